"""``python -m oxibonsai_b200`` runs the command line (see ``oxibonsai_b200.cli``)."""
import sys

from .cli import main

sys.exit(main())
