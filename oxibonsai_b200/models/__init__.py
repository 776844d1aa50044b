"""Model families.  The one served family is the Qwen3 decoder (``qwen3``); ``registry`` maps shapes to variants."""
