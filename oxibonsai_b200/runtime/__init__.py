"""Runtime layer: engine, builders, presets, sampling, schedulers, controllers."""
from .presets import SamplingParams, SamplingPreset
from .builders import EngineBuilder, SamplerBuilder
