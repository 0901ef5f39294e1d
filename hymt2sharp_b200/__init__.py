"""hymt2sharp_b200: a small, whole inference library for the Hunyuan dense
architecture on one B200 GPU — configuration and registry, weights by name,
layers from parts, a paged cache, one step function, a generation loop, GPU
sampling, a command line and trace replay, on hand-written sm_100a kernels."""

__version__ = "0.1.0"


def load(model_dir: str, dtype="bfloat16", **options):
    """Loads the model folder (config.json + model.safetensors) into an Engine."""
    from .engine.engine import Engine
    return Engine(model_dir, dtype=dtype, **options)


def __getattr__(name):
    if name in ("Engine", "StepEntry", "EngineError"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    if name == "write_random_model":
        from .weights.random_init import write_random_model
        return write_random_model
    raise AttributeError(name)
