"""A small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

Model folder (config.json, model.safetensors) -> typed configuration -> parts -> paged cache ->
step function -> scheduler -> sampled tokens, with hand-written CUDA kernels on the device.
"""
from . import architectures  # noqa: F401  (fills the architecture registry)
from . import cache, config, weights

__all__ = ["cache", "config", "weights", "load_model", "StepEngine", "StepEntry", "Engine", "Scheduler",
           "SchedulerConfig", "GenerationRequest", "RequestResult", "SamplingParams", "RandomStream"]


def __getattr__(name):
    # The parts that need the GPU library are imported on first use, so that configuration, weights,
    # cache bookkeeping and scheduling can be used (and tested) on a machine without a GPU.
    if name in ("load_model",):
        from .engine.loading import load_model
        return load_model
    if name in ("StepEngine", "StepEntry"):
        from .engine import step as _step
        return getattr(_step, name)
    if name == "Engine":
        from .engine.generate import Engine
        return Engine
    if name in ("Scheduler", "SchedulerConfig", "GenerationRequest", "RequestResult"):
        from .engine import scheduler as _sched
        return getattr(_sched, name)
    if name in ("SamplingParams", "RandomStream"):
        from .sampling import params as _params
        return getattr(_params, name)
    raise AttributeError(name)
