"""air_b200: a single-GPU inference engine for the Qwen2 dense decoder on NVIDIA B200.

    from air_b200 import InferenceService, GenerationConfig, SamplingConfig, SchedulerConfig
    service = InferenceService.create("/path/to/model", dtype="bfloat16")
    response = service.generate([5, 17, 3], GenerationConfig(max_new_tokens=16))
"""
__version__ = "0.1.0"

from .sampling.sampler import GenerationConfig, SamplingConfig  # noqa: F401


def __getattr__(name):
    # the engine's modules load torch and the CUDA library; import them on first use
    if name in ("InferenceService", "SchedulerConfig", "InferenceResponse", "CancellationSource", "CancellationToken"):
        from .engine import service
        return getattr(service, name)
    if name in ("Engine", "EngineConfig", "write_random_model"):
        from .engine import engine
        return getattr(engine, name)
    if name == "Entry":
        from .engine.batch import Entry
        return Entry
    raise AttributeError(name)
