"""lily_b200: a small, whole, single-GPU inference engine for the Llama / Qwen3 dense decoder,
written for NVIDIA B200 (sm_100a)."""

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "EngineConfig"):
        from lily_b200.engine import engine
        return getattr(engine, name)
    if name == "SamplingParams":
        from lily_b200.sampling.params import SamplingParams
        return SamplingParams
    if name == "ServerArgs":
        from lily_b200.config.server_args import ServerArgs
        return ServerArgs
    raise AttributeError(name)
