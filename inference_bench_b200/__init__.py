"""A small, whole, B200-native inference engine for the Qwen3 dense decoder.

    from inference_bench_b200 import Engine, SamplingParams
    engine = Engine.load("path/to/model", max_ctx=4096)
    reply = engine.generate([1, 2, 3], max_tokens=16)
"""
from .sampling.params import SamplingParams  # noqa: F401


def __getattr__(name):
    if name in ("Engine", "Reply"):
        from .engine import engine as _e
        return getattr(_e, name)
    raise AttributeError(name)
