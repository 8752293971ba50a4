"""sglang-rs_b200: a small, whole inference engine for one GPU (B200, sm_100a).

    from sglang_rs_b200 import Engine
    engine = Engine(model_path="...", dtype="bfloat16")
    engine.generate([1, 2, 3], {"max_new_tokens": 8})
"""
__version__ = "0.1.0"

from .sampling.params import SamplingParams  # noqa: E402,F401


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
