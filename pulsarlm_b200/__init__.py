"""pulsarlm_b200: a single-GPU inference engine for B200 (sm_100a).

    from pulsarlm_b200 import Engine, SamplingParams
    engine = Engine("model_dir", dtype="bfloat16")
    engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0), max_tokens=8)
"""

__version__ = "0.1.0"

_EXPORTS = {
    "Engine": ("pulsarlm_b200.engine.engine", "Engine"),
    "complete": ("pulsarlm_b200.engine.engine", "complete"),
    "SamplingParams": ("pulsarlm_b200.sampling.params", "SamplingParams"),
    "write_random_model": ("pulsarlm_b200.weights.random_init", "write_random_model"),
    "register_architecture": ("pulsarlm_b200.config.registry", "register_architecture"),
    "register_part": ("pulsarlm_b200.parts.registry", "register_part"),
}


def __getattr__(name):
    if name in _EXPORTS:
        import importlib

        module, attr = _EXPORTS[name]
        return getattr(importlib.import_module(module), attr)
    raise AttributeError(f"module 'pulsarlm_b200' has no attribute {name!r}")
