"""miniinfer_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

    from miniinfer_b200 import LLMEngine, SamplingParams
    engine = LLMEngine("/path/to/model", dtype="bfloat16")
    outputs = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=16))
"""

__version__ = "0.1.0"

_LAZY = {
  "LLMEngine": ("miniinfer_b200.engine.llm_engine", "LLMEngine"),
  "RequestOutput": ("miniinfer_b200.engine.llm_engine", "RequestOutput"),
  "SamplingParams": ("miniinfer_b200.sampling.params", "SamplingParams"),
  "EngineConfig": ("miniinfer_b200.config.engine_config", "EngineConfig"),
}


def __getattr__(name):
  if name in _LAZY:
    import importlib
    mod, attr = _LAZY[name]
    return getattr(importlib.import_module(mod), attr)
  raise AttributeError(name)
