"""fastdms_b200: B200-native (sm_100a) implementation of the compact-DMS decode path.

The module layout mirrors the reference project (`fastdms.layers.compact_attention`,
`fastdms.engine.compact_kv`, `fastdms.engine.dms`, `fastdms.layers.attention`,
`fastdms.utils.context`, ...), so switching is `import fastdms_b200 as fastdms`.
"""
__version__ = "0.1.0"


def __getattr__(name):
    # LLM / SamplingParams are imported lazily: they pull in the model stack.
    if name == "LLM":
        from fastdms_b200.llm import LLM
        return LLM
    if name == "SamplingParams":
        from fastdms_b200.sampling_params import SamplingParams
        return SamplingParams
    raise AttributeError(name)
