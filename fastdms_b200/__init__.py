"""fastdms_b200: B200-native (sm_100a) implementation of the compact-DMS decode path.

The module layout mirrors the reference project (`fastdms.layers.compact_attention`,
`fastdms.engine.compact_kv`, `fastdms.engine.dms`, `fastdms.layers.attention`,
`fastdms.utils.context`, ...).  `import fastdms_b200 as fastdms` switches code that reaches everything
through the package object; `install_as_fastdms()` also makes `from fastdms.layers.compact_attention
import ...` style imports resolve to this package.
"""
__version__ = "0.1.0"

_MIRRORED = (
    "config", "llm", "sampling_params",
    "engine", "engine.compact_kv", "engine.dms", "engine.llm_engine", "engine.model_runner", "engine.scheduler",
    "engine.sequence",
    "layers", "layers.activation", "layers.attention", "layers.compact_attention", "layers.embed_head",
    "layers.layernorm", "layers.linear", "layers.rotary_embedding", "layers.sampler",
    "models", "models.llama", "models.qwen3",
    "utils", "utils.context", "utils.loader", "utils.profiler",
)


def install_as_fastdms(force: bool = False) -> None:
    """Registers this package and its sub-modules under the reference's names in `sys.modules`
    (`fastdms`, `fastdms.layers.compact_attention`, ...), so that unchanged application code written
    against the reference imports this implementation.  Refuses to shadow a `fastdms` package that is
    already imported unless `force` is given."""
    import importlib
    import sys
    if "fastdms" in sys.modules and sys.modules["fastdms"] is not sys.modules[__name__] and not force:
        raise RuntimeError("a different `fastdms` package is already imported; pass force=True to replace it")
    sys.modules["fastdms"] = sys.modules[__name__]
    for name in _MIRRORED:
        sys.modules[f"fastdms.{name}"] = importlib.import_module(f"{__name__}.{name}")


def __getattr__(name):
    # LLM / SamplingParams are imported lazily: they pull in the model stack.
    if name == "LLM":
        from fastdms_b200.llm import LLM
        return LLM
    if name == "SamplingParams":
        from fastdms_b200.sampling_params import SamplingParams
        return SamplingParams
    raise AttributeError(name)
