"""CPU checks of the C-ABI boundary: the library builds/loads, exports exactly what the header
declares, and the ctypes signatures have the header's arity.  No kernel is launched."""
from __future__ import annotations

import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "fastdms_b200.h").read_text()


def _declared():
    """name -> number of parameters, parsed from the header."""
    text = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:int32_t|int64_t|const char\*)\s+(fdms_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
    return out


@pytest.fixture(scope="module")
def lib():
    from fastdms_b200 import _lib, build
    if build.needs_build():
        build.build()
    return _lib.lib()


def test_header_and_bindings_agree(lib):
    from fastdms_b200 import _lib
    decl = _declared()
    assert len(decl) >= 14
    assert set(decl) == set(_lib.exported_symbols())
    for name, nargs in decl.items():
        fn = getattr(lib, name)          # raises AttributeError if the symbol is not exported
        assert len(fn.argtypes) == nargs, f"{name}: header has {nargs} parameters, binding {len(fn.argtypes)}"


def test_version_and_workspace_size(lib):
    assert lib.fdms_abi_version() == 1
    assert lib.fdms_last_error() == b""
    n = lib.fdms_attn_decode_workspace_bytes(8, 8, 64)
    assert n > 0 and n % 4 == 0
    assert lib.fdms_attn_decode_workspace_bytes(8, 8, 128) > n
    assert lib.fdms_attn_decode_workspace_bytes(-1, 8, 64) < 0


def test_argument_errors_are_reported_without_a_gpu(lib):
    from fastdms_b200 import _lib
    # null pointers / bad sizes are rejected on the host before any CUDA call
    rc = lib.fdms_kv_quant(None, 0, None, None, 4, 2, 64, None)
    assert rc == _lib.FDMS_E_ARG and b"null pointer" in lib.fdms_last_error()
    with pytest.raises(ValueError):
        _lib.check(rc)
    rc = lib.fdms_extract_decisions(1 << 12, 0, 64, 64, 1 << 12, 2, 4, 5, 2, 64, 100.0, 5.0, None)
    assert rc == _lib.FDMS_E_ARG and b"divisible" in lib.fdms_last_error()


def test_product_fails_loudly_without_cuda():
    import torch
    from fastdms_b200.layers.compact_attention import compact_decode_attention
    q = torch.zeros((1, 4, 64))
    k = torch.zeros((16, 64))
    meta = torch.ones((1, 1), dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        compact_decode_attention(q, k, k, meta, meta)
    from fastdms_b200.engine.compact_kv import CompactKVManager
    with pytest.raises(RuntimeError, match="CUDA"):
        CompactKVManager(num_layers=1, num_kv_heads=1, capacity_tokens=16, max_model_len=16, device="cpu",
                         head_dim=16, compact_dtype=torch.float32)


def test_product_does_not_import_the_oracle():
    pkg = ROOT / "fastdms_b200"
    for path in pkg.rglob("*.py"):
        src = path.read_text()
        assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f"{path} imports the oracle"
