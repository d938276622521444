"""The allocation-free attention entry point (fdms_attn_decode_noalloc) against the ordinary one.

Some callers of this library have no way to obtain a split-K workspace: a serving process that gave
all device memory to its KV pool at start-up and bans later cudaMalloc calls, or a runtime written
in another language that loads the library as a plugin and owns no device allocator.  For them the
scratch is an array inside the library.  The test drives both entry points through the C ABI on the
same inputs, twice in a row (the built-in scratch keeps the first call's contents, so the second
call checks that stale data does no harm), with a shape whose spans are split over several clusters
so that the scratch is really used, and checks the documented size limits.

Collected last on purpose: if it fails, `pytest -x` has already run every other test."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, q, k, v, base, live, out, ws=None):
    from fastdms_b200 import _lib
    B, Hq, D = q.shape
    Hk = base.shape[1]
    args = [q.data_ptr(), _lib.BF16, q.stride(0), q.stride(1), k.data_ptr(), v.data_ptr(), _lib.dtype_code(k.dtype), k.shape[0],
            base.data_ptr(), live.data_ptr(), live.stride(0), None, 0, 0, 0, None, None,
            out.data_ptr(), _lib.BF16, out.stride(0), out.stride(1), B, Hq, Hk, D, float(D ** -0.5), None, None, 0, 0]
    if ws is not None:
        args += [ws.data_ptr(), ws.numel(), 0]
    args += [None, torch.cuda.current_stream().cuda_stream]
    return fn(*args)


@pytest.mark.parametrize("B,Hk,G,D,lens,pool", [
    (1, 2, 4, 64, (3000, 1700), torch.float8_e4m3fn), (1, 1, 8, 128, (2500,), torch.float8_e4m3fn),
    (8, 8, 4, 64, None, torch.float8_e4m3fn),
    (2, 2, 4, 64, (300, 170, 90, 411), torch.bfloat16)])     # a bf16 pool takes the generic kernel (no scratch use)
def test_noalloc_matches_workspace_entry_point(B, Hk, G, D, lens, pool):
    from fastdms_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(7 + B + D)
    if lens is None:
        live = torch.randint(1100, 1400, (B, Hk), device=dev, generator=g, dtype=torch.int32)
    else:
        live = torch.tensor(lens, device=dev, dtype=torch.int32).view(B, Hk)
    base = (torch.cumsum(live.flatten().to(torch.int64) + 5, 0) - live.flatten() - 5).to(torch.int32).view(B, Hk).contiguous()
    rows = int((live.to(torch.int64) + 5).sum())
    k = torch.randn((rows, D), device=dev, generator=g).to(pool)
    v = torch.randn((rows, D), device=dev, generator=g).to(pool)
    ws = torch.zeros(lib.fdms_attn_decode_workspace_bytes(B, Hk, D), dtype=torch.uint8, device=dev)
    for round_ in range(2):                               # two calls in a row, new q each time
        q = torch.randn((B, Hk * G, D), device=dev, generator=g).to(torch.bfloat16)
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        _lib.check(_call(lib.fdms_attn_decode, q, k, v, base, live, want, ws))
        _lib.check(_call(lib.fdms_attn_decode_noalloc, q, k, v, base, live, got))
        torch.cuda.synchronize(dev)
        # both entry points run the same kernel with the same split of the spans: identical bits
        assert torch.equal(got, want), f"call {round_}: outputs differ"
    assert _lib.read_device_status(dev) == 0


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch():
    from fastdms_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    k = torch.zeros((64, 64), device=dev, dtype=torch.float8_e4m3fn)
    # 4097 spans: one more than the scratch has counters for
    q = torch.zeros((4097, 4, 64), device=dev, dtype=torch.bfloat16)
    meta = torch.ones((4097, 1), device=dev, dtype=torch.int32)
    rc = _call(lib.fdms_attn_decode_noalloc, q, k, k, meta, meta, torch.empty_like(q))
    assert rc == _lib.FDMS_E_CAPACITY and b"4096" in lib.fdms_last_error()
    with pytest.raises(RuntimeError, match="scratch limit"):
        _lib.check(rc)
    # head_dim 256 is beyond the 128 the scratch is sized for
    q = torch.zeros((1, 4, 256), device=dev, dtype=torch.bfloat16)
    k = torch.zeros((64, 256), device=dev, dtype=torch.float8_e4m3fn)
    meta = torch.ones((1, 1), device=dev, dtype=torch.int32)
    rc = _call(lib.fdms_attn_decode_noalloc, q, k, k, meta, meta, torch.empty_like(q))
    assert rc == _lib.FDMS_E_CAPACITY and b"head_dim=256" in lib.fdms_last_error()
    # argument errors are reported before anything is enqueued (9 q heads over 2 KV heads)
    q = torch.zeros((1, 9, 64), device=dev, dtype=torch.bfloat16)
    k = torch.zeros((64, 64), device=dev, dtype=torch.float8_e4m3fn)
    meta = torch.ones((1, 2), device=dev, dtype=torch.int32)
    rc = _call(lib.fdms_attn_decode_noalloc, q, k, k, meta, meta, torch.empty_like(q))
    assert rc == _lib.FDMS_E_ARG and b"divisible" in lib.fdms_last_error()
