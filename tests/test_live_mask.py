"""`build_dms_live_mask` of the package against the vectors the reference's own function produced
(tests/golden/make_golden_ops.py: `livemask_*`; reference fastdms/engine/dms.py:235-262): the mask of
tokens that are still visible, live = not evicted, or inside the delayed window."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from fastdms_b200.engine.dms import build_dms_live_mask


def _check(z, device):
    ev = torch.from_numpy(z["livemask_evict"].astype(bool)).to(device)
    for cur, w, pos_key, want_key in ((39, 8, None, "livemask_cur39_w8"), (50, 0, None, "livemask_cur50_w0"),
                                      (60, 16, "livemask_positions", "livemask_cur60_w16_pos")):
        pos = None if pos_key is None else torch.from_numpy(z[pos_key].astype(np.int64)).to(device)
        got = build_dms_live_mask(ev, current_position=cur, window_size=w, positions=pos)
        assert got.dtype == torch.bool and got.shape == ev.shape
        assert np.array_equal(got.cpu().numpy(), z[want_key].astype(bool)), want_key
    # a single layer's [kv_heads, tokens] slice gives that layer's rows
    got = build_dms_live_mask(ev[0], current_position=39, window_size=8)
    assert np.array_equal(got.cpu().numpy(), z["livemask_cur39_w8"][0].astype(bool))


def test_live_mask_matches_reference_vectors(ops_golden):
    _check(ops_golden, "cpu")


def test_live_mask_argument_errors():
    ev = torch.zeros((2, 5), dtype=torch.bool)
    with pytest.raises(ValueError):
        build_dms_live_mask(ev.view(-1), current_position=3, window_size=1)
    with pytest.raises(ValueError):
        build_dms_live_mask(ev, current_position=3, window_size=-1)
    with pytest.raises(ValueError):
        build_dms_live_mask(ev, current_position=3, window_size=1, positions=torch.arange(4))


@pytest.mark.gpu
def test_live_mask_on_device_tensors(ops_golden):
    _check(ops_golden, "cuda:0")
