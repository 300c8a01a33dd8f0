"""Failure detection on the device, without faulting anything: the per-head barrier of the
split-head_d kernel is made to wait (with a short limit) for an arrival that never comes.  The
kernel gives up, reports its error bits, the call returns B200ATTN_ERR_KERNEL, and the next call on
the same context cleans the scratch and is correct again."""
import numpy as np
import pytest
import torch

import oracle_lib as O

pytestmark = pytest.mark.gpu
ERR_KERNEL = 4
FLAG_ASYNC = 1


def _case(seed, B=1, H=4, L=64, D=2048):
    rng = np.random.default_rng(seed)
    q, k, v = (rng.uniform(-1, 1, (B, H, L, D)).astype(np.float32) for _ in range(3))
    return q, k, v, O.attention(q, k, v)


def _run(pkg, q, k, v, flags=0):
    Q, K, V = (torch.from_numpy(x).cuda() for x in (q, k, v))
    out = pkg.forward(Q, K, V, flags=flags)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_lost_arrival_is_reported_and_the_context_recovers(pkg, cuda):
    L = pkg.lib()
    q, k, v, want = _case(7)
    assert np.abs(_run(pkg, q, k, v) - want).max() <= 1e-4
    assert pkg.last_path() == "splitd_tc"
    L.b200attn_debug_lost_arrival(1, 20000)
    try:
        with pytest.raises(pkg.B200AttnError) as ei:
            _run(pkg, q, k, v)
        assert ei.value.status == ERR_KERNEL and "0x1" in str(ei.value)
        # an asynchronous call cannot report its own failure: the next call on the device does
        _run(pkg, q, k, v, flags=FLAG_ASYNC)
        with pytest.raises(pkg.B200AttnError) as ei:
            _run(pkg, q, k, v)
        assert ei.value.status == ERR_KERNEL and "earlier asynchronous call" in str(ei.value)
    finally:
        L.b200attn_debug_lost_arrival(0, 0)
    # same context, scratch cleaned by the library: results are right again, twice in a row
    for seed in (8, 9):
        q, k, v, want = _case(seed)
        assert np.abs(_run(pkg, q, k, v) - want).max() <= 1e-4
