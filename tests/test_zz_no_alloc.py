"""forge_attention_flash_static: the decode attention with its split-KV workspace in a fixed array of the
library instead of per-call allocations, for hosts that cannot let the library allocate device memory.

Collected last on purpose (file name): a run that stops at the first failure has then already run every
other test.  The checks are against the allocating entry point on the same inputs and against the CPU restatement of
attention_flash, several calls in a row, so that a later call meets the scratch exactly as an earlier one left it."""
import numpy as np
import pytest

from util import dev, rel_l2

pytestmark = pytest.mark.gpu


def _case(rng, nq, nkv, hd, seq):
    q = rng.standard_normal(nq * hd, dtype=np.float32)
    k = (rng.standard_normal((seq, nkv * hd), dtype=np.float32) * 0.5).astype(np.float16)
    v = rng.standard_normal((seq, nkv * hd), dtype=np.float32).astype(np.float16)
    return q, k, v


def test_static_scratch_attention_matches_allocating_entry_point(oracle):
    import torch
    from forge_llm_b200._lib import check, lib
    rng = np.random.default_rng(77)
    # two calls in a row: a long context with many splits, then a short one that uses fewer splits and
    # fewer heads, so stale partials and tickets of the first call are still lying in the array
    for nq, nkv, hd, seq in ((32, 8, 64, 3257), (9, 3, 64, 70), (4, 4, 128, 1629), (14, 2, 96, 200)):
        q, k, v = _case(rng, nq, nkv, hd, seq)
        dq, dk, dv = dev(q), dev(k.view(np.uint16)), dev(v.view(np.uint16))
        ref = torch.empty(nq * hd, dtype=torch.float32, device="cuda")
        got = torch.full((nq * hd,), float("nan"), dtype=torch.float32, device="cuda")
        check(lib.forge_attention_flash(ref.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), seq, nq, nkv, hd, None))
        check(lib.forge_attention_flash_static(got.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), seq, nq, nkv, hd, None))
        torch.cuda.synchronize()
        a, b = got.cpu().numpy(), ref.cpu().numpy()
        assert np.isfinite(a).all()
        assert rel_l2(a, b) < 3e-6  # the tolerance of the decode-attention parity test
        # and against the CPU restatement (fp16 K/V stand-in), with the same bound as the allocating entry point's own test
        want = oracle.attention_flash(q, oracle.KV_F16, k.astype(np.float32), v.astype(np.float32), None, None, seq, nq, nkv, hd)
        assert rel_l2(a, want) < 3e-6


def test_static_scratch_attention_rejects_oversized_shapes():
    import torch
    from forge_llm_b200._lib import lib
    t = torch.zeros(256, device="cuda")
    p = t.data_ptr()
    assert lib.forge_attention_flash_static(p, p, p, p, 16, 65, 1, 64, None) == 2      # too many heads
    assert lib.forge_attention_flash_static(p, p, p, p, 16, 4, 4, 256, None) == 2      # head_dim beyond the array
    assert lib.forge_attention_flash_static(p, p, p, p, (1 << 20) + 1, 4, 4, 64, None) == 2
    assert b"exceeds the built-in scratch" in lib.forge_last_error()
    assert lib.forge_attention_flash_static(None, p, p, p, 16, 4, 4, 64, None) == 1
