"""Session-level behaviour around the decode step: scratch growth with several caches on one model, and the status
a bounded device-side wait returns when it runs out.  Nothing here faults or hangs the GPU: the waits that are made
to run out are the kernels' own bounded polls, and the kernels return by themselves."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-2


def _tiny(quant=4):
    from forge_llm_b200 import configs, synth
    c = configs.tiny(quant, hd=64, nq=4, nkv=2, layers=2)
    return c, synth.make_weights_bin(c), synth.prompt_tokens(c, 40)


def test_scratch_growth_between_caches(oracle):
    """A batch-1 cache and a batch-4 cache share one model: the second grows the decode scratch after the first has
    already decoded and captured its step as a graph; both must keep matching the CPU restatement."""
    from forge_llm_b200 import runtime
    c, blob, toks = _tiny()
    gm = runtime.Model(c, blob)
    kv1 = gm.new_cache(max_seq=128)
    kv4 = gm.new_cache(max_seq=128, batch=4)
    oms = [oracle.OracleModel(c, blob, kv_mode=oracle.KV_F16) for _ in range(5)]
    lo = [om.forward_prefill(toks[: 20 + 3 * i]) for i, om in enumerate(oms)]
    gm.forward_prefill(toks[:20], kv1)
    for b in range(4):
        gm.forward_prefill(toks[: 23 + 3 * b], kv4, seq=b)
    for rnd in range(3):
        # batch-1 step on the first cache
        t = oracle.argmax(lo[0])
        lo[0] = oms[0].forward(t)
        assert np.abs(gm.forward(t, kv1) - lo[0]).max() < LOGIT_TOL
        # batched step on the second cache: the scratch grows in the first round
        ts = [oracle.argmax(lo[1 + b]) for b in range(4)]
        lg = gm.forward_batch(ts, kv4)
        for b in range(4):
            lo[1 + b] = oms[1 + b].forward(ts[b])
            assert np.abs(lg[b] - lo[1 + b]).max() < LOGIT_TOL
        # single-sequence steps on the batched cache
        t2 = oracle.argmax(lo[3])
        lo[3] = oms[3].forward(t2)
        assert np.abs(gm.forward(t2, kv4, seq=2) - lo[3]).max() < LOGIT_TOL
    kv1.close(); kv4.close(); gm.close()


def test_peer_sum_that_never_arrives_reports_timeout():
    """Tensor-parallel decode over peer memory on ONE GPU: rank 0 of a two-rank cut is attached to an exchange in which
    the slot of rank 1 is its own buffer, so nobody ever pushes rank 1's partial sums.  The consumer's bounded wait runs
    out, the kernels return, the call reports TIMEOUT and the position is not advanced."""
    from forge_llm_b200 import runtime
    from forge_llm_b200._lib import ForgeError
    c, blob, toks = _tiny(4)
    gm = runtime.Model(c, blob, tp_rank=0, tp_world=2)
    h = gm.tp_exchange_handle()
    gm.tp_exchange_attach(np.concatenate([h, h]))
    gm.set_wait_limit(64)
    kv = gm.new_cache(max_seq=64)
    with pytest.raises(ForgeError) as ei:
        gm.forward(int(toks[0]), kv)
    assert ei.value.code == 5, ei.value
    assert kv.len() == 0
    kv.close(); gm.close()
