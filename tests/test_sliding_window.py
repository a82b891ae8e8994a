"""Sliding-window attention (attention_sliding, attention_sliding_batch; Mistral-class configurations).

The reference's own tests for these functions only check that the code is emitted (emit.rs:6168-6260), so the CPU cases
pin the restatement against an independent float64 computation and against its unwindowed twins; the GPU cases compare
the CUDA kernels and a whole model with the restatement."""
import numpy as np
import pytest

from util import dev, rel_l2


def _kv(rng, seq, nkv, hd):
    k = (rng.standard_normal((seq, nkv * hd), dtype=np.float32) * 0.5).astype(np.float16)
    v = (rng.standard_normal((seq, nkv * hd), dtype=np.float32) * 0.5).astype(np.float16)
    return k, v


def _ref64(q, k, v, pos, window, nq, nkv, hd):
    """float64 attention of one query at position `pos` over keys [max(0, pos - window + 1), pos]."""
    lo = max(0, pos - window + 1)
    out = np.zeros(nq * hd)
    g = nq // nkv
    for h in range(nq):
        kk = k[lo:pos + 1, (h // g) * hd:(h // g + 1) * hd].astype(np.float64)
        vv = v[lo:pos + 1, (h // g) * hd:(h // g + 1) * hd].astype(np.float64)
        s = kk @ q[h * hd:(h + 1) * hd].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        out[h * hd:(h + 1) * hd] = (p / p.sum()) @ vv
    return out


@pytest.mark.parametrize("seq,window", [(5, 64), (64, 64), (65, 64), (200, 32), (200, 1), (130, 100)])
def test_oracle_sliding_single_query(oracle, seq, window):
    nq, nkv, hd = 6, 2, 64
    rng = np.random.default_rng(seq * 31 + window)
    q = rng.standard_normal(nq * hd, dtype=np.float32)
    k, v = _kv(rng, seq, nkv, hd)
    got = oracle.attention_sliding(q, oracle.KV_F16, k.astype(np.float32), v.astype(np.float32), None, None, seq, window, nq, nkv, hd)
    assert rel_l2(got, _ref64(q, k, v, seq - 1, window, nq, nkv, hd)) < 2e-6
    if window >= seq:  # a window that covers the context is plain attention, bit for bit
        plain = oracle.attention(q, oracle.KV_F16, k.astype(np.float32), v.astype(np.float32), None, None, seq, nq, nkv, hd)
        assert np.array_equal(got, plain)


@pytest.mark.parametrize("m,base,window", [(1, 0, 8), (40, 0, 16), (70, 0, 64), (100, 30, 32), (33, 100, 200), (17, 64, 1)])
def test_oracle_sliding_batch(oracle, m, base, window):
    nq, nkv, hd = 4, 2, 64
    rng = np.random.default_rng(m + 7 * base + window)
    seq = base + m
    q = rng.standard_normal((m, nq * hd), dtype=np.float32)
    k, v = _kv(rng, seq, nkv, hd)
    kf, vf = k.astype(np.float32), v.astype(np.float32)
    got = oracle.attention_sliding_batch(q, oracle.KV_F16, kf, vf, None, None, m, base, window, nq, nkv, hd)
    for r in range(m):  # each row equals the single-query function at its position (online vs two-pass softmax)
        one = oracle.attention_sliding(q[r], oracle.KV_F16, kf[:base + r + 1], vf[:base + r + 1], None, None, base + r + 1, window, nq, nkv, hd)
        assert rel_l2(got[r], one) < 2e-6
    if window >= seq:
        full = oracle.attention_flash_batch(q, oracle.KV_F16, kf, vf, None, None, m, base, nq, nkv, hd)
        assert rel_l2(got, full) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("hd,nq,nkv", [(64, 8, 2), (128, 4, 4)])
@pytest.mark.parametrize("seq,window", [(5, 64), (64, 64), (65, 64), (200, 32), (1000, 100), (513, 512), (300, 1)])
def test_cuda_attention_sliding(oracle, hd, nq, nkv, seq, window):
    import torch
    from forge_llm_b200._lib import check, lib
    rng = np.random.default_rng(hd + seq + window)
    q = rng.standard_normal(nq * hd, dtype=np.float32)
    k, v = _kv(rng, seq, nkv, hd)
    ref = oracle.attention_sliding(q, oracle.KV_F16, k.astype(np.float32), v.astype(np.float32), None, None, seq, window, nq, nkv, hd)
    dq, dk, dv = dev(q), dev(k.view(np.uint16)), dev(v.view(np.uint16))
    out = torch.empty(nq * hd, dtype=torch.float32, device="cuda")
    check(lib.forge_attention_sliding(out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), seq, window, nq, nkv, hd, None))
    torch.cuda.synchronize()
    assert rel_l2(out.cpu().numpy(), ref) < 3e-6


@pytest.mark.gpu
@pytest.mark.parametrize("hd,nq,nkv", [(64, 8, 2), (128, 4, 2)])
@pytest.mark.parametrize("m,base,window", [(1, 0, 8), (70, 0, 64), (100, 30, 32), (300, 0, 100), (33, 100, 200), (64, 64, 1), (200, 500, 128)])
def test_cuda_attention_sliding_batch(oracle, hd, nq, nkv, m, base, window):
    import torch
    from forge_llm_b200._lib import check, lib
    rng = np.random.default_rng(hd + m + base + window)
    seq = base + m
    q = rng.standard_normal((m, nq * hd), dtype=np.float32)
    k, v = _kv(rng, seq, nkv, hd)
    ref = oracle.attention_sliding_batch(q, oracle.KV_F16, k.astype(np.float32), v.astype(np.float32), None, None, m, base, window, nq, nkv, hd)
    pad = (-seq) % 64
    kp = np.concatenate([k, np.full((pad, nkv * hd), np.nan, np.float16)])
    vp = np.concatenate([v, np.full((pad, nkv * hd), np.nan, np.float16)])
    dq, dk, dv = dev(q), dev(kp.view(np.uint16)), dev(vp.view(np.uint16))
    out = torch.empty((m, nq * hd), dtype=torch.float32, device="cuda")
    check(lib.forge_attention_sliding_batch(out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), m, base, window, nq, nkv, hd, None))
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_l2(got, ref) < 2e-5  # q and p enter the tensor-core products as fp16 hi + lo pairs


@pytest.mark.gpu
@pytest.mark.parametrize("quant,window", [(8, 32), (4, 64), (4, 100)])
def test_model_with_sliding_window(oracle, quant, window):
    from forge_llm_b200 import configs, runtime, synth
    c = dict(configs.tiny(quant, hd=64, nq=4, nkv=2, layers=2), sliding_window=window)
    blob = synth.make_weights_bin(c)
    toks = synth.prompt_tokens(c, 150)
    gm = runtime.Model(c, blob)
    kv = gm.new_cache(max_seq=200)
    om = oracle.OracleModel(c, blob, kv_mode=oracle.KV_F16)
    lo = om.forward_prefill(toks)
    lg = gm.forward_prefill(toks, kv)
    assert np.abs(lg - lo).max() < 2e-2
    full = oracle.OracleModel(dict(c, sliding_window=0), blob, kv_mode=oracle.KV_F16).forward_prefill(toks)
    assert np.abs(full - lo).max() > 1e-3  # the window really changes the result at this length
    for _ in range(4):
        t = oracle.argmax(lo)
        lo = om.forward(t)
        lg = gm.forward(t, kv)
        assert np.abs(lg - lo).max() < 2e-2
    kv.reset()
    om.reset()
    assert np.array_equal(gm.generate_greedy(toks, 24, kv), om.generate_greedy(toks, 24)[0])
    kv.close()
    gm.close()
