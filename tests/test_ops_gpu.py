"""Operator-level parity: each C-ABI operator against the oracle on the same seeded inputs.

Tolerances: the decode GEMV and all elementwise operators are f32 arithmetic in a different
summation order, so they must agree to ~1e-6 relative; the batched GEMM (m >= 8) is the
split-precision tensor-core form (~3e-5 at K = 8192); attention kernels read an fp16 cache and
are compared with the oracle's attention run on the same fp16-rounded K/V."""
import ctypes as C

import numpy as np
import pytest

from util import dev, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from forge_llm_b200._lib import check, lib
    return lib, check


def _sync():
    import torch
    torch.cuda.synchronize()


@pytest.mark.parametrize("quant", [8, 4])
@pytest.mark.parametrize("m,K,N", [(1, 32, 2), (1, 576, 192), (1, 2048, 512), (1, 8192, 2048), (1, 11008, 130),
                                   (3, 896, 130), (7, 576, 576), (8, 576, 576), (9, 896, 128), (17, 3072, 96),
                                   (100, 576, 1536), (130, 2048, 300), (37, 8192, 256)])
def test_matmul_mat(L, oracle, quant, m, K, N):
    import torch
    from forge_llm_b200 import synth
    lib, check = L
    rng = np.random.default_rng(1000 * quant + m + K + N)
    w = synth.quantize(quant, rng.standard_normal((N, K), dtype=np.float32) * 0.02)
    x = rng.standard_normal((m, K), dtype=np.float32)
    ref = oracle.matmul_mat(quant, x, w, K, N)
    dx, dw = dev(x), dev(w)
    out = torch.empty((m, N), dtype=torch.float32, device="cuda")
    fn = lib.forge_matmul_mat_q8_0 if quant == 8 else lib.forge_matmul_mat_q4_0
    check(fn(out.data_ptr(), m, dx.data_ptr(), dw.data_ptr(), K, N, None))
    _sync()
    got = out.cpu().numpy()
    tol = 4e-6 if m < 8 else 6e-5
    assert rel_l2(got, ref) < tol
    assert np.abs(got - ref).max() < 50 * tol * np.abs(ref).max()


@pytest.mark.parametrize("quant", [8, 4])
@pytest.mark.parametrize("nb,K,N", [(1, 32, 2), (2, 576, 192), (4, 2048, 512), (5, 896, 130), (8, 8192, 2048), (9, 11008, 4096),
                                    (16, 2048, 128), (16, 4096, 22016), (13, 3072, 9216), (16, 576, 49152), (7, 8192, 3072)])
def test_matmul_decode_batch(L, oracle, quant, nb, K, N):
    """The batched decode product (weights streamed once for up to 16 rows) against the per-row CPU products: the rows
    enter as fp16 hi + lo pairs (22 bits), the block scales are applied in f32."""
    import ctypes as C
    import torch
    from forge_llm_b200 import synth
    lib, check = L
    rng = np.random.default_rng(77 * quant + nb + K + N)
    w = synth.quantize(quant, rng.standard_normal((N, K), dtype=np.float32) * 0.02)
    x = rng.standard_normal((nb, K), dtype=np.float32)
    ref = oracle.matmul_mat(quant, x, w, K, N)
    dx, dw = dev(x), dev(w)
    out = torch.empty((nb, N), dtype=torch.float32, device="cuda")
    pk = C.c_void_p()
    check(lib.forge_packed_create(quant, dw.data_ptr(), K, N, None, C.byref(pk)))
    for _ in range(2):   # the second call reuses the buffers (and the self-resetting tickets)
        out.zero_()
        check(lib.forge_matmul_decode_batch(out.data_ptr(), nb, dx.data_ptr(), pk, None))
        check(lib.forge_packed_check(pk, None))
        got = out.cpu().numpy()
        assert rel_l2(got, ref) < 2e-6
        assert np.abs(got - ref).max() < 1e-4 * np.abs(ref).max()
    lib.forge_packed_destroy(pk)


@pytest.mark.parametrize("quant", [12, 14])
@pytest.mark.parametrize("m,K,N", [(1, 256, 2), (1, 512, 130), (1, 2048, 512), (1, 8192, 2048), (1, 11008 // 256 * 256, 19000),
                                   (3, 768, 130), (7, 1536, 144), (1, 2048, 32000),
                                   (9, 1536, 144), (37, 512, 256), (37, 256, 512), (100, 2048, 520), (130, 8192, 256)])
def test_matmul_vec_kquant(L, oracle, quant, m, K, N):
    """matmul_vec_q4_k / matmul_vec_q6_k: the input row is quantised to Q8_0 blocks as in the reference, the block dots
    are exact integers, so the result agrees with the oracle up to the f32 summation order.  From 8 rows on the rows
    go through the tensor-core GEMM together (same Q8_0 rounding of the input, weights dequantised to split fp16)."""
    import torch
    lib, check = L
    rng = np.random.default_rng(100 * quant + m + K + N)
    w = oracle.random_kquant_rows(quant, rng, N, K)
    x = rng.standard_normal((m, K), dtype=np.float32)
    x[:, 32:64] = 0.0  # an all-zero block (scale 1, zeros)
    ref = oracle.matmul_vec_kquant(quant, x, w, K, N)
    dx, dw = dev(x), dev(w)
    out = torch.empty((m, N), dtype=torch.float32, device="cuda")
    fn = lib.forge_matmul_vec_q4_k if quant == 12 else lib.forge_matmul_vec_q6_k
    check(fn(out.data_ptr(), m, dx.data_ptr(), dw.data_ptr(), K, N, None))
    _sync()
    got = out.cpu().numpy()
    if m < 8:
        assert rel_l2(got, ref) < 4e-6
        assert np.abs(got - ref).max() < 2e-4 * np.abs(ref).max()
    else:
        # the batched form rounds hi + lo of the f32 input (22 bits of it), so a value on a rounding boundary may land on
        # the other side: allow a few such rows, everything else agrees to the GEMM's split-precision accuracy
        rows = np.array([rel_l2(got[r], ref[r]) for r in range(m)])
        assert np.median(rows) < 6e-5 and (rows > 6e-5).sum() <= max(1, m // 10) and rows.max() < 2e-2


def test_matmul_vec_kquant_known_answer(L, oracle):
    # weight_loader.rs:2545-2569 through the C-ABI: every weight 4, every input 2 -> 2048 (the input is exactly
    # representable in Q8_0 here, so the product is exact)
    import torch
    lib, check = L
    blk = oracle.pack_q4_k_superblock(1.0, 0.0, [1] * 8, [0] * 8, np.full((4, 32), 4), np.full((4, 32), 4))
    dx, dw = dev(np.full(256, 2.0, np.float32)), dev(blk)
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    check(lib.forge_matmul_vec_q4_k(out.data_ptr(), 1, dx.data_ptr(), dw.data_ptr(), 256, 1, None))
    _sync()
    assert abs(out.item() - 2048.0) < 2048.0 * 2e-3
    assert out.item() == oracle.matmul_vec_kquant(12, np.full(256, 2.0, np.float32), blk, 256, 1)[0, 0]
    assert lib.forge_matmul_vec_q6_k(out.data_ptr(), 1, dx.data_ptr(), dw.data_ptr(), 224, 1, None) == 2  # K % 256


def test_matmul_known_answer(L):
    # crates/forgellm-runtime/src/kernels.rs:327-335 through the C-ABI: [1,2] x [[1,2],[3,4]]^T = [5,11]
    import torch
    lib, check = L
    scale = np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8)
    rows = []
    for a, b in ((1, 2), (3, 4)):
        q = np.zeros(32, np.int8)
        q[:2] = [a, b]
        rows.append(np.concatenate([scale, q.view(np.uint8)]))
    x = np.zeros(32, np.float32)
    x[:2] = [1, 2]
    dx, dw = dev(x), dev(np.concatenate(rows))
    out = torch.empty(2, dtype=torch.float32, device="cuda")
    check(lib.forge_matmul_mat_q8_0(out.data_ptr(), 1, dx.data_ptr(), dw.data_ptr(), 32, 2, None))
    _sync()
    assert out.cpu().tolist() == [5.0, 11.0]


def test_matmul_rejects_bad_shapes(L):
    import torch
    lib, _ = L
    t = torch.zeros(64, device="cuda")
    assert lib.forge_matmul_mat_q8_0(t.data_ptr(), 1, t.data_ptr(), t.data_ptr(), 48, 1, None) == 2
    assert lib.forge_matmul_mat_q8_0(None, 1, t.data_ptr(), t.data_ptr(), 32, 1, None) == 1
    assert lib.forge_matmul_mat_q4_0(t.data_ptr(), 0, t.data_ptr(), t.data_ptr(), 32, 1, None) == 0  # empty batch


@pytest.mark.parametrize("rows,n", [(1, 576), (5, 2048), (33, 3072), (2, 4)])
def test_rms_norm(L, oracle, rows, n):
    import torch
    lib, check = L
    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, n), dtype=np.float32) * 3
    w = rng.standard_normal(n, dtype=np.float32)
    dx, dw = dev(x), dev(w)
    out = torch.empty_like(dx)
    check(lib.forge_rms_norm(out.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, n, C.c_float(1e-5), None))
    _sync()
    ref = np.stack([oracle.rms_norm(x[r], w, 1e-5) for r in range(rows)])
    assert rel_l2(out.cpu().numpy(), ref) < 1e-6


@pytest.mark.parametrize("hd,heads,theta", [(64, 9, 1e5), (96, 4, 1e4), (128, 2, 5e5)])
def test_rope(L, oracle, hd, heads, theta):
    import torch
    lib, check = L
    rows, base = 11, 3000
    rng = np.random.default_rng(hd)
    x = rng.standard_normal((rows, heads * hd), dtype=np.float32)
    tab = np.empty((base + rows, hd // 2, 2), np.float32)
    check(lib.forge_rope_table(tab.ctypes.data_as(C.c_void_p), base + rows, hd, C.c_float(theta)))
    dx, dt = dev(x), dev(tab)
    check(lib.forge_rope(dx.data_ptr(), rows, base, hd, heads, dt.data_ptr(), None))
    _sync()
    f = oracle.rope_freqs(hd, theta)
    ref = np.stack([oracle.rope(x[r], base + r, hd, heads, f) for r in range(rows)])
    assert np.abs(dx.cpu().numpy() - ref).max() < 1e-6  # same table, one rounding order apart (FMA)


def test_silu_mul_and_residual_add(L, oracle):
    import torch
    lib, check = L
    rng = np.random.default_rng(5)
    g = rng.standard_normal(10001, dtype=np.float32) * 4
    u = rng.standard_normal(10001, dtype=np.float32)
    dg, du = dev(g), dev(u)
    out = torch.empty_like(dg)
    check(lib.forge_silu_mul(out.data_ptr(), dg.data_ptr(), du.data_ptr(), g.size, None))
    check(lib.forge_residual_add(dg.data_ptr(), du.data_ptr(), g.size, None))
    _sync()
    ref = oracle.silu_mul(g, u)
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-6 * max(1.0, np.abs(ref).max())
    assert np.array_equal(dg.cpu().numpy(), g + u)
    check(lib.forge_silu_mul(out.data_ptr(), dg.data_ptr(), du.data_ptr(), 0, None))  # empty input is a no-op


def _kv(rng, seq, nkv, hd, scale=1.0):
    k = (rng.standard_normal((seq, nkv * hd), dtype=np.float32) * scale).astype(np.float16)
    v = rng.standard_normal((seq, nkv * hd), dtype=np.float32).astype(np.float16)
    return k, v


@pytest.mark.parametrize("hd,nq,nkv", [(64, 9, 3), (64, 14, 2), (64, 32, 8), (96, 4, 4), (128, 4, 4), (128, 8, 1)])
@pytest.mark.parametrize("seq", [1, 5, 64, 70, 200, 1629, 3257])
def test_attention_flash_decode(L, oracle, hd, nq, nkv, seq):
    import torch
    lib, check = L
    rng = np.random.default_rng(hd * 7 + nq + seq)
    q = rng.standard_normal(nq * hd, dtype=np.float32)
    k, v = _kv(rng, seq, nkv, hd, 0.5)
    ref = oracle.attention_flash(q, oracle.KV_F16, k.astype(np.float32), v.astype(np.float32), None, None, seq, nq, nkv, hd)
    dq, dk, dv = dev(q), dev(k.view(np.uint16)), dev(v.view(np.uint16))
    out = torch.empty(nq * hd, dtype=torch.float32, device="cuda")
    check(lib.forge_attention_flash(out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), seq, nq, nkv, hd, None))
    _sync()
    assert rel_l2(out.cpu().numpy(), ref) < 3e-6


def test_attention_golden_inputs(L, oracle):
    # the closed-form inputs of emit.rs:6687-6701 cannot run as they are (head_dim 8); the same
    # generators at head_dim 64 exercise one-block, exact-block and multi-block contexts
    import torch
    lib, check = L
    nh, nkv, hd = 3, 1, 64
    for seq in (5, 64, 70, 128, 200):
        q = (((np.arange(nh * hd) * 7 + 3) % 23).astype(np.float32) * np.float32(0.1) - 1.0) * np.float32(0.5)
        k = ((((np.arange(seq * hd) * 11 + 5) % 29).astype(np.float32) * np.float32(0.07) - 1.0) * np.float32(0.3)).astype(np.float16)
        v = ((((np.arange(seq * hd) * 13 + 7) % 31).astype(np.float32) * np.float32(0.05) - 0.5) * np.float32(0.4)).astype(np.float16)
        ref = oracle.attention(q, oracle.KV_F16, k.astype(np.float32), v.astype(np.float32), None, None, seq, nh, nkv, hd)
        dq, dk, dv = dev(q), dev(k.view(np.uint16)), dev(v.view(np.uint16))
        out = torch.empty(nh * hd, dtype=torch.float32, device="cuda")
        check(lib.forge_attention_flash(out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), seq, nh, nkv, hd, None))
        _sync()
        assert np.abs(out.cpu().numpy() - ref).max() < 1e-4  # the reference test's own bound


@pytest.mark.parametrize("hd,nq,nkv", [(64, 9, 3), (64, 14, 2), (96, 4, 4), (128, 4, 2)])
@pytest.mark.parametrize("m,base", [(1, 0), (8, 0), (17, 0), (64, 0), (65, 0), (100, 0), (300, 0), (33, 100), (64, 64), (5, 700)])
def test_attention_flash_batch(L, oracle, hd, nq, nkv, m, base):
    import torch
    lib, check = L
    rng = np.random.default_rng(hd + nq + m + base)
    seq = base + m
    q = rng.standard_normal((m, nq * hd), dtype=np.float32)
    k, v = _kv(rng, seq, nkv, hd, 0.5)
    ref = oracle.attention_flash_batch(q, oracle.KV_F16, k.astype(np.float32), v.astype(np.float32), None, None, m, base, nq, nkv, hd)
    # pad the cache to a whole page: the kernel reads 64-position tiles
    pad = (-seq) % 64
    kp = np.concatenate([k, np.full((pad, nkv * hd), np.nan, np.float16)])
    vp = np.concatenate([v, np.full((pad, nkv * hd), np.nan, np.float16)])
    dq, dk, dv = dev(q), dev(kp.view(np.uint16)), dev(vp.view(np.uint16))
    out = torch.empty((m, nq * hd), dtype=torch.float32, device="cuda")
    check(lib.forge_attention_flash_batch(out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), m, base, nq, nkv, hd, None))
    _sync()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()  # NaN padding behind the causal limit must never leak
    assert rel_l2(got, ref) < 2e-5  # q and p enter the tensor-core products as fp16 hi + lo pairs


def test_kv_append_rounds_to_fp16(L):
    import torch
    lib, check = L
    rng = np.random.default_rng(3)
    kvd, rows, base = 192, 5, 7
    k = rng.standard_normal((rows, kvd), dtype=np.float32)
    v = rng.standard_normal((rows, kvd), dtype=np.float32)
    kc = torch.zeros((base + rows) * kvd, dtype=torch.uint16, device="cuda")
    vc = torch.zeros_like(kc)
    dk, dv = dev(k), dev(v)
    check(lib.forge_kv_append_f16(kc.data_ptr(), vc.data_ptr(), dk.data_ptr(), dv.data_ptr(), rows, base, kvd, None))
    _sync()
    got = kc.cpu().numpy().view(np.float16).reshape(base + rows, kvd)
    assert np.array_equal(got[base:], k.astype(np.float16)) and not got[:base].any()
    assert np.array_equal(vc.cpu().numpy().view(np.float16).reshape(base + rows, kvd)[base:], v.astype(np.float16))


def test_argmax_last_index_on_ties(L, oracle):
    import torch
    lib, check = L
    rng = np.random.default_rng(9)
    for n in (3, 1000, 151936):
        x = rng.standard_normal(n, dtype=np.float32)
        x[[n // 3, n // 2, n - 2]] = 9.0  # three equal maxima
        dx = dev(x)
        res = torch.zeros(1, dtype=torch.int32, device="cuda")
        check(lib.forge_argmax(res.data_ptr(), dx.data_ptr(), n, None))
        _sync()
        assert int(res.item()) == oracle.argmax(x) == n - 2
