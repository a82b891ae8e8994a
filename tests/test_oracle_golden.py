"""The oracle against every known-answer vector the reference's own tests hold for this path.

Each case names the reference test it reproduces (paths relative to the reference tree)."""
import numpy as np
import pytest


def test_f16_basic_values(oracle):
    # crates/forgellm-frontend/src/weight_loader.rs:2470-2482 (f16_conversion_basic)
    assert oracle.f16_to_f32(0x0000) == 0.0
    for bits, val in ((0x3C00, 1.0), (0xBC00, -1.0), (0x3800, 0.5), (0x4000, 2.0)):
        assert abs(oracle.f16_to_f32(bits) - val) < 1e-6


def test_f16_special_values(oracle):
    # weight_loader.rs:2484-2492 (f16_special_values)
    assert np.isinf(oracle.f16_to_f32(0x7C00))
    assert np.isnan(oracle.f16_to_f32(0x7E00))
    v = oracle.f16_to_f32(0x8000)
    assert v == 0.0 and np.signbit(v)


def test_f16_widening_matches_ieee_for_all_bit_patterns(oracle):
    bits = np.arange(0x10000, dtype=np.uint16)
    ieee = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in bits], np.float32)
    nan = np.isnan(ieee)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), ieee[~nan].view(np.uint32))


def test_f32_to_f16_round_to_nearest_even(oracle):
    # weight_loader.rs:1361-1442: RNE; f32 subnormals and magnitudes below 2^-25 flush to zero
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-3, 1.0, 100.0)])
    x = np.concatenate([x, np.float32([0.0, -0.0, 65504.0, 65520.0, 1e6, -1e6, 6.1e-5, 5.97e-8, 2.0 ** -24, 2.0 ** -14])])
    got = np.array([oracle.f32_to_f16(float(v)) for v in x], np.uint16)
    with np.errstate(over="ignore"):
        ieee = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, ieee)
    assert oracle.f32_to_f16(np.float32(2.0 ** -26)) == 0
    assert oracle.f32_to_f16(np.float32(1e-40)) == 0


def test_dequant_q8_0_basic(oracle):
    # weight_loader.rs:3210-3224: scale 1.0 (0x3C00), int8 values 0..31 -> 0..31
    block = np.concatenate([np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8), np.arange(32, dtype=np.uint8)])
    out = oracle.dequant_q8_0(block, 32)
    assert np.allclose(out, np.arange(32), atol=1e-6)


def test_dequant_q4_0_basic(oracle):
    # weight_loader.rs:3227-3242: scale 1.0, bytes 0x88 -> all zeros
    block = np.concatenate([np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8), np.full(16, 0x88, np.uint8)])
    out = oracle.dequant_q4_0(block, 32)
    assert np.all(np.abs(out) < 1e-6)


def test_q4_0_nibble_order(oracle):
    # emit.rs:2337-2359 / weight_loader.rs:908-921: byte j = element j (low) and element j+16 (high)
    qs = np.arange(16, dtype=np.uint8) | ((15 - np.arange(16, dtype=np.uint8)) << 4)
    block = np.concatenate([np.frombuffer(np.uint16(0x4000).tobytes(), np.uint8), qs])  # d = 2.0
    out = oracle.dequant_q4_0(block, 32)
    assert np.array_equal(out[:16], (np.arange(16) - 8) * 2.0)
    assert np.array_equal(out[16:], (15 - np.arange(16) - 8) * 2.0)


def test_quantize_q8_0_round_trip(oracle):
    # weight_loader.rs:3003-3018: ramp (i-32)*0.05 over two blocks, error < 0.02
    v = ((np.arange(64) - 32) * 0.05).astype(np.float32)
    q = oracle.quantize_q8_0(v)
    assert q.size == 2 * 34
    assert np.all(np.abs(oracle.dequant_q8_0(q, 64) - v) < 0.02)


def test_quantize_q8_0_zero_block(oracle):
    # weight_loader.rs:3021-3028
    q = oracle.quantize_q8_0(np.zeros(32, np.float32))
    assert np.all(oracle.dequant_q8_0(q, 32) == 0.0)


def test_quantize_q4_0_round_trip(oracle):
    # weight_loader.rs:3341-3362: ramp (i-32)*0.1, |error| <= step + 0.01 with step = max|x|/8
    v = ((np.arange(64) - 32) * 0.1).astype(np.float32)
    q = oracle.quantize_q4_0(v, "ref")
    assert q.size == 2 * 18
    step = np.abs(v).max() / 8.0
    assert np.all(np.abs(oracle.dequant_q4_0(q, 64) - v) <= step + 0.01)


def test_quantize_q4_0_zeros(oracle):
    # weight_loader.rs:3365-3379: zero input -> zero scale bits, zero output
    for rule in ("ref", "signed"):
        q = oracle.quantize_q4_0(np.zeros(32, np.float32), rule)
        assert q.size == 18 and q[0] == 0 and q[1] == 0
        assert np.all(oracle.dequant_q4_0(q, 32) == 0.0)


def test_quantize_q4_0_signed_rule_reaches_minus_eight(oracle):
    # signed-max rule: the largest-magnitude value maps to nibble 0 (= -8 * d) exactly
    v = np.zeros(32, np.float32)
    v[5] = 0.8
    v[9] = -0.3
    q = oracle.quantize_q4_0(v, "signed")
    out = oracle.dequant_q4_0(q, 32)
    assert abs(out[5] - 0.8) < 1e-3 and (q[2 + 5] & 0x0F) == 0


@pytest.mark.parametrize("seq_len", [5, 64, 70, 128, 200])
def test_flash_attention_matches_plain(oracle, seq_len):
    # emit.rs:6558-6741 (flash_attention_numerical_equivalence): 3 heads, 1 kv head, head_dim 8,
    # closed-form inputs, |flash - plain| < 1e-4 on f32 K/V
    nh, nkv, hd = 3, 1, 8
    q = (((np.arange(nh * hd) * 7 + 3).astype(np.float32) * np.float32(0.1) - 1.0) * 0.5).astype(np.float32)
    k = (((np.arange(seq_len * hd) * 11 + 5).astype(np.float32) * np.float32(0.07) - 1.0) * 0.3).astype(np.float32)
    v = (((np.arange(seq_len * hd) * 13 + 7).astype(np.float32) * np.float32(0.05) - 0.5) * 0.4).astype(np.float32)
    plain = oracle.attention(q, oracle.KV_F32, k, v, None, None, seq_len, nh, nkv, hd)
    flash = oracle.attention_flash(q, oracle.KV_F32, k, v, None, None, seq_len, nh, nkv, hd)
    assert np.abs(plain - flash).max() < 1e-4
    # the batched kernel with one query at the last position must agree too
    fb = oracle.attention_flash_batch(q, oracle.KV_F32, k, v, None, None, 1, seq_len - 1, nh, nkv, hd)
    assert np.abs(plain - fb).max() < 1e-4
    # independent float64 statement of softmax attention
    K = k.reshape(seq_len, hd).astype(np.float64)
    V = v.reshape(seq_len, hd).astype(np.float64)
    for h in range(nh):
        s = K @ q[h * hd:(h + 1) * hd].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        p /= p.sum()
        ref = p @ V
        assert np.abs(ref - plain[h * hd:(h + 1) * hd]).max() < 1e-6 * max(1.0, np.abs(ref).max())


def test_kv_quantize_round_trip(oracle):
    # emit.rs:6814-6852: ((7i+3)*0.1-3)*0.5, max round-trip error <= one step
    v = (((np.arange(64) * 7 + 3).astype(np.float32) * np.float32(0.1) - 3.0) * 0.5).astype(np.float32)
    q, scale = oracle.quantize_kv(v)
    assert abs(scale - np.abs(v).max() / 127.0) < 1e-7
    assert np.abs(q.astype(np.float32) * scale - v).max() <= scale + 1e-6
    q0, s0 = oracle.quantize_kv(np.zeros(8, np.float32))
    assert s0 == 0.0 and not q0.any()


def test_matmul_vec_basic(oracle):
    # crates/forgellm-runtime/src/kernels.rs:327-335: [1,2] x [[1,2],[3,4]]^T = [5,11], with the
    # two weight rows written as hand-built Q8_0 (scale 1.0) and Q4_0 (scale 1.0) blocks
    scale = np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8)
    x = np.zeros(32, np.float32)
    x[:2] = [1, 2]
    rows8 = []
    rows4 = []
    for a, b in ((1, 2), (3, 4)):
        q = np.zeros(32, np.int8)
        q[:2] = [a, b]
        rows8.append(np.concatenate([scale, q.view(np.uint8)]))
        nib = np.full(16, 0x88, np.uint8)  # all zeros after the -8 offset
        nib[0] = (a + 8) | (8 << 4)
        nib[1] = (b + 8) | (8 << 4)
        rows4.append(np.concatenate([scale, nib]))
    assert np.array_equal(oracle.matmul_vec(8, x, np.concatenate(rows8), 32, 2), np.float32([5, 11]))
    assert np.array_equal(oracle.matmul_vec(4, x, np.concatenate(rows4), 32, 2), np.float32([5, 11]))
    assert np.array_equal(oracle.matmul_mat(8, x[None], np.concatenate(rows8), 32, 2)[0], np.float32([5, 11]))


def test_rms_norm_basic(oracle):
    # crates/forgellm-runtime/src/kernels.rs:396-413
    x = np.float32([1, 2, 3, 4])
    out = oracle.rms_norm(x, np.ones(4, np.float32), 1e-5)
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-5)
    assert np.abs(out - ref).max() < 1e-5


def test_rope_preserves_norm(oracle):
    # crates/forgellm-runtime/src/interpreter.rs:293-303
    rng = np.random.default_rng(1)
    x = rng.standard_normal(4 * 64).astype(np.float32)
    f = oracle.rope_freqs(64, 1e4)
    y = oracle.rope(x, 17, 64, 4, f)
    assert abs(np.linalg.norm(y) - np.linalg.norm(x)) < 1e-4
    assert np.array_equal(oracle.rope(x, 0, 64, 4, f), x)  # position 0 is the identity
    # adjacent-pair convention (emit.rs:523-525)
    ang = np.float32(17) * f[3]
    assert abs(y[6] - (x[6] * np.cos(ang) - x[7] * np.sin(ang))) < 1e-5


def test_argmax_cases(oracle):
    # crates/forgellm-runtime/src/sampling.rs:165-169, plus the last-index tie rule of max_by
    # (crates/forgellm-codegen-cpu/src/project.rs:501-503)
    assert oracle.argmax(np.float32([1.0, 3.0, 2.0])) == 1
    assert oracle.argmax(np.float32([5.0, 1.0, 2.0])) == 0
    assert oracle.argmax(np.float32([-1.0, -2.0, -0.5])) == 2
    assert oracle.argmax(np.float32([1.0, 7.0, 7.0, 0.0])) == 2


def test_silu_mul_formula(oracle):
    g = np.float32([-3.0, -0.5, 0.0, 0.5, 3.0])
    u = np.float32([2.0, 2.0, 2.0, 2.0, 2.0])
    ref = (g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64)))) * u
    assert np.abs(oracle.silu_mul(g, u) - ref).max() < 1e-6


@pytest.mark.parametrize("quant", [8, 4])
def test_row_vectorised_matmul_is_bit_identical(oracle, quant):
    from forge_llm_b200 import synth
    rng = np.random.default_rng(2)
    K, N, m = 576, 77, 9
    w = synth.quantize(quant, rng.standard_normal((N, K), dtype=np.float32) * 0.02)
    x = rng.standard_normal((m, K), dtype=np.float32)
    a = oracle.matmul_mat(quant, x, w, K, N, fast=True)
    b = oracle.matmul_mat(quant, x, w, K, N, fast=False)
    assert np.array_equal(a, b)
    ref = x.astype(np.float64) @ synth.dequantize(quant, w, N * K).reshape(N, K).astype(np.float64).T
    assert np.abs(a - ref).max() < 1e-5


def test_batched_prefill_equals_per_token_path(oracle):
    # emit.rs:4576-4587: both paths of forward_prefill compute the same values on x86 except for
    # the f32 summation order inside P.V; also checks the fp16 and f32 KV stand-ins stay close
    from forge_llm_b200 import configs, synth
    c = configs.tiny(8, layers=2)
    blob = synth.make_weights_bin(c)
    toks = synth.prompt_tokens(c, 150)
    outs = {}
    for mode in (oracle.KV_INT8, oracle.KV_F16, oracle.KV_F32):
        a = oracle.OracleModel(c, blob, kv_mode=mode)
        b = oracle.OracleModel(c, blob, kv_mode=mode)
        la, ta = a.forward_prefill(toks, trace=True)
        lb, tb = b.forward_prefill(toks, trace=True, force_per_token=True)
        assert np.abs(la - lb).max() < 2e-5
        assert np.abs(ta - tb).max() < 2e-5
        assert a.len == b.len == 150
        outs[mode] = la
    assert np.abs(outs[oracle.KV_F16] - outs[oracle.KV_F32]).max() < 5e-3
    # short prompts (< PREFILL_BATCH_THRESHOLD) take the per-token path
    s = oracle.OracleModel(c, blob)
    l1 = s.forward_prefill(toks[:5])
    t = oracle.OracleModel(c, blob)
    for tok in toks[:5]:
        l2 = t.forward(int(tok))
    assert np.array_equal(l1, l2)


# ---- K-quants: the reference's own known-answer tests (crates/forgellm-frontend/src/weight_loader.rs)
def _f16_bytes(bits):
    return np.frombuffer(np.uint16(bits).tobytes(), np.uint8)


def test_dequant_q4_k_basic_and_values(oracle):
    # WL:3422-3450: d = 1, dmin = 0, all scales 1, all q = 0 -> zeros
    b = np.zeros(144, np.uint8)
    b[0:2] = _f16_bytes(0x3C00)
    b[4:8] = 1
    b[12:16] = 0x01
    assert np.all(np.abs(oracle.dequant_kquant(oracle.Q4_K, b, 256)) < 1e-6)
    # WL:3453-3478: d = 2, dmin = 1, sub-block 0 scale 3 and min 2, low nibbles 5 -> 2*3*5 - 1*2 = 28
    b = np.zeros(144, np.uint8)
    b[0:2] = _f16_bytes(0x4000)
    b[2:4] = _f16_bytes(0x3C00)
    b[4], b[8] = 3, 2
    b[16:48] = 0x05
    out = oracle.dequant_kquant(oracle.Q4_K, b, 256)
    assert np.all(np.abs(out[:32] - 28.0) < 1e-4)


def test_dequant_q6_k_known_answers(oracle):
    # WL:3562-3583: all quants 0 -> (0 - 32) * 1 * 1
    b = np.zeros(210, np.uint8)
    b[208:210] = _f16_bytes(0x3C00)
    b[192:208] = 1
    assert np.all(np.abs(oracle.dequant_kquant(oracle.Q6_K, b, 256) + 32.0) < 1e-4)
    # WL:3586-3609: d = 0.5, scale[0] = 2, ql[0] = 0x0A, qh[0] = 2 -> 0.5 * 2 * ((10 | 32) - 32) = 10
    c = np.zeros(210, np.uint8)
    c[208:210] = _f16_bytes(0x3800)
    c[192], c[0], c[128] = 2, 0x0A, 0x02
    assert abs(oracle.dequant_kquant(oracle.Q6_K, c, 256)[0] - 10.0) < 1e-4
    # WL:3612-3657: the four values interleaved in one (ql, ql+32, qh) triple
    b[0], b[32], b[128] = 0x31, 0x52, 0xE4
    out = oracle.dequant_kquant(oracle.Q6_K, b, 256)
    assert [out[0], out[32], out[64], out[96]] == [-31.0, -14.0, 3.0, 21.0]


def test_dot_q4_k_uniform_block(oracle):
    # WL:2545-2569: every weight dequantises to 4, every input is 2 -> 256 * 2 * 4 = 2048 within 1 %
    blk = oracle.pack_q4_k_superblock(1.0, 0.0, [1] * 8, [0] * 8, np.full((4, 32), 4), np.full((4, 32), 4))
    assert np.all(np.abs(oracle.dequant_kquant(oracle.Q4_K, blk, 256) - 4.0) < 1e-5)
    got = oracle.matmul_vec_kquant(oracle.Q4_K, np.full(256, 2.0, np.float32), blk, 256, 1)[0, 0]
    assert abs(got - 2048.0) / 2048.0 < 0.01


def test_dot_q4_k_varied_block(oracle):
    # WL:2572-2605: varied scales / mins / nibbles against the f32 product of the dequantised weights, within 2 %
    c, i = np.arange(4)[:, None], np.arange(32)[None, :]
    blk = oracle.pack_q4_k_superblock(0.03, 0.01, [3, 5, 7, 2, 10, 4, 6, 8], [1, 2, 3, 1, 2, 1, 1, 2],
                                      (c * 4 + i // 8) % 16, (c * 2 + i % 16) % 16)
    x = (np.sin(np.arange(256, dtype=np.float32) * np.float32(0.1)) * 0.5).astype(np.float32)
    want = float(np.sum(oracle.dequant_kquant(oracle.Q4_K, blk, 256) * x, dtype=np.float32))
    got = oracle.matmul_vec_kquant(oracle.Q4_K, x, blk, 256, 1)[0, 0]
    assert abs(got - want) / max(abs(want), 1e-6) < 0.02


@pytest.mark.parametrize("quant", [12, 14])
def test_kquant_dot_equals_product_of_dequantised_operands(oracle, quant):
    # the property behind WL:2979-3001: the integer block dots reproduce dequant(W) . dequant(Q8_0(x)) up to f32 rounding
    rng = np.random.default_rng(quant)
    K, N = 1024, 24
    w = oracle.random_kquant_rows(quant, rng, N, K)
    x = rng.standard_normal((3, K)).astype(np.float32)
    got = oracle.matmul_vec_kquant(quant, x, w, K, N)
    W = oracle.dequant_kquant(quant, w, N * K).reshape(N, K).astype(np.float64)
    for r in range(3):
        q, s = oracle.quantize_act_q8_0(x[r])
        xd = (q.reshape(-1, 32).astype(np.float64) * s[:, None]).ravel()
        assert np.abs(got[r] - W @ xd).max() < 2e-5 * np.abs(W @ xd).max()


def test_activation_q8_0_blocks(oracle):
    # emit.rs:1412-1440: absmax maps to +-127, a zero block keeps scale 1 and zeros, ties round away from zero
    x = np.zeros(96, np.float32)
    x[0:32] = np.linspace(-1.0, 1.0, 32)
    x[64:96] = 127.0
    x[64] = 0.5
    x[65] = -2.5
    q, s = oracle.quantize_act_q8_0(x)
    assert q[0] == -127 and q[31] == 127 and np.all(q[32:64] == 0) and s[1] == 1.0
    assert s[2] == 1.0 and q[64] == 1 and q[65] == -3 and np.all(q[66:96] == 127)


# ---- K-quant quantisers: the reference's own tests (weight_loader.rs:2733-2975), run on the CPU restatement
def test_quantize_q4_k_round_trips(oracle):
    ramp = ((np.arange(512, dtype=np.float32) - np.float32(256.0)) * np.float32(0.005)).astype(np.float32)
    q = oracle.quantize_kquant(oracle.Q4_K, ramp)
    assert q.size == 2 * 144
    assert np.abs(oracle.dequant_kquant(oracle.Q4_K, q, 512) - ramp).max() < 0.05          # WL:2735-2755
    state, vals = 0xDEADBEEF, []
    for _ in range(512):                                                                  # WL:2758-2780
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        vals.append((np.float32(state >> 16) / np.float32(65535.0) - np.float32(0.5)) * np.float32(0.2))
    v = np.array(vals, np.float32)
    d = oracle.dequant_kquant(oracle.Q4_K, oracle.quantize_kquant(oracle.Q4_K, v), 512)
    assert np.sqrt(np.mean((d.astype(np.float64) - v) ** 2)) < 0.005
    z = oracle.dequant_kquant(oracle.Q4_K, oracle.quantize_kquant(oracle.Q4_K, np.zeros(256, np.float32)), 256)
    assert np.all(np.abs(z) < 1e-3)                                                        # WL:2895-2903


def test_quantize_q6_k_round_trips_and_is_unbiased(oracle):
    ramp = ((np.arange(512, dtype=np.float32) - np.float32(256.0)) * np.float32(0.005)).astype(np.float32)
    q = oracle.quantize_kquant(oracle.Q6_K, ramp)
    assert q.size == 2 * 210
    assert np.abs(oracle.dequant_kquant(oracle.Q6_K, q, 512) - ramp).max() < 0.02          # WL:2906-2921
    v = (np.random.default_rng(0xFEED).standard_normal(4096) * 0.05).astype(np.float32)    # WL:2924-2966 (Gaussian weights)
    d = oracle.dequant_kquant(oracle.Q6_K, oracle.quantize_kquant(oracle.Q6_K, v), 4096).astype(np.float64)
    err = d - v
    assert abs(err.mean()) < 5.0 * np.sqrt(np.mean(err ** 2)) / np.sqrt(4096)
    z = oracle.dequant_kquant(oracle.Q6_K, oracle.quantize_kquant(oracle.Q6_K, np.zeros(256, np.float32)), 256)
    assert np.all(np.abs(z) < 1e-3)                                                        # WL:2969-2976
