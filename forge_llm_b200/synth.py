"""Seeded synthetic models in the reference's ``weights.bin`` layout.

The layout is the one the reference's exporter writes and its generated loader reads
(crates/forgellm-cli/src/main.rs:2714-2757, crates/forgellm-codegen-cpu/src/project.rs:341-407):
``embed_tokens`` f32 ``[V, h]``; per layer ``attn_norm`` f32, ``q``, ``k``, ``v`` raw blocks,
optional f32 ``q_bias, k_bias, v_bias``, ``o``, ``ffn_norm`` f32, ``gate``, ``up``, ``down``;
``final_norm`` f32; ``lm_head`` raw blocks.  Projection bytes are GGUF Q8_0 (34 B per 32 values)
or Q4_0 (18 B per 32 values), rows of ``K/32`` blocks, ``N`` rows.

Values: every linear weight ~ N(0, 0.02) f32 from ``numpy.random.default_rng(seed)`` (PCG64),
drawn in file order and quantised at once; norm weights 1.0; biases N(0, 0.02).  For a tied
model the embedding is the dequantised lm_head, which is what the reference's exporter
produces from a tied quantised checkpoint (main.rs:2655-2693).
"""
from __future__ import annotations

import numpy as np


def _f16_round(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16)  # IEEE round-to-nearest-even, as weight_loader.rs:1361-1442


def _round_half_away(x: np.ndarray) -> np.ndarray:
    return np.copysign(np.floor(np.abs(x) + np.float32(0.5)), x)  # Rust f32::round


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """weight_loader.rs:1454-1486: d = amax/127 (stored f16), q = round(x * (1/d_f32)), clamp +-127."""
    b = np.ascontiguousarray(x, np.float32).reshape(-1, 32)
    amax = np.abs(b).max(axis=1)
    scale = np.where(amax == 0, np.float32(0), amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(scale != 0, np.float32(1.0) / scale, np.float32(0)).astype(np.float32)
    q = np.clip(_round_half_away(b * inv[:, None]), -127, 127).astype(np.int8)
    out = np.empty((b.shape[0], 34), np.uint8)
    out[:, :2] = _f16_round(scale).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """Signed-max rule of the benchmark configurations: d = (largest-magnitude value) / -8 stored
    as f16, nibble = clamp(round(x * (1/d_f32)) + 8, 0, 15); element j in the low nibble of byte j,
    element j+16 in the high nibble (weight_loader.rs:1494-1544 packs the same way)."""
    b = np.ascontiguousarray(x, np.float32).reshape(-1, 32)
    idx = np.abs(b).argmax(axis=1)
    vmax = b[np.arange(b.shape[0]), idx]
    d = np.where(vmax == 0, np.float32(0), vmax / np.float32(-8.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    q = np.clip(_round_half_away(b * inv[:, None]).astype(np.int32) + 8, 0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 18), np.uint8)
    out[:, :2] = _f16_round(d).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def dequantize(quant: int, raw: np.ndarray, n: int) -> np.ndarray:
    """weight_loader.rs:860-926."""
    if quant == 8:
        b = raw.reshape(-1, 34)
        d = b[:, :2].copy().view(np.float16).astype(np.float32)
        return (b[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)[:n]
    b = raw.reshape(-1, 18)
    d = b[:, :2].copy().view(np.float16).astype(np.float32)
    lo = (b[:, 2:] & 0x0F).astype(np.int32) - 8
    hi = (b[:, 2:] >> 4).astype(np.int32) - 8
    return (np.concatenate([lo, hi], axis=1).astype(np.float32) * d).reshape(-1)[:n]


_native = None


def quantize(quant: int, x: np.ndarray) -> np.ndarray:
    """Quantise with the library's host quantisers (multithreaded C++) when the shared object is
    built, else with the numpy statements above; the two are bit-identical (tests/)."""
    global _native
    if _native is None:
        try:
            from . import runtime
            _native = runtime
        except Exception:
            _native = False
    if _native:
        return _native.quantize_q8_0(x) if quant == 8 else _native.quantize_q4_0(x, True)
    return quantize_q8_0(x) if quant == 8 else quantize_q4_0(x)


def random_kquant(quant: int, rng: np.random.Generator, n: int, k: int, std: float) -> np.ndarray:
    """n rows of K-quant super-blocks drawn field by field (no quantiser is involved: every bit pattern of the
    scale and quant fields is a legal block); the f16 super-block scales are sized so that the dequantised weights
    have about the magnitude ``std``.  Q4_K: 144 bytes {d, dmin, 12 scale bytes, 128 nibble bytes}; Q6_K: 210 bytes
    {128 low-nibble bytes, 64 two-bit bytes, 16 int8 scales, d} (emit.rs:2962-2969, :3542-3546)."""
    nsb = n * (k // 256)
    if quant == 12:
        blk = rng.integers(0, 256, (nsb, 144), dtype=np.uint8)
        blk[:, 0:2] = (std / 256 * (0.5 + rng.random(nsb))).astype(np.float16).view(np.uint8).reshape(nsb, 2)
        blk[:, 2:4] = (std / 256 * (0.5 + rng.random(nsb))).astype(np.float16).view(np.uint8).reshape(nsb, 2)
    else:
        blk = rng.integers(0, 256, (nsb, 210), dtype=np.uint8)
        blk[:, 208:210] = (std / 1024 * (0.5 + rng.random(nsb))).astype(np.float16).view(np.uint8).reshape(nsb, 2)
    return blk.reshape(-1)


def weights_bin_size(c: dict) -> int:
    from .configs import proj_quants, raw_row_bytes
    h, qk, kv = c["hidden_size"], c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"]
    ff, V = c["intermediate_size"], c["vocab_size"]
    pq = proj_quants(c)
    mb = lambda cat, n, k: n * raw_row_bytes(pq[cat], k)
    per = h * 4 + mb(0, qk, h) + mb(1, kv, h) + mb(2, kv, h) + ((qk + 2 * kv) * 4 if c.get("qkv_bias") else 0) + mb(3, h, qk) + h * 4 \
        + mb(4, ff, h) + mb(5, ff, h) + mb(6, h, ff)
    return V * h * 4 + per * c["num_layers"] + h * 4 + mb(7, V, h)


def make_weights_bin(c: dict, seed: int = 0, std: float = 0.02, chunk_rows: int = 8192, quantize_fn=None,
                     repeat_layers: bool = False) -> np.ndarray:
    """Return the whole ``weights.bin`` image as a uint8 array.

    ``quantize_fn(quant, f32 array) -> uint8 array`` replaces the default quantiser (callers that must not load the
    CUDA library pass their own).  ``repeat_layers``: layer 0 is drawn from the generator and its bytes are repeated
    for the other layers - same shapes, sizes and value distribution at a fraction of the host time (timing runs of
    the multi-billion-parameter shapes, and the full-depth parity runs of those two shapes; every other test draws every layer)."""
    rng = np.random.default_rng(seed)
    qfn = quantize_fn or quantize
    h, qk, kv = c["hidden_size"], c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"]
    from .configs import proj_quants
    ff, V = c["intermediate_size"], c["vocab_size"]
    pq = proj_quants(c)
    out = np.empty(weights_bin_size(c), np.uint8)
    off = 0

    def put(a: np.ndarray):
        nonlocal off
        b = a.view(np.uint8).reshape(-1)
        out[off:off + b.size] = b
        off += b.size

    def draw_quant(n: int, k: int, cat: int) -> np.ndarray:
        quant = pq[cat]
        if quant in (12, 14):
            return random_kquant(quant, rng, n, k, std)
        parts = []
        for r0 in range(0, n, chunk_rows):
            r = min(chunk_rows, n - r0)
            w = rng.standard_normal((r, k), dtype=np.float32) * np.float32(std)
            parts.append(qfn(quant, w))
        return np.concatenate(parts) if len(parts) > 1 else parts[0]

    embed_off = off
    off += V * h * 4  # filled below (tied: from lm_head; untied: drawn first)
    if not c.get("tied"):
        save = off
        off = embed_off
        for r0 in range(0, V, chunk_rows):
            r = min(chunk_rows, V - r0)
            put(rng.standard_normal((r, h), dtype=np.float32) * np.float32(std))
        off = save
    ones = np.ones(h, np.float32)
    layer0 = off
    for li in range(c["num_layers"]):
        if repeat_layers and li > 0:
            n = off - layer0 if li == 1 else layer_bytes
            if li == 1:
                layer_bytes = n
            out[off:off + layer_bytes] = out[layer0:layer0 + layer_bytes]
            off += layer_bytes
            continue
        put(ones)
        put(draw_quant(qk, h, 0))
        put(draw_quant(kv, h, 1))
        put(draw_quant(kv, h, 2))
        if c.get("qkv_bias"):
            put(rng.standard_normal(qk, dtype=np.float32) * np.float32(std))
            put(rng.standard_normal(kv, dtype=np.float32) * np.float32(std))
            put(rng.standard_normal(kv, dtype=np.float32) * np.float32(std))
        put(draw_quant(h, qk, 3))
        put(ones)
        put(draw_quant(ff, h, 4))
        put(draw_quant(ff, h, 5))
        put(draw_quant(h, ff, 6))
    put(ones)
    lm = draw_quant(V, h, 7)
    put(lm)
    assert off == out.size
    if c.get("tied"):
        assert pq[7] in (8, 4), "tied synthetic models need a Q8_0 / Q4_0 head"
        emb = dequantize(pq[7], lm, V * h)
        out[embed_off:embed_off + V * h * 4] = emb.view(np.uint8)
    return out


def prompt_tokens(c: dict, n: int, seed: int = 1) -> np.ndarray:
    """Uniform token ids, ``numpy.random.default_rng(seed).integers(0, V)``."""
    return np.random.default_rng(seed).integers(0, c["vocab_size"], size=n).astype(np.uint32)
