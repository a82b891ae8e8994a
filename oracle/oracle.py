"""ctypes binding of the CPU oracle (``oracle/forge_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by
``bench.py`` for the CPU-baseline / reference arm.  The shipped package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libforge_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (no-op when up to date)."""
    src = os.path.join(_HERE, "forge_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


class FoConfig(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_int32), ("intermediate_size", C.c_int32), ("num_layers", C.c_int32),
        ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("vocab_size", C.c_int32), ("max_seq_len", C.c_int32),
        ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float),
        ("quant", C.c_int32), ("qkv_bias", C.c_int32), ("sliding_window", C.c_int32),
        ("proj_quant", C.c_int32 * 8),
    ]


_lib = None
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")


def lib():
    global _lib
    if _lib is not None:
        return _lib
    try:
        so = build()
    except Exception:  # no compiler on this host: fall back to the prebuilt file
        so = _SO
    L = C.CDLL(so)
    vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    sigs = {
        "fo_f32_to_f16": (C.c_uint16, [f]),
        "fo_f16_to_f32": (f, [C.c_uint16]),
        "fo_quantize_q8_0": (None, [_f32p, sz, _u8p]),
        "fo_quantize_q4_0_ref": (None, [_f32p, sz, _u8p]),
        "fo_quantize_q4_0_signed": (None, [_f32p, sz, _u8p]),
        "fo_dequant_q8_0": (None, [_u8p, sz, _f32p]),
        "fo_dequant_q4_0": (None, [_u8p, sz, _f32p]),
        "fo_dot_q8_0": (f, [_f32p, _u8p, i]),
        "fo_dot_q4_0": (f, [_f32p, _u8p, i]),
        "fo_matmul_vec_q8_0": (None, [_f32p, _f32p, _u8p, i, i]),
        "fo_matmul_vec_q4_0": (None, [_f32p, _f32p, _u8p, i, i]),
        "fo_matmul_mat_q8_0": (None, [_f32p, i, _f32p, _u8p, i, i, i]),
        "fo_matmul_mat_q4_0": (None, [_f32p, i, _f32p, _u8p, i, i, i]),
        "fo_quantize_act_q8_0": (None, [_f32p, i, np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS"), _f32p]),
        "fo_matmul_vec_kquant": (None, [i, _f32p, i, _f32p, _u8p, i, i]),
        "fo_quantize_q4_k": (None, [_f32p, sz, _u8p]),
        "fo_quantize_q6_k": (None, [_f32p, sz, _u8p]),
        "fo_dequant_q4_k": (None, [_u8p, sz, _f32p]),
        "fo_dequant_q6_k": (None, [_u8p, sz, _f32p]),
        "fo_rms_norm": (None, [_f32p, _f32p, _f32p, i, f]),
        "fo_silu_mul": (None, [_f32p, _f32p, _f32p, i]),
        "fo_residual_add": (None, [_f32p, _f32p, i]),
        "fo_rope_freqs": (None, [_f32p, i, f]),
        "fo_rope": (None, [_f32p, i, i, i, _f32p]),
        "fo_quantize_kv": (f, [_f32p, i, np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")]),
        "fo_argmax": (C.c_uint32, [_f32p, i]),
        "fo_attention": (None, [_f32p, _f32p, i, vp, vp, vp, vp, i, i, i, i]),
        "fo_attention_flash": (None, [_f32p, _f32p, i, vp, vp, vp, vp, i, i, i, i]),
        "fo_attention_flash_batch": (None, [_f32p, _f32p, i, vp, vp, vp, vp, i, i, i, i, i]),
        "fo_attention_sliding": (None, [_f32p, _f32p, i, vp, vp, vp, vp, i, i, i, i, i]),
        "fo_attention_sliding_batch": (None, [_f32p, _f32p, i, vp, vp, vp, vp, i, i, i, i, i, i]),
        "fo_weights_bin_size": (sz, [C.POINTER(FoConfig)]),
        "fo_model_create": (vp, [C.POINTER(FoConfig), vp, sz]),
        "fo_model_set_fast": (None, [vp, i]),
        "fo_model_destroy": (None, [vp]),
        "fo_kv_create": (vp, [vp, i]),
        "fo_kv_reset": (None, [vp]),
        "fo_kv_len": (i, [vp]),
        "fo_kv_destroy": (None, [vp]),
        "fo_kv_read": (None, [vp, i, i, _f32p]),
        "fo_forward": (i, [vp, vp, C.c_uint32, _f32p, vp]),
        "fo_forward_prefill": (i, [vp, vp, _u32p, i, _f32p, vp, i]),
        "fo_num_threads": (i, []),
        "fo_set_num_threads": (None, [i]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


KV_INT8, KV_F16, KV_F32 = 0, 1, 2


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------------ element ops
def f32_to_f16(x: float) -> int:
    return int(lib().fo_f32_to_f16(x))


def f16_to_f32(h: int) -> float:
    return float(lib().fo_f16_to_f32(h))


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).ravel()
    out = np.empty(((x.size + 31) // 32) * 34, np.uint8)
    lib().fo_quantize_q8_0(x, x.size, out)
    return out


def quantize_q4_0(x: np.ndarray, rule: str = "ref") -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).ravel()
    out = np.empty(((x.size + 31) // 32) * 18, np.uint8)
    (lib().fo_quantize_q4_0_ref if rule == "ref" else lib().fo_quantize_q4_0_signed)(x, x.size, out)
    return out


def dequant_q8_0(b: np.ndarray, n: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().fo_dequant_q8_0(np.ascontiguousarray(b, np.uint8), n, out)
    return out


def dequant_q4_0(b: np.ndarray, n: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().fo_dequant_q4_0(np.ascontiguousarray(b, np.uint8), n, out)
    return out


def matmul_mat(quant: int, x: np.ndarray, w: np.ndarray, K: int, N: int, fast: bool = True) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    out = np.empty((x.shape[0], N), np.float32)
    fn = lib().fo_matmul_mat_q8_0 if quant == 8 else lib().fo_matmul_mat_q4_0
    fn(out, x.shape[0], x, np.ascontiguousarray(w, np.uint8), K, N, int(fast))
    return out


def matmul_vec(quant: int, x: np.ndarray, w: np.ndarray, K: int, N: int) -> np.ndarray:
    out = np.empty(N, np.float32)
    fn = lib().fo_matmul_vec_q8_0 if quant == 8 else lib().fo_matmul_vec_q4_0
    fn(out, np.ascontiguousarray(x, np.float32), np.ascontiguousarray(w, np.uint8), K, N)
    return out


# ---- K-quants (quant 12 = Q4_K, 14 = Q6_K: the GGML type numbers)
Q4_K, Q6_K = 12, 14


def kquant_row_bytes(quant: int, K: int) -> int:
    return (K // 256) * (144 if quant == Q4_K else 210)


def quantize_act_q8_0(x: np.ndarray):
    """The Q8_0 form every K-quant product gives its input row: (int8 values, f16-rounded block scales)."""
    x = np.ascontiguousarray(x, np.float32).ravel()
    q = np.empty(((x.size + 31) // 32) * 32, np.int8)
    s = np.empty((x.size + 31) // 32, np.float32)
    lib().fo_quantize_act_q8_0(x, x.size, q, s)
    return q, s


def matmul_vec_kquant(quant: int, x: np.ndarray, w: np.ndarray, K: int, N: int) -> np.ndarray:
    """matmul_vec_q4_k_KxN / matmul_vec_q6_k_KxN applied to every row of x."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    out = np.empty((x.shape[0], N), np.float32)
    lib().fo_matmul_vec_kquant(quant, out, x.shape[0], x, np.ascontiguousarray(w, np.uint8), K, N)
    return out


def dequant_kquant(quant: int, b: np.ndarray, n: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    (lib().fo_dequant_q4_k if quant == Q4_K else lib().fo_dequant_q6_k)(np.ascontiguousarray(b, np.uint8), n, out)
    return out


def quantize_kquant(quant: int, x: np.ndarray) -> np.ndarray:
    """quantize_f32_to_q4_k / quantize_f32_to_q6_k (WL:1773-1900, :2025-2125); x.size must be a multiple of 256."""
    x = np.ascontiguousarray(x, np.float32).ravel()
    assert x.size % 256 == 0
    out = np.empty(x.size // 256 * (144 if quant == Q4_K else 210), np.uint8)
    (lib().fo_quantize_q4_k if quant == Q4_K else lib().fo_quantize_q6_k)(x, x.size, out)
    return out


def pack_q4_k_superblock(d: float, dmin: float, scales, mins, q_lo, q_hi) -> np.ndarray:
    """One 144-byte Q4_K super-block from its fields: scales/mins are the eight 6-bit values, q_lo[c] / q_hi[c]
    the 32 nibbles of sub-blocks 2c / 2c+1 (the inverse of the scale unpacking, WL:2499-2542)."""
    out = np.zeros(144, np.uint8)
    out[0:2] = np.frombuffer(np.uint16(f32_to_f16(d)).tobytes(), np.uint8)
    out[2:4] = np.frombuffer(np.uint16(f32_to_f16(dmin)).tobytes(), np.uint8)
    sc, mn = [int(v) for v in scales], [int(v) for v in mins]
    for i in range(4):
        out[4 + i] = (sc[i] & 63) | (((sc[i + 4] >> 4) & 3) << 6)
        out[8 + i] = (mn[i] & 63) | (((mn[i + 4] >> 4) & 3) << 6)
        out[12 + i] = (sc[i + 4] & 15) | ((mn[i + 4] & 15) << 4)
    lo = np.asarray(q_lo, np.uint8).reshape(4, 32) & 15
    hi = np.asarray(q_hi, np.uint8).reshape(4, 32) & 15
    out[16:144] = (lo | (hi << 4)).ravel()
    return out


def random_kquant_rows(quant: int, rng: np.random.Generator, N: int, K: int, scale: float = 0.02) -> np.ndarray:
    """N rows of valid K-quant super-blocks with random fields (no quantiser involved): every byte pattern of the
    quant fields is legal, only the f16 scales are drawn from a sane range."""
    nsb = N * (K // 256)
    if quant == Q4_K:
        blk = rng.integers(0, 256, (nsb, 144), dtype=np.uint8)
        d = (scale / 32 * (0.5 + rng.random(nsb))).astype(np.float16)
        dmin = (scale / 32 * (0.5 + rng.random(nsb))).astype(np.float16)
        blk[:, 0:2] = d.view(np.uint8).reshape(nsb, 2)
        blk[:, 2:4] = dmin.view(np.uint8).reshape(nsb, 2)
    else:
        blk = rng.integers(0, 256, (nsb, 210), dtype=np.uint8)
        d = (scale / 1024 * (0.5 + rng.random(nsb))).astype(np.float16)
        blk[:, 208:210] = d.view(np.uint8).reshape(nsb, 2)
    return blk.reshape(-1)


def rms_norm(x, w, eps):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    lib().fo_rms_norm(out, x, np.ascontiguousarray(w, np.float32), x.size, eps)
    return out


def silu_mul(g, u):
    g = np.ascontiguousarray(g, np.float32)
    out = np.empty_like(g)
    lib().fo_silu_mul(out, g, np.ascontiguousarray(u, np.float32), g.size)
    return out


def rope_freqs(head_dim: int, theta: float) -> np.ndarray:
    f = np.empty(head_dim // 2, np.float32)
    lib().fo_rope_freqs(f, head_dim, theta)
    return f


def rope(data, pos, head_dim, heads, freqs):
    d = np.array(data, np.float32, copy=True).ravel()
    lib().fo_rope(d, pos, head_dim, heads, np.ascontiguousarray(freqs, np.float32))
    return d


def quantize_kv(v):
    v = np.ascontiguousarray(v, np.float32)
    q = np.empty(v.size, np.int8)
    s = lib().fo_quantize_kv(v, v.size, q)
    return q, float(s)


def argmax(v) -> int:
    v = np.ascontiguousarray(v, np.float32)
    return int(lib().fo_argmax(v, v.size))


def _attn(fn, q, mode, k, v, ks, vs, *tail):
    q = np.ascontiguousarray(q, np.float32)
    out = np.empty_like(q)
    fn(out, q, mode, _ptr(k), _ptr(v), _ptr(ks), _ptr(vs), *tail)
    return out


def _kv_args(mode, k, v, ks, vs):
    if mode == KV_INT8:
        return (np.ascontiguousarray(k, np.int8), np.ascontiguousarray(v, np.int8),
                np.ascontiguousarray(ks, np.float32), np.ascontiguousarray(vs, np.float32))
    return np.ascontiguousarray(k, np.float32), np.ascontiguousarray(v, np.float32), None, None


def attention(q, mode, k, v, ks, vs, seq, nh, nkv, hd):
    return _attn(lib().fo_attention, q, mode, *_kv_args(mode, k, v, ks, vs), seq, nh, nkv, hd)


def attention_flash(q, mode, k, v, ks, vs, seq, nh, nkv, hd):
    return _attn(lib().fo_attention_flash, q, mode, *_kv_args(mode, k, v, ks, vs), seq, nh, nkv, hd)


def attention_flash_batch(qb, mode, k, v, ks, vs, m, base_pos, nh, nkv, hd):
    return _attn(lib().fo_attention_flash_batch, qb, mode, *_kv_args(mode, k, v, ks, vs), m, base_pos, nh, nkv, hd)


def attention_sliding(q, mode, k, v, ks, vs, seq, window, nh, nkv, hd):
    return _attn(lib().fo_attention_sliding, q, mode, *_kv_args(mode, k, v, ks, vs), seq, window, nh, nkv, hd)


def attention_sliding_batch(qb, mode, k, v, ks, vs, m, base_pos, window, nh, nkv, hd):
    return _attn(lib().fo_attention_sliding_batch, qb, mode, *_kv_args(mode, k, v, ks, vs), m, base_pos, window, nh, nkv, hd)


# ------------------------------------------------------------------ model
def make_config(d: dict) -> FoConfig:
    return FoConfig(d["hidden_size"], d["intermediate_size"], d["num_layers"], d["num_heads"], d["num_kv_heads"],
                    d["head_dim"], d["vocab_size"], d["max_seq_len"], d["rms_norm_eps"], d["rope_theta"],
                    d["quant"], int(d.get("qkv_bias", 0)), int(d.get("sliding_window", 0) or 0),
                    (C.c_int32 * 8)(*[int(v) for v in (d.get("proj_quant") or [0] * 8)]))


class OracleModel:
    """Mirror of the generated ``model::{Weights, KVCache, forward, forward_prefill}``."""

    def __init__(self, cfg: dict, weights_bin: np.ndarray, kv_mode: int = KV_INT8, fast: bool = True):
        self.cfg = dict(cfg)
        self._c = make_config(cfg)
        self._blob = np.ascontiguousarray(weights_bin, np.uint8)  # must outlive the model
        L = lib()
        if L.fo_weights_bin_size(C.byref(self._c)) != self._blob.size:
            raise ValueError("weights.bin length does not match the configuration")
        self._m = L.fo_model_create(C.byref(self._c), _ptr(self._blob), self._blob.size)
        L.fo_model_set_fast(self._m, int(fast))
        self.kv_mode = kv_mode
        self._kv = L.fo_kv_create(self._m, kv_mode)

    def set_fast(self, fast: bool):
        lib().fo_model_set_fast(self._m, int(fast))

    def reset(self):
        lib().fo_kv_reset(self._kv)

    @property
    def len(self) -> int:
        return lib().fo_kv_len(self._kv)

    def forward(self, token: int, trace: bool = False):
        c = self.cfg
        logits = np.empty(c["vocab_size"], np.float32)
        tr = np.empty((c["num_layers"], c["hidden_size"]), np.float32) if trace else None
        rc = lib().fo_forward(self._m, self._kv, int(token), logits, _ptr(tr))
        if rc:
            raise RuntimeError(f"oracle forward failed: {rc}")
        return (logits, tr) if trace else logits

    def forward_prefill(self, tokens, trace: bool = False, force_per_token: bool = False):
        c = self.cfg
        t = np.ascontiguousarray(tokens, np.uint32)
        logits = np.empty(c["vocab_size"], np.float32)
        tr = np.empty((c["num_layers"], t.size, c["hidden_size"]), np.float32) if trace else None
        rc = lib().fo_forward_prefill(self._m, self._kv, t, t.size, logits, _ptr(tr), int(force_per_token))
        if rc:
            raise RuntimeError(f"oracle forward_prefill failed: {rc}")
        return (logits, tr) if trace else logits

    def kv_read(self, layer: int, which: int) -> np.ndarray:
        kvs = self.cfg["num_kv_heads"] * self.cfg["head_dim"]
        out = np.empty((self.len, kvs), np.float32)
        lib().fo_kv_read(self._kv, layer, which, out)
        return out

    def generate_greedy(self, prompt, n_new: int):
        """Prefill, then greedy decode with plain argmax (repeat penalty 1.0)."""
        logits = self.forward_prefill(prompt)
        out = []
        for _ in range(n_new):
            tok = argmax(logits)
            out.append(tok)
            logits = self.forward(tok)
        return np.array(out, np.uint32), logits

    def __del__(self):
        try:
            lib().fo_kv_destroy(self._kv)
            lib().fo_model_destroy(self._m)
        except Exception:
            pass
