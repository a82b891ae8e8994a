"""Model shapes of the five benchmark configurations and reduced twins for fast parity runs.

Field names follow the reference's ``ModelConfig`` (crates/forgellm-frontend/src/ir.rs:484-519).
``quant`` is 8 for GGUF Q8_0 and 4 for Q4_0.  ``max_seq_len`` is 4096 everywhere so that the
flash-attention variants are the ones selected (the reference needs ``max_seq_len > 512``,
crates/forgellm-codegen-cpu/src/emit.rs:126-128) and its 4096 cap (emit.rs:178) is not hit.
``rms_norm_eps`` is the reference's GGUF default 1e-5 (crates/forgellm-cli/src/main.rs:748-750).
"""
from __future__ import annotations


def _cfg(name, hidden, layers, nq, nkv, hd, ffn, vocab, theta, quant, bias=0, tied=False):
    return dict(name=name, hidden_size=hidden, intermediate_size=ffn, num_layers=layers, num_heads=nq,
                num_kv_heads=nkv, head_dim=hd, vocab_size=vocab, max_seq_len=4096, rms_norm_eps=1e-5,
                rope_theta=float(theta), quant=quant, qkv_bias=bias, tied=tied)


CONFIGS = {
    # SmolLM2-135M-shaped, Q8_0, tied embeddings
    "c1": _cfg("smollm2-135m-q8_0", 576, 30, 9, 3, 64, 1536, 49152, 1e5, 8, tied=True),
    # Llama-3.2-1B-shaped, Q4_0
    "c2": _cfg("llama-3.2-1b-q4_0", 2048, 16, 32, 8, 64, 8192, 128256, 5e5, 4),
    # Qwen2.5-0.5B-shaped, Q8_0, QKV bias
    "c3": _cfg("qwen2.5-0.5b-q8_0", 896, 24, 14, 2, 64, 4864, 151936, 1e6, 8, bias=1),
    # Phi-3-mini-shaped, Q8_0, MHA, head_dim 96
    "c4": _cfg("phi-3-mini-q8_0", 3072, 32, 32, 32, 96, 8192, 32064, 1e4, 8),
    # Llama-2-7B-shaped, Q4_0, MHA, head_dim 128
    "c5": _cfg("llama-2-7b-q4_0", 4096, 32, 32, 32, 128, 11008, 32000, 1e4, 4),
}


def reduced(key: str, layers: int = 2, vocab: int | None = None) -> dict:
    """Same per-layer shapes, fewer layers (and optionally a smaller vocabulary)."""
    c = dict(CONFIGS[key])
    c["num_layers"] = layers
    if vocab is not None:
        c["vocab_size"] = vocab
    c["name"] = f"{c['name']}-L{layers}" + (f"-V{vocab}" if vocab else "")
    return c


def tiny(quant: int = 8, hd: int = 64, nq: int = 4, nkv: int = 2, bias: int = 0, layers: int = 2,
         hidden: int | None = None, ffn: int = 256, vocab: int = 512) -> dict:
    """A toy decoder for CPU-speed parity cases."""
    hidden = hidden or nq * hd
    return _cfg(f"tiny-q{quant}-hd{hd}", hidden, layers, nq, nkv, hd, ffn, vocab, 1e4, quant, bias=bias)


PROJ_ORDER = ("q", "k", "v", "o", "gate", "up", "down", "lm_head")
Q4_K, Q6_K = 12, 14  # K-quants carry their GGML type numbers


def proj_quants(c: dict) -> list[int]:
    """Storage format of every projection category in PROJ_ORDER: ``c["proj_quant"][i]`` (the reference's
    ``ProjectionDTypes``, ir.rs:411-421), or ``c["quant"]`` where that is absent or 0."""
    pq = c.get("proj_quant") or [0] * 8
    return [int(v) or int(c["quant"]) for v in pq]


def with_proj_quant(c: dict, **cats: int) -> dict:
    """Copy of ``c`` with the named categories (PROJ_ORDER names) stored in the given formats."""
    d = dict(c)
    pq = list(c.get("proj_quant") or [0] * 8)
    for name, q in cats.items():
        pq[PROJ_ORDER.index(name)] = int(q)
    d["proj_quant"] = pq
    d["name"] = c["name"] + "-" + "-".join(f"{n}{q}" for n, q in cats.items())
    return d


def raw_row_bytes(quant: int, k: int) -> int:
    if quant in (Q4_K, Q6_K):
        return (k // 256) * (144 if quant == Q4_K else 210)
    return (k // 32) * (34 if quant == 8 else 18)


def weight_elems(c: dict) -> int:
    """Quantised weight elements streamed per decoded token (projections + lm_head)."""
    h, qk, kv, ff = c["hidden_size"], c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"], c["intermediate_size"]
    per_layer = h * qk + 2 * h * kv + qk * h + 3 * h * ff
    return per_layer * c["num_layers"] + h * c["vocab_size"]


def block_bytes(c: dict) -> int:
    return 34 if c["quant"] == 8 else 18


def decode_bytes_per_token(c: dict, ctx: int) -> float:
    """Algorithmic HBM bytes for one batch-1 decode step at context length ``ctx``:
    every quantised weight byte once, plus fp16 K and V of all cached positions once."""
    w = weight_elems(c) * block_bytes(c) / 32
    kv = c["num_layers"] * 2 * c["num_kv_heads"] * c["head_dim"] * ctx * 2
    return w + kv


def prefill_flops(c: dict, m: int) -> float:
    """Useful flops of an m-token causal prefill: projections for every row, QK^T and PV over
    the causal triangle, lm_head for the last row only."""
    h, qk, kv, ff = c["hidden_size"], c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"], c["intermediate_size"]
    per_layer = h * qk + 2 * h * kv + qk * h + 3 * h * ff
    gemm = 2.0 * m * per_layer * c["num_layers"]
    attn = c["num_layers"] * 4.0 * qk * m * (m + 1) / 2
    return gemm + attn + 2.0 * h * c["vocab_size"]
