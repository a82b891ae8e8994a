"""GGUF reader and weights.bin exporter (host code of the library; no GPU needed).

The parser cases restate the reference's own parser tests (crates/forgellm-frontend/src/gguf.rs:562-700: minimal v3,
several tensors with metadata, v2, bad magic, unsupported version).  The export cases write a synthetic GGUF from the
same seeded tensors `synth.make_weights_bin` uses and require the exported image to equal it byte for byte."""
import os
import struct
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from forge_llm_b200 import configs, gguf, synth  # noqa: E402
from forge_llm_b200._lib import ForgeError  # noqa: E402

MAGIC = 0x46554747
F32, F16, Q4_0, Q8_0, BF16 = 0, 1, 2, 8, 30


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def build_gguf(version, metadata, tensors, alignment=32, data=b""):
    """metadata: [(key, type_id, raw value bytes)]; tensors: [(name, dims, ggml_type, offset)]; data: tensor section."""
    out = struct.pack("<IIQQ", MAGIC, version, len(tensors), len(metadata))
    for key, tid, raw in metadata:
        out += _s(key) + struct.pack("<I", tid) + raw
    for name, dims, typ, off in tensors:
        out += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, off)
    pad = (-len(out)) % alignment
    return out + b"\0" * pad + data


def u32(v): return struct.pack("<I", v)
def f32(v): return struct.pack("<f", v)


def test_parse_minimal_v3():
    g = gguf.GgufFile(build_gguf(3, [("general.architecture", 8, _s("llama"))], [("token_embd.weight", [32000, 2048], F16, 0)]))
    assert g.version == 3
    t = g.tensors()
    assert len(t) == 1 and t[0]["name"] == "token_embd.weight" and t[0]["dims"] == [32000, 2048] and t[0]["type"] == F16
    assert t[0]["size"] == 32000 * 2048 * 2


def test_parse_several_tensors_and_block_sizes():
    g = gguf.GgufFile(build_gguf(3, [("general.architecture", 8, _s("llama")), ("llama.embedding_length", 4, u32(2048)),
                                     ("llama.attention.layer_norm_rms_epsilon", 6, f32(1e-5))],
                                 [("token_embd.weight", [32000, 2048], F16, 0), ("blk.0.attn_q.weight", [2048, 2048], Q8_0, 4096),
                                  ("blk.0.ffn_gate.weight", [5632, 2048], Q4_0, 8192)]))
    t = {x["name"]: x for x in g.tensors()}
    assert t["blk.0.attn_q.weight"]["size"] == 2048 * 2048 // 32 * 34   # 34 bytes per 32 weights
    assert t["blk.0.ffn_gate.weight"]["size"] == 5632 * 2048 // 32 * 18  # 18 bytes per 32 weights
    assert t["blk.0.attn_q.weight"]["offset"] == 4096


def test_parse_v2_and_alignment():
    g = gguf.GgufFile(build_gguf(2, [], []))
    assert g.version == 2 and g.tensors() == []
    raw = build_gguf(3, [("general.alignment", 4, u32(64))], [("a", [4], F32, 0)], alignment=64, data=b"\0" * 16)
    g = gguf.GgufFile(raw)
    assert g.data_offset % 64 == 0 and g.data_offset == len(raw) - 16
    # every metadata value type, arrays of scalars and of strings included, is skipped correctly
    arr = struct.pack("<IQ", 4, 3) + struct.pack("<III", 1, 2, 3)
    sarr = struct.pack("<IQ", 8, 2) + _s("a") + _s("bc")
    meta = [("k0", 0, b"\1"), ("k1", 1, b"\xff"), ("k2", 2, b"\1\0"), ("k3", 3, b"\1\0"), ("k5", 5, u32(7)), ("k7", 7, b"\1"),
            ("k9", 9, arr), ("k9s", 9, sarr), ("k10", 10, struct.pack("<Q", 9)), ("k11", 11, struct.pack("<q", -9)),
            ("k12", 12, struct.pack("<d", 0.5))]
    assert gguf.GgufFile(build_gguf(3, meta, [("a", [4], F32, 0)], data=b"\0" * 16)).tensors()[0]["name"] == "a"


def test_rejects_bad_files():
    with pytest.raises(ForgeError):
        gguf.GgufFile(struct.pack("<I", 0xDEADBEEF) + b"\0" * 28)           # bad magic
    with pytest.raises(ForgeError):
        gguf.GgufFile(struct.pack("<IIQQ", MAGIC, 99, 0, 0))                # unsupported version
    with pytest.raises(ForgeError):
        gguf.GgufFile(build_gguf(3, [], [("t", [1, 1, 1, 1, 1], F32, 0)]))   # five dimensions
    good = build_gguf(3, [("general.architecture", 8, _s("llama"))], [("token_embd.weight", [8, 8], F16, 0)])
    for cut in (3, 11, 30, len(good) - 40):
        with pytest.raises(ForgeError):
            gguf.GgufFile(good[:cut]).tensors()                              # truncated header / tables


def synthetic_gguf(c: dict, tied: bool, embed_type: int = F32, arch: str = "llama"):
    """A GGUF file holding exactly the tensors of synth.make_weights_bin(c), under GGUF names."""
    blob = synth.make_weights_bin(c)
    h, qk, kv = c["hidden_size"], c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"]
    ff, V = c["intermediate_size"], c["vocab_size"]
    pq = configs.proj_quants(c)
    gtype = {8: Q8_0, 4: Q4_0, 12: 12, 14: 14}  # the K-quants carry their GGML type numbers
    off = 0

    def proj(name, dims, cat, n, k):
        return (name, dims, gtype[pq[cat]], take(n * configs.raw_row_bytes(pq[cat], k)))

    def take(n):
        nonlocal off
        b = blob[off:off + n].tobytes()
        off += n
        return b

    tensors = []
    embed = np.frombuffer(take(V * h * 4), np.float32)
    if embed_type == F16:
        tensors.append(("token_embd.weight", [h, V], F16, embed.astype(np.float16).tobytes()))
    else:
        tensors.append(("token_embd.weight", [h, V], F32, embed.tobytes()))
    for l in range(c["num_layers"]):
        p = f"blk.{l}."
        tensors.append((p + "attn_norm.weight", [h], F32, take(h * 4)))
        tensors.append(proj(p + "attn_q.weight", [h, qk], 0, qk, h))
        tensors.append(proj(p + "attn_k.weight", [h, kv], 1, kv, h))
        tensors.append(proj(p + "attn_v.weight", [h, kv], 2, kv, h))
        if c.get("qkv_bias"):
            tensors.append((p + "attn_q.bias", [qk], F32, take(qk * 4)))
            tensors.append((p + "attn_k.bias", [kv], F32, take(kv * 4)))
            tensors.append((p + "attn_v.bias", [kv], F32, take(kv * 4)))
        tensors.append(proj(p + "attn_output.weight", [qk, h], 3, h, qk))
        tensors.append((p + "ffn_norm.weight", [h], F32, take(h * 4)))
        tensors.append(proj(p + "ffn_gate.weight", [h, ff], 4, ff, h))
        tensors.append(proj(p + "ffn_up.weight", [h, ff], 5, ff, h))
        tensors.append(proj(p + "ffn_down.weight", [ff, h], 6, h, ff))
    tensors.append(("output_norm.weight", [h], F32, take(h * 4)))
    head = proj("output.weight", [h, V], 7, V, h)
    assert off == blob.size
    if not tied:
        tensors.append(head)
    data, table = b"", []
    for name, dims, typ, raw in tensors[::-1]:  # file order differs from export order on purpose
        data += b"\0" * ((-len(data)) % 32)
        table.append((name, dims, typ, len(data)))
        data += raw
    meta = [("general.architecture", 8, _s(arch)), (f"{arch}.embedding_length", 4, u32(h)), (f"{arch}.block_count", 4, u32(c["num_layers"])),
            (f"{arch}.attention.head_count", 4, u32(c["num_heads"])), (f"{arch}.attention.head_count_kv", 4, u32(c["num_kv_heads"])),
            (f"{arch}.feed_forward_length", 4, u32(ff)), (f"{arch}.vocab_size", 4, u32(V)), (f"{arch}.context_length", 4, u32(c["max_seq_len"])),
            (f"{arch}.attention.layer_norm_rms_epsilon", 6, f32(c["rms_norm_eps"])), (f"{arch}.rope.freq_base", 6, f32(c["rope_theta"]))]
    return build_gguf(3, meta, table, data=data), blob, embed


@pytest.mark.parametrize("quant,bias", [(8, 0), (4, 0), (4, 1)])
def test_export_equals_the_reference_order_image(quant, bias):
    c = configs.tiny(quant, hd=64, nq=4, nkv=2, bias=bias, layers=2)
    raw, blob, _ = synthetic_gguf(c, tied=False, arch="qwen2" if bias else "llama")
    g = gguf.GgufFile(raw)
    got = g.config()
    for k in ("hidden_size", "intermediate_size", "num_layers", "num_heads", "num_kv_heads", "head_dim", "vocab_size", "max_seq_len", "quant", "qkv_bias"):
        assert got[k] == c[k] if k != "qkv_bias" else got[k] == bias, k
    assert abs(got["rms_norm_eps"] - c["rms_norm_eps"]) < 1e-12 and got["rope_theta"] == c["rope_theta"]
    assert np.array_equal(g.weights_bin(), blob)


def test_k_quant_file_keeps_its_per_category_formats(oracle):
    """A Q4_K_M-shaped file (main.rs:603-607): Q4_K for q/k/o/gate/up, Q6_K for v/down/output.  The configuration
    reports the mix, the projections are exported verbatim, and a K-quant embedding is dequantised to f32."""
    base = configs.tiny(12, hd=64, nq=4, nkv=2, layers=2, ffn=512)
    c = configs.with_proj_quant(base, v=14, down=14, lm_head=14)
    raw, blob, _ = synthetic_gguf(c, tied=False)
    g = gguf.GgufFile(raw)
    got = g.config()
    assert got["quant"] == 12 and got["proj_quant"] == [12, 12, 14, 12, 12, 12, 14, 14]
    assert np.array_equal(g.weights_bin(), blob)
    # uniform Q6_K projections under the same vote rules: other block formats count towards Q8_0 (main.rs:512-536),
    # so the model format is Q8_0 and every category reports Q6_K
    c6 = configs.tiny(14, hd=64, nq=4, nkv=2, layers=1, ffn=512)
    raw6, blob6, _ = synthetic_gguf(c6, tied=False)
    got6 = gguf.GgufFile(raw6).config()
    assert got6["quant"] == 8 and got6["proj_quant"] == [14] * 8
    assert np.array_equal(gguf.GgufFile(raw6).weights_bin(), blob6)


def test_tensors_off_their_category_format_are_requantised(oracle):
    """A real Q4_K_M file alternates Q4_K and Q6_K for attn_v / ffn_down from layer to layer.  The category takes the
    majority format (ties go to the higher precision, main.rs:628-660) and the other tensors are dequantised and
    quantised again in it (weight_loader.rs:193-218)."""
    base = configs.tiny(12, hd=64, nq=4, nkv=2, layers=2, ffn=512)
    c = configs.with_proj_quant(base, v=14, down=14, lm_head=14)
    raw, blob, _ = synthetic_gguf(c, tied=False)
    g0 = gguf.GgufFile(raw)
    h, kv, ff = c["hidden_size"], c["num_kv_heads"] * c["head_dim"], c["intermediate_size"]
    # layer 1 keeps attn_v and ffn_down as Q4_K (1:1 tie -> Q6_K wins), layer 0 has them in Q6_K
    rng = np.random.default_rng(77)
    swapped = {"blk.1.attn_v.weight": synth.random_kquant(12, rng, kv, h, 0.02), "blk.1.ffn_down.weight": synth.random_kquant(12, rng, h, ff, 0.02)}
    tensors, data = [], b""
    for t in g0.tensors():
        payload = raw[g0.data_offset + t["offset"]:g0.data_offset + t["offset"] + t["size"]]
        typ = t["type"]
        if t["name"] in swapped:
            payload, typ = swapped[t["name"]].tobytes(), 12
        data += b"\0" * ((-len(data)) % 32)
        tensors.append((t["name"], t["dims"], typ, len(data)))
        data += payload
    meta = [("general.architecture", 8, _s("llama")), ("llama.embedding_length", 4, u32(h)), ("llama.block_count", 4, u32(2)),
            ("llama.attention.head_count", 4, u32(c["num_heads"])), ("llama.attention.head_count_kv", 4, u32(c["num_kv_heads"])),
            ("llama.feed_forward_length", 4, u32(ff)), ("llama.vocab_size", 4, u32(c["vocab_size"])),
            ("llama.context_length", 4, u32(c["max_seq_len"]))]
    g = gguf.GgufFile(build_gguf(3, meta, tensors, data=data))
    assert g.config()["proj_quant"] == [12, 12, 14, 12, 12, 12, 14, 14]
    out = g.weights_bin()
    assert out.size == blob.size
    # locate layer 1's v_proj and down_proj in the image and compare with dequantise -> quantise of the Q4_K payloads
    V, qk = c["vocab_size"], c["num_heads"] * c["head_dim"]
    rb = configs.raw_row_bytes
    per_layer = h * 4 + qk * rb(12, h) + kv * rb(12, h) + kv * rb(14, h) + h * rb(12, qk) + h * 4 + 2 * ff * rb(12, h) + h * rb(14, ff)
    l1 = V * h * 4 + per_layer
    v_off = l1 + h * 4 + qk * rb(12, h) + kv * rb(12, h)
    want_v = oracle.quantize_kquant(14, oracle.dequant_kquant(12, swapped["blk.1.attn_v.weight"], kv * h))
    assert np.array_equal(out[v_off:v_off + kv * rb(14, h)], want_v)
    d_off = l1 + per_layer - h * rb(14, ff)
    want_d = oracle.quantize_kquant(14, oracle.dequant_kquant(12, swapped["blk.1.ffn_down.weight"], h * ff))
    assert np.array_equal(out[d_off:d_off + h * rb(14, ff)], want_d)
    # everything else is the verbatim image
    keep = np.ones(out.size, bool)
    keep[v_off:v_off + kv * rb(14, h)] = False
    keep[d_off:d_off + h * rb(14, ff)] = False
    assert np.array_equal(out[keep], blob[keep])


def test_k_quant_embedding_is_dequantised_and_tied_head_stays_raw(oracle):
    c = configs.tiny(12, hd=64, nq=4, nkv=2, layers=1, ffn=512)
    V, h = c["vocab_size"], c["hidden_size"]
    raw, blob, _ = synthetic_gguf(c, tied=False)
    # rebuild the file with the head tensor renamed to the embedding: a tied model whose token_embd is Q4_K
    head_bytes = V * configs.raw_row_bytes(12, h)
    head = blob[-head_bytes:]
    g0 = gguf.GgufFile(raw)
    tensors, data = [], b""
    for t in g0.tensors():
        name, typ, dims, off, size = t["name"], t["type"], t["dims"], t["offset"], t["size"]
        if name == "output.weight":
            continue
        payload = head.tobytes() if name == "token_embd.weight" else raw[g0.data_offset + off:g0.data_offset + off + size]
        data += b"\0" * ((-len(data)) % 32)
        tensors.append((name, dims, 12 if name == "token_embd.weight" else typ, len(data)))
        data += payload
    meta = [("general.architecture", 8, _s("llama")), ("llama.embedding_length", 4, u32(h)), ("llama.block_count", 4, u32(1)),
            ("llama.attention.head_count", 4, u32(c["num_heads"])), ("llama.attention.head_count_kv", 4, u32(c["num_kv_heads"])),
            ("llama.feed_forward_length", 4, u32(c["intermediate_size"])), ("llama.vocab_size", 4, u32(V))]
    out = gguf.GgufFile(build_gguf(3, meta, tensors, data=data)).weights_bin()
    assert np.array_equal(out[:V * h * 4].view(np.float32), oracle.dequant_kquant(12, head, V * h))
    assert np.array_equal(out[-head_bytes:], head)


@pytest.mark.parametrize("quant", [8, 4])
def test_tied_head_and_f16_embedding(quant, oracle):
    c = configs.tiny(quant, hd=64, nq=4, nkv=2, layers=1)
    raw, blob, embed = synthetic_gguf(c, tied=True, embed_type=F16)
    out = gguf.GgufFile(raw).weights_bin()
    V, h = c["vocab_size"], c["hidden_size"]
    e16 = embed.astype(np.float16).astype(np.float32)
    assert np.array_equal(out[:V * h * 4].view(np.float32), e16)             # embedding widened from f16
    head_bytes = V * h // 32 * (34 if quant == 8 else 18)
    assert np.array_equal(out[V * h * 4:-head_bytes], blob[V * h * 4:-head_bytes])  # everything between is verbatim
    # head = the embedding re-quantised with the exporter's own rules (the CPU restatement's quantisers)
    want = oracle.quantize_q8_0(e16) if quant == 8 else oracle.quantize_q4_0(e16, rule="ref")
    assert np.array_equal(out[-head_bytes:], np.asarray(want).reshape(-1).view(np.uint8))


def test_defaults_and_unsupported():
    # missing optional keys take the reference's defaults: kv heads = heads, ffn = 4 * hidden, eps 1e-5, theta 1e4, ctx 2048
    meta = [("general.architecture", 8, _s("llama")), ("llama.embedding_length", 4, u32(256)), ("llama.block_count", 4, u32(1)),
            ("llama.attention.head_count", 4, u32(4)), ("tokenizer.ggml.tokens", 9, struct.pack("<IQ", 8, 3) + _s("a") + _s("b") + _s("c"))]
    g = gguf.GgufFile(build_gguf(3, meta, [("blk.0.attn_q.weight", [256, 256], Q8_0, 0)], data=b"\0" * (256 * 256 // 32 * 34)))
    c = g.config()
    assert (c["num_kv_heads"], c["intermediate_size"], c["vocab_size"], c["max_seq_len"], c["head_dim"]) == (4, 1024, 3, 2048, 64)
    assert abs(c["rms_norm_eps"] - 1e-5) < 1e-12 and c["rope_theta"] == 10000.0 and c["quant"] == 8
    with pytest.raises(ForgeError):
        g.weights_bin()  # tensors are missing
    meta[0] = ("general.architecture", 8, _s("gemma"))
    with pytest.raises(ForgeError):
        gguf.GgufFile(build_gguf(3, meta, [("blk.0.attn_q.weight", [256, 256], Q8_0, 0)], data=b"\0" * 69632)).config()


def test_phi3_fused_tensors_are_split():
    """Phi-3 files carry q|k|v as one attn_qkv tensor and gate|up as one double-height ffn_up tensor
    (weight_loader.rs:543-582): the exported image must equal the one of the unfused file."""
    c = configs.tiny(8, hd=64, nq=4, nkv=4, layers=2)
    raw, blob, _ = synthetic_gguf(c, tied=False, arch="phi3")
    g = gguf.GgufFile(raw)
    t = {x["name"]: x for x in g.tensors()}
    off0 = g.data_offset
    table, data = [], b""
    def add(name, dims, typ, payload):
        nonlocal data
        data += b"\0" * ((-len(data)) % 32)
        table.append((name, dims, typ, len(data)))
        data += payload
    def payload(name):
        return raw[off0 + t[name]["offset"]: off0 + t[name]["offset"] + t[name]["size"]]
    h, ff = c["hidden_size"], c["intermediate_size"]
    rows_qkv = (c["num_heads"] + 2 * c["num_kv_heads"]) * c["head_dim"]
    for name, x in t.items():
        if name.endswith(("attn_k.weight", "attn_v.weight", "ffn_gate.weight")):
            continue
        if name.endswith("attn_q.weight"):
            p = name[:-len("attn_q.weight")]
            add(p + "attn_qkv.weight", [h, rows_qkv], Q8_0, payload(p + "attn_q.weight") + payload(p + "attn_k.weight") + payload(p + "attn_v.weight"))
        elif name.endswith("ffn_up.weight"):
            p = name[:-len("ffn_up.weight")]
            add(name, [h, 2 * ff], Q8_0, payload(p + "ffn_gate.weight") + payload(name))
        else:
            add(name, x["dims"], x["type"], payload(name))
    arch = "phi3"
    meta = [("general.architecture", 8, _s(arch)), (f"{arch}.embedding_length", 4, u32(h)), (f"{arch}.block_count", 4, u32(c["num_layers"])),
            (f"{arch}.attention.head_count", 4, u32(c["num_heads"])), (f"{arch}.attention.head_count_kv", 4, u32(c["num_kv_heads"])),
            (f"{arch}.feed_forward_length", 4, u32(ff)), (f"{arch}.vocab_size", 4, u32(c["vocab_size"])),
            (f"{arch}.context_length", 4, u32(c["max_seq_len"])), (f"{arch}.attention.layer_norm_rms_epsilon", 6, f32(c["rms_norm_eps"])),
            (f"{arch}.rope.freq_base", 6, f32(c["rope_theta"]))]
    fused = gguf.GgufFile(build_gguf(3, meta, table, data=data))
    assert fused.config()["num_kv_heads"] == 4
    assert np.array_equal(fused.weights_bin(), blob)


# ---- tensor -> f32 for the block formats the exporter reads (dequantize, weight_loader.rs:809-826)
def _one_tensor_file(typ, dims, payload):
    return gguf.GgufFile(build_gguf(3, [("general.architecture", 8, _s("llama"))], [("t.weight", dims, typ, 0)], data=bytes(payload)))


def _scale_min_k4(j, sc):
    if j < 4:
        return int(sc[j] & 63), int(sc[j + 4] & 63)
    return int((sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4)), int((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4))


def _dq_q4_1(raw, n):  # weight_loader.rs:931-966
    b = np.frombuffer(raw, np.uint8).reshape(-1, 20)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    m = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    lo, hi = (b[:, 4:] & 0x0F).astype(np.float32), (b[:, 4:] >> 4).astype(np.float32)
    return (np.concatenate([lo, hi], axis=1) * d + m).reshape(-1)[:n]


def _dq_q5_k(raw, n):  # weight_loader.rs:1071-1140
    out = np.zeros(n, np.float32)
    blocks = np.frombuffer(raw, np.uint8).reshape(-1, 176)
    for sb, blk in enumerate(blocks):
        d = blk[0:2].copy().view(np.float16).astype(np.float32)[0]
        dmin = blk[2:4].copy().view(np.float16).astype(np.float32)[0]
        sc, qh, qs = blk[4:16], blk[16:48], blk[48:176]
        for j in range(8):
            s6, m6 = _scale_min_k4(j, sc)
            by = qs[(j >> 1) * 32:(j >> 1) * 32 + 32]
            q = ((by >> 4) if j & 1 else (by & 0x0F)).astype(np.uint32) + (((qh >> j) & 1).astype(np.uint32) << 4)
            out[sb * 256 + j * 32:sb * 256 + j * 32 + 32] = (d * np.float32(s6)) * q.astype(np.float32) - dmin * np.float32(m6)
    return out


def test_dequant_q4_1_and_q5_k_known_answers():
    # weight_loader.rs:3245-3260: scale 2, min 1, all nibbles 0 -> 1.0
    blk = np.zeros(20, np.uint8)
    blk[0:2] = np.frombuffer(np.uint16(0x4000).tobytes(), np.uint8)
    blk[2:4] = np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8)
    assert np.all(_one_tensor_file(3, [32], blk).tensor_f32(0) == 1.0)
    # weight_loader.rs:3509-3533: d = 1, sub-block 0 scale 1, qs[0] low nibble 3, qh[0] bit 0 -> 3 + 16 = 19
    b = np.zeros(176, np.uint8)
    b[0:2] = np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8)
    b[4], b[16], b[48] = 1, 0x01, 0x03
    assert _one_tensor_file(13, [256], b).tensor_f32(0)[0] == 19.0
    # weight_loader.rs:3536-3558: sub-block 1 scale 2, qs[0] high nibble 7, qh[0] bit 1 -> 2 * (7 + 16) = 46 at element 32
    b = np.zeros(176, np.uint8)
    b[0:2] = np.frombuffer(np.uint16(0x3C00).tobytes(), np.uint8)
    b[5], b[16], b[48] = 2, 0x02, 0x70
    assert _one_tensor_file(13, [256], b).tensor_f32(0)[32] == 46.0


def test_tensor_to_f32_matches_the_restatements(oracle):
    rng = np.random.default_rng(21)
    n = 256 * 6

    def blocks(count, size, scale_cols, mag):
        raw = rng.integers(0, 256, (count, size), dtype=np.uint8)
        for c in scale_cols:
            raw[:, c:c + 2] = (mag * (0.5 + rng.random(count))).astype(np.float16).view(np.uint8).reshape(count, 2)
        return raw.reshape(-1)

    q41 = blocks(n // 32, 20, (0, 2), 0.01)
    assert np.array_equal(_one_tensor_file(3, [n], q41).tensor_f32(0), _dq_q4_1(q41.tobytes(), n))
    q5k = blocks(n // 256, 176, (0, 2), 1e-4)
    assert np.array_equal(_one_tensor_file(13, [n], q5k).tensor_f32(0), _dq_q5_k(q5k.tobytes(), n))
    q4k = synth.random_kquant(12, rng, 1, n, 0.02)
    assert np.array_equal(_one_tensor_file(12, [n], q4k).tensor_f32(0), oracle.dequant_kquant(12, q4k, n))
    q6k = synth.random_kquant(14, rng, 1, n, 0.02)
    assert np.array_equal(_one_tensor_file(14, [n], q6k).tensor_f32(0), oracle.dequant_kquant(14, q6k, n))
    q80 = oracle.quantize_q8_0(rng.standard_normal(n).astype(np.float32))
    assert np.array_equal(_one_tensor_file(8, [n], q80).tensor_f32(0), oracle.dequant_q8_0(q80, n))
    q40 = oracle.quantize_q4_0(rng.standard_normal(n).astype(np.float32))
    assert np.array_equal(_one_tensor_file(2, [n], q40).tensor_f32(0), oracle.dequant_q4_0(q40, n))
