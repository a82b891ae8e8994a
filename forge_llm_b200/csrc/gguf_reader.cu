// GGUF reader and weights.bin exporter (host code only): lets a GGUF checkpoint drive the backend directly.
// Follows the reference's parser (crates/forgellm-frontend/src/gguf.rs:484-551; type table :207-258), its
// GGUF -> ModelConfig rules (crates/forgellm-cli/src/main.rs:689-811, dtype vote :479-560), its tensor name map
// (crates/forgellm-frontend/src/weight_loader.rs:400-441) and the write order of `export-weights`
// (crates/forgellm-cli/src/main.rs:2506-2757) for the two block formats of this backend, Q8_0 and Q4_0:
//   embed_tokens as f32 | per layer: input norm f32, q, k, v blocks, (q, k, v bias f32), o blocks, post-attention
//   norm f32, gate, up, down blocks | final norm f32 | lm_head blocks (the embedding, re-quantised, when the file
//   has no output.weight).
// Everything is bounds-checked against the mapped length; nothing is read past it.
#include <cstdint>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace {

using namespace forge;

constexpr uint32_t kMagic = 0x46554747u;  // "GGUF"
constexpr uint64_t kDefaultAlignment = 32;
enum : int32_t { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30 };

struct MetaValue {
    int type = -1;         // GGUF value type id (0..12)
    uint64_t u = 0;        // integers, bool
    double f = 0.0;        // floats
    std::string s;         // strings
    int elem_type = -1;    // arrays
    uint64_t count = 0;    // arrays: number of elements
};

struct TensorInfo {
    std::string name;
    int n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    int32_t type = 0;
    uint64_t offset = 0;  // from the start of the tensor data section
    uint64_t numel() const { return dims[0] * dims[1] * dims[2] * dims[3]; }
};

// elements per block and bytes per block (gguf.rs:207-258); 0 = a type this reader does not size
bool type_layout(int32_t t, uint64_t& block, uint64_t& bytes) {
    switch (t) {
        case 0: block = 1; bytes = 4; return true;     // F32
        case 1: block = 1; bytes = 2; return true;     // F16
        case 2: block = 32; bytes = 18; return true;   // Q4_0
        case 3: block = 32; bytes = 20; return true;   // Q4_1
        case 6: block = 32; bytes = 22; return true;   // Q5_0
        case 7: block = 32; bytes = 24; return true;   // Q5_1
        case 8: block = 32; bytes = 34; return true;   // Q8_0
        case 9: block = 32; bytes = 40; return true;   // Q8_1
        case 10: block = 256; bytes = 84; return true;   // Q2_K
        case 11: block = 256; bytes = 110; return true;  // Q3_K
        case 12: block = 256; bytes = 144; return true;  // Q4_K
        case 13: block = 256; bytes = 176; return true;  // Q5_K
        case 14: block = 256; bytes = 210; return true;  // Q6_K
        case 15: block = 256; bytes = 292; return true;  // Q8_K
        case 24: block = 1; bytes = 1; return true;    // I8
        case 25: block = 1; bytes = 2; return true;    // I16
        case 26: block = 1; bytes = 4; return true;    // I32
        case 27: block = 1; bytes = 8; return true;    // I64
        case 28: block = 1; bytes = 8; return true;    // F64
        case 30: block = 1; bytes = 2; return true;    // BF16
        default: return false;
    }
}

struct Reader {
    const uint8_t* p;
    size_t len, pos = 0;
    bool ok = true;
    bool need(size_t n) {
        if (!ok || n > len - pos) { ok = false; return false; }
        return true;
    }
    template <typename T> T get() {
        T v{};
        if (need(sizeof(T))) { memcpy(&v, p + pos, sizeof(T)); pos += sizeof(T); }
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        std::string s;
        if (ok && n <= len - pos) { s.assign(reinterpret_cast<const char*>(p + pos), size_t(n)); pos += size_t(n); }
        else ok = false;
        return s;
    }
};

size_t scalar_size(int t) {
    switch (t) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}

bool read_value(Reader& r, int type, MetaValue& v, int depth) {
    v.type = type;
    switch (type) {
        case 0: v.u = r.get<uint8_t>(); break;
        case 1: v.u = uint64_t(int64_t(r.get<int8_t>())); break;
        case 2: v.u = r.get<uint16_t>(); break;
        case 3: v.u = uint64_t(int64_t(r.get<int16_t>())); break;
        case 4: v.u = r.get<uint32_t>(); break;
        case 5: v.u = uint64_t(int64_t(r.get<int32_t>())); break;
        case 6: v.f = r.get<float>(); break;
        case 7: v.u = r.get<uint8_t>() != 0; break;
        case 8: v.s = r.str(); break;
        case 9: {
            v.elem_type = int(r.get<uint32_t>());
            v.count = r.get<uint64_t>();
            if (!r.ok) return false;
            if (const size_t sz = scalar_size(v.elem_type)) {      // skip fixed-size elements in one step
                if (v.count > (r.len - r.pos) / sz) { r.ok = false; return false; }
                r.pos += size_t(v.count) * sz;
            } else if (v.elem_type == 8) {
                for (uint64_t i = 0; i < v.count && r.ok; ++i) {   // strings: only the lengths matter here
                    const uint64_t n = r.get<uint64_t>();
                    if (!r.ok || n > r.len - r.pos) { r.ok = false; return false; }
                    r.pos += size_t(n);
                }
            } else if (v.elem_type == 9 && depth < 4) {
                for (uint64_t i = 0; i < v.count && r.ok; ++i) { MetaValue e; if (!read_value(r, 9, e, depth + 1)) return false; }
            } else {
                r.ok = false;
            }
            break;
        }
        case 10: v.u = r.get<uint64_t>(); break;
        case 11: v.u = uint64_t(r.get<int64_t>()); break;
        case 12: v.f = r.get<double>(); break;
        default: return false;
    }
    return r.ok;
}

float f16_to_f32(uint16_t h) { __half_raw r; r.x = h; return __half2float(__half(r)); }
float bf16_to_f32(uint16_t h) { uint32_t u = uint32_t(h) << 16; float f; memcpy(&f, &u, 4); return f; }

// GGUF tensor name -> HuggingFace name (weight_loader.rs:400-441)
std::string hf_name(const std::string& n) {
    if (n == "token_embd.weight") return "model.embed_tokens.weight";
    if (n == "output_norm.weight") return "model.norm.weight";
    if (n == "output.weight") return "lm_head.weight";
    if (n.rfind("blk.", 0) == 0) {
        const size_t dot = n.find('.', 4);
        if (dot != std::string::npos) {
            const std::string layer = n.substr(4, dot - 4), suffix = n.substr(dot + 1);
            static const std::unordered_map<std::string, std::string> map = {
                {"attn_norm.weight", "input_layernorm.weight"},       {"attn_q.weight", "self_attn.q_proj.weight"},
                {"attn_k.weight", "self_attn.k_proj.weight"},         {"attn_v.weight", "self_attn.v_proj.weight"},
                {"attn_q.bias", "self_attn.q_proj.bias"},             {"attn_k.bias", "self_attn.k_proj.bias"},
                {"attn_v.bias", "self_attn.v_proj.bias"},             {"attn_output.weight", "self_attn.o_proj.weight"},
                {"attn_qkv.weight", "self_attn.qkv_proj.weight"},     {"ffn_norm.weight", "post_attention_layernorm.weight"},
                {"ffn_gate.weight", "mlp.gate_proj.weight"},          {"ffn_up.weight", "mlp.up_proj.weight"},
                {"ffn_down.weight", "mlp.down_proj.weight"}};
            auto it = map.find(suffix);
            return "model.layers." + layer + "." + (it == map.end() ? suffix : it->second);
        }
    }
    return n;
}

}  // namespace

struct ForgeGguf {
    const uint8_t* data = nullptr;
    size_t len = 0;
    uint32_t version = 0;
    uint64_t alignment = kDefaultAlignment, data_offset = 0;
    std::unordered_map<std::string, MetaValue> meta;
    std::vector<TensorInfo> tensors;
    std::unordered_map<std::string, size_t> by_hf_name;

    const MetaValue* get(const std::string& k) const { auto it = meta.find(k); return it == meta.end() ? nullptr : &it->second; }
    bool get_u32(const std::string& k, uint64_t& out) const { const MetaValue* v = get(k); if (!v || v->type != 4) return false; out = v->u; return true; }
    bool get_u64(const std::string& k, uint64_t& out) const { const MetaValue* v = get(k); if (!v || (v->type != 4 && v->type != 10)) return false; out = v->u; return true; }
    bool get_f32(const std::string& k, float& out) const { const MetaValue* v = get(k); if (!v || v->type != 6) return false; out = float(v->f); return true; }
    const TensorInfo* tensor(const std::string& hf) const { auto it = by_hf_name.find(hf); return it == by_hf_name.end() ? nullptr : &tensors[it->second]; }
    bool span(const TensorInfo& t, const uint8_t*& ptr, uint64_t& bytes) const {
        uint64_t block, tsz;
        if (!type_layout(t.type, block, tsz)) return false;
        bytes = (t.numel() + block - 1) / block * tsz;
        const uint64_t start = data_offset + t.offset;
        if (start > len || bytes > len - start) return false;
        ptr = data + start;
        return true;
    }
};

namespace {

// the projection dtype of the model: majority vote over the projection tensors (detect_gguf_dtype, main.rs:479-556).
// Other block formats count towards Q8_0 as there; a dense (f16 / f32) majority has no kernel in this backend.
int32_t vote_quant(const ForgeGguf& g, int32_t& quant) {
    size_t q8 = 0, q4 = 0, q4k = 0, dense = 0;
    for (const TensorInfo& t : g.tensors) {
        const std::string& n = t.name;
        const bool proj = n.find(".weight") != std::string::npos && n.find("token_embd") == std::string::npos &&
                          n.find("output.weight") == std::string::npos && n.find("_norm") == std::string::npos;
        if (!proj) continue;
        if (t.type == T_Q8_0) ++q8;
        else if (t.type == T_Q4_0) ++q4;
        else if (t.type == T_Q4_K) ++q4k;
        else if (t.type == T_F32 || t.type == T_F16 || t.type == T_BF16) ++dense;
        else if (t.type == 3 || (t.type >= 6 && t.type <= 23) || t.type == 29) ++q8;  // Q4_1, Q5_x, Q8_1, the other K- and I-quants (IQ1_M = 29)
    }
    const size_t total = q8 + q4 + q4k + dense;
    if (total > 0 && q4k > total / 2) quant = FORGE_Q4_K;
    else if (total > 0 && q8 > total / 2) quant = FORGE_Q8_0;
    else if (total > 0 && q4 > total / 2) quant = FORGE_Q4_0;
    else { set_error("GGUF projections have no Q8_0 / Q4_0 / Q4_K majority (%zu dense, %zu Q8_0-class, %zu Q4_0, %zu Q4_K)", dense, q8, q4, q4k); return FORGE_ERR_UNSUPPORTED; }
    return FORGE_OK;
}

// Storage format per projection category (detect_gguf_proj_dtypes, main.rs:603-690): the majority format of the
// category's tensors, count ties going to the higher precision (dense > Q8_0 > Q6_K > Q4_K > Q4_0); formats without
// a kernel do not vote; an empty category, or one with a dense majority (which the exporter quantises), takes the
// model's format; without an output tensor the head follows the embedding.  pq: q, k, v, o, gate, up, down, lm_head.
void detect_proj_quants(const ForgeGguf& g, int32_t fallback, int32_t (&pq)[8]) {
    static const char* const suffix[8] = {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                                          "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
                                          "mlp.down_proj.weight", "lm_head.weight"};
    auto pick = [&](auto&& in_category) -> int32_t {
        // index: 0 dense, 1 Q8_0, 2 Q6_K, 3 Q4_K, 4 Q4_0 (precision order)
        size_t count[5] = {0, 0, 0, 0, 0};
        static const int32_t fmt[5] = {0, FORGE_Q8_0, FORGE_Q6_K, FORGE_Q4_K, FORGE_Q4_0};
        for (const TensorInfo& t : g.tensors) {
            if (!in_category(hf_name(t.name))) continue;
            if (t.type == T_F32 || t.type == T_F16 || t.type == T_BF16) ++count[0];
            else if (t.type == T_Q8_0) ++count[1];
            else if (t.type == T_Q6_K) ++count[2];
            else if (t.type == T_Q4_K) ++count[3];
            else if (t.type == T_Q4_0) ++count[4];
        }
        int best = -1;
        for (int i = 0; i < 5; ++i) if (count[i] > 0 && (best < 0 || count[i] > count[best])) best = i;
        return best <= 0 ? fallback : fmt[best];
    };
    for (int i = 0; i < 8; ++i) {
        const std::string sfx = suffix[i];
        pq[i] = pick([&](const std::string& n) {
            if (i == 7) return n == sfx;
            return n.compare(0, 13, "model.layers.") == 0 && n.size() > sfx.size() && n.compare(n.size() - sfx.size(), sfx.size(), sfx) == 0 &&
                   n[n.size() - sfx.size() - 1] == '.';
        });
    }
    if (!g.tensor("lm_head.weight")) pq[7] = pick([](const std::string& n) { return n == "model.embed_tokens.weight"; });
    // fused Phi-3 tensors carry several categories at once
    const int32_t qkv = pick([](const std::string& n) { return n.find(".self_attn.qkv_proj.weight") != std::string::npos; });
    if (!g.tensor("model.layers.0.self_attn.q_proj.weight") && g.tensor("model.layers.0.self_attn.qkv_proj.weight")) pq[0] = pq[1] = pq[2] = qkv;
    if (!g.tensor("model.layers.0.mlp.gate_proj.weight")) pq[4] = pq[5];
}

// dense tensor -> f32 (F32 / F16 / BF16), or Q8_0 blocks -> f32 (dequantize_q8_0, weight_loader.rs:860-888)
// `first`: first element of the range [first, first + expect) inside the tensor (a part of a fused tensor)
int32_t to_f32(const ForgeGguf& g, const TensorInfo& t, uint64_t expect, std::vector<float>& out, uint64_t first = 0) {
    const uint8_t* p; uint64_t bytes;
    if (!g.span(t, p, bytes)) { set_error("tensor %s extends past the end of the file", t.name.c_str()); return FORGE_ERR_SHAPE; }
    if (first > t.numel() || expect > t.numel() - first) { set_error("tensor %s has %llu elements, expected %llu from %llu", t.name.c_str(), (unsigned long long)t.numel(), (unsigned long long)expect, (unsigned long long)first); return FORGE_ERR_SHAPE; }
    uint64_t block, tsz;
    type_layout(t.type, block, tsz);
    if (first % block) { set_error("tensor %s: part does not start on a block", t.name.c_str()); return FORGE_ERR_SHAPE; }
    p += first / block * tsz;
    out.resize(size_t(expect));
    if (t.type == T_F32) { memcpy(out.data(), p, size_t(expect) * 4); return FORGE_OK; }
    if (t.type == T_F16 || t.type == T_BF16) {
        for (uint64_t i = 0; i < expect; ++i) {
            uint16_t h; memcpy(&h, p + 2 * i, 2);
            out[size_t(i)] = t.type == T_F16 ? f16_to_f32(h) : bf16_to_f32(h);
        }
        return FORGE_OK;
    }
    if (t.type == T_Q8_0 && expect % 32 == 0) {
        for (uint64_t b = 0; b < expect / 32; ++b) {
            uint16_t h; memcpy(&h, p + 34 * b, 2);
            const float d = f16_to_f32(h);
            for (int i = 0; i < 32; ++i) out[size_t(b * 32 + i)] = float(int8_t(p[34 * b + 2 + i])) * d;
        }
        return FORGE_OK;
    }
    if (t.type == T_Q4_0 && expect % 32 == 0) {  // weight_loader.rs:893-926
        for (uint64_t b = 0; b < expect / 32; ++b) {
            uint16_t h; memcpy(&h, p + 18 * b, 2);
            const float d = f16_to_f32(h);
            for (int i = 0; i < 16; ++i) {
                out[size_t(b * 32 + i)] = float(int(p[18 * b + 2 + i] & 0x0F) - 8) * d;
                out[size_t(b * 32 + i + 16)] = float(int(p[18 * b + 2 + i] >> 4) - 8) * d;
            }
        }
        return FORGE_OK;
    }
    if (t.type == T_Q4_1 && expect % 32 == 0) {  // weight_loader.rs:931-966: {f16 scale, f16 min, 16 nibble bytes}, q * scale + min
        for (uint64_t b = 0; b < expect / 32; ++b) {
            uint16_t h0, h1; memcpy(&h0, p + 20 * b, 2); memcpy(&h1, p + 20 * b + 2, 2);
            const float d = f16_to_f32(h0), mn = f16_to_f32(h1);
            for (int i = 0; i < 16; ++i) {
                out[size_t(b * 32 + i)] = float(p[20 * b + 4 + i] & 0x0F) * d + mn;
                out[size_t(b * 32 + i + 16)] = float(p[20 * b + 4 + i] >> 4) * d + mn;
            }
        }
        return FORGE_OK;
    }
    if (t.type == T_Q5_K && expect % 256 == 0) {  // weight_loader.rs:1071-1140: Q4_K's layout plus one high bit per value
        for (uint64_t sb = 0; sb < expect / 256; ++sb) {
            const uint8_t* blk = p + 176 * sb;
            uint16_t h0, h1; memcpy(&h0, blk, 2); memcpy(&h1, blk + 2, 2);
            const float d = f16_to_f32(h0), dmin = f16_to_f32(h1);
            const uint8_t *sc = blk + 4, *qh = blk + 16, *qs = blk + 48;
            for (int j = 0; j < 8; ++j) {  // sub-block j: nibble (j & 1) of qs[(j / 2) * 32 + l], high bit = bit j of qh[l]
                int s6, m6;
                if (j < 4) { s6 = sc[j] & 63; m6 = sc[j + 4] & 63; }
                else { s6 = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); m6 = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
                const float dw = d * float(s6), mw = dmin * float(m6);
                for (int l = 0; l < 32; ++l) {
                    const uint8_t by = qs[(j >> 1) * 32 + l];
                    const uint32_t q5 = uint32_t((j & 1) ? (by >> 4) : (by & 0x0F)) + (((qh[l] >> j) & 1) ? 16u : 0u);
                    out[size_t(sb * 256 + j * 32 + l)] = dw * float(q5) - mw;
                }
            }
        }
        return FORGE_OK;
    }
    if (t.type == T_Q4_K && expect % 256 == 0) {  // weight_loader.rs:1146-1200: d * sc * q - dmin * m per 32-element sub-block
        for (uint64_t sb = 0; sb < expect / 256; ++sb) {
            const uint8_t* blk = p + 144 * sb;
            uint16_t h0, h1; memcpy(&h0, blk, 2); memcpy(&h1, blk + 2, 2);
            const float d = f16_to_f32(h0), dmin = f16_to_f32(h1);
            const uint8_t* sc = blk + 4;
            for (int j = 0; j < 8; ++j) {
                int s6, m6;
                if (j < 4) { s6 = sc[j] & 63; m6 = sc[j + 4] & 63; }
                else { s6 = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); m6 = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
                const float dw = d * float(s6), mw = dmin * float(m6);
                for (int l = 0; l < 32; ++l) {
                    const uint8_t by = blk[16 + (j >> 1) * 32 + l];
                    out[size_t(sb * 256 + j * 32 + l)] = dw * float((j & 1) ? (by >> 4) : (by & 0x0F)) - mw;
                }
            }
        }
        return FORGE_OK;
    }
    if (t.type == T_Q6_K && expect % 256 == 0) {  // weight_loader.rs:997-1060: d * scale[group of 16] * (q6 - 32)
        for (uint64_t sb = 0; sb < expect / 256; ++sb) {
            const uint8_t* blk = p + 210 * sb;
            uint16_t h; memcpy(&h, blk + 208, 2);
            const float d = f16_to_f32(h);
            for (int j = 0; j < 8; ++j) {  // 32-element group j: see the block table of dot_q6_k_q8_0 (emit.rs:3560-3570)
                const uint8_t* ql = blk + (j >> 2) * 64 + (j & 1) * 32;
                const uint8_t* qh = blk + 128 + (j >> 2) * 32;
                const int nib = ((j >> 1) & 1) * 4, hsh = (j & 3) * 2;
                for (int l = 0; l < 32; ++l) {
                    const int q6 = int(((ql[l] >> nib) & 0x0F) | (((qh[l] >> hsh) & 3) << 4)) - 32;
                    out[size_t(sb * 256 + j * 32 + l)] = d * float(int(int8_t(blk[192 + 2 * j + (l >> 4)]))) * float(q6);
                }
            }
        }
        return FORGE_OK;
    }
    set_error("tensor %s: type %d cannot be read as f32 here", t.name.c_str(), t.type);
    return FORGE_ERR_UNSUPPORTED;
}

bool is_kquant(int32_t q) { return q == FORGE_Q4_K || q == FORGE_Q6_K; }
uint64_t row_bytes(int32_t quant, uint64_t cols) {
    if (is_kquant(quant)) return cols / 256 * (quant == FORGE_Q4_K ? 144 : 210);
    return cols / 32 * (quant == FORGE_Q8_0 ? 34 : 18);
}
int32_t quant_of(const ForgeModelConfig& c, int cat) { return c.proj_quant[cat] ? c.proj_quant[cat] : c.quant; }

struct Sink {  // counts bytes, and writes them when there is a buffer
    uint8_t* out; size_t cap, n = 0; bool overflow = false;
    void put(const void* src, size_t bytes) {
        if (out) { if (bytes > cap - n) { overflow = true; return; } memcpy(out + n, src, bytes); }
        n += bytes;
    }
};

int32_t put_f32_tensor(const ForgeGguf& g, const std::string& hf, uint64_t expect, Sink& s) {
    const TensorInfo* t = g.tensor(hf);
    if (!t) { set_error("weight not found: %s", hf.c_str()); return FORGE_ERR_SHAPE; }
    if (!s.out) { s.n += size_t(expect) * 4; return t->numel() == expect ? FORGE_OK : (set_error("tensor %s has the wrong size", hf.c_str()), FORGE_ERR_SHAPE); }
    if (t->numel() != expect) { set_error("tensor %s has the wrong size", hf.c_str()); return FORGE_ERR_SHAPE; }
    std::vector<float> v;
    FORGE_TRY(to_f32(g, *t, expect, v));
    s.put(v.data(), v.size() * 4);
    return FORGE_OK;
}

int32_t put_quantised(const std::vector<float>& v, int32_t quant, Sink& s) {
    const bool kq = quant == FORGE_Q4_K || quant == FORGE_Q6_K;
    std::vector<uint8_t> q(kq ? v.size() / 256 * (quant == FORGE_Q4_K ? 144 : 210) : v.size() / 32 * (quant == FORGE_Q8_0 ? 34 : 18));
    if (quant == FORGE_Q8_0) FORGE_TRY(forge_quantize_q8_0_host(v.data(), v.size(), q.data()));
    else if (quant == FORGE_Q4_K) FORGE_TRY(forge_quantize_q4_k_host(v.data(), v.size(), q.data()));
    else if (quant == FORGE_Q6_K) FORGE_TRY(forge_quantize_q6_k_host(v.data(), v.size(), q.data()));
    else FORGE_TRY(forge_quantize_q4_0_host(v.data(), v.size(), q.data(), 0));
    s.put(q.data(), q.size());
    return FORGE_OK;
}

// Where a projection's rows live: a tensor of its own, or a row range of a fused Phi-3 tensor - q | k | v in
// attn_qkv.weight, gate | up in a double-height ffn_up.weight (split_fused_tensors, weight_loader.rs:543-582).
struct Part { const TensorInfo* t = nullptr; uint64_t first = 0; bool fused = false; };

Part find_projection(const ForgeGguf& g, const std::string& hf, uint64_t numel, const ForgeModelConfig& c) {
    const uint64_t H = uint64_t(c.hidden_size), QK = uint64_t(c.num_heads) * c.head_dim, KV = uint64_t(c.num_kv_heads) * c.head_dim;
    const uint64_t FF = uint64_t(c.intermediate_size);
    const size_t dot = hf.rfind(".self_attn."), mlp = hf.rfind(".mlp.");
    if (const TensorInfo* t = g.tensor(hf)) {
        // a double-height up_proj without a gate_proj is the fused gate | up tensor: up is its second half
        if (mlp != std::string::npos && hf.compare(mlp, std::string::npos, ".mlp.up_proj.weight") == 0 && t->numel() == 2 * numel &&
            !g.tensor(hf.substr(0, mlp) + ".mlp.gate_proj.weight"))
            return {t, FF * H, true};
        return {t, 0, false};
    }
    if (dot != std::string::npos) {
        if (const TensorInfo* t = g.tensor(hf.substr(0, dot) + ".self_attn.qkv_proj.weight")) {
            const std::string which = hf.substr(dot);
            if (which == ".self_attn.q_proj.weight") return {t, 0, true};
            if (which == ".self_attn.k_proj.weight") return {t, QK * H, true};
            if (which == ".self_attn.v_proj.weight") return {t, (QK + KV) * H, true};
        }
    }
    if (mlp != std::string::npos && hf.compare(mlp, std::string::npos, ".mlp.gate_proj.weight") == 0) {
        const TensorInfo* t = g.tensor(hf.substr(0, mlp) + ".mlp.up_proj.weight");
        if (t && t->numel() == 2 * numel) return {t, 0, true};
    }
    return {};
}

// a projection [rows][cols] of category `cat`: raw blocks when the tensor already has the category's block format.
// Otherwise the tensor is dequantised and quantised again in the category's format, as the reference's loader does
// for K-quant categories (load_from_file_mixed_per_tensor, weight_loader.rs:193-218: the alternating Q4_K / Q6_K
// attn_v and ffn_down tensors of a Q4_K_M file) and its exporter for dense projections of Q4_0 models
// (main.rs:2601-2607).  Source formats this reader cannot dequantise (Q5_0, Q5_1, Q8_1, Q2_K, Q3_K, Q8_K, I-quants) are reported.
int32_t put_projection(const ForgeGguf& g, const std::string& hf, int cat, uint64_t rows, uint64_t cols, const ForgeModelConfig& c, Sink& s) {
    const int32_t quant = quant_of(c, cat);
    const uint64_t numel = rows * cols, rb = row_bytes(quant, cols);
    const uint64_t blk = is_kquant(quant) ? 256 : 32;
    if (cols % blk) { set_error("tensor %s: %llu columns are not a multiple of the %llu-element block", hf.c_str(), (unsigned long long)cols, (unsigned long long)blk); return FORGE_ERR_SHAPE; }
    const Part part = find_projection(g, hf, numel, c);
    const TensorInfo* t = part.t;
    if (!t) { set_error("weight not found: %s", hf.c_str()); return FORGE_ERR_SHAPE; }
    if (part.first > t->numel() || numel > t->numel() - part.first || t->dims[0] != cols) { set_error("tensor %s does not hold a [%llu][%llu] projection", t->name.c_str(), (unsigned long long)rows, (unsigned long long)cols); return FORGE_ERR_SHAPE; }
    if (!part.fused && t->numel() != numel) { set_error("tensor %s is not [%llu][%llu]", hf.c_str(), (unsigned long long)rows, (unsigned long long)cols); return FORGE_ERR_SHAPE; }
    if (!s.out) { s.n += size_t(rows * rb); return FORGE_OK; }
    const int32_t want = quant == FORGE_Q8_0 ? T_Q8_0 : quant == FORGE_Q4_0 ? T_Q4_0 : quant == FORGE_Q4_K ? T_Q4_K : T_Q6_K;
    if (t->type == want) {
        const uint8_t* p; uint64_t bytes;
        if (!g.span(*t, p, bytes)) { set_error("tensor %s extends past the end of the file", t->name.c_str()); return FORGE_ERR_SHAPE; }
        s.put(p + part.first / cols * rb, size_t(rows * rb));
        return FORGE_OK;
    }
    const bool dense = t->type == T_F32 || t->type == T_F16 || t->type == T_BF16;
    const bool blocks = t->type == T_Q8_0 || t->type == T_Q4_0 || t->type == T_Q4_1 || t->type == T_Q4_K || t->type == T_Q5_K || t->type == T_Q6_K;
    if ((dense && !is_kquant(quant)) || (blocks && (is_kquant(quant) || quant == FORGE_Q8_0 || t->type == T_Q8_0))) {
        std::vector<float> v;
        FORGE_TRY(to_f32(g, *t, numel, v, part.first));
        return put_quantised(v, quant, s);
    }
    set_error("tensor %s: type %d cannot be converted to the format %d of its category here", t->name.c_str(), t->type, quant);
    return FORGE_ERR_UNSUPPORTED;
}

int32_t export_to(const ForgeGguf& g, Sink& s) {
    ForgeModelConfig c;
    FORGE_TRY(forge_gguf_model_config(&g, &c));
    const uint64_t H = uint64_t(c.hidden_size), QK = uint64_t(c.num_heads) * c.head_dim, KV = uint64_t(c.num_kv_heads) * c.head_dim;
    const uint64_t FF = uint64_t(c.intermediate_size), V = uint64_t(c.vocab_size);
    if (H % 32 || QK % 32 || FF % 32) { set_error("hidden, attention and FFN widths must be multiples of 32"); return FORGE_ERR_SHAPE; }
    FORGE_TRY(put_f32_tensor(g, "model.embed_tokens.weight", V * H, s));
    for (int l = 0; l < c.num_layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        FORGE_TRY(put_f32_tensor(g, p + "input_layernorm.weight", H, s));
        FORGE_TRY(put_projection(g, p + "self_attn.q_proj.weight", 0, QK, H, c, s));
        FORGE_TRY(put_projection(g, p + "self_attn.k_proj.weight", 1, KV, H, c, s));
        FORGE_TRY(put_projection(g, p + "self_attn.v_proj.weight", 2, KV, H, c, s));
        if (c.qkv_bias) {
            FORGE_TRY(put_f32_tensor(g, p + "self_attn.q_proj.bias", QK, s));
            FORGE_TRY(put_f32_tensor(g, p + "self_attn.k_proj.bias", KV, s));
            FORGE_TRY(put_f32_tensor(g, p + "self_attn.v_proj.bias", KV, s));
        }
        FORGE_TRY(put_projection(g, p + "self_attn.o_proj.weight", 3, H, QK, c, s));
        FORGE_TRY(put_f32_tensor(g, p + "post_attention_layernorm.weight", H, s));
        FORGE_TRY(put_projection(g, p + "mlp.gate_proj.weight", 4, FF, H, c, s));
        FORGE_TRY(put_projection(g, p + "mlp.up_proj.weight", 5, FF, H, c, s));
        FORGE_TRY(put_projection(g, p + "mlp.down_proj.weight", 6, H, FF, c, s));
    }
    FORGE_TRY(put_f32_tensor(g, "model.norm.weight", H, s));
    // lm_head: output.weight, else the (tied) embedding in the model's block format (main.rs:2625-2667)
    FORGE_TRY(put_projection(g, g.tensor("lm_head.weight") ? "lm_head.weight" : "model.embed_tokens.weight", 7, V, H, c, s));
    if (s.overflow) { set_error("output buffer too small"); return FORGE_ERR_INVALID_ARG; }
    return FORGE_OK;
}

}  // namespace

extern "C" {

int32_t forge_gguf_open(const void* data, size_t len, ForgeGguf** out) {
    if (!data || !out) { set_error("bad argument to forge_gguf_open"); return FORGE_ERR_INVALID_ARG; }
    *out = nullptr;
    Reader r{static_cast<const uint8_t*>(data), len};
    const uint32_t magic = r.get<uint32_t>();
    if (!r.ok || magic != kMagic) { set_error("not a GGUF file (magic 0x%08x)", magic); return FORGE_ERR_SHAPE; }
    const uint32_t version = r.get<uint32_t>();
    if (!r.ok || (version != 2 && version != 3)) { set_error("unsupported GGUF version %u", version); return FORGE_ERR_UNSUPPORTED; }
    const uint64_t n_tensors = r.get<uint64_t>(), n_meta = r.get<uint64_t>();
    if (!r.ok || n_tensors > len || n_meta > len) { set_error("truncated GGUF header"); return FORGE_ERR_SHAPE; }
    ForgeGguf* g = new ForgeGguf();
    g->data = r.p; g->len = len; g->version = version;
    auto fail = [&](int32_t code) { delete g; return code; };
    for (uint64_t i = 0; i < n_meta; ++i) {
        std::string key = r.str();
        const uint32_t type = r.get<uint32_t>();
        MetaValue v;
        if (!r.ok || !read_value(r, int(type), v, 0)) { set_error("bad metadata entry %llu (value type %u)", (unsigned long long)i, type); return fail(r.ok ? FORGE_ERR_UNSUPPORTED : FORGE_ERR_SHAPE); }
        g->meta.emplace(std::move(key), std::move(v));
    }
    g->tensors.reserve(size_t(n_tensors));
    for (uint64_t i = 0; i < n_tensors; ++i) {
        TensorInfo t;
        t.name = r.str();
        const uint32_t nd = r.get<uint32_t>();
        if (!r.ok) { set_error("truncated tensor table"); return fail(FORGE_ERR_SHAPE); }
        if (nd > 4) { set_error("tensor %s has %u dimensions", t.name.c_str(), nd); return fail(FORGE_ERR_SHAPE); }
        t.n_dims = int(nd);
        for (uint32_t d = 0; d < nd; ++d) t.dims[d] = r.get<uint64_t>();
        t.type = int32_t(r.get<uint32_t>());
        t.offset = r.get<uint64_t>();
        if (!r.ok) { set_error("truncated tensor table"); return fail(FORGE_ERR_SHAPE); }
        uint64_t prod = 1;
        for (uint32_t d = 0; d < nd; ++d) { if (t.dims[d] && prod > UINT64_MAX / t.dims[d]) { set_error("tensor %s overflows", t.name.c_str()); return fail(FORGE_ERR_SHAPE); } prod *= t.dims[d]; }
        g->by_hf_name.emplace(hf_name(t.name), g->tensors.size());
        g->tensors.push_back(std::move(t));
    }
    uint64_t a = 0;
    if (g->get_u32("general.alignment", a) && a > 0) {
        // a power of two no larger than the file: anything else cannot be a real alignment and would overflow the round-up below
        if ((a & (a - 1)) != 0 || uint64_t(a) > uint64_t(len)) { set_error("GGUF general.alignment %llu is not a power of two within the file", (unsigned long long)a); return fail(FORGE_ERR_SHAPE); }
        g->alignment = a;
    }
    g->data_offset = (uint64_t(r.pos) + g->alignment - 1) / g->alignment * g->alignment;
    *out = g;
    return FORGE_OK;
}

void forge_gguf_close(ForgeGguf* g) { delete g; }

int32_t forge_gguf_version(const ForgeGguf* g) { return g ? int32_t(g->version) : -1; }
int64_t forge_gguf_tensor_count(const ForgeGguf* g) { return g ? int64_t(g->tensors.size()) : -1; }
uint64_t forge_gguf_data_offset(const ForgeGguf* g) { return g ? g->data_offset : 0; }

int32_t forge_gguf_tensor_info(const ForgeGguf* g, int64_t index, const char** name, int32_t* ggml_type, int32_t* n_dims,
                               uint64_t* dims, uint64_t* offset, uint64_t* data_size) {
    if (!g || index < 0 || size_t(index) >= g->tensors.size()) { set_error("tensor index out of range"); return FORGE_ERR_INVALID_ARG; }
    const TensorInfo& t = g->tensors[size_t(index)];
    if (name) *name = t.name.c_str();
    if (ggml_type) *ggml_type = t.type;
    if (n_dims) *n_dims = t.n_dims;
    if (dims) for (int d = 0; d < 4; ++d) dims[d] = d < t.n_dims ? t.dims[d] : 0;
    if (offset) *offset = t.offset;
    if (data_size) {
        uint64_t block, tsz;
        if (!type_layout(t.type, block, tsz)) { set_error("tensor %s has unknown type %d", t.name.c_str(), t.type); return FORGE_ERR_UNSUPPORTED; }
        *data_size = (t.numel() + block - 1) / block * tsz;
    }
    return FORGE_OK;
}

int32_t forge_gguf_model_config(const ForgeGguf* g, ForgeModelConfig* c) {
    if (!g || !c) { set_error("bad argument to forge_gguf_model_config"); return FORGE_ERR_INVALID_ARG; }
    const MetaValue* av = g->get("general.architecture");
    const std::string arch = av && av->type == 8 ? av->s : "unknown";
    if (arch != "llama" && arch != "qwen2" && arch != "mistral" && arch != "phi3" && arch != "phi") { set_error("unsupported GGUF architecture for this backend: %s", arch.c_str()); return FORGE_ERR_UNSUPPORTED; }
    uint64_t hidden = 0, layers = 0, heads = 0, kv_heads = 0, ff = 0, ctx = 0, vocab = 0, window = 0;
    g->get_u32(arch + ".embedding_length", hidden);
    g->get_u32(arch + ".block_count", layers);
    g->get_u32(arch + ".attention.head_count", heads);
    if (!g->get_u32(arch + ".attention.head_count_kv", kv_heads)) kv_heads = heads;
    if (hidden == 0 || layers == 0 || heads == 0) { set_error("could not extract the model configuration from the GGUF metadata"); return FORGE_ERR_SHAPE; }
    g->get_u32(arch + ".attention.sliding_window", window);
    if (!g->get_u32(arch + ".feed_forward_length", ff)) ff = hidden * 4;
    const MetaValue* toks = g->get("tokenizer.ggml.tokens");
    if (toks && toks->type == 9) vocab = toks->count;
    else if (!g->get_u64(arch + ".vocab_size", vocab)) vocab = 32000;
    if (!g->get_u64(arch + ".context_length", ctx)) ctx = 2048;
    float eps = 1e-5f, theta = 10000.0f;
    g->get_f32(arch + ".attention.layer_norm_rms_epsilon", eps);
    g->get_f32(arch + ".rope.freq_base", theta);
    int32_t quant = 0;
    FORGE_TRY(vote_quant(*g, quant));
    memset(c, 0, sizeof(*c));
    c->hidden_size = int32_t(hidden); c->intermediate_size = int32_t(ff); c->num_layers = int32_t(layers);
    c->num_heads = int32_t(heads); c->num_kv_heads = int32_t(kv_heads); c->head_dim = int32_t(hidden / heads);
    c->vocab_size = int32_t(vocab); c->max_seq_len = int32_t(ctx);
    c->rms_norm_eps = eps; c->rope_theta = theta;
    c->quant = quant; c->qkv_bias = arch == "qwen2" ? 1 : 0;
    c->tp_rank = 0; c->tp_world = 1;
    c->sliding_window = int32_t(window);
    int32_t pq[8];
    detect_proj_quants(*g, quant, pq);
    bool uniform = true;
    for (int i = 0; i < 8; ++i) uniform = uniform && pq[i] == quant;
    if (!uniform) memcpy(c->proj_quant, pq, sizeof(pq));
    return FORGE_OK;
}

int32_t forge_gguf_tensor_to_f32(const ForgeGguf* g, int64_t index, float* out, size_t capacity) {
    if (!g || !out || index < 0 || size_t(index) >= g->tensors.size()) { set_error("bad argument to forge_gguf_tensor_to_f32"); return FORGE_ERR_INVALID_ARG; }
    const TensorInfo& t = g->tensors[size_t(index)];
    if (capacity < t.numel()) { set_error("tensor %s has %llu elements, the buffer holds %zu", t.name.c_str(), (unsigned long long)t.numel(), capacity); return FORGE_ERR_INVALID_ARG; }
    std::vector<float> v;
    FORGE_TRY(to_f32(*g, t, t.numel(), v));
    memcpy(out, v.data(), v.size() * sizeof(float));
    return FORGE_OK;
}

size_t forge_gguf_weights_bin_size(const ForgeGguf* g) {
    if (!g) return 0;
    Sink s{nullptr, 0};
    return export_to(*g, s) == FORGE_OK ? s.n : 0;
}

int32_t forge_gguf_export_weights_bin(const ForgeGguf* g, void* out, size_t capacity) {
    if (!g || !out) { set_error("bad argument to forge_gguf_export_weights_bin"); return FORGE_ERR_INVALID_ARG; }
    Sink s{static_cast<uint8_t*>(out), capacity};
    return export_to(*g, s);
}

}  // extern "C"
