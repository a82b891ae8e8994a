// Operator-level C entry points: device-pointer twins of the generated kernels, taking raw
// GGUF block bytes like the functions they replace.  Each call repacks the weight it is given
// into the kernels' aligned layout in stream-ordered scratch memory, so these are meant for
// parity tests and one-off use; the session API (forge_model_create) packs weights once.
#include <cmath>
#include <vector>

#include "common.cuh"

using namespace forge;

namespace {

struct AsyncBuf {
    void* p = nullptr; cudaStream_t st;
    explicit AsyncBuf(cudaStream_t s) : st(s) {}
    cudaError_t alloc(size_t bytes) { return cudaMallocAsync(&p, bytes ? bytes : 1, st); }
    ~AsyncBuf() { if (p) cudaFreeAsync(p, st); }
};

int32_t need_device() {
    if (forge_device_count() == 0) { set_error("no CUDA device: this backend has no CPU fallback"); return FORGE_ERR_CUDA; }
    return FORGE_OK;
}

int32_t matmul_mat(int quant, float* out, int32_t m, const float* in, const uint8_t* w, int32_t K, int32_t N, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !in || !w || m < 0 || K <= 0 || N <= 0) { set_error("bad argument to forge_matmul_mat"); return FORGE_ERR_INVALID_ARG; }
    if (K % 32) { set_error("K=%d must be a multiple of 32", K); return FORGE_ERR_SHAPE; }
    if (m == 0) return FORGE_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int BS = quant == FORGE_Q8_0 ? 34 : 18;
    if (m < FORGE_PREFILL_BATCH_THRESHOLD) {  // per-token path: the streaming GEMV, f32-exact up to summation order
        QTiled qt;
        qt.K = K; qt.N = N; qt.quant = quant; qt.row_tiles = (N + 15) / 16;
        AsyncBuf td(st), tab(st), err(st);
        FORGE_CUDA(td.alloc(qtiled_bytes(quant, K, N)));
        FORGE_CUDA(tab.alloc(size_t(qt.row_tiles) * 16 * sizeof(uint8_t*)));
        FORGE_CUDA(err.alloc(sizeof(int)));
        FORGE_CUDA(cudaMemsetAsync(err.p, 0, sizeof(int), st));
        std::vector<const uint8_t*> rows(size_t(qt.row_tiles) * 16, nullptr);
        for (int r = 0; r < N; ++r) rows[r] = w + size_t(r) * (K / 32) * BS;
        FORGE_CUDA(cudaMemcpyAsync(tab.p, rows.data(), rows.size() * sizeof(uint8_t*), cudaMemcpyHostToDevice, st));
        FORGE_CUDA(cudaStreamSynchronize(st));  // `rows` leaves scope
        qt.data = static_cast<uint8_t*>(td.p);
        FORGE_TRY(tile_pack(static_cast<const uint8_t* const*>(tab.p), qt, st));
        GemvArgs ga;
        ga.x = in; ga.out = out; ga.batch = m;
        FORGE_TRY(gemv_tc(qt, EPI_STORE, ga, static_cast<int*>(err.p), st));
        int herr = 0;
        FORGE_CUDA(cudaMemcpyAsync(&herr, err.p, sizeof(int), cudaMemcpyDeviceToHost, st));
        FORGE_CUDA(cudaStreamSynchronize(st));
        if (herr) { set_error("gemv: a bounded device-side wait gave up"); return FORGE_ERR_TIMEOUT; }
        return FORGE_OK;
    }
    QWeight qw;
    qw.K = K; qw.N = N; qw.quant = quant;
    AsyncBuf qs(st), d(st), a16(st), a16lo(st);
    FORGE_CUDA(qs.alloc(size_t(N) * qw.qs_row_bytes()));
    FORGE_CUDA(d.alloc(size_t(N) * (K / 32) * sizeof(__half)));
    qw.qs = static_cast<uint8_t*>(qs.p); qw.d = static_cast<__half*>(d.p);
    FORGE_TRY(pack_rows(w, quant, K, 0, N, 0, K / 32, qw, 0, 1, st));
    FORGE_CUDA(a16.alloc(size_t(m) * K * sizeof(__half)));
    FORGE_CUDA(a16lo.alloc(size_t(m) * K * sizeof(__half)));
    FORGE_TRY(f32_to_f16(static_cast<__half*>(a16.p), static_cast<__half*>(a16lo.p), in, size_t(m) * K, st));
    return gemm_f16a(out, static_cast<const __half*>(a16.p), static_cast<const __half*>(a16lo.p), qw, m, nullptr, st);
}

}  // namespace

extern "C" {

int32_t forge_matmul_mat_q8_0(float* out, int32_t m, const float* in, const uint8_t* w, int32_t K, int32_t N, void* stream) {
    return matmul_mat(FORGE_Q8_0, out, m, in, w, K, N, stream);
}
int32_t forge_matmul_mat_q4_0(float* out, int32_t m, const float* in, const uint8_t* w, int32_t K, int32_t N, void* stream) {
    return matmul_mat(FORGE_Q4_0, out, m, in, w, K, N, stream);
}

int32_t forge_rms_norm(float* out, const float* in, const float* weight, int32_t rows, int32_t n, float eps, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !in || !weight || rows < 0 || n <= 0) { set_error("bad argument to forge_rms_norm"); return FORGE_ERR_INVALID_ARG; }
    return rms_norm_f32(out, in, weight, rows, n, eps, static_cast<cudaStream_t>(stream));
}

int32_t forge_rope_table(float* table, int32_t n_pos, int32_t head_dim, float theta) {
    if (!table || n_pos < 0 || head_dim <= 0 || (head_dim & 1)) { set_error("bad argument to forge_rope_table"); return FORGE_ERR_INVALID_ARG; }
    const int half = head_dim / 2;
    std::vector<float> freq(half);
    for (int i = 0; i < half; ++i) freq[i] = 1.0f / powf(theta, 2.0f * float(i) / float(head_dim));
    for (int pos = 0; pos < n_pos; ++pos)
        for (int i = 0; i < half; ++i) {
            float ang = float(pos) * freq[i];
            table[(size_t(pos) * half + i) * 2] = cosf(ang);
            table[(size_t(pos) * half + i) * 2 + 1] = sinf(ang);
        }
    return FORGE_OK;
}

int32_t forge_rope(float* data, int32_t rows, int32_t base_pos, int32_t head_dim, int32_t num_heads, const float* table, void* stream) {
    FORGE_TRY(need_device());
    if (!data || !table || rows < 0 || base_pos < 0 || head_dim <= 0 || (head_dim & 1) || num_heads <= 0) { set_error("bad argument to forge_rope"); return FORGE_ERR_INVALID_ARG; }
    return rope_rows(data, rows, base_pos, head_dim, num_heads, table, static_cast<cudaStream_t>(stream));
}

int32_t forge_silu_mul(float* out, const float* gate, const float* up, size_t n, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !gate || !up) { set_error("bad argument to forge_silu_mul"); return FORGE_ERR_INVALID_ARG; }
    return silu_mul_f32(out, gate, up, n, static_cast<cudaStream_t>(stream));
}

int32_t forge_residual_add(float* a, const float* b, size_t n, void* stream) {
    FORGE_TRY(need_device());
    if (!a || !b) { set_error("bad argument to forge_residual_add"); return FORGE_ERR_INVALID_ARG; }
    return residual_add_f32(a, b, n, static_cast<cudaStream_t>(stream));
}

int32_t forge_kv_append_f16(uint16_t* k_cache, uint16_t* v_cache, const float* k, const float* v, int32_t rows, int32_t base_pos,
                            int32_t kv_dim, void* stream) {
    FORGE_TRY(need_device());
    if (!k_cache || !v_cache || !k || !v || rows < 0 || base_pos < 0 || kv_dim <= 0) { set_error("bad argument to forge_kv_append_f16"); return FORGE_ERR_INVALID_ARG; }
    return kv_append_contig(reinterpret_cast<__half*>(k_cache), reinterpret_cast<__half*>(v_cache), k, v, rows, base_pos, kv_dim,
                            static_cast<cudaStream_t>(stream));
}

int32_t forge_attention_flash(float* out, const float* q, const uint16_t* k_cache, const uint16_t* v_cache, int32_t seq_len,
                              int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !q || !k_cache || !v_cache || seq_len <= 0 || num_heads <= 0 || num_kv_heads <= 0) { set_error("bad argument to forge_attention_flash"); return FORGE_ERR_INVALID_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int splits = std::min(32, std::max(1, seq_len / 64));
    AsyncBuf ws(st), cnt(st);
    FORGE_CUDA(ws.alloc(sizeof(float) * attn_decode_ws_floats(1, num_heads, head_dim, splits)));
    FORGE_CUDA(cnt.alloc(sizeof(int) * num_kv_heads));
    FORGE_CUDA(cudaMemsetAsync(cnt.p, 0, sizeof(int) * num_kv_heads, st));
    AttnDecodeArgs a{out, q, reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache), nullptr, 0, nullptr,
                     seq_len, 1, num_heads, num_kv_heads, head_dim, seq_len, static_cast<float*>(ws.p), static_cast<int*>(cnt.p), splits};
    return attn_decode(a, st);
}

int32_t forge_attention_flash_batch(float* out, const float* q_batch, const uint16_t* k_cache, const uint16_t* v_cache, int32_t m,
                                    int32_t base_pos, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !q_batch || !k_cache || !v_cache || m < 0 || base_pos < 0 || num_heads <= 0 || num_kv_heads <= 0) { set_error("bad argument to forge_attention_flash_batch"); return FORGE_ERR_INVALID_ARG; }
    AttnPrefillArgs a{nullptr, nullptr, out, nullptr, reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache), nullptr,
                      m, base_pos, num_heads, num_kv_heads, head_dim};
    return attn_prefill_q32(a, q_batch, static_cast<cudaStream_t>(stream));
}

int32_t forge_argmax(uint32_t* result, const float* logits, int32_t n, void* stream) {
    FORGE_TRY(need_device());
    if (!result || !logits || n <= 0) { set_error("bad argument to forge_argmax"); return FORGE_ERR_INVALID_ARG; }
    return argmax_last(result, logits, n, 1, static_cast<cudaStream_t>(stream));
}

// ---- host-side quantisers of the exporter (weight_loader.rs:1454-1544)
static inline uint16_t f32_to_f16_bits(float x) { return __half_as_ushort(__float2half_rn(x)); }

int32_t forge_quantize_q8_0_host(const float* x, size_t n, uint8_t* out) {
    if (!x || !out || (n % 32)) { set_error("forge_quantize_q8_0_host: n must be a multiple of 32"); return FORGE_ERR_INVALID_ARG; }
    const long nb = long(n / 32);
#pragma omp parallel for schedule(static)
    for (long b = 0; b < nb; ++b) {
        const float* v = x + size_t(b) * 32;
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
        float scale = amax == 0.f ? 0.f : amax / 127.0f;
        float inv = scale != 0.f ? 1.0f / scale : 0.f;
        uint8_t* o = out + size_t(b) * 34;
        uint16_t hb = f32_to_f16_bits(scale);
        o[0] = uint8_t(hb); o[1] = uint8_t(hb >> 8);
        for (int j = 0; j < 32; ++j) {
            float q = fminf(127.f, fmaxf(-127.f, roundf(v[j] * inv)));
            o[2 + j] = uint8_t(int8_t(q));
        }
    }
    return FORGE_OK;
}

int32_t forge_quantize_q4_0_host(const float* x, size_t n, uint8_t* out, int32_t signed_max) {
    if (!x || !out || (n % 32)) { set_error("forge_quantize_q4_0_host: n must be a multiple of 32"); return FORGE_ERR_INVALID_ARG; }
    const long nb = long(n / 32);
#pragma omp parallel for schedule(static)
    for (long b = 0; b < nb; ++b) {
        const float* v = x + size_t(b) * 32;
        float amax = 0.f, vmax = 0.f;
        for (int j = 0; j < 32; ++j) { float a = fabsf(v[j]); if (a > amax) { amax = a; vmax = v[j]; } }
        float d = signed_max ? (vmax == 0.f ? 0.f : vmax / -8.0f) : amax / 8.0f;
        float inv = d != 0.f ? 1.0f / d : 0.f;
        uint8_t* o = out + size_t(b) * 18;
        uint16_t hb = f32_to_f16_bits(d);
        o[0] = uint8_t(hb); o[1] = uint8_t(hb >> 8);
        for (int j = 0; j < 16; ++j) {
            int lo = int(roundf(v[j] * inv)) + 8, hi = int(roundf(v[j + 16] * inv)) + 8;
            lo = lo < 0 ? 0 : (lo > 15 ? 15 : lo);
            hi = hi < 0 ? 0 : (hi > 15 ? 15 : hi);
            o[2 + j] = uint8_t(lo | (hi << 4));
        }
    }
    return FORGE_OK;
}

}  // extern "C"
