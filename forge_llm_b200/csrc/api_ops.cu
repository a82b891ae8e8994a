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

}  // namespace

// A projection repacked once into both kernel layouts (see forge_packed_create).
struct ForgePacked {
    QWeight soa;
    QTiled tiled;
    int* err = nullptr;
    GemvSplit split;
    GemvSplit bsplit;         // split-K scratch of the batched decode product
    uint2* bact = nullptr;    // its packed activations (sixteen rows)
};

namespace {

bool is_kquant(int quant) { return quant == FORGE_Q4_K || quant == FORGE_Q6_K; }
// bytes of one raw weight row
size_t raw_row_bytes(int quant, int K) {
    if (is_kquant(quant)) return size_t(K / 256) * (quant == FORGE_Q4_K ? 144 : 210);
    return size_t(K / 32) * (quant == FORGE_Q8_0 ? 34 : 18);
}

int32_t packed_build(int quant, const uint8_t* w, int K, int N, cudaStream_t st, ForgePacked* pk) {
    pk->soa.K = K; pk->soa.N = N; pk->soa.quant = quant;
    pk->tiled.K = K; pk->tiled.N = N; pk->tiled.quant = quant;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    pk->tiled.bt = gemv_band_tiles(N, sms);
    pk->tiled.bands = (N + 16 * pk->tiled.bt - 1) / (16 * pk->tiled.bt);
    const bool kq = is_kquant(quant);
    if (kq) pk->soa.quant = FORGE_KQ_SOA;  // K-quant rows of either kind share the expanded row-major layout
    FORGE_CUDA(cudaMalloc(&pk->soa.qs, size_t(N) * pk->soa.qs_row_bytes()));
    if (kq) FORGE_CUDA(cudaMalloc(&pk->soa.sf, size_t(N) * (K / 32) * sizeof(float4)));
    else FORGE_CUDA(cudaMalloc(&pk->soa.d, size_t(N) * (K / 32) * sizeof(__half)));
    FORGE_CUDA(cudaMalloc(&pk->tiled.data, qtiled_bytes(quant, K, N, pk->tiled.bt)));
    FORGE_CUDA(cudaMalloc(&pk->err, sizeof(int)));
    FORGE_CUDA(cudaMemsetAsync(pk->err, 0, sizeof(int), st));
    FORGE_TRY(pack_rows(w, quant, K, 0, N, 0, K / 32, pk->soa, 0, 1, st));
    if (pk->tiled.bands * 16 * pk->tiled.bt <= kGemvSplitRows) {
        FORGE_CUDA(cudaMalloc(&pk->split.scratch, sizeof(float) * kGemvMaxSlices * size_t(pk->tiled.bands) * 16 * pk->tiled.bt));
        FORGE_CUDA(cudaMalloc(&pk->split.tickets, sizeof(int) * size_t(pk->tiled.bands) * pk->tiled.bt));
        FORGE_CUDA(cudaMemsetAsync(pk->split.tickets, 0, sizeof(int) * size_t(pk->tiled.bands) * pk->tiled.bt, st));
        pk->split.max_slices = kGemvMaxSlices;
    }
    std::vector<const uint8_t*> rows(size_t(pk->tiled.bands) * 16 * pk->tiled.bt, nullptr);
    for (int r = 0; r < N; ++r) rows[r] = w + size_t(r) * raw_row_bytes(quant, K);
    const uint8_t** tab = nullptr;
    FORGE_CUDA(cudaMalloc(&tab, rows.size() * sizeof(uint8_t*)));
    cudaError_t e = cudaMemcpyAsync(tab, rows.data(), rows.size() * sizeof(uint8_t*), cudaMemcpyHostToDevice, st);
    int32_t rc = e == cudaSuccess ? tile_pack(tab, pk->tiled, st) : FORGE_ERR_CUDA;
    cudaStreamSynchronize(st);
    cudaFree(tab);
    if (e != cudaSuccess) set_error("row table upload failed: %s", cudaGetErrorString(e));
    return rc;
}

void packed_free(ForgePacked* pk) {
    if (!pk) return;
    cudaFree(pk->soa.qs); cudaFree(pk->soa.d); cudaFree(pk->soa.sf); cudaFree(pk->tiled.data); cudaFree(pk->err); cudaFree(pk->split.scratch); cudaFree(pk->split.tickets);
    cudaFree(pk->bsplit.scratch); cudaFree(pk->bsplit.tickets); cudaFree(pk->bact);
    delete pk;
}

// Reads the error word a bounded device-side wait sets when it gives up, and clears it so that one timeout does not
// mark every later call on the same packed matrix.  Synchronises the stream.
int32_t packed_check_err(const ForgePacked* pk, cudaStream_t st) {
    int herr = 0;
    FORGE_CUDA(cudaMemcpyAsync(&herr, pk->err, sizeof(int), cudaMemcpyDeviceToHost, st));
    FORGE_CUDA(cudaStreamSynchronize(st));
    if (!herr) return FORGE_OK;
    FORGE_CUDA(cudaMemsetAsync(pk->err, 0, sizeof(int), st));
    set_error("matmul: a bounded device-side wait gave up");
    return FORGE_ERR_TIMEOUT;
}

int32_t matmul_packed(float* out, int32_t m, const float* in, const ForgePacked* pk, cudaStream_t st, bool check_err) {
    const int K = pk->soa.K;
    if (m < FORGE_PREFILL_BATCH_THRESHOLD) {  // per-token path: the streaming GEMV, f32-exact up to summation order
        GemvArgs ga;
        ga.x = in; ga.out = out; ga.batch = m;
        FORGE_TRY(gemv_tc(pk->tiled, EPI_STORE, ga, pk->split, pk->err, st));
        return check_err ? packed_check_err(pk, st) : FORGE_OK;
    }
    AsyncBuf a16(st), a16lo(st);
    FORGE_CUDA(a16.alloc(size_t(m) * K * sizeof(__half)));
    FORGE_CUDA(a16lo.alloc(size_t(m) * K * sizeof(__half)));
    FORGE_TRY(f32_to_f16(static_cast<__half*>(a16.p), static_cast<__half*>(a16lo.p), in, size_t(m) * K, st));
    // K-quant products take their input rows as Q8_0 blocks (emit.rs:1412-1440); the batched form keeps that rounding
    if (pk->soa.quant == FORGE_KQ_SOA) FORGE_TRY(q8_round_f16(static_cast<__half*>(a16.p), static_cast<__half*>(a16lo.p), size_t(m) * K, st));
    FORGE_TRY(gemm_f16a(out, static_cast<const __half*>(a16.p), static_cast<const __half*>(a16lo.p), pk->soa, m, nullptr, pk->err, st));
    return check_err ? packed_check_err(pk, st) : FORGE_OK;
}

int32_t matmul_mat(int quant, float* out, int32_t m, const float* in, const uint8_t* w, int32_t K, int32_t N, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !in || !w || m < 0 || K <= 0 || N <= 0) { set_error("bad argument to forge_matmul_mat"); return FORGE_ERR_INVALID_ARG; }
    if (K % (is_kquant(quant) ? 256 : 32)) { set_error("K=%d must be a multiple of %d", K, is_kquant(quant) ? 256 : 32); return FORGE_ERR_SHAPE; }
    if (m == 0) return FORGE_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ForgePacked* pk = new ForgePacked();
    int32_t rc = packed_build(quant, w, K, N, st, pk);
    if (rc == FORGE_OK) rc = matmul_packed(out, m, in, pk, st, true);
    cudaStreamSynchronize(st);
    packed_free(pk);
    return rc;
}

}  // namespace

extern "C" {

int32_t forge_matmul_mat_q8_0(float* out, int32_t m, const float* in, const uint8_t* w, int32_t K, int32_t N, void* stream) {
    return matmul_mat(FORGE_Q8_0, out, m, in, w, K, N, stream);
}
int32_t forge_matmul_mat_q4_0(float* out, int32_t m, const float* in, const uint8_t* w, int32_t K, int32_t N, void* stream) {
    return matmul_mat(FORGE_Q4_0, out, m, in, w, K, N, stream);
}

int32_t forge_matmul_vec_q4_k(float* out, int32_t m, const float* in, const uint8_t* w, int32_t K, int32_t N, void* stream) {
    return matmul_mat(FORGE_Q4_K, out, m, in, w, K, N, stream);
}
int32_t forge_matmul_vec_q6_k(float* out, int32_t m, const float* in, const uint8_t* w, int32_t K, int32_t N, void* stream) {
    return matmul_mat(FORGE_Q6_K, out, m, in, w, K, N, stream);
}

int32_t forge_packed_create(int32_t quant, const uint8_t* w, int32_t K, int32_t N, void* stream, ForgePacked** out) {
    FORGE_TRY(need_device());
    if (!out) { set_error("null out pointer"); return FORGE_ERR_INVALID_ARG; }
    *out = nullptr;
    if (!w || K <= 0 || N <= 0 || (quant != FORGE_Q8_0 && quant != FORGE_Q4_0 && !is_kquant(quant))) { set_error("bad argument to forge_packed_create"); return FORGE_ERR_INVALID_ARG; }
    if (K % (is_kquant(quant) ? 256 : 32)) { set_error("K=%d must be a multiple of %d", K, is_kquant(quant) ? 256 : 32); return FORGE_ERR_SHAPE; }
    ForgePacked* pk = new ForgePacked();
    int32_t rc = packed_build(quant, w, K, N, static_cast<cudaStream_t>(stream), pk);
    if (rc != FORGE_OK) { packed_free(pk); return rc; }
    *out = pk;
    return FORGE_OK;
}

void forge_packed_destroy(ForgePacked* pk) { packed_free(pk); }

int32_t forge_matmul_mat_packed(float* out, int32_t m, const float* in, const ForgePacked* w, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !in || !w || m < 0) { set_error("bad argument to forge_matmul_mat_packed"); return FORGE_ERR_INVALID_ARG; }
    if (m == 0) return FORGE_OK;
    return matmul_packed(out, m, in, w, static_cast<cudaStream_t>(stream), false);
}

int32_t forge_matmul_decode_batch(float* out, int32_t nb, const float* in, ForgePacked* w, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !in || !w || nb < 0 || nb > 16) { set_error("bad argument to forge_matmul_decode_batch (1..16 rows)"); return FORGE_ERR_INVALID_ARG; }
    if (nb == 0) return FORGE_OK;
    if (is_kquant(w->tiled.quant)) { set_error("forge_matmul_decode_batch takes Q8_0 / Q4_0 weights"); return FORGE_ERR_UNSUPPORTED; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!w->bact) {   // first use: the product's buffers
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        FORGE_CUDA(cudaMalloc(&w->bact, sizeof(uint2) * gemv_batch_act_words(w->tiled.K, 16)));
        const size_t fl = gemv_batch_scratch_floats(w->tiled.N, w->tiled.K, w->tiled.quant, sms), tk = gemv_batch_tickets(w->tiled.N);
        if (fl) {
            FORGE_CUDA(cudaMalloc(&w->bsplit.scratch, sizeof(float) * fl));
            FORGE_CUDA(cudaMalloc(&w->bsplit.tickets, sizeof(int) * tk));
            FORGE_CUDA(cudaMemsetAsync(w->bsplit.tickets, 0, sizeof(int) * tk, st));
            w->bsplit.max_slices = kGemvMaxSlices;
        }
    }
    FORGE_TRY(gemv_batch_pack(w->bact, const_cast<float*>(in), size_t(w->tiled.K), nb, w->tiled.K, w->tiled.quant, 0, nullptr, 0.f, st));
    return gemv_batch(w->tiled, w->bact, nb, out, nullptr, w->bsplit, w->err, st);
}

int32_t forge_packed_check(const ForgePacked* w, void* stream) {
    FORGE_TRY(need_device());
    if (!w) { set_error("bad argument to forge_packed_check"); return FORGE_ERR_INVALID_ARG; }
    return packed_check_err(w, static_cast<cudaStream_t>(stream));
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
    int splits = attn_decode_splits((seq_len + FORGE_KV_PAGE - 1) / FORGE_KV_PAGE, num_kv_heads, 148, head_dim, num_heads / num_kv_heads);
    AsyncBuf ws(st), cnt(st);
    FORGE_CUDA(ws.alloc(sizeof(float) * attn_decode_ws_floats(1, num_heads, head_dim, splits)));
    FORGE_CUDA(cnt.alloc(sizeof(int) * num_kv_heads));
    FORGE_CUDA(cudaMemsetAsync(cnt.p, 0, sizeof(int) * num_kv_heads, st));
    AttnDecodeArgs a{out, q, reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache), nullptr, 0, nullptr,
                     seq_len, 1, num_heads, num_kv_heads, head_dim, seq_len, static_cast<float*>(ws.p), static_cast<int*>(cnt.p), splits};
    return attn_decode(a, st);
}

// the batched attention of the operator surface: f32 queries become fp16 hi + lo pairs (the tensor-core kernel's precise
// form), the contiguous cache is addressed as pages of 64 positions, rows past the last position read as zero
static int32_t attention_batch_f32(float* out, const float* q_batch, const uint16_t* k_cache, const uint16_t* v_cache, int32_t m, int32_t base_pos,
                                   int32_t window, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, cudaStream_t st) {
    if (m == 0) return FORGE_OK;
    const size_t nq = size_t(m) * num_heads * head_dim;
    AsyncBuf q16(st), q16lo(st), err(st);
    FORGE_CUDA(q16.alloc(nq * sizeof(__half)));
    FORGE_CUDA(q16lo.alloc(nq * sizeof(__half)));
    FORGE_CUDA(err.alloc(sizeof(int)));
    FORGE_CUDA(cudaMemsetAsync(err.p, 0, sizeof(int), st));
    FORGE_TRY(f32_to_f16(static_cast<__half*>(q16.p), static_cast<__half*>(q16lo.p), q_batch, nq, st));
    AttnPrefillArgs a{nullptr, nullptr, out, static_cast<const __half*>(q16.p), reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache),
                      nullptr, m, base_pos, num_heads, num_kv_heads, head_dim, window};
    a.q16_lo = static_cast<const __half*>(q16lo.p);
    a.precise = 1;
    a.pool_rows = size_t(base_pos) + size_t(m);
    a.err = static_cast<int*>(err.p);
    FORGE_TRY(attn_prefill(a, st));
    int h_err = 0;
    FORGE_CUDA(cudaMemcpyAsync(&h_err, err.p, sizeof(int), cudaMemcpyDeviceToHost, st));
    FORGE_CUDA(cudaStreamSynchronize(st));
    if (h_err) { set_error("attention: a bounded device-side wait gave up"); return FORGE_ERR_TIMEOUT; }
    return FORGE_OK;
}

int32_t forge_attention_flash_batch(float* out, const float* q_batch, const uint16_t* k_cache, const uint16_t* v_cache, int32_t m,
                                    int32_t base_pos, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !q_batch || !k_cache || !v_cache || m < 0 || base_pos < 0 || num_heads <= 0 || num_kv_heads <= 0) { set_error("bad argument to forge_attention_flash_batch"); return FORGE_ERR_INVALID_ARG; }
    return attention_batch_f32(out, q_batch, k_cache, v_cache, m, base_pos, 0, num_heads, num_kv_heads, head_dim, static_cast<cudaStream_t>(stream));
}

int32_t forge_attention_sliding(float* out, const float* q, const uint16_t* k_cache, const uint16_t* v_cache, int32_t seq_len,
                                int32_t window, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, void* stream) {
    FORGE_TRY(need_device());
    if (!out || !q || !k_cache || !v_cache || seq_len <= 0 || window <= 0 || num_heads <= 0 || num_kv_heads <= 0) { set_error("bad argument to forge_attention_sliding"); return FORGE_ERR_INVALID_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int splits = attn_decode_splits((seq_len + FORGE_KV_PAGE - 1) / FORGE_KV_PAGE, num_kv_heads, 148, head_dim, num_heads / num_kv_heads);
    AsyncBuf ws(st), cnt(st);
    FORGE_CUDA(ws.alloc(sizeof(float) * attn_decode_ws_floats(1, num_heads, head_dim, splits)));
    FORGE_CUDA(cnt.alloc(sizeof(int) * num_kv_heads));
    FORGE_CUDA(cudaMemsetAsync(cnt.p, 0, sizeof(int) * num_kv_heads, st));
    AttnDecodeArgs a{out, q, reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache), nullptr, 0, nullptr,
                     seq_len, 1, num_heads, num_kv_heads, head_dim, seq_len, static_cast<float*>(ws.p), static_cast<int*>(cnt.p), splits, window};
    return attn_decode(a, st);
}

int32_t forge_attention_sliding_batch(float* out, const float* q_batch, const uint16_t* k_cache, const uint16_t* v_cache, int32_t m,
                                      int32_t base_pos, int32_t window, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                      void* stream) {
    FORGE_TRY(need_device());
    if (!out || !q_batch || !k_cache || !v_cache || m < 0 || base_pos < 0 || window <= 0 || num_heads <= 0 || num_kv_heads <= 0) { set_error("bad argument to forge_attention_sliding_batch"); return FORGE_ERR_INVALID_ARG; }
    return attention_batch_f32(out, q_batch, k_cache, v_cache, m, base_pos, window, num_heads, num_kv_heads, head_dim, static_cast<cudaStream_t>(stream));
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
