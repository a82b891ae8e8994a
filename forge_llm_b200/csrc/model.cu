// Host side of the backend: Weights / KVCache / forward / forward_prefill of the generated
// module (crates/forgellm-codegen-cpu/src/emit.rs:3875-4015, :4029-4500, :4553-4587, :5118-5486)
// and the greedy loop of the generated main (crates/forgellm-codegen-cpu/src/project.rs:714-751),
// re-stated as kernel launches on one CUDA stream per model.  The decode step is captured once
// into a CUDA graph (positions and the sampled token live in device memory, so the same graph
// replays for every step).
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstring>
#include <string>
#include <vector>

#include "gemv_core.cuh"

namespace forge {

thread_local std::string g_error;
thread_local long long g_launches = 0;

void set_error(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
}

}  // namespace forge

using namespace forge;

// ------------------------------------------------------------------------------ structures
struct ForgeLayer {
    float* attn_norm = nullptr;
    QWeight qkv;           // rows: [q ; k ; v] of this rank (row-major split layout: prefill GEMM)
    QTiled qkv_t;          // the same matrix in the tiled streaming layout (decode GEMV)
    QTiled v_t;            // only when v_proj is stored in another format than q/k: qkv holds [q ; k], this holds v
    float* qkv_bias = nullptr;
    QWeight o;
    QTiled o_t;
    float* ffn_norm = nullptr;
    QWeight gateup;        // rows interleaved: 2j = gate_j, 2j+1 = up_j
    QTiled gateup_t;
    QWeight down;
    QTiled down_t;
};

struct ForgeModel {
    ForgeModelConfig cfg;
    int device = 0;
    cudaStream_t stream = nullptr;
    // local (per tensor-parallel rank) sizes
    int h = 0, qk = 0, kv = 0, ff = 0, V = 0, hd = 0, nq = 0, nkv = 0;
    float* embed = nullptr;
    std::vector<ForgeLayer> layers;
    float* final_norm = nullptr;
    QWeight lm_head;
    QTiled lm_head_t;
    int* d_err = nullptr;  // set by a kernel whose bounded wait gave up
    GemvSplit split;       // split-K scratch shared by the decode GEMVs (one launch at a time on the stream)
    GemvSplit bsplit;      // the same for the batched decode products
    uint2* d_bact = nullptr;  // packed activations of one batched product (sixteen rows)
    float* rope = nullptr;  // [max_seq][hd/2]{cos,sin}
    int max_seq = 0;
    std::vector<void*> allocs;
    // prefill scratch (grown on demand)
    int scratch_rows = 0, tok_cap = 0;
    float* p_hidden = nullptr; __half* p_normed = nullptr; float* p_qkv = nullptr; __half* p_q16 = nullptr; __half* p_q16_lo = nullptr;
    __half* p_attn16 = nullptr; float* p_gu = nullptr; __half* p_act16 = nullptr; uint32_t* p_tokens = nullptr;
    __half* p_normed_lo = nullptr; __half* p_attn16_lo = nullptr; __half* p_act16_lo = nullptr;
    float* p_parts = nullptr;   // [4][rows][h] partial products of the K-sliced o / down projections
    float* p_qkv_parts = nullptr;   // [4][rows][qk + 2 kv] the same for the QKV projection
    int gemm_passes = 3;  // 3: split-precision prefill GEMMs (default); 1: single fp16 pass
    std::vector<struct ForgeKV*> caches;   // live caches of this model (released with it if the caller did not)
    int pq[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // storage format of q, k, v, o, gate, up, down, lm_head (cfg.proj_quant or cfg.quant)
    bool uniform_basic = true;             // every projection is stored in cfg.quant (Q8_0 / Q4_0): what the whole-step kernel takes
    bool per_token_prefill = false;        // no batched layout for this mix of formats: the prompt always runs token by token
    bool any_kquant = false;               // a projection is stored as Q4_K / Q6_K
    bool kquant_batched = false;           // K-quant models: prompt through the batched GEMMs (forge_model_set_prefill_mode)
    TpComm* tp = nullptr;  // tensor-parallel communicator (cfg.tp_world > 1)
    // peer-memory exchange of the decode step (forge_model_tp_exchange_*): local buffer, peers' mappings, device tables
    void* tpx_local = nullptr; std::vector<void*> tpx_peer; bool tpx_ready = false;
    uint2** d_tpx_ll = nullptr; uint32_t* d_tpx_step = nullptr;  // peers' buffers (device table), decode step counter
    float* p_part = nullptr; float* d_part = nullptr;  // this rank's partial sums of a row-sliced projection
    uint32_t wait_limit = 1u << 20;     // polls per device-side peer wait (forge_model_set_wait_limit)
    // decode scratch (per batch row).  Growing it moves every buffer: scratch_gen counts the moves, and whatever holds the
    // old addresses (a cache's captured decode graph) is rebuilt when its generation differs.
    int dec_batch = 0; int scratch_gen = 0;
    float* d_hidden2 = nullptr;
    float* d_hidden = nullptr; float* d_q = nullptr; float* d_attn = nullptr; float* d_act = nullptr; float* d_logits = nullptr;
    uint32_t* d_tok = nullptr; uint32_t* d_hist = nullptr; int hist_cap = 0; int32_t* d_step = nullptr;
    float* d_amax_val = nullptr; int* d_amax_idx = nullptr; int* d_amax_ticket = nullptr;
    // parity trace
    bool trace_on = false; float* trace = nullptr; size_t trace_cap = 0; int trace_rows = 0;
    // timing of the last generate call
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
    float prefill_ms = 0.f, decode_ms = 0.f; long long last_launches = 0;
};

struct ForgeKV {
    ForgeModel* model = nullptr;
    int max_seq = 0, batch = 0, pages_per_seq = 0, num_pages = 0;
    __half* k_pool = nullptr; __half* v_pool = nullptr;
    size_t layer_stride = 0;  // halfs per layer pool
    int32_t* d_page_table = nullptr; int32_t* d_seq_len = nullptr;
    std::vector<int32_t> h_page_table; std::vector<int> free_pages; std::vector<int> pages_used; std::vector<int> len;
    float* attn_ws = nullptr; int* attn_counters = nullptr; int splits = 1;
    alignas(64) unsigned char k_map[128], v_map[128];   // CUtensorMap of the two pools (all layers), for the decode attention's page copies
    cudaGraphExec_t graph = nullptr; int graph_batch = 0; bool graph_greedy = false; int graph_gen = -1;  // scratch generation the graph was captured with
};

namespace {

template <typename T>
int32_t dev_alloc(ForgeModel* m, T** p, size_t count) {
    void* q = nullptr;
    FORGE_CUDA(cudaMalloc(&q, std::max<size_t>(count, 1) * sizeof(T)));
    m->allocs.push_back(q);
    *p = static_cast<T*>(q);
    return FORGE_OK;
}

int32_t alloc_qweight(ForgeModel* m, QWeight& w, int quant, int K, int N) {
    w.K = K; w.N = N; w.quant = quant;
    FORGE_TRY(dev_alloc(m, &w.qs, size_t(N) * w.qs_row_bytes()));
    if (quant == FORGE_KQ_SOA) FORGE_TRY(dev_alloc(m, &w.sf, size_t(N) * (K / 32)));
    else FORGE_TRY(dev_alloc(m, &w.d, size_t(N) * (K / 32)));
    return FORGE_OK;
}

bool is_kquant(int quant) { return quant == FORGE_Q4_K || quant == FORGE_Q6_K; }
size_t raw_row_bytes(int quant, size_t k) {
    if (is_kquant(quant)) return (k / 256) * (quant == FORGE_Q4_K ? 144 : 210);
    return (k / 32) * (quant == FORGE_Q8_0 ? 34 : 18);
}
size_t raw_bytes(int quant, size_t n, size_t k) { return n * raw_row_bytes(quant, k); }

enum ProjIndex { PQ_Q = 0, PQ_K, PQ_V, PQ_O, PQ_GATE, PQ_UP, PQ_DOWN, PQ_LM };
// storage format of every projection category: cfg.proj_quant[i], or cfg.quant where that is 0
void proj_quants(const ForgeModelConfig* c, int (&pq)[8]) {
    for (int i = 0; i < 8; ++i) pq[i] = c->proj_quant[i] ? c->proj_quant[i] : c->quant;
}

int32_t check_cfg(const ForgeModelConfig* c) {
    if (!c) { set_error("null config"); return FORGE_ERR_INVALID_ARG; }
    int pq[8];
    proj_quants(c, pq);
    bool anyk = false;
    for (int i = 0; i < 8; ++i) {
        if (pq[i] != FORGE_Q8_0 && pq[i] != FORGE_Q4_0 && !is_kquant(pq[i])) { set_error("quant / proj_quant[%d] = %d is not FORGE_Q8_0, FORGE_Q4_0, FORGE_Q4_K or FORGE_Q6_K", i, pq[i]); return FORGE_ERR_INVALID_ARG; }
        anyk = anyk || is_kquant(pq[i]);
    }
    if (pq[PQ_Q] != pq[PQ_K] || pq[PQ_GATE] != pq[PQ_UP]) { set_error("q/k and gate/up must share a storage format (they are fused into one product)"); return FORGE_ERR_UNSUPPORTED; }
    if (c->hidden_size <= 0 || c->intermediate_size <= 0 || c->num_layers <= 0 || c->num_heads <= 0 || c->num_kv_heads <= 0 ||
        c->vocab_size <= 0 || c->max_seq_len <= 0) { set_error("non-positive dimension in config"); return FORGE_ERR_INVALID_ARG; }
    if (c->head_dim != 64 && c->head_dim != 96 && c->head_dim != 128) { set_error("head_dim %d unsupported (64, 96, 128)", c->head_dim); return FORGE_ERR_SHAPE; }
    if (c->hidden_size % 32 || c->intermediate_size % 32 || (c->num_heads * c->head_dim) % 32) { set_error("hidden, intermediate and heads*head_dim must be multiples of 32"); return FORGE_ERR_SHAPE; }
    if (c->num_heads % c->num_kv_heads) { set_error("num_heads must be a multiple of num_kv_heads"); return FORGE_ERR_SHAPE; }
    int tp = c->tp_world < 1 ? 1 : c->tp_world;
    if (c->tp_rank < 0 || c->tp_rank >= tp) { set_error("tp_rank out of range"); return FORGE_ERR_INVALID_ARG; }
    if (c->num_kv_heads % tp || (c->intermediate_size / tp) % 32 || c->intermediate_size % tp) { set_error("tensor-parallel world %d does not divide kv heads / intermediate blocks", tp); return FORGE_ERR_SHAPE; }
    if ((anyk || pq[PQ_V] != pq[PQ_Q]) && tp > 1) { set_error("K-quant and mixed q/v formats are not sharded over tensor-parallel ranks"); return FORGE_ERR_UNSUPPORTED; }
    const int kdim[8] = {c->hidden_size, c->hidden_size, c->hidden_size, c->num_heads * c->head_dim, c->hidden_size, c->hidden_size,
                         c->intermediate_size, c->hidden_size};
    for (int i = 0; i < 8; ++i)
        if (is_kquant(pq[i]) && kdim[i] % 256) { set_error("projection %d is a K-quant but its input width %d is not a multiple of 256", i, kdim[i]); return FORGE_ERR_SHAPE; }
    return FORGE_OK;
}

int32_t ensure_batch_buffers(ForgeModel* m);

int32_t ensure_prefill_scratch(ForgeModel* m, int rows) {
    if (rows <= m->scratch_rows) return FORGE_OK;
    // scratch is only ever grown between calls; old buffers stay alive until model destroy
    size_t r = size_t(rows);
    FORGE_TRY(dev_alloc(m, &m->p_hidden, r * m->h));
    FORGE_TRY(dev_alloc(m, &m->p_normed, r * m->h));
    FORGE_TRY(dev_alloc(m, &m->p_qkv, r * (m->qk + 2 * m->kv)));
    FORGE_TRY(dev_alloc(m, &m->p_q16, r * m->qk));
    FORGE_TRY(dev_alloc(m, &m->p_q16_lo, r * m->qk));
    FORGE_TRY(dev_alloc(m, &m->p_attn16, r * m->qk));
    FORGE_TRY(dev_alloc(m, &m->p_gu, r * 2 * m->ff));
    FORGE_TRY(dev_alloc(m, &m->p_act16, r * m->ff));
    FORGE_TRY(dev_alloc(m, &m->p_tokens, r));
    FORGE_TRY(dev_alloc(m, &m->p_normed_lo, r * m->h));
    FORGE_TRY(dev_alloc(m, &m->p_attn16_lo, r * m->qk));
    FORGE_TRY(dev_alloc(m, &m->p_act16_lo, r * m->ff));
    if (m->cfg.tp_world > 1) FORGE_TRY(dev_alloc(m, &m->p_part, r * m->h));
    else if (m->h % 4 == 0 && m->h <= 8192) {   // K-slice partials of o / down and of q/k/v
        FORGE_TRY(dev_alloc(m, &m->p_parts, 4 * r * m->h));
        FORGE_TRY(dev_alloc(m, &m->p_qkv_parts, 4 * r * (m->qk + 2 * m->kv)));
    }
    m->scratch_rows = rows;
    ++m->scratch_gen;   // a captured batched decode step holds these addresses
    return FORGE_OK;
}

int32_t ensure_decode_scratch(ForgeModel* m, int batch) {
    if (batch <= m->dec_batch) return FORGE_OK;
    size_t b = size_t(batch);
    FORGE_TRY(dev_alloc(m, &m->d_hidden, b * m->h));
    FORGE_TRY(dev_alloc(m, &m->d_hidden2, b * m->h));
    FORGE_TRY(dev_alloc(m, &m->d_q, b * m->qk));
    FORGE_TRY(dev_alloc(m, &m->d_attn, b * m->qk));
    FORGE_TRY(dev_alloc(m, &m->d_act, b * m->ff));
    FORGE_TRY(dev_alloc(m, &m->d_logits, b * m->V));
    FORGE_TRY(dev_alloc(m, &m->d_tok, b));
    FORGE_TRY(dev_alloc(m, &m->d_amax_val, b * kArgmaxSlices));
    FORGE_TRY(dev_alloc(m, &m->d_amax_idx, b * kArgmaxSlices));
    FORGE_TRY(dev_alloc(m, &m->d_amax_ticket, b));
    FORGE_CUDA(cudaMemsetAsync(m->d_amax_ticket, 0, sizeof(int) * b, m->stream));
    if (!m->d_step) { FORGE_TRY(dev_alloc(m, &m->d_step, 1)); }
    if (m->cfg.tp_world > 1) FORGE_TRY(dev_alloc(m, &m->d_part, b * m->h));
    if (batch >= 2) {   // batched steps keep their q/k/v and gate/up rows in the prompt scratch; their buffers must exist before a capture
        FORGE_TRY(ensure_prefill_scratch(m, batch));
        FORGE_TRY(ensure_batch_buffers(m));
    }
    m->dec_batch = batch;
    ++m->scratch_gen;
    return FORGE_OK;
}

int32_t ensure_trace(ForgeModel* m, int rows) {
    size_t need = size_t(m->cfg.num_layers) * rows * m->h;
    if (need > m->trace_cap) {
        FORGE_TRY(dev_alloc(m, &m->trace, need));
        m->trace_cap = need;
    }
    m->trace_rows = rows;
    return FORGE_OK;
}

// hand out pages so that sequence `seq` can hold `new_len` positions; uploads the table row if it changed
int32_t ensure_pages(ForgeKV* kv, int seq, int new_len) {
    if (new_len > kv->max_seq) { set_error("KV cache full: position %d >= max_seq %d", new_len - 1, kv->max_seq); return FORGE_ERR_KV_FULL; }
    int need = (new_len + FORGE_KV_PAGE - 1) / FORGE_KV_PAGE;
    bool dirty = false;
    while (kv->pages_used[seq] < need) {
        if (kv->free_pages.empty()) { set_error("KV page pool exhausted"); return FORGE_ERR_KV_FULL; }
        int pg = kv->free_pages.back();
        kv->free_pages.pop_back();
        kv->h_page_table[size_t(seq) * kv->pages_per_seq + kv->pages_used[seq]++] = pg;
        dirty = true;
    }
    if (dirty) {
        FORGE_CUDA(cudaMemcpyAsync(kv->d_page_table + size_t(seq) * kv->pages_per_seq, &kv->h_page_table[size_t(seq) * kv->pages_per_seq],
                                   sizeof(int32_t) * kv->pages_per_seq, cudaMemcpyHostToDevice, kv->model->stream));
        FORGE_CUDA(cudaStreamSynchronize(kv->model->stream));  // the host vector may change before an async copy runs
    }
    return FORGE_OK;
}

int32_t upload_len(ForgeKV* kv) {
    std::vector<int32_t> l(kv->len.begin(), kv->len.end());
    FORGE_CUDA(cudaMemcpyAsync(kv->d_seq_len, l.data(), sizeof(int32_t) * kv->batch, cudaMemcpyHostToDevice, kv->model->stream));
    FORGE_CUDA(cudaStreamSynchronize(kv->model->stream));
    return FORGE_OK;
}

// The synchronisation point of a session call.  Also reads the word the bounded device-side waits raise when they give
// up (a pipeline stage, a peer's contribution or another CTA's result never arrived): the call then fails with
// FORGE_ERR_TIMEOUT, the word is cleared and the device-side positions are put back to the host's (`kv`, may be null).
int32_t sync_and_check(ForgeModel* m, ForgeKV* kv) {
    int herr = 0;
    FORGE_CUDA(cudaMemcpyAsync(&herr, m->d_err, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    FORGE_CUDA(cudaStreamSynchronize(m->stream));
    if (!herr) return FORGE_OK;
    FORGE_CUDA(cudaMemsetAsync(m->d_err, 0, sizeof(int), m->stream));
    if (kv) FORGE_TRY(upload_len(kv));
    FORGE_CUDA(cudaStreamSynchronize(m->stream));
    set_error("a bounded device-side wait gave up: the step did not complete");
    return FORGE_ERR_TIMEOUT;
}

// hidden += W x for a projection whose K dimension is sliced over the tensor-parallel ranks: the ranks' partial
// products are summed (all-reduce) before the residual is added, so every rank holds the same hidden state
int32_t row_sliced_gemm(ForgeModel* m, const QWeight& w, const __half* a, const __half* alo, int n, cudaStream_t st) {
    if (m->cfg.tp_world == 1) return gemm_f16a(m->p_hidden, a, alo, w, n, m->p_hidden, m->d_err, st);
    FORGE_TRY(gemm_f16a(m->p_part, a, alo, w, n, nullptr, m->d_err, st));
    FORGE_TRY(tp_allreduce_sum(m->tp, m->p_part, size_t(n) * m->h, st));
    return residual_add_f32(m->p_hidden, m->p_part, size_t(n) * m->h, st);
}
// hidden += W x, then (next_norm given) normed = RMSNorm(hidden) * next_norm as the fp16 hi/lo input of the next
// product.  On one GPU a long-K product runs as K slices whose partial products are added by the normalisation pass
// itself (residual add + RMSNorm fused, emit.rs:455-459 and :327-334): shorter accumulation chains in tensor memory
// and more CTAs for these few-row-tile matrices.
int32_t row_sliced_gemm_norm(ForgeModel* m, const QWeight& w, const __half* a, const __half* alo, int n, const float* next_norm, __half* nlo, cudaStream_t st) {
    const int ks = gemm_tc5_ksplit(w);
    if (m->cfg.tp_world == 1 && ks > 1 && gemm_tc5_supported(w) && m->p_parts) {
        const size_t stride = size_t(n) * m->h;
        FORGE_TRY(gemm_tc5(m->p_parts, a, alo, w, n, nullptr, m->d_err, st, ks, stride));
        return add_parts_rms_norm_f16(m->p_hidden, m->p_parts, ks, stride, m->p_normed, nlo, next_norm, n, m->h, m->cfg.rms_norm_eps, st);
    }
    FORGE_TRY(row_sliced_gemm(m, w, a, alo, n, st));
    if (next_norm) FORGE_TRY(rms_norm_f16(m->p_normed, nlo, m->p_hidden, next_norm, n, m->h, m->cfg.rms_norm_eps, st));
    return FORGE_OK;
}
// act = SiLU(gate) * up of the normed rows, as fp16 hi (+ lo): the GEMM's own epilogue where the tcgen05 kernel runs
// (fusion pattern gate/up + SiLU, forgellm-optimizer/src/fusion.rs:12-27), else the product followed by the element-wise pass
int32_t gateup_silu(ForgeModel* m, const QWeight& w, const __half* nlo, __half* flo, int n, cudaStream_t st) {
    if (gemm_tc5_supported(w)) return gemm_tc5(nullptr, m->p_normed, nlo, w, n, nullptr, m->d_err, st, 1, 0, m->p_act16, flo);
    FORGE_TRY(gemm_f16a(m->p_gu, m->p_normed, nlo, w, n, nullptr, m->d_err, st));
    return silu_mul_f16(m->p_act16, flo, m->p_gu, n, m->ff, st);
}
int32_t row_sliced_gemv(ForgeModel* m, const QTiled& w, GemvArgs a, int batch, cudaStream_t st) {
    if (m->cfg.tp_world == 1) return gemv_tc(w, EPI_RESID, a, m->split, m->d_err, st);
    a.out = m->d_part; a.resid = nullptr;
    FORGE_TRY(gemv_tc(w, EPI_STORE, a, m->split, m->d_err, st));
    FORGE_TRY(tp_allreduce_sum(m->tp, m->d_part, size_t(batch) * m->h, st));
    return residual_add_f32(m->d_hidden, m->d_part, size_t(batch) * m->h, st);
}

// exchange buffer of {value, tag} pairs: ll[2 slots][world][h] for the single-sequence step, then
// [2 slots][world][kTpxRows * h] for the rows of a batched step
constexpr int kTpxRows = 32;
inline size_t tpx_region_pairs(const ForgeModel* m) { return 2 * size_t(m->cfg.tp_world) * m->h; }
inline size_t tpx_bytes(const ForgeModel* m) { return sizeof(uint2) * tpx_region_pairs(m) * (1 + kTpxRows); }

int32_t decode_launches(ForgeModel* m, ForgeKV* kv, int batch, bool greedy, bool record, const struct PrefillToken* pt);
int32_t prefill_per_token(ForgeModel* m, ForgeKV* kv, int seq, const uint32_t* tokens_host, int n);

// ------------------------------------------------------------------ prefill of one sequence
// forward_prefill_batched, emit.rs:5118-5486.  Leaves the last row's logits in m->d_logits[0..V).
int32_t prefill_seq(ForgeModel* m, ForgeKV* kv, int seq, const uint32_t* tokens_host, int n) {
    const ForgeModelConfig& c = m->cfg;
    cudaStream_t st = m->stream;
    const int base = kv->len[seq];
    FORGE_TRY(ensure_pages(kv, seq, base + n));
    if (m->per_token_prefill || (m->any_kquant && !m->kquant_batched)) return prefill_per_token(m, kv, seq, tokens_host, n);
    FORGE_TRY(ensure_prefill_scratch(m, n));
    FORGE_TRY(ensure_decode_scratch(m, 1));
    if (m->trace_on) FORGE_TRY(ensure_trace(m, n));
    FORGE_CUDA(cudaMemcpyAsync(m->p_tokens, tokens_host, sizeof(uint32_t) * n, cudaMemcpyHostToDevice, st));
    FORGE_TRY(embedding_rows(m->p_hidden, m->embed, m->p_tokens, n, m->h, nullptr, nullptr, st));
    const int32_t* page_row = kv->d_page_table + size_t(seq) * kv->pages_per_seq;
    const bool split = m->gemm_passes == 3;
    __half* nlo = split ? m->p_normed_lo : nullptr;
    __half* alo = split ? m->p_attn16_lo : nullptr;
    __half* flo = split ? m->p_act16_lo : nullptr;
    FORGE_TRY(rms_norm_f16(m->p_normed, nlo, m->p_hidden, m->layers[0].attn_norm, n, m->h, c.rms_norm_eps, st));
    for (int l = 0; l < c.num_layers; ++l) {
        ForgeLayer& L = m->layers[l];
        __half* kp = kv->k_pool + size_t(l) * kv->layer_stride;
        __half* vp = kv->v_pool + size_t(l) * kv->layer_stride;
        // (normed = RMSNorm(hidden) * attn_norm was formed together with the residual add in front of it)
        if (L.qkv.quant == FORGE_KQ_SOA) FORGE_TRY(q8_round_f16(m->p_normed, nlo, size_t(n) * m->h, st));
        // K and V are rounded to fp16 on their way into the cache, which turns a difference of e before the rounding into
        // ~sqrt(e * 2^-11) after it: the QKV product therefore runs as K slices (shorter accumulation chains in tensor
        // memory, see gemm_tc5_ksplit) whose partials the epilogue kernel adds
        const int qks = (m->cfg.tp_world == 1 && gemm_tc5_supported(L.qkv) && m->p_qkv_parts) ? std::max(1, std::min(4, L.qkv.K / 1024)) : 1;
        const size_t qstride = size_t(n) * (m->qk + 2 * m->kv);
        if (qks > 1) FORGE_TRY(gemm_tc5(m->p_qkv_parts, m->p_normed, nlo, L.qkv, n, nullptr, m->d_err, st, qks, qstride));
        else FORGE_TRY(gemm_f16a(m->p_qkv, m->p_normed, nlo, L.qkv, n, nullptr, m->d_err, st));
        const float* qkv_src = qks > 1 ? m->p_qkv_parts : m->p_qkv;
        // The attention runs in its precise form (queries and probabilities as fp16 hi + lo pairs, output to ~1e-6) whenever
        // the products are split-precision too: with fp16 queries and probabilities alone the layer error is ~3e-4, which
        // compounds past the 1e-3 per-layer gate on 32-layer models.  K-quant models need it in any case (their attention
        // output is rounded to 8 bits in front of o_proj).
        const bool precise = m->any_kquant || m->gemm_passes == 3;
        FORGE_TRY(qkv_post(qkv_src, n, base, L.qkv_bias, m->rope, m->p_q16, precise ? m->p_q16_lo : nullptr, kp, vp, page_row, m->qk, m->kv, m->hd, st, qks, qstride));
        AttnPrefillArgs pa{m->p_attn16, alo, nullptr, m->p_q16, kp, vp, page_row, n, base, m->nq, m->nkv, m->hd, c.sliding_window};
        if (precise) { pa.q16_lo = m->p_q16_lo; pa.precise = 1; }
        pa.pool_rows = size_t(kv->num_pages) * FORGE_KV_PAGE; pa.err = m->d_err;
        FORGE_TRY(attn_prefill(pa, st));
        if (L.o.quant == FORGE_KQ_SOA) FORGE_TRY(q8_round_f16(m->p_attn16, alo, size_t(n) * m->qk, st));
        FORGE_TRY(row_sliced_gemm_norm(m, L.o, m->p_attn16, alo, n, L.ffn_norm, nlo, st));
        if (L.gateup.quant == FORGE_KQ_SOA) FORGE_TRY(q8_round_f16(m->p_normed, nlo, size_t(n) * m->h, st));
        FORGE_TRY(gateup_silu(m, L.gateup, nlo, flo, n, st));
        if (L.down.quant == FORGE_KQ_SOA) FORGE_TRY(q8_round_f16(m->p_act16, flo, size_t(n) * m->ff, st));
        FORGE_TRY(row_sliced_gemm_norm(m, L.down, m->p_act16, flo, n, l + 1 < c.num_layers ? m->layers[l + 1].attn_norm : nullptr, nlo, st));
        if (m->trace_on)
            FORGE_CUDA(cudaMemcpyAsync(m->trace + size_t(l) * n * m->h, m->p_hidden, sizeof(float) * n * m->h, cudaMemcpyDeviceToDevice, st));
    }
    // final rms_norm + lm_head on the last row only (emit.rs:5439-5482): exact-f32 GEMV
    GemvArgs ga;
    ga.x = m->p_hidden + size_t(n - 1) * m->h; ga.norm_w = m->final_norm; ga.eps = c.rms_norm_eps; ga.out = m->d_logits; ga.batch = 1;
    FORGE_TRY(gemv_tc(m->lm_head_t, EPI_STORE, ga, m->split, m->d_err, st));
    kv->len[seq] += n;
    return FORGE_OK;
}


// ------------------------------------------------------------------ one decode step (launch sequence)
// forward(), emit.rs:4029-4500, for `batch` sequences.  Tokens are read from m->d_tok, positions
// from kv->d_seq_len; with `greedy` the next token is selected on the device into m->d_tok.
// `pt` (per-token prefill): the step runs for sequence pt->seq with the token at pt->tok, without the head unless
// pt->head, and leaves the step counter of the generation history alone.
struct PrefillToken { int seq; const uint32_t* tok; bool head; float* trace_dst; size_t trace_stride; };

// A decode step of several sequences: every projection streams its weights ONCE for up to sixteen sequences (the
// generated module has no batched decode: a batch there is B calls of forward(), emit.rs:4029-4500, whose operator
// order this follows).  Activations are packed as fp16 hi/lo fragments in front of each product (with the RMSNorm or
// SiLU*up that feeds it), bias + RoPE + cache append and the single-query attention run per sequence.
constexpr int kBatchGroup = 16;
int32_t ensure_batch_buffers(ForgeModel* m) {
    if (m->d_bact) return FORGE_OK;
    const int maxK = std::max({m->h, m->qk, m->ff});
    FORGE_TRY(dev_alloc(m, &m->d_bact, gemv_batch_act_words(maxK, kBatchGroup)));
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, m->device);
    size_t fl = 1, tk = 1;   // the largest need over the model's matrices (one product at a time on the stream)
    auto need = [&](const QTiled& w) {
        fl = std::max(fl, gemv_batch_scratch_floats(w.N, w.K, w.quant, sms));
        tk = std::max(tk, gemv_batch_tickets(w.N));
    };
    for (const ForgeLayer& L : m->layers) { need(L.qkv_t); need(L.o_t); need(L.gateup_t); need(L.down_t); }
    need(m->lm_head_t);
    FORGE_TRY(dev_alloc(m, &m->bsplit.scratch, fl));
    FORGE_TRY(dev_alloc(m, &m->bsplit.tickets, tk));
    FORGE_CUDA(cudaMemsetAsync(m->bsplit.tickets, 0, sizeof(int) * tk, m->stream));
    m->bsplit.max_slices = kGemvMaxSlices;
    return FORGE_OK;
}

// The pair exchange of sum `index` of a step (see BatchTp): slot = parity of the index, tag = step * (2 L + 1) + index + 1
BatchTp batch_tp(const ForgeModel* m, int index) {
    BatchTp t;
    t.peer_ll = m->d_tpx_ll; t.local_ll = static_cast<const uint2*>(m->tpx_local);
    t.cap = size_t(kTpxRows) * m->h;
    t.base = tpx_region_pairs(m) + size_t(index & 1) * m->cfg.tp_world * t.cap;
    t.world = m->cfg.tp_world; t.rank = m->cfg.tp_rank;
    t.step_counter = m->d_tpx_step; t.step_mul = uint32_t(2 * m->cfg.num_layers + 1); t.step_add = uint32_t(index + 1);
    t.wait_limit = m->wait_limit; t.err = m->d_err;
    return t;
}

// out[n][N] (+ resid) = f(x)[n][K] . W^T in groups of sixteen rows.  consume / push: the tensor-parallel sum in front of
// this product is taken in while its rows are packed / this product's values go to the ranks' exchange buffers (both
// for a single group of rows only).
int32_t batched_product(ForgeModel* m, const QTiled& w, float* x, size_t x_stride, int mode, const float* norm_w, int n,
                        float* out, const float* resid, cudaStream_t st, const BatchTp* consume = nullptr, const BatchTp* push = nullptr) {
    if ((consume || push) && n > kBatchGroup) { set_error("batched product: fused tensor-parallel sums take one group of rows"); return FORGE_ERR_INVALID_ARG; }
    for (int g0 = 0; g0 < n; g0 += kBatchGroup) {
        const int nb = std::min(kBatchGroup, n - g0);
        FORGE_TRY(gemv_batch_pack(m->d_bact, x + size_t(g0) * x_stride, x_stride, nb, w.K, w.quant, mode, norm_w, m->cfg.rms_norm_eps, st, consume));
        FORGE_TRY(gemv_batch(w, m->d_bact, nb, out ? out + size_t(g0) * w.N : nullptr, resid ? resid + size_t(g0) * w.N : nullptr, m->bsplit, m->d_err, st, push));
    }
    return FORGE_OK;
}

// hidden += W f(x) for a projection whose K dimension is sliced over the tensor-parallel ranks; `sum_index` numbers
// the step's sums (the pair exchange tags them with it)
// (`pending`: set when the sum was only pushed - the next normalising product has to consume it)
int32_t batched_row_sliced(ForgeModel* m, const QTiled& w, float* x, size_t x_stride, int mode, int n, int* sum_index, int* pending, cudaStream_t st) {
    if (m->cfg.tp_world == 1) return batched_product(m, w, x, x_stride, mode, nullptr, n, m->d_hidden, m->d_hidden, st);
    if (m->tpx_ready && n <= kBatchGroup) {
        // the product's epilogue pushes the pairs; the next product's packing adds them to the residual stream
        const int index = (*sum_index)++;
        const BatchTp push = batch_tp(m, index);
        *pending = index;
        return batched_product(m, w, x, x_stride, mode, nullptr, n, nullptr, nullptr, st, nullptr, &push);
    }
    FORGE_TRY(batched_product(m, w, x, x_stride, mode, nullptr, n, m->d_part, nullptr, st));
    if (m->tpx_ready && n <= kTpxRows) {
        const int index = (*sum_index)++;
        return tp_pair_sum(m->d_hidden, m->d_part, m->d_tpx_ll, static_cast<const uint2*>(m->tpx_local), tpx_region_pairs(m),
                           size_t(kTpxRows) * m->h, n * m->h, m->cfg.tp_world, m->cfg.tp_rank, index & 1, m->d_tpx_step,
                           uint32_t(2 * m->cfg.num_layers + 1), uint32_t(index + 1), m->wait_limit, m->d_err, st);
    }
    FORGE_TRY(tp_allreduce_sum(m->tp, m->d_part, size_t(n) * m->h, st));
    return residual_add_f32(m->d_hidden, m->d_part, size_t(n) * m->h, st);
}

int32_t decode_launches_batched(ForgeModel* m, ForgeKV* kv, int batch, bool greedy, bool record) {
    const ForgeModelConfig& c = m->cfg;
    cudaStream_t st = m->stream;
    const int n = batch;
    enum { PLAIN = 0, NORM = 1, SILU = 2 };
    int sums = 0;      // tensor-parallel sums issued in this step
    int pending = -1;  // index of a sum that was pushed and not consumed yet
    auto normed_product = [&](const QTiled& w, const float* norm_w, float* out) -> int32_t {   // out = W RMSNorm(hidden), taking a pending sum in
        if (pending < 0) return batched_product(m, w, m->d_hidden, m->h, NORM, norm_w, n, out, nullptr, st);
        const BatchTp consume = batch_tp(m, pending);
        pending = -1;
        return batched_product(m, w, m->d_hidden, m->h, NORM, norm_w, n, out, nullptr, st, &consume);
    };
    FORGE_TRY(embedding_rows(m->d_hidden, m->embed, m->d_tok, n, m->h, record ? m->d_hist : nullptr, m->d_step, st));
    for (int l = 0; l < c.num_layers; ++l) {
        ForgeLayer& L = m->layers[l];
        __half* kp = kv->k_pool + size_t(l) * kv->layer_stride;
        __half* vp = kv->v_pool + size_t(l) * kv->layer_stride;
        FORGE_TRY(normed_product(L.qkv_t, L.attn_norm, m->p_qkv));
        FORGE_TRY(qkv_post_rows(m->p_qkv, n, L.qkv_bias, m->rope, m->d_q, kp, vp, kv->d_page_table, kv->d_seq_len, kv->pages_per_seq,
                                m->qk, m->kv, m->hd, st));
        AttnDecodeArgs da{m->d_attn, m->d_q, kp, vp, kv->d_page_table, kv->pages_per_seq, kv->d_seq_len, 0,
                          n, m->nq, m->nkv, m->hd, kv->max_seq, kv->attn_ws, kv->attn_counters, kv->splits, c.sliding_window};
        da.map_k = kv->k_map; da.map_v = kv->v_map; da.row_base = int(size_t(l) * kv->num_pages * FORGE_KV_PAGE); da.err = m->d_err;
        FORGE_TRY(attn_decode(da, st));
        FORGE_TRY(batched_row_sliced(m, L.o_t, m->d_attn, m->qk, PLAIN, n, &sums, &pending, st));
        FORGE_TRY(normed_product(L.gateup_t, L.ffn_norm, m->p_gu));
        FORGE_TRY(batched_row_sliced(m, L.down_t, m->p_gu, size_t(2) * m->ff, SILU, n, &sums, &pending, st));
    }
    FORGE_TRY(normed_product(m->lm_head_t, m->final_norm, m->d_logits));
    if (greedy) FORGE_TRY(argmax_slices(m->d_tok, m->d_logits, m->V, n, m->d_amax_val, m->d_amax_idx, m->d_amax_ticket, st));
    return step_advance(kv->d_seq_len, n, m->d_step, st, sums ? m->d_tpx_step : nullptr);
}

// A decode step of more than 8 sequences: every projection is one tcgen05 product over the batch rows (the rule the
// generated module applies to prompts, PREFILL_BATCH_THRESHOLD, emit.rs:203-206 and :4576-4587): up to 32 rows its
// weight-streaming form, beyond that the tile form; the weights are read once per step either way.  Operator order of
// forward() (emit.rs:4029-4500) with the batched products of forward_prefill_batched (emit.rs:5118-5486); the rows live
// in the prompt scratch (fp16 hi/lo operands).
int32_t decode_launches_gemm(ForgeModel* m, ForgeKV* kv, int batch, bool greedy, bool record) {
    const ForgeModelConfig& c = m->cfg;
    cudaStream_t st = m->stream;
    const int n = batch;
    const bool split = m->gemm_passes == 3;
    __half* nlo = split ? m->p_normed_lo : nullptr;
    __half* alo = split ? m->p_attn16_lo : nullptr;
    __half* flo = split ? m->p_act16_lo : nullptr;
    FORGE_TRY(embedding_rows(m->p_hidden, m->embed, m->d_tok, n, m->h, record ? m->d_hist : nullptr, m->d_step, st));
    FORGE_TRY(rms_norm_f16(m->p_normed, nlo, m->p_hidden, m->layers[0].attn_norm, n, m->h, c.rms_norm_eps, st));
    for (int l = 0; l < c.num_layers; ++l) {
        ForgeLayer& L = m->layers[l];
        __half* kp = kv->k_pool + size_t(l) * kv->layer_stride;
        __half* vp = kv->v_pool + size_t(l) * kv->layer_stride;
        // q/k/v as K slices like the prompt's (more CTAs for a product of few row tiles; the epilogue adds the slices)
        const int qks = (c.tp_world == 1 && split && gemm_tc5_supported(L.qkv) && m->p_qkv_parts) ? std::max(1, std::min(4, L.qkv.K / 1024)) : 1;
        const size_t qstride = size_t(n) * (m->qk + 2 * m->kv);
        if (qks > 1) FORGE_TRY(gemm_tc5(m->p_qkv_parts, m->p_normed, nlo, L.qkv, n, nullptr, m->d_err, st, qks, qstride));
        else FORGE_TRY(gemm_f16a(m->p_qkv, m->p_normed, nlo, L.qkv, n, nullptr, m->d_err, st));
        FORGE_TRY(qkv_post_rows(qks > 1 ? m->p_qkv_parts : m->p_qkv, n, L.qkv_bias, m->rope, m->d_q, kp, vp, kv->d_page_table, kv->d_seq_len,
                                kv->pages_per_seq, m->qk, m->kv, m->hd, st, qks, qstride));
        AttnDecodeArgs da{m->d_attn, m->d_q, kp, vp, kv->d_page_table, kv->pages_per_seq, kv->d_seq_len, 0,
                          n, m->nq, m->nkv, m->hd, kv->max_seq, kv->attn_ws, kv->attn_counters, kv->splits, c.sliding_window};
        da.map_k = kv->k_map; da.map_v = kv->v_map; da.row_base = int(size_t(l) * kv->num_pages * FORGE_KV_PAGE); da.err = m->d_err;
        da.out16 = m->p_attn16; da.out16_lo = alo;   // straight into the o-projection's operand form
        FORGE_TRY(attn_decode(da, st));
        FORGE_TRY(row_sliced_gemm_norm(m, L.o, m->p_attn16, alo, n, L.ffn_norm, nlo, st));
        FORGE_TRY(gateup_silu(m, L.gateup, nlo, flo, n, st));
        FORGE_TRY(row_sliced_gemm_norm(m, L.down, m->p_act16, flo, n, l + 1 < c.num_layers ? m->layers[l + 1].attn_norm : m->final_norm, nlo, st));
    }
    FORGE_TRY(gemm_f16a(m->d_logits, m->p_normed, nlo, m->lm_head, n, nullptr, m->d_err, st));
    if (greedy) FORGE_TRY(argmax_slices(m->d_tok, m->d_logits, m->V, n, m->d_amax_val, m->d_amax_idx, m->d_amax_ticket, st));
    return step_advance(kv->d_seq_len, n, m->d_step, st, nullptr);
}

int32_t decode_launches(ForgeModel* m, ForgeKV* kv, int batch, bool greedy, bool record, const PrefillToken* pt = nullptr) {
    const ForgeModelConfig& c = m->cfg;
    cudaStream_t st = m->stream;
    const int32_t* page_table = kv->d_page_table + (pt ? size_t(pt->seq) * kv->pages_per_seq : 0);
    int32_t* seq_len = kv->d_seq_len + (pt ? pt->seq : 0);
    // tensor-parallel sums over peer memory: the residual stream alternates between two buffers, because the kernel
    // that forms hidden + sum(parts) while staging writes it for its successors and other CTAs still read the old one
    const bool px = c.tp_world > 1 && m->tpx_ready && batch == 1 && !m->trace_on;
    float* hid[2] = {m->d_hidden, m->d_hidden2};
    int cur = 0;
    bool pending = false;  // a pushed sum has not been consumed yet
    int sums = 0;          // sums issued in this step so far (numbers them; slot = parity)
    auto tp_common = [&](GemvArgs& a, int index) {
        a.tp.world = c.tp_world; a.tp.rank = c.tp_rank; a.tp.slot = index & 1;
        a.tp.step_counter = m->d_tpx_step; a.tp.step_mul = uint32_t(2 * c.num_layers + 1); a.tp.step_add = uint32_t(index + 1);
        a.tp.wait_limit = m->wait_limit;
    };
    auto tp_consume = [&](GemvArgs& a) {   // a.x is the residual stream: take the pending sum in while staging
        if (!pending) return;
        tp_common(a, sums - 1);
        a.tp.consume = 1; a.tp.ll = static_cast<const uint2*>(m->tpx_local);
        a.tp.x_writeback = hid[cur ^ 1];
        cur ^= 1;
        pending = false;
    };
    auto tp_push = [&](const QTiled& w, GemvArgs a) -> int32_t {
        a.out = nullptr; a.resid = nullptr;
        tp_common(a, sums++);
        a.tp.consume = 0; a.tp.peer_ll = m->d_tpx_ll;
        pending = true;
        return gemv_tc(w, EPI_TP_PUSH, a, m->split, m->d_err, st);
    };
    if (batch >= 2 && !pt && m->uniform_basic && !m->trace_on) {
        // up to 8 sequences: the mma.sync streaming product; beyond: the tcgen05 products (their weight-streaming form up to
        // 32 rows, measured faster from about 16 rows on; the tile form for more)
        if (batch > kBatchGroup / 2 && m->lm_head.qs) return decode_launches_gemm(m, kv, batch, greedy, record);
        return decode_launches_batched(m, kv, batch, greedy, record);
    }
    FORGE_TRY(embedding_rows(m->d_hidden, m->embed, pt ? pt->tok : m->d_tok, batch, m->h, record ? m->d_hist : nullptr, m->d_step, st));
    for (int l = 0; l < c.num_layers; ++l) {
        ForgeLayer& L = m->layers[l];
        __half* kp = kv->k_pool + size_t(l) * kv->layer_stride;
        __half* vp = kv->v_pool + size_t(l) * kv->layer_stride;
        GemvArgs a;
        a.x = hid[cur]; a.norm_w = L.attn_norm; a.eps = c.rms_norm_eps; a.batch = batch;
        if (px) tp_consume(a);
        a.bias = L.qkv_bias; a.rope = m->rope; a.q_out = m->d_q; a.k_pool = kp; a.v_pool = vp;
        a.page_table = page_table; a.seq_len = seq_len; a.pages_per_seq = kv->pages_per_seq;
        a.qk = m->qk; a.kv = m->kv; a.kv_stride = m->kv; a.head_dim = m->hd;
        a.next_w = L.o_t.data; a.next_bytes = qtiled_bytes(L.o_t);
        if (L.v_t.data) { a.next_w = L.v_t.data; a.next_bytes = qtiled_bytes(L.v_t); }
        FORGE_TRY(gemv_tc(L.qkv_t, EPI_QKV, a, m->split, m->d_err, st));
        if (L.v_t.data) {
            // v_proj stored in its own format: a second product whose rows all land in the V cache (no rotation)
            GemvArgs v = a;
            v.tp = GemvArgs::Tp();
            v.qk = 0; v.kv = 0; v.q_out = nullptr;
            v.bias = L.qkv_bias ? L.qkv_bias + m->qk + m->kv : nullptr;
            v.next_w = L.o_t.data; v.next_bytes = qtiled_bytes(L.o_t);
            FORGE_TRY(gemv_tc(L.v_t, EPI_QKV, v, m->split, m->d_err, st));
        }
        AttnDecodeArgs da{m->d_attn, m->d_q, kp, vp, page_table, kv->pages_per_seq, seq_len, 0,
                          batch, m->nq, m->nkv, m->hd, kv->max_seq, kv->attn_ws, kv->attn_counters, kv->splits, c.sliding_window};
        da.map_k = kv->k_map; da.map_v = kv->v_map; da.row_base = int(size_t(l) * kv->num_pages * FORGE_KV_PAGE); da.err = m->d_err;
        FORGE_TRY(attn_decode(da, st));
        GemvArgs o;
        o.x = m->d_attn; o.out = hid[cur]; o.resid = hid[cur]; o.batch = batch;
        o.next_w = L.gateup_t.data; o.next_bytes = qtiled_bytes(L.gateup_t);
        if (px) FORGE_TRY(tp_push(L.o_t, o)); else FORGE_TRY(row_sliced_gemv(m, L.o_t, o, batch, st));
        GemvArgs g;
        g.x = hid[cur]; g.norm_w = L.ffn_norm; g.eps = c.rms_norm_eps; g.out = m->d_act; g.batch = batch;
        if (px) tp_consume(g);
        g.next_w = L.down_t.data; g.next_bytes = qtiled_bytes(L.down_t);
        FORGE_TRY(gemv_tc(L.gateup_t, EPI_SILU, g, m->split, m->d_err, st));
        GemvArgs d;
        d.x = m->d_act; d.out = hid[cur]; d.resid = hid[cur]; d.batch = batch;
        {   // the next projection on the stream: the next layer's QKV, or the head (a part of it: it is larger than L2)
            const QTiled& nx = l + 1 < c.num_layers ? m->layers[l + 1].qkv_t : m->lm_head_t;
            d.next_w = nx.data; d.next_bytes = std::min(qtiled_bytes(nx), size_t(48) << 20);
        }
        if (px) FORGE_TRY(tp_push(L.down_t, d)); else FORGE_TRY(row_sliced_gemv(m, L.down_t, d, batch, st));
        if (pt && pt->trace_dst)
            FORGE_CUDA(cudaMemcpyAsync(pt->trace_dst + size_t(l) * pt->trace_stride, m->d_hidden, sizeof(float) * m->h, cudaMemcpyDeviceToDevice, st));
        else if (m->trace_on && !pt)
            FORGE_CUDA(cudaMemcpyAsync(m->trace + size_t(l) * batch * m->h, m->d_hidden, sizeof(float) * batch * m->h, cudaMemcpyDeviceToDevice, st));
    }
    if (!pt || pt->head) {
        GemvArgs lm;
        lm.x = hid[cur]; lm.norm_w = m->final_norm; lm.eps = c.rms_norm_eps; lm.out = m->d_logits; lm.batch = batch;
        if (px) tp_consume(lm);
        FORGE_TRY(gemv_tc(m->lm_head_t, EPI_STORE, lm, m->split, m->d_err, st));
    }
    if (greedy) FORGE_TRY(argmax_slices(m->d_tok, m->d_logits, m->V, batch, m->d_amax_val, m->d_amax_idx, m->d_amax_ticket, st));
    FORGE_TRY(step_advance(seq_len, batch, pt ? nullptr : m->d_step, st, px ? m->d_tpx_step : nullptr));
    return FORGE_OK;
}

// forward_prefill, emit.rs:4511-5050: the generated module has batched products only for Q8_0 / Q4_0, so a model with
// K-quant projections takes its prompt through the per-token step, the head running for the last token only.  Pages
// for [base, base + n) are already reserved; the device-side length of the sequence advances with every token.
int32_t prefill_per_token(ForgeModel* m, ForgeKV* kv, int seq, const uint32_t* tokens_host, int n) {
    cudaStream_t st = m->stream;
    FORGE_TRY(ensure_decode_scratch(m, 1));
    if (m->trace_on) FORGE_TRY(ensure_trace(m, n));
    if (n > m->tok_cap) {
        FORGE_TRY(dev_alloc(m, &m->p_tokens, size_t(n)));
        m->tok_cap = n;
    }
    FORGE_CUDA(cudaMemcpyAsync(m->p_tokens, tokens_host, sizeof(uint32_t) * n, cudaMemcpyHostToDevice, st));
    FORGE_TRY(upload_len(kv));
    for (int i = 0; i < n; ++i) {
        PrefillToken pt{seq, m->p_tokens + i, i == n - 1, m->trace_on ? m->trace + size_t(i) * m->h : nullptr, size_t(n) * m->h};
        FORGE_TRY(decode_launches(m, kv, 1, false, false, &pt));
    }
    kv->len[seq] += n;
    return FORGE_OK;
}

// host bookkeeping before a decode step: pages for the new position of every sequence
int32_t decode_prepare(ForgeKV* kv, int batch) {
    for (int b = 0; b < batch; ++b) FORGE_TRY(ensure_pages(kv, b, kv->len[b] + 1));
    return FORGE_OK;
}

int32_t decode_step_graph(ForgeModel* m, ForgeKV* kv, int batch, bool greedy) {
    if (m->trace_on) return decode_launches(m, kv, batch, greedy, greedy);
    if (!kv->graph || kv->graph_batch != batch || kv->graph_greedy != greedy || kv->graph_gen != m->scratch_gen) {
        if (kv->graph) { cudaGraphExecDestroy(kv->graph); kv->graph = nullptr; }
        cudaGraph_t g = nullptr;
        FORGE_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        long long before = g_launches;
        int32_t rc = decode_launches(m, kv, batch, greedy, greedy);
        cudaError_t ce = cudaStreamEndCapture(m->stream, &g);
        if (rc != FORGE_OK) { if (g) cudaGraphDestroy(g); return rc; }
        if (ce != cudaSuccess) { set_error("graph capture: %s", cudaGetErrorString(ce)); return FORGE_ERR_CUDA; }
        g_launches = before;  // captured, not launched
        cudaError_t ie = cudaGraphInstantiate(&kv->graph, g, 0);
        cudaGraphDestroy(g);
        if (ie != cudaSuccess) { set_error("graph instantiate: %s", cudaGetErrorString(ie)); return FORGE_ERR_CUDA; }
        kv->graph_batch = batch; kv->graph_greedy = greedy; kv->graph_gen = m->scratch_gen;
    }
    FORGE_CUDA(cudaGraphLaunch(kv->graph, m->stream));
    // kernels inside one replay: embedding + 5 per layer + lm_head + (argmax) + advance
    g_launches += 1 + 5LL * m->cfg.num_layers + 1 + (greedy ? 1 : 0) + 1;
    return FORGE_OK;
}

int32_t check_seq(const ForgeKV* kv, int seq) {
    if (!kv || seq < 0 || seq >= kv->batch) { set_error("sequence index out of range"); return FORGE_ERR_INVALID_ARG; }
    if (!kv->model) { set_error("the model of this cache has been destroyed"); return FORGE_ERR_INVALID_ARG; }
    return FORGE_OK;
}

}  // namespace

// ------------------------------------------------------------------------------ C API
extern "C" {

const char* forge_last_error(void) { return g_error.c_str(); }

int32_t forge_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

size_t forge_weights_bin_size(const ForgeModelConfig* c) {
    if (!c) return 0;
    size_t h = c->hidden_size, qk = size_t(c->num_heads) * c->head_dim, kv = size_t(c->num_kv_heads) * c->head_dim;
    size_t ff = c->intermediate_size, V = c->vocab_size;
    int pq[8];
    proj_quants(c, pq);
    size_t per = h * 4 + raw_bytes(pq[PQ_Q], qk, h) + raw_bytes(pq[PQ_K], kv, h) + raw_bytes(pq[PQ_V], kv, h) + (c->qkv_bias ? (qk + 2 * kv) * 4 : 0) +
                 raw_bytes(pq[PQ_O], h, qk) + h * 4 + raw_bytes(pq[PQ_GATE], ff, h) + raw_bytes(pq[PQ_UP], ff, h) + raw_bytes(pq[PQ_DOWN], h, ff);
    return V * h * 4 + per * c->num_layers + h * 4 + raw_bytes(pq[PQ_LM], V, h);
}

int32_t forge_model_create(const ForgeModelConfig* cfg, const void* weights_bin, size_t len, int32_t device, ForgeModel** out) {
    if (!out) { set_error("null out pointer"); return FORGE_ERR_INVALID_ARG; }
    *out = nullptr;
    FORGE_TRY(check_cfg(cfg));
    if (!weights_bin) { set_error("null weights"); return FORGE_ERR_INVALID_ARG; }
    if (len != forge_weights_bin_size(cfg)) { set_error("weights.bin is %zu bytes, configuration needs %zu", len, forge_weights_bin_size(cfg)); return FORGE_ERR_SHAPE; }
    int ndev = forge_device_count();
    if (ndev == 0) { set_error("no CUDA device: this backend has no CPU fallback"); return FORGE_ERR_CUDA; }
    if (device < 0 || device >= ndev) { set_error("device %d out of range (%d visible)", device, ndev); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(device));
    ForgeModel* m = new ForgeModel();
    m->cfg = *cfg;
    if (m->cfg.tp_world < 1) { m->cfg.tp_world = 1; m->cfg.tp_rank = 0; }
    m->device = device;
    const int tp = m->cfg.tp_world, rk = m->cfg.tp_rank;
    proj_quants(cfg, m->pq);
    const int* pq = m->pq;
    const bool split_v = pq[PQ_V] != pq[PQ_Q];
    // The prompt takes the batched GEMMs unless q/k and v differ in a way the row-major layout cannot hold in one
    // matrix (a basic format next to anything else); K-quant inputs are rounded to Q8_0 blocks in front of each GEMM.
    m->per_token_prefill = split_v && !(is_kquant(pq[PQ_Q]) && is_kquant(pq[PQ_V]));
    for (int i = 0; i < 8; ++i) m->any_kquant = m->any_kquant || is_kquant(pq[i]);
    for (int i = 0; i < 8; ++i) m->uniform_basic = m->uniform_basic && pq[i] == cfg->quant && !is_kquant(pq[i]);
    const int H = cfg->hidden_size, QK = cfg->num_heads * cfg->head_dim, KV = cfg->num_kv_heads * cfg->head_dim, FF = cfg->intermediate_size;
    m->h = H; m->hd = cfg->head_dim; m->V = cfg->vocab_size;
    m->nq = cfg->num_heads / tp; m->nkv = cfg->num_kv_heads / tp;
    m->qk = QK / tp; m->kv = KV / tp; m->ff = FF / tp;
    m->max_seq = std::min(cfg->max_seq_len, 4096);  // emit.rs:178
    int32_t rc = FORGE_OK;
    auto fail = [&](int32_t code) { forge_model_destroy(m); return code; };
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) { set_error("cudaStreamCreate failed"); return fail(FORGE_ERR_CUDA); }
    for (auto& e : m->ev) if (cudaEventCreate(&e) != cudaSuccess) { set_error("cudaEventCreate failed"); return fail(FORGE_ERR_CUDA); }
    cudaStream_t st = m->stream;

    // Staging buffer for the raw blocks of one group of tensors (q,k,v | o | gate,up | down | lm_head): the
    // group is repacked on the device into (a) the row-major split layout the prefill GEMM reads and (b) the
    // tiled layout the decode GEMV streams, then the stage is reused.
    int sm_count = 148;
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    size_t max_raw = std::max({raw_bytes(pq[PQ_LM], size_t(cfg->vocab_size), H), 2 * raw_bytes(pq[PQ_GATE], FF, H) + 64,
                               raw_bytes(pq[PQ_Q], QK, H) + raw_bytes(pq[PQ_K], KV, H) + raw_bytes(pq[PQ_V], KV, H) + 64,
                               raw_bytes(pq[PQ_O], H, QK), raw_bytes(pq[PQ_DOWN], H, FF)});
    size_t max_rows = std::max({size_t(cfg->vocab_size), size_t(2 * FF), size_t(QK + 2 * KV), size_t(H)}) + 128;
    uint8_t* stage = nullptr;
    const uint8_t** d_rowsrc = nullptr;
    if (cudaMalloc(&stage, max_raw) != cudaSuccess || cudaMalloc(&d_rowsrc, max_rows * sizeof(uint8_t*)) != cudaSuccess) {
        set_error("staging allocation of %zu bytes failed", max_raw); cudaFree(stage); return fail(FORGE_ERR_CUDA);
    }
    const uint8_t* p = static_cast<const uint8_t*>(weights_bin);
    auto upload_f32 = [&](float** dst, size_t n, const uint8_t* src) -> int32_t {
        FORGE_TRY(dev_alloc(m, dst, n));
        FORGE_CUDA(cudaMemcpyAsync(*dst, src, n * 4, cudaMemcpyHostToDevice, st));
        return FORGE_OK;
    };
    // one source tensor of a group: raw [N_full][K_full/32] blocks on the host; this rank keeps rows
    // [row0, row0+rows) and blocks [blk0, blk0+blks), landing at destination rows dst_row0 + r*step
    struct Part { const uint8_t* host; int N_full, K_full, row0, rows, blk0, blks, dst_row0, step; int quant = 0; };
    // `quant`: the format of the parts (a part may name its own: K-quant rows of both kinds share the row-major
    // layout).  soa / tiled: which of the two layouts to build (null = skip).
    auto load_group = [&](int quant, const std::vector<Part>& parts, QWeight* soa, QTiled* tiled, int K_local, int N_local) -> int32_t {
        bool kq = false;
        for (const Part& pt : parts) kq = kq || is_kquant(pt.quant ? pt.quant : quant);
        if (soa) FORGE_TRY(alloc_qweight(m, *soa, kq ? FORGE_KQ_SOA : quant, K_local, N_local));
        std::vector<const uint8_t*> table;
        if (tiled) {
            tiled->K = K_local; tiled->N = N_local; tiled->quant = quant; tiled->bt = gemv_band_tiles(N_local, sm_count); tiled->bands = (N_local + 16 * tiled->bt - 1) / (16 * tiled->bt);
            FORGE_TRY(dev_alloc(m, &tiled->data, qtiled_bytes(quant, K_local, N_local, tiled->bt)));
            table.assign(size_t(tiled->bands) * 16 * tiled->bt, nullptr);
        }
        size_t off = 0;
        for (const Part& pt : parts) {
            const int pquant = pt.quant ? pt.quant : quant;
            const size_t bytes = raw_bytes(pquant, pt.N_full, pt.K_full);
            FORGE_CUDA(cudaMemcpyAsync(stage + off, pt.host, bytes, cudaMemcpyHostToDevice, st));
            if (soa) FORGE_TRY(pack_rows(stage + off, pquant, pt.K_full, pt.row0, pt.rows, pt.blk0, pt.blks, *soa, pt.dst_row0, pt.step, st));
            const size_t blk_bytes = is_kquant(pquant) ? 0 : (pquant == FORGE_Q8_0 ? 34 : 18);  // K-quant rows are never sliced along K (one rank)
            if (tiled)
                for (int r = 0; r < pt.rows; ++r)
                    table[size_t(pt.dst_row0) + size_t(r) * pt.step] = stage + off + size_t(pt.row0 + r) * raw_row_bytes(pquant, pt.K_full) + pt.blk0 * blk_bytes;
            off += (bytes + 15) & ~size_t(15);
        }
        if (tiled) {
            FORGE_CUDA(cudaMemcpyAsync(d_rowsrc, table.data(), table.size() * sizeof(uint8_t*), cudaMemcpyHostToDevice, st));
            FORGE_TRY(tile_pack(d_rowsrc, *tiled, st));
        }
        FORGE_CUDA(cudaStreamSynchronize(st));  // stage, table and the host vector are reused by the next group
        return FORGE_OK;
    };
#define MC(expr) do { rc = (expr); if (rc != FORGE_OK) { cudaFree(stage); cudaFree(d_rowsrc); return fail(rc); } } while (0)
    MC(upload_f32(&m->embed, size_t(cfg->vocab_size) * H, p));
    p += size_t(cfg->vocab_size) * H * 4;
    m->layers.resize(cfg->num_layers);
    for (int l = 0; l < cfg->num_layers; ++l) {
        ForgeLayer& L = m->layers[l];
        MC(upload_f32(&L.attn_norm, H, p)); p += size_t(H) * 4;
        const uint8_t* wq = p; p += raw_bytes(pq[PQ_Q], QK, H);
        const uint8_t* wk = p; p += raw_bytes(pq[PQ_K], KV, H);
        const uint8_t* wv = p; p += raw_bytes(pq[PQ_V], KV, H);
        if (!split_v) {
            MC(load_group(pq[PQ_Q], {{wq, QK, H, rk * m->qk, m->qk, 0, H / 32, 0, 1},
                                     {wk, KV, H, rk * m->kv, m->kv, 0, H / 32, m->qk, 1},
                                     {wv, KV, H, rk * m->kv, m->kv, 0, H / 32, m->qk + m->kv, 1}}, &L.qkv, &L.qkv_t, H, m->qk + 2 * m->kv));
        } else {
            // the streamed layout keeps V apart (its tiles differ); the row-major layout of the batched GEMM holds
            // [q ; k ; v] in one matrix when both formats are K-quants (they share that layout)
            MC(load_group(pq[PQ_Q], {{wq, QK, H, 0, m->qk, 0, H / 32, 0, 1}, {wk, KV, H, 0, m->kv, 0, H / 32, m->qk, 1}}, nullptr, &L.qkv_t, H, m->qk + m->kv));
            MC(load_group(pq[PQ_V], {{wv, KV, H, 0, m->kv, 0, H / 32, 0, 1}}, nullptr, &L.v_t, H, m->kv));
            if (!m->per_token_prefill)
                MC(load_group(pq[PQ_Q], {{wq, QK, H, 0, m->qk, 0, H / 32, 0, 1, pq[PQ_Q]}, {wk, KV, H, 0, m->kv, 0, H / 32, m->qk, 1, pq[PQ_K]},
                                         {wv, KV, H, 0, m->kv, 0, H / 32, m->qk + m->kv, 1, pq[PQ_V]}}, &L.qkv, nullptr, H, m->qk + 2 * m->kv));
        }
        if (cfg->qkv_bias) {
            MC(dev_alloc(m, &L.qkv_bias, size_t(m->qk + 2 * m->kv)));
            const float* bq = reinterpret_cast<const float*>(p);
            const float* bk = bq + QK; const float* bv = bk + KV;
            if (cudaMemcpyAsync(L.qkv_bias, bq + rk * m->qk, size_t(m->qk) * 4, cudaMemcpyHostToDevice, st) != cudaSuccess ||
                cudaMemcpyAsync(L.qkv_bias + m->qk, bk + rk * m->kv, size_t(m->kv) * 4, cudaMemcpyHostToDevice, st) != cudaSuccess ||
                cudaMemcpyAsync(L.qkv_bias + m->qk + m->kv, bv + rk * m->kv, size_t(m->kv) * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) {
                set_error("bias upload failed"); cudaFree(stage); cudaFree(d_rowsrc); return fail(FORGE_ERR_CUDA);
            }
            p += size_t(QK + 2 * KV) * 4;
        }
        MC(load_group(pq[PQ_O], {{p, H, QK, 0, H, rk * (m->qk / 32), m->qk / 32, 0, 1}}, &L.o, &L.o_t, m->qk, H)); p += raw_bytes(pq[PQ_O], H, QK);
        MC(upload_f32(&L.ffn_norm, H, p)); p += size_t(H) * 4;
        const uint8_t* pg = p; p += raw_bytes(pq[PQ_GATE], FF, H);
        const uint8_t* pu = p; p += raw_bytes(pq[PQ_UP], FF, H);
        MC(load_group(pq[PQ_GATE], {{pg, FF, H, rk * m->ff, m->ff, 0, H / 32, 0, 2}, {pu, FF, H, rk * m->ff, m->ff, 0, H / 32, 1, 2}},
                      &L.gateup, &L.gateup_t, H, 2 * m->ff));
        MC(load_group(pq[PQ_DOWN], {{p, H, FF, 0, H, rk * (m->ff / 32), m->ff / 32, 0, 1}}, &L.down, &L.down_t, m->ff, H)); p += raw_bytes(pq[PQ_DOWN], H, FF);
    }
    MC(upload_f32(&m->final_norm, H, p)); p += size_t(H) * 4;
    MC(load_group(pq[PQ_LM], {{p, cfg->vocab_size, H, 0, cfg->vocab_size, 0, H / 32, 0, 1}}, pq[PQ_LM] == FORGE_Q8_0 || pq[PQ_LM] == FORGE_Q4_0 ? &m->lm_head : nullptr, &m->lm_head_t, H, cfg->vocab_size));
    MC(dev_alloc(m, &m->d_err, 1));
    MC(dev_alloc(m, &m->split.scratch, size_t(kGemvMaxSlices) * kGemvSplitRows));
    MC(dev_alloc(m, &m->split.tickets, size_t(kGemvSplitRows) / 16));
    m->split.max_slices = kGemvMaxSlices;
    if (cudaMemsetAsync(m->split.tickets, 0, sizeof(int) * kGemvSplitRows / 16, st) != cudaSuccess) { set_error("memset failed"); cudaFree(stage); cudaFree(d_rowsrc); return fail(FORGE_ERR_CUDA); }
    if (cudaMemsetAsync(m->d_err, 0, sizeof(int), st) != cudaSuccess) { set_error("memset failed"); cudaFree(stage); cudaFree(d_rowsrc); return fail(FORGE_ERR_CUDA); }
    cudaFree(d_rowsrc);
    cudaFree(stage);
    // RoPE table with the host libm, f32 (emit.rs:502-519)
    {
        std::vector<float> tab(size_t(m->max_seq) * m->hd);
        forge_rope_table(tab.data(), m->max_seq, m->hd, cfg->rope_theta);
        rc = dev_alloc(m, &m->rope, tab.size());
        if (rc != FORGE_OK) return fail(rc);
        if (cudaMemcpyAsync(m->rope, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) { set_error("rope table upload failed"); return fail(FORGE_ERR_CUDA); }
    }
#undef MC
    if (cudaStreamSynchronize(st) != cudaSuccess) { set_error("weight upload failed: %s", cudaGetErrorString(cudaGetLastError())); return fail(FORGE_ERR_CUDA); }
    *out = m;
    return FORGE_OK;
}

static void kv_release_device(ForgeKV* kv);

void forge_model_destroy(ForgeModel* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    if (m->stream) cudaStreamSynchronize(m->stream);
    for (ForgeKV* kv : m->caches) kv_release_device(kv);
    m->caches.clear();
    tp_destroy(m->tp);
    for (void* q : m->tpx_peer) if (q) cudaIpcCloseMemHandle(q);
    if (m->tpx_local) cudaFree(m->tpx_local);
    for (void* q : m->allocs) cudaFree(q);
    for (auto& e : m->ev) if (e) cudaEventDestroy(e);
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
}

void* forge_model_stream(ForgeModel* m) { return m ? static_cast<void*>(m->stream) : nullptr; }
size_t forge_model_vocab_size(const ForgeModel* m) { return m ? size_t(m->V) : 0; }

int32_t forge_model_tp_exchange_export(ForgeModel* m, uint8_t* handle_out) {
    if (!m || !handle_out) { set_error("bad argument to forge_model_tp_exchange_export"); return FORGE_ERR_INVALID_ARG; }
    if (m->cfg.tp_world < 2 || m->cfg.tp_world > 16) { set_error("peer exchange needs 2..16 tensor-parallel ranks"); return FORGE_ERR_INVALID_ARG; }
    static_assert(sizeof(cudaIpcMemHandle_t) == FORGE_TP_HANDLE_BYTES, "FORGE_TP_HANDLE_BYTES must match cudaIpcMemHandle_t");
    FORGE_CUDA(cudaSetDevice(m->device));
    if (!m->tpx_local) {
        FORGE_CUDA(cudaMalloc(&m->tpx_local, tpx_bytes(m)));
        FORGE_CUDA(cudaMemset(m->tpx_local, 0, tpx_bytes(m)));
        FORGE_CUDA(cudaDeviceSynchronize());
    }
    cudaIpcMemHandle_t h;
    FORGE_CUDA(cudaIpcGetMemHandle(&h, m->tpx_local));
    memcpy(handle_out, &h, sizeof(h));
    return FORGE_OK;
}

int32_t forge_model_tp_exchange_attach(ForgeModel* m, const uint8_t* handles) {
    if (!m || !handles) { set_error("bad argument to forge_model_tp_exchange_attach"); return FORGE_ERR_INVALID_ARG; }
    if (!m->tpx_local) { set_error("call forge_model_tp_exchange_export first"); return FORGE_ERR_INVALID_ARG; }
    if (m->tpx_ready) { set_error("the exchange is already attached"); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    const int world = m->cfg.tp_world, rank = m->cfg.tp_rank;
    m->tpx_peer.assign(world, nullptr);
    std::vector<uint2*> ll(world);
    for (int r = 0; r < world; ++r) {
        void* base = m->tpx_local;
        cudaIpcMemHandle_t own;
        FORGE_CUDA(cudaIpcGetMemHandle(&own, m->tpx_local));
        // a peer entry that repeats this rank's own handle maps the local buffer: nothing will ever be pushed into that
        // slot, which is how a single-process test makes the bounded peer wait run out
        if (r != rank && memcmp(&own, handles + size_t(r) * FORGE_TP_HANDLE_BYTES, sizeof(own)) != 0) {
            cudaIpcMemHandle_t h;
            memcpy(&h, handles + size_t(r) * FORGE_TP_HANDLE_BYTES, sizeof(h));
            cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) { set_error("cudaIpcOpenMemHandle(rank %d): %s", r, cudaGetErrorString(e)); return FORGE_ERR_COMM; }
            m->tpx_peer[r] = base;
        }
        ll[r] = static_cast<uint2*>(base);
    }
    FORGE_TRY(dev_alloc(m, &m->d_tpx_ll, size_t(world)));
    FORGE_TRY(dev_alloc(m, &m->d_tpx_step, 1));
    FORGE_CUDA(cudaMemcpy(m->d_tpx_ll, ll.data(), sizeof(uint2*) * world, cudaMemcpyHostToDevice));
    FORGE_CUDA(cudaMemset(m->d_tpx_step, 0, sizeof(uint32_t)));
    FORGE_CUDA(cudaDeviceSynchronize());
    m->tpx_ready = true;
    return FORGE_OK;
}

int32_t forge_tp_unique_id(uint8_t* id_out) {
    if (!id_out) { set_error("null id buffer"); return FORGE_ERR_INVALID_ARG; }
    return tp_unique_id(id_out);
}

int32_t forge_model_tp_init(ForgeModel* m, const uint8_t* id) {
    if (!m || !id) { set_error("bad argument to forge_model_tp_init"); return FORGE_ERR_INVALID_ARG; }
    if (m->cfg.tp_world < 2) { set_error("the model was created with tp_world = 1"); return FORGE_ERR_INVALID_ARG; }
    if (m->tp) { set_error("the model already has a communicator"); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    return tp_init(&m->tp, id, m->cfg.tp_rank, m->cfg.tp_world);
}

int32_t forge_kv_create(ForgeModel* m, int32_t max_seq, int32_t batch, ForgeKV** out) {
    if (!m || !out || max_seq <= 0 || batch <= 0) { set_error("bad argument to forge_kv_create"); return FORGE_ERR_INVALID_ARG; }
    *out = nullptr;
    FORGE_CUDA(cudaSetDevice(m->device));
    ForgeKV* kv = new ForgeKV();
    kv->model = m;
    kv->max_seq = std::min(max_seq, m->max_seq);
    kv->batch = batch;
    kv->pages_per_seq = (kv->max_seq + FORGE_KV_PAGE - 1) / FORGE_KV_PAGE;
    kv->num_pages = kv->pages_per_seq * batch;
    kv->layer_stride = size_t(kv->num_pages) * FORGE_KV_PAGE * m->kv;
    size_t pool = kv->layer_stride * m->cfg.num_layers;
    auto fail = [&](int32_t code) { forge_kv_destroy(kv); return code; };
    if (cudaMalloc(&kv->k_pool, pool * sizeof(__half)) != cudaSuccess || cudaMalloc(&kv->v_pool, pool * sizeof(__half)) != cudaSuccess) {
        set_error("KV pool allocation of %zu bytes failed", 2 * pool * sizeof(__half)); cudaGetLastError(); return fail(FORGE_ERR_CUDA);
    }
    static_assert(sizeof(kv->k_map) >= 128, "CUtensorMap is 128 bytes");
    {
        const size_t rows = size_t(kv->num_pages) * FORGE_KV_PAGE * m->cfg.num_layers;
        int32_t rc = make_kv_map(kv->k_map, kv->k_pool, m->hd, m->nkv, rows);
        if (rc == FORGE_OK) rc = make_kv_map(kv->v_map, kv->v_pool, m->hd, m->nkv, rows);
        if (rc != FORGE_OK) return fail(rc);
    }
    cudaMemsetAsync(kv->k_pool, 0, pool * sizeof(__half), m->stream);
    cudaMemsetAsync(kv->v_pool, 0, pool * sizeof(__half), m->stream);
    if (cudaMalloc(&kv->d_page_table, sizeof(int32_t) * kv->num_pages) != cudaSuccess || cudaMalloc(&kv->d_seq_len, sizeof(int32_t) * batch) != cudaSuccess)
        { set_error("KV table allocation failed"); return fail(FORGE_ERR_CUDA); }
    cudaMemsetAsync(kv->d_page_table, 0, sizeof(int32_t) * kv->num_pages, m->stream);
    cudaMemsetAsync(kv->d_seq_len, 0, sizeof(int32_t) * batch, m->stream);
    kv->h_page_table.assign(kv->num_pages, 0);
    kv->pages_used.assign(batch, 0);
    kv->len.assign(batch, 0);
    for (int i = kv->num_pages - 1; i >= 0; --i) kv->free_pages.push_back(i);
    // split-KV: enough CTAs to fill the SMs
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, m->device);
    kv->splits = attn_decode_splits(kv->pages_per_seq, batch * m->nkv, sms, m->hd, m->nq / m->nkv);
    if (cudaMalloc(&kv->attn_ws, sizeof(float) * attn_decode_ws_floats(batch, m->nq, m->hd, kv->splits)) != cudaSuccess ||
        cudaMalloc(&kv->attn_counters, sizeof(int) * batch * m->nkv) != cudaSuccess) { set_error("attention workspace allocation failed"); return fail(FORGE_ERR_CUDA); }
    cudaMemsetAsync(kv->attn_counters, 0, sizeof(int) * batch * m->nkv, m->stream);
    if (cudaStreamSynchronize(m->stream) != cudaSuccess) { set_error("KV init failed"); return fail(FORGE_ERR_CUDA); }
    m->caches.push_back(kv);
    *out = kv;
    return FORGE_OK;
}

int32_t forge_kv_reset(ForgeKV* kv) {
    if (!kv || !kv->model) { set_error("null kv, or a cache whose model has been destroyed"); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(kv->model->device));
    FORGE_CUDA(cudaStreamSynchronize(kv->model->stream));
    std::fill(kv->len.begin(), kv->len.end(), 0);
    std::fill(kv->pages_used.begin(), kv->pages_used.end(), 0);
    kv->free_pages.clear();
    for (int i = kv->num_pages - 1; i >= 0; --i) kv->free_pages.push_back(i);
    return upload_len(kv);
}

int32_t forge_kv_len(const ForgeKV* kv, int32_t seq) { return (kv && seq >= 0 && seq < kv->batch) ? kv->len[seq] : -1; }

void forge_kv_destroy(ForgeKV* kv) {
    if (!kv) return;
    if (!kv->model) { delete kv; return; }  // the model went first and took the device memory with it
    cudaSetDevice(kv->model->device);
    cudaStreamSynchronize(kv->model->stream);
    auto& reg = kv->model->caches;
    reg.erase(std::remove(reg.begin(), reg.end(), kv), reg.end());
    if (kv->graph) cudaGraphExecDestroy(kv->graph);
    cudaFree(kv->k_pool); cudaFree(kv->v_pool); cudaFree(kv->d_page_table); cudaFree(kv->d_seq_len);
    cudaFree(kv->attn_ws); cudaFree(kv->attn_counters);
    delete kv;
}

// device memory of a cache whose model is being destroyed; the handle itself stays valid for forge_kv_destroy
static void kv_release_device(ForgeKV* kv) {
    if (kv->graph) cudaGraphExecDestroy(kv->graph);
    cudaFree(kv->k_pool); cudaFree(kv->v_pool); cudaFree(kv->d_page_table); cudaFree(kv->d_seq_len);
    cudaFree(kv->attn_ws); cudaFree(kv->attn_counters);
    kv->graph = nullptr; kv->k_pool = kv->v_pool = nullptr; kv->d_page_table = kv->d_seq_len = nullptr;
    kv->attn_ws = nullptr; kv->attn_counters = nullptr;
    kv->model = nullptr;
}

int32_t forge_kv_read(ForgeKV* kv, int32_t seq, int32_t layer, int32_t which, float* out_host) {
    FORGE_TRY(check_seq(kv, seq));
    ForgeModel* m = kv->model;
    if (layer < 0 || layer >= m->cfg.num_layers || !out_host) { set_error("bad argument to forge_kv_read"); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    int len = kv->len[seq];
    if (len == 0) return FORGE_OK;
    float* tmp = nullptr;
    FORGE_CUDA(cudaMalloc(&tmp, sizeof(float) * len * m->kv));
    const __half* pool = (which ? kv->v_pool : kv->k_pool) + size_t(layer) * kv->layer_stride;
    int32_t rc = gather_rows_f16(tmp, pool, kv->d_page_table + size_t(seq) * kv->pages_per_seq, len, m->kv, m->stream);
    if (rc == FORGE_OK && (cudaMemcpyAsync(out_host, tmp, sizeof(float) * len * m->kv, cudaMemcpyDeviceToHost, m->stream) != cudaSuccess ||
                           cudaStreamSynchronize(m->stream) != cudaSuccess)) { set_error("kv read copy failed"); rc = FORGE_ERR_CUDA; }
    cudaFree(tmp);
    return rc;
}

// ---- corpus scoring (--score-corpus, project.rs:652-712): per-token forward() over one chunk from an empty cache; the
// negative log-likelihood of every next token is formed on the device from the logits row, so no logits leave the GPU
int32_t forge_score_chunk(ForgeModel* m, ForgeKV* kv, const uint32_t* chunk, size_t n, double* nll_host) {
    if (!m || !chunk || !nll_host || n < 2 || n > (1u << 20)) { set_error("bad argument to forge_score_chunk"); return FORGE_ERR_INVALID_ARG; }
    FORGE_TRY(check_seq(kv, 0));
    if (kv->model != m) { set_error("kv belongs to another model"); return FORGE_ERR_INVALID_ARG; }
    if (int(n) - 1 > kv->max_seq) { set_error("chunk of %zu tokens does not fit the cache (max_seq %d)", n, kv->max_seq); return FORGE_ERR_KV_FULL; }
    for (size_t i = 0; i < n; ++i) if (chunk[i] >= uint32_t(m->V)) { set_error("token id %u out of vocabulary", chunk[i]); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    FORGE_TRY(forge_kv_reset(kv));
    double* d_nll = nullptr;
    FORGE_CUDA(cudaMalloc(&d_nll, sizeof(double) * (n - 1)));
    int32_t rc = FORGE_OK;
    for (size_t i = 0; i + 1 < n && rc == FORGE_OK; ++i) {
        rc = forge_forward_seq(m, kv, 0, chunk[i], nullptr);                       // logits of position i stay in d_logits
        if (rc == FORGE_OK) rc = token_nll(d_nll + i, m->d_logits, m->V, chunk[i + 1], m->stream);
    }
    if (rc == FORGE_OK && (cudaMemcpyAsync(nll_host, d_nll, sizeof(double) * (n - 1), cudaMemcpyDeviceToHost, m->stream) != cudaSuccess ||
                           cudaStreamSynchronize(m->stream) != cudaSuccess)) { set_error("score copy failed"); rc = FORGE_ERR_CUDA; }
    cudaFree(d_nll);
    return rc;
}

// ---- persistence (project.rs:456-499)
namespace {
constexpr char kKvMagic[4] = {'F', 'K', 'V', '1'};
// 24 bytes on disk: magic 'FKV1' | u32 layers | u32 width (values per cache row) | u32 zero | u64 positions
struct KvHeader { char magic[4]; uint32_t layers, width, reserved; uint64_t len; };
static_assert(sizeof(KvHeader) == 24, "the saved-cache header is a fixed 24-byte layout");

// one layer's rows [0, len) of K or V between the paged pool and a contiguous host array [len][width] of fp16
int32_t kv_copy_rows(ForgeKV* kv, int seq, int layer, int which, int len, __half* host, bool to_host) {
    ForgeModel* m = kv->model;
    __half* pool = (which ? kv->v_pool : kv->k_pool) + size_t(layer) * kv->layer_stride;
    for (int lp = 0; lp * FORGE_KV_PAGE < len; ++lp) {
        const int rows = std::min(FORGE_KV_PAGE, len - lp * FORGE_KV_PAGE);
        const int page = kv->h_page_table[size_t(seq) * kv->pages_per_seq + lp];
        __half* dev = pool + size_t(page) * FORGE_KV_PAGE * m->kv;
        __half* hst = host + size_t(lp) * FORGE_KV_PAGE * m->kv;
        const size_t bytes = sizeof(__half) * size_t(rows) * m->kv;
        FORGE_CUDA(to_host ? cudaMemcpyAsync(hst, dev, bytes, cudaMemcpyDeviceToHost, m->stream)
                           : cudaMemcpyAsync(dev, hst, bytes, cudaMemcpyHostToDevice, m->stream));
    }
    return FORGE_OK;
}
}  // namespace

size_t forge_kv_save_size(const ForgeKV* kv, int32_t seq) {
    if (!kv || !kv->model || seq < 0 || seq >= kv->batch) return 0;
    const ForgeModel* m = kv->model;
    return sizeof(KvHeader) + size_t(2) * m->cfg.num_layers * kv->len[seq] * m->kv * sizeof(__half);
}

int32_t forge_kv_save(ForgeKV* kv, int32_t seq, void* out_host, size_t capacity) {
    FORGE_TRY(check_seq(kv, seq));
    ForgeModel* m = kv->model;
    if (!out_host || capacity < forge_kv_save_size(kv, seq)) { set_error("forge_kv_save: buffer too small"); return FORGE_ERR_INVALID_ARG; }
    if (m->cfg.tp_world > 1) { set_error("forge_kv_save: a tensor-parallel cache holds only this rank's heads"); return FORGE_ERR_UNSUPPORTED; }
    FORGE_CUDA(cudaSetDevice(m->device));
    const int len = kv->len[seq], L = m->cfg.num_layers;
    KvHeader h{};
    memcpy(h.magic, kKvMagic, 4); h.layers = uint32_t(L); h.width = uint32_t(m->kv); h.len = uint64_t(len);
    memcpy(out_host, &h, sizeof(h));
    __half* dst = reinterpret_cast<__half*>(static_cast<char*>(out_host) + sizeof(h));
    for (int which = 0; which < 2; ++which)
        for (int l = 0; l < L; ++l) FORGE_TRY(kv_copy_rows(kv, seq, l, which, len, dst + (size_t(which) * L + l) * len * m->kv, true));
    FORGE_CUDA(cudaStreamSynchronize(m->stream));
    return FORGE_OK;
}

int32_t forge_kv_load(ForgeKV* kv, int32_t seq, const void* data_host, size_t n) {
    FORGE_TRY(check_seq(kv, seq));
    ForgeModel* m = kv->model;
    if (!data_host || n < 8) { set_error("forge_kv_load: no data"); return FORGE_ERR_INVALID_ARG; }
    if (m->cfg.tp_world > 1) { set_error("forge_kv_load: a tensor-parallel cache holds only this rank's heads"); return FORGE_ERR_UNSUPPORTED; }
    FORGE_CUDA(cudaSetDevice(m->device));
    const int L = m->cfg.num_layers;
    const size_t W = size_t(m->kv);
    const uint8_t* p = static_cast<const uint8_t*>(data_host);
    std::vector<__half> rows;  // [2][L][len][W]
    uint64_t len = 0;
    if (n >= sizeof(KvHeader) && memcmp(p, kKvMagic, 4) == 0) {
        KvHeader h;
        memcpy(&h, p, sizeof(h));
        if (h.layers != uint32_t(L) || h.width != uint32_t(W)) { set_error("forge_kv_load: the file is for %u layers x %u, the model has %d x %zu", h.layers, h.width, L, W); return FORGE_ERR_SHAPE; }
        len = h.len;
        if (len > uint64_t(kv->max_seq) || n != sizeof(h) + size_t(2) * L * len * W * sizeof(__half)) { set_error("forge_kv_load: bad length"); return FORGE_ERR_SHAPE; }
        rows.resize(size_t(2) * L * len * W);
        memcpy(rows.data(), p + sizeof(h), rows.size() * sizeof(__half));
    } else {
        // the reference's int8 file: u64 len | K i8 [L][len*W] | V i8 [L][len*W] | k_scales f32 [L][len] | v_scales f32 [L][len]
        memcpy(&len, p, 8);
        if (len > uint64_t(kv->max_seq) || n != 8 + size_t(2) * L * len * W + size_t(2) * L * len * 4) { set_error("forge_kv_load: not a cache file of this model (%zu bytes)", n); return FORGE_ERR_SHAPE; }
        const int8_t* q = reinterpret_cast<const int8_t*>(p + 8);
        const uint8_t* sc = p + 8 + size_t(2) * L * len * W;
        rows.resize(size_t(2) * L * len * W);
        for (size_t wl = 0; wl < size_t(2) * L; ++wl)
            for (size_t t = 0; t < len; ++t) {
                float s;
                memcpy(&s, sc + (wl * len + t) * 4, 4);
                for (size_t i = 0; i < W; ++i) rows[(wl * len + t) * W + i] = __float2half_rn(float(q[(wl * len + t) * W + i]) * s);
            }
    }
    // the sequence starts over: its pages go back to the pool, then the saved rows are written
    FORGE_CUDA(cudaStreamSynchronize(m->stream));
    for (int i = 0; i < kv->pages_used[seq]; ++i) kv->free_pages.push_back(kv->h_page_table[size_t(seq) * kv->pages_per_seq + i]);
    kv->pages_used[seq] = 0;
    kv->len[seq] = 0;
    FORGE_TRY(ensure_pages(kv, seq, int(len)));
    for (int which = 0; which < 2; ++which)
        for (int l = 0; l < L; ++l) FORGE_TRY(kv_copy_rows(kv, seq, l, which, int(len), rows.data() + (size_t(which) * L + l) * len * W, false));
    FORGE_CUDA(cudaStreamSynchronize(m->stream));
    kv->len[seq] = int(len);
    return upload_len(kv);
}

int32_t forge_forward_prefill_seq(ForgeModel* m, ForgeKV* kv, int32_t seq, const uint32_t* tokens, size_t n, float* logits_host) {
    if (!m || !tokens || n == 0 || n > (1u << 20)) { set_error("bad argument to forge_forward_prefill"); return FORGE_ERR_INVALID_ARG; }
    FORGE_TRY(check_seq(kv, seq));
    if (kv->model != m) { set_error("kv belongs to another model"); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    for (size_t i = 0; i < n; ++i) if (tokens[i] >= uint32_t(m->V)) { set_error("token id %u out of vocabulary", tokens[i]); return FORGE_ERR_INVALID_ARG; }
    if (kv->len[seq] + int(n) > kv->max_seq) { set_error("KV cache full: %d + %zu > max_seq %d", kv->len[seq], n, kv->max_seq); return FORGE_ERR_KV_FULL; }
    if (n < FORGE_PREFILL_BATCH_THRESHOLD && !m->trace_on) {
        // emit.rs:4581: short prompts take the per-token path
        for (size_t i = 0; i < n; ++i) FORGE_TRY(forge_forward_seq(m, kv, seq, tokens[i], (i + 1 == n) ? logits_host : nullptr));
        return FORGE_OK;
    }
    const int len0 = kv->len[seq];
    FORGE_TRY(prefill_seq(m, kv, seq, tokens, int(n)));
    FORGE_TRY(upload_len(kv));
    if (logits_host) FORGE_CUDA(cudaMemcpyAsync(logits_host, m->d_logits, sizeof(float) * m->V, cudaMemcpyDeviceToHost, m->stream));
    kv->len[seq] = len0;   // until the check has passed
    FORGE_TRY(sync_and_check(m, kv));
    kv->len[seq] = len0 + int(n);
    return upload_len(kv);
}

int32_t forge_forward_prefill(ForgeModel* m, ForgeKV* kv, const uint32_t* tokens, size_t n, float* logits_host) {
    return forge_forward_prefill_seq(m, kv, 0, tokens, n, logits_host);
}

// single sequence `seq` of a multi-sequence cache: runs the batch-1 launch sequence on views of that sequence
int32_t forge_forward_seq(ForgeModel* m, ForgeKV* kv, int32_t seq, uint32_t token, float* logits_host) {
    if (!m) { set_error("null model"); return FORGE_ERR_INVALID_ARG; }
    FORGE_TRY(check_seq(kv, seq));
    if (kv->model != m) { set_error("kv belongs to another model"); return FORGE_ERR_INVALID_ARG; }
    if (token >= uint32_t(m->V)) { set_error("token id %u out of vocabulary", token); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    FORGE_TRY(ensure_decode_scratch(m, 1));
    FORGE_TRY(ensure_pages(kv, seq, kv->len[seq] + 1));
    if (m->trace_on) FORGE_TRY(ensure_trace(m, 1));
    FORGE_CUDA(cudaMemcpyAsync(m->d_tok, &token, sizeof(uint32_t), cudaMemcpyHostToDevice, m->stream));
    // view of sequence `seq` as a batch of one
    ForgeKV view = *kv;
    view.d_page_table = kv->d_page_table + size_t(seq) * kv->pages_per_seq;
    view.d_seq_len = kv->d_seq_len + seq;
    view.graph = nullptr;
    int32_t rc;
    if (seq == 0 && kv->batch >= 1 && !m->trace_on) {
        rc = decode_step_graph(m, kv, 1, false);
    } else {
        rc = decode_launches(m, &view, 1, false, false);
    }
    view.h_page_table.clear();
    FORGE_TRY(rc);
    if (logits_host) FORGE_CUDA(cudaMemcpyAsync(logits_host, m->d_logits, sizeof(float) * m->V, cudaMemcpyDeviceToHost, m->stream));
    FORGE_TRY(sync_and_check(m, kv));
    kv->len[seq] += 1;
    return FORGE_OK;
}

int32_t forge_forward(ForgeModel* m, ForgeKV* kv, uint32_t token, float* logits_host) { return forge_forward_seq(m, kv, 0, token, logits_host); }

int32_t forge_forward_batch(ForgeModel* m, ForgeKV* kv, int32_t batch, const uint32_t* tokens, float* logits_host) {
    if (!m || !kv || !tokens || batch <= 0 || batch > kv->batch || kv->model != m) { set_error("bad argument to forge_forward_batch"); return FORGE_ERR_INVALID_ARG; }
    for (int b = 0; b < batch; ++b) if (tokens[b] >= uint32_t(m->V)) { set_error("token id %u out of vocabulary", tokens[b]); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    FORGE_TRY(ensure_decode_scratch(m, batch));
    FORGE_TRY(decode_prepare(kv, batch));
    if (m->trace_on) FORGE_TRY(ensure_trace(m, batch));
    FORGE_CUDA(cudaMemcpyAsync(m->d_tok, tokens, sizeof(uint32_t) * batch, cudaMemcpyHostToDevice, m->stream));
    FORGE_TRY(decode_step_graph(m, kv, batch, false));
    if (logits_host) FORGE_CUDA(cudaMemcpyAsync(logits_host, m->d_logits, sizeof(float) * size_t(batch) * m->V, cudaMemcpyDeviceToHost, m->stream));
    FORGE_TRY(sync_and_check(m, kv));
    for (int b = 0; b < batch; ++b) kv->len[b] += 1;
    return FORGE_OK;
}

static int32_t ensure_hist(ForgeModel* m, int n) {
    if (n > m->hist_cap) { FORGE_TRY(dev_alloc(m, &m->d_hist, size_t(n))); m->hist_cap = n; }
    return FORGE_OK;
}

int32_t forge_decode_greedy_batch(ForgeModel* m, ForgeKV* kv, int32_t batch, const uint32_t* first_tokens, int32_t n_new, uint32_t* out_tokens) {
    if (!m || !kv || !first_tokens || !out_tokens || batch <= 0 || batch > kv->batch || n_new <= 0 || kv->model != m) { set_error("bad argument to forge_decode_greedy_batch"); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    for (int b = 0; b < batch; ++b) {
        if (first_tokens[b] >= uint32_t(m->V)) { set_error("token id out of vocabulary"); return FORGE_ERR_INVALID_ARG; }
        if (kv->len[b] + n_new > kv->max_seq) { set_error("KV cache full: %d + %d > max_seq %d", kv->len[b], n_new, kv->max_seq); return FORGE_ERR_KV_FULL; }
    }
    FORGE_TRY(ensure_decode_scratch(m, batch));
    FORGE_TRY(ensure_hist(m, n_new * batch));
    long long l0 = g_launches;
    FORGE_CUDA(cudaMemcpyAsync(m->d_tok, first_tokens, sizeof(uint32_t) * batch, cudaMemcpyHostToDevice, m->stream));
    FORGE_CUDA(cudaMemsetAsync(m->d_step, 0, sizeof(int32_t), m->stream));
    FORGE_CUDA(cudaEventRecord(m->ev[1], m->stream));
    bool saved_trace = m->trace_on;
    m->trace_on = false;
    const std::vector<int> len0 = kv->len;
    int32_t rc = FORGE_OK;
    for (int i = 0; i < n_new && rc == FORGE_OK; ++i) {
        rc = decode_prepare(kv, batch);
        if (rc == FORGE_OK) rc = decode_step_graph(m, kv, batch, true);
        if (rc == FORGE_OK) for (int b = 0; b < batch; ++b) kv->len[b] += 1;
    }
    m->trace_on = saved_trace;
    if (rc != FORGE_OK) { cudaStreamSynchronize(m->stream); kv->len = len0; upload_len(kv); return rc; }
    FORGE_CUDA(cudaEventRecord(m->ev[2], m->stream));
    FORGE_CUDA(cudaMemcpyAsync(out_tokens, m->d_hist, sizeof(uint32_t) * size_t(n_new) * batch, cudaMemcpyDeviceToHost, m->stream));
    {
        const std::vector<int> len1 = kv->len;
        kv->len = len0;   // what the device is put back to if the check fails
        FORGE_TRY(sync_and_check(m, kv));
        kv->len = len1;
    }
    FORGE_CUDA(cudaEventElapsedTime(&m->decode_ms, m->ev[1], m->ev[2]));
    m->last_launches = g_launches - l0;
    return FORGE_OK;
}

int32_t forge_generate_greedy(ForgeModel* m, ForgeKV* kv, const uint32_t* prompt, size_t n, int32_t n_new, uint32_t* out_tokens) {
    if (!m || !kv || !prompt || !out_tokens || n == 0 || n_new <= 0 || kv->model != m) { set_error("bad argument to forge_generate_greedy"); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    if (kv->len[0] + int(n) + n_new > kv->max_seq) { set_error("KV cache full: %d + %zu + %d > max_seq %d", kv->len[0], n, n_new, kv->max_seq); return FORGE_ERR_KV_FULL; }
    for (size_t i = 0; i < n; ++i) if (prompt[i] >= uint32_t(m->V)) { set_error("token id %u out of vocabulary", prompt[i]); return FORGE_ERR_INVALID_ARG; }
    FORGE_TRY(ensure_decode_scratch(m, 1));
    long long l0 = g_launches;
    const int len_entry = kv->len[0];
    FORGE_CUDA(cudaEventRecord(m->ev[0], m->stream));
    if (n < FORGE_PREFILL_BATCH_THRESHOLD) {
        for (size_t i = 0; i < n; ++i) FORGE_TRY(forge_forward_seq(m, kv, 0, prompt[i], nullptr));
    } else {
        FORGE_TRY(prefill_seq(m, kv, 0, prompt, int(n)));
        FORGE_TRY(upload_len(kv));
    }
    // first token: sample() of the prefill logits (project.rs:722)
    FORGE_TRY(argmax_slices(m->d_tok, m->d_logits, m->V, 1, m->d_amax_val, m->d_amax_idx, m->d_amax_ticket, m->stream));
    uint32_t first = 0;
    FORGE_CUDA(cudaMemcpyAsync(&first, m->d_tok, sizeof(uint32_t), cudaMemcpyDeviceToHost, m->stream));
    {
        const int len1 = kv->len[0];
        kv->len[0] = len_entry;
        FORGE_TRY(sync_and_check(m, kv));
        kv->len[0] = len1;
    }
    long long lp = g_launches - l0;
    int32_t rc = forge_decode_greedy_batch(m, kv, 1, &first, n_new, out_tokens);
    if (rc != FORGE_OK) return rc;
    FORGE_CUDA(cudaEventElapsedTime(&m->prefill_ms, m->ev[0], m->ev[1]));
    m->last_launches += lp;
    return FORGE_OK;
}

int32_t forge_model_set_gemm_passes(ForgeModel* m, int32_t passes) {
    if (!m || (passes != 1 && passes != 3)) { set_error("gemm passes must be 1 or 3"); return FORGE_ERR_INVALID_ARG; }
    m->gemm_passes = passes;
    return FORGE_OK;
}

int32_t forge_model_set_prefill_mode(ForgeModel* m, int32_t mode) {
    if (!m || (mode != 0 && mode != 1)) { set_error("prefill mode must be 0 or 1"); return FORGE_ERR_INVALID_ARG; }
    if (mode == 1 && m->per_token_prefill) { set_error("this mix of storage formats has no batched prompt path"); return FORGE_ERR_UNSUPPORTED; }
    m->kquant_batched = mode == 1;
    return FORGE_OK;
}

int32_t forge_model_set_wait_limit(ForgeModel* m, uint32_t polls) {
    if (!m || polls == 0) { set_error("the wait limit must be at least one poll"); return FORGE_ERR_INVALID_ARG; }
    m->wait_limit = polls;
    return FORGE_OK;
}

int32_t forge_hidden_trace_enable(ForgeModel* m, int32_t enable) {
    if (!m) { set_error("null model"); return FORGE_ERR_INVALID_ARG; }
    m->trace_on = enable != 0;
    return FORGE_OK;
}

int32_t forge_hidden_trace_read(ForgeModel* m, float* out_host, size_t capacity_floats, int32_t* rows) {
    if (!m || !out_host || !rows) { set_error("bad argument to forge_hidden_trace_read"); return FORGE_ERR_INVALID_ARG; }
    size_t n = size_t(m->cfg.num_layers) * m->trace_rows * m->h;
    if (n == 0 || !m->trace) { set_error("no trace recorded"); return FORGE_ERR_INVALID_ARG; }
    if (capacity_floats < n) { set_error("trace needs %zu floats", n); return FORGE_ERR_INVALID_ARG; }
    FORGE_CUDA(cudaSetDevice(m->device));
    FORGE_CUDA(cudaMemcpyAsync(out_host, m->trace, n * 4, cudaMemcpyDeviceToHost, m->stream));
    FORGE_CUDA(cudaStreamSynchronize(m->stream));
    *rows = m->trace_rows;
    return FORGE_OK;
}

int32_t forge_last_timing(ForgeModel* m, float* prefill_ms, float* decode_ms, int64_t* launches) {
    if (!m) { set_error("null model"); return FORGE_ERR_INVALID_ARG; }
    if (prefill_ms) *prefill_ms = m->prefill_ms;
    if (decode_ms) *decode_ms = m->decode_ms;
    if (launches) *launches = m->last_launches;
    return FORGE_OK;
}

}  // extern "C"
