// Shared declarations of the sm_100a backend: status plumbing, packed-weight descriptors,
// the kernel launch prototypes each .cu file exports to the host-side model code.
#pragma once

#include <cuda_fp16.h>
#include <utility>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/forge_b200.h"

namespace forge {

// ------------------------------------------------------------------ errors
void set_error(const char* fmt, ...);
extern thread_local long long g_launches;  // kernels of this library launched on this thread

#define FORGE_CUDA(call)                                                                   \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess) {                                                           \
            forge::set_error("%s:%d %s: %s", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
            return FORGE_ERR_CUDA;                                                         \
        }                                                                                  \
    } while (0)

#define FORGE_LAUNCH_CHECK()                                                               \
    do {                                                                                   \
        ++forge::g_launches;                                                               \
        cudaError_t e_ = cudaGetLastError();                                               \
        if (e_ != cudaSuccess) {                                                           \
            forge::set_error("%s:%d kernel launch: %s", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            return FORGE_ERR_CUDA;                                                         \
        }                                                                                  \
    } while (0)

#define FORGE_TRY(expr)                     \
    do {                                    \
        int32_t s_ = (expr);                \
        if (s_ != FORGE_OK) return s_;      \
    } while (0)

// ------------------------------------------------------------------ packed weights
// Load-time layout of one projection: the 32 (Q8_0) or 16 (Q4_0) quant bytes of every block,
// verbatim and contiguous per row, and the f16 block scales in a second array.  Same bytes
// per weight as the GGUF stream (34/32 and 18/32), but every row starts 16-byte aligned.
// Row-major layout of the batched GEMM.  Q8_0 / Q4_0: quant bytes verbatim + f16 block scales.  K-quant rows
// (Q4_K and Q6_K alike, so rows of both may share one matrix) are expanded to FORGE_KQ_SOA: one int8 per weight
// (the nibble 0..15, or q6 - 32) and per 32-element block a float4 {s_lo, s_hi, mn, 0} with
// value = s_lo * q (k < 16) or s_hi * q (k >= 16), minus mn  (Q4_K: s_lo = s_hi = d*sc, mn = dmin*m; Q6_K: mn = 0).
constexpr int FORGE_KQ_SOA = 100;
struct QWeight {
    uint8_t* qs = nullptr;  // [N][K] int8  or  [N][K/2] nibble pairs
    __half* d = nullptr;    // [N][K/32]  (Q8_0 / Q4_0)
    float4* sf = nullptr;   // [N][K/32]  (FORGE_KQ_SOA)
    int K = 0, N = 0, quant = 0;
    size_t qs_row_bytes() const { return quant == FORGE_Q4_0 ? size_t(K) / 2 : size_t(K); }
};

// raw GGUF rows [row0, row0+rows) x blocks [blk0, blk0+blks) of a [N][K/32] block matrix ->
// packed rows dst_row0.. with optional row interleave: dst row = dst_row0 + r*row_step.
int32_t pack_rows(const uint8_t* raw_dev, int quant, int K_full, int row0, int rows, int blk0, int blks,
                  QWeight& dst, int dst_row0, int row_step, cudaStream_t st);

// ------------------------------------------------------------------ tensor-parallel sum (tp_comm.cu)
struct TpComm;
int32_t tp_unique_id(uint8_t* out);
int32_t tp_init(TpComm** out, const uint8_t* id_bytes, int rank, int world);
int32_t tp_allreduce_sum(TpComm* c, float* buf, size_t n, cudaStream_t st);  // in place, on st
// hidden[0..count) += sum over ranks of part, through {value, tag} pairs in the ranks' exchange buffers (peer memory);
// `region` and `cap` (pairs) place the [slot][rank][cap] area inside every rank's buffer
int32_t tp_pair_sum(float* hidden, const float* part, uint2* const* peer_ll, const uint2* local_ll, size_t region, size_t cap, int count,
                    int world, int rank, int slot, const uint32_t* step_counter, uint32_t step_mul, uint32_t step_add, uint32_t limit,
                    int* err, cudaStream_t st);
void tp_destroy(TpComm* c);

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with launch_pdl() may start while the kernel before it on the stream is still running.
// It must execute pdl_wait() before it touches anything an earlier kernel writes (the wait returns when the earlier
// kernels have completed and their writes are visible); what it does before the wait (barrier set-up, streaming
// constant weights into shared memory) overlaps the tail of its predecessor.  pdl_trigger() lets the next kernel
// on the stream be scheduled as soon as every CTA of this one has called it.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}
#endif

// ------------------------------------------------------------------ GEMV (decode)
// EPI_PARTIAL: every K slice stores its raw partial sums at scratch[slice][row]; the reader adds them
enum GemvEpilogue { EPI_STORE = 0, EPI_RESID = 1, EPI_QKV = 2, EPI_SILU = 3, EPI_PARTIAL = 4, EPI_TP_PUSH = 5 };

struct GemvArgs {
    const float* x = nullptr;       // [batch][K] input rows
    const float* norm_w = nullptr;  // if set: RMSNorm(x) * norm_w is applied before the product
    float eps = 0.f;
    float* out = nullptr;           // EPI_STORE / EPI_RESID / EPI_SILU target, [batch][N or N/2]
    const float* resid = nullptr;   // EPI_RESID: out = resid + W x (may alias out)
    int batch = 1;
    // EPI_QKV
    const float* bias = nullptr;    // [N] or null
    const float* rope = nullptr;    // [pos][hd/2]{cos,sin}
    float* q_out = nullptr;         // [batch][qk]
    __half* k_pool = nullptr;       // this layer's page pool
    __half* v_pool = nullptr;
    const int32_t* page_table = nullptr;  // [batch][pages_per_seq]
    const int32_t* seq_len = nullptr;     // [batch] device positions (the new row's position)
    int pages_per_seq = 0;
    int qk = 0, kv = 0, head_dim = 0;
    int kv_stride = 0;              // values per cache row (= kv of the layer; a V-only matrix passes qk = kv = 0)
    // optional: constant data the NEXT kernel on the stream will read (its weights).  Every CTA asks L2 to fetch its
    // share while this kernel runs, so HBM keeps streaming across the kernel boundary.
    const void* next_w = nullptr;
    size_t next_bytes = 0;
    // Tensor-parallel sum over peer memory (decode, batch 1).  Every rank owns an exchange buffer
    // ll[2 slots][world][h] of {value, step} pairs that its peers map (CUDA IPC).
    //  * EPI_TP_PUSH (the row-sliced projection): each finished row of this rank's partial product is stored as one
    //    8-byte {value, step} pair into ll[slot][tp.rank] of EVERY rank's buffer (NVLink stores).  The pair is written
    //    atomically, so the value needs no fence and no completion flag: a reader sees it as soon as the step matches.
    //  * tp.consume (the kernel that reads the result next): stages x = x + sum over ranks of ll[slot][r] in rank
    //    order (every rank forms the same bits), spinning - bounded - on pairs whose step is not the current one yet,
    //    and writes the sum once to x_writeback (the residual stream for the kernels after it).
    // step = *step_counter * step_mul + step_add: the device-side decode step counter makes it unique across graph
    // replays; step_add (>= 1) numbers the sums inside a step.  Two slots alternate: a rank can be at most one sum
    // ahead of its slowest peer.
    struct Tp {
        int world = 0, rank = 0, consume = 0, slot = 0;
        uint2* const* peer_ll = nullptr;        // device array [world]: exchange buffer of every rank (own entry = local)
        const uint2* ll = nullptr;              // local exchange buffer
        const uint32_t* step_counter = nullptr; // device, advanced once per decode step
        uint32_t step_mul = 0, step_add = 0;
        uint32_t wait_limit = 1u << 20;         // polls per pair before the wait gives up
        float* x_writeback = nullptr;
    } tp;
};
// Streaming layout of one projection for the decode GEMV: 16-row x 32-column tiles, each
// {8 x half2 block scales}{quant bytes in MMA-fragment order}, K-major inside a 16-row band.
struct QTiled {
    uint8_t* data = nullptr;
    int K = 0, N = 0, quant = 0, bands = 0, bt = 1;  // bt row tiles per band; bands = ceil(N/(16*bt)); padding rows are zero
};
// Scratch for the split-K form of the GEMV (used when a matrix has fewer 128-row bands than SMs):
// partial sums [max_slices][bands*128] and one self-resetting ticket per 16-row tile.
struct GemvSplit {
    float* scratch = nullptr;
    int* tickets = nullptr;
    int max_slices = 0;
};
int gemv_slices(const QTiled& w, const GemvSplit& sp, int sms, int batch);
constexpr int kGemvMaxSlices = 16;
constexpr int kGemvSplitRows = 256 * 128;  // split only happens up to this many (padded) rows
size_t qtiled_bytes(int quant, int K, int N, int bt);
inline size_t qtiled_bytes(const QTiled& w) { return qtiled_bytes(w.quant, w.K, w.N, w.bt); }
int gemv_band_tiles(int N, int sms);
// row_src_dev[r] (device array of bands*16*bt device pointers): first raw GGUF block of the K
// slice of destination row r, or null for a padding row
int32_t tile_pack(const uint8_t* const* row_src_dev, QTiled& dst, cudaStream_t st);
// err: device int set to 1 if a bounded wait inside the kernel gave up (may be null)
int32_t gemv_tc(const QTiled& w, GemvEpilogue epi, const GemvArgs& a, const GemvSplit& sp, int* err, cudaStream_t st);

// ------------------------------------------------------------------ batched decode products (gemv_batch.cu)
// out[b][N] (+ resid) = x[b][K] . W^T for nb <= 16 rows per launch, the tiled weights streamed once.  The activations
// are packed first (gemv_batch_pack) into fp16 hi/lo B fragments; mode: 0 plain rows, 1 RMSNorm(x) * norm_w,
// 2 SiLU(gate) * up of interleaved [2 * K] rows.
int gemv_batch_ncg(int nb);
size_t gemv_batch_act_words(int K, int nb);          // uint2 entries the packed activations take
size_t gemv_batch_scratch_floats(int N, int K, int quant, int sms);   // split-K scratch a matrix needs (0: not split)
size_t gemv_batch_tickets(int N);
int gemv_batch_slices(int groups, int chunks, int sms);
// Tensor-parallel sum of a batched product over peer memory, fused into its two neighbours: the product's epilogue stores
// every finished value as a {value, tag} pair into every rank's exchange buffer (push), and the packing kernel of the
// next product forms hidden + sum over ranks while it reads its rows (consume), polling - bounded - for pairs whose tag is
// not the expected one yet.  Element (row b, column j) of rank r's part lies at base + r * cap + b * N + j.
struct BatchTp {
    uint2* const* peer_ll = nullptr;         // device array [world]: every rank's exchange buffer (push)
    const uint2* local_ll = nullptr;         // this rank's exchange buffer (consume)
    size_t base = 0, cap = 0;                // pairs
    int world = 0, rank = 0;
    const uint32_t* step_counter = nullptr;  // device, advanced once per decode step
    uint32_t step_mul = 0, step_add = 0;     // tag = *step_counter * step_mul + step_add
    uint32_t wait_limit = 1u << 20;
    int* err = nullptr;
};
// consume != null (mode 1 only): the rows are x + the ranks' pairs, and that sum is written back to x first
int32_t gemv_batch_pack(uint2* dst, float* x, size_t x_stride, int nb, int K, int quant, int mode, const float* norm_w, float eps, cudaStream_t st,
                        const BatchTp* consume = nullptr);
// push != null: the product goes to the ranks' exchange buffers instead of `out`
int32_t gemv_batch(const QTiled& w, const uint2* act, int nb, float* out, const float* resid, const GemvSplit& sp, int* err, cudaStream_t st,
                   const BatchTp* push = nullptr);

// ------------------------------------------------------------------ elementwise
int32_t rms_norm_f32(float* out, const float* in, const float* w, int rows, int n, float eps, cudaStream_t st);
// fp16 outputs come as a hi/lo pair when `lo` is given: hi = fp16(x), lo = fp16(x - hi)
int32_t rms_norm_f16(__half* out, __half* lo, const float* in, const float* w, int rows, int n, float eps, cudaStream_t st);
// hidden[r] += parts[0][r] + parts[1][r] + ... (fixed order; part s at parts + s * pstride), then, if w is given,
// out / lo = RMSNorm(hidden[r]) * w as an fp16 hi/lo pair: the residual add and the next operator's normalisation in one pass
int32_t add_parts_rms_norm_f16(float* hidden, const float* parts, int nparts, size_t pstride, __half* out, __half* lo, const float* w,
                               int rows, int n, float eps, cudaStream_t st);
int32_t rope_rows(float* data, int rows, int base_pos, int head_dim, int heads, const float* table, cudaStream_t st);
int32_t silu_mul_f32(float* out, const float* g, const float* u, size_t n, cudaStream_t st);
int32_t silu_mul_f16(__half* out, __half* lo, const float* gu, int rows, int ffn, cudaStream_t st);  // gu = interleaved [rows][2*ffn]
int32_t residual_add_f32(float* a, const float* b, size_t n, cudaStream_t st);
// hist/step (optional): also records tokens[r] at hist[*step * rows + r] (greedy loop bookkeeping)
int32_t embedding_rows(float* out, const float* table, const uint32_t* tokens, int rows, int h, uint32_t* hist, const int32_t* step, cudaStream_t st);
int32_t kv_append_contig(__half* kc, __half* vc, const float* k, const float* v, int rows, int base_pos, int kvd, cudaStream_t st);
// prefill QKV epilogue: bias, RoPE, q -> fp16 [m][qk], k/v -> paged fp16 cache
// nparts > 1: the product arrives as K-slice partials (pstride floats apart), added in slice order
int32_t qkv_post(const float* qkv, int m, int base_pos, const float* bias, const float* rope, __half* q16, __half* q16_lo,
                 __half* k_pool, __half* v_pool, const int32_t* page_row, int qk, int kv, int hd, cudaStream_t st, int nparts = 1, size_t pstride = 0);
// batched decode QKV epilogue: row b is sequence b at position seq_len[b]; q stays f32, k/v go to the sequence's page
int32_t qkv_post_rows(const float* qkv, int batch, const float* bias, const float* rope, float* q_out, __half* k_pool, __half* v_pool,
                      const int32_t* page_table, const int32_t* seq_len, int pages_per_seq, int qk, int kv, int hd, cudaStream_t st, int nparts = 1,
                      size_t pstride = 0);  // nparts > 1: the product arrives as K-slice partials, pstride floats apart
int32_t argmax_last(uint32_t* result, const float* logits, int n, int batch, cudaStream_t st);
// many-CTA form; sval/sidx: [batch][kArgmaxSlices] scratch, ticket: [batch] zero-initialised counters
constexpr int kArgmaxSlices = 148;
int32_t argmax_slices(uint32_t* result, const float* logits, int n, int batch, float* sval, int* sidx, int* ticket, cudaStream_t st);
int32_t f32_to_f16(__half* out, __half* lo, const float* in, size_t n, cudaStream_t st);
// In place: the rows (hi + lo) become their Q8_0 form q * f16(scale) per 32 values (emit.rs:1412-1440), the input of
// every K-quant product, again split into hi + lo (exact: an 8-bit integer times an f16).
int32_t q8_round_f16(__half* hi, __half* lo, size_t n, cudaStream_t st);
int32_t step_advance(int32_t* seq_len, int batch, int32_t* step, cudaStream_t st, uint32_t* extra_counter = nullptr);
int32_t token_nll(double* out, const float* logits, int n, uint32_t target, cudaStream_t st);  // -log softmax(logits)[target], f64
int32_t gather_rows_f16(float* out, const __half* pool, const int32_t* page_row, int len, int kvd, cudaStream_t st);

// ------------------------------------------------------------------ attention
struct AttnDecodeArgs {
    float* out; const float* q;              // [batch][nq*hd]
    const __half* k_pool; const __half* v_pool;
    const int32_t* page_table; int pages_per_seq;  // null table = contiguous cache
    const int32_t* seq_len;                  // device [batch]: attends to positions <= seq_len[b]
    int seq_len_host;                        // used when seq_len == nullptr (op-level call): count of positions
    int batch, nq, nkv, hd, max_ctx;
    float* ws; int* counters;                // split workspace
    int splits;
    int window = 0;                          // > 0: only the last `window` positions are attended to
    // tensor maps (CUtensorMap, host memory) of the K and V pools as {head_dim, kv heads, rows}: a paged cache passes its
    // own (made once, see make_kv_map) with row_base = first row of the layer; a contiguous cache may leave them null
    const void* map_k = nullptr; const void* map_v = nullptr;
    int row_base = 0;
    int* err = nullptr;                      // set when a bounded wait gave up
    // out16 != null: the result is stored as fp16 hi (+ lo) rows [batch][nq*hd] (the operand of a tensor-core product)
    // instead of f32 `out`
    __half* out16 = nullptr; __half* out16_lo = nullptr;
};
// context splits for `groups` = batch * kv_heads independent (sequence, KV head) pairs over `pages` pages
int attn_decode_splits(int pages, int groups, int sms, int hd, int heads_per_group);
size_t attn_decode_ws_floats(int batch, int nq, int hd, int splits);
// Tiled tensor map over an fp16 K or V pool of `rows` rows of kv_heads * head_dim values: dimensions {head_dim, kv_heads,
// rows}, box {head_dim, 1, 64} = one page of one KV head (`out`: a CUtensorMap in host memory)
int32_t make_kv_map(void* out, const __half* pool, int head_dim, int kv_heads, size_t rows);
int32_t attn_decode(const AttnDecodeArgs& a, cudaStream_t st);

struct AttnPrefillArgs {
    __half* out16; __half* out16_lo; float* out32;  // out16 (+ optional lo part) or out32: [m][nq*hd]
    const __half* q16;                       // [m][nq*hd]
    const __half* k_pool; const __half* v_pool;
    const int32_t* page_row;                 // device [pages] physical page of logical page i (null = contiguous)
    int m, base_pos, nq, nkv, hd;
    int window = 0;                          // > 0: query position p sees keys [max(0, p - window + 1), p]
    // precise: queries and probabilities enter the tensor cores as fp16 hi + lo pairs (two MMAs each), which takes the
    // output from ~1e-4 to ~1e-6 of the f32 result; used where the output feeds an 8-bit rounding (K-quant models)
    const __half* q16_lo = nullptr;          // [m][nq*hd] low parts of q16 (precise mode)
    int precise = 0;
    size_t pool_rows = 0;                    // rows of k_pool / v_pool (positions); rows beyond them read as zero
    int* err = nullptr;                      // set when a bounded wait gave up
};
int32_t attn_prefill(const AttnPrefillArgs& a, cudaStream_t st);

// ------------------------------------------------------------------ GEMM (prefill)
// out f32 [m][N] = A f16 [m][K] x W^T; optional resid: out = resid + A W^T (may alias out)
// Alo != null selects the split-precision form (A = A + Alo, weights split the same way)
// err: device word set when a bounded wait in the tcgen05 kernel gives up (may be null)
int32_t gemm_f16a(float* out, const __half* A, const __half* Alo, const QWeight& w, int m, const float* resid, int* err, cudaStream_t st);
int32_t gemm_f16a_mma(float* out, const __half* A, const __half* Alo, const QWeight& w, int m, const float* resid, cudaStream_t st);
bool gemm_tc5_supported(const QWeight& w);
// ksplit > 1: K slice z leaves its partial product (no residual) at out + z * part_stride; the caller adds the slices
// act_hi != null (gate/up product, rows 2j = gate_j, 2j + 1 = up_j, one K slice): the epilogue stores SiLU(gate) * up as
// fp16 hi (+ lo) rows [m][N / 2] and `out` is not written
int32_t gemm_tc5(float* out, const __half* A, const __half* Alo, const QWeight& w, int m, const float* resid, int* err, cudaStream_t st,
                 int ksplit = 1, size_t part_stride = 0, __half* act_hi = nullptr, __half* act_lo = nullptr);
int gemm_tc5_ksplit(const QWeight& w);

}  // namespace forge
