/* forge_b200.h — C ABI of the B200 (sm_100a) backend for ForgeLLM's quantized forward path.
 *
 * The reference has no FFI: its boundary is the function surface of the Rust module that
 * its CPU code generator emits (`model::forward`, `model::forward_prefill`, the shape-
 * specialised `matmul_vec_*` / `matmul_mat_*`, `attention_flash*`, `rms_norm`, `rope`,
 * `silu_mul`, `residual_add`) plus the `weights.bin` file format.  Each entry point below
 * names the generated function it replaces (file:line in the reference tree, where
 * E = crates/forgellm-codegen-cpu/src/emit.rs, P = crates/forgellm-codegen-cpu/src/project.rs,
 * WL = crates/forgellm-frontend/src/weight_loader.rs, CLI = crates/forgellm-cli/src/main.rs).
 *
 * Conventions
 *  - Every function returns a ForgeStatus (0 = ok); nothing aborts the process.
 *  - "device pointer" arguments are CUDA global-memory addresses on the current device;
 *    "host pointer" arguments are ordinary process memory.  No torch types appear here.
 *  - `stream` is a `cudaStream_t` passed as `void*` (NULL = the default stream).
 *  - Shapes are run-time arguments (the reference bakes them into function names).
 *  - Calls that touch one ForgeKV must be serialised by the caller (the reference enforces
 *    the same with `&mut KVCache`).
 *  - There is no CPU fallback: without a CUDA device every compute entry point returns
 *    FORGE_ERR_CUDA.
 */
#ifndef FORGE_B200_H
#define FORGE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ForgeStatus {
    FORGE_OK = 0,
    FORGE_ERR_INVALID_ARG = 1, /* null pointer, negative size, unknown enum value */
    FORGE_ERR_SHAPE = 2,       /* K not a multiple of 32, unsupported head_dim, blob length mismatch */
    FORGE_ERR_KV_FULL = 3,     /* position would pass max_seq (the reference panics on the slice bound) */
    FORGE_ERR_CUDA = 4,        /* a CUDA runtime call failed; forge_last_error() has the text */
    FORGE_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up */
    FORGE_ERR_UNSUPPORTED = 6,
    FORGE_ERR_COMM = 7         /* tensor-parallel collective failed */
} ForgeStatus;

#define FORGE_Q8_0 8 /* GGUF Q8_0: 34-byte blocks {f16 d; int8 q[32]}        (E:1266-1268, WL:860-888) */
#define FORGE_Q4_0 4 /* GGUF Q4_0: 18-byte blocks {f16 d; u8 qs[16]}, value = nibble-8,
                        byte j = element j (low) and j+16 (high)          (E:2337-2359, WL:893-926) */
/* K-quants (256-element super-blocks; the numbers are the GGML type ids).  Operator level only:
 * per-token products only, as in the generated module (no batched K-quant product exists there). */
#define FORGE_Q4_K 12 /* 144 bytes {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]},
                         value = d*sc[j]*q - dmin*m[j] per 32-element sub-block j   (E:2962-2969, WL:1146-1200) */
#define FORGE_Q6_K 14 /* 210 bytes {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d},
                         value = d*scales[i/16]*(q6-32)                             (E:3542-3546, WL:997-1060) */

#define FORGE_PREFILL_BATCH_THRESHOLD 8 /* E:203-206 */
#define FORGE_KV_PAGE 64                /* positions per KV page (= FLASH_ATTN_BLOCK_SIZE, E:199-202) */

/* Mirrors the reference's ModelConfig (crates/forgellm-frontend/src/ir.rs:484-519), reduced
 * to the fields the emitted constants use (E:151-206). */
typedef struct ForgeModelConfig {
    int32_t hidden_size;
    int32_t intermediate_size;
    int32_t num_layers;
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t head_dim; /* 64, 96 or 128 */
    int32_t vocab_size;
    int32_t max_seq_len; /* capped at 4096 like MAX_SEQ_LEN (E:178) */
    float rms_norm_eps;
    float rope_theta;
    int32_t quant;    /* FORGE_Q8_0, FORGE_Q4_0, FORGE_Q4_K or FORGE_Q6_K: every projection and lm_head, unless proj_quant says otherwise */
    int32_t qkv_bias; /* 1: f32 q,k,v biases follow v_proj in weights.bin (Qwen2, E:4108-4118) */
    int32_t tp_rank;  /* tensor-parallel rank / world size; 0 / 1 when not sharded */
    int32_t tp_world;
    int32_t sliding_window; /* > 0: position p attends to [max(0, p - window + 1), p] (Mistral, E:601-626,
                               E:916-1046); 0: full causal attention */
    int32_t proj_quant[8];  /* storage format per projection category, in the order q, k, v, o, gate, up, down, lm_head
                               (ProjectionDTypes, crates/forgellm-frontend/src/ir.rs:411-421, without the f32 embedding);
                               0 = `quant`.  q/k and gate/up must agree.  A model with a K-quant category runs its prompt
                               token by token like the generated forward_prefill (E:4511-5050) and takes one GPU. */
} ForgeModelConfig;

typedef struct ForgeModel ForgeModel;
typedef struct ForgeKV ForgeKV;

/* Text of the last error on the calling thread ("" if none). */
const char* forge_last_error(void);
/* Number of CUDA devices visible; 0 when there is no driver or no device. */
int32_t forge_device_count(void);

/* ------------------------------------------------------------------------------------
 * Operator surface (device pointers).  Weights are raw GGUF block bytes, row-major
 * [N][K/32][block], exactly what the generated functions take.
 * ------------------------------------------------------------------------------------ */

/* matmul_vec_q8_0_{K}x{N}(output, input, weight)              E:2047-2087 (dot_q8_0 E:1359-1377)
 * matmul_mat_q8_0_{K}x{N}(output, m, input, weight)           E:2278-2299
 *   out f32 [m][N], in f32 [m][K], w u8 [N][K/32][34].  m == 1 is the decode GEMV. */
int32_t forge_matmul_mat_q8_0(float* out, int32_t m, const float* in, const uint8_t* w,
                              int32_t K, int32_t N, void* stream);
/* matmul_vec_q4_0_{K}x{N} E:2910-2953 (dot_q4_0 E:2337-2359); matmul_mat_q4_0_{K}x{N} E:3792-3813 */
int32_t forge_matmul_mat_q4_0(float* out, int32_t m, const float* in, const uint8_t* w,
                              int32_t K, int32_t N, void* stream);

/* matmul_vec_q4_k_{K}x{N}(output, input, weight)  E:3411-3487 (dot_q4_k_q8_0 E:3246-3303)
 * matmul_vec_q6_k_{K}x{N}(output, input, weight)  E:3636-3652 (dot_q6_k_q8_0 E:3553-3611)
 *   applied to each of the m rows of `in` (the generated module has no batched K-quant product).  As there, every
 *   input row is first quantised to Q8_0 blocks (E:1412-1440); below 8 rows the block dots are exact integers, from
 *   8 rows on the rows share one tensor-core GEMM (weights dequantised to split fp16, ~1e-5 relative).
 *   out f32 [m][N], in f32 [m][K], w u8 [N][K/256][144 or 210]; K must be a multiple of 256. */
int32_t forge_matmul_vec_q4_k(float* out, int32_t m, const float* in, const uint8_t* w,
                              int32_t K, int32_t N, void* stream);
int32_t forge_matmul_vec_q6_k(float* out, int32_t m, const float* in, const uint8_t* w,
                              int32_t K, int32_t N, void* stream);

/* The same products on a weight repacked once: forge_packed_create converts raw GGUF blocks
 * (device pointer, [N][K/32][block]) into the kernels' aligned layouts (same bytes per weight),
 * forge_matmul_mat_packed then runs without any per-call repacking or allocation for m < 8
 * (the `Weights` struct of the generated module, E:3875-3939, plays this role there). */
typedef struct ForgePacked ForgePacked;
int32_t forge_packed_create(int32_t quant, const uint8_t* w, int32_t K, int32_t N, void* stream, ForgePacked** out);
void forge_packed_destroy(ForgePacked* w);
int32_t forge_matmul_mat_packed(float* out, int32_t m, const float* in, const ForgePacked* w, void* stream);
/* The product of a decode step for nb <= 16 sequences at once (the reference has no batched decode: it calls
 * matmul_vec_* once per sequence, E:2047-2087 / E:2910-2953, and this returns those calls' values): out f32 [nb][N],
 * in f32 [nb][K], the weights streamed once for all rows.  Q8_0 / Q4_0.  The first call on a packed matrix allocates
 * the product's buffers; it only enqueues work (see forge_packed_check). */
int32_t forge_matmul_decode_batch(float* out, int32_t nb, const float* in, ForgePacked* w, void* stream);
/* forge_matmul_mat_packed only enqueues work.  This call synchronises `stream` and reports whether a bounded
 * device-side wait of any product on `w` since the last check gave up (FORGE_ERR_TIMEOUT; the word is cleared). */
int32_t forge_packed_check(const ForgePacked* w, void* stream);

/* rms_norm(output, input, weight, eps)  E:327-334, applied to `rows` rows of n values. */
int32_t forge_rms_norm(float* out, const float* in, const float* weight, int32_t rows, int32_t n,
                       float eps, void* stream);
/* rope_freqs + the per-position sin/cos table of rope()  E:502-519.  Host function: fills
 * table[pos][i] = {cos, sin}(pos * 1/theta^(2i/head_dim)) for pos < n_pos, i < head_dim/2,
 * with the host libm in f32 (the arithmetic the reference's CPU path performs). */
int32_t forge_rope_table(float* table_host, int32_t n_pos, int32_t head_dim, float theta);
/* rope(data, pos, head_dim, num_heads, freqs)  E:509-528, for `rows` rows; row r uses
 * position base_pos + r.  `table` is a device copy of forge_rope_table's output. */
int32_t forge_rope(float* data, int32_t rows, int32_t base_pos, int32_t head_dim, int32_t num_heads,
                   const float* table, void* stream);
/* silu_mul(output, gate, up)  E:381-386 */
int32_t forge_silu_mul(float* out, const float* gate, const float* up, size_t n, void* stream);
/* residual_add(a, b)  E:455-459 */
int32_t forge_residual_add(float* a, const float* b, size_t n, void* stream);

/* Cache write that replaces quantize_kv + copy_from_slice (E:533-545, E:4136-4153): rounds
 * `rows` K and V rows (f32 [rows][num_kv_heads*head_dim]) to fp16 and stores them at
 * positions base_pos.. of a contiguous fp16 cache [pos][kv_head][d]. */
int32_t forge_kv_append_f16(uint16_t* k_cache, uint16_t* v_cache, const float* k, const float* v,
                            int32_t rows, int32_t base_pos, int32_t kv_dim, void* stream);
/* attention_flash(output, q, k_cache, v_cache, .., seq_len, num_heads, num_kv_heads, head_dim)
 * E:657-715, over a contiguous fp16 cache [pos][kv_head][d] (the reference CPU cache is int8
 * with per-token scales; fp16 is the cache type of this backend). out, q: f32 [nh*hd]. */
int32_t forge_attention_flash(float* out, const float* q, const uint16_t* k_cache,
                              const uint16_t* v_cache, int32_t seq_len, int32_t num_heads,
                              int32_t num_kv_heads, int32_t head_dim, void* stream);
/* No counterpart in the reference.  The same operation as forge_attention_flash for callers that cannot
 * let the library allocate device memory (a host whose own pool owns the whole GPU, or a loop that cannot
 * afford the synchronisation an allocation may imply): the split-KV workspace is a fixed array inside the
 * library image, about 1.1 MB on every GPU that loads the library, held until the process exits.
 * Limits: num_heads <= 64, num_kv_heads <= 64, head_dim <= 128 (64, 96 or 128), seq_len <= 1048576;
 * anything larger returns FORGE_ERR_SHAPE.  The first call on each device looks up the array's address
 * (that device must be current); make that first call before any stream capture begins.  All calls on a
 * device share the one array: two calls that overlap on the GPU (different streams) race on it, so issue
 * them on one stream or order them yourself.  It performs no cudaMalloc / cudaFree and uses no allocating
 * library routine. */
int32_t forge_attention_flash_static(float* out, const float* q, const uint16_t* k_cache,
                                     const uint16_t* v_cache, int32_t seq_len, int32_t num_heads,
                                     int32_t num_kv_heads, int32_t head_dim, void* stream);
/* attention_flash_batch(output, q_batch, k_cache, v_cache, .., m, base_pos, ...)  E:755-883.
 * Query row r sits at position base_pos + r and sees cache positions <= its own.  The caches hold base_pos + m rows
 * (rows past that are never read).  The call converts the queries to fp16 hi + lo pairs in a temporary buffer of the
 * stream-ordered allocator, runs the tensor-core kernel and synchronises the stream to read the kernel's status
 * (FORGE_ERR_TIMEOUT if a bounded device-side wait gave up); the sliding-window twin below does the same. */
int32_t forge_attention_flash_batch(float* out, const float* q_batch, const uint16_t* k_cache,
                                    const uint16_t* v_cache, int32_t m, int32_t base_pos,
                                    int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                    void* stream);
/* argmax of the generated main (P:501-503): on ties the LAST maximal index wins.
 * logits: device f32 [n]; result: device u32. */
int32_t forge_argmax(uint32_t* result, const float* logits, int32_t n, void* stream);

/* attention_sliding (E:601-626) and attention_sliding_batch (E:916-1046): the two calls above restricted to the last
 * `window` positions: the query at position p sees the cache positions [max(0, p - window + 1), p]. */
int32_t forge_attention_sliding(float* out, const float* q, const uint16_t* k_cache, const uint16_t* v_cache, int32_t seq_len,
                                int32_t window, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, void* stream);
int32_t forge_attention_sliding_batch(float* out, const float* q_batch, const uint16_t* k_cache, const uint16_t* v_cache, int32_t m,
                                      int32_t base_pos, int32_t window, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                      void* stream);

/* Host-side quantisers of the reference's exporter (quantize_f32_to_q8_0 WL:1454-1486;
 * Q4_0 packing WL:1494-1544 with `signed_max` = 0, or the signed-max scale rule
 * d = largest-magnitude value / -8 with `signed_max` = 1).  n must be a multiple of 32. */
int32_t forge_quantize_q8_0_host(const float* x, size_t n, uint8_t* out);
int32_t forge_quantize_q4_0_host(const float* x, size_t n, uint8_t* out, int32_t signed_max);
/* quantize_f32_to_q4_k (WL:1773-1900) / quantize_f32_to_q6_k (WL:2025-2125): n a multiple of 256; out receives
 * n/256 super-blocks of 144 / 210 bytes.  The exporter uses them where a tensor is not stored in its category's
 * format (load_from_file_mixed_per_tensor, WL:193-218). */
int32_t forge_quantize_q4_k_host(const float* x, size_t n, uint8_t* out);
int32_t forge_quantize_q6_k_host(const float* x, size_t n, uint8_t* out);

/* ------------------------------------------------------------------------------------
 * Session surface: Weights / KVCache / forward / forward_prefill of the generated module.
 * ------------------------------------------------------------------------------------ */

/* Byte length of weights.bin for a configuration (layout: CLI:2714-2757, P:341-407). */
size_t forge_weights_bin_size(const ForgeModelConfig* cfg);

/* Weights (E:3875-3939) from a host image of weights.bin; uploads to `device` and repacks
 * the blocks into the kernels' aligned layout (same bytes per weight).  With tp_world > 1
 * the rank keeps its column slice of q/k/v/gate/up and its row slice of o/down. */
int32_t forge_model_create(const ForgeModelConfig* cfg, const void* weights_bin, size_t len,
                           int32_t device, ForgeModel** out);
/* Also releases the device memory of caches of this model that are still alive; their handles stay valid for
 * forge_kv_destroy only (every other call on them reports an error), so the two can be destroyed in either order. */
void forge_model_destroy(ForgeModel* model);
/* The CUDA stream (cudaStream_t) all work of this model is launched on. */
void* forge_model_stream(ForgeModel* model);

/* Tensor parallelism (one process per GPU, cfg.tp_world ranks).  The attention-output and FFN-down projections are
 * row-sliced, so their results are summed over the ranks (an NCCL all-reduce on the model's stream) before the
 * residual is added; every rank ends with the same hidden state and computes the full logits.
 *   forge_tp_unique_id: rank 0 creates the rendezvous id (FORGE_TP_ID_BYTES bytes) and hands it to the other
 *     ranks by any host channel (a process-group broadcast, MPI, a file);
 *   forge_model_tp_init: every rank, after forge_model_create with the same tp_world; collective.
 * A model created with tp_world > 1 returns FORGE_ERR_INVALID_ARG from the forward calls until it has a communicator.
 * NCCL (libnccl.so.2) is bound at run time; without it these two calls return FORGE_ERR_UNSUPPORTED. */
#define FORGE_TP_ID_BYTES 128
int32_t forge_tp_unique_id(uint8_t* id_out);
int32_t forge_model_tp_init(ForgeModel* model, const uint8_t* id);

/* Optional, after forge_model_tp_init: sum the decode step's partial products over peer memory instead of calling the
 * collective library.  Each rank exports a handle (CUDA IPC) to a small exchange buffer it owns; after every rank has
 * all `tp_world` handles (rank order, FORGE_TP_HANDLE_BYTES each, gathered over any host channel) it attaches them.
 * From then on the batch-1 decode step pushes each row-sliced projection's partial rows straight into the peers'
 * buffers from the GEMV epilogue (NVLink stores) and the next kernel adds the ranks' parts while it stages its input;
 * a batched decode step of up to 8 sequences does the same through the batched product's epilogue and the next
 * packing kernel; prompts and larger batches keep the library all-reduce.  Needs peer access between the GPUs (one process per GPU, all GPUs visible to every process). */
#define FORGE_TP_HANDLE_BYTES 64
int32_t forge_model_tp_exchange_export(ForgeModel* model, uint8_t* handle_out);
int32_t forge_model_tp_exchange_attach(ForgeModel* model, const uint8_t* handles);

/* Numeric form of the prefill GEMMs (matmul_mat_*, E:2278-2299).  3 (default): both operands
 * are carried as fp16 hi+lo pairs and three tensor-core passes are accumulated in f32 (~1e-6
 * relative to the reference's all-f32 arithmetic); 1: one fp16 pass (~3e-4 relative per GEMM,
 * which exceeds 1e-3 on the hidden state after ~20 layers). */
int32_t forge_model_set_gemm_passes(ForgeModel* model, int32_t passes);
/* Prompt path of a model with K-quant projections.  0 (default): token by token through the per-token products, the
 * structure of the generated forward_prefill (E:4511-5050), which has no batched K-quant product.  1: the batched
 * GEMMs, every K-quant product still taking its input rows as Q8_0 blocks, and the attention in its precise form
 * (queries and probabilities as fp16 hi + lo pairs); ~75x faster on a 1500-token prompt.  The GEMMs carry their
 * operands as 22-bit fp16 pairs, so their outputs differ from the per-token integer dots by ~1e-6, which moves a
 * value across an 8-bit rounding boundary in about one row of five on the tiny test models (per-layer deviation
 * 1e-3 .. 4e-3 there, against < 1e-3 for mode 0).  No effect on Q8_0 / Q4_0 models (always batched). */
int32_t forge_model_set_prefill_mode(ForgeModel* model, int32_t mode);

/* Polls a device-side wait for a tensor-parallel peer's contribution makes before it gives up (the reference has no
 * counterpart: its CPU threads join).  Every wait inside the kernels - a pipeline stage, a peer's partial sums - is
 * bounded; when one runs out the kernel finishes by itself, and the session call that launched it returns
 * FORGE_ERR_TIMEOUT at its synchronisation point, with the cache positions as they were before the call.
 * The default (2^20 polls, about a second) suits production; tests set it small. */
int32_t forge_model_set_wait_limit(ForgeModel* model, uint32_t polls);


/* KVCache::new (E:3978-4000) for `batch` independent sequences of up to max_seq positions,
 * fp16, paged (FORGE_KV_PAGE positions per page, pages handed out on demand). */
int32_t forge_kv_create(ForgeModel* model, int32_t max_seq, int32_t batch, ForgeKV** out);
/* KVCache::reset (E:4002-4005): all sequences back to length 0, pages returned. */
int32_t forge_kv_reset(ForgeKV* kv);
/* cache.len of sequence `seq`; -1 on a bad argument. */
int32_t forge_kv_len(const ForgeKV* kv, int32_t seq);
void forge_kv_destroy(ForgeKV* kv);
/* Copy K (which = 0) or V (1) rows [0, len) of `layer`, sequence `seq`, widened to f32, into
 * a host buffer [len][num_kv_heads*head_dim] (used by parity tests). */
int32_t forge_kv_read(ForgeKV* kv, int32_t seq, int32_t layer, int32_t which, float* out_host);

/* KV cache persistence (save_kv_cache / load_kv_cache of the generated main.rs, project.rs:456-499).
 * forge_kv_save writes sequence `seq` as {"FKV1", u32 layers, u32 kv_width, u64 len} followed by the K rows of every
 * layer and then the V rows of every layer, fp16 [layer][len][kv_width]; forge_kv_save_size is the byte count.
 * forge_kv_load replaces sequence `seq` with the saved state.  It also accepts the reference's own file - u64 len,
 * int8 K [layer][len*kv_width], int8 V, f32 k_scales [layer][len], f32 v_scales - and converts it: every value
 * becomes fp16(int8 * scale).  A file of another model (layer count, width) or past max_seq is refused. */
size_t forge_kv_save_size(const ForgeKV* kv, int32_t seq);
int32_t forge_kv_save(ForgeKV* kv, int32_t seq, void* out_host, size_t capacity);
int32_t forge_kv_load(ForgeKV* kv, int32_t seq, const void* data_host, size_t len);

/* forward(token_id, &weights, &mut cache) -> Vec<f32>  E:4029-4500, sequence 0.
 * logits_host: V floats (may be NULL to skip the copy). */
int32_t forge_forward(ForgeModel* model, ForgeKV* kv, uint32_t token, float* logits_host);
/* forward_prefill(tokens, &weights, &mut cache) -> Vec<f32>  E:4553-4587 / E:5118-5486,
 * sequence 0; returns the logits of the last prompt row only (E:5439-5443). */
int32_t forge_forward_prefill(ForgeModel* model, ForgeKV* kv, const uint32_t* tokens, size_t m,
                              float* logits_host);
/* The same two calls for sequence `seq` of a multi-sequence cache. */
int32_t forge_forward_seq(ForgeModel* model, ForgeKV* kv, int32_t seq, uint32_t token, float* logits_host);
int32_t forge_forward_prefill_seq(ForgeModel* model, ForgeKV* kv, int32_t seq, const uint32_t* tokens,
                                  size_t m, float* logits_host);
/* One decode step for the first `batch` sequences of the cache at once (the reference has no
 * batched decode: this equals `batch` independent forward() calls).  tokens: host u32 [batch];
 * logits_host: [batch][V] or NULL. */
int32_t forge_forward_batch(ForgeModel* model, ForgeKV* kv, int32_t batch, const uint32_t* tokens,
                            float* logits_host);
/* The generated main's greedy loop (P:714-751 with temperature 0 and repeat penalty 1.0):
 * prefill the prompt, then n_new times {argmax, forward}, token selection on the device.
 * out_tokens: host u32 [n_new]. */
int32_t forge_generate_greedy(ForgeModel* model, ForgeKV* kv, const uint32_t* prompt, size_t m,
                              int32_t n_new, uint32_t* out_tokens);
/* Batched twin of the loop above for the first `batch` sequences after they were prefilled:
 * first_tokens host u32 [batch]; out_tokens host u32 [n_new][batch]. */
int32_t forge_decode_greedy_batch(ForgeModel* model, ForgeKV* kv, int32_t batch,
                                  const uint32_t* first_tokens, int32_t n_new, uint32_t* out_tokens);

/* Token selection of the generated main.rs, on the host logits (project.rs:501-551): argmax when temperature <= 0
 * (last index on ties), else temperature, softmax, top-k, top-p, renormalisation and one draw of the xorshift
 * generator, in the reference's arithmetic order; both calls modify `logits` in place.  The repeat penalty divides a
 * positive logit and multiplies a non-positive one, once per occurrence in `recent`. */
int32_t forge_apply_repeat_penalty(float* logits_host, int32_t n, const uint32_t* recent, size_t n_recent, float penalty);
int32_t forge_sample(float* logits_host, int32_t n, float temperature, int32_t top_k, float top_p, uint64_t* rng_state,
                     uint32_t* token);

/* The prompt -> tokens loop of the generated main.rs (project.rs:714-751): prefill, sample, then until an EOS id or
 * max_tokens: emit, forward, repeat penalty over prompt + emitted tokens, sample.  The reference's command-line
 * defaults are temperature 0, top_k 0, top_p 0.9, repeat_penalty 1.1, seed 0xdeadbeef12345678 (project.rs:608-613).
 * out_tokens: max_tokens entries; *n_out: how many were emitted. */
typedef struct ForgeSampling {
    float temperature;
    int32_t top_k;
    float top_p;
    float repeat_penalty;
    uint64_t seed;
} ForgeSampling;
int32_t forge_generate(ForgeModel* model, ForgeKV* kv, const uint32_t* prompt, size_t n_prompt, int32_t max_tokens,
                       const ForgeSampling* sampling, const uint32_t* eos_tokens, size_t n_eos, uint32_t* out_tokens,
                       int32_t* n_out);
/* One chunk of the reference's corpus scorer (--score-corpus, project.rs:652-712): from an empty cache, per-token
 * forward() over chunk[0 .. n-2]; nll_host[i] = -log softmax(logits after chunk[i])[chunk[i+1]] for i < n-1, formed
 * in f64 from the f32 logits as the reference does.  Perplexity of a corpus = exp(sum of all nll / count). */
int32_t forge_score_chunk(ForgeModel* model, ForgeKV* kv, const uint32_t* chunk, size_t n, double* nll_host);
/* Vocabulary size of the model (the length of a logits row). */
size_t forge_model_vocab_size(const ForgeModel* model);

/* Parity hook: when enabled, the next forward / forward_prefill call records the hidden
 * state after every layer.  forge_hidden_trace_read copies [num_layers][rows][hidden] f32 of
 * the last call to a host buffer and returns the row count through *rows. */
int32_t forge_hidden_trace_enable(ForgeModel* model, int32_t enable);
int32_t forge_hidden_trace_read(ForgeModel* model, float* out_host, size_t capacity_floats, int32_t* rows);

/* Device time (CUDA events on the model's stream) of the prefill part and the decode part of
 * the last forge_generate_greedy / forge_decode_greedy_batch call, in milliseconds, and the
 * number of kernels of this library launched by that call. */
int32_t forge_last_timing(ForgeModel* model, float* prefill_ms, float* decode_ms, int64_t* launches);

/* ------------------------------------------------------------------------------------
 * GGUF input (host only): the reference's `export-weights` step, so a GGUF checkpoint can feed
 * forge_model_create directly.  Parser: crates/forgellm-frontend/src/gguf.rs:484-551 (v2 / v3,
 * little endian); configuration rules: crates/forgellm-cli/src/main.rs:689-811 (head_dim =
 * hidden / heads, defaults, Qwen2 has QKV bias) and the dtype vote :479-560; tensor names:
 * crates/forgellm-frontend/src/weight_loader.rs:400-441; write order: main.rs:2506-2757.
 * Supported: llama / qwen2 / mistral / phi3 (fused attn_qkv and gate|up tensors are split, WL:543-582)
 * whose projections are Q8_0 or Q4_0;
 * embedding and norms F32 / F16 / BF16 (or a Q8_0 embedding); dense or Q8_0 projections in a
 * Q4_0 model are re-quantised with the reference's rule; a missing output.weight ties the head
 * to the embedding.  Anything else returns FORGE_ERR_UNSUPPORTED; a malformed or truncated
 * file returns FORGE_ERR_SHAPE.  `data` must stay mapped while the handle lives.
 * ------------------------------------------------------------------------------------ */
typedef struct ForgeGguf ForgeGguf;
int32_t forge_gguf_open(const void* data, size_t len, ForgeGguf** out);
void forge_gguf_close(ForgeGguf* gguf);
int32_t forge_gguf_version(const ForgeGguf* gguf);
int64_t forge_gguf_tensor_count(const ForgeGguf* gguf);
/* Byte offset of the tensor data section (aligned to general.alignment, default 32). */
uint64_t forge_gguf_data_offset(const ForgeGguf* gguf);
/* Descriptor `index`: dims[4] (innermost first, unused = 0), offset from the data section,
 * size in bytes.  Any output pointer may be null. */
int32_t forge_gguf_tensor_info(const ForgeGguf* gguf, int64_t index, const char** name, int32_t* ggml_type,
                               int32_t* n_dims, uint64_t* dims, uint64_t* offset, uint64_t* data_size);
/* Tensor `index` as f32 (dequantize, weight_loader.rs:809-826): F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q4_K, Q5_K, Q6_K;
 * `capacity` in floats. */
int32_t forge_gguf_tensor_to_f32(const ForgeGguf* gguf, int64_t index, float* out, size_t capacity);
int32_t forge_gguf_model_config(const ForgeGguf* gguf, ForgeModelConfig* cfg);
/* Size of the weights.bin image (0 on error, see forge_last_error) and the image itself. */
size_t forge_gguf_weights_bin_size(const ForgeGguf* gguf);
int32_t forge_gguf_export_weights_bin(const ForgeGguf* gguf, void* out, size_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* FORGE_B200_H */
