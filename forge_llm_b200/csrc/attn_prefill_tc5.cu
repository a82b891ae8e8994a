// Prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM) over the paged fp16 KV cache (replaces
// attention_flash_batch, crates/forgellm-codegen-cpu/src/emit.rs:755-883): query row r sits at position
// base_pos + r and sees cache positions <= its own (:815-818); key tiles stop at the tile's last query (:782,
// :792-793); GQA mapping kv_head = h / (nq/nkv) (:763, :775).
//
// One CTA = 128 query rows of one head; keys and values stream in 64-position tiles (one KV page).  Per tile:
//   S = Q K^T      tcgen05.mma, both operands in shared memory (K-major, SWIZZLE_128B), S[query][key] f32 in TMEM;
//   softmax        four warps, one query row per thread (TMEM lane = query): tcgen05.ld of the row, mask, running
//                  maximum and sum in the base-2 domain, probabilities back into TMEM as packed fp16 (tcgen05.st);
//   O += P V       tcgen05.mma with P as the TMEM operand and the V page as an MN-major shared-memory operand (the
//                  page is [key][dim], dims contiguous); O[query][dim] f32 stays in TMEM for the whole key loop and
//                  is rescaled in place by the row's thread when its maximum moves.
// PRECISE: Q and P enter the products as fp16 hi + lo pairs (S = Q_hi K + Q_lo K, O += P_hi V + P_lo V); K and V are
// the cache's fp16 values either way, so the result is the f32 attention over those values to ~1e-5.
// Warp roles (192 threads): warp 0 = TMA producer (3-D tiled copies: {64 dims, 1 head, rows}), warp 1 = TMEM
// allocation and MMA issue (one lane), warps 2..5 = softmax, rescale and the final store.
// The three stages overlap: S of tile j + 1 is issued as soon as the softmax warps have read S of tile j into registers;
// the probabilities alternate between two buffers, so the softmax of tile j + 1 does not wait for P V of tile j; and the
// running maximum is lazy - a row keeps its reference maximum (probabilities may then exceed 1, up to 2^8) until the
// true maximum has moved by more than 8 in the base-2 domain, so O is rescaled (which does wait for the P V in flight)
// only a few times per row.  Tensor memory: S [0,64), P0 [64,128), P1 [128,192) (hi | lo halves), O from 192: 256 columns
// for 64-wide heads (two CTAs per SM), 512 for wider ones (one CTA per SM, which is also what their shared memory
// allows).  Every wait is bounded; one that gives up sets the error word and the CTA still frees its tensor memory.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"

namespace forge {

namespace {

constexpr int BM = 128;   // query rows per CTA
constexpr int BN = 64;    // keys per tile = one KV page
constexpr int kThreads = 192;
constexpr int KVS = 3;    // K/V stages
constexpr uint32_t kSpinLimit = 1u << 22;
// tensor memory: the scores, two probability buffers (hi | lo each), the output
constexpr uint32_t kColS = 0, kColP = 64, kColO = 192;
template <int HD> struct Tmem { static constexpr uint32_t cols = HD == 64 ? 256 : 512; };
constexpr float kLazy = 8.f;   // a row's reference maximum moves only when the true one exceeds it by 2^8

struct Tc5AttnParams {
    AttnPrefillArgs a;
    float scale_log2;     // 1/sqrt(head_dim) * log2(e)
    int* err;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// bounded wait; also gives up as soon as another role of the CTA has reported a failure
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* cta_err) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if ((i & 1023u) == 1023u && *cta_err) return false;
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
// shared-memory matrix descriptors, SWIZZLE_128B, 8-row groups 1024 bytes apart.
// K-major (rows = M or N index, 64 K values = one 128-byte swizzle row): leading offset unused.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
    return uint64_t((saddr & 0x3FFFF) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// MN-major (rows = K index, 64 N values contiguous in a 128-byte swizzle row): groups of 8 K rows 1024 bytes apart,
// the next 64 N values `chunk` bytes further
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t chunk) {
    return uint64_t((saddr & 0x3FFFF) >> 4) | (uint64_t(chunk >> 4) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// instruction descriptors: D f32, A/B f16, M = 128
template <int N, bool B_MN_MAJOR> struct Idesc {
    static constexpr uint32_t value = (1u << 4) | (B_MN_MAJOR ? (1u << 16) : 0u) | (uint32_t(N >> 3) << 17) | (uint32_t(128 >> 4) << 24);
};

__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_h2_lo(float a, float b, uint32_t hi) {  // what pack_h2 dropped
    const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    return pack_h2(a - hf.x, b - hf.y);
}

// HD: head_dim (64, 96, 128); SW: sliding window; PRECISE: hi + lo operands
template <int HD, bool SW, bool PRECISE>
__global__ void __launch_bounds__(kThreads) attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_qlo,
                                                                     const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                                                     Tc5AttnParams p) {
    constexpr int NCH = (HD + 63) / 64;              // 64-dim chunks of a row (the last may be half used)
    constexpr int NP = PRECISE ? 2 : 1;
    constexpr int Q_CHUNK = BM * 128;                // bytes: 128 rows x 128-byte swizzle row
    constexpr int KV_CHUNK = BN * 128;
    constexpr int Q_BYTES = NP * NCH * Q_CHUNK;
    constexpr int STAGE = 2 * NCH * KV_CHUNK;        // K chunks, then V chunks
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* sQ = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sKV = sQ + Q_BYTES;
    __shared__ uint64_t q_full, kv_full[KVS], kv_empty[KVS], s_full, s_free, p_full[2], pv_done[2];
    constexpr uint32_t kTmemCols = Tmem<HD>::cols;
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;

    const AttnPrefillArgs& a = p.a;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // CTAs in the order of their work: all heads of the last query tile (the most key tiles) first, the first tile last
    const int linear = int(blockIdx.x + gridDim.x * blockIdx.y);
    const int h_ = linear % a.nq, tile = int(gridDim.x) - 1 - linear / a.nq;
    const int h = h_, kvh = h / (a.nq / a.nkv);
    const int q0 = tile * BM;
    const int q_last = min(q0 + BM, a.m) - 1;
    const int lp_last = (a.base_pos + q_last) / BN;
    const int lp_first = (SW && a.base_pos + q0 - a.window + 1 > 0) ? (a.base_pos + q0 - a.window + 1) / BN : 0;
    const int nblk = lp_last - lp_first + 1;

    if (tid == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < KVS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        mbar_init(&s_full, 1);
        mbar_init(&s_free, 4);
        for (int s = 0; s < 2; ++s) { mbar_init(&p_full[s], 4); mbar_init(&pv_done[s], 1); }
        s_err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "n"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == 0) {
        // ---------------- TMA producer: the query tile once, then the K and V pages of every key tile
        if (lane == 0) {
            mbar_expect_tx(&q_full, uint32_t(Q_BYTES));
            for (int c = 0; c < NCH; ++c) {
                tma_load_3d(sQ + c * Q_CHUNK, &map_q, c * 64, h, q0, &q_full);
                if (PRECISE) tma_load_3d(sQ + (NCH + c) * Q_CHUNK, &map_qlo, c * 64, h, q0, &q_full);
            }
            for (int j = 0; j < nblk; ++j) {
                const int s = j % KVS, use = j / KVS;
                if (use > 0 && !mbar_wait(&kv_empty[s], (use - 1) & 1, &s_err)) { atomicExch(&s_err, 1); break; }
                const int lp = lp_first + j;
                const int row = (a.page_row ? a.page_row[lp] : lp) * BN;
                unsigned char* dst = sKV + size_t(s) * STAGE;
                mbar_expect_tx(&kv_full[s], uint32_t(STAGE));
                for (int c = 0; c < NCH; ++c) {
                    tma_load_3d(dst + c * KV_CHUNK, &map_k, c * 64, kvh, row, &kv_full[s]);
                    tma_load_3d(dst + (NCH + c) * KV_CHUNK, &map_v, c * 64, kvh, row, &kv_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: S of the next tile as soon as the score buffer has been read, then P V of this one
        if (lane == 0) {
            bool ok = mbar_wait(&q_full, 0, &s_err);
            const uint32_t q_base = smem_u32(sQ);
            auto issue_s = [&](int j) {   // S = Q K_j^T
                const uint32_t k_base = smem_u32(sKV + size_t(j % KVS) * STAGE);
#pragma unroll
                for (int pass = 0; pass < NP; ++pass)
#pragma unroll
                    for (int k16 = 0; k16 < HD / 16; ++k16) {
                        const uint32_t off = uint32_t(k16 / 4), in = uint32_t((k16 % 4) * 32);
                        umma_ss(tmem + kColS, desc_kmajor(q_base + (pass * NCH + off) * Q_CHUNK + in), desc_kmajor(k_base + off * KV_CHUNK + in),
                                Idesc<BN, false>::value, (pass > 0 || k16 > 0) ? 1u : 0u);
                    }
                umma_commit(&s_full);
            };
            if (ok && mbar_wait(&kv_full[0], 0, &s_err)) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_s(0);
            } else {
                ok = false;
            }
            for (int j = 0; j < nblk && ok; ++j) {
                if (j + 1 < nblk) {
                    if (!mbar_wait(&kv_full[(j + 1) % KVS], ((j + 1) / KVS) & 1, &s_err) || !mbar_wait(&s_free, j & 1, &s_err)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_s(j + 1);
                }
                if (!mbar_wait(&p_full[j & 1], (j >> 1) & 1, &s_err)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t v_base = smem_u32(sKV + size_t(j % KVS) * STAGE) + NCH * KV_CHUNK;
                const uint32_t p_base = tmem + kColP + uint32_t((j & 1) * 64);
#pragma unroll
                for (int pass = 0; pass < NP; ++pass)
#pragma unroll
                    for (int k16 = 0; k16 < BN / 16; ++k16)
                        umma_ts(tmem + kColO, p_base + uint32_t(pass * 32 + k16 * 8), desc_mnmajor(v_base + k16 * 2048, KV_CHUNK),
                                Idesc<HD, true>::value, (j > 0 || pass > 0 || k16 > 0) ? 1u : 0u);
                umma_commit(&pv_done[j & 1]);
                umma_commit(&kv_empty[j % KVS]);
            }
            if (!ok) atomicExch(&s_err, 1);
        }
    } else {
        // ---------------- softmax (warps 2..5): TMEM lane = query row; a warp may only touch its lane quadrant
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const int pq = a.base_pos + q0 + r;           // position of this thread's query
        const uint32_t lane_addr = tmem + (uint32_t(quad * 32) << 16);
        float m_ref = -INFINITY, l_run = 0.f;         // reference maximum (base-2 domain, scaled) and the sum relative to it
        bool ok = true;
        for (int j = 0; j < nblk; ++j) {
            const int t0 = (lp_first + j) * BN;
            if (ok && !mbar_wait(&s_full, j & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t sv[2][32];
            tmem_ld32(lane_addr + kColS, sv[0]);
            tmem_ld32(lane_addr + kColS + 32, sv[1]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free);   // the scores are in registers: the next tile's S may be formed
            // scores stay raw; the maximum and the exponent's argument take the scale (s * c - m * c is one fused
            // multiply-add).  Only a tile that reaches past some row's position (or starts before its window) is masked.
            const bool masked = t0 + BN - 1 > a.base_pos + q0 || (SW && t0 <= a.base_pos + q0 + BM - 1 - a.window);
            if (masked) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int t = t0 + c;
                    const bool seen = t <= pq && (!SW || t > pq - a.window);
                    if (!seen) sv[c >> 5][c & 31] = 0xff800000u;  // -inf
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four independent chains
#pragma unroll
            for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c >> 5][c & 31]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;   // scale > 0: max(s) * c = max(s * c)
            // a row that had seen nothing takes the tile's maximum (its O is still exactly zero); otherwise the reference
            // moves, and O and l are rescaled, only when the maximum has grown past the slack
            float alpha = 1.f;
            if (m_ref == -INFINITY) m_ref = mx;
            else if (mx > m_ref + kLazy) { alpha = ex2(m_ref - mx); m_ref = mx; }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;   // nothing seen yet: every p is 0
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t ph[32], pl[32];
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
                const float p0 = ex2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), p.scale_log2, -m_use));
                const float p1 = ex2(fmaf(__uint_as_float(sv[c >> 5][(c & 31) + 1]), p.scale_log2, -m_use));
                sum4[(c >> 1) & 3] += p0 + p1;
                ph[c >> 1] = pack_h2(p0, p1);
                if (PRECISE) pl[c >> 1] = pack_h2_lo(p0, p1, ph[c >> 1]);
            }
            l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            // this tile's probability buffer was last read by P V of tile j - 2
            if (j >= 2 && ok && !mbar_wait(&pv_done[j & 1], ((j >> 1) - 1) & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // O changes scale: every P V issued so far must be complete (the next one waits for this tile's probabilities)
                if (ok && !mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(lane_addr + kColO + c0, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_addr + kColO + c0, o);
                }
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t p_addr = lane_addr + kColP + uint32_t((j & 1) * 64);
            tmem_st32(p_addr, ph);
            if (PRECISE) tmem_st32(p_addr + 32, pl);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[j & 1]);
        }
        // ---------------- the tile's output: O / l
        if (ok && !mbar_wait(&pv_done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        const int qr = q0 + r;
        const size_t row_off = (size_t(qr) * a.nq + h) * HD;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(lane_addr + kColO + c0, o);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (qr < a.m && ok) {
                if (a.out32) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(a.out32 + row_off + c0 + i) =
                            make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv, __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float x0 = __uint_as_float(o[i + 2 * e]) * inv, x1 = __uint_as_float(o[i + 2 * e + 1]) * inv;
                            hi[e] = pack_h2(x0, x1);
                            lo[e] = pack_h2_lo(x0, x1, hi[e]);
                        }
                        *reinterpret_cast<uint4*>(a.out16 + row_off + c0 + i) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        if (a.out16_lo) *reinterpret_cast<uint4*>(a.out16_lo + row_off + c0 + i) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kTmemCols) : "memory");
    }
    if (tid == 0 && s_err && p.err) atomicExch(p.err, 1);
}

// ---- host: tensor maps through the driver entry point (no link-time dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// {head_dim, heads, rows} fp16, box {64 dims, 1 head, box_rows}, SWIZZLE_128B; dims beyond head_dim and rows beyond
// `rows` read as zero
int32_t make_map3(CUtensorMap* map, const __half* base, int hd, int heads, size_t rows, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return FORGE_ERR_UNSUPPORTED; }
    const cuuint64_t dims[3] = {cuuint64_t(hd), cuuint64_t(heads), cuuint64_t(rows)};
    const cuuint64_t strides[2] = {cuuint64_t(hd) * 2, cuuint64_t(heads) * hd * 2};
    const cuuint32_t box[3] = {64, 1, cuuint32_t(box_rows)};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed for an attention operand (%d)", int(r)); return FORGE_ERR_CUDA; }
    return FORGE_OK;
}

template <int HD, bool SW, bool PRECISE>
int32_t launch(const CUtensorMap& mq, const CUtensorMap& mql, const CUtensorMap& mk, const CUtensorMap& mv, const Tc5AttnParams& p, cudaStream_t st) {
    constexpr int NCH = (HD + 63) / 64;
    const size_t smem = size_t(PRECISE ? 2 : 1) * NCH * BM * 128 + size_t(KVS) * 2 * NCH * BN * 128 + 1024;
    auto kern = attn_prefill_tc5_kernel<HD, SW, PRECISE>;
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    dim3 grid((p.a.m + BM - 1) / BM, p.a.nq);
    kern<<<grid, kThreads, smem, st>>>(mq, mql, mk, mv, p);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

template <int HD>
int32_t launch_hd(const CUtensorMap& mq, const CUtensorMap& mql, const CUtensorMap& mk, const CUtensorMap& mv, const Tc5AttnParams& p, cudaStream_t st) {
    const bool sw = p.a.window > 0;
    if (p.a.precise) return sw ? launch<HD, true, true>(mq, mql, mk, mv, p, st) : launch<HD, false, true>(mq, mql, mk, mv, p, st);
    return sw ? launch<HD, true, false>(mq, mql, mk, mv, p, st) : launch<HD, false, false>(mq, mql, mk, mv, p, st);
}

}  // namespace

int32_t attn_prefill(const AttnPrefillArgs& a, cudaStream_t st) {
    if (a.m <= 0) return FORGE_OK;
    if (a.nq % a.nkv) { set_error("attention: num_heads %d not a multiple of num_kv_heads %d", a.nq, a.nkv); return FORGE_ERR_SHAPE; }
    if (a.hd != 64 && a.hd != 96 && a.hd != 128) { set_error("attention: head_dim %d unsupported (64, 96, 128)", a.hd); return FORGE_ERR_SHAPE; }
    if (!a.q16 || (a.precise && !a.q16_lo) || a.pool_rows == 0) { set_error("attention: fp16 queries and the cache's row count are required"); return FORGE_ERR_INVALID_ARG; }
    CUtensorMap mq, mql, mk, mv;
    FORGE_TRY(make_map3(&mq, a.q16, a.hd, a.nq, size_t(a.m), BM));
    FORGE_TRY(make_map3(&mql, a.precise ? a.q16_lo : a.q16, a.hd, a.nq, size_t(a.m), BM));
    FORGE_TRY(make_map3(&mk, a.k_pool, a.hd, a.nkv, a.pool_rows, BN));
    FORGE_TRY(make_map3(&mv, a.v_pool, a.hd, a.nkv, a.pool_rows, BN));
    Tc5AttnParams p{a, 1.0f / sqrtf(float(a.hd)) * 1.4426950408889634f, a.err};
    switch (a.hd) {
        case 64: return launch_hd<64>(mq, mql, mk, mv, p, st);
        case 96: return launch_hd<96>(mq, mql, mk, mv, p, st);
    }
    return launch_hd<128>(mq, mql, mk, mv, p, st);
}

}  // namespace forge
