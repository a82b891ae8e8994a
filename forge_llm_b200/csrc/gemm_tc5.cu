// Prefill GEMM on the 5th-generation tensor cores (tcgen05 + TMEM): out[m][N] = A[m][K] x W[N][K]^T with W
// streamed as Q8_0 / Q4_0 blocks and dequantised on the fly (replaces matmul_mat_q8_0_KxN /
// matmul_mat_q4_0_KxN, crates/forgellm-codegen-cpu/src/emit.rs:2278-2299 and :3792-3813).
//
// CTA tile: 128 weight rows (MMA M) x NT tokens (MMA N = 128, 192 or 256), K step 64.  The dequantised weight
// tile is the A operand and lives in TENSOR memory; the activation tile is the B operand in shared memory;
// D[weight row][token] accumulates in tensor memory (f32).  Warp roles (320 threads):
//   warp 0      TMA producer: 2-D tiled bulk copies (SWIZZLE_128B) of the fp16 activation tiles (hi and lo
//               parts) into a ring of shared-memory stages, completion on an mbarrier;
//   warp 1      allocates TMEM and issues tcgen05.mma (one lane), K = 16 per instruction: per K step three products
//               accumulate into the same tile, w_hi*x_hi + w_hi*x_lo + w_lo*x_hi (split precision, see
//               gemm_mma.cu); tcgen05.commit releases the activation stage and the weight stage and finally
//               publishes the accumulator;
//   warps 2..9  dequantise: each thread owns one 32-value block of one weight row per K step, reads it and its
//               f16 scale from global memory (through a register queue four K steps deep), forms
//               hi = rn16(q*d) and lo = rn16(q*d - hi) with packed-half arithmetic and writes both with
//               tcgen05.st into one of four weight stages in tensor memory (row = TMEM lane, two fp16 per
//               32-bit column); after the main loop the same warps read the accumulator with tcgen05.ld (two
//               warps per lane quadrant) and store f32 rows (+ residual): a warp writes 32 consecutive output
//               columns of one token, so the stores are coalesced.
// Shared memory carries only the activations: one operand read per product.  (With both operands in shared memory
// the reads of a 128 x 128 x 16 product, 8 KB per ~68 clocks, saturate the 128 B/clk shared-memory port.)
// Every wait is bounded; a wait that gives up sets an error word, and the CTA still frees its TMEM.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace forge {

namespace {

constexpr int BK = 64;  // K step: one 128-byte swizzle row of fp16
constexpr int kThreads = 320;
constexpr uint32_t kSpinLimit = 1u << 22;

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
    uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if ((i & 1023u) == 1023u && *cta_err) return false;
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// shared-memory matrix descriptor: K-major, SWIZZLE_128B, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= uint64_t((saddr & 0x3FFFF) >> 4);   // start address, 16-byte units
    d |= uint64_t(1) << 16;                  // leading byte offset (unused for swizzled K-major)
    d |= uint64_t(1024 >> 4) << 32;          // stride byte offset between 8-row groups
    d |= uint64_t(1) << 46;                  // descriptor version (Blackwell)
    d |= uint64_t(2) << 61;                  // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct Tc5Params {
    float* out; const float* resid;
    const uint8_t* qs; const __half* d; const float4* sf;
    int m, N, K;
    int* err;
    int ksplit;            // K slices (grid.z); slice z leaves its partial product at out + z * part_stride
    size_t part_stride;
    // gate/up product (weight rows 2j = gate_j, 2j + 1 = up_j): when act_hi is set the epilogue stores
    // SiLU(gate_j) * up_j as fp16 hi (+ lo) into act[token][N / 2] instead of the f32 rows
    __half* act_hi; __half* act_lo;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// two integer weights (exact in fp16) times the block scale: hi = rn16(q*d), lo = rn16(q*d - hi).  The fp16 multiply
// rounds the exact product once and the fused multiply-add forms q*d - hi exactly before its one rounding, so
// hi + lo carries the 19-bit product q*d to the last bit (|lo| <= ulp(hi)/2 is itself exact in fp16).
__device__ __forceinline__ void scale_split(__half2 q, __half2 d, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __hmul2(q, d);
    hi = as_u32(h);
    lo = as_u32(__hfma2(q, d, __hneg2(h)));
}

// instruction descriptor: D f32, A/B f16, both K-major, M = 128 weight rows, N = NT tokens
template <int NT> struct TsIdesc { static constexpr uint32_t value = (1u << 4) | (uint32_t(NT >> 3) << 17) | (uint32_t(128 >> 4) << 24); };

template <int NT>
__device__ __forceinline__ void umma_ts_f16(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(TsIdesc<NT>::value), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                   "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
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

// 32 consecutive weights of one row (one quantisation block) -> 16 + 16 packed fp16 pairs (hi, lo)
template <int QUANT, bool SPLIT>
__device__ __forceinline__ void dequant_block(const uint32_t* cur, __half2 d2, uint32_t (&hi)[16], uint32_t (&lo)[16]) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {      // 8 values per group
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // 2 values per register
            __half2 q;
            const uint32_t sel = (i & 1) ? 0x4342u : 0x4140u;
            if (QUANT == FORGE_Q8_0) {
                const uint32_t word = cur[2 * c + (i >> 1)];
                q = __hsub2(as_h2(prmt(word ^ 0x80808080u, 0x64646464u, sel)), __float2half2_rn(1152.f));
            } else {
                const uint32_t word = cur[2 * (c & 1) + (i >> 1)];
                const uint32_t two = prmt(word, 0u, sel) >> ((c >> 1) * 4);
                q = __hsub2(as_h2((two & 0x000F000Fu) | 0x64006400u), __float2half2_rn(1032.f));
            }
            if (SPLIT) scale_split(q, d2, hi[4 * c + i], lo[4 * c + i]);
            else hi[4 * c + i] = as_u32(__hmul2(q, d2));
        }
    }
}

// K-quant rows in the expanded row-major layout (FORGE_KQ_SOA): 32 int8 values and {s_lo, s_hi, mn}; the value
// s * q - mn is formed in f32 (one fused rounding) and split into hi = rn16(w), lo = rn16(w - hi): 22 bits of w.
template <bool SPLIT>
__device__ __forceinline__ void dequant_block_kq(const uint32_t* cur, float4 sc, uint32_t (&hi)[16], uint32_t (&lo)[16]) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {  // register j = elements 2j, 2j + 1
        const uint32_t word = cur[j >> 1];
        const int q0 = int(int8_t(word >> (16 * (j & 1)))), q1 = int(int8_t(word >> (16 * (j & 1) + 8)));
        const float s = j < 8 ? sc.x : sc.y;
        const float w0 = fmaf(s, float(q0), -sc.z), w1 = fmaf(s, float(q1), -sc.z);
        const __half2 h = __floats2half2_rn(w0, w1);
        hi[j] = as_u32(h);
        if (SPLIT) {
            const float2 hf = __half22float2(h);
            lo[j] = as_u32(__floats2half2_rn(w0 - hf.x, w1 - hf.y));
        }
    }
}

template <int QUANT, int NT, bool SPLIT, int XS>
__global__ void __launch_bounds__(kThreads, 1) gemm_ts_kernel(const __grid_constant__ CUtensorMap map_hi,
                                                              const __grid_constant__ CUtensorMap map_lo, Tc5Params p) {
    constexpr int NP = SPLIT ? 2 : 1;
    constexpr int X_TILE = NT * BK * 2;          // bytes of one activation tile (NT tokens x 64 k fp16)
    constexpr int X_STAGE = NP * X_TILE;
    constexpr int WS = 4;                        // weight stages in tensor memory
    constexpr int W_COLS = NP * (BK / 2);        // 32-bit columns of one weight stage (hi | lo)
    constexpr uint32_t kTmemCols = 512;          // accumulator at columns [0, NT), weight stages from column 256
    constexpr uint32_t kWBase = 256;
    static_assert(NT <= 256 && kWBase + WS * W_COLS <= kTmemCols, "tensor memory budget");
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* sX = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_x[XS], empty_x[XS], full_w[WS], empty_w[WS], accum_full;
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * 128, m0 = blockIdx.y * NT;
    // K steps of this CTA: the whole K, or slice blockIdx.z of it (a shorter accumulation chain per accumulator, and
    // more CTAs for matrices with few row tiles; the slices' partial products are added by the consumer)
    const int nk_all = p.K / BK;
    const int kt_begin = (nk_all * int(blockIdx.z)) / p.ksplit;
    const int nk = (nk_all * (int(blockIdx.z) + 1)) / p.ksplit - kt_begin;

    if (tid == 0) {
        for (int s = 0; s < XS; ++s) { mbar_init(&full_x[s], 1); mbar_init(&empty_x[s], 1); }
        for (int s = 0; s < WS; ++s) { mbar_init(&full_w[s], 8); mbar_init(&empty_w[s], 1); }
        mbar_init(&accum_full, 1);
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
        // ---------------- TMA producer: activation tiles (B operand)
        if (lane == 0) {
            for (int kt = 0; kt < nk; ++kt) {
                const int s = kt % XS, use = kt / XS;
                if (use > 0 && !mbar_wait(&empty_x[s], (use - 1) & 1, &s_err)) { atomicExch(&s_err, 1); break; }
                mbar_expect_tx(&full_x[s], uint32_t(X_STAGE));
                unsigned char* dst = sX + size_t(s) * X_STAGE;
                tma_load_2d(dst, &map_hi, (kt_begin + kt) * BK, m0, &full_x[s]);
                if (SPLIT) tma_load_2d(dst + X_TILE, &map_lo, (kt_begin + kt) * BK, m0, &full_x[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: D[weight row][token] += W(TMEM) * X(smem)^T
        if (lane == 0) {
            for (int kt = 0; kt < nk; ++kt) {
                const int sx = kt % XS, sw = kt % WS;
                if (!mbar_wait(&full_x[sx], (kt / XS) & 1, &s_err) || !mbar_wait(&full_w[sw], (kt / WS) & 1, &s_err)) { atomicExch(&s_err, 1); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t x_base = smem_u32(sX + size_t(sx) * X_STAGE);
                const uint32_t w_base = tmem + kWBase + uint32_t(sw * W_COLS);
#pragma unroll
                for (int pass = 0; pass < (SPLIT ? 3 : 1); ++pass) {
                    // pass 0: w_hi x_hi   pass 1: w_hi x_lo   pass 2: w_lo x_hi
                    const uint32_t x_tile = x_base + uint32_t(pass == 1 ? X_TILE : 0);
                    const uint32_t w_tile = w_base + uint32_t(pass == 2 ? BK / 2 : 0);
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16) {
                        const uint32_t acc = (kt > 0 || pass > 0 || k16 > 0) ? 1u : 0u;
                        umma_ts_f16<NT>(tmem, w_tile + uint32_t(k16 * 8), umma_desc(x_tile + k16 * 32), acc);
                    }
                }
                umma_commit(&empty_x[sx]);
                umma_commit(&empty_w[sw]);
            }
            umma_commit(&accum_full);
        }
    } else {
        // ---------------- dequantise (warps 2..9): TMEM lane = weight row; a warp may only touch its lane quadrant
        const int quad = warp & 3, blk = (warp - 2) >> 2;
        const int r = quad * 32 + lane;
        const int n = n0 + r;
        const bool n_ok = n < p.N;
        constexpr bool KQ = QUANT == FORGE_KQ_SOA;
        const size_t qrow = QUANT == FORGE_Q4_0 ? size_t(p.K) / 2 : size_t(p.K);
        constexpr int QB = QUANT == FORGE_Q4_0 ? 16 : 32;
        constexpr int QV = QB / 16;
        const uint8_t* qsrc = p.qs + size_t(n_ok ? n : 0) * qrow + size_t(blk) * QB + size_t(kt_begin) * (2 * QB);
        const __half* dsrc = KQ ? nullptr : p.d + size_t(n_ok ? n : 0) * (p.K / 32) + blk + 2 * kt_begin;
        const float4* fsrc = KQ ? p.sf + size_t(n_ok ? n : 0) * (p.K / 32) + blk + 2 * kt_begin : nullptr;
        constexpr int kPrefetch = 4;
        uint4 q[kPrefetch][QV];
        __half dsc[kPrefetch];
        float4 fsc[KQ ? kPrefetch : 1];
        auto gload = [&](int kt, int slot) {
            if (n_ok && kt < nk) {
#pragma unroll
                for (int i = 0; i < QV; ++i) q[slot][i] = __ldg(reinterpret_cast<const uint4*>(qsrc + size_t(kt) * (2 * QB)) + i);
                if (KQ) fsc[KQ ? slot : 0] = __ldg(fsrc + 2 * kt);
                else dsc[slot] = dsrc[2 * kt];
            } else {
#pragma unroll
                for (int i = 0; i < QV; ++i) q[slot][i] = make_uint4(0, 0, 0, 0);
                if (KQ) fsc[KQ ? slot : 0] = make_float4(0.f, 0.f, 0.f, 0.f);
                else dsc[slot] = __float2half(0.f);
            }
        };
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) gload(j, j);
        bool ok = true;
        const uint32_t lane_base = tmem + (uint32_t(quad * 32) << 16) + kWBase + uint32_t(blk * 16);
        // The queue is a ring with compile-time slot indices (the K loop is unrolled by its depth): a slot is refilled
        // right after it is read and not touched again until kPrefetch steps later.  (Shifting the queue instead
        // would make every step wait for the youngest load.)
        // The stores of step i into tensor memory complete under the arithmetic of step i + 1: a stage is published
        // (wait::st, fence, arrive) one step late.
        static_assert(kPrefetch == WS, "one unrolled round covers the weight stages once");
        auto publish = [&](int stage) {
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_w[stage]);
        };
        for (int kt0 = 0; kt0 < nk; kt0 += kPrefetch) {
#pragma unroll
            for (int j = 0; j < kPrefetch; ++j) {
                const int kt = kt0 + j;
                if (kt >= nk) break;
                const int sw = j, use = kt0 / WS;
                uint32_t cur[4 * QV];
#pragma unroll
                for (int i = 0; i < QV; ++i) { cur[4 * i] = q[j][i].x; cur[4 * i + 1] = q[j][i].y; cur[4 * i + 2] = q[j][i].z; cur[4 * i + 3] = q[j][i].w; }
                const __half2 d2 = __half2half2(dsc[j]);
                const float4 f4 = fsc[KQ ? j : 0];
                gload(kt + kPrefetch, j);
                uint32_t hi[16], lo[16];
                if (KQ) dequant_block_kq<SPLIT>(cur, f4, hi, lo);
                else dequant_block<QUANT == FORGE_KQ_SOA ? FORGE_Q8_0 : QUANT, SPLIT>(cur, d2, hi, lo);
                if (kt > 0) publish((j + WS - 1) % WS);
                if (ok && use > 0 && !mbar_wait(&empty_w[sw], (use - 1) & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t col = lane_base + uint32_t(sw * W_COLS);
                tmem_st16(col, hi);
                if (SPLIT) tmem_st16(col + BK / 2, lo);
            }
        }
        publish((nk - 1) % WS);

        // ---------------- epilogue: lane = weight row, columns = tokens; two warps per lane quadrant split the tokens
        if (!mbar_wait(&accum_full, 0, &s_err)) atomicExch(&s_err, 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int col_n = n0 + r;
        float* const outp = p.out + size_t(blockIdx.z) * p.part_stride;
#pragma unroll 1
        for (int c0 = blk * (NT / 2); c0 < (blk + 1) * (NT / 2); c0 += 32) {
            uint32_t v[32];
            const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16) + uint32_t(c0);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                  "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                  "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                  "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (p.act_hi) {
                // neighbouring lanes hold gate_j and up_j of the same tokens: the even lane takes the first sixteen
                // tokens of the chunk, the odd lane the other sixteen, each getting the partner's half by shuffle
                const bool even = !(lane & 1);
                const size_t half_n = size_t(p.N) / 2;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t got = __shfl_xor_sync(0xffffffffu, even ? v[16 + j] : v[j], 1);
                    const float g = __uint_as_float(even ? v[j] : got), u = __uint_as_float(even ? got : v[16 + j]);
                    const int row = m0 + c0 + (even ? j : 16 + j);
                    if (col_n < p.N && row < p.m) {
                        const float x = (g / (1.0f + expf(-g))) * u;
                        const __half hx = __float2half_rn(x);
                        const size_t off = size_t(row) * half_n + size_t(col_n >> 1);
                        p.act_hi[off] = hx;
                        if (p.act_lo) p.act_lo[off] = __float2half_rn(x - __half2float(hx));
                    }
                }
            } else if (col_n < p.N) {
                // the residual may be the output buffer itself: all of its loads are issued before the first store,
                // otherwise every load would have to wait for the store in front of it (one memory round trip each)
                float rv[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int row = m0 + c0 + j;
                    rv[j] = (p.resid && row < p.m) ? p.resid[size_t(row) * p.N + col_n] : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int row = m0 + c0 + j;
                    if (row < p.m) outp[size_t(row) * p.N + col_n] = rv[j] + __uint_as_float(v[j]);
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

// ------------------------------------------------------------------------------------------------
// The same product for a few rows (m <= 32: batched decode steps, short prompts), bound by the weight stream instead of
// the tensor pipe.  Differences from the kernel above:
//   * the A operand in tensor memory holds the INTEGER weights (exact in fp16), one copy, no block scale;
//   * the rows' hi and lo fp16 parts are the two halves of ONE B operand (MMA N = 2 * NT columns), so a K step is one
//     pass of two K = 16 products per 32-column block;
//   * every block's 128 x 2 NT sums are read out of tensor memory by four scale warps (tcgen05.ld, one weight row per
//     thread) and added into register accumulators with the row's f16 block scale in f32;
//   * every hand-off covers a GROUP of G K steps (rows by TMA, weights from the dequantising warps, block sums to the
//     scale warps and back): a query of an mbarrier costs ~150 clocks even when its phase is complete (measured; a
//     tcgen05.mma or commit issues in ~45), so the single issuing thread must meet few barriers per K step.
// The products are exact in the weights and carry the rows to 22 bits; a tensor-memory chain is two products long.
//   * the quantised bytes reach the dequantising threads through shared memory: 128 rows x 128 bytes per bulk tensor copy
//     (SWIZZLE_128B, so a thread reads its row's 16-byte pieces without bank conflicts), four K steps per stage - a
//     thread-per-row read from global memory fetches one sector per request and cannot keep HBM busy.
// Warps (480 threads): 0 TMA for the rows, 1 MMA issue, 2..9 dequantise (one block of one row per thread and K step),
// 10..13 scale + epilogue, 14 TMA for the weights.
constexpr int kSmallThreads = 480;
constexpr int kSuper = 4;   // K steps per weight stage

// several barriers at once: the queries are issued together, so their latencies overlap
__device__ __forceinline__ bool mbar_wait3(uint64_t* a, uint32_t pa, uint64_t* b, uint32_t pb, uint64_t* c, uint32_t pc, const volatile int* cta_err) {
    const uint32_t aa = smem_u32(a), ab = smem_u32(b), ac = c ? smem_u32(c) : 0;
    uint32_t da = 0, db = 0, dc = c ? 0u : 1u;
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if ((i & 1023u) == 1023u && *cta_err) return false;
        uint32_t ta = 1, tb = 1, tc = 1;
        if (!da) asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ta) : "r"(aa), "r"(pa) : "memory");
        if (!db) asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(tb) : "r"(ab), "r"(pb) : "memory");
        if (!dc) asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(tc) : "r"(ac), "r"(pc) : "memory");
        da |= ta; db |= tb; dc |= tc;
        if (da && db && dc) return true;
    }
    return false;
}

template <int QUANT>
__device__ __forceinline__ void raw_block(const uint32_t* cur, uint32_t (&out)[16]) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t sel = (i & 1) ? 0x4342u : 0x4140u;
            if (QUANT == FORGE_Q8_0) {
                const uint32_t word = cur[2 * c + (i >> 1)];
                out[4 * c + i] = as_u32(__hsub2(as_h2(prmt(word ^ 0x80808080u, 0x64646464u, sel)), __float2half2_rn(1152.f)));
            } else {
                const uint32_t word = cur[2 * (c & 1) + (i >> 1)];
                const uint32_t two = prmt(word, 0u, sel) >> ((c >> 1) * 4);
                out[4 * c + i] = as_u32(__hsub2(as_h2((two & 0x000F000Fu) | 0x64006400u), __float2half2_rn(1032.f)));
            }
        }
    }
}

// NT rows (16 or 32); G = K steps per hand-off group
template <int QUANT, int NT>
__global__ void __launch_bounds__(kSmallThreads, 1) gemm_small_kernel(const __grid_constant__ CUtensorMap map_hi,
                                                                      const __grid_constant__ CUtensorMap map_lo,
                                                                      const __grid_constant__ CUtensorMap map_w, Tc5Params p) {
    constexpr int NC = 2 * NT;                   // MMA N: hi columns, then lo columns
    constexpr int G = NT == 16 ? 2 : 1;          // K steps per group
    constexpr int BG = 2 * G;                    // 32-column blocks per group
    constexpr int X_TILE = NT * BK * 2;          // bytes of one part (hi or lo) of one K step
    constexpr int X_STAGE = G * 2 * X_TILE;
    constexpr int XS = 4;                        // row stages (groups)
    constexpr int W_COLS = BK / 2;               // 32-bit columns of one K step of weights
    constexpr int WG = 256 / (G * W_COLS);       // weight stages (groups) in tensor memory
    constexpr uint32_t kTmemCols = 512, kWBase = 256;   // two sets of BG block-sum buffers in [0, 256), weights from 256
    static_assert(2 * BG * NC <= 256 && NC % 16 == 0 && WG >= 2, "tensor memory budget");
    constexpr int Q_BOXES = QUANT == FORGE_Q4_0 ? 1 : 2;   // 128-byte boxes per row and weight stage (256 columns)
    constexpr int Q_STAGE = Q_BOXES * 128 * 128;
    constexpr int QS = QUANT == FORGE_Q4_0 ? 6 : 4;        // weight stages in shared memory
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* sX = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = sX + XS * X_STAGE;
    __shared__ uint64_t full_x[XS], empty_x[XS], full_w[WG], empty_w[WG], d_full[2], d_free[2], full_q[QS], empty_q[QS];
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * 128;
    const int nk_all = p.K / BK;
    const int kt_begin = (nk_all * int(blockIdx.z)) / p.ksplit;
    const int nk = (nk_all * (int(blockIdx.z) + 1)) / p.ksplit - kt_begin;
    const int ng = (nk + G - 1) / G;             // groups; the K steps of the last one beyond nk carry zero scales

    if (tid == 0) {
        for (int s = 0; s < XS; ++s) { mbar_init(&full_x[s], 1); mbar_init(&empty_x[s], 1); }
        for (int s = 0; s < WG; ++s) { mbar_init(&full_w[s], 8); mbar_init(&empty_w[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&d_full[s], 1); mbar_init(&d_free[s], 4); }
        for (int s = 0; s < QS; ++s) { mbar_init(&full_q[s], 1); mbar_init(&empty_q[s], 8); }
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
    const int nss = (ng * G + kSuper - 1) / kSuper;   // weight stages of this CTA

    if (warp == 14) {
        // ---------------- TMA producer for the weights: 128 rows x 256 columns of quantised bytes per stage
        if (lane == 0) {
            const int bytes_per_col_num = QUANT == FORGE_Q4_0 ? 1 : 2;   // bytes per column, in halves
            for (int ss = 0; ss < nss; ++ss) {
                const int s = ss % QS, use = ss / QS;
                if (use > 0 && !mbar_wait(&empty_q[s], (use - 1) & 1, &s_err)) { atomicExch(&s_err, 1); break; }
                mbar_expect_tx(&full_q[s], uint32_t(Q_STAGE));
                const int x0 = ((kt_begin + ss * kSuper) * BK * bytes_per_col_num) / 2;   // byte offset in the row
#pragma unroll
                for (int b = 0; b < Q_BOXES; ++b) tma_load_2d(sQ + size_t(s) * Q_STAGE + b * 16384, &map_w, x0 + b * 128, n0, &full_q[s]);
            }
        }
    } else if (warp == 0) {
        // ---------------- TMA producer: per group, the rows' hi and lo tiles of its K steps (columns past K read as zero)
        if (lane == 0) {
            for (int gi = 0; gi < ng; ++gi) {
                const int s = gi % XS, use = gi / XS;
                if (use > 0 && !mbar_wait(&empty_x[s], (use - 1) & 1, &s_err)) { atomicExch(&s_err, 1); break; }
                mbar_expect_tx(&full_x[s], uint32_t(X_STAGE));
                unsigned char* dst = sX + size_t(s) * X_STAGE;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    tma_load_2d(dst + g * 2 * X_TILE, &map_hi, (kt_begin + gi * G + g) * BK, 0, &full_x[s]);
                    tma_load_2d(dst + g * 2 * X_TILE + X_TILE, &map_lo, (kt_begin + gi * G + g) * BK, 0, &full_x[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: per group one meeting with its three partners, then 4 G products and three commits
        if (lane == 0) {
            for (int gi = 0; gi < ng; ++gi) {
                const int sx = gi % XS, sw = gi % WG, ds = gi & 1;
                if (!mbar_wait3(&full_x[sx], (gi / XS) & 1, &full_w[sw], (gi / WG) & 1, gi >= 2 ? &d_free[ds] : nullptr, ((gi >> 1) - 1) & 1, &s_err)) {
                    atomicExch(&s_err, 1);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t xd = umma_desc(smem_u32(sX + size_t(sx) * X_STAGE));
                const uint32_t w_base = tmem + kWBase + uint32_t(sw * G * W_COLS);
                const uint32_t d_base = tmem + uint32_t(ds * BG * NC);
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)   // block k16 / 2 of this K step
                        umma_ts_f16<NC>(d_base + uint32_t((2 * g + (k16 >> 1)) * NC), w_base + uint32_t(g * W_COLS + k16 * 8),
                                        xd + uint64_t((g * 2 * X_TILE + k16 * 32) >> 4), (k16 & 1) ? 1u : 0u);
                umma_commit(&d_full[ds]);
                umma_commit(&empty_x[sx]);
                umma_commit(&empty_w[sw]);
            }
        }
    } else if (warp < 10) {
        // ---------------- dequantise (warps 2..9): integer weights as fp16 into tensor memory, lane = weight row
        const int quad = warp & 3, blk = (warp - 2) >> 2;
        const int r = quad * 32 + lane;
        constexpr int QV = QUANT == FORGE_Q4_0 ? 1 : 2;   // 16-byte pieces per block
        constexpr int kUnroll = 8;
        static_assert(kUnroll % G == 0 && (WG * G) % kUnroll == 0 && kUnroll % kSuper == 0, "one unrolled round covers whole groups and stages");
        bool ok = true;
        const uint32_t lane_base = tmem + (uint32_t(quad * 32) << 16) + kWBase + uint32_t(blk * 16);
        const uint32_t sw7 = uint32_t(r & 7);
        for (int kt0 = 0; kt0 < ng * G; kt0 += kUnroll) {
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int kt = kt0 + j;
                if (kt >= ng * G) break;
                const int gi = kt / G, g = kt % G, sw = gi % WG;
                const int ss = kt / kSuper, qi = kt % kSuper, sq = ss % QS;
                if (qi == 0 && ok && !mbar_wait(&full_q[sq], (ss / QS) & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
                // this thread's block: 16-byte pieces of its row, un-swizzled (piece index ^ (row & 7))
                uint32_t cur[4 * QV];
                const unsigned char* stage = sQ + size_t(sq) * Q_STAGE;
#pragma unroll
                for (int i = 0; i < QV; ++i) {
                    const int piece = QUANT == FORGE_Q4_0 ? qi * 2 + blk : ((qi & 1) * 2 + blk) * 2 + i;   // within the row's 128 bytes
                    const int box = QUANT == FORGE_Q4_0 ? 0 : qi >> 1;
                    const uint4 v = *reinterpret_cast<const uint4*>(stage + box * 16384 + r * 128 + ((uint32_t(piece) ^ sw7) << 4));
                    cur[4 * i] = v.x; cur[4 * i + 1] = v.y; cur[4 * i + 2] = v.z; cur[4 * i + 3] = v.w;
                }
                if (qi == kSuper - 1 || kt == ng * G - 1) {   // the stage's bytes are in registers
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty_q[sq]);
                }
                uint32_t w16[16];
                raw_block<QUANT>(cur, w16);
                if (g == 0) {   // first K step of a group: its stage must have been read by the products that used it last
                    const int use = gi / WG;
                    if (ok && use > 0 && !mbar_wait(&empty_w[sw], (use - 1) & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                tmem_st16(lane_base + uint32_t((sw * G + g) * W_COLS), w16);
                if (g == G - 1) {   // the group is complete
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_w[sw]);
                }
            }
        }
    } else {
        // ---------------- scale warps (10..13): block sums out of tensor memory, times the row's block scale, in f32
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const int n = n0 + r;
        const bool n_ok = n < p.N;
        const __half2* dsrc = reinterpret_cast<const __half2*>(p.d + size_t(n_ok ? n : 0) * (p.K / 32) + 2 * kt_begin);   // two scales per K step
        const uint32_t lane_addr = tmem + (uint32_t(quad * 32) << 16);
        float acc[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[c] = 0.f;
        constexpr int kAhead = 4;                // groups of scales in flight
        __half2 dq[kAhead][G];
        auto dload = [&](int gi, int slot) {
#pragma unroll
            for (int g = 0; g < G; ++g) dq[slot][g] = (n_ok && gi * G + g < nk) ? dsrc[gi * G + g] : __float2half2_rn(0.f);
        };
#pragma unroll
        for (int j = 0; j < kAhead; ++j) dload(j, j);
        bool ok = true;
        for (int g0 = 0; g0 < ng; g0 += kAhead) {
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const int gi = g0 + j;
                if (gi >= ng) break;
                const int ds = gi & 1;
                float dsc[BG];
#pragma unroll
                for (int g = 0; g < G; ++g) { const float2 d2 = __half22float2(dq[j][g]); dsc[2 * g] = d2.x; dsc[2 * g + 1] = d2.y; }
                dload(gi + kAhead, j);
                if (ok && !mbar_wait(&d_full[ds], (gi >> 1) & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int b = 0; b < BG; ++b) {
#pragma unroll
                    for (int c0 = 0; c0 < NC; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld32(lane_addr + uint32_t((ds * BG + b) * NC + c0), v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (b == BG - 1 && c0 + 32 >= NC) {   // the group's sums are in registers: its buffers may be overwritten
                            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&d_free[ds]);
                        }
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[c0 + i] = fmaf(dsc[b], __uint_as_float(v[i]), acc[c0 + i]);
                    }
                }
            }
        }
        // ---------------- epilogue: row n, tokens 0..m-1; hi and lo columns added
        float* const outp = p.out + size_t(blockIdx.z) * p.part_stride;
        if (p.act_hi) {
            // neighbouring lanes hold gate_j and up_j: the even lane takes the first half of the tokens, the odd lane the rest
            const bool even = !(lane & 1);
            const size_t half_n = size_t(p.N) / 2;
#pragma unroll
            for (int j = 0; j < NT / 2; ++j) {
                const float first = acc[j] + acc[NT + j], second = acc[NT / 2 + j] + acc[NT + NT / 2 + j];   // tokens j and NT/2 + j
                const float got = __shfl_xor_sync(0xffffffffu, even ? second : first, 1);
                const float g = even ? first : got, u = even ? got : second;
                const int row = even ? j : NT / 2 + j;
                if (n_ok && row < p.m) {
                    const float x = (g / (1.0f + expf(-g))) * u;
                    const __half hx = __float2half_rn(x);
                    const size_t off = size_t(row) * half_n + size_t(n >> 1);
                    p.act_hi[off] = hx;
                    if (p.act_lo) p.act_lo[off] = __float2half_rn(x - __half2float(hx));
                }
            }
        } else if (n_ok) {
            float rv[NT];
#pragma unroll
            for (int j = 0; j < NT; ++j) rv[j] = (p.resid && j < p.m) ? p.resid[size_t(j) * p.N + n] : 0.f;
#pragma unroll
            for (int j = 0; j < NT; ++j)
                if (j < p.m) outp[size_t(j) * p.N + n] = rv[j] + (acc[j] + acc[NT + j]);
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

int32_t make_map(CUtensorMap* map, const __half* base, int m, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return FORGE_ERR_UNSUPPORTED; }
    const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(m)};
    const cuuint64_t strides[1] = {cuuint64_t(K) * 2};
    const cuuint32_t box[2] = {BK, cuuint32_t(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", int(r)); return FORGE_ERR_CUDA; }
    return FORGE_OK;
}

}  // namespace

int32_t make_kv_map(void* out, const __half* pool, int head_dim, int kv_heads, size_t rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return FORGE_ERR_UNSUPPORTED; }
    const cuuint64_t dims[3] = {cuuint64_t(head_dim), cuuint64_t(kv_heads), cuuint64_t(rows)};
    const cuuint64_t strides[2] = {cuuint64_t(head_dim) * 2, cuuint64_t(kv_heads) * head_dim * 2};
    const cuuint32_t box[3] = {cuuint32_t(head_dim), 1, cuuint32_t(FORGE_KV_PAGE)};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(static_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(pool), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed for a KV pool (%d)", int(r)); return FORGE_ERR_CUDA; }
    return FORGE_OK;
}

namespace {

template <int QUANT, int NT, bool SPLIT>
int32_t launch_ts(const __half* A, const __half* Alo, const Tc5Params& p, cudaStream_t st) {
    constexpr int NP = SPLIT ? 2 : 1;
    constexpr int STAGE = NP * NT * BK * 2;
    constexpr int XS = (200 * 1024) / STAGE >= 4 ? 4 : (200 * 1024) / STAGE;
    static_assert(XS >= 2, "pipeline needs at least two stages");
    CUtensorMap mh, ml;
    FORGE_TRY(make_map(&mh, A, p.m, p.K, NT));
    FORGE_TRY(make_map(&ml, Alo ? Alo : A, p.m, p.K, NT));
    const size_t smem = size_t(XS) * STAGE + 1024;
    auto kern = gemm_ts_kernel<QUANT, NT, SPLIT, XS>;
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    dim3 grid((p.N + 127) / 128, (p.m + NT - 1) / NT, p.ksplit);
    kern<<<grid, kThreads, smem, st>>>(mh, ml, p);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

template <int QUANT, int NT>
int32_t launch_small(const __half* A, const __half* Alo, const Tc5Params& p, cudaStream_t st) {
    CUtensorMap mh, ml;
    FORGE_TRY(make_map(&mh, A, p.m, p.K, NT));
    FORGE_TRY(make_map(&ml, Alo, p.m, p.K, NT));
    // the quantised bytes as a 2-D byte tensor {row bytes, N}, box {128 bytes, 128 rows}
    CUtensorMap mw;
    {
        EncodeTiledFn fn = encode_fn();
        if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return FORGE_ERR_UNSUPPORTED; }
        const cuuint64_t row_bytes = QUANT == FORGE_Q4_0 ? cuuint64_t(p.K) / 2 : cuuint64_t(p.K);
        const cuuint64_t dims[2] = {row_bytes, cuuint64_t(p.N)};
        const cuuint64_t strides[1] = {row_bytes};
        const cuuint32_t box[2] = {128, 128};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = fn(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(p.qs), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed for the weight bytes (%d)", int(r)); return FORGE_ERR_CUDA; }
    }
    constexpr int kQStage = (QUANT == FORGE_Q4_0 ? 1 : 2) * 128 * 128, kQStages = QUANT == FORGE_Q4_0 ? 6 : 4;
    const size_t smem = size_t(4) * (NT == 16 ? 2 : 1) * 2 * NT * BK * 2 + size_t(kQStages) * kQStage + 1024;
    auto kern = gemm_small_kernel<QUANT, NT>;
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    dim3 grid((p.N + 127) / 128, 1, p.ksplit);
    kern<<<grid, kSmallThreads, smem, st>>>(mh, ml, mw, p);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace

bool gemm_tc5_supported(const QWeight& w) { return w.K % BK == 0 && w.K >= BK; }

// K slices for a product whose result is added to a residual stream anyway (the consumer adds the slices): as many as
// keep at least 16 K steps (1024 columns) per slice, at most 4.  A tensor-memory accumulator rounds toward zero at every
// accumulation, a bias that grows with the chain (measured: 7e-6 of the result at K = 2048, 2.7e-5 at K = 8192) and,
// being one-sided, adds up over the layers; shorter chains keep it at the K = 2048 level.
int gemm_tc5_ksplit(const QWeight& w) { return std::max(1, std::min(4, w.K / 1024)); }

int32_t gemm_tc5(float* out, const __half* A, const __half* Alo, const QWeight& w, int m, const float* resid, int* err, cudaStream_t st,
                 int ksplit, size_t part_stride, __half* act_hi, __half* act_lo) {
    if (m <= 0) return FORGE_OK;
    if (!gemm_tc5_supported(w)) { set_error("tcgen05 gemm: K=%d must be a multiple of %d", w.K, BK); return FORGE_ERR_SHAPE; }
    if (ksplit < 1 || ksplit > w.K / BK || (ksplit > 1 && (resid || act_hi))) { set_error("tcgen05 gemm: bad K split"); return FORGE_ERR_INVALID_ARG; }
    if (act_hi && ((w.N & 1) || resid)) { set_error("tcgen05 gemm: the SiLU epilogue needs gate/up row pairs and no residual"); return FORGE_ERR_INVALID_ARG; }
    Tc5Params p{out, resid, w.qs, w.d, w.sf, m, w.N, w.K, err, ksplit, part_stride, act_hi, act_lo};
    const bool split = Alo != nullptr;
    // a few rows: the weight-streaming form (exact integer weights, block scales applied to the block sums in f32)
    if (split && m <= 32 && w.quant != FORGE_KQ_SOA) {
        if (w.quant == FORGE_Q8_0) return m <= 16 ? launch_small<FORGE_Q8_0, 16>(A, Alo, p, st) : launch_small<FORGE_Q8_0, 32>(A, Alo, p, st);
        return m <= 16 ? launch_small<FORGE_Q4_0, 16>(A, Alo, p, st) : launch_small<FORGE_Q4_0, 32>(A, Alo, p, st);
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // Token tile: 128, 192 or 256.  A tile's cost is a fixed share (dequantising the 128 x K weight panel, prologue,
    // epilogue) plus a share proportional to its tokens (measured on B200: 0.77 / 0.90 / 1.0 per CTA round); CTAs run
    // in whole rounds over the SMs.  Pick the cheapest.
    const long nt = (w.N + 127) / 128;
    int best = 128;
    double best_cost = 1e30;
    for (int cand : {128, 192, 256}) {
        if (cand > 128 && m <= cand - 64) continue;
        const long ctas = nt * ((m + cand - 1) / cand) * ksplit;
        const double cost = double((ctas + sms - 1) / sms) * (0.55 + 0.45 * cand / 256.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = cand; }
    }
#define FORGE_TS(Q)                                                                  \
    do {                                                                             \
        if (split) {                                                                 \
            if (best == 256) return launch_ts<Q, 256, true>(A, Alo, p, st);          \
            if (best == 192) return launch_ts<Q, 192, true>(A, Alo, p, st);          \
            return launch_ts<Q, 128, true>(A, Alo, p, st);                           \
        }                                                                            \
        if (best == 256) return launch_ts<Q, 256, false>(A, Alo, p, st);             \
        if (best == 192) return launch_ts<Q, 192, false>(A, Alo, p, st);             \
        return launch_ts<Q, 128, false>(A, Alo, p, st);                              \
    } while (0)
    if (w.quant == FORGE_Q8_0) FORGE_TS(FORGE_Q8_0);
    if (w.quant == FORGE_KQ_SOA) FORGE_TS(FORGE_KQ_SOA);
    FORGE_TS(FORGE_Q4_0);
#undef FORGE_TS
}

}  // namespace forge
