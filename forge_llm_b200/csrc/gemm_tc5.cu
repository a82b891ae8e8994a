// Prefill GEMM on the 5th-generation tensor cores (tcgen05 + TMEM): out[m][N] = A[m][K] x W[N][K]^T with W
// streamed as Q8_0 / Q4_0 blocks and dequantised on the fly (replaces matmul_mat_q8_0_KxN /
// matmul_mat_q4_0_KxN, crates/forgellm-codegen-cpu/src/emit.rs:2278-2299 and :3792-3813).
//
// CTA tile: (MT x 128) activation rows x 128 weight rows, K step 64.  Warp roles (320 threads):
//   warp 0      TMA producer: 2-D tiled bulk copies (SWIZZLE_128B) of the fp16 activation tiles (hi and lo
//               parts) into shared memory, completion on an mbarrier;
//   warp 1      allocates TMEM and issues tcgen05.mma (one elected lane): per K step and per 128-row
//               sub-tile three products accumulate into the same f32 TMEM tile,
//               x_hi*w_hi + x_lo*w_hi + x_hi*w_lo (split precision, see gemm_mma.cu), K = 16 per instruction;
//               tcgen05.commit releases the shared-memory stage and finally publishes the accumulator;
//   warps 2..9  dequantise: each thread owns one 32-value block of one weight row per K step, reads it and its
//               f16 scale from global memory, forms hi = rn16(q*d) and lo = rn16(q*d - hi) with packed-half
//               arithmetic and writes both into the K-major SWIZZLE_128B operand tiles (generic-proxy stores +
//               fence.proxy.async); after the main loop the same warps read the accumulator with tcgen05.ld
//               (two warps per TMEM lane quadrant) and write f32 rows (+ residual).
// Every wait is bounded; a wait that gives up sets an error word, and the CTA still frees its TMEM.
#include <cuda.h>

#include "common.cuh"

namespace forge {

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kThreads = 320;
constexpr int kTileBytes = BM * BK * 2;  // one 128 x 64 fp16 operand tile = 16 KB (1024-byte aligned)
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
// instruction descriptor: D f32, A/B f16, both K-major, M = 128, N = 128
constexpr uint32_t kIdesc = (1u << 4) | (uint32_t(BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct Tc5Params {
    float* out; const float* resid;
    const uint8_t* qs; const __half* d;
    int m, N, K;
    int* err;
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

// eight consecutive weights of one row -> one 16-byte chunk of the hi tile and of the lo tile.
// K-major SWIZZLE_128B: row r at r*128 bytes, 16-byte chunk c stored at chunk (c ^ (r & 7)).
// w0, w1: for Q8_0 the eight int8 values; for Q4_0 eight bytes whose nibbles at bit `sh` are the values.
template <int QUANT, bool SPLIT>
__device__ __forceinline__ void dequant_chunk(unsigned char* hi_tile, unsigned char* lo_tile, int row, int chunk, uint32_t w0,
                                              uint32_t w1, int sh, __half2 d2) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t word = i < 2 ? w0 : w1;
        const uint32_t sel = (i & 1) ? 0x4342u : 0x4140u;  // bytes (2,3) or (0,1) into the low bytes of each half
        __half2 q;
        if (QUANT == FORGE_Q8_0) {
            // int8 b -> fp16: 0x6400 | (b + 128) is 1024 + b + 128
            q = __hsub2(as_h2(prmt(word ^ 0x80808080u, 0x64646464u, sel)), __float2half2_rn(1152.f));
        } else {
            // nibble n -> fp16: 0x6400 | n is 1024 + n; the stored value is n - 8
            const uint32_t two = prmt(word, 0u, sel) >> sh;
            q = __hsub2(as_h2((two & 0x000F000Fu) | 0x64006400u), __float2half2_rn(1032.f));
        }
        if (SPLIT) scale_split(q, d2, h[i], l[i]);
        else h[i] = as_u32(__hmul2(q, d2));
    }
    const uint32_t off = uint32_t(row) * 128u + uint32_t((chunk ^ (row & 7)) << 4);
    *reinterpret_cast<uint4*>(hi_tile + off) = make_uint4(h[0], h[1], h[2], h[3]);
    if (SPLIT) *reinterpret_cast<uint4*>(lo_tile + off) = make_uint4(l[0], l[1], l[2], l[3]);
}

// MT: 128-row activation sub-tiles per CTA; SPLIT: hi/lo split precision (3 passes) or one fp16 pass; STAGES: ring depth
template <int QUANT, int MT, bool SPLIT, int STAGES>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_hi,
                                                               const __grid_constant__ CUtensorMap map_lo, Tc5Params p) {
    constexpr int NP = SPLIT ? 2 : 1;                     // operand parts (hi, lo)
    constexpr int A_STAGE = MT * NP * kTileBytes, B_STAGE = NP * kTileBytes;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment for the swizzle atoms
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = smem;                              // [STAGES][MT][NP][16 KB]
    unsigned char* sB = smem + size_t(STAGES) * A_STAGE;   // [STAGES][NP][16 KB]
    __shared__ uint64_t full_a[STAGES], full_b[STAGES], empty[STAGES], accum_full;
    __shared__ uint32_t s_tmem;
    __shared__ int s_err;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * (BM * MT);
    const int nk = p.K / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_a[s], 1); mbar_init(&full_b[s], 8); mbar_init(&empty[s], 1); }
        mbar_init(&accum_full, 1);
        s_err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM: MT accumulators of 128 lanes x 128 f32 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "n"(MT * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == 0) {
        // ---------------- TMA producer (activation tiles)
        if (lane == 0) {
            for (int kt = 0; kt < nk; ++kt) {
                const int s = kt % STAGES, use = kt / STAGES;
                if (use > 0 && !mbar_wait(&empty[s], (use - 1) & 1, &s_err)) { atomicExch(&s_err, 1); break; }
                mbar_expect_tx(&full_a[s], uint32_t(A_STAGE));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    unsigned char* dst = sA + size_t(s) * A_STAGE + size_t(mt) * NP * kTileBytes;
                    tma_load_2d(dst, &map_hi, kt * BK, m0 + mt * BM, &full_a[s]);
                    if (SPLIT) tma_load_2d(dst + kTileBytes, &map_lo, kt * BK, m0 + mt * BM, &full_a[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < nk && ok; ++kt) {
                const int s = kt % STAGES, use = kt / STAGES;
                if (!mbar_wait(&full_a[s], use & 1, &s_err) || !mbar_wait(&full_b[s], use & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_base = smem_u32(sA + size_t(s) * A_STAGE), b_base = smem_u32(sB + size_t(s) * B_STAGE);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int pass = 0; pass < (SPLIT ? 3 : 1); ++pass) {
                        // pass 0: x_hi w_hi   pass 1: x_lo w_hi   pass 2: x_hi w_lo
                        const uint32_t a_tile = a_base + uint32_t(mt * NP + (pass == 1 ? 1 : 0)) * kTileBytes;
                        const uint32_t b_tile = b_base + uint32_t(pass == 2 ? 1 : 0) * kTileBytes;
#pragma unroll
                        for (int k16 = 0; k16 < BK / 16; ++k16) {
                            const uint32_t acc = (kt > 0 || pass > 0 || k16 > 0) ? 1u : 0u;
                            umma_f16(tmem + uint32_t(mt * BN), umma_desc(a_tile + k16 * 32), umma_desc(b_tile + k16 * 32), acc);
                        }
                    }
                }
                umma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
            }
            umma_commit(&accum_full);    // all MMAs done: the accumulators are complete
        }
    } else {
        // ---------------- dequantise (warps 2..9): thread -> weight row n0 + r, 32-value block blk of the K step
        const int r = (tid - 64) & 127, blk = (tid - 64) >> 7;
        const int n = n0 + r;
        const bool n_ok = n < p.N;
        const size_t qrow = QUANT == FORGE_Q8_0 ? size_t(p.K) : size_t(p.K) / 2;
        constexpr int QB = QUANT == FORGE_Q8_0 ? 32 : 16;  // bytes of quantised values per block
        constexpr int QV = QB / 16;
        const uint8_t* qsrc = p.qs + size_t(n_ok ? n : 0) * qrow + size_t(blk) * QB;
        const __half* dsrc = p.d + size_t(n_ok ? n : 0) * (p.K / 32) + blk;
        // the quantised values travel through a small register queue, kPrefetch K steps ahead of their use: the
        // rows are far apart in memory, so each load is a separate L2 / HBM round trip that must be hidden
        constexpr int kPrefetch = 4;
        uint4 q[kPrefetch][QV];
        __half dsc[kPrefetch];
        auto gload = [&](int kt, int slot) {
            if (n_ok && kt < nk) {
#pragma unroll
                for (int i = 0; i < QV; ++i) q[slot][i] = __ldg(reinterpret_cast<const uint4*>(qsrc + size_t(kt) * (2 * QB)) + i);
                dsc[slot] = dsrc[2 * kt];
            } else {
#pragma unroll
                for (int i = 0; i < QV; ++i) q[slot][i] = make_uint4(0, 0, 0, 0);
                dsc[slot] = __float2half(0.f);
            }
        };
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) gload(j, j);
        bool ok = true;
        for (int kt = 0; kt < nk; ++kt) {
            const int s = kt % STAGES, use = kt / STAGES;
            uint32_t cur[4 * QV];
#pragma unroll
            for (int i = 0; i < QV; ++i) { cur[4 * i] = q[0][i].x; cur[4 * i + 1] = q[0][i].y; cur[4 * i + 2] = q[0][i].z; cur[4 * i + 3] = q[0][i].w; }
            const __half2 d2 = __half2half2(dsc[0]);
#pragma unroll
            for (int j = 0; j + 1 < kPrefetch; ++j) {
#pragma unroll
                for (int i = 0; i < QV; ++i) q[j][i] = q[j + 1][i];
                dsc[j] = dsc[j + 1];
            }
            gload(kt + kPrefetch, kPrefetch - 1);
            if (ok && use > 0 && !mbar_wait(&empty[s], (use - 1) & 1, &s_err)) { atomicExch(&s_err, 1); ok = false; }
            unsigned char* hi_tile = sB + size_t(s) * B_STAGE;
            unsigned char* lo_tile = hi_tile + kTileBytes;
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // 8 values per 16-byte fp16 chunk
                if (QUANT == FORGE_Q8_0) {
                    dequant_chunk<QUANT, SPLIT>(hi_tile, lo_tile, r, blk * 4 + c, cur[2 * c], cur[2 * c + 1], 0, d2);
                } else {
                    // block bytes j = 0..15: element j in the low nibble, element j + 16 in the high nibble
                    dequant_chunk<QUANT, SPLIT>(hi_tile, lo_tile, r, blk * 4 + c, cur[2 * (c & 1)], cur[2 * (c & 1) + 1], (c >> 1) * 4, d2);
                }
            }
            // make the generic-proxy stores visible to the tensor core (async proxy), then signal
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_b[s]);
        }

        // ---------------- epilogue: TMEM -> registers -> global (warp w reads lane quadrant w % 4)
        if (!mbar_wait(&accum_full, 0, &s_err)) atomicExch(&s_err, 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quad = warp & 3, chalf = (warp - 2) >> 2;  // two warps per lane quadrant, 64 columns each
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int row = m0 + mt * BM + quad * 32 + lane;
#pragma unroll
            for (int c0 = chalf * 64; c0 < chalf * 64 + 64; c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16) + uint32_t(mt * BN + c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                    "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                      "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                      "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < p.m) {
                    float* orow = p.out + size_t(row) * p.N + n0 + c0;
                    const float* rrow = p.resid ? p.resid + size_t(row) * p.N + n0 + c0 : nullptr;
                    if (n0 + c0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                            if (rrow) { const float4 rr = *reinterpret_cast<const float4*>(rrow + j); o.x += rr.x; o.y += rr.y; o.z += rr.z; o.w += rr.w; }
                            *reinterpret_cast<float4*>(orow + j) = o;
                        }
                    } else {
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c0 + j < p.N) orow[j] = (rrow ? rrow[j] : 0.f) + __uint_as_float(v[j]);
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(MT * BN) : "memory");
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

int32_t make_map(CUtensorMap* map, const __half* base, int m, int K) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return FORGE_ERR_UNSUPPORTED; }
    const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(m)};
    const cuuint64_t strides[1] = {cuuint64_t(K) * 2};
    const cuuint32_t box[2] = {BK, BM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", int(r)); return FORGE_ERR_CUDA; }
    return FORGE_OK;
}

template <int QUANT, int MT, bool SPLIT>
int32_t launch(const CUtensorMap& mh, const CUtensorMap& ml, const Tc5Params& p, cudaStream_t st) {
    constexpr int NP = SPLIT ? 2 : 1;
    constexpr int STAGE = (MT * NP + NP) * kTileBytes;
    constexpr int STAGES = (200 * 1024) / STAGE >= 4 ? 4 : (200 * 1024) / STAGE;
    static_assert(STAGES >= 2, "pipeline needs at least two stages");
    const size_t smem = size_t(STAGES) * STAGE + 1024;
    auto kern = gemm_tc5_kernel<QUANT, MT, SPLIT, STAGES>;
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    dim3 grid((p.N + BN - 1) / BN, (p.m + BM * MT - 1) / (BM * MT));
    kern<<<grid, kThreads, smem, st>>>(mh, ml, p);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace

bool gemm_tc5_supported(const QWeight& w) { return w.K % BK == 0 && w.K >= BK; }

int32_t gemm_tc5(float* out, const __half* A, const __half* Alo, const QWeight& w, int m, const float* resid, int* err, cudaStream_t st) {
    if (m <= 0) return FORGE_OK;
    if (!gemm_tc5_supported(w)) { set_error("tcgen05 gemm: K=%d must be a multiple of %d", w.K, BK); return FORGE_ERR_SHAPE; }
    CUtensorMap mh, ml;
    FORGE_TRY(make_map(&mh, A, m, w.K));
    FORGE_TRY(make_map(&ml, Alo ? Alo : A, m, w.K));
    Tc5Params p{out, resid, w.qs, w.d, m, w.N, w.K, err};
    const bool split = Alo != nullptr;
    // two activation sub-tiles per CTA reuse every dequantised weight tile twice; use it when the grid still fills the GPU
    // (a CTA with two sub-tiles costs about 1.5x one with a single sub-tile; compare whole rounds over the SMs)
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long nt = (w.N + BN - 1) / BN;
    const long ctas1 = nt * ((m + BM - 1) / BM), ctas2 = nt * ((m + 2 * BM - 1) / (2 * BM));
    const bool mt2 = m > BM && 3 * ((ctas2 + sms - 1) / sms) <= 2 * ((ctas1 + sms - 1) / sms);
#define FORGE_TC5(Q)                                                                             \
    do {                                                                                         \
        if (split) return mt2 ? launch<Q, 2, true>(mh, ml, p, st) : launch<Q, 1, true>(mh, ml, p, st);   \
        return mt2 ? launch<Q, 2, false>(mh, ml, p, st) : launch<Q, 1, false>(mh, ml, p, st);   \
    } while (0)
    if (w.quant == FORGE_Q8_0) FORGE_TC5(FORGE_Q8_0);
    FORGE_TC5(FORGE_Q4_0);
#undef FORGE_TC5
}

}  // namespace forge
