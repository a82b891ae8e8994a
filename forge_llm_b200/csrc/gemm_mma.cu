// Prefill GEMM, warp-level tensor-core version: out[m][N] = A[m][K] (fp16) x W[N][K]^T with W
// streamed as packed Q8_0 / Q4_0 blocks and dequantised to fp16 tiles in shared memory
// (replaces matmul_mat_q8_0_KxN / matmul_mat_q4_0_KxN, crates/forgellm-codegen-cpu/src/emit.rs
// :2278-2299 and :3792-3813).  f32 accumulation.  A single fp16 pass rounds both operands to 11
// bits (~3e-4 relative per product row, which compounds past 1e-3 over ~30 layers), so the
// default is the split-precision form: x = x_hi + x_lo and w = w_hi + w_lo, each an fp16 pair,
// and out = x_hi w_hi + x_lo w_hi + x_hi w_lo (three MMA passes, ~1e-6 relative).
// 128x128x32 CTA tile, 8 warps of 64x32, m16n8k16 MMAs, double-buffered shared memory.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace forge {

namespace {

constexpr int BM = 128, BN = 128, BK = 32, LDS = BK + 8, kThreads = 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

struct GemmParams {
    float* out; const __half* A; const __half* Alo; const uint8_t* qs; const __half* d; const float* resid;
    int m, N, K;
};

__device__ __forceinline__ void split_h2(float a, float b, uint32_t& hi, uint32_t& lo) {
    __half2 h = __floats2half2_rn(a, b);
    float2 hf = __half22float2(h);
    __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<uint32_t*>(&h);
    lo = *reinterpret_cast<uint32_t*>(&l);
}

template <int QUANT, bool SPLIT>
__global__ void __launch_bounds__(kThreads) gemm_kernel(GemmParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int NT = SPLIT ? 2 : 1;  // hi (and lo) tiles
    // layout: [buf][A hi, A lo][BM*LDS] then [buf][B hi, B lo][BN*LDS]
    __half* sAbase = reinterpret_cast<__half*>(smem_raw);
    __half* sBbase = sAbase + 2 * NT * BM * LDS;
    auto sA = [&](int buf, int part) { return sAbase + (buf * NT + part) * BM * LDS; };
    auto sB = [&](int buf, int part) { return sBbase + (buf * NT + part) * BN * LDS; };
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nk = p.K / BK;
    const size_t qrow = QUANT == FORGE_Q8_0 ? size_t(p.K) : size_t(p.K) / 2;

    // A loader: 128 rows x 4 chunks of 16 B; thread -> (row = tid/2, chunks 2*(tid%2), +1)
    const int a_row = tid >> 1, a_c = (tid & 1) * 2;
    const bool a_ok = (m0 + a_row) < p.m;
    const __half* a_src = p.A + size_t(a_ok ? m0 + a_row : 0) * p.K + a_c * 8;
    const __half* al_src = SPLIT ? p.Alo + size_t(a_ok ? m0 + a_row : 0) * p.K + a_c * 8 : nullptr;
    // W loader: thread -> (row = tid/2, half = tid%2): elements half*16 .. +15 of the row's block
    const int b_row = tid >> 1, b_half = tid & 1;
    const bool b_ok = (n0 + b_row) < p.N;
    const uint8_t* q_src = p.qs + size_t(b_ok ? n0 + b_row : 0) * qrow;
    const __half* d_src = p.d + size_t(b_ok ? n0 + b_row : 0) * (p.K / 32);

    uint4 ra[2], ral[2], rb;
    float rd;
    auto gload = [&](int kt) {
        if (a_ok) {
            ra[0] = *reinterpret_cast<const uint4*>(a_src + size_t(kt) * BK);
            ra[1] = *reinterpret_cast<const uint4*>(a_src + size_t(kt) * BK + 8);
            if (SPLIT) {
                ral[0] = *reinterpret_cast<const uint4*>(al_src + size_t(kt) * BK);
                ral[1] = *reinterpret_cast<const uint4*>(al_src + size_t(kt) * BK + 8);
            }
        } else {
            ra[0] = ra[1] = ral[0] = ral[1] = make_uint4(0, 0, 0, 0);
        }
        if (b_ok) {
            if (QUANT == FORGE_Q8_0) rb = *reinterpret_cast<const uint4*>(q_src + size_t(kt) * 32 + b_half * 16);
            else rb = *reinterpret_cast<const uint4*>(q_src + size_t(kt) * 16);
            rd = __half2float(d_src[kt]);
        } else {
            rb = make_uint4(0, 0, 0, 0);
            rd = 0.f;
        }
    };
    auto sstore = [&](int buf) {
        *reinterpret_cast<uint4*>(sA(buf, 0) + a_row * LDS + a_c * 8) = ra[0];
        *reinterpret_cast<uint4*>(sA(buf, 0) + a_row * LDS + a_c * 8 + 8) = ra[1];
        if (SPLIT) {
            *reinterpret_cast<uint4*>(sA(buf, 1) + a_row * LDS + a_c * 8) = ral[0];
            *reinterpret_cast<uint4*>(sA(buf, 1) + a_row * LDS + a_c * 8 + 8) = ral[1];
        }
        const uint32_t w[4] = {rb.x, rb.y, rb.z, rb.w};
        uint32_t h[8], hl[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float f0, f1, f2, f3;
            if (QUANT == FORGE_Q8_0) {
                f0 = float(int(int8_t(w[i]))) * rd; f1 = float(int(int8_t(w[i] >> 8))) * rd;
                f2 = float(int(int8_t(w[i] >> 16))) * rd; f3 = float(int(int8_t(w[i] >> 24))) * rd;
            } else {
                const int sh = b_half * 4;  // low nibbles = elements 0..15, high nibbles = 16..31
                f0 = float(int((w[i] >> sh) & 15u) - 8) * rd; f1 = float(int((w[i] >> (8 + sh)) & 15u) - 8) * rd;
                f2 = float(int((w[i] >> (16 + sh)) & 15u) - 8) * rd; f3 = float(int((w[i] >> (24 + sh)) & 15u) - 8) * rd;
            }
            if (SPLIT) {
                split_h2(f0, f1, h[2 * i], hl[2 * i]);
                split_h2(f2, f3, h[2 * i + 1], hl[2 * i + 1]);
            } else {
                h[2 * i] = pack_h2(f0, f1);
                h[2 * i + 1] = pack_h2(f2, f3);
            }
        }
        *reinterpret_cast<uint4*>(sB(buf, 0) + b_row * LDS + b_half * 16) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(sB(buf, 0) + b_row * LDS + b_half * 16 + 8) = make_uint4(h[4], h[5], h[6], h[7]);
        if (SPLIT) {
            *reinterpret_cast<uint4*>(sB(buf, 1) + b_row * LDS + b_half * 16) = make_uint4(hl[0], hl[1], hl[2], hl[3]);
            *reinterpret_cast<uint4*>(sB(buf, 1) + b_row * LDS + b_half * 16 + 8) = make_uint4(hl[4], hl[5], hl[6], hl[7]);
        }
    };

    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f; }

    gload(0);
    sstore(0);
    __syncthreads();
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) gload(kt + 1);
#pragma unroll
        for (int pass = 0; pass < (SPLIT ? 3 : 1); ++pass) {
            // pass 0: x_hi w_hi   pass 1: x_lo w_hi   pass 2: x_hi w_lo
            const int pa = (pass == 1) ? 1 : 0, pb = (pass == 2) ? 1 : 0;
            uint32_t bf[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                ldsm_x4(bf[j], smem_u32(sB(buf, pb) + (wn * 32 + j * 8 + (lane & 7)) * LDS + (lane >> 3) * 8));
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t af[2][4];
#pragma unroll
                for (int ks = 0; ks < 2; ++ks)
                    ldsm_x4(af[ks], smem_u32(sA(buf, pa) + (wm * 64 + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + ks * 16 + (lane >> 4) * 8));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    mma16816(acc[i][j], af[0], bf[j][0], bf[j][1]);
                    mma16816(acc[i][j], af[1], bf[j][2], bf[j][3]);
                }
            }
        }
        if (kt + 1 < nk) sstore(buf ^ 1);
        __syncthreads();
    }
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int r = m0 + wm * 64 + i * 16 + g + rr * 8;
            if (r >= p.m) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = n0 + wn * 32 + j * 8 + 2 * t;
                if (c >= p.N) continue;
                float v0 = acc[i][j][rr * 2], v1 = acc[i][j][rr * 2 + 1];
                const size_t off = size_t(r) * p.N + c;
                if (c + 1 < p.N && !(p.N & 1)) {
                    if (p.resid) { float2 rs = *reinterpret_cast<const float2*>(p.resid + off); v0 += rs.x; v1 += rs.y; }
                    *reinterpret_cast<float2*>(p.out + off) = make_float2(v0, v1);
                } else {
                    p.out[off] = p.resid ? p.resid[off] + v0 : v0;
                    if (c + 1 < p.N) p.out[off + 1] = p.resid ? p.resid[off + 1] + v1 : v1;
                }
            }
        }
    }
}

}  // namespace

// mma.sync tile kernel: the path for K that is not a multiple of 64, and the cross-check for the tcgen05 kernel
int32_t gemm_f16a_mma(float* out, const __half* A, const __half* Alo, const QWeight& w, int m, const float* resid, cudaStream_t st) {
    if (m <= 0) return FORGE_OK;
    if (w.K % 32) { set_error("gemm: K=%d must be a multiple of 32", w.K); return FORGE_ERR_SHAPE; }
    GemmParams p{out, A, Alo, w.qs, w.d, resid, m, w.N, w.K};
    dim3 grid((w.N + BN - 1) / BN, (m + BM - 1) / BM);
    const bool split = Alo != nullptr;
    const size_t smem = size_t(2) * (split ? 2 : 1) * (BM + BN) * LDS * sizeof(__half);
#define FORGE_GEMM_LAUNCH(Q, S)                                                                                   \
    do {                                                                                                          \
        FORGE_CUDA(cudaFuncSetAttribute(gemm_kernel<Q, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))); \
        gemm_kernel<Q, S><<<grid, kThreads, smem, st>>>(p);                                                       \
    } while (0)
    if (w.quant == FORGE_Q8_0) { if (split) FORGE_GEMM_LAUNCH(FORGE_Q8_0, true); else FORGE_GEMM_LAUNCH(FORGE_Q8_0, false); }
    else { if (split) FORGE_GEMM_LAUNCH(FORGE_Q4_0, true); else FORGE_GEMM_LAUNCH(FORGE_Q4_0, false); }
#undef FORGE_GEMM_LAUNCH
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

int32_t gemm_f16a(float* out, const __half* A, const __half* Alo, const QWeight& w, int m, const float* resid, int* err, cudaStream_t st) {
    if (w.quant == FORGE_KQ_SOA) {  // K-quant rows exist in the tcgen05 kernel only (K is a multiple of 256 there)
        if (!gemm_tc5_supported(w)) { set_error("gemm: K-quant rows need K to be a multiple of 64"); return FORGE_ERR_SHAPE; }
        return gemm_tc5(out, A, Alo, w, m, resid, err, st);
    }
    if (gemm_tc5_supported(w)) return gemm_tc5(out, A, Alo, w, m, resid, err, st);
    return gemm_f16a_mma(out, A, Alo, w, m, resid, st);
}

}  // namespace forge
