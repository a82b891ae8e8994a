// Decode GEMV on packed Q8_0 / Q4_0 weights (replaces matmul_vec_q8_0_KxN / matmul_vec_q4_0_KxN,
// crates/forgellm-codegen-cpu/src/emit.rs:2047-2087 and :2910-2953) with the reference's
// fusion patterns folded in (crates/forgellm-optimizer/src/fusion.rs:12-27):
//   prologue  RMSNorm(x) * w                      (emit.rs:327-334)
//   epilogue  + residual                          (emit.rs:455-459)
//             + bias, RoPE, fp16 KV append        (emit.rs:4108-4153, cache type fp16)
//             silu(gate) * up                     (emit.rs:381-386)
// HBM-bound: every weight byte is read once with 128-bit loads (one uint4 per lane per row),
// dequantised in registers against f32 activations held in shared memory, reduced with warp
// shuffles.  Activations stay f32 and are never quantised (the x86 branch of the reference).
#include "common.cuh"

namespace forge {

namespace {

constexpr int kWarps = 4;
constexpr int kRows = 4;  // rows per warp; even, so RoPE pairs and gate/up pairs stay in one warp

struct GemvParams {
    const uint8_t* qs; const __half* d;
    int K, N, nblk;       // nblk = K/32
    GemvArgs a;
};

template <int QUANT> struct Geo;
template <> struct Geo<FORGE_Q8_0> { static constexpr int C = 16, J = 4; };  // floats per lane-chunk, float4s
template <> struct Geo<FORGE_Q4_0> { static constexpr int C = 32, J = 8; };

// shared-memory slot of activation element e: lane-chunks are interleaved so that the 32
// lanes of a warp read 32 consecutive float4 (no bank conflicts).
template <int QUANT>
__device__ __forceinline__ int xslot(int e) {
    constexpr int C = Geo<QUANT>::C, J = Geo<QUANT>::J;
    int it = e / (32 * C), rem = e % (32 * C);
    int l = rem / C, j = (rem % C) >> 2, c = e & 3;
    return (((it * J + j) << 5) + l) * 4 + c;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float s8(uint32_t w, int i) { return float(int(int8_t(w >> (8 * i)))); }

template <int QUANT, int EPI>
__global__ void __launch_bounds__(kWarps * 32) gemv_kernel(GemvParams p) {
    extern __shared__ float4 xs4[];
    float* xs = reinterpret_cast<float*>(xs4);
    __shared__ float red[kWarps];
    constexpr int C = Geo<QUANT>::C, J = Geo<QUANT>::J;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, N = p.N;
    const int iters = (K + 32 * C - 1) / (32 * C);
    const int ngroups = (N + kWarps * kRows - 1) / (kWarps * kRows);
    const size_t qrow = (QUANT == FORGE_Q8_0) ? size_t(K) : size_t(K) / 2;

    for (int b = 0; b < p.a.batch; ++b) {
        // ---- stage (optionally normalised) activations
        const float* x = p.a.x + size_t(b) * K;
        float inv = 1.0f;
        if (p.a.norm_w) {
            float ss = 0.f;
            for (int e = tid; e < K; e += kWarps * 32) { float v = x[e]; ss += v * v; }
            ss = warp_sum(ss);
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            ss = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) ss += red[w];
            inv = 1.0f / sqrtf(ss / float(K) + p.a.eps);
        }
        __syncthreads();  // previous batch row's readers are done
        for (int e = tid; e < iters * 32 * C; e += kWarps * 32) {
            float v = 0.f;
            if (e < K) {
                v = x[e];
                if (p.a.norm_w) v = v * inv * p.a.norm_w[e];
            }
            xs[xslot<QUANT>(e)] = v;
        }
        __syncthreads();

        for (int g = blockIdx.x; g < ngroups; g += gridDim.x) {
            const int row0 = (g * kWarps + warp) * kRows;
            float acc[kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r) acc[r] = 0.f;
            for (int it = 0; it < iters; ++it) {
                const int e0 = (it * 32 + lane) * C;
                if (e0 >= K) break;
                float4 xv[J];
#pragma unroll
                for (int j = 0; j < J; ++j) xv[j] = xs4[((it * J + j) << 5) + lane];
                uint4 wv[kRows];
                float dv[kRows];
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    int row = row0 + r;
                    if (row < N) {
                        wv[r] = ld_stream(reinterpret_cast<const uint4*>(p.qs + size_t(row) * qrow + (QUANT == FORGE_Q8_0 ? e0 : e0 / 2)));
                        dv[r] = __half2float(p.d[size_t(row) * p.nblk + e0 / 32]);
                    } else {
                        wv[r] = make_uint4(0, 0, 0, 0);
                        dv[r] = 0.f;
                    }
                }
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    const uint32_t w[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
                    float s = 0.f;
                    if (QUANT == FORGE_Q8_0) {
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            s += xv[t].x * s8(w[t], 0);
                            s += xv[t].y * s8(w[t], 1);
                            s += xv[t].z * s8(w[t], 2);
                            s += xv[t].w * s8(w[t], 3);
                        }
                    } else {
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            // byte i of the block = element i (low nibble) and element i+16 (high nibble)
                            s += xv[t].x * float(int(w[t] & 15u) - 8);
                            s += xv[t].y * float(int((w[t] >> 8) & 15u) - 8);
                            s += xv[t].z * float(int((w[t] >> 16) & 15u) - 8);
                            s += xv[t].w * float(int((w[t] >> 24) & 15u) - 8);
                            s += xv[4 + t].x * float(int((w[t] >> 4) & 15u) - 8);
                            s += xv[4 + t].y * float(int((w[t] >> 12) & 15u) - 8);
                            s += xv[4 + t].z * float(int((w[t] >> 20) & 15u) - 8);
                            s += xv[4 + t].w * float(int((w[t] >> 28) & 15u) - 8);
                        }
                    }
                    acc[r] += dv[r] * s;
                }
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r) acc[r] = warp_sum(acc[r]);

            // ---- epilogue: lane r/2 of each pair handles rows (row0+2i, row0+2i+1)
            if (lane < kRows / 2) {
                const int ra = row0 + 2 * lane;
                float v0 = lane == 0 ? acc[0] : acc[2], v1 = lane == 0 ? acc[1] : acc[3];
                if (ra < N) {
                    const bool has1 = (ra + 1) < N;
                    if (EPI == EPI_STORE) {
                        p.a.out[size_t(b) * N + ra] = v0;
                        if (has1) p.a.out[size_t(b) * N + ra + 1] = v1;
                    } else if (EPI == EPI_RESID) {
                        p.a.out[size_t(b) * N + ra] = p.a.resid[size_t(b) * N + ra] + v0;
                        if (has1) p.a.out[size_t(b) * N + ra + 1] = p.a.resid[size_t(b) * N + ra + 1] + v1;
                    } else if (EPI == EPI_SILU) {
                        // rows are interleaved at pack time: 2j = gate_j, 2j+1 = up_j
                        float gt = v0;
                        p.a.out[size_t(b) * (N / 2) + (ra >> 1)] = (gt / (1.0f + expf(-gt))) * v1;
                    } else {  // EPI_QKV
                        if (p.a.bias) { v0 += p.a.bias[ra]; v1 += p.a.bias[ra + 1]; }
                        const int pos = p.a.seq_len[b];
                        const int qk = p.a.qk, kv = p.a.kv, hd = p.a.head_dim;
                        int col = ra;  // column inside q, k or v
                        int region = 0;
                        if (col >= qk) { col -= qk; region = 1; }
                        if (region == 1 && col >= kv) { col -= kv; region = 2; }
                        if (region < 2) {
                            const float2 cs = reinterpret_cast<const float2*>(p.a.rope)[size_t(pos) * (hd / 2) + (col % hd) / 2];
                            float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;
                            v0 = r0; v1 = r1;
                        }
                        if (region == 0) {
                            float2* dst = reinterpret_cast<float2*>(p.a.q_out + size_t(b) * qk + col);
                            *dst = make_float2(v0, v1);
                        } else {
                            const int page = p.a.page_table[size_t(b) * p.a.pages_per_seq + pos / FORGE_KV_PAGE];
                            __half* pool = region == 1 ? p.a.k_pool : p.a.v_pool;
                            __half2* dst = reinterpret_cast<__half2*>(pool + (size_t(page) * FORGE_KV_PAGE + pos % FORGE_KV_PAGE) * kv + col);
                            *dst = __floats2half2_rn(v0, v1);
                        }
                    }
                }
            }
        }
    }
}

template <int QUANT>
int32_t launch(const QWeight& w, GemvEpilogue epi, const GemvArgs& a, cudaStream_t st) {
    GemvParams p;
    p.qs = w.qs; p.d = w.d; p.K = w.K; p.N = w.N; p.nblk = w.K / 32; p.a = a;
    constexpr int C = Geo<QUANT>::C;
    int iters = (w.K + 32 * C - 1) / (32 * C);
    size_t smem = size_t(iters) * 32 * C * sizeof(float);
    if (smem > 48 * 1024) { set_error("gemv: K=%d too large for the activation stage", w.K); return FORGE_ERR_SHAPE; }
    int ngroups = (w.N + kWarps * kRows - 1) / (kWarps * kRows);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int grid = ngroups < sms * 8 ? ngroups : sms * 8;
    dim3 blk(kWarps * 32);
    switch (epi) {
        case EPI_STORE: gemv_kernel<QUANT, EPI_STORE><<<grid, blk, smem, st>>>(p); break;
        case EPI_RESID: gemv_kernel<QUANT, EPI_RESID><<<grid, blk, smem, st>>>(p); break;
        case EPI_QKV: gemv_kernel<QUANT, EPI_QKV><<<grid, blk, smem, st>>>(p); break;
        case EPI_SILU: gemv_kernel<QUANT, EPI_SILU><<<grid, blk, smem, st>>>(p); break;
    }
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace

int32_t gemv(const QWeight& w, GemvEpilogue epi, const GemvArgs& a, cudaStream_t st) {
    if (w.K % 32 != 0 || w.K <= 0 || w.N <= 0) { set_error("gemv: K=%d must be a positive multiple of 32", w.K); return FORGE_ERR_SHAPE; }
    if ((epi == EPI_SILU || epi == EPI_QKV) && (w.N % 2)) { set_error("gemv: paired epilogue needs even N"); return FORGE_ERR_SHAPE; }
    return w.quant == FORGE_Q8_0 ? launch<FORGE_Q8_0>(w, epi, a, st) : launch<FORGE_Q4_0>(w, epi, a, st);
}

}  // namespace forge
