// Prefill attention on tensor cores over the paged fp16 KV cache (replaces
// attention_flash_batch, crates/forgellm-codegen-cpu/src/emit.rs:755-883): query row r sits at
// position base_pos + r and sees cache positions <= its own (:815-818); K/V tiles stop at the
// tile's last query (:782, :792-793); GQA mapping kv_head = h / (nq/nkv) (:763, :775).
// One CTA = 64 query rows of one head (16 per warp); K/V stream in 64-key tiles (one KV page);
// S = Q K^T and O += P V are m16n8k16 fp16 MMAs with f32 accumulators.  The softmax state is f32 in the base-2
// domain (scores are scaled by scale * log2(e) once, probabilities are ex2 of the difference: the hardware
// exponential, relative error ~2^-22, far below the fp16 rounding of P); the causal mask is applied only on tiles
// that reach past a query's position.  K/V tiles are double-buffered with cp.async; CTAs with the most key tiles
// (the last query tiles) are scheduled first.
#include "common.cuh"

namespace forge {

namespace {

constexpr int BM = 64, BN = 64, kThreads = 128;

struct PrefillParams {
    AttnPrefillArgs a;
    const float* q32;
    float scale;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 16-byte global -> shared copy that bypasses registers; src_bytes = 0 writes zeros
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t pack_h2_lo(float a, float b, uint32_t hi) {  // what pack_h2 dropped
    const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    return pack_h2(a - hf.x, b - hf.y);
}

// SW: sliding-window instantiation (the full-attention one carries no window tests)
// PRECISE: Q and P enter the MMAs as fp16 hi + lo pairs (S = Q_hi K + Q_lo K, O += P_hi V + P_lo V); K and V are the
// cache's fp16 values either way, so the result is the f32 attention over those values to ~1e-6
template <int HD, bool SW, bool PRECISE>
__global__ void __launch_bounds__(kThreads) attn_prefill_kernel(PrefillParams p) {
    constexpr int LD = HD + 8;       // padded row (halfs): keeps ldmatrix rows on distinct banks
    constexpr int CH = HD / 8;       // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sQ = reinterpret_cast<__half*>(smem_raw);
    __half* sKV = sQ + BM * LD;  // [2 buffers][K | V][BN][LD]
    __half* sQlo = sKV + 4 * BN * LD;  // PRECISE only
    const AttnPrefillArgs& a = p.a;
    const int qt = int(gridDim.x) - 1 - int(blockIdx.x), h = blockIdx.y;  // longest CTAs first
    const int G = a.nq / a.nkv, kvh = h / G, kvd = a.nkv * HD;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int row0 = qt * BM;
    const size_t qstride = size_t(a.nq) * HD;

    for (int idx = tid; idx < BM * CH; idx += kThreads) {
        int r = idx / CH, c = idx % CH, qr = row0 + r;
        uint4 v = make_uint4(0, 0, 0, 0), vl = make_uint4(0, 0, 0, 0);
        if (qr < a.m) {
            if (p.q32) {
                const float4* s = reinterpret_cast<const float4*>(p.q32 + qr * qstride + h * HD + c * 8);
                float4 x0 = s[0], x1 = s[1];
                v.x = pack_h2(x0.x, x0.y); v.y = pack_h2(x0.z, x0.w); v.z = pack_h2(x1.x, x1.y); v.w = pack_h2(x1.z, x1.w);
                if (PRECISE) {
                    vl.x = pack_h2_lo(x0.x, x0.y, v.x); vl.y = pack_h2_lo(x0.z, x0.w, v.y);
                    vl.z = pack_h2_lo(x1.x, x1.y, v.z); vl.w = pack_h2_lo(x1.z, x1.w, v.w);
                }
            } else {
                v = *reinterpret_cast<const uint4*>(a.q16 + qr * qstride + h * HD + c * 8);
                if (PRECISE && a.q16_lo) vl = *reinterpret_cast<const uint4*>(a.q16_lo + qr * qstride + h * HD + c * 8);
            }
        }
        *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
        if (PRECISE) *reinterpret_cast<uint4*>(sQlo + r * LD + c * 8) = vl;
    }
    __syncthreads();
    uint32_t qf[HD / 16][4];
    uint32_t qfl[PRECISE ? HD / 16 : 1][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        ldsm_x4(qf[ks], smem_u32(sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8));
        if (PRECISE) ldsm_x4(qfl[PRECISE ? ks : 0], smem_u32(sQlo + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8));
    }

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

    const int q_hi = min(a.m, row0 + BM) - 1;
    const int n_keys = a.base_pos + q_hi + 1;
    const int ntiles = (n_keys + BN - 1) / BN;
    const int qpos0 = a.base_pos + row0 + warp * 16 + g;  // position of this thread's first row

    auto load_tile = [&](int j, int buf) {
        const int page = a.page_row ? a.page_row[j] : j;
        __half* dK = sKV + size_t(buf) * 2 * BN * LD;
        __half* dV = dK + BN * LD;
        for (int idx = tid; idx < BN * CH; idx += kThreads) {
            const int r = idx / CH, c = idx % CH;
            const bool in = j * BN + r < n_keys;
            const size_t off = (size_t(page) * FORGE_KV_PAGE + (in ? r : 0)) * kvd + kvh * HD + c * 8;
            cp_async16(dK + r * LD + c * 8, a.k_pool + off, in ? 16 : 0);
            cp_async16(dV + r * LD + c * 8, a.v_pool + off, in ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const float sl2 = p.scale * 1.4426950408889634f;  // scores in the base-2 domain
    // sliding window: the first query of the tile sees keys from (its position - window + 1); earlier tiles are skipped
    const int k_first = SW ? max(a.base_pos + row0 - (a.window - 1), 0) : 0;
    const int j0 = k_first / BN;
    load_tile(j0, j0 & 1);
    for (int j = j0; j < ntiles; ++j) {
        if (j + 1 < ntiles) {
            load_tile(j + 1, (j + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __half* sK = sKV + size_t(j & 1) * 2 * BN * LD;
        const __half* sV = sK + BN * LD;

        float s[BN / 8][4];
#pragma unroll
        for (int nb = 0; nb < BN / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks += 2) {
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
                uint32_t r[4];
                ldsm_x4(r, smem_u32(sK + (nb * 8 + (lane & 7)) * LD + ks * 16 + (lane >> 3) * 8));
                mma16816(s[nb], qf[ks], r[0], r[1]);
                mma16816(s[nb], qf[ks + 1], r[2], r[3]);
                if (PRECISE) {
                    mma16816(s[nb], qfl[PRECISE ? ks : 0], r[0], r[1]);
                    mma16816(s[nb], qfl[PRECISE ? ks + 1 : 0], r[2], r[3]);
                }
            }
        }
        // scale, causal mask (only where the tile reaches past the row), online softmax in base 2
        // (rows g and g+8 of the warp's 16)
        // some key of the tile may be masked for this warp: past a query's position, or before its window
        const bool diag = j * BN + BN - 1 > a.base_pos + row0 + warp * 16 ||
                          (SW && j * BN < a.base_pos + row0 + warp * 16 + 15 - (a.window - 1));
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int qpos = qpos0 + rr * 8;
            float mx = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float v = s[nb][rr * 2 + e] * sl2;
                    const int key = j * BN + nb * 8 + 2 * t + e;
                    if (diag && (key > qpos || (SW && key < qpos - (a.window - 1)))) v = -INFINITY;
                    s[nb][rr * 2 + e] = v;
                    mx = fmaxf(mx, v);
                }
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(mrow[rr], mx);
            const float msub = (mn == -INFINITY) ? 0.f : mn;  // a fully masked row keeps exponent arguments finite
            const float es = ex2(mrow[rr] - msub);            // ex2(-inf) = 0
            float ls = 0.f;
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pr = ex2(s[nb][rr * 2 + e] - msub);
                    s[nb][rr * 2 + e] = pr;
                    ls += pr;
                }
            }
            lrow[rr] = lrow[rr] * es + ls;
            mrow[rr] = mn;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) { o[i][rr * 2] *= es; o[i][rr * 2 + 1] *= es; }
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_h2(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_h2(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            uint32_t pl[4] = {0u, 0u, 0u, 0u};
            if (PRECISE) {
                pl[0] = pack_h2_lo(s[2 * kk][0], s[2 * kk][1], pa[0]);
                pl[1] = pack_h2_lo(s[2 * kk][2], s[2 * kk][3], pa[1]);
                pl[2] = pack_h2_lo(s[2 * kk + 1][0], s[2 * kk + 1][1], pa[2]);
                pl[3] = pack_h2_lo(s[2 * kk + 1][2], s[2 * kk + 1][3], pa[3]);
            }
#pragma unroll
            for (int nb2 = 0; nb2 < HD / 16; ++nb2) {
                uint32_t r[4];
                ldsm_x4_t(r, smem_u32(sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + nb2 * 16 + (lane >> 4) * 8));
                mma16816(o[2 * nb2], pa, r[0], r[1]);
                mma16816(o[2 * nb2 + 1], pa, r[2], r[3]);
                if (PRECISE) {
                    mma16816(o[2 * nb2], pl, r[0], r[1]);
                    mma16816(o[2 * nb2 + 1], pl, r[2], r[3]);
                }
            }
        }
        __syncthreads();  // the buffer is refilled by the prefetch of the next iteration
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        float l = lrow[rr];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = 1.0f / l;
        const int qr = row0 + warp * 16 + g + rr * 8;
        if (qr < a.m) {
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                float v0 = o[i][rr * 2] * inv, v1 = o[i][rr * 2 + 1] * inv;
                size_t off = qr * qstride + h * HD + i * 8 + 2 * t;
                if (a.out16) {
                    __half2 hv = __floats2half2_rn(v0, v1);
                    *reinterpret_cast<__half2*>(a.out16 + off) = hv;
                    if (a.out16_lo) {
                        float2 hf = __half22float2(hv);
                        *reinterpret_cast<__half2*>(a.out16_lo + off) = __floats2half2_rn(v0 - hf.x, v1 - hf.y);
                    }
                } else {
                    *reinterpret_cast<float2*>(a.out32 + off) = make_float2(v0, v1);
                }
            }
        }
    }
}

template <int HD>
int32_t launch(const PrefillParams& p, cudaStream_t st) {
    const size_t smem = size_t((p.a.precise ? 2 : 1) * BM + 4 * BN) * (HD + 8) * sizeof(__half);
    auto kern = p.a.precise ? (p.a.window > 0 ? attn_prefill_kernel<HD, true, true> : attn_prefill_kernel<HD, false, true>)
                            : (p.a.window > 0 ? attn_prefill_kernel<HD, true, false> : attn_prefill_kernel<HD, false, false>);
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    dim3 grid((p.a.m + BM - 1) / BM, p.a.nq);
    kern<<<grid, kThreads, smem, st>>>(p);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace

int32_t attn_prefill_q32(const AttnPrefillArgs& a, const float* q32, cudaStream_t st) {
    if (a.m <= 0) return FORGE_OK;
    if (a.nq % a.nkv) { set_error("attention: num_heads %d not a multiple of num_kv_heads %d", a.nq, a.nkv); return FORGE_ERR_SHAPE; }
    PrefillParams p{a, q32, 1.0f / sqrtf(float(a.hd))};
    switch (a.hd) {
        case 64: return launch<64>(p, st);
        case 96: return launch<96>(p, st);
        case 128: return launch<128>(p, st);
    }
    set_error("attention: head_dim %d unsupported (64, 96, 128)", a.hd);
    return FORGE_ERR_SHAPE;
}

int32_t attn_prefill(const AttnPrefillArgs& a, cudaStream_t st) { return attn_prefill_q32(a, nullptr, st); }

}  // namespace forge
