// Row-wise and elementwise operators of the forward path and the prefill glue kernels.
// Reference statements (crates/forgellm-codegen-cpu/src/emit.rs): rms_norm :327-334,
// rope :509-528, silu_mul :381-386, residual_add :455-459, embedding :586-589, bias adds
// :4108-4118, cache write :4136-4153 (fp16 here instead of int8), argmax project.rs:501-503.
#include "common.cuh"

namespace forge {

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < nw; ++w) s += red[w];
    return s;
}

// one CTA per row: out = x * (1/sqrt(mean(x^2)+eps)) * w
__device__ __forceinline__ void store_split(__half* hi, __half* lo, size_t i, float v) {
    __half h = __float2half_rn(v);
    hi[i] = h;
    if (lo) lo[i] = __float2half_rn(v - __half2float(h));
}

template <typename OutT>
__global__ void rms_norm_kernel(OutT* __restrict__ out, __half* __restrict__ lo, const float* __restrict__ in, const float* __restrict__ w, int n, float eps) {
    __shared__ float red[32];
    const float* x = in + size_t(blockIdx.x) * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { float v = x[i]; ss += v * v; }
    ss = block_sum(ss, red);
    float inv = 1.0f / sqrtf(ss / float(n) + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[i] * inv * w[i];
        if constexpr (sizeof(OutT) == 2) store_split(out, lo, size_t(blockIdx.x) * n + i, v);
        else out[size_t(blockIdx.x) * n + i] = v;
    }
}

// fp16 hi/lo output for rows of at most 256 * 4 * NV floats: the row is read once with 128-bit loads and stays in
// registers between the sum of squares and the scaling
template <int NV>
__global__ void __launch_bounds__(256) rms_norm_f16_vec_kernel(__half* __restrict__ out, __half* __restrict__ lo, const float* __restrict__ in,
                                                                const float* __restrict__ w, int n, float eps) {
    __shared__ float red[32];
    const float* x = in + size_t(blockIdx.x) * n;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = (threadIdx.x + i * 256) * 4;
        v[i] = e < n ? *reinterpret_cast<const float4*>(x + e) : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / float(n) + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = (threadIdx.x + i * 256) * 4;
        if (e >= n) continue;
        const float4 ww = *reinterpret_cast<const float4*>(w + e);
        const float r[4] = {v[i].x * inv * ww.x, v[i].y * inv * ww.y, v[i].z * inv * ww.z, v[i].w * inv * ww.w};
        const __half2 h0 = __floats2half2_rn(r[0], r[1]), h1 = __floats2half2_rn(r[2], r[3]);
        const size_t o = size_t(blockIdx.x) * n + e;
        *reinterpret_cast<uint2*>(out + o) = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        if (lo) {
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
            const __half2 l0 = __floats2half2_rn(r[0] - f0.x, r[1] - f0.y), l1 = __floats2half2_rn(r[2] - f1.x, r[3] - f1.y);
            *reinterpret_cast<uint2*>(lo + o) = make_uint2(*reinterpret_cast<const uint32_t*>(&l0), *reinterpret_cast<const uint32_t*>(&l1));
        }
    }
}

// residual_add (emit.rs:455-459) of a product that arrives as K-slice partials, fused with the rms_norm (emit.rs:327-334)
// of the next operator: hidden += part_0 + part_1 + ... in slice order, the row stays in registers for the normalisation
template <int NV>
__global__ void __launch_bounds__(256) add_parts_norm_kernel(float* __restrict__ hidden, const float* __restrict__ parts, int nparts, size_t pstride,
                                                              __half* __restrict__ out, __half* __restrict__ lo, const float* __restrict__ w, int n, float eps) {
    __shared__ float red[32];
    float* x = hidden + size_t(blockIdx.x) * n;
    const float* pr = parts + size_t(blockIdx.x) * n;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = (threadIdx.x + i * 256) * 4;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < n) {
            // all loads first (one memory round trip), then the sum in slice order
            v[i] = *reinterpret_cast<const float4*>(x + e);
            float4 a[4];
#pragma unroll
            for (int s = 0; s < 4; ++s)
                a[s] = s < nparts ? *reinterpret_cast<const float4*>(pr + size_t(s) * pstride + e) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < 4; ++s) { v[i].x += a[s].x; v[i].y += a[s].y; v[i].z += a[s].z; v[i].w += a[s].w; }
            *reinterpret_cast<float4*>(x + e) = v[i];
        }
        ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    if (!w) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / float(n) + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = (threadIdx.x + i * 256) * 4;
        if (e >= n) continue;
        const float4 ww = *reinterpret_cast<const float4*>(w + e);
        const float r[4] = {v[i].x * inv * ww.x, v[i].y * inv * ww.y, v[i].z * inv * ww.z, v[i].w * inv * ww.w};
        const __half2 h0 = __floats2half2_rn(r[0], r[1]), h1 = __floats2half2_rn(r[2], r[3]);
        const size_t o = size_t(blockIdx.x) * n + e;
        *reinterpret_cast<uint2*>(out + o) = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        if (lo) {
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
            const __half2 l0 = __floats2half2_rn(r[0] - f0.x, r[1] - f0.y), l1 = __floats2half2_rn(r[2] - f1.x, r[3] - f1.y);
            *reinterpret_cast<uint2*>(lo + o) = make_uint2(*reinterpret_cast<const uint32_t*>(&l0), *reinterpret_cast<const uint32_t*>(&l1));
        }
    }
}

// thread per (row, head, pair): adjacent-pair rotation, table = {cos, sin}[pos][hd/2]
__global__ void rope_kernel(float* data, int rows, int base_pos, int hd, int heads, const float2* __restrict__ table) {
    int half = hd / 2;
    long total = long(rows) * heads * half;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        int pr = int(i % half);
        long rh = i / half;
        int r = int(rh / heads);
        float2 cs = table[size_t(base_pos + r) * half + pr];
        float2* p = reinterpret_cast<float2*>(data) + rh * half + pr;
        float2 v = *p;
        *p = make_float2(v.x * cs.x - v.y * cs.y, v.x * cs.y + v.y * cs.x);
    }
}

__global__ void silu_mul_kernel(float* out, const float* g, const float* u, size_t n) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
        float x = g[i];
        out[i] = (x / (1.0f + expf(-x))) * u[i];
    }
}

// gu: [rows][2*ffn] with gate_j at column 2j and up_j at 2j+1  ->  out f16 [rows][ffn]
__global__ void silu_mul_f16_kernel(__half* out, __half* lo, const float2* gu, size_t n) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
        float2 v = gu[i];
        store_split(out, lo, i, (v.x / (1.0f + expf(-v.x))) * v.y);
    }
}

__global__ void residual_add_kernel(float* a, const float* b, size_t n) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) a[i] += b[i];
}

__global__ void embedding_kernel(float* out, const float* table, const uint32_t* tokens, int h, uint32_t* hist, const int32_t* step) {
    if (hist && threadIdx.x == 0) hist[size_t(*step) * gridDim.x + blockIdx.x] = tokens[blockIdx.x];
    const float4* src = reinterpret_cast<const float4*>(table + size_t(tokens[blockIdx.x]) * h);
    float4* dst = reinterpret_cast<float4*>(out + size_t(blockIdx.x) * h);
    for (int i = threadIdx.x; i < h / 4; i += blockDim.x) dst[i] = src[i];
}

__global__ void kv_append_contig_kernel(__half* kc, __half* vc, const float* k, const float* v, size_t n, size_t off) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
        kc[off + i] = __float2half_rn(k[i]);
        vc[off + i] = __float2half_rn(v[i]);
    }
}

// prefill glue: fused [q;k;v] f32 rows -> (+bias) -> RoPE on q,k -> q fp16, k/v into the paged cache
// (the product may arrive as `nparts` K-slice partials, pstride floats apart: they are added in slice order)
__global__ void qkv_post_kernel(const float* __restrict__ qkv, int nparts, size_t pstride, int m, int base_pos, const float* __restrict__ bias,
                                const float2* __restrict__ rope, __half* __restrict__ q16, __half* __restrict__ q16_lo, __half* __restrict__ k_pool,
                                __half* __restrict__ v_pool, const int32_t* __restrict__ page_row, int qk, int kv, int hd) {
    const int npairs = (qk + 2 * kv) / 2;
    const int r = blockIdx.x;
    const int pos = base_pos + r;
    const float2* src = reinterpret_cast<const float2*>(qkv + size_t(r) * (qk + 2 * kv));
    const int lp = pos / FORGE_KV_PAGE;
    const size_t prow = (size_t(page_row ? page_row[lp] : lp) * FORGE_KV_PAGE + pos % FORGE_KV_PAGE) * kv;
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        float2 v = src[i];
        for (int s = 1; s < nparts; ++s) {
            const float2 a = reinterpret_cast<const float2*>(qkv + size_t(s) * pstride + size_t(r) * (qk + 2 * kv))[i];
            v.x += a.x; v.y += a.y;
        }
        int col = 2 * i;
        if (bias) { v.x += bias[col]; v.y += bias[col + 1]; }
        int region = 0;
        if (col >= qk) { col -= qk; region = 1; }
        if (region == 1 && col >= kv) { col -= kv; region = 2; }
        if (region < 2) {
            float2 cs = rope[size_t(pos) * (hd / 2) + (col % hd) / 2];
            v = make_float2(v.x * cs.x - v.y * cs.y, v.x * cs.y + v.y * cs.x);
        }
        __half2 hv = __floats2half2_rn(v.x, v.y);
        if (region == 0) {
            *reinterpret_cast<__half2*>(q16 + size_t(r) * qk + col) = hv;
            if (q16_lo) {  // the part of the query fp16 drops, for the precise attention
                const float2 hf = __half22float2(hv);
                *reinterpret_cast<__half2*>(q16_lo + size_t(r) * qk + col) = __floats2half2_rn(v.x - hf.x, v.y - hf.y);
            }
        } else *reinterpret_cast<__half2*>((region == 1 ? k_pool : v_pool) + prow + col) = hv;
    }
}

// batched decode glue: row b of the fused [q;k;v] product belongs to sequence b at position seq_len[b]:
// (+bias) -> RoPE on q,k -> q f32 [b][qk], k/v into that sequence's cache page
__global__ void qkv_post_rows_kernel(const float* __restrict__ qkv, int nparts, size_t pstride, const float* __restrict__ bias, const float2* __restrict__ rope,
                                     float* __restrict__ q_out, __half* __restrict__ k_pool, __half* __restrict__ v_pool,
                                     const int32_t* __restrict__ page_table, const int32_t* __restrict__ seq_len, int pages_per_seq,
                                     int qk, int kv, int hd) {
    const int npairs = (qk + 2 * kv) / 2;
    const int b = blockIdx.x;
    const int pos = seq_len[b];
    const float2* src = reinterpret_cast<const float2*>(qkv + size_t(b) * (qk + 2 * kv));
    const size_t prow = (size_t(page_table[size_t(b) * pages_per_seq + pos / FORGE_KV_PAGE]) * FORGE_KV_PAGE + pos % FORGE_KV_PAGE) * kv;
    // one pair per thread: blockIdx.y walks the row in pieces of blockDim.x pairs (a few rows must not mean a few CTAs)
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < npairs; i += gridDim.y * blockDim.x) {
        float2 v = src[i];
        {   // further K-slice partials of the product (pstride floats apart), added in slice order; loads first
            float2 a[3];
#pragma unroll
            for (int s = 0; s < 3; ++s) a[s] = s + 1 < nparts ? *reinterpret_cast<const float2*>(qkv + size_t(s + 1) * pstride + size_t(b) * (qk + 2 * kv) + 2 * i) : make_float2(0.f, 0.f);
#pragma unroll
            for (int s = 0; s < 3; ++s) { v.x += a[s].x; v.y += a[s].y; }
        }
        int col = 2 * i;
        if (bias) { v.x += bias[col]; v.y += bias[col + 1]; }
        int region = 0;
        if (col >= qk) { col -= qk; region = 1; }
        if (region == 1 && col >= kv) { col -= kv; region = 2; }
        if (region < 2) {
            const float2 cs = rope[size_t(pos) * (hd / 2) + (col % hd) / 2];
            v = make_float2(v.x * cs.x - v.y * cs.y, v.x * cs.y + v.y * cs.x);
        }
        if (region == 0) *reinterpret_cast<float2*>(q_out + size_t(b) * qk + col) = v;
        else *reinterpret_cast<__half2*>((region == 1 ? k_pool : v_pool) + prow + col) = __floats2half2_rn(v.x, v.y);
    }
}

// Greedy pick with the generated main's tie rule: the LAST index among equal maxima.
__global__ void argmax_kernel(uint32_t* result, const float* logits, int n) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* x = logits + size_t(blockIdx.x) * n;
    float best = -INFINITY;
    int idx = -1;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[i];
        if (idx < 0 || v > best || (v == best && i > idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi > idx))) { best = ov; idx = oi; }
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < nw; ++w)
            if (bi[w] >= 0 && (idx < 0 || bv[w] > best || (bv[w] == best && bi[w] > idx))) { best = bv[w]; idx = bi[w]; }
        result[blockIdx.x] = uint32_t(idx < 0 ? 0 : idx);
    }
}

// Two-stage variant for large vocabularies: every CTA scans a slice, the last CTA to finish (atomic
// ticket) reduces the per-CTA winners with the same tie rule.  scratch: [batch][gridDim.x] pairs.
__global__ void argmax_slices_kernel(uint32_t* result, const float* logits, int n, float* sval, int* sidx, int* ticket) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    __shared__ int s_last;
    const int b = blockIdx.y, nb = gridDim.x;
    const float* x = logits + size_t(b) * n;
    const int per = (n + nb - 1) / nb, lo = blockIdx.x * per, hi = min(n, lo + per);
    float best = -INFINITY;
    int idx = -1;
    auto better = [](float v, int i, float bv_, int bi_) { return i >= 0 && (bi_ < 0 || v > bv_ || (v == bv_ && i > bi_)); };
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float v = x[i];
        if (better(v, i, best, idx)) { best = v; idx = i; }
    }
    auto block_reduce = [&]() {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
        }
        int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
        __syncthreads();
        if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
        __syncthreads();
        if (threadIdx.x == 0)
            for (int w = 1; w < nw; ++w)
                if (better(bv[w], bi[w], best, idx)) { best = bv[w]; idx = bi[w]; }
    };
    block_reduce();
    if (threadIdx.x == 0) {
        sval[b * nb + blockIdx.x] = best;
        sidx[b * nb + blockIdx.x] = idx;
        __threadfence();
        int old = atomicAdd(ticket + b, 1);
        s_last = (old == nb - 1);
        if (s_last) ticket[b] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    best = -INFINITY;
    idx = -1;
    for (int i = threadIdx.x; i < nb; i += blockDim.x) {
        float v = __ldcg(sval + b * nb + i);
        int vi = __ldcg(sidx + b * nb + i);
        if (better(v, vi, best, idx)) { best = v; idx = vi; }
    }
    block_reduce();
    if (threadIdx.x == 0) result[b] = uint32_t(idx < 0 ? 0 : idx);
}

__global__ void f32_to_f16_kernel(__half* out, __half* lo, const float* in, size_t n) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) store_split(out, lo, i, in[i]);
}

// -log p(target) of one logits row: log_z = max + ln(sum exp((l - max) as f64)) as the reference's corpus scorer forms it
// (crates/forgellm-codegen-cpu/src/project.rs:684-689); one CTA, f64 tree sums
__global__ void __launch_bounds__(1024) token_nll_kernel(double* out, const float* __restrict__ logits, int n, uint32_t target) {
    __shared__ float smax[32];
    __shared__ double ssum[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, logits[i]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) smax[warp] = mx;
    __syncthreads();
    mx = smax[0];
    for (int w = 1; w < int(blockDim.x >> 5); ++w) mx = fmaxf(mx, smax[w]);
    double s = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += exp(double(logits[i] - mx));
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) ssum[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int w = 0; w < int(blockDim.x >> 5); ++w) tot += ssum[w];
        *out = -(double(logits[target]) - (double(mx) + log(tot)));
    }
}

__global__ void step_advance_kernel(int32_t* seq_len, int batch, int32_t* step, uint32_t* extra_counter) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < batch) seq_len[i] += 1;
    if (i == 0 && step) *step += 1;
    if (i == 0 && extra_counter) *extra_counter += 1;
}

__global__ void gather_rows_kernel(float* out, const __half* pool, const int32_t* page_row, int len, int kvd) {
    size_t n = size_t(len) * kvd;
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
        int t = int(i / kvd), c = int(i % kvd);
        int lp = t / FORGE_KV_PAGE;
        out[i] = __half2float(pool[(size_t(page_row ? page_row[lp] : lp) * FORGE_KV_PAGE + t % FORGE_KV_PAGE) * kvd + c]);
    }
}

inline int grid_for(size_t n, int threads = 256) {
    size_t g = (n + threads - 1) / threads;
    return int(g < 148 * 32 ? (g ? g : 1) : 148 * 32);
}

}  // namespace

int32_t rms_norm_f32(float* out, const float* in, const float* w, int rows, int n, float eps, cudaStream_t st) {
    if (rows <= 0) return FORGE_OK;
    rms_norm_kernel<float><<<rows, 256, 0, st>>>(out, nullptr, in, w, n, eps);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t rms_norm_f16(__half* out, __half* lo, const float* in, const float* w, int rows, int n, float eps, cudaStream_t st) {
    if (rows <= 0) return FORGE_OK;
    if (n % 4 == 0 && n <= 2048) rms_norm_f16_vec_kernel<2><<<rows, 256, 0, st>>>(out, lo, in, w, n, eps);
    else if (n % 4 == 0 && n <= 4096) rms_norm_f16_vec_kernel<4><<<rows, 256, 0, st>>>(out, lo, in, w, n, eps);
    else if (n % 4 == 0 && n <= 8192) rms_norm_f16_vec_kernel<8><<<rows, 256, 0, st>>>(out, lo, in, w, n, eps);
    else rms_norm_kernel<__half><<<rows, 256, 0, st>>>(out, lo, in, w, n, eps);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t add_parts_rms_norm_f16(float* hidden, const float* parts, int nparts, size_t pstride, __half* out, __half* lo, const float* w,
                               int rows, int n, float eps, cudaStream_t st) {
    if (rows <= 0) return FORGE_OK;
    if (n % 4 || n > 8192 || nparts < 1 || nparts > 4) { set_error("add_parts_rms_norm: row length %d / %d slices unsupported", n, nparts); return FORGE_ERR_SHAPE; }
    if (n <= 2048) add_parts_norm_kernel<2><<<rows, 256, 0, st>>>(hidden, parts, nparts, pstride, out, lo, w, n, eps);
    else if (n <= 4096) add_parts_norm_kernel<4><<<rows, 256, 0, st>>>(hidden, parts, nparts, pstride, out, lo, w, n, eps);
    else add_parts_norm_kernel<8><<<rows, 256, 0, st>>>(hidden, parts, nparts, pstride, out, lo, w, n, eps);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t rope_rows(float* data, int rows, int base_pos, int head_dim, int heads, const float* table, cudaStream_t st) {
    size_t n = size_t(rows) * heads * (head_dim / 2);
    if (n == 0) return FORGE_OK;
    rope_kernel<<<grid_for(n), 256, 0, st>>>(data, rows, base_pos, head_dim, heads, reinterpret_cast<const float2*>(table));
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t silu_mul_f32(float* out, const float* g, const float* u, size_t n, cudaStream_t st) {
    if (n == 0) return FORGE_OK;
    silu_mul_kernel<<<grid_for(n), 256, 0, st>>>(out, g, u, n);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t silu_mul_f16(__half* out, __half* lo, const float* gu, int rows, int ffn, cudaStream_t st) {
    size_t n = size_t(rows) * ffn;
    if (n == 0) return FORGE_OK;
    silu_mul_f16_kernel<<<grid_for(n), 256, 0, st>>>(out, lo, reinterpret_cast<const float2*>(gu), n);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t residual_add_f32(float* a, const float* b, size_t n, cudaStream_t st) {
    if (n == 0) return FORGE_OK;
    residual_add_kernel<<<grid_for(n), 256, 0, st>>>(a, b, n);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t embedding_rows(float* out, const float* table, const uint32_t* tokens, int rows, int h, uint32_t* hist, const int32_t* step, cudaStream_t st) {
    if (rows <= 0) return FORGE_OK;
    embedding_kernel<<<rows, 128, 0, st>>>(out, table, tokens, h, hist, step);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t kv_append_contig(__half* kc, __half* vc, const float* k, const float* v, int rows, int base_pos, int kvd, cudaStream_t st) {
    size_t n = size_t(rows) * kvd;
    if (n == 0) return FORGE_OK;
    kv_append_contig_kernel<<<grid_for(n), 256, 0, st>>>(kc, vc, k, v, n, size_t(base_pos) * kvd);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t qkv_post(const float* qkv, int m, int base_pos, const float* bias, const float* rope, __half* q16, __half* q16_lo,
                 __half* k_pool, __half* v_pool, const int32_t* page_row, int qk, int kv, int hd, cudaStream_t st, int nparts, size_t pstride) {
    if (m <= 0) return FORGE_OK;
    qkv_post_kernel<<<m, 256, 0, st>>>(qkv, nparts, pstride, m, base_pos, bias, reinterpret_cast<const float2*>(rope), q16, q16_lo, k_pool, v_pool, page_row, qk, kv, hd);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t qkv_post_rows(const float* qkv, int batch, const float* bias, const float* rope, float* q_out, __half* k_pool, __half* v_pool,
                      const int32_t* page_table, const int32_t* seq_len, int pages_per_seq, int qk, int kv, int hd, cudaStream_t st, int nparts,
                      size_t pstride) {
    if (batch <= 0) return FORGE_OK;
    const int npairs = (qk + 2 * kv) / 2;
    if (nparts < 1 || nparts > 4) { set_error("qkv_post_rows: %d slices unsupported", nparts); return FORGE_ERR_INVALID_ARG; }
    qkv_post_rows_kernel<<<dim3(batch, (npairs + 255) / 256), 256, 0, st>>>(qkv, nparts, pstride, bias, reinterpret_cast<const float2*>(rope), q_out, k_pool, v_pool, page_table, seq_len,
                                                pages_per_seq, qk, kv, hd);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t argmax_last(uint32_t* result, const float* logits, int n, int batch, cudaStream_t st) {
    argmax_kernel<<<batch, 1024, 0, st>>>(result, logits, n);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t argmax_slices(uint32_t* result, const float* logits, int n, int batch, float* sval, int* sidx, int* ticket, cudaStream_t st) {
    dim3 grid(kArgmaxSlices, batch);
    argmax_slices_kernel<<<grid, 256, 0, st>>>(result, logits, n, sval, sidx, ticket);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
// four threads per 32-value block, eight values each; whole warps stay in the loop (shuffles)
__global__ void q8_round_f16_kernel(__half* __restrict__ hi, __half* __restrict__ lo, size_t groups) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < ((groups + 31) & ~size_t(31)); i += size_t(gridDim.x) * blockDim.x) {
        const bool on = i < groups;
        float x[8];
        uint4 h = make_uint4(0, 0, 0, 0), l = make_uint4(0, 0, 0, 0);
        if (on) { h = reinterpret_cast<const uint4*>(hi)[i]; if (lo) l = reinterpret_cast<const uint4*>(lo)[i]; }
        const __half2* hp = reinterpret_cast<const __half2*>(&h);
        const __half2* lp = reinterpret_cast<const __half2*>(&l);
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 a = __half22float2(hp[j]), b = __half22float2(lp[j]);
            x[2 * j] = a.x + b.x; x[2 * j + 1] = a.y + b.y;
            amax = fmaxf(amax, fmaxf(fabsf(x[2 * j]), fabsf(x[2 * j + 1])));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        float bs = 1.0f, binv = 0.0f;
        if (amax != 0.f) { bs = __fdiv_rn(amax, 127.0f); binv = __fdiv_rn(1.0f, bs); }
        const float s16 = bs < 5.9604644775390625e-8f ? 0.f : __half2float(__float2half_rn(bs));  // the reference's f16 conversion flushes below 2^-24
        uint4 oh, ol;
        __half2* ohp = reinterpret_cast<__half2*>(&oh);
        __half2* olp = reinterpret_cast<__half2*>(&ol);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float v0 = s16 * fminf(127.f, fmaxf(-127.f, roundf(x[2 * j] * binv)));
            const float v1 = s16 * fminf(127.f, fmaxf(-127.f, roundf(x[2 * j + 1] * binv)));
            ohp[j] = __floats2half2_rn(v0, v1);
            const float2 hf = __half22float2(ohp[j]);
            olp[j] = __floats2half2_rn(v0 - hf.x, v1 - hf.y);
        }
        if (on) { reinterpret_cast<uint4*>(hi)[i] = oh; if (lo) reinterpret_cast<uint4*>(lo)[i] = ol; }
    }
}

int32_t q8_round_f16(__half* hi, __half* lo, size_t n, cudaStream_t st) {
    if (n % 32) { set_error("q8_round_f16: n must be a multiple of 32"); return FORGE_ERR_SHAPE; }
    if (n == 0) return FORGE_OK;
    q8_round_f16_kernel<<<grid_for(n / 8), 256, 0, st>>>(hi, lo, n / 8);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

int32_t f32_to_f16(__half* out, __half* lo, const float* in, size_t n, cudaStream_t st) {
    if (n == 0) return FORGE_OK;
    f32_to_f16_kernel<<<grid_for(n), 256, 0, st>>>(out, lo, in, n);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t token_nll(double* out, const float* logits, int n, uint32_t target, cudaStream_t st) {
    token_nll_kernel<<<1, 1024, 0, st>>>(out, logits, n, target);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t step_advance(int32_t* seq_len, int batch, int32_t* step, cudaStream_t st, uint32_t* extra_counter) {
    step_advance_kernel<<<(batch + 127) / 128, 128, 0, st>>>(seq_len, batch, step, extra_counter);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}
int32_t gather_rows_f16(float* out, const __half* pool, const int32_t* page_row, int len, int kvd, cudaStream_t st) {
    size_t n = size_t(len) * kvd;
    if (n == 0) return FORGE_OK;
    gather_rows_kernel<<<grid_for(n), 256, 0, st>>>(out, pool, page_row, len, kvd);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace forge
