// Decode products for a batch of sequences: out[b][N] = x[b][K] . W[N][K]^T for up to 16 rows b per launch, with the
// weights streamed ONCE per launch (the generated module has no batched decode - a batch there is B calls of
// matmul_vec_q8_0_KxN / matmul_vec_q4_0_KxN, crates/forgellm-codegen-cpu/src/emit.rs:2047-2087 and :2910-2953 - so the
// values are those calls' values; what changes is how often the weight bytes cross HBM).
//
// Same streaming structure as the single-row kernel (gemv_tc.cu): a persistent CTA per SM, a producer lane feeding a
// ring of shared-memory stages with bulk copies (mbarrier completion), sixteen consumer warps = 8 row tiles x 2 halves
// of the k-blocks of a stage.  Differences:
//   * the tile product runs on the fp16 tensor-core path (mma.sync m16n8k16, f32 accumulate): the integer weights are
//     exact in fp16 and are multiplied by the block scale AFTER the product, in f32, like the single-row kernel does;
//     every activation enters as an fp16 pair hi + lo (hi = rn16(x), lo = rn16(x - hi): 22 bits), two B columns per
//     row b, so 8 columns = 4 rows per instruction and sixteen rows take four column groups;
//   * the activations do not fit in shared memory for a whole K (K x 64 bytes for sixteen rows): they are packed once
//     per product by a small kernel into B-fragment order, [k-block][16-element half][column group][lane] x 8 bytes,
//     and travel through the ring beside the weights, one more bulk copy per stage;
//   * a unit of work is 128 output rows (8 row tiles) x one K slice, whatever layout the matrix was packed in (in the
//     16-row-band layout a stage takes eight copies, one per row tile); matrices with few 128-row groups are split
//     along K over the CTAs, the slices' partial sums meet in scratch memory and the last slice to arrive (atomic
//     ticket) adds them in slice order, so results do not depend on timing.
// The k order inside a 16-element half is free as long as both operands agree: a lane's four weight bytes
// (k = 4t..4t+3 of the half) become its two A registers directly, (k0, k1 | k2, k3) for Q8_0 and (k0, k2 | k1, k3) for
// Q4_0 (the cheap nibble split), and the packed activations use the same order.
#include <algorithm>

#include "gemv_core.cuh"

namespace forge {

namespace {

using namespace core;

constexpr int kBatchRows = 16;                 // rows b per launch
constexpr int kGroupRows = 16 * kBandTiles;    // output rows per unit

// k-blocks per stage, bytes of the weight and activation parts of a stage, and stages in the ring (<= 200 KB, <= 8)
template <int QUANT, int NCG> struct BTile {
    static constexpr int CKB = QUANT == FORGE_Q8_0 ? 4 : 8;
    static constexpr int W_BYTES = Tile<QUANT>::BYTES * CKB * kBandTiles;   // 17408 / 18432
    static constexpr int A_BYTES = CKB * 2 * NCG * 256;
    static constexpr int STAGE = W_BYTES + A_BYTES;
    static constexpr int STAGES = (200 * 1024) / STAGE > 8 ? 8 : (200 * 1024) / STAGE;
};

struct BatchParams {
    const uint8_t* w;        // tiled weights
    const uint2* act;        // packed activations: [kb][2][NCG][32] x 8 bytes
    float* out;              // [rows b][N]
    const float* resid;      // optional: out = resid + product (may alias out)
    float* scratch;          // [slices][16][groups * 128] partial sums (slices > 1)
    int* tickets;            // [groups * 8] zero-initialised, self-resetting
    int K, N, kb, bt, groups, slices, units, nb;
    int bands16;             // 16-row bands the packed matrix really has (the last 128-row group may be short of them)
    int* err;
    BatchTp tp;              // tp.peer_ll != null: the product is pushed to the ranks' exchange buffers
};

struct BShared {
    uint64_t full_bar[8], empty_bar[8];
    int err;
};

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// NCG: column groups of 8 columns (4 rows b as hi/lo pairs) -> up to 4 * NCG rows
template <int QUANT, int NCG>
__global__ void __launch_bounds__(kThreads, 1) gemv_batch_kernel(BatchParams p) {
    using T = Tile<QUANT>;
    using B = BTile<QUANT, NCG>;
    constexpr int CKB = B::CKB, STAGES = B::STAGES, STAGE = B::STAGE;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ BShared sh;
    __shared__ float s_pair[kBandTiles][NCG * 2][32];   // the odd-k warp of a row tile hands its sums to the even-k warp
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full_bar[s], 1); mbar_init(&sh.empty_bar[s], kConsumerWarps); }
        sh.err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int chunks = (p.kb + CKB - 1) / CKB;
    const bool wide = p.bt == kBandTiles;

    if (warp == kConsumerWarps) {
        // ---- producer lane: for every unit of this CTA, the stages of its K slice: weights (one copy in the 128-row
        // layout, one per row tile in the 16-row layout) and the packed activations of the same k-blocks
        if (lane == 0) {
            int cc = 0;
            for (int u = blockIdx.x; u < p.units; u += gridDim.x) {
                const int grp = u / p.slices, slice = u - grp * p.slices;
                int c0, c1;
                slice_range(chunks, p.slices, slice, c0, c1);
                for (int c = c0; c < c1; ++c, ++cc) {
                    const int st = cc % STAGES, use = cc / STAGES;
                    if (use > 0 && !mbar_wait(&sh.empty_bar[st], (use - 1) & 1, &sh.err)) { atomicExch(&sh.err, 1); return; }
                    if (*reinterpret_cast<volatile int*>(&sh.err)) return;
                    const int kb0 = c * CKB, nkb = min(CKB, p.kb - kb0);
                    unsigned char* dst = smem + size_t(st) * STAGE;
                    const int tiles = wide ? kBandTiles : min(kBandTiles, p.bands16 - grp * kBandTiles);   // row tiles of the group that exist
                    const uint32_t wbytes = uint32_t(nkb) * tiles * T::BYTES, abytes = uint32_t(nkb) * 2 * NCG * 256;
                    mbar_expect_tx(&sh.full_bar[st], wbytes + abytes);
                    if (wide) {
                        bulk_g2s(dst, p.w + (size_t(grp) * p.kb + kb0) * kBandTiles * T::BYTES, wbytes, &sh.full_bar[st]);
                    } else {
#pragma unroll 1
                        for (int r8 = 0; r8 < tiles; ++r8)   // row tile r8 of the group is band grp * 8 + r8 of the 16-row layout
                            bulk_g2s(dst + size_t(r8) * CKB * T::BYTES, p.w + (size_t(grp * kBandTiles + r8) * p.kb + kb0) * T::BYTES,
                                     uint32_t(nkb) * T::BYTES, &sh.full_bar[st]);
                    }
                    bulk_g2s(dst + B::W_BYTES, p.act + size_t(kb0) * 2 * NCG * 32, abytes, &sh.full_bar[st]);
                }
            }
        }
        return;
    }

    // ---- consumers: warp = row tile r8 + 8 * (k half of the stage)
    const int r8 = warp % kBandTiles, khalf = warp / kBandTiles;
    int cc = 0;
    for (int u = blockIdx.x; u < p.units; u += gridDim.x) {
        const int grp = u / p.slices, slice = u - grp * p.slices;
        int c0, c1;
        slice_range(chunks, p.slices, slice, c0, c1);
        float acc[NCG][4];
#pragma unroll
        for (int cg = 0; cg < NCG; ++cg) acc[cg][0] = acc[cg][1] = acc[cg][2] = acc[cg][3] = 0.f;
        for (int c = c0; c < c1; ++c, ++cc) {
            const int st = cc % STAGES, use = cc / STAGES;
            if (!mbar_wait(&sh.full_bar[st], use & 1, &sh.err)) atomicExch(&sh.err, 1);
            const int nkb = min(CKB, p.kb - c * CKB);
            const unsigned char* stage = smem + size_t(st) * STAGE;
            const unsigned char* acts = stage + B::W_BYTES;
#pragma unroll
            for (int jj = 0; jj < CKB / 2; ++jj) {
                const int j = 2 * jj + khalf;   // k-block of the stage
                if (j >= nkb) break;
                const unsigned char* tp = stage + (wide ? size_t(j * kBandTiles + r8) : size_t(r8 * CKB + j)) * T::BYTES;
                const float2 d = __half22float2(*reinterpret_cast<const __half2*>(tp + g * 4));
                // A registers of the two 16-element halves: {row g (k pair 0), row g+8 (k pair 0), row g (k pair 1), row g+8 (k pair 1)}
                uint32_t a[2][4];
                if (QUANT == FORGE_Q4_0) {
                    // byte j of a word: low nibble = row g, high nibble = row g+8, k = 4t + j; fp16 1024 + n built in place,
                    // pairs (k0, k2) and (k1, k3); n - 8 = (1024 + n) - 1032 is exact
                    const uint2 wq = *reinterpret_cast<const uint2*>(tp + 32 + lane * 8);
                    const uint32_t bias = 0x64086408u;   // half2(1032, 1032)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t w = h ? wq.y : wq.x;
                        a[h][0] = hsub2_u32((w & 0x000F000Fu) | 0x64006400u, bias);
                        a[h][1] = hsub2_u32(((w >> 4) & 0x000F000Fu) | 0x64006400u, bias);
                        a[h][2] = hsub2_u32(((w >> 8) & 0x000F000Fu) | 0x64006400u, bias);
                        a[h][3] = hsub2_u32(((w >> 12) & 0x000F000Fu) | 0x64006400u, bias);
                    }
                } else {
                    // words: row g k lo, row g+8 k lo, row g k hi, row g+8 k hi (int8); fp16 1024 + (q + 128) built with a byte
                    // permute, pairs (k0, k1) and (k2, k3); q = (1152 + q) - 1152 is exact
                    const uint4 wq = *reinterpret_cast<const uint4*>(tp + 32 + lane * 16);
                    const uint32_t bias = 0x64806480u;   // half2(1152, 1152)
                    const uint32_t w0 = wq.x ^ 0x80808080u, w1 = wq.y ^ 0x80808080u, w2 = wq.z ^ 0x80808080u, w3 = wq.w ^ 0x80808080u;
                    a[0][0] = hsub2_u32(prmt(w0, 0x64646464u, 0x4140u), bias); a[0][2] = hsub2_u32(prmt(w0, 0x64646464u, 0x4342u), bias);
                    a[0][1] = hsub2_u32(prmt(w1, 0x64646464u, 0x4140u), bias); a[0][3] = hsub2_u32(prmt(w1, 0x64646464u, 0x4342u), bias);
                    a[1][0] = hsub2_u32(prmt(w2, 0x64646464u, 0x4140u), bias); a[1][2] = hsub2_u32(prmt(w2, 0x64646464u, 0x4342u), bias);
                    a[1][1] = hsub2_u32(prmt(w3, 0x64646464u, 0x4140u), bias); a[1][3] = hsub2_u32(prmt(w3, 0x64646464u, 0x4342u), bias);
                }
#pragma unroll
                for (int cg = 0; cg < NCG; ++cg) {
                    const uint2 b0 = *reinterpret_cast<const uint2*>(acts + ((size_t(j) * 2 + 0) * NCG + cg) * 256 + lane * 8);
                    const uint2 b1 = *reinterpret_cast<const uint2*>(acts + ((size_t(j) * 2 + 1) * NCG + cg) * 256 + lane * 8);
                    float cfr[4] = {0.f, 0.f, 0.f, 0.f};
                    mma16816(cfr, a[0], b0.x, b0.y);
                    mma16816(cfr, a[1], b1.x, b1.y);
                    acc[cg][0] += d.x * cfr[0]; acc[cg][1] += d.x * cfr[1];
                    acc[cg][2] += d.y * cfr[2]; acc[cg][3] += d.y * cfr[3];
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.empty_bar[st]);
        }
        // ---- this warp's part of the unit: per lane, rows g / g+8 of its row tile x rows b = 4 cg + t (hi + lo columns added)
        float v[NCG][2];
#pragma unroll
        for (int cg = 0; cg < NCG; ++cg) { v[cg][0] = acc[cg][0] + acc[cg][1]; v[cg][1] = acc[cg][2] + acc[cg][3]; }
        if (khalf == 1) {
#pragma unroll
            for (int cg = 0; cg < NCG; ++cg) { s_pair[r8][2 * cg][lane] = v[cg][0]; s_pair[r8][2 * cg + 1][lane] = v[cg][1]; }
        }
        asm volatile("bar.sync %0, 64;" ::"r"(2 + r8) : "memory");
        if (khalf == 1) {
            asm volatile("bar.sync %0, 64;" ::"r"(2 + r8) : "memory");  // s_pair consumed
            continue;
        }
#pragma unroll
        for (int cg = 0; cg < NCG; ++cg) { v[cg][0] += s_pair[r8][2 * cg][lane]; v[cg][1] += s_pair[r8][2 * cg + 1][lane]; }
        asm volatile("bar.sync %0, 64;" ::"r"(2 + r8) : "memory");
        const int rt = grp * kBandTiles + r8;
        const int row0 = rt * 16 + g;   // and row0 + 8
        const size_t npad = size_t(p.groups) * kGroupRows;
        bool finish = true;
        if (p.slices > 1) {
            // split K: publish this slice's partial sums; the last slice to arrive adds all of them in slice order
#pragma unroll
            for (int cg = 0; cg < NCG; ++cg) {
                float* sp = p.scratch + (size_t(slice) * kBatchRows + 4 * cg + t) * npad;
                sp[row0] = v[cg][0];
                sp[row0 + 8] = v[cg][1];
            }
            __threadfence();
            __syncwarp();
            int old = 0;
            if (lane == 0) old = atomicAdd(p.tickets + rt, 1);
            old = __shfl_sync(0xffffffffu, old, 0);
            finish = old == p.slices - 1;
            if (finish) {
                __threadfence();
                if (lane == 0) p.tickets[rt] = 0;  // ready for the next use
#pragma unroll
                for (int cg = 0; cg < NCG; ++cg) {
                    float s0 = 0.f, s1 = 0.f;
                    for (int s = 0; s < p.slices; ++s) {
                        const float* sp = p.scratch + (size_t(s) * kBatchRows + 4 * cg + t) * npad;
                        s0 += __ldcg(sp + row0);
                        s1 += __ldcg(sp + row0 + 8);
                    }
                    v[cg][0] = s0; v[cg][1] = s1;
                }
            }
        }
        if (finish) {
            const uint32_t tag = p.tp.peer_ll ? __ldcg(p.tp.step_counter) * p.tp.step_mul + p.tp.step_add : 0u;
#pragma unroll
            for (int cg = 0; cg < NCG; ++cg) {
                const int b = 4 * cg + t;
                if (b >= p.nb) continue;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int row = row0 + 8 * hh;
                    if (row < p.N) {
                        const size_t off = size_t(b) * p.N + row;
                        if (p.tp.peer_ll) {
                            // one 8-byte store per rank: value and tag travel together (own buffer included)
                            const uint2 pair = make_uint2(__float_as_uint(v[cg][hh]), tag);
                            for (int r = 0; r < p.tp.world; ++r) p.tp.peer_ll[r][p.tp.base + size_t(p.tp.rank) * p.tp.cap + off] = pair;
                        } else {
                            p.out[off] = (p.resid ? p.resid[off] : 0.f) + v[cg][hh];
                        }
                    }
                }
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kCT) : "memory");
    if (tid == 0 && sh.err && p.err) atomicExch(p.err, 1);
}

// ---------------------------------------------------------------------------------------------- activation packing
// One CTA per row b: x (optionally RMS-normalised, or SiLU(gate) * up of an interleaved [2 * K] row) -> fp16 hi / lo
// B fragments.  Column 2 * (b % 4) holds hi, the next one lo; lane = 4 * column + t carries k = 4t..4t+3 of a half.
enum PackMode { PACK_PLAIN = 0, PACK_NORM = 1, PACK_SILU = 2 };

template <int QUANT>
__global__ void __launch_bounds__(256) act_pack_kernel(float* x, size_t x_stride, const float* __restrict__ norm_w, float eps,
                                                       int mode, int K, int ncg, uint2* __restrict__ dst, BatchTp tp) {
    __shared__ float s_red[8];
    const int b = blockIdx.x;
    float* row = x + size_t(b) * x_stride;
    float inv = 1.0f;
    if (mode == PACK_NORM) {
        const uint32_t tag = tp.local_ll ? __ldcg(tp.step_counter) * tp.step_mul + tp.step_add : 0u;
        float ss = 0.f;
        for (int i = threadIdx.x * 4; i < K; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(row + i);
            if (tp.local_ll) {
                // the row-sliced product in front of this one: add the ranks' parts in rank order (four pairs = two 16-byte
                // loads per rank, polled until all four carry this sum's tag) and put the residual stream back
                for (int r = 0; r < tp.world; ++r) {
                    const uint2* src = tp.local_ll + tp.base + size_t(r) * tp.cap + size_t(b) * K + i;
                    uint4 p0 = make_uint4(0, 0, 0, 0), p1 = p0;
                    bool ok = false;
                    for (uint32_t it = 0; it < tp.wait_limit && !ok; ++it) {
                        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(p0.x), "=r"(p0.y), "=r"(p0.z), "=r"(p0.w) : "l"(src) : "memory");
                        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(p1.x), "=r"(p1.y), "=r"(p1.z), "=r"(p1.w) : "l"(src + 2) : "memory");
                        ok = p0.y == tag && p0.w == tag && p1.y == tag && p1.w == tag;
                        if (!ok && (it & 1023u) == 1023u && *reinterpret_cast<volatile int*>(tp.err)) break;   // somebody already gave up
                    }
                    if (!ok) { atomicExch(tp.err, 1); p0.x = p0.z = p1.x = p1.z = 0; }
                    v.x += __uint_as_float(p0.x); v.y += __uint_as_float(p0.z); v.z += __uint_as_float(p1.x); v.w += __uint_as_float(p1.z);
                }
                *reinterpret_cast<float4*>(row + i) = v;
            }
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float s2 = 0.f;
        for (int w = 0; w < int(blockDim.x >> 5); ++w) s2 += s_red[w];
        inv = 1.0f / sqrtf(s2 / float(K) + eps);
    }
    const int cg = b >> 2, col = 2 * (b & 3);
    for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {   // i: four consecutive k
        float4 v;
        if (mode == PACK_SILU) {
            const float4 a = *reinterpret_cast<const float4*>(row + 8 * i), c = *reinterpret_cast<const float4*>(row + 8 * i + 4);
            v = make_float4((a.x / (1.0f + expf(-a.x))) * a.y, (a.z / (1.0f + expf(-a.z))) * a.w,
                            (c.x / (1.0f + expf(-c.x))) * c.y, (c.z / (1.0f + expf(-c.z))) * c.w);
        } else {
            v = *reinterpret_cast<const float4*>(row + 4 * i);
            if (mode == PACK_NORM) {
                const float4 nw = *reinterpret_cast<const float4*>(norm_w + 4 * i);
                v = make_float4(v.x * inv * nw.x, v.y * inv * nw.y, v.z * inv * nw.z, v.w * inv * nw.w);
            }
        }
        const float e[4] = {v.x, v.y, v.z, v.w};
        const int o1 = QUANT == FORGE_Q4_0 ? 2 : 1, o2 = QUANT == FORGE_Q4_0 ? 1 : 2;   // (k0, k2 | k1, k3) or (k0, k1 | k2, k3)
        const __half2 h0 = __floats2half2_rn(e[0], e[o1]), h1 = __floats2half2_rn(e[o2], e[3]);
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        const __half2 l0 = __floats2half2_rn(e[0] - f0.x, e[o1] - f0.y), l1 = __floats2half2_rn(e[o2] - f1.x, e[3] - f1.y);
        const int kb = i >> 3, h = (i >> 2) & 1, t = i & 3;
        uint2* d = dst + ((size_t(kb) * 2 + h) * ncg + cg) * 32 + t;
        d[4 * col] = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        d[4 * (col + 1)] = make_uint2(*reinterpret_cast<const uint32_t*>(&l0), *reinterpret_cast<const uint32_t*>(&l1));
    }
}

template <int QUANT, int NCG>
int32_t launch_batch(const BatchParams& p, int grid, cudaStream_t st) {
    using B = BTile<QUANT, NCG>;
    const size_t smem = size_t(B::STAGES) * B::STAGE;
    auto kern = gemv_batch_kernel<QUANT, NCG>;
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    kern<<<grid, kThreads, smem, st>>>(p);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace

int gemv_batch_ncg(int nb) { return nb <= 4 ? 1 : nb <= 8 ? 2 : 4; }

// K slices per 128-row group: the count (1..8, never finer than one stage) that fills whole rounds of CTAs best, the
// smaller count on ties (every slice costs a pass through scratch memory)
constexpr int kBatchMaxSlices = 8;
int gemv_batch_slices(int groups, int chunks, int sms) {
    int best = 1;
    double best_eff = 0.0;
    for (int s = 1; s <= std::min(kBatchMaxSlices, chunks); ++s) {
        const long units = long(groups) * s;
        const double eff = double(units) / double(((units + sms - 1) / sms) * sms);
        if (eff > best_eff + 0.03) { best_eff = eff; best = s; }
    }
    return best;
}
size_t gemv_batch_act_words(int K, int nb) { return size_t(K / 32) * 2 * gemv_batch_ncg(nb) * 32; }   // uint2 entries
// split-K scratch (floats) and tickets (ints) a matrix of N rows and K columns needs on a GPU with `sms` SMs
size_t gemv_batch_scratch_floats(int N, int K, int quant, int sms) {
    const int groups = (N + kGroupRows - 1) / kGroupRows, ckb = quant == FORGE_Q8_0 ? 4 : 8;
    const int slices = gemv_batch_slices(groups, (K / 32 + ckb - 1) / ckb, sms);
    return slices > 1 ? size_t(slices) * kBatchRows * groups * kGroupRows : 0;
}
size_t gemv_batch_tickets(int N) { return size_t((N + kGroupRows - 1) / kGroupRows) * kBandTiles; }

int32_t gemv_batch_pack(uint2* dst, float* x, size_t x_stride, int nb, int K, int quant, int mode, const float* norm_w, float eps, cudaStream_t st,
                        const BatchTp* consume) {
    if (nb <= 0) return FORGE_OK;
    if (nb > kBatchRows || K % 32 || (quant != FORGE_Q8_0 && quant != FORGE_Q4_0)) { set_error("batched product: %d rows / K=%d / format %d unsupported", nb, K, quant); return FORGE_ERR_SHAPE; }
    const int ncg = gemv_batch_ncg(nb);
    if (consume && (mode != PACK_NORM || !consume->local_ll || size_t(nb) * K > consume->cap)) { set_error("batched product: bad tensor-parallel consume"); return FORGE_ERR_INVALID_ARG; }
    const BatchTp tp = consume ? *consume : BatchTp();
    if (quant == FORGE_Q8_0) act_pack_kernel<FORGE_Q8_0><<<nb, 256, 0, st>>>(x, x_stride, norm_w, eps, mode, K, ncg, dst, tp);
    else act_pack_kernel<FORGE_Q4_0><<<nb, 256, 0, st>>>(x, x_stride, norm_w, eps, mode, K, ncg, dst, tp);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

int32_t gemv_batch(const QTiled& w, const uint2* act, int nb, float* out, const float* resid, const GemvSplit& sp, int* err, cudaStream_t st,
                   const BatchTp* push) {
    if (nb <= 0) return FORGE_OK;
    if (nb > kBatchRows || w.K % 32 || (w.quant != FORGE_Q8_0 && w.quant != FORGE_Q4_0) || (w.bt != 1 && w.bt != core::kBandTiles)) {
        set_error("batched product: %d rows / K=%d / format %d unsupported", nb, w.K, w.quant);
        return FORGE_ERR_SHAPE;
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    BatchParams p{};
    p.w = w.data; p.act = act; p.out = out; p.resid = resid; p.K = w.K; p.N = w.N; p.kb = w.K / 32; p.bt = w.bt; p.nb = nb; p.err = err;
    if (push) {
        if (!push->peer_ll || size_t(nb) * w.N > push->cap) { set_error("batched product: bad tensor-parallel push"); return FORGE_ERR_INVALID_ARG; }
        p.tp = *push;
    }
    // 128-row groups; in the 16-row layout the matrix is padded to whole 16-row bands only, so the last group may be
    // short of bands (the kernel copies the ones that exist; rows beyond N are never stored)
    const int bands16 = w.bt == 1 ? w.bands : w.bands * core::kBandTiles;
    p.bands16 = bands16;
    p.groups = (bands16 + core::kBandTiles - 1) / core::kBandTiles;
    const int ckb = w.quant == FORGE_Q8_0 ? 4 : 8;
    const int chunks = (p.kb + ckb - 1) / ckb;
    p.slices = gemv_batch_slices(p.groups, chunks, sms);
    if (p.slices > 1 && (!sp.scratch || !sp.tickets || p.slices > sp.max_slices)) p.slices = 1;
    p.units = p.groups * p.slices;
    p.scratch = sp.scratch; p.tickets = sp.tickets;
    const int grid = std::min(p.units, sms);
    const int ncg = gemv_batch_ncg(nb);
#define FORGE_GB(Q)                                                   \
    do {                                                              \
        if (ncg == 1) return launch_batch<Q, 1>(p, grid, st);         \
        if (ncg == 2) return launch_batch<Q, 2>(p, grid, st);         \
        return launch_batch<Q, 4>(p, grid, st);                       \
    } while (0)
    if (w.quant == FORGE_Q8_0) FORGE_GB(FORGE_Q8_0);
    FORGE_GB(FORGE_Q4_0);
#undef FORGE_GB
}

}  // namespace forge
