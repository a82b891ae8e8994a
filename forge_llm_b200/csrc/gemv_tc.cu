// Decode GEMV, streaming form (replaces matmul_vec_q8_0_KxN / matmul_vec_q4_0_KxN,
// crates/forgellm-codegen-cpu/src/emit.rs:2047-2087 and :2910-2953, with the reference's fusion
// patterns as prologue/epilogue: RMSNorm :327-334, residual :455-459, bias + RoPE + cache write
// :4108-4153, silu_mul :381-386).
//
// HBM-bound by design: one persistent CTA per SM pulls its share of the weight stream with 1-D
// bulk copies (cp.async.bulk, completion on an mbarrier) into a ring of shared-memory stages, so
// the bytes in flight (~140 KB per SM) do not depend on the instruction stream.  Eight consumer
// warps turn each 16-row x 32-column tile into two m16n8k16 tensor-core products: the quantised
// integers are exact in fp16 (nibble / byte spliced into the mantissa of 1024.0), the f32
// activation is carried as an fp16 pair hi + lo (after an exact power-of-two pre-scale) in two
// columns of the B operand, accumulation is f32, and the f16 block scale multiplies the 32-wide
// partial sum in f32 - so the result is the reference's f32 arithmetic up to summation order.
//
// Weight layout ("tiled"): the matrix is cut into tiles of 16 rows x one 32-value block per row,
// stored K-major per 16-row band.  A tile is {8 x half2 (d[row g], d[row g+8])}{quant bytes in
// MMA-fragment order, 8 (Q4_0) or 16 (Q8_0) bytes per lane}: 288 or 544 bytes, i.e. exactly the
// 18 / 34 bytes per block of the GGUF stream, every tile 16-byte aligned.
#include "common.cuh"

namespace forge {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;  // + one producer warp
constexpr int kStages = 8;
constexpr uint32_t kSpinLimit = 1u << 24;

template <int QUANT> struct Tile {
    static constexpr int BYTES = (QUANT == FORGE_Q4_0) ? 288 : 544;
    static constexpr int CHUNK_TILES = (QUANT == FORGE_Q4_0) ? 64 : 32;   // tiles per pipeline stage
    static constexpr int STAGE_BYTES = BYTES * CHUNK_TILES;                 // 18432 / 17408
};

// ------------------------------------------------------------------ PTX helpers
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
// bounded wait: returns false when the limit ran out (the caller records an error and unwinds)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lop3_or_and(uint32_t w, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "r"(mask), "r"(orv));  // (w & mask) | orv
    return r;
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
// 8 nibbles (n0..n7) of a Q4_0 fragment word -> the four fp16x2 A registers of one k16 step,
// value = nibble - 8 exactly.  n0,n4 -> a[0]; n1,n5 -> a[1]; n2,n6 -> a[2]; n3,n7 -> a[3].
__device__ __forceinline__ void dequant_q4(uint32_t w, uint32_t (&a)[4]) {
    const uint32_t magic = 0x64006400u;                  // (1024.0, 1024.0)
    const uint32_t c1032 = 0x64086408u;                  // 1032.0
    const uint32_t sixteenth = 0x2C002C00u, m72 = 0xD480D480u;  // 1/16, -72.0
    uint32_t w8 = w >> 8;
    a[0] = h2_sub(lop3_or_and(w, 0x000F000Fu, magic), c1032);
    a[1] = h2_fma(lop3_or_and(w, 0x00F000F0u, magic), sixteenth, m72);   // (1024 + 16 n)/16 - 72 = n - 8
    a[2] = h2_sub(lop3_or_and(w8, 0x000F000Fu, magic), c1032);
    a[3] = h2_fma(lop3_or_and(w8, 0x00F000F0u, magic), sixteenth, m72);
}
// 4 bytes (stored as q + 128) -> two fp16x2 registers holding q exactly
__device__ __forceinline__ void dequant_q8(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t c1152 = 0x64806480u;                  // 1024 + 128
    lo = h2_sub(__byte_perm(w, 0x64646464u, 0x4140), c1152);
    hi = h2_sub(__byte_perm(w, 0x64646464u, 0x4342), c1152);
}

struct TcParams {
    const uint8_t* w;      // tiled weights
    int K, N, kb, row_tiles;
    GemvArgs a;
    int* err;              // device error word (set when a bounded wait gives up)
};

// x fragments in shared memory: for k-block kb, column c (0 = hi, 1 = lo), quad lane t:
// uint4 {k16 step 0: (k=2t,2t+1), (k=2t+8,2t+9); step 1: the same + 16}
template <int QUANT, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemv_tc_kernel(TcParams p) {
    using T = Tile<QUANT>;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t full_bar[kStages], empty_bar[kStages];
    __shared__ float red[2][kConsumerWarps][16];
    __shared__ float s_part[32];
    __shared__ float s_inv, s_unscale, s_scale;
    __shared__ int s_err;
    unsigned char* ring = smem;
    uint4* xf = reinterpret_cast<uint4*>(smem + size_t(kStages) * T::STAGE_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int K = p.K, KB = p.kb;
    const int chunks_per_rt = (KB + T::CHUNK_TILES - 1) / T::CHUNK_TILES;
    // row tiles of this CTA: rt = blockIdx.x, + gridDim.x, ...
    const int my_rts = (p.row_tiles > int(blockIdx.x)) ? (p.row_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;
    const int total_chunks = my_rts * chunks_per_rt;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kConsumerWarps); }
        s_err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // ---- producer warp: streams this CTA's chunks, once per batch row, as fast as stages free up.
    // It starts right away: the weights do not depend on the activations being staged below.
    if (warp == kConsumerWarps) {
        if (lane == 0) {
            const int all = total_chunks * p.a.batch;
            for (int cc = 0; cc < all; ++cc) {
                const int st = cc % kStages, use = cc / kStages;
                if (use > 0 && !mbar_wait(&empty_bar[st], (use - 1) & 1)) { atomicExch(&s_err, 1); break; }
                if (*reinterpret_cast<volatile int*>(&s_err)) break;
                const int c = cc % total_chunks;
                const int rt = int(blockIdx.x) + (c / chunks_per_rt) * int(gridDim.x);
                const int kb0 = (c % chunks_per_rt) * T::CHUNK_TILES;
                const int nt = min(T::CHUNK_TILES, KB - kb0);
                const uint32_t bytes = uint32_t(nt) * T::BYTES;
                mbar_expect_tx(&full_bar[st], bytes);
                bulk_g2s(ring + size_t(st) * T::STAGE_BYTES, p.w + (size_t(rt) * KB + kb0) * T::BYTES, bytes, &full_bar[st]);
            }
        }
        return;
    }

    // ---- consumer warps (256 threads, named barrier 1)
    constexpr int kCT = kConsumerWarps * 32;
    auto csync = [] { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); };
    for (int b = 0; b < p.a.batch; ++b) {
        // stage the activation row as hi/lo fp16 MMA fragments (optionally RMS-normalised)
        const float* x = p.a.x + size_t(b) * K;
        float ss = 0.f, mx = 0.f;
        for (int e = tid; e < K; e += kCT) { float v = x[e]; ss += v * v; mx = fmaxf(mx, fabsf(p.a.norm_w ? v * p.a.norm_w[e] : v)); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { ss += __shfl_xor_sync(0xffffffffu, ss, o); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); }
        csync();  // the previous batch row's fragments are no longer read
        if (lane == 0) { s_part[warp] = ss; s_part[16 + warp] = mx; }
        csync();
        if (tid == 0) {
            float s2 = 0.f, m2 = 0.f;
            for (int w = 0; w < kConsumerWarps; ++w) { s2 += s_part[w]; m2 = fmaxf(m2, s_part[16 + w]); }
            const float inv = p.a.norm_w ? 1.0f / sqrtf(s2 / float(K) + p.a.eps) : 1.0f;
            m2 *= inv;
            // exact power-of-two pre-scale that puts max|x| in [2^13, 2^14): hi and lo stay normal fp16
            int ex = 0;
            float sc = 1.0f;
            if (m2 > 0.f && m2 < 3.0e38f) { frexpf(m2, &ex); sc = ldexpf(1.0f, 14 - ex); }
            s_inv = inv;
            s_unscale = 1.0f / sc;
            s_scale = sc;
        }
        csync();
        const float inv = s_inv, sc = s_scale;
        for (int i = tid; i < KB * 4; i += kCT) {
            const int kbi = i >> 2, tt = i & 3;
            float v[8];
#pragma unroll
            for (int s = 0; s < 2; ++s)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int k = kbi * 32 + s * 16 + 2 * tt + (j & 1) + (j >> 1) * 8;
                    float xv = x[k];
                    if (p.a.norm_w) xv = xv * inv * p.a.norm_w[k];
                    v[s * 4 + j] = xv * sc;
                }
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                __half2 h = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
                float2 hf = __half22float2(h);
                __half2 l = __floats2half2_rn(v[2 * q] - hf.x, v[2 * q + 1] - hf.y);
                hi[q] = *reinterpret_cast<uint32_t*>(&h);
                lo[q] = *reinterpret_cast<uint32_t*>(&l);
            }
            xf[(kbi * 2 + 0) * 4 + tt] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            xf[(kbi * 2 + 1) * 4 + tt] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
        csync();

        const float unscale = s_unscale;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int c = 0; c < total_chunks; ++c) {
            const int cc = b * total_chunks + c;
            const int st = cc % kStages, use = cc / kStages;
            if (!mbar_wait(&full_bar[st], use & 1)) atomicExch(&s_err, 1);
            const int rti = c / chunks_per_rt, ci = c % chunks_per_rt;
            const int kb0 = ci * T::CHUNK_TILES;
            const int nt = min(T::CHUNK_TILES, KB - kb0);
            const unsigned char* base = ring + size_t(st) * T::STAGE_BYTES;
            for (int ti = warp; ti < nt; ti += kConsumerWarps) {
                const unsigned char* tp = base + size_t(ti) * T::BYTES;
                const uint4 bx = (g < 2) ? xf[((kb0 + ti) * 2 + g) * 4 + t] : make_uint4(0, 0, 0, 0);
                const float2 d = __half22float2(*reinterpret_cast<const __half2*>(tp + g * 4));
                float cfrag[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t a0[4], a1[4];
                if (QUANT == FORGE_Q4_0) {
                    const uint2 wq = *reinterpret_cast<const uint2*>(tp + 32 + lane * 8);
                    dequant_q4(wq.x, a0);
                    dequant_q4(wq.y, a1);
                } else {
                    const uint4 wq = *reinterpret_cast<const uint4*>(tp + 32 + lane * 16);
                    dequant_q8(wq.x, a0[0], a0[1]);
                    dequant_q8(wq.y, a0[2], a0[3]);
                    dequant_q8(wq.z, a1[0], a1[1]);
                    dequant_q8(wq.w, a1[2], a1[3]);
                }
                mma16816(cfrag, a0, bx.x, bx.y);
                mma16816(cfrag, a1, bx.z, bx.w);
                acc[0] += d.x * cfrag[0]; acc[1] += d.x * cfrag[1];
                acc[2] += d.y * cfrag[2]; acc[3] += d.y * cfrag[3];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[st]);
            if (ci != chunks_per_rt - 1) continue;

            // ---- row tile complete: combine the warps' partial sums, then the epilogue
            const int rb = rti & 1;
            if (t == 0) { red[rb][warp][g] = acc[0] + acc[1]; red[rb][warp][g + 8] = acc[2] + acc[3]; }
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            csync();
            if (warp != 0) continue;
            if (tid < 16) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) v += red[rb][w][tid];
                red[rb][0][tid] = v * unscale;
            }
            __syncwarp();
            const int row = (int(blockIdx.x) + rti * int(gridDim.x)) * 16 + tid;
            if (tid >= 16 || row >= p.N) continue;
            const float v = red[rb][0][tid];
            if (EPI == EPI_STORE) {
                p.a.out[size_t(b) * p.N + row] = v;
            } else if (EPI == EPI_RESID) {
                p.a.out[size_t(b) * p.N + row] = p.a.resid[size_t(b) * p.N + row] + v;
            } else if (EPI == EPI_SILU) {
                if ((tid & 1) == 0) {  // rows interleaved at pack time: 2j = gate_j, 2j+1 = up_j
                    const float up = red[rb][0][tid + 1];
                    p.a.out[size_t(b) * (p.N / 2) + (row >> 1)] = (v / (1.0f + expf(-v))) * up;
                }
            } else if ((tid & 1) == 0) {  // EPI_QKV: the thread of the even row handles the (even, odd) pair
                float v0 = v, v1 = red[rb][0][tid + 1];
                if (p.a.bias) { v0 += p.a.bias[row]; v1 += p.a.bias[row + 1]; }
                const int pos = p.a.seq_len[b];
                const int qk = p.a.qk, kv = p.a.kv, hd = p.a.head_dim;
                int col = row, region = 0;
                if (col >= qk) { col -= qk; region = 1; }
                if (region == 1 && col >= kv) { col -= kv; region = 2; }
                if (region < 2) {
                    const float2 cs = reinterpret_cast<const float2*>(p.a.rope)[size_t(pos) * (hd / 2) + (col % hd) / 2];
                    const float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;
                    v0 = r0; v1 = r1;
                }
                if (region == 0) {
                    *reinterpret_cast<float2*>(p.a.q_out + size_t(b) * qk + col) = make_float2(v0, v1);
                } else {
                    const int page = p.a.page_table[size_t(b) * p.a.pages_per_seq + pos / FORGE_KV_PAGE];
                    __half* pool = region == 1 ? p.a.k_pool : p.a.v_pool;
                    *reinterpret_cast<__half2*>(pool + (size_t(page) * FORGE_KV_PAGE + pos % FORGE_KV_PAGE) * kv + col) =
                        __floats2half2_rn(v0, v1);
                }
            }
        }
    }
    csync();
    if (tid == 0 && s_err && p.err) atomicExch(p.err, 1);
}

// ------------------------------------------------------------------ packing
// thread per (tile, lane): gathers the lane's fragment bytes from the two raw GGUF rows it owns
template <int QUANT>
__global__ void tile_pack_kernel(const uint8_t* const* __restrict__ row_src, int KB, int row_tiles, uint8_t* __restrict__ dst) {
    constexpr int BS = QUANT == FORGE_Q8_0 ? 34 : 18;
    using T = Tile<QUANT>;
    const long total = long(row_tiles) * KB * 32;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        const int lane = int(i & 31);
        const long tile = i >> 5;
        const int kb = int(tile % KB), rt = int(tile / KB);
        const int g = lane >> 2, t = lane & 3;
        const uint8_t* r0 = row_src[rt * 16 + g];
        const uint8_t* r1 = row_src[rt * 16 + g + 8];
        const uint8_t* b0 = r0 ? r0 + size_t(kb) * BS : nullptr;
        const uint8_t* b1 = r1 ? r1 + size_t(kb) * BS : nullptr;
        uint8_t* tp = dst + size_t(tile) * T::BYTES;
        if (t == 0) {
            uint16_t d0 = b0 ? uint16_t(b0[0] | (b0[1] << 8)) : 0, d1 = b1 ? uint16_t(b1[0] | (b1[1] << 8)) : 0;
            *reinterpret_cast<uint32_t*>(tp + g * 4) = uint32_t(d0) | (uint32_t(d1) << 16);
        }
        // element k of a block: Q8_0 byte 2+k; Q4_0 byte 2 + (k & 15), low nibble for k < 16 else high
        auto q8 = [&](const uint8_t* blk, int k) -> uint32_t { return blk ? uint32_t(uint8_t(blk[2 + k] ^ 0x80)) : 0x80u; };
        auto q4 = [&](const uint8_t* blk, int k) -> uint32_t { return blk ? uint32_t((blk[2 + (k & 15)] >> ((k >> 4) * 4)) & 15u) : 8u; };
        if (QUANT == FORGE_Q4_0) {
            uint32_t w[2];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const int k = s * 16 + 2 * t;
                // nibble order n0..n7: (row g,k) (row g+8,k) (row g,k+8) (row g+8,k+8) then the same for k+1
                w[s] = q4(b0, k) | (q4(b1, k) << 4) | (q4(b0, k + 8) << 8) | (q4(b1, k + 8) << 12) |
                       (q4(b0, k + 1) << 16) | (q4(b1, k + 1) << 20) | (q4(b0, k + 9) << 24) | (q4(b1, k + 9) << 28);
            }
            *reinterpret_cast<uint2*>(tp + 32 + lane * 8) = make_uint2(w[0], w[1]);
        } else {
            uint32_t w[4];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const int k = s * 16 + 2 * t;
                // bytes: a0a1 = (row g: k,k+1), a2a3 = (row g+8: k,k+1) | a4a5 = (row g: k+8,k+9), a6a7 = (row g+8: k+8,k+9)
                w[2 * s] = q8(b0, k) | (q8(b0, k + 1) << 8) | (q8(b1, k) << 16) | (q8(b1, k + 1) << 24);
                w[2 * s + 1] = q8(b0, k + 8) | (q8(b0, k + 9) << 8) | (q8(b1, k + 8) << 16) | (q8(b1, k + 9) << 24);
            }
            *reinterpret_cast<uint4*>(tp + 32 + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

template <int QUANT>
int32_t launch(const QTiled& w, GemvEpilogue epi, const GemvArgs& a, int* err, cudaStream_t st) {
    using T = Tile<QUANT>;
    TcParams p;
    p.w = w.data; p.K = w.K; p.N = w.N; p.kb = w.K / 32; p.row_tiles = w.row_tiles; p.a = a; p.err = err;
    const size_t smem = size_t(kStages) * T::STAGE_BYTES + size_t(p.kb) * 2 * 4 * sizeof(uint4);
    if (smem > 220 * 1024) { set_error("gemv: K=%d needs %zu bytes of shared memory", w.K, smem); return FORGE_ERR_SHAPE; }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = w.row_tiles < sms ? w.row_tiles : sms;
#define FORGE_TC_LAUNCH(E)                                                                                              \
    do {                                                                                                                \
        FORGE_CUDA(cudaFuncSetAttribute(gemv_tc_kernel<QUANT, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))); \
        gemv_tc_kernel<QUANT, E><<<grid, kThreads, smem, st>>>(p);                                                      \
    } while (0)
    switch (epi) {
        case EPI_STORE: FORGE_TC_LAUNCH(EPI_STORE); break;
        case EPI_RESID: FORGE_TC_LAUNCH(EPI_RESID); break;
        case EPI_QKV: FORGE_TC_LAUNCH(EPI_QKV); break;
        case EPI_SILU: FORGE_TC_LAUNCH(EPI_SILU); break;
    }
#undef FORGE_TC_LAUNCH
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace

size_t qtiled_bytes(int quant, int K, int N) {
    const size_t rt = size_t((N + 15) / 16);
    return rt * size_t(K / 32) * (quant == FORGE_Q4_0 ? 288 : 544);
}

int32_t tile_pack(const uint8_t* const* row_src_dev, QTiled& dst, cudaStream_t st) {
    const long total = long(dst.row_tiles) * (dst.K / 32) * 32;
    if (total == 0) return FORGE_OK;
    const int grid = int((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
    if (dst.quant == FORGE_Q8_0) tile_pack_kernel<FORGE_Q8_0><<<grid, 256, 0, st>>>(row_src_dev, dst.K / 32, dst.row_tiles, dst.data);
    else tile_pack_kernel<FORGE_Q4_0><<<grid, 256, 0, st>>>(row_src_dev, dst.K / 32, dst.row_tiles, dst.data);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

int32_t gemv_tc(const QTiled& w, GemvEpilogue epi, const GemvArgs& a, int* err, cudaStream_t st) {
    if (w.K % 32 != 0 || w.K <= 0 || w.N <= 0) { set_error("gemv: K=%d must be a positive multiple of 32", w.K); return FORGE_ERR_SHAPE; }
    if ((epi == EPI_SILU || epi == EPI_QKV) && (w.N % 2)) { set_error("gemv: paired epilogue needs even N"); return FORGE_ERR_SHAPE; }
    return w.quant == FORGE_Q8_0 ? launch<FORGE_Q8_0>(w, epi, a, err, st) : launch<FORGE_Q4_0>(w, epi, a, err, st);
}

}  // namespace forge
