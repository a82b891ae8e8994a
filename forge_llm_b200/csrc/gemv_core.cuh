// Device-side core of the streaming decode GEMV (gemv_tc.cu).
//
// One CTA = 16 consumer warps + 1 producer warp.  The producer lane issues 1-D bulk copies
// (cp.async.bulk, mbarrier completion) of "chunks" - runs of k-blocks of one 128-row band of the
// tiled weight layout - into a ring of shared-memory stages.  Two consumer warps share each of
// the band's eight 16-row tiles (even / odd k-blocks) and turn every 16 x 32 tile into one
// integer tensor-core product (mma.sync m16n8k32, s8/u8 x s8 -> s32) against the activation held
// in shared memory as the four balanced base-256 digits (bytes) of a 31-bit fixed-point value; digit
// sums are scaled by the f16 block scale and accumulated in f32.  See gemv_tc.cu for the layout.
#pragma once

#include "common.cuh"

namespace forge {
namespace core {

constexpr int kBandTiles = 8;                        // 16-row tiles per band in the wide layout (bt = 8); bt = 1: one tile
constexpr int kConsumerWarps = 16;                   // two warps per row tile (even / odd k-blocks of a chunk)
constexpr int kCT = kConsumerWarps * 32;             // consumer threads
constexpr int kThreads = (kConsumerWarps + 1) * 32;  // + one producer warp
constexpr int kStages = 8;                           // most stages any format uses (Tile<QUANT>::STAGES)
constexpr int kMaxKB = 352;                          // K <= 11264
constexpr uint32_t kSpinLimit = 1u << 24;

// K-quants (256-element super-blocks) are re-tiled at load time into the same 16-row x 32-column tiles with the
// super-block fields expanded per tile, so the tile loop stays one MMA per tile:
//   Q4_K: 8 x float4 {d*sc[g], dmin*m[g], d*sc[g+8] / 16, dmin*m[g+8]} + nibbles as for Q4_0 (unsigned)   = 384 bytes
//   Q6_K: 8 x float4 {d*sc_lo[g], d*sc_hi[g], d*sc_lo[g+8], d*sc_hi[g+8]} + (q6 - 32) as int8, Q8_0 order = 640 bytes
// (all products of an f16 and a small integer: exact in f32).
inline bool is_kquant(int quant) { return quant == FORGE_Q4_K || quant == FORGE_Q6_K; }  // host side
template <int QUANT> struct KQuant { static constexpr bool value = QUANT == FORGE_Q4_K || QUANT == FORGE_Q6_K; };
template <int QUANT> struct Tile {
    static constexpr int BYTES = QUANT == FORGE_Q4_0 ? 288 : QUANT == FORGE_Q8_0 ? 544 : QUANT == FORGE_Q4_K ? 384 : 640;
    // k-blocks per pipeline stage and stages in the ring.  The per-stage work of a warp (wait, arrive, loop) is
    // amortised over CHUNK_KB / 2 tiles, so the K-quants take 8 k-blocks per stage and fewer, larger stages
    // (the bytes in flight stay at 144-160 KB per SM).
    static constexpr int CHUNK_KB = (QUANT == FORGE_Q8_0) ? 4 : 8;
    static constexpr int STAGES = QUANT == FORGE_Q4_K ? 6 : QUANT == FORGE_Q6_K ? 4 : kStages;
    static constexpr int STAGE_BYTES = BYTES * CHUNK_KB * kBandTiles;       // 18432 / 17408 / 24576 / 40960
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
// bounded wait: returns false when the limit ran out, or as soon as *stop is set (somebody in the CTA has already
// given up, so whatever this wait is for may never come); the caller records an error and goes on
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const int* stop = nullptr) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (stop && (i & 15) == 15 && *reinterpret_cast<const volatile int*>(stop)) return false;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// D(16x8, s32) = A(16x32, row) * B(32x8, s8, col) + C, A unsigned (Q4_0 nibbles) or signed (Q8_0).
// Not volatile: independent tiles interleave.
__device__ __forceinline__ void imma16832_u8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma16832_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(kCT) : "memory"); }

// chunk range [c0, c1) of slice s when `chunks` chunks are cut into `slices` near-equal slices
__device__ __forceinline__ void slice_range(int chunks, int slices, int s, int& c0, int& c1) {
    if (slices == 1) { c0 = 0; c1 = chunks; return; }
    c0 = (chunks * s) / slices;  // chunks * slices is far below 2^31
    c1 = (chunks * (s + 1)) / slices;
}
// band and slice of unit u
__device__ __forceinline__ void unit_split(int u, int slices, int& band, int& slice) {
    if (slices == 1) { band = u; slice = 0; return; }
    band = u / slices;
    slice = u - band * slices;
}
// k-blocks per chunk (a power of two: a chunk is always CHUNK_KB * 8 tiles) and chunks per band
template <int QUANT>
__device__ __forceinline__ int chunk_kb_shift(int bt) {
    constexpr int base = Tile<QUANT>::CHUNK_KB == 8 ? 3 : 2;  // log2(CHUNK_KB)
    return bt == kBandTiles ? base : base + 3;
}

// One GEMV ("phase") as the kernels see it.
struct Phase {
    const uint8_t* w;      // tiled weights
    int K, N, kb, bands;   // kb = K/32, bands = ceil(N / (16 * bt))
    int bt;                // row tiles per band: 8 (two warps per tile) or 1 (all sixteen warps share the tile)
    int slices;            // K slices per band (1 = no split)
    int units;             // bands * slices
    int rot;               // unit u is served by CTA (u + rot) % gridDim.x
    int epi;               // GemvEpilogue
    float* scratch;        // [slices][bands*16*bt] partial sums (slices > 1 or EPI_PARTIAL)
    int* tickets;          // [bands*bt] zero-initialised, self-resetting (slices > 1)
    GemvArgs a;
};

__device__ __host__ inline size_t phase_npad(const Phase& ph) { return size_t(ph.bands) * 16 * ph.bt; }

// Shared-memory state of the pipeline; `cc` counts chunks and must advance identically in the
// producer and in every consumer warp.
struct Shared {
    uint64_t full_bar[kStages], empty_bar[kStages];
    float part[32];
    float pair[kBandTiles][16];
    float red[2][kConsumerWarps][16];
    int err;
};

// first unit of CTA `cta` and the stride between its units
__device__ __forceinline__ int first_unit(const Phase& ph, int cta, int grid) {
    if (ph.rot == 0) return cta;
    int r = (cta - ph.rot) % grid;
    return r < 0 ? r + grid : r;
}

// Ask L2 to fetch this CTA's share of [p, p + bytes) (16-byte aligned; 8 KB pieces dealt round-robin over the grid).
__device__ __forceinline__ void l2_prefetch_share(const void* p, size_t bytes) {
    constexpr size_t kPiece = 8192;
    const char* base = static_cast<const char*>(p);
    for (size_t off = size_t(blockIdx.x) * kPiece; off < bytes; off += size_t(gridDim.x) * kPiece) {
        const uint32_t n = uint32_t(min(kPiece, bytes - off)) & ~15u;
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(n) : "memory");
    }
}

// ---- producer side: issue all chunks of this CTA's units of one phase (one batch row).
// `when_ring_full()` runs once: when the ring is full for the first time, or after the last chunk if it never fills.
template <int QUANT, typename Hook>
__device__ __forceinline__ bool produce_phase(const Phase& ph, Shared& sh, unsigned char* ring, int& cc, Hook when_ring_full) {
    using T = Tile<QUANT>;
    const int cshift = chunk_kb_shift<QUANT>(ph.bt), ckb = 1 << cshift;
    const int chunks_per_band = (ph.kb + ckb - 1) >> cshift;
    bool hooked = false;
    for (int u = first_unit(ph, blockIdx.x, gridDim.x); u < ph.units; u += gridDim.x) {
        int band, slice, c0, c1;
        unit_split(u, ph.slices, band, slice);
        slice_range(chunks_per_band, ph.slices, slice, c0, c1);
        for (int c = c0; c < c1; ++c, ++cc) {
            const int st = cc % T::STAGES, use = cc / T::STAGES;
            if (use > 0 && !hooked) { hooked = true; when_ring_full(); }
            if (use > 0 && !mbar_wait(&sh.empty_bar[st], (use - 1) & 1, &sh.err)) { atomicExch(&sh.err, 1); return false; }
            if (*reinterpret_cast<volatile int*>(&sh.err)) return false;
            const int kb0 = c * ckb;
            const int nkb = min(ckb, ph.kb - kb0);
            const uint32_t bytes = uint32_t(nkb) * ph.bt * T::BYTES;
            mbar_expect_tx(&sh.full_bar[st], bytes);
            bulk_g2s(ring + size_t(st) * T::STAGE_BYTES, ph.w + (size_t(band) * ph.kb + kb0) * ph.bt * T::BYTES, bytes, &sh.full_bar[st]);
        }
    }
    if (!hooked) when_ring_full();
    return true;
}
template <int QUANT>
__device__ __forceinline__ bool produce_phase(const Phase& ph, Shared& sh, unsigned char* ring, int& cc) {
    return produce_phase<QUANT>(ph, sh, ring, cc, [] {});
}

// ---- consumer side, step 1: stage one activation row as int8 digit fragments.
// xf: for k-block kb, digit column c (0..3), quad lane t: uint2 {digits of k = 4t..4t+3, of k = 16+4t..+3}
// (the B fragment of m16n8k32).  The row is first written as plain floats into the fragment area
// ("fill": stage_fill_global below, or a caller's own loop), then converted in place by stage_finish:
// the 32 floats of a k-block and its 4 x 4 x 8-byte fragments occupy the same 128 bytes, and the four
// threads that convert a k-block sit in one warp.  All consumer warps take part in both steps.

// running sum(x^2) and max|x * norm_w| of the values a thread wrote during the fill
struct FillStat { float ss = 0.f, mx = 0.f; };

__device__ __forceinline__ void fill_note(FillStat& st, const float4& v, const float* norm_w, int e) {
    st.ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    if (norm_w) {
        const float4 nw = *reinterpret_cast<const float4*>(norm_w + e);
        st.mx = fmaxf(fmaxf(st.mx, fmaxf(fabsf(v.x * nw.x), fabsf(v.y * nw.y))), fmaxf(fabsf(v.z * nw.z), fabsf(v.w * nw.w)));
    } else {
        st.mx = fmaxf(fmaxf(st.mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
}

// Fill from global memory: x = base (may be null) + the sum of `nparts` partial vectors
// (parts + s * pstride), added in slice order.  With `writeback`, element group i (4 floats) is also
// stored by CTA i % gridDim.x, so the summed vector exists once in global memory afterwards.
// CG: read through L2 (data written by other CTAs of the same kernel).
template <bool CG>
__device__ __forceinline__ FillStat stage_fill_global(uint2* xf, const float* base, const float* parts, int nparts, size_t pstride,
                                                     float* writeback, int K, const float* norm_w) {
    float* xraw = reinterpret_cast<float*>(xf);
    FillStat st;
    csync();  // the previous contents of the fragment area are no longer read
    for (int e = threadIdx.x * 4; e < K; e += kCT * 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (base) v = CG ? __ldcg(reinterpret_cast<const float4*>(base + e)) : *reinterpret_cast<const float4*>(base + e);
        if (nparts > 0) {
            float4 pv[kGemvMaxSlices];
#pragma unroll
            for (int s = 0; s < kGemvMaxSlices; ++s)
                pv[s] = (s < nparts) ? __ldcg(reinterpret_cast<const float4*>(parts + size_t(s) * pstride + e)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < kGemvMaxSlices; ++s) { v.x += pv[s].x; v.y += pv[s].y; v.z += pv[s].z; v.w += pv[s].w; }
            if (writeback && ((e >> 2) % int(gridDim.x)) == int(blockIdx.x)) *reinterpret_cast<float4*>(writeback + e) = v;
        }
        fill_note(st, v, norm_w, e);
        *reinterpret_cast<float4*>(xraw + e) = v;
    }
    return st;
}

// Fill for the tensor-parallel sum: x = base + the ranks' partial rows, which arrive as {value, step} pairs written by
// peer GPUs (see GemvArgs::Tp).  A pair is valid once its step is `step`; the wait is bounded and reports through *err.
// Rank order is fixed, so every rank forms the same bits.  The sum is written once (element group i by CTA
// i % gridDim.x) to `writeback`.
__device__ __forceinline__ FillStat stage_fill_pairs(uint2* xf, const float* base, const uint2* ll, int world, uint32_t step,
                                                     float* writeback, int K, const float* norm_w, int* err, uint32_t limit) {
    float* xraw = reinterpret_cast<float*>(xf);
    FillStat st;
    csync();  // the previous contents of the fragment area are no longer read
    for (int e = threadIdx.x * 4; e < K; e += kCT * 4) {
        float4 v = __ldcg(reinterpret_cast<const float4*>(base + e));
        for (int r = 0; r < world; ++r) {
            const uint2* src = ll + size_t(r) * K + e;
            uint4 a, b;
            bool ok = false;
            for (uint32_t i = 0; i < limit && !ok && !*reinterpret_cast<volatile int*>(err); ++i) {  // the default limit is about a second
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src) : "memory");
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(src + 2) : "memory");
                ok = a.y == step && a.w == step && b.y == step && b.w == step;
            }
            if (!ok) atomicExch(err, 1);
            v.x += __uint_as_float(a.x); v.y += __uint_as_float(a.z); v.z += __uint_as_float(b.x); v.w += __uint_as_float(b.z);
        }
        if (writeback && ((e >> 2) % int(gridDim.x)) == int(blockIdx.x)) *reinterpret_cast<float4*>(writeback + e) = v;
        fill_note(st, v, norm_w, e);
        *reinterpret_cast<float4*>(xraw + e) = v;
    }
    return st;
}

// Convert the filled row in place; returns 1/scale.
template <int QUANT>
__device__ __forceinline__ float stage_finish(uint2* xf, int4* xoff, Shared& sh, FillStat st, int K, const float* norm_w, float eps) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int KB = K / 32;
    float* xraw = reinterpret_cast<float*>(xf);
    float ss = st.ss, mx = st.mx;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { ss += __shfl_xor_sync(0xffffffffu, ss, o); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); }
    if (lane == 0) { sh.part[warp] = ss; sh.part[16 + warp] = mx; }
    csync();
    float s2 = 0.f, m2 = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) { s2 += sh.part[w]; m2 = fmaxf(m2, sh.part[16 + w]); }
    const float inv = norm_w ? 1.0f / sqrtf(s2 / float(K) + eps) : 1.0f;
    if (KQuant<QUANT>::value) {
        // K-quant products take the row quantised to Q8_0 blocks, as the functions they replace do
        // (emit.rs:1412-1440): scale = absmax / 127 kept as f16 (1 for a zero block), q = round-half-away(x / scale)
        // in [-127, 127].  A k-block's 128-byte slot then holds {4 x uint2 B fragments (column 0), f32 scale,
        // f32 sum of q}; the dots are exact integers and the scale is applied per block.
        for (int i0 = 0; i0 < KB * 4; i0 += kCT) {
            const int i = i0 + tid;
            const bool on = i < KB * 4;
            const int kbi = i >> 2, tt = i & 3;
            float xv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (on) {
                const float4 r0 = *reinterpret_cast<const float4*>(xraw + kbi * 32 + 4 * tt);
                const float4 r1 = *reinterpret_cast<const float4*>(xraw + kbi * 32 + 16 + 4 * tt);
                xv[0] = r0.x; xv[1] = r0.y; xv[2] = r0.z; xv[3] = r0.w; xv[4] = r1.x; xv[5] = r1.y; xv[6] = r1.z; xv[7] = r1.w;
                if (norm_w) {
                    const float4 n0 = *reinterpret_cast<const float4*>(norm_w + kbi * 32 + 4 * tt);
                    const float4 n1 = *reinterpret_cast<const float4*>(norm_w + kbi * 32 + 16 + 4 * tt);
                    const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                    for (int q = 0; q < 8; ++q) xv[q] = xv[q] * inv * nw[q];
                }
            }
            float amax = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(xv[q]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            float bs = 1.0f, binv = 0.0f;
            if (amax != 0.f) { bs = __fdiv_rn(amax, 127.0f); binv = __fdiv_rn(1.0f, bs); }
            int qv[8], qsum = 0;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                qv[q] = int(fminf(127.f, fmaxf(-127.f, roundf(xv[q] * binv))));
                qsum += qv[q];
            }
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
            __syncwarp();  // all four readers of a k-block are done before it is overwritten
            if (on) {
                const uint32_t w0 = uint32_t(qv[0] & 255) | (uint32_t(qv[1] & 255) << 8) | (uint32_t(qv[2] & 255) << 16) | (uint32_t(qv[3] & 255) << 24);
                const uint32_t w1 = uint32_t(qv[4] & 255) | (uint32_t(qv[5] & 255) << 8) | (uint32_t(qv[6] & 255) << 16) | (uint32_t(qv[7] & 255) << 24);
                xf[kbi * 16 + tt] = make_uint2(w0, w1);
                if (tt == 0) *reinterpret_cast<float2*>(xraw + kbi * 32 + 8) = make_float2(bs < 5.9604644775390625e-8f ? 0.f : __half2float(__float2half_rn(bs)), float(qsum));  // the reference's f16 conversion flushes below 2^-24
            }
        }
        csync();
        return 1.0f;
    }
    m2 *= inv;
    // exact power-of-two scale that puts max|x| * 2^s in [2^29, 2^30): 31-bit signed fixed point
    float sc = 1.0f;
    if (m2 > 0.f && m2 < 3.0e38f) {
        const int E = int(__float_as_uint(m2) >> 23);  // biased exponent: m2 = f * 2^(E - 126), f in [0.5, 1)
        if (E >= 29) sc = __uint_as_float(uint32_t(283 - E) << 23);
        else { int ex = 0; frexpf(m2, &ex); sc = ldexpf(1.0f, 30 - ex); }
    }
    // Balanced base-256 digits without carries or bit-field extraction: with y = x + 0x80808080 (no wrap for
    // |x| < 2^30), byte c of y is digit c of x plus 128, so the digits are the bytes of y ^ 0x80808080.  Four
    // values are turned into four digit words (byte j = value j) by a 4 x 4 byte transpose.
    for (int i0 = 0; i0 < KB * 4; i0 += kCT) {
        const int i = i0 + tid;
        const bool on = i < KB * 4;
        const int kbi = i >> 2, tt = i & 3;
        uint32_t y[8];
        if (on) {
            const float4 r0 = *reinterpret_cast<const float4*>(xraw + kbi * 32 + 4 * tt);
            const float4 r1 = *reinterpret_cast<const float4*>(xraw + kbi * 32 + 16 + 4 * tt);
            float xv[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
            if (norm_w) {
                const float4 n0 = *reinterpret_cast<const float4*>(norm_w + kbi * 32 + 4 * tt);
                const float4 n1 = *reinterpret_cast<const float4*>(norm_w + kbi * 32 + 16 + 4 * tt);
                const float nw[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                for (int q = 0; q < 8; ++q) xv[q] = xv[q] * inv * nw[q];
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) y[q] = uint32_t(__float2int_rn(xv[q] * sc)) + 0x80808080u;
        }
        __syncwarp();  // all four readers of a k-block are done before it is overwritten
        int dsum[4] = {0, 0, 0, 0};
        if (on) {
            uint32_t w[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t a = __byte_perm(y[4 * h], y[4 * h + 1], 0x5140), b = __byte_perm(y[4 * h + 2], y[4 * h + 3], 0x5140);
                const uint32_t c = __byte_perm(y[4 * h], y[4 * h + 1], 0x7362), d = __byte_perm(y[4 * h + 2], y[4 * h + 3], 0x7362);
                w[h][0] = __byte_perm(a, b, 0x5410) ^ 0x80808080u;
                w[h][1] = __byte_perm(a, b, 0x7632) ^ 0x80808080u;
                w[h][2] = __byte_perm(c, d, 0x5410) ^ 0x80808080u;
                w[h][3] = __byte_perm(c, d, 0x7632) ^ 0x80808080u;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                dsum[c] = __dp4a(int(w[0][c]), 0x01010101, __dp4a(int(w[1][c]), 0x01010101, 0));
                xf[(kbi * 4 + c) * 4 + tt] = make_uint2(w[0][c], w[1][c]);
            }
        }
        if (QUANT == FORGE_Q4_0) {
            // Nibbles enter the product unsigned: rows g as n = q + 8, rows g+8 as 16 n (high nibble in
            // place).  The accumulators start at -8 * sum(digits) and -128 * sum(digits).
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                dsum[c] += __shfl_xor_sync(0xffffffffu, dsum[c], 1);
                dsum[c] += __shfl_xor_sync(0xffffffffu, dsum[c], 2);
            }
            if (on && tt == 0) {
                xoff[2 * kbi] = make_int4(-8 * dsum[0], -8 * dsum[1], -128 * dsum[0], -128 * dsum[1]);
                xoff[2 * kbi + 1] = make_int4(-8 * dsum[2], -8 * dsum[3], -128 * dsum[2], -128 * dsum[3]);
            }
        }
    }
    csync();
    return 1.0f / sc;
}

// the common case: one plain row from global memory
template <int QUANT, bool CG>
__device__ __forceinline__ float stage_activation(uint2* xf, int4* xoff, Shared& sh, const float* x, int K,
                                                  const float* norm_w, float eps) {
    const FillStat st = stage_fill_global<CG>(xf, x, nullptr, 0, 0, nullptr, K, norm_w);
    return stage_finish<QUANT>(xf, xoff, sh, st, K, norm_w, eps);
}

// The same for Q8_0 / Q4_0 in one pass: item i of a thread covers elements 4tt..4tt+3 and 16+4tt..16+4tt+3 of k-block kb
// (i = 4 kb + tt), exactly the values whose digits that thread writes, so they stay in registers from the load to
// the conversion.  The row and the norm weights are requested together (one memory round trip), warps without an
// item only take part in the barriers, and there are two barriers instead of three.  `fresh`: nobody can still be
// reading the fragment area (first row of a launch).
constexpr int kStageItems = 3;
// the register form takes rows of up to kStageItems items per thread; a normalised row must fit one item per thread
__device__ __forceinline__ bool stage_regs_ok(int K, const float* norm_w) { return K <= (norm_w ? 1 : kStageItems) * kCT * 8; }
template <int QUANT>
__device__ __forceinline__ float stage_activation_regs(uint2* xf, int4* xoff, Shared& sh, const float* x, int K,
                                                       const float* norm_w, float eps, bool fresh) {
    static_assert(!KQuant<QUANT>::value, "K-quant inputs are staged as Q8_0 blocks");
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nitems = K / 8;
    const bool busy = (warp << 5) < nitems;
    float xv[kStageItems][8], nw[8];
    float ss = 0.f, mx = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) nw[q] = 1.0f;
#pragma unroll
    for (int it = 0; it < kStageItems; ++it) {
        const int i = it * kCT + tid;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (i < nitems) {
            const int e0 = (i >> 2) * 32 + 4 * (i & 3);
            a = *reinterpret_cast<const float4*>(x + e0);
            b = *reinterpret_cast<const float4*>(x + e0 + 16);
            if (norm_w && it == 0) {
                const float4 na = __ldg(reinterpret_cast<const float4*>(norm_w + e0)), nb = __ldg(reinterpret_cast<const float4*>(norm_w + e0 + 16));
                nw[0] = na.x; nw[1] = na.y; nw[2] = na.z; nw[3] = na.w; nw[4] = nb.x; nw[5] = nb.y; nw[6] = nb.z; nw[7] = nb.w;
            }
        }
        xv[it][0] = a.x; xv[it][1] = a.y; xv[it][2] = a.z; xv[it][3] = a.w; xv[it][4] = b.x; xv[it][5] = b.y; xv[it][6] = b.z; xv[it][7] = b.w;
    }
    if (busy) {
#pragma unroll
        for (int it = 0; it < kStageItems; ++it)
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                ss += xv[it][q] * xv[it][q];
                mx = fmaxf(mx, fabsf(it == 0 ? xv[it][q] * nw[q] : xv[it][q]));
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { ss += __shfl_xor_sync(0xffffffffu, ss, o); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); }
    }
    if (!fresh) csync();  // the previous contents of the fragment area (and of sh.part) are no longer read
    if (lane == 0) { sh.part[warp] = ss; sh.part[16 + warp] = mx; }
    csync();
    float s2 = 0.f, m2 = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) { s2 += sh.part[w]; m2 = fmaxf(m2, sh.part[16 + w]); }
    const float inv = norm_w ? 1.0f / sqrtf(s2 / float(K) + eps) : 1.0f;
    m2 *= inv;
    // exact power-of-two scale that puts max|x| * 2^s in [2^29, 2^30): 31-bit signed fixed point
    float sc = 1.0f;
    if (m2 > 0.f && m2 < 3.0e38f) {
        const int E = int(__float_as_uint(m2) >> 23);  // biased exponent: m2 = f * 2^(E - 126), f in [0.5, 1)
        if (E >= 29) sc = __uint_as_float(uint32_t(283 - E) << 23);
        else { int ex = 0; frexpf(m2, &ex); sc = ldexpf(1.0f, 30 - ex); }
    }
    // balanced base-256 digits (see stage_finish)
#pragma unroll
    for (int it = 0; it < kStageItems; ++it) {
        if (it * kCT + (warp << 5) >= nitems) break;   // nothing left for this warp (warp-uniform)
        const int i = it * kCT + tid;
        const bool on = i < nitems;
        const int kbi = i >> 2, tt = i & 3;
        uint32_t y[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float v = (norm_w && it == 0) ? xv[it][q] * inv * nw[q] : xv[it][q];
            y[q] = uint32_t(__float2int_rn(v * sc)) + 0x80808080u;
        }
        int dsum[4] = {0, 0, 0, 0};
        if (on) {
            uint32_t w[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t a = __byte_perm(y[4 * h], y[4 * h + 1], 0x5140), b = __byte_perm(y[4 * h + 2], y[4 * h + 3], 0x5140);
                const uint32_t c = __byte_perm(y[4 * h], y[4 * h + 1], 0x7362), d = __byte_perm(y[4 * h + 2], y[4 * h + 3], 0x7362);
                w[h][0] = __byte_perm(a, b, 0x5410) ^ 0x80808080u;
                w[h][1] = __byte_perm(a, b, 0x7632) ^ 0x80808080u;
                w[h][2] = __byte_perm(c, d, 0x5410) ^ 0x80808080u;
                w[h][3] = __byte_perm(c, d, 0x7632) ^ 0x80808080u;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                dsum[c] = __dp4a(int(w[0][c]), 0x01010101, __dp4a(int(w[1][c]), 0x01010101, 0));
                xf[(kbi * 4 + c) * 4 + tt] = make_uint2(w[0][c], w[1][c]);
            }
        }
        if (QUANT == FORGE_Q4_0) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                dsum[c] += __shfl_xor_sync(0xffffffffu, dsum[c], 1);
                dsum[c] += __shfl_xor_sync(0xffffffffu, dsum[c], 2);
            }
            if (on && tt == 0) {
                xoff[2 * kbi] = make_int4(-8 * dsum[0], -8 * dsum[1], -128 * dsum[0], -128 * dsum[1]);
                xoff[2 * kbi + 1] = make_int4(-8 * dsum[2], -8 * dsum[3], -128 * dsum[2], -128 * dsum[3]);
            }
        }
    }
    csync();
    return 1.0f / sc;
}

// ---- epilogue of one finished output row (runtime-selected fusion)
// Operands that do not depend on the product, for the rows row0 (index 0) and row0 + 8 (index 1) of a thread.
struct EpiPre {
    float resid[2];  // EPI_RESID
    float bias[2][2];  // EPI_QKV: bias of (row, row + 1)
    float2 cs[2];    // EPI_QKV: rotation of the pair
    int pos, page;   // EPI_QKV: position and physical page of the new cache row
};

// pos_hint: the sequence position if the caller has already fetched it (saves a dependent load), else -1
template <bool TP>
__device__ __forceinline__ EpiPre epilogue_prefetch(const Phase& ph, int b, int row0, bool mine, int pos_hint) {
    EpiPre e;
    e.resid[0] = e.resid[1] = 0.f;
    e.bias[0][0] = e.bias[0][1] = e.bias[1][0] = e.bias[1][1] = 0.f;
    e.cs[0] = e.cs[1] = make_float2(1.f, 0.f);
    e.pos = 0; e.page = 0;
    if (!mine) return e;
    const GemvArgs& a = ph.a;
    if (ph.epi == EPI_RESID) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int row = row0 + 8 * j;
            if (row < ph.N) e.resid[j] = __ldcg(a.resid + size_t(b) * ph.N + row);
        }
    } else if (TP && ph.epi == EPI_TP_PUSH) {
        e.pos = int(__ldcg(a.tp.step_counter) * a.tp.step_mul + a.tp.step_add);  // the step this kernel publishes
    } else if (ph.epi == EPI_QKV && (row0 & 1) == 0) {
        e.pos = pos_hint >= 0 ? pos_hint : a.seq_len[b];
        e.page = a.page_table[size_t(b) * a.pages_per_seq + e.pos / FORGE_KV_PAGE];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int row = row0 + 8 * j;
            if (row >= ph.N) continue;
            if (a.bias) { e.bias[j][0] = a.bias[row]; e.bias[j][1] = a.bias[row + 1]; }
            if (row < a.qk + a.kv) {
                const int col = row < a.qk ? row : row - a.qk;
                e.cs[j] = reinterpret_cast<const float2*>(a.rope)[size_t(e.pos) * (a.head_dim / 2) + (col % a.head_dim) / 2];
            }
        }
    }
    return e;
}

template <bool TP>
__device__ __forceinline__ void epilogue_row(const Phase& ph, int b, int row, float v, float partner, const EpiPre& pre, int j) {
    if (row >= ph.N) return;
    const GemvArgs& a = ph.a;
    if (ph.epi == EPI_STORE) {
        a.out[size_t(b) * ph.N + row] = v;
    } else if (ph.epi == EPI_RESID) {
        a.out[size_t(b) * ph.N + row] = pre.resid[j] + v;
    } else if (TP && ph.epi == EPI_TP_PUSH) {
        const size_t off = (size_t(a.tp.slot) * a.tp.world + a.tp.rank) * ph.N + row;
        const uint2 pair = make_uint2(__float_as_uint(v), uint32_t(pre.pos));
        for (int r = 0; r < a.tp.world; ++r) a.tp.peer_ll[r][off] = pair;  // one 8-byte store: value and step together
    } else if (ph.epi == EPI_SILU) {
        if ((row & 1) == 0)  // rows interleaved at pack time: 2j = gate_j, 2j+1 = up_j
            a.out[size_t(b) * (ph.N / 2) + (row >> 1)] = (v / (1.0f + expf(-v))) * partner;
    } else if ((row & 1) == 0) {  // EPI_QKV: the thread of the even row handles the (even, odd) pair
        float q0 = v + pre.bias[j][0], q1 = partner + pre.bias[j][1];
        const int pos = pre.pos;
        const int qk = a.qk, kv = a.kv;
        int col = row, region = 0;
        if (col >= qk) { col -= qk; region = 1; }
        if (region == 1 && col >= kv) { col -= kv; region = 2; }
        if (region < 2) {
            const float2 cs = pre.cs[j];
            const float r0 = q0 * cs.x - q1 * cs.y, r1 = q0 * cs.y + q1 * cs.x;
            q0 = r0; q1 = r1;
        }
        if (region == 0) {
            *reinterpret_cast<float2*>(a.q_out + size_t(b) * qk + col) = make_float2(q0, q1);
        } else {
            __half* pool = region == 1 ? a.k_pool : a.v_pool;
            *reinterpret_cast<__half2*>(pool + (size_t(pre.page) * FORGE_KV_PAGE + pos % FORGE_KV_PAGE) * a.kv_stride + col) =
                __floats2half2_rn(q0, q1);
        }
    }
}

// ---- consumer side, step 2: all units of this CTA for one phase and one batch row.
// `on_row(row, value, partner)` is called by the finishing thread after the epilogue, `partner` being the value of
// row ^ 1; pass a no-op when there is nothing to add.  It is also called for the padding rows (row >= N).
// Row pair (row0, row0 + 8) a thread finishes in unit u, and whether it is the thread that runs the epilogue
// (shared by the consumer loop and by callers that fetch the first unit's epilogue operands ahead of time).
__device__ __forceinline__ void unit_rows(const Phase& ph, int u, int ui, int& row0, bool& mine) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bool wide = ph.bt == kBandTiles;
    const int r8 = wide ? warp % kBandTiles : 0, khalf = wide ? warp / kBandTiles : warp;
    int band, slice;
    unit_split(u, ph.slices, band, slice);
    row0 = (band * ph.bt + r8) * 16 + g;
    mine = t == 0 && (wide ? khalf == 0 : warp == ui % kConsumerWarps);
}

// pre_first: the first unit's epilogue operands if the caller has fetched them already (have_pre_first)
template <int QUANT, typename RowHook, bool TP = false>
__device__ __forceinline__ void consume_phase(const Phase& ph, Shared& sh, const unsigned char* ring, const uint2* xf,
                                              const int4* xoff, float unscale, int b, int& cc, RowHook on_row, int pos_hint = -1,
                                              bool have_pre_first = false, const EpiPre pre_first = EpiPre()) {
    using T = Tile<QUANT>;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int bt = ph.bt;
    const bool wide = bt == kBandTiles;
    const int kparts = wide ? kConsumerWarps / kBandTiles : kConsumerWarps;  // warps sharing one row tile
    const int r8 = wide ? warp % kBandTiles : 0;                              // row tile within the band
    const int khalf = wide ? warp / kBandTiles : warp;                        // k part of this warp
    const int KB = ph.kb;
    const int cshift = chunk_kb_shift<QUANT>(bt), ckb = 1 << cshift;
    const int chunks_per_band = (KB + ckb - 1) >> cshift;
    int ui = 0;
    for (int u = first_unit(ph, blockIdx.x, gridDim.x); u < ph.units; u += gridDim.x, ++ui) {
        int band, slice, c0, c1;
        unit_split(u, ph.slices, band, slice);
        slice_range(chunks_per_band, ph.slices, slice, c0, c1);
        const int rt = band * bt + r8;
        const int row0 = rt * 16 + g;  // and row0 + 8
        // operands of the epilogue that do not depend on the product are fetched now, under the tile loop
        // (the warp that will finish the unit: the even-k warp of the tile, or the unit's turn in the 16-row form)
        const EpiPre pre = (ui == 0 && have_pre_first) ? pre_first
                                                       : epilogue_prefetch<TP>(ph, b, row0, t == 0 && (wide ? khalf == 0 : warp == ui % kConsumerWarps), pos_hint);
        // per-lane accumulators: rows g / g+8 of this warp's row tile x digit columns 2t / 2t+1
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int c = c0; c < c1; ++c, ++cc) {
            const int st = cc % T::STAGES, use = cc / T::STAGES;
            if (!mbar_wait(&sh.full_bar[st], use & 1, &sh.err)) atomicExch(&sh.err, 1);
            const int kb0 = c * ckb;
            const int nkb = min(ckb, KB - kb0);
            const unsigned char* base = ring + size_t(st) * T::STAGE_BYTES + size_t(r8) * T::BYTES;
            auto tile = [&](int j) {  // k-block kb0 + j of this warp's row tile
                const unsigned char* tp = base + size_t(j) * (bt * T::BYTES);
                if (KQuant<QUANT>::value) {
                    // one int8 B column (the Q8_0 row); C columns 0 / 1 of lanes t == 0 carry the sums
                    const uint2 bx = xf[(kb0 + j) * 16 + t];
                    const float2 xs = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(xf) + (kb0 + j) * 32 + 8);
                    const float4 sc = *reinterpret_cast<const float4*>(tp + g * 16);
                    int cf[4] = {0, 0, 0, 0};
                    uint32_t a[4];
                    if (QUANT == FORGE_Q4_K) {
                        const uint2 wq = *reinterpret_cast<const uint2*>(tp + 128 + lane * 8);
                        a[0] = wq.x & 0x0F0F0F0Fu; a[1] = wq.x & 0xF0F0F0F0u;
                        a[2] = wq.y & 0x0F0F0F0Fu; a[3] = wq.y & 0xF0F0F0F0u;
                        imma16832_u8(cf, a, bx.x, bx.y);
                        // x_scale * (d*sc * dot - dmin*m * sum(q)); rows g+8 entered as 16 q, their scale as d*sc / 16
                        acc[0] += xs.x * (sc.x * float(cf[0]) - sc.y * xs.y);
                        acc[2] += xs.x * (sc.z * float(cf[2]) - sc.w * xs.y);
                    } else {
                        // column 0 sees k 0..15 only, column 1 k 16..31 only: the two 16-element scale groups
                        const uint4 wq = *reinterpret_cast<const uint4*>(tp + 128 + lane * 16);
                        a[0] = wq.x; a[1] = wq.y; a[2] = wq.z; a[3] = wq.w;
                        imma16832_s8(cf, a, (g & 1) ? 0u : bx.x, (g & 1) ? bx.y : 0u);
                        acc[0] += xs.x * (sc.x * float(cf[0]) + sc.y * float(cf[1]));
                        acc[2] += xs.x * (sc.z * float(cf[2]) + sc.w * float(cf[3]));
                    }
                    return;
                }
                // B fragment: digit column (g & 3); lanes g >= 4 duplicate columns whose results are never read
                const uint2 bx = xf[((kb0 + j) * 4 + (g & 3)) * 4 + t];
                const float2 d = __half22float2(*reinterpret_cast<const __half2*>(tp + g * 4));
                int cf[4];
                uint32_t a[4];
                if (QUANT == FORGE_Q4_0) {
                    const uint2 wq = *reinterpret_cast<const uint2*>(tp + 32 + lane * 8);
                    a[0] = wq.x & 0x0F0F0F0Fu; a[1] = wq.x & 0xF0F0F0F0u;
                    a[2] = wq.y & 0x0F0F0F0Fu; a[3] = wq.y & 0xF0F0F0F0u;
                    const int4 xo = xoff[2 * (kb0 + j) + (t & 1)];
                    cf[0] = xo.x; cf[1] = xo.y; cf[2] = xo.z; cf[3] = xo.w;
                    imma16832_u8(cf, a, bx.x, bx.y);
                } else {
                    const uint4 wq = *reinterpret_cast<const uint4*>(tp + 32 + lane * 16);
                    a[0] = wq.x; a[1] = wq.y; a[2] = wq.z; a[3] = wq.w;
                    cf[0] = cf[1] = cf[2] = cf[3] = 0;
                    imma16832_s8(cf, a, bx.x, bx.y);
                }
                acc[0] += d.x * float(cf[0]); acc[1] += d.x * float(cf[1]);
                acc[2] += d.y * float(cf[2]); acc[3] += d.y * float(cf[3]);
            };
            if (nkb == ckb) {  // full chunk: straight-line code, the tiles' loads and MMAs interleave
#pragma unroll
                for (int j = 0; j < T::CHUNK_KB / 2; ++j) tile(j * kparts + khalf);
            } else {
                for (int j = khalf; j < nkb; j += kparts) tile(j);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.empty_bar[st]);
        }
        // ---- the warp's part of this unit is complete: combine digits (quad lanes 0 and 1)
        const float wgt = (t == 0) ? 1.0f : 65536.0f;  // lane 0: digits 0,1; lane 1: digits 2,3 (base 256)
        const float w1 = (QUANT == FORGE_Q4_0) ? wgt * 0.0625f : wgt;  // Q4_0 rows g+8 were carried as 16 n
        float v0 = (acc[0] + 256.0f * acc[1]) * wgt, v1 = (acc[2] + 256.0f * acc[3]) * w1;
        if (KQuant<QUANT>::value) {
            v0 = t == 0 ? acc[0] : 0.f;  // the other quad lanes hold MMA columns nobody asked for
            v1 = t == 0 ? acc[2] : 0.f;
        }
        v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
        v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
        if (bt == kBandTiles) {
            // the two warps of a row tile (even / odd k-blocks) meet here: the odd one hands over its sums
            if (khalf == 1 && t == 0) { sh.pair[r8][g] = v0; sh.pair[r8][g + 8] = v1; }
            asm volatile("bar.sync %0, 64;" ::"r"(2 + r8) : "memory");
            if (khalf == 1) {
                asm volatile("bar.sync %0, 64;" ::"r"(2 + r8) : "memory");  // pair[] consumed
                continue;
            }
            v0 += sh.pair[r8][g];
            v1 += sh.pair[r8][g + 8];
            asm volatile("bar.sync %0, 64;" ::"r"(2 + r8) : "memory");
        } else {
            // All sixteen warps worked on the same row tile: one of them adds their sums and runs the epilogue, the
            // others go straight on to the next unit.  The duty rotates (unit ui -> warp ui % 16), so no warp is the
            // bottleneck, and nobody waits for the epilogue: the sums travel through red[ui & 1], guarded by two
            // pairs of named barriers in producer/consumer form -
            //   "full" (ids 12, 13): 15 warps arrive after writing, the finisher syncs before reading;
            //   "free" (ids 10, 11): the finisher arrives after reading, the other 15 warps sync before they write the
            //                        same buffer again two units later (only armed if that unit exists).
            const int par = ui & 1;
            const int fin = ui % kConsumerWarps;
            if (ui >= 2 && warp != (ui - 2) % kConsumerWarps) asm volatile("bar.sync %0, %1;" ::"r"(10 + par), "n"(kCT) : "memory");
            if (t == 0) { sh.red[par][warp][g] = v0; sh.red[par][warp][g + 8] = v1; }
            if (warp != fin) {
                asm volatile("bar.arrive %0, %1;" ::"r"(12 + par), "n"(kCT) : "memory");
                continue;
            }
            asm volatile("bar.sync %0, %1;" ::"r"(12 + par), "n"(kCT) : "memory");
            v0 = 0.f; v1 = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) { v0 += sh.red[par][w][g]; v1 += sh.red[par][w][g + 8]; }
            if (u + 2 * int(gridDim.x) < ph.units) asm volatile("bar.arrive %0, %1;" ::"r"(10 + par), "n"(kCT) : "memory");
        }
        v0 *= unscale;
        v1 *= unscale;
        bool finish = true;
        if (ph.epi == EPI_PARTIAL) {
            // raw partial sums of this K slice; whoever reads them adds the slices in order
            if (t == 0) {
                const size_t npad = size_t(ph.bands) * 16 * bt;
                ph.scratch[size_t(slice) * npad + row0] = v0;
                ph.scratch[size_t(slice) * npad + row0 + 8] = v1;
            }
            continue;
        }
        if (ph.slices > 1) {
            // split K: publish this slice's partial sums; the last slice to arrive adds all of them
            const size_t npad = size_t(ph.bands) * 16 * bt;
            if (t == 0) {
                ph.scratch[size_t(slice) * npad + row0] = v0;
                ph.scratch[size_t(slice) * npad + row0 + 8] = v1;
            }
            __threadfence();
            __syncwarp();
            int old = 0;
            if (lane == 0) old = atomicAdd(ph.tickets + rt, 1);
            old = __shfl_sync(0xffffffffu, old, 0);
            finish = (old == ph.slices - 1);
            if (finish) {
                __threadfence();
                if (lane == 0) ph.tickets[rt] = 0;  // ready for the next use
                // all loads are issued before the first add (one L2 round trip); the sum runs in slice
                // order, independent of which slice came last
                float p0[kGemvMaxSlices], p1[kGemvMaxSlices];
#pragma unroll
                for (int s = 0; s < kGemvMaxSlices; ++s) {
                    const bool in = s < ph.slices;
                    p0[s] = in ? __ldcg(ph.scratch + size_t(s) * npad + row0) : 0.f;
                    p1[s] = in ? __ldcg(ph.scratch + size_t(s) * npad + row0 + 8) : 0.f;
                }
                v0 = 0.f; v1 = 0.f;
#pragma unroll
                for (int s = 0; s < kGemvMaxSlices; ++s) { v0 += p0[s]; v1 += p1[s]; }
            }
        }
        // pair partners (rows r^1) live in the neighbouring quad
        const float o0 = __shfl_xor_sync(0xffffffffu, v0, 4), o1 = __shfl_xor_sync(0xffffffffu, v1, 4);
        if (finish && t == 0) {
            epilogue_row<TP>(ph, b, row0, v0, o0, pre, 0);
            epilogue_row<TP>(ph, b, row0 + 8, v1, o1, pre, 1);
            on_row(row0, v0, o0);
            on_row(row0 + 8, v1, o1);
        }
    }
}

// shared-memory bytes of the ring plus the activation fragments for the largest K in use
template <int QUANT>
inline size_t dyn_smem_bytes(int max_kb) { return size_t(Tile<QUANT>::STAGES) * Tile<QUANT>::STAGE_BYTES + size_t(max_kb) * 128; }

}  // namespace core
}  // namespace forge
