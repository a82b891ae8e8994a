// Decode GEMV, streaming form (replaces matmul_vec_q8_0_KxN / matmul_vec_q4_0_KxN,
// crates/forgellm-codegen-cpu/src/emit.rs:2047-2087 and :2910-2953, with the reference's fusion
// patterns as prologue/epilogue: RMSNorm :327-334, residual :455-459, bias + RoPE + cache write
// :4108-4153, silu_mul :381-386).
//
// One persistent CTA per SM pulls its share of the weight stream with 1-D bulk copies (cp.async.bulk,
// completion on an mbarrier) into a ring of shared-memory stages, so the bytes in flight (~140 KB per
// SM) do not depend on the instruction stream.  Sixteen consumer warps turn every 16-row x 32-column
// tile (one quantisation block per row) into ONE integer tensor-core product, mma.sync m16n8k32
// s8/u8 x s8 -> s32:
//   A = the quantised weights as they are (Q8_0 bytes; Q4_0 nibbles split into bytes),
//   B = the f32 activation in fixed point, x * 2^s rounded to a 31-bit integer whose four balanced
//       base-256 digits (the bytes of x + 0x80808080, each minus 128) fill one B column each,
// so the 32-term integer dot products are exact; each digit's sum is converted to f32,
// multiplied by the row's f16 block scale and accumulated in f32, and the four digit
// accumulators are combined once per row.  The result is the reference's f32 arithmetic up to
// summation order (the activation keeps 2^-30 of its largest magnitude; it is never quantised
// to 8 bits).
//
// Units of work: a "wide" band is 128 rows (8 row tiles, two warps per tile taking the even / odd
// k-blocks, no CTA-level reduction); a "narrow" band is one row tile shared by all sixteen warps
// (16-row units for matrices too small to fill the SMs with 128-row bands; the warps' sums meet in
// shared memory and the finishing duty rotates over the warps).  Small matrices are also split along
// K over several CTAs ("slices"): every slice writes its partial sums to scratch and the warp that
// completes a row tile (atomic ticket) adds the slices in fixed order and runs the epilogue, so
// results do not depend on timing.
//
// Latency: a batch-1 decode step is a chain of short dependent kernels, so the kernel is launched
// with programmatic dependent launch (barrier set-up and the weight stream start under the previous
// kernel's tail, griddepcontrol.wait precedes the first dependent read), asks L2 for the next
// kernel's weights, and fetches its epilogue operands under the tile loop.  All decode GEMVs share
// this one kernel on purpose: its code stays in the instruction caches from launch to launch
// (specialising it per epilogue made the step 3 % slower, merging rarely used code into it 1-3 %).
//
// Weight layout ("tiled"): 16-row x 32-column tiles; a tile is {8 x half2 (d[row g], d[row g+8])}
// {quant bytes in A-fragment order, 16 (Q8_0) or 8 (Q4_0) bytes per lane} = 544 or 288 bytes:
// exactly the 34 / 18 bytes per block of the GGUF stream.  Tiles are ordered
// [128-row band][k-block][row tile within band], so a chunk (a run of k-blocks of one band) is
// one contiguous, 16-byte aligned bulk copy.
//
// K-quants (matmul_vec_q4_k_KxN / matmul_vec_q6_k_KxN, emit.rs:3411-3487 and :3636-3652) run through the same
// kernel: their 256-element super-blocks are re-tiled at load time into 16 x 32 tiles that carry the block's own
// f32 scale fields (see Tile in gemv_core.cuh), and the activation is staged as the Q8_0 blocks those functions
// quantise their input to (one int8 B column instead of four digit columns), so the integer dots are the
// reference's own.  Q6_K's two 16-element scale groups per block come out of ONE MMA: B column 0 holds k 0..15
// only and column 1 holds k 16..31 only.  Their pipeline stages hold 8 k-blocks (6 / 4 stages in the ring): a warp's
// per-stage work (barrier wait, arrive, loop) is then spread over four tiles instead of two.
#include <algorithm>
#include <cstdlib>

#include "gemv_core.cuh"
#include "kquant_decode.cuh"

namespace forge {

namespace {

using namespace core;

struct TcParams {
    Phase ph;
    int* err;  // device error word (set when a bounded wait gives up)
};

// TP: the instantiation that can take part in the tensor-parallel sums over peer memory (its extra code stays out
// of the single-GPU kernel: every decode kernel starts with a cold instruction cache, so size matters)
template <int QUANT, bool TP>
__global__ void __launch_bounds__(kThreads, 1) gemv_tc_kernel(TcParams p) {
    using T = Tile<QUANT>;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ Shared sh;
    __shared__ int4 s_xoff[QUANT == FORGE_Q4_0 ? 2 * kMaxKB : 1];
    unsigned char* ring = smem;
    uint2* xf = reinterpret_cast<uint2*>(smem + size_t(T::STAGES) * T::STAGE_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5;
    pdl_trigger();  // the next kernel may be scheduled; it waits for this one before it reads any result
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&sh.full_bar[s], 1); mbar_init(&sh.empty_bar[s], kConsumerWarps); }
        sh.err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const Phase& ph = p.ph;
    int cc = 0;
    // producer warp: streams this CTA's chunks, once per batch row, as fast as stages free up; it starts
    // right away because the weights do not depend on the activations being staged by the consumers
    if (warp == kConsumerWarps) {
        if ((tid & 31) == 0)
            for (int b = 0; b < ph.a.batch; ++b)
                if (!produce_phase<QUANT>(ph, sh, ring, cc, [&] { if (b == 0) l2_prefetch_share(ph.a.next_w, ph.a.next_bytes); })) break;
        return;
    }
    // everything above (and the producer's weight stream) is independent of earlier kernels; the activation is not
    pdl_wait();
    for (int b = 0; b < ph.a.batch; ++b) {
        // the position of the new cache row is needed late (epilogue) but heads a chain of dependent loads: ask now
        const int pos = ph.epi == EPI_QKV ? ph.a.seq_len[b] : -1;
        float unscale;
        EpiPre pre0 = EpiPre();
        bool have_pre0 = false;
        if (TP && ph.a.tp.consume) {
            // the input is a sum over the tensor-parallel ranks that arrives through peer stores (see GemvArgs::Tp)
            const GemvArgs::Tp& tp = ph.a.tp;
            const uint32_t step = __ldcg(tp.step_counter) * tp.step_mul + tp.step_add;
            const FillStat st = stage_fill_pairs(xf, ph.a.x, tp.ll + size_t(tp.slot) * tp.world * ph.K, tp.world, step, tp.x_writeback,
                                                 ph.K, ph.a.norm_w, &sh.err, tp.wait_limit);
            unscale = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, ph.a.norm_w, ph.a.eps);
        } else {
            bool staged = false;
            if constexpr (!KQuant<QUANT>::value) {
                if (stage_regs_ok(ph.K, ph.a.norm_w)) {
                    // the first unit's epilogue operands (residual, position -> page -> rotation) are asked for now, so
                    // their round trips run under the staging
                    const int u0 = first_unit(ph, blockIdx.x, gridDim.x);
                    if (u0 < ph.units) {
                        int row0;
                        bool mine;
                        unit_rows(ph, u0, 0, row0, mine);
                        pre0 = epilogue_prefetch<TP>(ph, b, row0, mine, pos);
                        have_pre0 = true;
                    }
                    unscale = stage_activation_regs<QUANT>(xf, s_xoff, sh, ph.a.x + size_t(b) * ph.K, ph.K, ph.a.norm_w, ph.a.eps, b == 0);
                    staged = true;
                }
            }
            if (!staged) unscale = stage_activation<QUANT, false>(xf, s_xoff, sh, ph.a.x + size_t(b) * ph.K, ph.K, ph.a.norm_w, ph.a.eps);
        }
        auto no_hook = [](int, float, float) {};
        consume_phase<QUANT, decltype(no_hook), TP>(ph, sh, ring, xf, s_xoff, unscale, b, cc, no_hook, pos, have_pre0, pre0);
    }
    csync();
    if (tid == 0 && sh.err && p.err) atomicExch(p.err, 1);
}

// ------------------------------------------------------------------ packing
// thread per (tile, lane): gathers the lane's A-fragment bytes from the two raw GGUF rows it owns
// (rows g and g+8 of the 16-row tile; k = 4t..4t+3 and 16+4t..16+4t+3 of the block)
template <int QUANT>
__global__ void tile_pack_kernel(const uint8_t* const* __restrict__ row_src, int KB, int bands, int bt, uint8_t* __restrict__ dst) {
    constexpr int BS = QUANT == FORGE_Q8_0 ? 34 : 18;
    using T = core::Tile<QUANT>;
    const long total = long(bands) * KB * bt * 32;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        const int lane = int(i & 31);
        const long tile = i >> 5;                      // ((band * KB + kb) * bt + r8)
        const int r8 = int(tile % bt);
        const int kb = int((tile / bt) % KB), band = int(tile / (long(bt) * KB));
        const int rt = band * bt + r8;
        const int g = lane >> 2, t = lane & 3;
        const uint8_t* r0 = row_src[rt * 16 + g];
        const uint8_t* r1 = row_src[rt * 16 + g + 8];
        if (QUANT == FORGE_Q4_K) {
            uint8_t* tp = dst + size_t(tile) * T::BYTES;
            const KBlock4 b0 = kblock_q4_k(r0, kb), b1 = kblock_q4_k(r1, kb);
            if (t == 0) *reinterpret_cast<float4*>(tp + g * 16) = make_float4(b0.s, b0.mn, b1.s * 0.0625f, b1.mn);
            uint32_t w[2] = {0u, 0u};
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int k = h * 16 + 4 * t + j;  // byte j: low nibble = row g, high nibble = row g+8
                    const uint32_t q0 = b0.q(k), q1 = b1.q(k);
                    w[h] |= (q0 | (q1 << 4)) << (8 * j);
                }
            *reinterpret_cast<uint2*>(tp + 128 + lane * 8) = make_uint2(w[0], w[1]);
            continue;
        }
        if (QUANT == FORGE_Q6_K) {
            uint8_t* tp = dst + size_t(tile) * T::BYTES;
            const KBlock6 b0 = kblock_q6_k(r0, kb), b1 = kblock_q6_k(r1, kb);
            if (t == 0) *reinterpret_cast<float4*>(tp + g * 16) = make_float4(b0.s_lo, b0.s_hi, b1.s_lo, b1.s_hi);
            auto q6 = [](const KBlock6& b, int l) -> uint32_t { return uint32_t(b.q(l)) & 255u; };
            uint32_t w[4] = {0u, 0u, 0u, 0u};  // a0: row g, k lo; a1: row g+8, k lo; a2: row g, k hi; a3: row g+8, k hi
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int k = h * 16 + 4 * t + j;
                    w[2 * h] |= q6(b0, k) << (8 * j);
                    w[2 * h + 1] |= q6(b1, k) << (8 * j);
                }
            *reinterpret_cast<uint4*>(tp + 128 + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            continue;
        }
        const uint8_t* b0 = r0 ? r0 + size_t(kb) * BS : nullptr;
        const uint8_t* b1 = r1 ? r1 + size_t(kb) * BS : nullptr;
        uint8_t* tp = dst + size_t(tile) * T::BYTES;
        if (t == 0) {
            uint16_t d0 = b0 ? uint16_t(b0[0] | (b0[1] << 8)) : 0, d1 = b1 ? uint16_t(b1[0] | (b1[1] << 8)) : 0;
            *reinterpret_cast<uint32_t*>(tp + g * 4) = uint32_t(d0) | (uint32_t(d1) << 16);
        }
        // element k of a block: Q8_0 byte 2+k; Q4_0 byte 2 + (k & 15), low nibble for k < 16 else high
        auto q8 = [&](const uint8_t* blk, int k) -> uint32_t { return blk ? uint32_t(blk[2 + k]) : 0u; };
        auto q4 = [&](const uint8_t* blk, int k) -> uint32_t { return blk ? uint32_t((blk[2 + (k & 15)] >> ((k >> 4) * 4)) & 15u) : 8u; };
        if (QUANT == FORGE_Q4_0) {
            uint32_t w[2] = {0u, 0u};
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int k = h * 16 + 4 * t + j;  // byte j: low nibble = row g, high nibble = row g+8
                    w[h] |= (q4(b0, k) | (q4(b1, k) << 4)) << (8 * j);
                }
            *reinterpret_cast<uint2*>(tp + 32 + lane * 8) = make_uint2(w[0], w[1]);
        } else {
            uint32_t w[4] = {0u, 0u, 0u, 0u};  // a0: row g, k lo; a1: row g+8, k lo; a2: row g, k hi; a3: row g+8, k hi
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int k = h * 16 + 4 * t + j;
                    w[2 * h] |= q8(b0, k) << (8 * j);
                    w[2 * h + 1] |= q8(b1, k) << (8 * j);
                }
            *reinterpret_cast<uint4*>(tp + 32 + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

template <int QUANT>
int32_t launch(const QTiled& w, GemvEpilogue epi, const GemvArgs& a, const GemvSplit& sp, int* err, cudaStream_t st) {
    using T = Tile<QUANT>;
    TcParams p;
    Phase& ph = p.ph;
    ph.w = w.data; ph.K = w.K; ph.N = w.N; ph.kb = w.K / 32; ph.bands = w.bands; ph.bt = w.bt; ph.a = a; ph.epi = epi; ph.rot = 0;
    p.err = err;
    const size_t smem = dyn_smem_bytes<QUANT>(ph.kb);
    if (smem > 220 * 1024 || ph.kb > kMaxKB) { set_error("gemv: K=%d is beyond the supported %d", w.K, kMaxKB * 32); return FORGE_ERR_SHAPE; }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    ph.slices = gemv_slices(w, sp, sms, a.batch);
    ph.units = w.bands * ph.slices;
    ph.scratch = sp.scratch;
    ph.tickets = sp.tickets;
    const int grid = ph.units < sms ? ph.units : sms;
    // one limit for every launch of this kernel: a launch replayed later (a graph node re-issued by a profiler) must
    // not find a smaller limit left behind by another matrix
    const bool tp = !KQuant<QUANT>::value && (a.tp.consume || epi == EPI_TP_PUSH);
    auto kern = tp ? gemv_tc_kernel<QUANT, !KQuant<QUANT>::value> : gemv_tc_kernel<QUANT, false>;
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn_smem_bytes<QUANT>(kMaxKB))));
    FORGE_CUDA(launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, p));
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace

// K slices per band: split (ticketed cross-CTA reduction) only when the matrix has so few bands that at
// least half of the SMs would idle; one batch row only (the scratch holds one row), never finer than one
// pipeline chunk.
int gemv_slices(const QTiled& w, const GemvSplit& sp, int sms, int batch) {
    const int ckb = (w.quant == FORGE_Q8_0 ? 4 : 8) * (core::kBandTiles / w.bt);
    const int chunks = (w.K / 32 + ckb - 1) / ckb;
    if (!sp.scratch || !sp.tickets || batch != 1 || 2 * w.bands > sms) return 1;
    int slices = (sms + w.bands - 1) / w.bands;
    slices = std::min({slices, chunks, sp.max_slices, kGemvMaxSlices});
    return slices < 1 ? 1 : slices;
}

// Row tiles per band for an N-row matrix.  The wide form (8 tiles = 128 rows per band, two warps per tile, no
// CTA-level reduction per unit) streams fastest but comes in coarse units; it is used when whole rounds of 128-row
// bands keep at least 80 % of the SMs busy.  Otherwise one tile per band (16-row units, all warps share the tile).
int gemv_band_tiles(int N, int sms) {
    const int wide = (N + 127) / 128;
    const int rounds = (wide + sms - 1) / sms;
    return (5 * wide >= 4 * rounds * sms) ? core::kBandTiles : 1;
}

size_t qtiled_bytes(int quant, int K, int N, int bt) {
    const size_t bands = size_t((N + 16 * bt - 1) / (16 * bt));
    const size_t tile = quant == FORGE_Q4_0 ? 288 : quant == FORGE_Q8_0 ? 544 : quant == FORGE_Q4_K ? 384 : 640;
    return bands * bt * size_t(K / 32) * tile;
}

int32_t tile_pack(const uint8_t* const* row_src_dev, QTiled& dst, cudaStream_t st) {
    const long total = long(dst.bands) * (dst.K / 32) * dst.bt * 32;
    if (total == 0) return FORGE_OK;
    const int grid = int((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
    if (dst.quant == FORGE_Q8_0) tile_pack_kernel<FORGE_Q8_0><<<grid, 256, 0, st>>>(row_src_dev, dst.K / 32, dst.bands, dst.bt, dst.data);
    else if (dst.quant == FORGE_Q4_0) tile_pack_kernel<FORGE_Q4_0><<<grid, 256, 0, st>>>(row_src_dev, dst.K / 32, dst.bands, dst.bt, dst.data);
    else if (dst.quant == FORGE_Q4_K) tile_pack_kernel<FORGE_Q4_K><<<grid, 256, 0, st>>>(row_src_dev, dst.K / 32, dst.bands, dst.bt, dst.data);
    else tile_pack_kernel<FORGE_Q6_K><<<grid, 256, 0, st>>>(row_src_dev, dst.K / 32, dst.bands, dst.bt, dst.data);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

int32_t gemv_tc(const QTiled& w, GemvEpilogue epi, const GemvArgs& a, const GemvSplit& sp, int* err, cudaStream_t st) {
    if (w.K % 32 != 0 || w.K <= 0 || w.N <= 0) { set_error("gemv: K=%d must be a positive multiple of 32", w.K); return FORGE_ERR_SHAPE; }
    if ((epi == EPI_SILU || epi == EPI_QKV) && (w.N % 2)) { set_error("gemv: paired epilogue needs even N"); return FORGE_ERR_SHAPE; }
    if (core::is_kquant(w.quant)) {
        if (w.K % 256) { set_error("gemv: K=%d must be a multiple of 256 for K-quants", w.K); return FORGE_ERR_SHAPE; }
        if (a.tp.consume || epi == EPI_TP_PUSH) { set_error("gemv: K-quants take no part in the tensor-parallel sums"); return FORGE_ERR_UNSUPPORTED; }
        return w.quant == FORGE_Q4_K ? launch<FORGE_Q4_K>(w, epi, a, sp, err, st) : launch<FORGE_Q6_K>(w, epi, a, sp, err, st);
    }
    return w.quant == FORGE_Q8_0 ? launch<FORGE_Q8_0>(w, epi, a, sp, err, st) : launch<FORGE_Q4_0>(w, epi, a, sp, err, st);
}

}  // namespace forge
