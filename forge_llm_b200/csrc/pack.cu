// Load-time repack of raw GGUF Q8_0 / Q4_0 block rows into the aligned split layout the
// kernels stream (see QWeight): quant bytes verbatim in one array, f16 block scales in
// another.  Block semantics: crates/forgellm-frontend/src/weight_loader.rs:860-926.
// Also used for the tensor-parallel slices (a column slice of o/down is a strided gather of
// blocks from every row) and for interleaving gate/up rows so their SiLU epilogue sees both.
#include "common.cuh"
#include "kquant_decode.cuh"

namespace forge {

namespace {
template <int QUANT>
__global__ void pack_kernel(const uint8_t* __restrict__ raw, int nblk_full, int row0, int rows, int blk0, int blks,
                            uint8_t* __restrict__ qs, __half* __restrict__ d, int dst_row0, int row_step) {
    constexpr int BS = QUANT == FORGE_Q8_0 ? 34 : 18, QB = BS - 2;
    long total = long(rows) * blks;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        int r = int(i / blks), j = int(i % blks);
        const uint8_t* src = raw + (size_t(row0 + r) * nblk_full + blk0 + j) * BS;
        int drow = dst_row0 + r * row_step;
        uint16_t hb = uint16_t(src[0]) | (uint16_t(src[1]) << 8);
        d[size_t(drow) * blks + j] = __ushort_as_half(hb);
        uint16_t* dq = reinterpret_cast<uint16_t*>(qs + (size_t(drow) * blks + j) * QB);
        const uint16_t* sq = reinterpret_cast<const uint16_t*>(src + 2);  // blocks are 2-byte aligned
#pragma unroll
        for (int t = 0; t < QB / 2; ++t) dq[t] = sq[t];
    }
}
// raw K-quant rows -> FORGE_KQ_SOA: thread per (row, 32-element block)
template <int QUANT>
__global__ void pack_kq_kernel(const uint8_t* __restrict__ raw, int K_full, int row0, int rows, uint8_t* __restrict__ qs,
                               float4* __restrict__ sf, int dst_row0, int row_step) {
    const int blks = K_full / 32;
    const size_t row_bytes = size_t(K_full / 256) * (QUANT == FORGE_Q4_K ? 144 : 210);
    long total = long(rows) * blks;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        const int r = int(i / blks), kb = int(i % blks);
        const uint8_t* row = raw + size_t(row0 + r) * row_bytes;
        const int drow = dst_row0 + r * row_step;
        uint32_t w[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        float4 f;
        if (QUANT == FORGE_Q4_K) {
            const KBlock4 b = kblock_q4_k(row, kb);
            for (int k = 0; k < 32; ++k) w[k >> 2] |= b.q(k) << (8 * (k & 3));
            f = make_float4(b.s, b.s, b.mn, 0.f);
        } else {
            const KBlock6 b = kblock_q6_k(row, kb);
            for (int k = 0; k < 32; ++k) w[k >> 2] |= (uint32_t(b.q(k)) & 255u) << (8 * (k & 3));
            f = make_float4(b.s_lo, b.s_hi, 0.f, 0.f);
        }
        uint4* dq = reinterpret_cast<uint4*>(qs + (size_t(drow) * blks + kb) * 32);
        dq[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dq[1] = make_uint4(w[4], w[5], w[6], w[7]);
        sf[size_t(drow) * blks + kb] = f;
    }
}
}  // namespace

int32_t pack_rows(const uint8_t* raw_dev, int quant, int K_full, int row0, int rows, int blk0, int blks,
                  QWeight& dst, int dst_row0, int row_step, cudaStream_t st) {
    const bool kq = quant == FORGE_Q4_K || quant == FORGE_Q6_K;
    if (dst.K != blks * 32 || dst.quant != (kq ? FORGE_KQ_SOA : quant) || (kq && (blk0 != 0 || blks * 32 != K_full))) { set_error("pack_rows: destination shape mismatch"); return FORGE_ERR_SHAPE; }
    long total = long(rows) * blks;
    if (total == 0) return FORGE_OK;
    int grid = int((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (kq) {
        if (quant == FORGE_Q4_K) pack_kq_kernel<FORGE_Q4_K><<<grid, 256, 0, st>>>(raw_dev, K_full, row0, rows, dst.qs, dst.sf, dst_row0, row_step);
        else pack_kq_kernel<FORGE_Q6_K><<<grid, 256, 0, st>>>(raw_dev, K_full, row0, rows, dst.qs, dst.sf, dst_row0, row_step);
        FORGE_LAUNCH_CHECK();
        return FORGE_OK;
    }
    if (quant == FORGE_Q8_0)
        pack_kernel<FORGE_Q8_0><<<grid, 256, 0, st>>>(raw_dev, K_full / 32, row0, rows, blk0, blks, dst.qs, dst.d, dst_row0, row_step);
    else
        pack_kernel<FORGE_Q4_0><<<grid, 256, 0, st>>>(raw_dev, K_full / 32, row0, rows, blk0, blks, dst.qs, dst.d, dst_row0, row_step);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace forge
