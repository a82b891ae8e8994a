// Load-time repack of raw GGUF Q8_0 / Q4_0 block rows into the aligned split layout the
// kernels stream (see QWeight): quant bytes verbatim in one array, f16 block scales in
// another.  Block semantics: crates/forgellm-frontend/src/weight_loader.rs:860-926.
// Also used for the tensor-parallel slices (a column slice of o/down is a strided gather of
// blocks from every row) and for interleaving gate/up rows so their SiLU epilogue sees both.
#include "common.cuh"

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
}  // namespace

int32_t pack_rows(const uint8_t* raw_dev, int quant, int K_full, int row0, int rows, int blk0, int blks,
                  QWeight& dst, int dst_row0, int row_step, cudaStream_t st) {
    if (dst.K != blks * 32 || dst.quant != quant) { set_error("pack_rows: destination shape mismatch"); return FORGE_ERR_SHAPE; }
    long total = long(rows) * blks;
    if (total == 0) return FORGE_OK;
    int grid = int((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (quant == FORGE_Q8_0)
        pack_kernel<FORGE_Q8_0><<<grid, 256, 0, st>>>(raw_dev, K_full / 32, row0, rows, blk0, blks, dst.qs, dst.d, dst_row0, row_step);
    else
        pack_kernel<FORGE_Q4_0><<<grid, 256, 0, st>>>(raw_dev, K_full / 32, row0, rows, blk0, blks, dst.qs, dst.d, dst_row0, row_step);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

}  // namespace forge
