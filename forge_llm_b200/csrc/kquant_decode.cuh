// Field decoding of raw K-quant super-blocks, shared by the two load-time repackers (tiles for the streaming GEMV
// in gemv_tc.cu, the row-major layout of the batched GEMM in pack.cu).  Every product below is an f16 times a small
// integer and therefore exact in f32.
#pragma once

#include "common.cuh"

namespace forge {

__device__ __forceinline__ float kq_f16_at(const uint8_t* p) { return __half2float(__ushort_as_half(uint16_t(p[0] | (p[1] << 8)))); }

// One 32-element block (k-block kb of the row) of a raw K-quant row, as the fields a consumer needs.
// Q4_K (emit.rs:3013-3021, :3246-3303): sub-block j = kb % 8 of super-block kb / 8; s = d * sc_j, mn = dmin * m_j;
// element k is the low (j even) or high (j odd) nibble of qs[(j / 2) * 32 + k].
struct KBlock4 {
    float s = 0.f, mn = 0.f; const uint8_t* qs = nullptr; int shift = 0;
    __device__ __forceinline__ uint32_t q(int k) const { return qs ? (qs[k] >> shift) & 15u : 0u; }
};
__device__ __forceinline__ KBlock4 kblock_q4_k(const uint8_t* row, int kb) {
    KBlock4 b;
    if (!row) return b;
    const uint8_t* sb = row + size_t(kb >> 3) * 144;
    const int j = kb & 7;
    const uint8_t* sc = sb + 4;
    int s6, m6;
    if (j < 4) { s6 = sc[j] & 63; m6 = sc[j + 4] & 63; }
    else { s6 = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); m6 = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
    b.s = kq_f16_at(sb) * float(s6);
    b.mn = kq_f16_at(sb + 2) * float(m6);
    b.qs = sb + 16 + (j >> 1) * 32;
    b.shift = (j & 1) * 4;
    return b;
}
// Q6_K (emit.rs:3560-3607): block j = kb % 8 reads ql[ql_off + l] >> nib and qh[qh_off + l] >> hsh; scale groups 2j, 2j+1.
struct KBlock6 {
    float s_lo = 0.f, s_hi = 0.f; const uint8_t* ql = nullptr; const uint8_t* qh = nullptr; int nib = 0, hsh = 0;
    __device__ __forceinline__ int q(int l) const {  // the signed value q6 - 32
        return ql ? int(((ql[l] >> nib) & 0x0F) | (((qh[l] >> hsh) & 3) << 4)) - 32 : 0;
    }
};
__device__ __forceinline__ KBlock6 kblock_q6_k(const uint8_t* row, int kb) {
    KBlock6 b;
    if (!row) return b;
    const uint8_t* sb = row + size_t(kb >> 3) * 210;
    const int j = kb & 7;
    const float d = kq_f16_at(sb + 208);
    b.s_lo = d * float(int(int8_t(sb[192 + 2 * j])));
    b.s_hi = d * float(int(int8_t(sb[192 + 2 * j + 1])));
    b.ql = sb + (j >> 2) * 64 + (j & 1) * 32;
    b.qh = sb + 128 + (j >> 2) * 32;
    b.nib = ((j >> 1) & 1) * 4;
    b.hsh = (j & 3) * 2;
    return b;
}

}  // namespace forge
