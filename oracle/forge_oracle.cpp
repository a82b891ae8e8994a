// forge_oracle.cpp — CPU oracle for the quantized transformer forward path.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain C++, the arithmetic of the
// Rust source that ForgeLLM's CPU code generator emits (the `#[cfg(not(target_arch =
// "aarch64"))]` branch, which is the one an x86_64 host executes).  It is the checker
// the CUDA path is compared against; nothing in the shipped library links, imports or
// calls it.  Every function cites the reference range it follows
// (E = crates/forgellm-codegen-cpu/src/emit.rs, P = crates/forgellm-codegen-cpu/src/project.rs,
//  WL = crates/forgellm-frontend/src/weight_loader.rs).
//
// Pinning status: the element-level pieces (f16 conversion, Q8_0/Q4_0 block semantics,
// quantisers, flash-vs-plain attention agreement, int8 KV round trip, argmax) are pinned
// by the reference's own known-answer tests, reproduced in tests/.  The composed path
// (a quantised matmul value, attention_flash_batch, logits of a whole model) has no
// golden value in the reference's tests and the reference (Rust) cannot be built where
// this oracle runs, so for the composed path: PARITY UNPINNED.
//
// Floating-point discipline: every reduction is a sequential f32 sum in the reference's
// loop order, multiplies and adds are separate roundings (compile with -ffp-contract=off),
// `round` is half-away-from-zero (Rust f32::round), exp/sin/cos/pow come from libm.
// Threads (OpenMP) only split independent outputs (rows, heads, tokens), as rayon does
// in the reference, so results do not depend on the thread count.

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>
#include <algorithm>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr int kFlashBlock = 64;  // FLASH_ATTN_BLOCK_SIZE, E:199-202
constexpr int kQTile = 16;       // Q_TILE, E:762

// ---------------------------------------------------------------- f16 <-> f32
// E:1246-1264 / WL:1326-1357: field-by-field widening, subnormals renormalised.
inline float f16_bits_to_f32(uint16_t h) {
    uint32_t s = (h >> 15) & 1u, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, out;
    if (e == 0) {
        if (m == 0) {
            out = s << 31;
        } else {
            int ex = -14;
            while ((m & 0x400u) == 0) { m <<= 1; --ex; }
            m &= 0x3FFu;
            out = (s << 31) | ((uint32_t(ex + 127) & 0xFFu) << 23) | (m << 13);
        }
    } else if (e == 31) {
        out = (s << 31) | (0xFFu << 23) | (m << 13);
    } else {
        out = (s << 31) | ((e - 15 + 127) << 23) | (m << 13);
    }
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}

// WL:1361-1442: round-to-nearest-even narrowing; f32 subnormals flush to signed zero,
// magnitudes past 2^16 go to infinity, NaN keeps a non-zero mantissa.
inline uint16_t f32_to_f16_bits(float x) {
    uint32_t b;
    std::memcpy(&b, &x, 4);
    uint32_t s = (b >> 31) & 1u;
    int e = int((b >> 23) & 0xFFu);
    uint32_t man = b & 0x7FFFFFu;
    if (e == 0xFF) {
        uint32_t hm = (man >> 13) & 0x3FFu;
        if (man != 0 && hm == 0) hm = 1;
        return uint16_t((s << 15) | (0x1Fu << 10) | hm);
    }
    if (e == 0) return uint16_t(s << 15);
    int ub = e - 127;
    if (ub > 15) return uint16_t((s << 15) | (0x1Fu << 10));
    if (ub < -24) return uint16_t(s << 15);
    uint32_t full = man | 0x800000u;
    uint32_t shift = (ub < -14) ? uint32_t(-1 - ub) : 13u;
    uint32_t dropped = full & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    uint32_t t = full >> shift;
    if (dropped > half || (dropped == half && (t & 1u))) t += 1;
    if (ub < -14) {
        if (t >= 0x400u) return uint16_t((s << 15) | (1u << 10));
        return uint16_t((s << 15) | t);
    }
    uint32_t he = uint32_t(ub + 15);
    if (t >= 0x800u) {
        he += 1;
        if (he >= 0x1Fu) return uint16_t((s << 15) | (0x1Fu << 10));
        return uint16_t((s << 15) | (he << 10));
    }
    return uint16_t((s << 15) | (he << 10) | (t & 0x3FFu));
}

// Rust `f32::round`: half away from zero == C roundf.
inline float rround(float v) { return roundf(v); }

// ---------------------------------------------------------------- block dots
// E:1359-1377: f32 activation x (int8 * f16 scale), one running f32 sum over the row.
float dot_q8_0(const float* in, const uint8_t* row, int k) {
    int nb = (k + 31) / 32;
    float sum = 0.0f;
    for (int b = 0; b < nb; ++b) {
        const uint8_t* blk = row + size_t(b) * 34;
        float d = f16_bits_to_f32(uint16_t(blk[0] | (blk[1] << 8)));
        int lim = std::min(32, k - b * 32);
        for (int j = 0; j < lim; ++j) {
            float w = float(int8_t(blk[2 + j])) * d;
            sum += in[b * 32 + j] * w;
        }
    }
    return sum;
}

// E:2337-2359: byte j carries element j (low nibble) and element j+16 (high nibble),
// value = nibble - 8; the sum visits lo then hi for each byte.
float dot_q4_0(const float* in, const uint8_t* row, int k) {
    int nb = (k + 31) / 32;
    float sum = 0.0f;
    for (int b = 0; b < nb; ++b) {
        const uint8_t* blk = row + size_t(b) * 18;
        float d = f16_bits_to_f32(uint16_t(blk[0] | (blk[1] << 8)));
        for (int j = 0; j < 16; ++j) {
            uint8_t by = blk[2 + j];
            int lo = int(by & 0x0F) - 8, hi = int(by >> 4) - 8;
            int il = b * 32 + j, ih = il + 16;
            if (il < k) sum += in[il] * (float(lo) * d);
            if (ih < k) sum += in[ih] * (float(hi) * d);
        }
    }
    return sum;
}

// Row-vectorised twin of the two dots: 16 output rows advance together, lane r of every
// vector holding row r's own sequential sum, so each lane performs exactly the scalar
// sequence above and the results are bit-identical.  The dequantised 16-row x 32-element
// tile (the reference's `q as f32 * scale` products) is formed once and reused for all m
// input rows.  Only used to make large parity cases finish quickly; the timed CPU
// baseline uses the scalar loops.
template <int QUANT>
void mat16_rows(const float* in, int m, int k, const uint8_t* w, size_t row_bytes, int rows,
                float* out, int n_stride) {
    constexpr int BS = (QUANT == 8) ? 34 : 18;
    int nb = k / 32;
    std::vector<float> accv(size_t(m) * 16, 0.0f);
    alignas(64) float wt[32][16];
    for (int b = 0; b < nb; ++b) {
        for (int r = 0; r < 16; ++r) {
            if (r < rows) {
                const uint8_t* blk = w + size_t(r) * row_bytes + size_t(b) * BS;
                float d = f16_bits_to_f32(uint16_t(blk[0] | (blk[1] << 8)));
                if (QUANT == 8) {
                    for (int j = 0; j < 32; ++j) wt[j][r] = float(int8_t(blk[2 + j])) * d;
                } else {
                    // visit order of dot_q4_0: (j, j+16) pairs -> slots 2j, 2j+1
                    for (int j = 0; j < 16; ++j) {
                        uint8_t by = blk[2 + j];
                        wt[2 * j][r] = float(int(by & 0x0F) - 8) * d;
                        wt[2 * j + 1][r] = float(int(by >> 4) - 8) * d;
                    }
                }
            } else {
                for (int j = 0; j < 32; ++j) wt[j][r] = 0.0f;
            }
        }
        for (int t = 0; t < m; ++t) {
            const float* __restrict x = in + size_t(t) * k + b * 32;
            float* __restrict accp = &accv[size_t(t) * 16];
            float acc[16];
            for (int r = 0; r < 16; ++r) acc[r] = accp[r];
            if (QUANT == 8) {
                for (int j = 0; j < 32; ++j) {
                    float xv = x[j];
#pragma omp simd
                    for (int r = 0; r < 16; ++r) acc[r] += xv * wt[j][r];
                }
            } else {
                for (int j = 0; j < 16; ++j) {
                    float xl = x[j], xh = x[j + 16];
#pragma omp simd
                    for (int r = 0; r < 16; ++r) acc[r] += xl * wt[2 * j][r];
#pragma omp simd
                    for (int r = 0; r < 16; ++r) acc[r] += xh * wt[2 * j + 1][r];
                }
            }
            for (int r = 0; r < 16; ++r) accp[r] = acc[r];
        }
    }
    for (int t = 0; t < m; ++t)
        for (int r = 0; r < rows; ++r) out[size_t(t) * n_stride + r] = accv[size_t(t) * 16 + r];
}

inline size_t row_bytes_of(int quant, int k) {
    if (quant == 12 || quant == 14) return size_t(k / 256) * (quant == 12 ? 144 : 210);
    return size_t((k + 31) / 32) * (quant == 8 ? 34 : 18);
}
void matmul_vec_kquant(int quant, float* out, const float* in, const uint8_t* w, int k, int n);

// E:2047-2087 (Q8_0) / E:2910-2953 (Q4_0): one dot per output row.
void matmul_vec(int quant, float* out, const float* in, const uint8_t* w, int k, int n) {
    size_t rb = row_bytes_of(quant, k);
    for (int j = 0; j < n; ++j)
        out[j] = (quant == 8) ? dot_q8_0(in, w + size_t(j) * rb, k) : dot_q4_0(in, w + size_t(j) * rb, k);
}

// E:2278-2299 / E:3792-3813: the non-aarch64 batched matmul runs the per-token GEMV once
// per input row.  Rows and row chunks are independent, so they are split over threads
// (the reference splits rows in chunks of 256 through rayon, E:2053).  `fast` selects the
// row-vectorised twin (same values).
void matmul_mat(int quant, float* out, int m, const float* in, const uint8_t* w, int k, int n, bool fast) {
    if (quant == 12 || quant == 14) {  // K-quants: the per-token product, row by row (there is no batched form)
        for (int r = 0; r < m; ++r) matmul_vec_kquant(quant, out + size_t(r) * n, in + size_t(r) * k, w, k, n);
        return;
    }
    size_t rb = row_bytes_of(quant, k);
    if (fast && (k % 32) == 0) {
        int groups = (n + 15) / 16;
#pragma omp parallel for schedule(dynamic, 4)
        for (int gi = 0; gi < groups; ++gi) {
            int j0 = gi * 16, rows = std::min(16, n - j0);
            if (quant == 8) mat16_rows<8>(in, m, k, w + size_t(j0) * rb, rb, rows, out + j0, n);
            else mat16_rows<4>(in, m, k, w + size_t(j0) * rb, rb, rows, out + j0, n);
        }
        return;
    }
    const int chunk = 256;
    int nchunks = (n + chunk - 1) / chunk;
    long total = long(m) * nchunks;
#pragma omp parallel for schedule(dynamic, 1)
    for (long it = 0; it < total; ++it) {
        int c = int(it / m), r = int(it % m);  // chunk-major so a weight chunk stays cached
        int j0 = c * chunk, cnt = std::min(chunk, n - j0);
        matmul_vec(quant, out + size_t(r) * n + j0, in + size_t(r) * k, w + size_t(j0) * rb, k, cnt);
    }
}

// ---------------------------------------------------------------- K-quants (per-token products only)
// The generated module has no batched K-quant product: every matmul_vec_q4_k / matmul_vec_q6_k call first
// quantises its input row to Q8_0 blocks (E:3413-3416, E:3636-3640) and then takes one integer dot per
// output row against the 256-element super-blocks.

// E:1412-1440 (also WL `quantize_f32_to_q8_0`): per 32 values, scale = absmax / 127 stored as f16 (1.0 for an
// all-zero block), q = round-half-away(x * (1 / scale)) clamped to [-127, 127].  Returns the scales as the f32
// values the dots read back from the f16 bits.
void quantize_act_q8_0(const float* in, int k, int8_t* q, float* scale) {
    int nb = (k + 31) / 32;
    for (int b = 0; b < nb; ++b) {
        int lim = std::min(32, k - b * 32);
        float absmax = 0.0f;
        for (int j = 0; j < lim; ++j) absmax = std::max(absmax, std::fabs(in[b * 32 + j]));
        float s = 1.0f, inv = 0.0f;
        if (absmax != 0.0f) { s = absmax / 127.0f; inv = 1.0f / s; }
        scale[b] = f16_bits_to_f32(f32_to_f16_bits(s));
        for (int j = 0; j < 32; ++j) {
            float v = j < lim ? rround(in[b * 32 + j] * inv) : 0.0f;
            q[b * 32 + j] = int8_t(std::min(127.0f, std::max(-127.0f, v)));
        }
    }
}

// E:3013-3021: the 6-bit (scale, min) pair of sub-block j from the 12 packed bytes.
inline void scale_min_k4(int j, const uint8_t* sc, int& s, int& m) {
    if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
    else { s = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
}

// E:3246-3303: Q4_K super-block = {f16 d, f16 dmin, 12 scale bytes, 128 nibble bytes}; 64-element chunk c holds
// sub-block 2c in the low nibbles and 2c+1 in the high nibbles of qs[32c .. 32c+31].
float dot_q4_k_q8_0(const uint8_t* row, const int8_t* xq, const float* xs, int k) {
    float acc = 0.0f;
    for (int sb = 0; sb < k / 256; ++sb) {
        const uint8_t* blk = row + size_t(sb) * 144;
        float d = f16_bits_to_f32(uint16_t(blk[0] | (blk[1] << 8)));
        float dmin = f16_bits_to_f32(uint16_t(blk[2] | (blk[3] << 8)));
        const uint8_t* qs = blk + 16;
        for (int chunk = 0; chunk < 4; ++chunk) {
            for (int half = 0; half < 2; ++half) {
                int is = chunk * 2 + half, sc, mn;
                scale_min_k4(is, blk + 4, sc, mn);
                float dw = d * float(sc), mw = dmin * float(mn);
                const int8_t* x = xq + (size_t(sb) * 8 + is) * 32;
                int dot = 0, sum = 0;
                for (int i = 0; i < 32; ++i) {
                    int q4 = half ? (qs[chunk * 32 + i] >> 4) : (qs[chunk * 32 + i] & 0x0F);
                    dot += int(x[i]) * q4;
                    sum += int(x[i]);
                }
                acc += xs[sb * 8 + is] * (dw * float(dot) - mw * float(sum));
            }
        }
    }
    return acc;
}

// E:3553-3611: Q6_K super-block = {128 low-nibble bytes, 64 two-bit bytes, 16 int8 scales, f16 d}; the eight
// 32-element input blocks address it through the table below (two 16-element scale groups per block).
float dot_q6_k_q8_0(const uint8_t* row, const int8_t* xq, const float* xs, int k) {
    static const int tab[8][5] = {{0, 0, 0, 0, 0}, {32, 0, 0, 2, 2}, {0, 0, 4, 4, 4}, {32, 0, 4, 6, 6},
                                  {64, 32, 0, 0, 8}, {96, 32, 0, 2, 10}, {64, 32, 4, 4, 12}, {96, 32, 4, 6, 14}};
    float acc = 0.0f;
    for (int sb = 0; sb < k / 256; ++sb) {
        const uint8_t* blk = row + size_t(sb) * 210;
        const uint8_t *ql = blk, *qh = blk + 128, *sc = blk + 192;
        float d = f16_bits_to_f32(uint16_t(blk[208] | (blk[209] << 8)));
        for (int b = 0; b < 8; ++b) {
            const int8_t* x = xq + (size_t(sb) * 8 + b) * 32;
            int dots[2] = {0, 0};
            for (int l = 0; l < 32; ++l) {
                int q6 = int((ql[tab[b][0] + l] >> tab[b][2]) & 0x0F) | (int((qh[tab[b][1] + l] >> tab[b][3]) & 3) << 4);
                dots[l >> 4] += (q6 - 32) * int(x[l]);
            }
            float slo = float(int(int8_t(sc[tab[b][4]]))), shi = float(int(int8_t(sc[tab[b][4] + 1])));
            acc += d * xs[sb * 8 + b] * (slo * float(dots[0]) + shi * float(dots[1]));
        }
    }
    return acc;
}

inline size_t kquant_row_bytes(int quant, int k) { return size_t(k / 256) * (quant == 12 ? 144 : 210); }

// E:3411-3487 (Q4_K) / E:3636-3652 (Q6_K); quant: 12 = Q4_K, 14 = Q6_K (the GGML type numbers)
void matmul_vec_kquant(int quant, float* out, const float* in, const uint8_t* w, int k, int n) {
    std::vector<int8_t> xq((size_t(k) + 31) / 32 * 32);
    std::vector<float> xs((size_t(k) + 31) / 32);
    quantize_act_q8_0(in, k, xq.data(), xs.data());
    size_t rb = kquant_row_bytes(quant, k);
#pragma omp parallel for schedule(static) if (size_t(n) * rb > 1000000)
    for (int j = 0; j < n; ++j)
        out[j] = quant == 12 ? dot_q4_k_q8_0(w + size_t(j) * rb, xq.data(), xs.data(), k)
                             : dot_q6_k_q8_0(w + size_t(j) * rb, xq.data(), xs.data(), k);
}

// WL:1146-1200: value = d * sc * q - dmin * m
void dequant_q4_k(const uint8_t* in, size_t n, float* out) {
    for (size_t sb = 0; sb * 256 < n; ++sb) {
        const uint8_t* blk = in + sb * 144;
        float d = f16_bits_to_f32(uint16_t(blk[0] | (blk[1] << 8)));
        float dmin = f16_bits_to_f32(uint16_t(blk[2] | (blk[3] << 8)));
        for (int is = 0; is < 8; ++is) {
            int sc, mn;
            scale_min_k4(is, blk + 4, sc, mn);
            float dw = d * float(sc), mw = dmin * float(mn);
            for (int l = 0; l < 32; ++l) {
                size_t o = sb * 256 + size_t(is) * 32 + l;
                uint8_t by = blk[16 + (is >> 1) * 32 + l];
                if (o < n) out[o] = dw * float((is & 1) ? (by >> 4) : (by & 0x0F)) - mw;
            }
        }
    }
}

// WL:997-1060: value = d * scale[group of 16] * (q6 - 32)
void dequant_q6_k(const uint8_t* in, size_t n, float* out) {
    for (size_t sb = 0; sb * 256 < n; ++sb) {
        const uint8_t* blk = in + sb * 210;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192);
        float d = f16_bits_to_f32(uint16_t(blk[208] | (blk[209] << 8)));
        for (int half = 0; half < 2; ++half)
            for (int l = 0; l < 32; ++l) {
                int is = l / 16;
                const uint8_t* q = ql + half * 64;
                uint8_t h = qh[half * 32 + l];
                int q1 = int((q[l] & 0x0F) | (((h >> 0) & 3) << 4)) - 32, q2 = int((q[l + 32] & 0x0F) | (((h >> 2) & 3) << 4)) - 32;
                int q3 = int((q[l] >> 4) | (((h >> 4) & 3) << 4)) - 32, q4 = int((q[l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32;
                size_t o = sb * 256 + size_t(half) * 128 + l;
                const int8_t* s = sc + half * 8 + is;
                if (o < n) out[o] = d * float(s[0]) * float(q1);
                if (o + 32 < n) out[o + 32] = d * float(s[2]) * float(q2);
                if (o + 64 < n) out[o + 64] = d * float(s[4]) * float(q3);
                if (o + 96 < n) out[o + 96] = d * float(s[6]) * float(q4);
            }
    }
}

// ---------------------------------------------------------------- K-quant quantisers (exporter side)
// WL:1663-1771 make_qkx2_quants(x, nmax = 15, rmin = -1, rdelta = 0.1, nstep = 20) on one 32-element sub-block:
// returns scale and the_min (= -min) and fills L.
void qkx2_fit(const float* x, float& scale_out, float& the_min_out, uint8_t* L) {
    const int n = 32;
    const float nmax = 15.0f;
    float mn = x[0], mx = x[0];
    for (int i = 1; i < n; ++i) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
    if (mx == mn) { scale_out = 0.0f; the_min_out = -mn; std::fill(L, L + n, uint8_t(0)); return; }
    if (mn > 0.0f) mn = 0.0f;
    float iscale = nmax / (mx - mn), scale = 1.0f / iscale, best_mad = 0.0f;
    auto level = [&](float v, float is) { return std::min(nmax, std::max(0.0f, rround((v - mn) * is))); };
    for (int i = 0; i < n; ++i) {
        float li = level(x[i], iscale);
        L[i] = uint8_t(li);
        float diff = scale * li + mn - x[i];
        best_mad += diff * diff;
    }
    float best_scale = scale, best_min = mn;
    std::vector<uint8_t> laux(n);
    for (int is = 0; is <= 20; ++is) {
        float iscale_try = (-1.0f + 0.1f * float(is) + nmax) / (mx - mn);
        float sum_l = 0, sum_l2 = 0, sum_x = 0, sum_xl = 0;
        for (int i = 0; i < n; ++i) {
            float li = level(x[i], iscale_try);
            laux[i] = uint8_t(li);
            sum_l += li; sum_l2 += li * li; sum_x += x[i]; sum_xl += li * x[i];
        }
        float det = float(n) * sum_l2 - sum_l * sum_l;
        if (det > 0.0f) {
            float this_scale = (float(n) * sum_xl - sum_x * sum_l) / det;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / det;
            if (this_min > 0.0f) { this_min = 0.0f; if (sum_l2 > 0.0f) this_scale = sum_xl / sum_l2; }
            if (this_scale > 0.0f) {
                float mad = 0.0f;
                for (int i = 0; i < n; ++i) { float diff = this_scale * float(laux[i]) + this_min - x[i]; mad += diff * diff; }
                if (mad < best_mad) { std::copy(laux.begin(), laux.end(), L); best_mad = mad; best_scale = this_scale; best_min = this_min; }
            }
        }
    }
    scale_out = best_scale;
    the_min_out = -best_min;
}

// WL:1773-1900
void quantize_q4_k(const float* data, size_t n, uint8_t* out) {
    for (size_t sb = 0; sb < n / 256; ++sb) {
        const float* x = data + sb * 256;
        uint8_t* o = out + sb * 144;
        float scales[8], mins[8];
        uint8_t q[8][32];
        for (int j = 0; j < 8; ++j) qkx2_fit(x + j * 32, scales[j], mins[j], q[j]);
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; ++j) { if (scales[j] > max_scale) max_scale = scales[j]; if (mins[j] > max_min) max_min = mins[j]; }
        float inv_scale = max_scale > 0 ? 63.0f / max_scale : 0.0f, inv_min = max_min > 0 ? 63.0f / max_min : 0.0f;
        float d = max_scale > 0 ? max_scale / 63.0f : 0.0f, dmin = max_min > 0 ? max_min / 63.0f : 0.0f;
        uint8_t sq[8], mq[8];
        for (int j = 0; j < 8; ++j) {
            sq[j] = uint8_t(std::min(63.0f, std::max(0.0f, rround(scales[j] * inv_scale))));
            mq[j] = uint8_t(std::min(63.0f, std::max(0.0f, rround(mins[j] * inv_min))));
        }
        uint16_t d_bits = f32_to_f16_bits(d), dmin_bits = f32_to_f16_bits(dmin);
        float d_stored = f16_bits_to_f32(d_bits), dmin_stored = f16_bits_to_f32(dmin_bits);
        for (int j = 0; j < 8; ++j) {
            float s_eff = d_stored * float(sq[j]);
            if (s_eff == 0.0f) { std::fill(q[j], q[j] + 32, uint8_t(0)); continue; }
            float inv_s = 1.0f / s_eff, dm = dmin_stored * float(mq[j]);
            for (int i = 0; i < 32; ++i) q[j][i] = uint8_t(std::min(15.0f, std::max(0.0f, rround((x[j * 32 + i] + dm) * inv_s))));
        }
        o[0] = uint8_t(d_bits); o[1] = uint8_t(d_bits >> 8); o[2] = uint8_t(dmin_bits); o[3] = uint8_t(dmin_bits >> 8);
        for (int i = 0; i < 4; ++i) {
            o[4 + i] = uint8_t((sq[i] & 63) | (((sq[i + 4] >> 4) & 3) << 6));
            o[8 + i] = uint8_t((mq[i] & 63) | (((mq[i + 4] >> 4) & 3) << 6));
            o[12 + i] = uint8_t((sq[i + 4] & 0x0F) | ((mq[i + 4] & 0x0F) << 4));
        }
        for (int c = 0; c < 4; ++c)
            for (int i = 0; i < 32; ++i) o[16 + c * 32 + i] = uint8_t((q[2 * c][i] & 0x0F) | ((q[2 * c + 1][i] & 0x0F) << 4));
    }
}

// WL:1989-2125
void quantize_q6_k(const float* data, size_t n, uint8_t* out) {
    for (size_t sb = 0; sb < n / 256; ++sb) {
        const float* x = data + sb * 256;
        uint8_t* o = out + sb * 210;
        float sub[16];
        for (int j = 0; j < 16; ++j) {
            float mx = 0.0f, amax = 0.0f;
            for (int i = 0; i < 16; ++i) { float av = std::fabs(x[j * 16 + i]); if (av > amax) { amax = av; mx = x[j * 16 + i]; } }
            if (amax < 1e-30f) { sub[j] = 0.0f; continue; }
            float iscale = -32.0f / mx;
            sub[j] = 1.0f / iscale;
        }
        float max_scale = 0.0f, max_abs = 0.0f;
        for (int j = 0; j < 16; ++j) if (std::fabs(sub[j]) > max_abs) { max_abs = std::fabs(sub[j]); max_scale = sub[j]; }
        if (max_abs < 1e-30f) { std::fill(o, o + 210, uint8_t(0)); continue; }
        float super_iscale = -128.0f / max_scale, super_d = 1.0f / super_iscale;
        uint16_t d_bits = f32_to_f16_bits(super_d);
        o[208] = uint8_t(d_bits); o[209] = uint8_t(d_bits >> 8);
        float d_stored = f16_bits_to_f32(d_bits);
        int8_t L[256] = {0};
        for (int j = 0; j < 16; ++j) {
            int qs = std::min(127, std::max(-128, int(rround(super_iscale * sub[j]))));
            o[192 + j] = uint8_t(int8_t(qs));
            float s_eff = d_stored * float(qs);
            if (s_eff == 0.0f) continue;
            float inv = 1.0f / s_eff;
            for (int i = 0; i < 16; ++i) L[j * 16 + i] = int8_t(std::min(31, std::max(-32, int(rround(inv * x[j * 16 + i])))));
        }
        for (int chunk = 0; chunk < 256; chunk += 128)
            for (int l = 0; l < 32; ++l) {
                uint8_t q1 = uint8_t(L[chunk + l] + 32), q2 = uint8_t(L[chunk + l + 32] + 32), q3 = uint8_t(L[chunk + l + 64] + 32), q4 = uint8_t(L[chunk + l + 96] + 32);
                o[chunk / 2 + l] = uint8_t((q1 & 0x0F) | ((q3 & 0x0F) << 4));
                o[chunk / 2 + l + 32] = uint8_t((q2 & 0x0F) | ((q4 & 0x0F) << 4));
                o[128 + chunk / 4 + l] = uint8_t((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
            }
    }
}

// ---------------------------------------------------------------- elementwise
// E:298-304
inline float dot_f32(const float* a, const float* b, int n) {
    float s = 0.0f;
    for (int i = 0; i < n; ++i) s += a[i] * b[i];
    return s;
}
// E:327-334: x * inv_rms * w, inv_rms = 1/sqrt(mean + eps)
void rms_norm(float* out, const float* in, const float* w, int n, float eps) {
    float ss = dot_f32(in, in, n);
    float inv = 1.0f / std::sqrt(ss / float(n) + eps);
    for (int i = 0; i < n; ++i) out[i] = in[i] * inv * w[i];
}
// E:381-386
void silu_mul(float* out, const float* g, const float* u, int n) {
    for (int i = 0; i < n; ++i) {
        float x = g[i];
        out[i] = (x / (1.0f + std::exp(-x))) * u[i];
    }
}
// E:455-459
void residual_add(float* a, const float* b, int n) {
    for (int i = 0; i < n; ++i) a[i] += b[i];
}
// E:502-504
void rope_freqs(float* f, int head_dim, float theta) {
    for (int i = 0; i < head_dim / 2; ++i) f[i] = 1.0f / std::pow(theta, 2.0f * float(i) / float(head_dim));
}
// E:509-528: adjacent pairs, one sin/cos table per position shared by all heads
void rope(float* data, int pos, int head_dim, int heads, const float* freqs) {
    int half = head_dim / 2;
    std::vector<float> c(half), s(half);
    for (int i = 0; i < half; ++i) {
        float ang = float(pos) * freqs[i];
        s[i] = std::sin(ang);
        c[i] = std::cos(ang);
    }
    for (int h = 0; h < heads; ++h) {
        float* p = data + size_t(h) * head_dim;
        for (int i = 0; i < half; ++i) {
            float x0 = p[2 * i], x1 = p[2 * i + 1];
            p[2 * i] = x0 * c[i] - x1 * s[i];
            p[2 * i + 1] = x0 * s[i] + x1 * c[i];
        }
    }
}
// E:533-545
float quantize_kv(const float* v, int n, int8_t* out) {
    float mx = 0.0f;
    for (int i = 0; i < n; ++i) {
        float a = std::fabs(v[i]);
        if (a > mx) mx = a;
    }
    float scale = mx / 127.0f;
    float inv = (mx > 0.0f) ? 127.0f / mx : 0.0f;
    for (int i = 0; i < n; ++i) {
        float q = rround(v[i] * inv);
        q = std::min(127.0f, std::max(-127.0f, q));
        out[i] = int8_t(q);
    }
    return scale;
}

// ---------------------------------------------------------------- KV storage
// mode 0: int8 + per-token f32 scale (the reference CPU path, E:3954-3974)
// mode 1: fp16 values (the GPU design; values are rounded to fp16 when appended)
// mode 2: f32 values
struct KVView {
    int mode;
    const int8_t* k8; const int8_t* v8; const float* ks; const float* vs;   // mode 0
    const float* kf; const float* vf;                                      // mode 1/2 (already widened)
};

// score of q against the cached key at position t (before the 1/sqrt(hd) factor)
// mode 0 follows dot_f32_i8 (E:550-556): sum(q*k_i8) then * k_scale.
inline float k_dot(const KVView& c, const float* q, size_t off, int t, int hd) {
    float s = 0.0f;
    if (c.mode == 0) {
        const int8_t* k = c.k8 + off;
        for (int i = 0; i < hd; ++i) s += q[i] * float(k[i]);
        return s * c.ks[t];
    }
    const float* k = c.kf + off;
    for (int i = 0; i < hd; ++i) s += q[i] * k[i];
    return s;
}
inline float v_at(const KVView& c, size_t idx, int t) {
    return c.mode == 0 ? float(c.v8[idx]) * c.vs[t] : c.vf[idx];
}

// E:559-583 (plain two-pass softmax attention; E:490-498 softmax)
void attention_plain(float* out, const float* q, const KVView& c, int seq, int nh, int nkv, int hd) {
    int g = nh / nkv;
    float scale = 1.0f / std::sqrt(float(hd));
    size_t stride = size_t(nkv) * hd;
    std::vector<float> sc(seq);
    for (int h = 0; h < nh; ++h) {
        int kvh = h / g;
        const float* qh = q + size_t(h) * hd;
        for (int t = 0; t < seq; ++t) sc[t] = k_dot(c, qh, t * stride + size_t(kvh) * hd, t, hd) * scale;
        float mx = -std::numeric_limits<float>::infinity();
        for (int t = 0; t < seq; ++t) mx = std::max(mx, sc[t]);
        float sum = 0.0f;
        for (int t = 0; t < seq; ++t) { sc[t] = std::exp(sc[t] - mx); sum += sc[t]; }
        float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        for (int t = 0; t < seq; ++t) sc[t] *= inv;
        for (int d = 0; d < hd; ++d) {
            float a = 0.0f;
            for (int t = 0; t < seq; ++t) a += sc[t] * v_at(c, t * stride + size_t(kvh) * hd + d, t);
            out[size_t(h) * hd + d] = a;
        }
    }
}

// E:601-626 (attention_sliding): the plain two-pass attention over the last `window` positions only.
void attention_sliding(float* out, const float* q, const KVView& c, int seq, int window, int nh, int nkv, int hd) {
    int start = seq > window ? seq - window : 0, wl = seq - start;
    int g = nh / nkv;
    float scale = 1.0f / std::sqrt(float(hd));
    size_t stride = size_t(nkv) * hd;
    std::vector<float> sc(wl);
    for (int h = 0; h < nh; ++h) {
        int kvh = h / g;
        const float* qh = q + size_t(h) * hd;
        for (int si = 0; si < wl; ++si) { int t = start + si; sc[si] = k_dot(c, qh, t * stride + size_t(kvh) * hd, t, hd) * scale; }
        float mx = -std::numeric_limits<float>::infinity();
        for (int si = 0; si < wl; ++si) mx = std::max(mx, sc[si]);
        float sum = 0.0f;
        for (int si = 0; si < wl; ++si) { sc[si] = std::exp(sc[si] - mx); sum += sc[si]; }
        float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        for (int si = 0; si < wl; ++si) sc[si] *= inv;
        for (int d = 0; d < hd; ++d) {
            float a = 0.0f;
            for (int si = 0; si < wl; ++si) { int t = start + si; a += sc[si] * v_at(c, t * stride + size_t(kvh) * hd + d, t); }
            out[size_t(h) * hd + d] = a;
        }
    }
}

// E:657-715: single-query attention, keys in blocks of 64, online softmax, per-block
// partial P.V sum added to the accumulator.
void attention_flash(float* out, const float* q, const KVView& c, int seq, int nh, int nkv, int hd) {
    int g = nh / nkv;
    float scale = 1.0f / std::sqrt(float(hd));
    size_t stride = size_t(nkv) * hd;
    float sc[kFlashBlock];
    std::vector<float> acc(hd);
    for (int h = 0; h < nh; ++h) {
        int kvh = h / g;
        const float* qh = q + size_t(h) * hd;
        float mi = -std::numeric_limits<float>::infinity(), li = 0.0f;
        std::fill(acc.begin(), acc.end(), 0.0f);
        for (int b0 = 0; b0 < seq; b0 += kFlashBlock) {
            int bl = std::min(kFlashBlock, seq - b0);
            float mb = -std::numeric_limits<float>::infinity();
            for (int bi = 0; bi < bl; ++bi) {
                int t = b0 + bi;
                float s = k_dot(c, qh, t * stride + size_t(kvh) * hd, t, hd) * scale;
                sc[bi] = s;
                if (s > mb) mb = s;
            }
            float mp = mi;
            if (mb > mi) mi = mb;
            float es = std::exp(mp - mi);
            li *= es;
            for (int d = 0; d < hd; ++d) acc[d] *= es;
            float lb = 0.0f;
            for (int bi = 0; bi < bl; ++bi) {
                float e = std::exp(sc[bi] - mi);
                sc[bi] = e;
                lb += e;
            }
            li += lb;
            for (int d = 0; d < hd; ++d) {
                float sum = 0.0f;
                for (int bi = 0; bi < bl; ++bi) {
                    int t = b0 + bi;
                    sum += sc[bi] * v_at(c, t * stride + size_t(kvh) * hd + d, t);
                }
                acc[d] += sum;
            }
        }
        float il = 1.0f / li;
        for (int d = 0; d < hd; ++d) out[size_t(h) * hd + d] = acc[d] * il;
    }
}

// E:755-883: m queries, tiles of 16 queries x blocks of 64 keys; query row r (global
// position base_pos + r) sees keys <= its own position; blocks past the tile's last
// query are never visited; a block wholly in a query's future is skipped for it.
void attention_flash_batch(float* out, const float* qb, const KVView& c, int m, int base_pos,
                           int nh, int nkv, int hd) {
    int g = nh / nkv;
    float scale = 1.0f / std::sqrt(float(hd));
    size_t stride = size_t(nkv) * hd;
    size_t ostride = size_t(nh) * hd;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < nh; ++h) {
        int kvh = h / g;
        size_t qo = size_t(h) * hd;
        std::vector<float> acc(size_t(kQTile) * hd);
        std::vector<float> sc(size_t(kQTile) * kFlashBlock);
        float ms[kQTile], ls[kQTile];
        for (int t0 = 0; t0 < m; t0 += kQTile) {
            int tl = std::min(kQTile, m - t0);
            int maxq = base_pos + t0 + tl - 1;
            for (int i = 0; i < kQTile; ++i) { ms[i] = -std::numeric_limits<float>::infinity(); ls[i] = 0.0f; }
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (int b0 = 0; b0 <= maxq; b0 += kFlashBlock) {
                int be = std::min(b0 + kFlashBlock, maxq + 1), bl = be - b0;
                std::fill(sc.begin(), sc.end(), 0.0f);
                for (int bi = 0; bi < bl; ++bi) {
                    int t = b0 + bi;
                    size_t ko = t * stride + size_t(kvh) * hd;
                    for (int qi = 0; qi < tl; ++qi) {
                        const float* qr = qb + size_t(t0 + qi) * ostride + qo;
                        sc[qi * kFlashBlock + bi] = k_dot(c, qr, ko, t, hd) * scale;
                    }
                }
                for (int qi = 0; qi < tl; ++qi) {
                    int qpos = base_pos + t0 + qi;
                    int ve = std::min(std::max(qpos + 1 - b0, 0), bl);
                    float* s = &sc[qi * kFlashBlock];
                    if (ve == 0) { for (int bi = 0; bi < bl; ++bi) s[bi] = 0.0f; continue; }
                    float mb = -std::numeric_limits<float>::infinity();
                    for (int bi = 0; bi < ve; ++bi) if (s[bi] > mb) mb = s[bi];
                    float mp = ms[qi], mn = std::max(mp, mb);
                    ms[qi] = mn;
                    float es = std::exp(mp - mn);
                    ls[qi] *= es;
                    for (int d = 0; d < hd; ++d) acc[size_t(qi) * hd + d] *= es;
                    float lb = 0.0f;
                    for (int bi = 0; bi < ve; ++bi) { float e = std::exp(s[bi] - mn); s[bi] = e; lb += e; }
                    for (int bi = ve; bi < bl; ++bi) s[bi] = 0.0f;
                    ls[qi] += lb;
                }
                for (int bi = 0; bi < bl; ++bi) {
                    int t = b0 + bi;
                    size_t vo = t * stride + size_t(kvh) * hd;
                    for (int d = 0; d < hd; ++d) {
                        float vv = v_at(c, vo + d, t);
                        for (int qi = 0; qi < tl; ++qi) acc[size_t(qi) * hd + d] += sc[qi * kFlashBlock + bi] * vv;
                    }
                }
            }
            for (int qi = 0; qi < tl; ++qi) {
                float il = 1.0f / ls[qi];
                float* o = out + size_t(t0 + qi) * ostride + qo;
                for (int d = 0; d < hd; ++d) o[d] = acc[size_t(qi) * hd + d] * il;
            }
        }
    }
}

// E:916-1046 (attention_sliding_batch): as attention_flash_batch, but query position p sees the keys
// [max(0, p - window + 1), p]; the key blocks start at the 64-aligned block that holds the tile's first valid key.
void attention_sliding_batch(float* out, const float* qb, const KVView& c, int m, int base_pos, int window,
                             int nh, int nkv, int hd) {
    int g = nh / nkv;
    float scale = 1.0f / std::sqrt(float(hd));
    size_t stride = size_t(nkv) * hd;
    size_t ostride = size_t(nh) * hd;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < nh; ++h) {
        int kvh = h / g;
        size_t qo = size_t(h) * hd;
        std::vector<float> acc(size_t(kQTile) * hd);
        std::vector<float> sc(size_t(kQTile) * kFlashBlock);
        float ms[kQTile], ls[kQTile];
        for (int t0 = 0; t0 < m; t0 += kQTile) {
            int tl = std::min(kQTile, m - t0);
            int first_q = base_pos + t0, maxq = base_pos + t0 + tl - 1;
            int min_k = std::max(first_q - (window - 1), 0);
            for (int i = 0; i < kQTile; ++i) { ms[i] = -std::numeric_limits<float>::infinity(); ls[i] = 0.0f; }
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (int b0 = (min_k / kFlashBlock) * kFlashBlock; b0 <= maxq; b0 += kFlashBlock) {
                int be = std::min(b0 + kFlashBlock, maxq + 1), bl = be - b0;
                std::fill(sc.begin(), sc.end(), 0.0f);
                for (int bi = 0; bi < bl; ++bi) {
                    int t = b0 + bi;
                    size_t ko = t * stride + size_t(kvh) * hd;
                    for (int qi = 0; qi < tl; ++qi) {
                        const float* qr = qb + size_t(t0 + qi) * ostride + qo;
                        sc[qi * kFlashBlock + bi] = k_dot(c, qr, ko, t, hd) * scale;
                    }
                }
                for (int qi = 0; qi < tl; ++qi) {
                    int qpos = base_pos + t0 + qi;
                    int ws = std::max(qpos - (window - 1), 0);
                    int lo = std::max(ws, b0) - b0;
                    int hi = std::min(std::max(qpos + 1 - b0, 0), bl);
                    float* s = &sc[qi * kFlashBlock];
                    if (lo >= hi) { for (int bi = 0; bi < bl; ++bi) s[bi] = 0.0f; continue; }
                    float mb = -std::numeric_limits<float>::infinity();
                    for (int bi = lo; bi < hi; ++bi) if (s[bi] > mb) mb = s[bi];
                    float mp = ms[qi], mn = std::max(mp, mb);
                    ms[qi] = mn;
                    float es = std::exp(mp - mn);
                    ls[qi] *= es;
                    for (int d = 0; d < hd; ++d) acc[size_t(qi) * hd + d] *= es;
                    float lb = 0.0f;
                    for (int bi = lo; bi < hi; ++bi) { float e = std::exp(s[bi] - mn); s[bi] = e; lb += e; }
                    for (int bi = 0; bi < lo; ++bi) s[bi] = 0.0f;
                    for (int bi = hi; bi < bl; ++bi) s[bi] = 0.0f;
                    ls[qi] += lb;
                }
                for (int bi = 0; bi < bl; ++bi) {
                    int t = b0 + bi;
                    size_t vo = t * stride + size_t(kvh) * hd;
                    for (int d = 0; d < hd; ++d) {
                        float vv = v_at(c, vo + d, t);
                        for (int qi = 0; qi < tl; ++qi) acc[size_t(qi) * hd + d] += sc[qi * kFlashBlock + bi] * vv;
                    }
                }
            }
            for (int qi = 0; qi < tl; ++qi) {
                float il = ls[qi] > 0.0f ? 1.0f / ls[qi] : 0.0f;
                float* o = out + size_t(t0 + qi) * ostride + qo;
                for (int d = 0; d < hd; ++d) o[d] = acc[size_t(qi) * hd + d] * il;
            }
        }
    }
}

// P:501-503: max_by(partial_cmp) keeps the LAST of equal maxima.
uint32_t argmax_last(const float* v, int n) {
    int best = 0;
    for (int i = 1; i < n; ++i) if (v[i] >= v[best]) best = i;
    return uint32_t(best);
}

}  // namespace

// ======================================================================= C API
extern "C" {

struct FoConfig {
    int32_t hidden_size, intermediate_size, num_layers, num_heads, num_kv_heads, head_dim;
    int32_t vocab_size, max_seq_len;
    float rms_norm_eps, rope_theta;
    int32_t quant;     // 8 = Q8_0, 4 = Q4_0
    int32_t qkv_bias;  // 1: f32 q/k/v biases follow v in weights.bin (Qwen2)
    int32_t sliding_window;  // > 0: sliding-window attention over that many positions (Mistral), E:97, E:191
    int32_t proj_quant[8];   // ProjectionDTypes (ir.rs:411-421) as q, k, v, o, gate, up, down, lm_head; 0 = quant; 12 = Q4_K, 14 = Q6_K
};
inline int pq_of(const FoConfig& c, int i) { return c.proj_quant[i] ? c.proj_quant[i] : c.quant; }

uint16_t fo_f32_to_f16(float x) { return f32_to_f16_bits(x); }
float fo_f16_to_f32(uint16_t h) { return f16_bits_to_f32(h); }

// WL:1454-1486
void fo_quantize_q8_0(const float* x, size_t n, uint8_t* out) {
    size_t nb = (n + 31) / 32;
#pragma omp parallel for if (nb > 4096)
    for (long b = 0; b < long(nb); ++b) {
        size_t base = size_t(b) * 32, end = std::min(base + 32, n);
        float amax = 0.0f;
        for (size_t i = base; i < end; ++i) { float a = std::fabs(x[i]); if (a > amax) amax = a; }
        float scale = (amax == 0.0f) ? 0.0f : amax / 127.0f;
        float inv = (scale != 0.0f) ? 1.0f / scale : 0.0f;
        uint8_t* o = out + size_t(b) * 34;
        uint16_t hb = f32_to_f16_bits(scale);
        o[0] = uint8_t(hb); o[1] = uint8_t(hb >> 8);
        for (int j = 0; j < 32; ++j) {
            float v = (base + j < end) ? x[base + j] : 0.0f;
            float q = std::min(127.0f, std::max(-127.0f, rround(v * inv)));
            o[2 + j] = uint8_t(int8_t(q));
        }
    }
}

// WL:1494-1544: the reference's own Q4_0 quantiser, scale = amax/8 (always >= 0).
void fo_quantize_q4_0_ref(const float* x, size_t n, uint8_t* out) {
    size_t nb = (n + 31) / 32;
#pragma omp parallel for if (nb > 4096)
    for (long b = 0; b < long(nb); ++b) {
        size_t base = size_t(b) * 32, end = std::min(base + 32, n);
        float amax = 0.0f;
        for (size_t i = base; i < end; ++i) { float a = std::fabs(x[i]); if (a > amax) amax = a; }
        float scale = amax / 8.0f;
        float inv = (scale != 0.0f) ? 1.0f / scale : 0.0f;
        uint8_t* o = out + size_t(b) * 18;
        uint16_t hb = f32_to_f16_bits(scale);
        o[0] = uint8_t(hb); o[1] = uint8_t(hb >> 8);
        for (int j = 0; j < 16; ++j) {
            float lo = (base + j < end) ? x[base + j] : 0.0f;
            float hi = (base + j + 16 < end) ? x[base + j + 16] : 0.0f;
            int ql = std::min(15, std::max(0, int(rround(lo * inv)) + 8));
            int qh = std::min(15, std::max(0, int(rround(hi * inv)) + 8));
            o[2 + j] = uint8_t(ql | (qh << 4));
        }
    }
}

// The benchmark configurations specify the signed-max rule instead: d = (value of largest
// magnitude, sign kept) / -8, nibble = clamp(round(x/d) + 8, 0, 15).  Dequantisation is
// the same as for the rule above (WL:893-926), so the kernels see no difference.
void fo_quantize_q4_0_signed(const float* x, size_t n, uint8_t* out) {
    size_t nb = (n + 31) / 32;
#pragma omp parallel for if (nb > 4096)
    for (long b = 0; b < long(nb); ++b) {
        size_t base = size_t(b) * 32, end = std::min(base + 32, n);
        float amax = 0.0f, vmax = 0.0f;
        for (size_t i = base; i < end; ++i) { float a = std::fabs(x[i]); if (a > amax) { amax = a; vmax = x[i]; } }
        float d = (vmax == 0.0f) ? 0.0f : vmax / -8.0f;
        float inv = (d != 0.0f) ? 1.0f / d : 0.0f;
        uint8_t* o = out + size_t(b) * 18;
        uint16_t hb = f32_to_f16_bits(d);
        o[0] = uint8_t(hb); o[1] = uint8_t(hb >> 8);
        for (int j = 0; j < 16; ++j) {
            float lo = (base + j < end) ? x[base + j] : 0.0f;
            float hi = (base + j + 16 < end) ? x[base + j + 16] : 0.0f;
            int ql = std::min(15, std::max(0, int(rround(lo * inv)) + 8));
            int qh = std::min(15, std::max(0, int(rround(hi * inv)) + 8));
            o[2 + j] = uint8_t(ql | (qh << 4));
        }
    }
}

// WL:860-888
void fo_dequant_q8_0(const uint8_t* in, size_t n, float* out) {
    size_t nb = (n + 31) / 32;
#pragma omp parallel for if (nb > 4096)
    for (long b = 0; b < long(nb); ++b) {
        const uint8_t* blk = in + size_t(b) * 34;
        float d = f16_bits_to_f32(uint16_t(blk[0] | (blk[1] << 8)));
        for (int j = 0; j < 32 && size_t(b) * 32 + j < n; ++j) out[size_t(b) * 32 + j] = float(int8_t(blk[2 + j])) * d;
    }
}
// WL:893-926
void fo_dequant_q4_0(const uint8_t* in, size_t n, float* out) {
    size_t nb = (n + 31) / 32;
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t* blk = in + b * 18;
        float d = f16_bits_to_f32(uint16_t(blk[0] | (blk[1] << 8)));
        for (int j = 0; j < 16; ++j) {
            size_t il = b * 32 + j, ih = il + 16;
            if (il < n) out[il] = float(int(blk[2 + j] & 0x0F) - 8) * d;
            if (ih < n) out[ih] = float(int(blk[2 + j] >> 4) - 8) * d;
        }
    }
}

float fo_dot_q8_0(const float* in, const uint8_t* row, int k) { return dot_q8_0(in, row, k); }
float fo_dot_q4_0(const float* in, const uint8_t* row, int k) { return dot_q4_0(in, row, k); }

void fo_matmul_vec_q8_0(float* out, const float* in, const uint8_t* w, int k, int n) { matmul_mat(8, out, 1, in, w, k, n, false); }
void fo_matmul_vec_q4_0(float* out, const float* in, const uint8_t* w, int k, int n) { matmul_mat(4, out, 1, in, w, k, n, false); }
// fast != 0 picks the row-vectorised twin (bit-identical values)
void fo_matmul_mat_q8_0(float* out, int m, const float* in, const uint8_t* w, int k, int n, int fast) { matmul_mat(8, out, m, in, w, k, n, fast != 0); }
void fo_matmul_mat_q4_0(float* out, int m, const float* in, const uint8_t* w, int k, int n, int fast) { matmul_mat(4, out, m, in, w, k, n, fast != 0); }

// K-quants: quant 12 = Q4_K, 14 = Q6_K
void fo_quantize_act_q8_0(const float* in, int k, int8_t* q, float* scale) { quantize_act_q8_0(in, k, q, scale); }
void fo_matmul_vec_kquant(int quant, float* out, int m, const float* in, const uint8_t* w, int k, int n) {
    for (int r = 0; r < m; ++r) matmul_vec_kquant(quant, out + size_t(r) * n, in + size_t(r) * k, w, k, n);
}
void fo_quantize_q4_k(const float* x, size_t n, uint8_t* out) { quantize_q4_k(x, n, out); }
void fo_quantize_q6_k(const float* x, size_t n, uint8_t* out) { quantize_q6_k(x, n, out); }
void fo_dequant_q4_k(const uint8_t* in, size_t n, float* out) { dequant_q4_k(in, n, out); }
void fo_dequant_q6_k(const uint8_t* in, size_t n, float* out) { dequant_q6_k(in, n, out); }

void fo_rms_norm(float* out, const float* in, const float* w, int n, float eps) { rms_norm(out, in, w, n, eps); }
void fo_silu_mul(float* out, const float* g, const float* u, int n) { silu_mul(out, g, u, n); }
void fo_residual_add(float* a, const float* b, int n) { residual_add(a, b, n); }
void fo_rope_freqs(float* f, int head_dim, float theta) { rope_freqs(f, head_dim, theta); }
void fo_rope(float* data, int pos, int head_dim, int heads, const float* freqs) { rope(data, pos, head_dim, heads, freqs); }
float fo_quantize_kv(const float* v, int n, int8_t* out) { return quantize_kv(v, n, out); }
uint32_t fo_argmax(const float* v, int n) { return argmax_last(v, n); }

// Attention on caller-provided caches.  kv_mode 0: k/v are int8 with scales; 1 or 2: k/v
// are float arrays (mode 1 callers pass values already rounded through fp16).
static KVView make_view(int mode, const void* k, const void* v, const float* ks, const float* vs) {
    KVView c{};
    c.mode = mode;
    if (mode == 0) { c.k8 = (const int8_t*)k; c.v8 = (const int8_t*)v; c.ks = ks; c.vs = vs; }
    else { c.kf = (const float*)k; c.vf = (const float*)v; }
    return c;
}
void fo_attention(float* out, const float* q, int kv_mode, const void* k, const void* v, const float* ks,
                  const float* vs, int seq, int nh, int nkv, int hd) {
    attention_plain(out, q, make_view(kv_mode, k, v, ks, vs), seq, nh, nkv, hd);
}
void fo_attention_flash(float* out, const float* q, int kv_mode, const void* k, const void* v, const float* ks,
                        const float* vs, int seq, int nh, int nkv, int hd) {
    attention_flash(out, q, make_view(kv_mode, k, v, ks, vs), seq, nh, nkv, hd);
}
void fo_attention_sliding(float* out, const float* q, int kv_mode, const void* k, const void* v, const float* ks,
                          const float* vs, int seq, int window, int nh, int nkv, int hd) {
    attention_sliding(out, q, make_view(kv_mode, k, v, ks, vs), seq, window, nh, nkv, hd);
}
void fo_attention_sliding_batch(float* out, const float* qb, int kv_mode, const void* k, const void* v,
                                const float* ks, const float* vs, int m, int base_pos, int window, int nh, int nkv, int hd) {
    attention_sliding_batch(out, qb, make_view(kv_mode, k, v, ks, vs), m, base_pos, window, nh, nkv, hd);
}
void fo_attention_flash_batch(float* out, const float* qb, int kv_mode, const void* k, const void* v,
                              const float* ks, const float* vs, int m, int base_pos, int nh, int nkv, int hd) {
    attention_flash_batch(out, qb, make_view(kv_mode, k, v, ks, vs), m, base_pos, nh, nkv, hd);
}

// ------------------------------------------------------------------ model
// E:3875-3939 Weights/LayerWeights; pointers into the caller's weights.bin image in the
// order P:341-407 reads it.
struct FoLayer {
    const float* attn_norm; const uint8_t *q, *k, *v; const float *qb, *kb, *vb;
    const uint8_t* o; const float* ffn_norm; const uint8_t *gate, *up, *down;
};
struct FoModel {
    FoConfig cfg;
    const float* embed; std::vector<FoLayer> layers; const float* final_norm; const uint8_t* lm_head;
    std::vector<float> freqs;
    int fast;
};
// E:3954-4015 KVCache (mode 0) and its fp16 / f32 stand-ins
struct FoKV {
    int mode, max_seq, kv_size, layers; int len;
    std::vector<std::vector<int8_t>> k8, v8; std::vector<std::vector<float>> ks, vs, kf, vf;
};

size_t fo_weights_bin_size(const FoConfig* c) {
    size_t h = c->hidden_size, qk = size_t(c->num_heads) * c->head_dim, kv = size_t(c->num_kv_heads) * c->head_dim;
    size_t ff = c->intermediate_size, V = c->vocab_size;
    auto mb = [&](int cat, size_t n, size_t k) { return n * row_bytes_of(pq_of(*c, cat), int(k)); };
    size_t per = h * 4 + mb(0, qk, h) + mb(1, kv, h) + mb(2, kv, h) + (c->qkv_bias ? (qk + 2 * kv) * 4 : 0) + mb(3, h, qk) + h * 4 +
                 mb(4, ff, h) + mb(5, ff, h) + mb(6, h, ff);
    return V * h * 4 + per * c->num_layers + h * 4 + mb(7, V, h);
}

FoModel* fo_model_create(const FoConfig* c, const uint8_t* blob, size_t len) {
    if (len != fo_weights_bin_size(c)) return nullptr;
    FoModel* m = new FoModel();
    m->cfg = *c;
    m->fast = 0;
    size_t h = c->hidden_size, qk = size_t(c->num_heads) * c->head_dim, kv = size_t(c->num_kv_heads) * c->head_dim;
    size_t ff = c->intermediate_size, V = c->vocab_size;
    auto mb = [&](int cat, size_t n, size_t k) { return n * row_bytes_of(pq_of(*c, cat), int(k)); };
    const uint8_t* p = blob;
    m->embed = (const float*)p; p += V * h * 4;
    for (int l = 0; l < c->num_layers; ++l) {
        FoLayer L{};
        L.attn_norm = (const float*)p; p += h * 4;
        L.q = p; p += mb(0, qk, h);
        L.k = p; p += mb(1, kv, h);
        L.v = p; p += mb(2, kv, h);
        if (c->qkv_bias) {
            L.qb = (const float*)p; p += qk * 4;
            L.kb = (const float*)p; p += kv * 4;
            L.vb = (const float*)p; p += kv * 4;
        }
        L.o = p; p += mb(3, h, qk);
        L.ffn_norm = (const float*)p; p += h * 4;
        L.gate = p; p += mb(4, ff, h);
        L.up = p; p += mb(5, ff, h);
        L.down = p; p += mb(6, h, ff);
        m->layers.push_back(L);
    }
    m->final_norm = (const float*)p; p += h * 4;
    m->lm_head = p;
    m->freqs.resize(c->head_dim / 2);
    rope_freqs(m->freqs.data(), c->head_dim, c->rope_theta);
    return m;
}
void fo_model_set_fast(FoModel* m, int fast) { m->fast = fast; }
void fo_model_destroy(FoModel* m) { delete m; }

FoKV* fo_kv_create(const FoModel* m, int mode) {
    FoKV* kv = new FoKV();
    kv->mode = mode;
    kv->max_seq = std::min(m->cfg.max_seq_len, 4096);  // E:178
    kv->kv_size = m->cfg.num_kv_heads * m->cfg.head_dim;
    kv->layers = m->cfg.num_layers;
    kv->len = 0;
    size_t n = size_t(kv->max_seq) * kv->kv_size;
    for (int l = 0; l < kv->layers; ++l) {
        if (mode == 0) {
            kv->k8.emplace_back(n, int8_t(0)); kv->v8.emplace_back(n, int8_t(0));
            kv->ks.emplace_back(kv->max_seq, 0.0f); kv->vs.emplace_back(kv->max_seq, 0.0f);
        } else {
            kv->kf.emplace_back(n, 0.0f); kv->vf.emplace_back(n, 0.0f);
        }
    }
    return kv;
}
void fo_kv_reset(FoKV* kv) { kv->len = 0; }
int fo_kv_len(const FoKV* kv) { return kv->len; }
void fo_kv_destroy(FoKV* kv) { delete kv; }
// copy out layer `l` K (which=0) or V (which=1) rows [0,len) as floats (dequantised for mode 0)
void fo_kv_read(const FoKV* kv, int l, int which, float* out) {
    size_t n = size_t(kv->len) * kv->kv_size;
    if (kv->mode == 0) {
        const auto& q = which ? kv->v8[l] : kv->k8[l];
        const auto& s = which ? kv->vs[l] : kv->ks[l];
        for (size_t i = 0; i < n; ++i) out[i] = float(q[i]) * s[i / kv->kv_size];
    } else {
        const auto& f = which ? kv->vf[l] : kv->kf[l];
        std::memcpy(out, f.data(), n * 4);
    }
}

static void kv_store(FoKV* kv, int l, int pos, const float* k, const float* v) {
    int n = kv->kv_size;
    if (kv->mode == 0) {  // E:4136-4153
        kv->ks[l][pos] = quantize_kv(k, n, &kv->k8[l][size_t(pos) * n]);
        kv->vs[l][pos] = quantize_kv(v, n, &kv->v8[l][size_t(pos) * n]);
    } else if (kv->mode == 1) {
        for (int i = 0; i < n; ++i) {
            kv->kf[l][size_t(pos) * n + i] = f16_bits_to_f32(f32_to_f16_bits(k[i]));
            kv->vf[l][size_t(pos) * n + i] = f16_bits_to_f32(f32_to_f16_bits(v[i]));
        }
    } else {
        std::memcpy(&kv->kf[l][size_t(pos) * n], k, n * 4);
        std::memcpy(&kv->vf[l][size_t(pos) * n], v, n * 4);
    }
}
static KVView kv_view(const FoKV* kv, int l) {
    KVView c{};
    c.mode = kv->mode;
    if (kv->mode == 0) { c.k8 = kv->k8[l].data(); c.v8 = kv->v8[l].data(); c.ks = kv->ks[l].data(); c.vs = kv->vs[l].data(); }
    else { c.kf = kv->kf[l].data(); c.vf = kv->vf[l].data(); }
    return c;
}

// E:4029-4500: one token.  `trace` (optional) receives the hidden state after every layer,
// [num_layers][hidden].  Returns 0, or -1 when the cache is full.
int fo_forward(const FoModel* m, FoKV* kv, uint32_t token, float* logits, float* trace) {
    const FoConfig& c = m->cfg;
    int h = c.hidden_size, qk = c.num_heads * c.head_dim, kvs = c.num_kv_heads * c.head_dim, ff = c.intermediate_size;
    int pos = kv->len;
    if (pos >= kv->max_seq) return -1;
    std::vector<float> hid(h), nrm(h), q(qk), k(kvs), v(kvs), ao(qk), ap(h), g(ff), u(ff), fh(ff), fo(h);
    std::memcpy(hid.data(), m->embed + size_t(token) * h, size_t(h) * 4);  // E:586-589
    for (int l = 0; l < c.num_layers; ++l) {
        const FoLayer& L = m->layers[l];
        rms_norm(nrm.data(), hid.data(), L.attn_norm, h, c.rms_norm_eps);
        matmul_mat(pq_of(c, 0), q.data(), 1, nrm.data(), L.q, h, qk, m->fast);
        matmul_mat(pq_of(c, 1), k.data(), 1, nrm.data(), L.k, h, kvs, m->fast);
        matmul_mat(pq_of(c, 2), v.data(), 1, nrm.data(), L.v, h, kvs, m->fast);
        if (c.qkv_bias) {  // E:4108-4118
            for (int i = 0; i < qk; ++i) q[i] += L.qb[i];
            for (int i = 0; i < kvs; ++i) k[i] += L.kb[i];
            for (int i = 0; i < kvs; ++i) v[i] += L.vb[i];
        }
        rope(q.data(), pos, c.head_dim, c.num_heads, m->freqs.data());
        rope(k.data(), pos, c.head_dim, c.num_kv_heads, m->freqs.data());
        kv_store(kv, l, pos, k.data(), v.data());
        KVView view = kv_view(kv, l);
        if (c.sliding_window > 0) attention_sliding(ao.data(), q.data(), view, pos + 1, c.sliding_window, c.num_heads, c.num_kv_heads, c.head_dim);  // E:4156
        else if (c.max_seq_len > 512) attention_flash(ao.data(), q.data(), view, pos + 1, c.num_heads, c.num_kv_heads, c.head_dim);  // E:126-128
        else attention_plain(ao.data(), q.data(), view, pos + 1, c.num_heads, c.num_kv_heads, c.head_dim);
        matmul_mat(pq_of(c, 3), ap.data(), 1, ao.data(), L.o, qk, h, m->fast);
        residual_add(hid.data(), ap.data(), h);
        rms_norm(nrm.data(), hid.data(), L.ffn_norm, h, c.rms_norm_eps);
        matmul_mat(pq_of(c, 4), g.data(), 1, nrm.data(), L.gate, h, ff, m->fast);
        matmul_mat(pq_of(c, 5), u.data(), 1, nrm.data(), L.up, h, ff, m->fast);
        silu_mul(fh.data(), g.data(), u.data(), ff);
        matmul_mat(pq_of(c, 6), fo.data(), 1, fh.data(), L.down, ff, h, m->fast);
        residual_add(hid.data(), fo.data(), h);
        if (trace) std::memcpy(trace + size_t(l) * h, hid.data(), size_t(h) * 4);
    }
    rms_norm(nrm.data(), hid.data(), m->final_norm, h, c.rms_norm_eps);
    matmul_mat(pq_of(c, 7), logits, 1, nrm.data(), m->lm_head, h, c.vocab_size, m->fast);
    kv->len += 1;
    return 0;
}

// E:5118-5486: batched prefill.  `trace` (optional): [num_layers][m][hidden].
static int forward_prefill_batched(const FoModel* m, FoKV* kv, const uint32_t* tokens, int n, float* logits, float* trace) {
    const FoConfig& c = m->cfg;
    int h = c.hidden_size, qk = c.num_heads * c.head_dim, kvs = c.num_kv_heads * c.head_dim, ff = c.intermediate_size;
    int base = kv->len;
    if (base + n > kv->max_seq) return -1;
    size_t M = size_t(n);
    std::vector<float> hid(M * h), nrm(M * h), q(M * qk), k(M * kvs), v(M * kvs), ao(M * qk), ap(M * h), g(M * ff), u(M * ff), fh(M * ff), fo(M * h);
    for (int r = 0; r < n; ++r) std::memcpy(&hid[size_t(r) * h], m->embed + size_t(tokens[r]) * h, size_t(h) * 4);
    for (int l = 0; l < c.num_layers; ++l) {
        const FoLayer& L = m->layers[l];
#pragma omp parallel for
        for (int r = 0; r < n; ++r) rms_norm(&nrm[size_t(r) * h], &hid[size_t(r) * h], L.attn_norm, h, c.rms_norm_eps);
        matmul_mat(pq_of(c, 0), q.data(), n, nrm.data(), L.q, h, qk, m->fast);
        matmul_mat(pq_of(c, 1), k.data(), n, nrm.data(), L.k, h, kvs, m->fast);
        matmul_mat(pq_of(c, 2), v.data(), n, nrm.data(), L.v, h, kvs, m->fast);
#pragma omp parallel for
        for (int r = 0; r < n; ++r) {  // E:5232-5285
            float *qr = &q[size_t(r) * qk], *kr = &k[size_t(r) * kvs], *vr = &v[size_t(r) * kvs];
            if (c.qkv_bias) {
                for (int i = 0; i < qk; ++i) qr[i] += L.qb[i];
                for (int i = 0; i < kvs; ++i) kr[i] += L.kb[i];
                for (int i = 0; i < kvs; ++i) vr[i] += L.vb[i];
            }
            rope(qr, base + r, c.head_dim, c.num_heads, m->freqs.data());
            rope(kr, base + r, c.head_dim, c.num_kv_heads, m->freqs.data());
            kv_store(kv, l, base + r, kr, vr);
        }
        KVView view = kv_view(kv, l);
        if (c.max_seq_len > 512 && c.sliding_window <= 0) {
            attention_flash_batch(ao.data(), q.data(), view, n, base, c.num_heads, c.num_kv_heads, c.head_dim);
        } else if (c.sliding_window > 0) {  // E:5312
            attention_sliding_batch(ao.data(), q.data(), view, n, base, c.sliding_window, c.num_heads, c.num_kv_heads, c.head_dim);
        } else {  // E: short-context fallback, per-token plain attention
#pragma omp parallel for
            for (int r = 0; r < n; ++r)
                attention_plain(&ao[size_t(r) * qk], &q[size_t(r) * qk], view, base + r + 1, c.num_heads, c.num_kv_heads, c.head_dim);
        }
        matmul_mat(pq_of(c, 3), ap.data(), n, ao.data(), L.o, qk, h, m->fast);
        for (int r = 0; r < n; ++r) residual_add(&hid[size_t(r) * h], &ap[size_t(r) * h], h);
#pragma omp parallel for
        for (int r = 0; r < n; ++r) rms_norm(&nrm[size_t(r) * h], &hid[size_t(r) * h], L.ffn_norm, h, c.rms_norm_eps);
        matmul_mat(pq_of(c, 4), g.data(), n, nrm.data(), L.gate, h, ff, m->fast);
        matmul_mat(pq_of(c, 5), u.data(), n, nrm.data(), L.up, h, ff, m->fast);
#pragma omp parallel for
        for (int r = 0; r < n; ++r) silu_mul(&fh[size_t(r) * ff], &g[size_t(r) * ff], &u[size_t(r) * ff], ff);
        matmul_mat(pq_of(c, 6), fo.data(), n, fh.data(), L.down, ff, h, m->fast);
        for (int r = 0; r < n; ++r) residual_add(&hid[size_t(r) * h], &fo[size_t(r) * h], h);
        if (trace) std::memcpy(trace + size_t(l) * M * h, hid.data(), M * h * 4);
    }
    std::vector<float> last(h);
    rms_norm(last.data(), &hid[(M - 1) * h], m->final_norm, h, c.rms_norm_eps);  // E:5439-5443
    matmul_mat(pq_of(c, 7), logits, 1, last.data(), m->lm_head, h, c.vocab_size, m->fast);
    kv->len += n;
    return 0;
}

// E:4553-4587: prompts of at least PREFILL_BATCH_THRESHOLD (8) tokens take the batched
// path unless force_per_token is set (the reference's FORGE_BATCHED_PREFILL=0 switch);
// shorter ones run the per-token loop and keep the last token's logits (E:4626-4814).
int fo_forward_prefill(const FoModel* m, FoKV* kv, const uint32_t* tokens, int n, float* logits, float* trace, int force_per_token) {
    if (n <= 0) return -2;
    if (!force_per_token && n >= 8) return forward_prefill_batched(m, kv, tokens, n, logits, trace);
    int h = m->cfg.hidden_size, L = m->cfg.num_layers;
    std::vector<float> tr(trace ? size_t(L) * h : 0);
    for (int r = 0; r < n; ++r) {
        int rc = fo_forward(m, kv, tokens[r], logits, trace ? tr.data() : nullptr);
        if (rc) return rc;
        if (trace)
            for (int l = 0; l < L; ++l) std::memcpy(trace + (size_t(l) * n + r) * h, &tr[size_t(l) * h], size_t(h) * 4);
    }
    return 0;
}

int fo_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Host threads the row / head loops may use (rayon's pool size in the reference).  Launchers that pin
// OMP_NUM_THREADS=1 for their workers (torchrun) would otherwise leave the CPU baseline on one core.
void fo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"
