// Host-side K-quant quantisers of the weights exporter: f32 -> Q4_K / Q6_K super-blocks with the rules of
// quantize_f32_to_q4_k (crates/forgellm-frontend/src/weight_loader.rs:1773-1900, per-sub-block fit
// make_qkx2_quants :1663-1771) and quantize_f32_to_q6_k (:2025-2125, make_q6k_quants :1989-2010).  The exporter
// needs them when a tensor's format differs from the format its projection category is stored in
// (load_from_file_mixed_per_tensor, :193-218).  Plain f32 arithmetic in the reference's order, one multiply and one
// add per rounding; super-blocks are independent and spread over the host threads.
#include <cmath>
#include <cstring>

#include "common.cuh"

using namespace forge;

namespace {

inline float half_round(float x) { return __half2float(__float2half_rn(x)); }
inline void put_half(uint8_t* p, float x) {
    const uint16_t b = __half_as_ushort(__float2half_rn(x));
    p[0] = uint8_t(b); p[1] = uint8_t(b >> 8);
}
inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

// ---- Q4_K: a 32-element sub-block as scale * L - offset with L in 0..15.
// Start from the [min(x, 0), max] bracket, then try 21 slightly narrower / wider level spacings; for each, refit
// (scale, min) to its levels by two-parameter least squares (min held at 0 if it comes out positive) and keep the
// candidate with the smallest squared error.
struct SubFit { float scale, offset; uint8_t level[32]; };

void fit_sub_q4(const float* x, SubFit& out) {
    float lo = x[0], hi = x[0];
    for (int i = 1; i < 32; ++i) { if (x[i] < lo) lo = x[i]; if (x[i] > hi) hi = x[i]; }
    if (hi == lo) { out.scale = 0.f; out.offset = -lo; memset(out.level, 0, 32); return; }
    if (lo > 0.f) lo = 0.f;
    const float span = hi - lo;
    float inv = 15.0f / span;
    float best_scale = 1.0f / inv, best_lo = lo, best_err = 0.f;
    for (int i = 0; i < 32; ++i) {
        const float l = clampf(roundf((x[i] - lo) * inv), 0.f, 15.f);
        out.level[i] = uint8_t(l);
        const float e = best_scale * l + lo - x[i];
        best_err += e * e;
    }
    uint8_t trial[32];
    for (int step = 0; step <= 20; ++step) {
        inv = (-1.0f + 0.1f * float(step) + 15.0f) / span;
        float sl = 0.f, sl2 = 0.f, sx = 0.f, sxl = 0.f;
        for (int i = 0; i < 32; ++i) {
            const float l = clampf(roundf((x[i] - lo) * inv), 0.f, 15.f);
            trial[i] = uint8_t(l);
            sl += l; sl2 += l * l; sx += x[i]; sxl += l * x[i];
        }
        const float det = 32.0f * sl2 - sl * sl;
        if (!(det > 0.f)) continue;
        float s = (32.0f * sxl - sx * sl) / det;
        float m = (sl2 * sx - sl * sxl) / det;
        if (m > 0.f) { m = 0.f; if (sl2 > 0.f) s = sxl / sl2; }
        if (!(s > 0.f)) continue;  // a negative scale would mirror the unsigned levels
        float err = 0.f;
        for (int i = 0; i < 32; ++i) { const float e = s * float(trial[i]) + m - x[i]; err += e * e; }
        if (err < best_err) { best_err = err; best_scale = s; best_lo = m; memcpy(out.level, trial, 32); }
    }
    out.scale = best_scale;
    out.offset = -best_lo;
}

void quantize_superblock_q4_k(const float* x, uint8_t* out) {
    SubFit fit[8];
    float top_scale = 0.f, top_offset = 0.f;
    for (int j = 0; j < 8; ++j) {
        fit_sub_q4(x + 32 * j, fit[j]);
        if (fit[j].scale > top_scale) top_scale = fit[j].scale;
        if (fit[j].offset > top_offset) top_offset = fit[j].offset;
    }
    const float to_sc = top_scale > 0.f ? 63.0f / top_scale : 0.f, to_mn = top_offset > 0.f ? 63.0f / top_offset : 0.f;
    const float d = top_scale > 0.f ? top_scale / 63.0f : 0.f, dmin = top_offset > 0.f ? top_offset / 63.0f : 0.f;
    uint8_t sc[8], mn[8];
    for (int j = 0; j < 8; ++j) {
        sc[j] = uint8_t(clampf(roundf(fit[j].scale * to_sc), 0.f, 63.f));
        mn[j] = uint8_t(clampf(roundf(fit[j].offset * to_mn), 0.f, 63.f));
    }
    // the levels are taken again against the scales as they will be read back (f16 d / dmin, 6-bit factors)
    const float d16 = half_round(d), dmin16 = half_round(dmin);
    uint8_t lv[8][32];
    for (int j = 0; j < 8; ++j) {
        const float s = d16 * float(sc[j]);
        if (s == 0.f) { memset(lv[j], 0, 32); continue; }
        const float inv = 1.0f / s, off = dmin16 * float(mn[j]);
        for (int i = 0; i < 32; ++i) lv[j][i] = uint8_t(clampf(roundf((x[32 * j + i] + off) * inv), 0.f, 15.f));
    }
    put_half(out, d);
    put_half(out + 2, dmin);
    for (int i = 0; i < 4; ++i) {  // the inverse of the 6-bit unpacking (emit.rs:3013-3021)
        out[4 + i] = uint8_t((sc[i] & 63) | (((sc[i + 4] >> 4) & 3) << 6));
        out[8 + i] = uint8_t((mn[i] & 63) | (((mn[i + 4] >> 4) & 3) << 6));
        out[12 + i] = uint8_t((sc[i + 4] & 15) | ((mn[i + 4] & 15) << 4));
    }
    for (int c = 0; c < 4; ++c)
        for (int i = 0; i < 32; ++i) out[16 + 32 * c + i] = uint8_t((lv[2 * c][i] & 15) | ((lv[2 * c + 1][i] & 15) << 4));
}

// ---- Q6_K: sixteen 16-element groups, each scale = (value of largest magnitude) / -32; the group scales become int8
// multiples of d = (group scale of largest magnitude) / -128, and the 6-bit levels are taken against d16 * int8.
void quantize_superblock_q6_k(const float* x, uint8_t* out) {
    float gs[16];
    float top = 0.f, top_abs = 0.f;
    for (int j = 0; j < 16; ++j) {
        float peak = 0.f, peak_abs = 0.f;
        for (int i = 0; i < 16; ++i) { const float a = fabsf(x[16 * j + i]); if (a > peak_abs) { peak_abs = a; peak = x[16 * j + i]; } }
        gs[j] = peak_abs < 1e-30f ? 0.f : 1.0f / (-32.0f / peak);
        if (fabsf(gs[j]) > top_abs) { top_abs = fabsf(gs[j]); top = gs[j]; }
    }
    if (top_abs < 1e-30f) { memset(out, 0, 210); return; }
    const float to_int = -128.0f / top;
    const float d = 1.0f / to_int;
    put_half(out + 208, d);
    const float d16 = half_round(d);
    int8_t level[256];
    for (int j = 0; j < 16; ++j) {
        int q = int(roundf(to_int * gs[j]));
        q = q < -128 ? -128 : (q > 127 ? 127 : q);
        out[192 + j] = uint8_t(int8_t(q));
        const float s = d16 * float(q);
        for (int i = 0; i < 16; ++i) {
            int l = 0;
            if (s != 0.f) { l = int(roundf((1.0f / s) * x[16 * j + i])); l = l < -32 ? -32 : (l > 31 ? 31 : l); }
            level[16 * j + i] = int8_t(l);
        }
    }
    for (int half = 0; half < 2; ++half)  // 128 values: low nibbles of (l, l+64) and (l+32, l+96) share bytes, top bits four to a byte
        for (int l = 0; l < 32; ++l) {
            const int8_t* v = level + 128 * half + l;
            const uint8_t q1 = uint8_t(v[0] + 32), q2 = uint8_t(v[32] + 32), q3 = uint8_t(v[64] + 32), q4 = uint8_t(v[96] + 32);
            out[64 * half + l] = uint8_t((q1 & 15) | ((q3 & 15) << 4));
            out[64 * half + l + 32] = uint8_t((q2 & 15) | ((q4 & 15) << 4));
            out[128 + 32 * half + l] = uint8_t((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
        }
}

}  // namespace

extern "C" {

int32_t forge_quantize_q4_k_host(const float* x, size_t n, uint8_t* out) {
    if (!x || !out || (n % 256)) { set_error("forge_quantize_q4_k_host: n must be a multiple of 256"); return FORGE_ERR_INVALID_ARG; }
    const long nsb = long(n / 256);
#pragma omp parallel for schedule(static)
    for (long b = 0; b < nsb; ++b) quantize_superblock_q4_k(x + size_t(b) * 256, out + size_t(b) * 144);
    return FORGE_OK;
}

int32_t forge_quantize_q6_k_host(const float* x, size_t n, uint8_t* out) {
    if (!x || !out || (n % 256)) { set_error("forge_quantize_q6_k_host: n must be a multiple of 256"); return FORGE_ERR_INVALID_ARG; }
    const long nsb = long(n / 256);
#pragma omp parallel for schedule(static)
    for (long b = 0; b < nsb; ++b) quantize_superblock_q6_k(x + size_t(b) * 256, out + size_t(b) * 210);
    return FORGE_OK;
}

}  // extern "C"
