// Batch-1 decode (forward(), crates/forgellm-codegen-cpu/src/emit.rs:4029-4500, and the greedy loop around it,
// crates/forgellm-codegen-cpu/src/project.rs:727-751) as ONE persistent kernel for any number of consecutive steps.
//
// A CTA per SM, launched cooperatively so that all of them are resident.  The producer warp of every CTA streams that
// CTA's share of every projection of every layer of every step through the shared-memory ring without ever waiting for
// activations (weights are static), so HBM keeps streaming across the dependent operators.  The sixteen consumer warps
// walk the operators
//   [RMSNorm + QKV GEMV + bias/RoPE/KV append] | attention | [O GEMV] | [RMSNorm + gate/up GEMV + SiLU*up] | [down GEMV]
// per layer, then [RMSNorm + lm_head GEMV + arg-max].
//
// There is no grid-wide barrier.  Every vector that crosses CTAs (q, the new k/v row, the attention partials, the O,
// SiLU and down outputs, the per-CTA arg-max) is published as {value, tag} pairs in global memory, each pair written
// with one 8-byte store; tag = epoch + step is unique per step and each (layer, operator) has its own buffer, so a
// reader simply polls the pairs it needs until the tag matches - the poll IS the load, no fence and no flag are
// involved - and a CTA starts an operator the moment its own inputs have arrived.  Every wait is bounded: when it runs
// out the CTA raises the error word, stops waiting anywhere else, and the kernel drains.
//
// The residual stream never leaves the SM: every CTA keeps the whole hidden vector in shared memory and adds the O and
// down outputs to it as they arrive (all CTAs add the same values in the same order, so they hold the same bits).
// Attention: a unit is (KV head, context split); at most four splits, whose (m, l, acc) partials are merged by the
// readers while they stage the O projection's input.  The unit that covers the newest position takes this step's k/v
// from the pairs (the fp16 cache row is written for the later steps).
// Greedy decoding (argmax with the last-index tie rule, project.rs:501-503): every CTA publishes the best logit of its
// rows, every CTA reads all of them and so knows the next token without a host round trip.
#include "gemv_core.cuh"

namespace forge {

namespace {

using namespace core;

constexpr int kGC = 4;          // query heads per pass over a KV split
constexpr int kMaxQ = 512;      // query values per KV group (heads per group x head_dim)
constexpr int kMaxSplits = 4;   // context splits per KV head
constexpr int kMaxHS = 512;     // heads x splits the merge handles

template <int HD> struct Seg { static constexpr int W = (HD == 64) ? 8 : 16, ACTIVE = HD / 8, RPW = 32 / W; };

// ------------------------------------------------------------------ pairs
__device__ __forceinline__ void st_pair(uint2* p, float v, uint32_t tag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ void st_pair2(uint2* p, float a, float b, uint32_t tag) {  // p 16-byte aligned
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(a)), "r"(tag), "r"(__float_as_uint(b)), "r"(tag) : "memory");
}
struct Waiter {
    uint32_t tag, limit;
    int* sh_err;   // shared: set when any wait of this CTA gave up
    int* g_err;    // global error word
};
// The two pairs at p (16-byte aligned), once both carry the tag.  Bounded: gives up after `limit` polls, or as soon
// as this CTA or another one has reported an error; the values are then zero.
__device__ __forceinline__ float2 wait2(const uint2* p, const Waiter& w) {
    for (uint32_t i = 0; i < w.limit; ++i) {
        uint4 v;
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
        if (v.y == w.tag && v.w == w.tag) return make_float2(__uint_as_float(v.x), __uint_as_float(v.z));
        if (i >= 4) {
            __nanosleep(32);
            if ((i & 63) == 4 && *reinterpret_cast<volatile int*>(w.sh_err)) break;
            if ((i & 1023) == 1023 && __ldcg(w.g_err)) break;
        }
    }
    *reinterpret_cast<volatile int*>(w.sh_err) = 1;
    atomicExch(w.g_err, 1);
    return make_float2(0.f, 0.f);
}

// ------------------------------------------------------------------ staging fills (all consumer threads)
// The caller runs csync() first: the previous contents of the fragment area are no longer read (the same barrier
// publishes the operator description that warp 0 prefetched).
// x = embedding row; also starts the residual stream
__device__ __forceinline__ FillStat fill_embed(uint2* xf, float* resid, const float* row, int K, const float* norm_w) {
    float* xraw = reinterpret_cast<float*>(xf);
    FillStat st;
    for (int e = threadIdx.x * 4; e < K; e += kCT * 4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(row + e));
        *reinterpret_cast<float4*>(resid + e) = v;
        fill_note(st, v, norm_w, e);
        *reinterpret_cast<float4*>(xraw + e) = v;
    }
    return st;
}
// residual stream += the published vector; x = the new residual stream
__device__ __forceinline__ FillStat fill_add_pairs(uint2* xf, float* resid, const uint2* src, int K, const float* norm_w, const Waiter& w) {
    float* xraw = reinterpret_cast<float*>(xf);
    FillStat st;
    for (int e = threadIdx.x * 4; e < K; e += kCT * 4) {
        const float2 a = wait2(src + e, w), b = wait2(src + e + 2, w);
        float4 v = *reinterpret_cast<const float4*>(resid + e);
        v.x += a.x; v.y += a.y; v.z += b.x; v.w += b.y;
        *reinterpret_cast<float4*>(resid + e) = v;
        fill_note(st, v, norm_w, e);
        *reinterpret_cast<float4*>(xraw + e) = v;
    }
    return st;
}
// x = the published vector
__device__ __forceinline__ FillStat fill_pairs(uint2* xf, const uint2* src, int K, const Waiter& w) {
    float* xraw = reinterpret_cast<float*>(xf);
    FillStat st;
    for (int e = threadIdx.x * 4; e < K; e += kCT * 4) {
        const float2 a = wait2(src + e, w), b = wait2(src + e + 2, w);
        const float4 v = make_float4(a.x, a.y, b.x, b.y);
        fill_note(st, v, nullptr, e);
        *reinterpret_cast<float4*>(xraw + e) = v;
    }
    return st;
}
// x = attention output: per head, the softmax-weighted merge of the context splits' partials (m, l, acc[HD])
template <int HD>
__device__ __forceinline__ FillStat fill_attention_merge(uint2* xf, const uint2* xatt, int nq, int S, float (*s_w)[kMaxHS], const Waiter& w) {
    float* xraw = reinterpret_cast<float*>(xf);
    FillStat st;
    csync();  // the previous contents of the fragment area and of s_w are no longer read
    const int i1 = threadIdx.x;  // (head, split) handled by this thread; nq * S <= kMaxHS = kCT
    if (i1 < nq * S) {
        const float2 ml = wait2(xatt + size_t(i1) * (HD + 2), w);
        s_w[0][i1] = ml.x;
        s_w[1][i1] = ml.y;
    }
    csync();
    float wt = 0.f;
    if (i1 < nq * S) {
        const int head = i1 / S;
        float M = -INFINITY, L = 0.f;
        for (int s = 0; s < S; ++s) M = fmaxf(M, s_w[0][head * S + s]);
        for (int s = 0; s < S; ++s) {
            const float m = s_w[0][head * S + s];
            L += (m == -INFINITY) ? 0.f : s_w[1][head * S + s] * expf(m - M);
        }
        const float m = s_w[0][i1];
        wt = (m == -INFINITY) ? 0.f : expf(m - M) * (1.0f / L);
    }
    csync();
    if (i1 < nq * S) s_w[0][i1] = wt;
    csync();
    const int K = nq * HD;
    for (int e = threadIdx.x * 4; e < K; e += kCT * 4) {
        const int head = e / HD, dd = e % HD;
        const uint2* a0 = xatt + size_t(head) * S * (HD + 2) + 2 + dd;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kMaxSplits; ++s) {
            if (s < S) {
                const float2 lo = wait2(a0 + size_t(s) * (HD + 2), w), hi = wait2(a0 + size_t(s) * (HD + 2) + 2, w);
                const float ws = s_w[0][head * S + s];
                v.x += lo.x * ws; v.y += lo.y * ws; v.z += hi.x * ws; v.w += hi.y * ws;
            }
        }
        fill_note(st, v, nullptr, e);
        *reinterpret_cast<float4*>(xraw + e) = v;
    }
    return st;
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// attention_flash (emit.rs:657-715) for the current token, split over the CTAs: a unit is (kv head, context split).
// The unit waits for its group's queries (and, if it covers the newest position, for this step's k / v), runs the
// online softmax over its positions of the fp16 cache and publishes (m, l, acc) per query head.  `buf` is shared
// memory of at least (16 * kGC * (HD + 2) + kMaxQ + 2 * HD) floats.
template <int HD>
__device__ void attention_phase(const FlowParams& p, int layer, int pos, const uint2* xq, const uint2* xkv, uint2* xatt, float* buf,
                                const Waiter& w) {
    constexpr int W = Seg<HD>::W, ACTIVE = Seg<HD>::ACTIVE, RPW = Seg<HD>::RPW;
    constexpr int PARTS = kConsumerWarps * RPW;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = lane / W, sl = lane % W;
    const bool act = sl < ACTIVE;
    const int G = p.nq / p.nkv, kvd = p.kvd, S = p.attn_splits;
    const int n_ctx = pos + 1;
    int chunk = (n_ctx + S - 1) / S;
    chunk = (chunk + PARTS - 1) / PARTS * PARTS;
    const __half* kp = p.k_pool + size_t(layer) * p.layer_stride;
    const __half* vp = p.v_pool + size_t(layer) * p.layer_stride;
    const float scale = 1.0f / sqrtf(float(HD));
    float (*s_ml)[kGC][2] = reinterpret_cast<float (*)[kGC][2]>(buf);
    float (*s_acc)[kGC][HD] = reinterpret_cast<float (*)[kGC][HD]>(buf + kConsumerWarps * kGC * 2);
    float* sq = buf + kConsumerWarps * kGC * (HD + 2);   // [G][HD] queries of the group
    float* snew = sq + kMaxQ;                            // [2][HD] this step's k and v (fp16-rounded)

    for (int u = blockIdx.x; u < p.nkv * S; u += gridDim.x) {
        const int kvh = u / S, split = u % S;
        const int t_begin = split * chunk, t_end = min(n_ctx, t_begin + chunk);
        const bool covers = pos >= t_begin && pos < t_end;
        csync();  // shared buffers of the previous unit (or operator) are no longer read
        if (t_begin < t_end) {
            const int npairs = (G * HD + (covers ? 2 * HD : 0)) / 2;
            for (int pr = threadIdx.x; pr < npairs; pr += kCT) {
                int e = 2 * pr;
                if (e < G * HD) {
                    const float2 v = wait2(xq + size_t(kvh) * G * HD + e, w);
                    sq[e] = v.x; sq[e + 1] = v.y;
                } else {
                    e -= G * HD;
                    const int which = e / HD, d = e % HD;
                    const float2 v = wait2(xkv + size_t(which) * kvd + kvh * HD + d, w);
                    snew[which * HD + d] = v.x; snew[which * HD + d + 1] = v.y;
                }
            }
        }
        csync();
        for (int g0 = 0; g0 < G; g0 += kGC) {
            const int gc = min(kGC, G - g0);
            float q[kGC][8], acc[kGC][8], mi[kGC], li[kGC];
#pragma unroll
            for (int g = 0; g < kGC; ++g) {
                mi[g] = -INFINITY; li[g] = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) { acc[g][i] = 0.f; q[g][i] = (g < gc && act && t_begin < t_end) ? sq[(g0 + g) * HD + sl * 8 + i] : 0.f; }
            }
            constexpr int UNR = 2;
            for (int base = t_begin + warp * RPW; base < t_end; base += PARTS * UNR) {
                uint4 kr[UNR], vr[UNR];
#pragma unroll
                for (int un = 0; un < UNR; ++un) {
                    const int t = base + un * PARTS + seg;
                    kr[un] = make_uint4(0, 0, 0, 0);
                    vr[un] = make_uint4(0, 0, 0, 0);
                    if (t < t_end && t != pos && act) {
                        const size_t row = size_t(p.page_table[t / FORGE_KV_PAGE]) * FORGE_KV_PAGE + t % FORGE_KV_PAGE;
                        const size_t off = row * kvd + kvh * HD + sl * 8;
                        kr[un] = __ldcg(reinterpret_cast<const uint4*>(kp + off));
                        vr[un] = __ldcg(reinterpret_cast<const uint4*>(vp + off));
                    }
                }
#pragma unroll
                for (int un = 0; un < UNR; ++un) {
                    const int t = base + un * PARTS + seg;
                    const bool valid = t < t_end;
                    float kf[8], vf[8];
                    unpack8(kr[un], kf);
                    unpack8(vr[un], vf);
                    if (t == pos && act) {  // this step's row: taken from the pairs, not from the cache
#pragma unroll
                        for (int i = 0; i < 8; ++i) { kf[i] = snew[sl * 8 + i]; vf[i] = snew[HD + sl * 8 + i]; }
                    }
#pragma unroll
                    for (int g = 0; g < kGC; ++g) {
                        float s = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) s += q[g][i] * kf[i];
#pragma unroll
                        for (int o = W / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                        s *= scale;
                        if (valid && g < gc) {
                            float mn = fmaxf(mi[g], s);
                            float es = expf(mi[g] - mn), pr = expf(s - mn);
                            mi[g] = mn;
                            li[g] = li[g] * es + pr;
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * es + pr * vf[i];
                        }
                    }
                }
            }
            // merge the RPW segments of the warp (butterfly over lane offsets W, 2W, ...)
#pragma unroll
            for (int off = W; off < 32; off <<= 1) {
#pragma unroll
                for (int g = 0; g < kGC; ++g) {
                    const float mo = __shfl_xor_sync(0xffffffffu, mi[g], off), lo = __shfl_xor_sync(0xffffffffu, li[g], off);
                    const float M = fmaxf(mi[g], mo);
                    const float a = (mi[g] == -INFINITY) ? 0.f : expf(mi[g] - M), bq = (mo == -INFINITY) ? 0.f : expf(mo - M);
                    li[g] = li[g] * a + lo * bq;
                    mi[g] = M;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][i], off);
                        acc[g][i] = acc[g][i] * a + ao * bq;
                    }
                }
            }
            csync();  // the merge buffer of the previous pass is no longer read
            if (seg == 0) {
#pragma unroll
                for (int g = 0; g < kGC; ++g) {
                    if (sl == 0) { s_ml[warp][g][0] = mi[g]; s_ml[warp][g][1] = li[g]; }
                    if (act) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) s_acc[warp][g][sl * 8 + i] = acc[g][i];
                    }
                }
            }
            csync();
            for (int idx = threadIdx.x; idx < gc * HD; idx += kCT) {
                const int g = idx / HD, dd = idx % HD;
                float M = -INFINITY;
#pragma unroll
                for (int wi = 0; wi < kConsumerWarps; ++wi) M = fmaxf(M, s_ml[wi][g][0]);
                float L = 0.f, A = 0.f;
#pragma unroll
                for (int wi = 0; wi < kConsumerWarps; ++wi) {
                    const float m = s_ml[wi][g][0];
                    const float wt = (m == -INFINITY) ? 0.f : expf(m - M);
                    L += s_ml[wi][g][1] * wt;
                    A += s_acc[wi][g][dd] * wt;
                }
                uint2* wsp = xatt + (size_t(kvh * G + g0 + g) * S + split) * (HD + 2);
                st_pair(wsp + 2 + dd, A, w.tag);
                if (dd == 0) st_pair2(wsp, M, L, w.tag);
            }
        }
    }
}

template <int QUANT, int HD>
__global__ void __launch_bounds__(kThreads, 1) decode_flow_kernel(FlowParams p) {
    using T = Tile<QUANT>;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ Shared sh;
    __shared__ int4 s_xoff[QUANT == FORGE_Q4_0 ? 2 * kMaxKB : 1];
    __shared__ float s_w[2][kMaxHS];
    __shared__ float s_best[kConsumerWarps];
    __shared__ int s_bidx[kConsumerWarps];
    __shared__ float2 s_rope[HD / 2];
    __shared__ Phase s_ph[2];      // the current operator's description and, prefetched under it, the next one's
    unsigned char* ring = smem;
    const int region_floats = max(p.max_kb * 32, kConsumerWarps * kGC * (HD + 2) + kMaxQ + 2 * HD);
    uint2* xf = reinterpret_cast<uint2*>(smem + size_t(T::STAGES) * T::STAGE_BYTES);
    float* resid = reinterpret_cast<float*>(xf) + region_floats;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&sh.full_bar[s], 1); mbar_init(&sh.empty_bar[s], kConsumerWarps); }
        sh.err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int L = p.num_layers, NPH = 4 * L + 1;
    int cc = 0;

    if (warp == kConsumerWarps) {
        // ---- producer: every projection of every layer of every step, in order, bounded only by ring space
        if (lane == 0) {
            bool ok = true;
            for (int s = 0; s < p.n_steps && ok; ++s)
                for (int i = 0; i < NPH && ok; ++i) {
                    const Phase ph = p.phases[i];
                    ok = produce_phase<QUANT>(ph, sh, ring, cc);
                }
        }
        return;
    }

    // ---- consumers
    const int pos0 = p.seq_len[0];
    const int step0 = p.step ? *p.step : 0;
    uint32_t tok = *p.tok;
    const int h = p.h, qk = p.qk, kvd = p.kvd;
    const size_t natt = size_t(p.nq) * p.attn_splits * (HD + 2);
    // operator i's description moves into s_ph[i & 1] while operator i - 1 runs (warp 0 copies, the csync that opens
    // every staging fill publishes it)
    auto fetch_phase = [&](int i) {
        if (warp == 0) {
            const uint32_t* src = reinterpret_cast<const uint32_t*>(p.phases + (i % NPH));
            uint32_t* dst = reinterpret_cast<uint32_t*>(&s_ph[i & 1]);
            for (int j = lane; j < int(sizeof(Phase) / 4); j += 32) dst[j] = __ldg(src + j);
        }
    };
    fetch_phase(0);
    int pi = 0;   // running operator index (parity selects the s_ph slot)
    auto noop = [](int, float, float) {};
    (void)noop;
    for (int s = 0; s < p.n_steps; ++s) {
        const int pos = pos0 + s;
        Waiter w{p.epoch + uint32_t(s), p.wait_limit, &sh.err, p.err};
        const uint32_t tag = w.tag;
        if (blockIdx.x == 0 && tid == 0 && p.hist) p.hist[step0 + s] = tok;
        if (tid < HD / 2) s_rope[tid] = __ldg(reinterpret_cast<const float2*>(p.rope) + size_t(pos) * (HD / 2) + tid);
        const int page = p.page_table[pos / FORGE_KV_PAGE];
        const size_t new_row = (size_t(page) * FORGE_KV_PAGE + pos % FORGE_KV_PAGE) * kvd;
        for (int l = 0; l < L; ++l) {
            uint2* xq = p.xbuf + size_t(l) * p.x_layer_stride;
            uint2* xkv = xq + qk;
            uint2* xatt = xkv + 2 * kvd;
            uint2* xo = xatt + natt;
            uint2* xact = xo + h;
            uint2* xdown = xact + p.ff;
            {   // residual stream (+ the previous layer's down output) -> RMSNorm -> QKV -> bias, RoPE -> q pairs, k/v pairs + cache
                csync();
                const Phase& ph = s_ph[pi & 1];
                const FillStat st = l == 0 ? fill_embed(xf, resid, p.embed + size_t(tok) * h, h, ph.a.norm_w)
                                           : fill_add_pairs(xf, resid, xdown - p.x_layer_stride, h, ph.a.norm_w, w);
                const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, ph.a.norm_w, ph.a.eps);
                fetch_phase(pi + 1);
                const float* bias = ph.a.bias;
                __half* kc = p.k_pool + size_t(l) * p.layer_stride + new_row;
                __half* vc = p.v_pool + size_t(l) * p.layer_stride + new_row;
                const int N = ph.N;
                consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, [&](int row, float v, float partner) {
                    if (row >= N || (row & 1)) return;   // the thread of the even row handles the (even, odd) pair
                    float q0 = v, q1 = partner;
                    if (bias) { q0 += __ldg(bias + row); q1 += __ldg(bias + row + 1); }
                    int col = row, region = 0;
                    if (col >= qk) { col -= qk; region = 1; }
                    if (region == 1 && col >= kvd) { col -= kvd; region = 2; }
                    if (region < 2) {
                        const float2 cs = s_rope[(col % HD) / 2];
                        const float r0 = q0 * cs.x - q1 * cs.y, r1 = q0 * cs.y + q1 * cs.x;
                        q0 = r0; q1 = r1;
                    }
                    if (region == 0) {
                        st_pair2(xq + col, q0, q1, tag);
                    } else {
                        const __half2 hv = __floats2half2_rn(q0, q1);
                        const float2 back = __half22float2(hv);
                        st_pair2(xkv + size_t(region - 1) * kvd + col, back.x, back.y, tag);
                        *reinterpret_cast<__half2*>((region == 1 ? kc : vc) + col) = hv;
                    }
                });
                ++pi;
            }
            attention_phase<HD>(p, l, pos, xq, xkv, xatt, reinterpret_cast<float*>(xf), w);
            {   // merge of the attention splits -> O projection -> o pairs
                const FillStat st = fill_attention_merge<HD>(xf, xatt, p.nq, p.attn_splits, s_w, w);
                const Phase& ph = s_ph[pi & 1];
                const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, nullptr, 0.f);
                fetch_phase(pi + 1);
                const int N = ph.N;
                consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, [&](int row, float v, float) {
                    if (row < N) st_pair(xo + row, v, tag);
                });
                ++pi;
            }
            {   // residual stream += o -> RMSNorm -> gate/up -> SiLU * up -> act pairs
                csync();
                const Phase& ph = s_ph[pi & 1];
                const FillStat st = fill_add_pairs(xf, resid, xo, h, ph.a.norm_w, w);
                const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, ph.a.norm_w, ph.a.eps);
                fetch_phase(pi + 1);
                const int N = ph.N;
                consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, [&](int row, float v, float partner) {
                    // rows interleaved at pack time: 2j = gate_j, 2j+1 = up_j
                    if (row < N && (row & 1) == 0) st_pair(xact + (row >> 1), (v / (1.0f + expf(-v))) * partner, tag);
                });
                ++pi;
            }
            {   // act -> down projection -> down pairs
                csync();
                const Phase& ph = s_ph[pi & 1];
                const FillStat st = fill_pairs(xf, xact, p.ff, w);
                const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, nullptr, 0.f);
                fetch_phase(pi + 1);
                const int N = ph.N;
                consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, [&](int row, float v, float) {
                    if (row < N) st_pair(xdown + row, v, tag);
                });
                ++pi;
            }
        }
        // residual stream += the last down output -> final RMSNorm -> lm_head, tracking the arg-max (last index wins ties)
        float best = -INFINITY;
        int bidx = -1;
        {
            const uint2* xdown_last = p.xbuf + size_t(L - 1) * p.x_layer_stride + qk + 2 * kvd + natt + h + p.ff;
            csync();
            const Phase& ph = s_ph[pi & 1];
            const FillStat st = fill_add_pairs(xf, resid, xdown_last, h, ph.a.norm_w, w);
            const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, ph.a.norm_w, ph.a.eps);
            fetch_phase(pi + 1);
            const int N = ph.N;
            float* logits = p.logits;
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, [&](int row, float v, float) {
                if (row >= N) return;
                logits[row] = v;
                if (bidx < 0 || v > best || (v == best && row > bidx)) { best = v; bidx = row; }
            });
            ++pi;
        }
        if (!p.greedy) break;   // n_steps is 1: the caller reads the logits
        // ---- per-CTA winner -> pairs -> every CTA picks the same token
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
            if (oi >= 0 && (bidx < 0 || ov > best || (ov == best && oi > bidx))) { best = ov; bidx = oi; }
        }
        csync();   // s_best of the previous step is no longer read
        if (lane == 0) { s_best[warp] = best; s_bidx[warp] = bidx; }
        csync();
        if (tid == 0) {
            for (int wi = 1; wi < kConsumerWarps; ++wi)
                if (s_bidx[wi] >= 0 && (bidx < 0 || s_best[wi] > best || (s_best[wi] == best && s_bidx[wi] > bidx))) { best = s_best[wi]; bidx = s_bidx[wi]; }
            __threadfence();   // this CTA's cache rows of the step precede its arg-max pair
            st_pair2(p.xamax + 2 * blockIdx.x, best, __int_as_float(bidx), tag);
        }
        best = -INFINITY; bidx = -1;
        for (int c = tid; c < int(gridDim.x); c += kCT) {
            const float2 v = wait2(p.xamax + 2 * c, w);
            const int i = __float_as_int(v.y);
            if (i >= 0 && (bidx < 0 || v.x > best || (v.x == best && i > bidx))) { best = v.x; bidx = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
            if (oi >= 0 && (bidx < 0 || ov > best || (ov == best && oi > bidx))) { best = ov; bidx = oi; }
        }
        csync();
        if (lane == 0) { s_best[warp] = best; s_bidx[warp] = bidx; }
        csync();
        for (int wi = 0; wi < kConsumerWarps; ++wi)
            if (s_bidx[wi] >= 0 && (bidx < 0 || s_best[wi] > best || (s_best[wi] == best && s_bidx[wi] > bidx))) { best = s_best[wi]; bidx = s_bidx[wi]; }
        __threadfence();       // the other CTAs' cache rows of the step precede the next step's reads
        if (bidx >= 0) tok = uint32_t(bidx);
    }
    // ---- bookkeeping for the host and the next launch
    csync();
    if (tid == 0) {
        if (sh.err) atomicExch(p.err, 1);
        if (blockIdx.x == 0) {
            if (p.greedy) *p.tok = tok;
            if (!*reinterpret_cast<volatile int*>(&sh.err) && !__ldcg(p.err)) {
                p.seq_len[0] = pos0 + p.n_steps;
                if (p.step) *p.step = step0 + p.n_steps;
            }
        }
    }
}

template <int QUANT, int HD>
int32_t launch(const FlowParams& p, int max_kb, int grid, cudaStream_t st) {
    size_t region = size_t(max_kb) * 128;
    const size_t attn = (size_t(kConsumerWarps) * kGC * (HD + 2) + kMaxQ + 2 * HD) * sizeof(float);
    if (attn > region) region = attn;
    const size_t smem = size_t(Tile<QUANT>::STAGES) * Tile<QUANT>::STAGE_BYTES + region + size_t(p.h) * sizeof(float);
    auto kern = decode_flow_kernel<QUANT, HD>;
    cudaFuncAttributes fa;
    FORGE_CUDA(cudaFuncGetAttributes(&fa, kern));
    int dev = 0, optin = 0;
    FORGE_CUDA(cudaGetDevice(&dev));
    FORGE_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    if (smem + fa.sharedSizeBytes > size_t(optin)) { set_error("decode kernel: %zu bytes of shared memory needed", smem + fa.sharedSizeBytes); return FORGE_ERR_UNSUPPORTED; }
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    int per_sm = 0;
    FORGE_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem));
    if (per_sm < 1) { set_error("decode kernel does not fit on an SM"); return FORGE_ERR_UNSUPPORTED; }
    FlowParams pc = p;
    pc.max_kb = max_kb;
    void* args[] = {&pc};
    FORGE_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), dim3(grid), dim3(kThreads), args, smem, st));
    ++g_launches;
    return FORGE_OK;
}

}  // namespace

// context splits per KV head: cover the SMs if possible, at most kMaxSplits
int flow_attn_splits(int nkv, int sms) { return std::max(1, std::min((sms + nkv - 1) / nkv, kMaxSplits)); }

// {value, tag} pairs one layer exchanges: q | new k, v | attention partials | o | act | down
size_t flow_layer_pairs(int h, int qk, int kvd, int ff, int nq, int hd, int splits) {
    return size_t(qk) + 2 * size_t(kvd) + size_t(nq) * splits * (hd + 2) + size_t(h) + size_t(ff) + size_t(h);
}

int32_t decode_flow(const FlowParams& p, int quant, int max_kb, int grid, cudaStream_t st) {
    if (max_kb > core::kMaxKB) { set_error("decode kernel: K beyond %d", core::kMaxKB * 32); return FORGE_ERR_SHAPE; }
    if (p.nq * p.attn_splits > kMaxHS || (p.nq / p.nkv) * p.hd > kMaxQ || p.attn_splits > kMaxSplits) { set_error("decode kernel: %d heads x %d splits unsupported", p.nq, p.attn_splits); return FORGE_ERR_UNSUPPORTED; }
    if (p.h % 4 || p.qk % 4 || p.ff % 4 || p.kvd % 2) { set_error("decode kernel: widths must be multiples of 4"); return FORGE_ERR_SHAPE; }
#define FORGE_FLOW(Q, H) return launch<Q, H>(p, max_kb, grid, st)
    if (quant == FORGE_Q4_0) {
        if (p.hd == 64) FORGE_FLOW(FORGE_Q4_0, 64);
        if (p.hd == 96) FORGE_FLOW(FORGE_Q4_0, 96);
        if (p.hd == 128) FORGE_FLOW(FORGE_Q4_0, 128);
    } else {
        if (p.hd == 64) FORGE_FLOW(FORGE_Q8_0, 64);
        if (p.hd == 96) FORGE_FLOW(FORGE_Q8_0, 96);
        if (p.hd == 128) FORGE_FLOW(FORGE_Q8_0, 128);
    }
#undef FORGE_FLOW
    set_error("decode kernel: head_dim %d unsupported", p.hd);
    return FORGE_ERR_SHAPE;
}

}  // namespace forge
