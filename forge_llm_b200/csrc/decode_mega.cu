// One decode step (forward(), crates/forgellm-codegen-cpu/src/emit.rs:4029-4500, batch 1) as ONE
// persistent kernel: a CTA per SM, launched cooperatively.  The producer lane of every CTA streams
// that CTA's share of every projection of every layer through the shared-memory ring without ever
// waiting for activations (weights are static), so HBM stays busy across the dependent phases;
// the 16 consumer warps walk the phases
//   [RMSNorm + QKV GEMV + bias/RoPE/KV append] | attention | [O GEMV + residual] |
//   [RMSNorm + gate/up GEMV + SiLU*up] | [down GEMV + residual]            per layer, then
//   [RMSNorm + lm_head GEMV (+ arg-max)]
// separated by grid-wide barriers (an atomic counter in global memory, bounded spin).  Units of
// work are dealt round-robin across phases, so every SM streams the same number of bytes per step.
// Cross-CTA reductions are done by the READER: a projection that is split along K leaves its raw
// per-slice partial sums in scratch, and the phase that consumes the vector adds the slices (in slice
// order, so the result does not depend on timing) while it stages its input - the residual stream is
// rebuilt that way (h' = h + sum of O partials, h'' = h' + sum of down partials), the attention phase
// rebuilds q / k / v (+ bias, RoPE, cache append), and the O projection's input is the merge of the
// attention splits.
// Greedy sampling (argmax with the last-index tie rule, project.rs:501-503), the position counter
// and the token history are updated by the last CTA to finish, so consecutive steps need no host
// work besides the launch.
#include "gemv_core.cuh"

namespace forge {

namespace {

using namespace core;

constexpr int kGC = 4;                       // query heads per pass over a KV split
constexpr uint32_t kBarSpinLimit = 1u << 22;
constexpr int kMaxSplits = 16;                // KV splits per head in the whole-step kernel

template <int HD> struct Seg { static constexpr int W = (HD == 64) ? 8 : 16, ACTIVE = HD / 8, RPW = 32 / W; };

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Grid-wide barrier for the consumer warps of all CTAs.  Returns false (for every thread of the CTA)
// when the wait gave up or another CTA reported an error.
__device__ __forceinline__ bool grid_barrier(const MegaParams& p, Shared& sh, unsigned target) {
    csync();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(p.bar, 1u);
        bool ok = false;
        for (uint32_t i = 0; i < kBarSpinLimit; ++i) {
            if (ld_acquire(p.bar) >= target) { ok = true; break; }
            if ((i & 63) == 63 && __ldcg(p.err)) break;
        }
        if (!ok) { atomicExch(p.err, 1); sh.err = 1; }
        __threadfence();
    }
    csync();
    return *reinterpret_cast<volatile int*>(&sh.err) == 0;
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// attention_flash (emit.rs:657-715) for the current token of sequence 0, split over the CTAs: a unit is
// (kv head, context split).  Each unit first rebuilds what it needs of this step's q / k / v from the QKV
// projection's partial sums (+ bias, RoPE; the unit that covers the current position also appends k / v to
// the fp16 cache), then writes its online-softmax partial (m, l, acc) to attn_ws.  `buf` is shared memory
// of at least (16 * kGC * (HD + 2) + kMaxQ + 2 * HD) floats.
constexpr int kMaxQ = 512;  // query values per KV group (heads per group x head_dim)

template <int HD>
__device__ void attention_phase(const MegaParams& p, int layer, int pos, float* buf) {
    constexpr int W = Seg<HD>::W, ACTIVE = Seg<HD>::ACTIVE, RPW = Seg<HD>::RPW;
    constexpr int PARTS = kConsumerWarps * RPW;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = lane / W, sl = lane % W;
    const bool act = sl < ACTIVE;
    const int G = p.nq / p.nkv, kvd = p.nkv * HD, S = p.attn_splits, qk = p.nq * HD;
    const int n_ctx = pos + 1;
    int chunk = (n_ctx + S - 1) / S;
    chunk = (chunk + PARTS - 1) / PARTS * PARTS;
    __half* kp = p.k_pool + size_t(layer) * p.layer_stride;
    __half* vp = p.v_pool + size_t(layer) * p.layer_stride;
    const float scale = 1.0f / sqrtf(float(HD));
    float (*s_ml)[kGC][2] = reinterpret_cast<float (*)[kGC][2]>(buf);
    float (*s_acc)[kGC][HD] = reinterpret_cast<float (*)[kGC][HD]>(buf + kConsumerWarps * kGC * 2);
    float* sq = buf + kConsumerWarps * kGC * (HD + 2);   // [G][HD] finished queries of the group
    float* snew = sq + kMaxQ;                            // [2][HD] this step's k and v (fp16-rounded)
    const Phase& qph = p.phases[4 * layer];
    const float* scr = qph.scratch;
    const size_t npad = phase_npad(qph);
    const int Sq = qph.slices;
    const float* bias = qph.a.bias;
    const float2* rope = reinterpret_cast<const float2*>(qph.a.rope) + size_t(pos) * (HD / 2);

    for (int u = blockIdx.x; u < p.nkv * S; u += gridDim.x) {
        const int kvh = u / S, split = u % S;
        const int t_begin = split * chunk, t_end = min(n_ctx, t_begin + chunk);
        const bool covers = pos >= t_begin && pos < t_end;
        csync();  // shared buffers of the previous unit are no longer read
        // ---- rebuild q (and, in the covering unit, k / v) from the projection's K slices
        const int npairs = (G * HD + (covers ? 2 * HD : 0)) / 2;
        for (int pr = threadIdx.x; pr < npairs; pr += kCT) {
            int e = 2 * pr, row, which = -1, d;
            if (e < G * HD) { d = e % HD; row = (kvh * G + e / HD) * HD + d; }
            else { e -= G * HD; which = e / HD; d = e % HD; row = qk + which * kvd + kvh * HD + d; }
            float2 pv[kGemvMaxSlices];
#pragma unroll
            for (int s = 0; s < kGemvMaxSlices; ++s)
                pv[s] = (s < Sq) ? __ldcg(reinterpret_cast<const float2*>(scr + size_t(s) * npad + row)) : make_float2(0.f, 0.f);
            float v0 = 0.f, v1 = 0.f;
#pragma unroll
            for (int s = 0; s < kGemvMaxSlices; ++s) { v0 += pv[s].x; v1 += pv[s].y; }
            if (bias) { v0 += bias[row]; v1 += bias[row + 1]; }
            if (which != 1) {  // q and k rotate (adjacent pairs, emit.rs:523-525)
                const float2 cs = rope[d / 2];
                const float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;
                v0 = r0; v1 = r1;
            }
            if (which < 0) {
                sq[2 * pr] = v0; sq[2 * pr + 1] = v1;
            } else {
                const __half2 hv = __floats2half2_rn(v0, v1);
                const size_t rowoff = (size_t(p.page_table[pos / FORGE_KV_PAGE]) * FORGE_KV_PAGE + pos % FORGE_KV_PAGE) * kvd + kvh * HD + d;
                *reinterpret_cast<__half2*>((which == 0 ? kp : vp) + rowoff) = hv;
                const float2 back = __half22float2(hv);
                snew[which * HD + d] = back.x; snew[which * HD + d + 1] = back.y;
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
                for (int i = 0; i < 8; ++i) { acc[g][i] = 0.f; q[g][i] = (g < gc && act) ? sq[(g0 + g) * HD + sl * 8 + i] : 0.f; }
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
                    if (t == pos && act) {  // this step's row: taken from shared memory, not from the cache
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
                for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, s_ml[w][g][0]);
                float L = 0.f, A = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) {
                    const float m = s_ml[w][g][0];
                    const float wt = (m == -INFINITY) ? 0.f : expf(m - M);
                    L += s_ml[w][g][1] * wt;
                    A += s_acc[w][g][dd] * wt;
                }
                float* wsp = p.attn_ws + (size_t(kvh * G + g0 + g) * S + split) * (HD + 2);
                wsp[2 + dd] = A;
                if (dd == 0) { wsp[0] = M; wsp[1] = L; }
            }
        }
    }
}

// Fill the staging area with the attention output: for every head, the softmax-weighted merge of the
// context splits' partials (m, l, acc).  Two L2 round trips: the (m, l) pairs, then the accumulators.
template <int HD>
__device__ __forceinline__ FillStat fill_attention_merge(const MegaParams& p, uint2* xf, float (*s_w)[512]) {
    float* xraw = reinterpret_cast<float*>(xf);
    const int S = p.attn_splits, nq = p.nq;
    FillStat st;
    csync();  // the previous contents of the fragment area and of s_w are no longer read
    for (int i = threadIdx.x; i < nq * S; i += kCT) {
        const float* w = p.attn_ws + size_t(i) * (HD + 2);
        s_w[0][i] = __ldcg(w);
        s_w[1][i] = __ldcg(w + 1);
    }
    csync();
    float wt = 0.f;
    const int i1 = threadIdx.x;  // (head, split) handled by this thread; nq * S <= 512
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
        const float* a0 = p.attn_ws + size_t(head) * S * (HD + 2) + 2 + dd;
        float2 lo[kMaxSplits], hi[kMaxSplits];   // (HD + 2) floats per record: 8-byte aligned, not 16
#pragma unroll
        for (int s = 0; s < kMaxSplits; ++s) {
            const bool in = s < S;
            lo[s] = in ? __ldcg(reinterpret_cast<const float2*>(a0 + size_t(s) * (HD + 2))) : make_float2(0.f, 0.f);
            hi[s] = in ? __ldcg(reinterpret_cast<const float2*>(a0 + size_t(s) * (HD + 2) + 2)) : make_float2(0.f, 0.f);
        }
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kMaxSplits; ++s) {
            const float w = (s < S) ? s_w[0][head * S + s] : 0.f;
            v.x += lo[s].x * w; v.y += lo[s].y * w; v.z += hi[s].x * w; v.w += hi[s].y * w;
        }
        fill_note(st, v, nullptr, e);
        *reinterpret_cast<float4*>(xraw + e) = v;
    }
    return st;
}

template <int QUANT, int HD>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(MegaParams p) {
    using T = Tile<QUANT>;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ Shared sh;
    __shared__ int4 s_xoff[QUANT == FORGE_Q4_0 ? 2 * kMaxKB : 1];
    __shared__ float s_w[2][512];
    __shared__ float s_best[kConsumerWarps];
    __shared__ int s_bidx[kConsumerWarps];
    unsigned char* ring = smem;
    uint2* xf = reinterpret_cast<uint2*>(smem + size_t(kStages) * T::STAGE_BYTES);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&sh.full_bar[s], 1); mbar_init(&sh.empty_bar[s], kConsumerWarps); }
        sh.err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int L = p.num_layers;
    int cc = 0;

    if (warp == kConsumerWarps) {
        // ---- producer: every projection of every layer, in phase order, bounded only by ring space
        if (lane == 0) {
            for (int i = 0; i < 4 * L + 1; ++i) {
                const Phase ph = p.phases[i];
                if (!produce_phase<QUANT>(ph, sh, ring, cc)) break;
            }
        }
        return;
    }

    // ---- consumers
    const uint32_t tok = *p.tok;
    const int pos = p.seq_len[0];
    if (blockIdx.x == 0 && tid == 0 && p.hist) p.hist[*p.step] = tok;
    const float* embed_row = p.embed + size_t(tok) * p.h;
    unsigned target = 0;
    bool ok = true;
    auto nohook = [](int, float) {};
    // partial sums of the down projection of the previous layer (none before layer 0)
    const float* dparts = nullptr;
    int dn = 0;
    size_t dstride = 0;
    for (int l = 0; l < L && ok; ++l) {
        {   // residual stream h = h_prev + down partials -> RMSNorm -> QKV (raw partials)
            const Phase ph = p.phases[4 * l];
            const FillStat st = stage_fill_global<true>(xf, l == 0 ? embed_row : p.hidden0, dparts, dn, dstride, p.hidden1, ph.K, ph.a.norm_w);
            const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, ph.a.norm_w, ph.a.eps);
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, nohook);
        }
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
        attention_phase<HD>(p, l, pos, reinterpret_cast<float*>(xf));
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
        {   // merge of the attention splits -> O projection (raw partials)
            const Phase ph = p.phases[4 * l + 1];
            const FillStat st = fill_attention_merge<HD>(p, xf, s_w);
            const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, nullptr, 0.f);
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, nohook);
        }
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
        {   // h' = h + O partials -> RMSNorm -> gate/up -> SiLU * up
            const Phase ph = p.phases[4 * l + 2];
            const Phase& oph = p.phases[4 * l + 1];
            const float* hin = (l == 0) ? embed_row : p.hidden1;   // layer 0 has no pending down partials: h is the embedding row
            const FillStat st = stage_fill_global<true>(xf, hin, oph.scratch, oph.slices, phase_npad(oph), p.hidden0, ph.K, ph.a.norm_w);
            const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, ph.a.norm_w, ph.a.eps);
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, nohook);
        }
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
        {   // down projection (raw partials)
            const Phase ph = p.phases[4 * l + 3];
            const FillStat st = stage_fill_global<true>(xf, ph.a.x, nullptr, 0, 0, nullptr, ph.K, nullptr);
            const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, nullptr, 0.f);
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, nohook);
            dparts = ph.scratch; dn = ph.slices; dstride = phase_npad(ph);
        }
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
    }
    float best = -INFINITY;
    int bidx = -1;
    if (ok) {   // h_final = h + down partials -> RMSNorm -> lm_head, tracking the arg-max (last index wins ties)
        const Phase ph = p.phases[4 * L];
        const FillStat st = stage_fill_global<true>(xf, p.hidden0, dparts, dn, dstride, nullptr, ph.K, ph.a.norm_w);
        const float un = stage_finish<QUANT>(xf, s_xoff, sh, st, ph.K, ph.a.norm_w, ph.a.eps);
        const int N = ph.N;
        consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, [&](int row, float v) {
            if (row < N && (bidx < 0 || v > best || (v == best && row > bidx))) { best = v; bidx = row; }
        });
    }
    // ---- per-CTA winner, then the last CTA to arrive picks the token and advances the counters
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
        if (oi >= 0 && (bidx < 0 || ov > best || (ov == best && oi > bidx))) { best = ov; bidx = oi; }
    }
    if (lane == 0) { s_best[warp] = best; s_bidx[warp] = bidx; }
    csync();
    if (tid == 0) {
        for (int w = 1; w < kConsumerWarps; ++w)
            if (s_bidx[w] >= 0 && (bidx < 0 || s_best[w] > best || (s_best[w] == best && s_bidx[w] > bidx))) { best = s_best[w]; bidx = s_bidx[w]; }
        p.amax_val[blockIdx.x] = best;
        p.amax_idx[blockIdx.x] = bidx;
        if (sh.err) atomicExch(p.err, 1);
        __threadfence();
        const int old = atomicAdd(p.amax_ticket, 1);
        if (old == int(gridDim.x) - 1) {
            __threadfence();
            float bv = -INFINITY;
            int bi = -1;
            for (int c = 0; c < int(gridDim.x); ++c) {
                const float v = __ldcg(p.amax_val + c);
                const int i = __ldcg(p.amax_idx + c);
                if (i >= 0 && (bi < 0 || v > bv || (v == bv && i > bi))) { bv = v; bi = i; }
            }
            if (p.greedy && bi >= 0) *p.tok = uint32_t(bi);
            if (!__ldcg(p.err)) {
                p.seq_len_mut[0] = pos + 1;
                *p.step += 1;
            }
            *p.amax_ticket = 0;
            *p.bar = 0u;   // every CTA has passed its last barrier by now
        }
    }
}

template <int QUANT, int HD>
int32_t launch(const MegaParams& p, int max_kb, int grid, cudaStream_t st) {
    size_t region = size_t(max_kb) * 128;
    const size_t attn = (size_t(kConsumerWarps) * kGC * (HD + 2) + kMaxQ + 2 * HD) * sizeof(float);
    if (attn > region) region = attn;
    const size_t smem = size_t(kStages) * Tile<QUANT>::STAGE_BYTES + region;
    if (smem > 220 * 1024) { set_error("decode step kernel: %zu bytes of shared memory needed", smem); return FORGE_ERR_SHAPE; }
    auto kern = decode_step_kernel<QUANT, HD>;
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    int per_sm = 0;
    FORGE_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem));
    if (per_sm < 1) { set_error("decode step kernel does not fit on an SM"); return FORGE_ERR_UNSUPPORTED; }
    MegaParams pc = p;
    void* args[] = {&pc};
    FORGE_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), dim3(grid), dim3(kThreads), args, smem, st));
    ++g_launches;
    return FORGE_OK;
}

}  // namespace

int32_t decode_step_mega(const MegaParams& p, int quant, int hd, int max_kb, int grid, cudaStream_t st) {
    if (max_kb > core::kMaxKB) { set_error("decode step kernel: K beyond %d", core::kMaxKB * 32); return FORGE_ERR_SHAPE; }
#define FORGE_MEGA(Q, H) return launch<Q, H>(p, max_kb, grid, st)
    if (quant == FORGE_Q4_0) {
        if (hd == 64) FORGE_MEGA(FORGE_Q4_0, 64);
        if (hd == 96) FORGE_MEGA(FORGE_Q4_0, 96);
        if (hd == 128) FORGE_MEGA(FORGE_Q4_0, 128);
    } else {
        if (hd == 64) FORGE_MEGA(FORGE_Q8_0, 64);
        if (hd == 96) FORGE_MEGA(FORGE_Q8_0, 96);
        if (hd == 128) FORGE_MEGA(FORGE_Q8_0, 128);
    }
#undef FORGE_MEGA
    set_error("decode step kernel: head_dim %d unsupported", hd);
    return FORGE_ERR_SHAPE;
}

}  // namespace forge
