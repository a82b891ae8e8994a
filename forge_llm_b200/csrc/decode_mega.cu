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
// Greedy sampling (argmax with the last-index tie rule, project.rs:501-503), the position counter
// and the token history are updated by the last CTA to finish, so consecutive steps need no host
// work besides the launch.
#include "gemv_core.cuh"

namespace forge {

namespace {

using namespace core;

constexpr int kGC = 4;                       // query heads per pass over a KV split
constexpr uint32_t kBarSpinLimit = 1u << 22;

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

// attention_flash (emit.rs:657-715) for the current token of sequence 0: split-KV over the CTAs,
// per-unit partial (m, l, acc) to scratch, last unit of a KV head merges.  `buf` is shared memory of
// at least 16 * kGC * (HD + 2) floats.
template <int HD>
__device__ void attention_phase(const MegaParams& p, int layer, int pos, float* buf, int* s_flag) {
    constexpr int W = Seg<HD>::W, ACTIVE = Seg<HD>::ACTIVE, RPW = Seg<HD>::RPW;
    constexpr int PARTS = kConsumerWarps * RPW;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = lane / W, sl = lane % W;
    const bool act = sl < ACTIVE;
    const int G = p.nq / p.nkv, kvd = p.nkv * HD, S = p.attn_splits;
    const int n_ctx = pos + 1;
    int chunk = (n_ctx + S - 1) / S;
    chunk = (chunk + PARTS - 1) / PARTS * PARTS;
    const __half* kp = p.k_pool + size_t(layer) * p.layer_stride;
    const __half* vp = p.v_pool + size_t(layer) * p.layer_stride;
    const float scale = 1.0f / sqrtf(float(HD));
    float (*s_ml)[kGC][2] = reinterpret_cast<float (*)[kGC][2]>(buf);
    float (*s_acc)[kGC][HD] = reinterpret_cast<float (*)[kGC][HD]>(buf + kConsumerWarps * kGC * 2);

    for (int u = blockIdx.x; u < p.nkv * S; u += gridDim.x) {
        const int kvh = u / S, split = u % S;
        const int t_begin = split * chunk, t_end = min(n_ctx, t_begin + chunk);
        for (int g0 = 0; g0 < G; g0 += kGC) {
            const int gc = min(kGC, G - g0);
            float q[kGC][8], acc[kGC][8], mi[kGC], li[kGC];
#pragma unroll
            for (int g = 0; g < kGC; ++g) {
                mi[g] = -INFINITY; li[g] = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) { acc[g][i] = 0.f; q[g][i] = 0.f; }
                if (g < gc && act) {
                    const float4* qp = reinterpret_cast<const float4*>(p.q + size_t(kvh * G + g0 + g) * HD + sl * 8);
                    float4 x0 = __ldcg(qp), x1 = __ldcg(qp + 1);
                    q[g][0] = x0.x; q[g][1] = x0.y; q[g][2] = x0.z; q[g][3] = x0.w;
                    q[g][4] = x1.x; q[g][5] = x1.y; q[g][6] = x1.z; q[g][7] = x1.w;
                }
            }
            constexpr int UNR = 2;
            for (int base = t_begin + warp * RPW; base < t_end; base += PARTS * UNR) {
                uint4 kr[UNR], vr[UNR];
#pragma unroll
                for (int un = 0; un < UNR; ++un) {
                    const int t = base + un * PARTS + seg;
                    kr[un] = make_uint4(0, 0, 0, 0);
                    vr[un] = make_uint4(0, 0, 0, 0);
                    if (t < t_end && act) {
                        const size_t row = size_t(p.page_table[t / FORGE_KV_PAGE]) * FORGE_KV_PAGE + t % FORGE_KV_PAGE;
                        const size_t off = row * kvd + kvh * HD + sl * 8;
                        kr[un] = __ldcg(reinterpret_cast<const uint4*>(kp + off));  // through L2: this step's row was
                        vr[un] = __ldcg(reinterpret_cast<const uint4*>(vp + off));  // written by another CTA
                    }
                }
#pragma unroll
                for (int un = 0; un < UNR; ++un) {
                    const bool valid = (base + un * PARTS + seg) < t_end;
                    float kf[8], vf[8];
                    unpack8(kr[un], kf);
                    unpack8(vr[un], vf);
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
                const int head = kvh * G + g0 + g;
                if (S == 1) {
                    p.attn_out[size_t(head) * HD + dd] = A * (1.0f / L);
                } else {
                    float* wsp = p.attn_ws + (size_t(head) * S + split) * (HD + 2);
                    wsp[2 + dd] = A;
                    if (dd == 0) { wsp[0] = M; wsp[1] = L; }
                }
            }
        }
        if (S == 1) continue;
        // last unit of this KV head merges the splits (fixed order)
        __threadfence();
        csync();
        if (threadIdx.x == 0) {
            const int old = atomicAdd(p.attn_tickets + kvh, 1);
            *s_flag = (old == S - 1);
            if (old == S - 1) p.attn_tickets[kvh] = 0;
        }
        csync();
        if (!*s_flag) continue;
        __threadfence();
        for (int idx = threadIdx.x; idx < G * HD; idx += kCT) {
            const int g = idx / HD, dd = idx % HD, head = kvh * G + g;
            const float* w0 = p.attn_ws + size_t(head) * S * (HD + 2);
            float M = -INFINITY;
            for (int s = 0; s < S; ++s) M = fmaxf(M, __ldcg(w0 + size_t(s) * (HD + 2)));
            float L = 0.f, A = 0.f;
            for (int s = 0; s < S; ++s) {
                const float* w = w0 + size_t(s) * (HD + 2);
                const float m = __ldcg(w);
                const float wt = (m == -INFINITY) ? 0.f : expf(m - M);
                L += __ldcg(w + 1) * wt;
                A += __ldcg(w + 2 + dd) * wt;
            }
            p.attn_out[size_t(head) * HD + dd] = A * (1.0f / L);
        }
    }
}

template <int QUANT, int HD>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(MegaParams p) {
    using T = Tile<QUANT>;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ Shared sh;
    __shared__ int4 s_xoff[QUANT == FORGE_Q4_0 ? 2 * kMaxKB : 1];
    __shared__ float s_best[kConsumerWarps];
    __shared__ int s_bidx[kConsumerWarps];
    __shared__ int s_flag;
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
    for (int l = 0; l < L && ok; ++l) {
        {   // RMSNorm + QKV + bias / RoPE / KV append
            Phase ph = p.phases[4 * l];
            ph.a.x = (l == 0) ? embed_row : p.hidden;
            const float un = stage_activation<QUANT, true>(xf, s_xoff, sh, ph.a.x, ph.K, ph.a.norm_w, ph.a.eps);
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, nohook);
        }
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
        attention_phase<HD>(p, l, pos, reinterpret_cast<float*>(xf), &s_flag);
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
        {   // O projection + residual
            Phase ph = p.phases[4 * l + 1];
            if (l == 0) ph.a.resid = embed_row;
            const float un = stage_activation<QUANT, true>(xf, s_xoff, sh, ph.a.x, ph.K, nullptr, 0.f);
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, nohook);
        }
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
        {   // RMSNorm + gate/up + SiLU * up
            const Phase ph = p.phases[4 * l + 2];
            const float un = stage_activation<QUANT, true>(xf, s_xoff, sh, ph.a.x, ph.K, ph.a.norm_w, ph.a.eps);
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, nohook);
        }
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
        {   // down projection + residual
            const Phase ph = p.phases[4 * l + 3];
            const float un = stage_activation<QUANT, true>(xf, s_xoff, sh, ph.a.x, ph.K, nullptr, 0.f);
            consume_phase<QUANT>(ph, sh, ring, xf, s_xoff, un, 0, cc, nohook);
        }
        target += gridDim.x;
        if (!(ok = grid_barrier(p, sh, target))) break;
    }
    float best = -INFINITY;
    int bidx = -1;
    if (ok) {   // final RMSNorm + lm_head, tracking the arg-max (last index wins ties)
        const Phase ph = p.phases[4 * L];
        const float un = stage_activation<QUANT, true>(xf, s_xoff, sh, ph.a.x, ph.K, ph.a.norm_w, ph.a.eps);
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
    const size_t attn = size_t(kConsumerWarps) * kGC * (HD + 2) * sizeof(float);
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
