// Single-query decode attention over the paged fp16 KV cache (replaces attention_flash,
// crates/forgellm-codegen-cpu/src/emit.rs:657-715; GQA mapping kv_head = h / (nq/nkv), :660-666).
// HBM-bound on K/V: the context is split over CTAs (split-KV); a producer lane pulls the CTA's pages - 64 rows of one
// KV head, K and V - into a ring of shared-memory stages with 3-D tiled TMA copies (cp.async.bulk.tensor, mbarrier
// completion; the tensor map spans this GPU's own pool), so the bytes in flight do not depend on registers or on
// the instruction stream, and it starts before the dependency wait: every cached row but the newest was written by
// earlier steps.  Four consumer warps read the rows from shared memory with 128-bit loads, every row shared by the
// query heads of its group; the online-softmax state (m, l, acc) is f32.  Split partials are merged by the last CTA
// to finish a KV head (atomic ticket), so no second launch is needed.  Every wait is bounded.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace forge {

namespace {

constexpr int kThreads = 128;     // consumer threads (four warps); warp 4 is the producer
constexpr int kBlock = kThreads + 32;
constexpr int kStages = 4;        // most pages (K and V) in flight per CTA (a CTA with one or two pages takes a ring of two)
constexpr int kMaxGroup = 16;  // query heads per KV head
constexpr int kMaxSplits = 32;    // context splits per KV head (the merge keeps one partial per split in registers)
constexpr uint32_t kSpin = 1u << 22;

template <int HD> struct Seg { static constexpr int W = (HD == 64) ? 8 : 16, ACTIVE = HD / 8, RPW = 32 / W; };

struct DecParams {
    AttnDecodeArgs a;
    float scale;
    int stages;   // ring depth of this launch (<= kStages)
};

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// exp(x - m) with exp(-inf) = 0 and no NaN when both are -inf
__device__ __forceinline__ float exp_rel(float x, float m) { return (x == -INFINITY) ? 0.f : __expf(x - m); }

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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < kSpin; ++i) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// one page of one KV head: box {head_dim, 1, 64 rows} at {0, kv head, row}
__device__ __forceinline__ void tma_page(void* dst, const CUtensorMap* map, int kvh, int row, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(0), "r"(kvh), "r"(row), "r"(smem_u32(bar)) : "memory");
}
// the result in the form the caller asked for: f32, or fp16 hi (+ lo)
__device__ __forceinline__ void store_out(const AttnDecodeArgs& a, size_t i, float x) {
    if (a.out16) {
        const __half h = __float2half_rn(x);
        a.out16[i] = h;
        if (a.out16_lo) a.out16_lo[i] = __float2half_rn(x - __half2float(h));
    } else {
        a.out[i] = x;
    }
}
__device__ __forceinline__ void store_out2(const AttnDecodeArgs& a, size_t i, float2 x) {
    if (a.out16) {
        const __half2 h = __floats2half2_rn(x.x, x.y);
        *reinterpret_cast<__half2*>(a.out16 + i) = h;
        if (a.out16_lo) {
            const float2 hf = __half22float2(h);
            *reinterpret_cast<__half2*>(a.out16_lo + i) = __floats2half2_rn(x.x - hf.x, x.y - hf.y);
        }
    } else {
        *reinterpret_cast<float2*>(a.out + i) = x;
    }
}
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }

// SW: sliding-window instantiation (the full-attention one carries no window tests)
// GC: query heads folded per pass over the keys: min(4, query heads per KV head), so that multi-head attention (one
// query head per KV head) forms one score per key, not four
template <int HD, bool SW, int GC>
__global__ void __launch_bounds__(kBlock, (HD == 128 || GC == 4) ? 2 : 3) attn_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                                             DecParams p) {
    constexpr int W = Seg<HD>::W, ACTIVE = Seg<HD>::ACTIVE, RPW = Seg<HD>::RPW;
    constexpr int PARTS = (kThreads / 32) * RPW;
    constexpr int PAGE_BYTES = FORGE_KV_PAGE * HD * 2;
    extern __shared__ __align__(1024) unsigned char ring[];   // [kStages][K page | V page]
    __shared__ uint64_t full_bar[kStages], empty_bar[kStages];
    __shared__ float s_m[PARTS][GC], s_l[PARTS][GC], s_w[PARTS][GC];
    __shared__ float s_acc[PARTS][GC][HD];
    __shared__ float s_fw[kMaxSplits][kMaxGroup];  // final merge: weight of split s for query head g
    __shared__ int s_last;
    const AttnDecodeArgs& a = p.a;
    pdl_trigger();
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = lane / W, sl = lane % W;
    const bool act = sl < ACTIVE;
    const int G = a.nq / a.nkv, kvd = a.nkv * HD;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kThreads / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Split s owns the logical pages s, s + splits, ...: which pages a CTA reads does not depend on the context
    // length.  The length, the page table and every cached row but the newest were written before the kernel in front
    // of this one started, so they are read without waiting for it.
    const int32_t* pt = a.page_table ? a.page_table + size_t(b) * a.pages_per_seq : nullptr;
    const int n_ctx = a.seq_len ? a.seq_len[b] + 1 : a.seq_len_host;
    const int n_pages = (n_ctx + FORGE_KV_PAGE - 1) / FORGE_KV_PAGE;
    const int t_first = (SW && n_ctx > a.window) ? n_ctx - a.window : 0;  // sliding window: first position seen
    const size_t seq_base = a.page_table ? 0 : size_t(b) * a.max_ctx;  // contiguous: [batch][max_ctx][kvd]
    const int part = warp * RPW + seg;
    // positions per segment folded into the running softmax state in one step (a whole page per warp step when one
    // query head leaves the registers for it)
    constexpr int UNR = (GC == 1 && W == 16) ? 8 : 4;

    if (warp == kThreads / 32) {
        // ---- producer: the CTA's pages, once per pass over the query heads, as ring space frees up
        if (lane == 0) {
            int i = 0;
            for (int g0 = 0; g0 < G; g0 += GC)
                for (int lp = split; lp < n_pages; lp += a.splits) {
                    if (SW && (lp + 1) * FORGE_KV_PAGE <= t_first) continue;
                    const int st = i % p.stages, use = i / p.stages;
                    if (use > 0 && !mbar_wait(&empty_bar[st], (use - 1) & 1)) { if (a.err) atomicExch(a.err, 1); return; }
                    const int row = a.row_base + int(seq_base) + (pt ? pt[lp] : lp) * FORGE_KV_PAGE;
                    unsigned char* dst = ring + size_t(st) * 2 * PAGE_BYTES;
                    mbar_expect_tx(&full_bar[st], 2 * PAGE_BYTES);
                    tma_page(dst, &map_k, kvh, row, &full_bar[st]);
                    tma_page(dst + PAGE_BYTES, &map_v, kvh, row, &full_bar[st]);
                    ++i;
                }
        }
        return;
    }
    pdl_wait();  // q and the newest cache row come from the kernel before this one
    int pi = 0;  // pages consumed so far (ring position)

    for (int g0 = 0; g0 < G; g0 += GC) {
        const int gc = min(GC, G - g0);
        float q[GC][8], acc[GC][8], mi[GC], li[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            mi[g] = -INFINITY; li[g] = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[g][i] = 0.f; q[g][i] = 0.f; }
            if (g < gc && act) {
                const float4* qp = reinterpret_cast<const float4*>(a.q + (size_t(b) * a.nq + kvh * G + g0 + g) * HD + sl * 8);
                float4 x0 = qp[0], x1 = qp[1];
                q[g][0] = x0.x * p.scale; q[g][1] = x0.y * p.scale; q[g][2] = x0.z * p.scale; q[g][3] = x0.w * p.scale;
                q[g][4] = x1.x * p.scale; q[g][5] = x1.y * p.scale; q[g][6] = x1.z * p.scale; q[g][7] = x1.w * p.scale;
            }
        }
        for (int lp = split; lp < n_pages; lp += a.splits) {
            if (SW && (lp + 1) * FORGE_KV_PAGE <= t_first) continue;  // the whole page lies before the window
            const int t_page = lp * FORGE_KV_PAGE;
            const int st = pi % p.stages;
            if (!mbar_wait(&full_bar[st], (pi / p.stages) & 1) && a.err) atomicExch(a.err, 1);
            const unsigned char* ks = ring + size_t(st) * 2 * PAGE_BYTES;
            const unsigned char* vs = ks + PAGE_BYTES;
            for (int base = warp * RPW; base < FORGE_KV_PAGE; base += PARTS * UNR) {
                uint4 kr[UNR], vr[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int tp = base + u * PARTS + seg;
                    kr[u] = make_uint4(0, 0, 0, 0);
                    vr[u] = make_uint4(0, 0, 0, 0);
                    if (tp < FORGE_KV_PAGE && t_page + tp < n_ctx && (!SW || t_page + tp >= t_first) && act) {
                        if (t_page + tp == n_ctx - 1) {
                            // the newest row is being written by the kernel in front while the page is copied: it is
                            // read from global memory, after the wait
                            const size_t off = (size_t(seq_base) + size_t(pt ? pt[lp] : lp) * FORGE_KV_PAGE + tp) * kvd + size_t(kvh) * HD + sl * 8;
                            kr[u] = __ldcg(reinterpret_cast<const uint4*>(a.k_pool + off));
                            vr[u] = __ldcg(reinterpret_cast<const uint4*>(a.v_pool + off));
                        } else {
                            kr[u] = *reinterpret_cast<const uint4*>(ks + size_t(tp) * HD * 2 + sl * 16);
                            vr[u] = *reinterpret_cast<const uint4*>(vs + size_t(tp) * HD * 2 + sl * 16);
                        }
                    }
                }
                // the UNR scores of a head are formed independently, then folded into the running state in one
                // softmax step (one rescale per group instead of one per position)
                float sc[UNR][GC];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    float kf[8];
                    unpack8(kr[u], kf);
#pragma unroll
                    for (int g = 0; g < GC; ++g) {
                        float d = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) d += q[g][i] * kf[i];
                        sc[u][g] = d;
                    }
                }
#pragma unroll
                for (int o = W / 2; o > 0; o >>= 1)
#pragma unroll
                    for (int u = 0; u < UNR; ++u)
#pragma unroll
                        for (int g = 0; g < GC; ++g) sc[u][g] += __shfl_xor_sync(0xffffffffu, sc[u][g], o);
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int tp = base + u * PARTS + seg;
                    if (!(tp < FORGE_KV_PAGE && t_page + tp < n_ctx && (!SW || t_page + tp >= t_first))) {
#pragma unroll
                        for (int g = 0; g < GC; ++g) sc[u][g] = -INFINITY;
                    }
                }
                float vf[UNR][8];
#pragma unroll
                for (int u = 0; u < UNR; ++u) unpack8(vr[u], vf[u]);
#pragma unroll
                for (int g = 0; g < GC; ++g) {
                    float mn = mi[g];
#pragma unroll
                    for (int u = 0; u < UNR; ++u) mn = fmaxf(mn, sc[u][g]);
                    if (mn == -INFINITY || g >= gc) continue;
                    const float es = exp_rel(mi[g], mn);
                    float pr[UNR], ps = 0.f;
#pragma unroll
                    for (int u = 0; u < UNR; ++u) { pr[u] = exp_rel(sc[u][g], mn); ps += pr[u]; }
                    mi[g] = mn;
                    li[g] = li[g] * es + ps;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float t = acc[g][i] * es;
#pragma unroll
                        for (int u = 0; u < UNR; ++u) t += pr[u] * vf[u][i];
                        acc[g][i] = t;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[st]);
            ++pi;
        }
        // ---- merge the CTA's parts: weights once per (part, head), then one weighted sum per output
        csync();
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            if (sl == 0) { s_m[part][g] = mi[g]; s_l[part][g] = li[g]; }
            if (act) {
                *reinterpret_cast<float4*>(&s_acc[part][g][sl * 8]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
                *reinterpret_cast<float4*>(&s_acc[part][g][sl * 8 + 4]) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
            }
        }
        csync();
        if (threadIdx.x < PARTS * GC) {
            const int pp = threadIdx.x % PARTS, g = threadIdx.x / PARTS;
            float M = -INFINITY;
#pragma unroll
            for (int j = 0; j < PARTS; ++j) M = fmaxf(M, s_m[j][g]);
            s_w[pp][g] = exp_rel(s_m[pp][g], M);
        }
        csync();
        for (int idx = threadIdx.x; idx < gc * HD; idx += kThreads) {
            const int g = idx / HD, dd = idx % HD;
            float A = 0.f;
#pragma unroll
            for (int pp = 0; pp < PARTS; ++pp) A += s_acc[pp][g][dd] * s_w[pp][g];
            const int head = kvh * G + g0 + g;
            float M = -INFINITY, L = 0.f;
            if (dd == 0 || a.splits == 1) {
#pragma unroll
                for (int pp = 0; pp < PARTS; ++pp) { M = fmaxf(M, s_m[pp][g]); L += s_l[pp][g] * s_w[pp][g]; }
            }
            if (a.splits == 1) {
                store_out(a, (size_t(b) * a.nq + head) * HD + dd, A * (1.0f / L));
            } else {
                float* w = a.ws + ((size_t(b) * a.nq + head) * a.splits + split) * (HD + 2);
                w[2 + dd] = A;
                if (dd == 0) { w[0] = M; w[1] = L; }
            }
        }
    }
    if (a.splits == 1) return;

    // ---- last CTA of this (batch, kv head) merges the splits
    __threadfence();
    csync();
    if (threadIdx.x == 0) {
        int old = atomicAdd(a.counters + b * a.nkv + kvh, 1);
        s_last = (old == a.splits - 1);
        if (s_last) a.counters[b * a.nkv + kvh] = 0;  // ready for the next launch
    }
    csync();
    if (!s_last) return;
    __threadfence();
    // One round trip: every thread first issues the loads of its two output columns from all splits, then the
    // warps turn the splits' (max, sum) pairs into normalised weights (lane = split), then the weighted sums.
    const float* ws_kvh = a.ws + (size_t(b) * a.nq + size_t(kvh) * G) * a.splits * (HD + 2);
    const int nout2 = G * HD / 2;
    for (int i0 = 0; i0 < nout2; i0 += kThreads) {
        const int idx = i0 + threadIdx.x;
        const bool on = idx < nout2;
        const int g = on ? idx / (HD / 2) : 0, d2 = on ? idx % (HD / 2) : 0;
        const float* w0 = ws_kvh + size_t(g) * a.splits * (HD + 2) + 2 + 2 * d2;
        float2 pa[kMaxSplits];
#pragma unroll
        for (int s = 0; s < kMaxSplits; ++s)
            pa[s] = (on && s < a.splits) ? __ldcg(reinterpret_cast<const float2*>(w0 + size_t(s) * (HD + 2))) : make_float2(0.f, 0.f);
        if (i0 == 0) {
            for (int g2 = warp; g2 < G; g2 += kThreads / 32) {
                const float* w = ws_kvh + (size_t(g2) * a.splits + lane) * (HD + 2);
                const float m = lane < a.splits ? __ldcg(w) : -INFINITY;
                const float l = lane < a.splits ? __ldcg(w + 1) : 0.f;
                float M = m;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
                const float wt = exp_rel(m, M);
                float L = l * wt;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
                s_fw[lane][g2] = wt * (1.0f / L);
            }
            csync();
        }
        float2 A = make_float2(0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kMaxSplits; ++s) {
            const float wt = s < a.splits ? s_fw[s][g] : 0.f;
            A.x += pa[s].x * wt;
            A.y += pa[s].y * wt;
        }
        if (on) store_out2(a, (size_t(b) * a.nq + kvh * G + g) * HD + 2 * d2, A);
    }
}

}  // namespace

int attn_decode_splits(int pages, int groups, int sms, int hd, int heads_per_group) {
    // CTAs run in rounds over the resident slots (three CTAs per SM; two with 128-wide heads or four query heads per pass):
    // pick the split count whose rounds waste the least, a CTA's work being 1 / splits of a sequence plus a few per cent
    // per extra split for the merge.  Never more splits than pages.
    const int per_sm = (hd == 128 || heads_per_group >= 3) ? 2 : 3;
    const long slots = long(sms) * per_sm;
    const int smax = std::max(1, std::min(pages, kMaxSplits));
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= smax; ++s) {
        const long rounds = (long(groups) * s + slots - 1) / slots;
        const double cost = double(rounds) / s * (1.0 + 0.03 * (s - 1));
        if (cost < best_cost - 1e-12) { best_cost = cost; best = s; }
    }
    return best;
}

size_t attn_decode_ws_floats(int batch, int nq, int hd, int splits) { return size_t(batch) * nq * splits * (hd + 2); }

template <int HD, bool SW, int GC>
int32_t launch_decode(const CUtensorMap& mk, const CUtensorMap& mv, const DecParams& p, dim3 grid, cudaStream_t st) {
    const size_t smem = size_t(p.stages) * 2 * FORGE_KV_PAGE * HD * 2;
    auto kern = attn_decode_kernel<HD, SW, GC>;
    FORGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(size_t(kStages) * 2 * FORGE_KV_PAGE * HD * 2)));
    FORGE_CUDA(launch_pdl(kern, grid, dim3(kBlock), smem, st, mk, mv, p));
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

template <int GC>
int32_t launch_decode_hd(int hd, bool sw, const CUtensorMap& mk, const CUtensorMap& mv, const DecParams& p, dim3 grid, cudaStream_t st) {
    if (hd == 64) return sw ? launch_decode<64, true, GC>(mk, mv, p, grid, st) : launch_decode<64, false, GC>(mk, mv, p, grid, st);
    if (hd == 96) return sw ? launch_decode<96, true, GC>(mk, mv, p, grid, st) : launch_decode<96, false, GC>(mk, mv, p, grid, st);
    return sw ? launch_decode<128, true, GC>(mk, mv, p, grid, st) : launch_decode<128, false, GC>(mk, mv, p, grid, st);
}

int32_t attn_decode(const AttnDecodeArgs& a, cudaStream_t st) {
    if (a.nq % a.nkv) { set_error("attention: num_heads %d not a multiple of num_kv_heads %d", a.nq, a.nkv); return FORGE_ERR_SHAPE; }
    if (a.splits < 1 || (a.splits > 1 && (!a.ws || !a.counters))) { set_error("attention: split workspace missing"); return FORGE_ERR_INVALID_ARG; }
    if (a.nq / a.nkv > kMaxGroup) { set_error("attention: at most %d query heads per KV head", kMaxGroup); return FORGE_ERR_SHAPE; }
    if (a.splits > kMaxSplits) { set_error("attention: at most %d context splits", kMaxSplits); return FORGE_ERR_INVALID_ARG; }
    if (a.hd != 64 && a.hd != 96 && a.hd != 128) { set_error("attention: head_dim %d unsupported (64, 96, 128)", a.hd); return FORGE_ERR_SHAPE; }
    // tensor maps of the two pools: the caller's (a paged cache keeps them), or made here for a contiguous cache
    CUtensorMap mk, mv;
    if (a.map_k && a.map_v) {
        mk = *static_cast<const CUtensorMap*>(a.map_k);
        mv = *static_cast<const CUtensorMap*>(a.map_v);
    } else {
        const size_t rows = a.page_table ? 0 : size_t(a.batch) * a.max_ctx;
        if (!rows) { set_error("attention: a paged cache needs its tensor maps"); return FORGE_ERR_INVALID_ARG; }
        FORGE_TRY(make_kv_map(&mk, a.k_pool, a.hd, a.nkv, rows));
        FORGE_TRY(make_kv_map(&mv, a.v_pool, a.hd, a.nkv, rows));
    }
    // ring depth: the pages a CTA will see (per pass over the query heads), at most kStages
    const int ctx = a.seq_len ? a.max_ctx : a.seq_len_host;
    const int pages_per_cta = ((ctx + FORGE_KV_PAGE - 1) / FORGE_KV_PAGE + a.splits - 1) / a.splits;
    // three CTAs per SM (two with 128-wide heads) share its shared memory with their merge buffers: a ring of 48 KB
    // each for 64- and 96-wide heads (3 and 2 pages of K and V), 64 KB (2 pages) for 128-wide
    const int fit = std::max(2, int((56u << 10) / (2u * FORGE_KV_PAGE * a.hd * sizeof(__half))));
    DecParams p{a, 1.0f / sqrtf(float(a.hd)), pages_per_cta <= 2 ? 2 : std::min(kStages, fit)};
    dim3 grid(a.splits, a.nkv, a.batch);
    const int group = a.nq / a.nkv;
    if (group == 1) return launch_decode_hd<1>(a.hd, a.window > 0, mk, mv, p, grid, st);
    if (group == 2) return launch_decode_hd<2>(a.hd, a.window > 0, mk, mv, p, grid, st);
    return launch_decode_hd<4>(a.hd, a.window > 0, mk, mv, p, grid, st);
}

}  // namespace forge

// ------------------------------------------------------------------------------------------------
// forge_attention_flash_static: the same single-query attention for callers that must not allocate.
//
// Some hosts cannot let a library call cudaMalloc: a serving process whose own pool has already claimed
// the whole device (an allocation here would fail or fragment it), or a loop with a latency budget that
// cannot absorb the device-wide synchronisation an allocation or a free may imply.  forge_attention_flash
// gets its split-KV workspace from the stream-ordered allocator on every call; this variant keeps that
// workspace in a fixed array inside the library image instead (about 1.1 MB on every GPU that loads the
// library, until the process exits) and therefore accepts only shapes that fit it.
namespace {

constexpr int kStaticMaxHeads = 64;    // query heads (and KV heads)
constexpr int kStaticMaxSplits = 32;   // context splits, the same rule as forge_attention_flash
constexpr int kStaticMaxHeadDim = 128;
constexpr int kStaticMaxSeq = 1 << 20;

struct StaticScratch {
    float ws[size_t(kStaticMaxHeads) * kStaticMaxSplits * (kStaticMaxHeadDim + 2)];  // partial (m, l, acc) per head and split
    int counters[kStaticMaxHeads];                                                  // arrival tickets per KV head
};

// In host code this name is only a handle for the runtime; the device address comes from
// cudaGetSymbolAddress below and is what the kernel receives.
static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
StaticScratch* g_static_ptr[kMaxDevices] = {};

// Device address of the scratch on the current device; resolved once per device.
int32_t static_scratch(StaticScratch** out) {
    int dev = -1;
    FORGE_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) { forge::set_error("device index %d beyond %d", dev, kMaxDevices); return FORGE_ERR_UNSUPPORTED; }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        FORGE_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        g_static_ptr[dev] = static_cast<StaticScratch*>(p);
    }
    *out = g_static_ptr[dev];
    return FORGE_OK;
}

}  // namespace

extern "C" int32_t forge_attention_flash_static(float* out, const float* q, const uint16_t* k_cache, const uint16_t* v_cache,
                                                int32_t seq_len, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                                void* stream) {
    using namespace forge;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        set_error("no CUDA device: this backend has no CPU fallback");
        return FORGE_ERR_CUDA;
    }
    if (!out || !q || !k_cache || !v_cache || seq_len <= 0 || num_heads <= 0 || num_kv_heads <= 0) {
        set_error("bad argument to forge_attention_flash_static");
        return FORGE_ERR_INVALID_ARG;
    }
    if (num_heads > kStaticMaxHeads || num_kv_heads > kStaticMaxHeads || head_dim > kStaticMaxHeadDim || seq_len > kStaticMaxSeq) {
        set_error("forge_attention_flash_static: shape (%d heads, %d kv heads, head_dim %d, %d positions) exceeds the built-in scratch "
                  "(%d heads, head_dim %d, %d positions); use forge_attention_flash",
                  num_heads, num_kv_heads, head_dim, seq_len, kStaticMaxHeads, kStaticMaxHeadDim, kStaticMaxSeq);
        return FORGE_ERR_SHAPE;
    }
    StaticScratch* sc = nullptr;
    FORGE_TRY(static_scratch(&sc));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int splits = std::min(kStaticMaxSplits, attn_decode_splits((seq_len + FORGE_KV_PAGE - 1) / FORGE_KV_PAGE, num_kv_heads, 148, head_dim, num_heads / num_kv_heads));
    // the tickets must start at zero; the partials are fully rewritten by every call that reads them
    FORGE_CUDA(cudaMemsetAsync(sc->counters, 0, sizeof(int) * num_kv_heads, st));
    AttnDecodeArgs a{out, q, reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache), nullptr, 0, nullptr,
                     seq_len, 1, num_heads, num_kv_heads, head_dim, seq_len, sc->ws, sc->counters, splits};
    return attn_decode(a, st);
}
