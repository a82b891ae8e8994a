// Tensor-parallel collective of the forward path: the sum over ranks after the row-sliced projections (attention
// output and FFN down), as the reference's tensor-parallel plan would need it.  One process per GPU; the sum is an
// NCCL all-reduce on the model's stream (NVLink / NVSwitch, in-switch reduction when NCCL enables it), so it is
// captured into the decode graph like any kernel.  NCCL is bound at run time (dlopen of libnccl.so.2): a
// single-GPU user of the library needs no NCCL at all.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "common.cuh"

namespace forge {

struct TpComm {
    void* lib = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    decltype(&ncclGetUniqueId) get_id = nullptr;
    decltype(&ncclCommInitRank) init_rank = nullptr;
    decltype(&ncclAllReduce) all_reduce = nullptr;
    decltype(&ncclCommDestroy) destroy = nullptr;
    decltype(&ncclGetErrorString) err_string = nullptr;
};

namespace {

int32_t bind(TpComm& c) {
    c.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!c.lib) { set_error("tensor parallelism needs libnccl.so.2: %s", dlerror()); return FORGE_ERR_UNSUPPORTED; }
    c.get_id = reinterpret_cast<decltype(c.get_id)>(dlsym(c.lib, "ncclGetUniqueId"));
    c.init_rank = reinterpret_cast<decltype(c.init_rank)>(dlsym(c.lib, "ncclCommInitRank"));
    c.all_reduce = reinterpret_cast<decltype(c.all_reduce)>(dlsym(c.lib, "ncclAllReduce"));
    c.destroy = reinterpret_cast<decltype(c.destroy)>(dlsym(c.lib, "ncclCommDestroy"));
    c.err_string = reinterpret_cast<decltype(c.err_string)>(dlsym(c.lib, "ncclGetErrorString"));
    if (!c.get_id || !c.init_rank || !c.all_reduce || !c.destroy || !c.err_string) { set_error("libnccl.so.2 lacks a required symbol"); return FORGE_ERR_UNSUPPORTED; }
    return FORGE_OK;
}

}  // namespace

static_assert(sizeof(ncclUniqueId) == FORGE_TP_ID_BYTES, "FORGE_TP_ID_BYTES must match ncclUniqueId");

int32_t tp_unique_id(uint8_t* out) {
    TpComm c;
    FORGE_TRY(bind(c));
    ncclUniqueId id;
    ncclResult_t r = c.get_id(&id);
    if (r != ncclSuccess) { set_error("ncclGetUniqueId: %s", c.err_string(r)); return FORGE_ERR_COMM; }
    memcpy(out, &id, sizeof(id));
    return FORGE_OK;
}

int32_t tp_init(TpComm** out, const uint8_t* id_bytes, int rank, int world) {
    TpComm* c = new TpComm();
    int32_t rc = bind(*c);
    if (rc != FORGE_OK) { delete c; return rc; }
    ncclUniqueId id;
    memcpy(&id, id_bytes, sizeof(id));
    ncclResult_t r = c->init_rank(&c->comm, world, id, rank);
    if (r != ncclSuccess) { set_error("ncclCommInitRank: %s", c->err_string(r)); delete c; return FORGE_ERR_COMM; }
    c->rank = rank; c->world = world;
    *out = c;
    return FORGE_OK;
}

int32_t tp_allreduce_sum(TpComm* c, float* buf, size_t n, cudaStream_t st) {
    if (!c) { set_error("tensor-parallel model without a communicator: call forge_model_tp_init first"); return FORGE_ERR_INVALID_ARG; }
    ncclResult_t r = c->all_reduce(buf, buf, n, ncclFloat32, ncclSum, c->comm, st);
    if (r != ncclSuccess) { set_error("ncclAllReduce: %s", c->err_string(r)); return FORGE_ERR_COMM; }
    ++g_launches;
    return FORGE_OK;
}

// ------------------------------------------------------------------ the sum over peer memory, batched rows
// hidden[i] += sum over ranks of part_r[i], for the `count` values (rows x hidden) of a batched decode step, in one
// kernel instead of an all-reduce and an add.  Every thread owns two values: it stores them as {value, tag} pairs
// (8 bytes each, written whole, so a pair whose tag matches is complete) into every peer's exchange buffer, then
// polls its own buffer for the peers' pairs of the same two values and adds the parts in rank order, which makes the
// result the same bits on every rank.  The tag numbers the sum (decode step x sums per step + index), so nothing is
// ever cleared; two slots alternate, and a rank cannot run two sums ahead of a peer because its next sum needs that
// peer's contribution.  The wait is bounded: when it gives up the error word is set and the thread moves on.
namespace {

constexpr int kPairThreads = 256;

__global__ void __launch_bounds__(kPairThreads) tp_pair_sum_kernel(float* hidden, const float* part, uint2* const* peer_ll, const uint2* local_ll,
                                                                   size_t region, size_t cap, int count, int world, int rank, int slot,
                                                                   const uint32_t* step_counter, uint32_t step_mul, uint32_t step_add,
                                                                   uint32_t limit, int* err) {
    const int i = (blockIdx.x * kPairThreads + threadIdx.x) * 2;
    if (i >= count) return;
    const uint32_t tag = *step_counter * step_mul + step_add;
    const float2 mine = *reinterpret_cast<const float2*>(part + i);
    const uint4 out = make_uint4(__float_as_uint(mine.x), tag, __float_as_uint(mine.y), tag);
    const size_t at = region + (size_t(slot) * world + rank) * cap + i;
    for (int d = 1; d < world; ++d) {
        const int r = (rank + d) % world;  // every rank starts with a different peer
        asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(peer_ll[r] + at), "r"(out.x), "r"(out.y), "r"(out.z), "r"(out.w) : "memory");
    }
    float2 acc = make_float2(0.f, 0.f);
    for (int r = 0; r < world; ++r) {
        if (r == rank) { acc.x += mine.x; acc.y += mine.y; continue; }
        const uint2* src = local_ll + region + (size_t(slot) * world + r) * cap + i;
        uint4 a = make_uint4(0, 0, 0, 0);
        bool ok = false;
        for (uint32_t t = 0; t < limit && !ok; ++t) {
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src) : "memory");
            ok = a.y == tag && a.w == tag;
            if (!ok && (t & 1023) == 1023 && *reinterpret_cast<volatile int*>(err)) break;  // another thread already gave up
        }
        if (!ok) { atomicExch(err, 1); a.x = 0; a.z = 0; }
        acc.x += __uint_as_float(a.x); acc.y += __uint_as_float(a.z);
    }
    float2 h = *reinterpret_cast<const float2*>(hidden + i);
    h.x += acc.x; h.y += acc.y;
    *reinterpret_cast<float2*>(hidden + i) = h;
}

}  // namespace

int32_t tp_pair_sum(float* hidden, const float* part, uint2* const* peer_ll, const uint2* local_ll, size_t region, size_t cap, int count,
                    int world, int rank, int slot, const uint32_t* step_counter, uint32_t step_mul, uint32_t step_add, uint32_t limit,
                    int* err, cudaStream_t st) {
    if (count <= 0 || (count & 1) || size_t(count) > cap) { set_error("peer sum: %d values do not fit the exchange buffer", count); return FORGE_ERR_INVALID_ARG; }
    const int blocks = (count / 2 + kPairThreads - 1) / kPairThreads;
    tp_pair_sum_kernel<<<blocks, kPairThreads, 0, st>>>(hidden, part, peer_ll, local_ll, region, cap, count, world, rank, slot, step_counter,
                                                        step_mul, step_add, limit, err);
    FORGE_LAUNCH_CHECK();
    return FORGE_OK;
}

void tp_destroy(TpComm* c) {
    if (!c) return;
    if (c->comm) c->destroy(c->comm);
    delete c;
}

}  // namespace forge
