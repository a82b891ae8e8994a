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

void tp_destroy(TpComm* c) {
    if (!c) return;
    if (c->comm) c->destroy(c->comm);
    delete c;
}

}  // namespace forge
