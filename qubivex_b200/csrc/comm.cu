// The one exchange of the head-sharded decode path: an all-gather of the per-head attention outputs over
// NVLink with NCCL, then a transpose, both on the caller's stream.
//
// The reference has nothing here: one device per engine (crates/qubivex-runtime/src/engine.rs:1290; "More than
// one device" is not decided, docs/decisions/ADR-018-DISCRETE-DEVICE-MEMORY.md:106-113).  What makes the
// division by KV head free of any collective inside attention is the reference's own structure: a (token,
// head) result needs nothing from any other (crates/qubivex-arch/src/lib.rs:1304-1306), and a GQA group shares
// its keys and values with no other group.
//
// Each rank runs attention for its own KV heads and has it write [token][local head][d] straight into its
// slot of a gather buffer in its own memory; ncclAllGather (in place) fills the other ranks' slots of every
// rank's buffer; a small kernel turns [rank][token][local head][d] into the [token][head][d] the caller wants.
// No kernel here reads a peer's memory: NCCL moves the bytes, everything else works on local copies.
//
// NCCL is bound at run time (dlopen of libnccl.so.2; a process that already has one loaded -- PyTorch brings
// its own -- gets that one), so the library loads and the single-GPU path runs on hosts without NCCL.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <algorithm>

#include "qvx_common.cuh"

namespace qvx {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
    std::string why;
};

static const NcclApi& nccl() {
    static const NcclApi api = [] {
        NcclApi a;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            a.why = std::string("libnccl.so.2 cannot be loaded: ") + (dlerror() ? dlerror() : "unknown");
            return a;
        }
        a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(h, "ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))dlsym(h, "ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))dlsym(h, "ncclCommDestroy");
        a.AllGather = (decltype(a.AllGather))dlsym(h, "ncclAllGather");
        a.GetErrorString = (decltype(a.GetErrorString))dlsym(h, "ncclGetErrorString");
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllGather && a.GetErrorString;
        if (!a.ok) a.why = "libnccl.so.2 lacks a function this library needs";
        return a;
    }();
    return api;
}

static int32_t check_nccl(qvx_device* dev, ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return QVX_OK;
    return fail(dev, QVX_ERR_DEVICE, "cuda device error: %s: %s", what, nccl().GetErrorString(r));
}

// [rank][token][local head][d] -> [token][rank * local heads + local head][d], 16 bytes per thread.
__global__ void __launch_bounds__(256) gather_heads_kernel(const float4* __restrict__ g, float4* __restrict__ out, uint32_t nranks,
                                                           uint32_t s, uint32_t row4 /* local heads * d / 4 */) {
    const uint64_t total = (uint64_t)nranks * s * row4;
    for (uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x; i < total; i += (uint64_t)gridDim.x * 256u) {
        const uint32_t x = (uint32_t)(i % row4);
        const uint64_t rt = i / row4;
        const uint32_t t = (uint32_t)(rt % s), r = (uint32_t)(rt / s);
        out[((uint64_t)t * nranks + r) * row4 + x] = g[i];
    }
}

}  // namespace qvx

struct qvx_comm {
    qvx_device* dev = nullptr;
    ncclComm_t comm = nullptr;
    int nranks = 1, rank = 0;
    float* gather = nullptr;   // [rank][token][local head][d], this GPU's own memory
    size_t gather_floats = 0;  // one slot's capacity x nranks
    size_t slot_floats = 0;
};

using namespace qvx;

extern "C" {

int32_t qvx_comm_unique_id(uint8_t* id_out) {
    if (!id_out) return QVX_ERR_SHAPE;
    static_assert(sizeof(ncclUniqueId) == QVX_COMM_ID_BYTES, "the id the header promises is NCCL's");
    const NcclApi& api = nccl();
    if (!api.ok) return fail(nullptr, QVX_ERR_UNSUPPORTED, "head-sharded decode needs NCCL: %s", api.why.c_str());
    ncclUniqueId id;
    int32_t rc = check_nccl(nullptr, api.GetUniqueId(&id), "ncclGetUniqueId");
    if (rc) return rc;
    memcpy(id_out, &id, sizeof id);
    return QVX_OK;
}

int32_t qvx_comm_init(qvx_device* dev, int32_t nranks, int32_t rank, const uint8_t* id, size_t max_tokens, size_t heads_local,
                      size_t head_dim, qvx_comm** out) {
    if (!dev || !out || nranks < 1 || rank < 0 || rank >= nranks || (nranks > 1 && !id)) return QVX_ERR_SHAPE;
    *out = nullptr;
    if (max_tokens == 0 || heads_local == 0 || head_dim == 0 || head_dim % 4 != 0)
        return fail(dev, QVX_ERR_SHAPE, "shape mismatch in head gather: %zu tokens, %zu local heads of %zu", max_tokens, heads_local, head_dim);
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaError_t e = cudaSetDevice(dev->ordinal);
    if (e != cudaSuccess) return check_cuda(dev, e, "cudaSetDevice");
    qvx_comm* c = new qvx_comm;
    c->dev = dev; c->nranks = nranks; c->rank = rank;
    c->slot_floats = max_tokens * heads_local * head_dim;
    c->gather_floats = c->slot_floats * (size_t)nranks;
    // The gather buffer is allocated here, once: nothing is allocated per step.
    e = cudaMalloc((void**)&c->gather, c->gather_floats * 4);
    if (e != cudaSuccess) { delete c; return check_cuda(dev, e, "gather buffer"); }
    if (nranks > 1) {
        const NcclApi& api = nccl();
        if (!api.ok) { cudaFree(c->gather); delete c; return fail(dev, QVX_ERR_UNSUPPORTED, "head-sharded decode needs NCCL: %s", api.why.c_str()); }
        ncclUniqueId uid;
        memcpy(&uid, id, sizeof uid);
        int32_t rc = check_nccl(dev, api.CommInitRank(&c->comm, nranks, uid, rank), "ncclCommInitRank");
        if (rc) { cudaFree(c->gather); delete c; return rc; }
    }
    *out = c;
    return QVX_OK;
}

void qvx_comm_destroy(qvx_comm* c) {
    if (!c) return;
    {
        std::lock_guard<std::mutex> lk(c->dev->mu);
        cudaSetDevice(c->dev->ordinal);
        cudaDeviceSynchronize();
        if (c->comm) nccl().CommDestroy(c->comm);
        if (c->gather) cudaFree(c->gather);
    }
    delete c;
}

float* qvx_comm_send_slot(qvx_comm* c, size_t s, size_t heads_local, size_t head_dim) {
    if (!c || s * heads_local * head_dim > c->slot_floats) return nullptr;
    return c->gather + (size_t)c->rank * s * heads_local * head_dim;
}

int32_t qvx_allgather_heads(qvx_device* dev, qvx_comm* c, float* out_full, size_t s, size_t heads_local, size_t head_dim,
                            void* stream) {
    if (!dev || !c || c->dev != dev || !out_full) return QVX_ERR_SHAPE;
    const size_t count = s * heads_local * head_dim;
    if (count > c->slot_floats || head_dim % 4 != 0 || ((uintptr_t)out_full & 15u))
        return fail(dev, QVX_ERR_SHAPE, "shape mismatch in head gather: %zu tokens x %zu local heads of %zu (the buffer holds %zu floats per rank; "
                    "out must be 16-byte aligned)", s, heads_local, head_dim, c->slot_floats);
    if (count == 0) return QVX_OK;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaError_t e = cudaSetDevice(dev->ordinal);
    if (e != cudaSuccess) return check_cuda(dev, e, "cudaSetDevice");
    cudaStream_t st = (cudaStream_t)stream;
    if (c->nranks > 1) {
        // In place: this rank's slot already holds what attention wrote; the others' slots are filled.
        int32_t rc = check_nccl(dev, nccl().AllGather(c->gather + (size_t)c->rank * count, c->gather, count, ncclFloat, c->comm, st),
                                "ncclAllGather");
        if (rc) return rc;
    }
    const uint64_t total4 = (uint64_t)c->nranks * count / 4;
    const unsigned grid = (unsigned)std::min<uint64_t>((total4 + 255) / 256, 4u * 148u * 8u);
    gather_heads_kernel<<<grid, 256, 0, st>>>((const float4*)c->gather, (float4*)out_full, (uint32_t)c->nranks, (uint32_t)s,
                                              (uint32_t)(heads_local * head_dim / 4));
    return check_cuda(dev, cudaGetLastError(), "head gather launch");
}

}  // extern "C"
