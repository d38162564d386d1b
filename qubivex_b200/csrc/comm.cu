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
// A second way for the same exchange needs no NCCL call per step (qvx_comm_peer_*): every rank maps the others' result
// buffers (CUDA IPC between processes, peer access inside one process) and, after attention, one kernel stores the
// rank's rows straight into every rank's buffer over NVLink, already transposed, and raises a flag there; a second
// kernel waits (bounded) for every rank's flag and hands the gathered rows to the caller.  Stores and flag words
// only: no load and no bulk copy ever reads another GPU's memory.
//
// NCCL is bound at run time (dlopen of libnccl.so.2; a process that already has one loaded -- PyTorch brings
// its own -- gets that one), so the library loads and the single-GPU path runs on hosts without NCCL.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>
#include <unistd.h>

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

extern int* device_status_word(qvx_device* dev);
#ifndef QVX_WAIT_LIMIT
#define QVX_WAIT_LIMIT (1u << 20)
#endif
constexpr uint32_t WAIT_LIMIT = QVX_WAIT_LIMIT;  // polls of the bounded wait below (with its back-off: about a second)

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

constexpr int MAX_PEERS = 16;
struct PeerArgs {
    float4* full[MAX_PEERS];      // every rank's result buffer (this step's half), [token][rank][row4]
    uint32_t* flags[MAX_PEERS];   // every rank's flag words: flags[p][r] = the last step rank r has finished writing to rank p
};

// This rank's [token][row4] rows into every rank's [token][rank][row4] buffer, then (the last CTA to finish) this rank's
// flag on every rank.  `done` is a counter in this GPU's memory, zero between launches.
__global__ void __launch_bounds__(256) scatter_heads_kernel(const float4* __restrict__ local, PeerArgs pa, uint32_t nranks,
                                                            uint32_t rank, uint32_t s, uint32_t row4, uint32_t step, uint32_t* done) {
    const uint64_t total = (uint64_t)s * row4;
    for (uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x; i < total; i += (uint64_t)gridDim.x * 256u) {
        const uint32_t x = (uint32_t)(i % row4), t = (uint32_t)(i / row4);
        const float4 v = local[i];
        const uint64_t at = ((uint64_t)t * nranks + rank) * row4 + x;
        for (uint32_t p = 0; p < nranks; p++) pa.full[(p + rank) % nranks][at] = v;  // (each rank starts with itself: the links share the load)
    }
    __threadfence_system();  // this thread's stores are visible on every GPU before the arrival is counted
    __syncthreads();
    __shared__ uint32_t last;
    if (threadIdx.x == 0) last = atomicAdd(done, 1u) == gridDim.x - 1 ? 1u : 0u;
    __syncthreads();
    if (!last) return;
    __threadfence_system();
    if (threadIdx.x < nranks) *reinterpret_cast<volatile uint32_t*>(pa.flags[threadIdx.x] + rank) = step;
    if (threadIdx.x == 0) *done = 0;
}

// Waits (bounded) until every rank's flag in this GPU's memory shows `step`, then copies the gathered rows out.
__global__ void __launch_bounds__(256) collect_heads_kernel(const float4* __restrict__ full, float4* __restrict__ out,
                                                            const uint32_t* flags, uint32_t nranks, uint64_t total4, uint32_t step,
                                                            int* status) {
    __shared__ uint32_t ok;
    if (threadIdx.x == 0) {
        bool all = false;
        for (uint32_t i = 0; i < WAIT_LIMIT && !all; i++) {
            all = true;
            for (uint32_t r = 0; r < nranks; r++)
                all = all && (int32_t)(*reinterpret_cast<const volatile uint32_t*>(flags + r) - step) >= 0;
            if (!all && i > 64) __nanosleep(64);
        }
        if (!all) atomicExch(status, STATUS_WAIT_TIMEOUT);
        __threadfence_system();
        ok = all ? 1u : 0u;
    }
    __syncthreads();
    if (!ok) return;  // a rank never arrived: nothing is handed over, the host reads the status
    for (uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x; i < total4; i += (uint64_t)gridDim.x * 256u) out[i] = __ldcg(full + i);
}

}  // namespace qvx

struct qvx_comm {
    qvx_device* dev = nullptr;
    ncclComm_t comm = nullptr;
    int nranks = 1, rank = 0;
    float* gather = nullptr;   // [rank][token][local head][d], this GPU's own memory
    size_t gather_floats = 0;  // one slot's capacity x nranks
    size_t slot_floats = 0;
    // the peer-memory path (qvx_comm_peer_*): one allocation the other ranks map: two result buffers, used by
    // alternate steps, then the flag words and the scatter kernel's counter
    uint8_t* shared = nullptr;
    size_t full_bytes = 0;                    // one result buffer: nranks slots
    void* peer_base[qvx::MAX_PEERS] = {};     // every rank's `shared` as this process sees it
    bool peer_ipc[qvx::MAX_PEERS] = {};       // opened through CUDA IPC (to be closed)
    bool peers_open = false;
    uint32_t step = 0;
};

struct qvx_peer_handle {                      // what qvx_comm_peer_handle writes: QVX_COMM_HANDLE_BYTES
    int64_t pid;
    int32_t device;
    int32_t reserved;
    uint64_t pointer;
    cudaIpcMemHandle_t ipc;
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
        for (int p = 0; p < c->nranks && p < MAX_PEERS; p++)
            if (c->peer_ipc[p] && c->peer_base[p]) cudaIpcCloseMemHandle(c->peer_base[p]);
        if (c->shared) cudaFree(c->shared);
    }
    delete c;
}

float* qvx_comm_send_slot(qvx_comm* c, size_t s, size_t heads_local, size_t head_dim) {
    if (!c || s * heads_local * head_dim > c->slot_floats) return nullptr;
    return c->gather + (size_t)c->rank * s * heads_local * head_dim;
}

int32_t qvx_comm_peer_handle(qvx_comm* c, uint8_t* handle_out) {
    static_assert(sizeof(qvx_peer_handle) <= QVX_COMM_HANDLE_BYTES, "the handle fits what the header promises");
    if (!c || !handle_out) return QVX_ERR_SHAPE;
    qvx_device* dev = c->dev;
    if (c->nranks > MAX_PEERS) return fail(dev, QVX_ERR_UNSUPPORTED, "the peer-memory gather serves at most %d ranks", MAX_PEERS);
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaError_t e = cudaSetDevice(dev->ordinal);
    if (e != cudaSuccess) return check_cuda(dev, e, "cudaSetDevice");
    if (!c->shared) {
        c->full_bytes = (c->gather_floats * 4 + 255) & ~(size_t)255;
        const size_t bytes = 2 * c->full_bytes + 256;
        e = cudaMalloc((void**)&c->shared, bytes);
        if (e == cudaSuccess) e = cudaMemset(c->shared, 0, bytes);
        if (e != cudaSuccess) { c->shared = nullptr; return check_cuda(dev, e, "peer gather buffer"); }
    }
    qvx_peer_handle h{};
    h.pid = (int64_t)getpid(); h.device = dev->ordinal; h.pointer = (uint64_t)(uintptr_t)c->shared;
    e = cudaIpcGetMemHandle(&h.ipc, c->shared);
    if (e != cudaSuccess) return check_cuda(dev, e, "cudaIpcGetMemHandle");
    memset(handle_out, 0, QVX_COMM_HANDLE_BYTES);
    memcpy(handle_out, &h, sizeof h);
    return QVX_OK;
}

int32_t qvx_comm_peer_open(qvx_comm* c, const uint8_t* handles) {
    if (!c || !handles) return QVX_ERR_SHAPE;
    qvx_device* dev = c->dev;
    if (!c->shared || c->nranks > MAX_PEERS)
        return fail(dev, QVX_ERR_SHAPE, "qvx_comm_peer_open: call qvx_comm_peer_handle on every rank first");
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaError_t e = cudaSetDevice(dev->ordinal);
    if (e != cudaSuccess) return check_cuda(dev, e, "cudaSetDevice");
    for (int p = 0; p < c->nranks; p++) {
        qvx_peer_handle h;
        memcpy(&h, handles + (size_t)p * QVX_COMM_HANDLE_BYTES, sizeof h);
        if (p == c->rank) { c->peer_base[p] = c->shared; continue; }
        if (h.pid == (int64_t)getpid()) {
            // Another rank of this process (ranks as threads): its pointer is valid here once peer access is on.
            int can = 0;
            e = cudaDeviceCanAccessPeer(&can, dev->ordinal, h.device);
            if (e == cudaSuccess && !can) return fail(dev, QVX_ERR_UNSUPPORTED, "device %d cannot reach device %d's memory", dev->ordinal, h.device);
            if (e == cudaSuccess) {
                e = cudaDeviceEnablePeerAccess(h.device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
            }
            if (e != cudaSuccess) return check_cuda(dev, e, "peer access");
            c->peer_base[p] = (void*)(uintptr_t)h.pointer;
        } else {
            void* mapped = nullptr;
            e = cudaIpcOpenMemHandle(&mapped, h.ipc, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) { cudaGetLastError(); return check_cuda(dev, e, "cudaIpcOpenMemHandle (peer gather buffer)"); }
            c->peer_base[p] = mapped;
            c->peer_ipc[p] = true;
        }
    }
    c->peers_open = true;
    return QVX_OK;
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
    if (c->nranks > 1 && c->peers_open) {
        // Over peer memory: this rank's rows go straight into every rank's result buffer, transposed; then the flags.
        const uint32_t step = ++c->step, half = step & 1u;
        PeerArgs pa{};
        for (int p = 0; p < c->nranks; p++) {
            pa.full[p] = (float4*)((uint8_t*)c->peer_base[p] + half * c->full_bytes);
            pa.flags[p] = (uint32_t*)((uint8_t*)c->peer_base[p] + 2 * c->full_bytes);
        }
        uint32_t* my_flags = (uint32_t*)(c->shared + 2 * c->full_bytes);
        const uint32_t row4 = (uint32_t)(heads_local * head_dim / 4);
        const uint64_t mine4 = (uint64_t)s * row4, total4 = mine4 * (uint64_t)c->nranks;
        const unsigned g1 = (unsigned)std::min<uint64_t>((mine4 + 255) / 256, 2u * 148u);
        scatter_heads_kernel<<<g1, 256, 0, st>>>((const float4*)(c->gather + (size_t)c->rank * count), pa, (uint32_t)c->nranks,
                                                 (uint32_t)c->rank, (uint32_t)s, row4, step, my_flags + MAX_PEERS);
        const unsigned g2 = (unsigned)std::min<uint64_t>((total4 + 255) / 256, 4u * 148u);
        collect_heads_kernel<<<g2, 256, 0, st>>>((const float4*)(c->shared + half * c->full_bytes), (float4*)out_full, my_flags,
                                                 (uint32_t)c->nranks, total4, step, device_status_word(dev));
        return check_cuda(dev, cudaGetLastError(), "peer gather launch");
    }
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
