/*
 * qvx — CUDA (sm_100a) backend for qubivex's paged KV-cache decode path.
 *
 * This is the whole boundary: a C ABI a `qubivex-backend-cuda` crate binds with
 * `extern "C"` to implement `qubivex_compute::discrete::DiscreteDevice` for the decode
 * attention stage (KV sync, KV append, paged decode attention) plus the block copies
 * that copy-on-write and compaction need, and the host-side block bookkeeping that in
 * the reference lives in `qubivex-runtime` and `qubivex-kv-cache`.
 *
 * Conventions
 *  - Every call returns an int32 status: 0 ok, 1 declined (nothing written), < 0 error,
 *    mirroring `ComputeError` (crates/qubivex-compute/src/lib.rs:26-83).  The text of
 *    the last error of a device is kept per device (`qvx_last_error`).
 *  - Pointers are DEVICE pointers unless the parameter name ends in `_host`.
 *  - `stream` is a `cudaStream_t` passed as `void*`; NULL is the legacy default stream.
 *    Calls whose name ends in `_host` are synchronous: complete on return, as
 *    `DiscreteDevice::routed_moe` is (crates/qubivex-compute/src/discrete.rs:561-569).
 *  - What a kernel finds out too late for a return code (a block id in device memory that is not
 *    the pool's, a position beyond a bound the caller gave, a bounded wait that ran out) goes
 *    into a per-device status word.  The host reads it at its next wait on that device
 *    (`qvx_wait`, any synchronous `_host` call, `qvx_get_kernel_times`), returns
 *    QVX_ERR_DEVICE with the reason in `qvx_last_error`, and clears it: the word is sticky
 *    until then, and the report may land on a later, unrelated call.
 *  - There is no CPU fallback anywhere: without a CUDA device `qvx_open` fails.
 *  - Paths cited are relative to the reference project's root.
 */
#ifndef QVX_H
#define QVX_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status (ComputeError, crates/qubivex-compute/src/lib.rs:26-83) ----------------- */
#define QVX_OK 0
#define QVX_DECLINED 1              /* Ok(false): nothing written                        */
#define QVX_ERR_SHAPE (-1)          /* ComputeError::Shape                               */
#define QVX_ERR_UNSUPPORTED (-2)    /* ComputeError::Unsupported                         */
#define QVX_ERR_CORE (-3)           /* ComputeError::Core (a size computation failed)    */
#define QVX_ERR_ELEMENT_TYPE (-4)   /* ComputeError::ElementType                         */
#define QVX_ERR_SHARED (-5)         /* ComputeError::Shared                              */
#define QVX_ERR_OUT_OF_MEMORY (-6)  /* ComputeError::OutOfDeviceMemory                   */
#define QVX_ERR_DEVICE (-7)         /* ComputeError::Device                              */

/* ---- element types (qubivex_core::DType names) and pool layouts ----------------------- */
#define QVX_F32 0
#define QVX_BF16 1
#define QVX_F16 2

/* The reference's block: keys [kv_head][d][B] then values [B][kv_head][d]
 * (crates/qubivex-compute/src/discrete.rs:247-256, :317-329), B generalised from 256. */
#define QVX_LAYOUT_REFERENCE 0
/* [block][kv_head][K|V][slot][d], the 16-byte chunk index of a row XORed with (slot & 7).
 * One position's row is contiguous (16-byte stores), one (block, kv head) page pair is
 * contiguous (one bulk copy).  Needs head_dim * element size to be a multiple of 128. */
#define QVX_LAYOUT_NATIVE 1

typedef struct qvx_geometry {
    uint32_t block_tokens; /* KV_BLOCK, discrete.rs:248 */
    uint32_t kv_heads;
    uint32_t head_dim;
    uint32_t dtype;
    uint32_t layout;
} qvx_geometry;

/* kv_block_words x element size (discrete.rs:253-256).  0 for a geometry that is not valid. */
size_t qvx_block_bytes(const qvx_geometry *geo);
/* Byte offset in the pool of key (kv = 0) or value (kv = 1) element (g, i) at pool position
 * `at` = block * block_tokens + slot: kv_key_word / kv_value_word (discrete.rs:317-329). */
size_t qvx_elem_offset(const qvx_geometry *geo, size_t at, int kv, size_t g, size_t i);

/* ---- the device (trait DiscreteDevice, crates/qubivex-compute/src/discrete.rs:433-570) -- */
typedef struct qvx_device qvx_device;
typedef struct qvx_buffer qvx_buffer;

/* As SimConfig / VulkanConfig (crates/qubivex-backend-cpu/src/sim.rs:46-72,
 * crates/qubivex-backend-vulkan/src/lib.rs:88-122). */
typedef struct qvx_config {
    int32_t device;     /* CUDA ordinal                                                   */
    uint64_t capacity;  /* bytes alloc/upload may hold in all; 0 = the device's free memory */
    uint64_t kv_pool;   /* DiscreteDevice::kv_pool(); 0 = None (the runtime's default)     */
    uint32_t timing;    /* n > 0: time every n-th launch of each kernel with CUDA events (TransferStats.timed) */
} qvx_config;

int32_t qvx_open(const qvx_config *cfg, qvx_device **dev);
void qvx_close(qvx_device *dev);
const char *qvx_name(void);                                          /* "cuda", :435   */
int32_t qvx_describe(qvx_device *dev, char *out, size_t cap);          /* :438           */
int32_t qvx_supports(qvx_device *dev, uint32_t dtype);                 /* :441, KV dtypes */
const char *qvx_last_error(qvx_device *dev);
uint64_t qvx_kv_pool(qvx_device *dev);                                 /* :554-559       */
uint64_t qvx_max_arena(qvx_device *dev);                               /* :525-529       */
int32_t qvx_routes_moe_attention(qvx_device *dev, size_t experts, size_t k, size_t s); /* :546-552 */

/* upload / alloc / write (discrete.rs:443-448, :493-523).  A buffer is reference counted
 * like the Arc inside DeviceBuffer (discrete.rs:28-63): qvx_retain adds a holder,
 * qvx_free drops one, the memory goes with the last. */
int32_t qvx_upload(qvx_device *dev, const void *data_host, size_t len, qvx_buffer **out);
int32_t qvx_alloc(qvx_device *dev, size_t len, qvx_buffer **out);
int32_t qvx_write(qvx_device *dev, qvx_buffer *buf, size_t offset, const void *data_host, size_t len);
int32_t qvx_read(qvx_device *dev, qvx_buffer *buf, size_t offset, void *data_host, size_t len);
void qvx_retain(qvx_buffer *buf);
void qvx_free(qvx_buffer *buf);
void *qvx_buffer_ptr(qvx_buffer *buf);
size_t qvx_buffer_len(qvx_buffer *buf);

/* DeviceUsage / TransferStats (discrete.rs:361-427). */
typedef struct qvx_usage {
    uint64_t capacity, used, peak, refused;
} qvx_usage;
typedef struct qvx_transfer_stats {
    uint64_t uploads, upload_bytes, activations_in, activations_out, submissions, transfer_ns,
        fence_waits, submit_ns, wait_ns, timed, gpu_ns, gpu_busy_ns;
} qvx_transfer_stats;
int32_t qvx_get_usage(qvx_device *dev, qvx_usage *out);
int32_t qvx_get_transfers(qvx_device *dev, qvx_transfer_stats *out);

/* Per-kernel device time, when the device was opened with timing = 1: launches and summed
 * nanoseconds per kernel family since the last reset.  (The reference times whole
 * submissions with timestamp queries, TransferStats.timed / gpu_ns.) */
#define QVX_K_SYNC 0
#define QVX_K_APPEND 1
#define QVX_K_ATTN 2     /* the split decode-attention kernel                              */
#define QVX_K_PRELUDE 3  /* clip, Q/K norms and RoPE before the store and attention            */
#define QVX_K_EXACT 4    /* the reference-order decode-attention kernel                    */
#define QVX_K_COPY 5     /* block copies (copy-on-write, compaction)                       */
#define QVX_K_COUNT 6
typedef struct qvx_kernel_times {
    uint64_t launches[QVX_K_COUNT];
    uint64_t gpu_ns[QVX_K_COUNT];
} qvx_kernel_times;
int32_t qvx_get_kernel_times(qvx_device *dev, qvx_kernel_times *out); /* drains pending events */
int32_t qvx_reset_kernel_times(qvx_device *dev);

/* ---- the kernels, on device memory ------------------------------------------------------ */

/* Rows the host cache holds and the pool does not: `kv_sync.comp`
 * (crates/qubivex-backend-vulkan/shaders/kv_sync.comp:1-51) and the sync loop of `put`
 * (crates/qubivex-backend-cpu/src/sim.rs:391-393).  rows: n x 2*kv_out f32 (key row, value
 * row); sync_to[r] = block * block_tokens + slot.  Positions must be distinct (the _host
 * call below resolves duplicates the reference's way: the later row wins).  `pool_blocks` is
 * the number of blocks `pool` holds: sync_to lives in device memory, so the kernel does the
 * check sim.rs:372-376 does on the host — a row for a block at or past pool_blocks is not
 * written and the device status reports it. */
int32_t qvx_kv_sync(qvx_device *dev, const qvx_geometry *geo, void *pool, size_t pool_blocks,
                    const float *rows, const uint32_t *sync_to, size_t n, void *stream);

/* Each token's new key and value row at its position: the store of `attn_prelude.comp`
 * (shaders/attn_prelude.comp:92-104, :169-173) and sim.rs:394-398.  k_new, v_new:
 * s x kv_out f32.  Token t's row goes to blocks[table_at[t] + pos[t] / B], slot pos[t] % B.
 * A row whose block id is at or past pool_blocks is not written (device status, as above);
 * the tables' own extent is the caller's to get right. */
int32_t qvx_kv_append(qvx_device *dev, const qvx_geometry *geo, void *pool, size_t pool_blocks,
                      const float *k_new, const float *v_new, const uint32_t *pos,
                      const uint32_t *blocks, const uint32_t *table_at, size_t s, void *stream);

/* Block tables of one decode op, resident on the device with the work list the split
 * kernel walks.  Built from host arrays, as DeviceMoeAttention carries them
 * (discrete.rs:292-297); validated as sim.rs:313-324, :359-376 does. */
typedef struct qvx_tables qvx_tables;
int32_t qvx_tables_create(qvx_device *dev, const qvx_geometry *geo, size_t pool_blocks, size_t heads,
                          size_t s, const uint32_t *pos_host, const uint32_t *blocks_host,
                          size_t n_blocks, const uint32_t *table_at_host, qvx_tables **out);
void qvx_tables_free(qvx_tables *t);
const uint32_t *qvx_tables_pos(qvx_tables *t);      /* device copies, for qvx_kv_append */
const uint32_t *qvx_tables_blocks(qvx_tables *t);
const uint32_t *qvx_tables_table_at(qvx_tables *t);

/* Which decode-attention kernel runs. */
#define QVX_ATTN_AUTO 0   /* the split kernel */
#define QVX_ATTN_SPLIT 1  /* GQA-grouped, online softmax, split over the context: within tolerance */
#define QVX_ATTN_EXACT 2  /* the order of math::attend, bit for bit (math.rs:142-155) */
/* May be or-ed into `variant` of the device-memory calls: the caller's word that nothing still
 * running in the stream writes the pool blocks or the tables this launch reads (e.g. the launch
 * before it served another layer, whose blocks are others).  Only q, k_new and v_new are then
 * taken to come from the stream's earlier work: the launch is made a programmatic dependent
 * launch, starts streaming the old positions while the launch before it drains, and waits
 * (griddepcontrol.wait) before it reads q, k_new or v_new or writes anything. */
#define QVX_ATTN_POOL_SETTLED 0x100
/* On the host-memory calls (qvx_paged_attention_host_async) the same flag says: no op still in flight
 * on this device writes the blocks this op reads or writes.  Ops so marked (with no sync rows) may run
 * their kernels side by side with the previous op's; an op without it waits for every op before it. */

/* Paged decode attention: `attn_decode.comp` (shaders/attn_decode.comp:60-175), the gather
 * and `attend` of sim.rs:400-429.  q, out: s x heads x head_dim f32, [token][head][d].
 * Token t reads positions 0..=pos[t] of its own table; query head h reads KV head
 * h / (heads / kv_heads). */
int32_t qvx_attn_decode(qvx_device *dev, qvx_tables *tables, const void *pool, const float *q,
                        float *out, uint32_t variant, void *stream);

/* The two stages of a decode step in the reference's order — each token's new row stored at
 * pos[t], then attention over 0..=pos[t] (crates/qubivex-backend-cpu/src/sim.rs:394-429;
 * `attn_prelude.comp` then `attn_decode.comp`) — as one call.  On native-layout pools the rows are
 * stored inside the attention launch (by the CTA that reads them); otherwise this is
 * qvx_kv_append followed by qvx_attn_decode.  k_new, v_new: s x kv_out f32. */
int32_t qvx_kv_append_attn_decode(qvx_device *dev, qvx_tables *tables, void *pool, const float *k_new,
                                  const float *v_new, const float *q, float *out, uint32_t variant, void *stream);

/* Paged decode attention for a caller that must not allocate device memory.  It has no
 * counterpart in the reference.  qubivex's runtime charges every device byte to a ledger and
 * gives the KV pool whatever the budget leaves, so a host that has committed the whole device
 * cannot have its backend call cudaMalloc later (it can fail, it is outside the ledger, and
 * cudaMalloc / cudaFree stall every stream in the middle of a decode step).  qvx_attn_decode
 * grows its scratch on demand and needs a qvx_tables object; this call needs neither: pos,
 * blocks and table_at are the caller's own device arrays (unchecked: a block id past the pool
 * is the caller's fault, as with qvx_kv_append), max_pos is a bound on pos[] the host knows
 * (a position beyond it is refused through the device status, nothing written for it), and
 * the scratch is a fixed array inside the library: 16 MiB of partial results + 16384
 * arrival counters, held on every GPU that loads the library until the process exits.
 * An op that needs more ((sequences x head groups) > 16384, or
 * sequences x head groups x ceil((max_pos + 1) / chunk) x (8 * head_dim + 16) x 4 bytes > 16 MiB, chunk = 576
 * positions rounded down to whole blocks, as in qvx_attn_decode)
 * returns QVX_ERR_UNSUPPORTED with the sizes in qvx_last_error.  bf16 or f16 pools in the native
 * layout, head_dim 64 or 128.  The first call on a device looks the array's address up: make
 * that call outside any stream capture.  All calls share the array: calls that overlap on
 * the GPU race on it, so keep them on one stream or order them. */
int32_t qvx_attn_decode_static(qvx_device *dev, const qvx_geometry *geo, const void *pool, size_t heads,
                               size_t s, const float *q, const uint32_t *pos, const uint32_t *blocks,
                               const uint32_t *table_at, uint32_t max_pos, float *out, void *stream);

/* The attention prelude: what SimDevice::attention does between the projections and the store
 * (crates/qubivex-backend-cpu/src/sim.rs:333-357; the device statement is
 * crates/qubivex-backend-vulkan/shaders/attn_prelude.comp:1-176), with the reference's bits:
 * z.clamp(-clip, clip) on q, k and v; the full-width RMS norms of each token's q row
 * (heads * head_dim values, weights q_norm) and k row (kv_heads * head_dim, k_norm) with the
 * 64-lane sum of squares (crates/qubivex-compute/src/math.rs:88-117, reduce.rs:12-47); NeoX RoPE
 * on every head of q and k from the token's table row [cos.., sin..] (math.rs:159-168).
 * Mirrors DeviceMoeAttention's clip / qk_norm / eps / rope fields (discrete.rs:281-289). */
typedef struct qvx_prelude {
    uint32_t has_clip;    /* Option<f32>: 0 = None                                          */
    float clip;           /* >= 0                                                           */
    const float *q_norm;  /* Option<(&[f32], &[f32])>: both NULL, or heads * head_dim and   */
    const float *k_norm;  /* kv_heads * head_dim weights                                    */
    double eps;           /* narrowed to f32 before use, as the reference does              */
    const float *rope;    /* s x head_dim, one row per token                                */
} qvx_prelude;
/* Device pointers throughout (the struct itself is read on the host); q [s][heads][d], k_new and
 * v_new [s][kv_heads][d] are changed in place: afterwards they are what attention and the store
 * take, and k_new / v_new what the host cache keeps (attn_prelude.comp's binding 2). */
int32_t qvx_attn_prelude(qvx_device *dev, const qvx_geometry *geo, size_t heads, size_t s, float *q,
                         float *k_new, float *v_new, const qvx_prelude *prelude, void *stream);

/* Whole-block copies src[i] -> dst[i]: the copy of a shared block before the first
 * divergent append, and the moves of a compaction pass.  No counterpart in the reference,
 * which copies a whole cache (crates/qubivex-arch/src/lib.rs:409-432) and never moves a
 * block.  src and dst are device arrays; no dst may also be a src or another dst.  A move
 * with either id at or past pool_blocks is skipped whole (device status, as above). */
int32_t qvx_block_copy(qvx_device *dev, const qvx_geometry *geo, void *pool, size_t pool_blocks,
                       const uint32_t *src, const uint32_t *dst, size_t n, void *stream);

/* ---- the head-sharded division over the GPUs of one box ----------------------------------- */

/* No counterpart in the reference, which has one device per engine
 * (crates/qubivex-runtime/src/engine.rs:1290).  Attention of a (token, head) needs nothing from any
 * other (crates/qubivex-arch/src/lib.rs:1304-1306), so each GPU can hold the pool of some KV heads
 * only and run the calls above on them unchanged; the single exchange is afterwards: every rank
 * has [token][its heads][d] and the caller wants [token][head][d].  One rank per GPU, ranks as
 * processes or as threads of one process; ranks own equal numbers of heads, in rank order.
 *
 * qvx_comm_unique_id: rank 0 makes the 128-byte id and the host hands it to the other ranks by
 * whatever means it has.  qvx_comm_init: every rank, at the same time (it is NCCL's
 * ncclCommInitRank and blocks until all have called); it also allocates, once, the gather buffer
 * for ops of up to max_tokens tokens, so that no step allocates.  nranks == 1 needs no id and no
 * NCCL.  NCCL is loaded at run time (libnccl.so.2): without it these calls return
 * QVX_ERR_UNSUPPORTED and everything else in this header still works. */
typedef struct qvx_comm qvx_comm;
#define QVX_COMM_ID_BYTES 128
int32_t qvx_comm_unique_id(uint8_t *id_out_host);
int32_t qvx_comm_init(qvx_device *dev, int32_t nranks, int32_t rank, const uint8_t *id_host, size_t max_tokens,
                      size_t heads_local, size_t head_dim, qvx_comm **out);
void qvx_comm_destroy(qvx_comm *comm);
/* Optional: the same exchange over peer memory, with no NCCL call per step.  Every rank calls
 * qvx_comm_peer_handle (it allocates the rank's result buffers, once, and describes them in
 * QVX_COMM_HANDLE_BYTES bytes), the host gathers the nranks handles in rank order and every rank calls
 * qvx_comm_peer_open with all of them (CUDA IPC between processes, peer access between threads of one
 * process).  From then on qvx_allgather_heads stores this rank's rows straight into every rank's
 * buffer over NVLink, already transposed, raises a flag on every rank, waits (bounded: a rank that
 * never arrives leaves "gave up a bounded wait" in the device status and nothing is handed over) for
 * every rank's flag and copies the result out.  Stores and flag words only cross GPUs.  If either call
 * fails (no peer access between the devices), the communicator keeps working over NCCL. */
#define QVX_COMM_HANDLE_BYTES 128
int32_t qvx_comm_peer_handle(qvx_comm *comm, uint8_t *handle_out_host);
int32_t qvx_comm_peer_open(qvx_comm *comm, const uint8_t *handles_host);
/* Where this rank's attention launch should write its [s][heads_local][d] outputs (pass it as `out` of
 * qvx_attn_decode / qvx_kv_append_attn_decode): the rank's own slot of the gather buffer, so that the
 * all-gather needs no copy in.  NULL if the op is larger than qvx_comm_init provided for. */
float *qvx_comm_send_slot(qvx_comm *comm, size_t s, size_t heads_local, size_t head_dim);
/* ncclAllGather (in place, over NVLink) of every rank's slot, then the transpose into out_full
 * [s][heads_local * nranks][d] (device memory of this GPU), all on `stream`, after whatever wrote the
 * slot there.  Every rank calls it, with the same s.  Nothing here reads another GPU's memory
 * directly: NCCL moves the bytes into this GPU's buffer first. */
int32_t qvx_allgather_heads(qvx_device *dev, qvx_comm *comm, float *out_full, size_t s, size_t heads_local,
                            size_t head_dim, void *stream);

/* ---- the op as the reference's device sees it, host memory in and out ------------------- */

/* DeviceMoeAttention after the projections, clip, norms and RoPE
 * (discrete.rs:266-307; SimDevice::attention, sim.rs:359-429): validate everything, write
 * the sync rows (a later duplicate wins), write each token's new row, then attention over
 * 0..=pos[t].  Synchronous.  QVX_ERR_SHAPE before anything is written. */
int32_t qvx_paged_attention_host(qvx_device *dev, qvx_buffer *pool, const qvx_geometry *geo,
                                 size_t heads, size_t s, const float *q_host,
                                 const float *k_new_host, const float *v_new_host,
                                 const uint32_t *pos_host, const uint32_t *blocks_host,
                                 size_t n_blocks, const uint32_t *table_at_host,
                                 const float *sync_host, const uint32_t *sync_to_host,
                                 size_t n_sync, float *out_host, uint32_t variant);

/* The same op with the waits taken out: the copies and kernels are queued on the device's
 * streams and `qvx_wait` (or the next synchronous call) completes them, so several layers' ops
 * overlap their copies with each other's kernels.  q, k_new, v_new, sync and out are copied
 * straight from / to the caller's arrays (only the block tables and the work list built from
 * them pass through the library's pinned staging ring): give PINNED host memory
 * (cudaHostAlloc / cudaHostRegister) for the copies to be asynchronous; from pageable memory
 * the CUDA runtime stages each copy and the call blocks for as long, which serialises the ops.
 * An out_host page-locked under this device and 16-byte aligned is not copied to at all: the attention kernel stores the
 * outputs into it over the bus while it runs (both calls; the bytes are the same either way).
 * The host arrays must stay unchanged until the wait; out_host is written by then. */
int32_t qvx_paged_attention_host_async(qvx_device *dev, qvx_buffer *pool, const qvx_geometry *geo,
                                       size_t heads, size_t s, const float *q_host,
                                       const float *k_new_host, const float *v_new_host,
                                       const uint32_t *pos_host, const uint32_t *blocks_host,
                                       size_t n_blocks, const uint32_t *table_at_host,
                                       const float *sync_host, const uint32_t *sync_to_host,
                                       size_t n_sync, float *out_host, uint32_t variant);
int32_t qvx_wait(qvx_device *dev);

/* DeviceMoeAttention after the projections only: the prelude above on the host's q, k_new and
 * v_new (the raw projections; `prelude` holds host pointers here), then the op of
 * qvx_paged_attention_host.  k_new_host and v_new_host are written back (clipped, normed,
 * rotated), as SimDevice::attention leaves them for the host cache (sim.rs:325-357).
 * Synchronous.  QVX_ERR_SHAPE (also for a negative or NaN clip) before anything is written. */
int32_t qvx_attention_stage_host(qvx_device *dev, qvx_buffer *pool, const qvx_geometry *geo,
                                 size_t heads, size_t s, const float *q_host, float *k_new_host,
                                 float *v_new_host, const qvx_prelude *prelude,
                                 const uint32_t *pos_host, const uint32_t *blocks_host,
                                 size_t n_blocks, const uint32_t *table_at_host,
                                 const float *sync_host, const uint32_t *sync_to_host,
                                 size_t n_sync, float *out_host, uint32_t variant);

/* Host-side block copy: lists in host memory, synchronous. */
int32_t qvx_block_copy_host(qvx_device *dev, qvx_buffer *pool, const qvx_geometry *geo,
                            const uint32_t *src_host, const uint32_t *dst_host, size_t n);

/* ---- block bookkeeping (host only; integers) -------------------------------------------- */

/* KvPool + KvFree (crates/qubivex-runtime/src/discrete.rs:215-243): the free list, LIFO,
 * first pop is block 0 (:447-449); plus one reference count per block, which the reference
 * does not have (a prefix hit there is a copy, docs/decisions/ADR-016-KV-SUBSYSTEM.md:32-37). */
typedef struct qvx_kvpool qvx_kvpool;
/* KvPoolStats (discrete.rs:91-108) and the counters of what the reference does not do. */
typedef struct qvx_kvpool_stats {
    uint64_t bytes, allocated, blocks, free, layers, synced_rows, full;
    uint64_t cow_copies, compaction_moves, bytes_moved, shared_blocks;
} qvx_kvpool_stats;

/* The pool's size rule (discrete.rs:429-455): min(configured or 512 MiB, 1 GiB, budget left,
 * max_arena) / block bytes.  `uncapped` != 0 skips the 512 MiB default and the 1 GiB cap and
 * takes `configured` as is (180 GB parts hold far larger pools). */
uint64_t qvx_kvpool_blocks_for(const qvx_geometry *geo, uint64_t configured, uint64_t budget_left,
                               uint64_t max_arena, int uncapped);
qvx_kvpool *qvx_kvpool_new(const qvx_geometry *geo, uint32_t blocks);
void qvx_kvpool_delete(qvx_kvpool *p);
/* Replaces the free list (in pop order: order[0] is handed out first).  Every free block
 * must appear once.  Lets a test hand blocks out in a seeded permutation. */
int32_t qvx_kvpool_set_free_order(qvx_kvpool *p, const uint32_t *order, size_t n);
int32_t qvx_kvpool_stats_get(qvx_kvpool *p, qvx_kvpool_stats *out);
uint32_t qvx_kvpool_refcount(qvx_kvpool *p, uint32_t block);
void qvx_kvpool_note_allocated(qvx_kvpool *p, int allocated); /* the buffer exists (kv_buffer, :502-512) */

/* Mirror / LayerMirror (discrete.rs:245-280): one sequence's blocks per layer, in position
 * order, and how many positions of each layer the pool holds.  Deleting it gives every block
 * back (Drop, :276-280). */
typedef struct qvx_seq qvx_seq;
qvx_seq *qvx_seq_new(qvx_kvpool *p, uint64_t epoch);
void qvx_seq_delete(qvx_seq *q);
size_t qvx_seq_blocks(qvx_seq *q, size_t layer, uint32_t *out, size_t cap); /* returns the count */
size_t qvx_seq_synced(qvx_seq *q, size_t layer);
/* A new sequence that shares the blocks holding positions 0..tokens of every layer of
 * `parent` (reference counts go up; nothing is copied): what a prefix hit becomes when the
 * retained value is a set of pages (ADR-016:82-89). */
qvx_seq *qvx_seq_fork(qvx_seq *parent, size_t tokens, uint64_t epoch);

/* attention_plan (discrete.rs:951-1009) for one layer over `s` sequences at positions
 * pos_host[]: epoch check and release, synced = min(synced, pos), blocks grown to
 * pos / B + 1, the flat tables, and the unsynced positions lmirror.synced..pos.
 * New here: a sequence about to write into a block someone else also holds gets a fresh
 * block and a (src, dst) copy is listed — copy-on-write.  Returns QVX_DECLINED when the
 * free list runs dry (blocks already taken stay with their sequence, `full` counts it). */
typedef struct qvx_plan qvx_plan;
int32_t qvx_plan_build(qvx_kvpool *p, qvx_seq *const *seqs, const uint64_t *epochs,
                       const uint32_t *pos_host, size_t s, size_t layer, qvx_plan **out);
void qvx_plan_free(qvx_plan *pl);
size_t qvx_plan_counts(qvx_plan *pl, size_t *n_blocks, size_t *n_sync, size_t *n_copies); /* returns s */
const uint32_t *qvx_plan_pos(qvx_plan *pl);
const uint32_t *qvx_plan_table_at(qvx_plan *pl);
const uint32_t *qvx_plan_blocks(qvx_plan *pl);
/* Unsynced rows: pool positions, and (sequence index, position) for the caller to fetch the
 * host cache's rows from. */
const uint32_t *qvx_plan_sync_to(qvx_plan *pl);
const uint32_t *qvx_plan_sync_seq(qvx_plan *pl);
const uint32_t *qvx_plan_sync_pos(qvx_plan *pl);
const uint32_t *qvx_plan_copy_src(qvx_plan *pl);
const uint32_t *qvx_plan_copy_dst(qvx_plan *pl);
/* After the device ran the op (discrete.rs:929-943): synced = pos + 1 per sequence, the
 * `layers` and `synced_rows` counters. */
void qvx_plan_commit(qvx_kvpool *p, qvx_plan *pl, qvx_seq *const *seqs, size_t layer);

/* Compaction (no counterpart in the reference, whose blocks never move,
 * crates/qubivex-runtime/src/discrete.rs:227-243).  With L live blocks: every live block
 * with id >= L, ascending, moves to the free ids < L, ascending; the tables of every live
 * sequence of the pool are rewritten; the free list becomes L..blocks, lowest first.  The
 * moves are returned for qvx_block_copy (cap too small: QVX_ERR_SHAPE, nothing changed). */
int32_t qvx_kvpool_compact(qvx_kvpool *p, uint32_t *src_out, uint32_t *dst_out, size_t cap,
                           size_t *n_moves);

/* ---- the prefix index (crates/qubivex-kv-cache/src/lib.rs:22-209) ----------------------- */
#define QVX_MIN_REUSE 32 /* lib.rs:22 */
typedef struct qvx_prefix_cache qvx_prefix_cache;
typedef struct qvx_prefix_stats {
    uint64_t lookups, hits, tokens_reused, inserted, evicted, entries, cost;
} qvx_prefix_stats;
/* The value is an opaque u64 handle with a release callback standing in for Arc<V>: the
 * callback runs when the index has dropped the value and every hit on it was released. */
typedef void (*qvx_release_fn)(uint64_t value, void *user);
qvx_prefix_cache *qvx_prefix_new(uint64_t budget, qvx_release_fn release, void *user);
void qvx_prefix_delete(qvx_prefix_cache *c);
/* lookup (lib.rs:119-140): 1 and *value, *reuse, *hit on a hit, else 0.  scope NULL = None. */
int32_t qvx_prefix_lookup(qvx_prefix_cache *c, const char *scope, const uint32_t *prompt, size_t n,
                          uint64_t *value, size_t *reuse, uint64_t *hit);
void qvx_prefix_hit_release(qvx_prefix_cache *c, uint64_t hit);
/* insert (lib.rs:146-181): 1 kept, 0 not kept (the value is released at once). */
int32_t qvx_prefix_insert(qvx_prefix_cache *c, const char *scope, const uint32_t *tokens, size_t n,
                          uint64_t cost, uint64_t value);
int32_t qvx_prefix_evict_oldest(qvx_prefix_cache *c); /* lib.rs:184-199 */
void qvx_prefix_clear(qvx_prefix_cache *c);             /* lib.rs:202-204 */
void qvx_prefix_stats_get(qvx_prefix_cache *c, qvx_prefix_stats *out);
uint64_t qvx_prefix_budget(qvx_prefix_cache *c);

#ifdef __cplusplus
}
#endif
#endif /* QVX_H */
