/*
 * b200q.h -- C ABI of the B200 (sm_100a) quantized weight mat-mul: ggml's
 * GGML_OP_MUL_MAT and GGML_OP_MUL_MAT_ID over Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL and IQ4_XS
 * weights with f32 activations and f32 results.
 *
 * The entry points are what a ggml backend binds for this path. Each one names the
 * interface of marfrit/arcint's ggml-opencl backend it stands in for; "P01" etc. are
 * patch files under contrib/llama.cpp/patches/ of that tree and the numbers are
 * lines of the .patch file:
 *   P01  0000-01-kquant-integer-dpas.patch      P09  0000-09-moe-routing-gemm-tiles.patch
 *   P99  0099-opencl-q4_0-q8_0-int8-gemm.patch  P100 0100-opencl-downgrade-lines-and-counts.patch
 *   P103 0103-opencl-id-int8-sg8.patch          P115 0115-opencl-few-column-int8-q4_0-q8_0-iq4.patch
 *
 * Conventions
 *   - plain pointers and sizes only; every call returns a b200q_status and never aborts;
 *   - one context per GPU, used from one host thread at a time (ggml drives a backend
 *     instance from one thread); work is enqueued on the context's stream and is
 *     asynchronous to the host unless the call says otherwise;
 *   - tensor storage belongs to the caller; scratch belongs to the context, grows on
 *     demand and is never shrunk (the reference's prealloc_* buffers, P01:66-88);
 *   - there is no CPU fallback: a shape the kernels do not take is B200Q_UNSUPPORTED.
 */
#ifndef B200Q_H
#define B200Q_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B200Q_API
#else
#define B200Q_API __attribute__((visibility("default")))
#endif

typedef enum {
    B200Q_OK = 0,
    B200Q_UNSUPPORTED = 1,   /* shape / type / layout outside what the kernels take */
    B200Q_INVALID = 2,       /* null pointer, inconsistent sizes, id out of range    */
    B200Q_CUDA_ERROR = 3,
    B200Q_NO_MEMORY = 4,
    B200Q_NCCL_ERROR = 5,
    B200Q_TIMEOUT = 6,       /* a bounded device-side wait gave up                   */
    B200Q_PEER_FAILED = 7    /* a collective call that every rank left together because another rank reported an error */
} b200q_status;

/* ggml type ids (ggml.h enum ggml_type) */
enum {
    B200Q_TYPE_F32 = 0,
    B200Q_TYPE_Q4_0 = 2,
    B200Q_TYPE_Q8_0 = 8,
    B200Q_TYPE_Q4_K = 12,
    B200Q_TYPE_Q5_K = 13,
    B200Q_TYPE_Q6_K = 14,
    B200Q_TYPE_IQ4_NL = 20,
    B200Q_TYPE_IQ4_XS = 23,
    B200Q_TYPE_I32 = 26
};

enum { B200Q_OP_MUL_MAT = 0, B200Q_OP_MUL_MAT_ID = 1 };

/*
 * The fields of ggml_tensor this path reads (P01:817-857, 1174-1219): type, ne[4]
 * (elements per dimension, ne[0] fastest), nb[4] (strides in bytes) and the device
 * address of element 0 (ggml: extra->data_device + offset + view_offs).
 * `id` is the tensor's identity for the per-graph caches (ggml: the ggml_tensor pointer
 * itself, as the reference keys its caches: `c.src1 == src1`, P01:683-688; `rc.ids == ids`,
 * P01:1264-1287): ggml-alloc gives one address to several tensors of a graph in turn, so an
 * address alone does not say whose contents a buffer holds. NULL: no identity is known and the
 * caches compare address, shape and strides only -- then the caller must start a new
 * generation (b200q_graph_begin) whenever a buffer's contents may have changed.
 */
typedef struct {
    int32_t type;
    int64_t ne[4];
    size_t  nb[4];
    void   *data;
    const void *id;
} b200q_tensor;

typedef struct b200q_ctx b200q_ctx;

/* ggml_backend_opencl_init / ggml_backend_opencl_reg (P100:11-25): one context per
 * device. `stream` is a cudaStream_t (NULL: the context creates its own). */
B200Q_API b200q_status b200q_init(b200q_ctx **ctx, int device, void *stream);
B200Q_API void         b200q_free(b200q_ctx *ctx);
B200Q_API const char  *b200q_last_error(const b200q_ctx *ctx);
/* the cudaStream_t the context enqueues on (the caller's, or the one the context made) */
B200Q_API b200q_status b200q_get_stream(const b200q_ctx *ctx, void **stream);
B200Q_API const char  *b200q_version(void);

/* ggml_opencl_supports_op (P01:615-652) with the shape gate ggml_cl_kq_mul_mat_shape
 * (P01:807-812). B200Q_OK when b200q_mul_mat / b200q_mul_mat_id will take the op.
 * ctx may be NULL (the answer does not depend on the device). */
B200Q_API b200q_status b200q_supports(const b200q_ctx *ctx, int op, const b200q_tensor *src0,
                                      const b200q_tensor *src1, const b200q_tensor *ids,
                                      const b200q_tensor *dst);

/* ggml_cl_mul_mat (P01:1135-1158; Q4_0/Q8_0 arms P99:120-290; few-column arm
 * P115:588-594): dst[M, N] = src0[K, M] (quantized rows) x src1[K, N] (f32), the
 * weight broadcast over src1's dimensions 2 and 3. */
B200Q_API b200q_status b200q_mul_mat(b200q_ctx *ctx, const b200q_tensor *src0,
                                     const b200q_tensor *src1, b200q_tensor *dst);

/* ggml_cl_mul_mat_id (P01:1316-1328, ggml_cl_mul_mat_id_kq P01:1174-1313): src0
 * [K, M, n_expert], src1 [K, ne11 in {1, n_used}, n_tok] f32, ids [n_used, n_tok] i32
 * (row stride nb[1], may be a view), dst [M, n_used, n_tok]:
 * dst[:, i, t] = src0[ids[i, t]] x src1[:, i % ne11, t]  (P01:3917-3934). */
B200Q_API b200q_status b200q_mul_mat_id(b200q_ctx *ctx, const b200q_tensor *src0,
                                        const b200q_tensor *src1, const b200q_tensor *ids,
                                        b200q_tensor *dst);

/* The steps either side of MUL_MAT_ID in a mixture-of-experts feed-forward block.
 * b200q_moe_router: the reference's fused router kernel_topk_moe_softmax_norm_n* (P09:928-987): per token, softmax over
 * logits [n_expert, n_tok] f32, the n_used largest in descending order (ties: the lower expert id) into ids [n_used, n_tok]
 * i32, and their probabilities divided by clamp(their sum, cmin, cmax) into weights [n_used, n_tok] f32. At most 1024
 * experts and 32 used.
 * b200q_moe_ffn: router, gate and up MUL_MAT_ID over x [d_model, n_tok] (one route, one gathered activation), SwiGLU
 * h = silu(gate) * up, down MUL_MAT_ID over h, and y[:, t] = sum_i weights[i, t] * down[:, i, t] into y [d_model, n_tok],
 * as one launch sequence on the context's stream (scratch from the context, no host synchronisation). gate_w, up_w:
 * [d_model, d_ff, n_expert]; down_w: [d_ff, d_model, n_expert]. ids_out / weights_out may be NULL. The reference runs
 * these as separate graph nodes (no matmul + GLU fusion on its Intel path, P01:65). */
B200Q_API b200q_status b200q_moe_router(b200q_ctx *ctx, const b200q_tensor *logits, int n_used, float cmin, float cmax,
                                        b200q_tensor *ids, b200q_tensor *weights);
B200Q_API b200q_status b200q_moe_ffn(b200q_ctx *ctx, const b200q_tensor *gate_w, const b200q_tensor *up_w, const b200q_tensor *down_w,
                                     const b200q_tensor *x, const b200q_tensor *logits, int n_used, float cmin, float cmax,
                                     b200q_tensor *y, b200q_tensor *ids_out, b200q_tensor *weights_out);

/* ggml_backend_opencl_graph_compute's generation bump (P01:609-611): starts a new
 * graph. Within one graph an activation tensor that feeds several products (q/k/v,
 * gate/up) is quantized once (P01:670-688) and a MoE route is computed once per ids
 * tensor (P01:1264-1287); both caches are keyed by (identity, address, shape, strides,
 * generation): call this once per graph when tensors carry their `id`, and whenever tensor
 * contents may have changed when they do not. */
B200Q_API b200q_status b200q_graph_begin(b200q_ctx *ctx);

/* CUDA-graph replay of a recorded call sequence (what ggml's CUDA backend does for its
 * graph_compute; the reference's OpenCL backend enqueues each node, P01:855). Calls made on
 * the context between capture_begin and capture_end are recorded instead of run; the graph
 * then replays them on the context's stream with one launch. Scratch must already be large
 * enough (run the sequence once before capturing: growth inside a capture is refused), and
 * a graph is stale once the context's scratch has grown ("workspace_grow" in b200q_stats)
 * or any tensor it touched has moved. capture_begin and capture_end each start a new cache
 * generation, so a recorded sequence always holds its own quantize / route kernels and a replay
 * sees the tensors' current contents. */
typedef struct b200q_graph b200q_graph;
B200Q_API b200q_status b200q_capture_begin(b200q_ctx *ctx);
B200Q_API b200q_status b200q_capture_end(b200q_ctx *ctx, b200q_graph **graph);
B200Q_API b200q_status b200q_graph_launch(b200q_ctx *ctx, b200q_graph *graph);
B200Q_API void         b200q_graph_free(b200q_graph *graph);

/* Multi-GPU, one process and one context per GPU, NCCL over NVLink/NVSwitch. The reference
 * has no tensor- or expert-parallel mode (only a layer split through ggml's scheduler), so
 * these have no counterpart there; the single-GPU op result is what they must reproduce.
 *   column split: each rank owns a row range of the weight (b200q_tp_shard with unit 1) and
 *                 runs b200q_mul_mat on it; b200q_all_gather joins the row blocks if wanted;
 *   row split:    each rank owns a K range on block boundaries (unit = the type's block
 *                 size) of the weight and of the activation and runs b200q_mul_mat into a
 *                 full-size partial result; b200q_all_reduce_f32 sums the partials;
 *   expert split: each rank owns an expert range; b200q_all_to_all_v carries the routed
 *                 activations to their owners and the results back.
 * Rank 0 makes the 128-byte id, the launcher hands it to every rank. */
B200Q_API b200q_status b200q_tp_unique_id(void *id128);
B200Q_API b200q_status b200q_tp_init(b200q_ctx *ctx, const void *id128, int rank, int nranks);
B200Q_API b200q_status b200q_tp_rank(const b200q_ctx *ctx, int *rank, int *nranks);
B200Q_API b200q_status b200q_tp_shard(int64_t total, int64_t unit, int nranks, int rank, int64_t *first, int64_t *count);
B200Q_API b200q_status b200q_all_reduce_f32(b200q_ctx *ctx, void *dev_buf, size_t count);
B200Q_API b200q_status b200q_all_gather(b200q_ctx *ctx, const void *dev_send, void *dev_recv, size_t bytes_per_rank);
/* Row split in one call: dst [M, N] (packed) = the sum over the ranks of src0 (this rank's K shard) x src1 (its K range),
 * the same on every rank. At decode widths (1, 2, 4 or 8 columns) the product and the all-reduce are one kernel: the
 * partial sums leave the GEMV's registers as stores into every rank's mapped receive buffer over NVLink and the same
 * kernel adds them up in rank order; otherwise b200q_mul_mat followed by b200q_all_reduce_f32. Collective. */
B200Q_API b200q_status b200q_mul_mat_allreduce(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1, b200q_tensor *dst);
B200Q_API b200q_status b200q_all_to_all_v(b200q_ctx *ctx, const void *dev_send, const size_t *send_offsets,
                                          const size_t *send_bytes, void *dev_recv, const size_t *recv_offsets,
                                          const size_t *recv_bytes);
/* MUL_MAT_ID with the experts split over the ranks: src0_local holds this rank's experts
 * [K, M, n_expert_total / nranks]; src1, ids (global expert ids) and dst are this rank's tokens.
 * After b200q_ep_reserve dispatch and combine are the library's own kernels over peer memory; otherwise they are
 * NCCL all-to-alls and the call synchronizes the stream once (the exchange sizes must reach the host).
 * Every rank must make the same sequence of calls (the ranks wait for one another inside them).
 * Errors: in the NCCL form no rank leaves between collectives alone -- a rank-local error travels as a status word
 * beside the exchange sizes, and again before dispatch and combine, and every rank returns from the same point, the
 * failing rank with its own status, the others with B200Q_PEER_FAILED; the communicator stays usable. In the peer-memory
 * form a failing rank returns at once and the others' bounded waits end in B200Q_TIMEOUT; a call outside the reserved
 * bounds is B200Q_INVALID on the rank that made it. */
B200Q_API b200q_status b200q_mul_mat_id_ep(b200q_ctx *ctx, const b200q_tensor *src0_local, const b200q_tensor *src1,
                                           const b200q_tensor *ids, b200q_tensor *dst, int n_expert_total);
/* Collective (every rank, same arguments): reserves and maps, on every rank, the regions of peer memory that let
 * b200q_mul_mat_id_ep dispatch and combine from its own kernels, with no host synchronisation, so that the call
 * can be captured in a CUDA graph. max_pairs: the most (token, expert) pairs one rank brings to a call;
 * max_k / max_m: the longest activation / result rows (multiples of 4). Calls beyond the reserved bounds, and
 * every call when the mapping was refused or B200Q_NO_PEER_EP=1 is set, take the NCCL send/receive route. */
B200Q_API b200q_status b200q_ep_reserve(b200q_ctx *ctx, int64_t max_pairs, int64_t max_k, int64_t max_m);
B200Q_API b200q_status b200q_tp_check(b200q_ctx *ctx);

/* ggml backend buffer interface (buffer alloc, set_tensor, get_tensor, synchronize):
 * device memory for tensors and stream-ordered copies between host and device. */
B200Q_API b200q_status b200q_buffer_alloc(b200q_ctx *ctx, size_t bytes, void **dev_ptr);
B200Q_API b200q_status b200q_buffer_free(b200q_ctx *ctx, void *dev_ptr);
B200Q_API b200q_status b200q_tensor_set(b200q_ctx *ctx, void *dev_dst, const void *host_src, size_t bytes);
B200Q_API b200q_status b200q_tensor_get(b200q_ctx *ctx, void *host_dst, const void *dev_src, size_t bytes);
B200Q_API b200q_status b200q_tensor_copy(b200q_ctx *ctx, void *dev_dst, const void *dev_src, size_t bytes);
B200Q_API b200q_status b200q_synchronize(b200q_ctx *ctx);
/* The same copies on a second stream of the context, so that they overlap kernels instead of queueing
 * between them (ggml-cuda's copy-stream pattern for split buffers): _stage is host -> device and every
 * kernel queued after the call waits for it; _fetch is device -> host after everything queued before the
 * call and completes at the next b200q_synchronize. The caller double-buffers: a buffer being staged
 * must not still be read by queued kernels, one being fetched must not be rewritten before the synchronize. */
B200Q_API b200q_status b200q_tensor_stage(b200q_ctx *ctx, void *dev_dst, const void *host_src, size_t bytes);
B200Q_API b200q_status b200q_tensor_fetch(b200q_ctx *ctx, void *host_dst, const void *dev_src, size_t bytes);
/* page-locked host memory, so set/get copies run at full PCIe rate and asynchronously */
B200Q_API b200q_status b200q_host_alloc(size_t bytes, void **host_ptr);
B200Q_API b200q_status b200q_host_free(void *host_ptr);

/* The reference's "a path other than the promised one says so" counters
 * (ggml_cl_downgrade*, P100:51-64, 255-266): "key\tcount\n" lines, one per kernel
 * path taken since the context was made (or since b200q_stats_reset). The string
 * belongs to the context and is valid until the next call on it. */
B200Q_API const char  *b200q_stats(b200q_ctx *ctx);
B200Q_API void         b200q_stats_reset(b200q_ctx *ctx);

/* No counterpart in the reference (its backend always owns scratch buffers it may grow).
 * b200q_mul_mat for at most 8 activation columns of at most 32768 values each, for callers
 * that cannot allocate device memory: a host whose own pool took all of the GPU's memory at
 * start-up, or a serving loop that must not meet the device-wide synchronisation of
 * cudaMalloc / cudaFree. It needs no context and allocates nothing; the quantized activation
 * passes through a fixed 320 KiB array inside the library image (held by every GPU that loads
 * the library until the process exits). Larger shapes are refused with B200Q_UNSUPPORTED and a
 * message in b200q_noalloc_last_error(). All calls share that array and it keeps the last
 * call's contents (each call overwrites what it reads, so nothing needs clearing); calls that
 * overlap on one GPU race on it, so keep them ordered. The first call on a device looks up the
 * array's device address, so make that call before opening any stream capture; the first call for a
 * weight type and column count asks the driver for that kernel's attributes (and may make it load the
 * kernel's code), so a host about to take all device memory should first make one call per weight type
 * and column count it will use. `stream` is a cudaStream_t (NULL: the default stream); work is
 * enqueued, not waited for. b200q_noalloc_device_error reads (with a blocking copy) the word a kernel
 * of an earlier call set when one of its bounded waits gave up; zero means none did. */
B200Q_API b200q_status b200q_mul_mat_noalloc(int device, void *stream, const b200q_tensor *src0,
                                             const b200q_tensor *src1, b200q_tensor *dst);
B200Q_API const char  *b200q_noalloc_last_error(void);
B200Q_API b200q_status b200q_noalloc_device_error(int device, int *error);

/* Measurement and test helpers (device timers, an L2 flush, debug views of the kernels' operands, the failure-path
 * check) are declared in b200q_test.h: they are exported by the same library but are not part of the boundary a
 * backend binds. */

#ifdef __cplusplus
}
#endif
#endif
