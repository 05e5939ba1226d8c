// common.cuh -- shared host/device declarations of the b200q library (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/b200q.h"
#include "../../include/b200q_test.h"

#define QK   32
#define QK_K 256

namespace b200q {

// ---- block formats ------------------------------------------------------------------

struct TypeInfo {
    int    block;        // weights per block
    int    bytes;        // bytes per block
    int    act_form;     // 0: per-32 activation (fp16 scale), 1: per-256 (f32 scale + sums)
    const char *name;
};

__host__ __device__ inline bool type_info(int type, TypeInfo *ti) {
    switch (type) {
        case B200Q_TYPE_Q4_0:   *ti = { 32, 18, 0, "q4_0" };    return true;
        case B200Q_TYPE_Q8_0:   *ti = { 32, 34, 0, "q8_0" };    return true;
        case B200Q_TYPE_Q4_K:   *ti = { 256, 144, 1, "q4_K" };  return true;
        case B200Q_TYPE_Q5_K:   *ti = { 256, 176, 1, "q5_K" };  return true;
        case B200Q_TYPE_Q6_K:   *ti = { 256, 210, 1, "q6_K" };  return true;
        case B200Q_TYPE_IQ4_XS: *ti = { 256, 136, 1, "iq4_xs" }; return true;
        case B200Q_TYPE_IQ4_NL: *ti = { 32, 18, 0, "iq4_nl" };   return true;
        default: return false;
    }
}

enum { ACT_Q8_0 = 0, ACT_Q8_256 = 1, ACT_Q8_0_TILED = 2, ACT_Q8_256_TILED = 3 };   // TILED: the tensor-core GEMM's chunk layout

// Quantized activation as the kernels read it: column c of K values at
//   codes  + c*K            int8
//   d16    + c*(K/32)       fp16 bits, per-32 form
//   d32    + c*(K/256)      f32,       per-256 form
//   s32    + c*(K/32)       int16 sums of each 32 codes, both forms
//   s16    + c*(K/16)       int16 sums of each 16 codes, per-256 form
struct ActView {
    const int8_t   *codes;
    const uint16_t *d16;
    const float    *d32;
    const int16_t  *s32;
    const int16_t  *s16;
    int             form;
    int64_t         K;
    int64_t         N;
};

// ---- context ------------------------------------------------------------------------

struct Workspace {
    void  *ptr = nullptr;
    size_t cap = 0;
    void  *base = nullptr;   // start of the allocation: ptr, or WS_GUARD bytes before it when guard words surround the block
};

constexpr size_t WS_GUARD = 256;          // bytes of guard words on each side of a scratch block (B200Q_CANARY=1)
constexpr int    WS_GUARD_BYTE = 0xC5;

struct ActKey {
    const void *data;
    const void *id;          // the caller's tensor identity (NULL: unknown)
    int64_t ne[4];
    size_t  nb[4];
    int     form;
    uint64_t gen;
    bool operator==(const ActKey &o) const {
        if (data != o.data || id != o.id || form != o.form || gen != o.gen) return false;
        for (int i = 0; i < 4; ++i) if (ne[i] != o.ne[i] || nb[i] != o.nb[i]) return false;
        return true;
    }
};

struct ActEntry {
    ActKey    key;
    Workspace codes, scales, sums, sums16;
    bool      valid = false;
};

struct RouteEntry;

// Path-taken counters (the reference's downgrade counters, P100:51-64): fixed slots so a
// launch does not pay for a string.
enum Stat {
    ST_QUANT_Q8_0, ST_QUANT_Q8_256, ST_ACT_CACHE_HIT, ST_WORKSPACE_GROW, ST_MUL_MAT_GEMV_CHUNKS,
    ST_GEMV_COL0,                                 // + ncols (1..8)
    ST_GEMV_UNALIGNED_COL0 = ST_GEMV_COL0 + 9,    // + ncols
    ST_GEMV_ID = ST_GEMV_UNALIGNED_COL0 + 9, ST_GEMV_ID_UNALIGNED, ST_MOE_ROUTE, ST_ROUTE_CACHE_HIT, ST_MOE_GEMM,
    ST_MOE_PACK, ST_GEMM_TC, ST_GEMM_TC_QUANT, ST_GEMM_FALLBACK_SHAPE, ST_TP_ALLREDUCE, ST_TP_ALLGATHER,
    ST_EP_DISPATCH, ST_EP_COMBINE, ST_GRAPH_LAUNCH, ST_NO_ALLOC, ST_GEMM_KQ_MINS, ST_GEMV_STREAM, ST_TP_ALLREDUCE_PEER, ST_GEMM_TC_F16, ST_EP_PEER, ST_EP_DISPATCH_CACHED, ST_MOE_ROUTER, ST_MOE_FFN, ST_GEMV_KNOB_IGNORED, ST_GEMM_KSPLIT, ST_GEMV_FUSED_QUANT, ST_GEMV_ALLREDUCE_FUSED,
    ST_EP_AGREED_EXIT, ST_GEMM_KQ_ROWCOPY, ST_GEMV_MMA,
    ST_COUNT
};
const char *stat_name(int s);

}  // namespace b200q

struct b200q_ctx {
    int          device = 0;
    cudaStream_t stream = nullptr;
    bool         own_stream = false;
    int          sm_count = 148;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;   // overlapped host copies (b200q_tensor_stage / _fetch), one stream per direction
    cudaEvent_t  ev_fork = nullptr, ev_join = nullptr;
    bool         copy_pending = false;    // the copy streams hold work the compute stream has not joined
    uint64_t     generation = 1;
    // what the gathered, tiled activation scratch of the tensor-core MUL_MAT_ID holds (gate and up of a layer
    // read the same src1 through the same ids: the second call finds it ready)
    struct { const void *src1 = nullptr, *ids = nullptr, *src1_id = nullptr, *ids_id = nullptr; int64_t ne[4] = {0, 0, 0, 0}; size_t nb[4] = {0, 0, 0, 0}; uint64_t gen = 0; int per32 = -1, n_expert = 0; } moe_act;
    bool         route_skip_negative = false;   // expert-parallel local product: negative ids are empty slots
    int          route_pinned = -1;       // a route entry in use across a nested call: not a victim
    uint64_t     private_generation = 0;  // expert-parallel calls: generations of their internal products
    bool         capturing = false;
    bool         no_tc = false;           // B200Q_NO_TC=1: never take the tensor-core GEMM
    bool         no_pdl = false;          // B200Q_NO_PDL=1: plain stream order between the decode kernels
    bool         tc_f16 = true;           // B200Q_TC_I8=1: the per-32 prompt GEMM on the int8 MMA instead of exact fp16 operands
    // decode GEMV tile knobs (read once from the environment; 0 / -1: the measured defaults): rows per ring stage,
    // warps per block, and which column counts take the slice-resident kernel (bit c = c columns)
    int          gemv_rows = 0, gemv_block_warps = 0, gemv_stream_mask = -1;
    // B200Q_FUSE_QUANT_BYTES: per-32 decode products up to this many weight bytes quantize their activation inside the GEMV.
    // Off (0) by default: it saves a launch, but every warp then starts with two dependent global loads and the quantizer's
    // arithmetic in front of its first row, where the separate quantizer runs under the previous GEMV's tail (programmatic
    // dependent launch). Measured on the 7B decode trace: -2 % at two GPUs, +38 % at eight (1.48 against 1.08 ms).
    int64_t      fuse_quant_bytes = 0;
    bool         no_ksplit = false;       // B200Q_NO_KSPLIT=1: never cut a prompt product along K
    bool         canary = false;          // B200Q_CANARY=1: guard words around every scratch block, exact sizes (b200q_debug_check_guards)
    bool         gemv_mma_sets3 = false;  // B200Q_GEMV_MMA_SETS=3: a three-stage ring for the warp-MMA GEMV even where four stages fit
    int          gemv_mma_groups = 0;     // B200Q_GEMV_MMA_GROUPS=1: blocks of one group (several blocks per SM) instead of one block per SM
    int          gemv_mma_slice = 0;      // B200Q_GEMV_MMA_SLICE=2|3|4: super-blocks per warp of the warp-MMA GEMV (0: by row length)
    int          gemv_mma_min = 0;        // B200Q_GEMV_MMA_MIN: fewest columns at which a product takes the warp-MMA GEMV (99: never; 0: Q6_K 3, Q8_0 7, the others 4, measured)
    bool         gemv_no_small = false;   // B200Q_GEMV_NO_SMALL=1: never the 128-thread, 170-register build of the wide Q6_K GEMV
    bool         moe_mins_pass = false;   // B200Q_MOE_MINS_PASS=1: Q4_K route tiles take the mins term in a separate pass
    bool         no_stream = false;       // B200Q_NO_STREAM=1: every GEMV through the per-warp ring kernel (comparisons)
    std::string  last_error;
    std::string  stats_text;
    uint64_t     counters[b200q::ST_COUNT] = {};
    // quantized-activation cache: a few entries, reused round-robin
    std::vector<b200q::ActEntry> act_cache;
    size_t       act_next = 0;
    b200q::Workspace flush_buf;
    b200q::Workspace moe_ws[10];
    b200q::RouteEntry *routes[2] = { nullptr, nullptr };
    size_t       route_next = 0;
    cudaEvent_t  ev0 = nullptr, ev1 = nullptr;
    void        *tp = nullptr;   // tensor/expert-parallel state (tp.cu)
    int         *error_word = nullptr;   // device word a kernel sets when a bounded wait runs out
};

namespace b200q {

b200q_status fail(b200q_ctx *ctx, b200q_status st, const char *fmt, ...);
b200q_status ws_reserve(b200q_ctx *ctx, Workspace *ws, size_t bytes);
void ws_release(Workspace *ws);
int moe_route_workspaces(b200q_ctx *ctx, Workspace **out, const char **names);   // the route caches' blocks, for the guard check
inline void  count(b200q_ctx *ctx, int stat) { ++ctx->counters[stat]; }

#define B200Q_CUDA(ctx, expr)                                                                       \
    do {                                                                                            \
        cudaError_t e_ = (expr);                                                                    \
        if (e_ != cudaSuccess)                                                                      \
            return b200q::fail((ctx), B200Q_CUDA_ERROR, "%s: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                               __FILE__, __LINE__);                                                 \
    } while (0)

// quantize.cu
b200q_status launch_quantize_act(b200q_ctx *ctx, int form, const b200q_tensor *src1, int8_t *codes, void *scales,
                                 int16_t *sums32, int16_t *sums16);
b200q_status launch_dequantize(b200q_ctx *ctx, int type, const void *w, int64_t M, int64_t K, size_t row_stride,
                               float *out);

// gemv.cu: dst[m + c*ldd] for c < ncols (<= 8), rows [0, M)
b200q_status launch_gemv(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                         const ActView &act, int64_t col0, int ncols, float *dst, int64_t ldd);
// the same for one or two columns of a small Q4_0 / Q8_0 product, quantizing src1 inside the kernel;
// B200Q_UNSUPPORTED: not that case, take the quantizer + launch_gemv
b200q_status launch_gemv_fused(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                               const b200q_tensor *src1, int ncols, float *dst, int64_t ldd);

// MUL_MAT_ID over route tiles of at most tile_pairs (1, 2, 4 or 8) pairs of one expert; tiles == NULL:
// direct mode, one pair per unit with its expert read from ids on the device (small token counts)
b200q_status launch_gemv_id(b200q_ctx *ctx, int type, const void *w, size_t row_stride, size_t expert_stride,
                            int64_t M, int64_t K, const ActView &av, int tile_pairs, const int32_t *tiles,
                            const int32_t *n_tiles, int64_t max_tiles, const int32_t *pairs, const b200q_tensor *ids,
                            int n_expert, int n_used, int ne11, float *dst, int64_t ld1, int64_t ld2);
// the product of a K shard and the all-reduce of the ranks' partial results in one kernel (gemv_stream.cuh); av: the
// quantized activation, or NULL with src1 to quantize inside the kernel; peers / state: the all-reduce's mapped
// buffers and device words (tp.cu). B200Q_UNSUPPORTED: the shape does not qualify.
b200q_status launch_gemv_allreduce(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K, const ActView *av,
                                   const b200q_tensor *src1, int ncols, float *dst, int64_t ldd, uint64_t *const *peers, uint32_t *state,
                                   int rank, int nranks);
bool gemv_ar_shape_ok(int type, const void *w, size_t row_stride, int64_t M, int64_t K, int ncols, int64_t ldd);
// api.cu: the quantized activation of src1 in the decode layout of the weight type's form (cached per graph)
b200q_status get_decode_activation(b200q_ctx *ctx, int weight_type, const b200q_tensor *src1, ActView *out);
// moe.cu: route (pairs sorted by expert, tile lists by size class)
// Kernel attributes (dynamic shared memory opt-in, occupancy) belong to a device, and one process may hold
// contexts on several: per-kernel tables indexed by device ordinal replace per-process flags.
constexpr int B200Q_MAX_DEVICES = 64;

struct RouteView {
    const int32_t *pairs;          // [n_pairs]
    const int32_t *tiles[4];       // class k: tiles of at most 1, 2, 4, 8 pairs (int4 each)
    const int32_t *tiles128;       // tiles of at most 128 pairs (tensor-core path), every pair once
    const int32_t *n_tiles;        // [5] device counters: the four classes, then the 128-pair list
    int64_t        max_tiles;      // upper bound of every list
    int64_t        max_tiles128;   // upper bound of the 128-pair list
    int            slot;           // which of the context's route entries holds this view
    const int32_t *owner_counts;   // expert parallelism: pairs per owner rank (device), else unused
};
// MUL_MAT_ID view of the tensor-core GEMM: column c of tile n is pair pairs[first + c] of expert
// tiles[4n] (tiles == nullptr: a dense product, column = token).
struct TileRoute {
    const int32_t *tiles;      // [n][4]: expert, first pair, count, -
    const int32_t *n_tiles;    // device scalar
    const int32_t *pairs;      // pairs sorted by expert
    int            n_used, ne11;
    size_t         nb1, nb2;   // src1: bytes between slot rows and between tokens
    int64_t        ld1, ld2;   // dst: floats between slots and between tokens
};
b200q_status make_weight_tmap3(b200q_ctx *ctx, void *tmap_out, const void *w, size_t row_stride, int64_t M, int64_t row_bytes,
                               int box_bytes, int64_t n_mat, size_t mat_stride);
// tensor map of a packed weight matrix seen as [M rows][row_bytes / 4] 32-bit elements, box = 128 rows x box_bytes
b200q_status make_weight_tmap(b200q_ctx *ctx, void *tmap_out, const void *w, size_t row_stride, int64_t M, int64_t row_bytes,
                              int box_bytes);
b200q_status moe_route(b200q_ctx *ctx, const b200q_tensor *ids, int n_expert, RouteView *out, int experts_per_owner = 0);
b200q_status launch_ep_pack(b200q_ctx *ctx, const b200q_tensor *src1, const b200q_tensor *ids, int n_expert,
                            int experts_per_owner, const int32_t *pairs, float *send_x, int32_t *send_e);
b200q_status launch_ep_unpack(b200q_ctx *ctx, const float *back, const int32_t *pairs, int n_used, int n_pairs, int M,
                              float *dst, int64_t ld1, int64_t ld2);
void         moe_free(b200q_ctx *ctx);

// tp.cu
void         tp_free(b200q_ctx *ctx);

// gemm_tc.cu: tensor-core prefill GEMM (Q4_0, Q8_0)
bool         gemm_tc_supported(int type, int64_t M, int64_t K, int64_t N, const void *w, size_t row_stride);
size_t       gemm_tc_act_bytes(int64_t K, int64_t N);
b200q_status launch_quantize_tiled(b200q_ctx *ctx, const b200q_tensor *src1, uint8_t *out);
size_t       gemm_tc_id_act_bytes(int64_t K, int64_t max_tiles);
b200q_status launch_gemm_tc_id(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1, const TileRoute &tr,
                               int64_t max_tiles, uint8_t *act, float *dst, bool act_ready);
b200q_status launch_gemm_tc(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                            const uint8_t *act, int64_t N, float *dst, int64_t ldd);

// gemm_kq.cu: tensor-core prefill GEMM for the super-block types IQ4_XS, Q4_K and Q6_K (integer sub-scales folded into two int8 limbs)
bool         gemm_kq_supported(int type, int64_t M, int64_t K, int64_t N, const void *w, size_t row_stride);
size_t       gemm_kq_act_bytes(int64_t K, int64_t N);
b200q_status launch_quantize_tiled256(b200q_ctx *ctx, const b200q_tensor *src1, uint8_t *out);
size_t       gemm_kq_id_act_bytes(int64_t K, int64_t max_tiles);
b200q_status launch_gemm_kq_id(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1, const TileRoute &tr,
                               int64_t max_tiles, uint8_t *act, float *dst, bool act_ready);
b200q_status launch_gemm_kq(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                            const uint8_t *act, int64_t N, float *dst, int64_t ldd);

}  // namespace b200q
