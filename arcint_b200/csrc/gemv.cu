// gemv.cu -- decode GEMV for 1..8 activation columns: dst[:, c] = W x_c.
//
// HBM-bound (every packed weight byte is read once for all columns), CUDA cores only:
// each warp streams R rows through a private ring of shared-memory stages filled with
// 16-byte asynchronous copies (coalesced 128-bit reads of the packed GGUF blocks, several
// stages in flight per warp), every lane decodes 32 weights of a stage and runs dp4a
// against the int8 activation codes it holds in registers for all columns, and the warp
// reduces with shuffles. No tensor cores. Rows whose byte length or address is not a
// multiple of 16 take the same kernel with a plain 2-byte copy loop as the loader.
//
// Stands in for the reference's kernel_mul_mv_*_q8_1 family
// (marfrit/arcint contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch:3882-3915,
// host side ggml_cl_mul_mv_kq_q8_1 at :817-857).
#include "gemv_kernel.cuh"
#include "gemv_stream.cuh"
#include "gemv_mma.cuh"
#include "common.cuh"

#include <limits.h>

namespace b200q {

template <int TYPE, int NC, int B, int WARPS, int NSETS, bool ID>
static b200q_status launch_one(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K,
                               const GemvAct &act, float *dst, int64_t ldd, bool aligned, const GemvId &id,
                               int64_t max_tiles) {
    typedef GemvStage<TYPE> S;
    const size_t smem = (size_t)WARPS * NSETS * B * S::SLOT;
    if (M > INT32_MAX / 2 || K / GemvFmt<TYPE>::BLK_W > INT32_MAX / 256 || ldd > INT32_MAX)
        return fail(ctx, B200Q_UNSUPPORTED, "gemv: dimensions beyond 32-bit indexing");
    auto kern_a = gemv_kernel<TYPE, NC, B, WARPS, NSETS, true, ID>;
    auto kern_u = gemv_kernel<TYPE, NC, B, WARPS, NSETS, false, ID>;
    auto kern = aligned ? kern_a : kern_u;
    // resident CTAs per SM of this instantiation, asked once: the grid is one full wave of
    // persistent CTAs (or fewer when the work is small) and each warp strides over its units
    static int occ_dev[B200Q_MAX_DEVICES][2] = {};
    int *occ = occ_dev[ctx->device % B200Q_MAX_DEVICES];
    if (occ[aligned] == 0) {
        if (smem > 48 * 1024)
            B200Q_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int n = 0;
        B200Q_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, WARPS * 32, smem));
        occ[aligned] = n > 0 ? n : 1;
    }
    const int64_t n_bt = (M + B - 1) / B;
    const int64_t n_units = ID ? n_bt * max_tiles : n_bt;      // ID: an upper bound, the kernel reads the count
    int64_t blocks = (n_units + WARPS - 1) / WARPS;
    const int64_t cap = (int64_t)ctx->sm_count * occ[aligned];
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    B200Q_CUDA(ctx, launch_pdl(!ctx->no_pdl, kern, dim3((unsigned)blocks), dim3(WARPS * 32), smem, ctx->stream,
                               (const uint8_t *)w, row_stride, (int)M, (int)(K / GemvFmt<TYPE>::BLK_W), act, dst, (int)ldd, id));
    B200Q_CUDA(ctx, cudaGetLastError());
    return B200Q_OK;
}

// One launch of the slice-resident kernel built with the launch bounds (MAXT, MINB); resident blocks per SM for the
// block shape are asked once per (device, shape).
template <int TYPE, int NC, int R, int NSETS, bool QX, bool AR, int MAXT, int MINB>
static b200q_status launch_stream_kernel(b200q_ctx *ctx, int threads, size_t smem, int groups, const void *w, size_t row_stride, int64_t M,
                                         int nblk, const GemvAct &act, float *dst, int64_t ldd, const GemvAr &ar_args) {
    auto kern = gemv_stream_kernel<TYPE, NC, R, NSETS, QX, AR, MAXT, MINB>;
    struct Occ { int threads; size_t smem; int blocks; bool attr; };
    static Occ occ_dev[B200Q_MAX_DEVICES] = {};
    Occ &o = occ_dev[ctx->device % B200Q_MAX_DEVICES];
    if (!o.attr) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return fail(ctx, B200Q_CUDA_ERROR, "gemv_stream attribute: %s", cudaGetErrorString(e));
        o.attr = true;
    }
    if (o.threads != threads || o.smem != smem) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem);
        if (e != cudaSuccess) return fail(ctx, B200Q_CUDA_ERROR, "gemv_stream occupancy: %s", cudaGetErrorString(e));
        o.threads = threads;
        o.smem = smem;
        o.blocks = n > 0 ? n : 1;
    }
    const int64_t n_units = (M + R - 1) / R;
    int64_t blocks = (n_units + groups - 1) / groups;
    const int64_t cap = (int64_t)ctx->sm_count * o.blocks;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaError_t e = launch_pdl(!ctx->no_pdl, kern, dim3((unsigned)blocks), dim3(threads), smem, ctx->stream, (const uint8_t *)w,
                               row_stride, (int)M, nblk, act, dst, (int)ldd, groups, ctx->error_word, ar_args);
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? B200Q_OK : fail(ctx, B200Q_CUDA_ERROR, "gemv_stream launch: %s", cudaGetErrorString(e));
}

// The slice-resident kernel (gemv_stream.cuh) for rows that bulk copies can fetch (16-byte aligned
// start, stride and length). Returns false when the shape does not fit it: more than 16 warps per
// group (K beyond 16 slices, or 8 for more than four columns) or a ring beyond shared memory.
template <int TYPE, int NC, int R, bool QX = false, bool AR = false>
static bool try_launch_stream(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K, const GemvAct &act,
                              float *dst, int64_t ldd, b200q_status *st, const GemvAr *ar = nullptr) {
    typedef GemvFmt<TYPE> F;
    constexpr int CW = NC > 4 ? 2 : 1, NSETS = 3;      // a four-stage ring at one and two columns measured 5-15 % slower
    const int nblk = (int)(K / F::BLK_W), nsl = (nblk + F::STAGE_BLOCKS - 1) / F::STAGE_BLOCKS, nw = nsl * CW;
    if (nw > GEMV_STREAM_MAX_THREADS / 32) return false;
    const int row_bytes = nblk * F::BLK_B;
    const size_t gb = (gemv_stream_group_smem(row_bytes, R, NSETS, nw) + 15) / 16 * 16;
    if (gb > 200 * 1024) return false;
    int target_warps = 4;                                  // blocks of about four warps measured best
    if (ctx->gemv_block_warps) {
        if (ctx->gemv_block_warps >= 1 && ctx->gemv_block_warps <= GEMV_STREAM_MAX_THREADS / 32) target_warps = ctx->gemv_block_warps;
        else count(ctx, ST_GEMV_KNOB_IGNORED);
    }
    int groups = target_warps / nw < 1 ? 1 : target_warps / nw;
    if (groups * nw > GEMV_STREAM_MAX_THREADS / 32) groups = (GEMV_STREAM_MAX_THREADS / 32) / nw;
    while (groups > 1 && groups * gb > 200 * 1024) --groups;
    const size_t smem = groups * gb;
    const int threads = groups * nw * 32;
    GemvAr ar_args = {};
    if (ar) ar_args = *ar;
    // Q6_K at four and more columns in blocks of one 128-thread group: the build with room for 170 registers
    constexpr bool has_small = ((TYPE == B200Q_TYPE_Q6_K && NC >= 2) || (TYPE == B200Q_TYPE_Q4_K && NC >= 4)) && !QX && !AR;
    if constexpr (has_small) {
        if (threads <= 128 && !ctx->gemv_no_small) {
            // (two blocks per SM with up to 255 registers measured slower: Q6_K 8 columns 60.4 against 55.5 us)
            *st = launch_stream_kernel<TYPE, NC, R, NSETS, QX, AR, 128, 3>(ctx, threads, smem, groups, w, row_stride, M, nblk, act, dst, ldd, ar_args);
            return true;
        }
    }
    *st = launch_stream_kernel<TYPE, NC, R, NSETS, QX, AR, GEMV_STREAM_MAX_THREADS, 0>(ctx, threads, smem, groups, w, row_stride, M, nblk, act, dst,
                                                                                      ldd, ar_args);
    return true;
}

// The warp-MMA kernel (gemv_mma.cuh) for rows that bulk copies can fetch. Returns false when the shape does not fit it:
// more than twelve warps per group (K beyond 12288) or a ring beyond shared memory.
template <int TYPE, int NSETS, int SLICE>
static bool try_launch_mma(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K, const GemvAct &act, int ncols,
                           float *dst, int64_t ldd, b200q_status *st) {
    typedef GemvFmt<TYPE> F;
    constexpr int MAX_WARPS = gemv_mma_max_threads(SLICE) / 32;
    constexpr size_t SMEM_CAP = 227 * 1024;
    if (K % 256) return false;                                     // the kernel counts in chunks of 256 weights
    const int nblk = (int)(K / 256), nw = (nblk + SLICE - 1) / SLICE;
    if (nw > MAX_WARPS) return false;
    const int row_bytes = nblk * gemv_mma_chunk_bytes<TYPE>();
    const size_t gb = (gemv_mma_group_smem(row_bytes, NSETS, nw) + 127) / 128 * 128;
    if (gb > SMEM_CAP || gemv_mma_xstages((int)K, row_bytes) > NSETS - 1) return false;
    int groups = MAX_WARPS / nw;
    while (groups > 1 && groups * gb > SMEM_CAP) --groups;
    const int per_sm = groups;                                     // groups an SM holds
    if (ctx->gemv_mma_groups == 1) groups = 1;                     // ... as blocks of one group each
    const int64_t n_units = (M + GEMV_MMA_ROWS - 1) / GEMV_MMA_ROWS;
    // few rows: rather more blocks than full ones
    while (groups > 1 && n_units < (int64_t)groups * ctx->sm_count) --groups;
    const size_t smem = groups * gb;
    const int threads = groups * nw * 32;
    auto kern = gemv_mma_kernel<TYPE, NSETS, SLICE>;
    static bool attr_dev[B200Q_MAX_DEVICES] = {};
    bool &attr = attr_dev[ctx->device % B200Q_MAX_DEVICES];
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_CAP);
        if (e != cudaSuccess) { *st = fail(ctx, B200Q_CUDA_ERROR, "gemv_mma attribute: %s", cudaGetErrorString(e)); return true; }
        attr = true;
    }
    int64_t blocks = (n_units + groups - 1) / groups;
    const int64_t cap = (int64_t)ctx->sm_count * (per_sm / groups);
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaError_t e = launch_pdl(!ctx->no_pdl, kern, dim3((unsigned)blocks), dim3(threads), smem, ctx->stream, (const uint8_t *)w, row_stride,
                               (int)M, nblk, act, ncols, dst, (int)ldd, groups, ctx->error_word);
    if (e == cudaSuccess) e = cudaGetLastError();
    *st = e == cudaSuccess ? B200Q_OK : fail(ctx, B200Q_CUDA_ERROR, "gemv_mma launch: %s", cudaGetErrorString(e));
    return true;
}

// Which kernel takes a dense, aligned product of NC columns (measured on B200, CUDA-graph replay over
// rotating weight copies): the slice-resident kernel everywhere except the 210-byte Q6_K blocks at one
// column, where the per-warp ring kernel is 10 % faster (23.1 against 25.9 us on the 32000x4096 head). With four
// rows per ring stage it also wins at two columns (Q4_K 4096x11008: 8.9 against 10.8 us).
template <int TYPE, int NC>
static bool stream_preferred() {
    if (NC == 1 && TYPE == B200Q_TYPE_Q6_K) return false;
    return true;
}

template <int TYPE, int NC>
static b200q_status launch_nc(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K,
                              const GemvAct &act, float *dst, int64_t ldd, bool aligned) {
    // rows per warp batch: four; eight for three or four columns of a small-block type, where
    // the activation registers are worth sharing further (measured on B200)
    constexpr bool wide = (NC == 3 || NC == 4) && GemvStage<TYPE>::BYTES <= 1152;
    const bool want_stream = ctx->gemv_stream_mask >= 0 ? ((ctx->gemv_stream_mask >> NC) & 1) != 0 : stream_preferred<TYPE, NC>();
    if constexpr (TYPE == B200Q_TYPE_Q4_K || TYPE == B200Q_TYPE_Q5_K || TYPE == B200Q_TYPE_Q6_K || TYPE == B200Q_TYPE_IQ4_XS ||
                  TYPE == B200Q_TYPE_Q4_0 || TYPE == B200Q_TYPE_IQ4_NL || TYPE == B200Q_TYPE_Q8_0) {
        // from how many columns the warp-MMA kernel wins (measured): Q6_K 3, Q8_0 7, the others 4
        if (aligned && !ctx->no_stream && M <= INT32_MAX / 2 && ldd <= INT32_MAX &&
            NC >= (ctx->gemv_mma_min ? ctx->gemv_mma_min : (TYPE == B200Q_TYPE_Q6_K ? 3 : TYPE == B200Q_TYPE_Q8_0 ? 7 : 4))) {
            b200q_status st = B200Q_OK;
            // the narrowest slice per warp that covers a row with sixteen warps (twelve at four super-blocks)
            const int nblk = (int)(K / 256);
            int slice = nblk <= 32 ? 2 : nblk <= 48 ? 3 : 4;
            if (ctx->gemv_mma_slice >= 2 && ctx->gemv_mma_slice <= 4) slice = ctx->gemv_mma_slice;
            if (TYPE == B200Q_TYPE_Q6_K && slice == 3) slice = 4;      // Q6_K: even slices only
            const bool four = !ctx->gemv_mma_sets3;
            bool took = false;
            if (slice == 2) took = (four && try_launch_mma<TYPE, 4, 2>(ctx, w, row_stride, M, K, act, NC, dst, ldd, &st)) ||
                                   try_launch_mma<TYPE, 3, 2>(ctx, w, row_stride, M, K, act, NC, dst, ldd, &st);
            else if (slice == 3) {
                if constexpr (TYPE != B200Q_TYPE_Q6_K)
                    took = (four && try_launch_mma<TYPE, 4, 3>(ctx, w, row_stride, M, K, act, NC, dst, ldd, &st)) ||
                           try_launch_mma<TYPE, 3, 3>(ctx, w, row_stride, M, K, act, NC, dst, ldd, &st);
            }
            else took = (four && try_launch_mma<TYPE, 4, 4>(ctx, w, row_stride, M, K, act, NC, dst, ldd, &st)) ||
                        try_launch_mma<TYPE, 3, 4>(ctx, w, row_stride, M, K, act, NC, dst, ldd, &st);
            if (took) {
                if (st == B200Q_OK) count(ctx, ST_GEMV_MMA);
                return st;
            }
        }
    }
    if (aligned && !ctx->no_stream && M <= INT32_MAX / 2 && ldd <= INT32_MAX && want_stream) {
        typedef GemvFmt<TYPE> F;
        const int row_bytes = (int)(K / F::BLK_W) * F::BLK_B;
        // rows per ring stage: four; two at a single column unless the rows are long (measured: Q4_K 11008x4096 at one
        // column 7.4 us with two and 7.6 with four, 4096x11008 7.55 with two and 7.1 with four; at 4 and 8 columns four rows
        // win everywhere, by up to 25 % on the long rows), and two when a ring of four rows does not fit shared memory
        bool two = NC == 1 && row_bytes <= 4096;
        if (ctx->gemv_rows == 2 || ctx->gemv_rows == 4) two = ctx->gemv_rows == 2;
        else if (ctx->gemv_rows) count(ctx, ST_GEMV_KNOB_IGNORED);
        b200q_status st = B200Q_OK;
        bool took = !two && try_launch_stream<TYPE, NC, 4>(ctx, w, row_stride, M, K, act, dst, ldd, &st);
        if (!took) took = try_launch_stream<TYPE, NC, 2>(ctx, w, row_stride, M, K, act, dst, ldd, &st);
        if (took) {
            if (st == B200Q_OK) count(ctx, ST_GEMV_STREAM);
            return st;
        }
    }
    GemvId none = {};
    return launch_one<TYPE, NC, wide ? 8 : 4, 4, 2, false>(ctx, w, row_stride, M, K, act, dst, ldd, aligned, none, 0);
}

template <int TYPE>
static b200q_status launch_type(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K,
                                const GemvAct &act, int nc, float *dst, int64_t ldd, bool aligned) {
    switch (nc) {
    case 1: return launch_nc<TYPE, 1>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 2: return launch_nc<TYPE, 2>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 3: return launch_nc<TYPE, 3>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 4: return launch_nc<TYPE, 4>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 5: return launch_nc<TYPE, 5>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 6: return launch_nc<TYPE, 6>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 7: return launch_nc<TYPE, 7>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 8: return launch_nc<TYPE, 8>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    }
    return fail(ctx, B200Q_INVALID, "gemv: %d columns", nc);
}

// MUL_MAT_ID over route tiles of at most nc pairs (nc = 1, 2, 4 or 8)
template <int TYPE>
static b200q_status launch_id_type(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K,
                                   const GemvAct &act, int nc, float *dst, bool aligned, const GemvId &id,
                                   int64_t max_tiles) {
    switch (nc) {
    case 1: return launch_one<TYPE, 1, 4, 4, 2, true>(ctx, w, row_stride, M, K, act, dst, 0, aligned, id, max_tiles);
    case 2: return launch_one<TYPE, 2, 4, 4, 2, true>(ctx, w, row_stride, M, K, act, dst, 0, aligned, id, max_tiles);
    case 4: return launch_one<TYPE, 4, 4, 4, 2, true>(ctx, w, row_stride, M, K, act, dst, 0, aligned, id, max_tiles);
    case 8: return launch_one<TYPE, 8, 4, 4, 2, true>(ctx, w, row_stride, M, K, act, dst, 0, aligned, id, max_tiles);
    }
    return fail(ctx, B200Q_INVALID, "gemv_id: tile of %d pairs", nc);
}

static GemvAct make_act(const ActView &av, int64_t col0, int64_t K) {
    GemvAct act;
    act.q = av.codes + col0 * K;
    act.d16 = av.d16 ? av.d16 + col0 * (K / 32) : nullptr;
    act.d32 = av.d32 ? av.d32 + col0 * (K / 256) : nullptr;
    act.s32 = av.s32 ? av.s32 + col0 * (K / 32) : nullptr;
    act.s16 = av.s16 ? av.s16 + col0 * (K / 16) : nullptr;
    act.K = (int)K;
    return act;
}

b200q_status launch_gemv_id(b200q_ctx *ctx, int type, const void *w, size_t row_stride, size_t expert_stride,
                            int64_t M, int64_t K, const ActView &av, int tile_pairs, const int32_t *tiles,
                            const int32_t *n_tiles, int64_t max_tiles, const int32_t *pairs, const b200q_tensor *ids,
                            int n_expert, int n_used, int ne11, float *dst, int64_t ld1, int64_t ld2) {
    TypeInfo ti;
    if (!type_info(type, &ti)) return fail(ctx, B200Q_UNSUPPORTED, "gemv_id: type %d", type);
    const size_t row_bytes = (size_t)(K / ti.block) * ti.bytes;
    const bool aligned = ((uintptr_t)w % 16 == 0) && (row_stride % 16 == 0) && (row_bytes % 16 == 0) &&
                         (expert_stride % 16 == 0);
    GemvId id;
    id.tiles = tiles;
    id.n_tiles = n_tiles;
    id.pairs = pairs;
    id.ids = (const uint8_t *)ids->data;
    id.ids_stride = ids->nb[1];
    id.n_pairs = (int)(ids->ne[0] * ids->ne[1]);
    id.n_expert = n_expert;
    id.n_used = n_used;
    id.ne11 = ne11;
    id.expert_stride = expert_stride;
    id.ld1 = ld1;
    id.ld2 = ld2;
    const GemvAct act = make_act(av, 0, K);
    count(ctx, aligned ? ST_GEMV_ID : ST_GEMV_ID_UNALIGNED);
    switch (type) {
    case B200Q_TYPE_Q4_0:   return launch_id_type<B200Q_TYPE_Q4_0>(ctx, w, row_stride, M, K, act, tile_pairs, dst, aligned, id, max_tiles);
    case B200Q_TYPE_Q8_0:   return launch_id_type<B200Q_TYPE_Q8_0>(ctx, w, row_stride, M, K, act, tile_pairs, dst, aligned, id, max_tiles);
    case B200Q_TYPE_Q4_K:   return launch_id_type<B200Q_TYPE_Q4_K>(ctx, w, row_stride, M, K, act, tile_pairs, dst, aligned, id, max_tiles);
    case B200Q_TYPE_Q5_K:   return launch_id_type<B200Q_TYPE_Q5_K>(ctx, w, row_stride, M, K, act, tile_pairs, dst, aligned, id, max_tiles);
    case B200Q_TYPE_Q6_K:   return launch_id_type<B200Q_TYPE_Q6_K>(ctx, w, row_stride, M, K, act, tile_pairs, dst, aligned, id, max_tiles);
    case B200Q_TYPE_IQ4_XS: return launch_id_type<B200Q_TYPE_IQ4_XS>(ctx, w, row_stride, M, K, act, tile_pairs, dst, aligned, id, max_tiles);
    case B200Q_TYPE_IQ4_NL: return launch_id_type<B200Q_TYPE_IQ4_NL>(ctx, w, row_stride, M, K, act, tile_pairs, dst, aligned, id, max_tiles);
    }
    return fail(ctx, B200Q_UNSUPPORTED, "gemv_id: type %d", type);
}

static GemvAct make_act(const ActView &av, int64_t col0, int64_t K);

// One or two columns of a small per-32 product with the activation quantized inside the GEMV (no quantizer launch):
// B200Q_UNSUPPORTED when the shape does not qualify and the caller should take the two-kernel route.
template <int TYPE>
static b200q_status launch_fused_t(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K, const GemvAct &act, int nc,
                                   float *dst, int64_t ldd) {
    b200q_status st = B200Q_OK;
    bool took = false;
    if (nc == 1) took = try_launch_stream<TYPE, 1, 2, true>(ctx, w, row_stride, M, K, act, dst, ldd, &st);
    else if (nc == 2) took = try_launch_stream<TYPE, 2, 4, true>(ctx, w, row_stride, M, K, act, dst, ldd, &st);
    if (!took) return B200Q_UNSUPPORTED;
    if (st == B200Q_OK) { count(ctx, ST_GEMV_STREAM); count(ctx, ST_GEMV_FUSED_QUANT); count(ctx, ST_GEMV_COL0 + nc); }
    return st;
}

b200q_status launch_gemv_fused(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                               const b200q_tensor *src1, int ncols, float *dst, int64_t ldd) {
    if (type != B200Q_TYPE_Q4_0 && type != B200Q_TYPE_Q8_0) return B200Q_UNSUPPORTED;
    if (ncols < 1 || ncols > 2 || ctx->no_stream || ctx->fuse_quant_bytes <= 0) return B200Q_UNSUPPORTED;
    TypeInfo ti;
    type_info(type, &ti);
    const size_t row_bytes = (size_t)(K / ti.block) * ti.bytes;
    if ((uintptr_t)w % 16 || row_stride % 16 || row_bytes % 16) return B200Q_UNSUPPORTED;
    if ((int64_t)(row_bytes * (size_t)M) > ctx->fuse_quant_bytes || M > INT32_MAX / 2 || ldd > INT32_MAX) return B200Q_UNSUPPORTED;
    // the activation as plain columns of f32
    if (src1->ne[2] != 1 || src1->ne[3] != 1 || src1->nb[0] != 4 || src1->nb[1] % 16 || (uintptr_t)src1->data % 16) return B200Q_UNSUPPORTED;
    GemvAct act = {};
    act.K = (int)K;
    act.xf = (const float *)src1->data;
    act.xf_stride = (int64_t)(src1->nb[1] / 4);
    return type == B200Q_TYPE_Q4_0 ? launch_fused_t<B200Q_TYPE_Q4_0>(ctx, w, row_stride, M, K, act, ncols, dst, ldd)
                                   : launch_fused_t<B200Q_TYPE_Q8_0>(ctx, w, row_stride, M, K, act, ncols, dst, ldd);
}

// Product + all-reduce in one kernel (row split over several GPUs): 1, 2, 4 or 8 columns of a shape the slice-resident
// kernel takes, NC * M results within the all-reduce buffer. src1 != NULL: quantize inside the kernel (per-32 types,
// 1-2 columns). B200Q_UNSUPPORTED: not that case.
template <int TYPE, int NC, bool QX>
static b200q_status launch_ar_t(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K, const GemvAct &act, float *dst,
                                int64_t ldd, const GemvAr &ar) {
    typedef GemvFmt<TYPE> F;
    const int row_bytes = (int)(K / F::BLK_W) * F::BLK_B;
    const bool two = NC == 1 && row_bytes <= 4096;              // as in launch_nc
    b200q_status st = B200Q_OK;
    bool took = !two && try_launch_stream<TYPE, NC, 4, QX, true>(ctx, w, row_stride, M, K, act, dst, ldd, &st, &ar);
    if (!took) took = try_launch_stream<TYPE, NC, 2, QX, true>(ctx, w, row_stride, M, K, act, dst, ldd, &st, &ar);
    if (!took) return B200Q_UNSUPPORTED;
    if (st == B200Q_OK) { count(ctx, ST_GEMV_STREAM); count(ctx, ST_GEMV_ALLREDUCE_FUSED); count(ctx, ST_GEMV_COL0 + NC); if (QX) count(ctx, ST_GEMV_FUSED_QUANT); }
    return st;
}

template <int TYPE>
static b200q_status launch_ar_type(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K, const GemvAct &act, int nc,
                                   bool qx, float *dst, int64_t ldd, const GemvAr &ar) {
    constexpr bool per32 = TYPE == B200Q_TYPE_Q4_0 || TYPE == B200Q_TYPE_Q8_0;
    if constexpr (per32) {
        if (qx && nc == 1) return launch_ar_t<TYPE, 1, true>(ctx, w, row_stride, M, K, act, dst, ldd, ar);
        if (qx && nc == 2) return launch_ar_t<TYPE, 2, true>(ctx, w, row_stride, M, K, act, dst, ldd, ar);
    }
    if (qx) return B200Q_UNSUPPORTED;
    switch (nc) {
    case 1: return launch_ar_t<TYPE, 1, false>(ctx, w, row_stride, M, K, act, dst, ldd, ar);
    case 2: return launch_ar_t<TYPE, 2, false>(ctx, w, row_stride, M, K, act, dst, ldd, ar);
    case 4: return launch_ar_t<TYPE, 4, false>(ctx, w, row_stride, M, K, act, dst, ldd, ar);
    case 8: return launch_ar_t<TYPE, 8, false>(ctx, w, row_stride, M, K, act, dst, ldd, ar);
    }
    return B200Q_UNSUPPORTED;
}

bool gemv_ar_shape_ok(int type, const void *w, size_t row_stride, int64_t M, int64_t K, int ncols, int64_t ldd) {
    TypeInfo ti;
    if (!type_info(type, &ti)) return false;
    const size_t row_bytes = (size_t)(K / ti.block) * ti.bytes;
    if ((uintptr_t)w % 16 || row_stride % 16 || row_bytes % 16) return false;
    if (ncols != 1 && ncols != 2 && ncols != 4 && ncols != 8) return false;
    return (int64_t)ncols * M <= PEER_AR_MAX_FLOATS && M <= INT32_MAX / 2 && ldd <= INT32_MAX;
}

b200q_status launch_gemv_allreduce(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K, const ActView *av,
                                   const b200q_tensor *src1, int ncols, float *dst, int64_t ldd, uint64_t *const *peers, uint32_t *state,
                                   int rank, int nranks) {
    if (ctx->no_stream || !gemv_ar_shape_ok(type, w, row_stride, M, K, ncols, ldd)) return B200Q_UNSUPPORTED;
    GemvAr ar = {};
    for (int p = 0; p < nranks && p < PEER_AR_MAX_RANKS; ++p) ar.peer[p] = peers[p];
    ar.state = state;
    ar.rank = rank;
    ar.nranks = nranks;
    GemvAct act = {};
    bool qx = false;
    if (av) {
        act = make_act(*av, 0, K);
    } else {
        if (!src1 || src1->ne[2] != 1 || src1->ne[3] != 1 || src1->nb[0] != 4 || src1->nb[1] % 16 || (uintptr_t)src1->data % 16) return B200Q_UNSUPPORTED;
        act.K = (int)K;
        act.xf = (const float *)src1->data;
        act.xf_stride = (int64_t)(src1->nb[1] / 4);
        qx = true;
    }
    switch (type) {
    case B200Q_TYPE_Q4_0:   return launch_ar_type<B200Q_TYPE_Q4_0>(ctx, w, row_stride, M, K, act, ncols, qx, dst, ldd, ar);
    case B200Q_TYPE_Q8_0:   return launch_ar_type<B200Q_TYPE_Q8_0>(ctx, w, row_stride, M, K, act, ncols, qx, dst, ldd, ar);
    case B200Q_TYPE_Q4_K:   return launch_ar_type<B200Q_TYPE_Q4_K>(ctx, w, row_stride, M, K, act, ncols, qx, dst, ldd, ar);
    case B200Q_TYPE_Q6_K:   return launch_ar_type<B200Q_TYPE_Q6_K>(ctx, w, row_stride, M, K, act, ncols, qx, dst, ldd, ar);
    case B200Q_TYPE_IQ4_XS: return launch_ar_type<B200Q_TYPE_IQ4_XS>(ctx, w, row_stride, M, K, act, ncols, qx, dst, ldd, ar);
    }
    return B200Q_UNSUPPORTED;                 // other types (Q5_K): the caller runs the product and the all-reduce one after the other
}

b200q_status launch_gemv(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                         const ActView &av, int64_t col0, int ncols, float *dst, int64_t ldd) {
    const GemvAct act = make_act(av, col0, K);
    TypeInfo ti;
    if (!type_info(type, &ti)) return fail(ctx, B200Q_UNSUPPORTED, "gemv: type %d", type);
    const size_t row_bytes = (size_t)(K / ti.block) * ti.bytes;
    const bool aligned = ((uintptr_t)w % 16 == 0) && (row_stride % 16 == 0) && (row_bytes % 16 == 0);
    count(ctx, (aligned ? ST_GEMV_COL0 : ST_GEMV_UNALIGNED_COL0) + ncols);
    switch (type) {
    case B200Q_TYPE_Q4_0:   return launch_type<B200Q_TYPE_Q4_0>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_Q8_0:   return launch_type<B200Q_TYPE_Q8_0>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_Q4_K:   return launch_type<B200Q_TYPE_Q4_K>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_Q5_K:   return launch_type<B200Q_TYPE_Q5_K>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_Q6_K:   return launch_type<B200Q_TYPE_Q6_K>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_IQ4_XS: return launch_type<B200Q_TYPE_IQ4_XS>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_IQ4_NL: return launch_type<B200Q_TYPE_IQ4_NL>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    }
    return fail(ctx, B200Q_UNSUPPORTED, "gemv: type %d", type);
}

}  // namespace b200q
