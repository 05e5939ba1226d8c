// api.cu -- the C ABI: context, scratch, shape gates and dispatch of MUL_MAT.
//
// Host side of the path, the counterpart of the reference's dispatch in ggml-opencl.cpp
// (marfrit/arcint contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch):
// ggml_cl_kq_type_index / ggml_cl_kq_mul_mat_shape (:781-812), the per-graph activation
// conversion cache (:670-715), ggml_cl_mul_mat (:1135-1158) and supports_op (:615-652).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace b200q {

// A wait that cannot succeed, for the failure-path test: one thread polls a shared-memory mbarrier that
// nobody ever arrives at, at most `polls` times, then does what every kernel of the library does when a
// bounded wait runs out -- it records the fact in the context's error word and returns. No trap, no
// fault, no unbounded loop: the context stays usable.
__global__ void debug_wait_timeout_kernel(unsigned polls, int *error_word) {
    __shared__ __align__(8) uint64_t bar;
    const uint32_t b = tc::smem_u32(&bar);
    tc::mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    bool done = false;
    for (unsigned i = 0; i < polls && !done; ++i) done = tc::mbar_try(b, 0);
    if (!done) atomicExch(error_word, 3);
}

const char *stat_name(int s) {
    static const char *fixed[] = { "quantize_act_q8_0", "quantize_act_q8_256", "act_cache_hit", "workspace_grow",
                                   "mul_mat_gemv_chunks" };
    static char cols[18][32];
    if (s < ST_GEMV_COL0) return fixed[s];
    if (s < ST_GEMV_ID) {
        const bool un = s >= ST_GEMV_UNALIGNED_COL0;
        const int n = s - (un ? ST_GEMV_UNALIGNED_COL0 : ST_GEMV_COL0);
        char *b = cols[(un ? 9 : 0) + n];
        snprintf(b, 32, "gemv_%s%dcol", un ? "unaligned_" : "", n);
        return b;
    }
    static const char *rest[] = { "gemv_id", "gemv_id_unaligned", "moe_route", "route_cache_hit", "moe_gemm", "moe_pack",
                                  "gemm_tc", "gemm_tc_quantize", "gemm_fallback_shape", "tp_allreduce", "tp_allgather",
                                  "ep_dispatch", "ep_combine", "graph_launch", "no_alloc", "gemm_kq_mins", "gemv_stream", "tp_allreduce_peer", "gemm_tc_f16", "ep_peer", "ep_dispatch_cached", "moe_router", "moe_ffn", "gemv_knob_ignored", "gemm_ksplit", "gemv_fused_quant", "gemv_allreduce_fused",
                                  "ep_agreed_exit", "gemm_kq_rowcopy", "gemv_mma" };
    return rest[s - ST_GEMV_ID];
}

b200q_status fail(b200q_ctx *ctx, b200q_status st, const char *fmt, ...) {
    if (ctx) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof(buf), fmt, ap);
        va_end(ap);
        ctx->last_error = buf;
    }
    return st;
}

// grow-only scratch (the reference's prealloc_* buffers never shrink either)
b200q_status ws_reserve(b200q_ctx *ctx, Workspace *ws, size_t bytes) {
    if (bytes <= ws->cap) return B200Q_OK;
    if (ctx->capturing)
        return fail(ctx, B200Q_INVALID, "scratch would grow inside a capture: run the sequence once before capturing");
    if (ws->ptr) {
        // the old block may still be in use by work already enqueued on the stream
        B200Q_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        B200Q_CUDA(ctx, cudaFree(ws->base));
        ws->ptr = ws->base = nullptr;
        ws->cap = 0;
    }
    // Normally whole megabytes, so that a slowly growing request does not reallocate every time. With guard words the block
    // has the size asked for (to 256 bytes), so that a write past the request lands in the guard and not in rounding slack.
    const size_t guard = ctx->canary ? WS_GUARD : 0;
    const size_t unit = ctx->canary ? 256 : (size_t)1 << 20;
    const size_t want = (bytes + unit - 1) / unit * unit;
    // (behind the tail guard another 64 KiB, so that a read past the block -- which no guard can see -- stays inside the allocation)
    const size_t total = want + 2 * guard + (guard ? (size_t)64 << 10 : 0);
    cudaError_t e = cudaMalloc(&ws->base, total);
    if (e != cudaSuccess) {
        ws->base = nullptr;
        return fail(ctx, B200Q_NO_MEMORY, "cudaMalloc(%zu): %s", total, cudaGetErrorString(e));
    }
    ws->ptr = (uint8_t *)ws->base + guard;
    ws->cap = want;
    if (guard) {
        B200Q_CUDA(ctx, cudaMemsetAsync(ws->base, WS_GUARD_BYTE, guard, ctx->stream));
        B200Q_CUDA(ctx, cudaMemsetAsync((uint8_t *)ws->ptr + want, WS_GUARD_BYTE, guard, ctx->stream));
    }
    count(ctx, ST_WORKSPACE_GROW);
    return B200Q_OK;
}

void ws_release(Workspace *ws) {
    if (ws->base) cudaFree(ws->base);
    ws->ptr = ws->base = nullptr;
    ws->cap = 0;
}

static bool is_contiguous_f32(const b200q_tensor *t) {
    return t->type == B200Q_TYPE_F32 && t->nb[0] == sizeof(float);
}

// The gate of ggml_cl_kq_mul_mat_shape plus what the kernels' loads need.
static b200q_status check_mul_mat(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1,
                                  const b200q_tensor *dst, bool id_form) {
    if (!src0 || !src1 || !dst) return fail(ctx, B200Q_INVALID, "null tensor");
    TypeInfo ti;
    if (!type_info(src0->type, &ti)) return fail(ctx, B200Q_UNSUPPORTED, "weight type %d", src0->type);
    const int64_t K = src0->ne[0], M = src0->ne[1];
    if (K <= 0 || K % ti.block) return fail(ctx, B200Q_UNSUPPORTED, "K=%lld not a multiple of %d", (long long)K, ti.block);
    const size_t row_bytes = (size_t)(K / ti.block) * ti.bytes;
    if (src0->nb[0] != (size_t)ti.bytes) return fail(ctx, B200Q_UNSUPPORTED, "weight nb[0]=%zu", src0->nb[0]);
    if (src0->nb[1] < row_bytes || src0->nb[1] % 2) return fail(ctx, B200Q_UNSUPPORTED, "weight row stride %zu", src0->nb[1]);
    if (!id_form && (src0->ne[2] != 1 || src0->ne[3] != 1))
        return fail(ctx, B200Q_UNSUPPORTED, "3-D weights for MUL_MAT");
    if (src0->ne[3] != 1) return fail(ctx, B200Q_UNSUPPORTED, "4-D weights");
    if ((uintptr_t)src0->data % 2) return fail(ctx, B200Q_UNSUPPORTED, "weight address not 2-byte aligned");
    if (!is_contiguous_f32(src1)) return fail(ctx, B200Q_UNSUPPORTED, "src1 must be f32 with unit element stride");
    if (!is_contiguous_f32(dst)) return fail(ctx, B200Q_UNSUPPORTED, "dst must be f32 with unit element stride");
    if (src1->ne[0] != K) return fail(ctx, B200Q_INVALID, "src1 ne[0]=%lld, K=%lld", (long long)src1->ne[0], (long long)K);
    if (dst->ne[0] != M) return fail(ctx, B200Q_INVALID, "dst ne[0]=%lld, M=%lld", (long long)dst->ne[0], (long long)M);
    if ((uintptr_t)src1->data % 16 || src1->nb[1] % 16 || src1->nb[2] % 16 || src1->nb[3] % 16)
        return fail(ctx, B200Q_UNSUPPORTED, "src1 columns must be 16-byte aligned");
    if ((uintptr_t)dst->data % 4 || dst->nb[1] % 4 || dst->nb[2] % 4 || dst->nb[3] % 4)
        return fail(ctx, B200Q_UNSUPPORTED, "dst columns must be 4-byte aligned");
    if (!src0->data || !src1->data || !dst->data) {
        const bool empty = M == 0 || src1->ne[1] * src1->ne[2] * src1->ne[3] == 0;
        if (!empty) return fail(ctx, B200Q_INVALID, "null data pointer");
    }
    return B200Q_OK;
}

// MUL_MAT_ID shapes: src0 [K, M, n_expert], src1 [K, ne11 in {1, n_used}, n_tok], ids [n_used, n_tok] i32,
// dst [M, n_used, n_tok] (P01:1174-1219; the column rule kq_i8_col, P09:573-577)
static b200q_status check_ids(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1,
                              const b200q_tensor *ids, const b200q_tensor *dst) {
    if (!ids) return fail(ctx, B200Q_INVALID, "null ids");
    if (ids->type != B200Q_TYPE_I32 || ids->nb[0] != sizeof(int32_t)) return fail(ctx, B200Q_UNSUPPORTED, "ids must be packed i32");
    if (ids->ne[2] != 1 || ids->ne[3] != 1 || src1->ne[3] != 1 || dst->ne[3] != 1) return fail(ctx, B200Q_UNSUPPORTED, "4-D MUL_MAT_ID");
    const int64_t n_used = ids->ne[0], n_tok = ids->ne[1];
    if (src1->ne[2] != n_tok || (src1->ne[1] != 1 && src1->ne[1] != n_used))
        return fail(ctx, B200Q_INVALID, "src1 [K, %lld, %lld] against ids [%lld, %lld]", (long long)src1->ne[1],
                    (long long)src1->ne[2], (long long)n_used, (long long)n_tok);
    if (dst->ne[1] != n_used || dst->ne[2] != n_tok) return fail(ctx, B200Q_INVALID, "dst shape against ids");
    if (ids->nb[1] % 4 || (uintptr_t)ids->data % 4) return fail(ctx, B200Q_UNSUPPORTED, "ids rows must be 4-byte aligned");
    if (src0->ne[2] < 1 || src0->ne[2] > 4096) return fail(ctx, B200Q_UNSUPPORTED, "%lld experts", (long long)src0->ne[2]);
    if (src0->ne[2] > 1 && src0->nb[2] % 2) return fail(ctx, B200Q_UNSUPPORTED, "expert stride %zu", src0->nb[2]);
    if (n_used * n_tok > (1 << 28)) return fail(ctx, B200Q_UNSUPPORTED, "too many pairs");
    if (!ids->data && n_used * n_tok) return fail(ctx, B200Q_INVALID, "null ids data");
    return B200Q_OK;
}

// Quantize src1 once per graph: q/k/v and gate/up share their input (P01:670-688).
static b200q_status get_activation(b200q_ctx *ctx, int form, const b200q_tensor *src1, ActView *out) {
    ActKey key;
    key.data = src1->data;
    key.id = src1->id;
    key.form = form;
    key.gen = ctx->generation;
    for (int i = 0; i < 4; ++i) { key.ne[i] = src1->ne[i]; key.nb[i] = src1->nb[i]; }
    ActEntry *hit = nullptr;
    for (auto &e : ctx->act_cache)
        if (e.valid && e.key == key) { hit = &e; break; }
    const int64_t K = src1->ne[0], N = src1->ne[1] * src1->ne[2] * src1->ne[3];
    if (!hit) {
        if (ctx->act_cache.size() < 4) ctx->act_cache.resize(4);
        // victim: an entry of an older graph (its contents are dead), the first one if several,
        // so a steady sequence of graphs keeps landing in the same, already sized, buffers;
        // only when all four belong to this graph do they rotate
        size_t pick = ctx->act_cache.size();
        for (size_t i = 0; i < ctx->act_cache.size(); ++i)
            if (!ctx->act_cache[i].valid || ctx->act_cache[i].key.gen != ctx->generation) { pick = i; break; }
        if (pick == ctx->act_cache.size()) {
            pick = ctx->act_next;
            ctx->act_next = (ctx->act_next + 1) % ctx->act_cache.size();
        }
        ActEntry &e = ctx->act_cache[pick];
        e.valid = false;
        b200q_status st;
        if (form == ACT_Q8_0_TILED || form == ACT_Q8_256_TILED) {
            const bool per32 = form == ACT_Q8_0_TILED;
            if ((st = ws_reserve(ctx, &e.codes, per32 ? gemm_tc_act_bytes(K, N) : gemm_kq_act_bytes(K, N))) != B200Q_OK) return st;
            st = per32 ? launch_quantize_tiled(ctx, src1, (uint8_t *)e.codes.ptr)
                       : launch_quantize_tiled256(ctx, src1, (uint8_t *)e.codes.ptr);
            if (st != B200Q_OK) return st;
            e.key = key;
            e.valid = true;
            out->codes = (const int8_t *)e.codes.ptr;
            out->form = form;
            out->K = K;
            out->N = N;
            return B200Q_OK;
        }
        if ((st = ws_reserve(ctx, &e.codes, (size_t)(N * K) + 64)) != B200Q_OK) return st;
        const size_t sbytes = form == ACT_Q8_0 ? sizeof(uint16_t) * (size_t)(N * (K / 32)) : sizeof(float) * (size_t)(N * (K / 256));
        if ((st = ws_reserve(ctx, &e.scales, sbytes + 64)) != B200Q_OK) return st;
        if ((st = ws_reserve(ctx, &e.sums, sizeof(int16_t) * (size_t)(N * (K / 32)) + 64)) != B200Q_OK) return st;
        if (form == ACT_Q8_256 && (st = ws_reserve(ctx, &e.sums16, sizeof(int16_t) * (size_t)(N * (K / 16)) + 64)) != B200Q_OK)
            return st;
        if ((st = launch_quantize_act(ctx, form, src1, (int8_t *)e.codes.ptr, e.scales.ptr, (int16_t *)e.sums.ptr,
                                      (int16_t *)e.sums16.ptr)) != B200Q_OK)
            return st;
        e.key = key;
        e.valid = true;
        hit = &e;
    } else {
        count(ctx, ST_ACT_CACHE_HIT);
    }
    out->codes = (const int8_t *)hit->codes.ptr;
    out->d16 = form == ACT_Q8_0 ? (const uint16_t *)hit->scales.ptr : nullptr;
    out->d32 = form == ACT_Q8_256 ? (const float *)hit->scales.ptr : nullptr;
    out->s32 = (const int16_t *)hit->sums.ptr;
    out->s16 = form == ACT_Q8_256 ? (const int16_t *)hit->sums16.ptr : nullptr;
    out->form = form;
    out->K = K;
    out->N = N;
    return B200Q_OK;
}

b200q_status get_decode_activation(b200q_ctx *ctx, int weight_type, const b200q_tensor *src1, ActView *out) {
    TypeInfo ti;
    if (!type_info(weight_type, &ti)) return fail(ctx, B200Q_UNSUPPORTED, "weight type %d", weight_type);
    return get_activation(ctx, ti.act_form, src1, out);
}

// dst column c (flattened like src1) -> element offset; the kernels take a single column
// stride, so a dst whose flattened columns are not evenly spaced is walked in runs
static bool dst_uniform(const b200q_tensor *dst, int64_t *ldd) {
    const size_t s1 = dst->nb[1];
    const bool ok2 = dst->ne[2] == 1 || dst->nb[2] == s1 * (size_t)dst->ne[1];
    const bool ok3 = dst->ne[3] == 1 || dst->nb[3] == s1 * (size_t)dst->ne[1] * (size_t)dst->ne[2];
    *ldd = (int64_t)(s1 / sizeof(float));
    return ok2 && ok3;
}

}  // namespace b200q

using namespace b200q;

extern "C" {

const char *b200q_version(void) { return "b200q 0.1 (sm_100a)"; }

b200q_status b200q_init(b200q_ctx **out, int device, void *stream) {
    if (!out) return B200Q_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return B200Q_CUDA_ERROR;
    if (cudaSetDevice(device) != cudaSuccess) return B200Q_CUDA_ERROR;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return B200Q_CUDA_ERROR;
    if (prop.major != 10) return B200Q_UNSUPPORTED;            // sm_100a kernels only
    b200q_ctx *ctx = new b200q_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return B200Q_CUDA_ERROR;
        }
        ctx->own_stream = true;
    }
    if (cudaEventCreate(&ctx->ev0) != cudaSuccess || cudaEventCreate(&ctx->ev1) != cudaSuccess ||
        cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ctx->ev_join, cudaEventDisableTiming) != cudaSuccess) {
        b200q_free(ctx);
        return B200Q_CUDA_ERROR;
    }
    if (cudaMalloc(&ctx->error_word, sizeof(int)) != cudaSuccess || cudaMemset(ctx->error_word, 0, sizeof(int)) != cudaSuccess) {
        b200q_free(ctx);
        return B200Q_NO_MEMORY;
    }
    const char *no_tc = getenv("B200Q_NO_TC");      // read once: force the CUDA-core path (tests, comparisons)
    ctx->no_tc = no_tc && no_tc[0] == '1';
    const char *no_pdl = getenv("B200Q_NO_PDL");     // plain stream order in the decode chain (comparisons)
    ctx->no_pdl = no_pdl && no_pdl[0] == '1';
    const char *tc_i8 = getenv("B200Q_TC_I8");           // the int8 arm of the per-32 prompt GEMM (comparisons)
    ctx->tc_f16 = !(tc_i8 && tc_i8[0] == '1');
    // tile knobs for the tuner (arcint_b200/tune.py): each is validated where it is used, a value the kernels do
    // not take falls back to the default and is counted as "gemv_knob_ignored"
    if (const char *v = getenv("B200Q_GEMV_ROWS")) ctx->gemv_rows = atoi(v);
    if (const char *v = getenv("B200Q_GEMV_BLOCK_WARPS")) ctx->gemv_block_warps = atoi(v);
    if (const char *v = getenv("B200Q_GEMV_STREAM_MASK")) ctx->gemv_stream_mask = (int)strtol(v, nullptr, 0);
    if (const char *v = getenv("B200Q_FUSE_QUANT_BYTES")) ctx->fuse_quant_bytes = atoll(v);
    const char *no_ks = getenv("B200Q_NO_KSPLIT");
    ctx->no_ksplit = no_ks && no_ks[0] == '1';
    const char *no_small = getenv("B200Q_GEMV_NO_SMALL");
    ctx->gemv_no_small = no_small && no_small[0] == '1';
    const char *mma_min = getenv("B200Q_GEMV_MMA_MIN");  // fewest columns for the warp-MMA GEMV (99: never)
    if (mma_min && mma_min[0]) ctx->gemv_mma_min = atoi(mma_min);
    const char *mma_sets = getenv("B200Q_GEMV_MMA_SETS");
    ctx->gemv_mma_sets3 = mma_sets && mma_sets[0] == '3';
    const char *mma_groups = getenv("B200Q_GEMV_MMA_GROUPS");
    if (mma_groups && mma_groups[0]) ctx->gemv_mma_groups = atoi(mma_groups);
    const char *mma_slice = getenv("B200Q_GEMV_MMA_SLICE");
    if (mma_slice && mma_slice[0]) ctx->gemv_mma_slice = atoi(mma_slice);
    const char *canary = getenv("B200Q_CANARY");         // debugging: guard words around every scratch block
    ctx->canary = canary && canary[0] == '1';
    const char *mins_pass = getenv("B200Q_MOE_MINS_PASS");
    ctx->moe_mins_pass = mins_pass && mins_pass[0] == '1';
    const char *no_stream = getenv("B200Q_NO_STREAM");   // the older GEMV kernel for every shape (comparisons)
    ctx->no_stream = no_stream && no_stream[0] == '1';
    *out = ctx;
    return B200Q_OK;
}

void b200q_free(b200q_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto &e : ctx->act_cache) {
        ws_release(&e.codes);
        ws_release(&e.scales);
        ws_release(&e.sums);
        ws_release(&e.sums16);
    }
    ws_release(&ctx->flush_buf);
    if (ctx->error_word) cudaFree(ctx->error_word);
    for (auto &w : ctx->moe_ws) ws_release(&w);
    moe_free(ctx);
    tp_free(ctx);
    if (ctx->copy_in) { cudaStreamSynchronize(ctx->copy_in); cudaStreamDestroy(ctx->copy_in); }
    if (ctx->copy_out) { cudaStreamSynchronize(ctx->copy_out); cudaStreamDestroy(ctx->copy_out); }
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    if (ctx->ev_join) cudaEventDestroy(ctx->ev_join);
    if (ctx->ev0) cudaEventDestroy(ctx->ev0);
    if (ctx->ev1) cudaEventDestroy(ctx->ev1);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *b200q_last_error(const b200q_ctx *ctx) { return ctx ? ctx->last_error.c_str() : ""; }

b200q_status b200q_get_stream(const b200q_ctx *ctx, void **stream) {
    if (!ctx || !stream) return B200Q_INVALID;
    *stream = (void *)ctx->stream;
    return B200Q_OK;
}

b200q_status b200q_supports(const b200q_ctx *ctx, int op, const b200q_tensor *src0, const b200q_tensor *src1,
                            const b200q_tensor *ids, const b200q_tensor *dst) {
    (void)ctx;
    if (op == B200Q_OP_MUL_MAT) {
        b200q_status st = check_mul_mat(nullptr, src0, src1, dst, false);
        if (st != B200Q_OK) return st;
        if (dst->ne[1] != src1->ne[1] || dst->ne[2] != src1->ne[2] || dst->ne[3] != src1->ne[3]) return B200Q_INVALID;
        return B200Q_OK;
    }
    if (op == B200Q_OP_MUL_MAT_ID) {
        b200q_status st = check_mul_mat(nullptr, src0, src1, dst, true);
        return st != B200Q_OK ? st : check_ids(nullptr, src0, src1, ids, dst);
    }
    return B200Q_UNSUPPORTED;
}

b200q_status b200q_graph_begin(b200q_ctx *ctx) {
    if (!ctx) return B200Q_INVALID;
    ++ctx->generation;
    return B200Q_OK;
}

b200q_status b200q_mul_mat(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1, b200q_tensor *dst) {
    if (!ctx) return B200Q_INVALID;
    b200q_status st = check_mul_mat(ctx, src0, src1, dst, false);
    if (st != B200Q_OK) return st;
    if (dst->ne[1] != src1->ne[1] || dst->ne[2] != src1->ne[2] || dst->ne[3] != src1->ne[3])
        return fail(ctx, B200Q_INVALID, "dst shape does not match src1");
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    TypeInfo ti;
    type_info(src0->type, &ti);
    const int64_t K = src0->ne[0], M = src0->ne[1];
    const int64_t N = src1->ne[1] * src1->ne[2] * src1->ne[3];
    if (M == 0 || N == 0) return B200Q_OK;
    ActView act;
    int64_t ldd;
    const bool uniform = dst_uniform(dst, &ldd);
    // prompt widths of the per-32 types go to the tensor cores
    if (N > 8 && uniform && !ctx->no_tc && gemm_tc_supported(src0->type, M, K, N, src0->data, src0->nb[1])) {
        if ((st = get_activation(ctx, ACT_Q8_0_TILED, src1, &act)) != B200Q_OK) return st;
        return launch_gemm_tc(ctx, src0->type, src0->data, src0->nb[1], M, K, (const uint8_t *)act.codes, N,
                              (float *)dst->data, ldd);
    }
    if (N > 8 && uniform && !ctx->no_tc && gemm_kq_supported(src0->type, M, K, N, src0->data, src0->nb[1])) {
        if ((st = get_activation(ctx, ACT_Q8_256_TILED, src1, &act)) != B200Q_OK) return st;
        return launch_gemm_kq(ctx, src0->type, src0->data, src0->nb[1], M, K, (const uint8_t *)act.codes, N,
                              (float *)dst->data, ldd);
    }
    if (N > 8) count(ctx, ST_GEMM_FALLBACK_SHAPE);
    // small per-32 products at one or two columns: the GEMV quantizes its own slice of the activation, one launch
    // instead of two (what matters once a tensor-parallel shard is a microsecond of weights)
    if (N <= 2 && uniform) {
        st = launch_gemv_fused(ctx, src0->type, src0->data, src0->nb[1], M, K, src1, (int)N, (float *)dst->data, ldd);
        if (st != B200Q_UNSUPPORTED) return st;
    }
    if ((st = get_activation(ctx, ti.act_form, src1, &act)) != B200Q_OK) return st;
    // decode widths go to the GEMV; wider products walk it in groups of eight columns
    // until the tensor-core GEMM takes them
    const int64_t run = uniform ? N : dst->ne[1];     // columns that share one stride
    for (int64_t c0 = 0; c0 < N; c0 += run) {
        const int64_t c23 = c0 / dst->ne[1], c2 = c23 % dst->ne[2], c3 = c23 / dst->ne[2];
        float *base = uniform ? (float *)dst->data
                              : (float *)((uint8_t *)dst->data + c2 * dst->nb[2] + c3 * dst->nb[3]);
        if (N > 8) count(ctx, ST_MUL_MAT_GEMV_CHUNKS);
        for (int64_t c = 0; c < run; c += 8) {
            const int nc = (int)(run - c < 8 ? run - c : 8);
            st = launch_gemv(ctx, src0->type, src0->data, src0->nb[1], M, K, act, c0 + c, nc, base + c * ldd, ldd);
            if (st != B200Q_OK) return st;
        }
    }
    return B200Q_OK;
}

b200q_status b200q_mul_mat_id(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1,
                              const b200q_tensor *ids, b200q_tensor *dst) {
    if (!ctx) return B200Q_INVALID;
    b200q_status st = check_mul_mat(ctx, src0, src1, dst, true);
    if (st != B200Q_OK) return st;
    st = check_ids(ctx, src0, src1, ids, dst);
    if (st != B200Q_OK) return st;
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    TypeInfo ti;
    type_info(src0->type, &ti);
    const int64_t K = src0->ne[0], M = src0->ne[1];
    const int n_expert = (int)src0->ne[2], n_used = (int)ids->ne[0], n_tok = (int)ids->ne[1], ne11 = (int)src1->ne[1];
    if (M == 0 || n_used == 0 || n_tok == 0) return B200Q_OK;
    const int64_t ld1 = (int64_t)(dst->nb[1] / sizeof(float)), ld2 = (int64_t)(dst->nb[2] / sizeof(float));
    // prompt-sized batches of the super-block types go to the tensor cores: the route's 128-pair tiles
    // are the GEMM's column tiles (an expert with few pairs pays a whole tile, so the batch must carry
    // enough pairs per expert on average to beat the per-tile GEMV below)
    const bool per32 = gemm_tc_supported(src0->type, M, K, 1, src0->data, src0->nb[1]);
    const bool per256 = gemm_kq_supported(src0->type, M, K, 1, src0->data, src0->nb[1]);
    if ((int64_t)n_used * n_tok >= 8 * (int64_t)n_expert && (int64_t)n_used * n_tok >= 256 && !ctx->no_tc && (per32 || per256) &&
        src0->nb[2] % 16 == 0 && src1->nb[1] % 16 == 0 && src1->nb[2] % 16 == 0 && (uintptr_t)src1->data % 16 == 0) {
        RouteView rv;
        if ((st = moe_route(ctx, ids, n_expert, &rv)) != B200Q_OK) return st;
        const size_t bytes = per32 ? gemm_tc_id_act_bytes(K, rv.max_tiles128) : gemm_kq_id_act_bytes(K, rv.max_tiles128);
        const void *before = ctx->moe_ws[7].ptr;
        if ((st = ws_reserve(ctx, &ctx->moe_ws[7], bytes)) != B200Q_OK) return st;
        const bool grew = ctx->moe_ws[7].ptr != before;
        TileRoute tr = { rv.tiles128, rv.n_tiles + 4, rv.pairs, n_used, ne11, src1->nb[1], src1->nb[2], ld1, ld2 };
        count(ctx, ST_MOE_GEMM);
        // the scratch may already hold this very activation, gathered for these ids in this graph
        auto &ma = ctx->moe_act;
        bool ready = !grew && ma.src1 == src1->data && ma.ids == ids->data && ma.src1_id == src1->id && ma.ids_id == ids->id && ma.gen == ctx->generation && ma.per32 == (int)per32 &&
                     ma.n_expert == n_expert;
        for (int i = 0; i < 4 && ready; ++i) ready = ma.ne[i] == src1->ne[i] && ma.nb[i] == src1->nb[i];
        if (ready) count(ctx, ST_ACT_CACHE_HIT);
        ma.src1 = src1->data;
        ma.ids = ids->data;
        ma.src1_id = src1->id;
        ma.ids_id = ids->id;
        ma.gen = ctx->generation;
        ma.per32 = (int)per32;
        ma.n_expert = n_expert;
        for (int i = 0; i < 4; ++i) { ma.ne[i] = src1->ne[i]; ma.nb[i] = src1->nb[i]; }
        return per32 ? launch_gemm_tc_id(ctx, src0, src1, tr, rv.max_tiles128, (uint8_t *)ctx->moe_ws[7].ptr, (float *)dst->data, ready)
                     : launch_gemm_kq_id(ctx, src0, src1, tr, rv.max_tiles128, (uint8_t *)ctx->moe_ws[7].ptr, (float *)dst->data, ready);
    }
    ActView act;
    if ((st = get_activation(ctx, ti.act_form, src1, &act)) != B200Q_OK) return st;
    // a handful of tokens: one unit per pair, its expert read on the device (the reference's
    // per-pair GEMV below GGML_OPENCL_KQ_MM_ID_MIN_TOK); more: route once per ids tensor
    // and graph, then one launch per tile size class
    if (n_tok <= 4)
        return launch_gemv_id(ctx, src0->type, src0->data, src0->nb[1], src0->nb[2], M, K, act, 1, nullptr, nullptr,
                              (int64_t)n_used * n_tok, nullptr, ids, n_expert, n_used, ne11, (float *)dst->data, ld1, ld2);
    RouteView rv;
    if ((st = moe_route(ctx, ids, n_expert, &rv)) != B200Q_OK) return st;
    static const int widths[4] = { 1, 2, 4, 8 };
    for (int k = 3; k >= 0; --k) {
        st = launch_gemv_id(ctx, src0->type, src0->data, src0->nb[1], src0->nb[2], M, K, act, widths[k], rv.tiles[k],
                            rv.n_tiles + k, rv.max_tiles, rv.pairs, ids, n_expert, n_used, ne11, (float *)dst->data, ld1, ld2);
        if (st != B200Q_OK) return st;
    }
    return B200Q_OK;
}

static b200q_status join_copy_stream(b200q_ctx *ctx);

// ---- CUDA graphs ----------------------------------------------------------------------

struct b200q_graph {
    cudaGraph_t     graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

b200q_status b200q_capture_begin(b200q_ctx *ctx) {
    if (!ctx) return B200Q_INVALID;
    if (ctx->capturing) return fail(ctx, B200Q_INVALID, "capture already open");
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    B200Q_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    // a recorded sequence must contain its own quantizers, routes and gathers: nothing cached by the
    // warm-up run before the capture may be reused inside it, or every replay would multiply by the
    // warm-up's activation
    ++ctx->generation;
    ctx->moe_act.src1 = nullptr;
    // the copy stream joins the capture, so staged and fetched copies become nodes of the graph
    B200Q_CUDA(ctx, cudaEventRecord(ctx->ev_fork, ctx->stream));
    B200Q_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->ev_fork, 0));
    B200Q_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->ev_fork, 0));
    ctx->copy_pending = true;
    return B200Q_OK;
}

b200q_status b200q_capture_end(b200q_ctx *ctx, b200q_graph **out) {
    if (!ctx || !out) return B200Q_INVALID;
    *out = nullptr;
    if (!ctx->capturing) return fail(ctx, B200Q_INVALID, "no capture open");
    ctx->capturing = false;
    ++ctx->generation;                                      // and nothing cached inside the capture outlives it
    ctx->moe_act.src1 = nullptr;
    join_copy_stream(ctx);                                  // every forked stream must be back before the capture ends
    b200q_graph *g = new b200q_graph();
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
        if (g->graph) cudaGraphDestroy(g->graph);
        delete g;
        return fail(ctx, B200Q_CUDA_ERROR, "graph capture: %s", cudaGetErrorString(e));
    }
    *out = g;
    return B200Q_OK;
}

b200q_status b200q_graph_launch(b200q_ctx *ctx, b200q_graph *g) {
    if (!ctx || !g || !g->exec) return B200Q_INVALID;
    B200Q_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
    count(ctx, ST_GRAPH_LAUNCH);
    return B200Q_OK;
}

void b200q_graph_free(b200q_graph *g) {
    if (!g) return;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
}

// ---- buffers and copies --------------------------------------------------------------

b200q_status b200q_buffer_alloc(b200q_ctx *ctx, size_t bytes, void **dev_ptr) {
    if (!ctx || !dev_ptr) return B200Q_INVALID;
    *dev_ptr = nullptr;
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaError_t e = cudaMalloc(dev_ptr, bytes ? bytes : 1);
    if (e != cudaSuccess) return fail(ctx, B200Q_NO_MEMORY, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    return B200Q_OK;
}

b200q_status b200q_buffer_free(b200q_ctx *ctx, void *dev_ptr) {
    if (!ctx) return B200Q_INVALID;
    if (!dev_ptr) return B200Q_OK;
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    B200Q_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    B200Q_CUDA(ctx, cudaFree(dev_ptr));
    return B200Q_OK;
}

b200q_status b200q_tensor_set(b200q_ctx *ctx, void *dev_dst, const void *host_src, size_t bytes) {
    if (!ctx || (bytes && (!dev_dst || !host_src))) return B200Q_INVALID;
    B200Q_CUDA(ctx, cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return B200Q_OK;
}

b200q_status b200q_tensor_get(b200q_ctx *ctx, void *host_dst, const void *dev_src, size_t bytes) {
    if (!ctx || (bytes && (!host_dst || !dev_src))) return B200Q_INVALID;
    B200Q_CUDA(ctx, cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return B200Q_OK;
}

b200q_status b200q_tensor_copy(b200q_ctx *ctx, void *dev_dst, const void *dev_src, size_t bytes) {
    if (!ctx || (bytes && (!dev_dst || !dev_src))) return B200Q_INVALID;
    B200Q_CUDA(ctx, cudaMemcpyAsync(dev_dst, dev_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return B200Q_OK;
}

// Overlapped copies. They run on the context's two copy streams (one per direction, like the GPU's copy
// engines), so they do not sit in the queue between two kernels of the compute stream: an upload runs while earlier kernels compute, a download while later ones do.
// stage: host -> device; every kernel queued after the call waits for it. fetch: device -> host, after
// everything queued before the call; complete at the next b200q_synchronize. The caller keeps the usual
// double-buffering discipline: a device buffer being staged must not still be read by queued kernels, a
// buffer being fetched must not be rewritten before the synchronize.
b200q_status b200q_tensor_stage(b200q_ctx *ctx, void *dev_dst, const void *host_src, size_t bytes) {
    if (!ctx || (bytes && (!dev_dst || !host_src))) return B200Q_INVALID;
    B200Q_CUDA(ctx, cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->copy_in));
    B200Q_CUDA(ctx, cudaEventRecord(ctx->ev_join, ctx->copy_in));
    B200Q_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
    return B200Q_OK;
}

b200q_status b200q_tensor_fetch(b200q_ctx *ctx, void *host_dst, const void *dev_src, size_t bytes) {
    if (!ctx || (bytes && (!host_dst || !dev_src))) return B200Q_INVALID;
    B200Q_CUDA(ctx, cudaEventRecord(ctx->ev_fork, ctx->stream));
    B200Q_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->ev_fork, 0));
    B200Q_CUDA(ctx, cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, ctx->copy_out));
    ctx->copy_pending = true;
    return B200Q_OK;
}

// the compute stream waits for what the copy stream still holds (before a capture ends, before a synchronize)
static b200q_status join_copy_stream(b200q_ctx *ctx) {
    if (!ctx->copy_pending) return B200Q_OK;
    B200Q_CUDA(ctx, cudaEventRecord(ctx->ev_join, ctx->copy_out));
    B200Q_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
    B200Q_CUDA(ctx, cudaEventRecord(ctx->ev_join, ctx->copy_in));
    B200Q_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
    ctx->copy_pending = false;
    return B200Q_OK;
}

b200q_status b200q_synchronize(b200q_ctx *ctx) {
    if (!ctx) return B200Q_INVALID;
    b200q_status js = join_copy_stream(ctx);
    if (js != B200Q_OK) return js;
    B200Q_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    // a kernel whose bounded wait ran out says so here
    int err = 0;
    B200Q_CUDA(ctx, cudaMemcpy(&err, ctx->error_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (err) {
        cudaMemset(ctx->error_word, 0, sizeof(int));
        return fail(ctx, B200Q_TIMEOUT, "a device-side wait gave up (error word %d)", err);
    }
    return B200Q_OK;
}

b200q_status b200q_host_alloc(size_t bytes, void **host_ptr) {
    if (!host_ptr) return B200Q_INVALID;
    return cudaMallocHost(host_ptr, bytes ? bytes : 1) == cudaSuccess ? B200Q_OK : B200Q_NO_MEMORY;
}

b200q_status b200q_host_free(void *host_ptr) {
    return (!host_ptr || cudaFreeHost(host_ptr) == cudaSuccess) ? B200Q_OK : B200Q_CUDA_ERROR;
}

// ---- stats, timing --------------------------------------------------------------------

const char *b200q_stats(b200q_ctx *ctx) {
    if (!ctx) return "";
    ctx->stats_text.clear();
    for (int i = 0; i < ST_COUNT; ++i)
        if (ctx->counters[i]) ctx->stats_text += std::string(stat_name(i)) + "\t" + std::to_string(ctx->counters[i]) + "\n";
    return ctx->stats_text.c_str();
}

void b200q_stats_reset(b200q_ctx *ctx) {
    if (ctx) memset(ctx->counters, 0, sizeof(ctx->counters));
}

b200q_status b200q_timer_start(b200q_ctx *ctx) {
    if (!ctx) return B200Q_INVALID;
    B200Q_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    return B200Q_OK;
}

b200q_status b200q_timer_stop(b200q_ctx *ctx, float *elapsed_ms) {
    if (!ctx || !elapsed_ms) return B200Q_INVALID;
    B200Q_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    B200Q_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
    B200Q_CUDA(ctx, cudaEventElapsedTime(elapsed_ms, ctx->ev0, ctx->ev1));
    return B200Q_OK;
}

b200q_status b200q_flush_l2(b200q_ctx *ctx) {
    if (!ctx) return B200Q_INVALID;
    const size_t bytes = 256u << 20;                     // twice the 126 MB L2
    b200q_status st = ws_reserve(ctx, &ctx->flush_buf, bytes);
    if (st != B200Q_OK) return st;
    B200Q_CUDA(ctx, cudaMemsetAsync(ctx->flush_buf.ptr, 0, bytes, ctx->stream));
    return B200Q_OK;
}

// ---- debug views ----------------------------------------------------------------------

b200q_status b200q_debug_quantize_act(b200q_ctx *ctx, int weight_type, const b200q_tensor *src1, void *dev_codes,
                                      void *dev_scales, void *dev_sums) {
    if (!ctx || !src1 || !dev_codes || !dev_scales) return B200Q_INVALID;
    TypeInfo ti;
    if (!type_info(weight_type, &ti)) return fail(ctx, B200Q_UNSUPPORTED, "weight type %d", weight_type);
    if (!is_contiguous_f32(src1) || src1->ne[0] % ti.block) return fail(ctx, B200Q_UNSUPPORTED, "src1 layout");
    if (!dev_sums) return B200Q_INVALID;
    const int64_t K = src1->ne[0], N = src1->ne[1] * src1->ne[2] * src1->ne[3];
    ctx->moe_act.src1 = nullptr;                            // the scratch below is shared with the MUL_MAT_ID activation
    b200q_status st = ws_reserve(ctx, &ctx->moe_ws[7], sizeof(int16_t) * (size_t)(N * (K / 16)) + 64);
    if (st != B200Q_OK) return st;
    return launch_quantize_act(ctx, ti.act_form, src1, (int8_t *)dev_codes, dev_scales, (int16_t *)dev_sums,
                               (int16_t *)ctx->moe_ws[7].ptr);
}

b200q_status b200q_debug_wait_timeout(b200q_ctx *ctx, unsigned polls) {
    if (!ctx) return B200Q_INVALID;
    if (polls > (1u << 20)) polls = 1u << 20;
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    debug_wait_timeout_kernel<<<1, 1, 0, ctx->stream>>>(polls, ctx->error_word);
    B200Q_CUDA(ctx, cudaGetLastError());
    return B200Q_OK;
}

b200q_status b200q_debug_check_guards(b200q_ctx *ctx, int *blocks, int *violated) {
    if (!ctx || !blocks || !violated) return B200Q_INVALID;
    *blocks = *violated = 0;
    if (!ctx->canary) return fail(ctx, B200Q_INVALID, "guard words are off: create the context with B200Q_CANARY=1");
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    B200Q_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    Workspace *list[64];
    const char *names[64];
    int n = 0;
    for (auto &e : ctx->act_cache) {
        list[n] = &e.codes;  names[n++] = "activation codes";
        list[n] = &e.scales; names[n++] = "activation scales";
        list[n] = &e.sums;   names[n++] = "activation sums";
        list[n] = &e.sums16; names[n++] = "activation sums16";
    }
    static const char *ws_names[10] = { "moe_ws[0]", "moe_ws[1]", "moe_ws[2]", "moe_ws[3]", "moe_ws[4]",
                                        "moe_ws[5]", "moe_ws[6]", "moe_ws[7]", "moe_ws[8]", "moe_ws[9]" };
    for (int i = 0; i < 10; ++i) { list[n] = &ctx->moe_ws[i]; names[n++] = ws_names[i]; }
    list[n] = &ctx->flush_buf; names[n++] = "flush buffer";
    n += moe_route_workspaces(ctx, list + n, names + n);
    uint8_t host[2 * WS_GUARD];
    for (int i = 0; i < n; ++i) {
        const Workspace *w = list[i];
        if (!w->base) continue;
        ++*blocks;
        B200Q_CUDA(ctx, cudaMemcpy(host, w->base, WS_GUARD, cudaMemcpyDeviceToHost));
        B200Q_CUDA(ctx, cudaMemcpy(host + WS_GUARD, (const uint8_t *)w->ptr + w->cap, WS_GUARD, cudaMemcpyDeviceToHost));
        for (size_t b = 0; b < 2 * WS_GUARD; ++b)
            if (host[b] != (uint8_t)WS_GUARD_BYTE) {
                if (!*violated)
                    fail(ctx, B200Q_INVALID, "%s (%zu bytes): guard byte %zu %s the block was overwritten", names[i], w->cap,
                         b % WS_GUARD, b < WS_GUARD ? "before" : "after");
                ++*violated;
                break;
            }
    }
    return B200Q_OK;
}

b200q_status b200q_debug_dequantize(b200q_ctx *ctx, const b200q_tensor *src0, float *dev_out) {
    if (!ctx || !src0 || !dev_out) return B200Q_INVALID;
    TypeInfo ti;
    if (!type_info(src0->type, &ti) || src0->ne[0] % ti.block) return fail(ctx, B200Q_UNSUPPORTED, "weight layout");
    return launch_dequantize(ctx, src0->type, src0->data, src0->ne[1] * src0->ne[2] * src0->ne[3], src0->ne[0],
                             src0->nb[1], dev_out);
}

}  // extern "C"
