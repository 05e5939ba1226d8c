// moe_ffn.cu -- the steps either side of MUL_MAT_ID in a mixture-of-experts feed-forward block, and the
// block as one call:
//
//   router   softmax over a token's expert logits, the n_used largest in descending order (ties: the lower
//            expert id) and their probabilities divided by their clamped sum -- the reference's fused router
//            kernel_topk_moe_softmax_norm_n* (marfrit/arcint contrib/llama.cpp/patches/
//            0000-09-moe-routing-gemm-tiles.patch:2062-2115 of the kernel file's added text, lines 928-987 of
//            the patch): p = exp(x - max), s = sum p, pick k times the largest unpicked p, w_j = p_j / s,
//            w_j /= clamp(sum_j w_j, cmin, cmax);
//   gate/up  two MUL_MAT_ID over the token's activation (they share the route, the gathered activation and,
//            under expert parallelism, the dispatch);
//   SwiGLU   h = silu(gate) * up, elementwise;
//   down     MUL_MAT_ID over h;
//   combine  y[:, t] = sum_i w[i, t] * down[:, i, t].
//
// One warp per token in the router: a lane holds experts lane, lane + 32, ... in registers (up to 1024
// experts), maximum / sum / selection are warp shuffles, no shared memory and no block barrier.
#include <math.h>

#include "common.cuh"

namespace b200q {

constexpr int ROUTER_MAX_EXPERT = 1024, ROUTER_MAX_USED = 32;

template <int NPER>
__global__ void __launch_bounds__(128)
moe_router_kernel(const uint8_t *__restrict__ logits, size_t nb1, int n_expert, int n_used, int n_tok, float cmin, float cmax,
                  uint8_t *__restrict__ ids, size_t ids_nb1, uint8_t *__restrict__ wts, size_t wts_nb1) {
    const int lane = threadIdx.x & 31, t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tok) return;                                    // whole warps leave together
    const float *x = reinterpret_cast<const float *>(logits + (size_t)t * nb1);
    int32_t *io = reinterpret_cast<int32_t *>(ids + (size_t)t * ids_nb1);
    float *wo = reinterpret_cast<float *>(wts + (size_t)t * wts_nb1);
    float p[NPER];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
        const int i = lane + 32 * j;
        p[j] = i < n_expert ? x[i] : -INFINITY;
        m = fmaxf(m, p[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
        const int i = lane + 32 * j;
        p[j] = i < n_expert ? expf(p[j] - m) : -1.f;           // -1: never selected (probabilities are >= 0)
        if (i < n_expert) s += p[j];
    }
    // the sum in a fixed order (butterfly), so every lane holds the same s
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    float wsum = 0.f, wsel = 0.f;                              // lane j keeps weight j (n_used <= 32)
    for (int j = 0; j < n_used; ++j) {
        float bv = -1.f;
        int bi = INT_MAX;
#pragma unroll
        for (int q = 0; q < NPER; ++q)
            if (p[q] > bv) { bv = p[q]; bi = lane + 32 * q; }   // strict: the lowest index among equals stays
        float gv = bv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gv = fmaxf(gv, __shfl_xor_sync(0xFFFFFFFFu, gv, o));
        int gi = bv == gv ? bi : INT_MAX;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gi = min(gi, __shfl_xor_sync(0xFFFFFFFFu, gi, o));
        const float w = gv / s;
        wsum += w;
        if (lane == j) wsel = w;
        if (lane == 0) io[j] = gi;
        if ((gi & 31) == lane) {
#pragma unroll
            for (int q = 0; q < NPER; ++q)
                if (q == (gi >> 5)) p[q] = -1.f;                // taken
        }
    }
    const float denom = fminf(fmaxf(wsum, cmin), cmax);
    if (lane < n_used) wo[lane] = wsel / denom;
}

// h = silu(g) * u over n elements; g, u, h may be the same buffers (h may overwrite g)
__global__ void __launch_bounds__(256)
swiglu_kernel(const float *__restrict__ g, const float *__restrict__ u, float *__restrict__ h, int64_t n4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 a = reinterpret_cast<const float4 *>(g)[i], b = reinterpret_cast<const float4 *>(u)[i];
        float4 r;
        r.x = a.x / (1.f + expf(-a.x)) * b.x;
        r.y = a.y / (1.f + expf(-a.y)) * b.y;
        r.z = a.z / (1.f + expf(-a.z)) * b.z;
        r.w = a.w / (1.f + expf(-a.w)) * b.w;
        reinterpret_cast<float4 *>(h)[i] = r;
    }
}

// y[m, t] = sum_i w[i, t] * d[m, i, t]; d is [M][n_used][n_tok] packed, y has column stride ldy, added in slot order
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float *__restrict__ d, const uint8_t *__restrict__ wts, size_t wts_nb1, int M, int n_used, int n_tok,
                   float *__restrict__ y, int64_t ldy) {
    const int t = blockIdx.y;
    const float *w = reinterpret_cast<const float *>(wts + (size_t)t * wts_nb1);
    const float *dt = d + (size_t)t * n_used * M;
    for (int m = blockIdx.x * blockDim.x + threadIdx.x; m < M; m += gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < n_used; ++i) acc = fmaf(w[i], dt[(size_t)i * M + m], acc);
        y[(size_t)t * ldy + m] = acc;
    }
}

static b200q_status launch_router(b200q_ctx *ctx, const b200q_tensor *logits, int n_used, float cmin, float cmax,
                                  const b200q_tensor *ids, const b200q_tensor *wts) {
    const int n_expert = (int)logits->ne[0], n_tok = (int)logits->ne[1];
    if (n_tok == 0) return B200Q_OK;
    const dim3 grid((unsigned)((n_tok + 3) / 4));
#define B200Q_ROUTER(NPER)                                                                                                   \
    moe_router_kernel<NPER><<<grid, 128, 0, ctx->stream>>>((const uint8_t *)logits->data, logits->nb[1], n_expert, n_used, n_tok, \
                                                           cmin, cmax, (uint8_t *)ids->data, ids->nb[1], (uint8_t *)wts->data, wts->nb[1])
    if (n_expert <= 64) B200Q_ROUTER(2);
    else if (n_expert <= 128) B200Q_ROUTER(4);
    else if (n_expert <= 256) B200Q_ROUTER(8);
    else if (n_expert <= 512) B200Q_ROUTER(16);
    else B200Q_ROUTER(32);
#undef B200Q_ROUTER
    B200Q_CUDA(ctx, cudaGetLastError());
    count(ctx, ST_MOE_ROUTER);
    return B200Q_OK;
}

}  // namespace b200q

using namespace b200q;

extern "C" {

b200q_status b200q_moe_router(b200q_ctx *ctx, const b200q_tensor *logits, int n_used, float cmin, float cmax, b200q_tensor *ids,
                              b200q_tensor *weights) {
    if (!ctx || !logits || !ids || !weights) return B200Q_INVALID;
    if (logits->type != B200Q_TYPE_F32 || ids->type != B200Q_TYPE_I32 || weights->type != B200Q_TYPE_F32 || logits->nb[0] != 4 ||
        ids->nb[0] != 4 || weights->nb[0] != 4 || logits->ne[2] != 1 || logits->ne[3] != 1)
        return fail(ctx, B200Q_UNSUPPORTED, "router: f32 logits [n_expert, n_tok], i32 ids and f32 weights [n_used, n_tok]");
    if (logits->ne[0] < 1 || logits->ne[0] > ROUTER_MAX_EXPERT || n_used < 1 || n_used > ROUTER_MAX_USED || n_used > logits->ne[0])
        return fail(ctx, B200Q_UNSUPPORTED, "router: %lld experts, %d used (limits %d, %d)", (long long)logits->ne[0], n_used,
                    ROUTER_MAX_EXPERT, ROUTER_MAX_USED);
    if (ids->ne[0] != n_used || weights->ne[0] != n_used || ids->ne[1] != logits->ne[1] || weights->ne[1] != logits->ne[1])
        return fail(ctx, B200Q_INVALID, "router: output shapes");
    if ((uintptr_t)logits->data % 4 || logits->nb[1] % 4 || (uintptr_t)ids->data % 4 || ids->nb[1] % 4 || (uintptr_t)weights->data % 4 ||
        weights->nb[1] % 4)
        return fail(ctx, B200Q_UNSUPPORTED, "router: 4-byte aligned rows");
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    return launch_router(ctx, logits, n_used, cmin, cmax, ids, weights);
}

b200q_status b200q_moe_ffn(b200q_ctx *ctx, const b200q_tensor *gate_w, const b200q_tensor *up_w, const b200q_tensor *down_w,
                           const b200q_tensor *x, const b200q_tensor *logits, int n_used, float cmin, float cmax, b200q_tensor *y,
                           b200q_tensor *ids_out, b200q_tensor *weights_out) {
    if (!ctx || !gate_w || !up_w || !down_w || !x || !logits || !y) return B200Q_INVALID;
    const int64_t d_model = gate_w->ne[0], d_ff = gate_w->ne[1], n_expert = gate_w->ne[2], n_tok = x->ne[1];
    if (up_w->ne[0] != d_model || up_w->ne[1] != d_ff || up_w->ne[2] != n_expert || down_w->ne[0] != d_ff || down_w->ne[1] != d_model ||
        down_w->ne[2] != n_expert || x->ne[0] != d_model || x->ne[2] != 1 || x->ne[3] != 1 || logits->ne[0] != n_expert ||
        logits->ne[1] != n_tok || y->ne[0] != d_model || y->ne[1] != n_tok || y->ne[2] != 1 || y->ne[3] != 1)
        return fail(ctx, B200Q_INVALID, "moe_ffn: shapes");
    if (x->type != B200Q_TYPE_F32 || y->type != B200Q_TYPE_F32 || x->nb[0] != 4 || y->nb[0] != 4 || y->nb[1] % 4 || d_ff % 4)
        return fail(ctx, B200Q_UNSUPPORTED, "moe_ffn: packed f32 activations, d_ff a multiple of 4");
    if (n_tok == 0) return B200Q_OK;
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    // scratch: ids, weights, gate, up (becomes h), down
    const size_t pairs = (size_t)n_used * (size_t)n_tok;
    auto up256 = [](size_t v) { return (v + 255) / 256 * 256; };
    const size_t o_ids = 0, o_w = up256(pairs * 4), o_g = o_w + up256(pairs * 4), o_u = o_g + up256(pairs * d_ff * 4),
                 o_d = o_u + up256(pairs * d_ff * 4), total = o_d + up256(pairs * d_model * 4);
    b200q_status st = ws_reserve(ctx, &ctx->moe_ws[8], total);
    if (st != B200Q_OK) return st;
    uint8_t *ws = (uint8_t *)ctx->moe_ws[8].ptr;
    auto tensor = [](int type, void *data, int64_t e0, int64_t e1, int64_t e2, const void *ident) {
        b200q_tensor t;
        t.type = type;
        t.data = data;
        t.id = ident;
        t.ne[0] = e0; t.ne[1] = e1; t.ne[2] = e2; t.ne[3] = 1;
        t.nb[0] = 4; t.nb[1] = 4 * (size_t)e0; t.nb[2] = t.nb[1] * (size_t)e1; t.nb[3] = t.nb[2] * (size_t)e2;
        return t;
    };
    b200q_tensor ids = ids_out ? *ids_out : tensor(B200Q_TYPE_I32, ws + o_ids, n_used, n_tok, 1, ws + o_ids);
    b200q_tensor wts = weights_out ? *weights_out : tensor(B200Q_TYPE_F32, ws + o_w, n_used, n_tok, 1, ws + o_w);
    if ((st = b200q_moe_router(ctx, logits, n_used, cmin, cmax, &ids, &wts)) != B200Q_OK) return st;
    // the block's own tensors live under a cache generation of its own: their buffers are reused by the next call
    const uint64_t caller_gen = ctx->generation;
    ctx->generation = (1ull << 61) + ++ctx->private_generation;
    b200q_tensor x3 = *x;                                      // [d_model, 1, n_tok]: every used expert reads the token's row
    x3.ne[1] = 1; x3.ne[2] = n_tok; x3.nb[2] = x->nb[1]; x3.nb[1] = x->nb[1]; x3.nb[3] = x->nb[1] * (size_t)n_tok;
    b200q_tensor g = tensor(B200Q_TYPE_F32, ws + o_g, d_ff, n_used, n_tok, ws + o_g);
    b200q_tensor u = tensor(B200Q_TYPE_F32, ws + o_u, d_ff, n_used, n_tok, ws + o_u);
    b200q_tensor d = tensor(B200Q_TYPE_F32, ws + o_d, d_model, n_used, n_tok, ws + o_d);
    st = b200q_mul_mat_id(ctx, gate_w, &x3, &ids, &g);
    if (st == B200Q_OK) st = b200q_mul_mat_id(ctx, up_w, &x3, &ids, &u);
    if (st == B200Q_OK) {
        const int64_t n4 = (int64_t)(pairs * d_ff / 4);
        const int64_t blocks = (n4 + 255) / 256;
        swiglu_kernel<<<(unsigned)(blocks > 148 * 8 ? 148 * 8 : blocks), 256, 0, ctx->stream>>>((const float *)g.data, (const float *)u.data,
                                                                                                (float *)u.data, n4);
        if (cudaGetLastError() != cudaSuccess) st = fail(ctx, B200Q_CUDA_ERROR, "swiglu launch");
    }
    if (st == B200Q_OK) st = b200q_mul_mat_id(ctx, down_w, &u, &ids, &d);
    if (st == B200Q_OK) {
        const dim3 grid((unsigned)((d_model + 255) / 256), (unsigned)n_tok);
        moe_combine_kernel<<<grid, 256, 0, ctx->stream>>>((const float *)d.data, (const uint8_t *)wts.data, wts.nb[1], (int)d_model, n_used,
                                                          (int)n_tok, (float *)y->data, (int64_t)(y->nb[1] / 4));
        if (cudaGetLastError() != cudaSuccess) st = fail(ctx, B200Q_CUDA_ERROR, "combine launch");
    }
    ctx->generation = caller_gen;
    if (st == B200Q_OK) count(ctx, ST_MOE_FFN);
    return st;
}

}  // extern "C"
