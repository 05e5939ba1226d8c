// moe.cu -- MUL_MAT_ID routing: the (token, slot) pairs sorted by expert and cut into tiles
// of pairs of one expert, as the reference's kernel_moe_route_tiles does (marfrit/arcint
// contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch:2417-2444: count per expert
// with shared-memory atomics, prefix, emit (expert, first, count) tiles, scatter), with two
// differences: the tiles are split into four lists by size (at most 1, 2, 4, 8 pairs) so
// each list runs on the kernel instantiation of that many columns, and the route is kept
// per ids tensor for the rest of the graph (the reference's route cache, :1264-1287) so
// gate, up and down of a layer share one.
//
// Pair p = t*n_used + i. Ids outside [0, n_expert) are clamped, as in the reference kernel.
// The order of pairs inside an expert is whatever the atomics give: every pair's result is
// computed independently of its tile mates, so the order does not reach the output.
#include "common.cuh"

namespace b200q {

struct RouteEntry {
    const void *ids_data = nullptr;
    const void *ids_id = nullptr;      // the caller's tensor identity (NULL: unknown)
    int64_t ne[2] = { 0, 0 };
    size_t  nb1 = 0;
    int     n_expert = 0;
    uint64_t gen = 0;
    bool    valid = false;
    int     experts_per_owner = 0;
    bool    skip_negative = false;
    Workspace buf;               // pairs | 5 tile lists | 8 counters | owner counts
    RouteView view;
};

__global__ void __launch_bounds__(1024)
moe_route_kernel(const uint8_t *ids, size_t nb1, int n_used, int n_tok, int n_expert, int32_t *pairs,
                 int32_t *tiles0, int32_t *tiles1, int32_t *tiles2, int32_t *tiles3, int32_t *tiles128, int32_t *n_tiles,
                 int32_t *owner_counts, int experts_per_owner, int n_groups, int skip_negative) {
    // Counters are kept once per group of warps (a skewed router sends a tenth of all pairs to one
    // expert: one shared-memory counter would serialize them): cntg / fillg [n_groups][n_expert].
    extern __shared__ int sm[];
    int *cnt = sm, *base = sm + n_expert, *toff = sm + 2 * n_expert;          // cnt: totals; toff: [5][n_expert]
    int *cntg = sm + 7 * n_expert, *fillg = cntg + n_groups * n_expert;
    const int tid = threadIdx.x, nth = blockDim.x;
    const int grp = (tid >> 5) * n_groups / (nth >> 5);                          // this warp's counter group
    const int n_pairs = n_used * n_tok;
    auto expert_of = [&](int p) {
        const int t = p / n_used, i = p - t * n_used;
        const int e = reinterpret_cast<const int32_t *>(ids + (size_t)t * nb1)[i];
        // skip_negative: a negative id marks an empty slot (expert-parallel receive regions are only partly
        // filled) and takes no part in the route; otherwise ids are clamped like the reference's route kernel
        if (skip_negative && e < 0) return -1;
        return min(max(e, 0), n_expert - 1);
    };
    for (int i = tid; i < 2 * n_groups * n_expert; i += nth) cntg[i] = 0;      // cntg and fillg
    __syncthreads();
    // eight independent loads in flight per thread (the ids come from global memory)
    const int lane = tid & 31;
    for (int p0 = tid; p0 < n_pairs; p0 += 8 * nth) {
        int e8[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) e8[k] = p0 + k * nth < n_pairs ? expert_of(p0 + k * nth) : -1;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (e8[k] >= 0) atomicAdd(&cntg[grp * n_expert + e8[k]], 1);
    }
    __syncthreads();
    // per expert: the groups' counts become the groups' offsets inside the expert's run; their sum is the count
    for (int e = tid; e < n_expert; e += nth) {
        int run = 0;
        for (int g = 0; g < n_groups; ++g) {
            const int t = cntg[g * n_expert + e];
            cntg[g * n_expert + e] = run;
            run += t;
        }
        cnt[e] = run;
    }
    __syncthreads();
    // six exclusive prefix sums over the experts at once (block-wide scan, 1024 experts per round): the pair
    // offsets, the tile offsets of the four decode size classes, and of the 128-pair tiles of the tensor-core
    // path (which covers every pair once more, in its own list)
    __shared__ int warp_tot[6][32], carry[6], round_tot[6];
    const int warp = tid >> 5, n_warps = nth >> 5;
    if (tid < 6) carry[tid] = 0;
    __syncthreads();
    for (int e0 = 0; e0 < n_expert; e0 += nth) {
        const int e = e0 + tid;
        const int c = e < n_expert ? cnt[e] : 0, rem = c & 7;
        int v[6], incl[6];
        v[0] = rem == 1;
        v[1] = rem == 2;
        v[2] = rem == 3 || rem == 4;
        v[3] = (c >> 3) + (rem >= 5);
        v[4] = (c + 127) >> 7;
        v[5] = c;
#pragma unroll
        for (int k = 0; k < 6; ++k) {
            int x = v[k];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int y = __shfl_up_sync(0xFFFFFFFFu, x, off);
                if (lane >= off) x += y;
            }
            incl[k] = x;
            if (lane == 31) warp_tot[k][warp] = x;
        }
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int k = 0; k < 6; ++k) {
                const int t = lane < n_warps ? warp_tot[k][lane] : 0;
                int x = t;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int y = __shfl_up_sync(0xFFFFFFFFu, x, off);
                    if (lane >= off) x += y;
                }
                warp_tot[k][lane] = x - t;                         // exclusive over the warps
                if (lane == 31) round_tot[k] = x;
            }
        }
        __syncthreads();
        if (e < n_expert) {
#pragma unroll
            for (int k = 0; k < 6; ++k) {
                const int ex = carry[k] + warp_tot[k][warp] + incl[k] - v[k];
                if (k == 5) base[e] = ex; else toff[k * n_expert + e] = ex;
            }
        }
        __syncthreads();
        if (tid < 6) carry[tid] += round_tot[tid];
        __syncthreads();
    }
    if (tid < 5) n_tiles[tid] = carry[tid];
    __syncthreads();
    for (int e = tid; e < n_expert; e += nth) {
        const int c = cnt[e], rem = c & 7, full = c >> 3, first = base[e];
        int32_t *t3 = tiles3 + 4 * toff[3 * n_expert + e];
        for (int k = 0; k < full; ++k) { t3[4 * k] = e; t3[4 * k + 1] = first + 8 * k; t3[4 * k + 2] = 8; t3[4 * k + 3] = 0; }
        if (rem) {
            int32_t *t = rem >= 5 ? t3 + 4 * full
                       : rem >= 3 ? tiles2 + 4 * toff[2 * n_expert + e]
                       : rem == 2 ? tiles1 + 4 * toff[1 * n_expert + e]
                                  : tiles0 + 4 * toff[e];
            t[0] = e; t[1] = first + 8 * full; t[2] = rem; t[3] = 0;
        }
        int32_t *tb = tiles128 + 4 * toff[4 * n_expert + e];
        for (int k = 0; 128 * k < c; ++k) { tb[4 * k] = e; tb[4 * k + 1] = first + 128 * k; tb[4 * k + 2] = min(128, c - 128 * k); tb[4 * k + 3] = 0; }
    }
    // the same thread meets the same pairs as in the counting pass, so its group's share of the run is its own
    for (int p0 = tid; p0 < n_pairs; p0 += 8 * nth) {
        int e8[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) e8[k] = p0 + k * nth < n_pairs ? expert_of(p0 + k * nth) : -1;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (e8[k] >= 0) {
                const int g = grp * n_expert + e8[k];
                pairs[base[e8[k]] + cntg[g] + atomicAdd(&fillg[g], 1)] = p0 + k * nth;
            }
    }
    // expert parallelism: how many pairs go to each owner (experts are owned in contiguous ranges)
    if (owner_counts) {
        const int n_owner = n_expert / experts_per_owner;
        for (int g = tid; g < n_owner; g += nth) {
            int c = 0;
            for (int e = g * experts_per_owner; e < (g + 1) * experts_per_owner; ++e) c += cnt[e];
            owner_counts[g] = c;
        }
    }
}

// expert-parallel dispatch: the activation row and the owner-local expert index of every pair, in
// the order of the sorted pair list (which groups pairs by owner because owners hold expert ranges)
__global__ void ep_pack_kernel(const uint8_t *src1, size_t nb1, size_t nb2, int ne11, const uint8_t *ids, size_t ids_nb1,
                               int n_used, int n_pairs, int K, int n_expert, int experts_per_owner,
                               const int32_t *pairs, float *send_x, int32_t *send_e) {
    const int pos = blockIdx.x;
    if (pos >= n_pairs) return;
    const int p = pairs[pos], t = p / n_used, i = p - t * n_used;
    const float4 *x = reinterpret_cast<const float4 *>(src1 + (size_t)(i % ne11) * nb1 + (size_t)t * nb2);
    float4 *o = reinterpret_cast<float4 *>(send_x + (size_t)pos * K);
    for (int k = threadIdx.x; k < K / 4; k += blockDim.x) o[k] = x[k];
    if (threadIdx.x == 0) {
        const int e = min(max(reinterpret_cast<const int32_t *>(ids + (size_t)t * ids_nb1)[i], 0), n_expert - 1);
        send_e[pos] = e % experts_per_owner;
    }
}

// expert-parallel combine: result row pos of the returned buffer belongs to pair pairs[pos]
__global__ void ep_unpack_kernel(const float *back, const int32_t *pairs, int n_used, int n_pairs, int M, float *dst,
                                 int64_t ld1, int64_t ld2) {
    const int pos = blockIdx.x;
    if (pos >= n_pairs) return;
    const int p = pairs[pos], t = p / n_used, i = p - t * n_used;
    const float *b = back + (size_t)pos * M;
    float *o = dst + t * ld2 + i * ld1;
    for (int m = threadIdx.x; m < M; m += blockDim.x) o[m] = b[m];
}

b200q_status launch_ep_pack(b200q_ctx *ctx, const b200q_tensor *src1, const b200q_tensor *ids, int n_expert,
                            int experts_per_owner, const int32_t *pairs, float *send_x, int32_t *send_e) {
    const int n_pairs = (int)(ids->ne[0] * ids->ne[1]);
    if (n_pairs == 0) return B200Q_OK;
    ep_pack_kernel<<<n_pairs, 128, 0, ctx->stream>>>((const uint8_t *)src1->data, src1->nb[1], src1->nb[2], (int)src1->ne[1],
                                                   (const uint8_t *)ids->data, ids->nb[1], (int)ids->ne[0], n_pairs,
                                                   (int)src1->ne[0], n_expert, experts_per_owner, pairs, send_x, send_e);
    B200Q_CUDA(ctx, cudaGetLastError());
    count(ctx, ST_MOE_PACK);
    return B200Q_OK;
}

b200q_status launch_ep_unpack(b200q_ctx *ctx, const float *back, const int32_t *pairs, int n_used, int n_pairs, int M,
                              float *dst, int64_t ld1, int64_t ld2) {
    if (n_pairs == 0) return B200Q_OK;
    ep_unpack_kernel<<<n_pairs, 128, 0, ctx->stream>>>(back, pairs, n_used, n_pairs, M, dst, ld1, ld2);
    B200Q_CUDA(ctx, cudaGetLastError());
    return B200Q_OK;
}

b200q_status moe_route(b200q_ctx *ctx, const b200q_tensor *ids, int n_expert, RouteView *out, int experts_per_owner) {
    const int n_used = (int)ids->ne[0], n_tok = (int)ids->ne[1];
    const int64_t n_pairs = (int64_t)n_used * n_tok;
    RouteEntry *hit = nullptr;
    for (RouteEntry *e : ctx->routes)
        if (e && e->valid && e->ids_data == ids->data && e->ids_id == ids->id && e->ne[0] == ids->ne[0] && e->ne[1] == ids->ne[1] &&
            e->nb1 == ids->nb[1] && e->n_expert == n_expert && e->gen == ctx->generation &&
            e->experts_per_owner == experts_per_owner && e->skip_negative == ctx->route_skip_negative) { hit = e; break; }
    if (hit) {
        count(ctx, ST_ROUTE_CACHE_HIT);
        *out = hit->view;
        return B200Q_OK;
    }
    // victim: an entry of an older graph first, else round robin; never the entry a caller up the stack
    // still reads (the expert-parallel call keeps its route across the local product)
    size_t pick = 2;
    for (size_t i = 0; i < 2; ++i)
        if ((int)i != ctx->route_pinned &&
            (!ctx->routes[i] || !ctx->routes[i]->valid || ctx->routes[i]->gen != ctx->generation)) { pick = i; break; }
    if (pick == 2) {
        pick = ctx->route_next;
        ctx->route_next ^= 1;
        if ((int)pick == ctx->route_pinned) pick ^= 1;
    }
    if (!ctx->routes[pick]) ctx->routes[pick] = new RouteEntry();
    RouteEntry &e = *ctx->routes[pick];
    e.valid = false;
    const int64_t max_tiles = (n_pairs + 7) / 8 + (n_expert < n_pairs ? n_expert : n_pairs);
    const size_t bytes = sizeof(int32_t) * (size_t)(n_pairs + 5 * 4 * max_tiles + 8 + 4096) + 64;   // + owner counts
    b200q_status st = ws_reserve(ctx, &e.buf, bytes);
    if (st != B200Q_OK) return st;
    int32_t *p = (int32_t *)e.buf.ptr;
    int32_t *pairs = p;
    int32_t *tl[5];
    for (int k = 0; k < 5; ++k) tl[k] = p + n_pairs + (size_t)k * 4 * max_tiles;
    int32_t *n_tiles = p + n_pairs + (size_t)20 * max_tiles;
    int32_t *owner_counts = n_tiles + 8;
    // counter groups: as many as fit beside the seven per-expert arrays (eight for up to ~1000 experts)
    int n_groups = 8;
    while (n_groups > 1 && sizeof(int) * (size_t)n_expert * (7 + 2 * n_groups) > 200 * 1024) n_groups >>= 1;
    const size_t smem = sizeof(int) * (size_t)n_expert * (7 + 2 * n_groups);
    if (smem > 200 * 1024) return fail(ctx, B200Q_UNSUPPORTED, "route: %d experts", n_expert);
    static bool attr_dev[B200Q_MAX_DEVICES] = {};
    bool &attr = attr_dev[ctx->device % B200Q_MAX_DEVICES];
    if (!attr) {
        B200Q_CUDA(ctx, cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr = true;
    }
    moe_route_kernel<<<1, 1024, smem, ctx->stream>>>((const uint8_t *)ids->data, ids->nb[1], n_used, n_tok, n_expert, pairs,
                                                     tl[0], tl[1], tl[2], tl[3], tl[4], n_tiles,
                                                     experts_per_owner > 0 ? owner_counts : nullptr,
                                                     experts_per_owner > 0 ? experts_per_owner : 1, n_groups,
                                                     ctx->route_skip_negative ? 1 : 0);
    B200Q_CUDA(ctx, cudaGetLastError());
    count(ctx, ST_MOE_ROUTE);
    e.ids_data = ids->data;
    e.ids_id = ids->id;
    e.ne[0] = ids->ne[0];
    e.ne[1] = ids->ne[1];
    e.nb1 = ids->nb[1];
    e.n_expert = n_expert;
    e.gen = ctx->generation;
    e.view.pairs = pairs;
    for (int k = 0; k < 4; ++k) e.view.tiles[k] = tl[k];
    e.view.tiles128 = tl[4];
    e.view.max_tiles128 = (n_pairs + 127) / 128 + (n_expert < n_pairs ? n_expert : n_pairs);
    e.view.n_tiles = n_tiles;
    e.view.max_tiles = max_tiles;
    e.view.owner_counts = owner_counts;
    e.view.slot = (int)pick;
    e.experts_per_owner = experts_per_owner;
    e.skip_negative = ctx->route_skip_negative;
    e.valid = true;
    *out = e.view;
    return B200Q_OK;
}

int moe_route_workspaces(b200q_ctx *ctx, Workspace **out, const char **names) {
    int n = 0;
    for (RouteEntry *e : ctx->routes)
        if (e) { out[n] = &e->buf; names[n++] = "route tables"; }
    return n;
}

void moe_free(b200q_ctx *ctx) {
    for (RouteEntry *&e : ctx->routes) {
        if (e) {
            ws_release(&e->buf);
            delete e;
            e = nullptr;
        }
    }
}

}  // namespace b200q
