// gemv_kernel.cuh -- the decode GEMV kernel template (see gemv.cu for the description).
#pragma once

#include "gemv_core.cuh"
#include "pdl.cuh"

namespace b200q {

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// index of column c of the second column group (0 when there is no second group, so the
// never-used instantiation still indexes inside its arrays)
template <int NCG, int NC2> __host__ __device__ constexpr int second_group_index(int c) {
    return (NC2 > 0 && c < NC2) ? NCG + c : 0;
}

// MUL_MAT_ID view of the same kernel: the "columns" of a unit are the pairs of one route
// tile (all of one expert), so a unit is (tile, row batch) and its weight base, activation
// columns and output addresses come from the tile. Pair p = t*n_used + i has expert
// ids[t][i], activation column (i % ne11) + t*ne11 and output dst + t*ld2 + i*ld1
// (the reference's ID_PROLOGUE, marfrit/arcint contrib/llama.cpp/patches/
// 0000-01-kquant-integer-dpas.patch:3917-3934).
struct GemvId {
    const int32_t *tiles;      // [n][4]: expert, first pair, count, - ; NULL: direct mode, tile p = pair p
    const int32_t *n_tiles;    // device scalar (direct mode: unused)
    const int32_t *pairs;      // pairs sorted by expert (direct mode: unused)
    const uint8_t *ids;        // direct mode: ids[t][i] at ids + t*ids_stride + 4*i
    size_t         ids_stride;
    int            n_pairs, n_expert;
    int            n_used, ne11;
    size_t         expert_stride;   // bytes between expert matrices
    int64_t        ld1, ld2;        // dst strides of slot i and token t, in floats
};

// One warp owns a batch of B consecutive rows at a time and walks the row in stages of 2048
// weights. For each stage it holds the activation side (64 codes per lane and column, scales,
// block sums) in registers and runs the B staged row chunks against it, so the activation
// loads, address arithmetic and pipeline bookkeeping are paid once per B rows. The chunks
// arrive through a per-warp ring of NSETS sets of B slots filled with 16-byte asynchronous
// copies: NSETS-1 sets are in flight while the current one is consumed. More
// than four columns are taken as two column groups over the same staged set.
template <int TYPE, int NC, int B, int WARPS, int NSETS, bool ALIGNED, bool ID>
__global__ void __launch_bounds__(WARPS * 32)
gemv_kernel(const uint8_t *__restrict__ W, size_t row_stride, int M, int nblk, GemvAct act,
            float *__restrict__ dst, int ldd, GemvId id) {
    typedef GemvFmt<TYPE> F;
    typedef GemvStage<TYPE> S;
    constexpr int NCG = NC <= 4 ? NC : (NC + 1) / 2;      // columns of the first group
    constexpr int NC2 = NC - NCG;                         // columns of the second group (0: none)
    constexpr int N2 = NC2 > 0 ? NC2 : 1;
    constexpr int PIECES = (S::BYTES + 511) / 512;        // 16-byte copies per lane and chunk
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t *ring = smem + warp * (NSETS * B * S::SLOT);
    if (ID) pdl_wait();                  // the route (tile lists, counts) comes from the kernel before

    const int row_bytes = nblk * F::BLK_B;
    const int nstages = (nblk + F::STAGE_BLOCKS - 1) / F::STAGE_BLOCKS;
    const int n_bt = (M + B - 1) / B;                     // row batches per matrix
    const bool direct = ID && id.tiles == nullptr;
    const int n_units = ID ? (direct ? id.n_pairs : __ldg(id.n_tiles)) * n_bt : n_bt;
    // direct mode: the expert of pair p, read from ids and clamped like the reference's route kernel
    auto pair_expert = [&](int p) {
        const int t = p / id.n_used, i = p - t * id.n_used;
        const int e = __ldg(reinterpret_cast<const int32_t *>(id.ids + (size_t)t * id.ids_stride) + i);
        return min(max(e, 0), id.n_expert - 1);
    };
    const int gw = blockIdx.x * WARPS + warp, tw = gridDim.x * WARPS;

    // producer cursor: unit and stage of the next set to fetch, and its place in the ring
    int p_u = gw, p_s = 0, p_set = 0;
    auto issue = [&]() {
        if (p_u < n_units) {
            const int off = p_s * S::BYTES;
            const int bytes = min((int)S::BYTES, row_bytes - off);
            const int row0 = (ID ? p_u % n_bt : p_u) * B;
            const uint8_t *src = W + (size_t)row0 * row_stride + off;
            if (ID) src += (size_t)(direct ? pair_expert(p_u / n_bt) : __ldg(id.tiles + 4 * (p_u / n_bt))) * id.expert_stride;
            uint8_t *d = ring + p_set * (B * S::SLOT);
#pragma unroll
            for (int r = 0; r < B; ++r) {
                if (row0 + r < M) {              // rows past the end keep stale bytes; never stored
                    if (ALIGNED) {
#pragma unroll
                        for (int j = 0; j < PIECES; ++j) {
                            const int b = lane * 16 + j * 512;
                            if (b < bytes) cp_async16(d + b, src + b);
                        }
                    } else {
                        for (int b = lane * 2; b < bytes; b += 64)
                            *reinterpret_cast<uint16_t *>(d + b) = *reinterpret_cast<const uint16_t *>(src + b);
                    }
                }
                src += row_stride;
                d += S::SLOT;
            }
            if (++p_s == nstages) { p_s = 0; p_u += tw; }
        }
        p_set = p_set + 1 == NSETS ? 0 : p_set + 1;
        cp_async_commit();
    };

    float acc[B][NC];
#pragma unroll
    for (int i = 0; i < NSETS - 1; ++i) issue();
    // the first weight stages are in flight; the activation (the quantizer's output) and dst (which
    // an earlier kernel may still be writing or reading) are touched only after this
    if (!ID) pdl_wait();
    int c_set = 0;
    for (int u = gw; u < n_units; u += tw) {
        // this unit's columns: where each reads its activation and writes its result
        int cols[NC];
        int64_t outs[NC];
        int ncol = NC;
        if (ID) {
            const int tile = u / n_bt;
            const int first = direct ? tile : __ldg(id.tiles + 4 * tile + 1);
            ncol = direct ? 1 : __ldg(id.tiles + 4 * tile + 2);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int p = direct ? tile : __ldg(id.pairs + first + min(c, ncol - 1));   // short tiles repeat their last pair
                const int t = p / id.n_used, i = p - t * id.n_used;
                cols[c] = (i % id.ne11) + t * id.ne11;
                outs[c] = t * id.ld2 + i * id.ld1;
            }
        } else {
#pragma unroll
            for (int c = 0; c < NC; ++c) { cols[c] = c; outs[c] = (int64_t)c * ldd; }
        }
        int cols1[NCG], cols2[N2];
#pragma unroll
        for (int c = 0; c < NCG; ++c) cols1[c] = cols[c];
#pragma unroll
        for (int c = 0; c < N2; ++c) cols2[c] = cols[second_group_index<NCG, NC2>(c)];
#pragma unroll
        for (int r = 0; r < B; ++r)
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
        for (int s = 0; s < nstages; ++s) {
            __syncwarp();                    // every lane is done with the set about to be refilled
            issue();
            cp_async_wait<NSETS - 1>();      // all but the NSETS-1 newest sets have landed
            __syncwarp();
            const uint8_t *set = ring + c_set * (B * S::SLOT);
            c_set = c_set + 1 == NSETS ? 0 : c_set + 1;
            {
                GemvX<NCG> X;
                gemv_load_x<TYPE, NCG>(lane, s, nblk, act, cols1, X);
#pragma unroll
                for (int r = 0; r < B; ++r) {
                    float a[NCG];
#pragma unroll
                    for (int c = 0; c < NCG; ++c) a[c] = acc[r][c];
                    gemv_lane_row<TYPE, NCG>(reinterpret_cast<const uint32_t *>(set + r * S::SLOT), lane, X, a);
#pragma unroll
                    for (int c = 0; c < NCG; ++c) acc[r][c] = a[c];
                }
            }
            if (NC2 > 0) {
                GemvX<N2> X;
                gemv_load_x<TYPE, N2>(lane, s, nblk, act, cols2, X);
#pragma unroll
                for (int r = 0; r < B; ++r) {
                    float a[N2];
#pragma unroll
                    for (int c = 0; c < N2; ++c) a[c] = acc[r][second_group_index<NCG, NC2>(c)];
                    gemv_lane_row<TYPE, N2>(reinterpret_cast<const uint32_t *>(set + r * S::SLOT), lane, X, a);
#pragma unroll
                    for (int c = 0; c < N2; ++c)
                        if (c < NC2) acc[r][second_group_index<NCG, NC2>(c)] = a[c];
                }
            }
        }
        const int row0 = (ID ? u % n_bt : u) * B;
#pragma unroll
        for (int r = 0; r < B; ++r)
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float v = acc[r][c];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                if (lane == 0 && row0 + r < M && c < ncol) dst[outs[c] + row0 + r] = v;
            }
    }
    // this block's work is done: once every block is here the next kernel of the stream may be
    // scheduled (any earlier and its blocks would take this wave's places on the SMs)
    pdl_trigger();
    cp_async_wait<0>();
}

}  // namespace b200q
