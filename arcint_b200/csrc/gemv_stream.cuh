// gemv_stream.cuh -- the decode GEMV for dense products whose rows are 16-byte aligned.
//
// HBM-bound by intent: every packed weight byte crosses HBM once for all columns. What bounds it in
// practice is instruction issue and the load/store pipe, so the kernel keeps both out of the inner loop:
//   - a row is cut into slices of 2048 weights (64 per lane) and a warp owns ONE slice for the whole
//     launch: its activation codes, scales and block sums for that slice are loaded into registers once,
//     never again. A warp holds at most four columns (the form in which the lane code of gemv_core.cuh
//     needs about 120 registers); 5..8 columns are split over two warps per slice;
//   - the S slices x 1 or 2 column halves of a row are a "group" of warps. A group takes R consecutive
//     rows at a time; the R whole rows arrive in a shared-memory ring by bulk asynchronous copies
//     (cp.async.bulk, one instruction per row, issued by one lane of the group) that complete on an
//     mbarrier; a second mbarrier per ring stage hands the space back. All warps of the group read the
//     same staged bytes, so the weights are fetched once;
//   - the R x columns partial sums of a lane are reduced across the warp by a transposing butterfly
//     (half of the values change hands at each step: 31 shuffles for 32 values instead of 160), the
//     slices' partial sums meet in shared memory and one warp of the group (they take turns) adds them
//     in a fixed order and stores the results, while the others go on with the next rows.
// Every mbarrier wait is bounded; a wait that runs out sets the context's error word and the warp ends.
//
// Stands in for the reference's kernel_mul_mv_*_q8_1 family (marfrit/arcint contrib/llama.cpp/patches/
// 0000-01-kquant-integer-dpas.patch:3882-3915) at 1..8 columns and for its few-column kernels
// (0115-opencl-few-column-int8-q4_0-q8_0-iq4.patch:904-984), without tensor cores.
#pragma once

#include "gemv_core.cuh"
#include "pdl.cuh"
#include "tc_common.cuh"
#include "peer_ar.cuh"

namespace b200q {

constexpr uint32_t GEMV_SPIN_LIMIT = 1u << 22;
constexpr int GEMV_STREAM_MAX_THREADS = 512;      // 16 warps: the compiler may use up to 128 registers per thread

// bounded wait of one thread on an mbarrier phase; false when the limit ran out
__device__ __forceinline__ bool gemv_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < GEMV_SPIN_LIMIT; ++i)
        if (tc::mbar_try(bar, parity)) return true;
    return false;
}

// Weights are read once per product: their lines are marked evict-first in L2 so that the stream does
// not push out what is read again (the quantized activation, the next product's inputs).
__device__ __forceinline__ uint64_t gemv_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void gemv_bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}

// Sum of v[i] over the 32 lanes for every i < V (V a power of two up to 32). On return v[0] of lane l
// holds the total of index l >> (5 - log2 V); lanes that share an index hold the same total.
template <int V>
__device__ __forceinline__ void warp_reduce_transposed(float (&v)[V], int lane) {
    int n = V;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        if (n > 1) {
            const int half = n / 2;
            const bool upper = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < V / 2; ++i) {
                if (i < half) {
                    const float keep = upper ? v[i + half] : v[i];
                    const float send = upper ? v[i] : v[i + half];
                    v[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, o);
                }
            }
            n = half;
        } else {
            v[0] += __shfl_xor_sync(0xFFFFFFFFu, v[0], o);
        }
    }
}

constexpr int gemv_pow2_at_least(int v) { return v <= 1 ? 1 : v <= 2 ? 2 : v <= 4 ? 4 : v <= 8 ? 8 : v <= 16 ? 16 : 32; }

// Shared memory of one group: the ring of NSETS stages of R rows, the slices' partial sums of two
// row batches in flight, and the barriers.
struct GemvGroupSmem {
    uint32_t ring, part, bar_full, bar_empty, bar_done, bar_free;   // shared-space addresses
    uint8_t *ring_ptr;
    float   *part_ptr;
};

__host__ __device__ inline int gemv_stream_slot(int row_bytes) { return ((row_bytes + 15) / 16) * 16 + 16; }
// bytes of shared memory per group of nw warps
__host__ __device__ inline size_t gemv_stream_group_smem(int row_bytes, int R, int nsets, int nw) {
    return (size_t)nsets * R * gemv_stream_slot(row_bytes) + (size_t)2 * nw * 32 * sizeof(float) + (size_t)(2 * nsets + 4) * 8;
}

// Row split over several GPUs: the product and the all-reduce of its partial results as ONE kernel. Instead of
// storing a finished partial sum to dst, a warp stores it (with the all-reduce's sequence number, peer_ar.cuh)
// into its rank's slot of EVERY rank's mapped receive buffer -- plain 8-byte stores over NVLink, issued while the
// other rows are still being computed; after its last row batch a group goes back over its outputs, polls the G
// slots of each element in its own buffer (bounded), adds them in rank order and writes dst. The last block
// advances the sequence number. nranks == 0: a plain product.
struct GemvAr {
    uint64_t *peer[PEER_AR_MAX_RANKS];
    uint32_t *state;                   // [0] sequence number of the last all-reduce, [1] blocks finished
    int       rank, nranks;
};

__device__ __forceinline__ void gemv_ar_emit(const GemvAr &ar, uint32_t seq, int e, float v) {
    const uint64_t w = peer_ar_pack(v, seq);
    const int set = (int)(seq & 1u);
    for (int p = 0; p < ar.nranks; ++p) {
        const int q = (ar.rank + p) % ar.nranks;
        asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(ar.peer[q] + peer_ar_index(set, ar.rank, e)), "l"(w) : "memory");
    }
}

// The lane's activation registers for its slice straight from the f32 activation, for the per-32 weight types
// (Q4_0, Q8_0): the lane's two 32-blocks (numbers 64 slice + lane and + 32) are whole quantization blocks, so ggml's
// block_q8_0 rule needs nothing from other lanes. Same arithmetic as quantize_q8_0_kernel, operation for operation
// (d = amax / 127, codes roundf(x * (1 / d)), the scale rounded to fp16), so the product is bit-identical to the one
// over the separately quantized activation. For small products this removes the quantizer's launch from the chain.
template <int TYPE, int NC>
__device__ __forceinline__ void gemv_quant_x(int lane, int slice, int nblk, const GemvAct &act, const int (&cols)[NC], GemvX<NC> &X) {
    static_assert(TYPE == B200Q_TYPE_Q4_0 || TYPE == B200Q_TYPE_Q8_0, "per-32 activation form only");
    const int b0 = slice * 64 + lane, b1 = b0 + 32;
    X.live = b0 < nblk;
    X.live2 = b1 < nblk;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const float *xp = act.xf + (int64_t)cols[c] * act.xf_stride;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!(u ? X.live2 : X.live)) continue;
            const float4 *p = reinterpret_cast<const float4 *>(xp + 32 * (u ? b1 : b0));
            float4 v[8];
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = __ldg(p + i);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
            }
            const float d = __fdiv_rn(amax, 127.f);
            const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;
            int w[8], sum = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int q0 = (int)roundf(__fmul_rn(v[i].x, id)), q1 = (int)roundf(__fmul_rn(v[i].y, id));
                const int q2 = (int)roundf(__fmul_rn(v[i].z, id)), q3 = (int)roundf(__fmul_rn(v[i].w, id));
                sum += q0 + q1 + q2 + q3;
                w[i] = (int)((uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24));
            }
            X.x[c][2 * u] = I4{ w[0], w[1], w[2], w[3] };
            X.x[c][2 * u + 1] = I4{ w[4], w[5], w[6], w[7] };
            float f = __half2float(__float2half_rn(d));
            int off = 0;
            if (TYPE == B200Q_TYPE_Q4_0) {
                off = -128 * sum;                      // -8 * 16 * sum(x)
                f *= 0.0625f;                          // the nibble dot is kept x16
            }
            if (u) { X.f1[c] = f; X.i1[c] = off; } else { X.f0[c] = f; X.i0[c] = off; }
        }
    }
}

// What one warp of a group does: slice `slice` of every row, columns [col0, col0 + NCW) of the launch.
// wi: the warp's index in its group of nw warps; warp 0 of the group also runs the producer side.
template <int TYPE, int NC, int NCW, int R, int NSETS, bool QX, bool AR>
__device__ __forceinline__ void gemv_stream_warp(const uint8_t *__restrict__ W, size_t row_stride, int M, int nblk,
                                                 const GemvAct &act, float *__restrict__ dst, int ldd, const GemvGroupSmem &sm,
                                                 int gg, int tg, int lane, int wi, int nw, int slice, int col0,
                                                 int *error_word, const GemvAr &ar, uint32_t seq) {
    constexpr int CW = NC > 4 ? 2 : 1;                             // warps per slice (column halves)
    typedef GemvFmt<TYPE> F;
    typedef GemvStage<TYPE> S;
    const int row_bytes = nblk * F::BLK_B;
    const int slot = gemv_stream_slot(row_bytes);
    const int n_units = (M + R - 1) / R;
    const bool leader = wi == 0;
    bool ok = true;
    const uint64_t policy = gemv_policy_evict_first();

    // producer cursor (lane 0 of the group's first warp acts): the next row batch to request
    int p_n = 0, p_set = 0;
    auto issue = [&]() {
        const int u = gg + p_n * tg;
        if (u < n_units && lane == 0) {
            // the stage's previous rows must have been released by every warp of the group
            if (p_n >= NSETS && !gemv_mbar_wait(sm.bar_empty + 8 * p_set, (uint32_t)((p_n / NSETS - 1) & 1))) ok = false;
            if (ok) {
                const int row0 = u * R, rows = min(R, M - row0);
                const uint8_t *src = W + (size_t)row0 * row_stride;
                const uint32_t d = sm.ring + p_set * (R * slot);
                tc::mbar_expect_tx(sm.bar_full + 8 * p_set, (uint32_t)row_bytes * (uint32_t)rows);
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (r < rows) gemv_bulk_g2s(d + r * slot, src + (size_t)r * row_stride, (uint32_t)row_bytes, sm.bar_full + 8 * p_set, policy);
            }
        }
        p_set = p_set + 1 == NSETS ? 0 : p_set + 1;
        ++p_n;
    };
    // The producer runs NSETS - 2 batches ahead of the consumers, not NSETS - 1: the stage it refills was
    // read one batch earlier than the newest finished one, so its wait for the other warps' release is
    // normally over before it begins and the warps of a group do not fall into lockstep.
    static_assert(NSETS >= 3, "the ring needs a stage being read, one draining and at least one in flight");
    if (leader) {
#pragma unroll
        for (int i = 0; i < NSETS - 2; ++i) issue();
    }
    // the first rows are in flight; the activation (the quantizer's output) and dst (which an earlier
    // kernel may still be using) are touched only after this
    pdl_wait();

    int cols[NCW];
#pragma unroll
    for (int c = 0; c < NCW; ++c) cols[c] = col0 + c;
    GemvX<NCW> X;
    if constexpr (QX) gemv_quant_x<TYPE, NCW>(lane, slice, nblk, act, cols, X);      // ... quantized here from the f32 activation
    else gemv_load_x<TYPE, NCW>(lane, slice, nblk, act, cols, X);                    // once: this warp's slice of every column

    constexpr int V = gemv_pow2_at_least(R * NCW);
    constexpr int SHARE = 32 / V;                                  // lanes that end up with the same value
    const int slice_off = slice * S::BYTES;
    int c_set = 0;
    for (int n = 0, u = gg; u < n_units; u += tg, ++n) {
        if (leader) issue();
        float acc[R][NCW];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < NCW; ++c) acc[r][c] = 0.f;
        ok = ok && gemv_mbar_wait(sm.bar_full + 8 * c_set, (uint32_t)((n / NSETS) & 1));
        if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
        const uint8_t *set = sm.ring_ptr + c_set * (R * slot) + slice_off;
#pragma unroll
        for (int r = 0; r < R; ++r) gemv_lane_row<TYPE, NCW>(reinterpret_cast<const uint32_t *>(set + r * slot), lane, X, acc[r]);
        __syncwarp();                                              // every lane has read the stage
        if (lane == 0) tc::mbar_arrive(sm.bar_empty + 8 * c_set);
        c_set = c_set + 1 == NSETS ? 0 : c_set + 1;

        // value index i = c * R + r, so neighbouring lanes hold neighbouring rows
        float v[V];
#pragma unroll
        for (int i = 0; i < V; ++i) v[i] = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < NCW; ++c) v[c * R + r] = acc[r][c];
        warp_reduce_transposed<V>(v, lane);
        const int i = lane / SHARE;
        if (nw == 1) {
            const int c = i / R, r = i - c * R, row = u * R + r;
            if ((lane & (SHARE - 1)) == 0 && c < NCW && row < M) {
                if (AR) gemv_ar_emit(ar, seq, (col0 + c) * M + row, v[0]);
                else dst[(size_t)(col0 + c) * ldd + row] = v[0];
            }
            continue;
        }
        // the slices meet in shared memory: part[par][warp][i]
        const int par = n & 1;
        if (n >= 2) {                                              // the batch two back has been added up and stored
            ok = gemv_mbar_wait(sm.bar_free + 8 * par, (uint32_t)((n / 2 - 1) & 1));
            if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
        }
        float *part = sm.part_ptr + (size_t)par * nw * 32;
        if ((lane & (SHARE - 1)) == 0) part[wi * 32 + i] = v[0];
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(sm.bar_done + 8 * par);
        if (wi == n % nw) {                                        // this batch's finisher
            ok = gemv_mbar_wait(sm.bar_done + 8 * par, (uint32_t)((n / 2) & 1));
            if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
            // warps of a group: wi = slice * CW + half; every lane adds up one (column, row) of a half
#pragma unroll
            for (int h = 0; h < CW; ++h) {
                const int hcol0 = h == 0 ? 0 : (NC + 1) / 2, hn = CW == 1 ? NC : (h == 0 ? (NC + 1) / 2 : NC / 2);
                const int c = lane / R, r = lane - c * R, row = u * R + r;
                if (c < hn && row < M) {
                    float t = 0.f;
                    for (int s = h; s < nw; s += CW) t += part[s * 32 + lane];
                    if (AR) gemv_ar_emit(ar, seq, (hcol0 + c) * M + row, t);
                    else dst[(size_t)(hcol0 + c) * ldd + row] = t;
                }
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(sm.bar_free + 8 * par);
        }
    }
    if (AR && ok) {
        // second pass: the group's outputs (its row batches x R rows x NC columns) are shared out over ALL lanes of ALL its
        // warps; a lane first issues the loads of the G ranks' slots of its element together, then waits (bounded) for
        // those that have not arrived, and adds them in rank order. (One lane per (column, row) of a batch, batch after
        // batch, left 30 of 32 lanes idle at one column and cost more than the all-reduce it replaced at eight ranks.)
        bool got = !(error_word && *(volatile int *)error_word);
        auto load = [](const uint64_t *p) {
            uint64_t w;
            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
            return w;
        };
        const uint64_t *mine = ar.peer[ar.rank];
        const int set = (int)(seq & 1u);
        constexpr int PER = R * NC;
        const int my_units = gg < n_units ? (n_units - gg + tg - 1) / tg : 0;
        for (int f = wi * 32 + lane; f < my_units * PER; f += nw * 32) {
            const int k = f / PER, j = f - k * PER, c = j / R, r = j - c * R, row = (gg + k * tg) * R + r;
            if (row >= M) continue;
            const int e = c * M + row;
            uint64_t w[PEER_AR_MAX_RANKS];
#pragma unroll
            for (int q = 0; q < PEER_AR_MAX_RANKS; ++q)
                if (q < ar.nranks) w[q] = load(mine + peer_ar_index(set, q, e));
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < PEER_AR_MAX_RANKS; ++q) {
                if (q < ar.nranks) {
                    if ((uint32_t)(w[q] >> 32) != seq) w[q] = peer_ar_wait(mine + peer_ar_index(set, q, e), seq, PEER_AR_SPIN_LIMIT, load, &got);
                    sum += peer_ar_value(w[q]);
                }
            }
            dst[(size_t)c * ldd + row] = sum;
        }
        if (!got && error_word) atomicExch(error_word, 4);
    }
    if (!ok && lane == 0 && error_word) atomicExch(error_word, 2);
}

// dst[m + c*ldd] = sum_k W[m][k] x_c[k] for c < NC (1..8), rows [0, M). A block holds `groups` groups of
// nslices * (NC > 4 ? 2 : 1) warps; the grid is one wave of persistent blocks and group number gg takes the
// row batches gg, gg + (all groups), ...
// MAXT, MINB: the launch bounds. The default (512 threads) caps a thread at 128 registers, which the wide Q6_K forms
// reach: they are also built for blocks of at most 128 threads, three to an SM (170 registers).
template <int TYPE, int NC, int R, int NSETS, bool QX = false, bool AR = false, int MAXT = GEMV_STREAM_MAX_THREADS, int MINB = 0>
__global__ void __launch_bounds__(MAXT, MINB)
gemv_stream_kernel(const uint8_t *__restrict__ W, size_t row_stride, int M, int nblk, GemvAct act, float *__restrict__ dst,
                   int ldd, int groups, int *__restrict__ error_word, GemvAr ar) {
    typedef GemvFmt<TYPE> F;
    constexpr int CW = NC > 4 ? 2 : 1;
    constexpr int NCA = CW == 2 ? (NC + 1) / 2 : NC, NCB = NC - NCA;
    extern __shared__ __align__(128) uint8_t smem[];
    const int nslices = (nblk + F::STAGE_BLOCKS - 1) / F::STAGE_BLOCKS, nw = nslices * CW;
    const int row_bytes = nblk * F::BLK_B, slot = gemv_stream_slot(row_bytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = warp / nw, wi = warp - g * nw;
    const int slice = wi / CW, sub = wi - slice * CW;
    const size_t gbytes = (gemv_stream_group_smem(row_bytes, R, NSETS, nw) + 15) / 16 * 16;
    GemvGroupSmem sm;
    sm.ring_ptr = smem + g * gbytes;
    sm.part_ptr = reinterpret_cast<float *>(sm.ring_ptr + (size_t)NSETS * R * slot);
    sm.ring = tc::smem_u32(sm.ring_ptr);
    sm.part = tc::smem_u32(sm.part_ptr);
    sm.bar_full = sm.part + 2 * nw * 32 * (uint32_t)sizeof(float);
    sm.bar_empty = sm.bar_full + 8 * NSETS;
    sm.bar_done = sm.bar_empty + 8 * NSETS;
    sm.bar_free = sm.bar_done + 16;
    if (wi == 0 && lane == 0) {
#pragma unroll
        for (int i = 0; i < NSETS; ++i) {
            tc::mbar_init(sm.bar_full + 8 * i, 1);
            tc::mbar_init(sm.bar_empty + 8 * i, (uint32_t)nw);
        }
        tc::mbar_init(sm.bar_done, (uint32_t)nw);
        tc::mbar_init(sm.bar_done + 8, (uint32_t)nw);
        tc::mbar_init(sm.bar_free, 1);
        tc::mbar_init(sm.bar_free + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int gg = blockIdx.x * groups + g, tg = gridDim.x * groups;
    uint32_t seq = 0;
    if (AR) seq = *(volatile uint32_t *)ar.state + 1;
    if (g < groups) {
        // one copy of the warp code when both column halves are equally wide (8 and 6 columns): the instruction
        // cache is a measured bottleneck of the wide forms
        if (CW == 1 || NCA == NCB)
            gemv_stream_warp<TYPE, NC, NCA, R, NSETS, QX, AR>(W, row_stride, M, nblk, act, dst, ldd, sm, gg, tg, lane, wi, nw, slice, sub * NCA,
                                                              error_word, ar, seq);
        else if (sub == 0)
            gemv_stream_warp<TYPE, NC, NCA, R, NSETS, QX, AR>(W, row_stride, M, nblk, act, dst, ldd, sm, gg, tg, lane, wi, nw, slice, 0, error_word, ar,
                                                              seq);
        else
            gemv_stream_warp<TYPE, NC, (NCB > 0 ? NCB : 1), R, NSETS, QX, AR>(W, row_stride, M, nblk, act, dst, ldd, sm, gg, tg, lane, wi, nw,
                                                                              slice, NCA, error_word, ar, seq);
    }
    if (AR) {
        // the last block to finish advances the all-reduce's sequence number (for the next launch)
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(ar.state + 1, 1u) == gridDim.x - 1) {
                ar.state[1] = 0;
                *(volatile uint32_t *)ar.state = seq;
            }
        }
    }
    // this block's rows are done: once every block is here the next kernel of the stream may be scheduled
    pdl_trigger();
}

}  // namespace b200q
