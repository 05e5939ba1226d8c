// ep_peer.cuh -- expert-parallel dispatch and combine over peer memory (NVLink / NVSwitch), device-initiated.
//
// Every rank owns a "symmetric region" that all ranks have mapped (cudaIpc, exchanged in b200q_ep_reserve):
//     x      [G source ranks][cap pairs][K]  f32   activation rows received for this rank's experts
//     e      [G][cap]                        i32   the pair's expert, as an index into this rank's experts
//     y      [G owner ranks][cap][M]         f32   result rows coming back for this rank's own pairs
//     flags  2 x [G] + 2 x [G]               u64   (sequence number << 32 | count), by parity of the sequence number
// One MUL_MAT_ID over experts split across G ranks is then four small kernels around the local product, all
// enqueued on the context's stream without any host synchronisation (the sequence is capturable):
//   dispatch   (source)  pair number s of the route-sorted list (sorted by expert = grouped by owner) goes to
//                        region [this rank] of its owner, position s - (first pair of that owner); the last
//                        block publishes (sequence, count) to every owner after a system-wide fence;
//   wait+build (owner)   waits until every source has published, then marks the filled slots with their expert
//                        and the empty ones with -1 (the local route skips those);
//   product    (owner)   b200q_mul_mat_id over all G x cap slots as tokens with one used expert each;
//   combine    (owner)   result row of slot (r, i) goes to y region [this rank] of rank r, position i; the last
//                        block publishes the sequence number to every source;
//   unpack     (source)  waits for its owners, scatters the rows into dst, and the last block advances the
//                        sequence number.
// A rank cannot start call n+1 before every owner has finished call n (it waits for all G owners' flags, also
// those it sent nothing to), so data regions need no double buffering; the flags alternate by parity.
// gate and up of a layer read the same activation through the same ids: the second call finds the dispatch
// (and, on the owner, the route and the gathered activation) already done and only runs product, combine, unpack.
//
// Plain loads and stores to peer memory; every wait is bounded and reports through the context's error word.
// The reference has no expert-parallel mode; this has no counterpart there.
#pragma once

#include <stdint.h>

namespace b200q {

constexpr int      EP_MAX_RANKS = 8;
constexpr uint32_t EP_SPIN_LIMIT = 1u << 22;

struct EpLayout {
    int64_t cap;                      // pairs per (source, owner) region
    int64_t K, M;                     // row lengths of this call, in floats
    size_t  off_e, off_y, off_flags;  // byte offsets inside a symmetric region (x is at 0)
    int     G, rank;
    uint8_t *base[EP_MAX_RANKS];      // every rank's region as mapped here (this rank's own at [rank])
};

__device__ __forceinline__ float *ep_x(const EpLayout &L, int on, int src, int64_t i) {
    return reinterpret_cast<float *>(L.base[on]) + ((size_t)src * L.cap + (size_t)i) * L.K;
}
__device__ __forceinline__ int32_t *ep_e(const EpLayout &L, int on, int src, int64_t i) {
    return reinterpret_cast<int32_t *>(L.base[on] + L.off_e) + (size_t)src * L.cap + (size_t)i;
}
__device__ __forceinline__ float *ep_y(const EpLayout &L, int on, int owner, int64_t i) {
    return reinterpret_cast<float *>(L.base[on] + L.off_y) + ((size_t)owner * L.cap + (size_t)i) * L.M;
}
// flag words: kind 0 = activations published by source `who`, kind 1 = results published by owner `who`
__device__ __forceinline__ uint64_t *ep_flag(const EpLayout &L, int on, int kind, int parity, int who) {
    return reinterpret_cast<uint64_t *>(L.base[on] + L.off_flags) + ((size_t)kind * 2 + (size_t)parity) * EP_MAX_RANKS + who;
}
__device__ __forceinline__ void ep_store_flag(uint64_t *p, uint64_t v) {
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ep_load_flag(const uint64_t *p) {
    uint64_t v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait for a flag of this sequence number; false when it gave up: after EP_WAIT_NS, after the poll limit,
// or at once when an earlier wait of this context already gave up (its error word is set) -- a peer that has gone
// away costs the others two seconds once, not per flag and per kernel.
constexpr unsigned long long EP_WAIT_NS = 2000000000ull;
__device__ __forceinline__ bool ep_wait_flag(const uint64_t *p, uint32_t seq, uint32_t *count, const int *error_word) {
    *count = 0;
    if (error_word && *(volatile const int *)error_word) return false;
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < EP_SPIN_LIMIT; ++i) {
        const uint64_t v = ep_load_flag(p);
        if ((uint32_t)(v >> 32) == seq) {
            *count = (uint32_t)v;
            __threadfence_system();            // what the publisher wrote before the flag is read after it
            return true;
        }
        if (i > 256) __nanosleep(100);
        if ((i & 1023u) == 1023u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > EP_WAIT_NS) break;
        }
    }
    return false;
}

// which owner sorted position `pos` belongs to, and its place among that owner's pairs
__device__ __forceinline__ bool ep_owner_of(const int32_t *owner_counts, int G, int pos, int *owner, int *idx) {
    int off = 0;
    for (int o = 0; o < G; ++o) {
        const int c = owner_counts[o];
        if (pos < off + c) { *owner = o; *idx = pos - off; return true; }
        off += c;
    }
    return false;
}

// The copy kernels are persistent: a few blocks per SM walk the rows with a grid stride, one warp per row, and
// each block fences and counts itself in once at its end (a system-wide fence per row-sized block measured ten
// times slower than the copies themselves).
constexpr int EP_COPY_THREADS = 256;

// state words: [0] sequence number of the last finished call, [1..3] block counters of dispatch, combine, unpack
__global__ void __launch_bounds__(EP_COPY_THREADS)
ep_dispatch_kernel(const uint8_t *src1, size_t nb1, size_t nb2, int ne11, const uint8_t *ids, size_t ids_nb1, int n_used,
                   int n_pairs, int n_expert, int per_owner, const int32_t *pairs, const int32_t *owner_counts, EpLayout L,
                   uint32_t *state) {
    const uint32_t seq = *(volatile uint32_t *)state + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    for (int pos = blockIdx.x * wpb + warp; pos < n_pairs; pos += gridDim.x * wpb) {
        int owner = 0, idx = 0;
        if (!ep_owner_of(owner_counts, L.G, pos, &owner, &idx)) continue;
        const int p = pairs[pos], t = p / n_used, i = p - t * n_used;
        const float4 *x = reinterpret_cast<const float4 *>(src1 + (size_t)(i % ne11) * nb1 + (size_t)t * nb2);
        float4 *o = reinterpret_cast<float4 *>(ep_x(L, owner, L.rank, idx));
        for (int k = lane; k < (int)(L.K / 4); k += 32) o[k] = x[k];
        if (lane == 0) {
            const int e = min(max(reinterpret_cast<const int32_t *>(ids + (size_t)t * ids_nb1)[i], 0), n_expert - 1);
            *ep_e(L, owner, L.rank, idx) = e - owner * per_owner;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(state + 1, 1u) == gridDim.x - 1) {
            state[1] = 0;
            __threadfence_system();
            for (int o = 0; o < L.G; ++o)
                ep_store_flag(ep_flag(L, o, 0, (int)(seq & 1u), L.rank), ((uint64_t)seq << 32) | (uint32_t)owner_counts[o]);
        }
    }
}

// owner side: counts[r] = pairs received from rank r; ids_local[slot] = expert of a filled slot, -1 otherwise
__global__ void __launch_bounds__(256)
ep_wait_build_kernel(EpLayout L, const uint32_t *state, int32_t *ids_local, int32_t *counts, int *error_word) {
    __shared__ uint32_t cnt[EP_MAX_RANKS];
    __shared__ int bad;
    const uint32_t seq = *(volatile const uint32_t *)state + 1;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    if ((int)threadIdx.x < L.G) {
        uint32_t c;
        if (!ep_wait_flag(ep_flag(L, L.rank, 0, (int)(seq & 1u), threadIdx.x), seq, &c, error_word)) bad = 1;
        cnt[threadIdx.x] = c > (uint32_t)L.cap ? (uint32_t)L.cap : c;
        counts[threadIdx.x] = (int32_t)cnt[threadIdx.x];
    }
    __syncthreads();
    __threadfence_system();
    const int64_t total = (int64_t)L.G * L.cap;
    for (int64_t s = threadIdx.x; s < total; s += blockDim.x) {
        const int r = (int)(s / L.cap);
        const int64_t i = s - (int64_t)r * L.cap;
        ids_local[s] = i < (int64_t)cnt[r] ? __ldcg(ep_e(L, L.rank, r, i)) : -1;     // L2: a peer wrote it
    }
    if (threadIdx.x == 0 && bad && error_word) atomicExch(error_word, 5);
}

// owner side: out is the local product's result, one row of M floats per slot; filled slot g of all regions
// together is slot (r, i) with i below counts[r]
__global__ void __launch_bounds__(EP_COPY_THREADS)
ep_combine_kernel(const float *out, const int32_t *counts, EpLayout L, uint32_t *state) {
    const uint32_t seq = *(volatile uint32_t *)state + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    int total = 0;
    for (int r = 0; r < L.G; ++r) total += counts[r];
    for (int g = blockIdx.x * wpb + warp; g < total; g += gridDim.x * wpb) {
        int r = 0, i = 0;
        if (!ep_owner_of(counts, L.G, g, &r, &i)) continue;
        const float4 *s = reinterpret_cast<const float4 *>(out + ((size_t)r * L.cap + (size_t)i) * L.M);
        float4 *d = reinterpret_cast<float4 *>(ep_y(L, r, L.rank, i));
        for (int m = lane; m < (int)(L.M / 4); m += 32) d[m] = s[m];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(state + 2, 1u) == gridDim.x - 1) {
            state[2] = 0;
            __threadfence_system();
            for (int q = 0; q < L.G; ++q) ep_store_flag(ep_flag(L, q, 1, (int)(seq & 1u), L.rank), ((uint64_t)seq << 32) | 1u);
        }
    }
}

// source side: every block first waits for all G owners' flags (also the owners nothing was sent to, so that no
// rank runs a whole call ahead of another), then scatters rows
__global__ void __launch_bounds__(EP_COPY_THREADS)
ep_unpack_kernel2(const int32_t *pairs, const int32_t *owner_counts, int n_pairs, int n_used, float *dst, int64_t ld1,
                  int64_t ld2, EpLayout L, uint32_t *state, int *error_word) {
    __shared__ int bad;
    const uint32_t seq = *(volatile uint32_t *)state + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    if ((int)threadIdx.x < L.G) {
        uint32_t c;
        if (!ep_wait_flag(ep_flag(L, L.rank, 1, (int)(seq & 1u), threadIdx.x), seq, &c, error_word)) bad = 1;
    }
    __syncthreads();
    if (!bad) {
        for (int pos = blockIdx.x * wpb + warp; pos < n_pairs; pos += gridDim.x * wpb) {
            int owner = 0, idx = 0;
            if (!ep_owner_of(owner_counts, L.G, pos, &owner, &idx)) continue;
            const int p = pairs[pos], t = p / n_used, i = p - t * n_used;
            const float4 *s = reinterpret_cast<const float4 *>(ep_y(L, L.rank, owner, idx));
            float4 *d = reinterpret_cast<float4 *>(dst + t * ld2 + i * ld1);
            for (int m = lane; m < (int)(L.M / 4); m += 32) d[m] = __ldcg(s + m);        // L2: a peer wrote it
        }
    } else if (threadIdx.x == 0 && error_word) {
        atomicExch(error_word, 6);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(state + 3, 1u) == gridDim.x - 1) {
            state[3] = 0;
            *(volatile uint32_t *)state = seq;            // the call is over on this rank
        }
    }
}

}  // namespace b200q
