// peer_ar.cuh -- the one-shot all-reduce of small f32 vectors over peer memory (NVLink / NVSwitch).
//
// A row-split decode product leaves every rank with a partial result of a few thousand floats; NCCL's
// all-reduce of 16 KB costs more than the GEMV that made it. Here every rank holds a receive buffer that
// all peers have mapped (cudaIpc handles exchanged once at b200q_tp_init). One kernel per all-reduce:
//   1. every rank stores its vector into slot [set][its rank] of EVERY rank's buffer (its own included)
//      with plain 8-byte stores: the low word is the float, the high word the sequence number of this
//      all-reduce. An aligned 8-byte store arrives whole, so a reader that sees the sequence number
//      sees the float next to it -- no fence, no separate flag (the "LL" idea of collective libraries);
//   2. it then reads the nranks slots of its own buffer, polling each 8-byte element until its high word
//      is the sequence number, and adds the floats in rank order (the same order on every rank: results
//      are identical across ranks and from run to run).
// Two sets of slots alternate, so a fast rank's next all-reduce does not overwrite what a slow rank is
// still reading: a rank cannot finish all-reduce n+1 before every rank has begun it, i.e. has finished n.
// The sequence number lives in device memory and is advanced by the kernel itself (the last block to
// finish), so a captured CUDA graph replays correctly.
//
// Plain loads and stores to peer memory only: no TMA, no tensor map over peer memory, no multicast.
// Every poll loop is bounded; when it runs out the rank sets its context's error word, takes the value
// it has and goes on, so nothing hangs a GPU (the host sees B200Q_TIMEOUT at its next synchronize).
// The reference has no tensor-parallel mode; this has no counterpart there.
#pragma once

#include <stdint.h>

#include "intrin.cuh"

namespace b200q {

constexpr int      PEER_AR_MAX_RANKS = 8;
constexpr int      PEER_AR_MAX_FLOATS = 64 * 1024;          // per all-reduce: 8 decode columns of 8192 rows
constexpr uint32_t PEER_AR_SPIN_LIMIT = 1u << 22;
// a wait on another GPU also ends after this long, and once one wait of a context has given up (its error word is
// set) no later wait of that context spins at all: a peer that has gone away costs the others two seconds once,
// not per element and per kernel
constexpr unsigned long long PEER_WAIT_NS = 2000000000ull;

// element e of rank r's slot in set s of a receive buffer (8-byte elements)
B200Q_HD size_t peer_ar_index(int set, int r, int e) {
    return ((size_t)set * PEER_AR_MAX_RANKS + (size_t)r) * PEER_AR_MAX_FLOATS + (size_t)e;
}
constexpr size_t PEER_AR_BUFFER_BYTES = (size_t)2 * PEER_AR_MAX_RANKS * PEER_AR_MAX_FLOATS * 8;

B200Q_HD uint64_t peer_ar_pack(float v, uint32_t seq) {
    uint32_t bits;
    memcpy(&bits, &v, 4);
    return ((uint64_t)seq << 32) | bits;
}
B200Q_HD float peer_ar_value(uint64_t w) {
    const uint32_t bits = (uint32_t)w;
    float v;
    memcpy(&v, &bits, 4);
    return v;
}

// Polls *slot until its sequence word is `seq`, at most `limit` times. Returns the element as last read and
// sets *ok to false when the limit ran out (the wait gave up). `load` is how the caller reads 8 bytes that
// another GPU writes (a volatile load on the device, a plain read in the host replay).
template <typename Load>
B200Q_HD uint64_t peer_ar_wait(const uint64_t *slot, uint32_t seq, uint32_t limit, Load load, bool *ok) {
    uint64_t w = load(slot);
#ifdef __CUDA_ARCH__
    unsigned long long t0 = 0;
    for (uint32_t i = 0; (uint32_t)(w >> 32) != seq && i < limit && *ok; ++i) {
        w = load(slot);
        if ((i & 1023u) == 1023u) {                              // the clock every thousand polls
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > PEER_WAIT_NS) break;
        }
    }
#else
    for (uint32_t i = 0; (uint32_t)(w >> 32) != seq && i < limit; ++i) w = load(slot);
#endif
    if ((uint32_t)(w >> 32) != seq) *ok = false;
    return w;
}

}  // namespace b200q
