// ep_agree.h -- what every rank of an expert-parallel call concludes from the ranks' status words.
//
// The NCCL form of b200q_mul_mat_id_ep is a sequence of collectives. A rank that found a rank-local error
// (a refused shape, no memory for its scratch, a failed launch) must not leave alone: the others would wait
// in the next collective for a peer that never arrives. So the ranks exchange a status word beside the
// per-owner counts (and again before the dispatch and before the combine) and all leave together, the
// failing rank with its own error, the others with B200Q_PEER_FAILED. This header is the decision rule, plain
// host C++ so that the host replay can test it without a communicator. The reference has no multi-GPU
// mode; this has no counterpart there.
#pragma once

#include <stdint.h>

namespace b200q {

// records: G records of `stride` int32 each, the status word at index `status_at` of a record.
// Returns 0 when every rank reported 0; else the own status when it is not 0; else `peer_failed`, with the
// lowest failing rank in *who.
inline int ep_agree_decide(const int32_t *records, int G, int stride, int status_at, int rank, int peer_failed, int *who) {
    int first_bad = -1;
    for (int p = 0; p < G; ++p)
        if (records[(size_t)p * stride + status_at] != 0 && first_bad < 0) first_bad = p;
    if (who) *who = first_bad;
    if (first_bad < 0) return 0;
    const int own = records[(size_t)rank * stride + status_at];
    return own != 0 ? own : peer_failed;
}

}  // namespace b200q
