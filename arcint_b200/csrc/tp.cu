// tp.cu -- the exchanges the multi-GPU splits of the path need, over NCCL (NVLink 5 /
// NVSwitch): all-reduce of the f32 partial results of a row (K) split, all-gather of the
// row blocks of a column (output-feature) split, and the variable all-to-all of expert
// parallelism (dispatch of routed activations to the ranks that own the experts, combine of
// their results). One process per GPU; a context joins a communicator from a 128-byte id
// made by rank 0 and handed over by whatever launcher the caller uses.
//
// The reference has no tensor- or expert-parallel mode (its only multi-device mode is a
// layer split through ggml's scheduler, lines 782-788 of the design notes at the root of marfrit/arcint), so there is no
// reference behaviour to match here beyond the single-GPU op result.
//
// NCCL is opened at run time (dlopen "libnccl.so.2"): a single-GPU user never needs it, and a
// process that already carries an NCCL (PyTorch's) shares that copy instead of loading a
// second one. One kernel here touches peers' memory itself: the one-shot all-reduce of decode-sized
// vectors (peer_ar.cuh), with plain loads and stores; every other byte crosses in NCCL.
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "common.cuh"
#include "pdl.cuh"
#include "peer_ar.cuh"
#include "ep_peer.cuh"
#include "ep_agree.h"

namespace b200q {

struct Nccl {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

static Nccl *nccl_api(std::string *err) {
    static Nccl api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.lib) api.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (api.lib) {
#define B200Q_SYM(name) *(void **)(&api.name) = dlsym(api.lib, "nccl" #name)
            B200Q_SYM(GetUniqueId); B200Q_SYM(CommInitRank); B200Q_SYM(CommDestroy); B200Q_SYM(CommAbort);
            B200Q_SYM(CommGetAsyncError); B200Q_SYM(AllReduce); B200Q_SYM(AllGather); B200Q_SYM(Send); B200Q_SYM(Recv);
            B200Q_SYM(GroupStart); B200Q_SYM(GroupEnd); B200Q_SYM(GetErrorString);
#undef B200Q_SYM
        }
    }
    if (!api.lib || !api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.AllGather || !api.Send || !api.Recv ||
        !api.GroupStart || !api.GroupEnd) {
        if (err) *err = api.lib ? "libnccl.so.2 lacks a needed symbol" : "libnccl.so.2 not found";
        return nullptr;
    }
    return &api;
}

struct TpState {
    ncclComm_t comm = nullptr;
    int rank = 0, nranks = 1;
    // one-shot all-reduce over peer memory (peer_ar.cuh): this rank's receive buffer, the peers' buffers as
    // mapped into this process, and the device words the kernel keeps its sequence number and block count in
    bool      peer_ok = false;
    uint64_t *ar_local = nullptr;
    uint64_t *ar_peer[PEER_AR_MAX_RANKS] = {};
    uint32_t *ar_state = nullptr;            // [0] sequence number of the last all-reduce, [1] blocks finished
    // status agreement of the NCCL form of expert parallelism (ep_agree.h): G gathered records of G counts and a
    // status word, then this rank's own record; allocated with the communicator so that no later failure can keep a
    // rank out of the agreement
    int32_t  *agree_dev = nullptr;
    int32_t   agree_host = 0;                // the status word on its way to the device
    // expert parallelism over peer memory (ep_peer.cuh), after b200q_ep_reserve
    bool      ep_ok = false;
    int64_t   ep_cap = 0, ep_k = 0, ep_m = 0;          // reserved: pairs per region, longest rows in floats
    size_t    ep_off_e = 0, ep_off_y = 0, ep_off_flags = 0;
    uint8_t  *ep_local = nullptr, *ep_peer[EP_MAX_RANKS] = {};
    float    *ep_out = nullptr;              // local product's results, one row per slot
    int32_t  *ep_ids = nullptr, *ep_counts = nullptr;
    uint32_t *ep_state = nullptr;
    // what the owners hold from this rank's last dispatch (gate and up of a layer share it)
    struct { const void *src1 = nullptr, *src1_id = nullptr, *ids = nullptr, *ids_id = nullptr; uint64_t gen = 0; int64_t ne[4] = {0, 0, 0, 0};
             size_t nb[4] = {0, 0, 0, 0}; uint64_t private_gen = 0; } ep_sent;
};

struct PeerArArgs {
    uint64_t *peer[PEER_AR_MAX_RANKS];       // every rank's receive buffer (this rank's own at [rank])
    int       rank, nranks;
};

// One all-reduce: buf[0..count) += the other ranks' buf, in place, the same sum on every rank.
__global__ void __launch_bounds__(512)
peer_allreduce_kernel(float *__restrict__ buf, int count, PeerArArgs a, uint32_t *state, int *error_word) {
    pdl_wait();                                                   // buf comes from the kernel before
    const uint32_t seq = *(volatile uint32_t *)state + 1;
    const int set = (int)(seq & 1u);
    const int stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;
    for (int e = first; e < count; e += stride) {
        const uint64_t w = peer_ar_pack(buf[e], seq);
        for (int p = 0; p < a.nranks; ++p) {
            const int q = (a.rank + p) % a.nranks;                // ranks start on different peers
            asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(a.peer[q] + peer_ar_index(set, a.rank, e)), "l"(w) : "memory");
        }
    }
    // a context whose earlier wait gave up does not wait again (the host has not yet looked at the error word)
    bool ok = !(error_word && *(volatile int *)error_word);
    auto load = [](const uint64_t *p) {
        uint64_t v;
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
        return v;
    };
    const uint64_t *mine = a.peer[a.rank];
    for (int e = first; e < count; e += stride) {
        float sum = 0.f;
        for (int r = 0; r < a.nranks; ++r)
            sum += peer_ar_value(peer_ar_wait(mine + peer_ar_index(set, r, e), seq, PEER_AR_SPIN_LIMIT, load, &ok));
        buf[e] = sum;
    }
    if (!ok && error_word) atomicExch(error_word, 4);
    // the last block to finish advances the sequence number for the next all-reduce (a later launch)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(state + 1, 1u) == gridDim.x - 1) {
            state[1] = 0;
            *(volatile uint32_t *)state = seq;
        }
    }
    pdl_trigger();
}

#define B200Q_NCCL(ctx, api, expr)                                                                     \
    do {                                                                                               \
        ncclResult_t r_ = (expr);                                                                      \
        if (r_ != ncclSuccess)                                                                         \
            return fail((ctx), B200Q_NCCL_ERROR, "%s: %s", #expr,                                      \
                        (api)->GetErrorString ? (api)->GetErrorString(r_) : "nccl error");             \
    } while (0)

static void peer_ar_close(b200q_ctx *ctx, TpState *tp) {
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int p = 0; p < tp->nranks && p < PEER_AR_MAX_RANKS; ++p)
        if (p != tp->rank && tp->ar_peer[p]) cudaIpcCloseMemHandle(tp->ar_peer[p]);
    if (tp->ar_local) cudaFree(tp->ar_local);
    if (tp->ar_state) cudaFree(tp->ar_state);
    tp->ar_local = nullptr;
    tp->ar_state = nullptr;
    tp->peer_ok = false;
}

// Maps every rank's receive buffer into every rank (cudaIpc handles travel through one NCCL all-gather).
// The fast path is switched on only when every rank mapped every peer; otherwise all ranks stay on NCCL.
static void peer_ar_setup(b200q_ctx *ctx, TpState *tp, Nccl *api) {
    const char *off = getenv("B200Q_NO_PEER_AR");
    if ((off && off[0] == '1') || tp->nranks < 2 || tp->nranks > PEER_AR_MAX_RANKS) return;
    const int G = tp->nranks;
    bool mine = cudaMalloc(&tp->ar_local, PEER_AR_BUFFER_BYTES) == cudaSuccess &&
                cudaMemset(tp->ar_local, 0, PEER_AR_BUFFER_BYTES) == cudaSuccess &&
                cudaMalloc(&tp->ar_state, 2 * sizeof(uint32_t)) == cudaSuccess &&
                cudaMemset(tp->ar_state, 0, 2 * sizeof(uint32_t)) == cudaSuccess;
    cudaIpcMemHandle_t h;
    memset(&h, 0, sizeof(h));
    if (mine) mine = cudaIpcGetMemHandle(&h, tp->ar_local) == cudaSuccess;
    // record: [handle 64 B][ok 1 B] padded to 80 bytes per rank
    constexpr size_t REC = 80;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed as 64 bytes");
    std::vector<uint8_t> all(REC * G), rec(REC, 0);
    memcpy(rec.data(), &h, 64);
    rec[64] = mine ? 1 : 0;
    uint8_t *d = nullptr;
    bool ok = cudaMalloc(&d, REC * (G + 1)) == cudaSuccess;
    auto gather = [&]() {
        return ok && cudaMemcpyAsync(d + REC * G, rec.data(), REC, cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
               api->AllGather(d + REC * G, d, REC, ncclInt8, tp->comm, ctx->stream) == ncclSuccess &&
               cudaMemcpyAsync(all.data(), d, REC * G, cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess &&
               cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    };
    bool agreed = gather();
    for (int p = 0; agreed && p < G; ++p) agreed = all[REC * p + 64] == 1;
    bool mapped = agreed;
    if (agreed) {
        for (int p = 0; p < G && mapped; ++p) {
            if (p == tp->rank) { tp->ar_peer[p] = tp->ar_local; continue; }
            cudaIpcMemHandle_t hp;
            memcpy(&hp, all.data() + REC * p, 64);
            void *ptr = nullptr;
            mapped = cudaIpcOpenMemHandle(&ptr, hp, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
            tp->ar_peer[p] = (uint64_t *)ptr;
        }
        if (!mapped) cudaGetLastError();                           // a refused mapping is not a sticky error
    }
    // second round: did every rank map every peer?
    rec[64] = mapped ? 1 : 0;
    bool all_mapped = gather();
    for (int p = 0; all_mapped && p < G; ++p) all_mapped = all[REC * p + 64] == 1;
    if (d) cudaFree(d);
    tp->peer_ok = all_mapped;
    if (!all_mapped) peer_ar_close(ctx, tp);
}

static void ep_close(b200q_ctx *ctx, TpState *tp) {
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int p = 0; p < tp->nranks && p < EP_MAX_RANKS; ++p)
        if (p != tp->rank && tp->ep_peer[p]) cudaIpcCloseMemHandle(tp->ep_peer[p]);
    for (int p = 0; p < EP_MAX_RANKS; ++p) tp->ep_peer[p] = nullptr;
    if (tp->ep_local) cudaFree(tp->ep_local);
    if (tp->ep_out) cudaFree(tp->ep_out);
    if (tp->ep_ids) cudaFree(tp->ep_ids);
    if (tp->ep_state) cudaFree(tp->ep_state);
    tp->ep_local = nullptr;
    tp->ep_out = nullptr;
    tp->ep_ids = nullptr;
    tp->ep_state = nullptr;
    tp->ep_ok = false;
}

void tp_free(b200q_ctx *ctx) {
    TpState *tp = (TpState *)ctx->tp;
    if (!tp) return;
    ep_close(ctx, tp);
    peer_ar_close(ctx, tp);
    if (tp->agree_dev) cudaFree(tp->agree_dev);
    Nccl *api = nccl_api(nullptr);
    if (api && tp->comm && api->CommDestroy) api->CommDestroy(tp->comm);
    delete tp;
    ctx->tp = nullptr;
}

static b200q_status tp_get(b200q_ctx *ctx, TpState **tp, Nccl **api) {
    if (!ctx) return B200Q_INVALID;
    *tp = (TpState *)ctx->tp;
    if (!*tp || !(*tp)->comm) return fail(ctx, B200Q_INVALID, "b200q_tp_init was not called on this context");
    std::string err;
    *api = nccl_api(&err);
    if (!*api) return fail(ctx, B200Q_NCCL_ERROR, "%s", err.c_str());
    return B200Q_OK;
}

}  // namespace b200q

using namespace b200q;

extern "C" {

b200q_status b200q_tp_unique_id(void *id128) {
    if (!id128) return B200Q_INVALID;
    Nccl *api = nccl_api(nullptr);
    if (!api) return B200Q_NCCL_ERROR;
    static_assert(sizeof(ncclUniqueId) == 128, "the id is passed as 128 bytes");
    ncclUniqueId id;
    if (api->GetUniqueId(&id) != ncclSuccess) return B200Q_NCCL_ERROR;
    memcpy(id128, &id, 128);
    return B200Q_OK;
}

b200q_status b200q_tp_init(b200q_ctx *ctx, const void *id128, int rank, int nranks) {
    if (!ctx || !id128 || nranks < 1 || rank < 0 || rank >= nranks) return B200Q_INVALID;
    if (ctx->tp) return fail(ctx, B200Q_INVALID, "the context already belongs to a communicator");
    std::string err;
    Nccl *api = nccl_api(&err);
    if (!api) return fail(ctx, B200Q_NCCL_ERROR, "%s", err.c_str());
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    TpState *tp = new TpState();
    tp->rank = rank;
    tp->nranks = nranks;
    ncclResult_t r = api->CommInitRank(&tp->comm, nranks, id, rank);
    if (r != ncclSuccess) {
        delete tp;
        return fail(ctx, B200Q_NCCL_ERROR, "ncclCommInitRank: %s", api->GetErrorString ? api->GetErrorString(r) : "error");
    }
    if (cudaMalloc(&tp->agree_dev, sizeof(int32_t) * (size_t)(nranks + 1) * (nranks + 1)) != cudaSuccess) {
        cudaGetLastError();
        if (api->CommDestroy) api->CommDestroy(tp->comm);
        delete tp;
        return fail(ctx, B200Q_NO_MEMORY, "status records of %d ranks", nranks);
    }
    ctx->tp = tp;
    peer_ar_setup(ctx, tp, api);
    return B200Q_OK;
}

b200q_status b200q_tp_rank(const b200q_ctx *ctx, int *rank, int *nranks) {
    if (!ctx || !ctx->tp) return B200Q_INVALID;
    const TpState *tp = (const TpState *)ctx->tp;
    if (rank) *rank = tp->rank;
    if (nranks) *nranks = tp->nranks;
    return B200Q_OK;
}

// Which slice of `total` rank `rank` of `nranks` owns, in units of `unit` (rows: 1; K of a row
// split: the weight type's block size, so every shard is whole blocks; experts: 1). The first
// total/unit % nranks ranks get one unit more.
b200q_status b200q_tp_shard(int64_t total, int64_t unit, int nranks, int rank, int64_t *first, int64_t *count) {
    if (!first || !count || unit <= 0 || nranks < 1 || rank < 0 || rank >= nranks || total < 0 || total % unit)
        return B200Q_INVALID;
    const int64_t units = total / unit, q = units / nranks, r = units % nranks;
    *first = ((int64_t)rank * q + (rank < r ? rank : r)) * unit;
    *count = (q + (rank < r ? 1 : 0)) * unit;
    return B200Q_OK;
}

b200q_status b200q_all_reduce_f32(b200q_ctx *ctx, void *dev_buf, size_t count) {
    TpState *tp;
    Nccl *api;
    b200q_status st = tp_get(ctx, &tp, &api);
    if (st != B200Q_OK) return st;
    if (!dev_buf && count) return B200Q_INVALID;
    if (count == 0 || tp->nranks == 1) return B200Q_OK;
    // decode-sized vectors: one kernel over peer memory instead of a library collective
    if (tp->peer_ok && count <= (size_t)PEER_AR_MAX_FLOATS && (uintptr_t)dev_buf % 4 == 0) {
        PeerArArgs a;
        for (int p = 0; p < PEER_AR_MAX_RANKS; ++p) a.peer[p] = tp->ar_peer[p];
        a.rank = tp->rank;
        a.nranks = tp->nranks;
        const int threads = 512;
        int blocks = (int)((count + threads - 1) / threads);
        if (blocks > 16) blocks = 16;                             // all blocks of all ranks must be resident together: far below one wave
        B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
        B200Q_CUDA(ctx, launch_pdl(!ctx->no_pdl, peer_allreduce_kernel, dim3(blocks), dim3(threads), 0, ctx->stream, (float *)dev_buf,
                                   (int)count, a, tp->ar_state, ctx->error_word));
        B200Q_CUDA(ctx, cudaGetLastError());
        b200q::count(ctx, ST_TP_ALLREDUCE);
        b200q::count(ctx, ST_TP_ALLREDUCE_PEER);
        return B200Q_OK;
    }
    B200Q_NCCL(ctx, api, api->AllReduce(dev_buf, dev_buf, count, ncclFloat32, ncclSum, tp->comm, ctx->stream));
    b200q::count(ctx, ST_TP_ALLREDUCE);
    return B200Q_OK;
}

// Row split, decode widths: dst = sum over the ranks of src0 (this rank's K shard) x src1 (its K range), the same on
// every rank. When the shape allows (1, 2, 4 or 8 columns, rows the slice-resident GEMV takes, at most 65536 results,
// peer buffers mapped) the product and the all-reduce are ONE kernel: partial sums go straight from the GEMV's
// registers into every rank's receive buffer over NVLink and are added up by the same kernel (gemv_stream.cuh).
// Otherwise b200q_mul_mat followed by b200q_all_reduce_f32.
b200q_status b200q_mul_mat_allreduce(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1, b200q_tensor *dst) {
    TpState *tp;
    Nccl *api;
    b200q_status st = tp_get(ctx, &tp, &api);
    if (st != B200Q_OK) return st;
    if (!src0 || !src1 || !dst) return B200Q_INVALID;
    const int64_t N = src1->ne[1] * src1->ne[2] * src1->ne[3], M = src0->ne[1], K = src0->ne[0];
    const bool plain = b200q_supports(nullptr, B200Q_OP_MUL_MAT, src0, src1, nullptr, dst) == B200Q_OK && dst->ne[2] == 1 && dst->ne[3] == 1 &&
                       src1->ne[2] == 1 && src1->ne[3] == 1 && dst->nb[1] == (size_t)M * 4;      // packed [M, N] result: element c * M + m
    static const bool off = [] { const char *v = getenv("B200Q_NO_FUSED_AR"); return v && v[0] == '1'; }();
    if (plain && !off && tp->peer_ok && tp->nranks > 1 && N >= 1 && N <= 8 && M > 0 &&
        gemv_ar_shape_ok(src0->type, src0->data, src0->nb[1], M, K, (int)N, M)) {
        B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
        // small per-32 products quantize inside the kernel; the rest take the cached quantized activation
        TypeInfo ti;
        type_info(src0->type, &ti);
        const bool qx = (src0->type == B200Q_TYPE_Q4_0 || src0->type == B200Q_TYPE_Q8_0) && N <= 2 && ctx->fuse_quant_bytes > 0 &&
                        (int64_t)((size_t)(K / ti.block) * ti.bytes * (size_t)M) <= ctx->fuse_quant_bytes;
        ActView av;
        if (!qx && (st = get_decode_activation(ctx, src0->type, src1, &av)) != B200Q_OK) return st;
        st = launch_gemv_allreduce(ctx, src0->type, src0->data, src0->nb[1], M, K, qx ? nullptr : &av, src1, (int)N, (float *)dst->data, M,
                                   tp->ar_peer, tp->ar_state, tp->rank, tp->nranks);
        if (st == B200Q_OK) count(ctx, ST_TP_ALLREDUCE);
        if (st != B200Q_UNSUPPORTED) return st;
    }
    if ((st = b200q_mul_mat(ctx, src0, src1, dst)) != B200Q_OK) return st;
    if (!plain) return fail(ctx, B200Q_UNSUPPORTED, "mul_mat_allreduce needs a packed 2-D result");
    return b200q_all_reduce_f32(ctx, dst->data, (size_t)(M * N));
}

b200q_status b200q_all_gather(b200q_ctx *ctx, const void *dev_send, void *dev_recv, size_t bytes_per_rank) {
    TpState *tp;
    Nccl *api;
    b200q_status st = tp_get(ctx, &tp, &api);
    if (st != B200Q_OK) return st;
    if ((!dev_send || !dev_recv) && bytes_per_rank) return B200Q_INVALID;
    if (bytes_per_rank == 0) return B200Q_OK;
    B200Q_NCCL(ctx, api, api->AllGather(dev_send, dev_recv, bytes_per_rank, ncclInt8, tp->comm, ctx->stream));
    b200q::count(ctx, ST_TP_ALLGATHER);
    return B200Q_OK;
}

// Variable all-to-all (expert-parallel dispatch and combine): rank r's slice for peer p starts at
// send_offsets[p] bytes of dev_send and is send_bytes[p] long; what peer p sends lands at
// recv_offsets[p] of dev_recv. Host arrays of nranks entries each. One grouped send/recv.
b200q_status b200q_all_to_all_v(b200q_ctx *ctx, const void *dev_send, const size_t *send_offsets, const size_t *send_bytes,
                                void *dev_recv, const size_t *recv_offsets, const size_t *recv_bytes) {
    TpState *tp;
    Nccl *api;
    b200q_status st = tp_get(ctx, &tp, &api);
    if (st != B200Q_OK) return st;
    if (!send_offsets || !send_bytes || !recv_offsets || !recv_bytes) return B200Q_INVALID;
    B200Q_NCCL(ctx, api, api->GroupStart());
    // a group that was opened is always closed, also after a refused send or receive: the first error is kept
    ncclResult_t first = ncclSuccess;
    for (int p = 0; p < tp->nranks && first == ncclSuccess; ++p) {
        if (send_bytes[p])
            first = api->Send((const uint8_t *)dev_send + send_offsets[p], send_bytes[p], ncclInt8, p, tp->comm, ctx->stream);
        if (recv_bytes[p] && first == ncclSuccess)
            first = api->Recv((uint8_t *)dev_recv + recv_offsets[p], recv_bytes[p], ncclInt8, p, tp->comm, ctx->stream);
    }
    const ncclResult_t end = api->GroupEnd();
    if (first == ncclSuccess) first = end;
    if (first != ncclSuccess)
        return fail(ctx, B200Q_NCCL_ERROR, "all-to-all: %s", api->GetErrorString ? api->GetErrorString(first) : "nccl error");
    b200q::count(ctx, ST_EP_DISPATCH);
    return B200Q_OK;
}

// Collective: every rank calls it with the same bounds, before its expert-parallel products (and again when the
// bounds grow): the largest number of (token, expert) pairs one rank brings to a call, and the longest
// activation and result rows. It allocates the symmetric regions of ep_peer.cuh, exchanges their cudaIpc
// handles through one NCCL all-gather and maps the peers' regions. After it, b200q_mul_mat_id_ep runs without
// any host synchronisation; without it (or when a mapping was refused) the call uses NCCL send/receive.
b200q_status b200q_ep_reserve(b200q_ctx *ctx, int64_t max_pairs, int64_t max_k, int64_t max_m) {
    TpState *tp;
    Nccl *api;
    b200q_status st = tp_get(ctx, &tp, &api);
    if (st != B200Q_OK) return st;
    if (max_pairs <= 0 || max_k <= 0 || max_m <= 0 || max_k % 4 || max_m % 4) return fail(ctx, B200Q_INVALID, "ep_reserve bounds");
    const int G = tp->nranks;
    const char *off = getenv("B200Q_NO_PEER_EP");
    if ((off && off[0] == '1') || G < 2 || G > EP_MAX_RANKS) return B200Q_OK;        // stays on NCCL
    if (tp->ep_ok && max_pairs <= tp->ep_cap && max_k <= tp->ep_k && max_m <= tp->ep_m) return B200Q_OK;
    B200Q_CUDA(ctx, cudaSetDevice(ctx->device));
    ep_close(ctx, tp);
    const int64_t cap = (max_pairs + 3) / 4 * 4;
    const size_t x_bytes = (size_t)G * cap * max_k * 4, e_bytes = (size_t)G * cap * 4, y_bytes = (size_t)G * cap * max_m * 4;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    tp->ep_off_e = up(x_bytes);
    tp->ep_off_y = tp->ep_off_e + up(e_bytes);
    tp->ep_off_flags = tp->ep_off_y + up(y_bytes);
    const size_t total = tp->ep_off_flags + 4 * 2 * EP_MAX_RANKS * 8;
    bool mine = cudaMalloc(&tp->ep_local, total) == cudaSuccess &&
                cudaMemset(tp->ep_local + tp->ep_off_flags, 0, total - tp->ep_off_flags) == cudaSuccess &&
                cudaMalloc(&tp->ep_out, (size_t)G * cap * max_m * 4) == cudaSuccess &&
                cudaMalloc(&tp->ep_ids, ((size_t)G * cap + EP_MAX_RANKS) * 4) == cudaSuccess &&
                cudaMalloc(&tp->ep_state, 4 * sizeof(uint32_t)) == cudaSuccess &&
                cudaMemset(tp->ep_state, 0, 4 * sizeof(uint32_t)) == cudaSuccess;
    if (!mine) cudaGetLastError();
    tp->ep_counts = tp->ep_ids ? tp->ep_ids + (size_t)G * cap : nullptr;
    cudaIpcMemHandle_t h;
    memset(&h, 0, sizeof(h));
    if (mine) mine = cudaIpcGetMemHandle(&h, tp->ep_local) == cudaSuccess;
    constexpr size_t REC = 80;
    std::vector<uint8_t> all(REC * G), rec(REC, 0);
    memcpy(rec.data(), &h, 64);
    rec[64] = mine ? 1 : 0;
    uint8_t *d = nullptr;
    bool ok = cudaMalloc(&d, REC * (G + 1)) == cudaSuccess;
    auto gather = [&]() {
        return ok && cudaMemcpyAsync(d + REC * G, rec.data(), REC, cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
               api->AllGather(d + REC * G, d, REC, ncclInt8, tp->comm, ctx->stream) == ncclSuccess &&
               cudaMemcpyAsync(all.data(), d, REC * G, cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess &&
               cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    };
    bool agreed = gather();
    for (int p = 0; agreed && p < G; ++p) agreed = all[REC * p + 64] == 1;
    bool mapped = agreed;
    if (agreed) {
        for (int p = 0; p < G && mapped; ++p) {
            if (p == tp->rank) { tp->ep_peer[p] = tp->ep_local; continue; }
            cudaIpcMemHandle_t hp;
            memcpy(&hp, all.data() + REC * p, 64);
            void *ptr = nullptr;
            mapped = cudaIpcOpenMemHandle(&ptr, hp, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
            tp->ep_peer[p] = (uint8_t *)ptr;
        }
        if (!mapped) cudaGetLastError();
    }
    rec[64] = mapped ? 1 : 0;
    bool all_mapped = gather();
    for (int p = 0; all_mapped && p < G; ++p) all_mapped = all[REC * p + 64] == 1;
    if (d) cudaFree(d);
    if (!all_mapped) {
        ep_close(ctx, tp);
        return B200Q_OK;                                                       // every rank stays on NCCL
    }
    tp->ep_ok = true;
    tp->ep_cap = cap;
    tp->ep_k = max_k;
    tp->ep_m = max_m;
    tp->ep_sent.src1 = nullptr;
    return B200Q_OK;
}

// Expert-parallel MUL_MAT_ID. Every rank holds its own tokens (src1 [K, ne11, n_tok], ids [n_used, n_tok]
// with GLOBAL expert ids, dst [M, n_used, n_tok]) and the experts [rank * n_local, (rank + 1) * n_local)
// as src0 [K, M, n_local]; n_expert_total = n_local * nranks. After b200q_ep_reserve the exchange is
// device-initiated over peer memory (ep_peer.cuh) and the call neither synchronises nor allocates. Without it
// the call routes the local pairs by owner, exchanges the per-owner counts (one small all-gather and one host
// synchronisation: the send and receive sizes must be known on the host), sends every pair's f32 activation row
// and owner-local expert index to the owner (all-to-all), runs b200q_mul_mat_id over what it received, returns
// the result rows (all-to-all) and scatters them into dst. The local product runs under a private cache
// generation (the receive buffers are reused with other contents by the next call); the caller's caches, the
// route of `ids` among them, stay valid across the gate, up and down calls of a layer.
//
// Errors. In the NCCL form no rank leaves between collectives alone: a rank-local error (a refused argument, no
// memory for the scratch, a failed launch or local product) travels as a status word beside the counts and again
// before the dispatch and before the combine (ep_agree.h), and every rank returns from the same point -- the
// failing rank with its own error, the others with B200Q_PEER_FAILED. In the peer-memory form a rank that fails
// returns at once; the others' bounded waits for its rows run out and they report B200Q_TIMEOUT.
b200q_status b200q_mul_mat_id_ep(b200q_ctx *ctx, const b200q_tensor *src0_local, const b200q_tensor *src1,
                                 const b200q_tensor *ids, b200q_tensor *dst, int n_expert_total) {
    TpState *tp;
    Nccl *api;
    b200q_status st = tp_get(ctx, &tp, &api);
    if (st != B200Q_OK) return st;
    const int G = tp->nranks;
    int n_local = 0, n_used = 0, n_tok = 0, n_pairs = 0;
    int64_t K = 0, M = 0;
    // everything this rank can refuse by itself
    auto validate = [&]() -> b200q_status {
        if (!src0_local || !src1 || !ids || !dst) return fail(ctx, B200Q_INVALID, "expert-parallel MUL_MAT_ID: null tensor");
        if (n_expert_total <= 0 || n_expert_total % G || src0_local->ne[2] != n_expert_total / G)
            return fail(ctx, B200Q_INVALID, "experts: %d in total over %d ranks, %lld here", n_expert_total, G,
                        (long long)src0_local->ne[2]);
        if (n_expert_total > 4096 || G > 64) return fail(ctx, B200Q_UNSUPPORTED, "expert-parallel limits: 4096 experts, 64 ranks");
        if (ids->type != B200Q_TYPE_I32 || src1->type != B200Q_TYPE_F32 || dst->type != B200Q_TYPE_F32 || src1->nb[0] != 4 ||
            dst->nb[0] != 4 || (uintptr_t)src1->data % 16 || src1->nb[1] % 16 || src1->nb[2] % 16 || src1->ne[0] % 4)
            return fail(ctx, B200Q_UNSUPPORTED, "expert-parallel MUL_MAT_ID needs packed f32 activations and i32 ids");
        n_local = n_expert_total / G;
        n_used = (int)ids->ne[0];
        n_tok = (int)ids->ne[1];
        K = src0_local->ne[0];
        M = src0_local->ne[1];
        n_pairs = n_used * n_tok;
        if (src1->ne[0] != K || dst->ne[0] != M || dst->ne[1] != n_used || dst->ne[2] != n_tok ||
            (src1->ne[1] != 1 && src1->ne[1] != n_used) || src1->ne[2] != n_tok)
            return fail(ctx, B200Q_INVALID, "expert-parallel MUL_MAT_ID shapes");
        if (cudaSetDevice(ctx->device) != cudaSuccess) return fail(ctx, B200Q_CUDA_ERROR, "cudaSetDevice(%d)", ctx->device);
        return B200Q_OK;
    };
    // B200Q_EP_INJECT_FAIL=<rank>:<stage> makes that rank report a host-side error at agreement <stage> (0 counts,
    // 1 dispatch, 2 combine): how the multi-GPU test exercises the joint exit without any device fault
    auto injected = [&](int stage, b200q_status s) -> b200q_status {
        int r = -1, g = -1;
        const char *inj = getenv("B200Q_EP_INJECT_FAIL");                 // read per call: the NCCL form synchronises anyway
        if (s == B200Q_OK && inj && sscanf(inj, "%d:%d", &r, &g) == 2 && r == tp->rank && g == stage)
            return fail(ctx, B200Q_INVALID, "injected failure at stage %d", stage);
        return s;
    };
    b200q_status local = validate();

    RouteView rv;
    if (local == B200Q_OK) local = moe_route(ctx, ids, n_expert_total, &rv, n_local);
    if (tp->ep_ok) {
        if (local != B200Q_OK) return local;
        // regions are reserved: a call that does not fit them is refused here, on this rank alone, rather than sent
        // down the NCCL form while the peers run the peer-memory form
        if (!(n_pairs <= tp->ep_cap && K <= tp->ep_k && M <= tp->ep_m && K % 4 == 0 && M % 4 == 0 && (uintptr_t)dst->data % 16 == 0 &&
              dst->nb[1] % 16 == 0 && dst->nb[2] % 16 == 0 && G <= EP_MAX_RANKS))
            return fail(ctx, B200Q_INVALID, "expert-parallel call outside the reserved bounds (%lld pairs, rows %lld / %lld): b200q_ep_reserve again",
                        (long long)tp->ep_cap, (long long)tp->ep_k, (long long)tp->ep_m);
    }
    // device-initiated exchange over peer memory when the regions are reserved
    if (tp->ep_ok) {
        EpLayout L;
        L.cap = tp->ep_cap;
        L.K = K;
        L.M = M;
        L.off_e = tp->ep_off_e;
        L.off_y = tp->ep_off_y;
        L.off_flags = tp->ep_off_flags;
        L.G = G;
        L.rank = tp->rank;
        for (int p = 0; p < EP_MAX_RANKS; ++p) L.base[p] = tp->ep_peer[p];
        // B200Q_EP_TRACE=1: time the phases of this call with events and print them (synchronizes: debugging only)
        static const bool trace = [] { const char *v = getenv("B200Q_EP_TRACE"); return v && v[0] == '1'; }();
        cudaEvent_t ev[6] = {};
        int nev = 0;
        auto mark = [&]() { if (trace && nev < 6) { cudaEventCreate(&ev[nev]); cudaEventRecord(ev[nev], ctx->stream); ++nev; } };
        mark();
        // persistent copy kernels: eight rows per block at a time, at most four blocks per SM
        auto copy_blocks = [&](int64_t rows) {
            int64_t b = (rows + 7) / 8;
            const int64_t cap_b = (int64_t)ctx->sm_count * 4;
            return (unsigned)(b < 1 ? 1 : b > cap_b ? cap_b : b);
        };
        auto &sent = tp->ep_sent;
        bool cached = sent.src1 == src1->data && sent.src1_id == src1->id && sent.ids == ids->data && sent.ids_id == ids->id &&
                      sent.gen == ctx->generation;
        for (int i = 0; i < 4 && cached; ++i) cached = sent.ne[i] == src1->ne[i] && sent.nb[i] == src1->nb[i];
        if (!cached) {
            ep_dispatch_kernel<<<copy_blocks(n_pairs), EP_COPY_THREADS, 0, ctx->stream>>>(
                (const uint8_t *)src1->data, src1->nb[1], src1->nb[2], (int)src1->ne[1], (const uint8_t *)ids->data, ids->nb[1], n_used,
                n_pairs, n_expert_total, n_local, rv.pairs, rv.owner_counts, L, tp->ep_state);
            B200Q_CUDA(ctx, cudaGetLastError());
            ep_wait_build_kernel<<<1, 256, 0, ctx->stream>>>(L, tp->ep_state, tp->ep_ids, tp->ep_counts, ctx->error_word);
            B200Q_CUDA(ctx, cudaGetLastError());
            sent.src1 = src1->data; sent.src1_id = src1->id; sent.ids = ids->data; sent.ids_id = ids->id; sent.gen = ctx->generation;
            for (int i = 0; i < 4; ++i) { sent.ne[i] = src1->ne[i]; sent.nb[i] = src1->nb[i]; }
            sent.private_gen = (1ull << 62) + ++ctx->private_generation;
            count(ctx, ST_EP_DISPATCH);
        } else {
            count(ctx, ST_EP_DISPATCH_CACHED);
        }
        mark();
        // the local experts over all slots: slot = one token with one used expert (-1: empty, skipped by the route)
        const int64_t slots = (int64_t)G * L.cap;
        b200q_tensor x1, id1, y1;
        x1.id = id1.id = y1.id = nullptr;
        x1.type = B200Q_TYPE_F32; x1.data = tp->ep_local;
        x1.ne[0] = K; x1.ne[1] = 1; x1.ne[2] = slots; x1.ne[3] = 1;
        x1.nb[0] = 4; x1.nb[1] = (size_t)K * 4; x1.nb[2] = (size_t)K * 4; x1.nb[3] = (size_t)K * 4 * slots;
        id1.type = B200Q_TYPE_I32; id1.data = tp->ep_ids;
        id1.ne[0] = 1; id1.ne[1] = slots; id1.ne[2] = 1; id1.ne[3] = 1;
        id1.nb[0] = 4; id1.nb[1] = 4; id1.nb[2] = 4 * (size_t)slots; id1.nb[3] = 4 * (size_t)slots;
        y1.type = B200Q_TYPE_F32; y1.data = tp->ep_out;
        y1.ne[0] = M; y1.ne[1] = 1; y1.ne[2] = slots; y1.ne[3] = 1;
        y1.nb[0] = 4; y1.nb[1] = (size_t)M * 4; y1.nb[2] = (size_t)M * 4; y1.nb[3] = (size_t)M * 4 * slots;
        // The regions are refilled by the next dispatch, so what the local product caches about them lives under a
        // private generation: a new one per dispatch, the same one for the calls that share a dispatch (their
        // route and gathered activation are reused).
        const uint64_t caller_gen = ctx->generation;
        ctx->generation = sent.private_gen;
        ctx->route_pinned = rv.slot;
        ctx->route_skip_negative = true;
        st = b200q_mul_mat_id(ctx, src0_local, &x1, &id1, &y1);
        ctx->route_skip_negative = false;
        ctx->route_pinned = -1;
        ctx->generation = caller_gen;
        if (st != B200Q_OK) return st;
        mark();
        ep_combine_kernel<<<copy_blocks(slots), EP_COPY_THREADS, 0, ctx->stream>>>(tp->ep_out, tp->ep_counts, L, tp->ep_state);
        B200Q_CUDA(ctx, cudaGetLastError());
        mark();
        ep_unpack_kernel2<<<copy_blocks(n_pairs), EP_COPY_THREADS, 0, ctx->stream>>>(rv.pairs, rv.owner_counts, n_pairs, n_used, (float *)dst->data,
                                                           (int64_t)(dst->nb[1] / 4), (int64_t)(dst->nb[2] / 4), L, tp->ep_state,
                                                           ctx->error_word);
        B200Q_CUDA(ctx, cudaGetLastError());
        mark();
        if (trace && !ctx->capturing) {
            cudaStreamSynchronize(ctx->stream);
            float ms[4] = {0, 0, 0, 0};
            for (int i = 0; i + 1 < nev; ++i) cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]);
            fprintf(stderr, "ep_trace rank %d M=%lld K=%lld pairs=%d%s: dispatch+wait %.3f product %.3f combine %.3f unpack %.3f ms\n", tp->rank,
                    (long long)M, (long long)K, n_pairs, cached ? " (dispatch cached)" : "", ms[0], ms[1], ms[2], ms[3]);
        }
        for (int i = 0; i < nev; ++i) cudaEventDestroy(ev[i]);
        count(ctx, ST_EP_PEER);
        count(ctx, ST_EP_COMBINE);
        return B200Q_OK;
    }
    // 2. everyone learns everyone's counts, and whether every rank got this far (ep_agree.h)
    const int REC = G + 1;
    int32_t *gathered = tp->agree_dev, *mine = tp->agree_dev + (size_t)G * REC;
    std::vector<int32_t> h((size_t)G * REC);
    // One agreement round: this rank's record (its per-owner counts when it has them, its status word) goes to every
    // rank; B200Q_OK only when all ranks reported B200Q_OK. A CUDA or NCCL failure inside the round itself cannot be
    // agreed on and is returned as it is.
    auto agree = [&](int stage, b200q_status mine_st, const int32_t *dev_counts) -> b200q_status {
        mine_st = injected(stage, mine_st);
        tp->agree_host = (int32_t)mine_st;
        if (dev_counts) B200Q_CUDA(ctx, cudaMemcpyAsync(mine, dev_counts, sizeof(int32_t) * G, cudaMemcpyDeviceToDevice, ctx->stream));
        else B200Q_CUDA(ctx, cudaMemsetAsync(mine, 0, sizeof(int32_t) * G, ctx->stream));
        B200Q_CUDA(ctx, cudaMemcpyAsync(mine + G, &tp->agree_host, sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        B200Q_NCCL(ctx, api, api->AllGather(mine, gathered, (size_t)REC, ncclInt32, tp->comm, ctx->stream));
        B200Q_CUDA(ctx, cudaMemcpyAsync(h.data(), gathered, sizeof(int32_t) * h.size(), cudaMemcpyDeviceToHost, ctx->stream));
        B200Q_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        int who = -1;
        const int verdict = ep_agree_decide(h.data(), G, REC, G, tp->rank, (int)B200Q_PEER_FAILED, &who);
        if (verdict == 0) return B200Q_OK;
        count(ctx, ST_EP_AGREED_EXIT);
        if (verdict == (int)B200Q_PEER_FAILED)
            return fail(ctx, B200Q_PEER_FAILED, "rank %d reported status %d at stage %d of the expert-parallel call; every rank leaves", who,
                        (int)h[(size_t)who * REC + G], stage);
        return (b200q_status)verdict;                        // this rank's own error: its message is already recorded
    };
    if (ctx->capturing) local = local != B200Q_OK ? local : fail(ctx, B200Q_UNSUPPORTED, "the NCCL form of expert parallelism synchronises: not capturable");
    if ((st = agree(0, local, local == B200Q_OK ? rv.owner_counts : nullptr)) != B200Q_OK) return st;
    std::vector<size_t> so(G), sb(G), ro(G), rb(G), zo(G), zb(G), wo(G), wb(G);
    size_t n_send = 0, n_recv = 0;
    for (int g = 0; g < G; ++g) {
        const size_t cs = (size_t)h[(size_t)tp->rank * REC + g], cr = (size_t)h[(size_t)g * REC + tp->rank];
        so[g] = n_send; sb[g] = cs; ro[g] = n_recv; rb[g] = cr;
        n_send += cs;
        n_recv += cr;
    }
    // 3. scratch and packing are rank-local too: agree again before the first exchange
    const size_t rowx = (size_t)K * 4, rowy = (size_t)M * 4;
    float *send_x = nullptr, *recv_x = nullptr, *out = nullptr, *back = nullptr;
    int32_t *send_e = nullptr, *recv_e = nullptr;
    auto prepare = [&]() -> b200q_status {
        if ((int64_t)n_send != n_pairs) return fail(ctx, B200Q_INVALID, "route counted %zu of %d pairs", n_send, n_pairs);
        b200q_status r;
        if ((r = ws_reserve(ctx, &ctx->moe_ws[1], rowx * (n_send ? n_send : 1))) != B200Q_OK) return r;
        if ((r = ws_reserve(ctx, &ctx->moe_ws[2], 4 * (n_send ? n_send : 1))) != B200Q_OK) return r;
        if ((r = ws_reserve(ctx, &ctx->moe_ws[3], rowx * (n_recv ? n_recv : 1))) != B200Q_OK) return r;
        if ((r = ws_reserve(ctx, &ctx->moe_ws[4], 4 * (n_recv ? n_recv : 1))) != B200Q_OK) return r;
        if ((r = ws_reserve(ctx, &ctx->moe_ws[5], rowy * (n_recv ? n_recv : 1))) != B200Q_OK) return r;
        if ((r = ws_reserve(ctx, &ctx->moe_ws[6], rowy * (n_send ? n_send : 1))) != B200Q_OK) return r;
        send_x = (float *)ctx->moe_ws[1].ptr; recv_x = (float *)ctx->moe_ws[3].ptr;
        send_e = (int32_t *)ctx->moe_ws[2].ptr; recv_e = (int32_t *)ctx->moe_ws[4].ptr;
        out = (float *)ctx->moe_ws[5].ptr; back = (float *)ctx->moe_ws[6].ptr;
        return launch_ep_pack(ctx, src1, ids, n_expert_total, n_local, rv.pairs, send_x, send_e);
    };
    if ((st = agree(1, prepare(), nullptr)) != B200Q_OK) return st;
    for (int g = 0; g < G; ++g) { zo[g] = so[g] * rowx; zb[g] = sb[g] * rowx; wo[g] = ro[g] * rowx; wb[g] = rb[g] * rowx; }
    if ((st = b200q_all_to_all_v(ctx, send_x, zo.data(), zb.data(), recv_x, wo.data(), wb.data())) != B200Q_OK) return st;
    for (int g = 0; g < G; ++g) { zo[g] = so[g] * 4; zb[g] = sb[g] * 4; wo[g] = ro[g] * 4; wb[g] = rb[g] * 4; }
    if ((st = b200q_all_to_all_v(ctx, send_e, zo.data(), zb.data(), recv_e, wo.data(), wb.data())) != B200Q_OK) return st;
    // 4. the local experts over everything received: one slot per received pair
    b200q_status prod = B200Q_OK;
    if (n_recv) {
        b200q_tensor x1, id1, y1;
        x1.id = id1.id = y1.id = nullptr;
        x1.type = B200Q_TYPE_F32; x1.data = recv_x;
        x1.ne[0] = K; x1.ne[1] = 1; x1.ne[2] = (int64_t)n_recv; x1.ne[3] = 1;
        x1.nb[0] = 4; x1.nb[1] = rowx; x1.nb[2] = rowx; x1.nb[3] = rowx * n_recv;
        id1.type = B200Q_TYPE_I32; id1.data = recv_e;
        id1.ne[0] = 1; id1.ne[1] = (int64_t)n_recv; id1.ne[2] = 1; id1.ne[3] = 1;
        id1.nb[0] = 4; id1.nb[1] = 4; id1.nb[2] = 4 * n_recv; id1.nb[3] = 4 * n_recv;
        y1.type = B200Q_TYPE_F32; y1.data = out;
        y1.ne[0] = M; y1.ne[1] = 1; y1.ne[2] = (int64_t)n_recv; y1.ne[3] = 1;
        y1.nb[0] = 4; y1.nb[1] = rowy; y1.nb[2] = rowy; y1.nb[3] = rowy * n_recv;
        // The receive buffers are reused with other contents by the next call, so what the local product
        // caches about them (quantized activation, route) must not outlive it: it runs under a cache
        // generation of its own, and the caller's generation -- with the route of `ids`, which gate, up and
        // down of a layer share -- comes back afterwards.
        const uint64_t caller_gen = ctx->generation;
        ctx->generation = (1ull << 62) + ++ctx->private_generation;
        ctx->route_pinned = rv.slot;                      // rv.pairs is read again after the local product
        prod = b200q_mul_mat_id(ctx, src0_local, &x1, &id1, &y1);
        ctx->route_pinned = -1;
        ctx->generation = caller_gen;
    }
    // 5. combine: results travel back the way the activations came -- if every rank's product went through
    if ((st = agree(2, prod, nullptr)) != B200Q_OK) return st;
    for (int g = 0; g < G; ++g) { zo[g] = ro[g] * rowy; zb[g] = rb[g] * rowy; wo[g] = so[g] * rowy; wb[g] = sb[g] * rowy; }
    if ((st = b200q_all_to_all_v(ctx, out, zo.data(), zb.data(), back, wo.data(), wb.data())) != B200Q_OK) return st;
    b200q::count(ctx, ST_EP_COMBINE);
    st = launch_ep_unpack(ctx, back, rv.pairs, n_used, n_pairs, (int)M, (float *)dst->data, (int64_t)(dst->nb[1] / 4),
                          (int64_t)(dst->nb[2] / 4));
    return st;
}

// The communicator's asynchronous error state, for callers that watch a stuck peer from the
// host: B200Q_OK, or B200Q_NCCL_ERROR after aborting the communicator.
b200q_status b200q_tp_check(b200q_ctx *ctx) {
    TpState *tp;
    Nccl *api;
    b200q_status st = tp_get(ctx, &tp, &api);
    if (st != B200Q_OK) return st;
    if (!api->CommGetAsyncError) return B200Q_OK;
    ncclResult_t async = ncclSuccess;
    B200Q_NCCL(ctx, api, api->CommGetAsyncError(tp->comm, &async));
    if (async != ncclSuccess && async != ncclInProgress) {
        if (api->CommAbort) api->CommAbort(tp->comm);
        tp->comm = nullptr;
        return fail(ctx, B200Q_NCCL_ERROR, "communicator failed: %s", api->GetErrorString ? api->GetErrorString(async) : "error");
    }
    return B200Q_OK;
}

}  // extern "C"
