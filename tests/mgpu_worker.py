"""One rank of the multi-GPU parity check; launched by tests/test_gpu_multi.py as
  python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 ... tests/mgpu_worker.py
Every rank: its own GPU and b200q context, joins the NCCL communicator (id broadcast over a gloo
group), runs a column split (Q8_0 prompt GEMM, all-gather), a row split (Q4_0 and Q4_K, all-reduce
of the f32 partials), a variable all-to-all and an expert-parallel MUL_MAT_ID, and compares with the CPU oracle."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import torch
import torch.distributed as dist

import arcint_b200 as A
import oracle as O
from gpu_util import TOL, rel_err


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo")
    ctx = A.Context(local)
    idt = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        idt = torch.frombuffer(bytearray(A.tp_unique_id()), dtype=torch.uint8).clone()
    dist.broadcast(idt, 0)
    ctx.tp_init(bytes(idt.numpy().tobytes()), rank, world)

    # column split: Q8_0, 64 tokens (tensor-core path), rows sharded, results gathered
    t, m, k, n = A.Q8_0, 512 * world, 1024, 64
    w = O.quantize(t, O.fill_normal(m * k, 21, 0.02).reshape(m, k))
    x = O.fill_normal(n * k, 22, 1.0).reshape(n, k)
    r0, rc = A.tp_shard(m, 1, world, rank)
    dw, dx = ctx.upload(w[r0:r0 + rc]), ctx.upload(x)
    dpart, dall = ctx.alloc(n * rc * 4), ctx.alloc(world * n * rc * 4)
    ctx.graph_begin()
    ctx.mul_mat(A.Tensor.weights(t, dw, k, rc), A.Tensor.f32(dx, [k, n]), A.Tensor.f32(dpart, [rc, n]))
    ctx.all_gather(dpart, dall, n * rc * 4)
    got = ctx.download(dall, (world, n, rc), np.float32)
    got = np.concatenate([got[r] for r in range(world)], axis=1)
    e1 = rel_err(got, O.mul_mat_f64(t, w, k, x, True))
    assert e1 < TOL, ("column split", e1)

    # row split: K sharded on block boundaries, f32 partials all-reduced
    errs = []
    for t, k in ((A.Q4_0, 2048), (A.Q4_K, 2816)):
        m, n = 256, 3
        w = O.quantize(t, O.fill_normal(m * k, 31 + t, 0.02).reshape(m, k))
        x = O.fill_normal(n * k, 32, 1.0).reshape(n, k)
        k0, kc = A.tp_shard(k, A.block_size(t), world, rank)
        b0, bc = k0 // A.block_size(t) * A.block_bytes(t), kc // A.block_size(t) * A.block_bytes(t)
        wk = np.ascontiguousarray(w[:, b0:b0 + bc])
        dw, dx, dy = ctx.upload(wk), ctx.upload(np.ascontiguousarray(x[:, k0:k0 + kc])), ctx.alloc(n * m * 4)
        ctx.graph_begin()
        if kc:
            ctx.mul_mat(A.Tensor.weights(t, dw, kc, m), A.Tensor.f32(dx, [kc, n]), A.Tensor.f32(dy, [m, n]))
        else:
            ctx.upload(np.zeros((n, m), dtype=np.float32), dy)
        ctx.all_reduce_f32(dy, n * m)
        got = ctx.download(dy, (n, m), np.float32)
        errs.append(rel_err(got, O.mul_mat_f64(t, w, k, x, True)))
        assert errs[-1] < TOL, ("row split", t, errs[-1])
        # the same as one call (at 1, 2, 4, 8 columns product and all-reduce are one kernel), twice in a row
        if kc:
            for nn in (1, 2, 4):
                xs = np.ascontiguousarray(x[:nn, k0:k0 + kc]) if nn <= n else np.ascontiguousarray(np.tile(x, (2, 1))[:nn, k0:k0 + kc])
                xfull = x[:nn] if nn <= n else np.tile(x, (2, 1))[:nn]
                dxs, dy2 = ctx.upload(xs), ctx.alloc(nn * m * 4)
                for rep in range(2):
                    ctx.graph_begin()
                    ctx.upload(np.full((nn, m), np.nan, dtype=np.float32), dy2)
                    ctx.mul_mat_allreduce(A.Tensor.weights(t, dw, kc, m), A.Tensor.f32(dxs, [kc, nn]), A.Tensor.f32(dy2, [m, nn]))
                    got = ctx.download(dy2, (nn, m), np.float32)
                    e = rel_err(got, O.mul_mat_f64(t, w, k, xfull, True))
                    assert e < TOL, ("fused row split", t, nn, rep, e)
                ctx.free(dxs)
                ctx.free(dy2)

    # the one-shot all-reduce over peer memory, many times in a row (both sets of slots, the device-side sequence
    # number), eagerly and replayed from a CUDA graph: every rank must end with the same, exact sums
    # (small integers: any order of the additions gives the same float)
    cnt = 3000
    vals = (np.arange(cnt, dtype=np.float32) % 97) + rank
    dv = ctx.alloc(cnt * 4)
    want = sum(((np.arange(cnt, dtype=np.float32) % 97) + r) for r in range(world))
    for rep in range(5):
        ctx.upload(vals, dv)
        ctx.all_reduce_f32(dv, cnt)
        assert np.array_equal(ctx.download(dv, (cnt,), np.float32), want), ("peer all-reduce", rep)
    ctx.upload(vals, dv)
    ctx.sync()
    dist.barrier()

    def three():
        for _ in range(3):
            ctx.all_reduce_f32(dv, cnt)

    g = ctx.capture(three)
    for rep in range(2):
        ctx.graph_launch(g)
        ctx.sync()
        dist.barrier()
    ctx.graph_free(g)
    # six all-reduces of the running sums: value * world^6 (exact in f32 for these sizes)
    got6 = ctx.download(dv, (cnt,), np.float32)
    # after the first all-reduce every rank holds `want`; each further one multiplies by world
    assert np.array_equal(got6, want * float(world) ** 5), "peer all-reduce in a graph"
    peer_used = ctx.stats().get("tp_allreduce_peer", 0)

    # variable all-to-all: rank r sends (r + p + 1) floats of value 100 r + p to peer p
    send_counts = [rank + p + 1 for p in range(world)]
    recv_counts = [p + rank + 1 for p in range(world)]
    send = np.concatenate([np.full(c, 100 * rank + p, dtype=np.float32) for p, c in enumerate(send_counts)])
    ds, dr = ctx.upload(send), ctx.alloc(sum(recv_counts) * 4)
    so, ro = np.concatenate([[0], np.cumsum(send_counts)[:-1]]) * 4, np.concatenate([[0], np.cumsum(recv_counts)[:-1]]) * 4
    ctx.all_to_all_v(ds, so, [4 * c for c in send_counts], dr, ro, [4 * c for c in recv_counts])
    got = ctx.download(dr, (sum(recv_counts),), np.float32)
    want = np.concatenate([np.full(c, 100 * p + rank, dtype=np.float32) for p, c in enumerate(recv_counts)])
    assert np.array_equal(got, want), "all_to_all_v"

    # expert parallelism: 8 experts split over the ranks, every rank brings its own tokens (a different
    # count per rank) with global expert ids; against the oracle's MUL_MAT_ID over all experts
    ep_errs = []
    cases = ((A.Q4_K, 192, 512, 5 + 3 * rank, 1), (A.Q4_0, 96, 256, 37 + rank, 2), (A.Q6_K, 64, 256, 1, 1),
             (A.Q4_K, 128, 1024, 150 + 7 * rank, 1))
    for mode in ("nccl", "peer"):
        if mode == "peer":
            # collective, same bounds on every rank: the largest pair count, the longest rows
            ctx.ep_reserve(2 * (150 + 7 * (world - 1)), 1024, 192)
        for t, m, k, n_tok, ne11 in cases:
            n_exp, n_used = 4 * world, 2
            per = n_exp // world
            w = np.stack([O.quantize(t, O.fill_normal(m * k, 500 + 10 * t + e, 0.05).reshape(m, k)) for e in range(n_exp)])
            x = O.fill_normal(n_tok * ne11 * k, 600 + rank, 1.0).reshape(n_tok, ne11, k)
            ids = O.route_ids(n_used, n_tok, n_exp, 700 + rank)
            dw = ctx.upload(np.ascontiguousarray(w[rank * per:(rank + 1) * per]))
            dx, di, dy = ctx.upload(x), ctx.upload(ids), ctx.alloc(n_tok * n_used * m * 4)
            rb = w.shape[-1]
            src0 = A.Tensor.make(t, [k, m, per, 1], [A.block_bytes(t), rb, rb * m, rb * m * per], dw)
            X, I = A.Tensor.f32(dx, [k, ne11, n_tok]), A.Tensor.make(A.I32, [n_used, n_tok, 1, 1], [4, 4 * n_used], di)
            Y = A.Tensor.f32(dy, [m, n_used, n_tok])
            want = O.mul_mat_id(t, w, m, k, x, ids, f64=True).reshape(-1, m)
            ctx.graph_begin()
            for rep in range(2):          # twice in one graph generation: the second finds the dispatch done (gate, up)
                ctx.upload(np.zeros((n_tok, n_used, m), dtype=np.float32), dy)
                ctx.mul_mat_id_ep(src0, X, I, Y, n_exp)
                got = ctx.download(dy, (n_tok, n_used, m), np.float32)
                ep_errs.append(rel_err(got.reshape(-1, m), want))
                assert ep_errs[-1] < TOL, ("expert parallel", mode, t, rep, ep_errs[-1])
            if mode == "nccl" and (t, n_tok) == (A.Q4_0, 37 + rank):
                # a host-injected error on the last rank at each of the three agreement points: every rank must come
                # back from the call (nobody waits in a collective for a rank that left), the failing rank with its
                # own status, the others with PEER_FAILED; the next call is an ordinary one and must be right
                for stage in range(3):
                    os.environ["B200Q_EP_INJECT_FAIL"] = "%d:%d" % (world - 1, stage)
                    try:
                        ctx.mul_mat_id_ep(src0, X, I, Y, n_exp)
                        status = A.binding.OK
                    except A.B200QError as e:
                        status = e.status
                    finally:
                        del os.environ["B200Q_EP_INJECT_FAIL"]
                    assert status == (A.binding.INVALID if rank == world - 1 else A.binding.PEER_FAILED), (stage, rank, status)
                    ctx.graph_begin()
                    ctx.upload(np.zeros((n_tok, n_used, m), dtype=np.float32), dy)
                    ctx.mul_mat_id_ep(src0, X, I, Y, n_exp)
                    got = ctx.download(dy, (n_tok, n_used, m), np.float32)
                    assert rel_err(got.reshape(-1, m), want) < TOL, ("after an agreed exit", stage)
                assert ctx.stats().get("ep_agreed_exit") == 3, ctx.stats()
            for ptr in (dw, dx, di, dy):
                ctx.free(ptr)
        dist.barrier()
    ep_stats = ctx.stats()
    peer_ep = ep_stats.get("ep_peer", 0)
    # when the peer regions could be mapped every call of the second round went through them, half of them
    # on a cached dispatch
    assert peer_ep in (0, 2 * len(cases)), ep_stats
    if peer_ep:
        assert ep_stats.get("ep_dispatch_cached") == len(cases), ep_stats
    ctx.sync()

    st = ctx.stats()
    assert st.get("tp_allgather") == 1 and st.get("tp_allreduce", 0) >= 2 + 5 + 3 and st.get("gemm_tc", 0) >= 1, st
    # the decode-sized all-reduces went over peer memory unless the mapping was refused or switched off
    assert peer_used in (0, 10) or os.environ.get("B200Q_NO_PEER_AR") == "1", st
    if peer_used:
        assert st.get("gemv_allreduce_fused", 0) >= 6, st
    dist.barrier()
    print("MGPU_OK rank %d/%d colsplit %.2e rowsplit %s ep %s peer_allreduce %d" % (rank, world, e1, ["%.2e" % e for e in errs],
                                                                                       ["%.2e" % max(ep_errs)], peer_used) + " peer_ep %d" % peer_ep, flush=True)
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
