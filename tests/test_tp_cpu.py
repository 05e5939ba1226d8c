"""Host-side logic of the multi-GPU splits, on CPU: the shard arithmetic exported by the C ABI,
and world_size-2 gloo runs in which each rank computes its shard with the CPU oracle and the
exchange the split needs (concatenate / all-reduce / dispatch-combine) goes through
torch.distributed -- the result must be the unsharded product."""
import os
import sys

import numpy as np
import pytest

import arcint_b200 as A
import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_covers_and_respects_units():
    for total, unit in ((4096, 1), (11008, 32), (11008, 256), (512, 1), (4096, 256), (96, 32)):
        for n in (1, 2, 3, 4, 8):
            pos = 0
            for r in range(n):
                first, count = A.tp_shard(total, unit, n, r)
                assert first == pos and count % unit == 0 and count >= 0
                pos += count
            assert pos == total
    # 11008 = 43 blocks of 256: 8 ranks get 6,6,6,5,5,5,5,5 blocks
    assert [A.tp_shard(11008, 256, 8, r)[1] // 256 for r in range(8)] == [6, 6, 6, 5, 5, 5, 5, 5]
    with pytest.raises(A.B200QError):
        A.tp_shard(100, 32, 2, 0)                       # not whole units
    with pytest.raises(A.B200QError):
        A.tp_shard(128, 32, 2, 2)                       # rank out of range


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        t, m, k, n = O.Q4_K, 48, 1024, 5
        w = O.quantize(t, O.fill_normal(m * k, 5, 0.02).reshape(m, k))
        x = O.fill_normal(n * k, 6, 1.0).reshape(n, k)
        full = O.mul_mat_f64(t, w, k, x, True)
        rb = O.row_bytes(t, k)
        # column split: a row range of the weight per rank, results concatenated
        r0, rc = A.tp_shard(m, 1, world, rank)
        part = torch.from_numpy(O.mul_mat(t, w[r0:r0 + rc], k, x).copy())
        parts = [torch.empty((n, A.tp_shard(m, 1, world, r)[1]), dtype=torch.float32) for r in range(world)]
        dist.all_gather(parts, part)
        col = torch.cat(parts, dim=1).numpy()
        # row split: a K range on block boundaries per rank (weight and activation), partials summed
        k0, kc = A.tp_shard(k, O.block_size(t), world, rank)
        b0, bc = k0 // O.block_size(t) * O.block_bytes(t), kc // O.block_size(t) * O.block_bytes(t)
        wk = np.ascontiguousarray(w.reshape(m, rb)[:, b0:b0 + bc])
        partial = torch.from_numpy(O.mul_mat(t, wk, kc, np.ascontiguousarray(x[:, k0:k0 + kc])).copy())
        dist.all_reduce(partial)
        row = partial.numpy()
        # expert split: tokens sharded, experts sharded; dispatch by owner, compute, combine
        n_expert, n_used, n_tok, me, ke = 8, 2, 6, 16, 256
        rng = np.random.default_rng(11)
        we = np.stack([O.random_blocks(t, me, ke, rng) for _ in range(n_expert)])
        ids_all = np.stack([rng.permutation(n_expert)[:n_used] for _ in range(n_tok * world)]).astype(np.int32)
        xe_all = rng.normal(0, 1, size=(n_tok * world, 1, ke)).astype(np.float32)
        want = O.mul_mat_id(t, we, me, ke, xe_all, ids_all)[rank * n_tok:(rank + 1) * n_tok]
        ids, xe = ids_all[rank * n_tok:(rank + 1) * n_tok], xe_all[rank * n_tok:(rank + 1) * n_tok]
        e0, ec = A.tp_shard(n_expert, 1, world, rank)
        pairs = [(tk, i) for tk in range(n_tok) for i in range(n_used)]
        owner = lambda e: next(r for r in range(world) if A.tp_shard(n_expert, 1, world, r)[0] <= e < sum(A.tp_shard(n_expert, 1, world, r)))
        send = [[p for p in pairs if owner(ids[p]) == r] for r in range(world)]
        out_lists = [None] * world
        dist.all_gather_object(out_lists, [[(int(ids[p]), xe[p[0], 0].copy()) for p in send[r]] for r in range(world)])
        mine = [out_lists[src][rank] for src in range(world)]           # what each source sent to this rank
        results = []
        for src_items in mine:
            res = []
            for e, xv in src_items:
                assert e0 <= e < e0 + ec
                res.append(O.mul_mat(t, we[e], ke, xv[None])[0])
            results.append(res)
        back_lists = [None] * world
        dist.all_gather_object(back_lists, results)
        got = np.zeros((n_tok, n_used, me), dtype=np.float32)
        for r in range(world):
            for p, v in zip(send[r], back_lists[r][rank]):
                got[p[0], p[1]] = v
        ok = (np.abs(col - full).max() < 1e-4 * np.abs(full).max() and np.abs(row - full).max() < 1e-4 * np.abs(full).max()
              and np.array_equal(got, want))
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_splits_world_size_2_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    res = dict(q.get(timeout=5) for _ in range(2))
    assert res == {0: True, 1: True}


def _agree_worker(rank, world, port, q, fail_rank, fail_stage):
    """A replay of the NCCL form of b200q_mul_mat_id_ep's control flow on gloo ranks: three agreement rounds
    (after the counts, before the dispatch, before the combine) decided by the library's own rule
    (ep_agree_decide, through the host replay). One rank reports a host-side error at one stage."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from arcint_b200 import build as B
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E = C.CDLL(B.build_emul())
        E.emul_ep_agree.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]
        rec = world + 1
        left_at, status, exchanges = None, A.binding.OK, 0
        for stage in range(3):
            mine = torch.zeros(rec, dtype=torch.int32)
            mine[:world] = torch.arange(world, dtype=torch.int32) + 10 * rank          # the per-owner counts
            mine[world] = A.binding.INVALID if (rank == fail_rank and stage == fail_stage) else A.binding.OK
            allr = [torch.empty(rec, dtype=torch.int32) for _ in range(world)]
            dist.all_gather(allr, mine)
            flat = torch.cat(allr).numpy().copy()
            who = C.c_int(-2)
            v = E.emul_ep_agree(flat.ctypes.data, world, rec, world, rank, A.binding.PEER_FAILED, C.byref(who))
            if v != 0:
                left_at, status = stage, v
                assert who.value == fail_rank
                break
            # the collective that follows the agreement: every rank that got here must find all the others here
            t = torch.ones(1)
            dist.all_reduce(t)
            assert int(t.item()) == world
            exchanges += 1
        q.put((rank, left_at, int(status), exchanges))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_rank,fail_stage", [(1, 0), (0, 1), (1, 2), (-1, -1)])
def test_ep_ranks_leave_together_gloo(fail_rank, fail_stage):
    """No rank of an expert-parallel call leaves between collectives alone: with a host-injected error on one rank
    at one stage, both ranks stop at that stage -- the failing rank with its own status, the other with PEER_FAILED --
    and every collective before it saw both ranks."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() + 7 * (fail_rank + 2) + 3 * (fail_stage + 2)) % 2000
    procs = [ctx.Process(target=_agree_worker, args=(r, 2, port, q, fail_rank, fail_stage)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    res = {r: (at, st, ex) for r, at, st, ex in (q.get(timeout=5) for _ in range(2))}
    if fail_rank < 0:
        assert res == {0: (None, A.binding.OK, 3), 1: (None, A.binding.OK, 3)}
    else:
        other = 1 - fail_rank
        assert res[fail_rank] == (fail_stage, A.binding.INVALID, fail_stage)
        assert res[other] == (fail_stage, A.binding.PEER_FAILED, fail_stage)
