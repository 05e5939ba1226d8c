#!/usr/bin/env python
"""bench.py -- the path's headline measurement on B200.

Default workload ("decode_gemv", benchmark config 2): the decode GEMV over a Llama-7B-shaped
set of quantized weights -- Q4_K gate/up 11008x4096, Q4_K down 4096x11008, Q6_K LM head
32000x4096 -- at batch 1, 2, 4 and 8 f32 activation columns. One step = all twelve
products once, each through b200q_mul_mat (activation quantize + GEMV).

  value      algorithmic GB/s of the whole step with inputs resident in HBM
  roofline   the GEMV kernel alone (activation already quantized), CUDA events on the
             launching stream, against the measured HBM copy peak
  e2e        the same step through the C ABI with HOST buffers: pinned f32 activations
             copied in and f32 results copied out inside the timed region (weights are
             resident, as after ggml's set_tensor at model load)
  cpu_baseline  the CPU oracle (a port of the reference math, not ggml) on the host cores

Weights rotate over distinct device copies whose total footprint is several times the
126 MB L2, so no product finds its weights in cache. Under torchrun each rank runs a
replica (the decode configuration of the benchmark definition is single-GPU; it does not shard).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "quant mul_mat prefill TFLOPS + decode GEMV HBM GB/s (% roofline), 1/2/4/8 GPU"
L2_BYTES = 126 << 20
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, copy read+write)"
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ---- the decode workload -------------------------------------------------------------------

def decode_shapes():
    import arcint_b200 as A
    return [("gate_up", A.Q4_K, 11008, 4096), ("down", A.Q4_K, 4096, 11008), ("lm_head", A.Q6_K, 32000, 4096)]


BATCHES = (1, 2, 4, 8)


def algo_bytes(t, m, k, n):
    import arcint_b200 as A
    return m * A.row_bytes(t, k) + 4 * n * (k + m)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.rows, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "window": "warm-up, the timed steps, one more second of the same step, the end-to-end and roofline legs"}


def build_decode_inputs(seed=0x5EED0001):
    """Seeded synthetic tensors of config 2: N(0,0.02) weights quantized on the host by the
    oracle's quantizers (stand-ins for ggml's K-quant quantizers), N(0,1) activations."""
    import oracle as O
    out = []
    for i, (name, t, m, k) in enumerate(decode_shapes()):
        w = O.quantize(t, O.fill_normal(m * k, seed + i, 0.02).reshape(m, k))
        out.append((name, t, m, k, w))
    x = {k: O.fill_normal(8 * k, seed + 100 + k, 1.0).reshape(8, k) for k in (4096, 11008)}
    return out, x


def prefill_section(ctx, world, rank, dist):
    """Prompt GEMM on the tensor cores (tcgen05 int8 MMA), reported beside the decode headline:
    config 1 (Q4_0 4096x4096, 512 tokens) on one GPU, and config 3's Q8_0 12288x3072 at 4096
    tokens column-split over the ranks (each rank owns a row range; no collective is needed
    for the compute, activations are replicated). Each timed product is quantize + GEMM."""
    import arcint_b200 as A
    import oracle as O
    peaks = {}
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            peaks = json.load(f)
    # the int8 tensor pipe runs at twice the bf16 rate; MEASURED_PEAKS has the bf16 number
    peak_tops = 2.0 * float(peaks.get("bf16_tflops", 1590.0))
    peak_src = "2 x measured bf16 burst (MEASURED_PEAKS.json)" if peaks else "2 x fallback bf16 1.59 PF"
    tag = " column-split" if world > 1 else ""
    cases = [("config1 q4_0 4096x4096 x 512", A.Q4_0, 4096, 4096, 512, False),
             ("config3 q8_0 3072x3072 x 4096" + tag, A.Q8_0, 3072, 3072, 4096, True),
             ("config3 q8_0 12288x3072 x 4096" + tag, A.Q8_0, 12288, 3072, 4096, True),
             ("config3 iq4_xs 17408x5120 x 512" + tag, A.IQ4_XS, 17408, 5120, 512, True),
             ("config3 iq4_xs 5120x17408 x 512" + tag, A.IQ4_XS, 5120, 17408, 512, True),
             ("config3 iq4_xs 17408x5120 x 2048" + tag, A.IQ4_XS, 17408, 5120, 2048, True),
             ("config3 iq4_xs 5120x17408 x 2048" + tag, A.IQ4_XS, 5120, 17408, 2048, True),
             # beyond the listed configs: the decode config's matrices at a prompt width (Q4_K and Q6_K on the tensor cores)
             ("extra q4_K 11008x4096 x 512" + tag, A.Q4_K, 11008, 4096, 512, True),
             ("extra q6_K 32000x4096 x 512" + tag, A.Q6_K, 32000, 4096, 512, True)]
    out = []
    for name, t, m, k, n, split in cases:
        if world > 1 and not split:
            continue
        r0, rc = A.tp_shard(m, 1, world, rank) if split else (0, m)
        base = O.quantize(t, O.fill_normal(256 * k, 0x5EED0300 + t, 0.02).reshape(256, k))
        w = np.tile(base, (-(-rc // 256), 1))[:rc]
        x = O.fill_normal(256 * k, 0x5EED0400, 1.0).reshape(256, k)
        x = np.tile(x, (-(-n // 256), 1))[:n]
        dw, dx, dy = ctx.upload(w), ctx.upload(x), ctx.alloc(n * rc * 4)
        W, X, Y = A.Tensor.weights(t, dw, k, rc), A.Tensor.f32(dx, [k, n]), A.Tensor.f32(dy, [rc, n])
        ctx.graph_begin()
        ctx.mul_mat(W, X, Y)
        got = ctx.download(dy, (n, rc), np.float32)
        rows = np.arange(0, rc, max(1, rc // 16))
        ref = O.mul_mat_f64(t, w[rows], k, x[:32], True)
        floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
        err = float((np.abs(got[:32][:, rows] - ref) / np.maximum(np.abs(ref), floor)).max())
        if not err < 1e-3:
            raise SystemExit("bench: prefill parity check failed on rank %d, %s (max rel err %.3e)" % (rank, name, err))
        reps = 5

        def seq():
            for _ in range(reps):
                ctx.graph_begin()
                ctx.mul_mat(W, X, Y)

        seq()
        g = ctx.capture(seq)
        ctx.graph_launch(g)
        ctx.sync()
        if dist:
            dist.barrier()
        ctx.timer_start()
        for _ in range(3):
            ctx.graph_launch(g)
        ms = ctx.timer_stop() / (3 * reps)
        if dist:
            import torch
            tt = torch.tensor([ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        ctx.graph_free(g)
        tops = 2.0 * m * k * n / (ms * 1e-3) / 1e12
        out.append({"workload": name, "ms": ms, "tops": tops, "roofline": {"bound": "tensor", "achieved": tops,
                    "peak": peak_tops * world, "unit": "TOP/s", "frac": tops / (peak_tops * world), "peak_source": peak_src},
                    "parity_max_rel_err": err, "timed": "activation quantize + tcgen05 int8 GEMM, CUDA-graph replay"})
        for ptr in (dw, dx, dy):
            ctx.free(ptr)
    return out


def _max_over_ranks(ms, dist):
    if dist:
        import torch
        tt = torch.tensor([ms], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    return ms


def tp_trace_section(ctx, world, rank, dist):
    """Config 4: the weight mat-muls of a Llama-2-7B-shaped model in Q4_0 (32 layers of q/k/v/o
    4096x4096, gate/up 11008x4096, down 4096x11008, LM head 32000x4096), as pp512 (512-token GEMMs on
    the tensor cores) and tg (sequential batch-1 GEMVs). Tensor parallel over the ranks: q/k/v/gate/
    up/head split by rows (column-parallel), o/down split along K (row-parallel) with an all-reduce of
    the f32 partial outputs. One layer's weights are generated and reused by every layer (two rotating
    device copies: 2 x 114 MB per GPU at N=1, beyond L2); the timed region is a CUDA-graph replay of the
    whole trace."""
    import arcint_b200 as A
    import oracle as O
    t = A.Q4_0
    shapes = [("q", 4096, 4096, "col"), ("k", 4096, 4096, "col"), ("v", 4096, 4096, "col"), ("o", 4096, 4096, "row"),
              ("gate", 11008, 4096, "col"), ("up", 11008, 4096, "col"), ("down", 4096, 11008, "row")]
    head = ("head", 32000, 4096, "col")
    bs, bb = A.block_size(t), A.block_bytes(t)
    dev = {}
    seed_of = {}

    def wfull_shard(name, r, kc_r):
        """the 256 distinct rows rank r tiles its shard of `name` from (row-split ranks differ in K range
        only by length: every rank draws its own block from the same seed, so the unsharded weight of the
        parity check is the ranks' blocks side by side)"""
        return O.quantize(t, O.fill_normal(256 * kc_r, seed_of[name], 0.02).reshape(256, kc_r))

    for name, m, k, how in shapes + [head]:
        seed_of[name] = 0x5EED0500 + len(dev)
        if how == "col":
            _, mc = A.tp_shard(m, 1, world, rank)
            kc = k
        else:
            mc = m
            _, kc = A.tp_shard(k, 256, world, rank)          # whole k-stages of the prompt GEMM per rank
        base = O.quantize(t, O.fill_normal(256 * kc, 0x5EED0500 + len(dev), 0.02).reshape(256, kc))
        w = np.tile(base, (-(-mc // 256), 1))[:mc]
        copies = [ctx.upload(w)]
        if name != "head":
            p2 = ctx.alloc(w.nbytes)
            ctx.copy(p2, copies[0], w.nbytes)
            copies.append(p2)
        dev[name] = (mc, kc, how, copies)
    out = []
    n_layers = 32
    for label, n, reps in (("pp512", 512, 1), ("tg128", 1, 8)):
        kmax = 11008
        # four activations per layer, as in the model's graph: the attention input feeds q, k and v, the
        # attention output feeds o, the FFN input feeds gate and up, their product feeds down. One cache
        # generation per layer, so the library quantizes each of them once (as under a ggml graph).
        x = O.fill_normal(n * kmax, 0x5EED0600 + n, 1.0).reshape(n, kmax)
        dxs = {key: ctx.upload(x) for key in ("attn_in", "attn_out", "ffn_in", "ffn_mid")}
        feeds = {"q": "attn_in", "k": "attn_in", "v": "attn_in", "o": "attn_out", "gate": "ffn_in", "up": "ffn_in",
                 "down": "ffn_mid", "head": "attn_in"}
        dy = ctx.alloc(n * 32000 * 4)

        def product(name, layer):
            mc, kc, how, copies = dev[name]
            xin = A.Tensor.make(A.F32, [kc, n, 1, 1], [4, 4 * kmax], dxs[feeds[name]])
            if how == "row" and world > 1:
                # product + all-reduce: one kernel at decode widths, product then collective at prompt widths
                ctx.mul_mat_allreduce(A.Tensor.weights(t, copies[layer % len(copies)], kc, mc), xin, A.Tensor.f32(dy, [mc, n]))
            else:
                ctx.mul_mat(A.Tensor.weights(t, copies[layer % len(copies)], kc, mc), xin, A.Tensor.f32(dy, [mc, n]))

        def trace():
            for _ in range(reps):
                for layer in range(n_layers):
                    ctx.graph_begin()
                    for name, _, _, _ in shapes:
                        product(name, layer)
                ctx.graph_begin()
                product("head", 0)

        for layer in range(2):
            ctx.graph_begin()
            for name, _, _, _ in shapes:
                product(name, layer)
        ctx.graph_begin()
        product("head", 0)
        ctx.sync()
        # parity before timing, on every rank: the row-split products (o, down) after their all-reduce and one
        # column-split product (q) against the oracle's product with the unsharded weight, sampled rows
        errs = {}
        for name in ("o", "down", "q"):
            mc, kc, how, copies = dev[name]
            m_full, k_full = [(m, k) for nm, m, k, _ in shapes if nm == name][0]
            ctx.graph_begin()
            product(name, 0)
            got = ctx.download(dy, (n, mc), np.float32)
            nchk = min(n, 4)
            if how == "row":
                rows = np.arange(0, m_full, max(1, m_full // 24))
                # the full weight is the ranks' K shards side by side, each the seeded block of its rank
                parts = []
                for r in range(world):
                    _, kr = A.tp_shard(k_full, 256, world, r)
                    parts.append(wfull_shard(name, r, kr)[rows % 256])
                ref, k0 = 0.0, 0
                for r, pw in enumerate(parts):
                    _, kr = A.tp_shard(k_full, 256, world, r)
                    ref = ref + O.mul_mat_f64(t, pw, kr, np.ascontiguousarray(x[:nchk, :kr]), True)
                    k0 += kr
                sub = got[:nchk][:, rows]
            else:
                rows = np.arange(0, mc, max(1, mc // 24))
                ref = O.mul_mat_f64(t, wfull_shard(name, rank, kc)[rows % 256], kc, np.ascontiguousarray(x[:nchk, :kc]), True)
                sub = got[:nchk][:, rows]
            floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
            errs[name] = float((np.abs(sub - ref) / np.maximum(np.abs(ref), floor)).max())
            if not errs[name] < 1e-3:
                raise SystemExit("bench: tensor-parallel parity check failed on rank %d, %s %s (max rel err %.3e)"
                                 % (rank, label, name, errs[name]))
        how_run = "CUDA-graph replay"
        g = None
        try:
            g = ctx.capture(trace)
        except Exception as e:                     # a collective that cannot be captured: run the trace eagerly
            how_run = "eager launches (capture failed: %s)" % str(e)[:60]
        run = (lambda: ctx.graph_launch(g)) if g is not None else trace
        run()
        ctx.sync()
        if dist:
            dist.barrier()
        ctx.timer_start()
        for _ in range(2):
            run()
        ms = _max_over_ranks(ctx.timer_stop() / (2 * reps), dist)
        if g is not None:
            ctx.graph_free(g)
        ops = 2.0 * n * (n_layers * sum(m * k for _, m, k, _ in shapes) + head[1] * head[2])
        bytes_w = (n_layers * sum(m * k for _, m, k, _ in shapes) + head[1] * head[2]) // bs * bb
        rec = {"workload": "config4 llama-2-7b q4_0 %s" % label, "tokens": n, "ms_per_pass": ms,
               "tokens_per_s": n / (ms * 1e-3), "parallelism": "tp%d column/row split, all-reduce of row-split outputs" % world
               if world > 1 else "single GPU", "timed": how_run + " of 32 layers x 7 mat-muls + LM head",
               "parity_max_rel_err": max(errs.values())}
        if n > 8:
            rec["tops"] = ops / (ms * 1e-3) / 1e12
        else:
            rec["weight_gbs"] = bytes_w / (ms * 1e-3) / 1e9
        out.append(rec)
        for ptr in dxs.values():
            ctx.free(ptr)
        ctx.free(dy)
    for mc, kc, how, copies in dev.values():
        for ptr in copies:
            ctx.free(ptr)
    return out


def moe_section(ctx, world, rank, dist):
    """Config 5: MUL_MAT_ID over 512 Q4_K experts, top-10 routing from seeded Zipf(1.1) logits,
    d_model 2048, expert FFN 512 (gate/up 512x2048, down 2048x512), token batches 1 and 2048. With
    more than one rank the experts are split in contiguous ranges (512 / N per GPU), the tokens are
    split evenly, and dispatch / combine are all-to-alls (b200q_mul_mat_id_ep). Eight distinct experts
    are generated and tiled to 512 (the timing does not depend on the values)."""
    import arcint_b200 as A
    import oracle as O
    t, n_exp, n_used, d_model, d_ff = A.Q4_K, 512, 10, 2048, 512
    per = n_exp // world
    mats = {}
    for name, m, k in (("gate", d_ff, d_model), ("up", d_ff, d_model), ("down", d_model, d_ff)):
        base = np.stack([O.quantize(t, O.fill_normal(m * k, 0x5EED0700 + 8 * len(mats) + e, 0.02).reshape(m, k)) for e in range(8)])
        w = np.tile(base, (per // 8, 1, 1))
        mats[name] = (m, k, base, ctx.upload(w), w.shape[-1])
    out = []
    for n_total in (1, 2048):
        n_tok = max(1, n_total // world)
        ids = O.route_ids(n_used, n_tok, n_exp, 0x5EED0800 + rank)
        x = O.fill_normal(n_tok * d_model, 0x5EED0900 + rank, 1.0).reshape(n_tok, 1, d_model)
        h = O.fill_normal(n_tok * n_used * d_ff, 0x5EED0A00 + rank, 1.0).reshape(n_tok, n_used, d_ff)
        dxi, dh, di = ctx.upload(x), ctx.upload(h), ctx.upload(ids)
        dg = ctx.alloc(n_tok * n_used * d_ff * 4)
        dd = ctx.alloc(n_tok * n_used * d_model * 4)
        I = A.Tensor.make(A.I32, [n_used, n_tok, 1, 1], [4, 4 * n_used], di)

        def src0(name):
            m, k, _, dw, rb = mats[name]
            return A.Tensor.make(t, [k, m, per, 1], [A.block_bytes(t), rb, rb * m, rb * m * per], dw)

        if world > 1:
            ctx.ep_reserve(n_tok * n_used, d_model, d_model)        # collective; maps the peer regions (no-op when refused)

        def block():
            # gate and up read the token's activation (ne11 = 1), down reads one row per used expert
            ctx.graph_begin()
            for name, xin, yout, m in (("gate", A.Tensor.f32(dxi, [d_model, 1, n_tok]), dg, d_ff),
                                       ("up", A.Tensor.f32(dxi, [d_model, 1, n_tok]), dg, d_ff),
                                       ("down", A.Tensor.f32(dh, [d_ff, n_used, n_tok]), dd, d_model)):
                y = A.Tensor.f32(yout, [m, n_used, n_tok])
                if world > 1:
                    ctx.mul_mat_id_ep(src0(name), xin, I, y, n_exp)
                else:
                    ctx.mul_mat_id(src0(name), xin, I, y)

        block()
        got = ctx.download(dd, (n_tok, n_used, d_model), np.float32)
        err = None
        if True:                                          # parity of the last product on a sample of this rank's tokens
            ts = np.arange(0, n_tok, max(1, n_tok // 4))[:4]
            wfull = np.tile(mats["down"][2], (n_exp // 8, 1, 1))
            ref = O.mul_mat_id(t, wfull, d_model, d_ff, h[ts], np.ascontiguousarray(ids[ts]), f64=True)
            floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
            err = float((np.abs(got[ts] - ref) / np.maximum(np.abs(ref), floor)).max())
            if not err < 1e-3:
                raise SystemExit("bench: MoE parity check failed on rank %d (max rel err %.3e)" % (rank, err))
        reps = 5
        g = None
        peer_ep = world > 1 and ctx.stats().get("ep_peer", 0) > 0
        if world == 1 or peer_ep:                         # over NCCL the expert-parallel call synchronizes: not capturable
            g = ctx.capture(lambda: [block() for _ in range(reps)])
            ctx.graph_launch(g)
        ctx.sync()
        if dist:
            dist.barrier()
        g_used = g is not None
        ctx.timer_start()
        if g is not None:
            for _ in range(3):
                ctx.graph_launch(g)
            ms = ctx.timer_stop() / (3 * reps)
            ctx.graph_free(g)
        else:
            for _ in range(reps):
                block()
            ms = ctx.timer_stop() / reps
        ms = _max_over_ranks(ms, dist)
        tokens = n_tok * world
        ops = 2.0 * tokens * n_used * 3 * d_ff * d_model
        out.append({"workload": "config5 moe q4_K 512 experts top-10, %d token%s" % (tokens, "" if tokens == 1 else "s"),
                    "ms": ms, "tokens_per_s": tokens / (ms * 1e-3), "tops": ops / (ms * 1e-3) / 1e12,
                    "parallelism": ("ep%d: %d experts per GPU, all-to-all dispatch/combine" % (world, per)) if world > 1 else "single GPU",
                    "parity_max_rel_err": err,
                    "timed": "gate + up + down MUL_MAT_ID" + (", CUDA-graph replay" if g_used else ", eager (one host synchronisation per call)"),
                    "exchange": "none" if world == 1 else ("own kernels over peer memory" if peer_ep else "NCCL send/receive")})
        if world == 1:
            # the whole feed-forward block as one call: router (seeded logits of the same Zipf shape), gate, up,
            # SwiGLU, down, weighted combine
            logits = O.fill_normal(n_tok * n_exp, 0x5EED0B00, 1.0).reshape(n_tok, n_exp) - \
                1.1 * np.log(1.0 + np.random.default_rng(0x5EED0B01).permutation(n_exp))[None, :].astype(np.float32)
            dlg, dyo = ctx.upload(logits.astype(np.float32)), ctx.alloc(n_tok * d_model * 4)

            def ffn():
                ctx.graph_begin()
                ctx.moe_ffn(src0("gate"), src0("up"), src0("down"), A.Tensor.f32(dxi, [d_model, n_tok]), A.Tensor.f32(dlg, [n_exp, n_tok]),
                            n_used, 6.103515625e-5, float("inf"), A.Tensor.f32(dyo, [d_model, n_tok]))

            ffn()
            y = ctx.download(dyo, (n_tok, d_model), np.float32)
            ts = np.arange(0, n_tok, max(1, n_tok // 3))[:3]
            wg, wu, wd = (np.tile(mats[nm][2], (n_exp // 8, 1, 1)) for nm in ("gate", "up", "down"))
            ref, _, _ = O.moe_ffn(t, wg, wu, wd, d_model, d_ff, x[ts, 0], logits[ts].astype(np.float32), n_used, 6.103515625e-5, float("inf"))
            e_ffn = float(((y[ts] - ref) ** 2).sum() / max((ref ** 2).sum(), 1e-300))
            if not e_ffn < 5e-4:
                raise SystemExit("bench: fused MoE block parity check failed (NMSE %.3e)" % e_ffn)
            g2 = ctx.capture(lambda: [ffn() for _ in range(reps)])
            ctx.graph_launch(g2)
            ctx.sync()
            ctx.timer_start()
            for _ in range(3):
                ctx.graph_launch(g2)
            ms2 = ctx.timer_stop() / (3 * reps)
            ctx.graph_free(g2)
            out.append({"workload": "config5 moe block (router + gate/up + SwiGLU + down + combine), %d token%s" % (tokens, "" if tokens == 1 else "s"),
                        "ms": ms2, "tokens_per_s": tokens / (ms2 * 1e-3), "tops": ops / (ms2 * 1e-3) / 1e12, "parallelism": "single GPU",
                        "parity_max_rel_err": e_ffn, "timed": "b200q_moe_ffn, CUDA-graph replay", "exchange": "none"})
            ctx.free(dlg)
            ctx.free(dyo)
        for ptr in (dxi, dh, di, dg, dd):
            ctx.free(ptr)
    for m, k, base, dw, rb in mats.values():
        ctx.free(dw)
    return out


def run_case(args):
    """One product, a few times, for profiling and tile sweeps: --case <type>:<M>x<K>x<N>[:id].
    Seeded tensors are uploaded, every repeat is one b200q_mul_mat (or, with :id, one b200q_mul_mat_id over
    512 experts, top-10 routing, N tokens) in a cache generation of its own, over rotating weight copies
    beyond L2; the CUDA-event time per call and the path counters are printed as one JSON line. This is
    the command line the summaries under profiles/ give."""
    import arcint_b200 as A
    import oracle as O
    parts = args.case.split(":")
    tname, dims = parts[0], [int(v) for v in parts[1].lower().split("x")]
    is_id = len(parts) > 2 and parts[2] == "id"
    t = {v: k for k, v in O.TYPE_NAMES.items()}[tname]
    m, k, n = dims
    ctx = A.Context(0)
    base = O.quantize(t, O.fill_normal(256 * k, 0x5EED0C00 + t, 0.02).reshape(256, k))
    if is_id:
        n_exp, n_used = 512, 10
        w = np.tile(base, (-(-m // 256), 1))[:m]
        w = np.tile(w[None], (n_exp, 1, 1))
        rb = w.shape[-1]
        ids = O.route_ids(n_used, n, n_exp, 0x5EED0C10)
        x = O.fill_normal(n * k, 0x5EED0C20, 1.0).reshape(n, 1, k)
        dw, dx, di, dy = ctx.upload(w), ctx.upload(x), ctx.upload(ids), ctx.alloc(n * n_used * m * 4)
        W = [A.Tensor.make(t, [k, m, n_exp, 1], [A.block_bytes(t), rb, rb * m, rb * m * n_exp], dw)]
        X, I = A.Tensor.f32(dx, [k, 1, n]), A.Tensor.make(A.I32, [n_used, n, 1, 1], [4, 4 * n_used], di)
        Y = A.Tensor.f32(dy, [m, n_used, n])
        call = lambda i: ctx.mul_mat_id(W[0], X, I, Y)
        ops = 2.0 * m * k * n * n_used
    else:
        w = np.tile(base, (-(-m // 256), 1))[:m]
        copies = max(2, min(16, -(-3 * L2_BYTES // w.nbytes)))
        first = ctx.upload(w)
        ptrs = [first]
        for _ in range(copies - 1):
            p2 = ctx.alloc(w.nbytes)
            ctx.copy(p2, first, w.nbytes)
            ptrs.append(p2)
        x = O.fill_normal(min(n, 256) * k, 0x5EED0C20, 1.0).reshape(min(n, 256), k)
        x = np.tile(x, (-(-n // 256), 1))[:n]
        dx, dy = ctx.upload(x), ctx.alloc(n * m * 4)
        W = [A.Tensor.weights(t, p2, k, m) for p2 in ptrs]
        X, Y = A.Tensor.f32(dx, [k, n]), A.Tensor.f32(dy, [m, n])
        call = lambda i: ctx.mul_mat(W[i % len(W)], X, Y)
        ops = 2.0 * m * k * n
    ctx.graph_begin()
    call(0)
    ctx.sync()
    ctx.stats_reset()
    times = []
    for i in range(args.reps):
        ctx.graph_begin()
        ctx.timer_start()
        call(i + 1)
        times.append(ctx.timer_stop())
    ms = float(np.median(times))
    wbytes = m * A.row_bytes(t, k)
    print(json.dumps({"case": args.case, "reps": args.reps, "ms_per_call_median": ms, "ms_all": [round(v, 4) for v in times],
                      "tops": ops / (ms * 1e-3) / 1e12, "weight_gbs": wbytes / (ms * 1e-3) / 1e9, "stats": ctx.stats(),
                      "timed": "one eager call (activation quantize + product), CUDA events"}))
    ctx.close()


def run_reference(args, rank):
    """The CPU arm: the oracle (a port of the reference math; ggml's CPU backend is not
    in this image) on all host cores, same workload, metric and unit."""
    if rank != 0:
        return
    import oracle as O
    mats, xs = build_decode_inputs()
    total = sum(algo_bytes(t, m, k, n) for _, t, m, k, _ in mats for n in BATCHES)

    cpu_threads = len(os.sched_getaffinity(0))       # asked for explicitly: torchrun pins OMP_NUM_THREADS to 1

    def step():
        for _, t, m, k, w in mats:
            for n in BATCHES:
                O.mul_mat(t, w, k, xs[k][:n], nthreads=cpu_threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    v = total / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 block dots, f32 accumulate", "data": "synthetic",
        "config": {"workload": "decode_gemv: Q4_K 11008x4096 + Q4_K 4096x11008 + Q6_K 32000x4096, batch 1/2/4/8"},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": cpu_threads, "kind": "port",
                         "sample": "the full step (12 products) per timed step"},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_gpu(args, rank, world):
    import arcint_b200 as A
    import oracle as O

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist_mod.init_process_group("nccl")
        dist = dist_mod
    device = int(os.environ.get("LOCAL_RANK", 0)) if world > 1 else 0
    ctx = A.Context(device)
    if world > 1:
        # the library's own communicator (tensor-parallel trace, expert-parallel MoE): rank 0's id to all
        import torch
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt = torch.frombuffer(bytearray(A.tp_unique_id()), dtype=torch.uint8).clone().cuda()
        dist.broadcast(idt, 0)
        ctx.tp_init(bytes(idt.cpu().numpy().tobytes()), rank, world)
    mats, xs = build_decode_inputs()

    # device copies: each shape rotates over enough copies to exceed 4x L2
    dev = []
    for name, t, m, k, w in mats:
        copies = max(2, -(-4 * L2_BYTES // w.nbytes))
        first = ctx.upload(w)
        ptrs = [first]
        for _ in range(copies - 1):
            p = ctx.alloc(w.nbytes)
            ctx.copy(p, first, w.nbytes)
            ptrs.append(p)
        dev.append((name, t, m, k, ptrs))
    ctx.sync()
    dx = {k: ctx.upload(v) for k, v in xs.items()}
    max_m = max(m for _, _, m, _ in decode_shapes())
    dy = ctx.alloc(8 * max_m * 4)
    hx = {k: A.binding.PinnedArray((8, k), np.float32) for k in xs}
    for k in xs:
        hx[k].array[:] = xs[k]
    hy = A.binding.PinnedArray((8, max_m), np.float32)

    products = [(name, t, m, k, ptrs, n) for name, t, m, k, ptrs in dev for n in BATCHES]
    total_bytes = sum(algo_bytes(t, m, k, n) for _, t, m, k, _, n in products)
    ROT = 4                                 # step graphs, each on its own rotation of the weight copies

    def step_device(rot):
        for name, t, m, k, ptrs, n in products:
            ctx.graph_begin()
            ctx.mul_mat(A.Tensor.weights(t, ptrs[(rot * 5 + n) % len(ptrs)], k, m), A.Tensor.f32(dx[k], [k, n]),
                        A.Tensor.f32(dy, [m, n]))

    # end to end: every product has its own device input and output and its own pinned host output, so
    # the uploads run ahead of the kernels and the downloads behind them on the context's copy streams
    e2e_in = [ctx.alloc(4 * n * k) for _, _, _, k, _, n in products]
    e2e_out = [ctx.alloc(4 * n * m) for _, _, m, _, _, n in products]
    e2e_host = [A.binding.PinnedArray((n, m), np.float32) for _, _, m, _, _, n in products]

    # the step's twelve products are independent: the ones with the largest results go first, so that the download
    # left over after the last kernel is the smallest one (4096 x 1 floats instead of 32000 x 8)
    e2e_order = sorted(range(len(products)), key=lambda i: -products[i][5] * products[i][2])

    def step_e2e(rot):
        # host buffers in, host buffers out; the caller reads the results at the end of the step
        for i in e2e_order:
            name, t, m, k, ptrs, n = products[i]
            ctx.graph_begin()
            ctx.stage(e2e_in[i], hx[k].ptr, 4 * n * k)
            ctx.mul_mat(A.Tensor.weights(t, ptrs[(rot * 5 + n) % len(ptrs)], k, m), A.Tensor.f32(e2e_in[i], [k, n]),
                        A.Tensor.f32(e2e_out[i], [m, n]))
            ctx.fetch(e2e_host[i].ptr, e2e_out[i], 4 * n * m)

    def barrier():
        ctx.sync()
        if dist:
            dist.barrier()

    def timed(fn, steps):
        barrier()
        ctx.timer_start()
        for i in range(steps):
            fn(i)
        ms = ctx.timer_stop()
        if dist:
            import torch
            tt = torch.tensor([ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms

    # parity spot check before timing: sampled rows of one product against the oracle
    name, t, m, k, ptrs = dev[0]
    ctx.graph_begin()
    ctx.mul_mat(A.Tensor.weights(t, ptrs[0], k, m), A.Tensor.f32(dx[k], [k, 8]), A.Tensor.f32(dy, [m, 8]))
    got = ctx.download(dy, (8, m), np.float32)
    rows = np.arange(0, m, max(1, m // 64))
    ref = O.mul_mat_f64(t, mats[0][4][rows], k, xs[k], True)
    floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
    err = float((np.abs(got[:, rows] - ref) / np.maximum(np.abs(ref), floor)).max())
    if not err < 1e-3:
        raise SystemExit("bench: parity check failed before timing (max rel err %.3e)" % err)

    sampler = ClockSampler(device)
    if rank == 0:
        sampler.start()
    # the step as CUDA graphs (one per rotation): scratch is sized by an eager pass first
    for r in range(ROT):
        step_device(r)
    ctx.sync()
    ctx.stats_reset()
    graphs = [ctx.capture(lambda r=r: step_device(r)) for r in range(ROT)]
    st = ctx.stats()
    # one kernel per counted product (its column-count key) and per quantizer call
    launches_per_step = sum(v for key, v in st.items() if key.startswith("quantize_") or
                            (key.startswith("gemv_") and key.endswith("col"))) // ROT
    for i in range(max(args.warmup, 3)):
        ctx.graph_launch(graphs[i % ROT])
    ms = timed(lambda i: ctx.graph_launch(graphs[i % ROT]), args.steps)
    ms_step = ms / args.steps
    # the timed region lasts milliseconds, shorter than one nvidia-smi period: keep the same step running for
    # about a second more (not timed) so that the clock samples are taken under this load
    t_load = time.perf_counter()
    i = 0
    while time.perf_counter() - t_load < 1.0:
        for _ in range(50):
            ctx.graph_launch(graphs[i % ROT])
            i += 1
        ctx.sync()
    value = world * total_bytes / (ms_step * 1e-3) / 1e9
    launches = launches_per_step * args.steps

    # end to end through the C ABI with host buffers (eager calls, and the same as graphs)
    for i in range(3):
        step_e2e(i)
        ctx.sync()

    def e2e_eager(i):
        step_e2e(i)
        ctx.sync()

    ms_e2e_eager = timed(e2e_eager, args.steps) / args.steps
    # what arrived in the host buffers is the product (checked on the widest one against the oracle)
    name, t, m, k, ptrs, n = products[3]
    rows = np.arange(0, m, max(1, m // 64))
    ref = O.mul_mat_f64(t, mats[0][4][rows], k, xs[k][:n], True)
    floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
    err_e2e = float((np.abs(e2e_host[3].array[:, rows] - ref) / np.maximum(np.abs(ref), floor)).max())
    assert err_e2e < 1e-3, ("e2e parity", err_e2e)
    egraphs = [ctx.capture(lambda r=r: step_e2e(r)) for r in range(ROT)]

    def e2e_graph(i):
        ctx.graph_launch(egraphs[i % ROT])
        ctx.sync()

    for i in range(3):
        e2e_graph(i)
    e2e_host[3].array[:] = 0.0                           # the replays must bring the product back again
    ms_e2e_graph = timed(e2e_graph, args.steps) / args.steps
    err_e2e = float((np.abs(e2e_host[3].array[:, rows] - ref) / np.maximum(np.abs(ref), floor)).max())
    assert err_e2e < 1e-3, ("e2e parity (graph replay)", err_e2e)
    # The end-to-end figure is the step as a decode loop runs it: recorded once through the C ABI (b200q_capture_begin /
    # _end around the stage, product and fetch calls), then one b200q_graph_launch and one synchronize per step; every
    # replay copies the inputs from the pinned host buffers and the results back into them. The same calls issued one
    # by one from Python are reported beside it.
    ms_e2e = ms_e2e_graph
    e2e = world * total_bytes / (ms_e2e * 1e-3) / 1e9
    h2d = sum(4 * n * k for _, _, _, k, _, n in products)
    d2h = sum(4 * n * m for _, _, m, _, _, n in products)

    # roofline of the dominant kernel: the GEMV alone (activation quantized once per graph),
    # a graph of back-to-back launches over the rotating weight copies
    peak, peak_src = measured_peaks()
    detail, tot_b, tot_ms, tot_traffic = [], 0, 0.0, 0.0
    reps = 50
    for name, t, m, k, ptrs, n in products:
        W = [A.Tensor.weights(t, p, k, m) for p in ptrs]
        X, Y = A.Tensor.f32(dx[k], [k, n]), A.Tensor.f32(dy, [m, n])
        ctx.graph_begin()
        ctx.mul_mat(W[0], X, Y)

        def gemv_only():
            for i in range(reps):
                ctx.mul_mat(W[i % len(W)], X, Y)

        g = ctx.capture(gemv_only)
        for _ in range(3):
            ctx.graph_launch(g)
        ctx.sync()
        nl = 4
        ctx.timer_start()
        for _ in range(nl):
            ctx.graph_launch(g)
        kms = ctx.timer_stop() / (reps * nl)
        ctx.graph_free(g)
        b = algo_bytes(t, m, k, n)
        detail.append({"shape": "%s %dx%d" % (O.TYPE_NAMES[t], m, k), "batch": n, "us": round(kms * 1e3, 2),
                       "gbs": round(b / (kms * 1e-3) / 1e9, 1), "frac": round(b / (kms * 1e-3) / 1e9 / peak, 3)})
        tot_b += b
        tot_ms += kms
        # DRAM bytes per launch as ncu captured them (dram__bytes_read.sum + dram__bytes_write.sum): 25.39 to 25.46 MB for
        # the 25.36 MB Q4_K matrix at 1 and 8 columns; for the 107.52 MB Q6_K head 111.7 to 114.2 MB from the dp4a
        # kernels (1 and 2 columns) and 107.83 MB from the warp-MMA kernel (4 and 8 columns)
        tot_traffic += b * ((1.05 if n < 3 else 1.003) if t == A.Q6_K else 1.003)
    achieved = tot_b / (tot_ms * 1e-3) / 1e9
    clocks = sampler.stop() if rank == 0 else None

    # the sections beside the headline (all by default; --sections picks some, e.g. to compare one of them across builds)
    want = set(args.sections.split(",")) if args.sections else {"prefill", "tp_trace", "moe"}
    prefill = prefill_section(ctx, world, rank, dist) if "prefill" in want else []
    tp_trace = tp_trace_section(ctx, world, rank, dist) if "tp_trace" in want else []
    moe = moe_section(ctx, world, rank, dist) if "moe" in want else []

    cpu = None
    if rank == 0 and world == 1:           # the CPU leg runs at N=1 only (idle ranks would spin on the host cores it needs)
        cpu_threads = len(os.sched_getaffinity(0))       # torchrun pins OMP_NUM_THREADS to 1: ask for the cores explicitly
        t0 = time.perf_counter()
        reps_cpu = 0
        while time.perf_counter() - t0 < 10.0:
            for _, t, m, k, w in mats:
                for n in BATCHES:
                    O.mul_mat(t, w, k, xs[k][:n], nthreads=cpu_threads)
            reps_cpu += 1
        dt = (time.perf_counter() - t0) / reps_cpu
        cpu = {"value": total_bytes / dt / 1e9, "unit": "GB/s", "cores": cpu_threads, "kind": "port",
               "sample": "the full step (12 products), %d repeats in ~10 s" % reps_cpu}

    if dist:
        dist.barrier()
    if rank == 0:
        # one short line per section first, so a truncated tail of the output still carries the sharded numbers
        for r in prefill:
            print("# prefill %-44s %8.4f ms %7.1f TOP/s frac %.3f err %.1e" % (r["workload"], r["ms"], r["tops"], r["roofline"]["frac"],
                                                                             r["parity_max_rel_err"]), file=sys.stderr)
        for r in tp_trace:
            print("# tp_trace %-34s %8.3f ms/pass %10.1f tok/s err %.1e (%s)" % (r["workload"], r["ms_per_pass"], r["tokens_per_s"],
                                                                                 r["parity_max_rel_err"], r["parallelism"][:24]), file=sys.stderr)
        for r in moe:
            print("# moe %-52s %8.4f ms err %.1e (%s)" % (r["workload"], r["ms"], r["parity_max_rel_err"], r["parallelism"][:24]),
                  file=sys.stderr)
        summary = {"prefill": {r["workload"]: [round(r["ms"], 4), round(r["tops"], 1)] for r in prefill},
                   "tp_trace_ms": {r["workload"].split()[-1]: round(r["ms_per_pass"], 3) for r in tp_trace},
                   "moe_ms": {r["workload"].replace("config5 ", "")[:40]: round(r["ms"], 4) for r in moe}}
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 block dots (dp4a; warp MMA from 3-4 columns), f32 accumulate", "data": "synthetic",
            "config": {"workload": "decode_gemv: Q4_K 11008x4096 + Q4_K 4096x11008 + Q6_K 32000x4096, batch 1/2/4/8",
                       "l2": "weights rotate over device copies totalling >= 4x L2 per shape",
                       "launch": "each step is one CUDA-graph replay of 12 x (quantize, GEMV)",
                       "parallelism": "replicas" if world > 1 else "single GPU", "parity_max_rel_err": err},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         # DRAM bytes per GEMV launch, mean over the 12 products, scaled from the ncu captures
                         "traffic": tot_traffic / len(detail), "algorithmic_bytes_per_launch": tot_b / len(detail),
                         "peak_source": peak_src, "kernel": "gemv_stream_kernel / gemv_kernel at 1-2 (Q4_K: 1-3) columns, gemv_mma_kernel above (activation pre-quantized), back-to-back launches in a CUDA graph",
                         "detail": detail},
            "prefill": prefill,
            "tp_trace": tp_trace,
            "moe": moe,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e, "how": "per product tensor_stage (pinned host -> device, copy stream), mul_mat, tensor_fetch "
                    "(device -> pinned host, copy stream) through the C ABI, recorded once with capture_begin/_end; per step one "
                    "graph_launch (the copies run in every replay) and one synchronize",
                    "eager_value": world * total_bytes / (ms_e2e_eager * 1e-3) / 1e9, "eager_ms_per_step": ms_e2e_eager},
            "gpu_launches": launches,
            "clocks": clocks,
            "sections_ms": summary,
        }
        print(json.dumps(line))
    ctx.close()
    if dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200q", choices=["b200q", "reference"])
    ap.add_argument("--case", default=None, help="<type>:<M>x<K>x<N>[:id] -- one product a few times (profiling)")
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--sections", default=None, help="comma list of prefill,tp_trace,moe (default: all)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args, rank)
    else:
        run_gpu(args, rank, world)


if __name__ == "__main__":
    main()
