"""Tile search for the decode GEMV, in the manner of the reference's tools/kq_tune (marfrit/arcint
tools/kq_tune/README.md: genomes of environment knobs scored on the benchmark shapes, exhaustive or by a small
genetic search, one JSON file rewritten after every evaluation so a rerun resumes).

  python -m arcint_b200.tune exhaustive|ga out.json [--cases q4_K:11008x4096x1,...] [--budget N] [--seed S]

Genome = the library's environment knobs, read once when a context is made:
  B200Q_GEMV_ROWS          rows per ring stage of the slice-resident GEMV (2, 4; 0 = default rule)
  B200Q_GEMV_BLOCK_WARPS   warps per block (2..16; 0 = default 4)
  B200Q_GEMV_STREAM_MASK   which column counts take the slice-resident kernel (bit c; -1 = default rule)
  B200Q_GEMV_NO_SMALL      1: never the 128-thread / 170-register build of the wide Q4_K / Q6_K forms
  B200Q_GEMV_MMA_MIN       fewest columns at which a product takes the warp-MMA GEMV (0 = measured rule per type: 3 to 6; 99 = never)
  B200Q_GEMV_MMA_SLICE     super-blocks per warp of the warp-MMA GEMV (2, 3, 4; 0 = by row length)
Fitness = sum over the cases of the median CUDA-event time of `bench.py --case` (lower is better), each case in
its own process. A genome the library ignored (stats key "gemv_knob_ignored") scores nothing, so a fallback to
the defaults is never credited to the genome that asked for something else; the default genome is re-measured
every 8 evaluations and scores are kept as ratios to the latest re-measure (drift between GPU boxes and clocks).
Needs a GPU: run it where the library runs."""
import argparse
import itertools
import json
import os
import random
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEFAULT_CASES = ["q4_K:11008x4096x1", "q4_K:11008x4096x4", "q4_K:11008x4096x8", "q4_K:4096x11008x1", "q4_K:4096x11008x8",
                 "q6_K:32000x4096x1", "q6_K:32000x4096x8", "q4_0:4096x4096x1"]
GENES = {"B200Q_GEMV_ROWS": [0, 2, 4], "B200Q_GEMV_BLOCK_WARPS": [0, 2, 4, 8, 16],
         "B200Q_GEMV_STREAM_MASK": [-1, 0x1F2, 0x1FE, 0x1F0, 0x112], "B200Q_GEMV_NO_SMALL": [0, 1],
         "B200Q_GEMV_MMA_MIN": [0, 2, 3, 4, 5, 99], "B200Q_GEMV_MMA_SLICE": [0, 2, 4]}
DEFAULT = {"B200Q_GEMV_ROWS": 0, "B200Q_GEMV_BLOCK_WARPS": 0, "B200Q_GEMV_STREAM_MASK": -1, "B200Q_GEMV_NO_SMALL": 0,
           "B200Q_GEMV_MMA_MIN": 0, "B200Q_GEMV_MMA_SLICE": 0}


def key(g):
    return ",".join("%s=%s" % (k, g[k]) for k in sorted(g))


def evaluate(genome, cases, reps):
    """sum of median ms over the cases, or None when a run failed or the library ignored a knob"""
    env = {k: v for k, v in os.environ.items() if not k.startswith("B200Q_GEMV_")}
    env.update({k: str(v) for k, v in genome.items() if (k, v) != ("B200Q_GEMV_STREAM_MASK", -1) and v != 0 or k == "B200Q_GEMV_STREAM_MASK" and v >= 0})
    total = 0.0
    for case in cases:
        try:
            r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--case", case, "--reps", str(reps)], env=env,
                               capture_output=True, text=True, timeout=600)
            line = json.loads(r.stdout.strip().splitlines()[-1])
        except (subprocess.TimeoutExpired, ValueError, IndexError):
            return None
        if r.returncode != 0 or line["stats"].get("gemv_knob_ignored"):
            return None
        total += line["ms_per_call_median"]
    return total


def mutate(g, rng):
    g = dict(g)
    k = rng.choice(sorted(GENES))
    vals = GENES[k]
    i = vals.index(g[k])
    g[k] = vals[max(0, min(len(vals) - 1, i + rng.choice((-1, 1))))]
    return g


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("mode", choices=["exhaustive", "ga"])
    ap.add_argument("out")
    ap.add_argument("--cases", default=",".join(DEFAULT_CASES))
    ap.add_argument("--budget", type=int, default=40)
    ap.add_argument("--pop", type=int, default=8)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--reps", type=int, default=8)
    a = ap.parse_args()
    cases = a.cases.split(",")
    rng = random.Random(a.seed)
    db = {"cases": cases, "evals": {}, "order": []}
    if os.path.exists(a.out):
        with open(a.out) as f:
            old = json.load(f)
        if old.get("cases") == cases:
            db = old                                              # resume: genomes already measured are skipped
    ref = {"ms": None, "age": 8}

    def score(g):
        k = key(g)
        if k in db["evals"]:
            return db["evals"][k]["ratio"]
        if ref["age"] >= 8:                                       # drift: the default genome again
            ref["ms"], ref["age"] = evaluate(DEFAULT, cases, a.reps), 0
        ms = evaluate(g, cases, a.reps)
        ref["age"] += 1
        ratio = ms / ref["ms"] if ms and ref["ms"] else None
        db["evals"][k] = {"genome": g, "ms": ms, "ratio": ratio}
        db["order"].append(k)
        with open(a.out, "w") as f:
            json.dump(db, f, indent=1)
        print("%-70s %s" % (k, "failed / ignored" if ratio is None else "%.4f ms  x%.3f of default" % (ms, ratio)), flush=True)
        return ratio

    if a.mode == "exhaustive":
        names = sorted(GENES)
        for vals in itertools.product(*(GENES[n] for n in names)):
            score(dict(zip(names, vals)))
    else:
        pop = [dict(DEFAULT)] + [{k: rng.choice(v) for k, v in GENES.items()} for _ in range(a.pop - 1)]
        while len(db["order"]) < a.budget:
            ranked = sorted(pop, key=lambda g: (score(g) is None, score(g) or 9e9))
            nxt = ranked[:2]                                      # elitism
            while len(nxt) < a.pop:
                pa = min(rng.sample(ranked, 3), key=lambda g: (score(g) is None, score(g) or 9e9))      # tournament of 3
                pb = min(rng.sample(ranked, 3), key=lambda g: (score(g) is None, score(g) or 9e9))
                child = {k: rng.choice((pa[k], pb[k])) for k in GENES}
                if rng.random() < 0.7:
                    child = mutate(child, rng)
                nxt.append(child)
            if all(key(g) in db["evals"] for g in nxt) and len(db["evals"]) >= len(list(itertools.product(*GENES.values()))):
                break
            pop = nxt
    best = min((e for e in db["evals"].values() if e["ratio"]), key=lambda e: e["ratio"], default=None)
    print("best:", json.dumps(best))


if __name__ == "__main__":
    main()
