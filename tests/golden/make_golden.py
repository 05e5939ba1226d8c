"""Generate tests/golden/quant_golden.npz with gguf-py (the ggml authors' numpy
implementation of the block formats, gguf/quants.py).

Run in a container that has the `gguf` package:  python tests/golden/make_golden.py
The tests only read the .npz, so they do not need gguf at run time.

Contents, per block type T in {q4_0, q8_0, q4_K, q6_K, iq4_xs, q5_K, iq4_nl}:
  T_blocks  uint8 [rows, row_bytes]  random-field blocks with sane fp16 scales
  T_deq     f32   [rows, k]          gguf.quants.dequantize(T_blocks)
and for the two types gguf-py can quantize bit-exactly like ggml-quants.c:
  T_src     f32   [rows, k]          inputs (N(0,0.02), zeros, exact .5 ties, large values)
  T_quant   uint8 [rows, row_bytes]  gguf.quants.quantize(T_src)
plus the per-32 activation form (ggml block_q8_0 of N(0,1) columns):
  act_src f32 [n, k], act_q int8 [n, k], act_d uint16 [n, k/32] (fp16 bits)
"""
import os

import numpy as np
from gguf import quants
from gguf.constants import GGML_QUANT_SIZES, GGMLQuantizationType as T

TYPES = {"q4_0": T.Q4_0, "q8_0": T.Q8_0, "q4_K": T.Q4_K, "q6_K": T.Q6_K, "iq4_xs": T.IQ4_XS}
MORE_TYPES = {"q5_K": T.Q5_K, "iq4_nl": T.IQ4_NL}
HALF_FIELDS = {  # byte offset of each fp16 field, (lo, hi) magnitude, signed?
    "q4_0": [(0, 1e-3, 2e-2, True)], "q8_0": [(0, 1e-3, 2e-2, True)], "iq4_xs": [(0, 1e-3, 2e-2, True)],
    "q4_K": [(0, 1e-4, 2e-3, False), (2, 1e-4, 2e-3, False)], "q6_K": [(208, 1e-5, 5e-4, True)],
    "q5_K": [(0, 1e-4, 2e-3, False), (2, 1e-4, 2e-3, False)], "iq4_nl": [(0, 1e-3, 2e-2, True)],
}


def random_blocks(name, rows, k, rng):
    bs, bb = GGML_QUANT_SIZES[TYPES[name] if name in TYPES else MORE_TYPES[name]]
    nb = k // bs
    raw = rng.integers(0, 256, size=(rows, nb, bb), dtype=np.uint8)
    for off, lo, hi, signed in HALF_FIELDS[name]:
        v = rng.uniform(lo, hi, size=(rows, nb)).astype(np.float32)
        if signed:
            v *= rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=(rows, nb))
        h = v.astype(np.float16).view(np.uint16)
        raw[:, :, off] = (h & 0xFF).astype(np.uint8)
        raw[:, :, off + 1] = (h >> 8).astype(np.uint8)
    return raw.reshape(rows, nb * bb)


def quant_inputs(rng, k):
    rows = [rng.normal(0, 0.02, size=k) for _ in range(5)]
    rows.append(np.zeros(k))
    tie = np.tile(np.arange(-16, 16) + 0.5, k // 32)       # x/d lands on .5 for d = 1 (q8_0: amax 127)
    tie[::32] = 127.0
    rows.append(tie)
    rows.append(rng.normal(0, 300.0, size=k))
    neg = rng.normal(0, 0.02, size=k)
    neg[5::32] = -0.2                                      # the largest magnitude is negative
    rows.append(neg)
    pos = rng.normal(0, 0.02, size=k)
    pos[7::32] = 0.2                                       # ... and positive
    rows.append(pos)
    return np.stack(rows).astype(np.float32)


def main():
    rng = np.random.default_rng(0xB200)
    out = {}
    k = 512
    for name, t in TYPES.items():
        blocks = random_blocks(name, 6, k, rng)
        out[name + "_blocks"] = blocks
        out[name + "_deq"] = quants.dequantize(blocks, t).astype(np.float32)
    for name in ("q4_0", "q8_0"):
        src = quant_inputs(rng, 256)
        out[name + "_src"] = src
        out[name + "_quant"] = quants.quantize(src, TYPES[name])
    act = rng.normal(0, 1.0, size=(6, 512)).astype(np.float32)
    act[4, :64] = 0.0
    act[5] = np.round(act[5] * 4) / 4
    qb = quants.quantize(act, T.Q8_0).reshape(6, 512 // 32, 34)
    out["act_src"] = act
    out["act_d"] = qb[:, :, :2].copy().view(np.uint16).reshape(6, 16)
    out["act_q"] = qb[:, :, 2:].copy().view(np.int8).reshape(6, 512)
    # types added later draw from a generator of their own, so the entries above keep their values
    rng2 = np.random.default_rng(0xB201)
    for name, t in MORE_TYPES.items():
        blocks = random_blocks(name, 6, k, rng2)
        out[name + "_blocks"] = blocks
        out[name + "_deq"] = quants.dequantize(blocks, t).astype(np.float32)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
