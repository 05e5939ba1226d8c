"""Generate tests/golden/tiny.gguf (+ tiny_gguf_expect.npz) with gguf-py's GGUFWriter: a few small tensors in the
block formats of the path, quantized by the oracle, plus metadata of every kv value type, so that the GGUF reader
under adapters/gguf has a file written by the format's own reference implementation to read.

Run in a container that has the `gguf` package:  python tests/golden/make_gguf_fixture.py
The tests only read the two files."""
import os
import sys

import numpy as np
import gguf

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import oracle as O                                                  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
T = gguf.GGMLQuantizationType
QT = {O.Q4_0: T.Q4_0, O.Q8_0: T.Q8_0, O.Q4_K: T.Q4_K, O.Q5_K: T.Q5_K, O.Q6_K: T.Q6_K, O.IQ4_XS: T.IQ4_XS, O.IQ4_NL: T.IQ4_NL}


def main():
    path = os.path.join(HERE, "tiny.gguf")
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("b200q.test.u32", 4242)
    w.add_string("b200q.test.str", "hello gguf")
    w.add_float32("b200q.test.f32", 1.5)
    w.add_bool("b200q.test.bool", True)
    w.add_array("b200q.test.arr_i32", [1, 2, 3, 4, 5])
    w.add_array("b200q.test.arr_str", ["a", "bc", "def"])
    w.add_uint64("b200q.test.u64", 1 << 40)
    expect = {}
    shapes = {O.Q4_0: (24, 256), O.Q8_0: (8, 128), O.Q4_K: (16, 512), O.Q5_K: (5, 256), O.Q6_K: (12, 512), O.IQ4_XS: (7, 256),
              O.IQ4_NL: (9, 96)}
    for t, (m, k) in shapes.items():
        blocks = O.quantize(t, O.fill_normal(m * k, 900 + t, 0.02).reshape(m, k))          # uint8 [m, row_bytes]
        name = "blk.0.%s.weight" % O.TYPE_NAMES[t]
        w.add_tensor(name, blocks, raw_dtype=QT[t])
        expect[name] = blocks
        expect[name + ".meta"] = np.array([t, k, m], dtype=np.int64)
    # a stack of expert matrices (three dimensions) and a plain f32 tensor
    ex = np.stack([O.quantize(O.Q4_K, O.fill_normal(8 * 256, 950 + e, 0.02).reshape(8, 256)) for e in range(3)])
    w.add_tensor("blk.0.ffn_gate_exps.weight", ex, raw_dtype=T.Q4_K)
    expect["blk.0.ffn_gate_exps.weight"] = ex
    expect["blk.0.ffn_gate_exps.weight.meta"] = np.array([O.Q4_K, 256, 8, 3], dtype=np.int64)
    f = O.fill_normal(6 * 10, 999, 1.0).reshape(6, 10)
    w.add_tensor("norm.weight", f)
    expect["norm.weight"] = f
    expect["norm.weight.meta"] = np.array([0, 10, 6], dtype=np.int64)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    np.savez_compressed(os.path.join(HERE, "tiny_gguf_expect.npz"), **expect)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
