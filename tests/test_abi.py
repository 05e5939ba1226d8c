"""The C-ABI library loads and exports every symbol include/b200q.h and include/b200q_test.h declare (no compute)."""
import ctypes as C
import os
import re

import numpy as np

import arcint_b200 as A
from arcint_b200 import binding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    # the boundary (b200q.h) and the measurement / test helpers exported beside it (b200q_test.h)
    text = open(os.path.join(ROOT, "include", "b200q.h")).read() + open(os.path.join(ROOT, "include", "b200q_test.h")).read()
    return sorted(set(re.findall(r"B200Q_API\s+[\w\s\*]+?\b(b200q_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    syms = declared_symbols()
    assert len(syms) >= 20
    L = A.lib()
    for s in syms:
        assert hasattr(L, s), s
    assert sorted(binding.EXPORTS) == syms


def test_version_and_block_tables():
    assert b"sm_100a" in A.lib().b200q_version()
    assert A.row_bytes(A.Q4_K, 4096) == 2304 and A.row_bytes(A.Q6_K, 4096) == 3360
    assert A.row_bytes(A.Q4_0, 4096) == 2304 and A.row_bytes(A.Q8_0, 3072) == 3264 and A.row_bytes(A.IQ4_XS, 5120) == 2720


def test_tensor_struct_layout():
    t = A.Tensor.weights(A.Q4_K, 0x1000, 4096, 11008)
    assert C.sizeof(A.Tensor) == 88 and A.Tensor.id.offset == 80      # type, ne[4], nb[4], data, id
    assert list(t.ne) == [4096, 11008, 1, 1] and list(t.nb)[:2] == [144, 2304]
    f = A.Tensor.f32(0x2000, [4096, 8])
    assert list(f.nb) == [4, 16384, 131072, 131072]


def test_supports_gate_needs_no_device():
    """supports_op answers from shapes alone (ctx may be NULL): the reference's gate
    (0000-01-kquant-integer-dpas.patch:619-634, 807-812)."""
    L = A.lib()

    def sup(w, x, y, op=A.OP_MUL_MAT, ids=None):
        return L.b200q_supports(None, op, w, x, ids, y)

    k, m, n = 4096, 64, 4
    w = A.Tensor.weights(A.Q4_K, 0x10000, k, m)
    x, y = A.Tensor.f32(0x20000, [k, n]), A.Tensor.f32(0x30000, [m, n])
    assert sup(w, x, y) == A.OK
    assert sup(A.Tensor.weights(A.Q4_K, 0x10000, 4000 // 256 * 256 + 32, m), x, y) != A.OK       # K % 256
    bad = A.Tensor.weights(A.Q4_K, 0x10000, k, m, 2)
    assert sup(bad, x, y) == A.UNSUPPORTED                                                       # 3-D weights
    xi = A.Tensor.make(A.I32, [k, n], [4, 4 * k], 0x20000)
    assert sup(w, xi, y) == A.UNSUPPORTED                                                        # non-f32 src1
    wf = A.Tensor.make(A.F32, [k, m], [4, 4 * k], 0x10000)
    assert sup(wf, x, y) == A.UNSUPPORTED                                                        # unquantized weights
    assert sup(w, A.Tensor.f32(0x20000, [k // 2, n]), y) == A.INVALID
    assert sup(A.Tensor.weights(A.Q4_0, 0x10000, 96, m), A.Tensor.f32(0x20000, [96, n]), y) == A.OK
