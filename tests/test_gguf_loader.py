"""The GGUF reader under adapters/gguf against a file written by gguf-py's GGUFWriter (tests/golden/tiny.gguf, made
by tests/golden/make_gguf_fixture.py): header, key/value section with every value kind, tensor table, data offsets,
and the b200q_tensor it describes; malformed files are refused, not read past. The GPU test feeds a loaded weight
to b200q_mul_mat."""
import ctypes as C
import os

import numpy as np
import pytest

import arcint_b200 as A
import oracle as O
from arcint_b200 import build as B

HERE = os.path.dirname(os.path.abspath(__file__))
FIX = os.path.join(HERE, "golden", "tiny.gguf")


class GT(C.Structure):
    _fields_ = [("name", C.c_char_p), ("type", C.c_int32), ("n_dims", C.c_int32), ("ne", C.c_int64 * 4), ("offset", C.c_uint64),
                ("nbytes", C.c_uint64), ("data", C.c_void_p)]


@pytest.fixture(scope="module")
def G():
    L = C.CDLL(B.build_gguf())
    L.b200q_gguf_open.restype = C.c_void_p
    L.b200q_gguf_open.argtypes = [C.c_char_p]
    L.b200q_gguf_close.argtypes = [C.c_void_p]
    L.b200q_gguf_error.restype = C.c_char_p
    for f in ("b200q_gguf_version", "b200q_gguf_alignment"):
        getattr(L, f).restype = C.c_uint32
        getattr(L, f).argtypes = [C.c_void_p]
    for f in ("b200q_gguf_tensor_count", "b200q_gguf_kv_count"):
        getattr(L, f).restype = C.c_int64
        getattr(L, f).argtypes = [C.c_void_p]
    L.b200q_gguf_tensor_at.argtypes = [C.c_void_p, C.c_int64, C.POINTER(GT)]
    L.b200q_gguf_find.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(GT)]
    L.b200q_gguf_get_u32.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint32)]
    L.b200q_gguf_get_str.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(C.c_uint64)]
    L.b200q_gguf_row_bytes.restype = C.c_size_t
    L.b200q_gguf_row_bytes.argtypes = [C.c_int32, C.c_int64]
    L.b200q_gguf_describe.argtypes = [C.POINTER(GT), C.c_void_p, C.POINTER(A.Tensor)]
    return L


def _bytes(t):
    return np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_uint8)), shape=(t.nbytes,)).copy()


def test_reads_what_gguf_py_wrote(G):
    exp = np.load(os.path.join(HERE, "golden", "tiny_gguf_expect.npz"))
    g = G.b200q_gguf_open(FIX.encode())
    assert g, G.b200q_gguf_error()
    try:
        assert G.b200q_gguf_version(g) == 3 and G.b200q_gguf_alignment(g) == 32
        names = [k for k in exp.files if not k.endswith(".meta")]
        assert G.b200q_gguf_tensor_count(g) == len(names)
        assert G.b200q_gguf_kv_count(g) >= 8                         # the seven test keys and general.architecture
        v = C.c_uint32()
        assert G.b200q_gguf_get_u32(g, b"b200q.test.u32", C.byref(v)) == 0 and v.value == 4242
        s, n = C.c_char_p(), C.c_uint64()
        assert G.b200q_gguf_get_str(g, b"b200q.test.str", C.byref(s), C.byref(n)) == 0
        assert C.string_at(s, n.value) == b"hello gguf"
        assert G.b200q_gguf_get_str(g, b"general.architecture", C.byref(s), C.byref(n)) == 0 and C.string_at(s, n.value) == b"llama"
        assert G.b200q_gguf_get_u32(g, b"no.such.key", C.byref(v)) != 0
        seen = set()
        for i in range(len(names)):
            t = GT()
            assert G.b200q_gguf_tensor_at(g, i, C.byref(t)) == 0
            name = t.name.decode()
            seen.add(name)
            meta = exp[name + ".meta"]
            want = exp[name]
            assert t.type == meta[0] and list(t.ne[:len(meta) - 1]) == [int(x) for x in meta[1:]], (name, t.type, list(t.ne))
            assert t.offset % 32 == 0 and t.nbytes == want.nbytes
            assert np.array_equal(_bytes(t), want.view(np.uint8).reshape(-1))
            d = A.Tensor()
            st = G.b200q_gguf_describe(C.byref(t), 0x1000, C.byref(d))
            if t.type == 0:
                assert st == A.OK and d.nb[0] == 4 and d.nb[1] == 4 * t.ne[0]
            else:
                assert st == A.OK and d.type == t.type and d.nb[1] == A.row_bytes(t.type, t.ne[0]) and d.nb[2] == d.nb[1] * t.ne[1]
                assert d.data == 0x1000 and d.id == 0x1000 and list(d.ne) == list(t.ne)
        assert seen == set(names)
        t = GT()
        assert G.b200q_gguf_find(g, b"blk.0.ffn_gate_exps.weight", C.byref(t)) == 0 and t.n_dims == 3 and t.ne[2] == 3
        assert G.b200q_gguf_find(g, b"missing", C.byref(t)) != 0
        assert G.b200q_gguf_tensor_at(g, len(names), C.byref(t)) != 0
    finally:
        G.b200q_gguf_close(g)


def test_row_bytes_of_every_type_of_the_path(G):
    for t in O.QUANT_TYPES:
        assert G.b200q_gguf_row_bytes(t, 4096) == O.row_bytes(t, 4096)
    assert G.b200q_gguf_row_bytes(O.Q4_K, 100) == 0 and G.b200q_gguf_row_bytes(99, 256) == 0


@pytest.mark.parametrize("cut", [3, 10, 23, 40, 200, 900])
def test_truncated_and_foreign_files_are_refused(G, tmp_path, cut):
    raw = open(FIX, "rb").read()
    p = tmp_path / "cut.gguf"
    p.write_bytes(raw[:cut])
    assert not G.b200q_gguf_open(str(p).encode())
    assert G.b200q_gguf_error()
    q = tmp_path / "foreign.gguf"
    q.write_bytes(b"GGML" + raw[4:])
    assert not G.b200q_gguf_open(str(q).encode())
    v = tmp_path / "v9.gguf"
    v.write_bytes(raw[:4] + (9).to_bytes(4, "little") + raw[8:])
    assert not G.b200q_gguf_open(str(v).encode())


def test_tensor_past_the_end_of_the_file_is_refused(G, tmp_path):
    """The header parses, but the last tensors' bytes are missing: opening works, asking for such a tensor does not."""
    raw = open(FIX, "rb").read()
    p = tmp_path / "short.gguf"
    p.write_bytes(raw[:len(raw) - 4000])
    g = G.b200q_gguf_open(str(p).encode())
    assert g
    try:
        bad = 0
        for i in range(G.b200q_gguf_tensor_count(g)):
            t = GT()
            if G.b200q_gguf_tensor_at(g, i, C.byref(t)) != 0:
                bad += 1
                assert not t.data
        assert bad >= 1
    finally:
        G.b200q_gguf_close(g)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["blk.0.q4_K.weight", "blk.0.q6_K.weight", "blk.0.q4_0.weight", "blk.0.q5_K.weight", "blk.0.iq4_nl.weight"])
def test_loaded_weight_goes_through_mul_mat(G, name):
    g = G.b200q_gguf_open(FIX.encode())
    assert g
    try:
        t = GT()
        assert G.b200q_gguf_find(g, name.encode(), C.byref(t)) == 0
        w = _bytes(t).reshape(t.ne[1], -1)
        k, m = int(t.ne[0]), int(t.ne[1])
        x = np.random.default_rng(k + m).normal(0, 1, size=(3, k)).astype(np.float32)
        with A.Context(0) as ctx:
            dw, dx, dy = ctx.upload(w), ctx.upload(x), ctx.alloc(3 * m * 4)
            W = A.Tensor()
            assert G.b200q_gguf_describe(C.byref(t), dw, C.byref(W)) == A.OK
            ctx.mul_mat(W, A.Tensor.f32(dx, [k, 3]), A.Tensor.f32(dy, [m, 3]))
            got = ctx.download(dy, (3, m), np.float32)
        ref = O.mul_mat_f64(int(t.type), w, k, x, True)
        assert np.abs(got - ref).max() <= 1e-3 * max(np.abs(ref).max(), 1e-6)
    finally:
        G.b200q_gguf_close(g)
