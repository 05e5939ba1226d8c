"""Device-free checks of the kernels' own text: the GEMV lane code, the block decoders and
the bit tricks are host+device functions; arcint_b200/csrc/emul.cpp compiles them with g++
and replays the kernel's loops on the CPU. What is checked here is the same source the GPU
runs (the method of the reference's tests/test-opencl-kq-i8.cpp)."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle as O
from arcint_b200 import build as B

_emul = None
_mutants = {}


def _load(so):
    E = C.CDLL(so)
    vp, i64 = C.c_void_p, C.c_int64
    E.emul_gemv.argtypes = [C.c_int, vp, C.c_size_t, i64, i64, vp, vp, vp, vp, vp, C.c_int, C.c_int, vp, i64]
    return E


def mutant(define):
    if define not in _mutants:
        _mutants[define] = _load(B.build_emul(define=define))
    return _mutants[define]


def emul():
    global _emul
    if _emul is None:
        so = B.build_emul()
        E = C.CDLL(so)
        vp, i64 = C.c_void_p, C.c_int64
        E.emul_gemv.argtypes = [C.c_int, vp, C.c_size_t, i64, i64, vp, vp, vp, vp, vp, C.c_int, C.c_int, vp, i64]
        E.emul_dequantize_row.argtypes = [C.c_int, vp, i64, vp]
        E.emul_lookup4_tab.argtypes = [vp, C.c_uint32]
        E.emul_lookup4_tab.restype = C.c_uint32
        E.emul_iq4xs_limbs.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        for f in ("emul_iq4nl_lookup4", "emul_nib_minus8", "emul_six_minus32"):
            getattr(E, f).argtypes = [C.c_uint32]
            getattr(E, f).restype = C.c_uint32
        _emul = E
    return _emul


def test_bit_tricks_exhaustive_per_byte():
    E = emul()
    for a in range(16):
        for b in range(16):
            idx = a | (b << 8) | (((a * 7 + 3) % 16) << 16) | (((b * 5 + 1) % 16) << 24)
            got = E.emul_iq4nl_lookup4(idx)
            want = 0
            for i in range(4):
                want |= (int(O.KVALUES_IQ4NL[(idx >> (8 * i)) & 0xF]) & 0xFF) << (8 * i)
            assert got == want
            got8 = E.emul_nib_minus8(idx)
            assert [((got8 >> (8 * i)) & 0xFF) for i in range(4)] == [(((idx >> (8 * i)) & 0xF) - 8) & 0xFF for i in range(4)]
    for a in range(64):
        t = a | ((63 - a) << 8) | (((a * 11) % 64) << 16) | (((a * 29 + 5) % 64) << 24)
        got = E.emul_six_minus32(t)
        assert [((got >> (8 * i)) & 0xFF) for i in range(4)] == [(((t >> (8 * i)) & 0x3F) - 32) & 0xFF for i in range(4)]


def test_iq4xs_two_limbs():
    """The tensor-core IQ4_XS path folds (ls - 32) * kvalues[n] into two int8 limbs, computed eight
    weights (one packed word) at a time in registers (biased lookup, one multiply-add per pair of
    16-bit halves): every (ls, n) must satisfy 256 hi + lo = product with both limbs in int8, and
    the packed form must agree with the scalar one for low and high nibbles."""
    E = emul()
    E.emul_iq4xs_limbs8.argtypes = [C.c_uint32, C.c_int, C.POINTER(C.c_uint32)]
    rng = np.random.default_rng(0)
    for ls in range(64):
        his, los = [], []
        for n in range(16):
            hi, lo = C.c_int(), C.c_int()
            E.emul_iq4xs_limbs(ls, n, C.byref(hi), C.byref(lo))
            assert 256 * hi.value + lo.value == (ls - 32) * int(O.KVALUES_IQ4NL[n])
            assert -128 <= lo.value <= 127 and -16 <= hi.value <= 16
            his.append(hi.value & 0xFF)
            los.append(lo.value & 0xFF)
        words = [0x10325476, 0x98BADCFE, 0x00000000, 0xFFFFFFFF, 0x88888888, 0x77777777] + \
                [int(x) for x in rng.integers(0, 1 << 32, 10, dtype=np.uint64)]
        for q in words:
            out = (C.c_uint32 * 4)()
            E.emul_iq4xs_limbs8(q, ls - 32, out)
            low = [(q >> (8 * b)) & 0xF for b in range(4)]
            high = [(q >> (8 * b + 4)) & 0xF for b in range(4)]
            assert out[0] == sum(his[i] << (8 * b) for b, i in enumerate(low))
            assert out[1] == sum(los[i] << (8 * b) for b, i in enumerate(low))
            assert out[2] == sum(his[i] << (8 * b) for b, i in enumerate(high))
            assert out[3] == sum(los[i] << (8 * b) for b, i in enumerate(high))


def test_q6k_two_limbs():
    """Q6_K on the tensor cores: sc * (q - 32) as 256 hi + lo with int8 limbs, for every scale and code."""
    E = emul()
    E.emul_q6k_limbs4.argtypes = [C.c_uint32, C.c_int, C.POINTER(C.c_uint32)]
    for sc in range(-128, 128):
        for q0 in range(0, 64, 4):
            q6 = q0 | ((q0 + 1) << 8) | ((q0 + 2) << 16) | ((q0 + 3) << 24)
            out = (C.c_uint32 * 2)()
            E.emul_q6k_limbs4(q6, sc, out)
            for b in range(4):
                hi = (out[0] >> (8 * b)) & 0xFF
                lo = (out[1] >> (8 * b)) & 0xFF
                hi = hi - 256 if hi >= 128 else hi
                lo = lo - 256 if lo >= 128 else lo
                assert 256 * hi + lo == sc * (q0 + b - 32) and -16 <= hi <= 16


def test_q4k_two_limbs_and_packed_scales():
    """Q4_K on the tensor cores: sc * q as 256 hi + lo with int8 limbs, four codes at a time; the packed
    extraction of the eight scales and mins must agree with the scalar one."""
    E = emul()
    E.emul_q4k_limbs4.argtypes = [C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32)]
    E.emul_q4k_scales_mins.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32)]
    E.emul_q4k_scale_min.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    rng = np.random.default_rng(1)
    for sc in range(64):
        # codes 0..15 (Q4_K) and 0..31 (Q5_K: the same limbs, sc * q <= 63 * 31)
        for idx4 in [np.arange(4) + 4 * g for g in range(8)] + [rng.integers(0, 32, 4) for _ in range(4)]:
            idx = int(idx4[0]) | (int(idx4[1]) << 8) | (int(idx4[2]) << 16) | (int(idx4[3]) << 24)
            out = (C.c_uint32 * 2)()
            E.emul_q4k_limbs4(idx, sc, out)
            for b, q in enumerate(idx4):
                hi = (out[0] >> (8 * b)) & 0xFF
                lo = (out[1] >> (8 * b)) & 0xFF
                hi = hi - 256 if hi >= 128 else hi
                lo = lo - 256 if lo >= 128 else lo
                assert 256 * hi + lo == sc * int(q) and 0 <= hi <= 8 and -128 <= lo <= 127
    for _ in range(200):
        s0, s1, s2 = (int(v) for v in rng.integers(0, 1 << 32, 3, dtype=np.uint64))
        out = (C.c_uint32 * 4)()
        E.emul_q4k_scales_mins(s0, s1, s2, out)
        for j in range(8):
            sc, m = C.c_int(), C.c_int()
            E.emul_q4k_scale_min(s0, s1, s2, j, C.byref(sc), C.byref(m))
            assert (out[j // 4] >> (8 * (j % 4))) & 0xFF == sc.value
            assert (out[2 + j // 4] >> (8 * (j % 4))) & 0xFF == m.value


@pytest.mark.parametrize("name,t", [("q4_0", O.Q4_0), ("q8_0", O.Q8_0), ("q4_K", O.Q4_K), ("q5_K", O.Q5_K), ("q6_K", O.Q6_K), ("iq4_xs", O.IQ4_XS),
                                    ("iq4_nl", O.IQ4_NL)])
def test_device_decoder_text_matches_gguf_golden(golden, name, t):
    E = emul()
    blocks, want = golden[name + "_blocks"], golden[name + "_deq"]
    got = np.empty_like(want)
    for r in range(blocks.shape[0]):
        row = np.ascontiguousarray(blocks[r])
        E.emul_dequantize_row(t, row.ctypes.data, want.shape[1], got[r].ctypes.data)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def _run_emul(t, w, k, x, R, E=None):
    E = E or emul()
    m, n = w.shape[0], x.shape[0]
    if O.act_form(t) == O.ACT_Q8_0:
        q, d = O.quantize_act_q8_0(x)
        d16, d32 = d.ctypes.data, None
    else:
        q, d, _ = O.quantize_act_q8_256(x)
        d16, d32 = None, d.ctypes.data
    s32 = q.reshape(n, k // 32, 32).astype(np.int32).sum(-1).astype(np.int16)
    s16 = q.reshape(n, k // 16, 16).astype(np.int32).sum(-1).astype(np.int16)
    out = np.full((n, m), np.nan, dtype=np.float32)
    rc = E.emul_gemv(t, w.ctypes.data, w.shape[1], m, k, q.ctypes.data, d16, d32, s32.ctypes.data, s16.ctypes.data, n, R,
                     out.ctypes.data, m)
    assert rc == 0
    return out


def rel_err(got, ref):
    floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), floor)).max())


# K values: one full stage, several stages, a ragged last stage, a single block
KS = {O.Q4_0: [32, 96, 1024, 2080, 4096, 6176], O.Q8_0: [32, 96, 1024, 2080, 4128], O.Q4_K: [256, 1024, 2816, 4096, 5120],
      O.Q5_K: [256, 1024, 2816, 4096, 5120],
      O.Q6_K: [256, 2048, 2816, 4096, 4352], O.IQ4_XS: [256, 1024, 2816, 5120], O.IQ4_NL: [32, 96, 1024, 2080, 4096, 6176]}


@pytest.mark.parametrize("t", O.QUANT_TYPES)
@pytest.mark.parametrize("n,R", [(1, 4), (2, 1), (3, 4), (4, 4), (5, 4), (7, 1), (8, 4)])
def test_gemv_lane_code_matches_oracle(t, n, R):
    rng = np.random.default_rng(1000 * t + n)
    for k in KS[t]:
        m = 7                                               # odd: exercises the ragged row group
        w = O.random_blocks(t, m, k, rng)
        x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
        got = _run_emul(t, w, k, x, R)
        ref = O.mul_mat_f64(t, w, k, x, True)
        assert np.isfinite(got).all()
        assert rel_err(got, ref) < 1e-4, (t, k, n)
        assert rel_err(got, O.mul_mat(t, w, k, x)) < 1e-4


def test_gemv_lane_code_red_case():
    """The comparison must be able to fail: a wrong activation scale has to show."""
    t, k = O.Q4_K, 1024
    rng = np.random.default_rng(5)
    w = O.random_blocks(t, 4, k, rng)
    x = rng.normal(0, 1, size=(1, k)).astype(np.float32)
    ref = O.mul_mat_f64(t, w, k, x, True)
    x2 = x.copy()
    x2[0, 700] += 0.5
    assert rel_err(_run_emul(t, w, k, x2, 4), ref) > 1e-3


@pytest.mark.parametrize("define,t", [("B200Q_RED_Q40", O.Q4_0), ("B200Q_RED_SCALE", O.Q4_K), ("B200Q_RED_DROP", O.Q8_0),
                                      ("B200Q_RED_DROP", O.Q4_0)])
def test_kernel_mutants_turn_the_suite_red(define, t):
    """The reference ships a mutant switch with every kernel patch and records that the suite fails under it
    (0099-opencl-q4_0-q8_0-int8-gemm.patch:304-310, 576-581; 0103-opencl-id-int8-sg8.patch:338-343;
    0115-...patch:742-746). The same lane text, built with the switch, must miss the tolerance the real build
    meets on every case here."""
    E = mutant(define)
    rng = np.random.default_rng(7)
    red = green = 0
    for k in (1024, 4096):
        for n in (1, 4, 8):
            w = O.random_blocks(t, 7, k, rng)
            x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
            ref = O.mul_mat_f64(t, w, k, x, True)
            green += rel_err(_run_emul(t, w, k, x, 4), ref) < 1e-4
            red += rel_err(_run_emul(t, w, k, x, 4, E), ref) > 1e-3
    assert green == 6 and red == 6, (define, green, red)


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_peer_allreduce_slot_protocol_and_give_up(nranks):
    """The one-shot all-reduce's slot protocol (sequence number beside each float, two alternating sets of
    slots, sum in rank order) replayed on the host from the kernel's own text: two all-reduces in a row give
    the same sum on every rank; with one rank silent in the second, every reader's bounded wait gives up
    after its poll limit instead of spinning."""
    E = emul()
    E.emul_peer_allreduce.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_uint, C.c_void_p]
    rng = np.random.default_rng(nranks)
    count = 1000
    x = rng.normal(0, 1, size=(2, nranks, count)).astype(np.float32)
    out = np.empty_like(x)
    gave = np.zeros(nranks, dtype=np.int32)
    assert E.emul_peer_allreduce(nranks, count, x.ctypes.data, out.ctypes.data, -1, 100, gave.ctypes.data) == 0
    assert not gave.any()
    for call in range(2):
        want = np.zeros(count, dtype=np.float32)
        for r in range(nranks):                                  # the kernel's order: rank 0 first
            want = want + x[call, r]
        for r in range(nranks):
            assert np.array_equal(out[call, r], want)
    assert E.emul_peer_allreduce(nranks, count, x.ctypes.data, out.ctypes.data, nranks - 1, 50, gave.ctypes.data) == 0
    assert gave.all()                                            # nobody hung: every rank gave up and said so
    assert np.array_equal(out[0, 0], x[0].sum(axis=0, dtype=np.float32)) or np.allclose(out[0, 0], x[0].sum(axis=0), atol=1e-5)
