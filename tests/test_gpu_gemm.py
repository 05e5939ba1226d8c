"""GPU parity of the tensor-core prefill GEMM (Q4_0 / Q8_0, more than 8 tokens) through the
C ABI against the CPU oracle: f32 outputs within max relative error 1e-3 of the fp64 product
of the same quantized operands; NMSE against the unquantized-activation product under the
reference's op-suite bound (5e-4). Shapes follow the reference's cases (marfrit/arcint
contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch:3965-4035: 300 x {17,40,64,100}
x 1024, 1023 x n x 4096)."""
import numpy as np
import pytest

import arcint_b200 as A
import oracle as O
from gpu_util import TOL, make_weights, nmse, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = A.Context(0)
    yield c
    c.close()


def run(ctx, t, w, k, x):
    ctx.stats_reset()
    got = ctx.run_mul_mat(t, w, k, x)
    return got, ctx.stats()


@pytest.mark.parametrize("t", [A.Q4_0, A.Q8_0, A.IQ4_NL])
@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (128, 16, 256), (256, 128, 512), (300, 17, 1024), (300, 40, 1024),
                                   (300, 64, 1024), (300, 100, 1024), (1023, 33, 4096), (77, 9, 4096), (512, 300, 2560)])
def test_gemm_tc_matches_oracle(ctx, t, m, n, k):
    rng = np.random.default_rng(m * 7 + n)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1, st                  # the tensor-core path ran, not the fallback
    assert np.isfinite(got).all()
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


@pytest.mark.parametrize("t", [A.Q4_0, A.Q8_0, A.IQ4_NL])
def test_gemm_tc_nmse_against_f32_activations(ctx, t):
    m, n, k = 384, 200, 2048
    w = make_weights(t, m, k, 60 + t)
    x = O.fill_normal(n * k, 61, 1.0).reshape(n, k)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    assert nmse(got, O.mul_mat_f64(t, w, k, x, False)) < 5e-4


def test_gemm_tc_agrees_with_gemv_path(ctx):
    """The same product through the decode kernel (8 columns at a time) and the tensor cores."""
    t, m, n, k = A.Q4_0, 256, 24, 1024
    rng = np.random.default_rng(5)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    got, _ = run(ctx, t, w, k, x)
    parts = np.concatenate([ctx.run_mul_mat(t, w, k, x[i:i + 8]) for i in range(0, n, 8)])
    assert rel_err(got, parts.astype(np.float64)) < 1e-4


def test_gemm_shapes_outside_the_tensor_core_gate_fall_back(ctx):
    """K not a multiple of 256: the product still runs (decode kernel in column groups) and says so."""
    t, m, n, k = A.Q4_0, 64, 20, 2080
    rng = np.random.default_rng(6)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 0 and st.get("gemm_fallback_shape", 0) == 1
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


def test_config1_full_size(ctx):
    """benchmark config 1: Q4_0 4096 x 4096 weights, 512 tokens; sampled rows against the oracle."""
    t, m, n, k = A.Q4_0, 4096, 512, 4096
    w = make_weights(t, m, k, 0x5EED0000)
    x = O.fill_normal(n * k, 0x5EED0100, 1.0).reshape(n, k)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    rows = np.unique(np.concatenate([[0, 1, 127, 128, m - 1], np.random.default_rng(1).integers(0, m, 40)]))
    ref = O.mul_mat_f64(t, w[rows], k, x, True)
    assert rel_err(got[:, rows], ref) < TOL
    assert np.isfinite(got).all()


# ---- IQ4_XS: integer sub-scales folded into two int8 limbs, float once per 256 ----

@pytest.mark.parametrize("m,n,k", [(128, 128, 512), (128, 16, 512), (300, 17, 1024), (300, 100, 1024), (512, 300, 2560),
                                   (1023, 33, 4096), (77, 9, 5120)])
def test_gemm_iq4_xs_matches_oracle(ctx, m, n, k):
    rng = np.random.default_rng(m * 3 + n)
    t = A.IQ4_XS
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1, st
    assert np.isfinite(got).all()
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


def test_gemm_iq4_xs_extreme_codes(ctx):
    """Every sub-scale at its extremes and every nibble equal: the largest limb sums the accumulators see."""
    t, m, n, k = A.IQ4_XS, 128, 32, 512
    rng = np.random.default_rng(1)
    w = O.random_blocks(t, m, k, rng).reshape(m, k // 256, 136)
    w[:, :, 2:8] = 0xFF                                   # ls = 63 everywhere
    w[: m // 2, :, 2:8] = 0x00                            # ... and ls = 0 (factor -32) in half the rows
    w[:, :, 8:] = 0x00                                    # codebook entry -127 everywhere
    w = w.reshape(m, -1)
    x = np.full((n, k), 3.0, dtype=np.float32)
    x[::2] *= -1
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


@pytest.mark.parametrize("m,k,n", [(64, 768, 20), (200, 11008, 40), (129, 256, 9), (1000, 1280, 128)])
def test_gemm_iq4_xs_odd_superblock_count(ctx, m, k, n):
    """An odd number of 136-byte super-blocks makes rows 8-byte multiples only (K = 11008: the down projection of the 7B
    models): staged row by row, one super-block per stage, still on the tensor cores."""
    t = A.IQ4_XS
    rng = np.random.default_rng(2 + m + k)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1 and st.get("gemm_kq_rowcopy", 0) == 1 and st.get("gemm_fallback_shape", 0) == 0, st
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


def test_config3_iq4_xs_full_size(ctx):
    """benchmark config 3: IQ4_XS 17408 x 5120 at 512 tokens; sampled rows against the oracle."""
    t, m, n, k = A.IQ4_XS, 17408, 512, 5120
    base = make_weights(t, 512, k, 0x5EED0002)
    w = np.tile(base, (m // 512, 1))
    x = O.fill_normal(n * k, 0x5EED0102, 1.0).reshape(n, k)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    rows = np.unique(np.concatenate([[0, 127, 128, m - 1], np.random.default_rng(1).integers(0, m, 28)]))
    assert rel_err(got[:, rows], O.mul_mat_f64(t, w[rows], k, x, True)) < TOL
    assert np.isfinite(got).all()


# ---- Q4_K: sc * q as two int8 limbs on the tensor cores, mins term subtracted by a dp4a kernel ----

@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (128, 16, 512), (300, 17, 1024), (300, 100, 1024), (512, 300, 2560),
                                   (1023, 33, 4096), (77, 9, 768), (200, 130, 11008)])
@pytest.mark.parametrize("t", [A.Q4_K, A.Q5_K])
def test_gemm_q4_K_matches_oracle(ctx, t, m, n, k):
    """Q4_K and Q5_K (the same block with a fifth code bit): two-limb tensor-core product plus the mins term."""
    rng = np.random.default_rng(m * 5 + n + t)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1 and st.get("gemm_kq_mins", 0) == 1, st
    assert np.isfinite(got).all()
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


@pytest.mark.parametrize("t,bb", [(A.Q4_K, 144), (A.Q5_K, 176)])
def test_gemm_q4_K_extreme_codes(ctx, t, bb):
    """All scales and mins at 63, all codes at their maximum (15, 31), activations of one sign: the largest limb sums
    and block sums."""
    m, n, k = 128, 32, 512
    rng = np.random.default_rng(3)
    w = O.random_blocks(t, m, k, rng).reshape(m, k // 256, bb)
    w[:, :, 4:16] = 0xFF
    w[: m // 2, :, 16:] = 0xFF
    w[m // 2:, :, 16:] = 0x00
    w = w.reshape(m, -1)
    x = np.full((n, k), 2.5, dtype=np.float32)
    x[1::2] *= -1
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


@pytest.mark.parametrize("t", [A.Q4_K, A.Q5_K])
def test_gemm_q4_K_nmse_and_gemv_agreement(ctx, t):
    m, n, k = 384, 72, 2048
    w = make_weights(t, m, k, 70)
    x = O.fill_normal(n * k, 71, 1.0).reshape(n, k)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    assert nmse(got, O.mul_mat_f64(t, w, k, x, False)) < 5e-4
    parts = np.concatenate([ctx.run_mul_mat(t, w, k, x[i:i + 8]) for i in range(0, n, 8)])
    assert rel_err(got, parts.astype(np.float64)) < TOL


def test_config2_shape_q4_K_prompt(ctx):
    """The decode config's gate/up shape at a prompt width: Q4_K 11008 x 4096, 512 tokens; sampled rows."""
    t, m, n, k = A.Q4_K, 11008, 512, 4096
    base = make_weights(t, 256, k, 0x5EED0003)
    w = np.tile(base, (m // 256, 1))
    x = O.fill_normal(n * k, 0x5EED0103, 1.0).reshape(n, k)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    rows = np.unique(np.concatenate([[0, 127, 128, m - 1], np.random.default_rng(2).integers(0, m, 28)]))
    assert rel_err(got[:, rows], O.mul_mat_f64(t, w[rows], k, x, True)) < TOL


# ---- Q6_K: sc * (q - 32) as two int8 limbs; 210-byte blocks staged through a 224-byte box (K % 2048 == 0) ----

@pytest.mark.parametrize("m,n,k", [(128, 128, 2048), (300, 17, 2048), (300, 100, 4096), (77, 9, 4096), (1023, 33, 6144),
                                   (512, 300, 2048)])
def test_gemm_q6_K_matches_oracle(ctx, m, n, k):
    rng = np.random.default_rng(m * 11 + n)
    t = A.Q6_K
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1 and st.get("gemm_kq_mins", 0) == 0, st
    assert np.isfinite(got).all()
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


def test_gemm_q6_K_extreme_codes_and_other_k_fall_back(ctx):
    """Scales at -128 / 127 with codes 0 / 63 (the largest limb sums); a K that is not a multiple of 2048 walks the GEMV."""
    t, m, n, k = A.Q6_K, 128, 32, 2048
    rng = np.random.default_rng(4)
    w = O.random_blocks(t, m, k, rng).reshape(m, k // 256, 210)
    w[:, :, 192:208] = 0x80                               # every scale -128
    w[m // 2:, :, 192:208] = 0x7F                         # ... and 127 in the other half of the rows
    w[:, :, :192] = 0x00                                  # code 0 (q - 32 = -32)
    w[::2, :, :192] = 0xFF                                # code 63 in every other row
    w = w.reshape(m, -1)
    x = np.full((n, k), 1.5, dtype=np.float32)
    x[::2] *= -1
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL
    k2 = 1280
    w2 = O.random_blocks(t, 64, k2, rng)
    x2 = rng.normal(0, 1, size=(20, k2)).astype(np.float32)
    got2, st2 = run(ctx, t, w2, k2, x2)
    # five super-blocks: 1050-byte rows, not a 16-byte multiple -- staged row by row, still on the tensor cores
    assert st2.get("gemm_tc", 0) == 1 and st2.get("gemm_kq_rowcopy", 0) == 1 and st2.get("gemm_fallback_shape", 0) == 0
    assert rel_err(got2, O.mul_mat_f64(t, w2, k2, x2, True)) < TOL


@pytest.mark.parametrize("m,k,n", [(200, 11008, 40), (129, 256, 9), (64, 3328, 300), (1000, 1280, 128)])
def test_gemm_q6_k_rows_that_are_not_16_byte_multiples(ctx, m, k, n):
    """Q6_K rows of 210-byte blocks are 16-byte multiples only when K is a multiple of 2048. Other lengths (K = 11008, the
    down projection of the 7B models) are staged row by row from the 16-byte boundary below each row's block; every row
    then sits at its own offset inside its slot. Ragged M and N, one and many super-blocks, odd block counts."""
    t = A.Q6_K
    rng = np.random.default_rng(m + k + n)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1 and st.get("gemm_kq_rowcopy", 0) == 1 and st.get("gemm_fallback_shape", 0) == 0, st
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


def test_config2_head_q6_K_prompt(ctx):
    """The decode config's LM head at a prompt width: Q6_K 32000 x 4096, 128 tokens; sampled rows, NMSE against f32 activations."""
    t, m, n, k = A.Q6_K, 32000, 128, 4096
    base = make_weights(t, 256, k, 0x5EED0004)
    w = np.tile(base, (m // 256, 1))
    x = O.fill_normal(n * k, 0x5EED0104, 1.0).reshape(n, k)
    got, st = run(ctx, t, w, k, x)
    assert st.get("gemm_tc", 0) == 1
    rows = np.unique(np.concatenate([[0, 127, 128, m - 1], np.random.default_rng(3).integers(0, m, 28)]))
    assert rel_err(got[:, rows], O.mul_mat_f64(t, w[rows], k, x, True)) < TOL
    assert nmse(got[:, rows], O.mul_mat_f64(t, w[rows], k, x, False)) < 5e-4


@pytest.mark.parametrize("t,m,k,n", [(A.Q4_0, 300, 1024, 100), (A.Q8_0, 256, 2048, 129), (A.Q4_0, 128, 4096, 16)])
def test_fp16_and_int8_arms_give_identical_results(t, m, k, n):
    """The per-32 prompt GEMM has two arms: int8 operands (tcgen05 kind::i8, int32 block dots converted to float)
    and integer-valued fp16 operands (kind::f16, f32 block dots). Every product and partial sum of a 32-block is
    an integer below 2^24, so both give the same float for every block dot and the outputs must match bit for bit."""
    import os
    w = make_weights(t, m, k, 700 + t)
    x = np.random.default_rng(n).normal(0, 1, size=(n, k)).astype(np.float32)
    outs = {}
    for arm in ("f16", "i8"):
        if arm == "i8":
            os.environ["B200Q_TC_I8"] = "1"
        try:
            with A.Context(0) as c:
                outs[arm] = c.run_mul_mat(t, w, k, x)
                st = c.stats()
                assert st.get("gemm_tc") == 1 and (st.get("gemm_tc_f16", 0) == 1) == (arm == "f16"), st
        finally:
            os.environ.pop("B200Q_TC_I8", None)
    assert np.array_equal(outs["f16"], outs["i8"])
    assert rel_err(outs["f16"], O.mul_mat_f64(t, w, k, x, True)) < TOL
