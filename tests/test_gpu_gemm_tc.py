"""The TMA + tcgen05 int4 GEMM against the oracle and against the check GEMM."""
import numpy as np
import pytest

from test_gpu_ops import bf16_round, make_matrix

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,n,k,ksplit", [
    (128, 128, 64, 1), (128, 128, 256, 1), (100, 96, 128, 1), (1, 128, 64, 1), (300, 1536, 1152, 1),
    (257, 1152, 1024, 4), (200, 1152, 6912, 4), (64, 384, 1024, 2), (130, 2064, 384, 1),
])
def test_tcgen05_gemm_matches_oracle(pkg, orc, mio, t, n, k, ksplit):
    packed, scale = make_matrix(mio, n, k, 5 * n + k)
    a = bf16_round(np.random.Generator(np.random.PCG64(t + 1)).standard_normal((t, k), dtype=np.float32))
    want = orc.matmul_w4(packed, scale, a)
    got, _ = pkg.ops.gemm_w4(packed, scale, a, mode=pkg.GEMM_TCGEN05, ksplit=ksplit)
    # int4 weights and bf16 activations are exact in the MMA; only fp32 accumulation order differs
    assert np.abs(got - want).max() / np.abs(want).max() < 2e-5, np.abs(got - want).max() / np.abs(want).max()


def test_tcgen05_gemm_agrees_with_check_gemm(pkg, mio):
    packed, scale = make_matrix(mio, 768, 384, 77)
    a = bf16_round(np.random.Generator(np.random.PCG64(6)).standard_normal((150, 384), dtype=np.float32))
    tc, _ = pkg.ops.gemm_w4(packed, scale, a, mode=pkg.GEMM_TCGEN05)
    ck, _ = pkg.ops.gemm_w4(packed, scale, a, mode=pkg.GEMM_CHECK)
    assert np.abs(tc - ck).max() / np.abs(ck).max() < 2e-5


@pytest.mark.parametrize("t,ffn,k", [(128, 64, 64), (70, 128, 64), (300, 1024, 384), (129, 6912, 1152)])
def test_tcgen05_geglu_epilogue(pkg, orc, mio, t, ffn, k):
    gp, gs = make_matrix(mio, ffn, k, 1)
    up, us = make_matrix(mio, ffn, k, 2)
    a = bf16_round(np.random.Generator(np.random.PCG64(3)).standard_normal((t, k), dtype=np.float32))
    g = orc.matmul_w4(gp, gs, a).astype(np.float64)
    u = orc.matmul_w4(up, us, a).astype(np.float64)
    want = 0.5 * g * (1 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * u
    got = pkg.ops.gemm_geglu_w4(gp, gs, up, us, a, mode=pkg.GEMM_TCGEN05)
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-2          # output stored as bf16


def test_tcgen05_linearity_at_full_size(pkg, mio):
    """Size-independent property at the 1B model's largest projection: G(a + b) = G(a) + G(b)
    for activations that stay exact in bf16."""
    n, k, t = 13824, 1152, 1024
    packed, scale = make_matrix(mio, n, k, 9)
    rng = np.random.Generator(np.random.PCG64(10))
    a = rng.integers(-8, 9, (t, k)).astype(np.float32)
    b = rng.integers(-8, 9, (t, k)).astype(np.float32)
    ga, _ = pkg.ops.gemm_w4(packed, scale, a, mode=pkg.GEMM_TCGEN05)
    gb, _ = pkg.ops.gemm_w4(packed, scale, b, mode=pkg.GEMM_TCGEN05)
    gab, _ = pkg.ops.gemm_w4(packed, scale, a + b, mode=pkg.GEMM_TCGEN05)
    assert np.abs(gab - (ga + gb)).max() / np.abs(gab).max() < 1e-6
