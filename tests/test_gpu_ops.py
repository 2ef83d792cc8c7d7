"""Operator parity on a B200, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bf16_round(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def make_matrix(mio, n, k, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return mio.quantize_int4(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))


@pytest.mark.parametrize("n,k", [(16, 64), (96, 128), (1536, 1152), (1152, 6912), (4096, 384)])
def test_int4_unpack_is_bit_exact(pkg, orc, mio, n, k):
    packed, _ = make_matrix(mio, n, k, n + k)
    got = pkg.ops.unpack_w4(packed)
    assert got.dtype == np.int8 and np.array_equal(got, orc.unpack_int4(packed))


@pytest.mark.parametrize("n,k,ncols,nterms,kslices", [
    (96, 64, 1, 3, 1), (1536, 1152, 1, 3, 1), (1152, 1024, 1, 3, 4), (1152, 6912, 1, 3, 2),
    (13824, 1152, 1, 3, 1), (4096, 384, 2, 3, 1), (1152, 1024, 4, 2, 2), (2048, 512, 3, 2, 1), (512, 256, 1, 1, 1),
    (512, 256, 1, 2, 1), (262144 // 8, 1152, 1, 3, 1),
])
def test_decode_gemv_matches_oracle(pkg, orc, mio, n, k, ncols, nterms, kslices):
    packed, scale = make_matrix(mio, n, k, 3 * n + k)
    rng = np.random.Generator(np.random.PCG64(99))
    x = rng.standard_normal((ncols, k), dtype=np.float32)
    x[:, ::7] *= 5.0
    want = orc.matmul_w4(packed, scale, x)
    got = pkg.ops.gemv_w4(packed, scale, x, nterms=nterms, kslices=kslices)
    tol = {3: 2e-5, 2: 2e-3, 1: 6e-2}[nterms]
    for c in range(ncols):
        denom = np.abs(want[c]).max()
        assert np.abs(got[c] - want[c]).max() / denom < tol, (c, np.abs(got[c] - want[c]).max() / denom)


def test_decode_gemv_zero_and_constant_inputs(pkg, orc, mio):
    packed, scale = make_matrix(mio, 64, 128, 5)
    x0 = np.zeros((1, 128), np.float32)
    assert np.all(pkg.ops.gemv_w4(packed, scale, x0) == 0)
    x1 = np.full((1, 128), 0.25, np.float32)
    np.testing.assert_allclose(pkg.ops.gemv_w4(packed, scale, x1), orc.matmul_w4(packed, scale, x1), rtol=1e-5, atol=1e-7)


def test_decode_gemv_is_deterministic(pkg, mio):
    packed, scale = make_matrix(mio, 1152, 6912, 8)
    x = np.random.Generator(np.random.PCG64(1)).standard_normal((1, 6912), dtype=np.float32)
    a = pkg.ops.gemv_w4(packed, scale, x, kslices=2)
    b = pkg.ops.gemv_w4(packed, scale, x, kslices=2)
    assert np.array_equal(a, b)            # integer accumulation: order cannot matter


@pytest.mark.parametrize("t,n,k", [(5, 96, 64), (40, 192, 128), (64, 384, 1024)])
def test_check_gemm_matches_oracle(pkg, orc, mio, t, n, k):
    packed, scale = make_matrix(mio, n, k, n * 3 + k)
    a = bf16_round(np.random.Generator(np.random.PCG64(t)).standard_normal((t, k), dtype=np.float32))
    want = orc.matmul_w4(packed, scale, a)
    got, _ = pkg.ops.gemm_w4(packed, scale, a, mode=pkg.GEMM_CHECK)
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-5


def test_check_gemm_geglu(pkg, orc, mio):
    t, ffn, k = 9, 128, 64
    gp, gs = make_matrix(mio, ffn, k, 1)
    up, us = make_matrix(mio, ffn, k, 2)
    a = bf16_round(np.random.Generator(np.random.PCG64(3)).standard_normal((t, k), dtype=np.float32))
    g = orc.matmul_w4(gp, gs, a).astype(np.float64)
    u = orc.matmul_w4(up, us, a).astype(np.float64)
    want = 0.5 * g * (1 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * u
    got = pkg.ops.gemm_geglu_w4(gp, gs, up, us, a, mode=pkg.GEMM_CHECK)
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-2          # output stored as bf16


@pytest.mark.parametrize("hq,hkv,hd,t,s,qpos0,window,kv_bf16", [
    (4, 1, 256, 16, 300, 284, 0, False),       # global, queries at the end of the cache
    (4, 1, 256, 40, 600, 560, 512, False),     # window 512, crosses two pages
    (4, 1, 32, 8, 20, 12, 8, False),           # tiny-model geometry
    (8, 4, 128, 12, 200, 188, 48, True),       # several kv heads, bf16 pages
    (2, 2, 64, 5, 5, 0, 0, False),             # no grouping, query i sees keys 0..i
    (4, 1, 256, 3, 700, 0, 0, False),          # queries at the start: 1, 2, 3 keys
])
def test_prefill_attention_matches_oracle(pkg, orc, hq, hkv, hd, t, s, qpos0, window, kv_bf16):
    rng = np.random.Generator(np.random.PCG64(2))
    q = rng.standard_normal((t, hq, hd), dtype=np.float32)
    k = rng.standard_normal((s, hkv, hd), dtype=np.float32)
    v = rng.standard_normal((s, hkv, hd), dtype=np.float32)
    kk, vv = (bf16_round(k), bf16_round(v)) if kv_bf16 else (k, v)
    want = orc.attention(q, kk, vv, qpos0, window)
    got, _ = pkg.ops.attention(q, k, v, qpos0=qpos0, window=window, kv_bf16=kv_bf16, nsplit=1)
    assert np.abs(got - want).max() < 2e-4, np.abs(got - want).max()


@pytest.mark.parametrize("hq,hkv,hd,s,window", [
    (4, 1, 256, 300, 0),         # global causal, two pages, ragged last tile
    (4, 1, 256, 700, 512),       # window 512: tiles fall out of the window on the left
    (8, 4, 128, 200, 48),        # several kv heads, G = 2, head_dim 128
    (2, 2, 128, 130, 0),         # no grouping: 128-token tiles, two of them
    (4, 1, 256, 1023, 0),        # the benchmark's prefill length
])
def test_tensor_core_prefill_attention_matches_oracle(pkg, orc, hq, hkv, hd, s, window):
    """The tcgen05 flash kernel (bf16 operands, bf16 probabilities) against the fp32 oracle on
    bf16-rounded inputs.  Tolerance: bf16 rounding of P and of the output, 3e-2 absolute on
    outputs of unit scale."""
    rng = np.random.Generator(np.random.PCG64(2))
    q = rng.standard_normal((s, hq, hd), dtype=np.float32)
    k = rng.standard_normal((s, hkv, hd), dtype=np.float32)
    v = rng.standard_normal((s, hkv, hd), dtype=np.float32)
    want = orc.attention(bf16_round(q), bf16_round(k), bf16_round(v), 0, window)
    got, _ = pkg.ops.attention_prefill_tc(q, k, v, window=window)
    assert np.isfinite(got).all()
    err = np.abs(got - want).max()
    assert err < 3e-2, err
    # the first token attends to itself only: its output is v[0] (bf16-rounded twice)
    assert np.abs(got[0] - np.repeat(bf16_round(v[0]), hq // hkv, axis=0)).max() < 2e-2


def test_tensor_core_prefill_attention_rejects_unbounded_scores(pkg):
    q = np.full((64, 4, 256), 3.0, dtype=np.float32)
    k = np.full((64, 1, 256), 3.0, dtype=np.float32)
    with pytest.raises(pkg.StatusError) as e:
        pkg.ops.attention_prefill_tc(q, k, k)
    assert e.value.code == pkg.FAILED_PRECONDITION


@pytest.mark.parametrize("hq,hkv,hd,batch,s,window,kv_bf16,nsplit", [
    (4, 1, 256, 1, 1100, 0, False, 32), (4, 1, 256, 1, 1100, 512, False, 8), (4, 1, 256, 4, 4096, 0, True, 16),
    (8, 4, 128, 3, 300, 48, True, 4), (4, 1, 32, 2, 7, 8, False, 2), (4, 1, 256, 2, 5, 0, False, 32),
])
def test_split_kv_decode_attention_matches_oracle(pkg, orc, hq, hkv, hd, batch, s, window, kv_bf16, nsplit):
    """Batch of single-token queries at position s-1; more splits than keys is legal (empty splits)."""
    rng = np.random.Generator(np.random.PCG64(4))
    q = rng.standard_normal((batch, hq, hd), dtype=np.float32)
    k = rng.standard_normal((s, hkv, hd), dtype=np.float32)
    v = rng.standard_normal((s, hkv, hd), dtype=np.float32)
    kk, vv = (bf16_round(k), bf16_round(v)) if kv_bf16 else (k, v)
    want = np.concatenate([orc.attention(q[i:i + 1], kk, vv, s - 1, window) for i in range(batch)])
    got, _ = pkg.ops.attention(q, k, v, window=window, kv_bf16=kv_bf16, nsplit=nsplit)
    assert np.abs(got - want).max() < 2e-4, np.abs(got - want).max()
    # a batch of independent sequences (own cache copy and page table each) gives the same rows, bit for bit
    own, _ = pkg.ops.attention(q, k, v, window=window, kv_bf16=kv_bf16, nsplit=nsplit, private_caches=True)
    assert np.array_equal(own, got)
    # the streaming kernel of the wide decode step on the same request
    st, _ = pkg.ops.attention(q, k, v, window=window, kv_bf16=kv_bf16, nsplit=nsplit, streaming_kernel=True)
    assert np.abs(st - want).max() < 2e-4, np.abs(st - want).max()
    st, _ = pkg.ops.attention(q, k, v, window=window, kv_bf16=kv_bf16, nsplit=nsplit, streaming_kernel=True, private_caches=True)
    assert np.abs(st - want).max() < 2e-4, np.abs(st - want).max()
