"""The allocation-free decode attention entry point against the ordinary one.

B200LmOps_AttentionDecodeStatic is meant for callers that cannot allocate device memory when
they call in (inside another runtime's callback, a warm serving loop that bans allocator
calls, a process whose GPU memory is fully pre-assigned).  It keeps its split partials in a
fixed array inside the library instead of allocating them.  Here it runs twice in a row on
different inputs -- the shared array still holds the first call's partials during the second --
and each result must equal what B200LmOps_Attention (which allocates its scratch) returns.
The file name makes pytest collect it last.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def to_pages(x, hkv, hd, bf16):
    """[S][hkv][hd] -> paged layout [page][hkv][256][hd] (zero padded)."""
    import torch
    s = x.shape[0]
    npages = (s + 255) // 256
    buf = np.zeros((npages * 256, hkv, hd), dtype=np.float32)
    buf[:s] = x
    pages = buf.reshape(npages, 256, hkv, hd).transpose(0, 2, 1, 3).copy()
    t = torch.from_numpy(pages).cuda()
    return t.to(torch.bfloat16).contiguous() if bf16 else t.contiguous()


@pytest.mark.parametrize("hq,hkv,hd,window,kv_bf16,nsplit", [(4, 1, 256, 0, False, 16), (8, 4, 128, 48, True, 4)])
def test_static_scratch_attention_matches_allocating_entry_point(pkg, orc, hq, hkv, hd, window, kv_bf16, nsplit):
    import torch
    rng = np.random.Generator(np.random.PCG64(17))
    for call, (batch, s) in enumerate([(3, 700), (2, 333)]):          # two calls in a row, different shapes
        q = rng.standard_normal((batch, hq, hd), dtype=np.float32)
        k = rng.standard_normal((s, hkv, hd), dtype=np.float32)
        v = rng.standard_normal((s, hkv, hd), dtype=np.float32)
        want, _ = pkg.ops.attention(q, k, v, window=window, kv_bf16=kv_bf16, nsplit=nsplit)
        rows = np.zeros((batch, (hq + 2 * hkv) * hd), dtype=np.float32)
        rows[:, :hq * hd] = q.reshape(batch, -1)
        q_dev = torch.from_numpy(rows).cuda()
        kp, vp = to_pages(k, hkv, hd, kv_bf16), to_pages(v, hkv, hd, kv_bf16)
        ptab = torch.arange((s + 255) // 256, dtype=torch.int32, device="cuda")
        out = torch.full((batch, hq, hd), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        pkg.ops.attention_decode_static(q_dev.data_ptr(), kp.data_ptr(), vp.data_ptr(), ptab.data_ptr(), out.data_ptr(),
                                        batch, s, hq, hkv, hd, window=window, kv_bf16=kv_bf16, nsplit=nsplit)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.isfinite(got).all(), call
        assert np.abs(got - want).max() < 2e-4, (call, np.abs(got - want).max())
        assert pkg.ops.attention_decode_static_status() == 0          # the error word its kernels keep is clean
        # ... and against the CPU oracle directly (every query sits at position s - 1); a bf16 cache
        # carries the rounding of K and V, so the oracle sees the rounded rows
        if kv_bf16:
            k = torch.from_numpy(k).to(torch.bfloat16).float().numpy()
            v = torch.from_numpy(v).to(torch.bfloat16).float().numpy()
        for b in range(batch):
            ref = orc.attention(q[b:b + 1], k, v, s - 1, window)
            assert np.abs(got[b:b + 1] - ref).max() < 2e-4, (call, b, np.abs(got[b:b + 1] - ref).max())
        # the allocating entry point at a much smaller shape in between: it must not shrink a kernel
        # limit that the next static call (head_dim 256, group of 4) depends on
        qs = rng.standard_normal((1, 1, 32), dtype=np.float32)
        ks = rng.standard_normal((40, 1, 32), dtype=np.float32)
        small, _ = pkg.ops.attention(qs, ks, ks, nsplit=2)
        assert np.abs(small - orc.attention(qs, ks, ks, 39, 0)).max() < 2e-4


def test_static_scratch_limits_are_enforced(pkg):
    import torch
    dummy = torch.zeros(16, device="cuda")
    ptr = dummy.data_ptr()
    with pytest.raises(pkg.StatusError) as e:      # 4096 queries x 4 heads x 64 splits x 258 floats > 8 MiB
        pkg.ops.attention_decode_static(ptr, ptr, ptr, ptr, ptr, 4096, 1024, 4, 1, 256, nsplit=64)
    assert e.value.code == pkg.INVALID_ARGUMENT and "static scratch" in e.value.message
    with pytest.raises(pkg.StatusError) as e:
        pkg.ops.attention_decode_static(ptr, ptr, ptr, ptr, ptr, 20000, 1024, 4, 1, 32, nsplit=1)
    assert e.value.code == pkg.INVALID_ARGUMENT
