"""Host-side logic of the CUDA library, exercised without a GPU: the C ABI exports, the
tile repacks (checked by re-deriving every element from the documented layouts), input
validation and the loud failure when no CUDA device exists."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def test_every_declared_symbol_is_exported(pkg):
    lib = pkg.load_library()
    declared = []
    for hdr in ("b200lm.h", "b200lm_ops.h"):
        text = open(os.path.join(ROOT, "include", hdr)).read()
        declared += re.findall(r"\b(B200Lm(?:Ops)?_[A-Za-z0-9]+)\s*\(", text)
    assert len(set(declared)) >= 20
    for name in set(declared):
        assert hasattr(lib, name), name


def test_header_compiles_as_c():
    src = '#include "b200lm.h"\n#include "b200lm_ops.h"\nint main(void){return sizeof(B200LmConfig) > 0 ? 0 : 1;}\n'
    r = subprocess.run(["/usr/bin/gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                        "-x", "c", "-", "-fsyntax-only"], input=src, text=True, capture_output=True)
    assert r.returncode == 0, r.stderr


def w4t_elements(buf, n, k):
    """Expands the decode layout exactly as documented: 16x64 tiles of 512 bytes, lane 4g+t,
    word j covers k = 32*(j/2) + 16*(j%2) + 4t + i, nibble 2i = row g, 2i+1 = row g+8, two's complement."""
    words = buf.view(np.uint32).reshape(n // 16, k // 64, 32, 4)
    out = np.zeros((n, k), dtype=np.int8)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for j in range(4):
            w = words[:, :, lane, j]
            for i in range(4):
                kk = 32 * (j // 2) + 16 * (j % 2) + 4 * t + i
                lo = ((w >> (8 * i)) & 0xF).astype(np.int16)
                hi = ((w >> (8 * i + 4)) & 0xF).astype(np.int16)
                lo = np.where(lo >= 8, lo - 16, lo)
                hi = np.where(hi >= 8, hi - 16, hi)
                out[g::16, kk::64] = lo
                out[g + 8::16, kk::64] = hi
    return out


def w4g_elements(buf, n_pad, k):
    """128-row x 64-k blocks of 4096 bytes; word wi of a row holds k = 8*wi + e with nibble
    order k0,k2,k4,k6,k1,k3,k5,k7, each q+8."""
    words = buf.view(np.uint32).reshape(n_pad // 128, k // 64, 128, 8)
    out = np.zeros((n_pad, k), dtype=np.int8)
    for wi in range(8):
        for e in range(8):
            nib = 4 + (e >> 1) if e & 1 else e >> 1
            v = ((words[:, :, :, wi] >> (4 * nib)) & 0xF).astype(np.int16) - 8      # [tiles, kb, 128]
            out.reshape(n_pad // 128, 128, k // 64, 64)[:, :, :, wi * 8 + e] = v.transpose(0, 2, 1)
    return out


@pytest.mark.parametrize("n,k", [(16, 64), (96, 128), (48, 1152), (256, 192)])
def test_repack_w4t_is_a_permutation_of_the_canonical_values(pkg, mio, n, k):
    rng = np.random.Generator(np.random.PCG64(n * 7 + k))
    packed, _ = mio.quantize_int4(rng.standard_normal((n, k), dtype=np.float32))
    buf = pkg.ops.repack_w4t(packed)
    assert buf.size == n * k // 2
    assert np.array_equal(w4t_elements(buf, n, k), mio.unpack_int4(packed))


@pytest.mark.parametrize("n,k", [(128, 64), (96, 128), (300, 256)])
def test_repack_w4g_matches_layout_and_pads_with_zero_weights(pkg, mio, n, k):
    rng = np.random.Generator(np.random.PCG64(n + k))
    packed, _ = mio.quantize_int4(rng.standard_normal((n, k), dtype=np.float32))
    buf = pkg.ops.repack_w4g(packed)
    n_pad = (n + 127) // 128 * 128
    got = w4g_elements(buf, n_pad, k)
    assert np.array_equal(got[:n], mio.unpack_int4(packed))
    assert np.all(got[n:] == 0)


def test_repack_rejects_bad_shapes(pkg):
    with pytest.raises(pkg.StatusError) as e:
        pkg.ops.repack_w4t(np.zeros((16, 10), np.uint8))       # k = 20, not a multiple of 64
    assert e.value.code == pkg.INVALID_ARGUMENT


def test_create_rejects_malformed_images(pkg, mio, models):
    _, rec, img = models("tiny")
    cases = [
        (b"NOTLITER" + b"\0" * 100, pkg.INVALID_ARGUMENT),                  # bad magic
        (img[:20000], pkg.INVALID_ARGUMENT),                                # truncated section
        (mio.write_litertlm([(mio.SECTION_GENERIC, b"no weights here", [])]), pkg.NOT_FOUND),
    ]
    major2 = bytearray(img); major2[8] = 2
    cases.append((bytes(major2), pkg.UNIMPLEMENTED))
    bad_rec = bytearray(rec); bad_rec[16 + 4 * 4] = 48                      # head_dim 48
    cases.append((bytes(bad_rec), pkg.UNIMPLEMENTED))
    for data, code in cases:
        with pytest.raises(pkg.StatusError) as e:
            pkg.B200LlmExecutor(data)
        assert e.value.code == code, (code, str(e.value))
    with pytest.raises(pkg.StatusError) as e:
        pkg.B200LlmExecutor("/nonexistent/model.litertlm")
    assert e.value.code == pkg.NOT_FOUND


@pytest.mark.skipif(_has_gpu(), reason="checks the no-GPU failure path")
def test_no_gpu_means_failed_precondition_not_a_fallback(pkg, models):
    _, _, img = models("tiny")
    with pytest.raises(pkg.StatusError) as e:
        pkg.B200LlmExecutor(img)
    assert e.value.code == pkg.FAILED_PRECONDITION and "no CPU fallback" in e.value.message
    with pytest.raises(pkg.StatusError) as e:
        pkg.ops.unpack_w4(np.zeros((16, 32), np.uint8))
    assert e.value.code == pkg.FAILED_PRECONDITION


def test_missing_library_fails_loudly(pkg, monkeypatch):
    monkeypatch.setattr(pkg, "_lib", None)
    monkeypatch.setattr(pkg, "LIB_PATH", "/nonexistent/libb200lm.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        pkg.load_library()


def test_null_handle_calls_are_rejected(pkg):
    lib = pkg.load_library()
    err = ctypes.c_char_p()
    v = ctypes.c_int32()
    assert lib.B200Lm_GetVocabSize(None, ctypes.byref(v), ctypes.byref(err)) == pkg.INVALID_ARGUMENT
    assert err.value
    assert lib.B200Lm_Reset(None, None) == pkg.INVALID_ARGUMENT        # err pointer is optional
    lib.B200Lm_Destroy(None)


def test_algorithmic_work_formulas(mio):
    cfg = mio.config_gemma3_1b()
    assert cfg.layer_params() * cfg.n_layers // 2 == 348_880_896
    assert cfg.vocab * cfg.d_model // 2 == 150_994_944
    assert cfg.decode_bytes_per_token() == 536_848_896
    assert abs(cfg.prefill_flops(1024) - 1.473e12) / 1.473e12 < 2e-3


def test_xnnpack_timing_baseline_tracks_the_oracle(orc, models):
    """The XNNPACK leg of the CPU arm (int8 activations) is a timing baseline, not a parity reference, but it must
    compute the same model: same arg-max and a high cosine on a small case.  Skipped where torch's XNNPACK symbols
    cannot be bound."""
    import numpy as np
    cfg, rec, _ = models("small")
    ids = np.random.Generator(np.random.PCG64(5)).integers(0, cfg.vocab, 48).astype(np.int32)
    ref = orc.OracleExecutor(orc.OracleModel(rec))
    assert ref.prefill(ids) == 0
    rc, want = ref.decode_logits()
    assert rc == 0
    if not orc.use_xnnpack(2):
        orc.use_plain_matmul()
        import pytest
        pytest.skip("XNNPACK symbols of libtorch_cpu.so not available")
    try:
        ex = orc.OracleExecutor(orc.OracleModel(rec))
        assert ex.prefill(ids) == 0
        rc, got = ex.decode_logits()
        assert rc == 0
    finally:
        orc.use_plain_matmul()
    cos = float(np.dot(got, want) / (np.linalg.norm(got) * np.linalg.norm(want)))
    assert cos >= 0.995 and int(np.argmax(got)) == int(np.argmax(want))
    # and the hook is gone again: the oracle is bit-identical to before
    ex = orc.OracleExecutor(orc.OracleModel(rec))
    assert ex.prefill(ids) == 0
    assert np.array_equal(ex.decode_logits()[1], want)
