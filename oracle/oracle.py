"""ctypes binding of the CPU oracle (``oracle/oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  The CUDA executor never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import List, Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_xnnb = None


def build_xnnpack_baseline() -> str:
    """Compiles xnn_baseline.c against torch's copy of xnnpack.h (no torch import: the header path comes from the
    package's location).  Raises when the header or the compiler is missing."""
    import importlib.util
    spec = importlib.util.find_spec("torch")
    if spec is None or not spec.origin:
        raise RuntimeError("torch is not installed: no xnnpack.h to compile against")
    inc = os.path.join(os.path.dirname(spec.origin), "include")
    out = os.path.join(_HERE, "libxnnb.so")
    src = os.path.join(_HERE, "xnn_baseline.c")
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libxnnb.so", f"TORCH_INC={inc}"], stdout=subprocess.DEVNULL,
                              stderr=subprocess.DEVNULL)
    return out


def use_xnnpack(threads: int) -> bool:
    """Timing baseline only: routes the oracle's matrix products through XNNPACK's fully-connected operator with
    dynamically quantised int8 activations (the XNNPACK build inside torch) on a pool of `threads` workers, and
    limits the OpenMP parts to the same count.  False when it cannot be set up."""
    global _xnnb
    try:
        out = build_xnnpack_baseline()
        import torch  # noqa: F401  (loads libtorch_cpu.so, which exports the xnn_* symbols)
        if _xnnb is None:
            _xnnb = C.CDLL(out, mode=C.RTLD_GLOBAL)
            _xnnb.xnnb_init.argtypes = [C.c_int, C.c_char_p]
            _xnnb.xnnb_init.restype = C.c_int
        cpu_lib = os.path.join(os.path.dirname(torch.__file__), "lib", "libtorch_cpu.so")
        if _xnnb.xnnb_init(int(threads), cpu_lib.encode()) != 0:
            return False
        lib().orc_set_matmul_hook(C.cast(_xnnb.xnnb_matmul, C.c_void_p))
        lib().orc_set_threads(int(threads))
        return True
    except Exception:
        return False


def use_plain_matmul(threads: int = 0) -> None:
    """Back to the oracle's own matrix product (the parity configuration)."""
    lib().orc_set_matmul_hook(None)
    if threads:
        lib().orc_set_threads(int(threads))


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        vp, i32p, f32p, u8p, i8p = C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_float), \
            C.POINTER(C.c_uint8), C.POINTER(C.c_int8)
        sig = {
            "orc_unpack_int4": (None, [vp, C.c_int64, C.c_int64, vp]),
            "orc_quantize_int4": (None, [vp, C.c_int64, C.c_int64, vp, vp]),
            "orc_kv_index": (None, [C.c_int, i32p, i32p]),
            "orc_kv_offset": (C.c_int64, [C.c_int] * 5),
            "orc_greedy": (C.c_int, [vp, C.c_int64, C.c_int, vp]),
            "orc_softmax": (C.c_int, [vp, C.c_int64, vp, C.c_int64, C.c_float, C.c_int, vp, vp]),
            "orc_plan_work_groups": (C.c_int, [vp, C.c_int, C.c_int, vp, vp, C.c_int]),
            "orc_fill_mask": (None, [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
            "orc_rope_table": (None, [C.c_double, C.c_int, C.c_int, vp, vp]),
            "orc_model_create": (vp, [vp, C.c_uint64]),
            "orc_model_destroy": (None, [vp]),
            "orc_model_cfg": (None, [vp, vp]),
            "orc_exec_create": (vp, [vp]),
            "orc_exec_destroy": (None, [vp]),
            "orc_exec_prefill": (C.c_int, [vp, vp, C.c_int]),
            "orc_exec_decode_logits": (C.c_int, [vp, vp, vp]),
            "orc_exec_decode_token": (C.c_int, [vp, vp, vp]),
            "orc_exec_reset": (None, [vp]),
            "orc_exec_current_step": (C.c_int, [vp]),
            "orc_exec_internal_step": (C.c_int, [vp]),
            "orc_exec_pending_token": (C.c_int, [vp]),
            "orc_exec_last_plan": (C.c_int, [vp, vp, vp]),
            "orc_exec_read_kv": (None, [vp, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
            "orc_matmul_w4": (None, [vp, vp, C.c_int, C.c_int, vp, C.c_int, vp]),
            "orc_attention": (None, [vp, vp, vp] + [C.c_int] * 7 + [vp]),
            "orc_set_matmul_hook": (None, [vp]),
            "orc_set_threads": (None, [C.c_int]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _p(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


# ---------------------------------------------------------------- free functions

def unpack_int4(packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    n, kb = packed.shape
    out = np.empty((n, kb * 2), dtype=np.int8)
    lib().orc_unpack_int4(_p(packed), n, kb * 2, _p(out))
    return out


def quantize_int4(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    packed = np.empty((n, k // 2), dtype=np.uint8)
    scale = np.empty(n, dtype=np.float32)
    lib().orc_quantize_int4(_p(w), n, k, _p(packed), _p(scale))
    return packed, scale


def kv_index(pos: int) -> Tuple[int, int]:
    page, slot = C.c_int32(), C.c_int32()
    lib().orc_kv_index(pos, C.byref(page), C.byref(slot))
    return page.value, slot.value


def kv_offset(phys_page: int, kv_head: int, slot: int, n_kv_heads: int, head_dim: int) -> int:
    return lib().orc_kv_offset(phys_page, kv_head, slot, n_kv_heads, head_dim)


def greedy(logits: np.ndarray, batch: int = 1) -> np.ndarray:
    logits = np.ascontiguousarray(logits, dtype=np.float32).ravel()
    out = np.empty(batch, dtype=np.int32)
    rc = lib().orc_greedy(_p(logits), logits.size, batch, _p(out))
    if rc:
        raise ValueError(f"status {rc}")
    return out


def softmax(logits, topk, temperature: float, batch: int) -> Tuple[np.ndarray, np.ndarray]:
    logits = np.ascontiguousarray(logits, dtype=np.float32).ravel()
    topk = np.ascontiguousarray(topk, dtype=np.int32).ravel()
    probs = np.empty(topk.size, dtype=np.float32)
    mx = np.empty(batch, dtype=np.float32)
    rc = lib().orc_softmax(_p(logits), logits.size, _p(topk), topk.size, temperature, batch, _p(probs), _p(mx))
    if rc:
        raise ValueError(f"status {rc}")
    return probs, mx


def plan_work_groups(buckets, input_length: int) -> List[Tuple[int, int]]:
    b = np.ascontiguousarray(sorted(buckets, reverse=True), dtype=np.int32)
    ob = np.empty(256, dtype=np.int32)
    ol = np.empty(256, dtype=np.int32)
    n = lib().orc_plan_work_groups(_p(b), b.size, input_length, _p(ob), _p(ol), 256)
    if n < 0:
        raise ValueError("too many groups")
    return [(int(ob[i]), int(ol[i])) for i in range(n)]


def fill_mask(rows: int, ctx: int, start: int, steps: int, is_f16: bool = True) -> np.ndarray:
    m = np.empty((rows, ctx), dtype=np.float32)
    lib().orc_fill_mask(_p(m), rows, ctx, start, steps, int(is_f16))
    return m


def rope_table(base: float, head_dim: int, max_ctx: int) -> Tuple[np.ndarray, np.ndarray]:
    c = np.empty((max_ctx, head_dim // 2), dtype=np.float32)
    s = np.empty_like(c)
    lib().orc_rope_table(base, head_dim, max_ctx, _p(c), _p(s))
    return c, s


def matmul_w4(packed: np.ndarray, scale: np.ndarray, x: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = packed.shape[0], packed.shape[1] * 2
    t = x.shape[0]
    y = np.empty((t, n), dtype=np.float32)
    lib().orc_matmul_w4(_p(packed), _p(scale), n, k, _p(x), t, _p(y))
    return y


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, qpos0: int, window: int) -> np.ndarray:
    """q [T, hq, hd]; k, v [S, hkv, hd]; fp32.  window <= 0: global."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    t, hq, hd = q.shape
    s, hkv, _ = k.shape
    out = np.empty_like(q)
    lib().orc_attention(_p(q), _p(k), _p(v), t, s, hq, hkv, hd, qpos0, window, _p(out))
    return out


# ---------------------------------------------------------------- model / executor

class OracleModel:
    def __init__(self, record: bytes) -> None:
        self._buf = np.frombuffer(record, dtype=np.uint8)       # keeps the bytes alive
        self.h = lib().orc_model_create(_p(self._buf), self._buf.size)
        if not self.h:
            raise ValueError("bad weights record")
        cfg = np.zeros(16, dtype=np.int32)
        lib().orc_model_cfg(self.h, _p(cfg))
        (self.n_layers, self.d_model, self.n_q_heads, self.n_kv_heads, self.head_dim, self.ffn, self.vocab,
         self.max_ctx, self.window, self.period, self.kv_dtype, self.n_buckets) = (int(v) for v in cfg[:12])

    def close(self) -> None:
        if self.h:
            lib().orc_model_destroy(self.h)
            self.h = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class OracleExecutor:
    """Same call surface and status codes as the reference executor."""

    def __init__(self, model: OracleModel) -> None:
        self.model = model
        self.h = lib().orc_exec_create(model.h)
        self._logits = np.empty(model.vocab, dtype=np.float32)

    def prefill(self, ids) -> int:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        return lib().orc_exec_prefill(self.h, _p(ids), ids.size)

    def decode_logits(self, token: Optional[int] = None) -> Tuple[int, Optional[np.ndarray]]:
        out = np.empty(self.model.vocab, dtype=np.float32)
        if token is None:
            rc = lib().orc_exec_decode_logits(self.h, None, _p(out))
        else:
            t = C.c_int32(token)
            rc = lib().orc_exec_decode_logits(self.h, C.byref(t), _p(out))
        return rc, (out if rc == 0 else None)

    def decode_token(self) -> Tuple[int, int]:
        t = C.c_int32(-1)
        rc = lib().orc_exec_decode_token(self.h, C.byref(t), _p(self._logits))
        return rc, t.value

    def reset(self) -> None:
        lib().orc_exec_reset(self.h)

    @property
    def current_step(self) -> int:
        return lib().orc_exec_current_step(self.h)

    @property
    def internal_step(self) -> int:
        return lib().orc_exec_internal_step(self.h)

    @property
    def pending_token(self) -> int:
        return lib().orc_exec_pending_token(self.h)

    def last_plan(self) -> List[Tuple[int, int]]:
        b = np.empty(64, dtype=np.int32)
        l = np.empty(64, dtype=np.int32)
        n = lib().orc_exec_last_plan(self.h, _p(b), _p(l))
        return [(int(b[i]), int(l[i])) for i in range(n)]

    def read_kv(self, layer: int, is_v: bool, kv_head: int, pos: int) -> np.ndarray:
        out = np.empty(self.model.head_dim, dtype=np.float32)
        lib().orc_exec_read_kv(self.h, layer, int(is_v), kv_head, pos, _p(out))
        return out

    def close(self) -> None:
        if self.h:
            lib().orc_exec_destroy(self.h)
            self.h = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
