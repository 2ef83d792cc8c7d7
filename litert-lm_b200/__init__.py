"""litert_lm_b200 — host-side binding of the B200 LlmExecutor backend.

The product is ``libb200lm.so`` (hand-written sm_100a CUDA behind the C ABI of
``include/b200lm.h``).  This module is the thin Python host layer over that ABI:
:class:`B200LlmExecutor` mirrors the reference's ``LlmExecutorBase`` call surface
(runtime/executor/llm_executor_base.h:33-121) — ``Prefill``, ``Decode``,
``DecodeLogits``, ``Reset``, ``GetVocabSize``, ``GetCurrentStep``,
``ExecutorBackendName`` — with the same argument meaning and status codes, and
:mod:`ops` exposes the operator-level entry points of ``include/b200lm_ops.h``.

There is no CPU fallback: a missing library raises, and on a machine without a
CUDA device every device entry point reports ``FAILED_PRECONDITION``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import model_io  # noqa: F401  (re-exported)
from . import sharding  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200lm.so")

# absl::StatusCode
OK, CANCELLED, INVALID_ARGUMENT, DEADLINE_EXCEEDED, NOT_FOUND = 0, 1, 3, 4, 5
FAILED_PRECONDITION, OUT_OF_RANGE, UNIMPLEMENTED, INTERNAL = 9, 11, 12, 13
_CODE_NAMES = {0: "OK", 1: "CANCELLED", 3: "INVALID_ARGUMENT", 4: "DEADLINE_EXCEEDED", 5: "NOT_FOUND",
               9: "FAILED_PRECONDITION", 11: "OUT_OF_RANGE", 12: "UNIMPLEMENTED", 13: "INTERNAL"}

DECODE_AUTO, DECODE_PHASE_KERNELS, DECODE_PERSISTENT, DECODE_PERSISTENT_BASIC, DECODE_CHAINED, DECODE_WIDE = 0, 1, 2, 3, 4, 5
GEMM_AUTO, GEMM_CHECK, GEMM_TCGEN05 = 0, 1, 2


class StatusError(RuntimeError):
    """A non-OK absl-style status returned by the library."""

    def __init__(self, code: int, message: str) -> None:
        super().__init__(f"{_CODE_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


class B200LmConfig(C.Structure):
    _fields_ = [("struct_size", C.c_int32), ("device", C.c_int32), ("max_num_tokens", C.c_int32),
                ("decode_mode", C.c_int32), ("prefill_gemm", C.c_int32), ("page_order", C.c_int32),
                ("stream", C.c_void_p), ("n_sessions", C.c_int32), ("reserved1", C.c_int32),
                ("tp_rank", C.c_int32), ("tp_world", C.c_int32), ("tp_unique_id", C.c_void_p)]


_lib: Optional[C.CDLL] = None

_EXEC_SYMBOLS = ["B200Lm_Create", "B200Lm_CreateShared", "B200Lm_Destroy", "B200Lm_Prefill", "B200Lm_DecodeLogits",
                 "B200Lm_DecodeToken", "B200Lm_DecodeTokens", "B200Lm_Reset", "B200Lm_GetVocabSize",
                 "B200Lm_GetCurrentStep", "B200Lm_GetMaxNumTokens", "B200Lm_GetDecodeMode", "B200Lm_TpUniqueId", "B200Lm_TpAllReduceProbe", "B200Lm_BackendName", "B200Lm_Synchronize",
                 "B200Lm_GetLastPrefillPlan", "B200Lm_ReadKvRow", "B200Lm_GetLaunchCount", "B200Lm_TraceDecodeStep",
                 "B200Lm_SelectSession", "B200Lm_GetNumSessions", "B200Lm_PrefillSession", "B200Lm_DecodeTokensBatch"]
_OPS_SYMBOLS = ["B200LmOps_RepackW4T", "B200LmOps_RepackW4G", "B200LmOps_UnpackW4", "B200LmOps_GemvW4",
                "B200LmOps_GemmW4", "B200LmOps_GemmGegluW4", "B200LmOps_Attention", "B200LmOps_AttentionPrefillTc",
                "B200LmOps_AttentionDecodeStatic", "B200LmOps_AttentionDecodeStaticStatus"]


def load_library() -> C.CDLL:
    """Loads libb200lm.so.  Raises if it has not been built (python litert-lm_b200/build.py)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python litert-lm_b200/build.py` "
                           "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64
    errp = C.POINTER(C.c_char_p)
    sig = {
        "B200Lm_Create": [C.POINTER(B200LmConfig), vp, u64, C.c_char_p, C.POINTER(vp), errp],
        "B200Lm_CreateShared": [vp, C.POINTER(B200LmConfig), C.POINTER(vp), errp],
        "B200Lm_Prefill": [vp, vp, i32, i32, vp, errp],
        "B200Lm_DecodeLogits": [vp, vp, vp, errp],
        "B200Lm_DecodeToken": [vp, vp, errp],
        "B200Lm_DecodeTokens": [vp, i32, vp, errp],
        "B200Lm_Reset": [vp, errp],
        "B200Lm_GetVocabSize": [vp, vp, errp],
        "B200Lm_GetCurrentStep": [vp, vp, errp],
        "B200Lm_GetMaxNumTokens": [vp, vp, errp],
        "B200Lm_GetDecodeMode": [vp, vp, errp],
        "B200Lm_TpUniqueId": [vp, errp],
        "B200Lm_TpAllReduceProbe": [vp, i64, i32, vp, errp],
        "B200Lm_Synchronize": [vp, errp],
        "B200Lm_GetLastPrefillPlan": [vp, vp, vp, i32, vp, errp],
        "B200Lm_ReadKvRow": [vp, i32, i32, i32, i32, vp, vp, vp, errp],
        "B200Lm_GetLaunchCount": [vp, vp, errp],
        "B200Lm_TraceDecodeStep": [vp, vp, vp, i64, vp, vp, vp, errp],
        "B200Lm_SelectSession": [vp, i32, errp],
        "B200Lm_GetNumSessions": [vp, vp, errp],
        "B200Lm_PrefillSession": [vp, i32, vp, i32, i32, vp, errp],
        "B200Lm_DecodeTokensBatch": [vp, i32, vp, errp],
        "B200LmOps_RepackW4T": [vp, i64, i64, vp, errp],
        "B200LmOps_RepackW4G": [vp, i64, i64, vp, errp],
        "B200LmOps_UnpackW4": [i32, vp, i64, i64, vp, errp],
        "B200LmOps_GemvW4": [i32, vp, vp, i64, i64, vp, i32, i32, i32, vp, errp],
        "B200LmOps_GemmW4": [i32, i32, vp, vp, i64, i64, vp, i32, i32, i32, vp, vp, errp],
        "B200LmOps_GemmGegluW4": [i32, i32, vp, vp, vp, vp, i64, i64, vp, i32, vp, errp],
        "B200LmOps_Attention": [i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, errp],
        "B200LmOps_AttentionPrefillTc": [i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, errp],
        "B200LmOps_AttentionDecodeStatic": [i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, errp],
        "B200LmOps_AttentionDecodeStaticStatus": [i32, vp, vp, errp],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int
    lib.B200Lm_Destroy.argtypes = [vp]
    lib.B200Lm_Destroy.restype = None
    lib.B200Lm_BackendName.argtypes = []
    lib.B200Lm_BackendName.restype = C.c_char_p
    _lib = lib
    return lib


def tp_unique_id() -> bytes:
    """128 bytes identifying a new tensor-parallel group (an ncclUniqueId): make it on one rank and hand
    the same bytes to every rank's executor."""
    buf = C.create_string_buffer(128)
    _call("B200Lm_TpUniqueId", C.cast(buf, C.c_void_p))
    return buf.raw


_libc = C.CDLL(None)
_libc.free.argtypes = [C.c_void_p]
_libc.free.restype = None


def _check(code: int, err: C.c_char_p) -> None:
    if code == OK:
        return
    msg = err.value.decode(errors="replace") if err.value else ""
    if err.value is not None:
        _libc.free(C.cast(err, C.c_void_p))
    raise StatusError(code, msg)


def _call(name: str, *args) -> None:
    lib = load_library()
    err = C.c_char_p()
    code = getattr(lib, name)(*args, C.byref(err))
    _check(code, err)


def _ptr(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


class B200LlmExecutor:
    """Counterpart of ``LlmLiteRtCompiledModelExecutor`` on one B200.

    ``model`` is a `.litertlm` image (bytes) or a path to one.  Batch is 1, as in the
    reference (llm_litert_compiled_model_executor.cc:95).
    """

    def __init__(self, model, device: int = 0, max_num_tokens: int = 0, decode_mode: int = DECODE_AUTO,
                 prefill_gemm: int = GEMM_AUTO, stream: int = 0, reversed_pages: bool = False,
                 n_sessions: int = 1, tp_rank: int = 0, tp_world: int = 1, tp_unique_id: Optional[bytes] = None,
                 _shared_from: "Optional[B200LlmExecutor]" = None) -> None:
        self._h = C.c_void_p()
        self._tp_id = C.create_string_buffer(bytes(tp_unique_id), 128) if tp_unique_id is not None else None
        cfg = B200LmConfig(C.sizeof(B200LmConfig), device, max_num_tokens, decode_mode, prefill_gemm,
                           1 if reversed_pages else 0, stream or None, n_sessions, 0, tp_rank, tp_world,
                           C.cast(self._tp_id, C.c_void_p) if self._tp_id is not None else None)
        if _shared_from is not None:
            _call("B200Lm_CreateShared", _shared_from._h, C.byref(cfg), C.byref(self._h))
        elif isinstance(model, (bytes, bytearray, memoryview)):
            buf = np.frombuffer(model, dtype=np.uint8)
            _call("B200Lm_Create", C.byref(cfg), _ptr(buf), buf.size, None, C.byref(self._h))
        else:
            _call("B200Lm_Create", C.byref(cfg), None, 0, os.fsencode(model), C.byref(self._h))
        v = C.c_int32()
        _call("B200Lm_GetVocabSize", self._h, C.byref(v))
        self._vocab = v.value

    # -- LlmExecutorBase surface -------------------------------------------------------
    def Prefill(self, ids: Sequence[int], wait_for_completion: bool = True, cancel: Optional[np.ndarray] = None) -> None:
        """ids: token ids [1, n].  The last id of every work group is held back."""
        a = np.ascontiguousarray(ids, dtype=np.int32).ravel()
        cp = _ptr(cancel) if cancel is not None else None
        _call("B200Lm_Prefill", self._h, _ptr(a) if a.size else None, a.size, int(wait_for_completion), cp)

    def DecodeLogits(self, token: Optional[int] = None, out: Optional[np.ndarray] = None) -> np.ndarray:
        """One step on `token` (or the pending id); returns float32 logits [1, 1, vocab]."""
        logits = out if out is not None else np.empty((1, 1, self._vocab), dtype=np.float32)
        if token is None:
            _call("B200Lm_DecodeLogits", self._h, None, _ptr(logits))
        else:
            t = C.c_int32(int(token))
            _call("B200Lm_DecodeLogits", self._h, C.byref(t), _ptr(logits))
        return logits

    def Decode(self) -> int:
        """One step on the pending id with greedy sampling on the device; returns the token."""
        t = C.c_int32(-1)
        _call("B200Lm_DecodeToken", self._h, C.byref(t))
        return t.value

    def DecodeTokens(self, n_steps: int) -> np.ndarray:
        out = np.empty(max(n_steps, 0), dtype=np.int32)
        _call("B200Lm_DecodeTokens", self._h, n_steps, _ptr(out))
        return out

    def Reset(self) -> None:
        _call("B200Lm_Reset", self._h)

    # -- several sessions in one executor (no reference counterpart) -----------------------
    def SelectSession(self, session: int) -> None:
        """Makes `session` the one the single-session calls act on."""
        _call("B200Lm_SelectSession", self._h, session)

    def GetNumSessions(self) -> int:
        v = C.c_int32()
        _call("B200Lm_GetNumSessions", self._h, C.byref(v))
        return v.value

    def PrefillSession(self, session: int, ids: Sequence[int], wait_for_completion: bool = True) -> None:
        a = np.ascontiguousarray(ids, dtype=np.int32).ravel()
        _call("B200Lm_PrefillSession", self._h, session, _ptr(a) if a.size else None, a.size, int(wait_for_completion),
              None)

    def DecodeTokensBatch(self, n_steps: int) -> np.ndarray:
        """All sessions take n_steps greedy steps in lockstep; returns ids [n_steps, n_sessions]."""
        out = np.empty((max(n_steps, 0), self.GetNumSessions()), dtype=np.int32)
        _call("B200Lm_DecodeTokensBatch", self._h, n_steps, _ptr(out))
        return out

    def GetVocabSize(self) -> int:
        return self._vocab

    def GetCurrentStep(self) -> int:
        v = C.c_int32()
        _call("B200Lm_GetCurrentStep", self._h, C.byref(v))
        return v.value

    def GetDecodeMode(self) -> int:
        v = C.c_int32(0)
        _call("B200Lm_GetDecodeMode", self._h, C.byref(v))
        return v.value

    def TpAllReduceProbe(self, count: int, iters: int = 50) -> float:
        """Mean device time in ms of one all-reduce of `count` floats over the tensor-parallel group."""
        ms = C.c_float(0)
        _call("B200Lm_TpAllReduceProbe", self._h, count, iters, C.byref(ms))
        return ms.value

    def GetMaxNumTokens(self) -> int:
        v = C.c_int32()
        _call("B200Lm_GetMaxNumTokens", self._h, C.byref(v))
        return v.value

    @staticmethod
    def ExecutorBackendName() -> str:
        return load_library().B200Lm_BackendName().decode()

    # -- extras -----------------------------------------------------------------------
    def CreateShared(self, **kw) -> "B200LlmExecutor":
        """Another session (own KV cache and counters) over the same device weights."""
        return B200LlmExecutor(None, _shared_from=self, **kw)

    def Synchronize(self) -> None:
        _call("B200Lm_Synchronize", self._h)

    def GetLastPrefillPlan(self) -> List[Tuple[int, int]]:
        b = np.zeros(64, dtype=np.int32)
        l = np.zeros(64, dtype=np.int32)
        n = C.c_int32()
        _call("B200Lm_GetLastPrefillPlan", self._h, _ptr(b), _ptr(l), 64, C.byref(n))
        return [(int(b[i]), int(l[i])) for i in range(min(n.value, 64))]

    def ReadKvRow(self, layer: int, is_v: bool, kv_head: int, pos: int) -> Tuple[np.ndarray, int, int]:
        row = np.empty(4096, dtype=np.float32)
        page, slot = C.c_int32(), C.c_int32()
        _call("B200Lm_ReadKvRow", self._h, layer, int(is_v), kv_head, pos, _ptr(row), C.byref(page), C.byref(slot))
        return row, page.value, slot.value

    def TraceDecodeStep(self):
        """One greedy decode step with the per-barrier device timeline.  Returns (token,
        stamps[n_barriers, n_cta, 2] in SM cycles, sm_clock_khz)."""
        cap = 1 << 20
        buf = np.zeros(cap, dtype=np.int64)
        tok, nb, nc, khz = C.c_int32(-1), C.c_int32(), C.c_int32(), C.c_int32()
        _call("B200Lm_TraceDecodeStep", self._h, C.byref(tok), _ptr(buf), cap, C.byref(nb), C.byref(nc), C.byref(khz))
        n2 = nb.value * nc.value * 2
        self.last_trace_points = buf[n2:n2 + nb.value * nc.value * 8].reshape(nb.value, nc.value, 8).copy()
        return tok.value, buf[:n2].reshape(nb.value, nc.value, 2).copy(), khz.value

    def GetLaunchCount(self) -> int:
        v = C.c_int64()
        _call("B200Lm_GetLaunchCount", self._h, C.byref(v))
        return v.value

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            load_library().B200Lm_Destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class ops:
    """Operator-level entry points (include/b200lm_ops.h)."""

    @staticmethod
    def repack_w4t(packed: np.ndarray) -> np.ndarray:
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        n, k = packed.shape[0], packed.shape[1] * 2
        out = np.zeros(((n + 15) // 16 * 16) * k // 2, dtype=np.uint8)
        _call("B200LmOps_RepackW4T", _ptr(packed), n, k, _ptr(out))
        return out

    @staticmethod
    def repack_w4g(packed: np.ndarray) -> np.ndarray:
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        n, k = packed.shape[0], packed.shape[1] * 2
        out = np.zeros(((n + 127) // 128 * 128) * k // 2, dtype=np.uint8)
        _call("B200LmOps_RepackW4G", _ptr(packed), n, k, _ptr(out))
        return out

    @staticmethod
    def unpack_w4(packed: np.ndarray, device: int = 0) -> np.ndarray:
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        n, k = packed.shape[0], packed.shape[1] * 2
        out = np.empty((n, k), dtype=np.int8)
        _call("B200LmOps_UnpackW4", device, _ptr(packed), n, k, _ptr(out))
        return out

    @staticmethod
    def gemv_w4(packed: np.ndarray, scale: np.ndarray, x: np.ndarray, nterms: int = 3, kslices: int = 1,
                device: int = 0) -> np.ndarray:
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        scale = np.ascontiguousarray(scale, dtype=np.float32)
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, packed.shape[1] * 2)
        n, k = packed.shape[0], packed.shape[1] * 2
        y = np.empty((x.shape[0], n), dtype=np.float32)
        _call("B200LmOps_GemvW4", device, _ptr(packed), _ptr(scale), n, k, _ptr(x), x.shape[0], nterms, kslices, _ptr(y))
        return y

    @staticmethod
    def gemm_w4(packed: np.ndarray, scale: np.ndarray, a: np.ndarray, mode: int = GEMM_TCGEN05, ksplit: int = 1,
                repeat: int = 1, device: int = 0) -> Tuple[np.ndarray, float]:
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        scale = np.ascontiguousarray(scale, dtype=np.float32)
        a = np.ascontiguousarray(a, dtype=np.float32)
        n, k = packed.shape[0], packed.shape[1] * 2
        out = np.empty((a.shape[0], n), dtype=np.float32)
        ms = C.c_float(0)
        _call("B200LmOps_GemmW4", device, mode, _ptr(packed), _ptr(scale), n, k, _ptr(a), a.shape[0], ksplit, repeat,
              _ptr(out), C.byref(ms))
        return out, ms.value

    @staticmethod
    def gemm_geglu_w4(gate: np.ndarray, gate_scale: np.ndarray, up: np.ndarray, up_scale: np.ndarray, a: np.ndarray,
                      mode: int = GEMM_TCGEN05, device: int = 0) -> np.ndarray:
        gate = np.ascontiguousarray(gate, dtype=np.uint8)
        up = np.ascontiguousarray(up, dtype=np.uint8)
        gs = np.ascontiguousarray(gate_scale, dtype=np.float32)
        us = np.ascontiguousarray(up_scale, dtype=np.float32)
        a = np.ascontiguousarray(a, dtype=np.float32)
        ffn, k = gate.shape[0], gate.shape[1] * 2
        out = np.empty((a.shape[0], ffn), dtype=np.float32)
        _call("B200LmOps_GemmGegluW4", device, mode, _ptr(gate), _ptr(gs), _ptr(up), _ptr(us), ffn, k, _ptr(a),
              a.shape[0], _ptr(out))
        return out

    @staticmethod
    def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, qpos0: int = 0, window: int = 0, kv_bf16: bool = False,
                  nsplit: int = 1, repeat: int = 1, device: int = 0, private_caches: bool = False,
                  streaming_kernel: bool = False) -> Tuple[np.ndarray, float]:
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        t, hq, hd = q.shape
        s, hkv, _ = k.shape
        out = np.empty_like(q)
        ms = C.c_float(0)
        _call("B200LmOps_Attention", device, _ptr(q), _ptr(k), _ptr(v), t, s, hq, hkv, hd, qpos0, window,
              int(kv_bf16) | (2 if private_caches else 0) | (4 if streaming_kernel else 0), nsplit, repeat, _ptr(out),
              C.byref(ms))
        return out, ms.value

    @staticmethod
    def attention_prefill_tc(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int = 0, repeat: int = 1,
                             device: int = 0) -> Tuple[np.ndarray, float]:
        """Causal self-attention of s tokens with the tensor-core prefill kernel (bf16 operands)."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        s, hq, hd = q.shape
        _, hkv, _ = k.shape
        out = np.empty_like(q)
        ms = C.c_float(0)
        _call("B200LmOps_AttentionPrefillTc", device, _ptr(q), _ptr(k), _ptr(v), s, hq, hkv, hd, window, repeat,
              _ptr(out), C.byref(ms))
        return out, ms.value

    @staticmethod
    def attention_decode_static(q_dev: int, k_pages_dev: int, v_pages_dev: int, page_table_dev: int, out_dev: int,
                                batch: int, s: int, hq: int, hkv: int, hd: int, window: int = 0, kv_bf16: bool = False,
                                nsplit: int = 8, stream: int = 0, device: int = 0) -> None:
        """Split-KV decode attention over caller-owned DEVICE buffers (raw addresses); allocates
        nothing: the split partials live in a fixed array inside the library (8 MiB per GPU).
        For callers that must not allocate device memory at call time."""
        _call("B200LmOps_AttentionDecodeStatic", device, C.c_void_p(q_dev), C.c_void_p(k_pages_dev),
              C.c_void_p(v_pages_dev), C.c_void_p(page_table_dev), batch, s, hq, hkv, hd, window, int(kv_bf16), nsplit,
              C.c_void_p(out_dev), C.c_void_p(stream) if stream else None)

    @staticmethod
    def attention_decode_static_status(stream: int = 0, device: int = 0) -> int:
        """Waits for `stream` and returns the device error word of the static-scratch attention
        (0 = clean); raises StatusError when the word is set.  Allocates nothing."""
        word = C.c_int32(-1)
        _call("B200LmOps_AttentionDecodeStaticStatus", device, C.c_void_p(stream) if stream else None, C.byref(word))
        return word.value
