"""Synthetic Gemma3-style int4 models and the `.litertlm` container.

Two things live here, both host-side tooling around the executor:

* the seeded random-init models the benchmark configurations name (shapes only;
  no checkpoint is read), quantised to int4 per output channel and serialised
  as one self-describing *weights record* (magic ``B2LMWT01``);
* a writer/reader for the `.litertlm` container the reference ships models in:
  ``LITERTLM`` magic, version triple, header-end offset at byte 24, a
  flatbuffer ``LiteRTLMMetaData`` header at byte 32 and 16 KiB-aligned sections
  (reference: schema/core/litertlm_export.cc:94-180,
  schema/core/litertlm_read.cc:38-109, schema/core/litertlm_header_schema.fbs).
  The flatbuffer is encoded and decoded by hand (no flatbuffers package).

The weights record travels as a ``GenericBinaryData`` section next to an
``LlmMetadataProto`` section, so the file opens with the reference's own
section logic while the B200 executor reads its section by index.
"""
from __future__ import annotations

import dataclasses
import struct
import zlib
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

BLOCK = 16 * 1024
WEIGHTS_MAGIC = b"B2LMWT01"
KV_PAGE = 256

# AnySectionDataType (litertlm_header_schema.fbs:70-78)
SECTION_NONE, SECTION_GENERIC, SECTION_DEPRECATED, SECTION_TFLITE, SECTION_SP_TOKENIZER, \
    SECTION_LLM_METADATA, SECTION_HF_TOKENIZER_ZLIB = range(7)
SECTION_NAMES = ["NONE", "GenericBinaryData", "Deprecated", "TFLiteModel", "SP_Tokenizer",
                 "LlmMetadataProto", "HF_Tokenizer_Zlib"]

# VData union members (litertlm_header_schema.fbs:37-49)
(VD_NONE, VD_UINT8, VD_INT8, VD_UINT16, VD_INT16, VD_UINT32, VD_INT32, VD_FLOAT32, VD_BOOL,
 VD_STRING, VD_UINT64, VD_INT64) = range(12)
_VD_STRUCT_FMT = {VD_UINT8: "<B", VD_INT8: "<b", VD_UINT16: "<H", VD_INT16: "<h", VD_UINT32: "<I",
                  VD_INT32: "<i", VD_FLOAT32: "<f", VD_BOOL: "<?", VD_UINT64: "<Q", VD_INT64: "<q"}


# --------------------------------------------------------------------------- configs

@dataclasses.dataclass
class ModelConfig:
    name: str
    n_layers: int
    d_model: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    max_ctx: int
    window: int
    global_period: int = 6          # layer i is global iff i % period == period - 1
    kv_dtype: int = 0               # 0 = fp32 cache, 1 = bf16 cache
    buckets: Tuple[int, ...] = (1024, 256, 64)   # prefill signatures, descending
    rope_local: float = 1.0e4
    rope_global: float = 1.0e6
    rms_eps: float = 1.0e-6
    seed: int = 0

    def is_global(self, layer: int) -> bool:
        return layer % self.global_period == self.global_period - 1

    @property
    def n_qkv_rows(self) -> int:
        return (self.n_q_heads + 2 * self.n_kv_heads) * self.head_dim

    def layer_params(self) -> int:
        d, hq, hkv, hd, f = self.d_model, self.n_q_heads, self.n_kv_heads, self.head_dim, self.ffn
        return d * hq * hd + 2 * d * hkv * hd + hq * hd * d + 3 * d * f

    def decode_bytes_per_token(self, kv_len_avg_fn=None, s_lo: int = 1024, s_hi: int = 1280) -> int:
        """Algorithmic HBM bytes one decode step must move (batch 1): int4 layer
        weights + tied int4 head + fp32 scales + norm gains + KV read + logits write."""
        L, d, hq, hkv, hd, f, V = (self.n_layers, self.d_model, self.n_q_heads, self.n_kv_heads,
                                   self.head_dim, self.ffn, self.vocab)
        e_kv = 4 if self.kv_dtype == 0 else 2
        n_glob = sum(1 for i in range(L) if self.is_global(i))
        weights = L * self.layer_params() // 2 + V * d // 2
        scales = 4 * (L * (hq * hd + 2 * hkv * hd + 2 * d + 2 * f) + V)
        norms = 4 * (L * (4 * d + 2 * hd) + d)
        kv = 0.0
        steps = range(s_lo, s_hi)
        for s in steps:
            kv += 2 * hkv * hd * e_kv * (n_glob * s + (L - n_glob) * min(s, self.window))
        kv /= len(steps)
        return int(weights + scales + norms + kv + 4 * V)

    def prefill_flops(self, t: int, start: int = 0) -> float:
        """Projection FLOPs (2*T*P) + masked attention FLOPs for t tokens from `start`."""
        L, hq, hd = self.n_layers, self.n_q_heads, self.head_dim
        n_glob = sum(1 for i in range(L) if self.is_global(i))
        proj = 2.0 * t * L * self.layer_params()
        g = sum(p + 1 for p in range(start, start + t))
        l = sum(min(p + 1, self.window) for p in range(start, start + t))
        return proj + 4.0 * hd * hq * (n_glob * g + (L - n_glob) * l)


def config_tiny(seed: int = 0) -> ModelConfig:
    """Stand-in for the reference's tiny test LM (its file is not distributed):
    2 layers (one local, one global), window 8, context 64."""
    return ModelConfig("tiny-lm", n_layers=2, d_model=64, n_q_heads=4, n_kv_heads=1, head_dim=32,
                       ffn=128, vocab=256, max_ctx=64, window=8, global_period=2,
                       buckets=(32, 8), seed=seed)


def config_small(seed: int = 7) -> ModelConfig:
    """Mid-size case with the 1B model's head geometry (4 query heads on 1 kv head,
    head_dim 256): every tile shape is exercised, the CPU oracle finishes in seconds."""
    return ModelConfig("small-lm", n_layers=6, d_model=384, n_q_heads=4, n_kv_heads=1, head_dim=256,
                       ffn=1024, vocab=4096, max_ctx=1024, window=64, global_period=3,
                       buckets=(256, 64, 16), seed=seed)


def config_small_gqa(seed: int = 8) -> ModelConfig:
    """Mid-size case with several kv heads (group of 2), head_dim 128 and a bf16 cache."""
    return ModelConfig("small-gqa-lm", n_layers=4, d_model=512, n_q_heads=8, n_kv_heads=4, head_dim=128,
                       ffn=1536, vocab=2048, max_ctx=512, window=48, global_period=2, kv_dtype=1,
                       buckets=(128, 32), seed=seed)


def config_gemma3_1b(seed: int = 1) -> ModelConfig:
    return ModelConfig("gemma3-1b-shape", n_layers=26, d_model=1152, n_q_heads=4, n_kv_heads=1,
                       head_dim=256, ffn=6912, vocab=262144, max_ctx=4096, window=512,
                       buckets=(1024, 256, 64), seed=seed)


def config_gemma3_4b(seed: int = 3) -> ModelConfig:
    return ModelConfig("gemma3-4b-shape", n_layers=34, d_model=2560, n_q_heads=8, n_kv_heads=4,
                       head_dim=256, ffn=10240, vocab=262144, max_ctx=8192, window=1024,
                       buckets=(1024, 256, 64), seed=seed)


def config_gemma3_27b(seed: int = 4) -> ModelConfig:
    return ModelConfig("gemma3-27b-shape", n_layers=62, d_model=5376, n_q_heads=32, n_kv_heads=16,
                       head_dim=128, ffn=21504, vocab=262144, max_ctx=4096, window=1024,
                       buckets=(2048, 512, 128), seed=seed)


def config_gemma3_4b_slice(seed: int = 3) -> ModelConfig:
    """The 4B shape's layer geometry (hidden 2560, 8 query / 4 kv heads of 256, ffn 10240, window 1024)
    on 6 layers (one global) and a 16 k vocabulary: every per-layer kernel shape of the full model, small
    enough for the CPU oracle and a quick build."""
    return ModelConfig("gemma3-4b-slice", n_layers=6, d_model=2560, n_q_heads=8, n_kv_heads=4,
                       head_dim=256, ffn=10240, vocab=16384, max_ctx=2048, window=1024,
                       buckets=(1024, 256, 64), seed=seed)


def config_gemma3_27b_slice(seed: int = 4) -> ModelConfig:
    """The 27B shape's layer geometry (hidden 5376, 32 query / 16 kv heads of 128, ffn 21504, window
    1024) on 2 layers (one local, one global) and a 16 k vocabulary, one GPU (no tensor parallelism)."""
    return ModelConfig("gemma3-27b-slice", n_layers=2, d_model=5376, n_q_heads=32, n_kv_heads=16,
                       head_dim=128, ffn=21504, vocab=16384, max_ctx=2048, window=1024, global_period=2,
                       buckets=(2048, 512, 128), seed=seed)


CONFIGS = {"tiny": config_tiny, "small": config_small, "small-gqa": config_small_gqa, "gemma3-1b": config_gemma3_1b,
           "gemma3-4b": config_gemma3_4b, "gemma3-27b": config_gemma3_27b,
           "gemma3-4b-slice": config_gemma3_4b_slice, "gemma3-27b-slice": config_gemma3_27b_slice}


# --------------------------------------------------------------------------- int4

def quantize_int4(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Symmetric per-output-row int4: scale = max|w|/7, q = rint(w/scale) in [-7, 7];
    element 2j in the low nibble of byte j (two's complement)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    amax = np.abs(w).max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(7.0), np.float32(1.0)).astype(np.float32)
    q = np.rint(w / scale[:, None]).astype(np.int32)
    np.clip(q, -7, 7, out=q)
    qu = (q & 0xF).astype(np.uint8)
    packed = (qu[:, 0::2] | (qu[:, 1::2] << 4)).astype(np.uint8)
    return packed, scale


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    lo = (packed & 0xF).astype(np.int8)
    hi = (packed >> 4).astype(np.int8)
    lo = np.where(lo >= 8, lo - 16, lo).astype(np.int8)
    hi = np.where(hi >= 8, hi - 16, hi).astype(np.int8)
    out = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.int8)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return out


# --------------------------------------------------------------------------- weights record

_ENTRY = struct.Struct("<48sIIIIQQ")   # name, dtype, rows, cols, pad, offset, nbytes  (80 bytes)


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


def pack_weights_record(cfg: ModelConfig, tensors: "Dict[str, np.ndarray]") -> bytes:
    """Serialise named tensors.  uint8 2-D arrays are packed int4 (cols = 2 * bytes per row)."""
    names = list(tensors)
    header = bytearray(256)
    header[0:8] = WEIGHTS_MAGIC
    index_bytes = _ENTRY.size * len(names)
    data_start = _align(256 + index_bytes, 256)
    struct.pack_into("<II", header, 8, data_start, len(names))
    icfg = [cfg.n_layers, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab,
            cfg.max_ctx, cfg.window, cfg.global_period, cfg.kv_dtype, len(cfg.buckets), cfg.seed, 0, 0, 0]
    struct.pack_into("<16i", header, 16, *icfg)
    struct.pack_into("<8f", header, 80, cfg.rope_local, cfg.rope_global, cfg.rms_eps, 0, 0, 0, 0, 0)
    bk = list(cfg.buckets) + [0] * (8 - len(cfg.buckets))
    struct.pack_into("<8i", header, 112, *bk)
    entries = bytearray()
    chunks: List[bytes] = []
    off = data_start
    for nm in names:
        a = tensors[nm]
        if a.dtype == np.uint8:
            dtype, rows, cols = 0, a.shape[0], a.shape[1] * 2
        else:
            a = np.ascontiguousarray(a, dtype=np.float32)
            dtype, rows, cols = 1, (a.shape[0] if a.ndim == 2 else 1), a.shape[-1]
        raw = np.ascontiguousarray(a).tobytes()
        entries += _ENTRY.pack(nm.encode(), dtype, rows, cols, 0, off, len(raw))
        pad = _align(len(raw), 256) - len(raw)
        chunks.append(raw + b"\0" * pad)
        off += len(raw) + pad
    head = bytes(header) + bytes(entries)
    head += b"\0" * (data_start - len(head))
    return head + b"".join(chunks)


def parse_weights_record(blob: bytes) -> Tuple[ModelConfig, "Dict[str, np.ndarray]"]:
    if blob[:8] != WEIGHTS_MAGIC:
        raise ValueError("not a weights record")
    _, n = struct.unpack_from("<II", blob, 8)
    ic = struct.unpack_from("<16i", blob, 16)
    fc = struct.unpack_from("<8f", blob, 80)
    bk = struct.unpack_from("<8i", blob, 112)
    cfg = ModelConfig("from-record", *ic[:9], global_period=ic[9], kv_dtype=ic[10],
                      buckets=tuple(bk[:ic[11]]), rope_local=fc[0], rope_global=fc[1], rms_eps=fc[2],
                      seed=ic[12])
    out: Dict[str, np.ndarray] = {}
    for i in range(n):
        nm, dtype, rows, cols, _, off, nbytes = _ENTRY.unpack_from(blob, 256 + i * _ENTRY.size)
        nm = nm.rstrip(b"\0").decode()
        if dtype == 0:
            out[nm] = np.frombuffer(blob, dtype=np.uint8, count=nbytes, offset=off).reshape(rows, cols // 2)
        else:
            a = np.frombuffer(blob, dtype=np.float32, count=nbytes // 4, offset=off)
            out[nm] = a.reshape(rows, cols) if rows > 1 else a
    return cfg, out


def generate_tensors(cfg: ModelConfig) -> "Dict[str, np.ndarray]":
    """Random-init weights: N(0, 0.02) before quantisation, gains 1 + N(0, 0.02).
    Draw order is fixed: embedding; per layer wqkv (q heads, k heads, v heads), wo, wgate,
    wup, wdown, then the six norm gains; final norm last."""
    rng = np.random.Generator(np.random.PCG64(cfg.seed))
    t: Dict[str, np.ndarray] = {}

    def mat(name: str, rows: int, cols: int) -> None:
        w = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
        t[name + ".q"], t[name + ".scale"] = quantize_int4(w)

    def gain(name: str, n: int) -> None:
        t[name] = (1.0 + 0.02 * rng.standard_normal(n, dtype=np.float32)).astype(np.float32)

    d, hd = cfg.d_model, cfg.head_dim
    mat("embed", cfg.vocab, d)
    for i in range(cfg.n_layers):
        p = f"L{i}."
        mat(p + "wqkv", cfg.n_qkv_rows, d)
        mat(p + "wo", d, cfg.n_q_heads * hd)
        mat(p + "wgate", cfg.ffn, d)
        mat(p + "wup", cfg.ffn, d)
        mat(p + "wdown", d, cfg.ffn)
        for nm, n in (("pre_attn", d), ("post_attn", d), ("pre_ffn", d), ("post_ffn", d),
                      ("q_norm", hd), ("k_norm", hd)):
            gain(p + nm, n)
    gain("final_norm", d)
    return t


def build_weights_record(cfg: ModelConfig) -> bytes:
    return pack_weights_record(cfg, generate_tensors(cfg))


def shard_for_tensor_parallel(cfg: ModelConfig, tensors: "Dict[str, np.ndarray]", rank: int, world: int):
    """The sub-model one tensor-parallel rank holds: query / kv heads and FFN columns are split over the
    ranks (W_q / W_k / W_v and gate / up by output rows, W_o and W_down by input columns), norms and the
    tied embedding are replicated.  Quantised values and their per-row scales are SLICED, never
    re-quantised, so the partial O and down outputs of the ranks add up exactly to the unsplit products;
    the executor sums them across the ranks (all-reduce) before the post-norms.  Returns (config, tensors)
    of a valid smaller model."""
    hq, hkv, hd, f, d = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.d_model
    if hq % world or hkv % world or f % world or (f // world) % 64 or ((hq // world) * hd) % 64:
        raise ValueError("heads / ffn columns do not divide over the ranks in 64-wide units")
    import dataclasses
    hq_r, hkv_r, f_r = hq // world, hkv // world, f // world
    sub = dataclasses.replace(cfg, name=f"{cfg.name}-tp{rank}of{world}", n_q_heads=hq_r, n_kv_heads=hkv_r, ffn=f_r)
    out: Dict[str, np.ndarray] = {}
    for nm, a in tensors.items():
        base = nm.split(".")[-2] if nm.endswith((".q", ".scale")) else nm.split(".")[-1]
        is_q, is_s = nm.endswith(".q"), nm.endswith(".scale")
        if base == "wqkv":
            rows = np.concatenate([np.arange(rank * hq_r * hd, (rank + 1) * hq_r * hd),
                                   hq * hd + np.arange(rank * hkv_r * hd, (rank + 1) * hkv_r * hd),
                                   (hq + hkv) * hd + np.arange(rank * hkv_r * hd, (rank + 1) * hkv_r * hd)])
            out[nm] = np.ascontiguousarray(a[rows])
        elif base in ("wgate", "wup"):
            out[nm] = np.ascontiguousarray(a[rank * f_r:(rank + 1) * f_r])
        elif base == "wo" and is_q:          # input columns = this rank's heads; two int4 per byte
            out[nm] = np.ascontiguousarray(a[:, rank * hq_r * hd // 2:(rank + 1) * hq_r * hd // 2])
        elif base == "wdown" and is_q:
            out[nm] = np.ascontiguousarray(a[:, rank * f_r // 2:(rank + 1) * f_r // 2])
        else:                                 # scales of W_o / W_down (per output row), norms, embedding
            out[nm] = a
        del is_s
    return sub, out


# --------------------------------------------------------------------------- flatbuffer (by hand)

class _FbWriter:
    """Forward-laid-out flatbuffer encoder: every object is appended after its parent and
    the parent's uoffset is patched, so all uoffsets point forward as the format requires."""

    def __init__(self) -> None:
        self.buf = bytearray(4)          # root uoffset placeholder

    def _pad(self, a: int) -> None:
        while len(self.buf) % a:
            self.buf.append(0)

    def _patch(self, at: int, target: int) -> None:
        struct.pack_into("<I", self.buf, at, target - at)

    def string(self, at: int, s: str) -> None:
        raw = s.encode()
        self._pad(4)
        self._patch(at, len(self.buf))
        self.buf += struct.pack("<I", len(raw)) + raw + b"\0"
        self._pad(4)

    def table(self, at: int, fields: "List[Tuple[str, object]]") -> None:
        """fields: list of (kind, payload) in field-id order.  kinds: 'absent', 'u8', 'u64',
        'string', 'table' (payload = field list), 'vector' (payload = list of field lists),
        'struct' (payload = raw bytes, alignment = len)."""
        sizes = {"u8": 1, "u64": 8}
        # Table body layout: soffset32, then fields in id order with natural alignment.
        body_off = 4
        offs = []
        for kind, payload in fields:
            if kind == "absent":
                offs.append(0)
                continue
            sz = sizes.get(kind, 4)
            body_off = _align(body_off, sz)
            offs.append(body_off)
            body_off += sz
        body_size = _align(body_off, 4)
        vt_size = 4 + 2 * len(fields)
        # vtable immediately precedes the table; align so the table's u64s land on 8.
        self._pad(2)
        while (len(self.buf) + vt_size) % 8:
            self.buf.append(0)
        vt_pos = len(self.buf)
        self.buf += struct.pack("<HH", vt_size, body_size) + b"".join(struct.pack("<H", o) for o in offs)
        tpos = len(self.buf)
        self._patch(at, tpos)
        self.buf += bytearray(body_size)
        struct.pack_into("<i", self.buf, tpos, tpos - vt_pos)
        deferred = []
        for (kind, payload), o in zip(fields, offs):
            if kind == "absent":
                continue
            if kind == "u8":
                self.buf[tpos + o] = int(payload) & 0xFF
            elif kind == "u64":
                struct.pack_into("<Q", self.buf, tpos + o, int(payload))
            else:
                deferred.append((kind, payload, tpos + o))
        for kind, payload, where in deferred:
            if kind == "string":
                self.string(where, payload)
            elif kind == "table":
                self.table(where, payload)
            elif kind == "struct":
                self._pad(max(4, len(payload)))
                self._patch(where, len(self.buf))
                self.buf += payload
                self._pad(4)
            elif kind == "vector":
                self._pad(4)
                self._patch(where, len(self.buf))
                self.buf += struct.pack("<I", len(payload))
                slots = len(self.buf)
                self.buf += bytearray(4 * len(payload))
                for i, sub in enumerate(payload):
                    self.table(slots + 4 * i, sub)
            else:
                raise ValueError(kind)


def _kv_fields(key: str, value) -> "List[Tuple[str, object]]":
    """KeyValuePair {key, value_type, value}.  Python ints map to Int32 unless they overflow
    (then Int64), floats to Float32, bools to Bool, str to StringValue; a (tag, value) tuple
    forces a VData member."""
    if isinstance(value, tuple):
        tag, v = value
    elif isinstance(value, bool):
        tag, v = VD_BOOL, value
    elif isinstance(value, int):
        tag, v = (VD_INT32, value) if -2 ** 31 <= value < 2 ** 31 else (VD_INT64, value)
    elif isinstance(value, float):
        tag, v = VD_FLOAT32, value
    else:
        tag, v = VD_STRING, str(value)
    if tag == VD_STRING:
        val = ("table", [("string", v)])
    else:
        val = ("struct", struct.pack(_VD_STRUCT_FMT[tag], v))
    return [("string", key), ("u8", tag), val]


def encode_header(system_kv: Sequence[Tuple[str, object]],
                  sections: Sequence[Tuple[int, int, int, Sequence[Tuple[str, object]]]]) -> bytes:
    """sections: (data_type, begin, end, items)."""
    w = _FbWriter()
    sys_tbl = [("vector", [_kv_fields(k, v) for k, v in system_kv])]
    objs = []
    for dtype, begin, end, items in sections:
        objs.append([("vector", [_kv_fields(k, v) for k, v in items]) if items else ("absent", None),
                     ("u64", begin), ("u64", end), ("u8", dtype)])
    sec_tbl = [("vector", objs)]
    w.table(0, [("table", sys_tbl), ("table", sec_tbl)])
    return bytes(w.buf)


class _FbReader:
    def __init__(self, buf: bytes) -> None:
        self.b = buf

    def u32(self, p: int) -> int:
        return struct.unpack_from("<I", self.b, p)[0]

    def indirect(self, p: int) -> int:
        return p + self.u32(p)

    def field(self, tpos: int, idx: int) -> int:
        vt = tpos - struct.unpack_from("<i", self.b, tpos)[0]
        vt_size = struct.unpack_from("<H", self.b, vt)[0]
        slot = 4 + 2 * idx
        if slot >= vt_size:
            return 0
        o = struct.unpack_from("<H", self.b, vt + slot)[0]
        return tpos + o if o else 0

    def string(self, p: int) -> str:
        s = self.indirect(p)
        n = self.u32(s)
        return self.b[s + 4:s + 4 + n].decode()

    def vector(self, p: int) -> Tuple[int, int]:
        v = self.indirect(p)
        return self.u32(v), v + 4

    def kv(self, tpos: int) -> Tuple[str, object, int]:
        key = self.string(self.field(tpos, 0))
        tf = self.field(tpos, 1)
        tag = self.b[tf] if tf else VD_NONE
        vf = self.field(tpos, 2)
        if tag == VD_STRING:
            st = self.indirect(vf)
            val = self.string(self.field(st, 0))
        elif tag in _VD_STRUCT_FMT:
            val = struct.unpack_from(_VD_STRUCT_FMT[tag], self.b, self.indirect(vf))[0]
        else:
            val = None
        return key, val, tag

    def kv_vector(self, fieldpos: int) -> "List[Tuple[str, object, int]]":
        if not fieldpos:
            return []
        n, base = self.vector(fieldpos)
        return [self.kv(self.indirect(base + 4 * i)) for i in range(n)]


@dataclasses.dataclass
class Section:
    data_type: int
    begin: int
    end: int
    items: "List[Tuple[str, object, int]]"


@dataclasses.dataclass
class LitertLmFile:
    version: Tuple[int, int, int]
    header_end: int
    system: "List[Tuple[str, object, int]]"
    sections: "List[Section]"


def decode_header(fb: bytes) -> Tuple["List[Tuple[str, object, int]]", "List[Section]"]:
    r = _FbReader(fb)
    root = r.indirect(0)
    system, sections = [], []
    f = r.field(root, 0)
    if f:
        st = r.indirect(f)
        system = r.kv_vector(r.field(st, 0))
    f = r.field(root, 1)
    if f:
        sm = r.indirect(f)
        n, base = r.vector(r.field(sm, 0))
        for i in range(n):
            so = r.indirect(base + 4 * i)
            bf, ef, tf = r.field(so, 1), r.field(so, 2), r.field(so, 3)
            sections.append(Section(
                data_type=r.b[tf] if tf else 0,
                begin=struct.unpack_from("<Q", r.b, bf)[0] if bf else 0,
                end=struct.unpack_from("<Q", r.b, ef)[0] if ef else 0,
                items=r.kv_vector(r.field(so, 0))))
    return system, sections


def read_litertlm(data: bytes) -> LitertLmFile:
    """Header parse with the reference reader's checks (litertlm_read.cc:38-109):
    magic, major version must be 1, header end >= 32."""
    if len(data) < 32 or data[:8] != b"LITERTLM":
        raise ValueError("Invalid magic number or failed to read")
    major, minor, patch = struct.unpack_from("<III", data, 8)
    if major != 1:
        raise NotImplementedError(f"This reader doesn't support version {major}, expected version 1.")
    header_end = struct.unpack_from("<Q", data, 24)[0]
    if header_end < 32:
        raise ValueError("Invalid header end offset: smaller than current position.")
    if header_end > len(data):
        raise ValueError("Failed to read header data.")
    system, sections = decode_header(data[32:header_end])
    return LitertLmFile((major, minor, patch), header_end, system, sections)


def write_litertlm(sections: Sequence[Tuple[int, bytes, Sequence[Tuple[str, object]]]],
                   system_kv: Sequence[Tuple[str, object]] = ()) -> bytes:
    """Writer constants 1.1.0; sections start on 16 KiB boundaries; the header must end
    inside the first block (litertlm_export.cc:126-173)."""
    if not sections:
        raise ValueError("Input sections list is empty.")
    body = bytearray()
    offs = []
    pos = BLOCK
    for _, payload, _ in sections:
        begin = pos
        end = begin + len(payload)
        offs.append((begin, end))
        body += payload
        pad = _align(end, BLOCK) - end
        if pad == 0:
            pad = 0
        body += b"\0" * pad
        pos = end + pad
    fb = encode_header(system_kv, [(t, b, e, items) for (t, _, items), (b, e) in zip(sections, offs)])
    header_end = 32 + len(fb)
    if header_end > BLOCK:
        raise ValueError("Header size exceeds 16KB limit.")
    head = bytearray(BLOCK)
    head[0:8] = b"LITERTLM"
    struct.pack_into("<III", head, 8, 1, 1, 0)
    struct.pack_into("<Q", head, 24, header_end)
    head[32:header_end] = fb
    return bytes(head) + bytes(body)


def hf_tokenizer_section(json_bytes: bytes) -> bytes:
    """HF_Tokenizer_Zlib payload: u64 uncompressed size + one zlib stream
    (schema/core/litertlm_section.h:239-337)."""
    return struct.pack("<Q", len(json_bytes)) + zlib.compress(json_bytes)


def read_hf_tokenizer_section(payload: bytes) -> bytes:
    n = struct.unpack_from("<Q", payload, 0)[0]
    out = zlib.decompress(payload[8:])
    if len(out) != n:
        raise ValueError("uncompressed size mismatch")
    return out


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def llm_metadata_proto(max_num_tokens: int, start_token_id: int = 2, stop_token_ids: Sequence[int] = (1,),
                       start_token_str: Optional[str] = None, stop_token_strs: Sequence[str] = ()) -> bytes:
    """Minimal `LlmMetadata` protobuf (runtime/proto/llm_metadata.proto:67-84): start token,
    stop tokens (each a TokenUnion with token_ids) and max_num_tokens, wire-encoded by hand."""
    def token_union(ids: Sequence[int]) -> bytes:
        packed = b"".join(_varint(i) for i in ids)
        tok_ids = b"\x0a" + _varint(len(packed)) + packed          # TokenIds.ids (field 1, packed)
        return b"\x0a" + _varint(len(tok_ids)) + tok_ids           # TokenUnion.token_ids (field 1)
    def token_str(s: str) -> bytes:
        raw = s.encode()
        return b"\x12" + _varint(len(raw)) + raw                   # TokenUnion.token_str (field 2)
    out = b""
    st = token_str(start_token_str) if start_token_str is not None else token_union([start_token_id])
    out += b"\x0a" + _varint(len(st)) + st                         # start_token = 1
    stops = [token_str(s) for s in stop_token_strs] or [token_union([s]) for s in stop_token_ids]
    for tu in stops:
        out += b"\x12" + _varint(len(tu)) + tu                     # stop_tokens = 2
    if max_num_tokens <= 0:
        return out
    out += b"\x28" + _varint(max_num_tokens)                       # max_num_tokens = 5
    return out


def export_model_litertlm(cfg: ModelConfig, record: Optional[bytes] = None) -> bytes:
    """A `.litertlm` file holding the metadata proto and the weights record."""
    record = record if record is not None else build_weights_record(cfg)
    items = [("model_type", "b200_int4_decoder"), ("n_layers", cfg.n_layers), ("d_model", cfg.d_model),
             ("n_q_heads", cfg.n_q_heads), ("n_kv_heads", cfg.n_kv_heads), ("head_dim", cfg.head_dim),
             ("ffn", cfg.ffn), ("vocab", cfg.vocab), ("max_ctx", cfg.max_ctx), ("window", cfg.window)]
    return write_litertlm(
        [(SECTION_LLM_METADATA, llm_metadata_proto(cfg.max_ctx), []),
         (SECTION_GENERIC, record, items)],
        system_kv=[("generator", "litert_lm_b200.model_io"), ("seed", cfg.seed)])


def find_weights_record(data: bytes) -> bytes:
    f = read_litertlm(data)
    for s in f.sections:
        if s.data_type == SECTION_GENERIC and data[s.begin:s.begin + 8] == WEIGHTS_MAGIC:
            return data[s.begin:s.end]
    raise ValueError("no weights record section")
