"""Attention-only micro-benchmark: one JSON line per shape.

Inputs are seeded synthetic N(0,1) tensors (seed 2), head_dim 256, GQA 4:1, page size 256.

  prefill  causal self-attention over S tokens (S = 512 .. 8192), global and window 512,
           on the tcgen05 flash kernel; reported against the measured bf16 tensor peak.
           FLOPs counted: 4 * head_dim per (query, visible key) pair per query head.
  decode   a batch of 1 .. 64 independent sequences, each with its own bf16 KV cache of S keys
           (1k .. 32k) and one query at position S - 1; split-KV kernel + log-sum-exp combine;
           reported against the measured HBM copy bandwidth.  Bytes counted: the K and V rows
           of every sequence once (batch * 2 * S * hkv * head_dim * 2).

    python litert-lm_b200/attention_bench.py [--quick] [--repeat N]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402

HQ, HKV, HD, WINDOW = 4, 1, 256, 512


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def visible_pairs(s: int, window: int) -> int:
    """Number of (query, key) pairs a causal (optionally windowed) mask leaves open."""
    if window <= 0 or window >= s:
        return s * (s + 1) // 2
    return window * (window + 1) // 2 + (s - window) * window


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="two prefill and two decode shapes only")
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--streaming-kernel", action="store_true", help="decode: the streaming kernel of the wide decode step instead of the register-resident split kernel")
    args = ap.parse_args()
    graft.build()
    pkg = graft.load_package()
    hbm, tensor, src = peaks()
    rng = np.random.Generator(np.random.PCG64(2))
    seqs = (512, 2048) if args.quick else (512, 1024, 2048, 4096, 8192)
    for s in seqs:
        q = rng.standard_normal((s, HQ, HD), dtype=np.float32)
        k = rng.standard_normal((s, HKV, HD), dtype=np.float32)
        v = rng.standard_normal((s, HKV, HD), dtype=np.float32)
        for window in (0, WINDOW):
            _, ms = pkg.ops.attention_prefill_tc(q, k, v, window=window, repeat=args.repeat)
            flops = 4.0 * HD * HQ * visible_pairs(s, window)
            tf = flops / (ms * 1e-3) / 1e12
            print(json.dumps({"op": "prefill_attention", "kernel": "flash_prefill_tc_kernel<256>", "seq": s,
                              "mask": "causal" if window == 0 else f"causal+window{window}", "hq": HQ, "hkv": HKV,
                              "head_dim": HD, "dtype": "bf16 operands, fp32 accumulate", "ms": ms, "flops": flops,
                              "roofline": {"bound": "tensor", "achieved": tf, "peak": tensor, "unit": "TFLOP/s",
                                           "frac": tf / tensor, "of": src}}), flush=True)
    shapes = ((1024, 1), (32768, 64)) if args.quick else tuple((s, b) for s in (1024, 2048, 4096, 8192, 16384, 32768)
                                                              for b in (1, 4, 16, 64))
    for s, batch in shapes:
        k = rng.standard_normal((s, HKV, HD), dtype=np.float32)
        v = rng.standard_normal((s, HKV, HD), dtype=np.float32)
        q = rng.standard_normal((batch, HQ, HD), dtype=np.float32)
        nsplit = max(2, min(64, s // 256))
        if args.streaming_kernel:       # one CTA per SM there: about two (sequence, kv head, split) items per SM
            nsplit = max(2, min(nsplit, -(-2 * 148 // (batch * HKV))))
        _, ms = pkg.ops.attention(q, k, v, nsplit=nsplit, repeat=args.repeat, kv_bf16=True, private_caches=True,
                                  streaming_kernel=args.streaming_kernel)
        nbytes = 2.0 * s * HKV * HD * 2 * batch
        gbs = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"op": "decode_attention", "kernel": ("wide_attn_kernel + wide_attn_combine_kernel" if args.streaming_kernel else
                                                            "attn_decode_kernel + attn_combine_kernel"), "kv_len": s,
                          "batch": batch, "nsplit": nsplit, "page": 256, "kv_dtype": "bf16", "ms": ms, "bytes": nbytes,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s",
                                       "frac": gbs / hbm, "of": src,
                                       "note": "caches up to 126 MB in total can be served from L2 on repeated runs"}}),
              flush=True)


if __name__ == "__main__":
    main()
