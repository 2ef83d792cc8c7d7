"""Benchmark of the B200 executor on the reference's headline protocol: a 1024-token
prefill followed by 256 greedy decode steps, batch 1, on the Gemma3-1B-shaped int4 model
(random-init weights, seeded synthetic prompt).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one prefill + 256 decode steps of one session per GPU (sessions are independent:
with N > 1 every rank runs its own, no collective on the data path; "weak" scaling).
Prints ONE JSON line on rank 0.  `value` is decode tok/s with the arg-max fed back on the
device; `prefill` carries the prefill tok/s; `e2e` is the same protocol through the
reference-facing calls with host buffers (ids host->device, 1 MiB of logits device->host
per step, host arg-max as the reference's CPU sampler does).

`--impl reference` times the CPU implementation of the same path on the host cores.  The
reference's own CPU backend (LiteRT + XNNPACK) cannot be built in this environment, so this
arm runs the CPU oracle port (oracle/), on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402

PREFILL_TOKENS = 1024
DECODE_STEPS = 256
# DRAM bytes per decode step: an ncu capture (2026-11-25) of one launch of two decode steps of the chained
# kernel read 1079.5 MB and wrote 48.3 MB
DECODE_DRAM_BYTES_PER_STEP = 563.9e6
# The CPU arm's sample of the workload, used by `--impl reference` and by the in-line `cpu_baseline` alike:
# the full 1024-token prefill once, then short runs of greedy decode steps that stay inside the protocol's
# context range (1024 .. 1280 positions).
CPU_DECODE_TOKENS_PER_STEP = 8
METRIC = "decode tok/s (256 greedy steps after a 1024-token prefill), Gemma3-1B-shaped int4, batch 1 per GPU"


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_model(name: str, quiet: bool = True, kv_dtype: str = ""):
    """Seeded synthetic model, cached on local disk so both bench arms reuse it.  kv_dtype "fp32" / "bf16"
    overrides the configuration's KV-cache type (the weights are the same)."""
    pkg = graft.load_package()
    mio = pkg.model_io
    cfg = mio.CONFIGS[name]()
    if kv_dtype:
        cfg.kv_dtype = {"fp32": 0, "bf16": 1}[kv_dtype]
    cache_dir = os.environ.get("B200LM_CACHE", os.path.join(os.sep, "tmp", "b200lm_cache"))
    path = os.path.join(cache_dir, f"{name}-seed{cfg.seed}-kv{cfg.kv_dtype}.litertlm")
    if os.path.exists(path):
        with open(path, "rb") as f:
            img = f.read()
        try:
            rec = mio.find_weights_record(img)
            return cfg, rec, img
        except Exception:
            pass
    rec = mio.build_weights_record(cfg)
    img = mio.export_model_litertlm(cfg, rec)
    try:
        os.makedirs(cache_dir, exist_ok=True)
        tmp = path + f".{os.getpid()}.tmp"
        with open(tmp, "wb") as f:
            f.write(img)
        os.replace(tmp, path)
    except OSError:
        pass
    return cfg, rec, img


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons while the timed region runs (read-only NVML)."""

    def __init__(self, index: int) -> None:
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self) -> None:
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._halt.wait(0.1)

    def finish(self):
        self._halt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


class CpuArm:
    """The CPU oracle on the benchmark workload: `prefill()` runs the whole 1024-id prompt (timed once),
    `decode_step(n)` times n greedy steps that continue from there (context 1024 + steps so far)."""

    def __init__(self, rec, cfg) -> None:
        from oracle import oracle as orc
        self.model = orc.OracleModel(rec)
        self.ex = orc.OracleExecutor(self.model)
        self.ids = np.random.Generator(np.random.PCG64(cfg.seed)).integers(0, cfg.vocab, PREFILL_TOKENS).astype(np.int32)
        self.done = 0

    def prefill(self) -> float:
        t0 = time.perf_counter()
        assert self.ex.prefill(self.ids) == 0
        self.done = 0
        return PREFILL_TOKENS / (time.perf_counter() - t0)

    def decode_step(self, n: int) -> float:
        if self.done + n > DECODE_STEPS:          # stay inside the protocol's context range
            self.ex.reset()
            self.prefill()
        t0 = time.perf_counter()
        for _ in range(n):
            rc, _tok = self.ex.decode_token()
            assert rc == 0
        self.done += n
        return n / (time.perf_counter() - t0)


def xnnpack_baseline(rec, cfg, thread_counts) -> dict:
    """The same CPU sample with the matrix products on XNNPACK's dynamically-quantised int8 fully-connected
    operator (the XNNPACK build inside torch; not LiteRT).  A timing baseline beside the oracle port, never a
    parity reference: activations are quantised to int8 per row."""
    from oracle import oracle as orc
    out = {"library": "XNNPACK as bundled in torch (qd8-f32-qc8w fully-connected; int4 values held as int8)", "runs": []}
    try:
        for th in thread_counts:
            if not orc.use_xnnpack(th):
                out["unavailable"] = "XNNPACK symbols could not be bound from libtorch_cpu.so"
                break
            arm = CpuArm(rec, cfg)
            assert arm.ex.prefill(arm.ids[:8]) == 0    # first use creates and packs the operators
            arm.ex.reset()
            p = arm.prefill()
            arm.decode_step(2)
            d = float(np.mean([arm.decode_step(CPU_DECODE_TOKENS_PER_STEP) for _ in range(3)]))
            out["runs"].append({"threads": th, "decode_tok_s": d, "prefill_tok_s": p})
            del arm
    finally:
        orc.use_plain_matmul(host_threads())
    return out


def xnnpack_leg(model: str, thread_counts) -> dict:
    """Runs xnnpack_baseline in a child process: OpenMP's and pthreadpool's workers must not both spin on the
    same cores, and the wait policy can only be chosen before the OpenMP runtime loads."""
    import subprocess
    env = dict(os.environ, OMP_WAIT_POLICY="passive")
    t0 = time.perf_counter()
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "xnnpack", "--model", model, "--threads",
                            ",".join(str(t) for t in thread_counts)], env=env, capture_output=True, text=True, timeout=600)
        out = json.loads(r.stdout.strip().splitlines()[-1])
    except Exception as e:  # a timing extra: its absence must not fail the arm
        out = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    out["wall_s"] = time.perf_counter() - t0
    return out


def cpu_sample_text(n: int) -> str:
    return (f"CPU oracle port (plain C, OpenMP, all host threads), same weights and seeded prompt: the {PREFILL_TOKENS}-id "
            f"prefill once, then {n} greedy decode steps per bench step at context {PREFILL_TOKENS}+")


def host_threads() -> int:
    env = os.environ.get("OMP_NUM_THREADS")
    if env and env.isdigit():
        return int(env)
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def use_all_host_threads() -> None:
    """torchrun exports OMP_NUM_THREADS=1 to its children; the CPU arm wants every core it may
    run on.  Must be called before the oracle library (OpenMP) is loaded."""
    if "TORCHELASTIC_RUN_ID" in os.environ or "B200LM_CPU_THREADS" in os.environ:
        try:
            n = len(os.sched_getaffinity(0))
        except Exception:
            n = os.cpu_count() or 1
        os.environ["OMP_NUM_THREADS"] = os.environ.get("B200LM_CPU_THREADS", str(n))


def workload_config(cfg, world: int, decode_mode: int) -> dict:
    return {"workload": f"{cfg.name}: {PREFILL_TOKENS}-token prefill + {DECODE_STEPS} greedy decode steps, batch 1 per GPU",
            "seed": cfg.seed, "kv_cache": "fp32" if cfg.kv_dtype == 0 else "bf16", "context": cfg.max_ctx,
            "sessions": world, "parallelism": f"independent sessions x{world}, no collective",
            "l2": "every decode step streams 537 MB of weights and KV (> 126 MB L2); no flush needed",
            "decode_mode": "persistent kernel" if decode_mode in (0, 2, 4) else "one kernel per phase (CUDA graph)"}


def run_reference(args, rank: int) -> None:
    if rank != 0:
        return
    use_all_host_threads()
    cfg, rec, _ = load_model(args.model)
    n = max(1, min(CPU_DECODE_TOKENS_PER_STEP, DECODE_STEPS // max(1, args.warmup + args.steps)))
    arm = CpuArm(rec, cfg)
    t_all = time.perf_counter()
    prefill_tok_s = arm.prefill()
    vals = []
    for i in range(args.warmup + args.steps):
        v = arm.decode_step(n)
        if i >= args.warmup:
            vals.append(v)
    wall = time.perf_counter() - t_all
    value = float(np.mean(vals))
    cores = host_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * n / value, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights x fp32 activations (CPU)", "data": "synthetic",
        "config": workload_config(cfg, 1, 0),
        "prefill": {"value": prefill_tok_s, "unit": "tok/s"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": cpu_sample_text(n),
                         "prefill_tok_s": prefill_tok_s},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": wall,
        "note": "the reference's LiteRT/XNNPACK CPU backend cannot be built here; this is the CPU restatement",
    }
    if not args.no_xnnpack:
        line["xnnpack"] = xnnpack_leg(args.model, sorted({cores, min(4, cores)}, reverse=True))
        runs = line["xnnpack"].get("runs") or []
        best = max(runs, key=lambda r: r["decode_tok_s"]) if runs else None
        if best and best["decode_tok_s"] > value:
            # the stronger of the two CPU stand-ins is the arm's value, so that the GPU / CPU ratio is not flattered
            line["port"] = {"value": value, "prefill_tok_s": prefill_tok_s, "cores": cores}
            value = best["decode_tok_s"]
            line["value"] = value
            line["ms_per_step"] = 1000.0 * n / value
            line["prefill"] = {"value": best["prefill_tok_s"], "unit": "tok/s"}
            line["e2e"]["value"] = value
            line["cpu_baseline"].update({"value": value, "cores": best["threads"], "prefill_tok_s": best["prefill_tok_s"],
                                         "sample": cpu_sample_text(n) + "; matrix products on XNNPACK (torch-bundled build, "
                                                   "int8 activations x int8-held int4 weights), the rest the oracle's C"})
            line["dtype"] = "int4 values as int8 weights x dynamically quantised int8 activations (XNNPACK), fp32 elsewhere (CPU)"
    print(json.dumps(line), flush=True)


def run_cfg4(args, pkg, cfg, img, stream, rank: int, world: int, local_rank: int) -> None:
    """BASELINE config 4: `--sessions` concurrent sessions (1024-id prompt + 256 greedy steps each) of the
    4B-shaped model, sharded over the ranks with no collective on the data path.  On a GPU the sessions run
    in lockstep groups (one pass over the weights per decode step for a whole group) over ONE weight copy;
    the group size is the largest the decode kernels hold for this model."""
    import torch
    import torch.distributed as dist
    mine = pkg.sharding.shard_sessions(args.sessions, world, rank)
    cap = PREFILL_TOKENS + DECODE_STEPS + 256
    # the largest lockstep group first: all of this GPU's sessions in one wide group (tensor-core GEMM decode),
    # then what the persistent GEMV kernels carry
    owner, group = None, 0
    for group in ([args.group] if args.group > 0 else []) + [min(len(mine), 128), 4, 2, 1]:
        try:
            owner = pkg.B200LlmExecutor(img, device=local_rank, stream=stream.cuda_stream, n_sessions=group, max_num_tokens=cap)
            break
        except pkg.StatusError:
            if group == 1:
                raise
    decode_mode = owner.GetDecodeMode()
    groups = [mine[i:i + group] for i in range(0, len(mine), group)]
    execs = [owner]
    for g in groups[1:]:
        execs.append(owner.CreateShared(n_sessions=group, max_num_tokens=cap, stream=stream.cuda_stream))
    prompts = {sid: np.random.Generator(np.random.PCG64(pkg.sharding.session_seed(cfg.seed, sid))).integers(
        0, cfg.vocab, PREFILL_TOKENS).astype(np.int32) for sid in mine}

    def step():
        pf, dec = 0.0, 0.0
        for ex, g in zip(execs, groups):
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            for i in range(group):
                ex.SelectSession(i)
                ex.Reset()
            e0.record(stream)
            for i in range(group):        # a short last group repeats its last session: the lockstep step is the same work
                ex.PrefillSession(i, prompts[g[min(i, len(g) - 1)]], wait_for_completion=False)
            e1.record(stream)
            if group > 1:
                ex.DecodeTokensBatch(DECODE_STEPS)
            else:
                ex.DecodeTokens(DECODE_STEPS)
            e2.record(stream)
            e2.synchronize()
            pf += e0.elapsed_time(e1)
            dec += e1.elapsed_time(e2)
        return pf, dec

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(1, min(args.warmup, 1))):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    launches0 = sum(ex.GetLaunchCount() for ex in execs)
    res = [step() for _ in range(max(1, min(args.steps, 3)))]
    barrier()
    launches = sum(ex.GetLaunchCount() for ex in execs) - launches0       # this rank's kernels in the timed region
    clocks = sampler.finish()
    n = len(res)
    tok, (pf_ms, dec_ms) = pkg.sharding.reduce_throughput(n * len(mine) * DECODE_STEPS, [sum(r[0] for r in res), sum(r[1] for r in res)])
    if rank != 0:
        return
    peaks = measured_peaks()
    # per decode step of a group: the weights once, the KV of every session of the group
    full = cfg.decode_bytes_per_token(s_lo=PREFILL_TOKENS, s_hi=PREFILL_TOKENS + DECODE_STEPS)
    kv_only = full - cfg.decode_bytes_per_token(s_lo=0, s_hi=1)
    per_step = full + (group - 1) * (kv_only + 4 * cfg.vocab)
    steps_per_gpu = n * len(groups) * DECODE_STEPS
    achieved = per_step * steps_per_gpu / (dec_ms / 1e3) / 1e9
    line = {
        "metric": "aggregate decode tok/s, 64 concurrent sessions (1024-token prompt + 256 greedy steps each), Gemma3-4B-shaped int4",
        "value": tok / (dec_ms / 1e3), "unit": "tok/s", "n_gpus": world, "steps": n, "warmup": 1,
        "ms_per_step": (pf_ms + dec_ms) / n, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": ("int4 weights; bf16 activations on the tensor-core GEMM (prefill and wide decode), fp32 accumulate"
                  if decode_mode == pkg.DECODE_WIDE else
                  "int4 weights; int8 activation terms (decode), bf16 MMA (prefill), fp32 accumulate"), "data": "synthetic",
        "config": {"workload": f"{cfg.name}: {args.sessions} sessions x ({PREFILL_TOKENS}-token prefill + {DECODE_STEPS} decode steps), "
                               f"sharded over {world} GPU(s), no collective", "seed": cfg.seed, "sessions_per_gpu": len(mine),
                   "lockstep_group": group, "decode_mode": {pkg.DECODE_WIDE: "wide (tensor-core GEMM per step, CUDA graph)",
                                                            pkg.DECODE_CHAINED: "chained persistent kernel"}.get(decode_mode, str(decode_mode)),
                   "kv_cache": "fp32" if cfg.kv_dtype == 0 else "bf16", "context": cfg.max_ctx,
                   "kv_capacity_per_session": cap},
        "prefill": {"value": world * n * len(mine) * PREFILL_TOKENS / (pf_ms / 1e3), "unit": "tok/s"},
        "decode_ms_per_group_step": dec_ms / steps_per_gpu,
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": None, "of": peaks["source"], "algorithmic_bytes_per_group_step": per_step,
                     "note": "weights once + KV of every session of the lockstep group, per GPU"},
    }
    print(json.dumps(line), flush=True)


def run_cfg5(args, pkg, rank: int, world: int, local_rank: int) -> None:
    """BASELINE config 5's partitioning on `world` GPUs: query / kv heads and FFN columns split over the ranks,
    an NCCL all-reduce after the O and the down projection.  The model is a slice of a few layers of the
    27B shape (the full 62 layers take too long to generate on the host); one sequence, a 2048-id prompt,
    256 greedy steps.  Reports tok/s and the share of the all-reduces in a decode step."""
    import torch
    import torch.distributed as dist
    mio = pkg.model_io
    cfg = mio.CONFIGS[args.model]()
    tensors = mio.generate_tensors(cfg)
    prompt_len = min(2048, cfg.max_ctx - DECODE_STEPS - 1)
    ids = np.random.Generator(np.random.PCG64(cfg.seed)).integers(0, cfg.vocab, prompt_len).astype(np.int32)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    if world > 1:
        sub_cfg, sub = mio.shard_for_tensor_parallel(cfg, tensors, rank, world)
        ident = [pkg.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, src=0)
        kw = dict(tp_rank=rank, tp_world=world, tp_unique_id=ident[0])
    else:
        sub_cfg, sub, kw = cfg, tensors, dict(decode_mode=pkg.DECODE_PHASE_KERNELS)
    img = mio.export_model_litertlm(sub_cfg, mio.pack_weights_record(sub_cfg, sub))
    del tensors, sub
    ex = pkg.B200LlmExecutor(img, device=local_rank, stream=stream.cuda_stream, **kw)

    def step():
        ex.Reset()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(stream)
        ex.Prefill(ids, wait_for_completion=False)
        e1.record(stream)
        toks = ex.DecodeTokens(DECODE_STEPS)
        e2.record(stream)
        e2.synchronize()
        return e0.elapsed_time(e1), e1.elapsed_time(e2), toks

    step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    res = [step() for _ in range(max(1, min(args.steps, 3)))]
    pf = float(np.mean([r[0] for r in res]))
    dec = float(np.mean([r[1] for r in res]))
    t = torch.tensor([pf, dec], dtype=torch.float64, device="cuda")
    ar_ms = 0.0
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # the two buffers summed per layer: the O partials (one d-vector per head slice of the rank) and the down partials
        ar_counts = [(cfg.n_q_heads // world) * cfg.d_model, 4 * cfg.d_model]
        ar_ms = float(np.mean([ex.TpAllReduceProbe(c, 100) for c in ar_counts]))
    if rank != 0:
        return
    pf, dec = float(t[0]), float(t[1])
    n_ar = 2 * cfg.n_layers
    line = {
        "metric": "decode tok/s, one sequence, tensor parallel over the GPUs, Gemma3-27B layer geometry (slice)",
        "value": DECODE_STEPS / (dec / 1e3), "unit": "tok/s", "n_gpus": world, "steps": len(res), "warmup": 1,
        "ms_per_step": pf + dec, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int4 weights; int8 activation terms (decode), bf16 MMA (prefill), fp32 all-reduce", "data": "synthetic",
        "config": {"workload": f"{cfg.name} ({cfg.n_layers} layers): {prompt_len}-token prefill + {DECODE_STEPS} decode steps, batch 1, "
                               f"tensor parallel x{world}", "seed": cfg.seed, "decode": "one kernel per phase, all-reduce after O and down"},
        "prefill": {"value": prompt_len / (pf / 1e3), "unit": "tok/s", "ms": pf},
        "decode_ms_per_token": dec / DECODE_STEPS,
        "allreduce": {"per_decode_step": n_ar, "ms_each": ar_ms, "share_of_decode_step": (n_ar * ar_ms) / (dec / DECODE_STEPS) if world > 1 else 0.0,
                      "floats_each": [(cfg.n_q_heads // world) * cfg.d_model, 4 * cfg.d_model] if world > 1 else []},
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    global DECODE_STEPS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "xnnpack"])
    ap.add_argument("--model", default="gemma3-1b")
    ap.add_argument("--decode-mode", type=int, default=0)
    ap.add_argument("--prefill-gemm", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-xnnpack", action="store_true", help="skip the XNNPACK leg of the CPU arms")
    ap.add_argument("--threads", default="", help="thread counts of the XNNPACK leg (--impl xnnpack)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--batched-sessions", type=int, default=4,
                    help="extra leg: this many sessions per GPU decoded in lockstep (0 = skip)")
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg4", "cfg5"],
                    help="cfg2: the headline protocol (default); cfg4: 64 concurrent sessions of the 4B shape, sharded over the GPUs; "
                         "cfg5: tensor parallelism over the GPUs at the 27B shape's layer geometry")
    ap.add_argument("--sessions", type=int, default=64, help="cfg4: concurrent sessions over all GPUs")
    ap.add_argument("--kv-dtype", default="", choices=["", "fp32", "bf16"],
                    help="KV-cache type instead of the configuration's (cfg4 leaves it open; cfg2 specifies fp32)")
    ap.add_argument("--group", type=int, default=0, help="cfg4: sessions per lockstep group (0 = all of a GPU's sessions, at most 128)")
    ap.add_argument("--decode-steps", type=int, default=DECODE_STEPS,
                    help="decode steps per bench step (256 is the protocol; fewer only for profiler captures)")
    args = ap.parse_args()
    DECODE_STEPS = args.decode_steps
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "xnnpack":                   # child process of the CPU arms, prints one JSON object
        if int(os.environ.get("RANK", "0")) == 0:
            cfg, rec, _ = load_model(args.model)
            print(json.dumps(xnnpack_baseline(rec, cfg, [int(t) for t in args.threads.split(",") if t] or [host_threads()])),
                  flush=True)
        return
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "cfg4" and args.model == "gemma3-1b":
        args.model = "gemma3-4b"
    if args.workload == "cfg5" and args.model == "gemma3-1b":
        args.model = "gemma3-27b-slice"

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 executor has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    graft.build()
    pkg = graft.load_package()
    if args.workload == "cfg5":
        run_cfg5(args, pkg, rank, world, local_rank)
        if world > 1:
            dist.destroy_process_group()
        return
    if world > 1:
        # rank 0 generates (or finds) the cached model file; the others read it afterwards
        if rank == 0:
            cfg, rec, img = load_model(args.model, kv_dtype=args.kv_dtype)
        dist.barrier()
        if rank != 0:
            cfg, rec, img = load_model(args.model, kv_dtype=args.kv_dtype)
    else:
        cfg, rec, img = load_model(args.model, kv_dtype=args.kv_dtype)
    stream = torch.cuda.Stream()          # a real (non-default) stream: CUDA events below are recorded on it
    torch.cuda.set_stream(stream)
    if args.workload == "cfg4":
        run_cfg4(args, pkg, cfg, img, stream, rank, world, local_rank)
        if world > 1:
            dist.destroy_process_group()
        return
    ex = pkg.B200LlmExecutor(img, device=local_rank, decode_mode=args.decode_mode, prefill_gemm=args.prefill_gemm,
                             stream=stream.cuda_stream)
    # one session per GPU; session ids are sharded over the ranks, each with its own seeded prompt
    session = pkg.sharding.shard_sessions(world, world, rank)[0]
    ids = np.random.Generator(np.random.PCG64(pkg.sharding.session_seed(cfg.seed, session))).integers(
        0, cfg.vocab, PREFILL_TOKENS).astype(np.int32)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def device_step():
        ex.Reset()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(stream)
        ex.Prefill(ids, wait_for_completion=False)
        e1.record(stream)
        toks = ex.DecodeTokens(DECODE_STEPS)
        e2.record(stream)
        e2.synchronize()
        return e0.elapsed_time(e1), e1.elapsed_time(e2), toks

    logits_host = torch.empty((1, 1, cfg.vocab), dtype=torch.float32, pin_memory=True).numpy()

    def e2e_step():
        ex.Reset()
        logits = logits_host                  # page-locked: the device-to-host copy lands in it directly
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ex.Prefill(ids, wait_for_completion=True)
        t1 = time.perf_counter()
        tok = None
        toks = []
        for _ in range(DECODE_STEPS):
            ex.DecodeLogits(tok, out=logits)
            tok = int(np.argmax(logits))          # first maximum, as std::max_element
            toks.append(tok)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        return (t1 - t0) * 1e3, (t2 - t1) * 1e3, toks

    for _ in range(args.warmup):
        device_step()
    launches0 = ex.GetLaunchCount()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    pf_ms, dec_ms = [], []
    toks_dev = None
    for _ in range(args.steps):
        a, b, toks_dev = device_step()
        pf_ms.append(a)
        dec_ms.append(b)
    barrier()
    clocks = sampler.finish()
    launches = ex.GetLaunchCount() - launches0
    # whole job: tokens summed over ranks, device times (CUDA events) maxed over ranks
    dec_tokens, (pf_total, dec_total) = pkg.sharding.reduce_throughput(args.steps * DECODE_STEPS, [sum(pf_ms), sum(dec_ms)])
    decode_tok_s = dec_tokens / (dec_total / 1e3)
    prefill_tok_s = world * args.steps * PREFILL_TOKENS / (pf_total / 1e3)

    e2e = None
    if not args.no_e2e:
        e2e_step()
        ep, ed = [], []
        toks_e2e = None
        barrier()
        for _ in range(max(1, min(args.steps, 3))):
            a, b, toks_e2e = e2e_step()
            ep.append(a)
            ed.append(b)
        barrier()
        te = torch.tensor([float(np.mean(ep)), float(np.mean(ed))], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = {"value": world * DECODE_STEPS / (float(te[1]) / 1e3), "unit": "tok/s",
               "h2d_bytes_per_step": PREFILL_TOKENS * 4 + DECODE_STEPS * 8,
               "d2h_bytes_per_step": DECODE_STEPS * (cfg.vocab * 4 + 4),
               "prefill_tok_s": world * PREFILL_TOKENS / (float(te[0]) / 1e3),
               "api": "B200Lm_Prefill(host ids) + 256 x B200Lm_DecodeLogits(host logits) + host arg-max",
               "tokens_match_device_loop": bool(toks_dev is not None and list(toks_dev) == toks_e2e)}
    # extra leg (BASELINE config 4's way of running): several sessions per GPU in one executor, all
    # advanced by every decode step, weights read once per step.  Not the headline value.
    batched = None
    if args.batched_sessions > 1 and not args.no_e2e:
        nb = args.batched_sessions
        del ex
        exb = None
        while exb is None and nb > 1:
            try:
                exb = pkg.B200LlmExecutor(img, device=local_rank, decode_mode=args.decode_mode,
                                          prefill_gemm=args.prefill_gemm, stream=stream.cuda_stream, n_sessions=nb)
            except pkg.StatusError:
                nb -= 1          # the staging of that many sessions does not fit this model: try fewer
    if batched is None and args.batched_sessions > 1 and not args.no_e2e and exb is not None:
        prompts = [np.random.Generator(np.random.PCG64(pkg.sharding.session_seed(cfg.seed, world * (1 + i) + rank)))
                   .integers(0, cfg.vocab, PREFILL_TOKENS).astype(np.int32) for i in range(nb)]

        def batched_step():
            for i in range(nb):
                exb.SelectSession(i)
                exb.Reset()
                exb.PrefillSession(i, prompts[i], wait_for_completion=False)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            exb.DecodeTokensBatch(DECODE_STEPS)
            e1.record(stream)
            e1.synchronize()
            return e0.elapsed_time(e1)

        batched_step()
        barrier()
        bms = [batched_step() for _ in range(max(1, min(args.steps, 3)))]
        barrier()
        btok, (bt,) = pkg.sharding.reduce_throughput(len(bms) * nb * DECODE_STEPS, [sum(bms)])
        batched = {"sessions_per_gpu": nb, "value": btok / (bt / 1e3), "unit": "tok/s",
                   "ms_per_decode_step": float(np.mean(bms)) / DECODE_STEPS,
                   "note": "aggregate decode tok/s of all sessions on all GPUs; one pass over the weights per step"}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    bytes_per_tok = cfg.decode_bytes_per_token(s_lo=PREFILL_TOKENS, s_hi=PREFILL_TOKENS + DECODE_STEPS)
    per_gpu_dec_ms = float(np.mean(dec_ms))
    achieved_gbs = bytes_per_tok * DECODE_STEPS / (per_gpu_dec_ms / 1e3) / 1e9
    flops = cfg.prefill_flops(PREFILL_TOKENS - 1)       # the last prompt id is held back
    per_gpu_pf_ms = float(np.mean(pf_ms))
    achieved_tf = flops / (per_gpu_pf_ms / 1e3) / 1e12
    line = {
        "metric": METRIC, "value": decode_tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": (pf_total + dec_total) / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights; int8x3 activations (decode), bf16 MMA (prefill), fp32 accumulate",
        "data": "synthetic",
        "config": workload_config(cfg, world, args.decode_mode),
        "prefill": {"value": prefill_tok_s, "unit": "tok/s", "ms": per_gpu_pf_ms,
                    "roofline": {"bound": "tensor", "achieved": achieved_tf, "peak": peaks["bf16_tflops"],
                                 "unit": "TFLOP/s", "frac": achieved_tf / peaks["bf16_tflops"], "traffic": None,
                                 "flops_per_prefill": flops, "of": peaks["source"]}},
        "decode_ms_per_token": per_gpu_dec_ms / DECODE_STEPS,
        "clocks": clocks,
        "e2e": e2e,
        "batched_sessions": batched,
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved_gbs / peaks["hbm_gbs"], "traffic": DECODE_DRAM_BYTES_PER_STEP, "of": peaks["source"],
                     "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum per decode step, from an ncu capture of "
                                     "one two-step launch of the decode kernel",
                     "kernel": "decode step (all phases)", "algorithmic_bytes_per_token": bytes_per_tok,
                     "frac_of_nominal_8TBs": achieved_gbs / 8000.0},
    }
    if not args.no_cpu_baseline and world == 1:
        # the same sample as `--impl reference`: about 20 s of CPU work on 16 cores
        t0 = time.perf_counter()
        arm = CpuArm(rec, cfg)
        p = arm.prefill()
        d = float(np.mean([arm.decode_step(CPU_DECODE_TOKENS_PER_STEP) for _ in range(4)][1:]))
        line["cpu_baseline"] = {"value": d, "unit": "tok/s", "cores": host_threads(), "kind": "port",
                                "prefill_tok_s": p, "wall_s": time.perf_counter() - t0,
                                "sample": cpu_sample_text(CPU_DECODE_TOKENS_PER_STEP)}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
