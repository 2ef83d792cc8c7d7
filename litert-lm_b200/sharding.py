"""Session sharding across the GPUs of one node.

Independent sessions (the reference runs one `LlmExecutor` per session,
runtime/core/session_basic.cc) are partitioned over ranks with no collective on
the data path: every rank owns whole sessions, KV cache included.  The only
communication is the timing reduction a benchmark does at the end (max over
ranks of the elapsed time, sum of the tokens).  Works on any torch.distributed
backend; the unit tests drive it with gloo on CPU.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_sessions(n_sessions: int, world: int, rank: int) -> List[int]:
    """Session ids owned by `rank`: contiguous blocks, sizes differing by at most one.

    Contiguous (not strided) so that a rank's sessions keep the order of the
    request list, which is the order their results are reported in."""
    if n_sessions < 0 or world <= 0 or not 0 <= rank < world:
        raise ValueError("bad sharding arguments")
    base, extra = divmod(n_sessions, world)
    lo = rank * base + min(rank, extra)
    return list(range(lo, lo + base + (1 if rank < extra else 0)))


def session_seed(model_seed: int, session: int) -> int:
    """Prompt seed of a session: independent of how sessions are sharded."""
    return model_seed + 1000 * session


def reduce_throughput(tokens: float, elapsed_ms: Sequence[float]) -> Tuple[float, List[float]]:
    """Whole-job totals: (sum of tokens over ranks, element-wise max of the elapsed times).

    Without an initialised process group this is the identity (single GPU)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(tokens), [float(x) for x in elapsed_ms]
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([float(tokens)], dtype=torch.float64, device=dev)
    e = torch.tensor([float(x) for x in elapsed_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    dist.all_reduce(e, op=dist.ReduceOp.MAX)
    return float(t[0]), [float(x) for x in e]
