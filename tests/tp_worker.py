"""One tensor-parallel rank of the 2-GPU parity test (launched by tests/test_gpu_tensor_parallel.py through
torch.distributed.run).  Every rank loads ITS shard of the model, all ranks make the same calls; rank 0 writes
the logits of every decode step and the device-loop tokens to an .npz file for the test to compare with the
CPU oracle of the unsplit model.

    python -m torch.distributed.run --nproc-per-node 2 tests/tp_worker.py <model> <prompt_len> <steps> <out.npz>
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402


def main() -> None:
    import torch
    import torch.distributed as dist
    name, prompt_len, steps, out_path = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")               # only carries the 128-byte group id; the data path is NCCL inside the library
    pkg = graft.load_package()
    mio = pkg.model_io
    cfg = mio.CONFIGS[name]()
    tensors = mio.generate_tensors(cfg)
    sub_cfg, sub = mio.shard_for_tensor_parallel(cfg, tensors, rank, world)
    img = mio.export_model_litertlm(sub_cfg, mio.pack_weights_record(sub_cfg, sub))
    ident = [pkg.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ident, src=0)
    ex = pkg.B200LlmExecutor(img, device=local, tp_rank=rank, tp_world=world, tp_unique_id=ident[0])
    ids = np.random.Generator(np.random.PCG64(51)).integers(0, cfg.vocab, prompt_len).astype(np.int32)
    ex.Prefill(ids)
    logits, tok = [], None
    forced = np.load(out_path + ".forced.npy") if os.path.exists(out_path + ".forced.npy") else None
    for s in range(steps):
        l = ex.DecodeLogits(tok).ravel().copy()
        logits.append(l)
        tok = int(forced[s]) if forced is not None else int(np.argmax(l))     # teacher-forced on the oracle's tokens
    free = list(ex.DecodeTokens(4)) if forced is None else []
    if forced is not None:
        ex.Prefill(np.array([int(forced[steps])], dtype=np.int32))
        free = list(ex.DecodeTokens(4))
    rows = np.stack([ex.ReadKvRow(sub_cfg.n_layers - 1, False, 0, p)[0][:cfg.head_dim] for p in (0, prompt_len - 2, prompt_len + 1)])
    if rank == 0:
        np.savez(out_path, logits=np.stack(logits), free=np.array(free, dtype=np.int64), rows=rows,
                 step=ex.GetCurrentStep(), mode=ex.GetDecodeMode())
    dist.barrier()
    ex.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
