"""Tensor parallelism over two GPUs (BASELINE config 5's partitioning: query / kv heads and FFN columns split
over the ranks, NCCL all-reduce of the partial O and down projections) against the CPU oracle of the UNSPLIT
model, at the 27B shape's layer geometry.  Needs two B200s; skipped on a single-GPU box."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import logits_close, seeded_ids

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _two_gpus() -> bool:
    import torch
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


@pytest.mark.parametrize("name,prompt_len", [("small-gqa", 150), ("gemma3-27b-slice", 300)])
def test_two_rank_tensor_parallel_matches_the_unsplit_oracle(pkg, orc, models, tmp_path, name, prompt_len):
    if not _two_gpus():
        pytest.skip("needs two GPUs")
    cfg, rec, img = models(name)
    steps = 6
    prompt = seeded_ids(51, cfg.vocab, prompt_len)
    ref = orc.OracleExecutor(orc.OracleModel(rec))
    assert ref.prefill(prompt) == 0
    want, forced, tok = [], [], None
    for _ in range(steps):
        rc, l = ref.decode_logits(tok)
        assert rc == 0
        want.append(l.copy())
        tok = int(orc.greedy(l)[0])
        forced.append(tok)
    ref.prefill(np.array([tok], dtype=np.int32))
    free_want = [ref.decode_token()[1] for _ in range(4)]
    out = str(tmp_path / "tp.npz")
    np.save(out + ".forced.npy", np.array(forced + [tok], dtype=np.int64))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", os.path.join(ROOT, "tests", "tp_worker.py"), name, str(prompt_len), str(steps), out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    got = np.load(out)
    assert int(got["mode"]) == pkg.DECODE_PHASE_KERNELS          # a collective cannot run inside a persistent kernel
    for s in range(steps):
        cos, err = logits_close(got["logits"][s], want[s])
        assert cos >= 0.999 and err <= 2e-2, (s, cos, err)
        assert int(np.argmax(got["logits"][s])) == forced[s], s
    assert list(got["free"]) == free_want
    # rank 0 holds kv head 0 of the unsplit model
    for i, pos in enumerate((0, prompt_len - 2, prompt_len + 1)):
        w = ref.read_kv(cfg.n_layers - 1, False, 0, pos)
        assert np.abs(got["rows"][i] - w).max() <= 2e-2 * max(1.0, np.abs(w).max()), pos
