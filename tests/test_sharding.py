"""Session sharding over ranks: pure logic, then a world-size-2 gloo run on CPU in which
each rank decodes its own sessions with the CPU oracle and the totals are reduced the way
bench.py does it."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402

pkg = graft.load_package()
sharding = pkg.sharding


def test_shards_partition_sessions():
    for n in (0, 1, 2, 7, 64):
        for world in (1, 2, 3, 4, 8):
            seen = []
            sizes = []
            for r in range(world):
                s = sharding.shard_sessions(n, world, r)
                assert s == sorted(s)
                seen += s
                sizes.append(len(s))
            assert seen == list(range(n))
            assert max(sizes) - min(sizes) <= 1


def test_shard_arguments_are_checked():
    with pytest.raises(ValueError):
        sharding.shard_sessions(4, 0, 0)
    with pytest.raises(ValueError):
        sharding.shard_sessions(4, 2, 2)
    with pytest.raises(ValueError):
        sharding.shard_sessions(-1, 2, 0)


def test_reduce_is_identity_without_a_process_group():
    tok, ms = sharding.reduce_throughput(12, [1.5, 2.5])
    assert tok == 12.0 and ms == [1.5, 2.5]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _decode_session(session, steps=4):
    """Tokens of one session on the tiny model with the CPU oracle."""
    from oracle import oracle as orc
    mio = pkg.model_io
    cfg = mio.CONFIGS["tiny"]()
    rec = mio.build_weights_record(cfg)
    model = orc.OracleModel(rec)
    ex = orc.OracleExecutor(model)
    seed = sharding.session_seed(cfg.seed, session)
    ids = np.random.Generator(np.random.PCG64(seed)).integers(0, cfg.vocab, 9).astype(np.int32)
    assert ex.prefill(ids) == 0
    toks = []
    for _ in range(steps):
        rc, t = ex.decode_token()
        assert rc == 0
        toks.append(int(t))
    ex.close()
    return toks


def _rank_main(rank, world, port, n_sessions, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = sharding.shard_sessions(n_sessions, world, rank)
        out = {s: _decode_session(s) for s in mine}
        ntok = sum(len(v) for v in out.values())
        total, ms = sharding.reduce_throughput(ntok, [10.0 * (rank + 1), 3.0])
        q.put((rank, out, total, ms))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo_cover_all_sessions_and_match_single_process():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, n_sessions, port = 2, 3, _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, n_sessions, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    merged = {}
    for rank, out, total, ms in got:
        assert total == 4.0 * n_sessions            # sum over ranks
        assert ms == [10.0 * world, 3.0]             # max over ranks
        assert not set(out) & set(merged)
        merged.update(out)
    assert sorted(merged) == list(range(n_sessions))
    for s in range(n_sessions):                      # sharding does not change any session's tokens
        assert merged[s] == _decode_session(s)
