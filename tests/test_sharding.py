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


def _tp_partial_products_worker(rank, world, port, q):
    """Each rank multiplies its slice of W_o and W_down with its slice of the input; the gloo all-reduce of
    the partial products must equal the product with the unsplit matrices."""
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as graft
    mio = graft.load_package().model_io
    cfg = mio.config_small_gqa()
    t = mio.generate_tensors(cfg)
    sub_cfg, sub = mio.shard_for_tensor_parallel(cfg, t, rank, world)
    rng = np.random.default_rng(3)
    x_attn = rng.standard_normal(cfg.n_q_heads * cfg.head_dim)
    x_act = rng.standard_normal(cfg.ffn)
    errs = []
    for nm, x, per in (("L1.wo", x_attn, cfg.n_q_heads * cfg.head_dim // world), ("L1.wdown", x_act, cfg.ffn // world)):
        full = (mio.unpack_int4(t[nm + ".q"]).astype(np.float64) * t[nm + ".scale"][:, None]) @ x
        part = (mio.unpack_int4(sub[nm + ".q"]).astype(np.float64) * sub[nm + ".scale"][:, None]) @ x[rank * per:(rank + 1) * per]
        tot = torch.from_numpy(part.copy())
        dist.all_reduce(tot)
        errs.append(float(np.abs(tot.numpy() - full).max()))
    q.put((rank, errs, sub_cfg.n_q_heads, sub_cfg.n_kv_heads, sub_cfg.ffn))
    dist.destroy_process_group()


def test_tensor_parallel_shards_reassemble_and_partial_products_add_up():
    """World size 2 on CPU (gloo): the shards of the head-split and column-split matrices re-assemble to the
    unsplit ones, and the all-reduced partial O / down products equal the unsplit products."""
    import multiprocessing as mp
    import __graft_entry__ as graft
    mio = graft.load_package().model_io
    cfg = mio.config_small_gqa()
    t = mio.generate_tensors(cfg)
    world = 2
    shards = [mio.shard_for_tensor_parallel(cfg, t, r, world)[1] for r in range(world)]
    hq, hkv, hd = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
    q_rows = np.concatenate([s["L0.wqkv.q"][:hq // world * hd] for s in shards])
    k_rows = np.concatenate([s["L0.wqkv.q"][hq // world * hd:(hq + hkv) // world * hd] for s in shards])
    v_rows = np.concatenate([s["L0.wqkv.q"][(hq + hkv) // world * hd:] for s in shards])
    assert np.array_equal(np.concatenate([q_rows, k_rows, v_rows]), t["L0.wqkv.q"])
    assert np.array_equal(np.concatenate([s["L0.wgate.q"] for s in shards]), t["L0.wgate.q"])
    assert np.array_equal(np.concatenate([s["L0.wo.q"] for s in shards], axis=1), t["L0.wo.q"])
    assert np.array_equal(np.concatenate([s["L0.wdown.q"] for s in shards], axis=1), t["L0.wdown.q"])
    assert all(np.array_equal(s["L0.wo.scale"], t["L0.wo.scale"]) and np.array_equal(s["embed.q"], t["embed.q"]) for s in shards)
    with pytest.raises(ValueError):
        mio.shard_for_tensor_parallel(cfg, t, 0, 3)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tp_partial_products_worker, args=(r, world, 29533, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, errs, nq, nkv, ffn in res:
        assert max(errs) < 1e-9, (rank, errs)
        assert (nq, nkv, ffn) == (hq // world, hkv // world, cfg.ffn // world)
