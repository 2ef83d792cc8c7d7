"""The oracle against the reference's own known answers.

Each case cites the reference test or source lines it is taken from.  These pin the
parts of the hot path the reference does define: greedy / soft-max sampling, the prefill
work-group plan, the attention-mask rule and the executor's token hold-back.
"""
import json
import os

import numpy as np
import pytest

from conftest import seeded_ids

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


# ---- runtime/components/sampling_cpu_util_test.cc:16-96

def test_greedy_batch2_lowest_index(orc):
    # TopKIndicies_BatchSize2: logits {0.1,0.5,0.4,0.2}, k=1, batch 2 -> {1, 0}
    assert list(orc.greedy(np.array([0.1, 0.5, 0.4, 0.2], np.float32), batch=2)) == [1, 0]


def test_greedy_ties_take_first(orc):
    # std::max_element returns the first maximum (sampling_cpu_util.cc:32-41)
    assert list(orc.greedy(np.array([1.0, 3.0, 3.0, 2.0, 3.0], np.float32))) == [1]


def test_greedy_bad_batch(orc):
    with pytest.raises(ValueError):
        orc.greedy(np.zeros(5, np.float32), batch=2)


def test_softmax_batch1(orc):
    p, m = orc.softmax([0.1, 0.1], [0, 1], 1.0, 1)
    assert list(p) == [0.5, 0.5] and list(m) == [np.float32(0.1)]


def test_softmax_all_zero(orc):
    p, m = orc.softmax([0.0, 0.0], [0, 1], 1.0, 1)
    assert list(p) == [0.5, 0.5] and list(m) == [0.0]


def test_softmax_tiny_temperature(orc):
    p, m = orc.softmax([0.0, 1.0, 2.0], [0, 1, 2], 1e-8, 1)
    assert list(p) == [0.0, 0.0, 1.0] and list(m) == [2.0]


def test_softmax_huge_temperature(orc):
    p, m = orc.softmax([0.0, 1.0, 2.0, 3.0], [0, 1, 2, 3], 1e11, 1)
    assert list(p) == [0.25, 0.25, 0.25, 0.25] and list(m) == [3.0]


def test_softmax_batch3(orc):
    p, m = orc.softmax([0.1, 0.1, 0.0, 5.0, 1.0, 0.0], [0, 1, 0, 1, 0, 1], 1.0, 3)
    np.testing.assert_allclose(p, [0.5, 0.5, 0.00669285096, 0.993307173, 0.731058598, 0.268941432], rtol=1e-6)
    assert list(m) == [np.float32(0.1), 5.0, 1.0]


def test_softmax_rejects_zero_temperature(orc):
    with pytest.raises(ValueError):
        orc.softmax([0.0, 1.0], [0, 1], 0.0, 1)


# ---- runtime/executor/litert_compiled_model_executor_utils.cc:300-330 (no reference test exists)

@pytest.mark.parametrize("buckets,n,want", [
    ([1024, 128], 1100, [(1024, 1024), (128, 76)]),
    ([1024, 128], 1024, [(1024, 1024)]),
    ([1024, 512, 128], 100, [(128, 100)]),
    ([1024, 512, 128], 129, [(512, 129)]),
    ([1024, 512, 128], 2048 + 513, [(1024, 1024), (1024, 1024), (1024, 513)]),
    ([32, 8], 32, [(32, 32)]),
    ([32, 8], 41, [(32, 32), (32, 9)]),
    ([32, 8], 1, [(8, 1)]),
])
def test_work_group_plan(orc, buckets, n, want):
    assert orc.plan_work_groups(buckets, n) == want


# ---- litert_compiled_model_executor_utils.cc:332-397

def test_mask_rule(orc):
    m = orc.fill_mask(rows=4, ctx=16, start=5, steps=3, is_f16=True)
    for i in range(3):
        assert np.all(m[i, :5 + i + 1] == 0.0)
        assert np.all(m[i, 5 + i + 1:] == np.float32(-45824))
    assert np.all(m[3] == np.float32(-45824))          # padded row stays closed
    m32 = orc.fill_mask(rows=1, ctx=4, start=0, steps=1, is_f16=False)
    assert m32[0, 0] == 0.0 and m32[0, 1] == np.float32(-0.7 * 3.402823466e+38)


# ---- llm_litert_compiled_model_executor.cc:157-298,416-574 and .h:95-97

def test_hold_back_and_step_counter(orc, models):
    cfg, rec, _ = models("tiny")
    ex = orc.OracleExecutor(orc.OracleModel(rec))
    ids = seeded_ids(0, cfg.vocab, 12)
    assert ex.prefill(ids[:3]) == 0
    # 3 ids: two processed, the third pending (fake_llm_executor_test.cc: GetCurrentStep()==3 after a 3-id prefill)
    assert ex.internal_step == 2 and ex.pending_token == ids[2] and ex.current_step == 3
    rc, tok = ex.decode_token()
    assert rc == 0 and ex.internal_step == 3 and ex.pending_token == tok and ex.current_step == 4
    # pending id goes first in the next prefill and does not consume an input id
    assert ex.prefill(ids[3:6]) == 0
    assert ex.internal_step == 6 and ex.pending_token == ids[5] and ex.current_step == 7


def test_one_id_prefill_drops_pending(orc, models):
    cfg, rec, _ = models("tiny")
    ex = orc.OracleExecutor(orc.OracleModel(rec))
    assert ex.prefill([5, 6, 7]) == 0
    assert ex.prefill([9]) == 0            # loop bound ids.size()-1 == 0: nothing runs, pending replaced
    assert ex.internal_step == 2 and ex.pending_token == 9 and ex.current_step == 3


def test_work_groups_and_hold_back_across_buckets(orc, models):
    cfg, rec, _ = models("tiny")           # buckets (32, 8)
    ex = orc.OracleExecutor(orc.OracleModel(rec))
    ids = seeded_ids(3, cfg.vocab, 41)
    assert ex.prefill(ids) == 0
    assert ex.last_plan() == [(32, 32), (32, 9)]
    # group 1 runs ids[0..30] and holds ids[31]; group 2 runs ids[31] + ids[32..39], holds ids[40]
    assert ex.internal_step == 40 and ex.pending_token == ids[40] and ex.current_step == 41


def test_decode_without_id_is_invalid_argument(orc, models):
    cfg, rec, _ = models("tiny")
    ex = orc.OracleExecutor(orc.OracleModel(rec))
    rc, _ = ex.decode_logits()
    assert rc == 3                          # "No id available to be decoded."
    rc, logits = ex.decode_logits(token=4)  # an explicit id is accepted
    assert rc == 0 and logits.shape == (cfg.vocab,)
    assert ex.current_step == 1 and ex.pending_token == -1


def test_reset_keeps_cache(orc, models):
    cfg, rec, _ = models("tiny")
    ex = orc.OracleExecutor(orc.OracleModel(rec))
    ex.prefill([1, 2, 3, 4])
    row = ex.read_kv(0, False, 0, 1).copy()
    ex.reset()
    assert ex.current_step == 0 and ex.pending_token == -1
    assert np.array_equal(ex.read_kv(0, False, 0, 1), row)


def test_prefill_split_is_invariant(orc, models):
    """Feeding the same ids in one call or in pieces gives the same logits: the hold-back
    only moves chunk boundaries."""
    cfg, rec, _ = models("tiny")
    m = orc.OracleModel(rec)
    ids = seeded_ids(5, cfg.vocab, 20)
    a, b = orc.OracleExecutor(m), orc.OracleExecutor(m)
    a.prefill(ids)
    b.prefill(ids[:7]); b.prefill(ids[7:13]); b.prefill(ids[13:])
    la, lb = a.decode_logits()[1], b.decode_logits()[1]
    np.testing.assert_allclose(la, lb, rtol=0, atol=1e-5)


# ---- frozen outputs of the oracle itself (regression pin; see tests/golden/make_golden.py)

def test_oracle_matches_committed_vectors(orc, models):
    with open(os.path.join(GOLDEN, "tiny_lm_oracle.json")) as f:
        g = json.load(f)
    cfg, rec, _ = models("tiny")
    ex = orc.OracleExecutor(orc.OracleModel(rec))
    ids = seeded_ids(g["prompt_seed"], cfg.vocab, g["prompt_len"])
    assert ex.prefill(ids) == 0
    toks = []
    for step in range(len(g["greedy_tokens"])):
        rc, logits = ex.decode_logits(None if step == 0 else toks[-1])
        assert rc == 0
        toks.append(int(orc.greedy(logits)[0]))
        np.testing.assert_allclose(logits[:8], g["logits_head"][step], rtol=1e-4, atol=1e-5)
    assert toks == g["greedy_tokens"]


def test_int4_convention(orc, mio):
    rng = np.random.Generator(np.random.PCG64(11))
    w = rng.standard_normal((32, 128), dtype=np.float32) * 0.02
    p_np, s_np = mio.quantize_int4(w)
    p_c, s_c = orc.quantize_int4(w)
    assert np.array_equal(p_np, p_c) and np.array_equal(s_np, s_c)
    q = orc.unpack_int4(p_c)
    assert np.array_equal(q, mio.unpack_int4(p_np))
    assert q.min() >= -7 and q.max() <= 7
    assert np.all(np.abs(q).max(axis=1) == 7)          # scale = max|w| / 7
    # low nibble = even element
    assert (p_c[0, 0] & 0xF) == (int(q[0, 0]) & 0xF) and (p_c[0, 0] >> 4) == (int(q[0, 1]) & 0xF)


def test_kv_index_rule(orc):
    assert orc.kv_index(0) == (0, 0)
    assert orc.kv_index(255) == (0, 255)
    assert orc.kv_index(256) == (1, 0)
    assert orc.kv_index(4095) == (15, 255)
    assert orc.kv_offset(3, 1, 7, 4, 128) == ((3 * 4 + 1) * 256 + 7) * 128
