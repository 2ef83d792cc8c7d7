"""Wide lockstep decode (B200LM_DECODE_WIDE): more sessions per executor than the GEMV kernels carry, the
projections of a step on the tensor-core int4 GEMM with the sessions as its token rows.  Activations are bf16
(as in prefill), so logits are held to the prefill tolerance and greedy ids are checked against the oracle
teacher-forced on the device's own ids: the id the device picked must be the oracle's arg-max, or within the
logit tolerance of it."""
import numpy as np
import pytest

from conftest import logits_close, seeded_ids

pytestmark = pytest.mark.gpu

COS_MIN, ERR_MAX = 0.999, 2e-2


def check_against_oracle(orc, rec, prompt, ids):
    """Teacher-forced on `ids` (what the device produced): every id must be (nearly) the oracle's arg-max."""
    ref = orc.OracleExecutor(orc.OracleModel(rec))
    assert ref.prefill(prompt) == 0
    exact = 0
    for step, tok in enumerate(ids):
        rc, want = ref.decode_logits(None if step == 0 else int(ids[step - 1]))
        assert rc == 0
        top = int(orc.greedy(want)[0])
        span = float(want.max() - want.min())
        assert want[tok] >= want[top] - ERR_MAX * span, (step, tok, top, float(want[top] - want[tok]), span)
        exact += int(tok == top)
    return exact


@pytest.mark.parametrize("name,n_sessions,prompt_len", [("small", 6, 70), ("small-gqa", 9, 40), ("tiny", 5, 20)])
def test_wide_batch_matches_oracle(pkg, orc, models, name, n_sessions, prompt_len):
    cfg, rec, img = models(name)
    ex = pkg.B200LlmExecutor(img, n_sessions=n_sessions)
    assert ex.GetDecodeMode() == pkg.DECODE_WIDE
    prompts = [seeded_ids(10 + s, cfg.vocab, prompt_len + 3 * s) for s in range(n_sessions)]
    for s, p in enumerate(prompts):
        ex.PrefillSession(s, p, wait_for_completion=(s % 2 == 0))
    steps = 12
    out = ex.DecodeTokensBatch(steps)                  # [steps, n_sessions]
    assert out.shape == (steps, n_sessions)
    exact = 0
    for s, p in enumerate(prompts):
        exact += check_against_oracle(orc, rec, p, [int(t) for t in out[:, s]])
        ex.SelectSession(s)
        assert ex.GetCurrentStep() == len(p) + steps      # the last id is pending, and counted
    assert exact >= 0.9 * steps * n_sessions           # bf16 activations: a near-tie may flip, most ids are exact


def test_wide_single_session_logits_and_kv(pkg, orc, models):
    """The same step with one row: logits against the oracle, and the appended K / V rows."""
    cfg, rec, img = models("small")
    prompt = seeded_ids(3, cfg.vocab, 90)
    ex = pkg.B200LlmExecutor(img, decode_mode=pkg.DECODE_WIDE, n_sessions=3)
    ex.PrefillSession(1, prompt)
    ref = orc.OracleExecutor(orc.OracleModel(rec))
    assert ref.prefill(prompt) == 0
    tok = None
    for step in range(4):
        got = ex.DecodeLogits(tok).ravel()
        rc, want = ref.decode_logits(tok)
        assert rc == 0
        cos, err = logits_close(got, want)
        assert cos >= COS_MIN and err <= ERR_MAX, (step, cos, err)
        tok = int(orc.greedy(want)[0])
    pos = len(prompt) - 1 + 3
    for layer in (0, cfg.n_layers - 1):
        for is_v in (0, 1):
            row, _, _ = ex.ReadKvRow(layer, is_v, 0, pos)
            want = ref.read_kv(layer, is_v, 0, pos)
            got = row[:cfg.head_dim]
            assert np.abs(got - want).max() <= 2e-2 * max(1.0, np.abs(want).max()), (layer, is_v)


def test_wide_equals_wide_in_any_grouping(pkg, models):
    """A session's ids do not depend on which other sessions share its steps (rows are independent)."""
    cfg, rec, img = models("small")
    prompts = [seeded_ids(40 + s, cfg.vocab, 50 + s) for s in range(7)]
    ex = pkg.B200LlmExecutor(img, n_sessions=7)
    for s, p in enumerate(prompts):
        ex.PrefillSession(s, p)
    together = ex.DecodeTokensBatch(10)
    solo = pkg.B200LlmExecutor(img, decode_mode=pkg.DECODE_WIDE, n_sessions=1)
    for s in (0, 3, 6):
        solo.Reset()
        solo.Prefill(prompts[s])
        assert [int(t) for t in solo.DecodeTokens(10)] == [int(t) for t in together[:, s]]


def test_wide_8_sessions_on_the_4b_slice(pkg, orc, models):
    """BASELINE config 4's regime: 8 lockstep sessions of the 4B layer geometry against the oracle."""
    cfg, rec, img = models("gemma3-4b-slice")
    n = 8
    prompts = [seeded_ids(70 + s, cfg.vocab, 120 + 17 * s) for s in range(n)]
    ex = pkg.B200LlmExecutor(img, n_sessions=n, max_num_tokens=512)
    assert ex.GetDecodeMode() == pkg.DECODE_WIDE
    for s, p in enumerate(prompts):
        ex.PrefillSession(s, p, wait_for_completion=False)
    out = ex.DecodeTokensBatch(8)
    exact = sum(check_against_oracle(orc, rec, prompts[s], [int(t) for t in out[:, s]]) for s in range(n))
    assert exact >= 0.9 * 8 * n


def test_wide_rejects_more_than_its_capacity(pkg, models):
    cfg, rec, img = models("tiny")
    with pytest.raises(pkg.StatusError):
        pkg.B200LlmExecutor(img, n_sessions=129)
