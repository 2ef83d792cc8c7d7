"""Several sessions in one executor, decoded in lockstep (one pass over the weights per step
for the whole batch): every session's tokens must be the ones it produces alone, which are
the CPU oracle's."""
import numpy as np
import pytest

from conftest import logits_close, seeded_ids

pytestmark = pytest.mark.gpu


def oracle_tokens(orc, rec, prompt, steps):
    ref = orc.OracleExecutor(orc.OracleModel(rec))
    assert ref.prefill(prompt) == 0
    out = [ref.decode_token()[1] for _ in range(steps)]
    step = ref.current_step
    ref.close()
    return out, step


@pytest.mark.parametrize("name,n_sessions,lens", [
    ("tiny", 2, (32, 9)), ("tiny", 4, (32, 9, 17, 40)), ("small", 2, (200, 300)), ("small", 3, (64, 257, 100)),
    ("small-gqa", 4, (150, 20, 33, 128)),
])
def test_lockstep_sessions_match_single_session_and_oracle(pkg, orc, models, name, n_sessions, lens):
    cfg, rec, img = models(name)
    steps = 16
    prompts = [seeded_ids(20 + i, cfg.vocab, n) for i, n in enumerate(lens)]
    ex = pkg.B200LlmExecutor(img, n_sessions=n_sessions)
    assert ex.GetNumSessions() == n_sessions
    for i, p in enumerate(prompts):
        ex.PrefillSession(i, p)
    got = ex.DecodeTokensBatch(steps)
    assert got.shape == (steps, n_sessions)
    for i, p in enumerate(prompts):
        want, want_step = oracle_tokens(orc, rec, p, steps)
        assert list(got[:, i]) == want, (i, list(got[:, i]), want)
        ex.SelectSession(i)
        assert ex.GetCurrentStep() == want_step               # processed ids + the pending one
    # a session alone (one column, three int8 terms) gives the same ids
    solo = pkg.B200LlmExecutor(img)
    solo.Prefill(prompts[-1])
    assert list(solo.DecodeTokens(steps)) == list(got[:, -1])


def test_single_session_calls_leave_the_other_sessions_alone(pkg, orc, models):
    cfg, rec, img = models("small")
    a, b = seeded_ids(31, cfg.vocab, 120), seeded_ids(32, cfg.vocab, 70)
    ex = pkg.B200LlmExecutor(img, n_sessions=2)
    ex.PrefillSession(0, a)
    ex.PrefillSession(1, b)
    first = ex.DecodeTokensBatch(4)
    # session 1 goes on alone through the logits path; session 0 must not move
    ex.SelectSession(1)
    ref = orc.OracleExecutor(orc.OracleModel(rec))
    ref.prefill(b)
    want_b = [ref.decode_token()[1] for _ in range(4)]
    assert list(first[:, 1]) == want_b
    rc, want_logits = ref.decode_logits(None)
    got_logits = ex.DecodeLogits().ravel()
    cos, err = logits_close(got_logits, want_logits)
    assert cos >= 0.999 and err <= 2e-2
    ex.SelectSession(0)
    assert ex.GetCurrentStep() == 120 + 4
    # session 1 has no pending id now (the logits path does not sample): a lockstep step is refused, nothing changes
    with pytest.raises(pkg.StatusError) as e:
        ex.DecodeTokensBatch(1)
    assert e.value.code == pkg.INVALID_ARGUMENT
    assert ex.GetCurrentStep() == 120 + 4
    # session 0 alone continues exactly as the oracle does
    want_a, _ = oracle_tokens(orc, rec, a, 8)
    assert list(first[:, 0]) == want_a[:4]
    assert list(ex.DecodeTokens(4)) == want_a[4:]


def test_session_count_is_checked(pkg, models):
    cfg, rec, img = models("tiny")
    with pytest.raises(pkg.StatusError) as e:
        pkg.B200LlmExecutor(img, n_sessions=129)
    assert e.value.code == pkg.INVALID_ARGUMENT
    ex = pkg.B200LlmExecutor(img, n_sessions=2)
    with pytest.raises(pkg.StatusError):
        ex.SelectSession(2)


def test_two_sessions_at_the_benchmark_shape(pkg, models):
    cfg, rec, img = models("gemma3-1b")
    p0, p1 = seeded_ids(41, cfg.vocab, 1024), seeded_ids(42, cfg.vocab, 700)
    ex = pkg.B200LlmExecutor(img, n_sessions=2)
    ex.PrefillSession(0, p0)
    ex.PrefillSession(1, p1)
    got = ex.DecodeTokensBatch(32)
    for i, p in enumerate((p0, p1)):
        solo = pkg.B200LlmExecutor(img)
        solo.Prefill(p)
        assert list(solo.DecodeTokens(32)) == list(got[:, i]), i
