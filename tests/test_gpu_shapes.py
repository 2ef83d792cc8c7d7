"""Parity at the per-layer geometry of the two larger benchmark shapes (4B: hidden 2560, 8 query /
4 kv heads of 256, ffn 10240; 27B: hidden 5376, 32 query / 16 kv heads of 128, ffn 21504), on
slices of a few layers so the CPU oracle keeps up.  One GPU, no tensor parallelism.  The prompts
are longer than the 1024-position window, so the local layers really drop keys."""
import numpy as np
import pytest

from conftest import logits_close, seeded_ids

pytestmark = pytest.mark.gpu

COS_MIN, ERR_MAX = 0.999, 2e-2


@pytest.mark.parametrize("name,prompt_len", [("gemma3-4b-slice", 1100), ("gemma3-27b-slice", 1100)])
def test_logits_and_tokens_match_oracle_on_large_layer_shapes(pkg, orc, models, name, prompt_len):
    cfg, rec, img = models(name)
    prompt = seeded_ids(51, cfg.vocab, prompt_len)
    ex = pkg.B200LlmExecutor(img)
    ref = orc.OracleExecutor(orc.OracleModel(rec))
    ex.Prefill(prompt)
    assert ref.prefill(prompt) == 0
    tok = None
    for step in range(8):
        got = ex.DecodeLogits(tok).ravel()
        rc, want = ref.decode_logits(tok)
        assert rc == 0
        cos, err = logits_close(got, want)
        assert cos >= COS_MIN and err <= ERR_MAX, (step, cos, err)
        tok = int(orc.greedy(want)[0])
        order = np.sort(want)[::-1]
        assert int(np.argmax(got)) == tok, (step, "oracle margin", float(order[0] - order[1]),
                                            "max abs err", float(np.abs(got - want).max()))
    # the device loop continues from the same state with the same ids as the oracle
    ex.Prefill([tok])                       # 1-id prefill: replaces the pending id, processes nothing
    ref.prefill(np.array([tok], dtype=np.int32))
    assert list(ex.DecodeTokens(4)) == [ref.decode_token()[1] for _ in range(4)]
    for pos in (0, prompt_len - 2, prompt_len + 3):
        for is_v in (False, True):
            row = ex.ReadKvRow(cfg.n_layers - 1, is_v, cfg.n_kv_heads - 1, pos)[0][:cfg.head_dim]
            want = ref.read_kv(cfg.n_layers - 1, is_v, cfg.n_kv_heads - 1, pos)
            assert np.abs(row - want).max() <= 2e-2 * max(1.0, np.abs(want).max()), (pos, is_v)
