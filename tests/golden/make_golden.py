"""Regenerates the committed fixtures in this directory.

  python tests/golden/make_golden.py

* tiny_lm_oracle.json — greedy tokens and the first logits of every step of the CPU
  oracle on the seeded tiny model (a regression pin of the oracle itself);
* litertlm_fixture.json — what the reference's own container fixture
  schema/testdata/test_hf_tokenizer.litertlm decodes to (header fields, flatbuffer
  bytes, section table, SHA-256 of the inflated tokenizer JSON) and the bytes of
  schema/testdata/llm_metadata.pb.  Needs the reference checkout; skipped when absent.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402
from oracle import oracle as orc  # noqa: E402

REF = os.environ.get("LITERT_LM_REFERENCE", os.path.join(os.sep, "root", "reference"))


def main() -> None:
    pkg = graft.load_package()
    mio = pkg.model_io
    cfg = mio.config_tiny()
    rec = mio.build_weights_record(cfg)
    ex = orc.OracleExecutor(orc.OracleModel(rec))
    seed, n = 0, 32
    ids = np.random.Generator(np.random.PCG64(seed)).integers(0, cfg.vocab, n).astype(np.int32)
    assert ex.prefill(ids) == 0
    toks, heads = [], []
    for step in range(16):
        rc, logits = ex.decode_logits(None if step == 0 else toks[-1])
        assert rc == 0
        toks.append(int(orc.greedy(logits)[0]))
        heads.append([float(x) for x in logits[:8]])
    with open(os.path.join(HERE, "tiny_lm_oracle.json"), "w") as f:
        json.dump({"config": "tiny", "prompt_seed": seed, "prompt_len": n, "greedy_tokens": toks,
                   "logits_head": heads, "record_sha256": hashlib.sha256(rec).hexdigest()}, f, indent=1)
    fixture = os.path.join(REF, "schema/testdata/test_hf_tokenizer.litertlm")
    if os.path.exists(fixture):
        data = open(fixture, "rb").read()
        lf = mio.read_litertlm(data)
        sec = lf.sections[0]
        tok = mio.read_hf_tokenizer_section(data[sec.begin:sec.end])
        ref_json = open(os.path.join(REF, "schema/testdata/tokenizer.json"), "rb").read()
        assert tok == ref_json
        out = {
            "file_size": len(data), "version": list(lf.version), "header_end": lf.header_end,
            "header_flatbuffer_hex": data[32:lf.header_end].hex(),
            "system": [[k, v, t] for k, v, t in lf.system],
            "sections": [{"data_type": s.data_type, "begin": s.begin, "end": s.end,
                          "items": [[k, v, t] for k, v, t in s.items]} for s in lf.sections],
            "tokenizer_json_sha256": hashlib.sha256(tok).hexdigest(), "tokenizer_json_size": len(tok),
            "llm_metadata_pb_hex": open(os.path.join(REF, "schema/testdata/llm_metadata.pb"), "rb").read().hex(),
        }
        with open(os.path.join(HERE, "litertlm_fixture.json"), "w") as f:
            json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
