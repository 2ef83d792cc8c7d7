"""The C++ LlmExecutorBase adapter (litert-lm_b200/adapter) compiled against the shim and
linked to libb200lm.so."""
import os
import subprocess

import numpy as np
import pytest

from conftest import seeded_ids

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "litert-lm_b200")


@pytest.fixture(scope="module")
def driver(pkg, tmp_path_factory):
    out = tmp_path_factory.mktemp("adapter") / "adapter_driver"
    cmd = ["/usr/bin/g++", "-std=c++17", "-Wall", "-O1", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(PKG, "adapter"), os.path.join(ROOT, "tests", "cpp", "adapter_driver.cc"),
           "-L", PKG, "-lb200lm", "-Wl,-rpath," + PKG, "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return str(out)


def run_driver(driver, model_path, n_decode, ids):
    r = subprocess.run([driver, model_path, str(n_decode)] + [str(int(i)) for i in ids], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    return dict(line.split("=", 1) for line in r.stdout.strip().splitlines() if "=" in line)


def test_adapter_compiles_and_reports_missing_gpu_or_runs(driver, models, tmp_path):
    import torch
    cfg, rec, img = models("tiny")
    path = tmp_path / "tiny.litertlm"
    path.write_bytes(img)
    out = run_driver(driver, str(path), 4, seeded_ids(0, cfg.vocab, 12))
    if not torch.cuda.is_available():
        assert out["create_code"] == "9" and "no CPU fallback" in out["create_msg"]
    else:
        assert out["prefill_code"] == "0"


@pytest.mark.gpu
def test_adapter_matches_c_abi(driver, pkg, models, tmp_path):
    cfg, rec, img = models("tiny")
    path = tmp_path / "tiny.litertlm"
    path.write_bytes(img)
    ids = seeded_ids(0, cfg.vocab, 12)
    out = run_driver(driver, str(path), 6, ids)
    ex = pkg.B200LlmExecutor(img)
    ex.Prefill(ids)
    want = [ex.Decode() for _ in range(6)]
    assert out["backend"] == ex.ExecutorBackendName()
    assert out["prefill_code"] == "0" and out["step_after_prefill"] == "12" and out["vocab"] == str(cfg.vocab)
    assert [int(t) for t in out["tokens"].strip(",").split(",")] == want
    logits = ex.DecodeLogits(int(ids[0])).ravel()
    assert out["logits_dims"] == "3" and int(out["logits_argmax"]) == int(np.argmax(logits))
    assert out["live_locks"] == "0"                                # no mapping outlives the call that wrote the logits
    assert out["max_num_tokens"] == str(cfg.max_ctx)               # GetExecutorSettings().GetMaxNumTokens() = KV capacity
    assert out["cancelled_prefill_code"] == "1" and out["float_ids_code"] == "3"
    assert out["step_end"] == str(ex.GetCurrentStep())
    assert out["undersized_logits_code"] == "3"
    assert out["reset_code"] == "0" and out["step_after_reset"] == "0"
    assert out["decode_without_id_code"] == "3"


@pytest.mark.gpu
def test_executor_settings_report_the_kv_capacity_of_a_long_context_model(driver, mio, tmp_path):
    """The caller loop falls back to 4096 tokens when GetExecutorSettings is not implemented
    (runtime/core/pipeline.cc:51-62); an 8192-position model must report 8192."""
    import dataclasses
    cfg = dataclasses.replace(mio.config_tiny(), max_ctx=8192)
    img = mio.export_model_litertlm(cfg, mio.build_weights_record(cfg))
    path = tmp_path / "tiny8k.litertlm"
    path.write_bytes(img)
    out = run_driver(driver, str(path), 2, seeded_ids(0, cfg.vocab, 12))
    assert out["prefill_code"] == "0" and out["max_num_tokens"] == "8192"
