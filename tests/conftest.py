import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    graft.build()
    return graft.load_package()


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def mio(pkg):
    return pkg.model_io


_MODEL_CACHE = {}


@pytest.fixture(scope="session")
def models(mio):
    """name -> (config, weights record bytes, .litertlm image bytes), built once per session."""
    def get(name):
        if name not in _MODEL_CACHE:
            cfg = mio.CONFIGS[name]()
            rec = mio.build_weights_record(cfg)
            _MODEL_CACHE[name] = (cfg, rec, mio.export_model_litertlm(cfg, rec))
        return _MODEL_CACHE[name]
    return get


def seeded_ids(seed, vocab, n):
    return np.random.Generator(np.random.PCG64(seed)).integers(0, vocab, n).astype(np.int32)


def logits_close(got, want):
    """The parity bar: cosine >= 0.999 and max-abs error <= 2e-2 of the logit range."""
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    cos = float(np.dot(got, want) / (np.linalg.norm(got) * np.linalg.norm(want) + 1e-300))
    err = float(np.abs(got - want).max() / (want.max() - want.min() + 1e-300))
    return cos, err
