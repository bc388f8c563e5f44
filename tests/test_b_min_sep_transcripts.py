"""Stored b-min-sep Monte-Carlo transcripts: same numbers as the streaming accountant, prefix queries, bounded registry."""
import numpy as np
import pytest

from opaque_b200.accounting.core import DiscretizationConfig, native, set_discretization
from opaque_b200.dpftrl import _transcripts as tr
from opaque_b200.dpftrl import accounting as facc
from opaque_b200.dpftrl import band_mf_strategy


@pytest.fixture(autouse=True)
def _fresh_registry():
    tr.clear()
    yield
    tr.clear()


def _cfg(samples=4000, seed=7):
    return DiscretizationConfig(num_mc_samples=samples, seed=seed)


def test_corpus_matches_streaming_accountant_and_serves_prefixes():
    cfg = _cfg().to_native()
    coef = [1.0, 0.6, 0.3]
    corpus = native.BMinSepCorpus(coef, 64, 4, 0.1, True, cfg.num_mc_samples, cfg.seed)
    assert corpus.nbytes == tr.estimate_nbytes(64, cfg.num_mc_samples)
    for nm in (0.7, 1.5):
        for n in (64, 40, 5):                        # the full horizon and two prefixes
            a = native.b_min_sep_mc_pld(coef, n, 4, 0.1, nm, True, cfg)
            b = corpus.pld(nm, n, cfg)
            assert a.epsilon_at(1e-5) == b.epsilon_at(1e-5)
            assert a.delta_at(1.0) == b.delta_at(1.0)
    with pytest.raises(ValueError):
        corpus.pld(1.0, 65, cfg)


def test_registry_reuses_extends_and_evicts(monkeypatch):
    calls = []
    real = native.BMinSepCorpus

    def counting(*a, **k):
        calls.append(a[1])
        return real(*a, **k)
    monkeypatch.setattr(tr.native, "BMinSepCorpus", counting)
    args = dict(min_sep=3, sampling_prob=0.2, warm_start=False, num_samples=500, seed=1)
    get = lambda coef, n: tr.with_corpus(coef, n, use=lambda c: c.n_steps, **args)
    assert get([1.0, 0.5], 30) == 30 and get([1.0, 0.5], 30) == 30 and get([1.0, 0.5], 12) == 30
    assert calls == [30]                                            # one draw served three queries
    assert get([1.0, 0.5], 50) == 50 and calls == [30, 50]          # a longer horizon replaces the stored corpus
    assert tr.info()["entries"] == 1
    for k in range(tr.MAX_ENTRIES):                                 # other keys push the first one out (LRU)
        get([1.0, 0.1 * (k + 1)], 10)
    assert tr.info()["entries"] == tr.MAX_ENTRIES and tr.info()["evictions"] >= 1
    monkeypatch.setenv(tr.ENV_MAX_BYTES, str(tr.estimate_nbytes(10, 500) - 1))
    assert get([2.0], 10) is None and tr.info()["too_large"] == 1   # would not fit: caller falls back to streaming


def test_process_gives_same_epsilon_with_and_without_the_registry(monkeypatch):
    strategy = band_mf_strategy(bands=3)
    with set_discretization(_cfg(samples=3000)):
        proc = facc.b_min_sep(facc.mf_gaussian(1.2, strategy, n_steps=24), bands=3, n_steps=24, sampling_prob=0.15,
                              warm_start=True)
        with_registry = proc.pld_at(24).epsilon_at(1e-5)
        assert tr.info()["entries"] == 1
        again = facc.b_min_sep(facc.mf_gaussian(0.9, strategy, n_steps=24), bands=3, n_steps=24, sampling_prob=0.15,
                               warm_start=True).pld_at(24).epsilon_at(1e-5)
        assert tr.info()["hits"] >= 1 and again > with_registry      # less noise, same transcripts: larger epsilon
        monkeypatch.setenv(tr.ENV_MAX_BYTES, "0")
        tr.clear()
        assert proc.pld_at(24).epsilon_at(1e-5) == with_registry
