"""DP-FTRL: matrix-factorisation noise, participation-aware samplers and accounting.

Parity: packages/opaque-dpftrl/src/opaque/dpftrl/__init__.py.
"""
from ..dpsgd import clipping
from ..dpsgd.clipping import auto_clipped_grad, clipped_grad, per_group
from . import noise, sampling

import sys as _sys
_sys.modules[__name__ + ".clipping"] = clipping          # ``import opaque_b200.dpftrl.clipping`` is the DP-SGD clipping module
from .noise import (band_mf_strategy, bisr_strategy, blt_strategy, bsr_strategy, identity_strategy,
                    lambda_cgd_strategy, mf_gaussian_noise)
from .. import __version__  # noqa: F401
from .sampling import BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler, SequentialBatchSampler


def __getattr__(name):
    if name == "accounting":
        import importlib
        return importlib.import_module(".accounting", __name__)
    raise AttributeError(name)


__all__ = ["BMinSepSampler", "BallsInBinsSampler", "CyclicPoissonSampler", "SequentialBatchSampler", "accounting",
           "auto_clipped_grad", "band_mf_strategy", "bisr_strategy", "blt_strategy", "bsr_strategy", "clipped_grad",
           "clipping", "identity_strategy", "lambda_cgd_strategy", "mf_gaussian_noise", "noise", "per_group", "sampling"]
