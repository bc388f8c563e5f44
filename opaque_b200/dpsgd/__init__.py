"""DP-SGD: clipping, Gaussian noise, samplers and accounting front-ends.

Parity: packages/opaque-dpsgd/src/opaque/dpsgd/__init__.py.
"""
from . import clipping, noise, sampling
from .clipping import adaptive_clipped_grad, auto_clipped_grad, clipped_grad, per_group
from .noise import gaussian_noise
from .. import __version__  # noqa: F401
from .sampling import BalancedRankSampler, KOutOfTSampler, PoissonSampler, RandomAllocationSampler


def __getattr__(name):
    if name == "accounting":
        import importlib
        return importlib.import_module(".accounting", __name__)
    raise AttributeError(name)


__all__ = ["KOutOfTSampler", "PoissonSampler", "RandomAllocationSampler", "accounting", "adaptive_clipped_grad",
           "BalancedRankSampler", "auto_clipped_grad", "clipped_grad", "clipping", "gaussian_noise", "noise", "per_group", "sampling"]
