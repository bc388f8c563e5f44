"""Privacy accounting: process algebra, budgets and calibration over the C++ PLD core.

Parity: packages/opaque-accounting/src/opaque/accounting/__init__.py.
"""
from . import core as composition  # noqa: F401  (``accounting.composition`` namespace)
from . import core as calibration  # noqa: F401
from . import core as discretization  # noqa: F401
from . import core as mechanisms  # noqa: F401
from . import core as amplification  # noqa: F401
from .. import __version__  # noqa: F401
from .core import (Accountant, DiscretizationConfig, DpProcess, advantage_budget, beta_budget, cached, calibrate,
                   compose, delta_budget, eps_delta, epsilon_budget, get_discretization, identity, nonprivate,
                   per_step, register_budget_serializer, repeat, risk_budget, set_discretization)

__all__ = ["Accountant", "DiscretizationConfig", "DpProcess", "advantage_budget", "amplification", "beta_budget",
           "cached", "calibrate", "calibration", "compose", "composition", "delta_budget", "discretization",
           "eps_delta", "epsilon_budget", "get_discretization", "identity", "mechanisms", "nonprivate", "per_step",
           "register_budget_serializer", "repeat", "risk_budget", "set_discretization"]

from . import core as _core  # noqa: E402
from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "types", "Classes of the accounting façade.", {n: getattr(_core, n) for n in (
    "Accountant AdvantageBudget BetaBudget Budget CachedProcess CalibrateResult Composed DeltaBudget DiscretizationConfig "
    "DpHorizonProcess DpProcess EpsDelta EpsilonBudget Identity NonPrivate PerStep Repeated RiskBudget").split()}, bind=False)
