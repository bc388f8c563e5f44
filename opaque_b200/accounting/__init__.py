"""Privacy accounting: process algebra, budgets and calibration over the C++ PLD core.

Parity: packages/opaque-accounting/src/opaque/accounting/__init__.py.
"""
from . import core as composition  # noqa: F401  (``accounting.composition`` namespace)
from . import core as calibration  # noqa: F401
from . import core as discretization  # noqa: F401
from . import core as mechanisms  # noqa: F401
from . import core as amplification  # noqa: F401
from .core import (Accountant, DiscretizationConfig, DpProcess, advantage_budget, beta_budget, cached, calibrate,
                   compose, delta_budget, eps_delta, epsilon_budget, get_discretization, identity, nonprivate,
                   per_step, register_budget_serializer, repeat, risk_budget, set_discretization)

__all__ = ["Accountant", "DiscretizationConfig", "DpProcess", "advantage_budget", "amplification", "beta_budget",
           "cached", "calibrate", "calibration", "compose", "composition", "delta_budget", "discretization",
           "eps_delta", "epsilon_budget", "get_discretization", "identity", "mechanisms", "nonprivate", "per_step",
           "register_budget_serializer", "repeat", "risk_budget", "set_discretization"]
