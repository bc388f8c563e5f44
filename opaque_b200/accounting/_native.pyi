"""Typed surface of the C++17 privacy-accounting core (built by ``opaque_b200.utils.build.build_accounting``).

Counterpart of packages/opaque-accounting/src/opaque/api/accounting/core/opaque_accounting.pyi in the reference (a Rust
crate there).  tests/test_api_surface.py checks that every public name of the built module is declared here.
"""
from collections.abc import Sequence


class BMinSepCorpus:
    def __init__(self: BMinSepCorpus, coef: Sequence[float], n_steps: int, min_sep: int, sampling_prob: float, warm_start: bool, num_samples: int, seed: int) -> None: ...
    n_steps: object
    nbytes: object
    num_samples: object
    def pld(self: BMinSepCorpus, noise_multiplier: float, n_steps: int, config: DiscretizationConfig) -> Pld: ...
    seed: object

class DiscretizationConfig:
    def __init__(self: DiscretizationConfig, discretization: float = 0.0001, log_mass_truncation_bound: float = -50.0, max_grid_size: int = 10000000, tail_mass_truncation: float = 1e-15, max_conv_grid: int = 32768, num_mc_samples: int = 100000, seed: int = 42, proportional_normalization: bool = False) -> None: ...
    discretization: object
    log_mass_truncation_bound: object
    max_conv_grid: object
    max_grid_size: object
    num_mc_samples: object
    proportional_normalization: object
    seed: object
    tail_mass_truncation: object

class Pld:
    def advantage(self: Pld) -> float: ...
    def beta_at(self: Pld, alpha: float) -> float: ...
    def compose(self: Pld, arg0: Pld) -> Pld: ...
    def delta_at(self: Pld, epsilon: float) -> float: ...
    discretization: object
    def epsilon_at(self: Pld, delta: float) -> float: ...
    grid_size: object
    def infinity_mass(self: Pld) -> float: ...
    def is_symmetric(self: Pld) -> bool: ...
    def pmf(self: Pld, add: bool = False) -> tuple[int, float, list[float], float]: ...
    def risk_at(self: Pld, prior: float) -> float: ...
    def self_compose(self: Pld, arg0: int) -> Pld: ...

def adaclip_effective_noise_multiplier(arg0: float, arg1: float, arg2: float, arg3: int) -> float:
    """Noise multiplier left for the gradients after the quantile release of adaptive clipping."""

def b_min_sep_mc_pld(coef: Sequence[float], n_steps: int, min_sep: int, sampling_prob: float, noise_multiplier: float, warm_start: bool, config: DiscretizationConfig) -> Pld:
    """Monte-Carlo PLD of b-min-sep subsampling of a banded mechanism."""

def balls_in_bins_mc_pld(arg0: Sequence[float], arg1: int, arg2: int, arg3: float, arg4: DiscretizationConfig) -> Pld:
    """Monte-Carlo PLD of balls-in-bins participation from the b x b Gram matrix."""

def banded_sensitivity_squared(gram: Sequence[float], n: int, bands: int, min_sep: int, max_participations: int | None = None) -> float:
    """banded sensitivity squared"""

def bisr_gram_matrix(coefficients: Sequence[float], n_steps: int, min_sep: int = 1, max_participations: int | None = None, normalized: bool = True, momentum: float = 0.0) -> list[float]:
    """Balls-in-bins Gram matrix of the banded-inverse-square-root strategy."""

def bisr_gram_matrix_lr(coefficients: Sequence[float], momentum: float, n_steps: int, min_sep: int, max_participations: int | None, normalized: bool, lr_weights: Sequence[float]) -> list[float]:
    """The same with per-step learning-rate weights."""

def bisr_normalized_sensitivity_squared(coefficients: Sequence[float], n_steps: int, min_sep: int = 1, max_participations: int | None = None, momentum: float = 0.0) -> float:
    """The same, column-normalised."""

def bisr_sensitivity_squared(coefficients: Sequence[float], n_steps: int, min_sep: int = 1, max_participations: int | None = None, momentum: float = 0.0) -> float:
    """Squared sensitivity of the banded-inverse-square-root strategy."""

def bisr_strategy_coefficients(coefficients: Sequence[float], n: int) -> list[float]:
    """First n entries of column 0 of C for the banded inverse with the given taps."""

def blt_sensitivity_squared(scale: Sequence[float], decay: Sequence[float], n: int, min_sep: int = 1, max_participations: int | None = None) -> float:
    """blt sensitivity squared"""

def eps_delta_pld(arg0: float, arg1: float, arg2: DiscretizationConfig) -> Pld:
    """PLD of a generic (epsilon, delta)-DP mechanism."""

def fixed_epoch_sensitivity_squared(arg0: Sequence[float], arg1: int, arg2: int) -> float:
    """fixed epoch sensitivity squared"""

def gaussian_delta(noise_multiplier: float, epsilon: float, sensitivity: float = 1.0) -> float:
    """Exact delta(epsilon) of the Gaussian mechanism."""

def gaussian_pld(arg0: float, arg1: DiscretizationConfig) -> Pld:
    """PLD of the Gaussian mechanism at the given noise multiplier (sensitivity 1)."""

def general_sensitivity_squared_upper_bound(gram: Sequence[float], n: int, min_sep: int, max_participations: int | None = None) -> float:
    """general sensitivity squared upper bound"""

def identity_pld(arg0: DiscretizationConfig) -> Pld:
    """PLD of a mechanism that releases nothing."""

def lambda_cgd_gram_matrix(lambda_: float, n_steps: int, min_sep: int = 1, max_participations: int | None = None, normalized: bool = True, momentum: float = 0.0) -> list[float]:
    """Balls-in-bins Gram matrix of (column-normalised) DP-lambda-CGD, optional momentum filter."""

def lambda_cgd_gram_matrix_lr(lambda_: float, momentum: float, n_steps: int, min_sep: int, max_participations: int | None, normalized: bool, lr_weights: Sequence[float]) -> list[float]:
    """The same with per-step learning-rate weights."""

def lambda_cgd_max_column_norm(lambda_: float, n_steps: int) -> float:
    """sqrt((1 - lambda^(2n)) / (1 - lambda^2))."""

def lambda_cgd_normalized_sensitivity_squared(lambda_: float, n_steps: int, min_sep: int = 1, max_participations: int | None = None, momentum: float = 0.0) -> float:
    """The same for the column-normalised matrix (1 for a single participation)."""

def lambda_cgd_sensitivity_squared(lambda_: float, n_steps: int, min_sep: int = 1, max_participations: int | None = None, momentum: float = 0.0) -> float:
    """Squared sensitivity of C = (I - lambda S)^-1 under min-sep / max participations."""

def max_participation_for_linear_fn(x: Sequence[float], min_sep: int, max_participations: int | None = None) -> float:
    """max participation for linear fn"""

def mf_gaussian_pld(arg0: float, arg1: float, arg2: DiscretizationConfig) -> Pld:
    """Gaussian PLD at noise_multiplier / sensitivity (matrix-factorisation mechanisms)."""

def minsep_true_max_participations(n: int, min_sep: int, max_participations: int | None = None) -> int:
    """minsep true max participations"""

def mixture_gaussian_pld(arg0: float, arg1: Sequence[float], arg2: Sequence[float], arg3: float, arg4: float, arg5: DiscretizationConfig) -> Pld:
    """Gaussian mixture dominating pair from log-probabilities and sensitivities of the components."""

def nonprivate_pld(arg0: DiscretizationConfig) -> Pld:
    """PLD with all mass at infinite loss."""

def norm_cdf(arg0: float) -> float:
    """norm cdf"""

def norm_ppf(arg0: float) -> float:
    """norm ppf"""

def parallel_poisson_gaussian_pld(arg0: float, arg1: float, arg2: int, arg3: DiscretizationConfig) -> Pld:
    """Several workers Poisson-sample the same dataset at the same rate."""

def poisson_gaussian_pld(arg0: float, arg1: float, arg2: DiscretizationConfig) -> Pld:
    """Poisson-subsampled Gaussian (remove direction dominating pair, connect-the-dots discretisation)."""

def random_allocation_gaussian_pld(arg0: float, arg1: int, arg2: int, arg3: DiscretizationConfig) -> Pld:
    """Each record takes part in k of t steps chosen uniformly (k = 1: random allocation)."""

def single_participation_sensitivity_squared(arg0: Sequence[float], arg1: int) -> float:
    """single participation sensitivity squared"""

def toeplitz_bnb_gram_matrix(strategy_coef: Sequence[float], n_steps: int, min_sep: int = 1, max_participations: int | None = None, normalized: bool = True) -> list[float]:
    """Balls-in-bins Gram matrix of a Toeplitz strategy with known forward coefficients."""

def toeplitz_gram_matrix(arg0: Sequence[float], arg1: int) -> list[float]:
    """Dense n x n Gram matrix C^T C (row-major) of a Toeplitz strategy."""

def toeplitz_minsep_sensitivity_squared(coef: Sequence[float], n: int, min_sep: int, max_participations: int | None = None) -> float:
    """toeplitz minsep sensitivity squared"""

def truncated_poisson_gaussian_pld(arg0: float, arg1: float, arg2: int, arg3: int, arg4: DiscretizationConfig) -> Pld:
    """Poisson-subsampled Gaussian with a hard cap on the batch size over a dataset of the given size."""

