"""Numerical parity with the UNMODIFIED reference on the CPU, when it is installed (``baseline/install_reference.sh`` puts it
into ``baseline/_ref``): same key derivation, schedules, clipped gradients, even the same noise realisation and the same
Poisson / random-allocation / balls-in-bins draws; band-MF coefficients and the correlated-noise
realisations of four matrix-factorisation strategies; the (ε, δ) and μ-GDP order-statistics audits; twelve optimizer configurations, automatic / adaptive / second-moment clipping, every
preference-loss piece, the factory collators and the shift-inside SFT losses to rounding."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref", "opaque")


@pytest.mark.skipif(not os.path.isdir(REF), reason="the reference is not installed under baseline/_ref")
def test_building_blocks_equal_the_reference():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    run = subprocess.run([sys.executable, "-W", "ignore", os.path.join(ROOT, "tests", "reference_parity_worker.py")], capture_output=True,
                         text=True, timeout=600, env=env)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-3000:]
    d = json.loads([line for line in run.stdout.splitlines() if line.startswith("{")][-1])
    assert d["rng_equal"] and d["poisson_draws_equal"] and d["random_allocation_draws_equal"] and d["balls_in_bins_draws_equal"], d
    assert d["schedules"] < 1e-9 and d["clipped_grad"] < 1e-6 and d["grad_norms"] < 1e-6, d
    assert d["noise_realisation"] < 1e-6 and d["noise_std"] > 0.01, d          # the SAME noise, and it is noise
    assert d["adamw_bc"] < 1e-6 and d["other_optimizers"] < 1e-5 and d["clipping_variants"] < 1e-6, d      # adaptive clipping: 3 steps of its state too
    # band-MF coefficients from the same objective; identity / band-MF / BSR / λ-CGD noise: the same realisation and published std
    assert d["band_mf_coefficients"] < 1e-6 and d["bsr_sensitivity"] < 1e-9, d
    assert d["mf_noise_realisation"] < 1e-5 and d["mf_noise_std"] > 0.1, d
    assert d["order_statistics_audits"] < 1e-8, d              # eps_delta() and gdp() of the estimate on the same scores
    assert d["preference_losses"] < 1e-5 and d["collators_equal"] and d["sft_losses_and_metrics"] < 1e-5, d
