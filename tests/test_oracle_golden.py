"""The CPU oracle against outputs of the reference's own FP32 kernels captured on
a B200 (tests/golden/README.md says how).  This is what pins the oracle: the
reference has no tests, vectors or CPU code of its own."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_ffma_b200.npz")
N, P = 58368, 961


@pytest.fixture(scope="module")
def case(built):
    m, O = built
    g = np.load(GOLD)
    x, y, _ = m.synth_window(int(g["seed"]), 0, N)
    x = (x * np.float32(float(g["x_scale"]))).astype(np.float32)
    # the regenerated inputs are the ones the reference kernel saw
    assert abs(x.astype(np.float64).sum() - float(g["x_checksum"])) < 1e-6 * max(1.0, abs(float(g["x_checksum"])))
    assert abs(y.astype(np.float64).sum() - float(g["y_checksum"])) < 1e-6 * abs(float(g["y_checksum"]))
    return O, g, x, y


def test_loss_only_call_matches_reference_kernel(case):
    O, g, x, y = case
    r = O.logp_grad(O.reference_model(), x, y, g["w"], want_losses=True)
    assert np.abs(r["grad"] - g["eval_grad"]).max() < 1e-5 * np.abs(g["eval_grad"]).max()
    assert abs(r["loglik"] - float(g["eval_loglik"])) < 1e-6 * abs(float(g["eval_loglik"]))
    assert abs(r["logprior"] - float(g["eval_logprior"])) < 1e-6 * abs(float(g["eval_logprior"]))
    assert np.allclose(r["row_loss"][:256], g["eval_row_loss_head"], rtol=1e-5, atol=1e-5)


def test_ten_leapfrog_steps_and_accept_ratio_match_reference_kernel(case):
    O, g, x, y = case
    model = O.reference_model()
    eps = float(g["eps"])
    r0 = O.logp_grad(model, x, y, g["w"], want_losses=True)
    r = O.mcmc_step(model, x, y, 10, eps, g["w"], g["mom"], g["eval_grad"])
    for key, ref in (("w_next", "step10_w"), ("mom_next", "step10_mom"), ("grad_cur", "step10_grad")):
        assert np.abs(r[key] - g[ref]).max() < 1e-5 * np.abs(g[ref]).max(), key
    assert abs(r["loglik"] - float(g["step10_loglik"])) < 1e-6 * abs(float(g["step10_loglik"]))
    # kernel_helpers.h:163-175
    prev = np.concatenate([r0["row_loss"], r0["prior_loss"]]).astype(np.float64)
    mf = r["mom_next"].astype(np.float64) + 0.5 * np.float32(eps) * r["grad_cur"].astype(np.float64)
    la = float(np.sum(r["loss_values"].astype(np.float64) - prev) +
               0.5 * (np.sum(g["mom"].astype(np.float64) ** 2) - np.sum(mf ** 2)))
    assert abs(la - float(g["log_acpt"])) < 2e-2  # the reference sums 60290 FP32 terms in FP32
