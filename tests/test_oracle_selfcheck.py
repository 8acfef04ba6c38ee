"""The oracle against facts that can be checked without any GPU: the reference's
hard-coded constants, finite differences, hand-computable cases, the leapfrog
and accept semantics of the reference driver, and row-shard additivity."""
import math

import numpy as np
import pytest

import oracle as O

D, H, P = 22, 40, 961


def _data(n, seed=0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, D)).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    w = (0.2 * rng.standard_normal(P)).astype(np.float32)
    return x, y, w


def test_constants_match_reference():
    # include/mcmc/global_params.h:45,52 hard-code these two normalisers
    m = O.reference_model()
    assert abs(O.lib().oracle_lik_norm(O.C.byref(m)) - 5.63448313353184) < 1e-12
    assert abs(O.lib().oracle_prior_norm(O.C.byref(m)) - 6.21725589975271) < 1e-12
    assert O.num_params(22, 40) == 961 and O.num_params(22, 128) == 3073


def test_tanh_identity_branch():
    # include/mcmc/kernel_helpers.h:43: |x| below the cut-off returns x itself
    cut = float(np.float32(0.0048176045529544353485))
    t = O.lib().oracle_tanh
    assert t(cut * 0.999) == cut * 0.999
    assert t(-cut * 0.5) == -cut * 0.5
    assert abs(t(cut * 1.001) - math.tanh(cut * 1.001)) < 1e-15
    assert abs(t(1.3) - math.tanh(1.3)) < 1e-15


@pytest.mark.parametrize("model", [O.reference_model(), O.baseline_model()])
def test_gradient_matches_finite_differences(model):
    x, y, w = _data(300, 1)
    r = O.logp_grad(model, x, y, w)
    rng = np.random.default_rng(2)
    w64 = w.astype(np.float64)
    scale = np.abs(r["grad"]).max()
    for p in rng.choice(P, 40, replace=False):
        h = 1e-4
        wp, wm = w64.copy(), w64.copy()
        wp[p] += h
        wm[p] -= h
        fd = (O.logp_f64(model, x, y, wp) - O.logp_f64(model, x, y, wm)) / (2 * h)
        assert abs(fd - r["grad"][p]) <= 2e-6 * scale + 1e-6 * abs(fd)
    assert abs(O.logp_f64(model, x, y, w64) - (r["loglik"] + r["logprior"])) < 1e-6 * abs(r["loglik"])


@pytest.mark.parametrize("tf32", [False, True])
def test_wide_model_gradient_matches_finite_differences(tf32):
    """22 -> 128 -> 1 (3073 parameters, the scaled stress configuration): the oracle's gradient against
    central differences of its own double-precision log density; the TF32 mode within its tolerance."""
    Hw = 128
    Pw = O.num_params(D, Hw)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((200, D)).astype(np.float32)
    y = rng.standard_normal(200).astype(np.float32)
    w = (0.1 * rng.standard_normal(Pw)).astype(np.float32)
    exact = O.baseline_model(H=Hw)
    r = O.logp_grad(O.baseline_model(tf32=tf32, H=Hw), x, y, w)
    w64 = w.astype(np.float64)
    scale = np.abs(r["grad"]).max()
    tol = 2e-3 if tf32 else 2e-6
    for p in rng.choice(Pw, 30, replace=False):
        h = 1e-4
        wp, wm = w64.copy(), w64.copy()
        wp[p] += h
        wm[p] -= h
        fd = (O.logp_f64(exact, x, y, wp) - O.logp_f64(exact, x, y, wm)) / (2 * h)
        assert abs(fd - r["grad"][p]) <= tol * scale + 1e-6 * abs(fd)


def test_zero_weights_only_output_bias_gets_likelihood_gradient():
    # tanh(0) = 0 and W1 = 0: every likelihood gradient vanishes except db1 = sum dL/dpred
    x, y, _ = _data(64, 3)
    m = O.baseline_model()
    r = O.logp_grad(m, x, y, np.zeros(P, np.float32), add_prior=False)
    assert np.all(r["grad"][:P - 1] == 0)
    assert abs(r["grad"][P - 1] - float(np.sum(y.astype(np.float64)))) < 1e-9
    assert abs(r["loglik"] - float(np.sum(-0.5 * y.astype(np.float64) ** 2 - 0.5 * math.log(2 * math.pi)))) < 1e-9


def test_single_row_single_case_by_hand():
    m = O.baseline_model()
    x = np.zeros((1, D), np.float32)
    x[0, 0] = 2.0
    y = np.array([1.0], np.float32)
    w = np.zeros(P, np.float32)
    w[0] = 0.5          # W0[0][0]
    w[D * H] = 0.25     # b0[0]
    w[D * H + H] = 2.0  # W1[0]
    w[P - 1] = -0.5     # b1
    h = math.tanh(2.0 * 0.5 + 0.25)
    pred = -0.5 + 2.0 * h
    dy = 1.0 - pred
    r = O.logp_grad(m, x, y, w, add_prior=False)
    assert abs(r["grad"][P - 1] - dy) < 1e-12
    assert abs(r["grad"][D * H + H] - dy * h) < 1e-12
    dz = (1 - h * h) * 2.0 * dy
    assert abs(r["grad"][D * H] - dz) < 1e-12
    assert abs(r["grad"][0] - 2.0 * dz) < 1e-12


def test_row_shards_add_up():
    x, y, w = _data(1000, 4)
    m = O.reference_model()
    full = O.logp_grad(m, x, y, w)
    a = O.logp_grad(m, x, y, w, rows=(0, 400), add_prior=False)
    b = O.logp_grad(m, x, y, w, rows=(400, 1000), add_prior=True)
    assert np.allclose(a["grad"] + b["grad"], full["grad"], rtol=1e-12, atol=1e-12)
    assert abs(a["loglik"] + b["loglik"] - full["loglik"]) < 1e-9


def test_mcmc_step_first_kick_is_half_and_eps0_is_pure_evaluation():
    x, y, w = _data(200, 5)
    m = O.baseline_model()
    g0 = O.logp_grad(m, x, y, w)["grad"].astype(np.float32)
    mom = np.random.default_rng(6).standard_normal(P).astype(np.float32)
    # eps = 0: the reference's loss-only idiom (main.h:85-99)
    r = O.mcmc_step(m, x, y, 1, 0.0, w, np.zeros(P, np.float32), np.zeros(P, np.float32))
    assert np.array_equal(r["w_next"], w)
    assert np.allclose(r["grad_cur"], g0, rtol=1e-6)
    assert abs(float(np.sum(r["loss_values"][:200].astype(np.float64))) - r["loglik"]) < 1e-3
    # one step: m1 = m0 + eps/2 g0 ; w1 = w0 + eps m1 (mcmc_step_ffma.h:106-120, MOM_CORRECTION = 2)
    eps = 1e-2
    r = O.mcmc_step(m, x, y, 1, eps, w, mom, g0)
    m1 = mom.astype(np.float64) + np.float32(eps) * g0.astype(np.float64) / 2
    assert np.allclose(r["mom_next"], m1, rtol=1e-6, atol=1e-7)
    assert np.allclose(r["w_next"], w + np.float32(eps) * m1, rtol=1e-6, atol=1e-7)
    # two steps: the second kick is a full kick with the gradient at w1
    r2 = O.mcmc_step(m, x, y, 2, eps, w, mom, g0)
    m2 = r["mom_next"].astype(np.float64) + np.float32(eps) * r["grad_cur"].astype(np.float64)
    assert np.allclose(r2["mom_next"], m2, rtol=1e-6, atol=1e-7)


def test_chain_accept_reject_and_adaptation():
    x, y, _ = _data(256, 7)
    m = O.baseline_model()
    n_iter = 6
    rng = np.random.default_rng(8)
    mom = rng.standard_normal((n_iter, P)).astype(np.float32)
    s = O.Sampler(3, 4, 1e-3, 0.2, 0.1, 0.01)
    # log u = -inf-ish accepts everything, +large rejects everything
    acc = O.hmc_chain(m, s, x, y, mom, np.full(n_iter, -1e30, np.float32))
    rej = O.hmc_chain(m, s, x, y, mom, np.full(n_iter, 1e30, np.float32))
    assert acc["accepted"].all() and not rej["accepted"].any()
    assert np.all(rej["samples"] == 0)  # the chain starts at w = 0 (main.h:52) and never moves
    # main.h:266-276: eps grows by 1% per adapted iteration while the ratio is above target
    assert np.allclose(acc["eps"][:5], 1e-3 * 1.01 ** np.arange(5), rtol=1e-6)
    assert acc["eps"][5] == acc["eps"][4]  # adaptation stops after adapt_steps = 4 iterations
    # rejected: ratio vs target decides shrink factor 1 - 0.1/1.1
    la = rej["log_acpt"]
    exp = [1e-3]
    for i in range(4):
        exp.append(exp[-1] * ((1 - 0.1 / 1.1) if min(la[i], 0) < math.log(0.2) else 1.01))
    assert np.allclose(rej["eps"][:5], exp, rtol=1e-6)
    # Hamiltonian bookkeeping: the accept ratio equals the energy difference recomputed by hand
    it = 0
    m0 = mom[it]
    st = O.mcmc_step(m, x, y, 3, 1e-3, np.zeros(P, np.float32), m0,
                     O.logp_grad(m, x, y, np.zeros(P, np.float32))["grad"].astype(np.float32))
    boot = O.logp_grad(m, x, y, np.zeros(P, np.float32))
    mf = st["mom_next"].astype(np.float64) + 0.5 * np.float32(1e-3) * st["grad_cur"].astype(np.float64)
    by_hand = (st["loglik"] + st["logprior"]) - (boot["loglik"] + boot["logprior"]) + \
        0.5 * (np.sum(m0.astype(np.float64) ** 2) - np.sum(mf ** 2))
    assert abs(by_hand - acc["log_acpt"][0]) < 5e-3  # per-row FP32 rounding of the loss vector


def test_f32_port_tracks_double_oracle():
    x, y, w = _data(2048, 9)
    m = O.reference_model()
    g, ll = O.port_f32_grad(m, x, y, w, nthreads=2)
    r = O.logp_grad(m, x, y, w)
    assert np.abs(g - r["grad"]).max() < 1e-4 * np.abs(r["grad"]).max()
    assert abs(ll - r["loglik"]) < 1e-5 * abs(r["loglik"])
    n_iter = 5
    rng = np.random.default_rng(10)
    mom = rng.standard_normal((n_iter, P)).astype(np.float32)
    lu = np.log(rng.uniform(size=n_iter)).astype(np.float32)
    mb = O.baseline_model()
    s = O.baseline_sampler(L=4)
    n_acc, samples = O.port_f32_chain(mb, s, x, y, mom, lu, nthreads=2)
    ref = O.hmc_chain(mb, s, x, y, mom, lu)
    assert n_acc == int(ref["accepted"].sum())
    assert np.allclose(samples, ref["samples"], rtol=1e-3, atol=1e-5)


def test_tf32_mode_truncates_but_stays_close():
    x, y, w = _data(512, 11)
    a = O.logp_grad(O.baseline_model(tf32=False), x, y, w)
    b = O.logp_grad(O.baseline_model(tf32=True), x, y, w)
    rel = np.abs(a["grad"] - b["grad"]).max() / np.abs(a["grad"]).max()
    assert 0 < rel < 2e-3


def test_predict_mean_and_final_loss():
    x, y, _ = _data(100, 12)
    rng = np.random.default_rng(13)
    S = rng.standard_normal((5, P)).astype(np.float32) * 0.1
    m = O.baseline_model()
    pm = O.predict_mean(m, x, S)
    one = np.stack([O.predict_mean(m, x, S[i:i + 1]) for i in range(5)]).mean(0)
    assert np.allclose(pm, one, rtol=1e-12)
    ll, lp = O.final_loss(m, x, y, S)
    each = [O.logp_grad(m, x, y, S[i]) for i in range(5)]
    assert abs(ll - np.mean([e["loglik"] for e in each])) < 1e-9
    assert abs(lp - np.mean([e["logprior"] for e in each])) < 1e-9
