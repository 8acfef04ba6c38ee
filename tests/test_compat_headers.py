"""include/mcmc/*.h keep the reference's spellings (mcmc::mcmc_step, Network,
DeviceMatrix, log_acpt_prec, main_loop) over the C-ABI: a program written like
the reference's main.cu must build against them (CPU check) and give the
oracle's numbers (GPU check)."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "_build", "compat_main")


def _build(m):
    src = os.path.join(ROOT, "tests", "compat_main.cu")
    deps = [src, m.LIB_PATH] + [os.path.join(ROOT, "include", "mcmc", f) for f in
                                ("main.h", "utils_matrix.h", "global_params.h", "io.h")]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) >= os.path.getmtime(d) for d in deps):
        return
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    subprocess.check_call([
        "nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + os.path.join(ROOT, "include"),
        "-o", EXE, src, "-L" + os.path.dirname(m.LIB_PATH), "-lmcmc_b200",
        "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../mcmc_bnn_example_b200"])


def test_reference_style_program_builds_against_compat_headers(built):
    m, _ = built
    _build(m)
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_reference_style_program_matches_oracle(built):
    m, O = built
    if not os.path.exists(EXE):
        _build(m)
    out = subprocess.run([EXE], check=True, capture_output=True, text=True).stdout.splitlines()
    la = float(out[0].split()[1])
    assert float(out[1].split()[1]) == 0.0  # grad_next is left zeroed
    vals = np.array([[float(t) for t in ln.split()[2:4]] for ln in out[2:]])
    assert vals.shape == (961, 2)
    N, P = 58368, 961
    x, y, _ = m.synth_window(5, 0, N)
    x = (x * np.float32(0.05)).astype(np.float32)
    model = O.reference_model()
    zero = np.zeros(P, np.float32)
    boot = O.logp_grad(model, x, y, zero, want_losses=True)
    mom = np.array([0.5 * ((i * 37) % 11 - 5) / 5.0 for i in range(P)], np.float32)
    ref = O.mcmc_step(model, x, y, 10, 0.02, zero, mom, boot["grad"].astype(np.float32))
    assert np.abs(vals[:, 0] - ref["w_next"]).max() < 1e-5 * np.abs(ref["w_next"]).max()
    assert np.abs(vals[:, 1] - ref["grad_cur"]).max() < 1e-5 * np.abs(ref["grad_cur"]).max()
    prev = np.concatenate([boot["row_loss"], boot["prior_loss"]]).astype(np.float64)
    mf = ref["mom_next"].astype(np.float64) + 0.5 * np.float32(0.02) * ref["grad_cur"].astype(np.float64)
    exp = float(np.sum(ref["loss_values"].astype(np.float64) - prev) +
                0.5 * (np.sum(mom.astype(np.float64) ** 2) - np.sum(mf ** 2)))
    assert abs(la - exp) < 2e-2 + 1e-4 * abs(exp)


SHORT = dict(MCMC_LEAPFROG_STEPS=10, MCMC_BURN_IN_STEPS=8, MCMC_SAMPLE_STEPS=12, MCMC_N_SAMPLES=8192)
EXE_SHORT = os.path.join(ROOT, "tests", "_build", "compat_main_short")


def _build_short(m):
    """The same program with the header's chain lengths given on the compiler command line."""
    src = os.path.join(ROOT, "tests", "compat_main.cu")
    deps = [src, m.LIB_PATH, __file__] + [os.path.join(ROOT, "include", "mcmc", f) for f in
                                          ("main.h", "utils_matrix.h", "global_params.h", "io.h")]
    if os.path.exists(EXE_SHORT) and all(os.path.getmtime(EXE_SHORT) >= os.path.getmtime(d) for d in deps):
        return
    os.makedirs(os.path.dirname(EXE_SHORT), exist_ok=True)
    subprocess.check_call([
        "nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + os.path.join(ROOT, "include"),
        *["-D%s=%d" % kv for kv in SHORT.items()],
        "-o", EXE_SHORT, src, "-L" + os.path.dirname(m.LIB_PATH), "-lmcmc_b200",
        "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../mcmc_bnn_example_b200"])


def test_short_main_loop_program_builds(built):
    m, _ = built
    _build_short(m)
    assert os.path.exists(EXE_SHORT)


@pytest.mark.gpu
def test_main_loop_runs_reference_preset_end_to_end(built, tmp_path):
    """mcmc::main_loop<float>() (the reference's one executable path, main.cu:28-31 -> main.h:117-308) with
    the reference's model and sampler constants, shortened on the compiler command line to 8 + 12
    iterations of 10 leapfrog steps on 8192 rows so that the CPU oracle can replay it: the accept
    count, the final step size and the mean losses over the kept samples must be the oracle's."""
    import re
    m, O = built
    _build_short(m)
    out = subprocess.run([EXE_SHORT, "main_loop"], check=True, capture_output=True, text=True,
                         cwd=str(tmp_path)).stdout
    acc, n_it, eps_final = re.search(r"accepted (\d+) of (\d+), final step size (\S+)", out).groups()
    ll, lp, full = (float(v) for v in re.search(r"Final loss1: (\S+), loss2: (\S+), full loss: (\S+)", out).groups())
    L, burn, keep, N = (SHORT[k] for k in ("MCMC_LEAPFROG_STEPS", "MCMC_BURN_IN_STEPS", "MCMC_SAMPLE_STEPS",
                                            "MCMC_N_SAMPLES"))
    n_iter = burn + keep
    assert int(n_it) == n_iter
    # the program's inputs and draws, recomputed on the host: synthetic window (seed 0, window 0) scaled by
    # 0.001, Philox momenta and accept uniforms keyed by (SEED_INIT = 0, window 0, iteration)
    x, y, _ = m.synth_window(0, 0, N)
    x = (x * np.float32(0.001)).astype(np.float32)
    P = 961
    mom = np.array([[m.lib().mcmc_b200_philox_normal(0, 0, it, 0, p) for p in range(P)] for it in range(n_iter)],
                   np.float32)
    log_u = np.empty(n_iter, np.float32)
    for it in range(n_iter):
        r = m.philox_raw([0, it, 0, 1], [0, 0])
        log_u[it] = np.log(np.float32((np.float32(r[0] >> 8) + np.float32(1.0)) * np.float32(1.0 / 16777216.0)),
                           dtype=np.float32)
    ref = O.hmc_chain(O.reference_model(), O.Sampler(L, burn, 0.01, 0.2, 0.1, 0.01), x, y, mom, log_u)
    assert int(acc) == int(ref["accepted"].sum())
    eps_next = ref["eps"][-1]  # the adaptation has ended by the last iteration: the step size no longer moves
    assert abs(float(eps_final) - eps_next) <= 1e-5 * eps_next
    ell, elp = O.final_loss(O.reference_model(), x, y, ref["samples"][burn:])
    assert abs(ll - ell) <= 1e-5 * abs(ell) and abs(lp - elp) <= 1e-5 * abs(elp)
    assert abs(full - (ell + elp)) <= 1e-5 * abs(ell + elp)
