"""Pins the CPU oracle (and the CUDA path) against the reference's own FP32
kernel, built unmodified from the reference's headers (oracle/ref_harness.cu)
and run here on the GPU, at the shapes the reference fixes at compile time
(58368 rows, 22 -> 40 -> 1, Student-t(100, 2.2), N(0, 200^2) prior).

Also writes the captured reference outputs into $MCMC_B200_GOLDEN_OUT (pytest's
temporary directory when unset) so that they can be committed under
tests/golden/ for the CPU-only suite."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_ffma.so")
N, P = 58368, 961


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _ref_step(ref, x, y, L, eps, w, mom, g):
    wn, mn, gc = (np.zeros(P, np.float32) for _ in range(3))
    loss = np.zeros(N + P, np.float32)
    rc = ref.ref_ffma_mcmc_step(_fp(x), _fp(y), L, C.c_float(eps), _fp(w), _fp(mom), _fp(g), _fp(wn),
                                _fp(mn), _fp(gc), _fp(loss))
    assert rc == 0
    return dict(w_next=wn, mom_next=mn, grad_cur=gc, loss_values=loss)


def test_oracle_and_cuda_path_against_reference_kernel(built, tmp_path):
    if not os.path.exists(REF_LIB):
        pytest.skip("reference harness not built (needs the reference tree at build time)")
    m, O = built
    ref = C.CDLL(REF_LIB)
    assert ref.ref_n_samples() == N and ref.ref_n_params() == P
    x, y, _ = m.synth_window(2024, 0, N)
    x = (x * np.float32(0.05)).astype(np.float32)
    rng = np.random.default_rng(1)
    w = (0.3 * rng.standard_normal(P)).astype(np.float32)
    mom = rng.standard_normal(P).astype(np.float32)
    zeros = np.zeros(P, np.float32)
    model = O.reference_model()

    # (1) the loss-only idiom: mcmc_step<T,1>, eps = 0 (main.h:85-99)
    r1 = _ref_step(ref, x, y, 1, 0.0, w, zeros, zeros)
    o1 = O.logp_grad(model, x, y, w, want_losses=True)
    gscale = np.abs(o1["grad"]).max()
    assert np.abs(r1["grad_cur"] - o1["grad"]).max() < 1e-5 * gscale
    assert np.allclose(r1["loss_values"][:N], o1["row_loss"], rtol=1e-5, atol=1e-5)
    assert np.allclose(r1["loss_values"][N:], o1["prior_loss"], rtol=1e-6)
    assert np.array_equal(r1["w_next"], w)

    # (2) ten leapfrog steps: mcmc_step<T,10>
    eps = 0.02  # stable for 58368 rows: the trajectory does not amplify rounding differences
    g0 = o1["grad"].astype(np.float32)
    r10 = _ref_step(ref, x, y, 10, eps, w, mom, g0)
    o10 = O.mcmc_step(model, x, y, 10, eps, w, mom, g0)
    assert np.abs(r10["w_next"] - o10["w_next"]).max() < 1e-5 * np.abs(o10["w_next"]).max()
    assert np.abs(r10["mom_next"] - o10["mom_next"]).max() < 1e-5 * np.abs(o10["mom_next"]).max()
    assert np.abs(r10["grad_cur"] - o10["grad_cur"]).max() < 1e-5 * np.abs(o10["grad_cur"]).max()
    assert np.allclose(r10["loss_values"], o10["loss_values"], rtol=1e-5, atol=1e-5)

    # (3) accept ratio: log_acpt_prec (kernel_helpers.h:153-188)
    out = C.c_float()
    prev = np.concatenate([o1["row_loss"], o1["prior_loss"]]).astype(np.float32)
    rc = ref.ref_log_acpt(_fp(prev), _fp(r10["loss_values"]), _fp(mom), _fp(r10["mom_next"]),
                          _fp(r10["grad_cur"]), C.c_float(eps), C.byref(out))
    assert rc == 0
    mf = o10["mom_next"].astype(np.float64) + 0.5 * np.float32(eps) * o10["grad_cur"].astype(np.float64)
    exp = float(np.sum(o10["loss_values"].astype(np.float64) - prev.astype(np.float64)) +
                0.5 * (np.sum(mom.astype(np.float64) ** 2) - np.sum(mf ** 2)))
    assert abs(out.value - exp) < 2e-2 + 1e-4 * abs(exp)

    # (4) this library against the reference kernel directly
    ctx = m.Context(m.reference_config(leapfrog_steps=10), n_windows=1, rows=N)
    ctx.set_window_data(0, x, y)
    mine = ctx.potential_and_grad(0, w, want_row_loss=True)
    assert np.abs(mine["grad"] - r1["grad_cur"]).max() < 1e-5 * gscale
    assert np.allclose(mine["row_loss"], r1["loss_values"][:N], rtol=1e-5, atol=1e-5)
    lf = ctx.leapfrog(0, 10, eps, w, mom, g0)
    assert np.abs(lf["w_next"] - r10["w_next"]).max() < 1e-5 * np.abs(r10["w_next"]).max()
    assert np.abs(lf["mom_next"] - r10["mom_next"]).max() < 1e-5 * np.abs(r10["mom_next"]).max()
    assert np.abs(lf["grad_cur"] - r10["grad_cur"]).max() < 1e-5 * np.abs(r10["grad_cur"]).max()
    ctx.close()

    # capture for the CPU-only suite: inputs are regenerated from the seed there,
    # so only small vectors and checksums are stored
    out_dir = os.environ.get("MCMC_B200_GOLDEN_OUT") or str(tmp_path)
    os.makedirs(out_dir, exist_ok=True)
    np.savez_compressed(
        os.path.join(out_dir, "reference_ffma_b200.npz"),
        seed=2024, x_scale=0.05, eps=eps, w=w, mom=mom,
        x_checksum=np.float64(x.astype(np.float64).sum()), y_checksum=np.float64(y.astype(np.float64).sum()),
        eval_grad=r1["grad_cur"], eval_loglik=np.float64(r1["loss_values"][:N].astype(np.float64).sum()),
        eval_logprior=np.float64(r1["loss_values"][N:].astype(np.float64).sum()),
        eval_row_loss_head=r1["loss_values"][:256],
        step10_w=r10["w_next"], step10_mom=r10["mom_next"], step10_grad=r10["grad_cur"],
        step10_loglik=np.float64(r10["loss_values"][:N].astype(np.float64).sum()),
        log_acpt=np.float32(out.value))
