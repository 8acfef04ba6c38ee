"""ctypes binding of the CPU oracle (oracle/hmc_oracle.c).

Test infrastructure only: the tests, the smoke check and the benchmark's CPU
baseline import this; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")

LIK_STUDENT_T = 0
LIK_GAUSSIAN = 1


class Model(C.Structure):
    _fields_ = [("D", C.c_int32), ("H", C.c_int32), ("likelihood", C.c_int32), ("tf32", C.c_int32),
                ("lik_scale", C.c_double), ("lik_df", C.c_double), ("prior_scale", C.c_double)]


class Sampler(C.Structure):
    _fields_ = [("leapfrog_steps", C.c_int32), ("adapt_steps", C.c_int32), ("eps0", C.c_double),
                ("target_rate", C.c_double), ("decrement", C.c_double), ("increment", C.c_double)]


def reference_model(tf32=False, H=40, D=22):
    """The reference's shipped preset (global_params.h:39-58)."""
    return Model(D, H, LIK_STUDENT_T, int(tf32), 100.0, 2.2, 200.0)


def baseline_model(tf32=False, H=40, D=22):
    """Gaussian sigma = 1 likelihood, N(0,1) prior: the benchmark preset."""
    return Model(D, H, LIK_GAUSSIAN, int(tf32), 1.0, 0.0, 1.0)


def reference_sampler(L=1000):
    return Sampler(L, 100, 0.01, 0.2, 0.1, 0.01)


def baseline_sampler(L=10, eps=1e-3):
    return Sampler(L, 0, eps, 0.2, 0.1, 0.01)


def build(force=False):
    if force or not os.path.exists(_LIB_PATH) or \
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "hmc_oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_lik_norm.restype = C.c_double
        _lib.oracle_prior_norm.restype = C.c_double
        _lib.oracle_tanh.restype = C.c_double
        _lib.oracle_tanh.argtypes = [C.c_double]
        _lib.oracle_logp_f64.restype = C.c_double
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a, t=C.c_float):
    return None if a is None else a.ctypes.data_as(C.POINTER(t))


def num_params(D, H):
    return D * H + 2 * H + 1


def logp_grad(model, X, y, w, rows=None, add_prior=True, want_losses=False):
    """-> dict(loglik, logprior, grad[P] float64, row_loss, prior_loss)."""
    X, y, w = _f32(X), _f32(y), _f32(w)
    N = X.shape[0]
    P = num_params(model.D, model.H)
    assert X.shape == (N, model.D) and y.shape[0] == N and w.shape[0] == P
    ll, lp = C.c_double(), C.c_double()
    grad = np.zeros(P, np.float64)
    row_loss = np.zeros(N, np.float32) if want_losses else None
    prior_loss = np.zeros(P, np.float32) if want_losses else None
    r0, r1 = (0, N) if rows is None else rows
    lib().oracle_logp_grad_rows(C.byref(model), C.c_int64(N), _p(X), _p(y), _p(w), C.c_int64(r0),
                                C.c_int64(r1), C.c_int(int(add_prior)), C.byref(ll), C.byref(lp),
                                _p(grad, C.c_double), _p(row_loss), _p(prior_loss))
    return dict(loglik=ll.value, logprior=lp.value, grad=grad, row_loss=row_loss,
                prior_loss=prior_loss)


def logp_f64(model, X, y, w64):
    X, y = _f32(X), _f32(y)
    w64 = np.ascontiguousarray(w64, np.float64)
    return lib().oracle_logp_f64(C.byref(model), C.c_int64(X.shape[0]), _p(X), _p(y),
                                 _p(w64, C.c_double))


def mcmc_step(model, X, y, L, eps, w_prev, mom_prev, grad_prev, want_losses=True):
    X, y = _f32(X), _f32(y)
    N = X.shape[0]
    P = num_params(model.D, model.H)
    w_next, mom_next, grad_cur = (np.zeros(P, np.float32) for _ in range(3))
    loss = np.zeros(N + P, np.float32) if want_losses else None
    ll, lp = C.c_double(), C.c_double()
    lib().oracle_mcmc_step(C.byref(model), C.c_int64(N), _p(X), _p(y), C.c_int(L), C.c_double(eps),
                           _p(_f32(w_prev)), _p(_f32(mom_prev)), _p(_f32(grad_prev)), _p(w_next),
                           _p(mom_next), _p(grad_cur), _p(loss), C.byref(ll), C.byref(lp))
    return dict(w_next=w_next, mom_next=mom_next, grad_cur=grad_cur, loss_values=loss,
                loglik=ll.value, logprior=lp.value)


def hmc_chain(model, sampler, X, y, momenta, log_u):
    X, y = _f32(X), _f32(y)
    momenta, log_u = _f32(momenta), _f32(log_u)
    n_iter = log_u.shape[0]
    N = X.shape[0]
    P = num_params(model.D, model.H)
    assert momenta.shape == (n_iter, P)
    samples = np.zeros((n_iter, P), np.float32)
    log_acpt = np.zeros(n_iter, np.float64)
    accepted = np.zeros(n_iter, np.int32)
    eps_tr = np.zeros(n_iter, np.float64)
    ll_tr = np.zeros(n_iter, np.float64)
    lp_tr = np.zeros(n_iter, np.float64)
    lib().oracle_hmc_chain(C.byref(model), C.byref(sampler), C.c_int64(N), _p(X), _p(y),
                           C.c_int(n_iter), _p(momenta), _p(log_u), _p(samples),
                           _p(log_acpt, C.c_double), _p(accepted, C.c_int32),
                           _p(eps_tr, C.c_double), _p(ll_tr, C.c_double), _p(lp_tr, C.c_double))
    return dict(samples=samples, log_acpt=log_acpt, accepted=accepted, eps=eps_tr, loglik=ll_tr,
                logprior=lp_tr)


def predict_mean(model, Xs, samples):
    Xs, samples = _f32(Xs), _f32(samples)
    n, S = Xs.shape[0], samples.shape[0]
    out = np.zeros(n, np.float64)
    lib().oracle_predict_mean(C.byref(model), C.c_int64(n), _p(Xs), C.c_int(S), _p(samples),
                              _p(out, C.c_double))
    return out


def final_loss(model, X, y, samples):
    X, y, samples = _f32(X), _f32(y), _f32(samples)
    a, b = C.c_double(), C.c_double()
    lib().oracle_final_loss(C.byref(model), C.c_int64(X.shape[0]), _p(X), _p(y),
                            C.c_int(samples.shape[0]), _p(samples), C.byref(a), C.byref(b))
    return a.value, b.value


def port_f32_chain(model, sampler, X, y, momenta, log_u, nthreads=0, want_samples=True):
    X, y = _f32(X), _f32(y)
    momenta, log_u = _f32(momenta), _f32(log_u)
    n_iter = log_u.shape[0]
    P = num_params(model.D, model.H)
    samples = np.zeros((n_iter, P), np.float32) if want_samples else None
    n_acc = lib().oracle_port_f32_chain(C.byref(model), C.byref(sampler), C.c_int64(X.shape[0]),
                                        _p(X), _p(y), C.c_int(n_iter), _p(momenta), _p(log_u),
                                        _p(samples), C.c_int(nthreads))
    return n_acc, samples


def port_f32_grad(model, X, y, w, nthreads=0):
    X, y, w = _f32(X), _f32(y), _f32(w)
    P = num_params(model.D, model.H)
    grad = np.zeros(P, np.float32)
    ll = C.c_double()
    lib().oracle_port_f32_grad(C.byref(model), C.c_int64(X.shape[0]), _p(X), _p(y), _p(w),
                               _p(grad), C.byref(ll), C.c_int(nthreads))
    return grad, ll.value


def max_threads():
    return lib().oracle_max_threads()
