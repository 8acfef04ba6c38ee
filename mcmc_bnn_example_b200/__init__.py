"""B200-native HMC hot path of NVIDIA/mcmc-bnn-example.

The product is the C-ABI shared library built from ``csrc/`` (declared in
``include/mcmc_b200.h``); this package is a thin ctypes mirror of it, shaped
after the reference's driver (``include/mcmc/main.h``): a :class:`Context`
holds what ``main_loop`` allocates, ``run_chain`` is its sampling loop,
``mcmc_step`` / ``log_acpt`` are the drop-ins for ``mcmc::mcmc_step`` and
``mcmc::log_acpt_prec``.

There is no CPU fallback: without the built library, or without a B200, every
compute call raises.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "libmcmc_b200.so")
_SOURCES = ["api.cu", "chain.cu", "grad_fp32.cu", "grad_tf32.cu", "grad_tf32_wide.cu", "synth.cu", "noalloc.cu", "io.cu",
            "microbench.cu", "forward.cu"]
_HEADERS = ["common.cuh", "chain.cuh", "philox.h", "tc05.cuh"]

OK = 0
LIK_STUDENT_T, LIK_GAUSSIAN = 0, 1
PREC_FP32, PREC_TF32 = 0, 1
RNG_PHILOX, RNG_REFERENCE = 0, 1

EXPORTS = [
    "mcmc_b200_config_reference", "mcmc_b200_config_baseline", "mcmc_b200_last_error",
    "mcmc_b200_has_tf32", "mcmc_b200_create", "mcmc_b200_destroy", "mcmc_b200_num_params",
    "mcmc_b200_set_window_data", "mcmc_b200_potential_and_grad", "mcmc_b200_leapfrog",
    "mcmc_b200_run_chain", "mcmc_b200_run_chain_async", "mcmc_b200_synchronize", "mcmc_b200_stream",
    "mcmc_b200_reset_chain", "mcmc_b200_chain_info", "mcmc_b200_get_state", "mcmc_b200_get_samples",
    "mcmc_b200_get_trace", "mcmc_b200_predict_mean", "mcmc_b200_final_loss",
    "mcmc_b200_nccl_unique_id", "mcmc_b200_enable_row_sharding", "mcmc_b200_mcmc_step",
    "mcmc_b200_log_acpt", "mcmc_b200_synth_window", "mcmc_b200_philox_normal", "mcmc_b200_philox_raw",
    "mcmc_b200_launch_count", "mcmc_b200_chain_geometry", "mcmc_b200_potential_and_grad_static",
    "mcmc_b200_checkpoint_size", "mcmc_b200_checkpoint_save", "mcmc_b200_checkpoint_load",
    "mcmc_b200_read_table", "mcmc_b200_plan_work_table", "mcmc_b200_rebind_data",
    "mcmc_b200_selftest_wait_timeout", "mcmc_b200_philox_device", "mcmc_b200_refstream_momentum_device",
    "mcmc_b200_refstream_engine", "mcmc_b200_refstream_engine0", "mcmc_b200_refstream_log_uniform",
    "mcmc_b200_microbench_l2_read", "mcmc_b200_microbench_mufu", "mcmc_b200_enable_oneshot_allreduce",
    "mcmc_b200_time_allreduce", "mcmc_b200_selftest_oneshot_timeout",
]


class Config(C.Structure):
    """Mirror of ``mcmc_b200_config`` (the reference's global_params.h:27-58)."""
    _fields_ = [("D", C.c_int32), ("H", C.c_int32), ("likelihood", C.c_int32), ("precision", C.c_int32),
                ("lik_scale", C.c_double), ("lik_df", C.c_double), ("prior_scale", C.c_double),
                ("leapfrog_steps", C.c_int32), ("burn_in", C.c_int32), ("adapt_steps", C.c_int32),
                ("sample_capacity", C.c_int32), ("eps0", C.c_double), ("target_rate", C.c_double),
                ("decrement", C.c_double), ("increment", C.c_double), ("seed", C.c_uint64),
                ("trace_iters", C.c_int32), ("slices", C.c_int32), ("rng_streams", C.c_int32)]


class McmcError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"mcmc_b200 error {code}: {msg}")
        self.code = code


def build(force=False, verbose=False):
    """Compile csrc/*.cu for sm_100a into libmcmc_b200.so (nvcc cross-compiles without a GPU)."""
    src = [os.path.join(_HERE, "csrc", s) for s in _SOURCES]
    deps = src + [os.path.join(_HERE, "csrc", h) for h in _HEADERS] + \
        [os.path.join(_ROOT, "include", "mcmc_b200.h")]
    if not force and os.path.exists(LIB_PATH) and \
            all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(d) for d in deps):
        return LIB_PATH
    cmd = ["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo",
           "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", "-cudart", "static",
           "-o", LIB_PATH] + src + ["-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.check_call(cmd)
    return LIB_PATH


_lib = None


def lib():
    """Loads the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise McmcError(-1, f"{LIB_PATH} is missing: run __graft_entry__.build() "
                                "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        L.mcmc_b200_last_error.restype = C.c_char_p
        L.mcmc_b200_stream.restype = C.c_void_p
        L.mcmc_b200_stream.argtypes = [C.c_void_p]
        L.mcmc_b200_launch_count.restype = C.c_int64
        L.mcmc_b200_launch_count.argtypes = [C.c_void_p, C.c_int]
        L.mcmc_b200_philox_normal.restype = C.c_float
        L.mcmc_b200_philox_normal.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
        L.mcmc_b200_refstream_engine.restype = C.c_uint32
        L.mcmc_b200_refstream_engine.argtypes = [C.c_uint64]
        L.mcmc_b200_refstream_engine0.restype = C.c_uint32
        L.mcmc_b200_refstream_engine0.argtypes = [C.c_uint64]
        L.mcmc_b200_refstream_log_uniform.restype = C.c_float
        L.mcmc_b200_refstream_log_uniform.argtypes = [C.c_uint64]
        L.mcmc_b200_destroy.argtypes = [C.c_void_p]
        L.mcmc_b200_destroy.restype = None
        _lib = L
    return _lib


def _check(code):
    if code != OK:
        raise McmcError(code, lib().mcmc_b200_last_error().decode())


def _fp(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


def _vp(ptr):
    return C.c_void_p(int(ptr)) if ptr is not None else None


def reference_config(**kw):
    cfg = Config()
    lib().mcmc_b200_config_reference(C.byref(cfg))
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


def baseline_config(**kw):
    cfg = Config()
    lib().mcmc_b200_config_baseline(C.byref(cfg))
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


def num_params(D, H):
    return D * H + 2 * H + 1


def synth_window(seed, window, rows, D=22, H=40):
    """Synthetic (X, y, teacher) of one window; host code, needs no GPU."""
    x = np.empty((rows, D), np.float32)
    y = np.empty(rows, np.float32)
    t = np.empty(num_params(D, H), np.float32)
    _check(lib().mcmc_b200_synth_window(C.c_uint64(seed), C.c_int64(window), C.c_int64(rows), D, H,
                                        _fp(x), _fp(y), _fp(t)))
    return x, y, t


def philox_raw(ctr, key):
    c = (C.c_uint32 * 4)(*ctr)
    k = (C.c_uint32 * 2)(*key)
    o = (C.c_uint32 * 4)()
    lib().mcmc_b200_philox_raw(c, k, o)
    return list(o)


def potential_and_grad_static(cfg, x_ptr, y_ptr, rows, w_ptr, grad_ptr, scalars_ptr, stream=None):
    """Allocation-free log p / gradient on device pointers (see include/mcmc_b200.h); asynchronous."""
    _check(lib().mcmc_b200_potential_and_grad_static(C.byref(cfg), _vp(x_ptr), _vp(y_ptr), C.c_int64(rows),
                                                     _vp(w_ptr), _vp(grad_ptr), _vp(scalars_ptr),
                                                     _vp(stream)))


def microbench_l2_read(nbytes, device=0):
    """GB/s at which all SMs re-read an L2-resident buffer of nbytes (ld.global.cg, 128-bit)."""
    out = C.c_double()
    _check(lib().mcmc_b200_microbench_l2_read(device, C.c_int64(nbytes), C.byref(out)))
    return out.value


def microbench_mufu(kind=0, device=0):
    """10^9 values/s through the MUFU pipe: kind 0 = tanh.approx.f32, kind 1 = ex2.approx + rcp.approx."""
    out = C.c_double()
    _check(lib().mcmc_b200_microbench_mufu(device, kind, C.byref(out)))
    return out.value


def read_table(path, rows, total_cols=149, skip_cols=2, D=22, feature_scale=0.001):
    """The reference's dataset text layout (io.h:42-80 there): header of total_cols tokens, then per row
    skip_cols ignored, one label, D features, the rest ignored.  Returns (x [rows][D] scaled, y [rows])."""
    x = np.empty((rows, D), np.float32)
    y = np.empty(rows, np.float32)
    _check(lib().mcmc_b200_read_table(os.fsencode(path), C.c_int64(rows), total_cols, skip_cols, D,
                                      C.c_float(feature_scale), _fp(x), _fp(y)))
    return x, y


def plan_work_table(windows, tiles_per_window, max_ctas=148, slices=0):
    """The persistent kernels' work partition: list (one entry per CTA) of lists of
    (window, first_tile, end_tile, slot).  Host arithmetic only."""
    n_ctas, n_segs = C.c_int32(), C.c_int32()
    _check(lib().mcmc_b200_plan_work_table(windows, C.c_int64(tiles_per_window), max_ctas, slices, None, 0,
                                           None, 0, C.byref(n_ctas), C.byref(n_segs)))
    sp = np.empty(n_ctas.value + 1, np.int32)
    sg = np.empty((n_segs.value, 4), np.int32)
    _check(lib().mcmc_b200_plan_work_table(windows, C.c_int64(tiles_per_window), max_ctas, slices,
                                           sp.ctypes.data_as(C.POINTER(C.c_int32)), sp.size,
                                           sg.ctypes.data_as(C.POINTER(C.c_int32)), n_segs.value,
                                           C.byref(n_ctas), C.byref(n_segs)))
    return [[tuple(int(v) for v in sg[i]) for i in range(sp[b], sp[b + 1])] for b in range(n_ctas.value)]


def nccl_unique_id():
    buf = (C.c_ubyte * 128)()
    _check(lib().mcmc_b200_nccl_unique_id(buf))
    return bytes(buf)


class Context:
    """What the reference's main_loop allocates (main.h:153-183), for n_windows windows."""

    def __init__(self, cfg: Config, n_windows=1, rows=58368, device=0):
        self.cfg = cfg
        self.n_windows = n_windows
        self.rows = rows
        self._h = C.c_void_p()
        _check(lib().mcmc_b200_create(C.byref(cfg), device, n_windows, C.c_int64(rows), C.byref(self._h)))
        self.P = lib().mcmc_b200_num_params(self._h)

    def close(self):
        if self._h:
            lib().mcmc_b200_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- data ------------------------------------------------------------
    def set_window_data(self, window, x, y, global_window=None):
        x = np.ascontiguousarray(x, np.float32)
        y = np.ascontiguousarray(y, np.float32)
        assert x.shape == (self.rows, self.cfg.D) and y.shape == (self.rows,)
        gw = window if global_window is None else global_window
        _check(lib().mcmc_b200_set_window_data(self._h, window, C.c_int64(gw), _fp(x), _fp(y), 0))

    def set_window_data_ptr(self, window, x_ptr, y_ptr, is_device, global_window=None):
        gw = window if global_window is None else global_window
        _check(lib().mcmc_b200_set_window_data(self._h, window, C.c_int64(gw), _vp(x_ptr), _vp(y_ptr),
                                               int(is_device)))

    # -- per-call probes ---------------------------------------------------
    def potential_and_grad(self, window, w, want_row_loss=False):
        w = np.ascontiguousarray(w, np.float32)
        assert w.shape == (self.P,)
        ll, lp = C.c_double(), C.c_double()
        grad = np.empty(self.P, np.float32)
        rl = np.empty(self.rows, np.float32) if want_row_loss else None
        _check(lib().mcmc_b200_potential_and_grad(self._h, window, _fp(w), C.byref(ll), C.byref(lp),
                                                  _fp(grad), _fp(rl)))
        return dict(loglik=ll.value, logprior=lp.value, grad=grad, row_loss=rl)

    def leapfrog(self, window, L, eps, w_prev, mom_prev, grad_prev):
        a = [np.ascontiguousarray(v, np.float32) for v in (w_prev, mom_prev, grad_prev)]
        w_next, mom_next, grad_cur = (np.empty(self.P, np.float32) for _ in range(3))
        ll, lp = C.c_double(), C.c_double()
        _check(lib().mcmc_b200_leapfrog(self._h, window, L, C.c_float(eps), _fp(a[0]), _fp(a[1]), _fp(a[2]),
                                        _fp(w_next), _fp(mom_next), _fp(grad_cur), C.byref(ll),
                                        C.byref(lp)))
        return dict(w_next=w_next, mom_next=mom_next, grad_cur=grad_cur, loglik=ll.value,
                    logprior=lp.value)

    # -- chain -------------------------------------------------------------
    def run_chain(self, n_iter, sync=True):
        fn = lib().mcmc_b200_run_chain if sync else lib().mcmc_b200_run_chain_async
        _check(fn(self._h, n_iter))

    def synchronize(self):
        _check(lib().mcmc_b200_synchronize(self._h))

    def reset_chain(self):
        _check(lib().mcmc_b200_reset_chain(self._h))

    @property
    def stream(self):
        return lib().mcmc_b200_stream(self._h)

    def chain_info(self, window=0):
        it, acc, eps = C.c_int32(), C.c_int32(), C.c_float()
        _check(lib().mcmc_b200_chain_info(self._h, window, C.byref(it), C.byref(acc), C.byref(eps)))
        return dict(iterations=it.value, accepted=acc.value, eps=eps.value)

    def get_state(self, window=0):
        w, g = np.empty(self.P, np.float32), np.empty(self.P, np.float32)
        ll, lp = C.c_double(), C.c_double()
        _check(lib().mcmc_b200_get_state(self._h, window, _fp(w), _fp(g), C.byref(ll), C.byref(lp)))
        return dict(w=w, grad=g, loglik=ll.value, logprior=lp.value)

    def get_samples(self, window=0, first=0, count=None, out=None):
        count = self.cfg.sample_capacity - first if count is None else count
        if out is None:
            out = np.empty((count, self.P), np.float32)
        _check(lib().mcmc_b200_get_samples(self._h, window, first, count, _fp(out)))
        return out

    def get_samples_ptr(self, window, first, count, host_ptr):
        _check(lib().mcmc_b200_get_samples(self._h, window, first, count, _vp(host_ptr)))

    def get_trace(self, window=0, first=0, count=None):
        count = self.cfg.trace_iters - first if count is None else count
        mom = np.empty((count, self.P), np.float32)
        log_u = np.empty(count, np.float32)
        la = np.empty(count, np.float64)
        acc = np.empty(count, np.int32)
        eps = np.empty(count, np.float32)
        _check(lib().mcmc_b200_get_trace(self._h, window, first, count, _fp(mom), _fp(log_u),
                                         la.ctypes.data_as(C.POINTER(C.c_double)),
                                         acc.ctypes.data_as(C.POINTER(C.c_int32)), _fp(eps)))
        return dict(momenta=mom, log_u=log_u, log_acpt=la, accepted=acc, eps=eps)

    def predict_mean(self, window, xs, first=0, count=None):
        xs = np.ascontiguousarray(xs, np.float32)
        count = self.cfg.sample_capacity - first if count is None else count
        out = np.empty(xs.shape[0], np.float32)
        _check(lib().mcmc_b200_predict_mean(self._h, window, _fp(xs), C.c_int64(xs.shape[0]), first, count,
                                            _fp(out)))
        return out

    def final_loss(self, window=0, first=0, count=None):
        count = self.cfg.sample_capacity - first if count is None else count
        a, b = C.c_double(), C.c_double()
        _check(lib().mcmc_b200_final_loss(self._h, window, first, count, C.byref(a), C.byref(b)))
        return a.value, b.value

    # -- checkpoint / resume / export -----------------------------------------
    def checkpoint(self):
        """The chain state of every window (position, momentum, carried gradient, step size, counters,
        stored samples, trace) as one bytes object; the dataset is not included."""
        n = C.c_uint64()
        _check(lib().mcmc_b200_checkpoint_size(self._h, C.byref(n)))
        buf = np.empty(n.value, np.uint8)
        _check(lib().mcmc_b200_checkpoint_save(self._h, buf.ctypes.data_as(C.c_void_p), n))
        return buf

    def restore(self, blob):
        """Resume from ``checkpoint()`` output (same configuration, data already uploaded)."""
        buf = np.ascontiguousarray(np.frombuffer(blob, np.uint8) if not isinstance(blob, np.ndarray) else blob)
        _check(lib().mcmc_b200_checkpoint_load(self._h, buf.ctypes.data_as(C.c_void_p), C.c_uint64(buf.size)))

    def save_checkpoint(self, path):
        self.checkpoint().tofile(path)

    def load_checkpoint(self, path):
        self.restore(np.fromfile(path, np.uint8))

    def export_samples(self, prefix, first=0, count=None):
        """Writes ``prefix.samples.f32`` (raw little-endian float32 [windows][count][P]) and
        ``prefix.json`` (shape, configuration, per-window counters and the recorded trace)."""
        import json
        count = self.cfg.sample_capacity - first if count is None else count
        with open(prefix + ".samples.f32", "wb") as f:
            for w in range(self.n_windows):
                self.get_samples(w, first, count).tofile(f)
        meta = {"shape": [self.n_windows, count, self.P], "dtype": "float32", "first_sample": first,
                "config": {k: getattr(self.cfg, k) for k, _ in Config._fields_},
                "windows": [self.chain_info(w) for w in range(self.n_windows)]}
        if self.cfg.trace_iters > 0:
            done = min(self.cfg.trace_iters, min(i["iterations"] for i in meta["windows"]))
            meta["trace"] = []
            for w in range(self.n_windows):
                t = self.get_trace(w, 0, done)
                meta["trace"].append({"log_u": t["log_u"].tolist(), "log_acpt": t["log_acpt"].tolist(),
                                      "accepted": t["accepted"].tolist(), "eps": t["eps"].tolist()})
        with open(prefix + ".json", "w") as f:
            json.dump(meta, f)

    # -- multi-GPU -----------------------------------------------------------
    def enable_row_sharding(self, unique_id: bytes, rank, nranks):
        buf = (C.c_ubyte * 128).from_buffer_copy(unique_id)
        _check(lib().mcmc_b200_enable_row_sharding(self._h, buf, rank, nranks))

    def enable_oneshot_allreduce(self):
        """The per-step all-reduce over peer memory instead of NCCL (after enable_row_sharding)."""
        _check(lib().mcmc_b200_enable_oneshot_allreduce(self._h))

    def time_allreduce(self, reps=200):
        us = C.c_float()
        _check(lib().mcmc_b200_time_allreduce(self._h, reps, C.byref(us)))
        return us.value

    def selftest_oneshot_timeout(self, polls=2000):
        code = lib().mcmc_b200_selftest_oneshot_timeout(self._h, int(polls))
        return code, lib().mcmc_b200_last_error().decode()

    # -- drop-ins on device pointers ------------------------------------------
    def mcmc_step(self, x, y, weights_prev, weights_next, mom_prev, mom_next, grad_prev, grad_cur,
                  grad_next, loss_values, L, eps, stream=None):
        """mcmc::mcmc_step<float, L> on device pointers (ints)."""
        _check(lib().mcmc_b200_mcmc_step(self._h, _vp(x), _vp(y), _vp(weights_prev), _vp(weights_next),
                                         _vp(mom_prev), _vp(mom_next), _vp(grad_prev), _vp(grad_cur),
                                         _vp(grad_next), _vp(loss_values), L, C.c_float(eps),
                                         _vp(stream if stream is not None else self.stream)))

    def rebind_data(self):
        """The next mcmc_step repacks the dataset even when x and y are the same pointers as before."""
        _check(lib().mcmc_b200_rebind_data(self._h))

    def selftest_wait_timeout(self, limit_us=1000):
        """Runs a bounded device-side wait into its limit; returns the status code the context reports
        (4 = MCMC_B200_ERR_TIMEOUT when the time-out route works) and its message."""
        code = lib().mcmc_b200_selftest_wait_timeout(self._h, int(limit_us))
        return code, lib().mcmc_b200_last_error().decode()

    def philox_device(self, ctr, key, n):
        """The device's evaluation of the random streams: (raw [n][4] uint32, normals [n], accept uniform)."""
        c = (C.c_uint32 * 4)(*ctr)
        k = (C.c_uint32 * 2)(*key)
        raw = np.empty((n, 4), np.uint32)
        nrm = np.empty(n, np.float32)
        u = C.c_float()
        _check(lib().mcmc_b200_philox_device(self._h, c, k, n, raw.ctypes.data_as(C.POINTER(C.c_uint32)),
                                             _fp(nrm), C.byref(u)))
        return raw, nrm, u.value

    def refstream_momentum_device(self, first_n, count):
        """The reference's momentum stream evaluated on the device: draws first_n .. first_n + count - 1."""
        out = np.empty(count, np.float32)
        _check(lib().mcmc_b200_refstream_momentum_device(self._h, C.c_uint64(first_n), count, _fp(out)))
        return out

    def log_acpt(self, prev_loss, new_loss, n_loss, prev_mom, new_mom, grad_cur, eps, stream=None):
        """mcmc::log_acpt_prec on device pointers (ints); returns the host scalar."""
        out = C.c_float()
        _check(lib().mcmc_b200_log_acpt(self._h, _vp(prev_loss), _vp(new_loss), C.c_int64(n_loss),
                                        _vp(prev_mom), _vp(new_mom), _vp(grad_cur), C.c_float(eps),
                                        _vp(stream if stream is not None else self.stream),
                                        C.byref(out)))
        return out.value

    # -- bookkeeping ---------------------------------------------------------
    def launch_count(self, reset=False):
        return lib().mcmc_b200_launch_count(self._h, int(reset))

    def geometry(self):
        s, c, t = C.c_int(), C.c_int(), C.c_int()
        _check(lib().mcmc_b200_chain_geometry(self._h, C.byref(s), C.byref(c), C.byref(t)))
        return dict(slices=s.value, ctas_per_sm=c.value, tile_rows=t.value)
