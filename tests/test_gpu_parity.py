"""Parity of the CUDA path (through the C-ABI) with the CPU oracle on the same
seeded inputs.  Tolerances are the ones the task states: per-call potential and
gradient within rel 1e-5 (FP32) / 2e-3 (TF32), identical accept decisions over
the first 50 iterations, posterior-mean predictions over 800 samples within 1 %."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

D, H, P = 22, 40, 961
TOL = {0: 1e-5, 1: 2e-3}


def _w(seed, scale=0.15, p=P):
    return (scale * np.random.default_rng(seed).standard_normal(p)).astype(np.float32)


def _presets(m, O, prec):
    tf = prec == m.PREC_TF32
    return {
        "baseline": (m.baseline_config(precision=prec), O.baseline_model(tf32=tf)),
        "reference": (m.reference_config(precision=prec), O.reference_model(tf32=tf)),
    }


def _grad_err(got, ref):
    return float(np.abs(got - ref).max() / np.abs(ref).max())


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("preset", ["baseline", "reference"])
@pytest.mark.parametrize("rows", [1, 2, 127, 129, 1000, 58368])
def test_potential_and_grad(built, prec, preset, rows):
    m, O = built
    cfg, model = _presets(m, O, prec)[preset]
    x, y, _ = m.synth_window(11, rows % 7, rows)
    if preset == "reference":
        x = x * np.float32(0.05)  # keep tanh out of saturation with wider weights
    w = _w(rows, 0.3 if preset == "reference" else 0.15)
    ctx = m.Context(cfg, n_windows=1, rows=rows)
    ctx.set_window_data(0, x, y)
    got = ctx.potential_and_grad(0, w, want_row_loss=True)
    ref = O.logp_grad(model, x, y, w, want_losses=True)
    tol = TOL[prec]
    assert _grad_err(got["grad"], ref["grad"]) < tol
    assert abs(got["loglik"] - ref["loglik"]) <= tol * abs(ref["loglik"])
    assert abs(got["logprior"] - ref["logprior"]) <= 1e-6 * abs(ref["logprior"])
    assert np.allclose(got["row_loss"], ref["row_loss"], rtol=10 * tol, atol=10 * tol)
    ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_tf32_and_fp32_modes_agree_with_exact_oracle(built, prec):
    """Both modes against the untruncated oracle: FP32 at 1e-5, TF32 at 2e-3."""
    m, O = built
    rows = 20000
    x, y, _ = m.synth_window(5, 1, rows)
    w = _w(77)
    ctx = m.Context(m.baseline_config(precision=prec), n_windows=1, rows=rows)
    ctx.set_window_data(0, x, y)
    got = ctx.potential_and_grad(0, w)
    ref = O.logp_grad(O.baseline_model(tf32=False), x, y, w)
    assert _grad_err(got["grad"], ref["grad"]) < TOL[prec]
    assert abs(got["loglik"] - ref["loglik"]) <= TOL[prec] * abs(ref["loglik"])
    ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("rows", [100, 3000, 40000])
def test_wide_model(built, prec, rows):
    """22-128-1 (3073 parameters, the scaled stress configuration) in both precisions."""
    m, O = built
    Hw = 128
    Pw = 22 * Hw + 2 * Hw + 1
    x, y, _ = m.synth_window(3, 0, rows, H=Hw)
    w = _w(5, 0.1, Pw)
    ctx = m.Context(m.baseline_config(H=Hw, precision=prec), n_windows=1, rows=rows)
    ctx.set_window_data(0, x, y)
    got = ctx.potential_and_grad(0, w, want_row_loss=True)
    ref = O.logp_grad(O.baseline_model(tf32=bool(prec), H=Hw), x, y, w, want_losses=True)
    tol = TOL[prec]
    assert _grad_err(got["grad"], ref["grad"]) < tol
    assert abs(got["loglik"] - ref["loglik"]) <= tol * abs(ref["loglik"])
    assert np.allclose(got["row_loss"], ref["row_loss"], rtol=tol * 10, atol=tol)
    ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_wide_model_chain_matches_oracle(built, prec):
    """A short multi-window chain at 128 hidden units: device draws replayed through the oracle."""
    m, O = built
    Hw, rows, W, iters = 128, 6000, 3, 6
    Pw = 22 * Hw + 2 * Hw + 1
    cfg = m.baseline_config(H=Hw, precision=prec, leapfrog_steps=4, eps0=2e-4, sample_capacity=iters,
                            trace_iters=iters, seed=9)
    ctx = m.Context(cfg, n_windows=W, rows=rows)
    data = []
    for w in range(W):
        x, y, _ = m.synth_window(8, w, rows, H=Hw)
        ctx.set_window_data(w, x, y, global_window=w)
        data.append((x, y))
    ctx.run_chain(iters)
    model = O.baseline_model(tf32=bool(prec), H=Hw)
    sampler = O.baseline_sampler(L=4, eps=2e-4)
    for w in range(W):
        tr = ctx.get_trace(w)
        ref = O.hmc_chain(model, sampler, data[w][0], data[w][1], tr["momenta"], tr["log_u"])
        # decisions must agree wherever the draw is not within the kernel tolerance of the ratio
        clear = np.abs(ref["log_acpt"] - tr["log_u"]) > 0.05
        assert np.array_equal(ref["accepted"][clear], tr["accepted"][clear])
        if np.array_equal(ref["accepted"], tr["accepted"]):
            got = ctx.get_samples(w)
            tol = TOL[prec]
            assert np.abs(got - ref["samples"]).max() <= tol * max(1e-3, np.abs(ref["samples"]).max())
            assert np.allclose(tr["log_acpt"], ref["log_acpt"], rtol=1e-2, atol=5e-2)
    ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("L", [1, 2, 10])
def test_leapfrog_matches_oracle_mcmc_step(built, prec, L):
    m, O = built
    rows = 5000
    x, y, _ = m.synth_window(21, 2, rows)
    cfg, model = _presets(m, O, prec)["baseline"]
    w0 = _w(1)
    mom = np.random.default_rng(2).standard_normal(P).astype(np.float32)
    ctx = m.Context(cfg, n_windows=1, rows=rows)
    ctx.set_window_data(0, x, y)
    g0 = ctx.potential_and_grad(0, w0)["grad"]
    got = ctx.leapfrog(0, L, 1e-3, w0, mom, g0)
    ref = O.mcmc_step(model, x, y, L, 1e-3, w0, mom, g0)
    tol = TOL[prec]
    assert np.allclose(got["w_next"], ref["w_next"], rtol=tol, atol=tol * 1e-2)
    assert np.allclose(got["mom_next"], ref["mom_next"], rtol=tol, atol=tol)
    assert _grad_err(got["grad_cur"], ref["grad_cur"]) < tol
    assert abs(got["loglik"] - ref["loglik"]) <= tol * abs(ref["loglik"])
    ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("preset", ["baseline", "reference"])
def test_accept_decisions_identical_over_first_50_iterations(built, preset, prec):
    """The device chain replayed on the CPU with the draws the device used, in both precisions (the oracle
    runs in the same mode: TF32 truncates the tensor-core operands as the device does)."""
    m, O = built
    rows, n_iter = 58368 if preset == "baseline" else 8192, 50
    x, y, _ = m.synth_window(9, 0, rows)
    tf = bool(prec)
    if preset == "baseline":
        cfg = m.baseline_config(precision=prec, sample_capacity=n_iter, trace_iters=n_iter, seed=1234)
        model, sampler = O.baseline_model(tf32=tf), O.baseline_sampler()
    else:
        # the reference's Student-t / N(0,200^2) preset with its adaptive burn-in, shortened to
        # L = 10 so that the CPU replay finishes in seconds; eps0 = 0.2 gives accepts, rejections and both
        # branches of the step-size adaptation within 50 iterations
        cfg = m.reference_config(precision=prec, leapfrog_steps=10, burn_in=0, adapt_steps=30,
                                 sample_capacity=n_iter, trace_iters=n_iter, seed=99, eps0=0.2)
        x = x * np.float32(0.05)
        model, sampler = O.reference_model(tf32=tf), O.Sampler(10, 30, 0.2, 0.2, 0.1, 0.01)
    ctx = m.Context(cfg, n_windows=1, rows=rows)
    ctx.set_window_data(0, x, y)
    ctx.run_chain(n_iter)
    tr = ctx.get_trace(0)
    samples = ctx.get_samples(0, 0, n_iter)
    ref = O.hmc_chain(model, sampler, x, y, tr["momenta"], tr["log_u"])
    differ = np.flatnonzero(tr["accepted"] != ref["accepted"])
    margin = np.abs(ref["log_acpt"] - tr["log_u"])
    assert differ.size == 0, ("decisions differ at iterations %s; |log_acpt - log_u| there: %s; device "
                              "log_acpt %s, oracle %s" % (differ, margin[differ], tr["log_acpt"][differ],
                                                           ref["log_acpt"][differ]))
    assert np.allclose(tr["eps"], ref["eps"], rtol=1e-6)
    if prec == 0:
        assert np.allclose(tr["log_acpt"], ref["log_acpt"], rtol=1e-3, atol=2e-2)
        assert np.allclose(samples, ref["samples"], rtol=1e-4, atol=1e-5)
    else:
        # same decisions, so the two chains visit the same states up to the TF32 mode's per-call tolerance
        assert np.abs(samples - ref["samples"]).max() <= TOL[1] * max(1e-3, np.abs(ref["samples"]).max())
    info = ctx.chain_info(0)
    assert info["iterations"] == n_iter and info["accepted"] == int(ref["accepted"].sum())
    if preset == "reference":
        assert 0 < ref["accepted"].sum() < n_iter  # the case exercises both branches
    # draws are N(0,1) / log U(0,1]
    assert abs(tr["momenta"].std() - 1) < 0.02 and np.all(tr["log_u"] <= 0)
    ctx.close()


def _host_accept_log_u(m, seed, gwin, it):
    """log of the accept uniform of (seed, window, iteration), from the host's Philox."""
    r = m.philox_raw([0, it, gwin, 1], [seed & 0xFFFFFFFF, seed >> 32])
    u = np.float32((np.float32(r[0] >> 8) + np.float32(1.0)) * np.float32(1.0 / 16777216.0))
    return np.log(u, dtype=np.float32)


def test_device_random_streams_equal_the_host_functions(built):
    """Momentum normals and accept uniforms drawn inside the accept kernel are the host functions'
    values for (seed, GLOBAL window, iteration): raw Philox words bit-exact, normals to 2e-6 relative (the device
    uses sincospif, the host sinf/cosf), log-uniforms to float rounding."""
    m, _ = built
    rows, n_iter, W, seed = 512, 6, 3, 0x1234567ABCDEF
    gwins = (7, 1000, 65536 + 3)
    cfg = m.baseline_config(sample_capacity=n_iter, trace_iters=n_iter, seed=seed)
    ctx = m.Context(cfg, n_windows=W, rows=rows)
    for w in range(W):
        x, y, _ = m.synth_window(3, w, rows)
        ctx.set_window_data(w, x, y, global_window=gwins[w])
    ctx.run_chain(n_iter)
    key = [seed & 0xFFFFFFFF, seed >> 32]
    for w in range(W):
        tr = ctx.get_trace(w)
        for it in range(n_iter):
            host = np.array([m.lib().mcmc_b200_philox_normal(seed, gwins[w], it, 0, p) for p in range(P)],
                            np.float32)
            assert np.all(np.abs(tr["momenta"][it] - host) <= 2e-6 * np.maximum(1.0, np.abs(host))), (w, it)
            lu = _host_accept_log_u(m, seed, gwins[w], it)
            assert abs(tr["log_u"][it] - lu) <= 1e-6 * max(1.0, abs(lu)), (w, it)
        # the generator itself, evaluated on the device: bit-exact words
        raw, nrm, u = ctx.philox_device([5, 2, gwins[w], 0], key, 100)
        for i in (0, 1, 57, 99):
            assert list(raw[i]) == m.philox_raw([5 + i, 2, gwins[w], 0], key)
        host = np.array([m.lib().mcmc_b200_philox_normal(seed, gwins[w], 2, 0, p) for p in range(100)], np.float32)
        assert np.all(np.abs(nrm - host) <= 2e-6 * np.maximum(1.0, np.abs(host)))
        assert abs(np.log(np.float32(u)) - _host_accept_log_u(m, seed, gwins[w], 2)) <= 1e-6
    ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_posterior_mean_prediction_over_800_samples(built, prec):
    """Posterior-mean prediction over 800 samples against the CPU replay, three seeds.  The stated bound is
    1 %.  It holds whenever the device chain and the replay take the same 800 decisions.  When they do
    not (possible in TF32 mode only: a proposal whose ratio is within rounding of the draw), the two
    chains decorrelate from that iteration on and the difference is Monte-Carlo, not kernel, error; its
    size is measured in the same test as the oracle's own exact-vs-TF32 divergence on the same draws,
    and the device must stay within 1.5x of it."""
    m, O = built
    rows, n_iter = 2048, 800
    for seed in (5, 6, 7):
        x, y, _ = m.synth_window(31, 0, rows)
        cfg = m.baseline_config(precision=prec, sample_capacity=n_iter, trace_iters=n_iter, seed=seed)
        ctx = m.Context(cfg, n_windows=1, rows=rows)
        ctx.set_window_data(0, x, y)
        ctx.run_chain(n_iter)
        tr = ctx.get_trace(0)
        ref = O.hmc_chain(O.baseline_model(tf32=bool(prec)), O.baseline_sampler(), x, y, tr["momenta"],
                          tr["log_u"])
        assert ref["accepted"].sum() > n_iter // 2  # the chain moves
        xs, _, _ = m.synth_window(31, 1, 512)
        got = ctx.predict_mean(0, xs)
        exp = O.predict_mean(O.baseline_model(), xs, ref["samples"])
        rel_l2 = np.linalg.norm(got - exp) / np.linalg.norm(exp)
        same = np.array_equal(tr["accepted"], ref["accepted"])
        if prec == 0:
            assert same and rel_l2 < 1e-2, (seed, rel_l2)
        elif same:
            assert rel_l2 < 1e-2, (seed, rel_l2)
        else:
            other = O.hmc_chain(O.baseline_model(tf32=False), O.baseline_sampler(), x, y, tr["momenta"],
                                tr["log_u"])
            exp2 = O.predict_mean(O.baseline_model(), xs, other["samples"])
            own_div = np.linalg.norm(exp2 - exp) / np.linalg.norm(exp)
            first = int(np.flatnonzero(tr["accepted"] != ref["accepted"])[0])
            margin = abs(ref["log_acpt"][first] - tr["log_u"][first])
            assert margin < 0.05, (seed, first, margin)  # only a borderline proposal may flip
            assert rel_l2 <= max(1e-2, 1.5 * own_div), (seed, rel_l2, own_div)
            assert np.mean(tr["accepted"] == ref["accepted"]) > 0.97
        # and the device's own forward pass over its own samples is exact to FP32
        own = O.predict_mean(O.baseline_model(), xs, ctx.get_samples(0))
        assert np.linalg.norm(got - own) / np.linalg.norm(own) < 1e-5
        if seed == 5:
            ll, lp = ctx.final_loss(0, 0, 16)
            ell, elp = O.final_loss(O.baseline_model(tf32=bool(prec)), x, y, ctx.get_samples(0, 0, 16))
            assert abs(ll - ell) <= TOL[prec] * abs(ell) and abs(lp - elp) <= 1e-5 * abs(elp)
        ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_batched_windows_equal_single_window_chains_bitwise(built, prec):
    """Windows are independent: a window gives the same chain alone or batched,
    wherever it sits (the random streams are keyed by the global window id)."""
    m, _ = built
    rows, n_iter, W = 3000, 12, 3
    data = [m.synth_window(8, g, rows) for g in (10, 11, 12)]
    cfg = m.baseline_config(precision=prec, sample_capacity=n_iter, slices=5, seed=3)
    batched = m.Context(cfg, n_windows=W, rows=rows)
    for i, (x, y, _) in enumerate(data):
        batched.set_window_data(i, x, y, global_window=10 + i)
    batched.run_chain(n_iter)
    for i, (x, y, _) in enumerate(data):
        single = m.Context(cfg, n_windows=1, rows=rows)
        single.set_window_data(0, x, y, global_window=10 + i)
        single.run_chain(5)
        single.run_chain(n_iter - 5)  # split runs continue the same chain
        assert np.array_equal(single.get_samples(0), batched.get_samples(i))
        single.close()
    # and a second identical run is bit-identical (no atomics anywhere)
    again = m.Context(cfg, n_windows=W, rows=rows)
    for i, (x, y, _) in enumerate(data):
        again.set_window_data(i, x, y, global_window=10 + i)
    again.run_chain(n_iter)
    for i in range(W):
        assert np.array_equal(again.get_samples(i), batched.get_samples(i))
    assert not np.array_equal(batched.get_samples(0), batched.get_samples(1))
    again.close()
    batched.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_mcmc_step_and_log_acpt_drop_ins_on_device_buffers(built, prec):
    """mcmc::mcmc_step / mcmc::log_acpt_prec semantics on caller-owned device buffers."""
    import torch
    m, O = built
    rows, L, eps = 4096, 3, 2e-3
    x, y, _ = m.synth_window(2, 0, rows)
    cfg, model = _presets(m, O, prec)["baseline"]
    dev = torch.device("cuda:0")
    tx, ty = torch.from_numpy(x).to(dev), torch.from_numpy(y).to(dev)
    w0 = _w(3)
    mom = np.random.default_rng(4).standard_normal(P).astype(np.float32)
    ref0 = O.logp_grad(model, x, y, w0, want_losses=True)
    g0 = ref0["grad"].astype(np.float32)
    t = {k: torch.from_numpy(v).to(dev) for k, v in dict(wp=w0, mp=mom, gp=g0).items()}
    out = {k: torch.full((P,), 7.0, device=dev) for k in ("wn", "mn", "gc", "gn")}
    loss = torch.zeros(rows + P, device=dev)
    ctx = m.Context(cfg, n_windows=1, rows=rows)
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(2):  # second call reuses the repacked dataset
        ctx.mcmc_step(tx.data_ptr(), ty.data_ptr(), t["wp"].data_ptr(), out["wn"].data_ptr(),
                      t["mp"].data_ptr(), out["mn"].data_ptr(), t["gp"].data_ptr(), out["gc"].data_ptr(),
                      out["gn"].data_ptr(), loss.data_ptr(), L, eps, stream=s)
    torch.cuda.synchronize()
    ref = O.mcmc_step(model, x, y, L, eps, w0, mom, g0)
    tol = TOL[prec]
    assert np.allclose(out["wn"].cpu().numpy(), ref["w_next"], rtol=tol, atol=tol * 1e-2)
    assert np.allclose(out["mn"].cpu().numpy(), ref["mom_next"], rtol=tol, atol=tol)
    assert _grad_err(out["gc"].cpu().numpy(), ref["grad_cur"]) < tol
    assert np.all(out["gn"].cpu().numpy() == 0)
    assert np.allclose(loss.cpu().numpy(), ref["loss_values"], rtol=10 * tol, atol=10 * tol)
    # accept ratio on device buffers
    prev_loss = torch.from_numpy(np.concatenate([ref0["row_loss"], ref0["prior_loss"]])).to(dev)
    la = ctx.log_acpt(prev_loss.data_ptr(), loss.data_ptr(), rows + P, t["mp"].data_ptr(),
                      out["mn"].data_ptr(), out["gc"].data_ptr(), eps, stream=s)
    mf = ref["mom_next"].astype(np.float64) + 0.5 * np.float32(eps) * ref["grad_cur"].astype(np.float64)
    exp = float(np.sum(ref["loss_values"].astype(np.float64)) -
                np.sum(prev_loss.cpu().numpy().astype(np.float64)) +
                0.5 * (np.sum(mom.astype(np.float64) ** 2) - np.sum(mf ** 2)))
    assert abs(la - exp) < max(5e-3, 20 * tol * abs(exp))
    ctx.close()


def test_errors_are_reported_not_fatal(built):
    m, _ = built
    with pytest.raises(m.McmcError):
        m.Context(m.baseline_config(D=21), n_windows=1, rows=128)
    ctx = m.Context(m.baseline_config(), n_windows=2, rows=256)
    with pytest.raises(m.McmcError) as e:
        ctx.run_chain(1)  # no data yet
    assert "no data" in str(e.value)
    with pytest.raises(m.McmcError):
        ctx.get_samples(5)
    ctx.close()


@pytest.mark.gpu
@pytest.mark.parametrize("prec", [0, 1])
def test_checkpoint_resume_is_bit_identical(built, prec, tmp_path):
    """12 iterations in one go == 5 iterations, checkpoint, new context, restore, 7 more (3 windows,
    adaptive preset so that the step size and the counters matter)."""
    m, O = built
    rows, W = 3000, 3
    cfg = m.reference_config(precision=prec, leapfrog_steps=5, burn_in=4, adapt_steps=4, sample_capacity=8,
                             trace_iters=12, eps0=0.02, seed=77)

    def make():
        ctx = m.Context(cfg, n_windows=W, rows=rows)
        for w in range(W):
            x, y, _ = m.synth_window(5, w, rows)
            ctx.set_window_data(w, x * np.float32(0.05), y, global_window=10 + w)
        return ctx

    a = make()
    a.run_chain(12)
    b = make()
    b.run_chain(5)
    path = str(tmp_path / "chain.ckpt")
    b.save_checkpoint(path)
    b.close()
    c = make()
    c.load_checkpoint(path)
    c.run_chain(7)
    for w in range(W):
        assert a.chain_info(w) == c.chain_info(w)
        sa, sc = a.get_state(w), c.get_state(w)
        assert np.array_equal(sa["w"], sc["w"]) and np.array_equal(sa["grad"], sc["grad"])
        assert sa["loglik"] == sc["loglik"]
        assert np.array_equal(a.get_samples(w), c.get_samples(w))
        ta, tc = a.get_trace(w), c.get_trace(w)
        assert np.array_equal(ta["accepted"], tc["accepted"]) and np.array_equal(ta["log_acpt"], tc["log_acpt"])
    # a checkpoint of another configuration is refused
    other = m.Context(m.reference_config(precision=prec, leapfrog_steps=6, burn_in=4, adapt_steps=4,
                                         sample_capacity=8, trace_iters=12, eps0=0.02, seed=77),
                      n_windows=W, rows=rows)
    for w in range(W):
        x, y, _ = m.synth_window(5, w, rows)
        other.set_window_data(w, x, y, global_window=10 + w)
    with pytest.raises(m.McmcError):
        other.load_checkpoint(path)
    # export: raw samples + JSON side file
    prefix = str(tmp_path / "out")
    c.export_samples(prefix)
    raw = np.fromfile(prefix + ".samples.f32", np.float32).reshape(W, 8, c.P)
    assert np.array_equal(raw[1], c.get_samples(1))
    import json
    meta = json.load(open(prefix + ".json"))
    assert meta["shape"] == [W, 8, c.P] and len(meta["trace"]) == W and meta["windows"][0]["iterations"] == 12


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("shape", [(58368, 40), (1048576, 128)])
def test_full_size_additivity_over_row_blocks(built, prec, shape):
    """Size-independent property at the full BASELINE sizes, where the CPU oracle would take minutes:
    the likelihood part of log p and of the gradient is a sum over rows, so evaluating two row blocks
    separately and adding must give the evaluation of the whole window.  A row's contribution does not
    depend on the partition in either precision, so the tolerance is FP32 summation error."""
    m, _ = built
    rows, Hw = shape
    Pw = 22 * Hw + 2 * Hw + 1
    x, y, _ = m.synth_window(17, 3, rows, H=Hw)
    w = _w(4, 0.1, Pw)
    cfg = m.baseline_config(H=Hw, precision=prec)

    def ev(xb, yb):
        ctx = m.Context(cfg, n_windows=1, rows=xb.shape[0])
        ctx.set_window_data(0, xb, yb)
        out = ctx.potential_and_grad(0, w)
        ctx.close()
        return out

    cut = rows // 2 + 77  # not a multiple of the tile size
    full, a, b = ev(x, y), ev(x[:cut], y[:cut]), ev(x[cut:], y[cut:])
    # the prior (gradient -w / s^2, s = 1 in this preset) is in every evaluation once
    prior_grad = -w
    lik_full = full["grad"] - prior_grad
    lik_sum = (a["grad"] - prior_grad) + (b["grad"] - prior_grad)
    scale = np.abs(lik_full).max()
    assert np.abs(lik_full - lik_sum).max() <= 2e-5 * scale
    assert abs(full["loglik"] - (a["loglik"] + b["loglik"])) <= 1e-6 * abs(full["loglik"])
    assert full["logprior"] == a["logprior"] == b["logprior"]


def test_multistep_launch_matches_per_step_launches(built, monkeypatch):
    """One window in TF32 mode runs the L leapfrog steps of an iteration as ONE cooperative launch (grid
    barrier + cross-CTA sum inside the kernel).  The same chain with one launch per step must agree: same
    accept decisions, states equal up to the order of the cross-CTA sums."""
    m, O = built
    rows, n_iter = 58368, 12
    x, y, _ = m.synth_window(41, 0, rows)
    x = x * np.float32(0.05)

    def run():
        cfg = m.reference_config(precision=m.PREC_TF32, leapfrog_steps=10, burn_in=0, adapt_steps=8,
                                 sample_capacity=n_iter, trace_iters=n_iter, seed=7, eps0=0.02)
        ctx = m.Context(cfg, n_windows=1, rows=rows)
        ctx.set_window_data(0, x, y)
        n0 = ctx.launch_count(reset=True)
        ctx.run_chain(n_iter)
        out = (ctx.get_samples(0), ctx.get_trace(0), ctx.chain_info(0), ctx.launch_count())
        ctx.close()
        return out

    monkeypatch.setenv("MCMC_B200_MULTISTEP", "1")
    monkeypatch.delenv("MCMC_B200_NO_MULTISTEP", raising=False)
    s_multi, t_multi, i_multi, l_multi = run()
    monkeypatch.delenv("MCMC_B200_MULTISTEP")
    monkeypatch.setenv("MCMC_B200_NO_MULTISTEP", "1")
    s_step, t_step, i_step, l_step = run()
    assert l_multi < l_step  # 2 launches per iteration instead of 21
    assert i_multi == i_step
    assert np.array_equal(t_multi["accepted"], t_step["accepted"])
    assert 0 < t_multi["accepted"].sum()
    assert np.allclose(t_multi["log_acpt"], t_step["log_acpt"], rtol=1e-3, atol=1e-3)
    assert np.abs(s_multi - s_step).max() <= 1e-4 * np.abs(s_step).max()
    # and against the oracle with the device's draws
    ref = O.hmc_chain(O.reference_model(tf32=True), O.Sampler(10, 8, 0.02, 0.2, 0.1, 0.01), x, y,
                      t_multi["momenta"], t_multi["log_u"])
    clear = np.abs(ref["log_acpt"] - t_multi["log_u"]) > 0.05
    assert np.array_equal(ref["accepted"][clear], t_multi["accepted"][clear])


@pytest.mark.parametrize("prec", [0, 1])
def test_ragged_sizes_sweep(built, prec):
    """Seeded sweep over window counts and ragged row counts (tile edges, fewer tiles than CTAs, more
    windows than fit one launch slot each): the batched per-call gradient of every window against the
    oracle, the free partition (slices = 0) against a fixed one, and two short chains for determinism."""
    m, O = built
    rng = np.random.default_rng(20241)
    model = O.baseline_model(tf32=bool(prec))
    tol = TOL[prec]
    cases = [(1, 1), (2, 127), (3, 128), (2, 129), (5, 383), (7, 385), (4, 1027), (9, 2049), (160, 200)]
    cases += [(int(rng.integers(1, 7)), int(rng.integers(1, 6000))) for _ in range(6)]
    for W, rows in cases:
        data = [m.synth_window(13, g, rows) for g in range(W)]
        w = _w(rows + W)
        outs = []
        for slices in (0, 3):
            ctx = m.Context(m.baseline_config(precision=prec, slices=slices, sample_capacity=3), n_windows=W,
                            rows=rows)
            for i, (x, y, _) in enumerate(data):
                ctx.set_window_data(i, x, y, global_window=i)
            got = [ctx.potential_and_grad(i, w) for i in (0, W - 1)]
            ctx.run_chain(3)
            outs.append((got, ctx.get_samples(W - 1).copy()))
            ctx.run_chain(0)
            ctx.close()
        for i, widx in enumerate((0, W - 1)):
            ref = O.logp_grad(model, data[widx][0], data[widx][1], w)
            for got, _ in outs:
                assert _grad_err(got[i]["grad"], ref["grad"]) < tol, (W, rows)
                assert abs(got[i]["loglik"] - ref["loglik"]) <= tol * abs(ref["loglik"]) + 1e-6, (W, rows)
        # the partition changes the summation order only
        assert np.abs(outs[0][1] - outs[1][1]).max() <= 1e-4 * max(1e-3, np.abs(outs[1][1]).max()), (W, rows)


def test_bounded_wait_runs_out_into_a_status_code_and_the_context_stays_usable(built):
    """A device-side wait that nothing ever satisfies returns by itself after its limit, the context
    reports MCMC_B200_ERR_TIMEOUT once, and the same context then evaluates a gradient correctly."""
    m, O = built
    rows = 3000
    x, y, _ = m.synth_window(4, 0, rows)
    w = _w(9)
    for prec in (0, 1):
        ctx = m.Context(m.baseline_config(precision=prec), n_windows=1, rows=rows)
        ctx.set_window_data(0, x, y)
        before = ctx.potential_and_grad(0, w)
        code, msg = ctx.selftest_wait_timeout(limit_us=1000)
        assert code == 4 and "901" in msg, (code, msg)
        ctx.synchronize()  # the status word was cleared: no second report
        after = ctx.potential_and_grad(0, w)
        assert np.array_equal(before["grad"], after["grad"]) and before["loglik"] == after["loglik"]
        ref = O.logp_grad(O.baseline_model(tf32=bool(prec)), x, y, w)
        assert _grad_err(after["grad"], ref["grad"]) < TOL[prec]
        ctx.run_chain(2)
        assert ctx.chain_info(0)["iterations"] == 2
        ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_mcmc_step_sees_a_dataset_overwritten_in_place_after_rebind(built, prec):
    """mcmc_step recognises its dataset by the two pointers.  Refilling the same buffers with another
    window must be announced with rebind_data(); without it the old repacked copy is used (documented)."""
    import torch
    m, O = built
    rows, eps = 2048, 1e-3
    cfg, model = _presets(m, O, prec)["baseline"]
    dev = torch.device("cuda:0")
    xa, ya, _ = m.synth_window(2, 0, rows)
    xb, yb, _ = m.synth_window(2, 1, rows)
    tx, ty = torch.from_numpy(xa).to(dev), torch.from_numpy(ya).to(dev)
    w0 = _w(3)
    zero = np.zeros(P, np.float32)
    t = {k: torch.from_numpy(v).to(dev) for k, v in dict(wp=w0, mp=zero, gp=zero).items()}
    out = {k: torch.zeros(P, device=dev) for k in ("wn", "mn", "gc", "gn")}
    loss = torch.zeros(rows + P, device=dev)
    ctx = m.Context(cfg, n_windows=1, rows=rows)
    s = torch.cuda.current_stream().cuda_stream

    def step():
        ctx.mcmc_step(tx.data_ptr(), ty.data_ptr(), t["wp"].data_ptr(), out["wn"].data_ptr(),
                      t["mp"].data_ptr(), out["mn"].data_ptr(), t["gp"].data_ptr(), out["gc"].data_ptr(),
                      out["gn"].data_ptr(), loss.data_ptr(), 1, 0.0, stream=s)
        torch.cuda.synchronize()
        return out["gc"].cpu().numpy().copy()

    ga = step()
    tx.copy_(torch.from_numpy(xb))
    ty.copy_(torch.from_numpy(yb))
    torch.cuda.synchronize()
    assert np.array_equal(step(), ga)        # same pointers, no rebind: still the first window
    ctx.rebind_data()
    gb = step()
    ra, rb = O.logp_grad(model, xa, ya, w0), O.logp_grad(model, xb, yb, w0)
    assert _grad_err(ga, ra["grad"]) < TOL[prec] and _grad_err(gb, rb["grad"]) < TOL[prec]
    assert _grad_err(gb, ra["grad"]) > 100 * TOL[prec]
    ctx.close()


def test_reset_chain_restarts_the_same_chain(built):
    """reset_chain drops the captured iteration graph and restarts at w = 0: the same samples again."""
    m, _ = built
    rows, n_iter = 3000, 6
    x, y, _ = m.synth_window(6, 0, rows)
    for prec in (0, 1):
        ctx = m.Context(m.baseline_config(precision=prec, sample_capacity=n_iter, seed=11), n_windows=1, rows=rows)
        ctx.set_window_data(0, x, y)
        ctx.run_chain(n_iter)
        first = ctx.get_samples(0).copy()
        ctx.reset_chain()
        ctx.run_chain(n_iter)
        assert np.array_equal(first, ctx.get_samples(0))
        ctx.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_reference_random_streams_mode(built, prec):
    """cfg.rng_streams = RNG_REFERENCE: the chain is driven by the reference's own streams (Thrust minstd_rand
    + normal_distribution on the device for the momenta, libstdc++ minstd_rand0 + uniform_real_distribution
    + log on the host for the accept draw, include/mcmc/main.h:207-216, 235-239, with its bookkeeping of 962
    draws per iteration).  The trace must hold exactly those draws, every window gets the same ones, and
    the CPU replay with them takes the same decisions."""
    from scipy.special import ndtr
    m, O = built
    rows, n_iter, seed, W = 4096, 14, 5, 2
    cfg = m.reference_config(precision=prec, leapfrog_steps=10, burn_in=0, adapt_steps=8, sample_capacity=n_iter,
                             trace_iters=n_iter, seed=seed, eps0=0.2, rng_streams=m.RNG_REFERENCE)
    ctx = m.Context(cfg, n_windows=W, rows=rows)
    data = []
    for w in range(W):
        x, y, _ = m.synth_window(9, w, rows)
        data.append((x * np.float32(0.05), y))
        ctx.set_window_data(w, data[w][0], y, global_window=100 + w)
    ctx.run_chain(5)
    ctx.run_chain(n_iter - 5)       # the second call continues the streams where the first stopped
    L = m.lib()
    tr = [ctx.get_trace(w) for w in range(W)]
    assert np.array_equal(tr[0]["momenta"], tr[1]["momenta"]) and np.array_equal(tr[0]["log_u"], tr[1]["log_u"])
    for it in range(n_iter):
        dev = ctx.refstream_momentum_device(seed + 962 * it, P)
        assert np.array_equal(tr[0]["momenta"][it], dev), it
        assert tr[0]["log_u"][it] == np.float32(L.mcmc_b200_refstream_log_uniform(seed + 962 * it + 961)), it
    # the normal draw is the inverse normal CDF of ONE engine value: its CDF gives back the engine's
    # value scaled to (0,1) (or its complement), and the draws are standard normal
    n0 = 12345
    v = ctx.refstream_momentum_device(n0, 2000)
    u = np.array([L.mcmc_b200_refstream_engine(n0 + i) for i in range(2000)], np.float64) / 2147483647.0
    c = ndtr(v.astype(np.float64))
    assert min(np.abs(c - u).max(), np.abs(c - (1.0 - u)).max()) < 1e-5
    big = ctx.refstream_momentum_device(0, 4096)
    assert abs(big.mean()) < 0.06 and abs(big.std() - 1.0) < 0.05
    model = O.reference_model(tf32=bool(prec))
    for w in range(W):
        ref = O.hmc_chain(model, O.Sampler(10, 8, 0.2, 0.2, 0.1, 0.01), data[w][0], data[w][1], tr[w]["momenta"],
                          tr[w]["log_u"])
        clear = np.abs(ref["log_acpt"] - tr[w]["log_u"]) > (0.0 if prec == 0 else 0.05)
        assert np.array_equal(ref["accepted"][clear], tr[w]["accepted"][clear]), w
    ctx.close()


@pytest.mark.parametrize("Hw", [40, 128])
def test_forward_only_pass_over_samples_ragged_sizes(built, Hw):
    """predict_mean / final_loss (one forward-only launch over samples x rows) at sizes that are no multiple
    of its 512-row tiles or of its sample chunks, for both widths, against the oracle's forward pass."""
    m, O = built
    rows, n_iter, n_pred = 1531, 7, 777
    x, y, _ = m.synth_window(12, 0, rows, H=Hw)
    cfg = m.baseline_config(H=Hw, sample_capacity=n_iter, seed=3, eps0=2e-4)
    ctx = m.Context(cfg, n_windows=2, rows=rows)
    ctx.set_window_data(0, x, y, global_window=0)
    x1, y1, _ = m.synth_window(12, 1, rows, H=Hw)
    ctx.set_window_data(1, x1, y1, global_window=1)
    ctx.run_chain(n_iter)
    model = O.baseline_model(H=Hw)
    xs, _, _ = m.synth_window(12, 5, n_pred, H=Hw)
    for w, (xw, yw) in enumerate(((x, y), (x1, y1))):
        smp = ctx.get_samples(w)
        for first, count in ((0, n_iter), (2, 3), (6, 1)):
            got = ctx.predict_mean(w, xs, first, count)
            exp = O.predict_mean(model, xs, smp[first:first + count])
            assert np.abs(got - exp).max() <= 1e-5 * max(1.0, np.abs(exp).max()), (w, first, count)
            ll, lp = ctx.final_loss(w, first, count)
            ell, elp = O.final_loss(model, xw, yw, smp[first:first + count])
            assert abs(ll - ell) <= 1e-5 * abs(ell) and abs(lp - elp) <= 1e-5 * max(1.0, abs(elp)), (w, first, count)
    ctx.close()
