"""The allocation-free entry point against the regular one.

mcmc_b200_potential_and_grad_static exists for hosts that may not call
cudaMalloc while they evaluate the model (all GPU memory owned by the host's own
arena; loops where the allocator's device-wide synchronisation is not allowed).
Its scratch is a fixed array inside the library image, shared by every call on a
GPU, so two calls in a row must both be right: nothing may depend on what the
previous call left behind.  This file sorts last on purpose: a run that stops at
the first failure has then already run every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

P = 961


@pytest.mark.parametrize("preset", ["baseline", "reference"])
def test_static_scratch_entry_matches_regular_entry_twice_in_a_row(built, preset):
    import torch
    m, O = built
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    cfg = m.baseline_config() if preset == "baseline" else m.reference_config()
    model = O.baseline_model() if preset == "baseline" else O.reference_model()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back, the larger one first, so that stale scratch would show
    for call, (rows, seed) in enumerate([(58368, 3), (4097, 4)]):
        x, y, _ = m.synth_window(17, seed, rows)
        w = (0.2 * np.random.default_rng(seed).standard_normal(P)).astype(np.float32)
        ctx = m.Context(cfg, n_windows=1, rows=rows)
        ctx.set_window_data(0, x, y)
        ref = ctx.potential_and_grad(0, w)
        ctx.close()
        tx, ty, tw = (torch.from_numpy(a).to(dev) for a in (x, y, w))
        grad = torch.full((P,), float("nan"), device=dev)
        scal = torch.full((2,), float("nan"), device=dev, dtype=torch.float64)
        torch.cuda.synchronize()
        m.potential_and_grad_static(cfg, tx.data_ptr(), ty.data_ptr(), rows, tw.data_ptr(), grad.data_ptr(),
                                    scal.data_ptr(), stream)
        torch.cuda.synchronize()
        g = grad.cpu().numpy()
        ll, lp = scal.cpu().numpy()
        assert np.abs(g - ref["grad"]).max() <= 1e-5 * np.abs(ref["grad"]).max(), (call, rows)
        assert abs(ll - ref["loglik"]) <= 1e-5 * abs(ref["loglik"])
        assert abs(lp - ref["logprior"]) <= 1e-6 * abs(ref["logprior"])
        if rows == 4097:  # and against the CPU oracle directly, at a size it finishes at once
            exact = O.logp_grad(model, x, y, w)
            assert np.abs(g - exact["grad"]).max() <= 1e-5 * np.abs(exact["grad"]).max()
            assert abs(ll - exact["loglik"]) <= 1e-5 * abs(exact["loglik"])
            assert abs(lp - exact["logprior"]) <= 1e-6 * abs(exact["logprior"])


def test_static_scratch_entry_alternating_datasets_without_host_synchronisation(built):
    """Many calls queued back to back on one stream, alternating between two datasets of different
    sizes, with no host synchronisation in between: every call repacks into the shared array right
    before its gradient kernel reads it, so each result must be its own dataset's, never the previous
    call's rows."""
    import torch
    m, _ = built
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    cfg = m.baseline_config()
    stream = torch.cuda.current_stream().cuda_stream
    sets, refs = [], []
    for rows, seed in ((9000, 1), (5000, 2)):
        x, y, _ = m.synth_window(23, seed, rows)
        w = (0.2 * np.random.default_rng(seed).standard_normal(P)).astype(np.float32)
        ctx = m.Context(cfg, n_windows=1, rows=rows)
        ctx.set_window_data(0, x, y)
        refs.append(ctx.potential_and_grad(0, w))
        ctx.close()
        sets.append((rows,) + tuple(torch.from_numpy(a).to(dev) for a in (x, y, w)))
    n_calls = 40
    grads = torch.zeros((n_calls, P), device=dev)
    scal = torch.zeros((n_calls, 2), device=dev, dtype=torch.float64)
    torch.cuda.synchronize()
    for i in range(n_calls):
        rows, tx, ty, tw = sets[i & 1]
        m.potential_and_grad_static(cfg, tx.data_ptr(), ty.data_ptr(), rows, tw.data_ptr(),
                                    grads[i].data_ptr(), scal[i].data_ptr(), stream)
    torch.cuda.synchronize()
    g, sc = grads.cpu().numpy(), scal.cpu().numpy()
    for i in range(n_calls):
        ref = refs[i & 1]
        assert np.abs(g[i] - ref["grad"]).max() <= 1e-5 * np.abs(ref["grad"]).max(), i
        assert abs(sc[i, 0] - ref["loglik"]) <= 1e-5 * abs(ref["loglik"]), i


def test_static_scratch_entry_refuses_what_does_not_fit(built):
    import torch
    m, _ = built
    dev = torch.device("cuda:0")
    t = torch.zeros(8, device=dev)
    d = torch.zeros(2, device=dev, dtype=torch.float64)
    with pytest.raises(m.McmcError) as e:
        m.potential_and_grad_static(m.baseline_config(), t.data_ptr(), t.data_ptr(), 65537, t.data_ptr(),
                                    t.data_ptr(), d.data_ptr())
    assert "max 65536" in str(e.value)
    with pytest.raises(m.McmcError):
        m.potential_and_grad_static(m.baseline_config(precision=m.PREC_TF32), t.data_ptr(), t.data_ptr(), 8,
                                    t.data_ptr(), t.data_ptr(), d.data_ptr())
