"""The multi-rank host logic on CPU ranks (gloo, world size 2): window blocks
cover every window exactly once, and a row-sharded evaluation (each rank its
rows, one all-reduce of P+1 doubles, prior added once after it) equals the
unsharded one — the arithmetic the NCCL path performs on the GPUs."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import mcmc_bnn_example_b200 as m
    import oracle as O
    from mcmc_bnn_example_b200.sharding import row_block, window_block

    # windows: every global window on exactly one rank
    w0, w1 = window_block(rank, world, 201)
    mine = torch.zeros(201, dtype=torch.int32)
    mine[w0:w1] = 1
    dist.all_reduce(mine)
    assert bool((mine == 1).all())

    # rows of one window: partial sums, all-reduce, prior once
    rows, P = 3001, 961
    x, y, _ = m.synth_window(3, 0, rows)
    w = (0.2 * np.random.default_rng(1).standard_normal(P)).astype(np.float32)
    model = O.baseline_model()
    r0, r1 = row_block(rank, world, rows)
    part = O.logp_grad(model, x, y, w, rows=(r0, r1), add_prior=False)
    buf = torch.from_numpy(np.concatenate([part["grad"], [part["loglik"]]]))
    dist.all_reduce(buf)
    full = O.logp_grad(model, x, y, w)
    prior = O.logp_grad(model, x[:1], y[:1], w, rows=(0, 0), add_prior=True)  # prior terms only
    grad = buf[:P].numpy() + prior["grad"]
    assert np.allclose(grad, full["grad"], rtol=1e-12, atol=1e-12)
    assert abs(float(buf[P]) - full["loglik"]) < 1e-9 * abs(full["loglik"])
    # identical inputs on every rank => identical accept decision without a broadcast
    la = torch.tensor([float(buf[P]) + prior["logprior"]], dtype=torch.float64)
    lo, hi = la.clone(), la.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    assert float(lo) == float(hi)
    open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
    dist.destroy_process_group()


def test_window_and_row_sharding_on_two_cpu_ranks(tmp_path, built):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
