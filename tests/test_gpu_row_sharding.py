"""Row sharding of one window over two GPUs (one process per GPU; the gradient
partials are all-reduced each leapfrog step either by NCCL or by the library's
one-shot all-reduce over peer memory) gives the chain the unsharded window gives.  Needs two GPUs; NVLS is switched off for the children
(a rank that leaves while its memory is bound to an in-switch reduction group can fault
the other ranks' GPUs)."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
import mcmc_bnn_example_b200 as m
from mcmc_bnn_example_b200.sharding import row_block
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")
rows, n_iter, prec = 58368, 6, int(sys.argv[1])
x, y, _ = m.synth_window(4, 0, rows)
uid = [m.nccl_unique_id() if rank == 0 else None]
dist.broadcast_object_list(uid, src=0)
r0, r1 = row_block(rank, world, rows)
cfg = m.baseline_config(precision=prec, sample_capacity=n_iter, trace_iters=n_iter, seed=11, eps0=2e-4)
ctx = m.Context(cfg, n_windows=1, rows=r1 - r0, device=rank)
ctx.enable_row_sharding(uid[0], rank, world)
if sys.argv[3] == "oneshot":
    ctx.enable_oneshot_allreduce()
ctx.set_window_data(0, x[r0:r1], y[r0:r1], global_window=0)
ctx.run_chain(n_iter)
np.save(sys.argv[2] + "/samples%%d.npy" %% rank, ctx.get_samples(0))
np.save(sys.argv[2] + "/acc%%d.npy" %% rank, ctx.get_trace(0)["accepted"])
ctx.close()
dist.barrier()
dist.destroy_process_group()
'''


@pytest.mark.parametrize("allreduce", ["nccl", "oneshot"])
@pytest.mark.parametrize("prec", [0, 1])
def test_two_gpu_row_sharded_chain_matches_single_gpu(built, tmp_path, prec, allreduce):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    m, _ = built
    script = tmp_path / "child.py"
    script.write_text(CHILD % {"root": ROOT})
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1",
               MASTER_PORT=str(29600 + os.getpid() % 1000), WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), str(prec), str(tmp_path), allreduce],
                              env=dict(env, RANK=str(r))) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    s0, s1 = np.load(tmp_path / "samples0.npy"), np.load(tmp_path / "samples1.npy")
    assert np.array_equal(s0, s1)  # every rank holds the same chain
    assert np.array_equal(np.load(tmp_path / "acc0.npy"), np.load(tmp_path / "acc1.npy"))
    rows, n_iter = 58368, 6
    x, y, _ = m.synth_window(4, 0, rows)
    cfg = m.baseline_config(precision=prec, sample_capacity=n_iter, trace_iters=n_iter, seed=11, eps0=2e-4)
    ctx = m.Context(cfg, n_windows=1, rows=rows)
    ctx.set_window_data(0, x, y)
    ctx.run_chain(n_iter)
    single = ctx.get_samples(0)
    assert np.array_equal(ctx.get_trace(0)["accepted"], np.load(tmp_path / "acc0.npy"))
    tol = 1e-5 if prec == 0 else 2e-3
    assert np.abs(single - s0).max() <= tol * max(np.abs(single).max(), 1e-6)
    ctx.close()


def test_oneshot_allreduce_wait_is_bounded(built):
    """One GPU: the context plays rank 0 of 2 and the other rank never sends.  The wait inside the
    all-reduce kernel runs out after its poll limit, the kernel returns by itself, the call reports
    MCMC_B200_ERR_TIMEOUT, and the context then works as an ordinary unsharded one."""
    m, O = built
    rows = 3000
    x, y, _ = m.synth_window(4, 0, rows)
    w = (0.15 * np.random.default_rng(9).standard_normal(961)).astype(np.float32)
    ctx = m.Context(m.baseline_config(precision=m.PREC_TF32, sample_capacity=4), n_windows=1, rows=rows)
    ctx.set_window_data(0, x, y)
    code, msg = ctx.selftest_oneshot_timeout(polls=2000)
    assert code == 4 and "501" in msg, (code, msg)
    got = ctx.potential_and_grad(0, w)
    ref = O.logp_grad(O.baseline_model(tf32=True), x, y, w)
    assert np.abs(got["grad"] - ref["grad"]).max() <= 2e-3 * np.abs(ref["grad"]).max()
    ctx.run_chain(3)
    assert ctx.chain_info(0)["iterations"] == 3
    ctx.close()
