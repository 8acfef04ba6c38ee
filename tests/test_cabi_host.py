"""CPU-only checks of the product library: it loads, exports everything the
header declares, fails loudly without a GPU, and its host-side pieces (Philox
streams, synthetic window generator) behave."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    hdr = open(os.path.join(ROOT, "include", "mcmc_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(mcmc_b200_[a-z0-9_]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol(built):
    m, _ = built
    lib = C.CDLL(m.LIB_PATH)
    names = _declared()
    assert len(names) >= 28
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert set(m.EXPORTS) == set(names)


def test_config_presets_match_reference_constants(built):
    m, _ = built
    # include/mcmc/global_params.h:27-58
    r = m.reference_config()
    assert (r.D, r.H, r.likelihood, r.leapfrog_steps, r.burn_in, r.adapt_steps, r.sample_capacity) == \
        (22, 40, m.LIK_STUDENT_T, 1000, 100, 100, 800)
    assert (r.lik_scale, r.lik_df, r.prior_scale, r.eps0, r.target_rate, r.decrement, r.increment) == \
        (100.0, 2.2, 200.0, 0.01, 0.2, 0.1, 0.01)
    b = m.baseline_config()
    assert (b.likelihood, b.lik_scale, b.prior_scale, b.leapfrog_steps, b.eps0) == \
        (m.LIK_GAUSSIAN, 1.0, 1.0, 10, 1e-3)


def test_no_gpu_means_a_loud_error_not_a_fallback(built):
    m, _ = built
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(m.McmcError) as e:
        m.Context(m.baseline_config(), n_windows=1, rows=128)
    assert "no CPU path" in str(e.value)


def test_philox_known_answers(built):
    m, _ = built
    # Philox4x32-10 known-answer vectors of the Random123 distribution (kat_vectors)
    assert m.philox_raw([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert m.philox_raw([0xffffffff] * 4, [0xffffffff] * 2) == \
        [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert m.philox_raw([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_philox_normal_stream_statistics(built):
    m, _ = built
    f = m.lib().mcmc_b200_philox_normal
    v = np.array([f(123, 5, 9, 0, i) for i in range(20000)])
    assert abs(v.mean()) < 0.03 and abs(v.std() - 1) < 0.03
    assert abs(np.mean(v ** 3)) < 0.1 and abs(np.mean(v ** 4) - 3) < 0.25
    # keyed by window / iteration / stream
    assert f(123, 5, 9, 0, 0) != f(123, 6, 9, 0, 0) != f(123, 5, 10, 0, 0)
    assert f(123, 5, 9, 0, 7) == f(123, 5, 9, 0, 7)


def test_synthetic_window_is_deterministic_and_teacher_consistent(built):
    m, O = built
    x, y, t = m.synth_window(42, 3, 5000)
    x2, y2, t2 = m.synth_window(42, 3, 5000)
    assert np.array_equal(x, x2) and np.array_equal(y, y2) and np.array_equal(t, t2)
    xo, _, _ = m.synth_window(42, 4, 5000)
    assert not np.array_equal(x, xo)
    # a prefix of the same window is the same data (index-keyed streams)
    xp, yp, _ = m.synth_window(42, 3, 1000)
    assert np.array_equal(xp, x[:1000]) and np.array_equal(yp, y[:1000])
    assert abs(x.mean()) < 0.02 and abs(x.std() - 1) < 0.02
    assert abs(t.std() - 0.3) < 0.03
    # y = teacher(x) + N(0, 0.05^2)
    pred = O.predict_mean(O.baseline_model(), x, t[None, :])
    resid = y - pred
    assert abs(resid.std() - 0.05) < 0.005 and abs(resid.mean()) < 0.005


def test_read_table_matches_a_plain_parse(tmp_path):
    """The reference's dataset layout (io.h:42-80 there): 149 header tokens, rows of 149 tokens =
    2 ignored + label + 22 features + rest ignored.  Host-only: runs without a GPU."""
    import mcmc_bnn_example_b200 as m
    m.build()
    rng = np.random.default_rng(3)
    rows, total, skip, D = 37, 149, 2, 22
    table = rng.standard_normal((rows, total)) * 10.0
    path = tmp_path / "returns_and_features_for_mcmc.txt"
    with open(path, "w") as f:
        f.write(" ".join("col%d" % j for j in range(total)) + "\n")
        for i in range(rows):
            toks = ["%.9g" % v for v in table[i]]
            toks[0] = "2019-01-%02d" % (i % 28 + 1)      # the skipped columns need not be numbers
            toks[1] = "TICK%d" % i
            f.write(("\t" if i % 2 else " ").join(toks) + "\n")
    x, y = m.read_table(str(path), rows)
    want_y = table[:, skip].astype(np.float32)
    want_x = (table[:, skip + 1:skip + 1 + D].astype(np.float32) * np.float32(0.001)).astype(np.float32)
    # the file holds 9 significant digits: the parse may differ from the float32 of the double by one ulp
    assert np.allclose(y, want_y, rtol=2e-7, atol=0)
    assert np.allclose(x, want_x, rtol=3e-7, atol=0)
    # fewer rows than asked for, and a missing file, are errors with a message (the reference aborts)
    with pytest.raises(m.McmcError, match="row 37"):
        m.read_table(str(path), rows + 1)
    with pytest.raises(m.McmcError, match="cannot open"):
        m.read_table(str(tmp_path / "nope.txt"), 1)


@pytest.mark.parametrize("slices", [0, 3])
def test_work_partition_covers_every_tile_once_and_is_balanced(slices):
    """The persistent kernels' work table (host arithmetic): every (window, tile) is owned by exactly one
    CTA, a CTA's segments are contiguous in the flattened order, slots number a window's pieces 0..k-1,
    and with the free partition no CTA costs more than equal tile counts would cost the worst CTA."""
    import mcmc_bnn_example_b200 as m
    m.build()
    seg_cost = 8.0
    for W, tpw, G in [(1, 456, 148), (25, 456, 148), (200, 456, 148), (64, 8192, 148), (3, 24, 148), (7, 3, 148),
                      (5, 1, 148), (148, 1, 148), (149, 2, 148), (2, 1000, 7)]:
        plan = m.plan_work_table(W, tpw, G, slices)
        assert 1 <= len(plan) <= G
        owned = np.zeros((W, tpw), np.int32)
        slots = [[] for _ in range(W)]
        costs = []
        flat_pos = 0
        for cta in plan:
            assert cta, "a CTA of the table owns at least one segment"
            tiles = 0
            for (w, t0, t1, slot) in cta:
                assert 0 <= w < W and 0 <= t0 < t1 <= tpw
                owned[w, t0:t1] += 1
                slots[w].append(slot)
                tiles += t1 - t0
                if slices == 0:  # contiguous in the flattened (window, tile) order
                    assert w * tpw + t0 == flat_pos
                    flat_pos = w * tpw + t1
            costs.append(tiles + seg_cost * len(cta))
        assert np.all(owned == 1)
        for w in range(W):
            assert sorted(slots[w]) == list(range(len(slots[w])))
            if slices:
                assert len(slots[w]) == min(slices, tpw)
        if slices == 0:
            T = W * tpw
            n = min(G, T)
            even_tiles = -(-T // n)
            worst_segments = (even_tiles + tpw - 2) // tpw + 1  # windows an even range can touch
            assert max(costs) <= even_tiles + seg_cost * worst_segments + 1e-9


def test_reference_stream_engines_are_the_published_generators():
    """The reference draws its momenta from Thrust's default engine (minstd_rand, multiplier 48271) and its
    accept uniforms from libstdc++'s (minstd_rand0, multiplier 16807), both modulo 2^31 - 1 (Park-Miller;
    the reference's include/mcmc/main.h:207-216, 235-239).  The C++ standard pins the 10000th value of
    both engines seeded with 1; the library calls the engines themselves, this checks the plumbing
    around them against a three-line restatement of the recurrence."""
    import mcmc_bnn_example_b200 as m
    L = m.lib()

    def lcg(a, x, n):
        for _ in range(n):
            x = x * a % 2147483647
        return x

    assert L.mcmc_b200_refstream_engine(9999) == 399268537      # minstd_rand, [rand.predef]
    assert lcg(16807, 1, 10000) == 1043618065                   # minstd_rand0, [rand.predef]
    for n in (0, 1, 961, 962 * 50 + 17, 962 * 900):
        assert L.mcmc_b200_refstream_engine(n) == lcg(48271, 1, n + 1)
    for seed in (1, 2, 961, 962 * 7 + 961, 2 ** 31 + 5):
        s0 = seed % 2147483647 or 1                             # seed 0 (mod m) is mapped to 1
        x = lcg(16807, s0, 1)
        assert L.mcmc_b200_refstream_engine0(seed) == x
        # U(FLT_MIN, 1) from one engine value, log in double, narrowed to float (main.h:235-239)
        u = (x - 1) / 2147483646.0
        lu = L.mcmc_b200_refstream_log_uniform(seed)
        assert abs(lu - np.log(max(u, 1.2e-38))) <= 2e-6 * max(1.0, abs(lu)), (seed, lu, np.log(u))
