"""CPU tests of the period search and codebook machinery.

Model: reference tests/test_partitioning_quantization_cpu.py,
tests/test_codebook_indices_parity.py, tests/test_dequant_indices_parity.py.
"""
import math

import numpy as np
import pytest
import torch

from gefen_x_b200.quant import codebook as C
from gefen_x_b200.quant import partitioning as P


def test_divisors_proper_and_sorted():
    assert P.divisors(12) == [1, 2, 3, 4, 6]
    assert P.divisors(7) == [1]
    assert P.divisors(1) == []
    assert P.divisors(16) == [1, 2, 4, 8]


def test_block_variance_matches_numpy():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(240) ** 2
    for p in P.divisors(240):
        want = math.sqrt(x.reshape(-1, p).var(axis=1).mean())
        got = P.average_within_block_variance_cpu(x, p)
        assert abs(want - got) < 1e-12


def test_period_search_matches_direct_statement():
    """find_period == argmin over divisors of err[p] - err[previous p], computed directly."""
    rng = np.random.default_rng(3)
    for n in (96, 360, 1024):
        g2 = rng.standard_normal(n) ** 2
        divs = P.divisors(n)
        errs = [math.sqrt(g2.reshape(-1, p).var(axis=1).mean()) for p in divs]
        scores = [1e-12] + [errs[i] - errs[i - 1] for i in range(1, len(errs))]
        best = min(zip(scores, divs))[1]
        want = 1 if best < 8 else best
        if want == 1:
            want = P.memory_safe_fallback_period(n, (n,))
        got = P.find_period_by_block_variance(torch.from_numpy(g2), print_results=False,
                                              parameter_shape=(n,), backend="cpu")
        assert got == want


def test_small_winner_collapses_and_fallback():
    # a flat curve has no structure: the winner is tiny -> 1 -> memory-safe fallback
    assert P.select_period([(1, 0.5), (2, 0.5), (4, 0.5)]) == 1
    assert P.memory_safe_fallback_period(4096 * 64, (4096, 64)) == 2048
    assert P.memory_safe_fallback_period(4096 * 4096, (4096, 4096)) == 4096
    assert P.memory_safe_fallback_period(7, (7,)) == 1
    assert P.memory_safe_fallback_period(2560, (2560,)) == 1280
    old = P.MEMORY_SAFE_FALLBACK
    try:
        P.MEMORY_SAFE_FALLBACK = False
        x = torch.ones(64)
        assert P.find_period_by_block_variance(x, print_results=False) == 1
    finally:
        P.MEMORY_SAFE_FALLBACK = old


def test_select_period_tie_prefers_smaller():
    assert P.select_period([(1, 1.0), (8, 0.5), (16, 0.0), (32, -0.5)]) == 8


def _brute_force_kmeans(xs, ws, k):
    """Exhaustive optimal contiguous partition for tiny inputs (endpoints pinned)."""
    import itertools

    n = len(xs)
    best = (float("inf"), None)
    for cuts in itertools.combinations(range(1, n), k - 1):
        b = (0,) + cuts + (n,)
        cost, cents = 0.0, []
        for c in range(k):
            seg_x, seg_w = xs[b[c]:b[c + 1]], ws[b[c]:b[c + 1]]
            if c == 0:
                cen = -1.0
            elif c == k - 1:
                cen = 1.0
            else:
                cen = float((seg_x * seg_w).sum() / seg_w.sum())
            cost += float((seg_w * (seg_x - cen) ** 2).sum())
            cents.append(cen)
        if cost < best[0] - 1e-15:
            best = (cost, cents)
    return best


def test_exact_dp_is_optimal_and_backends_agree():
    rng = np.random.default_rng(1)
    xs = np.sort(rng.uniform(-1, 1, 12)).astype(np.float32)
    ws = rng.integers(1, 20, 12).astype(np.float32)
    stats = {"active_centers": torch.from_numpy(xs), "active_counts": torch.from_numpy(ws)}
    cb = C.exact_dp(stats, 4, True)
    _, cents = _brute_force_kmeans(xs.astype(np.float64), ws.astype(np.float64), 4)
    assert torch.allclose(cb, torch.tensor(sorted(cents), dtype=torch.float32), atol=1e-6)
    # numpy fallback == C++ solver
    w = torch.from_numpy(ws).double()
    x = torch.from_numpy(xs).double()
    pw = torch.cat([torch.zeros(1, dtype=torch.float64), torch.cumsum(w, 0)]).numpy()
    pwx = torch.cat([torch.zeros(1, dtype=torch.float64), torch.cumsum(w * x, 0)]).numpy()
    pwx2 = torch.cat([torch.zeros(1, dtype=torch.float64), torch.cumsum(w * x * x, 0)]).numpy()
    alt = np.sort(C._exact_dp_numpy(pw, pwx, pwx2, 4, True))
    assert np.allclose(alt, cb.numpy(), atol=1e-7)


def test_exact_dp_pads_when_few_points():
    stats = {"active_centers": torch.tensor([-0.5, 0.25]), "active_counts": torch.tensor([3.0, 1.0])}
    cb = C.exact_dp(stats, 8, True)
    assert cb.numel() == 8 and cb[0] == -1.0 and cb[-1] == 1.0
    assert torch.all(cb[1:] >= cb[:-1])


def test_learned_codebook_is_sorted_with_endpoints():
    torch.manual_seed(0)
    g = torch.randn(64, 256) * 1e-3
    cb = C.learn_codebook_from_grad_periods([("w", g.reshape(-1), 256, g)], "cpu")
    assert cb.shape == (256,) and cb.dtype == torch.float32
    assert cb[0] == -1.0 and cb[-1] == 1.0
    assert torch.all(cb[1:] >= cb[:-1])


def test_nearest_index_ties_go_low_and_match_brute_force():
    cb = torch.tensor([-1.0, -0.5, 0.0, 0.5, 1.0])
    v = torch.tensor([-2.0, -0.75, -0.25, 0.25, 0.1, 0.75, 3.0, 0.0])
    got = C.nearest_codebook_indices(cb, v)
    assert got.tolist() == [0, 0, 1, 2, 2, 3, 4, 2]
    torch.manual_seed(1)
    cb = torch.sort(torch.rand(256) * 2 - 1).values
    cb[0], cb[-1] = -1.0, 1.0
    v = torch.rand(5000) * 2.2 - 1.1
    brute = (v[:, None] - cb[None, :]).abs().argmin(dim=1)
    got = C.nearest_codebook_indices(cb, v).long()
    assert torch.equal((v - cb[got]).abs(), (v - cb[brute]).abs())


def test_dequantize_round_trip():
    cb = torch.linspace(-1, 1, 256)
    idx = torch.randint(0, 256, (7, 33), dtype=torch.uint8)
    out = C.dequantize_indices(cb, idx, torch.float32)
    assert torch.equal(out, cb[idx.long()])
    assert torch.equal(C.nearest_codebook_indices(cb, out), idx)


def test_search_lut_brackets_every_value():
    torch.manual_seed(2)
    cb = torch.sort(torch.rand(256) * 2 - 1).values
    cb[0], cb[-1] = -1.0, 1.0
    thr = C.decision_thresholds(cb)
    assert thr.numel() == 255
    lut = C.codebook_search_lut(cb).long()
    assert lut.numel() == C.LUT_BUCKETS + 1 and lut[0] == 0 and lut[-1] == 255
    v = torch.rand(20000) * 2.4 - 1.2
    b = C._bucket(v, C.LUT_BUCKETS)
    ins = torch.bucketize(v, thr)                 # the index the search must return
    assert torch.all(ins >= lut[b]) and torch.all(ins <= lut[b + 1])
    packed = C.packed_search_lut(cb)
    assert packed.dtype == torch.int16 and packed.numel() == C.LUT_BUCKETS
    u = packed.int() & 0xFFFF
    assert torch.equal(u & 0xFF, lut[:-1].int()) and torch.equal(u >> 8, (lut[1:] - lut[:-1]).int())
    pt = C.padded_thresholds(cb)
    assert pt.numel() == 256 and torch.isinf(pt[-1]) and torch.equal(pt[:-1], thr)


def test_histogram_counts_total_and_symmetry():
    g = torch.tensor([1.0, -1.0, 0.5, 0.0, 2.0, -2.0, 0.0, 0.0])
    counts = C.block_normalised_histogram(g, 4)
    assert counts.sum().item() == 8
    assert counts[4095].item() == 2          # +1.0 of each block clamps into the last bin
    assert counts[0].item() == 2             # -1.0


def test_monotone_exact_dp_equals_the_full_scan():
    """The O(n k log n) solver returns the very codebook of the O(n^2 k) scan, ties included."""
    import torch

    from gefen_x_b200.quant import codebook as C

    g = torch.Generator().manual_seed(0)
    samples = [
        (torch.randn(1 << 16, generator=g) * 0.3).clamp(-1, 1),
        torch.rand(1 << 14, generator=g) * 2 - 1,
        torch.cat([torch.zeros(20000), (torch.randn(3000, generator=g) * 0.05).clamp(-1, 1)]),
        (torch.randn(1500, generator=g) * 0.5).clamp(-1, 1),                       # sparse histogram
        torch.cat([(torch.randn(2000, generator=g) * 0.2).clamp(-1, 1)] * 1
                  + [-(torch.randn(2000, generator=torch.Generator().manual_seed(0)) * 0.2).clamp(-1, 1)]),
        torch.randint(0, 400, (8000,), generator=g).float() / 200 - 1,              # few distinct values
    ]
    h = (torch.randn(3000, generator=g) * 0.2).clamp(-1, 1)
    samples.append(torch.cat([h, -h]))                                             # symmetric: exact ties
    for x in samples:
        counts = torch.histc(x, bins=C.HISTOGRAM_BINS, min=-1, max=1).long()
        st = C.histogram_stats_from_counts(counts)
        for k in (256, 16):
            a = C.exact_dp(st, k, method="scan")
            b = C.exact_dp(st, k, method="monotone")
            assert torch.equal(a, b)
    assert C.EXACT_DP_METHOD == "monotone"


def test_bucket_function_is_monotonic_saturating_and_total():
    """The bucket of the search table: rint(sat(x / 2 + 1 / 2) * 16383).  It must never decrease with x
    (the table's bracketing argument rests on that), map everything below -1 to 0 and above 1 to the
    last bucket, and give NaN a bucket (0, like the saturating fma of the kernels)."""
    x = torch.cat([torch.linspace(-1.5, 1.5, 200001), torch.tensor([-1.0, 1.0, 0.0, -0.0, 1e-45, -1e-45,
                                                                  float("inf"), float("-inf")])])
    x = torch.sort(x).values
    b = C._bucket(x, C.LUT_BUCKETS)
    assert int(b.min()) == 0 and int(b.max()) == C.LUT_BUCKETS - 1
    assert bool((b[1:] >= b[:-1]).all())
    assert int(C._bucket(torch.tensor([-1.0]), C.LUT_BUCKETS)) == 0
    assert int(C._bucket(torch.tensor([1.0]), C.LUT_BUCKETS)) == C.LUT_BUCKETS - 1
    assert int(C._bucket(torch.tensor([0.0]), C.LUT_BUCKETS)) in (8191, 8192)       # 8191.5 rounds to even: 8192
    assert int(C._bucket(torch.tensor([float("nan")]), C.LUT_BUCKETS)) == 0
