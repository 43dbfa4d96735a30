"""Codebook learning and (de)quantisation of the first moment.

The momentum of every parameter is stored as one ``uint8`` index per element
into a single optimizer-wide, sorted 256-entry fp32 codebook (end points pinned
to -1 and +1) plus one fp32 magnitude per block.  The codebook is the exact
weighted 1-D k-means solution over a 4096-bin histogram of the block-normalised
first-step gradients.

Parity: reference ``src/gefen/gefen.py:288-335`` (nearest index, ties to the
lower index), ``:337-377`` (dequantise), ``:417-517`` (histogram + solve) and
``src/gefen/quantization.py:197-253`` (exact DP).  The solver here is host C++
(``csrc/host/exact_dp.cpp``) with a vectorised numpy fallback.
"""
from __future__ import annotations

import ctypes
import logging
import warnings
from typing import Iterable, Optional, Tuple

import numpy as np
import torch

logger = logging.getLogger(__name__)

NUM_CODEWORDS = 256
HISTOGRAM_BINS = NUM_CODEWORDS * 16
LUT_BUCKETS = 16384


# Optional observability switches (reference ``gefen.py:3095-3155``): when
# ``LIST_STEPS_SAVE_HIST_GRAD`` holds optimizer step numbers, ``Gefen.step`` writes the histogram of
# the block-normalised gradients at those steps to ``<SAVE_CODEBOOK_PREFIX>_grad_hist_step_<n>.pt``.
LIST_STEPS_SAVE_HIST_GRAD = None
SAVE_CODEBOOK_PREFIX = None


# --------------------------------------------------------------------------
# histogram
# --------------------------------------------------------------------------
def save_distribution_histogram_pt_from_counts(hist: torch.Tensor, prefix: str, suffix: str, num_samples: int,
                                               value_range=(-1.0, 1.0)) -> None:
    """Write histogram counts with their bin geometry to ``<prefix stem>_<suffix>.pt`` beside
    ``prefix`` (same dictionary as the reference's ``quantization.py:12-56``)."""
    from pathlib import Path

    if prefix is None:
        raise ValueError("Cannot save gradient histogram because SAVE_CODEBOOK_PREFIX is None.")
    if hist.dim() != 1:
        raise ValueError("Expected 1D histogram counts, got dim={}.".format(hist.dim()))
    if hist.numel() <= 0:
        raise ValueError("Expected at least one histogram bin.")
    if num_samples < 0:
        raise ValueError("num_samples must be non-negative, got {}.".format(num_samples))
    base = Path(prefix).expanduser().resolve()
    base.parent.mkdir(parents=True, exist_ok=True)
    path = base.parent / "{}_{}.pt".format(base.stem, suffix)
    counts = hist.detach().cpu().to(torch.float32)
    left, right = float(value_range[0]), float(value_range[1])
    edges = torch.linspace(left, right, steps=counts.numel() + 1, dtype=torch.float32)
    torch.save({"hist": counts, "bin_edges": edges, "bin_centers": 0.5 * (edges[:-1] + edges[1:]),
                "bin_width": (right - left) / float(counts.numel()), "range": (left, right),
                "num_bins": counts.numel(), "num_samples": int(num_samples)}, path)
    logger.info("Saved distribution histogram data to %s", path)


def block_normalised_histogram(flat: torch.Tensor, period: int,
                               bins: int = HISTOGRAM_BINS) -> torch.Tensor:
    """int64 counts of ``g / absmax(block)`` over ``bins`` equal bins of [-1, 1].

    CUDA tensors go through the fused histogram kernel, everything else through
    torch ops; both produce the same counts (bin = ``floor((x + 1) / width)``
    clamped to the last bin).
    """
    flat = flat.detach().reshape(-1)
    if flat.numel() % period:
        raise ValueError("period {} does not divide numel {}".format(period, flat.numel()))
    if flat.is_cuda:
        from ..ops import quant as _q

        if _q.available():
            return _q.histogram(flat, period, bins)
    x = flat.float().view(-1, period)
    absmax = x.abs().amax(dim=1, keepdim=True)
    normed = torch.where(absmax > 0, x / absmax, torch.zeros_like(x)).reshape(-1)
    width = 2.0 / float(bins)
    idx = torch.floor((normed + 1.0) / width).to(torch.long).clamp_(0, bins - 1)
    return torch.bincount(idx, minlength=bins)


def _pad_codebook(active_centers: torch.Tensor, k: int, force_endpoints: bool) -> torch.Tensor:
    out = torch.empty(k, dtype=torch.float32)
    n = int(active_centers.numel())
    out[:n] = active_centers
    out[n:] = active_centers[-1]
    if force_endpoints:
        out[0] = -1.0
        out[-1] = 1.0
    return out.sort().values


def _exact_dp_numpy(pw, pwx, pwx2, k: int, force_endpoints: bool) -> np.ndarray:
    """Vectorised fallback of the DP (one cost matrix strip per cluster count)."""
    n = pw.shape[0] - 1
    inf = np.inf
    prev = np.full(n + 1, inf)
    prev[0] = 0.0
    back = np.full((n + 1, k + 1), -1, dtype=np.int64)
    s_all = np.arange(1, n + 1)
    for c in range(1, k + 1):
        cur = np.full(n + 1, inf)
        pin = force_endpoints and (c == 1 or c == k)
        centre = -1.0 if c == 1 else 1.0
        s = s_all[c - 1:]                      # candidate starts c..n
        base = prev[s - 1]
        for e0 in range(c, n + 1, 512):
            e = np.arange(e0, min(e0 + 512, n + 1))
            sw = pw[e][:, None] - pw[s - 1][None, :]
            swx = pwx[e][:, None] - pwx[s - 1][None, :]
            swx2 = pwx2[e][:, None] - pwx2[s - 1][None, :]
            valid = s[None, :] <= e[:, None]
            with np.errstate(divide="ignore", invalid="ignore"):
                if pin:
                    seg = swx2 - 2.0 * centre * swx + centre * centre * sw
                else:
                    seg = swx2 - (swx * swx) / sw
            cand = np.where(valid, base[None, :] + seg, inf)
            cand = np.where(np.isnan(cand), inf, cand)
            j = cand.argmin(axis=1)
            cur[e] = cand[np.arange(e.size), j]
            back[e, c] = s[j]
        prev = cur
    out = np.empty(k, dtype=np.float32)
    e = n
    for c in range(k, 0, -1):
        s = back[e, c]
        if force_endpoints and c == 1:
            out[c - 1] = -1.0
        elif force_endpoints and c == k:
            out[c - 1] = 1.0
        else:
            out[c - 1] = (pwx[e] - pwx[s - 1]) / (pw[e] - pw[s - 1])
        e = s - 1
    return out


EXACT_DP_METHOD = "monotone"   # "monotone": divide and conquer; "scan": every start for every end


def exact_dp(histogram_stats: dict, num_codebooks: int,
             force_endpoints: bool = True, method: Optional[str] = None) -> torch.Tensor:
    """Exact weighted k-means of the active histogram bins; returns a sorted codebook.

    ``method`` (default: the module flag ``EXACT_DP_METHOD``): ``"scan"`` evaluates every segment
    start for every end, O(n^2 k), like the reference's solver; ``"monotone"`` uses the
    monotonicity of the optimal start (the segment cost satisfies the quadrangle inequality) for
    O(n k log n) with the same tie rule."""
    method = method or EXACT_DP_METHOD
    if method not in ("scan", "monotone"):
        raise ValueError("exact_dp method must be 'scan' or 'monotone'")
    centers = histogram_stats["active_centers"].detach().cpu().to(torch.float32)
    counts = histogram_stats["active_counts"].detach().cpu().to(torch.float32)
    if centers.numel() == 0:
        raise ValueError("Cannot run exact DP on an empty histogram.")
    if not bool(torch.all(counts > 0)):
        raise ValueError("exact DP expects strictly positive counts for all active histogram bins.")
    if num_codebooks > centers.numel():
        return _pad_codebook(centers, num_codebooks, force_endpoints)

    n = int(centers.numel())
    w = counts.to(torch.float64)
    x = centers.to(torch.float64)
    pw = torch.zeros(n + 1, dtype=torch.float64)
    pwx = torch.zeros(n + 1, dtype=torch.float64)
    pwx2 = torch.zeros(n + 1, dtype=torch.float64)
    pw[1:] = torch.cumsum(w, 0)
    pwx[1:] = torch.cumsum(w * x, 0)
    pwx2[1:] = torch.cumsum(w * x.square(), 0)

    from .. import build as _build

    lib = _build.host_lib()
    if lib is not None:
        a, b, c = (t.contiguous().numpy() for t in (pw, pwx, pwx2))
        out = np.empty(num_codebooks, dtype=np.float32)
        solver = lib.gefen_exact_dp_monotone if method == "monotone" else lib.gefen_exact_dp
        rc = solver(
            a.ctypes.data_as(ctypes.c_void_p), b.ctypes.data_as(ctypes.c_void_p),
            c.ctypes.data_as(ctypes.c_void_p), n, int(num_codebooks),
            int(bool(force_endpoints)), out.ctypes.data_as(ctypes.c_void_p),
        )
        if rc != 0:
            raise RuntimeError("exact-DP solver failed with code {}".format(rc))
        codebook = torch.from_numpy(out)
    else:
        warnings.warn(
            "gefen_x_b200: host C++ library unavailable; using the numpy exact-DP "
            "fallback (slow for full 4096-bin histograms).", UserWarning, stacklevel=2)
        codebook = torch.from_numpy(
            _exact_dp_numpy(pw.numpy(), pwx.numpy(), pwx2.numpy(), num_codebooks,
                            force_endpoints))
    return codebook.sort().values


def histogram_stats_from_counts(counts_int64: torch.Tensor) -> dict:
    bins = int(counts_int64.numel())
    edges = torch.linspace(-1.0, 1.0, steps=bins + 1, dtype=torch.float32)
    centers = 0.5 * (edges[:-1] + edges[1:])
    counts = counts_int64.to("cpu").to(torch.float32)
    active = counts > 0
    return {
        "bin_edges": edges,
        "bin_centers": centers,
        "bin_counts": counts,
        "active_bins": active,
        "active_centers": centers[active],
        "active_counts": counts[active],
        "active_sums": centers[active] * counts[active],
    }


def learn_codebook_from_grad_periods(
    grad_periods: Iterable[Tuple[str, torch.Tensor, int, torch.Tensor]],
    codebook_device,
    num_codebooks: int = NUM_CODEWORDS,
    force_endpoints: bool = True,
    verbose: bool = False,
    reduce_counts=None,
) -> Optional[torch.Tensor]:
    """Learn the optimizer-wide codebook from ``(name, flat_grad, period, grad)`` items.

    ``reduce_counts`` (optional callable on the int64 count vector) lets a
    sharded run sum the histogram over ranks so that every rank learns the same
    codebook; the default keeps the reference's rank-local behaviour.
    """
    bins = num_codebooks * 16
    total = 0
    counts_by_dev = {}
    for _name, flat, period, _grad in grad_periods:
        flat = flat.reshape(-1)
        if flat.numel() == 0:
            continue
        c = block_normalised_histogram(flat, period, bins)
        key = c.device
        if key in counts_by_dev:
            counts_by_dev[key].add_(c)
        else:
            counts_by_dev[key] = c.clone()
        total += flat.numel()
    counts = torch.zeros(bins, dtype=torch.int64)
    for c in counts_by_dev.values():
        counts.add_(c.cpu())
    if reduce_counts is not None:
        counts = reduce_counts(counts)
        total = int(counts.sum().item())
    if total == 0:
        return None
    stats = histogram_stats_from_counts(counts)
    codebook = exact_dp(stats, num_codebooks, force_endpoints).to(codebook_device)
    if verbose:
        cb = codebook.cpu()
        ac = stats["active_centers"]
        idx = nearest_codebook_indices(cb, ac).long()
        mse = ((ac - cb[idx]).square() * stats["active_counts"]).sum().item() / total
        print("  exact DP: MSE_normalized={:.6e}".format(mse))
    return codebook


# --------------------------------------------------------------------------
# quantise / dequantise
# --------------------------------------------------------------------------
_SEARCH_CHUNK = 1 << 23


def decision_thresholds(codebook: torch.Tensor) -> torch.Tensor:
    """``thr[i] = fp32((cb[i] + cb[i + 1]) * 0.5)`` for the 255 neighbouring pairs."""
    cb = codebook.detach().float()
    return (cb[:-1] + cb[1:]) * 0.5


def nearest_codebook_indices(codebook: torch.Tensor, normalized: torch.Tensor) -> torch.Tensor:
    """uint8 index of the nearest codeword: ``#{i : thr[i] < v}`` over the decision
    thresholds, so a value exactly between two codewords goes to the lower one.

    The reference compares the two fp32 distances instead (``gefen.py:288-335``);
    the two rules differ only for values within an ulp of a midpoint.
    """
    if codebook.device != normalized.device:
        raise ValueError(
            "Gefen codebook device {} does not match normalized_vals device {}.".format(
                codebook.device, normalized.device))
    k = int(codebook.numel())
    out = torch.empty(normalized.shape, dtype=torch.uint8, device=normalized.device)
    if k <= 1:
        return out.zero_()
    thr = decision_thresholds(codebook)
    src = normalized.reshape(-1)
    dst = out.view(-1)
    for s in range(0, src.numel(), _SEARCH_CHUNK):
        v = src[s:s + _SEARCH_CHUNK].float()
        dst[s:s + _SEARCH_CHUNK] = torch.bucketize(v, thr).to(torch.uint8)
    return out


def dequantize_indices(codebook: torch.Tensor, indices: torch.Tensor,
                       dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``codebook[indices]`` as ``dtype`` without a full-size int64 temporary."""
    if codebook.device != indices.device:
        raise ValueError(
            "Gefen codebook device {} does not match stored index device {}.".format(
                codebook.device, indices.device))
    out = torch.empty(indices.shape, dtype=dtype, device=indices.device)
    o = out.view(-1)
    i = indices.reshape(-1)
    for s in range(0, i.numel(), _SEARCH_CHUNK):
        o[s:s + _SEARCH_CHUNK] = codebook.index_select(0, i[s:s + _SEARCH_CHUNK].long())
    return out


def _bucket(values: torch.Tensor, buckets: int) -> torch.Tensor:
    """``rint(sat(fma(x, 0.5, 0.5)) * (buckets - 1))`` with both fused multiply-adds rounded once to
    fp32, as on the device (the second one adds 2^23 there, which rounds the product to the nearest
    integer, ties to even)."""
    t = (values.double() * 0.5 + 0.5).float().clamp_(0.0, 1.0)      # exact product and sum, one rounding
    t = torch.nan_to_num(t, nan=0.0)
    return torch.round(t.double() * float(buckets - 1)).to(torch.long)   # exact product; round half to even


def codebook_search_lut(codebook: torch.Tensor, buckets: int = LUT_BUCKETS) -> torch.Tensor:
    """Bucket table that narrows the threshold search.

    ``lut[b]`` = number of decision thresholds whose bucket is below ``b`` (int16,
    ``buckets + 1`` entries), so the insertion point of any value of bucket ``b``
    among the thresholds lies in ``[lut[b], lut[b + 1]]``.  It is an accelerator
    only: the result is identical with or without it.  Same idea as the
    reference's table (``kernels/automatic_gefen_fused.py:81-121``), built over the
    thresholds instead of the codewords.
    """
    thr = decision_thresholds(codebook)
    hist = torch.bincount(_bucket(thr, buckets), minlength=buckets)
    lut = torch.zeros(buckets + 1, dtype=torch.long, device=thr.device)
    lut[1:] = torch.cumsum(hist, 0)
    return lut.to(torch.int16)


def packed_search_lut(codebook: torch.Tensor, buckets: int = LUT_BUCKETS) -> torch.Tensor:
    """The table the kernels load: ``lut[b] | (lut[b + 1] - lut[b]) << 8`` as int16[buckets]
    (bit pattern of an unsigned 16-bit value: thresholds below the bucket, thresholds inside it)."""
    lut = codebook_search_lut(codebook, buckets).to(torch.int32)
    packed = lut[:-1] | ((lut[1:] - lut[:-1]) << 8)
    packed = torch.where(packed >= 32768, packed - 65536, packed)
    return packed.to(torch.int16).contiguous()


def padded_thresholds(codebook: torch.Tensor) -> torch.Tensor:
    """The 255 thresholds followed by ``+inf`` (fp32[256]), the layout the kernels load."""
    thr = decision_thresholds(codebook)
    return torch.cat([thr, torch.full((1,), float("inf"), dtype=torch.float32, device=thr.device)]).contiguous()
