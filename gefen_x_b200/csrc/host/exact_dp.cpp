// Exact weighted 1-D k-means over a histogram, solved by dynamic programming.
//
// Host C++ (OpenMP) replacement for the reference's numba-compiled solver
// (reference src/gefen/quantization.py:83-136).  Input: prefix sums of the bin
// weights w, w*x and w*x^2 over the active (non-empty) histogram bins in
// ascending x.  Output: k cluster centres, the first and last pinned to -1/+1
// when force_endpoints is set.  Ties keep the smallest segment start, as a
// left-to-right scan with a strict "<" would.
//
// Layout chosen for the host cache: two rolling cost rows (the recurrence only
// needs the previous cluster count) and one int32 backtrack table; every
// end-index of a row is independent, so the row is split over threads.
//
// Plain C ABI so Python can load it with ctypes; no torch headers.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

extern "C" {

// Returns 0 on success, non-zero on bad arguments.
static int exact_dp_impl(const double* prefix_w, const double* prefix_wx,
                         const double* prefix_wx2, int64_t num_points,
                         int64_t num_codebooks, int force_endpoints, float* codebook_out,
                         bool use_monotone) {
    if (num_points <= 0 || num_codebooks <= 0 || num_codebooks > num_points) return 1;
    const int64_t n = num_points, k = num_codebooks;
    const double inf = std::numeric_limits<double>::infinity();
    std::vector<double> prev(n + 1, inf), cur(n + 1, inf);
    std::vector<int32_t> back((size_t)(n + 1) * (size_t)(k + 1), -1);
    prev[0] = 0.0;

    for (int64_t c = 1; c <= k; ++c) {
        const bool pin_lo = force_endpoints && c == 1;
        const bool pin_hi = force_endpoints && c == k;
        const double centre = pin_lo ? -1.0 : 1.0;
        for (int64_t e = 0; e <= n; ++e) cur[e] = inf;
        if (use_monotone) {
            // Divide and conquer over the end index: the segment cost is a sum over points (pinned
            // rows) or a within-cluster sum of squares (free rows); both satisfy the quadrangle
            // inequality, so the smallest optimal start is non-decreasing in the end index and
            // every end only scans the window its neighbours leave open: O(n log n) per row.
            struct Job { int64_t lo, hi, slo, shi; };
            std::vector<Job> stack;
            stack.push_back({c, n, c, n});
            while (!stack.empty()) {
                const Job j = stack.back();
                stack.pop_back();
                if (j.lo > j.hi) continue;
                const int64_t e = (j.lo + j.hi) / 2;
                double best = inf;
                int64_t best_s = -1;
                const double we = prefix_w[e], wxe = prefix_wx[e], wx2e = prefix_wx2[e];
                const int64_t s_end = std::min(e, j.shi);
                for (int64_t s = std::max(c, j.slo); s <= s_end; ++s) {
                    const double base = prev[s - 1];
                    if (!(base < inf)) continue;
                    const double sw = we - prefix_w[s - 1];
                    const double swx = wxe - prefix_wx[s - 1];
                    const double swx2 = wx2e - prefix_wx2[s - 1];
                    const double seg = (pin_lo || pin_hi) ? swx2 - 2.0 * centre * swx + centre * centre * sw
                                                          : swx2 - (swx * swx) / sw;
                    const double cand = base + seg;
                    if (cand < best) { best = cand; best_s = s; }
                }
                cur[e] = best;
                back[(size_t)e * (size_t)(k + 1) + (size_t)c] = (int32_t)best_s;
                const int64_t split = best_s < 0 ? j.slo : best_s;
                stack.push_back({j.lo, e - 1, j.slo, best_s < 0 ? j.shi : split});
                stack.push_back({e + 1, j.hi, split, j.shi});
            }
            prev.swap(cur);
            continue;
        }
#pragma omp parallel for schedule(dynamic, 16)
        for (int64_t e = c; e <= n; ++e) {
            double best = inf;
            int32_t best_s = -1;
            const double we = prefix_w[e], wxe = prefix_wx[e], wx2e = prefix_wx2[e];
            for (int64_t s = c; s <= e; ++s) {
                const double base = prev[s - 1];
                if (!(base < inf)) continue;
                const double sw = we - prefix_w[s - 1];
                const double swx = wxe - prefix_wx[s - 1];
                const double swx2 = wx2e - prefix_wx2[s - 1];
                double seg;
                if (pin_lo || pin_hi)
                    seg = swx2 - 2.0 * centre * swx + centre * centre * sw;
                else
                    seg = swx2 - (swx * swx) / sw;
                const double cand = base + seg;
                if (cand < best) { best = cand; best_s = (int32_t)s; }
            }
            cur[e] = best;
            back[(size_t)e * (size_t)(k + 1) + (size_t)c] = best_s;
        }
        prev.swap(cur);
    }

    int64_t e = n;
    for (int64_t c = k; c >= 1; --c) {
        const int64_t s = back[(size_t)e * (size_t)(k + 1) + (size_t)c];
        if (s < 1) return 2;
        if (force_endpoints && c == 1) codebook_out[c - 1] = -1.0f;
        else if (force_endpoints && c == k) codebook_out[c - 1] = 1.0f;
        else {
            const double sw = prefix_w[e] - prefix_w[s - 1];
            const double swx = prefix_wx[e] - prefix_wx[s - 1];
            codebook_out[c - 1] = (float)(swx / sw);
        }
        e = s - 1;
    }
    return 0;
}

// Full scan of every start for every end: O(n^2 k).
int gefen_exact_dp(const double* prefix_w, const double* prefix_wx,
                   const double* prefix_wx2, int64_t num_points,
                   int64_t num_codebooks, int force_endpoints, float* codebook_out) {
    return exact_dp_impl(prefix_w, prefix_wx, prefix_wx2, num_points, num_codebooks, force_endpoints,
                         codebook_out, false);
}

// Same recurrence, same tie rule (smallest start), monotone-optimum search: O(n k log n).
int gefen_exact_dp_monotone(const double* prefix_w, const double* prefix_wx,
                            const double* prefix_wx2, int64_t num_points,
                            int64_t num_codebooks, int force_endpoints, float* codebook_out) {
    return exact_dp_impl(prefix_w, prefix_wx, prefix_wx2, num_points, num_codebooks, force_endpoints,
                         codebook_out, true);
}

}  // extern "C"
