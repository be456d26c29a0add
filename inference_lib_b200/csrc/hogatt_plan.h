// Split-K decomposition shared by host and device code.
//
// The op is cut into *units* (one kv head of one block of query rows).  The visible keys of a
// unit are a sequence of *tiles*: up to `tile_tokens` consecutive keys of ONE fragment (tiles
// never straddle a fragment boundary, because the query changes at every boundary).  All units
// have the same tile count TH, so the whole call is a list of N = units * TH tiles, ordered
// unit-major.  The persistent grid cuts that list into `ctas` contiguous, balanced ranges:
// CTA c walks tiles [c*N/ctas, (c+1)*N/ctas).  Where a range ends inside a unit the CTA leaves a
// partial result (unnormalised output rows + running max + running sum) in the workspace; the
// merge step combines the partials of each unit.
//
// The reference instead gives each (kv head, worker, query token) `splits` CTAs that take keys
// interleaved with stride `splits` (src/kernels/kernel_v21.cuh:62-66,113,957-964) and re-reads
// the KV once per (worker, token); here one CTA serves every worker and GQA head of its kv head.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define HOGATT_HD __host__ __device__ __forceinline__
#else
#define HOGATT_HD inline
#endif

namespace hogatt {

// floor(num / den) for num >= 0, den > 0.  On the device a 64-bit division is a ~100-instruction routine; the
// quotients here almost always fit 32 bits, so that case divides in 32 bits and the general one is kept out
// of line (these run in kernels whose whole life is a few microseconds: code size and latency both show).
#if defined(__CUDACC__)
__host__ __device__ __noinline__ inline int64_t wide_div(int64_t num, int64_t den) { return num / den; }
#else
inline int64_t wide_div(int64_t num, int64_t den) { return num / den; }
#endif
HOGATT_HD int64_t floor_div(int64_t num, int64_t den) {
    if ((((uint64_t)num | (uint64_t)den) >> 32) == 0) return (int64_t)((uint32_t)num / (uint32_t)den);
    return wide_div(num, den);
}

// First global tile index of CTA c (c may equal ctas: end of the last range).
HOGATT_HD int64_t cta_first_tile(int64_t c, int64_t total_tiles, int64_t ctas) {
    return floor_div(c * total_tiles, ctas);
}

// CTAs that get work: never more than there are tiles, so every CTA owns at least one tile.
HOGATT_HD int effective_ctas(int64_t total_tiles, int grid) {
    return total_tiles < (int64_t)grid ? (int)total_tiles : grid;
}

// CTAs that get work when no CTA's range should cross a fragment or unit boundary.  `pre[0..F]` is the tile prefix of
// a unit's fragments.  If a whole number T of tiles per CTA divides every fragment's tile count and needs between
// three quarters of the grid and the whole grid, N / T CTAs of exactly T tiles each are used: their ranges start at
// multiples of T, so each lies inside one fragment of one unit.  A CTA whose range crosses a boundary rotates and
// stages a second set of query rows and, at a unit boundary, folds and stores twice; on B200 exactly those CTAs were
// the last to finish by about 2 us (16 K keys, 8 kv heads: 17.1 -> 15.5 us per call with 128 CTAs x 8 tiles instead of
// 148 x 6.9).  Otherwise (long contexts, ragged lengths): balanced ranges over effective_ctas().
HOGATT_HD int aligned_ctas(const int* pre, int F, int64_t units, int grid) {
    const int64_t TH = pre[F], N = units * TH;
    const int fallback = effective_ctas(N, grid);
    if (TH <= 0 || N <= (int64_t)grid) return fallback;
    int64_t g = 0;
    for (int f = 0; f < F; ++f) {
        int64_t t = pre[f + 1] - pre[f];
        while (t != 0) {                 // g = gcd(g, t)
            const int64_t r = g % t;
            g = t;
            t = r;
        }
    }
    const int64_t lo = (N + grid - 1) / grid, hi = floor_div(N * 4, (int64_t)grid * 3);
    for (int64_t T = lo; T <= hi && T <= g; ++T)
        if (g % T == 0) return (int)(N / T);
    return fallback;
}

// Smallest c whose range ends after tile x, i.e. the first CTA that touches tile x.
HOGATT_HD int cta_of_tile(int64_t x, int64_t total_tiles, int64_t ctas) {
    // floor((c+1)*N/n) > x  <=>  (c+1)*N >= (x+1)*n  <=>  c >= ceil((x+1)*n/N) - 1
    return (int)(floor_div((x + 1) * ctas + total_tiles - 1, total_tiles) - 1);
}

// First CTA touching unit u and how many consecutive CTAs touch it.
HOGATT_HD void unit_ctas(int64_t unit, int64_t tiles_per_unit, int64_t total_tiles, int64_t ctas,
                         int* first, int* count) {
    const int a = cta_of_tile(unit * tiles_per_unit, total_tiles, ctas);
    const int b = cta_of_tile((unit + 1) * tiles_per_unit - 1, total_tiles, ctas);
    *first = a;
    *count = b - a + 1;
}

// Upper bound on unit_ctas(...).count for any tile count: balanced range boundaries are spaced
// N/ctas apart, a unit is N/units long, so at most ctas/units boundaries (+ rounding) fall inside.
HOGATT_HD int max_parts_per_unit(int units, int grid) {
    return grid / units + 2;
}

HOGATT_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace hogatt
