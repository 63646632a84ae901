// Row blocks of the 1D row-sharded SpMM: which rows of the degree-ordered matrix each rank owns.
// Host code only (no device is touched), so the layout can be computed and tested anywhere.
// The reference is single-GPU (main.cu:53-182) and has no counterpart.
//
// Cutting the degree-ordered rows into contiguous ranges of equal nonzero count gives the first
// rank most of the (light) rows and the last rank a few heavy ones: the SpMM is balanced, but the
// dense transform X*W, the output rows and above all the all-gather of the dense operand are not
// (one rank sends most of the volume).  Here every rank gets TWO ranges instead, one from the
// light end and one from the heavy end of what is still unassigned, sized so that the rank holds
// rows_per_block rows AND about nnz / world nonzeros.  Removing an exactly average block leaves an
// average remainder, so the same step works for the next rank.  Blocks are equal in height, the
// exchange is one balanced all-gather, and rank g's rows are rows [g * rows_per_block, ...) of the
// gathered operand -- a permutation of the degree order that the column ids are renamed to.
#include "host_common.h"
#include "internal.h"

namespace agcn {

int balanced_blocks(const int *h_indptr, int64_t n_rows, int world, int64_t *h_ranges, int64_t *rows_per_block)
{
    AGCN_REQUIRE(h_indptr != nullptr && h_ranges != nullptr && rows_per_block != nullptr, "agcn_balanced_blocks: null pointer");
    AGCN_REQUIRE(n_rows > 0 && world >= 1 && world <= AGCN_MAX_WORLD, "agcn_balanced_blocks: n_rows > 0 and 1 <= world <= %d", AGCN_MAX_WORLD);
    const int64_t per = ceil_div(n_rows, world);
    *rows_per_block = per;
    const int64_t base = h_indptr[0];
    auto nz = [&](int64_t a, int64_t b) { return (int64_t)h_indptr[b] - (int64_t)h_indptr[a]; };   // nonzeros of rows [a, b)
    AGCN_REQUIRE(nz(0, n_rows) >= 0, "agcn_balanced_blocks: indptr decreases");
    (void)base;
    int64_t lo = 0, hi = n_rows;          // rows [lo, hi) are still unassigned
    for (int g = 0; g < world; g++) {
        const int64_t left = hi - lo;
        const int64_t take = left < per ? left : per;                  // the last blocks may be short or empty
        int64_t q = 0;                                                  // rows taken from the heavy end
        if (g + 1 < world && take > 0 && take < left) {
            // f(q) = nonzeros of the `take - q` lightest and the q heaviest unassigned rows: non-decreasing in q
            // when the rows are in degree order.  Target: this block's share of what is left.
            const double target = (double)nz(lo, hi) * (double)take / (double)left;
            auto f = [&](int64_t qq) { return nz(lo, lo + take - qq) + nz(hi - qq, hi); };
            int64_t a = 0, b = take;                                    // smallest q with f(q) >= target
            while (a < b) {
                const int64_t mid = a + (b - a) / 2;
                if ((double)f(mid) < target) a = mid + 1; else b = mid;
            }
            q = a;
            if (q > 0 && target - (double)f(q - 1) <= (double)f(q) - target) q--;      // whichever side is closer
        }
        const int64_t p = take - q;
        h_ranges[4 * g + 0] = lo;       h_ranges[4 * g + 1] = lo + p;
        h_ranges[4 * g + 2] = hi - q;   h_ranges[4 * g + 3] = hi;
        lo += p;
        hi -= q;
    }
    return AGCN_OK;
}

}  // namespace agcn

extern "C" int agcn_balanced_blocks(const int32_t *h_indptr, int64_t n_rows, int world, int64_t *h_ranges,
                                    int64_t *rows_per_block)
{
    agcn::clear_error();
    return agcn::balanced_blocks(h_indptr, n_rows, world, h_ranges, rows_per_block);
}
