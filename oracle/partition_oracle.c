/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement (oracle) of the Accel-GCN
 * block-level partitioner.  Nothing in the product library links, loads or
 * calls this file; only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark do, and only as a checker / reported baseline.
 *
 * Parity status: PINNED.  The output of this file is compared byte for byte
 * against the 16 golden `.block4` files the reference ships
 * (block_level_meta/<graph>.block4) and against outputs of the unmodified
 * reference script on seeded edge-case inputs (tests/golden/).
 *
 * Reference followed: block_level_partition.py
 *   :7-21   pattern tables  (agcn_oracle_pattern)
 *   :38     degree extraction
 *   :48-103 sequential walk (agcn_oracle_partition)
 *   :105-106 int32 AoS 4-tuple output
 */
#include <stdint.h>
#include <stddef.h>

#define ORACLE_DEG_BOUND 384   /* block_level_partition.py:7  (12 * 32) */
#define ORACLE_NUM_WARPS 12    /* block_level_partition.py:8 */

/* Pattern tables, block_level_partition.py:9-21.  The reference builds two
 * lists indexed by degree 0..191 by walking a factor list; degrees past the
 * end of the lists take the fall-back values at :56-63.  Returns the table
 * length (192) and fills warp_nz[] / block_rows[] (capacity >= 192). */
int agcn_oracle_pattern(int32_t *warp_nz, int32_t *block_rows)
{
    static const int factor[6] = {1, 2, 3, 4, 6, 12};
    const int warp_max_nz = ORACLE_DEG_BOUND / ORACLE_NUM_WARPS;
    int n = 0, jf = 0, i = 1;
    warp_nz[n] = 0; block_rows[n] = 0; n++;
    while (i < ORACLE_DEG_BOUND / 2) {
        if (factor[jf] * warp_max_nz >= i) {
            warp_nz[n] = (i + factor[jf] - 1) / factor[jf];
            block_rows[n] = ORACLE_NUM_WARPS / factor[jf];
            n++; i++;
        } else {
            jf++;
        }
    }
    return n;
}

/* Sequential walk, block_level_partition.py:48-103.
 * indptr has n_rows+1 entries.  out4 (may be NULL for a pure count) receives
 * up to cap 4-tuples {degree, row_begin, loc_begin, info}.  Returns the
 * number of tuples the walk produces (even when it exceeds cap), or -1 when
 * n_rows <= 0 (the reference raises IndexError on an empty graph). */
int64_t agcn_oracle_partition(const int32_t *indptr, int64_t n_rows,
                              int32_t *out4, int64_t cap)
{
    int32_t warp_nz[ORACLE_DEG_BOUND], block_rows[ORACLE_DEG_BOUND];
    const int tab_len = agcn_oracle_pattern(warp_nz, block_rows);
    if (n_rows <= 0) return -1;

    int64_t cur_row = 0, n_out = 0;
    int32_t cur_loc = 0;           /* numpy int32 scalar arithmetic in the reference */
    for (;;) {
        const int32_t cur_degree = indptr[cur_row + 1] - indptr[cur_row];
        if (cur_degree == 0) {
            cur_row += 1;                                   /* :52-53 */
        } else if (cur_degree >= 1 && cur_degree <= ORACLE_DEG_BOUND) {
            const int32_t w_nz  = cur_degree >= tab_len ? ORACLE_DEG_BOUND / ORACLE_NUM_WARPS
                                                        : warp_nz[cur_degree];    /* :56-59 */
            const int32_t b_row = cur_degree >= tab_len ? 1 : block_rows[cur_degree]; /* :60-63 */
            const int64_t row_begin = cur_row;
            const int32_t loc_begin = cur_loc;
            int32_t j = 0;
            while (indptr[cur_row + 1] - indptr[cur_row] == cur_degree) {  /* :69-75 */
                cur_row += 1;
                j += 1;
                if (j == b_row) break;
                if (cur_row == n_rows) break;
            }
            cur_loc += j * cur_degree;
            if (out4 && n_out < cap) {
                out4[4 * n_out + 0] = cur_degree;
                out4[4 * n_out + 1] = (int32_t)row_begin;
                out4[4 * n_out + 2] = loc_begin;
                out4[4 * n_out + 3] = (w_nz << 16) + j;                    /* :78 */
            }
            n_out++;
        } else if (cur_degree > ORACLE_DEG_BOUND) {          /* :80-96 */
            int32_t tmp_loc = 0;
            for (;;) {
                int32_t info;
                const int32_t loc_begin = cur_loc;
                if (tmp_loc + ORACLE_DEG_BOUND > cur_degree) {
                    info = cur_degree - tmp_loc;
                    cur_loc += cur_degree - tmp_loc;
                    tmp_loc = cur_degree;
                } else {
                    info = ORACLE_DEG_BOUND;
                    tmp_loc += ORACLE_DEG_BOUND;
                    cur_loc += ORACLE_DEG_BOUND;
                }
                if (out4 && n_out < cap) {
                    out4[4 * n_out + 0] = cur_degree;
                    out4[4 * n_out + 1] = (int32_t)cur_row;
                    out4[4 * n_out + 2] = loc_begin;
                    out4[4 * n_out + 3] = info;
                }
                n_out++;
                if (tmp_loc == cur_degree) break;
            }
            cur_row += 1;
        } else {
            return -2;   /* negative degree: the reference prints an error and stops (:98-100) */
        }
        if (cur_row == n_rows) break;                        /* :102-103 */
    }
    return n_out;
}
