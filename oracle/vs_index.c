/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle, never part of the shipped path.
 *
 * Plain-C restatement of the reference's vertical/slash index conversion
 * (csrc/vertical_slash_index.cu:27-99, the kernel body; :21-25, save_blocks;
 * :127-167, the zero-initialised outputs and row count).  One call walks every
 * (batch, head, 64-row query block) sequentially, exactly in the order the
 * reference's single thread per row block does.
 *
 * Parity status: pinned.  tests/test_oracle_index.py checks this file against
 * (a) the reference kernel body itself compiled for the host from the reference
 * tree (oracle/build_ref.py -> oracle/_ref/libref_vs_index_host.so) and
 * (b) fixtures under tests/golden/ produced from that library.
 *
 * One deliberate difference: the reference skips slash entries >= end_m with no
 * bounds check (vertical_slash_index.cu:65-67) and reads past the slash list
 * when no entry qualifies.  Here that case sets counts to 0 for the row block and
 * makes the function return the number of such row blocks, so callers can tell.
 */
#include <stdint.h>
#include <string.h>

#define BLK 64

static int imax(int a, int b) { return a > b ? a : b; }

/* csrc/vertical_slash_index.cu:21-25 */
static void emit_tiles(int32_t *dst, int lo, int hi, int *n)
{
    for (int t = lo; t < hi; t += BLK) dst[(*n)++] = t;
}

/*
 * seqlens          [B]
 * vertical_indexes [B, H, nnz_v]  ascending
 * slash_indexes    [B, H, nnz_s]  descending diagonal offsets
 * block_count      [B, H, rows]
 * block_offset     [B, H, rows, nnz_s]
 * column_count     [B, H, rows]
 * column_index     [B, H, rows, nnz_v]
 * rows = ceil(context_size / 64).  Outputs are fully written (zero tails).
 * Returns the number of row blocks that had no usable slash entry.
 */
int oracle_convert_vertical_slash_indexes(
    const int32_t *seqlens, const int32_t *vertical_indexes, const int32_t *slash_indexes,
    int32_t *block_count, int32_t *block_offset, int32_t *column_count, int32_t *column_index,
    int batch, int heads, int rows, int nnz_v, int nnz_s)
{
    int bad = 0;
    size_t nrow = (size_t)batch * heads * rows;
    memset(block_count, 0, nrow * sizeof(int32_t));
    memset(column_count, 0, nrow * sizeof(int32_t));
    memset(block_offset, 0, nrow * (size_t)nnz_s * sizeof(int32_t));
    memset(column_index, 0, nrow * (size_t)nnz_v * sizeof(int32_t));

    for (int b = 0; b < batch; ++b)
    for (int h = 0; h < heads; ++h)
    for (int m = 0; m < rows; ++m) {
        int seqlen = seqlens[b];
        int start_m = m * BLK;
        if (start_m >= seqlen) continue;                 /* :49-51 */
        int end_m = start_m + BLK;
        const int32_t *vi = vertical_indexes + ((size_t)b * heads + h) * nnz_v;
        const int32_t *si = slash_indexes + ((size_t)b * heads + h) * nnz_s;
        size_t row = ((size_t)b * heads + h) * rows + m;
        int32_t *bo = block_offset + row * nnz_s;
        int32_t *ci = column_index + row * nnz_v;

        int ncol = 0, nblk = 0;
        int s = 0, v = 0;
        int v_idx = vi[v++];
        /* :65-67, with the missing bounds check added */
        while (s < nnz_s && si[s] >= end_m) ++s;
        if (s == nnz_s) { ++bad; continue; }
        int s_idx = imax(end_m - si[s++], BLK);          /* :68 */
        int range_start = s_idx - BLK, range_end = s_idx;
        for (;;) {
            if (v_idx < range_end) {                     /* :71-79 */
                if (v_idx < range_start) ci[ncol++] = v_idx;
                v_idx = (v < nnz_v) ? vi[v++] : end_m + BLK;
            } else {                                     /* :80-94 */
                if (s < nnz_s) {
                    s_idx = imax(end_m - si[s++], BLK);
                } else {
                    emit_tiles(bo, range_start, range_end, &nblk);
                    break;
                }
                if (s_idx > range_end + BLK) {
                    emit_tiles(bo, range_start, range_end, &nblk);
                    range_start = s_idx - BLK;
                    range_end = s_idx;
                } else if (s_idx > range_end) {
                    range_end += BLK;
                }
            }
        }
        block_count[row] = nblk;
        column_count[row] = ncol;
    }
    return bad;
}
