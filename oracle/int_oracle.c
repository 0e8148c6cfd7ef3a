/*
 * CPU oracle for the integer part of the MoE hot path.  TEST INFRASTRUCTURE ONLY: nothing under
 * cute-kernels_b200/ links or calls this file; tests and the benchmark's CPU baseline do.
 *
 * Restates (paths inside open-lm-engine/cute-kernels):
 *   oracle_count       fma/ops/continuous_count/__init__.py:35-36 (torch branch: bincount, uint32),
 *                      with the documented rule that ids outside [0,size) are ignored (:16-18)
 *   oracle_sort_maps   selected_experts.flatten().sort() + continuous_count,
 *                      fma/modules/moe/__init__.py:213-217, in its stable form, plus the
 *                      expert-contiguous row maps with segments padded to row_align rows
 *                      (padding idea: fma/modules/moe/cuda_implementation/__init__.py:83-104,:133-135)
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

int oracle_count(const void* ids, int id_bytes, int64_t n, int32_t size, uint32_t* out) {
    if (size < 1 || n < 0 || (id_bytes != 4 && id_bytes != 8)) return 1;
    memset(out, 0, (size_t)size * sizeof(uint32_t));
    if (id_bytes == 4) {
        const int32_t* p = (const int32_t*)ids;
        for (int64_t i = 0; i < n; ++i)
            if (p[i] >= 0 && p[i] < size) out[p[i]]++;
    } else {
        const int64_t* p = (const int64_t*)ids;
        for (int64_t i = 0; i < n; ++i)
            if (p[i] >= 0 && p[i] < size) out[p[i]]++;
    }
    return 0;
}

/* Any output pointer may be NULL.  rows_cap is the length of slot_of_row; mtile_expert has rows_cap/128 entries. */
int oracle_sort_maps(const int64_t* selected, int64_t R, int32_t E, int32_t row_align, int64_t rows_cap,
                     int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, uint32_t* expert_count,
                     int32_t* pad_offsets, int32_t* row_of_slot, int32_t* slot_of_row, int32_t* mtile_expert) {
    if (E < 1 || R < 0 || row_align < 1) return 1;
    int64_t* count = (int64_t*)calloc((size_t)E, sizeof(int64_t));
    int64_t* plain = (int64_t*)calloc((size_t)E + 1, sizeof(int64_t));
    int64_t* padded = (int64_t*)calloc((size_t)E + 1, sizeof(int64_t));
    int64_t* next = (int64_t*)calloc((size_t)E, sizeof(int64_t));
    if (!count || !plain || !padded || !next) return 2;
    for (int64_t i = 0; i < R; ++i) {
        if (selected[i] < 0 || selected[i] >= E) return 3;
        count[selected[i]]++;
    }
    for (int32_t e = 0; e < E; ++e) {
        plain[e + 1] = plain[e] + count[e];
        padded[e + 1] = padded[e] + (count[e] + row_align - 1) / row_align * row_align;
    }
    if (expert_count) for (int32_t e = 0; e < E; ++e) expert_count[e] = (uint32_t)count[e];
    if (pad_offsets) for (int32_t e = 0; e <= E; ++e) pad_offsets[e] = (int32_t)padded[e];
    if (slot_of_row) for (int64_t p = 0; p < rows_cap; ++p) slot_of_row[p] = -1;
    for (int64_t i = 0; i < R; ++i) {  /* ascending flat index => stable */
        const int64_t e = selected[i];
        const int64_t rank = next[e]++;
        const int64_t q = plain[e] + rank;
        const int64_t row = padded[e] + rank;
        if (sorted_expert_idxs) sorted_expert_idxs[q] = e;
        if (sorted_scattered_idxs) sorted_scattered_idxs[q] = i;
        if (row_of_slot) row_of_slot[i] = (int32_t)row;
        if (slot_of_row) slot_of_row[row] = (int32_t)i;
    }
    if (mtile_expert) {
        int32_t e = 0;
        for (int64_t t = 0; t < rows_cap / 128; ++t) {
            const int64_t row = t * 128;
            if (row >= padded[E]) { mtile_expert[t] = -1; continue; }
            while (padded[e + 1] <= row) ++e;
            mtile_expert[t] = e;
        }
    }
    free(count); free(plain); free(padded); free(next);
    return 0;
}
