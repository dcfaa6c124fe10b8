// Prefill-time quantized linear (m >= 128).  Placeholder while the tcgen05 kernel is
// brought up: routes through the streaming kernel in groups of 32 rows (correct, re-reads W).
#include "common.cuh"

extern "C" size_t atlas_qlinear_gemm_workspace_bytes(int64_t m, int64_t n_cols) {
    (void)m; (void)n_cols;
    return 0;
}

extern "C" int atlas_qlinear_gemm(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                  const void *scales, const int32_t *outlier_row_ptr,
                                  const int32_t *outlier_col, const void *outlier_vals, int64_t n_rows,
                                  int64_t n_cols, int block_size, const void *bias, void *y, int64_t ldy,
                                  void *workspace, size_t workspace_bytes, void *stream) {
    (void)workspace; (void)workspace_bytes;
    return atlas_qlinear_gemv(x, dtype, m, ldx, tiles, scales, outlier_row_ptr, outlier_col, outlier_vals,
                              n_rows, n_cols, block_size, bias, y, ldy, stream);
}
