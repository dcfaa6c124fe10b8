// Inverse of the quantizer, and expansion of the compacted code stream into
// the tile-major kernel layout.
//
// Replaces dequantize_tensor (atlasinfer_core/quant/adaptive_quantizer.py:156-251).
// The reference keeps a running offset into the code stream and, per block,
// masks the whole outlier index list (:194-196, O(blocks x outliers)).  Here the
// sorted outlier index list is binary-searched once per block boundary: the
// number of outliers before a block both locates the block's outliers and
// gives the block's offset into the compacted code stream (position minus
// outliers before it), so every block is independent.
#include "common.cuh"

namespace atlas {
namespace {

constexpr int DQ_THREADS = 256;
constexpr int DQ_SPAN = 4096;  // padded elements per CTA

// first i in [0, n) with idx[i] >= key
__device__ __forceinline__ int64_t lower_bound_i64(const int64_t *idx, int64_t n, int64_t key) {
    int64_t lo = 0, hi = n;
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if (idx[mid] < key) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// Shared walk over one span of the padded tensor.  `emit(p, is_outlier, k, code)`
// is called for every padded position p of the span: k is the outlier's index
// in the outlier streams when is_outlier, else `code` is the int8 code.
template <class Emit>
__device__ __forceinline__ void walk_span(const int8_t *codes, int64_t n_codes, const int64_t *oidx,
                                          int64_t n_out, int64_t padded, Emit emit) {
    __shared__ int64_t s_lo, s_hi;
    const int64_t span0 = (int64_t)blockIdx.x * DQ_SPAN;
    const int64_t span1 = min(span0 + DQ_SPAN, padded);
    if (threadIdx.x == 0) s_lo = lower_bound_i64(oidx, n_out, span0);
    if (threadIdx.x == 32) s_hi = lower_bound_i64(oidx, n_out, span1);
    __syncthreads();
    const int64_t lo = s_lo, hi = s_hi;
    for (int64_t p = span0 + threadIdx.x; p < span1; p += DQ_THREADS) {
        // outliers of this span with index < p: search the (short) window [lo, hi)
        int64_t a = lo, b = hi;
        while (a < b) {
            int64_t mid = (a + b) >> 1;
            if (oidx[mid] < p) a = mid + 1; else b = mid;
        }
        const bool is_out = (a < hi) && (oidx[a] == p);
        int8_t code = 0;
        if (!is_out) {
            const int64_t ci = p - a;  // position in the compacted stream
            code = (ci < n_codes) ? codes[ci] : (int8_t)0;
        }
        emit(p, is_out, a, code);
    }
}

__global__ void __launch_bounds__(DQ_THREADS)
dequantize_kernel(const int8_t *codes, int64_t n_codes, const uint16_t *ovals, const int64_t *oidx,
                  int64_t n_out, const uint16_t *scales, int64_t numel, int64_t padded, int bs,
                  uint16_t *w) {
    walk_span(codes, n_codes, oidx, n_out, padded, [&](int64_t p, bool is_out, int64_t k, int8_t code) {
        if (p >= numel) return;
        uint16_t v;
        if (is_out) {
            v = ovals[k];
        } else {
            // fp16(code) * scale, one fp16 rounding (adaptive_quantizer.py:216)
            const float sc = __half2float(__ushort_as_half(scales[p / bs]));
            v = __half_as_ushort(__float2half_rn(__fmul_rn((float)code, sc)));
        }
        w[p] = v;
    });
}

// Byte offset of weight (row, col) inside the tile-major layout.
__device__ __forceinline__ int64_t tile_offset(int64_t row, int64_t col, int64_t k_tiles) {
    const int64_t rt = row >> 7, kt = col >> 6;
    const int strip = (int)(row & 127) >> 4, h = (int)(row & 15) >> 3, g = (int)(row & 7);
    const int tig = (int)(col & 63) >> 4, byte = (int)(col & 15);
    return ((((rt * k_tiles + kt) * 8 + strip) * 2 + h) * 32 + (g * 4 + tig)) * 16 + byte;
}

// One thread per 16 consecutive columns of a row = one 16-byte unit of the tile-major layout (n_cols is a multiple
// of 64, so a unit never straddles rows, and a span of DQ_SPAN positions is DQ_SPAN / 16 whole units).  The thread
// finds how many outliers precede its unit (binary search in the span's short window of the sorted index list),
// walks its 16 positions against the list and the compacted code stream, and stores the unit at once.
__global__ void __launch_bounds__(DQ_THREADS)
repack_kernel(const int8_t *codes, int64_t n_codes, const int64_t *oidx, int64_t n_out, int64_t n_rows,
              int64_t n_cols, uint8_t *tiles) {
    static_assert(DQ_SPAN == DQ_THREADS * 16, "one 16-byte unit per thread");
    __shared__ int64_t s_lo, s_hi;
    const int64_t numel = n_rows * n_cols;
    const int64_t span0 = (int64_t)blockIdx.x * DQ_SPAN;
    const int64_t span1 = min(span0 + DQ_SPAN, numel);
    if (threadIdx.x == 0) s_lo = lower_bound_i64(oidx, n_out, span0);
    if (threadIdx.x == 32) s_hi = lower_bound_i64(oidx, n_out, span1);
    __syncthreads();
    const int64_t p0 = span0 + (int64_t)threadIdx.x * 16;
    if (p0 >= span1) return;
    int64_t a = s_lo, b = s_hi;
    const int64_t hi = b;
    while (a < b) {
        const int64_t mid = (a + b) >> 1;
        if (oidx[mid] < p0) a = mid + 1; else b = mid;
    }
    int64_t next_out = a < hi ? oidx[a] : numel;   // the next outlier position at or after p0 (numel: none in this span)
    int64_t ci = p0 - a;                            // position of p0's code in the compacted stream
    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        uint32_t byte = 128u;                       // an outlier's place holds code 0
        if (p0 + j == next_out) {
            ++a;
            next_out = a < hi ? oidx[a] : numel;
        } else {
            if (ci < n_codes) byte = (uint32_t)((int)codes[ci] + 128);
            ++ci;
        }
        w[j >> 2] |= byte << (8 * (j & 3));
    }
    const int64_t row = p0 / n_cols, col = p0 - row * n_cols;
    *reinterpret_cast<uint4 *>(tiles + tile_offset(row, col, n_cols >> 6)) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Rows beyond n_rows inside the last 128-row tile: code 0.
__global__ void __launch_bounds__(DQ_THREADS)
repack_pad_kernel(int64_t n_rows, int64_t n_rows_padded, int64_t n_cols, uint8_t *tiles) {
    const int64_t k_tiles = n_cols >> 6;
    const int64_t total = (n_rows_padded - n_rows) * n_cols;
    for (int64_t i = (int64_t)blockIdx.x * DQ_THREADS + threadIdx.x; i < total; i += (int64_t)gridDim.x * DQ_THREADS) {
        const int64_t row = n_rows + i / n_cols, col = i % n_cols;
        tiles[tile_offset(row, col, k_tiles)] = 128;
    }
}

__global__ void __launch_bounds__(DQ_THREADS)
row_ptr_kernel(const int64_t *oidx, int64_t n_out, int64_t n_rows, int64_t n_cols, int32_t *row_ptr) {
    const int64_t r = (int64_t)blockIdx.x * DQ_THREADS + threadIdx.x;
    if (r <= n_rows) row_ptr[r] = (int32_t)lower_bound_i64(oidx, n_out, r * n_cols);
}

// Scales transposed per 128-row tile: [row/128][block][row%128], so that the scales of a
// run of rows for one K block are contiguous.
__global__ void __launch_bounds__(DQ_THREADS)
scales_tile_kernel(const uint16_t *scales, int64_t n_rows, int64_t n_rows_padded, int64_t blocks_per_row,
                   uint16_t *scales_t) {
    const int64_t total = n_rows_padded * blocks_per_row;
    for (int64_t i = (int64_t)blockIdx.x * DQ_THREADS + threadIdx.x; i < total; i += (int64_t)gridDim.x * DQ_THREADS) {
        const int64_t rt = i / (blocks_per_row * 128), rem = i - rt * blocks_per_row * 128;
        const int64_t kb = rem >> 7, r = rem & 127;
        const int64_t row = rt * 128 + r;
        scales_t[i] = row < n_rows ? scales[row * blocks_per_row + kb] : (uint16_t)0;
    }
}

// Outliers regrouped by 16-row strip and sorted by column inside a strip.  Entry = row%16 << 24 |
// column.  The position of an outlier is found by counting, over the 16 row lists of its strip
// (each sorted by column already), the entries that precede it: deterministic, no atomics.
__global__ void __launch_bounds__(DQ_THREADS)
strip_sort_kernel(const int64_t *oidx, const uint16_t *ovals, int64_t n_out, int64_t n_rows, int64_t n_cols,
                  const int32_t *row_ptr, uint32_t *entries, uint16_t *vals_sorted) {
    const int64_t i = (int64_t)blockIdx.x * DQ_THREADS + threadIdx.x;
    if (i >= n_out) return;
    const int64_t idx = oidx[i];
    const int64_t row = idx / n_cols, col = idx - row * n_cols;
    const int64_t r0 = row & ~(int64_t)15;
    int rank = 0;
    for (int64_t r = r0; r < r0 + 16 && r < n_rows; ++r) {
        // entries of row r with column < col (rows above) or <= col (rows below or equal: ties keep row order)
        const int64_t key = r * n_cols + col + (r < row ? 1 : 0);
        int lo = row_ptr[r], hi = row_ptr[r + 1];
        const int base = lo;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (oidx[mid] < key) lo = mid + 1; else hi = mid;
        }
        rank += lo - base;
    }
    const int pos = row_ptr[r0] + rank;
    entries[pos] = (uint32_t)(row & 15) << 24 | (uint32_t)col;
    vals_sorted[pos] = ovals[i];
}

// chunk_ptr[strip][c] = first entry of the strip with column >= 64 * c (c = 0 .. n_cols / 64).
__global__ void __launch_bounds__(DQ_THREADS)
chunk_ptr_kernel(const int64_t *oidx, int64_t n_rows, int64_t n_cols, const int32_t *row_ptr, int64_t n_strips,
                 int n_chunks, int32_t *chunk_ptr) {
    const int64_t i = (int64_t)blockIdx.x * DQ_THREADS + threadIdx.x;
    if (i >= n_strips * (n_chunks + 1)) return;
    const int64_t strip = i / (n_chunks + 1);
    const int c = (int)(i - strip * (n_chunks + 1));
    const int64_t r0 = strip * 16;
    if (r0 >= n_rows) { chunk_ptr[i] = row_ptr[n_rows]; return; }
    int count = 0;
    for (int64_t r = r0; r < r0 + 16 && r < n_rows; ++r) {
        const int64_t key = r * n_cols + (int64_t)c * 64;
        int lo = row_ptr[r], hi = row_ptr[r + 1];
        const int base = lo;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (oidx[mid] < key) lo = mid + 1; else hi = mid;
        }
        count += lo - base;
    }
    chunk_ptr[i] = row_ptr[r0] + count;
}

}  // namespace
}  // namespace atlas

extern "C" {

int atlas_dequantize(const int8_t *codes, int64_t n_codes, const void *outlier_vals,
                     const int64_t *outlier_idx, int64_t n_outliers, const void *scales, int64_t numel,
                     int block_size, void *w_out, void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(numel < 0 || n_codes < 0 || n_outliers < 0 || block_size < 1, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_dequantize: negative size or block_size < 1");
    if (numel == 0) return ATLAS_OK;
    const int64_t padded = ceil_div_i64(numel, block_size) * block_size;
    ATLAS_RETURN_IF(n_codes + n_outliers != padded, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_dequantize: %lld codes + %lld outliers do not cover %lld padded elements",
                    (long long)n_codes, (long long)n_outliers, (long long)padded);
    ATLAS_RETURN_IF(!w_out || !scales || (n_codes && !codes) || (n_outliers && (!outlier_vals || !outlier_idx)),
                    ATLAS_ERR_BAD_ARGUMENT, "atlas_dequantize: null buffer");
    int rc = check_device();
    if (rc) return rc;
    const int64_t grid = ceil_div_i64(padded, DQ_SPAN);
    ATLAS_RETURN_IF(grid > 0x7fffffff, ATLAS_ERR_UNSUPPORTED, "atlas_dequantize: tensor too large");
    dequantize_kernel<<<(unsigned)grid, DQ_THREADS, 0, (cudaStream_t)stream>>>(
        codes, n_codes, (const uint16_t *)outlier_vals, outlier_idx, n_outliers, (const uint16_t *)scales,
        numel, padded, block_size, (uint16_t *)w_out);
    return check_cuda(cudaGetLastError(), "dequantize_kernel launch");
}

size_t atlas_tiles_bytes(int64_t n_rows, int64_t n_cols) {
    if (n_rows <= 0 || n_cols <= 0) return 0;
    return (size_t)(atlas::ceil_div_i64(n_rows, 128) * 128 * n_cols);
}

int atlas_repack(const int8_t *codes, int64_t n_codes, const void *outlier_vals, const int64_t *outlier_idx,
                 int64_t n_outliers, const void *scales, int64_t n_rows, int64_t n_cols, int block_size,
                 uint8_t *tiles, void *scales_tiled, int32_t *outlier_row_ptr, int32_t *outlier_chunk_ptr,
                 uint32_t *outlier_entries, void *outlier_vals_sorted, void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(n_rows <= 0 || n_cols <= 0 || n_codes < 0 || n_outliers < 0 || block_size < 1,
                    ATLAS_ERR_BAD_ARGUMENT, "atlas_repack: bad size");
    ATLAS_RETURN_IF(n_cols % 64 != 0 || block_size % 16 != 0 || n_cols % block_size != 0,
                    ATLAS_ERR_UNSUPPORTED,
                    "atlas_repack: needs n_cols %% 64 == 0, block_size %% 16 == 0 and n_cols %% block_size == 0 "
                    "(got n_cols=%lld block_size=%d)", (long long)n_cols, block_size);
    ATLAS_RETURN_IF(n_cols >= (1 << 24) || n_outliers > 0x7fffffff, ATLAS_ERR_UNSUPPORTED,
                    "atlas_repack: n_cols >= 2^24 or more than 2^31 outliers");
    ATLAS_RETURN_IF(n_codes + n_outliers != n_rows * n_cols, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_repack: %lld codes + %lld outliers do not cover %lld x %lld",
                    (long long)n_codes, (long long)n_outliers, (long long)n_rows, (long long)n_cols);
    ATLAS_RETURN_IF(!tiles || !scales || !scales_tiled || !outlier_row_ptr || !outlier_chunk_ptr ||
                        (n_codes && !codes) ||
                        (n_outliers && (!outlier_idx || !outlier_vals || !outlier_entries || !outlier_vals_sorted)),
                    ATLAS_ERR_BAD_ARGUMENT, "atlas_repack: null buffer");
    ATLAS_RETURN_IF(((uintptr_t)tiles & 15) != 0, ATLAS_ERR_BAD_ARGUMENT, "atlas_repack: tiles must be 16-byte aligned");
    int rc = check_device();
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t numel = n_rows * n_cols;
    const int64_t grid = ceil_div_i64(numel, DQ_SPAN);
    ATLAS_RETURN_IF(grid > 0x7fffffff, ATLAS_ERR_UNSUPPORTED, "atlas_repack: tensor too large");
    repack_kernel<<<(unsigned)grid, DQ_THREADS, 0, st>>>(codes, n_codes, outlier_idx, n_outliers, n_rows,
                                                         n_cols, tiles);
    rc = check_cuda(cudaGetLastError(), "repack_kernel launch");
    if (rc) return rc;
    const int64_t rows_padded = ceil_div_i64(n_rows, 128) * 128;
    if (rows_padded > n_rows) {
        const int64_t total = (rows_padded - n_rows) * n_cols;
        const int64_t g = ceil_div_i64(total, DQ_THREADS);
        repack_pad_kernel<<<(unsigned)(g < 4096 ? g : 4096), DQ_THREADS, 0, st>>>(n_rows, rows_padded, n_cols, tiles);
        rc = check_cuda(cudaGetLastError(), "repack_pad_kernel launch");
        if (rc) return rc;
    }
    const int64_t bpr = n_cols / block_size;
    {
        const int64_t g = ceil_div_i64(rows_padded * bpr, DQ_THREADS);
        scales_tile_kernel<<<(unsigned)(g < 8192 ? g : 8192), DQ_THREADS, 0, st>>>(
            (const uint16_t *)scales, n_rows, rows_padded, bpr, (uint16_t *)scales_tiled);
        rc = check_cuda(cudaGetLastError(), "scales_tile_kernel launch");
        if (rc) return rc;
    }
    row_ptr_kernel<<<(unsigned)ceil_div_i64(n_rows + 1, DQ_THREADS), DQ_THREADS, 0, st>>>(
        outlier_idx, n_outliers, n_rows, n_cols, outlier_row_ptr);
    rc = check_cuda(cudaGetLastError(), "row_ptr_kernel launch");
    if (rc) return rc;
    if (n_outliers > 0) {
        strip_sort_kernel<<<(unsigned)ceil_div_i64(n_outliers, DQ_THREADS), DQ_THREADS, 0, st>>>(
            outlier_idx, (const uint16_t *)outlier_vals, n_outliers, n_rows, n_cols, outlier_row_ptr,
            outlier_entries, (uint16_t *)outlier_vals_sorted);
        rc = check_cuda(cudaGetLastError(), "strip_sort_kernel launch");
        if (rc) return rc;
    }
    const int64_t n_strips = rows_padded / 16;
    const int n_chunks = (int)(n_cols / 64);
    chunk_ptr_kernel<<<(unsigned)ceil_div_i64(n_strips * (n_chunks + 1), DQ_THREADS), DQ_THREADS, 0, st>>>(
        outlier_idx, n_rows, n_cols, outlier_row_ptr, n_strips, n_chunks, outlier_chunk_ptr);
    return check_cuda(cudaGetLastError(), "chunk_ptr_kernel launch");
}

}  // extern "C"
