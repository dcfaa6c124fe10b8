/*
 * atlas_b200.h -- C ABI of the B200 (sm_100a) implementation of AtlasInfer's
 * adaptive hybrid quantization path.
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes,
 * enqueues its work on the CUDA stream it is given and returns an int status
 * (0 = ok).  The library owns no memory: every buffer, workspace included,
 * belongs to the caller, and no pointer is kept after a call returns.  There
 * is no CPU fallback; a call made without a usable GPU returns an error.
 *
 * fp16 / bf16 buffers are passed as `void*` (raw 16-bit patterns).
 *
 * Citations name files of the reference project (nishantkluhera/AtlasInfer).
 */
#ifndef ATLAS_B200_H_
#define ATLAS_B200_H_

#include <stddef.h>
#include <stdint.h>

/* Exported with default visibility; everything else in the library is hidden. */
#if defined(__GNUC__)
#define ATLAS_API __attribute__((visibility("default")))
#else
#define ATLAS_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define ATLAS_OK 0
#define ATLAS_ERR_BAD_ARGUMENT 1   /* null pointer, negative size, bad dtype     */
#define ATLAS_ERR_UNSUPPORTED 2    /* shape / block size outside the fast path   */
#define ATLAS_ERR_CAPACITY 3       /* an output or workspace buffer is too small */
#define ATLAS_ERR_LAUNCH 4         /* CUDA reported an error (see last_error)    */
#define ATLAS_ERR_TIMEOUT 5        /* a bounded device-side wait ran out         */
#define ATLAS_ERR_NO_DEVICE 6      /* no CUDA device / wrong architecture        */

/* activation / output element types */
#define ATLAS_DTYPE_F16 0
#define ATLAS_DTYPE_BF16 1

/* Library version (major*10000 + minor*100 + patch). */
ATLAS_API int atlas_version(void);
/* Text of the last error raised on the calling thread ("" if none). */
ATLAS_API const char *atlas_last_error(void);
/* Fixed text for a status code. */
ATLAS_API const char *atlas_status_string(int status);

/* ---- quantize ------------------------------------------------------------
 * Replaces quantize_tensor(fp16_tensor, block_size, z_threshold)
 * (atlasinfer_core/quant/adaptive_quantizer.py:51-148) for a tensor already in
 * device memory.  The flat input is zero-padded to a whole number of blocks;
 * per block the z-score outlier test (:44-49, :106-107), the fp16 scale
 * absmax/127 (:121-123) and the int8 codes (:125-126) are evaluated exactly as
 * PyTorch's CPU kernels do, so all four output streams are bit-identical to
 * the reference's.
 *
 *   w              numel fp16 values
 *   block_size     multiple of 32, 32..512 (others: ATLAS_ERR_UNSUPPORTED);
 *                  32 / 64 / 128 / 256 take the fast kernel
 *   z_threshold    as given to the reference; rounded to fp16 inside
 *   codes          capacity padded_numel int8  (compacted non-outlier codes)
 *   outlier_vals   capacity outlier_capacity fp16
 *   outlier_idx    capacity outlier_capacity int64 (flat index, padded tensor)
 *   scales         n_blocks fp16
 *   counts         4 x int64 on the device: [0] n_codes, [1] n_outliers
 *                  (the true count even when it exceeds outlier_capacity, in
 *                  which case only the first outlier_capacity entries were
 *                  stored and the caller retries with more room), [2] non-zero
 *                  if a bounded wait ran out (results invalid), [3] reserved
 *   workspace      atlas_quantize_workspace_bytes(numel, block_size) bytes
 *                  of scratch, 16-byte aligned; contents are irrelevant
 *                  before and after the call
 */
ATLAS_API size_t atlas_quantize_workspace_bytes(int64_t numel, int block_size);
ATLAS_API int atlas_quantize(const void *w, int64_t numel, int block_size, double z_threshold,
                   int8_t *codes, void *outlier_vals, int64_t *outlier_idx,
                   int64_t outlier_capacity, void *scales, int64_t *counts,
                   void *workspace, size_t workspace_bytes, void *stream);

/* ---- quantize for callers that cannot allocate -------------------------------
 * No counterpart in the reference.  Same computation and outputs as
 * atlas_quantize, but the look-back scratch lives in a device array inside the
 * library instead of a caller-provided workspace, and the call performs no
 * device or host allocation (it issues two cudaMemsetAsync and one kernel).
 * Meant for hosts that must not allocate where they quantize: a fixed,
 * pre-reserved memory arena, a serving loop that forbids cudaMalloc after
 * start-up, a plug-in that does not own the allocator.
 *
 *  - limit: ceil(numel / block_size) * block_size <=
 *    ATLAS_QUANTIZE_NOALLOC_MAX_ELEMENTS (64 Mi elements, e.g. 8192 x 8192;
 *    about 0.4 % fewer for block sizes that do not divide 8192);
 *    larger inputs return ATLAS_ERR_CAPACITY and must use atlas_quantize.
 *    The array (64 KB + 16 B) is held by every GPU context that loads the
 *    library, until the process exits.
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress); make that first call outside any stream capture.
 *    The address is cached per device ordinal for the life of the process: a
 *    cudaDeviceReset() destroys the array it points to, so do not call this
 *    entry point again on a device that was reset.
 *  - all calls on a device share the array: it is cleared on the stream at the
 *    start of every call, and two calls whose kernels may overlap on the GPU
 *    (different streams without ordering) race.  Serialise them.
 */
#define ATLAS_QUANTIZE_NOALLOC_MAX_ELEMENTS ((int64_t)1 << 26)
ATLAS_API int atlas_quantize_noalloc(const void *w, int64_t numel, int block_size, double z_threshold,
                                     int8_t *codes, void *outlier_vals, int64_t *outlier_idx,
                                     int64_t outlier_capacity, void *scales, int64_t *counts,
                                     void *stream);

/* ---- dequantize ------------------------------------------------------------
 * Replaces dequantize_tensor(quant_data, target_device)
 * (adaptive_quantizer.py:156-251) minus its id()-keyed cache: writes the
 * numel fp16 values fp16(fp16(code) * scale) / raw outlier values (:216,
 * :221-235).  Any block_size >= 1 and any numel are accepted.
 */
ATLAS_API int atlas_dequantize(const int8_t *codes, int64_t n_codes, const void *outlier_vals,
                     const int64_t *outlier_idx, int64_t n_outliers, const void *scales,
                     int64_t numel, int block_size, void *w_out, void *stream);

/* ---- repack to the kernel layout -----------------------------------------------
 * No counterpart in the reference (which re-derives positions per block at
 * adaptive_quantizer.py:187-212 and caches an fp16 copy).  Expands the
 * compacted streams of a quantized [n_rows, n_cols] weight into the layout the
 * linear kernels stream:
 *
 *   tiles            atlas_tiles_bytes(n_rows, n_cols) bytes; code + 128 as
 *                    uint8 (outlier positions hold 128, i.e. code 0), ordered
 *                    [row/128][col/64][row%128][col%64] (every 128-row x
 *                    64-column tile is a contiguous 8 KB matrix of 64-byte
 *                    rows); rows padded to a multiple of 128; 16-byte aligned
 *   scales_tiled     atlas_tiles_bytes / block_size fp16: the scales ordered
 *                    [row/128][block][row%128] (0 for padding rows)
 *   outlier_row_ptr  n_rows + 1 int32: CSR row starts into the canonical
 *                    outlier streams
 *   outlier_chunk_ptr  (rows_padded/16) x (n_cols/64 + 1) int32: for each
 *                    16-row strip, the first entry with column >= 64*c
 *   outlier_entries  n_outliers uint32, (row%16) << 24 | column, grouped by
 *                    strip and sorted by column within a strip
 *   outlier_vals_sorted  n_outliers fp16 in the order of outlier_entries
 *
 * Requires n_cols % 64 == 0, n_cols < 2^24 and n_cols % block_size == 0 with
 * block_size a multiple of 16 (blocks never straddle rows), else
 * ATLAS_ERR_UNSUPPORTED.
 */
ATLAS_API size_t atlas_tiles_bytes(int64_t n_rows, int64_t n_cols);
ATLAS_API int atlas_repack(const int8_t *codes, int64_t n_codes, const void *outlier_vals,
                           const int64_t *outlier_idx, int64_t n_outliers, const void *scales,
                           int64_t n_rows, int64_t n_cols, int block_size, uint8_t *tiles,
                           void *scales_tiled, int32_t *outlier_row_ptr, int32_t *outlier_chunk_ptr,
                           uint32_t *outlier_entries, void *outlier_vals_sorted, void *stream);

/* ---- quantized linear forward ----------------------------------------------------
 * Replaces QuantizedLinear.forward (integration/atlas_wrappers.py:30-74):
 * y[m][n] = sum_k x[m][k] * W[n][k] + bias[n], W being the dequantized weight
 * of dequantize_tensor, never materialised.  The weight is given in the
 * layout atlas_repack writes.  x and y share `dtype` (ATLAS_DTYPE_F16 as in
 * the reference, or ATLAS_DTYPE_BF16); bias is fp16 or NULL.  ldx / ldy are
 * row strides in elements.  bf16 activations are used as fp16 inside
 * (|x| > 65504 saturates).  `status` is a caller-owned device int32 (or NULL)
 * that a kernel sets non-zero if one of its bounded waits ran out; the library
 * never clears it.
 *
 * atlas_qlinear_gemv: decode shapes, any m >= 1 (intended for m <= 16).  HBM-
 * bound: the rows of x are served up to 16 at a time by a kernel that gives
 * each CTA one 16-row strip of the weight, streams its codes with 16-byte
 * loads, dequantises in registers and adds the outlier products in the same
 * launch (passes after the first find most of the weight in L2).  Activations
 * that are not 16-byte aligned are read two bytes at a time.  Launched with
 * programmatic dependent launch: only weights are read before the stream's
 * earlier work has completed.  The kernel has no bounded wait: `status` is
 * accepted for symmetry and never written.
 *
 * atlas_qlinear_gemm: larger batches (any m >= 1 accepted).  The code tiles
 * come in by TMA, are dequantised by 16 warps straight into tensor memory as
 * the fp16 A operand of tcgen05.mma (the activations are the B operand, from
 * shared memory; fp32 accumulators in tensor memory); the token tile is 32,
 * 64, 128 or 256 wide by m, and for decode-sized batches K is sliced over CTAs
 * with the fp32 partial tiles added in slice order by a second kernel
 * (deterministic).
 * `workspace` must hold atlas_qlinear_gemm_workspace_bytes(m, n_rows, n_cols)
 * bytes, 256-byte aligned.
 */
ATLAS_API int atlas_qlinear_gemv(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                 const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                 const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                 int64_t n_rows, int64_t n_cols, int block_size, const void *bias, void *y,
                                 int64_t ldy, int32_t *status, void *stream);

/* atlas_qlinear_stream: decode shapes, the weight read once for up to 32 rows
 * of x per launch (more rows: one pass per 32).  One persistent CTA per SM; the
 * 8 KB code tiles, taken row-tile-major, are cut into equal contiguous ranges,
 * one per CTA, and stream through a shared-memory ring of bulk copies that the
 * CTA starts filling before the stream's earlier work has completed
 * (programmatic dependent launch; two consecutive launches are co-resident on
 * an SM).  Row tiles whose K range is shared between CTAs are finished by the
 * CTA that arrives last, which adds the fp32 partial tiles in CTA order
 * (deterministic; no CTA waits for another).
 *
 * `workspace`: atlas_qlinear_stream_workspace_bytes(m) bytes, 16-byte aligned,
 * ZERO-FILLED before its first use.  Every call leaves it zero-filled where it
 * must be, so one workspace serves any number of calls of any shape that are
 * ordered on one stream; calls that may overlap on the GPU need separate
 * workspaces.  After a call that reported a timed-out wait through `status`,
 * zero it again.
 *
 * Preconditions shared by the three linear entry points: the weight-side
 * buffers (tiles, scales_tiled, outlier_*) are read before the stream's
 * earlier work has completed, so they must be final before the kernel that
 * precedes the call on the stream was launched (synchronise once after
 * atlas_repack).  x, bias, y, workspace and status are only touched afterwards.
 */
ATLAS_API size_t atlas_qlinear_stream_workspace_bytes(int64_t m);
ATLAS_API int atlas_qlinear_stream(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                   const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                   const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                   int64_t n_rows, int64_t n_cols, int block_size, const void *bias, void *y,
                                   int64_t ldy, void *workspace, size_t workspace_bytes, int32_t *status,
                                   void *stream);

/* ---- column-parallel linear with the gather fused into the kernel ---------------
 * No counterpart in the reference (it is single-process; nothing to cite).
 * For a weight sharded by output rows over `world` GPUs of one node, each rank
 * computes its [m, n_rows] shard with atlas_qlinear_stream's kernel and stores
 * it straight into every rank's gathered output (plain peer stores over
 * NVLink; no TMA, no multicast), instead of writing y locally and calling an
 * all-gather.  When its last CTA has finished, the rank publishes an arrival
 * count into every rank's flag array; a consumer of the gathered buffer waits
 * until all `world` flags have reached its own rank's count.  That wait is part
 * of this kernel's prologue when `wait_flags` is given (its x is then a
 * gathered buffer: it is read only after the wait, through L2), and is
 * available on its own as atlas_peer_wait.  Every wait polls at most
 * `poll_limit` times; when it runs out the kernel sets `status` and goes on.
 *
 *   world, rank   ranks sharing the weight (1..ATLAS_MAX_PEERS), this rank
 *   y_dst[d]      address on rank d where element (row 0, first output
 *                 feature of THIS rank) goes; row stride `ldy` elements
 *                 (y_dst[rank] is local memory, the others are peer mappings)
 *   flags_dst[d]  rank d's arrival flags (`world` x uint32); this rank writes
 *                 entry [rank]
 *   state         local, 2 x uint32, zero before first use: CTAs finished,
 *                 gather launches completed (the arrival count)
 *   wait_flags    local arrival flags to wait on before x is read, or NULL
 *   poll_limit    polls per wait (each ~0.1 us)
 * The peer mappings come from atlas_peer_alloc / _export / _import below (or
 * any other inter-process mapping of plain device memory).
 */
#define ATLAS_MAX_PEERS 8
typedef struct AtlasPeerGather {
    int32_t world;
    int32_t rank;
    void *y_dst[ATLAS_MAX_PEERS];
    uint32_t *flags_dst[ATLAS_MAX_PEERS];
    uint32_t *state;
    const uint32_t *wait_flags;
    int64_t poll_limit;
} AtlasPeerGather;

ATLAS_API int atlas_qlinear_stream_gather(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                          const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                          const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                          int64_t n_rows, int64_t n_cols, int block_size, const void *bias,
                                          int64_t ldy, void *workspace, size_t workspace_bytes, int32_t *status,
                                          void *stream, const AtlasPeerGather *gather);

/* The same gather behind the tcgen05 path of atlas_qlinear_gemm, for m <= 64:
 * the kernel that adds the K-slice partial tiles writes y into every rank's
 * buffer and publishes the arrival; with `wait_flags` the kernel that copies x
 * to fp16 waits first (bounded).  No extra launch.  `workspace` as for
 * atlas_qlinear_gemm. */
ATLAS_API int atlas_qlinear_gemm_gather(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                        const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                        const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                        int64_t n_rows, int64_t n_cols, int block_size, const void *bias,
                                        int64_t ldy, void *workspace, size_t workspace_bytes, int32_t *status,
                                        void *stream, const AtlasPeerGather *gather);

/* Waits (one small kernel on `stream`) until all `world` entries of `flags`
 * have reached the count in state[1]; sets *status non-zero if `poll_limit`
 * polls were not enough.  For consumers of a gathered buffer that are not
 * atlas kernels. */
ATLAS_API int atlas_peer_wait(const uint32_t *flags, int world, const uint32_t *state, int64_t poll_limit,
                              int32_t *status, void *stream);

/* The gather without the linear: copies this rank's finished shard `src`
 * (`rows` x `row_bytes`, rows `src_pitch_bytes` apart) to gather->y_dst[d]
 * (rows `dst_pitch_bytes` apart) on every rank d with plain peer stores and
 * publishes the arrival exactly as atlas_qlinear_stream_gather does (same
 * flags, same state, interchangeable launch by launch).  For shards computed
 * by atlas_qlinear_gemv / atlas_qlinear_gemm: one small kernel instead of a
 * collective.  gather->wait_flags and poll_limit are not used (the kernel
 * waits for nothing; a consumer waits through atlas_peer_wait). */
ATLAS_API int atlas_peer_push(const void *src, int64_t rows, int64_t row_bytes, int64_t src_pitch_bytes,
                              int64_t dst_pitch_bytes, const AtlasPeerGather *gather, void *stream);

/* Device memory that other processes of the node can map: plain cudaMalloc
 * memory (zero-filled), exported / imported as CUDA IPC handles (64 bytes).
 * These four calls are the only ones in the library that own memory; it is
 * freed by atlas_peer_free (imports by atlas_peer_release). */
#define ATLAS_PEER_HANDLE_BYTES 64
ATLAS_API int atlas_peer_alloc(size_t bytes, void **ptr);
ATLAS_API int atlas_peer_free(void *ptr);
ATLAS_API int atlas_peer_export(void *ptr, unsigned char *handle);
ATLAS_API int atlas_peer_import(const unsigned char *handle, void **ptr);
ATLAS_API int atlas_peer_release(void *ptr);

ATLAS_API size_t atlas_qlinear_gemm_workspace_bytes(int64_t m, int64_t n_rows, int64_t n_cols);
ATLAS_API int atlas_qlinear_gemm(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                 const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                 const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                 int64_t n_rows, int64_t n_cols, int block_size, const void *bias, void *y,
                                 int64_t ldy, void *workspace, size_t workspace_bytes, int32_t *status,
                                 void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ATLAS_B200_H_ */
