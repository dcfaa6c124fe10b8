// Decode-time quantized linear: y[m][n] = sum_k x[m][k] * W[n][k] + bias[n], m <= 32.
//
// Replaces the steady state of QuantizedLinear.forward
// (integration/atlas_wrappers.py:56,67), which multiplies by a cached fp16
// copy of the weight (2 bytes per weight).  Here the kernel streams the
// tile-major uint8 codes (1 byte per weight) with 128-bit loads, rebuilds in
// registers exactly the fp16 weight the reference's dequantizer produces
// (adaptive_quantizer.py:216: fp16(fp16(code) * scale)), feeds it to the
// tensor cores as the 16-row operand with the activations as the 8-column
// operand, and adds the fp16 outlier products from the CSR side-table in the
// same launch.  The kernel is HBM-bound; the MMA is only the cheapest way to
// do the multiply-adds without unpacking to fp32.
//
// Work split: a CTA owns R = 16 * (8 / WK) weight rows and one slice of the
// K dimension; the S CTAs of a thread-block cluster own the S slices of the
// same rows and add their partial sums through distributed shared memory in
// a fixed order (deterministic, no atomics, no scratch in global memory).
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace atlas {
namespace {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = 8;
constexpr int GV_UNROLL = 4;  // k-tiles (64 columns each) loaded per batch and warp

struct GemvParams {
    const void *x;
    int dtype;
    int m;          // rows of x handled by this launch (<= 8 * MT)
    int64_t ldx;
    const uint8_t *tiles;
    const uint16_t *scales;
    const int32_t *row_ptr;
    const int32_t *ocol;
    const uint16_t *ovals;
    int n_rows;
    int n_cols;
    int bs;
    const uint16_t *bias;
    void *y;
    int64_t ldy;
    int k_tiles;     // n_cols / 64
    int kc_tiles;    // k-tiles staged per pass (x slice in shared memory)
    int splits;      // cluster size S
    int x_vec_ok;    // x rows allow 16-byte loads
};

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four biased codes (code + 128 per byte) -> two half2 of fp16(fp16(code) * scale).
__device__ __forceinline__ void dequant4(uint32_t w, __half2 scale2, uint32_t &lo, uint32_t &hi) {
    const uint32_t l = __byte_perm(w, 0x64646464u, 0x5140);  // halves 1024 + u0, 1024 + u1
    const uint32_t h = __byte_perm(w, 0x64646464u, 0x5342);  // halves 1024 + u2, 1024 + u3
    const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));  // 1152
    __half2 lv = __hsub2(*reinterpret_cast<const __half2 *>(&l), bias);  // exact integer code
    __half2 hv = __hsub2(*reinterpret_cast<const __half2 *>(&h), bias);
    lv = __hmul2(lv, scale2);  // the reference's single fp16 rounding
    hv = __hmul2(hv, scale2);
    lo = *reinterpret_cast<uint32_t *>(&lv);
    hi = *reinterpret_cast<uint32_t *>(&hv);
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    float lo = __uint_as_float(v << 16);
    float hi = __uint_as_float(v & 0xffff0000u);
    lo = fminf(fmaxf(lo, -65504.f), 65504.f);
    hi = fminf(fmaxf(hi, -65504.f), 65504.f);
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// MT: 8-column MMA tiles over the batch (m <= 8 * MT).  WK: warps sharing a 16-row strip along K.
template <int MT, int WK>
__global__ void __launch_bounds__(GV_THREADS) gemv_kernel(GemvParams p) {
    constexpr int MTOT = MT * 8;
    constexpr int WR = GV_WARPS / WK;  // 16-row strips per CTA
    constexpr int R = WR * 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int strip_local = warp / WK, wk = warp % WK;
    const int split = blockIdx.x;  // == rank in the cluster along K
    const int n0 = blockIdx.y * R;

    // this CTA's k-tiles
    const int kt_begin = (int)((int64_t)p.k_tiles * split / p.splits);
    const int kt_end = (int)((int64_t)p.k_tiles * (split + 1) / p.splits);

    const int xs_stride = p.kc_tiles * 64 + 8;  // halves; +8 keeps 128-bit reads conflict-free
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem_raw);
    float *ytile = reinterpret_cast<float *>(smem_raw + (((size_t)MTOT * xs_stride * 2 + 15) & ~(size_t)15));
    // ytile: [WK + 1][MTOT][R]; slab WK collects the outlier products

    for (int e = tid; e < (WK + 1) * MTOT * R; e += GV_THREADS) ytile[e] = 0.f;
    __syncthreads();

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // location of this warp's strip in the tile-major layout
    const int row_strip = n0 + strip_local * 16;          // first weight row of the strip
    const int64_t rt = row_strip >> 7;
    const int strip_in_tile = (row_strip & 127) >> 4;
    const uint8_t *strip_base = p.tiles + ((rt * p.k_tiles) * 8 + strip_in_tile) * 1024 + lane * 16;
    const int row_a = row_strip + g, row_b = row_a + 8;
    const int sc_per_row = p.n_cols / p.bs;
    const bool row_a_ok = row_a < p.n_rows, row_b_ok = row_b < p.n_rows;

    // outlier cursor: thread r < R walks row n0 + r of the CSR side-table
    int o_cur = 0, o_end = 0;
    if (tid < R && n0 + tid < p.n_rows) {
        o_cur = p.row_ptr[n0 + tid];
        o_end = p.row_ptr[n0 + tid + 1];
        const int kb = kt_begin * 64;
        int lo = o_cur, hi = o_end;
        while (lo < hi) {  // first outlier at or after this CTA's first column
            int mid = (lo + hi) >> 1;
            if (p.ocol[mid] < kb) lo = mid + 1; else hi = mid;
        }
        o_cur = lo;
    }

    for (int pass_begin = kt_begin; pass_begin < kt_end; pass_begin += p.kc_tiles) {
        const int pass_end = min(pass_begin + p.kc_tiles, kt_end);
        const int pass_cols = (pass_end - pass_begin) * 64;
        const int col0 = pass_begin * 64;
        __syncthreads();  // previous pass no longer reads xs (also orders the ytile zeroing)
        // ---- stage x[:, col0 : col0 + pass_cols] as fp16 ------------------------------
        {
            const int vec_per_row = pass_cols >> 3;
            for (int idx = tid; idx < MTOT * vec_per_row; idx += GV_THREADS) {
                const int m = idx / vec_per_row, v = idx - m * vec_per_row;
                uint4 val = make_uint4(0, 0, 0, 0);
                if (m < p.m) {
                    const uint16_t *src = reinterpret_cast<const uint16_t *>(p.x) + (int64_t)m * p.ldx + col0 + v * 8;
                    if (p.x_vec_ok) {
                        val = *reinterpret_cast<const uint4 *>(src);
                    } else {
                        val.x = src[0] | (uint32_t)src[1] << 16;
                        val.y = src[2] | (uint32_t)src[3] << 16;
                        val.z = src[4] | (uint32_t)src[5] << 16;
                        val.w = src[6] | (uint32_t)src[7] << 16;
                    }
                    if (p.dtype == ATLAS_DTYPE_BF16) {
                        val.x = bf16x2_to_f16x2(val.x);
                        val.y = bf16x2_to_f16x2(val.y);
                        val.z = bf16x2_to_f16x2(val.z);
                        val.w = bf16x2_to_f16x2(val.w);
                    }
                }
                *reinterpret_cast<uint4 *>(xs + m * xs_stride + v * 8) = val;
            }
        }
        __syncthreads();

        // ---- dense part: this warp's k-tiles of the pass, GV_UNROLL at a time ---------------
        for (int kt0 = pass_begin + wk; kt0 < pass_end; kt0 += WK * GV_UNROLL) {
            uint4 wa[GV_UNROLL], wb[GV_UNROLL];
#pragma unroll
            for (int u = 0; u < GV_UNROLL; ++u) {
                const int kt = kt0 + u * WK;
                if (kt < pass_end) {
                    const uint8_t *tp = strip_base + (int64_t)kt * 8192;
                    wa[u] = __ldcs(reinterpret_cast<const uint4 *>(tp));        // row g,   16 codes
                    wb[u] = __ldcs(reinterpret_cast<const uint4 *>(tp + 512));  // row g+8, 16 codes
                }
            }
#pragma unroll
            for (int u = 0; u < GV_UNROLL; ++u) {
                const int kt = kt0 + u * WK;
                if (kt < pass_end) {
                    const int kb = (kt * 64 + tig * 16) / p.bs;
                    const __half sa = row_a_ok ? __ushort_as_half(__ldg(p.scales + (int64_t)row_a * sc_per_row + kb))
                                               : __ushort_as_half((uint16_t)0);
                    const __half sb = row_b_ok ? __ushort_as_half(__ldg(p.scales + (int64_t)row_b * sc_per_row + kb))
                                               : __ushort_as_half((uint16_t)0);
                    const __half2 sa2 = __half2half2(sa), sb2 = __half2half2(sb);
                    const uint32_t wav[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w};
                    const uint32_t wbv[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
                    uint32_t a_lo[4], a_hi[4], b_lo[4], b_hi[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        dequant4(wav[i], sa2, a_lo[i], a_hi[i]);
                        dequant4(wbv[i], sb2, b_lo[i], b_hi[i]);
                    }
                    const int xoff = (kt - pass_begin) * 64 + tig * 16;
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt) {
                        const uint4 x0 = *reinterpret_cast<const uint4 *>(xs + (nt * 8 + g) * xs_stride + xoff);
                        const uint4 x1 = *reinterpret_cast<const uint4 *>(xs + (nt * 8 + g) * xs_stride + xoff + 8);
                        const uint32_t xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            mma_f16(acc[nt], a_lo[i], b_lo[i], a_hi[i], b_hi[i], xv[2 * i], xv[2 * i + 1]);
                    }
                }
            }
        }

        // ---- sparse part: outliers of rows n0..n0+R-1 inside this pass's columns -----------
        if (tid < R) {
            float *yo = ytile + (size_t)WK * MTOT * R + tid;
            const int col_end = col0 + pass_cols;
            while (o_cur < o_end) {
                const int c = __ldg(p.ocol + o_cur);
                if (c >= col_end) break;
                const float v = __half2float(__ushort_as_half(__ldg(p.ovals + o_cur)));
                const uint16_t *xc = xs + (c - col0);
#pragma unroll 4
                for (int m = 0; m < MTOT; ++m)
                    yo[m * R] = fmaf(v, __half2float(__ushort_as_half(xc[m * xs_stride])), yo[m * R]);
                ++o_cur;
            }
        }
    }

    // ---- accumulators -> this warp's slab ------------------------------------------------
    {
        float *slab = ytile + (size_t)wk * MTOT * R + strip_local * 16;
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            const int m0 = nt * 8 + tig * 2;
            slab[(m0 + 0) * R + g] = acc[nt][0];
            slab[(m0 + 1) * R + g] = acc[nt][1];
            slab[(m0 + 0) * R + g + 8] = acc[nt][2];
            slab[(m0 + 1) * R + g + 8] = acc[nt][3];
        }
    }
    __syncthreads();
    // fold the slabs of this CTA in a fixed order into slab 0
    for (int e = tid; e < MTOT * R; e += GV_THREADS) {
        float s = ytile[e];
#pragma unroll
        for (int k = 1; k <= WK; ++k) s += ytile[(size_t)k * MTOT * R + e];
        ytile[e] = s;
    }

    // ---- add the K slices across the cluster and write y -----------------------------------
    cg::cluster_group cluster = cg::this_cluster();
    if (p.splits > 1) cluster.sync(); else __syncthreads();
    {
        const int total = p.m * R;  // only real batch rows
        const int e_begin = (int)((int64_t)total * split / p.splits);
        const int e_end = (int)((int64_t)total * (split + 1) / p.splits);
        for (int e = e_begin + tid; e < e_end; e += GV_THREADS) {
            const int m = e / R, r = e - m * R;
            const int n = n0 + r;
            if (n >= p.n_rows) continue;
            float s = 0.f;
            if (p.splits > 1) {
                for (int c = 0; c < p.splits; ++c) {
                    const float *remote = cluster.map_shared_rank(ytile, c);
                    s += remote[e];
                }
            } else {
                s = ytile[e];
            }
            if (p.bias) s += __half2float(__ushort_as_half(__ldg(p.bias + n)));
            if (p.dtype == ATLAS_DTYPE_BF16)
                reinterpret_cast<__nv_bfloat16 *>(p.y)[(int64_t)m * p.ldy + n] = __float2bfloat16_rn(s);
            else
                reinterpret_cast<__half *>(p.y)[(int64_t)m * p.ldy + n] = __float2half_rn(s);
        }
    }
    if (p.splits > 1) cluster.sync();  // peers may still be reading this CTA's shared memory
}

template <int MT, int WK>
int launch_gemv(const GemvParams &p, int row_groups, size_t smem, cudaStream_t st) {
    auto kern = gemv_kernel<MT, WK>;
    static thread_local size_t configured = 0;
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != configured_dev) { configured = 0; configured_dev = dev; }
    if (smem > configured) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                            "cudaFuncSetAttribute(gemv smem)");
        if (rc) return rc;
        configured = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.splits, (unsigned)row_groups, 1);
    cfg.blockDim = dim3(GV_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p), "gemv_kernel launch");
}

template <int MT>
int dispatch_wk(int wk, const GemvParams &p, int row_groups, size_t smem, cudaStream_t st) {
    switch (wk) {
        case 1: return launch_gemv<MT, 1>(p, row_groups, smem, st);
        case 2: return launch_gemv<MT, 2>(p, row_groups, smem, st);
        case 4: return launch_gemv<MT, 4>(p, row_groups, smem, st);
        default: return launch_gemv<MT, 8>(p, row_groups, smem, st);
    }
}

int sm_count() {
    static thread_local int dev_cached = -1, sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != dev_cached) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
        dev_cached = dev;
    }
    return sms;
}

}  // namespace
}  // namespace atlas

extern "C" int atlas_qlinear_gemv(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                  const void *scales, const int32_t *outlier_row_ptr,
                                  const int32_t *outlier_col, const void *outlier_vals, int64_t n_rows,
                                  int64_t n_cols, int block_size, const void *bias, void *y, int64_t ldy,
                                  void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(!x || !tiles || !scales || !outlier_row_ptr || !y, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemv: null buffer");
    ATLAS_RETURN_IF(m < 0 || n_rows <= 0 || n_cols <= 0 || ldx < n_cols || ldy < n_rows, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemv: bad size (m=%lld n_rows=%lld n_cols=%lld ldx=%lld ldy=%lld)",
                    (long long)m, (long long)n_rows, (long long)n_cols, (long long)ldx, (long long)ldy);
    ATLAS_RETURN_IF(dtype != ATLAS_DTYPE_F16 && dtype != ATLAS_DTYPE_BF16, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemv: dtype %d", dtype);
    ATLAS_RETURN_IF(n_cols % 64 != 0 || block_size < 16 || block_size % 16 != 0 || n_cols % block_size != 0,
                    ATLAS_ERR_UNSUPPORTED,
                    "atlas_qlinear_gemv: needs n_cols %% 64 == 0 and block_size a multiple of 16 dividing n_cols");
    ATLAS_RETURN_IF(n_rows > 0x7fffff00 || n_cols > 0x7fffff00, ATLAS_ERR_UNSUPPORTED, "atlas_qlinear_gemv: too large");
    ATLAS_RETURN_IF(((uintptr_t)tiles & 15) != 0, ATLAS_ERR_BAD_ARGUMENT, "atlas_qlinear_gemv: tiles not 16-byte aligned");
    int rc = check_device();
    if (rc) return rc;
    if (m == 0) return ATLAS_OK;
    cudaStream_t st = (cudaStream_t)stream;

    const int k_tiles = (int)(n_cols / 64);
    const int target = sm_count() * 3 / 2;
    for (int64_t m0 = 0; m0 < m; m0 += 32) {
        const int mg = (int)((m - m0) < 32 ? (m - m0) : 32);
        const int mt = mg <= 8 ? 1 : (mg <= 16 ? 2 : 4);
        // rows per CTA: the largest of 128/64/32/16 that still yields enough CTAs with 8 K slices
        int wk = 8;
        for (int cand = 1; cand <= 8; cand *= 2) {
            const int R = 16 * (GV_WARPS / cand);
            const int64_t groups = ceil_div_i64(n_rows, R);
            const int smax = k_tiles / cand >= 8 ? 8 : (k_tiles / cand >= 1 ? (k_tiles / cand) : 1);
            if (groups * smax >= target || cand == 8) { wk = cand; break; }
        }
        const int R = 16 * (GV_WARPS / wk);
        const int row_groups = (int)ceil_div_i64(n_rows, R);
        int smax = 1;
        while (smax * 2 <= 8 && k_tiles / (smax * 2) >= wk) smax *= 2;
        int splits = 1;
        while (splits < smax && (int64_t)row_groups * splits < target) splits *= 2;
        const int tiles_per_cta = (int)ceil_div_i64(k_tiles, splits);
        int kc_cap = 256 / (mt * 8);  // x slice <= 32 KB: 32 k-tiles at m<=8, 16 at m<=16, 8 at m<=32
        if (kc_cap < wk) kc_cap = wk;
        const int kc_tiles = tiles_per_cta < kc_cap ? tiles_per_cta : kc_cap;

        GemvParams p;
        p.x = (const char *)x + (size_t)m0 * ldx * 2;
        p.dtype = dtype;
        p.m = mg;
        p.ldx = ldx;
        p.tiles = tiles;
        p.scales = (const uint16_t *)scales;
        p.row_ptr = outlier_row_ptr;
        p.ocol = outlier_col;
        p.ovals = (const uint16_t *)outlier_vals;
        p.n_rows = (int)n_rows;
        p.n_cols = (int)n_cols;
        p.bs = block_size;
        p.bias = (const uint16_t *)bias;
        p.y = (char *)y + (size_t)m0 * ldy * 2;
        p.ldy = ldy;
        p.k_tiles = k_tiles;
        p.kc_tiles = kc_tiles;
        p.splits = splits;
        p.x_vec_ok = (((uintptr_t)x & 15) == 0) && (ldx % 8 == 0);

        const int mtot = mt * 8;
        const size_t xs_bytes = ((size_t)mtot * (kc_tiles * 64 + 8) * 2 + 15) & ~(size_t)15;
        const size_t y_bytes = (size_t)(wk + 1) * mtot * R * 4;
        const size_t smem = xs_bytes + y_bytes;
        if (mt == 1) rc = dispatch_wk<1>(wk, p, row_groups, smem, st);
        else if (mt == 2) rc = dispatch_wk<2>(wk, p, row_groups, smem, st);
        else rc = dispatch_wk<4>(wk, p, row_groups, smem, st);
        if (rc) return rc;
    }
    return ATLAS_OK;
}
