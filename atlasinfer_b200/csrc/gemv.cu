// Decode-time quantized linear: y[m][n] = sum_k x[m][k] * W[n][k] + bias[n], m <= 32.
//
// Replaces the steady state of QuantizedLinear.forward
// (integration/atlas_wrappers.py:56,67), which multiplies by a cached fp16
// copy of the weight (2 bytes per weight).  Here the kernel streams the
// tile-major uint8 codes (1 byte per weight), rebuilds in registers exactly
// the fp16 weight the reference's dequantizer produces
// (adaptive_quantizer.py:216: fp16(fp16(code) * scale)), feeds it to the
// tensor cores as the 16-row operand with the activations as the 8-column
// operand, and adds the fp16 outlier products in the same launch.  The
// kernel is HBM-bound; the MMA is only the cheapest way to do the
// multiply-adds without unpacking to fp32.
//
// Data movement: every warp owns a ring of 1 KB shared-memory slots that it
// fills with 1-D bulk asynchronous copies (one slot = the 16 rows x 64 columns
// of codes the warp consumes per step, contiguous in the tile-major layout)
// and drains through mbarrier waits, eight copies deep, so that the bytes in
// flight per SM do not depend on registers or occupancy.  The kernel is
// launched with programmatic dependent launch: barrier set-up, the first ring
// fills and the scale staging touch only weights and run before
// griddepcontrol.wait, i.e. while the previous kernel of the stream drains.
//
// Work split: a CTA owns R = 16 * (8 / WK) weight rows and one slice of the
// K dimension; the S CTAs of a thread-block cluster own the S slices of the
// same rows and add their partial sums through distributed shared memory in
// a fixed order (deterministic, no atomics, no scratch in global memory).
//
// Outliers: the side-table is regrouped by 16-row strip and sorted by column
// (atlas_repack).  A warp turns 16 outliers of its strip at a time into one
// more MMA: the A fragment holds each value in its own row and K slot, the B
// fragment gathers the matching activation columns from shared memory.
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace atlas {
namespace {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = 8;
constexpr int GV_PF = 8;            // ring depth: 1 KB slots in flight per warp
constexpr int GV_SLOT = 1024;       // bytes per slot: 16 rows x 64 columns of codes
constexpr int GV_SPIN_LIMIT = 1 << 20;

struct GemvParams {
    const void *x;
    int dtype;
    int m;          // rows of x handled by this launch (<= 8 * MT)
    int64_t ldx;
    const uint8_t *tiles;
    const uint16_t *scales_t;   // [row/128][block][row%128]
    const int32_t *chunk_ptr;   // [strip][k_tiles + 1]: first outlier entry with column >= 64 * c
    const uint32_t *entries;    // row%16 << 24 | column, strip-major, column-sorted
    const uint16_t *ovals;      // fp16 outlier values in the order of `entries`
    int n_rows;
    int n_cols;
    int bs;
    const uint16_t *bias;
    void *y;
    int64_t ldy;
    int k_tiles;        // n_cols / 64
    int n_chunks;       // ceil(n_cols / 256)
    int blocks_per_row; // n_cols / bs
    int kc_tiles;       // k-tiles staged per pass (x slice in shared memory); multiple of max(4, WK)
    int scale_rows;     // K blocks a CTA may need (capacity of the staged scales)
    int splits;         // cluster size S
    int x_vec_ok;       // x rows allow 16-byte loads
    int *status;        // device int, set non-zero if a bounded wait ran out (may be null)
    int bs_shift;       // log2(block size) when it is a power of two, else -1
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < GV_SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

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
    extern __shared__ __align__(128) unsigned char smem_raw[];

    // let the next kernel of the stream start its own weight prefetch as early as possible
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int strip_local = warp / WK, wk = warp % WK;
    const int split = blockIdx.x;  // == rank in the cluster along K
    const int n0 = blockIdx.y * R;

    // this CTA's K slice, in 256-column chunks (the granularity of the outlier table)
    const int c_begin = (int)((int64_t)p.n_chunks * split / p.splits);
    const int c_end = (int)((int64_t)p.n_chunks * (split + 1) / p.splits);
    const int kt_begin = c_begin * 4;
    const int kt_end = min(c_end * 4, p.k_tiles);

    // ---- shared memory carve-up ----------------------------------------------------------
    unsigned char *ring = smem_raw + (size_t)warp * GV_PF * GV_SLOT;             // this warp's slots
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar_u32 = smem_u32(smem_raw + (size_t)GV_WARPS * GV_PF * GV_SLOT) + (uint32_t)warp * GV_PF * 8;
    const int xs_stride = p.kc_tiles * 64 + 8;  // halves; +8 keeps 128-bit reads conflict-free
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem_raw + (size_t)GV_WARPS * GV_PF * (GV_SLOT + 8));
    uint16_t *s_scale = xs + (size_t)MTOT * xs_stride;                            // [block][R]
    float *ytile = reinterpret_cast<float *>(
        reinterpret_cast<unsigned char *>(s_scale) + (((size_t)p.scale_rows * R * 2 + 15) & ~(size_t)15));
    // ytile: [WK][MTOT][R]

    // ---- this warp's tile sequence and ring ------------------------------------------------
    const int row_strip = n0 + strip_local * 16;
    const int64_t rt = row_strip >> 7;
    const int strip_in_tile = (row_strip & 127) >> 4;
    const uint8_t *strip_base = p.tiles + ((rt * p.k_tiles) * 8 + strip_in_tile) * (int64_t)GV_SLOT;
    const int first_kt = kt_begin + wk;
    const int nj = first_kt < kt_end ? (kt_end - first_kt + WK - 1) / WK : 0;  // tiles of this warp
    if (lane == 0) {
        for (int sidx = 0; sidx < GV_PF; ++sidx) mbar_init(bar_u32 + 8 * sidx, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const int pre = nj < GV_PF ? nj : GV_PF;
        for (int j = 0; j < pre; ++j) {
            mbar_arrive_expect_tx(bar_u32 + 8 * j, GV_SLOT);
            bulk_load_1d(ring_u32 + j * GV_SLOT, strip_base + (int64_t)(first_kt + j * WK) * (8 * GV_SLOT), GV_SLOT,
                         bar_u32 + 8 * j);
        }
    }
    __syncwarp();

    // ---- scales of this CTA's rows and K slice (weights: may be read before the dependency wait) ---
    const int kb_begin = (kt_begin * 64) / p.bs;
    const int kb_end = min((kt_end * 64 + p.bs - 1) / p.bs, p.blocks_per_row);
    {
        const uint16_t *src = p.scales_t + ((int64_t)(n0 >> 7) * p.blocks_per_row) * 128 + (n0 & 127);
        const int nkb = kb_end - kb_begin;
        for (int e = tid; e < nkb * R; e += GV_THREADS) {
            const int kb = e / R, r = e - kb * R;
            s_scale[e] = __ldg(src + (int64_t)(kb_begin + kb) * 128 + r);
        }
    }
    // outlier ranges of this warp's strip, per pass, come from chunk_ptr (weights as well)
    const int32_t *cptr = p.chunk_ptr + (int64_t)(row_strip >> 4) * (p.k_tiles + 1);

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // everything below reads x (and later writes y): wait for the previous kernels of the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");

    bool alive = true;  // false once a bounded wait ran out: skip further waits
    int j = 0;          // index into this warp's tile sequence
    for (int pass_begin = kt_begin; pass_begin < kt_end; pass_begin += p.kc_tiles) {
        const int pass_end = min(pass_begin + p.kc_tiles, kt_end);
        const int pass_cols = (pass_end - pass_begin) * 64;
        const int col0 = pass_begin * 64;
        __syncthreads();  // previous pass no longer reads xs; also publishes s_scale
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

        // ---- dense part: this warp's k-tiles of the pass ------------------------------------
        for (int kt = pass_begin + wk; kt < pass_end; kt += WK, ++j) {
            const int slot = j % GV_PF;
            if (alive && !mbar_wait(bar_u32 + 8 * slot, (uint32_t)(j / GV_PF) & 1u)) {
                alive = false;
                if (lane == 0 && p.status) atomicExch(p.status, 1);
            }
            const uint4 wa = *reinterpret_cast<const uint4 *>(ring + slot * GV_SLOT + lane * 16);        // row g
            const uint4 wb = *reinterpret_cast<const uint4 *>(ring + slot * GV_SLOT + 512 + lane * 16);  // row g+8
            const int kb = (kt * 64 + tig * 16) / p.bs - kb_begin;
            const __half2 sa2 = __half2half2(__ushort_as_half(s_scale[kb * R + strip_local * 16 + g]));
            const __half2 sb2 = __half2half2(__ushort_as_half(s_scale[kb * R + strip_local * 16 + g + 8]));
            const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w};
            const uint32_t wbv[4] = {wb.x, wb.y, wb.z, wb.w};
            uint32_t a_lo[4], a_hi[4], b_lo[4], b_hi[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                dequant4(wav[i], sa2, a_lo[i], a_hi[i]);
                dequant4(wbv[i], sb2, b_lo[i], b_hi[i]);
            }
            // the slot has been consumed by every lane: refill it with the tile GV_PF steps ahead
            __syncwarp();
            if (lane == 0 && j + GV_PF < nj) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive_expect_tx(bar_u32 + 8 * slot, GV_SLOT);
                bulk_load_1d(ring_u32 + slot * GV_SLOT, strip_base + (int64_t)(kt + GV_PF * WK) * (8 * GV_SLOT),
                             GV_SLOT, bar_u32 + 8 * slot);
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

        // ---- sparse part: outliers of this warp's strip inside the pass, 16 per MMA ----------
        {
            const int e_begin = __ldg(cptr + pass_begin);
            const int e_end = __ldg(cptr + pass_end);
            for (int e0 = e_begin + wk * 16; e0 < e_end; e0 += WK * 16) {
                uint32_t av[4];   // A fragment: values of slots (2tig,2tig+1) and (2tig+8,2tig+9) for rows g, g+8
                int cols[4];
                uint16_t vals[4];
                int rws[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int slot_k = 2 * tig + (q & 1) + (q >> 1) * 8;
                    const int e = e0 + slot_k;
                    uint32_t ent = 0xff000000u | (uint32_t)col0;  // no row matches 255; column stays in range
                    uint16_t v = 0;
                    if (e < e_end) { ent = __ldg(p.entries + e); v = __ldg(p.ovals + e); }
                    cols[q] = (int)(ent & 0xffffffu) - col0;
                    rws[q] = (int)(ent >> 24);
                    vals[q] = v;
                }
                av[0] = (rws[0] == g ? vals[0] : 0u) | (uint32_t)(rws[1] == g ? vals[1] : 0u) << 16;
                av[1] = (rws[0] == g + 8 ? vals[0] : 0u) | (uint32_t)(rws[1] == g + 8 ? vals[1] : 0u) << 16;
                av[2] = (rws[2] == g ? vals[2] : 0u) | (uint32_t)(rws[3] == g ? vals[3] : 0u) << 16;
                av[3] = (rws[2] == g + 8 ? vals[2] : 0u) | (uint32_t)(rws[3] == g + 8 ? vals[3] : 0u) << 16;
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    const uint16_t *xr = xs + (nt * 8 + g) * xs_stride;
                    const uint32_t b0 = xr[cols[0]] | (uint32_t)xr[cols[1]] << 16;
                    const uint32_t b1 = xr[cols[2]] | (uint32_t)xr[cols[3]] << 16;
                    mma_f16(acc[nt], av[0], av[1], av[2], av[3], b0, b1);
                }
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
    if (WK > 1) {  // fold the slabs of this CTA in a fixed order into slab 0
        for (int e = tid; e < MTOT * R; e += GV_THREADS) {
            float s = ytile[e];
#pragma unroll
            for (int k = 1; k < WK; ++k) s += ytile[(size_t)k * MTOT * R + e];
            ytile[e] = s;
        }
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

// ---------------------------------------------------------------------------------------------
// m <= 8: one 16-row strip per CTA, its warps split K in 256-column chunks.
//
// The general kernel above spends most of its time in per-CTA set-up and reduction chains when
// the whole launch lasts a few microseconds.  This variant keeps the per-warp instruction chain
// short: no activation staging, no cluster, one __syncthreads.  A warp loads its codes (16-byte
// loads, 1 KB per warp and step, contiguous) and scales before the dependency wait, its
// activations after it (straight from global memory: x is a few KB and stays in L1/L2), and the
// CTA folds the per-warp partial sums through 8 KB of shared memory.  Codes, scales, the first
// outlier entries and the bias are requested before griddepcontrol.wait.
constexpr int GS_MAX_WARPS = 16;
constexpr int GS_UNROLL = 2;

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <bool BF16>
__device__ __forceinline__ void load_x16(const uint16_t *src, bool valid, uint32_t (&xv)[8]) {
    uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
    if (valid) {
        a = __ldg(reinterpret_cast<const uint4 *>(src));
        b = __ldg(reinterpret_cast<const uint4 *>(src) + 1);
    }
    xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
    xv[4] = b.x; xv[5] = b.y; xv[6] = b.z; xv[7] = b.w;
    if (BF16) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float lo = __uint_as_float(xv[i] << 16), hi = __uint_as_float(xv[i] & 0xffff0000u);
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(xv[i]) : "f"(hi), "f"(lo));
        }
    }
}

template <bool BF16>
__global__ void __launch_bounds__(GS_MAX_WARPS * 32, 2) gemv_strip_kernel(GemvParams p) {
    __shared__ float4 part[GS_MAX_WARPS][32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int strip = blockIdx.x;
    const int c0 = (p.n_chunks * warp) / nwarps, c1 = (p.n_chunks * (warp + 1)) / nwarps;
    const int kt0 = c0 * 4, kt1 = min(c1 * 4, p.k_tiles);

    const uint8_t *wbase = p.tiles + ((size_t)(strip >> 3) * p.k_tiles * 8 + (strip & 7)) * 1024 + lane * 16;
    const uint16_t *sbase = p.scales_t + (size_t)(strip >> 3) * p.blocks_per_row * 128 + (strip & 7) * 16 + g;
    // lanes whose batch row does not exist read row 0: their MMA columns are never stored
    const uint16_t *xg = reinterpret_cast<const uint16_t *>(p.x) + (size_t)(g < p.m ? g : 0) * p.ldx;
    const uint16_t *xrow = xg + tig * 16;

    // ---- weights first: none of this depends on earlier kernels of the stream ----------------------
    uint4 wa[GS_UNROLL], wb[GS_UNROLL];
    uint16_t sa[GS_UNROLL], sb[GS_UNROLL];
    auto load_batch = [&](int kt) {
#pragma unroll
        for (int u = 0; u < GS_UNROLL; ++u) {
            if (kt + u < kt1) {
                const uint8_t *tp = wbase + (size_t)(kt + u) * 8192;
                wa[u] = ldg_stream(tp);
                wb[u] = ldg_stream(tp + 512);
                const int kb = p.bs_shift >= 0 ? ((kt + u) * 64 + tig * 16) >> p.bs_shift : ((kt + u) * 64 + tig * 16) / p.bs;
                sa[u] = __ldg(sbase + (size_t)kb * 128);
                sb[u] = __ldg(sbase + (size_t)kb * 128 + 8);
            }
        }
    };
    load_batch(kt0);
    // first group of outlier entries of the strip inside this warp's columns, and the bias
    const int32_t *cptr = p.chunk_ptr + (size_t)strip * (p.k_tiles + 1);
    int e_begin = 0, e_end = 0;
    if (kt0 < kt1) { e_begin = __ldg(cptr + kt0); e_end = __ldg(cptr + kt1); }
    uint32_t pre_ent[4], pre_val[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int e = e_begin + 2 * tig + (q & 1) + (q >> 1) * 8;
        pre_ent[q] = 0xff000000u;
        pre_val[q] = 0;
        if (e < e_end) { pre_ent[q] = __ldg(p.entries + e); pre_val[q] = __ldg(p.ovals + e); }
    }
    const int rL = tid >> 2, rj = tid & 3;              // (lane, component) this thread reduces at the end
    const int out_row = (rL >> 2) + (rj >> 1) * 8, out_m = (rL & 3) * 2 + (rj & 1);
    const int out_n = strip * 16 + out_row;
    float bias_v = 0.f;
    if (tid < 128 && p.bias && out_n < p.n_rows) bias_v = __half2float(__ushort_as_half(__ldg(p.bias + out_n)));

    // ---- activations: only after the earlier kernels of the stream have completed ------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    auto outlier_mma = [&](const uint32_t (&ent)[4], const uint32_t (&val)[4]) {
        int rws[4];
        uint32_t xq[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            rws[q] = (int)(ent[q] >> 24);
            xq[q] = __ldg(xg + (ent[q] & 0xffffffu));
        }
        const uint32_t a0 = (rws[0] == g ? val[0] : 0u) | (rws[1] == g ? val[1] : 0u) << 16;
        const uint32_t a1 = (rws[0] == g + 8 ? val[0] : 0u) | (rws[1] == g + 8 ? val[1] : 0u) << 16;
        const uint32_t a2 = (rws[2] == g ? val[2] : 0u) | (rws[3] == g ? val[3] : 0u) << 16;
        const uint32_t a3 = (rws[2] == g + 8 ? val[2] : 0u) | (rws[3] == g + 8 ? val[3] : 0u) << 16;
        uint32_t b0 = xq[0] | xq[1] << 16, b1 = xq[2] | xq[3] << 16;
        if (BF16) {
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(b0) : "f"(__uint_as_float(xq[1] << 16)), "f"(__uint_as_float(xq[0] << 16)));
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(b1) : "f"(__uint_as_float(xq[3] << 16)), "f"(__uint_as_float(xq[2] << 16)));
        }
        mma_f16(acc, a0, a1, a2, a3, b0, b1);
    };
    if (e_begin < e_end) outlier_mma(pre_ent, pre_val);   // its activation gathers overlap the K loop's loads

    for (int kt = kt0; kt < kt1; kt += GS_UNROLL) {
        if (kt != kt0) load_batch(kt);
        uint32_t xv[GS_UNROLL][8];
#pragma unroll
        for (int u = 0; u < GS_UNROLL; ++u)
            if (kt + u < kt1) load_x16<BF16>(xrow + (kt + u) * 64, true, xv[u]);
#pragma unroll
        for (int u = 0; u < GS_UNROLL; ++u) {
            if (kt + u < kt1) {
                const __half2 sa2 = __half2half2(__ushort_as_half(sa[u])), sb2 = __half2half2(__ushort_as_half(sb[u]));
                const uint32_t wav[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w};
                const uint32_t wbv[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t alo, ahi, blo, bhi;
                    dequant4(wav[i], sa2, alo, ahi);
                    dequant4(wbv[i], sb2, blo, bhi);
                    mma_f16(acc, alo, blo, ahi, bhi, xv[u][2 * i], xv[u][2 * i + 1]);
                }
            }
        }
    }
    for (int e0 = e_begin + 16; e0 < e_end; e0 += 16) {    // remaining outlier groups, 16 per MMA
        uint32_t ent[4], val[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = e0 + 2 * tig + (q & 1) + (q >> 1) * 8;
            ent[q] = 0xff000000u;
            val[q] = 0;
            if (e < e_end) { ent[q] = __ldg(p.entries + e); val[q] = __ldg(p.ovals + e); }
        }
        outlier_mma(ent, val);
    }

    part[warp][lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    if (tid < 128) {
        float s = bias_v;
        for (int w = 0; w < nwarps; ++w) s += reinterpret_cast<const float *>(&part[w][rL])[rj];
        if (out_m < p.m && out_n < p.n_rows) {
            if (BF16) reinterpret_cast<__nv_bfloat16 *>(p.y)[(size_t)out_m * p.ldy + out_n] = __float2bfloat16_rn(s);
            else reinterpret_cast<__half *>(p.y)[(size_t)out_m * p.ldy + out_n] = __float2half_rn(s);
        }
    }
}

int launch_gemv_strip(const GemvParams &p, cudaStream_t st) {
    int nwarps = p.n_chunks < GS_MAX_WARPS ? p.n_chunks : GS_MAX_WARPS;
    if (nwarps < 4) nwarps = 4;  // the reduction needs 128 threads
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((p.n_rows + 15) / 16), 1, 1);
    cfg.blockDim = dim3((unsigned)(nwarps * 32), 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (p.dtype == ATLAS_DTYPE_BF16)
        return check_cuda(cudaLaunchKernelEx(&cfg, gemv_strip_kernel<true>, p), "gemv_strip_kernel launch");
    return check_cuda(cudaLaunchKernelEx(&cfg, gemv_strip_kernel<false>, p), "gemv_strip_kernel launch");
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
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
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
                                  const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                  const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                  int64_t n_rows, int64_t n_cols, int block_size, const void *bias, void *y,
                                  int64_t ldy, int32_t *status, void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(!x || !tiles || !scales_tiled || !outlier_chunk_ptr || !y, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemv: null buffer");
    ATLAS_RETURN_IF(m < 0 || n_rows <= 0 || n_cols <= 0 || ldx < n_cols || ldy < n_rows, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemv: bad size (m=%lld n_rows=%lld n_cols=%lld ldx=%lld ldy=%lld)",
                    (long long)m, (long long)n_rows, (long long)n_cols, (long long)ldx, (long long)ldy);
    ATLAS_RETURN_IF(dtype != ATLAS_DTYPE_F16 && dtype != ATLAS_DTYPE_BF16, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemv: dtype %d", dtype);
    ATLAS_RETURN_IF(n_cols % 64 != 0 || block_size < 16 || block_size % 16 != 0 || n_cols % block_size != 0,
                    ATLAS_ERR_UNSUPPORTED,
                    "atlas_qlinear_gemv: needs n_cols %% 64 == 0 and block_size a multiple of 16 dividing n_cols");
    ATLAS_RETURN_IF(n_rows > 0x7fffff00 || n_cols >= (1 << 24), ATLAS_ERR_UNSUPPORTED, "atlas_qlinear_gemv: too large");
    ATLAS_RETURN_IF(((uintptr_t)tiles & 15) != 0, ATLAS_ERR_BAD_ARGUMENT, "atlas_qlinear_gemv: tiles not 16-byte aligned");
    int rc = check_device();
    if (rc) return rc;
    if (m == 0) return ATLAS_OK;
    cudaStream_t st = (cudaStream_t)stream;

    const int k_tiles = (int)(n_cols / 64);
    const int n_chunks = (int)ceil_div_i64(n_cols, 256);
    const int target = sm_count() * 3 / 2;
    for (int64_t m0 = 0; m0 < m; m0 += 32) {
        const int mg = (int)((m - m0) < 32 ? (m - m0) : 32);
        const int mt = mg <= 8 ? 1 : (mg <= 16 ? 2 : 4);
        // rows per CTA: the largest of 128/64/32/16 that still yields enough CTAs with up to 8 K slices
        int wk = 8;
        for (int cand = 1; cand <= 8; cand *= 2) {
            const int R = 16 * (GV_WARPS / cand);
            const int64_t groups = ceil_div_i64(n_rows, R);
            const int smax = n_chunks >= 8 ? 8 : n_chunks;
            if (groups * smax >= target || cand == 8) { wk = cand; break; }
        }
        const int R = 16 * (GV_WARPS / wk);
        const int row_groups = (int)ceil_div_i64(n_rows, R);
        int smax = 1;
        while (smax * 2 <= 8 && smax * 2 <= n_chunks) smax *= 2;
        int splits = 1;
        while (splits < smax && (int64_t)row_groups * splits < target) splits *= 2;
        const int tiles_per_cta = (int)ceil_div_i64(n_chunks, splits) * 4;
        const int unit = wk > 4 ? wk : 4;            // passes hold whole chunks and whole warp rounds
        int kc_cap = 256 / (mt * 8);                 // x slice <= 32 KB: 32 k-tiles at m<=8, 16, 8 at m<=32
        kc_cap = (kc_cap / unit) * unit;
        if (kc_cap < unit) kc_cap = unit;
        int kc_tiles = ((tiles_per_cta + unit - 1) / unit) * unit;
        if (kc_tiles > kc_cap) kc_tiles = kc_cap;
        const int scale_rows = (tiles_per_cta * 64 + block_size - 1) / block_size + 2;

        GemvParams p;
        p.x = (const char *)x + (size_t)m0 * ldx * 2;
        p.dtype = dtype;
        p.m = mg;
        p.ldx = ldx;
        p.tiles = tiles;
        p.scales_t = (const uint16_t *)scales_tiled;
        p.chunk_ptr = outlier_chunk_ptr;
        p.entries = outlier_entries;
        p.ovals = (const uint16_t *)outlier_vals_sorted;
        p.n_rows = (int)n_rows;
        p.n_cols = (int)n_cols;
        p.bs = block_size;
        p.bias = (const uint16_t *)bias;
        p.y = (char *)y + (size_t)m0 * ldy * 2;
        p.ldy = ldy;
        p.k_tiles = k_tiles;
        p.n_chunks = n_chunks;
        p.blocks_per_row = (int)(n_cols / block_size);
        p.kc_tiles = kc_tiles;
        p.scale_rows = scale_rows;
        p.splits = splits;
        p.x_vec_ok = (((uintptr_t)x & 15) == 0) && (ldx % 8 == 0);
        p.status = status;
        p.bs_shift = (block_size & (block_size - 1)) == 0 ? __builtin_ctz((unsigned)block_size) : -1;

        if (mt <= 2 && p.x_vec_ok) {
            // up to 16 rows: one strip-kernel launch per 8 rows (the second pass over a weight finds most of it in L2)
            for (int r0 = 0; r0 < mg; r0 += 8) {
                GemvParams ps = p;
                ps.m = mg - r0 < 8 ? mg - r0 : 8;
                ps.x = (const char *)p.x + (size_t)r0 * ldx * 2;
                ps.y = (char *)p.y + (size_t)r0 * ldy * 2;
                rc = launch_gemv_strip(ps, st);
                if (rc) return rc;
            }
            continue;
        }
        const int mtot = mt * 8;
        const size_t ring_bytes = (size_t)GV_WARPS * GV_PF * (GV_SLOT + 8);
        const size_t xs_bytes = (size_t)mtot * (kc_tiles * 64 + 8) * 2;
        const size_t sc_bytes = ((size_t)scale_rows * R * 2 + 15) & ~(size_t)15;
        const size_t y_bytes = (size_t)wk * mtot * R * 4;
        const size_t smem = ring_bytes + xs_bytes + sc_bytes + y_bytes;
        if (mt == 1) rc = dispatch_wk<1>(wk, p, row_groups, smem, st);
        else if (mt == 2) rc = dispatch_wk<2>(wk, p, row_groups, smem, st);
        else rc = dispatch_wk<4>(wk, p, row_groups, smem, st);
        if (rc) return rc;
    }
    return ATLAS_OK;
}
