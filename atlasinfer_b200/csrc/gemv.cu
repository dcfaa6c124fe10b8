// Decode-time quantized linear: y[m][n] = sum_k x[m][k] * W[n][k] + bias[n], a few rows of x at a time.
//
// Replaces the steady state of QuantizedLinear.forward (integration/atlas_wrappers.py:56,67), which multiplies by
// a cached fp16 copy of the weight (2 bytes per weight).  Here the kernel streams the tile-major uint8 codes
// (1 byte per weight), rebuilds in registers exactly the fp16 weight the reference's dequantizer produces
// (adaptive_quantizer.py:216: fp16(fp16(code) * scale)), feeds it to the tensor cores as the 16-row operand with
// the activations as the 8-column operand, and adds the fp16 outlier products in the same launch.  The kernel is
// HBM-bound; the MMA is only the cheapest way to do the multiply-adds without unpacking to fp32.
//
// Work split: one CTA per 16-row strip of the weight, its (up to 16) warps split K in 256-column chunks.  The
// per-warp instruction chain is short, because a launch lasts only microseconds: no activation staging, no
// cluster, one __syncthreads.  A warp loads its codes (16-byte loads, 1 KB per warp and step, contiguous in the
// tile-major layout), scales, first outlier entries and the bias before the dependency wait of programmatic
// dependent launch, i.e. while the previous kernel of the stream drains; its activations come after the wait,
// straight from global memory (x is a few KB and stays in L1/L2) -- or, for one or two bf16 rows, through a
// per-warp fp16 copy in shared memory.  The CTA folds the per-warp partial sums
// through 8 KB of shared memory in warp order (deterministic, no atomics).
//
// Outliers: the side-table is regrouped by 16-row strip and sorted by column (atlas_repack).  A warp turns 16
// outliers of its strip at a time into one more MMA: the A fragment holds each value in its own row and K slot,
// the B fragment gathers the matching activations.
//
// Up to 8 rows of x take one 8-column MMA tile (two CTAs of 16 warps per SM); 9..16 rows take two tiles per step in
// one pass over the weight (two CTAs of 8 warps per SM at twice the registers).  More rows are served 16 at a time: the later passes
// find most of the weight in L2.
#include <cuda_bf16.h>

#include "common.cuh"

namespace atlas {
namespace {

struct GemvParams {
    const void *x;
    int dtype;
    int m;          // rows of x handled by this launch (<= 16)
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
    int bs_shift;       // log2(block size) when it is a power of two, else -1
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

constexpr int GS_MAX_WARPS = 16;
constexpr int GS_UNROLL = 2;
constexpr int GS_WARPS2 = 8;   // warps of the two-tile kernel: two CTAs per SM at 128 registers (1.95 -> 2.38 TB/s at 16 rows against 16 warps in one CTA)

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// 16 consecutive activations of one batch row.  VEC: the row allows 16-byte loads.
template <bool BF16, bool VEC>
__device__ __forceinline__ void load_x16(const uint16_t *src, uint32_t (&xv)[8]) {
    if (VEC) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(src));
        const uint4 b = __ldg(reinterpret_cast<const uint4 *>(src) + 1);
        xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
        xv[4] = b.x; xv[5] = b.y; xv[6] = b.z; xv[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = __ldg(src + 2 * i) | (uint32_t)__ldg(src + 2 * i + 1) << 16;
    }
    if (BF16) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float lo = __uint_as_float(xv[i] << 16), hi = __uint_as_float(xv[i] & 0xffff0000u);
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(xv[i]) : "f"(hi), "f"(lo));
        }
    }
}

// MT: 8-column MMA tiles over the batch (m <= 8 * MT).  One tile: two CTAs of 16 warps per SM at 64 registers, two
// k-tiles of codes in flight per warp.  Two tiles: two CTAs of 8 warps per SM at twice the registers, four k-tiles in
// flight per warp (the same bytes in flight per SM), the dequantised fragments of a step feeding two MMAs.
//
// STAGE (bf16 activations): every warp converts the columns of its K range to fp16 once, into shared memory (it reads
// no other columns, so no CTA-wide barrier is needed), instead of converting the fragments of every step in registers
// for each of its eight row groups -- the kernel is bound by instruction issue, not by bytes in flight.
//
// FAST (whole 256-column chunks, blocks of whole 64-column tiles): every batch of a warp is full and a step has one
// scale block, so the K loop carries no bounds predicates and no per-lane block index.
template <bool BF16, bool VEC, int MT, bool STAGE, bool FAST>
__global__ void __launch_bounds__((MT == 1 ? GS_MAX_WARPS : GS_WARPS2) * 32, 2) gemv_strip_kernel(GemvParams p) {
    constexpr int U = MT == 1 ? GS_UNROLL : 2 * GS_UNROLL;
    __shared__ float4 part[MT][MT == 1 ? GS_MAX_WARPS : GS_WARPS2][32];
    extern __shared__ __align__(16) unsigned char xs_raw[];   // STAGE: [m][n_cols fp16 + 16 bytes of padding]
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int strip = blockIdx.x;
    // (a CTA has 16 warps unless K is short: the split of the chunks over them then needs no division)
    const int c0 = nwarps == 16 ? (p.n_chunks * warp) >> 4 : (nwarps == 8 ? (p.n_chunks * warp) >> 3 : (p.n_chunks * warp) / nwarps);
    const int c1 = nwarps == 16 ? (p.n_chunks * (warp + 1)) >> 4 : (nwarps == 8 ? (p.n_chunks * (warp + 1)) >> 3 : (p.n_chunks * (warp + 1)) / nwarps);
    const int kt0 = c0 * 4, kt1 = min(c1 * 4, p.k_tiles);

    const uint8_t *wbase = p.tiles + ((size_t)(strip >> 3) * p.k_tiles * 8 + (strip & 7)) * 1024 + lane * 16;
    const uint16_t *sbase = p.scales_t + (size_t)(strip >> 3) * p.blocks_per_row * 128 + (strip & 7) * 16 + g;
    // lanes whose batch row does not exist read row 0: their MMA columns are never stored
    const uint16_t *xg[MT], *xrow[MT];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        xg[nt] = reinterpret_cast<const uint16_t *>(p.x) + (size_t)(nt * 8 + g < p.m ? nt * 8 + g : 0) * p.ldx;
        xrow[nt] = xg[nt] + tig * 16;
    }

    // ---- weights first: none of this depends on earlier kernels of the stream ----------------------
    uint4 wa[U], wb[U];
    uint16_t sa[U], sb[U];
    auto load_batch = [&](int kt) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (FAST || kt + u < kt1) {
                const uint8_t *tp = wbase + (FAST ? (size_t)((uint32_t)(kt + u) << 13) : (size_t)(kt + u) * 8192);
                wa[u] = ldg_stream(tp);
                wb[u] = ldg_stream(tp + 512);
                const int kb = FAST ? (kt + u) >> (p.bs_shift - 6)
                                    : (p.bs_shift >= 0 ? ((kt + u) * 64 + tig * 16) >> p.bs_shift : ((kt + u) * 64 + tig * 16) / p.bs);
                sa[u] = __ldg(sbase + (FAST ? (size_t)((uint32_t)kb << 7) : (size_t)kb * 128));
                sb[u] = __ldg(sbase + (FAST ? (size_t)((uint32_t)kb << 7) : (size_t)kb * 128) + 8);
            }
        }
    };
    load_batch(kt0);
    // first group of outlier entries of the strip inside this warp's columns, and the bias
    const int32_t *cptr = p.chunk_ptr + (size_t)strip * (p.k_tiles + 1);
    int e_begin = 0, e_end = 0;
    if (kt0 < kt1) { e_begin = __ldg(cptr + kt0); e_end = __ldg(cptr + kt1); }
    // an empty slot of an outlier group: row 255 matches no lane; its column is one of this warp's own (with the staged
    // row a warp reads only what it has written itself)
    const uint32_t no_entry = 0xff000000u | (uint32_t)(kt0 * 64);
    uint32_t pre_ent[4], pre_val[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int e = e_begin + 2 * tig + (q & 1) + (q >> 1) * 8;
        pre_ent[q] = no_entry;
        pre_val[q] = 0;
        if (e < e_end) { pre_ent[q] = __ldg(p.entries + e); pre_val[q] = __ldg(p.ovals + e); }
    }
    // (MMA tile, lane, component) this thread reduces at the end: 128 outputs per tile
    const int rT = tid >> 7, rL = (tid >> 2) & 31, rj = tid & 3;
    const int out_row = (rL >> 2) + (rj >> 1) * 8, out_m = rT * 8 + (rL & 3) * 2 + (rj & 1);
    const int out_n = strip * 16 + out_row;
    float bias_v = 0.f;
    if (tid < 128 * MT && p.bias && out_n < p.n_rows) bias_v = __half2float(__ushort_as_half(__ldg(p.bias + out_n)));

    // ---- activations: only after the earlier kernels of the stream have completed ------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int xs_row_bytes = p.n_cols * 2 + 16;
    if (STAGE) {
        // every warp converts the columns of its own K range, the only ones it reads: no CTA-wide barrier
        const int per_row = (kt1 - kt0) * 8;   // 16-byte pieces per batch row
        for (int row = 0; row < p.m; ++row) {
            const uint16_t *src = reinterpret_cast<const uint16_t *>(p.x) + (size_t)row * p.ldx + kt0 * 64;
            unsigned char *dst = xs_raw + (size_t)row * xs_row_bytes + kt0 * 128;
            for (int c = lane; c < per_row; c += 32) {
                uint4 v = __ldg(reinterpret_cast<const uint4 *>(src) + c);
                uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float lo = __uint_as_float(w4[e] << 16), hi = __uint_as_float(w4[e] & 0xffff0000u);
                    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(w4[e]) : "f"(hi), "f"(lo));
                }
                *reinterpret_cast<uint4 *>(dst + c * 16) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
        }
        __syncwarp();
    }
    // this lane's row of staged activations (rows that do not exist read row 0, as above)
    const unsigned char *xs_lane = xs_raw + (size_t)(g < p.m ? g : 0) * xs_row_bytes;

    float acc[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
    auto outlier_mma = [&](const uint32_t (&ent)[4], const uint32_t (&val)[4]) {
        int rws[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) rws[q] = (int)(ent[q] >> 24);
        const uint32_t a0 = (rws[0] == g ? val[0] : 0u) | (rws[1] == g ? val[1] : 0u) << 16;
        const uint32_t a1 = (rws[0] == g + 8 ? val[0] : 0u) | (rws[1] == g + 8 ? val[1] : 0u) << 16;
        const uint32_t a2 = (rws[2] == g ? val[2] : 0u) | (rws[3] == g ? val[3] : 0u) << 16;
        const uint32_t a3 = (rws[2] == g + 8 ? val[2] : 0u) | (rws[3] == g + 8 ? val[3] : 0u) << 16;
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            uint32_t xq[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
                xq[q] = STAGE ? *reinterpret_cast<const uint16_t *>(xs_lane + (size_t)(ent[q] & 0xffffffu) * 2)
                              : __ldg(xg[nt] + (ent[q] & 0xffffffu));
            uint32_t b0 = xq[0] | xq[1] << 16, b1 = xq[2] | xq[3] << 16;
            if (BF16 && !STAGE) {
                asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(b0) : "f"(__uint_as_float(xq[1] << 16)), "f"(__uint_as_float(xq[0] << 16)));
                asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(b1) : "f"(__uint_as_float(xq[3] << 16)), "f"(__uint_as_float(xq[2] << 16)));
            }
            mma_f16(acc[nt], a0, a1, a2, a3, b0, b1);
        }
    };
    if (e_begin < e_end) outlier_mma(pre_ent, pre_val);   // its activation gathers overlap the K loop's loads

    for (int kt = kt0; kt < kt1; kt += U) {
        if (kt != kt0) load_batch(kt);
        if (MT == 1) {
            // all activations of the batch first, then the arithmetic
            uint32_t xv[U][8];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (FAST || kt + u < kt1) {
                    if (STAGE) {
                        const uint4 a = *reinterpret_cast<const uint4 *>(xs_lane + ((kt + u) * 64 + tig * 16) * 2);
                        const uint4 b = *reinterpret_cast<const uint4 *>(xs_lane + ((kt + u) * 64 + tig * 16) * 2 + 16);
                        xv[u][0] = a.x; xv[u][1] = a.y; xv[u][2] = a.z; xv[u][3] = a.w;
                        xv[u][4] = b.x; xv[u][5] = b.y; xv[u][6] = b.z; xv[u][7] = b.w;
                    } else {
                        load_x16<BF16, VEC>(xrow[0] + (kt + u) * 64, xv[u]);
                    }
                }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (FAST || kt + u < kt1) {
                    const uint32_t wav[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w};
                    const uint32_t wbv[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
                    const __half2 sa2 = __half2half2(__ushort_as_half(sa[u])), sb2 = __half2half2(__ushort_as_half(sb[u]));
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t alo, ahi, blo, bhi;
                        dequant4(wav[i], sa2, alo, ahi);
                        dequant4(wbv[i], sb2, blo, bhi);
                        mma_f16(acc[0], alo, blo, ahi, bhi, xv[u][2 * i], xv[u][2 * i + 1]);
                    }
                }
            }
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (FAST || kt + u < kt1) {
                    uint32_t xv[MT][8];
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt) load_x16<BF16, VEC>(xrow[nt] + (kt + u) * 64, xv[nt]);
                    const __half2 sa2 = __half2half2(__ushort_as_half(sa[u])), sb2 = __half2half2(__ushort_as_half(sb[u]));
                    const uint32_t wav[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w};
                    const uint32_t wbv[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t alo, ahi, blo, bhi;
                        dequant4(wav[i], sa2, alo, ahi);
                        dequant4(wbv[i], sb2, blo, bhi);
#pragma unroll
                        for (int nt = 0; nt < MT; ++nt) mma_f16(acc[nt], alo, blo, ahi, bhi, xv[nt][2 * i], xv[nt][2 * i + 1]);
                    }
                }
            }
        }
    }
    for (int e0 = e_begin + 16; e0 < e_end; e0 += 16) {    // remaining outlier groups, 16 per MMA
        uint32_t ent[4], val[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = e0 + 2 * tig + (q & 1) + (q >> 1) * 8;
            ent[q] = no_entry;
            val[q] = 0;
            if (e < e_end) { ent[q] = __ldg(p.entries + e); val[q] = __ldg(p.ovals + e); }
        }
        outlier_mma(ent, val);
    }

#pragma unroll
    for (int nt = 0; nt < MT; ++nt) part[nt][warp][lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
    __syncthreads();
    if (tid < 128 * MT) {
        float s = bias_v;
        for (int w = 0; w < nwarps; ++w) s += reinterpret_cast<const float *>(&part[rT][w][rL])[rj];
        if (out_m < p.m && out_n < p.n_rows) {
            if (BF16) reinterpret_cast<__nv_bfloat16 *>(p.y)[(size_t)out_m * p.ldy + out_n] = __float2bfloat16_rn(s);
            else reinterpret_cast<__half *>(p.y)[(size_t)out_m * p.ldy + out_n] = __float2half_rn(s);
        }
    }
}

constexpr int GS_STAGE_MAX_BYTES = 48 * 1024;   // staged fp16 activations per CTA, at most (two CTAs per SM)

template <int MT>
int launch_gemv_strip(const GemvParams &p, bool vec, cudaStream_t st) {
    const int max_warps = MT == 1 ? GS_MAX_WARPS : GS_WARPS2;
    int nwarps = p.n_chunks < max_warps ? p.n_chunks : max_warps;
    if (nwarps < 4 * MT) nwarps = 4 * MT;  // the reduction needs 128 threads per MMA tile
    // one or two rows of bf16 activations are converted once per CTA into shared memory (measured at 1 / 2 / 4 / 8
    // rows: 3.7 / 3.5 / 3.1 / 2.6 TB/s staged against 3.4 / 3.3 / 3.3 / 3.1 converted per step)
    const size_t stage_bytes = (size_t)p.m * ((size_t)p.n_cols * 2 + 16);
    const bool fast = vec && (p.k_tiles & 3) == 0 && p.bs_shift >= 6;   // whole chunks, blocks of whole tiles
    const bool stage = MT == 1 && p.dtype == ATLAS_DTYPE_BF16 && vec && p.m <= 2 && stage_bytes <= (size_t)GS_STAGE_MAX_BYTES;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((p.n_rows + 15) / 16), 1, 1);
    cfg.blockDim = dim3((unsigned)(nwarps * 32), 1, 1);
    cfg.dynamicSmemBytes = stage ? stage_bytes : 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (stage) {
        auto kern = fast ? gemv_strip_kernel<true, true, 1, true, true> : gemv_strip_kernel<true, true, 1, true, false>;
        static thread_local int configured_dev[2] = {-1, -1};   // more than the default dynamic shared memory: opt in once
        int dev = 0;
        cudaGetDevice(&dev);
        if (configured_dev[fast] != dev) {
            int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GS_STAGE_MAX_BYTES),
                                "cudaFuncSetAttribute(gemv smem)");
            if (rc) return rc;
            configured_dev[fast] = dev;
        }
        return check_cuda(cudaLaunchKernelEx(&cfg, kern, p), "gemv_strip_kernel launch");
    }
    if (fast) {
        auto kern = p.dtype == ATLAS_DTYPE_BF16 ? gemv_strip_kernel<true, true, MT, false, true> : gemv_strip_kernel<false, true, MT, false, true>;
        return check_cuda(cudaLaunchKernelEx(&cfg, kern, p), "gemv_strip_kernel launch");
    }
    auto kern = p.dtype == ATLAS_DTYPE_BF16 ? (vec ? gemv_strip_kernel<true, true, MT, false, false> : gemv_strip_kernel<true, false, MT, false, false>)
                                            : (vec ? gemv_strip_kernel<false, true, MT, false, false> : gemv_strip_kernel<false, false, MT, false, false>);
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p), "gemv_strip_kernel launch");
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

    GemvParams p;
    p.dtype = dtype;
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
    p.ldy = ldy;
    p.k_tiles = (int)(n_cols / 64);
    p.n_chunks = (int)ceil_div_i64(n_cols, 256);
    p.blocks_per_row = (int)(n_cols / block_size);
    p.bs_shift = (block_size & (block_size - 1)) == 0 ? __builtin_ctz((unsigned)block_size) : -1;
    const bool vec = (((uintptr_t)x & 15) == 0) && (ldx % 8 == 0);   // x rows allow 16-byte loads
    (void)status;   // no bounded wait in this kernel: nothing to report
    for (int64_t m0 = 0; m0 < m; m0 += 16) {   // one launch per 16 rows: the later passes find most of the weight in L2
        p.m = (int)(m - m0 < 16 ? m - m0 : 16);
        p.x = (const char *)x + (size_t)m0 * ldx * 2;
        p.y = (char *)y + (size_t)m0 * ldy * 2;
        rc = p.m <= 8 ? launch_gemv_strip<1>(p, vec, st) : launch_gemv_strip<2>(p, vec, st);
        if (rc) return rc;
    }
    return ATLAS_OK;
}
