// Adaptive hybrid quantizer for sm_100a: one pass over the fp16 weights.
//
// Replaces quantize_tensor (atlasinfer_core/quant/adaptive_quantizer.py:51-148).
// The reference walks the blocks in a Python loop and concatenates four
// streams; here a persistent grid takes tiles of 8192 elements in order
// (dynamic tile ids), evaluates every block of a tile in shared memory, and
// finds where the tile's compacted codes and outliers start in the output
// through a decoupled look-back over per-tile outlier counts, so the input is
// read once and every output byte is written once.
//
// Bit-exactness contract (what PyTorch's CPU kernels compute for fp16 blocks):
//   mean  = fp16(S / n), S = fp32 sum in ATen's vectorised order: 8 lanes
//           (element i -> lane i % 8), four interleaved accumulators per lane
//           (8-wide chunk j -> accumulator j % 4), folded ((a0+a1)+a2)+a3,
//           lanes added 0..7                              (:46, torch.mean)
//   std   = fp16((float)sqrt(M2 / (n - 1))), M2 in fp64      (:47, torch.std)
//   z     = fp16(fp16(x - mean) / fp16(std + fp16(1e-6)))    (:49)
//   outlier iff |z| > fp16(z_threshold)                      (:107)
//   scale = max(fp16(max|non-outlier| / 127), fp16(1e-6)); 1.0 if none (:121-130)
//   code  = int8(clamp(rint(fp16(x / scale)), -127, 127))    (:125-126)
// The fp64 second moment is a two-pass sum here and a Welford recurrence in
// ATen; both carry ~1e-16 relative error, far below the fp16 rounding step.
#include <cmath>
#include <mutex>

#include "common.cuh"

namespace atlas {
namespace {

constexpr int QT_THREADS = 256;
constexpr int QT_TILE = 8192;             // elements per tile
constexpr int QT_WORDS = QT_TILE / 32;    // outlier-mask words per tile
constexpr int QT_MAX_BLOCKS = QT_TILE / 32;
constexpr int QT_SPIN_LIMIT = 1 << 20;    // bounded look-back wait (~0.1 s)

constexpr unsigned long long ST_AGG = 1ull << 62;     // tile's own outlier count is known
constexpr unsigned long long ST_PREFIX = 2ull << 62;  // inclusive count up to this tile is known
constexpr unsigned long long ST_VALUE = (1ull << 62) - 1;

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ float h2f_bits(uint16_t b) { return __half2float(__ushort_as_half(b)); }
__device__ __forceinline__ uint16_t f2h_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }

// int8 code of one value given the block's fp32 scale: adaptive_quantizer.py:125-126.
__device__ __forceinline__ int quant_code(float xf, float scale_f) {
    float q = h2f_bits(f2h_bits(__fdiv_rn(xf, scale_f)));  // quotient rounded to fp16 first
    float r = rintf(q);                                     // half to even, as torch.round
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    return (int)r;
}

struct QuantParams {
    const uint16_t *x;
    int64_t numel;
    int64_t padded;
    int64_t n_blocks;
    int64_t num_tiles;
    int bs;
    uint16_t thr_h;
    int8_t *codes;
    uint16_t *ovals;
    int64_t *oidx;
    int64_t ocap;
    uint16_t *scales;
    int64_t *counts;
    unsigned int *tile_counter;
    unsigned long long *status;
    int in_aligned;   // x is 16-byte aligned
    int out_aligned;  // codes is 16-byte aligned
    int tile;         // elements per tile: the largest multiple of the block size <= QT_TILE
};

__global__ void __launch_bounds__(QT_THREADS) quantize_kernel(QuantParams p) {
    __shared__ __align__(16) uint16_t s_x[QT_TILE];
    __shared__ __align__(16) uint8_t s_codes[QT_TILE + 32];
    __shared__ uint32_t s_mask[QT_WORDS];
    __shared__ uint32_t s_wordpre[QT_WORDS];
    __shared__ uint16_t s_scale[QT_MAX_BLOCKS];
    __shared__ uint32_t s_warp_tot[QT_THREADS / 32];
    __shared__ long long s_tile_prefix;
    __shared__ int s_tile_total;
    __shared__ unsigned int s_tile;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int bs = p.bs;
    const uint16_t eps_h = f2h_bits(1e-6f);
    const float eps_f = h2f_bits(eps_h);
    const float thr_f = h2f_bits(p.thr_h);

    for (;;) {
        __syncthreads();  // previous tile's shared state is no longer read
        if (tid == 0) s_tile = atomicAdd(p.tile_counter, 1u);
        __syncthreads();
        const int64_t tile = s_tile;
        if (tile >= p.num_tiles) break;
        const int64_t tile_base = tile * p.tile;   // tiles hold whole blocks
        const int tile_elems = (int)min((int64_t)p.tile, p.padded - tile_base);
        const int tile_real = (int)max((int64_t)0, min((int64_t)tile_elems, p.numel - tile_base));
        const int tile_blocks = tile_elems / bs;

        // ---- stage the tile (zero padding included) -------------------------------
        if (p.in_aligned) {
            const uint4 *src = reinterpret_cast<const uint4 *>(p.x + tile_base);
            for (int v = tid; v < QT_TILE / 8; v += QT_THREADS) {
                int e0 = v * 8;
                if (e0 + 8 <= tile_real) {
                    reinterpret_cast<uint4 *>(s_x)[v] = __ldg(src + v);
                } else if (e0 < tile_elems) {
                    for (int e = e0; e < e0 + 8; ++e) s_x[e] = (e < tile_real) ? p.x[tile_base + e] : (uint16_t)0;
                }
            }
        } else {
            for (int e = tid; e < tile_elems; e += QT_THREADS)
                s_x[e] = (e < tile_real) ? p.x[tile_base + e] : (uint16_t)0;
        }
        for (int w = tid; w < QT_WORDS; w += QT_THREADS) s_mask[w] = 0u;
        __syncthreads();

        // ---- phase A: per-block statistics, 8 threads per block ----------------------
        {
            const int l = tid & 7;    // ATen SIMD lane this thread plays
            const int grp = tid >> 3;
            const unsigned gmask = 0xffu << (lane & 24);
            const int nv = bs >> 3;   // 8-wide chunks per block (multiple of 4)
            for (int b = grp; b < tile_blocks; b += QT_THREADS / 8) {
                const uint16_t *xb = s_x + b * bs;
                // fp32 sum in ATen's order + exact fp64 sum
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                double dsum = 0.0;
                for (int j = 0; j < nv; j += 4) {
                    float f0 = h2f_bits(xb[(j + 0) * 8 + l]);
                    float f1 = h2f_bits(xb[(j + 1) * 8 + l]);
                    float f2 = h2f_bits(xb[(j + 2) * 8 + l]);
                    float f3 = h2f_bits(xb[(j + 3) * 8 + l]);
                    a0 = __fadd_rn(a0, f0);
                    a1 = __fadd_rn(a1, f1);
                    a2 = __fadd_rn(a2, f2);
                    a3 = __fadd_rn(a3, f3);
                    dsum += ((double)f0 + (double)f1) + ((double)f2 + (double)f3);  // exact
                }
                float lane_sum = __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3);
                float fin = 0.f;
#pragma unroll
                for (int s = 0; s < 8; ++s) fin = __fadd_rn(fin, __shfl_sync(gmask, lane_sum, s, 8));
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) dsum += __shfl_xor_sync(gmask, dsum, o, 8);
                const float mean_f = h2f_bits(f2h_bits(__fdiv_rn(fin, (float)bs)));
                const double mean_d = dsum / (double)bs;
                // second moment in fp64
                double m2 = 0.0;
                for (int j = 0; j < nv; ++j) {
                    double d = (double)h2f_bits(xb[j * 8 + l]) - mean_d;
                    m2 = fma(d, d, m2);
                }
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) m2 += __shfl_xor_sync(gmask, m2, o, 8);
                const double var = m2 / (double)(bs - 1);
                const float std_f = h2f_bits(f2h_bits(__double2float_rn(sqrt(var))));
                const float den_f = h2f_bits(f2h_bits(__fadd_rn(std_f, eps_f)));
                // z test, outlier mask, absmax of the rest
                int cnt = 0;
                unsigned int maxabs = 0;  // fp16 magnitude bits order like the values
                for (int j = 0; j < nv; ++j) {
                    const int e = j * 8 + l;
                    const uint16_t xbits = xb[e];
                    const float xf = h2f_bits(xbits);
                    const float d = h2f_bits(f2h_bits(__fsub_rn(xf, mean_f)));
                    const float z = h2f_bits(f2h_bits(__fdiv_rn(d, den_f)));
                    if (fabsf(z) > thr_f) {
                        const int pos = b * bs + e;
                        atomicOr(&s_mask[pos >> 5], 1u << (pos & 31));
                        cnt++;
                    } else {
                        maxabs = max(maxabs, (unsigned int)(xbits & 0x7fffu));
                    }
                }
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    cnt += __shfl_xor_sync(gmask, cnt, o, 8);
                    maxabs = max(maxabs, __shfl_xor_sync(gmask, maxabs, o, 8));
                }
                if (l == 0) {
                    uint16_t sc = 0x3c00u;  // 1.0 when the block has no non-outliers
                    if (cnt < bs) {
                        sc = f2h_bits(__fdiv_rn(h2f_bits((uint16_t)maxabs), 127.0f));
                        if (h2f_bits(sc) < eps_f) sc = eps_h;
                    }
                    s_scale[b] = sc;
                }
            }
        }
        __syncthreads();

        // ---- exclusive scan of outliers per mask word --------------------------------
        {
            const uint32_t c = __popc(s_mask[tid]);  // QT_WORDS == QT_THREADS
            uint32_t inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += n;
            }
            if (lane == 31) s_warp_tot[warp] = inc;
            __syncthreads();
            uint32_t wbase = 0;
            for (int w = 0; w < warp; ++w) wbase += s_warp_tot[w];
            s_wordpre[tid] = wbase + inc - c;
            if (tid == QT_THREADS - 1) s_tile_total = (int)(wbase + inc);
        }
        __syncthreads();

        // ---- decoupled look-back over tiles (warp 0) -------------------------------------
        if (warp == 0) {
            const unsigned long long agg = (unsigned long long)s_tile_total;
            long long prefix = 0;
            if (tile == 0) {
                if (lane == 0) st_release_u64(p.status, ST_PREFIX | agg);
            } else {
                if (lane == 0) st_release_u64(p.status + tile, ST_AGG | agg);
                int64_t look = tile - 1;
                bool done = false;
                while (!done) {
                    const int64_t idx = look - lane;
                    unsigned long long v = ST_PREFIX;  // tiles before the first count as prefix 0
                    int spins = 0;
                    bool gave_up = false;
                    for (;;) {
                        if (idx >= 0) v = ld_acquire_u64(p.status + idx);
                        const bool ready = (v >> 62) != 0;
                        if (__all_sync(0xffffffffu, ready)) break;
                        if (++spins > QT_SPIN_LIMIT) { gave_up = true; break; }
                        __nanosleep(64);
                    }
                    if (gave_up) {  // record and leave; the host reports ATLAS_ERR_TIMEOUT
                        if (lane == 0) atomicExch((unsigned long long *)&p.counts[2], 1ull);
                        break;
                    }
                    const unsigned pm = __ballot_sync(0xffffffffu, (v >> 62) == 2);
                    const int first = pm ? (__ffs(pm) - 1) : 32;
                    long long contrib = (lane <= first) ? (long long)(v & ST_VALUE) : 0;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
                    prefix += contrib;
                    if (pm) done = true; else look -= 32;
                }
                if (lane == 0) st_release_u64(p.status + tile, ST_PREFIX | (unsigned long long)(prefix + (long long)agg));
            }
            if (lane == 0) {
                s_tile_prefix = prefix;
                if (tile == p.num_tiles - 1) {
                    const long long total_out = prefix + (long long)agg;
                    p.counts[0] = p.padded - total_out;
                    p.counts[1] = total_out;
                }
            }
        }
        __syncthreads();

        // ---- phase B: codes into a shared staging buffer, outliers straight out --------
        const long long tile_prefix = s_tile_prefix;
        const int64_t code_base = tile_base - tile_prefix;  // where this tile's codes start
        const int shift = p.out_aligned ? (int)(code_base & 15) : 0;
        for (int i = tid * 4; i < tile_elems; i += QT_THREADS * 4) {
            const float sc_f = h2f_bits(s_scale[i / bs]);
            const uint32_t word = s_mask[i >> 5];
            const uint32_t m4 = (word >> (i & 31)) & 0xfu;
            int before = (int)s_wordpre[i >> 5] + __popc(word & ((1u << (i & 31)) - 1u));
            const uint2 raw = *reinterpret_cast<const uint2 *>(s_x + i);
            const uint16_t xs[4] = {(uint16_t)(raw.x & 0xffffu), (uint16_t)(raw.x >> 16),
                                    (uint16_t)(raw.y & 0xffffu), (uint16_t)(raw.y >> 16)};
            const int dst = shift + i - before;
            if (m4 == 0u && (dst & 3) == 0) {
                uint32_t packed = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    packed |= (uint32_t)(quant_code(h2f_bits(xs[e]), sc_f) & 0xff) << (8 * e);
                *reinterpret_cast<uint32_t *>(s_codes + dst) = packed;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if ((m4 >> e) & 1u) {
                        const long long pos = tile_prefix + before;
                        if (pos < p.ocap) {
                            p.ovals[pos] = xs[e];
                            p.oidx[pos] = tile_base + i + e;
                        }
                        before++;
                    } else {
                        s_codes[shift + i + e - before] = (uint8_t)quant_code(h2f_bits(xs[e]), sc_f);
                    }
                }
            }
        }
        __syncthreads();

        // ---- copy the compacted codes out: 16-byte stores inside, bytes at the ragged ends --
        {
            const int total = tile_elems - s_tile_total;  // code bytes of this tile
            const int end = shift + total;
            int8_t *gdst = p.codes + (code_base - shift);  // 16-byte aligned when out_aligned
            const int nchunks = (end + 15) >> 4;
            for (int c = tid; c < nchunks; c += QT_THREADS) {
                const int lo = c << 4;
                if (p.out_aligned && lo >= shift && lo + 16 <= end) {
                    *reinterpret_cast<uint4 *>(gdst + lo) = *reinterpret_cast<const uint4 *>(s_codes + lo);
                } else {
                    const int a = max(lo, shift), z = min(lo + 16, end);
                    for (int q = a; q < z; ++q) gdst[q] = (int8_t)s_codes[q];
                }
            }
            const int64_t block0 = tile_base / bs;
            for (int b = tid; b < tile_blocks; b += QT_THREADS) p.scales[block0 + b] = s_scale[b];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Fast variant for block sizes 32 / 64 / 128 / 256 (EPT = block_size / 8 values per thread, kept
// in registers).  Same results as quantize_kernel above, bit for bit, with most of the IEEE
// divisions and all of the fp64 work moved off the common path:
//   * the second moment is accumulated in fp32 (error <= ~1e-6 relative); only if rounding the
//     standard deviation to fp16 could go either way within 4e-6 is it recomputed in fp64;
//   * |fp16(d / den)| > thr is decided from d * (1 / den) against the real number at which the
//     rounded quotient crosses thr, with a 2^-21 guard band inside which the exact quotient is used;
//   * fp16(x / scale) is taken from x * (1 / scale) when nudging the product by 2^-22 either way
//     rounds to the same fp16 number, else from the exact quotient.
// Codes are written once, uncompacted, to shared memory by the threads that computed the block
// statistics; the compaction pass only moves bytes.
struct FastConsts {
    float t_lo, t_hi;  // guard band around the |z| decision boundary
    float thr_f;
};

template <int EPT>
__global__ void __launch_bounds__(QT_THREADS, (EPT <= 16 ? 5 : 2)) quantize_fast_kernel(QuantParams p, FastConsts fc) {
    constexpr int BS = EPT * 8;
    constexpr int TILE_BLOCKS = QT_TILE / BS;
    // Blocks are padded (16 bytes of values, 8 bytes of codes) so that the four blocks a warp works
    // on at a time fall on different banks.
    constexpr int XSTRIDE = BS * 2 + 16;  // bytes
    constexpr int DSTRIDE = BS + 8;
    __shared__ __align__(16) uint8_t s_xb[TILE_BLOCKS * XSTRIDE];
    __shared__ __align__(16) uint8_t s_dense[TILE_BLOCKS * DSTRIDE];
    auto xref = [&](int e) -> uint16_t & {
        return *reinterpret_cast<uint16_t *>(s_xb + (e / BS) * XSTRIDE + (e % BS) * 2);
    };
    __shared__ __align__(16) uint8_t s_codes[QT_TILE + 32];
    __shared__ uint32_t s_mask[QT_WORDS];
    __shared__ uint32_t s_wordpre[QT_WORDS];
    __shared__ uint16_t s_scale[TILE_BLOCKS];
    __shared__ uint32_t s_warp_tot[QT_THREADS / 32];
    __shared__ long long s_tile_prefix;
    __shared__ int s_tile_total;
    __shared__ unsigned int s_tile;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint16_t eps_h = f2h_bits(1e-6f);
    const float eps_f = h2f_bits(eps_h);

    for (;;) {
        __syncthreads();  // previous tile's shared state is no longer read
        if (tid == 0) s_tile = atomicAdd(p.tile_counter, 1u);
        __syncthreads();
        const int64_t tile = s_tile;
        if (tile >= p.num_tiles) break;
        const int64_t tile_base = tile * QT_TILE;
        const int tile_elems = (int)min((int64_t)QT_TILE, p.padded - tile_base);
        const int tile_real = (int)max((int64_t)0, min((int64_t)tile_elems, p.numel - tile_base));
        const int tile_blocks = tile_elems / BS;

        // ---- stage the tile (zero padding included) -------------------------------
        if (p.in_aligned) {
            const uint4 *src = reinterpret_cast<const uint4 *>(p.x + tile_base);
            for (int v = tid; v < QT_TILE / 8; v += QT_THREADS) {
                int e0 = v * 8;
                if (e0 + 8 <= tile_real) {
                    *reinterpret_cast<uint4 *>(s_xb + (e0 / BS) * XSTRIDE + (e0 % BS) * 2) = __ldg(src + v);
                } else if (e0 < tile_elems) {
                    for (int e = e0; e < e0 + 8; ++e) xref(e) = (e < tile_real) ? p.x[tile_base + e] : (uint16_t)0;
                }
            }
        } else {
            for (int e = tid; e < tile_elems; e += QT_THREADS)
                xref(e) = (e < tile_real) ? p.x[tile_base + e] : (uint16_t)0;
        }
        for (int w = tid; w < QT_WORDS; w += QT_THREADS) s_mask[w] = 0u;
        __syncthreads();

        // ---- phase A: statistics and codes of whole blocks, 8 threads per block ----------
        {
            const int l = tid & 7;    // ATen SIMD lane this thread plays
            const int grp = tid >> 3;
            const unsigned gmask = 0xffu << (lane & 24);
            for (int b = grp; b < tile_blocks; b += QT_THREADS / 8) {
                const uint16_t *xb = reinterpret_cast<const uint16_t *>(s_xb + b * XSTRIDE);
                float f[EPT];
#pragma unroll
                for (int j = 0; j < EPT; ++j) f[j] = h2f_bits(xb[j * 8 + l]);
                // fp32 sum in ATen's order
                float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < EPT; ++j) a4[j & 3] = __fadd_rn(a4[j & 3], f[j]);
                const float lane_sum = __fadd_rn(__fadd_rn(__fadd_rn(a4[0], a4[1]), a4[2]), a4[3]);
                float fin = 0.f;
#pragma unroll
                for (int s = 0; s < 8; ++s) fin = __fadd_rn(fin, __shfl_sync(gmask, lane_sum, s, 8));
                const float mean32 = __fdiv_rn(fin, (float)BS);
                const float mean_f = h2f_bits(f2h_bits(mean32));
                // second moment: fp32 first
                // (about mean32, with the first moment about it taken out again, so that the rounding
                // of mean32 itself only enters to second order)
                float m2f = 0.f, r1 = 0.f;
#pragma unroll
                for (int j = 0; j < EPT; ++j) {
                    const float d = f[j] - mean32;
                    r1 += d;
                    m2f = fmaf(d, d, m2f);
                }
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    m2f += __shfl_xor_sync(gmask, m2f, o, 8);
                    r1 += __shfl_xor_sync(gmask, r1, o, 8);
                }
                m2f = fmaxf(fmaf(-r1, r1 * (1.f / (float)BS), m2f), 0.f);
                const float std32 = __fsqrt_rn(__fdiv_rn(m2f, (float)(BS - 1)));
                uint16_t std_h = f2h_bits(std32 * (1.f - 4e-6f));
                if (std_h != f2h_bits(std32 * (1.f + 4e-6f))) {
                    // the fp16 rounding is within reach of the fp32 error: redo it in fp64 (group-uniform)
                    double dsum = 0.0;
#pragma unroll
                    for (int j = 0; j < EPT; ++j) dsum += (double)f[j];
#pragma unroll
                    for (int o = 1; o < 8; o <<= 1) dsum += __shfl_xor_sync(gmask, dsum, o, 8);
                    const double mean_d = dsum / (double)BS;
                    double m2 = 0.0;
#pragma unroll
                    for (int j = 0; j < EPT; ++j) {
                        const double d = (double)f[j] - mean_d;
                        m2 = fma(d, d, m2);
                    }
#pragma unroll
                    for (int o = 1; o < 8; o <<= 1) m2 += __shfl_xor_sync(gmask, m2, o, 8);
                    std_h = f2h_bits(__double2float_rn(sqrt(m2 / (double)(BS - 1))));
                }
                const float den_f = h2f_bits(f2h_bits(__fadd_rn(h2f_bits(std_h), eps_f)));
                // |d| / den against the threshold = |d| against threshold * den: the block's two bounds are one
                // rounding away from exact, well inside the guard band they delimit
                const float lo_b = fc.t_lo * den_f, hi_b = fc.t_hi * den_f;
                // z test, outlier mask, absmax of the rest
                unsigned int omask = 0;   // bit j: element j of this thread is an outlier
                unsigned int maxabs = 0;  // fp32 bits of the largest |x| kept (bit patterns order like the values)
#pragma unroll
                for (int j = 0; j < EPT; ++j) {
                    const float d = h2f_bits(f2h_bits(__fsub_rn(f[j], mean_f)));
                    const float a = fabsf(d);
                    bool is_out = a > hi_b;
                    if (!is_out && a >= lo_b) {   // inside the guard band: the exact rounded quotient decides
                        const float z = h2f_bits(f2h_bits(__fdiv_rn(d, den_f)));
                        is_out = fabsf(z) > fc.thr_f;
                    }
                    if (is_out) omask |= 1u << j;
                    else maxabs = max(maxabs, __float_as_uint(f[j]) & 0x7fffffffu);
                }
                int cnt = __popc(omask);
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    cnt += __shfl_xor_sync(gmask, cnt, o, 8);
                    maxabs = max(maxabs, __shfl_xor_sync(gmask, maxabs, o, 8));
                }
                uint16_t sc = 0x3c00u;  // 1.0 when the block has no non-outliers
                if (cnt < BS) {
                    sc = f2h_bits(__fdiv_rn(__uint_as_float(maxabs), 127.0f));
                    if (h2f_bits(sc) < eps_f) sc = eps_h;
                }
                if (l == 0) s_scale[b] = sc;
                const float sc_f = h2f_bits(sc);
                const float rsc = __frcp_rn(sc_f);
                uint8_t *db = s_dense + b * DSTRIDE + l;
#pragma unroll
                for (int j = 0; j < EPT; ++j) {
                    const float v = f[j] * rsc;   // within 2^-22 of x / scale
                    uint16_t qh = f2h_bits(v);
                    // fp16 keeps 10 of the 23 mantissa bits: v rounds the other way only if its 13 low bits are within a
                    // few units of the midpoint 0x1000 (results below the fp16 normal range give code 0 either way)
                    if (((__float_as_uint(v) & 0x1fffu) - (0x1000u - 8u)) <= 16u) qh = f2h_bits(__fdiv_rn(f[j], sc_f));
                    int r = __half2int_rn(__ushort_as_half(qh));   // half to even, as torch.round
                    r = max(-127, min(127, r));
                    db[j * 8] = (uint8_t)r;
                }
                if (omask) {
#pragma unroll
                    for (int j = 0; j < EPT; ++j)
                        if ((omask >> j) & 1u) {
                            const int pos = b * BS + j * 8 + l;
                            atomicOr(&s_mask[pos >> 5], 1u << (pos & 31));
                        }
                }
            }
        }
        __syncthreads();

        // ---- exclusive scan of outliers per mask word --------------------------------
        {
            const uint32_t c = __popc(s_mask[tid]);  // QT_WORDS == QT_THREADS
            uint32_t inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += n;
            }
            if (lane == 31) s_warp_tot[warp] = inc;
            __syncthreads();
            uint32_t wbase = 0;
            for (int w = 0; w < warp; ++w) wbase += s_warp_tot[w];
            s_wordpre[tid] = wbase + inc - c;
            if (tid == QT_THREADS - 1) s_tile_total = (int)(wbase + inc);
        }
        __syncthreads();

        // ---- decoupled look-back over tiles (warp 0) -------------------------------------
        if (warp == 0) {
            const unsigned long long agg = (unsigned long long)s_tile_total;
            long long prefix = 0;
            if (tile == 0) {
                if (lane == 0) st_release_u64(p.status, ST_PREFIX | agg);
            } else {
                if (lane == 0) st_release_u64(p.status + tile, ST_AGG | agg);
                int64_t look = tile - 1;
                bool done = false;
                while (!done) {
                    const int64_t idx = look - lane;
                    unsigned long long v = ST_PREFIX;  // tiles before the first count as prefix 0
                    int spins = 0;
                    bool gave_up = false;
                    for (;;) {
                        if (idx >= 0) v = ld_acquire_u64(p.status + idx);
                        const bool ready = (v >> 62) != 0;
                        if (__all_sync(0xffffffffu, ready)) break;
                        if (++spins > QT_SPIN_LIMIT) { gave_up = true; break; }
                        __nanosleep(64);
                    }
                    if (gave_up) {  // record and leave; the host reports ATLAS_ERR_TIMEOUT
                        if (lane == 0) atomicExch((unsigned long long *)&p.counts[2], 1ull);
                        break;
                    }
                    const unsigned pm = __ballot_sync(0xffffffffu, (v >> 62) == 2);
                    const int first = pm ? (__ffs(pm) - 1) : 32;
                    long long contrib = (lane <= first) ? (long long)(v & ST_VALUE) : 0;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
                    prefix += contrib;
                    if (pm) done = true; else look -= 32;
                }
                if (lane == 0) st_release_u64(p.status + tile, ST_PREFIX | (unsigned long long)(prefix + (long long)agg));
            }
            if (lane == 0) {
                s_tile_prefix = prefix;
                if (tile == p.num_tiles - 1) {
                    const long long total_out = prefix + (long long)agg;
                    p.counts[0] = p.padded - total_out;
                    p.counts[1] = total_out;
                }
            }
        } else {
            // ---- meanwhile, warps 1..7 compact the codes in shared memory (needs no prefix) ----------
            for (int i = (tid - 32) * 4; i < tile_elems; i += (QT_THREADS - 32) * 4) {
                const uint32_t word = s_mask[i >> 5];
                const uint32_t m4 = (word >> (i & 31)) & 0xfu;
                const int before = (int)s_wordpre[i >> 5] + __popc(word & ((1u << (i & 31)) - 1u));
                const uint32_t c4 = *reinterpret_cast<const uint32_t *>(s_dense + (i / BS) * DSTRIDE + (i % BS));
                int dst = i - before;
                if (m4 == 0u && (dst & 3) == 0) {
                    *reinterpret_cast<uint32_t *>(s_codes + dst) = c4;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (!((m4 >> e) & 1u)) s_codes[dst++] = (uint8_t)(c4 >> (8 * e));
                }
            }
        }
        __syncthreads();

        // ---- with the prefix: outliers straight out, one mask word per thread ------------------------
        const long long tile_prefix = s_tile_prefix;
        const int64_t code_base = tile_base - tile_prefix;  // where this tile's codes start
        const int shift = p.out_aligned ? (int)(code_base & 15) : 0;
        {
            uint32_t word = s_mask[tid];   // QT_WORDS == QT_THREADS
            long long pos = tile_prefix + s_wordpre[tid];
            while (word) {
                const int e = tid * 32 + __ffs(word) - 1;
                word &= word - 1;
                if (pos < p.ocap) {
                    p.ovals[pos] = xref(e);
                    p.oidx[pos] = tile_base + e;
                }
                ++pos;
            }
        }

        // ---- copy the compacted codes out: 16-byte stores to aligned global addresses, the shared-memory side is
        // read at whatever byte offset the tile's start in the code stream leaves (five words and a funnel shift)
        {
            const int total = tile_elems - s_tile_total;  // code bytes of this tile
            const int end = shift + total;
            int8_t *gdst = p.codes + (code_base - shift);  // 16-byte aligned when out_aligned
            const int nchunks = (end + 15) >> 4;
            const uint32_t *s32 = reinterpret_cast<const uint32_t *>(s_codes);
            for (int c = tid; c < nchunks; c += QT_THREADS) {
                const int lo = c << 4;
                if (p.out_aligned && lo >= shift && lo + 16 <= end) {
                    const int o = lo - shift;
                    const int wi = o >> 2, r = (o & 3) * 8;
                    const uint32_t w0 = s32[wi], w1 = s32[wi + 1], w2 = s32[wi + 2], w3 = s32[wi + 3], w4 = s32[wi + 4];
                    uint4 v;
                    v.x = __funnelshift_r(w0, w1, r);
                    v.y = __funnelshift_r(w1, w2, r);
                    v.z = __funnelshift_r(w2, w3, r);
                    v.w = __funnelshift_r(w3, w4, r);
                    *reinterpret_cast<uint4 *>(gdst + lo) = v;
                } else {
                    const int a = max(lo, shift), z = min(lo + 16, end);
                    for (int q = a; q < z; ++q) gdst[q] = (int8_t)s_codes[q - shift];
                }
            }
            const int64_t block0 = tile_base / BS;
            for (int b = tid; b < tile_blocks; b += QT_THREADS) p.scales[block0 + b] = s_scale[b];
        }
    }
}

// |fp16(q)| > thr_h  <=>  |q| beyond T, the midpoint between thr_h and the next fp16 number above it
// (a tie goes to the even neighbour).  Returns T; the kernel uses the exact quotient inside a guard band.
FastConsts make_fast_consts(uint16_t thr_h) {
    FastConsts fc;
    const float thr = __half2float(__ushort_as_half(thr_h));
    fc.thr_f = thr;
    float T;
    if ((thr_h & 0x7fffu) > 0x7c00u) T = INFINITY;            // NaN threshold: nothing compares greater
    else if (thr_h == 0x7c00u) T = INFINITY;                   // +inf
    else if (thr_h & 0x8000u) T = -1.f;                        // negative threshold: every |z| is greater
    else if (thr_h == 0x7bffu) T = 65520.f;                    // next above the largest finite is inf
    else T = 0.5f * (thr + __half2float(__ushort_as_half((uint16_t)(thr_h + 1))));
    if (T == INFINITY) { fc.t_lo = INFINITY; fc.t_hi = INFINITY; }
    else if (T < 0.f) { fc.t_lo = -2.f; fc.t_hi = -1.f; }
    else { fc.t_lo = T * (1.f - 4.8e-7f); fc.t_hi = T * (1.f + 4.8e-7f); }
    return fc;
}

struct DeviceInfo {
    int dev = -1;
    int sms = 0;
    int quant_ctas_per_sm = 0;
};

int device_info(DeviceInfo &out) {
    static thread_local DeviceInfo cache;
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (cache.dev != dev) {
        DeviceInfo d;
        d.dev = dev;
        rc = check_cuda(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev), "sm count");
        if (rc) return rc;
        rc = check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&d.quant_ctas_per_sm, quantize_kernel,
                                                                      QT_THREADS, 0),
                        "occupancy(quantize_kernel)");
        if (rc) return rc;
        if (d.quant_ctas_per_sm < 1) d.quant_ctas_per_sm = 1;
        cache = d;
    }
    out = cache;
    return ATLAS_OK;
}

}  // namespace
}  // namespace atlas

extern "C" {

size_t atlas_quantize_workspace_bytes(int64_t numel, int block_size) {
    if (numel <= 0 || block_size <= 0 || block_size > atlas::QT_TILE) return 16;
    const int64_t padded = atlas::ceil_div_i64(numel, block_size) * block_size;
    const int64_t tile = (atlas::QT_TILE / block_size) * block_size;   // a tile holds whole blocks
    const int64_t tiles = atlas::ceil_div_i64(padded, tile);
    return (size_t)(16 + 8 * tiles);
}

int atlas_quantize(const void *w, int64_t numel, int block_size, double z_threshold, int8_t *codes,
                   void *outlier_vals, int64_t *outlier_idx, int64_t outlier_capacity, void *scales,
                   int64_t *counts, void *workspace, size_t workspace_bytes, void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(numel < 0 || counts == nullptr || outlier_capacity < 0, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_quantize: negative size or null counts");
    ATLAS_RETURN_IF(block_size < 32 || block_size > 512 || block_size % 32 != 0, ATLAS_ERR_UNSUPPORTED,
                    "atlas_quantize: block_size %d is not a multiple of 32 in [32, 512]", block_size);
    int rc = check_device();
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    rc = check_cuda(cudaMemsetAsync(counts, 0, 4 * sizeof(int64_t), st), "memset(counts)");
    if (rc) return rc;
    if (numel == 0) return ATLAS_OK;
    ATLAS_RETURN_IF(!w || !codes || !scales || !workspace ||
                        (outlier_capacity > 0 && (!outlier_vals || !outlier_idx)),
                    ATLAS_ERR_BAD_ARGUMENT, "atlas_quantize: null buffer");
    const size_t need = atlas_quantize_workspace_bytes(numel, block_size);
    ATLAS_RETURN_IF(workspace_bytes < need, ATLAS_ERR_CAPACITY,
                    "atlas_quantize: workspace holds %zu bytes, %zu needed", workspace_bytes, need);
    ATLAS_RETURN_IF(((uintptr_t)workspace & 15) != 0 || ((uintptr_t)w & 1) != 0 ||
                        ((uintptr_t)outlier_idx & 7) != 0 || ((uintptr_t)counts & 7) != 0,
                    ATLAS_ERR_BAD_ARGUMENT, "atlas_quantize: misaligned buffer");

    QuantParams p;
    p.x = (const uint16_t *)w;
    p.numel = numel;
    p.n_blocks = ceil_div_i64(numel, block_size);
    p.padded = p.n_blocks * block_size;
    p.tile = (QT_TILE / block_size) * block_size;
    p.num_tiles = ceil_div_i64(p.padded, p.tile);
    p.bs = block_size;
    p.thr_h = __half_as_ushort(__float2half_rn((float)z_threshold));
    p.codes = codes;
    p.ovals = (uint16_t *)outlier_vals;
    p.oidx = outlier_idx;
    p.ocap = outlier_capacity;
    p.scales = (uint16_t *)scales;
    p.counts = counts;
    p.tile_counter = (unsigned int *)workspace;
    p.status = (unsigned long long *)((char *)workspace + 16);
    p.in_aligned = ((uintptr_t)w & 15) == 0;
    p.out_aligned = ((uintptr_t)codes & 15) == 0;

    rc = check_cuda(cudaMemsetAsync(workspace, 0, need, st), "memset(workspace)");
    if (rc) return rc;
    DeviceInfo di;
    rc = device_info(di);
    if (rc) return rc;
    const bool fast = block_size == 32 || block_size == 64 || block_size == 128 || block_size == 256;
    const int per_sm = fast ? (block_size == 256 ? 2 : 5) : di.quant_ctas_per_sm;   // resident CTAs of the fast kernels
    const int64_t max_ctas = (int64_t)di.sms * per_sm;
    const int grid = (int)(p.num_tiles < max_ctas ? p.num_tiles : max_ctas);
    if (fast) {
        const FastConsts fc = make_fast_consts(p.thr_h);
        switch (block_size) {
            case 32: quantize_fast_kernel<4><<<grid, QT_THREADS, 0, st>>>(p, fc); break;
            case 64: quantize_fast_kernel<8><<<grid, QT_THREADS, 0, st>>>(p, fc); break;
            case 128: quantize_fast_kernel<16><<<grid, QT_THREADS, 0, st>>>(p, fc); break;
            default: quantize_fast_kernel<32><<<grid, QT_THREADS, 0, st>>>(p, fc); break;
        }
        return check_cuda(cudaGetLastError(), "quantize_fast_kernel launch");
    }
    quantize_kernel<<<grid, QT_THREADS, 0, st>>>(p);
    return check_cuda(cudaGetLastError(), "quantize_kernel launch");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Quantize without any allocation by anyone: scratch in a file-scope device array.
//
// The look-back needs a tile counter and one status word per tile.  atlas_quantize takes them
// from a caller-provided workspace; callers that are not allowed to allocate device memory at
// the point of the call (a pre-allocated arena they may not grow, a fixed-memory serving loop
// where every cudaMalloc is a synchronisation and a fragmentation risk, a plug-in host that
// owns the allocator) cannot provide one.  For them the same kernel runs against the static
// array below, sized for ATLAS_QUANTIZE_NOALLOC_MAX_ELEMENTS padded elements (64 Mi: 8192 tiles,
// 64 KB + 16 B).  The array lives in every context that loads this library until it exits.
constexpr int64_t NOALLOC_MAX_TILES = ATLAS_QUANTIZE_NOALLOC_MAX_ELEMENTS / atlas::QT_TILE;
static __device__ __align__(256) unsigned char g_quantize_scratch[16 + 8 * NOALLOC_MAX_TILES];

namespace {
// In host code `g_quantize_scratch` is only a handle for the symbol, not a device address: the
// address is looked up once per device, with that device current, and cached.
int noalloc_scratch_ptr(void **out) {
    constexpr int kMaxDevices = 64;
    static void *cache[kMaxDevices] = {nullptr};
    static std::mutex mu;
    int dev = -1;
    int rc = atlas::check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= kMaxDevices) {
        atlas::set_error("atlas_quantize_noalloc: device ordinal %d outside [0, %d)", dev, kMaxDevices);
        return ATLAS_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == nullptr) {
        void *ptr = nullptr;
        rc = atlas::check_cuda(cudaGetSymbolAddress(&ptr, g_quantize_scratch),
                               "cudaGetSymbolAddress(g_quantize_scratch)");
        if (rc) return rc;
        cache[dev] = ptr;
    }
    *out = cache[dev];
    return ATLAS_OK;
}
}  // namespace

extern "C" int atlas_quantize_noalloc(const void *w, int64_t numel, int block_size, double z_threshold,
                                      int8_t *codes, void *outlier_vals, int64_t *outlier_idx,
                                      int64_t outlier_capacity, void *scales, int64_t *counts, void *stream) {
    using namespace atlas;
    clear_error();
    ATLAS_RETURN_IF(numel < 0 || block_size <= 0, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_quantize_noalloc: negative size or block size");
    const int64_t padded = ceil_div_i64(numel, block_size) * block_size;
    ATLAS_RETURN_IF(padded > ATLAS_QUANTIZE_NOALLOC_MAX_ELEMENTS, ATLAS_ERR_CAPACITY,
                    "atlas_quantize_noalloc: %lld padded elements exceed the static scratch limit of %lld; "
                    "use atlas_quantize with a caller-provided workspace",
                    (long long)padded, (long long)ATLAS_QUANTIZE_NOALLOC_MAX_ELEMENTS);
    // block sizes that do not divide the 8192-element tile use slightly smaller tiles, hence more status words
    ATLAS_RETURN_IF(block_size <= QT_TILE && atlas_quantize_workspace_bytes(numel, block_size) > sizeof(g_quantize_scratch),
                    ATLAS_ERR_CAPACITY,
                    "atlas_quantize_noalloc: %lld elements in blocks of %d exceed the static scratch limit; "
                    "use atlas_quantize with a caller-provided workspace", (long long)numel, block_size);
    void *scratch = nullptr;
    int rc = check_device();
    if (rc) return rc;
    rc = noalloc_scratch_ptr(&scratch);
    if (rc) return rc;
    // atlas_quantize zeroes the scratch it is given on the stream before the kernel runs
    return atlas_quantize(w, numel, block_size, z_threshold, codes, outlier_vals, outlier_idx, outlier_capacity,
                          scales, counts, scratch, sizeof(g_quantize_scratch), stream);
}
