// Decode-time quantized linear, m <= 32 rows of x per launch, the weight read once:
//     y[m][n] = sum_k x[m][k] * W[n][k] + bias[n]
//
// Replaces the steady state of QuantizedLinear.forward
// (integration/atlas_wrappers.py:56,67), which multiplies by a cached fp16 copy
// of the weight (2 bytes per weight).  This kernel streams the tile-major uint8
// codes (1 byte per weight), rebuilds in registers exactly the fp16 weight the
// reference's dequantizer produces (adaptive_quantizer.py:216:
// fp16(fp16(code) * scale)), multiplies on the tensor cores (mma.sync with the
// weights as the 16-row operand and the batch as 8-column tiles) and adds the
// fp16 outlier products in the same launch.  It is HBM-bound; everything here is
// about keeping HBM busy across a chain of launches that last microseconds.
//
// Work split.  The weight is a matrix of 8 KB tiles (128 rows x 64 columns,
// contiguous in the tile-major layout).  The tiles, taken row-tile-major, form
// one sequence of units that is cut into equal contiguous ranges, one per CTA
// (one CTA per SM), so every launch is balanced whatever its shape.  A range
// crosses row-tile boundaries: a row tile whose K range is shared by several
// CTAs is finished by whichever of them arrives last (a ticket per row tile),
// which adds the fp32 partial tiles in CTA order -- deterministic, and nobody
// ever waits for another CTA.
//
// Data movement.  Warp 0 issues one 8 KB bulk copy (plus the tile's scales) per
// unit into a ring of shared-memory stages and runs as far ahead as the ring
// allows; it touches only weights, so under programmatic dependent launch a CTA
// of the next linear fills its whole ring (~90 KB per SM, ~13 MB per GPU) while
// the previous linear still computes: the CTA is sized so that two launches are
// co-resident on an SM.  Warp 1 waits for the
// previous kernels, then puts each unit's 64 activation columns into the stage
// as fp16 (bf16 is converted here, once per CTA and unit, not once per warp).
// Eight consumer warps own one 16-row strip of the row tile each: 1 KB of codes
// per unit from shared memory, dequantised in registers, four MMAs per 8 batch
// rows.  A strip's outliers (sorted by column at repack time) are taken 16 at a
// time as one more MMA, interleaved with the dense steps; their activations are
// gathered from global memory (they stay in L1).
//
// Every wait is bounded; when one runs out the CTA sets the caller's status
// word, stops waiting and runs to its end on whatever data it has.
#include <cuda_bf16.h>

#include "common.cuh"

namespace atlas {
namespace {

constexpr int SK_CONSUMERS = 8;            // consumer warps = 16-row strips of a 128-row tile
constexpr int SK_TILE_BYTES = 8192;        // 128 rows x 64 codes
constexpr int SK_SPIN_LIMIT = 1 << 20;     // polls per bounded wait
constexpr int SK_MAX_GRID = 256;           // partial-tile slots in the workspace
constexpr int SK_MAX_TILE_ROWS = 16384;    // tickets in the workspace (n_rows <= 2 Mi)
constexpr size_t SK_TICKET_BYTES = (size_t)SK_MAX_TILE_ROWS * 4;
constexpr int SK_SMEM_BUDGET = 110 * 1024; // per CTA, so that two launches share an SM

struct StreamParams {
    const void *x;
    int dtype;
    int m;
    int64_t ldx;
    const uint8_t *tiles;
    const uint16_t *scales_t;   // [row/128][block][row%128]
    const int32_t *chunk_ptr;   // [strip][k_tiles + 1]: first outlier entry with column >= 64 * c
    const uint32_t *entries;    // row%16 << 24 | column, strip-major, column-sorted
    const uint16_t *ovals;      // fp16 outlier values in the order of `entries`
    const uint16_t *bias;
    void *y;
    int64_t ldy;
    int n_rows;
    int n_cols;
    int bs;
    int bs_shift;        // log2(block size) when it is a power of two, else -1
    int k_tiles;         // n_cols / 64
    int blocks_per_row;  // n_cols / bs
    int tile_rows;       // ceil(n_rows / 128)
    long long units;     // tile_rows * k_tiles
    int scale_cap;       // bytes reserved for scales in a stage (multiple of 256)
    int stage_stride;    // bytes per stage
    int n_stages;
    int x_vec_ok;        // x rows allow 16-byte loads
    unsigned int *tickets;   // [tile_rows], zero between launches
    float *partials;         // [grid][2][m][128] fp32
    int *status;             // device int, set non-zero if a bounded wait ran out (may be null)
    // column-parallel output: this rank's y goes straight into every rank's gathered buffer (world <= 1: plain y)
    int world;
    int rank;
    int wait_world;                          // arrival flags to wait on (the real number of ranks)
    void *y_dst[ATLAS_MAX_PEERS];            // where row 0, column 0 of this rank's y lands on each rank
    unsigned int *flags_dst[ATLAS_MAX_PEERS];   // each rank's arrival flags; this rank writes entry [rank]
    unsigned int *state;                     // local: [0] CTAs finished, [1] gather launches completed
    const unsigned int *wait_flags;          // local arrival flags to wait on before x is read (x was gathered), or null
    long long poll_limit;
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until every rank's arrival flag has reached `target` (a launch count); one lane per rank polls, at most
// `limit` times.  Returns false if the limit ran out.
__device__ __forceinline__ bool wait_arrivals(const unsigned int *flags, int world, unsigned int target, long long limit,
                                              int lane) {
    bool ok = true;
    if (lane < world) {
        ok = false;
        for (long long i = 0; i < limit; ++i) {
            if ((int)(ld_acquire_sys(flags + lane) - target) >= 0) { ok = true; break; }
            __nanosleep(64);
        }
    }
    return __all_sync(0xffffffffu, ok) != 0;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait that also gives up as soon as another thread of the CTA has.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int *abort_flag) {
    for (int i = 0; i < SK_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 63 && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(SK_CONSUMERS * 32) : "memory"); }

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm(
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

// Two bf16 (low, high half of v) -> two fp16, saturating at +-65504.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(v & 0xffff0000u)), "f"(__uint_as_float(v << 16)));
    return r;
}

__device__ __forceinline__ long long unit_begin(long long units, int grid, int cta) { return units * cta / grid; }

// MT: 8-column MMA tiles over the batch (m <= 8 * MT).
template <int MT>
struct StreamCfg {
    static constexpr int XP_WARPS = 1;                                     // activation producers
    static constexpr int FIRST_CONSUMER = 1 + XP_WARPS;
    static constexpr int THREADS = (FIRST_CONSUMER + SK_CONSUMERS) * 32;
    static constexpr int X_BYTES = MT * 8 * 128;                           // fp16 [MT*8 rows][64]
    static constexpr int OUT_LD = MT * 8;                                  // floats per row of the staging tile
    static constexpr int OUT_BYTES = 128 * OUT_LD * 4;
};

template <int MT>
__global__ void __launch_bounds__(StreamCfg<MT>::THREADS, 2) qlinear_stream_kernel(StreamParams p) {
    using C = StreamCfg<MT>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // let the next kernel of the stream become resident and start its own weight prefetch
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int NS = p.n_stages;
    // shared memory: stages | staging tile | barriers | flags
    const uint32_t smem0 = smem_u32(smem_raw);
    float *s_out = reinterpret_cast<float *>(smem_raw + (size_t)NS * p.stage_stride);
    const uint32_t bars = smem0 + (uint32_t)NS * p.stage_stride + C::OUT_BYTES;
    volatile int *s_flags = reinterpret_cast<volatile int *>(smem_raw + (size_t)NS * p.stage_stride + C::OUT_BYTES + 16 * NS);
    volatile int *s_abort = s_flags;        // [0] a bounded wait ran out somewhere in the CTA
    volatile int *s_ticket = s_flags + 1;   // [1] ticket drawn for the row tile being finished
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (NS + s); };
    const uint32_t w_off = 0, sc_off = SK_TILE_BYTES, x_off = SK_TILE_BYTES + (uint32_t)p.scale_cap;

    const long long u0 = unit_begin(p.units, grid, cta), u1 = unit_begin(p.units, grid, cta + 1);
    const int n_units = (int)(u1 - u0);
    const int r0 = (int)(u0 / p.k_tiles), kt0 = (int)(u0 - (long long)r0 * p.k_tiles);

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar(s), 2);                 // the code producer (with its bytes) + one activation producer
            mbar_init(empty_bar(s), SK_CONSUMERS);
        }
        s_flags[0] = 0;
        s_flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // batch rows that do not exist stay zero in every stage's activation tile
    for (int i = tid; i < NS * (C::X_BYTES / 16); i += C::THREADS) {
        const int s = i / (C::X_BYTES / 16), c = i - s * (C::X_BYTES / 16);
        *reinterpret_cast<uint4 *>(smem_raw + (size_t)s * p.stage_stride + x_off + c * 16) = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();

    if (warp == 0) {
        // ------------------------------ code producer (weights only: runs before the dependency wait) ----------
        if (lane == 0) {
            int r = r0, kt = kt0;
            for (int i = 0; i < n_units; ++i) {
                const int s = i % NS;
                if (i >= NS && !mbar_wait(empty_bar(s), (uint32_t)((i / NS - 1) & 1), s_abort)) { *s_abort = 1; break; }
                const int first_blk = (kt * 64) / p.bs, last_blk = (kt * 64 + 63) / p.bs;
                const uint32_t sc_bytes = (uint32_t)(last_blk - first_blk + 1) * 256u;
                const uint32_t dst = smem0 + (uint32_t)s * p.stage_stride;
                mbar_arrive_expect_tx(full_bar(s), SK_TILE_BYTES + sc_bytes);
                bulk_load(dst + w_off, p.tiles + ((size_t)r * p.k_tiles + kt) * SK_TILE_BYTES, SK_TILE_BYTES, full_bar(s));
                bulk_load(dst + sc_off, p.scales_t + ((size_t)r * p.blocks_per_row + first_blk) * 128, sc_bytes, full_bar(s));
                if (++kt == p.k_tiles) { kt = 0; ++r; }
            }
        }
    } else if (warp < C::FIRST_CONSUMER) {
        // ------------------------------ activation producers ------------------------------
        const int which = warp - 1;
        const bool bf16 = p.dtype == ATLAS_DTYPE_BF16;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // x comes from the earlier kernels of the stream
        const uint16_t *xg = reinterpret_cast<const uint16_t *>(p.x);
        int kt = kt0;
        bool alive = true;
        const bool gathered_x = p.wait_flags != nullptr;
        if (gathered_x) {
            // x is a gathered buffer the other ranks' kernels store into: wait until every rank has finished as many
            // gather launches as this rank (the count is final: this rank's previous kernel has completed)
            const unsigned int target = *reinterpret_cast<volatile unsigned int *>(p.state + 1);
            if (!wait_arrivals(p.wait_flags, p.wait_world, target, p.poll_limit, lane)) {
                alive = false;
                *s_abort = 1;
            }
        }
        for (int i = 0; i < n_units; ++i) {
            if (i % C::XP_WARPS == which) {
                const int s = i % NS;
                if (alive && i >= NS && !mbar_wait(empty_bar(s), (uint32_t)((i / NS - 1) & 1), s_abort)) {
                    alive = false;
                    *s_abort = 1;
                }
                unsigned char *xs = smem_raw + (size_t)s * p.stage_stride + x_off;
                // 16-byte chunk ch of row rr goes to position ch ^ (rr & 1): the consumers' paired reads of two rows
                // then fall on different banks
                for (int idx = lane; idx < p.m * 8; idx += 32) {
                    const int rr = idx >> 3, ch = idx & 7;
                    const uint16_t *src = xg + (size_t)rr * p.ldx + kt * 64 + ch * 8;
                    uint4 v;
                    if (p.x_vec_ok) {
                        // data stored by peers during this kernel's life must not come through the non-coherent path
                        v = gathered_x ? __ldcg(reinterpret_cast<const uint4 *>(src)) : __ldg(reinterpret_cast<const uint4 *>(src));
                    } else if (gathered_x) {
                        const volatile uint16_t *vs = src;
                        v.x = vs[0] | (uint32_t)vs[1] << 16;
                        v.y = vs[2] | (uint32_t)vs[3] << 16;
                        v.z = vs[4] | (uint32_t)vs[5] << 16;
                        v.w = vs[6] | (uint32_t)vs[7] << 16;
                    } else {
                        v.x = src[0] | (uint32_t)src[1] << 16;
                        v.y = src[2] | (uint32_t)src[3] << 16;
                        v.z = src[4] | (uint32_t)src[5] << 16;
                        v.w = src[6] | (uint32_t)src[7] << 16;
                    }
                    if (bf16) {
                        v.x = bf16x2_to_f16x2(v.x);
                        v.y = bf16x2_to_f16x2(v.y);
                        v.z = bf16x2_to_f16x2(v.z);
                        v.w = bf16x2_to_f16x2(v.w);
                    }
                    *reinterpret_cast<uint4 *>(xs + rr * 128 + ((ch ^ (rr & 1)) << 4)) = v;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar(s));
            }
            if (++kt == p.k_tiles) kt = 0;
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int w = warp - C::FIRST_CONSUMER;          // strip of the row tile
        const int ct = tid - C::FIRST_CONSUMER * 32;     // 0..255
        const int g = lane >> 2, tig = lane & 3;
        const bool bf16 = p.dtype == ATLAS_DTYPE_BF16;
        const bool gathered_x = p.wait_flags != nullptr;
        const uint16_t *xg = reinterpret_cast<const uint16_t *>(p.x);

        // outlier list of the first segment: weights only, requested before the dependency wait
        auto seg_end_kt = [&](int kt_begin, int left) { return min(p.k_tiles, kt_begin + left); };
        int e_cur = 0, e_end = 0, win_base = 0;
        uint32_t cur_ent = 0xff000000u, nxt_ent = 0xff000000u, cur_val = 0, nxt_val = 0;
        auto load_window = [&](int base, uint32_t &ent, uint32_t &val) {
            ent = 0xff000000u;
            val = 0;
            if (base + lane < e_end) { ent = __ldg(p.entries + base + lane); val = __ldg(p.ovals + base + lane); }
        };
        auto start_outliers = [&](int ea, int eb) {
            e_cur = ea;
            e_end = eb;
            win_base = ea;
            load_window(ea, cur_ent, cur_val);
            load_window(ea + 32, nxt_ent, nxt_val);
        };
        {
            const int32_t *cp = p.chunk_ptr + ((size_t)r0 * 8 + w) * (p.k_tiles + 1);
            start_outliers(__ldg(cp + kt0), __ldg(cp + seg_end_kt(kt0, n_units)));
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");   // x, y and the workspace belong to the stream from here on

        float acc[MT][4];
        uint32_t og_rv[4];          // pending outlier group: row << 16 | fp16 value per K slot of this lane
        uint32_t og_x[MT][4];       //   and the activations gathered for it (raw 16-bit patterns)
        bool og_pending = false;
        auto outlier_gather = [&]() {     // entries e_cur .. e_cur + 15: fetch their activations
            const int off = e_cur - win_base;   // 0 or 16
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int slot = 2 * tig + (q & 1) + (q >> 1) * 8;
                const uint32_t ent = __shfl_sync(0xffffffffu, cur_ent, off + slot);
                const uint32_t val = __shfl_sync(0xffffffffu, cur_val, off + slot);
                og_rv[q] = (ent >> 24) << 16 | val;     // row 255 (no entry) matches no lane
                const uint32_t col = ent & 0xffffffu;   // 0 for missing entries: stays in range
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    const int mm = nt * 8 + g;
                    const uint16_t *xp = xg + (size_t)(mm < p.m ? mm : 0) * p.ldx + col;
                    og_x[nt][q] = gathered_x ? (uint32_t)__ldcg(xp) : (uint32_t)__ldg(xp);
                }
            }
            og_pending = true;
            e_cur += 16;
            if (e_cur - win_base == 32) {
                cur_ent = nxt_ent;
                cur_val = nxt_val;
                win_base += 32;
                load_window(win_base + 32, nxt_ent, nxt_val);
            }
        };
        auto outlier_mma = [&]() {
            uint32_t rws[4], vals[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) { rws[q] = og_rv[q] >> 16; vals[q] = og_rv[q] & 0xffffu; }
            const uint32_t ug = (uint32_t)g;
            const uint32_t a0 = (rws[0] == ug ? vals[0] : 0u) | (rws[1] == ug ? vals[1] : 0u) << 16;
            const uint32_t a1 = (rws[0] == ug + 8 ? vals[0] : 0u) | (rws[1] == ug + 8 ? vals[1] : 0u) << 16;
            const uint32_t a2 = (rws[2] == ug ? vals[2] : 0u) | (rws[3] == ug ? vals[3] : 0u) << 16;
            const uint32_t a3 = (rws[2] == ug + 8 ? vals[2] : 0u) | (rws[3] == ug + 8 ? vals[3] : 0u) << 16;
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                uint32_t b0 = og_x[nt][0] | og_x[nt][1] << 16, b1 = og_x[nt][2] | og_x[nt][3] << 16;
                if (bf16) { b0 = bf16x2_to_f16x2(b0); b1 = bf16x2_to_f16x2(b1); }
                mma_f16(acc[nt], a0, a1, a2, a3, b0, b1);
            }
            og_pending = false;
        };

        bool alive = true;
        int r = r0, kt = kt0, left = n_units, i = 0, seg = 0;
        while (left > 0) {
            const int ka = kt, kb = seg_end_kt(kt, left);
            // the next segment's outlier range (its row tile starts at column 0): requested now, used when it starts
            int nxt_ea = 0, nxt_eb = 0;
            if (left > kb - ka) {
                const int32_t *cp = p.chunk_ptr + ((size_t)(r + 1) * 8 + w) * (p.k_tiles + 1);
                nxt_ea = __ldg(cp);
                nxt_eb = __ldg(cp + seg_end_kt(0, left - (kb - ka)));
            }
#pragma unroll
            for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[nt][j] = 0.f;
            // a segment that is not the first waits a few steps for its entry windows before touching them
            int o_hold = seg == 0 ? 0 : 4;

            for (; kt < kb; ++kt, ++i) {
                const int s = i % NS;
                bool got = !alive || mbar_wait(full_bar(s), (uint32_t)((i / NS) & 1), s_abort);
                // the first stage also stands for the activation producer's wait for the other ranks
                for (int extra = 0; !got && gathered_x && i == 0 && extra < 64 && !*s_abort; ++extra)
                    got = mbar_wait(full_bar(s), 0u, s_abort);
                if (!got) {
                    alive = false;
                    *s_abort = 1;
                }
                const unsigned char *stg = smem_raw + (size_t)s * p.stage_stride;
                const uint4 wa = *reinterpret_cast<const uint4 *>(stg + w_off + w * 1024 + lane * 16);          // row g of the strip
                const uint4 wb = *reinterpret_cast<const uint4 *>(stg + w_off + w * 1024 + 512 + lane * 16);    // row g + 8
                const int col = kt * 64 + tig * 16;
                const int kbl = (p.bs_shift >= 0 ? (col >> p.bs_shift) - ((kt * 64) >> p.bs_shift)
                                                 : col / p.bs - (kt * 64) / p.bs);
                const uint16_t *scs = reinterpret_cast<const uint16_t *>(stg + sc_off) + kbl * 128 + w * 16 + g;
                const __half2 sa2 = __half2half2(__ushort_as_half(scs[0]));
                const __half2 sb2 = __half2half2(__ushort_as_half(scs[8]));
                const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w};
                const uint32_t wbv[4] = {wb.x, wb.y, wb.z, wb.w};
                uint32_t a_lo[4], a_hi[4], b_lo[4], b_hi[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    dequant4(wav[q], sa2, a_lo[q], a_hi[q]);
                    dequant4(wbv[q], sb2, b_lo[q], b_hi[q]);
                }
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    const unsigned char *xr = stg + x_off + (nt * 8 + g) * 128;
                    const uint4 x0 = *reinterpret_cast<const uint4 *>(xr + (((2 * tig) ^ (g & 1)) << 4));
                    const uint4 x1 = *reinterpret_cast<const uint4 *>(xr + (((2 * tig + 1) ^ (g & 1)) << 4));
                    if (nt == MT - 1) {
                        // everything this warp needs from the stage is in registers: hand it back
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty_bar(s));
                    }
                    const uint32_t xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        mma_f16(acc[nt], a_lo[q], b_lo[q], a_hi[q], b_hi[q], xv[2 * q], xv[2 * q + 1]);
                }
                // outliers ride along: on odd steps the next 16 entries' activations are requested, on even steps the
                // group requested a step ago becomes one more MMA (an entry window of 32 then lasts four steps, about
                // the latency of the load that refills it)
                if (o_hold > 0) {
                    --o_hold;
                } else if (i & 1) {
                    if (!og_pending && e_cur < e_end) outlier_gather();
                } else if (og_pending) {
                    outlier_mma();
                }
            }
            while (og_pending || e_cur < e_end) {   // what the dense steps did not cover
                if (og_pending) outlier_mma();
                if (e_cur < e_end) outlier_gather();
            }

            // ---- the strip's sums go to the CTA's staging tile [row][batch column] ----------------------
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                *reinterpret_cast<float2 *>(s_out + (w * 16 + g) * C::OUT_LD + nt * 8 + 2 * tig) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2 *>(s_out + (w * 16 + g + 8) * C::OUT_LD + nt * 8 + 2 * tig) = make_float2(acc[nt][2], acc[nt][3]);
            }
            consumer_bar();
            const int n_base = r * 128;
            auto store_y = [&](int mm, int row, float v) {
                const int n = n_base + row;
                if (n >= p.n_rows) return;
                if (p.bias) v += __half2float(__ushort_as_half(__ldg(p.bias + n)));
                const uint16_t bits = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
                const size_t at = (size_t)mm * p.ldy + n;
                if (p.world <= 1) {
                    reinterpret_cast<uint16_t *>(p.y)[at] = bits;
                } else {
                    // plain stores into every rank's gathered buffer (the local one included), own rank first
                    for (int d = 0; d < p.world; ++d) {
                        const int dst = (p.rank + d) % p.world;
                        reinterpret_cast<uint16_t *>(p.y_dst[dst])[at] = bits;
                    }
                }
            };
            if (ka == 0 && kb == p.k_tiles) {
                // the whole K range of this row tile was ours
                for (int idx = ct; idx < p.m * 128; idx += SK_CONSUMERS * 32) {
                    const int mm = idx >> 7, row = idx & 127;
                    store_y(mm, row, s_out[row * C::OUT_LD + mm]);
                }
            } else {
                // shared row tile: publish the partial tile [m][128], draw a ticket, the last one adds them all up
                const long long t_lo = (long long)r * p.k_tiles, t_hi = t_lo + p.k_tiles;   // the row tile's units
                int c_lo = (int)(t_lo * grid / p.units), c_hi = (int)((t_hi - 1) * grid / p.units);
                while (c_lo > 0 && unit_begin(p.units, grid, c_lo) > t_lo) --c_lo;
                while (unit_begin(p.units, grid, c_lo + 1) <= t_lo) ++c_lo;
                while (c_hi + 1 < grid && unit_begin(p.units, grid, c_hi + 1) < t_hi) ++c_hi;
                while (unit_begin(p.units, grid, c_hi) >= t_hi) --c_hi;
                const size_t slot_floats = (size_t)p.m * 128;
                float *mine = p.partials + ((size_t)cta * 2 + (seg == 0 ? 0 : 1)) * slot_floats;
                for (int idx = ct; idx < p.m * 128; idx += SK_CONSUMERS * 32) {
                    const int mm = idx >> 7, row = idx & 127;
                    __stcg(mine + idx, s_out[row * C::OUT_LD + mm]);
                }
                __threadfence();
                consumer_bar();
                if (ct == 0) {
                    const unsigned int t = atomicAdd(p.tickets + r, 1u);
                    __threadfence();
                    *s_ticket = (int)t;
                }
                consumer_bar();
                if (*s_ticket == c_hi - c_lo) {
                    for (int idx = ct; idx < p.m * 128; idx += SK_CONSUMERS * 32) {
                        float sum = 0.f;
                        for (int cc = c_lo; cc <= c_hi; ++cc) {
                            // a CTA's first segment uses its slot 0, its last one slot 1
                            const int first_tile_row = (int)(unit_begin(p.units, grid, cc) / p.k_tiles);
                            const float *theirs = p.partials + ((size_t)cc * 2 + (first_tile_row == r ? 0 : 1)) * slot_floats;
                            sum += __ldcg(theirs + idx);
                        }
                        store_y(idx >> 7, idx & 127, sum);
                    }
                    if (ct == 0) p.tickets[r] = 0;   // left as found for the next launch
                }
            }
            consumer_bar();   // the staging tile is free again

            left -= kb - ka;
            kt = 0;
            ++r;
            ++seg;
            if (left > 0) start_outliers(nxt_ea, nxt_eb);
        }
    }

    if (p.world > 1) __threadfence_system();   // this thread's stores into the other ranks' buffers are out
    __syncthreads();
    if (p.world > 1 && tid == 0) {
        // the CTA that finishes last tells every rank that this rank's shard of the output is complete
        __threadfence_system();
        const unsigned int finished = atomicAdd(p.state, 1u);
        if (finished == (unsigned int)grid - 1) {
            __threadfence_system();
            const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(p.state + 1) + 1u;
            p.state[0] = 0;
            p.state[1] = seq;
            for (int d = 0; d < p.world; ++d) st_release_sys(p.flags_dst[(p.rank + d) % p.world] + p.rank, seq);
        }
    }
    if (*s_abort) {
        // a wait ran out: bulk copies may still be in flight towards this CTA's shared memory; give them time to land
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        if (tid == 0 && p.status) atomicExch(p.status, 1);
    }
}

int stream_sm_count() {
    static thread_local int dev_cached = -1, sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != dev_cached) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
        dev_cached = dev;
    }
    return sms;
}

template <int MT>
int launch_stream(const StreamParams &p, int grid, size_t smem, cudaStream_t st) {
    auto kern = qlinear_stream_kernel<MT>;
    static thread_local size_t configured = 0;
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != configured_dev) { configured = 0; configured_dev = dev; }
    if (smem > configured) {
        int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                            "cudaFuncSetAttribute(stream smem)");
        if (rc) return rc;
        configured = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(StreamCfg<MT>::THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kern, p), "qlinear_stream_kernel launch");
}

int mt_for(int64_t m) { return m <= 8 ? 1 : (m <= 16 ? 2 : 4); }

}  // namespace
}  // namespace atlas

extern "C" size_t atlas_qlinear_stream_workspace_bytes(int64_t m) {
    const int64_t rows = m <= 0 ? 1 : (m > 32 ? 32 : m);
    return atlas::SK_TICKET_BYTES + (size_t)atlas::SK_MAX_GRID * 2 * (size_t)rows * 128 * 4;
}

namespace atlas {
namespace {
int stream_entry(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles, const void *scales_tiled,
                 const int32_t *outlier_chunk_ptr, const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                 int64_t n_rows, int64_t n_cols, int block_size, const void *bias, void *y, int64_t ldy,
                 void *workspace, size_t workspace_bytes, int32_t *status, void *stream, const AtlasPeerGather *gather) {
    clear_error();
    ATLAS_RETURN_IF(!x || !tiles || !scales_tiled || !outlier_chunk_ptr || (!y && !gather) || !workspace,
                    ATLAS_ERR_BAD_ARGUMENT, "atlas_qlinear_stream: null buffer");
    if (gather) {
        ATLAS_RETURN_IF(gather->world < 1 || gather->world > ATLAS_MAX_PEERS || gather->rank < 0 ||
                            gather->rank >= gather->world || !gather->state || gather->poll_limit < 1,
                        ATLAS_ERR_BAD_ARGUMENT, "atlas_qlinear_stream_gather: bad world / rank / state / poll_limit");
        ATLAS_RETURN_IF(m > 32, ATLAS_ERR_UNSUPPORTED, "atlas_qlinear_stream_gather: at most 32 rows of x per call");
        for (int d = 0; d < gather->world; ++d)
            ATLAS_RETURN_IF(!gather->y_dst[d] || !gather->flags_dst[d], ATLAS_ERR_BAD_ARGUMENT,
                            "atlas_qlinear_stream_gather: null destination for rank %d", d);
    }
    ATLAS_RETURN_IF(m < 0 || n_rows <= 0 || n_cols <= 0 || ldx < n_cols || ldy < n_rows, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_stream: bad size (m=%lld n_rows=%lld n_cols=%lld ldx=%lld ldy=%lld)",
                    (long long)m, (long long)n_rows, (long long)n_cols, (long long)ldx, (long long)ldy);
    ATLAS_RETURN_IF(dtype != ATLAS_DTYPE_F16 && dtype != ATLAS_DTYPE_BF16, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_stream: dtype %d", dtype);
    ATLAS_RETURN_IF(n_cols % 64 != 0 || block_size < 16 || block_size % 16 != 0 || n_cols % block_size != 0,
                    ATLAS_ERR_UNSUPPORTED,
                    "atlas_qlinear_stream: needs n_cols %% 64 == 0 and block_size a multiple of 16 dividing n_cols");
    ATLAS_RETURN_IF(n_rows > (int64_t)SK_MAX_TILE_ROWS * 128 || n_cols >= (1 << 24), ATLAS_ERR_UNSUPPORTED,
                    "atlas_qlinear_stream: too large");
    ATLAS_RETURN_IF(((uintptr_t)tiles & 15) != 0 || ((uintptr_t)scales_tiled & 15) != 0 || ((uintptr_t)workspace & 15) != 0,
                    ATLAS_ERR_BAD_ARGUMENT, "atlas_qlinear_stream: tiles, scales_tiled and workspace must be 16-byte aligned");
    const size_t need = atlas_qlinear_stream_workspace_bytes(m);
    ATLAS_RETURN_IF(workspace_bytes < need, ATLAS_ERR_CAPACITY,
                    "atlas_qlinear_stream: workspace holds %zu bytes, %zu needed", workspace_bytes, need);
    int rc = check_device();
    if (rc) return rc;
    if (m == 0) return ATLAS_OK;
    cudaStream_t st = (cudaStream_t)stream;

    StreamParams p;
    p.dtype = dtype;
    p.ldx = ldx;
    p.tiles = tiles;
    p.scales_t = (const uint16_t *)scales_tiled;
    p.chunk_ptr = outlier_chunk_ptr;
    p.entries = outlier_entries;
    p.ovals = (const uint16_t *)outlier_vals_sorted;
    p.bias = (const uint16_t *)bias;
    p.ldy = ldy;
    p.n_rows = (int)n_rows;
    p.n_cols = (int)n_cols;
    p.bs = block_size;
    p.bs_shift = (block_size & (block_size - 1)) == 0 ? __builtin_ctz((unsigned)block_size) : -1;
    p.k_tiles = (int)(n_cols / 64);
    p.blocks_per_row = (int)(n_cols / block_size);
    p.tile_rows = (int)ceil_div_i64(n_rows, 128);
    p.units = (long long)p.tile_rows * p.k_tiles;
    // scale blocks a 64-column tile can touch: one when blocks are whole tiles, 64 / bs when they divide a tile
    const int max_blk = block_size % 64 == 0 ? 1 : (64 % block_size == 0 ? 64 / block_size : 64 / block_size + 2);
    p.scale_cap = max_blk * 256;
    p.x_vec_ok = (((uintptr_t)x & 15) == 0) && (ldx % 8 == 0);
    p.tickets = (unsigned int *)workspace;
    p.partials = (float *)((char *)workspace + SK_TICKET_BYTES);
    p.status = status;
    p.world = 0;
    p.rank = 0;
    p.wait_world = 0;
    p.state = nullptr;
    p.wait_flags = nullptr;
    p.poll_limit = 0;
    for (int d = 0; d < ATLAS_MAX_PEERS; ++d) { p.y_dst[d] = nullptr; p.flags_dst[d] = nullptr; }
    if (gather) {
        // world == 1 still goes through the peer path (stores to y_dst[0], arrival flag), so that one GPU exercises it
        p.world = gather->world == 1 ? 2 : gather->world;
        p.rank = gather->rank;
        p.wait_world = gather->world;
        for (int d = 0; d < gather->world; ++d) { p.y_dst[d] = gather->y_dst[d]; p.flags_dst[d] = gather->flags_dst[d]; }
        if (gather->world == 1) { p.y_dst[1] = gather->y_dst[0]; p.flags_dst[1] = gather->flags_dst[0]; }
        p.state = gather->state;
        p.wait_flags = gather->wait_flags;
        p.poll_limit = gather->poll_limit;
    }
    const int sms = stream_sm_count();
    int grid = sms < SK_MAX_GRID ? sms : SK_MAX_GRID;
    if ((long long)grid > p.units) grid = (int)p.units;

    for (int64_t m0 = 0; m0 < m; m0 += 32) {   // more than 32 rows: one pass over the weight per 32
        const int mg = (int)((m - m0) < 32 ? (m - m0) : 32);
        const int mt = mt_for(mg);
        p.m = mg;
        p.x = (const char *)x + (size_t)m0 * ldx * 2;
        p.y = (char *)y + (size_t)m0 * ldy * 2;
        const int x_bytes = mt * 8 * 128, out_bytes = 128 * mt * 8 * 4;
        p.stage_stride = (SK_TILE_BYTES + p.scale_cap + x_bytes + 127) & ~127;
        int ns = (SK_SMEM_BUDGET - out_bytes - 64) / (p.stage_stride + 16);
        if (ns > 16) ns = 16;
        ATLAS_RETURN_IF(ns < 2, ATLAS_ERR_UNSUPPORTED, "atlas_qlinear_stream: stage of %d bytes does not fit", p.stage_stride);
        p.n_stages = ns;
        const size_t smem = (size_t)ns * p.stage_stride + out_bytes + 16 * ns + 64;
        if (mt == 1) rc = launch_stream<1>(p, grid, smem, st);
        else if (mt == 2) rc = launch_stream<2>(p, grid, smem, st);
        else rc = launch_stream<4>(p, grid, smem, st);
        if (rc) return rc;
    }
    return ATLAS_OK;
}
}  // namespace
}  // namespace atlas

extern "C" int atlas_qlinear_stream(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                    const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                    const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                    int64_t n_rows, int64_t n_cols, int block_size, const void *bias, void *y,
                                    int64_t ldy, void *workspace, size_t workspace_bytes, int32_t *status,
                                    void *stream) {
    return atlas::stream_entry(x, dtype, m, ldx, tiles, scales_tiled, outlier_chunk_ptr, outlier_entries,
                               outlier_vals_sorted, n_rows, n_cols, block_size, bias, y, ldy, workspace, workspace_bytes,
                               status, stream, nullptr);
}

extern "C" int atlas_qlinear_stream_gather(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                           const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                           const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                           int64_t n_rows, int64_t n_cols, int block_size, const void *bias,
                                           int64_t ldy, void *workspace, size_t workspace_bytes, int32_t *status,
                                           void *stream, const AtlasPeerGather *gather) {
    if (!gather) {
        atlas::clear_error();
        atlas::set_error("atlas_qlinear_stream_gather: null gather descriptor");
        return ATLAS_ERR_BAD_ARGUMENT;
    }
    return atlas::stream_entry(x, dtype, m, ldx, tiles, scales_tiled, outlier_chunk_ptr, outlier_entries,
                               outlier_vals_sorted, n_rows, n_cols, block_size, bias, nullptr, ldy, workspace,
                               workspace_bytes, status, stream, gather);
}
