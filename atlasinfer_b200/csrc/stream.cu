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
// rows.  A strip's outliers (sorted by column at repack time) inside the columns
// of a ring stage are taken 16 at a time as one more MMA per stage, with their
// activations read from the stage in shared memory.
//
// Every wait is bounded; when one runs out the CTA sets the caller's status
// word, stops waiting and runs to its end on whatever data it has.
#include <cuda_bf16.h>

#include <cstdlib>

#include "common.cuh"

namespace atlas {
namespace {

constexpr int SK_CONSUMERS = 8;            // consumer warps = 16-row strips of a 128-row tile
constexpr int SK_TILE_BYTES = 8192;        // 128 rows x 64 codes
constexpr int SK_SKT = 2;                  // 64-column tiles per code stage (16 KB: what a warp can take to registers at once)
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
    int skt;             // 64-column tiles per ring stage (a stage never crosses a row tile)
    int scale_cap;       // bytes reserved for scales in a stage (multiple of 256)
    int x_row_bytes;     // skt * 128 + 16: stride of a batch row's activations in an activation stage
    int stage_stride;    // bytes per code stage (codes + scales)
    int n_stages;        // code stages
    int x_stride;        // bytes per activation stage (m rows)
    int x_stages;        // activation stages (a deeper ring than the codes': x cannot be requested before the wait)
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

// Four biased codes -> two half2 of the integer codes themselves (exact in fp16).
__device__ __forceinline__ void codes4(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t l = __byte_perm(w, 0x64646464u, 0x5140);
    const uint32_t h = __byte_perm(w, 0x64646464u, 0x5342);
    const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));  // 1152
    const __half2 lv = __hsub2(*reinterpret_cast<const __half2 *>(&l), bias);
    const __half2 hv = __hsub2(*reinterpret_cast<const __half2 *>(&h), bias);
    lo = *reinterpret_cast<const uint32_t *>(&lv);
    hi = *reinterpret_cast<const uint32_t *>(&hv);
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
    static constexpr int FIRST_CONSUMER = 2;                               // warp 0: codes, warp 1: activations
    static constexpr int THREADS = (FIRST_CONSUMER + SK_CONSUMERS) * 32;
    static constexpr int OUT_LD = MT * 8;                                  // floats per row of the staging tile
    static constexpr int OUT_BYTES = 128 * OUT_LD * 4;
};

// The CTA's units [u0, u1) cut into ring stages: runs of up to `skt` consecutive 64-column tiles of one row tile.
// Every role walks the same sequence.
struct StageWalk {
    int r, kt, left, k_tiles, skt;
    __device__ StageWalk(long long u0, int n_units, int k_tiles_, int skt_) : left(n_units), k_tiles(k_tiles_), skt(skt_) {
        r = (int)(u0 / k_tiles_);
        kt = (int)(u0 - (long long)r * k_tiles_);
    }
    // next stage: row tile, first tile column, tiles in the stage; false when the range is exhausted
    __device__ bool next(int &sr, int &skt0, int &snk) {
        if (left <= 0) return false;
        sr = r;
        skt0 = kt;
        snk = min(skt, min(k_tiles - kt, left));
        kt += snk;
        left -= snk;
        if (kt == k_tiles) { kt = 0; ++r; }
        return true;
    }
};

// POST: the MMAs take the integer codes themselves and a block's sum is multiplied by its scale afterwards (fp32),
// which needs blocks that are whole 64-column tiles; otherwise every code is turned into the reference's fp16 weight
// fp16(fp16(code) * scale) first.  Both are well inside the 1e-2 * rms tolerance of the linear's output; POST saves a
// third of the dequantisation instructions and is the more accurate of the two (one rounding per block and row
// instead of one per weight).
template <int MT, bool POST>
__global__ void __launch_bounds__(StreamCfg<MT>::THREADS, 2) qlinear_stream_kernel(StreamParams p) {
    using C = StreamCfg<MT>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // let the next kernel of the stream become resident and start its own weight prefetch
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int NS = p.n_stages;
    // shared memory: code stages | activation stages | zero row | staging tile | barriers | flags
    const int XS = p.x_stages;
    const uint32_t smem0 = smem_u32(smem_raw);
    unsigned char *x_ring = smem_raw + (size_t)NS * p.stage_stride;
    unsigned char *zero_row = x_ring + (size_t)XS * p.x_stride;
    float *s_out = reinterpret_cast<float *>(zero_row + p.x_row_bytes);
    unsigned char *bar_base = reinterpret_cast<unsigned char *>(s_out) + C::OUT_BYTES;
    const uint32_t bars = smem_u32(bar_base);
    volatile int *s_flags = reinterpret_cast<volatile int *>(bar_base + 16 * NS + 24 * XS);
    volatile int *s_abort = s_flags;        // [0] a bounded wait ran out somewhere in the CTA
    volatile int *s_ticket = s_flags + 1;   // [1] ticket drawn for the row tile being finished
    auto full_bar = [&](int s) { return bars + 8u * s; };                       // codes and scales of a stage have landed
    auto empty_bar = [&](int s) { return bars + 8u * (NS + s); };
    auto xraw_bar = [&](int s) { return bars + 8u * (2 * NS + s); };            // activation bytes have landed
    auto xfull_bar = [&](int s) { return bars + 8u * (2 * NS + XS + s); };      // ... and are fp16
    auto xempty_bar = [&](int s) { return bars + 8u * (2 * NS + 2 * XS + s); };
    const uint32_t sc_off = (uint32_t)p.skt * SK_TILE_BYTES;

    const long long u0 = unit_begin(p.units, grid, cta), u1 = unit_begin(p.units, grid, cta + 1);
    const int n_units = (int)(u1 - u0);
    const int r0 = (int)(u0 / p.k_tiles), kt0 = (int)(u0 - (long long)r0 * p.k_tiles);

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), SK_CONSUMERS);
        }
        for (int s = 0; s < XS; ++s) {
            mbar_init(xraw_bar(s), 1);
            mbar_init(xfull_bar(s), 1);
            mbar_init(xempty_bar(s), SK_CONSUMERS);
        }
        s_flags[0] = 0;
        s_flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // batch rows that do not exist read this row of zeros
    for (int i = tid; i < p.x_row_bytes / 16; i += C::THREADS) reinterpret_cast<uint4 *>(zero_row)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();

    if (warp == 0) {
        // ------------------------------ code producer (weights only: runs before the dependency wait) ----------
        // Lane s owns ring stage s.  A stage is one bulk copy of up to skt adjacent 8 KB tiles (they are contiguous in
        // the tile-major layout) plus one of their scales: what limits a ring is the number of stage hand-overs per
        // microsecond, not the bytes, so stages are made as large as the shared-memory budget allows.
        if (lane < NS) {
            StageWalk walk(u0, n_units, p.k_tiles, p.skt);
            int sr, skt0, snk;
            for (int i = 0; walk.next(sr, skt0, snk); ++i) {
                if (i % NS != lane) continue;
                if (i >= NS && !mbar_wait(empty_bar(lane), (uint32_t)((i / NS - 1) & 1), s_abort)) { *s_abort = 1; break; }
                const int first_blk = (skt0 * 64) / p.bs, last_blk = ((skt0 + snk) * 64 - 1) / p.bs;
                const uint32_t w_bytes = (uint32_t)snk * SK_TILE_BYTES, sc_bytes = (uint32_t)(last_blk - first_blk + 1) * 256u;
                const uint32_t dst = smem0 + (uint32_t)lane * p.stage_stride;
                mbar_arrive_expect_tx(full_bar(lane), w_bytes + sc_bytes);
                bulk_load(dst, p.tiles + ((size_t)sr * p.k_tiles + skt0) * SK_TILE_BYTES, w_bytes, full_bar(lane));
                bulk_load(dst + sc_off, p.scales_t + ((size_t)sr * p.blocks_per_row + first_blk) * 128, sc_bytes, full_bar(lane));
            }
        }
    } else if (warp == 1) {
        // ------------------------------ activation producer ------------------------------
        const bool bf16 = p.dtype == ATLAS_DTYPE_BF16;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // x comes from the earlier kernels of the stream
        const uint16_t *xg = reinterpret_cast<const uint16_t *>(p.x);
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
        // An activation stage holds, per batch row, the 64 * snk columns of a code stage as one run (rows
        // x_row_bytes apart: 16 bytes of padding keep the consumers' paired reads of two rows on different banks).
        // The ring is deeper than the codes' and is filled by one bulk copy per batch row, XS - 1 stages ahead, so
        // that the latency of x is paid once after the dependency wait; bf16 is converted in place once landed.
        StageWalk ahead(u0, n_units, p.k_tiles, p.skt), done(u0, n_units, p.k_tiles, p.skt);
        int issued = 0;
        // Requests the activations of up to `count` further stages.  Issuing a bulk copy occupies a thread for
        // hundreds of cycles, so the (stage, batch row) copies are spread over the lanes.
        auto issue = [&](int count) {
            int sr[12], skt0[12], snk[12], n = 0;
#pragma unroll
            for (int c = 0; c < 12; ++c)
                if (c < count && ahead.next(sr[n], skt0[n], snk[n])) ++n;
            if (n == 0) return;
            // stage `issued + c` must have been handed back by the consumers; then announce its bytes
            for (int c = 0; c < n; ++c) {
                const int st = issued + c, s = st % XS;
                if (alive && st >= XS && !mbar_wait(xempty_bar(s), (uint32_t)((st / XS - 1) & 1), s_abort)) {
                    alive = false;
                    *s_abort = 1;
                }
            }
            if (p.x_vec_ok) {
                if (lane < n) mbar_arrive_expect_tx(xraw_bar((issued + lane) % XS), (uint32_t)(p.m * snk[lane] * 128));
                __syncwarp();
                for (int pr = lane; pr < n * p.m; pr += 32) {
                    const int c = pr / p.m, rr = pr - c * p.m, s = (issued + c) % XS;
                    bulk_load(smem_u32(x_ring + (size_t)s * p.x_stride + rr * p.x_row_bytes),
                              xg + (size_t)rr * p.ldx + skt0[c] * 64, (uint32_t)snk[c] * 128u, xraw_bar(s));
                }
            } else {
                // rows of x that do not allow 16-byte accesses: plain 2-byte loads, published like a landed copy
                for (int c = 0; c < n; ++c) {
                    unsigned char *xs = x_ring + (size_t)((issued + c) % XS) * p.x_stride;
                    for (int idx = lane; idx < p.m * snk[c] * 32; idx += 32) {
                        const int rr = idx / (snk[c] * 32), c2 = idx - rr * (snk[c] * 32);
                        const volatile uint16_t *src = xg + (size_t)rr * p.ldx + skt0[c] * 64 + c2 * 2;
                        *reinterpret_cast<uint32_t *>(xs + rr * p.x_row_bytes + c2 * 4) = src[0] | (uint32_t)src[1] << 16;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(xraw_bar((issued + c) % XS));
                }
            }
            issued += n;
        };
        issue(XS - 1);   // everything the ring holds but one stage, at once
        int sr, skt0, snk;
        for (int i = 0; done.next(sr, skt0, snk); ++i) {
            const int s = i % XS;
            if (alive && !mbar_wait(xraw_bar(s), (uint32_t)((i / XS) & 1), s_abort)) {
                alive = false;
                *s_abort = 1;
            }
            if (bf16) {
                unsigned char *xs = x_ring + (size_t)s * p.x_stride;
                const int per_row = snk * 8;   // 16-byte pieces per batch row
                for (int idx = lane; idx < p.m * per_row; idx += 32) {
                    const int rr = idx / per_row, pc = idx - rr * per_row;
                    uint4 *at = reinterpret_cast<uint4 *>(xs + rr * p.x_row_bytes + pc * 16);
                    uint4 v = *at;
                    v.x = bf16x2_to_f16x2(v.x);
                    v.y = bf16x2_to_f16x2(v.y);
                    v.z = bf16x2_to_f16x2(v.z);
                    v.w = bf16x2_to_f16x2(v.w);
                    *at = v;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(xfull_bar(s));
            issue(1);
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int w = warp - C::FIRST_CONSUMER;          // strip of the row tile
        const int ct = tid - C::FIRST_CONSUMER * 32;     // 0..255
        const int g = lane >> 2, tig = lane & 3;
        const bool bf16 = p.dtype == ATLAS_DTYPE_BF16;
        const bool gathered_x = p.wait_flags != nullptr;
        const uint16_t *xg = reinterpret_cast<const uint16_t *>(p.x);

        // Outliers.  The strip's entries (row, column; sorted by column at repack time) of the columns a ring stage
        // covers are one contiguous run, whose end comes from the chunk_ptr table: lane l keeps the boundary after
        // stage cw_base + l of the segment (two windows of 32), and lane l of cur / nxt keeps entry win_base (+32) + l.
        // Everything here is weight-side data, requested ahead; the activations come from the stage in shared memory.
        auto seg_end_kt = [&](int kt_begin, int left) { return min(p.k_tiles, kt_begin + left); };
        int e_cur = 0, e_end = 0, win_base = 0, cw_base = 0, seg_ka = 0, seg_kb = 0;
        // three windows of 32 entries (the one in use and two requested ahead: ~16 stages of lead at the benchmark's
        // outlier density), and the first window of the next segment, requested a few stages before it starts
        uint32_t cur_ent = 0xff000000u, nxt_ent = 0xff000000u, nx2_ent = 0xff000000u, pre_ent = 0xff000000u;
        uint32_t cur_val = 0, nxt_val = 0, nx2_val = 0, pre_val = 0;
        int cwin = 0, cnext = 0, pre_cwin = 0;
        bool have_pre = false;
        const int32_t *seg_cp = nullptr;
        auto load_window = [&](int base, int end, uint32_t &ent, uint32_t &val) {
            ent = 0xff000000u;
            val = 0;
            if (base + lane < end) { ent = __ldg(p.entries + base + lane); val = __ldg(p.ovals + base + lane); }
        };
        auto bounds_of = [&](const int32_t *cp, int ka_, int kb_, int first_stage) {
            // boundary after stage first_stage + lane of a segment [ka_, kb_): the entry index at its end column
            return (int)__ldg(cp + min(ka_ + (first_stage + lane + 1) * p.skt, kb_));
        };
        auto load_bounds = [&](int first_stage) { return bounds_of(seg_cp, seg_ka, seg_kb, first_stage); };
        auto start_segment = [&](int row_tile, int ka_, int kb_, int ea, int eb) {
            seg_cp = p.chunk_ptr + ((size_t)row_tile * 8 + w) * (p.k_tiles + 1);
            seg_ka = ka_;
            seg_kb = kb_;
            e_cur = ea;
            e_end = eb;
            win_base = ea;
            cw_base = 0;
            if (have_pre) {
                cur_ent = pre_ent;
                cur_val = pre_val;
                cwin = pre_cwin;
                have_pre = false;
            } else {
                load_window(ea, eb, cur_ent, cur_val);
                cwin = load_bounds(0);
            }
            load_window(ea + 32, eb, nxt_ent, nxt_val);
            load_window(ea + 64, eb, nx2_ent, nx2_val);
            cnext = load_bounds(32);
        };
        {
            const int32_t *cp = p.chunk_ptr + ((size_t)r0 * 8 + w) * (p.k_tiles + 1);
            const int kb0 = seg_end_kt(kt0, n_units);
            start_segment(r0, kt0, kb0, __ldg(cp + kt0), __ldg(cp + kb0));
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");   // x, y and the workspace belong to the stream from here on

        float acc[MT][4];
        // where this lane finds the activations of batch row nt * 8 + g inside a stage: its own row, or the zero row
        int x_row_off[MT];
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) x_row_off[nt] = nt * 8 + g < p.m ? (nt * 8 + g) * p.x_row_bytes : -1;

        bool alive = true;
        int r = r0, kt = kt0, left = n_units, seg = 0;
        int s = 0, xsi = 0;                  // ring positions of the stage being consumed
        uint32_t ph = 0, xph = 0;            // and the parities of their current rounds
        bool first_stage = true;
        const int bt = POST ? p.bs >> 6 : 1; // tiles per scale block
        constexpr int NA = MT <= 2 ? 2 : 1;  // independent accumulator chains
        while (left > 0) {
            const int ka = kt, kb = seg_end_kt(kt, left);
            // the next segment's outlier range (its row tile starts at column 0): requested now, used when it starts
            int nxt_ea = 0, nxt_eb = 0;
            if (left > kb - ka) {
                const int32_t *cp = p.chunk_ptr + ((size_t)(r + 1) * 8 + w) * (p.k_tiles + 1);
                nxt_ea = __ldg(cp);
                nxt_eb = __ldg(cp + seg_end_kt(0, left - (kb - ka)));
            }
            float part[NA][MT][4];   // dense sums: of the current block (POST) or of the segment
#pragma unroll
            for (int a = 0; a < NA; ++a)
#pragma unroll
                for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) part[a][nt][j] = 0.f;
#pragma unroll
            for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[nt][j] = 0.f;
            int seg_stage = 0;                       // stage index inside the segment
            int blk_left = POST ? bt - kt % bt : 0;  // tiles until the current scale block ends

            while (kt < kb) {
                const int snk = min(p.skt, kb - kt);       // tiles in this stage (the same cut the producers make)
                bool got = !alive || mbar_wait(xfull_bar(xsi), xph, s_abort);
                // the first stage also stands for the activation producer's wait for the other ranks
                for (int extra = 0; !got && gathered_x && first_stage && extra < 64 && !*s_abort; ++extra)
                    got = mbar_wait(xfull_bar(xsi), 0u, s_abort);
                got = got && (!alive || mbar_wait(full_bar(s), ph, s_abort));
                first_stage = false;
                if (!got) {
                    alive = false;
                    *s_abort = 1;
                }
                const unsigned char *stg = smem_raw + (size_t)s * p.stage_stride;
                const unsigned char *xst = x_ring + (size_t)xsi * p.x_stride;
                const int first_blk = p.bs_shift >= 0 ? (kt * 64) >> p.bs_shift : (kt * 64) / p.bs;
                // ---- this warp's codes and scales of the whole stage go to registers and the stage goes back to the
                // producer at once: a code stage that is held while it is multiplied is a stage that is not in flight
                uint4 wreg[SK_SKT][2];
                uint32_t screg[SK_SKT];   // scale of row g | scale of row g + 8 << 16, per tile (of the lane's 16 columns)
                {
                    const unsigned char *wp = stg + w * 1024 + lane * 16;
                    const uint16_t *sc_lane = reinterpret_cast<const uint16_t *>(stg + sc_off) + w * 16 + g;
#pragma unroll
                    for (int j = 0; j < SK_SKT; ++j) {
                        if (j < snk) {
                            wreg[j][0] = *reinterpret_cast<const uint4 *>(wp + j * SK_TILE_BYTES);          // row g of the strip
                            wreg[j][1] = *reinterpret_cast<const uint4 *>(wp + j * SK_TILE_BYTES + 512);    // row g + 8
                            const int col = (kt + j) * 64 + (POST ? 0 : tig * 16);
                            const int kbl = (p.bs_shift >= 0 ? col >> p.bs_shift : col / p.bs) - first_blk;
                            screg[j] = (uint32_t)sc_lane[kbl * 128] | (uint32_t)sc_lane[kbl * 128 + 8] << 16;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar(s));
                }
                if (!have_pre && left > kb - ka && (seg_stage == 3 || kt + snk >= kb)) {
                    // the next segment's first entries and stage boundaries, a few stages before they are needed
                    const int32_t *ncp = p.chunk_ptr + ((size_t)(r + 1) * 8 + w) * (p.k_tiles + 1);
                    load_window(nxt_ea, nxt_eb, pre_ent, pre_val);
                    pre_cwin = bounds_of(ncp, 0, seg_end_kt(0, left - (kb - ka)), 0);
                    have_pre = true;
                }
                {
                    // ---- outliers of the stage's columns, 16 per MMA, activations from the stage itself ----------
                    int o = seg_stage - cw_base;
                    if (o >= 32) {
                        cwin = cnext;
                        cw_base += 32;
                        cnext = load_bounds(cw_base + 32);
                        o -= 32;
                    }
                    const int e_hi = __shfl_sync(0xffffffffu, cwin, o);
                    const int col_base = kt * 64;
                    while (e_cur < e_hi) {
                        if (e_cur - win_base >= 32) {
                            cur_ent = nxt_ent;
                            cur_val = nxt_val;
                            nxt_ent = nx2_ent;
                            nxt_val = nx2_val;
                            win_base += 32;
                            load_window(win_base + 64, e_end, nx2_ent, nx2_val);
                        }
                        const int off = e_cur - win_base;   // 0..31; the group may reach into the next window
                        uint32_t rv[4];
                        int xo[4];                           // byte offset of the entry's column inside a batch row of the stage
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int slot = 2 * tig + (q & 1) + (q >> 1) * 8;
                            const int at = off + slot;
                            uint32_t ent = __shfl_sync(0xffffffffu, cur_ent, at & 31);
                            uint32_t val = __shfl_sync(0xffffffffu, cur_val, at & 31);
                            if (off > 16) {                  // warp-uniform: only then can a slot fall into the next window
                                const uint32_t ent2 = __shfl_sync(0xffffffffu, nxt_ent, at & 31);
                                const uint32_t val2 = __shfl_sync(0xffffffffu, nxt_val, at & 31);
                                if (at >= 32) { ent = ent2; val = val2; }
                            }
                            const bool valid = e_cur + slot < e_hi;
                            rv[q] = valid ? (ent >> 24) << 16 | val : 0x00ff0000u;   // row 255 matches no lane
                            xo[q] = valid ? ((int)(ent & 0xffffffu) - col_base) * 2 : 0;    // 0 .. snk * 128 - 2
                        }
                        uint32_t rws[4], vals[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) { rws[q] = rv[q] >> 16; vals[q] = rv[q] & 0xffffu; }
                        const uint32_t ug = (uint32_t)g;
                        const uint32_t a0 = (rws[0] == ug ? vals[0] : 0u) | (rws[1] == ug ? vals[1] : 0u) << 16;
                        const uint32_t a1 = (rws[0] == ug + 8 ? vals[0] : 0u) | (rws[1] == ug + 8 ? vals[1] : 0u) << 16;
                        const uint32_t a2 = (rws[2] == ug ? vals[2] : 0u) | (rws[3] == ug ? vals[3] : 0u) << 16;
                        const uint32_t a3 = (rws[2] == ug + 8 ? vals[2] : 0u) | (rws[3] == ug + 8 ? vals[3] : 0u) << 16;
#pragma unroll
                        for (int nt = 0; nt < MT; ++nt) {
                            uint32_t xq[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                xq[q] = x_row_off[nt] >= 0 ? *reinterpret_cast<const uint16_t *>(xst + x_row_off[nt] + xo[q]) : 0u;
                            mma_f16(acc[nt], a0, a1, a2, a3, xq[0] | xq[1] << 16, xq[2] | xq[3] << 16);
                        }
                        e_cur = min(e_cur + 16, e_hi);
                    }
                }
                // ---- dense part, from registers; the activations come tile by tile from their own ring -------------
#pragma unroll
                for (int j = 0; j < SK_SKT; ++j) {
                    if (j < snk) {
                        const uint32_t wav[4] = {wreg[j][0].x, wreg[j][0].y, wreg[j][0].z, wreg[j][0].w};
                        const uint32_t wbv[4] = {wreg[j][1].x, wreg[j][1].y, wreg[j][1].z, wreg[j][1].w};
                        uint32_t a_lo[4], a_hi[4], b_lo[4], b_hi[4];
                        if (POST) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                codes4(wav[q], a_lo[q], a_hi[q]);
                                codes4(wbv[q], b_lo[q], b_hi[q]);
                            }
                        } else {
                            const __half2 sa2 = __half2half2(__ushort_as_half((unsigned short)(screg[j] & 0xffffu)));
                            const __half2 sb2 = __half2half2(__ushort_as_half((unsigned short)(screg[j] >> 16)));
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                dequant4(wav[q], sa2, a_lo[q], a_hi[q]);
                                dequant4(wbv[q], sb2, b_lo[q], b_hi[q]);
                            }
                        }
                        const bool fold = POST && (--blk_left == 0 || kt == kb - 1);   // this tile ends its scale block
                        const float sca_f = __half2float(__ushort_as_half((unsigned short)(screg[j] & 0xffffu)));
                        const float scb_f = __half2float(__ushort_as_half((unsigned short)(screg[j] >> 16)));
                        if (fold) blk_left = bt;
#pragma unroll
                        for (int nt = 0; nt < MT; ++nt) {
                            const unsigned char *xr = x_row_off[nt] >= 0 ? xst + x_row_off[nt] + j * 128 : zero_row;
                            const uint4 x0 = *reinterpret_cast<const uint4 *>(xr + tig * 32);
                            const uint4 x1 = *reinterpret_cast<const uint4 *>(xr + tig * 32 + 16);
                            if (nt == MT - 1 && j == snk - 1) {
                                // the last activations of the stage are in registers: hand the activation stage back
                                __syncwarp();
                                if (lane == 0) mbar_arrive(xempty_bar(xsi));
                            }
                            const uint32_t xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                mma_f16(part[q % NA][nt], a_lo[q], b_lo[q], a_hi[q], b_hi[q], xv[2 * q], xv[2 * q + 1]);
                            if (fold) {
#pragma unroll
                                for (int a = 0; a < NA; ++a) {
                                    acc[nt][0] = fmaf(sca_f, part[a][nt][0], acc[nt][0]);
                                    acc[nt][1] = fmaf(sca_f, part[a][nt][1], acc[nt][1]);
                                    acc[nt][2] = fmaf(scb_f, part[a][nt][2], acc[nt][2]);
                                    acc[nt][3] = fmaf(scb_f, part[a][nt][3], acc[nt][3]);
#pragma unroll
                                    for (int c = 0; c < 4; ++c) part[a][nt][c] = 0.f;
                                }
                            }
                        }
                        ++kt;
                    }
                }
                if (++s == NS) { s = 0; ph ^= 1u; }
                if (++xsi == XS) { xsi = 0; xph ^= 1u; }
                ++seg_stage;
            }
            if (!POST) {   // the dense sums were already in the weight's own units
#pragma unroll
                for (int a = 0; a < NA; ++a)
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[nt][c] += part[a][nt][c];
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
                consumer_bar();
                if (ct == 0) {
                    __threadfence();   // the other consumers' stores are ordered before this by the barrier
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
            if (left > 0) start_segment(r, 0, seg_end_kt(0, left), nxt_ea, nxt_eb);
        }
    }

    __syncthreads();
    if (p.world > 1 && tid == 0) {
        // The CTA that finishes last tells every rank that this rank's shard of the output is complete.  Each CTA counts
        // itself in with a release at GPU scope (the barrier orders its stores before it); the last one acquires the
        // others' releases by the same atomic and releases everything at system scope with the flag stores.
        unsigned int finished;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(finished) : "l"(p.state) : "memory");
        if (finished == (unsigned int)grid - 1) {
            const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(p.state + 1) + 1u;
            p.state[0] = 0;
            p.state[1] = seq;
            asm volatile("fence.acq_rel.sys;" ::: "memory");   // one system-scope release for all the flag stores
            for (int d = 0; d < p.world; ++d)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.flags_dst[(p.rank + d) % p.world] + p.rank), "r"(seq) : "memory");
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

template <int MT, bool POST>
int launch_stream(const StreamParams &p, int grid, size_t smem, cudaStream_t st) {
    auto kern = qlinear_stream_kernel<MT, POST>;
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
        // Ring geometry.  A code stage is SK_SKT tiles of 64 columns (8 KB each) plus their scales; a consumer warp
        // takes its share of a stage to registers and hands the stage back at once, so nearly the whole ring is in
        // flight.  The activations of a stage (m rows) live in a ring of their own, which can be deeper (they
        // can only be requested after the dependency wait, so their latency must be paid once, not per stage).
        const int out_bytes = 128 * mt * 8 * 4;
        const int skt = SK_SKT;
        const int max_blk = block_size % 64 == 0 ? (skt * 64 + block_size - 1) / block_size + 1 : (skt * 64) / block_size + 2;
        p.scale_cap = max_blk * 256;
        p.x_row_bytes = skt * 128 + 16;
        p.x_stride = mg * p.x_row_bytes;
        p.stage_stride = (skt * SK_TILE_BYTES + p.scale_cap + 127) & ~127;
        int ns = 6, xs = 0;
        for (; ns >= 2; --ns) {
            const int fixed = ns * (p.stage_stride + 16) + p.x_row_bytes + out_bytes + 64;
            xs = (SK_SMEM_BUDGET - fixed) / (p.x_stride + 24);
            if (xs >= 3) break;
        }
        if (xs > 12) xs = 12;
        ATLAS_RETURN_IF(ns < 2 || xs < 2, ATLAS_ERR_UNSUPPORTED, "atlas_qlinear_stream: the rings do not fit in shared memory");
        p.skt = skt;
        p.n_stages = ns;
        p.x_stages = xs;
        const size_t smem = (size_t)ns * p.stage_stride + (size_t)xs * p.x_stride + p.x_row_bytes + out_bytes +
                            16 * ns + 24 * xs + 64;
        const bool post = block_size % 64 == 0 && p.bs_shift >= 0;   // blocks of whole tiles: integer codes into the MMA
        if (mt == 1) rc = post ? launch_stream<1, true>(p, grid, smem, st) : launch_stream<1, false>(p, grid, smem, st);
        else if (mt == 2) rc = post ? launch_stream<2, true>(p, grid, smem, st) : launch_stream<2, false>(p, grid, smem, st);
        else rc = launch_stream<4, false>(p, grid, smem, st);
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


