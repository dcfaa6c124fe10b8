// Prefill-time quantized linear: y[m][n] = sum_k x[m][k] * W[n][k] + bias[n], m >= 128.
//
// Replaces the dequantize-then-F.linear of QuantizedLinear.forward
// (integration/atlas_wrappers.py:56,67) for prompt-sized batches.  The fp16
// weight the reference materialises (adaptive_quantizer.py:216:
// fp16(fp16(code) * scale), outliers patched in at :221-229) is rebuilt here
// tile by tile in shared memory and consumed at once by the 5th-generation
// tensor cores, so it never exists in global memory.
//
// One CTA computes a 128 (output features) x BN (tokens) tile.  The rebuilt fp16 weights never touch
// shared memory: the dequantizer warps write them straight into tensor memory and the MMA takes its A
// operand from there, so shared memory only carries what comes from global memory (the kernel is bound
// by the shared-memory data pipe, not by the tensor pipe).  A pipeline stage is two k-tiles (128 columns
// of K).  Rings: codes (4 stages of 2 x (8 KB + 256 B of scales)), activations (2 stages of 2 x BN x 64
// fp16, L2-resident), rebuilt weights (4 stages of 64 TMEM columns beside the accumulator; 2 for BN < 256).
//   warp 0      activation producer: per 64-wide K step a 2-D TMA load of the BN x 64 fp16
//               activation tile (128-byte swizzle) completing on the step's `ready` barrier
//   warp 2      code producer: a 1-D bulk copy of the step's 8 KB code tile (contiguous in the
//               tile-major layout) and of the 256 B of scales of its block, completing on `full_c`
//   warps 3-18  dequantizers.  A warp can only reach the TMEM lanes 32 * (warp % 4) .. + 31, and TMEM
//               lane = tile row for the MMA, so thread = row: warp (q, ph) rebuilds rows 32q .. 32q+31
//               of every fourth K step (it % 4 == ph, always into A stage ph): four 16-byte code loads
//               per thread (chunk order rotated per lane so that a quarter-warp covers all banks, then
//               rotated back with selects), codes -> fp16(fp16(code) * scale), the outliers of the
//               warp's two strips written over their (zero-coded) slots in registers (side-table
//               prefetched one step ahead), one tcgen05.st of 32 columns, arrive on `ready`; the
//               code slot is released on `empty_c` as soon as it is in registers
//   warp 1      one thread issues tcgen05.mma (M=128, N=BN, K=16, A from TMEM, B from shared memory,
//               fp32 accumulate in TMEM) four times per step and commits the slot's `mma_done`
//               mbarrier (which frees both the activation slot and the A stage); after the last step
//               it commits `acc_full`
//   warps 3-18  epilogue: tcgen05.ld of their TMEM lane quarter (four warps per quarter, a quarter of
//               the columns each), + bias, convert, transpose through shared memory, 16-byte stores
// Every mbarrier wait is bounded; if one runs out the CTA sets the caller's status word,
// skips the rest of its work, frees its TMEM and returns.
//
// bf16 activations are first converted to fp16 into the workspace (the MMA
// takes both operands as fp16; |x| > 65504 saturates).
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>

#include "common.cuh"

namespace atlas {
namespace {

constexpr int GM_DQ_WARPS = 16;                      // dequantizer warps: 4 TMEM lane quarters x 4 K-step phases
constexpr int GM_EPI_WARPS = 16;                     // all of them drain the accumulator: four per TMEM lane quarter
constexpr int GM_CTRL_WARPS = 3;                     // activation producer (and converter), MMA issuer, code producer
constexpr int GM_THREADS = (GM_CTRL_WARPS + GM_DQ_WARPS) * 32;
constexpr int GM_BM = 128;  // weight rows (output features) per CTA = UMMA M
constexpr int GM_BK = 64;   // K per pipeline step (one 128-byte swizzle row of fp16)
constexpr int GM_SK = 2;    // k-tiles per pipeline stage: one barrier round trip, poll and commit per 128 columns of K
// (the activation ring depth depends on the token tile too: Smem<BN>::XS)
// (the code ring depth depends on the token tile: Smem<BN>::CS)
constexpr int GM_PH = 4;    // K-stage phases of the dequantizers = `ready` / `mma_done` barriers
constexpr int GM_A_COLS = GM_SK * GM_BK / 2;     // TMEM columns of one A stage: two fp16 per 32-bit cell
constexpr uint32_t C_BYTES = GM_BM * GM_BK;      // 8 KB code tile
constexpr uint32_t S_BYTES = 256;                // one scale block: 128 rows x fp16
// shared-memory map for a tile of BN tokens (BN = 32, 64, 128 or 256 = UMMA N)
template <int BN>
struct Smem {
    static constexpr uint32_t B_BYTES = BN * GM_BK * 2;   // fp16 activation tile of one k-tile
    // Code ring depth, in stages of GM_SK k-tiles (16 KB): the bytes an SM keeps in flight.  Decode-sized token
    // tiles are HBM-bound and leave the room for a deep ring (160 KB in flight covers ~3 us of loaded DRAM latency
    // at an SM's share of the bandwidth); the 256-token tile is compute-bound and needs the room for activations.
    static constexpr int CS = BN <= 32 ? 10 : (BN == 64 ? 8 : (BN == 128 ? 6 : 4));
    // Activation ring depth, in stages.  Decode-sized token tiles are filled by a warp (loads, conversion, stores:
    // a microsecond of latency per stage), which a deeper ring hides; the wide tiles come in by TMA.
    static constexpr int XS = BN <= 64 ? 4 : 2;
    static constexpr uint32_t OFF_B = 0;
    static constexpr uint32_t OFF_C = OFF_B + XS * GM_SK * B_BYTES;
    static constexpr uint32_t OFF_BAR = OFF_C + CS * GM_SK * C_BYTES;
    static constexpr uint32_t OFF_S = OFF_BAR + 512;
    static constexpr uint32_t TOTAL = OFF_S + CS * GM_SK * S_BYTES + 1024 /*alignment slack*/;
    // A stages in tensor memory (64 columns each) beside the accumulator columns [0, BN); allocations are powers of two
    static constexpr int A_STAGES = BN == 256 ? 4 : 2;
    static constexpr uint32_t TMEM_COLS = BN + A_STAGES * GM_A_COLS <= 256 ? 256 : 512;
    static_assert(BN + A_STAGES * GM_A_COLS <= 512, "tensor memory");
    // the epilogue stages the output tile over the (then idle) activation and code rings
    static_assert((BN * (GM_BM + 4)) * 4 <= XS * GM_SK * B_BYTES + CS * GM_SK * C_BYTES, "epilogue staging does not fit");
    static_assert(TOTAL <= 227 * 1024, "shared memory");
};
constexpr int GM_SPIN_LIMIT = 1 << 20;       // polls per wait

// ---- PTX wrappers ----------------------------------------------------------------
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
// Bounded wait: false if the phase did not complete within the poll limit.  NS > 0 sleeps between polls, which
// keeps a waiting warp out of the issue slots of the warps that work on the same scheduler.
template <int NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < GM_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (NS > 0) __nanosleep(NS);
    }
    return false;
}
// Same, agreed on by the whole (converged) warp, so that warp-wide instructions after it stay warp-wide.
template <int NS = 0>
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const volatile int *abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait<NS>(bar, parity) && !*abort_flag) != 0;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: A is 128 lanes x 8 columns (16 fp16 along K, two per cell)
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 32 lanes (this warp's quarter) x 32 columns: thread t writes v[0..31] to lane t, columns taddr.col .. + 31
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand tile, rows of 128 bytes (64 fp16), 128-byte
// swizzle, 8-row groups 1024 bytes apart.  Fields: start address >> 4 at bit 0, leading byte
// offset >> 4 at bit 16 (not used by swizzled K-major layouts; 1), stride byte offset >> 4 at bit
// 32, descriptor version 1 at bit 46, swizzle mode 2 (128 B) at bit 61.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: D fp32 (1 at bit 4), A and B fp16 (0 at bits 7 and 10),
// both K-major (0 at bits 15, 16), N >> 3 at bit 17, M >> 4 at bit 24.
template <int BN>
constexpr uint32_t gm_idesc() { return (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(GM_BM >> 4) << 24); }

// Two bf16 (low, high half of v) -> two fp16, saturating at +-65504.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(v & 0xffff0000u)), "f"(__uint_as_float(v << 16)));
    return r;
}

// Four biased codes -> two half2 of fp16(fp16(code) * scale), as in the streaming kernel.
__device__ __forceinline__ void dequant4(uint32_t w, __half2 scale2, uint32_t &lo, uint32_t &hi) {
    const uint32_t l = __byte_perm(w, 0x64646464u, 0x5140);
    const uint32_t h = __byte_perm(w, 0x64646464u, 0x5342);
    const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
    __half2 lv = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&l), bias), scale2);
    __half2 hv = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&h), bias), scale2);
    lo = *reinterpret_cast<uint32_t *>(&lv);
    hi = *reinterpret_cast<uint32_t *>(&hv);
}

struct GemmParams {
    const uint8_t *tiles;
    const uint16_t *scales_t;   // [row/128][block][row%128]
    const int32_t *chunk_ptr;   // [strip][k_tiles + 1]
    const uint32_t *entries;    // row%16 << 24 | column, strip-major, column-sorted
    const uint16_t *ovals;      // values in the order of `entries`
    const uint16_t *bias;
    void *y;
    int64_t ldy;
    int m;
    int n_rows;
    int n_cols;
    int bs;
    int k_tiles;
    int n_chunks;
    int bs_tiles;   // k-tiles per scale block when block_size % 64 == 0 (scales staged by the producer), else 0
    int out_bf16;
    int splits;        // K slices (grid.z); > 1: fp32 partial tiles go to `partials`, a second kernel adds them
    float *partials;   // [splits][m][n_rows] fp32
    int to_partials;   // write the fp32 tile to `partials` even with one K slice (the second kernel writes y)
    int x_bf16;        // the tensor map delivers bf16 rows (decode-sized token tiles only): converted in the kernel
    const unsigned int *wait_flags;    // arrival flags of the ranks that fill x (gathered input), or null
    const unsigned int *gather_state;  // [1]: this rank's count of completed gather launches
    int wait_world;
    long long poll_limit;
    int *error_flag;
};

template <int BN>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap c_map, GemmParams p) {
    using SM = Smem<BN>;
    // the next kernel of the stream may start its own weight-only prologue right away
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr uint32_t B_BYTES = SM::B_BYTES, OFF_B = SM::OFF_B, OFF_C = SM::OFF_C, OFF_BAR = SM::OFF_BAR,
                       OFF_S = SM::OFF_S, TMEM_COLS = SM::TMEM_COLS;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;          // operand tiles need 1024-byte alignment
    unsigned char *base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + OFF_BAR;   // mbarriers, 8 bytes each
    // ready(s): the activation tile has landed (one arrival + its bytes) and the four dequantizer warps of the
    // stage have stored the weights (128 arrivals); the MMA thread waits on this one barrier per K step
    auto ready_bar = [&](int s) { return bars + 8u * s; };
    auto mma_done = [&](int s) { return bars + 8u * (GM_PH + s); };
    auto full_c = [&](int s) { return bars + 8u * (2 * GM_PH + s); };
    constexpr int CS = SM::CS, XS = SM::XS;
    auto empty_c = [&](int s) { return bars + 8u * (2 * GM_PH + CS + s); };
    auto x_landed = [&](int s) { return bars + 8u * (2 * GM_PH + 2 * CS + s); };   // bf16 tile in its slot, to be converted
    constexpr int N_BARS = 2 * GM_PH + 2 * CS + XS + 1;
    static_assert(N_BARS * 8 + 16 <= 512, "barrier area");
    const uint32_t accfull_bar = bars + 8u * (N_BARS - 1);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + OFF_BAR + 8 * N_BARS);
    volatile int *s_abort = reinterpret_cast<volatile int *>(base_ptr + OFF_BAR + 8 * N_BARS + 8);
    constexpr int AS = SM::A_STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * GM_BM;  // first weight row (output feature) of the tile
    const int m0 = blockIdx.y * BN;  // first token
    // this CTA's K steps (grid.z slices K)
    const int kt_begin = (int)((long long)p.k_tiles * blockIdx.z / p.splits);
    const int KT = (int)((long long)p.k_tiles * (blockIdx.z + 1) / p.splits) - kt_begin;
    const int NST = (KT + GM_SK - 1) / GM_SK;   // pipeline stages of GM_SK k-tiles (the last one may hold a single k-tile)
    // stage st uses barriers ready[st % 4] / mma_done[st % 4] in round st / 4, activation slot st % XS, code slot
    // st % CS and A stage st % AS; a resource used by stage st is free again when mma_done of stage st fired
    auto done_bar_of = [&](int st) { return mma_done(st % GM_PH); };
    auto done_par_of = [&](int st) { return (uint32_t)((st / GM_PH) & 1); };

    if (tid == 32 * 0 + 1 || tid == 32 * 2 + 1) {   // the TMA units fetch the 128-byte tensor maps on first use: start that now
        asm volatile("prefetch.tensormap [%0];" ::"l"(tid < 32 ? (const void *)&x_map : (const void *)&c_map) : "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < GM_PH; ++s) {
            mbar_init(ready_bar(s), 4 * 32 + 1);
            mbar_init(mma_done(s), 1);
        }
        for (int s = 0; s < XS; ++s) mbar_init(x_landed(s), 1);
        for (int s = 0; s < CS; ++s) {
            mbar_init(full_c(s), 1);
            mbar_init(empty_c(s), 4);
        }
        mbar_init(accfull_bar, 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation is warp-wide; the same warp frees it at the end
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ activation producer ------------------------------
        // activations come from earlier kernels of the stream; everything else so far read only weights
        asm volatile("griddepcontrol.wait;" ::: "memory");
        bool alive = true;
        if (p.wait_flags) {
            // x is a gathered buffer that the other ranks fill: wait (bounded) until every rank has completed as many
            // gather launches as this one; the code ring keeps filling meanwhile
            const unsigned int target = *reinterpret_cast<const volatile unsigned int *>(p.gather_state + 1);
            bool ok = true;
            if (lane < p.wait_world) {
                ok = false;
                for (long long i = 0; i < p.poll_limit; ++i) {
                    unsigned int v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait_flags + lane) : "memory");
                    if ((int)(v - target) >= 0) { ok = true; break; }
                    __nanosleep(64);
                }
            }
            if (!__all_sync(0xffffffffu, ok)) { alive = false; *s_abort = 1; }
        }
        // requests the activation tiles of stage `st` (lane 0); false if the slot never became free
        auto request = [&](int st) -> bool {
            const int slot = st % XS;
            if (st >= XS && !mbar_wait<32>(done_bar_of(st - XS), done_par_of(st - XS))) return false;
            const int nk = min(GM_SK, KT - st * GM_SK);
            // bf16 tiles land in their slot and are converted there by this warp, which then reports the stage ready
            const uint32_t rb = p.x_bf16 ? x_landed(slot) : ready_bar(st % GM_PH);
            mbar_arrive_expect_tx(rb, (uint32_t)nk * B_BYTES);
            for (int j = 0; j < nk; ++j)
                tma_load_2d(base + OFF_B + (slot * GM_SK + j) * B_BYTES, &x_map, (kt_begin + st * GM_SK + j) * GM_BK, m0, rb);
            return true;
        };
        if (BN <= 64 && p.x_bf16) {
            // bf16 input, decode-sized token tiles.  The tensor map delivers the bf16 rows with the same 128-byte
            // swizzle the MMA expects of the fp16 tile, so the conversion is element-wise in place: lane = token row,
            // eight 16-byte pieces per row and k-tile.  The ring is kept XS - 1 stages ahead: the slot of stage st - 1
            // is requested again after stage st has been converted, when its MMAs have normally finished.
            bool ok = alive;
            int requested = 0;
            if (lane == 0 && ok)
                for (; requested < NST && requested < XS - 1; ++requested) ok = request(requested);
            requested = __shfl_sync(0xffffffffu, requested, 0);
            for (int st = 0; st < NST && __all_sync(0xffffffffu, ok); ++st) {
                const int slot = st % XS;
                if (!mbar_wait_warp<32>(x_landed(slot), (uint32_t)((st / XS) & 1), s_abort)) { ok = false; break; }
                const int nk = min(GM_SK, KT - st * GM_SK);
                for (int j = 0; j < nk; ++j) {
#pragma unroll
                    for (int rr = 0; rr < BN / 32; ++rr) {
                        unsigned char *row = base_ptr + OFF_B + (slot * GM_SK + j) * B_BYTES + (rr * 32 + lane) * 128;
                        uint4 v[8];
#pragma unroll
                        for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint4 *>(row + ((c ^ (lane & 7)) << 4));
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            v[c].x = bf16x2_to_f16x2(v[c].x);
                            v[c].y = bf16x2_to_f16x2(v[c].y);
                            v[c].z = bf16x2_to_f16x2(v[c].z);
                            v[c].w = bf16x2_to_f16x2(v[c].w);
                            *reinterpret_cast<uint4 *>(row + ((c ^ (lane & 7)) << 4)) = v[c];
                        }
                    }
                }
                fence_async_smem();   // the tensor core reads the tile through the async proxy
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(ready_bar(st % GM_PH));
                    if (requested < NST) { ok = request(requested); }
                }
                if (requested < NST) ++requested;
            }
            if (!__all_sync(0xffffffffu, ok)) *s_abort = 1;
        } else if (lane == 0 && alive) {
            for (int st = 0; st < NST; ++st) {
                if (*s_abort) break;
                if (!request(st)) { *s_abort = 1; break; }
            }
        }
    } else if (warp == 2) {
        // ------------------------------ code producer ------------------------------
        if (lane == 0) {
            const int64_t crow0 = (int64_t)blockIdx.x * p.k_tiles + kt_begin;   // code tiles are rows of 128 in the map
            const int bpr = p.n_cols / p.bs;
            for (int st = 0; st < NST; ++st) {
                const int slot = st % CS, round = st / CS;
                if (round > 0 && !mbar_wait<200>(empty_c(slot), (round - 1) & 1)) { *s_abort = 1; break; }
                if (*s_abort) break;
                const int nk = min(GM_SK, KT - st * GM_SK);
                mbar_arrive_expect_tx(full_c(slot), (uint32_t)nk * (C_BYTES + (p.bs_tiles ? S_BYTES : 0)));
                for (int j = 0; j < nk; ++j) {
                    const int kt = st * GM_SK + j;
                    // an 8 KB code tile is a 128-row x 64-byte matrix; the 64-byte swizzle spreads a column of 16-byte
                    // chunks over all banks for the dequantizers (thread = row)
                    tma_load_2d(base + OFF_C + (slot * GM_SK + j) * C_BYTES, &c_map, 0, (int)((crow0 + kt) * GM_BM), full_c(slot));
                    if (p.bs_tiles)
                        bulk_load_1d(base + OFF_S + (slot * GM_SK + j) * S_BYTES,
                                     p.scales_t + ((size_t)blockIdx.x * bpr + (kt_begin + kt) / p.bs_tiles) * 128, S_BYTES, full_c(slot));
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            // One barrier poll, eight MMAs and one commit per stage.  An MMA issue, a poll and a commit each cost this
            // single thread 70-180 cycles and the tensor pipe needs 128 cycles per MMA, so the poll for the next stage
            // is issued between the MMAs of this one (its result is only looked at afterwards) and nothing but the
            // commit stands between the last MMA of a stage and the first of the next.
            bool ok = NST > 0 && mbar_wait(ready_bar(0), 0);
            const uint64_t db0 = make_smem_desc(base + OFF_B);
            const uint32_t ta0 = tmem_base + (uint32_t)BN;
            for (int st = 0; st < NST && ok; ++st) {
                tcgen05_fence_after();
                const uint64_t dbs = db0 + (uint64_t)(((st % XS) * GM_SK * B_BYTES) >> 4);   // the address field counts 16-byte units
                const uint32_t ta = ta0 + (uint32_t)((st % AS) * GM_A_COLS);
                const bool two = KT - st * GM_SK >= 2;
                umma_f16_ts(tmem_base, ta, dbs, gm_idesc<BN>(), st != 0);
                umma_f16_ts(tmem_base, ta + 8u, dbs + 2u, gm_idesc<BN>(), 1u);
                // the next stage's barrier: one poll now, looked at after the commit
                const uint32_t rbn = ready_bar((st + 1) % GM_PH);
                const uint32_t pn = (uint32_t)(((st + 1) / GM_PH) & 1);
                const bool next_ready = st + 1 < NST ? mbar_try_wait(rbn, pn) : true;
                umma_f16_ts(tmem_base, ta + 16u, dbs + 4u, gm_idesc<BN>(), 1u);
                umma_f16_ts(tmem_base, ta + 24u, dbs + 6u, gm_idesc<BN>(), 1u);
                if (two) {
                    const uint64_t db1 = dbs + (uint64_t)(B_BYTES >> 4);
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_f16_ts(tmem_base, ta + 32u + (uint32_t)(k * 8), db1 + (uint64_t)(k * 2), gm_idesc<BN>(), 1u);
                }
                umma_commit(done_bar_of(st));  // arrives when these MMAs have finished reading the slot and the A stage
                if (!next_ready) ok = mbar_wait(rbn, pn);
                if ((st & 7) == 7 && *s_abort) ok = false;
            }
            if (!ok) *s_abort = 1;
            umma_commit(accfull_bar);  // arrives when every MMA issued so far is complete
        }
    } else {
        // ------------------------------ dequantizers, then epilogue ------------------------------
        const int dwi = warp - GM_CTRL_WARPS;     // 0..15
        const int q = warp & 3;                   // TMEM lane quarter this warp may access: rows 32q .. 32q+31 of the tile
        const int ph = dwi >> 2;                  // this warp rebuilds the K steps it == ph (mod 4), always into A stage ph
        const int rl = q * 32 + lane;             // row of the tile (= TMEM lane) this thread rebuilds
        const int rs = lane & 15;                 // its row inside the 16-row strip
        const int swz = (lane >> 1) & 3;          // 64-byte swizzle of this row's 16-byte chunks
        const int bpr = p.n_cols / p.bs;
        const uint16_t *sc_tile = p.scales_t + (int64_t)blockIdx.x * bpr * 128;
        // outlier lists (sorted by column) of the warp's two strips: lanes 0-15 serve strip 2q, lanes 16-31 strip 2q+1
        const int64_t strip = (int64_t)blockIdx.x * 8 + 2 * q + (lane >> 4);
        const int32_t *cp = p.chunk_ptr + strip * (p.n_chunks + 1) + kt_begin;
        const int ej = lane & 15;                 // which entry of its strip's list this lane buffers
        const uint32_t code_off = (uint32_t)rl * 64u;   // the tile is a 128 x 64-byte row-major matrix
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)BN + (uint32_t)((ph % AS) * GM_A_COLS);
        // Side-table pipeline.  The warp's stages are numbered n = 0, 1, .. (stage st = ph + 4 n = k-tiles 2 st, 2 st + 1).
        // The entry ranges [cp[2 st], cp[2 st + 2]) of 16 consecutive stages sit in one register per lane (lane j of each
        // half-warp: stage 16 * block + j of its strip), two such blocks alternate; the entries of a stage are requested
        // two stages ahead, one per lane, and packed for the patch when the stage starts: owner lane (strip half * 16 +
        // row) << 23 | column inside the stage (0..127) << 16 | fp16 value; 63 in the lane field matches nobody.
        constexpr uint32_t NO_ENTRY = 63u << 23;
        const int nsteps = ph < NST ? (NST - ph + 3) >> 2 : 0;
        int rbA = 0, reA = 0, rbB = 0, reB = 0;
        auto load_ranges = [&](int block, int &rb, int &re) {
            const int nn = block * 16 + ej;
            rb = 0;
            re = 0;
            if (nn < nsteps) {
                const int kt = (ph + 4 * nn) * GM_SK;
                rb = __ldg(cp + kt);
                re = __ldg(cp + min(kt + GM_SK, KT));
            }
        };
        auto range_of = [&](int nn, int &b_, int &e_) {   // ranges of stage nn for both half-warps; (0, 0) past the end
            const bool odd = (nn >> 4) & 1;
            const int src = (lane & 16) | (nn & 15);
            b_ = __shfl_sync(0xffffffffu, odd ? rbB : rbA, src);
            e_ = __shfl_sync(0xffffffffu, odd ? reB : reA, src);
        };
        load_ranges(0, rbA, reA);
        load_ranges(1, rbB, reB);
        int b0, e0, b1, e1;
        uint32_t ent0 = 0, val0 = 0, ent1 = 0, val1 = 0;
        range_of(0, b0, e0);
        range_of(1, b1, e1);
        if (b0 + ej < e0) { ent0 = __ldg(p.entries + b0 + ej); val0 = __ldg(p.ovals + b0 + ej); }
        if (b1 + ej < e1) { ent1 = __ldg(p.entries + b1 + ej); val1 = __ldg(p.ovals + b1 + ej); }
        bool ok = true;
        for (int n = 0; n < nsteps && ok; ++n) {
            const int st = ph + 4 * n;
            // request the entries of stage n + 2; when that stage opens a new block of ranges, refill the idle block
            int b2, e2;
            range_of(n + 2, b2, e2);
            uint32_t ent2 = 0, val2 = 0;
            if (b2 + ej < e2) { ent2 = __ldg(p.entries + b2 + ej); val2 = __ldg(p.ovals + b2 + ej); }
            if (((n + 2) & 15) == 0) {
                const int block = (n + 2) >> 4;
                if (block & 1) load_ranges(block + 1, rbA, reA); else load_ranges(block + 1, rbB, reB);
            }
            const int k0 = (kt_begin + st * GM_SK) * GM_BK;   // first column of the stage
            const int nk = min(GM_SK, KT - st * GM_SK);
            auto pack = [&](uint32_t owner_base, uint32_t ent, uint32_t val) -> uint32_t {
                return (owner_base | (ent >> 24)) << 23 | ((ent & 0xffffffu) - (uint32_t)k0) << 16 | val;
            };
            const uint32_t pk0 = b0 + ej < e0 ? pack((uint32_t)(lane & 16), ent0, val0) : NO_ENTRY;
            // which buffered entries belong to this lane's row: five ballots over the owner field
            uint32_t mine_all;
            {
                const uint32_t own = pk0 >> 23;
                mine_all = __ballot_sync(0xffffffffu, own != 63u);
#pragma unroll
                for (int bit = 0; bit < 5; ++bit) {
                    const uint32_t bb = __ballot_sync(0xffffffffu, (own >> bit) & 1u);
                    mine_all &= ((lane >> bit) & 1) ? bb : ~bb;
                }
            }
            const uint32_t second = __ballot_sync(0xffffffffu, (pk0 >> 22) & 1u);   // entries of the stage's second k-tile

            const int sc_ = st % CS, cround = st / CS;   // code slot
            if (!mbar_wait_warp<40>(full_c(sc_), cround & 1, s_abort)) { ok = false; break; }
#pragma unroll
            for (int j = 0; j < GM_SK; ++j) {
                if (j < nk) {
                    const unsigned char *codes = base_ptr + OFF_C + (sc_ * GM_SK + j) * C_BYTES + code_off;
                    // the row's 64 codes: chunk c sits at c ^ ((row >> 1) & 3) under the 64-byte swizzle, so the 8 lanes
                    // of a quarter-warp (rows 64 bytes apart) cover all 32 banks
                    uint4 L[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) L[c] = *reinterpret_cast<const uint4 *>(codes + ((c ^ swz) << 4));
                    __half sh[4];
                    if (p.bs_tiles) {
                        const uint16_t *scs = reinterpret_cast<const uint16_t *>(base_ptr + OFF_S + (sc_ * GM_SK + j) * S_BYTES);
                        sh[0] = sh[1] = sh[2] = sh[3] = __ushort_as_half(scs[rl]);
                    } else {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            sh[c] = __ushort_as_half(__ldg(sc_tile + (int64_t)((k0 + j * GM_BK + c * 16) / p.bs) * 128 + rl));
                    }
                    if (j == nk - 1) {   // the code slot is in registers: hand it back (one arrival per warp)
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty_c(sc_));
                    }
                    uint32_t o[32];   // the row's 64 fp16 weights of this k-tile, two per register
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const __half2 s2 = __half2half2(sh[c]);
                        dequant4(L[c].x, s2, o[c * 8 + 0], o[c * 8 + 1]);
                        dequant4(L[c].y, s2, o[c * 8 + 2], o[c * 8 + 3]);
                        dequant4(L[c].z, s2, o[c * 8 + 4], o[c * 8 + 5]);
                        dequant4(L[c].w, s2, o[c * 8 + 6], o[c * 8 + 7]);
                    }
                    // outliers of the two strips inside this k-tile: every lane pulls the buffered entries of its own row
                    // with one shuffle per round and puts the raw fp16 value over the zero-coded slot; the rounds are
                    // the largest number of outliers any row has in this k-tile
                    auto put = [&](uint32_t pk, bool have) {
                        const uint32_t onehot = have ? 1u << ((pk >> 17) & 31u) : 0u;      // which of the row's 32 registers
                        const uint32_t sel = (pk & 0x10000u) ? 0x5410u : 0x3254u;          // odd column: high half, even: low half
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (onehot & (1u << i)) o[i] = __byte_perm(o[i], pk, sel);
                    };
                    {
                        uint32_t mine = mine_all & (j == 0 ? ~second : second);
                        const int rounds = __reduce_max_sync(0xffffffffu, __popc(mine));
                        for (int r = 0; r < rounds; ++r) {
                            const bool have = mine != 0;
                            const uint32_t pk = __shfl_sync(0xffffffffu, pk0, have ? __ffs(mine) - 1 : 0);
                            mine &= mine - 1;
                            put(pk, have);
                        }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {   // rare: more than 16 outliers of one strip inside one stage
                        const int cnt = __shfl_sync(0xffffffffu, e0 - b0, h * 16);
                        if (cnt > 16) {
                            const int bb = __shfl_sync(0xffffffffu, b0, h * 16);
                            for (int i = 16; i < cnt; ++i) {
                                const uint32_t pk = pack((uint32_t)(h * 16), __ldg(p.entries + bb + i), (uint32_t)__ldg(p.ovals + bb + i));
                                put(pk, (pk >> 23) == (uint32_t)lane && (int)((pk >> 22) & 1u) == j);
                            }
                        }
                    }
                    if (j == 0) {   // the A stage must have been read by the MMAs of its previous use
                        if (st >= AS && !mbar_wait_warp<40>(done_bar_of(st - AS), done_par_of(st - AS), s_abort)) { ok = false; break; }
                        tcgen05_fence_after();
                    }
                    tmem_st_32x32b_x32(taddr + (uint32_t)(j * (GM_BK / 2)), o);
                }
            }
            if (!ok) break;
            tmem_st_wait();
            tcgen05_fence_before();
            mbar_arrive(ready_bar(st % GM_PH));
            ent0 = ent1; val0 = val1; ent1 = ent2; val1 = val2;
            b0 = b1; e0 = e1; b1 = b2; e1 = e2;
        }
        if (!ok) *s_abort = 1;

        // epilogue: TMEM lane = output feature, column = token.  The accumulators go through shared
        // memory (the rings are idle by now) so that y is written in 16-byte pieces along a token row.
        // The 16 warps take ONE decision together (a barrier that ANDs their votes): the named barrier inside the
        // epilogue must be reached by all of them or by none, also when only some saw a wait run out.
        const bool acc_ok = mbar_wait_warp<200>(accfull_bar, 0, s_abort);
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "barrier.cta.red.and.pred q, 1, %2, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(all_ok) : "r"((uint32_t)acc_ok), "n"(GM_EPI_WARPS * 32) : "memory");
        if (all_ok) {
            tcgen05_fence_after();
            const int part = (warp - GM_CTRL_WARPS) >> 2;   // four warps share a TMEM lane quarter: 32-column chunks part, part + 4, ..
            const int nl = q * 32 + lane;                   // feature inside the tile
            const int n = n0 + nl;
            const float bv = (p.bias && n < p.n_rows) ? __half2float(__ushort_as_half(__ldg(p.bias + n))) : 0.f;
            // staging tile [BN tokens][128 features (+ pad)] in the idle rings: 16-bit outputs, or fp32
            // partial sums when K is split between CTAs
            const bool partial = p.splits > 1 || p.to_partials;
            unsigned char *stage = base_ptr + OFF_B;
            const int st_bytes = partial ? (GM_BM + 4) * 4 : (GM_BM + 8) * 2;   // row stride; pads keep banks apart
            for (int c = part; c < BN / 32; c += 4) {
                if (m0 + c * 32 >= p.m) break;  // warp-uniform: no tokens left in this tile
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    unsigned char *row = stage + (size_t)(c * 32 + j) * st_bytes;
                    if (partial) {
                        reinterpret_cast<uint32_t *>(row)[nl] = v[j];
                    } else {
                        const float f = __uint_as_float(v[j]) + bv;
                        reinterpret_cast<uint16_t *>(row)[nl] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(f))
                                                                          : __half_as_ushort(__float2half_rn(f));
                    }
                }
            }
            // all eight epilogue warps have staged their part
            asm volatile("bar.sync 1, %0;" ::"n"(GM_EPI_WARPS * 32) : "memory");
            const int et = tid - GM_CTRL_WARPS * 32;         // 0..511
            const int rows_left = min(BN, p.m - m0);
            if (partial) {
                // fp32 partial tile -> partials[z][m][n], 16 bytes (4 features) per thread and store
                float *dst0 = p.partials + (size_t)blockIdx.z * p.m * p.n_rows;
                const bool vec_ok = (n0 + GM_BM <= p.n_rows) && (p.n_rows % 4 == 0);
                for (int idx = et; idx < rows_left * (GM_BM / 4); idx += GM_EPI_WARPS * 32) {
                    const int row = idx >> 5, piece = idx & 31;
                    const float *src = reinterpret_cast<const float *>(stage + (size_t)row * st_bytes) + piece * 4;
                    float *dst = dst0 + (size_t)(m0 + row) * p.n_rows + n0 + piece * 4;
                    if (vec_ok) {
                        *reinterpret_cast<float4 *>(dst) = *reinterpret_cast<const float4 *>(src);
                    } else {
                        for (int e = 0; e < 4; ++e)
                            if (n0 + piece * 4 + e < p.n_rows) dst[e] = src[e];
                    }
                }
            } else {
                const bool vec_ok = (n0 + GM_BM <= p.n_rows) && (p.ldy % 8 == 0) && (((uintptr_t)p.y & 15) == 0);
                for (int idx = et; idx < rows_left * (GM_BM / 8); idx += GM_EPI_WARPS * 32) {
                    const int row = idx >> 4, piece = idx & 15;  // 16 pieces of 8 features per token row
                    const uint16_t *src = reinterpret_cast<const uint16_t *>(stage + (size_t)row * st_bytes) + piece * 8;
                    uint16_t *dst = reinterpret_cast<uint16_t *>(p.y) + (int64_t)(m0 + row) * p.ldy + n0 + piece * 8;
                    if (vec_ok) {
                        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
                    } else {
                        for (int e = 0; e < 8; ++e)
                            if (n0 + piece * 8 + e < p.n_rows) dst[e] = src[e];
                    }
                }
            }
        } else {
            *s_abort = 1;
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    if (tid == 0 && *s_abort && p.error_flag) atomicExch(p.error_flag, 1);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Where the second kernel writes y when the output is gathered over the ranks of a node: the same columns of
// every rank's buffer (plain peer stores), followed by the arrival count (see atlas_qlinear_stream_gather).
struct FinishGather {
    int world;   // 0: no gather, y is local
    int rank;
    void *y_dst[ATLAS_MAX_PEERS];
    unsigned int *flags_dst[ATLAS_MAX_PEERS];
    unsigned int *state;
};

// Adds the K-slice partial tiles in slice order (deterministic), adds the bias and writes y.
// VEC: 8 features (16 bytes of output) per thread; needs n_rows % 8 == 0 and 16-byte aligned output rows.
template <bool VEC>
__global__ void __launch_bounds__(256)
gemm_finish_kernel(const float *partials, int splits, int m, int n_rows, const uint16_t *bias, void *y, int64_t ldy,
                   int out_bf16, FinishGather fg) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr int W = VEC ? 8 : 1;
    const int64_t total = (int64_t)m * n_rows, pieces = total / W;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < pieces; i += (int64_t)gridDim.x * 256) {
        const int64_t e0 = i * W;
        const int row = (int)(e0 / n_rows), n = (int)(e0 - (int64_t)row * n_rows);
        float acc[W];
#pragma unroll
        for (int e = 0; e < W; ++e) acc[e] = 0.f;
        for (int z = 0; z < splits; ++z) {
            const float *src = partials + (size_t)z * total + e0;
            if (VEC) {
                const float4 a = __ldcg(reinterpret_cast<const float4 *>(src)), b = __ldcg(reinterpret_cast<const float4 *>(src) + 1);
                acc[0] += a.x; acc[1 % W] += a.y; acc[2 % W] += a.z; acc[3 % W] += a.w;
                acc[4 % W] += b.x; acc[5 % W] += b.y; acc[6 % W] += b.z; acc[7 % W] += b.w;
            } else {
                acc[0] += __ldcg(src);
            }
        }
        uint16_t out[W];
#pragma unroll
        for (int e = 0; e < W; ++e) {
            float v = acc[e];
            if (bias) v += __half2float(__ushort_as_half(__ldg(bias + n + e)));
            out[e] = out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
        }
        const int64_t off = (int64_t)row * ldy + n;
        const int dests = fg.world > 0 ? fg.world : 1;
        for (int d = 0; d < dests; ++d) {
            uint16_t *dst = reinterpret_cast<uint16_t *>(y);
            if (fg.world > 0) {
                int to = fg.rank + d;
                if (to >= fg.world) to -= fg.world;
                dst = reinterpret_cast<uint16_t *>(fg.y_dst[to]);
            }
            if (VEC) *reinterpret_cast<uint4 *>(dst + off) = make_uint4(out[0] | (uint32_t)out[1 % W] << 16, out[2 % W] | (uint32_t)out[3 % W] << 16,
                                                                        out[4 % W] | (uint32_t)out[5 % W] << 16, out[6 % W] | (uint32_t)out[7 % W] << 16);
            else dst[off] = out[0];
        }
    }
    if (fg.world > 0) {
        // the CTA that finishes last tells every rank that this rank's columns are complete
        // Each CTA counts itself in with a release at GPU scope (the barrier orders the CTA's stores before it); the
        // last one acquires the others' releases by the same atomic and releases everything at system scope with
        // the flag stores themselves.  No stand-alone system fence: two of them in a row cost ~8 us per launch.
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int finished;
            asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(finished) : "l"(fg.state) : "memory");
            if (finished == gridDim.x - 1) {
                const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(fg.state + 1) + 1u;
                fg.state[0] = 0;
                fg.state[1] = seq;
                asm volatile("fence.acq_rel.sys;" ::: "memory");   // one system-scope release for all the flag stores
                for (int d = 0; d < fg.world; ++d) {
                    int to = fg.rank + d;
                    if (to >= fg.world) to -= fg.world;
                    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(fg.flags_dst[to] + fg.rank), "r"(seq) : "memory");
                }
            }
        }
    }
}

// bf16 -> fp16 (saturating) into a dense [m][k] buffer; also used to make strided fp16 rows dense.  When x is a
// gathered buffer that the other ranks fill (`wait_flags`), every CTA first waits, bounded, until all ranks'
// arrival counts have reached this rank's own (state[1]).
__global__ void __launch_bounds__(256)
to_f16_kernel(const uint16_t *x, int64_t ldx, int m, int k, int from_bf16, uint16_t *out, const unsigned int *wait_flags,
              int wait_world, const unsigned int *state, long long poll_limit, int *status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (wait_flags) {
        if (threadIdx.x < 32) {
            const int lane = threadIdx.x;
            const unsigned int target = *reinterpret_cast<const volatile unsigned int *>(state + 1);
            bool ok = true;
            if (lane < wait_world) {
                ok = false;
                for (long long i = 0; i < poll_limit; ++i) {
                    unsigned int v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(wait_flags + lane) : "memory");
                    if ((int)(v - target) >= 0) { ok = true; break; }
                    __nanosleep(64);
                }
            }
            if (!__all_sync(0xffffffffu, ok) && lane == 0 && status) atomicExch(status, 1);   // reported; the copy goes on
        }
        __syncthreads();
    }
    const int64_t total = (int64_t)m * (k >> 1);
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        const int64_t row = i / (k >> 1), c2 = i - row * (k >> 1);
        // (read through L2: with wait_flags the rows were written by other GPUs)
        uint32_t v = __ldcg(x + row * ldx + 2 * c2) | (uint32_t)__ldcg(x + row * ldx + 2 * c2 + 1) << 16;
        if (from_bf16) v = bf16x2_to_f16x2(v);
        reinterpret_cast<uint32_t *>(out)[i] = v;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn *out) {
    static EncodeTiledFn cached = nullptr;
    if (!cached) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        int rc = check_cuda(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres),
                            "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
        if (rc) return rc;
        if (qres != cudaDriverEntryPointSuccess || !fn) {
            set_error("cuTensorMapEncodeTiled is not available in this driver");
            return ATLAS_ERR_LAUNCH;
        }
        cached = (EncodeTiledFn)fn;
    }
    *out = cached;
    return ATLAS_OK;
}

constexpr size_t GM_WS_HEADER = 256;  // reserved; the fp16 copy of x follows

}  // namespace
}  // namespace atlas

namespace atlas {
namespace {

// launch configuration with programmatic dependent launch allowed
cudaLaunchConfig_t pdl_config(dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
    static thread_local cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
}

// tokens per tile for a batch of m rows
int gemm_bn_for(int64_t m) { return m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256)); }

// K slices for decode-sized batches (one CTA per SM, `tiles` output tiles): the count that minimises
// waves x (k-tiles per CTA + the fixed cost of a CTA, about 12 k-tiles' worth of streaming), so that neither a
// nearly empty last wave nor many short CTAs dominate.
int gemm_splits_for(int64_t m, int64_t n_rows, int64_t n_cols, int sms) {
    const int bn = gemm_bn_for(m);
    if (bn > 64) return 1;
    const int64_t tiles = ceil_div_i64(n_rows, GM_BM) * ceil_div_i64(m, bn);
    const int k_tiles = (int)(n_cols / 64);
    int best = 1;
    int64_t best_cost = 0;
    for (int s = 1; s <= 16; s *= 2) {
        if (s > 1 && k_tiles / s < 8) break;
        const int64_t cost = ceil_div_i64(tiles * s, sms) * (ceil_div_i64(k_tiles, s) + 12);
        if (s == 1 || cost < best_cost) { best = s; best_cost = cost; }
    }
    return best;
}

int gemm_sm_count() {
    static thread_local int dev_cached = -1, sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != dev_cached) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
        dev_cached = dev;
    }
    return sms;
}

template <int BN>
int launch_gemm(const CUtensorMap &x_map, const CUtensorMap &c_map, const GemmParams &p, cudaStream_t st) {
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        int rc = check_cuda(cudaFuncSetAttribute(gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)Smem<BN>::TOTAL), "cudaFuncSetAttribute(gemm smem)");
        if (rc) return rc;
        configured_dev = dev;
    }
    cudaLaunchConfig_t cfg = pdl_config(dim3((unsigned)ceil_div_i64(p.n_rows, GM_BM), (unsigned)ceil_div_i64(p.m, BN), (unsigned)p.splits),
                                        dim3(GM_THREADS), Smem<BN>::TOTAL, st);
    return check_cuda(cudaLaunchKernelEx(&cfg, gemm_kernel<BN>, x_map, c_map, p), "gemm_kernel launch");
}

}  // namespace
}  // namespace atlas

extern "C" size_t atlas_qlinear_gemm_workspace_bytes(int64_t m, int64_t n_rows, int64_t n_cols) {
    if (m <= 0 || n_cols <= 0 || n_rows <= 0) return atlas::GM_WS_HEADER;
    // fp16 copy of x (bf16 or strided input), then room for up to 8 fp32 K-slice partial outputs
    // (only decode-sized batches are ever sliced)
    const size_t xcopy = ((size_t)m * (size_t)n_cols * 2 + 255) & ~(size_t)255;
    // (one fp32 slice of the output per K slice; one even without slicing, for the gathered form)
    const size_t part = atlas::gemm_bn_for(m) <= 64
                            ? (size_t)atlas::gemm_splits_for(m, n_rows, n_cols, atlas::gemm_sm_count()) * (size_t)m * (size_t)n_rows * 4
                            : 0;
    return atlas::GM_WS_HEADER + xcopy + part;
}

namespace atlas {
namespace {

int gemm_entry(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles, const void *scales_tiled,
               const int32_t *outlier_chunk_ptr, const uint32_t *outlier_entries, const void *outlier_vals_sorted,
               int64_t n_rows, int64_t n_cols, int block_size, const void *bias, void *y, int64_t ldy, void *workspace,
               size_t workspace_bytes, int32_t *status, void *stream, const AtlasPeerGather *gather) {
    clear_error();
    FinishGather fg;
    memset(&fg, 0, sizeof(fg));
    if (gather) {
        ATLAS_RETURN_IF(gather->world < 1 || gather->world > ATLAS_MAX_PEERS || gather->rank < 0 || gather->rank >= gather->world ||
                            !gather->state || gather->poll_limit < 1, ATLAS_ERR_BAD_ARGUMENT,
                        "atlas_qlinear_gemm_gather: bad gather descriptor");
        ATLAS_RETURN_IF(m > 64, ATLAS_ERR_UNSUPPORTED,
                        "atlas_qlinear_gemm_gather: decode-sized batches only (m <= 64); gather larger ones with a collective");
        fg.world = gather->world;
        fg.rank = gather->rank;
        fg.state = gather->state;
        for (int d = 0; d < gather->world; ++d) {
            ATLAS_RETURN_IF(!gather->y_dst[d] || !gather->flags_dst[d], ATLAS_ERR_BAD_ARGUMENT,
                            "atlas_qlinear_gemm_gather: null destination");
            fg.y_dst[d] = gather->y_dst[d];
            fg.flags_dst[d] = gather->flags_dst[d];
        }
        y = gather->y_dst[gather->rank];
    }
    ATLAS_RETURN_IF(!x || !tiles || !scales_tiled || !outlier_chunk_ptr || !y || !workspace, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemm: null buffer");
    ATLAS_RETURN_IF(m < 0 || n_rows <= 0 || n_cols <= 0 || ldx < n_cols || ldy < n_rows, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemm: bad size (m=%lld n_rows=%lld n_cols=%lld ldx=%lld ldy=%lld)",
                    (long long)m, (long long)n_rows, (long long)n_cols, (long long)ldx, (long long)ldy);
    ATLAS_RETURN_IF(dtype != ATLAS_DTYPE_F16 && dtype != ATLAS_DTYPE_BF16, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemm: dtype %d", dtype);
    ATLAS_RETURN_IF(n_cols % 64 != 0 || block_size < 16 || block_size % 16 != 0 || n_cols % block_size != 0,
                    ATLAS_ERR_UNSUPPORTED,
                    "atlas_qlinear_gemm: needs n_cols %% 64 == 0 and block_size a multiple of 16 dividing n_cols");
    ATLAS_RETURN_IF(n_rows > 0x7fffff00 || n_cols >= (1 << 24) || m > 0x7fffff00, ATLAS_ERR_UNSUPPORTED,
                    "atlas_qlinear_gemm: too large");
    ATLAS_RETURN_IF(((uintptr_t)tiles & 15) != 0 || ((uintptr_t)workspace & 255) != 0, ATLAS_ERR_BAD_ARGUMENT,
                    "atlas_qlinear_gemm: tiles must be 16-byte and workspace 256-byte aligned");
    const size_t need = atlas_qlinear_gemm_workspace_bytes(m, n_rows, n_cols);
    ATLAS_RETURN_IF(workspace_bytes < need, ATLAS_ERR_CAPACITY,
                    "atlas_qlinear_gemm: workspace holds %zu bytes, %zu needed", workspace_bytes, need);
    int rc = check_device();
    if (rc) return rc;
    if (m == 0) return ATLAS_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int bn = gemm_bn_for(m);

    // operand B must be fp16 with rows on 16-byte boundaries for the tensor map
    const void *xb = x;
    int64_t ldb = ldx;
    const size_t xcopy = ((size_t)m * (size_t)n_cols * 2 + 255) & ~(size_t)255;
    const unsigned int *wait_flags = gather ? gather->wait_flags : nullptr;
    // Rows the tensor map can take as they are: 16-byte aligned, fp16 -- or bf16 for decode-sized token tiles,
    // which the kernel converts in shared memory.  Anything else is copied to a dense fp16 buffer first.
    const bool tma_ok = ((uintptr_t)x & 15) == 0 && (ldx % 8) == 0;
    // (in the kernel when the weight is small: one more kernel in the chain then costs more than the conversion's
    // share of the producer warp over the few stages of a CTA)
    const bool small_weight = n_rows * n_cols <= ((int64_t)32 << 20);
    const bool in_kernel_bf16 = dtype == ATLAS_DTYPE_BF16 && bn <= 64 && tma_ok && small_weight;
    const bool direct = tma_ok && (dtype == ATLAS_DTYPE_F16 || in_kernel_bf16);
    // a gathered input is waited for by whichever kernel reads x first: the copy kernel, or the linear kernel itself
    const bool wait_in_copy = wait_flags && !direct;
    if (!direct) {
        uint16_t *xf = (uint16_t *)((char *)workspace + GM_WS_HEADER);
        const int64_t pairs = m * (n_cols / 2);
        const int64_t blocks = ceil_div_i64(pairs, 256);
        cudaLaunchConfig_t cfg = pdl_config(dim3((unsigned)(blocks < 65535 ? blocks : 65535)), dim3(256), 0, st);
        rc = check_cuda(cudaLaunchKernelEx(&cfg, to_f16_kernel, (const uint16_t *)x, ldx, (int)m, (int)n_cols,
                                           (int)(dtype == ATLAS_DTYPE_BF16), xf, wait_in_copy ? wait_flags : (const unsigned int *)nullptr,
                                           gather ? (int)gather->world : 0,
                                           gather ? (const unsigned int *)gather->state : (const unsigned int *)nullptr,
                                           gather ? (long long)gather->poll_limit : 0ll, (int *)status), "to_f16_kernel launch");
        if (rc) return rc;
        xb = xf;
        ldb = n_cols;
    }

    EncodeTiledFn encode = nullptr;
    rc = get_encode_fn(&encode);
    if (rc) return rc;
    CUtensorMap x_map;
    const cuuint64_t gdim[2] = {(cuuint64_t)n_cols, (cuuint64_t)m};
    const cuuint64_t gstride[1] = {(cuuint64_t)ldb * 2};
    const cuuint32_t box[2] = {(cuuint32_t)GM_BK, (cuuint32_t)bn};
    const cuuint32_t estride[2] = {1, 1};
    CUresult cr = encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(xb), gdim, gstride, box,
                         estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ATLAS_RETURN_IF(cr != CUDA_SUCCESS, ATLAS_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with %d", (int)cr);
    // the code tiles as one matrix of 64-byte rows: tile (row tile rt, k-tile kt) = rows (rt * k_tiles + kt) * 128 .. + 127
    CUtensorMap c_map;
    {
        const cuuint64_t cdim[2] = {(cuuint64_t)GM_BK, (cuuint64_t)(ceil_div_i64(n_rows, GM_BM) * (n_cols / GM_BK) * GM_BM)};
        const cuuint64_t cstride[1] = {(cuuint64_t)GM_BK};
        const cuuint32_t cbox[2] = {(cuuint32_t)GM_BK, (cuuint32_t)GM_BM};
        cr = encode(&c_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(tiles), cdim, cstride, cbox, estride,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        ATLAS_RETURN_IF(cr != CUDA_SUCCESS, ATLAS_ERR_LAUNCH, "cuTensorMapEncodeTiled (codes) failed with %d", (int)cr);
    }

    GemmParams p;
    p.tiles = tiles;
    p.scales_t = (const uint16_t *)scales_tiled;
    p.chunk_ptr = outlier_chunk_ptr;
    p.entries = outlier_entries;
    p.ovals = (const uint16_t *)outlier_vals_sorted;
    p.bias = (const uint16_t *)bias;
    p.y = y;
    p.ldy = ldy;
    p.m = (int)m;
    p.n_rows = (int)n_rows;
    p.n_cols = (int)n_cols;
    p.bs = block_size;
    p.k_tiles = (int)(n_cols / 64);
    p.n_chunks = (int)(n_cols / 64);
    p.bs_tiles = block_size % 64 == 0 ? block_size / 64 : 0;
    p.out_bf16 = dtype == ATLAS_DTYPE_BF16;
    p.splits = gemm_splits_for(m, n_rows, n_cols, gemm_sm_count());
    p.partials = (float *)((char *)workspace + GM_WS_HEADER + xcopy);
    p.to_partials = gather != nullptr;   // the gather is the second kernel's job
    p.x_bf16 = in_kernel_bf16;
    p.wait_flags = wait_in_copy ? nullptr : wait_flags;
    p.gather_state = gather ? (const unsigned int *)gather->state : nullptr;
    p.wait_world = gather ? gather->world : 0;
    p.poll_limit = gather ? (long long)gather->poll_limit : 0;
    p.error_flag = status;
    switch (bn) {
        case 32: rc = launch_gemm<32>(x_map, c_map, p, st); break;
        case 64: rc = launch_gemm<64>(x_map, c_map, p, st); break;
        case 128: rc = launch_gemm<128>(x_map, c_map, p, st); break;
        default: rc = launch_gemm<256>(x_map, c_map, p, st); break;
    }
    if (rc) return rc;
    if (p.splits > 1 || p.to_partials) {
        const bool vec = n_rows % 8 == 0 && ldy % 8 == 0 && (((uintptr_t)y & 15) == 0) &&
                         (((uintptr_t)p.partials & 15) == 0);
        bool vec_all = vec;
        for (int d = 0; d < fg.world; ++d) vec_all = vec_all && (((uintptr_t)fg.y_dst[d] & 15) == 0);
        const int64_t pieces = m * n_rows / (vec_all ? 8 : 1);
        const int64_t blocks = ceil_div_i64(pieces, 256);
        cudaLaunchConfig_t cfg = pdl_config(dim3((unsigned)(blocks < 2048 ? blocks : 2048)), dim3(256), 0, st);
        auto kern = vec_all ? gemm_finish_kernel<true> : gemm_finish_kernel<false>;
        rc = check_cuda(cudaLaunchKernelEx(&cfg, kern, (const float *)p.partials, p.splits, (int)m, (int)n_rows,
                                           (const uint16_t *)bias, y, ldy, p.out_bf16, fg), "gemm_finish_kernel launch");
    }
    return rc;
}

}  // namespace
}  // namespace atlas

extern "C" int atlas_qlinear_gemm(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                  const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                  const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                  int64_t n_rows, int64_t n_cols, int block_size, const void *bias, void *y,
                                  int64_t ldy, void *workspace, size_t workspace_bytes, int32_t *status,
                                  void *stream) {
    ATLAS_RETURN_IF(!y, ATLAS_ERR_BAD_ARGUMENT, "atlas_qlinear_gemm: null buffer");
    return atlas::gemm_entry(x, dtype, m, ldx, tiles, scales_tiled, outlier_chunk_ptr, outlier_entries, outlier_vals_sorted,
                             n_rows, n_cols, block_size, bias, y, ldy, workspace, workspace_bytes, status, stream, nullptr);
}

extern "C" int atlas_qlinear_gemm_gather(const void *x, int dtype, int64_t m, int64_t ldx, const uint8_t *tiles,
                                         const void *scales_tiled, const int32_t *outlier_chunk_ptr,
                                         const uint32_t *outlier_entries, const void *outlier_vals_sorted,
                                         int64_t n_rows, int64_t n_cols, int block_size, const void *bias,
                                         int64_t ldy, void *workspace, size_t workspace_bytes, int32_t *status,
                                         void *stream, const AtlasPeerGather *gather) {
    ATLAS_RETURN_IF(!gather, ATLAS_ERR_BAD_ARGUMENT, "atlas_qlinear_gemm_gather: null gather descriptor");
    return atlas::gemm_entry(x, dtype, m, ldx, tiles, scales_tiled, outlier_chunk_ptr, outlier_entries, outlier_vals_sorted,
                             n_rows, n_cols, block_size, bias, nullptr, ldy, workspace, workspace_bytes, status, stream, gather);
}
