// MUL_MAT for a batch of activation columns on the 5th-generation tensor cores (tcgen05, TMEM accumulators).
//
// Same arithmetic as mmq.cu (lm_ggml_compute_forward_mul_mat, cactus/ggml-cpu/ggml-cpu.c:1257-1449): one exact integer
// dot product per 32-element block, then d_w[row] * d_a[col] scaling into fp32 accumulators.  What differs is where the
// work runs:
//   * The integer dot is computed by tcgen05.mma.kind::f8f6f4 on e4m3 operands that hold small integers.  The
//     subnormals and the first binade of e4m3 are the integers 0..15 times 2^-9, so a weight nibble u = q + 8, zero
//     extended to a byte, already *is* the e4m3 encoding of u * 2^-9: expanding the packed weights is a mask and an
//     XOR.  An activation quant a = 16 h + l (h = a >> 4, l = a & 15) is two e4m3 bytes (h * 2^-5 and l * 2^-9, planes
//     written by the quantiser), multiplied by two MMAs that accumulate.  Every product and every partial sum is an
//     integer below 2^17 times 2^-18, so the fp32 accumulator holds the exact value of sum(u a) * 2^-18: the block dot
//     stays bit-exact, and it arrives as a float -- no int -> float conversion in the epilogue.
//   * sum(q a) = sum(u a) - 8 sum(a); the quantiser stores D = d_a * 2^18 and C = -8 d_a sum(a) per (column, block), so
//     t = fma(v, D, C) = d_a * dot and y = fma(t, d_w, y) are the only two operations per value and block, issued as
//     fma.rn.f32x2 on column pairs.
//   * The expanded weights never touch shared memory: a thread owns one weight row, expands 4 blocks of it in registers
//     and writes them into tensor memory (tcgen05.st), from where the MMA reads its A operand.
//
// A CTA (one per SM, 20 warps with fixed roles, joined by mbarriers only) owns 128 weight rows x up to 64 columns and
// walks K in groups of 4 blocks:
//   warps 0-3   MMA issue: warp w issues block w of every group -- two MMAs of 128 x 64 x 32 (hi plane, then lo plane
//               accumulating) -- so the accumulator tiles in flight turn over independently of each other;
//   warp 4      producer: five TMA tensor copies per group into a ring of stages -- the packed T16 weight tiles (one
//               box of 8 row tiles, written with the 128-byte swizzle so that the row-per-thread reads below are
//               conflict free), their fp16 scales, the two e4m3 activation planes and the activation scales;
//   warps 8-11  expand: thread = weight row; four 16-byte loads give the row's 4 blocks, 32 registers go to TMEM;
//   warps 12-19 epilogue: one per (TMEM lane quarter, 32-column half).  Accumulator tiles are read in the MMA fragment
//               order (16x256b: a thread holds 4 rows x 4 column pairs of a block, so a 16-byte load of column scales
//               serves 4 rows), the tile of block b+1 is in flight while block b is scaled.
// Tensor memory: six accumulator tiles of one block (64 columns each) and four A buffers of 4 blocks (32 columns each).
// Every wait is bounded; on time-out the CTA raises b200_kernel_status, all roles fall through, the producer waits
// (bounded) for its copies in flight, the issuing warps for their MMAs, the CTA frees its TMEM and returns.
//
// Measured on B200 (probes run on this pool; the figures that shaped the kernel and that bound it today):
//   * tcgen05.mma 128 x 64 x 32, e4m3 or s8, issued back to back: 48.6 clk with A in shared memory, 45.5 clk with A in
//     TMEM (the shared-memory operand fetch, not the 32 clk of arithmetic, sets the pace); 128 x 128 x 32: 64.6 clk = 8117
//     MAC/clk/SM; s8 and e4m3 run at the same rate.  Integer-valued e4m3 operands accumulate exactly (0 mismatches in
//     8192 dots including the extreme values).
//   * a hand-over between warps costs 230-280 clk whatever the mechanism (mbarrier try_wait / test_wait, a polled
//     shared-memory counter, bar.sync / bar.arrive all measured 460-560 clk per round trip), and a wait costs the
//     waiting warp well over a hundred cycles even when the phase is already complete;
//   * tcgen05.ld moves 253 B/clk/SM in the 16x256b shape, 476 in 16x128b, 652 in 32x32b;
//   * a 16-byte shared-memory load whose lanes share 4 addresses occupies the SM's load unit for about 6 clk.
// With one block (92 clk of MMA, 128 clk of FP32 work) as the unit that is handed from role to role, those costs add
// up to about 2900 clk per group of 4 blocks where the mma.sync kernel needs 2700: the kernel passes every parity
// case but is not the default (B200_MMQ_TC=1 selects it).
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace b200 {

void launch_mmq_reduce(const float *partial, int ks, int64_t M, int64_t N, float *dst, int64_t dst_nb_row, cudaStream_t st);
int launch_mmq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
               void *workspace, size_t workspace_bytes, cudaStream_t st, bool canon, const PeerDst &peers);

__device__ int g_tc_error = 0;   // non-zero after a bounded wait gave up
__device__ unsigned g_tc_spin_limit = 1u << 20;   // try_wait rounds before a wait gives up (each may suspend for a while)
constexpr uint32_t TC_DRAIN_LIMIT = 1u << 22;     // what a CTA that gave up still waits for: its own copies and MMAs in flight
#ifdef B200_TC_PROFILE
__device__ long long g_tc_prof[4][64];   // [role][iteration]: clock of CTA 0 when the role starts work on an iteration
#define TC_PROF(role, it) do { if (blockIdx.x == 0 && blockIdx.z == 0 && lane == 0 && (it) < 64) g_tc_prof[role][it] = clock64(); } while (0)
#else
#define TC_PROF(role, it) do { } while (0)
#endif

constexpr int TC_THREADS = 640;   // 20 warps: 0-3 MMA issue, 4 producer (5-7 idle), 8-11 expand, 12-19 epilogue
constexpr int TC_STAGES = 6;
constexpr int TC_ROWS = 128, TC_COLS = 64;
constexpr int TC_WQ = 8 * 1024, TC_WD = 8 * 128, TC_BH = 8 * 1024, TC_BL = 8 * 1024, TC_BS = 8 * 256;
constexpr int TC_OFF_WD = TC_WQ, TC_OFF_BH = TC_OFF_WD + TC_WD, TC_OFF_BL = TC_OFF_BH + TC_BH, TC_OFF_BS = TC_OFF_BL + TC_BL;
constexpr int TC_STAGE = TC_OFF_BS + TC_BS;   // 27648 = 27 * 1024: every stage starts on a swizzle-pattern boundary
constexpr int TC_BAR_OFFSET = TC_STAGES * TC_STAGE;
constexpr int TC_ACC = 6;    // accumulator tiles (one block each, 64 TMEM columns)
constexpr int TC_ABUF = 4;   // A buffers (the 4 blocks of a group each, 32 TMEM columns)
constexpr int TC_ISSUE_WARPS = 4, TC_EXP_WARPS = 4, TC_EPI_WARPS = 8;
// barriers (8 bytes each)
constexpr int BAR_FULL = 0, BAR_EMPTY = TC_STAGES, BAR_A_FULL = 2 * TC_STAGES, BAR_A_FREE = BAR_A_FULL + TC_ABUF, BAR_ACC_FULL = BAR_A_FREE + TC_ABUF,
              BAR_ACC_FREE = BAR_ACC_FULL + TC_ACC, BAR_DRAIN = BAR_ACC_FREE + TC_ACC, TC_N_BARS = BAR_DRAIN + TC_ISSUE_WARPS;
constexpr int TC_SMEM = TC_BAR_OFFSET + TC_N_BARS * 8 + 32;
constexpr uint32_t TC_A_COL = 64 * TC_ACC;   // TMEM columns 0..383: accumulators, 384..511: A buffers

struct TcMaps {
    CUtensorMap wq, wd, bh, bl, bs;
};

__device__ __forceinline__ uint64_t tc_pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t tc_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// K-major, no swizzle: core matrices of 8 rows x 16 bytes; lbo = byte step between the two core matrices along K,
// sbo = byte step between 8-row groups
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t) ((addr >> 4) & 0x3FFF) | ((uint64_t) ((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t) ((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ bool tc_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait of a whole (converged) warp.  A barrier operation costs the issuing warp more than a hundred cycles even
// when the phase is already complete, and those cycles add up within a warp, so a warp that needs several barriers at once
// hands one to each of its first lanes: lane i < n waits for (bar[i], parity[i]), the others pass true.  false = gave up
// (or the CTA already gave up elsewhere).
__device__ __forceinline__ bool tc_wait_lanes(bool mine, uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t limit) {
    bool ok = !mine || tc_try(bar, parity);
    if (__all_sync(0xffffffffu, ok)) return true;
    for (uint32_t i = 0; i < limit; ++i) {
        if (!ok) ok = tc_try(bar, parity);
        if (__all_sync(0xffffffffu, ok)) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(&g_tc_error, 1);
    return false;
}
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t limit) {
    return tc_wait_lanes(true, bar, parity, abort_flag, limit);
}
__device__ __forceinline__ void tc_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_tma_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem], 128 x 64 x 32, e4m3 x e4m3 -> f32
__device__ __forceinline__ void tc_mma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

#define TC_REGS16(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7]), \
                        "=r"(r[o + 8]), "=r"(r[o + 9]), "=r"(r[o + 10]), "=r"(r[o + 11]), "=r"(r[o + 12]), "=r"(r[o + 13]), "=r"(r[o + 14]), "=r"(r[o + 15])
// 16 TMEM lanes x 32 columns in the mma C-fragment order: r[4k + 0,1] = (lane g, columns 8k + 2t, + 1), r[4k + 2,3] = (lane g + 8, same)
#define TC_LD_16x32(r, o, taddr)                                                                                                  \
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n" \
                 : TC_REGS16(r, o) : "r"(taddr))

// debugging switches in `mode`: bit 0 no MMAs, bit 1 no scaling FMAs, bit 2 no accumulator reads, bit 3 no weight expansion,
// bits 4-6 leave out the activation planes / the packed weights / the scale planes of every copy
__global__ void __launch_bounds__(TC_THREADS, 1) mmq_tc_q4_kernel(const __grid_constant__ TcMaps maps, TiledDims dims, ActDims act,
                                                               float *__restrict__ dst, int64_t dst_nb_row,
                                                               float *__restrict__ partial, int ksplit, int mode) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t smem_u32 = (uint32_t) __cvta_generic_to_shared(smem);
    const uint32_t bars = smem_u32 + TC_BAR_OFFSET;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + TC_BAR_OFFSET + TC_N_BARS * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);
#define BAR(which, i) (bars + 8u * (uint32_t) ((which) + (i)))

    const int cta_rt0 = blockIdx.x * 8;
    const int cta_nt0 = blockIdx.y * 8;
    const int ks = blockIdx.z;
    const int per = (int) ((dims.n_bg + ksplit - 1) / ksplit);
    const int bg_begin = ks * per;
    const int bg_end = min((int) dims.n_bg, bg_begin + per);
    const int n_iter = max(0, bg_end - bg_begin);
    const uint32_t spin_limit = g_tc_spin_limit;

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < TC_N_BARS; ++i) {
            // empty: the issuing warps' commits (activation planes read), the expanding warps (packed weights read), the epilogue warps (scales read)
            const int count = (i >= BAR_EMPTY && i < BAR_A_FULL)            ? TC_ISSUE_WARPS + TC_EXP_WARPS + TC_EPI_WARPS
                            : (i >= BAR_A_FULL && i < BAR_A_FREE)            ? TC_EXP_WARPS
                            : (i >= BAR_A_FREE && i < BAR_ACC_FULL)          ? TC_ISSUE_WARPS
                            : (i >= BAR_ACC_FREE && i < BAR_DRAIN)           ? TC_EPI_WARPS : 1;
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(BAR(0, i)), "r"(count));
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {   // all 512 columns (the CTA is alone on its SM)
        const uint32_t slot = (uint32_t) __cvta_generic_to_shared(tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(slot) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    pdl_prologue();   // everything above touches no global memory

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;\n");
        // ---------------- MMA issue: warp w issues block w of every group, so the four accumulator tiles in flight turn over independently ----------------
        const int j = warp;
        const uint32_t idesc = (1u << 4) | ((uint32_t) (TC_COLS >> 3) << 17) | ((uint32_t) (TC_ROWS >> 4) << 24);   // e4m3 x e4m3 -> f32, K-major both
        const uint64_t bh0 = tc_smem_desc(smem_u32 + TC_OFF_BH + j * 256, 128, 1024), bl0 = tc_smem_desc(smem_u32 + TC_OFF_BL + j * 256, 128, 1024);
        int ti = j % TC_ACC, tpar = 0;   // accumulator tile of block 4 it + j and the parity of its use count
        for (int it = 0; it < n_iter; ++it) {
            const int s = it % TC_STAGES, ab = it % TC_ABUF;
            // lane 0: the stage has landed; lane 1: the expanded weights are in TMEM; lane 2: the accumulator tile has been read
            const uint32_t wbar = lane == 0 ? BAR(BAR_FULL, s) : lane == 1 ? BAR(BAR_A_FULL, ab) : BAR(BAR_ACC_FREE, ti);
            const uint32_t wpar = lane == 0 ? (uint32_t) ((it / TC_STAGES) & 1) : lane == 1 ? (uint32_t) ((it / TC_ABUF) & 1) : (uint32_t) (tpar ^ 1);
            if (!tc_wait_lanes(lane < 3, wbar, wpar, abort_flag, spin_limit)) break;
            if (warp == 0) TC_PROF(2, it);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (lane == 0) {
                if (mode & 1) {
                    tc_arrive(BAR(BAR_ACC_FULL, ti)); tc_arrive(BAR(BAR_A_FREE, ab)); tc_arrive(BAR(BAR_EMPTY, s));
                } else {
                    const uint64_t st16 = (uint64_t) ((s * TC_STAGE) >> 4);
                    const uint32_t d_t = tmem + 64u * (uint32_t) ti, a_t = tmem + TC_A_COL + 32u * ab + 8u * j;
                    tc_mma_f8_ts(d_t, a_t, bh0 + st16, idesc, 0u);
                    tc_mma_f8_ts(d_t, a_t, bl0 + st16, idesc, 1u);
                    tc_commit(BAR(BAR_ACC_FULL, ti)); tc_commit(BAR(BAR_A_FREE, ab)); tc_commit(BAR(BAR_EMPTY, s));
                }
            }
            __syncwarp();
            ti += 4;
            if (ti >= TC_ACC) { ti -= TC_ACC; tpar ^= 1; }
        }
        if (lane == 0) {   // no MMA of this CTA may be in flight when its tensor memory is freed, whatever happened elsewhere
            tc_commit(BAR(BAR_DRAIN, warp));
            for (uint32_t spin = 0; spin < TC_DRAIN_LIMIT && !tc_try(BAR(BAR_DRAIN, warp), 0); ++spin) {}
        }
        __syncwarp();
    } else if (warp < 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;\n");
        if (warp == 4) {
            // ---------------- producer: lanes 0..4 = the five tensor copies of a stage ----------------
            const CUtensorMap *map = lane == 0 ? &maps.wq : lane == 1 ? &maps.wd : lane == 2 ? &maps.bh : lane == 3 ? &maps.bl : &maps.bs;
            const uint32_t dst_off = lane == 0 ? 0 : lane == 1 ? TC_OFF_WD : lane == 2 ? TC_OFF_BH : lane == 3 ? TC_OFF_BL : TC_OFF_BS;
            int issued = 0;
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % TC_STAGES, n = it / TC_STAGES;
                if (!tc_wait_lanes(lane == 0, BAR(BAR_EMPTY, s), (uint32_t) ((n & 1) ^ 1), abort_flag, spin_limit)) break;
                TC_PROF(0, it);
                const uint32_t tx = TC_STAGE - ((mode & 16) ? TC_BH + TC_BL : 0) - ((mode & 32) ? TC_WQ : 0) - ((mode & 64) ? TC_WD + TC_BS : 0);
                if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(BAR(BAR_FULL, s)), "r"(tx) : "memory");
                __syncwarp();
                const int bg = bg_begin + it;
                const uint32_t to = smem_u32 + s * TC_STAGE + dst_off;
                if (lane == 0) { if (!(mode & 32)) tc_tma_3d(to, map, 0, bg * 8, cta_rt0, BAR(BAR_FULL, s)); }      // rows / columns past the end read as zero
                else if (lane == 1) { if (!(mode & 64)) tc_tma_2d(to, map, bg * 32, cta_rt0, BAR(BAR_FULL, s)); }
                else if (lane < 4) { if (!(mode & 16)) tc_tma_2d(to, map, bg * 256, cta_nt0, BAR(BAR_FULL, s)); }
                else if (lane == 4) { if (!(mode & 64)) tc_tma_2d(to, map, bg * 64, cta_nt0, BAR(BAR_FULL, s)); }
                issued = it + 1;
            }
            // copies in flight must land before the CTA may exit, whatever happened elsewhere
            for (int it = max(0, issued - TC_STAGES); it < issued && lane == 0; ++it) {
                const uint32_t bar = BAR(BAR_FULL, it % TC_STAGES), parity = (uint32_t) ((it / TC_STAGES) & 1);
                for (uint32_t spin = 0; spin < TC_DRAIN_LIMIT && !tc_try(bar, parity); ++spin) {}
            }
            __syncwarp();
        }
    } else if (warp < 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;\n");
        // ---------------- expand: thread = weight row m of the CTA's 128 ----------------
        const int m = tid - 256;
        const int tile = m >> 4, hrow = (m >> 3) & 1, g = m & 7;
        // the 128-byte line of (tile, g) holds the 16-byte chunks 2t + hrow = word t of blocks 0..3 of row g + 8 hrow; the TMA
        // swizzle stores chunk c at position c ^ (line & 7) = c ^ g
        const uint32_t line = smem_u32 + (uint32_t) ((tile * 8 + g) * 128);
        uint32_t chunk[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) chunk[t] = (uint32_t) (((2 * t + hrow) ^ g) * 16);
        const uint32_t a_lane = tmem + ((uint32_t) (32 * (warp - 8)) << 16) + TC_A_COL;
        for (int it = 0; it < n_iter; ++it) {
            const int s = it % TC_STAGES, ab = it % TC_ABUF;
            const uint32_t wbar = lane == 0 ? BAR(BAR_FULL, s) : BAR(BAR_A_FREE, ab);
            const uint32_t wpar = lane == 0 ? (uint32_t) ((it / TC_STAGES) & 1) : (uint32_t) (((it / TC_ABUF) & 1) ^ 1);
            if (!tc_wait_lanes(lane < 2, wbar, wpar, abort_flag, spin_limit)) break;
            if (warp == 8) TC_PROF(1, it);
            uint32_t r[4][4];   // r[t][j] = word t of block j
#pragma unroll
            for (int t = 0; t < 4; ++t)
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[t][0]), "=r"(r[t][1]), "=r"(r[t][2]), "=r"(r[t][3]) : "r"(line + s * TC_STAGE + chunk[t]));
            __syncwarp();
            if (lane == 0) tc_arrive(BAR(BAR_EMPTY, s));   // the packed weights of this stage are in registers (the arrive orders the loads before it)
            if (!(mode & 8)) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t a[16];     // a[8 jj + c]: bytes 4c..4c+3 of the row of block 2h + jj, element order
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const uint32_t w = r[t][2 * h + jj];
                            a[8 * jj + t] = (w & 0x0F0F0F0Fu) ^ 0x08080808u;              // elements 4t..4t+3: u = q + 8 (the nibbles hold q in two's complement)
                            a[8 * jj + 4 + t] = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;   // elements 16+4t..
                        }
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
                                 ::"r"(a_lane + 32u * ab + 16u * h), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]),
                                 "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]) : "memory");
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_arrive(BAR(BAR_A_FULL, ab));
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 152;\n");
        // -------- epilogue: rows 32 q + {g, g+8, g+16, g+24}, column pairs 32 cg + 8 k + 2 t (k < 4) --------
        const int q = warp & 3, cg = (warp - 12) >> 2, g = lane >> 2, t = lane & 3;
        uint64_t y[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int k = 0; k < 4; ++k) y[r][k] = 0ull;
        const uint32_t t_lo = tmem + ((uint32_t) (32 * q) << 16) + 32u * cg, t_hi = t_lo + (16u << 16);

        uint32_t c0[32], c1[32];   // the accumulator tiles of an even / odd block: [0..15] rows g, g+8, [16..31] rows g+16, g+24
        // y += d_w * (D * v + C) for one block: v = 2^-18 sum(u a), D = d_a 2^18, C = -8 d_a sum(a)
        auto scale_block = [&](const uint32_t (&cc)[32], const uint8_t *sj, const uint64_t (&dw)[4]) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint4 sc = *reinterpret_cast<const uint4 *>(sj + k * 256);   // {D0, D1, C0, C1} of columns 8k + 2t, + 1
                const uint64_t da = tc_pack2(sc.x, sc.y), ca = tc_pack2(sc.z, sc.w);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int i = (r >> 1) * 16 + 4 * k + 2 * (r & 1);
                    const uint64_t tt = tc_fma2(tc_pack2(cc[i], cc[i + 1]), da, ca);
                    y[r][k] = tc_fma2(tt, dw[r], y[r][k]);
                }
            }
        };
        auto dw_of = [&](const uint2 (&h4)[4], int j, uint64_t (&dw)[4]) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const uint32_t h = (j < 2) ? h4[r].x : h4[r].y;
                const __half2 h2 = *reinterpret_cast<const __half2 *>(&h);
                const uint32_t uu = __float_as_uint((j & 1) ? __high2float(h2) : __low2float(h2));
                dw[r] = tc_pack2(uu, uu);
            }
        };
        int ti = 0, tpar = 0;   // accumulator tile of the block being loaded (or the next to be loaded) and the parity of its use count
        bool ok = n_iter > 0 && tc_wait(BAR(BAR_ACC_FULL, 0), 0u, abort_flag, spin_limit);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (mode & 4) {
#pragma unroll
                for (int i = 0; i < 32; ++i) c0[i] = c1[i] = 0u;
            } else {
                TC_LD_16x32(c0, 0, t_lo); TC_LD_16x32(c0, 16, t_hi);
            }
        }
        for (int it = 0; ok && it < n_iter; ++it) {
            const int s = it % TC_STAGES;
            if (warp == 12) TC_PROF(3, it);
            const uint8_t *st = smem + s * TC_STAGE;
            // weight scales: fp16 at 4*row + block within a tile's 128 bytes; rows {g, g+8} of tiles 2q and 2q + 1
            const uint2 *sa = reinterpret_cast<const uint2 *>(st + TC_OFF_WD + (2 * q) * 128);
            const uint2 h4[4] = {sa[g], sa[g + 8], sa[16 + g], sa[24 + g]};
            const uint8_t *Ss = st + TC_OFF_BS + (4 * cg) * 256 + t * 16;
            uint64_t dw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // block j of this group sits in c0 (j even) or c1 (j odd); it is complete after this wait: hand its tile back
                if (!(mode & 4)) asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) tc_arrive(BAR(BAR_ACC_FREE, ti));
                if (++ti == TC_ACC) { ti = 0; tpar ^= 1; }
                // start reading the next block's tile before this one is scaled
                if (j < 3 || it + 1 < n_iter) {
                    ok = tc_wait(BAR(BAR_ACC_FULL, ti), (uint32_t) tpar, abort_flag, spin_limit);
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    if (!ok) break;
                    const uint32_t a = 64u * (uint32_t) ti;
                    if (!(mode & 4)) {
                        if (j & 1) { TC_LD_16x32(c0, 0, t_lo + a); TC_LD_16x32(c0, 16, t_hi + a); }
                        else { TC_LD_16x32(c1, 0, t_lo + a); TC_LD_16x32(c1, 16, t_hi + a); }
                    }
                }
                if (!(mode & 2)) {
                    dw_of(h4, j, dw);
                    if (j & 1) scale_block(c1, Ss + j * 64, dw);
                    else scale_block(c0, Ss + j * 64, dw);
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) tc_arrive(BAR(BAR_EMPTY, s));
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        // write back
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int64_t row = (int64_t) blockIdx.x * TC_ROWS + 32 * q + 8 * r + g;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int64_t col = (int64_t) cta_nt0 * 8 + 32 * cg + 8 * k + 2 * t;
                uint32_t lo, hi;
                asm("mov.b64 {%0,%1}, %2;" : "=r"(lo), "=r"(hi) : "l"(y[r][k]));
                const float v0 = __uint_as_float(lo), v1 = __uint_as_float(hi);
                if (row < dims.M) {
                    if (ksplit == 1) {
                        if (col < act.N) *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + col * dst_nb_row + row * 4) = v0;
                        if (col + 1 < act.N) *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + (col + 1) * dst_nb_row + row * 4) = v1;
                    } else {
                        if (col < act.N) partial[((int64_t) ks * act.N + col) * dims.M + row] = v0;
                        if (col + 1 < act.N) partial[((int64_t) ks * act.N + col + 1) * dims.M + row] = v1;
                    }
                }
            }
        }
    }
#undef BAR
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}

static int tc_sm_count() {   // every device of a process is the same model
    static const int n = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

// ---- tensor maps ----
typedef CUresult (*tc_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static tc_encode_fn tc_encoder() {
    static tc_encode_fn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) p = nullptr;
        return (tc_encode_fn) p;
    }();
    return fn;
}
// 2-D view: rows of `inner_words` 32-bit words, a box of box_words x 8 rows
static bool tc_encode(CUtensorMap *m, const void *base, uint64_t inner_words, uint64_t rows, uint32_t box_words) {
    tc_encode_fn enc = tc_encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {inner_words, rows};
    const cuuint64_t strides[1] = {inner_words * 4};
    const cuuint32_t box[2] = {box_words, 8};
    const cuuint32_t elem[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// The packed weight tiles as lines of 128 bytes (8 lines per tile): [row tile][block group * 8 + line][32 words], a box of
// 8 row tiles x one block group's 8 lines, written with the 128-byte swizzle (16-byte chunk c of line l at c ^ (l & 7)).
static bool tc_encode_wq(CUtensorMap *m, const void *base, uint64_t n_bg, uint64_t n_rt) {
    tc_encode_fn enc = tc_encoder();
    if (!enc) return false;
    const cuuint64_t dims[3] = {32, n_bg * 8, n_rt};
    const cuuint64_t strides[2] = {128, n_bg * 1024};
    const cuuint32_t box[3] = {32, 8, 8};
    const cuuint32_t elem[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// encoded maps are pure functions of (pointer, extents): keep them, a model has a few hundred weights
struct TcKey {
    const void *p;
    int64_t a, b;
    bool operator==(const TcKey &o) const { return p == o.p && a == o.a && b == o.b; }
};
struct TcKeyHash {
    size_t operator()(const TcKey &k) const { return std::hash<const void *>()(k.p) ^ (size_t) (k.a * 0x9E3779B97F4A7C15ull) ^ (size_t) (k.b * 0xC2B2AE3D27D4EB4Full); }
};
struct TcWeightMaps { CUtensorMap q, d; };
struct TcActMaps { CUtensorMap h, l, s; };
static bool tc_weight_maps(const TiledDims &d, const void *w, TcWeightMaps *out) {
    static std::mutex mu;
    static std::unordered_map<TcKey, TcWeightMaps, TcKeyHash> cache;
    const TcKey key{w, d.n_rt, d.n_bg};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        TcWeightMaps p;
        if (!tc_encode_wq(&p.q, w, (uint64_t) d.n_bg, (uint64_t) d.n_rt)) return false;
        if (!tc_encode(&p.d, (const uint8_t *) w + d.qs_bytes, (uint64_t) d.n_bg * 32, (uint64_t) d.n_rt, 32)) return false;
        if (cache.size() > 65536) cache.clear();
        it = cache.emplace(key, p).first;
    }
    *out = it->second;
    return true;
}
static bool tc_act_maps(const ActDims &a, const void *aq, TcActMaps *out) {
    static std::mutex mu;
    static std::unordered_map<TcKey, TcActMaps, TcKeyHash> cache;
    const TcKey key{aq, a.n_nt, a.n_bg};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        TcActMaps p;
        if (!tc_encode(&p.h, (const uint8_t *) aq + a.hi_offset, (uint64_t) a.nbp * 64, (uint64_t) a.n_nt, 256)) return false;
        if (!tc_encode(&p.l, (const uint8_t *) aq + a.lo_offset, (uint64_t) a.nbp * 64, (uint64_t) a.n_nt, 256)) return false;
        if (!tc_encode(&p.s, (const uint8_t *) aq + a.s2_offset, (uint64_t) a.n_bg * 64, (uint64_t) a.n_nt, 64)) return false;
        if (cache.size() > 65536) cache.clear();
        it = cache.emplace(key, p).first;
    }
    *out = it->second;
    return true;
}

int launch_mmq_tc(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
                  void *workspace, size_t workspace_bytes, cudaStream_t st) {
    TcWeightMaps wm;
    TcActMaps am;
    if (wtype != B200_TYPE_Q4_0 || a.hi_offset == 0 || !is_aligned(w, 16) || !is_aligned(aq, 16) || !tc_weight_maps(d, w, &wm) || !tc_act_maps(a, aq, &am)) {
        return launch_mmq(wtype, d, w, a, aq, dst, dst_nb_row, workspace, workspace_bytes, st, false, PeerDst{});
    }
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(mmq_tc_q4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        if (e != cudaSuccess) return set_error(B200_E_CUDA, "mmq_tc shared memory opt-in: %s", cudaGetErrorString(e));
        configured[dev & 63] = true;
    }
    static const int mode = [] {   // debugging switches, see the kernel
        const char *e = getenv("B200_TC_DEBUG");
        return e ? atoi(e) : 0;
    }();
    TcMaps maps;
    maps.wq = wm.q; maps.wd = wm.d; maps.bh = am.h; maps.bl = am.l; maps.bs = am.s;
    const int64_t row_groups = (d.n_rt + 7) / 8, col_chunks = (a.n_nt + 7) / 8;
    // K splits: whole waves of one CTA per SM, a few block groups of fixed cost per split
    const int64_t ctas = row_groups * col_chunks, slots = (int64_t) tc_sm_count();
    int ks = 1;
    int64_t best = -1;
    for (int k = 1; k <= 16; ++k) {
        const int64_t per = (d.n_bg + k - 1) / k;
        if (k > 1 && per < 2) break;
        const int64_t cost = ((ctas * k + slots - 1) / slots) * (per + 3) + (k > 1 ? 2 : 0);
        if (best < 0 || cost < best) { best = cost; ks = k; }
    }
    const size_t per_split = (size_t) a.N * d.M * sizeof(float);
    if (ks > 1 && (!workspace || workspace_bytes < per_split * ks)) ks = workspace ? (int) std::max<size_t>(1, workspace_bytes / per_split) : 1;
    dim3 grid((unsigned) row_groups, (unsigned) col_chunks, (unsigned) ks);
    cudaError_t le = launch_pdl(mmq_tc_q4_kernel, grid, dim3(TC_THREADS), (size_t) TC_SMEM, st, maps, d, a, dst, dst_nb_row, (float *) workspace, ks, mode);
    if (le != cudaSuccess) return set_error(B200_E_CUDA, "mmq_tc launch: %s", cudaGetErrorString(le));
    if (int e = check_launch("mmq_tc")) return e;
    if (ks > 1) {
        launch_mmq_reduce((const float *) workspace, ks, d.M, a.N, dst, dst_nb_row, st);
        return check_launch("mmq_reduce");
    }
    return B200_OK;
}

int tc_error_flag() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
    return v;
}
void tc_set_wait_limit(unsigned rounds) {
    const unsigned v = rounds ? rounds : 1u << 20;
    const int zero = 0;
    cudaMemcpyToSymbol(g_tc_spin_limit, &v, sizeof(v));
    cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(zero));
}

}  // namespace b200

namespace b200 { int tcf_error_flag(); void tcf_set_wait_limit(unsigned rounds); }
extern "C" B200_API int b200_kernel_status(void) { return b200::tc_error_flag() | (b200::tcf_error_flag() << 1); }
extern "C" B200_API void b200_kernel_set_wait_limit(unsigned rounds) {
    b200::tc_set_wait_limit(rounds);
    b200::tcf_set_wait_limit(rounds);
}
#ifdef B200_TC_PROFILE
extern "C" B200_API void b200_tc_profile(long long *out) { cudaMemcpyFromSymbol(out, b200::g_tc_prof, sizeof(long long) * 256); }
#endif
