// MUL_MAT for a batch of activation columns on the 5th-generation tensor cores, with the block scales folded into
// the operands so that one accumulator in tensor memory runs over the whole of K.
//
// lm_ggml_compute_forward_mul_mat (cactus/ggml-cpu/ggml-cpu.c:1257-1449) computes, per output value,
// sum over blocks b of d_w[row, b] * d_a[col, b] * dot_b with dot_b an integer.  Scaling after every block (mmq.cu,
// mmq_tc.cu) costs a pass over the accumulator tile per 32 values of K; here the scales go into the operands instead:
//   A[row, k] = d_w[row, b] * q[row, k]      (15 significant bits: 11 of the fp16 scale, 4 of the quant)
//   B[col, k] = d_a[col, b] * a[col, k]      (19 significant bits)
// Each is split into an fp16 value and the exact fp16 remainder (x_hi = rn(x), x_lo = x - x_hi, both fp16: the
// remainder of a product of an fp16 and a small integer always fits), and the product is
//   A_hi B_hi + A_hi B_lo + A_lo B_hi       (the missing A_lo B_lo is below 2^-22 of a term)
// accumulated in fp32 by tcgen05.mma.kind::f16.  Per 16 values of K that is one MMA of 128 x 128 (A_hi against the B_hi
// and B_lo planes stacked along N, two accumulator halves that the write-back adds) and one of 128 x 64 (A_lo against
// B_hi, into the first half).  Nothing is rounded that the reference does not round, except the order of the fp32 sums.
//
// A CTA (one per SM) owns 128 weight rows x 64 activation columns (up to 64 columns in all) or x 128 (more) and walks K in
// groups of 4 blocks.  A hand-over between warps costs a few hundred cycles whatever the mechanism, so the converting
// roles are held by several teams that take the groups in turn, one team per buffer of its ring (TfCfg):
//   warp 0       issues the MMAs of every group, in order (8 K-steps x 2), into the one accumulator;
//   warp 1       producer: four TMA tensor copies per group into a ring of stages -- the packed T16 weight tiles (128-byte
//                swizzle, so the row-per-thread reads are conflict free), their fp16 scales, the Q8_0 activation tiles in
//                the fragment order every mul_mat kernel reads, and the activation scales;
//   warps 4-15   weights, teams of 4 warps (as many as A buffers fit into tensor memory): thread = weight row; unpacks 128
//                nibbles with the 0x6400 trick (0x6400 | v is the fp16 1024 + v), multiplies by the block scale and writes
//                A_hi and A_lo straight into tensor memory (the MMA's A operand); after the last group two teams read
//                the accumulator (half of the columns each) and write the result;
//   warps 16-..  activations, teams of 4 or 8 warps: int8 -> fp16 (same trick), times the block scale, hi and lo planes
//                into a ring of shared memory tiles in the K-major core-matrix order of the MMA's B descriptor.
// Measured (B200, K 4096 x M 14336): 45.6 us at 64 columns with three terms, 35.3 with two, against 33.1 for the mma.sync
// kernel; at 128 columns 60.5 / 44.5 against 56.9.  The conversions cost 2300-3000 warp instructions per group on the CUDA
// cores, more than the group's HBM time, and they slow the issuing thread (103 clk per 128 x 128 x 16 MMA against 64.5 in
// isolation); the kernel is therefore opt-in (B200_MMQ_TC=2 three terms, =3 two).
// Within a block both operands use the same permutation of K (the order the nibbles come out of a 32-bit word).
// Every wait is bounded; on time-out the CTA raises b200_kernel_status, all roles fall through, the producer waits
// (bounded) for its copies in flight, the issuing warp for its MMAs, the CTA frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace b200 {

void launch_mmq_reduce(const float *partial, int ks, int64_t M, int64_t N, float *dst, int64_t dst_nb_row, cudaStream_t st);
int launch_mmq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
               void *workspace, size_t workspace_bytes, cudaStream_t st, bool canon, const PeerDst &peers);

__device__ int g_tcf_error = 0;                    // non-zero after a bounded wait gave up
__device__ unsigned g_tcf_spin_limit = 1u << 20;   // try_wait rounds before a wait gives up (each may suspend for a while)
constexpr uint32_t TF_DRAIN_LIMIT = 1u << 22;      // what a CTA that gave up still waits for: its own copies and MMAs in flight

#ifdef B200_TC_PROFILE
__device__ long long g_tcf_prof[8][64];   // [event][iteration]: clock of CTA 0
#define TF_PROF(ev, it) do { if (blockIdx.x == 0 && blockIdx.z == 0 && lane == 0 && (it) < 64) g_tcf_prof[ev][it] = clock64(); } while (0)
#else
#define TF_PROF(ev, it) do { } while (0)
#endif

constexpr int TF_ROWS = 128;
constexpr int TF_MAX_STAGES = 5, TF_MAX_BUF = 3;
// barriers (8 bytes each); rings are sized for the larger configuration
constexpr int TFB_FULL = 0, TFB_EMPTY = TF_MAX_STAGES, TFB_A_FULL = 2 * TF_MAX_STAGES, TFB_A_FREE = TFB_A_FULL + TF_MAX_BUF, TFB_B_FULL = TFB_A_FREE + TF_MAX_BUF,
              TFB_B_FREE = TFB_B_FULL + TF_MAX_BUF, TFB_ACC = TFB_B_FREE + TF_MAX_BUF, TFB_DRAIN = TFB_ACC + 1, TF_N_BARS = TFB_DRAIN + 1;

// Geometry of a CTA that owns 128 weight rows x NT tiles of 8 activation columns (NT 8: the width of a decode ubatch;
// NT 16: prefill -- the weights are converted once per 128 columns and the MMAs are twice as wide).
template <int NT, int TERMS>
struct TfCfg {
    static constexpr int NCH = 8 * NT;                      // activation columns of the CTA
    static constexpr int STAGES = NT == 8 ? 5 : 3;
    static constexpr int WQ = 8 * 1024, WD = 8 * 128, BQ = NT * 1024, BS = NT * 256;
    static constexpr int OFF_WD = WQ, OFF_BQ = OFF_WD + WD, OFF_BS = OFF_BQ + BQ;
    static constexpr int STAGE = OFF_BS + BS;               // 19 or 29 KiB: every stage starts on a swizzle-pattern boundary
    static constexpr int KSTEP = 2 * NT * 256;              // B tile of one K-step: NT column groups of the hi plane, NT of the lo plane, 256 bytes each
    static constexpr int BTILE = 8 * KSTEP;
    // TMEM: the accumulator takes 2 NCH columns (hi-hi + lo-hi | hi-lo), A buffers of 64 (A_hi) or 128 (A_hi, A_lo) columns the rest
    static constexpr uint32_t A_COL = 2 * NCH;
    static constexpr uint32_t A_STRIDE = TERMS >= 3 ? 128 : 64;
    static constexpr int ABUF = (512 - (int) A_COL) / (int) A_STRIDE > TF_MAX_BUF ? TF_MAX_BUF : (512 - (int) A_COL) / (int) A_STRIDE;
    static constexpr int BBUF = NT == 8 ? 3 : 2;
    static constexpr int ACT_WARPS = NT / 2;                // warps of an activation team: 2 column tiles each
    static constexpr int THREADS = 32 * (16 + BBUF * ACT_WARPS);   // 4 control warps, 12 weight warps (4 ABUF at work), the activation teams
    // registers: the launch gives every thread BASE; the roles then trade (an increase waits until the registers exist, so the
    // budgets must fit the CTA's allocation)
    static constexpr int BASE_REGS = THREADS == 1024 ? 64 : 72;
    static constexpr int W_REGS = TERMS >= 3 ? 88 : 80;
    static constexpr int A_REGS = NT == 8 ? (TERMS >= 3 ? 64 : 72) : 56;
    static constexpr int IDLE_WARPS = 12 - 4 * ABUF;
    static_assert(4 * 32 * 48 + 4 * ABUF * 32 * W_REGS + IDLE_WARPS * 32 * BASE_REGS + BBUF * ACT_WARPS * 32 * A_REGS <= THREADS * BASE_REGS,
                  "register budget of the roles exceeds the CTA's allocation");
    static constexpr int OFF_B = STAGES * STAGE;
    static constexpr int BAR_OFFSET = OFF_B + BBUF * BTILE;
    static constexpr int SMEM = BAR_OFFSET + TF_N_BARS * 8 + 32;
    static_assert(STAGE % 1024 == 0, "stages start on swizzle-pattern boundaries");
    static_assert(ABUF >= 2 && ABUF * 4 <= 12 && THREADS <= 1024 && THREADS * BASE_REGS <= 65536, "teams must fit the CTA");
    static_assert(SMEM <= 232448, "shared memory of an SM");
};

struct TfMaps {
    CUtensorMap wq, wd, bq, bs;
};

__device__ __forceinline__ uint64_t tf_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t) ((addr >> 4) & 0x3FFF) | ((uint64_t) ((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t) ((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ bool tf_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait of a whole (converged) warp; lane i < n waits for its own (bar, parity), the others pass true -- a barrier
// operation costs the issuing warp over a hundred cycles even when the phase is complete, so a warp that needs several
// barriers hands one to each of its first lanes.  false = gave up (or the CTA already gave up elsewhere).
__device__ __forceinline__ bool tf_wait_lanes(bool mine, uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t limit) {
    bool ok = !mine || tf_try(bar, parity);
    if (__all_sync(0xffffffffu, ok)) return true;
    for (uint32_t i = 0; i < limit; ++i) {
        if (!ok) ok = tf_try(bar, parity);
        if (__all_sync(0xffffffffu, ok)) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(&g_tcf_error, 1);
    return false;
}
__device__ __forceinline__ void tf_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tf_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tf_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tf_tma_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem], M 128, K 16, fp16 x fp16 -> f32; N comes with the instruction descriptor
__device__ __forceinline__ void tf_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ uint32_t tf_h2(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 tf_as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

#define TF_ST16(taddr, a)                                                                                                              \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"          \
                 ::"r"(taddr), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]), \
                 "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]) : "memory")
#define TF_LD16(r, taddr)                                                                                                          \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"      \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), \
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(taddr))

// TERMS 3: A_hi B_hi + A_hi B_lo + A_lo B_hi (exact to fp32 rounding); TERMS 2 leaves out A_lo B_hi (the weights
// rounded to fp16: 2^-12 relative per term), kept for measurements.
// debugging switches in `mode`: 1 no activation stores, 2 no weight stores, 4 no MMAs, 8 / 16 no activation / weight arithmetic,
// 32 the producer copies nothing (every consumer wait then runs into its limit: the test of the give-up path)
template <int NT, int TERMS>
__global__ void __launch_bounds__((TfCfg<NT, TERMS>::THREADS), 1) mmq_tcf_kernel(const __grid_constant__ TfMaps maps, TiledDims dims, ActDims act,
                                                              float *__restrict__ dst, int64_t dst_nb_row,
                                                              float *__restrict__ partial, int ksplit, int mode) {
    using C = TfCfg<NT, TERMS>;
    // Every ring of buffers has as many teams as buffers and team i owns buffer i; one warp issues all MMAs in order.  Each
    // barrier is then waited for by one warp (or team) phase after phase, which a parity wait can tell apart (a waiter two
    // phases ahead could not).
    constexpr int ABUF = C::ABUF, BBUF = C::BBUF, STAGES = C::STAGES;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t smem_u32 = (uint32_t) __cvta_generic_to_shared(smem);
    const uint32_t bars = smem_u32 + C::BAR_OFFSET;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + C::BAR_OFFSET + TF_N_BARS * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);
#define BAR(which, i) (bars + 8u * (uint32_t) ((which) + (i)))

    const int cta_rt0 = blockIdx.x * 8;
    const int cta_nt0 = blockIdx.y * NT;
    const int ks = blockIdx.z;
    const int per = (int) ((dims.n_bg + ksplit - 1) / ksplit);
    const int bg_begin = ks * per;
    const int bg_end = min((int) dims.n_bg, bg_begin + per);
    const int n_iter = max(0, bg_end - bg_begin);
    const uint32_t spin_limit = g_tcf_spin_limit;

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < TF_N_BARS; ++i) {
            const int count = (i >= TFB_EMPTY && i < TFB_A_FULL)    ? 4 + C::ACT_WARPS   // a weight team and an activation team have read the stage
                            : (i >= TFB_A_FULL && i < TFB_A_FREE)   ? 4
                            : (i >= TFB_B_FULL && i < TFB_B_FREE)   ? C::ACT_WARPS : 1;
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

    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 48;\n");
    else if (warp < 4 + 4 * ABUF) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(C::W_REGS));
    else if (warp >= 16 && C::A_REGS < C::BASE_REGS) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(C::A_REGS));

    if (warp == 0) {
        // ---------------- MMA issue ----------------
        const uint32_t idesc_wide = (1u << 4) | ((uint32_t) ((2 * C::NCH) >> 3) << 17) | ((uint32_t) (TF_ROWS >> 4) << 24);   // f16 x f16 -> f32, K-major both
        const uint32_t idesc_hi = (1u << 4) | ((uint32_t) (C::NCH >> 3) << 17) | ((uint32_t) (TF_ROWS >> 4) << 24);
        // B tile: per K-step 2 NT groups of 8 columns (the hi plane, then the lo plane), 256 bytes each: two core matrices of
        // 8 columns x 8 values along K
        const uint64_t b0 = tf_smem_desc(smem_u32 + C::OFF_B, 128, 256);
        for (int it = 0; it < n_iter; ++it) {
            const int ab = it % ABUF, bb = it % BBUF;
            const uint32_t wbar = lane == 0 ? BAR(TFB_A_FULL, ab) : BAR(TFB_B_FULL, bb);
            const uint32_t wpar = lane == 0 ? (uint32_t) ((it / ABUF) & 1) : (uint32_t) ((it / BBUF) & 1);
            if (!tf_wait_lanes(lane < 2, wbar, wpar, abort_flag, spin_limit)) break;
            TF_PROF(2, it);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (lane == 0 && (mode & 4)) {
                tf_arrive(BAR(TFB_A_FREE, ab)); tf_arrive(BAR(TFB_B_FREE, bb));
                if (it == n_iter - 1) tf_arrive(BAR(TFB_ACC, 0));
            } else if (lane == 0) {
                const uint32_t a_hi = tmem + C::A_COL + C::A_STRIDE * (uint32_t) ab, a_lo = a_hi + 64u;
                const uint64_t bd = b0 + (uint64_t) ((bb * C::BTILE) >> 4);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    tf_mma(tmem, a_hi + 8u * k, bd + (uint64_t) ((k * C::KSTEP) >> 4), idesc_wide, (it > 0 || k > 0) ? 1u : 0u);
                    if (TERMS >= 3) tf_mma(tmem, a_lo + 8u * k, bd + (uint64_t) ((k * C::KSTEP) >> 4), idesc_hi, 1u);
                }
                TF_PROF(7, it);
                tf_commit(BAR(TFB_A_FREE, ab));
                tf_commit(BAR(TFB_B_FREE, bb));
                if (it == n_iter - 1) tf_commit(BAR(TFB_ACC, 0));
            }
            TF_PROF(6, it);
            __syncwarp();
        }
        if (lane == 0) {   // no MMA of this CTA may be in flight when its tensor memory is freed, whatever happened elsewhere
            tf_commit(BAR(TFB_DRAIN, 0));
            for (uint32_t spin = 0; spin < TF_DRAIN_LIMIT && !tf_try(BAR(TFB_DRAIN, 0), 0); ++spin) {}
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- producer: lanes 0..3 = the four tensor copies of a stage ----------------
        const CUtensorMap *map = lane == 0 ? &maps.wq : lane == 1 ? &maps.wd : lane == 2 ? &maps.bq : &maps.bs;
        const uint32_t dst_off = lane == 0 ? 0 : lane == 1 ? C::OFF_WD : lane == 2 ? C::OFF_BQ : C::OFF_BS;
        int issued = 0;
        for (int it = 0; it < n_iter && !(mode & 32); ++it) {
            const int s = it % STAGES, n = it / STAGES;
            if (!tf_wait_lanes(lane == 0, BAR(TFB_EMPTY, s), (uint32_t) ((n & 1) ^ 1), abort_flag, spin_limit)) break;
            TF_PROF(0, it);
            if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(BAR(TFB_FULL, s)), "r"((uint32_t) C::STAGE) : "memory");
            __syncwarp();
            const int bg = bg_begin + it;
            const uint32_t to = smem_u32 + s * C::STAGE + dst_off;
            if (lane == 0) tf_tma_3d(to, map, 0, bg * 8, cta_rt0, BAR(TFB_FULL, s));      // rows / columns past the end read as zero
            else if (lane == 1) tf_tma_2d(to, map, bg * 32, cta_rt0, BAR(TFB_FULL, s));
            else if (lane == 2) tf_tma_2d(to, map, bg * 256, cta_nt0, BAR(TFB_FULL, s));
            else if (lane == 3) tf_tma_2d(to, map, bg * 64, cta_nt0, BAR(TFB_FULL, s));
            issued = it + 1;
        }
        // copies in flight must land before the CTA may exit, whatever happened elsewhere
        for (int it = max(0, issued - STAGES); it < issued && lane == 0; ++it) {
            const uint32_t bar = BAR(TFB_FULL, it % STAGES), parity = (uint32_t) ((it / STAGES) & 1);
            for (uint32_t spin = 0; spin < TF_DRAIN_LIMIT && !tf_try(bar, parity); ++spin) {}
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 16) {
        // ---------------- weights: thread = weight row m of the CTA's 128; team i takes the groups i, i + ABUF, ... ----------------
        const int team = (warp - 4) >> 2, m = (tid - 128) & 127;
        const int tile = m >> 4, hrow = (m >> 3) & 1, g = m & 7;
        // the 128-byte line of (tile, g) holds the 16-byte chunks 2t + hrow = word t of blocks 0..3 of row g + 8 hrow; the TMA
        // swizzle stores chunk c at position c ^ (line & 7) = c ^ g
        const uint32_t line = smem_u32 + (uint32_t) ((tile * 8 + g) * 128);
        uint32_t chunk[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) chunk[t] = (uint32_t) (((2 * t + hrow) ^ g) * 16);
        const uint32_t lane_base = tmem + ((uint32_t) (32 * (warp & 3)) << 16);
        const uint32_t a_lane = lane_base + C::A_COL;
        const __half2 bias = __half2half2(__float2half_rn(-1032.0f));
        bool ok = true;
        for (int it = team; it < n_iter && team < ABUF; it += ABUF) {
            const int s = it % STAGES, ab = team;
            const uint32_t wbar = lane == 0 ? BAR(TFB_FULL, s) : BAR(TFB_A_FREE, ab);
            const uint32_t wpar = lane == 0 ? (uint32_t) ((it / STAGES) & 1) : (uint32_t) (((it / ABUF) & 1) ^ 1);
            if (!tf_wait_lanes(lane < 2, wbar, wpar, abort_flag, spin_limit)) { ok = false; break; }
            if ((warp & 3) == 0) TF_PROF(1, it);
            uint32_t r[4][4];   // r[t][j] = word t of block j
#pragma unroll
            for (int t = 0; t < 4; ++t)
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[t][0]), "=r"(r[t][1]), "=r"(r[t][2]), "=r"(r[t][3]) : "r"(line + s * C::STAGE + chunk[t]));
            // fp16 scales of the row's 4 blocks: half index 4 * row + block within a tile's 128 bytes
            uint2 dw4;
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(dw4.x), "=r"(dw4.y) : "r"(smem_u32 + (uint32_t) (s * C::STAGE + C::OFF_WD + tile * 128 + (m & 15) * 8)));
            __syncwarp();
            if (lane == 0) tf_arrive(BAR(TFB_EMPTY, s));   // this stage's weights are in registers (the arrive orders the loads before it)
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int j = 0; j < 4 && !(mode & 16); ++j) {
                const uint32_t dbits = (j < 2) ? dw4.x : dw4.y;
                const __half2 d2 = (j & 1) ? __high2half2(tf_as_h2(dbits)) : __low2half2(tf_as_h2(dbits));
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const uint32_t w = r[t][j];
#pragma unroll
                    for (int si = 0; si < 4; ++si) {
                        // the nibbles at bits 4 si and 16 + 4 si hold q in two's complement; v = q + 8
                        const uint32_t x = ((w >> (4 * si)) & 0x000F000Fu) ^ 0x64086408u;
                        const __half2 q2 = __hadd2(tf_as_h2(x), bias);
                        const __half2 h = __hmul2(q2, d2);
                        hi[4 * t + si] = tf_h2(h);
                        if (TERMS >= 3) lo[4 * t + si] = tf_h2(__hfma2(q2, d2, __hneg2(h)));
                    }
                }
                if (!(mode & 2)) {
                    TF_ST16(a_lane + C::A_STRIDE * ab + 16u * j, hi);
                    if (TERMS >= 3) TF_ST16(a_lane + C::A_STRIDE * ab + 64u + 16u * j, lo);
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if ((warp & 3) == 0) TF_PROF(4, it);
            if (lane == 0) tf_arrive(BAR(TFB_A_FULL, ab));
        }
        // ---------------- write-back: the thread owns accumulator lane m; team 0 the first half of the columns, team 1 the second ----------------
        if (team < 2) {
            ok = ok && n_iter > 0 && tf_wait_lanes(lane == 0, BAR(TFB_ACC, 0), 0u, abort_flag, spin_limit);
            const int64_t row = (int64_t) blockIdx.x * TF_ROWS + m;
#pragma unroll 1
            for (int c0 = (C::NCH / 2) * team; c0 < (C::NCH / 2) * (team + 1); c0 += 16) {
                float y[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) y[i] = 0.0f;
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
                    for (int part = 0; part < 2; ++part) {   // hi-hi + lo-hi, then hi-lo
                        uint32_t u[16];
                        TF_LD16(u, lane_base + (uint32_t) (C::NCH * part + c0));
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 16; ++i) y[i] += __uint_as_float(u[i]);
                    }
                }
                if (row < dims.M && (ok || n_iter == 0)) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int64_t col = (int64_t) cta_nt0 * 8 + c0 + i;
                        if (col < act.N) {
                            if (ksplit == 1) *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + col * dst_nb_row + row * 4) = y[i];
                            else partial[((int64_t) ks * act.N + col) * dims.M + row] = y[i];
                        }
                    }
                }
            }
        }
    } else if (warp >= 16 && warp < 16 + BBUF * C::ACT_WARPS) {
        // ---------------- activations: team i takes the groups i, i + BBUF, ...; a warp takes 2 tiles of 8 columns, lane = 8 t + g ----------------
        const int team = (warp - 16) / C::ACT_WARPS, aw = (warp - 16) % C::ACT_WARPS, t = lane >> 3, g = lane & 7;
        const __half2 bias = __half2half2(__float2half_rn(-1152.0f));
        for (int it = team; it < n_iter; it += BBUF) {
            const int s = it % STAGES, bb = team;
            const uint32_t wbar = lane == 0 ? BAR(TFB_FULL, s) : BAR(TFB_B_FREE, bb);
            const uint32_t wpar = lane == 0 ? (uint32_t) ((it / STAGES) & 1) : (uint32_t) (((it / BBUF) & 1) ^ 1);
            if (!tf_wait_lanes(lane < 2, wbar, wpar, abort_flag, spin_limit)) break;
            if (aw == 0) TF_PROF(3, it);
            const uint32_t st = smem_u32 + s * C::STAGE;
            const uint32_t bt = smem_u32 + C::OFF_B + bb * C::BTILE;
            // fragment order: 8 bytes per (column g, word t): elements 4t..4t+3, then 16+4t..16+4t+3; all loads first
            uint2 q[8];
            float df[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int nt = 2 * aw + (i >> 2), j = i & 3;
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(q[i].x), "=r"(q[i].y) : "r"(st + (uint32_t) (C::OFF_BQ + nt * 1024 + j * 256 + (4 * g + t) * 8)));
                asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(df[i]) : "r"(st + (uint32_t) (C::OFF_BS + nt * 256 + act_scale_index(j, g) * 4)));
            }
            __syncwarp();
            if (lane == 0) tf_arrive(BAR(TFB_EMPTY, s));   // this stage's activations are in registers
#pragma unroll
            for (int i = 0; i < 8 && !(mode & 8); ++i) {
                const int nt = 2 * aw + (i >> 2), j = i & 3;
                const __half2 d2 = __half2half2(__float2half_rn(df[i]));   // the scale is an fp16 value widened
                const uint32_t w0 = q[i].x ^ 0x80808080u, w1 = q[i].y ^ 0x80808080u;   // a + 128
                uint32_t x[4];
                x[0] = __byte_perm(w0, 0x64646464u, 0x4240);   // elements 4t, 4t+2 as 1024 + (a + 128)
                x[1] = __byte_perm(w1, 0x64646464u, 0x4240);   // 16+4t, 16+4t+2
                x[2] = __byte_perm(w0, 0x64646464u, 0x4341);   // 4t+1, 4t+3
                x[3] = __byte_perm(w1, 0x64646464u, 0x4341);   // 16+4t+1, 16+4t+3
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const __half2 a2 = __hadd2(tf_as_h2(x[c]), bias);
                    const __half2 h = __hmul2(a2, d2);
                    hi[c] = tf_h2(h);
                    lo[c] = tf_h2(__hfma2(a2, d2, __hneg2(h)));
                }
                // K-step 2j + (t >> 1), column group nt (hi plane) / NT + nt (lo plane), K half t & 1, column g
                const uint32_t o = bt + (uint32_t) ((2 * j + (t >> 1)) * C::KSTEP + nt * 256 + (t & 1) * 128 + g * 16);
                if (!(mode & 1)) {
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(o), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(o + (uint32_t) (NT * 256)), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the tensor core reads these stores through the async proxy
            __syncwarp();
            if (aw == 0) TF_PROF(5, it);
            if (lane == 0) tf_arrive(BAR(TFB_B_FULL, bb));
        }
    }
#undef BAR
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}

static int tf_sm_count() {   // every device of a process is the same model
    static const int n = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

// ---- tensor maps ----
typedef CUresult (*tf_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static tf_encode_fn tf_encoder() {
    static tf_encode_fn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) p = nullptr;
        return (tf_encode_fn) p;
    }();
    return fn;
}
// 2-D view: rows of `inner_words` 32-bit words, a box of box_words x box_rows
static bool tf_encode(CUtensorMap *m, const void *base, uint64_t inner_words, uint64_t rows, uint32_t box_words, uint32_t box_rows = 8) {
    tf_encode_fn enc = tf_encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {inner_words, rows};
    const cuuint64_t strides[1] = {inner_words * 4};
    const cuuint32_t box[2] = {box_words, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// The packed weight tiles as lines of 128 bytes (8 lines per tile): [row tile][block group * 8 + line][32 words], a box of
// 8 row tiles x one block group's 8 lines, written with the 128-byte swizzle (16-byte chunk c of line l at c ^ (l & 7)).
static bool tf_encode_wq(CUtensorMap *m, const void *base, uint64_t n_bg, uint64_t n_rt) {
    tf_encode_fn enc = tf_encoder();
    if (!enc) return false;
    const cuuint64_t dims[3] = {32, n_bg * 8, n_rt};
    const cuuint64_t strides[2] = {128, n_bg * 1024};
    const cuuint32_t box[3] = {32, 8, 8};
    const cuuint32_t elem[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// encoded maps are pure functions of (pointer, extents): keep them, a model has a few hundred weights
struct TfKey {
    const void *p;
    int64_t a, b;
    bool operator==(const TfKey &o) const { return p == o.p && a == o.a && b == o.b; }
};
struct TfKeyHash {
    size_t operator()(const TfKey &k) const { return std::hash<const void *>()(k.p) ^ (size_t) (k.a * 0x9E3779B97F4A7C15ull) ^ (size_t) (k.b * 0xC2B2AE3D27D4EB4Full); }
};
struct TfPair { CUtensorMap x, y; };
static bool tf_weight_maps(const TiledDims &d, const void *w, TfPair *out) {
    static std::mutex mu;
    static std::unordered_map<TfKey, TfPair, TfKeyHash> cache;
    const TfKey key{w, d.n_rt, d.n_bg};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        TfPair p;
        if (!tf_encode_wq(&p.x, w, (uint64_t) d.n_bg, (uint64_t) d.n_rt)) return false;
        if (!tf_encode(&p.y, (const uint8_t *) w + d.qs_bytes, (uint64_t) d.n_bg * 32, (uint64_t) d.n_rt, 32)) return false;
        if (cache.size() > 65536) cache.clear();
        it = cache.emplace(key, p).first;
    }
    *out = it->second;
    return true;
}
static bool tf_act_maps(const ActDims &a, const void *aq, int nt, TfPair *out) {
    static std::mutex mu;
    static std::unordered_map<TfKey, TfPair, TfKeyHash> cache;
    const TfKey key{aq, a.n_nt * 32 + nt, a.n_bg};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        TfPair p;
        if (!tf_encode(&p.x, aq, (uint64_t) a.nbp * 64, (uint64_t) a.n_nt, 256, (uint32_t) nt)) return false;
        if (!tf_encode(&p.y, (const uint8_t *) aq + a.d_offset, (uint64_t) a.n_bg * 64, (uint64_t) a.n_nt, 64, (uint32_t) nt)) return false;
        if (cache.size() > 65536) cache.clear();
        it = cache.emplace(key, p).first;
    }
    *out = it->second;
    return true;
}

template <int NT, int TERMS>
static cudaError_t tf_launch(dim3 grid, cudaStream_t st, const TfMaps &maps, const TiledDims &d, const ActDims &a, float *dst, int64_t dst_nb_row,
                             float *partial, int ks, int mode) {
    static std::mutex mu;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[dev & 63]) {
            cudaError_t e = cudaFuncSetAttribute(mmq_tcf_kernel<NT, TERMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, TfCfg<NT, TERMS>::SMEM);
            if (e != cudaSuccess) return e;
            configured[dev & 63] = true;
        }
    }
    return launch_pdl(mmq_tcf_kernel<NT, TERMS>, grid, dim3(TfCfg<NT, TERMS>::THREADS), (size_t) TfCfg<NT, TERMS>::SMEM, st, maps, d, a, dst, dst_nb_row, partial, ks, mode);
}

// terms: 3 (exact) or 2.  Up to 64 columns a CTA takes 8 column tiles, beyond that 16.
int launch_mmq_tcf(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
                   void *workspace, size_t workspace_bytes, cudaStream_t st, int terms) {
    TfPair wm, am;
    const int nt = a.N > 64 ? 16 : 8;
    if (wtype != B200_TYPE_Q4_0 || !is_aligned(w, 16) || !is_aligned(aq, 16) || !tf_weight_maps(d, w, &wm) || !tf_act_maps(a, aq, nt, &am)) {
        return launch_mmq(wtype, d, w, a, aq, dst, dst_nb_row, workspace, workspace_bytes, st, false, PeerDst{});
    }
    static const int mode = [] {   // debugging switches, see the kernel
        const char *e = getenv("B200_TCF_DEBUG");
        return e ? atoi(e) : 0;
    }();
    TfMaps maps;
    maps.wq = wm.x; maps.wd = wm.y; maps.bq = am.x; maps.bs = am.y;
    const int64_t row_groups = (d.n_rt + 7) / 8, col_chunks = (a.n_nt + nt - 1) / nt;
    // K splits: whole waves of one CTA per SM, a few block groups of fixed cost per split
    const int64_t ctas = row_groups * col_chunks, slots = (int64_t) tf_sm_count();
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
    cudaError_t le;
    if (nt == 16) le = terms >= 3 ? tf_launch<16, 3>(grid, st, maps, d, a, dst, dst_nb_row, (float *) workspace, ks, mode)
                                  : tf_launch<16, 2>(grid, st, maps, d, a, dst, dst_nb_row, (float *) workspace, ks, mode);
    else le = terms >= 3 ? tf_launch<8, 3>(grid, st, maps, d, a, dst, dst_nb_row, (float *) workspace, ks, mode)
                         : tf_launch<8, 2>(grid, st, maps, d, a, dst, dst_nb_row, (float *) workspace, ks, mode);
    if (le != cudaSuccess) return set_error(B200_E_CUDA, "mmq_tcf launch: %s", cudaGetErrorString(le));
    if (int e = check_launch("mmq_tcf")) return e;
    if (ks > 1) {
        launch_mmq_reduce((const float *) workspace, ks, d.M, a.N, dst, dst_nb_row, st);
        return check_launch("mmq_reduce");
    }
    return B200_OK;
}

int tcf_error_flag() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_tcf_error, sizeof(int));
    return v;
}
void tcf_set_wait_limit(unsigned rounds) {
    const unsigned v = rounds ? rounds : 1u << 20;
    const int zero = 0;
    cudaMemcpyToSymbol(g_tcf_spin_limit, &v, sizeof(v));
    cudaMemcpyToSymbol(g_tcf_error, &zero, sizeof(zero));
}

}  // namespace b200
#ifdef B200_TC_PROFILE
extern "C" B200_API void b200_tcf_profile(long long *out) { cudaMemcpyFromSymbol(out, b200::g_tcf_prof, sizeof(long long) * 512); }
#endif
