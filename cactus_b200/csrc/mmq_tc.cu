// MUL_MAT for many activation columns on the 5th-generation tensor cores (tcgen05, TMEM accumulators).
//
// Same arithmetic as mmq.cu (lm_ggml_compute_forward_mul_mat, cactus/ggml-cpu/ggml-cpu.c:1257-1449): one int8
// MMA step per 32-element block, then d_w[row] * d_a[col] scaling into fp32 accumulators.  Here one
// tcgen05.mma.kind::i8 of shape 128 x 64 x 32 covers a CTA's 128 weight rows and up to 64 activation columns;
// its int32 result lives in tensor memory and is read back with tcgen05.ld, one row per thread (32x32b).
//
// A CTA is twenty warps with fixed roles, connected by mbarriers only (no __syncthreads in the main loop); one CTA
// per SM owns all 512 TMEM columns: two groups of four 64-column accumulator buffers, one buffer per block of a
// 4-block group, so the MMAs of group i+1 run while group i is being scaled.
//   warp 0      producer: four TMA tensor copies per stage bring a 4-block group of the packed T16 weight tiles
//               (8 row tiles x 1 KB, one box), their scales, the canonical-order activation tiles (quantize.cu,
//               LAYOUT 2) and the activation scales into an 8-stage ring.  Plain bulk copies, one per tile, cost
//               twice the time: the copy engine's rate is per instruction;
//   warp 1      one thread issues the four MMAs of a group and commits them to one barrier;
//   warps 2-3   expand the packed nibbles into int8 K-major core matrices (8 rows x 16 bytes, no swizzle; the layout
//               the shared-memory matrix descriptor names), double-buffered;
//   warps 4-19  epilogue, one per (TMEM lane quarter, 16-column group): read the four accumulator buffers of a
//               group refill them and release the group, then apply the
//               block scales with packed FMAs.
// A hand-over through an mbarrier costs about 400 cycles from arrive to a polling thread's next instruction, and an
// already satisfied wait about 150, so there is one wait per role and 4-block group, and one lane polls for its warp.
// The accumulator buffers are pre-filled with 0x4B400000 and the MMA accumulates onto that, so the value read back is
// the float 12582912 + dot; t = fma(d_a, v, -d_a * 12582912) and y = fma(d_w, t, y) follow as fma.rn.f32x2, exactly
// as in the mma.sync kernel.
//
// Every wait on an mbarrier is bounded: on time-out the CTA raises a flag in global memory (b200_kernel_status),
// every role stops issuing work and falls through its remaining waits, the producer waits (bounded) for its own
// copies in flight, the MMA thread for its MMAs, the CTA frees its TMEM and returns.
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
#ifdef B200_TC_PROFILE
__device__ long long g_tc_prof[64];
#define TC_PROF(slot) do { if (blockIdx.x == 3 && blockIdx.z == 0 && lane == 0) g_tc_prof[slot] = clock64(); } while (0)
#else
#define TC_PROF(slot) do { } while (0)
#endif

constexpr int TC_THREADS = 640;
constexpr int TC_STAGES = 8;
constexpr int TC_EPI_WARPS = 16;
constexpr int TC_ROWS = 128, TC_COLS = 64;
constexpr int TC_A_RAW = 8 * 1024, TC_AS = 8 * 128, TC_B = 8 * 1024, TC_BS = 8 * 256;
constexpr int TC_STAGE = TC_A_RAW + TC_AS + TC_B + TC_BS;   // 19456
constexpr int TC_A8 = 4 * 4096;                             // four blocks of 128 rows x 32 int8
constexpr int TC_BAR_OFFSET = TC_STAGES * TC_STAGE + 2 * TC_A8;
// barriers (8 bytes each): ready[S] stage_free[S] a8_ready[2] a8_free[2] acc_full[2] acc_free[2] drain
constexpr int BAR_READY = 0, BAR_STAGE_FREE = TC_STAGES, BAR_A8_READY = 2 * TC_STAGES, BAR_A8_FREE = BAR_A8_READY + 2, BAR_ACC_FULL = BAR_A8_FREE + 2,
              BAR_ACC_FREE = BAR_ACC_FULL + 2, BAR_DRAIN = BAR_ACC_FREE + 2, TC_N_BARS = BAR_DRAIN + 1;
constexpr int TC_SMEM = TC_BAR_OFFSET + TC_N_BARS * 8 + 32;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;   // polls of about 100 cycles: a fraction of a second

struct TcMaps {
    CUtensorMap wq, wd, aq, ad;   // weight quants / scales, activation quants / scales
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
__device__ __forceinline__ bool tc_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait for the completion of the barrier phase with this parity; false = gave up (or the CTA already gave up elsewhere)
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
        if (tc_test(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(&g_tc_error, 1);
    return false;
}
// the same for a whole (converged) warp: one lane polls, since every polling thread is a separate operation on the barrier
__device__ __forceinline__ bool tc_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, int lane) {
    int ok = 0;
    if (lane == 0) ok = tc_wait(bar, parity, abort_flag) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void tc_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

#define TC_LD_REGS(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7])

// 32 TMEM lanes x 16 columns: thread = lane (row), r[i] = column i.  This shape moves twice the bytes per cycle of 16x256b.
#define TC_REGS16(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7]), \
                        "=r"(r[o + 8]), "=r"(r[o + 9]), "=r"(r[o + 10]), "=r"(r[o + 11]), "=r"(r[o + 12]), "=r"(r[o + 13]), "=r"(r[o + 14]), "=r"(r[o + 15])
#define TC_LD_32x16(r, o, taddr)                                                                                                   \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n" \
                 : TC_REGS16(r, o) : "r"(taddr))
// 16 TMEM lanes x 16 columns in the mma C-fragment order: r[4k + 0,1] = (row g, columns 8k + 2t, + 1), r[4k + 2,3] = (row g + 8, same).
// Half the bytes per cycle of the shape above, but a thread then holds four rows, which share their column scales.
#define TC_LD_16x16(r, o, taddr)                                                                    \
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n" \
                 : TC_LD_REGS(r, o) : "r"(taddr))
__device__ __forceinline__ void tc_st_32x16(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};\n" ::"r"(taddr), "r"(v));
}

// debugging switches in `mode`: bit 0 no MMAs, bit 1 no scaling FMAs, bit 2 no accumulator reads, bit 3 no weight expansion
__global__ void __launch_bounds__(TC_THREADS, 1) mmq_tc_q4_kernel(const __grid_constant__ TcMaps maps, TiledDims dims, ActDims act,
                                                               float *__restrict__ dst, int64_t dst_nb_row,
                                                               float *__restrict__ partial, int ksplit, int mode) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t smem_u32 = (uint32_t) __cvta_generic_to_shared(smem);
    const uint32_t a8_u32 = smem_u32 + TC_STAGES * TC_STAGE;
    const uint32_t bars = smem_u32 + TC_BAR_OFFSET;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + TC_BAR_OFFSET + TC_N_BARS * 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);
#define BAR(which, i) (bars + 8u * (uint32_t) ((which) + (i)))
    if (warp == 0) TC_PROF(0);

    const int cta_rt0 = blockIdx.x * 8;
    const int cta_nt0 = blockIdx.y * 8;
    const int ks = blockIdx.z;
    const int per = (int) ((dims.n_bg + ksplit - 1) / ksplit);
    const int bg_begin = ks * per;
    const int bg_end = min((int) dims.n_bg, bg_begin + per);
    const int n_iter = max(0, bg_end - bg_begin);

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < TC_N_BARS; ++i) {
            // stage_free: the MMA commit (activations read), two expanding warps (packed weights read), the epilogue warps (scales read)
            const int count = (i >= BAR_STAGE_FREE && i < BAR_A8_READY) ? 3 + TC_EPI_WARPS
                            : (i >= BAR_A8_READY && i < BAR_A8_FREE)    ? 2
                            : (i >= BAR_ACC_FREE && i < BAR_DRAIN)      ? TC_EPI_WARPS : 1;
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(BAR(0, i)), "r"(count));
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {   // all 512 columns: 2 groups x 4 accumulator buffers x 64 columns (the CTA is alone on its SM)
        const uint32_t slot = (uint32_t) __cvta_generic_to_shared(tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(slot) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    if (warp == 0) TC_PROF(1);

    // registers move from the first warpgroup (copy / MMA issue / expansion) to the four epilogue warpgroups
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 24;\n");
    if (warp == 0) {
        // ---------------- producer: lanes 0..3 = the four tensor copies of a stage ----------------
        const CUtensorMap *map = lane == 0 ? &maps.wq : lane == 1 ? &maps.wd : lane == 2 ? &maps.aq : &maps.ad;
        const int xmul = lane == 0 ? 256 : lane == 1 ? 32 : lane == 2 ? 256 : 64;   // 32-bit words per block group and row
        const int ycoord = lane < 2 ? cta_rt0 : cta_nt0;                            // rows / columns past the end read as zero
        const uint32_t dst_off = lane == 0 ? 0 : lane == 1 ? TC_A_RAW : lane == 2 ? TC_A_RAW + TC_AS : TC_A_RAW + TC_AS + TC_B;
        int issued = 0;
        for (int it = 0; it < n_iter; ++it) {
            const int s = it % TC_STAGES, n = it / TC_STAGES;
            if (!tc_wait_warp(BAR(BAR_STAGE_FREE, s), (uint32_t) ((n & 1) ^ 1), abort_flag, lane)) break;
            if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(BAR(BAR_READY, s)), "r"(TC_STAGE) : "memory");
            __syncwarp();
            if (lane < 4) tc_tma_2d(smem_u32 + s * TC_STAGE + dst_off, map, (bg_begin + it) * xmul, ycoord, BAR(BAR_READY, s));
            issued = it + 1;
        }
        TC_PROF(2);
        // copies in flight must land before the CTA may exit, whatever happened elsewhere
        for (int it = max(0, issued - TC_STAGES); it < issued && lane == 0; ++it) {
            const uint32_t bar = BAR(BAR_READY, it % TC_STAGES), parity = (uint32_t) ((it / TC_STAGES) & 1);
            for (uint32_t spin = 0; spin < TC_SPIN_LIMIT && !tc_test(bar, parity); ++spin) {}
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issue: lane 0 issues; lanes 0 and 1 poll the two barriers of a group side by side ----------------
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (TC_COLS >> 3) << 17) | ((uint32_t) (TC_ROWS >> 4) << 24);
        for (int it = 0; it < n_iter; ++it) {
            const int s = it % TC_STAGES, u = it & 1, m = it >> 1;
            // the expanded weights are ready (their warps saw the stage land: the activation tiles are there too); the accumulator group is free
            int ok = 1;
            if (lane == 0) ok = tc_wait(BAR(BAR_A8_READY, u), (uint32_t) (m & 1), abort_flag) ? 1 : 0;
            if (lane == 1) ok = tc_wait(BAR(BAR_ACC_FREE, u), (uint32_t) ((m & 1) ^ 1), abort_flag) ? 1 : 0;
            if (__any_sync(0xffffffffu, !ok)) break;
            if (lane == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (mode & 1) {
                    tc_arrive(BAR(BAR_ACC_FULL, u)); tc_arrive(BAR(BAR_A8_FREE, u)); tc_arrive(BAR(BAR_STAGE_FREE, s));
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // leading-dimension byte offset = step between the two core matrices along K, stride byte offset = step between 8-row groups
                        const uint64_t adesc = tc_smem_desc(a8_u32 + u * TC_A8 + j * 4096, 128, 256);
                        const uint64_t bdesc = tc_smem_desc(smem_u32 + s * TC_STAGE + TC_A_RAW + TC_AS + j * 256, 128, 1024);
                        asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n"
                                     ::"r"(tmem + 256 * u + 64 * j), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
                    }
                    tc_commit(BAR(BAR_ACC_FULL, u)); tc_commit(BAR(BAR_A8_FREE, u)); tc_commit(BAR(BAR_STAGE_FREE, s));
                }
            }
            __syncwarp();
        }
        TC_PROF(3);
        if (lane == 0) {   // no MMA of this CTA may be in flight when its tensor memory is freed, whatever happened elsewhere
            tc_commit(BAR(BAR_DRAIN, 0));
            for (uint32_t spin = 0; spin < TC_SPIN_LIMIT && !tc_test(BAR(BAR_DRAIN, 0), 0); ++spin) {}
        }
        __syncwarp();
    } else if (warp < 4) {
        // ---------------- expand packed nibbles to int8 core matrices: warp = four tiles of 16 rows ----------------
        const int g = lane >> 2, t = lane & 3;
        for (int it = 0; it < n_iter; ++it) {
            const int s = it % TC_STAGES, n = it / TC_STAGES, u = it & 1, m = it >> 1;
            int ok = 1;
            if (lane == 0) ok = tc_wait(BAR(BAR_READY, s), (uint32_t) (n & 1), abort_flag) ? 1 : 0;
            if (lane == 1) ok = tc_wait(BAR(BAR_A8_FREE, u), (uint32_t) ((m & 1) ^ 1), abort_flag) ? 1 : 0;
            if (__any_sync(0xffffffffu, !ok)) break;
            if (!(mode & 8)) {
                const uint8_t *raw = smem + s * TC_STAGE;
                uint8_t *a8 = smem + TC_STAGES * TC_STAGE + u * TC_A8 + g * 16 + t * 4;
#pragma unroll
                for (int tt = 0; tt < 4; ++tt) {
                    const int tile = (warp - 2) * 4 + tt;
                    const uint4 *p = reinterpret_cast<const uint4 *>(raw + tile * 1024) + lane * 2;
                    const uint4 u0 = p[0], u1 = p[1];
                    const uint32_t wg[4] = {u0.x, u0.y, u0.z, u0.w}, wh[4] = {u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // rows 16*tile + g (8-row group 2*tile) and 16*tile + 8 + g (group 2*tile + 1); low nibbles = elements 0..15
                        uint8_t *blk = a8 + j * 4096 + (2 * tile) * 256;
                        *reinterpret_cast<uint32_t *>(blk) = (wg[j] << 4) & 0xF0F0F0F0u;
                        *reinterpret_cast<uint32_t *>(blk + 128) = wg[j] & 0xF0F0F0F0u;
                        *reinterpret_cast<uint32_t *>(blk + 256) = (wh[j] << 4) & 0xF0F0F0F0u;
                        *reinterpret_cast<uint32_t *>(blk + 384) = wh[j] & 0xF0F0F0F0u;
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy stores -> tensor-core reads
            __syncwarp();
            if (lane == 0) { tc_arrive(BAR(BAR_A8_READY, u)); tc_arrive(BAR(BAR_STAGE_FREE, s)); }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 112;\n");
        // -------- epilogue: rows 32*q + {g, g+8, g+16, g+24}, column pairs 16*cq + 8k + 2t (k < 2) --------
        const int q = warp & 3, cq = (warp - 4) >> 2, g = lane >> 2, t = lane & 3;
        uint64_t y[4][2];
#pragma unroll
        for (int r = 0; r < 4; ++r) y[r][0] = y[r][1] = 0ull;
        const uint32_t t_lo = tmem + ((uint32_t) (32 * q) << 16) + 16 * cq, t_hi = t_lo + (16u << 16);
        if (warp == 4) TC_PROF(4);

        uint32_t c0[32], c1[32];   // blocks {0,1} and {2,3} of a group: per block lo[8] (rows g, g+8) then hi[8] (rows g+16, g+24)
        // y += d_w * (d_a * v - d_a * 12582912) for one block, where v = as_float(dot + 0x4B400000) = 12582912 + dot
        auto scale_block = [&](const uint32_t (&cc)[32], int o, const uint8_t *sj, const uint64_t (&dw)[4]) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint4 sc = *reinterpret_cast<const uint4 *>(sj + k * 256);   // {d0, d1, nd0, nd1} of columns 8k + 2t, + 1
                const uint64_t da = tc_pack2(sc.x, sc.y), nda = tc_pack2(sc.z, sc.w);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int i = o + (r >> 1) * 8 + 4 * k + 2 * (r & 1);
                    const uint64_t tt = tc_fma2(tc_pack2(cc[i] + 0x4B400000u, cc[i + 1] + 0x4B400000u), da, nda);
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
        bool ok = n_iter > 0 && tc_wait_warp(BAR(BAR_ACC_FULL, 0), 0u, abort_flag, lane);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (mode & 4) {
#pragma unroll
                for (int i = 0; i < 32; ++i) c0[i] = c1[i] = 0u;
            } else {
                TC_LD_16x16(c0, 0, t_lo); TC_LD_16x16(c0, 8, t_hi);
                TC_LD_16x16(c0, 16, t_lo + 64); TC_LD_16x16(c0, 24, t_hi + 64);
            }
        }
        for (int it = 0; ok && it < n_iter; ++it) {
            const int s = it % TC_STAGES, u = it & 1;
            if (warp == 4 && it < 8) TC_PROF(8 + it);
            // the group's MMAs are done: their thread was told so by warps that saw the stage land, so the scales are there too
            const uint8_t *st = smem + s * TC_STAGE;
            // weight scales: fp16 at 4*row + block within a tile's 128 bytes; rows {g, g+8} of tiles 2q and 2q + 1
            const uint2 *sa = reinterpret_cast<const uint2 *>(st + TC_A_RAW + (2 * q) * 128);
            const uint2 h4[4] = {sa[g], sa[g + 8], sa[16 + g], sa[24 + g]};
            const uint8_t *Ss = st + TC_A_RAW + TC_AS + TC_B + (2 * cq) * 256 + t * 16;
            const uint32_t a_lo = t_lo + 256 * u, a_hi = t_hi + 256 * u;
            uint64_t dw[4];
            if (!(mode & 4)) {
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                TC_LD_16x16(c1, 0, a_lo + 128); TC_LD_16x16(c1, 8, a_hi + 128);
                TC_LD_16x16(c1, 16, a_lo + 192); TC_LD_16x16(c1, 24, a_hi + 192);
            }
            if (!(mode & 2)) {
                dw_of(h4, 0, dw); scale_block(c0, 0, Ss, dw);
                dw_of(h4, 1, dw); scale_block(c0, 16, Ss + 64, dw);
            }
            if (!(mode & 4)) asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            // everything of this group is in registers: the MMAs overwrite, so it can be handed back at once
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_arrive(BAR(BAR_ACC_FREE, u));
            if (it + 1 < n_iter) {   // start reading the next group before the second half of this one is scaled
                ok = tc_wait_warp(BAR(BAR_ACC_FULL, u ^ 1), (uint32_t) (((it + 1) >> 1) & 1), abort_flag, lane);
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (ok && !(mode & 4)) {
                    const uint32_t b_lo = t_lo + 256 * (u ^ 1), b_hi = t_hi + 256 * (u ^ 1);
                    TC_LD_16x16(c0, 0, b_lo); TC_LD_16x16(c0, 8, b_hi);
                    TC_LD_16x16(c0, 16, b_lo + 64); TC_LD_16x16(c0, 24, b_hi + 64);
                }
            }
            if (!(mode & 2)) {
                dw_of(h4, 2, dw); scale_block(c1, 0, Ss + 128, dw);
                dw_of(h4, 3, dw); scale_block(c1, 16, Ss + 192, dw);
            }
            __syncwarp();
            if (lane == 0) tc_arrive(BAR(BAR_STAGE_FREE, s));
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (warp == 4) TC_PROF(5);
        // write back (Q4_0 quants were used as 16 * value)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int64_t row = (int64_t) blockIdx.x * TC_ROWS + 32 * q + 8 * r + g;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int64_t col = (int64_t) cta_nt0 * 8 + 16 * cq + 8 * k + 2 * t;
                uint32_t lo, hi;
                asm("mov.b64 {%0,%1}, %2;" : "=r"(lo), "=r"(hi) : "l"(y[r][k]));
                const float v0 = __uint_as_float(lo) * 0.0625f, v1 = __uint_as_float(hi) * 0.0625f;
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
    if (warp == 4) TC_PROF(6);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) TC_PROF(7);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}

static int tc_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// ---- tensor maps: 2-D views (row = tile row / column tile, inner = 32-bit words along K) of the four planes ----
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
// encoded maps are pure functions of (pointer, extents): keep them, a model has a few hundred weights
struct TcKey {
    const void *p;
    int64_t a, b;
    bool operator==(const TcKey &o) const { return p == o.p && a == o.a && b == o.b; }
};
struct TcKeyHash {
    size_t operator()(const TcKey &k) const { return std::hash<const void *>()(k.p) ^ (size_t) (k.a * 0x9E3779B97F4A7C15ull) ^ (size_t) (k.b * 0xC2B2AE3D27D4EB4Full); }
};
struct TcPair { CUtensorMap q, d; };
static bool tc_weight_maps(const TiledDims &d, const void *w, TcPair *out) {
    static std::mutex mu;
    static std::unordered_map<TcKey, TcPair, TcKeyHash> cache;
    const TcKey key{w, d.n_rt, d.n_bg};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        TcPair p;
        if (!tc_encode(&p.q, w, (uint64_t) d.n_bg * 256, (uint64_t) d.n_rt, 256)) return false;
        if (!tc_encode(&p.d, (const uint8_t *) w + d.qs_bytes, (uint64_t) d.n_bg * 32, (uint64_t) d.n_rt, 32)) return false;
        if (cache.size() > 65536) cache.clear();
        it = cache.emplace(key, p).first;
    }
    *out = it->second;
    return true;
}
static bool tc_act_maps(const ActDims &a, const void *aq, TcPair *out) {
    static std::mutex mu;
    static std::unordered_map<TcKey, TcPair, TcKeyHash> cache;
    const TcKey key{aq, a.n_nt, a.n_bg};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        TcPair p;
        if (!tc_encode(&p.q, aq, (uint64_t) a.nbp * 64, (uint64_t) a.n_nt, 256)) return false;
        if (!tc_encode(&p.d, (const uint8_t *) aq + a.d_offset, (uint64_t) a.n_bg * 64, (uint64_t) a.n_nt, 64)) return false;
        if (cache.size() > 65536) cache.clear();
        it = cache.emplace(key, p).first;
    }
    *out = it->second;
    return true;
}

int launch_mmq_tc(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
                  void *workspace, size_t workspace_bytes, cudaStream_t st) {
    // Q8_0 weights stay on the mma.sync kernel, reading the canonical activation order
    if (wtype != B200_TYPE_Q4_0) return launch_mmq(wtype, d, w, a, aq, dst, dst_nb_row, workspace, workspace_bytes, st, true, PeerDst{});
    TcPair wm, am;
    if (!is_aligned(w, 16) || !is_aligned(aq, 16) || !tc_weight_maps(d, w, &wm) || !tc_act_maps(a, aq, &am)) {
        return launch_mmq(wtype, d, w, a, aq, dst, dst_nb_row, workspace, workspace_bytes, st, true, PeerDst{});
    }
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(mmq_tc_q4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        if (e != cudaSuccess) return set_error(B200_E_CUDA, "mmq_tc shared memory opt-in: %s", cudaGetErrorString(e));
        configured[dev & 63] = true;
    }
    static int mode = -1;   // debugging switches, see the kernel
    if (mode < 0) {
        const char *e = getenv("B200_TC_DEBUG");
        mode = e ? atoi(e) : 0;
    }
    TcMaps maps;
    maps.wq = wm.q; maps.wd = wm.d; maps.aq = am.q; maps.ad = am.d;
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
    mmq_tc_q4_kernel<<<grid, TC_THREADS, TC_SMEM, st>>>(maps, d, a, dst, dst_nb_row, (float *) workspace, ks, mode);
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

}  // namespace b200

extern "C" B200_API int b200_kernel_status(void) { return b200::tc_error_flag(); }
#ifdef B200_TC_PROFILE
extern "C" B200_API void b200_tc_profile(long long *out) { cudaMemcpyFromSymbol(out, b200::g_tc_prof, sizeof(long long) * 64); }
#endif
