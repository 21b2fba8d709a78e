// MUL_MAT for more than a couple of activation columns: int8 tensor-core kernel with per-block fp16 scales.
//
// Replaces the chunked vec_dot loop of lm_ggml_compute_forward_mul_mat
// (cactus/ggml-cpu/ggml-cpu.c:1257-1449).  Every 32-element block has its own pair of scales, so each
// k=32 MMA step produces a fresh integer tile that must be scaled by d_w[row] * d_a[col] and added to an
// fp32 accumulator.  That epilogue, not the MMA, is the cost; it is kept to two packed instructions per
// pair of values:
//   * the MMA accumulator starts at 0x4B400000, so the int32 result read as a float is 12582912 + dot
//     (exact, |dot| < 2^22);  t = fma(d_a, that, -d_a * 12582912) equals d_a * dot rounded once, with the
//     constant term precomputed per (column, block) by the quantiser -- no int->float conversion;
//   * y = fma(d_w, t, y).
//   Both run as fma.rn.f32x2 on the (column 2t, column 2t+1) pair an MMA thread owns.
//
// Work split: a warp owns 32 weight rows (two 16-row tiles) and every column of the CTA's column chunk.
// The 4 warps of a CTA walk the same block groups; weight tiles and activation tiles are both stored in
// fragment order, so a 4-stage cp.async ring copies them verbatim (16-byte chunks, three block groups in
// flight per CTA to cover HBM latency) and the fragments are plain 128/64-bit shared loads.
// grid = (row groups of 128, column chunks, K splits); with K splits > 1 partial tiles go to a workspace
// and a second kernel adds them in a fixed order.
#include <cstdlib>

#include <mutex>

#include "common.cuh"

namespace b200 {


__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const uint32_t s = (uint32_t) __cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_s8_magic(uint32_t (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    const uint32_t magic = 0x4B400000u;
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(magic));
}
// One k=32 step of a 16x8 tile and its epilogue in a single block, so the accumulator pairs stay in aligned
// register pairs: c = A.B + 0x4B400000 (bits of 12582912 + dot); t = d_a * c - d_a * 12582912; y += d_w * t.
__device__ __forceinline__ void mma_scale_acc(uint64_t &y01, uint64_t &y23, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1, uint64_t da, uint64_t nda, uint64_t dw01, uint64_t dw23) {
    asm("{\n"
        ".reg .b32 c0, c1, c2, c3;\n"
        ".reg .b64 p01, p23;\n"
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {c0,c1,c2,c3}, {%2,%3,%4,%5}, {%6,%7}, {%12,%12,%12,%12};\n"
        "mov.b64 p01, {c0,c1};\n"
        "mov.b64 p23, {c2,c3};\n"
        "fma.rn.f32x2 p01, p01, %8, %9;\n"
        "fma.rn.f32x2 p23, p23, %8, %9;\n"
        "fma.rn.f32x2 %0, p01, %10, %0;\n"
        "fma.rn.f32x2 %1, p23, %11, %1;\n"
        "}\n"
        : "+l"(y01), "+l"(y23)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "l"(da), "l"(nda), "l"(dw01), "l"(dw23), "r"(0x4B400000u));
}
// k=32 MMA step alone, accumulator pairs returned packed (aligned register pairs for the f32x2 epilogue)
__device__ __forceinline__ void mma_s8_magic2(uint64_t &p01, uint64_t &p23, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("{\n"
        ".reg .b32 c0, c1, c2, c3;\n"
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {c0,c1,c2,c3}, {%2,%3,%4,%5}, {%6,%7}, {%8,%8,%8,%8};\n"
        "mov.b64 %0, {c0,c1};\n"
        "mov.b64 %1, {c2,c3};\n"
        "}\n"
        : "=l"(p01), "=l"(p23)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0x4B400000u));
}
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
    uint32_t a, b;
    asm("mov.b64 {%0,%1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a);
    hi = __uint_as_float(b);
}

template <int WTYPE>
struct WFrag {  // one block group of one 16-row tile: quants of rows g / g+8 and their four block scales
    static constexpr int NW = (WTYPE == B200_TYPE_Q4_0) ? 4 : 8;
    uint32_t a[NW], b[NW];
    uint2 sa, sb;
};

template <int WTYPE>
__device__ __forceinline__ void load_wfrag(WFrag<WTYPE> &f, const uint8_t *__restrict__ wq, const uint8_t *__restrict__ wd, int lane) {
    const int g = lane >> 2;
    if (WTYPE == B200_TYPE_Q4_0) {
        // lane i owns the 16-byte chunks 2i and 2i + 1 of the tile; in the ring chunk c sits at c ^ ((c >> 3) & 1) (see the
        // copy plan), which spreads the eight lanes of a quarter warp over all eight 16-byte bank groups
        const int sw = (lane >> 2) & 1;
        const uint4 *p = reinterpret_cast<const uint4 *>(wq);
        const uint4 u0 = p[(lane * 2) ^ sw], u1 = p[(lane * 2 + 1) ^ sw];
        f.a[0] = u0.x; f.a[1] = u0.y; f.a[2] = u0.z; f.a[3] = u0.w;
        f.b[0] = u1.x; f.b[1] = u1.y; f.b[2] = u1.z; f.b[3] = u1.w;
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 u = (reinterpret_cast<const uint4 *>(wq + j * 512))[lane];
            f.a[2 * j] = u.x; f.b[2 * j] = u.y; f.a[2 * j + 1] = u.z; f.b[2 * j + 1] = u.w;
        }
    }
    f.sa = reinterpret_cast<const uint2 *>(wd)[g];
    f.sb = reinterpret_cast<const uint2 *>(wd)[g + 8];
}

// Shape of a CTA: WM x WN warps; a warp owns MT 16-row tiles and NTW 8-column tiles.
template <int WTYPE, int NTW, int WN, int MT, int WM, int STAGES>
struct MmqCfg {
    static constexpr int WARPS = WM * WN;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int CTA_TILES = WM * MT;      // 16-row tiles per CTA
    static constexpr int NT = WN * NTW;            // 8-column tiles per CTA
    static constexpr int TILE = (WTYPE == B200_TYPE_Q4_0) ? 1024 : 2048;
    static constexpr int A_BYTES = CTA_TILES * TILE;       // weight tiles of the CTA's rows, one block group
    static constexpr int AS_BYTES = CTA_TILES * 128;       // their scales
    static constexpr int B_BYTES = NT * 1024;              // NT n-tiles x 4 blocks x 256 B
    static constexpr int S_BYTES = NT * 256;               // their scale groups
    static constexpr int STAGE = A_BYTES + AS_BYTES + B_BYTES + S_BYTES;
    static constexpr int TOTAL = STAGE * STAGES;
};

// MODE 1 (peer): the write-back also stores into the other GPUs' buffers of a row split; a separate instantiation so
// that the one-GPU kernel is the same machine code as without the feature (it measured 7 % slower on the widest shape
// otherwise).
// MODE 2 (stream-K): the grid is one CTA per resident slot of the device, and the (row group, block group) iterations
// of the whole product are dealt out evenly and contiguously, so every SM is busy for the same time whatever the row
// count.  A CTA whose range ends inside a row group parks its partial tile in the workspace; the CTA that arrives last
// at a row group (a counter per row group) adds the parts in K order and writes the result, so the sum does not
// depend on the arrival order and nobody waits for anybody.
// MMQ_PEER and MMQ_STREAMK_SEG know row ranges (other GPUs' buffers, separate weight / destination tensors); the plain
// kernels carry none of that code: the hot shapes of a decode step must not pay for it
constexpr int MMQ_PLAIN = 0, MMQ_PEER = 1, MMQ_STREAMK = 2, MMQ_STREAMK_SEG = 3;
#ifndef MMQ_DEPTH
#define MMQ_DEPTH 2
#endif
template <int WTYPE, int NTW, int WN, int MT, int WM, int STAGES, int MINB, int MODE = MMQ_PLAIN>
__global__ void __launch_bounds__(WM * WN * 32, MINB) mmq_kernel(TiledDims dims, const uint8_t *__restrict__ w, ActDims act,
                                                          const uint8_t *__restrict__ aq, float *__restrict__ dst,
                                                          int64_t dst_nb_row, float *__restrict__ partial, int ksplit, int canon, int cluster, PeerDst peers) {
    pdl_prologue();
    using S = MmqCfg<WTYPE, NTW, WN, MT, WM, STAGES>;
    constexpr int MMQ_STAGES = STAGES;
    constexpr int NT = NTW;              // n-tiles of this warp
    constexpr int MMQ_MT = MT;
    constexpr int MMQ_THREADS = S::THREADS;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp / WN, wn = warp % WN;
    const int64_t rt0 = (int64_t) blockIdx.x * S::CTA_TILES + wm * MT;  // first row tile of this warp
    const int64_t cta_nt0 = (int64_t) blockIdx.y * S::NT;
    const int64_t nt0 = cta_nt0 + wn * NTW;                               // first column tile of this warp
    const int ks = blockIdx.z;
    const int64_t per = (dims.n_bg + ksplit - 1) / ksplit;
    const int64_t bg_begin = ks * per;
    const int64_t bg_end = min(dims.n_bg, bg_begin + per);
    constexpr bool SK = MODE == MMQ_STREAMK || MODE == MMQ_STREAMK_SEG;
    constexpr bool SEGS = MODE == MMQ_PEER || MODE == MMQ_STREAMK_SEG;
    // Stream-K.  Iteration i of the product is block group i % n_bg of row group i / n_bg.  Two ways to deal them out:
    //   even deal (ksplit <= 1): CTA j owns the contiguous iterations [j * total / G, (j + 1) * total / G) -- for
    //     products with more row groups than CTAs; a CTA first does the piece its range ends with, then the rest, so it
    //     finishes with whole row groups;
    //   head/tail deal (ksplit = h > 1): fewer row groups than CTAs.  CTA b < groups does block groups [0, h) of row
    //     group b; the other Gs CTAs share the tails [h, n_bg) of all row groups, contiguously, and are done first (h is
    //     chosen that way), so every head finds its tail parked and finishes with one read and the store.
    const uint32_t sk_nbg = (uint32_t) dims.n_bg;
    const uint32_t sk_groups = SK ? (uint32_t) (dims.n_rt / S::CTA_TILES) : 0u;
    const uint32_t sk_total = sk_groups * sk_nbg;
    const uint32_t sk_h = SK && ksplit > 1 ? (uint32_t) ksplit : 0u;       // 0: even deal
    const uint32_t sk_sl = sk_nbg - sk_h;                                    // tail length of a row group (head/tail deal)
    const uint32_t sk_gs = SK ? gridDim.x - sk_groups : 1u;                  // CTAs that share the tails
    const bool sk_tails = sk_h != 0 && blockIdx.x >= sk_groups;
    // this CTA's range [sk_it0, sk_it0 + n_iter): in iteration space, or for a tail CTA in the space of all tails laid end to end
    uint32_t sk_it0 = 0, sk_n = 0;
    if (SK) {
        if (sk_h == 0) {
            sk_it0 = (uint32_t) ((uint64_t) blockIdx.x * sk_total / gridDim.x);
            sk_n = (uint32_t) ((uint64_t) (blockIdx.x + 1) * sk_total / gridDim.x) - sk_it0;
        } else if (!sk_tails) {
            sk_it0 = blockIdx.x * sk_nbg;
            sk_n = sk_h;
        } else {
            const uint64_t c = blockIdx.x - sk_groups, all = (uint64_t) sk_groups * sk_sl;
            sk_it0 = (uint32_t) (c * all / sk_gs);
            sk_n = (uint32_t) ((c + 1) * all / sk_gs) - sk_it0;
        }
    }
    const int64_t n_iter = SK ? (int64_t) sk_n : max((int64_t) 0, bg_end - bg_begin);

    // Copy plan of this thread, fixed for the whole K loop: 16-byte chunk c of a stage comes from
    // base + (src16[k] + bg * step16) * 16.  Offsets are in 16-byte units and fit 32 bits.
    const int64_t cta_rt0 = SK ? 0 : (int64_t) blockIdx.x * S::CTA_TILES;   // stream-K adds the row group per iteration
    constexpr int A_CH = S::A_BYTES / 16, AS_CH = S::AS_BYTES / 16, B_CH = S::B_BYTES / 16, S_CH = S::S_BYTES / 16;
    constexpr int A_N = (A_CH + MMQ_THREADS - 1) / MMQ_THREADS, AS_N = (AS_CH + MMQ_THREADS - 1) / MMQ_THREADS;
    constexpr int B_N = (B_CH + MMQ_THREADS - 1) / MMQ_THREADS, S_N = (S_CH + MMQ_THREADS - 1) / MMQ_THREADS;
    uint32_t a_src[A_N], as_src[AS_N], b_src[B_N], s_src[S_N];
    uint32_t a_dst[A_N];   // Q4_0: chunk c of a tile lands at chunk position c ^ ((c >> 3) & 1): conflict-free for the fragment loads
    const uint8_t *w_sc = w + dims.qs_bytes, *a_sc = aq + act.d_offset;
#pragma unroll
    for (int k = 0; k < A_N; ++k) {
        const int c = tid + k * MMQ_THREADS;
        const int tile = c / (S::TILE / 16), off = c % (S::TILE / 16);
        const int64_t rt = min(cta_rt0 + tile, dims.n_rt - 1);  // rows beyond the matrix are never written back
        a_src[k] = (uint32_t) (rt * dims.n_bg * (S::TILE / 16) + off);
        a_dst[k] = (WTYPE == B200_TYPE_Q4_0) ? (uint32_t) (tile * S::TILE + (off ^ ((off >> 3) & 1)) * 16) : (uint32_t) (c * 16);
    }
#pragma unroll
    for (int k = 0; k < AS_N; ++k) {
        const int c = tid + k * MMQ_THREADS;
        const int64_t rt = min(cta_rt0 + (c >> 3), dims.n_rt - 1);
        as_src[k] = (uint32_t) (rt * dims.n_bg * 8 + (c & 7));
    }
#pragma unroll
    for (int k = 0; k < B_N; ++k) {
        const int c = tid + k * MMQ_THREADS;
        const int64_t nt = min(cta_nt0 + (c >> 6), act.n_nt - 1);  // columns beyond N are never written back
        b_src[k] = (uint32_t) (nt * act.nbp * 16 + (c & 63));
    }
#pragma unroll
    for (int k = 0; k < S_N; ++k) {
        const int c = tid + k * MMQ_THREADS;
        const int64_t nt = min(cta_nt0 + (c >> 4), act.n_nt - 1);
        s_src[k] = (uint32_t) (nt * act.n_bg * 16 + (c & 15));
    }
    // Stream-K order inside a CTA: a range that ends inside a row group (or tail) starts with that last piece and then
    // walks the rest from its beginning.  The pieces shared with a neighbour are then parked early, long before the CTA
    // that completes the row group looks for them.
    const uint32_t sk_unit = sk_tails ? sk_sl : sk_nbg;   // length of what the range is cut at
    uint32_t sk_head = 0, sk_head_at = 0;
    if (SK) {
        const uint32_t it1 = sk_it0 + sk_n;
        sk_head_at = it1 / sk_unit * sk_unit;
        if (sk_head_at > sk_it0 && it1 > sk_head_at) sk_head = it1 - sk_head_at;
    }
    // local iteration -> (row group, block group)
    auto sk_where = [&](int64_t it, uint32_t &ct, uint32_t &bg) {
        const uint32_t u = it < (int64_t) sk_head ? sk_head_at + (uint32_t) it : sk_it0 + (uint32_t) it - sk_head;
        ct = u / sk_unit;
        bg = u - ct * sk_unit + (sk_tails ? sk_h : 0u);
    };
    uint32_t iss_ct = 0, iss_bg = 0;   // stream-K: where the next copy reads
    if (SK) sk_where(0, iss_ct, iss_bg);
    auto issue = [&](int64_t it) {
        uint8_t *st = smem + (it % MMQ_STAGES) * S::STAGE;
        uint32_t bg = (uint32_t) (bg_begin + it);
        uint32_t wbg = bg;   // block-group index into the weight stream, row group included
        int64_t first_row = cta_rt0 * 16;   // of the row group this copy belongs to
        if (SK) {
            if (sk_head != 0 && it == (int64_t) sk_head) sk_where(it, iss_ct, iss_bg);   // the last piece is copied: on to the start of the range
            bg = iss_bg;
            wbg = iss_ct * (uint32_t) S::CTA_TILES * sk_nbg + iss_bg;
            first_row = (int64_t) iss_ct * S::CTA_TILES * 16;
            if (++iss_bg == sk_nbg) {
                iss_bg = sk_tails ? sk_h : 0u;
                ++iss_ct;
            }
        }
        // row ranges from separate weight tensors (PeerDst::wseg): the range's tensor, and its first row tile taken off the offsets
        const uint8_t *wq_base = w, *ws_base = w_sc;
        if (SEGS && peers.n_wseg > 0) {
            const int k = first_row < peers.seg_end[0] ? 0 : ((peers.n_seg > 2 && first_row >= peers.seg_end[1]) ? 2 : 1);
            wq_base = peers.wseg[k];
            ws_base = wq_base + peers.wseg_qs[k];
            if (k > 0) wbg -= (uint32_t) (peers.seg_end[k - 1] / 16) * (uint32_t) dims.n_bg;   // (the sums below stay non-negative)
        }
#pragma unroll
        for (int k = 0; k < A_N; ++k) {
            const int c = tid + k * MMQ_THREADS;
            if (A_CH % MMQ_THREADS == 0 || c < A_CH) cp_async16(st + a_dst[k], wq_base + (size_t) (uint32_t) (a_src[k] + wbg * (S::TILE / 16)) * 16);
        }
#pragma unroll
        for (int k = 0; k < AS_N; ++k) {
            const int c = tid + k * MMQ_THREADS;
            if (AS_CH % MMQ_THREADS == 0 || c < AS_CH) cp_async16(st + S::A_BYTES + c * 16, ws_base + (size_t) (uint32_t) (as_src[k] + wbg * 8) * 16);
        }
        uint8_t *sb = st + S::A_BYTES + S::AS_BYTES;
#pragma unroll
        for (int k = 0; k < B_N; ++k) {
            const int c = tid + k * MMQ_THREADS;
            if (B_CH % MMQ_THREADS == 0 || c < B_CH) cp_async16(sb + c * 16, aq + (size_t) (b_src[k] + bg * 64) * 16);
        }
#pragma unroll
        for (int k = 0; k < S_N; ++k) {
            const int c = tid + k * MMQ_THREADS;
            if (S_CH % MMQ_THREADS == 0 || c < S_CH) cp_async16(sb + S::B_BYTES + c * 16, a_sc + (size_t) (s_src[k] + bg * 16) * 16);
        }
    };
    uint64_t y[MMQ_MT][NT][2];  // packed (col 2t, col 2t+1) for row g ([0]) and row g+8 ([1])
#pragma unroll
    for (int mt = 0; mt < MMQ_MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) y[mt][nt][0] = y[mt][nt][1] = 0ull;

    for (int s = 0; s < MMQ_STAGES - 1; ++s) {
        if (s < n_iter) issue(s);
        cp_async_commit();
    }

    auto body = [&](int64_t it) {
        cp_async_wait<MMQ_STAGES - 2>();
        __syncthreads();
        if (it + MMQ_STAGES - 1 < n_iter) issue(it + MMQ_STAGES - 1);
        cp_async_commit();

        const uint8_t *As = smem + (it % MMQ_STAGES) * S::STAGE;
        const uint8_t *Bs = As + S::A_BYTES + S::AS_BYTES;
        const uint8_t *Ss = Bs + S::B_BYTES;
        WFrag<WTYPE> cur[MMQ_MT];
#pragma unroll
        for (int mt = 0; mt < MMQ_MT; ++mt) {
            const int tile = wm * MT + mt;
            load_wfrag<WTYPE>(cur[mt], As + tile * S::TILE, As + S::A_BYTES + tile * 128, lane);
        }

        // 4 blocks x NT/2 column-tile pairs = a flat sequence of steps.  The MMAs of step s+1 are issued before the
        // epilogue FMAs of step s, so the tensor-pipe latency of one step hides behind the FP32 work of the previous one.
        constexpr int NP = NT / 2;
        constexpr int NSTEP = 4 * NP;
        uint32_t a0[MMQ_MT], a1[MMQ_MT], a2[MMQ_MT], a3[MMQ_MT];
        // DEPTH steps are in flight: the MMAs of steps s+1 .. s+DEPTH-1 are issued before the epilogue of step s
        constexpr int DEPTH = MMQ_DEPTH;
        uint64_t dwa[2][MMQ_MT], dwb[2][MMQ_MT];   // weight scales of the block of the step in flight / the step being finished
        uint64_t p01[DEPTH][2][MMQ_MT], p23[DEPTH][2][MMQ_MT];
        uint2 sc[DEPTH][2];                          // {d0, d1} of the two column tiles of a step (-d * 12582912 is recomputed: half the shared-memory traffic)
        auto start = [&](int step, int buf) {
            const int j = step / NP, np = step % NP;
            if (np == 0) {
                // A fragments of block j for the warp's row tiles, and the block's weight scales as packed (d, d) pairs
#pragma unroll
                for (int mt = 0; mt < MMQ_MT; ++mt) {
                    const uint32_t ha = (j < 2) ? cur[mt].sa.x : cur[mt].sa.y, hb = (j < 2) ? cur[mt].sb.x : cur[mt].sb.y;
                    const __half2 h2a = *reinterpret_cast<const __half2 *>(&ha), h2b = *reinterpret_cast<const __half2 *>(&hb);
                    const uint32_t ua = __float_as_uint((j & 1) ? __high2float(h2a) : __low2float(h2a));
                    const uint32_t ub = __float_as_uint((j & 1) ? __high2float(h2b) : __low2float(h2b));
                    dwa[j & 1][mt] = pack2(ua, ua);
                    dwb[j & 1][mt] = pack2(ub, ub);
                    if (WTYPE == B200_TYPE_Q4_0) {
                        a0[mt] = (cur[mt].a[j] << 4) & 0xF0F0F0F0u; a2[mt] = cur[mt].a[j] & 0xF0F0F0F0u;
                        a1[mt] = (cur[mt].b[j] << 4) & 0xF0F0F0F0u; a3[mt] = cur[mt].b[j] & 0xF0F0F0F0u;
                    } else {
                        a0[mt] = cur[mt].a[2 * j]; a2[mt] = cur[mt].a[2 * j + 1];
                        a1[mt] = cur[mt].b[2 * j]; a3[mt] = cur[mt].b[2 * j + 1];
                    }
                }
            }
            const int ntl = wn * NTW + 2 * np;
            uint2 b0, b1;
            if (canon) {   // activations kept as two 8-column x 16-byte core matrices per block (the tcgen05 kernel's order)
                const uint8_t *q0 = Bs + ntl * 1024 + j * 256 + g * 16 + t * 4, *q1 = q0 + 1024;
                b0 = make_uint2(*reinterpret_cast<const uint32_t *>(q0), *reinterpret_cast<const uint32_t *>(q0 + 128));
                b1 = make_uint2(*reinterpret_cast<const uint32_t *>(q1), *reinterpret_cast<const uint32_t *>(q1 + 128));
            } else {
                b0 = reinterpret_cast<const uint2 *>(Bs + ntl * 1024 + j * 256)[lane];
                b1 = reinterpret_cast<const uint2 *>(Bs + (ntl + 1) * 1024 + j * 256)[lane];
            }
            sc[buf][0] = *reinterpret_cast<const uint2 *>(Ss + ntl * 256 + (j * 4 + t) * 16);
            sc[buf][1] = *reinterpret_cast<const uint2 *>(Ss + (ntl + 1) * 256 + (j * 4 + t) * 16);
#pragma unroll
            for (int mt = 0; mt < MMQ_MT; ++mt) {
                mma_s8_magic2(p01[buf][0][mt], p23[buf][0][mt], a0[mt], a1[mt], a2[mt], a3[mt], b0.x, b0.y);
                mma_s8_magic2(p01[buf][1][mt], p23[buf][1][mt], a0[mt], a1[mt], a2[mt], a3[mt], b1.x, b1.y);
            }
        };
        auto finish = [&](int step, int buf) {
            const int j = step / NP, np = step % NP;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint64_t da = pack2(sc[buf][i].x, sc[buf][i].y);
                const uint64_t nda = fma2(da, pack2(0xCB400000u, 0xCB400000u), 0ull);   // -d * 12582912, exact (d is an fp16 value)
#pragma unroll
                for (int mt = 0; mt < MMQ_MT; ++mt) {
                    const uint64_t t01 = fma2(p01[buf][i][mt], da, nda), t23 = fma2(p23[buf][i][mt], da, nda);
                    y[mt][2 * np + i][0] = fma2(t01, dwa[j & 1][mt], y[mt][2 * np + i][0]);
                    y[mt][2 * np + i][1] = fma2(t23, dwb[j & 1][mt], y[mt][2 * np + i][1]);
                }
            }
        };
#pragma unroll
        for (int step = 0; step < DEPTH - 1; ++step) start(step, step % DEPTH);
#pragma unroll
        for (int step = 0; step < NSTEP; ++step) {
            if (step + DEPTH - 1 < NSTEP) start(step + DEPTH - 1, (step + DEPTH - 1) % DEPTH);
            finish(step, step % DEPTH);
        }
    };
    // write back; Q4_0 quants were used as 16 * value
    constexpr float WS = (WTYPE == B200_TYPE_Q4_0) ? 0.0625f : 1.0f;
    if constexpr (SK) {
        // workspace: one arrival counter per row group (zeroed before the launch), then the slots partial tiles are parked
        // in, each holding the accumulator registers of every thread in thread order -- all CTAs have the same shape, so
        // the CTA that sums reads the values of its own (row, column) positions
        constexpr int NACC = MMQ_MT * NT * 2;
        constexpr int64_t SLOT = (int64_t) NACC * MMQ_THREADS;   // 8-byte pairs
        const int64_t n_groups = dims.n_rt / S::CTA_TILES;
        unsigned *arrived = reinterpret_cast<unsigned *>(partial);
        uint64_t *slots = reinterpret_cast<uint64_t *>(reinterpret_cast<char *>(partial) + ((n_groups * 4 + 255) / 256) * 256);
        __shared__ int sk_flag;
        auto store_group = [&](uint32_t ct) {
#pragma unroll
            for (int mt = 0; mt < MMQ_MT; ++mt) {
                const int64_t row_base = ((int64_t) ct * S::CTA_TILES + wm * MT + mt) * 16 + g;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int64_t col = (nt0 + nt) * 8 + 2 * t;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int64_t row = row_base + h * 8;
                        float v0, v1;
                        unpack2(y[mt][nt][h], v0, v1);
                        if (row < dims.M) {
                            const int64_t sh = SEGS ? peer_row_shift(peers, row) : 0;   // row ranges that belong to different destination tensors
                            if (col < act.N) *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + col * dst_nb_row + row * 4 + sh) = v0 * WS;
                            if (col + 1 < act.N) *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + (col + 1) * dst_nb_row + row * 4 + sh) = v1 * WS;
                        }
                    }
                }
            }
        };
        auto add_part = [&](int64_t slot) {   // y += the part parked in that slot
            const uint64_t *src = slots + slot * SLOT + tid;
            unsigned long long v[NACC];
#pragma unroll
            for (int i = 0; i < NACC; ++i) v[i] = __ldcg(reinterpret_cast<const unsigned long long *>(src + i * MMQ_THREADS));
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                uint64_t &acc = y[i / (NT * 2)][(i / 2) % NT][i & 1];
                float a0, a1;
                unpack2(acc, a0, a1);
                a0 += __uint_as_float((uint32_t) v[i]);
                a1 += __uint_as_float((uint32_t) (v[i] >> 32));
                acc = pack2(__float_as_uint(a0), __float_as_uint(a1));
            }
        };
        const uint64_t G = gridDim.x;
        int64_t it = 0;
        while (it < n_iter) {
            uint32_t ct, bg0;
            sk_where(it, ct, bg0);
            const int64_t seg_end = it < (int64_t) sk_head ? (int64_t) sk_head : min(n_iter, it + (int64_t) (sk_nbg - bg0));
            const int64_t seg_len = seg_end - it;
#pragma unroll
            for (int mt = 0; mt < MMQ_MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) y[mt][nt][0] = y[mt][nt][1] = 0ull;
            for (; it < seg_end; ++it) body(it);
            if (it == n_iter) pdl_trigger();
            if (seg_len == (int64_t) sk_nbg) {   // the whole K range of this row group: no parts
                store_group(ct);
                continue;
            }
            // The parts of row group ct in K order, their slots, and which of them this one is.
            //   even deal: the CTA of iteration i is the largest j with j * total / G <= i; CTA j parks a piece that starts
            //     where its range starts in slot 2j, the piece its range ends with in slot 2j + 1;
            //   head/tail deal: slot 3 ct is the head, 3 ct + 1 the tail from block group h, 3 ct + 2 the rest of a tail
            //     that two CTAs share.
            uint32_t parts, own;
            uint32_t first = 0;
            if (sk_h == 0) {
                first = (uint32_t) ((((uint64_t) ct * sk_nbg + 1) * G - 1) / sk_total);
                parts = (uint32_t) ((((uint64_t) (ct + 1) * sk_nbg) * G - 1) / sk_total) - first + 1;
                own = blockIdx.x - first;
            } else {
                const uint64_t all = (uint64_t) sk_groups * sk_sl;
                const uint32_t ca = (uint32_t) ((((uint64_t) ct * sk_sl + 1) * sk_gs - 1) / all);
                const uint32_t cb = (uint32_t) ((((uint64_t) (ct + 1) * sk_sl) * sk_gs - 1) / all);
                parts = 2 + (cb - ca);
                own = bg0 == 0 ? 0u : (bg0 == sk_h ? 1u : 2u);
            }
            auto slot_of = [&](uint32_t p) -> int64_t {
                if (sk_h != 0) return (int64_t) ct * 3 + p;
                const uint32_t j = first + p;
                const uint32_t j_it0 = (uint32_t) ((uint64_t) j * sk_total / G);
                return (int64_t) j * 2 + (j_it0 >= ct * sk_nbg ? 0 : 1);
            };
            // If every other part is already parked, add them to the registers and write the rows out: nothing of this
            // part goes through memory.  Only for the first or second part in K order, where (own + p0) + p2 ... are the
            // same bits as the sum from zero in K order (a + b = b + a), so the result does not depend on who finishes.
            if (tid == 0) {
                unsigned seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(arrived + ct) : "memory");
                sk_flag = own <= 1 && seen == parts - 1;
            }
            __syncthreads();
            if (sk_flag) {
                for (uint32_t p = 0; p < parts; ++p)
                    if (p != own) add_part(slot_of(p));
                store_group(ct);
                __syncthreads();   // sk_flag is rewritten by the next part
                continue;
            }
            uint64_t *mine = slots + slot_of(own) * SLOT + tid;
#pragma unroll
            for (int i = 0; i < NACC; ++i) __stcg(reinterpret_cast<unsigned long long *>(mine + i * MMQ_THREADS), (unsigned long long) y[i / (NT * 2)][(i / 2) % NT][i & 1]);
            __threadfence();
            __syncthreads();
            if (tid == 0) sk_flag = atomicAdd(arrived + ct, 1u) == parts - 1;
            __syncthreads();
            if (sk_flag) {   // arrived last: add all parts in K order, this CTA's own from memory too
                __threadfence();
#pragma unroll
                for (int mt = 0; mt < MMQ_MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) y[mt][nt][0] = y[mt][nt][1] = 0ull;
                for (uint32_t p = 0; p < parts; ++p) add_part(slot_of(p));
                store_group(ct);
            }
            __syncthreads();
        }
        cp_async_wait<0>();
        return;
    } else {
        for (int64_t it = 0; it < n_iter; ++it) body(it);
    }
    cp_async_wait<0>();
    pdl_trigger();

    if (cluster) {
        // The K splits of one output tile form a thread-block cluster (cluster dimension z = ksplit).  Every CTA parks its
        // partial tile in its own shared memory; after a cluster barrier CTA r sums slice r of the tile over all CTAs,
        // in split order, through distributed shared memory and writes it out.  No partial sums in global memory, no
        // second kernel, and the summation order is fixed.
        constexpr int ROWS = S::CTA_TILES * 16, COLS = S::NT * 8, TOTAL4 = ROWS * COLS / 4;
        static_assert(ROWS * COLS * 4 <= S::TOTAL, "the partial tile reuses the copy ring");
        __syncthreads();   // every warp is done with the ring
        float *red = reinterpret_cast<float *>(smem);   // [col][row]
#pragma unroll
        for (int mt = 0; mt < MMQ_MT; ++mt) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float v0, v1;
                    unpack2(y[mt][nt][h], v0, v1);
                    const int r = (wm * MT + mt) * 16 + g + h * 8, c = (wn * NTW + nt) * 8 + 2 * t;
                    red[c * ROWS + r] = v0 * WS;
                    red[(c + 1) * ROWS + r] = v1 * WS;
                }
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        const int per4 = (TOTAL4 + ksplit - 1) / ksplit;   // float4 groups (4 consecutive rows of one column) per CTA
        const uint32_t red_u32 = (uint32_t) __cvta_generic_to_shared(red);
        for (int i = tid; i < per4; i += MMQ_THREADS) {
            const int q4 = ks * per4 + i;
            if (q4 >= TOTAL4) break;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < ksplit; ++k) {
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(red_u32 + (uint32_t) q4 * 16u), "r"(k));
                float4 v;
                asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            const int c = (q4 * 4) / ROWS, r = (q4 * 4) % ROWS;
            const int64_t col = cta_nt0 * 8 + c, row = cta_rt0 * 16 + r;
            if (col < act.N) {
                const int64_t off = col * dst_nb_row + row * 4 + (MODE == MMQ_PEER ? peer_row_shift(peers, row) : 0);
                const int n_peers = MODE == MMQ_PEER ? peers.n : 0;
                for (int pi = -1; pi < n_peers; ++pi) {   // own buffer, then the other GPUs' of a row split
                    float *o = reinterpret_cast<float *>(reinterpret_cast<char *>(pi < 0 ? dst : peers.p[pi]) + off);
                    if (row + 3 < dims.M && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
                        *reinterpret_cast<float4 *>(o) = acc;
                    } else {
                        if (row < dims.M) o[0] = acc.x;
                        if (row + 1 < dims.M) o[1] = acc.y;
                        if (row + 2 < dims.M) o[2] = acc.z;
                        if (row + 3 < dims.M) o[3] = acc.w;
                    }
                }
            }
        }
        // nobody leaves while a neighbour may still read its tile
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        return;
    }
#pragma unroll
    for (int mt = 0; mt < MMQ_MT; ++mt) {
        const int64_t row_base = (rt0 + mt) * 16 + g;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int64_t col = (nt0 + nt) * 8 + 2 * t;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t row = row_base + h * 8;
                float v0, v1;
                unpack2(y[mt][nt][h], v0, v1);
                v0 *= WS;
                v1 *= WS;
                if (row < dims.M) {
                    if (ksplit == 1) {
                        if (MODE == MMQ_PEER) {
                            const int64_t sh = peer_row_shift(peers, row);
                            if (col < act.N) store_f32(dst, peers, col * dst_nb_row + row * 4 + sh, v0);
                            if (col + 1 < act.N) store_f32(dst, peers, (col + 1) * dst_nb_row + row * 4 + sh, v1);
                        } else {
                            if (col < act.N) *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + col * dst_nb_row + row * 4) = v0;
                            if (col + 1 < act.N) *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + (col + 1) * dst_nb_row + row * 4) = v1;
                        }
                    } else {
                        if (col < act.N) partial[((int64_t) ks * act.N + col) * dims.M + row] = v0;
                        if (col + 1 < act.N) partial[((int64_t) ks * act.N + col + 1) * dims.M + row] = v1;
                    }
                }
            }
        }
    }
}

// dst[n][m] = sum over splits of partial[s][n][m], in split order
__global__ void __launch_bounds__(256) mmq_reduce_kernel(const float *__restrict__ partial, int ksplit, int64_t M, int64_t N,
                                                        float *__restrict__ dst, int64_t dst_nb_row, PeerDst peers) {
    pdl_prologue();
    const int64_t gid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= M * N) return;
    const int64_t n = gid / M, m = gid - n * M;
    float s = 0.0f;
    for (int k = 0; k < ksplit; ++k) s += partial[((int64_t) k * N + n) * M + m];
    store_f32(dst, peers, n * dst_nb_row + m * 4 + peer_row_shift(peers, m), s);
}

// The per-device tables below are filled on first use; calls may come from several host threads (one backend per thread
// is a supported way to drive the C ABI), so every table has its lock.
static int sm_count() {
    static int n[64] = {0};
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    std::lock_guard<std::mutex> lock(mu);
    if (!n[dev]) {
        cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
        if (n[dev] <= 0) n[dev] = 148;
    }
    return n[dev];
}

// One launchable CTA shape: how many rows / columns a CTA covers, how many CTAs fit on an SM, and the launcher.
struct MmqVariant {
    int cta_tiles;   // 16-row tiles per CTA
    int cta_nt;      // 8-column tiles per CTA
    int ctas_per_sm; // resident CTAs per SM (filled on first use)
    int (*launch)(const TiledDims &, const uint8_t *, const ActDims &, const uint8_t *, float *, int64_t, float *, int, int, int, const PeerDst &, cudaStream_t);
    int (*max_clusters)(int);   // resident clusters of `ksplit` CTAs on this device (0 = cannot be launched that way)
    int (*launch_streamk)(const TiledDims &, const uint8_t *, const ActDims &, const uint8_t *, float *, int64_t, void *, int, int, int, const PeerDst &, cudaStream_t);
    size_t streamk_slot_bytes;  // one partial tile of a CTA in the stream-K workspace
};

__global__ void zero_u32_kernel(unsigned *p, int n) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = 0u;
}

static size_t streamk_counter_bytes(int64_t n_groups) { return (size_t) ((n_groups * 4 + 255) / 256) * 256; }

// stream-K launch: `ctas` CTAs (one per resident slot), arrival counters zeroed first; head = 0 for the even deal, else
// the block groups of a head in the head/tail deal
template <int WTYPE, int NTW, int WN, int MT, int WM, int STAGES, int MINB>
static int launch_variant_streamk(const TiledDims &d, const uint8_t *w, const ActDims &a, const uint8_t *aq, float *dst, int64_t dst_nb_row,
                                  void *workspace, int ctas, int head, int canon, const PeerDst &segs, cudaStream_t st) {
    using S = MmqCfg<WTYPE, NTW, WN, MT, WM, STAGES>;
    const int n_groups = (int) (d.n_rt / S::CTA_TILES);
    launch_pdl(zero_u32_kernel, dim3((unsigned) ((n_groups + 255) / 256)), dim3(256), 0, st, (unsigned *) workspace, n_groups);
    if (int e = check_launch("mmq stream-K counters")) return e;
    if (segs.n_seg > 1) launch_pdl(mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_STREAMK_SEG>, dim3((unsigned) ctas), dim3(S::THREADS), S::TOTAL, st, d, w, a,
                                   aq, dst, dst_nb_row, (float *) workspace, head, canon, 0, segs);   // segs: row ranges only, never peers
    else launch_pdl(mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_STREAMK>, dim3((unsigned) ctas), dim3(S::THREADS), S::TOTAL, st, d, w, a, aq, dst,
                    dst_nb_row, (float *) workspace, head, canon, 0, PeerDst{});
    return check_launch("mmq stream-K");
}

template <int WTYPE, int NTW, int WN, int MT, int WM, int STAGES, int MINB>
static int launch_variant(const TiledDims &d, const uint8_t *w, const ActDims &a, const uint8_t *aq, float *dst, int64_t dst_nb_row,
                          float *partial, int ksplit, int canon, int cluster, const PeerDst &peers, cudaStream_t st) {
    using S = MmqCfg<WTYPE, NTW, WN, MT, WM, STAGES>;
    dim3 grid((unsigned) ((d.n_rt + S::CTA_TILES - 1) / S::CTA_TILES), (unsigned) ((a.n_nt + S::NT - 1) / S::NT), (unsigned) ksplit);
    const bool peer = peers.n > 0 || peers.n_seg > 1;
    if (!cluster) {
        if (peer) launch_pdl(mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_PEER>, grid, dim3(S::THREADS), S::TOTAL, st, d, w, a, aq, dst, dst_nb_row, partial, ksplit, canon, 0, peers);
        else launch_pdl(mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_PLAIN>, grid, dim3(S::THREADS), S::TOTAL, st, d, w, a, aq, dst, dst_nb_row, partial, ksplit, canon, 0, peers);
        return check_launch("mmq");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(S::THREADS);
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned) ksplit;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = peer ? cudaLaunchKernelEx(&cfg, mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_PEER>, d, w, a, aq, dst, dst_nb_row, partial, ksplit, canon, 1, peers)
                         : cudaLaunchKernelEx(&cfg, mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_PLAIN>, d, w, a, aq, dst, dst_nb_row, partial, ksplit, canon, 1, peers);
    if (e != cudaSuccess) return set_error(B200_E_CUDA, "mmq cluster launch: %s", cudaGetErrorString(e));
    count_launch();
    return B200_OK;
}

template <int WTYPE, int NTW, int WN, int MT, int WM, int STAGES, int MINB>
static int max_clusters_variant(int ksplit) {
    using S = MmqCfg<WTYPE, NTW, WN, MT, WM, STAGES>;
    static int cache[64][9];   // per device and cluster size: 0 = not asked yet, -1 = none, else the count
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (ksplit < 2 || ksplit > 8) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev][ksplit] != 0) return cache[dev][ksplit] < 0 ? 0 : cache[dev][ksplit];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, (unsigned) ksplit);
    cfg.blockDim = dim3(S::THREADS);
    cfg.dynamicSmemBytes = S::TOTAL;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned) ksplit;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    cache[dev][ksplit] = n > 0 ? n : -1;
    return n;
}

template <int WTYPE, int NTW, int WN, int MT, int WM, int STAGES = 4, int MINB = 1>
static MmqVariant make_variant() {
    using S = MmqCfg<WTYPE, NTW, WN, MT, WM, STAGES>;
    MmqVariant v;
    v.cta_tiles = S::CTA_TILES;
    v.cta_nt = S::NT;
    v.launch = launch_variant<WTYPE, NTW, WN, MT, WM, STAGES, MINB>;
    v.max_clusters = max_clusters_variant<WTYPE, NTW, WN, MT, WM, STAGES, MINB>;
    v.launch_streamk = launch_variant_streamk<WTYPE, NTW, WN, MT, WM, STAGES, MINB>;
    v.streamk_slot_bytes = (size_t) S::CTA_TILES * 16 * S::NT * 8 * sizeof(float);
    cudaFuncSetAttribute(mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_STREAMK>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    cudaFuncSetAttribute(mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_STREAMK_SEG>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    cudaFuncSetAttribute(mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    cudaFuncSetAttribute(mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB, MMQ_PEER>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, mmq_kernel<WTYPE, NTW, WN, MT, WM, STAGES, MINB>, S::THREADS, S::TOTAL) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 1;
    }
    v.ctas_per_sm = n;
    return v;
}

// Variants per (weight type, column class).  Column classes: <= 16, <= 32, more (64-column chunks).
// Index 0 is the default; B200_MMQ_VARIANT=<i> selects another one (tuning aid).
template <int WTYPE>
static const MmqVariant &pick_variant(int64_t N) {
    // per device: kernel attributes and occupancy are per-context properties
    static MmqVariant table[64][3][4];
    static bool ready[64] = {false};
    static std::mutex mu;
    static const int forced = [] {
        const char *e = getenv("B200_MMQ_VARIANT");
        return e ? atoi(e) : -1;
    }();
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    std::lock_guard<std::mutex> lock(mu);
    if (!ready[dev]) {
        MmqVariant(*t)[4] = table[dev];
        t[0][0] = make_variant<WTYPE, 2, 1, 2, 4>();   // 128 rows x 16 cols, 4 warps
        t[0][1] = make_variant<WTYPE, 2, 1, 1, 4>();   //  64 rows x 16 cols
        t[0][2] = t[0][0]; t[0][3] = t[0][0];
        t[1][0] = make_variant<WTYPE, 4, 1, 2, 4>();   // 128 rows x 32 cols
        t[1][1] = make_variant<WTYPE, 4, 1, 1, 4>();
        t[1][2] = t[1][0]; t[1][3] = t[1][0];
        t[2][0] = make_variant<WTYPE, 8, 1, 2, 4, 4, 2>();   // 128 rows x 64 cols, a warp owns all 64 columns, 2 CTAs/SM
        t[2][1] = make_variant<WTYPE, 8, 1, 2, 4, 3, 3>();   // as [0] with 3 stages and 168 registers: 3 CTAs/SM
        t[2][2] = make_variant<WTYPE, 4, 2, 4, 1, 4, 3>();   //  64 rows x 64 cols, 2 warps, warp tile 64 x 32
        t[2][3] = make_variant<WTYPE, 4, 2, 2, 4, 3, 2>();   // 128 rows x 64 cols, 8 warps as 4 x 2, 3 stages
        ready[dev] = true;
    }
    static const int forced_cls = [] {   // B200_MMQ_CLASS=<0..2>: column class whatever N (tuning aid: narrower CTAs, more column chunks)
        const char *e = getenv("B200_MMQ_CLASS");
        return e ? atoi(e) : -1;
    }();
    const int cls = (forced_cls >= 0 && forced_cls <= 2) ? forced_cls : (N > 32 ? 2 : (N > 16 ? 1 : 0));
    return table[dev][cls][(forced >= 0 && forced < 4) ? forced : 0];
}

// K splits: the CTA count is made to fit whole waves of resident CTAs; each split pays about three block
// groups of fixed cost (pipeline fill, write-back).  Up to 8 splits can run as one thread-block cluster that sums
// its partial tiles through distributed shared memory; more splits, or a device that cannot place such clusters,
// write partial sums to the workspace for the reduction kernel (about two block groups' worth of time more).
static int choose_ksplit(const MmqVariant &v, const TiledDims &d, int64_t n_nt, bool *cluster) {
    static const int allow = [] {
        const char *e = getenv("B200_MMQ_CLUSTER");
        return (e && atoi(e) == 0) ? 0 : 1;
    }();
    const int64_t ctas = ((d.n_rt + v.cta_tiles - 1) / v.cta_tiles) * ((n_nt + v.cta_nt - 1) / v.cta_nt);
    const int64_t slots = (int64_t) sm_count() * v.ctas_per_sm;
    int best = 1;
    int64_t best_cost = -1;
    *cluster = false;
    for (int ks = 1; ks <= 16; ++ks) {
        const int64_t per = (d.n_bg + ks - 1) / ks;
        if (ks > 1 && per < 2) break;
        const int64_t waves = (ctas * ks + slots - 1) / slots;
        const int64_t cost = 2 * (waves * (per + 3) + (ks > 1 ? 2 : 0));
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = ks;
            *cluster = false;
        }
        if (allow && ks >= 2 && ks <= 8) {
            const int64_t cslots = (int64_t) v.max_clusters(ks) * ks;
            if (cslots > 0) {
                const int64_t cwaves = (ctas * ks + cslots - 1) / cslots;
                const int64_t ccost = 2 * cwaves * (per + 3) + 1;
                if (ccost < best_cost) {
                    best_cost = ccost;
                    best = ks;
                    *cluster = true;
                }
            }
        }
    }
    return best;
}

static const MmqVariant &variant_for(int wtype, int64_t N) {
    return wtype == B200_TYPE_Q4_0 ? pick_variant<B200_TYPE_Q4_0>(N) : pick_variant<B200_TYPE_Q8_0>(N);
}

// Up to this many activation columns the dp4a kernel (mmvq.cu) runs; its time grows with the columns (9.9, 10.9, 14.9,
// 17.0 us for 1..4 columns of a 14336 x 4096 Q4_0 weight on B200), where the tensor-core kernel's 16-column tile costs
// 13.4 us for any count up to 16.
int mmvq_max_n() {
    static const int v = [] {
        const char *e = getenv("B200_MMVQ_MAX_N");
        return e ? std::max(2, std::min(8, atoi(e))) : 2;
    }();
    return v;
}

size_t mmq_workspace_bytes(int wtype, int64_t K, int64_t M, int64_t N) {
    if (N <= 2) return 0;   // never the tensor-core kernel (mmvq_max_n() is 2 ... 8: columns 3..8 may need it)
    // upper bound over every K split the launcher may choose (the choice depends on the device): never more
    // than 16, than half the block groups, or than what two waves of the largest plausible device need
    const TiledDims d = tiled_dims(wtype, K, M);
    const int64_t ctas = ((d.n_rt + 7) / 8) * ((N + 63) / 64);
    int64_t ks = std::min<int64_t>(16, std::max<int64_t>(1, d.n_bg / 2));
    ks = std::min<int64_t>(ks, std::max<int64_t>(1, (2368 + ctas - 1) / ctas));
    const size_t splitk = ks > 1 ? align_up((size_t) ks * N * M * sizeof(float), 256) : 0;
    // stream-K (one column chunk only): counters + three partial tiles of 128 rows x 64 columns for each of at most 3 CTAs per SM
    const size_t streamk = N <= 64 ? streamk_counter_bytes(d.n_rt) + (size_t) sm_count() * 3 * 3 * (128 * 64 * sizeof(float)) : 0;
    return std::max(splitk, streamk);
}

// Stream-K is taken when the product has a single column chunk, whole row groups, and dealing the iterations out beats
// the best wave-quantised split.  With at least as many row groups as resident CTAs
// the deal is even; with between half as many and as many, heads and tails (*head = block groups of a head, chosen so
// that the CTAs sharing the tails are done two block groups before the heads).  Fewer row groups are left to the
// cluster split.  B200_MMQ_STREAMK=0 turns it off, =2 takes it whenever it is legal.
static int streamk_ctas(const MmqVariant &v, const TiledDims &d, const ActDims &a, int ks, bool cluster, size_t workspace_bytes, int *head) {
    static const int mode = [] {
        const char *e = getenv("B200_MMQ_STREAMK");
        return e ? atoi(e) : 1;
    }();
    *head = 0;
    if (mode == 0 || a.n_nt > v.cta_nt || d.n_rt % v.cta_tiles != 0) return 0;
    const int64_t groups = d.n_rt / v.cta_tiles, total = groups * d.n_bg;
    const int64_t slots = (int64_t) sm_count() * v.ctas_per_sm;
    if (total >= (1ll << 31) || groups == slots) return 0;
    if (workspace_bytes < streamk_counter_bytes(groups) + (size_t) slots * 3 * v.streamk_slot_bytes) return 0;
    if (groups < slots) {
        if (2 * groups < slots) return 0;
        const int64_t gs = slots - groups;
        const int64_t h = (total + 2 * gs + slots - 1) / slots;
        if (h < 2 || h >= d.n_bg || groups * (d.n_bg - h) < gs) return 0;
        *head = (int) h;
    }
    if (mode >= 2) return (int) slots;
    // An SM works through its CTAs' block groups at about the same rate whether one or two CTAs are resident (measured:
    // 1.07 us per block group alone, 1.85 us for one of each of two), so what counts is the block groups per SM: the
    // fullest SM of the wave-quantised launch against the even share plus about eight block groups for the counter
    // reset, the parked parts and the last read.
    const int64_t sms = sm_count();
    const int64_t per = (d.n_bg + ks - 1) / ks;
    const int64_t now = (groups * ks + sms - 1) / sms * (per + 3);
    const int64_t sk = (total + sms - 1) / sms + 8;
    (void) cluster;
    return sk < now ? (int) slots : 0;
}

void launch_mmq_reduce(const float *partial, int ks, int64_t M, int64_t N, float *dst, int64_t dst_nb_row, cudaStream_t st) {
    const int64_t total = M * N;
    launch_pdl(mmq_reduce_kernel, dim3((unsigned) ((total + 255) / 256)), dim3(256), 0, st, partial, ks, M, N, dst, dst_nb_row, PeerDst{});
}

int launch_mmq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
               void *workspace, size_t workspace_bytes, cudaStream_t st, bool canon, const PeerDst &peers) {
    const MmqVariant &v = variant_for(wtype, a.N);
    bool cluster = false;
    int ks = choose_ksplit(v, d, a.n_nt, &cluster);
    const size_t per_split = (size_t) a.N * d.M * sizeof(float);
    if (ks > 1 && !cluster && (!workspace || workspace_bytes < per_split * ks)) {
        ks = workspace ? (int) std::max<size_t>(1, workspace_bytes / per_split) : 1;  // fewer splits fit: still correct, only slower
    }
    if (peers.n == 0 && (peers.n_seg <= 1 || peers.n_wseg > 0) && workspace) {   // (the ranges of a row-split rank keep the plain grid)
        int head = 0;
        if (const int ctas = streamk_ctas(v, d, a, ks, cluster, workspace_bytes, &head))
            return v.launch_streamk(d, (const uint8_t *) w, a, (const uint8_t *) aq, dst, dst_nb_row, workspace, ctas, head, canon ? 1 : 0, peers, st);
    }
    if (int e = v.launch(d, (const uint8_t *) w, a, (const uint8_t *) aq, dst, dst_nb_row, (float *) workspace, ks, canon ? 1 : 0, cluster ? 1 : 0, peers, st)) return e;
    if (ks > 1 && !cluster) {
        const int64_t total = d.M * a.N;
        launch_pdl(mmq_reduce_kernel, dim3((unsigned) ((total + 255) / 256)), dim3(256), 0, st, (const float *) workspace, ks, d.M, a.N, dst, dst_nb_row, peers);
        return check_launch("mmq_reduce");
    }
    return B200_OK;
}

}  // namespace b200
