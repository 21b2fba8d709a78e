// MUL_MAT for few activation columns (1 or 2 by default, at most 8): the HBM-bound decode kernel.
//
// Replaces lm_ggml_vec_dot_q4_0_q8_0 / lm_ggml_vec_dot_q8_0_q8_0 under mul_mat
// (cactus/ggml-cpu/ggml-cpu-quants.c:1906, :3591; cactus/ggml-cpu/ggml-cpu.c:1167-1255).
//
// One CTA per 16-row tile of the weight matrix, 4, 8 or 16 warps splitting the K dimension by block group (launch_mmvq_n
// picks the count with which all row tiles are resident at once).
// A warp streams 1 KB (Q4_0) / 2 KB (Q8_0) tiles with two/four 128-bit loads per lane, lane (g, t)
// holding word t of every block of rows g and g+8, multiplies them against the Q8_0 activation words
// with dp4a and applies the two fp16 block scales per (row, column, block).  Partial sums are folded
// over the four t lanes with shuffles and over the warps through shared memory in a fixed order, so
// the result does not depend on scheduling.
#include <cstdlib>

#include "common.cuh"

namespace b200 {


// MMVQ_WARPS warps split the block groups of a row tile: many when there are few row tiles (a 4096-row weight has only 256
// CTAs, and more warps per CTA are what keeps enough loads in flight), fewer for tall matrices
// DEPTH: tiles a warp has requested beyond the one it works on (1 or 2)
template <int WTYPE, int NC, int MMVQ_WARPS, int DEPTH = 1>
__global__ void __launch_bounds__(MMVQ_WARPS * 32) mmvq_kernel(TiledDims dims, const uint8_t *__restrict__ w, ActDims act,
                                                              const uint8_t *__restrict__ aq, float *__restrict__ dst,
                                                              int64_t dst_nb_row, PeerDst peers, int early) {
    const int64_t rt = blockIdx.x;
    if (early) {
        // the weights of this row tile (one contiguous run of tiles, one of scales) do not depend on the kernel ahead:
        // let the next kernel in, ask for the weights in L2, and only then wait for the activations
        pdl_trigger();
        const uint8_t *q0 = w + rt * dims.n_bg * dims.tile_bytes;
        for (int64_t bg = threadIdx.x; bg < dims.n_bg; bg += MMVQ_WARPS * 32) prefetch_l2_bulk(q0 + bg * dims.tile_bytes, (uint32_t) dims.tile_bytes);
        const uint8_t *s0 = w + dims.qs_bytes + rt * dims.n_bg * 128;
        for (int64_t c = threadIdx.x; c * 16 < dims.n_bg; c += MMVQ_WARPS * 32)
            prefetch_l2_bulk(s0 + c * 2048, (uint32_t) (min((int64_t) 16, dims.n_bg - c * 16) * 128));
    }
    pdl_prologue();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    float y[2][NC];
#pragma unroll
    for (int n = 0; n < NC; ++n) y[0][n] = y[1][n] = 0.0f;

    const uint8_t *wq = w + rt * dims.n_bg * dims.tile_bytes;
    const uint2 *wd = reinterpret_cast<const uint2 *>(w + dims.qs_bytes + rt * dims.n_bg * 128);
    const float *ad = reinterpret_cast<const float *>(aq + act.d_offset);
    constexpr float WS = (WTYPE == B200_TYPE_Q4_0) ? 0.0625f : 1.0f;  // Q4_0 nibbles sit in the high half of each byte: x16

    // the weight tile and its scales of one block group, as loaded: the next group's are requested before this one's are used
    struct Tile {
        uint4 q[WTYPE == B200_TYPE_Q4_0 ? 2 : 4];
        uint2 sa, sb;
    };
    auto load_tile = [&](int64_t bg, Tile &tl) {
        if (WTYPE == B200_TYPE_Q4_0) {
            const uint4 *p = reinterpret_cast<const uint4 *>(wq + bg * 1024) + lane * 2;
            tl.q[0] = __ldg(p);
            tl.q[1] = __ldg(p + 1);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) tl.q[j] = __ldg(reinterpret_cast<const uint4 *>(wq + bg * 2048 + j * 512) + lane);
        }
        tl.sa = __ldg(wd + bg * 16 + g);
        tl.sb = __ldg(wd + bg * 16 + g + 8);
    };
    Tile nxt, nxt2;
    if (warp < dims.n_bg) load_tile(warp, nxt);
    if (DEPTH >= 2 && warp + MMVQ_WARPS < dims.n_bg) load_tile(warp + MMVQ_WARPS, nxt2);
    for (int64_t bg = warp; bg < dims.n_bg; bg += MMVQ_WARPS) {
        const Tile cur = nxt;
        if (DEPTH >= 2) {
            nxt = nxt2;
            if (bg + 2 * MMVQ_WARPS < dims.n_bg) load_tile(bg + 2 * MMVQ_WARPS, nxt2);
        } else if (bg + MMVQ_WARPS < dims.n_bg) {
            load_tile(bg + MMVQ_WARPS, nxt);
        }
        // weights of this tile
        uint32_t wa[8], wb[8];  // row g / row g+8: Q4_0 uses [0..3] (blocks), Q8_0 [2*j], [2*j+1] (word t, word 4+t)
        if (WTYPE == B200_TYPE_Q4_0) {
            const uint4 u0 = cur.q[0], u1 = cur.q[1];
            wa[0] = u0.x; wa[1] = u0.y; wa[2] = u0.z; wa[3] = u0.w;
            wb[0] = u1.x; wb[1] = u1.y; wb[2] = u1.z; wb[3] = u1.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 u = cur.q[j];
                wa[2 * j] = u.x; wb[2 * j] = u.y; wa[2 * j + 1] = u.z; wb[2 * j + 1] = u.w;
            }
        }
        const uint2 sa = cur.sa, sb = cur.sb;
        float dwa[4], dwb[4];
        {
            const __half2 a01 = *reinterpret_cast<const __half2 *>(&sa.x), a23 = *reinterpret_cast<const __half2 *>(&sa.y);
            const __half2 b01 = *reinterpret_cast<const __half2 *>(&sb.x), b23 = *reinterpret_cast<const __half2 *>(&sb.y);
            dwa[0] = __low2float(a01) * WS; dwa[1] = __high2float(a01) * WS; dwa[2] = __low2float(a23) * WS; dwa[3] = __high2float(a23) * WS;
            dwb[0] = __low2float(b01) * WS; dwb[1] = __high2float(b01) * WS; dwb[2] = __low2float(b23) * WS; dwb[3] = __high2float(b23) * WS;
        }
#pragma unroll
        for (int n = 0; n < NC; ++n) {
            float da[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) da[j] = __ldg(ad + bg * 64 + act_scale_index(j, n));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint2 a = __ldg(reinterpret_cast<const uint2 *>(aq + (bg * 4 + j) * 256) + n * 4 + t);
                int s0, s1;
                if (WTYPE == B200_TYPE_Q4_0) {
                    s0 = __dp4a((int) ((wa[j] << 4) & 0xF0F0F0F0u), (int) a.x, 0);
                    s0 = __dp4a((int) (wa[j] & 0xF0F0F0F0u), (int) a.y, s0);
                    s1 = __dp4a((int) ((wb[j] << 4) & 0xF0F0F0F0u), (int) a.x, 0);
                    s1 = __dp4a((int) (wb[j] & 0xF0F0F0F0u), (int) a.y, s1);
                } else {
                    s0 = __dp4a((int) wa[2 * j], (int) a.x, 0);
                    s0 = __dp4a((int) wa[2 * j + 1], (int) a.y, s0);
                    s1 = __dp4a((int) wb[2 * j], (int) a.x, 0);
                    s1 = __dp4a((int) wb[2 * j + 1], (int) a.y, s1);
                }
                y[0][n] = fmaf(dwa[j] * da[j], (float) s0, y[0][n]);
                y[1][n] = fmaf(dwb[j] * da[j], (float) s1, y[1][n]);
            }
        }
    }

    // fold the four t lanes
#pragma unroll
    for (int n = 0; n < NC; ++n) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            y[h][n] += __shfl_xor_sync(0xffffffffu, y[h][n], 1);
            y[h][n] += __shfl_xor_sync(0xffffffffu, y[h][n], 2);
        }
    }
    __shared__ float red[MMVQ_WARPS][16][NC];
    if (t == 0) {
#pragma unroll
        for (int n = 0; n < NC; ++n) {
            red[warp][g][n] = y[0][n];
            red[warp][g + 8][n] = y[1][n];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * NC; i += MMVQ_WARPS * 32) {
        const int n = i >> 4, r = i & 15;
        const int64_t row = rt * 16 + r;
        if (row < dims.M) {
            float s = 0.0f;
#pragma unroll
            for (int wv = 0; wv < MMVQ_WARPS; ++wv) s += red[wv][r][n];
            store_f32(dst, peers, n * dst_nb_row + row * 4 + peer_row_shift(peers, row), s);
        }
    }
}

template <int WTYPE, int NC, int WARPS, int DEPTH>
static int mmvq_ctas_per_sm() {   // resident CTAs of one variant (every device of a process is the same model)
    static const int n = [] {
        int v = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, mmvq_kernel<WTYPE, NC, WARPS, DEPTH>, WARPS * 32, 0) != cudaSuccess || v <= 0) {
            cudaGetLastError();
            v = 1;
        }
        return v;
    }();
    return n;
}
static int mmvq_sm_count() {
    static const int n = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

// A launch of this kernel lasts about as long as one CTA does, so a second, partly filled wave of CTAs costs as much as
// the first: the row tiles should all be resident at once.  More warps per CTA keep more loads in flight per row tile
// (what small matrices need), fewer warps let more CTAs reside.  Taken: the most warps (16, 8, 4) with which all row tiles
// fit at once; with 16 warps a warp requests two tiles ahead.  Measured on B200 at one column (us per launch, 16 / 8 / 4
// warps): 4096 x 4096 (K x M) 4.7 / 5.7 / 8.6, 14336 x 4096 10.1 / 13.9 / 25.6, 4096 x 6144 8.2 / 6.2 / 8.6 (384 row tiles:
// 16 warps need 1.3 waves), 4096 x 14336 12.7 / 12.5 / 9.7 (896 row tiles: 8 warps need 1.2 waves), 4096 x 128256
// 88.9 / 67.8 / 65.0.  B200_MMVQ_CFG=<warps><depth> (42, 81, 162, ...) forces a variant (tuning aid).
template <int WTYPE, int NC>
static int launch_mmvq_n(const TiledDims &d, const uint8_t *w, const ActDims &a, const uint8_t *aq, float *dst, int64_t dst_nb_row, const PeerDst &peers,
                         cudaStream_t st) {
    static const int forced = [] {
        const char *e = getenv("B200_MMVQ_CFG");
        return e ? atoi(e) : 0;
    }();
    const dim3 grid((unsigned) d.n_rt);
    const int early = (peers.n == 0 && a.N <= pdl_early_rows()) ? 1 : 0;
    const int64_t sms = mmvq_sm_count();
    int cfg = forced;
    if (cfg != 41 && cfg != 42 && cfg != 81 && cfg != 82 && cfg != 161 && cfg != 162) {
        if (d.n_bg >= 16 && d.n_rt <= sms * mmvq_ctas_per_sm<WTYPE, NC, 16, 2>()) cfg = 162;
        else if (d.n_rt <= sms * mmvq_ctas_per_sm<WTYPE, NC, 8, 1>()) cfg = 81;
        else if (d.n_rt <= sms * mmvq_ctas_per_sm<WTYPE, NC, 4, 1>()) cfg = 41;
        else cfg = 42;
    }
    switch (cfg) {
        case 41: launch_pdl(mmvq_kernel<WTYPE, NC, 4, 1>, grid, dim3(128), 0, st, d, w, a, aq, dst, dst_nb_row, peers, early); break;
        case 42: launch_pdl(mmvq_kernel<WTYPE, NC, 4, 2>, grid, dim3(128), 0, st, d, w, a, aq, dst, dst_nb_row, peers, early); break;
        case 81: launch_pdl(mmvq_kernel<WTYPE, NC, 8, 1>, grid, dim3(256), 0, st, d, w, a, aq, dst, dst_nb_row, peers, early); break;
        case 82: launch_pdl(mmvq_kernel<WTYPE, NC, 8, 2>, grid, dim3(256), 0, st, d, w, a, aq, dst, dst_nb_row, peers, early); break;
        case 161: launch_pdl(mmvq_kernel<WTYPE, NC, 16, 1>, grid, dim3(512), 0, st, d, w, a, aq, dst, dst_nb_row, peers, early); break;
        default: launch_pdl(mmvq_kernel<WTYPE, NC, 16, 2>, grid, dim3(512), 0, st, d, w, a, aq, dst, dst_nb_row, peers, early); break;
    }
    return check_launch("mmvq");
}

template <int WTYPE>
static int launch_mmvq_t(const TiledDims &d, const uint8_t *w, const ActDims &a, const uint8_t *aq, float *dst,
                         int64_t dst_nb_row, const PeerDst &peers, cudaStream_t st) {
    switch (a.N) {
        case 1: return launch_mmvq_n<WTYPE, 1>(d, w, a, aq, dst, dst_nb_row, peers, st);
        case 2: return launch_mmvq_n<WTYPE, 2>(d, w, a, aq, dst, dst_nb_row, peers, st);
        case 3: return launch_mmvq_n<WTYPE, 3>(d, w, a, aq, dst, dst_nb_row, peers, st);
        case 4: return launch_mmvq_n<WTYPE, 4>(d, w, a, aq, dst, dst_nb_row, peers, st);
        case 5: return launch_mmvq_n<WTYPE, 5>(d, w, a, aq, dst, dst_nb_row, peers, st);
        case 6: return launch_mmvq_n<WTYPE, 6>(d, w, a, aq, dst, dst_nb_row, peers, st);
        case 7: return launch_mmvq_n<WTYPE, 7>(d, w, a, aq, dst, dst_nb_row, peers, st);
        case 8: return launch_mmvq_n<WTYPE, 8>(d, w, a, aq, dst, dst_nb_row, peers, st);
        default: return set_error(B200_E_INVALID, "mmvq handles 1..8 columns, got %lld", (long long) a.N);
    }
}

int launch_mmvq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
                const PeerDst &peers, cudaStream_t st) {
    if (wtype == B200_TYPE_Q4_0) return launch_mmvq_t<B200_TYPE_Q4_0>(d, (const uint8_t *) w, a, (const uint8_t *) aq, dst, dst_nb_row, peers, st);
    return launch_mmvq_t<B200_TYPE_Q8_0>(d, (const uint8_t *) w, a, (const uint8_t *) aq, dst, dst_nb_row, peers, st);
}

}  // namespace b200
