// MUL_MAT for many activation columns (N > 8): int8 tensor-core kernel with per-block fp16 scales.
//
// Replaces the chunked vec_dot loop of lm_ggml_compute_forward_mul_mat
// (cactus/ggml-cpu/ggml-cpu.c:1257-1449).  Every 32-element block has its own pair of scales, so each
// k=32 MMA step produces a fresh int32 tile that is converted and folded into fp32 accumulators with
// the outer product of the weight and activation block scales.
//
// CTA tile 64 rows x BN columns, 4 warps as 2 (rows) x 2 (columns), warp tile 32 x BN/2.  Weight tiles
// (already in A-fragment order) and activation tiles (B-fragment order) are copied verbatim into a
// 4-stage cp.async ring, one block group (K = 128) per stage; fragments are then plain 128/64-bit shared
// loads without bank conflicts.  grid = (row groups, column chunks, K splits); with K splits > 1 the
// partial tiles go to a workspace and a second kernel adds them in a fixed order.
#include "common.cuh"

namespace b200 {

constexpr int MMQ_STAGES = 4;
constexpr int MMQ_BM_TILES = 4;  // 16-row tiles per CTA

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const uint32_t s = (uint32_t) __cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

template <int WTYPE, int BN>
struct MmqSmem {
    static constexpr int TILE = (WTYPE == B200_TYPE_Q4_0) ? 1024 : 2048;
    static constexpr int A_BYTES = MMQ_BM_TILES * TILE;
    static constexpr int AS_BYTES = MMQ_BM_TILES * 128;
    static constexpr int B_BYTES = (BN / 8) * 1024;
    static constexpr int BS_BYTES = (BN / 8) * 64;
    static constexpr int STAGE = A_BYTES + AS_BYTES + B_BYTES + BS_BYTES;
    static constexpr int TOTAL = STAGE * MMQ_STAGES;
};

template <int WTYPE, int BN>
__global__ void __launch_bounds__(128) mmq_kernel(TiledDims dims, const uint8_t *__restrict__ w, ActDims act,
                                                 const uint8_t *__restrict__ aq, float *__restrict__ dst, int64_t dst_nb_row,
                                                 float *__restrict__ partial, int ksplit) {
    using S = MmqSmem<WTYPE, BN>;
    constexpr int NTW = BN / 16;  // n-tiles per warp
    extern __shared__ __align__(128) uint8_t smem[];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp >> 1, wn = warp & 1;
    const int64_t rt0 = (int64_t) blockIdx.x * MMQ_BM_TILES;
    const int64_t nt0 = (int64_t) blockIdx.y * (BN / 8);
    const int ks = blockIdx.z;
    // block groups of this K split
    const int64_t per = (dims.n_bg + ksplit - 1) / ksplit;
    const int64_t bg_begin = ks * per;
    const int64_t bg_end = min(dims.n_bg, bg_begin + per);
    const int64_t n_iter = max((int64_t) 0, bg_end - bg_begin);

    auto issue = [&](int64_t it) {
        uint8_t *st = smem + (it % MMQ_STAGES) * S::STAGE;
        const int64_t bg = bg_begin + it;
        // weights: MMQ_BM_TILES tiles of TILE bytes, then their scales
        constexpr int A_CH = S::A_BYTES / 16;
        for (int c = tid; c < A_CH; c += 128) {
            const int tile = c / (S::TILE / 16), off = c % (S::TILE / 16);
            const int64_t rt = min(rt0 + tile, dims.n_rt - 1);  // clamp: rows beyond the matrix are never written back
            cp_async16(st + c * 16, w + (rt * dims.n_bg + bg) * S::TILE + off * 16);
        }
        constexpr int AS_CH = S::AS_BYTES / 16;
        for (int c = tid; c < AS_CH; c += 128) {
            const int tile = c / 8, off = c % 8;
            const int64_t rt = min(rt0 + tile, dims.n_rt - 1);
            cp_async16(st + S::A_BYTES + c * 16, w + dims.qs_bytes + (rt * dims.n_bg + bg) * 128 + off * 16);
        }
        constexpr int B_CH = S::B_BYTES / 16;
        for (int c = tid; c < B_CH; c += 128) {
            const int tile = c / 64, off = c % 64;
            const int64_t nt = min(nt0 + tile, act.n_nt - 1);
            cp_async16(st + S::A_BYTES + S::AS_BYTES + c * 16, aq + (nt * act.nbp + bg * 4) * 256 + off * 16);
        }
        constexpr int BS_CH = S::BS_BYTES / 16;
        for (int c = tid; c < BS_CH; c += 128) {
            const int tile = c / 4, off = c % 4;
            const int64_t nt = min(nt0 + tile, act.n_nt - 1);
            cp_async16(st + S::A_BYTES + S::AS_BYTES + S::B_BYTES + c * 16, aq + act.d_offset + (nt * act.n_bg + bg) * 64 + off * 16);
        }
    };

    float y[2][NTW][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) y[mt][nt][c] = 0.0f;

    for (int s = 0; s < MMQ_STAGES - 1; ++s) {
        if (s < n_iter) issue(s);
        cp_async_commit();
    }

    constexpr float WS = (WTYPE == B200_TYPE_Q4_0) ? 0.0625f : 1.0f;

    for (int64_t it = 0; it < n_iter; ++it) {
        cp_async_wait<MMQ_STAGES - 2>();
        __syncthreads();
        if (it + MMQ_STAGES - 1 < n_iter) issue(it + MMQ_STAGES - 1);
        cp_async_commit();

        const uint8_t *st = smem + (it % MMQ_STAGES) * S::STAGE;
        const uint8_t *As = st, *Asc = st + S::A_BYTES, *Bs = st + S::A_BYTES + S::AS_BYTES, *Bsc = Bs + S::B_BYTES;

        // weight fragments and scales of the warp's two row tiles
        uint32_t wa[2][8], wb[2][8];
        float dwa[2][4], dwb[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const int tile = wm * 2 + mt;
            if (WTYPE == B200_TYPE_Q4_0) {
                const uint4 *p = reinterpret_cast<const uint4 *>(As + tile * 1024) + lane * 2;
                const uint4 u0 = p[0], u1 = p[1];
                wa[mt][0] = u0.x; wa[mt][1] = u0.y; wa[mt][2] = u0.z; wa[mt][3] = u0.w;
                wb[mt][0] = u1.x; wb[mt][1] = u1.y; wb[mt][2] = u1.z; wb[mt][3] = u1.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 u = reinterpret_cast<const uint4 *>(As + tile * 2048 + j * 512)[lane];
                    wa[mt][2 * j] = u.x; wb[mt][2 * j] = u.y; wa[mt][2 * j + 1] = u.z; wb[mt][2 * j + 1] = u.w;
                }
            }
            const uint2 sa = reinterpret_cast<const uint2 *>(Asc + tile * 128)[g];
            const uint2 sb = reinterpret_cast<const uint2 *>(Asc + tile * 128)[g + 8];
            const __half2 a01 = *reinterpret_cast<const __half2 *>(&sa.x), a23 = *reinterpret_cast<const __half2 *>(&sa.y);
            const __half2 b01 = *reinterpret_cast<const __half2 *>(&sb.x), b23 = *reinterpret_cast<const __half2 *>(&sb.y);
            dwa[mt][0] = __low2float(a01) * WS; dwa[mt][1] = __high2float(a01) * WS;
            dwa[mt][2] = __low2float(a23) * WS; dwa[mt][3] = __high2float(a23) * WS;
            dwb[mt][0] = __low2float(b01) * WS; dwb[mt][1] = __high2float(b01) * WS;
            dwb[mt][2] = __low2float(b23) * WS; dwb[mt][3] = __high2float(b23) * WS;
        }

#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            const int ntl = wn * NTW + nt;
            // activation scales of columns 2t and 2t+1, four blocks each
            const uint2 s0 = reinterpret_cast<const uint2 *>(Bsc + ntl * 64)[2 * t];
            const uint2 s1 = reinterpret_cast<const uint2 *>(Bsc + ntl * 64)[2 * t + 1];
            const __half2 e01 = *reinterpret_cast<const __half2 *>(&s0.x), e23 = *reinterpret_cast<const __half2 *>(&s0.y);
            const __half2 f01 = *reinterpret_cast<const __half2 *>(&s1.x), f23 = *reinterpret_cast<const __half2 *>(&s1.y);
            const float da0[4] = {__low2float(e01), __high2float(e01), __low2float(e23), __high2float(e23)};
            const float da1[4] = {__low2float(f01), __high2float(f01), __low2float(f23), __high2float(f23)};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint2 b = reinterpret_cast<const uint2 *>(Bs + ntl * 1024 + j * 256)[lane];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    uint32_t a0, a1, a2, a3;
                    if (WTYPE == B200_TYPE_Q4_0) {
                        a0 = (wa[mt][j] << 4) & 0xF0F0F0F0u; a2 = wa[mt][j] & 0xF0F0F0F0u;
                        a1 = (wb[mt][j] << 4) & 0xF0F0F0F0u; a3 = wb[mt][j] & 0xF0F0F0F0u;
                    } else {
                        a0 = wa[mt][2 * j]; a2 = wa[mt][2 * j + 1];
                        a1 = wb[mt][2 * j]; a3 = wb[mt][2 * j + 1];
                    }
                    int c[4];
                    mma_s8(c, a0, a1, a2, a3, b.x, b.y);
                    y[mt][nt][0] = fmaf(dwa[mt][j] * da0[j], (float) c[0], y[mt][nt][0]);
                    y[mt][nt][1] = fmaf(dwa[mt][j] * da1[j], (float) c[1], y[mt][nt][1]);
                    y[mt][nt][2] = fmaf(dwb[mt][j] * da0[j], (float) c[2], y[mt][nt][2]);
                    y[mt][nt][3] = fmaf(dwb[mt][j] * da1[j], (float) c[3], y[mt][nt][3]);
                }
            }
        }
    }
    cp_async_wait<0>();

    // write back: c0 (row g, col 2t), c1 (g, 2t+1), c2 (g+8, 2t), c3 (g+8, 2t+1)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        const int64_t row_base = (rt0 + wm * 2 + mt) * 16;
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            const int64_t col_base = (nt0 + wn * NTW + nt) * 8 + 2 * t;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int64_t row = row_base + g + (c >> 1) * 8;
                const int64_t col = col_base + (c & 1);
                if (row < dims.M && col < act.N) {
                    if (ksplit == 1) {
                        *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + col * dst_nb_row + row * 4) = y[mt][nt][c];
                    } else {
                        partial[((int64_t) ks * act.N + col) * dims.M + row] = y[mt][nt][c];
                    }
                }
            }
        }
    }
}

// dst[n][m] = sum over splits of partial[s][n][m], in split order
__global__ void __launch_bounds__(256) mmq_reduce_kernel(const float *__restrict__ partial, int ksplit, int64_t M, int64_t N,
                                                        float *__restrict__ dst, int64_t dst_nb_row) {
    const int64_t gid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= M * N) return;
    const int64_t n = gid / M, m = gid - n * M;
    float s = 0.0f;
    for (int k = 0; k < ksplit; ++k) s += partial[((int64_t) k * N + n) * M + m];
    *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + n * dst_nb_row + m * 4) = s;
}

static int g_sm_count = 0;
static int sm_count() {
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

// number of K splits: enough CTAs to fill the device twice over, at least 8 block groups per split
int mmq_ksplit(const TiledDims &d, int64_t N) {
    const int64_t row_groups = (d.n_rt + MMQ_BM_TILES - 1) / MMQ_BM_TILES;
    const int64_t col_chunks = (N + 63) / 64;
    const int64_t ctas = row_groups * col_chunks;
    const int64_t want = 2 * sm_count();
    if (ctas >= want) return 1;
    int64_t ks = (want + ctas - 1) / ctas;
    ks = min(ks, max((int64_t) 1, d.n_bg / 8));
    return (int) min(ks, (int64_t) 16);
}

size_t mmq_workspace_bytes(int wtype, int64_t K, int64_t M, int64_t N) {
    if (N <= 8) return 0;
    const TiledDims d = tiled_dims(wtype, K, M);
    const int ks = mmq_ksplit(d, N);
    return ks > 1 ? align_up((size_t) ks * N * M * sizeof(float), 256) : 0;
}

template <int WTYPE, int BN>
static int launch_mmq_t(const TiledDims &d, const uint8_t *w, const ActDims &a, const uint8_t *aq, float *dst, int64_t dst_nb_row,
                        float *partial, int ksplit, cudaStream_t st) {
    using S = MmqSmem<WTYPE, BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(mmq_kernel<WTYPE, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return set_error(B200_E_CUDA, "mmq smem opt-in: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((unsigned) ((d.n_rt + MMQ_BM_TILES - 1) / MMQ_BM_TILES), (unsigned) ((a.N + BN - 1) / BN), (unsigned) ksplit);
    mmq_kernel<WTYPE, BN><<<grid, 128, S::TOTAL, st>>>(d, w, a, aq, dst, dst_nb_row, partial, ksplit);
    if (int e = check_launch("mmq")) return e;
    if (ksplit > 1) {
        const int64_t total = d.M * a.N;
        mmq_reduce_kernel<<<(unsigned) ((total + 255) / 256), 256, 0, st>>>(partial, ksplit, d.M, a.N, dst, dst_nb_row);
        return check_launch("mmq_reduce");
    }
    return B200_OK;
}

int launch_mmq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
               void *workspace, size_t workspace_bytes, cudaStream_t st) {
    int ks = mmq_ksplit(d, a.N);
    if (ks > 1 && (!workspace || workspace_bytes < (size_t) ks * a.N * d.M * sizeof(float))) {
        return set_error(B200_E_SCRATCH, "mul_mat workspace too small for %d K splits", ks);
    }
    const bool wide = a.N > 32;
    if (wtype == B200_TYPE_Q4_0) {
        return wide ? launch_mmq_t<B200_TYPE_Q4_0, 64>(d, (const uint8_t *) w, a, (const uint8_t *) aq, dst, dst_nb_row, (float *) workspace, ks, st)
                    : launch_mmq_t<B200_TYPE_Q4_0, 32>(d, (const uint8_t *) w, a, (const uint8_t *) aq, dst, dst_nb_row, (float *) workspace, ks, st);
    }
    return wide ? launch_mmq_t<B200_TYPE_Q8_0, 64>(d, (const uint8_t *) w, a, (const uint8_t *) aq, dst, dst_nb_row, (float *) workspace, ks, st)
                : launch_mmq_t<B200_TYPE_Q8_0, 32>(d, (const uint8_t *) w, a, (const uint8_t *) aq, dst, dst_nb_row, (float *) workspace, ks, st);
}

}  // namespace b200
