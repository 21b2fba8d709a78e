// Activation quantiser (quantize_row_q8_0), the tiled weight layout converters, GET_ROWS on tiled
// weights and the exact block-dot debug kernel.
#include <cstdlib>

#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------------
// quantize_row_q8_0 (cactus/ggml-cpu/ggml-cpu-quants.c:732-1045).  8 threads per 32-element block,
// 4 elements each; the block maximum is reduced with three shuffles.  LAYOUT 0 writes the reference's
// block_q8_0 stream, LAYOUT 1 the B8 scratch layout (mma.sync fragment order), LAYOUT 3 that plus the e4m3 planes in
// the K-major core-matrix order the tcgen05 kernel's shared-memory descriptors expect (common.cuh, ACT_F8_MIN_N).
// ---------------------------------------------------------------------------------------------
template <int LAYOUT>
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float *__restrict__ x, int64_t x_nb_row, int64_t K,
                                                           int64_t N, int64_t n_rows_padded, int64_t nb, int64_t nbp,
                                                           uint8_t *__restrict__ out, size_t d_offset, int variant, int early) {
    pdl_prologue(early != 0);
    const int64_t gid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int j = (int) (gid & 7);             // which group of 4 elements inside the block
    const int64_t blk = gid >> 3;              // (row, block) index
    const int64_t nblk = (LAYOUT == 0) ? nb : nbp;
    const int64_t n = blk / nblk;
    const int64_t b = blk - n * nblk;
    if (n >= n_rows_padded) return;  // whole groups of 8 lanes leave together (gid>>3 is uniform per group)

    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const bool real = (n < N) && (b < nb);
    if (real) {
        const float *row = (const float *) ((const char *) x + n * x_nb_row) + b * 32 + j * 4;
        if ((((uintptr_t) row) & 15) == 0) {
            const float4 f = *reinterpret_cast<const float4 *>(row);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            v[0] = row[0]; v[1] = row[1]; v[2] = row[2]; v[3] = row[3];
        }
    }
    q8_quantize_store<LAYOUT>(v, out, d_offset, nb, nbp, n, b, j, real, variant);
}

// ---------------------------------------------------------------------------------------------
// Row-major block stream <-> T16.  One thread per (row, block) of the padded index space.
// ---------------------------------------------------------------------------------------------
template <int WTYPE, bool TO_TILED>
__global__ void __launch_bounds__(256) weight_convert_kernel(TiledDims dims, const uint8_t *__restrict__ src,
                                                            uint8_t *__restrict__ dst, int64_t row0, int64_t nrows_padded) {
    const int64_t gid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t r_local = gid / dims.nbp;
    const int64_t b = gid - r_local * dims.nbp;
    if (r_local >= nrows_padded) return;
    const int64_t row = row0 + r_local;
    const bool real = row < dims.M && b < dims.nb;
    constexpr int BB = (WTYPE == B200_TYPE_Q4_0) ? 18 : 34;  // bytes per reference block
    constexpr int NW = (WTYPE == B200_TYPE_Q4_0) ? 4 : 8;    // 32-bit words of quants per block

    const int64_t rt = row >> 4;
    const int r = (int) (row & 15);
    const int g = r & 7;
    const int hi_row = r >> 3;  // 0: row g, 1: row g+8
    const int64_t bg = b >> 2;
    const int jb = (int) (b & 3);
    const uint8_t *tiled_c = TO_TILED ? dst : src;
    uint8_t *tile = const_cast<uint8_t *>(tiled_c) + (rt * dims.n_bg + bg) * dims.tile_bytes;
    __half *dplane = reinterpret_cast<__half *>(const_cast<uint8_t *>(tiled_c) + dims.qs_bytes) + (rt * dims.n_bg + bg) * 64;
    // the row-major side addresses rows relative to row0 (the caller passes a pointer to the chunk)
    const uint8_t *rm_c = TO_TILED ? src : dst;
    uint8_t *rm = const_cast<uint8_t *>(rm_c) + (r_local * dims.nb + b) * BB;

    if (TO_TILED) {
        uint32_t w[NW];
        uint16_t dbits = 0;
        if (real) {
            const uint16_t *p = reinterpret_cast<const uint16_t *>(rm);
            dbits = p[0];
#pragma unroll
            for (int i = 0; i < NW; ++i) w[i] = (uint32_t) p[1 + 2 * i] | ((uint32_t) p[2 + 2 * i] << 16);
        } else {
#pragma unroll
            for (int i = 0; i < NW; ++i) w[i] = (WTYPE == B200_TYPE_Q4_0) ? 0x88888888u : 0u;
        }
        if (WTYPE == B200_TYPE_Q4_0) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                uint32_t *lane = reinterpret_cast<uint32_t *>(tile + (g * 4 + t) * 32);
                lane[hi_row * 4 + jb] = w[t] ^ 0x88888888u;
            }
        } else {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                uint32_t *lane = reinterpret_cast<uint32_t *>(tile + jb * 512 + (g * 4 + t) * 16);
                lane[hi_row] = w[t];
                lane[2 + hi_row] = w[4 + t];
            }
        }
        reinterpret_cast<uint16_t *>(dplane)[r * 4 + jb] = dbits;
    } else {
        if (!real) return;
        uint32_t w[NW];
        if (WTYPE == B200_TYPE_Q4_0) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint32_t *lane = reinterpret_cast<const uint32_t *>(tile + (g * 4 + t) * 32);
                w[t] = lane[hi_row * 4 + jb] ^ 0x88888888u;
            }
        } else {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint32_t *lane = reinterpret_cast<const uint32_t *>(tile + jb * 512 + (g * 4 + t) * 16);
                w[t] = lane[hi_row];
                w[4 + t] = lane[2 + hi_row];
            }
        }
        uint16_t *p = reinterpret_cast<uint16_t *>(rm);
        p[0] = reinterpret_cast<const uint16_t *>(dplane)[r * 4 + jb];
#pragma unroll
        for (int i = 0; i < NW; ++i) {
            p[1 + 2 * i] = (uint16_t) (w[i] & 0xffffu);
            p[2 + 2 * i] = (uint16_t) (w[i] >> 16);
        }
    }
}

// value of element e (0..31) of block (row, b) in a T16 tensor, as an integer (before the scale)
template <int WTYPE>
__device__ __forceinline__ int tiled_quant(const TiledDims &dims, const uint8_t *w, int64_t row, int64_t b, int e) {
    const int64_t rt = row >> 4;
    const int r = (int) (row & 15), g = r & 7, hi_row = r >> 3;
    const uint8_t *tile = w + (rt * dims.n_bg + (b >> 2)) * dims.tile_bytes;
    const int jb = (int) (b & 3);
    if (WTYPE == B200_TYPE_Q4_0) {
        const int ee = e & 15;  // byte index inside the 16 nibble bytes
        const int t = ee >> 2;
        const uint32_t word = reinterpret_cast<const uint32_t *>(tile + (g * 4 + t) * 32)[hi_row * 4 + jb];
        const uint32_t byte = (word >> (8 * (ee & 3))) & 0xffu;
        const int nib = (e < 16) ? (int) (byte & 0xf) : (int) (byte >> 4);
        return (nib ^ 8) - 8;  // 4-bit two's complement -> int
    } else {
        const int wi = e >> 2;  // word 0..7
        const int t = wi & 3;
        const uint32_t word = reinterpret_cast<const uint32_t *>(tile + jb * 512 + (g * 4 + t) * 16)[(wi >> 2) * 2 + hi_row];
        return (int) (int8_t) ((word >> (8 * (e & 3))) & 0xffu);
    }
}
template <int WTYPE>
__device__ __forceinline__ float tiled_scale(const TiledDims &dims, const uint8_t *w, int64_t row, int64_t b) {
    const __half *dplane = reinterpret_cast<const __half *>(w + dims.qs_bytes) + ((row >> 4) * dims.n_bg + (b >> 2)) * 64;
    return __half2float(dplane[(row & 15) * 4 + (b & 3)]);
}

// GET_ROWS on tiled weights (cactus/ggml-cpu/ops.cpp:4236-4300): dst[i] = dequantised row ids[i]
template <int WTYPE>
__global__ void __launch_bounds__(256) get_rows_q_kernel(TiledDims dims, const uint8_t *__restrict__ w,
                                                        const int32_t *__restrict__ ids, float *__restrict__ dst,
                                                        int64_t dst_nb_row, int64_t n_ids) {
    const int64_t gid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t i = gid / dims.K;
    const int64_t k = gid - i * dims.K;
    if (i >= n_ids) return;
    const int64_t row = ids[i];
    float *o = (float *) ((char *) dst + i * dst_nb_row);
    if (row < 0 || row >= dims.M) {
        o[k] = 0.0f;
        return;
    }
    const int64_t b = k >> 5;
    o[k] = (float) tiled_quant<WTYPE>(dims, w, row, b, (int) (k & 31)) * tiled_scale<WTYPE>(dims, w, row, b);
}

// exact integer dot of weight block (m, b) with activation block (n, b): out[(n*M + m)*nb + b].
// Uses the same word-level dp4a arithmetic as the mul_mat kernels (Q4_0 nibbles in the high half of each
// byte, i.e. 16x the value, undone by an exact shift).
template <int WTYPE>
__global__ void __launch_bounds__(256) block_dots_kernel(TiledDims dims, ActDims act, const uint8_t *__restrict__ w,
                                                        const uint8_t *__restrict__ aq, int32_t *__restrict__ out) {
    const int64_t gid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = act.N * dims.M * dims.nb;
    if (gid >= total) return;
    const int64_t b = gid % dims.nb;
    const int64_t m = (gid / dims.nb) % dims.M;
    const int64_t n = gid / (dims.nb * dims.M);
    const uint2 *atile = reinterpret_cast<const uint2 *>(aq + ((n >> 3) * act.nbp + b) * 256) + (n & 7) * 4;
    const int64_t rt = m >> 4;
    const int r = (int) (m & 15), g = r & 7, hi_row = r >> 3;
    const int jb = (int) (b & 3);
    const uint8_t *tile = w + (rt * dims.n_bg + (b >> 2)) * dims.tile_bytes;
    int sum = 0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const uint2 a = atile[t];
        if (WTYPE == B200_TYPE_Q4_0) {
            const uint32_t word = reinterpret_cast<const uint32_t *>(tile + (g * 4 + t) * 32)[hi_row * 4 + jb];
            sum = __dp4a((int) ((word << 4) & 0xF0F0F0F0u), (int) a.x, sum);
            sum = __dp4a((int) (word & 0xF0F0F0F0u), (int) a.y, sum);
        } else {
            const uint32_t *lane = reinterpret_cast<const uint32_t *>(tile + jb * 512 + (g * 4 + t) * 16);
            sum = __dp4a((int) lane[hi_row], (int) a.x, sum);
            sum = __dp4a((int) lane[2 + hi_row], (int) a.y, sum);
        }
    }
    out[gid] = (WTYPE == B200_TYPE_Q4_0) ? (sum >> 4) : sum;
}

static int check_wtype(int wtype) {
    if (wtype != B200_TYPE_Q4_0 && wtype != B200_TYPE_Q8_0) return set_error(B200_E_INVALID, "weight type %d is not Q4_0/Q8_0", wtype);
    return B200_OK;
}

int launch_quantize_b8(const float *x, int64_t x_nb_row, int64_t K, int64_t N, void *scratch, int variant, int layout, cudaStream_t st) {
    const ActDims a = act_dims(K, N);
    const int64_t threads = a.n_nt * 8 * a.nbp * 8;
    const int64_t grid = (threads + 255) / 256;
    const int early = N <= pdl_early_rows() ? 1 : 0;
    if (layout == 3) launch_pdl(quantize_q8_0_kernel<3>, dim3((unsigned) grid), dim3(256), 0, st, x, x_nb_row, K, N, a.n_nt * 8, a.nb, a.nbp, (uint8_t *) scratch, a.d_offset, variant, early);
    else launch_pdl(quantize_q8_0_kernel<1>, dim3((unsigned) grid), dim3(256), 0, st, x, x_nb_row, K, N, a.n_nt * 8, a.nb, a.nbp, (uint8_t *) scratch, a.d_offset, variant, early);
    return check_launch("quantize_q8_0 (activations)");
}

// What the quantised activations of an N-column product hold: 1 = the B8 tiles in fragment order, which the dp4a and
// mma.sync kernels read; 3 = those plus the e4m3 planes of the tcgen05 kernel (ACT_F8_MIN_N columns and more; the
// scratch of such a product always has room for them).  The tcgen05 kernel is taken with B200_MMQ_TC=1: it passes every
// parity case, but at the decode width of 64 columns it does not beat the mma.sync kernel yet (see mmq_tc.cu).
// B200_MMQ_TC: 0 mma.sync kernel, 1 the per-block tcgen05 kernel (mmq_tc.cu), 2 / 3 the folded-scale tcgen05 kernel
// (mmq_tcf.cu) with 3 / 2 product terms.
int mmq_tc_mode() {
    static const int mode = [] {
        const char *e = getenv("B200_MMQ_TC");
        int mode = e ? atoi(e) : 0;
        if (mode < 0 || mode > 3) mode = 0;
        return mode;
    }();
    return mode;
}
bool mmq_tc_enabled() { return mmq_tc_mode() == 1; }
int act_layout(int64_t N) { return (N >= ACT_F8_MIN_N && mmq_tc_enabled()) ? 3 : 1; }

}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_weight_bytes(int wtype, int64_t K, int64_t M) {
    if (check_wtype(wtype) || K <= 0 || M <= 0 || K % 32) return 0;
    return tiled_dims(wtype, K, M).total_bytes;
}

static int weight_convert(bool to_tiled, int wtype, int64_t K, int64_t M, const void *src, void *dst, int64_t rows_begin,
                          int64_t rows_count, cudaStream_t st) {
    if (int e = check_wtype(wtype)) return e;
    B200_REQUIRE(K > 0 && K % 32 == 0 && M > 0, "weight tensor needs K %% 32 == 0 (K=%lld M=%lld)", (long long) K, (long long) M);
    B200_REQUIRE(rows_begin >= 0 && rows_count > 0 && rows_begin + rows_count <= M, "row range out of bounds");
    B200_REQUIRE(rows_begin % 16 == 0, "rows_begin must be a multiple of 16");
    B200_REQUIRE(rows_count % 16 == 0 || rows_begin + rows_count == M, "rows_count must be a multiple of 16 unless the range ends at M");
    B200_REQUIRE(src && dst && is_aligned(src, 2) && is_aligned(dst, 2), "null or misaligned pointer");
    B200_REQUIRE(is_aligned(to_tiled ? dst : src, 16), "tiled tensor must be 16-byte aligned");
    const TiledDims d = tiled_dims(wtype, K, M);
    const int64_t rows_padded = (rows_count + 15) / 16 * 16;
    const int64_t threads = rows_padded * d.nbp;
    const unsigned grid = (unsigned) ((threads + 255) / 256);
    if (wtype == B200_TYPE_Q4_0) {
        if (to_tiled) weight_convert_kernel<B200_TYPE_Q4_0, true><<<grid, 256, 0, st>>>(d, (const uint8_t *) src, (uint8_t *) dst, rows_begin, rows_padded);
        else weight_convert_kernel<B200_TYPE_Q4_0, false><<<grid, 256, 0, st>>>(d, (const uint8_t *) src, (uint8_t *) dst, rows_begin, rows_padded);
    } else {
        if (to_tiled) weight_convert_kernel<B200_TYPE_Q8_0, true><<<grid, 256, 0, st>>>(d, (const uint8_t *) src, (uint8_t *) dst, rows_begin, rows_padded);
        else weight_convert_kernel<B200_TYPE_Q8_0, false><<<grid, 256, 0, st>>>(d, (const uint8_t *) src, (uint8_t *) dst, rows_begin, rows_padded);
    }
    return check_launch("weight_convert");
}

int b200_weight_upload(int wtype, int64_t K, int64_t M, const void *src_rowmajor, void *dst_tiled, int64_t rows_begin,
                       int64_t rows_count, b200_stream_t stream) {
    return weight_convert(true, wtype, K, M, src_rowmajor, dst_tiled, rows_begin, rows_count, (cudaStream_t) stream);
}

int b200_weight_download(int wtype, int64_t K, int64_t M, const void *src_tiled, void *dst_rowmajor, int64_t rows_begin,
                         int64_t rows_count, b200_stream_t stream) {
    return weight_convert(false, wtype, K, M, src_tiled, dst_rowmajor, rows_begin, rows_count, (cudaStream_t) stream);
}

int b200_quantize_q8_0(const float *x, int64_t x_row_stride_bytes, int64_t K, int64_t N, void *dst_blocks, int variant,
                       b200_stream_t stream) {
    B200_REQUIRE(x && dst_blocks, "null pointer");
    B200_REQUIRE(K > 0 && K % 32 == 0 && N >= 0, "K must be a positive multiple of 32");
    B200_REQUIRE(variant == B200_Q8_AVX2 || variant == B200_Q8_SCALAR, "unknown quantiser variant %d", variant);
    B200_REQUIRE(is_aligned(x, 4) && x_row_stride_bytes % 4 == 0 && is_aligned(dst_blocks, 2), "misaligned pointer or stride");
    if (N == 0) return B200_OK;
    const int64_t nb = K / 32;
    const int64_t threads = N * nb * 8;
    quantize_q8_0_kernel<0><<<(unsigned) ((threads + 255) / 256), 256, 0, (cudaStream_t) stream>>>(
        x, x_row_stride_bytes, K, N, N, nb, nb, (uint8_t *) dst_blocks, 0, variant, 0);
    return check_launch("quantize_q8_0");
}

size_t b200_act_bytes(int64_t K, int64_t N) {
    if (K <= 0 || K % 32 || N <= 0) return 0;
    return act_dims(K, N).total_bytes;
}

int b200_quantize_activations(const float *x, int64_t x_row_stride_bytes, int64_t K, int64_t N, void *scratch,
                              size_t scratch_bytes, int variant, b200_stream_t stream) {
    B200_REQUIRE(x && scratch, "null pointer");
    B200_REQUIRE(K > 0 && K % 32 == 0 && N > 0, "K must be a positive multiple of 32 and N positive");
    B200_REQUIRE(variant == B200_Q8_AVX2 || variant == B200_Q8_SCALAR, "unknown quantiser variant %d", variant);
    B200_REQUIRE(is_aligned(x, 4) && x_row_stride_bytes % 4 == 0, "misaligned activations");
    B200_REQUIRE(is_aligned(scratch, 256), "scratch must be 256-byte aligned");
    if (scratch_bytes < act_dims(K, N).total_bytes) return set_error(B200_E_SCRATCH, "scratch too small: %zu < %zu", scratch_bytes, act_dims(K, N).total_bytes);
    return launch_quantize_b8(x, x_row_stride_bytes, K, N, scratch, variant, act_layout(N), (cudaStream_t) stream);
}

int b200_block_dots(int wtype, const void *w, int64_t K, int64_t M, const float *x, int64_t x_row_stride_bytes, int64_t N,
                    int32_t *out, void *scratch, size_t scratch_bytes, int variant, b200_stream_t stream) {
    if (int e = check_wtype(wtype)) return e;
    B200_REQUIRE(w && out && is_aligned(w, 16), "null or misaligned pointer");
    B200_REQUIRE(x && scratch && is_aligned(scratch, 256) && scratch_bytes >= act_dims(K, N).total_bytes, "bad activation scratch");
    if (int e = launch_quantize_b8(x, x_row_stride_bytes, K, N, scratch, variant, 1, (cudaStream_t) stream)) return e;
    const TiledDims d = tiled_dims(wtype, K, M);
    const ActDims a = act_dims(K, N);
    const int64_t total = N * M * d.nb;
    const unsigned grid = (unsigned) ((total + 255) / 256);
    if (wtype == B200_TYPE_Q4_0) block_dots_kernel<B200_TYPE_Q4_0><<<grid, 256, 0, (cudaStream_t) stream>>>(d, a, (const uint8_t *) w, (const uint8_t *) scratch, out);
    else block_dots_kernel<B200_TYPE_Q8_0><<<grid, 256, 0, (cudaStream_t) stream>>>(d, a, (const uint8_t *) w, (const uint8_t *) scratch, out);
    return check_launch("block_dots");
}

int b200_get_rows_q(int wtype, const void *table_tiled, int64_t d, int64_t n_table_rows, const int32_t *ids, float *dst,
                    int64_t dst_nb_row, int64_t n_ids, b200_stream_t stream) {
    if (int e = check_wtype(wtype)) return e;
    B200_REQUIRE(table_tiled && ids && dst && d > 0 && d % 32 == 0 && n_table_rows > 0, "bad get_rows arguments");
    if (n_ids == 0) return B200_OK;
    const TiledDims dims = tiled_dims(wtype, d, n_table_rows);
    const int64_t total = n_ids * d;
    const unsigned grid = (unsigned) ((total + 255) / 256);
    if (wtype == B200_TYPE_Q4_0) get_rows_q_kernel<B200_TYPE_Q4_0><<<grid, 256, 0, (cudaStream_t) stream>>>(dims, (const uint8_t *) table_tiled, ids, dst, dst_nb_row, n_ids);
    else get_rows_q_kernel<B200_TYPE_Q8_0><<<grid, 256, 0, (cudaStream_t) stream>>>(dims, (const uint8_t *) table_tiled, ids, dst, dst_nb_row, n_ids);
    return check_launch("get_rows_q");
}

}  // extern "C"
