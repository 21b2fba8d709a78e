// Device-side pieces of the unified KV cache bookkeeping that the reference does on the host:
// the attention mask (llama_kv_cache_unified::set_input_kq_mask, cactus/llama-kv-cache.cpp:696-761),
// the K/V store into cache rows (cpy_k / cpy_v, :617-656) addressed by slot index, and greedy argmax over
// logits (the sampler step after llama_get_logits, cactus/cactus_completion.cpp:210).
#include <math_constants.h>

#include "common.cuh"

namespace b200 {

// mask[j][i] = 0 if cell i holds token j's sequence and cell_pos[i] <= tok_pos[j], else -inf; rows
// n_tokens..n_rows (the padding to a multiple of 64) are -inf.  One sequence id per cell.
__global__ void __launch_bounds__(256) kq_mask_kernel(const int32_t *__restrict__ cell_pos, const int32_t *__restrict__ cell_seq,
                                                     int64_t n_kv, const int32_t *__restrict__ tok_pos,
                                                     const int32_t *__restrict__ tok_seq, int64_t n_tokens, int64_t n_rows,
                                                     __half *__restrict__ mask, int64_t mask_nb_row) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t j = blockIdx.y;
    if (i >= n_kv || j >= n_rows) return;
    unsigned short v = 0xFC00u;  // -inf
    if (j < n_tokens) {
        const int32_t cs = cell_seq[i];
        if (cs >= 0 && cs == tok_seq[j] && cell_pos[i] <= tok_pos[j]) v = 0;
    }
    reinterpret_cast<unsigned short *>(reinterpret_cast<char *>(mask) + j * mask_nb_row)[i] = v;
}

__global__ void __launch_bounds__(256) scatter_i32_kernel(int32_t *__restrict__ dst, const int32_t *__restrict__ idx,
                                                         const int32_t *__restrict__ src, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[idx[i]] = src[i];
}

__global__ void __launch_bounds__(256) set_rows_f16_kernel(const float *__restrict__ x, int64_t x_nb_row,
                                                          const int32_t *__restrict__ slots, __half *__restrict__ dst,
                                                          int64_t dst_nb_row, int64_t d, int64_t rows) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d * rows) return;
    const int64_t r = i / d, c = i - r * d;
    const float v = reinterpret_cast<const float *>(reinterpret_cast<const char *>(x) + r * x_nb_row)[c];
    reinterpret_cast<__half *>(reinterpret_cast<char *>(dst) + (int64_t) slots[r] * dst_nb_row)[c] = __float2half_rn(v);
}

// first index of the maximum of each row (ties: lowest index, as a linear scan finds it).  One CTA of 1024 threads per row,
// 16-byte loads where the row allows them: a vocabulary-sized row is a chain of dependent compares per thread, so the time
// is the number of elements a thread walks
constexpr int ARGMAX_THREADS = 1024;
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_rows_kernel(const float *__restrict__ x, int64_t x_nb_row, int64_t d,
                                                                    int32_t *__restrict__ out) {
    const int64_t r = blockIdx.x;
    const float *row = reinterpret_cast<const float *>(reinterpret_cast<const char *>(x) + r * x_nb_row);
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    int64_t done = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        const int64_t n4 = d >> 2;
        const float4 *row4 = reinterpret_cast<const float4 *>(row);
#pragma unroll 4
        for (int64_t i = threadIdx.x; i < n4; i += ARGMAX_THREADS) {
            const float4 v = __ldg(row4 + i);
            const int b = (int) (i << 2);
            if (v.x > best) { best = v.x; bi = b; }
            if (v.y > best) { best = v.y; bi = b + 1; }
            if (v.z > best) { best = v.z; bi = b + 2; }
            if (v.w > best) { best = v.w; bi = b + 3; }
        }
        done = n4 << 2;
    }
    for (int64_t i = done + threadIdx.x; i < d; i += ARGMAX_THREADS) {
        const float v = row[i];
        if (v > best) { best = v; bi = (int) i; }
    }
    // a thread's candidate is the first maximum among its own elements; between threads the lower index wins a tie
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    __shared__ float sv[ARGMAX_THREADS / 32];
    __shared__ int si[ARGMAX_THREADS / 32];
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x];
        bi = si[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;   // nothing above -inf: a linear scan stays at index 0
    }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_kq_mask_build(const int32_t *cell_pos, const int32_t *cell_seq, int64_t n_kv, const int32_t *tok_pos,
                       const int32_t *tok_seq, int64_t n_tokens, void *mask, int64_t mask_nb_row, b200_stream_t stream) {
    B200_REQUIRE(cell_pos && cell_seq && tok_pos && tok_seq && mask && n_kv > 0 && n_tokens > 0, "bad kq_mask arguments");
    B200_REQUIRE(mask_nb_row % 2 == 0 && mask_nb_row >= n_kv * 2, "bad mask row stride");
    const int64_t n_rows = (n_tokens + 63) / 64 * 64;
    dim3 grid((unsigned) ((n_kv + 255) / 256), (unsigned) n_rows);
    kq_mask_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(cell_pos, cell_seq, n_kv, tok_pos, tok_seq, n_tokens, n_rows,
                                                            (__half *) mask, mask_nb_row);
    return check_launch("kq_mask");
}

int b200_scatter_i32(int32_t *dst, const int32_t *idx, const int32_t *src, int64_t n, b200_stream_t stream) {
    B200_REQUIRE(dst && idx && src && n >= 0, "bad scatter arguments");
    if (n == 0) return B200_OK;
    scatter_i32_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(dst, idx, src, n);
    return check_launch("scatter_i32");
}

int b200_set_rows_f16(const float *x, int64_t x_nb_row, const int32_t *slots, void *dst, int64_t dst_nb_row, int64_t d,
                      int64_t rows, b200_stream_t stream) {
    B200_REQUIRE(x && slots && dst && d > 0 && rows >= 0 && x_nb_row % 4 == 0 && dst_nb_row % 2 == 0, "bad set_rows arguments");
    if (rows == 0) return B200_OK;
    set_rows_f16_kernel<<<(unsigned) ((d * rows + 255) / 256), 256, 0, (cudaStream_t) stream>>>(x, x_nb_row, slots, (__half *) dst,
                                                                                              dst_nb_row, d, rows);
    return check_launch("set_rows_f16");
}

int b200_argmax_rows(const float *x, int64_t x_nb_row, int64_t d, int64_t rows, int32_t *out, b200_stream_t stream) {
    B200_REQUIRE(x && out && d > 0 && rows >= 0 && x_nb_row % 4 == 0, "bad argmax arguments");
    if (rows == 0) return B200_OK;
    argmax_rows_kernel<<<(unsigned) rows, ARGMAX_THREADS, 0, (cudaStream_t) stream>>>(x, x_nb_row, d, out);
    return check_launch("argmax_rows");
}

}  // extern "C"
