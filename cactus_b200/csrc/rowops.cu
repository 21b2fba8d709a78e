// The small row ops that keep a llama layer on the device: RMS_NORM(+MUL), ADD, MUL, SILU(+MUL), ROPE,
// CPY and GET_ROWS on f32 tables (cactus/ggml-cpu/ops.cpp, cactus/ggml-cpu/binary-ops.cpp).
#include "common.cuh"

namespace b200 {

// RMS_NORM: ops.cpp:3268-3316.  The reference sums squares in double and scales by 1/sqrtf(mean + eps);
// a following MUL by the weight row (binary-ops.cpp:152-154) is fused when w != NULL.
__global__ void __launch_bounds__(1024) rms_norm_kernel(const float *x, int64_t x_nb_row, const float *__restrict__ w,
                                                       float *dst, int64_t dst_nb_row, int64_t d, float eps) {
    const int64_t r = blockIdx.x;
    const float *xr = reinterpret_cast<const float *>(reinterpret_cast<const char *>(x) + r * x_nb_row);
    float *o = reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + r * dst_nb_row);
    double sum = 0.0;
    const int64_t groups = (d + 3) / 4;
    for (int64_t gi = threadIdx.x; gi < groups; gi += blockDim.x) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (gi * 4 + i < d) {
                const float v = xr[gi * 4 + i];
                sum += (double) (v * v);
            }
        }
    }
    const double tot = rms_block_sum(sum);
    const float mean = (float) (tot / (double) d);
    const float sc = 1.0f / sqrtf(mean + eps);
    for (int64_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = xr[i] * sc;
        o[i] = w ? v * w[i] : v;
    }
}

template <int OP>  // 0 add, 1 mul
__global__ void __launch_bounds__(256) binary_kernel(const float *a, const float *b, float *dst,
                                                    int64_t d, int64_t total, int64_t b_rows) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float bv = b_rows == 1 ? b[i % d] : b[i];
    dst[i] = OP == 0 ? a[i] + bv : a[i] * bv;
}

// SILU: ops.cpp:2902-2981 (x / (1 + exp(-x))), optionally times b
__global__ void __launch_bounds__(256) silu_kernel(const float *a, const float *b, float *dst, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = a[i];
    const float s = x / (1.0f + expf(-x));
    dst[i] = b ? s * b[i] : s;
}

// ROPE mode 0: ops.cpp:5080-5118, 5178-5362.  theta_i = pos * theta_scale^i is built by repeated
// multiplication in the reference; one thread of the token's CTA walks that recurrence (cheap), the cos/sin
// of the D/2 angles are then taken in parallel and applied to every head of the token, so the angles are
// bit-identical to the reference's.
__global__ void __launch_bounds__(128) rope_norm_kernel(const float *x, int64_t x_nb_head, int64_t x_nb_tok,
                                                       float *dst, int64_t dst_nb_head, int64_t dst_nb_tok, int64_t D,
                                                       int64_t H, int64_t T, int n_dims, const int32_t *__restrict__ pos,
                                                       const float *__restrict__ ff, float theta_scale, float freq_scale,
                                                       float attn_factor) {
    extern __shared__ float cs[];   // [n_dims/2] cos, [n_dims/2] sin
    const int64_t t = blockIdx.x;
    const int half_dims = n_dims / 2;
    if (threadIdx.x == 0) {
        float theta = (float) pos[t];
        for (int k = 0; k < half_dims; ++k) {
            cs[k] = theta;
            theta *= theta_scale;
        }
    }
    __syncthreads();
    for (int k = threadIdx.x; k < half_dims; k += blockDim.x) {
        const float f = ff ? ff[k] : 1.0f;
        const float th = freq_scale * (cs[k] / f);
        cs[half_dims + k] = sinf(th) * attn_factor;
    }
    __syncthreads();
    for (int k = threadIdx.x; k < half_dims; k += blockDim.x) {
        const float f = ff ? ff[k] : 1.0f;
        const float th = freq_scale * (cs[k] / f);
        cs[k] = cosf(th) * attn_factor;
    }
    __syncthreads();
    const int64_t pairs = D / 2;
    for (int64_t i = threadIdx.x; i < H * pairs; i += blockDim.x) {
        const int64_t h = i / pairs, k = i - h * pairs;
        const float *s = reinterpret_cast<const float *>(reinterpret_cast<const char *>(x) + t * x_nb_tok + h * x_nb_head) + 2 * k;
        float *o = reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + t * dst_nb_tok + h * dst_nb_head) + 2 * k;
        const float2 v = *reinterpret_cast<const float2 *>(s);
        if (k < half_dims) {
            const float c = cs[k], sn = cs[half_dims + k];
            *reinterpret_cast<float2 *>(o) = make_float2(v.x * c - v.y * sn, v.x * sn + v.y * c);
        } else {
            *reinterpret_cast<float2 *>(o) = v;
        }
    }
}

// The same rotation on f16 rows, as the K-shift graph applies it in place to the cached keys
// (lm_ggml_compute_forward_rope_f16, ops.cpp:5364-5520): values widened to f32, rotated, rounded back to f16.
// pos[t] is the shift of cell t; a zero shift returns the row unchanged bit for bit (cos 1, sin 0).
__global__ void __launch_bounds__(128) rope_norm_f16_kernel(const __half *x, int64_t x_nb_head, int64_t x_nb_tok,
                                                           __half *dst, int64_t dst_nb_head, int64_t dst_nb_tok, int64_t D,
                                                           int64_t H, int n_dims, const int32_t *__restrict__ pos,
                                                           const float *__restrict__ ff, float theta_scale, float freq_scale, float attn_factor) {
    extern __shared__ float cs[];   // [n_dims/2] cos, [n_dims/2] sin, [n_dims/2] theta
    const int64_t t = blockIdx.x;
    const int half_dims = n_dims / 2;
    float *th_s = cs + 2 * half_dims;
    if (threadIdx.x == 0) {
        float theta = (float) pos[t];
        for (int k = 0; k < half_dims; ++k) {
            th_s[k] = theta;
            theta *= theta_scale;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * half_dims; i += blockDim.x) {
        const int a = i < half_dims ? i : i - half_dims;
        const float f = ff ? ff[a] : 1.0f;
        const float th = freq_scale * (th_s[a] / f);
        cs[i] = (i < half_dims ? cosf(th) : sinf(th)) * attn_factor;
    }
    __syncthreads();
    const int64_t pairs = D / 2;
    for (int64_t i = threadIdx.x; i < H * pairs; i += blockDim.x) {
        const int64_t h = i / pairs, k = i - h * pairs;
        const __half2 v = *reinterpret_cast<const __half2 *>(reinterpret_cast<const char *>(x) + t * x_nb_tok + h * x_nb_head + 4 * k);
        __half2 *o = reinterpret_cast<__half2 *>(reinterpret_cast<char *>(dst) + t * dst_nb_tok + h * dst_nb_head + 4 * k);
        if (k < half_dims) {
            const float c = cs[k], sn = cs[half_dims + k];
            const float x0 = __low2float(v), x1 = __high2float(v);
            *o = __halves2half2(__float2half_rn(x0 * c - x1 * sn), __float2half_rn(x0 * sn + x1 * c));
        } else {
            *o = v;
        }
    }
}

// rows of 2-byte elements copied as they are (f16 -> f16: the moves of a cache defragmentation)
__global__ void __launch_bounds__(256) cpy_b16_kernel(const uint16_t *__restrict__ x, int64_t x_nb_row, uint16_t *__restrict__ dst,
                                                     int64_t dst_nb_row, int64_t d, int64_t rows) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d * rows) return;
    const int64_t r = i / d, c = i - r * d;
    reinterpret_cast<uint16_t *>(reinterpret_cast<char *>(dst) + r * dst_nb_row)[c] =
        reinterpret_cast<const uint16_t *>(reinterpret_cast<const char *>(x) + r * x_nb_row)[c];
}

template <typename TO>
__global__ void __launch_bounds__(256) cpy_kernel(const float *__restrict__ x, int64_t x_nb_row, TO *__restrict__ dst, int64_t dst_nb_row,
                                                 int64_t d, int64_t rows) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d * rows) return;
    const int64_t r = i / d, c = i - r * d;
    const float v = reinterpret_cast<const float *>(reinterpret_cast<const char *>(x) + r * x_nb_row)[c];
    TO *o = reinterpret_cast<TO *>(reinterpret_cast<char *>(dst) + r * dst_nb_row);
    if constexpr (sizeof(TO) == 2) o[c] = __float2half_rn(v);
    else o[c] = v;
}

__global__ void __launch_bounds__(256) get_rows_f32_kernel(const float *__restrict__ table, int64_t table_nb_row,
                                                          const int32_t *__restrict__ ids, float *__restrict__ dst, int64_t dst_nb_row,
                                                          int64_t d, int64_t n_ids) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d * n_ids) return;
    const int64_t r = i / d, c = i - r * d;
    const float *src = reinterpret_cast<const float *>(reinterpret_cast<const char *>(table) + (int64_t) ids[r] * table_nb_row);
    reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + r * dst_nb_row)[c] = src[c];
}

static inline unsigned blocks_for(int64_t n, int per = 256) { return (unsigned) ((n + per - 1) / per); }

}  // namespace b200

using namespace b200;

extern "C" {

int b200_rms_norm(const float *x, int64_t x_nb_row, const float *w, float *dst, int64_t dst_nb_row, int64_t d, int64_t rows,
                  float eps, b200_stream_t stream) {
    B200_REQUIRE(x && dst && d > 0 && rows >= 0 && x_nb_row % 4 == 0 && dst_nb_row % 4 == 0, "bad rms_norm arguments");
    if (rows == 0) return B200_OK;
    rms_norm_kernel<<<(unsigned) rows, rms_threads(d), 0, (cudaStream_t) stream>>>(x, x_nb_row, w, dst, dst_nb_row, d, eps);
    return check_launch("rms_norm");
}

int b200_add(const float *a, const float *b, float *dst, int64_t d, int64_t rows, int64_t b_rows, b200_stream_t stream) {
    B200_REQUIRE(a && b && dst && d > 0 && rows >= 0 && (b_rows == 1 || b_rows == rows), "bad add arguments");
    if (rows == 0) return B200_OK;
    binary_kernel<0><<<blocks_for(d * rows), 256, 0, (cudaStream_t) stream>>>(a, b, dst, d, d * rows, b_rows);
    return check_launch("add");
}

int b200_mul(const float *a, const float *b, float *dst, int64_t d, int64_t rows, int64_t b_rows, b200_stream_t stream) {
    B200_REQUIRE(a && b && dst && d > 0 && rows >= 0 && (b_rows == 1 || b_rows == rows), "bad mul arguments");
    if (rows == 0) return B200_OK;
    binary_kernel<1><<<blocks_for(d * rows), 256, 0, (cudaStream_t) stream>>>(a, b, dst, d, d * rows, b_rows);
    return check_launch("mul");
}

int b200_silu(const float *a, const float *b, float *dst, int64_t n, b200_stream_t stream) {
    B200_REQUIRE(a && dst && n >= 0, "bad silu arguments");
    if (n == 0) return B200_OK;
    silu_kernel<<<blocks_for(n), 256, 0, (cudaStream_t) stream>>>(a, b, dst, n);
    return check_launch("silu");
}

int b200_rope_norm(const float *x, int64_t x_nb_head, int64_t x_nb_tok, float *dst, int64_t dst_nb_head, int64_t dst_nb_tok,
                   int64_t D, int64_t H, int64_t T, int n_dims, const int32_t *pos, const float *freq_factors, float freq_base,
                   float freq_scale, float attn_factor, b200_stream_t stream) {
    B200_REQUIRE(x && dst && pos && D > 0 && D % 2 == 0 && H > 0 && T >= 0 && n_dims > 0 && n_dims <= D && n_dims % 2 == 0, "bad rope arguments");
    B200_REQUIRE(n_dims <= 8192 && is_aligned(x, 8) && is_aligned(dst, 8) && x_nb_head % 8 == 0 && x_nb_tok % 8 == 0 && dst_nb_head % 8 == 0 && dst_nb_tok % 8 == 0,
                 "rope rows must be 8-byte aligned");
    if (T == 0) return B200_OK;
    const float theta_scale = powf(freq_base, -2.0f / (float) n_dims);
    rope_norm_kernel<<<(unsigned) T, 128, (size_t) n_dims * sizeof(float), (cudaStream_t) stream>>>(x, x_nb_head, x_nb_tok, dst, dst_nb_head, dst_nb_tok, D, H, T,
                                                                              n_dims, pos, freq_factors, theta_scale, freq_scale, attn_factor);
    return check_launch("rope_norm");
}

int b200_rope_norm_f16(const void *x, int64_t x_nb_head, int64_t x_nb_tok, void *dst, int64_t dst_nb_head, int64_t dst_nb_tok, int64_t D,
                       int64_t H, int64_t T, int n_dims, const int32_t *pos, const float *freq_factors, float freq_base, float freq_scale,
                       float attn_factor, b200_stream_t stream) {
    B200_REQUIRE(x && dst && pos && D > 0 && D % 2 == 0 && H > 0 && T >= 0 && n_dims > 0 && n_dims <= D && n_dims % 2 == 0, "bad rope arguments");
    B200_REQUIRE(n_dims <= 8192 && is_aligned(x, 4) && is_aligned(dst, 4) && x_nb_head % 4 == 0 && x_nb_tok % 4 == 0 && dst_nb_head % 4 == 0 && dst_nb_tok % 4 == 0,
                 "f16 rope rows must be 4-byte aligned");
    if (T == 0) return B200_OK;
    const float theta_scale = powf(freq_base, -2.0f / (float) n_dims);
    rope_norm_f16_kernel<<<(unsigned) T, 128, (size_t) (n_dims + n_dims / 2) * sizeof(float), (cudaStream_t) stream>>>(
        (const __half *) x, x_nb_head, x_nb_tok, (__half *) dst, dst_nb_head, dst_nb_tok, D, H, n_dims, pos, freq_factors, theta_scale, freq_scale, attn_factor);
    return check_launch("rope_norm_f16");
}

int b200_cpy_f16_f16(const void *x, int64_t x_nb_row, void *dst, int64_t dst_nb_row, int64_t d, int64_t rows, b200_stream_t stream) {
    B200_REQUIRE(x && dst && d > 0 && rows >= 0 && x_nb_row % 2 == 0 && dst_nb_row % 2 == 0, "bad cpy arguments");
    if (rows == 0) return B200_OK;
    cpy_b16_kernel<<<blocks_for(d * rows), 256, 0, (cudaStream_t) stream>>>((const uint16_t *) x, x_nb_row, (uint16_t *) dst, dst_nb_row, d, rows);
    return check_launch("cpy_f16_f16");
}

int b200_cpy_f32_f16(const float *x, int64_t x_nb_row, void *dst, int64_t dst_nb_row, int64_t d, int64_t rows, b200_stream_t stream) {
    B200_REQUIRE(x && dst && d > 0 && rows >= 0 && x_nb_row % 4 == 0 && dst_nb_row % 2 == 0, "bad cpy arguments");
    if (rows == 0) return B200_OK;
    cpy_kernel<__half><<<blocks_for(d * rows), 256, 0, (cudaStream_t) stream>>>(x, x_nb_row, (__half *) dst, dst_nb_row, d, rows);
    return check_launch("cpy_f32_f16");
}

int b200_cpy_f32_f32(const float *x, int64_t x_nb_row, float *dst, int64_t dst_nb_row, int64_t d, int64_t rows, b200_stream_t stream) {
    B200_REQUIRE(x && dst && d > 0 && rows >= 0 && x_nb_row % 4 == 0 && dst_nb_row % 4 == 0, "bad cpy arguments");
    if (rows == 0) return B200_OK;
    cpy_kernel<float><<<blocks_for(d * rows), 256, 0, (cudaStream_t) stream>>>(x, x_nb_row, dst, dst_nb_row, d, rows);
    return check_launch("cpy_f32_f32");
}

int b200_get_rows_f32(const float *table, int64_t table_nb_row, const int32_t *ids, float *dst, int64_t dst_nb_row, int64_t d,
                      int64_t n_ids, b200_stream_t stream) {
    B200_REQUIRE(table && ids && dst && d > 0 && n_ids >= 0, "bad get_rows arguments");
    if (n_ids == 0) return B200_OK;
    get_rows_f32_kernel<<<blocks_for(d * n_ids), 256, 0, (cudaStream_t) stream>>>(table, table_nb_row, ids, dst, dst_nb_row, d, n_ids);
    return check_launch("get_rows_f32");
}

}  // extern "C"
