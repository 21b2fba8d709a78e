// Fused forms of the small ops between the mul_mats of a llama layer (llm_build_llama, cactus/llama-model.cpp:4517-4671).
// Each one computes exactly what the chain of separate ops computes -- same float operations in the same order -- and
// hands the result to the next mul_mat already quantised, so the intermediate f32 tensors need not be written:
//   residual ADD (ops.cpp:1283-1300) + RMS_NORM (ops.cpp:3268-3316) + MUL by the norm weight + quantize_row_q8_0
//   SILU (ops.cpp:2902-2981) * up + quantize_row_q8_0
//   ROPE of q and k (ops.cpp:5080-5362) + the f32 -> f16 stores of k and v into the cache rows (cpy_k / cpy_v,
//   cactus/llama-kv-cache.cpp:617-656)
#include "common.cuh"

namespace b200 {

int act_layout(int64_t N);

// One CTA per (padded) token row, one pass: a thread keeps its groups of 4 elements in registers from the load to the
// quantised store.  The sum of squares is accumulated in the order rms_norm_kernel uses (rms_block_sum), so the
// scale -- and with it every quantised value -- is bit-identical to the unfused chain.
template <int LAYOUT>
// (x, res and h carry no __restrict__: a graph allocator may hand the same memory to the residual and to the normalised output)
__global__ void __launch_bounds__(1024) add_rms_norm_quantize_kernel(float *x, int64_t x_nb_row, const float *res,
                                                                    int64_t res_nb_row, const float *__restrict__ w, float *h,
                                                                    int64_t h_nb_row, int64_t d, int64_t N, float eps, int64_t nb, int64_t nbp,
                                                                    uint8_t *__restrict__ out, size_t d_offset, int variant, int early) {
    pdl_prologue(early != 0);
    constexpr int GMAX = 4;   // groups of 4 elements per thread: d <= 16 * blockDim.x
    const int64_t n = blockIdx.x;
    const bool row_real = n < N;
    const int64_t groups = d / 4, groups_padded = nbp * 8;
    float v[GMAX][4];
    double sum = 0.0;
    float *xr = row_real ? reinterpret_cast<float *>(reinterpret_cast<char *>(x) + n * x_nb_row) : nullptr;
    const float *rr = (row_real && res) ? reinterpret_cast<const float *>(reinterpret_cast<const char *>(res) + n * res_nb_row) : nullptr;
#pragma unroll
    for (int k = 0; k < GMAX; ++k) {
        const int64_t gi = threadIdx.x + (int64_t) k * blockDim.x;
        v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.0f;
        if (row_real && gi < groups) {
            const float4 a = *reinterpret_cast<const float4 *>(xr + gi * 4);
            v[k][0] = a.x; v[k][1] = a.y; v[k][2] = a.z; v[k][3] = a.w;
            if (rr) {
                const float4 b = *reinterpret_cast<const float4 *>(rr + gi * 4);
                v[k][0] = v[k][0] + b.x; v[k][1] = v[k][1] + b.y; v[k][2] = v[k][2] + b.z; v[k][3] = v[k][3] + b.w;
                *reinterpret_cast<float4 *>(xr + gi * 4) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) sum += (double) (v[k][i] * v[k][i]);
        }
    }
    const double tot = rms_block_sum(sum);
    const float mean = (float) (tot / (double) d);
    const float sc = 1.0f / sqrtf(mean + eps);
    float *hr = (h && row_real) ? reinterpret_cast<float *>(reinterpret_cast<char *>(h) + n * h_nb_row) : nullptr;
#pragma unroll
    for (int k = 0; k < GMAX; ++k) {
        const int64_t gi = threadIdx.x + (int64_t) k * blockDim.x;
        if (gi >= groups_padded) continue;   // whole 8-lane block groups leave together
        const bool real = row_real && gi < groups;
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        if (real) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float t = v[k][i] * sc;
                o[i] = w ? t * w[gi * 4 + i] : t;
            }
            if (hr) *reinterpret_cast<float4 *>(hr + gi * 4) = make_float4(o[0], o[1], o[2], o[3]);
        }
        q8_quantize_store<LAYOUT>(o, out, d_offset, nb, nbp, n, gi >> 3, (int) (gi & 7), real, variant);
    }
}

// silu(gate) * up, quantised; the same index space as quantize_q8_0_kernel
template <int LAYOUT>
__global__ void __launch_bounds__(256) silu_mul_quantize_kernel(const float *gate, const float *up, int64_t nb_row,
                                                               float *dst, int64_t dst_nb_row,
                                                               int64_t N, int64_t n_rows_padded, int64_t nb, int64_t nbp,
                                                               uint8_t *__restrict__ out, size_t d_offset, int variant, int early) {
    pdl_prologue(early != 0);
    const int64_t gid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int j = (int) (gid & 7);
    const int64_t blk = gid >> 3;
    const int64_t n = blk / nbp;
    const int64_t b = blk - n * nbp;
    if (n >= n_rows_padded) return;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const bool real = (n < N) && (b < nb);
    if (real) {
        const float4 a = *reinterpret_cast<const float4 *>(reinterpret_cast<const char *>(gate) + n * nb_row + (b * 32 + j * 4) * 4);
        const float4 u = *reinterpret_cast<const float4 *>(reinterpret_cast<const char *>(up) + n * nb_row + (b * 32 + j * 4) * 4);
        const float ga[4] = {a.x, a.y, a.z, a.w}, ua[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float s = ga[i] / (1.0f + expf(-ga[i]));
            v[i] = s * ua[i];
        }
        if (dst) *reinterpret_cast<float4 *>(reinterpret_cast<char *>(dst) + n * dst_nb_row + (b * 32 + j * 4) * 4) = make_float4(v[0], v[1], v[2], v[3]);
    }
    q8_quantize_store<LAYOUT>(v, out, d_offset, nb, nbp, n, b, j, real, variant);
}

// One CTA per token: the angles as rope_norm_kernel builds them, q rotated into qo (which may be q itself, with the same
// strides), k rotated and stored as f16 into its cache row, v stored as f16 into its cache row.
__global__ void __launch_bounds__(512) rope_store_kernel(const float *q, float *qo, int64_t q_nb_head, int64_t q_nb_tok, const float *__restrict__ k,
                                                        int64_t k_nb_head, int64_t k_nb_tok, const float *__restrict__ v, int64_t v_nb_tok,
                                                        int64_t D, int64_t H, int64_t Hkv, int n_dims, const int32_t *__restrict__ pos,
                                                        const float *__restrict__ ff, float theta_scale, float freq_scale, float attn_factor,
                                                        const int32_t *__restrict__ slots, __half *__restrict__ kc, int64_t kc_nb_row,
                                                        __half *__restrict__ vc, int64_t vc_nb_row, int early) {
    pdl_prologue(early != 0);
    extern __shared__ float cs[];   // [n_dims/2] cos, [n_dims/2] sin, [n_dims/2] theta
    const int64_t t = blockIdx.x;
    const int half_dims = n_dims / 2;
    float *th_s = cs + 2 * half_dims;
    if (threadIdx.x == 0) {
        float theta = (float) pos[t];
        for (int i = 0; i < half_dims; ++i) {
            th_s[i] = theta;
            theta *= theta_scale;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * half_dims; i += blockDim.x) {   // first half of the threads: cosines, second half: sines
        const int a = i < half_dims ? i : i - half_dims;
        const float f = ff ? ff[a] : 1.0f;
        const float th = freq_scale * (th_s[a] / f);
        cs[i] = (i < half_dims ? cosf(th) : sinf(th)) * attn_factor;
    }
    __syncthreads();
    const int64_t pairs = D / 2;
    const int64_t slot = slots ? (int64_t) slots[t] : t;   // no slot list: token t goes to row t of the cache pointers given
    __half *krow = reinterpret_cast<__half *>(reinterpret_cast<char *>(kc) + slot * kc_nb_row);
    __half *vrow = reinterpret_cast<__half *>(reinterpret_cast<char *>(vc) + slot * vc_nb_row);
    for (int64_t i = threadIdx.x; i < (H + 2 * Hkv) * pairs; i += blockDim.x) {
        const int64_t hh = i / pairs, p = i - hh * pairs;
        if (hh < H) {
            const int64_t off = t * q_nb_tok + hh * q_nb_head;
            const float2 x = *(reinterpret_cast<const float2 *>(reinterpret_cast<const char *>(q) + off) + p);
            float2 *d = reinterpret_cast<float2 *>(reinterpret_cast<char *>(qo) + off) + p;
            if (p < half_dims) {
                const float c = cs[p], sn = cs[half_dims + p];
                *d = make_float2(x.x * c - x.y * sn, x.x * sn + x.y * c);
            } else if (qo != q) {
                *d = x;
            }
        } else if (hh < H + Hkv) {
            const int64_t hk = hh - H;
            const float2 x = *reinterpret_cast<const float2 *>(reinterpret_cast<const float *>(reinterpret_cast<const char *>(k) + t * k_nb_tok + hk * k_nb_head) + 2 * p);
            float2 r = x;
            if (p < half_dims) {
                const float c = cs[p], sn = cs[half_dims + p];
                r = make_float2(x.x * c - x.y * sn, x.x * sn + x.y * c);
            }
            *reinterpret_cast<__half2 *>(krow + hk * D + 2 * p) = __halves2half2(__float2half_rn(r.x), __float2half_rn(r.y));
        } else if (v) {
            const int64_t hv = hh - H - Hkv;
            const float2 x = *reinterpret_cast<const float2 *>(reinterpret_cast<const float *>(reinterpret_cast<const char *>(v) + t * v_nb_tok) + hv * D + 2 * p);
            *reinterpret_cast<__half2 *>(vrow + hv * D + 2 * p) = __halves2half2(__float2half_rn(x.x), __float2half_rn(x.y));
        }
    }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_add_rms_norm_quantize(float *x, int64_t x_nb_row, const float *residual, int64_t residual_nb_row, const float *w, float *h,
                               int64_t h_nb_row, int64_t d, int64_t rows, float eps, void *scratch, size_t scratch_bytes, int variant,
                               b200_stream_t stream) {
    B200_REQUIRE(x && scratch && d > 0 && d % 32 == 0 && rows > 0, "bad arguments");
    B200_REQUIRE(x_nb_row % 4 == 0 && residual_nb_row % 4 == 0 && h_nb_row % 4 == 0, "row strides must be multiples of 4 bytes");
    B200_REQUIRE(variant == B200_Q8_AVX2 || variant == B200_Q8_SCALAR, "unknown quantiser variant %d", variant);
    B200_REQUIRE(is_aligned(scratch, 256), "scratch must be 256-byte aligned");
    const ActDims a = act_dims(d, rows);
    if (scratch_bytes < a.total_bytes) return set_error(B200_E_SCRATCH, "scratch too small: %zu < %zu", scratch_bytes, a.total_bytes);
    B200_REQUIRE(d <= 16384, "rows of more than 16384 elements are not supported");
    B200_REQUIRE(x_nb_row % 16 == 0 && residual_nb_row % 16 == 0 && h_nb_row % 16 == 0 && is_aligned(x, 16) && (!residual || is_aligned(residual, 16)) &&
                     (!h || is_aligned(h, 16)) && (!w || is_aligned(w, 4)), "rows must be 16-byte aligned");
    const unsigned grid = (unsigned) (a.n_nt * 8);
    const unsigned threads = rms_threads(d);
    cudaStream_t st = (cudaStream_t) stream;
    const int early = rows <= pdl_early_rows() ? 1 : 0;
    if (act_layout(rows) == 3) {
        launch_pdl(add_rms_norm_quantize_kernel<3>, dim3(grid), dim3(threads), 0, st, x, x_nb_row, residual, residual_nb_row, w, h, h_nb_row, d, rows, eps, a.nb, a.nbp,
                                                                  (uint8_t *) scratch, a.d_offset, variant, early);
    } else {
        launch_pdl(add_rms_norm_quantize_kernel<1>, dim3(grid), dim3(threads), 0, st, x, x_nb_row, residual, residual_nb_row, w, h, h_nb_row, d, rows, eps, a.nb, a.nbp,
                                                                  (uint8_t *) scratch, a.d_offset, variant, early);
    }
    return check_launch("add_rms_norm_quantize");
}

int b200_silu_mul_quantize(const float *gate, const float *up, int64_t nb_row, float *dst, int64_t dst_nb_row, int64_t K, int64_t N,
                           void *scratch, size_t scratch_bytes, int variant, b200_stream_t stream) {
    B200_REQUIRE(gate && up && scratch && K > 0 && K % 32 == 0 && N > 0, "bad arguments");
    B200_REQUIRE(nb_row % 16 == 0 && is_aligned(gate, 16) && is_aligned(up, 16) && (!dst || (is_aligned(dst, 16) && dst_nb_row % 16 == 0)),
                 "rows must be 16-byte aligned");
    B200_REQUIRE(variant == B200_Q8_AVX2 || variant == B200_Q8_SCALAR, "unknown quantiser variant %d", variant);
    B200_REQUIRE(is_aligned(scratch, 256), "scratch must be 256-byte aligned");
    const ActDims a = act_dims(K, N);
    if (scratch_bytes < a.total_bytes) return set_error(B200_E_SCRATCH, "scratch too small: %zu < %zu", scratch_bytes, a.total_bytes);
    const int64_t rows_padded = a.n_nt * 8;
    const int64_t threads = rows_padded * a.nbp * 8;
    const unsigned grid = (unsigned) ((threads + 255) / 256);
    cudaStream_t st = (cudaStream_t) stream;
    const int early = N <= pdl_early_rows() ? 1 : 0;
    if (act_layout(N) == 3) {
        launch_pdl(silu_mul_quantize_kernel<3>, dim3(grid), dim3(256), 0, st, gate, up, nb_row, dst, dst_nb_row, N, rows_padded, a.nb, a.nbp, (uint8_t *) scratch, a.d_offset, variant, early);
    } else {
        launch_pdl(silu_mul_quantize_kernel<1>, dim3(grid), dim3(256), 0, st, gate, up, nb_row, dst, dst_nb_row, N, rows_padded, a.nb, a.nbp, (uint8_t *) scratch, a.d_offset, variant, early);
    }
    return check_launch("silu_mul_quantize");
}

int b200_rope_store(float *q, int64_t q_nb_head, int64_t q_nb_tok, const float *k, int64_t k_nb_head, int64_t k_nb_tok, const float *v,
                    int64_t v_nb_tok, int64_t D, int64_t H, int64_t Hkv, int64_t T, int n_dims, const int32_t *pos, const float *freq_factors,
                    float freq_base, float freq_scale, float attn_factor, const int32_t *slots, void *k_cache, int64_t k_cache_nb_row,
                    void *v_cache, int64_t v_cache_nb_row, b200_stream_t stream) {
    return b200_rope_store_to(q, q, q_nb_head, q_nb_tok, k, k_nb_head, k_nb_tok, v, v_nb_tok, D, H, Hkv, T, n_dims, pos, freq_factors, freq_base, freq_scale,
                              attn_factor, slots, k_cache, k_cache_nb_row, v_cache, v_cache_nb_row, stream);
}

int b200_rope_store_to(const float *q, float *q_dst, int64_t q_nb_head, int64_t q_nb_tok, const float *k, int64_t k_nb_head, int64_t k_nb_tok, const float *v,
                       int64_t v_nb_tok, int64_t D, int64_t H, int64_t Hkv, int64_t T, int n_dims, const int32_t *pos, const float *freq_factors,
                       float freq_base, float freq_scale, float attn_factor, const int32_t *slots, void *k_cache, int64_t k_cache_nb_row,
                       void *v_cache, int64_t v_cache_nb_row, b200_stream_t stream) {
    B200_REQUIRE(k && pos && k_cache && (H == 0 || (q && q_dst)) && (!v || v_cache), "null pointer");
    B200_REQUIRE(is_aligned(q_dst, 8), "pairs must be 8-byte aligned");
    B200_REQUIRE(D > 0 && D % 2 == 0 && H >= 0 && Hkv > 0 && T >= 0 && n_dims > 0 && n_dims <= D && n_dims % 2 == 0, "bad rope arguments");
    B200_REQUIRE(q_nb_head % 8 == 0 && q_nb_tok % 8 == 0 && k_nb_head % 8 == 0 && k_nb_tok % 8 == 0 && v_nb_tok % 8 == 0 && is_aligned(q, 8) &&
                     is_aligned(k, 8) && is_aligned(v, 8) && k_cache_nb_row % 4 == 0 && v_cache_nb_row % 4 == 0 && is_aligned(k_cache, 4) && is_aligned(v_cache, 4),
                 "pairs must be 8-byte aligned (f32) / 4-byte aligned (f16)");
    if (T == 0) return B200_OK;
    const float theta_scale = powf(freq_base, -2.0f / (float) n_dims);
    launch_pdl(rope_store_kernel, dim3((unsigned) T), dim3(512), (size_t) (n_dims + n_dims / 2) * sizeof(float), (cudaStream_t) stream,
        q, q_dst, q_nb_head, q_nb_tok, k, k_nb_head, k_nb_tok, v, v_nb_tok, D, H, Hkv, n_dims, pos, freq_factors, theta_scale, freq_scale, attn_factor,
        slots, (__half *) k_cache, k_cache_nb_row, (__half *) v_cache, v_cache_nb_row, T <= pdl_early_rows() ? 1 : 0);
    return check_launch("rope_store");
}

}  // extern "C"
