/*
 * CPU oracle: plain-C restatement of the reference's ggml-cpu arithmetic for the quantised mul_mat and
 * flash-attention path.  TEST INFRASTRUCTURE ONLY (see oracle.h).  Compiled with -ffp-contract=off so
 * that a fused multiply-add happens only where fmaf() is written, which is where the reference's AVX2
 * branch issues one.
 *
 * Every function cites the reference lines it follows (paths relative to the reference project root).
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------------------------------------
 * IEEE binary16 <-> binary32, round-to-nearest-even.  The reference uses the F16C instructions
 * (cactus/ggml-impl.h:346-362), which implement exactly this.
 * ------------------------------------------------------------------------------------------- */
uint16_t orc_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        return (uint16_t) (sign | 0x7c00u | ((absx > 0x7f800000u) ? (0x0200u | ((absx >> 13) & 0x03ffu)) : 0u));
    }
    if (absx >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t) (sign | 0x7c00u);
    }
    if (absx < 0x33000001u) { /* <= 2^-25 rounds to zero (2^-25 itself ties to even = 0) */
        return (uint16_t) sign;
    }
    int32_t e = (int32_t) (absx >> 23) - 127;
    uint32_t m = (absx & 0x007fffffu) | 0x00800000u; /* 24-bit significand */
    uint32_t shift, half_bits;
    if (e < -14) { /* subnormal half: value = m * 2^(e-23); unit = 2^-24 */
        shift = (uint32_t) (13 + (-14 - e));
        half_bits = 0;
    } else {
        shift = 13;
        half_bits = (uint32_t) (e + 15) << 10;
        m &= 0x007fffffu;
    }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    return (uint16_t) (sign | (half_bits + q)); /* carry into the exponent is the correct rounding */
}

float orc_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = ((uint32_t) h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x03ffu;
    uint32_t x;
    if (e == 0) {
        if (m == 0) {
            x = sign;
        } else { /* subnormal: normalise */
            int sh = 0;
            while (!(m & 0x0400u)) { m <<= 1; sh++; }
            m &= 0x03ffu;
            x = sign | ((uint32_t) (127 - 15 - sh + 1) << 23) | (m << 13);
        }
    } else if (e == 31) {
        x = sign | 0x7f800000u | (m << 13);
    } else {
        x = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* ---------------------------------------------------------------------------------------------
 * Weight quantisation, cactus/ggml-quants.c:25-60 (quantize_row_q4_0_ref).
 * ------------------------------------------------------------------------------------------- */
void orc_quantize_row_q4_0(const float *x, orc_block_q4_0 *y, int64_t k) {
    const int64_t nb = k / ORC_QK;
    for (int64_t i = 0; i < nb; i++) {
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < ORC_QK; j++) {
            const float v = x[i * ORC_QK + j];
            if (amax < fabsf(v)) { amax = fabsf(v); max = v; }
        }
        const float d = max / -8;
        const float id = d ? 1.0f / d : 0.0f;
        y[i].d = orc_fp32_to_fp16(d);
        for (int j = 0; j < ORC_QK / 2; ++j) {
            /* x*id + 8.5f: gcc fuses this into one FMA in the pinned reference build (-mfma, default
             * -ffp-contract=fast); 1 nibble in ~10^7 differs from the unfused form */
            int8_t a = (int8_t) fmaf(x[i * ORC_QK + j], id, 8.5f);
            int8_t b = (int8_t) fmaf(x[i * ORC_QK + ORC_QK / 2 + j], id, 8.5f);
            const uint8_t xi0 = (uint8_t) (a < 15 ? a : 15);
            const uint8_t xi1 = (uint8_t) (b < 15 ? b : 15);
            y[i].qs[j] = (uint8_t) (xi0 | (xi1 << 4));
        }
    }
}

/* cactus/ggml-quants.c:249-267 and :343-357 */
void orc_dequantize_row_q4_0(const orc_block_q4_0 *x, float *y, int64_t k) {
    for (int64_t i = 0; i < k / ORC_QK; i++) {
        const float d = orc_fp16_to_fp32(x[i].d);
        for (int j = 0; j < 16; ++j) {
            y[i * 32 + j] = (float) ((x[i].qs[j] & 0x0F) - 8) * d;
            y[i * 32 + j + 16] = (float) ((x[i].qs[j] >> 4) - 8) * d;
        }
    }
}
void orc_dequantize_row_q8_0(const orc_block_q8_0 *x, float *y, int64_t k) {
    for (int64_t i = 0; i < k / ORC_QK; i++) {
        const float d = orc_fp16_to_fp32(x[i].d);
        for (int j = 0; j < 32; ++j) y[i * 32 + j] = (float) x[i].qs[j] * d;
    }
}

/* round half to even without depending on the floating-point environment */
static float round_half_even(float v) {
    const float r = roundf(v); /* half away from zero */
    if (fabsf(v - truncf(v)) == 0.5f) {
        /* tie: pick the even neighbour */
        const float t = truncf(v);
        return (fmodf(t, 2.0f) == 0.0f) ? t : r;
    }
    return r;
}

/* ---------------------------------------------------------------------------------------------
 * Activation quantisation.
 *   ORC_Q8_AVX2   : cactus/ggml-cpu/ggml-cpu-quants.c:802-885.  d = max/127 ; id = 127/max ;
 *                   q = round_to_nearest_even(x * id)   (separate multiply, no FMA)
 *   ORC_Q8_SCALAR : cactus/ggml-quants.c:188-211.  d = amax/127 ; id = 1/d ; q = roundf(x * id)
 * ------------------------------------------------------------------------------------------- */
void orc_quantize_row_q8_0(const float *x, orc_block_q8_0 *y, int64_t k, int variant) {
    const int64_t nb = k / ORC_QK;
    for (int64_t i = 0; i < nb; i++) {
        float amax = 0.0f;
        for (int j = 0; j < ORC_QK; j++) {
            const float v = fabsf(x[i * ORC_QK + j]);
            if (v > amax) amax = v;
        }
        const float d = amax / 127.0f;
        y[i].d = orc_fp32_to_fp16(d);
        if (variant == ORC_Q8_AVX2) {
            const float id = (amax != 0.0f) ? 127.0f / amax : 0.0f;
            for (int j = 0; j < ORC_QK; ++j) {
                const float v = x[i * ORC_QK + j] * id;
                y[i].qs[j] = (int8_t) round_half_even(v);
            }
        } else {
            const float id = d ? 1.0f / d : 0.0f;
            for (int j = 0; j < ORC_QK; ++j) {
                y[i].qs[j] = (int8_t) roundf(x[i * ORC_QK + j] * id);
            }
        }
    }
}

/* ---------------------------------------------------------------------------------------------
 * Block dots.  Integer part: cactus/ggml-cpu/ggml-cpu-quants.c:2585-2601 (q4_0) and :3998-4008 (q8_0).
 * ------------------------------------------------------------------------------------------- */
static void block_lanes(int wtype, const void *w_row, int64_t ib, const orc_block_q8_0 *a, int32_t lane[8], float *scale) {
    /* lane l = sum over elements 4l..4l+3, the grouping mul_sum_i8_pairs_float produces (:108-128) */
    const int8_t *ay = a[ib].qs;
    int8_t wv[32];
    float dw;
    if (wtype == ORC_TYPE_Q4_0) {
        const orc_block_q4_0 *w = (const orc_block_q4_0 *) w_row + ib;
        for (int j = 0; j < 16; ++j) {
            wv[j] = (int8_t) ((w->qs[j] & 0x0F) - 8);
            wv[j + 16] = (int8_t) ((w->qs[j] >> 4) - 8);
        }
        dw = orc_fp16_to_fp32(w->d);
    } else {
        const orc_block_q8_0 *w = (const orc_block_q8_0 *) w_row + ib;
        memcpy(wv, w->qs, 32);
        dw = orc_fp16_to_fp32(w->d);
    }
    for (int l = 0; l < 8; ++l) {
        int32_t s = 0;
        for (int j = 0; j < 4; ++j) s += (int32_t) wv[4 * l + j] * (int32_t) ay[4 * l + j];
        lane[l] = s;
    }
    *scale = dw * orc_fp16_to_fp32(a[ib].d); /* dx*dy formed first (:2274, :3870) */
}

void orc_block_dots(int wtype, int64_t k, const void *w_row, const orc_block_q8_0 *a, int32_t *out) {
    for (int64_t ib = 0; ib < k / ORC_QK; ++ib) {
        int32_t lane[8];
        float sc;
        block_lanes(wtype, w_row, ib, a, lane, &sc);
        int32_t s = 0;
        for (int l = 0; l < 8; ++l) s += lane[l];
        out[ib] = s;
    }
}

/* AVX2 accumulation order: acc[l] = fma(scale, (float)lane[l], acc[l]) per block (:2267-2290,
 * :3863-3880), then hsum_float_8 (:43-49): (l + l+4) -> (0+2, 1+3) -> 0+1. */
float orc_vec_dot(int wtype, int64_t k, const void *w_row, const orc_block_q8_0 *a) {
    float acc[8] = { 0 };
    for (int64_t ib = 0; ib < k / ORC_QK; ++ib) {
        int32_t lane[8];
        float sc;
        block_lanes(wtype, w_row, ib, a, lane, &sc);
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(sc, (float) lane[l], acc[l]);
    }
    float r[4];
    for (int l = 0; l < 4; ++l) r[l] = acc[l + 4] + acc[l];
    const float s0 = r[2] + r[0];
    const float s1 = r[3] + r[1];
    return s0 + s1;
}

/* cactus/ggml-cpu/ggml-cpu.c:1257-1449: quantise every src1 row to Q8_0, then one vec_dot per (m, n). */
void orc_mul_mat(int wtype, int64_t M, int64_t K, int64_t N, const void *w, const float *x, int64_t x_stride,
                 float *dst, orc_block_q8_0 *q8, int variant) {
    const int64_t nb = K / ORC_QK;
    const size_t wrow = (size_t) nb * (wtype == ORC_TYPE_Q4_0 ? sizeof(orc_block_q4_0) : sizeof(orc_block_q8_0));
    orc_block_q8_0 *tmp = q8 ? q8 : (orc_block_q8_0 *) malloc((size_t) N * nb * sizeof(orc_block_q8_0));
    for (int64_t n = 0; n < N; ++n) orc_quantize_row_q8_0(x + n * x_stride, tmp + n * nb, K, variant);
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m)
            dst[n * M + m] = orc_vec_dot(wtype, K, (const char *) w + (size_t) m * wrow, tmp + n * nb);
    if (!q8) free(tmp);
}

/* ---------------------------------------------------------------------------------------------
 * Flash attention, cactus/ggml-cpu/ops.cpp:6948-7165 with the AVX2 f16 vector helpers:
 *   lm_ggml_vec_dot_f16 (vec.cpp:122-160): 4 accumulators x 8 lanes, f32 FMA, tree reduce
 *   (simd-mappings.h:251-269); lm_ggml_vec_mad_f16 / vec_scale_f16 (vec.h:180-209, 295-320): f32
 *   arithmetic on fp16-loaded values, stored back rounded to fp16.
 * ------------------------------------------------------------------------------------------- */
static float dot_f16(int64_t n, const uint16_t *x, const uint16_t *y) {
    float sum[4][8];
    memset(sum, 0, sizeof(sum));
    const int64_t np = n & ~(int64_t) 31;
    for (int64_t i = 0; i < np; i += 32)
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 8; ++l)
                sum[j][l] = fmaf(orc_fp16_to_fp32(x[i + j * 8 + l]), orc_fp16_to_fp32(y[i + j * 8 + l]), sum[j][l]);
    float t[8];
    for (int l = 0; l < 8; ++l) {
        const float a = sum[0][l] + sum[2][l];
        const float b = sum[1][l] + sum[3][l];
        t[l] = a + b;
    }
    float t0[4];
    for (int l = 0; l < 4; ++l) t0[l] = t[l] + t[l + 4];
    const float h0 = t0[0] + t0[1], h1 = t0[2] + t0[3];
    double sumf = (double) (h0 + h1);
    for (int64_t i = np; i < n; ++i) sumf += (double) (orc_fp16_to_fp32(x[i]) * orc_fp16_to_fp32(y[i]));
    return (float) sumf;
}

void orc_flash_attn_ext(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv,
                        const float *q, const uint16_t *kc, const uint16_t *vc, const uint16_t *mask,
                        float scale, float max_bias, float logit_softcap, float *dst, int acc_mode) {
    if (logit_softcap != 0.0f) scale /= logit_softcap;
    const uint32_t n_head_log2 = 1u << (uint32_t) floor(log2((double) H));
    const float m0 = powf(2.0f, -(max_bias) / n_head_log2);
    const float m1 = powf(2.0f, -(max_bias / 2.0f) / n_head_log2);
    const int64_t gqa = H / Hkv;
    const int64_t np = D & ~(int64_t) 31;
    uint16_t *Q16 = (uint16_t *) malloc((size_t) D * 2);
    uint16_t *A16 = (uint16_t *) malloc((size_t) D * 2);
    double *A64 = (double *) malloc((size_t) D * 8);
    for (int64_t h = 0; h < H; ++h) {
        const float slope = (max_bias > 0.0f)
            ? ((uint32_t) h < n_head_log2 ? powf(m0, (float) (h + 1)) : powf(m1, (float) (2 * (h - n_head_log2) + 1)))
            : 1.0f;
        const int64_t hk = h / gqa;
        for (int64_t t = 0; t < Nq; ++t) {
            const float *pq = q + (t * H + h) * D;
            for (int64_t d = 0; d < D; ++d) Q16[d] = orc_fp32_to_fp16(pq[d]);
            memset(A16, 0, (size_t) D * 2);
            for (int64_t d = 0; d < D; ++d) A64[d] = 0.0;
            float S = 0.0f, M = -INFINITY;
            double S64 = 0.0;
            const uint16_t *mp = mask ? mask + t * n_kv : NULL;
            for (int64_t ic = 0; ic < n_kv; ++ic) {
                const float mv = mp ? slope * orc_fp16_to_fp32(mp[ic]) : 0.0f;
                if (mv == -INFINITY) continue;
                const uint16_t *kr = kc + (ic * Hkv + hk) * D;
                const uint16_t *vr = vc + (ic * Hkv + hk) * D;
                float s = dot_f16(D, kr, Q16);
                /* gcc contracts the scale and the mask add of the reference build into one FMA when no
                 * soft cap sits between them (-mfma, default -ffp-contract=fast) */
                if (logit_softcap != 0.0f) {
                    s = s * scale;
                    s = logit_softcap * tanhf(s);
                    s += mv;
                } else {
                    s = fmaf(s, scale, mv);
                }
                const float Mold = M;
                float ms = 1.0f, vs = 1.0f;
                if (s > M) {
                    M = s;
                    ms = expf(Mold - M);
                    if (acc_mode == 0) {
                        for (int64_t d = 0; d < D; ++d) A16[d] = orc_fp32_to_fp16(orc_fp16_to_fp32(A16[d]) * ms);
                    } else {
                        for (int64_t d = 0; d < D; ++d) A64[d] *= (double) ms;
                    }
                } else {
                    vs = expf(s - M);
                }
                if (acc_mode == 0) {
                    for (int64_t d = 0; d < np; ++d) /* SIMD body: fused multiply-add */
                        A16[d] = orc_fp32_to_fp16(fmaf(orc_fp16_to_fp32(vr[d]), vs, orc_fp16_to_fp32(A16[d])));
                    for (int64_t d = np; d < D; ++d) /* scalar tail: separate multiply and add */
                        A16[d] = orc_fp32_to_fp16(orc_fp16_to_fp32(A16[d]) + orc_fp16_to_fp32(vr[d]) * vs);
                } else {
                    for (int64_t d = 0; d < D; ++d) A64[d] += (double) orc_fp16_to_fp32(vr[d]) * (double) vs;
                }
                S = fmaf(S, ms, vs);
                S64 = S64 * (double) ms + (double) vs;
            }
            float *o = dst + (t * H + h) * D;
            if (acc_mode == 0) {
                const float S_inv = 1.0f / S;
                for (int64_t d = 0; d < D; ++d) o[d] = orc_fp16_to_fp32(A16[d]) * S_inv;
            } else {
                for (int64_t d = 0; d < D; ++d) o[d] = (float) (A64[d] / S64);
            }
        }
    }
    free(Q16); free(A16); free(A64);
}

/* cactus/llama-kv-cache.cpp:696-761 restricted to one seq_id per cell and no sliding window. */
void orc_build_kq_mask(int64_t n_kv, int64_t n_tokens, const int32_t *cell_pos, const int32_t *cell_seq,
                       const int32_t *tok_pos, const int32_t *tok_seq, uint16_t *mask) {
    const int64_t n_pad = (n_tokens + 63) / 64 * 64;
    const uint16_t ninf = 0xfc00u;
    for (int64_t j = 0; j < n_pad; ++j)
        for (int64_t i = 0; i < n_kv; ++i) {
            uint16_t v = ninf;
            if (j < n_tokens && cell_seq[i] == tok_seq[j] && cell_seq[i] >= 0 && cell_pos[i] <= tok_pos[j]) v = 0;
            mask[j * n_kv + i] = v;
        }
}

/* ---------------------------------------------------------------------------------------------
 * Row ops of the llama layer.
 * ------------------------------------------------------------------------------------------- */
/* cactus/ggml-cpu/ops.cpp:3268-3316 (sum of squares in double, scale = 1/sqrtf(mean+eps)), then MUL by
 * the weight row (binary-ops.cpp:152-154) */
void orc_rms_norm_mul(int64_t d, int64_t T, const float *x, const float *w, float eps, float *dst) {
    for (int64_t t = 0; t < T; ++t) {
        double sum = 0.0;
        for (int64_t i = 0; i < d; ++i) sum += (double) (x[t * d + i] * x[t * d + i]);
        const float mean = (float) (sum / (double) d);
        const float sc = 1.0f / sqrtf(mean + eps);
        for (int64_t i = 0; i < d; ++i) dst[t * d + i] = (x[t * d + i] * sc) * w[i];
    }
}
/* cactus/ggml-cpu/ops.cpp:2902-2981; silu(x) = x / (1 + exp(-x)); the reference's SIMD branch uses a
 * polynomial expf, so this is tolerance-checked only */
void orc_silu_mul(int64_t n, const float *a, const float *b, float *dst) {
    for (int64_t i = 0; i < n; ++i) dst[i] = (a[i] / (1.0f + expf(-a[i]))) * b[i];
}
void orc_add(int64_t n, const float *a, const float *b, float *dst) {
    for (int64_t i = 0; i < n; ++i) dst[i] = a[i] + b[i];
}
/* cactus/ggml-cpu/ops.cpp:5080-5118, 5178-5362, mode 0 ("norm": adjacent pairs), freq_scale 1,
 * ext_factor 0, attn_factor 1: theta_i = pos * s^i with s = powf(base, -2/D) built by repeated
 * multiplication */
void orc_rope_norm(int64_t D, int64_t H, int64_t T, const float *x, const int32_t *pos, float freq_base, float *dst) {
    const float theta_scale = powf(freq_base, -2.0f / (float) D);
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < H; ++h) {
            float theta = (float) pos[t];
            const float *s = x + (t * H + h) * D;
            float *o = dst + (t * H + h) * D;
            for (int64_t i = 0; i < D; i += 2) {
                const float c = cosf(theta), sn = sinf(theta);
                const float x0 = s[i], x1 = s[i + 1];
                /* contraction as gcc emits it for the reference build (-mfma) */
                o[i] = fmaf(x0, c, -(x1 * sn));
                o[i + 1] = fmaf(x0, sn, x1 * c);
                theta *= theta_scale;
            }
        }
    }
}
/* the same on an f16 tensor, as the K-shift graph applies it in place to the cached keys
 * (cactus/llama-kv-cache.cpp:822-860 -> lm_ggml_compute_forward_rope_f16, cactus/ggml-cpu/ops.cpp:5364-5520):
 * values widened to f32, rotated, rounded back to f16; pos holds the per-cell position shift (may be negative) */
void orc_rope_norm_f16(int64_t D, int64_t H, int64_t T, const uint16_t *x, const int32_t *pos, float freq_base, uint16_t *dst) {
    const float theta_scale = powf(freq_base, -2.0f / (float) D);
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < H; ++h) {
            float theta = (float) pos[t];
            const uint16_t *s = x + (t * H + h) * D;
            uint16_t *o = dst + (t * H + h) * D;
            for (int64_t i = 0; i < D; i += 2) {
                const float c = cosf(theta), sn = sinf(theta);
                const float x0 = orc_fp16_to_fp32(s[i]), x1 = orc_fp16_to_fp32(s[i + 1]);
                o[i] = orc_fp32_to_fp16(fmaf(x0, c, -(x1 * sn)));
                o[i + 1] = orc_fp32_to_fp16(fmaf(x0, sn, x1 * c));
                theta *= theta_scale;
            }
        }
    }
}
void orc_cpy_f32_f16(int64_t n, const float *x, uint16_t *dst) {
    for (int64_t i = 0; i < n; ++i) dst[i] = orc_fp32_to_fp16(x[i]);
}
/* cactus/ggml-cpu/ops.cpp:4236-4300: dequantise the selected rows */
void orc_get_rows(int wtype, int64_t d, int64_t n_rows, const void *table, const int32_t *ids, float *dst) {
    const int64_t nb = d / ORC_QK;
    for (int64_t r = 0; r < n_rows; ++r) {
        if (wtype == ORC_TYPE_Q4_0)
            orc_dequantize_row_q4_0((const orc_block_q4_0 *) table + (int64_t) ids[r] * nb, dst + r * d, d);
        else
            orc_dequantize_row_q8_0((const orc_block_q8_0 *) table + (int64_t) ids[r] * nb, dst + r * d, d);
    }
}
