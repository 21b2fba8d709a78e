// FLASH_ATTN_EXT over the f16 unified KV cache for ragged multi-sequence batches.
//
// Replaces lm_ggml_compute_forward_flash_attn_ext_f16 (cactus/ggml-cpu/ops.cpp:6948-7165).
//
// The mask tensor is honoured exactly as the reference does (a cell takes part iff its mask value is
// not -inf, the finite value is added to the scaled score), but it is scanned only once per graph:
// b200_mask_index_build turns each token's mask row into one bit per cell, and the attention kernel
// walks the set bits, so a token of a 64-sequence batch touches only its own sequence's K/V rows.
//
// Kernel: one CTA per (token, kv-head, head group, KV split).  Sub-warps of 8 lanes each own one cell at
// a time: a lane holds D/8 contiguous elements of the K and V rows (128-bit loads), the score is reduced
// over the 8 lanes with three shuffles, and every sub-warp keeps its own online-softmax state which is
// merged at the end (shuffles inside the warp, shared memory across warps).  With KV splits the
// partial (max, sum, accumulator) triples go to scratch and a combine kernel finishes.
#include <math_constants.h>

#include "common.cuh"

namespace b200 {

constexpr int FA_THREADS = 128;
constexpr int FA_SUPER_WORDS = 32;  // 2048 cells listed per round

// ---- mask scan: one warp per 64 cells of one token row ------------------------------------------
__global__ void __launch_bounds__(256) mask_index_kernel(const __half *__restrict__ mask, int64_t mask_nb_row, int64_t Nq,
                                                        int64_t n_kv, int64_t nw, unsigned long long *__restrict__ words) {
    const int lane = threadIdx.x & 31;
    const int64_t wid = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wid >= Nq * nw) return;
    const int64_t j = wid / nw, wi = wid - j * nw;
    const __half *row = reinterpret_cast<const __half *>(reinterpret_cast<const char *>(mask) + j * mask_nb_row);
    const int64_t c0 = wi * 64 + lane, c1 = c0 + 32;
    const unsigned short ninf = 0xFC00u;
    const bool v0 = c0 < n_kv && __half_as_ushort(row[c0]) != ninf;
    const bool v1 = c1 < n_kv && __half_as_ushort(row[c1]) != ninf;
    const unsigned lo = __ballot_sync(0xffffffffu, v0), hi = __ballot_sync(0xffffffffu, v1);
    if (lane == 0) words[wid] = (unsigned long long) lo | ((unsigned long long) hi << 32);
}

struct FattnParams {
    int64_t H, Hkv, Nq, n_kv, nw;
    const float *q; int64_t q_nb_tok, q_nb_head;
    const char *k; int64_t k_nb_cell, k_nb_head;
    const char *v; int64_t v_nb_cell, v_nb_head;
    const char *mask; int64_t mask_nb_row;
    const unsigned long long *words;  // NULL: every cell takes part
    float scale, max_bias, softcap, m0, m1;
    uint32_t n_head_log2;
    float *dst;
    float *partial;  // [Nq][H][nsplit][D + 2]
    int nsplit, hgroups;
    int64_t words_per_split;
};

template <int D, int G>
__global__ void __launch_bounds__(FA_THREADS) fattn_vec_kernel(FattnParams p) {
    constexpr int E = D / 8;  // elements per lane
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int e = lane & 7;          // lane inside the sub-warp
    const int sg = warp * 4 + (lane >> 3);  // sub-warp 0..15
    const unsigned sub_mask = 0xFFu << (lane & 24);  // the 8 lanes of this sub-warp
    const int64_t j = blockIdx.x;    // token
    const int hk = blockIdx.y / p.hgroups, hg = blockIdx.y % p.hgroups;
    const int split = blockIdx.z;
    const int gqa = (int) (p.H / p.Hkv);
    const int h0 = hk * gqa + hg * G;  // first query head of this CTA

    __shared__ int cell_list[FA_SUPER_WORDS * 64];
    __shared__ int list_count;
    __shared__ float merge_m[4][G], merge_l[4][G];
    __shared__ float merge_acc[4][G][D];

    // Q rounded to fp16 as the reference does before its dot (ops.cpp:7072), kept as float
    float qf[G][E];
    float slope[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        const float *qp = reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.q) + j * p.q_nb_tok + (int64_t) (h0 + h) * p.q_nb_head) + e * E;
#pragma unroll
        for (int i = 0; i < E; ++i) qf[h][i] = __half2float(__float2half_rn(qp[i]));
        const uint32_t hh = (uint32_t) (h0 + h);
        slope[h] = (p.max_bias > 0.0f) ? (hh < p.n_head_log2 ? powf(p.m0, (float) (hh + 1)) : powf(p.m1, (float) (2 * (hh - p.n_head_log2) + 1))) : 1.0f;
    }
    float m[G], l[G], acc[G][E];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        m[h] = -CUDART_INF_F;
        l[h] = 0.0f;
#pragma unroll
        for (int i = 0; i < E; ++i) acc[h][i] = 0.0f;
    }

    const int64_t w_begin = (int64_t) split * p.words_per_split;
    const int64_t w_end = min(p.nw, w_begin + p.words_per_split);
    const unsigned long long *wrow = p.words ? p.words + j * p.nw : nullptr;
    const __half *mrow = p.mask ? reinterpret_cast<const __half *>(p.mask + j * p.mask_nb_row) : nullptr;

    for (int64_t w0 = w_begin; w0 < w_end; w0 += FA_SUPER_WORDS) {
        // list the participating cells of this round (warp 0 scans 32 words)
        if (warp == 0) {
            const int64_t wi = w0 + lane;
            unsigned long long bits = 0;
            if (wi < w_end) {
                if (wrow) {
                    bits = wrow[wi];
                } else {
                    const int64_t left = p.n_kv - wi * 64;
                    bits = left >= 64 ? ~0ull : ((1ull << left) - 1ull);
                }
            }
            const int cnt = __popcll(bits);
            int pre = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, pre, o);
                if (lane >= o) pre += t;
            }
            int pos = pre - cnt;
            while (bits) {
                const int b = __ffsll((long long) bits) - 1;
                bits &= bits - 1;
                cell_list[pos++] = (int) (wi * 64 + b);
            }
            if (lane == 31) list_count = pre;
        }
        __syncthreads();
        const int count = list_count;
        // sub-warps run the same number of rounds; the shuffles below name only the 8 lanes of a sub-warp,
        // and a sub-warp without a cell in the last round skips it as a whole
        for (int idx = sg; idx < count; idx += 16) {
            const int64_t cell = cell_list[idx];
            const char *kp = p.k + cell * p.k_nb_cell + (int64_t) hk * p.k_nb_head + e * E * 2;
            const char *vp = p.v + cell * p.v_nb_cell + (int64_t) hk * p.v_nb_head + e * E * 2;
            float kf[E];
#pragma unroll
            for (int c = 0; c < E / 8; ++c) {
                const uint4 u = __ldg(reinterpret_cast<const uint4 *>(kp) + c);
                const __half2 *hp = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(hp[i]);
                    kf[c * 8 + 2 * i] = f.x;
                    kf[c * 8 + 2 * i + 1] = f.y;
                }
            }
            // issue the V loads early
            uint4 vu[E / 8];
#pragma unroll
            for (int c = 0; c < E / 8; ++c) vu[c] = __ldg(reinterpret_cast<const uint4 *>(vp) + c);
            const float mval = mrow ? __half2float(mrow[cell]) : 0.0f;

            float s[G];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float a = 0.0f;
#pragma unroll
                for (int i = 0; i < E; ++i) a = fmaf(qf[h][i], kf[i], a);
                a += __shfl_xor_sync(sub_mask, a, 1);
                a += __shfl_xor_sync(sub_mask, a, 2);
                a += __shfl_xor_sync(sub_mask, a, 4);
                a *= p.scale;
                if (p.softcap != 0.0f) a = p.softcap * tanhf(a);
                s[h] = a + slope[h] * mval;
            }
            float vf[E];
#pragma unroll
            for (int c = 0; c < E / 8; ++c) {
                const __half2 *hp = reinterpret_cast<const __half2 *>(&vu[c]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(hp[i]);
                    vf[c * 8 + 2 * i] = f.x;
                    vf[c * 8 + 2 * i + 1] = f.y;
                }
            }
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float pw;
                if (s[h] > m[h]) {
                    const float ms = expf(m[h] - s[h]);
                    m[h] = s[h];
                    l[h] = l[h] * ms + 1.0f;
#pragma unroll
                    for (int i = 0; i < E; ++i) acc[h][i] *= ms;
                    pw = 1.0f;
                } else {
                    pw = expf(s[h] - m[h]);
                    l[h] += pw;
                }
#pragma unroll
                for (int i = 0; i < E; ++i) acc[h][i] = fmaf(pw, vf[i], acc[h][i]);
            }
        }
        __syncthreads();
    }

    // merge the four sub-warps of each warp (lanes e, e+8, e+16, e+24 hold the same elements)
#pragma unroll
    for (int h = 0; h < G; ++h) {
#pragma unroll
        for (int o = 8; o <= 16; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[h], o);
            const float lo = __shfl_xor_sync(0xffffffffu, l[h], o);
            const float mn = fmaxf(m[h], mo);
            const float sa = (m[h] == -CUDART_INF_F) ? 0.0f : expf(m[h] - mn);
            const float sb = (mo == -CUDART_INF_F) ? 0.0f : expf(mo - mn);
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const float ao = __shfl_xor_sync(0xffffffffu, acc[h][i], o);
                acc[h][i] = acc[h][i] * sa + ao * sb;
            }
            l[h] = l[h] * sa + lo * sb;
            m[h] = mn;
        }
    }
    if (lane < 8) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
            if (lane == 0) {
                merge_m[warp][h] = m[h];
                merge_l[warp][h] = l[h];
            }
#pragma unroll
            for (int i = 0; i < E; ++i) merge_acc[warp][h][e * E + i] = acc[h][i];
        }
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += FA_THREADS) {
        const int h = i / D, d = i - h * D;
        float mn = -CUDART_INF_F;
#pragma unroll
        for (int wv = 0; wv < 4; ++wv) mn = fmaxf(mn, merge_m[wv][h]);
        float a = 0.0f, ls = 0.0f;
#pragma unroll
        for (int wv = 0; wv < 4; ++wv) {
            const float sc = (merge_m[wv][h] == -CUDART_INF_F) ? 0.0f : expf(merge_m[wv][h] - mn);
            a += merge_acc[wv][h][d] * sc;
            ls += merge_l[wv][h] * sc;
        }
        const int64_t head = h0 + h;
        if (p.nsplit == 1) {
            p.dst[(j * p.H + head) * D + d] = a * (1.0f / ls);
        } else {
            float *pp = p.partial + ((j * p.H + head) * p.nsplit + split) * (D + 2);
            pp[d] = a;
            if (d == 0) {
                pp[D] = mn;
                pp[D + 1] = ls;
            }
        }
    }
}

template <int D>
__global__ void __launch_bounds__(D) fattn_combine_kernel(const float *__restrict__ partial, int nsplit, float *__restrict__ dst) {
    const int64_t row = blockIdx.x;  // token * H + head
    const int d = threadIdx.x;
    const float *pp = partial + row * nsplit * (D + 2);
    float mn = -CUDART_INF_F;
    for (int s = 0; s < nsplit; ++s) mn = fmaxf(mn, pp[s * (D + 2) + D]);
    float a = 0.0f, ls = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = pp[s * (D + 2) + D];
        const float sc = (ms == -CUDART_INF_F) ? 0.0f : expf(ms - mn);
        a += pp[s * (D + 2) + d] * sc;
        ls += pp[s * (D + 2) + D + 1] * sc;
    }
    dst[row * D + d] = a * (1.0f / ls);
}

static int fa_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

static int fattn_heads_per_cta(int gqa) { return gqa >= 4 && gqa % 4 == 0 ? 4 : (gqa % 2 == 0 ? 2 : 1); }

static int fattn_nsplit(int64_t Nq, int64_t Hkv, int hgroups, int64_t n_kv) {
    const int64_t ctas = Nq * Hkv * hgroups;
    const int64_t want = 2 * fa_sm_count();
    if (ctas >= want) return 1;
    int64_t ns = (want + ctas - 1) / ctas;
    ns = std::min<int64_t>(ns, std::max<int64_t>(1, n_kv / 512));
    return (int) std::min<int64_t>(ns, 64);
}

}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_mask_index_bytes(int64_t Nq, int64_t n_kv) {
    if (Nq <= 0 || n_kv <= 0) return 0;
    return align_up((size_t) Nq * ((n_kv + 63) / 64) * 8, 256);
}

int b200_mask_index_build(const void *mask, int64_t mask_nb_row, int64_t Nq, int64_t n_kv, void *index, size_t index_bytes,
                          b200_stream_t stream) {
    B200_REQUIRE(mask && index && Nq > 0 && n_kv > 0, "bad mask index arguments");
    B200_REQUIRE(is_aligned(mask, 2) && mask_nb_row % 2 == 0 && is_aligned(index, 8), "misaligned mask or index");
    if (index_bytes < b200_mask_index_bytes(Nq, n_kv)) return set_error(B200_E_SCRATCH, "mask index buffer too small");
    const int64_t nw = (n_kv + 63) / 64;
    const int64_t threads = Nq * nw * 32;
    mask_index_kernel<<<(unsigned) ((threads + 255) / 256), 256, 0, (cudaStream_t) stream>>>(
        (const __half *) mask, mask_nb_row, Nq, n_kv, nw, (unsigned long long *) index);
    return check_launch("mask_index");
}

size_t b200_flash_attn_scratch_bytes(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv) {
    if (D <= 0 || H <= 0 || Hkv <= 0 || Nq <= 0 || n_kv <= 0 || H % Hkv) return 0;
    const int hgroups = (int) (H / Hkv) / fattn_heads_per_cta((int) (H / Hkv));
    const int ns = fattn_nsplit(Nq, Hkv, hgroups, n_kv);
    const size_t part = ns > 1 ? align_up((size_t) Nq * H * ns * (D + 2) * sizeof(float), 256) : 0;
    return b200_mask_index_bytes(Nq, n_kv) + part;
}

int b200_flash_attn_ext_indexed(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv, const float *q, int64_t q_nb_tok,
                                int64_t q_nb_head, const void *k, int64_t k_nb_cell, int64_t k_nb_head, const void *v,
                                int64_t v_nb_cell, int64_t v_nb_head, const void *mask, int64_t mask_nb_row, const void *index,
                                float scale, float max_bias, float logit_softcap, float *dst, void *scratch, size_t scratch_bytes,
                                b200_stream_t stream) {
    B200_REQUIRE(D == 64 || D == 128, "head size %lld not supported (64 or 128)", (long long) D);
    B200_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0 && Nq > 0 && n_kv > 0, "bad attention shape");
    B200_REQUIRE(q && k && v && dst, "null pointer");
    B200_REQUIRE((mask == nullptr) == (index == nullptr), "mask and mask index must be given together");
    B200_REQUIRE(is_aligned(q, 4) && q_nb_tok % 4 == 0 && q_nb_head % 4 == 0, "misaligned q");
    B200_REQUIRE(is_aligned(k, 16) && k_nb_cell % 16 == 0 && k_nb_head % 16 == 0, "k rows must be 16-byte aligned");
    B200_REQUIRE(is_aligned(v, 16) && v_nb_cell % 16 == 0 && v_nb_head % 16 == 0, "v rows must be 16-byte aligned");
    B200_REQUIRE(!mask || (is_aligned(mask, 2) && mask_nb_row % 2 == 0), "misaligned mask");
    const int gqa = (int) (H / Hkv);
    const int G = fattn_heads_per_cta(gqa);
    const int hgroups = gqa / G;
    const int ns = fattn_nsplit(Nq, Hkv, hgroups, n_kv);
    const size_t part = ns > 1 ? (size_t) Nq * H * ns * (D + 2) * sizeof(float) : 0;
    if (part && (!scratch || scratch_bytes < part)) return set_error(B200_E_SCRATCH, "flash_attn scratch too small: %zu < %zu", scratch_bytes, part);
    B200_REQUIRE(!part || is_aligned(scratch, 16), "scratch must be 16-byte aligned");

    FattnParams p;
    p.H = H; p.Hkv = Hkv; p.Nq = Nq; p.n_kv = n_kv; p.nw = (n_kv + 63) / 64;
    p.q = q; p.q_nb_tok = q_nb_tok; p.q_nb_head = q_nb_head;
    p.k = (const char *) k; p.k_nb_cell = k_nb_cell; p.k_nb_head = k_nb_head;
    p.v = (const char *) v; p.v_nb_cell = v_nb_cell; p.v_nb_head = v_nb_head;
    p.mask = (const char *) mask; p.mask_nb_row = mask_nb_row;
    p.words = (const unsigned long long *) index;
    p.scale = logit_softcap != 0.0f ? scale / logit_softcap : scale;
    p.max_bias = max_bias; p.softcap = logit_softcap;
    p.n_head_log2 = 1u << (uint32_t) floor(log2((double) H));
    p.m0 = powf(2.0f, -(max_bias) / p.n_head_log2);
    p.m1 = powf(2.0f, -(max_bias / 2.0f) / p.n_head_log2);
    p.dst = dst; p.partial = (float *) scratch; p.nsplit = ns; p.hgroups = hgroups;
    p.words_per_split = (p.nw + ns - 1) / ns;

    dim3 grid((unsigned) Nq, (unsigned) (Hkv * hgroups), (unsigned) ns);
    cudaStream_t st = (cudaStream_t) stream;
#define FA_LAUNCH(DD, GG) fattn_vec_kernel<DD, GG><<<grid, FA_THREADS, 0, st>>>(p)
    if (D == 128) {
        if (G == 4) FA_LAUNCH(128, 4); else if (G == 2) FA_LAUNCH(128, 2); else FA_LAUNCH(128, 1);
    } else {
        if (G == 4) FA_LAUNCH(64, 4); else if (G == 2) FA_LAUNCH(64, 2); else FA_LAUNCH(64, 1);
    }
#undef FA_LAUNCH
    if (int e = check_launch("fattn_vec")) return e;
    if (ns > 1) {
        if (D == 128) fattn_combine_kernel<128><<<(unsigned) (Nq * H), 128, 0, st>>>(p.partial, ns, dst);
        else fattn_combine_kernel<64><<<(unsigned) (Nq * H), 64, 0, st>>>(p.partial, ns, dst);
        return check_launch("fattn_combine");
    }
    return B200_OK;
}

int b200_flash_attn_ext(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv, const float *q, int64_t q_nb_tok,
                        int64_t q_nb_head, const void *k, int64_t k_nb_cell, int64_t k_nb_head, const void *v, int64_t v_nb_cell,
                        int64_t v_nb_head, const void *mask, int64_t mask_nb_row, float scale, float max_bias, float logit_softcap,
                        float *dst, void *scratch, size_t scratch_bytes, b200_stream_t stream) {
    const size_t ib = mask ? b200_mask_index_bytes(Nq, n_kv) : 0;
    if (mask) {
        if (!scratch || scratch_bytes < ib) return set_error(B200_E_SCRATCH, "flash_attn scratch too small for the mask index");
        B200_REQUIRE(is_aligned(scratch, 256), "scratch must be 256-byte aligned");
        if (int e = b200_mask_index_build(mask, mask_nb_row, Nq, n_kv, scratch, ib, stream)) return e;
    }
    return b200_flash_attn_ext_indexed(D, H, Hkv, Nq, n_kv, q, q_nb_tok, q_nb_head, k, k_nb_cell, k_nb_head, v, v_nb_cell, v_nb_head,
                                       mask, mask_nb_row, mask ? scratch : nullptr, scale, max_bias, logit_softcap, dst,
                                       scratch ? (char *) scratch + ib : nullptr, scratch_bytes > ib ? scratch_bytes - ib : 0, stream);
}

}  // extern "C"
