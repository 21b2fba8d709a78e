// FLASH_ATTN_EXT over the f16 unified KV cache for ragged multi-sequence batches.
//
// Replaces lm_ggml_compute_forward_flash_attn_ext_f16 (cactus/ggml-cpu/ops.cpp:6948-7165).
//
// The mask tensor is honoured exactly as the reference does (a cell takes part iff its mask value is
// not -inf, the finite value is added to the scaled score), but it is scanned only once per graph:
// b200_mask_index_build turns each token's mask row into one bit per cell, and the attention kernel
// walks the set bits, so a token of a 64-sequence batch touches only its own sequence's K/V rows.
//
// Kernel: one CTA per (token, kv-head, group of up to 8 query heads, KV split), tensor-core MMAs for both
// Q K^T and P V (see fattn_mma_kernel).  With KV splits the partial (max, sum, accumulator) triples go to
// scratch and a combine kernel finishes.  A second, slow kernel reproduces the reference's own rounding
// sequence for validation (fattn_parity_kernel).
#include <math_constants.h>

#include <cstdlib>

#include "common.cuh"

namespace b200 {

int act_layout(int64_t N);   // quantize.cu: which B8 layout the mul_mat kernels expect for N columns


constexpr int FA_THREADS = 128;
#ifndef FA_MIN_CTAS
#define FA_MIN_CTAS 3
#endif
#ifndef FA_PREFETCH_V
#define FA_PREFETCH_V 0   // 1: the next chunk's V rows are requested as soon as the P V MMAs of the current one have read theirs (measured slower on B200: 67.9 us against 57.5 on 64 ragged sequences)
#endif
#ifndef FA_PREFETCH_K
#define FA_PREFETCH_K 1   // the next chunk's K rows are loaded during the softmax and P V MMAs of the current one (32 more registers)
#endif
constexpr int FA_SUPER_WORDS = 32;  // 2048 cells listed per round
constexpr int FA_MIN_SPLIT_WORDS = 2;   // 64-cell words a KV split walks at least (when the mask index gives a token's word count)
constexpr int FA_ADAPTIVE_SPLITS = 2;   // most KV splits a long sequence is cut into when the batch is small

// ---- mask scan: one warp per 64 cells of one token row ------------------------------------------
__global__ void __launch_bounds__(256) mask_index_kernel(const __half *__restrict__ mask, int64_t mask_nb_row, int64_t Nq,
                                                        int64_t n_kv, int64_t nw, unsigned long long *__restrict__ words, int32_t *soft) {
    const int lane = threadIdx.x & 31;
    const int64_t wid = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wid >= Nq * nw) return;
    const int64_t j = wid / nw, wi = wid - j * nw;
    const __half *row = reinterpret_cast<const __half *>(reinterpret_cast<const char *>(mask) + j * mask_nb_row);
    const int64_t c0 = wi * 64 + lane, c1 = c0 + 32;
    const unsigned short ninf = 0xFC00u;
    const unsigned short m0 = c0 < n_kv ? __half_as_ushort(row[c0]) : ninf, m1 = c1 < n_kv ? __half_as_ushort(row[c1]) : ninf;
    const bool v0 = m0 != ninf, v1 = m1 != ninf;
    // a participating cell whose mask value is not +-0 is added to the score: the mask is then more than its bits
    if (((v0 && (m0 & 0x7fffu)) || (v1 && (m1 & 0x7fffu))) && soft) *soft = 1;
    const unsigned lo = __ballot_sync(0xffffffffu, v0), hi = __ballot_sync(0xffffffffu, v1);
    if (lane == 0) words[wid] = (unsigned long long) lo | ((unsigned long long) hi << 32);
}

// Second pass of the mask scan: per token, the indices of the 64-cell words that have any participating cell,
// in ascending order, and their count.  A token of a 64-sequence batch owns a few dozen of the 1024 words of a
// 65536-cell cache, and the attention kernel walks only those.
__global__ void __launch_bounds__(256) mask_words_compact_kernel(const unsigned long long *__restrict__ words, int64_t Nq, int64_t nw,
                                                                int32_t *__restrict__ wlist, int32_t *__restrict__ wcount) {
    const int lane = threadIdx.x & 31;
    const int64_t j = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (j >= Nq) return;
    const unsigned long long *row = words + j * nw;
    int32_t *out = wlist + j * nw;
    int base = 0;
    for (int64_t w0 = 0; w0 < nw; w0 += 32) {
        const int64_t wi = w0 + lane;
        const bool nz = wi < nw && row[wi] != 0ull;
        const unsigned m = __ballot_sync(0xffffffffu, nz);
        if (nz) out[base + __popc(m & ((1u << lane) - 1u))] = (int32_t) wi;
        base += __popc(m);
    }
    if (lane == 0) wcount[j] = base;
}

// Third pass: the tokens ordered by decreasing word count (longest sequence first, so the scheduler hands the long
// walks out first and the short ones fill the gaps), and the total number of words, from which the attention kernel
// derives how many words one CTA should walk.
__global__ void __launch_bounds__(1024) fattn_plan_kernel(const int32_t *__restrict__ wcount, int64_t Nq, int32_t *__restrict__ order,
                                                         int32_t *__restrict__ plan) {
    __shared__ long long total_s;
    if (threadIdx.x == 0) total_s = 0;
    __syncthreads();
    long long part = 0;
    for (int64_t j = threadIdx.x; j < Nq; j += blockDim.x) {
        const int32_t c = wcount[j];
        part += c;
        int64_t rank = 0;   // tokens with more words, or as many and a lower index, come first
        for (int64_t i = 0; i < Nq; ++i) {
            const int32_t ci = wcount[i];
            rank += (ci > c || (ci == c && i < j)) ? 1 : 0;
        }
        order[rank] = (int32_t) j;
    }
    atomicAdd((unsigned long long *) &total_s, (unsigned long long) part);
    __syncthreads();
    if (threadIdx.x == 0) {
        plan[0] = (int32_t) min(total_s, (long long) 0x7fffffff);
        plan[1] = 0;   // filled by fattn_tile_vote_kernel
    }
}

// Fourth pass: how much the tokens of a ubatch share their cells.  plan[1] = the sum, over groups of 16 consecutive
// tokens, of the number of mask words any token of the group attends to.  Against plan[0] (the same sum token by token)
// it tells whether walking the cells once per group (fattn_tile_kernel) beats walking them once per token: a prompt's
// tokens share nearly all their words, the tokens of a decode batch share none.
__global__ void __launch_bounds__(256) fattn_tile_vote_kernel(const unsigned long long *__restrict__ words, int64_t Nq, int64_t nw, int32_t *__restrict__ plan) {
    const int64_t t0 = (int64_t) blockIdx.x * 16, t1 = min(Nq, t0 + 16);
    int cnt = 0;
    for (int64_t wi = threadIdx.x; wi < nw; wi += blockDim.x) {
        unsigned long long bits = 0;
        for (int64_t j = t0; j < t1; ++j) bits |= words[j * nw + wi];
        cnt += bits != 0ull;
    }
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if ((threadIdx.x & 31) == 0 && cnt) atomicAdd(plan + 1, cnt);
}
// the choice both attention kernels derive from the plan: true = the query-tiled kernel does the work
__device__ __forceinline__ bool fattn_tiled_chosen(const int32_t *plan) { return 2ll * plan[1] <= (long long) plan[0]; }

struct FattnParams {
    int64_t H, Hkv, Nq, n_kv, nw;
    const float *q; int64_t q_nb_tok, q_nb_head;
    const char *k; int64_t k_nb_cell, k_nb_head;
    const char *v; int64_t v_nb_cell, v_nb_head;
    const char *mask; int64_t mask_nb_row;
    const unsigned long long *words;  // NULL: every cell takes part
    const int32_t *wlist, *wcount;    // per token: indices of the non-empty words and their number (with words)
    float scale, max_bias, softcap, m0, m1;
    uint32_t n_head_log2;
    float *dst;      // may be null when qout is given
    uint8_t *qout;   // optional: the output rows quantised to Q8_0 in the B8 activation layout of the mul_mat that follows
    size_t q_d_offset;
    int64_t q_nb, q_nbp;
    int q_canon, q_variant;
    float *partial;  // [Nq][H][nsplit][D + 2]
    int nsplit, hgroups;
    int w0;          // > 0: a token gets ceil(words / w0) KV splits (at most nsplit), so long sequences are cut, short ones are not;
                     // < 0: w0 is derived on the device from the mask's total word count (fattn_target_words)
    const int32_t *order, *plan;   // tokens by decreasing word count; plan[0] = total words (NULL without a mask index)
    int slots;       // CTAs of this kernel the device holds at once
    int vote;        // both attention kernels were launched and the plan decides which one works (the other returns at once):
                     // 1 = these are the per-token kernel's launches, 2 = the query-tiled kernel's
    int early;       // one or two tokens: the combine pass lets the next kernel's CTAs in at once (pdl_early_rows)
};

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

}  // namespace b200
#include "fattn_tile.cuh"   // the query-tiled kernel for ubatches with many tokens
namespace b200 {

// Tensor-core kernel.  One CTA per (token, kv-head, head group of up to 8 query heads, KV split); its 4 warps take
// 16-cell chunks of the token's cell list in turn.  Per chunk and warp:
//   S = Q K^T   heads on the MMA rows (m16n8k16, f16 inputs, f32 accumulate), 8 cells per n-tile.  Lane (g, t)
//               loads 16-byte pieces d = 32u + 8t .. +7 of the K row of cell g -- the k index of the MMA is a fixed
//               permutation of d that makes those pieces B fragments as they are; Q is held in the same permutation
//               (rounded to fp16 as the reference rounds it).
//   online softmax on the accumulator rows (a head's four lanes share max and sum through two shuffles)
//   O^T += V^T P^T   d on the MMA rows, heads on the columns, so no accumulator row is wasted: lane (g, t) loads
//               d = 8g .. 8g+7 (and 64 + 8g ..) of the V rows of cells 2t, 2t+1, 2t+8, 2t+9 and pairs the halves of
//               two cells with byte permutes; P goes in as fp16 hi + lo parts (two MMAs), which keeps the
//               probabilities at fp32 accuracy.
// Every warp keeps its own (max, sum, accumulator) state; the states are merged through shared memory at the end.
// words one CTA should walk: 1.15 x the mean load of a CTA slot if the whole mask were spread evenly (at least 4 words)
__device__ __forceinline__ int fattn_target_words(const FattnParams &p, int ctas_per_token) {
    if (p.w0 >= 0) return p.w0;
    const long long total = p.plan ? p.plan[0] : p.Nq * p.nw;
    const long long w = (115ll * total * ctas_per_token + 100ll * p.slots - 1) / (100ll * p.slots);
    return (int) max(4ll, min(w, 0x7fffffffll));
}

// Called by the 32 lanes of a warp with 32 consecutive elements of one output row: quantises them as one Q8_0 block of
// column n.  A real call (not inlined): the attention kernel sits at its register limit and its main loop must not pay
// for this code.
__device__ __noinline__ void fattn_quant_block(uint8_t *qout, size_t d_offset, int64_t nb, int64_t nbp, int canon, int variant, int64_t n, int64_t b,
                                               float val, bool real) {
    if (canon) q8_quantize_store_warp<3>(val, qout, d_offset, nb, nbp, n, b, real, variant);
    else q8_quantize_store_warp<1>(val, qout, d_offset, nb, nbp, n, b, real, variant);
}

// One output element; a warp calls this for 32 consecutive d of one (token, head).  With QUANT the row is also (or only)
// stored as Q8_0 blocks -- quantize_row_q8_0 applied to the f32 value, bit for bit what the separate quantiser makes of
// dst -- and the last token's warps zero the padding columns of its 8-column tile.
template <int D, bool QUANT>
__device__ __forceinline__ void fattn_store_out(const FattnParams &p, int64_t j, int64_t head, int d, float val) {
    if (!QUANT) {
        p.dst[(j * p.H + head) * D + d] = val;
        return;
    }
    if (p.dst) p.dst[(j * p.H + head) * D + d] = val;
    const int64_t b = (head * D + d) >> 5;
    fattn_quant_block(p.qout, p.q_d_offset, p.q_nb, p.q_nbp, p.q_canon, p.q_variant, j, b, val, true);
    if (j == p.Nq - 1) {
        for (int64_t n = p.Nq; n < ((p.Nq + 7) & ~(int64_t) 7); ++n) fattn_quant_block(p.qout, p.q_d_offset, p.q_nb, p.q_nbp, p.q_canon, p.q_variant, n, b, 0.0f, false);
    }
}

// QUANT: the instantiation behind b200_flash_attn_ext_quant; kept apart because this kernel sits at its register limit
// and the plain one must not change with it
template <int D, bool QUANT>
__global__ void __launch_bounds__(FA_THREADS, FA_MIN_CTAS) fattn_mma_kernel(FattnParams p) {
    pdl_prologue();
    if (p.vote == 1 && fattn_tiled_chosen(p.plan)) return;   // the query-tiled kernel takes this ubatch
    constexpr int KS = D / 16;   // k-steps of the S MMA
    constexpr int NU = D / 32;   // 16-byte K pieces per lane and cell
    constexpr int NR = D / 64;   // 64-wide d ranges of V
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // blocks are handed out heads first, then tokens in the order of the plan: the longest sequences start first
    const int64_t j = p.order ? p.order[blockIdx.y] : blockIdx.y;
    const int hk = blockIdx.x / p.hgroups, hg = blockIdx.x % p.hgroups;
    const int split = blockIdx.z;
    const int gqa = (int) (p.H / p.Hkv);
    const int G = min(8, gqa - hg * 8);        // query heads of this CTA
    const int h0 = hk * gqa + hg * 8;

    __shared__ int cell_list[FA_SUPER_WORDS * 64];
    __shared__ int list_count;
    __shared__ float merge_m[4][8], merge_l[4][8];
    __shared__ float merge_acc[4][8][D];

    // Q fragments: row g = head h0 + g (zero rows beyond G)
    uint32_t qa0[KS], qa2[KS];
    {
        const bool valid = g < G;
        const float *qp = reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.q) + j * p.q_nb_tok + (int64_t) (h0 + (valid ? g : 0)) * p.q_nb_head);
#pragma unroll
        for (int u = 0; u < NU; ++u)
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const int d0 = 32 * u + 8 * t + 4 * v;
                const float4 f = valid ? *reinterpret_cast<const float4 *>(qp + d0) : make_float4(0.f, 0.f, 0.f, 0.f);
                qa0[2 * u + v] = pack_half2(f.x, f.y);
                qa2[2 * u + v] = pack_half2(f.z, f.w);
            }
    }
    const uint32_t hh = (uint32_t) (h0 + g);
    const float slope = (p.max_bias > 0.0f) ? (hh < p.n_head_log2 ? powf(p.m0, (float) (hh + 1)) : powf(p.m1, (float) (2 * (hh - p.n_head_log2) + 1))) : 1.0f;

    float oacc[8][4];   // O^T: d-tile q; [0],[1]: d = 8g+q, heads 2t, 2t+1; [2],[3]: d = 64+8g+q
#pragma unroll
    for (int q = 0; q < 8; ++q) oacc[q][0] = oacc[q][1] = oacc[q][2] = oacc[q][3] = 0.0f;
    float m_run = -CUDART_INF_F, l_run = 0.0f;   // state of head g (l: this lane's share of the row sum)

    // the words this CTA walks: entries [w_begin, w_end) of the token's list of non-empty words (or of all words
    // when there is no mask), an equal share per KV split
    const unsigned long long *wrow = p.words ? p.words + j * p.nw : nullptr;
    const int32_t *wl = p.words ? p.wlist + j * p.nw : nullptr;
    const int64_t n_words = p.words ? (int64_t) p.wcount[j] : p.nw;
    int ns_j = p.nsplit;   // KV splits of this token
    if (p.w0 != 0) {
        const int w0 = fattn_target_words(p, (int) gridDim.x);
        ns_j = (int) min((int64_t) p.nsplit, max((int64_t) 1, (n_words + w0 - 1) / w0));
        if (split >= ns_j) return;   // the whole CTA: nothing has been synchronised yet
    }
    const int64_t per_split = (n_words + ns_j - 1) / ns_j;
    const int64_t w_begin = (int64_t) split * per_split;
    const int64_t w_end = min(n_words, w_begin + per_split);
    const __half *mrow = p.mask ? reinterpret_cast<const __half *>(p.mask + j * p.mask_nb_row) : nullptr;
    const char *kbase = p.k + (int64_t) hk * p.k_nb_head;
    const char *vbase = p.v + (int64_t) hk * p.v_nb_head;

    for (int64_t w0 = w_begin; w0 < w_end; w0 += FA_SUPER_WORDS) {
        if (warp == 0) {   // list the participating cells of this round
            const int64_t e = w0 + lane;
            unsigned long long bits = 0;
            int64_t wi = 0;
            if (e < w_end) {
                if (wrow) {
                    wi = wl[e];
                    bits = wrow[wi];
                } else {
                    wi = e;
                    const int64_t left = p.n_kv - wi * 64;
                    bits = left >= 64 ? ~0ull : ((1ull << left) - 1ull);
                }
            }
            const int cnt = __popcll(bits);
            int pre = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int x = __shfl_up_sync(0xffffffffu, pre, o);
                if (lane >= o) pre += x;
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
        const int n_chunks = (count + 15) >> 4;
        const int last = count - 1;
        uint4 kr[2][NU];   // K rows of the two 8-cell tiles of a chunk: 16-byte pieces t, t+4, ... of cell g
        auto load_k = [&](int chunk) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int64_t cell = cell_list[min((chunk << 4) + 8 * c + g, last)];
                const uint4 *kp = reinterpret_cast<const uint4 *>(kbase + cell * p.k_nb_cell) + t;
#pragma unroll
                for (int u = 0; u < NU; ++u) kr[c][u] = __ldg(kp + 4 * u);
            }
        };
        uint4 vr[4][NR];   // V rows of a chunk: 16-byte piece g (and g + 8) of cells 2t, 2t+1, 2t+8, 2t+9
        auto load_v = [&](int chunk) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t cell = cell_list[min((chunk << 4) + 2 * t + (i & 1) + 8 * (i >> 1), last)];
                const uint4 *vp = reinterpret_cast<const uint4 *>(vbase + cell * p.v_nb_cell) + g;
#pragma unroll
                for (int r = 0; r < NR; ++r) vr[i][r] = __ldg(vp + 8 * r);
            }
        };
        if (FA_PREFETCH_K && warp < n_chunks) load_k(warp);
        if (FA_PREFETCH_V && warp < n_chunks) load_v(warp);
        for (int ch = warp; ch < n_chunks; ch += 4) {
            const int base = ch << 4;
            if (!FA_PREFETCH_K) load_k(ch);
            // ---- S = Q K^T for the two 8-cell tiles ----
            float sacc[2][4];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                sacc[c][0] = sacc[c][1] = sacc[c][2] = sacc[c][3] = 0.0f;
#pragma unroll
                for (int u = 0; u < NU; ++u) {
                    mma_f16(sacc[c], qa0[2 * u], 0u, qa2[2 * u], 0u, kr[c][u].x, kr[c][u].y);
                    mma_f16(sacc[c], qa0[2 * u + 1], 0u, qa2[2 * u + 1], 0u, kr[c][u].z, kr[c][u].w);
                }
            }
            // V rows of cells 2t, 2t+1, 2t+8, 2t+9 (already on their way with FA_PREFETCH_V)
            if (!FA_PREFETCH_V) load_v(ch);
            // the next chunk's K rows travel during the softmax and the P V MMAs of this one
            if (FA_PREFETCH_K && ch + 4 < n_chunks) load_k(ch + 4);
            // ---- scores of head g for cells base + {2t, 2t+1, 8+2t, 9+2t} ----
            float sc[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = base + 2 * t + (i & 1) + 8 * (i >> 1);
                float a = sacc[i >> 1][i & 1] * p.scale;
                if (p.softcap != 0.0f) a = p.softcap * tanhf(a);
                if (idx < count) {
                    if (mrow) a += slope * __half2float(mrow[cell_list[idx]]);
                } else {
                    a = -CUDART_INF_F;
                }
                sc[i] = a;
            }
            float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);   // finite: a chunk holds at least one participating cell
            const float alpha = __expf(m_run - m_new);
            float pr[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pr[i] = __expf(sc[i] - m_new);
            l_run = l_run * alpha + (pr[0] + pr[1]) + (pr[2] + pr[3]);
            m_run = m_new;
            // P^T fragments, fp16 hi + lo
            const __half2 h01 = __floats2half2_rn(pr[0], pr[1]), h23 = __floats2half2_rn(pr[2], pr[3]);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const uint32_t b0h = *reinterpret_cast<const uint32_t *>(&h01), b1h = *reinterpret_cast<const uint32_t *>(&h23);
            const uint32_t b0l = pack_half2(pr[0] - f01.x, pr[1] - f01.y), b1l = pack_half2(pr[2] - f23.x, pr[3] - f23.y);
            // rescale O^T columns (heads 2t, 2t+1) when some head's maximum moved
            if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                const float a_lo = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4);
                const float a_hi = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    oacc[q][0] *= a_lo; oacc[q][1] *= a_hi; oacc[q][2] *= a_lo; oacc[q][3] *= a_hi;
                }
            }
            // ---- O^T += V^T P^T ----
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint32_t sel = (q & 1) ? 0x7632u : 0x5410u;
                const uint32_t *wA0 = reinterpret_cast<const uint32_t *>(&vr[0][0]), *wB0 = reinterpret_cast<const uint32_t *>(&vr[1][0]);
                const uint32_t *wC0 = reinterpret_cast<const uint32_t *>(&vr[2][0]), *wD0 = reinterpret_cast<const uint32_t *>(&vr[3][0]);
                const uint32_t a0 = __byte_perm(wA0[q >> 1], wB0[q >> 1], sel);
                const uint32_t a2 = __byte_perm(wC0[q >> 1], wD0[q >> 1], sel);
                uint32_t a1 = 0u, a3 = 0u;
                if (NR == 2) {
                    const uint32_t *wA1 = reinterpret_cast<const uint32_t *>(&vr[0][NR - 1]), *wB1 = reinterpret_cast<const uint32_t *>(&vr[1][NR - 1]);
                    const uint32_t *wC1 = reinterpret_cast<const uint32_t *>(&vr[2][NR - 1]), *wD1 = reinterpret_cast<const uint32_t *>(&vr[3][NR - 1]);
                    a1 = __byte_perm(wA1[q >> 1], wB1[q >> 1], sel);
                    a3 = __byte_perm(wC1[q >> 1], wD1[q >> 1], sel);
                }
                mma_f16(oacc[q], a0, a1, a2, a3, b0h, b1h);
                mma_f16(oacc[q], a0, a1, a2, a3, b0l, b1l);
            }
            if (FA_PREFETCH_V && ch + 4 < n_chunks) load_v(ch + 4);
        }
        __syncthreads();
    }

    pdl_trigger();
    // ---- merge the four warps ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (t == 0) {
        merge_m[warp][g] = m_run;
        merge_l[warp][g] = l_run;
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        merge_acc[warp][2 * t][8 * g + q] = oacc[q][0];
        merge_acc[warp][2 * t + 1][8 * g + q] = oacc[q][1];
        if (NR == 2) {
            merge_acc[warp][2 * t][64 + 8 * g + q] = oacc[q][2];
            merge_acc[warp][2 * t + 1][64 + 8 * g + q] = oacc[q][3];
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
            const float scl = (merge_m[wv][h] == -CUDART_INF_F) ? 0.0f : expf(merge_m[wv][h] - mn);
            a += merge_acc[wv][h][d] * scl;
            ls += merge_l[wv][h] * scl;
        }
        const int64_t head = h0 + h;
        if (ns_j == 1) {
            fattn_store_out<D, QUANT>(p, j, head, d, a * (1.0f / ls));
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

// ---- validation variant: the reference's own order of operations ------------------------------------
// One warp per (token, head) walks the unmasked cells in ascending order and reproduces
// lm_ggml_compute_forward_flash_attn_ext_f16 step by step (cactus/ggml-cpu/ops.cpp:7072-7152) as the x86
// AVX2 build executes it: Q rounded to fp16; the K.Q dot as 4 x 8 fp32 FMA lanes folded in the order of
// LM_GGML_F32x8_REDUCE (lane l of the warp is accumulator l/8, SIMD lane l%8); scale and mask applied with one
// FMA; the output accumulator kept in fp16 and rounded after every cell (vec_scale_f16 / vec_mad_f16).
// It exists to show that what separates the fast kernel from the reference is that fp16 accumulator.
template <int D>
__global__ void __launch_bounds__(128) fattn_parity_kernel(FattnParams p) {
    constexpr int E = D / 32;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t) blockIdx.x * 4 + (threadIdx.x >> 5);   // token * H + head
    if (row >= p.Nq * p.H) return;
    const int64_t j = row / p.H;
    const int h = (int) (row - j * p.H);
    const int hk = h / (int) (p.H / p.Hkv);
    const float *qp = reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.q) + j * p.q_nb_tok + (int64_t) h * p.q_nb_head);
    float qf[E];
    __half acc[E];
#pragma unroll
    for (int i = 0; i < E; ++i) {
        qf[i] = __half2float(__float2half_rn(qp[lane + 32 * i]));
        acc[i] = __float2half_rn(0.0f);
    }
    const uint32_t hh = (uint32_t) h;
    const float slope = (p.max_bias > 0.0f) ? (hh < p.n_head_log2 ? powf(p.m0, (float) (hh + 1)) : powf(p.m1, (float) (2 * (hh - p.n_head_log2) + 1))) : 1.0f;
    float S = 0.0f, M = -CUDART_INF_F;
    const unsigned long long *wrow = p.words ? p.words + j * p.nw : nullptr;
    const __half *mrow = p.mask ? reinterpret_cast<const __half *>(p.mask + j * p.mask_nb_row) : nullptr;
    for (int64_t wi = 0; wi < p.nw; ++wi) {
        unsigned long long bits;
        if (wrow) {
            bits = wrow[wi];
        } else {
            const int64_t left = p.n_kv - wi * 64;
            bits = left >= 64 ? ~0ull : ((1ull << left) - 1ull);
        }
        while (bits) {
            const int b = __ffsll((long long) bits) - 1;
            bits &= bits - 1;
            const int64_t cell = wi * 64 + b;
            const __half *kr = reinterpret_cast<const __half *>(p.k + cell * p.k_nb_cell + (int64_t) hk * p.k_nb_head);
            const __half *vr = reinterpret_cast<const __half *>(p.v + cell * p.v_nb_cell + (int64_t) hk * p.v_nb_head);
            float a = 0.0f;
#pragma unroll
            for (int i = 0; i < E; ++i) a = __fmaf_rn(__half2float(kr[lane + 32 * i]), qf[i], a);
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 16));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 8));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 4));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
            a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
            const float mv = mrow ? __fmul_rn(slope, __half2float(mrow[cell])) : 0.0f;
            float s;
            if (p.softcap != 0.0f) {
                s = __fmul_rn(a, p.scale);
                s = __fmul_rn(p.softcap, tanhf(s));
                s = __fadd_rn(s, mv);
            } else {
                s = __fmaf_rn(a, p.scale, mv);
            }
            float ms = 1.0f, vs = 1.0f;
            if (s > M) {
                ms = (float) exp((double) __fsub_rn(M, s));   // correctly rounded, as the host libm's expf is in all but rare cases
                M = s;
#pragma unroll
                for (int i = 0; i < E; ++i) acc[i] = __float2half_rn(__fmul_rn(__half2float(acc[i]), ms));
            } else {
                vs = (float) exp((double) __fsub_rn(s, M));
            }
#pragma unroll
            for (int i = 0; i < E; ++i) acc[i] = __float2half_rn(__fmaf_rn(__half2float(vr[lane + 32 * i]), vs, __half2float(acc[i])));
            S = __fmaf_rn(S, ms, vs);
        }
    }
    const float S_inv = __fdiv_rn(1.0f, S);
#pragma unroll
    for (int i = 0; i < E; ++i) p.dst[row * D + lane + 32 * i] = __fmul_rn(__half2float(acc[i]), S_inv);
}

template <int D, bool QUANT>
__global__ void __launch_bounds__(D) fattn_combine_kernel(FattnParams p, int ctas_per_token) {
    pdl_prologue(p.early != 0);
    if (p.vote == 1 && fattn_tiled_chosen(p.plan)) return;    // the query-tiled kernel wrote the result
    if (p.vote == 2 && !fattn_tiled_chosen(p.plan)) return;   // this is the query-tiled kernel's combine pass and the per-token kernel worked
    const float *__restrict__ partial = p.partial;
    int nsplit = p.nsplit;
    const int64_t row = blockIdx.x;  // token * H + head
    const int d = threadIdx.x;
    const float *pp = partial + row * nsplit * (D + 2);
    if (p.w0 != 0) {   // the splits this token really has; a token with one split was written directly
        const int w0 = fattn_target_words(p, ctas_per_token);
        const int64_t n_words = p.wcount ? (int64_t) p.wcount[row / p.H] : p.nw;
        nsplit = (int) min((int64_t) nsplit, max((int64_t) 1, (n_words + w0 - 1) / w0));
        if (nsplit == 1) return;
    }
    float mn = -CUDART_INF_F;
    for (int s = 0; s < nsplit; ++s) mn = fmaxf(mn, pp[s * (D + 2) + D]);
    float a = 0.0f, ls = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = pp[s * (D + 2) + D];
        const float sc = (ms == -CUDART_INF_F) ? 0.0f : expf(ms - mn);
        a += pp[s * (D + 2) + d] * sc;
        ls += pp[s * (D + 2) + D + 1] * sc;
    }
    fattn_store_out<D, QUANT>(p, row / p.H, row % p.H, d, a * (1.0f / ls));
}


static int fattn_hgroups(int gqa) { return (gqa + 7) / 8; }   // a CTA takes up to 8 query heads of one KV head

static int fa_sm_count() {   // every device of a process is the same model
    static const int n = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

// Decode-sized batches over ragged sequences: one CTA per (token, kv head) makes the longest sequence the kernel's
// duration.  When the grid is small enough for spare CTAs to be cheap (at most two waves), a token whose mask has more
// words than fattn_target_words is cut into up to FA_ADAPTIVE_SPLITS KV splits; the rest are written directly.
static bool fattn_adaptive(int64_t Nq, int64_t Hkv, int hgroups, bool have_index) {
    static const int allow = [] {
        const char *e = getenv("B200_FA_ADAPTIVE");   // opt-in: on the 64-sequence decode batch the cuts cost more than they save
        return (e && atoi(e) == 1) ? 1 : 0;
    }();
    return allow && have_index && Nq * Hkv * hgroups <= 2 * (int64_t) FA_MIN_CTAS * fa_sm_count();
}

static int fattn_nsplit(int64_t Nq, int64_t Hkv, int hgroups, int64_t n_kv) {
    static const int forced = [] {
        const char *e = getenv("B200_FA_NSPLIT");
        return e ? atoi(e) : 0;
    }();
    if (forced > 0) return (int) std::min<int64_t>(forced, 64);
    const int64_t ctas = Nq * Hkv * hgroups;
    const int64_t want = 2 * fa_sm_count();
    if (ctas >= want) return 1;
    int64_t ns = (want + ctas - 1) / ctas;
    ns = std::min<int64_t>(ns, std::max<int64_t>(1, n_kv / 512));
    return (int) std::min<int64_t>(ns, 64);
}

static bool cuda_memset_ok(void *p, size_t n, cudaStream_t st) { return cudaMemsetAsync(p, 0, n, st) == cudaSuccess; }
int fattn_tile_min_nq();

// KV splits of the query-tiled kernel: enough CTAs for two per SM twice over, a split walks at least 256 cells
static int fattn_tile_nsplit(int64_t Nq, int64_t Hkv, int gqa, int64_t n_kv) {
    int gl = 0;
    while ((1 << gl) < gqa) ++gl;
    const int64_t tiles = (Nq + (64 >> gl) - 1) / (64 >> gl), ctas = tiles * Hkv, want = 4 * (int64_t) fa_sm_count();
    int64_t ns = ctas >= want ? 1 : (want + ctas - 1) / ctas;
    ns = std::min<int64_t>(ns, std::max<int64_t>(1, n_kv / 256));
    return (int) std::min<int64_t>(ns, 8);
}
static bool fattn_tile_possible(int64_t Nq, int gqa) {
    const int tile_min = fattn_tile_min_nq();
    return tile_min > 0 && Nq >= tile_min && (gqa & (gqa - 1)) == 0 && gqa >= 2 && gqa <= 16;   // a tile holds 64 / gqa tokens: at most 32
}

// token count from which the query-tiled kernel is considered (B200_FA_TILE_MIN_NQ; 0 turns it off)
int fattn_tile_min_nq() {
    static const int v = [] {
        const char *e = getenv("B200_FA_TILE_MIN_NQ");
        return e ? atoi(e) : 128;
    }();
    return v;
}

}  // namespace b200

using namespace b200;

extern "C" {

// index layout: words [Nq][nw] u64 | list of non-empty word indices [Nq][nw] i32 | their counts [Nq] i32 |
// tokens by decreasing count [Nq] i32 | plan: total words i32, words summed over 16-token groups i32, 1 if the mask
// holds values other than 0 and -inf in participating cells i32
static size_t index_list_offset(int64_t Nq, int64_t nw) { return align_up((size_t) Nq * nw * 8, 256); }
static size_t index_count_offset(int64_t Nq, int64_t nw) { return index_list_offset(Nq, nw) + align_up((size_t) Nq * nw * 4, 256); }

static size_t index_order_offset(int64_t Nq, int64_t nw) { return index_count_offset(Nq, nw) + align_up((size_t) Nq * 4, 256); }
static size_t index_plan_offset(int64_t Nq, int64_t nw) { return index_order_offset(Nq, nw) + align_up((size_t) Nq * 4, 256); }

size_t b200_mask_index_bytes(int64_t Nq, int64_t n_kv) {
    if (Nq <= 0 || n_kv <= 0) return 0;
    const int64_t nw = (n_kv + 63) / 64;
    return index_plan_offset(Nq, nw) + 256;
}

int b200_mask_index_build(const void *mask, int64_t mask_nb_row, int64_t Nq, int64_t n_kv, void *index, size_t index_bytes,
                          b200_stream_t stream) {
    B200_REQUIRE(mask && index && Nq > 0 && n_kv > 0, "bad mask index arguments");
    B200_REQUIRE(is_aligned(mask, 2) && mask_nb_row % 2 == 0 && is_aligned(index, 8), "misaligned mask or index");
    if (index_bytes < b200_mask_index_bytes(Nq, n_kv)) return set_error(B200_E_SCRATCH, "mask index buffer too small");
    const int64_t nw = (n_kv + 63) / 64;
    const int64_t threads = Nq * nw * 32;
    int32_t *plan = (int32_t *) ((char *) index + index_plan_offset(Nq, nw));
    if (!cuda_memset_ok(plan + 2, 4, (cudaStream_t) stream)) return set_error(B200_E_CUDA, "mask index: cudaMemsetAsync failed");
    mask_index_kernel<<<(unsigned) ((threads + 255) / 256), 256, 0, (cudaStream_t) stream>>>(
        (const __half *) mask, mask_nb_row, Nq, n_kv, nw, (unsigned long long *) index, plan + 2);
    if (int e = check_launch("mask_index")) return e;
    mask_words_compact_kernel<<<(unsigned) ((Nq * 32 + 255) / 256), 256, 0, (cudaStream_t) stream>>>(
        (const unsigned long long *) index, Nq, nw, (int32_t *) ((char *) index + index_list_offset(Nq, nw)),
        (int32_t *) ((char *) index + index_count_offset(Nq, nw)));
    if (int e = check_launch("mask_words_compact")) return e;
    fattn_plan_kernel<<<1, 1024, 0, (cudaStream_t) stream>>>((const int32_t *) ((char *) index + index_count_offset(Nq, nw)), Nq,
                                                             (int32_t *) ((char *) index + index_order_offset(Nq, nw)),
                                                             (int32_t *) ((char *) index + index_plan_offset(Nq, nw)));
    if (int e = check_launch("fattn_plan")) return e;
    if (Nq >= fattn_tile_min_nq() && fattn_tile_min_nq() > 0) {   // only ubatches the query-tiled kernel may take need the vote
        fattn_tile_vote_kernel<<<(unsigned) ((Nq + 15) / 16), 256, 0, (cudaStream_t) stream>>>((const unsigned long long *) index, Nq, nw,
                                                                                                 (int32_t *) ((char *) index + index_plan_offset(Nq, nw)));
        return check_launch("fattn_tile_vote");
    }
    return B200_OK;
}

size_t b200_flash_attn_scratch_bytes(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv) {
    if (D <= 0 || H <= 0 || Hkv <= 0 || Nq <= 0 || n_kv <= 0 || H % Hkv) return 0;
    const int hgroups = fattn_hgroups((int) (H / Hkv));
    int ns = fattn_nsplit(Nq, Hkv, hgroups, n_kv);
    if (ns == 1 && fattn_adaptive(Nq, Hkv, hgroups, true)) ns = FA_ADAPTIVE_SPLITS;
    if (fattn_tile_possible(Nq, (int) (H / Hkv))) ns = std::max(ns, fattn_tile_nsplit(Nq, Hkv, (int) (H / Hkv), n_kv));
    const size_t part = ns > 1 ? align_up((size_t) Nq * H * ns * (D + 2) * sizeof(float), 256) : 0;
    return b200_mask_index_bytes(Nq, n_kv) + part;
}

static int flash_attn_impl(bool parity, int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv, const float *q, int64_t q_nb_tok,
                           int64_t q_nb_head, const void *k, int64_t k_nb_cell, int64_t k_nb_head, const void *v,
                           int64_t v_nb_cell, int64_t v_nb_head, const void *mask, int64_t mask_nb_row, const void *index,
                           float scale, float max_bias, float logit_softcap, float *dst, void *scratch, size_t scratch_bytes,
                           b200_stream_t stream, void *act = nullptr, size_t act_bytes = 0, int variant = B200_Q8_AVX2) {
    B200_REQUIRE(D == 64 || D == 128, "head size %lld not supported (64 or 128)", (long long) D);
    B200_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0 && Nq > 0 && n_kv > 0, "bad attention shape");
    B200_REQUIRE(q && k && v && (dst || act), "null pointer");
    if (act) {
        B200_REQUIRE(!parity && (H * D) % 128 == 0, "quantised output needs H * D to be a multiple of 128");
        B200_REQUIRE(variant == B200_Q8_AVX2 || variant == B200_Q8_SCALAR, "unknown quantiser variant %d", variant);
        B200_REQUIRE(is_aligned(act, 256), "activation scratch must be 256-byte aligned");
        if (act_bytes < act_dims(H * D, Nq).total_bytes) return set_error(B200_E_SCRATCH, "activation scratch too small: %zu < %zu", act_bytes, act_dims(H * D, Nq).total_bytes);
    }
    B200_REQUIRE((mask == nullptr) == (index == nullptr), "mask and mask index must be given together");
    B200_REQUIRE(is_aligned(q, 4) && q_nb_tok % 4 == 0 && q_nb_head % 4 == 0, "misaligned q");
    B200_REQUIRE(is_aligned(k, 16) && k_nb_cell % 16 == 0 && k_nb_head % 16 == 0, "k rows must be 16-byte aligned");
    B200_REQUIRE(is_aligned(v, 16) && v_nb_cell % 16 == 0 && v_nb_head % 16 == 0, "v rows must be 16-byte aligned");
    B200_REQUIRE(!mask || (is_aligned(mask, 2) && mask_nb_row % 2 == 0), "misaligned mask");
    const int gqa = (int) (H / Hkv);
    const int hgroups = fattn_hgroups(gqa);
    int ns = parity ? 1 : fattn_nsplit(Nq, Hkv, hgroups, n_kv);
    int w0 = 0;
    if (!parity && ns == 1 && fattn_adaptive(Nq, Hkv, hgroups, index != nullptr)) {
        ns = FA_ADAPTIVE_SPLITS;
        w0 = -1;
    }
    // a split of fewer than two 64-cell words is more launch and combine work than it saves: a token takes at most half as
    // many splits as it has words (measured on one sequence of 2048 cells: 16 splits 2.41 ms per 8B step, 32 splits 2.45,
    // 8 splits 2.46).  The token's word count is known on the device only, so this needs the mask index.
    if (!parity && ns > 1 && w0 == 0 && index) w0 = FA_MIN_SPLIT_WORDS;
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
    p.wlist = index ? (const int32_t *) ((const char *) index + index_list_offset(Nq, p.nw)) : nullptr;
    p.wcount = index ? (const int32_t *) ((const char *) index + index_count_offset(Nq, p.nw)) : nullptr;
    p.scale = logit_softcap != 0.0f ? scale / logit_softcap : scale;
    p.max_bias = max_bias; p.softcap = logit_softcap;
    p.n_head_log2 = 1u << (uint32_t) floor(log2((double) H));
    p.m0 = powf(2.0f, -(max_bias) / p.n_head_log2);
    p.m1 = powf(2.0f, -(max_bias / 2.0f) / p.n_head_log2);
    p.dst = dst; p.partial = (float *) scratch; p.nsplit = ns; p.hgroups = hgroups; p.w0 = w0;
    const ActDims ad = act_dims(H * D, Nq);
    p.qout = (uint8_t *) act; p.q_d_offset = ad.d_offset; p.q_nb = ad.nb; p.q_nbp = ad.nbp;
    p.q_canon = act_layout(Nq) == 3 ? 1 : 0; p.q_variant = variant;
    p.order = index ? (const int32_t *) ((const char *) index + index_order_offset(Nq, p.nw)) : nullptr;
    p.plan = index ? (const int32_t *) ((const char *) index + index_plan_offset(Nq, p.nw)) : nullptr;
    p.slots = FA_MIN_CTAS * fa_sm_count();
    B200_REQUIRE(Nq <= 65535, "at most 65535 tokens per call");

    cudaStream_t st = (cudaStream_t) stream;
    if (parity) {
        const unsigned blocks = (unsigned) ((Nq * H + 3) / 4);
        if (D == 128) fattn_parity_kernel<128><<<blocks, 128, 0, st>>>(p);
        else fattn_parity_kernel<64><<<blocks, 128, 0, st>>>(p);
        return check_launch("fattn_parity");
    }
    // Many query tokens: the query-tiled kernel shares every staged K/V chunk between the 64 / gqa tokens of a tile.  That
    // pays when the tokens share their cells (a prompt), not when every token has its own sequence (a large decode batch);
    // with a mask index both kernels are launched and the plan the index holds decides on the device which one works.
    int gqa_log2 = 0;
    while ((1 << gqa_log2) < gqa) ++gqa_log2;
    p.vote = 0;
    p.early = Nq <= pdl_early_rows() ? 1 : 0;
    if (!act && dst && fattn_tile_possible(Nq, gqa) && p.nw <= 2048) {
        FattnParams pt = p;
        pt.vote = index ? 2 : 0;
        pt.w0 = 0;
        pt.nsplit = fattn_tile_nsplit(Nq, Hkv, gqa, n_kv);
        const size_t tpart = pt.nsplit > 1 ? (size_t) Nq * H * pt.nsplit * (D + 2) * sizeof(float) : 0;
        if (tpart && (!scratch || scratch_bytes < tpart || !is_aligned(scratch, 16))) pt.nsplit = 1;   // an older scratch size: no splits
        const int tile_tokens = 64 >> gqa_log2;
        dim3 tgrid((unsigned) Hkv, (unsigned) ((Nq + tile_tokens - 1) / tile_tokens), (unsigned) pt.nsplit);
        // the opt-in to more than 48 KB of shared memory is per function and device
        static thread_local int tile_smem_dev = -1;
        int dev_now = 0;
        cudaGetDevice(&dev_now);
        if (tile_smem_dev != dev_now) {
            cudaFuncSetAttribute(fattn_tile_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, fattn_tile_smem_bytes(128));
            cudaFuncSetAttribute(fattn_tile_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, fattn_tile_smem_bytes(64));
            tile_smem_dev = dev_now;
        }
        if (D == 128) launch_pdl(fattn_tile_kernel<128>, tgrid, dim3(FT_THREADS), (size_t) fattn_tile_smem_bytes(128), st, pt, gqa_log2);
        else launch_pdl(fattn_tile_kernel<64>, tgrid, dim3(FT_THREADS), (size_t) fattn_tile_smem_bytes(64), st, pt, gqa_log2);
        if (int e = check_launch("fattn_tile")) return e;
        if (pt.nsplit > 1) {
            if (D == 128) launch_pdl(fattn_combine_kernel<128, false>, dim3((unsigned) (Nq * H)), dim3(128), 0, st, pt, 1);
            else launch_pdl(fattn_combine_kernel<64, false>, dim3((unsigned) (Nq * H)), dim3(64), 0, st, pt, 1);
            if (int e = check_launch("fattn_combine")) return e;
        }
        if (!index) return B200_OK;   // no mask: every token attends every cell, nothing to vote on
        p.vote = 1;
    }
    dim3 grid((unsigned) (Hkv * hgroups), (unsigned) Nq, (unsigned) ns);
    const bool qo = act != nullptr;
    if (D == 128) {
        if (qo) launch_pdl(fattn_mma_kernel<128, true>, grid, dim3(FA_THREADS), 0, st, p);
        else launch_pdl(fattn_mma_kernel<128, false>, grid, dim3(FA_THREADS), 0, st, p);
    } else {
        if (qo) launch_pdl(fattn_mma_kernel<64, true>, grid, dim3(FA_THREADS), 0, st, p);
        else launch_pdl(fattn_mma_kernel<64, false>, grid, dim3(FA_THREADS), 0, st, p);
    }
    if (int e = check_launch("fattn_mma")) return e;
    if (ns > 1) {
        const dim3 cgrid((unsigned) (Nq * H));
        const int cpt = (int) (Hkv * hgroups);
        if (D == 128) {
            if (qo) launch_pdl(fattn_combine_kernel<128, true>, cgrid, dim3(128), 0, st, p, cpt);
            else launch_pdl(fattn_combine_kernel<128, false>, cgrid, dim3(128), 0, st, p, cpt);
        } else {
            if (qo) launch_pdl(fattn_combine_kernel<64, true>, cgrid, dim3(64), 0, st, p, cpt);
            else launch_pdl(fattn_combine_kernel<64, false>, cgrid, dim3(64), 0, st, p, cpt);
        }
        return check_launch("fattn_combine");
    }
    return B200_OK;
}

int b200_flash_attn_ext_indexed(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv, const float *q, int64_t q_nb_tok,
                                int64_t q_nb_head, const void *k, int64_t k_nb_cell, int64_t k_nb_head, const void *v,
                                int64_t v_nb_cell, int64_t v_nb_head, const void *mask, int64_t mask_nb_row, const void *index,
                                float scale, float max_bias, float logit_softcap, float *dst, void *scratch, size_t scratch_bytes,
                                b200_stream_t stream) {
    return flash_attn_impl(false, D, H, Hkv, Nq, n_kv, q, q_nb_tok, q_nb_head, k, k_nb_cell, k_nb_head, v, v_nb_cell, v_nb_head, mask, mask_nb_row,
                           index, scale, max_bias, logit_softcap, dst, scratch, scratch_bytes, stream);
}

int b200_flash_attn_ext_quant(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv, const float *q, int64_t q_nb_tok,
                              int64_t q_nb_head, const void *k, int64_t k_nb_cell, int64_t k_nb_head, const void *v,
                              int64_t v_nb_cell, int64_t v_nb_head, const void *mask, int64_t mask_nb_row, const void *index,
                              float scale, float max_bias, float logit_softcap, float *dst, void *act, size_t act_bytes, int variant,
                              void *scratch, size_t scratch_bytes, b200_stream_t stream) {
    B200_REQUIRE(act, "null activation scratch");
    return flash_attn_impl(false, D, H, Hkv, Nq, n_kv, q, q_nb_tok, q_nb_head, k, k_nb_cell, k_nb_head, v, v_nb_cell, v_nb_head, mask, mask_nb_row,
                           index, scale, max_bias, logit_softcap, dst, scratch, scratch_bytes, stream, act, act_bytes, variant);
}

int b200_flash_attn_ext_parity(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv, const float *q, int64_t q_nb_tok,
                               int64_t q_nb_head, const void *k, int64_t k_nb_cell, int64_t k_nb_head, const void *v,
                               int64_t v_nb_cell, int64_t v_nb_head, const void *mask, int64_t mask_nb_row, const void *index,
                               float scale, float max_bias, float logit_softcap, float *dst, b200_stream_t stream) {
    return flash_attn_impl(true, D, H, Hkv, Nq, n_kv, q, q_nb_tok, q_nb_head, k, k_nb_cell, k_nb_head, v, v_nb_cell, v_nb_head, mask, mask_nb_row,
                           index, scale, max_bias, logit_softcap, dst, nullptr, 0, stream);
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
