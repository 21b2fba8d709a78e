// FLASH_ATTN_EXT for ubatches with many query tokens (prefill): query-tiled kernel.
//
// Same computation as fattn_mma_kernel (lm_ggml_compute_forward_flash_attn_ext_f16, cactus/ggml-cpu/ops.cpp:6948-7165),
// different work split.  The decode kernel gives every (token, kv-head) its own CTA, so the tokens of one prompt walk the
// same K/V rows once each.  Here a CTA owns a tile of consecutive tokens of the ubatch and one kv-head: 4 warps x 16 MMA
// rows, a row being one (token, query head of the group) pair -- 16 / gqa tokens per warp, 64 / gqa per CTA.  The CTA walks
// the union of its tokens' cells (the OR of their mask words) in chunks of 32 cells; a chunk's K and V rows are staged in
// shared memory once (cp.async, three stages) and used by all 64 rows.  A row's own mask value (-inf outside its
// sequence and beyond its position) is added to every score, so the causal triangle and ragged tiles that straddle two
// sequences need no special case.  When the mask holds nothing but 0 and -inf (the index build records that) the row's
// mask value comes from its mask-word bits (turned, once per round of 1024 cells, into 32 bits per token and chunk in
// shared memory) instead of from the f16 mask in global memory.  Long tiles are cut into KV splits (grid z): split z takes every nsplit-th
// chunk of the union list, the partial (max, sum, accumulator) triples go to scratch and fattn_combine_kernel finishes.
//   S = Q K^T   m16n8k16, Q rounded to fp16 as the reference rounds it, K fragments straight from the staged rows
//   online softmax per row (the four lanes of a row share max and sum through two shuffles)
//   O += P V    P goes in as fp16 hi + lo parts (two MMAs), which keeps the probabilities at fp32 accuracy; V fragments
//               come from the staged rows through ldmatrix.trans
#pragma once

namespace b200 {

constexpr int FT_THREADS = 128;
constexpr int FT_CHUNK = 32;            // cells per step
constexpr int FT_RW = 16;               // mask words (of 64 cells) listed per round
constexpr int FT_LIST = FT_RW * 64;     // cells listed per round at most
constexpr int FT_STAGES = 3;            // K/V chunks in flight
constexpr int FT_MAX_TILE = 32;         // tokens of a tile at most (gqa 2)
constexpr int FT_MAX_WORDS = 2048;      // mask words of a row at most (131072 cells)

__device__ __forceinline__ void ft_cp16(uint32_t smem, const void *g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem), "l"(g) : "memory");
}
__device__ __forceinline__ void ft_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// dynamic shared memory of the kernel: FT_STAGES stages of K and V rows
constexpr int fattn_tile_smem_bytes(int D) { return FT_STAGES * 2 * FT_CHUNK * (D * 2 + 16); }

template <int D>
__global__ void __launch_bounds__(FT_THREADS, 3) fattn_tile_kernel(FattnParams p, int gqa_log2) {
    pdl_prologue();
    if (p.vote == 2 && !fattn_tiled_chosen(p.plan)) return;   // the tokens share too few cells: the per-token kernel takes this ubatch
    constexpr int KS = D / 16;            // k-steps of S
    constexpr int NT = D / 8;             // n-tiles of O
    constexpr int ROW = D * 2 + 16;       // bytes of a staged K / V row (the pad spreads the 8 rows of a fragment over all banks)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int gqa = 1 << gqa_log2;
    const int tw = 16 >> gqa_log2;                      // tokens per warp
    const int64_t tok0 = (int64_t) blockIdx.y * (4 * tw);   // first token of the tile
    const int hk = blockIdx.x;
    const int split = blockIdx.z, nsplit = p.nsplit;
    const bool binary_mask = p.words && p.plan && p.plan[2] == 0;   // only 0 / -inf in the mask: a row's bit says it all

    __shared__ int cell_list[FT_LIST];                    // the cells of this round, ascending
    __shared__ unsigned short cell_kb[FT_LIST];           // where each sits among the round's words: 64 * slot + bit
    __shared__ unsigned short uw_index[FT_MAX_WORDS];     // the mask words any token of the tile attends to, ascending
    __shared__ unsigned long long tile_words[FT_MAX_TILE][FT_RW];   // the round's words, token by token
    __shared__ unsigned long long ubits[FT_RW];           // their union
    __shared__ int wbase[FT_RW];                          // cells listed before each word
    __shared__ unsigned rmask[FT_MAX_TILE][FT_LIST / FT_CHUNK];   // per token and chunk: which of the chunk's 32 cells the token attends to
    __shared__ int list_count, uw_count, warp_cnt[4];
    extern __shared__ __align__(16) uint8_t kv_s[];   // [stage][K, V][FT_CHUNK rows of ROW bytes] (dynamic: fattn_tile_smem_bytes)

    // rows g and g + 8 of this warp: (token, head)
    int64_t tok[2];
    int head[2], tl[2];
    bool live[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        tl[i] = warp * tw + (r >> gqa_log2);   // token within the tile
        tok[i] = tok0 + tl[i];
        head[i] = hk * gqa + (r & (gqa - 1));
        live[i] = tok[i] < p.Nq;
    }
    // Q as A fragments: a0 = (row g, d 16 ks + 2t, +1), a1 = (row g + 8, same), a2 = (row g, d 16 ks + 8 + 2t, +1), a3 = (row g + 8, same)
    uint32_t qa[KS][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float *qp = reinterpret_cast<const float *>(reinterpret_cast<const char *>(p.q) + (live[i] ? tok[i] : 0) * p.q_nb_tok + (int64_t) head[i] * p.q_nb_head);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const float2 lo = live[i] ? *reinterpret_cast<const float2 *>(qp + 16 * ks + 2 * t) : make_float2(0.f, 0.f);
            const float2 hi = live[i] ? *reinterpret_cast<const float2 *>(qp + 16 * ks + 8 + 2 * t) : make_float2(0.f, 0.f);
            qa[ks][i] = pack_half2(lo.x, lo.y);
            qa[ks][2 + i] = pack_half2(hi.x, hi.y);
        }
    }
    float slope[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint32_t hh = (uint32_t) head[i];
        slope[i] = (p.max_bias > 0.0f) ? (hh < p.n_head_log2 ? powf(p.m0, (float) (hh + 1)) : powf(p.m1, (float) (2 * (hh - p.n_head_log2) + 1))) : 1.0f;
    }
    const __half *mrow[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) mrow[i] = (p.mask && live[i]) ? reinterpret_cast<const __half *>(p.mask + tok[i] * p.mask_nb_row) : nullptr;

    float o[NT][4];   // [nt][0,1]: row g, d = 8 nt + 2t, +1; [2,3]: row g + 8
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.0f, 0.0f};   // l: this lane's share of the row sum

    const char *kbase = p.k + (int64_t) hk * p.k_nb_head;
    const char *vbase = p.v + (int64_t) hk * p.v_nb_head;
    const uint32_t kv_u32 = (uint32_t) __cvta_generic_to_shared(kv_s);
    const int n_tile_tok = (int) min((int64_t) (4 * tw), p.Nq - tok0);

    // ---- the words the tile attends to at all (one pass over the tokens' word rows, 128 words at a time) ----
    if (tid == 0) uw_count = 0;
    __syncthreads();
    for (int64_t b0 = 0; b0 < p.nw; b0 += FT_THREADS) {
        const int64_t wi = b0 + tid;
        bool nz = false;
        if (wi < p.nw) {
            if (p.words) {
                unsigned long long bits = 0;
                for (int j = 0; j < n_tile_tok; ++j) bits |= p.words[(tok0 + j) * p.nw + wi];
                nz = bits != 0ull;
            } else {
                nz = true;
            }
        }
        const unsigned m = __ballot_sync(0xffffffffu, nz);
        if (lane == 0) warp_cnt[warp] = __popc(m);
        __syncthreads();
        int off = uw_count;
        for (int w = 0; w < warp; ++w) off += warp_cnt[w];
        if (nz) uw_index[off + __popc(m & ((1u << lane) - 1u))] = (unsigned short) wi;
        __syncthreads();
        if (tid == 0) uw_count += warp_cnt[0] + warp_cnt[1] + warp_cnt[2] + warp_cnt[3];
        __syncthreads();
    }
    const int n_uw = uw_count;

    // one 16-byte piece of a K or V row per copy: D / 8 pieces per row, 32 rows of K then 32 of V.  A thread's copies sit at
    // fixed places of a stage: copy n of thread tid is piece (tid + 128 n) % PIECES of row ((tid + 128 n) / PIECES) % 32.
    constexpr int PIECES = D / 8, COPIES = 2 * FT_CHUNK * PIECES / FT_THREADS, K_COPIES = COPIES / 2;
    const int st_row0 = tid / PIECES, st_piece = tid % PIECES;   // 128 / PIECES rows apart from copy to copy
    const uint32_t st_dst0 = kv_u32 + (uint32_t) (st_row0 * ROW + st_piece * 16);
    auto stage = [&](int chunk, int count, int s) {
#pragma unroll
        for (int n = 0; n < COPIES; ++n) {
            const int which = n / K_COPIES, r = st_row0 + (n % K_COPIES) * (FT_THREADS / PIECES);
            const int64_t cell = cell_list[min(chunk * FT_CHUNK + r, count - 1)];
            const char *src = (which == 0 ? kbase + cell * p.k_nb_cell : vbase + cell * p.v_nb_cell) + st_piece * 16;
            ft_cp16(st_dst0 + (uint32_t) ((s * 2 + which) * (FT_CHUNK * ROW) + (n % K_COPIES) * (FT_THREADS / PIECES) * ROW), src);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    for (int r0 = 0; r0 < n_uw; r0 += FT_RW) {
        __syncthreads();   // the previous round's lists and stages are no longer read
        // ---- the round's words, token by token; their union; the cells in ascending order ----
        for (int e = tid; e < n_tile_tok * FT_RW; e += FT_THREADS) {
            const int j = e / FT_RW, k = e - j * FT_RW;
            unsigned long long w = 0;
            if (r0 + k < n_uw) {
                const int64_t wi = uw_index[r0 + k];
                if (p.words) w = p.words[(tok0 + j) * p.nw + wi];
                else {
                    const int64_t left = p.n_kv - wi * 64;
                    w = left >= 64 ? ~0ull : ((1ull << left) - 1ull);
                }
            }
            tile_words[j][k] = w;
        }
        __syncthreads();
        if (warp == 0) {
            unsigned long long bits = 0;
            if (lane < FT_RW)
                for (int j = 0; j < n_tile_tok; ++j) bits |= tile_words[j][lane];
            const int cnt = __popcll(bits);
            int pre = cnt;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int x = __shfl_up_sync(0xffffffffu, pre, off);
                if (lane >= off) pre += x;
            }
            if (lane < FT_RW) {
                ubits[lane] = bits;
                wbase[lane] = pre - cnt;
            }
            if (lane == 31) list_count = pre;
        }
        __syncthreads();
        const int count = list_count;
        for (int e = tid; e < FT_LIST; e += FT_THREADS) {
            const int k = e >> 6, b = e & 63;
            const unsigned long long bits = ubits[k];
            if ((bits >> b) & 1ull) {
                const int at = wbase[k] + __popcll(bits & ((1ull << b) - 1ull));
                cell_list[at] = (int) uw_index[r0 + k] * 64 + b;
                cell_kb[at] = (unsigned short) e;
            }
        }
        __syncthreads();
        const int n_chunks = (count + FT_CHUNK - 1) / FT_CHUNK;
        // ---- which cells of each of this split's chunks every token attends to ----
        for (int e = tid; e < n_tile_tok * n_chunks; e += FT_THREADS) {
            const int j = e / n_chunks, c = e - j * n_chunks;
            if (c % nsplit != split) continue;
            unsigned m = 0;
            for (int x = 0; x < FT_CHUNK; ++x) {
                const int idx = c * FT_CHUNK + x;
                if (idx < count) {
                    const int kb = cell_kb[idx];
                    m |= (unsigned) ((tile_words[j][kb >> 6] >> (kb & 63)) & 1ull) << x;
                }
            }
            rmask[j][c] = m;
        }
        // this split's chunks: split, split + nsplit, ...; FT_STAGES - 1 of them are on their way while one is multiplied
        int issued = 0;
        for (int k = 0; k < FT_STAGES - 1; ++k) {
            const int c = split + k * nsplit;
            if (c < n_chunks) stage(c, count, k);
            else asm volatile("cp.async.commit_group;\n" ::: "memory");
            ++issued;
        }
        int it = 0;
        for (int ch = split; ch < n_chunks; ch += nsplit, ++it) {
            const int s = it % FT_STAGES;
            {
                const int c = split + issued * nsplit;
                if (c < n_chunks) stage(c, count, issued % FT_STAGES);
                else asm volatile("cp.async.commit_group;\n" ::: "memory");
                ++issued;
            }
            asm volatile("cp.async.wait_group %0;\n" ::"n"(FT_STAGES - 1) : "memory");
            __syncthreads();   // the stage has landed for every thread (and, first time round, the row masks are written)
            const uint8_t *Ks = kv_s + (s * 2) * (FT_CHUNK * ROW);
            const uint32_t Vs = kv_u32 + (uint32_t) ((s * 2 + 1) * (FT_CHUNK * ROW));
            // ---- S = Q K^T: four n-tiles of 8 cells (four independent accumulator chains) ----
            float sacc[4][4];
#pragma unroll
            for (int c = 0; c < 4; ++c) sacc[c][0] = sacc[c][1] = sacc[c][2] = sacc[c][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint8_t *krow = Ks + (8 * c + g) * ROW + 4 * t + 32 * ks;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(krow), b1 = *reinterpret_cast<const uint32_t *>(krow + 16);
                    mma_f16(sacc[c], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                }
            // ---- scores: element [c][2 i + e] is (row g + 8 i, cell 8 c + 2 t + e of the chunk) ----
            const int base = ch * FT_CHUNK;
            float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
            unsigned rm[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) rm[i] = live[i] ? rmask[tl[i]][ch] : 0u;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int x = 8 * c + 2 * t + e;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        float a = sacc[c][2 * i + e] * p.scale;
                        if (p.softcap != 0.0f) a = p.softcap * tanhf(a);
                        if (!((rm[i] >> x) & 1u)) a = -CUDART_INF_F;
                        else if (!binary_mask && mrow[i]) a += slope[i] * __half2float(mrow[i][cell_list[base + x]]);
                        sacc[c][2 * i + e] = a;
                        mx[i] = fmaxf(mx[i], a);
                    }
                }
            float alpha[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m_run[i], mx[i]);
                // a row that has seen no participating cell yet keeps a zero state (exp(-inf - -inf) must not be formed)
                alpha[i] = (m_new == -CUDART_INF_F) ? 1.0f : __expf(m_run[i] - m_new);
                const float m_use = (m_new == -CUDART_INF_F) ? 0.0f : m_new;
                float sum = 0.0f;
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float pr = __expf(sacc[c][2 * i + e] - m_use);
                        sacc[c][2 * i + e] = pr;
                        sum += pr;
                    }
                l_run[i] = l_run[i] * alpha[i] + sum;
                m_run[i] = m_new;
            }
            if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
                }
            }
            // P as A fragments, two k-steps of 16 cells, fp16 hi + lo
            uint32_t ph[2][4], pl[2][4];
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float x0 = sacc[c][2 * i], x1 = sacc[c][2 * i + 1];
                    const __half2 h = __floats2half2_rn(x0, x1);
                    const float2 f = __half22float2(h);
                    ph[c >> 1][2 * (c & 1) + i] = *reinterpret_cast<const uint32_t *>(&h);
                    pl[c >> 1][2 * (c & 1) + i] = pack_half2(x0 - f.x, x1 - f.y);
                }
            // ---- O += P V: V^T fragments of two n-tiles per ldmatrix ----
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    uint32_t vb[4];   // {cells 0-7, cells 8-15} of this k-step for n-tile nt, then for n-tile nt + 1
                    const int mi = lane >> 3, mr = lane & 7;
                    ft_ldmatrix_x4_trans(vb, Vs + (uint32_t) ((16 * kk + 8 * (mi & 1) + mr) * ROW + (8 * (nt + (mi >> 1))) * 2));
                    mma_f16(o[nt], ph[kk][0], ph[kk][1], ph[kk][2], ph[kk][3], vb[0], vb[1]);
                    mma_f16(o[nt], pl[kk][0], pl[kk][1], pl[kk][2], pl[kk][3], vb[0], vb[1]);
                    mma_f16(o[nt + 1], ph[kk][0], ph[kk][1], ph[kk][2], ph[kk][3], vb[2], vb[3]);
                    mma_f16(o[nt + 1], pl[kk][0], pl[kk][1], pl[kk][2], pl[kk][3], vb[2], vb[3]);
                }
            }
            __syncthreads();   // this stage may be refilled by the copy issued in the next step
        }
    }
    pdl_trigger();
    // ---- finish: every row's sum over its four lanes, then O / l (or the split's partial triple) ----
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
        if (!live[i]) continue;
        if (nsplit == 1) {
            const float inv = 1.0f / l_run[i];
            float *dst = p.dst + (tok[i] * p.H + head[i]) * D;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) *reinterpret_cast<float2 *>(dst + 8 * nt + 2 * t) = make_float2(o[nt][2 * i] * inv, o[nt][2 * i + 1] * inv);
        } else {
            float *pp = p.partial + ((tok[i] * p.H + head[i]) * nsplit + split) * (D + 2);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) *reinterpret_cast<float2 *>(pp + 8 * nt + 2 * t) = make_float2(o[nt][2 * i], o[nt][2 * i + 1]);
            if (t == 0) {
                pp[D] = m_run[i];
                pp[D + 1] = l_run[i];
            }
        }
    }
}

}  // namespace b200
