// Test driver for the ggml-b200 plug-in, built against a checkout of the reference (test infrastructure).
//
//   harness ops                      single-op graphs run node by node on the reference CPU backend and on the
//                                    B200 backend with lm_ggml_backend_compare_graph_backend
//                                    (cactus/ggml-backend.cpp:1821-1857)
//   harness model [options]          writes a synthetic llama GGUF with the reference's gguf writer, loads it
//                                    twice through llama.h (CPU only / all layers on the B200 device) and feeds
//                                    both contexts the same ragged multi-sequence batches
//
// The reference's runtime (llama-context, llama-graph, llama-kv-cache, the scheduler) is the unchanged caller;
// the plug-in is registered with lm_ggml_backend_register before the model is loaded.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "ggml-backend-impl.h"
#include "ggml-backend.h"
#include "ggml-cpu.h"
#include "ggml.h"
#include "gguf.h"
#include "llama.h"

#include "../../cactus_b200/backend/ggml-b200.h"

static double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

// ------------------------------------------------------------------------------------------------------
// ops
// ------------------------------------------------------------------------------------------------------
struct cmp_state {
    double worst[LM_GGML_OP_COUNT];
    int count[LM_GGML_OP_COUNT];
    bool nan_seen;
};

static std::vector<float> to_f32(lm_ggml_tensor * t) {
    const size_t n = lm_ggml_nelements(t);
    std::vector<uint8_t> raw(lm_ggml_nbytes(t));
    lm_ggml_backend_tensor_get(t, raw.data(), 0, raw.size());
    std::vector<float> out(n);
    if (t->type == LM_GGML_TYPE_F32) memcpy(out.data(), raw.data(), n * 4);
    else if (t->type == LM_GGML_TYPE_F16) lm_ggml_fp16_to_fp32_row((const lm_ggml_fp16_t *) raw.data(), out.data(), n);
    else out.assign(n, 0.0f);
    return out;
}

static bool cmp_cb(int, lm_ggml_tensor * t1, lm_ggml_tensor * t2, void * ud) {
    cmp_state * st = (cmp_state *) ud;
    if (!lm_ggml_is_contiguous(t1) || (t1->type != LM_GGML_TYPE_F32 && t1->type != LM_GGML_TYPE_F16)) return true;
    std::vector<float> a = to_f32(t1), b = to_f32(t2);
    double maxref = 0, maxdiff = 0;
    for (size_t i = 0; i < a.size(); ++i) {
        if (std::isnan(a[i]) && std::isnan(b[i])) continue;   // fully masked padding rows are NaN in the reference too
        if (std::isnan(a[i]) != std::isnan(b[i])) st->nan_seen = true;
        maxref = std::max(maxref, (double) std::fabs(a[i]));
        maxdiff = std::max(maxdiff, (double) std::fabs(a[i] - b[i]));
    }
    const double rel = maxdiff / (maxref + 1e-30);
    if (getenv("HARNESS_VERBOSE")) fprintf(stderr, "  node %-24s %-16s rel %.3g (max |ref| %.3g)\n", t1->name, lm_ggml_op_name(t1->op), rel, maxref);
    st->worst[t1->op] = std::max(st->worst[t1->op], rel);
    st->count[t1->op]++;
    return true;
}

static void fill_normal(std::vector<float> & v, std::mt19937 & rng, float std_) {
    std::normal_distribution<float> d(0.0f, std_);
    for (auto & x : v) x = d(rng);
}

static lm_ggml_tensor * new_weight(lm_ggml_context * ctx, lm_ggml_type type, int64_t K, int64_t M) { return lm_ggml_new_tensor_2d(ctx, type, K, M); }

static void set_quantized(lm_ggml_tensor * t, std::mt19937 & rng, float std_) {
    const int64_t K = t->ne[0], M = t->ne[1];
    std::vector<float> w((size_t) K * M);
    fill_normal(w, rng, std_);
    std::vector<uint8_t> q(lm_ggml_nbytes(t));
    lm_ggml_quantize_chunk(t->type, w.data(), q.data(), 0, M, K, nullptr);
    lm_ggml_backend_tensor_set(t, q.data(), 0, q.size());
}

static void set_f32(lm_ggml_tensor * t, std::mt19937 & rng, float std_, float mean = 0.0f) {
    std::vector<float> v(lm_ggml_nelements(t));
    fill_normal(v, rng, std_);
    for (auto & x : v) x += mean;
    lm_ggml_backend_tensor_set(t, v.data(), 0, v.size() * 4);
}

// One llama layer worth of ops (the node list the plug-in receives, cactus/llama-model.cpp:4517-4671) on small shapes.
// `inplace`: the norm, its weight multiply, SILU, the gate x up product and the last residual add overwrite their first
// operand (the _inplace forms of the graph builder), so the row kernels and the plug-in's peepholes see aliased pointers.
static int run_ops(int n_tokens, lm_ggml_type wtype, bool inplace = false) {
    lm_ggml_backend_t cpu = lm_ggml_backend_cpu_init();
    lm_ggml_backend_t gpu = lm_ggml_backend_b200_init(0);
    if (!gpu) { printf("{\"error\": \"no B200 backend\"}\n"); return 2; }
    const int64_t d = 512, H = 8, Hkv = 2, D = 64, ff = 1024, n_kv = 256, T = n_tokens, V = 320;
    lm_ggml_init_params ip = { 64 * 1024 * 1024, nullptr, true };
    lm_ggml_context * ctx = lm_ggml_init(ip);
    std::mt19937 rng(7);

    lm_ggml_tensor * x = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_F32, d, T);
    lm_ggml_tensor * wn = lm_ggml_new_tensor_1d(ctx, LM_GGML_TYPE_F32, d);
    lm_ggml_tensor * wq = new_weight(ctx, wtype, d, H * D), * wk = new_weight(ctx, wtype, d, Hkv * D), * wv = new_weight(ctx, wtype, d, Hkv * D);
    lm_ggml_tensor * wo = new_weight(ctx, wtype, H * D, d), * wg = new_weight(ctx, wtype, d, ff), * wu = new_weight(ctx, wtype, d, ff), * wd = new_weight(ctx, wtype, ff, d);
    lm_ggml_tensor * emb = new_weight(ctx, wtype, d, V);
    lm_ggml_tensor * ids = lm_ggml_new_tensor_1d(ctx, LM_GGML_TYPE_I32, T);
    lm_ggml_tensor * pos = lm_ggml_new_tensor_1d(ctx, LM_GGML_TYPE_I32, T);
    lm_ggml_tensor * kc = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_F16, Hkv * D, n_kv), * vc = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_F16, Hkv * D, n_kv);
    const int64_t Tp = (T + 63) / 64 * 64;
    lm_ggml_tensor * mask32 = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_F32, n_kv, Tp);
    for (lm_ggml_tensor * t : {x, wn, wq, wk, wv, wo, wg, wu, wd, emb, ids, pos, kc, vc, mask32}) lm_ggml_set_input(t);

    // graph
    lm_ggml_tensor * e = lm_ggml_get_rows(ctx, emb, ids);
    auto norm = [&](lm_ggml_tensor * a, bool fresh) { return inplace && fresh ? lm_ggml_rms_norm_inplace(ctx, a, 1e-5f) : lm_ggml_rms_norm(ctx, a, 1e-5f); };
    auto mul = [&](lm_ggml_tensor * a, lm_ggml_tensor * b) { return inplace ? lm_ggml_mul_inplace(ctx, a, b) : lm_ggml_mul(ctx, a, b); };
    lm_ggml_tensor * h = mul(norm(lm_ggml_add(ctx, x, e), true), wn);
    lm_ggml_tensor * q = lm_ggml_rope_ext(ctx, lm_ggml_reshape_3d(ctx, lm_ggml_mul_mat(ctx, wq, h), D, H, T), pos, nullptr, D, 0, 0, 500000.0f, 1.0f, 0.0f, 1.0f, 0.0f, 0.0f);
    lm_ggml_tensor * k = lm_ggml_rope_ext(ctx, lm_ggml_reshape_3d(ctx, lm_ggml_mul_mat(ctx, wk, h), D, Hkv, T), pos, nullptr, D, 0, 0, 500000.0f, 1.0f, 0.0f, 1.0f, 0.0f, 0.0f);
    lm_ggml_tensor * v = lm_ggml_mul_mat(ctx, wv, h);
    const int64_t head = 100;  // the ubatch occupies cells [head, head + T)
    lm_ggml_tensor * k_dst = lm_ggml_view_1d(ctx, kc, T * Hkv * D, head * lm_ggml_row_size(kc->type, Hkv * D));
    lm_ggml_tensor * v_dst = lm_ggml_view_1d(ctx, vc, T * Hkv * D, head * lm_ggml_row_size(vc->type, Hkv * D));
    lm_ggml_tensor * k_cpy = lm_ggml_cpy(ctx, k, k_dst), * v_cpy = lm_ggml_cpy(ctx, v, v_dst);
    lm_ggml_tensor * kq_mask = lm_ggml_cast(ctx, mask32, LM_GGML_TYPE_F16);
    lm_ggml_tensor * qp = lm_ggml_permute(ctx, q, 0, 2, 1, 3);
    lm_ggml_tensor * kp = lm_ggml_permute(ctx, lm_ggml_view_3d(ctx, kc, D, Hkv, n_kv, lm_ggml_row_size(kc->type, D), lm_ggml_row_size(kc->type, Hkv * D), 0), 0, 2, 1, 3);
    lm_ggml_tensor * vp = lm_ggml_permute(ctx, lm_ggml_view_3d(ctx, vc, D, Hkv, n_kv, lm_ggml_row_size(vc->type, D), lm_ggml_row_size(vc->type, Hkv * D), 0), 0, 2, 1, 3);
    lm_ggml_tensor * att = lm_ggml_flash_attn_ext(ctx, qp, kp, vp, kq_mask, 1.0f / sqrtf((float) D), 0.0f, 0.0f);
    lm_ggml_flash_attn_ext_set_prec(att, LM_GGML_PREC_F32);
    lm_ggml_tensor * ao = lm_ggml_mul_mat(ctx, wo, lm_ggml_reshape_2d(ctx, att, H * D, T));
    lm_ggml_tensor * r1 = lm_ggml_add(ctx, ao, x);
    lm_ggml_tensor * h2 = mul(norm(r1, false), wn);   // r1 is read again by the last add: its norm gets a buffer of its own
    lm_ggml_tensor * gate = inplace ? lm_ggml_silu_inplace(ctx, lm_ggml_mul_mat(ctx, wg, h2)) : lm_ggml_silu(ctx, lm_ggml_mul_mat(ctx, wg, h2));
    lm_ggml_tensor * par = mul(gate, lm_ggml_mul_mat(ctx, wu, h2));
    lm_ggml_tensor * out = inplace ? lm_ggml_add_inplace(ctx, lm_ggml_mul_mat(ctx, wd, par), r1) : lm_ggml_add(ctx, lm_ggml_mul_mat(ctx, wd, par), r1);
    lm_ggml_set_output(out);

    lm_ggml_cgraph * gf = lm_ggml_new_graph(ctx);
    lm_ggml_build_forward_expand(gf, k_cpy);
    lm_ggml_build_forward_expand(gf, v_cpy);
    lm_ggml_build_forward_expand(gf, out);

    lm_ggml_backend_buffer_t buf = lm_ggml_backend_alloc_ctx_tensors(ctx, cpu);
    if (!buf) { printf("{\"error\": \"alloc failed\"}\n"); return 2; }

    set_f32(x, rng, 1.0f);
    set_f32(wn, rng, 0.1f, 1.0f);
    for (lm_ggml_tensor * t : {wq, wk, wv, wg, wu}) set_quantized(t, rng, 1.0f / sqrtf((float) d));
    set_quantized(wo, rng, 1.0f / sqrtf((float) (H * D)));
    set_quantized(wd, rng, 1.0f / sqrtf((float) ff));
    set_quantized(emb, rng, 1.0f);
    std::vector<int32_t> idv(T), posv(T), seqv(T);
    for (int i = 0; i < T; ++i) { idv[i] = (int32_t) (rng() % V); seqv[i] = i % 3; posv[i] = 30 + i / 3; }
    lm_ggml_backend_tensor_set(ids, idv.data(), 0, T * 4);
    lm_ggml_backend_tensor_set(pos, posv.data(), 0, T * 4);
    // cache: cells [0, head) hold three earlier sequences round-robin with positions below the new tokens
    std::vector<lm_ggml_fp16_t> kv((size_t) Hkv * D * n_kv);
    std::vector<float> tmp(kv.size());
    fill_normal(tmp, rng, 1.0f);
    lm_ggml_fp32_to_fp16_row(tmp.data(), kv.data(), tmp.size());
    lm_ggml_backend_tensor_set(kc, kv.data(), 0, kv.size() * 2);
    fill_normal(tmp, rng, 1.0f);
    lm_ggml_fp32_to_fp16_row(tmp.data(), kv.data(), tmp.size());
    lm_ggml_backend_tensor_set(vc, kv.data(), 0, kv.size() * 2);
    std::vector<float> m((size_t) n_kv * Tp, -INFINITY);
    for (int j = 0; j < T; ++j)
        for (int i = 0; i < n_kv; ++i) {
            int cseq, cpos;
            if (i < 90) { cseq = i % 3; cpos = i / 3; }
            else if (i >= head && i < head + T) { cseq = seqv[i - head]; cpos = posv[i - head]; }
            else continue;
            if (cseq == seqv[j] && cpos <= posv[j]) m[(size_t) j * n_kv + i] = 0.0f;
        }
    lm_ggml_backend_tensor_set(mask32, m.data(), 0, m.size() * 4);

    cmp_state st;
    memset(&st, 0, sizeof(st));
    const bool ok = lm_ggml_backend_compare_graph_backend(cpu, gpu, gf, cmp_cb, &st);
    lm_ggml_b200_stats bs;
    lm_ggml_backend_b200_get_stats(gpu, &bs);
    printf("{\"case\": \"%s\", \"tokens\": %d, \"wtype\": \"%s\", \"compared\": %s, \"nan_mismatch\": %s", inplace ? "layer in place" : "layer", n_tokens, lm_ggml_type_name(wtype),
           ok ? "true" : "false", st.nan_seen ? "true" : "false");
    for (int op = 0; op < LM_GGML_OP_COUNT; ++op)
        if (st.count[op]) printf(", \"%s\": %.3g", lm_ggml_op_name((lm_ggml_op) op), st.worst[op]);
    printf(", \"b200_nodes\": %llu, \"b200_mul_mat\": %llu, \"b200_flash_attn\": %llu}\n", (unsigned long long) bs.nodes,
           (unsigned long long) bs.mul_mat, (unsigned long long) bs.flash_attn);
    int rc = ok && !st.nan_seen ? 0 : 1;
    if (st.worst[LM_GGML_OP_MUL_MAT] > 3e-2 || st.worst[LM_GGML_OP_FLASH_ATTN_EXT] > 6e-3 || st.worst[LM_GGML_OP_ROPE] > 1e-4 ||
        st.worst[LM_GGML_OP_MUL] > 3e-2 || st.worst[LM_GGML_OP_ADD] > 3e-2 || st.worst[LM_GGML_OP_CPY] > 1e-3 || st.worst[LM_GGML_OP_GET_ROWS] > 0)
        rc = 1;
    lm_ggml_backend_buffer_free(buf);
    lm_ggml_free(ctx);
    lm_ggml_backend_free(gpu);
    lm_ggml_backend_free(cpu);
    return rc;
}

// The two KV-cache maintenance graphs of the reference on single nodes: the K-shift (ROPE in place on the cached f16
// keys with a per-cell shift, llama_kv_cache_unified::build_graph_shift) and a defragmentation move (CPY f16 -> f16 of a
// run of cells, build_graph_defrag), CPU backend against the B200 backend.
static int run_kv_ops() {
    lm_ggml_backend_t cpu = lm_ggml_backend_cpu_init();
    lm_ggml_backend_t gpu = lm_ggml_backend_b200_init(0);
    if (!gpu) { printf("{\"error\": \"no B200 backend\"}\n"); return 2; }
    const int64_t Hkv = 2, D = 64, n_kv = 256;
    lm_ggml_init_params ip = { 16 * 1024 * 1024, nullptr, true };
    lm_ggml_context * ctx = lm_ggml_init(ip);
    std::mt19937 rng(11);
    lm_ggml_tensor * kc = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_F16, Hkv * D, n_kv);
    lm_ggml_tensor * vc = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_F16, Hkv * D, n_kv);
    lm_ggml_tensor * shift = lm_ggml_new_tensor_1d(ctx, LM_GGML_TYPE_I32, n_kv);
    for (lm_ggml_tensor * t : {kc, vc, shift}) lm_ggml_set_input(t);
    lm_ggml_tensor * k3 = lm_ggml_view_3d(ctx, kc, D, Hkv, n_kv, lm_ggml_row_size(kc->type, D), lm_ggml_row_size(kc->type, Hkv * D), 0);
    lm_ggml_tensor * shifted = lm_ggml_rope_ext_inplace(ctx, k3, shift, nullptr, D, 0, 0, 500000.0f, 1.0f, 0.0f, 1.0f, 0.0f, 0.0f);
    const int64_t from = 200, to = 40, nm = 17;   // cells [200, 217) move to [40, 57)
    lm_ggml_tensor * src = lm_ggml_view_2d(ctx, vc, Hkv * D, nm, lm_ggml_row_size(vc->type, Hkv * D), lm_ggml_row_size(vc->type, Hkv * D * from));
    lm_ggml_tensor * dst = lm_ggml_view_2d(ctx, vc, Hkv * D, nm, lm_ggml_row_size(vc->type, Hkv * D), lm_ggml_row_size(vc->type, Hkv * D * to));
    lm_ggml_tensor * moved = lm_ggml_cpy(ctx, src, dst);
    lm_ggml_cgraph * gf = lm_ggml_new_graph(ctx);
    lm_ggml_build_forward_expand(gf, shifted);
    lm_ggml_build_forward_expand(gf, moved);
    lm_ggml_backend_buffer_t buf = lm_ggml_backend_alloc_ctx_tensors(ctx, cpu);
    if (!buf) { printf("{\"error\": \"alloc failed\"}\n"); return 2; }
    std::vector<float> tmp((size_t) Hkv * D * n_kv);
    std::vector<lm_ggml_fp16_t> kv(tmp.size());
    for (lm_ggml_tensor * t : {kc, vc}) {
        fill_normal(tmp, rng, 1.0f);
        lm_ggml_fp32_to_fp16_row(tmp.data(), kv.data(), tmp.size());
        lm_ggml_backend_tensor_set(t, kv.data(), 0, kv.size() * 2);
    }
    std::vector<int32_t> sh(n_kv);
    for (int i = 0; i < n_kv; ++i) sh[i] = (i % 4 == 0) ? 0 : (int32_t) (rng() % 4096) - 2048;
    lm_ggml_backend_tensor_set(shift, sh.data(), 0, sh.size() * 4);
    cmp_state st;
    memset(&st, 0, sizeof(st));
    const bool ok = lm_ggml_backend_compare_graph_backend(cpu, gpu, gf, cmp_cb, &st);
    printf("{\"case\": \"kv maintenance\", \"compared\": %s, \"nan_mismatch\": %s, \"ROPE\": %.3g, \"CPY\": %.3g, \"rope_nodes\": %d, \"cpy_nodes\": %d}\n",
           ok ? "true" : "false", st.nan_seen ? "true" : "false", st.worst[LM_GGML_OP_ROPE], st.worst[LM_GGML_OP_CPY], st.count[LM_GGML_OP_ROPE],
           st.count[LM_GGML_OP_CPY]);
    // f16 results: at most one f16 step apart where the f32 rotation differs in its last bits; copies are exact
    int rc = (ok && !st.nan_seen && st.count[LM_GGML_OP_ROPE] == 1 && st.count[LM_GGML_OP_CPY] == 1 && st.worst[LM_GGML_OP_ROPE] < 2e-3 &&
              st.worst[LM_GGML_OP_CPY] == 0.0) ? 0 : 1;
    lm_ggml_backend_buffer_free(buf);
    lm_ggml_free(ctx);
    lm_ggml_backend_free(gpu);
    lm_ggml_backend_free(cpu);
    return rc;
}

// ------------------------------------------------------------------------------------------------------
// model
// ------------------------------------------------------------------------------------------------------
struct model_cfg {
    int n_layer = 2, d = 512, n_head = 8, n_kv = 2, ff = 1024, vocab = 1000, n_ctx = 1024;
    lm_ggml_type layer_type = LM_GGML_TYPE_Q4_0, head_type = LM_GGML_TYPE_Q8_0;
};

// Synthetic llama GGUF: keys as cactus/llama-arch.cpp:80-177 names them, tokenizer "no_vocab"
// (cactus/llama-vocab.cpp:1382-1399), tensors of cactus/llama-model.cpp:1723-1771.
static bool write_gguf(const model_cfg & c, const std::string & path, uint32_t seed) {
    lm_gguf_context * g = lm_gguf_init_empty();
    lm_gguf_set_val_str(g, "general.architecture", "llama");
    lm_gguf_set_val_str(g, "general.name", "synthetic");
    lm_gguf_set_val_u32(g, "llama.context_length", 131072);
    lm_gguf_set_val_u32(g, "llama.embedding_length", c.d);
    lm_gguf_set_val_u32(g, "llama.block_count", c.n_layer);
    lm_gguf_set_val_u32(g, "llama.feed_forward_length", c.ff);
    lm_gguf_set_val_u32(g, "llama.attention.head_count", c.n_head);
    lm_gguf_set_val_u32(g, "llama.attention.head_count_kv", c.n_kv);
    lm_gguf_set_val_f32(g, "llama.attention.layer_norm_rms_epsilon", 1e-5f);
    lm_gguf_set_val_f32(g, "llama.rope.freq_base", 500000.0f);
    lm_gguf_set_val_u32(g, "llama.rope.dimension_count", c.d / c.n_head);
    lm_gguf_set_val_u32(g, "llama.vocab_size", c.vocab);
    lm_gguf_set_val_str(g, "tokenizer.ggml.model", "no_vocab");

    size_t total = 0;
    auto tsize = [&](lm_ggml_type t, int64_t k, int64_t m) { return lm_ggml_row_size(t, k) * m; };
    const int D = c.d / c.n_head;
    total += 2 * tsize(c.head_type, c.d, c.vocab) + c.d * 4;
    total += (size_t) c.n_layer * (2 * tsize(c.layer_type, c.d, c.d) + 2 * tsize(c.layer_type, c.d, (int64_t) c.n_kv * D) + 3 * tsize(c.layer_type, c.d, c.ff) + 2 * c.d * 4);
    lm_ggml_init_params ip = { total + (size_t) (16 + 12 * c.n_layer) * lm_ggml_tensor_overhead() + (1 << 20), nullptr, false };
    lm_ggml_context * ctx = lm_ggml_init(ip);
    if (!ctx) return false;
    std::mt19937 rng(seed);
    std::vector<float> tmp;
    auto add_q = [&](const std::string & name, lm_ggml_type t, int64_t k, int64_t m, float std_) {
        lm_ggml_tensor * w = lm_ggml_new_tensor_2d(ctx, t, k, m);
        lm_ggml_set_name(w, name.c_str());
        const int64_t chunk = 1024;
        for (int64_t r0 = 0; r0 < m; r0 += chunk) {
            const int64_t rows = std::min(chunk, m - r0);
            tmp.resize((size_t) rows * k);
            if (m * k <= (1 << 24)) {
                fill_normal(tmp, rng, std_);
            } else {   // big (benchmark-sized) tensors: rows cut out of one table of normal values at random offsets, a hundred times faster
                static std::vector<float> table;
                if (table.empty()) { table.resize(1 << 22); fill_normal(table, rng, 1.0f); }
                for (int64_t r = 0; r < rows; ++r) {
                    const size_t off = rng() % (table.size() - (size_t) k);
                    for (int64_t i = 0; i < k; ++i) tmp[(size_t) r * k + i] = table[off + i] * std_;
                }
            }
            // (the chunk API offsets both source and destination by `start`: quantise chunk-local rows at offset 0)
            lm_ggml_quantize_chunk(t, tmp.data(), (char *) w->data + r0 * lm_ggml_row_size(t, k), 0, rows, k, nullptr);
        }
        lm_gguf_add_tensor(g, w);
    };
    auto add_norm = [&](const std::string & name) {
        lm_ggml_tensor * w = lm_ggml_new_tensor_1d(ctx, LM_GGML_TYPE_F32, c.d);
        lm_ggml_set_name(w, name.c_str());
        std::normal_distribution<float> dist(1.0f, 0.02f);
        for (int i = 0; i < c.d; ++i) ((float *) w->data)[i] = dist(rng);
        lm_gguf_add_tensor(g, w);
    };
    // embeddings ~ N(0,1) so the first layer sees unit-scale activations; projections ~ N(0, 1/sqrt(fan_in)) keep the
    // residual stream at unit scale, which a well-trained model has and the 0.02 of the benchmark weights would not
    add_q("token_embd.weight", c.head_type, c.d, c.vocab, 1.0f);
    add_norm("output_norm.weight");
    add_q("output.weight", c.head_type, c.d, c.vocab, 1.0f / sqrtf((float) c.d));
    for (int il = 0; il < c.n_layer; ++il) {
        const std::string p = "blk." + std::to_string(il) + ".";
        add_norm(p + "attn_norm.weight");
        add_q(p + "attn_q.weight", c.layer_type, c.d, c.d, 1.0f / sqrtf((float) c.d));
        add_q(p + "attn_k.weight", c.layer_type, c.d, (int64_t) c.n_kv * D, 1.0f / sqrtf((float) c.d));
        add_q(p + "attn_v.weight", c.layer_type, c.d, (int64_t) c.n_kv * D, 1.0f / sqrtf((float) c.d));
        add_q(p + "attn_output.weight", c.layer_type, c.d, c.d, 0.5f / sqrtf((float) c.d));
        add_norm(p + "ffn_norm.weight");
        add_q(p + "ffn_gate.weight", c.layer_type, c.d, c.ff, 1.0f / sqrtf((float) c.d));
        add_q(p + "ffn_up.weight", c.layer_type, c.d, c.ff, 1.0f / sqrtf((float) c.d));
        add_q(p + "ffn_down.weight", c.layer_type, c.ff, c.d, 0.5f / sqrtf((float) c.ff));
    }
    const bool ok = lm_gguf_write_to_file(g, path.c_str(), false);
    lm_gguf_free(g);
    lm_ggml_free(ctx);
    return ok;
}

struct runner {
    llama_model * model = nullptr;
    llama_context * ctx = nullptr;
    int vocab = 0;
};

// split_row_gpus > 0: LLAMA_SPLIT_MODE_ROW over that many B200 devices (the loader then asks the plug-in for its split
// buffer type by name, cactus/llama-model.cpp:333-356, and spreads the layers over the same devices)
static int split_row_gpus = 0;

static bool open_runner(runner & r, const std::string & path, bool gpu, const model_cfg & c, int n_seq, int n_threads) {
    llama_model_params mp = llama_model_default_params();
    static lm_ggml_backend_dev_t none[1] = { nullptr };
    static lm_ggml_backend_dev_t devs[LM_GGML_B200_MAX_DEVICES + 1] = { nullptr };
    static llama_model_tensor_buft_override ov[2];
    if (gpu) {
        devs[0] = lm_ggml_backend_reg_dev_get(lm_ggml_backend_b200_reg(), 0);
        devs[1] = nullptr;
        mp.devices = devs;
        mp.n_gpu_layers = 999;
        mp.split_mode = LLAMA_SPLIT_MODE_NONE;
        mp.main_gpu = 0;
        if (split_row_gpus > 0) {
            const int have = (int) lm_ggml_backend_reg_dev_count(lm_ggml_backend_b200_reg());
            const int n = std::min(split_row_gpus, have);
            for (int i = 0; i < n; ++i) devs[i] = lm_ggml_backend_reg_dev_get(lm_ggml_backend_b200_reg(), i);
            devs[n] = nullptr;
            mp.split_mode = LLAMA_SPLIT_MODE_ROW;
        }
        // the input layer is pinned to the CPU by the loader (cactus/llama-model.cpp:1517-1519); move the embedding table too
        ov[0] = { "token_embd\\.weight", lm_ggml_backend_b200_buffer_type(0) };
        ov[1] = { nullptr, nullptr };
        mp.tensor_buft_overrides = ov;
    } else {
        mp.devices = none;
        mp.n_gpu_layers = 0;
    }
    r.model = llama_model_load_from_file(path.c_str(), mp);
    if (!r.model) return false;
    llama_context_params cp = llama_context_default_params();
    cp.n_ctx = c.n_ctx;
    cp.n_batch = 2048;
    cp.n_ubatch = 512;
    cp.n_seq_max = n_seq;
    cp.n_threads = cp.n_threads_batch = n_threads;
    cp.flash_attn = true;
    cp.no_perf = true;
    r.ctx = llama_init_from_model(r.model, cp);
    r.vocab = c.vocab;
    return r.ctx != nullptr;
}

// One logical batch, submitted in pieces of at most n_batch tokens (llama_decode asserts n_tokens <= n_batch,
// cactus/llama-context.cpp:895), the way a serving loop feeds long prompts; the logits of the wanted tokens are collected in order.
static int decode_batch(runner & r, const std::vector<int32_t> & tok, const std::vector<int32_t> & pos, const std::vector<int32_t> & seq,
                        const std::vector<int8_t> & want, std::vector<float> & logits_out, bool collect = true) {
    const int n_all = (int) tok.size(), n_batch = 2048;
    logits_out.clear();
    for (int i0 = 0; i0 < n_all; i0 += n_batch) {
        const int n = std::min(n_batch, n_all - i0);
        llama_batch b = llama_batch_init(n, 0, 1);
        b.n_tokens = n;
        for (int i = 0; i < n; ++i) {
            b.token[i] = tok[i0 + i];
            b.pos[i] = pos[i0 + i];
            b.n_seq_id[i] = 1;
            b.seq_id[i][0] = seq[i0 + i];
            b.logits[i] = want[i0 + i];
        }
        const int rc = llama_decode(r.ctx, b);
        if (rc == 0 && !collect) {
            (void) llama_get_logits_ith(r.ctx, 0);   // waits for the step (the logits are in the context's pinned buffer)
        } else if (rc == 0) {
            for (int i = 0; i < n; ++i)
                if (want[i0 + i]) {
                    const float * l = llama_get_logits_ith(r.ctx, i);
                    logits_out.insert(logits_out.end(), l, l + r.vocab);
                }
        }
        llama_batch_free(b);
        if (rc != 0) return rc;
    }
    return 0;
}

extern bool g_b200_device_mask;
extern unsigned long long g_b200_device_mask_calls;
extern bool g_b200_mask_verify;
extern unsigned long long g_b200_mask_values, g_b200_mask_mismatches;

static int run_model(int argc, char ** argv) {
    model_cfg c;
    int n_seq = 3, n_decode = 4, max_prompt = 40, n_threads = 8, bench_steps = 0;
    std::string path = "/tmp/b200_synth.gguf";
    bool skip_cpu = false, cpu_only = false;
    for (int i = 2; i < argc; ++i) {
        std::string a = argv[i];
        auto val = [&]() { return atoi(argv[++i]); };
        if (a == "--layers") c.n_layer = val();
        else if (a == "--d") c.d = val();
        else if (a == "--heads") c.n_head = val();
        else if (a == "--kv") c.n_kv = val();
        else if (a == "--ff") c.ff = val();
        else if (a == "--vocab") c.vocab = val();
        else if (a == "--ctx") c.n_ctx = val();
        else if (a == "--seqs") n_seq = val();
        else if (a == "--decode") n_decode = val();
        else if (a == "--max-prompt") max_prompt = val();
        else if (a == "--threads") n_threads = val();
        else if (a == "--bench-steps") bench_steps = val();
        else if (a == "--head-q4") c.head_type = LM_GGML_TYPE_Q4_0;
        else if (a == "--skip-cpu") skip_cpu = true;
        else if (a == "--cpu-only") cpu_only = true;   // checks the GGUF writer and the driver without a GPU
        else if (a == "--path") path = argv[++i];
        else if (a == "--split-row") split_row_gpus = val();
        else if (a == "--device-mask") g_b200_device_mask = true;   // device_mask.cpp: the KQ mask is synthesised on the device
        else if (a == "--verify-mask") g_b200_mask_verify = true;   // ... and compared bit for bit with the reference's host mask
    }
    llama_log_set([](lm_ggml_log_level level, const char * text, void *) { if (level >= LM_GGML_LOG_LEVEL_ERROR) fputs(text, stderr); }, nullptr);
    if (!cpu_only) lm_ggml_backend_register(lm_ggml_backend_b200_reg());
    llama_backend_init();
    if (!write_gguf(c, path, 1234)) { printf("{\"error\": \"gguf write failed\"}\n"); return 2; }

    runner cpu, gpu;
    if (!skip_cpu && !open_runner(cpu, path, false, c, n_seq, n_threads)) { printf("{\"error\": \"cpu load failed\"}\n"); return 2; }
    if (!cpu_only && !open_runner(gpu, path, true, c, n_seq, n_threads)) { printf("{\"error\": \"b200 load failed\"}\n"); return 2; }

    std::mt19937 rng(99);
    std::vector<int> len(n_seq);
    for (auto & l : len) l = 1 + (int) (rng() % max_prompt);
    std::vector<int32_t> tok, pos, seq;
    std::vector<int8_t> want;
    for (int s = 0; s < n_seq; ++s)
        for (int p = 0; p < len[s]; ++p) {
            tok.push_back((int32_t) (rng() % c.vocab));
            pos.push_back(p);
            seq.push_back(s);
            want.push_back(p == len[s] - 1);
        }
    double worst = 0, sum_rows = 0, good_rows = 0;
    int agree = 0, total = 0;
    std::vector<float> lc, lg;
    std::vector<int32_t> cur(n_seq);
    auto compare = [&](int rows) {
        for (int r = 0; r < rows; ++r) {
            const float * a = lc.data() + (size_t) r * c.vocab, * b = lg.data() + (size_t) r * c.vocab;
            double mr = 0, md = 0;
            int am = 0, bm = 0;
            for (int i = 0; i < c.vocab; ++i) {
                mr = std::max(mr, (double) std::fabs(a[i]));
                md = std::max(md, (double) std::fabs(a[i] - b[i]));
                if (a[i] > a[am]) am = i;
                if (b[i] > b[bm]) bm = i;
            }
            const double rel = md / (mr + 1e-30);
            worst = std::max(worst, rel);
            sum_rows += 1;
            good_rows += rel < 1e-3;
            agree += am == bm;
            total += 1;
            cur[r] = am;   // both contexts continue with the reference's greedy token
        }
    };
    int rc_c = skip_cpu ? 0 : decode_batch(cpu, tok, pos, seq, want, lc);
    int rc_g = cpu_only ? 0 : decode_batch(gpu, tok, pos, seq, want, lg);
    if (cpu_only) lg = lc;
    if (rc_c || rc_g) { printf("{\"error\": \"decode failed\", \"cpu\": %d, \"b200\": %d}\n", rc_c, rc_g); return 2; }
    if (skip_cpu) { lc = lg; }
    compare(n_seq);
    for (int step = 0; step < n_decode; ++step) {
        tok.assign(cur.begin(), cur.end());
        pos.resize(n_seq); seq.resize(n_seq); want.assign(n_seq, 1);
        for (int s = 0; s < n_seq; ++s) { pos[s] = len[s] + step; seq[s] = s; }
        rc_c = skip_cpu ? 0 : decode_batch(cpu, tok, pos, seq, want, lc);
        rc_g = cpu_only ? 0 : decode_batch(gpu, tok, pos, seq, want, lg);
        if (cpu_only) lg = lc;
        if (rc_c || rc_g) { printf("{\"error\": \"decode failed\", \"cpu\": %d, \"b200\": %d}\n", rc_c, rc_g); return 2; }
        if (skip_cpu) { lc = lg; }
        compare(n_seq);
    }
    // optional timing of further decode steps on the B200 context
    double step_ms = 0, bench_device_ms = 0;
    if (bench_steps > 0) {
        auto totals = (lm_ggml_b200_timing_totals_t) lm_ggml_backend_reg_get_proc_address(lm_ggml_backend_b200_reg(), "lm_ggml_backend_b200_timing_totals");
        double ms0 = 0, ms1 = 0;
        uint64_t g0 = 0, g1 = 0;
        if (totals) totals(&ms0, &g0);
        for (int s = 0; s < n_seq; ++s) seq[s] = s;
        const double t0 = now_s();
        for (int step = 0; step < bench_steps; ++step) {
            for (int s = 0; s < n_seq; ++s) pos[s] = len[s] + n_decode + step;
            decode_batch(gpu, tok, pos, seq, want, lg, false);
        }
        step_ms = (now_s() - t0) * 1e3 / bench_steps;
        if (totals) totals(&ms1, &g1);
        if (g1 > g0) bench_device_ms = (ms1 - ms0) / (double) (g1 - g0);   // only with B200_TIMING=1
    }
    uint64_t n_rope_store = 0, n_add_norm = 0, n_recorded = 0, n_replayed = 0;
    if (!cpu_only) {
        auto counts = (lm_ggml_b200_fused_group_counts_t) lm_ggml_backend_reg_get_proc_address(lm_ggml_backend_b200_reg(), "lm_ggml_backend_b200_fused_group_counts");
        if (counts) counts(&n_rope_store, &n_add_norm);
        auto gc = (lm_ggml_b200_graph_counts_t) lm_ggml_backend_reg_get_proc_address(lm_ggml_backend_b200_reg(), "lm_ggml_backend_b200_graph_counts");
        if (gc) gc(&n_recorded, &n_replayed);
    }
    printf("{\"case\": \"model\", \"layers\": %d, \"d\": %d, \"seqs\": %d, \"decode_steps\": %d, \"rows\": %d, \"worst_rel\": %.3g, "
           "\"rows_within_1e-3\": %.3f, \"greedy_agree\": %.3f, \"b200_step_ms\": %.3f, \"split_mul_mats\": %llu, \"device_masks\": %llu, "
           "\"device_ms_per_graph\": %.3f, \"rope_store_groups\": %llu, \"add_norm_groups\": %llu, \"mask_values_checked\": %llu, \"mask_mismatches\": %llu, \"graphs_recorded\": %llu, \"graphs_replayed\": %llu}\n",
           c.n_layer, c.d, n_seq, n_decode, total, worst, good_rows / sum_rows, (double) agree / total, step_ms,
           (unsigned long long) (cpu_only ? 0 : lm_ggml_backend_b200_split_mul_mat_count()), g_b200_device_mask_calls, bench_device_ms, (unsigned long long) n_rope_store, (unsigned long long) n_add_norm,
           g_b200_mask_values, g_b200_mask_mismatches, (unsigned long long) n_recorded, (unsigned long long) n_replayed);
    if (cpu.ctx) llama_free(cpu.ctx);
    if (cpu.model) llama_model_free(cpu.model);
    if (gpu.ctx) llama_free(gpu.ctx);
    if (gpu.model) llama_model_free(gpu.model);
    remove(path.c_str());
    return (worst < 3e-2 && agree >= 0.95 * total) ? 0 : 1;
}

// A quantised tensor placed in the plug-in's split buffer type (rows spread over all B200 devices, ragged row count):
// what set_tensor scatters must come back from get_tensor byte for byte.
static int run_split_roundtrip() {
    lm_ggml_backend_reg_t reg = lm_ggml_backend_b200_reg();
    auto fn = (lm_ggml_backend_split_buffer_type_t) lm_ggml_backend_reg_get_proc_address(reg, "lm_ggml_backend_split_buffer_type");
    if (!fn) { printf("{\"case\": \"split roundtrip\", \"error\": \"no split buffer type\"}\n"); return 2; }
    lm_ggml_backend_buffer_type_t buft = fn(0, nullptr);
    if (!buft) { printf("{\"case\": \"split roundtrip\", \"error\": \"null buffer type\"}\n"); return 2; }
    std::mt19937 rng(5);
    bool equal = true;
    for (lm_ggml_type type : {LM_GGML_TYPE_Q4_0, LM_GGML_TYPE_Q8_0}) {
        for (int64_t M : {300, 128, 2064}) {
            const int64_t K = 256;
            lm_ggml_init_params ip = { lm_ggml_tensor_overhead() * 4, nullptr, true };
            lm_ggml_context * ctx = lm_ggml_init(ip);
            lm_ggml_tensor * t = lm_ggml_new_tensor_2d(ctx, type, K, M);
            lm_ggml_backend_buffer_t buf = lm_ggml_backend_alloc_ctx_tensors_from_buft(ctx, buft);
            if (!buf) { printf("{\"case\": \"split roundtrip\", \"error\": \"allocation failed\"}\n"); return 2; }
            std::vector<float> w((size_t) M * K);
            fill_normal(w, rng, 0.05f);
            std::vector<uint8_t> q(lm_ggml_nbytes(t)), back(lm_ggml_nbytes(t), 0xAB);
            lm_ggml_quantize_chunk(type, w.data(), q.data(), 0, M, K, nullptr);
            lm_ggml_backend_tensor_set(t, q.data(), 0, q.size());
            lm_ggml_backend_tensor_get(t, back.data(), 0, back.size());
            equal = equal && memcmp(q.data(), back.data(), q.size()) == 0;
            lm_ggml_backend_buffer_free(buf);
            lm_ggml_free(ctx);
        }
    }
    printf("{\"case\": \"split roundtrip\", \"equal\": %s, \"devices\": %d, \"buffer_type\": \"%s\"}\n", equal ? "true" : "false",
           (int) lm_ggml_backend_reg_dev_count(reg), lm_ggml_backend_buft_name(buft));
    return equal ? 0 : 1;
}

int run_faults();   // faults.cpp

int main(int argc, char ** argv) {
    if (argc >= 2 && strcmp(argv[1], "faults") == 0) return run_faults();
    if (argc >= 2 && strcmp(argv[1], "split") == 0) return run_split_roundtrip();
    if (argc >= 2 && strcmp(argv[1], "ops") == 0) {
        int rc = 0;
        for (lm_ggml_type t : {LM_GGML_TYPE_Q4_0, LM_GGML_TYPE_Q8_0})
            for (int n : {1, 5, 24, 70}) rc |= run_ops(n, t);
        for (int n : {1, 24, 70}) rc |= run_ops(n, LM_GGML_TYPE_Q4_0, true);
        rc |= run_kv_ops();
        return rc;
    }
    if (argc >= 2 && strcmp(argv[1], "model") == 0) return run_model(argc, argv);
    fprintf(stderr, "usage: harness ops | harness split | harness faults | harness model [--layers N --d N --heads N --kv N --ff N --vocab N --ctx N --seqs N --decode N]\n");
    return 64;
}
