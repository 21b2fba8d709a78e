// Checker infrastructure, not product code.
//
// A thin C shim over the reference's own ggml + ggml-cpu (compiled unmodified into libggml_ref.so by
// the Makefile beside this file).  Each function builds the one-node graph a llama graph would hold
// for that op and runs it on the reference CPU backend, so tests can compare the CUDA kernels and the
// plain-C restatement (oracle.c) with what the reference really computes, and the bench can time the
// reference's CPU path on the host cores.
//
// Reference entry points used: lm_ggml_mul_mat (cactus/ggml.c:2740), lm_ggml_flash_attn_ext
// (cactus/ggml.c:4405), lm_ggml_graph_compute (cactus/ggml-cpu/ggml-cpu.c:3083), type traits
// (cactus/ggml-cpu/ggml-cpu.c:198-367), lm_ggml_quantize_chunk (cactus/ggml.c:6449).

#include "ggml.h"
#include "ggml-cpu.h"
#include "ggml-backend.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

namespace {

struct ctx_guard {
    lm_ggml_context * ctx;
    explicit ctx_guard(size_t mem) {
        lm_ggml_init_params p = { mem, nullptr, /*no_alloc=*/true };
        ctx = lm_ggml_init(p);
    }
    ~ctx_guard() { lm_ggml_free(ctx); }
};

// Runs `gf` with a persistent threadpool `reps` times; returns the median seconds per run.
double run_graph(lm_ggml_cgraph * gf, int n_threads, int warmup, int reps) {
    lm_ggml_threadpool_params tpp = lm_ggml_threadpool_params_default(n_threads);
    lm_ggml_threadpool * tp = lm_ggml_threadpool_new(&tpp);
    lm_ggml_cplan plan = lm_ggml_graph_plan(gf, n_threads, tp);
    std::vector<uint8_t> work(plan.work_size + 64);
    plan.work_data = work.data();
    std::vector<double> t;
    for (int i = 0; i < warmup + reps; ++i) {
        auto t0 = std::chrono::steady_clock::now();
        lm_ggml_graph_compute(gf, &plan);
        auto t1 = std::chrono::steady_clock::now();
        if (i >= warmup) t.push_back(std::chrono::duration<double>(t1 - t0).count());
    }
    lm_ggml_threadpool_free(tp);
    std::sort(t.begin(), t.end());
    return t.empty() ? 0.0 : t[t.size() / 2];
}

lm_ggml_tensor * wrap(lm_ggml_context * ctx, lm_ggml_type type, int nd, const int64_t * ne, const void * data) {
    lm_ggml_tensor * t = lm_ggml_new_tensor(ctx, type, nd, ne);
    t->data = const_cast<void *>(data);
    return t;
}

}  // namespace

extern "C" {

int ref_init(void) {
    lm_ggml_cpu_init();
    return 0;
}

// Weight-side quantisers as the reference uses them when a model file is produced
// (lm_ggml_quantize_chunk -> quantize_row_q4_0_ref / quantize_row_q8_0_ref). type: 2 = Q4_0, 8 = Q8_0.
int64_t ref_quantize_weights(int type, const float * src, void * dst, int64_t nrows, int64_t k) {
    return (int64_t) lm_ggml_quantize_chunk((lm_ggml_type) type, src, dst, 0, nrows, k, nullptr);
}

// Activation-side quantiser exactly as mul_mat calls it: type_traits_cpu[Q8_0].from_float, i.e. the
// SIMD branch this build was compiled for (AVX2 with the pinned flags).
void ref_quantize_row_q8_0(const float * x, void * y, int64_t k) {
    lm_ggml_get_type_traits_cpu(LM_GGML_TYPE_Q8_0)->from_float(x, y, k);
}

// The scalar variant (quantize_row_q8_0_ref) for comparison.
void ref_quantize_row_q8_0_scalar(const float * x, void * y, int64_t k) {
    lm_ggml_get_type_traits(LM_GGML_TYPE_Q8_0)->from_float_ref(x, y, k);
}

void ref_dequantize_row(int type, const void * x, float * y, int64_t k) {
    lm_ggml_get_type_traits((lm_ggml_type) type)->to_float(x, y, k);
}

// One weight row against one Q8_0 activation column: lm_ggml_vec_dot_q4_0_q8_0 / q8_0_q8_0.
float ref_vec_dot(int wtype, int64_t k, const void * w_row, const void * a_q8) {
    float s = 0.0f;
    lm_ggml_get_type_traits_cpu((lm_ggml_type) wtype)->vec_dot((int) k, &s, 0, w_row, 0, a_q8, 0, 1);
    return s;
}

// dst[M,N] = W[K,M]^T x[K,N]; W quantised (wtype 2 or 8), x f32 with row stride x_stride elements.
// Returns the median seconds per run (reps >= 1).
double ref_mul_mat(int wtype, int64_t M, int64_t K, int64_t N, const void * w, const float * x, int64_t x_stride,
                   float * dst, int n_threads, int warmup, int reps) {
    ctx_guard g(16 * 1024 * 1024);
    const int64_t new_[2] = { K, M };
    lm_ggml_tensor * W = wrap(g.ctx, (lm_ggml_type) wtype, 2, new_, w);
    const int64_t nex[2] = { K, N };
    lm_ggml_tensor * X = wrap(g.ctx, LM_GGML_TYPE_F32, 2, nex, x);
    if (x_stride != K) {
        X->nb[1] = (size_t) x_stride * sizeof(float);
        X->nb[2] = X->nb[1] * N;
        X->nb[3] = X->nb[2];
    }
    lm_ggml_tensor * Y = lm_ggml_mul_mat(g.ctx, W, X);
    Y->data = dst;
    lm_ggml_cgraph * gf = lm_ggml_new_graph(g.ctx);
    lm_ggml_build_forward_expand(gf, Y);
    return run_graph(gf, n_threads, warmup, reps);
}

// FLASH_ATTN_EXT with the tensor shapes and strides llama's unified KV cache produces
// (cactus/llama-graph.cpp:1059-1174, cactus/llama-kv-cache.cpp:583-615):
//   q    f32 [D, H, Nq] contiguous (token-major), permuted to [D, Nq, H]
//   kc/vc f16 cache [Hkv*D, n_cells]; the op sees the first n_kv cells as [D, n_kv, Hkv]
//   mask f16 [n_kv, pad64(Nq)] contiguous
//   dst  f32 [D, H, Nq]
double ref_flash_attn_ext(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv,
                          const float * q, const void * kc, const void * vc, const void * mask,
                          float scale, float max_bias, float logit_softcap,
                          float * dst, int n_threads, int warmup, int reps) {
    ctx_guard g(16 * 1024 * 1024);
    const int64_t neq[3] = { D, H, Nq };
    lm_ggml_tensor * Q = lm_ggml_permute(g.ctx, wrap(g.ctx, LM_GGML_TYPE_F32, 3, neq, q), 0, 2, 1, 3);
    const int64_t nek[3] = { D, Hkv, n_kv };
    lm_ggml_tensor * Kt = lm_ggml_permute(g.ctx, wrap(g.ctx, LM_GGML_TYPE_F16, 3, nek, kc), 0, 2, 1, 3);
    lm_ggml_tensor * Vt = lm_ggml_permute(g.ctx, wrap(g.ctx, LM_GGML_TYPE_F16, 3, nek, vc), 0, 2, 1, 3);
    const int64_t nem[2] = { n_kv, (Nq + 63) / 64 * 64 };
    lm_ggml_tensor * Mk = wrap(g.ctx, LM_GGML_TYPE_F16, 2, nem, mask);
    lm_ggml_tensor * O = lm_ggml_flash_attn_ext(g.ctx, Q, Kt, Vt, Mk, scale, max_bias, logit_softcap);
    lm_ggml_flash_attn_ext_set_prec(O, LM_GGML_PREC_F32);
    O->data = dst;
    // permute results are views: give them their parent's data
    Q->data = Q->view_src->data; Kt->data = Kt->view_src->data; Vt->data = Vt->view_src->data;
    lm_ggml_cgraph * gf = lm_ggml_new_graph(g.ctx);
    lm_ggml_build_forward_expand(gf, O);
    return run_graph(gf, n_threads, warmup, reps);
}

// Small row ops of the llama layer, for checking the device versions.
//   op 0: RMS_NORM(x, eps) * w      x [d,T], w [d]
//   op 1: SILU(a) * b               a,b [d,T]
//   op 2: ADD(a, b)                 a,b [d,T]
//   op 3: ROPE mode 0 on a [D,H,T] with int32 positions in b, freq_base in p0, n_dims = D
//   op 4: CPY f32 -> f16            a [d,T] -> dst f16
//   op 5: ROPE mode 0 on an f16 a [D,H,T] (passed through the float pointer) -> dst f16: the K-shift of the cache
int ref_row_op(int op, int64_t d, int64_t h, int64_t T, const float * a, const void * b, float p0, void * dst, int n_threads) {
    ctx_guard g(16 * 1024 * 1024);
    lm_ggml_tensor * out = nullptr;
    const int64_t ne2[2] = { d, T };
    switch (op) {
        case 0: {
            lm_ggml_tensor * x = wrap(g.ctx, LM_GGML_TYPE_F32, 2, ne2, a);
            const int64_t new_[1] = { d };
            lm_ggml_tensor * w = wrap(g.ctx, LM_GGML_TYPE_F32, 1, new_, b);
            lm_ggml_tensor * n = lm_ggml_rms_norm(g.ctx, x, p0);
            // intermediate needs storage
            static thread_local std::vector<float> tmp;
            tmp.resize((size_t) d * T);
            n->data = tmp.data();
            out = lm_ggml_mul(g.ctx, n, w);
        } break;
        case 1: {
            lm_ggml_tensor * x = wrap(g.ctx, LM_GGML_TYPE_F32, 2, ne2, a);
            lm_ggml_tensor * y = wrap(g.ctx, LM_GGML_TYPE_F32, 2, ne2, b);
            lm_ggml_tensor * s = lm_ggml_silu(g.ctx, x);
            static thread_local std::vector<float> tmp;
            tmp.resize((size_t) d * T);
            s->data = tmp.data();
            out = lm_ggml_mul(g.ctx, s, y);
        } break;
        case 2: {
            lm_ggml_tensor * x = wrap(g.ctx, LM_GGML_TYPE_F32, 2, ne2, a);
            lm_ggml_tensor * y = wrap(g.ctx, LM_GGML_TYPE_F32, 2, ne2, b);
            out = lm_ggml_add(g.ctx, x, y);
        } break;
        case 3: {
            const int64_t ne3[3] = { d, h, T };
            lm_ggml_tensor * x = wrap(g.ctx, LM_GGML_TYPE_F32, 3, ne3, a);
            const int64_t nep[1] = { T };
            lm_ggml_tensor * pos = wrap(g.ctx, LM_GGML_TYPE_I32, 1, nep, b);
            out = lm_ggml_rope_ext(g.ctx, x, pos, nullptr, (int) d, 0, 0, p0, 1.0f, 0.0f, 1.0f, 0.0f, 0.0f);
        } break;
        case 4: {
            lm_ggml_tensor * x = wrap(g.ctx, LM_GGML_TYPE_F32, 2, ne2, a);
            lm_ggml_tensor * y = lm_ggml_new_tensor(g.ctx, LM_GGML_TYPE_F16, 2, ne2);
            y->data = dst;
            out = lm_ggml_cpy(g.ctx, x, y);
        } break;
        case 5: {   // ROPE on an f16 tensor (the K-shift of the cache); a is f16 here
            const int64_t ne3[3] = { d, h, T };
            lm_ggml_tensor * x = wrap(g.ctx, LM_GGML_TYPE_F16, 3, ne3, a);
            const int64_t nep[1] = { T };
            lm_ggml_tensor * pos = wrap(g.ctx, LM_GGML_TYPE_I32, 1, nep, b);
            out = lm_ggml_rope_ext(g.ctx, x, pos, nullptr, (int) d, 0, 0, p0, 1.0f, 0.0f, 1.0f, 0.0f, 0.0f);
        } break;
        default: return -1;
    }
    out->data = dst;
    lm_ggml_cgraph * gf = lm_ggml_new_graph(g.ctx);
    lm_ggml_build_forward_expand(gf, out);
    run_graph(gf, n_threads, 0, 1);
    return 0;
}

}  // extern "C"
