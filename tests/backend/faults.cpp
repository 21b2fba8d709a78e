// Failure paths of the plug-in, with every failure made on the host (no GPU fault, trap or hang):
//   * an abort callback that says "stop" (the hook of cactus/ggml-backend.h lm_ggml_backend_set_abort_callback_t, reached
//     through the registry's get_proc_address): graph_compute returns LM_GGML_STATUS_ABORTED and the backend stays usable;
//   * a device allocator that fails: cudaMalloc of this executable (preferred by the dynamic linker over the CUDA runtime's)
//     returns cudaErrorMemoryAllocation while the switch is on.  A buffer allocation then yields no buffer, a graph whose
//     scratch has to grow returns LM_GGML_STATUS_ALLOC_FAILED, and with the switch off the same backend computes again.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "../../cactus_b200/backend/ggml-b200.h"
#include "ggml-backend.h"
#include "ggml-cpu.h"
#include "ggml.h"

static bool g_fail_cuda_malloc = false;
static unsigned long long g_failed_mallocs = 0;

extern "C" cudaError_t cudaMalloc(void ** ptr, size_t bytes) {
    typedef cudaError_t (*fn_t)(void **, size_t);
    static fn_t real = (fn_t) dlsym(RTLD_NEXT, "cudaMalloc");
    if (g_fail_cuda_malloc || !real) {
        ++g_failed_mallocs;
        if (ptr) *ptr = nullptr;
        return cudaErrorMemoryAllocation;
    }
    return real(ptr, bytes);
}

static bool stop_now(void *) { return true; }

int run_faults() {
    lm_ggml_backend_t gpu = lm_ggml_backend_b200_init(0);
    if (!gpu) { printf("{\"error\": \"no B200 backend\"}\n"); return 2; }
    const int64_t K = 512, M = 192, T = 24;
    lm_ggml_init_params ip = { 8 * 1024 * 1024, nullptr, true };
    lm_ggml_context * ctx = lm_ggml_init(ip);
    lm_ggml_tensor * x = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_F32, K, T);
    lm_ggml_tensor * w = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_Q4_0, K, M);
    lm_ggml_tensor * b = lm_ggml_new_tensor_2d(ctx, LM_GGML_TYPE_F32, M, T);
    for (lm_ggml_tensor * t : {x, w, b}) lm_ggml_set_input(t);
    lm_ggml_tensor * y = lm_ggml_add(ctx, lm_ggml_mul_mat(ctx, w, x), b);
    lm_ggml_set_output(y);
    lm_ggml_cgraph * gf = lm_ggml_new_graph(ctx);
    lm_ggml_build_forward_expand(gf, y);
    lm_ggml_backend_buffer_t buf = lm_ggml_backend_alloc_ctx_tensors(ctx, gpu);
    if (!buf) { printf("{\"error\": \"alloc failed\"}\n"); return 2; }
    std::mt19937 rng(3);
    std::normal_distribution<float> nd(0.0f, 1.0f);
    std::vector<float> xv((size_t) K * T), wv((size_t) K * M), bv((size_t) M * T);
    for (auto & v : xv) v = nd(rng);
    for (auto & v : wv) v = nd(rng) * 0.05f;
    for (auto & v : bv) v = nd(rng);
    std::vector<uint8_t> wq(lm_ggml_nbytes(w));
    lm_ggml_quantize_chunk(w->type, wv.data(), wq.data(), 0, M, K, nullptr);
    lm_ggml_backend_tensor_set(x, xv.data(), 0, xv.size() * 4);
    lm_ggml_backend_tensor_set(w, wq.data(), 0, wq.size());
    lm_ggml_backend_tensor_set(b, bv.data(), 0, bv.size() * 4);

    auto read_y = [&](std::vector<float> & out) {
        out.resize((size_t) M * T);
        lm_ggml_backend_tensor_get(y, out.data(), 0, out.size() * 4);
    };
    std::vector<float> y0, y1, y2;
    const lm_ggml_status s_first = lm_ggml_backend_graph_compute(gpu, gf);
    read_y(y0);

    // ---- abort callback ----
    auto set_abort = (lm_ggml_backend_set_abort_callback_t) lm_ggml_backend_reg_get_proc_address(lm_ggml_backend_b200_reg(), "lm_ggml_backend_set_abort_callback");
    lm_ggml_status s_abort = LM_GGML_STATUS_FAILED, s_after_abort = LM_GGML_STATUS_FAILED;
    if (set_abort) {
        set_abort(gpu, stop_now, nullptr);
        s_abort = lm_ggml_backend_graph_compute(gpu, gf);
        set_abort(gpu, nullptr, nullptr);
        std::vector<float> zero((size_t) M * T, 0.0f);
        lm_ggml_backend_tensor_set(y, zero.data(), 0, zero.size() * 4);
        s_after_abort = lm_ggml_backend_graph_compute(gpu, gf);
        read_y(y1);
    }

    // ---- failing allocator: a fresh backend has no scratch yet, so its first graph must allocate ----
    lm_ggml_backend_t gpu2 = lm_ggml_backend_b200_init(0);
    g_fail_cuda_malloc = true;
    lm_ggml_backend_buffer_t no_buf = lm_ggml_backend_buft_alloc_buffer(lm_ggml_backend_b200_buffer_type(0), 1 << 20);
    const lm_ggml_status s_alloc = gpu2 ? lm_ggml_backend_graph_compute(gpu2, gf) : LM_GGML_STATUS_FAILED;
    const unsigned long long refused = g_failed_mallocs;
    g_fail_cuda_malloc = false;
    const lm_ggml_status s_after_alloc = gpu2 ? lm_ggml_backend_graph_compute(gpu2, gf) : LM_GGML_STATUS_FAILED;
    read_y(y2);

    const bool same1 = y1.size() == y0.size() && memcmp(y0.data(), y1.data(), y0.size() * 4) == 0;
    const bool same2 = y2.size() == y0.size() && memcmp(y0.data(), y2.data(), y0.size() * 4) == 0;
    bool finite = true;
    for (float v : y0) finite = finite && std::isfinite(v);
    printf("{\"case\": \"faults\", \"first\": %d, \"aborted\": %d, \"after_abort\": %d, \"after_abort_same\": %s, \"buffer_refused\": %s, "
           "\"alloc_failed\": %d, \"refused_mallocs\": %llu, \"after_alloc\": %d, \"after_alloc_same\": %s, \"finite\": %s}\n",
           (int) s_first, (int) s_abort, (int) s_after_abort, same1 ? "true" : "false", no_buf ? "false" : "true", (int) s_alloc, refused,
           (int) s_after_alloc, same2 ? "true" : "false", finite ? "true" : "false");
    const bool ok = s_first == LM_GGML_STATUS_SUCCESS && s_abort == LM_GGML_STATUS_ABORTED && s_after_abort == LM_GGML_STATUS_SUCCESS && same1 && !no_buf &&
                    s_alloc == LM_GGML_STATUS_ALLOC_FAILED && refused > 0 && s_after_alloc == LM_GGML_STATUS_SUCCESS && same2 && finite;
    if (no_buf) lm_ggml_backend_buffer_free(no_buf);
    lm_ggml_backend_buffer_free(buf);
    lm_ggml_free(ctx);
    if (gpu2) lm_ggml_backend_free(gpu2);
    lm_ggml_backend_free(gpu);
    return ok ? 0 : 1;
}
