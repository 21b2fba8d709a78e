// Driver-side half of the device-side KQ mask: a replacement for llama_kv_cache_unified::set_input_kq_mask
// (cactus/llama-kv-cache.cpp:696-761) that the dynamic linker prefers over the one in the reference's library because it
// lives in the executable.  When switched on (harness flag --device-mask) and the case is one the backend's kernel covers
// -- causal attention, no ALiBi, no sliding window, one sequence per cell -- it does not walk n_tokens x n_kv cells on
// the host: it gathers position and sequence of the n cells of the attended window (one pass) and of the ubatch's
// tokens, and hands them to the backend through its extension proc together with the address of the mask it left
// unfilled.  Everything else goes to the reference's own function.
//
// With --verify-mask the reference's function runs as well, and what b200_kq_mask_build writes for the same cells and
// tokens is read back and compared bit for bit with the f16 cast of the reference's f32 mask (0 -> 0x0000, -inf -> 0xFC00).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <math.h>

#include <algorithm>
#include <cstdio>
#include <vector>

#include "../../cactus_b200/backend/ggml-b200.h"
#include "../../include/cactus_b200.h"
#include "ggml-backend.h"
#include "llama-batch.h"
#include "llama-hparams.h"
#include "llama-kv-cache.h"

bool g_b200_device_mask = false;               // set by the harness
unsigned long long g_b200_device_mask_calls = 0;
bool g_b200_mask_verify = false;               // set by the harness
unsigned long long g_b200_mask_values = 0, g_b200_mask_mismatches = 0;

// the reference's host mask (already in dst->data) against the device-built f16 mask of the same ubatch
static void verify_mask(const lm_ggml_tensor * dst, const std::vector<int32_t> & cell_pos, const std::vector<int32_t> & cell_seq,
                        const std::vector<int32_t> & tok_pos, const std::vector<int32_t> & tok_seq) {
    const int64_t n_kv = dst->ne[0], rows = dst->ne[1], n_tokens = (int64_t) tok_pos.size();
    const int64_t rows_dev = (n_tokens + 63) / 64 * 64;
    int32_t * d_ints = nullptr;
    uint16_t * d_mask = nullptr;
    const size_t n_ints = 2 * (size_t) n_kv + 2 * (size_t) n_tokens;
    if (cudaMalloc(&d_ints, n_ints * 4) != cudaSuccess || cudaMalloc(&d_mask, (size_t) std::max(rows, rows_dev) * n_kv * 2) != cudaSuccess) {
        ++g_b200_mask_mismatches;
        return;
    }
    cudaMemcpy(d_ints, cell_pos.data(), n_kv * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_ints + n_kv, cell_seq.data(), n_kv * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_ints + 2 * n_kv, tok_pos.data(), n_tokens * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_ints + 2 * n_kv + n_tokens, tok_seq.data(), n_tokens * 4, cudaMemcpyHostToDevice);
    const int rc = b200_kq_mask_build(d_ints, d_ints + n_kv, n_kv, d_ints + 2 * n_kv, d_ints + 2 * n_kv + n_tokens, n_tokens, d_mask, n_kv * 2, nullptr);
    std::vector<uint16_t> got((size_t) rows_dev * n_kv);
    if (rc != 0 || cudaMemcpy(got.data(), d_mask, got.size() * 2, cudaMemcpyDeviceToHost) != cudaSuccess) ++g_b200_mask_mismatches;
    const float * want = (const float *) dst->data;
    for (int64_t j = 0; j < std::min(rows, rows_dev); ++j)
        for (int64_t i = 0; i < n_kv; ++i) {
            const float w = want[j * n_kv + i];
            const uint16_t bits = w == 0.0f ? 0x0000 : (isinf(w) && w < 0 ? 0xFC00 : 0x7E00);   // anything else is not a causal mask value
            ++g_b200_mask_values;
            if (got[(size_t) j * n_kv + i] != bits) ++g_b200_mask_mismatches;
        }
    if (rows != rows_dev) ++g_b200_mask_mismatches;   // the padding the graph builder chose is the padding the kernel writes
    cudaFree(d_ints);
    cudaFree(d_mask);
}

typedef void (*set_mask_fn)(const llama_kv_cache_unified *, lm_ggml_tensor *, const llama_ubatch *, bool);

void llama_kv_cache_unified::set_input_kq_mask(lm_ggml_tensor * dst, const llama_ubatch * ubatch, bool causal_attn) const {
    static set_mask_fn original = (set_mask_fn) dlsym(RTLD_NEXT, "_ZNK22llama_kv_cache_unified17set_input_kq_maskEP14lm_ggml_tensorPK12llama_ubatchb");
    static lm_ggml_b200_kq_mask_from_cells_t give = nullptr;
    if (!give && g_b200_device_mask) {
        give = (lm_ggml_b200_kq_mask_from_cells_t) lm_ggml_backend_reg_get_proc_address(lm_ggml_backend_b200_reg(), "lm_ggml_backend_b200_kq_mask_from_cells");
    }
    // only for a context that computes on the B200 backend: its graph inputs live in that backend's pinned host buffer type
    // (cactus/llama-context.cpp:199-206); a CPU context in the same process keeps the host loop
    bool device = g_b200_device_mask && give && causal_attn && !hparams.use_alibi && swa_type == LLAMA_SWA_TYPE_NONE && dst->type == LM_GGML_TYPE_F32 &&
                  dst->buffer && lm_ggml_backend_buffer_get_type(dst->buffer) == lm_ggml_backend_b200_host_buffer_type();
    static std::vector<int32_t> cell_pos, cell_seq, tok_pos, tok_seq;
    const int64_t n_kv = n, n_tokens = ubatch->n_tokens;
    if (device) {
        cell_pos.resize(n_kv);
        cell_seq.resize(n_kv);
        for (int64_t i = 0; i < n_kv && device; ++i) {
            const kv_cell & c = cells[i];
            cell_pos[i] = c.pos;
            if (c.seq_id.empty()) cell_seq[i] = -1;
            else if (c.seq_id.size() == 1) cell_seq[i] = *c.seq_id.begin();
            else device = false;   // a cell shared by sequences: the host loop handles it
        }
    }
    if (device) {
        tok_pos.resize(n_tokens);
        tok_seq.resize(n_tokens);
        for (int64_t s = 0; s < ubatch->n_seqs; ++s)
            for (int64_t j = 0; j < ubatch->n_seq_tokens; ++j) {
                tok_pos[s * ubatch->n_seq_tokens + j] = ubatch->pos[s * ubatch->n_seq_tokens + j];
                tok_seq[s * ubatch->n_seq_tokens + j] = ubatch->seq_id[s][0];
            }
        if (g_b200_mask_verify && original) {
            original(this, dst, ubatch, causal_attn);
            verify_mask(dst, cell_pos, cell_seq, tok_pos, tok_seq);
        }
        give(dst->data, lm_ggml_nbytes(dst), cell_pos.data(), cell_seq.data(), n_kv, tok_pos.data(), tok_seq.data(), n_tokens);
        ++g_b200_device_mask_calls;
        return;
    }
    if (give && dst->buffer && lm_ggml_backend_buffer_get_type(dst->buffer) == lm_ggml_backend_b200_host_buffer_type()) {
        give(nullptr, 0, nullptr, nullptr, 0, nullptr, nullptr, 0);   // withdraw a hint of an earlier ubatch
    }
    if (!original) {
        fprintf(stderr, "device_mask: the reference's set_input_kq_mask was not found\n");
        abort();
    }
    original(this, dst, ubatch, causal_attn);
}
