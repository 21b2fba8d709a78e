// Driver-side half of the device-side KQ mask: a replacement for llama_kv_cache_unified::set_input_kq_mask
// (cactus/llama-kv-cache.cpp:696-761) that the dynamic linker prefers over the one in the reference's library because it
// lives in the executable.  When switched on (harness flag --device-mask) and the case is one the backend's kernel covers
// -- causal attention, no ALiBi, no sliding window, one sequence per cell -- it does not walk n_tokens x n_kv cells on
// the host: it gathers position and sequence of the n cells of the attended window (one pass) and of the ubatch's
// tokens, and hands them to the backend through its extension proc together with the address of the mask it left
// unfilled.  Everything else goes to the reference's own function.
#include <dlfcn.h>

#include <cstdio>
#include <vector>

#include "../../cactus_b200/backend/ggml-b200.h"
#include "ggml-backend.h"
#include "llama-batch.h"
#include "llama-hparams.h"
#include "llama-kv-cache.h"

bool g_b200_device_mask = false;               // set by the harness
unsigned long long g_b200_device_mask_calls = 0;

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
