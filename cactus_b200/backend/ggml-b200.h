// ggml backend for NVIDIA B200 (sm_100a) -- public entry points of the plug-in.
//
// The plug-in implements the backend interface of cactus's vendored ggml (cactus/ggml-backend-impl.h:
// reg, device, buffer type, buffer and backend vtables) on top of the C ABI in include/cactus_b200.h.
// A host program either links this library and calls
//     lm_ggml_backend_register(lm_ggml_backend_b200_reg());
// before it loads a model (registry: cactus/ggml-backend-reg.cpp:305), or loads it dynamically with
// lm_ggml_backend_load("libggml-b200.so") (cactus/ggml-backend-reg.cpp:401), which looks up the exported
// lm_ggml_backend_init.
#pragma once

#include "ggml-backend.h"
#include "ggml.h"

#ifdef __cplusplus
extern "C" {
#endif

#define LM_GGML_B200_NAME "B200"
#define LM_GGML_B200_MAX_DEVICES 16

LM_GGML_BACKEND_API lm_ggml_backend_reg_t lm_ggml_backend_b200_reg(void);
// a backend (stream) on device `device`; NULL if the device does not exist
LM_GGML_BACKEND_API lm_ggml_backend_t lm_ggml_backend_b200_init(int device);
LM_GGML_BACKEND_API bool lm_ggml_backend_is_b200(lm_ggml_backend_t backend);
LM_GGML_BACKEND_API lm_ggml_backend_buffer_type_t lm_ggml_backend_b200_buffer_type(int device);
LM_GGML_BACKEND_API lm_ggml_backend_buffer_type_t lm_ggml_backend_b200_host_buffer_type(void);

// counters of one backend since creation (for tests and benchmarks)
struct lm_ggml_b200_stats {
    uint64_t graphs;          // graph_compute calls
    uint64_t nodes;           // nodes executed (views excluded)
    uint64_t mul_mat;         // MUL_MAT nodes
    uint64_t flash_attn;      // FLASH_ATTN_EXT nodes
    uint64_t act_quantized;   // activation tensors quantised (shared by consecutive mul_mats)
    uint64_t mask_indexed;    // mask scans (shared by all layers of a graph)
    uint64_t rope_stores;     // ROPE(q), ROPE(k), CPY(k), CPY(v) groups done by one kernel
    double   device_ms;       // CUDA-event time of all graph_compute calls when timing is on (B200_TIMING=1)
};
LM_GGML_BACKEND_API void lm_ggml_backend_b200_get_stats(lm_ggml_backend_t backend, struct lm_ggml_b200_stats * out);
// Extension procs behind lm_ggml_backend_reg_get_proc_address (private to this backend):
//   "lm_ggml_backend_b200_kq_mask_from_cells": the driver did not fill the f32 KQ mask whose host data is
//   `mask_host_data` (n_kv * pad64(n_tokens) floats); the next upload from that address is skipped and the CPY node
//   that casts the uploaded tensor to f16 writes, on the device, what llama_kv_cache_unified::set_input_kq_mask
//   (cactus/llama-kv-cache.cpp:696-761) would have written: 0 where cell i holds sequence tok_seq[j] and
//   cell_pos[i] <= tok_pos[j], -inf elsewhere and in the padding rows.  cell_seq[i] = -1 for an empty cell; one sequence
//   per cell.  The arrays are copied before the call returns.  A null mask_host_data withdraws the hint.
//   "lm_ggml_backend_b200_kq_masks_built": how many masks were synthesised that way since the process started.
typedef void (*lm_ggml_b200_kq_mask_from_cells_t)(const void * mask_host_data, size_t mask_bytes, const int32_t * cell_pos, const int32_t * cell_seq,
                                                  int64_t n_kv, const int32_t * tok_pos, const int32_t * tok_seq, int64_t n_tokens);
typedef uint64_t (*lm_ggml_b200_kq_masks_built_t)(void);
//   "lm_ggml_backend_b200_timing_totals": CUDA-event time and count of all graph_compute calls of all backends of the
//   process while B200_TIMING=1 (for drivers that cannot reach the backends a llama_context owns).
typedef void (*lm_ggml_b200_timing_totals_t)(double * device_ms, uint64_t * graphs);
//   "lm_ggml_backend_b200_fused_group_counts": groups of nodes that ran as one kernel since the process started --
//   ROPE(q), ROPE(k), CPY(k), CPY(v) of a layer; residual ADD + RMS_NORM + MUL + activation quantiser.
typedef void (*lm_ggml_b200_fused_group_counts_t)(uint64_t * rope_stores, uint64_t * add_norms);
//   "lm_ggml_backend_b200_graph_counts": node lists recorded into a CUDA graph and node lists replayed from one since the
//   process started (B200_GRAPHS=0 switches the replay off: every list is then launched kernel by kernel).
typedef void (*lm_ggml_b200_graph_counts_t)(uint64_t * recorded, uint64_t * replayed);
// MUL_MAT nodes computed on weights of the split buffer type since the process started (all backends)
LM_GGML_BACKEND_API uint64_t lm_ggml_backend_b200_split_mul_mat_count(void);

#ifdef __cplusplus
}
#endif
