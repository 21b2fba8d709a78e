// ggml backend for NVIDIA B200: the host side of the plug-in (see ggml-b200.h).
//
// Everything that computes is a call into the C ABI of libcactus_b200.so (include/cactus_b200.h); this file
// holds the vtables of cactus/ggml-backend-impl.h, the device buffers, and graph_compute's node dispatch.
#include "ggml-b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/cactus_b200.h"
#include "ggml-backend-impl.h"
#include "ggml-impl.h"

#define B200_LOG_ERROR(...) LM_GGML_LOG_ERROR(__VA_ARGS__)

namespace {

constexpr size_t B200_ALIGNMENT = 256;
constexpr size_t B200_STAGE_BYTES = 64u << 20;  // bounce buffer for weight layout conversion

bool cuda_ok(cudaError_t e, const char * what) {
    if (e == cudaSuccess) return true;
    B200_LOG_ERROR("ggml-b200: %s failed: %s\n", what, cudaGetErrorString(e));
    return false;
}

struct device_guard {
    int prev = 0;
    explicit device_guard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~device_guard() {
        int cur = 0;
        cudaGetDevice(&cur);
        if (cur != prev) cudaSetDevice(prev);
    }
};

// ---------------------------------------------------------------------------------------------
// devices
// ---------------------------------------------------------------------------------------------
struct b200_device_ctx {
    int device;
    std::string name, description;
};

lm_ggml_backend_buffer_type_t device_buffer_type(int device);
bool buft_is_b200(lm_ggml_backend_buffer_type_t buft);
bool buft_is_b200_host(lm_ggml_backend_buffer_type_t buft);

// A quantised tensor that owns its storage in a B200 device buffer is kept in the tiled layout.
bool is_tiled_type(lm_ggml_type t) { return t == LM_GGML_TYPE_Q4_0 || t == LM_GGML_TYPE_Q8_0; }
bool tensor_is_tiled(const lm_ggml_tensor * t) {
    return is_tiled_type(t->type) && t->view_src == nullptr && t->ne[0] % 32 == 0;
}
int64_t tensor_rows(const lm_ggml_tensor * t) { return t->ne[1] * t->ne[2] * t->ne[3]; }
size_t block_bytes(lm_ggml_type t) { return t == LM_GGML_TYPE_Q4_0 ? 18 : 34; }

// ---------------------------------------------------------------------------------------------
// device buffer
// ---------------------------------------------------------------------------------------------
struct b200_buffer_ctx {
    int device;
    void * base = nullptr;
    void * stage = nullptr;  // lazily allocated bounce buffer (row-major block stream on the device)
    size_t stage_bytes = 0;
    ~b200_buffer_ctx() {
        device_guard g(device);
        if (stage) cudaFree(stage);
        if (base) cudaFree(base);
    }
    void * get_stage(size_t bytes) {
        if (stage_bytes < bytes) {
            if (stage) cudaFree(stage);
            stage = nullptr;
            stage_bytes = 0;
            if (!cuda_ok(cudaMalloc(&stage, bytes), "cudaMalloc(stage)")) return nullptr;
            stage_bytes = bytes;
        }
        return stage;
    }
};

void buffer_free(lm_ggml_backend_buffer_t buffer) { delete (b200_buffer_ctx *) buffer->context; }
void * buffer_get_base(lm_ggml_backend_buffer_t buffer) { return ((b200_buffer_ctx *) buffer->context)->base; }

// Moves bytes [offset, offset+size) of a tiled tensor between its row-major block stream and the device.
// Works on whole 16-row groups: rows that are only partly covered are first brought back to the stream.
bool tiled_transfer(b200_buffer_ctx * ctx, const lm_ggml_tensor * t, void * host, size_t offset, size_t size, bool to_device, int fill = -1) {
    const int64_t K = t->ne[0], M = tensor_rows(t);
    const size_t rb = (size_t) (K / 32) * block_bytes(t->type);
    const int64_t max_rows = std::max<int64_t>(16, (int64_t) (B200_STAGE_BYTES / rb) / 16 * 16);
    size_t done = 0;
    while (done < size) {
        const size_t off = offset + done;
        const int64_t r0 = (int64_t) (off / rb) / 16 * 16;
        const int64_t r1 = std::min<int64_t>(M, r0 + max_rows);
        const size_t chunk_begin = (size_t) r0 * rb, chunk_end = (size_t) r1 * rb;
        const size_t n = std::min(size - done, chunk_end - off);
        // rows actually touched, extended to the 16-row group
        const int64_t t1 = std::min<int64_t>(M, ((int64_t) ((off + n + rb - 1) / rb) + 15) / 16 * 16);
        const int64_t rows = t1 - r0;
        uint8_t * stage = (uint8_t *) ctx->get_stage((size_t) rows * rb);
        if (!stage) return false;
        const bool whole = (off == chunk_begin) && (off + n == (size_t) t1 * rb);
        if (!to_device || !whole) {
            if (b200_weight_download(t->type, K, M, t->data, stage, r0, rows, nullptr) != B200_OK) {
                B200_LOG_ERROR("ggml-b200: weight_download: %s\n", b200_last_error());
                return false;
            }
        }
        if (to_device) {
            if (fill >= 0) {
                if (!cuda_ok(cudaMemset(stage + (off - chunk_begin), fill, n), "cudaMemset")) return false;
            } else if (!cuda_ok(cudaMemcpy(stage + (off - chunk_begin), (const uint8_t *) host + done, n, cudaMemcpyHostToDevice), "cudaMemcpy H2D")) {
                return false;
            }
            if (b200_weight_upload(t->type, K, M, stage, t->data, r0, rows, nullptr) != B200_OK) {
                B200_LOG_ERROR("ggml-b200: weight_upload: %s\n", b200_last_error());
                return false;
            }
            if (!cuda_ok(cudaStreamSynchronize(nullptr), "sync after upload")) return false;
        } else {
            if (!cuda_ok(cudaMemcpy((uint8_t *) host + done, stage + (off - chunk_begin), n, cudaMemcpyDeviceToHost), "cudaMemcpy D2H")) return false;
        }
        done += n;
        (void) chunk_end;
    }
    return true;
}

void buffer_memset_tensor(lm_ggml_backend_buffer_t buffer, lm_ggml_tensor * tensor, uint8_t value, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    device_guard g(ctx->device);
    if (tensor_is_tiled(tensor)) {
        LM_GGML_ASSERT(tiled_transfer(ctx, tensor, nullptr, offset, size, true, value));
        return;
    }
    LM_GGML_ASSERT(cuda_ok(cudaMemset((char *) tensor->data + offset, value, size), "cudaMemset"));
    cudaStreamSynchronize(nullptr);
}

// ---------------------------------------------------------------------------------------------
// KQ mask synthesised on the device (extension proc "lm_ggml_backend_b200_kq_mask_from_cells").
// llama_kv_cache_unified::set_input_kq_mask (cactus/llama-kv-cache.cpp:696-761) fills an f32 mask of n_kv x pad64(n_tokens)
// on the host, one std::set lookup per (token, cell), the scheduler uploads it and a CPY node casts it to f16.  A driver
// that knows the cells hands over what the loop reads instead -- position and sequence of every cell of the attended
// window, position and sequence of every token -- together with the host address of the mask tensor it did NOT fill.
// When the scheduler then uploads from that address, the upload is skipped (the small arrays go up instead), and the CPY
// node that reads the uploaded tensor writes the f16 mask with b200_kq_mask_build.  One sequence per cell; the driver
// keeps the host loop for anything else (ALiBi, sliding windows, cells shared by sequences).
// ---------------------------------------------------------------------------------------------
struct kq_mask_hint_t {
    std::mutex mu;
    const void * host_mask = nullptr;
    size_t host_bytes = 0;
    std::vector<int32_t> cell_pos, cell_seq, tok_pos, tok_seq;
    uint64_t serial = 0;
    struct dev_state {
        int32_t * buf = nullptr;      // [cell_pos | cell_seq | tok_pos | tok_seq]
        size_t cap = 0;               // in int32
        const void * dev_mask = nullptr;   // the uploaded f32 tensor that stands for the mask
        int64_t n_kv = 0, n_tokens = 0;
        uint64_t serial = 0;
    } dev[LM_GGML_B200_MAX_DEVICES];
    std::atomic<uint64_t> masks_built{0};
};
kq_mask_hint_t g_kq_hint;

// true: `data` is the mask the driver left unfilled; its description is now on device `device`, `dst` stands for it
bool kq_hint_take_upload(int device, const void * data, size_t size, const void * dst) {
    kq_mask_hint_t & h = g_kq_hint;
    std::lock_guard<std::mutex> lock(h.mu);
    if (!h.host_mask || data != h.host_mask || size != h.host_bytes || device < 0 || device >= LM_GGML_B200_MAX_DEVICES) return false;
    kq_mask_hint_t::dev_state & d = h.dev[device];
    const size_t n_kv = h.cell_pos.size(), n_tok = h.tok_pos.size(), need = 2 * n_kv + 2 * n_tok;
    if (need > d.cap) {
        if (d.buf) cudaFree(d.buf);
        d.buf = nullptr;
        d.cap = 0;
        if (!cuda_ok(cudaMalloc((void **) &d.buf, need * 2 * sizeof(int32_t)), "cudaMalloc(kq mask cells)")) return false;
        d.cap = need * 2;
    }
    bool ok = cuda_ok(cudaMemcpy(d.buf, h.cell_pos.data(), n_kv * 4, cudaMemcpyHostToDevice), "cudaMemcpy(cells)");
    ok = ok && cuda_ok(cudaMemcpy(d.buf + n_kv, h.cell_seq.data(), n_kv * 4, cudaMemcpyHostToDevice), "cudaMemcpy(cells)");
    ok = ok && cuda_ok(cudaMemcpy(d.buf + 2 * n_kv, h.tok_pos.data(), n_tok * 4, cudaMemcpyHostToDevice), "cudaMemcpy(tokens)");
    ok = ok && cuda_ok(cudaMemcpy(d.buf + 2 * n_kv + n_tok, h.tok_seq.data(), n_tok * 4, cudaMemcpyHostToDevice), "cudaMemcpy(tokens)");
    if (!ok) return false;
    d.dev_mask = dst;
    d.n_kv = (int64_t) n_kv;
    d.n_tokens = (int64_t) n_tok;
    d.serial = h.serial;
    return true;
}

void buffer_set_tensor(lm_ggml_backend_buffer_t buffer, lm_ggml_tensor * tensor, const void * data, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    device_guard g(ctx->device);
    if (offset == 0 && tensor->type == LM_GGML_TYPE_F32 && kq_hint_take_upload(ctx->device, data, size, tensor->data)) return;
    if (tensor_is_tiled(tensor)) {
        LM_GGML_ASSERT(tiled_transfer(ctx, tensor, const_cast<void *>(data), offset, size, true));
        return;
    }
    LM_GGML_ASSERT(cuda_ok(cudaMemcpy((char *) tensor->data + offset, data, size, cudaMemcpyHostToDevice), "cudaMemcpy H2D"));
}

void buffer_get_tensor(lm_ggml_backend_buffer_t buffer, const lm_ggml_tensor * tensor, void * data, size_t offset, size_t size) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    device_guard g(ctx->device);
    if (tensor_is_tiled(tensor)) {
        LM_GGML_ASSERT(tiled_transfer(ctx, tensor, data, offset, size, false));
        return;
    }
    LM_GGML_ASSERT(cuda_ok(cudaMemcpy(data, (const char *) tensor->data + offset, size, cudaMemcpyDeviceToHost), "cudaMemcpy D2H"));
}

bool buffer_cpy_tensor(lm_ggml_backend_buffer_t buffer, const lm_ggml_tensor * src, lm_ggml_tensor * dst) {
    // device-to-device copies between plain (not tiled) contiguous tensors of B200 buffers; everything else
    // goes through the generic host path of the caller (cactus/ggml-backend.cpp:370-391)
    if (!src->buffer || !buft_is_b200(src->buffer->buft)) return false;
    if (tensor_is_tiled(src) || tensor_is_tiled(dst) || is_tiled_type(src->type)) return false;
    if (!lm_ggml_is_contiguous(src) || !lm_ggml_is_contiguous(dst) || lm_ggml_nbytes(src) != lm_ggml_nbytes(dst)) return false;
    b200_buffer_ctx * dctx = (b200_buffer_ctx *) buffer->context;
    b200_buffer_ctx * sctx = (b200_buffer_ctx *) src->buffer->context;
    device_guard g(dctx->device);
    cudaError_t e = (dctx->device == sctx->device) ? cudaMemcpy(dst->data, src->data, lm_ggml_nbytes(src), cudaMemcpyDeviceToDevice)
                                                   : cudaMemcpyPeer(dst->data, dctx->device, src->data, sctx->device, lm_ggml_nbytes(src));
    return cuda_ok(e, "cudaMemcpy D2D");
}

void buffer_clear(lm_ggml_backend_buffer_t buffer, uint8_t value) {
    b200_buffer_ctx * ctx = (b200_buffer_ctx *) buffer->context;
    device_guard g(ctx->device);
    cuda_ok(cudaMemset(ctx->base, value, buffer->size), "cudaMemset");
    cudaStreamSynchronize(nullptr);
}

const lm_ggml_backend_buffer_i b200_buffer_iface = {
    /* .free_buffer   = */ buffer_free,
    /* .get_base      = */ buffer_get_base,
    /* .init_tensor   = */ nullptr,
    /* .memset_tensor = */ buffer_memset_tensor,
    /* .set_tensor    = */ buffer_set_tensor,
    /* .get_tensor    = */ buffer_get_tensor,
    /* .cpy_tensor    = */ buffer_cpy_tensor,
    /* .clear         = */ buffer_clear,
    /* .reset         = */ nullptr,
};

// ---------------------------------------------------------------------------------------------
// device buffer type
// ---------------------------------------------------------------------------------------------
struct b200_buft_ctx {
    int device;
    std::string name;
};

const char * buft_get_name(lm_ggml_backend_buffer_type_t buft) { return ((b200_buft_ctx *) buft->context)->name.c_str(); }

lm_ggml_backend_buffer_t buft_alloc_buffer(lm_ggml_backend_buffer_type_t buft, size_t size) {
    b200_buft_ctx * bc = (b200_buft_ctx *) buft->context;
    device_guard g(bc->device);
    b200_buffer_ctx * ctx = new b200_buffer_ctx;
    ctx->device = bc->device;
    const size_t bytes = std::max<size_t>(size, 1);
    cudaError_t e = cudaMalloc(&ctx->base, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        B200_LOG_ERROR("ggml-b200: allocating %.2f MiB on device %d failed: %s\n", bytes / 1048576.0, bc->device, cudaGetErrorString(e));
        ctx->base = nullptr;
        delete ctx;
        return nullptr;  // the caller reports LM_GGML_STATUS_ALLOC_FAILED / fails the model load
    }
    return lm_ggml_backend_buffer_init(buft, b200_buffer_iface, ctx, size);
}

size_t buft_get_alignment(lm_ggml_backend_buffer_type_t) { return B200_ALIGNMENT; }

size_t buft_get_alloc_size(lm_ggml_backend_buffer_type_t, const lm_ggml_tensor * tensor) {
    size_t size = lm_ggml_nbytes(tensor);
    if (tensor_is_tiled(tensor)) {
        // rows padded to 16 and blocks to 4 in the tiled layout
        const size_t tiled = b200_weight_bytes(tensor->type, tensor->ne[0], tensor_rows(tensor));
        size = std::max(size, tiled);
    }
    return size;
}

bool buft_is_host(lm_ggml_backend_buffer_type_t) { return false; }

const lm_ggml_backend_buffer_type_i b200_buft_iface = {
    /* .get_name       = */ buft_get_name,
    /* .alloc_buffer   = */ buft_alloc_buffer,
    /* .get_alignment  = */ buft_get_alignment,
    /* .get_max_size   = */ nullptr,
    /* .get_alloc_size = */ buft_get_alloc_size,
    /* .is_host        = */ buft_is_host,
};

// ---------------------------------------------------------------------------------------------
// pinned host buffer type: what the context uses for graph inputs and the logits it reads back
// (cactus/llama-context.cpp:199-206, 1193-1199)
// ---------------------------------------------------------------------------------------------
const char * host_buft_get_name(lm_ggml_backend_buffer_type_t) { return LM_GGML_B200_NAME "_Host"; }

void host_buffer_free(lm_ggml_backend_buffer_t buffer) { cudaFreeHost(buffer->context); }

lm_ggml_backend_buffer_t host_buft_alloc_buffer(lm_ggml_backend_buffer_type_t buft, size_t size) {
    void * ptr = nullptr;
    cudaError_t e = cudaMallocHost(&ptr, std::max<size_t>(size, 1));
    if (e != cudaSuccess) {
        cudaGetLastError();
        // fall back to pageable memory of the CPU buffer type, as the caller would do without a host type
        return lm_ggml_backend_buft_alloc_buffer(lm_ggml_backend_cpu_buffer_type(), size);
    }
    lm_ggml_backend_buffer_t buffer = lm_ggml_backend_cpu_buffer_from_ptr(ptr, size);
    buffer->buft = buft;
    buffer->iface.free_buffer = host_buffer_free;
    return buffer;
}

size_t host_buft_get_alignment(lm_ggml_backend_buffer_type_t) { return 64; }
bool host_buft_is_host(lm_ggml_backend_buffer_type_t) { return true; }

const lm_ggml_backend_buffer_type_i b200_host_buft_iface = {
    /* .get_name       = */ host_buft_get_name,
    /* .alloc_buffer   = */ host_buft_alloc_buffer,
    /* .get_alignment  = */ host_buft_get_alignment,
    /* .get_max_size   = */ nullptr,
    /* .get_alloc_size = */ nullptr,
    /* .is_host        = */ host_buft_is_host,
};

bool buft_is_b200(lm_ggml_backend_buffer_type_t buft) { return buft && buft->iface.get_name == buft_get_name; }
bool buft_is_b200_host(lm_ggml_backend_buffer_type_t buft) { return buft && buft->iface.get_name == host_buft_get_name; }

// ---------------------------------------------------------------------------------------------
// split buffer type: the rows of a quantised weight matrix spread over the devices
// (lm_ggml_backend_split_buffer_type_t, cactus/ggml-backend.h:188; the loader asks for it by name for
// LLAMA_SPLIT_MODE_ROW, cactus/llama-model.cpp:333-356).  Device i holds rows [row0[i], row0[i+1]) as a T16 weight of
// its own; MUL_MAT on the main device's backend lets every device multiply its rows and store them straight into the
// main device's dst over NVLink (compute_mul_mat_split).  Nothing else can read such a tensor: supports_op says so
// and the loader then takes the next buffer type of its list (cactus/llama-model.cpp:262-275).
// ---------------------------------------------------------------------------------------------
struct b200_split_buft_ctx {
    int main_device;
    int n_dev;
    float cum[LM_GGML_B200_MAX_DEVICES + 1];   // cumulative share of the rows: device i owns [cum[i], cum[i+1])
    std::string name;
};

struct b200_split_tensor {   // tensor->extra of a tensor in a split buffer
    int n_dev = 0;
    int64_t row0[LM_GGML_B200_MAX_DEVICES + 1] = {0};
    void * data[LM_GGML_B200_MAX_DEVICES] = {nullptr};
};

struct b200_split_buffer_ctx {
    std::vector<b200_split_tensor *> tensors;
    ~b200_split_buffer_ctx() {
        for (b200_split_tensor * t : tensors) {
            for (int i = 0; i < t->n_dev; ++i) {
                if (!t->data[i]) continue;
                device_guard g(i);
                cudaFree(t->data[i]);
            }
            delete t;
        }
    }
};

// rows of device i: cut on multiples of 128 rows (the row group of the tensor-core kernel), the last device takes the rest
void split_rows(const b200_split_buft_ctx * bc, int64_t M, int64_t * row0) {
    row0[0] = 0;
    for (int i = 1; i < bc->n_dev; ++i) {
        int64_t r = (int64_t) ((double) M * bc->cum[i]) / 128 * 128;
        row0[i] = std::min(M, std::max(r, row0[i - 1]));
    }
    row0[bc->n_dev] = M;
}

const char * split_buft_get_name(lm_ggml_backend_buffer_type_t buft) { return ((b200_split_buft_ctx *) buft->context)->name.c_str(); }
bool buft_is_b200_split(lm_ggml_backend_buffer_type_t buft) { return buft && buft->iface.get_name == split_buft_get_name; }

void split_buffer_free(lm_ggml_backend_buffer_t buffer) { delete (b200_split_buffer_ctx *) buffer->context; }
void * split_buffer_get_base(lm_ggml_backend_buffer_t) { return (void *) 0x1000; }   // never dereferenced: the data hangs off tensor->extra

lm_ggml_status split_buffer_init_tensor(lm_ggml_backend_buffer_t buffer, lm_ggml_tensor * tensor) {
    LM_GGML_ASSERT(tensor->view_src == nullptr && "views of split tensors are not supported");
    LM_GGML_ASSERT(is_tiled_type(tensor->type) && tensor->ne[0] % 32 == 0 && tensor->ne[2] == 1 && tensor->ne[3] == 1);
    b200_split_buffer_ctx * ctx = (b200_split_buffer_ctx *) buffer->context;
    const b200_split_buft_ctx * bc = (const b200_split_buft_ctx *) buffer->buft->context;
    b200_split_tensor * st = new b200_split_tensor;
    st->n_dev = bc->n_dev;
    split_rows(bc, tensor->ne[1], st->row0);
    ctx->tensors.push_back(st);
    for (int i = 0; i < bc->n_dev; ++i) {
        const int64_t rows = st->row0[i + 1] - st->row0[i];
        if (rows <= 0) continue;
        device_guard g(i);
        const size_t bytes = b200_weight_bytes(tensor->type, tensor->ne[0], rows);
        if (!cuda_ok(cudaMalloc(&st->data[i], bytes), "cudaMalloc(split weight)")) return LM_GGML_STATUS_ALLOC_FAILED;
    }
    tensor->extra = st;
    return LM_GGML_STATUS_SUCCESS;
}

// host block stream <-> the per-device T16 weights, staged through a bounce buffer on each device
bool split_transfer(const lm_ggml_tensor * tensor, void * host, bool to_device) {
    const b200_split_tensor * st = (const b200_split_tensor *) tensor->extra;
    const int64_t K = tensor->ne[0];
    const size_t rb = (size_t) (K / 32) * block_bytes(tensor->type);
    const int64_t max_rows = std::max<int64_t>(16, (int64_t) (B200_STAGE_BYTES / rb) / 16 * 16);
    for (int i = 0; i < st->n_dev; ++i) {
        const int64_t Mi = st->row0[i + 1] - st->row0[i];
        if (Mi <= 0) continue;
        device_guard g(i);
        void * stage = nullptr;
        if (!cuda_ok(cudaMalloc(&stage, (size_t) std::min(Mi, max_rows) * rb), "cudaMalloc(stage)")) return false;
        bool ok = true;
        for (int64_t r = 0; r < Mi && ok; r += max_rows) {
            const int64_t rows = std::min(max_rows, Mi - r);
            uint8_t * hp = (uint8_t *) host + (size_t) (st->row0[i] + r) * rb;
            if (to_device) {
                ok = cuda_ok(cudaMemcpy(stage, hp, (size_t) rows * rb, cudaMemcpyHostToDevice), "cudaMemcpy H2D") &&
                     b200_weight_upload(tensor->type, K, Mi, stage, st->data[i], r, rows, nullptr) == B200_OK &&
                     cuda_ok(cudaStreamSynchronize(nullptr), "sync after upload");
            } else {
                ok = b200_weight_download(tensor->type, K, Mi, st->data[i], stage, r, rows, nullptr) == B200_OK &&
                     cuda_ok(cudaMemcpy(hp, stage, (size_t) rows * rb, cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
            }
        }
        cudaFree(stage);
        if (!ok) {
            B200_LOG_ERROR("ggml-b200: split tensor %s transfer on device %d failed: %s\n", tensor->name, i, b200_last_error());
            return false;
        }
    }
    return true;
}

void split_buffer_set_tensor(lm_ggml_backend_buffer_t, lm_ggml_tensor * tensor, const void * data, size_t offset, size_t size) {
    // whole tensors only, as the loader writes them (cactus/llama-model-loader.cpp:1034)
    LM_GGML_ASSERT(offset == 0 && size == lm_ggml_nbytes(tensor));
    LM_GGML_ASSERT(split_transfer(tensor, const_cast<void *>(data), true));
}

void split_buffer_get_tensor(lm_ggml_backend_buffer_t, const lm_ggml_tensor * tensor, void * data, size_t offset, size_t size) {
    LM_GGML_ASSERT(offset == 0 && size == lm_ggml_nbytes(tensor));
    LM_GGML_ASSERT(split_transfer(tensor, data, false));
}

void split_buffer_clear(lm_ggml_backend_buffer_t, uint8_t) {}

const lm_ggml_backend_buffer_i b200_split_buffer_iface = {
    /* .free_buffer   = */ split_buffer_free,
    /* .get_base      = */ split_buffer_get_base,
    /* .init_tensor   = */ split_buffer_init_tensor,
    /* .memset_tensor = */ nullptr,
    /* .set_tensor    = */ split_buffer_set_tensor,
    /* .get_tensor    = */ split_buffer_get_tensor,
    /* .cpy_tensor    = */ nullptr,
    /* .clear         = */ split_buffer_clear,
    /* .reset         = */ nullptr,
};

lm_ggml_backend_buffer_t split_buft_alloc_buffer(lm_ggml_backend_buffer_type_t buft, size_t size) {
    // the device memory is allocated tensor by tensor in init_tensor, where the row ranges are known
    return lm_ggml_backend_buffer_init(buft, b200_split_buffer_iface, new b200_split_buffer_ctx, size);
}

size_t split_buft_get_alloc_size(lm_ggml_backend_buffer_type_t buft, const lm_ggml_tensor * tensor) {
    size_t total = lm_ggml_nbytes(tensor);
    if (is_tiled_type(tensor->type) && tensor->ne[0] % 32 == 0) {
        const b200_split_buft_ctx * bc = (const b200_split_buft_ctx *) buft->context;
        int64_t row0[LM_GGML_B200_MAX_DEVICES + 1];
        split_rows(bc, tensor->ne[1], row0);
        size_t sum = 0;
        for (int i = 0; i < bc->n_dev; ++i)
            if (row0[i + 1] > row0[i]) sum += b200_weight_bytes(tensor->type, tensor->ne[0], row0[i + 1] - row0[i]);
        total = std::max(total, sum);
    }
    return total;
}

const lm_ggml_backend_buffer_type_i b200_split_buft_iface = {
    /* .get_name       = */ split_buft_get_name,
    /* .alloc_buffer   = */ split_buft_alloc_buffer,
    /* .get_alignment  = */ buft_get_alignment,
    /* .get_max_size   = */ nullptr,
    /* .get_alloc_size = */ split_buft_get_alloc_size,
    /* .is_host        = */ buft_is_host,
};

// ---------------------------------------------------------------------------------------------
// backend (one CUDA stream) and its scratch memory
// ---------------------------------------------------------------------------------------------
// While a node list is being recorded into a CUDA graph nothing may synchronise or allocate: a scratch block that would
// have to grow fails the recording instead (the list then runs directly, which grows the block, and is recorded next time).
thread_local bool t_recording = false, t_recording_failed = false;

struct scratch_buf {
    void * ptr = nullptr;
    size_t bytes = 0;
    // grows when needed; growing synchronises the stream first because earlier kernels may still use the old block
    void * get(size_t need, cudaStream_t st) {
        if (need <= bytes) return ptr;
        if (t_recording) {
            t_recording_failed = true;
            return nullptr;
        }
        if (ptr) {
            cudaStreamSynchronize(st);
            cudaFree(ptr);
            ptr = nullptr;
            bytes = 0;
        }
        const size_t want = (need + (1u << 20)) / (1u << 20) * (1u << 20);
        if (!cuda_ok(cudaMalloc(&ptr, want), "cudaMalloc(scratch)")) {
            ptr = nullptr;
            return nullptr;
        }
        bytes = want;
        return ptr;
    }
    void release() {
        if (ptr) cudaFree(ptr);
        ptr = nullptr;
        bytes = 0;
    }
};

// what a backend keeps on another device for MUL_MAT on split weights: a stream there, the copy of the quantised
// activations, the kernel workspace, and the event the main stream waits for
struct split_peer {
    bool ready = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t done = nullptr;
    scratch_buf act, workspace;
    const lm_ggml_tensor * act_src = nullptr;
};

struct rope_store_state {
    const lm_ggml_tensor * cpy_k = nullptr;   // the K store that the kernel of the preceding ROPE has already done
};

struct b200_backend_ctx {
    int device;
    std::string name;
    cudaStream_t stream = nullptr;
    scratch_buf act, workspace, fa_scratch, mask_index;
    split_peer peers[LM_GGML_B200_MAX_DEVICES];
    cudaEvent_t ev_act = nullptr;   // recorded on `stream` when the quantised activations are ready
    // what the scratch currently holds, valid inside one graph_compute
    const lm_ggml_tensor * act_src = nullptr;
    const lm_ggml_tensor * index_mask = nullptr;
    lm_ggml_abort_callback abort_cb = nullptr;
    void * abort_cb_data = nullptr;
    int q8_variant = B200_Q8_AVX2;
    bool fa_parity = false;  // B200_FA_PARITY=1: the reference-order attention kernel (validation)
    bool fuse = true;        // B200_FUSE=0: one kernel per node (except the norm and silu pairs)
    bool stack = true;       // B200_STACK=0: adjacent products on the same activations run one by one
    rope_store_state rs;
    bool timing = false;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    lm_ggml_b200_stats stats = {};
    // CUDA-graph replay of node lists (graph_cache below)
    bool graphs = true;      // B200_GRAPHS=0: every node list is launched kernel by kernel
    bool warmed = false;     // one node list has run directly (lazy per-device set-up of the kernel library is done)
    struct graph_entry {
        uint64_t h1 = 0, h2 = 0, stamp = 0;
        int n_nodes = 0;
        cudaGraphExec_t exec = nullptr;
        lm_ggml_b200_stats delta = {};               // what one run adds to the counters
        uint64_t rope_stores = 0, add_norms = 0, masks = 0;
    } cache[4];
    uint64_t stamp = 0, last_h1 = 0, last_h2 = 0;
    int cold_records = 0;    // recordings since the last replay
    cudaStream_t cap_stream = nullptr;   // recordings are captured here; nothing ever runs on it
    std::vector<uint64_t> dbg_trail;
    // rows of the KV cache that the ubatch's K / V stores write: the one thing that moves from step to step in a decode
    // graph.  The stores take (cache tensor, list of rows); the lists sit in device memory and are refreshed before every run.
    int32_t * slots_dev = nullptr;
    size_t slots_cap = 0;
    std::vector<int32_t> slots_host;
    std::vector<std::pair<const lm_ggml_tensor *, int>> slot_of;   // CPY node -> offset of its row list
    std::vector<int64_t> slot_first;                                // first cache row of each list
    std::vector<uint8_t> node_done;                                 // per node of the list being run: it ran ahead of its place
    scratch_buf parked[2];                                          // results of products that ran ahead but whose destination was not free yet
    struct parked_result { int node, block; size_t stride; };      // stride: the row stride of the launch it ran in
    std::vector<parked_result> parked_for;
};

lm_ggml_guid_t b200_guid() {
    static lm_ggml_guid guid = {0xb2, 0x00, 0x5a, 0x10, 0x0a, 0x47, 0x47, 0x4d, 0x4c, 0x2d, 0x62, 0x32, 0x30, 0x30, 0x00, 0x01};
    return &guid;
}

const char * backend_get_name(lm_ggml_backend_t backend) { return ((b200_backend_ctx *) backend->context)->name.c_str(); }

void backend_free(lm_ggml_backend_t backend) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    {
        device_guard g(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        ctx->act.release();
        ctx->workspace.release();
        ctx->fa_scratch.release();
        ctx->mask_index.release();
        ctx->parked[0].release();
        ctx->parked[1].release();
        if (ctx->ev0) cudaEventDestroy(ctx->ev0);
        if (ctx->ev1) cudaEventDestroy(ctx->ev1);
        if (ctx->ev_act) cudaEventDestroy(ctx->ev_act);
        for (auto & e : ctx->cache) if (e.exec) cudaGraphExecDestroy(e.exec);
        if (ctx->cap_stream) cudaStreamDestroy(ctx->cap_stream);
        if (ctx->slots_dev) cudaFree(ctx->slots_dev);
        cudaStreamDestroy(ctx->stream);
    }
    for (int i = 0; i < LM_GGML_B200_MAX_DEVICES; ++i) {
        split_peer & p = ctx->peers[i];
        if (!p.ready) continue;
        device_guard g(i);
        cudaStreamSynchronize(p.stream);
        p.act.release();
        p.workspace.release();
        cudaEventDestroy(p.done);
        cudaStreamDestroy(p.stream);
    }
    delete ctx;
    delete backend;
}

void backend_synchronize(lm_ggml_backend_t backend) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    device_guard g(ctx->device);
    cuda_ok(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
}

void backend_set_tensor_async(lm_ggml_backend_t backend, lm_ggml_tensor * tensor, const void * data, size_t offset, size_t size) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    lm_ggml_backend_buffer_t buf = tensor->view_src ? tensor->view_src->buffer : tensor->buffer;
    LM_GGML_ASSERT(buf && buft_is_b200(buf->buft) && "tensor is not in a B200 buffer");
    device_guard g(ctx->device);
    if (tensor_is_tiled(tensor)) {
        cudaStreamSynchronize(ctx->stream);
        buffer_set_tensor(buf, tensor, data, offset, size);
        return;
    }
    LM_GGML_ASSERT(cuda_ok(cudaMemcpyAsync((char *) tensor->data + offset, data, size, cudaMemcpyHostToDevice, ctx->stream), "cudaMemcpyAsync H2D"));
}

void backend_get_tensor_async(lm_ggml_backend_t backend, const lm_ggml_tensor * tensor, void * data, size_t offset, size_t size) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    lm_ggml_backend_buffer_t buf = tensor->view_src ? tensor->view_src->buffer : tensor->buffer;
    LM_GGML_ASSERT(buf && buft_is_b200(buf->buft) && "tensor is not in a B200 buffer");
    device_guard g(ctx->device);
    if (tensor_is_tiled(tensor)) {
        cudaStreamSynchronize(ctx->stream);
        buffer_get_tensor(buf, tensor, data, offset, size);
        return;
    }
    LM_GGML_ASSERT(cuda_ok(cudaMemcpyAsync(data, (const char *) tensor->data + offset, size, cudaMemcpyDeviceToHost, ctx->stream), "cudaMemcpyAsync D2H"));
}

bool backend_cpy_tensor_async(lm_ggml_backend_t backend_src, lm_ggml_backend_t backend_dst, const lm_ggml_tensor * src, lm_ggml_tensor * dst) {
    if (!lm_ggml_backend_is_b200(backend_src) || !lm_ggml_backend_is_b200(backend_dst)) return false;
    lm_ggml_backend_buffer_t sbuf = src->view_src ? src->view_src->buffer : src->buffer;
    lm_ggml_backend_buffer_t dbuf = dst->view_src ? dst->view_src->buffer : dst->buffer;
    if (!sbuf || !dbuf || !buft_is_b200(sbuf->buft) || !buft_is_b200(dbuf->buft)) return false;
    if (is_tiled_type(src->type) || !lm_ggml_is_contiguous(src) || !lm_ggml_is_contiguous(dst) || lm_ggml_nbytes(src) != lm_ggml_nbytes(dst)) return false;
    b200_backend_ctx * sctx = (b200_backend_ctx *) backend_src->context;
    b200_backend_ctx * dctx = (b200_backend_ctx *) backend_dst->context;
    device_guard g(sctx->device);
    // issue on the source stream, then make the destination stream wait for it
    cudaError_t e = (sctx->device == dctx->device)
        ? cudaMemcpyAsync(dst->data, src->data, lm_ggml_nbytes(src), cudaMemcpyDeviceToDevice, sctx->stream)
        : cudaMemcpyPeerAsync(dst->data, dctx->device, src->data, sctx->device, lm_ggml_nbytes(src), sctx->stream);
    if (!cuda_ok(e, "cudaMemcpyAsync D2D")) return false;
    if (backend_src != backend_dst) {
        cudaEvent_t ev;
        if (!cuda_ok(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate")) return false;
        cudaEventRecord(ev, sctx->stream);
        device_guard g2(dctx->device);
        cudaStreamWaitEvent(dctx->stream, ev, 0);
        cudaEventDestroy(ev);
    }
    return true;
}

// ---------------------------------------------------------------------------------------------
// op support and dispatch
// ---------------------------------------------------------------------------------------------
bool f32_rows(const lm_ggml_tensor * t) { return t->type == LM_GGML_TYPE_F32 && t->nb[0] == sizeof(float); }

// higher dimensions collapse onto dimension 1 (rows are evenly strided)
bool rows_collapsible(const lm_ggml_tensor * t) {
    return t->nb[2] == t->nb[1] * (size_t) t->ne[1] && t->nb[3] == t->nb[2] * (size_t) t->ne[2];
}

bool weight_ok(const lm_ggml_tensor * w) {
    // the tensor itself must be the tiled tensor (not a view of one) and two-dimensional
    return w && is_tiled_type(w->type) && w->view_src == nullptr && w->ne[2] == 1 && w->ne[3] == 1 && w->ne[0] % 32 == 0 &&
           w->buffer && buft_is_b200(w->buffer->buft);
}

// a weight in a split buffer: usable by MUL_MAT only (the probe of the loader hangs a dummy buffer of the split type on
// the tensor, cactus/llama-model.cpp:246-251, so only the buffer type may be looked at here)
bool split_weight_ok(const lm_ggml_tensor * w) {
    return w && is_tiled_type(w->type) && w->view_src == nullptr && w->ne[2] == 1 && w->ne[3] == 1 && w->ne[0] % 32 == 0 &&
           w->buffer && buft_is_b200_split(w->buffer->buft);
}

bool supports_mul_mat(const lm_ggml_tensor * op) {
    const lm_ggml_tensor * a = op->src[0], * b = op->src[1];
    if ((!weight_ok(a) && !split_weight_ok(a)) || !b) return false;
    if (!f32_rows(b) || b->ne[0] != a->ne[0] || !rows_collapsible(b)) return false;
    return op->type == LM_GGML_TYPE_F32 && lm_ggml_is_contiguous(op);
}

bool supports_flash_attn(const lm_ggml_tensor * op) {
    const lm_ggml_tensor * q = op->src[0], * k = op->src[1], * v = op->src[2], * m = op->src[3];
    if (!q || !k || !v) return false;
    if (q->type != LM_GGML_TYPE_F32 || k->type != LM_GGML_TYPE_F16 || v->type != LM_GGML_TYPE_F16) return false;
    if (q->nb[0] != 4 || k->nb[0] != 2 || v->nb[0] != 2) return false;
    const int64_t D = q->ne[0];
    if ((D != 64 && D != 128) || k->ne[0] != D || v->ne[0] != D) return false;
    if (q->ne[3] != 1 || k->ne[3] != 1 || v->ne[3] != 1) return false;
    if (k->ne[2] != v->ne[2] || k->ne[1] != v->ne[1] || q->ne[2] % k->ne[2] != 0) return false;
    if (k->nb[1] % 16 || k->nb[2] % 16 || v->nb[1] % 16 || v->nb[2] % 16) return false;
    if (m && (m->type != LM_GGML_TYPE_F16 || m->nb[0] != 2 || m->ne[0] < k->ne[1] || m->ne[1] < q->ne[1] || m->ne[2] != 1 || m->ne[3] != 1)) return false;
    if (op->src[4]) return false;  // no attention sinks in this runtime's graphs
    return op->type == LM_GGML_TYPE_F32 && lm_ggml_is_contiguous(op);
}

bool supports_cpy(const lm_ggml_tensor * src, const lm_ggml_tensor * dst) {
    if (src && src->type == LM_GGML_TYPE_F16 && dst->type == LM_GGML_TYPE_F16) {   // cache defragmentation moves
        if (lm_ggml_nelements(src) != lm_ggml_nelements(dst)) return false;
        if (lm_ggml_is_contiguous(src) && lm_ggml_is_contiguous(dst)) return true;
        return lm_ggml_are_same_shape(src, dst) && src->nb[0] == 2 && dst->nb[0] == 2;
    }
    if (!src || src->type != LM_GGML_TYPE_F32) return false;
    if (dst->type != LM_GGML_TYPE_F32 && dst->type != LM_GGML_TYPE_F16) return false;
    if (lm_ggml_nelements(src) != lm_ggml_nelements(dst)) return false;
    if (lm_ggml_is_contiguous(src) && lm_ggml_is_contiguous(dst)) return true;
    return lm_ggml_are_same_shape(src, dst) && src->nb[0] == 4 && dst->nb[0] == lm_ggml_type_size(dst->type);
}

bool supports_binary(const lm_ggml_tensor * op) {
    const lm_ggml_tensor * a = op->src[0], * b = op->src[1];
    if (!a || !b || a->type != LM_GGML_TYPE_F32 || b->type != LM_GGML_TYPE_F32 || op->type != LM_GGML_TYPE_F32) return false;
    if (!lm_ggml_is_contiguous(a) || !lm_ggml_is_contiguous(b) || !lm_ggml_is_contiguous(op) || !lm_ggml_are_same_shape(a, op)) return false;
    return lm_ggml_are_same_shape(a, b) || (b->ne[0] == a->ne[0] && lm_ggml_nelements(b) == b->ne[0]);
}

bool supports_rope(const lm_ggml_tensor * op) {
    const lm_ggml_tensor * a = op->src[0], * pos = op->src[1], * ff = op->src[2];
    if (!a || !pos || pos->type != LM_GGML_TYPE_I32) return false;
    const bool f32 = f32_rows(a) && op->type == LM_GGML_TYPE_F32 && op->nb[0] == 4;
    // f16 in, f16 out: the K-shift of the cache (llama_kv_cache_unified::build_rope_shift)
    const bool f16 = a->type == LM_GGML_TYPE_F16 && op->type == LM_GGML_TYPE_F16 && a->nb[0] == 2 && op->nb[0] == 2 && a->nb[1] % 4 == 0 &&
                     a->nb[2] % 4 == 0 && op->nb[1] % 4 == 0 && op->nb[2] % 4 == 0;
    if (!f32 && !f16) return false;
    const int32_t * p = (const int32_t *) op->op_params;
    const int n_dims = p[1], mode = p[2];
    float ext_factor;
    memcpy(&ext_factor, p + 7, sizeof(float));
    if (mode != 0 || ext_factor != 0.0f || n_dims <= 0 || n_dims > a->ne[0] || (n_dims & 1)) return false;
    if (ff && (ff->type != LM_GGML_TYPE_F32 || ff->ne[0] < n_dims / 2)) return false;
    return a->ne[3] == 1 && lm_ggml_are_same_shape(a, op);
}

bool b200_supports_op(const lm_ggml_tensor * op) {
    switch (op->op) {
        case LM_GGML_OP_NONE:
        case LM_GGML_OP_RESHAPE:
        case LM_GGML_OP_VIEW:
        case LM_GGML_OP_PERMUTE:
        case LM_GGML_OP_TRANSPOSE:
            return true;
        case LM_GGML_OP_MUL_MAT:
            return supports_mul_mat(op);
        case LM_GGML_OP_FLASH_ATTN_EXT:
            return supports_flash_attn(op);
        case LM_GGML_OP_RMS_NORM:
            return op->src[0] && f32_rows(op->src[0]) && op->type == LM_GGML_TYPE_F32 && lm_ggml_is_contiguous(op) && rows_collapsible(op->src[0]);
        case LM_GGML_OP_ADD:
        case LM_GGML_OP_MUL:
            return supports_binary(op);
        case LM_GGML_OP_UNARY:
            return lm_ggml_get_unary_op(op) == LM_GGML_UNARY_OP_SILU && op->src[0] && op->src[0]->type == LM_GGML_TYPE_F32 &&
                   lm_ggml_is_contiguous(op->src[0]) && lm_ggml_is_contiguous(op) && op->type == LM_GGML_TYPE_F32;
        case LM_GGML_OP_ROPE:
            return supports_rope(op);
        case LM_GGML_OP_CPY:
            return supports_cpy(op->src[0], op->src[1] ? op->src[1] : op);
        case LM_GGML_OP_CONT:
        case LM_GGML_OP_DUP:
            return supports_cpy(op->src[0], op);
        case LM_GGML_OP_GET_ROWS: {
            const lm_ggml_tensor * a = op->src[0], * ids = op->src[1];
            if (!a || !ids || ids->type != LM_GGML_TYPE_I32 || !lm_ggml_is_contiguous(ids) || op->type != LM_GGML_TYPE_F32 || !lm_ggml_is_contiguous(op)) return false;
            if (a->ne[2] != 1 || a->ne[3] != 1) return false;
            return f32_rows(a) || weight_ok(a);
        }
        default:
            return false;
    }
}

#define B200_CHECK(call)                                                           \
    do {                                                                           \
        if ((call) != B200_OK) {                                                   \
            B200_LOG_ERROR("ggml-b200: %s: %s\n", lm_ggml_op_name(node->op), b200_last_error()); \
            return LM_GGML_STATUS_FAILED;                                             \
        }                                                                          \
    } while (0)

bool only_user_is(const lm_ggml_cgraph * g, const lm_ggml_tensor * t, const lm_ggml_tensor * user) {
    for (int i = 0; i < g->n_nodes; ++i) {
        const lm_ggml_tensor * n = g->nodes[i];
        if (n == user) continue;
        for (int s = 0; s < LM_GGML_MAX_SRC; ++s) {
            if (n->src[s] == t) return false;
            if (n->src[s] && n->src[s]->view_src == t) return false;
        }
        if (n->view_src == t) return false;
    }
    return !(t->flags & LM_GGML_TENSOR_FLAG_OUTPUT);
}

lm_ggml_status compute_cpy(b200_backend_ctx * ctx, const lm_ggml_tensor * node, const lm_ggml_tensor * src, const lm_ggml_tensor * dst) {
    const bool to_f16 = dst->type == LM_GGML_TYPE_F16, from_f16 = src->type == LM_GGML_TYPE_F16;
    auto run = [&](const void * s, int64_t snb, void * d, int64_t dnb, int64_t n, int64_t rows) {
        if (from_f16) return b200_cpy_f16_f16(s, snb, d, dnb, n, rows, ctx->stream);
        return to_f16 ? b200_cpy_f32_f16((const float *) s, snb, d, dnb, n, rows, ctx->stream)
                      : b200_cpy_f32_f32((const float *) s, snb, (float *) d, dnb, n, rows, ctx->stream);
    };
    if (lm_ggml_is_contiguous(src) && lm_ggml_is_contiguous(dst)) {
        const int64_t n = lm_ggml_nelements(src);
        B200_CHECK(run(src->data, n * (int64_t) lm_ggml_type_size(src->type), dst->data, n * (int64_t) lm_ggml_type_size(dst->type), n, 1));
        return LM_GGML_STATUS_SUCCESS;
    }
    for (int64_t i3 = 0; i3 < src->ne[3]; ++i3)
        for (int64_t i2 = 0; i2 < src->ne[2]; ++i2)
            B200_CHECK(run((const char *) src->data + i2 * src->nb[2] + i3 * src->nb[3], src->nb[1],
                           (char *) dst->data + i2 * dst->nb[2] + i3 * dst->nb[3], dst->nb[1], src->ne[0], src->ne[1]));
    return LM_GGML_STATUS_SUCCESS;
}

// MUL_MAT with the weight rows spread over the devices (split buffer).  The activations are quantised once on this
// backend's device; every other device gets a copy over NVLink, multiplies its rows and stores them straight into
// this device's dst (plain peer stores from the kernel's write-back: dst columns [row0[i], row0[i+1]) of every
// activation row), all in stream order: the peers wait for the event behind the quantiser, this stream waits for
// theirs.  Only this device needs the result -- the next node runs here (cactus/llama-model.cpp:342-351 makes the
// layer's device the main device of its split buffer).
std::atomic<uint64_t> g_split_mul_mats{0};
// CUDA-event time of every graph_compute of every backend of the process (B200_TIMING=1), for drivers that cannot reach
// the backends a llama_context owns
std::atomic<uint64_t> g_rope_store_groups{0}, g_add_norm_groups{0};   // fused groups of all backends of the process
std::atomic<uint64_t> g_stacked_products{0};                          // launches that multiplied several weights (recordings included)
std::mutex g_totals_mu;
double g_total_device_ms = 0.0;
uint64_t g_total_timed_graphs = 0;

bool split_peer_init(b200_backend_ctx * ctx, int dev) {
    split_peer & p = ctx->peers[dev];
    if (p.ready) return true;
    int can = 0;
    cudaDeviceCanAccessPeer(&can, dev, ctx->device);
    if (!can) {
        B200_LOG_ERROR("ggml-b200: device %d cannot store into device %d: no peer access\n", dev, ctx->device);
        return false;
    }
    device_guard g(dev);
    cudaError_t e = cudaDeviceEnablePeerAccess(ctx->device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        e = cudaSuccess;
    }
    if (!cuda_ok(e, "cudaDeviceEnablePeerAccess")) return false;
    if (!cuda_ok(cudaStreamCreateWithFlags(&p.stream, cudaStreamNonBlocking), "cudaStreamCreate(peer)")) return false;
    if (!cuda_ok(cudaEventCreateWithFlags(&p.done, cudaEventDisableTiming), "cudaEventCreate(peer)")) return false;
    p.ready = true;
    return true;
}

lm_ggml_status compute_mul_mat_split(b200_backend_ctx * ctx, lm_ggml_tensor * node) {
    const lm_ggml_tensor * s0 = node->src[0], * s1 = node->src[1];
    const b200_split_tensor * sw = (const b200_split_tensor *) s0->extra;
    LM_GGML_ASSERT(sw != nullptr);
    cudaStream_t st = ctx->stream;
    const int64_t K = s0->ne[0], N = s1->ne[1] * s1->ne[2] * s1->ne[3];
    const size_t ab = b200_act_bytes(K, N);
    if (ctx->act_src != s1) {
        void * act = ctx->act.get(ab, st);
        if (!act) return LM_GGML_STATUS_ALLOC_FAILED;
        B200_CHECK(b200_quantize_activations((const float *) s1->data, s1->nb[1], K, N, act, ctx->act.bytes, ctx->q8_variant, st));
        ctx->act_src = s1;
        ctx->stats.act_quantized++;
        for (split_peer & p : ctx->peers) p.act_src = nullptr;
    }
    if (!ctx->ev_act && !cuda_ok(cudaEventCreateWithFlags(&ctx->ev_act, cudaEventDisableTiming), "cudaEventCreate")) return LM_GGML_STATUS_FAILED;
    if (!cuda_ok(cudaEventRecord(ctx->ev_act, st), "cudaEventRecord")) return LM_GGML_STATUS_FAILED;
    bool waited[LM_GGML_B200_MAX_DEVICES] = {false};
    for (int i = 0; i < sw->n_dev; ++i) {
        const int64_t Mi = sw->row0[i + 1] - sw->row0[i];
        if (Mi <= 0) continue;
        float * dst = (float *) node->data + sw->row0[i];
        const size_t wb = b200_mul_mat_workspace_bytes(s0->type, K, Mi, N);
        if (i == ctx->device) {
            void * ws = wb ? ctx->workspace.get(wb, st) : nullptr;
            if (wb && !ws) return LM_GGML_STATUS_ALLOC_FAILED;
            B200_CHECK(b200_mul_mat_q_prequant(s0->type, sw->data[i], K, Mi, ctx->act.ptr, N, dst, node->nb[1], ws, ws ? ctx->workspace.bytes : 0, st));
            continue;
        }
        if (!split_peer_init(ctx, i)) return LM_GGML_STATUS_FAILED;
        split_peer & p = ctx->peers[i];
        device_guard g(i);
        if (!cuda_ok(cudaStreamWaitEvent(p.stream, ctx->ev_act, 0), "cudaStreamWaitEvent")) return LM_GGML_STATUS_FAILED;
        if (p.act_src != s1) {
            void * act = p.act.get(ab, p.stream);
            if (!act) return LM_GGML_STATUS_ALLOC_FAILED;
            if (!cuda_ok(cudaMemcpyPeerAsync(act, i, ctx->act.ptr, ctx->device, ab, p.stream), "cudaMemcpyPeerAsync")) return LM_GGML_STATUS_FAILED;
            p.act_src = s1;
        }
        void * ws = wb ? p.workspace.get(wb, p.stream) : nullptr;
        if (wb && !ws) return LM_GGML_STATUS_ALLOC_FAILED;
        B200_CHECK(b200_mul_mat_q_prequant(s0->type, sw->data[i], K, Mi, p.act.ptr, N, dst, node->nb[1], ws, ws ? p.workspace.bytes : 0, p.stream));
        if (!cuda_ok(cudaEventRecord(p.done, p.stream), "cudaEventRecord")) return LM_GGML_STATUS_FAILED;
        waited[i] = true;
    }
    for (int i = 0; i < sw->n_dev; ++i)
        if (waited[i] && !cuda_ok(cudaStreamWaitEvent(st, ctx->peers[i].done, 0), "cudaStreamWaitEvent")) return LM_GGML_STATUS_FAILED;
    ctx->stats.mul_mat++;
    g_split_mul_mats.fetch_add(1, std::memory_order_relaxed);
    return LM_GGML_STATUS_SUCCESS;
}

// A CPY that stores f32 rows as f16 into whole consecutive rows of a cache tensor (cpy_k / cpy_v,
// cactus/llama-kv-cache.cpp:617-656: the destination is a view of the layer's cache at the rows the ubatch was given).
// Such a store runs as "rows r[0..T) of the cache tensor", with the row numbers in device memory, so that its launch is the
// same for every position of the ubatch in the cache.
bool row_store(const lm_ggml_tensor * cpy, int64_t * rows, int64_t * row_elems, int64_t * first_row) {
    const lm_ggml_tensor * src = cpy->src[0], * dst = cpy->src[1];
    if (cpy->op != LM_GGML_OP_CPY || !src || !dst || !dst->view_src || src->type != LM_GGML_TYPE_F32 || dst->type != LM_GGML_TYPE_F16) return false;
    const lm_ggml_tensor * cache = dst->view_src;
    if (cache->type != LM_GGML_TYPE_F16 || !lm_ggml_is_contiguous(cache) || !lm_ggml_is_contiguous(dst) || !lm_ggml_is_contiguous(src)) return false;
    if (!cache->buffer || !buft_is_b200(cache->buffer->buft) || tensor_is_tiled(cache)) return false;
    const int64_t n = lm_ggml_nelements(dst), re = cache->ne[0];
    if (re <= 0 || n <= 0 || n % re || lm_ggml_nelements(src) != n || cache->nb[1] != (size_t) re * 2 || dst->view_offs % cache->nb[1]) return false;
    if (((uintptr_t) src->data % 4) || dst->data != (char *) cache->data + dst->view_offs) return false;
    *rows = n / re;
    *row_elems = re;
    *first_row = (int64_t) (dst->view_offs / cache->nb[1]);
    return true;
}

int slot_offset(const b200_backend_ctx * ctx, const lm_ggml_tensor * cpy) {
    for (const auto & e : ctx->slot_of) if (e.first == cpy) return e.second;
    return -1;
}

// finds the row stores of a node list, writes their row numbers to the device (in stream order, before the list runs)
bool prepare_row_lists(b200_backend_ctx * ctx, const lm_ggml_cgraph * g) {
    ctx->slot_of.clear();
    ctx->slots_host.clear();
    ctx->slot_first.clear();
    for (int i = 0; i < g->n_nodes; ++i) {
        int64_t rows, re, first;
        if (!row_store(g->nodes[i], &rows, &re, &first) || rows > (1 << 20)) continue;
        ctx->slot_of.emplace_back(g->nodes[i], (int) ctx->slots_host.size());
        ctx->slot_first.push_back(first);
        for (int64_t r = 0; r < rows; ++r) ctx->slots_host.push_back((int32_t) (first + r));
    }
    if (ctx->slots_host.empty()) return true;
    if (ctx->slots_host.size() > ctx->slots_cap) {
        cudaStreamSynchronize(ctx->stream);
        if (ctx->slots_dev) cudaFree(ctx->slots_dev);
        ctx->slots_dev = nullptr;
        ctx->slots_cap = 0;
        const size_t want = std::max<size_t>(4096, ctx->slots_host.size() * 2);
        if (!cuda_ok(cudaMalloc((void **) &ctx->slots_dev, want * sizeof(int32_t)), "cudaMalloc(row lists)")) {
            ctx->slot_of.clear();   // the stores fall back to their absolute addresses
            return false;
        }
        ctx->slots_cap = want;
    }
    // pageable source: the copy is staged before the call returns, so the vector may be reused
    if (!cuda_ok(cudaMemcpyAsync(ctx->slots_dev, ctx->slots_host.data(), ctx->slots_host.size() * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream),
                 "cudaMemcpyAsync(row lists)")) {
        ctx->slot_of.clear();
        return false;
    }
    return true;
}

const lm_ggml_tensor * through_views(const lm_ggml_tensor * t) {
    while (t && (t->op == LM_GGML_OP_RESHAPE || t->op == LM_GGML_OP_VIEW) && t->src[0]) t = t->src[0];
    return t;
}

// ROPE(k) and the CPY that stores the rotated k as f16 into the cache rows of the ubatch (cpy_k,
// cactus/llama-kv-cache.cpp:617-628) as one kernel, run in the place of the ROPE.  The store is only moved EARLIER: the
// rows it writes are read by nothing before the attention of the same layer.  (Moving a node LATER is not possible under
// ggml-alloc: the ROPE's source is handed to the next product as soon as the ROPE's place in the node order has passed, so
// ROPE(q) and the V store stay where they are.)  Needs: the rotated k feeds nothing but that store, which writes whole
// consecutive f16 rows of Hkv * D values.
bool rope_store_group(b200_backend_ctx * ctx, const lm_ggml_cgraph * g, int i) {
    const lm_ggml_tensor * rk = g->nodes[i];
    if (rk->src[0]->type != LM_GGML_TYPE_F32 || !lm_ggml_is_contiguous(rk) || !lm_ggml_is_contiguous(rk->src[0]) || rk->ne[3] != 1) return false;
    const lm_ggml_tensor * ck = nullptr;
    for (int j = i + 1; j < g->n_nodes && j < i + 24 && !ck; ++j) {
        const lm_ggml_tensor * n = g->nodes[j];
        if (n->op == LM_GGML_OP_FLASH_ATTN_EXT) return false;
        if (n->op == LM_GGML_OP_CPY && n->src[0] == rk) ck = n;
    }
    if (!ck || !ck->src[1]) return false;
    const lm_ggml_tensor * kdst = ck->src[1];
    const int64_t D = rk->ne[0], Hkv = rk->ne[1], T = rk->ne[2];
    if (kdst->type != LM_GGML_TYPE_F16 || !lm_ggml_is_contiguous(kdst) || lm_ggml_nelements(kdst) != Hkv * D * T) return false;
    if (!only_user_is(g, rk, ck)) return false;
    if (((uintptr_t) rk->src[0]->data % 8) || ((uintptr_t) kdst->data % 4)) return false;
    const lm_ggml_tensor * node = rk;   // for B200_CHECK's message
    const int32_t * p = (const int32_t *) rk->op_params;
    float freq_base, freq_scale, attn_factor;
    memcpy(&freq_base, p + 5, sizeof(float));
    memcpy(&freq_scale, p + 6, sizeof(float));
    memcpy(&attn_factor, p + 8, sizeof(float));
    // through the row list when the store is a cache-row store (see row_store): nothing in the launch then depends on where
    // in the cache the ubatch lands
    const int32_t * rows_list = nullptr;
    void * k_base = kdst->data;
    int64_t k_nb_row = Hkv * D * 2;
    const int at = slot_offset(ctx, ck);
    if (at >= 0) {
        rows_list = ctx->slots_dev + at;
        k_base = kdst->view_src->data;
        k_nb_row = (int64_t) kdst->view_src->nb[1];
    }
    if (b200_rope_store_to(nullptr, nullptr, 0, 0, (const float *) rk->src[0]->data, rk->src[0]->nb[1], rk->src[0]->nb[2], nullptr, 0, D, 0, Hkv, T, p[1],
                           (const int32_t *) rk->src[1]->data, rk->src[2] ? (const float *) rk->src[2]->data : nullptr, freq_base, freq_scale, attn_factor,
                           rows_list, k_base, k_nb_row, nullptr, 0, ctx->stream) != B200_OK) {
        B200_LOG_ERROR("ggml-b200: %s: %s\n", lm_ggml_op_name(node->op), b200_last_error());
        return false;   // the separate kernels take over
    }
    ctx->rs.cpy_k = ck;
    ctx->stats.nodes += 1;
    ctx->stats.rope_stores++;
    g_rope_store_groups.fetch_add(1, std::memory_order_relaxed);
    return true;
}

// the mask-cast CPY of a mask that the driver described instead of filling (kq_mask_hint_t)
bool mask_hint_serves(const b200_backend_ctx * ctx, const lm_ggml_tensor * node) {
    if (node->op != LM_GGML_OP_CPY) return false;
    const lm_ggml_tensor * s0 = node->src[0], * dstt = node->src[1] ? node->src[1] : node;
    const kq_mask_hint_t::dev_state & d = g_kq_hint.dev[ctx->device];
    return d.dev_mask && s0->data == d.dev_mask && d.serial == g_kq_hint.serial && s0->type == LM_GGML_TYPE_F32 && dstt->type == LM_GGML_TYPE_F16 &&
           lm_ggml_is_contiguous(dstt) && s0->ne[0] == d.n_kv && s0->ne[1] == (d.n_tokens + 63) / 64 * 64 && lm_ggml_nelements(s0) == lm_ggml_nelements(dstt);
}

static bool debug_lists() {
    static const bool v = [] { const char * e = getenv("B200_GRAPH_DEBUG"); return e && atoi(e) != 0; }();
    return v;
}

// ---- running a node before its place in the node order ----
// ggml-alloc gives a node's destination to it from the node's own place on: earlier, the same memory may still hold a
// tensor that a node in between reads or writes.  Node j may therefore run together with node i < j only if, for every
// node k in between that has yet to run, j's destination overlaps neither k's destination nor any of k's sources, and
// none of j's sources overlaps k's destination (j's inputs exist already).  Checked on the addresses of the graph at hand.
bool ranges_overlap(const lm_ggml_tensor * a, const lm_ggml_tensor * b) {
    if (!a || !b || !a->data || !b->data) return false;
    const char * a0 = (const char *) a->data, * b0 = (const char *) b->data;
    return a0 < b0 + lm_ggml_nbytes(b) && b0 < a0 + lm_ggml_nbytes(a);
}

// j's sources are not written by any node between i and j that has yet to run
bool inputs_ready(const b200_backend_ctx * ctx, const lm_ggml_cgraph * g, int i, int j) {
    const lm_ggml_tensor * nj = g->nodes[j];
    for (int k = i + 1; k < j; ++k) {
        if (ctx->node_done[k]) continue;
        for (int s = 0; s < LM_GGML_MAX_SRC; ++s)
            if (nj->src[s] && ranges_overlap(nj->src[s], g->nodes[k])) return false;
    }
    return true;
}

// j's destination is not memory that a node between i and j that has yet to run reads or writes
bool destination_free(const b200_backend_ctx * ctx, const lm_ggml_cgraph * g, int i, int j) {
    const lm_ggml_tensor * nj = g->nodes[j];
    for (int k = i + 1; k < j; ++k) {
        if (ctx->node_done[k]) continue;
        const lm_ggml_tensor * nk = g->nodes[k];
        if (ranges_overlap(nj, nk)) return false;
        for (int s = 0; s < LM_GGML_MAX_SRC; ++s)
            if (nk->src[s] && ranges_overlap(nj, nk->src[s])) return false;
    }
    return true;
}

bool can_run_early(const b200_backend_ctx * ctx, const lm_ggml_cgraph * g, int i, int j) {
    return inputs_ready(ctx, g, i, j) && destination_free(ctx, g, i, j);
}

// every node that reads t, directly or through reshapes and views, is `reader`, and t is no graph output
bool only_reader_is(const lm_ggml_cgraph * g, const lm_ggml_tensor * t, const lm_ggml_tensor * reader) {
    for (int i = 0; i < g->n_nodes; ++i) {
        const lm_ggml_tensor * n = g->nodes[i];
        if (n == reader || n->op == LM_GGML_OP_RESHAPE || n->op == LM_GGML_OP_VIEW) continue;
        for (int s = 0; s < LM_GGML_MAX_SRC; ++s)
            if (n->src[s] && through_views(n->src[s]) == t) return false;
    }
    for (int i = 0; i < g->n_nodes; ++i) {
        const lm_ggml_tensor * n = g->nodes[i];
        if ((n->op == LM_GGML_OP_RESHAPE || n->op == LM_GGML_OP_VIEW) && through_views(n) == t && (n->flags & LM_GGML_TENSOR_FLAG_OUTPUT)) return false;
    }
    return !(t->flags & LM_GGML_TENSOR_FLAG_OUTPUT);
}

// ROPE(q) when the k and v products of the same layer have run ahead into scratch (they joined q's launch): one kernel
// rotates q into its destination, rotates k out of scratch into its cache rows and stores v out of scratch into its cache
// rows -- what ROPE(q), the two copies out of scratch, ROPE(k) + K store and the V store would do in five steps.  The k and
// v products, ROPE(k) and the two CPY nodes are then done: nothing else reads their results (checked), and the cache rows
// they write are read by nothing before the attention of the layer.
bool rope_all_group(b200_backend_ctx * ctx, const lm_ggml_cgraph * g, int i) {
    const lm_ggml_tensor * rq = g->nodes[i], * q_in = rq->src[0];
    if (q_in->type != LM_GGML_TYPE_F32 || !lm_ggml_is_contiguous(rq) || !lm_ggml_is_contiguous(q_in) || rq->ne[3] != 1) return false;
    int i_rk = -1, i_ck = -1, i_cv = -1, i_k = -1, i_v = -1;
    for (int j = i + 1; j < g->n_nodes && j < i + 24; ++j) {
        const lm_ggml_tensor * n = g->nodes[j];
        if (n->op == LM_GGML_OP_FLASH_ATTN_EXT) break;
        if (n->op == LM_GGML_OP_ROPE && i_rk < 0 && !ctx->node_done[j]) i_rk = j;
        else if (n->op == LM_GGML_OP_CPY && i_rk >= 0 && i_ck < 0 && n->src[0] == g->nodes[i_rk]) i_ck = j;
        else if (n->op == LM_GGML_OP_CPY && i_cv < 0 && n->src[0] && through_views(n->src[0])->op == LM_GGML_OP_MUL_MAT) i_cv = j;
    }
    if (i_rk < 0 || i_ck < 0 || i_cv < 0) return false;
    const lm_ggml_tensor * rk = g->nodes[i_rk], * ck = g->nodes[i_ck], * cv = g->nodes[i_cv];
    const lm_ggml_tensor * kp = through_views(rk->src[0]), * vp = through_views(cv->src[0]);
    const b200_backend_ctx::parked_result * pk = nullptr, * pv = nullptr;
    for (int j = 0; j < g->n_nodes && (i_k < 0 || i_v < 0); ++j) {
        if (g->nodes[j] == kp) i_k = j;
        if (g->nodes[j] == vp) i_v = j;
    }
    if (i_k < 0 || i_v < 0 || ctx->node_done[i_k] != 2 || ctx->node_done[i_v] != 2) return false;   // both wait in scratch
    for (const auto & e : ctx->parked_for) {
        if (e.node == i_k) pk = &e;
        if (e.node == i_v) pv = &e;
    }
    if (!pk || !pv) return false;
    // same rotation for q and k
    if (memcmp(rq->op_params, rk->op_params, sizeof(rq->op_params)) != 0 || rq->src[1] != rk->src[1] || rq->src[2] != rk->src[2]) return false;
    const int64_t D = rq->ne[0], H = rq->ne[1], T = rq->ne[2], Hkv = rk->ne[1];
    if (rk->ne[0] != D || rk->ne[2] != T || rk->ne[3] != 1 || kp->ne[0] != Hkv * D || vp->ne[0] != Hkv * D) return false;
    const int at_k = slot_offset(ctx, ck), at_v = slot_offset(ctx, cv);
    if (at_k < 0 || at_v < 0) return false;
    for (int64_t r = 0; r < T; ++r)
        if (ctx->slots_host[(size_t) at_k + r] != ctx->slots_host[(size_t) at_v + r]) return false;   // one row list serves both stores
    const lm_ggml_tensor * kc = ck->src[1]->view_src, * vc = cv->src[1]->view_src;
    if (kc->ne[0] != Hkv * D || vc->ne[0] != Hkv * D) return false;
    if (!only_reader_is(g, kp, rk) || !only_user_is(g, rk, ck) || !only_reader_is(g, vp, cv)) return false;
    if (((uintptr_t) q_in->data % 8) || ((uintptr_t) rq->data % 8) || (pk->stride % 8) || (pv->stride % 8)) return false;
    const int32_t * p = (const int32_t *) rq->op_params;
    float freq_base, freq_scale, attn_factor;
    memcpy(&freq_base, p + 5, sizeof(float));
    memcpy(&freq_scale, p + 6, sizeof(float));
    memcpy(&attn_factor, p + 8, sizeof(float));
    if (b200_rope_store_to((const float *) q_in->data, (float *) rq->data, q_in->nb[1], q_in->nb[2], (const float *) ctx->parked[pk->block].ptr, D * 4,
                           (int64_t) pk->stride, (const float *) ctx->parked[pv->block].ptr, (int64_t) pv->stride, D, H, Hkv, T, p[1],
                           (const int32_t *) rq->src[1]->data, rq->src[2] ? (const float *) rq->src[2]->data : nullptr, freq_base, freq_scale, attn_factor,
                           ctx->slots_dev + at_k, kc->data, (int64_t) kc->nb[1], vc->data, (int64_t) vc->nb[1], ctx->stream) != B200_OK) {
        B200_LOG_ERROR("ggml-b200: ROPE group: %s\n", b200_last_error());
        return false;   // the separate kernels take over
    }
    ctx->node_done[i_k] = ctx->node_done[i_v] = ctx->node_done[i_rk] = ctx->node_done[i_ck] = ctx->node_done[i_cv] = 1;
    ctx->stats.nodes += 3;
    ctx->stats.rope_stores++;
    g_rope_store_groups.fetch_add(1, std::memory_order_relaxed);
    if (debug_lists() && i < 64) fprintf(stderr, "ggml-b200: %s, %s and the K / V stores as one kernel\n", rq->name, rk->name);
    return true;
}

// launches the kernels of a node list on the backend's stream (directly, or into a stream capture)
lm_ggml_status run_nodes(b200_backend_ctx * ctx, lm_ggml_cgraph * cgraph, bool check_abort) {
    cudaStream_t st = ctx->stream;
    ctx->act_src = nullptr;
    for (split_peer & p : ctx->peers) p.act_src = nullptr;
    ctx->index_mask = nullptr;
    ctx->rs.cpy_k = nullptr;
    ctx->node_done.assign((size_t) cgraph->n_nodes, 0);   // nodes that ran ahead of their place
    ctx->parked_for.clear();

    for (int i = 0; i < cgraph->n_nodes; ++i) {
        lm_ggml_tensor * node = cgraph->nodes[i];
        if (ctx->node_done[i] == 2) {   // a product that ran ahead into scratch: its destination is its own from here on
            for (const auto & pk : ctx->parked_for)
                if (pk.node == i) {
                    if (!cuda_ok(cudaMemcpy2DAsync(node->data, node->nb[1], ctx->parked[pk.block].ptr, pk.stride, (size_t) node->ne[0] * 4,
                                                   (size_t) (node->ne[1] * node->ne[2] * node->ne[3]), cudaMemcpyDeviceToDevice, st), "cudaMemcpy2DAsync(parked product)"))
                        return LM_GGML_STATUS_FAILED;
                }
            continue;
        }
        if (lm_ggml_is_empty(node) || ctx->node_done[i]) continue;
        switch (node->op) {
            case LM_GGML_OP_NONE: case LM_GGML_OP_RESHAPE: case LM_GGML_OP_VIEW: case LM_GGML_OP_PERMUTE: case LM_GGML_OP_TRANSPOSE:
                continue;
            default:
                break;
        }
        if (check_abort && ctx->abort_cb && (i & 63) == 0 && ctx->abort_cb(ctx->abort_cb_data)) {
            cudaStreamSynchronize(st);
            return LM_GGML_STATUS_ABORTED;
        }
        ctx->stats.nodes++;
        const lm_ggml_tensor * s0 = node->src[0], * s1 = node->src[1];
        switch (node->op) {
            case LM_GGML_OP_MUL_MAT: {
                if (s0->buffer && buft_is_b200_split(s0->buffer->buft)) {
                    const lm_ggml_status rc = compute_mul_mat_split(ctx, node);
                    if (rc != LM_GGML_STATUS_SUCCESS) return rc;
                    break;
                }
                const int64_t K = s0->ne[0], M = s0->ne[1], N = s1->ne[1] * s1->ne[2] * s1->ne[3];
                const size_t ab = b200_act_bytes(K, N);
                if (ctx->act_src != s1) {  // consecutive mul_mats on the same activations (wq/wk/wv, gate/up) quantise once
                    void * act = ctx->act.get(ab, st);
                    if (!act) return LM_GGML_STATUS_ALLOC_FAILED;
                    B200_CHECK(b200_quantize_activations((const float *) s1->data, s1->nb[1], K, N, act, ctx->act.bytes, ctx->q8_variant, st));
                    ctx->act_src = s1;
                    ctx->stats.act_quantized++;
                }
                // Other products of the same activations a few nodes on (q, k and v; ffn_gate and ffn_up) join this launch: one
                // launch fills the GPU better than three small ones.  A product whose inputs exist runs ahead of its place --
                // into its own destination when that memory is free already and has this product's row stride
                // (destination_free), else into scratch of the backend, from where a device copy moves the result to its
                // destination when the node's turn comes (q, k, v: ggml-alloc gives k the block that q's product vacates).
                int n_w = 1;
                const void * wv[3] = {s0->data, nullptr, nullptr};
                int64_t Mv[3] = {M, 0, 0};
                float * dv[3] = {(float *) node->data, nullptr, nullptr};
                int at[3] = {i, -1, -1};
                int n_parked = 0;
                for (int j = i + 1; ctx->stack && n_w < 3 && j < cgraph->n_nodes && j < i + 12 && N > 8; ++j) {
                    const lm_ggml_tensor * nx = cgraph->nodes[j];
                    if (nx->op == LM_GGML_OP_FLASH_ATTN_EXT) break;
                    if (ctx->node_done[j] || nx->op != LM_GGML_OP_MUL_MAT || nx->src[1] != s1) continue;
                    if (nx->src[0]->type != s0->type || nx->src[0]->ne[0] != K || !nx->src[0]->buffer || buft_is_b200_split(nx->src[0]->buffer->buft) ||
                        Mv[n_w - 1] % 128 != 0 || ((uintptr_t) nx->src[0]->data % 16) || nx->ne[1] * nx->ne[2] * nx->ne[3] != N || nx->nb[0] != 4 ||
                        (int64_t) nx->src[0]->ne[1] * 4 > (int64_t) node->nb[1] || !inputs_ready(ctx, cgraph, i, j))
                        continue;
                    bool direct = nx->nb[1] == node->nb[1] && destination_free(ctx, cgraph, i, j);
                    for (int k = 0; direct && k < n_w; ++k) direct = !ranges_overlap(nx, cgraph->nodes[at[k]]);   // (the allocator may have given two of them the same memory)
                    float * to = (float *) nx->data;
                    if (!direct) {
                        if (n_parked >= 2) continue;
                        to = (float *) ctx->parked[n_parked].get((size_t) N * node->nb[1], st);
                        if (!to) continue;
                        ctx->parked_for.push_back({j, n_parked, (size_t) node->nb[1]});
                        ++n_parked;
                    }
                    if (debug_lists() && i < 64) fprintf(stderr, "ggml-b200: %s (node %d) joins %s (node %d)%s\n", nx->name, j, node->name, i, direct ? "" : " through scratch");
                    wv[n_w] = nx->src[0]->data;
                    Mv[n_w] = nx->src[0]->ne[1];
                    dv[n_w] = to;
                    at[n_w] = j;
                    ctx->node_done[j] = direct ? 1 : 2;   // 2: the result waits in scratch for the node's turn
                    ++n_w;
                }
                int64_t M_all = 0;
                for (int k = 0; k < n_w; ++k) M_all += Mv[k];
                const size_t wb = b200_mul_mat_workspace_bytes(s0->type, K, M_all, N);
                void * ws = wb ? ctx->workspace.get(wb, st) : nullptr;
                if (wb && !ws) return LM_GGML_STATUS_ALLOC_FAILED;
                if (n_w > 1) {
                    B200_CHECK(b200_mul_mat_q_prequant_multi(s0->type, n_w, wv, Mv, K, ctx->act.ptr, N, dv, node->nb[1], ws, ws ? ctx->workspace.bytes : 0, st));
                    ctx->stats.mul_mat += n_w;
                    ctx->stats.nodes += n_w - 1;
                    g_stacked_products.fetch_add(1, std::memory_order_relaxed);
                    break;
                }
                B200_CHECK(b200_mul_mat_q_prequant(s0->type, s0->data, K, M, ctx->act.ptr, N, (float *) node->data, node->nb[1], ws,
                                                   ws ? ctx->workspace.bytes : 0, st));
                ctx->stats.mul_mat++;
            } break;
            case LM_GGML_OP_FLASH_ATTN_EXT: {
                const lm_ggml_tensor * q = s0, * k = s1, * v = node->src[2], * m = node->src[3];
                const int64_t D = q->ne[0], Nq = q->ne[1], H = q->ne[2], Hkv = k->ne[2], n_kv = k->ne[1];
                float scale, max_bias, softcap;
                memcpy(&scale, (const float *) node->op_params + 0, sizeof(float));
                memcpy(&max_bias, (const float *) node->op_params + 1, sizeof(float));
                memcpy(&softcap, (const float *) node->op_params + 2, sizeof(float));
                void * index = nullptr;
                if (m) {
                    const size_t ib = b200_mask_index_bytes(Nq, n_kv);
                    if (ctx->index_mask != m) {  // every layer of a graph attends through the same mask tensor
                        index = ctx->mask_index.get(ib, st);
                        if (!index) return LM_GGML_STATUS_ALLOC_FAILED;
                        B200_CHECK(b200_mask_index_build(m->data, m->nb[1], Nq, n_kv, index, ctx->mask_index.bytes, st));
                        ctx->index_mask = m;
                        ctx->stats.mask_indexed++;
                    }
                    index = ctx->mask_index.ptr;
                }
                const size_t sb = b200_flash_attn_scratch_bytes(D, H, Hkv, Nq, n_kv);
                void * scratch = ctx->fa_scratch.get(std::max<size_t>(sb, 256), st);
                if (!scratch) return LM_GGML_STATUS_ALLOC_FAILED;
                if (ctx->fa_parity) {
                    B200_CHECK(b200_flash_attn_ext_parity(D, H, Hkv, Nq, n_kv, (const float *) q->data, q->nb[1], q->nb[2], k->data, k->nb[1], k->nb[2],
                                                          v->data, v->nb[1], v->nb[2], m ? m->data : nullptr, m ? m->nb[1] : 0, index, scale, max_bias,
                                                          softcap, (float *) node->data, st));
                    ctx->stats.flash_attn++;
                    break;
                }
                B200_CHECK(b200_flash_attn_ext_indexed(D, H, Hkv, Nq, n_kv, (const float *) q->data, q->nb[1], q->nb[2], k->data, k->nb[1], k->nb[2],
                                                       v->data, v->nb[1], v->nb[2], m ? m->data : nullptr, m ? m->nb[1] : 0, index, scale, max_bias,
                                                       softcap, (float *) node->data, scratch, ctx->fa_scratch.bytes, st));
                ctx->stats.flash_attn++;
            } break;
            case LM_GGML_OP_RMS_NORM: {
                float eps;
                memcpy(&eps, node->op_params, sizeof(float));
                const int64_t d = s0->ne[0], rows = lm_ggml_nrows(s0);
                // RMS_NORM followed by MUL with a weight row is how every llama norm is built: one kernel
                lm_ggml_tensor * next = i + 1 < cgraph->n_nodes ? cgraph->nodes[i + 1] : nullptr;
                if (next && next->op == LM_GGML_OP_MUL && next->src[0] == node && next->src[1] && next->src[1]->type == LM_GGML_TYPE_F32 &&
                    next->src[1]->ne[0] == d && lm_ggml_nelements(next->src[1]) == d && lm_ggml_is_contiguous(next->src[1]) &&
                    lm_ggml_is_contiguous(next) && only_user_is(cgraph, node, next)) {
                    // ... and when the next node multiplies a quantised weight by the result, the same kernel also
                    // leaves it quantised for that mul_mat (and the ones after it that read the same tensor)
                    lm_ggml_tensor * mm = i + 2 < cgraph->n_nodes ? cgraph->nodes[i + 2] : nullptr;
                    const bool feeds_mul_mat = mm && mm->op == LM_GGML_OP_MUL_MAT && mm->src[1] == next && d % 32 == 0 && d <= 16384 &&
                                               s0->nb[1] % 16 == 0 && ((uintptr_t) s0->data % 16) == 0 && ((uintptr_t) next->data % 16) == 0;
                    void * act = feeds_mul_mat ? ctx->act.get(b200_act_bytes(d, rows), st) : nullptr;
                    if (act) {
                        B200_CHECK(b200_add_rms_norm_quantize((float *) s0->data, s0->nb[1], nullptr, 0, (const float *) next->src[1]->data, (float *) next->data,
                                                              d * 4, d, rows, eps, act, ctx->act.bytes, ctx->q8_variant, st));
                        ctx->act_src = next;
                        ctx->stats.act_quantized++;
                    } else {
                        B200_CHECK(b200_rms_norm((const float *) s0->data, s0->nb[1], (const float *) next->src[1]->data, (float *) next->data, d * 4, d, rows, eps, st));
                    }
                    ++i;
                } else {
                    B200_CHECK(b200_rms_norm((const float *) s0->data, s0->nb[1], nullptr, (float *) node->data, d * 4, d, rows, eps, st));
                }
            } break;
            case LM_GGML_OP_ADD:
            case LM_GGML_OP_MUL: {
                if (node->op == LM_GGML_OP_ADD && ctx->fuse) {
                    // residual ADD written over one of its operands, then RMS_NORM, MUL by the norm weight and a MUL_MAT on the
                    // result (ffn_inp -> ffn_norm -> gate/up, l_out -> next layer's attn_norm -> q/k/v): one kernel
                    lm_ggml_tensor * rn = i + 1 < cgraph->n_nodes ? cgraph->nodes[i + 1] : nullptr;
                    lm_ggml_tensor * mu = i + 2 < cgraph->n_nodes ? cgraph->nodes[i + 2] : nullptr;
                    lm_ggml_tensor * mm = i + 3 < cgraph->n_nodes ? cgraph->nodes[i + 3] : nullptr;
                    const int64_t d = s0->ne[0], rows = lm_ggml_nrows(s0);
                    const bool in_place = node->data == s0->data || node->data == s1->data;
                    if (in_place && lm_ggml_are_same_shape(s0, s1) && rn && mu && mm && rn->op == LM_GGML_OP_RMS_NORM && rn->src[0] == node &&
                        mu->op == LM_GGML_OP_MUL && mu->src[0] == rn && mu->src[1] && mu->src[1]->type == LM_GGML_TYPE_F32 && mu->src[1]->ne[0] == d &&
                        lm_ggml_nelements(mu->src[1]) == d && lm_ggml_is_contiguous(mu->src[1]) && lm_ggml_is_contiguous(mu) && only_user_is(cgraph, rn, mu) &&
                        mm->op == LM_GGML_OP_MUL_MAT && mm->src[1] == mu && d % 32 == 0 && d <= 16384 && ((uintptr_t) s0->data % 16) == 0 &&
                        ((uintptr_t) s1->data % 16) == 0 && ((uintptr_t) mu->data % 16) == 0 && mu->data != node->data) {
                        void * act = ctx->act.get(b200_act_bytes(d, rows), st);
                        if (act) {
                            float eps;
                            memcpy(&eps, rn->op_params, sizeof(float));
                            float * x = (float *) node->data;
                            const float * res = node->data == s0->data ? (const float *) s1->data : (const float *) s0->data;
                            B200_CHECK(b200_add_rms_norm_quantize(x, d * 4, res, d * 4, (const float *) mu->src[1]->data, (float *) mu->data, d * 4, d, rows, eps,
                                                                  act, ctx->act.bytes, ctx->q8_variant, st));
                            ctx->act_src = mu;
                            ctx->stats.act_quantized++;
                            ctx->stats.nodes += 2;
                            g_add_norm_groups.fetch_add(1, std::memory_order_relaxed);
                            i += 2;
                            break;
                        }
                    }
                }
                const int64_t d = s0->ne[0], rows = lm_ggml_nrows(s0);
                const int64_t brows = lm_ggml_are_same_shape(s0, s1) ? rows : 1;
                if (node->op == LM_GGML_OP_ADD) B200_CHECK(b200_add((const float *) s0->data, (const float *) s1->data, (float *) node->data, d, rows, brows, st));
                else B200_CHECK(b200_mul((const float *) s0->data, (const float *) s1->data, (float *) node->data, d, rows, brows, st));
            } break;
            case LM_GGML_OP_UNARY: {
                // SILU(gate) * up: the llama FFN gate, fused when the SILU result has no other reader.  The multiply is the next
                // node that has yet to run (ffn_up sits between the two in the node order and may have run with ffn_gate), and
                // runs here, ahead of its place, when that is safe.
                int jn = i + 1;
                while (jn < cgraph->n_nodes && jn < i + 4 && ctx->node_done[jn]) ++jn;
                lm_ggml_tensor * next = jn < cgraph->n_nodes ? cgraph->nodes[jn] : nullptr;
                if (next && next->op == LM_GGML_OP_MUL && (next->src[0] == node || next->src[1] == node) && supports_binary(next) &&
                    lm_ggml_are_same_shape(next->src[0], next->src[1]) && only_user_is(cgraph, node, next) && (jn == i + 1 || can_run_early(ctx, cgraph, i, jn))) {
                    const lm_ggml_tensor * other = next->src[0] == node ? next->src[1] : next->src[0];
                    // the product is the input of ffn_down: the same kernel leaves it quantised for that mul_mat
                    lm_ggml_tensor * mm = jn + 1 < cgraph->n_nodes ? cgraph->nodes[jn + 1] : nullptr;
                    const int64_t d = s0->ne[0], rows = lm_ggml_nrows(s0);
                    const bool feeds_mul_mat = mm && mm->op == LM_GGML_OP_MUL_MAT && mm->src[1] == next && d % 32 == 0 && lm_ggml_is_contiguous(s0) &&
                                               lm_ggml_is_contiguous(other) && lm_ggml_is_contiguous(next) && ((uintptr_t) s0->data % 16) == 0 &&
                                               ((uintptr_t) other->data % 16) == 0 && ((uintptr_t) next->data % 16) == 0;
                    void * act = feeds_mul_mat ? ctx->act.get(b200_act_bytes(d, rows), st) : nullptr;
                    if (act) {
                        B200_CHECK(b200_silu_mul_quantize((const float *) s0->data, (const float *) other->data, d * 4, (float *) next->data, d * 4, d, rows,
                                                          act, ctx->act.bytes, ctx->q8_variant, st));
                        ctx->act_src = next;
                        ctx->stats.act_quantized++;
                    } else {
                        B200_CHECK(b200_silu((const float *) s0->data, (const float *) other->data, (float *) next->data, lm_ggml_nelements(s0), st));
                    }
                    ctx->node_done[jn] = 1;
                    ctx->stats.nodes++;
                } else {
                    B200_CHECK(b200_silu((const float *) s0->data, nullptr, (float *) node->data, lm_ggml_nelements(s0), st));
                }
            } break;
            case LM_GGML_OP_ROPE: {
                if (ctx->fuse && ctx->stack && s0->type == LM_GGML_TYPE_F32 && rope_all_group(ctx, cgraph, i)) break;   // q, k and both cache stores by one kernel
                if (ctx->fuse && s0->type == LM_GGML_TYPE_F32 && rope_store_group(ctx, cgraph, i)) break;   // rotated and stored into the cache by one kernel
                const int32_t * p = (const int32_t *) node->op_params;
                float freq_base, freq_scale, attn_factor;
                memcpy(&freq_base, p + 5, sizeof(float));
                memcpy(&freq_scale, p + 6, sizeof(float));
                memcpy(&attn_factor, p + 8, sizeof(float));
                if (s0->type == LM_GGML_TYPE_F16) {
                    B200_CHECK(b200_rope_norm_f16(s0->data, s0->nb[1], s0->nb[2], node->data, node->nb[1], node->nb[2], s0->ne[0], s0->ne[1], s0->ne[2], p[1],
                                                  (const int32_t *) s1->data, node->src[2] ? (const float *) node->src[2]->data : nullptr, freq_base,
                                                  freq_scale, attn_factor, st));
                    break;
                }
                B200_CHECK(b200_rope_norm((const float *) s0->data, s0->nb[1], s0->nb[2], (float *) node->data, node->nb[1], node->nb[2], s0->ne[0],
                                          s0->ne[1], s0->ne[2], p[1], (const int32_t *) s1->data, node->src[2] ? (const float *) node->src[2]->data : nullptr,
                                          freq_base, freq_scale, attn_factor, st));
            } break;
            case LM_GGML_OP_CPY: {
                if (node == ctx->rs.cpy_k) {   // already stored by the kernel that rotated k
                    ctx->rs.cpy_k = nullptr;
                    break;
                }
                if (mask_hint_serves(ctx, node)) {   // the f32 -> f16 cast of a mask the driver described instead of filling: synthesise the f16 mask
                    kq_mask_hint_t::dev_state & d = g_kq_hint.dev[ctx->device];
                    const lm_ggml_tensor * dstt = s1 ? s1 : node;
                    B200_CHECK(b200_kq_mask_build(d.buf, d.buf + d.n_kv, d.n_kv, d.buf + 2 * d.n_kv, d.buf + 2 * d.n_kv + d.n_tokens, d.n_tokens,
                                                  dstt->data, d.n_kv * 2, st));
                    g_kq_hint.masks_built.fetch_add(1, std::memory_order_relaxed);
                    break;
                }
                {   // a store into cache rows goes through its row list (row_store)
                    const int at = slot_offset(ctx, node);
                    if (at >= 0) {
                        const lm_ggml_tensor * cache = s1->view_src;
                        B200_CHECK(b200_set_rows_f16((const float *) s0->data, cache->ne[0] * 4, ctx->slots_dev + at, cache->data, (int64_t) cache->nb[1],
                                                     cache->ne[0], lm_ggml_nelements(s1) / cache->ne[0], st));
                        break;
                    }
                }
                lm_ggml_status rc = compute_cpy(ctx, node, s0, s1 ? s1 : node);
                if (rc != LM_GGML_STATUS_SUCCESS) return rc;
            } break;
            case LM_GGML_OP_CONT:
            case LM_GGML_OP_DUP: {
                lm_ggml_status rc = compute_cpy(ctx, node, s0, node);
                if (rc != LM_GGML_STATUS_SUCCESS) return rc;
            } break;
            case LM_GGML_OP_GET_ROWS: {
                const int64_t n_ids = lm_ggml_nelements(s1);
                if (s0->type == LM_GGML_TYPE_F32) {
                    B200_CHECK(b200_get_rows_f32((const float *) s0->data, s0->nb[1], (const int32_t *) s1->data, (float *) node->data, node->nb[1], s0->ne[0], n_ids, st));
                } else {
                    B200_CHECK(b200_get_rows_q(s0->type, s0->data, s0->ne[0], s0->ne[1], (const int32_t *) s1->data, (float *) node->data, node->nb[1], n_ids, st));
                }
            } break;
            default:
                B200_LOG_ERROR("ggml-b200: op %s reached graph_compute but supports_op does not list it\n", lm_ggml_op_name(node->op));
                return LM_GGML_STATUS_FAILED;
        }
    }
    return LM_GGML_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------------------------
// CUDA-graph replay.  The reference rebuilds its graph for every ubatch (cactus/llama-context.cpp, graph_build) but a
// decode step's node list comes out the same every time: same ops, shapes, addresses (ggml-alloc is deterministic) --
// except where the ubatch lands in the cache, which the row lists above take out of the launches, and the attended
// window n_kv, which grows by 256 cells now and then.  A node list is reduced to two 64-bit hashes over everything a
// launch depends on; a list seen for the first time runs kernel by kernel and is recorded into a CUDA graph meanwhile, a known one is
// replayed with one cudaGraphLaunch.  Lists on split weights (several devices and streams) always run directly.
// ---------------------------------------------------------------------------------------------
std::atomic<uint64_t> g_graph_records{0}, g_graph_replays{0}, g_graph_updates{0};   // updates: recordings that re-used an instance

struct hash2 {   // two independent 64-bit mixes over 8-byte words (a node list is a few hundred KB: byte-wise hashing would cost milliseconds)
    uint64_t a = 0xcbf29ce484222325ull, b = 0x9e3779b97f4a7c15ull;
    void word(uint64_t w) {
        a = (a ^ w) * 0x9e3779b97f4a7c15ull;
        a ^= a >> 29;
        b = (b + w) * 0xd6e8feb86659fd93ull;
        b ^= b >> 32;
    }
    void add(const void * p, size_t n) {
        const uint8_t * c = (const uint8_t *) p;
        for (; n >= 8; n -= 8, c += 8) {
            uint64_t w;
            memcpy(&w, c, 8);
            word(w);
        }
        if (n) {
            uint64_t w = 0;
            memcpy(&w, c, n);
            word(w ^ ((uint64_t) n << 56));
        }
    }
    template <typename T> void val(const T & v) {
        uint64_t w = 0;
        static_assert(sizeof(T) <= 8, "scalar");
        memcpy(&w, &v, sizeof(T));
        word(w);
    }
};

void hash_tensor(hash2 & h, const lm_ggml_tensor * t, bool with_address) {
    if (!t) { h.val((int) -1); return; }
    h.val((int) t->type);
    h.val((int) t->op);
    h.add(t->ne, sizeof(t->ne));
    h.add(t->nb, sizeof(t->nb));
    if (with_address) h.val((uintptr_t) t->data);
    else h.val((uintptr_t) (t->view_src ? t->view_src->data : nullptr));
}

// false: the list cannot be replayed (weights on a split buffer)
bool graph_signature(const b200_backend_ctx * ctx, const lm_ggml_cgraph * g, uint64_t * h1, uint64_t * h2, std::vector<uint64_t> * trail) {
    hash2 h;
    if (trail) trail->clear();
    h.val(g->n_nodes);
    h.val((uintptr_t) ctx->act.ptr); h.val((uintptr_t) ctx->workspace.ptr); h.val((uintptr_t) ctx->fa_scratch.ptr); h.val((uintptr_t) ctx->mask_index.ptr);
    h.val((uintptr_t) ctx->slots_dev);
    h.val((uintptr_t) ctx->parked[0].ptr); h.val((uintptr_t) ctx->parked[1].ptr);
    // where the row lists start relative to the first one (a kernel that serves two stores with one list relies on it)
    for (size_t k = 0; k < ctx->slot_first.size(); ++k) h.val(ctx->slot_first[k] - ctx->slot_first[0]);
    h.val(ctx->fuse); h.val(ctx->stack); h.val(ctx->fa_parity); h.val(ctx->q8_variant);
    for (int i = 0; i < g->n_nodes; ++i) {
        const lm_ggml_tensor * n = g->nodes[i];
        const int at = slot_offset(ctx, n);
        h.val(at);   // -1, or where the node's row list starts: the launch reads its rows from there
        // view nodes launch nothing (their readers hash what they read): the view into the cache that a row store writes
        // through is such a node, and it moves
        const bool is_view = n->op == LM_GGML_OP_NONE || n->op == LM_GGML_OP_RESHAPE || n->op == LM_GGML_OP_VIEW || n->op == LM_GGML_OP_PERMUTE ||
                             n->op == LM_GGML_OP_TRANSPOSE;
        hash_tensor(h, n, at < 0 && !is_view);
        if (!is_view) h.add(n->op_params, sizeof(n->op_params));   // a view keeps its byte offset there
        h.val(n->flags);
        for (int k = 0; k < LM_GGML_MAX_SRC; ++k) {
            const lm_ggml_tensor * sk = n->src[k];
            if (!sk) { h.val((int) -1); continue; }
            if (n->op == LM_GGML_OP_MUL_MAT && k == 0 && sk->buffer && buft_is_b200_split(sk->buffer->buft)) return false;
            hash_tensor(h, sk, !(at >= 0 && k == 1));   // the destination view of a row store moves; its cache tensor does not
        }
        if (mask_hint_serves(ctx, n)) {
            const kq_mask_hint_t::dev_state & d = g_kq_hint.dev[ctx->device];
            h.val((uintptr_t) d.buf); h.val(d.n_kv); h.val(d.n_tokens);
        } else {
            h.val((int) 0);
        }
        if (trail) trail->push_back(h.a);
    }
    *h1 = h.a;
    *h2 = h.b;
    return true;
}

// Records the launches of a node list into a CUDA graph without running them: the backend's stream is swapped for a
// capture stream for the duration.  A list that differs from a recorded one only in sizes and addresses (the attended
// window grew) updates that instance in place, which is much cheaper than a new one.
bool shadow_record(b200_backend_ctx * ctx, lm_ggml_cgraph * cgraph, uint64_t h1, uint64_t h2, b200_backend_ctx::graph_entry * victim) {
    if (!ctx->cap_stream && cudaStreamCreateWithFlags(&ctx->cap_stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        ctx->cap_stream = nullptr;
        return false;
    }
    const lm_ggml_b200_stats before = ctx->stats;
    const uint64_t r0 = g_rope_store_groups.load(), a0 = g_add_norm_groups.load(), m0 = g_kq_hint.masks_built.load();
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    bool ok = false;
    if (cudaStreamBeginCapture(ctx->cap_stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    cudaStream_t own = ctx->stream;
    ctx->stream = ctx->cap_stream;
    t_recording = true;
    t_recording_failed = false;
    const lm_ggml_status rrc = run_nodes(ctx, cgraph, false);
    t_recording = false;
    ctx->stream = own;
    const cudaError_t ee = cudaStreamEndCapture(ctx->cap_stream, &graph);
    // what one run adds to the counters; the recording itself ran nothing
    lm_ggml_b200_stats delta = {};
    delta.nodes = ctx->stats.nodes - before.nodes; delta.mul_mat = ctx->stats.mul_mat - before.mul_mat;
    delta.flash_attn = ctx->stats.flash_attn - before.flash_attn; delta.act_quantized = ctx->stats.act_quantized - before.act_quantized;
    delta.mask_indexed = ctx->stats.mask_indexed - before.mask_indexed; delta.rope_stores = ctx->stats.rope_stores - before.rope_stores;
    const uint64_t dr = g_rope_store_groups.load() - r0, da = g_add_norm_groups.load() - a0, dm = g_kq_hint.masks_built.load() - m0;
    ctx->stats = before;
    g_rope_store_groups.store(r0); g_add_norm_groups.store(a0); g_kq_hint.masks_built.store(m0);
    if (rrc == LM_GGML_STATUS_SUCCESS && ee == cudaSuccess && graph && !t_recording_failed) {
        b200_backend_ctx::graph_entry * like = nullptr;
        for (auto & e : ctx->cache)
            if (e.exec && e.n_nodes == cgraph->n_nodes && (!like || e.stamp > like->stamp)) like = &e;
        if (like) {
            cudaGraphExecUpdateResultInfo info;
            if (cudaGraphExecUpdate(like->exec, graph, &info) == cudaSuccess) {
                exec = like->exec;
                like->exec = nullptr;
                victim = like;
                g_graph_updates.fetch_add(1, std::memory_order_relaxed);
            } else {
                cudaGetLastError();
                cudaGraphExecDestroy(like->exec);   // it may be half updated
                like->exec = nullptr;
            }
        }
        if (!exec && cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) exec = nullptr;
        if (exec && victim) {
            if (victim->exec) cudaGraphExecDestroy(victim->exec);
            victim->exec = exec;
            victim->h1 = h1; victim->h2 = h2;
            victim->n_nodes = cgraph->n_nodes;
            victim->stamp = ++ctx->stamp;
            victim->delta = delta;
            victim->rope_stores = dr; victim->add_norms = da; victim->masks = dm;
            g_graph_records.fetch_add(1, std::memory_order_relaxed);
            ctx->cold_records++;
            ok = true;
        } else if (exec) {
            cudaGraphExecDestroy(exec);
        }
    }
    if (!ok) cudaGetLastError();   // a failed recording leaves no sticky error
    if (graph) cudaGraphDestroy(graph);
    return ok;
}

lm_ggml_status backend_graph_compute(lm_ggml_backend_t backend, lm_ggml_cgraph * cgraph) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    device_guard g(ctx->device);
    cudaStream_t st = ctx->stream;
    ctx->stats.graphs++;
    if (ctx->timing) cudaEventRecord(ctx->ev0, st);
    prepare_row_lists(ctx, cgraph);

    lm_ggml_status rc = LM_GGML_STATUS_SUCCESS;
    uint64_t h1 = 0, h2 = 0;
    bool done = false, want_record = false;
    b200_backend_ctx::graph_entry * victim = nullptr;   // where a new recording goes: a free entry, else the least recently used
    // B200_GRAPH_DEBUG=1: when a list differs from the one before, say at which node
    static const bool debug = [] { const char * e = getenv("B200_GRAPH_DEBUG"); return e && atoi(e) != 0; }();
    std::vector<uint64_t> trail;
    if (ctx->graphs && ctx->warmed && graph_signature(ctx, cgraph, &h1, &h2, debug ? &trail : nullptr)) {
        if (debug) {
            static bool listed = false;
            if (!listed && cgraph->n_nodes > 60) {   // once: the node order of a layer, which decides what can run as one kernel
                listed = true;
                for (int k = 0; k < 60; ++k) fprintf(stderr, "ggml-b200: node %d %s %s\n", k, lm_ggml_op_name(cgraph->nodes[k]->op), cgraph->nodes[k]->name);
            }
            if (h1 != ctx->last_h1 && !ctx->dbg_trail.empty()) {
                size_t k = 0;
                while (k < trail.size() && k < ctx->dbg_trail.size() && trail[k] == ctx->dbg_trail[k]) ++k;
                if (k < (size_t) cgraph->n_nodes) {
                    const lm_ggml_tensor * n = cgraph->nodes[k];
                    fprintf(stderr, "ggml-b200: node list differs from the previous one at node %zu of %d (%zu before): %s %s\n", k, cgraph->n_nodes, ctx->dbg_trail.size(),
                            lm_ggml_op_name(n->op), n->name);
                }
            }
            ctx->dbg_trail = trail;
        }
        if (ctx->abort_cb && ctx->abort_cb(ctx->abort_cb_data)) {
            cudaStreamSynchronize(st);
            return LM_GGML_STATUS_ABORTED;
        }
        b200_backend_ctx::graph_entry * hit = nullptr;
        for (auto & e : ctx->cache) {
            if (e.exec && e.h1 == h1 && e.h2 == h2) hit = &e;
            if (!victim || (victim->exec && (!e.exec || e.stamp < victim->stamp))) victim = &e;
        }
        // A recording costs more than a direct run.  Lists that keep changing (two recordings in a row that were never
        // replayed) are therefore recorded only once they repeat.
        const bool repeats = h1 == ctx->last_h1 && h2 == ctx->last_h2;
        ctx->last_h1 = h1;
        ctx->last_h2 = h2;
        if (hit) {
            if (cuda_ok(cudaGraphLaunch(hit->exec, st), "cudaGraphLaunch")) {
                hit->stamp = ++ctx->stamp;
                ctx->stats.nodes += hit->delta.nodes; ctx->stats.mul_mat += hit->delta.mul_mat; ctx->stats.flash_attn += hit->delta.flash_attn;
                ctx->stats.act_quantized += hit->delta.act_quantized; ctx->stats.mask_indexed += hit->delta.mask_indexed; ctx->stats.rope_stores += hit->delta.rope_stores;
                g_rope_store_groups.fetch_add(hit->rope_stores, std::memory_order_relaxed);
                g_add_norm_groups.fetch_add(hit->add_norms, std::memory_order_relaxed);
                g_kq_hint.masks_built.fetch_add(hit->masks, std::memory_order_relaxed);
                g_graph_replays.fetch_add(1, std::memory_order_relaxed);
                ctx->cold_records = 0;
                done = true;
            }
        } else if (ctx->cold_records < 2 || repeats) {
            want_record = true;
        }
    }
    if (!done) {
        rc = run_nodes(ctx, cgraph, true);
        if (rc == LM_GGML_STATUS_SUCCESS) ctx->warmed = true;
    }
    if (rc != LM_GGML_STATUS_SUCCESS) return rc;
    // An unknown list has just been launched kernel by kernel; while the device works on it the host records the same
    // launches on a capture stream (nothing runs there), so that the next such list is one cudaGraphLaunch.  Recording
    // instead of running would leave the device idle for as long as the recording takes (1.6 ms for a 1031-node list).
    if (want_record) {
        const auto t_rec0 = std::chrono::steady_clock::now();
        const uint64_t l0 = b200_launch_count();
        const bool ok = shadow_record(ctx, cgraph, h1, h2, victim);
        if (debug) fprintf(stderr, "ggml-b200: recording %d nodes (%llu launches) took %.2f ms on the host (%s)\n", cgraph->n_nodes,
                           (unsigned long long) (b200_launch_count() - l0),
                           std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_rec0).count(), ok ? "ok" : "failed");
    }
    if (ctx->timing) {
        cudaEventRecord(ctx->ev1, st);
        cudaEventSynchronize(ctx->ev1);
        float ms = 0;
        cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1);
        ctx->stats.device_ms += ms;
        std::lock_guard<std::mutex> lock(g_totals_mu);
        g_total_device_ms += ms;
        g_total_timed_graphs++;
    }
    return LM_GGML_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------------------------
// events
// ---------------------------------------------------------------------------------------------
void backend_event_record(lm_ggml_backend_t backend, lm_ggml_backend_event_t event) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    device_guard g(ctx->device);
    cuda_ok(cudaEventRecord((cudaEvent_t) event->context, ctx->stream), "cudaEventRecord");
}

void backend_event_wait(lm_ggml_backend_t backend, lm_ggml_backend_event_t event) {
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    device_guard g(ctx->device);
    cuda_ok(cudaStreamWaitEvent(ctx->stream, (cudaEvent_t) event->context, 0), "cudaStreamWaitEvent");
}

const lm_ggml_backend_i b200_backend_iface = {
    /* .get_name           = */ backend_get_name,
    /* .free               = */ backend_free,
    /* .set_tensor_async   = */ backend_set_tensor_async,
    /* .get_tensor_async   = */ backend_get_tensor_async,
    /* .cpy_tensor_async   = */ backend_cpy_tensor_async,
    /* .synchronize        = */ backend_synchronize,
    /* .graph_plan_create  = */ nullptr,
    /* .graph_plan_free    = */ nullptr,
    /* .graph_plan_update  = */ nullptr,
    /* .graph_plan_compute = */ nullptr,
    /* .graph_compute      = */ backend_graph_compute,
    /* .event_record       = */ backend_event_record,
    /* .event_wait         = */ backend_event_wait,
};

// ---------------------------------------------------------------------------------------------
// device
// ---------------------------------------------------------------------------------------------
struct b200_registry {
    std::vector<b200_device_ctx *> ctxs;
    std::vector<lm_ggml_backend_device> devices;
    std::vector<lm_ggml_backend_buffer_type> bufts;
    std::vector<b200_buft_ctx *> buft_ctxs;
    lm_ggml_backend_buffer_type host_buft;
    lm_ggml_backend_reg reg;
};
b200_registry * registry();

const char * dev_get_name(lm_ggml_backend_dev_t dev) { return ((b200_device_ctx *) dev->context)->name.c_str(); }
const char * dev_get_description(lm_ggml_backend_dev_t dev) { return ((b200_device_ctx *) dev->context)->description.c_str(); }

void dev_get_memory(lm_ggml_backend_dev_t dev, size_t * free, size_t * total) {
    b200_device_ctx * ctx = (b200_device_ctx *) dev->context;
    if (b200_device_info(ctx->device, nullptr, 0, free, total, nullptr) != B200_OK) *free = *total = 0;
}

enum lm_ggml_backend_dev_type dev_get_type(lm_ggml_backend_dev_t) { return LM_GGML_BACKEND_DEVICE_TYPE_GPU; }

void dev_get_props(lm_ggml_backend_dev_t dev, lm_ggml_backend_dev_props * props) {
    props->name = dev_get_name(dev);
    props->description = dev_get_description(dev);
    props->type = dev_get_type(dev);
    dev_get_memory(dev, &props->memory_free, &props->memory_total);
    props->caps = {
        /* .async                = */ true,
        /* .host_buffer          = */ true,
        /* .buffer_from_host_ptr = */ false,
        /* .events               = */ true,
    };
}

lm_ggml_backend_t dev_init_backend(lm_ggml_backend_dev_t dev, const char *) {
    return lm_ggml_backend_b200_init(((b200_device_ctx *) dev->context)->device);
}

lm_ggml_backend_buffer_type_t dev_get_buffer_type(lm_ggml_backend_dev_t dev) { return device_buffer_type(((b200_device_ctx *) dev->context)->device); }
lm_ggml_backend_buffer_type_t dev_get_host_buffer_type(lm_ggml_backend_dev_t) { return lm_ggml_backend_b200_host_buffer_type(); }

bool dev_supports_op(lm_ggml_backend_dev_t dev, const lm_ggml_tensor * op) {
    // tensors that already live somewhere must live in a buffer of this device
    b200_device_ctx * ctx = (b200_device_ctx *) dev->context;
    for (int i = 0; i < LM_GGML_MAX_SRC; ++i) {
        const lm_ggml_tensor * s = op->src[i];
        if (s && s->buffer && buft_is_b200(s->buffer->buft) && ((b200_buft_ctx *) s->buffer->buft->context)->device != ctx->device) return false;
        if (s && s->buffer && buft_is_b200_split(s->buffer->buft)) {
            // a split tensor is the weight of a MUL_MAT on its main device and nothing else (norm weights, biases and the
            // embedding table that the loader probes with MUL / ADD / GET_ROWS go to the next buffer type of its list)
            if (op->op != LM_GGML_OP_MUL_MAT || i != 0) return false;
            if (((b200_split_buft_ctx *) s->buffer->buft->context)->main_device != ctx->device) return false;
        }
    }
    return b200_supports_op(op);
}

bool dev_supports_buft(lm_ggml_backend_dev_t dev, lm_ggml_backend_buffer_type_t buft) {
    const int device = ((b200_device_ctx *) dev->context)->device;
    if (buft_is_b200_split(buft)) return ((b200_split_buft_ctx *) buft->context)->main_device == device;
    return buft_is_b200(buft) && ((b200_buft_ctx *) buft->context)->device == device;
}

bool dev_offload_op(lm_ggml_backend_dev_t, const lm_ggml_tensor *) { return false; }

lm_ggml_backend_event_t dev_event_new(lm_ggml_backend_dev_t dev) {
    device_guard g(((b200_device_ctx *) dev->context)->device);
    cudaEvent_t ev;
    if (!cuda_ok(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate")) return nullptr;
    return new lm_ggml_backend_event{dev, ev};
}

void dev_event_free(lm_ggml_backend_dev_t dev, lm_ggml_backend_event_t event) {
    device_guard g(((b200_device_ctx *) dev->context)->device);
    cudaEventDestroy((cudaEvent_t) event->context);
    delete event;
}

void dev_event_synchronize(lm_ggml_backend_dev_t dev, lm_ggml_backend_event_t event) {
    device_guard g(((b200_device_ctx *) dev->context)->device);
    cuda_ok(cudaEventSynchronize((cudaEvent_t) event->context), "cudaEventSynchronize");
}

const lm_ggml_backend_device_i b200_device_iface = {
    /* .get_name             = */ dev_get_name,
    /* .get_description      = */ dev_get_description,
    /* .get_memory           = */ dev_get_memory,
    /* .get_type             = */ dev_get_type,
    /* .get_props            = */ dev_get_props,
    /* .init_backend         = */ dev_init_backend,
    /* .get_buffer_type      = */ dev_get_buffer_type,
    /* .get_host_buffer_type = */ dev_get_host_buffer_type,
    /* .buffer_from_host_ptr = */ nullptr,
    /* .supports_op          = */ dev_supports_op,
    /* .supports_buft        = */ dev_supports_buft,
    /* .offload_op           = */ dev_offload_op,
    /* .event_new            = */ dev_event_new,
    /* .event_free           = */ dev_event_free,
    /* .event_synchronize    = */ dev_event_synchronize,
};

// ---------------------------------------------------------------------------------------------
// reg
// ---------------------------------------------------------------------------------------------
const char * reg_get_name(lm_ggml_backend_reg_t) { return LM_GGML_B200_NAME; }
size_t reg_get_device_count(lm_ggml_backend_reg_t) { return registry()->devices.size(); }
lm_ggml_backend_dev_t reg_get_device(lm_ggml_backend_reg_t, size_t index) {
    LM_GGML_ASSERT(index < registry()->devices.size());
    return &registry()->devices[index];
}

void set_abort_callback(lm_ggml_backend_t backend, lm_ggml_abort_callback cb, void * data) {
    if (!lm_ggml_backend_is_b200(backend)) return;
    b200_backend_ctx * ctx = (b200_backend_ctx *) backend->context;
    ctx->abort_cb = cb;
    ctx->abort_cb_data = data;
}

lm_ggml_backend_feature * get_features(lm_ggml_backend_reg_t) {
    static lm_ggml_backend_feature features[] = {
        {"ARCH", "sm_100a"}, {"MMQ", "int8 mma + f32x2"}, {"FLASH_ATTN", "1"}, {"Q8_0_QUANTIZER", "AVX2-exact"}, {nullptr, nullptr},
    };
    return features;
}

// lm_ggml_backend_split_buffer_type_t (cactus/ggml-backend.h:188): tensor_split holds one share per device, all zero
// (or null) meaning equal shares.  One buffer type per distinct (main device, shares), never freed.
lm_ggml_backend_buffer_type_t split_buffer_type(int main_device, const float * tensor_split) {
    static std::mutex mu;
    static std::vector<lm_ggml_backend_buffer_type *> made;
    b200_registry * r = registry();
    const int n = (int) r->devices.size();
    if (main_device < 0 || main_device >= n) return nullptr;
    float share[LM_GGML_B200_MAX_DEVICES], sum = 0.0f;
    for (int i = 0; i < n; ++i) {
        share[i] = tensor_split ? std::max(0.0f, tensor_split[i]) : 0.0f;
        sum += share[i];
    }
    if (sum <= 0.0f) {
        for (int i = 0; i < n; ++i) share[i] = 1.0f;
        sum = (float) n;
    }
    float cum[LM_GGML_B200_MAX_DEVICES + 1] = {0.0f};
    for (int i = 0; i < n; ++i) cum[i + 1] = cum[i] + share[i] / sum;
    std::lock_guard<std::mutex> lock(mu);
    for (lm_ggml_backend_buffer_type * t : made) {
        const b200_split_buft_ctx * bc = (const b200_split_buft_ctx *) t->context;
        if (bc->main_device == main_device && bc->n_dev == n && memcmp(bc->cum, cum, sizeof(float) * (n + 1)) == 0) return t;
    }
    b200_split_buft_ctx * bc = new b200_split_buft_ctx;
    bc->main_device = main_device;
    bc->n_dev = n;
    memcpy(bc->cum, cum, sizeof(cum));
    bc->name = std::string(LM_GGML_B200_NAME) + "_Split";
    made.push_back(new lm_ggml_backend_buffer_type{b200_split_buft_iface, &r->devices[main_device], bc});
    return made.back();
}

// Extension proc: the next upload from `mask_host_data` (mask_bytes = n_kv * pad64(n_tokens) * 4) is a mask that was not
// filled; what it would hold follows from the cells and tokens given here.  Null mask_host_data withdraws the hint.
void kq_mask_from_cells(const void * mask_host_data, size_t mask_bytes, const int32_t * cell_pos, const int32_t * cell_seq, int64_t n_kv,
                        const int32_t * tok_pos, const int32_t * tok_seq, int64_t n_tokens) {
    kq_mask_hint_t & h = g_kq_hint;
    std::lock_guard<std::mutex> lock(h.mu);
    h.serial++;
    h.host_mask = nullptr;
    if (!mask_host_data || !cell_pos || !cell_seq || !tok_pos || !tok_seq || n_kv <= 0 || n_tokens <= 0) return;
    if (mask_bytes != (size_t) n_kv * (size_t) ((n_tokens + 63) / 64 * 64) * sizeof(float)) return;
    h.cell_pos.assign(cell_pos, cell_pos + n_kv);
    h.cell_seq.assign(cell_seq, cell_seq + n_kv);
    h.tok_pos.assign(tok_pos, tok_pos + n_tokens);
    h.tok_seq.assign(tok_seq, tok_seq + n_tokens);
    h.host_mask = mask_host_data;
    h.host_bytes = mask_bytes;
}
uint64_t kq_masks_built() { return g_kq_hint.masks_built.load(); }
void graph_counts(uint64_t * recorded, uint64_t * replayed) {
    if (recorded) *recorded = g_graph_records.load();
    if (replayed) *replayed = g_graph_replays.load();
}

void fused_group_counts(uint64_t * rope_stores, uint64_t * add_norms) {
    if (rope_stores) *rope_stores = g_rope_store_groups.load();
    if (add_norms) *add_norms = g_add_norm_groups.load();
}
void timing_totals(double * device_ms, uint64_t * graphs) {
    std::lock_guard<std::mutex> lock(g_totals_mu);
    if (device_ms) *device_ms = g_total_device_ms;
    if (graphs) *graphs = g_total_timed_graphs;
}

void * reg_get_proc_address(lm_ggml_backend_reg_t, const char * name) {
    if (strcmp(name, "lm_ggml_backend_b200_kq_mask_from_cells") == 0) return (void *) kq_mask_from_cells;
    if (strcmp(name, "lm_ggml_backend_b200_kq_masks_built") == 0) return (void *) kq_masks_built;
    if (strcmp(name, "lm_ggml_backend_b200_timing_totals") == 0) return (void *) timing_totals;
    if (strcmp(name, "lm_ggml_backend_b200_fused_group_counts") == 0) return (void *) fused_group_counts;
    if (strcmp(name, "lm_ggml_backend_b200_graph_counts") == 0) return (void *) graph_counts;
    if (strcmp(name, "lm_ggml_backend_split_buffer_type") == 0) return (void *) split_buffer_type;
    if (strcmp(name, "lm_ggml_backend_set_abort_callback") == 0) return (void *) set_abort_callback;
    if (strcmp(name, "lm_ggml_backend_get_features") == 0) return (void *) get_features;
    if (strcmp(name, "lm_ggml_backend_b200_get_stats") == 0) return (void *) lm_ggml_backend_b200_get_stats;
    return nullptr;
}

const lm_ggml_backend_reg_i b200_reg_iface = {
    /* .get_name         = */ reg_get_name,
    /* .get_device_count = */ reg_get_device_count,
    /* .get_device       = */ reg_get_device,
    /* .get_proc_address = */ reg_get_proc_address,
};

b200_registry * registry() {
    static b200_registry * r = nullptr;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (r) return r;
    r = new b200_registry;  // never freed: the registry of the host keeps pointers into it (cactus/ggml-backend-reg.cpp:195-203)
    const int n = std::min(b200_device_count(), LM_GGML_B200_MAX_DEVICES);
    r->reg = {LM_GGML_BACKEND_API_VERSION, b200_reg_iface, nullptr};
    r->devices.reserve(n);
    r->bufts.reserve(n);
    for (int i = 0; i < n; ++i) {
        char name[128] = "";
        b200_device_info(i, name, sizeof(name), nullptr, nullptr, nullptr);
        b200_device_ctx * dc = new b200_device_ctx{i, std::string(LM_GGML_B200_NAME) + "_" + std::to_string(i), name};
        r->ctxs.push_back(dc);
        r->devices.push_back({b200_device_iface, &r->reg, dc});
        b200_buft_ctx * bc = new b200_buft_ctx{i, std::string(LM_GGML_B200_NAME) + "_" + std::to_string(i)};
        r->buft_ctxs.push_back(bc);
        r->bufts.push_back({b200_buft_iface, &r->devices[i], bc});
    }
    r->host_buft = {b200_host_buft_iface, n > 0 ? &r->devices[0] : nullptr, nullptr};
    return r;
}

lm_ggml_backend_buffer_type_t device_buffer_type(int device) {
    b200_registry * r = registry();
    if (device < 0 || device >= (int) r->bufts.size()) return nullptr;
    return &r->bufts[device];
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// public entry points
// ---------------------------------------------------------------------------------------------
extern "C" {

lm_ggml_backend_reg_t lm_ggml_backend_b200_reg(void) { return &registry()->reg; }

lm_ggml_backend_buffer_type_t lm_ggml_backend_b200_buffer_type(int device) { return device_buffer_type(device); }

lm_ggml_backend_buffer_type_t lm_ggml_backend_b200_host_buffer_type(void) { return &registry()->host_buft; }

bool lm_ggml_backend_is_b200(lm_ggml_backend_t backend) { return backend != nullptr && lm_ggml_guid_matches(backend->guid, b200_guid()); }

lm_ggml_backend_t lm_ggml_backend_b200_init(int device) {
    b200_registry * r = registry();
    if (device < 0 || device >= (int) r->devices.size()) {
        B200_LOG_ERROR("ggml-b200: no B200 device %d (found %zu)\n", device, r->devices.size());
        return nullptr;
    }
    device_guard g(device);
    b200_backend_ctx * ctx = new b200_backend_ctx;
    ctx->device = device;
    ctx->name = std::string(LM_GGML_B200_NAME) + "_" + std::to_string(device);
    if (!cuda_ok(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking), "cudaStreamCreate")) {
        delete ctx;
        return nullptr;
    }
    const char * v = getenv("B200_Q8_VARIANT");
    if (v && strcmp(v, "scalar") == 0) ctx->q8_variant = B200_Q8_SCALAR;
    const char * fu = getenv("B200_FUSE");
    ctx->fuse = !(fu && atoi(fu) == 0);
    const char * sk = getenv("B200_STACK");
    ctx->stack = !(sk && atoi(sk) == 0);
    const char * gr = getenv("B200_GRAPHS");
    ctx->graphs = !(gr && atoi(gr) == 0);
    const char * fp = getenv("B200_FA_PARITY");
    ctx->fa_parity = fp && atoi(fp) != 0;
    const char * t = getenv("B200_TIMING");
    ctx->timing = t && atoi(t) != 0;
    cudaEventCreate(&ctx->ev0);
    cudaEventCreate(&ctx->ev1);
    return new lm_ggml_backend{b200_guid(), b200_backend_iface, &r->devices[device], ctx};
}

uint64_t lm_ggml_backend_b200_split_mul_mat_count(void) { return g_split_mul_mats.load(); }

void lm_ggml_backend_b200_get_stats(lm_ggml_backend_t backend, struct lm_ggml_b200_stats * out) {
    if (!lm_ggml_backend_is_b200(backend)) {
        memset(out, 0, sizeof(*out));
        return;
    }
    *out = ((b200_backend_ctx *) backend->context)->stats;
}

// dynamic loading: lm_ggml_backend_load() looks this symbol up (cactus/ggml-backend-reg.cpp:236-252)
LM_GGML_BACKEND_API lm_ggml_backend_reg_t lm_ggml_backend_init(void) { return lm_ggml_backend_b200_reg(); }
LM_GGML_BACKEND_API int lm_ggml_backend_score(void) { return b200_device_count() > 0 ? 100 : 0; }

}  // extern "C"
