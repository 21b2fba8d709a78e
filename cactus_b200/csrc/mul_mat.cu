// C ABI of MUL_MAT: argument checks and the choice between the dp4a kernel (few columns, mmvq_max_n()) and the
// tensor-core kernels.
#include <mutex>

#include "common.cuh"

namespace b200 {
int act_layout(int64_t N);
int launch_mmq_tc(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
                  void *workspace, size_t workspace_bytes, cudaStream_t st);
int launch_mmq_tcf(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
                   void *workspace, size_t workspace_bytes, cudaStream_t st, int terms);
int mmq_tc_mode();
int mmvq_max_n();
int launch_mmvq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row, const PeerDst &peers,
                cudaStream_t st);
int launch_mmq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
               void *workspace, size_t workspace_bytes, cudaStream_t st, bool canon, const PeerDst &peers);
int launch_peer_signal_wait(void *const *flags_of_rank, int rank, int g, cudaStream_t st);
size_t mmq_workspace_bytes(int wtype, int64_t K, int64_t M, int64_t N);
}  // namespace b200

using namespace b200;

// ---------------------------------------------------------------------------------------------
// Scratch for b200_mul_mat_q_noalloc: room for the quantised activations of up to 8 columns of
// B200_NOALLOC_MAX_K values (one 8-column tile of 256-byte block groups plus its scale plane).
// The array lives in every device that loads this library, from load until the process exits.
// In host code the name below is only a handle for cudaGetSymbolAddress, never a device address.
// ---------------------------------------------------------------------------------------------
constexpr size_t NOALLOC_SCRATCH_BYTES = (size_t) B200_NOALLOC_MAX_K / 32 * 256 + (size_t) B200_NOALLOC_MAX_K / 128 * 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// device address of the array on the current device, looked up once per device
static int noalloc_scratch_ptr(void **out) {
    static void *ptrs[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(B200_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return set_error(B200_E_INVALID, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return set_error(B200_E_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return B200_OK;
}

static bool shape_ok(int wtype, int64_t K, int64_t M, int64_t N) {
    return (wtype == B200_TYPE_Q4_0 || wtype == B200_TYPE_Q8_0) && K > 0 && K % 32 == 0 && M > 0 && N > 0;
}

extern "C" {

size_t b200_mul_mat_workspace_bytes(int wtype, int64_t K, int64_t M, int64_t N) {
    if (!shape_ok(wtype, K, M, N)) return 0;
    return mmq_workspace_bytes(wtype, K, M, N);
}

size_t b200_mul_mat_scratch_bytes(int wtype, int64_t K, int64_t M, int64_t N) {
    if (!shape_ok(wtype, K, M, N)) return 0;
    return b200_act_bytes(K, N) + mmq_workspace_bytes(wtype, K, M, N);
}

static int mul_mat_prequant(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, float *dst, int64_t dst_row_stride_bytes,
                            void *workspace, size_t workspace_bytes, const PeerDst &peers, b200_stream_t stream);

int b200_mul_mat_q_prequant(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, float *dst,
                            int64_t dst_row_stride_bytes, void *workspace, size_t workspace_bytes, b200_stream_t stream) {
    return mul_mat_prequant(wtype, w, K, M, act, N, dst, dst_row_stride_bytes, workspace, workspace_bytes, PeerDst{}, stream);
}

static int rowsplit_impl(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, int rank, int g, void *const *dst_of_rank,
                         int64_t dst_row_stride_bytes, int64_t first_column, PeerDst peers, void *workspace, size_t workspace_bytes,
                         void *const *flags_of_rank, b200_stream_t stream);

int b200_mul_mat_q_rowsplit(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, int rank, int g, void *const *dst_of_rank,
                            int64_t dst_row_stride_bytes, int64_t first_column, void *workspace, size_t workspace_bytes,
                            void *const *flags_of_rank, b200_stream_t stream) {
    return rowsplit_impl(wtype, w, K, M, act, N, rank, g, dst_of_rank, dst_row_stride_bytes, first_column, PeerDst{}, workspace, workspace_bytes,
                         flags_of_rank, stream);
}

int b200_mul_mat_q_rowsplit_stacked(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, int rank, int g,
                                    void *const *dst_of_rank, int64_t dst_row_stride_bytes, int n_parts, const int64_t *part_rows,
                                    const int64_t *part_first_column, void *workspace, size_t workspace_bytes, void *const *flags_of_rank,
                                    b200_stream_t stream) {
    B200_REQUIRE(n_parts >= 1 && n_parts <= 3 && part_rows && part_first_column, "a stacked weight has 1 to 3 parts");
    PeerDst peers = {};
    peers.n_seg = n_parts;
    int64_t row = 0;
    for (int i = 0; i < n_parts; ++i) {
        B200_REQUIRE(part_rows[i] > 0 && part_first_column[i] >= 0 && (i == n_parts - 1 || part_rows[i] % 16 == 0), "parts but the last hold a multiple of 16 rows");
        // a plain mapping puts local row r at column part_first_column[0] + r
        peers.seg_shift[i] = (part_first_column[i] - (part_first_column[0] + row)) * 4;
        row += part_rows[i];
        if (i < 2) peers.seg_end[i] = (int) row;
    }
    B200_REQUIRE(row == M, "the parts hold %lld rows, the weight %lld", (long long) row, (long long) M);
    return rowsplit_impl(wtype, w, K, M, act, N, rank, g, dst_of_rank, dst_row_stride_bytes, part_first_column[0], peers, workspace, workspace_bytes,
                         flags_of_rank, stream);
}

static int rowsplit_impl(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, int rank, int g, void *const *dst_of_rank,
                         int64_t dst_row_stride_bytes, int64_t first_column, PeerDst peers, void *workspace, size_t workspace_bytes,
                         void *const *flags_of_rank, b200_stream_t stream) {
    B200_REQUIRE(dst_of_rank && flags_of_rank && g >= 1 && g <= 8 && rank >= 0 && rank < g && first_column >= 0, "bad row-split arguments");
    float *own = nullptr;
    for (int r = 0; r < g; ++r) {
        B200_REQUIRE(dst_of_rank[r] && flags_of_rank[r], "null buffer of rank %d", r);
        float *p = reinterpret_cast<float *>(dst_of_rank[r]) + first_column;
        if (r == rank) own = p;
        else peers.p[peers.n++] = p;
    }
    if (int e = mul_mat_prequant(wtype, w, K, M, act, N, own, dst_row_stride_bytes, workspace, workspace_bytes, peers, stream)) return e;
    return launch_peer_signal_wait(flags_of_rank, rank, g, (cudaStream_t) stream);
}

static int mul_mat_prequant(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, float *dst, int64_t dst_row_stride_bytes,
                            void *workspace, size_t workspace_bytes, const PeerDst &peers, b200_stream_t stream) {
    B200_REQUIRE(shape_ok(wtype, K, M, N), "bad mul_mat shape/type: type %d K %lld M %lld N %lld", wtype, (long long) K, (long long) M, (long long) N);
    B200_REQUIRE(w && act && dst, "null pointer");
    B200_REQUIRE(is_aligned(w, 16) && is_aligned(act, 256) && is_aligned(dst, 4), "misaligned pointer");
    B200_REQUIRE(dst_row_stride_bytes % 4 == 0 && dst_row_stride_bytes >= M * 4, "bad dst row stride");
    B200_REQUIRE(!workspace || is_aligned(workspace, 256), "workspace must be 256-byte aligned");
    const TiledDims d = tiled_dims(wtype, K, M);
    const ActDims a = act_dims(K, N);
    if (N <= mmvq_max_n()) return launch_mmvq(wtype, d, w, a, act, dst, dst_row_stride_bytes, peers, (cudaStream_t) stream);
    // the tcgen05 kernel reads the e4m3 planes, multiplies Q4_0 weights and writes one destination; everything else (Q8_0
    // weights, a row-split product) takes the mma.sync kernel on the fragment-order plane that is always there
    if (act_layout(N) == 3 && wtype == B200_TYPE_Q4_0 && peers.n == 0 && peers.n_seg <= 1) {
        return launch_mmq_tc(wtype, d, w, a, act, dst, dst_row_stride_bytes, workspace, workspace_bytes, (cudaStream_t) stream);
    }
    if (mmq_tc_mode() >= 2 && N >= 16 && wtype == B200_TYPE_Q4_0 && peers.n == 0 && peers.n_seg <= 1) {
        return launch_mmq_tcf(wtype, d, w, a, act, dst, dst_row_stride_bytes, workspace, workspace_bytes, (cudaStream_t) stream, mmq_tc_mode() == 2 ? 3 : 2);
    }
    return launch_mmq(wtype, d, w, a, act, dst, dst_row_stride_bytes, workspace, workspace_bytes, (cudaStream_t) stream, false, peers);
}

int b200_mul_mat_q_prequant_multi(int wtype, int n_weights, const void *const *w, const int64_t *M, int64_t K, const void *act, int64_t N,
                                  float *const *dst, int64_t dst_row_stride_bytes, void *workspace, size_t workspace_bytes, b200_stream_t stream) {
    B200_REQUIRE(n_weights >= 1 && n_weights <= 3 && w && M && dst, "1 to 3 weights");
    int64_t total = 0;
    bool whole_groups = true;
    for (int i = 0; i < n_weights; ++i) {
        B200_REQUIRE(w[i] && dst[i] && M[i] > 0 && is_aligned(w[i], 16) && is_aligned(dst[i], 4), "null or misaligned weight / destination %d", i);
        whole_groups = whole_groups && (i == n_weights - 1 || M[i] % 128 == 0);
        total += M[i];
    }
    // one launch needs whole row groups per tensor and the tensor-core kernel; otherwise one product after the other
    if (n_weights == 1 || !whole_groups || N <= mmvq_max_n()) {
        for (int i = 0; i < n_weights; ++i)
            if (int e = b200_mul_mat_q_prequant(wtype, w[i], K, M[i], act, N, dst[i], dst_row_stride_bytes, workspace, workspace_bytes, stream)) return e;
        return B200_OK;
    }
    B200_REQUIRE(shape_ok(wtype, K, total, N), "bad mul_mat shape/type: type %d K %lld M %lld N %lld", wtype, (long long) K, (long long) total, (long long) N);
    B200_REQUIRE(act && is_aligned(act, 256), "null or misaligned activations");
    B200_REQUIRE(dst_row_stride_bytes % 4 == 0, "bad dst row stride");
    B200_REQUIRE(!workspace || is_aligned(workspace, 256), "workspace must be 256-byte aligned");
    PeerDst segs = {};
    segs.n_seg = n_weights;
    segs.n_wseg = n_weights;
    int64_t row = 0;
    for (int i = 0; i < n_weights; ++i) {
        B200_REQUIRE(dst_row_stride_bytes >= M[i] * 4, "bad dst row stride");
        segs.wseg[i] = (const unsigned char *) w[i];
        segs.wseg_qs[i] = (unsigned long long) tiled_dims(wtype, K, M[i]).qs_bytes;
        // a plain mapping puts row r of the stacked product at dst[0] + r floats
        segs.seg_shift[i] = (int64_t) ((const char *) dst[i] - (const char *) dst[0]) - row * 4;
        row += M[i];
        if (i < 2) segs.seg_end[i] = (int) row;
    }
    const TiledDims d = tiled_dims(wtype, K, total);
    const ActDims a = act_dims(K, N);
    return launch_mmq(wtype, d, w[0], a, act, dst[0], dst_row_stride_bytes, workspace, workspace_bytes, (cudaStream_t) stream, false, segs);
}

int b200_mul_mat_q(int wtype, const void *w, int64_t K, int64_t M, const float *x, int64_t x_row_stride_bytes, int64_t N,
                   float *dst, int64_t dst_row_stride_bytes, void *scratch, size_t scratch_bytes, int variant, b200_stream_t stream) {
    B200_REQUIRE(shape_ok(wtype, K, M, N), "bad mul_mat shape/type: type %d K %lld M %lld N %lld", wtype, (long long) K, (long long) M, (long long) N);
    const size_t ab = b200_act_bytes(K, N);
    const size_t wb = mmq_workspace_bytes(wtype, K, M, N);
    if (!scratch || scratch_bytes < ab + wb) return set_error(B200_E_SCRATCH, "scratch too small: %zu < %zu", scratch_bytes, ab + wb);
    if (int e = b200_quantize_activations(x, x_row_stride_bytes, K, N, scratch, ab, variant, stream)) return e;
    return b200_mul_mat_q_prequant(wtype, w, K, M, scratch, N, dst, dst_row_stride_bytes, wb ? (char *) scratch + ab : nullptr, wb, stream);
}

int b200_mul_mat_q_noalloc(int wtype, const void *w, int64_t K, int64_t M, const float *x, int64_t x_row_stride_bytes, int64_t N,
                           float *dst, int64_t dst_row_stride_bytes, int variant, b200_stream_t stream) {
    B200_REQUIRE(shape_ok(wtype, K, M, N), "bad mul_mat shape/type: type %d K %lld M %lld N %lld", wtype, (long long) K, (long long) M, (long long) N);
    B200_REQUIRE(N <= B200_NOALLOC_MAX_N, "b200_mul_mat_q_noalloc handles at most %d columns, got %lld", B200_NOALLOC_MAX_N, (long long) N);
    B200_REQUIRE(K <= B200_NOALLOC_MAX_K, "b200_mul_mat_q_noalloc handles rows of at most %d values, got %lld", B200_NOALLOC_MAX_K, (long long) K);
    const size_t ab = b200_act_bytes(K, N);
    B200_REQUIRE(ab <= NOALLOC_SCRATCH_BYTES, "built-in scratch too small for K %lld", (long long) K);
    void *scratch = nullptr;
    if (int e = noalloc_scratch_ptr(&scratch)) return e;
    // the quantiser rewrites every byte of the region it uses (padding included), so nothing has to be cleared
    if (int e = b200_quantize_activations(x, x_row_stride_bytes, K, N, scratch, ab, variant, stream)) return e;
    return b200_mul_mat_q_prequant(wtype, w, K, M, scratch, N, dst, dst_row_stride_bytes, nullptr, 0, stream);
}

}  // extern "C"
