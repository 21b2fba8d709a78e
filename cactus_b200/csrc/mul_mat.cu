// C ABI of MUL_MAT: argument checks and the choice between the dp4a kernel (N <= 8) and the
// tensor-core kernel (N > 8).
#include "common.cuh"

namespace b200 {
int launch_quantize_b8(const float *x, int64_t x_nb_row, int64_t K, int64_t N, void *scratch, int variant, cudaStream_t st);
int launch_mmvq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row, cudaStream_t st);
int launch_mmq(int wtype, const TiledDims &d, const void *w, const ActDims &a, const void *aq, float *dst, int64_t dst_nb_row,
               void *workspace, size_t workspace_bytes, cudaStream_t st);
size_t mmq_workspace_bytes(int wtype, int64_t K, int64_t M, int64_t N);
}  // namespace b200

using namespace b200;

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

int b200_mul_mat_q_prequant(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, float *dst,
                            int64_t dst_row_stride_bytes, void *workspace, size_t workspace_bytes, b200_stream_t stream) {
    B200_REQUIRE(shape_ok(wtype, K, M, N), "bad mul_mat shape/type: type %d K %lld M %lld N %lld", wtype, (long long) K, (long long) M, (long long) N);
    B200_REQUIRE(w && act && dst, "null pointer");
    B200_REQUIRE(is_aligned(w, 16) && is_aligned(act, 256) && is_aligned(dst, 4), "misaligned pointer");
    B200_REQUIRE(dst_row_stride_bytes % 4 == 0 && dst_row_stride_bytes >= M * 4, "bad dst row stride");
    B200_REQUIRE(!workspace || is_aligned(workspace, 256), "workspace must be 256-byte aligned");
    const TiledDims d = tiled_dims(wtype, K, M);
    const ActDims a = act_dims(K, N);
    if (N <= 8) return launch_mmvq(wtype, d, w, a, act, dst, dst_row_stride_bytes, (cudaStream_t) stream);
    return launch_mmq(wtype, d, w, a, act, dst, dst_row_stride_bytes, workspace, workspace_bytes, (cudaStream_t) stream);
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

}  // extern "C"
