// Row-split mul_mat across the GPUs of one node: the exchange step.
//
// With the rows of every mul_mat weight split over g GPUs (what a split buffer type does for
// LLAMA_SPLIT_MODE_ROW, cactus/ggml-backend.h:188, cactus/llama-model.cpp:339-351), each GPU computes
// dst[:, r*M/g : (r+1)*M/g] and every GPU needs the whole dst for the next (replicated) op.  One process drives one
// GPU; the dst buffers live in memory shared through CUDA IPC, and the join is done by our own kernels over NVLink:
//   push     each GPU stores its slice into every GPU's dst buffer (plain stores to peer memory) -- from the write-back
//            of the mul_mat kernel itself (b200_mul_mat_q_rowsplit: no local copy of the slice, no separate pass), or
//            from a slice that already exists (b200_allgather_rows);
//   signal   after the push has completed in stream order, one thread per peer writes this collective's number into
//            that peer's flag word for us (st.release.sys);
//   wait     the same kernel then polls our own flag words until every peer's number has arrived.  The poll is
//            bounded: when it runs out, the kernel records the peer in an error word and returns; the host reads it
//            with b200_peer_status.
// The collective number lives in device memory and is advanced by the kernel, so a captured CUDA graph can be
// replayed.  No rank can be more than one collective ahead of another (it needs their flags to go on), and a dst
// buffer is reused at the earliest one layer later, so pushes never overwrite data a slower peer still reads.
#include "common.cuh"

namespace b200 {

constexpr uint32_t PEER_SPIN_LIMIT = 1u << 24;   // polls of a few hundred ns: seconds, then give up

struct PeerPtrs {
    void *p[8];
};

__global__ void __launch_bounds__(256) allgather_push_kernel(const float *__restrict__ src, int64_t src_nb_row, int64_t T, int64_t Mg,
                                                            PeerPtrs dst, int64_t dst_nb_row, int64_t col0, int g) {
    // one 16-byte chunk of the slice per thread and step, written to all g destinations
    const int64_t chunks_per_row = Mg / 4;
    const int64_t total = T * chunks_per_row;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t t = i / chunks_per_row, c = i - t * chunks_per_row;
        const float4 v = *reinterpret_cast<const float4 *>(reinterpret_cast<const char *>(src) + t * src_nb_row + c * 16);
#pragma unroll 8
        for (int r = 0; r < g; ++r) {
            *reinterpret_cast<float4 *>(reinterpret_cast<char *>(dst.p[r]) + t * dst_nb_row + (col0 + c * 4) * 4) = v;
        }
    }
}

// flags layout in every rank's shared block: uint32 arrived[8] (written by peers), then (local use only) uint32 counter, uint32 error,
// uint32 poll limit (0 = PEER_SPIN_LIMIT)
__global__ void allgather_signal_wait_kernel(PeerPtrs flags, int rank, int g) {
    uint32_t *mine = reinterpret_cast<uint32_t *>(flags.p[rank]);
    __shared__ uint32_t epoch;
    if (threadIdx.x == 0) epoch = mine[8] + 1;
    __syncthreads();
    const uint32_t e = epoch, limit = mine[10] ? mine[10] : PEER_SPIN_LIMIT;
    const int r = threadIdx.x;
    if (r < g) {
        uint32_t *theirs = reinterpret_cast<uint32_t *>(flags.p[r]) + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(theirs), "r"(e) : "memory");
        const uint32_t *from_r = mine + r;
        uint32_t spin = 0, v = 0;
        for (; spin < limit; ++spin) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(from_r) : "memory");
            if ((int32_t) (v - e) >= 0) break;
            __nanosleep(100);
        }
        if (spin == limit) atomicExch(mine + 9, (uint32_t) (r + 1));   // gave up on peer r
    }
    __syncthreads();
    if (threadIdx.x == 0) mine[8] = e;
}

int launch_peer_signal_wait(void *const *flags_of_rank, int rank, int g, cudaStream_t st) {
    PeerPtrs f;
    for (int r = 0; r < 8; ++r) f.p[r] = r < g ? flags_of_rank[r] : nullptr;
    allgather_signal_wait_kernel<<<1, 32, 0, st>>>(f, rank, g);
    return check_launch("allgather_signal_wait");
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_peer_alloc(size_t bytes, void **ptr, unsigned char handle[64]) {
    B200_REQUIRE(ptr && handle && bytes > 0, "null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return set_error(B200_E_CUDA, "peer_alloc %zu bytes: %s", bytes, cudaGetErrorString(e));
    e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return set_error(B200_E_CUDA, "peer_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, 64);
    *ptr = p;
    return B200_OK;
}

int b200_peer_open(const unsigned char handle[64], void **ptr) {
    B200_REQUIRE(ptr && handle, "null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return set_error(B200_E_CUDA, "peer_open: %s", cudaGetErrorString(e));
    *ptr = p;
    return B200_OK;
}

int b200_peer_close(void *ptr) {
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? B200_OK : set_error(B200_E_CUDA, "peer_close: %s", cudaGetErrorString(e));
}

int b200_peer_free(void *ptr) {
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? B200_OK : set_error(B200_E_CUDA, "peer_free: %s", cudaGetErrorString(e));
}

int b200_allgather_rows(const float *src, int64_t src_nb_row, int64_t T, int64_t Mg, int rank, int g, void *const *dst_of_rank,
                        int64_t dst_nb_row, void *const *flags_of_rank, b200_stream_t stream) {
    B200_REQUIRE(src && dst_of_rank && flags_of_rank, "null pointer");
    B200_REQUIRE(g >= 1 && g <= 8 && rank >= 0 && rank < g, "rank %d of %d: at most 8 GPUs", rank, g);
    B200_REQUIRE(T > 0 && Mg > 0 && Mg % 4 == 0 && src_nb_row % 16 == 0 && dst_nb_row % 16 == 0 && is_aligned(src, 16), "rows must be multiples of 16 bytes");
    PeerPtrs d, f;
    for (int r = 0; r < 8; ++r) {
        d.p[r] = r < g ? dst_of_rank[r] : nullptr;
        f.p[r] = r < g ? flags_of_rank[r] : nullptr;
        if (r < g) B200_REQUIRE(d.p[r] && f.p[r] && is_aligned(d.p[r], 16), "null or misaligned peer buffer %d", r);
    }
    cudaStream_t st = (cudaStream_t) stream;
    const int64_t total = T * (Mg / 4);
    const unsigned grid = (unsigned) std::min<int64_t>((total + 255) / 256, 592);
    allgather_push_kernel<<<grid, 256, 0, st>>>(src, src_nb_row, T, Mg, d, dst_nb_row, (int64_t) rank * Mg, g);
    if (int e = check_launch("allgather_push")) return e;
    return launch_peer_signal_wait(flags_of_rank, rank, g, st);
}

int b200_peer_set_wait_limit(void *flags, unsigned polls) {
    B200_REQUIRE(flags, "null pointer");
    const uint32_t v[2] = {0u, (uint32_t) polls};   // the error word and the limit sit side by side
    cudaError_t e = cudaMemcpy(reinterpret_cast<uint32_t *>(flags) + 9, v, sizeof(v), cudaMemcpyHostToDevice);
    return e == cudaSuccess ? B200_OK : set_error(B200_E_CUDA, "peer_set_wait_limit: %s", cudaGetErrorString(e));
}

int b200_peer_status(const void *flags) {
    B200_REQUIRE(flags, "null pointer");
    uint32_t v = 0;
    cudaError_t e = cudaMemcpy(&v, reinterpret_cast<const uint32_t *>(flags) + 9, sizeof(v), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return set_error(B200_E_CUDA, "peer_status: %s", cudaGetErrorString(e));
    return (int) v;
}

}  // extern "C"
