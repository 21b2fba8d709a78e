// Measures the issue-to-completion rate of tcgen05.mma on one SM (or all SMs): one thread issues 512 MMAs of a given
// kind and shape back to back (operands static zeros in shared / tensor memory, every wait bounded), the commit's
// arrival is timed with clock64.  Prints clocks per MMA and multiply-accumulates per clock and SM: the tensor-core
// peaks the roofline notes quote (s8 and e4m3 run at the same rate; fp16 at half of it; M = 64 or N = 64 at a reduced
// rate).  Built and run by `python -m cactus_b200.microbench umma-rate`.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t) ((addr >> 4) & 0x3FFF) | ((uint64_t) ((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t) ((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
template <int KIND, int TS, int ACC>
__device__ __forceinline__ void mma(uint32_t d, uint64_t adesc, uint32_t a_t, uint64_t bdesc, uint32_t idesc) {
    if (KIND == 2) {
        if (TS) asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d), "r"(a_t), "l"(bdesc), "r"(idesc), "r"(ACC) : "memory");
        else    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(ACC) : "memory");
        return;
    }
    if (KIND == 0) {
        if (TS) asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d), "r"(a_t), "l"(bdesc), "r"(idesc) : "memory");
        else    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
    } else if (KIND == 1) {
        if (TS) asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\ntcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d), "r"(a_t), "l"(bdesc), "r"(idesc) : "memory");
        else    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\ntcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
    } else {
        asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
    }
}
template <int KIND, int TS, int M, int N, int ACC, int NT>
__global__ void __launch_bounds__(128) rate(int reps, long long *clk, int *err) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t slot;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < 12288 / 4; i += 128) reinterpret_cast<uint32_t *>(smem)[i] = 0;
    const uint32_t bar_u = (uint32_t) __cvta_generic_to_shared(&bar);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_u));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"((uint32_t) __cvta_generic_to_shared(&slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = slot;
    for (int c = 0; c < 512; c += 8)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};\n" ::"r"(tmem + ((uint32_t) (32 * warp) << 16) + c), "r"(0) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t fmt = KIND == 0 ? ((2u << 4) | (1u << 7) | (1u << 10)) : (1u << 4);
    const uint32_t idesc = fmt | ((uint32_t) (N >> 3) << 17) | ((uint32_t) (M >> 4) << 24);
    const uint32_t sa = (uint32_t) __cvta_generic_to_shared(smem);
    const uint64_t adesc = smem_desc(sa, 128, 256), bdesc = smem_desc(sa + 4096, 128, 256);
    constexpr int TILES = NT;   // D tiles used in turn
    const uint32_t a_t = tmem + 504;
    if (tid == 0) {
        const long long t0 = clock64();
        for (int r = 0; r < reps; ++r) {
#pragma unroll
            for (int j = 0; j < 8; ++j) mma<KIND, TS, ACC>(tmem + (uint32_t) ((j % TILES) * N), adesc, a_t, bdesc, idesc);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar_u) : "memory");
        if (!bar_wait(bar_u, 0)) *err = 1;
        const long long t1 = clock64();
        if (blockIdx.x == 0) clk[0] = t1 - t0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}
long long *dclk; int *derr;
template <int KIND, int TS, int M, int N, int ACC, int NT>
void run(int grid) {
    const char *kn[3] = {"i8 ", "f8 ", "f16"};
    cudaFuncSetAttribute(rate<KIND, TS, M, N, ACC, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384);
    rate<KIND, TS, M, N, ACC, NT><<<grid, 128, 16384>>>(64, dclk, derr);
    cudaError_t e = cudaDeviceSynchronize();
    long long clk = 0; int err = 0;
    cudaMemcpy(&clk, dclk, 8, cudaMemcpyDeviceToHost); cudaMemcpy(&err, derr, 4, cudaMemcpyDeviceToHost);
    const double per = (double) clk / 512;
    printf("  %s M %3d N %3d %s acc %d tiles %d: %7.1f clk per MMA, %6.0f MAC/clk/SM  (%s, err %d)\n", kn[KIND], M, N, TS ? "TS" : "SS", ACC, NT, per, (double) M * N * (KIND == 2 ? 16 : 32) / per, cudaGetErrorString(e), err);
    if (e != cudaSuccess) exit(1);
}
int main() {
    cudaMalloc(&dclk, 64); cudaMalloc(&derr, 4); cudaMemset(derr, 0, 4);
    for (int grid : {1, 148}) {
        printf("grid %d\n", grid);
        run<0, 0, 128, 64, 0, 4>(grid); run<0, 0, 128, 128, 0, 4>(grid); run<0, 0, 128, 256, 0, 2>(grid);
        run<1, 0, 128, 64, 0, 4>(grid); run<1, 0, 128, 128, 0, 4>(grid); run<1, 0, 128, 256, 0, 2>(grid);
        run<1, 1, 128, 64, 1, 1>(grid); run<1, 1, 128, 128, 1, 1>(grid); run<1, 0, 64, 256, 0, 2>(grid);
        run<2, 0, 128, 64, 1, 1>(grid); run<2, 0, 128, 128, 1, 1>(grid); run<2, 0, 128, 256, 1, 1>(grid);
        run<2, 1, 128, 64, 1, 1>(grid); run<2, 1, 128, 128, 1, 1>(grid); run<2, 1, 128, 256, 1, 1>(grid);
    }
    return 0;
}
