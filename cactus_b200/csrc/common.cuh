// Shared device/host helpers for the sm_100a kernels: error plumbing, the tiled weight layout ("T16")
// and the activation scratch layout ("B8").
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cactus_b200.h"

namespace b200 {

// ---- error plumbing ---------------------------------------------------------------------------
int set_error(int code, const char *fmt, ...);
void count_launch(int n = 1);
int check_launch(const char *what);  // cudaGetLastError after a launch -> B200_E_CUDA or 0

#define B200_REQUIRE(cond, ...)                                   \
    do {                                                          \
        if (!(cond)) return b200::set_error(B200_E_INVALID, __VA_ARGS__); \
    } while (0)

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- programmatic dependent launch ---------------------------------------------------------------
// The kernels of a decode step run back to back on one stream, each a few to a few dozen microseconds long.  A kernel
// launched with launch_pdl may have its CTAs placed on the SMs while the previous kernel's last CTAs are still running;
// its first statement (pdl_prologue) waits until the previous kernel has completed and its writes are visible, so only
// the launch itself and the CTA start-up overlap.  B200_PDL=0 turns the launch attribute off.
bool pdl_enabled();
// With a single token row every kernel of a step is a few microseconds of latency and the weight stream of a product
// waits behind each of them.  Up to this many rows (B200_PDL_EARLY_ROWS, default 1; 0 switches it off) the row kernels
// let the next kernel's CTAs take their places at once (pdl_prologue(true)), and the few-column product asks for its
// weights -- which no kernel of a step writes -- to be brought into L2 before it waits for the kernel ahead of it.
int pdl_early_rows();
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_prologue() {
#ifdef B200_PDL_EARLY_TRIGGER   // lets the next kernel's CTAs take their places for the whole run of this one: measured slower
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
#endif
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_prologue(bool early) {
    if (early) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
}
// a hint without effect on results: `bytes` (a multiple of 16) from the 16-byte aligned global address p are wanted in L2
__device__ __forceinline__ void prefetch_l2_bulk(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(__cvta_generic_to_global(p)), "r"(bytes) : "memory");
}
// placed where a long kernel's CTA has only its write-back left: once every CTA of the grid is there (or gone), the next
// kernel's CTAs may be placed
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
template <typename... P, typename... A>
static inline cudaError_t launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}
#endif
static inline bool is_aligned(const void *p, size_t a) { return ((uintptr_t) p % a) == 0; }

// ---- row split: the other GPUs' copies of a product ------------------------------------------------
// A mul_mat kernel stores every result value into its own dst and, when the weight is one row slice of a split, into
// the same place of the other GPUs' output buffers (peer memory mapped through CUDA IPC): p[i] is the address in peer
// i's buffer that corresponds to `dst`, the row stride is the same everywhere.
// A stacked weight (the q, k, v rows -- or gate and up rows -- of one rank, one after the other) produces up to three
// row ranges that belong at different columns of dst: rows from seg_end[i-1] on land seg_shift[i] bytes further than a
// plain row-to-column mapping would put them (n_seg <= 1: no such ranges).  Ranges start on multiples of 16 rows.
struct PeerDst {
    float *p[7];
    int n;
    int n_seg;
    int seg_end[2];
    int64_t seg_shift[3];
    // The same row ranges can also come from separate weight tensors (ggml allocates a layer's gate and up projections
    // one by one; multiplying both by the same activations in one launch fills the GPU better than two launches): range i
    // then reads wseg[i] (scales wseg_qs[i] bytes further) instead of a slice of one stacked tensor.  n_wseg = 0: one
    // tensor.  Ranges then start on multiples of 128 rows (whole row groups of every kernel shape).
    int n_wseg;
    const unsigned char *wseg[3];
    unsigned long long wseg_qs[3];
};
#ifdef __CUDACC__
__device__ __forceinline__ int64_t peer_row_shift(const PeerDst &peers, int64_t row) {
    if (peers.n_seg <= 1 || row < peers.seg_end[0]) return 0;
    return (peers.n_seg > 2 && row >= peers.seg_end[1]) ? peers.seg_shift[2] : peers.seg_shift[1];
}
__device__ __forceinline__ void store_f32(float *dst, const PeerDst &peers, int64_t byte_off, float v) {
    *reinterpret_cast<float *>(reinterpret_cast<char *>(dst) + byte_off) = v;
    for (int i = 0; i < peers.n; ++i) *reinterpret_cast<float *>(reinterpret_cast<char *>(peers.p[i]) + byte_off) = v;
}
#endif

// ---- T16: tiled quantised weights ---------------------------------------------------------------
// A [K, M] tensor (M rows of K/32 blocks) is padded to Mp = ceil16(M) rows and nbp = ceil4(K/32) blocks and cut
// into tiles of 16 rows x 4 blocks.  Tile (rt, bg) is stored in the register order of an m16n8k32
// tensor-core A fragment, lane = 4*g + t owning rows g and g+8:
//   Q4_0: 1024 B per tile, 32 B per lane: [row g : word t of blocks 0..3][row g+8 : word t of blocks 0..3]
//         where "word t" is bytes 4t..4t+3 of the block's 16 nibble bytes, each byte XOR 0x88 so that
//         both nibbles hold (value - 8) as 4-bit two's complement.  Low nibbles are elements 4t..4t+3,
//         high nibbles elements 16+4t..16+4t+3.
//   Q8_0: 2048 B per tile = 4 blocks x 512 B, 16 B per lane and block:
//         [row g word t][row g+8 word t][row g word 4+t][row g+8 word 4+t]   (word = 4 consecutive int8)
// The fp16 scales follow in a second plane: 128 B per tile, half index 4*r + j for row r and block j.
struct TiledDims {
    int64_t M, K, nb;        // logical rows, columns, blocks per row
    int64_t Mp, nbp;         // padded rows (x16) and blocks (x4)
    int64_t n_rt, n_bg;      // row tiles, block groups
    int64_t tile_bytes;      // 1024 (Q4_0) or 2048 (Q8_0)
    size_t qs_bytes;         // size of the quant plane = offset of the scale plane
    size_t total_bytes;
};

__host__ __device__ static inline TiledDims tiled_dims(int wtype, int64_t K, int64_t M) {
    TiledDims d;
    d.M = M;
    d.K = K;
    d.nb = K / 32;
    d.Mp = (M + 15) / 16 * 16;
    d.nbp = (d.nb + 3) / 4 * 4;
    d.n_rt = d.Mp / 16;
    d.n_bg = d.nbp / 4;
    d.tile_bytes = (wtype == B200_TYPE_Q4_0) ? 1024 : 2048;
    d.qs_bytes = (size_t) d.n_rt * d.n_bg * d.tile_bytes;
    d.total_bytes = d.qs_bytes + (size_t) d.n_rt * d.n_bg * 128;
    return d;
}

// ---- B8: quantised activations (internal scratch) ------------------------------------------------
// N rows (columns of the product) of K floats are quantised to Q8_0 and stored in groups of 8 rows
// ("n-tiles") in the register order of an m16n8k32 B fragment: for n-tile nt and block b, 256 B at
// (nt*nbp + b)*256, lane = 4*g + t (row 8*nt + g) owning 8 B: [elements 4t..4t+3][elements 16+4t..16+4t+3].
// Scales: a plane of f32 at d_offset, 256 B per (nt, bg): for block j of the group and column pair cp the
// four floats {d[2cp], d[2cp+1], nd[2cp], nd[2cp+1]} at float index ((j*4 + cp)*4), where d is the block's
// fp16 scale widened to f32 and nd = -d * 12582912 (exact), the constant that turns the tensor-core
// kernel's "integer dot + 0x4B400000" accumulator bits into d * dot with one fused multiply-add.
// Rows beyond N and blocks beyond K/32 are zero.
constexpr float ACT_MAGIC = 12582912.0f;   // 1.5 * 2^23 = as_float(0x4B400000)
__host__ __device__ static inline int act_scale_index(int j, int col) { return ((j * 4 + (col >> 1)) * 4) + (col & 1); }
// Products of ACT_F8_MIN_N and more columns also carry what the tcgen05 kernel (mmq_tc.cu) reads: after the scale plane
// two more quant planes in K-major core-matrix order (per n-tile and block two 8-column x 16-byte matrices, elements
// 0..15 then 16..31), holding each quant a = 16 h + l (h = a >> 4, l = a & 15) as two e4m3 bytes -- `hi` the byte whose
// value is h * 2^-5, `lo` the byte l, whose value is l * 2^-9 (the subnormals and first binade of e4m3 are the
// integers 0..15 times 2^-9) -- and a second scale plane with {D[2cp], D[2cp+1], C[2cp], C[2cp+1]} at the same float
// indices, D = d * 2^18 and C = -8 * d * sum(a) (the kernel multiplies unsigned weight nibbles u = q + 8).
constexpr int ACT_F8_MIN_N = 16;
struct ActDims {
    int64_t N, K, nb, nbp, n_bg, n_nt;
    size_t d_offset;     // byte offset of the scale plane
    size_t hi_offset, lo_offset, s2_offset;   // the e4m3 planes and their scale plane (0 when absent)
    size_t total_bytes;
};

__host__ __device__ static inline ActDims act_dims(int64_t K, int64_t N) {
    ActDims a;
    a.N = N;
    a.K = K;
    a.nb = K / 32;
    a.nbp = (a.nb + 3) / 4 * 4;
    a.n_bg = a.nbp / 4;
    a.n_nt = (N + 7) / 8;
    a.d_offset = (size_t) a.n_nt * a.nbp * 256;
    a.total_bytes = a.d_offset + (size_t) a.n_nt * a.n_bg * 256;
    a.hi_offset = a.lo_offset = a.s2_offset = 0;
    if (N >= ACT_F8_MIN_N) {   // every offset below follows from d_offset alone: the scale planes are a quarter of a quant plane
        a.hi_offset = a.total_bytes;
        a.lo_offset = a.hi_offset + a.d_offset;
        a.s2_offset = a.lo_offset + a.d_offset;
        a.total_bytes = a.s2_offset + a.d_offset / 4;
    }
    return a;
}

// the shared arithmetic of quantize_row_q8_0 for one value, given the block's amax-derived multiplier
__device__ __forceinline__ int q8_round(float x, float id, int variant) {
    const float v = __fmul_rn(x, id);
    return variant == B200_Q8_AVX2 ? __float2int_rn(v) : (int) roundf(v);
}
// d (stored as fp16) and id for a block with maximum magnitude amax
__device__ __forceinline__ void q8_scales(float amax, int variant, __half *d_out, float *id_out) {
    const float d = __fdiv_rn(amax, 127.0f);
    *d_out = __float2half_rn(d);
    if (variant == B200_Q8_AVX2) {
        *id_out = (amax != 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
    } else {
        *id_out = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    }
}

// RMS_NORM's sum of squares (ops.cpp:3268-3316 accumulates in double).  The order both kernels that need it use: a
// row is cut into groups of 4 elements, thread i takes groups i, i + blockDim, ...; then a shuffle tree per warp, then
// the warps in order.  rms_threads(d) threads per row: one group per thread up to 4096 elements.
static inline unsigned rms_threads(int64_t d) {
    const int64_t g = (d / 4 + 31) / 32 * 32;
    return (unsigned) (g < 32 ? 32 : (g > 1024 ? 1024 : g));
}
__device__ __forceinline__ double rms_block_sum(double sum) {
    __shared__ double red[32];
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    double tot = 0.0;
    for (int i = 0; i < (int) ((blockDim.x + 31) >> 5); ++i) tot += red[i];
    return tot;
}

// e4m3 byte of h * 2^-5 for the signed nibble h (index = h & 15)
__device__ __forceinline__ uint32_t e4m3_hi_byte(uint32_t nib) {
    const uint64_t tab = (nib & 8) ? 0x90989CA0A2A4A6A8ull : 0x262422201C181000ull;   // h = -8..-1 | h = 0..7, lowest byte first
    return (uint32_t) (tab >> (8 * (nib & 7))) & 0xffu;
}
// Stores one lane's share (4 quants, element group j of 8) of a quantised block (row n, block b).  LAYOUT 0: the
// reference's block_q8_0 stream; 1: B8 tiles in mma.sync B-fragment order; 2: B8 tiles as K-major core matrices;
// 3: layout 1 plus the e4m3 planes of ACT_F8_MIN_N (qsum = the sum of the block's 32 quants).
// Lane j == 0 also stores the block scale (layouts 1/2/3: the f32 pair {d, -d * 12582912}; zero for padding).
template <int LAYOUT>
__device__ __forceinline__ void q8_store(uint8_t *__restrict__ out, size_t d_offset, int64_t nb, int64_t nbp, int64_t n, int64_t b, int j,
                                         uint32_t packed, __half d, bool real, int qsum = 0) {
    if (LAYOUT == 0) {
        uint8_t *blkp = out + (n * nb + b) * 34;
        if (j == 0) *reinterpret_cast<__half *>(blkp) = d;
        uint16_t *q = reinterpret_cast<uint16_t *>(blkp + 2 + 4 * j);
        q[0] = (uint16_t) (packed & 0xffffu);
        q[1] = (uint16_t) (packed >> 16);
    } else {
        const int64_t nt = n >> 3;
        const int g = (int) (n & 7);
        const int t = j & 3;
        uint8_t *tile = out + (nt * nbp + b) * 256;
        if (LAYOUT == 1 || LAYOUT == 3) {
            *reinterpret_cast<uint32_t *>(tile + (g * 4 + t) * 8 + (j >= 4 ? 4 : 0)) = packed;
            if (LAYOUT == 3) {
                const size_t hi_off = d_offset + d_offset / 4, lo_off = hi_off + d_offset;
                const size_t at = (size_t) (nt * nbp + b) * 256 + (j >> 2) * 128 + g * 16 + t * 4;
                const uint32_t nib = (packed >> 4) & 0x0F0F0F0Fu;
                const uint32_t hi = e4m3_hi_byte(nib & 0xff) | (e4m3_hi_byte((nib >> 8) & 0xff) << 8) | (e4m3_hi_byte((nib >> 16) & 0xff) << 16) |
                                    (e4m3_hi_byte(nib >> 24) << 24);
                *reinterpret_cast<uint32_t *>(out + hi_off + at) = hi;
                *reinterpret_cast<uint32_t *>(out + lo_off + at) = packed & 0x0F0F0F0Fu;
            }
        } else {
            // two 8-column x 16-byte core matrices: elements 0..15 of each column, then elements 16..31
            *reinterpret_cast<uint32_t *>(tile + (j >> 2) * 128 + g * 16 + t * 4) = packed;
        }
        if (j == 0) {
            float *dp = reinterpret_cast<float *>(out + d_offset) + (nt * (nbp >> 2) + (b >> 2)) * 64 + act_scale_index((int) (b & 3), g);
            const float df = real ? __half2float(d) : 0.0f;
            dp[0] = df;
            dp[2] = -df * ACT_MAGIC;
            if (LAYOUT == 3) {
                float *dp2 = reinterpret_cast<float *>(out + d_offset + d_offset / 4 + 2 * d_offset) + (dp - reinterpret_cast<float *>(out + d_offset));
                dp2[0] = df * 262144.0f;
                dp2[2] = __fmul_rn((float) (-8 * qsum), df);
            }
        }
    }
}

// quantises the 4 values of one lane of an 8-lane block group (all 8 lanes of the group must call it) and stores them
template <int LAYOUT>
__device__ __forceinline__ void q8_quantize_store(const float (&v)[4], uint8_t *__restrict__ out, size_t d_offset, int64_t nb, int64_t nbp,
                                                  int64_t n, int64_t b, int j, bool real, int variant) {
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    const unsigned grp = 0xFFu << (threadIdx.x & 24);  // the 8 lanes that share this block
    amax = fmaxf(amax, __shfl_xor_sync(grp, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(grp, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(grp, amax, 4));
    __half d;
    float id;
    q8_scales(amax, variant, &d, &id);
    uint32_t packed = 0;
    int qsum = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q = q8_round(v[i], id, variant);
        qsum += q;
        packed |= ((uint32_t) (q & 0xff)) << (8 * i);
    }
    if (LAYOUT == 3) {
        qsum += __shfl_xor_sync(grp, qsum, 1);
        qsum += __shfl_xor_sync(grp, qsum, 2);
        qsum += __shfl_xor_sync(grp, qsum, 4);
    }
    q8_store<LAYOUT>(out, d_offset, nb, nbp, n, b, j, packed, d, real, qsum);
}

// the same for one value per lane: the 32 lanes of a (fully active) warp hold one block in element order
template <int LAYOUT>
__device__ __forceinline__ void q8_quantize_store_warp(float v, uint8_t *__restrict__ out, size_t d_offset, int64_t nb, int64_t nbp, int64_t n,
                                                       int64_t b, bool real, int variant) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __half d;
    float id;
    q8_scales(amax, variant, &d, &id);
    const int qi = q8_round(v, id, variant);
    int qsum = qi;
    if (LAYOUT == 3) {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
    }
    const uint32_t q = (uint32_t) (qi & 0xff);
    uint32_t packed = q;
    packed |= __shfl_down_sync(0xffffffffu, q, 1) << 8;
    packed |= __shfl_down_sync(0xffffffffu, q, 2) << 16;
    packed |= __shfl_down_sync(0xffffffffu, q, 3) << 24;
    const int lane = threadIdx.x & 31;
    if ((lane & 3) == 0) q8_store<LAYOUT>(out, d_offset, nb, nbp, n, b, lane >> 2, packed, d, real, qsum);
}

}  // namespace b200
