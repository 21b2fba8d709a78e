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
static inline bool is_aligned(const void *p, size_t a) { return ((uintptr_t) p % a) == 0; }

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
struct ActDims {
    int64_t N, K, nb, nbp, n_bg, n_nt;
    size_t d_offset;     // byte offset of the scale plane
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

}  // namespace b200
