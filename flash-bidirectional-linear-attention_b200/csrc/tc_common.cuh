// Shared pieces of the tensor-core kernels: the kernel parameter block, the static tile
// schedule, and small device helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fbla_common.cuh"
#include "tc_ptx.cuh"

namespace fbla {
namespace tc {

#ifndef FBLA_PREFETCH_TILES
#define FBLA_PREFETCH_TILES 0
#endif
constexpr int kTileTokens = 128;      // tokens per tile = rows of one MMA
constexpr int kBlockBytes = 16384;    // one [128 tokens][64 features] 16-bit block in shared memory
constexpr int kThreads = 192;         // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue
constexpr int kEpiThreads = 128;
constexpr int kSmemLimit = 227 * 1024;

// Operator variant a kernel is instantiated for.
constexpr int kSimple = 0;      // no normaliser
constexpr int kLinear = 1;      // normalised, one q / k
constexpr int kDecoupled = 2;   // normalised, rotary q/k in the numerator

// Static schedule: the tiles of all units form one list (unit-major); CTA c owns the
// contiguous range [c * tiles_per_cta, (c+1) * tiles_per_cta).  A maximal run of tiles of one
// unit inside a CTA's range is a segment; reducing kernels emit one partial per segment into
// slot (unit, c - first_cta(unit)).
struct Schedule {
    int units;
    int tiles_per_unit;
    int total_tiles;
    int tiles_per_cta;
    int slots_per_unit;   // upper bound on segments per unit
    int ctas;
};

struct Params {
    Schedule sch;
    int seq_len;          // tokens per unit
    float scale;
    float inv_norm;       // 1 / (length the key sum is divided by)
    float eps;
    int is_bf16;          // 1: bf16, 0: fp16
    int* status;          // host-visible status word (0 = ok)
    // forward state / backward state: per-segment partials; others: the reduced state
    float* part;
    const float* state;
    int state_stride;     // floats per unit in state / partial slots
    // kernels that write an output with plain global stores (no staged tile): its base address
    void* out_a;
    void* out_b;
};

__host__ __device__ inline int first_cta_of_unit(const Schedule& s, int unit) {
    return (int)(((long long)unit * s.tiles_per_unit) / s.tiles_per_cta);
}
__host__ __device__ inline int last_cta_of_unit(const Schedule& s, int unit) {
    return (int)((((long long)unit + 1) * s.tiles_per_unit - 1) / s.tiles_per_cta);
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack2(uint32_t u, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
        return __bfloat1622float2(h);
    }
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
}
__device__ __forceinline__ uint16_t pack1(float a, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat16 h = __float2bfloat16_rn(a);
        return *reinterpret_cast<uint16_t*>(&h);
    }
    __half h = __float2half_rn(a);
    return *reinterpret_cast<uint16_t*>(&h);
}
__device__ __forceinline__ float unpack1(uint16_t u, int is_bf16) {
    if (is_bf16) return __bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&u));
    return __half2float(*reinterpret_cast<__half*>(&u));
}

// Copies a finished [DK x DV] fp32 accumulator (rows = key features) from tensor memory to a
// partial slot in global memory, plus one extra per-row value (the sum of NVEC columns starting
// at column `vec_col`) stored after the matrix.  Executed by the four epilogue warps.  With
// M = 128 accumulator row r sits in TMEM lane r; with M = 64 it sits in lane (r % 16) + 32 * (r / 16).
template <int DK, int DV, int NVEC>
__device__ __forceinline__ void drain_state_acc(uint32_t tmem_acc, uint32_t vec_col, float* out, int warp, int lane) {
    const int quarter = warp & 3;
    const int row = DK == 128 ? quarter * 32 + lane : quarter * 16 + lane;
    const bool row_ok = DK == 128 ? true : lane < 16;
    const uint32_t t_lane = tmem_acc + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
    for (int c0 = 0; c0 < DV; c0 += 32) {
        float v[32];
        ptx::tmem_ld32(t_lane + c0, v);
        ptx::tmem_ld_wait();
        if (row_ok) {
            float4* dst = reinterpret_cast<float4*>(out + row * DV + c0);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
    }
    if (NVEC > 0) {
        float v[16];
        ptx::tmem_ld16(t_lane + vec_col, v);
        ptx::tmem_ld_wait();
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NVEC; ++j) s += v[j];
        if (row_ok) out[DK * DV + row] = s;
    }
}

// Dynamic shared memory starts at an address the swizzled tiles can use (1024-byte aligned).
__device__ __forceinline__ uint8_t* align_1024(uint8_t* p) {
    const uint32_t a = ptx::smem_u32(p);
    return p + ((1024u - (a & 1023u)) & 1023u);
}

}  // namespace tc
}  // namespace fbla
