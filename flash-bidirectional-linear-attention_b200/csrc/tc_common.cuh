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
// Packed layout: every kernel keeps the tile plan (one int per sequence + 1) at the end of its
// dynamic shared memory, so at most kMaxPackedSeqs sequences per call take the tensor-core path.
constexpr int kPlanBytes = 8192;
constexpr int kMaxPackedSeqs = kPlanBytes / 4 - 1;

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

__host__ __device__ inline int first_cta_of_unit(const Schedule& s, int unit) {
    return (int)(((long long)unit * s.tiles_per_unit) / s.tiles_per_cta);
}
__host__ __device__ inline int last_cta_of_unit(const Schedule& s, int unit) {
    return (int)((((long long)unit + 1) * s.tiles_per_unit - 1) / s.tiles_per_cta);
}

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
    float* state_out;     // packed layout: reducing kernels write whole-unit states here directly
    const float* state;
    const float* state_parts;   // non-null: `state` is not used, the consuming pass adds the per-segment pieces itself
    int state_stride;     // floats per unit in state / partial slots
    // kernels that write an output with plain global stores (no staged tile): its base address
    void* out_a;
    void* out_b;
    int mem_dk, mem_dv;   // key / value features per row of those outputs in memory (<= the kernel's DK, DV)
    // packed variable-length layout (total_tokens, heads, D); all null / zero for fixed length
    const int32_t* cu;    // cu_seqlens, device
    const int32_t* plan;  // plan[s] = heads * (tiles of sequences before s), plan[num_seqs] = all tiles
    int num_seqs;
    int heads;
    int scale_per_seq;    // scale = 1 / length of the sequence
    float inv_norm_fixed; // > 0: divide the key sum by this length for every sequence; 0: by its own
};

// The state of one unit as a consuming pass reads it: one vector, or the per-segment pieces that the
// reducing pass left (added here in CTA order, the order tc_reduce_partials_kernel uses, so both
// routes give the same bits).
struct StateSrc {
    const float* p;
    int n;
    size_t stride;
    __device__ __forceinline__ float operator[](int i) const {
        float a = p[i];
        for (int j = 1; j < n; ++j) a += p[(size_t)j * stride + i];
        return a;
    }
    // N values first + u * step (u = 0..N-1) at once: all loads of one piece are in flight together
    // before the next piece is added (the sum per element still runs in piece order).
    template <int N>
    __device__ __forceinline__ void load(int first, int step, float (&x)[N]) const {
#pragma unroll
        for (int u = 0; u < N; ++u) x[u] = p[first + u * step];
        for (int j = 1; j < n; ++j) {
            const float* pj = p + (size_t)j * stride;
            float y[N];
#pragma unroll
            for (int u = 0; u < N; ++u) y[u] = pj[first + u * step];
#pragma unroll
            for (int u = 0; u < N; ++u) x[u] += y[u];
        }
    }
    template <int N>
    __device__ __forceinline__ void load2(int first, int step, float2 (&x)[N]) const {    // first, step even
#pragma unroll
        for (int u = 0; u < N; ++u) x[u] = *reinterpret_cast<const float2*>(p + first + u * step);
        for (int j = 1; j < n; ++j) {
            const float* pj = p + (size_t)j * stride;
            float2 y[N];
#pragma unroll
            for (int u = 0; u < N; ++u) y[u] = *reinterpret_cast<const float2*>(pj + first + u * step);
#pragma unroll
            for (int u = 0; u < N; ++u) {
                x[u].x += y[u].x;
                x[u].y += y[u].y;
            }
        }
    }
    __device__ __forceinline__ float2 pair(int i) const {     // i even
        float2 a = *reinterpret_cast<const float2*>(p + i);
        for (int j = 1; j < n; ++j) {
            const float2 b = *reinterpret_cast<const float2*>(p + (size_t)j * stride + i);
            a.x += b.x;
            a.y += b.y;
        }
        return a;
    }
};
__device__ __forceinline__ StateSrc state_source(const Params& p, int unit) {
    StateSrc s;
    if (p.state_parts != nullptr) {
        s.p = p.state_parts + (size_t)unit * p.sch.slots_per_unit * p.state_stride;
        s.n = last_cta_of_unit(p.sch, unit) - first_cta_of_unit(p.sch, unit) + 1;
    } else {
        s.p = p.state + (size_t)unit * p.state_stride;
        s.n = 1;
    }
    s.stride = (size_t)p.state_stride;
    return s;
}

// One 128-token tile of the work list, as every role of a kernel sees it.
struct Tile {
    int unit;          // state index
    int tile;          // index of the tile inside its unit
    int c1, c2;        // TMA coordinates after the feature coordinate
    int valid;         // tokens of the tile that belong to the unit (1..128)
    long long row0;    // row of the tile's first token in the (rows, D) view of the tensor
    int row_stride;    // rows between consecutive tokens (1, or heads when packed)
    bool first, last;  // first / last tile of a segment (run of one unit inside this CTA's range)
    bool starts_here, ends_here;   // the unit's first / last tile lies inside this CTA's range
    float scale, inv_norm;
};

// plan[s] = number of 128-token tiles of the sequences before s (per head), plan[num_seqs] = all of
// them; built by every CTA for itself from cu_seqlens (all threads of the block must call this).
__device__ __forceinline__ void build_plan(int32_t* plan, const int32_t* __restrict__ cu, int num_seqs) {
    for (int i = threadIdx.x; i <= num_seqs; i += blockDim.x) plan[i] = cu[i];
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, prev = plan[0];
        for (int s = 0; s < num_seqs; ++s) {
            const int next = plan[s + 1];
            plan[s] = acc;
            acc += (next - prev + kTileTokens - 1) / kTileTokens;
            prev = next;
        }
        plan[num_seqs] = acc;
    }
    __syncthreads();
}

template <bool VARLEN>
struct TileMap;

template <>
struct TileMap<false> {
    __device__ static __forceinline__ void range(const Params& p, int& g0, int& g1) {
        g0 = blockIdx.x * p.sch.tiles_per_cta;
        g1 = min(p.sch.total_tiles, g0 + p.sch.tiles_per_cta);
    }
    __device__ static __forceinline__ Tile get(const Params& p, int g, int g0, int g1) {
        Tile t;
        const int tpu = p.sch.tiles_per_unit;
        t.unit = g / tpu;
        t.tile = g - t.unit * tpu;
        t.c1 = t.tile * kTileTokens;
        t.c2 = t.unit;
        t.valid = min(kTileTokens, p.seq_len - t.c1);
        t.row0 = (long long)t.unit * p.seq_len + t.c1;
        t.row_stride = 1;
        t.first = (g == g0) || t.tile == 0;
        t.last = (g == g1 - 1) || t.tile == tpu - 1;
        t.starts_here = (g - t.tile) >= g0;
        t.ends_here = (g - t.tile + tpu) <= g1;
        t.scale = p.scale;
        t.inv_norm = p.inv_norm;
        return t;
    }
};

// Packed layout.  Token rows of one head are heads*D elements apart, so the heads of a token share
// DRAM pages: CTA c works on head c % heads, and the heads*G CTAs of a launch split the per-head tile
// list into G = gridDim.x / heads contiguous ranges, so that at any time the CTAs of a group stream
// the same tokens (one head each).  Tile index g below counts tiles of ONE head.
template <>
struct TileMap<true> {
    __device__ static __forceinline__ void range(const Params& p, int& g0, int& g1) {
        const int total = p.plan[p.num_seqs];
        const int groups = (int)gridDim.x / p.heads;
        const int grp = (int)blockIdx.x / p.heads;
        const int per = (total + groups - 1) / groups;
        g0 = min(total, grp * per);
        g1 = min(total, g0 + per);
    }
    __device__ static __forceinline__ Tile get(const Params& p, int g, int g0, int g1) {
        // sequence s with plan[s] <= g < plan[s+1]
        int lo = 0, hi = p.num_seqs;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.plan[mid] <= g) lo = mid; else hi = mid;
        }
        const int s = lo;
        const int a0 = p.plan[s];
        const int nt = p.plan[s + 1] - a0;
        const int h = (int)blockIdx.x % p.heads;
        Tile t;
        t.tile = g - a0;
        t.unit = s * p.heads + h;
        const int bos = p.cu[s];
        const int len = p.cu[s + 1] - bos;
        t.c1 = h;
        t.c2 = bos + t.tile * kTileTokens;
        t.valid = min(kTileTokens, len - t.tile * kTileTokens);
        t.row0 = (long long)t.c2 * p.heads + h;
        t.row_stride = p.heads;
        t.first = (g == g0) || t.tile == 0;
        t.last = (g == g1 - 1) || t.tile == nt - 1;
        t.starts_here = a0 >= g0;
        t.ends_here = (a0 + nt) <= g1;
        const float inv_len = 1.f / (float)len;
        t.scale = p.scale_per_seq ? inv_len : p.scale;
        t.inv_norm = p.inv_norm_fixed > 0.f ? p.inv_norm_fixed : inv_len;
        return t;
    }
};

// Where a reducing kernel puts the state of a finished segment.
//   fixed length : slot (unit, cta - first_cta(unit)) of the partial buffer, added by
//                  tc_reduce_partials_kernel.
//   packed       : a unit that lies wholly inside this CTA's range goes straight to the state; a
//                  piece of a unit that started in an earlier CTA goes to partial slot (cta, 0), a
//                  unit that starts here but continues in the next CTA to slot (cta, 1);
//                  tc_reduce_varlen_kernel adds the pieces in CTA order.
template <bool VARLEN>
__device__ __forceinline__ float* segment_destination(const Params& p, const Tile& t, float* state_out) {
    if (!VARLEN) {
        const int slot = t.unit * p.sch.slots_per_unit + ((int)blockIdx.x - first_cta_of_unit(p.sch, t.unit));
        return p.part + (size_t)slot * p.state_stride;
    }
    if (t.starts_here && t.ends_here) return state_out + (size_t)t.unit * p.state_stride;
    return p.part + ((size_t)blockIdx.x * 2 + (t.starts_here ? 1 : 0)) * p.state_stride;
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
