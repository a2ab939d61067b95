// Tensor-core forward of the piecewise_sparse_attention attention stage for the common shape:
// 16-bit inputs, block size 64, dk = dv = D in {64, 128}.
//
// One CTA of four warps per (query block, batch*head); a warp owns 16 query rows and keeps their
// online-softmax state and the 16 x D output accumulator in registers (warp-level mma.sync
// m16n8k16, fp32 accumulate -- the per-row rescaling between blocks makes a register-resident
// accumulator the natural fit here; the contraction-heavy passes of the other operators use
// tcgen05).  Key/value blocks, the block statistics (kc as keys, vc as values, in chunks of 64
// blocks) and the first-order state h all go through the same two shared-memory tiles, stored
// with a 16-byte-chunk XOR swizzle so that ldmatrix is conflict-free.
#pragma once

#include "fbla_common.cuh"

namespace fbla {
namespace pisa_mma {

constexpr int kBS = 64;        // block size
constexpr int kThreads = 128;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] 16-bit tile
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack(float a, float b) {
    if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

struct Params {
    int heads, ns, nt, T;
    float scale;
};

// Copies `nrows` rows (each D 16-bit elements, contiguous) from global memory into a swizzled tile,
// zero-filling rows [nrows, 64).
template <int D>
__device__ __forceinline__ void load_tile16(uint8_t* tile, const void* src, int nrows) {
    constexpr int CH = D / 8;                       // 16-byte chunks per row
    for (int i = threadIdx.x; i < kBS * CH; i += kThreads) {
        const int r = i / CH, c = i - r * CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows) v = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(src) + (size_t)r * D * 2 + c * 16);
        *reinterpret_cast<uint4*>(tile + tile_off<D>(r, c)) = v;
    }
}
// Asynchronous variant (cp.async, 16 bytes per request): the caller commits the group and waits for it
// before the tile is read.  Rows past `nrows` are zeroed with ordinary stores.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
template <int D>
__device__ __forceinline__ void load_tile16_async(uint8_t* tile, const void* src, int nrows) {
    constexpr int CH = D / 8;
    for (int i = threadIdx.x; i < kBS * CH; i += kThreads) {
        const int r = i / CH, c = i - r * CH;
        if (r < nrows)
            cp_async16(smem_addr(tile) + tile_off<D>(r, c), static_cast<const uint8_t*>(src) + (size_t)r * D * 2 + c * 16);
        else
            *reinterpret_cast<uint4*>(tile + tile_off<D>(r, c)) = make_uint4(0, 0, 0, 0);
    }
}
// Same from fp32 rows (block statistics, first-order state), converting to the 16-bit type.
template <int D, bool BF16>
__device__ __forceinline__ void load_tile32(uint8_t* tile, const float* src, int nrows, int tile_rows) {
    constexpr int CH = D / 8;
    for (int i = threadIdx.x; i < tile_rows * CH; i += kThreads) {
        const int r = i / CH, c = i - r * CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows) {
            const float4 a = *reinterpret_cast<const float4*>(src + (size_t)r * D + c * 8);
            const float4 b = *reinterpret_cast<const float4*>(src + (size_t)r * D + c * 8 + 4);
            v = make_uint4(pack<BF16>(a.x, a.y), pack<BF16>(a.z, a.w), pack<BF16>(b.x, b.y), pack<BF16>(b.z, b.w));
        }
        *reinterpret_cast<uint4*>(tile + tile_off<D>(r, c)) = v;
    }
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads)
pisa_fwd_mma_kernel(Params p, const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                    const float* __restrict__ kc, const float* __restrict__ vc, const float* __restrict__ h,
                    const int32_t* __restrict__ indices, void* __restrict__ o, float* __restrict__ row_stats) {
    constexpr int NT8 = D / 8;        // n-tiles of the output
    constexpr int KS = D / 16;        // k-steps over the feature dim
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kTile = kBS * D * 2;
    uint8_t* qs = smem;                         // [64][D]   queries; reused to stage the output
    uint8_t* kv0 = qs + kTile;                  // two (keys, values) buffer pairs: the selected blocks are
    uint8_t* kv1 = kv0 + 2 * kTile;             // prefetched with cp.async one block ahead
    uint8_t* ks = kv0;                          // [64][D]   keys / block means      } together [D][D] for h
    uint8_t* vs = ks + kTile;                   // [64][D]   values / block sums     }
    unsigned char* sel = kv1 + 2 * kTile;       // [nt] selected?

    const int i_blk = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = i_blk * kBS;
    const int nrows = min(kBS, p.T - t0);
    const size_t base_row = (size_t)bh * p.T;
    const float sm = p.scale * 1.44269504f;
    const int32_t* idx = indices + ((size_t)bh * p.nt + i_blk) * p.ns;
    const uint8_t* qg = static_cast<const uint8_t*>(q) + (base_row + t0) * D * 2;

    load_tile16<D>(qs, qg, nrows);
    for (int i = threadIdx.x; i < p.nt; i += kThreads) sel[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < p.ns; i += kThreads) {
        const int c = idx[i];
        if (c >= 0 && c < p.nt) sel[c] = 1;
    }
    // query fragments of this warp's 16 rows, kept for the whole kernel
    uint32_t qa[KS][4];
    {
        const int row = warp * 16 + (lane & 15);
#pragma unroll
        for (int s = 0; s < KS; ++s) ldsm_x4(qa[s], smem_addr(qs) + tile_off<D>(row, 2 * s + (lane >> 4)));
    }
    float acc[NT8][4];
#pragma unroll
    for (int n = 0; n < NT8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};    // rows lane/4 and lane/4 + 8
    float l_part[2] = {0.f, 0.f};               // per-thread partial sums (reduced over the quad at the end)
    float g_part[2] = {0.f, 0.f};
    const int col0 = (lane & 3) * 2;            // this thread's columns inside an 8-wide tile

    // scores of 64 keys (rows of ks) for this warp's rows -> online softmax -> acc += P . vs.
    // `approx`: keys are block means c0 + j (masked when selected or past NT), weights go to g.
    auto block = [&](int nvalid, bool approx, int c0) {
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
        // groups of 16 keys past `nvalid` are skipped (their scores stay 0 and are masked below)
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {        // two 8-key tiles per ldmatrix.x4
                if (n2 * 16 >= nvalid) continue;
                uint32_t b[4];
                const int key = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                ldsm_x4(b, smem_addr(ks) + tile_off<D>(key, 2 * kk + ((lane >> 3) & 1)));
                mma16816<BF16>(s[2 * n2], qa[kk], b[0], b[1]);
                mma16816<BF16>(s[2 * n2 + 1], qa[kk], b[2], b[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = n * 8 + col0 + (e & 1);
                bool ok = j < nvalid;
                if (approx && ok) ok = !sel[c0 + j];
                s[n][e] = ok ? s[n][e] * sm : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            alpha[r] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
            l_part[r] *= alpha[r];
            g_part[r] *= alpha[r];
        }
#pragma unroll
        for (int n = 0; n < NT8; ++n) {
            acc[n][0] *= alpha[0];
            acc[n][1] *= alpha[0];
            acc[n][2] *= alpha[1];
            acc[n][3] *= alpha[1];
        }
        uint32_t pa[4][4];                          // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            float pe[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float mr = m_run[e >> 1];
                pe[e] = (mr == -INFINITY) ? 0.f : exp2f(s[n][e] - mr);
                if (approx) {
                    const int cblk = c0 + n * 8 + col0 + (e & 1);
                    const float len = (cblk == p.nt - 1) ? (float)(p.T - (p.nt - 1) * kBS) : (float)kBS;
                    g_part[e >> 1] += pe[e] * len;
                } else {
                    l_part[e >> 1] += pe[e];
                }
            }
            pa[n >> 1][(n & 1) * 2 + 0] = pack<BF16>(pe[0], pe[1]);
            pa[n >> 1][(n & 1) * 2 + 1] = pack<BF16>(pe[2], pe[3]);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            if (kk * 16 >= nvalid) continue;        // weights of these keys are all zero
#pragma unroll
            for (int n2 = 0; n2 < NT8 / 2; ++n2) {
                uint32_t b[4];
                const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                ldsm_x4_trans(b, smem_addr(vs) + tile_off<D>(key, 2 * n2 + (lane >> 4)));
                mma16816<BF16>(acc[2 * n2], pa[kk], b[0], b[1]);
                mma16816<BF16>(acc[2 * n2 + 1], pa[kk], b[2], b[3]);
            }
        }
    };

    // ---- phase 1: exact attention on the selected key blocks (block n+1 in flight during block n) ----
    auto valid_rows = [&](int n) {
        const int cb = idx[n];
        return (cb < 0 || cb >= p.nt) ? 0 : min(kBS, p.T - cb * kBS);    // a bad index selects nothing
    };
    auto prefetch = [&](int n) {
        uint8_t* buf = (n & 1) ? kv1 : kv0;
        const int nvalid = valid_rows(n);
        const size_t off = (base_row + (size_t)(nvalid ? idx[n] : 0) * kBS) * D * 2;
        load_tile16_async<D>(buf, static_cast<const uint8_t*>(k) + off, nvalid);
        load_tile16_async<D>(buf + kTile, static_cast<const uint8_t*>(v) + off, nvalid);
        cp_async_commit();
    };
    if (p.ns > 0) prefetch(0);
    for (int n = 0; n < p.ns; ++n) {
        cp_async_wait_all();
        __syncthreads();            // block n has landed; every warp is done with block n-1
        if (n + 1 < p.ns) prefetch(n + 1);
        ks = (n & 1) ? kv1 : kv0;
        vs = ks + kTile;
        block(valid_rows(n), false, 0);
    }
    ks = kv0;
    vs = ks + kTile;
    // ---- phase 2: zeroth order on the unselected blocks, 64 blocks at a time ----
    for (int c0 = 0; c0 < p.nt; c0 += kBS) {
        __syncthreads();
        const int nvalid = min(kBS, p.nt - c0);
        load_tile32<D, BF16>(ks, kc + ((size_t)bh * p.nt + c0) * D, nvalid, kBS);
        load_tile32<D, BF16>(vs, vc + ((size_t)bh * p.nt + c0) * D, nvalid, kBS);
        __syncthreads();
        block(nvalid, true, c0);
    }
    // ---- reduce the per-thread partial sums over the four threads of a row ----
    float l_row[2], g_row[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_row[r] = l_part[r] + __shfl_xor_sync(0xffffffffu, l_part[r], 1);
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
        g_row[r] = g_part[r] + __shfl_xor_sync(0xffffffffu, g_part[r], 1);
        g_row[r] += __shfl_xor_sync(0xffffffffu, g_row[r], 2);
    }
    // ---- phase 3: first order, acc += (q h) g scale / T; h ([D][D]) fills the key+value tiles ----
    __syncthreads();
    {
        constexpr int CH = D / 8;
        const float* hb = h + (size_t)bh * D * D;
        for (int i = threadIdx.x; i < D * CH; i += kThreads) {
            const int r = i / CH, c = i - r * CH;
            const float4 a = *reinterpret_cast<const float4*>(hb + (size_t)r * D + c * 8);
            const float4 b = *reinterpret_cast<const float4*>(hb + (size_t)r * D + c * 8 + 4);
            *reinterpret_cast<uint4*>(ks + tile_off<D>(r, c)) =
                make_uint4(pack<BF16>(a.x, a.y), pack<BF16>(a.z, a.w), pack<BF16>(b.x, b.y), pack<BF16>(b.z, b.w));
        }
    }
    __syncthreads();
    const float w = p.scale / (float)p.T;
    const float corr[2] = {g_row[0] * w, g_row[1] * w};
#pragma unroll
    for (int n2 = 0; n2 < NT8 / 2; ++n2) {
        float r0[4] = {0.f, 0.f, 0.f, 0.f}, r1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            uint32_t b[4];
            const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            ldsm_x4_trans(b, smem_addr(ks) + tile_off<D>(row, 2 * n2 + (lane >> 4)));
            mma16816<BF16>(r0, qa[kk], b[0], b[1]);
            mma16816<BF16>(r1, qa[kk], b[2], b[3]);
        }
        acc[2 * n2][0] += r0[0] * corr[0];
        acc[2 * n2][1] += r0[1] * corr[0];
        acc[2 * n2][2] += r0[2] * corr[1];
        acc[2 * n2][3] += r0[3] * corr[1];
        acc[2 * n2 + 1][0] += r1[0] * corr[0];
        acc[2 * n2 + 1][1] += r1[1] * corr[0];
        acc[2 * n2 + 1][2] += r1[2] * corr[1];
        acc[2 * n2 + 1][3] += r1[3] * corr[1];
    }
    // ---- normalise, stage the tile in shared memory (the query tile is no longer needed), store ----
    const float rden[2] = {1.f / (l_row[0] + g_row[0]), 1.f / (l_row[1] + g_row[1])};
    __syncthreads();        // every warp has loaded its query fragments long ago; h reads are done too
    {
        const int r_lo = warp * 16 + (lane >> 2);
#pragma unroll
        for (int n = 0; n < NT8; ++n) {
            const int col = n * 8 + col0;
            *reinterpret_cast<uint32_t*>(qs + tile_off<D>(r_lo, col >> 3) + (col & 7) * 2) =
                pack<BF16>(acc[n][0] * rden[0], acc[n][1] * rden[0]);
            *reinterpret_cast<uint32_t*>(qs + tile_off<D>(r_lo + 8, col >> 3) + (col & 7) * 2) =
                pack<BF16>(acc[n][2] * rden[1], acc[n][3] * rden[1]);
        }
        if (row_stats != nullptr && (lane & 3) == 0) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = r_lo + 8 * r;
                if (row < nrows)
                    *reinterpret_cast<float4*>(row_stats + (base_row + t0 + row) * 4) =
                        make_float4(m_run[r], l_row[r] + g_row[r], g_row[r], rden[r]);
            }
        }
    }
    __syncthreads();
    {
        constexpr int CH = D / 8;
        uint8_t* og = static_cast<uint8_t*>(o) + (base_row + t0) * D * 2;
        for (int i = threadIdx.x; i < nrows * CH; i += kThreads) {
            const int r = i / CH, c = i - r * CH;
            *reinterpret_cast<uint4*>(og + (size_t)r * D * 2 + c * 16) = *reinterpret_cast<const uint4*>(qs + tile_off<D>(r, c));
        }
    }
}

template <int D>
constexpr size_t smem_bytes(int nt) { return (size_t)5 * kBS * D * 2 + (size_t)nt + 16; }

}  // namespace pisa_mma
}  // namespace fbla
