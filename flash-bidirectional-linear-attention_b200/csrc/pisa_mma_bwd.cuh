// Tensor-core backward of the piecewise_sparse_attention attention stage for the common shape
// (16-bit inputs, block size 64, dk = dv = D in {64, 128}); the formulas are stated where the
// backward entry point is defined.  Two kernels, both warp-level mma.sync m16n8k16 with fp32
// accumulators held in registers, shared-memory tiles in the forward kernel's swizzled layout:
//
//   pisa_bwd_q_mma_kernel   one CTA per query block; a warp owns 16 query rows.  Writes dq, the
//                           per-row dD, the rows dr = dnum g scale / T (16-bit; the first-order
//                           state gradient dh = q^T dr is formed from them by the state pass of
//                           the linear operators), and adds this block's share of dkc, dvc into
//                           fp32 buffers with red.global.
//   pisa_bwd_kv_mma_kernel  one CTA per key block; a warp owns 16 keys and visits the query blocks
//                           that selected the block.  Everything is computed transposed (keys as
//                           the M dimension) so that the softmax weights feed the dk, dv products
//                           straight from registers.  The statistics terms (dkc, dvc, dh) are
//                           added at the end.
//
// The final row maximum and denominator come from the forward's row statistics, so nothing is
// rescaled on the way.  Keys (or query rows) are processed 32 at a time to bound register use.
#pragma once

#include "pisa_mma.cuh"

namespace fbla {
namespace pisa_mma {

template <bool BF16>
__device__ __forceinline__ float2 unpack(uint32_t u) {
    if (BF16) return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
    return __half22float2(*reinterpret_cast<__half2*>(&u));
}

// 16-bit pair plus the pair of rounding residuals.  bf16 keeps 8 significant bits: a gradient that
// is dominated by one large term would otherwise carry that term's rounding error on top of its own.
template <bool BF16>
__device__ __forceinline__ void pack_split(float a, float b, uint32_t& hi, uint32_t& lo) {
    hi = pack<BF16>(a, b);
    const float2 f = unpack<BF16>(hi);
    lo = pack<BF16>(a - f.x, b - f.y);
}

__device__ __forceinline__ void red_add2(float* addr, float a, float b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

// 32-bit element pair (row, col), col even, of a swizzled [rows][D] 16-bit tile
template <int D>
__device__ __forceinline__ uint32_t* pair_at(uint8_t* tile, int row, int col) {
    return reinterpret_cast<uint32_t*>(tile + tile_off<D>(row, col >> 3) + (col & 7) * 2);
}

// Converts a [D][D] fp32 matrix to a 16-bit swizzled tile.
template <int D, bool BF16>
__device__ __forceinline__ void load_square32(uint8_t* tile, const float* src) {
    load_tile32<D, BF16>(tile, src, D, D);
}

// The scratch tile of the query kernel holds a [64][D] tile or two [64][64] tiles, whichever is larger.
template <int D>
constexpr int scratch_tile_bytes() { return kBS * D * 2 > 2 * kBS * 64 * 2 ? kBS * D * 2 : 2 * kBS * 64 * 2; }
template <int D>
constexpr size_t bwd_q_smem_bytes(int nt) {
    return (size_t)6 * kBS * D * 2 + scratch_tile_bytes<D>() + (size_t)nt + 16;
}
template <int D>
constexpr size_t bwd_kv_smem_bytes(int nt) {
    return (size_t)6 * kBS * D * 2 + 2 * kBS * (16 + 4) + (size_t)((nt + 3) / 4 * 4) + (size_t)nt * 4 + 32;
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// ------------------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads)
pisa_bwd_q_mma_kernel(Params p, const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                      const void* __restrict__ o, const void* __restrict__ d_o, const float* __restrict__ kc,
                      const float* __restrict__ vc, const float* __restrict__ h, const int32_t* __restrict__ indices,
                      const float* __restrict__ row_stats, void* __restrict__ dq, void* __restrict__ dr_out,
                      float* __restrict__ dkc, float* __restrict__ dvc, float* __restrict__ drow) {
    constexpr int NT8 = D / 8, KS = D / 16, CH = D / 8;
    constexpr int kTile = kBS * D * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* qs = smem;                 // [64][D] queries; at the end the dq tile
    uint8_t* dos = qs + kTile;          // [64][D] dO
    uint8_t* ks = dos + kTile;          // [64][D] keys / block means      } together [D][D] for h
    uint8_t* vs = ks + kTile;           // [64][D] values / block sums     }
    uint8_t* ts = vs + kTile;           // [64][D] o, then dr; later two [64][64] tiles: scale*da and pi/den
    uint8_t* kvb = ts + scratch_tile_bytes<D>();    // second (keys, values) pair: selected blocks are prefetched
    unsigned char* sel = kvb + 2 * kTile;
    uint8_t* const kva = ks;

    const int i_blk = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g8 = lane >> 2, col0 = (lane & 3) * 2;
    const int t0 = i_blk * kBS;
    const int nrows = min(kBS, p.T - t0);
    const size_t base_row = (size_t)bh * p.T;
    const float sm = p.scale * 1.44269504f;
    const float w = p.scale / (float)p.T;
    const int32_t* idx = indices + ((size_t)bh * p.nt + i_blk) * p.ns;
    const size_t tile_g = (base_row + t0) * D * 2;

    load_tile16<D>(qs, static_cast<const uint8_t*>(q) + tile_g, nrows);
    load_tile16<D>(dos, static_cast<const uint8_t*>(d_o) + tile_g, nrows);
    load_tile16<D>(ts, static_cast<const uint8_t*>(o) + tile_g, nrows);
    load_square32<D, BF16>(ks, h + (size_t)bh * D * D);
    for (int i = threadIdx.x; i < p.nt; i += kThreads) sel[i] = 0;
    // selected block n is loaded with cp.async while block n-1 is processed; even n -> kvb, odd n -> (ks, vs)
    auto valid_rows = [&](int n) {
        const int cb = idx[n];
        return (cb < 0 || cb >= p.nt) ? 0 : min(kBS, p.T - cb * kBS);    // a bad index selects nothing
    };
    auto prefetch = [&](int n) {
        uint8_t* buf = (n & 1) ? kva : kvb;
        const int nvalid = valid_rows(n);
        const size_t off = (base_row + (size_t)(nvalid ? idx[n] : 0) * kBS) * D * 2;
        load_tile16_async<D>(buf, static_cast<const uint8_t*>(k) + off, nvalid);
        load_tile16_async<D>(buf + kTile, static_cast<const uint8_t*>(v) + off, nvalid);
        cp_async_commit();
    };
    if (p.ns > 0) prefetch(0);
    __syncthreads();
    for (int i = threadIdx.x; i < p.ns; i += kThreads) {
        const int c = idx[i];
        if (c >= 0 && c < p.nt) sel[c] = 1;
    }

    uint32_t qa[KS][4], doa[KS][4];
    {
        const int row = warp * 16 + (lane & 15);
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            ldsm_x4(qa[s], smem_addr(qs) + tile_off<D>(row, 2 * s + (lane >> 4)));
            ldsm_x4(doa[s], smem_addr(dos) + tile_off<D>(row, 2 * s + (lane >> 4)));
        }
    }
    // per-row scalars of this thread's two rows (g8 and g8 + 8 of the warp's 16)
    const int r_lo = warp * 16 + g8;
    float m_row[2], rD[2], g_row[2], dD[2], dg[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = r_lo + 8 * r;
        m_row[r] = 0.f; rD[r] = 0.f; g_row[r] = 0.f;
        if (row < nrows) {
            const float4 st = *reinterpret_cast<const float4*>(row_stats + (base_row + t0 + row) * 4);
            m_row[r] = st.x;
            rD[r] = 1.f / st.y;
            g_row[r] = st.z;
        }
    }
    // ---- od = o . dO,  nr = dO . (q h) ----
    float od[2] = {0.f, 0.f}, nr[2] = {0.f, 0.f};
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
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const float* rr = half ? r1 : r0;
            const int col = (2 * n2 + half) * 8 + col0;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float2 dv2 = unpack<BF16>(*pair_at<D>(dos, r_lo + 8 * r, col));
                const float2 ov2 = unpack<BF16>(*pair_at<D>(ts, r_lo + 8 * r, col));
                od[r] += dv2.x * ov2.x + dv2.y * ov2.y;
                nr[r] += dv2.x * rr[2 * r] + dv2.y * rr[2 * r + 1];
            }
        }
    }
    float gw[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        od[r] += __shfl_xor_sync(0xffffffffu, od[r], 1);
        od[r] += __shfl_xor_sync(0xffffffffu, od[r], 2);
        nr[r] += __shfl_xor_sync(0xffffffffu, nr[r], 1);
        nr[r] += __shfl_xor_sync(0xffffffffu, nr[r], 2);
        dD[r] = -od[r] * rD[r];
        dg[r] = dD[r] + nr[r] * rD[r] * w;
        gw[r] = g_row[r] * w * rD[r];
    }
    if ((lane & 3) == 0) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
            if (r_lo + 8 * r < nrows) drow[base_row + t0 + r_lo + 8 * r] = dD[r];
    }
    // ---- dr = dO g w / den into this warp's rows of ts (o is no longer needed there) ----
    __syncwarp();
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
        const int col = n * 8 + col0;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float2 dv2 = unpack<BF16>(*pair_at<D>(dos, r_lo + 8 * r, col));
            *pair_at<D>(ts, r_lo + 8 * r, col) = pack<BF16>(dv2.x * gw[r], dv2.y * gw[r]);
        }
    }
    __syncwarp();
    // ---- dq = dr h^T (first-order part) ----
    float acc[NT8][4];
#pragma unroll
    for (int n = 0; n < NT8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
        uint32_t a[4];
        ldsm_x4(a, smem_addr(ts) + tile_off<D>(warp * 16 + (lane & 15), 2 * kk + (lane >> 4)));
#pragma unroll
        for (int n2 = 0; n2 < NT8 / 2; ++n2) {
            uint32_t b[4];
            const int drow_ = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
            ldsm_x4(b, smem_addr(ks) + tile_off<D>(drow_, 2 * kk + ((lane >> 3) & 1)));
            mma16816<BF16>(acc[2 * n2], a, b[0], b[1]);
            mma16816<BF16>(acc[2 * n2 + 1], a, b[2], b[3]);
        }
    }
    __syncthreads();
    {   // dr rows to global memory
        uint8_t* dg_ = static_cast<uint8_t*>(dr_out) + tile_g;
        for (int i = threadIdx.x; i < nrows * CH; i += kThreads) {
            const int r = i / CH, c = i - r * CH;
            *reinterpret_cast<uint4*>(dg_ + (size_t)r * D * 2 + c * 16) = *reinterpret_cast<const uint4*>(ts + tile_off<D>(r, c));
        }
    }
    uint8_t* das = ts;                    // [64 rows][64 blocks] scale * da
    uint8_t* pis = ts + kBS * 64 * 2;     // [64 rows][64 blocks] pi / den

    // 32 keys (rows j0 .. j0+31 of ks / vs) against this warp's rows
    auto half_block = [&](int j0, int nvalid, bool approx, int c0) {
        float s[4][4], dp[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) { s[n][e] = 0.f; dp[n][e] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2) {
                uint32_t b[4];
                const int key = j0 + n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                ldsm_x4(b, smem_addr(ks) + tile_off<D>(key, 2 * kk + ((lane >> 3) & 1)));
                mma16816<BF16>(s[2 * n2], qa[kk], b[0], b[1]);
                mma16816<BF16>(s[2 * n2 + 1], qa[kk], b[2], b[3]);
                ldsm_x4(b, smem_addr(vs) + tile_off<D>(key, 2 * kk + ((lane >> 3) & 1)));
                mma16816<BF16>(dp[2 * n2], doa[kk], b[0], b[1]);
                mma16816<BF16>(dp[2 * n2 + 1], doa[kk], b[2], b[3]);
            }
        }
        uint32_t dsa[2][4], dsl[2][4];              // scale * ds and, for bf16, its rounding residual
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            float de[4], pe[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + n * 8 + col0 + (e & 1);
                const int r = e >> 1;
                bool ok = j < nvalid;
                if (approx && ok) ok = !sel[c0 + j];
                const float pj = ok ? exp2f(s[n][e] * sm - m_row[r]) : 0.f;
                float dpj = dp[n][e] * rD[r];
                if (approx) {
                    const int cblk = c0 + j;
                    const float len = (cblk == p.nt - 1) ? (float)(p.T - (p.nt - 1) * kBS) : (float)kBS;
                    dpj += dg[r] * len;
                } else {
                    dpj += dD[r];
                }
                de[e] = pj * dpj * p.scale;
                pe[e] = pj * rD[r];
            }
            pack_split<BF16>(de[0], de[1], dsa[n >> 1][(n & 1) * 2 + 0], dsl[n >> 1][(n & 1) * 2 + 0]);
            pack_split<BF16>(de[2], de[3], dsa[n >> 1][(n & 1) * 2 + 1], dsl[n >> 1][(n & 1) * 2 + 1]);
            if (approx) {
                const int col = j0 + n * 8 + col0;
                *pair_at<64>(das, r_lo, col) = dsa[n >> 1][(n & 1) * 2 + 0];
                *pair_at<64>(das, r_lo + 8, col) = dsa[n >> 1][(n & 1) * 2 + 1];
                *pair_at<64>(pis, r_lo, col) = pack<BF16>(pe[0], pe[1]);
                *pair_at<64>(pis, r_lo + 8, col) = pack<BF16>(pe[2], pe[3]);
            }
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < NT8 / 2; ++n2) {
                uint32_t b[4];
                const int key = j0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                ldsm_x4_trans(b, smem_addr(ks) + tile_off<D>(key, 2 * n2 + (lane >> 4)));
                mma16816<BF16>(acc[2 * n2], dsa[kk], b[0], b[1]);
                mma16816<BF16>(acc[2 * n2 + 1], dsa[kk], b[2], b[3]);
                if (BF16) {
                    mma16816<BF16>(acc[2 * n2], dsl[kk], b[0], b[1]);
                    mma16816<BF16>(acc[2 * n2 + 1], dsl[kk], b[2], b[3]);
                }
            }
        }
    };

    // ---- exact part ----
    for (int n = 0; n < p.ns; ++n) {
        cp_async_wait_all();
        __syncthreads();            // block n has landed; every warp is done with block n-1 (and with h)
        if (n + 1 < p.ns) prefetch(n + 1);
        ks = (n & 1) ? kva : kvb;
        vs = ks + kTile;
        const int nvalid = valid_rows(n);
        half_block(0, nvalid, false, 0);
        if (nvalid > 32) half_block(32, nvalid, false, 0);
    }
    ks = kva;
    vs = ks + kTile;
    // ---- zeroth-order part, 64 blocks at a time; dkc, dvc of the chunk ----
    for (int c0 = 0; c0 < p.nt; c0 += kBS) {
        __syncthreads();
        const int nvalid = min(kBS, p.nt - c0);
        load_tile32<D, BF16>(ks, kc + ((size_t)bh * p.nt + c0) * D, nvalid, kBS);
        load_tile32<D, BF16>(vs, vc + ((size_t)bh * p.nt + c0) * D, nvalid, kBS);
        __syncthreads();
        half_block(0, nvalid, true, c0);
        if (nvalid > 32) half_block(32, nvalid, true, c0);     // columns >= 32 are read below only by warps 2, 3
        __syncthreads();
        // warp w: blocks c0 + 16 w .. + 15.   dkc_c += sum_rows das[row][c] q[row],  dvc_c += sum_rows pis[row][c] dO[row]
        if (warp * 16 < nvalid) {
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                const uint8_t* wt = which ? pis : das;
                const uint8_t* xt = which ? dos : qs;
                float* outp = (which ? dvc : dkc) + ((size_t)bh * p.nt + c0) * D;
                uint32_t a[4][4];
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    ldsm_x4_trans(a[kk], smem_addr(wt) + tile_off<64>(kk * 16 + ((lane >> 4) << 3) + (lane & 7),
                                                                      2 * warp + ((lane >> 3) & 1)));
#pragma unroll
                for (int n2 = 0; n2 < NT8 / 2; ++n2) {
                    float c_lo[4] = {0.f, 0.f, 0.f, 0.f}, c_hi[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        uint32_t b[4];
                        const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                        ldsm_x4_trans(b, smem_addr(xt) + tile_off<D>(row, 2 * n2 + (lane >> 4)));
                        mma16816<BF16>(c_lo, a[kk], b[0], b[1]);
                        mma16816<BF16>(c_hi, a[kk], b[2], b[3]);
                    }
                    const int cb_lo = warp * 16 + g8;
                    const int col = n2 * 16 + col0;
                    if (cb_lo < nvalid) {
                        red_add2(outp + (size_t)cb_lo * D + col, c_lo[0], c_lo[1]);
                        red_add2(outp + (size_t)cb_lo * D + col + 8, c_hi[0], c_hi[1]);
                    }
                    if (cb_lo + 8 < nvalid) {
                        red_add2(outp + (size_t)(cb_lo + 8) * D + col, c_lo[2], c_lo[3]);
                        red_add2(outp + (size_t)(cb_lo + 8) * D + col + 8, c_hi[2], c_hi[3]);
                    }
                }
            }
        }
    }
    // ---- dq out through the query tile ----
    __syncthreads();
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
        const int col = n * 8 + col0;
        *pair_at<D>(qs, r_lo, col) = pack<BF16>(acc[n][0], acc[n][1]);
        *pair_at<D>(qs, r_lo + 8, col) = pack<BF16>(acc[n][2], acc[n][3]);
    }
    __syncthreads();
    {
        uint8_t* og = static_cast<uint8_t*>(dq) + tile_g;
        for (int i = threadIdx.x; i < nrows * CH; i += kThreads) {
            const int r = i / CH, c = i - r * CH;
            *reinterpret_cast<uint4*>(og + (size_t)r * D * 2 + c * 16) = *reinterpret_cast<const uint4*>(qs + tile_off<D>(r, c));
        }
    }
}

// ------------------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads)
pisa_bwd_kv_mma_kernel(Params p, const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                       const void* __restrict__ d_o, const float* __restrict__ kc, const float* __restrict__ vc,
                       const int32_t* __restrict__ indices, const float* __restrict__ row_stats,
                       const float* __restrict__ drow, const float* __restrict__ dkc, const float* __restrict__ dvc,
                       const float* __restrict__ dh, void* __restrict__ dk, void* __restrict__ dv) {
    constexpr int NT8 = D / 8, KS = D / 16, CH = D / 8;
    constexpr int kTile = kBS * D * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ks = smem;                 // [64][D] keys of this block; later k - kc, then dk
    uint8_t* vs = ks + kTile;           // [64][D] values;             later v - vc/len, then dv
    uint8_t* qd0 = vs + kTile;          // two (q, dO) tile pairs of the visiting query blocks, filled one block
    uint8_t* qd1 = qd0 + 2 * kTile;     // ahead with cp.async; qd0 later holds dh as a [D][D] tile
    float4* rst = reinterpret_cast<float4*>(qd1 + 2 * kTile);    // [2][64] (m, den, g, 1/den) of the query rows
    float* dds = reinterpret_cast<float*>(rst + 2 * kBS);        // [2][64] dD of the query rows
    int* hlist = reinterpret_cast<int*>(dds + 2 * kBS);          // query blocks that selected this key block
    unsigned char* hit = reinterpret_cast<unsigned char*>(hlist + p.nt);
    __shared__ int n_hit;

    const int c_blk = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g8 = lane >> 2, col0 = (lane & 3) * 2;
    const int bos = c_blk * kBS;
    const int nkeys = min(kBS, p.T - bos);
    const size_t base_row = (size_t)bh * p.T;
    const float sm = p.scale * 1.44269504f;
    const size_t tile_g = (base_row + bos) * D * 2;

    load_tile16<D>(ks, static_cast<const uint8_t*>(k) + tile_g, nkeys);
    load_tile16<D>(vs, static_cast<const uint8_t*>(v) + tile_g, nkeys);
    for (int i = threadIdx.x; i < p.nt; i += kThreads) {
        const int32_t* idx = indices + ((size_t)bh * p.nt + i) * p.ns;
        bool any = false;
        for (int n = 0; n < p.ns; ++n) any |= (idx[n] == c_blk);
        hit[i] = any ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {             // in block order: the accumulation order is fixed
        int n = 0;
        for (int i = 0; i < p.nt; ++i)
            if (hit[i]) hlist[n++] = i;
        n_hit = n;
    }
    __syncthreads();
    const int nh = n_hit;
    float dka[NT8][4], dva[NT8][4];
#pragma unroll
    for (int n = 0; n < NT8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) { dka[n][e] = 0.f; dva[n][e] = 0.f; }
    const int arow = warp * 16 + (lane & 15);       // A-fragment row of this lane (key)

    auto prefetch = [&](int j) {
        const int t0 = hlist[j] * kBS;
        const int nrows = min(kBS, p.T - t0);
        uint8_t* buf = (j & 1) ? qd1 : qd0;
        load_tile16_async<D>(buf, static_cast<const uint8_t*>(q) + (base_row + t0) * D * 2, nrows);
        load_tile16_async<D>(buf + kTile, static_cast<const uint8_t*>(d_o) + (base_row + t0) * D * 2, nrows);
        for (int r = threadIdx.x; r < kBS; r += kThreads) {
            float4* st = rst + (j & 1) * kBS + r;
            float* dd = dds + (j & 1) * kBS + r;
            if (r < nrows) {
                cp_async16(smem_addr(st), row_stats + (base_row + t0 + r) * 4);
                cp_async4(smem_addr(dd), drow + base_row + t0 + r);
            } else {                    // 1/den = 0 and dD = 0 make a padded row contribute nothing
                *st = make_float4(0.f, 1.f, 0.f, 0.f);
                *dd = 0.f;
            }
        }
        cp_async_commit();
    };
    if (nh > 0) prefetch(0);
    for (int j = 0; j < nh; ++j) {
        cp_async_wait_all();
        __syncthreads();                // block j has landed; every warp is done with block j-1
        if (j + 1 < nh) prefetch(j + 1);
        const uint8_t* qs = (j & 1) ? qd1 : qd0;
        const uint8_t* dos = qs + kTile;
        const float4* rs = rst + (j & 1) * kBS;
        const float* dd = dds + (j & 1) * kBS;
        const int nrows = min(kBS, p.T - hlist[j] * kBS);
#pragma unroll 1
        for (int r0 = 0; r0 < kBS; r0 += 32) {
            if (r0 >= nrows) break;
            float st_[4][4], dpt[4][4];               // transposed scores / dp: 16 keys x 32 query rows
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) { st_[n][e] = 0.f; dpt[n][e] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
                uint32_t ak[4], av[4];
                ldsm_x4(ak, smem_addr(ks) + tile_off<D>(arow, 2 * kk + (lane >> 4)));
                ldsm_x4(av, smem_addr(vs) + tile_off<D>(arow, 2 * kk + (lane >> 4)));
#pragma unroll
                for (int n2 = 0; n2 < 2; ++n2) {
                    uint32_t b[4];
                    const int row = r0 + n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
                    ldsm_x4(b, smem_addr(qs) + tile_off<D>(row, 2 * kk + ((lane >> 3) & 1)));
                    mma16816<BF16>(st_[2 * n2], ak, b[0], b[1]);
                    mma16816<BF16>(st_[2 * n2 + 1], ak, b[2], b[3]);
                    ldsm_x4(b, smem_addr(dos) + tile_off<D>(row, 2 * kk + ((lane >> 3) & 1)));
                    mma16816<BF16>(dpt[2 * n2], av, b[0], b[1]);
                    mma16816<BF16>(dpt[2 * n2 + 1], av, b[2], b[3]);
                }
            }
            uint32_t pa[2][4], dsa[2][4], pl[2][4], dsl[2][4];      // weights, scale * ds; bf16 residuals
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                float pe[4], de[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = r0 + n * 8 + col0 + (e & 1);
                    const float4 st = rs[r];
                    const float pj = exp2f(st_[n][e] * sm - st.x);
                    pe[e] = pj * st.w;
                    de[e] = pj * (dpt[n][e] * st.w + dd[r]) * p.scale;
                }
                pack_split<BF16>(pe[0], pe[1], pa[n >> 1][(n & 1) * 2 + 0], pl[n >> 1][(n & 1) * 2 + 0]);
                pack_split<BF16>(pe[2], pe[3], pa[n >> 1][(n & 1) * 2 + 1], pl[n >> 1][(n & 1) * 2 + 1]);
                pack_split<BF16>(de[0], de[1], dsa[n >> 1][(n & 1) * 2 + 0], dsl[n >> 1][(n & 1) * 2 + 0]);
                pack_split<BF16>(de[2], de[3], dsa[n >> 1][(n & 1) * 2 + 1], dsl[n >> 1][(n & 1) * 2 + 1]);
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
                for (int n2 = 0; n2 < NT8 / 2; ++n2) {
                    uint32_t b[4];
                    const int row = r0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldsm_x4_trans(b, smem_addr(dos) + tile_off<D>(row, 2 * n2 + (lane >> 4)));
                    mma16816<BF16>(dva[2 * n2], pa[kk], b[0], b[1]);
                    mma16816<BF16>(dva[2 * n2 + 1], pa[kk], b[2], b[3]);
                    if (BF16) {
                        mma16816<BF16>(dva[2 * n2], pl[kk], b[0], b[1]);
                        mma16816<BF16>(dva[2 * n2 + 1], pl[kk], b[2], b[3]);
                    }
                    ldsm_x4_trans(b, smem_addr(qs) + tile_off<D>(row, 2 * n2 + (lane >> 4)));
                    mma16816<BF16>(dka[2 * n2], dsa[kk], b[0], b[1]);
                    mma16816<BF16>(dka[2 * n2 + 1], dsa[kk], b[2], b[3]);
                    if (BF16) {
                        mma16816<BF16>(dka[2 * n2], dsl[kk], b[0], b[1]);
                        mma16816<BF16>(dka[2 * n2 + 1], dsl[kk], b[2], b[3]);
                    }
                }
            }
        }
    }
    uint8_t* qs = qd0;                  // from here on the [D][D] tile of dh
    // ---- statistics terms: dk += dkc/len + (v - vc/len) dh^T,   dv += dvc + (k - kc) dh ----
    __syncthreads();
    load_square32<D, BF16>(qs, dh + (size_t)bh * D * D);
    const float inv_len = 1.f / (float)nkeys;
    const float* kcb = kc + ((size_t)bh * p.nt + c_blk) * D;
    const float* vcb = vc + ((size_t)bh * p.nt + c_blk) * D;
    const float* dkcb = dkc + ((size_t)bh * p.nt + c_blk) * D;
    const float* dvcb = dvc + ((size_t)bh * p.nt + c_blk) * D;
    const int r_lo = warp * 16 + g8;
    // centre this warp's rows in place (rows past the block's end stay zero: their results are dropped)
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
        const int col = n * 8 + col0;
        const float2 kc2 = *reinterpret_cast<const float2*>(kcb + col);
        const float2 vc2 = *reinterpret_cast<const float2*>(vcb + col);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = r_lo + 8 * r;
            if (row < nkeys) {
                const float2 k2 = unpack<BF16>(*pair_at<D>(ks, row, col));
                const float2 v2 = unpack<BF16>(*pair_at<D>(vs, row, col));
                *pair_at<D>(ks, row, col) = pack<BF16>(k2.x - kc2.x, k2.y - kc2.y);
                *pair_at<D>(vs, row, col) = pack<BF16>(v2.x - vc2.x * inv_len, v2.y - vc2.y * inv_len);
            }
        }
    }
    __syncthreads();        // dh tile complete, centred rows visible to the whole warp
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
        uint32_t ak[4], av[4];
        ldsm_x4(ak, smem_addr(ks) + tile_off<D>(arow, 2 * kk + (lane >> 4)));
        ldsm_x4(av, smem_addr(vs) + tile_off<D>(arow, 2 * kk + (lane >> 4)));
#pragma unroll
        for (int n2 = 0; n2 < NT8 / 2; ++n2) {
            uint32_t b[4];
            // dk[key][d] += sum_vv v'[key][vv] dh[d][vv]: dh rows as the N dimension
            const int drow_ = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
            ldsm_x4(b, smem_addr(qs) + tile_off<D>(drow_, 2 * kk + ((lane >> 3) & 1)));
            mma16816<BF16>(dka[2 * n2], av, b[0], b[1]);
            mma16816<BF16>(dka[2 * n2 + 1], av, b[2], b[3]);
            // dv[key][vv] += sum_d k'[key][d] dh[d][vv]: dh rows as the K dimension
            const int krow = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            ldsm_x4_trans(b, smem_addr(qs) + tile_off<D>(krow, 2 * n2 + (lane >> 4)));
            mma16816<BF16>(dva[2 * n2], ak, b[0], b[1]);
            mma16816<BF16>(dva[2 * n2 + 1], ak, b[2], b[3]);
        }
    }
    __syncwarp();           // this warp's A-fragment reads of its own rows are done: reuse them for the output
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
        const int col = n * 8 + col0;
        const float2 a2 = *reinterpret_cast<const float2*>(dkcb + col);
        const float2 b2 = *reinterpret_cast<const float2*>(dvcb + col);
        *pair_at<D>(ks, r_lo, col) = pack<BF16>(dka[n][0] + a2.x * inv_len, dka[n][1] + a2.y * inv_len);
        *pair_at<D>(ks, r_lo + 8, col) = pack<BF16>(dka[n][2] + a2.x * inv_len, dka[n][3] + a2.y * inv_len);
        *pair_at<D>(vs, r_lo, col) = pack<BF16>(dva[n][0] + b2.x, dva[n][1] + b2.y);
        *pair_at<D>(vs, r_lo + 8, col) = pack<BF16>(dva[n][2] + b2.x, dva[n][3] + b2.y);
    }
    __syncthreads();
    {
        uint8_t* gk = static_cast<uint8_t*>(dk) + tile_g;
        uint8_t* gv = static_cast<uint8_t*>(dv) + tile_g;
        for (int i = threadIdx.x; i < nkeys * CH; i += kThreads) {
            const int r = i / CH, c = i - r * CH;
            *reinterpret_cast<uint4*>(gk + (size_t)r * D * 2 + c * 16) = *reinterpret_cast<const uint4*>(ks + tile_off<D>(r, c));
            *reinterpret_cast<uint4*>(gv + (size_t)r * D * 2 + c * 16) = *reinterpret_cast<const uint4*>(vs + tile_off<D>(r, c));
        }
    }
}

}  // namespace pisa_mma
}  // namespace fbla
