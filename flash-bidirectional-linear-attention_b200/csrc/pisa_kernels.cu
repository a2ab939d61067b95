// piecewise_sparse_attention (PISA), forward: block statistics, the first-order state and the
// attention kernel.  CUDA-core (fp32 FMA) implementation for any dk, dv, block size <= 128.
//
// Per query row (all logits in the log2 domain, sm = scale * log2(e)):
//   exact   : s_j = sm q.k_j on the tokens j of the selected key blocks,  p_j = 2^(s_j - m)
//   zeroth  : a_c = sm q.kc_c on the unselected blocks c,                 pi_c = 2^(a_c - m)
//   g = sum_c pi_c * len_c,   l = sum_j p_j,   m = running maximum of all s_j, a_c
//   o = ( sum_j p_j v_j + sum_c pi_c vc_c + (q h) g scale / T ) / (l + g)
// The reference rescales l and the numerator when the maximum grows between groups of blocks
// but not g (kernel.py:262-276), so its result depends on the autotuned GROUP_SIZE once there
// are more blocks than one group; here g is rescaled too, which equals the reference whenever
// one group covers all blocks.
#include <cstdlib>

#include "fbla_common.cuh"
#include "pisa_mma.cuh"
#include "pisa_mma_bwd.cuh"
#include "pisa_tc.cuh"
#include "tc_kernels.cuh"

namespace fbla {
namespace {

constexpr int kPisaThreads = 256;
constexpr int kPisaWarps = kPisaThreads / 32;
constexpr int kChunkRows = 64;       // block statistics are consumed 64 blocks at a time
constexpr int kMaxRowsPerWarp = 16;  // block_size <= 128

__device__ __forceinline__ float wsum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ float wmax(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

struct PisaParams {
    int heads, dk, dv, bs, ns, nt;
    int T;
    float scale;
};

// qc, kc = block means (divided by the true length of a ragged last block), vc = block sums.
template <typename T>
__global__ void __launch_bounds__(128)
pisa_block_stats_kernel(PisaParams p, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                        float* __restrict__ qc, float* __restrict__ kc, float* __restrict__ vc) {
    const int c = blockIdx.x, bh = blockIdx.y, d = threadIdx.x;
    const int t0 = c * p.bs;
    const int len = min(p.bs, p.T - t0);
    const size_t row0 = (size_t)bh * p.T + t0;
    float sq = 0.f, sk = 0.f, sv = 0.f;
    const bool has_k = d < p.dk, has_v = d < p.dv;
    // eight rows in flight per thread: the loads of a group are issued before the first of them is added
    // (a row-at-a-time loop waits out one memory latency per row); the order of the sums is unchanged
    int t = 0;
    for (; t + 8 <= len; t += 8) {
        T a[8], b[8], e[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (has_k) {
                a[u] = q[(row0 + t + u) * p.dk + d];
                b[u] = k[(row0 + t + u) * p.dk + d];
            }
            if (has_v) e[u] = v[(row0 + t + u) * p.dv + d];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (has_k) {
                sq += to_f<T>(a[u]);
                sk += to_f<T>(b[u]);
            }
            if (has_v) sv += to_f<T>(e[u]);
        }
    }
    for (; t < len; ++t) {
        if (has_k) {
            sq += to_f<T>(q[(row0 + t) * p.dk + d]);
            sk += to_f<T>(k[(row0 + t) * p.dk + d]);
        }
        if (has_v) sv += to_f<T>(v[(row0 + t) * p.dv + d]);
    }
    const size_t blk = (size_t)bh * p.nt + c;
    if (d < p.dk) {
        qc[blk * p.dk + d] = sq / (float)len;
        kc[blk * p.dk + d] = sk / (float)len;
    }
    if (d < p.dv) vc[blk * p.dv + d] = sv;
}

// h = K^T V - sum_c kc_c (x) vc_c.  One CTA per (16 rows of h, batch*head): the block statistics are
// staged through shared memory 64 blocks at a time; a thread owns one row and dv/16 columns.
constexpr int kFoRows = 16;
__global__ void __launch_bounds__(256)
pisa_first_order_kernel(PisaParams p, const float* __restrict__ kv, const float* __restrict__ kc,
                        const float* __restrict__ vc, float* __restrict__ h) {
    __shared__ float ks[kChunkRows][kFoRows];
    __shared__ float vs[kChunkRows][128];
    const int bh = blockIdx.y, a0 = blockIdx.x * kFoRows;
    const int r = threadIdx.x >> 4, cg = threadIdx.x & 15;      // row a0 + r, columns cg, cg + 16, ...
    const float* kcb = kc + (size_t)bh * p.nt * p.dk;
    const float* vcb = vc + (size_t)bh * p.nt * p.dv;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int c0 = 0; c0 < p.nt; c0 += kChunkRows) {
        const int nc = min(kChunkRows, p.nt - c0);
        __syncthreads();
#pragma unroll 4
        for (int i = threadIdx.x; i < nc * kFoRows; i += 256) {
            const int c = i / kFoRows, a = i - c * kFoRows;
            ks[c][a] = (a0 + a < p.dk) ? kcb[(size_t)(c0 + c) * p.dk + a0 + a] : 0.f;
        }
        // rows of vc are contiguous in memory: a flat copy, eight loads in flight per thread
        {
            const float* src = vcb + (size_t)c0 * p.dv;
            const int n = nc * p.dv;
            const bool flat = p.dv == 128;
            for (int i0 = 0; i0 < n; i0 += 256 * 8) {
                float tmp[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * 256 + threadIdx.x;
                    tmp[u] = i < n ? src[i] : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * 256 + threadIdx.x;
                    if (i < n) {
                        if (flat) (&vs[0][0])[i] = tmp[u];
                        else vs[i / p.dv][i % p.dv] = tmp[u];
                    }
                }
            }
        }
        __syncthreads();
        for (int c = 0; c < nc; ++c) {
            const float kk = ks[c][r];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int b = cg + 16 * j;
                if (b < p.dv) acc[j] = fmaf(kk, vs[c][b], acc[j]);
            }
        }
    }
    if (a0 + r >= p.dk) return;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int b = cg + 16 * j;
        if (b < p.dv) {
            const size_t at = (size_t)bh * p.dk * p.dv + (size_t)(a0 + r) * p.dv + b;
            h[at] = kv[at] - acc[j];
        }
    }
}

// p-norm of each block's first-order state hc_c = (K_c - kc_c)^T V_c over its dk*dv entries (the
// selection bias of use_bias=True).  One CTA per (block, batch*head): the centred keys and the values
// of the block sit in shared memory as fp32, every thread forms dk*dv/256 entries of hc_c.
template <typename T>
__global__ void __launch_bounds__(256)
pisa_block_hnorm_kernel(PisaParams p, const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ kc,
                        float pnorm, float* __restrict__ hnorm) {
    extern __shared__ float smem[];
    const int K = p.dk, V = p.dv;
    float* ks = smem;                   // [bs][K]  k - kc
    float* vs = ks + p.bs * K;          // [bs][V]
    __shared__ float red[8];
    const int c = blockIdx.x, bh = blockIdx.y;
    const int t0 = c * p.bs;
    const int len = min(p.bs, p.T - t0);
    const size_t row0 = (size_t)bh * p.T + t0;
    const float* kcb = kc + ((size_t)bh * p.nt + c) * K;
    for (int i = threadIdx.x; i < len * K; i += 256) ks[i] = to_f<T>(k[row0 * K + i]) - kcb[i % K];
    for (int i = threadIdx.x; i < len * V; i += 256) vs[i] = to_f<T>(v[row0 * V + i]);
    __syncthreads();
    float acc = 0.f;
    for (int e = threadIdx.x; e < K * V; e += 256) {
        const int a = e / V, b = e - a * V;
        float h = 0.f;
        for (int t = 0; t < len; ++t) h = fmaf(ks[t * K + a], vs[t * V + b], h);
        const float m = fabsf(h);
        acc += pnorm == 2.f ? m * m : (pnorm == 1.f ? m : __powf(m, pnorm));
    }
    acc = wsum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int w = 0; w < 8; ++w) s += red[w];
        hnorm[(size_t)bh * p.nt + c] = pnorm == 2.f ? sqrtf(s) : (pnorm == 1.f ? s : __powf(s, 1.f / pnorm));
    }
}

// One CTA per (query block, batch*head); warp w owns query rows w, w+8, ...; inside a group of 32
// keys the lanes own one key each for the logits and a slice of the value columns for p.V.
template <typename T>
__global__ void __launch_bounds__(kPisaThreads)
pisa_fwd_kernel(PisaParams p, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                const float* __restrict__ kc, const float* __restrict__ vc, const float* __restrict__ h,
                const int32_t* __restrict__ indices, T* __restrict__ o, float* __restrict__ row_stats) {
    extern __shared__ float smem[];
    const int K = p.dk, V = p.dv, KP = K + 1, VP = V + 1;
    const int rows_buf = max(p.bs, kChunkRows);
    float* qs = smem;                          // [bs][K]
    float* kb = qs + p.bs * K;                 // [rows_buf][K+1]   keys / block means / (h, flat)
    float* vb = kb + rows_buf * KP;            // [rows_buf][V+1]   values / block sums
    unsigned char* sel = reinterpret_cast<unsigned char*>(vb + rows_buf * VP);   // [nt] selected?

    const int i_blk = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = i_blk * p.bs;
    const int nrows = min(p.bs, p.T - t0);
    const size_t base_row = (size_t)bh * p.T;
    const float sm = p.scale * 1.44269504f;
    const int32_t* idx = indices + ((size_t)bh * p.nt + i_blk) * p.ns;

    for (int i = threadIdx.x; i < p.bs * K; i += kPisaThreads) {
        const int r = i / K, d = i - r * K;
        qs[i] = r < nrows ? to_f<T>(q[(base_row + t0 + r) * K + d]) : 0.f;
    }
    for (int i = threadIdx.x; i < p.nt; i += kPisaThreads) sel[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < p.ns; i += kPisaThreads) {
        const int c = idx[i];
        if (c >= 0 && c < p.nt) sel[c] = 1;
    }

    float m[kMaxRowsPerWarp], l[kMaxRowsPerWarp], g[kMaxRowsPerWarp], acc[kMaxRowsPerWarp][4];
#pragma unroll
    for (int i = 0; i < kMaxRowsPerWarp; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
        g[i] = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
    }

    // One group of up to 32 keys (rows j0.. of kb / vb) against one query row.
    // weight_len < 0: exact keys (l accumulates); otherwise block means: g accumulates pi * len.
    auto group = [&](int ri, int r, int j0, int nvalid, bool approx, int c0) {
        const int j = j0 + lane;
        float s = -INFINITY;
        bool ok = j < nvalid;
        if (approx && ok) ok = !sel[c0 + j];
        if (ok) {
            float a = 0.f;
            const float* qrow = qs + r * K;
            const float* krow = kb + j * KP;
            for (int d = 0; d < K; ++d) a = fmaf(qrow[d], krow[d], a);
            s = a * sm;
        }
        const float gmax = wmax(s);
        if (gmax == -INFINITY) return;                       // nothing valid in this group
        const float new_m = fmaxf(m[ri], gmax);
        const float alpha = exp2f(m[ri] - new_m);            // 0 on the first group (m = -inf)
        const float pj = ok ? exp2f(s - new_m) : 0.f;
        l[ri] *= alpha;
        g[ri] *= alpha;
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[ri][c] *= alpha;
        if (approx) {
            const int cblk = c0 + j;
            const float len = (cblk == p.nt - 1) ? (float)(p.T - (p.nt - 1) * p.bs) : (float)p.bs;
            g[ri] += wsum(pj * len);
        } else {
            l[ri] += wsum(pj);
        }
        const int jn = min(32, nvalid - j0);
        for (int jj = 0; jj < jn; ++jj) {
            const float pb = __shfl_sync(0xffffffffu, pj, jj);
            const float* vrow = vb + (j0 + jj) * VP;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = lane + 32 * c;
                if (col < V) acc[ri][c] = fmaf(pb, vrow[col], acc[ri][c]);
            }
        }
        m[ri] = new_m;
    };

    // ---- phase 1: exact attention on the selected key blocks ----
    for (int n = 0; n < p.ns; ++n) {
        __syncthreads();
        const int cb = idx[n];
        const bool cb_ok = cb >= 0 && cb < p.nt;                   // a bad index selects nothing (and reads nothing)
        const int bos = cb_ok ? cb * p.bs : 0;
        const int nvalid = cb_ok ? max(0, min(p.bs, p.T - bos)) : 0;
        for (int i = threadIdx.x; i < p.bs * K; i += kPisaThreads) {
            const int r = i / K, d = i - r * K;
            kb[r * KP + d] = r < nvalid ? to_f<T>(k[(base_row + bos + r) * K + d]) : 0.f;
        }
        for (int i = threadIdx.x; i < p.bs * V; i += kPisaThreads) {
            const int r = i / V, d = i - r * V;
            vb[r * VP + d] = r < nvalid ? to_f<T>(v[(base_row + bos + r) * V + d]) : 0.f;
        }
        __syncthreads();
        for (int r = warp, ri = 0; r < nrows; r += kPisaWarps, ++ri)
            for (int j0 = 0; j0 < nvalid; j0 += 32) group(ri, r, j0, nvalid, false, 0);
    }
    // ---- phase 2: zeroth order on the unselected blocks, 64 blocks at a time ----
    for (int c0 = 0; c0 < p.nt; c0 += kChunkRows) {
        __syncthreads();
        const int nvalid = min(kChunkRows, p.nt - c0);
        const float* kcb = kc + ((size_t)bh * p.nt + c0) * K;
        const float* vcb = vc + ((size_t)bh * p.nt + c0) * V;
        for (int i = threadIdx.x; i < nvalid * K; i += kPisaThreads) {
            const int r = i / K, d = i - r * K;
            kb[r * KP + d] = kcb[i];
        }
        for (int i = threadIdx.x; i < nvalid * V; i += kPisaThreads) {
            const int r = i / V, d = i - r * V;
            vb[r * VP + d] = vcb[i];
        }
        __syncthreads();
        for (int r = warp, ri = 0; r < nrows; r += kPisaWarps, ++ri)
            for (int j0 = 0; j0 < nvalid; j0 += 32) group(ri, r, j0, nvalid, true, c0);
    }
    // ---- phase 3: first order, (q h) g scale / T; h (K x V, flat) reuses the key/value buffers ----
    __syncthreads();
    float* hs = kb;
    const float* hb = h + (size_t)bh * K * V;
    for (int i = threadIdx.x; i < K * V; i += kPisaThreads) hs[i] = hb[i];
    __syncthreads();
    const float w = p.scale / (float)p.T;
    for (int r = warp, ri = 0; r < nrows; r += kPisaWarps, ++ri) {
        const float* qrow = qs + r * K;
        const float corr = g[ri] * w;
        const float den = l[ri] + g[ri];
        const float rden = 1.f / den;
        const size_t row = base_row + t0 + r;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            if (col < V) {
                float rr = 0.f;
                for (int d = 0; d < K; ++d) rr = fmaf(qrow[d], hs[d * V + col], rr);
                o[row * V + col] = from_f<T>((acc[ri][c] + rr * corr) * rden);
            }
        }
        if (row_stats != nullptr && lane == 0)
            *reinterpret_cast<float4*>(row_stats + row * 4) = make_float4(m[ri], den, g[ri], 1.f / den);
    }
}

size_t fwd_smem_bytes(const PisaParams& p) {
    const int rows_buf = p.bs > kChunkRows ? p.bs : kChunkRows;
    return sizeof(float) * ((size_t)p.bs * p.dk + (size_t)rows_buf * (p.dk + 1 + p.dv + 1)) + (size_t)p.nt + 16;
}

}  // namespace

// Test hook: route fbla_pisa_fwd to the CUDA-core kernel whatever the shape (FBLA_PISA_GENERIC=1).
static const bool g_pisa_force_generic = [] {
    const char* e = getenv("FBLA_PISA_GENERIC");
    return e != nullptr && e[0] == '1';
}();

struct PisaArgs {
    PisaParams kp;
    int bh;
    int dtype;
};

static int resolve_pisa(const fbla_pisa_problem* p, PisaArgs* a) {
    if (p == nullptr) return api_fail(FBLA_ERR_INVALID, "problem is NULL");
    if (p->dtype != FBLA_F32 && p->dtype != FBLA_BF16 && p->dtype != FBLA_F16)
        return api_fail(FBLA_ERR_INVALID, "dtype %d is not one of FBLA_F32/FBLA_BF16/FBLA_F16", p->dtype);
    if (p->dk < 1 || p->dk > 128 || p->dv < 1 || p->dv > 128)
        return api_fail(FBLA_ERR_UNSUPPORTED, "dk=%d, dv=%d: feature dims must be in [1, 128]", p->dk, p->dv);
    if (p->block_size < 1 || p->block_size > 128)
        return api_fail(FBLA_ERR_UNSUPPORTED, "block_size=%d must be in [1, 128]", p->block_size);
    if (p->batch < 1 || p->heads < 1 || p->seq_len < 1 || p->seq_len > 0x7fffffffLL)
        return api_fail(FBLA_ERR_INVALID, "batch, heads and seq_len must be positive");
    const long long nt = (p->seq_len + p->block_size - 1) / p->block_size;
    if (p->num_selected < 1 || p->num_selected > nt)
        return api_fail(FBLA_ERR_INVALID, "num_selected=%d must be in [1, %lld]", p->num_selected, nt);
    if ((long long)p->batch * p->heads > 65535 || nt > 0x7fffffffLL)
        return api_fail(FBLA_ERR_UNSUPPORTED, "problem too large");
    a->kp.heads = p->heads;
    a->kp.dk = p->dk;
    a->kp.dv = p->dv;
    a->kp.bs = p->block_size;
    a->kp.ns = p->num_selected;
    a->kp.nt = (int)nt;
    a->kp.T = (int)p->seq_len;
    a->kp.scale = p->scale;
    a->bh = p->batch * p->heads;
    a->dtype = p->dtype;
    return FBLA_OK;
}

#define PISA_BY_DTYPE(dtype, ...)                                            \
    switch (dtype) {                                                         \
        case FBLA_F32: { using T = float; __VA_ARGS__; break; }              \
        case FBLA_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }     \
        default: { using T = __half; __VA_ARGS__; break; }                   \
    }

// ---- block selection: scores of the block means, top-k per query block ------------------------------
// One warp per query block.  score[j] = qc_i . (kc_j * scale), with the operands and the result rounded
// to the element type of q, k, v the way the reference forms them (block means stored in that type, the
// product taken in it; kernel.py:313); with a bias, score[j] + log(hnorm_j + 1e-5), whose softmax over j
// the reference ranks (kernel.py:314-315: softmax is monotone, so the order is the same).  The ns largest
// are written in descending order; equal scores go to the lower block index, NaN counts as smallest.
constexpr int kSelectWarps = 8;
constexpr int kSelectMaxBlocks = 1024;              // 32 scores per lane
constexpr int kSelectChunk = 128;                   // key blocks staged in shared memory per pass

__device__ __forceinline__ float round_like(float x, int dtype) {
    if (dtype == FBLA_BF16) return __bfloat162float(__float2bfloat16_rn(x));
    if (dtype == FBLA_F16) return __half2float(__float2half_rn(x));
    return x;
}

// (score, block) as one integer whose order is: larger score first, then lower block index; 0 = nothing.
__device__ __forceinline__ unsigned long long select_key(float x, int j) {
    unsigned int u = __float_as_uint(x);
    u = (x != x) ? 1u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));
    if (u < 2u) u = (x != x) ? 1u : 2u;
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (unsigned int)j);
}

// The CTA serves eight query blocks of one (batch, head): the key means, scaled and rounded, are staged
// in shared memory 128 blocks at a time (rows padded by four floats, so that the lanes' 128-bit reads of
// 32 different rows are free of bank conflicts), and every warp forms the scores of its query block from
// there.  PER = score slots per lane (PER * 32 >= number of blocks).
template <int PER>
__global__ void __launch_bounds__(kSelectWarps * 32)
pisa_select_kernel(PisaParams p, int dtype, const float* __restrict__ qc, const float* __restrict__ kc,
                   const float* __restrict__ hnorm, int32_t* __restrict__ indices) {
    extern __shared__ __align__(16) float select_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i_blk = blockIdx.x * kSelectWarps + warp, bh = blockIdx.y;
    const bool valid = i_blk < p.nt;
    const int K = p.dk, K4 = (K + 3) & ~3, KS = K4 + 4;
    float* kcs = select_smem;                                   // [kSelectChunk][KS]
    float* qrow = select_smem + kSelectChunk * KS + warp * K4;  // [K4], zero past K
    if (valid) {
        const float* qsrc = qc + ((size_t)bh * p.nt + i_blk) * K;
        for (int d = lane; d < K4; d += 32) qrow[d] = d < K ? round_like(qsrc[d], dtype) : 0.f;
    }
    unsigned long long key[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) key[u] = 0ull;
#pragma unroll
    for (int c = 0; c < PER / 4; ++c) {
        const int c0 = c * kSelectChunk;
        const int rows = min(kSelectChunk, p.nt - c0);
        if (rows <= 0) continue;                    // uniform over the CTA
        __syncthreads();
        const float* src = kc + ((size_t)bh * p.nt + c0) * K;
        for (int i0 = 0; i0 < rows * K4; i0 += kSelectWarps * 32 * 8) {      // eight loads in flight per thread
            float tmp[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * kSelectWarps * 32 + threadIdx.x;
                const int r = i / K4, d = i - r * K4;
                tmp[u] = (i < rows * K4 && d < K) ? src[(size_t)r * K + d] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * kSelectWarps * 32 + threadIdx.x;
                const int r = i / K4, d = i - r * K4;
                if (i < rows * K4) kcs[r * KS + d] = d < K ? round_like(tmp[u] * p.scale, dtype) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int jl = u * 32 + lane, j = c0 + jl;
            if (valid && jl < rows) {
                const float4* krow = reinterpret_cast<const float4*>(kcs + jl * KS);
                const float4* q4 = reinterpret_cast<const float4*>(qrow);
                float acc = 0.f;
                for (int d = 0; d < K4 / 4; ++d) {
                    const float4 a = q4[d], b = krow[d];
                    acc = fmaf(a.x, b.x, acc);
                    acc = fmaf(a.y, b.y, acc);
                    acc = fmaf(a.z, b.z, acc);
                    acc = fmaf(a.w, b.w, acc);
                }
                acc = round_like(acc, dtype);
                if (hnorm != nullptr)
                    acc = round_like(acc + round_like(logf(round_like(hnorm[(size_t)bh * p.nt + j], dtype) + 1e-5f), dtype), dtype);
                key[c * 4 + u] = select_key(acc, j);
            }
        }
    }
    if (!valid) return;
    int32_t* out = indices + ((size_t)bh * p.nt + i_blk) * p.ns;
    for (int n = 0; n < p.ns; ++n) {
        unsigned long long best = 0ull;
#pragma unroll
        for (int u = 0; u < PER; ++u) best = key[u] > best ? key[u] : best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        const int at = (int)(0xffffffffu - (unsigned int)(best & 0xffffffffull));
        if (lane == 0) out[n] = best != 0ull ? at : 0;
#pragma unroll
        for (int u = 0; u < PER; ++u)
            if (key[u] == best) key[u] = 0ull;          // retire the winner (keys are unique: they carry the index)
    }
}

}  // namespace fbla

extern "C" {

int fbla_pisa_block_stats(const fbla_pisa_problem* p, const void* q, const void* k, const void* v, float* qc,
                          float* kc, float* vc, fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!q || !k || !v || !qc || !kc || !vc) return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    dim3 grid(a.kp.nt, a.bh);
    cudaStream_t st = (cudaStream_t)stream;
    PISA_BY_DTYPE(a.dtype, (fbla::pisa_block_stats_kernel<T><<<grid, 128, 0, st>>>(a.kp, (const T*)q, (const T*)k,
                                                                                  (const T*)v, qc, kc, vc)));
    fbla::note_launches(1);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "block statistics: %s", cudaGetErrorString(e));
}

int fbla_pisa_select_blocks(const fbla_pisa_problem* p, const float* qc, const float* kc, const float* hnorm,
                            int32_t* indices, fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!qc || !kc || !indices) return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    if (a.kp.nt > fbla::kSelectMaxBlocks || a.kp.ns > a.kp.nt)
        return fbla::api_fail(FBLA_ERR_UNSUPPORTED, "block selection serves up to %d blocks (%d given) and at most as many "
                              "selected blocks as there are blocks", fbla::kSelectMaxBlocks, a.kp.nt);
    dim3 grid((a.kp.nt + fbla::kSelectWarps - 1) / fbla::kSelectWarps, a.bh);
    const int k4 = (a.kp.dk + 3) & ~3;
    const size_t smem = sizeof(float) * ((size_t)fbla::kSelectChunk * (k4 + 4) + (size_t)fbla::kSelectWarps * k4);
    auto run = [&](auto kern) {
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return;
        kern<<<grid, fbla::kSelectWarps * 32, smem, (cudaStream_t)stream>>>(a.kp, a.dtype, qc, kc, hnorm, indices);
    };
    if (a.kp.nt <= 128) run(fbla::pisa_select_kernel<4>);
    else run(fbla::pisa_select_kernel<32>);
    fbla::note_launches(1);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "block selection: %s", cudaGetErrorString(e));
}

int fbla_pisa_block_hnorm(const fbla_pisa_problem* p, const void* k, const void* v, const float* kc, float pnorm,
                          float* hnorm, fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!k || !v || !kc || !hnorm) return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    if (!(pnorm > 0.f)) return fbla::api_fail(FBLA_ERR_INVALID, "the norm order must be positive");
    dim3 grid(a.kp.nt, a.bh);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = sizeof(float) * (size_t)a.kp.bs * (a.kp.dk + a.kp.dv);
    cudaError_t e = cudaSuccess;
    PISA_BY_DTYPE(a.dtype, {
        auto kern = fbla::pisa_block_hnorm_kernel<T>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) kern<<<grid, 256, smem, st>>>(a.kp, (const T*)k, (const T*)v, kc, pnorm, hnorm);
    });
    fbla::note_launches(1);
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "block norms: %s", cudaGetErrorString(e));
}

int fbla_pisa_first_order_state(const fbla_pisa_problem* p, const float* kv, const float* kc, const float* vc,
                                float* h, fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!kv || !kc || !vc || !h) return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    dim3 grid((a.kp.dk + fbla::kFoRows - 1) / fbla::kFoRows, a.bh);
    fbla::pisa_first_order_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a.kp, kv, kc, vc, h);
    fbla::note_launches(1);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "first-order state: %s", cudaGetErrorString(e));
}

int64_t fbla_pisa_fwd_scratch_bytes(const fbla_pisa_problem* p) {
    fbla::PisaArgs a;
    if (fbla::resolve_pisa(p, &a)) return -1;
    if (!fbla::pisa_tc_supported(a.dtype, a.kp.dk, a.kp.dv, a.kp.bs, a.kp.nt, a.kp.ns) || fbla::g_pisa_force_generic) return 0;
    return fbla::pisa_tc_scratch_bytes(a.bh, a.kp.dk, a.kp.nt);
}

int fbla_pisa_fwd_ws(const fbla_pisa_problem* p, const void* q, const void* k, const void* v, const float* kc,
                     const float* vc, const float* h, const int32_t* indices, void* o, float* row_stats, void* scratch,
                     size_t scratch_bytes, fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!q || !k || !v || !kc || !vc || !h || !indices || !o)
        return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    const int64_t need = fbla_pisa_fwd_scratch_bytes(p);
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                           reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc) |
                           reinterpret_cast<uintptr_t>(h)) & 15u) == 0 &&
                         (reinterpret_cast<uintptr_t>(scratch) & 127u) == 0;
    // (the tensor-core kernel takes row maxima before scaling: it needs a positive scale)
    if (need <= 0 || scratch == nullptr || (int64_t)scratch_bytes < need || !aligned || !(a.kp.scale > 0.f))
        return fbla_pisa_fwd(p, q, k, v, kc, vc, h, indices, o, row_stats, stream);
    if (const int site = fbla::tc_device_status())
        return fbla::api_fail(FBLA_ERR_DEVICE, "a kernel gave up a bounded wait (site %d); results are invalid", site);
    const cudaError_t e = fbla::pisa_tc_fwd(a.dtype, a.bh, a.kp.dk, a.kp.nt, a.kp.ns, a.kp.T, a.kp.scale, q, k, v, kc, vc, h,
                                            indices, o, row_stats, scratch, (cudaStream_t)stream);
    fbla::note_launches(2);
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "attention kernel: %s", cudaGetErrorString(e));
}

int fbla_pisa_fwd(const fbla_pisa_problem* p, const void* q, const void* k, const void* v, const float* kc,
                  const float* vc, const float* h, const int32_t* indices, void* o, float* row_stats,
                  fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!q || !k || !v || !kc || !vc || !h || !indices || !o)
        return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    dim3 grid(a.kp.nt, a.bh);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
    // tensor-core kernel for the common shape; the CUDA-core kernel serves everything else
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                           reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc) |
                           reinterpret_cast<uintptr_t>(h)) & 15u) == 0;
    if (a.dtype != FBLA_F32 && a.kp.bs == 64 && a.kp.dk == a.kp.dv && (a.kp.dk == 64 || a.kp.dk == 128) && aligned &&
        !fbla::g_pisa_force_generic) {
        fbla::pisa_mma::Params mp{a.kp.heads, a.kp.ns, a.kp.nt, a.kp.T, a.kp.scale};
        auto run = [&](auto kern, size_t smem) {
            if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess)
                kern<<<grid, fbla::pisa_mma::kThreads, smem, st>>>(mp, q, k, v, kc, vc, h, indices, o, row_stats);
        };
        const bool bf = a.dtype == FBLA_BF16;
        if (a.kp.dk == 64) {
            const size_t smem = fbla::pisa_mma::smem_bytes<64>(a.kp.nt);
            if (bf) run(fbla::pisa_mma::pisa_fwd_mma_kernel<64, true>, smem);
            else run(fbla::pisa_mma::pisa_fwd_mma_kernel<64, false>, smem);
        } else {
            const size_t smem = fbla::pisa_mma::smem_bytes<128>(a.kp.nt);
            if (bf) run(fbla::pisa_mma::pisa_fwd_mma_kernel<128, true>, smem);
            else run(fbla::pisa_mma::pisa_fwd_mma_kernel<128, false>, smem);
        }
        fbla::note_launches(1);
        if (e == cudaSuccess) e = cudaGetLastError();
        return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "attention kernel: %s", cudaGetErrorString(e));
    }
    const size_t smem = fbla::fwd_smem_bytes(a.kp);
    PISA_BY_DTYPE(a.dtype, {
        auto kern = fbla::pisa_fwd_kernel<T>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            kern<<<grid, fbla::kPisaThreads, smem, st>>>(a.kp, (const T*)q, (const T*)k, (const T*)v, kc, vc, h, indices,
                                                          (T*)o, row_stats);
    });
    fbla::note_launches(1);
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "attention kernel: %s", cudaGetErrorString(e));
}

}  // extern "C"

// =========================================================================================
// Backward.  The reference has no backward for this operator; these kernels differentiate the
// forward above with the block selection held constant (gradients flow through the block
// statistics kc, vc, h as well).  Per query row, with dnum = dO / D, dD = -(o . dO) / D,
// r = q h, w = scale / T:
//   dg = dD + (dnum . r) w            dr = dnum g w
//   exact keys j : dp_j = dnum . v_j + dD      ds_j = p_j dp_j
//   blocks c     : dpi_c = dnum . vc_c + dg len_c   da_c = pi_c dpi_c
//   dq  = scale (sum_j ds_j k_j + sum_c da_c kc_c) + h dr
//   dk_j += scale ds_j q      dv_j += p_j dnum
//   dkc_c += scale da_c q     dvc_c += pi_c dnum     dh += q (x) dr
// and through the statistics:  dk_t += dkc_c / len_c + dh (v_t - vc_c / len_c),
//                              dv_t += dvc_c + dh^T (k_t - kc_c).
// Kernel 1 (one CTA per query block) writes dq and the per-row dD, and adds dkc, dvc, dh into
// fp32 buffers with atomics; kernel 2 (one CTA per key block) gathers the exact-attention part
// of dk, dv from the query blocks that selected it and adds the statistics terms.
// =========================================================================================
namespace fbla {
namespace {

template <typename T>
__global__ void __launch_bounds__(kPisaThreads)
pisa_bwd_q_kernel(PisaParams p, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                  const T* __restrict__ o, const T* __restrict__ d_o, const float* __restrict__ kc,
                  const float* __restrict__ vc, const float* __restrict__ h, const int32_t* __restrict__ indices,
                  const float* __restrict__ row_stats, T* __restrict__ dq, float* __restrict__ dkc,
                  float* __restrict__ dvc, float* __restrict__ dh, float* __restrict__ drow) {
    extern __shared__ float smem[];
    const int K = p.dk, V = p.dv, KP = K + 1, VP = V + 1;
    const int rows_buf = max(p.bs, kChunkRows);
    float* qs = smem;                          // [bs][K]
    float* dos = qs + p.bs * K;                // [bs][V]   dO rows
    float* drs = dos + p.bs * V;               // [bs][V]   dr rows
    float* kb = drs + p.bs * V;                // [rows_buf][K+1]
    float* vb = kb + rows_buf * KP;            // [rows_buf][V+1]
    float* das = vb + rows_buf * VP;           // [bs][64]  scale * da   (one chunk of blocks)
    float* pis = das + p.bs * kChunkRows;      // [bs][64]  pi / D
    unsigned char* sel = reinterpret_cast<unsigned char*>(pis + p.bs * kChunkRows);

    const int i_blk = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = i_blk * p.bs;
    const int nrows = min(p.bs, p.T - t0);
    const size_t base_row = (size_t)bh * p.T;
    const float sm = p.scale * 1.44269504f;
    const float w = p.scale / (float)p.T;
    const int32_t* idx = indices + ((size_t)bh * p.nt + i_blk) * p.ns;

    for (int i = threadIdx.x; i < p.bs * K; i += kPisaThreads) {
        const int r = i / K, d = i - r * K;
        qs[i] = r < nrows ? to_f<T>(q[(base_row + t0 + r) * K + d]) : 0.f;
    }
    for (int i = threadIdx.x; i < p.bs * V; i += kPisaThreads) {
        const int r = i / V, d = i - r * V;
        dos[i] = r < nrows ? to_f<T>(d_o[(base_row + t0 + r) * V + d]) : 0.f;
        drs[i] = 0.f;
    }
    for (int i = threadIdx.x; i < p.nt; i += kPisaThreads) sel[i] = 0;
    // h, padded rows: hs[d * (V+1) + col]
    float* hs = kb;
    const float* hb = h + (size_t)bh * K * V;
    for (int i = threadIdx.x; i < K * V; i += kPisaThreads) {
        const int d = i / V, c = i - d * V;
        hs[d * VP + c] = hb[i];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.ns; i += kPisaThreads) {
        const int c = idx[i];
        if (c >= 0 && c < p.nt) sel[c] = 1;
    }

    float mrow[kMaxRowsPerWarp], rD[kMaxRowsPerWarp], dD[kMaxRowsPerWarp], dg[kMaxRowsPerWarp];
    float dqa[kMaxRowsPerWarp][4];
    // ---- per row: dD, r = q h, dg, dr, and the first-order part of dq ----
    for (int r = warp, ri = 0; r < p.bs; r += kPisaWarps, ++ri) {
#pragma unroll
        for (int c = 0; c < 4; ++c) dqa[ri][c] = 0.f;
        mrow[ri] = 0.f; rD[ri] = 0.f; dD[ri] = 0.f; dg[ri] = 0.f;
        if (r >= nrows) continue;
        const size_t row = base_row + t0 + r;
        const float4 st = *reinterpret_cast<const float4*>(row_stats + row * 4);
        mrow[ri] = st.x;
        rD[ri] = 1.f / st.y;
        const float g = st.z;
        float od = 0.f, nr = 0.f, rr[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            rr[c] = 0.f;
            if (col < V) {
                od = fmaf(to_f<T>(o[row * V + col]), dos[r * V + col], od);
                float a = 0.f;
                for (int d = 0; d < K; ++d) a = fmaf(qs[r * K + d], hs[d * VP + col], a);
                rr[c] = a;
                nr = fmaf(dos[r * V + col], a, nr);
            }
        }
        dD[ri] = -wsum(od) * rD[ri];
        dg[ri] = dD[ri] + wsum(nr) * rD[ri] * w;
        const float gw = g * w * rD[ri];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            if (col < V) drs[r * V + col] = dos[r * V + col] * gw;
        }
        __syncwarp();
        // dq += h dr  (lanes over the key-feature columns)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            if (col < K) {
                float a = 0.f;
                for (int vv = 0; vv < V; ++vv) a = fmaf(hs[col * VP + vv], drs[r * V + vv], a);
                dqa[ri][c] = a;
            }
        }
        if (lane == 0) drow[row] = dD[ri];
    }
    __syncthreads();
    // dh += q^T dr over the rows of this block
    {
        float* dhb = dh + (size_t)bh * K * V;
        for (int i = threadIdx.x; i < K * V; i += kPisaThreads) {
            const int d = i / V, c = i - d * V;
            float a = 0.f;
            for (int r = 0; r < nrows; ++r) a = fmaf(qs[r * K + d], drs[r * V + c], a);
            atomicAdd(dhb + i, a);
        }
    }

    // one group of up to 32 keys / blocks against one query row
    auto group = [&](int ri, int r, int j0, int nvalid, bool approx, int c0) {
        const int j = j0 + lane;
        bool ok = j < nvalid;
        if (approx && ok) ok = !sel[c0 + j];
        float pj = 0.f, dsj = 0.f;
        if (ok) {
            float a = 0.f, b = 0.f;
            const float* qrow = qs + r * K;
            const float* krow = kb + j * KP;
            for (int d = 0; d < K; ++d) a = fmaf(qrow[d], krow[d], a);
            const float* dorow = dos + r * V;
            const float* vrow = vb + j * VP;
            for (int d = 0; d < V; ++d) b = fmaf(dorow[d], vrow[d], b);
            pj = exp2f(a * sm - mrow[ri]);
            float dp = b * rD[ri];
            if (approx) {
                const int cblk = c0 + j;
                const float len = (cblk == p.nt - 1) ? (float)(p.T - (p.nt - 1) * p.bs) : (float)p.bs;
                dp += dg[ri] * len;
            } else {
                dp += dD[ri];
            }
            dsj = pj * dp * p.scale;
        }
        if (approx) {
            das[r * kChunkRows + j0 + lane] = dsj;
            pis[r * kChunkRows + j0 + lane] = pj * rD[ri];
        }
        const int jn = min(32, nvalid - j0);
        for (int jj = 0; jj < jn; ++jj) {
            const float sb = __shfl_sync(0xffffffffu, dsj, jj);
            const float* krow = kb + (j0 + jj) * KP;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = lane + 32 * c;
                if (col < K) dqa[ri][c] = fmaf(sb, krow[col], dqa[ri][c]);
            }
        }
    };

    // ---- exact part ----
    for (int n = 0; n < p.ns; ++n) {
        __syncthreads();
        const int cb = idx[n];
        const bool cb_ok = cb >= 0 && cb < p.nt;                   // a bad index selects nothing (and reads nothing)
        const int bos = cb_ok ? cb * p.bs : 0;
        const int nvalid = cb_ok ? max(0, min(p.bs, p.T - bos)) : 0;
        for (int i = threadIdx.x; i < p.bs * K; i += kPisaThreads) {
            const int r = i / K, d = i - r * K;
            kb[r * KP + d] = r < nvalid ? to_f<T>(k[(base_row + bos + r) * K + d]) : 0.f;
        }
        for (int i = threadIdx.x; i < p.bs * V; i += kPisaThreads) {
            const int r = i / V, d = i - r * V;
            vb[r * VP + d] = r < nvalid ? to_f<T>(v[(base_row + bos + r) * V + d]) : 0.f;
        }
        __syncthreads();
        for (int r = warp, ri = 0; r < nrows; r += kPisaWarps, ++ri)
            for (int j0 = 0; j0 < nvalid; j0 += 32) group(ri, r, j0, nvalid, false, 0);
    }
    // ---- zeroth-order part, 64 blocks at a time ----
    for (int c0 = 0; c0 < p.nt; c0 += kChunkRows) {
        __syncthreads();
        const int nvalid = min(kChunkRows, p.nt - c0);
        const float* kcb = kc + ((size_t)bh * p.nt + c0) * K;
        const float* vcb = vc + ((size_t)bh * p.nt + c0) * V;
        for (int i = threadIdx.x; i < nvalid * K; i += kPisaThreads) {
            const int r = i / K, d = i - r * K;
            kb[r * KP + d] = kcb[i];
        }
        for (int i = threadIdx.x; i < nvalid * V; i += kPisaThreads) {
            const int r = i / V, d = i - r * V;
            vb[r * VP + d] = vcb[i];
        }
        for (int i = threadIdx.x; i < p.bs * kChunkRows; i += kPisaThreads) {
            das[i] = 0.f;
            pis[i] = 0.f;
        }
        __syncthreads();
        for (int r = warp, ri = 0; r < nrows; r += kPisaWarps, ++ri)
            for (int j0 = 0; j0 < nvalid; j0 += 32) group(ri, r, j0, nvalid, true, c0);
        __syncthreads();
        // dkc_c += sum_rows (scale da_c) q,  dvc_c += sum_rows (pi_c / D) dO
        float* dkcb = dkc + ((size_t)bh * p.nt + c0) * K;
        float* dvcb = dvc + ((size_t)bh * p.nt + c0) * V;
        for (int i = threadIdx.x; i < nvalid * K; i += kPisaThreads) {
            const int cc = i / K, d = i - cc * K;
            float a = 0.f;
            for (int r = 0; r < nrows; ++r) a = fmaf(das[r * kChunkRows + cc], qs[r * K + d], a);
            if (a != 0.f) atomicAdd(dkcb + i, a);
        }
        for (int i = threadIdx.x; i < nvalid * V; i += kPisaThreads) {
            const int cc = i / V, d = i - cc * V;
            float a = 0.f;
            for (int r = 0; r < nrows; ++r) a = fmaf(pis[r * kChunkRows + cc], dos[r * V + d], a);
            if (a != 0.f) atomicAdd(dvcb + i, a);
        }
    }
    for (int r = warp, ri = 0; r < nrows; r += kPisaWarps, ++ri) {
        const size_t row = base_row + t0 + r;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            if (col < K) dq[row * K + col] = from_f<T>(dqa[ri][c]);
        }
    }
}

// One CTA per key block c.  Warp w owns the keys w, w+8, ... of the block; the lanes split the
// feature columns.
template <typename T>
__global__ void __launch_bounds__(kPisaThreads)
pisa_bwd_kv_kernel(PisaParams p, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const T* __restrict__ d_o, const float* __restrict__ kc, const float* __restrict__ vc,
                   const int32_t* __restrict__ indices, const float* __restrict__ row_stats,
                   const float* __restrict__ drow, const float* __restrict__ dkc, const float* __restrict__ dvc,
                   const float* __restrict__ dh, T* __restrict__ dk, T* __restrict__ dv) {
    extern __shared__ float smem[];
    const int K = p.dk, V = p.dv, VP = V + 1;
    float* qs = smem;                  // [bs][K]   q rows of one query block; later the k rows of this block
    float* dos = qs + p.bs * K;        // [bs][V]   dO rows;                   later the v rows of this block
    float* rst = dos + p.bs * V;       // [bs][4]   m, 1/D, dD per query row
    float* dhs = rst + p.bs * 4;       // [K][V+1]

    const int c_blk = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bos = c_blk * p.bs;
    const int nkeys = min(p.bs, p.T - bos);
    const size_t base_row = (size_t)bh * p.T;
    const float sm = p.scale * 1.44269504f;
    constexpr int KPW = kMaxRowsPerWarp;   // keys per warp (block_size <= 128)

    float kr[KPW][4], vr[KPW][4], dka[KPW][4], dva[KPW][4];
#pragma unroll
    for (int i = 0; i < KPW; ++i) {
        const int key = warp + kPisaWarps * i;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            kr[i][c] = (key < nkeys && col < K) ? to_f<T>(k[(base_row + bos + key) * K + col]) : 0.f;
            vr[i][c] = (key < nkeys && col < V) ? to_f<T>(v[(base_row + bos + key) * V + col]) : 0.f;
            dka[i][c] = 0.f;
            dva[i][c] = 0.f;
        }
    }
    const int nkw = (nkeys - warp + kPisaWarps - 1) / kPisaWarps;   // keys this warp owns (may be <= 0)

    for (int i_blk = 0; i_blk < p.nt; ++i_blk) {
        const int32_t* idx = indices + ((size_t)bh * p.nt + i_blk) * p.ns;
        bool hit = false;
        for (int n = 0; n < p.ns; ++n) hit |= (idx[n] == c_blk);
        if (!hit) continue;                                        // uniform over the CTA
        const int t0 = i_blk * p.bs;
        const int nrows = min(p.bs, p.T - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nrows * K; i += kPisaThreads) qs[i] = to_f<T>(q[(base_row + t0) * K + i]);
        for (int i = threadIdx.x; i < nrows * V; i += kPisaThreads) dos[i] = to_f<T>(d_o[(base_row + t0) * V + i]);
        for (int r = threadIdx.x; r < nrows; r += kPisaThreads) {
            const float4 st = *reinterpret_cast<const float4*>(row_stats + (base_row + t0 + r) * 4);
            rst[r * 4 + 0] = st.x;
            rst[r * 4 + 1] = 1.f / st.y;
            rst[r * 4 + 2] = drow[base_row + t0 + r];
        }
        __syncthreads();
        for (int r = 0; r < nrows; ++r) {
            float qv[4], dv_[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = lane + 32 * c;
                qv[c] = col < K ? qs[r * K + col] : 0.f;
                dv_[c] = col < V ? dos[r * V + col] : 0.f;
            }
            const float m = rst[r * 4], rD = rst[r * 4 + 1], dDr = rst[r * 4 + 2];
#pragma unroll
            for (int i = 0; i < KPW; ++i) {
                if (i >= nkw) break;
                float a = 0.f, b = 0.f;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    a = fmaf(qv[c], kr[i][c], a);
                    b = fmaf(dv_[c], vr[i][c], b);
                }
                a = wsum(a);
                b = wsum(b);
                const float pj = exp2f(a * sm - m);
                const float ds = pj * (b * rD + dDr) * p.scale;
                const float pd = pj * rD;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    dka[i][c] = fmaf(ds, qv[c], dka[i][c]);
                    dva[i][c] = fmaf(pd, dv_[c], dva[i][c]);
                }
            }
        }
    }
    // ---- statistics terms: dkc / len, dvc, and the first-order state ----
    __syncthreads();
    const float* dhb = dh + (size_t)bh * K * V;
    for (int i = threadIdx.x; i < K * V; i += kPisaThreads) {
        const int d = i / V, c = i - d * V;
        dhs[d * VP + c] = dhb[i];
    }
    for (int i = threadIdx.x; i < nkeys * K; i += kPisaThreads) qs[i] = to_f<T>(k[(base_row + bos) * K + i]);
    for (int i = threadIdx.x; i < nkeys * V; i += kPisaThreads) dos[i] = to_f<T>(v[(base_row + bos) * V + i]);
    __syncthreads();
    const float inv_len = 1.f / (float)nkeys;
    const float* kcb = kc + ((size_t)bh * p.nt + c_blk) * K;
    const float* vcb = vc + ((size_t)bh * p.nt + c_blk) * V;
    const float* dkcb = dkc + ((size_t)bh * p.nt + c_blk) * K;
    const float* dvcb = dvc + ((size_t)bh * p.nt + c_blk) * V;
#pragma unroll
    for (int i = 0; i < KPW; ++i) {
        const int key = warp + kPisaWarps * i;
        if (key >= nkeys) break;
        const size_t row = base_row + bos + key;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int col = lane + 32 * c;
            if (col < K) {
                float a = 0.f;   // dh (v_t - mean v)
                for (int vv = 0; vv < V; ++vv) a = fmaf(dhs[col * VP + vv], dos[key * V + vv] - vcb[vv] * inv_len, a);
                dk[row * K + col] = from_f<T>(dka[i][c] + dkcb[col] * inv_len + a);
            }
            if (col < V) {
                float a = 0.f;   // dh^T (k_t - kc)
                for (int d = 0; d < K; ++d) a = fmaf(dhs[d * VP + col], qs[key * K + d] - kcb[d], a);
                dv[row * V + col] = from_f<T>(dva[i][c] + dvcb[col] + a);
            }
        }
    }
}

size_t bwd_q_smem_bytes(const PisaParams& p) {
    const int rows_buf = p.bs > kChunkRows ? p.bs : kChunkRows;
    return sizeof(float) * ((size_t)p.bs * p.dk + 2 * (size_t)p.bs * p.dv + (size_t)rows_buf * (p.dk + 1 + p.dv + 1) +
                            2 * (size_t)p.bs * kChunkRows) + (size_t)p.nt + 16;
}
size_t bwd_kv_smem_bytes(const PisaParams& p) {
    return sizeof(float) * ((size_t)p.bs * p.dk + (size_t)p.bs * p.dv + (size_t)p.bs * 4 + (size_t)p.dk * (p.dv + 1));
}

}  // namespace
}  // namespace fbla

namespace fbla {
namespace {

bool pisa_mma_shape(const PisaArgs& a) {
    return a.dtype != FBLA_F32 && a.kp.bs == 64 && a.kp.dk == a.kp.dv && (a.kp.dk == 64 || a.kp.dk == 128) &&
           !g_pisa_force_generic;
}

size_t round64(size_t n) { return (n + 63) / 64 * 64; }

// Scratch layout (fp32 elements, every part starting on a 256-byte boundary):
//   dkc [BH,NT,dk] | dvc [BH,NT,dv] | dh [BH,dk,dv] | drow [BH,T]
//   tensor-core path only: | dr [BH,T,dv] 16-bit | workspace of the state pass that forms dh
struct BwdScratch {
    size_t dkc, dvc, dh, drow, dr, ws, c16, dh16, total;
    int64_t ws_bytes;
    fbla_problem state_problem;
};

BwdScratch bwd_scratch(const PisaArgs& a) {
    const PisaParams& kp = a.kp;
    BwdScratch s{};
    s.dkc = 0;
    s.dvc = s.dkc + round64((size_t)a.bh * kp.nt * kp.dk);
    s.dh = s.dvc + round64((size_t)a.bh * kp.nt * kp.dv);
    s.drow = s.dh + round64((size_t)a.bh * kp.dk * kp.dv);
    s.dr = s.drow + round64((size_t)a.bh * kp.T);
    s.ws = s.dr;
    s.total = s.dr;
    s.ws_bytes = 0;
    if (pisa_mma_shape(a)) {
        fbla_problem& sp = s.state_problem;
        sp = fbla_problem{};
        sp.dtype = a.dtype;
        sp.batch = a.bh / kp.heads;
        sp.heads = kp.heads;
        sp.dk = kp.dk;
        sp.dv = kp.dv;
        sp.seq_len = kp.T;
        sp.scale = 1.f;
        sp.normalize = 0;
        s.ws_bytes = fbla_workspace_bytes(&sp);
        if (s.ws_bytes < 0) s.ws_bytes = 0;
        s.ws = s.dr + round64(((size_t)a.bh * kp.T * kp.dv + 1) / 2);
        s.c16 = s.ws + round64(((size_t)s.ws_bytes + 3) / 4);      // 16-bit copies of kc, vc, h for the tcgen05 kernel
        s.dh16 = s.c16 + round64(((size_t)pisa_tc_scratch_bytes(a.bh, kp.dk, kp.nt) + 3) / 4);   // dh as the key-side kernel reads it
        s.total = s.dh16 + round64(((size_t)a.bh * kp.dk * kp.dv + 1) / 2);
    }
    return s;
}

}  // namespace
}  // namespace fbla

extern "C" int64_t fbla_pisa_bwd_scratch_floats(const fbla_pisa_problem* p) {
    fbla::PisaArgs a;
    if (fbla::resolve_pisa(p, &a)) return -1;
    return (int64_t)fbla::bwd_scratch(a).total;
}

extern "C" int fbla_pisa_bwd(const fbla_pisa_problem* p, const void* q, const void* k, const void* v, const void* o,
                             const void* d_o, const float* kc, const float* vc, const float* h, const int32_t* indices,
                             const float* row_stats, void* dq, void* dk, void* dv, float* scratch,
                             size_t scratch_floats, fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!q || !k || !v || !o || !d_o || !kc || !vc || !h || !indices || !row_stats || !dq || !dk || !dv || !scratch)
        return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    const fbla::PisaParams& kp = a.kp;
    const fbla::BwdScratch lay = fbla::bwd_scratch(a);
    if (scratch_floats < lay.total)
        return fbla::api_fail(FBLA_ERR_WORKSPACE, "scratch of %lld floats needed, %lld given", (long long)lay.total,
                              (long long)scratch_floats);
    float* dkc = scratch + lay.dkc;
    float* dvc = scratch + lay.dvc;
    float* dh = scratch + lay.dh;
    float* drow = scratch + lay.drow;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(kp.nt, a.bh);
    const uintptr_t all_ptrs = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                               reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(d_o) | reinterpret_cast<uintptr_t>(kc) |
                               reinterpret_cast<uintptr_t>(vc) | reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(dq) |
                               reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv) |
                               reinterpret_cast<uintptr_t>(scratch) | reinterpret_cast<uintptr_t>(row_stats);
    if (fbla::pisa_mma_shape(a) && (all_ptrs & 15u) == 0) {
        // dh comes from the state pass, which overwrites it: only dkc, dvc are accumulated into
        cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(float) * lay.dh, st);
        if (e != cudaSuccess) return fbla::api_fail(FBLA_ERR_CUDA, "memset: %s", cudaGetErrorString(e));
        void* dr = scratch + lay.dr;
        void* ws = scratch + lay.ws;
        fbla::pisa_mma::Params mp{kp.heads, kp.ns, kp.nt, kp.T, kp.scale};
        const bool bf = a.dtype == FBLA_BF16;
        auto run_q = [&](auto kern, size_t smem) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess)
                kern<<<grid, fbla::pisa_mma::kThreads, smem, st>>>(mp, q, k, v, o, d_o, kc, vc, h, indices, row_stats, dq,
                                                                  dr, dkc, dvc, drow);
        };
        auto run_kv = [&](auto kern, size_t smem) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess)
                kern<<<grid, fbla::pisa_mma::kThreads, smem, st>>>(mp, q, k, v, d_o, kc, vc, indices, row_stats, drow, dkc,
                                                                  dvc, dh, dk, dv);
        };
        static const bool tc_off = [] {
            const char* v = getenv("FBLA_PISA_TC");
            return v != nullptr && v[0] == '0';
        }();
        if (!tc_off && kp.scale > 0.f && fbla::pisa_tc_supported(a.dtype, kp.dk, kp.dv, kp.bs, kp.nt, kp.ns)) {
            // tcgen05 kernel; it reads the statistics and h as 16-bit copies
            if (const int site = fbla::tc_device_status())
                return fbla::api_fail(FBLA_ERR_DEVICE, "a kernel gave up a bounded wait (site %d); results are invalid", site);
            const int64_t n_stats = (int64_t)a.bh * kp.nt * kp.dk, n_h = (int64_t)a.bh * kp.dk * kp.dk;
            uint16_t* c16 = reinterpret_cast<uint16_t*>(scratch + lay.c16);
            fbla::pisa_tc_cast16(a.dtype, kc, vc, h, n_stats, n_h, c16, st);
            e = fbla::pisa_tc_bwd_q(a.dtype, a.bh, kp.dk, kp.nt, kp.ns, kp.T, kp.scale, q, k, v, o, d_o, c16, c16 + n_stats,
                                    c16 + 2 * n_stats, indices, row_stats, dq, dr, dkc, dvc, drow, st);
            fbla::note_launches(1);
        } else if (kp.dk == 64) {
            const size_t smem = fbla::pisa_mma::bwd_q_smem_bytes<64>(kp.nt);
            if (bf) run_q(fbla::pisa_mma::pisa_bwd_q_mma_kernel<64, true>, smem);
            else run_q(fbla::pisa_mma::pisa_bwd_q_mma_kernel<64, false>, smem);
        } else {
            const size_t smem = fbla::pisa_mma::bwd_q_smem_bytes<128>(kp.nt);
            if (bf) run_q(fbla::pisa_mma::pisa_bwd_q_mma_kernel<128, true>, smem);
            else run_q(fbla::pisa_mma::pisa_bwd_q_mma_kernel<128, false>, smem);
        }
        fbla::note_launches(1);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e != cudaSuccess) return fbla::api_fail(FBLA_ERR_CUDA, "backward query kernel: %s", cudaGetErrorString(e));
        // dh = q^T dr
        if (int rc = fbla_simple_la_fwd_state(&lay.state_problem, q, dr, dh, ws, (size_t)lay.ws_bytes, stream)) return rc;
        static const bool tc_kv_off = [] {
            const char* v = getenv("FBLA_PISA_TC_KV");
            return v != nullptr && v[0] == '0';
        }();
        if (!tc_off && !tc_kv_off && kp.scale > 0.f && fbla::pisa_tc_supported(a.dtype, kp.dk, kp.dv, kp.bs, kp.nt, kp.ns) &&
            fbla::pisa_tc_bwd_kv_fits(kp.dk, kp.nt)) {
            e = fbla::pisa_tc_bwd_kv(a.dtype, a.bh, kp.dk, kp.nt, kp.ns, kp.T, kp.scale, q, k, v, d_o, kc, vc, indices, row_stats,
                                     drow, dkc, dvc, dh, scratch + lay.dh16, dk, dv, st);
            fbla::note_launches(1);
        } else if (kp.dk == 64) {
            const size_t smem = fbla::pisa_mma::bwd_kv_smem_bytes<64>(kp.nt);
            if (bf) run_kv(fbla::pisa_mma::pisa_bwd_kv_mma_kernel<64, true>, smem);
            else run_kv(fbla::pisa_mma::pisa_bwd_kv_mma_kernel<64, false>, smem);
        } else {
            const size_t smem = fbla::pisa_mma::bwd_kv_smem_bytes<128>(kp.nt);
            if (bf) run_kv(fbla::pisa_mma::pisa_bwd_kv_mma_kernel<128, true>, smem);
            else run_kv(fbla::pisa_mma::pisa_bwd_kv_mma_kernel<128, false>, smem);
        }
        fbla::note_launches(1);
        if (e == cudaSuccess) e = cudaGetLastError();
        return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "backward key kernel: %s", cudaGetErrorString(e));
    }
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(float) * lay.drow, st);
    if (e != cudaSuccess) return fbla::api_fail(FBLA_ERR_CUDA, "memset: %s", cudaGetErrorString(e));
    const size_t smem1 = fbla::bwd_q_smem_bytes(kp), smem2 = fbla::bwd_kv_smem_bytes(kp);
    if (smem1 > 227 * 1024 || smem2 > 227 * 1024)
        return fbla::api_fail(FBLA_ERR_UNSUPPORTED, "block_size, dk, dv too large for the backward kernels");
    PISA_BY_DTYPE(a.dtype, {
        auto k1 = fbla::pisa_bwd_q_kernel<T>;
        auto k2 = fbla::pisa_bwd_kv_kernel<T>;
        if (smem1 > 48 * 1024) e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        if (e == cudaSuccess && smem2 > 48 * 1024)
            e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        if (e == cudaSuccess) {
            k1<<<grid, fbla::kPisaThreads, smem1, st>>>(kp, (const T*)q, (const T*)k, (const T*)v, (const T*)o,
                                                        (const T*)d_o, kc, vc, h, indices, row_stats, (T*)dq, dkc, dvc,
                                                        dh, drow);
            k2<<<grid, fbla::kPisaThreads, smem2, st>>>(kp, (const T*)q, (const T*)k, (const T*)v, (const T*)d_o, kc, vc,
                                                        indices, row_stats, drow, dkc, dvc, dh, (T*)dk, (T*)dv);
        }
    });
    fbla::note_launches(2);
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "backward kernels: %s", cudaGetErrorString(e));
}
