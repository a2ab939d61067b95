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
#include "fbla_common.cuh"

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
    for (int t = 0; t < len; ++t) {
        if (d < p.dk) {
            sq += to_f<T>(q[(row0 + t) * p.dk + d]);
            sk += to_f<T>(k[(row0 + t) * p.dk + d]);
        }
        if (d < p.dv) sv += to_f<T>(v[(row0 + t) * p.dv + d]);
    }
    const size_t blk = (size_t)bh * p.nt + c;
    if (d < p.dk) {
        qc[blk * p.dk + d] = sq / (float)len;
        kc[blk * p.dk + d] = sk / (float)len;
    }
    if (d < p.dv) vc[blk * p.dv + d] = sv;
}

// h = K^T V - sum_c kc_c (x) vc_c
__global__ void __launch_bounds__(256)
pisa_first_order_kernel(PisaParams p, const float* __restrict__ kv, const float* __restrict__ kc,
                        const float* __restrict__ vc, float* __restrict__ h) {
    const int bh = blockIdx.y;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= p.dk * p.dv) return;
    const int a = i / p.dv, b = i - a * p.dv;
    const float* kcb = kc + (size_t)bh * p.nt * p.dk;
    const float* vcb = vc + (size_t)bh * p.nt * p.dv;
    float s = 0.f;
    for (int c = 0; c < p.nt; ++c) s = fmaf(kcb[c * p.dk + a], vcb[c * p.dv + b], s);
    h[(size_t)bh * p.dk * p.dv + i] = kv[(size_t)bh * p.dk * p.dv + i] - s;
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
        const int bos = cb * p.bs;
        const int nvalid = max(0, min(p.bs, p.T - bos));
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
            *reinterpret_cast<float4*>(row_stats + row * 4) = make_float4(m[ri], den, g[ri], 0.f);
    }
}

size_t fwd_smem_bytes(const PisaParams& p) {
    const int rows_buf = p.bs > kChunkRows ? p.bs : kChunkRows;
    return sizeof(float) * ((size_t)p.bs * p.dk + (size_t)rows_buf * (p.dk + 1 + p.dv + 1)) + (size_t)p.nt + 16;
}

}  // namespace

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

int fbla_pisa_first_order_state(const fbla_pisa_problem* p, const float* kv, const float* kc, const float* vc,
                                float* h, fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!kv || !kc || !vc || !h) return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    dim3 grid((a.kp.dk * a.kp.dv + 255) / 256, a.bh);
    fbla::pisa_first_order_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a.kp, kv, kc, vc, h);
    fbla::note_launches(1);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "first-order state: %s", cudaGetErrorString(e));
}

int fbla_pisa_fwd(const fbla_pisa_problem* p, const void* q, const void* k, const void* v, const float* kc,
                  const float* vc, const float* h, const int32_t* indices, void* o, float* row_stats,
                  fbla_stream_t stream) {
    fbla::PisaArgs a;
    if (int rc = fbla::resolve_pisa(p, &a)) return rc;
    if (!q || !k || !v || !kc || !vc || !h || !indices || !o)
        return fbla::api_fail(FBLA_ERR_INVALID, "a tensor pointer is NULL");
    const size_t smem = fbla::fwd_smem_bytes(a.kp);
    dim3 grid(a.kp.nt, a.bh);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
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
