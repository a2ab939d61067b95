// CUDA-core (fp32 FMA) kernels for the four streaming passes.  They serve every
// shape the tensor-core kernels do not: fp32 inputs (which need full fp32 products
// to stay within 1e-5 of the reference's torch path), feature dims that are not a
// multiple of 64, and any dk, dv in [1, 128].
//
// Work decomposition (all kernels): blockIdx.y = unit, blockIdx.x = slice of the
// unit's tokens.  The two reducing passes write one fp32 partial per (unit, slice)
// into the workspace and a second small kernel adds the slices in a fixed order, so
// results are bit-reproducible from run to run.
#include "fbla_common.cuh"

namespace fbla {
namespace {

constexpr int kThreads = 256;
constexpr int kTT = 16;           // tokens staged per step in the reducing passes
constexpr int kReduceChunk = 512; // most tokens per slice in the reducing passes (fewer when there are few units)
constexpr int kOutTokens = 128;   // tokens per block in the streaming passes

// Tokens per slice: 512, halved (down to 64) while the launch would have fewer than ~2 CTAs per SM of a
// large GPU.  A function of the problem only, so the workspace size and the order of the sums are fixed.
__host__ __device__ inline int chunk_of(const KParams& p) {
    int chunk = kReduceChunk;
    while (chunk > 64 && (long long)p.units * ((p.max_len + chunk - 1) / chunk) < 296) chunk >>= 1;
    return chunk;
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Stage `nt` (<= kTT) token rows of width D into shared memory as fp32, zero-filling
// the rows past nt.
template <typename T>
__device__ __forceinline__ void stage_rows(float* dst, const T* __restrict__ src, const UnitGeom& g, int D,
                                           int t0, int nt) {
    for (int i = threadIdx.x; i < kTT * D; i += kThreads) {
        const int t = i / D, d = i - t * D;
        float x = 0.f;
        if (t < nt) x = to_f<T>(src[(g.row0 + (int64_t)(t0 + t) * g.rs) * D + d]);
        dst[i] = x;
    }
}

// acc[i][j] += sum_t a[t][ty+16i] * b[t][tx+16j] over the staged tile.
template <int R>
__device__ __forceinline__ void outer_accumulate(float (&acc)[R][R], const float* a_s, const float* b_s,
                                                 int DK, int DV, int ty, int tx) {
#pragma unroll 4
    for (int t = 0; t < kTT; ++t) {
        float a[R], b[R];
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int r = ty + 16 * i;
            a[i] = r < DK ? a_s[t * DK + r] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int c = tx + 16 * j;
            b[j] = c < DV ? b_s[t * DV + c] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < R; ++i)
#pragma unroll
            for (int j = 0; j < R; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
}

template <int R>
__device__ __forceinline__ void store_partial(float* out, const float (&acc)[R][R], int DK, int DV, int ty,
                                              int tx) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = ty + 16 * i;
        if (r >= DK) continue;
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int c = tx + 16 * j;
            if (c < DV) out[r * DV + c] = acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------------------
// forward pass 1: partial [ S = sum_t kr_t (x) v_t | sum_t k_t ] over one slice of a unit
// ---------------------------------------------------------------------------------------
template <typename T, int R>
__global__ void __launch_bounds__(kThreads)
simt_fwd_state_kernel(KParams p, const T* __restrict__ k, const T* __restrict__ kr, const T* __restrict__ v,
                      float* __restrict__ part, int nslices) {
    extern __shared__ float smem[];
    const int DK = p.dk, DV = p.dv;
    float* a_s = smem;                 // kr tile
    float* b_s = a_s + kTT * DK;       // v tile
    float* c_s = b_s + kTT * DV;       // k tile (only when k != kr)
    const bool split = (k != kr) && p.normalize;

    const int u = blockIdx.y, sl = blockIdx.x;
    const UnitGeom g = unit_geom(p, u);
    const int chunk = chunk_of(p);
    const int t_begin = sl * chunk;
    const int t_end = min(g.len, t_begin + chunk);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;

    float acc[R][R];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) acc[i][j] = 0.f;
    float ks = 0.f;

    for (int t0 = t_begin; t0 < t_end; t0 += kTT) {
        const int nt = min(kTT, t_end - t0);
        stage_rows<T>(a_s, kr, g, DK, t0, nt);
        stage_rows<T>(b_s, v, g, DV, t0, nt);
        if (split) stage_rows<T>(c_s, k, g, DK, t0, nt);
        __syncthreads();
        outer_accumulate<R>(acc, a_s, b_s, DK, DV, ty, tx);
        if (p.normalize && threadIdx.x < DK) {
            const float* src = split ? c_s : a_s;
#pragma unroll
            for (int t = 0; t < kTT; ++t) ks += src[t * DK + threadIdx.x];
        }
        __syncthreads();
    }
    float* out = part + ((int64_t)u * nslices + sl) * p.state_stride;
    store_partial<R>(out, acc, DK, DV, ty, tx);
    if (p.normalize && threadIdx.x < DK) out[DK * DV + threadIdx.x] = ks;
}

// Adds the slices of every unit in slice order.
__global__ void __launch_bounds__(kThreads)
reduce_slices_kernel(const float* __restrict__ part, float* __restrict__ state, int nslices, int stride,
                     int64_t total) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= total) return;
    const int64_t u = i / stride;
    const int e = (int)(i - u * stride);
    const float* src = part + u * nslices * (int64_t)stride + e;
    float s = 0.f;
    for (int j = 0; j < nslices; ++j) s += src[(int64_t)j * stride];
    state[i] = s;
}

// ---------------------------------------------------------------------------------------
// forward pass 2: o_t = scale * (qr_t S) / (q_t . ksum * inv_norm + eps)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
simt_fwd_out_kernel(KParams p, const T* __restrict__ q, const T* __restrict__ qr,
                    const float* __restrict__ state, T* __restrict__ o) {
    extern __shared__ float smem[];
    const int DK = p.dk, DV = p.dv;
    float* S = smem;                    // [DK][DV], already multiplied by the scale
    float* km = S + DK * DV;            // [DK]
    float* qbuf = km + DK;              // [8 warps][2][DK]
    const int u = blockIdx.y;
    const UnitGeom g = unit_geom(p, u);
    const int t_begin = blockIdx.x * kOutTokens;
    if (t_begin >= g.len) return;
    const int t_end = min(g.len, t_begin + kOutTokens);

    const float* st = state + (int64_t)u * p.state_stride;
    for (int i = threadIdx.x; i < DK * DV; i += kThreads) S[i] = st[i] * g.scale;
    if (p.normalize)
        for (int i = threadIdx.x; i < DK; i += kThreads) km[i] = st[DK * DV + i] * g.inv_norm;
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qn = qbuf + warp * 2 * DK;   // numerator query (rotary when decoupled)
    float* qd = qn + DK;                // normaliser query
    for (int t = t_begin + warp; t < t_end; t += kThreads / 32) {
        const int64_t row = g.row0 + (int64_t)t * g.rs;
        for (int d = lane; d < DK; d += 32) {
            const float x = to_f<T>(q[row * DK + d]);
            qd[d] = x;
            qn[d] = (qr == q) ? x : to_f<T>(qr[row * DK + d]);
        }
        __syncwarp();
        float z = 1.f;
        if (p.normalize) {
            float zp = 0.f;
            for (int d = lane; d < DK; d += 32) zp = fmaf(qd[d], km[d], zp);
            z = warp_sum(zp) + p.eps;
        }
        for (int c = lane; c < DV; c += 32) {
            float a = 0.f;
            for (int d = 0; d < DK; ++d) a = fmaf(qn[d], S[d * DV + c], a);
            o[row * DV + c] = from_f<T>(a / z);
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------
// backward pass 1: per token  t = dO S^T,  z = q.km + eps,  dz = -(qr.t)/z^2,
//   dqr = t/z, dq = dz km (summed into one dq when the op is not decoupled), and the
//   partial [ dS = sum (qr/z) (x) dO | sum dz q ] over one slice of a unit.
// ---------------------------------------------------------------------------------------
template <typename T, int R>
__global__ void __launch_bounds__(kThreads)
simt_bwd_state_kernel(KParams p, const T* __restrict__ q, const T* __restrict__ qr, const T* __restrict__ d_o,
                      const float* __restrict__ state, T* __restrict__ dq, T* __restrict__ dqr,
                      float* __restrict__ part, int nslices) {
    extern __shared__ float smem[];
    const int DK = p.dk, DV = p.dv, DVP = DV + 1;
    float* S = smem;                    // [DK][DV+1] scaled state, padded rows
    float* km = S + DK * DVP;           // [DK]
    float* a_s = km + DK;               // [kTT][DK]  qr tile, becomes qr/z
    float* c_s = a_s + kTT * DK;        // [kTT][DK]  q tile, becomes dz*q
    float* b_s = c_s + kTT * DK;        // [kTT][DV]  dO tile

    const int u = blockIdx.y, sl = blockIdx.x;
    const UnitGeom g = unit_geom(p, u);
    const int chunk = chunk_of(p);
    const int t_begin = sl * chunk;
    const int t_end = min(g.len, t_begin + chunk);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool decoupled = (dqr != nullptr);

    const float* st = state + (int64_t)u * p.state_stride;
    for (int i = threadIdx.x; i < DK * DV; i += kThreads) {
        const int r = i / DV, c = i - r * DV;
        S[r * DVP + c] = st[i] * g.scale;
    }
    for (int i = threadIdx.x; i < DK; i += kThreads)
        km[i] = p.normalize ? st[DK * DV + i] * g.inv_norm : 0.f;

    float acc[R][R];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) acc[i][j] = 0.f;
    float dkm = 0.f;
    __syncthreads();

    for (int t0 = t_begin; t0 < t_end; t0 += kTT) {
        const int nt = min(kTT, t_end - t0);
        stage_rows<T>(a_s, qr, g, DK, t0, nt);
        if (qr != q) stage_rows<T>(c_s, q, g, DK, t0, nt);
        stage_rows<T>(b_s, d_o, g, DV, t0, nt);
        __syncthreads();
        if (qr == q)
            for (int i = threadIdx.x; i < kTT * DK; i += kThreads) c_s[i] = a_s[i];
        __syncthreads();
        // per-token part: one warp per token
        for (int t = warp; t < kTT; t += kThreads / 32) {
            float* qn = a_s + t * DK;
            float* qd = c_s + t * DK;
            const float* g_o = b_s + t * DV;
            float tk[4];
            float zp = 0.f, wp = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int d = lane + 32 * j;
                tk[j] = 0.f;
                if (d < DK) {
                    float a = 0.f;
                    const float* srow = S + d * DVP;
                    for (int c = 0; c < DV; ++c) a = fmaf(srow[c], g_o[c], a);
                    tk[j] = a;
                    zp = fmaf(qd[d], km[d], zp);
                    wp = fmaf(qn[d], a, wp);
                }
            }
            float z = 1.f, dz = 0.f;
            if (p.normalize) {
                z = warp_sum(zp) + p.eps;
                dz = -warp_sum(wp) / (z * z);
            }
            const float rz = 1.f / z;
            const int64_t row = g.row0 + (int64_t)(t0 + t) * g.rs;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int d = lane + 32 * j;
                if (d < DK) {
                    const float g_qr = tk[j] * rz;
                    const float g_q = dz * km[d];
                    if (t < nt) {
                        if (decoupled) {
                            dqr[row * DK + d] = from_f<T>(g_qr);
                            dq[row * DK + d] = from_f<T>(g_q);
                        } else {
                            dq[row * DK + d] = from_f<T>(g_qr + g_q);
                        }
                    }
                    const float qn_d = qn[d], qd_d = qd[d];
                    qn[d] = qn_d * rz;
                    qd[d] = dz * qd_d;
                }
            }
        }
        __syncthreads();
        outer_accumulate<R>(acc, a_s, b_s, DK, DV, ty, tx);
        if (p.normalize && threadIdx.x < DK) {
#pragma unroll
            for (int t = 0; t < kTT; ++t) dkm += c_s[t * DK + threadIdx.x];
        }
        __syncthreads();
    }
    float* out = part + ((int64_t)u * nslices + sl) * p.state_stride;
    store_partial<R>(out, acc, DK, DV, ty, tx);
    if (p.normalize && threadIdx.x < DK) out[DK * DV + threadIdx.x] = dkm;
}

// ---------------------------------------------------------------------------------------
// backward pass 2: dkr_t = scale * dS v_t (+ dkm*inv_norm), dv_t = scale * dS^T kr_t,
//   and dk_t = dkm*inv_norm on its own when the op is decoupled.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
simt_bwd_in_kernel(KParams p, const T* __restrict__ kr, const T* __restrict__ v,
                   const float* __restrict__ dstate, T* __restrict__ dk, T* __restrict__ dkr,
                   T* __restrict__ dv) {
    extern __shared__ float smem[];
    const int DK = p.dk, DV = p.dv, DVP = DV + 1;
    float* dS = smem;                   // [DK][DV+1], multiplied by the scale
    float* dkm = dS + DK * DVP;         // [DK], multiplied by inv_norm
    float* buf = dkm + DK;              // [8 warps][DK + DV]
    const int u = blockIdx.y;
    const UnitGeom g = unit_geom(p, u);
    const int t_begin = blockIdx.x * kOutTokens;
    if (t_begin >= g.len) return;
    const int t_end = min(g.len, t_begin + kOutTokens);
    const bool decoupled = (dkr != nullptr);

    const float* st = dstate + (int64_t)u * p.state_stride;
    for (int i = threadIdx.x; i < DK * DV; i += kThreads) {
        const int r = i / DV, c = i - r * DV;
        dS[r * DVP + c] = st[i] * g.scale;
    }
    for (int i = threadIdx.x; i < DK; i += kThreads)
        dkm[i] = p.normalize ? st[DK * DV + i] * g.inv_norm : 0.f;
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* kb = buf + warp * (DK + DV);
    float* vb = kb + DK;
    for (int t = t_begin + warp; t < t_end; t += kThreads / 32) {
        const int64_t row = g.row0 + (int64_t)t * g.rs;
        for (int d = lane; d < DK; d += 32) kb[d] = to_f<T>(kr[row * DK + d]);
        for (int c = lane; c < DV; c += 32) vb[c] = to_f<T>(v[row * DV + c]);
        __syncwarp();
        for (int d = lane; d < DK; d += 32) {
            float a = 0.f;
            const float* srow = dS + d * DVP;
            for (int c = 0; c < DV; ++c) a = fmaf(srow[c], vb[c], a);
            if (decoupled) {
                dkr[row * DK + d] = from_f<T>(a);
                dk[row * DK + d] = from_f<T>(dkm[d]);
            } else {
                dk[row * DK + d] = from_f<T>(a + dkm[d]);
            }
        }
        for (int c = lane; c < DV; c += 32) {
            float a = 0.f;
            for (int d = 0; d < DK; ++d) a = fmaf(kb[d], dS[d * DVP + c], a);
            dv[row * DV + c] = from_f<T>(a);
        }
        __syncwarp();
    }
}

inline int slices_of(const KParams& p) {
    const int chunk = chunk_of(p);
    return (p.max_len + chunk - 1) / chunk;
}

template <typename K>
cudaError_t opt_in_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

cudaError_t reduce_slices(const KParams& p, const float* part, float* state, int nslices, cudaStream_t st) {
    const int64_t total = (int64_t)p.units * p.state_stride;
    const int64_t blocks = (total + kThreads - 1) / kThreads;
    reduce_slices_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(part, state, nslices, p.state_stride, total);
    note_launches(1);
    return cudaGetLastError();
}

template <typename T>
cudaError_t fwd_state_t(const KParams& p, const T* k, const T* kr, const T* v, float* state, float* ws,
                        cudaStream_t st) {
    const int ns = slices_of(p);
    float* part = ns == 1 ? state : ws;
    const size_t smem = sizeof(float) * kTT * (2 * p.dk + p.dv);
    dim3 grid(ns, p.units);
    if (p.dk <= 64 && p.dv <= 64)
        simt_fwd_state_kernel<T, 4><<<grid, kThreads, smem, st>>>(p, k, kr, v, part, ns);
    else
        simt_fwd_state_kernel<T, 8><<<grid, kThreads, smem, st>>>(p, k, kr, v, part, ns);
    note_launches(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || ns == 1) return e;
    return reduce_slices(p, part, state, ns, st);
}

template <typename T>
cudaError_t fwd_out_t(const KParams& p, const T* q, const T* qr, const float* state, T* o, cudaStream_t st) {
    const size_t smem = sizeof(float) * (p.dk * p.dv + p.dk + (kThreads / 32) * 2 * p.dk);
    cudaError_t e = opt_in_smem(simt_fwd_out_kernel<T>, smem);
    if (e != cudaSuccess) return e;
    dim3 grid((p.max_len + kOutTokens - 1) / kOutTokens, p.units);
    simt_fwd_out_kernel<T><<<grid, kThreads, smem, st>>>(p, q, qr, state, o);
    note_launches(1);
    return cudaGetLastError();
}

template <typename T>
cudaError_t bwd_state_t(const KParams& p, const T* q, const T* qr, const T* d_o, const float* state, T* dq,
                        T* dqr, float* dstate, float* ws, cudaStream_t st) {
    const int ns = slices_of(p);
    float* part = ns == 1 ? dstate : ws;
    const size_t smem = sizeof(float) * (p.dk * (p.dv + 1) + p.dk + kTT * (2 * p.dk + p.dv));
    dim3 grid(ns, p.units);
    cudaError_t e;
    if (p.dk <= 64 && p.dv <= 64) {
        e = opt_in_smem(simt_bwd_state_kernel<T, 4>, smem);
        if (e != cudaSuccess) return e;
        simt_bwd_state_kernel<T, 4><<<grid, kThreads, smem, st>>>(p, q, qr, d_o, state, dq, dqr, part, ns);
    } else {
        e = opt_in_smem(simt_bwd_state_kernel<T, 8>, smem);
        if (e != cudaSuccess) return e;
        simt_bwd_state_kernel<T, 8><<<grid, kThreads, smem, st>>>(p, q, qr, d_o, state, dq, dqr, part, ns);
    }
    note_launches(1);
    e = cudaGetLastError();
    if (e != cudaSuccess || ns == 1) return e;
    return reduce_slices(p, part, dstate, ns, st);
}

template <typename T>
cudaError_t bwd_in_t(const KParams& p, const T* kr, const T* v, const float* dstate, T* dk, T* dkr, T* dv,
                     cudaStream_t st) {
    const size_t smem = sizeof(float) * (p.dk * (p.dv + 1) + p.dk + (kThreads / 32) * (p.dk + p.dv));
    cudaError_t e = opt_in_smem(simt_bwd_in_kernel<T>, smem);
    if (e != cudaSuccess) return e;
    dim3 grid((p.max_len + kOutTokens - 1) / kOutTokens, p.units);
    simt_bwd_in_kernel<T><<<grid, kThreads, smem, st>>>(p, kr, v, dstate, dk, dkr, dv);
    note_launches(1);
    return cudaGetLastError();
}

}  // namespace

int64_t simt_workspace_bytes(const KParams& p) {
    const int ns = slices_of(p);
    return ns <= 1 ? 0 : (int64_t)p.units * ns * p.state_stride * (int64_t)sizeof(float);
}

#define FBLA_BY_DTYPE(CALL)                                             \
    switch (dtype) {                                                    \
        case FBLA_F32: { using T = float; return CALL; }                \
        case FBLA_BF16: { using T = __nv_bfloat16; return CALL; }       \
        case FBLA_F16: { using T = __half; return CALL; }               \
        default: return cudaErrorInvalidValue;                          \
    }

cudaError_t simt_fwd_state(const KParams& p, int dtype, const void* k, const void* k_rope, const void* v,
                           float* state, void* ws, cudaStream_t st) {
    if (k_rope == nullptr) k_rope = k;
    FBLA_BY_DTYPE(fwd_state_t<T>(p, (const T*)k, (const T*)k_rope, (const T*)v, state, (float*)ws, st));
}

cudaError_t simt_fwd_out(const KParams& p, int dtype, const void* q, const void* q_rope, const float* state,
                         void* o, cudaStream_t st) {
    if (q_rope == nullptr) q_rope = q;
    FBLA_BY_DTYPE(fwd_out_t<T>(p, (const T*)q, (const T*)q_rope, state, (T*)o, st));
}

cudaError_t simt_bwd_state(const KParams& p, int dtype, const void* q, const void* q_rope, const void* d_o,
                           const float* state, void* dq, void* dq_rope, float* dstate, void* ws,
                           cudaStream_t st) {
    if (q_rope == nullptr) q_rope = q;
    FBLA_BY_DTYPE(bwd_state_t<T>(p, (const T*)q, (const T*)q_rope, (const T*)d_o, state, (T*)dq, (T*)dq_rope,
                                 dstate, (float*)ws, st));
}

cudaError_t simt_bwd_in(const KParams& p, int dtype, const void* k_rope, const void* v, const float* dstate,
                        void* dk, void* dk_rope, void* dv, cudaStream_t st) {
    FBLA_BY_DTYPE(bwd_in_t<T>(p, (const T*)k_rope, (const T*)v, dstate, (T*)dk, (T*)dk_rope, (T*)dv, st));
}

}  // namespace fbla
