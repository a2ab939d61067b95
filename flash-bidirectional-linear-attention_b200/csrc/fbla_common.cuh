// Shared declarations of the flash_bla_sm100 library: the resolved kernel
// parameters, the token-layout helper and the launcher prototypes that the C ABI
// (fbla_api.cu) dispatches to.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flash_bla_sm100.h"

namespace fbla {

// Everything a kernel needs to locate the tokens of one unit.  A unit is one
// (batch, head) pair in the fixed-length layout, one (sequence, head) pair in the
// packed layout.
// A sequence-sharded exchange: the peers' buffers (see fbla_peer_group in the public header), resolved.
struct PeerArgs {
    int world, rank;
    unsigned int epoch;
    void* parts[8];
    void* full[8];
    void* flags[8];
};

struct KParams {
    int units;            // B*H or num_seqs*H
    int heads;
    int dk, dv;           // feature dims the kernels compute with
    int mem_dk, mem_dv;   // feature dims of the tensors in memory (smaller than dk, dv only on the narrow route of
                          // the tensor-core kernels, whose TMA boxes zero-fill / clip the missing features)
    int64_t seq_len;      // fixed length: T; packed: total tokens
    int max_len;          // longest unit (fixed: T; packed: caller's max_seqlen)
    const int32_t* cu;    // packed layout only
    float scale;
    int scale_per_seq;
    float inv_norm;       // 1 / norm_len when given, else 0 (= use the unit's own length)
    float eps;
    int normalize;
    int state_stride;     // floats per unit in state / dstate
    int unreduced;        // tensor-core kernels, fixed length: 1 = the state stays in its per-segment pieces
                          // (the consuming pass adds them while staging; no reduce kernel); 2 = only the
                          // OUTPUT of a reducing pass stays in pieces, the state it reads is a reduced one
};

struct UnitGeom {
    int64_t row0;   // row of token 0 in the (rows, D) view of the tensor
    int64_t rs;     // rows between consecutive tokens
    int len;        // tokens in this unit
    float scale;    // value scale of this unit
    float inv_norm; // 1 / length the key sum is divided by
};

__device__ __forceinline__ UnitGeom unit_geom(const KParams& p, int u) {
    UnitGeom g;
    if (p.cu == nullptr) {
        g.row0 = (int64_t)u * p.seq_len;
        g.rs = 1;
        g.len = (int)p.seq_len;
        g.scale = p.scale;
        g.inv_norm = p.inv_norm > 0.f ? p.inv_norm : 1.f / (float)p.seq_len;
    } else {
        const int s = u / p.heads, h = u - s * p.heads;
        const int bos = p.cu[s], eos = p.cu[s + 1];
        g.len = eos - bos;
        g.row0 = (int64_t)bos * p.heads + h;
        g.rs = p.heads;
        const float inv_len = g.len > 0 ? 1.f / (float)g.len : 0.f;
        g.scale = p.scale_per_seq ? inv_len : p.scale;
        g.inv_norm = p.inv_norm > 0.f ? p.inv_norm : inv_len;
    }
    return g;
}

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// Used by entry points that live outside fbla_api.cu: record an error text for the calling thread
// (returns `code`), and validate a fixed-length linear_attention problem.
int api_fail(int code, const char* fmt, ...);
int api_resolve_linear(const fbla_problem* p, KParams* kp);

// Kernel-launch counter behind fbla_launch_count(): every launcher reports what it enqueued.
void note_launches(int n);

// ---- launchers (each returns a cudaError_t from the launch) ----------------------------
// CUDA-core path (simt_kernels.cu): any dk, dv in [1, 128], any dtype.
int64_t simt_workspace_bytes(const KParams& p);
cudaError_t simt_fwd_state(const KParams& p, int dtype, const void* k, const void* k_rope, const void* v,
                           float* state, void* ws, cudaStream_t st);
cudaError_t simt_fwd_out(const KParams& p, int dtype, const void* q, const void* q_rope, const float* state,
                         void* o, cudaStream_t st);
cudaError_t simt_bwd_state(const KParams& p, int dtype, const void* q, const void* q_rope, const void* d_o,
                           const float* state, void* dq, void* dq_rope, float* dstate, void* ws,
                           cudaStream_t st);
cudaError_t simt_bwd_in(const KParams& p, int dtype, const void* k_rope, const void* v, const float* dstate,
                        void* dk, void* dk_rope, void* dv, cudaStream_t st);

}  // namespace fbla
