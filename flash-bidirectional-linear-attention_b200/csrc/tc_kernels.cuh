// Launchers of the tensor-core path (tcgen05 MMA with TMEM accumulators, operands
// staged by TMA): 16-bit inputs with dk, dv in {64, 128}.
#pragma once

#include "fbla_common.cuh"

namespace fbla {

bool tc_supported(const KParams& p, int dtype);
// The decoupled operator has tensor-core kernels at dk = dv = 64 only.
bool tc_supported_decoupled(const KParams& p);
// Status word written by a kernel whose bounded wait gave up (0 = none did).
int tc_device_status();
// Device-visible address of that word (NULL if the pinned allocation failed).
int* tc_status_word();
int64_t tc_workspace_bytes(const KParams& p);
// Sequence-sharded calls: floats of one receive buffer (fbla_peer_group.recv) for `world` ranks.
int64_t tc_peer_recv_floats(const KParams& p, int world);
// Limit of a kernel's wait for a peer GPU, nanoseconds (FBLA_PEER_WAIT_MS in the environment).
unsigned long long tc_peer_wait_ns();
// Measurement aid: device buffer of 256 x 16 64-bit words that receives the timestamps of the
// sequence-sharded exchanges (NULL switches it off).
void tc_set_peer_trace(unsigned long long* dev);
// Clears the status word after a reported failure.
void tc_clear_device_status();
cudaError_t tc_fwd_state(const KParams& p, int dtype, const void* k, const void* k_rope, const void* v,
                         float* state, void* ws, cudaStream_t st);
// Same pass with the kernels' status word supplied by the caller (device-accessible memory).
cudaError_t tc_fwd_state_status(const KParams& p, int dtype, const void* k, const void* k_rope, const void* v,
                                float* state, void* ws, int* status, cudaStream_t st);
cudaError_t tc_fwd_out(const KParams& p, int dtype, const void* q, const void* q_rope, const float* state,
                       void* o, cudaStream_t st);
cudaError_t tc_bwd_state(const KParams& p, int dtype, const void* q, const void* q_rope, const void* d_o,
                         const float* state, void* dq, void* dq_rope, float* dstate, void* ws,
                         cudaStream_t st);
cudaError_t tc_bwd_in(const KParams& p, int dtype, const void* k_rope, const void* v, const float* dstate,
                      void* dk, void* dk_rope, void* dv, cudaStream_t st);

}  // namespace fbla
