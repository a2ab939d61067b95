// Launchers of the tensor-core path (tcgen05 MMA with TMEM accumulators, operands
// staged by TMA): 16-bit inputs with dk, dv in {64, 128}.
#pragma once

#include <cuda.h>

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
// TMA map of a (units, rows, D) 16-bit tensor as {D, rows, units}, box = 64 features x box_rows rows,
// 128-byte swizzle; rows past the end read as zero and are dropped on stores.
cudaError_t tc_encode_map_rows(CUtensorMap* m, const void* base, int dtype, int D, int64_t rows, int units, int box_rows);
// How the per-segment pieces of the reducing passes lie in the workspace (fixed length): unit u has
// pieces (u * slots + j), j < n(u), n(u) = last_cta(u) - first_cta(u) + 1 with the two tile counts.
struct PieceLayout {
    int units, slots, tiles_per_unit, tiles_per_cta;
};
PieceLayout tc_piece_layout(const KParams& p);
// The exchange kernel of the sequence-sharded tensor-core passes (peer_exchange.cu): sums the pieces of
// all ranks into `out` ([units][state_stride] floats of ordinary memory).
cudaError_t peer_piece_sum(const PeerArgs& g, const PieceLayout& lay, int state_stride, int two_round, float* out,
                           cudaStream_t st);
// Limit of a kernel's wait for a peer GPU, nanoseconds (FBLA_PEER_WAIT_MS in the environment, 5000).
unsigned long long tc_peer_wait_ns();
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
