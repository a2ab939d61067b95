// Launcher of the tcgen05 forward of the piecewise sparse attention stage (pisa_tc.cu):
// 16-bit inputs, dk = dv in {64, 128}, block size 64, up to 2048 blocks.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "fbla_common.cuh"

namespace fbla {

bool pisa_tc_supported(int dtype, int dk, int dv, int bs, int nt, int ns);
// Bytes of 16-bit scratch (copies of the block statistics and of h), 128-byte aligned.
int64_t pisa_tc_scratch_bytes(int bh, int d, int nt);
cudaError_t pisa_tc_fwd(int dtype, int bh, int d, int nt, int ns, int T, float scale, const void* q, const void* k,
                        const void* v, const float* kc, const float* vc, const float* h, const int32_t* indices, void* o,
                        float* row_stats, void* scratch, cudaStream_t st);

// fp32 -> 16-bit copies [kc | vc | h] (n_stats elements each of kc, vc; n_h of h) into `out`.
void pisa_tc_cast16(int dtype, const float* kc, const float* vc, const float* h, int64_t n_stats, int64_t n_h, void* out,
                    cudaStream_t st);
// Query-side backward on tcgen05 (pisa_tc_bwd.cu): dq, dr rows, dD per row, and the block's share of dkc, dvc.
cudaError_t pisa_tc_bwd_q(int dtype, int bh, int d, int nt, int ns, int T, float scale, const void* q, const void* k,
                          const void* v, const void* o, const void* d_o, const void* kc16, const void* vc16, const void* h16,
                          const int32_t* indices, const float* row_stats, void* dq, void* dr, float* dkc, float* dvc,
                          float* drow, cudaStream_t st);

// Key-side backward on tcgen05: dk, dv of every key block from the query blocks that selected it, plus the
// statistics terms.  dkc, dvc are overwritten (the per-block terms every key receives alike); dh16: 16-bit
// scratch of bh * d * d elements.  Usable while pisa_tc_bwd_kv_fits() (shared memory grows with nt).
cudaError_t pisa_tc_bwd_kv(int dtype, int bh, int d, int nt, int ns, int T, float scale, const void* q, const void* k,
                           const void* v, const void* d_o, const float* kc, const float* vc, const int32_t* indices,
                           const float* row_stats, const float* drow, float* dkc, float* dvc, const float* dh, void* dh16,
                           void* dk, void* dv, cudaStream_t st);
bool pisa_tc_bwd_kv_fits(int d, int nt);

}  // namespace fbla
