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

}  // namespace fbla
