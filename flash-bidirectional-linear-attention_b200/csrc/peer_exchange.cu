// Sum of the per-rank fp32 states of a sequence-sharded operator over the GPUs of one node, read
// straight from the peers' memory over NVLink (plain peer loads, no multicast): one kernel per
// exchange instead of a library all-reduce.  This serves the shapes that run on the CUDA-core
// kernels; on the tensor-core kernels the exchange happens inside the passes (tc_common.cuh).
//
// Every rank owns a buffer that its peers have mapped (symmetric memory) and a small array of flag
// words, one per peer.  The pass that produces the local state writes it into the buffer; then, in
// this kernel,
//   1. one CTA stores `epoch` into slot [rank] of every peer's flag array (release, system scope);
//   2. every CTA waits until the local slots of all peers have reached `epoch` (acquire, system
//      scope; bounded: after `wait_ns` it records the site in the status word and the CTA fills
//      its share of the result with NaN);
//   3. the CTAs add the `world` buffers in rank order -- the same order on every rank, so all ranks
//      hold bit-identical sums -- and write the result to ordinary local memory.
// The caller alternates between two buffers: a rank reaches the exchange after next only when every
// peer has entered the next one, i.e. has finished reading this one, so no second barrier is needed.
// Each GPU runs exactly one of these kernels per exchange; they wait on one another ACROSS GPUs only.
#include "fbla_common.cuh"
#include "tc_kernels.cuh"

namespace fbla {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kPeerThreads = 256;

struct PeerTable {
    const float4* buf[kMaxWorld];
    unsigned int* flag[kMaxWorld];
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kPeerThreads)
peer_state_sum_kernel(PeerTable t, int world, int rank, long long n4, unsigned int epoch, float4* __restrict__ out,
                      int* status, unsigned long long wait_ns) {
    __shared__ int gave_up;
    if (threadIdx.x == 0) gave_up = 0;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x < world && (int)threadIdx.x != rank) {
        __threadfence_system();
        st_release_sys(t.flag[threadIdx.x] + rank, epoch);
    }
    if (threadIdx.x < world && (int)threadIdx.x != rank) {
        const unsigned int* mine = t.flag[rank] + threadIdx.x;
        unsigned long long t0, now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - t0 > wait_ns) {
                gave_up = 1;
                if (status != nullptr) *status = 901;
                break;
            }
        }
    }
    __syncthreads();
    if (gave_up) {
        // no sum without the peers: make the failure impossible to miss downstream
        const float nan = __int_as_float(0x7fc00000);
        for (long long i = (long long)blockIdx.x * kPeerThreads + threadIdx.x; i < n4; i += (long long)gridDim.x * kPeerThreads)
            out[i] = make_float4(nan, nan, nan, nan);
        return;
    }
    // All peers' loads of an element are issued before the first add (NVLink latency is paid once, not
    // `world` times); the adds then run in rank order.  __ldcg = L2 only: a peer's line may differ from
    // the one read two exchanges ago.
    for (long long i = (long long)blockIdx.x * kPeerThreads + threadIdx.x; i < n4; i += (long long)gridDim.x * kPeerThreads) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r0 = 0; r0 < world; r0 += 8) {
            float4 x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (r0 + u < world) x[u] = __ldcg(t.buf[r0 + u] + i);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (r0 + u < world) { acc.x += x[u].x; acc.y += x[u].y; acc.z += x[u].z; acc.w += x[u].w; }
        }
        out[i] = acc;
    }
}

}  // namespace
}  // namespace fbla

extern "C" int fbla_peer_state_sum(int world, int rank, const void* const* peer_states, void* const* peer_flags,
                                   int64_t n_floats, uint32_t epoch, float* out, fbla_stream_t stream) {
    if (world < 1 || world > fbla::kMaxWorld || rank < 0 || rank >= world)
        return fbla::api_fail(FBLA_ERR_INVALID, "world %d / rank %d out of range (at most %d ranks)", world, rank,
                              fbla::kMaxWorld);
    if (peer_states == nullptr || peer_flags == nullptr || out == nullptr)
        return fbla::api_fail(FBLA_ERR_INVALID, "a pointer is NULL");
    if (n_floats < 0 || (n_floats & 3) != 0)
        return fbla::api_fail(FBLA_ERR_INVALID, "the state size must be a multiple of 4 floats");
    fbla::PeerTable t{};
    uintptr_t all = reinterpret_cast<uintptr_t>(out);
    for (int r = 0; r < world; ++r) {
        if (peer_states[r] == nullptr || peer_flags[r] == nullptr)
            return fbla::api_fail(FBLA_ERR_INVALID, "peer %d: NULL buffer or flag pointer", r);
        t.buf[r] = static_cast<const float4*>(peer_states[r]);
        t.flag[r] = static_cast<unsigned int*>(peer_flags[r]);
        all |= reinterpret_cast<uintptr_t>(peer_states[r]);
    }
    if ((all & 15u) != 0) return fbla::api_fail(FBLA_ERR_INVALID, "buffers must be 16-byte aligned");
    if (n_floats == 0) return FBLA_OK;
    const int s = fbla::tc_device_status();
    if (s != 0)
        return fbla::api_fail(FBLA_ERR_DEVICE, "a kernel gave up a bounded wait (site %d); results are invalid", s);
    const long long n4 = n_floats / 4;
    long long blocks = (n4 + fbla::kPeerThreads - 1) / fbla::kPeerThreads;
    if (blocks > 592) blocks = 592;
    fbla::peer_state_sum_kernel<<<(unsigned)blocks, fbla::kPeerThreads, 0, (cudaStream_t)stream>>>(
        t, world, rank, n4, epoch, reinterpret_cast<float4*>(out), fbla::tc_status_word(), fbla::tc_peer_wait_ns());
    fbla::note_launches(1);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FBLA_OK : fbla::api_fail(FBLA_ERR_CUDA, "peer state sum: %s", cudaGetErrorString(e));
}
