// fbla_linear_attn_fwd_state_noalloc: the forward state pass of linear_attention for
// callers that have no scratch buffer to hand over.
//
// The regular entry point, fbla_linear_attn_fwd_state, wants a caller-allocated workspace
// for the per-segment partial states.  Some embedders cannot provide one: a plugin that is
// invoked from inside another runtime's operator with nothing but that operator's input and
// output buffers, or a serving loop that fixed its device-memory budget at start-up, has no
// allocator to ask, and calling cudaMalloc there is not an option (it may fail against the
// host's budget, and it serialises the whole device).  For them this variant keeps the
// scratch inside the library: a file-scope device array of kScratchBytes that every GPU
// which loads the library holds until the process exits.
#include <mutex>

#include "fbla_common.cuh"
#include "tc_kernels.cuh"

namespace {

constexpr size_t kScratchBytes = 8u << 20;   // 8 MiB: e.g. 128 (batch, head) units of a 64 x 64 state

// In host code these names are host-side stand-ins, not device addresses: the address a kernel
// may use comes from cudaGetSymbolAddress (set_up below).
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];
static __device__ int g_status;   // written by a kernel whose bounded wait gave up

struct DeviceSide {
    bool ready = false;
    void* scratch = nullptr;
    int* status = nullptr;
    int failed = 0;       // last non-zero status read back by fbla_noalloc_status (until cleared)
};
DeviceSide g_dev[64];
std::mutex g_mu;

// Once per device, with that device current: resolve the device addresses of the two arrays.
int set_up(DeviceSide** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fbla::api_fail(FBLA_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fbla::api_fail(FBLA_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceSide& d = g_dev[dev];
    if (!d.ready) {
        void* scratch = nullptr;
        void* status = nullptr;
        e = cudaGetSymbolAddress(&scratch, g_scratch);
        if (e != cudaSuccess)
            return fbla::api_fail(FBLA_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        e = cudaGetSymbolAddress(&status, g_status);
        if (e != cudaSuccess)
            return fbla::api_fail(FBLA_ERR_CUDA, "cudaGetSymbolAddress(status): %s", cudaGetErrorString(e));
        d.scratch = scratch;
        d.status = static_cast<int*>(status);
        d.ready = true;
    }
    *out = &d;
    return FBLA_OK;
}

}  // namespace

// Same result as fbla_linear_attn_fwd_state (the state is bit-identical), without a workspace
// argument and without allocating: no cudaMalloc / cudaFree / cudaHostAlloc, no library that
// allocates.
//
//  * Limit: the scratch the tensor-core kernels need for the problem (one fp32 state per segment
//    of the tile schedule; never more than fbla_workspace_bytes of the same problem) must not
//    exceed 8 MiB; larger problems are refused with FBLA_ERR_WORKSPACE and a message.  Only
//    shapes served by the tensor-core kernels are accepted (16-bit inputs, dk, dv in {64, 128},
//    16-byte aligned tensors): the CUDA-core kernels need far more scratch.
//  * The first call on each device resolves the address of the library's scratch array
//    (cudaGetSymbolAddress) with that device current; make that first call before any stream
//    capture begins.
//  * Every call on a device shares the one array.  It keeps the previous call's partials, which
//    is harmless -- each call overwrites every slot it later reads, nothing has to start at zero
//    -- but two calls whose kernels overlap on the GPU (different streams, no dependency) race on
//    it: order them.
//  * A kernel whose bounded wait gives up records that in a device word of the library; this entry
//    point never synchronises, so the failure is not in its own return value.
//    fbla_noalloc_status() reads the word back (it synchronises; it allocates nothing); once it
//    has seen a failure, this entry point returns FBLA_ERR_DEVICE until the word is cleared.
extern "C" int fbla_linear_attn_fwd_state_noalloc(const fbla_problem* p, const void* k, const void* v,
                                                  float* state, fbla_stream_t stream) {
    fbla::KParams kp;
    if (int rc = fbla::api_resolve_linear(p, &kp)) return rc;
    if (k == nullptr || v == nullptr || state == nullptr)
        return fbla::api_fail(FBLA_ERR_INVALID, "k, v and state must not be NULL");
    if (kp.units == 0 || kp.seq_len == 0)
        return fbla::api_fail(FBLA_ERR_UNSUPPORTED, "empty problem: use fbla_linear_attn_fwd_state");
    if ((p->flags & FBLA_FLAG_GENERIC) || !fbla::tc_supported(kp, p->dtype) ||
        ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u) != 0)
        return fbla::api_fail(FBLA_ERR_UNSUPPORTED,
                              "the no-allocation variant serves 16-bit inputs with dk, dv in {64, 128} and "
                              "16-byte aligned tensors only");
    const int64_t need = fbla::tc_workspace_bytes(kp);
    if (need > (int64_t)kScratchBytes)
        return fbla::api_fail(FBLA_ERR_WORKSPACE,
                              "problem needs %lld bytes of scratch, the built-in array holds %lld: use "
                              "fbla_linear_attn_fwd_state with a caller-allocated workspace",
                              (long long)need, (long long)kScratchBytes);
    DeviceSide* d = nullptr;
    if (int rc = set_up(&d)) return rc;
    if (d->failed != 0)
        return fbla::api_fail(FBLA_ERR_DEVICE, "an earlier no-allocation call gave up a bounded wait (site %d); "
                              "clear it with fbla_noalloc_status(&v, 1)", d->failed);
    const cudaError_t e = fbla::tc_fwd_state_status(kp, p->dtype, k, nullptr, v, state, d->scratch, d->status,
                                                    (cudaStream_t)stream);
    if (e != cudaSuccess) return fbla::api_fail(FBLA_ERR_CUDA, "forward state pass: %s", cudaGetErrorString(e));
    return FBLA_OK;
}

// Reads the status word of the no-allocation entry point on the current device into *value (0 = no
// kernel of it has given up a wait; otherwise the number of the wait) and, with `clear` non-zero,
// resets it.  Synchronous 4-byte copies (the call waits for the device); nothing is allocated.
extern "C" int fbla_noalloc_status(int* value, int clear) {
    if (value == nullptr) return fbla::api_fail(FBLA_ERR_INVALID, "value is NULL");
    DeviceSide* d = nullptr;
    if (int rc = set_up(&d)) return rc;
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, d->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fbla::api_fail(FBLA_ERR_CUDA, "reading the status word: %s", cudaGetErrorString(e));
    *value = v;
    std::lock_guard<std::mutex> lock(g_mu);
    if (v != 0) d->failed = v;
    if (clear) {
        const int zero = 0;
        e = cudaMemcpy(d->status, &zero, sizeof(int), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) return fbla::api_fail(FBLA_ERR_CUDA, "clearing the status word: %s", cudaGetErrorString(e));
        d->failed = 0;
    }
    return FBLA_OK;
}
