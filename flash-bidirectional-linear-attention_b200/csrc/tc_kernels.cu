// Host side of the tensor-core path: TMA tensor maps, the static tile schedule, shared
// memory opt-in and the launches of the kernels in tc_fwd.cuh / tc_bwd.cuh.
#include "tc_kernels.cuh"

#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <utility>

#include "tc_bwd_in.cuh"
#include "tc_bwd_state.cuh"
#include "tc_fwd.cuh"

namespace fbla {
namespace {

using namespace tc;

#ifndef FBLA_L2_PROMOTION
#define FBLA_L2_PROMOTION CU_TENSOR_MAP_L2_PROMOTION_L2_256B
#endif

// ---- driver entry point for tensor-map encoding (no link-time dependency on libcuda) ------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// The driver call needs a CUDA context bound to the calling thread.  A thread that has made no
// context-binding runtime call yet (an autograd worker whose first work is this library) has none
// and gets CUDA_ERROR_INVALID_CONTEXT: bind the current device's primary context and try again.
CUresult encode_tiled(CUtensorMap* m, CUtensorMapDataType dt, const void* base, const cuuint64_t* dims,
                      const cuuint64_t* strides, const cuuint32_t* box) {
    EncodeTiledFn fn = encode_fn();
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = CUDA_ERROR_INVALID_CONTEXT;
    for (int attempt = 0; attempt < 2 && r == CUDA_ERROR_INVALID_CONTEXT; ++attempt) {
        if (attempt == 1) {
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) break;
        }
        r = fn(m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, FBLA_L2_PROMOTION, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    return r;
}

// (units, T, D) 16-bit tensor viewed as a 3-D map {D, T, units}; one box = 64 features x 128
// tokens of one unit, written to shared memory in the 128-byte-swizzled layout.  Tokens past T
// read as zero and are dropped on stores.
struct MapKey {
    const void* base;
    int dtype, D, units;
    int64_t T;
    bool operator==(const MapKey& o) const {
        return base == o.base && dtype == o.dtype && D == o.D && units == o.units && T == o.T;
    }
};
struct MapSlot {
    MapKey key{nullptr, 0, 0, 0, 0};
    CUtensorMap map;
};

cudaError_t encode_map(CUtensorMap* m, const void* base, int dtype, int D, int64_t T, int units);

// Encoding a tensor map costs a few microseconds on the host; training loops call with the same
// buffers again and again, so each thread keeps the last maps it made.  A map is a pure function
// of its key (address, type, extents), so a stale entry can never be wrong.
cudaError_t make_map(CUtensorMap* m, const void* base, int dtype, int D, int64_t T, int units) {
    constexpr int kSlots = 64;
    thread_local MapSlot cache[kSlots];
    const MapKey key{base, dtype, D, units, T};
    const size_t h = (reinterpret_cast<uintptr_t>(base) >> 8) * 0x9E3779B97F4A7C15ull + (size_t)T * 31 + (size_t)D;
    MapSlot& slot = cache[(h >> 20) % kSlots];
    if (slot.key == key) {
        *m = slot.map;
        return cudaSuccess;
    }
    const cudaError_t e = encode_map(m, base, dtype, D, T, units);
    if (e == cudaSuccess) {
        slot.key = key;
        slot.map = *m;
    }
    return e;
}

cudaError_t encode_map(CUtensorMap* m, const void* base, int dtype, int D, int64_t T, int units) {
    if (encode_fn() == nullptr) return cudaErrorNotSupported;
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)units};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)T * D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)kTileTokens, 1};
    const CUtensorMapDataType dt = dtype == FBLA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = encode_tiled(m, dt, base, dims, strides, box);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace

// Same view with a box of `box_rows` rows (the attention stage works on blocks of 64 tokens).
cudaError_t tc_encode_map_rows(CUtensorMap* m, const void* base, int dtype, int D, int64_t rows, int units, int box_rows) {
    if (encode_fn() == nullptr) return cudaErrorNotSupported;
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)units};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)rows * D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    const CUtensorMapDataType dt = dtype == FBLA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = encode_tiled(m, dt, base, dims, strides, box);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

namespace {

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

Schedule make_schedule(const KParams& p, int sms) {
    Schedule s;
    s.units = p.units;
    s.tiles_per_unit = (int)((p.seq_len + kTileTokens - 1) / kTileTokens);
    s.total_tiles = s.units * s.tiles_per_unit;
    const int ctas = s.total_tiles < sms ? s.total_tiles : sms;
    s.tiles_per_cta = (s.total_tiles + ctas - 1) / ctas;
    s.ctas = (s.total_tiles + s.tiles_per_cta - 1) / s.tiles_per_cta;
    s.slots_per_unit = (s.tiles_per_unit + s.tiles_per_cta - 1) / s.tiles_per_cta + 1;
    return s;
}

// Host-visible status word the kernels write when a bounded wait gives up.
int* g_status_host = nullptr;
int* g_status_dev = nullptr;
std::once_flag g_status_once;

int* status_word() {
    std::call_once(g_status_once, [] {
        void* h = nullptr;
        if (cudaHostAlloc(&h, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
            *static_cast<int*>(h) = 0;
            void* d = nullptr;
            if (cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess) {
                g_status_host = static_cast<int*>(h);
                g_status_dev = static_cast<int*>(d);
            }
        }
    });
    return g_status_dev;
}

Params make_params(const KParams& p, int dtype, const Schedule& s, int* status);

Params make_params(const KParams& p, int dtype, const Schedule& s) { return make_params(p, dtype, s, status_word()); }

Params make_params(const KParams& p, int dtype, const Schedule& s, int* status) {
    Params q;
    q.sch = s;
    q.seq_len = (int)p.seq_len;
    q.scale = p.scale;
    q.inv_norm = p.inv_norm > 0.f ? p.inv_norm : 1.f / (float)p.seq_len;
    q.eps = p.eps;
    q.is_bf16 = dtype == FBLA_BF16;
    q.status = status;
    q.part = nullptr;
    q.state = nullptr;
    q.state_parts = nullptr;
    q.state_stride = p.state_stride;
    q.out_a = nullptr;
    q.out_b = nullptr;
    q.state_out = nullptr;
    q.cu = nullptr;
    q.plan = nullptr;
    q.num_seqs = 0;
    q.heads = p.heads;
    q.mem_dk = p.mem_dk;
    q.mem_dv = p.mem_dv;
    q.scale_per_seq = 0;
    q.inv_norm_fixed = 0.f;
    return q;
}

// Opt in to the large dynamic shared memory once per kernel and device; `done` is the
// per-kernel record kept by the caller (one per template instantiation).
template <typename K>
cudaError_t set_smem(K kernel, int bytes, bool (&done)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (done[dev]) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done[dev] = true;
    return e;
}

// Launch with the programmatic-serialization attribute: the kernel may become resident while the
// previous kernel of the stream is still draining (it calls griddepcontrol.wait before it touches
// global memory).  FBLA_NO_PDL=1 in the environment restores ordinary launches.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), int grid, int block, int smem, cudaStream_t st, Args&&... args) {
    static const bool plain = [] {
        const char* e = getenv("FBLA_NO_PDL");
        return e != nullptr && e[0] == '1';
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = plain ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

int mode_of(const KParams& p, bool decoupled) { return !p.normalize ? kSimple : (decoupled ? kDecoupled : kLinear); }

cudaError_t reduce_partials(const Params& q, float* state, cudaStream_t st) {
    const long long total = (long long)q.sch.units * q.state_stride;
    tc_reduce_partials_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(q.part, state, q.sch, q.state_stride);
    note_launches(1);
    return cudaGetLastError();
}

// ---- per-shape launch helpers ----------------------------------------------------------------
template <int DK, int DV, int MODE, bool BF16, bool VARLEN = false>
cudaError_t launch_fwd_state(const Params& q, const CUtensorMap& tkr, const CUtensorMap& tk, const CUtensorMap& tv,
                             cudaStream_t st) {
    using Cfg = FwdStateCfg<DK, DV, MODE>;
    static_assert(Cfg::kSmemBytes <= kSmemLimit, "shared memory budget");
    auto kernel = tc_fwd_state_kernel<DK, DV, MODE, BF16, VARLEN>;
    static bool smem_set[64] = {false};
    cudaError_t e = set_smem(kernel, Cfg::kSmemBytes, smem_set);
    if (e != cudaSuccess) return e;
    e = launch_dependent(kernel, q.sch.ctas, kThreads, Cfg::kSmemBytes, st, tkr, tk, tv, q);
    note_launches(1);
    return e != cudaSuccess ? e : cudaGetLastError();
}

template <int DK, int DV, int MODE, bool BF16, bool VARLEN = false>
cudaError_t launch_fwd_out(const Params& q, const CUtensorMap& tqr, const CUtensorMap& tq, const CUtensorMap& to,
                           cudaStream_t st) {
    using Cfg = FwdOutCfg<DK, DV, MODE>;
    static_assert(Cfg::kSmemBytes <= kSmemLimit, "shared memory budget");
    static_assert(Cfg::kStages >= 2, "pipeline depth");
    auto kernel = tc_fwd_out_kernel<DK, DV, MODE, BF16, VARLEN>;
    static bool smem_set[64] = {false};
    cudaError_t e = set_smem(kernel, Cfg::kSmemBytes, smem_set);
    if (e != cudaSuccess) return e;
    e = launch_dependent(kernel, q.sch.ctas, kThreads, Cfg::kSmemBytes, st, tqr, tq, to, q);
    note_launches(1);
    return e != cudaSuccess ? e : cudaGetLastError();
}

template <int DK, int DV, int MODE, bool BF16, bool VARLEN = false>
cudaError_t launch_bwd_state(const Params& q, const CUtensorMap& tqr, const CUtensorMap& tq, const CUtensorMap& tdo,
                             const CUtensorMap& tdq, const CUtensorMap& tdqr, cudaStream_t st) {
    using Cfg = BwdStateCfg<DK, DV, MODE, VARLEN>;
    static_assert(Cfg::kSmemBytes <= kSmemLimit, "shared memory budget");
    static_assert(Cfg::kStages >= 2, "pipeline depth");
    auto go = [&](auto kernel, bool (&smem_set)[64]) -> cudaError_t {
        cudaError_t e = set_smem(kernel, Cfg::kSmemBytes, smem_set);
        if (e != cudaSuccess) return e;
        e = launch_dependent(kernel, q.sch.ctas, kBwdStateThreads, Cfg::kSmemBytes, st, tqr, tq, tdo, tdq, tdqr, q);
        note_launches(1);
        return e != cudaSuccess ? e : cudaGetLastError();
    };
    static bool set_wide[64] = {false}, set_narrow[64] = {false};
    if (q.mem_dk != DK) return go(tc_bwd_state_kernel<DK, DV, MODE, BF16, VARLEN, true>, set_narrow);
    return go(tc_bwd_state_kernel<DK, DV, MODE, BF16, VARLEN, false>, set_wide);
}

template <int DK, int DV, int MODE, bool BF16, bool VARLEN = false>
cudaError_t launch_bwd_in(const Params& q, const CUtensorMap& tkr, const CUtensorMap& tv, const CUtensorMap& tdk,
                          const CUtensorMap& tdkr, const CUtensorMap& tdv, cudaStream_t st) {
    using Cfg = BwdInCfg<DK, DV, MODE>;
    static_assert(Cfg::kSmemBytes <= kSmemLimit, "shared memory budget");
    static_assert(Cfg::kStages >= 2, "pipeline depth");
    auto kernel = tc_bwd_in_kernel<DK, DV, MODE, BF16, VARLEN>;
    static bool smem_set[64] = {false};
    cudaError_t e = set_smem(kernel, Cfg::kSmemBytes, smem_set);
    if (e != cudaSuccess) return e;
    e = launch_dependent(kernel, q.sch.ctas, kThreads, Cfg::kSmemBytes, st, tkr, tv, tdk, tdkr, tdv, q);
    note_launches(1);
    return e != cudaSuccess ? e : cudaGetLastError();
}

// Expands to a switch over (dk, dv, mode, 16-bit type); `CALL` names one of the launch_* templates.
#define FBLA_TC_CASES(CALL, BF, ...)                                                                    \
    switch (mode * 4 + key) {                                                                           \
        case 0: return CALL<64, 64, kSimple, BF>(__VA_ARGS__);                                          \
        case 1: return CALL<64, 128, kSimple, BF>(__VA_ARGS__);                                         \
        case 2: return CALL<128, 64, kSimple, BF>(__VA_ARGS__);                                         \
        case 3: return CALL<128, 128, kSimple, BF>(__VA_ARGS__);                                        \
        case 4: return CALL<64, 64, kLinear, BF>(__VA_ARGS__);                                          \
        case 5: return CALL<64, 128, kLinear, BF>(__VA_ARGS__);                                         \
        case 6: return CALL<128, 64, kLinear, BF>(__VA_ARGS__);                                         \
        case 7: return CALL<128, 128, kLinear, BF>(__VA_ARGS__);                                        \
        case 8: return CALL<64, 64, kDecoupled, BF>(__VA_ARGS__);                                       \
        default: return cudaErrorNotSupported;                                                          \
    }
#define FBLA_TC_DISPATCH(CALL, ...)                                                                     \
    do {                                                                                                \
        const int key = (p.dk == 128 ? 2 : 0) + (p.dv == 128 ? 1 : 0);                                  \
        if (dtype == FBLA_BF16) {                                                                       \
            FBLA_TC_CASES(CALL, true, __VA_ARGS__)                                                      \
        } else {                                                                                        \
            FBLA_TC_CASES(CALL, false, __VA_ARGS__)                                                     \
        }                                                                                               \
    } while (0)

// Packed (varlen) layout: normalised operator only.
#define FBLA_TC_VARLEN_DISPATCH(CALL, ...)                                                              \
    do {                                                                                                \
        const int key = (p.dk == 128 ? 2 : 0) + (p.dv == 128 ? 1 : 0) + (dtype == FBLA_BF16 ? 4 : 0);   \
        switch (key) {                                                                                  \
            case 0: return CALL<64, 64, kLinear, false, true>(__VA_ARGS__);                             \
            case 1: return CALL<64, 128, kLinear, false, true>(__VA_ARGS__);                            \
            case 2: return CALL<128, 64, kLinear, false, true>(__VA_ARGS__);                            \
            case 3: return CALL<128, 128, kLinear, false, true>(__VA_ARGS__);                           \
            case 4: return CALL<64, 64, kLinear, true, true>(__VA_ARGS__);                              \
            case 5: return CALL<64, 128, kLinear, true, true>(__VA_ARGS__);                             \
            case 6: return CALL<128, 64, kLinear, true, true>(__VA_ARGS__);                             \
            default: return CALL<128, 128, kLinear, true, true>(__VA_ARGS__);                           \
        }                                                                                               \
    } while (0)

// ---- packed layout: tensor maps, tile plan, workspace split ---------------------------------------
// (total_tokens, heads, D) 16-bit tensor as a 3-D map {D, heads, total_tokens}; one box = 64 features
// of one head over 128 consecutive tokens, same shared-memory tile as the fixed-length box.
cudaError_t make_map_packed(CUtensorMap* m, const void* base, int dtype, int D, int heads, int64_t tokens) {
    if (encode_fn() == nullptr) return cudaErrorNotSupported;
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)heads * D * 2};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t)kTileTokens};
    const CUtensorMapDataType dt = dtype == FBLA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = encode_tiled(m, dt, base, dims, strides, box);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Fills the packed-layout fields of the kernel parameters (each kernel builds its tile plan itself).
Params make_params_packed(const KParams& p, int dtype) {
    Schedule s{};
    s.units = p.units;
    s.ctas = (sm_count() / p.heads) * p.heads;       // groups of `heads` CTAs, one head each
    Params q = make_params(p, dtype, s);
    q.cu = p.cu;
    q.plan = nullptr;
    q.num_seqs = p.units / p.heads;
    q.heads = p.heads;
    q.scale_per_seq = p.scale_per_seq;
    q.inv_norm_fixed = p.inv_norm > 0.f ? p.inv_norm : 0.f;
    return q;
}

}  // namespace

// The tensor-core kernels serve 16-bit inputs in the fixed-length layout with dk, dv in
// {64, 128}; the decoupled operator at 64 x 64 only (its extra tiles do not fit the shared
// memory budget at 128).
bool tc_supported(const KParams& p, int dtype) {
    if (dtype != FBLA_BF16 && dtype != FBLA_F16) return false;
    if (p.cu != nullptr &&
        (!p.normalize || p.seq_len >= (1LL << 31) - 256 || p.units / p.heads > kMaxPackedSeqs ||
         p.heads > sm_count()))
        return false;
    if ((p.dk != 64 && p.dk != 128) || (p.dv != 64 && p.dv != 128)) return false;
    if (p.seq_len < 1 || p.units < 1) return false;
    if (encode_fn() == nullptr) return false;
    return true;
}

bool tc_supported_decoupled(const KParams& p) { return p.dk == 64 && p.dv == 64; }

int64_t tc_workspace_bytes(const KParams& p) {
    if (p.cu != nullptr)   // two partial slots per CTA
        return (int64_t)sm_count() * 2 * p.state_stride * (int64_t)sizeof(float);
    const Schedule s = make_schedule(p, sm_count());
    return (int64_t)s.units * s.slots_per_unit * p.state_stride * (int64_t)sizeof(float);
}


PieceLayout tc_piece_layout(const KParams& p) {
    const Schedule s = make_schedule(p, sm_count());
    return PieceLayout{s.units, s.slots_per_unit, s.tiles_per_unit, s.tiles_per_cta};
}

// How long a kernel waits for a peer GPU before it gives up and reports through the status word:
// FBLA_PEER_WAIT_MS in the environment, 5 s by default.  Ranks that may be further apart than this
// (one of them writing a checkpoint, say) should meet at a host-side barrier before the call.
unsigned long long tc_peer_wait_ns() {
    static const unsigned long long ns = [] {
        const char* e = getenv("FBLA_PEER_WAIT_MS");
        double ms = e != nullptr ? atof(e) : 0.0;
        if (!(ms > 0.0)) ms = 5000.0;
        return (unsigned long long)(ms * 1e6);
    }();
    return ns;
}

int tc_device_status() { return g_status_host != nullptr ? *static_cast<volatile int*>(g_status_host) : 0; }
void tc_clear_device_status() {
    if (g_status_host != nullptr) *static_cast<volatile int*>(g_status_host) = 0;
}
int* tc_status_word() { return status_word(); }

cudaError_t tc_fwd_state(const KParams& p, int dtype, const void* k, const void* k_rope, const void* v, float* state,
                         void* ws, cudaStream_t st) {
    return tc_fwd_state_status(p, dtype, k, k_rope, v, state, ws, status_word(), st);
}

cudaError_t tc_fwd_state_status(const KParams& p, int dtype, const void* k, const void* k_rope, const void* v,
                                float* state, void* ws, int* status, cudaStream_t st) {
    if (p.cu != nullptr) {
        // packed layout: zeroed state (units without tokens stay zero), state kernel, reduce
        cudaError_t e;
        if ((e = cudaMemsetAsync(state, 0, sizeof(float) * (size_t)p.units * p.state_stride, st)) != cudaSuccess) return e;
        Params q = make_params_packed(p, dtype);
        q.status = status;
        q.state_out = state;
        q.part = static_cast<float*>(ws);
        CUtensorMap tk, tv;
        if ((e = make_map_packed(&tk, k, dtype, p.mem_dk, p.heads, p.seq_len)) != cudaSuccess) return e;
        if ((e = make_map_packed(&tv, v, dtype, p.mem_dv, p.heads, p.seq_len)) != cudaSuccess) return e;
        auto launch = [&]() -> cudaError_t { FBLA_TC_VARLEN_DISPATCH(launch_fwd_state, q, tk, tk, tv, st); };
        if ((e = launch()) != cudaSuccess) return e;
        tc_reduce_varlen_kernel<<<q.sch.ctas, 256, 0, st>>>(q, state, q.sch.ctas);
        note_launches(1);
        return cudaGetLastError();
    }
    const bool dec = k_rope != nullptr && k_rope != k;
    const int mode = mode_of(p, dec);
    const Schedule s = make_schedule(p, sm_count());
    if (status == nullptr) return cudaErrorMemoryAllocation;
    Params q = make_params(p, dtype, s, status);
    q.part = static_cast<float*>(ws);
    CUtensorMap tkr, tk, tv;
    cudaError_t e;
    if ((e = make_map(&tkr, dec ? k_rope : k, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tk, k, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tv, v, dtype, p.mem_dv, p.seq_len, p.units)) != cudaSuccess) return e;
    auto launch = [&]() -> cudaError_t { FBLA_TC_DISPATCH(launch_fwd_state, q, tkr, tk, tv, st); };
    if ((e = launch()) != cudaSuccess) return e;
    if (p.unreduced) return cudaSuccess;        // the pieces in `ws` are the result
    return reduce_partials(q, state, st);
}

cudaError_t tc_fwd_out(const KParams& p, int dtype, const void* q_, const void* q_rope, const float* state, void* o,
                       cudaStream_t st) {
    if (p.cu != nullptr) {
        Params q = make_params_packed(p, dtype);
        if (q.status == nullptr) return cudaErrorMemoryAllocation;
        q.state = state;
        q.out_a = o;
        CUtensorMap tq, to;
        cudaError_t e;
        if ((e = make_map_packed(&tq, q_, dtype, p.mem_dk, p.heads, p.seq_len)) != cudaSuccess) return e;
        if ((e = make_map_packed(&to, o, dtype, p.mem_dv, p.heads, p.seq_len)) != cudaSuccess) return e;
        FBLA_TC_VARLEN_DISPATCH(launch_fwd_out, q, tq, tq, to, st);
    }
    const bool dec = q_rope != nullptr && q_rope != q_;
    const int mode = mode_of(p, dec);
    const Schedule s = make_schedule(p, sm_count());
    Params q = make_params(p, dtype, s);
    if (q.status == nullptr) return cudaErrorMemoryAllocation;
    q.state = state;
    if (p.unreduced == 1) q.state_parts = state;
    q.out_a = o;
    CUtensorMap tqr, tq, to;
    cudaError_t e;
    if ((e = make_map(&tqr, dec ? q_rope : q_, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tq, q_, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&to, o, dtype, p.mem_dv, p.seq_len, p.units)) != cudaSuccess) return e;
    FBLA_TC_DISPATCH(launch_fwd_out, q, tqr, tq, to, st);
}

cudaError_t tc_bwd_state(const KParams& p, int dtype, const void* q_, const void* q_rope, const void* d_o,
                         const float* state, void* dq, void* dq_rope, float* dstate, void* ws, cudaStream_t st) {
    if (p.cu != nullptr) {
        cudaError_t e;
        if ((e = cudaMemsetAsync(dstate, 0, sizeof(float) * (size_t)p.units * p.state_stride, st)) != cudaSuccess) return e;
        Params q = make_params_packed(p, dtype);
        if (q.status == nullptr) return cudaErrorMemoryAllocation;
        q.state = state;
        q.state_out = dstate;
        q.part = static_cast<float*>(ws);
        q.out_a = dq;
        q.out_b = dq;
        CUtensorMap tq, tdo, tdq;
        if ((e = make_map_packed(&tq, q_, dtype, p.mem_dk, p.heads, p.seq_len)) != cudaSuccess) return e;
        if ((e = make_map_packed(&tdo, d_o, dtype, p.mem_dv, p.heads, p.seq_len)) != cudaSuccess) return e;
        if ((e = make_map_packed(&tdq, dq, dtype, p.mem_dk, p.heads, p.seq_len)) != cudaSuccess) return e;
        auto launch = [&]() -> cudaError_t { FBLA_TC_VARLEN_DISPATCH(launch_bwd_state, q, tq, tq, tdo, tdq, tdq, st); };
        if ((e = launch()) != cudaSuccess) return e;
        tc_reduce_varlen_kernel<<<q.sch.ctas, 256, 0, st>>>(q, dstate, q.sch.ctas);
        note_launches(1);
        return cudaGetLastError();
    }
    const bool dec = dq_rope != nullptr;
    const int mode = mode_of(p, dec);
    const Schedule s = make_schedule(p, sm_count());
    Params q = make_params(p, dtype, s);
    if (q.status == nullptr) return cudaErrorMemoryAllocation;
    q.state = state;
    if (p.unreduced == 1) q.state_parts = state;
    q.part = static_cast<float*>(ws);
    q.out_a = dec ? dq_rope : dq;
    q.out_b = dq;
    CUtensorMap tqr, tq, tdo, tdq, tdqr;
    cudaError_t e;
    if ((e = make_map(&tqr, dec ? q_rope : q_, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tq, q_, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tdo, d_o, dtype, p.mem_dv, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tdq, dq, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tdqr, dec ? dq_rope : dq, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    auto launch = [&]() -> cudaError_t { FBLA_TC_DISPATCH(launch_bwd_state, q, tqr, tq, tdo, tdq, tdqr, st); };
    if ((e = launch()) != cudaSuccess) return e;
    if (p.unreduced) return cudaSuccess;
    return reduce_partials(q, dstate, st);
}

cudaError_t tc_bwd_in(const KParams& p, int dtype, const void* k_rope, const void* v, const float* dstate, void* dk,
                      void* dk_rope, void* dv, cudaStream_t st) {
    if (p.cu != nullptr) {
        Params q = make_params_packed(p, dtype);
        if (q.status == nullptr) return cudaErrorMemoryAllocation;
        q.state = dstate;
        q.out_a = dk;
        q.out_b = dv;
        CUtensorMap tk, tv, tdk, tdv;
        cudaError_t e;
        if ((e = make_map_packed(&tk, k_rope, dtype, p.mem_dk, p.heads, p.seq_len)) != cudaSuccess) return e;
        if ((e = make_map_packed(&tv, v, dtype, p.mem_dv, p.heads, p.seq_len)) != cudaSuccess) return e;
        if ((e = make_map_packed(&tdk, dk, dtype, p.mem_dk, p.heads, p.seq_len)) != cudaSuccess) return e;
        if ((e = make_map_packed(&tdv, dv, dtype, p.mem_dv, p.heads, p.seq_len)) != cudaSuccess) return e;
        FBLA_TC_VARLEN_DISPATCH(launch_bwd_in, q, tk, tv, tdk, tdk, tdv, st);
    }
    const bool dec = dk_rope != nullptr;
    const int mode = mode_of(p, dec);
    const Schedule s = make_schedule(p, sm_count());
    Params q = make_params(p, dtype, s);
    if (q.status == nullptr) return cudaErrorMemoryAllocation;
    q.state = dstate;
    if (p.unreduced == 1) q.state_parts = dstate;
    q.out_a = dec ? dk_rope : dk;      // kernels without a staged output tile store through these
    q.out_b = dv;
    CUtensorMap tkr, tv, tdk, tdkr, tdv;
    cudaError_t e;
    if ((e = make_map(&tkr, k_rope, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tv, v, dtype, p.mem_dv, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tdk, dk, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tdkr, dec ? dk_rope : dk, dtype, p.mem_dk, p.seq_len, p.units)) != cudaSuccess) return e;
    if ((e = make_map(&tdv, dv, dtype, p.mem_dv, p.seq_len, p.units)) != cudaSuccess) return e;
    FBLA_TC_DISPATCH(launch_bwd_in, q, tkr, tv, tdk, tdkr, tdv, st);
}

}  // namespace fbla
