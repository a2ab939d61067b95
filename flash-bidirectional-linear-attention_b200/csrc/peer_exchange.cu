// Sum of the per-rank fp32 states of a sequence-sharded operator over the GPUs of one node, with plain
// loads from the peers' memory over NVLink (no multicast, no library collective): one kernel per
// exchange, launched between the reducing and the consuming pass.
//
// Two kernels:
//   peer_piece_sum_kernel : for the tensor-core passes.  Its input is the per-segment pieces the
//       reducing pass left in this rank's (peer-mapped) workspace, so no separate reduction runs first.
//       Each unit is summed once, by its owner (rank u / ceil(units / world)), into a peer-mapped
//       buffer, a second flag round follows, and every rank then reads the units it does not own from
//       their owners: 2 (world-1)/world of the state crosses NVLink per rank instead of (world-1) times
//       the state.  (FBLA_PEER_TWO_ROUND=0 selects the one-round form in which every rank adds the
//       pieces of ALL units from all ranks; it was no faster at two ranks.)  Either way a unit is added
//       in one fixed order (ranks in order, pieces in CTA order), so all ranks hold the same bits.
//   peer_state_sum_kernel : the one-round sum over already reduced states, for the CUDA-core passes.
//
// No payload is ever STORED to a peer: on a busy B200 a system-scope fence behind remote stores was
// measured at 10 us, a device-scope fence behind local stores at 0.5 us (peers read this GPU's memory
// through its L2); only flag words cross NVLink as stores.  Flags carry the exchange number, so they are
// never reset; the caller alternates between two buffer sets (a rank reaches exchange e+2 only after
// every peer has entered e+1, i.e. has finished reading the buffers of e).  One thread of the grid does
// the system-scope work (signalling, polling the flags the peers write, one fence each); the other
// CTAs follow a device-local word.  Every wait is bounded: on giving up the kernel records it in the
// status word and fills the result with NaN.  Each GPU runs exactly one of these kernels per exchange;
// they wait on one another ACROSS GPUs only.
#include <cstdlib>

#include "fbla_common.cuh"
#include "tc_kernels.cuh"

namespace fbla {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kMaxRanks = 8;           // piece sum
constexpr int kPeerThreads = 256;

// words of a rank's flag array
constexpr int kFlagRound1 = 0;         // [0, 16)  rank q has entered the exchange (its pieces can be read)
constexpr int kFlagRound2 = 16;        // [16, 32) rank q has summed its units
constexpr int kFlagTicket = 32;        // CTAs of this rank that have finished their share of the sums
constexpr int kFlagGo1 = 40;           // device-local: first flag round complete (written by the polling thread)
constexpr int kFlagGo2 = 41;           // device-local: second flag round complete
constexpr int kFlagAbort = 42;         // device-local: the polling thread gave up in this exchange

__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_relaxed_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

struct PieceSum {
    const float4* parts[kMaxRanks];    // rank r's pieces, [units][slots][s4]
    float4* full[kMaxRanks];           // rank r's sums of the units it owns, [units][s4]
    unsigned int* flags[kMaxRanks];
    int world, rank;
    unsigned int epoch;
    int units, units_per_rank, slots, tiles_per_unit, tiles_per_cta;
    int s4;                            // float4 per unit
    int two_round;
    float4* out;                       // [units][s4], ordinary local memory
    unsigned long long wait_ns;
    int* status;
};

// One thread (block 0, thread 0) polls the `world` words the peers write until all have reached
// `epoch`, fences once at system scope and publishes `go`; everybody else waits for `go` (or for the
// abort word).  Returns false when the exchange was given up.
__device__ __forceinline__ bool wait_round(const PieceSum& a, int round_base, int go_word, int site, int* s_ok) {
    unsigned int* mine = a.flags[a.rank];
    if (threadIdx.x == 0) {
        bool ok = true;
        const unsigned long long t0 = global_ns();
        if (blockIdx.x == 0) {
            int spins = 0;
            while (true) {
                bool all = true;
                for (int r = 0; r < a.world; ++r) all = all && (int)(ld_relaxed_sys(mine + round_base + r) - a.epoch) >= 0;
                if (all) break;
                if ((++spins & 7) == 0 && global_ns() - t0 > a.wait_ns) {
                    ok = false;
                    break;
                }
            }
            __threadfence_system();     // acquire: what the peers wrote before their flags is visible from here on
            if (ok) {
                st_relaxed_gpu(mine + go_word, a.epoch);
            } else {
                if (a.status != nullptr) *a.status = site;
                st_relaxed_gpu(mine + kFlagAbort, a.epoch);
            }
        } else {
            int spins = 0;
            while ((int)(ld_relaxed_gpu(mine + go_word) - a.epoch) < 0) {
                if ((++spins & 7) == 0) {
                    if (ld_relaxed_gpu(mine + kFlagAbort) == a.epoch || global_ns() - t0 > 2 * a.wait_ns) {
                        ok = false;
                        break;
                    }
                }
            }
            __threadfence();            // the polling thread's fence made the peers' data visible to this GPU
        }
        *s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    const bool ok = *s_ok != 0;
    __syncthreads();
    return ok;
}

// Sum of one float4 element of unit u over all ranks' pieces: the loads of all ranks (two pieces each)
// are in flight together, the adds run in rank, piece order.
__device__ __forceinline__ float4 sum_pieces(const PieceSum& a, int u, int e4) {
    const int first = (int)(((long long)u * a.tiles_per_unit) / a.tiles_per_cta);
    const int last = (int)((((long long)u + 1) * a.tiles_per_unit - 1) / a.tiles_per_cta);
    const int n = last - first + 1;
    const size_t off = ((size_t)u * a.slots) * a.s4 + e4;
    float4 y[kMaxRanks][2];
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
        if (q < a.world) {
            y[q][0] = __ldcg(a.parts[q] + off);
            if (n > 1) y[q][1] = __ldcg(a.parts[q] + off + a.s4);
        }
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
        if (q < a.world) {
            acc.x += y[q][0].x; acc.y += y[q][0].y; acc.z += y[q][0].z; acc.w += y[q][0].w;
            if (n > 1) { acc.x += y[q][1].x; acc.y += y[q][1].y; acc.z += y[q][1].z; acc.w += y[q][1].w; }
            for (int j = 2; j < n; ++j) {
                const float4 z = __ldcg(a.parts[q] + off + (size_t)j * a.s4);
                acc.x += z.x; acc.y += z.y; acc.z += z.z; acc.w += z.w;
            }
        }
    }
    return acc;
}

__global__ void __launch_bounds__(kPeerThreads)
peer_piece_sum_kernel(const __grid_constant__ PieceSum a) {
    __shared__ int s_ok;
    unsigned int* mine = a.flags[a.rank];
    const long long tid = (long long)blockIdx.x * kPeerThreads + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * kPeerThreads;
    const long long all4 = (long long)a.units * a.s4;
    const float nan = __int_as_float(0x7fc00000);
    // launched with programmatic stream serialization: let the consuming pass start its prologue now, and
    // wait here until the reducing pass (the previous kernel of the stream) has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // first flag round: this rank's pieces were written by the previous kernel of the stream
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        __threadfence_system();
        for (int r = 0; r < a.world; ++r) st_relaxed_sys(a.flags[r] + kFlagRound1 + a.rank, a.epoch);
    }
    if (!wait_round(a, kFlagRound1, kFlagGo1, 911, &s_ok)) {
        for (long long i = tid; i < all4; i += nthreads) a.out[i] = make_float4(nan, nan, nan, nan);
        return;
    }
    if (!a.two_round) {
        for (long long i = tid; i < all4; i += nthreads) {
            const int u = (int)(i / a.s4);
            a.out[i] = sum_pieces(a, u, (int)(i - (long long)u * a.s4));
        }
        return;
    }
    // the units this rank owns
    const int u0 = a.rank * a.units_per_rank;
    const int u1 = min(a.units, u0 + a.units_per_rank);
    const long long own4 = (long long)max(0, u1 - u0) * a.s4;
    for (long long i = tid; i < own4; i += nthreads) {
        const int u = u0 + (int)(i / a.s4);
        const long long at = (long long)u0 * a.s4 + i;
        const float4 acc = sum_pieces(a, u, (int)(at - (long long)u * a.s4));
        a.full[a.rank][at] = acc;
        a.out[at] = acc;
    }
    __threadfence();                    // the sums are in L2, where the peers read them
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int ticket = atomicAdd(mine + kFlagTicket, 1u);
        if (ticket == gridDim.x - 1) {
            mine[kFlagTicket] = 0;          // every CTA has drawn: ready for the next launch
            __threadfence_system();
            for (int r = 0; r < a.world; ++r) st_relaxed_sys(a.flags[r] + kFlagRound2 + a.rank, a.epoch);
        }
    }
    // second flag round: the other ranks' sums
    if (!wait_round(a, kFlagRound2, kFlagGo2, 912, &s_ok)) {
        for (long long i = tid; i < all4; i += nthreads) a.out[i] = make_float4(nan, nan, nan, nan);
        return;
    }
    const long long before4 = (long long)u0 * a.s4, after4 = (long long)u1 * a.s4;
    for (long long i = tid; i < all4 - own4; i += nthreads) {
        const long long at = i < before4 ? i : i + (after4 - before4);
        const int owner = (int)(at / a.s4) / a.units_per_rank;
        a.out[at] = __ldcg(a.full[owner] + at);
    }
}

struct PeerTable {
    const float4* buf[kMaxWorld];
    unsigned int* flag[kMaxWorld];
};

__global__ void __launch_bounds__(kPeerThreads)
peer_state_sum_kernel(PeerTable t, int world, int rank, long long n4, unsigned int epoch, float4* __restrict__ out,
                      int* status, unsigned long long wait_ns) {
    __shared__ int gave_up;
    if (threadIdx.x == 0) gave_up = 0;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x < world && (int)threadIdx.x != rank) {
        __threadfence_system();
        st_relaxed_sys(t.flag[threadIdx.x] + rank, epoch);
    }
    if (threadIdx.x < world && (int)threadIdx.x != rank) {
        const unsigned int* mine = t.flag[rank] + threadIdx.x;
        const unsigned long long t0 = global_ns();
        int spins = 0;
        while ((int)(ld_relaxed_sys(mine) - epoch) < 0) {
            if ((++spins & 7) == 0 && global_ns() - t0 > wait_ns) {
                gave_up = 1;
                if (status != nullptr) *status = 901;
                break;
            }
        }
        __threadfence_system();
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

// CTAs of the piece-sum kernel that are resident at the same time (its CTAs wait for one another in the
// two-round form, so the grid must not be larger).
int resident_blocks() {
    static int cached[64] = {0};
    int sms = 0, dev = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 64;
    if (cached[dev] == 0) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 64;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_piece_sum_kernel, kPeerThreads, 0) != cudaSuccess ||
            per_sm < 1)
            per_sm = 1;
        cached[dev] = sms * per_sm;
    }
    return cached[dev];
}

}  // namespace

cudaError_t peer_piece_sum(const PeerArgs& g, const PieceLayout& lay, int state_stride, int two_round, float* out,
                           cudaStream_t st) {
    PieceSum a{};
    for (int r = 0; r < g.world; ++r) {
        a.parts[r] = static_cast<const float4*>(g.parts[r]);
        a.full[r] = static_cast<float4*>(g.full[r]);
        a.flags[r] = static_cast<unsigned int*>(g.flags[r]);
    }
    a.world = g.world;
    a.rank = g.rank;
    a.epoch = g.epoch;
    a.units = lay.units;
    a.units_per_rank = (lay.units + g.world - 1) / g.world;
    a.slots = lay.slots;
    a.tiles_per_unit = lay.tiles_per_unit;
    a.tiles_per_cta = lay.tiles_per_cta;
    a.s4 = state_stride / 4;
    a.two_round = two_round;
    a.out = reinterpret_cast<float4*>(out);
    a.wait_ns = tc_peer_wait_ns();
    a.status = tc_status_word();
    long long blocks = ((long long)lay.units * a.s4 + kPeerThreads - 1) / kPeerThreads;
    const int cap = resident_blocks();
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(kPeerThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool plain = [] {                      // FBLA_NO_PDL=1: ordinary launches everywhere
        const char* e = getenv("FBLA_NO_PDL");
        return e != nullptr && e[0] == '1';
    }();
    cfg.numAttrs = plain ? 0 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, peer_piece_sum_kernel, a);
    note_launches(1);
    return e != cudaSuccess ? e : cudaGetLastError();
}

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
