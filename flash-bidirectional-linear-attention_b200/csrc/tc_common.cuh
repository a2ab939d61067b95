// Shared pieces of the tensor-core kernels: the kernel parameter block, the static tile
// schedule, and small device helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fbla_common.cuh"
#include "tc_ptx.cuh"

namespace fbla {
namespace tc {

#ifndef FBLA_PREFETCH_TILES
#define FBLA_PREFETCH_TILES 0
#endif
constexpr int kTileTokens = 128;      // tokens per tile = rows of one MMA
constexpr int kBlockBytes = 16384;    // one [128 tokens][64 features] 16-bit block in shared memory
constexpr int kThreads = 192;         // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue
constexpr int kEpiThreads = 128;
constexpr int kSmemLimit = 227 * 1024;
// Packed layout: every kernel keeps the tile plan (one int per sequence + 1) at the end of its
// dynamic shared memory, so at most kMaxPackedSeqs sequences per call take the tensor-core path.
constexpr int kPlanBytes = 8192;
constexpr int kMaxPackedSeqs = kPlanBytes / 4 - 1;

// Operator variant a kernel is instantiated for.
constexpr int kSimple = 0;      // no normaliser
constexpr int kLinear = 1;      // normalised, one q / k
constexpr int kDecoupled = 2;   // normalised, rotary q/k in the numerator

// Static schedule: the tiles of all units form one list (unit-major); CTA c owns the
// contiguous range [c * tiles_per_cta, (c+1) * tiles_per_cta).  A maximal run of tiles of one
// unit inside a CTA's range is a segment; reducing kernels emit one partial per segment into
// slot (unit, c - first_cta(unit)).
struct Schedule {
    int units;
    int tiles_per_unit;
    int total_tiles;
    int tiles_per_cta;
    int slots_per_unit;   // upper bound on segments per unit
    int ctas;
};

__host__ __device__ inline int first_cta_of_unit(const Schedule& s, int unit) {
    return (int)(((long long)unit * s.tiles_per_unit) / s.tiles_per_cta);
}
__host__ __device__ inline int last_cta_of_unit(const Schedule& s, int unit) {
    return (int)((((long long)unit + 1) * s.tiles_per_unit - 1) / s.tiles_per_cta);
}

// Sequence sharding over the GPUs of one node: how the per-segment states of this rank reach the
// ranks that add them, and how the sums come back.  Unit u is summed by its owner, rank
// u / units_per_rank.
//   recv[r]  : rank r's receive buffer, [world][units_per_rank][slots_per_unit][state_stride] fp32 --
//              the reducing pass of rank q stores the pieces of a unit that r owns into block q of
//              recv[r] (plain stores to the peer's memory);
//   full[r]  : rank r's copy of the summed state of ALL units, [units][state_stride] fp32 -- the head
//              of the consuming pass adds the pieces of its own units (ranks in order, pieces in CTA
//              order, so every rank ends up with the same bits) and stores the sums into full[] of
//              every rank;
//   flags[r] : rank r's flag words: [0, 8) "the reducing pass of rank q has stored all its pieces",
//              [16, 24) "rank q has stored the sums of its units", [32], [33] CTA tickets of the
//              local kernels.  Flags carry the exchange number `epoch` (1, 2, 3, ...).
// world == 1 switches all of it off.  The kernels take it as a kernel parameter of its own (its pointer
// tables are indexed with run-time values, which a by-value copy of the parameters would pay for with
// local memory).
constexpr int kMaxPeers = 8;
struct PeerXchg {
    int world, rank;
    int units_per_rank;
    unsigned int epoch;
    unsigned long long wait_ns;     // limit of every wait for a peer
    float* recv[kMaxPeers];
    float* full[kMaxPeers];
    unsigned int* flags[kMaxPeers];
    float* state_copy;              // consuming pass: private copy of the summed state (may be null)
    unsigned long long* trace;      // measurement aid (may be null): 16 timestamps of this exchange, written by
                                    // one thread per kernel: [0] last CTA of the reducing pass signals,
                                    // [8..12] consuming pass, CTA 0: gather entered, pieces of all ranks in
                                    // place, own sums stored, sums of all ranks in place, private copy done
};

struct Params {
    Schedule sch;
    int seq_len;          // tokens per unit
    float scale;
    float inv_norm;       // 1 / (length the key sum is divided by)
    float eps;
    int is_bf16;          // 1: bf16, 0: fp16
    int* status;          // host-visible status word (0 = ok)
    // forward state / backward state: per-segment partials; others: the reduced state
    float* part;
    float* state_out;     // packed layout: reducing kernels write whole-unit states here directly
    const float* state;
    const float* state_parts;   // non-null: `state` is not used, the consuming pass adds the per-segment pieces itself
    int state_stride;     // floats per unit in state / partial slots
    // kernels that write an output with plain global stores (no staged tile): its base address
    void* out_a;
    void* out_b;
    // packed variable-length layout (total_tokens, heads, D); all null / zero for fixed length
    const int32_t* cu;    // cu_seqlens, device
    const int32_t* plan;  // plan[s] = heads * (tiles of sequences before s), plan[num_seqs] = all tiles
    int num_seqs;
    int heads;
    int scale_per_seq;    // scale = 1 / length of the sequence
    float inv_norm_fixed; // > 0: divide the key sum by this length for every sequence; 0: by its own
};

// The state of one unit as a consuming pass reads it: one vector, or the per-segment pieces that the
// reducing pass left (added here in CTA order, the order tc_reduce_partials_kernel uses, so both
// routes give the same bits).
// All loads bypass L1 (every element is read once, and the state may have been written by another
// GPU, with which only L2 is coherent).
struct StateSrc {
    const float* p;
    int n;
    size_t stride;
    __device__ __forceinline__ float operator[](int i) const {
        float a = __ldcg(p + i);
        for (int j = 1; j < n; ++j) a += __ldcg(p + (size_t)j * stride + i);
        return a;
    }
    // N values first + u * step (u = 0..N-1) at once: all loads of one piece are in flight together
    // before the next piece is added (the sum per element still runs in piece order).
    template <int N>
    __device__ __forceinline__ void load(int first, int step, float (&x)[N]) const {
#pragma unroll
        for (int u = 0; u < N; ++u) x[u] = __ldcg(p + first + u * step);
        for (int j = 1; j < n; ++j) {
            const float* pj = p + (size_t)j * stride;
            float y[N];
#pragma unroll
            for (int u = 0; u < N; ++u) y[u] = __ldcg(pj + first + u * step);
#pragma unroll
            for (int u = 0; u < N; ++u) x[u] += y[u];
        }
    }
    template <int N>
    __device__ __forceinline__ void load2(int first, int step, float2 (&x)[N]) const {    // first, step even
#pragma unroll
        for (int u = 0; u < N; ++u) x[u] = __ldcg(reinterpret_cast<const float2*>(p + first + u * step));
        for (int j = 1; j < n; ++j) {
            const float* pj = p + (size_t)j * stride;
            float2 y[N];
#pragma unroll
            for (int u = 0; u < N; ++u) y[u] = __ldcg(reinterpret_cast<const float2*>(pj + first + u * step));
#pragma unroll
            for (int u = 0; u < N; ++u) {
                x[u].x += y[u].x;
                x[u].y += y[u].y;
            }
        }
    }
    __device__ __forceinline__ float2 pair(int i) const {     // i even
        float2 a = __ldcg(reinterpret_cast<const float2*>(p + i));
        for (int j = 1; j < n; ++j) {
            const float2 b = __ldcg(reinterpret_cast<const float2*>(p + (size_t)j * stride + i));
            a.x += b.x;
            a.y += b.y;
        }
        return a;
    }
};
__device__ __forceinline__ StateSrc state_source(const Params& p, int unit) {
    StateSrc s;
    if (p.state_parts != nullptr) {
        s.p = p.state_parts + (size_t)unit * p.sch.slots_per_unit * p.state_stride;
        s.n = last_cta_of_unit(p.sch, unit) - first_cta_of_unit(p.sch, unit) + 1;
    } else {
        s.p = p.state + (size_t)unit * p.state_stride;
        s.n = 1;
    }
    s.stride = (size_t)p.state_stride;
    return s;
}

// One 128-token tile of the work list, as every role of a kernel sees it.
struct Tile {
    int unit;          // state index
    int tile;          // index of the tile inside its unit
    int c1, c2;        // TMA coordinates after the feature coordinate
    int valid;         // tokens of the tile that belong to the unit (1..128)
    long long row0;    // row of the tile's first token in the (rows, D) view of the tensor
    int row_stride;    // rows between consecutive tokens (1, or heads when packed)
    bool first, last;  // first / last tile of a segment (run of one unit inside this CTA's range)
    bool starts_here, ends_here;   // the unit's first / last tile lies inside this CTA's range
    float scale, inv_norm;
};

// plan[s] = number of 128-token tiles of the sequences before s (per head), plan[num_seqs] = all of
// them; built by every CTA for itself from cu_seqlens (all threads of the block must call this).
__device__ __forceinline__ void build_plan(int32_t* plan, const int32_t* __restrict__ cu, int num_seqs) {
    for (int i = threadIdx.x; i <= num_seqs; i += blockDim.x) plan[i] = cu[i];
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, prev = plan[0];
        for (int s = 0; s < num_seqs; ++s) {
            const int next = plan[s + 1];
            plan[s] = acc;
            acc += (next - prev + kTileTokens - 1) / kTileTokens;
            prev = next;
        }
        plan[num_seqs] = acc;
    }
    __syncthreads();
}

template <bool VARLEN>
struct TileMap;

template <>
struct TileMap<false> {
    __device__ static __forceinline__ void range(const Params& p, int& g0, int& g1) {
        g0 = blockIdx.x * p.sch.tiles_per_cta;
        g1 = min(p.sch.total_tiles, g0 + p.sch.tiles_per_cta);
    }
    __device__ static __forceinline__ Tile get(const Params& p, int g, int g0, int g1) {
        Tile t;
        const int tpu = p.sch.tiles_per_unit;
        t.unit = g / tpu;
        t.tile = g - t.unit * tpu;
        t.c1 = t.tile * kTileTokens;
        t.c2 = t.unit;
        t.valid = min(kTileTokens, p.seq_len - t.c1);
        t.row0 = (long long)t.unit * p.seq_len + t.c1;
        t.row_stride = 1;
        t.first = (g == g0) || t.tile == 0;
        t.last = (g == g1 - 1) || t.tile == tpu - 1;
        t.starts_here = (g - t.tile) >= g0;
        t.ends_here = (g - t.tile + tpu) <= g1;
        t.scale = p.scale;
        t.inv_norm = p.inv_norm;
        return t;
    }
};

// Packed layout.  Token rows of one head are heads*D elements apart, so the heads of a token share
// DRAM pages: CTA c works on head c % heads, and the heads*G CTAs of a launch split the per-head tile
// list into G = gridDim.x / heads contiguous ranges, so that at any time the CTAs of a group stream
// the same tokens (one head each).  Tile index g below counts tiles of ONE head.
template <>
struct TileMap<true> {
    __device__ static __forceinline__ void range(const Params& p, int& g0, int& g1) {
        const int total = p.plan[p.num_seqs];
        const int groups = (int)gridDim.x / p.heads;
        const int grp = (int)blockIdx.x / p.heads;
        const int per = (total + groups - 1) / groups;
        g0 = min(total, grp * per);
        g1 = min(total, g0 + per);
    }
    __device__ static __forceinline__ Tile get(const Params& p, int g, int g0, int g1) {
        // sequence s with plan[s] <= g < plan[s+1]
        int lo = 0, hi = p.num_seqs;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.plan[mid] <= g) lo = mid; else hi = mid;
        }
        const int s = lo;
        const int a0 = p.plan[s];
        const int nt = p.plan[s + 1] - a0;
        const int h = (int)blockIdx.x % p.heads;
        Tile t;
        t.tile = g - a0;
        t.unit = s * p.heads + h;
        const int bos = p.cu[s];
        const int len = p.cu[s + 1] - bos;
        t.c1 = h;
        t.c2 = bos + t.tile * kTileTokens;
        t.valid = min(kTileTokens, len - t.tile * kTileTokens);
        t.row0 = (long long)t.c2 * p.heads + h;
        t.row_stride = p.heads;
        t.first = (g == g0) || t.tile == 0;
        t.last = (g == g1 - 1) || t.tile == nt - 1;
        t.starts_here = a0 >= g0;
        t.ends_here = (a0 + nt) <= g1;
        const float inv_len = 1.f / (float)len;
        t.scale = p.scale_per_seq ? inv_len : p.scale;
        t.inv_norm = p.inv_norm_fixed > 0.f ? p.inv_norm_fixed : inv_len;
        return t;
    }
};

// Where a reducing kernel puts the state of a finished segment.
//   fixed length : slot (unit, cta - first_cta(unit)) of the partial buffer, added by
//                  tc_reduce_partials_kernel.
//   packed       : a unit that lies wholly inside this CTA's range goes straight to the state; a
//                  piece of a unit that started in an earlier CTA goes to partial slot (cta, 0), a
//                  unit that starts here but continues in the next CTA to slot (cta, 1);
//                  tc_reduce_varlen_kernel adds the pieces in CTA order.
template <bool VARLEN>
__device__ __forceinline__ float* segment_destination(const Params& p, const PeerXchg& px, const Tile& t,
                                                      float* state_out) {
    if (!VARLEN) {
        const int piece = (int)blockIdx.x - first_cta_of_unit(p.sch, t.unit);
        if (px.world > 1) {
            // sequence-sharded: straight into the receive buffer of the rank that sums this unit
            const int owner = t.unit / px.units_per_rank;
            const int local = t.unit - owner * px.units_per_rank;
            const size_t slot = ((size_t)px.rank * px.units_per_rank + local) * p.sch.slots_per_unit + piece;
            return px.recv[owner] + slot * p.state_stride;
        }
        const int slot = t.unit * p.sch.slots_per_unit + piece;
        return p.part + (size_t)slot * p.state_stride;
    }
    if (t.starts_here && t.ends_here) return state_out + (size_t)t.unit * p.state_stride;
    return p.part + ((size_t)blockIdx.x * 2 + (t.starts_here ? 1 : 0)) * p.state_stride;
}


__device__ __forceinline__ uint32_t pack2(float a, float b, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack2(uint32_t u, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
        return __bfloat1622float2(h);
    }
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
}
__device__ __forceinline__ uint16_t pack1(float a, int is_bf16) {
    if (is_bf16) {
        __nv_bfloat16 h = __float2bfloat16_rn(a);
        return *reinterpret_cast<uint16_t*>(&h);
    }
    __half h = __float2half_rn(a);
    return *reinterpret_cast<uint16_t*>(&h);
}
__device__ __forceinline__ float unpack1(uint16_t u, int is_bf16) {
    if (is_bf16) return __bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&u));
    return __half2float(*reinterpret_cast<__half*>(&u));
}

// Copies a finished [DK x DV] fp32 accumulator (rows = key features) from tensor memory to a
// partial slot in global memory, plus one extra per-row value (the sum of NVEC columns starting
// at column `vec_col`) stored after the matrix.  Executed by the four epilogue warps.  With
// M = 128 accumulator row r sits in TMEM lane r; with M = 64 it sits in lane (r % 16) + 32 * (r / 16).
template <int DK, int DV, int NVEC>
__device__ __forceinline__ void drain_state_acc(uint32_t tmem_acc, uint32_t vec_col, float* out, int warp, int lane) {
    const int quarter = warp & 3;
    const int row = DK == 128 ? quarter * 32 + lane : quarter * 16 + lane;
    const bool row_ok = DK == 128 ? true : lane < 16;
    const uint32_t t_lane = tmem_acc + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
    for (int c0 = 0; c0 < DV; c0 += 32) {
        float v[32];
        ptx::tmem_ld32(t_lane + c0, v);
        ptx::tmem_ld_wait();
        if (row_ok) {
            float4* dst = reinterpret_cast<float4*>(out + row * DV + c0);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
    }
    if (NVEC > 0) {
        float v[16];
        ptx::tmem_ld16(t_lane + vec_col, v);
        ptx::tmem_ld_wait();
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NVEC; ++j) s += v[j];
        if (row_ok) out[DK * DV + row] = s;
    }
}

// ---- sequence sharding: flags and sums over peer memory ---------------------------------------------
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Cycles an in-CTA wait may last: a CTA of a sequence-sharded call may sit behind a wait for peer
// GPUs, so its own waits must outlast that one (about two cycles per nanosecond).
__device__ __forceinline__ long long wait_limit(const PeerXchg& px) {
    return px.world > 1 ? ptx::kWaitCycles + 2 * (long long)px.wait_ns : ptx::kWaitCycles;
}
// Barrier among the 128 epilogue threads only (the other warps of the CTA are in their own loops).
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// The same barrier, returning to every thread whether ANY of the 128 passed a true predicate: a
// decision all of them take the same way (threads that left on different sides of it would meet at
// different barriers afterwards).
__device__ __forceinline__ bool epilogue_barrier_any(bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "bar.red.or.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}"
        : "=r"(out)
        : "r"((uint32_t)pred)
        : "memory");
    return out != 0;
}

// Waits until *flag has reached `epoch`, at most px.wait_ns; on giving up records `site` in the CTA's
// abort flag and in the library's status word and returns false.
__device__ __forceinline__ bool peer_wait(const unsigned int* flag, const PeerXchg& px, const ptx::Abort& ab,
                                          int site) {
    if ((int)(ld_acquire_sys(flag) - px.epoch) >= 0) return true;
    const unsigned long long t0 = global_ns();
    int spins = 0;
    while ((int)(ld_acquire_sys(flag) - px.epoch) < 0) {
        if ((++spins & 15) == 0) {
            if (*ab.cta_flag != 0) return false;
            if (global_ns() - t0 > px.wait_ns) {
                *ab.cta_flag = site;
                *ab.status = site;
                __threadfence_system();
                return false;
            }
        }
    }
    return true;
}

// End of a reducing pass of a sequence-sharded call, executed by ONE thread per CTA after every
// thread that stored pieces has executed __threadfence_system() and the CTA has synchronised: the
// last CTA of this rank to get here tells every rank that this rank's pieces are in place.
__device__ __forceinline__ void peer_signal_pieces(const PeerXchg& px) {
    unsigned int* mine = px.flags[px.rank];
    __threadfence();
    const unsigned int ticket = atomicAdd(mine + 32, 1u);
    if (ticket == gridDim.x - 1) {
        mine[32] = 0;                       // every CTA has drawn: ready for the next launch
        __threadfence_system();
        for (int r = 0; r < px.world; ++r) st_release_sys(px.flags[r] + px.rank, px.epoch);
        if (px.trace != nullptr) px.trace[0] = global_ns();
    }
}

// Head of a consuming pass of a sequence-sharded call, executed by the 128 epilogue threads of every
// CTA (et = 0..127) before the first state is staged:
//   1. wait until every rank's reducing pass has stored its pieces;
//   2. add the pieces of the units this rank owns -- ranks in order, pieces in CTA order -- and store
//      each sum into full[] of every rank (the CTAs of the grid share the elements);
//   3. the last CTA to finish tells every rank; wait until every rank has said so;
//   4. optionally copy the summed state of all units to private memory (the caller keeps it for the
//      backward; full[] is overwritten two exchanges later).
// Afterwards p.state (= full[rank]) is complete.  The CTAs of one launch wait for one another in step
// 3, so the grid must be resident as a whole (one CTA per SM at most, which the schedule guarantees).
// Returns false when a wait gave up.
__device__ __forceinline__ bool peer_gather_state(const Params& p, const PeerXchg& x, const ptx::Abort& ab, int et,
                                                  int site) {
    unsigned int* mine = x.flags[x.rank];
    const bool tracer = x.trace != nullptr && blockIdx.x == 0 && et == 0;
    if (tracer) x.trace[8] = global_ns();
    if (et < x.world) peer_wait(mine + et, x, ab, site);
    if (epilogue_barrier_any(*ab.cta_flag != 0)) return false;
    if (tracer) x.trace[9] = global_ns();
    const int s4 = p.state_stride >> 2;                       // float4 per unit (the stride is a multiple of 4)
    const int u0 = x.rank * x.units_per_rank;
    const int u1 = min(p.sch.units, u0 + x.units_per_rank);
    const long long n4 = (long long)max(0, u1 - u0) * s4;
    for (long long i = (long long)blockIdx.x * kEpiThreads + et; i < n4; i += (long long)gridDim.x * kEpiThreads) {
        const int ul = (int)(i / s4), e4 = (int)(i - (long long)ul * s4);
        const int u = u0 + ul;
        const int n = last_cta_of_unit(p.sch, u) - first_cta_of_unit(p.sch, u) + 1;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < x.world; ++q) {
            const float4* src = reinterpret_cast<const float4*>(
                                    x.recv[x.rank] + ((size_t)q * x.units_per_rank + ul) * p.sch.slots_per_unit * p.state_stride) + e4;
            for (int j = 0; j < n; ++j) {
                const float4 y = __ldcg(src + (size_t)j * s4);
                acc.x += y.x; acc.y += y.y; acc.z += y.z; acc.w += y.w;
            }
        }
        for (int r = 0; r < x.world; ++r)
            reinterpret_cast<float4*>(x.full[r] + (size_t)u * p.state_stride)[e4] = acc;
    }
    __threadfence_system();
    epilogue_barrier();
    if (tracer) x.trace[10] = global_ns();
    if (et == 0) {
        const unsigned int ticket = atomicAdd(mine + 33, 1u);
        if (ticket == gridDim.x - 1) {
            mine[33] = 0;
            __threadfence_system();
            for (int r = 0; r < x.world; ++r) st_release_sys(x.flags[r] + 16 + x.rank, x.epoch);
        }
    }
    if (et < x.world) peer_wait(mine + 16 + et, x, ab, site + 1);
    if (epilogue_barrier_any(*ab.cta_flag != 0)) return false;
    if (tracer) x.trace[11] = global_ns();
    if (x.state_copy != nullptr) {
        const long long all4 = (long long)p.sch.units * s4;
        const float4* src = reinterpret_cast<const float4*>(x.full[x.rank]);
        float4* dst = reinterpret_cast<float4*>(x.state_copy);
        for (long long i = (long long)blockIdx.x * kEpiThreads + et; i < all4; i += (long long)gridDim.x * kEpiThreads)
            dst[i] = __ldcg(src + i);
    }
    if (x.trace != nullptr) {
        epilogue_barrier();                 // all 128 threads: the copy of this CTA is complete
        if (tracer) x.trace[12] = global_ns();
    }
    return true;
}

// Dynamic shared memory starts at an address the swizzled tiles can use (1024-byte aligned).
__device__ __forceinline__ uint8_t* align_1024(uint8_t* p) {
    const uint32_t a = ptx::smem_u32(p);
    return p + ((1024u - (a & 1023u)) & 1023u);
}

}  // namespace tc
}  // namespace fbla
