// Tensor-core kernels of the forward direction.
//
//   tc_fwd_state_kernel : [ S = Kr^T V | sum_t k ] per segment.  TMA streams 128-token tiles of
//       k (kr) and v through a ring of shared-memory stages; one thread issues, per 16 tokens,
//       tcgen05.mma with BOTH operands MN-major (the tiles are token-major, the contraction
//       runs over tokens) accumulating fp32 in TMEM; the key sum is a second MMA of the key
//       tile against a tile of ones.  HBM traffic: k and v once.
//   tc_fwd_out_kernel   : o = (qr . scale*S) / (q . kmean + eps).  The bf16 state (and the key
//       mean split in a high and a low 16-bit part, as two extra columns) sits in shared
//       memory as the K-major B operand; per tile one MMA gives numerator and normaliser, the
//       epilogue divides, converts and hands the tile to a TMA store.  HBM traffic: q once, o once.
#pragma once

#include "tc_common.cuh"

#ifndef FBLA_FWD_STATE_SMEM_KB
#define FBLA_FWD_STATE_SMEM_KB 128
#endif

namespace fbla {
namespace tc {

// ------------------------------------------------------------------------------------------
template <int DK, int DV, int MODE>
struct FwdStateCfg {
    static constexpr int kKB = DK / 64, kVB = DV / 64;
    static constexpr int kStageBlocks = kKB + kVB + (MODE == kDecoupled ? kKB : 0);
    static constexpr int kStageBytes = kStageBlocks * kBlockBytes;
    static constexpr int kStages = (FBLA_FWD_STATE_SMEM_KB * 1024) / kStageBytes < 8 ? (FBLA_FWD_STATE_SMEM_KB * 1024) / kStageBytes : 8;
    // The key sum is K^T . ones.  With dv = 64 (and k the same tensor as kr) the ones are a full
    // 128-token block that the B descriptor reaches as the N-block after the v tile, so state and
    // key sum come from ONE MMA per 16 tokens (N = dv + 16) and the key tile is read once.
    // Otherwise a small ones tile feeds a second MMA (N = 16).
    static constexpr bool kMergedSum = (MODE == kLinear && DV == 64);
    static constexpr int kOnesBytes = kMergedSum ? kBlockBytes : 1024;
    static constexpr int kTmemCols = (DV + 16) <= 128 ? 128 : 256;
    static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kOnesBytes + 256 + kPlanBytes;
};

// Zeroes the rows [valid, 128) of `nblocks` swizzled [128][64] blocks (a tile whose tail belongs to
// the next packed sequence); executed by the 128 epilogue threads.
__device__ __forceinline__ void zero_tail_rows(uint8_t* blocks, int nblocks, int valid, int et) {
    const int rows = kTileTokens - valid;
    for (int i = et; i < nblocks * rows * 8; i += kEpiThreads) {
        const int b = i / (rows * 8), r = (i / 8) % rows, c = i & 7;
        *reinterpret_cast<uint4*>(blocks + b * kBlockBytes + (valid + r) * 128 + c * 16) = make_uint4(0, 0, 0, 0);
    }
}

template <int DK, int DV, int MODE, bool BF16, bool VARLEN>
__global__ void __launch_bounds__(kThreads, 1)
tc_fwd_state_kernel(const __grid_constant__ CUtensorMap tm_kr, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const Params p_in) {
    using Cfg = FwdStateCfg<DK, DV, MODE>;
    using Map = TileMap<VARLEN>;
    constexpr int NS = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_1024(smem_raw);
    uint8_t* stages = smem;
    uint8_t* ones = stages + NS * Cfg::kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(ones + Cfg::kOnesBytes);
    uint64_t* full = bars;              // [NS] TMA -> MMA
    uint64_t* empty = bars + NS;        // [NS] MMA -> TMA
    uint64_t* fixed = bars + 2 * NS;    // [NS] packed layout: tail rows of the stage zeroed
    uint64_t* acc_full = bars + 3 * NS; // MMA -> epilogue (segment finished)
    uint64_t* acc_empty = acc_full + 1; // epilogue -> MMA (accumulator drained)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ptx::griddep_launch();
    Params pv = p_in;
    if (VARLEN) {
        ptx::griddep_wait();                // cu_seqlens may come from the previous kernel
        int32_t* plan = reinterpret_cast<int32_t*>(smem_raw + (Cfg::kSmemBytes - kPlanBytes));
        build_plan(plan, p_in.cu, p_in.num_seqs);
        pv.plan = plan;
    }
    const Params& p = pv;
    int g0, g1;
    Map::range(p, g0, g1);
    const ptx::Abort ab{cta_abort, p.status};

    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; ++i) {
            ptx::mbar_init(&full[i], 1);
            ptx::mbar_init(&empty[i], 1);
            ptx::mbar_init(&fixed[i], kEpiThreads);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, kEpiThreads);
        *cta_abort = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tm_kr);
        ptx::prefetch_tensormap(&tm_v);
    }
    // a tile of ones (any layout of ones is ones): B operand of the key-sum MMA
    for (int i = threadIdx.x; i < Cfg::kOnesBytes / 2; i += kThreads)
        reinterpret_cast<uint16_t*>(ones)[i] = BF16 ? (uint16_t)0x3F80 : (uint16_t)0x3C00;
    ptx::fence_proxy_async_smem();
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (!VARLEN) ptx::griddep_wait();       // everything above overlaps the previous kernel's tail

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            if (!ptx::mbar_wait(&empty[s], ph ^ 1u, ab, 101)) break;
            ptx::mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
            const Tile t = Map::get(p, g, g0, g1);
            uint8_t* st = stages + s * Cfg::kStageBytes;
#pragma unroll
            for (int b = 0; b < Cfg::kKB; ++b) ptx::tma_load_3d(st + b * kBlockBytes, &tm_kr, &full[s], b * 64, t.c1, t.c2);
#pragma unroll
            for (int b = 0; b < Cfg::kVB; ++b)
                ptx::tma_load_3d(st + (Cfg::kKB + b) * kBlockBytes, &tm_v, &full[s], b * 64, t.c1, t.c2);
            if (MODE == kDecoupled) {
#pragma unroll
                for (int b = 0; b < Cfg::kKB; ++b)
                    ptx::tma_load_3d(st + (Cfg::kKB + Cfg::kVB + b) * kBlockBytes, &tm_k, &full[s], b * 64, t.c1, t.c2);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc_s = ptx::instr_desc(DK, Cfg::kMergedSum ? DV + 16 : DV, BF16, true, true);
        const uint32_t idesc_k = ptx::instr_desc(DK, 16, BF16, true, false);
        const uint32_t ones_base = ptx::smem_u32(ones);
        const uint64_t d_ones = ptx::smem_desc(ptx::smem_u32(ones), 128, 256, ptx::kLayoutNone);
        int seg = 0;
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            const Tile t = Map::get(p, g, g0, g1);
            const bool first = t.first, last = t.last;
            if (first && !ptx::mbar_wait(acc_empty, ((uint32_t)seg & 1u) ^ 1u, ab, 111)) break;
            // packed layout: the epilogue warps hand the stage over once its tail rows are zero
            if (!ptx::mbar_wait(VARLEN ? &fixed[s] : &full[s], ph, ab, 112)) break;
            ptx::tc_fence_after_sync();
            const uint32_t a_base = ptx::smem_u32(stages + s * Cfg::kStageBytes);
            const uint32_t b_base = a_base + Cfg::kKB * kBlockBytes;
            const uint32_t k_base = MODE == kDecoupled ? b_base + Cfg::kVB * kBlockBytes : a_base;
#pragma unroll
            for (int ks = 0; ks < kTileTokens / 16; ++ks) {
                const bool acc = !(first && ks == 0);
                const uint64_t da = ptx::smem_desc(a_base + ks * 2048, kBlockBytes, 1024, ptx::kLayoutSw128);
                // merged: the N-block after the v tile (leading byte offset) is the block of ones
                const uint64_t db = ptx::smem_desc(b_base + ks * 2048, Cfg::kMergedSum ? ones_base - b_base : kBlockBytes,
                                                   1024, ptx::kLayoutSw128);
                ptx::mma_ss(tmem, da, db, idesc_s, acc);
                if (MODE != kSimple && !Cfg::kMergedSum) {
                    const uint64_t dk = ptx::smem_desc(k_base + ks * 2048, kBlockBytes, 1024, ptx::kLayoutSw128);
                    ptx::mma_ss(tmem + DV, dk, d_ones, idesc_k, acc);
                }
            }
            ptx::mma_commit(&empty[s]);
            if (last) {
                ptx::mma_commit(acc_full);
                ++seg;
            }
        }
    } else if (warp >= 2) {
        // ---------------- epilogue: drain the accumulator of each finished segment ----------------
        const int et = threadIdx.x - 64;
        int seg = 0;
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const Tile t = Map::get(p, g, g0, g1);
            if (VARLEN) {
                const int s = it % NS;
                if (!ptx::mbar_wait(&full[s], (uint32_t)(it / NS) & 1u, ab, 122)) break;
                if (t.valid < kTileTokens) {
                    zero_tail_rows(stages + s * Cfg::kStageBytes, Cfg::kStageBlocks, t.valid, et);
                    ptx::fence_proxy_async_smem();
                }
                ptx::mbar_arrive(&fixed[s]);
            }
            if (!t.last) continue;
            if (!ptx::mbar_wait(acc_full, (uint32_t)seg & 1u, ab, 121)) break;
            ptx::tc_fence_after_sync();
            float* out = segment_destination<VARLEN>(p, t, p.state_out);
            drain_state_acc<DK, DV, (MODE != kSimple ? 1 : 0)>(tmem, DV, out, warp, lane);
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(acc_empty);
            ++seg;
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

// Packed layout: block b = (group, head) adds the pieces of the unit that starts inside its tile
// range and continues into later groups of the same head (slot (b, 1), then slot (b + heads*j, 0)
// for every later group the unit reaches), in group order, and writes the unit's state.
// `ctas` = grid size of the producing kernel.
__global__ void __launch_bounds__(256)
tc_reduce_varlen_kernel(const Params p_in, float* __restrict__ state, int ctas) {
    __shared__ int32_t plan_s[kMaxPackedSeqs + 1];
    build_plan(plan_s, p_in.cu, p_in.num_seqs);
    const Params& p = p_in;
    const int total = plan_s[p.num_seqs];
    if (total == 0) return;
    const int groups = ctas / p.heads;
    const int per = (total + groups - 1) / groups;
    const int b = blockIdx.x, grp = b / p.heads, h = b % p.heads;
    const int g0 = min(total, grp * per), g1 = min(total, g0 + per);
    if (g1 <= g0) return;
    const int g = g1 - 1;                               // the unit of this CTA's last tile
    int lo = 0, hi = p.num_seqs;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (plan_s[mid] <= g) lo = mid; else hi = mid;
    }
    const int us = plan_s[lo], ue = plan_s[lo + 1];     // per-head tile range of the sequence
    if (ue <= g1 || us < g0) return;                   // complete here, or owned by an earlier group
    const int unit = lo * p.heads + h;
    const int stride = p.state_stride;
    for (int e = threadIdx.x; e < stride; e += 256) {
        float s = p.part[((size_t)b * 2 + 1) * stride + e];
        for (int gg = grp + 1; gg < groups && gg * per < ue; ++gg)
            s += p.part[((size_t)(gg * p.heads + h) * 2) * stride + e];
        state[(size_t)unit * stride + e] = s;
    }
}

// Adds the per-segment partials of every unit, in CTA order (deterministic).
__global__ void __launch_bounds__(256)
tc_reduce_partials_kernel(const float* __restrict__ part, float* __restrict__ state, Schedule sch, int stride) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)sch.units * stride) return;
    const int unit = (int)(i / stride);
    const int e = (int)(i - (long long)unit * stride);
    const int n = last_cta_of_unit(sch, unit) - first_cta_of_unit(sch, unit) + 1;
    const float* src = part + (size_t)unit * sch.slots_per_unit * stride + e;
    float s = 0.f;
    for (int j = 0; j < n; ++j) s += src[(size_t)j * stride];
    state[i] = s;
}

// ------------------------------------------------------------------------------------------
template <int DK, int DV, int MODE>
struct FwdOutCfg {
    static constexpr int kKB = DK / 64, kVB = DV / 64;
    // B operand, per 64-wide K block: [dv rows: high part of scale*S^T][dv rows: rounding residual]
    // [16 rows: kmean high, kmean low, zeros].  With dv = 64 the three groups are the N range of ONE
    // MMA (N = 144): the accumulator holds [num_hi | num_lo | z] and the epilogue adds the halves.
    // With dv = 128 that would exceed N = 256, so high and residual accumulate into the same columns.
    static constexpr bool kWide = (DV == 64);
    static constexpr int kZRows = MODE != kSimple ? 16 : 0;
    static constexpr int kBopBlock = (2 * DV + kZRows) * 128;            // bytes per 64-wide K block
    static constexpr int kBopBytes = ((kKB * kBopBlock + 1023) / 1024) * 1024;
    static constexpr int kZCol = kWide ? 2 * DV : DV;                     // accumulator column of z
    static constexpr int kStageBlocks = kKB * (MODE == kDecoupled ? 2 : 1);
    static constexpr int kStageBytes = kStageBlocks * kBlockBytes;
    static constexpr int kOutBytes = kVB * kBlockBytes;                   // one staged output tile
    static constexpr int kAvail = 200 * 1024 - kBopBytes - 2 * kOutBytes;
    static constexpr int kStages = kAvail / kStageBytes < 8 ? kAvail / kStageBytes : 8;
    static constexpr int kAccCols = kZCol + 16;
    static constexpr int kTmemCols = 2 * kAccCols <= 256 ? 256 : 512;
    static constexpr int kSmemBytes = 1024 + kBopBytes + kStages * kStageBytes + 2 * kOutBytes + 512 + kPlanBytes;
};

template <int DK, int DV, int MODE, bool BF16, bool VARLEN>
__global__ void __launch_bounds__(kThreads, 1)
tc_fwd_out_kernel(const __grid_constant__ CUtensorMap tm_qr, const __grid_constant__ CUtensorMap tm_q,
                  const __grid_constant__ CUtensorMap tm_o, const Params p_in) {
    using Cfg = FwdOutCfg<DK, DV, MODE>;
    using Map = TileMap<VARLEN>;
    constexpr int NS = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_1024(smem_raw);
    uint8_t* bop = smem;
    uint8_t* stages = bop + Cfg::kBopBytes;
    uint8_t* outbuf = stages + NS * Cfg::kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(outbuf + 2 * Cfg::kOutBytes);
    uint64_t* full = bars;                 // [NS]
    uint64_t* empty = bars + NS;           // [NS]
    uint64_t* tfull = bars + 2 * NS;       // [2] accumulator ready
    uint64_t* tempty = tfull + 2;          // [2] accumulator drained
    uint64_t* bop_ready = tempty + 2;      // state of the segment is in shared memory
    uint64_t* out_free = bop_ready + 1;    // [2] staged tile no longer read by its TMA store
    uint64_t* out_written = out_free + 2;  // [2] staged tile written by all epilogue threads
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(out_written + 2);
    volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ptx::griddep_launch();
    Params pv = p_in;
    if (VARLEN) {
        ptx::griddep_wait();                // cu_seqlens may come from the previous kernel
        int32_t* plan = reinterpret_cast<int32_t*>(smem_raw + (Cfg::kSmemBytes - kPlanBytes));
        build_plan(plan, p_in.cu, p_in.num_seqs);
        pv.plan = plan;
    }
    const Params& p = pv;
    int g0, g1;
    Map::range(p, g0, g1);
    const ptx::Abort ab{cta_abort, p.status};

    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; ++i) {
            ptx::mbar_init(&full[i], 1);
            ptx::mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&tfull[i], 1);
            ptx::mbar_init(&tempty[i], kEpiThreads);
            ptx::mbar_init(&out_free[i], 1);
            ptx::mbar_init(&out_written[i], kEpiThreads);
        }
        ptx::mbar_init(bop_ready, kEpiThreads);
        *cta_abort = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tm_qr);
        ptx::prefetch_tensormap(&tm_o);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (!VARLEN) ptx::griddep_wait();       // everything above overlaps the previous kernel's tail

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            if (!ptx::mbar_wait(&empty[s], ph ^ 1u, ab, 201)) break;
            ptx::mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
            const Tile t = Map::get(p, g, g0, g1);
            uint8_t* st = stages + s * Cfg::kStageBytes;
#pragma unroll
            for (int b = 0; b < Cfg::kKB; ++b) ptx::tma_load_3d(st + b * kBlockBytes, &tm_qr, &full[s], b * 64, t.c1, t.c2);
            if (MODE == kDecoupled) {
#pragma unroll
                for (int b = 0; b < Cfg::kKB; ++b)
                    ptx::tma_load_3d(st + (Cfg::kKB + b) * kBlockBytes, &tm_q, &full[s], b * 64, t.c1, t.c2);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        constexpr bool kOneMma = Cfg::kWide && MODE != kDecoupled;   // numerator halves and z in one instruction
        const uint32_t idesc_n =
            ptx::instr_desc(128, kOneMma ? 2 * DV + Cfg::kZRows : (Cfg::kWide ? 2 * DV : DV), BF16, false, false);
        const uint32_t idesc_z = ptx::instr_desc(128, 16, BF16, false, false);
        const uint32_t bop_base = ptx::smem_u32(bop);
        int seg = 0;
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            const int a = it & 1;
            const bool first = Map::get(p, g, g0, g1).first;
            if (first) {
                if (!ptx::mbar_wait(bop_ready, (uint32_t)seg & 1u, ab, 211)) break;
                ++seg;
            }
            if (!ptx::mbar_wait(&full[s], ph, ab, 212)) break;
            if (!ptx::mbar_wait(&tempty[a], ((uint32_t)(it >> 1) & 1u) ^ 1u, ab, 213)) break;
            ptx::tc_fence_after_sync();
            const uint32_t qr_base = ptx::smem_u32(stages + s * Cfg::kStageBytes);
            const uint32_t q_base = MODE == kDecoupled ? qr_base + Cfg::kKB * kBlockBytes : qr_base;
            const uint32_t acc = tmem + a * Cfg::kAccCols;
#pragma unroll
            for (int kb = 0; kb < Cfg::kKB; ++kb) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const bool accum = !(kb == 0 && kk == 0);
                    const uint64_t da = ptx::smem_desc(qr_base + kb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    const uint64_t db = ptx::smem_desc(bop_base + kb * Cfg::kBopBlock + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    ptx::mma_ss(acc, da, db, idesc_n, accum);
                    if (!Cfg::kWide) {
                        const uint64_t dl = ptx::smem_desc(bop_base + kb * Cfg::kBopBlock + DV * 128 + kk * 32, 16, 1024,
                                                           ptx::kLayoutSw128);
                        ptx::mma_ss(acc, da, dl, idesc_n, true);
                    }
                    if (MODE != kSimple && !kOneMma) {
                        const uint64_t dq = ptx::smem_desc(q_base + kb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                        const uint64_t dz = ptx::smem_desc(bop_base + kb * Cfg::kBopBlock + 2 * DV * 128 + kk * 32, 16, 1024,
                                                           ptx::kLayoutSw128);
                        ptx::mma_ss(acc + Cfg::kZCol, dq, dz, idesc_z, accum);
                    }
                }
            }
            ptx::mma_commit(&empty[s]);
            ptx::mma_commit(&tfull[a]);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;
        const int et = threadIdx.x - 64;                 // 0..127
        const int row = quarter * 32 + lane;             // token row of this thread inside a tile
        const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        const bool issuer = (et == 0);
        int seg = 0;
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const Tile t = Map::get(p, g, g0, g1);
            const int unit = t.unit, tile = t.tile;
            const bool first = t.first;
            const int a = it & 1;
            const uint32_t ph2 = (uint32_t)(it >> 1) & 1u;
            if (first) {
                // Every MMA of the previous segment has completed (its accumulators were drained
                // below), so the B operand can be rewritten for this unit.
                const StateSrc st = state_source(p, unit);
                for (int i0 = et; i0 < DK * DV; i0 += 32 * kEpiThreads) {
                    float xs[32];
                    st.template load<32>(i0, kEpiThreads, xs);
#pragma unroll
                    for (int u = 0; u < 32; ++u) {
                        const int i = i0 + u * kEpiThreads;
                        const int k = i / DV, v = i - k * DV;
                        const float x = xs[u] * t.scale;
                        const uint16_t h = pack1(x, BF16);
                        *reinterpret_cast<uint16_t*>(bop + (k >> 6) * Cfg::kBopBlock + ptx::sw128_offset(v, k & 63)) = h;
                        // rounding residual: a second B operand accumulated into the same columns
                        *reinterpret_cast<uint16_t*>(bop + (k >> 6) * Cfg::kBopBlock + ptx::sw128_offset(DV + v, k & 63)) =
                            pack1(x - unpack1(h, BF16), BF16);
                    }
                }
                if (MODE != kSimple) {
                    for (int i = et; i < 16 * DK; i += kEpiThreads) {
                        const int r = i / DK, k = i - r * DK;
                        uint16_t h = 0;
                        if (r < 2) {
                            const float km = st[DK * DV + k] * t.inv_norm;
                            const uint16_t hi = pack1(km, BF16);
                            h = r == 0 ? hi : pack1(km - unpack1(hi, BF16), BF16);
                        }
                        *reinterpret_cast<uint16_t*>(bop + (k >> 6) * Cfg::kBopBlock + ptx::sw128_offset(2 * DV + r, k & 63)) = h;
                    }
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(bop_ready);
                ++seg;
            }
            if (!ptx::mbar_wait(&tfull[a], ph2, ab, 221)) break;
            ptx::tc_fence_after_sync();
            float rz = 1.f;
            if (MODE != kSimple) {
                float zc[16];
                ptx::tmem_ld16(t_lane + a * Cfg::kAccCols + Cfg::kZCol, zc);
                ptx::tmem_ld_wait();
                rz = 1.f / (zc[0] + zc[1] + p.eps);
            }
            // the staged tile of two tiles ago must have been read by its store
            if (issuer) {
                ptx::tma_store_wait_read<1>();
                ptx::mbar_arrive(&out_free[a]);
            }
            if (!ptx::mbar_wait(&out_free[a], ph2, ab, 222)) break;
            // packed layout: a tile may end inside the next sequence; such a tile leaves in row-guarded
            // 32-byte stores, every full tile as a staged tile through the TMA store like the fixed layout
            uint8_t* orow = static_cast<uint8_t*>(p.out_a) + (size_t)(t.row0 + (long long)row * t.row_stride) * p.mem_dv * 2;
            const bool row_ok = row < t.valid;
            const bool staged = !VARLEN || t.valid == kTileTokens;
            uint8_t* ob = outbuf + a * Cfg::kOutBytes;
#pragma unroll
            for (int c0 = 0; c0 < DV; c0 += 32) {
                float v[32];
                ptx::tmem_ld32(t_lane + a * Cfg::kAccCols + c0, v);
                if (Cfg::kWide) {
                    float lo[32];
                    ptx::tmem_ld32(t_lane + a * Cfg::kAccCols + DV + c0, lo);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += lo[j];
                } else {
                    ptx::tmem_ld_wait();
                }
                uint8_t* blk = ob + (c0 >> 6) * kBlockBytes + row * 128;
                uint4 keep[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint4 w;
                    w.x = pack2(v[8 * j] * rz, v[8 * j + 1] * rz, BF16);
                    w.y = pack2(v[8 * j + 2] * rz, v[8 * j + 3] * rz, BF16);
                    w.z = pack2(v[8 * j + 4] * rz, v[8 * j + 5] * rz, BF16);
                    w.w = pack2(v[8 * j + 6] * rz, v[8 * j + 7] * rz, BF16);
                    const int chunk = ((c0 & 63) >> 3) + j;
                    if (staged) *reinterpret_cast<uint4*>(blk + (((chunk ^ row) & 7) << 4)) = w;
                    keep[j] = w;
                }
                if (!staged && row_ok) {
                    // (rows in memory may be narrower than DV: multiples of 16 features)
                    if (c0 < p.mem_dv) ptx::st_global_32B(orow + c0 * 2, keep[0], keep[1]);
                    if (c0 + 16 < p.mem_dv) ptx::st_global_32B(orow + c0 * 2 + 32, keep[2], keep[3]);
                }
            }
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&tempty[a]);
            ptx::fence_proxy_async_smem();
            ptx::mbar_arrive(&out_written[a]);
            if (issuer) {
                if (!ptx::mbar_wait(&out_written[a], ph2, ab, 223)) break;
                if (staged) {
#pragma unroll
                    for (int b = 0; b < Cfg::kVB; ++b) ptx::tma_store_3d(&tm_o, ob + b * kBlockBytes, b * 64, t.c1, t.c2);
                }
                ptx::tma_store_commit();        // an empty group keeps the wait_read<1> bookkeeping uniform
            }
        }
        if (issuer) ptx::tma_store_wait_all<0>();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

}  // namespace tc
}  // namespace fbla
