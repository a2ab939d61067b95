// Tensor-core kernel of the second backward pass.
//
//   tc_bwd_in_kernel : dk = v . (scale*dS)^T + dkm/L,  dv = kr . (scale*dS)  per 128-token tile, both
//     from one copy of the 16-bit dS in shared memory (read K-major by the first MMA, MN-major by
//     the second).  HBM traffic: k, v once; dk, dv once.
#pragma once

#include "tc_common.cuh"

namespace fbla {
namespace tc {

// Writes the [DK x DV] fp32 matrix `src` (row-major), multiplied by `scale`, into shared memory as
// 16-bit DV/64 blocks of [DK rows][64 columns] in the 128-byte-swizzled layout.  Read K-major it is
// the operand B[n = row][k = column]; read MN-major it is B[k = row][n = column].
// With SPLIT a second copy holding the rounding residual (x - high part, again 16-bit) is written
// DV/64 blocks further on: issuing every MMA once per copy restores ~16 bits of the fp32 state.
template <int DK, int DV, bool SPLIT>
__device__ __forceinline__ void stage_matrix_sw128(uint8_t* dst, const StateSrc& src, float scale, int is_bf16,
                                                   int et) {
    for (int i0 = et; i0 < DK * DV / 2; i0 += 16 * kEpiThreads) {
        float2 xs[16];
        src.template load2<16>(2 * i0, 2 * kEpiThreads, xs);
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int i = i0 + u * kEpiThreads;
            const int k = (2 * i) / DV, v = (2 * i) - k * DV;
            float2 x = xs[u];
            x.x *= scale;
            x.y *= scale;
            const uint32_t h = pack2(x.x, x.y, is_bf16);
            uint8_t* at = dst + (v >> 6) * (DK * 128) + ptx::sw128_offset(k, v & 63);
            *reinterpret_cast<uint32_t*>(at) = h;
            if (SPLIT) {
                const float2 hf = unpack2(h, is_bf16);
                *reinterpret_cast<uint32_t*>(at + (DV / 64) * (DK * 128)) = pack2(x.x - hf.x, x.y - hf.y, is_bf16);
            }
        }
    }
}

// Every shape keeps the residual copy; the 128 x 128 kernel pays for it by writing its outputs
// with plain 16-byte global stores instead of a staged tile.
template <int DK, int DV>
struct SplitState {
    static constexpr bool value = true;
};

// ------------------------------------------------------------------------------------------
template <int DK, int DV, int MODE>
struct BwdInCfg {
    static constexpr int kKB = DK / 64, kVB = DV / 64;
    static constexpr bool kSplit = SplitState<DK, DV>::value;
    static constexpr int kBopOne = kVB * DK * 128;                          // one 16-bit copy of scale*dS
    static constexpr int kBopBytes = kBopOne * (kSplit ? 2 : 1);            // high part (+ residual)
    static constexpr int kVecBytes = 1024;                                  // fp32 dkm / L
    static constexpr int kStageBytes = (kKB + kVB) * kBlockBytes;           // v tile, kr tile
    static constexpr bool kDirect = (DK == 128 && DV == 128);               // no room for a staged output tile
    static constexpr int kOutBytes = kDirect ? 0 : (kKB + kVB) * kBlockBytes;   // staged dk (dkr) and dv tile
    static constexpr int kConstBytes = MODE == kDecoupled ? kKB * kBlockBytes : 0;  // dk tile of the decoupled op
    static constexpr int kOutBufs = (DK == 64 && DV == 64) ? 2 : 1;         // staged output tiles
    static constexpr int kFixed = 1024 + kBopBytes + kVecBytes + kOutBufs * kOutBytes + kConstBytes + 512 + kPlanBytes;
    static constexpr int kStagesRaw = (kSmemLimit - kFixed) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 4 ? 4 : kStagesRaw;
    static constexpr int kAccCols = DK + DV;
    static constexpr int kTmemCols = 2 * kAccCols <= 256 ? 256 : 512;
    static constexpr int kSmemBytes = kFixed + kStages * kStageBytes;
};

template <int DK, int DV, int MODE, bool BF16, bool VARLEN>
__global__ void __launch_bounds__(kThreads, 1)
tc_bwd_in_kernel(const __grid_constant__ CUtensorMap tm_kr, const __grid_constant__ CUtensorMap tm_v,
                 const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dkr,
                 const __grid_constant__ CUtensorMap tm_dv, const Params p_in) {
    using Cfg = BwdInCfg<DK, DV, MODE>;
    using Map = TileMap<VARLEN>;
    // packed layout: rows are strided and tiles may end inside the next sequence -> guarded stores
    constexpr bool kDirectOut = Cfg::kDirect;      // no staged tiles at all
    constexpr int NS = Cfg::kStages;
    constexpr int NO = Cfg::kOutBufs;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_1024(smem_raw);
    uint8_t* bop = smem;
    float* vec = reinterpret_cast<float*>(bop + Cfg::kBopBytes);
    uint8_t* stages = reinterpret_cast<uint8_t*>(vec) + Cfg::kVecBytes;
    uint8_t* outbuf = stages + NS * Cfg::kStageBytes;
    uint8_t* constbuf = outbuf + NO * Cfg::kOutBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(constbuf + Cfg::kConstBytes);
    uint64_t* full = bars;                  // [NS]
    uint64_t* empty = bars + NS;            // [NS]
    uint64_t* tfull = bars + 2 * NS;        // [2]
    uint64_t* tempty = tfull + 2;           // [2]
    uint64_t* bop_ready = tempty + 2;
    uint64_t* out_free = bop_ready + 1;     // [NO]
    uint64_t* out_written = out_free + NO;  // [NO]
    uint64_t* const_free = out_written + NO; // constant dk tile no longer read by a store
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(const_free + 1);
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
        }
        for (int i = 0; i < NO; ++i) {
            ptx::mbar_init(&out_free[i], 1);
            ptx::mbar_init(&out_written[i], kEpiThreads);
        }
        ptx::mbar_init(bop_ready, kEpiThreads);
        ptx::mbar_init(const_free, 1);
        *cta_abort = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tm_kr);
        ptx::prefetch_tensormap(&tm_v);
        ptx::prefetch_tensormap(&tm_dk);
        ptx::prefetch_tensormap(&tm_dv);
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
        // ---------------- TMA producer: v tile then kr tile ----------------
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            if (!ptx::mbar_wait(&empty[s], ph ^ 1u, ab, 401)) break;
            ptx::mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
            const Tile t = Map::get(p, g, g0, g1);
            uint8_t* st = stages + s * Cfg::kStageBytes;
#pragma unroll
            for (int b = 0; b < Cfg::kVB; ++b) ptx::tma_load_3d(st + b * kBlockBytes, &tm_v, &full[s], b * 64, t.c1, t.c2);
#pragma unroll
            for (int b = 0; b < Cfg::kKB; ++b)
                ptx::tma_load_3d(st + (Cfg::kVB + b) * kBlockBytes, &tm_kr, &full[s], b * 64, t.c1, t.c2);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc_dk = ptx::instr_desc(128, DK, BF16, false, false);
        const uint32_t idesc_dv = ptx::instr_desc(128, DV, BF16, false, true);
        const uint32_t bop_base = ptx::smem_u32(bop);
        int seg = 0;
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            const int a = it & 1;
            const bool first = Map::get(p, g, g0, g1).first;
            if (first) {
                if (!ptx::mbar_wait(bop_ready, (uint32_t)seg & 1u, ab, 411)) break;
                ++seg;
            }
            if (!ptx::mbar_wait(&full[s], ph, ab, 412)) break;
            if (!ptx::mbar_wait(&tempty[a], ((uint32_t)(it >> 1) & 1u) ^ 1u, ab, 413)) break;
            ptx::tc_fence_after_sync();
            const uint32_t v_base = ptx::smem_u32(stages + s * Cfg::kStageBytes);
            const uint32_t kr_base = v_base + Cfg::kVB * kBlockBytes;
            const uint32_t acc = tmem + a * Cfg::kAccCols;
            // dk[tok][k] = sum_v V[tok][v] * dS[k][v]   (B K-major: rows k, 128 bytes along v)
#pragma unroll
            for (int vb = 0; vb < Cfg::kVB; ++vb) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t da = ptx::smem_desc(v_base + vb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    const uint64_t db = ptx::smem_desc(bop_base + vb * (DK * 128) + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    ptx::mma_ss(acc, da, db, idesc_dk, !(vb == 0 && kk == 0));
                    if (Cfg::kSplit) {
                        const uint64_t dl = ptx::smem_desc(bop_base + Cfg::kBopOne + vb * (DK * 128) + kk * 32, 16, 1024,
                                                           ptx::kLayoutSw128);
                        ptx::mma_ss(acc, da, dl, idesc_dk, true);
                    }
                }
            }
            // dv[tok][v] = sum_k KR[tok][k] * dS[k][v]  (B MN-major: rows k, 128 bytes along v)
#pragma unroll
            for (int kb = 0; kb < Cfg::kKB; ++kb) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t da = ptx::smem_desc(kr_base + kb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    const uint64_t db = ptx::smem_desc(bop_base + (kb * 64 + kk * 16) * 128, DK * 128, 1024, ptx::kLayoutSw128);
                    ptx::mma_ss(acc + DK, da, db, idesc_dv, !(kb == 0 && kk == 0));
                    if (Cfg::kSplit) {
                        const uint64_t dl = ptx::smem_desc(bop_base + Cfg::kBopOne + (kb * 64 + kk * 16) * 128, DK * 128, 1024,
                                                           ptx::kLayoutSw128);
                        ptx::mma_ss(acc + DK, da, dl, idesc_dv, true);
                    }
                }
            }
            ptx::mma_commit(&empty[s]);
            ptx::mma_commit(&tfull[a]);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;
        const int et = threadIdx.x - 64;
        const int row = quarter * 32 + lane;
        const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        const bool issuer = (et == 0);
        int seg = 0;
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const Tile t = Map::get(p, g, g0, g1);
            const int unit = t.unit, tile = t.tile;
            const bool first = t.first;
            const int a = it & 1;
            const int ob_i = it % NO;
            const uint32_t ph2 = (uint32_t)(it >> 1) & 1u;
            const uint32_t pho = (uint32_t)(it / NO) & 1u;
            if (first) {
                const StateSrc st = state_source(p, unit);
                // `vec` (and the constant tile) of the previous unit are read by every epilogue thread
                // until it has arrived on out_written of the previous tile
                if (it > 0 && !ptx::mbar_wait(&out_written[(it - 1) % NO], (uint32_t)((it - 1) / NO) & 1u, ab, 424)) break;
                if (MODE == kDecoupled) {
                    if (issuer) {
                        ptx::tma_store_wait_read<0>();
                        ptx::mbar_arrive(const_free);
                    }
                    if (!ptx::mbar_wait(const_free, (uint32_t)seg & 1u, ab, 425)) break;
                }
                ++seg;
                stage_matrix_sw128<DK, DV, Cfg::kSplit>(bop, st, t.scale, BF16, et);
                if (MODE != kSimple)
                    for (int i = et; i < DK; i += kEpiThreads) vec[i] = st[DK * DV + i] * t.inv_norm;
                if (MODE == kDecoupled) {
                    // every token's dk is dkm / L: one constant tile, stored once per tile
                    for (int i = et; i < kTileTokens * DK / 2; i += kEpiThreads) {
                        const int r = (2 * i) / DK, k = (2 * i) - r * DK;
                        const float x0 = st[DK * DV + k] * t.inv_norm, x1 = st[DK * DV + k + 1] * t.inv_norm;
                        *reinterpret_cast<uint32_t*>(constbuf + (k >> 6) * kBlockBytes + ptx::sw128_offset(r, k & 63)) =
                            pack2(x0, x1, BF16);
                    }
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(bop_ready);
            }
            if (!ptx::mbar_wait(&tfull[a], ph2, ab, 421)) break;
            ptx::tc_fence_after_sync();
            if (!kDirectOut) {
                if (issuer) {
                    ptx::tma_store_wait_read<NO - 1>();
                    ptx::mbar_arrive(&out_free[ob_i]);
                }
                if (!ptx::mbar_wait(&out_free[ob_i], pho, ab, 422)) break;
            }
            uint8_t* ob = outbuf + ob_i * Cfg::kOutBytes;
            const bool tok_ok = row < t.valid;
            // packed layout: only full tiles go through the staged TMA store; a tile that ends inside the
            // next sequence leaves in row-guarded 32-byte stores
            const bool direct = kDirectOut || (VARLEN && t.valid != kTileTokens);
            const size_t grow = (size_t)(t.row0 + (long long)row * t.row_stride);   // this thread's row in the (rows, D) view
            // dk (or dk_rope) tile
#pragma unroll
            for (int c0 = 0; c0 < DK; c0 += 32) {
                float v[32];
                ptx::tmem_ld32(t_lane + a * Cfg::kAccCols + c0, v);
                ptx::tmem_ld_wait();
                if (MODE == kLinear) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += vec[c0 + j];
                }
                uint8_t* blk = ob + (c0 >> 6) * kBlockBytes + row * 128;
                uint4 w4[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    w4[j].x = pack2(v[8 * j], v[8 * j + 1], BF16);
                    w4[j].y = pack2(v[8 * j + 2], v[8 * j + 3], BF16);
                    w4[j].z = pack2(v[8 * j + 4], v[8 * j + 5], BF16);
                    w4[j].w = pack2(v[8 * j + 6], v[8 * j + 7], BF16);
                }
                if (direct) {
                    if (tok_ok) {
                        uint8_t* dst = static_cast<uint8_t*>(p.out_a) + (grow * p.mem_dk + c0) * 2;
                        if (c0 < p.mem_dk) ptx::st_global_32B(dst, w4[0], w4[1]);          // (rows may be narrower than DK)
                        if (c0 + 16 < p.mem_dk) ptx::st_global_32B(dst + 32, w4[2], w4[3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int chunk = ((c0 & 63) >> 3) + j;
                        *reinterpret_cast<uint4*>(blk + (((chunk ^ row) & 7) << 4)) = w4[j];
                    }
                }
            }
            // dv tile
#pragma unroll
            for (int c0 = 0; c0 < DV; c0 += 32) {
                float v[32];
                ptx::tmem_ld32(t_lane + a * Cfg::kAccCols + DK + c0, v);
                ptx::tmem_ld_wait();
                uint8_t* blk = ob + (Cfg::kKB + (c0 >> 6)) * kBlockBytes + row * 128;
                uint4 w4[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    w4[j].x = pack2(v[8 * j], v[8 * j + 1], BF16);
                    w4[j].y = pack2(v[8 * j + 2], v[8 * j + 3], BF16);
                    w4[j].z = pack2(v[8 * j + 4], v[8 * j + 5], BF16);
                    w4[j].w = pack2(v[8 * j + 6], v[8 * j + 7], BF16);
                }
                if (direct) {
                    if (tok_ok) {
                        uint8_t* dst = static_cast<uint8_t*>(p.out_b) + (grow * p.mem_dv + c0) * 2;
                        if (c0 < p.mem_dv) ptx::st_global_32B(dst, w4[0], w4[1]);
                        if (c0 + 16 < p.mem_dv) ptx::st_global_32B(dst + 32, w4[2], w4[3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int chunk = ((c0 & 63) >> 3) + j;
                        *reinterpret_cast<uint4*>(blk + (((chunk ^ row) & 7) << 4)) = w4[j];
                    }
                }
            }
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&tempty[a]);
            ptx::fence_proxy_async_smem();
            ptx::mbar_arrive(&out_written[ob_i]);
            if (!kDirectOut && issuer) {
                if (!ptx::mbar_wait(&out_written[ob_i], pho, ab, 423)) break;
                if (!direct) {
#pragma unroll
                    for (int b = 0; b < Cfg::kKB; ++b) ptx::tma_store_3d(&tm_dkr, ob + b * kBlockBytes, b * 64, t.c1, t.c2);
#pragma unroll
                    for (int b = 0; b < Cfg::kVB; ++b)
                        ptx::tma_store_3d(&tm_dv, ob + (Cfg::kKB + b) * kBlockBytes, b * 64, t.c1, t.c2);
                    if (MODE == kDecoupled) {
#pragma unroll
                        for (int b = 0; b < Cfg::kKB; ++b)
                            ptx::tma_store_3d(&tm_dk, constbuf + b * kBlockBytes, b * 64, t.c1, t.c2);
                    }
                }
                ptx::tma_store_commit();        // an empty group keeps the wait_read bookkeeping uniform
            }
        }
        if (!kDirectOut && issuer) ptx::tma_store_wait_all<0>();
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
