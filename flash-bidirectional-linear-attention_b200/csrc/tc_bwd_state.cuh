// Tensor-core kernel of the first backward pass.
//
//   tc_bwd_state_kernel : per 128-token tile
//         [ t | z ] = [ dO . (scale*S)^T | q . kmean ]   (MMA 1, K-major operands, accumulators in TMEM;
//                                                         kmean enters as a high and a low 16-bit column)
//         dz = -(qr . t) / (z + eps)^2
//         dq = t / z + dz * kmean                        (TMA store, or plain 16-byte stores where the
//                                                         shared memory has no room for a staged tile)
//         qs = qr / z                                    (written back over the qr tile in shared memory)
//         [ dS | dkm ] += qs^T . [ dO | dz*z ]           (MMA 2, MN-major operands: contraction over tokens)
//     and one fp32 partial [ dS | sum_t dz q ] per segment.  The saved output o is not read:
//     sum_v o*dO = (qr . t) / z.  HBM traffic: q, dO once; dq once.
//
//   The per-token arithmetic between the two MMAs is the longest stage of the pipeline, so two
//   epilogue warpgroups work on alternate tiles, and the two MMAs have an issuing thread each: the
//   thread of MMA 1 runs ahead (up to three t accumulators), the thread of MMA 2 follows the epilogue.
#pragma once

#include "tc_bwd_in.cuh"

namespace fbla {
namespace tc {

// producer warp, MMA-1 warp, two epilogue warpgroups, MMA-2 warp
constexpr int kBwdStateThreads = 64 + 2 * kEpiThreads + 32;


template <int DK, int DV, int MODE, bool VARLEN = false>
struct BwdStateCfg {
    static constexpr int kKB = DK / 64, kVB = DV / 64;
    static constexpr int kBopOne = kVB * DK * 128;                          // one 16-bit copy of scale*S
    static constexpr int kBopBytes = 2 * kBopOne;                           // high part + residual
    static constexpr int kVecBytes = 1024;                                  // fp32 kmean
    static constexpr int kKmOpBytes = MODE != kSimple ? kKB * 2048 : 0;     // 16-bit kmean rows (B of the z MMA)
    static constexpr int kDzBytes = MODE != kSimple ? 4096 : 0;             // [2 token blocks][16 rows][128 B]
    static constexpr int kQBlocks = kKB * (MODE == kDecoupled ? 2 : 1);
    static constexpr int kTmaBytes = (kQBlocks + kVB) * kBlockBytes;        // qr (, q), dO tiles
    static constexpr int kStageBytes = kTmaBytes + kDzBytes;
    // Fixed length: dq leaves in 32-byte global stores straight from registers (one full sector per
    // thread and store): measured as fast as a staged tile + TMA store, and the 16-32 KB per warpgroup
    // it saves buy a deeper load pipeline.  Packed layout: the rows of a head are heads*D elements apart,
    // so every 32-byte store opens a DRAM page of its own; there full tiles are staged in shared memory
    // and leave as one strided TMA store per warpgroup and tile (tiles that end inside the next sequence
    // keep the row-guarded direct stores).  The 128 x 128 shape has no room for staging.
    static constexpr bool kDirect = !(VARLEN && !(DK == 128 && DV == 128));
    static constexpr int kOutBytes = kDirect ? 0 : kQBlocks * kBlockBytes;  // per warpgroup
    static constexpr int kFixed = 1024 + kBopBytes + kVecBytes + kKmOpBytes + 2 * kOutBytes + 512 + kPlanBytes;
    static constexpr int kStagesRaw = (kSmemLimit - kFixed) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 5 ? 5 : kStagesRaw;
    static constexpr int kTCols = DK + (MODE != kSimple ? 16 : 0);          // t (+ z) accumulator
    // t accumulators: with three, MMA 1 runs ahead of the epilogue, so a warpgroup finds its next
    // accumulator complete when it finishes a tile
    static constexpr int kTBufs = (3 * kTCols + DV + 16 <= 512) ? 3 : 2;
    static constexpr int kColS = kTBufs * kTCols;                           // dS accumulator, DV columns
    static constexpr int kColM = kColS + DV;                                // dkm accumulator, 16 columns
    static constexpr int kTmemCols = (kColM + 16) <= 256 ? 256 : 512;
    static constexpr int kSmemBytes = kFixed + kStages * kStageBytes;
};

// NARROW: the rows of dq in memory may hold fewer than DK features (Params::mem_dk); otherwise the row width is
// the compile-time DK, which keeps the guard and the address arithmetic out of the issue-bound epilogue.
template <int DK, int DV, int MODE, bool BF16, bool VARLEN, bool NARROW = false>
__global__ void __launch_bounds__(kBwdStateThreads, 1)
tc_bwd_state_kernel(const __grid_constant__ CUtensorMap tm_qr, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_dq,
                    const __grid_constant__ CUtensorMap tm_dqr, const Params p_in) {
    using Cfg = BwdStateCfg<DK, DV, MODE, VARLEN>;
    using Map = TileMap<VARLEN>;
    constexpr int NS = Cfg::kStages;
    constexpr int NB = Cfg::kTBufs;
    constexpr int KB = Cfg::kKB, VB = Cfg::kVB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align_1024(smem_raw);
    uint8_t* bop = smem;
    float* km = reinterpret_cast<float*>(bop + Cfg::kBopBytes);
    uint8_t* kmop = reinterpret_cast<uint8_t*>(km) + Cfg::kVecBytes;
    uint8_t* stages = kmop + Cfg::kKmOpBytes;
    uint8_t* outbuf = stages + NS * Cfg::kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(outbuf + 2 * Cfg::kOutBytes);
    uint64_t* full = bars;                  // [NS] TMA landed
    uint64_t* empty = bars + NS;            // [NS] MMA 2 done with the stage
    uint64_t* qs_ready = bars + 2 * NS;     // [NS] epilogue wrote qr/z and the dz columns
    uint64_t* tfull = bars + 3 * NS;        // [NB] t accumulator ready
    uint64_t* tempty = tfull + NB;          // [NB] t accumulator drained
    uint64_t* bop_ready = tempty + NB;      // state of the segment is in shared memory
    uint64_t* acc_full = bop_ready + 1;     // dS / dkm of a segment complete
    uint64_t* acc_empty = acc_full + 1;
    uint64_t* out_free = acc_empty + 1;     // [2] staged tile of the warpgroup no longer read by its store
    uint64_t* out_written = out_free + 2;   // [2] warpgroup finished its tile (staged tile written, km read)
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
    const int mem_dk = NARROW ? p.mem_dk : DK;      // features per row of dq in memory
    int g0, g1;
    Map::range(p, g0, g1);
    const ptx::Abort ab{cta_abort, p.status};

    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; ++i) {
            ptx::mbar_init(&full[i], 1);
            ptx::mbar_init(&empty[i], 1);
            ptx::mbar_init(&qs_ready[i], kEpiThreads);
        }
        for (int i = 0; i < NB; ++i) {
            ptx::mbar_init(&tfull[i], 1);
            ptx::mbar_init(&tempty[i], kEpiThreads);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&out_free[i], 1);
            ptx::mbar_init(&out_written[i], kEpiThreads);
        }
        ptx::mbar_init(bop_ready, kEpiThreads);
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, kEpiThreads);
        *cta_abort = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tm_qr);
        ptx::prefetch_tensormap(&tm_do);
        ptx::prefetch_tensormap(&tm_dqr);
    }
    if (MODE != kSimple) {
        // rows 2..15 of every dz tile stay zero for the whole kernel
        for (int s = 0; s < NS; ++s) {
            uint32_t* dzt = reinterpret_cast<uint32_t*>(stages + s * Cfg::kStageBytes + Cfg::kTmaBytes);
            for (int i = threadIdx.x; i < Cfg::kDzBytes / 4; i += kBwdStateThreads) dzt[i] = 0u;
        }
        ptx::fence_proxy_async_smem();
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
        // ---------------- TMA producer: qr tile, (q tile,) dO tile ----------------
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            if (!ptx::mbar_wait(&empty[s], ph ^ 1u, ab, 301)) break;
            ptx::mbar_arrive_expect_tx(&full[s], Cfg::kTmaBytes);
            const Tile t = Map::get(p, g, g0, g1);
            uint8_t* st = stages + s * Cfg::kStageBytes;
#pragma unroll
            for (int b = 0; b < KB; ++b) ptx::tma_load_3d(st + b * kBlockBytes, &tm_qr, &full[s], b * 64, t.c1, t.c2);
            if (MODE == kDecoupled) {
#pragma unroll
                for (int b = 0; b < KB; ++b) ptx::tma_load_3d(st + (KB + b) * kBlockBytes, &tm_q, &full[s], b * 64, t.c1, t.c2);
            }
#pragma unroll
            for (int b = 0; b < VB; ++b)
                ptx::tma_load_3d(st + (Cfg::kQBlocks + b) * kBlockBytes, &tm_do, &full[s], b * 64, t.c1, t.c2);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- issuer of MMA 1: [t | z] = [dO . S^T | q . kmean] ----------------
        const uint32_t idesc_t = ptx::instr_desc(128, DK, BF16, false, false);
        const uint32_t idesc_z = ptx::instr_desc(128, 16, BF16, false, false);
        const uint32_t bop_base = ptx::smem_u32(bop);
        const uint32_t kmop_base = ptx::smem_u32(kmop);
        int seg_bop = 0;
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            const int tb = it % NB;
            const bool first = Map::get(p, g, g0, g1).first;
            if (first) {
                // the epilogue rewrites the state operand only after the first MMA of the previous
                // unit's last tile has completed, then arrives here
                if (!ptx::mbar_wait(bop_ready, (uint32_t)seg_bop & 1u, ab, 311)) break;
                ++seg_bop;
            }
            if (!ptx::mbar_wait(&full[s], ph, ab, 312)) break;
            if (!ptx::mbar_wait(&tempty[tb], ((uint32_t)(it / NB) & 1u) ^ 1u, ab, 313)) break;
            ptx::tc_fence_after_sync();
            const uint32_t qr_base = ptx::smem_u32(stages + s * Cfg::kStageBytes);
            const uint32_t q_base = MODE == kDecoupled ? qr_base + KB * kBlockBytes : qr_base;
            const uint32_t do_base = qr_base + Cfg::kQBlocks * kBlockBytes;
            const uint32_t t_acc = tmem + tb * Cfg::kTCols;
            // t[tok][k] = sum_v dO[tok][v] * S[k][v], high part and residual of S
#pragma unroll
            for (int vb = 0; vb < VB; ++vb) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t da = ptx::smem_desc(do_base + vb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    const uint64_t db = ptx::smem_desc(bop_base + vb * (DK * 128) + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    const uint64_t dl = ptx::smem_desc(bop_base + Cfg::kBopOne + vb * (DK * 128) + kk * 32, 16, 1024,
                                                       ptx::kLayoutSw128);
                    ptx::mma_ss(t_acc, da, db, idesc_t, !(vb == 0 && kk == 0));
                    ptx::mma_ss(t_acc, da, dl, idesc_t, true);
                }
            }
            // z[tok] = q[tok] . kmean (two columns: high and low part of kmean)
            if (MODE != kSimple) {
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t da = ptx::smem_desc(q_base + kb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                        const uint64_t db = ptx::smem_desc(kmop_base + kb * 2048 + kk * 32, 16, 1024, ptx::kLayoutSw128);
                        ptx::mma_ss(t_acc + DK, da, db, idesc_z, !(kb == 0 && kk == 0));
                    }
                }
            }
            ptx::mma_commit(&tfull[tb]);
        }
    } else if (warp == kBwdStateThreads / 32 - 1 && lane == 0) {
        // ---------------- issuer of MMA 2: [dS | dkm] += qs^T . [dO | dz] ----------------
        // A thread of its own: it follows the epilogue (qs_ready) while the issuer of MMA 1 runs
        // ahead of it by as many tiles as there are t accumulators and stages.
        const uint32_t idesc_s = ptx::instr_desc(DK, DV, BF16, true, true);
        const uint32_t idesc_m = ptx::instr_desc(DK, 16, BF16, true, false);
        int seg_acc = 0;
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            const Tile t = Map::get(p, g, g0, g1);
            const bool first = t.first, last = t.last;
            if (!ptx::mbar_wait(&qs_ready[s], ph, ab, 314)) break;
            if (first && !ptx::mbar_wait(acc_empty, ((uint32_t)seg_acc & 1u) ^ 1u, ab, 315)) break;
            ptx::tc_fence_after_sync();
            const uint32_t qr_base = ptx::smem_u32(stages + s * Cfg::kStageBytes);
            const uint32_t q_base = MODE == kDecoupled ? qr_base + KB * kBlockBytes : qr_base;
            const uint32_t do_base = qr_base + Cfg::kQBlocks * kBlockBytes;
            const uint32_t dz_base = qr_base + Cfg::kTmaBytes;
#pragma unroll
            for (int ks = 0; ks < kTileTokens / 16; ++ks) {
                const bool acc = !(first && ks == 0);
                const uint64_t da = ptx::smem_desc(qr_base + ks * 2048, kBlockBytes, 1024, ptx::kLayoutSw128);
                const uint64_t db = ptx::smem_desc(do_base + ks * 2048, kBlockBytes, 1024, ptx::kLayoutSw128);
                ptx::mma_ss(tmem + Cfg::kColS, da, db, idesc_s, acc);
                if (MODE != kSimple) {
                    const uint64_t dq_ = ptx::smem_desc(q_base + ks * 2048, kBlockBytes, 1024, ptx::kLayoutSw128);
                    const uint64_t dz_ = ptx::smem_desc(dz_base + (ks >> 2) * 2048 + (ks & 3) * 32, 16, 1024, ptx::kLayoutSw128);
                    ptx::mma_ss(tmem + Cfg::kColM, dq_, dz_, idesc_m, acc);
                }
            }
            ptx::mma_commit(&empty[s]);
            if (last) {
                ptx::mma_commit(acc_full);
                ++seg_acc;
            }
        }
    } else if (warp >= 2 && warp < 2 + 2 * (kEpiThreads / 32)) {
        // ---------------- epilogue: warpgroup wg owns the iterations with (it & 1) == wg ----------------
        const int wg = (warp - 2) >> 2;
        const int quarter = warp & 3;
        const int et = (threadIdx.x - 64) & (kEpiThreads - 1);
        const int row = quarter * 32 + lane;
        const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        const bool issuer = (et == 0);
        uint8_t* ob = outbuf + wg * Cfg::kOutBytes;
        const int a = wg;                                   // staged tile / out_* barriers of this warpgroup
        int nseg = 0;                                       // segments opened so far in this CTA's range
        for (int g = g0, it = 0; g < g1; ++g, ++it) {
            const Tile t = Map::get(p, g, g0, g1);
            if (t.first) ++nseg;
            if ((it & 1) != wg) continue;
            const int unit = t.unit;
            const bool first = t.first, last = t.last;
            const int s = it % NS;
            const uint32_t ph = (uint32_t)(it / NS) & 1u;
            const uint32_t ph2 = (uint32_t)(it >> 1) & 1u;   // phase of this warpgroup's out_* barriers
            const int tb = it % NB;                          // t accumulator of this tile
            const uint32_t pht = (uint32_t)(it / NB) & 1u;
            const uint32_t seg = (uint32_t)(nseg - 1);
            if (first) {
                if (it > 0) {
                    // tile it-1 (the other warpgroup's, last of the previous unit) must be past its
                    // first MMA, which reads the state operand, and past its reads of km
                    if (!ptx::mbar_wait(&tfull[(it - 1) % NB], (uint32_t)((it - 1) / NB) & 1u, ab, 326)) break;
                    if (!ptx::mbar_wait(&out_written[a ^ 1], (uint32_t)((it - 1) >> 1) & 1u, ab, 327)) break;
                }
                const StateSrc st = state_source(p, unit);
                stage_matrix_sw128<DK, DV, true>(bop, st, t.scale, BF16, et);
                if (MODE != kSimple) {
                    for (int i = et; i < DK; i += kEpiThreads) km[i] = st[DK * DV + i] * t.inv_norm;
                    for (int i = et; i < 16 * DK; i += kEpiThreads) {
                        const int r = i / DK, k = i - r * DK;
                        uint16_t h = 0;
                        if (r < 2) {
                            const float x = st[DK * DV + k] * t.inv_norm;
                            const uint16_t hi = pack1(x, BF16);
                            h = r == 0 ? hi : pack1(x - unpack1(hi, BF16), BF16);
                        }
                        *reinterpret_cast<uint16_t*>(kmop + (k >> 6) * 2048 + ptx::sw128_offset(r, k & 63)) = h;
                    }
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(bop_ready);
            }
            // km of this unit was written by whichever warpgroup opened the segment
            if (!ptx::mbar_wait(bop_ready, seg & 1u, ab, 328)) break;
            if (!ptx::mbar_wait(&full[s], ph, ab, 321)) break;       // the qr tile is read below
            if (!ptx::mbar_wait(&tfull[tb], pht, ab, 322)) break;
            ptx::tc_fence_after_sync();
            uint8_t* stg = stages + s * Cfg::kStageBytes;
            uint8_t* qr_row = stg + row * 128;                        // + block * kBlockBytes + swizzled chunk
            const uint32_t t_acc = t_lane + tb * Cfg::kTCols;
            const bool tok_ok = row < t.valid;
            const bool staged = !Cfg::kDirect && t.valid == kTileTokens;            // full tile of the packed layout
            const size_t grow = (size_t)(t.row0 + (long long)row * t.row_stride);   // this thread's row in the (rows, D) view
            float rz = 1.f, dz = 0.f, z = 1.f;

            // emits columns [c0, c0+32): dq to the staged tile (or global memory), qr/z over the qr tile
            auto emit32 = [&](int c0, const float (&t)[32], const uint4 (&qv)[4]) {
                uint4 keep1[4], keep2[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = c0 + 8 * j;
                    const uint32_t off = (uint32_t)(c >> 6) * kBlockBytes + (((((c & 63) >> 3) ^ row) & 7) << 4);
                    const uint32_t rw[4] = {qv[j].x, qv[j].y, qv[j].z, qv[j].w};
                    uint32_t o1[4], o2[4], qs[4];
                    float kmv[8];
                    if (MODE != kSimple) {
                        const float4 ka = *reinterpret_cast<const float4*>(km + c);
                        const float4 kb = *reinterpret_cast<const float4*>(km + c + 4);
                        kmv[0] = ka.x; kmv[1] = ka.y; kmv[2] = ka.z; kmv[3] = ka.w;
                        kmv[4] = kb.x; kmv[5] = kb.y; kmv[6] = kb.z; kmv[7] = kb.w;
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float ta = t[8 * j + 2 * e], tb = t[8 * j + 2 * e + 1];
                        if (MODE == kSimple) {
                            o1[e] = pack2(ta, tb, BF16);
                        } else {
                            const float ga = dz * kmv[2 * e], gb = dz * kmv[2 * e + 1];
                            if (MODE == kLinear) {
                                o1[e] = pack2(fmaf(ta, rz, ga), fmaf(tb, rz, gb), BF16);
                            } else {
                                o1[e] = pack2(ta * rz, tb * rz, BF16);   // dq_rope
                                o2[e] = pack2(ga, gb, BF16);             // dq
                            }
                            const float2 rf = unpack2(rw[e], BF16);
                            qs[e] = (VARLEN && !tok_ok) ? 0u : pack2(rf.x * rz, rf.y * rz, BF16);
                        }
                    }
                    if (!staged) {
                        keep1[j] = make_uint4(o1[0], o1[1], o1[2], o1[3]);
                        if (MODE == kDecoupled) keep2[j] = make_uint4(o2[0], o2[1], o2[2], o2[3]);
                        if ((j & 1) && tok_ok && c - 8 < mem_dk) {      // two 16-byte chunks = one 32-byte sector per store
                            const size_t at = (grow * mem_dk + c - 8) * 2;
                            ptx::st_global_32B(static_cast<uint8_t*>(p.out_a) + at, keep1[j - 1], keep1[j]);
                            if (MODE == kDecoupled)
                                ptx::st_global_32B(static_cast<uint8_t*>(p.out_b) + at, keep2[j - 1], keep2[j]);
                        }
                    } else {
                        *reinterpret_cast<uint4*>(ob + row * 128 + off) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
                        if (MODE == kDecoupled)
                            *reinterpret_cast<uint4*>(ob + KB * kBlockBytes + row * 128 + off) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
                    }
                    if (MODE != kSimple) *reinterpret_cast<uint4*>(qr_row + off) = make_uint4(qs[0], qs[1], qs[2], qs[3]);
                }
            };
            // loads columns [c0, c0+32) of t and of the packed qr row
            auto load32 = [&](int c0, float (&t)[32], uint4 (&qv)[4]) {
                ptx::tmem_ld32(t_acc + c0, t);
                if (MODE != kSimple) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int c = c0 + 8 * j;
                        const uint32_t off = (uint32_t)(c >> 6) * kBlockBytes + (((((c & 63) >> 3) ^ row) & 7) << 4);
                        qv[j] = *reinterpret_cast<const uint4*>(qr_row + off);
                    }
                }
            };
            auto dot32 = [&](const float (&t)[32], const uint4 (&qv)[4]) {
                float w[4] = {0.f, 0.f, 0.f, 0.f};   // independent chains
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t rw[4] = {qv[j].x, qv[j].y, qv[j].z, qv[j].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 rf = unpack2(rw[e], BF16);
                        w[e] = fmaf(rf.x, t[8 * j + 2 * e], w[e]);
                        w[e] = fmaf(rf.y, t[8 * j + 2 * e + 1], w[e]);
                    }
                }
                return (w[0] + w[1]) + (w[2] + w[3]);
            };
            auto wait_out_free = [&]() -> bool {
                if (Cfg::kDirect) return true;
                if (issuer) {
                    ptx::tma_store_wait_read<0>();      // the store of this warpgroup's previous tile
                    ptx::mbar_arrive(&out_free[a]);
                }
                return ptx::mbar_wait(&out_free[a], ph2, ab, 323);
            };

            if (DK == 64) {
                // one pass: the whole row of t stays in registers
                float t_lo[32], t_hi[32];
                uint4 qa[4], qb[4];
                float zc[16];
                load32(0, t_lo, qa);
                load32(32, t_hi, qb);
                if (MODE != kSimple) ptx::tmem_ld16(t_acc + DK, zc);
                ptx::tmem_ld_wait();
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(&tempty[tb]);
                if (MODE != kSimple) {
                    const float w = dot32(t_lo, qa) + dot32(t_hi, qb);
                    z = zc[0] + zc[1] + p.eps;
                    rz = 1.f / z;
                    dz = -w * rz * rz;
                }
                if (!wait_out_free()) break;
                emit32(0, t_lo, qa);
                emit32(32, t_hi, qb);
            } else {
                // two passes over the accumulator: first qr . t, then the outputs
                float w = 0.f;
                if (MODE != kSimple) {
                    float zc[16];
                    ptx::tmem_ld16(t_acc + DK, zc);
#pragma unroll
                    for (int c0 = 0; c0 < DK; c0 += 32) {
                        float t[32];
                        uint4 qv[4];
                        load32(c0, t, qv);
                        ptx::tmem_ld_wait();
                        w += dot32(t, qv);
                    }
                    z = zc[0] + zc[1] + p.eps;
                    rz = 1.f / z;
                    dz = -w * rz * rz;
                }
                if (!wait_out_free()) break;
#pragma unroll
                for (int c0 = 0; c0 < DK; c0 += 32) {
                    float t[32];
                    uint4 qv[4];
                    load32(c0, t, qv);
                    ptx::tmem_ld_wait();
                    emit32(c0, t, qv);
                }
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(&tempty[tb]);
            }
            if (MODE != kSimple) {
                // two 16-bit columns whose sum is dz*z (paired with qr/z) or dz (decoupled: paired with q)
                float x = MODE == kLinear ? dz * z : dz;
                if (VARLEN && !tok_ok) {
                    // rows past the end of a packed sequence belong to the next one: they must not
                    // reach the token contraction (qs is zero already; clear dO and dz as well)
                    x = 0.f;
                    uint8_t* do_row = stg + Cfg::kQBlocks * kBlockBytes + row * 128;
#pragma unroll
                    for (int b = 0; b < VB; ++b)
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(do_row + b * kBlockBytes + c * 16) = make_uint4(0, 0, 0, 0);
                }
                const uint16_t hi = pack1(x, BF16);
                const uint16_t lo = pack1(x - unpack1(hi, BF16), BF16);
                uint8_t* dzt = stg + Cfg::kTmaBytes + (row >> 6) * 2048;
                const int tc = row & 63;
                *reinterpret_cast<uint16_t*>(dzt + ptx::sw128_offset(0, tc)) = hi;
                *reinterpret_cast<uint16_t*>(dzt + ptx::sw128_offset(1, tc)) = lo;
            }
            ptx::fence_proxy_async_smem();
            ptx::mbar_arrive(&qs_ready[s]);
            ptx::mbar_arrive(&out_written[a]);
            if (!Cfg::kDirect && issuer) {
                if (!ptx::mbar_wait(&out_written[a], ph2, ab, 324)) break;
                if (staged) {
#pragma unroll
                    for (int b = 0; b < KB; ++b) ptx::tma_store_3d(&tm_dqr, ob + b * kBlockBytes, b * 64, t.c1, t.c2);
                    if (MODE == kDecoupled) {
#pragma unroll
                        for (int b = 0; b < KB; ++b)
                            ptx::tma_store_3d(&tm_dq, ob + (KB + b) * kBlockBytes, b * 64, t.c1, t.c2);
                    }
                }
                ptx::tma_store_commit();        // an empty group keeps the wait_read bookkeeping uniform
            }
            if (last) {
                if (!ptx::mbar_wait(acc_full, seg & 1u, ab, 325)) break;
                ptx::tc_fence_after_sync();
                float* out = segment_destination<VARLEN>(p, t, p.state_out);
                drain_state_acc<DK, DV, (MODE != kSimple ? 2 : 0)>(tmem + Cfg::kColS, DV, out, warp, lane);
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(acc_empty);
            }
        }
        if (!Cfg::kDirect && issuer) ptx::tma_store_wait_all<0>();
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
