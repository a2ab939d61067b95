// Query-side backward of the piecewise sparse attention stage on the 5th-generation tensor cores
// (the reference has no backward for this operator; the formulas are stated where fbla_pisa_bwd is
// defined).  One CTA per block of 64 queries of one (batch, head); same outputs as the mma.sync
// kernel it replaces: dq, the per-row dD, the rows dr = dO g scale / (T den) from which the state
// pass forms dh = q^T dr, and this block's share of dkc, dvc (fp32, red.global.add).
//
// Per selected key block (and per group of 64 unselected blocks, with their means / sums as keys /
// values):
//     S  = Q K^T,  dP = dO V^T      tcgen05.mma, M = 64, N = 64 each, accumulators in TMEM
//     p  = exp2(S scale log2e - m)  the row maximum m and denominator come from the forward's row
//     ds = p (dP / den + dD) scale  statistics: nothing is reduced or rescaled in the loop
//     dQ += ds K                    tcgen05.mma, ds staged in shared memory (bf16: plus its rounding
//                                   residual as a second product), accumulator in TMEM
// and for the groups of unselected blocks also dkc = ds^T Q and dvc = (p / den)^T dO, formed in the
// TMEM columns of S and dP and added to global memory by the element-wise warps.
//
//   warp 0      TMA producer: Q, dO, O, h once; then a two-deep ring of key tiles and one value tile
//   warp 1      MMA issuer (one thread) and owner of the TMEM allocation
//   warps 2-9   element-wise work: two warps per TMEM lane window, each on one half of the columns
//               (16x256b shape: thread t holds rows t / 4 and t / 4 + 8, two adjacent columns of
//               every group of eight)
//
// Before the loop: r = Q h (TMEM), od = rowsum(O dO), nr = rowsum(dO r), the per-row constants, the
// dr tile, and dQ = dr h^T as the initial value of the accumulator.
// Every wait is bounded and reports through the library's status word.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "pisa_tc.cuh"
#include "pisa_tc_common.cuh"
#include "tc_kernels.cuh"
#include "tc_ptx.cuh"

namespace fbla {

// Development aid (compile with -DFBLA_PISA_TRACE): one CTA writes clock64() stamps of its phases.
#ifdef FBLA_PISA_TRACE
__device__ long long g_pisa_bwd_trace[128];
#define PISA_BSTAMP(slot)                                                                     \
    do {                                                                                      \
        if (blockIdx.x == 36 && blockIdx.y == 20 && (slot) < 128) g_pisa_bwd_trace[(slot)] = clock64(); \
    } while (0)
extern "C" int fbla_debug_pisa_bwd_trace(long long* out128) {
    return (int)cudaMemcpyFromSymbol(out128, g_pisa_bwd_trace, sizeof(long long) * 128);
}
#else
#define PISA_BSTAMP(slot) do { } while (0)
#endif

namespace pisa_tc_bwd {

constexpr int kThreads = 320;
constexpr int kEwThreads = 256;
constexpr int kBS = 64;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColDq = 0;       // dQ accumulator: D columns (r = Q h before the loop)
constexpr uint32_t kColS = 128;      // S: 64 columns; dkc / dvc use [128, 128 + D)
constexpr uint32_t kColDp = 192;     // dP: 64 columns
using namespace pisa_tcx;

struct Params {
    int ns, nt, T;
    float scale;
    int* status;
};

enum Bar {
    kLoad0 = 0, kRFull, kDrFull, kInitDone, kKFull /*2*/, kKEmpty = kKFull + 2 /*2*/, kVFull = kKEmpty + 2, kVEmpty,
    kSFull, kSEmpty, kDeFull, kDeEmpty, kXFull, kXEmpty, kDone, kBars
};

template <int D>
constexpr int tile_bytes() { return kBS * D * 2; }
// [Q | dO | 2 key tiles | value tile | ds | ds residual | p / den | row exchange | barriers | bookkeeping]
template <int D>
size_t smem_bytes(int nt, int ns) {
    return (size_t)5 * tile_bytes<D>() + 3 * kBlockBytes + 1024 + 256 + (size_t)8 * ((nt + 63) / 64) + (size_t)4 * ns;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 2)
pisa_bwd_q_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_o, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kc,
                     const __grid_constant__ CUtensorMap tm_vc, const __grid_constant__ CUtensorMap tm_h,
                     const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_dr, const Params p,
                     const int32_t* __restrict__ indices, const float* __restrict__ row_stats, float* __restrict__ dkc,
                     float* __restrict__ dvc, float* __restrict__ drow) {
    constexpr int kNB = D / 64;
    constexpr int kTile = tile_bytes<D>();
    constexpr int kHalf = D / 2;            // feature columns per warp of a lane window
    extern __shared__ __align__(1024) uint8_t sm[];
    uint8_t* q_t = sm;
    uint8_t* do_t = q_t + kTile;
    uint8_t* k_ring = do_t + kTile;         // two key tiles; before the loop: O, and rows 0-63 of h
    uint8_t* v_t = k_ring + 2 * kTile;      // value tile; before the loop: rows 64-127 of h
    uint8_t* de_t = v_t + kTile;            // scale * ds, 16-bit; before the loop the dr tile starts here
    uint8_t* dl_t = de_t + kBlockBytes;     // its rounding residual (bf16)
    uint8_t* pe_t = dl_t + kBlockBytes;     // p / den (groups of unselected blocks)
    float* xch = reinterpret_cast<float*>(pe_t + kBlockBytes);          // [2][64][2] partial row sums
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xch) + 1024);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int nch = (p.nt + 63) / 64;
    unsigned long long* sel_mask = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(bars) + 256);
    int* sel_idx = reinterpret_cast<int*>(sel_mask + nch);

    const int qb = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NI = p.ns + nch;
    const int32_t* idx = indices + ((size_t)bh * p.nt + qb) * p.ns;
    if ((ptx::smem_u32(sm) & 1023u) != 0) {          // uniform over the CTA
        if (threadIdx.x == 0) *p.status = 798;
        return;
    }
    const ptx::Abort ab{abort_flag, p.status};
#ifdef FBLA_PISA_TRACE_Q
#define PISA_QSTAMP(slot) PISA_BSTAMP(slot)
#else
#define PISA_QSTAMP(slot) do { } while (0)
#endif
    if (threadIdx.x == 0) PISA_QSTAMP(0);

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars[kLoad0], 1);
        ptx::mbar_init(&bars[kRFull], 1);
        ptx::mbar_init(&bars[kDrFull], kEwThreads);
        ptx::mbar_init(&bars[kInitDone], 1);
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&bars[kKFull + s], 1);
            ptx::mbar_init(&bars[kKEmpty + s], 1);
        }
        ptx::mbar_init(&bars[kVFull], 1);
        ptx::mbar_init(&bars[kVEmpty], 1);
        ptx::mbar_init(&bars[kSFull], 1);
        ptx::mbar_init(&bars[kSEmpty], kEwThreads);
        ptx::mbar_init(&bars[kDeFull], kEwThreads);
        ptx::mbar_init(&bars[kDeEmpty], 1);
        ptx::mbar_init(&bars[kXFull], 1);
        ptx::mbar_init(&bars[kXEmpty], kEwThreads);
        ptx::mbar_init(&bars[kDone], 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        // everything the part before the loop needs, on one barrier
        ptx::mbar_arrive_expect_tx(&bars[kLoad0], (3 + kNB) * kTile);
        for (int cb = 0; cb < kNB; ++cb) {
            ptx::tma_load_3d(q_t + cb * kBlockBytes, &tm_q, &bars[kLoad0], cb * 64, qb * kBS, bh);
            ptx::tma_load_3d(do_t + cb * kBlockBytes, &tm_do, &bars[kLoad0], cb * 64, qb * kBS, bh);
            ptx::tma_load_3d(k_ring + cb * kBlockBytes, &tm_o, &bars[kLoad0], cb * 64, qb * kBS, bh);
        }
        for (int hb = 0; hb < kNB; ++hb) {
            uint8_t* dst = hb == 0 ? k_ring + kTile : v_t;
            for (int cb = 0; cb < kNB; ++cb) ptx::tma_load_3d(dst + cb * kBlockBytes, &tm_h, &bars[kLoad0], cb * 64, hb * 64, bh);
        }
    }
    for (int i = threadIdx.x; i < nch; i += kThreads) sel_mask[i] = 0ull;
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, kTmemCols);
        ptx::tmem_relinquish();
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.ns; i += kThreads) {
        const int c = idx[i];
        sel_idx[i] = c;
        if (c >= 0 && c < p.nt) atomicOr(&sel_mask[c >> 6], 1ull << (c & 63));      // a bad index selects nothing
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer: the ring, once the tiles of the first part are free ----------------
            auto block_of = [&](int i) {
                const int c = sel_idx[i];
                return (c < 0 || c >= p.nt) ? 0 : c;         // a bad index: fetched, then masked out entirely
            };
            auto load_k = [&](int i) -> bool {
                const int s = i & 1;
                if (!ptx::mbar_wait(&bars[kKEmpty + s], ((i >> 1) & 1) ^ 1, ab, 811)) return false;
                ptx::mbar_arrive_expect_tx(&bars[kKFull + s], kTile);
                const CUtensorMap* m = i < p.ns ? &tm_k : &tm_kc;
                const int r0 = i < p.ns ? block_of(i) * kBS : (i - p.ns) * 64;
                for (int cb = 0; cb < kNB; ++cb)
                    ptx::tma_load_3d(k_ring + s * kTile + cb * kBlockBytes, m, &bars[kKFull + s], cb * 64, r0, bh);
                return true;
            };
            auto load_v = [&](int i) -> bool {
                if (i > 0 && !ptx::mbar_wait(&bars[kVEmpty], (i - 1) & 1, ab, 812)) return false;
                ptx::mbar_arrive_expect_tx(&bars[kVFull], kTile);
                const CUtensorMap* m = i < p.ns ? &tm_v : &tm_vc;
                const int r0 = i < p.ns ? block_of(i) * kBS : (i - p.ns) * 64;
                for (int cb = 0; cb < kNB; ++cb) ptx::tma_load_3d(v_t + cb * kBlockBytes, m, &bars[kVFull], cb * 64, r0, bh);
                return true;
            };
            bool okay = ptx::mbar_wait(&bars[kInitDone], 0, ab, 810);
            if (okay) okay = load_k(0);
            if (okay) okay = load_v(0);
            for (int i = 1; i <= NI && okay; ++i) {
                if (i < NI) okay = load_k(i);            // K(i): its slot was freed by dQ of iteration i - 2
                if (okay && i < NI) okay = load_v(i);    // V(i): freed by dP of iteration i - 1
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc_nn = ptx::instr_desc(64, 64, BF16, false, false);     // both operands K-major
            const uint32_t idesc_o = ptx::instr_desc(64, D, BF16, false, true);        // B MN-major
            const uint32_t idesc_t = ptx::instr_desc(64, D, BF16, true, true);         // A and B MN-major
            // descriptors of the first k-step of every operand tile (K-major "k", MN-major "m"); the rest are offsets
            constexpr int kTileUnits = kTile / 16;
            auto dk_ = [](const void* t) { return ptx::smem_desc(ptx::smem_u32(t), 16, 1024, ptx::kLayoutSw128); };
            auto dm_ = [](const void* t) { return ptx::smem_desc(ptx::smem_u32(t), kBlockBytes, 1024, ptx::kLayoutSw128); };
            const uint64_t q_k = dk_(q_t), q_m = dm_(q_t), do_k = dk_(do_t), do_m = dm_(do_t);
            const uint64_t de_k = dk_(de_t), de_m = dm_(de_t), dl_k = dk_(dl_t), pe_m = dm_(pe_t);
            const uint64_t kr_k = dk_(k_ring), kr_m = dm_(k_ring), v_k = dk_(v_t), v_m = dm_(v_t);
            bool okay = ptx::mbar_wait(&bars[kLoad0], 0, ab, 820);
            if (okay) {
                // r = Q h -> columns [0, D); rows 0-63 of h lie in the second key tile, rows 64-127 in the value tile
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColDq, q_k + kb * ptx::kDescBlock,
                                                                      kb == 0 ? kr_m + kTileUnits : v_m, idesc_o, kb != 0);
                ptx::mma_commit(&bars[kRFull]);
                okay = ptx::mbar_wait(&bars[kDrFull], 0, ab, 821);
            }
            if (okay) {
                // dQ = dr h^T: dq[row][d] = sum_vv dr[row][vv] h[d][vv]; the rows d of h lie in two tiles
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int nb = 0; nb < kNB; ++nb)
#pragma unroll
                    for (int kb = 0; kb < kNB; ++kb)
                        ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepK>(tmem + kColDq + nb * 64, de_k + kb * ptx::kDescBlock,
                                                                         (nb == 0 ? kr_k + kTileUnits : v_k) + kb * ptx::kDescBlock,
                                                                         idesc_nn, kb != 0);
                ptx::mma_commit(&bars[kInitDone]);
            }
            auto scores = [&](int i) -> bool {       // S = Q K^T and dP = dO V^T of iteration i
                const int s = i & 1;
                if (!ptx::mbar_wait(&bars[kKFull + s], (i >> 1) & 1, ab, 822)) return false;
                if (!ptx::mbar_wait(&bars[kVFull], i & 1, ab, 823)) return false;
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepK>(tmem + kColS, q_k + kb * ptx::kDescBlock,
                                                                     kr_k + s * kTileUnits + kb * ptx::kDescBlock, idesc_nn, kb != 0);
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepK>(tmem + kColDp, do_k + kb * ptx::kDescBlock,
                                                                     v_k + kb * ptx::kDescBlock, idesc_nn, kb != 0);
                ptx::mma_commit(&bars[kSFull]);
                ptx::mma_commit(&bars[kVEmpty]);
                return true;
            };
            // The dr tile occupies the ds tiles until dQ = dr h^T has run; the element-wise warps wait for
            // that themselves.  The first scores may go out at once: S, dP do not overlap the dQ columns.
            if (okay && NI > 0) okay = scores(0);
            int x_events = 0;
            for (int i = 0; i < NI && okay; ++i) {
                const bool exact = i < p.ns;
                if (exact && i + 1 < NI) {
                    if (!ptx::mbar_wait(&bars[kSEmpty], i & 1, ab, 824) || !scores(i + 1)) { okay = false; break; }
                }
                if (!ptx::mbar_wait(&bars[kDeFull], i & 1, ab, 825)) { okay = false; break; }
                PISA_QSTAMP(10 + i);
                ptx::tc_fence_after_sync();
                ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColDq, de_k, kr_m + (i & 1) * kTileUnits, idesc_o, true);
                if (BF16)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColDq, dl_k, kr_m + (i & 1) * kTileUnits, idesc_o, true);
                ptx::mma_commit(&bars[kKEmpty + (i & 1)]);
                if (exact) {
                    ptx::mma_commit(&bars[kDeEmpty]);
                } else {
                    // dkc = ds^T Q, then dvc = (p / den)^T dO, each into the columns of S and dP (both read by now)
                    for (int which = 0; which < 2 && okay; ++which) {
                        ptx::mma_ss_k4<ptx::kDescStepMN, ptx::kDescStepMN>(tmem + kColS, which ? pe_m : de_m, which ? do_m : q_m, idesc_t,
                                                                           false);
                        ptx::mma_commit(&bars[kXFull]);
                        if (which == 1) ptx::mma_commit(&bars[kDeEmpty]);
                        okay = ptx::mbar_wait(&bars[kXEmpty], x_events & 1, ab, 826);
                        ++x_events;
                        ptx::tc_fence_after_sync();
                    }
                    if (okay && i + 1 < NI) okay = scores(i + 1);
                }
            }
            if (okay) ptx::mma_commit(&bars[kDone]);
        }
    } else {
        // ---------------- element-wise warps ----------------
        const int ew = warp - 2;
        const int quarter = warp & 3, half = ew >> 2;
        const int c2 = (lane & 3) * 2;
        const int row_a = quarter * 16 + (lane >> 2), row_b = row_a + 8;
        const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        const int t0 = qb * kBS;
        const int nrows = min(kBS, p.T - t0);
        const size_t base_row = (size_t)bh * p.T;
        const float sm2 = p.scale * 1.44269504f;
        const float w = p.scale / (float)p.T;
        const int last_len = p.T - (p.nt - 1) * kBS;
        float m_row[2], rD[2], dD[2], dg[2];
        bool okay = ptx::mbar_wait(&bars[kLoad0], 0, ab, 830) && ptx::mbar_wait(&bars[kRFull], 0, ab, 831);
        if (threadIdx.x == 64) PISA_QSTAMP(1);
        if (okay) {
            ptx::tc_fence_after_sync();
            // od = rowsum(O dO), nr = rowsum(dO r): this warp's half of the feature columns
            float od[2] = {0.f, 0.f}, nr[2] = {0.f, 0.f};
#pragma unroll
            for (int c = 0; c < kHalf; c += 32) {
                float r[16];
                tmem_ld_16x256b_x4(t_lane + kColDq + half * kHalf + c, r);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int x = 0; x < 16; x += 2) {
                    const int rr = (x >> 1) & 1;
                    const int row = rr ? row_b : row_a;
                    const int col = half * kHalf + c + (x >> 2) * 8 + c2;
                    const float2 d2 = unpack2<BF16>(*pair_at(do_t, row, col));
                    const float2 o2 = unpack2<BF16>(*pair_at(k_ring, row, col));
                    od[rr] += d2.x * o2.x + d2.y * o2.y;
                    nr[rr] += d2.x * r[x] + d2.y * r[x + 1];
                }
            }
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                od[rr] += __shfl_xor_sync(0xffffffffu, od[rr], 1);
                od[rr] += __shfl_xor_sync(0xffffffffu, od[rr], 2);
                nr[rr] += __shfl_xor_sync(0xffffffffu, nr[rr], 1);
                nr[rr] += __shfl_xor_sync(0xffffffffu, nr[rr], 2);
            }
            if ((lane & 3) == 0) {
                *reinterpret_cast<float2*>(xch + (half * 64 + row_a) * 2) = make_float2(od[0], nr[0]);
                *reinterpret_cast<float2*>(xch + (half * 64 + row_b) * 2) = make_float2(od[1], nr[1]);
            }
        }
        ptx::tc_fence_before_sync();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        float gw[2] = {0.f, 0.f};
        if (okay) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = rr ? row_b : row_a;
                const float2 a = *reinterpret_cast<const float2*>(xch + row * 2);
                const float2 b = *reinterpret_cast<const float2*>(xch + (64 + row) * 2);
                const float od = a.x + b.x, nr = a.y + b.y;
                float g_row = 0.f;
                m_row[rr] = 0.f;
                rD[rr] = 0.f;
                if (row < nrows) {
                    const float4 st = *reinterpret_cast<const float4*>(row_stats + (base_row + t0 + row) * 4);
                    m_row[rr] = st.x;
                    rD[rr] = 1.f / st.y;
                    g_row = st.z;
                }
                dD[rr] = -od * rD[rr];
                dg[rr] = dD[rr] + nr * rD[rr] * w;
                gw[rr] = g_row * w * rD[rr];
                if (half == 0 && (lane & 3) == 0 && row < nrows) drow[base_row + t0 + row] = dD[rr];
            }
            // dr = dO g w / den: this warp's columns of the dr tile (it starts where the ds tiles will be)
#pragma unroll
            for (int c = 0; c < kHalf; c += 8) {
                const int col = half * kHalf + c + c2;
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int row = rr ? row_b : row_a;
                    const float2 d2 = unpack2<BF16>(*pair_at(do_t, row, col));
                    *pair_at(de_t, row, col) = pack2<BF16>(d2.x * gw[rr], d2.y * gw[rr]);
                }
            }
            ptx::fence_proxy_async_smem();
        }
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(&bars[kDrFull]);
        if (threadIdx.x == 64 && okay) {
            // the dr rows also go to global memory (the state pass forms dh = q^T dr from them)
            if (ptx::mbar_wait(&bars[kDrFull], 0, ab, 832)) {
                for (int cb = 0; cb < kNB; ++cb) ptx::tma_store_3d(&tm_dr, de_t + cb * kBlockBytes, cb * 64, t0, bh);
                ptx::tma_store_commit();
                ptx::tma_store_wait_read<0>();
            }
        }
        // the ds tiles may be written once dQ = dr h^T has read the dr tile and the store above has, too
        if (okay) okay = ptx::mbar_wait(&bars[kInitDone], 0, ab, 833);
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (threadIdx.x == 64) PISA_QSTAMP(3);

        // scale folded into the per-row constants: scale * ds = p (dP rDs + dDs)
        const float neg_m[2] = {-m_row[0], -m_row[1]};
        const float rDs[2] = {rD[0] * p.scale, rD[1] * p.scale};
        const float dDs[2] = {dD[0] * p.scale, dD[1] * p.scale};
        const float dgs[2] = {dg[0] * p.scale, dg[1] * p.scale};
        int x_events = 0;
        for (int i = 0; i < NI && okay; ++i) {
            float s[16], dp[16];
            if (!ptx::mbar_wait(&bars[kSFull], i & 1, ab, 834)) { okay = false; break; }
            if (threadIdx.x == 64) PISA_QSTAMP(30 + i);
            ptx::tc_fence_after_sync();
            tmem_ld_16x256b_x4(t_lane + kColS + half * 32, s);
            tmem_ld_16x256b_x4(t_lane + kColDp + half * 32, dp);
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[kSEmpty]);
            const bool approx = i >= p.ns;
            int nvalid, jl = -1, c0 = 0;
            unsigned long long keep = ~0ull;
            if (!approx) {
                const int cb = sel_idx[i];
                nvalid = (cb < 0 || cb >= p.nt) ? 0 : min(kBS, p.T - cb * kBS);
            } else {
                c0 = (i - p.ns) * 64;
                nvalid = min(64, p.nt - c0);
                keep = ~sel_mask[i - p.ns];
                if (last_len != kBS) jl = p.nt - 1 - c0;     // position of the shorter last block, if in this group
            }
            keep &= nvalid >= 64 ? ~0ull : ((1ull << nvalid) - 1ull);
            const unsigned long long keep_t = keep >> (half * 32 + c2);      // bit 8 g + (x & 1): this thread's columns
            const int jl_t = jl - half * 32 - c2;
            uint32_t hi[8], lo[8], pe[8];
            if (!approx && keep == ~0ull) {
                // a full selected block (the common case): nothing to mask, p / den is not needed
#pragma unroll
                for (int x = 0; x < 16; x += 2) {
                    const int rr = (x >> 1) & 1;
                    const float d0 = exp2f(fmaf(s[x], sm2, neg_m[rr])) * fmaf(dp[x], rDs[rr], dDs[rr]);
                    const float d1 = exp2f(fmaf(s[x + 1], sm2, neg_m[rr])) * fmaf(dp[x + 1], rDs[rr], dDs[rr]);
                    hi[x >> 1] = pack2<BF16>(d0, d1);
                    if (BF16) {
                        const float2 f = unpack2<BF16>(hi[x >> 1]);
                        lo[x >> 1] = pack2<BF16>(d0 - f.x, d1 - f.y);
                    }
                }
            } else {
#pragma unroll
                for (int x = 0; x < 16; x += 2) {
                    const int rr = (x >> 1) & 1;
                    float de2[2], pe2[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int bit = (x >> 2) * 8 + u;
                        const bool ok = (keep_t >> bit) & 1ull;
                        const float pj = ok ? exp2f(fmaf(s[x + u], sm2, neg_m[rr])) : 0.f;
                        float dpj;
                        if (approx) {
                            const float len = (bit == jl_t) ? (float)last_len : (float)kBS;
                            dpj = fmaf(dp[x + u], rDs[rr], dgs[rr] * len);
                        } else {
                            dpj = fmaf(dp[x + u], rDs[rr], dDs[rr]);
                        }
                        de2[u] = pj * dpj;
                        pe2[u] = pj * rD[rr];
                    }
                    hi[x >> 1] = pack2<BF16>(de2[0], de2[1]);
                    if (BF16) {
                        const float2 f = unpack2<BF16>(hi[x >> 1]);
                        lo[x >> 1] = pack2<BF16>(de2[0] - f.x, de2[1] - f.y);
                    }
                    pe[x >> 1] = pack2<BF16>(pe2[0], pe2[1]);
                }
            }
            if (threadIdx.x == 64) PISA_QSTAMP(50 + i);
            if (i > 0 && !ptx::mbar_wait(&bars[kDeEmpty], (i - 1) & 1, ab, 835)) { okay = false; break; }
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const int row = (x & 1) ? row_b : row_a;
                const uint32_t off = row * 128 + ((((half * 4 + (x >> 1)) ^ row) & 7) << 4) + c2 * 2;
                *reinterpret_cast<uint32_t*>(de_t + off) = hi[x];
                if (BF16) *reinterpret_cast<uint32_t*>(dl_t + off) = lo[x];
                if (approx) *reinterpret_cast<uint32_t*>(pe_t + off) = pe[x];
            }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[kDeFull]);
            if (threadIdx.x == 64) PISA_QSTAMP(70 + i);
            if (approx) {
                // dkc, then dvc, of the 64 blocks of this group: rows = blocks, this warp's half of the features
                for (int which = 0; which < 2 && okay; ++which) {
                    if (!ptx::mbar_wait(&bars[kXFull], x_events & 1, ab, 836)) { okay = false; break; }
                    ++x_events;
                    ptx::tc_fence_after_sync();
                    float* outp = (which ? dvc : dkc) + ((size_t)bh * p.nt + c0) * D;
#pragma unroll
                    for (int c = 0; c < kHalf; c += 32) {
                        float r[16];
                        tmem_ld_16x256b_x4(t_lane + kColS + half * kHalf + c, r);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int x = 0; x < 16; x += 2) {
                            const int blk = ((x >> 1) & 1) ? row_b : row_a;
                            const int col = half * kHalf + c + (x >> 2) * 8 + c2;
                            if (blk < nvalid) red_add2(outp + (size_t)blk * D + col, r[x], r[x + 1]);
                        }
                    }
                    ptx::tc_fence_before_sync();
                    ptx::mbar_arrive(&bars[kXEmpty]);
                }
            }
        }
        if (okay) okay = ptx::mbar_wait(&bars[kDone], 0, ab, 837);
        if (threadIdx.x == 64) PISA_QSTAMP(92);
        if (okay) {
            ptx::tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < kHalf; c += 32) {
                float r[16];
                tmem_ld_16x256b_x4(t_lane + kColDq + half * kHalf + c, r);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int x = 0; x < 16; x += 2) {
                    const int row = ((x >> 1) & 1) ? row_b : row_a;
                    const int col = half * kHalf + c + (x >> 2) * 8 + c2;
                    *pair_at(q_t, row, col) = pack2<BF16>(r[x], r[x + 1]);     // the query tile is free: every product is done
                }
            }
            ptx::fence_proxy_async_smem();
        }
        ptx::tc_fence_before_sync();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (okay && threadIdx.x == 64) {
            for (int cb = 0; cb < kNB; ++cb) ptx::tma_store_3d(&tm_dq, q_t + cb * kBlockBytes, cb * 64, t0, bh);
            ptx::tma_store_commit();
            ptx::tma_store_wait_read<0>();
            PISA_QSTAMP(94);
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace pisa_tc_bwd

// ------------------------------------------------------------------------------------------------
// Key-side backward: one CTA per key block; it visits the query blocks that selected the block and
// works transposed (keys are the M dimension), so that the weights feed dV += P^T dO and
// dK += dS^T Q as K-major A operands:
//     S^T = K Q^T,  dP^T = V dO^T    tcgen05.mma, M = N = 64, two TMEM buffers
//     p / den, ds scale              16 element-wise warps (four per TMEM lane window, 16 columns each);
//                                    the per-column constants (m, 1 / den, dD of a query row) are
//                                    fetched from global memory while the scores are still in flight
//     dV += (p / den)^T-tile dO,  dK += ds^T-tile Q     accumulators in TMEM (bf16: plus residual tiles)
// The statistics terms dk += dkc / len + (v - vc / len) dh^T, dv += dvc + (k - kc) dh are split: the
// products with the uncentred tiles, dK = V dh^T and dV = K dh, are the first thing the tensor cores do
// (they initialise the accumulators), and what is the same for every key of a block,
// dkc / len - (vc / len) dh^T and dvc - kc dh, is formed per block by pisa_stats_terms_kernel beforehand
// (with the same 16-bit rounding of dh, so that the two halves cancel as they would in the centred form).
namespace pisa_tc_kvside {

constexpr int kEwThreads = 512;
constexpr int kThreads = 64 + kEwThreads;
constexpr int kBS = 64;
constexpr int kQStages = 3;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColDk = 0, kColDv = 128, kColS = 256;    // S^T buffer b at kColS + 128 b, dP^T 64 columns after it
using namespace pisa_tcx;
using pisa_tc_bwd::Params;

enum Bar { kKvFull = 0, kQFull = 1, kQEmpty = 4, kSFull = 7, kSEmpty = 9, kAFull = 11, kAEmpty = 13, kDhFull = 15, kDone = 16, kBars = 17 };

template <int D>
constexpr int tile_bytes() { return kBS * D * 2; }
// [K | V | 3 x (Q, dO) | dh | 2 x (p/den, its residual, ds, its residual) | barriers | visit list]
template <int D>
size_t smem_bytes(int nt) {
    return (size_t)(2 + 2 * kQStages) * tile_bytes<D>() + (size_t)D * D * 2 + 8 * kBlockBytes + 256 + (size_t)4 * nt +
           (size_t)((nt + 15) & ~15);
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
pisa_bwd_kv_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                      const __grid_constant__ CUtensorMap tm_dh, const Params p, const int32_t* __restrict__ indices,
                      const float* __restrict__ row_stats, const float* __restrict__ drow, const float* __restrict__ dkc,
                      const float* __restrict__ dvc) {
    constexpr int kNB = D / 64;
    constexpr int kTile = tile_bytes<D>();
    constexpr int kPart = D / 4;            // feature columns per warp of a lane window in the epilogue
    extern __shared__ __align__(1024) uint8_t sm[];
    uint8_t* k_t = sm;
    uint8_t* v_t = k_t + kTile;
    uint8_t* q_ring = v_t + kTile;                      // stage s: Q at + 2 s kTile, dO one tile after
    uint8_t* dh_t = q_ring + 2 * kQStages * kTile;      // dh as 64-column blocks of [D rows][64]
    uint8_t* a_t = dh_t + D * D * 2;                    // buffer b: + 4 b kBlockBytes: p/den, residual, ds, residual
    uint64_t* bars = reinterpret_cast<uint64_t*>(a_t + 8 * kBlockBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* n_hit = reinterpret_cast<int*>(tmem_slot + 2);
    int* hlist = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 256);
    unsigned char* hit = reinterpret_cast<unsigned char*>(hlist + p.nt);

    const int c_blk = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bos = c_blk * kBS;
    const int nkeys = min(kBS, p.T - bos);
    const size_t base_row = (size_t)bh * p.T;
    if ((ptx::smem_u32(sm) & 1023u) != 0) {          // uniform over the CTA
        if (threadIdx.x == 0) *p.status = 797;
        return;
    }
    const ptx::Abort ab{abort_flag, p.status};

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars[kKvFull], 1);
        for (int s = 0; s < kQStages; ++s) {
            ptx::mbar_init(&bars[kQFull + s], 1);
            ptx::mbar_init(&bars[kQEmpty + s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&bars[kSFull + s], 1);
            ptx::mbar_init(&bars[kSEmpty + s], kEwThreads);
            ptx::mbar_init(&bars[kAFull + s], kEwThreads);
            ptx::mbar_init(&bars[kAEmpty + s], 1);
        }
        ptx::mbar_init(&bars[kDhFull], 1);
        ptx::mbar_init(&bars[kDone], 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::mbar_arrive_expect_tx(&bars[kKvFull], 2 * kTile);
        for (int cb = 0; cb < kNB; ++cb) {
            ptx::tma_load_3d(k_t + cb * kBlockBytes, &tm_k, &bars[kKvFull], cb * 64, bos, bh);
            ptx::tma_load_3d(v_t + cb * kBlockBytes, &tm_v, &bars[kKvFull], cb * 64, bos, bh);
        }
        ptx::mbar_arrive_expect_tx(&bars[kDhFull], D * D * 2);
        for (int vb = 0; vb < kNB; ++vb)
            for (int db = 0; db < kNB; ++db)
                ptx::tma_load_3d(dh_t + vb * (D * 128) + db * kBlockBytes, &tm_dh, &bars[kDhFull], vb * 64, db * 64, bh);
    }
    if (threadIdx.x == 0) PISA_BSTAMP(0);
    // which query blocks selected this key block, in block order (the accumulation order is fixed)
    for (int i = threadIdx.x; i < p.nt; i += kThreads) {
        const int32_t* idx = indices + ((size_t)bh * p.nt + i) * p.ns;
        bool any = false;
        for (int n = 0; n < p.ns; ++n) any |= (idx[n] == c_blk);
        hit[i] = any ? 1 : 0;
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, kTmemCols);
        ptx::tmem_relinquish();
    }
    __syncthreads();
    if (warp == 0) {
        int count = 0;
        for (int base = 0; base < p.nt; base += 32) {
            const int i = base + lane;
            const bool bit = i < p.nt && hit[i] != 0;
            const unsigned mask = __ballot_sync(0xffffffffu, bit);
            if (bit) hlist[count + __popc(mask & ((1u << lane) - 1u))] = i;
            count += __popc(mask);
        }
        if (lane == 0) *n_hit = count;
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const int nh = *n_hit;
    if (threadIdx.x == 0) PISA_BSTAMP(1);

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer: (Q, dO) of the visiting query blocks ----------------
            for (int j = 0; j < nh; ++j) {
                const int s = j % kQStages;
                if (!ptx::mbar_wait(&bars[kQEmpty + s], ((j / kQStages) & 1) ^ 1, ab, 851)) break;
                ptx::mbar_arrive_expect_tx(&bars[kQFull + s], 2 * kTile);
                const int t0 = hlist[j] * kBS;
                for (int cb = 0; cb < kNB; ++cb) {
                    ptx::tma_load_3d(q_ring + 2 * s * kTile + cb * kBlockBytes, &tm_q, &bars[kQFull + s], cb * 64, t0, bh);
                    ptx::tma_load_3d(q_ring + (2 * s + 1) * kTile + cb * kBlockBytes, &tm_do, &bars[kQFull + s], cb * 64, t0, bh);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc_nn = ptx::instr_desc(64, 64, BF16, false, false);
            const uint32_t idesc_kk = ptx::instr_desc(64, D, BF16, false, false);
            const uint32_t idesc_o = ptx::instr_desc(64, D, BF16, false, true);
            constexpr int kTileUnits = kTile / 16;
            auto dk_ = [](const void* t) { return ptx::smem_desc(ptx::smem_u32(t), 16, 1024, ptx::kLayoutSw128); };
            auto dm_ = [](const void* t) { return ptx::smem_desc(ptx::smem_u32(t), kBlockBytes, 1024, ptx::kLayoutSw128); };
            const uint64_t k_k = dk_(k_t), v_k = dk_(v_t), ring_k = dk_(q_ring), ring_m = dm_(q_ring), a_k = dk_(a_t);
            const uint64_t dh_k = dk_(dh_t);
            const uint64_t dh_m = ptx::smem_desc(ptx::smem_u32(dh_t), D * 128, 1024, ptx::kLayoutSw128);
            auto scores = [&](int j) -> bool {
                const int s = j % kQStages, b = j & 1;
                if (!ptx::mbar_wait(&bars[kQFull + s], (j / kQStages) & 1, ab, 861)) return false;
                if (!ptx::mbar_wait(&bars[kSEmpty + b], ((j >> 1) & 1) ^ 1, ab, 862)) return false;
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepK>(tmem + kColS + b * 128, k_k + kb * ptx::kDescBlock,
                                                                     ring_k + 2 * s * kTileUnits + kb * ptx::kDescBlock, idesc_nn,
                                                                     kb != 0);
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepK>(tmem + kColS + b * 128 + 64, v_k + kb * ptx::kDescBlock,
                                                                     ring_k + (2 * s + 1) * kTileUnits + kb * ptx::kDescBlock, idesc_nn,
                                                                     kb != 0);
                ptx::mma_commit(&bars[kSFull + b]);
                return true;
            };
            bool okay = ptx::mbar_wait(&bars[kKvFull], 0, ab, 860) && ptx::mbar_wait(&bars[kDhFull], 0, ab, 864);
            if (okay) {
                ptx::tc_fence_after_sync();
                // dk[key][d] = sum_vv v[key][vv] dh[d][vv]: rows d of dh are the N dimension (blocks of 64 vv)
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepK>(tmem + kColDk, v_k + kb * ptx::kDescBlock, dh_k + kb * (D * 128 / 16),
                                                                     idesc_kk, kb != 0);
                // dv[key][vv] = sum_d k[key][d] dh[d][vv]: rows d of dh are the K dimension
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColDv, k_k + kb * ptx::kDescBlock, dh_m + kb * ptx::kDescBlock,
                                                                      idesc_o, kb != 0);
            }
            if (okay && nh > 0) okay = scores(0);
            for (int j = 0; j < nh && okay; ++j) {
                const int s = j % kQStages, b = j & 1;
                if (j + 1 < nh && !scores(j + 1)) { okay = false; break; }
                if (!ptx::mbar_wait(&bars[kAFull + b], (j >> 1) & 1, ab, 863)) { okay = false; break; }
                PISA_BSTAMP(10 + j);
                ptx::tc_fence_after_sync();
                const uint64_t q_m = ring_m + 2 * s * kTileUnits, do_m = q_m + kTileUnits;
                const uint64_t pe_k = a_k + 4 * b * ptx::kDescBlock;
                ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColDv, pe_k, do_m, idesc_o, true);
                if (BF16) ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColDv, pe_k + ptx::kDescBlock, do_m, idesc_o, true);
                ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColDk, pe_k + 2 * ptx::kDescBlock, q_m, idesc_o, true);
                if (BF16) ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColDk, pe_k + 3 * ptx::kDescBlock, q_m, idesc_o, true);
                ptx::mma_commit(&bars[kAEmpty + b]);
                ptx::mma_commit(&bars[kQEmpty + s]);
            }
            if (okay) ptx::mma_commit(&bars[kDone]);
        }
    } else {
        // ---------------- element-wise warps ----------------
        const int ew = warp - 2;
        const int quarter = warp & 3, part = ew >> 2;
        const int c2 = (lane & 3) * 2;
        const int key_a = quarter * 16 + (lane >> 2), key_b = key_a + 8;
        const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        const float sm2 = p.scale * 1.44269504f;
        bool okay = true;
        // Constants of this thread's four query rows (columns part * 16 + 8 g + c2 + u) of a visit: (m, 1 / den) and dD.
        // They are fetched one visit ahead and not touched before they are needed: the first use of a loaded
        // register is where a thread waits for the load.
        float4 st_next[2][2];
        float dd_next[2][2];
        auto fetch = [&](int j) {
            const int t0 = hlist[j] * kBS;
            const int nrows = min(kBS, p.T - t0);
#pragma unroll
            for (int g = 0; g < 2; ++g)
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int r = min(part * 16 + g * 8 + c2 + u, nrows - 1);      // padded rows are masked when used
                    st_next[g][u] = __ldg(reinterpret_cast<const float4*>(row_stats + (base_row + t0 + r) * 4));
                    dd_next[g][u] = __ldg(drow + base_row + t0 + r);
                }
        };
        if (nh > 0) fetch(0);
        for (int j = 0; j < nh; ++j) {
            const int b = j & 1;
            const int nrows = min(kBS, p.T - hlist[j] * kBS);
            float neg_m[2][2], rd[2][2], rds[2][2], dd[2][2];
#pragma unroll
            for (int g = 0; g < 2; ++g)
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const bool valid = part * 16 + g * 8 + c2 + u < nrows;      // 1/den = 0 and dD = 0: a padded row contributes nothing
                    neg_m[g][u] = valid ? -st_next[g][u].x : 0.f;
                    rd[g][u] = valid ? st_next[g][u].w : 0.f;
                    dd[g][u] = valid ? dd_next[g][u] * p.scale : 0.f;      // scale folded in: scale * ds = p (dP rds + dds)
                    rds[g][u] = rd[g][u] * p.scale;
                }
            if (j + 1 < nh) fetch(j + 1);
            float s[8], dp[8];
            if (threadIdx.x == 64) PISA_BSTAMP(100 + j);
            if (!ptx::mbar_wait(&bars[kSFull + b], (j >> 1) & 1, ab, 871)) { okay = false; break; }
            if (threadIdx.x == 64) PISA_BSTAMP(30 + j);
            ptx::tc_fence_after_sync();
            tmem_ld_16x256b_x2(t_lane + kColS + b * 128 + part * 16, s);
            tmem_ld_16x256b_x2(t_lane + kColS + b * 128 + 64 + part * 16, dp);
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[kSEmpty + b]);
            uint32_t pa[4], pl[4], da[4], dl[4];
#pragma unroll
            for (int x = 0; x < 8; x += 2) {
                const int g = x >> 2;
                float pe2[2], de2[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float pj = exp2f(fmaf(s[x + u], sm2, neg_m[g][u]));
                    pe2[u] = pj * rd[g][u];
                    de2[u] = pj * fmaf(dp[x + u], rds[g][u], dd[g][u]);
                }
                pa[x >> 1] = pack2<BF16>(pe2[0], pe2[1]);
                da[x >> 1] = pack2<BF16>(de2[0], de2[1]);
                if (BF16) {
                    const float2 f = unpack2<BF16>(pa[x >> 1]);
                    pl[x >> 1] = pack2<BF16>(pe2[0] - f.x, pe2[1] - f.y);
                    const float2 h2 = unpack2<BF16>(da[x >> 1]);
                    dl[x >> 1] = pack2<BF16>(de2[0] - h2.x, de2[1] - h2.y);
                }
            }
            if (threadIdx.x == 64) PISA_BSTAMP(50 + j);
            if (!ptx::mbar_wait(&bars[kAEmpty + b], ((j >> 1) & 1) ^ 1, ab, 872)) { okay = false; break; }
            uint8_t* ab_t = a_t + 4 * b * kBlockBytes;
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int row = (x & 1) ? key_b : key_a;
                const uint32_t off = row * 128 + ((((part * 2 + (x >> 1)) ^ row) & 7) << 4) + c2 * 2;
                *reinterpret_cast<uint32_t*>(ab_t + off) = pa[x];
                *reinterpret_cast<uint32_t*>(ab_t + 2 * kBlockBytes + off) = da[x];
                if (BF16) {
                    *reinterpret_cast<uint32_t*>(ab_t + kBlockBytes + off) = pl[x];
                    *reinterpret_cast<uint32_t*>(ab_t + 3 * kBlockBytes + off) = dl[x];
                }
            }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[kAFull + b]);
            if (threadIdx.x == 64) PISA_BSTAMP(70 + j);
        }
        if (threadIdx.x == 64) PISA_BSTAMP(90);
        if (okay) okay = ptx::mbar_wait(&bars[kDone], 0, ab, 875);
        if (threadIdx.x == 64) PISA_BSTAMP(92);
        if (okay) {
            ptx::tc_fence_after_sync();
            // what every key of the block receives alike (pisa_stats_terms_kernel left it in dkc, dvc)
            const float* dkcb = dkc + ((size_t)bh * p.nt + c_blk) * D;
            const float* dvcb = dvc + ((size_t)bh * p.nt + c_blk) * D;
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                uint8_t* tile = which ? v_t : k_t;          // the key and value tiles are free: every product is done
                const float* add = which ? dvcb : dkcb;
#pragma unroll
                for (int c = 0; c < kPart; c += 16) {
                    float r[8];
                    tmem_ld_16x256b_x2(t_lane + (which ? kColDv : kColDk) + part * kPart + c, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int x = 0; x < 8; x += 2) {
                        const int row = ((x >> 1) & 1) ? key_b : key_a;
                        const int col = part * kPart + c + (x >> 2) * 8 + c2;
                        const float2 a2 = *reinterpret_cast<const float2*>(add + col);
                        *pair_at(tile, row, col) = pack2<BF16>(a2.x + r[x], a2.y + r[x + 1]);
                    }
                }
            }
            ptx::fence_proxy_async_smem();
        }
        if (threadIdx.x == 64) PISA_BSTAMP(93);
        ptx::tc_fence_before_sync();
        asm volatile("bar.sync 1, 512;" ::: "memory");
        if (okay && threadIdx.x == 64) {
            for (int cb = 0; cb < kNB; ++cb) {
                ptx::tma_store_3d(&tm_dk, k_t + cb * kBlockBytes, cb * 64, bos, bh);
                ptx::tma_store_3d(&tm_dv, v_t + cb * kBlockBytes, cb * 64, bos, bh);
            }
            ptx::tma_store_commit();
            ptx::tma_store_wait_read<0>();
            PISA_BSTAMP(94);
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, kTmemCols);
    }
    if (threadIdx.x == 0) PISA_BSTAMP(2);
}

// dkc <- dkc / len - (vc / len) dh^T and dvc <- dvc - kc dh per key block (in place), with dh rounded to the
// 16-bit type as the tensor-core products see it; the CTAs of the first block group also write that copy out.
// Eight key blocks per CTA, one thread per feature.
constexpr int kTermBlocks = 8;
template <bool BF16>
__global__ void __launch_bounds__(128)
pisa_stats_terms_kernel(int D, int nt, int T, const float* __restrict__ kc, const float* __restrict__ vc,
                        const float* __restrict__ dh, float* __restrict__ dkc, float* __restrict__ dvc,
                        uint32_t* __restrict__ dh16) {
    __shared__ __align__(16) uint16_t dhs[128 * 130];   // rows padded by two elements: a column walk touches every bank
                                                        // (read and written as 32-bit pairs)
    __shared__ float kcs[128], vcs[128];
    const int bh = blockIdx.y, t = threadIdx.x;
    const int stride = D + 2;
    const float* dhb = dh + (size_t)bh * D * D;
    for (int i = t; i < D * D / 2; i += 128) {
        const float2 f = *reinterpret_cast<const float2*>(dhb + 2 * i);
        const uint32_t w = pack2<BF16>(f.x, f.y);
        const int d = (2 * i) / D, vv = 2 * i - d * D;
        *reinterpret_cast<uint32_t*>(&dhs[d * stride + vv]) = w;
        if (blockIdx.x == 0) dh16[(size_t)bh * D * D / 2 + i] = w;
    }
    for (int cc = 0; cc < kTermBlocks; ++cc) {
        const int c = blockIdx.x * kTermBlocks + cc;
        if (c >= nt) break;                     // uniform over the CTA
        const float inv_len = 1.f / (float)min(kBS, T - c * kBS);
        const size_t row = ((size_t)bh * nt + c) * D;
        __syncthreads();
        if (t < D) {
            kcs[t] = kc[row + t];
            vcs[t] = vc[row + t] * inv_len;
        }
        __syncthreads();
        if (t < D) {
            float uk = 0.f, uv = 0.f;
            for (int x = 0; x < D; x += 2) {
                const float2 r = unpack2<BF16>(*reinterpret_cast<const uint32_t*>(&dhs[t * stride + x]));   // dh[t][x], dh[t][x+1]
                uk = fmaf(vcs[x], r.x, uk);
                uk = fmaf(vcs[x + 1], r.y, uk);
            }
            for (int d = 0; d < D; ++d) {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(&dhs[d * stride + (t & ~1)]);
                const float2 r = unpack2<BF16>(w);
                uv = fmaf(kcs[d], (t & 1) ? r.y : r.x, uv);
            }
            dkc[row + t] = dkc[row + t] * inv_len - uk;
            dvc[row + t] = dvc[row + t] - uv;
        }
    }
}

}  // namespace pisa_tc_kvside

cudaError_t pisa_tc_bwd_kv(int dtype, int bh, int d, int nt, int ns, int T, float scale, const void* q, const void* k,
                           const void* v, const void* d_o, const float* kc, const float* vc, const int32_t* indices,
                           const float* row_stats, const float* drow, float* dkc, float* dvc, const float* dh, void* dh16,
                           void* dk, void* dv, cudaStream_t st) {
    using namespace pisa_tc_kvside;
    const bool bf = dtype == FBLA_BF16;
    {
        const dim3 grid((nt + kTermBlocks - 1) / kTermBlocks, bh);
        if (bf) pisa_stats_terms_kernel<true><<<grid, 128, 0, st>>>(d, nt, T, kc, vc, dh, dkc, dvc, static_cast<uint32_t*>(dh16));
        else pisa_stats_terms_kernel<false><<<grid, 128, 0, st>>>(d, nt, T, kc, vc, dh, dkc, dvc, static_cast<uint32_t*>(dh16));
    }
    CUtensorMap mk, mv, mq, mdo, mdk, mdv, mdh;
    cudaError_t e;
    if ((e = tc_encode_map_rows(&mk, k, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mv, v, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mq, q, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mdo, d_o, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mdk, dk, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mdv, dv, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mdh, dh16, dtype, d, d, bh, 64)) != cudaSuccess) return e;
    Params p{ns, nt, T, scale, tc_status_word()};
    if (p.status == nullptr) return cudaErrorMemoryAllocation;
    const dim3 grid(nt, bh);
    auto run = [&](auto kern, size_t smem) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            kern<<<grid, kThreads, smem, st>>>(mk, mv, mq, mdo, mdk, mdv, mdh, p, indices, row_stats, drow, dkc, dvc);
    };
    if (d == 64) {
        if (bf) run(pisa_bwd_kv_tc_kernel<64, true>, smem_bytes<64>(nt));
        else run(pisa_bwd_kv_tc_kernel<64, false>, smem_bytes<64>(nt));
    } else {
        if (bf) run(pisa_bwd_kv_tc_kernel<128, true>, smem_bytes<128>(nt));
        else run(pisa_bwd_kv_tc_kernel<128, false>, smem_bytes<128>(nt));
    }
    return e == cudaSuccess ? cudaGetLastError() : e;
}

// The key-side kernel keeps one CTA per SM busy with 3 (Q, dO) stages and dh resident: it fits up to this many blocks.
bool pisa_tc_bwd_kv_fits(int d, int nt) {
    return (d == 64 ? pisa_tc_kvside::smem_bytes<64>(nt) : pisa_tc_kvside::smem_bytes<128>(nt)) <= 232448;
}

cudaError_t pisa_tc_bwd_q(int dtype, int bh, int d, int nt, int ns, int T, float scale, const void* q, const void* k,
                          const void* v, const void* o, const void* d_o, const void* kc16, const void* vc16, const void* h16,
                          const int32_t* indices, const float* row_stats, void* dq, void* dr, float* dkc, float* dvc,
                          float* drow, cudaStream_t st) {
    using namespace pisa_tc_bwd;
    CUtensorMap mq, mdo, mo, mk, mv, mkc, mvc, mh, mdq, mdr;
    cudaError_t e;
    if ((e = tc_encode_map_rows(&mq, q, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mdo, d_o, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mo, o, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mk, k, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mv, v, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mkc, kc16, dtype, d, nt, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mvc, vc16, dtype, d, nt, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mh, h16, dtype, d, d, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mdq, dq, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mdr, dr, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    Params p{ns, nt, T, scale, tc_status_word()};
    if (p.status == nullptr) return cudaErrorMemoryAllocation;
    const dim3 grid(nt, bh);
    const bool bf = dtype == FBLA_BF16;
    auto run = [&](auto kern, size_t smem) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            kern<<<grid, kThreads, smem, st>>>(mq, mdo, mo, mk, mv, mkc, mvc, mh, mdq, mdr, p, indices, row_stats, dkc, dvc, drow);
    };
    if (d == 64) {
        if (bf) run(pisa_bwd_q_tc_kernel<64, true>, smem_bytes<64>(nt, ns));
        else run(pisa_bwd_q_tc_kernel<64, false>, smem_bytes<64>(nt, ns));
    } else {
        if (bf) run(pisa_bwd_q_tc_kernel<128, true>, smem_bytes<128>(nt, ns));
        else run(pisa_bwd_q_tc_kernel<128, false>, smem_bytes<128>(nt, ns));
    }
    return e == cudaSuccess ? cudaGetLastError() : e;
}

}  // namespace fbla
