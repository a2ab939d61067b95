// Forward of the piecewise sparse attention stage on the 5th-generation tensor cores
// (reference: piecewise_sparse_attention_fwd_kernel, flash_bla/ops/piecewise_attn/kernel.py:189-292).
//
// One CTA per block of 64 queries of one (batch, head).  Every key block the query block selected
// (exact softmax attention) and every group of 64 unselected blocks (their means as keys, their sums
// as values: the zeroth-order term) is one iteration of the same loop:
//     S = Q K^T          tcgen05.mma, M = 64, N = 64, accumulator in TMEM
//     P = exp2(S - m)    a warp reads its 16 rows of S from TMEM with all 32 lanes (16x256b shape)
//     O (+)= P V         tcgen05.mma, P staged in shared memory, accumulator in TMEM
// followed by r = Q h (the first-order term) and out = (O + r g scale / T) / (l + g).
//
//   warp 0      TMA producer: Q once, then a three-deep ring of key tiles and a two-deep ring of
//               value tiles (a key tile is free as soon as its scores are formed), then h
//   warp 1      MMA issuer (one thread) and owner of the TMEM allocation
//   warps 2-5   softmax and epilogue; with M = 64 the accumulator row r lives in TMEM lane
//               (r % 16) + 32 * (r / 16): each warp owns the 16 rows of its lane window
//
// The score MMA of iteration i + 1 is issued before the weights of iteration i are waited for, so
// the softmax of one block overlaps the tensor-core work of its neighbours; S is double-buffered.
// O is rescaled in TMEM (tcgen05.ld / tcgen05.st) only when a row's running maximum moved.
// The block statistics and h arrive as 16-bit copies so that TMA can fetch them like the keys.
// Every wait is bounded and reports through the library's status word.
#include "pisa_tc.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "pisa_tc_common.cuh"
#include "tc_kernels.cuh"
#include "tc_ptx.cuh"

namespace fbla {
namespace pisa_tc {

constexpr int kThreads = 192;
constexpr int kBS = 64;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColO = 0;        // O: D columns
constexpr uint32_t kColS = 128;      // S: two buffers of 64 columns; r = Q h reuses them at the end
using namespace pisa_tcx;

struct Params {
    int ns, nt, T;
    float scale;
    int* status;
};

constexpr int kKStages = 3, kVStages = 2;   // keys run further ahead than values: they are needed first
// Development aid (compile with -DFBLA_PISA_TRACE): one CTA writes clock64() stamps of its phases.
#ifdef FBLA_PISA_TRACE
__device__ long long g_pisa_trace[128];
#define PISA_STAMP(slot)                                                                  \
    do {                                                                                  \
        if (blockIdx.x == 36 && blockIdx.y == 20 && (slot) < 128) g_pisa_trace[(slot)] = clock64(); \
    } while (0)
#else
#define PISA_STAMP(slot) do { } while (0)
#endif

enum Bar { kQFull = 0, kKFull = 1, kKEmpty = 4, kVFull = 7, kVEmpty = 9, kSFull = 11, kSEmpty = 13, kPFull = 15, kPvDone = 16, kRFull = 17, kBars = 18 };

// Shared memory: [Q tile | 3 K tiles | 2 V tiles | P tile | barriers | bookkeeping]; tiles are
// D/64 swizzled blocks of [64 rows][64 elements] and need a 1024-byte aligned base, which the kernel
// checks (dynamic shared memory starts at the base of the CTA's window when there is no static part).
template <int D>
constexpr int tile_bytes() { return kBS * D * 2; }
template <int D>
size_t smem_bytes(int nt, int ns) {
    return (size_t)(1 + kKStages + kVStages) * tile_bytes<D>() + kBlockBytes + 256 + (size_t)8 * ((nt + 63) / 64) + (size_t)4 * ns;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 2)
pisa_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   const __grid_constant__ CUtensorMap tm_kc, const __grid_constant__ CUtensorMap tm_vc,
                   const __grid_constant__ CUtensorMap tm_h, const Params p, const int32_t* __restrict__ indices,
                   float* __restrict__ row_stats) {
    constexpr int kNB = D / 64;
    constexpr int kTile = tile_bytes<D>();
    extern __shared__ __align__(1024) uint8_t sm[];
    uint8_t* q_t = sm;
    uint8_t* k_ring = sm + kTile;
    uint8_t* v_ring = k_ring + kKStages * kTile;
    uint8_t* p_t = v_ring + kVStages * kTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_t + kBlockBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int nch = (p.nt + 63) / 64;
    unsigned long long* sel_mask = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(bars) + 256);
    int* sel_idx = reinterpret_cast<int*>(sel_mask + nch);

    const int qb = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NI = p.ns + nch;
    const int n_keys = NI + kNB;        // key tiles: one per iteration, then the 64-row halves of h
    const int32_t* idx = indices + ((size_t)bh * p.nt + qb) * p.ns;
    if ((ptx::smem_u32(sm) & 1023u) != 0) {          // uniform over the CTA: the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) *p.status = 799;
        return;
    }
    const ptx::Abort ab{abort_flag, p.status};

    // ---- loads (thread 0) ----
    // Issue order: K(t + 1) before V(t), so that the scores of the next iteration never wait for a load
    // that was started only when its slot fell free.  Indices are read straight from global memory.
    auto block_of = [&](int i) {
        const int c = __ldg(idx + i);
        return (c < 0 || c >= p.nt) ? 0 : c;         // a bad index: fetched, then masked out entirely
    };
    auto load_k = [&](int i) -> bool {
        const int s = i % kKStages;
        uint8_t* k_t = k_ring + s * kTile;
        if (!ptx::mbar_wait(&bars[kKEmpty + s], ((i / kKStages) & 1) ^ 1, ab, 711)) return false;
        ptx::mbar_arrive_expect_tx(&bars[kKFull + s], kTile);
        const CUtensorMap* m = i < p.ns ? &tm_k : (i < NI ? &tm_kc : &tm_h);
        const int r0 = i < p.ns ? block_of(i) * kBS : (i < NI ? (i - p.ns) * 64 : (i - NI) * 64);
        for (int cb = 0; cb < kNB; ++cb) ptx::tma_load_3d(k_t + cb * kBlockBytes, m, &bars[kKFull + s], cb * 64, r0, bh);
        return true;
    };
    auto load_v = [&](int i) -> bool {
        const int s = i % kVStages;
        uint8_t* v_t = v_ring + s * kTile;
        if (!ptx::mbar_wait(&bars[kVEmpty + s], ((i / kVStages) & 1) ^ 1, ab, 712)) return false;
        ptx::mbar_arrive_expect_tx(&bars[kVFull + s], kTile);
        const CUtensorMap* m = i < p.ns ? &tm_v : &tm_vc;
        const int r0 = i < p.ns ? block_of(i) * kBS : (i - p.ns) * 64;
        for (int cb = 0; cb < kNB; ++cb) ptx::tma_load_3d(v_t + cb * kBlockBytes, m, &bars[kVFull + s], cb * 64, r0, bh);
        return true;
    };

    if (threadIdx.x == 0) {
        PISA_STAMP(0);
        ptx::mbar_init(&bars[kQFull], 1);
        for (int s = 0; s < kKStages; ++s) {
            ptx::mbar_init(&bars[kKFull + s], 1);
            ptx::mbar_init(&bars[kKEmpty + s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&bars[kVFull + s], 1);
            ptx::mbar_init(&bars[kVEmpty + s], 1);
            ptx::mbar_init(&bars[kSFull + s], 1);
            ptx::mbar_init(&bars[kSEmpty + s], 128);
        }
        ptx::mbar_init(&bars[kPFull], 128);
        ptx::mbar_init(&bars[kPvDone], 1);
        ptx::mbar_init(&bars[kRFull], 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        // the first loads go out before the rest of the CTA has finished setting up
        ptx::mbar_arrive_expect_tx(&bars[kQFull], kTile);
        for (int cb = 0; cb < kNB; ++cb) ptx::tma_load_3d(q_t + cb * kBlockBytes, &tm_q, &bars[kQFull], cb * 64, qb * kBS, bh);
        load_k(0);
        if (n_keys > 1) load_k(1);
        if (NI > 0) load_v(0);
    }
    for (int i = threadIdx.x; i < nch; i += kThreads) sel_mask[i] = 0ull;
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, kTmemCols);
        ptx::tmem_relinquish();
    }
    __syncthreads();
    // one 64-bit word per group of 64 blocks: bit j set = block 64 c + j was selected
    for (int i = threadIdx.x; i < p.ns; i += kThreads) {
        const int c = idx[i];
        sel_idx[i] = c;
        if (c >= 0 && c < p.nt) atomicOr(&sel_mask[c >> 6], 1ull << (c & 63));      // a bad index selects nothing
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (threadIdx.x == 0) PISA_STAMP(1);

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer (continued) ----------------
            bool okay = true;
            for (int t = 1; t < n_keys && okay; ++t) {
                if (t + 1 < n_keys) okay = load_k(t + 1);
                if (okay && t < NI) okay = load_v(t);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc_s = ptx::instr_desc(64, 64, BF16, false, false);
            const uint32_t idesc_o = ptx::instr_desc(64, D, BF16, false, true);
            // descriptors of the first k-step of every operand tile; the rest are offsets from these
            const uint64_t d_q = ptx::smem_desc(ptx::smem_u32(q_t), 16, 1024, ptx::kLayoutSw128);
            const uint64_t d_p = ptx::smem_desc(ptx::smem_u32(p_t), 16, 1024, ptx::kLayoutSw128);
            const uint64_t d_k0 = ptx::smem_desc(ptx::smem_u32(k_ring), 16, 1024, ptx::kLayoutSw128);              // K-major
            const uint64_t d_kmn0 = ptx::smem_desc(ptx::smem_u32(k_ring), kBlockBytes, 1024, ptx::kLayoutSw128);    // MN-major (h)
            const uint64_t d_v0 = ptx::smem_desc(ptx::smem_u32(v_ring), kBlockBytes, 1024, ptx::kLayoutSw128);
            constexpr int kTileUnits = kTile / 16;
            auto scores = [&](int i) -> bool {
                const int s = i & 1, ks = i % kKStages;
                if (!ptx::mbar_wait(&bars[kKFull + ks], (i / kKStages) & 1, ab, 721)) return false;
                if (!ptx::mbar_wait(&bars[kSEmpty + s], ((i >> 1) & 1) ^ 1, ab, 722)) return false;
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepK>(tmem + kColS + s * 64, d_q + kb * ptx::kDescBlock,
                                                                     d_k0 + ks * kTileUnits + kb * ptx::kDescBlock, idesc_s, kb != 0);
                ptx::mma_commit(&bars[kSFull + s]);
                ptx::mma_commit(&bars[kKEmpty + ks]);
                return true;
            };
            bool okay = ptx::mbar_wait(&bars[kQFull], 0, ab, 720);
            PISA_STAMP(90);
            if (okay && NI > 0) okay = scores(0);
            for (int i = 0; i < NI && okay; ++i) {
                const int b = i & 1;
                if (i + 1 < NI && !scores(i + 1)) { okay = false; break; }
                if (!ptx::mbar_wait(&bars[kVFull + b], (i >> 1) & 1, ab, 725)) { okay = false; break; }
                if (!ptx::mbar_wait(&bars[kPFull], i & 1, ab, 723)) { okay = false; break; }
                PISA_STAMP(10 + i);
                ptx::tc_fence_after_sync();
                ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColO, d_p, d_v0 + b * kTileUnits, idesc_o, i != 0);
                ptx::mma_commit(&bars[kVEmpty + b]);
                ptx::mma_commit(&bars[kPvDone]);
            }
            for (int kb = 0; kb < kNB && okay; ++kb)
                okay = ptx::mbar_wait(&bars[kKFull + (NI + kb) % kKStages], ((NI + kb) / kKStages) & 1, ab, 724);
            if (okay) {
                // r = Q h into the columns of the score buffers (all scores have been read: the last
                // weights were waited for above)
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
                    ptx::mma_ss_k4<ptx::kDescStepK, ptx::kDescStepMN>(tmem + kColS, d_q + kb * ptx::kDescBlock,
                                                                      d_kmn0 + ((NI + kb) % kKStages) * kTileUnits, idesc_o, kb != 0);
                ptx::mma_commit(&bars[kRFull]);
                PISA_STAMP(91);
            }
        }
    } else {
        // ---------------- softmax and epilogue ----------------
        // A warp owns 16 query rows (TMEM lanes 32 q .. 32 q + 15) and reads them in the 16x256b shape:
        // thread t holds rows t / 4 and t / 4 + 8, and of every group of eight columns the two
        // columns 2 (t % 4), 2 (t % 4) + 1 (registers 4 i .. 4 i + 3 for column group i: first row,
        // then second row).  All 32 lanes carry data; row-wise maxima and sums take two shuffles.
        const int quarter = warp & 3;
        const int c2 = (lane & 3) * 2;
        const int row_a = quarter * 16 + (lane >> 2), row_b = row_a + 8;
        const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        const float sm2 = p.scale * 1.44269504f;
        const int nrows = min(kBS, p.T - qb * kBS);
        const int last_len = p.T - (p.nt - 1) * kBS;
        float m_run[2] = {-INFINITY, -INFINITY};      // running maxima of the scaled scores (log2 domain)
        float l_part[2] = {0.f, 0.f}, g_part[2] = {0.f, 0.f};   // this thread's share of the row sums
        bool okay = true;
        for (int i = 0; i < NI; ++i) {
            const int b = i & 1;
            float s[32];
            if (!ptx::mbar_wait(&bars[kSFull + b], (i >> 1) & 1, ab, 731)) { okay = false; break; }
            if (threadIdx.x == 64) PISA_STAMP(30 + i);
            ptx::tc_fence_after_sync();
            tmem_ld_16x256b_x8(t_lane + kColS + b * 64, s);
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[kSEmpty + b]);
            const bool approx = i >= p.ns;
            int nvalid, jl = -1;
            unsigned long long keep = ~0ull;
            if (!approx) {
                const int cb = sel_idx[i];
                nvalid = (cb < 0 || cb >= p.nt) ? 0 : min(kBS, p.T - cb * kBS);
            } else {
                const int c0 = (i - p.ns) * 64;
                nvalid = min(64, p.nt - c0);
                keep = ~sel_mask[i - p.ns];
                if (last_len != kBS) jl = p.nt - 1 - c0;     // position of the shorter last block, if in this group
            }
            keep &= nvalid >= 64 ? ~0ull : ((1ull << nvalid) - 1ull);
            if (keep != ~0ull) {
                const unsigned long long keep_t = keep >> c2;    // bit 8 i + (e & 1) = this thread's column of group i
#pragma unroll
                for (int x = 0; x < 32; ++x)
                    if (!((keep_t >> ((x >> 2) * 8 + (x & 1))) & 1ull)) s[x] = -INFINITY;
            }
            // row maxima: four independent chains per row, then the quad
            float mx[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float m4[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) m4[u] = fmaxf(s[8 * u + 2 * r], s[8 * u + 2 * r + 1]);
#pragma unroll
                for (int u = 0; u < 4; ++u) m4[u] = fmaxf(m4[u], fmaxf(s[8 * u + 4 + 2 * r], s[8 * u + 4 + 2 * r + 1]));
                mx[r] = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], 1));
            mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], 1));
            mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], 2));
            mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], 2));
            float alpha[2], neg_m[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float m_new = fmaxf(m_run[r], mx[r] * sm2);        // scale > 0: the order is kept
                alpha[r] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[r] - m_new);
                m_run[r] = m_new;
                l_part[r] *= alpha[r];
                g_part[r] *= alpha[r];
                neg_m[r] = (m_new == -INFINITY) ? 0.f : -m_new;          // exp2(-inf * sm2 + 0) = 0 for masked entries
            }
            if (threadIdx.x == 64) PISA_STAMP(110 + i);
            uint32_t pk[16];
            float sum[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
            if (!approx) {
#pragma unroll
                for (int x = 0; x < 32; x += 2) {
                    const int r = (x >> 1) & 1;
                    const float p0 = exp2f(fmaf(s[x], sm2, neg_m[r]));
                    const float p1 = exp2f(fmaf(s[x + 1], sm2, neg_m[r]));
                    pk[x >> 1] = pack2<BF16>(p0, p1);
                    sum[r][0] += p0;
                    sum[r][1] += p1;
                }
                l_part[0] += sum[0][0] + sum[0][1];
                l_part[1] += sum[1][0] + sum[1][1];
            } else {
                const int jl_t = jl - c2;                    // this thread holds block jl iff 8 i + (e & 1) == jl_t
                float p_last[2] = {0.f, 0.f};
#pragma unroll
                for (int x = 0; x < 32; x += 2) {
                    const int r = (x >> 1) & 1;
                    const float p0 = exp2f(fmaf(s[x], sm2, neg_m[r]));
                    const float p1 = exp2f(fmaf(s[x + 1], sm2, neg_m[r]));
                    pk[x >> 1] = pack2<BF16>(p0, p1);
                    sum[r][0] += p0;
                    sum[r][1] += p1;
                    p_last[r] = ((x >> 2) * 8 == jl_t) ? p0 : (((x >> 2) * 8 + 1 == jl_t) ? p1 : p_last[r]);
                }
                g_part[0] += (sum[0][0] + sum[0][1]) * (float)kBS - p_last[0] * (float)(kBS - last_len);
                g_part[1] += (sum[1][0] + sum[1][1]) * (float)kBS - p_last[1] * (float)(kBS - last_len);
            }
            if (threadIdx.x == 64) PISA_STAMP(50 + i);
            if (i > 0) {
                // the previous P V must be complete before P is overwritten and O is touched
                if (!ptx::mbar_wait(&bars[kPvDone], (i - 1) & 1, ab, 732)) { okay = false; break; }
                ptx::tc_fence_after_sync();
                if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                    for (int c = 0; c < D; c += 64) {
                        float o[32];
                        tmem_ld_16x256b_x8(t_lane + kColO + c, o);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int x = 0; x < 32; ++x) o[x] *= alpha[(x >> 1) & 1];
                        tmem_st_16x256b_x8(t_lane + kColO + c, o);
                    }
                    tmem_st_wait();
                }
            }
            uint8_t* pb = p_t;
#pragma unroll
            for (int x = 0; x < 16; ++x) {
                const int row = (x & 1) ? row_b : row_a;
                *reinterpret_cast<uint32_t*>(pb + row * 128 + ((((x >> 1) ^ row) & 7) << 4) + c2 * 2) = pk[x];
            }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[kPFull]);
            if (threadIdx.x == 64) PISA_STAMP(70 + i);
        }
        if (okay) okay = ptx::mbar_wait(&bars[kRFull], 0, ab, 733);
        if (threadIdx.x == 64) PISA_STAMP(92);
        if (okay) {
            ptx::tc_fence_after_sync();
            float corr[2], rden[2], l_row[2], g_row[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                l_row[r] = l_part[r] + __shfl_xor_sync(0xffffffffu, l_part[r], 1);
                l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
                g_row[r] = g_part[r] + __shfl_xor_sync(0xffffffffu, g_part[r], 1);
                g_row[r] += __shfl_xor_sync(0xffffffffu, g_row[r], 2);
                rden[r] = 1.f / (l_row[r] + g_row[r]);
                corr[r] = g_row[r] * p.scale / (float)p.T * rden[r];
            }
#pragma unroll
            for (int c = 0; c < D; c += 64) {
                float o[32], rr[32];
                tmem_ld_16x256b_x8(t_lane + kColO + c, o);
                tmem_ld_16x256b_x8(t_lane + kColS + c, rr);
                ptx::tmem_ld_wait();
                uint8_t* blk = q_t + (c >> 6) * kBlockBytes;      // the query tile is free: r = Q h is done
#pragma unroll
                for (int x = 0; x < 32; x += 2) {
                    const int r = (x >> 1) & 1;
                    const int row = r ? row_b : row_a;
                    *reinterpret_cast<uint32_t*>(blk + row * 128 + ((((x >> 2) ^ row) & 7) << 4) + c2 * 2) =
                        pack2<BF16>(fmaf(rr[x], corr[r], o[x] * rden[r]), fmaf(rr[x + 1], corr[r], o[x + 1] * rden[r]));
                }
            }
            if ((lane & 3) == 0 && row_stats != nullptr) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int row = r ? row_b : row_a;
                    if (row < nrows)
                        *reinterpret_cast<float4*>(row_stats + ((size_t)bh * p.T + qb * kBS + row) * 4) =
                            make_float4(m_run[r], l_row[r] + g_row[r], g_row[r], rden[r]);
                }
            }
            ptx::fence_proxy_async_smem();
        }
        if (threadIdx.x == 64) PISA_STAMP(93);
        ptx::tc_fence_before_sync();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (okay && threadIdx.x == 64) {
            for (int cb = 0; cb < kNB; ++cb) ptx::tma_store_3d(&tm_o, q_t + cb * kBlockBytes, cb * 64, qb * kBS, bh);
            ptx::tma_store_commit();
            ptx::tma_store_wait_read<0>();      // the tile may be released once it has been read
            PISA_STAMP(94);
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, kTmemCols);
    }
    if (threadIdx.x == 0) PISA_STAMP(2);
}

// fp32 -> 16-bit copies of the block statistics and of h, eight elements per thread
template <bool BF16>
__global__ void __launch_bounds__(256) cast16_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                     const float* __restrict__ c, int64_t na, int64_t nb, int64_t nc,
                                                     uint4* __restrict__ out) {
    const int64_t total = (na + nb + nc) / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = i * 8;
        const float* src = e < na ? a + e : (e < na + nb ? b + (e - na) : c + (e - na - nb));
        const float4 x = *reinterpret_cast<const float4*>(src);
        const float4 y = *reinterpret_cast<const float4*>(src + 4);
        out[i] = make_uint4(pack2<BF16>(x.x, x.y), pack2<BF16>(x.z, x.w), pack2<BF16>(y.x, y.y), pack2<BF16>(y.z, y.w));
    }
}

}  // namespace pisa_tc

#ifdef FBLA_PISA_TRACE
extern "C" int fbla_debug_pisa_trace(long long* out128) {
    return (int)cudaMemcpyFromSymbol(out128, pisa_tc::g_pisa_trace, sizeof(long long) * 128);
}
#endif

bool pisa_tc_supported(int dtype, int dk, int dv, int bs, int nt, int ns) {
    return (dtype == FBLA_BF16 || dtype == FBLA_F16) && dk == dv && (dk == 64 || dk == 128) && bs == 64 && nt <= 2048 &&
           ns <= nt;
}

void pisa_tc_cast16(int dtype, const float* kc, const float* vc, const float* h, int64_t n_stats, int64_t n_h, void* out,
                    cudaStream_t st) {
    const int64_t total = (2 * n_stats + n_h) / 8;
    const int grid = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
    if (dtype == FBLA_BF16)
        pisa_tc::cast16_kernel<true><<<grid, 256, 0, st>>>(kc, vc, h, n_stats, n_stats, n_h, static_cast<uint4*>(out));
    else
        pisa_tc::cast16_kernel<false><<<grid, 256, 0, st>>>(kc, vc, h, n_stats, n_stats, n_h, static_cast<uint4*>(out));
}

int64_t pisa_tc_scratch_bytes(int bh, int d, int nt) {
    return ((int64_t)2 * bh * nt * d + (int64_t)bh * d * d) * 2;
}

cudaError_t pisa_tc_fwd(int dtype, int bh, int d, int nt, int ns, int T, float scale, const void* q, const void* k,
                        const void* v, const float* kc, const float* vc, const float* h, const int32_t* indices, void* o,
                        float* row_stats, void* scratch, cudaStream_t st) {
    using namespace pisa_tc;
    const int64_t n_stats = (int64_t)bh * nt * d, n_h = (int64_t)bh * d * d;
    uint16_t* kc16 = static_cast<uint16_t*>(scratch);
    uint16_t* vc16 = kc16 + n_stats;
    uint16_t* h16 = vc16 + n_stats;
    const bool bf = dtype == FBLA_BF16;
    pisa_tc_cast16(dtype, kc, vc, h, n_stats, n_h, scratch, st);
    CUtensorMap mq, mk, mv, mo, mkc, mvc, mh;
    cudaError_t e;
    if ((e = tc_encode_map_rows(&mq, q, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mk, k, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mv, v, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mo, o, dtype, d, T, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mkc, kc16, dtype, d, nt, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mvc, vc16, dtype, d, nt, bh, 64)) != cudaSuccess) return e;
    if ((e = tc_encode_map_rows(&mh, h16, dtype, d, d, bh, 64)) != cudaSuccess) return e;
    Params p{ns, nt, T, scale, tc_status_word()};
    if (p.status == nullptr) return cudaErrorMemoryAllocation;
    const dim3 grid(nt, bh);
    auto run = [&](auto kern, size_t smem) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, mo, mkc, mvc, mh, p, indices, row_stats);
    };
    if (d == 64) {
        if (bf) run(pisa_fwd_tc_kernel<64, true>, smem_bytes<64>(nt, ns));
        else run(pisa_fwd_tc_kernel<64, false>, smem_bytes<64>(nt, ns));
    } else {
        if (bf) run(pisa_fwd_tc_kernel<128, true>, smem_bytes<128>(nt, ns));
        else run(pisa_fwd_tc_kernel<128, false>, smem_bytes<128>(nt, ns));
    }
    return e == cudaSuccess ? cudaGetLastError() : e;
}

}  // namespace fbla
