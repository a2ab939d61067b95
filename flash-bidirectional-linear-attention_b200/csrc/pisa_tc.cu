// Forward of the piecewise sparse attention stage on the 5th-generation tensor cores
// (reference: piecewise_sparse_attention_fwd_kernel, flash_bla/ops/piecewise_attn/kernel.py:189-292).
//
// One CTA per block of 64 queries of one (batch, head).  Every key block the query block selected
// (exact softmax attention) and every group of 64 unselected blocks (their means as keys, their sums
// as values: the zeroth-order term) is one iteration of the same loop:
//     S = Q K^T          tcgen05.mma, M = 64, N = 64, accumulator in TMEM
//     P = exp2(S - m)    one thread per query row reads its row of S from TMEM (no shuffles)
//     O (+)= P V         tcgen05.mma, P staged in shared memory, accumulator in TMEM
// followed by r = Q h (the first-order term) and out = (O + r g scale / T) / (l + g).
//
//   warp 0      TMA producer: Q once, then a two-stage ring of (K, V) tiles, then h
//   warp 1      MMA issuer (one thread) and owner of the TMEM allocation
//   warps 2-5   softmax and epilogue; with M = 64 the accumulator row r lives in TMEM lane
//               (r % 16) + 32 * (r / 16), so lanes 0-15 of each warp carry one row each
//
// The score MMA of iteration i + 1 is issued before the weights of iteration i are waited for, so
// the softmax of one block overlaps the tensor-core work of its neighbours; S is double-buffered.
// O is rescaled in TMEM (tcgen05.ld / tcgen05.st) only when a row's running maximum moved.
// The block statistics and h arrive as 16-bit copies so that TMA can fetch them like the keys.
// Every wait is bounded and reports through the library's status word.
#include "pisa_tc.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tc_kernels.cuh"
#include "tc_ptx.cuh"

namespace fbla {
namespace pisa_tc {

constexpr int kThreads = 192;
constexpr int kBS = 64;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColO = 0;        // O: D columns
constexpr uint32_t kColS = 128;      // S: two buffers of 64 columns; r = Q h reuses them at the end
constexpr int kBlockBytes = 64 * 128;   // one [64 rows][64 x 16-bit] swizzled block

struct Params {
    int ns, nt, T;
    float scale;
    int* status;
};

enum Bar { kQFull = 0, kKvFull = 1, kKvEmpty = 3, kSFull = 5, kSEmpty = 7, kPFull = 9, kPvDone = 10, kRFull = 11, kBars = 12 };

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if constexpr (BF16) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&t);
    } else {
        const __half2 t = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&t);
    }
}

// Shared memory: [Q tile | 2 x (K tile, V tile) | P tile | barriers | bookkeeping]; tiles are
// D/64 swizzled blocks of [64 rows][64 elements].
template <int D>
constexpr int tile_bytes() { return kBS * D * 2; }
template <int D>
size_t smem_bytes(int nt, int ns) {
    return 1024 + (size_t)5 * tile_bytes<D>() + kBlockBytes + 128 + (size_t)8 * ((nt + 63) / 64) + (size_t)4 * ns +
           (size_t)((nt + 15) & ~15);
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
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_t = sm;
    uint8_t* kv_t = sm + kTile;
    uint8_t* p_t = sm + 5 * kTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_t + kBlockBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int nch = (p.nt + 63) / 64;
    unsigned long long* sel_mask = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(bars) + 128);
    int* sel_idx = reinterpret_cast<int*>(sel_mask + nch);
    unsigned char* sel = reinterpret_cast<unsigned char*>(sel_idx + p.ns);

    const int qb = blockIdx.x, bh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NI = p.ns + nch;
    const int32_t* idx = indices + ((size_t)bh * p.nt + qb) * p.ns;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars[kQFull], 1);
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&bars[kKvFull + s], 1);
            ptx::mbar_init(&bars[kKvEmpty + s], 1);
            ptx::mbar_init(&bars[kSFull + s], 1);
            ptx::mbar_init(&bars[kSEmpty + s], 128);
        }
        ptx::mbar_init(&bars[kPFull], 128);
        ptx::mbar_init(&bars[kPvDone], 1);
        ptx::mbar_init(&bars[kRFull], 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tm_q);
        ptx::prefetch_tensormap(&tm_k);
        ptx::prefetch_tensormap(&tm_v);
    }
    for (int i = threadIdx.x; i < p.nt; i += kThreads) sel[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < p.ns; i += kThreads) {
        const int c = idx[i];
        sel_idx[i] = c;
        if (c >= 0 && c < p.nt) sel[c] = 1;          // a bad index selects nothing
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, kTmemCols);
        ptx::tmem_relinquish();
    }
    __syncthreads();
    // one 64-bit word per group of 64 blocks: bit j set = block 64 c + j was selected
    for (int c = warp; c < nch; c += kThreads / 32) {
        const int a = c * 64 + lane, b = a + 32;
        const unsigned lo = __ballot_sync(0xffffffffu, a < p.nt && sel[a] != 0);
        const unsigned hi = __ballot_sync(0xffffffffu, b < p.nt && sel[b] != 0);
        if (lane == 0) sel_mask[c] = ((unsigned long long)hi << 32) | lo;
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const ptx::Abort ab{abort_flag, p.status};

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer ----------------
            ptx::mbar_arrive_expect_tx(&bars[kQFull], kTile);
            for (int cb = 0; cb < kNB; ++cb) ptx::tma_load_3d(q_t + cb * kBlockBytes, &tm_q, &bars[kQFull], cb * 64, qb * kBS, bh);
            for (int i = 0; i <= NI; ++i) {
                const int s = i & 1;
                uint8_t* k_t = kv_t + s * 2 * kTile;
                if (!ptx::mbar_wait(&bars[kKvEmpty + s], ((i >> 1) & 1) ^ 1, ab, 711)) break;
                if (i < NI) {
                    ptx::mbar_arrive_expect_tx(&bars[kKvFull + s], 2 * kTile);
                    if (i < p.ns) {
                        int c = sel_idx[i];
                        if (c < 0 || c >= p.nt) c = 0;       // fetched, then masked out entirely
                        for (int cb = 0; cb < kNB; ++cb) {
                            ptx::tma_load_3d(k_t + cb * kBlockBytes, &tm_k, &bars[kKvFull + s], cb * 64, c * kBS, bh);
                            ptx::tma_load_3d(k_t + kTile + cb * kBlockBytes, &tm_v, &bars[kKvFull + s], cb * 64, c * kBS, bh);
                        }
                    } else {
                        const int r0 = (i - p.ns) * 64;
                        for (int cb = 0; cb < kNB; ++cb) {
                            ptx::tma_load_3d(k_t + cb * kBlockBytes, &tm_kc, &bars[kKvFull + s], cb * 64, r0, bh);
                            ptx::tma_load_3d(k_t + kTile + cb * kBlockBytes, &tm_vc, &bars[kKvFull + s], cb * 64, r0, bh);
                        }
                    }
                } else {
                    // h ([D][D]): rows 0-63 into the key tile, rows 64-127 into the value tile
                    ptx::mbar_arrive_expect_tx(&bars[kKvFull + s], kNB * kNB * kBlockBytes);
                    for (int hb = 0; hb < kNB; ++hb)
                        for (int cb = 0; cb < kNB; ++cb)
                            ptx::tma_load_3d(k_t + hb * kTile + cb * kBlockBytes, &tm_h, &bars[kKvFull + s], cb * 64, hb * 64, bh);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc_s = ptx::instr_desc(64, 64, BF16, false, false);
            const uint32_t idesc_o = ptx::instr_desc(64, D, BF16, false, true);
            const uint32_t q_base = ptx::smem_u32(q_t), p_base = ptx::smem_u32(p_t);
            auto scores = [&](int i) -> bool {
                const int s = i & 1;
                if (!ptx::mbar_wait(&bars[kKvFull + s], (i >> 1) & 1, ab, 721)) return false;
                if (!ptx::mbar_wait(&bars[kSEmpty + s], ((i >> 1) & 1) ^ 1, ab, 722)) return false;
                ptx::tc_fence_after_sync();
                const uint32_t k_base = ptx::smem_u32(kv_t + s * 2 * kTile);
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t da = ptx::smem_desc(q_base + kb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                        const uint64_t db = ptx::smem_desc(k_base + kb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                        ptx::mma_ss(tmem + kColS + s * 64, da, db, idesc_s, !(kb == 0 && kk == 0));
                    }
                ptx::mma_commit(&bars[kSFull + s]);
                return true;
            };
            bool okay = ptx::mbar_wait(&bars[kQFull], 0, ab, 720);
            if (okay && NI > 0) okay = scores(0);
            for (int i = 0; i < NI && okay; ++i) {
                if (i + 1 < NI && !scores(i + 1)) { okay = false; break; }
                if (!ptx::mbar_wait(&bars[kPFull], i & 1, ab, 723)) { okay = false; break; }
                ptx::tc_fence_after_sync();
                const uint32_t v_base = ptx::smem_u32(kv_t + (i & 1) * 2 * kTile + kTile);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t da = ptx::smem_desc(p_base + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    const uint64_t db = ptx::smem_desc(v_base + kk * 2048, kBlockBytes, 1024, ptx::kLayoutSw128);
                    ptx::mma_ss(tmem + kColO, da, db, idesc_o, !(i == 0 && kk == 0));
                }
                ptx::mma_commit(&bars[kKvEmpty + (i & 1)]);
                ptx::mma_commit(&bars[kPvDone]);
            }
            if (okay && ptx::mbar_wait(&bars[kKvFull + (NI & 1)], (NI >> 1) & 1, ab, 724)) {
                // r = Q h into the columns of the score buffers (all scores have been read: the last
                // weights were waited for above)
                ptx::tc_fence_after_sync();
                const uint32_t h_base = ptx::smem_u32(kv_t + (NI & 1) * 2 * kTile);
#pragma unroll
                for (int kb = 0; kb < kNB; ++kb)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t da = ptx::smem_desc(q_base + kb * kBlockBytes + kk * 32, 16, 1024, ptx::kLayoutSw128);
                        const uint64_t db = ptx::smem_desc(h_base + kb * kTile + kk * 2048, kBlockBytes, 1024, ptx::kLayoutSw128);
                        ptx::mma_ss(tmem + kColS, da, db, idesc_o, !(kb == 0 && kk == 0));
                    }
                ptx::mma_commit(&bars[kRFull]);
            }
        }
    } else {
        // ---------------- softmax and epilogue: one query row per thread (lanes 0-15) ----------------
        const int quarter = warp & 3;
        const bool active = lane < 16;
        const int row = quarter * 16 + (lane & 15);
        const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        const float sm2 = p.scale * 1.44269504f;
        const int nrows = min(kBS, p.T - qb * kBS);
        const int last_len = p.T - (p.nt - 1) * kBS;
        float m_run = -INFINITY, l = 0.f, g = 0.f;
        bool okay = true;
        for (int i = 0; i < NI; ++i) {
            const int b = i & 1;
            float s[64];
            if (!ptx::mbar_wait(&bars[kSFull + b], (i >> 1) & 1, ab, 731)) { okay = false; break; }
            ptx::tc_fence_after_sync();
            ptx::tmem_ld32(t_lane + kColS + b * 64, *reinterpret_cast<float(*)[32]>(&s[0]));
            ptx::tmem_ld32(t_lane + kColS + b * 64 + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[kSEmpty + b]);
            const bool approx = i >= p.ns;
            int nvalid, jl = -1;
            unsigned long long keep;
            if (!approx) {
                const int cb = sel_idx[i];
                nvalid = (cb < 0 || cb >= p.nt) ? 0 : min(kBS, p.T - cb * kBS);
                keep = ~0ull;
            } else {
                const int c0 = (i - p.ns) * 64;
                nvalid = min(64, p.nt - c0);
                keep = ~sel_mask[i - p.ns];
                jl = p.nt - 1 - c0;                 // position of the (possibly shorter) last block, if in this group
            }
            keep &= nvalid >= 64 ? ~0ull : ((1ull << nvalid) - 1ull);
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                s[j] = ((keep >> j) & 1ull) ? s[j] * sm2 : -INFINITY;
                mx = fmaxf(mx, s[j]);
            }
            const float m_new = fmaxf(m_run, mx);
            const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
            m_run = m_new;
            l *= alpha;
            g *= alpha;
            uint32_t pk[32];
            float sum = 0.f, p_last = 0.f;
#pragma unroll
            for (int j = 0; j < 64; j += 2) {
                const float p0 = (m_run == -INFINITY) ? 0.f : exp2f(s[j] - m_run);
                const float p1 = (m_run == -INFINITY) ? 0.f : exp2f(s[j + 1] - m_run);
                sum += p0 + p1;
                p_last = (j == jl) ? p0 : ((j + 1 == jl) ? p1 : p_last);
                pk[j >> 1] = pack2<BF16>(p0, p1);
            }
            if (approx) g += sum * (float)kBS - p_last * (float)(kBS - last_len);
            else l += sum;
            if (i > 0) {
                // the previous P V must be complete before P is overwritten and O is touched
                if (!ptx::mbar_wait(&bars[kPvDone], (i - 1) & 1, ab, 732)) { okay = false; break; }
                ptx::tc_fence_after_sync();
                if (__any_sync(0xffffffffu, active && alpha != 1.f)) {
#pragma unroll
                    for (int c = 0; c < D; c += 32) {
                        float o[32];
                        ptx::tmem_ld32(t_lane + kColO + c, o);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] *= alpha;
                        tmem_st32(t_lane + kColO + c, o);
                    }
                    tmem_st_wait();
                }
            }
            if (active) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4*>(p_t + row * 128 + (((c ^ row) & 7) << 4)) =
                        make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[kPFull]);
        }
        if (okay) okay = ptx::mbar_wait(&bars[kRFull], 0, ab, 733);
        if (okay) {
            ptx::tc_fence_after_sync();
            const float corr = g * p.scale / (float)p.T;
            const float rden = 1.f / (l + g);
#pragma unroll
            for (int c = 0; c < D; c += 32) {
                float o[32], r[32];
                ptx::tmem_ld32(t_lane + kColO + c, o);
                ptx::tmem_ld32(t_lane + kColS + c, r);
                ptx::tmem_ld_wait();
                if (active) {
                    uint8_t* blk = q_t + (c >> 6) * kBlockBytes + row * 128;      // the query tile is free: r = Q h is done
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        uint32_t w[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int x = e * 8 + u * 2;
                            w[u] = pack2<BF16>((o[x] + r[x] * corr) * rden, (o[x + 1] + r[x + 1] * corr) * rden);
                        }
                        const int chunk = ((c & 63) >> 3) + e;
                        *reinterpret_cast<uint4*>(blk + (((chunk ^ row) & 7) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            if (active && row < nrows && row_stats != nullptr)
                *reinterpret_cast<float4*>(row_stats + ((size_t)bh * p.T + qb * kBS + row) * 4) = make_float4(m_run, l + g, g, rden);
            ptx::fence_proxy_async_smem();
        }
        ptx::tc_fence_before_sync();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (okay && threadIdx.x == 64) {
            for (int cb = 0; cb < kNB; ++cb) ptx::tma_store_3d(&tm_o, q_t + cb * kBlockBytes, cb * 64, qb * kBS, bh);
            ptx::tma_store_commit();
            ptx::tma_store_wait_all<0>();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, kTmemCols);
    }
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

bool pisa_tc_supported(int dtype, int dk, int dv, int bs, int nt, int ns) {
    return (dtype == FBLA_BF16 || dtype == FBLA_F16) && dk == dv && (dk == 64 || dk == 128) && bs == 64 && nt <= 2048 &&
           ns <= nt;
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
    {
        const int64_t total = (2 * n_stats + n_h) / 8;
        const int grid = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
        if (bf) cast16_kernel<true><<<grid, 256, 0, st>>>(kc, vc, h, n_stats, n_stats, n_h, static_cast<uint4*>(scratch));
        else cast16_kernel<false><<<grid, 256, 0, st>>>(kc, vc, h, n_stats, n_stats, n_h, static_cast<uint4*>(scratch));
    }
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
