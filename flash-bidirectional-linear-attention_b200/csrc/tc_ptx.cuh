// sm_100a building blocks of the tensor-core kernels, as inline PTX:
//   mbarrier (with bounded waits), TMA tiled loads/stores (cp.async.bulk.tensor),
//   tcgen05 MMA / commit / TMEM alloc + load, shared-memory matrix descriptors.
// Nothing here uses cluster multicast; every kernel runs with cluster size 1.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fbla {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier -----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Every wait in the kernels is bounded: after kWaitCycles without progress, or as soon as
// another thread of the CTA has given up, the wait returns false, the caller leaves its
// loop, and the kernel reports the failure through the status word instead of hanging.
constexpr long long kWaitCycles = 10000000000LL;  // about five seconds

struct Abort {
    volatile int* cta_flag;   // shared memory: some thread of this CTA gave up
    int* status;              // host-visible status word of the library
};

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const Abort& ab, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        ++spins;
        // only waits of many microseconds back off (a sleeping waiter wakes up late)
        if (spins > 4096) __nanosleep(200);
        if ((spins & 63) == 0) {
            if (*ab.cta_flag != 0) return false;
            if (clock64() - t0 > kWaitCycles) {
                *ab.cta_flag = where;
                *ab.status = where;
                __threadfence_system();
                return false;
            }
        }
    }
}

// ---- proxies and tcgen05 fences -----------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA ----------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)m) : "memory");
}
// 3-D tiled load global -> shared, completion signalled on `bar` (transaction bytes).
// c0 is the innermost (feature) coordinate and must keep c0 * elemsize a multiple of 16.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Pulls one box into L2 without a destination in shared memory: lets a producer run the DRAM
// reads many tiles ahead of the few tiles its shared-memory stages can hold.
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* m, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"((uint64_t)m), "r"(c0),
                 "r"(c1), "r"(c2)
                 : "memory");
}
// 3-D tiled store shared -> global (bulk async group of the issuing thread).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     (uint64_t)m),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tensor memory ------------------------------------------------------------------------
// Allocation is warp-wide (.sync.aligned); the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 32 lanes x 32-bit, N consecutive columns: thread i of the warp receives columns
// [col, col+N) of TMEM lane (lane_base + i).  taddr = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
        "[%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- tcgen05.mma --------------------------------------------------------------------------
// Shared-memory matrix descriptor for the 128-byte-swizzled canonical layouts (rows of 128
// bytes, 8-row groups of 1024 bytes whose 16-byte chunks are XOR-ed with the row index):
//   bits  0-13 start address >> 4        bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4   bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 layout type (2 = 128-byte swizzle, 0 = none)
// K-major operand  : rows are M/N indices, the 128 bytes run along K; SBO = 1024 is the
//                    step to the next 8 rows; LBO is unused (1).
// MN-major operand : rows are K indices, the 128 bytes run along M/N (64 elements);
//                    SBO = 1024 is the step to the next 8 K-rows, LBO the step to the
//                    next 64 M/N elements.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(layout_type & 7) << 61;
    return d;
}
constexpr uint32_t kLayoutSw128 = 2;
constexpr uint32_t kLayoutNone = 0;

// Instruction descriptor of kind::f16 (fp32 accumulate):
//   bits 4-5 D format (1 = f32), 7-9 A format, 10-12 B format (0 = f16, 1 = bf16),
//   bit 15 A is MN-major, bit 16 B is MN-major, bits 17-22 N >> 3, bits 24-28 M >> 4.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, bool bf16, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
           ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// (Both operands must have the same 16-bit format: a descriptor that mixes f16 and bf16 raised an
// illegal-instruction fault on B200.)

// D[tmem] (+)= A[smem] * B[smem]; issued by a single thread.
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// Four MMAs over the consecutive k-steps of one 64-element block of the contraction dimension, as one
// statement: the descriptors advance by A_STEP / B_STEP (units of 16 bytes: 2 for a K-major operand,
// 128 for an MN-major one) from step to step.  The first accumulates iff `accumulate`, the others always.
// With small tiles (M = 64, N = 64 or 128) an MMA runs for 32-64 cycles, so the issuing thread must not
// spend dozens of instructions assembling descriptors for each.
template <int A_STEP, int B_STEP>
__device__ __forceinline__ void mma_ss_k4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, t;\n\t"
        ".reg .b64 a, b;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 t, %0, %0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "add.s64 a, %1, %5;\n\t"
        "add.s64 b, %2, %6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
        "add.s64 a, a, %5;\n\t"
        "add.s64 b, b, %6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
        "add.s64 a, a, %5;\n\t"
        "add.s64 b, b, %6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate), "n"(A_STEP), "n"(B_STEP)
        : "memory");
}
constexpr int kDescStepK = 2;        // K-major operand: 16 elements of 2 bytes
constexpr int kDescStepMN = 128;     // MN-major operand: 16 rows of 128 bytes
constexpr int kDescBlock = 512;      // next [64 rows][64 elements] block of a tile (8192 bytes)

// Arrives once on `bar` when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32-byte global store (one full sector per thread).
// Programmatic dependent launch: `griddep_launch` lets the next kernel of the stream (if it was
// launched with the programmatic-serialization attribute) start its prologue as soon as SM
// resources free up; `griddep_wait` blocks until the previous kernel of the stream has completed
// and its writes are visible.  Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void st_global_32B(void* ptr, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(a.x), "r"(a.y), "r"(a.z),
                 "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

// Byte offset of element (row, col) of a [rows][64] 16-bit tile in the 128-byte-swizzled
// layout (tile base 1024-byte aligned): what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B and
// what the descriptors above read.
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
    return (uint32_t)(row * 128 + ((((col >> 3) ^ row) & 7) << 4) + ((col & 7) << 1));
}

}  // namespace ptx
}  // namespace fbla
