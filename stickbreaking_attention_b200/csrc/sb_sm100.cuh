// Thin wrappers over the sm_100a instructions the tensor-core kernels use: mbarrier, TMA tile loads, tensor
// memory (TMEM) allocation / load / store and tcgen05.mma with its shared-memory and instruction descriptors.
// Every wait is bounded: after kWaitLimitNs the waiter gives up, and the kernel reports SBATTN_ST_TIMEOUT.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb {
namespace sm100 {

constexpr unsigned kProducerSleepNs = 100;  // between the polls of a producer's wait (30 ... 200 measured alike)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}
// Waits for the phase with the given parity to complete.  Returns false after kWaitLimitNs or as soon as
// *abort_flag (shared memory) is set by another waiter that gave up; the caller must then stop issuing work.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// The same for a producer that has time: it sleeps between polls instead of competing with the warps of its scheduler for
// issue slots (a tile load takes ~1 500 cycles anyway).  Worth 1 % in the dk/dv kernel, nothing in the others; the same
// in the row threads' long waits changed nothing.
__device__ __forceinline__ bool mbar_wait_idle(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    uint32_t spins = 0;
    while (true) {
        __nanosleep(kProducerSleepNs);
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// make generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma operand reads)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Rows [first, last) of a swizzled operand tile are set to zero by one warp.  The tile is a series of boxes of 128-byte
// rows, box_bytes apart; the 128-byte swizzle permutes 16-byte chunks inside a row only, so a row is 128 contiguous bytes
// of its box.  For the tiles at the ragged end of a sequence: the rows behind the end belong to the next sequence or to
// nobody, and although they only ever meet zero weights in a contraction, 0 * NaN is NaN.  zero_rows_done() makes the
// writes of all lanes visible to the tensor core.
__device__ __forceinline__ void zero_rows(uint8_t* tile, int boxes, int box_bytes, int first, int last, int lane) {
    for (int bx = 0; bx < boxes; ++bx)
        for (int i = first * 8 + lane; i < last * 8; i += 32) *(uint4*)(tile + bx * box_bytes + i * 16) = make_uint4(0u, 0u, 0u, 0u);
}
// The same for the rows from `first` to the next multiple of 16 (none if `first` is one): four stores per lane and box
__device__ __forceinline__ void zero_rows_to_16(uint8_t* tile, int boxes, int box_bytes, int first, int lane) {
    uint8_t* slice = tile + (first >> 4) * 2048;  // 16 rows of 128 bytes
    for (int bx = 0; bx < boxes; ++bx)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int chunk = lane + 32 * t;  // 16-byte chunk of the slice: row chunk / 8
            if ((chunk >> 3) >= (first & 15)) *(uint4*)(slice + bx * box_bytes + chunk * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
}
__device__ __forceinline__ void zero_rows_done() {
    fence_async_smem();
    __syncwarp();
}
// out of line, for kernels whose register allocation is better left alone
static __device__ __noinline__ void zero_rows_ool(uint8_t* tile, int boxes, int box_bytes, int first, int last, int lane) {
    zero_rows(tile, boxes, box_bytes, first, last, lane);
    zero_rows_done();
}

__device__ __forceinline__ void prefetch_l2(const void* gptr) { asm volatile("prefetch.global.L2 [%0];" ::"l"(gptr)); }

// 4-byte asynchronous copy global -> shared (a prefetched per-row scalar never occupies a register while in flight)
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)m) : "memory");
}
// 4-d tile load: coordinates (c0 = innermost element index, c1 = row, c2 = head, c3 = batch)
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// ---------------------------------------------------------------------------------------------- TMEM
// one full warp; writes the base address (lane 0, first column) to *dst (shared memory)
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Waits for this thread's tensor-memory loads.  The loaded registers are operands of the wait: an instruction that uses
// them depends on nothing else that orders it behind the wait, and the compiler is otherwise free to schedule it before
// (seen as garbage in a few lanes of an epilogue, now and then, when the load and its use were inlined into a longer loop).
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&a)[32], uint32_t (&b)[32]) {
    tmem_wait_ld(a);
    tmem_wait_ld(b);  // nothing left to wait for: orders the uses of b as well
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 columns of 32-bit cells: thread i of the warp receives lane (base lane + i), columns c..c+31
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---------------------------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for 128-byte-swizzled tiles made of rows of 128 bytes (what a TMA box
// with an inner extent of 64 two-byte elements and SWIZZLE_128B writes).  Byte offsets are multiples of 16.
//   K-major operand  (contraction index contiguous): rows = M/N index; `sbo` = bytes between groups of 8 rows.
//   MN-major operand (M/N index contiguous): rows = contraction index; `sbo` = bytes between groups of 8 rows,
//   `lbo` = bytes between consecutive blocks of 64 M/N indices.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of sm_100
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16 with fp32 accumulation.
//   ab_format: 0 = f16, 1 = bf16;  a_mn / b_mn: 1 when that operand is MN-major
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int ab_format, int a_mn, int b_mn) {
    return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)a_mn << 15) |
           ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// The issuing thread must stay cheap: a tcgen05.mma of 128 x 128 x 16 occupies the tensor pipe for about 64 cycles, and
// every instruction the single issuing thread spends between two of them (rebuilding a descriptor costs ~20) shows up
// as idle tensor time.  So descriptors are built once, kept as two 32-bit halves, and an operand tile further along
// is addressed by adding a constant (byte offset / 16) to the low half -- the address field cannot carry out of its
// 14 bits because shared memory ends below 256 KB.
// The warp that issues the MMAs runs its loops with all 32 lanes (waits, counters and descriptor arithmetic stay
// warp-uniform and cheap for the scheduler it shares with the row threads); only the tcgen05.mma / tcgen05.commit
// instructions themselves are predicated on one elected lane (`leader`).  Measured on B200: a single-lane issue loop
// drops from 65 to 80-100 cycles per MMA when the other warps of the scheduler are busy, the whole-warp form does not.
struct SmemDesc {
    uint32_t lo, hi;
};
__device__ __forceinline__ SmemDesc make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    SmemDesc d;
    d.lo = ((saddr & 0x3FFFFu) >> 4) | (((lbo >> 4) & 0x3FFFu) << 16);
    d.hi = ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);  // version 1, SWIZZLE_128B
    return d;
}

// D[tmem] (+)= A[smem] * B[smem] ; one thread issues.  a_off / b_off: byte offsets of the operand tiles.
template <bool kAccumulate>
__device__ __forceinline__ void mma_ss(bool leader, uint32_t d_tmem, SmemDesc a, uint32_t a_off, SmemDesc b, uint32_t b_off,
                                       uint32_t idesc) {
    if (leader) asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a.lo + (a_off >> 4)), "r"(a.hi), "r"(b.lo + (b_off >> 4)), "r"(b.hi), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
template <bool kAccumulate>
__device__ __forceinline__ void mma_ts(bool leader, uint32_t d_tmem, uint32_t a_tmem, SmemDesc b, uint32_t b_off, uint32_t idesc) {
    if (leader) asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b.lo + (b_off >> 4)), "r"(b.hi), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
// accumulate chosen at run time (first tile of a work item overwrites)
__device__ __forceinline__ void mma_ss_dyn(bool leader, uint32_t d_tmem, SmemDesc a, uint32_t a_off, SmemDesc b, uint32_t b_off,
                                           uint32_t idesc, bool accumulate) {
    if (accumulate) mma_ss<true>(leader, d_tmem, a, a_off, b, b_off, idesc);
    else mma_ss<false>(leader, d_tmem, a, a_off, b, b_off, idesc);
}
__device__ __forceinline__ void mma_ts_dyn(bool leader, uint32_t d_tmem, uint32_t a_tmem, SmemDesc b, uint32_t b_off, uint32_t idesc,
                                           bool accumulate) {
    if (accumulate) mma_ts<true>(leader, d_tmem, a_tmem, b, b_off, idesc);
    else mma_ts<false>(leader, d_tmem, a_tmem, b, b_off, idesc);
}
// the mbarrier receives one arrival when every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(bool leader, uint64_t* bar) {
    if (leader) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

}  // namespace sm100

// Host side: encode a 4-d tiled tensor map over a [B,H,T,D] tensor of 2-byte elements (box = 64 x rows x 1 x 1,
// 128-byte swizzle).  Returns 0 on success.
int encode_tile_map(CUtensorMap* map, const void* ptr, int elem_kind /*0 bf16, 2 f16*/, int64_t D, int64_t T, int64_t H,
                    int64_t B, int64_t stride_t, int64_t stride_h, int64_t stride_b, int box_rows);

}  // namespace sb
