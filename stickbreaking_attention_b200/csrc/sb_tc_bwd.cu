// Tensor-core backward (sm_100a) for bf16 / f16 inputs with head_dim 32, 64 or 128 (32 runs on the
// 64-column kernels: TMA pads the tiles with zeros and the second half of the columns is not stored): two kernels, no atomics and no
// locks on dq, dk, dv (the reference accumulates dk/dv tiles in global memory under a spin lock,
// stickbreaking_attention/sb_varlen/sb_varlen_bwd.py:11-53,454-465).
//
//   dq kernel     one work item = (head, sequence, 128-row query tile).  Walks the keys LEFT TO RIGHT in steps of 128,
//                 the direction of the reference's _backward_one_row (sb_varlen_bwd.py:401-473), because
//                 ds_ik = g_ik - beta_ik * (sum of g over keys <= k) needs a prefix over the keys.  The weights of a
//                 32-key quarter need the product W of (1 - beta) over everything to its right: the forward saved that
//                 value for every 32-key boundary (carry_w).  The kernel leaves the prefix of g through the right
//                 edge of every 32-key quarter in carry_c for the second kernel.
//   dk/dv kernel  one work item = (head, sequence, 128-key tile), kept stationary; walks the 128-row query tiles
//                 below it.  Every (query tile, 32-key quarter) pair is entered directly with carry_w and carry_c, the
//                 weights and ds are recomputed, written to shared memory as 16-bit operands, and
//                 dv += p^T do, dk += ds^T q accumulate in tensor memory for the whole walk; stored once.
//
// Both kernels: one persistent block of 608 threads per SM (warps 0-15: one thread per query row and 32-key quarter of
// a step; warps 16 and 18: TMA producers; warp 17 issues tcgen05.mma), all 512 tensor-memory columns, work drawn from a
// global counter.
#include "sb_tc_common.cuh"


namespace sb {

using namespace sm100;

namespace {

constexpr int kBM = 128;  // query rows per tile
constexpr int kBK = 64;   // keys per half of a step: the unit of masking and a 128-byte row of the p / ds buffers
constexpr int kQBox = 128 * 128;  // bytes of one TMA box of a 128-row tile (64 elements wide)
constexpr int kKBox = 64 * 128;   // bytes of one TMA box of a 64-row tile

// Element-wise core shared by both kernels, four adjacent scores at a time: om = 1 - beta = 1 / (1 + 2^(s * scale));
// masked keys get om = 1 (no stick broken, weight 0).  The operations without a dependency along the row are packed
// fp32x2 instructions, and the four reciprocals cost one MUFU operation: with d_i = 1 + e_i,
// 1 / d_i = (product of the other three) / (d_0 d_1 d_2 d_3).  The exponent is clamped at 30 so that the product of four
// stays finite (om = 2^-30 instead of something smaller: no visible difference).
template <bool kMasked, bool kGrouped = true>
__device__ __forceinline__ void stick4(float s0, float s1, float s2, float s3, float scale, int col, int lim, float2& om01,
                                       float2& om23) {
    float2 x01 = __fmul2_rn(make_float2(s0, s1), make_float2(scale, scale));
    float2 x23 = __fmul2_rn(make_float2(s2, s3), make_float2(scale, scale));
    if (kGrouped) {
        x01.x = fminf(x01.x, 30.f);
        x01.y = fminf(x01.y, 30.f);
        x23.x = fminf(x23.x, 30.f);
        x23.y = fminf(x23.y, 30.f);
    }
    if (kMasked) {
        if (col >= lim) x01.x = -INFINITY;
        if (col + 1 >= lim) x01.y = -INFINITY;
        if (col + 2 >= lim) x23.x = -INFINITY;
        if (col + 3 >= lim) x23.y = -INFINITY;
    }
    const float2 d01 = __fadd2_rn(make_float2(ex2_approx(x01.x), ex2_approx(x01.y)), make_float2(1.f, 1.f));
    const float2 d23 = __fadd2_rn(make_float2(ex2_approx(x23.x), ex2_approx(x23.y)), make_float2(1.f, 1.f));
    if (!kGrouped) {
        om01 = make_float2(rcp_approx(d01.x), rcp_approx(d01.y));
        om23 = make_float2(rcp_approx(d23.x), rcp_approx(d23.y));
        return;
    }
    const float2 m = __fmul2_rn(d01, d23);  // (d0 d2, d1 d3)
    const float r = rcp_approx(m.x * m.y);
    const float2 rm = make_float2(r * m.y, r * m.x);  // (1 / (d0 d2), 1 / (d1 d3))
    om01 = __fmul2_rn(rm, d23);
    om23 = __fmul2_rn(rm, d01);
}

// ================================================================================================ dq kernel
// One block per SM (608 threads: 19 warps put five on one scheduler, which caps a thread at 96 registers), one work item = (head, sequence, 128-row query tile) at a
// time, walked LEFT TO RIGHT in steps of 128 keys, so that every contraction runs at the widest shape: S and dP
// [128 q x 128 keys], dQ += dS K with K = 128 (an MMA instruction costs the same for N = 64 and N = 128; 64-key steps need
// 40 instructions per 128 x 128 scores, 128-key steps 24).
// Sixteen row warps: a thread owns one query row and a quarter (32 keys) of the step, warps 0-3 the rightmost quarter ...
// warps 12-15 the leftmost, so that every scheduler has four row warps to choose from (with eight row warps of 64 keys
// per thread the same arithmetic ran 20 % slower, and all of them waited at the same time).
//   * carry_w exists at every 32-key boundary: every quarter is entered independently with the forward's carry.
//   * The prefix of g that ds needs is local to a quarter up to a constant: a thread computes
//     a = g - beta * (prefix inside its quarter) and ds = a - beta * (prefix at the quarter's left edge).  That prefix
//     travels along the row as a chain through shared memory: a thread takes it from the quarter to its left (the leftmost
//     quarter from the rightmost one of the previous step), adds its total and passes it on.  Nobody waits for a quarter
//     to its right, so the quarters settle into a stagger and the waits of one overlap with the arithmetic of another.
//     The prefix through a quarter's right edge is also what the dk/dv kernel enters that quarter with (carry_c).
// Tensor memory: S in two buffers (S of the next step is computed while this one is worked on; a thread's dS overwrites
// the first half of its own 32 score columns as 16-bit operands), dP in one (released as soon as every thread has copied its values to
// registers), dQ.  Warp 16 loads Q, dO (once per item) and the K tiles (three-stage ring: a K tile is needed for S early
// and for dQ late), warp 18 the V tiles, warp 17 issues every tcgen05.mma.
constexpr int kDqThreads = 608;
constexpr int kDqKStages = 3, kDqVStages = 2;
enum DqBar { A_QDO_FULL, A_QDO_EMPTY, A_K_FULL0, A_K_FULL1, A_K_FULL2, A_K_EMPTY0, A_K_EMPTY1, A_K_EMPTY2, A_V_FULL0, A_V_FULL1,
             A_V_EMPTY0, A_V_EMPTY1, A_S_READY0, A_S_READY1, A_DP_READY, A_LOADED, A_DS_READY0, A_DS_READY1, A_DS_READY2, A_DS_READY3,
             A_DQ_READY,
             A_DQ_FREE, A_WORK_FULL0, A_WORK_FULL1, A_WORK_EMPTY0, A_WORK_EMPTY1,
             A_X_G0,  // 32 barriers for the prefixes: [quarter][step parity][warp & 3]
             kNumDqBars = A_X_G0 + 32 };

template <bool kMasked>
__device__ __forceinline__ void dq_half_pass1(uint32_t (&s)[32], uint32_t (&dp)[32], float scale, int col0, int lim,
                                              float drem, float& W) {
    // right to left: s <- beta, dp <- g = p * (dP - drem), with p = W * beta = W - W * om
#pragma unroll
    for (int q = 7; q >= 0; --q) {
        float2 om[2];
        stick4<kMasked, false>(__uint_as_float(s[4 * q]), __uint_as_float(s[4 * q + 1]), __uint_as_float(s[4 * q + 2]),
                               __uint_as_float(s[4 * q + 3]), scale, col0 + 4 * q, lim, om[0], om[1]);
#pragma unroll
        for (int h = 1; h >= 0; --h) {
            const int jj = 2 * q + h;
            const float2 beta = __ffma2_rn(om[h], make_float2(-1.f, -1.f), make_float2(1.f, 1.f));
            const float2 t = __fadd2_rn(make_float2(__uint_as_float(dp[2 * jj]), __uint_as_float(dp[2 * jj + 1])),
                                        make_float2(-drem, -drem));
            const float w1 = W * om[h].y, p1 = W - w1;
            const float w0 = w1 * om[h].x, p0 = w1 - w0;
            W = w0;
            const float2 g = __fmul2_rn(make_float2(p0, p1), t);
            dp[2 * jj] = __float_as_uint(g.x);
            dp[2 * jj + 1] = __float_as_uint(g.y);
            s[2 * jj] = __float_as_uint(beta.x);
            s[2 * jj + 1] = __float_as_uint(beta.y);
        }
    }
}
// left to right: g <- a = g - beta * (inclusive prefix of g inside the 32 columns); c carries the running prefix
__device__ __forceinline__ void dq_half_local(const uint32_t (&beta)[32], uint32_t (&g)[32], float& c) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        c += __uint_as_float(g[j]);
        g[j] = __float_as_uint(fmaf(-__uint_as_float(beta[j]), c, __uint_as_float(g[j])));
    }
}
// ds = a - beta * (prefix at the half's left edge), packed to 16 bits
template <bool kF16>
__device__ __forceinline__ void dq_half_finish(const uint32_t (&beta)[32], const uint32_t (&av)[32], float c_in, uint32_t (&packed)[16]) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float2 ds = __ffma2_rn(make_float2(__uint_as_float(beta[2 * j]), __uint_as_float(beta[2 * j + 1])),
                                     make_float2(-c_in, -c_in),
                                     make_float2(__uint_as_float(av[2 * j]), __uint_as_float(av[2 * j + 1])));
        packed[j] = pack16<kF16>(ds.x, ds.y);
    }
}

// kFused (both backward kernels): d_o is the gradient of out = o + rem * v; separate instantiations, the plain ones stay
// as they are
template <int D, bool kF16, bool kFused, bool kDefer>
__global__ void __launch_bounds__(kDqThreads, 1)
tc_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const KArgs a) {
    constexpr int kBoxes = D / 64;
    constexpr int kQBytes = kBM * D * 2;  // a 128-row tile of Q, dO, K or V
    constexpr int kStep = 128;            // keys per step
    constexpr uint32_t kColS = 0, kColDP = 256, kColDQ = 384;  // S buffer b at +128*b; dS overwrites 16 of every 32 columns of its S buffer
    constexpr uint32_t kCols = 512;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sDO = sQ + kQBytes;
    uint8_t* sK = sDO + kQBytes;              // kDqKStages tiles
    uint8_t* sV = sK + kDqKStages * kQBytes;  // kDqVStages tiles
    uint64_t* bars = (uint64_t*)(sV + kDqVStages * kQBytes);
    uint32_t* tmem_slot = (uint32_t*)(bars + kNumDqBars);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    SchedRing<Work>* ring = (SchedRing<Work>*)(tmem_slot + 2);
    float* xg = (float*)(tmem_slot + 32);  // [quarter][128 rows]: the exchange slots of the row threads
    static_assert(sizeof(SchedRing<Work>) <= 120, "ring does not fit its place");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < kNumDqBars; ++i) {
            uint32_t cnt = 1;
            if (i >= A_X_G0) cnt = 32;
            if (i == A_LOADED || i == A_DQ_FREE) cnt = 512;
            if (i >= A_DS_READY0 && i <= A_DS_READY3) cnt = kDefer ? 512 : 128;  // one per 32-key quarter of the step, or one for all
            if (i == A_WORK_EMPTY0 || i == A_WORK_EMPTY1) cnt = 514;  // MMA warp (one lane), V producer, 512 row threads
            mbar_init(&bars[i], cnt);
        }
        *abort_flag = (smem_u32(smem) & 1023u) ? 1u : 0u;  // the swizzled tiles need a 1024-byte aligned base
        fence_barrier_init();
    }
    if (warp == 17) {
        tmem_alloc(tmem_slot, kCols);
        tmem_relinquish();
    }
    if (warp == 16 && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int n_items = a.hdr->n_items;
    const int n_work = *abort_flag ? 0 : n_items * a.heads;
    // G counts 128-key steps over all items of this block: step G uses K stage G % 3, V stage G % 2 and S buffer G % 2;
    // a barrier that completes once per use is in phase (use count) & 1.

    if (warp == 16) {
        // ------------------------------------------------------------------ TMA: Q, dO per item, K ring
        if (lane == 0) {
            uint32_t G = 0, items = 0;
            bool ok = true;
            SchedProducer sched;
            int w;
            Work wk;
            const auto fetch = [&](int w_) { return fetch_work(a, n_items, w_); };
            while (ok && (w = sched.next(a.sched + 2, n_work, ring, &bars[A_WORK_FULL0], &bars[A_WORK_EMPTY0], abort_flag, fetch, wk)) >= 0) {
                ok = mbar_wait_idle(&bars[A_QDO_EMPTY], (items & 1) ^ 1, abort_flag);
                ++items;
                if (!ok) break;
                mbar_expect_tx(&bars[A_QDO_FULL], 2 * kQBytes);
#pragma unroll
                for (int bx = 0; bx < kBoxes; ++bx) {
                    tma_load_4d(sQ + bx * kQBox, &map_q, &bars[A_QDO_FULL], bx * 64, wk.start + wk.qt * kBM, wk.h, wk.b);
                    tma_load_4d(sDO + bx * kQBox, &map_do, &bars[A_QDO_FULL], bx * 64, wk.start + wk.qt * kBM, wk.h, wk.b);
                }
                for (int j = 0; j <= wk.qt; ++j, ++G) {
                    const uint32_t st = G % kDqKStages;
                    ok = mbar_wait_idle(&bars[A_K_EMPTY0 + st], ((G / kDqKStages) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&bars[A_K_FULL0 + st], kQBytes);
#pragma unroll
                    for (int bx = 0; bx < kBoxes; ++bx)
                        tma_load_4d(sK + st * kQBytes + bx * kQBox, &map_k, &bars[A_K_FULL0 + st], bx * 64, wk.start + j * kStep, wk.h, wk.b);
                }
            }
        }
    } else if (warp == 18) {
        // ------------------------------------------------------------------ TMA: V ring
        if (lane == 0) {
            uint32_t G = 0;
            bool ok = true;
            SchedConsumer sched;
            int w;
            Work wk;
            while (ok && (w = sched.next(ring, &bars[A_WORK_FULL0], &bars[A_WORK_EMPTY0], abort_flag, wk)) >= 0) {
                for (int j = 0; j <= wk.qt; ++j, ++G) {
                    const uint32_t st = G & 1;
                    ok = mbar_wait_idle(&bars[A_V_EMPTY0 + st], ((G >> 1) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&bars[A_V_FULL0 + st], kQBytes);
#pragma unroll
                    for (int bx = 0; bx < kBoxes; ++bx)
                        tma_load_4d(sV + st * kQBytes + bx * kQBox, &map_v, &bars[A_V_FULL0 + st], bx * 64, wk.start + j * kStep, wk.h, wk.b);
                }
            }
        }
    } else if (warp == 17) {
        // ------------------------------------------------------------------ MMA issuer
        {
            const bool leader = elect_one();  // the whole warp runs the loops; one lane issues
            constexpr uint32_t idesc_s = make_idesc(kBM, kStep, kF16 ? 0 : 1, 0, 0);
            constexpr uint32_t idesc_dq = make_idesc(kBM, D, kF16 ? 0 : 1, 0, 1);
            const SmemDesc desc_q = make_desc(smem_u32(sQ), 0, 1024), desc_do = make_desc(smem_u32(sDO), 0, 1024);
            const SmemDesc desc_k = make_desc(smem_u32(sK), 0, 1024), desc_v = make_desc(smem_u32(sV), 0, 1024);
            const SmemDesc desc_kmn = make_desc(smem_u32(sK), kQBox, 1024);  // K tile as MN-major operand of dQ
            uint32_t G = 0, items = 0;
            bool ok = true;
            // The item's last step is the diagonal tile; at the ragged end of a sequence its K and V rows behind the end are
            // set to zero (they meet dS = 0 and a masked dP only, but 0 * NaN is NaN): g_rag is that step, krows its rows
            uint32_t g_rag = ~0u;
            int krows = kStep;
            auto issue_s = [&](uint32_t g) {
                const uint32_t kst = g % kDqKStages;
                const SmemDesc dk = {desc_k.lo + kst * (kQBytes >> 4), desc_k.hi};
                ok = mbar_wait(&bars[A_K_FULL0 + kst], (g / kDqKStages) & 1, abort_flag);
                if (!ok) return;
                if (g == g_rag) zero_rows_ool(sK + kst * kQBytes, kBoxes, kQBox, krows, kStep, lane);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t o = (k >> 2) * kQBox + (k & 3) * 32;
                    if (k == 0) mma_ss<false>(leader, tmem + kColS + 128 * (g & 1), desc_q, o, dk, o, idesc_s);
                    else mma_ss<true>(leader, tmem + kColS + 128 * (g & 1), desc_q, o, dk, o, idesc_s);
                }
                mma_commit(leader, &bars[A_S_READY0 + (g & 1)]);
            };
            auto issue_dp = [&](uint32_t g, bool last_of_item) {
                const uint32_t vst = g & 1;
                const SmemDesc dv = {desc_v.lo + vst * (kQBytes >> 4), desc_v.hi};
                ok = mbar_wait(&bars[A_V_FULL0 + vst], (g >> 1) & 1, abort_flag);
                if (!ok) return;
                if (g == g_rag) zero_rows_ool(sV + vst * kQBytes, kBoxes, kQBox, krows, kStep, lane);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t o = (k >> 2) * kQBox + (k & 3) * 32;
                    if (k == 0) mma_ss<false>(leader, tmem + kColDP, desc_do, o, dv, o, idesc_s);
                    else mma_ss<true>(leader, tmem + kColDP, desc_do, o, dv, o, idesc_s);
                }
                mma_commit(leader, &bars[A_DP_READY]);
                mma_commit(leader, &bars[A_V_EMPTY0 + vst]);
                if (last_of_item) mma_commit(leader, &bars[A_QDO_EMPTY]);  // the item's last S was issued before
            };
            SchedConsumer sched;
            int w;
            Work wk;
            while (ok && (w = sched.next(ring, &bars[A_WORK_FULL0], &bars[A_WORK_EMPTY0], abort_flag, wk, leader, true)) >= 0) {
                const int n = wk.qt + 1;
                krows = wk.len - wk.qt * kBM;
                g_rag = krows < kStep ? G + n - 1 : ~0u;
                ok = mbar_wait(&bars[A_QDO_FULL], items & 1, abort_flag);
                if (!ok) break;
                issue_s(G);
                if (ok) issue_dp(G, n == 1);  // the row threads can start as soon as these two are complete
                if (ok && n > 1) issue_s(G + 1);
                for (int j = 0; ok && j < n; ++j) {
                    const uint32_t g = G + j, kst = g % kDqKStages;
                    if (j + 1 < n) {  // dP of the next step as soon as this step's is in registers
                        ok = mbar_wait(&bars[A_LOADED], g & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        issue_dp(g + 1, j + 2 == n);
                        if (!ok) break;
                    }
                    if (j == 0) ok = mbar_wait(&bars[A_DQ_FREE], (items & 1) ^ 1, abort_flag);  // previous dQ read out
                    if (!ok) break;
                    const SmemDesc dkmn = {desc_kmn.lo + kst * (kQBytes >> 4), desc_kmn.hi};
                    const uint32_t a_ds = tmem + kColS + 128 * (g & 1);
                    // dQ += dS K in slices of 32 keys, each as soon as that quarter's dS exists: the quarters finish one after
                    // the other (leftmost first, the prefix chain), and the tensor pipe does not wait for the last one before
                    // it starts on the first
                    // (-1.5 % on long sequences; on packs of short ones, the kDefer instantiation, one barrier for all four
                    // quarters is 3 % faster)
#pragma unroll
                    for (int qq = 0; qq < 4; ++qq) {
                        if (!kDefer || qq == 0) {
                            ok = mbar_wait(&bars[A_DS_READY0 + qq], g & 1, abort_flag);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        if (qq == 0) mma_ts_dyn(leader, tmem + kColDQ, a_ds, dkmn, 0, idesc_dq, j > 0);
                        else mma_ts<true>(leader, tmem + kColDQ, a_ds + qq * 32, dkmn, 2 * qq * 2048, idesc_dq);
                        mma_ts<true>(leader, tmem + kColDQ, a_ds + qq * 32 + 8, dkmn, (2 * qq + 1) * 2048, idesc_dq);
                    }
                    if (!ok) break;
                    mma_commit(leader, &bars[A_K_EMPTY0 + kst]);
                    if (j + 2 < n) issue_s(g + 2);  // into the buffer whose dS the contraction above reads: in order
                }
                if (!ok) break;
                mma_commit(leader, &bars[A_DQ_READY]);
                G += n;
                ++items;
            }
        }
    } else {
        // ------------------------------------------------------------------ row threads: warps 0-3 rightmost quarter ... 12-15 leftmost
        const int kq = 3 - (warp >> 2);        // 32-key quarter of the step this thread owns
        const int hf = kq >> 1, sub = kq & 1;  // its 64-key half (the unit of masking) and the quarter inside it
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const float scale = a.inv_temp * kLog2e;
        uint32_t G = 0, items = 0;
        bool ok = true;
        // With kDefer (chosen by the host for packs of short sequences) a finished item's dq leaves tensor memory one step
        // late: its last contraction needs a while to complete, and waiting for it at the end of the item idles the row
        // threads.  They work on the first step of the next item instead (whose S and dP exist already) and store dq then;
        // the first dQ contraction of the next item waits for A_DQ_FREE, i.e. for this store.
        struct PendingItem {
            int b, h;
            int64_t tok;
            uint32_t item;
            bool row_ok;
        };
        PendingItem pend{};
        bool have_pend = false;
        const auto store_item = [&]() {  // the quarters store 32 columns of every row each
            ok = mbar_wait(&bars[A_DQ_READY], pend.item & 1, abort_flag);
            have_pend = false;
            if (!ok) return;
            tc_fence_after();
            if (kq < D / 32) {
                const int d0 = kq * 32;
                char* orow = a.dq.ptr + 2 * ((int64_t)pend.b * a.dq.sb + (int64_t)pend.h * a.dq.sh + pend.tok * a.dq.st + d0);
                uint32_t v[32];
                tmem_ld32(lane_base + kColDQ + d0, v);
                tmem_wait_ld(v);
                const bool wr = pend.row_ok && (D == 128 || a.head_dim > d0);  // D == 64 serves head dim 32 too
                // two rows per lane pair where items are long (-0.8 %); on packs of short sequences it costs 3-5 %
                if (!kDefer) store_row32_pairs<kF16>(orow, v, a.inv_temp, (int64_t)a.dq.st * 2, wr, lane);
                else if (wr) store_row32<kF16>(orow, v, a.inv_temp);
            }
            tc_fence_before();
            mbar_arrive(&bars[A_DQ_FREE]);
        };
        SchedConsumer sched;
        int w;
        Work wk;
        while (ok && (w = sched.next(ring, &bars[A_WORK_FULL0], &bars[A_WORK_EMPTY0], abort_flag, wk)) >= 0) {
            const int n = wk.qt + 1;
            const int qi = wk.qt * kBM + r;
            const bool row_ok = qi < wk.len;
            const int64_t tok = wk.start + qi;
            float drem = 0.f;
            if (row_ok) {
                const char* dp = a.d_rem.ptr + 2 * ((int64_t)wk.b * a.d_rem.sb + (int64_t)wk.h * a.d_rem.sh + tok * a.d_rem.st);
                drem = kF16 ? __half2float(*(const __half*)dp) : __bfloat162float(*(const __nv_bfloat16*)dp);
            }
            if (kFused && row_ok) {
                // rem also receives do . v; the sum is left for the dk/dv kernel
                const char* dorow = a.d_o.ptr + 2 * ((int64_t)wk.b * a.d_o.sb + (int64_t)wk.h * a.d_o.sh + tok * a.d_o.st);
                const char* vrow = a.v.ptr + 2 * ((int64_t)wk.b * a.v.sb + (int64_t)wk.h * a.v.sh + tok * a.v.st);
                float dot = 0.f;
#pragma unroll 1
                for (int cidx = 0; cidx < D / 32; ++cidx) {
                    float x[32], y[32];
                    if (D == 64 && a.head_dim <= 32 * cidx) break;  // D == 64 serves head dim 32 as well
                    load_row32<kF16>(dorow + cidx * 64, x);
                    load_row32<kF16>(vrow + cidx * 64, y);
#pragma unroll
                    for (int i = 0; i < 32; ++i) dot = fmaf(x[i], y[i], dot);
                }
                drem += dot;
                if (kq == 3) a.drem_eff[(int64_t)wk.h * a.drem_rows + (int64_t)wk.b * a.tokens + wk.start + qi] = drem;
            }
            const float* cw = a.carry_w + ((int64_t)wk.h * a.slot_cap) * kTileQ + r;
            float* cc = a.carry_c + ((int64_t)wk.h * a.slot_cap) * kTileQ + r;
            // the half may lie beyond the end of the sequence (its carry slot does not exist): then W = 0, no weights
            const auto half_ok = [&](int j) { return row_ok && (2 * j + hf) * kBK < wk.len; };
            for (int j = 0; j < n; ++j) {
                const uint32_t g = G + j, buf = g & 1;
                const int kh = 2 * j + hf;
                const int64_t slot = carry_slot32(wk.slot_base, wk.qt, 4 * j + kq) * kTileQ;
                float W = half_ok(j) ? __ldg(cw + slot) : 0.f;
                ok = mbar_wait(&bars[A_S_READY0 + buf], (g >> 1) & 1, abort_flag) && mbar_wait(&bars[A_DP_READY], g & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const bool masked = kh >= 2 * wk.qt;  // the half reaches the diagonal
                const int lim = min(kBK, max(0, qi - kh * kBK + a.attend_current));
                uint32_t sv[32], gv[32], packed[16];
                tmem_ld32(lane_base + kColS + 128 * buf + 32 * kq, sv);
                tmem_ld32(lane_base + kColDP + 32 * kq, gv);
                tmem_wait_ld(sv, gv);
                tc_fence_before();
                mbar_arrive(&bars[A_LOADED]);  // dP is free once all have arrived; see the wait below
                if (j + 1 < n) prefetch_l2(cw + slot + 4 * kTileQ);  // the next step's carry on its way into the L2
                if (masked) dq_half_pass1<true>(sv, gv, scale, 32 * sub, lim, drem, W);
                else dq_half_pass1<false>(sv, gv, scale, 32 * sub, lim, drem, W);
                float cl = 0.f;  // prefix of g inside the quarter
                dq_half_local(sv, gv, cl);
                // Every thread has begun this step once it has arrived at A_LOADED.  The wait keeps the row threads within one
                // step of each other: the four warps of 32 rows exchange prefixes among themselves only, and without it one
                // such quartet could finish the next step (dP of which is computed as soon as everybody has loaded this one)
                // and complete this step's phase of its quarter's A_DS_READY with its arrivals before another quartet has written its dS
                // (seen as garbage in dq of 32 rows, now and then).  It also keeps the exchange slots and barriers safe across
                // items.  Barriers by step parity, so that a waiter is never two phases away from the phase it names.
                ok = mbar_wait(&bars[A_LOADED], g & 1, abort_flag);
                if (!ok) break;
                const uint32_t par = g & 1, ph = (g >> 1) & 1;
                // The prefix of g travels along the row as a chain: a thread takes the prefix at its left edge from the
                // quarter to its left (the leftmost one from the rightmost quarter of the previous step), adds its total
                // and passes it on.  Nobody waits for a quarter to its right, so the quarters settle into a stagger and
                // the waits of one overlap with the arithmetic of another.
                float c_edge = 0.f;
                if (kq > 0) {
                    ok = mbar_wait(&bars[A_X_G0 + 8 * (kq - 1) + 4 * par + (warp & 3)], ph, abort_flag);
                    if (!ok) break;
                    c_edge = xg[(kq - 1) * 128 + r];
                } else if (j > 0) {
                    ok = mbar_wait(&bars[A_X_G0 + 8 * 3 + 4 * (par ^ 1) + (warp & 3)], ((g - 1) >> 1) & 1, abort_flag);
                    if (!ok) break;
                    c_edge = xg[3 * 128 + r];
                }
                const float c_right = c_edge + cl;  // prefix through the quarter's right edge
                xg[kq * 128 + r] = c_right;
                mbar_arrive(&bars[A_X_G0 + 8 * kq + 4 * par + (warp & 3)]);
                if (half_ok(j)) cc[slot] = c_right;  // for the dk/dv kernel
                // dS goes over the first 16 of this thread's own 32 score columns, which nobody else reads or writes.  The
                // contraction finds the 16 keys of k-step k at columns 32 * (k / 2) + 8 * (k % 2).
                dq_half_finish<kF16>(sv, gv, c_edge, packed);
                tmem_st16(lane_base + kColS + 128 * buf + 32 * kq, packed);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bars[A_DS_READY0 + (kDefer ? 0 : kq)]);
                if (kDefer && j == 0 && have_pend) {
                    store_item();
                    if (!ok) break;
                }
            }
            if (!ok) break;
            pend = PendingItem{wk.b, wk.h, tok, items, row_ok};
            have_pend = true;
            if (!kDefer) {
                store_item();
                if (!ok) break;
            }
            G += n;
            ++items;
        }
        if (kDefer && ok && have_pend) store_item();  // the block's last item
    }
    tc_teardown(abort_flag, a.status, tmem, kCols, 17);
    sched_finish(a.sched + 2);
}

// ================================================================================================ dk/dv kernel
// One block per SM (608 threads: 19 warps put five on one scheduler, which caps a thread at 96 registers) keeps a 128-key tile stationary and walks the 128-row query
// tiles below it.  All four contractions run with M = 128 and N = 128 (N = D for the last two), the widest shape that 512
// columns of tensor memory allow: S and dP [128 q x 128 keys], dv and dk [128 keys x D] (an MMA instruction costs the same
// ~65 cycles for N = 64 and N = 128, so narrow tiles waste half of the tensor pipe).  Tensor memory is full with these
// four, so S and dP cannot be double-buffered; the step is pipelined another way:
//   * a row thread copies its 32 scores and 32 dP values to registers as soon as they exist and releases S / dP at once,
//     so the tensor cores compute S, dP of the next query tile while the threads work on this one;
//   * the row threads form two halves by query row (rows 0-63 / 64-127).  dv += p^T do and dk += ds^T q reduce
//     over query rows, so each half contributes its own four k-steps; the halves share ONE pair of p / ds buffers of
//     64 rows and take turns.  The buffers are two regions of 32 rows that are written and consumed alternately, four
//     contraction batches per step;
//   * Q and dO are loaded twice from the L2: whole tiles one step early for S, dP (one slot each), and as 64-row halves
//     just in time for dk, dv (one slot per half).  Holding a tile from its first use to its last would need three
//     slots per operand, which shared memory does not have;
//   * across items the issuing warp orders the contractions as: last dV, dK of the item, then the wait for the next item's
//     K, V and its first S, dP, which run while the row threads store dk, dv.
// Sixteen row warps: a thread owns one query row and a quarter (32 keys) of the tile, warps 0-3 the rightmost quarter ...
// warps 12-15 the leftmost; every quarter is entered independently with carry_w and carry_c of its right edge (both exist
// at every 32-key boundary), which the thread loads itself at the top of the step: with four row warps per scheduler the
// latency is covered.  Warp 16 loads K, V (once per item) and the early Q, dO tiles, warp 18 the late halves, warp 17
// issues every tcgen05.mma.
constexpr int kKvThreads = 608;
constexpr int kKT = 128;  // keys per stationary tile
enum KvBar { B_KV_FULL, B_KV_EMPTY, B_E_FULL, B_E_EMPTY, B_L_FULL0, B_L_FULL1, B_L_EMPTY0, B_L_EMPTY1, B_SDP_READY, B_LOADED,
             B_PDS_READY0, B_PDS_READY1, B_PDS_FREE0, B_PDS_FREE1, B_PDS_FREE2, B_PDS_FREE3, B_DKV_READY, B_DKV_FREE, B_WORK_FULL0,
             B_WORK_FULL1, B_WORK_EMPTY0, B_WORK_EMPTY1, kNumKvBars };

struct KvWork {
    int h, b, start, len, kt, slot_base, n_qt;
};
__device__ __forceinline__ KvWork fetch_kv_work(const KArgs& a, int n_items, int w) {
    // groups of head_group heads; inside a group the 128-key tiles heaviest first (key tiles are heaviest where
    // query tiles are lightest: the item table is walked backwards), the heads of the group innermost
    const int per_group = n_items * a.head_group;
    const int g = w / per_group, rest = w - g * per_group;
    const int hg = min(a.head_group, a.heads - g * a.head_group);
    const int idx = rest / hg;
    const int2 it = a.items[n_items - 1 - idx];
    const SeqInfo s = a.seqs[it.x];
    KvWork k;
    k.h = g * a.head_group + rest - idx * hg;
    k.b = s.batch; k.start = s.start; k.len = s.len; k.slot_base = s.slot_base;
    k.kt = it.y;
    k.n_qt = (s.len + kBM - 1) / kBM;
    return k;
}

template <bool kMasked, bool kF16>
__device__ __forceinline__ void kv_chunk(const uint32_t (&s)[32], const uint32_t (&dp)[32], float scale, int col0, int lim,
                                         float drem, float& c, float& W, uint32_t* pp, uint32_t* ps) {
    // right to left over 32 columns: p = W * beta = W - W * om and ds = g - beta * c = om * c - (c - g), where c enters as
    // the inclusive prefix of g at the chunk's right edge and loses every g it passes
#pragma unroll
    for (int q = 7; q >= 0; --q) {
        float2 om[2];
        stick4<kMasked>(__uint_as_float(s[4 * q]), __uint_as_float(s[4 * q + 1]), __uint_as_float(s[4 * q + 2]),
                        __uint_as_float(s[4 * q + 3]), scale, col0 + 4 * q, lim, om[0], om[1]);
#pragma unroll
        for (int h = 1; h >= 0; --h) {
            const int jj = 2 * q + h;
            const float2 t = __fadd2_rn(make_float2(__uint_as_float(dp[2 * jj]), __uint_as_float(dp[2 * jj + 1])),
                                        make_float2(-drem, -drem));
            const float w1 = W * om[h].y, p1 = W - w1;
            const float w0 = w1 * om[h].x, p0 = w1 - w0;
            W = w0;
            const float2 g = __fmul2_rn(make_float2(p0, p1), t);
            const float c1 = c - g.y;
            const float ds1 = fmaf(om[h].y, c, -c1);
            const float c0 = c1 - g.x;
            const float ds0 = fmaf(om[h].x, c1, -c0);
            c = c0;
            pp[jj] = pack16<kF16>(p0, p1);
            ps[jj] = pack16<kF16>(ds0, ds1);
        }
    }
}

// dk or dv of a finished item out of tensor memory: a thread holds one key row and D / 2 columns of the head dim, from
// chunk0 * 32 on.
// Not inlined: it runs once per item, and inside the step loop it would only dilute the instruction cache.
// With the fused remainder dv also receives rem * do of its own row: the direct path of out = o + rem * v.
template <int D, bool kF16, bool kFused>
__device__ __forceinline__ void kv_store_rows_inl(const KArgs& a, bool is_dv, const KvWork e, int r, uint32_t taddr, int chunk0,
                                                  int n_chunks) {
    tc_fence_after();
    const MatView m = is_dv ? a.dv : a.dk;
    const float sc = is_dv ? 1.f : a.inv_temp;
    const bool key_ok = e.kt * kKT + r < e.len;
    const int64_t tok = e.start + e.kt * kKT + r;
    char* orow = m.ptr + 2 * ((int64_t)e.b * m.sb + (int64_t)e.h * m.sh + tok * m.st);
    const char* add = nullptr;
    float mul = 0.f;
    if (kFused && is_dv && key_ok) {
        add = a.d_o.ptr + 2 * ((int64_t)e.b * a.d_o.sb + (int64_t)e.h * a.d_o.sh + tok * a.d_o.st);
        const char* rp = a.rem.ptr + 2 * ((int64_t)e.b * a.rem.sb + (int64_t)e.h * a.rem.sh + tok * a.rem.st);
        mul = kF16 ? __half2float(*(const __half*)rp) : __bfloat162float(*(const __nv_bfloat16*)rp);
    }
#pragma unroll
    for (int cc = 0; cc < D / 64; ++cc) {  // this thread's half of the head dim, 32 columns at a time
        const int cidx = chunk0 + cc;
        uint32_t v[32];
        tmem_ld32(taddr + cidx * 32, v);
        tmem_wait_ld(v);
        if (!(kFused && is_dv)) {  // two rows per lane pair: -7 % on a pack of 128-token sequences, -0.6 % on long ones
            // (the same in the forward and the dq kernel, whose threads store half as much, cost 1-5 %)
            store_row32_pairs<kF16>(orow + cidx * 64, v, sc, (int64_t)m.st * 2, key_ok && (D == 128 || cc < n_chunks), (int)(threadIdx.x & 31));
        } else if (key_ok && (D == 128 || cc < n_chunks)) {  // D == 64 serves head dim 32 as well: then fewer chunks exist
            if (kFused && add) {
                float x[32];
                load_row32<kF16>(add + cidx * 64, x);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(fmaf(mul, x[i], __uint_as_float(v[i])));
                store_row32<kF16>(orow + cidx * 64, v, 1.f);
            } else {
                store_row32<kF16>(orow + cidx * 64, v, sc);
            }
        }
    }
    tc_fence_before();
}
template <int D, bool kF16, bool kFused>
__device__ __noinline__ void kv_store_rows(const KArgs& a, bool is_dv, const KvWork e, int r, uint32_t taddr, int chunk0, int n_chunks) {
    kv_store_rows_inl<D, kF16, kFused>(a, is_dv, e, r, taddr, chunk0, n_chunks);
}

template <int D, bool kF16, bool kFused, bool kDefer>
__global__ void __launch_bounds__(kKvThreads, 1)
tc_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_q64, const __grid_constant__ CUtensorMap map_do64,
                   const __grid_constant__ KArgs a) {
    constexpr int kBoxes = D / 64;
    constexpr int kQBytes = kBM * D * 2;     // a 128-row tile of Q, dO, K or V
    constexpr int kHalfBytes = kQBytes / 2;  // 64 rows of Q or dO: kBoxes boxes of kKBox bytes
    constexpr int kBufBytes = 2 * 64 * 128;  // 64 query rows x 128 keys, 16-bit, as two 64-key blocks
    constexpr uint32_t kColS = 0, kColDP = 128, kColDK = 256, kColDV = 384;
    constexpr uint32_t kCols = 512;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;
    uint8_t* sV = sK + kQBytes;
    uint8_t* sQe = sV + kQBytes;     // Q of the step whose S is computed next
    uint8_t* sDOe = sQe + kQBytes;   // dO of the step whose dP is computed next
    uint8_t* sQl = sDOe + kQBytes;   // Q of the step whose dk is accumulated next: two 64-row halves
    uint8_t* sDOl = sQl + kQBytes;   // dO of the step whose dv is accumulated next: two 64-row halves
    uint8_t* sP = sDOl + kQBytes;
    uint8_t* sDS = sP + kBufBytes;
    uint64_t* bars = (uint64_t*)(sDS + kBufBytes);
    uint32_t* tmem_slot = (uint32_t*)(bars + kNumKvBars);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    SchedRing<KvWork>* ring = (SchedRing<KvWork>*)(tmem_slot + 2);
    static_assert(sizeof(SchedRing<KvWork>) <= 72, "ring does not fit its place");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < kNumKvBars; ++i) {
            uint32_t cnt = 1;
            if (i == B_LOADED || i == B_DKV_FREE) cnt = 512;
            if (i == B_PDS_READY0 || i == B_PDS_READY1) cnt = 128;  // the four warps of 32 query rows
            if (i == B_WORK_EMPTY0 || i == B_WORK_EMPTY1) cnt = 514;  // MMA warp (one lane), late producer, 512 row threads
            mbar_init(&bars[i], cnt);
        }
        *abort_flag = (smem_u32(smem) & 1023u) ? 1u : 0u;  // the swizzled tiles need a 1024-byte aligned base
        fence_barrier_init();
    }
    if (warp == 17) {
        tmem_alloc(tmem_slot, kCols);
        tmem_relinquish();
    }
    if (warp == 16 && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
        tma_prefetch_desc(&map_q64);
        tma_prefetch_desc(&map_do64);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int n_items = a.hdr->n_items;
    const int n_work = *abort_flag ? 0 : n_items * a.heads;
    // G counts query-tile steps over all items of this block; a barrier that completes once per step is in phase G & 1.

    if (warp == 16) {
        // ------------------------------------------------------------------ TMA: K, V per item; Q, dO tiles for S, dP
        if (lane == 0) {
            uint32_t G = 0, items = 0;
            bool ok = true;
            SchedProducer sched;
            int w;
            KvWork wk;
            const auto fetch = [&](int w_) { return fetch_kv_work(a, n_items, w_); };
            while (ok && (w = sched.next(a.sched + 4, n_work, ring, &bars[B_WORK_FULL0], &bars[B_WORK_EMPTY0], abort_flag, fetch, wk)) >= 0) {
                ok = mbar_wait_idle(&bars[B_KV_EMPTY], (items & 1) ^ 1, abort_flag);
                ++items;
                if (!ok) break;
                mbar_expect_tx(&bars[B_KV_FULL], 2 * kQBytes);
#pragma unroll
                for (int bx = 0; bx < kBoxes; ++bx) {
                    tma_load_4d(sK + bx * kQBox, &map_k, &bars[B_KV_FULL], bx * 64, wk.start + wk.kt * kKT, wk.h, wk.b);
                    tma_load_4d(sV + bx * kQBox, &map_v, &bars[B_KV_FULL], bx * 64, wk.start + wk.kt * kKT, wk.h, wk.b);
                }
                for (int i = wk.kt; i < wk.n_qt; ++i, ++G) {
                    ok = mbar_wait_idle(&bars[B_E_EMPTY], (G & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&bars[B_E_FULL], 2 * kQBytes);
#pragma unroll
                    for (int bx = 0; bx < kBoxes; ++bx) {
                        tma_load_4d(sQe + bx * kQBox, &map_q, &bars[B_E_FULL], bx * 64, wk.start + i * kBM, wk.h, wk.b);
                        tma_load_4d(sDOe + bx * kQBox, &map_do, &bars[B_E_FULL], bx * 64, wk.start + i * kBM, wk.h, wk.b);
                    }
                }
            }
        }
    } else if (warp == 18) {
        // ------------------------------------------------------------------ TMA: 64-row halves of Q, dO for dk, dv
        if (lane == 0) {
            uint32_t G = 0;
            bool ok = true;
            SchedConsumer sched;
            int w;
            KvWork wk;
            while (ok && (w = sched.next(ring, &bars[B_WORK_FULL0], &bars[B_WORK_EMPTY0], abort_flag, wk)) >= 0) {
                for (int i = wk.kt; ok && i < wk.n_qt; ++i, ++G) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        ok = mbar_wait_idle(&bars[B_L_EMPTY0 + hh], (G & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        mbar_expect_tx(&bars[B_L_FULL0 + hh], kQBytes);
#pragma unroll
                        for (int bx = 0; bx < kBoxes; ++bx) {
                            tma_load_4d(sQl + hh * kHalfBytes + bx * kKBox, &map_q64, &bars[B_L_FULL0 + hh], bx * 64,
                                        wk.start + i * kBM + hh * 64, wk.h, wk.b);
                            tma_load_4d(sDOl + hh * kHalfBytes + bx * kKBox, &map_do64, &bars[B_L_FULL0 + hh], bx * 64,
                                        wk.start + i * kBM + hh * 64, wk.h, wk.b);
                        }
                    }
                }
            }
        }
    } else if (warp == 17) {
        // ------------------------------------------------------------------ MMA issuer
        {
            const bool leader = elect_one();  // the whole warp runs the loops; one lane issues
            constexpr uint32_t idesc_s = make_idesc(kBM, kKT, kF16 ? 0 : 1, 0, 0);
            constexpr uint32_t idesc_t = make_idesc(kKT, D, kF16 ? 0 : 1, 1, 1);  // (P^T or dS^T)[128 keys x q] * (dO or Q)[q x D]
            const SmemDesc desc_q = make_desc(smem_u32(sQe), 0, 1024), desc_do = make_desc(smem_u32(sDOe), 0, 1024);  // K-major
            const SmemDesc desc_k = make_desc(smem_u32(sK), 0, 1024), desc_v = make_desc(smem_u32(sV), 0, 1024);
            const SmemDesc desc_qmn = make_desc(smem_u32(sQl), kKBox, 1024), desc_domn = make_desc(smem_u32(sDOl), kKBox, 1024);  // MN-major
            const SmemDesc desc_p = make_desc(smem_u32(sP), kKBox, 1024), desc_ds = make_desc(smem_u32(sDS), kKBox, 1024);
            bool ok = true;
            // Ragged ends.  The rows of a tile behind the end of its sequence belong to the next sequence or to nobody; they
            // meet zero weights only, but a zero weight does not silence a NaN.  K, V of the sequence's last key tile: the
            // rows behind the end are set to zero.  Q, dO of its last query tile, which is the last step of every item:
            // dk, dv contract over query rows in slices of 16, so the slices that lie behind the end are not issued at all,
            // and only the rows between the end and the next multiple of 16 are set to zero, in all four copies of the
            // tile (with Q and dO zero, S and dP of such a row are zero, and so are its p and ds).
            const auto zero_kv = [&](const KvWork& e) {
                const int krows = e.len - e.kt * kKT;
                if (krows < kKT) {
                    zero_rows(sK, kBoxes, kQBox, krows, kKT, lane);
                    zero_rows(sV, kBoxes, kQBox, krows, kKT, lane);
                    zero_rows_done();
                }
            };
            const auto last_rows = [](const KvWork& e) { return e.len - (e.n_qt - 1) * kBM; };  // 1 ... 128
            auto issue_sdp = [&](uint32_t g, bool last_of_item, int qrows) {
                ok = mbar_wait(&bars[B_E_FULL], g & 1, abort_flag);
                if (!ok) return;
                if (last_of_item && (qrows & 15)) {
                    zero_rows_to_16(sQe, kBoxes, kQBox, qrows, lane);
                    zero_rows_to_16(sDOe, kBoxes, kQBox, qrows, lane);
                    zero_rows_done();
                }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t o = (k >> 2) * kQBox + (k & 3) * 32;
                    if (k == 0) mma_ss<false>(leader, tmem + kColS, desc_q, o, desc_k, o, idesc_s);
                    else mma_ss<true>(leader, tmem + kColS, desc_q, o, desc_k, o, idesc_s);
                }
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t o = (k >> 2) * kQBox + (k & 3) * 32;
                    if (k == 0) mma_ss<false>(leader, tmem + kColDP, desc_do, o, desc_v, o, idesc_s);
                    else mma_ss<true>(leader, tmem + kColDP, desc_do, o, desc_v, o, idesc_s);
                }
                mma_commit(leader, &bars[B_SDP_READY]);
                mma_commit(leader, &bars[B_E_EMPTY]);
                if (last_of_item) mma_commit(leader, &bars[B_KV_EMPTY]);
            };
            // S, dP of step g + 1 are issued as soon as the row threads hold those of step g in registers. Across items
            // the order is: the last step's dV, dK contractions, then the wait for the next item's K, V (one buffer each,
            // free after the item's last S, dP) and its first S, dP, which run while the row threads store dk, dv.
            // Waiting for the next K, V before the last dV, dK measured 8% slower.
            SchedConsumer sched;
            KvWork wk, nx;
            uint32_t g = 0, items = 0;
            bool have = sched.next(ring, &bars[B_WORK_FULL0], &bars[B_WORK_EMPTY0], abort_flag, wk, leader, true) >= 0;
            if (have) {
                ok = mbar_wait(&bars[B_KV_FULL], 0, abort_flag);
                if (ok) {
                    zero_kv(wk);
                    issue_sdp(0, wk.n_qt - wk.kt == 1, last_rows(wk));
                }
            }
            while (ok && have) {
                const int n = wk.n_qt - wk.kt;
                const int qrows = last_rows(wk);
                for (int j = 0; ok && j < n; ++j, ++g) {
                    const int rows = j + 1 == n ? qrows : kBM;  // query rows of this step that belong to the sequence
                    if (j + 1 < n) {
                        ok = mbar_wait(&bars[B_LOADED], g & 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        issue_sdp(g + 1, j + 2 == n, qrows);
                    } else {  // the next item is fetched here, off the path between two items
                        have = sched.next(ring, &bars[B_WORK_FULL0], &bars[B_WORK_EMPTY0], abort_flag, nx, leader, true) >= 0;
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {  // 32 query rows at a time: region i & 1 of the p / ds buffers
                        const int hh = i >> 1, b = i & 1;
                        if (b == 0) {
                            ok = mbar_wait(&bars[B_L_FULL0 + hh], g & 1, abort_flag);
                            if (!ok) break;
                            // the slice of 16 rows that straddles the end, in its 64-row half: here, while the row threads
                            // are still at work on the region's p and ds, and not when the contractions are due
                            if ((rows & 15) && (rows >> 6) == hh) {
                                zero_rows_to_16(sQl + hh * kHalfBytes, kBoxes, kKBox, rows & 63, lane);
                                zero_rows_to_16(sDOl + hh * kHalfBytes, kBoxes, kKBox, rows & 63, lane);
                                zero_rows_done();
                            }
                        }
                        ok = mbar_wait(&bars[B_PDS_READY0 + b], hh, abort_flag);  // a region is used twice per step
                        if (ok && j == 0 && i == 0)  // the previous item's accumulators must have been read out
                            ok = mbar_wait(&bars[B_DKV_FREE], (items & 1) ^ 1, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        const SmemDesc ddo = {desc_domn.lo + hh * (kHalfBytes >> 4), desc_domn.hi};
                        const SmemDesc dq = {desc_qmn.lo + hh * (kHalfBytes >> 4), desc_qmn.hi};
                        if (32 * i < rows) {  // slices of 16 query rows that lie behind the end of the sequence are left out
                            mma_ss_dyn(leader, tmem + kColDV, desc_p, b * 4096, ddo, b * 4096, idesc_t, j > 0 || i > 0);
                            if (32 * i + 16 < rows) mma_ss<true>(leader, tmem + kColDV, desc_p, b * 4096 + 2048, ddo, b * 4096 + 2048, idesc_t);
                            mma_ss_dyn(leader, tmem + kColDK, desc_ds, b * 4096, dq, b * 4096, idesc_t, j > 0 || i > 0);
                            if (32 * i + 16 < rows) mma_ss<true>(leader, tmem + kColDK, desc_ds, b * 4096 + 2048, dq, b * 4096 + 2048, idesc_t);
                        }
                        mma_commit(leader, &bars[B_PDS_FREE0 + 2 * b + hh]);
                        if (b == 1) mma_commit(leader, &bars[B_L_EMPTY0 + hh]);
                    }
                }
                if (!ok) break;
                mma_commit(leader, &bars[B_DKV_READY]);
                ++items;
                wk = nx;
                if (have) {
                    ok = mbar_wait(&bars[B_LOADED], (g - 1) & 1, abort_flag) && mbar_wait(&bars[B_KV_FULL], items & 1, abort_flag);
                    if (!ok) break;
                    zero_kv(wk);
                    tc_fence_after();
                    issue_sdp(g, wk.n_qt - wk.kt == 1, last_rows(wk));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ row threads
        const int kq = 3 - (warp >> 2);        // 32-key quarter of the tile this thread owns
        const int hf = kq >> 1, sub = kq & 1;  // its 64-key half (a block of the p / ds buffers, the unit of masking)
        const int hh = (warp & 3) >> 1;        // half of the query rows this thread belongs to
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const float scale = a.inv_temp * kLog2e;
        uint8_t* prow = sP + hf * kKBox + (r & 63) * 128;
        uint8_t* srow = sDS + hf * kKBox + (r & 63) * 128;
        uint32_t G = 0, items = 0;
        bool ok = true;
        // dk (even quarters) / dv (odd quarters) are stored when the item's last contractions are complete, half of the
        // head dim per thread; S, dP of the next item's first step are computed meanwhile
        // 32-column chunks of the head dim this thread stores: D / 64 of them from chunk hf * (D / 64) on; none for the
        // second half of the columns when D == 64 serves head dim 32
        const int kv_chunks = max(0, min(D / 64, a.head_dim / 32 - hf * (D / 64)));
        auto store_dkdv = [&](const KvWork& e, uint32_t item) {
            ok = mbar_wait(&bars[B_DKV_READY], item & 1, abort_flag);
            if (!ok) return;
            if (kDefer) kv_store_rows_inl<D, kF16, kFused>(a, sub == 1, e, r, lane_base + (sub == 0 ? kColDK : kColDV), hf * (D / 64), kv_chunks);
            else kv_store_rows<D, kF16, kFused>(a, sub == 1, e, r, lane_base + (sub == 0 ? kColDK : kColDV), hf * (D / 64), kv_chunks);
            mbar_arrive(&bars[B_DKV_FREE]);
        };
        SchedConsumer sched;
        int w;
        KvWork wk;
        // With kDefer (packs of sequences of one tile) dk, dv of a finished item are stored inside the first step of the next
        // item: the item's last contractions need a while to complete; the first contraction of the next item waits for
        // B_DKV_FREE, i.e. for this store
        KvWork pend{};
        uint32_t pend_item = 0;
        bool have_pend = false;
        while (ok && (w = sched.next(ring, &bars[B_WORK_FULL0], &bars[B_WORK_EMPTY0], abort_flag, wk)) >= 0) {
            const int n = wk.n_qt - wk.kt;
            const int kh = 2 * wk.kt + hf;
            const float* cw = a.carry_w + ((int64_t)wk.h * a.slot_cap) * kTileQ + r;
            const float* cc = a.carry_c + ((int64_t)wk.h * a.slot_cap) * kTileQ + r;
            const bool half_ok = kh * kBK < wk.len;  // the half may lie beyond the end of the sequence
            // the scalars of a step: carry_w and the prefix of g at the quarter's right edge, drem of the row.  Those of the
            // next step are loaded after this step's arithmetic, so that they are in flight across the waits in between
            // and occupy no register during the arithmetic.
            // (drem stays in its 16-bit form until it is used: a conversion right behind the load would stall the warp
            // until the value has arrived)
            const auto load_scalars = [&](int i, float& W, float& c, uint32_t& drem) {
                const int qi = i * kBM + r;
                W = 0.f; c = 0.f; drem = 0u;
                if (qi < wk.len) {
                    if (half_ok) {
                        const int64_t slot = carry_slot32(wk.slot_base, i, 4 * wk.kt + kq) * kTileQ;
                        W = __ldg(cw + slot);
                        c = __ldg(cc + slot);  // loses every g it passes
                    }
                    if (kFused) {  // drem + do . v (float32), left behind by the dq kernel
                        drem = __ldg((const uint32_t*)a.drem_eff + (int64_t)wk.h * a.drem_rows + (int64_t)wk.b * a.tokens + wk.start + qi);
                    } else {
                        const char* dp = a.d_rem.ptr + 2 * ((int64_t)wk.b * a.d_rem.sb + (int64_t)wk.h * a.d_rem.sh +
                                                            (int64_t)(wk.start + qi) * a.d_rem.st);
                        drem = __ldg((const unsigned short*)dp);
                    }
                }
            };
            const auto drem_value = [](uint32_t raw) {
                if (kFused) return __uint_as_float(raw);
                return kF16 ? __half2float(__ushort_as_half((unsigned short)raw)) : __uint_as_float(raw << 16);
            };
            float W, c;
            uint32_t drem_raw;
            load_scalars(wk.kt, W, c, drem_raw);
            for (int j = 0; j < n; ++j) {
                const int i = wk.kt + j;
                const uint32_t g = G + j;
                const int qi = i * kBM + r;
                ok = mbar_wait(&bars[B_SDP_READY], g & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const bool masked = i == wk.kt;
                const int lim = min(kBK, max(0, qi - kh * kBK + a.attend_current));
                uint32_t pp[16], ps[16];
                {
                    uint32_t s1[32], d1[32];
                    tmem_ld32(lane_base + kColS + 32 * kq, s1);
                    tmem_ld32(lane_base + kColDP + 32 * kq, d1);
                    tmem_wait_ld(s1, d1);
                    tc_fence_before();
                    mbar_arrive(&bars[B_LOADED]);  // S and dP of this step are free
                    const float drem = drem_value(drem_raw);
                    if (masked) kv_chunk<true, kF16>(s1, d1, scale, 32 * sub, lim, drem, c, W, pp, ps);
                    else kv_chunk<false, kF16>(s1, d1, scale, 32 * sub, lim, drem, c, W, pp, ps);
                }
                if (j + 1 < n) load_scalars(i + 1, W, c, drem_raw);
                if (kDefer && j == 0 && have_pend) {
                    // Here and not after this step's p / ds have been written: the second row half can write only when the
                    // first half's contraction of this step is complete, and that contraction waits for B_DKV_FREE.
                    store_dkdv(pend, pend_item);
                    have_pend = false;
                    if (!ok) break;
                }
                // The 64-row p / ds buffers are two regions of 32 rows, each used by one warp quartet of either row half
                // in turn (rows 0-31 and 64-95 the first region, 32-63 and 96-127 the second).  A region is free once the
                // contractions of its previous use are complete: the other half's, of the previous step for half 0 and of
                // this step for half 1.  While one region is consumed the other is written, so the contractions of a step
                // follow each other without waiting for the row threads.  One "free" barrier per region and half, completing
                // once per step, and a thread waits for the other half's: a waiter is never two phases away from the phase
                // it names (with one barrier per region, completing twice per step, a thread of half 0 could arrive while
                // its own previous use was still pending and mistake the completion before that for the one it wants).
                ok = mbar_wait(&bars[B_PDS_FREE0 + 2 * (warp & 1) + (hh ^ 1)], (g & 1) ^ (hh ^ 1), abort_flag);
                if (!ok) break;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    const int off = ((4 * sub + ch) ^ (r & 7)) << 4;
                    *(uint4*)(prow + off) = make_uint4(pp[4 * ch], pp[4 * ch + 1], pp[4 * ch + 2], pp[4 * ch + 3]);
                    *(uint4*)(srow + off) = make_uint4(ps[4 * ch], ps[4 * ch + 1], ps[4 * ch + 2], ps[4 * ch + 3]);
                }
                fence_async_smem();
                mbar_arrive(&bars[B_PDS_READY0 + (warp & 1)]);
            }
            if (!ok) break;
            if (kDefer) {
                pend = wk;
                pend_item = items;
                have_pend = true;
            } else {
                store_dkdv(wk, items);
                if (!ok) break;
            }
            G += n;
            ++items;
        }
        if (kDefer && ok && have_pend) store_dkdv(pend, pend_item);  // the block's last item
    }
    tc_teardown(abort_flag, a.status, tmem, kCols, 17);
    sched_finish(a.sched + 4);
}

template <int D, bool kF16, bool kFused>
int launch_bwd_kernels(const SbParams& p, const KArgs& a, cudaStream_t st, const CUtensorMap& mq, const CUtensorMap& mk128,
                       const CUtensorMap& mv128, const CUtensorMap& mdo, const CUtensorMap& mq64, const CUtensorMap& mdo64,
                       int smem_a, int smem_b) {
    const auto launch_dq = [&](auto kernel) {
        const int e = ensure_kernel_attrs((const void*)kernel, smem_a, true);
        if (e != 0) return e;
        kernel<<<sm_count(), kDqThreads, smem_a, st>>>(mq, mk128, mv128, mdo, a);
        count_launch();
        return (int)cudaGetLastError();
    };
    const auto launch_dkdv = [&](auto kernel) {
        const int e = ensure_kernel_attrs((const void*)kernel, smem_b, true);
        if (e != 0) return e;
        kernel<<<sm_count(), kKvThreads, smem_b, st>>>(mq, mk128, mv128, mdo, mq64, mdo64, a);
        count_launch();
        return (int)cudaGetLastError();
    };
    if (p.bwd_phases != SBATTN_BWD_DKDV) {
        const int e = a.defer_dq ? launch_dq(tc_bwd_dq_kernel<D, kF16, kFused, true>) : launch_dq(tc_bwd_dq_kernel<D, kF16, kFused, false>);
        if (e != 0) return e;
    }
    if (p.bwd_phases != SBATTN_BWD_DQ) {
        const int e = a.defer_dkdv ? launch_dkdv(tc_bwd_dkdv_kernel<D, kF16, kFused, true>)
                                   : launch_dkdv(tc_bwd_dkdv_kernel<D, kF16, kFused, false>);
        if (e != 0) return e;
    }
    return 0;
}

template <int D, bool kF16>
int launch_bwd_t(const SbParams& p, const KArgs& a, cudaStream_t st) {
    // Q, dO, K, V as 128-row tiles; the dk/dv kernel loads Q and dO also as 64-row halves
    CUtensorMap mq, mdo, mk128, mv128, mq64, mdo64;
    const int kind = kF16 ? 2 : 0;
    const int64_t B = p.batch > 0 ? p.batch : 1;
    const int hd = p.head_dim;  // the maps carry the true head dim; TMA fills the columns up to D with zeros
    if (encode_tile_map(&mq, p.q.ptr, kind, hd, p.tokens, p.heads, B, p.q.stride_t, p.q.stride_h, p.q.stride_b, kBM) ||
        encode_tile_map(&mdo, p.d_o.ptr, kind, hd, p.tokens, p.heads, B, p.d_o.stride_t, p.d_o.stride_h, p.d_o.stride_b, kBM) ||
        encode_tile_map(&mk128, p.k.ptr, kind, hd, p.tokens, p.heads, B, p.k.stride_t, p.k.stride_h, p.k.stride_b, kBM) ||
        encode_tile_map(&mv128, p.v.ptr, kind, hd, p.tokens, p.heads, B, p.v.stride_t, p.v.stride_h, p.v.stride_b, kBM) ||
        encode_tile_map(&mq64, p.q.ptr, kind, hd, p.tokens, p.heads, B, p.q.stride_t, p.q.stride_h, p.q.stride_b, kBK) ||
        encode_tile_map(&mdo64, p.d_o.ptr, kind, hd, p.tokens, p.heads, B, p.d_o.stride_t, p.d_o.stride_h, p.d_o.stride_b, kBK))
        return kMapEncodeFailed;
    // dq kernel: q, do, three k stages, two v stages; dk/dv kernel: k, v, early q / do, late q / do, p, ds, scalars
    constexpr int need = 2 * kBM * D * 2 + (kDqKStages + kDqVStages) * kBM * D * 2 + 3072;
    constexpr int need_b = 6 * kBM * D * 2 + 2 * 2 * 64 * 128 + 3072;
    constexpr int smem_a = need > 120 * 1024 ? need : 120 * 1024;  // one block per SM: it owns all 512 tensor-memory columns
    constexpr int smem_b = need_b > 120 * 1024 ? need_b : 120 * 1024;  // one block per SM: it owns all 512 tensor-memory columns
    return a.fused ? launch_bwd_kernels<D, kF16, true>(p, a, st, mq, mk128, mv128, mdo, mq64, mdo64, smem_a, smem_b)
                   : launch_bwd_kernels<D, kF16, false>(p, a, st, mq, mk128, mv128, mdo, mq64, mdo64, smem_a, smem_b);
}

}  // namespace

int launch_tensor_bwd(const SbParams& p, const WsLayout&, const KArgs& a, cudaStream_t st) {
    const bool f16 = p.dtype == SBATTN_F16;
    if (p.head_dim > 64) return f16 ? launch_bwd_t<128, true>(p, a, st) : launch_bwd_t<128, false>(p, a, st);
    return f16 ? launch_bwd_t<64, true>(p, a, st) : launch_bwd_t<64, false>(p, a, st);
}

}  // namespace sb
