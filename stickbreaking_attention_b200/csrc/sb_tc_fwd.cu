// Tensor-core forward (sm_100a): o, rem, neg_log_acc and the carries of W at every 32-key boundary for bf16 / f16 inputs
// with head_dim 32, 64 or 128 (32 runs on the 64-column kernels; TMA pads the tiles with zeros).
//
// One work item = (head, sequence, 128-row query tile); one persistent thread block per SM draws items from a global
// counter (heaviest first, interleaved over small groups of heads so that their K and V stay in L2).  Per item the key
// tiles are visited right to left, from the diagonal to key 0 -- the order of the reference's _forward_one_row
// (stickbreaking_attention/sb_varlen/sb_varlen_fwd.py:155-193) -- because the weight of key j needs the product of
// (1 - beta) over the keys to its right.
//
// Warps of a block (608 threads: 19 warps put five on one scheduler, which caps a thread at 96 registers):
//   0-15       row warps: a thread owns one query row and a quarter (32 keys) of every tile, warps 0-3 the rightmost
//              quarter ... warps 12-15 the leftmost, so that every scheduler has four row warps to choose from.
//              S lives in three rotating buffers in tensor memory, so the tensor cores are always two tiles ahead:
//              while the threads turn scores into weights on the CUDA cores, S of later tiles and O += P V of earlier
//              ones are in flight.  A thread reads its 32 scores, computes the weights RELATIVE to a carry of 1, receives
//              the true carry W (product of 1 - beta over everything to the right of its quarter) from the thread of the
//              quarter to its right through shared memory (the rightmost quarter from the leftmost one of the previous
//              tile), passes its own on, rescales, and writes the weights back to tensor memory as 16-bit operands.
//   16 / 18    TMA producers: warp 16 loads Q once per item and the K tiles (three-stage ring, S runs ahead), warp 18
//              the V tiles (two-stage ring).
//   17         issues tcgen05.mma: S = Q K^T (both operands in shared memory) into the next S buffer of the rotation,
//              O += P V (P from tensor memory, V from shared memory).
// Tensor memory (512 columns): S buffers at columns 0, 128, 256; O [384,384+D).  P overwrites the right half of its S
// buffer: the weights of a quarter land on scores of quarters to its right, whose threads have read them before they
// passed the carry on.
#include "sb_tc_common.cuh"

namespace sb {

using namespace sm100;

namespace {

constexpr int kFwdThreads = 608;
constexpr int kBM = 128, kBN = 128;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColO = 384, kColPOff = 64;  // S buffer i at 128*i (i = step mod 3), its P at +64
constexpr int kKStages = 3, kVStages = 2;
// Eighths of every 32-key chunk whose exponential is computed on the FMA pipes (ex2_fma2) instead of the special-function
// unit.  Measured on the 16384-token benchmark pack (forward, one B200): 0 -> 0.4316 ms, 1 -> 0.4342 ms, 2 -> 0.4455 ms.
// The special-function unit is not what bounds the sweep (it is ~50 % busy), and the polynomial costs five more issue
// slots per score than ex2.approx, so the share stays at zero; the path is kept for shapes where that changes.
constexpr int kFmaExpEighths = 0;
enum FwdBar { Q_FULL, Q_EMPTY, K_FULL0, K_FULL1, K_FULL2, K_EMPTY0, K_EMPTY1, K_EMPTY2, V_FULL0, V_FULL1, V_EMPTY0, V_EMPTY1, S_READY0, S_READY1,
              S_READY2, P_READY0, P_READY1, P_READY2, O_READY, O_FREE, WORK_FULL0, WORK_FULL1, WORK_EMPTY0, WORK_EMPTY1,
              X_W0,  // 32 barriers for the carry chain: [quarter][tile parity][warp & 3]
              kNumBars = X_W0 + 32 };

// With e = exp(s) and d = 1 + e:  beta = e / d,  1 - beta = 1 / d.  For key m of a group of 8 keys entered with the
// carry W (product of 1 - beta over everything to its right)
//     p_m = beta_m * W * prod_{m' > m in group} 1/d_m'  =  e_m * (prod_{m' < m in group} d_m') * W / (prod over the group of d)
// which needs one reciprocal per GROUP instead of one per key.  Scores are clamped at 2^15 (beta = 1 - 3e-5 there)
// so that the product of 8 factors stays below 2^127.  Masked keys get e = 0: weight 0 and no stick broken.
//
// First pass over a chunk of 32 keys: s[idx] <- e * (product of d over the keys of its group to the LEFT);
// run[g] <- product of d over group g.  The four groups are swept side by side so that their chains overlap.
template <bool kMasked>
__device__ __forceinline__ void fwd_sweep(uint32_t (&s)[32], float scale, int col0, int lim, float (&run)[4]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) run[g] = 1.f;
#pragma unroll
    for (int m = 0; m < 8; m += 2) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const int idx = g * 8 + m;  // two adjacent keys: the scaling is one packed fp32x2 multiply
            const float2 x = __fmul2_rn(make_float2(__uint_as_float(s[idx]), __uint_as_float(s[idx + 1])), make_float2(scale, scale));
            float e0, e1;
            if (kFmaExpEighths > 0 && g == 3 && (kFmaExpEighths >= 2 || (m & 2))) {  // this share of the exponentials on the FMA pipes
                const float2 e = ex2_fma2(make_float2(fmaxf(fminf(x.x, 15.f), -125.f), fmaxf(fminf(x.y, 15.f), -125.f)));
                e0 = e.x;
                e1 = e.y;
            } else {
                e0 = ex2_approx(fminf(x.x, 15.f));
                e1 = ex2_approx(fminf(x.y, 15.f));
            }
            if (kMasked && col0 + idx >= lim) e0 = 0.f;
            if (kMasked && col0 + idx + 1 >= lim) e1 = 0.f;
            s[idx] = __float_as_uint(e0 * run[g]);
            run[g] = fmaf(run[g], e0, run[g]);
            s[idx + 1] = __float_as_uint(e1 * run[g]);
            run[g] = fmaf(run[g], e1, run[g]);
        }
    }
}
// carry entering each group from the right: f[g] = W / (product of d over groups g..3); W <- the chunk's exit carry
__device__ __forceinline__ void fwd_carries(const float (&run)[4], float& W, float* f) {
    f[3] = W * rcp_approx(run[3]);
    f[2] = f[3] * rcp_approx(run[2]);
    f[1] = f[2] * rcp_approx(run[1]);
    f[0] = f[1] * rcp_approx(run[0]);
    W = f[0];
}
template <bool kF16>
__device__ __forceinline__ void fwd_finish(const uint32_t (&s)[32], const float* f, float mul, uint32_t (&packed)[16]) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float fj = f[j >> 2] * mul;
        const float2 p = __fmul2_rn(make_float2(__uint_as_float(s[2 * j]), __uint_as_float(s[2 * j + 1])), make_float2(fj, fj));
        packed[j] = pack16<kF16>(p.x, p.y);
    }
}

// kFused: out = o + rem * v is formed in the epilogue (a separate instantiation: the plain one stays as it is)
// kDefer: an item's output is stored after the first step of the next item instead of at the item's end (chosen by the
// host for packs of short sequences, where the wait for the item's last contraction is a large share of the item)
template <int D, bool kF16, bool kFused, bool kDefer>
__global__ void __launch_bounds__(kFwdThreads, 1)
tc_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const KArgs a) {
    constexpr int kTileBytes = kBM * D * 2;
    constexpr int kBoxBytes = 128 * 128;  // one TMA box: 128 rows of 64 elements
    constexpr int kBoxes = D / 64;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + kTileBytes;             // kKStages tiles
    uint8_t* sV = sK + kKStages * kTileBytes;  // kVStages tiles
    uint64_t* bars = (uint64_t*)(sV + kVStages * kTileBytes);
    SchedRing<Work>* ring = (SchedRing<Work>*)(bars + kNumBars);
    uint32_t* tmem_slot = (uint32_t*)(ring + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* xw = (float*)(tmem_slot + 4);  // [quarter][128 rows]: carry leaving the quarter its thread has just swept
    float* wfin = xw + 512;               // [item mod 3][128 rows]: remainder of the row, for the fused epilogue (read one item late)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            uint32_t cnt = 1;
            if (i == P_READY0 || i == P_READY1 || i == P_READY2) cnt = 512;
            if (i >= X_W0) cnt = 32;  // a warp waits for the warp that holds the same rows in the quarter to its right
            if (i == O_FREE) cnt = 512;
            if (i == WORK_EMPTY0 || i == WORK_EMPTY1) cnt = 514;  // MMA thread, V producer, 512 row threads
            mbar_init(&bars[i], cnt);
        }
        *abort_flag = (smem_u32(smem) & 1023u) ? 1u : 0u;  // the swizzled tiles need a 1024-byte aligned base
        fence_barrier_init();
    }
    if (warp == 17) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    if (warp == 16 && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int n_items = a.hdr->n_items;
    const int n_work = *abort_flag ? 0 : n_items * a.heads;

    if (warp == 16) {
        // ------------------------------------------------------------------ TMA producer: Q and K
        if (lane == 0) {
            uint32_t ph_qe = 1, ph_ke = 7;  // "empty" barriers start released; bit i of ph_ke: K stage i
            uint32_t st = 0;                // K stage of the next tile
            bool ok = true;
            SchedProducer sched;
            int w;
            Work wk;
            const auto fetch = [&](int w_) { return fetch_work(a, n_items, w_); };
            while (ok && (w = sched.next(a.sched + 0, n_work, ring, &bars[WORK_FULL0], &bars[WORK_EMPTY0], abort_flag, fetch, wk)) >= 0) {
                ok = mbar_wait_idle(&bars[Q_EMPTY], ph_qe, abort_flag);
                ph_qe ^= 1;
                if (!ok) break;
                mbar_expect_tx(&bars[Q_FULL], kTileBytes);
#pragma unroll
                for (int bx = 0; bx < kBoxes; ++bx)
                    tma_load_4d(sQ + bx * kBoxBytes, &map_q, &bars[Q_FULL], bx * 64, wk.start + wk.qt * kBM, wk.h, wk.b);
                for (int kt = wk.qt; kt >= 0; --kt) {
                    ok = mbar_wait_idle(&bars[K_EMPTY0 + st], (ph_ke >> st) & 1, abort_flag);
                    ph_ke ^= 1u << st;
                    if (!ok) break;
                    mbar_expect_tx(&bars[K_FULL0 + st], kTileBytes);
#pragma unroll
                    for (int bx = 0; bx < kBoxes; ++bx)
                        tma_load_4d(sK + st * kTileBytes + bx * kBoxBytes, &map_k, &bars[K_FULL0 + st], bx * 64,
                                    wk.start + kt * kBN, wk.h, wk.b);
                    st = st == kKStages - 1 ? 0 : st + 1;
                }
            }
        }
    } else if (warp == 18) {
        // ------------------------------------------------------------------ TMA producer: V
        if (lane == 0) {
            uint32_t ph_ve0 = 1, ph_ve1 = 1;
            uint32_t kv = 0;
            bool ok = true;
            SchedConsumer sched;
            int w;
            Work wk;
            while (ok && (w = sched.next(ring, &bars[WORK_FULL0], &bars[WORK_EMPTY0], abort_flag, wk)) >= 0) {
                for (int kt = wk.qt; kt >= 0; --kt, ++kv) {
                    const int st = kv & 1;
                    uint32_t& ph_ve = st ? ph_ve1 : ph_ve0;
                    ok = mbar_wait_idle(&bars[V_EMPTY0 + st], ph_ve, abort_flag);
                    ph_ve ^= 1;
                    if (!ok) break;
                    mbar_expect_tx(&bars[V_FULL0 + st], kTileBytes);
#pragma unroll
                    for (int bx = 0; bx < kBoxes; ++bx)
                        tma_load_4d(sV + st * kTileBytes + bx * kBoxBytes, &map_v, &bars[V_FULL0 + st], bx * 64,
                                    wk.start + kt * kBN, wk.h, wk.b);
                }
            }
        }
    } else if (warp == 17) {
        // ------------------------------------------------------------------ MMA issuer
        {
            const bool leader = elect_one();  // the whole warp runs the loops; one lane issues
            constexpr uint32_t idesc_s = make_idesc(kBM, kBN, kF16 ? 0 : 1, 0, 0);
            constexpr uint32_t idesc_o = make_idesc(kBM, D, kF16 ? 0 : 1, 0, 1);
            const SmemDesc desc_q = make_desc(smem_u32(sQ), 0, 1024);          // K-major operands of S
            const SmemDesc desc_k = make_desc(smem_u32(sK), 0, 1024);
            const SmemDesc desc_v = make_desc(smem_u32(sV), kBoxBytes, 1024);  // MN-major operand of P V
            uint32_t ph_qf = 0, ph_kf = 0, ph_vf0 = 0, ph_vf1 = 0, ph_of = 1;  // bit i of ph_kf: K stage i
            uint32_t ph_p = 0;   // bit i: parity of P_READY of S buffer i
            uint32_t sbuf = 0;   // running step count modulo 3 = S buffer of the next S to issue
            uint32_t pbuf = 0;   // S buffer of the next P to consume
            uint32_t ks = 0, vs = 0;  // K stage of the next S; running count of V tiles consumed by P V
            bool ok = true;
            // S of step j of the current item into the next S buffer of the rotation
            auto issue_s = [&](int j, int n) {
                const uint32_t st = ks;
                ks = ks == kKStages - 1 ? 0 : ks + 1;
                ok = mbar_wait(&bars[K_FULL0 + st], (ph_kf >> st) & 1, abort_flag);
                ph_kf ^= 1u << st;
                if (!ok) return;
                tc_fence_after();
                const SmemDesc dk = {desc_k.lo + st * (kTileBytes >> 4), desc_k.hi};
                const uint32_t d_s = tmem + kColS0 + 128 * sbuf;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t off = (k >> 2) * kBoxBytes + (k & 3) * 32;
                    if (k == 0) mma_ss<false>(leader, d_s, desc_q, off, dk, off, idesc_s);
                    else mma_ss<true>(leader, d_s, desc_q, off, dk, off, idesc_s);
                }
                mma_commit(leader, &bars[S_READY0 + sbuf]);
                sbuf = sbuf == 2 ? 0 : sbuf + 1;
                mma_commit(leader, &bars[K_EMPTY0 + st]);
                if (j == n - 1) mma_commit(leader, &bars[Q_EMPTY]);
            };
            SchedConsumer sched;
            int w;
            Work wk;
            while (ok && (w = sched.next(ring, &bars[WORK_FULL0], &bars[WORK_EMPTY0], abort_flag, wk, leader, true)) >= 0) {
                const int n = wk.qt + 1;
                ok = mbar_wait(&bars[Q_FULL], ph_qf, abort_flag);
                ph_qf ^= 1;
                if (!ok) break;
                issue_s(0, n);
                if (ok && n > 1) issue_s(1, n);
                if (ok && n > 2) issue_s(2, n);
                for (int j = 0; ok && j < n; ++j) {
                    const uint32_t b = pbuf;
                    pbuf = pbuf == 2 ? 0 : pbuf + 1;
                    ok = mbar_wait(&bars[P_READY0 + b], (ph_p >> b) & 1, abort_flag);
                    ph_p ^= 1u << b;
                    if (!ok) break;
                    const int st = vs & 1;
                    ++vs;
                    uint32_t& ph_vf = st ? ph_vf1 : ph_vf0;
                    ok = mbar_wait(&bars[V_FULL0 + st], ph_vf, abort_flag);
                    ph_vf ^= 1;
                    if (!ok) break;
                    int vrows = kBN;  // keys of the step's tile that belong to the sequence
                    if (j == 0) {  // the previous item's O must have been read out
                        ok = mbar_wait(&bars[O_FREE], ph_of, abort_flag);
                        ph_of ^= 1;
                        if (!ok) break;
                        // Diagonal tile at the ragged end of a sequence: the V rows behind the end belong to the next sequence
                        // or to nobody.  They meet P = 0 only, but a zero weight does not silence a NaN: the slices of 16
                        // keys that lie behind the end are not issued, and the rows between the end and the next multiple of
                        // 16 are set to zero.
                        vrows = wk.len - wk.qt * kBM;
                        if (vrows < kBN && (vrows & 15)) {
                            zero_rows_to_16(sV + st * kTileBytes, kBoxes, kBoxBytes, vrows, lane);
                            zero_rows_done();
                        }
                    }
                    tc_fence_after();
                    const SmemDesc dv = {desc_v.lo + st * (kTileBytes >> 4), desc_v.hi};
                    const uint32_t a_p = tmem + kColS0 + 128 * b + kColPOff;
#pragma unroll
                    for (int k = 0; k < kBN / 16; ++k) {
                        if (k == 0) mma_ts_dyn(leader, tmem + kColO, a_p, dv, 0, idesc_o, j > 0);
                        else if (16 * k < vrows) mma_ts<true>(leader, tmem + kColO, a_p + k * 8, dv, k * 2048, idesc_o);
                    }
                    mma_commit(leader, &bars[V_EMPTY0 + st]);
                    if (j + 3 < n) issue_s(j + 3, n);
                }
                if (!ok) break;
                mma_commit(leader, &bars[O_READY]);
            }
        }
    } else {
        // ------------------------------------------------------------------ row threads: warps 0-3 rightmost quarter ... 12-15 leftmost
        const int kq = 3 - (warp >> 2);        // 32-key quarter of every tile this thread owns
        const int r = (warp & 3) * 32 + lane;  // row of the tile == TMEM lane
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        uint32_t step = 0;   // key tiles of all items so far: tile number g uses S buffer g % 3 for the (g / 3)-th time
        const float scale = a.inv_temp * kLog2e;
        uint32_t ph_o = 0, items = 0;
        bool ok = true;
        // With kDefer a finished item's output leaves tensor memory one step late: its last contraction needs a while to
        // complete, and waiting for it at the end of the item idles the row threads.  They sweep the first tile of the
        // next item instead (whose scores exist already) and store the output then; the first P V contraction of the next
        // item waits for O_FREE, i.e. for this store.  It pays for short items only: for long ones the few registers that
        // carry the pending item through the loop cost more than the wait.
        struct PendingItem {
            int b, h, tok, item;
            bool row_ok;
        };
        PendingItem pend{};
        bool have_pend = false;
        const auto store_item = [&]() {  // each quarter stores 32 columns of the head dim of every row
            ok = mbar_wait(&bars[O_READY], ph_o, abort_flag);
            ph_o ^= 1;
            have_pend = false;
            if (!ok) return;
            tc_fence_after();
            if (kq < D / 32) {
                const int d0 = kq * 32;
                char* orow = a.o.ptr + 2 * ((int64_t)pend.b * a.o.sb + (int64_t)pend.h * a.o.sh + (int64_t)pend.tok * a.o.st + d0);
                uint32_t v[32];
                tmem_ld32(lane_base + kColO + d0, v);
                tmem_wait_ld(v);
                if (pend.row_ok && (D == 128 || a.head_dim > d0)) {  // D == 64 serves head dim 32 as well
                    if (kFused) {  // out = o + rem * v, rem rounded to the output type first
                        const float remf = round16<kF16>(wfin[(pend.item % 3) * 128 + r]);
                        float x[32];
                        load_row32<kF16>(a.v.ptr + 2 * ((int64_t)pend.b * a.v.sb + (int64_t)pend.h * a.v.sh +
                                                         (int64_t)pend.tok * a.v.st + d0), x);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(fmaf(remf, x[i], __uint_as_float(v[i])));
                    }
                    store_row32<kF16>(orow, v, 1.f);
                }
            }
            tc_fence_before();
            mbar_arrive(&bars[O_FREE]);
        };
        SchedConsumer sched;
        int w;
        Work wk;
        while (ok && (w = sched.next(ring, &bars[WORK_FULL0], &bars[WORK_EMPTY0], abort_flag, wk)) >= 0) {
            const int n = wk.qt + 1;
            const int qi = wk.qt * kBM + r;
            const bool row_ok = qi < wk.len;
            float* cw = a.carry_w ? a.carry_w + ((int64_t)wk.h * a.slot_cap) * kTileQ + r : nullptr;
            const int lim = a.attend_current ? r + 1 : r;  // diagonal tile: columns < lim are visible
            float W = 1.f;  // carry leaving the last quarter this thread swept
            for (int j = 0; j < n; ++j) {
                const int kt = wk.qt - j;
                const uint32_t g = step + j, sb = g % 3;
                const uint32_t s_base = lane_base + kColS0 + 128 * sb;
                ok = mbar_wait(&bars[S_READY0 + sb], (g / 3) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                // sweep the quarter right to left relative to an entering carry of 1
                uint32_t u[32], packed[16];
                float run[4], f[4];
                float Wl = 1.f;
                tmem_ld32(s_base + 32 * kq, u);
                tmem_wait_ld(u);
                if (j == 0) fwd_sweep<true>(u, scale, 32 * kq, lim, run);
                else fwd_sweep<false>(u, scale, 32 * kq, lim, run);
                fwd_carries(run, Wl, f);
                // The true entering carry travels along the row as a chain through shared memory: a thread takes it from
                // the quarter to its right (the rightmost quarter from the leftmost one of the previous tile), multiplies
                // by its own product and passes it on.  Nobody waits for a quarter to its left, so the quarters settle into
                // a stagger.  The chain also orders the accesses to the S buffer: P of a quarter overwrites scores of
                // quarters to its right only (kColPOff = 64), whose threads have loaded them before they passed the carry.
                float Win = 1.f;
                if (kq < 3) {
                    ok = mbar_wait(&bars[X_W0 + 8 * (kq + 1) + 4 * (g & 1) + (warp & 3)], (g >> 1) & 1, abort_flag);
                    if (!ok) break;
                    Win = xw[(kq + 1) * 128 + r];
                } else if (j > 0) {
                    ok = mbar_wait(&bars[X_W0 + 4 * ((g - 1) & 1) + (warp & 3)], ((g - 1) >> 1) & 1, abort_flag);
                    if (!ok) break;
                    Win = xw[r];
                }
                W = Win * Wl;
                xw[kq * 128 + r] = W;
                mbar_arrive(&bars[X_W0 + 8 * kq + 4 * (g & 1) + (warp & 3)]);
                if (kFused && kq == 0 && j + 1 == n) wfin[(items % 3) * 128 + r] = W;  // visible to all once O_READY has completed
                if (cw) cw[carry_slot32(wk.slot_base, wk.qt, 4 * kt + kq) * kTileQ] = Win;  // the carry at the quarter's right edge
                fwd_finish<kF16>(u, f, Win, packed);
                tmem_st16(s_base + kColPOff + 16 * kq, packed);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bars[P_READY0 + sb]);
                if (kDefer && j == 0 && have_pend) {
                    store_item();
                    if (!ok) break;
                }
            }
            if (!ok) break;
            step += n;
            pend = PendingItem{wk.b, wk.h, wk.start + qi, (int)items, row_ok};
            have_pend = true;
            if (!kDefer) {
                store_item();
                if (!ok) break;
            }
            ++items;
            if (row_ok && kq == 0) {  // this thread swept the leftmost quarter: W is the remainder of the row
                const int64_t t = wk.start + qi;
                char* rp = a.rem.ptr + 2 * ((int64_t)wk.b * a.rem.sb + (int64_t)wk.h * a.rem.sh + t * a.rem.st);
                if (kF16) *(__half*)rp = __float2half_rn(W);
                else *(__nv_bfloat16*)rp = __float2bfloat16_rn(W);
                ((float*)a.nla.ptr)[(int64_t)wk.b * a.nla.sb + (int64_t)wk.h * a.nla.sh + t * a.nla.st] = lg2_approx(W);
            }
        }
        if (kDefer && ok && have_pend) store_item();  // the block's last item
    }
    tc_teardown(abort_flag, a.status, tmem, kTmemCols, 17);
    sched_finish(a.sched + 0);
}

template <int D, bool kF16>
int launch_fwd_t(const SbParams& p, const KArgs& a, cudaStream_t st) {
    // D is the padded head dim (64 or 128); the tensor maps carry the true one, and TMA fills the columns beyond it with zeros
    CUtensorMap mq, mk, mv;
    const int kind = kF16 ? 2 : 0;
    const int64_t B = p.batch > 0 ? p.batch : 1;
    const int hd = p.head_dim;
    if (encode_tile_map(&mq, p.q.ptr, kind, hd, p.tokens, p.heads, B, p.q.stride_t, p.q.stride_h, p.q.stride_b, kBM) ||
        encode_tile_map(&mk, p.k.ptr, kind, hd, p.tokens, p.heads, B, p.k.stride_t, p.k.stride_h, p.k.stride_b, kBN) ||
        encode_tile_map(&mv, p.v.ptr, kind, hd, p.tokens, p.heads, B, p.v.stride_t, p.v.stride_h, p.v.stride_b, kBN))
        return kMapEncodeFailed;
    // Q + three K stages + two V stages; at least 120 KB so that one block owns the SM and its tensor memory
    constexpr int need = (1 + kKStages + kVStages) * kBM * D * 2 + 1024 + 5120;  // tiles, alignment, barriers and exchange slots
    constexpr int smem = need > 120 * 1024 ? need : 120 * 1024;
    const auto launch = [&](auto kernel) {
        const int e = ensure_kernel_attrs((const void*)kernel, smem, false);
        if (e != 0) return e;
        kernel<<<sm_count(), kFwdThreads, smem, st>>>(mq, mk, mv, a);
        count_launch();
        return (int)cudaGetLastError();
    };
    if (a.fused) return a.defer_fwd ? launch(tc_fwd_kernel<D, kF16, true, true>) : launch(tc_fwd_kernel<D, kF16, true, false>);
    return a.defer_fwd ? launch(tc_fwd_kernel<D, kF16, false, true>) : launch(tc_fwd_kernel<D, kF16, false, false>);
}

}  // namespace

bool tensor_path_eligible(const SbParams& p, bool backward, int* why) {
    *why = SBATTN_EUNSUPPORTED;
    if (p.dtype != SBATTN_BF16 && p.dtype != SBATTN_F16) return false;
    // head dim 32 runs on the 64-column kernels: TMA pads the tiles with zeros, the epilogues skip the second 32-column chunk
    if (p.head_dim != 32 && p.head_dim != 64 && p.head_dim != 128) return false;
    *why = SBATTN_EALIGN;
    const auto ok = [&](const SbMat& m) {
        // outer strides of at least a row: a broadcast head (stride 0) is not something a tensor map can describe
        return aligned_mat(m) && m.stride_t >= p.head_dim && (p.heads <= 1 || m.stride_h >= p.head_dim) &&
               (p.batch <= 1 || m.stride_b >= p.head_dim);
    };
    if (!ok(p.q) || !ok(p.k) || !ok(p.v)) return false;
    if (backward) {
        if (!ok(p.d_o) || !ok(p.dq) || !ok(p.dk) || !ok(p.dv)) return false;
    } else if (!ok(p.o)) {
        return false;
    }
    return true;
}

int launch_tensor_fwd(const SbParams& p, const WsLayout&, const KArgs& a, cudaStream_t st) {
    const bool f16 = p.dtype == SBATTN_F16;
    if (p.head_dim > 64) return f16 ? launch_fwd_t<128, true>(p, a, st) : launch_fwd_t<128, false>(p, a, st);
    return f16 ? launch_fwd_t<64, true>(p, a, st) : launch_fwd_t<64, false>(p, a, st);
}

}  // namespace sb
