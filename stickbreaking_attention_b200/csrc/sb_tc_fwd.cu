// Tensor-core forward (sm_100a): o, rem, neg_log_acc and the per-64-key carries of W for bf16 / f16 inputs with
// head_dim 64 or 128.
//
// One work item = (head, sequence, 128-row query tile).  A persistent grid of 2 thread blocks per SM walks the
// item table built by the prep kernel (heaviest items first, round-robin over the blocks).  Per item the key tiles
// are visited right to left, from the diagonal to key 0 -- the order of the reference's _forward_one_row
// (stickbreaking_attention/sb_varlen/sb_varlen_fwd.py:155-193) -- because the weight of key j needs the product of
// (1 - beta) over the keys to its right.
//
// Roles inside a block (192 threads):
//   warps 0-3  one thread per query row: reads the 128 scores of its row from tensor memory, turns them into
//              attention weights in fp32 registers (beta = sigmoid(s), running product W of 1 - beta, p = beta * W),
//              writes them back to tensor memory as 16-bit operands; epilogue: o, rem, neg_log_acc to global memory.
//   warp 4     TMA producer: Q once per item, then K and V tiles (single stage each; K of tile t+1 arrives while
//              the weights of tile t are computed, V of tile t+1 while S of t+1 is computed).
//   warp 5     issues tcgen05.mma: S = Q K^T (both operands in shared memory) into TMEM columns [0,128),
//              O += P V (P from TMEM columns [64,128), V from shared memory) into columns [128,128+D).
// P overwrites the right half of S: a row is processed right to left in chunks of 32 columns and the packed
// weights of chunk c land in columns that were already read.
#include "sb_tc_common.cuh"

namespace sb {

using namespace sm100;

namespace {

constexpr int kFwdThreads = 192;
constexpr int kBM = 128, kBN = 128;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColP = 64, kColO = 128;
enum FwdBar { Q_FULL, Q_EMPTY, K_FULL, K_EMPTY, V_FULL, V_EMPTY, S_READY, P_READY, O_READY, O_FREE, WORK_FULL0, WORK_FULL1,
              WORK_EMPTY0, WORK_EMPTY1, kNumBars };

// Attention weights of 32 consecutive keys of one query row, right to left, in groups of 8 keys.
// With e = exp(s) and d = 1 + e:  beta = e / d,  1 - beta = 1 / d,  so for key m of a group entered with the carry W
// (product of 1 - beta over everything to its right)
//     p_m = beta_m * W * prod_{m' > m in group} 1/d_m'  =  e_m * (prod_{m' < m in group} d_m') * W / (prod over the group of d)
// which needs one reciprocal per GROUP instead of one per key.  Scores are clamped at 2^15 (beta = 1 - 3e-5 there)
// so that the product of 8 factors stays below 2^127.  Masked keys get e = 0: weight 0 and no stick broken.
template <bool kMasked, bool kF16>
__device__ __forceinline__ void fwd_chunk(uint32_t (&s)[32], float scale, int col0, int lim, float& W, uint32_t (&packed)[16]) {
#pragma unroll
    for (int g = 3; g >= 0; --g) {
        float e[8], pre[8];
        float run = 1.f;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            float x = fminf(__uint_as_float(s[g * 8 + m]) * scale, 15.f);
            e[m] = ex2_approx(x);
            if (kMasked && col0 + g * 8 + m >= lim) e[m] = 0.f;
            pre[m] = run;
            run = fmaf(run, e[m], run);
        }
        const float f = W * rcp_approx(run);
#pragma unroll
        for (int m = 0; m < 8; ++m) s[g * 8 + m] = __float_as_uint(e[m] * pre[m] * f);
        W = f;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) packed[j] = pack16<kF16>(__uint_as_float(s[2 * j]), __uint_as_float(s[2 * j + 1]));
}

template <int D, bool kF16>
__global__ void __launch_bounds__(kFwdThreads, 2)
tc_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const KArgs a) {
    constexpr int kTileBytes = kBM * D * 2;
    constexpr int kBoxBytes = 128 * 128;  // one TMA box: 128 rows of 64 elements
    constexpr int kBoxes = D / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + kTileBytes;
    uint8_t* sV = sK + kTileBytes;
    uint64_t* bars = (uint64_t*)(sV + kTileBytes);
    uint32_t* tmem_slot = (uint32_t*)(bars + kNumBars);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    SchedRing* ring = (SchedRing*)(tmem_slot + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(&bars[Q_FULL], 1);
        mbar_init(&bars[Q_EMPTY], 1);
        mbar_init(&bars[K_FULL], 1);
        mbar_init(&bars[K_EMPTY], 1);
        mbar_init(&bars[V_FULL], 1);
        mbar_init(&bars[V_EMPTY], 1);
        mbar_init(&bars[S_READY], 1);
        mbar_init(&bars[P_READY], 128);
        mbar_init(&bars[O_READY], 1);
        mbar_init(&bars[O_FREE], 128);
        mbar_init(&bars[WORK_FULL0], 1);
        mbar_init(&bars[WORK_FULL1], 1);
        mbar_init(&bars[WORK_EMPTY0], kRingConsumers);
        mbar_init(&bars[WORK_EMPTY1], kRingConsumers);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int n_items = a.hdr->n_items;
    const int n_work = n_items * a.heads;

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t ph_qe = 1, ph_ke = 1, ph_ve = 1;  // "empty" barriers start released
            bool ok = true;
            SchedProducer sched;
            int w;
            while (ok && (w = sched.next(a.sched + 0, n_work, ring, &bars[WORK_FULL0], &bars[WORK_EMPTY0], abort_flag)) >= 0) {
                const Work wk = fetch_work(a, n_items, w);
                ok = mbar_wait(&bars[Q_EMPTY], ph_qe, abort_flag);
                ph_qe ^= 1;
                if (!ok) break;
                mbar_expect_tx(&bars[Q_FULL], kTileBytes);
#pragma unroll
                for (int bx = 0; bx < kBoxes; ++bx)
                    tma_load_4d(sQ + bx * kBoxBytes, &map_q, &bars[Q_FULL], bx * 64, wk.start + wk.qt * kBM, wk.h, wk.b);
                for (int kt = wk.qt; kt >= 0; --kt) {
                    const int row = wk.start + kt * kBN;
                    ok = mbar_wait(&bars[K_EMPTY], ph_ke, abort_flag);
                    ph_ke ^= 1;
                    if (!ok) break;
                    mbar_expect_tx(&bars[K_FULL], kTileBytes);
#pragma unroll
                    for (int bx = 0; bx < kBoxes; ++bx)
                        tma_load_4d(sK + bx * kBoxBytes, &map_k, &bars[K_FULL], bx * 64, row, wk.h, wk.b);
                    ok = mbar_wait(&bars[V_EMPTY], ph_ve, abort_flag);
                    ph_ve ^= 1;
                    if (!ok) break;
                    mbar_expect_tx(&bars[V_FULL], kTileBytes);
#pragma unroll
                    for (int bx = 0; bx < kBoxes; ++bx)
                        tma_load_4d(sV + bx * kBoxBytes, &map_v, &bars[V_FULL], bx * 64, row, wk.h, wk.b);
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(kBM, kBN, kF16 ? 0 : 1, 0, 0);
            constexpr uint32_t idesc_o = make_idesc(kBM, D, kF16 ? 0 : 1, 0, 1);
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            uint32_t ph_qf = 0, ph_kf = 0, ph_vf = 0, ph_p = 0, ph_of = 1;
            bool ok = true;
            auto issue_s = [&](bool last_of_item) {
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t off = (k >> 2) * kBoxBytes + (k & 3) * 32;
                    mma_ss(tmem + kColS, make_smem_desc(q_addr + off, 0, 1024), make_smem_desc(k_addr + off, 0, 1024),
                           idesc_s, k > 0);
                }
                mma_commit(&bars[S_READY]);
                mma_commit(&bars[K_EMPTY]);
                if (last_of_item) mma_commit(&bars[Q_EMPTY]);
            };
            SchedConsumer sched;
            int w;
            while (ok && (w = sched.next(ring, &bars[WORK_FULL0], &bars[WORK_EMPTY0], abort_flag)) >= 0) {
                const Work wk = fetch_work(a, n_items, w);
                const int n_kt = wk.qt + 1;
                ok = mbar_wait(&bars[Q_FULL], ph_qf, abort_flag);
                ph_qf ^= 1;
                if (!ok) break;
                ok = mbar_wait(&bars[K_FULL], ph_kf, abort_flag);
                ph_kf ^= 1;
                if (!ok) break;
                issue_s(n_kt == 1);
                for (int t = 0; t < n_kt; ++t) {
                    ok = mbar_wait(&bars[P_READY], ph_p, abort_flag);
                    ph_p ^= 1;
                    if (!ok) break;
                    ok = mbar_wait(&bars[V_FULL], ph_vf, abort_flag);
                    ph_vf ^= 1;
                    if (!ok) break;
                    if (t == 0) {  // the previous item's O must have been read out
                        ok = mbar_wait(&bars[O_FREE], ph_of, abort_flag);
                        ph_of ^= 1;
                        if (!ok) break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < kBN / 16; ++k)
                        mma_ts(tmem + kColO, tmem + kColP + k * 8, make_smem_desc(v_addr + k * 2048, kBoxBytes, 1024),
                               idesc_o, (t > 0 || k > 0) ? 1u : 0u);
                    mma_commit(&bars[V_EMPTY]);
                    if (t + 1 < n_kt) {
                        ok = mbar_wait(&bars[K_FULL], ph_kf, abort_flag);
                        ph_kf ^= 1;
                        if (!ok) break;
                        issue_s(t + 2 == n_kt);
                    } else {
                        mma_commit(&bars[O_READY]);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ one thread per query row
        const int r = tid;  // row of the tile == TMEM lane
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        const float scale = a.inv_temp * kLog2e;
        uint32_t ph_s = 0, ph_o = 0;
        bool ok = true;
        SchedConsumer sched;
        int w;
        while (ok && (w = sched.next(ring, &bars[WORK_FULL0], &bars[WORK_EMPTY0], abort_flag)) >= 0) {
            const Work wk = fetch_work(a, n_items, w);
            const int qi = wk.qt * kBM + r;
            const bool row_ok = qi < wk.len;
            float* cw = a.carry_w ? a.carry_w + ((int64_t)wk.h * a.slot_cap) * kTileQ + r : nullptr;
            float W = 1.f;
            for (int kt = wk.qt; kt >= 0; --kt) {
                ok = mbar_wait(&bars[S_READY], ph_s, abort_flag);
                ph_s ^= 1;
                if (!ok) break;
                tc_fence_after();
                const bool diag = kt == wk.qt;
                // keys of the diagonal tile visible from row r: columns < lim
                const int lim = a.attend_current ? r + 1 : r;
                // chunks of 32 columns, right to left; the load of the next chunk is in flight while one is computed
                uint32_t sa[32], sb[32], packed[16];
                tmem_ld32(lane_base + kColS + 96, sa);
                tmem_wait_ld();
                tmem_ld32(lane_base + kColS + 64, sb);
                if (cw) cw[carry_slot(wk.slot_base, wk.qt, 2 * kt + 1) * kTileQ] = W;
                if (diag) fwd_chunk<true, kF16>(sa, scale, 96, lim, W, packed);
                else fwd_chunk<false, kF16>(sa, scale, 96, lim, W, packed);
                tmem_st16(lane_base + kColP + 48, packed);
                tmem_wait_ld();
                tmem_ld32(lane_base + kColS + 32, sa);
                if (diag) fwd_chunk<true, kF16>(sb, scale, 64, lim, W, packed);
                else fwd_chunk<false, kF16>(sb, scale, 64, lim, W, packed);
                tmem_st16(lane_base + kColP + 32, packed);
                tmem_wait_ld();
                tmem_ld32(lane_base + kColS + 0, sb);
                if (cw) cw[carry_slot(wk.slot_base, wk.qt, 2 * kt) * kTileQ] = W;
                if (diag) fwd_chunk<true, kF16>(sa, scale, 32, lim, W, packed);
                else fwd_chunk<false, kF16>(sa, scale, 32, lim, W, packed);
                tmem_st16(lane_base + kColP + 16, packed);
                tmem_wait_ld();
                if (diag) fwd_chunk<true, kF16>(sb, scale, 0, lim, W, packed);
                else fwd_chunk<false, kF16>(sb, scale, 0, lim, W, packed);
                tmem_st16(lane_base + kColP + 0, packed);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bars[P_READY]);
            }
            if (!ok) break;
            // epilogue
            ok = mbar_wait(&bars[O_READY], ph_o, abort_flag);
            ph_o ^= 1;
            if (!ok) break;
            tc_fence_after();
            char* orow = a.o.ptr + 2 * ((int64_t)wk.b * a.o.sb + (int64_t)wk.h * a.o.sh + (int64_t)(wk.start + qi) * a.o.st);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(lane_base + kColO + c * 32, v);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 u;
                        uint32_t* up = (uint32_t*)&u;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            up[j] = pack16<kF16>(__uint_as_float(v[g * 8 + 2 * j]), __uint_as_float(v[g * 8 + 2 * j + 1]));
                        *(uint4*)(orow + (c * 32 + g * 8) * 2) = u;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&bars[O_FREE]);
            if (row_ok) {
                const int64_t t = wk.start + qi;
                char* rp = a.rem.ptr + 2 * ((int64_t)wk.b * a.rem.sb + (int64_t)wk.h * a.rem.sh + t * a.rem.st);
                if (kF16) *(__half*)rp = __float2half_rn(W);
                else *(__nv_bfloat16*)rp = __float2bfloat16_rn(W);
                ((float*)a.nla.ptr)[(int64_t)wk.b * a.nla.sb + (int64_t)wk.h * a.nla.sh + t * a.nla.st] = lg2_approx(W);
            }
        }
    }
    tc_teardown(abort_flag, a.status, tmem, kTmemCols, 5);
    sched_finish(a.sched + 0);
}

template <int D, bool kF16>
int launch_fwd_t(const SbParams& p, const KArgs& a, cudaStream_t st) {
    CUtensorMap mq, mk, mv;
    const int kind = kF16 ? 2 : 0;
    const int64_t B = p.batch > 0 ? p.batch : 1;
    if (encode_tile_map(&mq, p.q.ptr, kind, D, p.tokens, p.heads, B, p.q.stride_t, p.q.stride_h, p.q.stride_b, kBM) ||
        encode_tile_map(&mk, p.k.ptr, kind, D, p.tokens, p.heads, B, p.k.stride_t, p.k.stride_h, p.k.stride_b, kBN) ||
        encode_tile_map(&mv, p.v.ptr, kind, D, p.tokens, p.heads, B, p.v.stride_t, p.v.stride_h, p.v.stride_b, kBN))
        return 1;
    // at least 80 KB so that never more than two blocks (2 x 256 TMEM columns) share an SM
    constexpr int smem = (3 * kBM * D * 2 + 1024 + 512) > 81920 ? (3 * kBM * D * 2 + 1024 + 512) : 81920;
    cudaError_t e = cudaFuncSetAttribute(tc_fwd_kernel<D, kF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(tc_fwd_kernel<D, kF16>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    tc_fwd_kernel<D, kF16><<<2 * sm_count(), kFwdThreads, smem, st>>>(mq, mk, mv, a);
    return (int)cudaGetLastError();
}

}  // namespace

bool tensor_path_eligible(const SbParams& p, bool backward, int* why) {
    *why = SBATTN_EUNSUPPORTED;
    if (p.dtype != SBATTN_BF16 && p.dtype != SBATTN_F16) return false;
    if (p.head_dim != 64 && p.head_dim != 128) return false;
    *why = SBATTN_EALIGN;
    if (!aligned_mat(p.q) || !aligned_mat(p.k) || !aligned_mat(p.v)) return false;
    if (backward) {
        if (!aligned_mat(p.d_o) || !aligned_mat(p.dq) || !aligned_mat(p.dk) || !aligned_mat(p.dv)) return false;
        if (p.d_o.stride_t < p.head_dim) return false;
    } else if (!aligned_mat(p.o)) {
        return false;
    }
    if (p.q.stride_t < p.head_dim || p.k.stride_t < p.head_dim || p.v.stride_t < p.head_dim) return false;
    return true;
}

int launch_tensor_fwd(const SbParams& p, const WsLayout&, const KArgs& a, cudaStream_t st) {
    const bool f16 = p.dtype == SBATTN_F16;
    if (p.head_dim == 128) return f16 ? launch_fwd_t<128, true>(p, a, st) : launch_fwd_t<128, false>(p, a, st);
    return f16 ? launch_fwd_t<64, true>(p, a, st) : launch_fwd_t<64, false>(p, a, st);
}

int launch_tensor_bwd(const SbParams& p, const WsLayout&, const KArgs& a, cudaStream_t st) {
    return launch_tensor_bwd_impl(p, a, st);
}

}  // namespace sb
