// fp32-arithmetic kernels (no tensor cores): forward, backward-dq and backward-dk/dv.
//
// They serve float32 inputs (where products must not be rounded to bf16/tf32), head dims other than 32, 64 and
// 128, and tensors whose strides the TMA path cannot take.  Structure mirrors the tensor-core kernels:
//   * forward walks the key tiles of one 64-row query block right to left and carries, per row, the running
//     product W = prod(1 - beta) of everything to the right (the reference carries its log,
//     stickbreaking_attention/sb_varlen/sb_varlen_fwd.py:53-66,155-193);
//   * the value of W at every 64-key boundary is saved ("carry_w") so that the backward can enter any tile
//     directly instead of subtracting from the row total as the reference does (sb_varlen_bwd.py:396-445);
//   * backward-dq walks left to right carrying the prefix sum of g = A * dA (sb_varlen_bwd.py:438-449) and saves
//     it at every boundary ("carry_c");
//   * backward-dk/dv keeps one 64-key tile stationary and walks the query blocks below it, entering each
//     tile with the two saved carries; dk and dv are accumulated in registers and stored once, so there is no
//     atomic or lock on the data (the reference uses a spin lock per key tile, sb_varlen_bwd.py:11-53).
#include "sb_common.cuh"

namespace sb {

namespace {

constexpr int kBM = 64;         // query rows per block
constexpr int kBN = 64;         // keys per tile
constexpr int kThreads = 256;   // 16 x 16 thread grid, 4 x 4 outputs each
constexpr int kSP = kBN + 1;    // padded row length of the score tiles

template <typename T>
__device__ inline void load_rows(float* dst, int DP, int D, const MatView& m, int b, int h, int row0, int rows_valid) {
    const T* base = (const T*)m.ptr + (int64_t)b * m.sb + (int64_t)h * m.sh;
    for (int idx = threadIdx.x; idx < kBM * D; idx += kThreads) {
        const int r = idx / D, d = idx - r * D;
        float x = 0.f;
        if (r < rows_valid) x = to_f32<T>(base[(int64_t)(row0 + r) * m.st + d]);
        dst[r * DP + d] = x;
    }
}

// C[64x64] = A[64xD] * B[64xD]^T ; thread (ty,tx) owns rows ty+16r, cols tx+16c
__device__ inline void gemm_nt(float* C, const float* A, const float* B, int DP, int D) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    for (int d = 0; d < D; ++d) {
        float a[4], bb[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) a[r] = A[(ty + 16 * r) * DP + d];
#pragma unroll
        for (int c = 0; c < 4; ++c) bb[c] = B[(tx + 16 * c) * DP + d];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(a[r], bb[c], acc[r][c]);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) C[(ty + 16 * r) * kSP + tx + 16 * c] = acc[r][c];
}

// acc[64 x D] += P[64 x 64] * V[64 x D] ; thread owns rows ty+16r, cols tx+16c (c < 8)
__device__ inline void gemm_pv(float (&acc)[4][8], const float* P, const float* V, int DP, int D) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int nc = (D + 15) >> 4;
    for (int j = 0; j < kBN; ++j) {
        float p[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) p[r] = P[(ty + 16 * r) * kSP + j];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (c < nc) {
                const float vv = V[j * DP + tx + 16 * c];  // columns beyond D read the zero padding
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[r][c] = fmaf(p[r], vv, acc[r][c]);
            }
        }
    }
}

// acc[64 keys x D] += P[64 q x 64 keys]^T * X[64 q x D]
__device__ inline void gemm_ptx(float (&acc)[4][8], const float* P, const float* X, int DP, int D) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int nc = (D + 15) >> 4;
    for (int i = 0; i < kBM; ++i) {
        float p[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) p[r] = P[i * kSP + ty + 16 * r];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (c < nc) {
                const float xv = X[i * DP + tx + 16 * c];
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[r][c] = fmaf(p[r], xv, acc[r][c]);
            }
        }
    }
}

template <typename T>
__device__ inline void store_acc(const float (&acc)[4][8], float scale, const MatView& m, int b, int h, int row0,
                                 int rows_valid, int D) {
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    T* base = (T*)m.ptr + (int64_t)b * m.sb + (int64_t)h * m.sh;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int row = ty + 16 * r;
        if (row >= rows_valid) continue;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int d = tx + 16 * c;
            if (d < D) base[(int64_t)(row0 + row) * m.st + d] = from_f32<T>(acc[r][c] * scale);
        }
    }
}

// sigmoid pieces with full relative accuracy on both sides: beta = sigmoid(s), r = 1 - beta
__device__ inline void sigmoid_pair(float s, float& beta, float& r) {
    const float e = expf(-fabsf(s));
    const float inv = 1.0f / (1.0f + e);
    const float big = inv, small = e * inv;
    beta = s >= 0.f ? big : small;
    r = s >= 0.f ? small : big;
}

// The 4 threads of a row (consecutive lanes) each own 16 consecutive keys of the 64-key tile.
struct RowPart {
    int row, part, lane_base;
};
__device__ inline RowPart row_part() {
    RowPart rp;
    rp.row = threadIdx.x >> 2;
    rp.part = threadIdx.x & 3;
    rp.lane_base = (threadIdx.x & 31) & ~3;
    return rp;
}
// product / sum over the 4 threads of a row, identical bits on all of them
__device__ inline float quad_prod(float x) {
    x *= __shfl_xor_sync(0xffffffffu, x, 1);
    x *= __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
}
__device__ inline float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
}
// product (sum) of the values held by the parts to the right (left) of this one
__device__ inline float quad_right_prod(float x, int part) {
    const float a = __shfl_down_sync(0xffffffffu, x, 1);
    const float b = __shfl_down_sync(0xffffffffu, x, 2);
    const float c = __shfl_down_sync(0xffffffffu, x, 3);
    return (part < 3 ? a : 1.f) * (part < 2 ? b : 1.f) * (part < 1 ? c : 1.f);
}
__device__ inline float quad_right_sum(float x, int part) {
    const float a = __shfl_down_sync(0xffffffffu, x, 1);
    const float b = __shfl_down_sync(0xffffffffu, x, 2);
    const float c = __shfl_down_sync(0xffffffffu, x, 3);
    return (part < 3 ? a : 0.f) + (part < 2 ? b : 0.f) + (part < 1 ? c : 0.f);
}
__device__ inline float quad_left_sum(float x, int part) {
    const float a = __shfl_up_sync(0xffffffffu, x, 1);
    const float b = __shfl_up_sync(0xffffffffu, x, 2);
    const float c = __shfl_up_sync(0xffffffffu, x, 3);
    return (part > 0 ? a : 0.f) + (part > 1 ? b : 0.f) + (part > 2 ? c : 0.f);
}

// key j (index inside the sequence) visible from query i?
__device__ inline bool visible(int i, int j, int len, int attend_current) {
    return j < len && (attend_current ? j <= i : j < i);
}

struct ItemCtx {
    int seq, qt, b, start, len, slot_base;
};
__device__ inline bool fetch_item(const KArgs& a, int item, ItemCtx& c) {
    if (item >= a.hdr->n_items) return false;
    const int2 it = a.items[item];
    const SeqInfo s = a.seqs[it.x];
    c.seq = it.x; c.qt = it.y; c.b = s.batch; c.start = s.start; c.len = s.len; c.slot_base = s.slot_base;
    return true;
}

// ------------------------------------------------------------------------------------------ forward
template <typename T>
__global__ void __launch_bounds__(kThreads, 1) simt_fwd_kernel(const KArgs a) {
    extern __shared__ float smem[];
    ItemCtx c;
    if (!fetch_item(a, blockIdx.x, c)) return;
    const int h = blockIdx.y;
    const int qb = 2 * c.qt + blockIdx.z;  // 64-row block inside the sequence
    const int row0 = qb * kBM;
    if (row0 >= c.len) return;
    // row pitch: odd (no bank conflicts) and with zero padding so that column reads up to 16*ceil(D/16) stay inside
    const int D = a.head_dim, DPP = (D | 1) + 16;
    float* Qs = smem;
    float* Ks = Qs + kBM * DPP;
    float* Vs = Ks + kBN * DPP;
    float* Ss = Vs + kBN * DPP;
    for (int idx = threadIdx.x; idx < 3 * kBM * DPP; idx += kThreads) smem[idx] = 0.f;
    __syncthreads();
    const int rows_valid = min(kBM, c.len - row0);
    load_rows<T>(Qs, DPP, D, a.q, c.b, h, c.start + row0, rows_valid);

    const RowPart rp = row_part();
    const int qi = row0 + rp.row;
    float W = 1.f;
    float acc[4][8] = {};
    float* cw = a.carry_w ? a.carry_w + ((int64_t)h * a.slot_cap) * kTileQ : nullptr;
    const int rloc = (qb & 1) * kBM + rp.row;  // row inside the 128-row tile

    for (int kh = qb; kh >= 0; --kh) {
        const int key0 = kh * kBN;
        const int keys_valid = min(kBN, c.len - key0);
        __syncthreads();
        load_rows<T>(Ks, DPP, D, a.k, c.b, h, c.start + key0, keys_valid);
        load_rows<T>(Vs, DPP, D, a.v, c.b, h, c.start + key0, keys_valid);
        __syncthreads();
        gemm_nt(Ss, Qs, Ks, DPP, D);
        __syncthreads();
        // element-wise part: 4 threads per row, 16 keys each
        if (cw && rp.part == 0) cw[carry_slot(c.slot_base, c.qt, kh) * kTileQ + rloc] = W;  // right edge of the half
        float beta[16], r[16];
        float prod = 1.f;
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
            const int j = rp.part * 16 + jj;
            const float s = Ss[rp.row * kSP + j] * a.inv_temp;
            float bt, rr;
            sigmoid_pair(s, bt, rr);
            const bool vis = visible(qi, key0 + j, c.len, a.attend_current);
            beta[jj] = vis ? bt : 0.f;
            r[jj] = vis ? rr : 1.f;
            prod *= r[jj];
        }
        const float win = W * quad_right_prod(prod, rp.part);
        // the carry in the middle of the half as well: a tensor-core backward may follow this forward (the two are
        // chosen independently, by the alignment of their own operands), and it enters every 32-key quarter directly
        if (cw && rp.part == 1) cw[carry_slot32(c.slot_base, c.qt, 2 * kh) * kTileQ + rloc] = win;
        float run = win;
#pragma unroll
        for (int jj = 15; jj >= 0; --jj) {
            Ss[rp.row * kSP + rp.part * 16 + jj] = beta[jj] * run;
            run *= r[jj];
        }
        W *= quad_prod(prod);
        __syncthreads();
        gemm_pv(acc, Ss, Vs, DPP, D);
    }
    store_acc<T>(acc, 1.f, a.o, c.b, h, c.start + row0, rows_valid, D);
    if (rp.part == 0 && rp.row < rows_valid) {
        const int64_t t = c.start + qi;
        ((T*)a.rem.ptr)[(int64_t)c.b * a.rem.sb + (int64_t)h * a.rem.sh + t * a.rem.st] = from_f32<T>(W);
        ((float*)a.nla.ptr)[(int64_t)c.b * a.nla.sb + (int64_t)h * a.nla.sh + t * a.nla.st] = log2f(W);
    }
}

// ------------------------------------------------------------------------------------------ backward: dq
template <typename T>
__global__ void __launch_bounds__(kThreads, 1) simt_bwd_dq_kernel(const KArgs a) {
    extern __shared__ float smem[];
    ItemCtx c;
    if (!fetch_item(a, blockIdx.x, c)) return;
    const int h = blockIdx.y;
    const int qb = 2 * c.qt + blockIdx.z;
    const int row0 = qb * kBM;
    if (row0 >= c.len) return;
    const int D = a.head_dim, DPP = (D | 1) + 16;
    float* Qs = smem;
    float* Gs = Qs + kBM * DPP;  // dO
    float* Ks = Gs + kBM * DPP;
    float* Vs = Ks + kBN * DPP;
    float* Ss = Vs + kBN * DPP;
    float* Ps = Ss + kBM * kSP;
    for (int idx = threadIdx.x; idx < 4 * kBM * DPP; idx += kThreads) smem[idx] = 0.f;
    __syncthreads();
    const int rows_valid = min(kBM, c.len - row0);
    load_rows<T>(Qs, DPP, D, a.q, c.b, h, c.start + row0, rows_valid);
    load_rows<T>(Gs, DPP, D, a.d_o, c.b, h, c.start + row0, rows_valid);

    const RowPart rp = row_part();
    const int qi = row0 + rp.row;
    const bool row_ok = rp.row < rows_valid;
    float drem = 0.f;
    if (row_ok)
        drem = to_f32<T>(((const T*)a.d_rem.ptr)[(int64_t)c.b * a.d_rem.sb + (int64_t)h * a.d_rem.sh +
                                                 (int64_t)(c.start + qi) * a.d_rem.st]);
    const float* cw = a.carry_w + ((int64_t)h * a.slot_cap) * kTileQ;
    float* cc = a.carry_c + ((int64_t)h * a.slot_cap) * kTileQ;
    const int rloc = (qb & 1) * kBM + rp.row;
    float cprefix = 0.f;  // sum of g over all keys left of the current tile
    float acc[4][8] = {};

    for (int kh = 0; kh <= qb; ++kh) {
        const int key0 = kh * kBN;
        const int keys_valid = min(kBN, c.len - key0);
        __syncthreads();
        load_rows<T>(Ks, DPP, D, a.k, c.b, h, c.start + key0, keys_valid);
        load_rows<T>(Vs, DPP, D, a.v, c.b, h, c.start + key0, keys_valid);
        __syncthreads();
        gemm_nt(Ss, Qs, Ks, DPP, D);
        gemm_nt(Ps, Gs, Vs, DPP, D);
        __syncthreads();
        const int64_t slot = carry_slot(c.slot_base, c.qt, kh) * kTileQ + rloc;
        const float W = row_ok ? cw[slot] : 0.f;
        float beta[16], g[16];
        float prod = 1.f;
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
            const int j = rp.part * 16 + jj;
            float bt, rr;
            sigmoid_pair(Ss[rp.row * kSP + j] * a.inv_temp, bt, rr);
            const bool vis = row_ok && visible(qi, key0 + j, c.len, a.attend_current);
            beta[jj] = vis ? bt : 0.f;
            g[jj] = vis ? rr : 1.f;  // holds r until the suffix pass below
            prod *= g[jj];
        }
        float run = W * quad_right_prod(prod, rp.part);
        float gsum = 0.f;
#pragma unroll
        for (int jj = 15; jj >= 0; --jj) {
            const float rr = g[jj];
            const float p = beta[jj] * run;
            g[jj] = p * (Ps[rp.row * kSP + rp.part * 16 + jj] - drem);
            gsum += g[jj];
            run *= rr;
        }
        float cin = cprefix + quad_left_sum(gsum, rp.part);
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
            cin += g[jj];
            Ss[rp.row * kSP + rp.part * 16 + jj] = g[jj] - beta[jj] * cin;
        }
        cprefix += quad_sum(gsum);
        if (rp.part == 0 && row_ok) cc[slot] = cprefix;  // prefix including this tile
        __syncthreads();
        gemm_pv(acc, Ss, Ks, DPP, D);
    }
    store_acc<T>(acc, a.inv_temp, a.dq, c.b, h, c.start + row0, rows_valid, D);
}

// ------------------------------------------------------------------------------------------ backward: dk, dv
template <typename T>
__global__ void __launch_bounds__(kThreads, 1) simt_bwd_dkdv_kernel(const KArgs a) {
    extern __shared__ float smem[];
    ItemCtx c;
    const int n_items = a.hdr->n_items;
    if ((int)blockIdx.x >= n_items) return;
    // the table is heaviest-first for query tiles; key tiles are heaviest at the other end
    if (!fetch_item(a, n_items - 1 - (int)blockIdx.x, c)) return;
    const int h = blockIdx.y;
    const int kh = 2 * c.qt + blockIdx.z;
    const int key0 = kh * kBN;
    if (key0 >= c.len) return;
    const int D = a.head_dim, DPP = (D | 1) + 16;
    float* Qs = smem;
    float* Gs = Qs + kBM * DPP;
    float* Ks = Gs + kBM * DPP;
    float* Vs = Ks + kBN * DPP;
    float* Ss = Vs + kBN * DPP;
    float* Ps = Ss + kBM * kSP;
    for (int idx = threadIdx.x; idx < 4 * kBM * DPP; idx += kThreads) smem[idx] = 0.f;
    __syncthreads();
    const int keys_valid = min(kBN, c.len - key0);
    load_rows<T>(Ks, DPP, D, a.k, c.b, h, c.start + key0, keys_valid);
    load_rows<T>(Vs, DPP, D, a.v, c.b, h, c.start + key0, keys_valid);

    const RowPart rp = row_part();
    const float* cw = a.carry_w + ((int64_t)h * a.slot_cap) * kTileQ;
    const float* cc = a.carry_c + ((int64_t)h * a.slot_cap) * kTileQ;
    float acc_k[4][8] = {}, acc_v[4][8] = {};
    const int n_qb = (c.len + kBM - 1) / kBM;

    for (int qb = kh; qb < n_qb; ++qb) {
        const int row0 = qb * kBM;
        const int rows_valid = min(kBM, c.len - row0);
        __syncthreads();
        load_rows<T>(Qs, DPP, D, a.q, c.b, h, c.start + row0, rows_valid);
        load_rows<T>(Gs, DPP, D, a.d_o, c.b, h, c.start + row0, rows_valid);
        __syncthreads();
        gemm_nt(Ss, Qs, Ks, DPP, D);
        gemm_nt(Ps, Gs, Vs, DPP, D);
        __syncthreads();
        const int qi = row0 + rp.row;
        const bool row_ok = rp.row < rows_valid;
        float drem = 0.f, W = 0.f, cright = 0.f;
        if (row_ok) {
            drem = to_f32<T>(((const T*)a.d_rem.ptr)[(int64_t)c.b * a.d_rem.sb + (int64_t)h * a.d_rem.sh +
                                                     (int64_t)(c.start + qi) * a.d_rem.st]);
            const int64_t slot = carry_slot(c.slot_base, qb >> 1, kh) * kTileQ + (qb & 1) * kBM + rp.row;
            W = cw[slot];
            cright = cc[slot];
        }
        float beta[16], g[16];
        float prod = 1.f;
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
            const int j = rp.part * 16 + jj;
            float bt, rr;
            sigmoid_pair(Ss[rp.row * kSP + j] * a.inv_temp, bt, rr);
            const bool vis = row_ok && visible(qi, key0 + j, c.len, a.attend_current);
            beta[jj] = vis ? bt : 0.f;
            g[jj] = vis ? rr : 1.f;
            prod *= g[jj];
        }
        float run = W * quad_right_prod(prod, rp.part);
        float gsum = 0.f;
        float pv[16];
#pragma unroll
        for (int jj = 15; jj >= 0; --jj) {
            const float rr = g[jj];
            pv[jj] = beta[jj] * run;
            g[jj] = pv[jj] * (Ps[rp.row * kSP + rp.part * 16 + jj] - drem);
            gsum += g[jj];
            run *= rr;
        }
        // inclusive prefix at key j = (prefix through the tile's right edge) - (sum of g right of j)
        float right = quad_right_sum(gsum, rp.part);
#pragma unroll
        for (int jj = 15; jj >= 0; --jj) {
            const float cin = cright - right;
            Ss[rp.row * kSP + rp.part * 16 + jj] = pv[jj];
            Ps[rp.row * kSP + rp.part * 16 + jj] = g[jj] - beta[jj] * cin;
            right += g[jj];
        }
        __syncthreads();
        gemm_ptx(acc_v, Ss, Gs, DPP, D);
        gemm_ptx(acc_k, Ps, Qs, DPP, D);
    }
    store_acc<T>(acc_k, a.inv_temp, a.dk, c.b, h, c.start + key0, keys_valid, D);
    store_acc<T>(acc_v, 1.f, a.dv, c.b, h, c.start + key0, keys_valid, D);
}

size_t simt_smem_bytes(int D, bool bwd) {
    const int DPP = (D | 1) + 16;
    return sizeof(float) * (size_t)((bwd ? 4 : 3) * kBM * DPP + (bwd ? 2 : 1) * kBM * kSP);
}

template <typename T>
int launch_fwd_t(const WsLayout& L, const KArgs& a, cudaStream_t st) {
    const size_t smem = simt_smem_bytes(a.head_dim, false);
    cudaError_t e = cudaFuncSetAttribute(simt_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(L.max_items, a.heads, 2);
    simt_fwd_kernel<T><<<grid, kThreads, smem, st>>>(a);
    count_launch();
    return (int)cudaGetLastError();
}

template <typename T>
int launch_bwd_t(const WsLayout& L, const KArgs& a, int phases, cudaStream_t st) {
    const size_t smem = simt_smem_bytes(a.head_dim, true);
    cudaError_t e = cudaFuncSetAttribute(simt_bwd_dq_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(simt_bwd_dkdv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(L.max_items, a.heads, 2);
    if (phases != SBATTN_BWD_DKDV) {
        simt_bwd_dq_kernel<T><<<grid, kThreads, smem, st>>>(a);
        count_launch();
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (phases != SBATTN_BWD_DQ) {
        simt_bwd_dkdv_kernel<T><<<grid, kThreads, smem, st>>>(a);
        count_launch();
    }
    return (int)cudaGetLastError();
}

}  // namespace

int launch_simt_fwd(const SbParams& p, const WsLayout& L, const KArgs& a, cudaStream_t st) {
    if (L.max_items <= 0) return 0;
    switch (p.dtype) {
        case SBATTN_BF16: return launch_fwd_t<__nv_bfloat16>(L, a, st);
        case SBATTN_F16: return launch_fwd_t<__half>(L, a, st);
        default: return launch_fwd_t<float>(L, a, st);
    }
}

int launch_simt_bwd(const SbParams& p, const WsLayout& L, const KArgs& a, cudaStream_t st) {
    if (L.max_items <= 0) return 0;
    switch (p.dtype) {
        case SBATTN_BF16: return launch_bwd_t<__nv_bfloat16>(L, a, p.bwd_phases, st);
        case SBATTN_F16: return launch_bwd_t<__half>(L, a, p.bwd_phases, st);
        default: return launch_bwd_t<float>(L, a, p.bwd_phases, st);
    }
}

}  // namespace sb
