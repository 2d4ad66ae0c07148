// Attention weights as a dense float32 matrix: the debugging output of the reference's forward launchers
// (return_attention=True, sb_varlen_fwd.py:194-201 and sb_fwd.py:145-147).  Not a hot path: one warp per query row,
// float32 arithmetic with the precise logarithm / exponential (this file is compiled without fast math).
#include "sb_common.cuh"

namespace sb {

namespace {

constexpr int kWeightWarps = 4;  // query rows per block

__device__ inline int64_t seq_end(const void* cu, int width, int s) {
    return width == 8 ? ((const int64_t*)cu)[s] : (int64_t)((const int32_t*)cu)[s];
}

// w[b][h][row][col] = sigmoid(s_ij) * prod_{j < k visible} (1 - sigmoid(s_ik)), s = q_i . k_j * inv_temp, for every visible
// pair; other entries are not touched.  Packed layout: row and col are token indices of the pack (block diagonal).
template <typename T>
__global__ void __launch_bounds__(32 * kWeightWarps)
weights_kernel(MatView q, MatView k, const void* cu, int cu_width, int num_seqs, int batch, int tokens, int D,
               int attend_current, float inv_temp, float* w, int64_t wsb, int64_t wsh, int64_t wsm) {
    __shared__ float qs[kWeightWarps][kMaxHeadDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWeightWarps + warp;
    const int h = blockIdx.y;
    const int64_t rows = (int64_t)tokens * (batch > 0 ? batch : 1);
    if (row >= rows) return;  // whole warps leave; nothing below synchronises the block
    int b = 0, t = (int)row, start = 0;
    if (batch > 0) {
        b = (int)(row / tokens);
        t = (int)(row % tokens);
    } else {
        // the sequence of token t: the first whose end is beyond t
        int lo = 0, hi = num_seqs;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (seq_end(cu, cu_width, mid) > t) hi = mid; else lo = mid + 1;
        }
        if (lo >= num_seqs) return;  // beyond the last sequence
        const int64_t s0 = lo > 0 ? seq_end(cu, cu_width, lo - 1) : 0;
        if (s0 < 0 || s0 > t || seq_end(cu, cu_width, lo) > tokens) return;  // inconsistent ends: the forward reports them
        start = (int)s0;
    }
    const int n = t - start + (attend_current ? 1 : 0);  // visible keys: start .. start + n - 1
    const T* qp = (const T*)q.ptr + (int64_t)b * q.sb + (int64_t)h * q.sh + (int64_t)t * q.st;
    for (int d = lane; d < D; d += 32) qs[warp][d] = to_f32(qp[d]);
    __syncwarp();
    float* wrow = w + (int64_t)b * wsb + (int64_t)h * wsh + (int64_t)t * wsm + (batch > 0 ? 0 : start);
    float right = 0.f;  // sum of log(1 - beta) over the keys to the right of this chunk
    for (int hi = n; hi > 0; hi -= 32) {
        const int j = hi - 1 - lane;  // lane 0 holds the rightmost key of the chunk
        const bool valid = j >= 0;
        float s = 0.f;
        if (valid) {
            const T* kp = (const T*)k.ptr + (int64_t)b * k.sb + (int64_t)h * k.sh + (int64_t)(start + j) * k.st;
            for (int d = 0; d < D; ++d) s = fmaf(qs[warp][d], to_f32(kp[d]), s);
        }
        s *= inv_temp;
        const float log_beta = fminf(s, 0.f) - log1pf(expf(-fabsf(s)));
        const float log_rest = valid ? log_beta - s : 0.f;  // log(1 - sigmoid(s))
        float x = log_rest;                                 // inclusive sum over the lanes to the right
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, x, off);
            if (lane >= off) x += y;
        }
        if (valid) wrow[j] = expf(log_beta + right + (x - log_rest));
        right += __shfl_sync(0xffffffffu, x, 31);
    }
}

template <typename T>
int launch_weights_t(const SbParams& p, float* w, int64_t sb_, int64_t sh, int64_t sm, cudaStream_t st) {
    const int64_t rows = (int64_t)p.tokens * (p.batch > 0 ? p.batch : 1);
    const dim3 grid((unsigned)((rows + kWeightWarps - 1) / kWeightWarps), (unsigned)p.heads);
    weights_kernel<T><<<grid, 32 * kWeightWarps, 0, st>>>(view(p.q), view(p.k), p.cu_seqlens, p.cu_width, p.num_seqs, p.batch,
                                                         p.tokens, p.head_dim, p.attend_current ? 1 : 0, p.inv_temp, w, sb_,
                                                         sh, sm);
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace

int launch_weights(const SbParams& p, float* w, int64_t stride_b, int64_t stride_h, int64_t stride_m, cudaStream_t st) {
    if (p.dtype == SBATTN_F32) return launch_weights_t<float>(p, w, stride_b, stride_h, stride_m, st);
    if (p.dtype == SBATTN_F16) return launch_weights_t<__half>(p, w, stride_b, stride_h, stride_m, st);
    return launch_weights_t<__nv_bfloat16>(p, w, stride_b, stride_h, stride_m, st);
}

}  // namespace sb
