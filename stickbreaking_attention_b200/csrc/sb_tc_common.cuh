// Helpers shared by the tensor-core forward and backward kernels.
#pragma once

#include "sb_common.cuh"
#include "sb_sm100.cuh"

namespace sb {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool kF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    return kF16 ? sm100::pack_f16(lo, hi) : sm100::pack_bf16(lo, hi);
}

// (head, sequence, 128-row tile) of a flat work index; items are ordered heaviest first
struct Work {
    int h, b, start, len, qt, slot_base;
};
__device__ __forceinline__ Work fetch_work(const KArgs& a, int w) {
    const int item = w / a.heads;
    const int2 it = a.items[item];
    const SeqInfo s = a.seqs[it.x];
    return Work{w - item * a.heads, s.batch, s.start, s.len, it.y, s.slot_base};
}

// teardown shared by the kernels: report a wait that ran out, let copies in flight land, free tensor memory
__device__ __forceinline__ void tc_teardown(volatile uint32_t* abort_flag, uint32_t* status, uint32_t tmem, uint32_t ncols,
                                            int alloc_warp) {
    __syncwarp();
    sm100::tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicOr(status, SBATTN_ST_TIMEOUT);
        for (int i = 0; i < 200; ++i) __nanosleep(5000);
        __syncthreads();
    }
    if ((int)(threadIdx.x >> 5) == alloc_warp) {
        sm100::tc_fence_after();
        sm100::tmem_dealloc(tmem, ncols);
    }
}

inline int sm_count() {
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

inline bool aligned_mat(const SbMat& m) {
    if (!m.ptr) return true;
    return ((uintptr_t)m.ptr & 15) == 0 && (m.stride_t & 7) == 0 && (m.stride_h & 7) == 0 && (m.stride_b & 7) == 0;
}

int launch_tensor_bwd_impl(const SbParams& p, const KArgs& a, cudaStream_t st);

}  // namespace sb
