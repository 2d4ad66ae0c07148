// Helpers shared by the tensor-core forward and backward kernels.
#pragma once

#include <mutex>
#include <unordered_map>

#include "sb_common.cuh"
#include "sb_sm100.cuh"

namespace sb {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^x for two values at once on the FMA pipes instead of the special-function unit (which delivers 16 results per clock
// and SM against 128 fused multiply-adds): x = n + f with n the nearest integer (the magic-number addition leaves n in
// the low mantissa bits of t), 2^f by a degree-4 polynomial on [-0.5, 0.5] (relative error 3.5e-6, far below the 16-bit
// rounding of the weights), and n added to the exponent field.  The caller keeps x within [-125, 15].
// Every multiply-add is a packed fp32x2 instruction.
__device__ __forceinline__ float2 ex2_fma2(float2 x) {
    const float kMagic = 12582912.f;  // 1.5 * 2^23
    const float2 t = __fadd2_rn(x, make_float2(kMagic, kMagic));
    const float2 n = __fadd2_rn(t, make_float2(-kMagic, -kMagic));
    const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
    // Chebyshev interpolant of 2^f on [-0.5, 0.5]
    float2 p = __ffma2_rn(f, make_float2(9.666368515e-3f, 9.666368515e-3f), make_float2(5.592197584e-2f, 5.592197584e-2f));
    p = __ffma2_rn(p, f, make_float2(2.402234904e-1f, 2.402234904e-1f));
    p = __ffma2_rn(p, f, make_float2(6.931210452e-1f, 6.931210452e-1f));
    p = __ffma2_rn(p, f, make_float2(1.f, 1.f));
    return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)),
                       __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
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

// 32 fp32 accumulator values of one row -> 32 16-bit values (64 bytes) at `dst`, scaled by `sc`.  256-bit stores where the
// address allows it: every lane of a warp writes its own row, so each store instruction touches 32 different lines and
// the number of instructions is what the epilogues cost.
template <bool kF16>
__device__ __forceinline__ void store_row32(char* dst, const uint32_t (&v)[32], float sc) {
    uint32_t u[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) u[j] = pack16<kF16>(__uint_as_float(v[2 * j]) * sc, __uint_as_float(v[2 * j + 1]) * sc);
    if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 32 * h), "r"(u[8 * h]),
                         "r"(u[8 * h + 1]), "r"(u[8 * h + 2]), "r"(u[8 * h + 3]), "r"(u[8 * h + 4]), "r"(u[8 * h + 5]),
                         "r"(u[8 * h + 6]), "r"(u[8 * h + 7])
                         : "memory");
    } else {
#pragma unroll
        for (int h = 0; h < 4; ++h) *(uint4*)(dst + 16 * h) = make_uint4(u[4 * h], u[4 * h + 1], u[4 * h + 2], u[4 * h + 3]);
    }
}

// The same for the two rows of a lane pair at once.  Lanes l and l ^ 1 own consecutive rows; after one exchange the even
// lane holds the first 32 bytes of both rows' 64 and the odd lane the second 32, so that the 64 bytes of a row leave in one
// instruction from two neighbouring lanes: 16 instead of 32 distinct lines per store instruction, and a 128 x 128 tile
// leaves the SM in ~1 100 instead of ~2 000 cycles (measured in isolation).  `dst` is this lane's own row, `row_bytes` the
// distance between consecutive rows, `ok` whether this lane's row is to be written.  All 32 lanes must call.
template <bool kF16>
__device__ __forceinline__ void store_row32_pairs(char* dst, const uint32_t (&v)[32], float sc, int64_t row_bytes, bool ok, int lane) {
    uint32_t u[16], s[8];
#pragma unroll
    for (int j = 0; j < 16; ++j) u[j] = pack16<kF16>(__uint_as_float(v[2 * j]) * sc, __uint_as_float(v[2 * j + 1]) * sc);
    const bool hi = lane & 1;
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] = __shfl_xor_sync(0xffffffffu, hi ? u[j] : u[8 + j], 1);  // the half the partner writes
    const bool ok_other = __shfl_xor_sync(0xffffffffu, (int)ok, 1) != 0;
    char* own = dst + (hi ? 32 : 0);
    char* oth = own + (hi ? -row_bytes : row_bytes);
    const auto put = [](char* p, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t a4, uint32_t a5, uint32_t a6, uint32_t a7) {
        if ((reinterpret_cast<uintptr_t>(p) & 31) == 0) {
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(a4),
                         "r"(a5), "r"(a6), "r"(a7)
                         : "memory");
        } else {
            *(uint4*)p = make_uint4(a0, a1, a2, a3);
            *(uint4*)(p + 16) = make_uint4(a4, a5, a6, a7);
        }
    };
    if (ok) {
        if (hi) put(own, u[8], u[9], u[10], u[11], u[12], u[13], u[14], u[15]);
        else put(own, u[0], u[1], u[2], u[3], u[4], u[5], u[6], u[7]);
    }
    if (ok_other) put(oth, s[0], s[1], s[2], s[3], s[4], s[5], s[6], s[7]);
}

// 32 16-bit values at `src` as fp32
template <bool kF16>
__device__ __forceinline__ void load_row32(const char* src, float (&x)[32]) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        const uint4 u = __ldg((const uint4*)(src + 16 * h));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (kF16) {
                const float2 f = __half22float2(*(const __half2*)&w[j]);
                x[8 * h + 2 * j] = f.x;
                x[8 * h + 2 * j + 1] = f.y;
            } else {
                x[8 * h + 2 * j] = __uint_as_float(w[j] << 16);
                x[8 * h + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
        }
    }
}
template <bool kF16>
__device__ __forceinline__ float round16(float x) {
    return kF16 ? __half2float(__float2half_rn(x)) : __bfloat162float(__float2bfloat16_rn(x));
}

// (head, sequence, 128-row tile) of a flat work index.  Order: groups of `head_group` heads; inside a group the
// items heaviest first, the heads of the group innermost.
struct Work {
    int h, b, start, len, qt, slot_base;
};
__device__ __forceinline__ Work fetch_work(const KArgs& a, int n_items, int w) {
    const int per_group = n_items * a.head_group;
    const int g = w / per_group, rest = w - g * per_group;
    const int hg = min(a.head_group, a.heads - g * a.head_group);
    const int item = rest / hg;
    const int2 it = a.items[item];
    const SeqInfo s = a.seqs[it.x];
    return Work{g * a.head_group + rest - item * hg, s.batch, s.start, s.len, it.y, s.slot_base};
}

// ---------------------------------------------------------------------------------------------- work scheduler
// One thread of the block (a TMA producer) draws work indices from a global counter, looks the item up (two dependent
// global loads) and hands index and item to the other roles through a two-slot ring in shared memory, so that nobody
// else pays the lookup latency when an item begins.  A negative index ends the block.
constexpr int kRing = 2;
template <typename T>
struct SchedRing {
    int32_t slot[kRing];
    T work[kRing];
};
struct SchedProducer {
    int i = 0;
    uint32_t ph[kRing] = {1, 1};
    // An item is drawn only when a slot of the ring is free, i.e. at most kRing items before it is worked on: drawing
    // further ahead hides more of the lookup latency but binds items to blocks earlier, and the blocks then finish
    // further apart (measured: one more item ahead cost 4-12 % on a pack of 7 long sequences).
    template <typename T, typename F>
    __device__ __forceinline__ int next(int32_t* counter, int n_work, SchedRing<T>* ring, uint64_t* full, uint64_t* empty,
                                        volatile uint32_t* abort_flag, F fetch, T& out) {
        const int sl = i & (kRing - 1);
        ++i;
        if (!sm100::mbar_wait(&empty[sl], ph[sl], abort_flag)) return -1;
        ph[sl] ^= 1;
        int w = atomicAdd(counter, 1);
        if (w >= n_work) w = -1;
        if (w >= 0) {
            out = fetch(w);
            ring->work[sl] = out;
        }
        ring->slot[sl] = w;
        sm100::mbar_arrive(&full[sl]);
        return w;
    }
};
struct SchedConsumer {
    int i = 0;
    uint32_t ph[kRing] = {0, 0};
    // A whole warp that consumes together (the slot counts it as one consumer) passes whole_warp = true and
    // arrive = true in one lane only.
    template <typename T>
    __device__ __forceinline__ int next(SchedRing<T>* ring, uint64_t* full, uint64_t* empty, volatile uint32_t* abort_flag,
                                        T& out, bool arrive = true, bool whole_warp = false) {
        const int sl = i & (kRing - 1);
        ++i;
        if (!sm100::mbar_wait(&full[sl], ph[sl], abort_flag)) return -1;
        ph[sl] ^= 1;
        const int w = ring->slot[sl];
        if (w >= 0) out = ring->work[sl];
        if (whole_warp) __syncwarp();  // every lane has its copy before one of them releases the slot
        if (arrive) sm100::mbar_arrive(&empty[sl]);
        return w;
    }
};
// the last block to finish re-arms the counters for the next launch
__device__ __forceinline__ void sched_finish(int32_t* counter) {
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(counter + 1, 1) == (int)gridDim.x - 1) {
            counter[0] = 0;
            counter[1] = 0;
            __threadfence();
        }
    }
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

// Dynamic shared memory size (and the carve-out preference) of a kernel, set once per kernel and device instead of on
// every launch: the two driver calls cost more than the launch itself for small problems.
inline int ensure_kernel_attrs(const void* kernel, int smem_bytes, bool prefer_shared) {
    static std::mutex mu;
    static std::unordered_map<const void*, uint64_t> done;  // bit d: set on device d
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return (int)cudaErrorInvalidDevice;
    const bool tracked = dev >= 0 && dev < 64;
    if (tracked) {
        std::lock_guard<std::mutex> lock(mu);
        auto it = done.find(kernel);
        if (it != done.end() && ((it->second >> dev) & 1)) return 0;
    }
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    if (prefer_shared) cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (tracked) {
        std::lock_guard<std::mutex> lock(mu);
        done[kernel] |= 1ull << dev;
    }
    return 0;
}

inline bool aligned_mat(const SbMat& m) {
    if (!m.ptr) return true;
    return ((uintptr_t)m.ptr & 15) == 0 && (m.stride_t & 7) == 0 && (m.stride_h & 7) == 0 && (m.stride_b & 7) == 0;
}

}  // namespace sb
