// Shared host/device definitions of the stick-breaking attention library: workspace layout, the work-item
// table that every kernel walks, and small device helpers.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/sbattn.h"

namespace sb {

constexpr int kTileQ = 128;    // query rows per work item
constexpr int kTileKV = 64;    // keys per slot of the slot count (each slot holds two 32-key carries)
constexpr int kMaxHeadDim = 128;

// One sequence of the pack (or one batch entry of the batched layout).
struct SeqInfo {
    int32_t batch;      // index along B (0 for the packed layout)
    int32_t start;      // first token along T
    int32_t len;        // tokens
    int32_t slot_base;  // first carry slot of this sequence (per head)
};

// Start of the forward workspace.  The prep kernel fills it; all later kernels only read it.
struct WsHeader {
    int32_t n_items;      // work items per head = sum over sequences of ceil(len/128)
    int32_t n_seqs;
    int32_t total_slots;  // carry slots per head actually used
    int32_t bad;          // non-zero: sequence table rejected, n_items is 0
    // work counters of the persistent kernels (forward, backward dq, backward dk/dv): [2k] next work index,
    // [2k+1] blocks that have finished; zeroed by the prep kernel, reset by the last block of every launch
    int32_t sched[8];
    int32_t covered_end;  // packed layout: end of the last sequence (tokens beyond it belong to no sequence)
    int32_t pad[51];
};
static_assert(sizeof(WsHeader) == 256, "header is one 256-byte line");

// Host-side description of where things live inside the workspaces (all offsets in bytes).
struct WsLayout {
    int32_t n_seqs;      // sequences (packed: num_seqs, batched: B)
    int32_t n_max;       // max 128-row tiles of one sequence
    int32_t max_items;   // upper bound on items per head
    int64_t slot_cap;    // upper bound on 64-key carry slots per head
    int32_t hb;          // heads (batched: heads; the batch index comes from the sequence)
    size_t off_seqs, off_items, off_bins, off_carry;
    size_t off_drem;     // inside the backward workspace
    size_t fwd_bytes;    // with carries if save_carries
    size_t bwd_bytes;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline WsLayout make_layout(const SbParams& p) {
    WsLayout L{};
    const bool batched = p.batch > 0;
    L.n_seqs = batched ? p.batch : p.num_seqs;
    const int64_t maxlen = batched ? p.tokens : (p.max_seqlen > 0 ? (p.max_seqlen < p.tokens ? p.max_seqlen : p.tokens) : p.tokens);
    L.n_max = (int32_t)((maxlen + kTileQ - 1) / kTileQ);
    if (L.n_max < 1) L.n_max = 1;
    if (batched) {
        L.max_items = L.n_seqs * L.n_max;
        L.slot_cap = (int64_t)L.n_seqs * L.n_max * (L.n_max + 1);
    } else {
        // sum ceil(len/128) <= T/128 + S ; sum n(n+1) <= (n_max+1) * sum n
        const int64_t items = p.tokens / kTileQ + L.n_seqs;
        L.max_items = (int32_t)items;
        L.slot_cap = items * (L.n_max + 1);
    }
    L.hb = p.heads;
    size_t off = sizeof(WsHeader);
    L.off_seqs = off;
    off = align_up(off + sizeof(SeqInfo) * (size_t)L.n_seqs, 256);
    L.off_items = off;
    off = align_up(off + sizeof(int2) * (size_t)L.max_items, 256);
    L.off_bins = off;
    off = align_up(off + sizeof(int32_t) * (size_t)(2 * (L.n_max + 2)), 256);
    L.off_carry = off;
    const size_t carry = sizeof(float) * (size_t)L.hb * (size_t)(2 * L.slot_cap) * kTileQ;  // two 32-key carries per slot
    L.fwd_bytes = off + (p.save_carries ? carry : 0);
    L.off_drem = align_up(carry, 256);  // after carry_c: drem + do . v per (head, token), fused-remainder backward
    L.bwd_bytes = L.off_drem + align_up(sizeof(float) * (size_t)p.heads * (size_t)p.tokens * (size_t)(batched ? p.batch : 1), 256);
    return L;
}

// What the kernels need of a [B,H,T,D] tensor.
struct MatView {
    char* ptr;
    int64_t sb, sh, st;  // element strides
};
struct VecView {
    char* ptr;
    int64_t sb, sh, st;
};
inline MatView view(const SbMat& m) { return MatView{(char*)m.ptr, m.stride_b, m.stride_h, m.stride_t}; }
inline VecView view(const SbVec& m) { return VecView{(char*)m.ptr, m.stride_b, m.stride_h, m.stride_t}; }

// Arguments common to every attention kernel.
struct KArgs {
    const WsHeader* hdr;
    const SeqInfo* seqs;
    const int2* items;      // (sequence, 128-row tile), heaviest first
    float* carry_w;         // forward carries  [heads][slot_cap][128], may be null in a no-grad forward; slot_cap: 32-key slots
    float* carry_c;         // backward carries [heads][slot_cap][128]
    int64_t slot_cap;
    int32_t heads, head_dim, attend_current;
    int32_t fused;          // SBATTN_FLAG_FUSED_REMAINDER
    int32_t tokens;         // tokens per batch entry (row index of drem_eff: batch * tokens + token)
    float* drem_eff;        // [heads][drem_rows]: drem + do . v, written by the dq kernel when fused
    int64_t drem_rows;      // batch * tokens (tokens for the packed layout)
    int32_t head_group;     // heads whose work is interleaved (sized so that their K and V stay in L2)
    int32_t defer_fwd, defer_dq, defer_dkdv;  // tensor-core kernels: store an item's result one step into the next item
    int32_t* sched;         // WsHeader::sched
    float inv_temp;
    MatView q, k, v, o, d_o, dq, dk, dv;
    VecView rem, nla, d_rem;
    uint32_t* status;
};

// Carries exist at every 32-key boundary.  carry_slot32: (128-row tile qt of a sequence, 32-key quarter kq in [0, 4*qt+3]),
// the value at the quarter's right edge.  carry_slot: the same for the 64-key half kh in [0, 2*qt+1], i.e. its right quarter
// (the fp32-arithmetic kernels work in 64-key halves and use these alone).  slot_base and WsLayout::slot_cap count
// 64-key slots, KArgs::slot_cap 32-key slots.
__host__ __device__ inline int64_t carry_slot32(int32_t slot_base, int32_t qt, int32_t kq) {
    return 2 * ((int64_t)slot_base + (int64_t)qt * (qt + 1)) + kq;
}
__host__ __device__ inline int64_t carry_slot(int32_t slot_base, int32_t qt, int32_t kh) {
    return carry_slot32(slot_base, qt, 2 * kh + 1);
}

template <typename T> __device__ inline float to_f32(T x);
template <> __device__ inline float to_f32<float>(float x) { return x; }
template <> __device__ inline float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ inline float to_f32<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ inline T from_f32(float x);
template <> __device__ inline float from_f32<float>(float x) { return x; }
template <> __device__ inline __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ inline __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Kernel launches made by the library in this process (sbattn_launch_count); every launch site calls count_launch().
extern unsigned long long g_launch_count;
inline void count_launch() { __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED); }

// launchers implemented in the .cu files (each returns a cudaError_t as int; the tensor-core launchers return
// kMapEncodeFailed when a tensor map could not be encoded, before anything has been launched)
constexpr int kMapEncodeFailed = -1000;
int launch_prep(const SbParams& p, const WsLayout& L, cudaStream_t st);
int launch_zero_tail(const SbParams& p, const KArgs& a, cudaStream_t st);
int launch_zero_tail_rows(const SbParams& p, const KArgs& a, cudaStream_t st);
int launch_simt_fwd(const SbParams& p, const WsLayout& L, const KArgs& a, cudaStream_t st);
int launch_simt_bwd(const SbParams& p, const WsLayout& L, const KArgs& a, cudaStream_t st);
bool tensor_path_eligible(const SbParams& p, bool backward, int* why);
int launch_tensor_fwd(const SbParams& p, const WsLayout& L, const KArgs& a, cudaStream_t st);
int launch_tensor_bwd(const SbParams& p, const WsLayout& L, const KArgs& a, cudaStream_t st);
int launch_weights(const SbParams& p, float* w, int64_t stride_b, int64_t stride_h, int64_t stride_m, cudaStream_t st);

}  // namespace sb
