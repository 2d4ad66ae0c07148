// Prep kernel: turns the sequence ends on the device into the tables every attention kernel walks -- one
// SeqInfo per sequence and the list of (sequence, 128-row tile) work items ordered heaviest first (a tile's
// cost is the number of key tiles to its left, i.e. its index inside the sequence + 1).  Runs as a single
// thread block on the caller's stream, so no host synchronisation is needed to learn the sequence lengths.
//
// Reference counterpart: the grid computation of varlen_fwd (stickbreaking_attention/sb_varlen/sb_varlen_fwd.py
// :476-479), which sizes the grid by max_seqlens and lets programs of short sequences exit early, and the
// per-program lookup of the sequence bounds (:283-288).
#include "sb_common.cuh"

namespace sb {

namespace {

constexpr int kPrepThreads = 1024;

__device__ inline int64_t read_end(const void* cu, int width, int i) {
    return width == 8 ? ((const int64_t*)cu)[i] : (int64_t)((const int32_t*)cu)[i];
}

// Exclusive block scan of two int values per thread (Hillis-Steele over shared memory).
__device__ inline void block_scan2(int& a, int& b, int* sh_a, int* sh_b, int& tot_a, int& tot_b) {
    const int t = threadIdx.x;
    sh_a[t] = a;
    sh_b[t] = b;
    __syncthreads();
    for (int off = 1; off < kPrepThreads; off <<= 1) {
        int va = 0, vb = 0;
        if (t >= off) { va = sh_a[t - off]; vb = sh_b[t - off]; }
        __syncthreads();
        sh_a[t] += va;
        sh_b[t] += vb;
        __syncthreads();
    }
    tot_a = sh_a[kPrepThreads - 1];
    tot_b = sh_b[kPrepThreads - 1];
    const int ia = sh_a[t] - a, ib = sh_b[t] - b;
    __syncthreads();
    a = ia;
    b = ib;
}

__global__ void __launch_bounds__(kPrepThreads, 1)
prep_kernel(WsHeader* hdr, SeqInfo* seqs, int2* items, int32_t* bins, const void* cu, int cu_width, int n_seqs,
            int batch, int tokens, int max_len, int n_max, int max_items, int64_t slot_cap, uint32_t* status) {
    __shared__ int sh_a[kPrepThreads];
    __shared__ int sh_b[kPrepThreads];
    __shared__ int sh_bad;
    const int t = threadIdx.x;
    int32_t* count = bins;               // [n_max+2] sequences per tile count, then items per cost class
    int32_t* cursor = bins + n_max + 2;  // [n_max+2] write position per cost class
    if (t == 0) sh_bad = 0;
    if (t < 8) hdr->sched[t] = 0;
    for (int i = t; i < 2 * (n_max + 2); i += kPrepThreads) bins[i] = 0;
    __syncthreads();

    // pass 1: sequence table, running offsets
    int item_carry = 0, slot_carry = 0;
    for (int base = 0; base < n_seqs; base += kPrepThreads) {
        const int s = base + t;
        int len = 0, start = 0, b = 0, bad = 0;
        if (s < n_seqs) {
            if (batch > 0) {
                b = s; start = 0; len = tokens;
            } else {
                const int64_t e1 = read_end(cu, cu_width, s);
                const int64_t e0 = s > 0 ? read_end(cu, cu_width, s - 1) : 0;
                if (e0 < 0 || e1 < e0 || e1 > tokens || e1 - e0 > max_len) bad = 1;
                start = (int)e0;
                len = bad ? 0 : (int)(e1 - e0);
            }
        }
        if (bad) sh_bad = 1;
        const int n = (len + kTileQ - 1) / kTileQ;
        int a_items = n, a_slots = n * (n + 1), tot_i, tot_s;
        block_scan2(a_items, a_slots, sh_a, sh_b, tot_i, tot_s);
        if (s < n_seqs) {
            seqs[s] = SeqInfo{b, start, len, slot_carry + a_slots};
            if (n > 0) atomicAdd(&count[n], 1);
        }
        item_carry += tot_i;
        slot_carry += tot_s;
    }
    __syncthreads();
    const bool bad = sh_bad != 0 || item_carry > max_items || (int64_t)slot_carry > slot_cap;

    // pass 2: items of cost c (tile index c-1) = sequences with at least c tiles; heaviest class first
    if (t == 0) {
        int run = 0;
        for (int c = n_max; c >= 1; --c) { run += count[c]; count[c] = run; }  // items in class c
        int pos = 0;
        for (int c = n_max; c >= 1; --c) { cursor[c] = pos; pos += count[c]; }
        hdr->n_items = bad ? 0 : item_carry;
        hdr->n_seqs = n_seqs;
        hdr->total_slots = slot_carry;
        hdr->bad = bad ? 1 : 0;
        hdr->covered_end = batch > 0 ? tokens : (n_seqs > 0 && !bad ? (int)read_end(cu, cu_width, n_seqs - 1) : 0);
        if (bad) atomicOr(status, SBATTN_ST_BAD_SEQLENS);
    }
    __syncthreads();
    if (bad) return;
    for (int s = t; s < n_seqs; s += kPrepThreads) {
        const int n = (seqs[s].len + kTileQ - 1) / kTileQ;
        for (int qt = 0; qt < n; ++qt) {
            const int pos = atomicAdd(&cursor[qt + 1], 1);
            items[pos] = make_int2(s, qt);
        }
    }
}

// Gradient rows of tokens that belong to no sequence (a pack whose last end is below T) are zero; every other row is
// written by the backward kernels, so the caller does not have to clear dq, dk, dv beforehand.
template <typename T>
__global__ void zero_tail_kernel(const WsHeader* hdr, MatView dq, MatView dk, MatView dv, int heads, int tokens, int D) {
    const int first = hdr->covered_end;
    const int rows = tokens - first;
    if (rows <= 0) return;
    const int64_t total = (int64_t)rows * heads * D;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % D);
        const int64_t rh = i / D;
        const int h = (int)(rh % heads);
        const int64_t t = first + rh / heads;
        ((T*)dq.ptr)[h * dq.sh + t * dq.st + d] = T(0.f);
        ((T*)dk.ptr)[h * dk.sh + t * dk.st + d] = T(0.f);
        ((T*)dv.ptr)[h * dv.sh + t * dv.st + d] = T(0.f);
    }
}

// rem and neg_log_acc of tokens that belong to no sequence are zero (what the reference's zero-initialised outputs hold
// there, sb_varlen_fwd.py:418-419); every other row is written by the forward kernels, so the caller need not clear them.
template <typename T>
__global__ void zero_tail_rows_kernel(const WsHeader* hdr, VecView rem, VecView nla, int heads, int tokens) {
    const int first = hdr->covered_end;
    const int rows = tokens - first;
    if (rows <= 0) return;
    const int64_t total = (int64_t)rows * heads;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int h = (int)(i % heads);
        const int64_t t = first + i / heads;
        ((T*)rem.ptr)[h * rem.sh + t * rem.st] = T(0.f);
        ((float*)nla.ptr)[h * nla.sh + t * nla.st] = 0.f;
    }
}

}  // namespace

int launch_zero_tail_rows(const SbParams& p, const KArgs& a, cudaStream_t st) {
    if (p.batch > 0) return 0;  // the batched layout covers every token
    if (p.dtype == SBATTN_F32) zero_tail_rows_kernel<float><<<16, 256, 0, st>>>(a.hdr, a.rem, a.nla, p.heads, p.tokens);
    else if (p.dtype == SBATTN_F16) zero_tail_rows_kernel<__half><<<16, 256, 0, st>>>(a.hdr, a.rem, a.nla, p.heads, p.tokens);
    else zero_tail_rows_kernel<__nv_bfloat16><<<16, 256, 0, st>>>(a.hdr, a.rem, a.nla, p.heads, p.tokens);
    count_launch();
    return (int)cudaGetLastError();
}

int launch_zero_tail(const SbParams& p, const KArgs& a, cudaStream_t st) {
    if (p.batch > 0) return 0;  // the batched layout covers every token
    if (p.dtype == SBATTN_F32)
        zero_tail_kernel<float><<<64, 256, 0, st>>>(a.hdr, a.dq, a.dk, a.dv, p.heads, p.tokens, p.head_dim);
    else if (p.dtype == SBATTN_F16)
        zero_tail_kernel<__half><<<64, 256, 0, st>>>(a.hdr, a.dq, a.dk, a.dv, p.heads, p.tokens, p.head_dim);
    else
        zero_tail_kernel<__nv_bfloat16><<<64, 256, 0, st>>>(a.hdr, a.dq, a.dk, a.dv, p.heads, p.tokens, p.head_dim);
    count_launch();
    return (int)cudaGetLastError();
}

int launch_prep(const SbParams& p, const WsLayout& L, cudaStream_t st) {
    char* ws = (char*)p.fwd_workspace;
    const int max_len = p.batch > 0 ? p.tokens : (p.max_seqlen > 0 ? p.max_seqlen : p.tokens);
    prep_kernel<<<1, kPrepThreads, 0, st>>>((WsHeader*)ws, (SeqInfo*)(ws + L.off_seqs), (int2*)(ws + L.off_items),
                                            (int32_t*)(ws + L.off_bins), p.cu_seqlens, p.cu_width, L.n_seqs, p.batch,
                                            p.tokens, max_len, L.n_max, L.max_items, L.slot_cap, p.status);
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace sb
