/*
 * sbattn.h -- C ABI of the B200 stick-breaking attention library (libsbattn.so).
 *
 * The library replaces the four host launchers of the reference and the Triton kernels below them:
 *
 *   sbattn_fwd  <->  varlen_fwd   stickbreaking_attention/sb_varlen/sb_varlen_fwd.py:411-521   (packed [H,T,D])
 *                    _fwd         stickbreaking_attention/sb_attn/sb_fwd.py:137-251            (batched [B,H,T,D])
 *   sbattn_bwd  <->  varlen_bwd   stickbreaking_attention/sb_varlen/sb_varlen_bwd.py:483-640
 *                    _bwd         stickbreaking_attention/sb_attn/sb_bwd.py:162-296
 *
 * Ownership: the caller allocates every buffer (inputs, outputs, workspaces, the status word); the library
 * allocates and frees no device memory and keeps no pointer after a call returns.  All work is enqueued on
 * the stream passed in; nothing synchronises with the host.
 * Errors: 0 on success, a negative SBATTN_E* code otherwise; nothing is launched when a code is returned
 * for bad arguments.  Conditions that only the device can see (non-monotone sequence ends, a wait inside a
 * kernel that ran out) are reported through the caller's status word, see SBATTN_ST_*.
 * Threading: re-entrant; the device the buffers live on must be current on the calling thread.
 */
#ifndef SBATTN_H_
#define SBATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SBATTN_VERSION 100

/* return codes */
#define SBATTN_OK 0
#define SBATTN_EINVAL (-1)       /* inconsistent sizes, negative strides, bad enum                       */
#define SBATTN_ENULL (-2)        /* a required pointer is NULL                                           */
#define SBATTN_EUNSUPPORTED (-3) /* head_dim > 128, dtype/path combination that has no kernel            */
#define SBATTN_EWORKSPACE (-4)   /* workspace missing or smaller than sbattn_workspace_bytes says        */
#define SBATTN_EALIGN (-5)       /* tensor-core path asked for, but pointers/strides are not 16-B aligned */
#define SBATTN_ECUDA (-6)        /* a CUDA runtime/driver call failed (launch error, no sm_100 device)   */
#define SBATTN_ECAPACITY (-7)    /* sbattn_fwd_static: the problem needs more than the built-in scratch  */

/* bits of the device status word (0 = fine) */
#define SBATTN_ST_BAD_SEQLENS 1u /* sequence ends decrease, exceed the token count or max_seqlen         */
#define SBATTN_ST_TIMEOUT 2u     /* a bounded wait inside a kernel gave up; results are invalid          */

/* element types of q, k, v, o, rem, do, drem, dq, dk, dv */
#define SBATTN_BF16 0
#define SBATTN_F32 1
#define SBATTN_F16 2

/* kernel family */
#define SBATTN_PATH_AUTO 0   /* tensor-core kernels when eligible (bf16/f16, head_dim 32, 64 or 128, aligned), else SIMT */
#define SBATTN_PATH_SIMT 1   /* fp32-arithmetic kernels: any dtype, any head_dim <= 128, any strides     */
#define SBATTN_PATH_TENSOR 2 /* tcgen05 kernels or SBATTN_EUNSUPPORTED / SBATTN_EALIGN                   */

/* backward phases */
#define SBATTN_BWD_ALL 0
#define SBATTN_BWD_DQ 1
#define SBATTN_BWD_DKDV 2

/* [B,H,T,D] matrix (B absent for the packed layout); strides in ELEMENTS, the D stride is 1 */
typedef struct SbMat {
    void* ptr;
    int64_t stride_b, stride_h, stride_t;
} SbMat;

/* [B,H,T] per-row vector; strides in elements */
typedef struct SbVec {
    void* ptr;
    int64_t stride_b, stride_h, stride_t;
} SbVec;

/* SbParams::flags.  SBATTN_FLAG_FUSED_REMAINDER: the forward writes out = o + rem * v into `o` (what every caller of the
 * reference computes next: tests/test_varlen.py:103, tests/test_attn.py:67, benchmarks/varlen.py:53), with rem rounded
 * to the output dtype first, as in that expression.  The backward then takes d_o = gradient of out and d_rem = gradient
 * of the separately returned rem, needs `rem` (the forward's output) and `v`, and returns dv including rem * d_o.
 * Tensor-core path only (16-bit inputs, head_dim 32, 64 or 128): otherwise SBATTN_EUNSUPPORTED. */
#define SBATTN_FLAG_FUSED_REMAINDER 1

typedef struct SbParams {
    int32_t dtype;          /* SBATTN_BF16 / F32 / F16                                                    */
    int32_t path;           /* SBATTN_PATH_*                                                              */
    int32_t batch;          /* 0: packed layout [H,T,D] with cu_seqlens; >0: batched [B,H,T,D]            */
    int32_t heads;
    int32_t tokens;         /* T: total tokens (packed) or tokens per batch entry (batched)               */
    int32_t head_dim;       /* D <= 128                                                                   */
    int32_t num_seqs;       /* packed: entries of cu_seqlens; batched: ignored                            */
    int32_t cu_width;       /* 4 or 8: bytes per entry of cu_seqlens                                      */
    const void* cu_seqlens; /* device; cumulative sequence ENDS, no leading zero (what varlen_fwd gets)   */
    int32_t max_seqlen;     /* upper bound on any sequence length (sizes the carry workspace)             */
    int32_t attend_current; /* 0: key j < query i; 1: key j <= i                                          */
    float inv_temp;         /* logits = q.k * inv_temp                                                    */
    int32_t save_carries;   /* forward: 1 if a backward will follow (fills the carry part of fwd_workspace) */
    int32_t bwd_phases;     /* backward: 0 = everything; SBATTN_BWD_DQ / SBATTN_BWD_DKDV run one kernel only
                               (for timing them apart; dk/dv needs the carries the dq kernel leaves behind)   */
    int32_t flags;          /* SBATTN_FLAG_*                                                              */

    SbMat q, k, v;          /* inputs                                                                     */
    SbMat o;                /* forward output, dtype                                                      */
    SbVec rem;              /* forward output, dtype: 1 - sum of attention                                */
    SbVec neg_log_acc;      /* forward output, float32: log2 of rem (the reference's saved tensor)        */

    SbMat d_o;              /* backward inputs                                                            */
    SbVec d_rem;
    SbMat dq, dk, dv;       /* backward outputs, dtype; every covered row is written (no zero-fill needed) */

    void* fwd_workspace;    /* written by forward, read by backward: keep it alive in between             */
    size_t fwd_workspace_bytes;
    void* bwd_workspace;    /* scratch of one backward call                                               */
    size_t bwd_workspace_bytes;

    uint32_t* status;       /* device word, OR-ed with SBATTN_ST_*; caller zeroes it                      */
    void* stream;           /* cudaStream_t                                                               */
} SbParams;

/* Bytes the two workspaces need for the shape fields of p (pointers are not looked at).
 * Reference counterpart: the allocations inside varlen_fwd / varlen_bwd (sb_varlen_fwd.py:417-424,
 * sb_varlen_bwd.py:506-508,569-572), moved to the caller. */
int sbattn_workspace_bytes(const SbParams* p, size_t* fwd_bytes, size_t* bwd_bytes);

/* o, rem, neg_log_acc <- q, k, v.  Replaces varlen_fwd (sb_varlen_fwd.py:411) and _fwd (sb_fwd.py:137). */
int sbattn_fwd(const SbParams* p);

/* dq, dk, dv <- do, drem, q, k, v and the forward's workspace.
 * Replaces varlen_bwd (sb_varlen_bwd.py:483) and _bwd (sb_bwd.py:162). */
int sbattn_bwd(const SbParams* p);

/* Forward without any allocation by anybody: the tables the forward needs live in a fixed 1 MiB array inside the
 * library (sbattn_static_scratch_bytes), which every GPU that loads the library holds until the process exits.
 * It has no counterpart in the reference.  It exists for callers that cannot allocate device memory at the call:
 * an inference server whose memory pool owns the whole device, a plugin that must not touch its host's allocator.
 *   - p->fwd_workspace, p->save_carries are ignored; no backward can follow (gradient-free forward only).  The caller
 *     still passes q, k, v, o, rem, neg_log_acc, cu_seqlens and the status word.
 *   - Returns SBATTN_ECAPACITY when the work-item tables of the shape do not fit (they need roughly
 *     16 bytes per sequence + 8 bytes per 128 tokens: a million tokens in tens of thousands of sequences fit).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress) with that device
 *     current; make that first call outside any stream capture.  Later calls only launch kernels.
 *   - All calls on one GPU share the array.  Every call rewrites the tables and zeroes its counters itself, so
 *     calls that follow each other on one stream are safe; calls that can overlap on the GPU (different streams,
 *     different threads) race on it and must be serialised by the caller.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine. */
int sbattn_fwd_static(const SbParams* p);

/* Size in bytes of the built-in scratch of sbattn_fwd_static.  No counterpart in the reference. */
size_t sbattn_static_scratch_bytes(void);

/* Attention weights as a dense float32 matrix, a debugging aid: w[b][h][i][j] = weight of key j in the output of
 * query i, written for every visible pair (j < i, or j <= i with attend_current); the other entries keep what the
 * caller put there (the reference fills the matrix with zeros first).  Replaces the return_attention=True mode of
 * varlen_fwd (sb_varlen_fwd.py:194-201, W allocated at :420-422 as [H,T,T]) and of _fwd (sb_fwd.py:145-147,
 * [B,H,T,T]).  Uses dtype, batch, heads, tokens, head_dim, num_seqs, cu_width, cu_seqlens, attend_current, inv_temp,
 * q, k and stream of p; no workspace.  Strides in elements; the column stride is 1 and stride_m >= tokens.
 * Packed layout: i and j are token indices of the pack, so each sequence fills its own diagonal block.  (The reference
 * offsets a sequence's block by its start along the columns only, sb_varlen_fwd.py:316; both agree for a pack of
 * one sequence.)  Float32 arithmetic whatever the dtype; cost O(T^2 D) per head with no tensor cores. */
int sbattn_attention_weights(const SbParams* p, float* w, int64_t stride_b, int64_t stride_h, int64_t stride_m);

/* Text for a return code.  No counterpart in the reference (it raises Python exceptions). */
const char* sbattn_strerror(int code);

/* SBATTN_VERSION the library was built with. */
int sbattn_version(void);

/* sizeof(SbParams) as the library was compiled: lets a foreign-function binding check its mirror of the struct.
 * No counterpart in the reference. */
size_t sbattn_params_size(void);

/* Number of GPU kernels this library has launched in the calling process so far (all entry points, all devices).
 * A benchmark reads it before and after a step to report how many kernels of the library the step ran.
 * No counterpart in the reference. */
unsigned long long sbattn_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SBATTN_H_ */
