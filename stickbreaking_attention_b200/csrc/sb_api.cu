// C ABI entry points: argument checking, workspace layout, dispatch to the kernel families.
#include "sb_common.cuh"

namespace sb {

unsigned long long g_launch_count = 0;

namespace {

int check_mat(const SbMat& m, bool required) {
    if (!m.ptr) return required ? SBATTN_ENULL : SBATTN_OK;
    if (m.stride_t < 0 || m.stride_h < 0 || m.stride_b < 0) return SBATTN_EINVAL;
    return SBATTN_OK;
}
int check_vec(const SbVec& m, bool required) {
    if (!m.ptr) return required ? SBATTN_ENULL : SBATTN_OK;
    if (m.stride_t < 0 || m.stride_h < 0 || m.stride_b < 0) return SBATTN_EINVAL;
    return SBATTN_OK;
}

int check_shape(const SbParams* p) {
    if (!p) return SBATTN_ENULL;
    if (p->dtype != SBATTN_BF16 && p->dtype != SBATTN_F32 && p->dtype != SBATTN_F16) return SBATTN_EINVAL;
    if (p->path != SBATTN_PATH_AUTO && p->path != SBATTN_PATH_SIMT && p->path != SBATTN_PATH_TENSOR)
        return SBATTN_EINVAL;
    if (p->bwd_phases < 0 || p->bwd_phases > 2) return SBATTN_EINVAL;
    if (p->batch < 0 || p->heads < 0 || p->tokens < 0 || p->head_dim <= 0) return SBATTN_EINVAL;
    if (p->head_dim > kMaxHeadDim) return SBATTN_EUNSUPPORTED;
    if (p->batch == 0) {
        if (p->num_seqs < 0) return SBATTN_EINVAL;
        if (p->cu_width != 4 && p->cu_width != 8) return SBATTN_EINVAL;
        if (p->max_seqlen < 0) return SBATTN_EINVAL;
    }
    // the token axis is indexed with 32-bit integers inside the kernels
    if ((int64_t)p->tokens > (int64_t)1 << 30) return SBATTN_EUNSUPPORTED;
    return SBATTN_OK;
}

bool empty_problem(const SbParams* p) {
    return p->heads == 0 || p->tokens == 0 || (p->batch == 0 && p->num_seqs == 0);
}

KArgs make_args(const SbParams& p, const WsLayout& L) {
    KArgs a{};
    char* ws = (char*)p.fwd_workspace;
    a.hdr = (const WsHeader*)ws;
    a.seqs = (const SeqInfo*)(ws + L.off_seqs);
    a.items = (const int2*)(ws + L.off_items);
    a.carry_w = p.save_carries ? (float*)(ws + L.off_carry) : nullptr;
    a.carry_c = (float*)p.bwd_workspace;
    a.drem_eff = p.bwd_workspace ? (float*)((char*)p.bwd_workspace + L.off_drem) : nullptr;
    a.fused = (p.flags & SBATTN_FLAG_FUSED_REMAINDER) ? 1 : 0;
    a.tokens = p.tokens;
    a.drem_rows = (int64_t)p.tokens * (p.batch > 0 ? p.batch : 1);
    a.slot_cap = 2 * L.slot_cap;  // 32-key slots
    a.heads = p.heads;
    a.head_dim = p.head_dim;
    a.attend_current = p.attend_current ? 1 : 0;
    a.inv_temp = p.inv_temp;
    a.sched = ((WsHeader*)ws)->sched;
    {   // heads worked on together: their K and V (2 x T x D 16-bit values each) should fit in a third of the L2
        const int64_t per_head = (int64_t)p.tokens * p.head_dim * 4;
        int64_t g = per_head > 0 ? (40ll << 20) / per_head : 8;
        a.head_group = (int32_t)(g < 1 ? 1 : (g > 8 ? 8 : g));
    }
    {   // Packs of short sequences: the persistent kernels then overlap the end of one item with the start of the next.
        // The host knows the average length only (the ends live on the device), which is what decides.
        const int64_t n_seq = p.batch > 0 ? 1 : (p.num_seqs > 0 ? p.num_seqs : 1);
        const int64_t avg = (int64_t)p.tokens / n_seq;
        // (measured: the forward gains up to an average of a few thousand tokens, 1.4 % at 2 340, and loses 1.3 % on one
        // sequence of 16 384; the dq kernel loses from about a thousand tokens on, the dk/dv kernel from a few hundred)
        a.defer_fwd = avg <= 3072;
        a.defer_dq = avg <= 1024;
        a.defer_dkdv = avg <= 192;
    }
    a.q = view(p.q); a.k = view(p.k); a.v = view(p.v); a.o = view(p.o);
    a.d_o = view(p.d_o); a.dq = view(p.dq); a.dk = view(p.dk); a.dv = view(p.dv);
    a.rem = view(p.rem); a.nla = view(p.neg_log_acc); a.d_rem = view(p.d_rem);
    a.status = p.status;
    return a;
}

// 0: SIMT, 1: tensor, <0: error
int choose_path(const SbParams& p, bool backward) {
    if (p.path == SBATTN_PATH_SIMT) return 0;
    int why = SBATTN_EUNSUPPORTED;
    const bool ok = tensor_path_eligible(p, backward, &why);
    if (ok) return 1;
    return p.path == SBATTN_PATH_TENSOR ? why : 0;
}

}  // namespace

}  // namespace sb

using namespace sb;

extern "C" int sbattn_version(void) { return SBATTN_VERSION; }

extern "C" size_t sbattn_params_size(void) { return sizeof(SbParams); }

extern "C" unsigned long long sbattn_launch_count(void) { return __atomic_load_n(&g_launch_count, __ATOMIC_RELAXED); }

extern "C" const char* sbattn_strerror(int code) {
    switch (code) {
        case SBATTN_OK: return "ok";
        case SBATTN_EINVAL: return "invalid argument (sizes, strides or enum value)";
        case SBATTN_ENULL: return "required pointer is NULL";
        case SBATTN_EUNSUPPORTED: return "unsupported shape or dtype for the requested kernel path";
        case SBATTN_EWORKSPACE: return "workspace missing or too small";
        case SBATTN_EALIGN: return "tensor-core path needs 16-byte aligned pointers and strides";
        case SBATTN_ECUDA: return "CUDA call failed";
        case SBATTN_ECAPACITY: return "problem too large for the built-in scratch of sbattn_fwd_static";
        default: return "unknown sbattn error";
    }
}

extern "C" int sbattn_workspace_bytes(const SbParams* p, size_t* fwd_bytes, size_t* bwd_bytes) {
    int rc = check_shape(p);
    if (rc != SBATTN_OK) return rc;
    const WsLayout L = make_layout(*p);
    if (fwd_bytes) *fwd_bytes = L.fwd_bytes;
    if (bwd_bytes) *bwd_bytes = L.bwd_bytes;
    return SBATTN_OK;
}

extern "C" int sbattn_fwd(const SbParams* p) {
    int rc = check_shape(p);
    if (rc != SBATTN_OK) return rc;
    if (empty_problem(p)) return SBATTN_OK;
    if ((rc = check_mat(p->q, true)) || (rc = check_mat(p->k, true)) || (rc = check_mat(p->v, true)) ||
        (rc = check_mat(p->o, true)) || (rc = check_vec(p->rem, true)) || (rc = check_vec(p->neg_log_acc, true)))
        return rc;
    if (p->batch == 0 && !p->cu_seqlens) return SBATTN_ENULL;
    if (!p->status) return SBATTN_ENULL;
    const WsLayout L = make_layout(*p);
    if (!p->fwd_workspace || p->fwd_workspace_bytes < L.fwd_bytes) return SBATTN_EWORKSPACE;
    if (((uintptr_t)p->fwd_workspace & 255) != 0) return SBATTN_EWORKSPACE;
    const int path = choose_path(*p, false);
    if (path < 0) return path;
    if ((p->flags & SBATTN_FLAG_FUSED_REMAINDER) && path != 1) return SBATTN_EUNSUPPORTED;  // tensor-core kernels only
    cudaStream_t st = (cudaStream_t)p->stream;
    if (launch_prep(*p, L, st) != 0) return SBATTN_ECUDA;
    const KArgs a = make_args(*p, L);
    if (launch_zero_tail_rows(*p, a, st) != 0) return SBATTN_ECUDA;
    int e = path == 1 ? launch_tensor_fwd(*p, L, a, st) : launch_simt_fwd(*p, L, a, st);
    // a layout the tensor-map encoder refuses (nothing has been launched yet): the other kernels take any strides
    if (e == kMapEncodeFailed && p->path == SBATTN_PATH_AUTO && !(p->flags & SBATTN_FLAG_FUSED_REMAINDER))
        e = launch_simt_fwd(*p, L, a, st);
    return e == 0 ? SBATTN_OK : (e == kMapEncodeFailed ? SBATTN_EUNSUPPORTED : SBATTN_ECUDA);
}

extern "C" int sbattn_bwd(const SbParams* p) {
    int rc = check_shape(p);
    if (rc != SBATTN_OK) return rc;
    if (empty_problem(p)) return SBATTN_OK;
    if ((rc = check_mat(p->q, true)) || (rc = check_mat(p->k, true)) || (rc = check_mat(p->v, true)) ||
        (rc = check_mat(p->d_o, true)) || (rc = check_vec(p->d_rem, true)) || (rc = check_mat(p->dq, true)) ||
        (rc = check_mat(p->dk, true)) || (rc = check_mat(p->dv, true)))
        return rc;
    if (!p->status) return SBATTN_ENULL;
    if (!p->save_carries) return SBATTN_EINVAL;  // the forward must have been run with save_carries
    const WsLayout L = make_layout(*p);
    if (!p->fwd_workspace || p->fwd_workspace_bytes < L.fwd_bytes) return SBATTN_EWORKSPACE;
    if (!p->bwd_workspace || p->bwd_workspace_bytes < L.bwd_bytes) return SBATTN_EWORKSPACE;
    if (((uintptr_t)p->fwd_workspace & 255) != 0 || ((uintptr_t)p->bwd_workspace & 255) != 0) return SBATTN_EWORKSPACE;
    const int path = choose_path(*p, true);
    if (path < 0) return path;
    if (p->flags & SBATTN_FLAG_FUSED_REMAINDER) {
        if (path != 1) return SBATTN_EUNSUPPORTED;
        if ((rc = check_vec(p->rem, true))) return rc;  // the forward's rem: dv includes rem * d_o
    }
    cudaStream_t st = (cudaStream_t)p->stream;
    const KArgs a = make_args(*p, L);
    if (p->bwd_phases == SBATTN_BWD_ALL && launch_zero_tail(*p, a, st) != 0) return SBATTN_ECUDA;
    int e = path == 1 ? launch_tensor_bwd(*p, L, a, st) : launch_simt_bwd(*p, L, a, st);
    if (e == kMapEncodeFailed && p->path == SBATTN_PATH_AUTO && !(p->flags & SBATTN_FLAG_FUSED_REMAINDER))
        e = launch_simt_bwd(*p, L, a, st);
    return e == 0 ? SBATTN_OK : (e == kMapEncodeFailed ? SBATTN_EUNSUPPORTED : SBATTN_ECUDA);
}

extern "C" int sbattn_attention_weights(const SbParams* p, float* w, int64_t stride_b, int64_t stride_h, int64_t stride_m) {
    int rc = check_shape(p);
    if (rc != SBATTN_OK) return rc;
    if (empty_problem(p)) return SBATTN_OK;
    if ((rc = check_mat(p->q, true)) || (rc = check_mat(p->k, true))) return rc;
    if (!w) return SBATTN_ENULL;
    if (p->batch == 0 && !p->cu_seqlens) return SBATTN_ENULL;
    if (stride_b < 0 || stride_h < 0 || stride_m < p->tokens) return SBATTN_EINVAL;
    return launch_weights(*p, w, stride_b, stride_h, stride_m, (cudaStream_t)p->stream) == 0 ? SBATTN_OK : SBATTN_ECUDA;
}
