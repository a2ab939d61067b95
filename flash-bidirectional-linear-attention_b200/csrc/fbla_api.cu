// The C ABI of flash_bla_sm100: argument validation, kernel-path selection and the
// per-operator entry points declared in include/flash_bla_sm100.h.  Every entry
// point only enqueues kernels on the caller's stream.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "fbla_common.cuh"
#include "tc_kernels.cuh"

namespace fbla {
static std::atomic<unsigned long long> g_launches{0};
void note_launches(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
}  // namespace fbla

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(FBLA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

enum OpKind { OP_LINEAR, OP_SIMPLE, OP_DECOUPLED, OP_VARLEN };

// Validates the problem for one operator and resolves the kernel parameters.
int resolve(const fbla_problem* p, OpKind op, fbla::KParams* kp) {
    if (p == nullptr) return fail(FBLA_ERR_INVALID, "problem is NULL");
    if (p->dtype != FBLA_F32 && p->dtype != FBLA_BF16 && p->dtype != FBLA_F16)
        return fail(FBLA_ERR_INVALID, "dtype %d is not one of FBLA_F32/FBLA_BF16/FBLA_F16", p->dtype);
    if (p->dk < 1 || p->dk > 128 || p->dv < 1 || p->dv > 128)
        return fail(FBLA_ERR_UNSUPPORTED, "dk=%d, dv=%d: feature dims must be in [1, 128]", p->dk, p->dv);
    if (p->heads < 1) return fail(FBLA_ERR_INVALID, "heads=%d must be positive", p->heads);
    if (p->seq_len < 0) return fail(FBLA_ERR_INVALID, "seq_len=%lld is negative", (long long)p->seq_len);
    if (p->norm_len < 0) return fail(FBLA_ERR_INVALID, "norm_len=%lld is negative", (long long)p->norm_len);
    const bool want_norm = (op != OP_SIMPLE);
    if ((p->normalize != 0) != want_norm)
        return fail(FBLA_ERR_INVALID, "normalize=%d does not match this operator", p->normalize);
    kp->heads = p->heads;
    kp->dk = kp->mem_dk = p->dk;
    kp->dv = kp->mem_dv = p->dv;
    if (p->flags & FBLA_FLAG_NARROW) {
        const bool wide = (p->dk == 64 || p->dk == 128) && (p->dv == 64 || p->dv == 128);
        const bool op_ok = op == OP_LINEAR || op == OP_SIMPLE || op == OP_VARLEN ||
                           (op == OP_DECOUPLED && p->dk <= 64 && p->dv <= 64);
        if (p->dtype == FBLA_F32 || !op_ok || (p->dk % 16) || (p->dv % 16) || wide || (p->flags & FBLA_FLAG_GENERIC))
            return fail(FBLA_ERR_UNSUPPORTED, "FBLA_FLAG_NARROW serves 16-bit linear_attn (fixed or packed) / simple_la (and "
                        "decoupled_la up to 64) with feature dims that are multiples of 16 and not both 64 or 128 "
                        "(dk=%d, dv=%d)", p->dk, p->dv);
        kp->dk = p->dk <= 64 ? 64 : 128;        // the kernels' tile widths; the tensors keep theirs
        kp->dv = p->dv <= 64 ? 64 : 128;
    }
    kp->seq_len = p->seq_len;
    kp->scale = p->scale;
    kp->eps = p->eps;
    kp->normalize = p->normalize != 0;
    kp->inv_norm = p->norm_len > 0 ? (float)(1.0 / (double)p->norm_len) : 0.f;
    kp->state_stride = kp->dk * kp->dv + (kp->normalize ? kp->dk : 0);
    kp->unreduced = 0;
    if (op == OP_VARLEN) {
        if (p->cu_seqlens == nullptr) return fail(FBLA_ERR_INVALID, "cu_seqlens is NULL");
        if (p->num_seqs < 1) return fail(FBLA_ERR_INVALID, "num_seqs=%d must be positive", p->num_seqs);
        if (p->max_seqlen < 1) return fail(FBLA_ERR_INVALID, "max_seqlen=%d must be positive", p->max_seqlen);
        if ((int64_t)p->num_seqs * p->heads > 0x7fffffffLL || p->seq_len * (int64_t)p->heads > (1LL << 40))
            return fail(FBLA_ERR_UNSUPPORTED, "problem too large");
        kp->cu = p->cu_seqlens;
        kp->units = p->num_seqs * p->heads;
        kp->max_len = p->max_seqlen;
        kp->scale_per_seq = p->scale_per_seq != 0;
    } else {
        if (p->cu_seqlens != nullptr)
            return fail(FBLA_ERR_INVALID, "cu_seqlens given to a fixed-length operator");
        if (p->batch < 1) return fail(FBLA_ERR_INVALID, "batch=%d must be positive", p->batch);
        if ((int64_t)p->batch * p->heads > 0x7fffffffLL || p->seq_len > 0x7fffffffLL)
            return fail(FBLA_ERR_UNSUPPORTED, "problem too large");
        kp->cu = nullptr;
        kp->units = p->batch * p->heads;
        kp->max_len = (int)p->seq_len;
        kp->scale_per_seq = 0;
    }
    return FBLA_OK;
}

OpKind kind_of(const fbla_problem* p) {
    if (p != nullptr && p->cu_seqlens != nullptr) return OP_VARLEN;
    if (p != nullptr && !p->normalize) return OP_SIMPLE;
    return OP_LINEAR;
}

bool use_tc(const fbla_problem* p, const fbla::KParams& kp) {
    return !(p->flags & FBLA_FLAG_GENERIC) && fbla::tc_supported(kp, p->dtype);
}

// TMA needs 16-byte aligned tensors; anything else takes the CUDA-core kernels.
bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr,
               const void* e = nullptr, const void* f = nullptr) {
    const void* ps[6] = {a, b, c, d, e, f};
    for (const void* x : ps)
        if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;
    return true;
}

// The workspace must serve whichever kernel path the pass ends up taking.
int64_t workspace_need(const fbla_problem* p, const fbla::KParams& kp) {
    const int64_t simt = fbla::simt_workspace_bytes(kp);
    if (!use_tc(p, kp)) return simt;
    const int64_t tc = fbla::tc_workspace_bytes(kp);
    return tc > simt ? tc : simt;
}

int check_device_status() {
    const int s = fbla::tc_device_status();
    if (s != 0) return fail(FBLA_ERR_DEVICE, "a kernel gave up a bounded wait (site %d); results are invalid", s);
    return FBLA_OK;
}

#define NOT_NULL(x) \
    if ((x) == nullptr) return fail(FBLA_ERR_INVALID, #x " is NULL")

int check_ws(const fbla_problem* p, const fbla::KParams& kp, void* ws, size_t ws_bytes) {
    const int64_t need = workspace_need(p, kp);
    if (need > 0 && (ws == nullptr || (int64_t)ws_bytes < need))
        return fail(FBLA_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given", (long long)need,
                    (long long)(ws ? ws_bytes : 0));
    return FBLA_OK;
}

// Empty problems (no tokens, or no units) have nothing to launch, but the state must
// still be defined for the caller.
bool is_empty(const fbla::KParams& kp) { return kp.units == 0 || kp.seq_len == 0; }

const char* const kUnreducedNeedsTc = "the unreduced-state mode needs the tensor-core kernels (16-byte aligned tensors)";
const char* const kNarrowNeedsTc = "FBLA_FLAG_NARROW needs the tensor-core kernels (16-byte aligned tensors)";
bool narrow(const fbla::KParams& kp) { return kp.mem_dk != kp.dk || kp.mem_dv != kp.dv; }

int fwd_state(const fbla_problem* p, OpKind op, const void* k, const void* k_rope, const void* v,
              float* state, void* ws, size_t ws_bytes, fbla_stream_t stream, bool unreduced = false) {
    fbla::KParams kp;
    if (int rc = resolve(p, op, &kp)) return rc;
    kp.unreduced = unreduced;
    if (!unreduced) NOT_NULL(state);
    cudaStream_t st = (cudaStream_t)stream;
    if (is_empty(kp)) {
        cudaError_t e = cudaMemsetAsync(state, 0, sizeof(float) * (size_t)kp.units * kp.state_stride, st);
        return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "memset of the state");
    }
    NOT_NULL(k);
    NOT_NULL(v);
    if (int rc = check_ws(p, kp, ws, ws_bytes)) return rc;
    if (int rc = check_device_status()) return rc;
    const bool tc = use_tc(p, kp) && aligned16(k, k_rope, v, ws) && (op != OP_DECOUPLED || fbla::tc_supported_decoupled(kp));
    if (unreduced && !tc) return fail(FBLA_ERR_INVALID, kUnreducedNeedsTc);
    if (narrow(kp) && !tc) return fail(FBLA_ERR_UNSUPPORTED, kNarrowNeedsTc);
    cudaError_t e = tc ? fbla::tc_fwd_state(kp, p->dtype, k, k_rope, v, state, ws, st)
                       : fbla::simt_fwd_state(kp, p->dtype, k, k_rope, v, state, ws, st);
    return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "forward state pass");
}

int fwd_out(const fbla_problem* p, OpKind op, const void* q, const void* q_rope, const float* state, void* o,
            fbla_stream_t stream, bool unreduced = false) {
    fbla::KParams kp;
    if (int rc = resolve(p, op, &kp)) return rc;
    kp.unreduced = unreduced;
    if (is_empty(kp)) return FBLA_OK;
    NOT_NULL(q);
    NOT_NULL(state);
    NOT_NULL(o);
    cudaStream_t st = (cudaStream_t)stream;
    if (int rc = check_device_status()) return rc;
    const bool tc = use_tc(p, kp) && aligned16(q, q_rope, o) && (op != OP_DECOUPLED || fbla::tc_supported_decoupled(kp));
    if (unreduced && !tc) return fail(FBLA_ERR_INVALID, kUnreducedNeedsTc);
    if (narrow(kp) && !tc) return fail(FBLA_ERR_UNSUPPORTED, kNarrowNeedsTc);
    cudaError_t e = tc ? fbla::tc_fwd_out(kp, p->dtype, q, q_rope, state, o, st)
                       : fbla::simt_fwd_out(kp, p->dtype, q, q_rope, state, o, st);
    return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "forward output pass");
}

int bwd_state(const fbla_problem* p, OpKind op, const void* q, const void* q_rope, const void* d_o,
              const float* state, void* dq, void* dq_rope, float* dstate, void* ws, size_t ws_bytes,
              fbla_stream_t stream, bool unreduced = false) {
    fbla::KParams kp;
    if (int rc = resolve(p, op, &kp)) return rc;
    kp.unreduced = unreduced;
    if (!unreduced) NOT_NULL(dstate);
    cudaStream_t st = (cudaStream_t)stream;
    if (is_empty(kp)) {
        if (dstate == nullptr) return FBLA_OK;
        cudaError_t e = cudaMemsetAsync(dstate, 0, sizeof(float) * (size_t)kp.units * kp.state_stride, st);
        return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "memset of the state gradient");
    }
    NOT_NULL(q);
    NOT_NULL(d_o);
    NOT_NULL(state);
    NOT_NULL(dq);
    if (op == OP_DECOUPLED) {
        NOT_NULL(q_rope);
        NOT_NULL(dq_rope);
    }
    if (int rc = check_ws(p, kp, ws, ws_bytes)) return rc;
    if (int rc = check_device_status()) return rc;
    const bool tc = use_tc(p, kp) && aligned16(q, q_rope, d_o, dq, dq_rope, ws) &&
                    (op != OP_DECOUPLED || fbla::tc_supported_decoupled(kp));
    if (unreduced && !tc) return fail(FBLA_ERR_INVALID, kUnreducedNeedsTc);
    if (narrow(kp) && !tc) return fail(FBLA_ERR_UNSUPPORTED, kNarrowNeedsTc);
    cudaError_t e = tc ? fbla::tc_bwd_state(kp, p->dtype, q, q_rope, d_o, state, dq, dq_rope, dstate, ws, st)
                       : fbla::simt_bwd_state(kp, p->dtype, q, q_rope, d_o, state, dq, dq_rope, dstate, ws, st);
    return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "backward state pass");
}

int bwd_in(const fbla_problem* p, OpKind op, const void* k_rope, const void* v, const float* dstate, void* dk,
           void* dk_rope, void* dv, fbla_stream_t stream, bool unreduced = false) {
    fbla::KParams kp;
    if (int rc = resolve(p, op, &kp)) return rc;
    kp.unreduced = unreduced;
    if (is_empty(kp)) return FBLA_OK;
    NOT_NULL(k_rope);
    NOT_NULL(v);
    NOT_NULL(dstate);
    NOT_NULL(dk);
    NOT_NULL(dv);
    if (op == OP_DECOUPLED) NOT_NULL(dk_rope);
    cudaStream_t st = (cudaStream_t)stream;
    if (int rc = check_device_status()) return rc;
    const bool tc = use_tc(p, kp) && aligned16(k_rope, v, dk, dk_rope, dv) &&
                    (op != OP_DECOUPLED || fbla::tc_supported_decoupled(kp));
    if (unreduced && !tc) return fail(FBLA_ERR_INVALID, kUnreducedNeedsTc);
    if (narrow(kp) && !tc) return fail(FBLA_ERR_UNSUPPORTED, kNarrowNeedsTc);
    cudaError_t e = tc ? fbla::tc_bwd_in(kp, p->dtype, k_rope, v, dstate, dk, dk_rope, dv, st)
                       : fbla::simt_bwd_in(kp, p->dtype, k_rope, v, dstate, dk, dk_rope, dv, st);
    return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "backward input pass");
}

}  // namespace

namespace fbla {
int api_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
int api_resolve_linear(const fbla_problem* p, KParams* kp) { return resolve(p, OP_LINEAR, kp); }
}  // namespace fbla

extern "C" {

int fbla_version(void) { return FBLA_ABI_VERSION; }

const char* fbla_last_error(void) { return g_err; }

uint64_t fbla_launch_count(void) { return fbla::g_launches.load(std::memory_order_relaxed); }

int64_t fbla_state_floats(const fbla_problem* p) {
    fbla::KParams kp;
    if (resolve(p, kind_of(p), &kp)) return -1;
    return (int64_t)kp.units * kp.state_stride;
}

int64_t fbla_workspace_bytes(const fbla_problem* p) {
    fbla::KParams kp;
    if (resolve(p, kind_of(p), &kp)) return -1;
    if (is_empty(kp)) return 0;
    return workspace_need(p, kp);
}

int fbla_kernel_path(const fbla_problem* p) {
    fbla::KParams kp;
    if (resolve(p, kind_of(p), &kp)) return -1;
    return use_tc(p, kp) ? 1 : 0;
}

// ---- linear_attention ------------------------------------------------------------------
int fbla_linear_attn_fwd_state(const fbla_problem* p, const void* k, const void* v, float* state, void* ws,
                               size_t ws_bytes, fbla_stream_t s) {
    return fwd_state(p, OP_LINEAR, k, nullptr, v, state, ws, ws_bytes, s);
}
int fbla_linear_attn_fwd_out(const fbla_problem* p, const void* q, const float* state, void* o,
                             fbla_stream_t s) {
    return fwd_out(p, OP_LINEAR, q, nullptr, state, o, s);
}
int fbla_linear_attn_bwd_state(const fbla_problem* p, const void* q, const void* d_o, const float* state,
                               void* dq, float* dstate, void* ws, size_t ws_bytes, fbla_stream_t s) {
    return bwd_state(p, OP_LINEAR, q, nullptr, d_o, state, dq, nullptr, dstate, ws, ws_bytes, s);
}
int fbla_linear_attn_bwd_in(const fbla_problem* p, const void* k, const void* v, const float* dstate, void* dk,
                            void* dv, fbla_stream_t s) {
    return bwd_in(p, OP_LINEAR, k, v, dstate, dk, nullptr, dv, s);
}

// ---- simple_la -------------------------------------------------------------------------
int fbla_simple_la_fwd_state(const fbla_problem* p, const void* k, const void* v, float* state, void* ws,
                             size_t ws_bytes, fbla_stream_t s) {
    return fwd_state(p, OP_SIMPLE, k, nullptr, v, state, ws, ws_bytes, s);
}
int fbla_simple_la_fwd_out(const fbla_problem* p, const void* q, const float* state, void* o, fbla_stream_t s) {
    return fwd_out(p, OP_SIMPLE, q, nullptr, state, o, s);
}
int fbla_simple_la_bwd_state(const fbla_problem* p, const void* q, const void* d_o, const float* state,
                             void* dq, float* dstate, void* ws, size_t ws_bytes, fbla_stream_t s) {
    return bwd_state(p, OP_SIMPLE, q, nullptr, d_o, state, dq, nullptr, dstate, ws, ws_bytes, s);
}
int fbla_simple_la_bwd_in(const fbla_problem* p, const void* k, const void* v, const float* dstate, void* dk,
                          void* dv, fbla_stream_t s) {
    return bwd_in(p, OP_SIMPLE, k, v, dstate, dk, nullptr, dv, s);
}

// ---- decoupled_la ----------------------------------------------------------------------
int fbla_decoupled_la_fwd_state(const fbla_problem* p, const void* k, const void* k_rope, const void* v,
                                float* state, void* ws, size_t ws_bytes, fbla_stream_t s) {
    if (k_rope == nullptr) return fail(FBLA_ERR_INVALID, "k_rope is NULL");
    return fwd_state(p, OP_DECOUPLED, k, k_rope, v, state, ws, ws_bytes, s);
}
int fbla_decoupled_la_fwd_out(const fbla_problem* p, const void* q, const void* q_rope, const float* state,
                              void* o, fbla_stream_t s) {
    if (q_rope == nullptr) return fail(FBLA_ERR_INVALID, "q_rope is NULL");
    return fwd_out(p, OP_DECOUPLED, q, q_rope, state, o, s);
}
int fbla_decoupled_la_bwd_state(const fbla_problem* p, const void* q, const void* q_rope, const void* d_o,
                                const float* state, void* dq, void* dq_rope, float* dstate, void* ws,
                                size_t ws_bytes, fbla_stream_t s) {
    return bwd_state(p, OP_DECOUPLED, q, q_rope, d_o, state, dq, dq_rope, dstate, ws, ws_bytes, s);
}
int fbla_decoupled_la_bwd_in(const fbla_problem* p, const void* k_rope, const void* v, const float* dstate,
                             void* dk, void* dk_rope, void* dv, fbla_stream_t s) {
    return bwd_in(p, OP_DECOUPLED, k_rope, v, dstate, dk, dk_rope, dv, s);
}

// ---- both passes of a direction in one call (saves a host round trip per pass) -----------
int fbla_unreduced_state(const fbla_problem* p) {
    if (p == nullptr || !(p->flags & FBLA_FLAG_UNREDUCED)) return 0;
    const OpKind op = kind_of(p);
    fbla::KParams kp;
    if (op == OP_VARLEN || resolve(p, op, &kp) != FBLA_OK) return 0;
    return (use_tc(p, kp) && !is_empty(kp) && workspace_need(p, kp) > 0) ? 1 : 0;
}
int fbla_linear_attn_fwd(const fbla_problem* p, const void* q, const void* k, const void* v, void* o, float* state,
                         void* ws, size_t ws_bytes, fbla_stream_t s) {
    const OpKind op = kind_of(p);
    const bool u = fbla_unreduced_state(p) != 0;
    if (int rc = fwd_state(p, op, k, nullptr, v, state, ws, ws_bytes, s, u)) return rc;
    return fwd_out(p, op, q, nullptr, u ? static_cast<const float*>(ws) : state, o, s, u);
}
int fbla_linear_attn_bwd(const fbla_problem* p, const void* q, const void* k, const void* v, const void* d_o,
                         const float* state, void* dq, void* dk, void* dv, float* dstate, void* ws, size_t ws_bytes,
                         fbla_stream_t s) {
    const OpKind op = kind_of(p);
    const bool u = fbla_unreduced_state(p) != 0;
    if (int rc = bwd_state(p, op, q, nullptr, d_o, state, dq, nullptr, dstate, ws, ws_bytes, s, u)) return rc;
    return bwd_in(p, op, k, v, u ? static_cast<const float*>(ws) : dstate, dk, nullptr, dv, s, u);
}

// ---- sequence-sharded calls on the tensor-core kernels ------------------------------------------
namespace {

OpKind sharded_kind(const fbla_problem* p, const void* rope) {
    if (p != nullptr && !p->normalize) return OP_SIMPLE;
    return rope != nullptr ? OP_DECOUPLED : OP_LINEAR;
}

// Validates the group and the problem for the sequence-sharded calls and resolves both.
int resolve_sharded(const fbla_problem* p, OpKind op, const fbla_peer_group* g, fbla::KParams* kp, fbla::PeerArgs* pa) {
    if (int rc = resolve(p, op, kp)) return rc;
    if (g == nullptr) return fail(FBLA_ERR_INVALID, "group is NULL");
    if (g->world < 2 || g->world > 8 || g->rank < 0 || g->rank >= g->world)
        return fail(FBLA_ERR_INVALID, "world %d / rank %d out of range (2 to 8 ranks)", g->world, g->rank);
    if (g->epoch == 0) return fail(FBLA_ERR_INVALID, "epoch must start at 1");
    if (g->parts == nullptr || g->full == nullptr || g->flags == nullptr)
        return fail(FBLA_ERR_INVALID, "a pointer table of the group is NULL");
    if (p->cu_seqlens != nullptr || is_empty(*kp) || !use_tc(p, *kp) ||
        (op == OP_DECOUPLED && !fbla::tc_supported_decoupled(*kp)))
        return fail(FBLA_ERR_UNSUPPORTED,
                    "the sequence-sharded calls serve what the tensor-core kernels serve (fixed length, 16-bit, "
                    "dk, dv in {64, 128}, decoupled at 64 x 64, at least one token)");
    pa->world = g->world;
    pa->rank = g->rank;
    pa->epoch = g->epoch;
    for (int r = 0; r < g->world; ++r) {
        if (g->parts[r] == nullptr || g->full[r] == nullptr || g->flags[r] == nullptr)
            return fail(FBLA_ERR_INVALID, "rank %d: NULL buffer or flag pointer", r);
        if (((reinterpret_cast<uintptr_t>(g->parts[r]) | reinterpret_cast<uintptr_t>(g->full[r])) & 15u) != 0 ||
            (reinterpret_cast<uintptr_t>(g->flags[r]) & 3u) != 0)
            return fail(FBLA_ERR_INVALID, "rank %d: buffers must be 16-byte aligned", r);
        pa->parts[r] = g->parts[r];
        pa->full[r] = g->full[r];
        pa->flags[r] = g->flags[r];
    }
    return check_device_status();
}

const char* const kShardedAlign = "the sequence-sharded calls need 16-byte aligned tensors";

}  // namespace

int fbla_seq_sharded_supported(const fbla_problem* p) {
    fbla::KParams kp;
    if (p == nullptr || p->cu_seqlens != nullptr || resolve(p, kind_of(p), &kp) != FBLA_OK) return 0;
    return (!is_empty(kp) && use_tc(p, kp)) ? 1 : 0;
}

int64_t fbla_seq_sharded_part_floats(const fbla_problem* p) {
    fbla::KParams kp;
    if (!fbla_seq_sharded_supported(p) || resolve(p, kind_of(p), &kp) != FBLA_OK) return -1;
    return fbla::tc_workspace_bytes(kp) / (int64_t)sizeof(float);
}

int fbla_seq_sharded_fwd_state(const fbla_problem* p, const void* k, const void* k_rope, const void* v,
                               const fbla_peer_group* g, fbla_stream_t s) {
    fbla::KParams kp;
    fbla::PeerArgs pa;
    const OpKind op = sharded_kind(p, k_rope);
    if (int rc = resolve_sharded(p, op, g, &kp, &pa)) return rc;
    NOT_NULL(k);
    NOT_NULL(v);
    if (!aligned16(k, k_rope, v)) return fail(FBLA_ERR_UNSUPPORTED, kShardedAlign);
    kp.unreduced = 1;           // the pieces in this rank's piece buffer are the result
    const cudaError_t e = fbla::tc_fwd_state(kp, p->dtype, k, k_rope, v, nullptr, pa.parts[pa.rank], (cudaStream_t)s);
    return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "forward state pass (sequence-sharded)");
}

int fbla_seq_sharded_bwd_state(const fbla_problem* p, const void* q, const void* q_rope, const void* d_o,
                               const float* state, const fbla_peer_group* g, void* dq, void* dq_rope,
                               fbla_stream_t s) {
    fbla::KParams kp;
    fbla::PeerArgs pa;
    const OpKind op = sharded_kind(p, q_rope);
    if (int rc = resolve_sharded(p, op, g, &kp, &pa)) return rc;
    NOT_NULL(q);
    NOT_NULL(d_o);
    NOT_NULL(state);
    NOT_NULL(dq);
    if (op == OP_DECOUPLED) NOT_NULL(dq_rope);
    if (!aligned16(q, q_rope, d_o, dq, dq_rope, state)) return fail(FBLA_ERR_UNSUPPORTED, kShardedAlign);
    // the state it reads is an ordinary reduced one; the pieces of the state GRADIENT stay unreduced
    kp.unreduced = 2;
    const cudaError_t e = fbla::tc_bwd_state(kp, p->dtype, q, q_rope, d_o, state, dq, dq_rope, nullptr, pa.parts[pa.rank],
                                             (cudaStream_t)s);
    return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "backward state pass (sequence-sharded)");
}

int fbla_seq_sharded_exchange(const fbla_problem* p, const fbla_peer_group* g, float* state_out, fbla_stream_t s) {
    fbla::KParams kp;
    fbla::PeerArgs pa;
    if (int rc = resolve_sharded(p, kind_of(p), g, &kp, &pa)) return rc;
    NOT_NULL(state_out);
    if (!aligned16(state_out)) return fail(FBLA_ERR_INVALID, "state_out must be 16-byte aligned");
    static const int forced = [] {
        const char* e = getenv("FBLA_PEER_TWO_ROUND");
        return e == nullptr ? -1 : (e[0] == '1' ? 1 : 0);
    }();
    const int two_round = forced >= 0 ? forced : 1;
    const cudaError_t e = fbla::peer_piece_sum(pa, fbla::tc_piece_layout(kp), kp.state_stride, two_round, state_out,
                                               (cudaStream_t)s);
    return e == cudaSuccess ? FBLA_OK : cuda_fail(e, "state exchange (sequence-sharded)");
}

int fbla_device_status(void) { return fbla::tc_device_status(); }
void fbla_clear_device_status(void) { fbla::tc_clear_device_status(); }

// ---- varlen_linear_attention -----------------------------------------------------------
int fbla_varlen_linear_attn_fwd_state(const fbla_problem* p, const void* k, const void* v, float* state,
                                      void* ws, size_t ws_bytes, fbla_stream_t s) {
    return fwd_state(p, OP_VARLEN, k, nullptr, v, state, ws, ws_bytes, s);
}
int fbla_varlen_linear_attn_fwd_out(const fbla_problem* p, const void* q, const float* state, void* o,
                                    fbla_stream_t s) {
    return fwd_out(p, OP_VARLEN, q, nullptr, state, o, s);
}
int fbla_varlen_linear_attn_bwd_state(const fbla_problem* p, const void* q, const void* d_o, const float* state,
                                      void* dq, float* dstate, void* ws, size_t ws_bytes, fbla_stream_t s) {
    return bwd_state(p, OP_VARLEN, q, nullptr, d_o, state, dq, nullptr, dstate, ws, ws_bytes, s);
}
int fbla_varlen_linear_attn_bwd_in(const fbla_problem* p, const void* k, const void* v, const float* dstate,
                                   void* dk, void* dv, fbla_stream_t s) {
    return bwd_in(p, OP_VARLEN, k, v, dstate, dk, nullptr, dv, s);
}

}  // extern "C"
