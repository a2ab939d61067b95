/*
 * flash_bla_sm100 -- C ABI of the B200 (sm_100a) bidirectional linear-attention library.
 *
 * Every operator of the reference is a pair of streaming passes per direction:
 *   forward   pass 1 (fwd_state): reduce over tokens into the per-(batch, head) state
 *                                 [ S = K^T V  |  sum_t k ]            (fp32)
 *             pass 2 (fwd_out)  : stream over tokens, o = scale * q S / (q . ksum/L + eps)
 *   backward  pass 1 (bwd_state): stream over tokens, write dq, reduce into
 *                                 [ dS = (q/z)^T dO  |  sum_t dz q ]    (fp32)
 *             pass 2 (bwd_in)   : stream over tokens, write dk, dv
 * The split into *_state / *_out entry points is what lets a caller that shards the
 * sequence over several GPUs all-reduce the state between the two passes.
 *
 * Conventions
 *   - plain pointers and sizes only; all tensor pointers are DEVICE pointers of the
 *     element type named by fbla_problem.dtype, contiguous in the layout stated below;
 *   - state / dstate buffers are fp32, fbla_state_floats() elements, caller-allocated;
 *   - the workspace is caller-allocated scratch of fbla_workspace_bytes() bytes (may be
 *     NULL when that returns 0); its contents need not be initialised;
 *   - every call only enqueues work on `stream` (a cudaStream_t) and returns; no call
 *     synchronises the device;
 *   - return value: FBLA_OK or an error code; fbla_last_error() gives the text for the
 *     calling thread.  No C++ exception crosses this boundary and nothing here exits.
 *   - there is no CPU fallback: a call on a machine without a CUDA device fails.
 *
 * Layouts
 *   fixed length : q, k, q_rope, k_rope  (batch, heads, seq_len, dk)
 *                  v, o, d_o             (batch, heads, seq_len, dv)
 *   varlen       : q, k (total_tokens, heads, dk); v, o, d_o (total_tokens, heads, dv);
 *                  cu_seqlens int32 [num_seqs + 1] on the device
 *   state        : per unit u (u = b*heads + h, varlen: u = seq*heads + h):
 *                  dk*dv floats of S (row-major dk x dv) followed, when normalize != 0,
 *                  by dk floats of the key sum.  dstate has the same shape.
 */
#ifndef FLASH_BLA_SM100_H
#define FLASH_BLA_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FBLA_ABI_VERSION 2

enum fbla_dtype { FBLA_F32 = 0, FBLA_BF16 = 1, FBLA_F16 = 2 };

enum fbla_status {
    FBLA_OK = 0,
    FBLA_ERR_INVALID = 1,      /* bad argument (null pointer, size out of range, ...) */
    FBLA_ERR_UNSUPPORTED = 2,  /* valid request this build has no kernel for          */
    FBLA_ERR_CUDA = 3,         /* a CUDA runtime / driver call failed                 */
    FBLA_ERR_WORKSPACE = 4,    /* workspace missing or too small                      */
    FBLA_ERR_DEVICE = 5        /* a kernel reported a device-side error status        */
};

enum fbla_flags {
    FBLA_FLAG_GENERIC = 1,     /* force the CUDA-core (fp32 FMA) kernels              */
    FBLA_FLAG_UNREDUCED = 2,   /* fbla_linear_attn_fwd / _bwd: see fbla_unreduced_state() */
    FBLA_FLAG_NARROW = 4       /* 16-bit linear_attn (fixed or packed) / simple_la (decoupled_la up to 64), feature dims: multiples
                                * of 16, at most 128 and not both 64 or 128 (the reference's layers use 32): served
                                * by the 64- / 128-wide tensor-core kernels, whose TMA boxes zero-fill the missing
                                * features on loads and clip them on stores, so the tensors are read and written
                                * once at their own width.  All tensors 16-byte aligned.  State, dstate and the
                                * workspace have the sizes of the widened problem (ask fbla_state_floats /
                                * fbla_workspace_bytes with the same flags).                                   */
};

typedef struct fbla_problem {
    int32_t dtype;          /* enum fbla_dtype                                              */
    int32_t batch;          /* B; 1 for varlen                                              */
    int32_t heads;          /* H                                                            */
    int32_t dk;             /* key / query feature dim                                      */
    int32_t dv;             /* value feature dim                                            */
    int64_t seq_len;        /* tokens per (batch, head) held by this call; varlen: total    */
    int64_t norm_len;       /* length the key sum is divided by; 0 means seq_len (varlen:   */
                            /* each sequence's own length).  A caller that shards the       */
                            /* sequence passes the global length here.                      */
    const int32_t *cu_seqlens; /* device int32 [num_seqs+1]; NULL selects fixed length      */
    int32_t num_seqs;       /* varlen only                                                  */
    int32_t max_seqlen;     /* varlen only: an upper bound on the sequence lengths          */
    float scale;            /* multiplies V inside the state                                */
    int32_t scale_per_seq;  /* varlen only: use 1/length of each sequence, ignore `scale`   */
    float eps;              /* added to the normaliser                                      */
    int32_t normalize;      /* 1: o = q S / (q.kmean + eps);  0: o = q S  (simple_la)       */
    int32_t flags;          /* enum fbla_flags                                              */
} fbla_problem;

typedef void *fbla_stream_t; /* a cudaStream_t */

/* ---- library ------------------------------------------------------------------------ */
int fbla_version(void);
const char *fbla_last_error(void);
/* Kernels this library has launched in this process so far (all threads, all devices): a
 * measurement aid, no counterpart in the reference.                                      */
uint64_t fbla_launch_count(void);
/* Number of fp32 elements of one state (or dstate) buffer for this problem; <0 on error. */
int64_t fbla_state_floats(const fbla_problem *p);
/* Bytes of scratch the *_state passes need for this problem; <0 on error.                */
int64_t fbla_workspace_bytes(const fbla_problem *p);
/* 1 when the tensor-core (tcgen05 + TMA) kernels serve this problem, 0 when the CUDA-core
 * kernels do, <0 on error.                                                               */
int fbla_kernel_path(const fbla_problem *p);

/* ---- linear_attention (normalised) ---------------------------------------------------
 * Replaces the kernels launched by LinearAttnFunction.forward / .backward,
 * flash_bla/ops/linear_attn/fused.py:350-398 and :400-453 (kernels :27-88, :103-165,
 * :169-266, :270-347).  p->normalize must be 1.                                          */
int fbla_linear_attn_fwd_state(const fbla_problem *p, const void *k, const void *v,
                               float *state, void *workspace, size_t workspace_bytes,
                               fbla_stream_t stream);
int fbla_linear_attn_fwd_out(const fbla_problem *p, const void *q, const float *state,
                             void *o, fbla_stream_t stream);
int fbla_linear_attn_bwd_state(const fbla_problem *p, const void *q, const void *d_o,
                               const float *state, void *dq, float *dstate,
                               void *workspace, size_t workspace_bytes, fbla_stream_t stream);
int fbla_linear_attn_bwd_in(const fbla_problem *p, const void *k, const void *v,
                            const float *dstate, void *dk, void *dv, fbla_stream_t stream);

/* Both passes of one direction in a single call, for callers on one GPU (nothing to exchange
 * between the passes): forward = fwd_state + fwd_out, backward = bwd_state + bwd_in.  They serve
 * linear_attention, simple_la (normalize = 0) and varlen_linear_attention (cu_seqlens set) alike;
 * `state` / `dstate` are outputs of the first pass and inputs of the second.
 *
 * With FBLA_FLAG_UNREDUCED in p->flags and fbla_unreduced_state(p) == 1 (tensor-core kernels,
 * fixed length) the state is never reduced to one vector per unit: the reducing pass leaves its
 * per-segment pieces in the workspace and the consuming pass adds them while it stages the state
 * (same order, same bits), which saves one kernel per direction.  Then
 *   fbla_linear_attn_fwd: `state` is not written (may be NULL); the WORKSPACE holds the state and
 *                         must be kept for the backward;
 *   fbla_linear_attn_bwd: `state` is that forward workspace; `dstate` is not written (may be NULL).
 * When fbla_unreduced_state(p) is 0 the flag has no effect.                                     */
int fbla_unreduced_state(const fbla_problem *p);
int fbla_linear_attn_fwd(const fbla_problem *p, const void *q, const void *k, const void *v, void *o,
                         float *state, void *workspace, size_t workspace_bytes, fbla_stream_t stream);
int fbla_linear_attn_bwd(const fbla_problem *p, const void *q, const void *k, const void *v,
                         const void *d_o, const float *state, void *dq, void *dk, void *dv,
                         float *dstate, void *workspace, size_t workspace_bytes, fbla_stream_t stream);

/* Forward state pass for callers that cannot hand over a workspace and must not allocate: same
 * result as fbla_linear_attn_fwd_state, with the scratch in an 8 MiB device array inside the
 * library (held by every GPU that loads it).  No counterpart in the reference.  Refuses problems
 * that the tensor-core kernels do not serve or whose tensor-core scratch (one fp32 state per
 * segment of the tile schedule, at most fbla_workspace_bytes()) exceeds 8 MiB.  The
 * first call on a device resolves the array's address and should precede any stream capture;
 * calls that overlap on the GPU race on the shared array.                                   */
int fbla_linear_attn_fwd_state_noalloc(const fbla_problem *p, const void *k, const void *v,
                                       float *state, fbla_stream_t stream);
/* The status word of that entry point on the current device: *value = 0 when none of its kernels
 * gave up a bounded wait, else the number of the wait; clear != 0 resets it.  Synchronises the
 * device (two 4-byte copies), allocates nothing.  Once a failure has been read, the entry point
 * above returns FBLA_ERR_DEVICE until it is cleared.  No counterpart in the reference.        */
int fbla_noalloc_status(int *value, int clear);

/* ---- simple_la (no normaliser) -------------------------------------------------------
 * Replaces SimpleLinearAttnFunction.forward / .backward,
 * flash_bla/ops/simple_la/fused.py:495-535 and :539-626 (kernels :26-79, :94-145,
 * :160-211, :324-426).  p->normalize must be 0.                                          */
int fbla_simple_la_fwd_state(const fbla_problem *p, const void *k, const void *v,
                             float *state, void *workspace, size_t workspace_bytes,
                             fbla_stream_t stream);
int fbla_simple_la_fwd_out(const fbla_problem *p, const void *q, const float *state,
                           void *o, fbla_stream_t stream);
int fbla_simple_la_bwd_state(const fbla_problem *p, const void *q, const void *d_o,
                             const float *state, void *dq, float *dstate,
                             void *workspace, size_t workspace_bytes, fbla_stream_t stream);
int fbla_simple_la_bwd_in(const fbla_problem *p, const void *k, const void *v,
                          const float *dstate, void *dk, void *dv, fbla_stream_t stream);

/* ---- decoupled_la (rotary numerator, plain normaliser) -------------------------------
 * Replaces DecoupledLAFunction.forward / .backward,
 * flash_bla/ops/linear_attn/decoupled.py:411-509 (kernels :27-100, :115-190, :194-316,
 * :320-408).  State = [ k_rope^T v | sum_t k ].  p->normalize must be 1.                  */
int fbla_decoupled_la_fwd_state(const fbla_problem *p, const void *k, const void *k_rope,
                                const void *v, float *state, void *workspace,
                                size_t workspace_bytes, fbla_stream_t stream);
int fbla_decoupled_la_fwd_out(const fbla_problem *p, const void *q, const void *q_rope,
                              const float *state, void *o, fbla_stream_t stream);
int fbla_decoupled_la_bwd_state(const fbla_problem *p, const void *q, const void *q_rope,
                                const void *d_o, const float *state, void *dq, void *dq_rope,
                                float *dstate, void *workspace, size_t workspace_bytes,
                                fbla_stream_t stream);
int fbla_decoupled_la_bwd_in(const fbla_problem *p, const void *k_rope, const void *v,
                             const float *dstate, void *dk, void *dk_rope, void *dv,
                             fbla_stream_t stream);

/* ---- varlen_linear_attention (packed sequences, cu_seqlens) --------------------------
 * Replaces VarlenLinearAttnFunction.forward / .backward,
 * flash_bla/ops/linear_attn/varlen.py:335-422 and :426-505 (kernels :30-88, :96-149,
 * :157-224, :232-332).  p->cu_seqlens must be set; p->normalize must be 1.               */
int fbla_varlen_linear_attn_fwd_state(const fbla_problem *p, const void *k, const void *v,
                                      float *state, void *workspace, size_t workspace_bytes,
                                      fbla_stream_t stream);
int fbla_varlen_linear_attn_fwd_out(const fbla_problem *p, const void *q, const float *state,
                                    void *o, fbla_stream_t stream);
int fbla_varlen_linear_attn_bwd_state(const fbla_problem *p, const void *q, const void *d_o,
                                      const float *state, void *dq, float *dstate,
                                      void *workspace, size_t workspace_bytes,
                                      fbla_stream_t stream);
int fbla_varlen_linear_attn_bwd_in(const fbla_problem *p, const void *k, const void *v,
                                   const float *dstate, void *dk, void *dv,
                                   fbla_stream_t stream);

/* ---- piecewise_sparse_attention (PISA) ------------------------------------------------
 * Softmax attention approximated piecewise: exact on the `num_selected` key blocks chosen per
 * query block, zeroth order (block means / sums) plus a global first-order term on the rest.
 * Replaces fused_chunk_reduce + fused_chunk_reduce_kernel
 * (flash_bla/ops/piecewise_attn/kernel.py:152-176, :89-128) and
 * piecewise_sparse_attention_fwd_kernel (:189-292).  The block scores and the top-k selection
 * between the two calls stay with the caller, as in the reference (:313-318).
 *   q, k (batch, heads, seq_len, dk), v, o (batch, heads, seq_len, dv); block statistics fp32:
 *   qc, kc (batch, heads, NT, dk) block means; vc (batch, heads, NT, dv) block sums;
 *   kv (batch, heads, dk, dv) = K^T V (the state of fbla_simple_la_fwd_state);
 *   h (batch, heads, dk, dv) = kv - sum_c kc_c (x) vc_c = sum_c (K_c - kc_c)^T V_c;
 *   indices int32 (batch, heads, NT, num_selected); NT = ceil(seq_len / block_size).
 *   row_stats fp32 (batch, heads, seq_len, 4): running max (log2 domain), denominator, g, 1/denominator;
 *   may be NULL when no backward follows.                                                   */
typedef struct fbla_pisa_problem {
    int32_t dtype;          /* enum fbla_dtype of q, k, v, o                        */
    int32_t batch, heads;
    int32_t dk, dv;         /* 1..128                                               */
    int32_t block_size;     /* tokens per block, 1..128                             */
    int32_t num_selected;   /* key blocks attended exactly per query block          */
    int64_t seq_len;
    float scale;            /* logit scale (reference default dk^-0.5)              */
} fbla_pisa_problem;

int fbla_pisa_block_stats(const fbla_pisa_problem *p, const void *q, const void *k, const void *v,
                          float *qc, float *kc, float *vc, fbla_stream_t stream);
/* hnorm (batch, heads, NT) fp32: p-norm (order `pnorm` > 0) of each block's first-order state
 * (K_c - kc_c)^T V_c over its dk*dv entries -- the selection bias of use_bias=True
 * (kernel.py:118 and :172-173, where the reference materialises all the per-block states).    */
int fbla_pisa_block_hnorm(const fbla_pisa_problem *p, const void *k, const void *v, const float *kc,
                          float pnorm, float *hnorm, fbla_stream_t stream);
/* Block selection: indices int32 (batch, heads, NT, num_selected) of the num_selected highest-scoring
 * key blocks per query block, in descending order of score.  score = qc . (kc * scale), operands and
 * result rounded to p->dtype as the reference forms them (kernel.py:313); with hnorm (may be NULL) the
 * score is score + log(hnorm + 1e-5), which ranks as the reference's softmax of it does
 * (kernel.py:314-315).  Replaces the einsum / softmax / topk between the reference's two kernels
 * (kernel.py:313-318); equal scores go to the lower block index.  Up to 1024 blocks.          */
int fbla_pisa_select_blocks(const fbla_pisa_problem *p, const float *qc, const float *kc,
                            const float *hnorm, int32_t *indices, fbla_stream_t stream);
int fbla_pisa_first_order_state(const fbla_pisa_problem *p, const float *kv, const float *kc,
                                const float *vc, float *h, fbla_stream_t stream);
int fbla_pisa_fwd(const fbla_pisa_problem *p, const void *q, const void *k, const void *v,
                  const float *kc, const float *vc, const float *h, const int32_t *indices,
                  void *o, float *row_stats, fbla_stream_t stream);

/* fbla_pisa_fwd on the tcgen05 tensor cores (TMEM accumulators, operands by TMA) for 16-bit inputs
 * with dk = dv in {64, 128}, block_size 64 and up to 2048 blocks: the caller passes 128-byte aligned
 * scratch of fbla_pisa_fwd_scratch_bytes() bytes (16-bit copies of kc, vc and h; 0 = this shape has
 * no such kernel, -1 = invalid problem).  With too little scratch or another shape the call is
 * fbla_pisa_fwd.  Same results contract and same row_stats as fbla_pisa_fwd.                     */
int64_t fbla_pisa_fwd_scratch_bytes(const fbla_pisa_problem *p);
int fbla_pisa_fwd_ws(const fbla_pisa_problem *p, const void *q, const void *k, const void *v,
                     const float *kc, const float *vc, const float *h, const int32_t *indices,
                     void *o, float *row_stats, void *scratch, size_t scratch_bytes,
                     fbla_stream_t stream);

/* Backward of fbla_pisa_fwd with the block selection held constant; gradients flow through the
 * block statistics as well.  The reference has no backward for this operator (no counterpart).
 * o, d_o: forward output and its gradient; row_stats: as written by fbla_pisa_fwd.
 * scratch: fp32, 256-byte aligned, at least fbla_pisa_bwd_scratch_floats() elements (holds the
 * gradients of the block statistics, the per-row terms and, on the tensor-core paths, the rows
 * from which the gradient of h is formed, the workspace of that state pass and 16-bit copies of
 * kc, vc, h and dh for the tcgen05 kernels); contents are undefined afterwards.
 * 16-bit inputs with block_size 64 and dk = dv in {64, 128} run on tcgen05 kernels (query side,
 * key side), other shapes on CUDA-core kernels; FBLA_PISA_TC=0 in the environment selects the
 * mma.sync kernels that served those shapes before.                                           */
int64_t fbla_pisa_bwd_scratch_floats(const fbla_pisa_problem *p);
int fbla_pisa_bwd(const fbla_pisa_problem *p, const void *q, const void *k, const void *v,
                  const void *o, const void *d_o, const float *kc, const float *vc, const float *h,
                  const int32_t *indices, const float *row_stats, void *dq, void *dk, void *dv,
                  float *scratch, size_t scratch_floats, fbla_stream_t stream);

/* ---- multi-GPU: sum of the sequence-sharded states over the GPUs of one node ---------------
 * The reference runs on one GPU (no counterpart).  A sequence split along T over `world` ranks
 * needs the sum of the ranks' fp32 states between *_fwd_state and *_fwd_out (and between
 * *_bwd_state and *_bwd_in).  For shapes the fused passes below do not serve (fp32, other feature
 * dims) this call does it in one kernel with plain loads from the peers' memory (NVLink).
 *   peer_states[r]: rank r's state buffer of n_floats floats, mapped into this process (this
 *                   rank's own buffer at index `rank`); the local state must already have been
 *                   written to it by earlier work on `stream`.
 *   peer_flags[r] : rank r's array of at least `world` 32-bit words, mapped likewise, zero before
 *                   the first exchange.
 *   epoch         : 1, 2, 3, ... the same on every rank for the same exchange.
 *   out           : ordinary device memory; receives sum_r peer_states[r], added in rank order
 *                   (bit-identical on all ranks).
 * Every rank of the group must make the matching call; each waits (bounded by FBLA_PEER_WAIT_MS,
 * then `out` is filled with NaN, the device status word is set and later calls return
 * FBLA_ERR_DEVICE) for all peers to enter theirs.  Use two buffers alternately for consecutive exchanges: a rank can enter exchange
 * e+2 only after all peers have entered e+1, i.e. have finished reading the buffer of e.      */
int fbla_peer_state_sum(int world, int rank, const void *const *peer_states,
                        void *const *peer_flags, int64_t n_floats, uint32_t epoch, float *out,
                        fbla_stream_t stream);

/* ---- multi-GPU: sequence-sharded calls for what the tensor-core kernels serve -----------------
 * No counterpart in the reference (it runs on one GPU).  Fixed length, 16-bit, dk, dv in {64, 128}
 * (decoupled at 64 x 64).  The reducing pass leaves its per-segment pieces in this rank's piece buffer
 * (no reduction kernel); fbla_seq_sharded_exchange, one kernel, sums the pieces of all ranks into an
 * ordinary state buffer, which the regular *_fwd_out / *_bwd_in (or *_bwd_state as `state`) then take.
 * With two ranks every rank adds all units from both ranks' pieces after one flag round.  With more,
 * each unit is summed once by its owner (rank u / ceil(units / world)) into full[owner], a second
 * flag round follows and every rank reads the other units from their owners: 2 (world-1)/world of the
 * state crosses NVLink per rank.  Either way a unit is added in one fixed order (ranks in order,
 * pieces in CTA order): all ranks hold the same bits.  Plain peer loads only; nothing but flag words
 * is stored to a peer; no multicast.
 *   parts[r] : rank r's piece buffer of fbla_seq_sharded_part_floats() floats, 16-byte aligned;
 *   full[r]  : rank r's buffer of fbla_state_floats() floats, 16-byte aligned;
 *   flags[r] : rank r's 64 32-bit flag words, zero before the first exchange;
 *   all three mapped into this process for every rank r (this rank's own memory at index `rank`);
 *   epoch    : 1, 2, 3, ... the same on every rank for the same exchange, counted per flags array.
 * Use two (parts, full) pairs alternately for consecutive exchanges and one flags array for all: a
 * rank can start exchange e+2 only after every peer has entered e+1, i.e. has finished reading the
 * buffers of e.  Every rank must make the same calls in the same order with the same problem (same
 * local seq_len: the ranks' tile schedules must agree).  The wait for the peers is bounded
 * (FBLA_PEER_WAIT_MS in the environment, default 5000): after that the kernel fills state_out with
 * NaN, fbla_device_status() becomes non-zero and every later call returns FBLA_ERR_DEVICE until
 * fbla_clear_device_status(); the flags arrays of all ranks must then be zeroed and the epochs
 * restarted.  Ranks that may be further apart should meet at a host barrier first.
 * k_rope / q_rope / dq_rope are NULL except for decoupled_la.                                      */
typedef struct fbla_peer_group {
    int32_t world;          /* 2..8 ranks, GPUs of one node                   */
    int32_t rank;
    uint32_t epoch;
    int32_t reserved;
    void *const *parts;     /* [world] */
    void *const *full;      /* [world] */
    void *const *flags;     /* [world] */
} fbla_peer_group;

int fbla_seq_sharded_supported(const fbla_problem *p);
int64_t fbla_seq_sharded_part_floats(const fbla_problem *p);
/* Pieces of [ S | sum k ] of this rank's tokens into parts[rank].                                   */
int fbla_seq_sharded_fwd_state(const fbla_problem *p, const void *k, const void *k_rope, const void *v,
                               const fbla_peer_group *group, fbla_stream_t stream);
/* dq (and dq_rope) of this rank's tokens; pieces of the state gradient into parts[rank].  `state` is
 * the summed state an earlier fbla_seq_sharded_exchange produced.                                  */
int fbla_seq_sharded_bwd_state(const fbla_problem *p, const void *q, const void *q_rope, const void *d_o,
                               const float *state, const fbla_peer_group *group, void *dq, void *dq_rope,
                               fbla_stream_t stream);
/* state_out (fbla_state_floats() floats, ordinary memory, 16-byte aligned) = sum over the ranks of the
 * pieces the preceding fbla_seq_sharded_fwd_state / _bwd_state of the same `group` left.           */
int fbla_seq_sharded_exchange(const fbla_problem *p, const fbla_peer_group *group, float *state_out,
                              fbla_stream_t stream);

/* The status word the kernels write when a bounded wait gives up (0 = none did; otherwise a number
 * naming the wait).  While it is non-zero every launching call returns FBLA_ERR_DEVICE.  Clear it
 * once the cause is dealt with; results of the failed call are invalid.  No counterpart in the
 * reference.                                                                                   */
int fbla_device_status(void);
void fbla_clear_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_BLA_SM100_H */
