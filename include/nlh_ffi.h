/*
 * nlh_ffi.h — C ABI of libnlh_b200.so, the sm_100a implementation of the
 * NL_Hecate memory-rule / SWA / AdamW hot path.
 *
 * Section 1 declares drop-in symbols: name, argument order, argument types and
 * return type are those of the `extern "C"` block in the reference's
 * core/src/cuda_ffi.rs (line of each Rust declaration cited). A host built
 * against that block links against this library unchanged.
 *
 * Conventions (same as the reference): every pointer is DEVICE memory owned by
 * the caller; dimensions are int32; uint16_t* is bf16 bits; outputs documented
 * as accumulated must be zeroed by the caller. Differences, all additive:
 *   - launches go to the stream set with nlh_set_stream() (default: the
 *     legacy default stream, as in the reference) and never synchronise;
 *   - private scratch comes from a grow-only per-device workspace instead of
 *     cudaMalloc/cudaFree inside each call;
 *   - an invalid argument or launch failure is recorded (nlh_last_status())
 *     and printed to stderr; the process is not aborted.
 *
 * Section 2 declares the additive entries of this library (status-returning,
 * per-problem outputs, recompute-style training path, multi-tensor AdamW).
 */
#ifndef NLH_FFI_H
#define NLH_FFI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ───────────────────────── runtime ───────────────────────── */
/* No counterpart in the reference (it has no stream/handle arguments). */
void nlh_set_stream(void* cuda_stream);
void* nlh_get_stream(void);
int32_t nlh_last_status(void);          /* NLH_OK (0) or the last recorded error */
const char* nlh_last_error(void);       /* text of the last recorded error ("" if none) */
void nlh_clear_status(void);
int32_t nlh_workspace_reserve(int64_t bytes); /* pre-grow scratch (e.g. before graph capture) */
void nlh_workspace_release(void);       /* free the scratch of the current device */
int64_t nlh_workspace_bytes(void);      /* scratch bytes held on the current device, all slots */
/* Scratch slot (0..7, default 0) used by the following calls. Launches that may overlap on the
 * GPU (different streams) must use different slots; each slot grows on its own. */
int32_t nlh_set_workspace_slot(int32_t slot);
int32_t nlh_abi_version(void);
/* The reference's parameter-init generator (SimpleRng, core/src/tensor.rs:380-408): xorshift64
 * (<<13, >>7, <<17), uniform = (2 * (u64 / u64::MAX) - 1) * scale. HOST pointers; *state is
 * advanced, so consecutive calls continue one stream (a zero state is replaced by 1 like a zero
 * seed). Lets a host reproduce StackedMAGParams::init (core/src/stacked_model.rs:69-119,172-208). */
void nlh_simple_rng_fill(uint64_t* state, float scale, float* out_host, int64_t n);

/* ═════════════ Section 1: drop-in symbols (core/src/cuda_ffi.rs) ═════════════ */

/* cuda_ffi.rs:26 — SWA forward. q,k,v,out [B,S,H*hd] bf16; attn_weights
 * [B,H,S,n_persistent+window] bf16 (may be NULL here: skipped). */
void swa_forward_f32_cuda(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out,
    uint16_t* attn_weights, int32_t seq_len, int32_t num_heads, int32_t head_dim,
    int32_t window_size, int32_t batch_size, int32_t n_persistent);
/* cuda_ffi.rs:62 — SWA backward. d_q,d_k,d_v f32, accumulated (caller zeroes). */
void swa_backward_f32_cuda(const uint16_t* q, const uint16_t* k, const uint16_t* v,
    const uint16_t* attn_weights, const float* d_attn_out, float* d_q, float* d_k, float* d_v,
    int32_t seq_len, int32_t num_heads, int32_t head_dim, int32_t window_size, int32_t batch_size,
    int32_t n_persistent);

/* cuda_ffi.rs:86 / :109 — Delta rule, full trajectory m_states [B,(S+1),d*d]. */
void delta_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int32_t seq_len, int32_t d, int32_t batch_size, int32_t input_stride, int32_t m_stride,
    float error_clip, float m_norm_max);
void delta_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta,
    float* d_m_initial, int32_t seq_len, int32_t d, int32_t batch_size, float error_clip);
/* cuda_ffi.rs:134 / :156 — Titans LMM. d_m_initial/d_s_initial [d*d] are summed
 * over the batch (caller zeroes); additive: both may be NULL, they are then not computed (the
 * same holds for every backward entry of this header). Additive: s_states may be NULL in both calls (head_dim 32/64,
 * no clip/projection): the forward then writes only the M trajectory and the backward derives
 * S_t = M_t - (1-alpha_{t-1}) M_{t-1} from it (needs eta_t > 0), halving the state traffic. */
void titans_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, int32_t seq_len, int32_t d,
    int32_t batch_size, int32_t input_stride, int32_t m_stride, float error_clip,
    float m_norm_max);
void titans_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states,
    const float* s_states, const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem,
    float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial, float* d_s_initial,
    int32_t seq_len, int32_t d, int32_t batch_size, float error_clip);
/* cuda_ffi.rs:186 / :202 — Hebbian (backward has no batch argument). */
void hebbian_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_initial, float* m_states, float* y, int32_t seq_len,
    int32_t d, int32_t batch_size, int32_t input_stride, int32_t m_stride);
void hebbian_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_states, const float* d_y, float* d_k_mem, float* d_v_mem,
    float* d_q_mem, float* d_alpha, float* d_m_initial, int32_t seq_len, int32_t d);

/* cuda_ffi.rs:221-240 — checkpointed forwards: slot 0 = initial state, then one
 * slot every checkpoint_interval tokens and the final state. Single problem. */
void delta_forward_ckpt_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int32_t seq_len, int32_t d, int32_t checkpoint_interval, float error_clip, float m_norm_max);
void titans_forward_ckpt_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, int32_t seq_len, int32_t d,
    int32_t checkpoint_interval, float error_clip, float m_norm_max);
void hebbian_forward_ckpt_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_initial, float* m_states, float* y, int32_t seq_len,
    int32_t d, int32_t checkpoint_interval);
/* cuda_ffi.rs:250-275 — segment backwards over tokens [t_start,t_end) with a
 * segment-local trajectory [B,(t_end-t_start+1),d*d], seeds and per-batch outputs. */
void delta_backward_segment_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y,
    const float* d_m_seed, float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha,
    float* d_theta, float* d_m_out, int32_t t_start, int32_t t_end, int32_t d, int32_t batch_size,
    int32_t seq_len, float error_clip);
void titans_backward_segment_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states,
    const float* s_states, const float* d_y, const float* d_m_seed, const float* d_s_seed,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_out, float* d_s_out, int32_t t_start, int32_t t_end, int32_t d, int32_t batch_size,
    int32_t seq_len, float error_clip);
void hebbian_backward_segment_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_states, const float* d_y, const float* d_m_seed,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_m_out,
    int32_t t_start, int32_t t_end, int32_t d, int32_t batch_size, int32_t seq_len);

/* cuda_ffi.rs:291-337 — DGD (same math as Delta with the L2 bias). */
void dgd_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int32_t seq_len, int32_t d, int32_t batch_size, int32_t input_stride, int32_t m_stride,
    float error_clip);
void dgd_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta,
    float* d_m_initial, int32_t seq_len, int32_t d, float error_clip);
void dgd_forward_ckpt_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int32_t seq_len, int32_t d, int32_t checkpoint_interval, float error_clip);
void dgd_backward_segment_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y,
    const float* d_m_seed, float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha,
    float* d_theta, float* d_m_out, int32_t t_start, int32_t t_end, int32_t d, int32_t batch_size,
    int32_t seq_len, float error_clip);

/* cuda_ffi.rs:356-386 — frozen-M0 chunkwise rule; *_chunk_states [B,(ceil(S/C)+1),d*d]. */
void delta_chunkwise_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_chunk_states,
    float* y, int32_t seq_len, int32_t d, int32_t batch_size, int32_t chunk_size,
    float error_clip, float m_norm_max);
void delta_chunkwise_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_chunk_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta,
    float* d_m_initial, int32_t seq_len, int32_t d, int32_t batch_size, int32_t chunk_size,
    float error_clip, float m_norm_max);
void titans_chunkwise_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_chunk_states, float* s_chunk_states, float* y,
    int32_t seq_len, int32_t d, int32_t batch_size, int32_t chunk_size, float error_clip,
    float m_norm_max);
void titans_chunkwise_backward_f32_cuda(const float* k_mem, const float* v_mem,
    const float* q_mem, const float* alpha, const float* theta, const float* eta,
    const float* m_chunk_states, const float* s_chunk_states, const float* d_y, float* d_k_mem,
    float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_initial, float* d_s_initial, int32_t seq_len, int32_t d, int32_t batch_size,
    int32_t chunk_size, float error_clip, float m_norm_max);

/* cuda_ffi.rs:401-440 — phase-1 epilogue and per-chunk phase-2 kernels. */
void error_subtract_clip_f32_cuda(float* predictions, const float* v, int32_t total_rows,
    int32_t d, float error_clip);
void delta_phase2_forward_f32_cuda(const float* k_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* errors, float* m_work, float* m_chunk_states, float* y,
    int32_t seq_len, int32_t d, int32_t batch_size, int32_t chunk_size, int32_t chunk_idx,
    float m_norm_max);
void titans_phase2_forward_f32_cuda(const float* k_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* eta, const float* errors, float* m_work, float* s_work,
    float* m_chunk_states, float* s_chunk_states, float* y, int32_t seq_len, int32_t d,
    int32_t batch_size, int32_t chunk_size, int32_t chunk_idx, float m_norm_max);
void delta_phase2_backward_f32_cuda(const float* k_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* errors, const float* m_chunk_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_M,
    float* d_M0, float* m_recompute, int32_t seq_len, int32_t d, int32_t batch_size,
    int32_t chunk_size, int32_t chunk_idx, float m_norm_max);
void titans_phase2_backward_f32_cuda(const float* k_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* eta, const float* errors, const float* m_chunk_states,
    const float* s_chunk_states, const float* d_y, float* d_k_mem, float* d_v_mem,
    float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta, float* d_M, float* d_S,
    float* d_M0, float* m_recompute, float* s_recompute, int32_t seq_len, int32_t d,
    int32_t batch_size, int32_t chunk_size, int32_t chunk_idx, float m_norm_max);

/* cuda_ffi.rs:467 / :471 — Frobenius-norm clamp of the carried memory. */
void m_norm_clamp_f32_cuda(float* m, int32_t d, float m_norm_max);
void m_norm_clamp_batch_f32_cuda(float* m, int32_t d, int32_t batch_size, float m_norm_max);

/* cuda_ffi.rs:674-714 — AdamW family; return value is a cudaError_t. */
uint32_t adamw_update_cuda(float* w, const float* g, float* m, float* v, int32_t n, float lr,
    float beta1, float beta2, float eps, float bc1_inv, float bc2_inv, float weight_decay);
uint32_t grad_norm_sq_cuda(const float* g, float* partial_sums, int32_t n,
    int32_t* out_num_blocks);
uint32_t dot_product_partial_f32_cuda(const float* a, const float* b, float* partial_sums,
    int32_t n, int32_t* out_num_blocks);
uint32_t grad_scale_cuda(float* g, float scale, int32_t n);
uint32_t reduce_partials_clip_cuda(const float* partial_sums, int32_t total_partials,
    float max_grad_norm, float* out_norm, float* out_scale);
uint32_t grad_scale_conditional_cuda(float* g, const float* scale_ptr, int32_t n);

/* cuda_ffi.rs:854 / :887 — Titans LMM with a two-layer MLP memory. The state of one problem is the
 * packed buffer W1[d_hidden,d], b1[d_hidden], W2[d,d_hidden], b2[d] (state_size floats); S has the
 * same shape. k/v/q/y [batch, seq_len, d] with input_stride = seq_len * d floats between problems;
 * gates [batch, seq_len]; m_initial / s_initial [batch, state_size]; m_states / s_states
 * [batch, (seq_len + 1) * state_size] with m_stride floats between problems (slot 0 = initial).
 * activation: 0 GELU (tanh form), 1 SiLU, 2 ReLU. m_norm_max: Frobenius bound on the whole packed
 * state after every token (<= 0 or >= 1e30: off); the backward passes gradients straight through
 * it. The backward ADDS d_m_initial / d_s_initial [state_size] over the batch (caller zeroes them)
 * and writes every other output. One CTA per problem with the state on the SM: supported for
 * d, d_hidden <= 512 and state_size <= 33280 floats (d = 64, d_hidden = 256); larger shapes record
 * NLH_ERR_UNSUPPORTED and launch nothing. */
void titans_mlp_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, int32_t seq_len, int32_t d,
    int32_t d_hidden, int32_t batch_size, int32_t input_stride, int32_t m_stride,
    int32_t activation, float m_norm_max);
void titans_mlp_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states,
    const float* s_states, const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem,
    float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial, float* d_s_initial,
    int32_t seq_len, int32_t d, int32_t d_hidden, int32_t batch_size, int32_t input_stride,
    int32_t m_stride, int32_t activation, float m_norm_max);

/* cuda_ffi.rs:973 / :1000 — fused forwards: L2-normalise k,q in place, compute
 * the gates, then run the recurrence. */
void dgd_fused_forward_f32_cuda(float* k_mem, const float* v_mem, float* q_mem,
    const float* w_alpha, const float* b_alpha_ptr, const float* w_theta,
    const float* b_theta_ptr, float alpha_floor, float alpha_ceil, float theta_floor,
    float theta_ceil, const float* m_initial, float* m_states, float* y, float* alpha_out,
    float* theta_out, float* k_norms_out, float* q_norms_out, int32_t seq_len, int32_t d,
    int32_t batch_size, float error_clip);
void titans_fused_forward_f32_cuda(float* k_mem, const float* v_mem, float* q_mem,
    const float* w_alpha, const float* b_alpha_ptr, const float* w_theta,
    const float* b_theta_ptr, const float* w_eta, const float* b_eta_ptr, float alpha_floor,
    float alpha_ceil, float theta_floor, float theta_ceil, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, float* alpha_out,
    float* theta_out, float* eta_out, float* k_norms_out, float* q_norms_out, int32_t seq_len,
    int32_t d, int32_t batch_size, float error_clip, float m_norm_max);

/* ═════════════ Section 2: additive entries of this library ═════════════ */

/* rule: 0 Delta/DGD, 1 Titans LMM, 2 Hebbian. All return NLH_OK or an error
 * code; nothing is printed or aborted. */

/* Training forward that keeps only what the recompute backward needs:
 * exact rule (chunk_size = 0): checkpoints every `interval` tokens,
 *   m_ckpt/s_ckpt [B, ceil(S/interval)+1, d*d] (slot j = state before token
 *   j*interval; last slot = final state);
 * frozen-M0 rule (chunk_size > 0): interval must equal chunk_size and the
 *   buffers are the reference's *_chunk_states; or interval = 1 with chunk_size > 1 (Titans,
 *   head_dim 32/64): EVERY state is stored, m_ckpt [B, S+1, d*d], s_ckpt may be NULL, and the
 *   backward streams the stored states instead of recomputing chunk windows (the momentum is
 *   derived from consecutive M states, which needs eta_t > 0) — the faster pair for short
 *   chunks, at (S+1) d*d floats per problem.
 * Replaces the trajectory-materialising pairs core/kernels/titans_forward.cu:83
 * + titans_backward.cu:66 (and the Delta/Hebbian twins) at the call sites
 * core/src/gpu_forward.rs:1521 and gpu_backward.rs:459. */
int32_t nlh_rule_forward(int32_t rule, const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_ckpt, float* s_ckpt, float* y, int32_t seq_len, int32_t d,
    int32_t batch_size, int32_t interval, int32_t chunk_size, float error_clip,
    float m_norm_max);
/* Matching backward. d_m_initial/d_s_initial are PER PROBLEM [B,d*d] (the
 * reference sums them over the batch with atomicAdd: titans_backward.cu:337); in the
 * full-trajectory frozen mode both may be NULL. */
int32_t nlh_rule_backward(int32_t rule, const float* k_mem, const float* v_mem,
    const float* q_mem, const float* alpha, const float* theta, const float* eta,
    const float* m_ckpt, const float* s_ckpt, const float* d_y, float* d_k_mem, float* d_v_mem,
    float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial,
    float* d_s_initial, int32_t seq_len, int32_t d, int32_t batch_size, int32_t interval,
    int32_t chunk_size, float error_clip, float m_norm_max);

/* SWA without the materialised weights tensor: forward writes out (bf16) and
 * the per-row log-sum-exp lse [B,H,S] f32; backward recomputes the
 * probabilities from lse. d_q,d_k,d_v f32 are overwritten (no pre-zeroing).
 * Replaces core/kernels/swa_forward.cu:23 / swa_backward.cu:24. */
int32_t nlh_swa_forward(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out,
    float* lse, int32_t seq_len, int32_t num_heads, int32_t head_dim, int32_t window_size,
    int32_t batch_size, int32_t n_persistent);
int32_t nlh_swa_backward(const uint16_t* q, const uint16_t* k, const uint16_t* v,
    const uint16_t* out, const float* lse, const float* d_attn_out, float* d_q, float* d_k,
    float* d_v, int32_t seq_len, int32_t num_heads, int32_t head_dim, int32_t window_size,
    int32_t batch_size, int32_t n_persistent);

/* Packed variants for callers that keep q|k|v as the rows of one projection output
 * qkv [batch, seq, 3*heads*head_dim] bf16: no split copies before the forward, and the backward
 * takes d_attn_out in bf16 and OVERWRITES d_qkv (same packed layout, bf16) — no casts or
 * concatenation around the attention. out and d_attn_out are dense [batch, seq, heads*head_dim]. */
int32_t nlh_swa_forward_packed(const uint16_t* qkv, uint16_t* out, float* lse, int32_t seq_len,
    int32_t num_heads, int32_t head_dim, int32_t window_size, int32_t batch_size, int32_t n_persistent);
int32_t nlh_swa_backward_packed(const uint16_t* qkv, const uint16_t* out, const float* lse,
    const uint16_t* d_attn_out, uint16_t* d_qkv, int32_t seq_len, int32_t num_heads, int32_t head_dim,
    int32_t window_size, int32_t batch_size, int32_t n_persistent);

/* SWA pair in fp32 end to end (q, k, v, out, gradients all fp32; same visibility rule): the
 * accuracy option for configurations stated in fp32, matching the reference's CPU path
 * (core/src/swa.rs:33-92, :163-235) to rounding. CUDA-core kernels without tiling, meant for small
 * shapes: head_dim <= 128, n_persistent + min(window, seq) <= 2048. d_q, d_k, d_v are overwritten. */
int32_t nlh_swa_forward_f32(const float* q, const float* k, const float* v, float* out, float* lse,
    int32_t seq_len, int32_t num_heads, int32_t head_dim, int32_t window_size, int32_t batch_size,
    int32_t n_persistent);
int32_t nlh_swa_backward_f32(const float* q, const float* k, const float* v, const float* out,
    const float* lse, const float* d_attn_out, float* d_q, float* d_k, float* d_v, int32_t seq_len,
    int32_t num_heads, int32_t head_dim, int32_t window_size, int32_t batch_size, int32_t n_persistent);

/* Library options (no counterpart in the reference). NLH_OPT_SWA_TCGEN05 (default 1) runs the
 * head_dim-64 SWA forward on the tcgen05/TMEM kernel; 0 selects the mma.sync kernel instead. nlh_swa_tc_timeout_flag()
 * synchronously reads a device flag that the tcgen05 kernel sets if one of its bounded mbarrier
 * waits ran out (0 = never, 1 = a wait expired and results are invalid, -1 = read failed). */
#define NLH_OPT_SWA_TCGEN05 1
/* NLH_OPT_CHUNK_MATRIX (default 1): frozen-M0 chunkwise Titans / Delta entries at head_dim 64 and
 * chunk sizes 16..64 run in chunk-parallel matrix form; 0 selects the per-token kernels. */
#define NLH_OPT_CHUNK_MATRIX 2
/* NLH_OPT_ROW_SPLIT (default 1): when a launch has at most half as many problems as the GPU has SMs, the exact
 * head_dim-64 forward and the M-only exact Titans backward divide every problem's rows over two
 * CTAs (the rows of the memory evolve independently; the backward then zeroes d_q, d_k and the gate
 * gradients itself and adds the two partial sums into them). 0 keeps one CTA per problem. */
#define NLH_OPT_ROW_SPLIT 3
/* NLH_OPT_SWA_TMA (default 1): the tcgen05 SWA forward stages its Q, K and V tiles with tiled TMA
 * copies (cp.async.bulk.tensor, one issuing thread, completion on an mbarrier; plain single-CTA
 * loads) instead of per-thread cp.async; 0 selects the cp.async staging. Results are identical. */
#define NLH_OPT_SWA_TMA 4
/* NLH_OPT_BULK_STAGING (default 1): the register-resident memory-rule forward kernels (head_dim
 * 32/64) stage their k, v, q tiles with one bulk asynchronous copy per stream and tile
 * (cp.async.bulk from one thread, completion counted on an mbarrier) instead of per-thread
 * cp.async; 0 selects the cp.async staging. Results are identical. nlh_bulk_timeout_flag() is
 * nonzero if a bounded mbarrier wait of these kernels ever ran out. */
#define NLH_OPT_BULK_STAGING 5
int32_t nlh_bulk_timeout_flag(void);
int32_t nlh_set_option(int32_t option, int32_t value);
/* How the last tcgen05 SWA forward of this process staged its operand tiles: 1 = tiled TMA copies,
 * 0 = cp.async (NLH_OPT_SWA_TMA off, or the driver's tensor-map encoder was not available or
 * rejected the shape), -1 = no such launch yet. */
int32_t nlh_swa_forward_staging(void);
int32_t nlh_swa_tc_timeout_flag(void);

/* Multi-tensor AdamW over one flat arena (w,g,m,v share the layout). The
 * per-tensor loop it replaces is core/src/gpu_stacked_optimizer.rs:554-677. */
typedef struct nlh_adamw_tensor_desc {
    float bc1_inv;       /* 1/(1-beta1^t), t = the tensor's own step count      */
    float bc2_inv;       /* 1/(1-beta2^t)                                       */
    float weight_decay;
    float lr_scale;      /* multiplies the call's lr                            */
    float clamp_lo;      /* post-update clamp (b_theta in [-10,2]) if has_clamp */
    float clamp_hi;
    int32_t has_clamp;
    int32_t active;      /* 0: tensor skipped (CMS level not fired this step)   */
} nlh_adamw_tensor_desc;

int32_t nlh_adamw_multi_tensor(float* w, const float* g, float* m, float* v,
    const nlh_adamw_tensor_desc* descs_dev, const int32_t* chunk_tensor_dev,
    const int64_t* chunk_start_dev, const int32_t* chunk_len_dev, int32_t n_chunks,
    const float* grad_scale_ptr, float lr, float beta1, float beta2, float eps);
/* Global L2 norm of a flat gradient arena and the clip scale
 * (norm > max ? max/norm : 1), replacing the per-tensor grad_norm_sq_cuda loop
 * at core/src/gpu_stacked_optimizer.rs:193-345. partial: >= partial_capacity floats. */
int32_t nlh_arena_grad_norm_clip(const float* g, int64_t n, float max_grad_norm, float* partial,
    int32_t partial_capacity, float* out_norm, float* out_scale);

/* Fused rule wrapper around the recurrence: the ~15 small launches per CMS level at
 * core/src/gpu_forward.rs:1339-1382 and gpu_backward.rs:2047-2115 as one kernel each way. kvq: [batch*seq, 3*d_model] rows (k | v | q) as produced by the projection GEMM, fp32 or
 * bf16. Outputs in the per-head layout the memory kernels consume: k_ph,v_ph,q_ph
 * [batch*heads, seq, head_dim] (k,q L2-normalised over d_model), gates [batch*heads, seq]
 * (one value per token, repeated per head); k_norm,q_norm [batch*seq] for the backward.
 * w_gates [3, 2*d_model] rows alpha, theta, eta; biases are device scalars. */
int32_t nlh_level_prep_forward(const void* kvq, int32_t kvq_is_bf16, const float* w_gates,
    const float* b_alpha, const float* b_theta, const float* b_eta, float* k_ph, float* v_ph,
    float* q_ph, float* alpha_ph, float* theta_ph, float* eta_ph, float* k_norm, float* q_norm,
    int32_t batch, int32_t seq, int32_t d_model, int32_t num_heads);
/* Backward twin: d_kvq [batch*seq, 3*d_model]; gate weight / bias gradients as per-CTA partial
 * sums dw_partial [rows, 3, 2*d_model], db_partial [rows, 3] with
 * rows = nlh_level_prep_partial_rows(batch*seq) (the caller sums over rows). */
int32_t nlh_level_prep_partial_rows(int32_t n_tokens);
int32_t nlh_level_prep_backward(const float* k_ph, const float* v_ph, const float* q_ph,
    const float* alpha_ph, const float* theta_ph, const float* eta_ph, const float* k_norm,
    const float* q_norm, const float* dk_ph, const float* dv_ph, const float* dq_ph,
    const float* dalpha_ph, const float* dtheta_ph, const float* deta_ph, const float* w_gates,
    void* d_kvq, int32_t kvq_is_bf16, float* dw_partial, float* db_partial, int32_t batch,
    int32_t seq, int32_t d_model, int32_t num_heads);
/* MAG gating of one block (core/src/gpu_stacked_forward.rs:1935-1960):
 * out = x + attn_proj * sigmoid(sum_l w_l * upsample(y_l)), y_l [batch*heads, seq/c_l, head_dim]
 * read in the per-head layout, level_weights [k] on the device (softmax of alpha_mem). */
int32_t nlh_mag_combine_forward(const float* x, const void* attn_proj, int32_t attn_is_bf16,
    const float* level_weights, const float* y0, const float* y1, const float* y2, const float* y3,
    int32_t c0, int32_t c1, int32_t c2, int32_t c3, int32_t k, float* out, int32_t batch,
    int32_t seq, int32_t d_model, int32_t num_heads);
/* Backward: d_attn_proj (dtype of attn_proj), d_ycomb [batch, seq, d_model] fp32 (gradient of the
 * weighted level sum) and dw_partial [n_partial_rows, 4] partial sums of d level_weights.
 * dy0..dy3 (each may be NULL): for a level with pool factor 1, receives that level's output
 * gradient level_weights[l] * d_ycomb in the per-head layout, saving its nlh_pool_to_heads pass. */
int32_t nlh_mag_combine_backward(const float* d_out, const void* attn_proj, int32_t attn_is_bf16,
    const float* level_weights, const float* y0, const float* y1, const float* y2, const float* y3,
    int32_t c0, int32_t c1, int32_t c2, int32_t c3, int32_t k, void* d_attn_proj, float* d_ycomb,
    float* dw_partial, int32_t n_partial_rows, float* dy0, float* dy1, float* dy2, float* dy3,
    int32_t batch, int32_t seq, int32_t d_model, int32_t num_heads);
/* Finishers of the per-CTA partial rows the two backward entries above leave: rows are summed
 * and ADDED into the caller's gradient buffers (no reduction or accumulation
 * pass on the caller's side). nlh_gate_grad_finish: dw_partial [rows, 3, 2*d_model] into
 * g_w_gates [3, 2*d_model], db_partial [rows, 3] into the three bias gradients (each [1]; a NULL
 * one is skipped). nlh_level_weight_grad_finish: dw_partial [rows, 4] of nlh_mag_combine_backward
 * through the softmax adjoint d_logit_i = w_i (dw_i - sum_j w_j dw_j), w = level_weights =
 * softmax(logits) (core/src/mag.rs aggregation weights), into g_logits [k]. */
int32_t nlh_gate_grad_finish(const float* dw_partial, const float* db_partial, int32_t rows,
    int32_t d_model, float* g_w_gates, float* g_b_alpha, float* g_b_theta, float* g_b_eta);
int32_t nlh_level_weight_grad_finish(const float* dw_partial, int32_t rows, int32_t k,
    const float* level_weights, float* g_logits);
/* dy_ph[(b*H+h), t', :] = level_weights[level] * sum_{i<pool} d_ycomb[b, t'*pool+i, h*hd:(h+1)*hd]
 * (adjoint of repeat_upsample_1d + head transpose, pool_ops.cu / elementwise.cu). */
int32_t nlh_pool_to_heads(const float* d_ycomb, const float* level_weights, int32_t level,
    int32_t pool, float* dy_ph, float* sum_out, int32_t batch, int32_t seq, int32_t d_model,
    int32_t num_heads);
/* A coarser level from a finer level's UNSCALED sums (sum_out of nlh_pool_to_heads or of this
 * entry; optional, same layout as dy_ph), both per-head: src_sums [rows, src_seq, head_dim] ->
 * dy_ph [rows, src_seq/factor, head_dim] = level_weights[level] * sum over factor source rows.
 * Pooling by 512 then reads 1/64 of the data a direct pass over d_ycomb would. */
int32_t nlh_pool_heads(const float* src_sums, const float* level_weights, int32_t level,
    int32_t factor, float* dy_ph, float* sum_out, int32_t rows, int32_t src_seq, int32_t head_dim);

/* Mean pooling of consecutive token rows (the input of a coarser CMS level,
 * core/src/gpu_stacked_forward.rs:1879-1890, pool_ops.cu): src [rows_out*factor, d_model] fp32 ->
 * out [rows_out, d_model] (fp32 or bf16) = scale * sum of factor rows; sum_out (optional, fp32)
 * keeps the unscaled sums so that the next coarser level pools those instead of src. */
int32_t nlh_mean_pool(const float* src, int32_t factor, float scale, void* out, int32_t out_is_bf16,
    float* sum_out, int32_t rows_out, int32_t d_model);
/* Adjoint of up to three mean pools in one pass: out[b, t, :] = sum_l g_l[b, t / c_l, :] / c_l,
 * g_l [batch, seq/c_l, d_model] fp32 or bf16. */
int32_t nlh_unpool_sum(const void* g0, int32_t c0, int32_t g0_is_bf16, const void* g1, int32_t c1,
    int32_t g1_is_bf16, const void* g2, int32_t c2, int32_t g2_is_bf16, int32_t n_src, float* out,
    int32_t batch, int32_t seq, int32_t d_model);

/* ── Stacked-block glue (drop-in) ─────────────────────────────────────────────────────────────
 * LayerNorm over the last axis of x [n, d]; mean/rstd caches [n] feed the backward
 * (core/src/cuda_ffi.rs:487-491, kernels core/kernels/layer_norm.cu; CPU statement
 * core/src/mag.rs:396-449). Backward ACCUMULATES into d_gamma/d_beta (caller zeroes). */
void layer_norm_forward_cuda(const float* x, const float* gamma, const float* beta, float* out,
    float* mean_cache, float* rstd_cache, int32_t n, int32_t d, float eps);
/* core/src/cuda_ffi.rs:495-500 */
void layer_norm_backward_cuda(const float* d_out, const float* x, const float* gamma,
    const float* mean_cache, const float* rstd_cache, float* d_x, float* d_gamma, float* d_beta,
    int32_t n, int32_t d);
/* output[t, :] = w_embed[input_ids[t], :] (core/src/cuda_ffi.rs:523-529, embedding.cu). */
void embedding_gather_cuda(const float* w_embed, const int32_t* input_ids, float* output,
    int32_t seq_len, int32_t d);
/* d_embed[input_ids[t], :] += d_embedded[t, :] (core/src/cuda_ffi.rs:532-538). */
void embedding_scatter_add_cuda(const float* d_embedded, const int32_t* input_ids, float* d_embed,
    int32_t seq_len, int32_t d);
/* loss_out[0] = sum over positions with 0 <= target < vocab of -log softmax(logits[t])[target];
 * the entry zeroes loss_out first (core/src/cuda_ffi.rs:766-770, cross_entropy.cu:20-96). */
void cross_entropy_forward_cuda(const float* logits, const int32_t* target_ids, float* loss_out,
    int32_t seq_len, int32_t vocab);
/* d_logits = (softmax - onehot) * inv_count; rows with an invalid target are zeroed
 * (core/src/cuda_ffi.rs:772-775, cross_entropy.cu:99-176). */
void cross_entropy_backward_cuda(const float* logits, const int32_t* target_ids, float* d_logits,
    int32_t seq_len, int32_t vocab, float inv_count);

/* ── Stacked-block glue (additive, no counterpart in the reference) ───────────────────────────
 * LayerNorm that can also emit a bf16 copy of its output (either output pointer may be NULL)
 * and whose backward takes the upstream gradient as an fp32 part plus a bf16 part (either may be
 * NULL; they are summed), so the bf16 GEMMs on both sides need no separate cast kernels. */
int32_t nlh_layer_norm_forward(const float* x, const float* gamma, const float* beta, float* out_f32,
    uint16_t* out_bf16, float* mean_cache, float* rstd_cache, int32_t n, int32_t d, float eps);
int32_t nlh_layer_norm_backward(const float* d_out_f32, const uint16_t* d_out_bf16, const float* x,
    const float* gamma, const float* mean_cache, const float* rstd_cache, float* d_x, float* d_gamma,
    float* d_beta, int32_t n, int32_t d);
/* The same backward with up to three more gradient sources: gradients of mean-pooled copies of
 * the LayerNorm output, g_l [n / c_l, d] fp32 or bf16, each adding g_l[b, t / c_l, :] / c_l to
 * the output gradient of row (b, t) (seq rows per sequence, seq % c_l == 0) — the adjoint of
 * nlh_mean_pool folded into this kernel, so the upsampled sum is never written to memory.
 * d_out_f32 and d_out_bf16 may both be NULL when n_src > 0. Needs d % 8 == 0, d <= 1024. */
int32_t nlh_layer_norm_backward_pooled(const float* d_out_f32, const uint16_t* d_out_bf16,
    const void* g0, int32_t c0, int32_t g0_is_bf16, const void* g1, int32_t c1, int32_t g1_is_bf16,
    const void* g2, int32_t c2, int32_t g2_is_bf16, int32_t n_src, int32_t seq, const float* x,
    const float* gamma, const float* mean_cache, const float* rstd_cache, float* d_x, float* d_gamma,
    float* d_beta, int32_t n, int32_t d);
/* LayerNorm of x + res with the neighbouring element-wise passes of a residual block folded in
 * (res fp32 or bf16 [n, d], may be NULL; the sum is never written). Backward twin: the general
 * form of the two backwards above. The kernel normalises x + res again, adds the pooled sources
 * (n_src may be 0) to the output gradient, and writes
 *   d_x      = input gradient + add_in            (add_in fp32 [n, d] or NULL: a gradient of x that
 *                                                  arrives from another consumer, summed here),
 *   d_x_bf16 = bf16(input gradient + add_in_bf16) (optional: the gradient of a bf16 res operand with
 *                                                  its own fan-in).
 * Needs d % 8 == 0, d <= 1024, 16-byte aligned buffers when any of these operands is given. */
int32_t nlh_layer_norm_residual_forward(const float* x, const void* res, int32_t res_is_bf16,
    const float* gamma, const float* beta, float* out_f32, uint16_t* out_bf16, float* mean_cache,
    float* rstd_cache, int32_t n, int32_t d, float eps);
int32_t nlh_layer_norm_backward_fused(const float* d_out_f32, const uint16_t* d_out_bf16,
    const void* g0, int32_t c0, int32_t g0_is_bf16, const void* g1, int32_t c1, int32_t g1_is_bf16,
    const void* g2, int32_t c2, int32_t g2_is_bf16, int32_t n_src, int32_t seq, const float* x,
    const void* res, int32_t res_is_bf16, const float* add_in, const float* gamma,
    const float* mean_cache, const float* rstd_cache, float* d_x, uint16_t* d_x_bf16,
    const uint16_t* add_in_bf16, float* d_gamma, float* d_beta, int32_t n, int32_t d);
/* Cross-entropy on fp32 or bf16 logits [n, vocab]. Forward ACCUMULATES the loss sum into
 * loss_sum[0] and the number of valid targets into valid_count[0] (optional) and stores the
 * per-row log-sum-exp in lse [n] (optional). Backward writes
 * (softmax - onehot) * inv_count * grad_scale[0] (grad_scale NULL = 1) in the logits' type;
 * d_logits may alias logits; lse NULL = recompute. */
int32_t nlh_cross_entropy_forward(const void* logits, int32_t logits_is_bf16, const int32_t* target_ids,
    float* loss_sum, float* lse, int32_t* valid_count, int32_t n, int32_t vocab);
int32_t nlh_cross_entropy_backward(const void* logits, int32_t logits_is_bf16, const int32_t* target_ids,
    const float* lse, const float* grad_scale, void* d_logits, int32_t n, int32_t vocab, float inv_count);

/* ── Host-slice dispatch layer (compiled counterpart of core/src/dispatch.rs `*_dispatch`) ────
 * Same argument order and meaning as the reference functions its kernel tests call
 * (swa_forward_dispatch dispatch.rs:378, swa_backward_dispatch :408, delta :746/:775, titans
 * :810/:842, hebbian :1083/:1110, dgd :1153/:1182): HOST pointers, one sequence, int64 sizes
 * (usize), int32 status instead of a panic. Each call uploads, runs the drop-in entry,
 * downloads and synchronises. SWA rounds q,k,v to bf16 on the device; its backward adds into
 * d_q,d_k,d_v (caller pre-zeroes) and does not read attn_weights (may be NULL). */
int32_t nlh_swa_forward_dispatch(const float* q, const float* k, const float* v, float* out,
    float* attn_weights, int64_t seq_len, int64_t num_heads, int64_t head_dim, int64_t window_size);
int32_t nlh_swa_backward_dispatch(const float* q, const float* k, const float* v, const float* attn_weights,
    const float* d_attn_out, float* d_q, float* d_k, float* d_v, int64_t seq_len, int64_t num_heads,
    int64_t head_dim, int64_t window_size);
int32_t nlh_delta_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int64_t seq_len, int64_t d, float error_clip, float m_norm_max);
int32_t nlh_delta_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y, float* d_k_mem,
    float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_m_initial, int64_t seq_len,
    int64_t d, float error_clip);
int32_t nlh_titans_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, int64_t seq_len, int64_t d,
    float error_clip, float m_norm_max);
int32_t nlh_titans_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states,
    const float* s_states, const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem,
    float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial, float* d_s_initial,
    int64_t seq_len, int64_t d, float error_clip);
int32_t nlh_hebbian_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_initial, float* m_states, float* y, int64_t seq_len, int64_t d);
int32_t nlh_hebbian_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_states, const float* d_y, float* d_k_mem, float* d_v_mem,
    float* d_q_mem, float* d_alpha, float* d_m_initial, int64_t seq_len, int64_t d);
int32_t nlh_dgd_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int64_t seq_len, int64_t d, float error_clip);
int32_t nlh_dgd_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y, float* d_k_mem,
    float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_m_initial, int64_t seq_len,
    int64_t d, float error_clip);

/* core/src/dispatch.rs:897 / :979 — titans_mlp_forward_cuda / titans_mlp_backward_cuda: the MLP-memory
 * pair on HOST slices, with a batch (k/v/q/y [batch, seq, d], gates [batch, seq], m_initial /
 * s_initial [batch, state], trajectories [batch, (seq+1)*state]); d_m_initial / d_s_initial [state]
 * are the sums over the batch and are overwritten. */
int32_t nlh_titans_mlp_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial, const float* s_initial,
    float* m_states, float* s_states, float* y, int64_t seq_len, int64_t d, int64_t d_hidden, int64_t batch_size,
    int32_t activation, float m_norm_max);
int32_t nlh_titans_mlp_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states, const float* s_states,
    const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_initial, float* d_s_initial, int64_t seq_len, int64_t d, int64_t d_hidden, int64_t batch_size,
    int32_t activation, float m_norm_max);

/* ── Opaque-VJP registry over the C ABI (boundary of core/src/tape.rs:98-182) ────────────────
 * Keys number the variants of the reference's OpaqueKey enum in declaration order
 * (core/src/tape.rs:100-134). nlh_opaque_backward is the C form of OpaqueBackwardFn
 * (tape.rs:141-145): HOST pointers, d_outputs[i] of out_len[i] floats, saved[i] of saved_len[i]
 * floats (saved[0] is the float-encoded meta buffer), d_inputs[i] of in_len[i] floats
 * caller-allocated and overwritten. GPU adapters exist for
 *   NLH_KEY_{DELTA_RULE,TITANS_LMM,HEBBIAN_RULE} — a whole rule block (opaque_adapters.rs:306-381,
 *     :402-590, :593-628): saved = [meta, level_params_flat, embedded, cache fields in the order
 *     record_on_tape stores them (:1180-1385)], d_inputs = [d_embedded, d_level_params_flat in the
 *     order of level_params_to_flat (:93-113)]; identity feature map, L2 bias, EMA / no momentum,
 *     linear memory, no conv1d (anything else: NLH_ERR_UNSUPPORTED);
 *   NLH_KEY_DGD (opaque_adapters.rs:1680-1725);
 *   NLH_KEY_SWA (:952-997; q,k,v are rounded to bf16 on the device, attn_weights is not read);
 *   the frozen reads NLH_KEY_FROZEN_{DELTA_RULE,TITANS_LMM,HEBBIAN_RULE} with the identity feature
 *     map (:999-1069).
 * Every other key returns NLH_ERR_UNSUPPORTED. The call synchronises its stream before returning. */
#define NLH_KEY_DELTA_RULE 0
#define NLH_KEY_TITANS_LMM 1
#define NLH_KEY_HEBBIAN_RULE 2
#define NLH_KEY_DGD 9
#define NLH_KEY_SWA 10
#define NLH_KEY_FROZEN_DELTA_RULE 11
#define NLH_KEY_FROZEN_TITANS_LMM 12
#define NLH_KEY_FROZEN_HEBBIAN_RULE 13
int32_t nlh_opaque_backward(int32_t key, int32_t n_out, const float* const* d_outputs,
    const int64_t* out_len, int32_t n_saved, const float* const* saved, const int64_t* saved_len,
    int32_t n_in, float* const* d_inputs, const int64_t* in_len);

/* No counterpart in the reference. Titans LMM backward (same arguments, layout and
 * batch-summed d_m_initial/d_s_initial as titans_backward_f32_cuda) for callers that must
 * not allocate device memory: its scratch is a fixed 2 MiB array inside the library image,
 * so the call never reaches cudaMalloc/cudaFree or the workspace. Limit:
 * batch_size*d*d <= NLH_NOALLOC_MAX_STATE_FLOATS, otherwise NLH_ERR_INVALID_ARG. All calls
 * on a device share the array: calls that overlap on the GPU race; issue them in order on
 * one stream. Every pointer is required: unlike titans_backward_f32_cuda this entry has no
 * M-only mode, s_states == NULL is rejected with NLH_ERR_INVALID_ARG. The first call on each device resolves the array's device address and should
 * be made while the stream is not being captured. */
#define NLH_NOALLOC_MAX_STATE_FLOATS 262144
#define NLH_NOALLOC_SCRATCH_BYTES (2 * NLH_NOALLOC_MAX_STATE_FLOATS * 4)
int32_t nlh_titans_backward_noalloc(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states,
    const float* s_states, const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem,
    float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial, float* d_s_initial,
    int32_t seq_len, int32_t d, int32_t batch_size, float error_clip);

#ifdef __cplusplus
}
#endif
#endif /* NLH_FFI_H */
