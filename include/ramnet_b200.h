/*
 * ramnet_b200 -- C ABI of the B200 (sm_100a) kernels for RAM-Net's sparse slot-memory path.
 *
 * Every entry point takes plain device pointers, sizes and element strides.  The library
 * never allocates, frees or synchronises: the caller owns inputs, outputs and workspaces and
 * passes the CUDA stream to launch on (as a cudaStream_t cast to void*).  Return value 0 means
 * the launch was enqueued; non-zero means nothing was launched and rn_last_error() describes
 * why (thread-local text).  Citations name the reference interface each entry point replaces,
 * by path inside the reference project.
 *
 * Symbols: B batch, T tokens, H heads, U address digits, P radix, A = P^U slots per head,
 * C value channels, Kw / Kr write / read Top-K, E number of leading heads with the CAPE shift.
 * dtype codes for logits / values / gamma / y: 0 = float32, 1 = float16, 2 = bfloat16.
 * Slot and mass state, weights and gradients of weights are float32; indices are int32.
 */
#ifndef RAMNET_B200_H
#define RAMNET_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { RN_F32 = 0, RN_F16 = 1, RN_BF16 = 2 };

/* Width of the index type used for slot indices (the reference exports the same number as
 * ramnet_ops._C.INT_BITS, packages/ramnet-ops/csrc/ram_attn_bind.cpp:120-129).  State element
 * offsets are 64-bit inside the kernels, so B*H*A*C may exceed 2^31. */
int rn_int_bits(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char *rn_last_error(void);

/* Library build tag, e.g. "ramnet_b200 sm_100a". */
const char *rn_version(void);

/* Benchmark aid (no counterpart in the reference).  After rn_prof_enable(1) the calling thread's
 * entry points record CUDA events around each of their kernel launches, on the launch stream;
 * rn_prof_read() waits for the last event of the most recent call and writes the duration of each
 * of its kernels in milliseconds (returns how many, -1 on a CUDA error). */
int rn_prof_enable(int on);
int rn_prof_read(float *ms, int n);

/*
 * Device-side failure report (the reference has no counterpart: its kernels have no waits that can
 * run out; host-side errors there are TORCH_CHECKs, packages/ramnet-ops/csrc/torch_compat.h:19-22).
 *
 * The decode and prefill kernels wait on asynchronous copies with a bound of about a second.  A wait
 * that runs out makes the kernel record a non-zero code (1 = wait timed out) in a per-device status
 * word, leave the state of the affected (batch, head) as it was where it still can, and return; the
 * entry point that launched it has already returned 0 by then.  The word is sticky.
 * rn_device_status() copies it to *status after SYNCHRONISING `stream` (so call it at a point that
 * may block, never inside a stream capture) and clears it when reset != 0.  0 means no kernel on
 * this device has reported a failure since the last reset.
 */
int rn_device_status(int device, void *stream, int reset, int *status);

/* Diagnostic for the mechanism above: launches one tiny kernel whose only bulk copy (256 bytes)
 * completes while its barrier expects `extra_bytes` more, so that the bounded wait (shortened to
 * 2^limit_log2 clock cycles) runs out exactly as it would in a product kernel; the kernel reports
 * through the status word and returns with nothing in flight.  With extra_bytes == 0 the wait
 * succeeds and the status word stays untouched.  No GPU fault, trap or hang is involved. */
int rn_selftest_wait_timeout(int extra_bytes, int limit_log2, int device, void *stream);

/*
 * Address decode (Product-Softmax over U digit sub-vectors + exact Top-K prefix search +
 * CAPE cyclic shift), write and read addresses in ONE launch.
 * Replaces ramnet_ops::topk_addr_forward / topk_addr_single_forward
 * (packages/ramnet-ops/csrc/ram_attn_ops.cpp:63-97,137-175 and the kernel
 *  packages/ramnet-ops/csrc/ram_attn_topk_addr.cu:52-117).
 *
 *  w_addr, r_addr : logits, logical shape (B,H,U,P,T) addressed through addr_strides[5]
 *                   (element strides in that order; both tensors share them).  r_addr may be
 *                   NULL (then Kr must be 0): single-tensor decode.
 *  pos            : int32 positions, element strides pos_strides[2] over (B,T).
 *  idx, val       : outputs, logical shape (B,H,Kw+Kr,T) through out_strides[4]; entries
 *                   [0,Kw) come from w_addr, [Kw,Kw+Kr) from r_addr.  Entry k is the k-th
 *                   address under (score descending, content index ascending).
 *  w_neg / r_neg  : store the weight negated (the joined decode of the reference stores reads
 *                   negated, packages/ramnet-ops/csrc/ram_attn_ops.cpp:152-153).
 *  encode_batch   : idx = (b*H+h)*A + a when non-zero, h*A + a otherwise.
 */
int rn_addr_fwd(const void *w_addr, const void *r_addr, int dtype, const int64_t *addr_strides,
                const int32_t *pos, const int64_t *pos_strides,
                int32_t *idx, float *val, const int64_t *out_strides,
                int64_t B, int64_t H, int64_t U, int64_t P, int64_t T, int64_t E,
                int64_t Kw, int64_t Kr, double w_re_norm, double r_re_norm,
                int w_neg, int r_neg, int encode_batch, int device, void *stream);

/*
 * Gradient of the decoded weights w.r.t. the logits.
 * Replaces ramnet_ops::topk_addr_backward / topk_addr_single_backward
 * (packages/ramnet-ops/csrc/ram_attn_ops.cpp:99-135,177-224, kernel
 *  packages/ramnet-ops/csrc/ram_attn_topk_addr.cu:119-226).
 *
 *  idx, val   : forward outputs, (B,H,Kw+Kr,T) through out_strides[4].
 *  d_val      : upstream gradient w.r.t. the POSITIVE weights, float32, same logical shape,
 *               strides dval_strides[4].
 *  d_w, d_r   : outputs in the logits dtype, logical shape (B,H,U,P,T) through dgrad_strides[5];
 *               d_r may be NULL when Kr == 0.
 *  w_neg/r_neg: sign convention val was stored with.
 */
int rn_addr_bwd(const int32_t *idx, const float *val, const int64_t *out_strides,
                const float *d_val, const int64_t *dval_strides,
                const void *w_addr, const void *r_addr, int dtype, const int64_t *addr_strides,
                const int32_t *pos, const int64_t *pos_strides,
                void *d_w, void *d_r, const int64_t *dgrad_strides,
                int64_t B, int64_t H, int64_t U, int64_t P, int64_t T, int64_t E,
                int64_t Kw, int64_t Kr, double w_re_norm, double r_re_norm,
                int w_neg, int r_neg, int device, void *stream);

/*
 * One fused autoregressive decode step: address decode for the write and read logits, gated
 * update of the Kw selected slots (slot and mass, in place), weighted read of the Kr selected
 * slots after the update, and optionally the layer epilogue (head-wise RMSNorm and sigmoid
 * gate).  Replaces ramnet_ops::topk_autoregressive_
 * (packages/ramnet-ops/csrc/ram_attn_ops.cpp:349-394, kernel
 *  packages/ramnet-ops/csrc/ram_attn_topk_autoregressive.cu:37-191); the epilogue replaces
 * packages/ramnet/src/ramnet/layers/ram_attn_block.py:342-348.
 *
 *  w_addr, r_addr : (B,H,U,P) contiguous logits;  x : (B,H,C);  gamma : (B,H)   [dtype]
 *  slot, mass     : float32 state (B,H,A,C) / (B,H,A), contiguous, updated in place
 *  mask           : (B) bytes, 0 = skip this batch row (state untouched, y = 0); may be NULL
 *  pos            : (B) int32
 *  y              : (B,H,C) output in dtype
 *  norm_weight    : (C) float32 or NULL;  gate_logits : (B,H,C) in dtype or NULL.
 *                   With either non-NULL, y = RMSNorm(y; norm_eps) * norm_weight * sigmoid(gate).
 */
int rn_decode_step(const void *w_addr, const void *r_addr, const void *x, const void *gamma, int dtype,
                   float *slot, float *mass, const uint8_t *mask, const int32_t *pos, void *y,
                   const float *norm_weight, const void *gate_logits, double norm_eps,
                   int64_t B, int64_t H, int64_t U, int64_t P, int64_t C, int64_t E,
                   int64_t Kw, int64_t Kr, double w_re_norm, double r_re_norm,
                   int mass_aware, double eps, int device, void *stream);

/*
 * The same step with the layer's address scaling folded into the load of the logits
 * (packages/ramnet/src/ramnet/layers/ram_attn_block.py:314-315: logits * exp(scale) / temperature):
 *  w_scale, r_scale : (H,U) factors in dtype, both or neither; a logit enters the decode as
 *                     round_to_dtype(factor * logit), exactly what the separate multiply produces.
 * Taken where rn_decode_scales_supported() returns 1 (16-bit logits, U=2, P=64, Kw=Kr=16, C in {128, 256});
 * elsewhere the call fails and the caller multiplies beforehand.
 *  batch_strides    : NULL (all inputs contiguous) or 5 element strides between the batch rows of w_addr, r_addr,
 *                     x, gamma and gate_logits; inside a batch row the heads are contiguous.  This lets the inputs
 *                     be column slices of ONE projection output (the layer's five projections merged into one GEMM).
 */
int rn_decode_scales_supported(int dtype, int64_t U, int64_t P, int64_t C, int64_t Kw, int64_t Kr);
int rn_decode_step_scaled(const void *w_addr, const void *r_addr, const void *x, const void *gamma, int dtype,
                          float *slot, float *mass, const uint8_t *mask, const int32_t *pos, void *y,
                          const float *norm_weight, const void *gate_logits, double norm_eps,
                          const void *w_scale, const void *r_scale, const int64_t *batch_strides,
                          int64_t B, int64_t H, int64_t U, int64_t P, int64_t C, int64_t E,
                          int64_t Kw, int64_t Kr, double w_re_norm, double r_re_norm,
                          int mass_aware, double eps, int device, void *stream);

/*
 * Prefill (T > 1) gated sparse update + read over decoded addresses.
 * Replaces gather_segment + ramnet_ops::topk_segment_forward / topk_segment_forward_
 * (packages/ramnet-ops/src/ramnet_ops/impl/cuda_impl.py:72-141,
 *  packages/ramnet-ops/csrc/ram_attn_ops.cpp:226-265,312-347, kernel
 *  packages/ramnet-ops/csrc/ram_attn_segment_parallel.cu:241-416).
 *
 *  idx, val     : decoded addresses, logical (B,H,Kw+Kr,T) through idx_strides[4] (shared by
 *                 both); entries [0,Kw) are writes, [Kw,Kw+Kr) reads; |val| is the weight,
 *                 val == 0 marks a no-op; idx may carry the (b*H+h)*A offset (idx mod A is used).
 *  x            : (B,H,T,C) values through x_strides[4] (channel stride 1);
 *  gamma        : (B,H,T) through gamma_strides[3];  mask: (B,T) bytes through mask_strides[2]
 *                 or NULL; a masked token neither writes nor reads and its y is zero.
 *  slot_in/mass_in, slot_out/mass_out : float32 contiguous (B,H,A,C)/(B,H,A); out may alias in.
 *  y            : (B,H,T,C) through y_strides[4] (channel stride 1), written in dtype.
 *  workspace    : caller-owned scratch of at least rn_gsu_workspace_bytes(...) bytes, 256-byte
 *                 aligned; holds the per-chunk event schedule between the two kernels.
 */
int64_t rn_gsu_workspace_bytes(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr,
                               int device);
/* The same query for a caller that knows the dtype and whether the rows of x start on 16-byte boundaries
 * (base pointer and the B, H, T strides in bytes all multiples of 16).  Model shapes (C = 128, A a multiple of
 * 16 up to 4096, Kr <= 16, Kw + Kr <= 32, 16-bit values) can run on the slot-owner kernel (when enabled, see
 * rn_gsu_owner_enable), which keeps the state of a (batch, head) in the shared memory of one 16-CTA cluster and
 * needs NO workspace: the answer is then 0 and rn_gsu_fwd accepts workspace == NULL.
 * rn_gsu_workspace_bytes() is always sufficient. */
/* Which kernels rn_gsu_fwd runs for a shape (no counterpart in the reference): 0 general apply kernel, 1 channel-slice
 * kernels with per-slot chains, 2 slot-owner cluster kernel; -1 on invalid dimensions.  rows_aligned as in
 * rn_gsu_fwd_workspace_bytes. */
int rn_gsu_fwd_path(int dtype, int rows_aligned, int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw,
                    int64_t Kr, int device);
/* The slot-owner kernel is an alternative forward path, off by default (on B200 the channel-slice kernels are
 * faster); rn_gsu_owner_enable(1) switches it on for the process, returns the previous setting (-1 = never set,
 * then the environment variable RN_PREFILL_OWNER=1 decides).  rn_gsu_owner_profile() hands it a device buffer
 * of 8 int64 cycle counters that CTA 0 fills (NULL = off); a benchmark aid.  No counterpart in the reference. */
int rn_gsu_owner_enable(int on);
int rn_gsu_owner_profile(long long *device_counters);
int64_t rn_gsu_fwd_workspace_bytes(int dtype, int rows_aligned, int64_t B, int64_t H, int64_t T, int64_t A, int64_t C,
                                   int64_t Kw, int64_t Kr, int device);
/* Launch plan of a prefill call of this shape (no counterpart in the reference; its launch geometry is fixed,
 * packages/ramnet-ops/csrc/ram_attn_segment_parallel.cu:785-830).  Fills out[0..7]: fast apply kernel (1/0),
 * channels per CTA, events per thread (forward), channel slices, chunk length, state slice in shared memory
 * (1/0), events per thread (backward sweeps), schedule tables in shared memory (1/0).  reverse != 0 plans the
 * backward pass.  Lets a test or benchmark prove that two shapes run the same template instances. */
int rn_gsu_plan_info(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr, int reverse,
                     int device, int32_t *out, int n);
int rn_gsu_fwd(const int32_t *idx, const float *val, const int64_t *idx_strides, const void *x,
               const int64_t *x_strides, const void *gamma, const int64_t *gamma_strides, int dtype,
               const uint8_t *mask, const int64_t *mask_strides, const float *slot_in, const float *mass_in,
               float *slot_out, float *mass_out, void *y, const int64_t *y_strides, void *workspace,
               int64_t workspace_bytes, int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw,
               int64_t Kr, int mass_aware, double eps, int device, void *stream);

/*
 * Backward of the prefill update / read (plain and mass-aware reads).
 * Replaces ramnet_ops::topk_segment_backward
 * (packages/ramnet-ops/csrc/ram_attn_ops.cpp:267-310, kernels
 *  packages/ramnet-ops/csrc/ram_attn_segment_parallel.cu:241-606).
 *
 *  idx, val, x, gamma, mask, slot_in, mass_in : the forward inputs (same layouts as rn_gsu_fwd).
 *  d_y          : (B,H,T,C) gradient of y in the dtype of x, strides dy_strides[4];
 *  d_slot_post, d_mass_post : gradients of the returned state, float32 contiguous.
 *  d_val        : output (B,H,Kw+Kr,T) through dval_strides[4], ZEROED BY THE CALLER; gradients
 *                 w.r.t. the positive weight of every event (writes and reads).
 *  d_x          : output (B,H,T,C) in the dtype of x;  d_gamma: (B,H,T) float32 contiguous;
 *  d_slot, d_mass : gradients of the initial state, float32 contiguous.
 *  workspace    : rn_gsu_bwd_workspace_bytes(...) bytes, 256-byte aligned (per write event it holds
 *                 x - slot_before, C floats, like the reference's replay cache, laid out per channel
 *                 slice; per event and channel slice one partial dot product; the event schedule).
 *                 Results are run-to-run deterministic: no float atomics are used.
 * Needs C % 4 == 0, A <= 65536 and a channel slice of the state that fits shared memory.
 */
int64_t rn_gsu_bwd_workspace_bytes(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr,
                                   int device);
int rn_gsu_bwd(const int32_t *idx, const float *val, const int64_t *idx_strides, const void *x,
               const int64_t *x_strides, const void *gamma, const int64_t *gamma_strides, int dtype,
               const uint8_t *mask, const int64_t *mask_strides, const float *slot_in, const float *mass_in,
               const void *d_y, const int64_t *dy_strides, const float *d_slot_post, const float *d_mass_post,
               float *d_val, const int64_t *dval_strides, void *d_x, const int64_t *dx_strides, float *d_gamma,
               float *d_slot, float *d_mass, void *workspace, int64_t workspace_bytes, int64_t B, int64_t H,
               int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr, int mass_aware, double eps, int device,
               void *stream);

/*
 * Prefill update without any allocation (no counterpart in the reference, which allocates its
 * event buffers with the framework allocator inside the operator).
 *
 * Same computation, arguments and results as rn_gsu_fwd, minus the workspace: the event schedule
 * is kept in a fixed array compiled into the library (rn_gsu_static_scratch_bytes() bytes of
 * device memory on every GPU that loads the library, held until the process exits).  Meant for
 * callers that cannot allocate device memory where they call from: an allocator or memory-pool
 * callback, a serving loop that sized its pools up front, a plugin whose host owns all device
 * memory.  The function calls no cudaMalloc / cudaFree nor any allocating library routine.
 *
 *  - Shapes whose schedule does not fit the array are rejected with a non-zero return and a
 *    message (nothing is launched); shorter calls with state carry-over give the same result.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
 *    caches it; make that first call outside any stream capture.
 *  - All calls on one device share the array and it keeps the previous call's contents.  Nothing
 *    in it has to start at zero (each call rewrites every entry it later reads), but two calls
 *    that overlap on the GPU (different streams, or different host threads without ordering) race
 *    on it: keep calls on one stream or order them with events.
 */
int64_t rn_gsu_static_scratch_bytes(void);
int rn_gsu_fwd_static(const int32_t *idx, const float *val, const int64_t *idx_strides, const void *x,
                      const int64_t *x_strides, const void *gamma, const int64_t *gamma_strides, int dtype,
                      const uint8_t *mask, const int64_t *mask_strides, const float *slot_in, const float *mass_in,
                      float *slot_out, float *mass_out, void *y, const int64_t *y_strides,
                      int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr,
                      int mass_aware, double eps, int device, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* RAMNET_B200_H */
