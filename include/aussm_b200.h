/* C ABI of libaussm_b200.so: the sm_100a (B200) implementation of the AUSSM
 * selective-scan operators.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream; it
 * allocates nothing on the device (scratch is always a caller-owned workspace),
 * enqueues its kernels on `stream` and returns without synchronising.  The
 * library depends on the CUDA runtime only (no cuBLAS or other library kernels).  Return value: 0 on
 * success, a negative AUSSM_E* code otherwise; aussm_b200_last_error() then
 * describes the failure (thread-local string).
 *
 * Tensors are float32, contiguous, row-major:
 *   u, dt, z, y, grad_y, du, ddt, dz : (B, D, L)
 *   theta, dtheta                    : (B, D, N, L)
 *   x, dx                            : (D, N, D)   indexed [i][j][r]
 *   x_bias, dx_bias                  : (D, N)
 *   B_r, B_theta, C_r, C_theta       : (N,)        Bc = B_r exp(i B_theta), Cc likewise
 *   Dskip                            : (D,)
 *   hidden states and their grads    : (B, D, N)   as separate real / imaginary arrays
 *
 * Operator (reference: extension-cpp/extension_cpp/csrc/cuda/ssm_adaptive_unitary_forward.cu:83-181):
 *   theta_t = sum_r x[i][j][r] u[b][r][t] + x_bias[i][j]
 *   h_t     = exp(i theta_t) h_{t-1} + Bc_j dt_t silu(u_t)
 *   y_t     = silu(z_t) (Dskip_i silu(u_t) + sum_j Re(Cc_j h_t))
 */
#ifndef AUSSM_B200_H
#define AUSSM_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AUSSM_OK 0
#define AUSSM_EINVAL (-1)     /* bad size, null pointer, unsupported state count */
#define AUSSM_EWORKSPACE (-2) /* workspace missing or too small */
#define AUSSM_ECUDA (-3)      /* a CUDA runtime call failed */
#define AUSSM_EDEVICE (-4)    /* a kernel reported a failure through the device status word */

#define AUSSM_MAX_STATES 128  /* largest N the kernels are instantiated for */

typedef void* aussm_stream_t; /* a cudaStream_t */

/* Library version (major*10000 + minor*100 + patch). */
int aussm_b200_version(void);

/* Message of the last failure on the calling thread ("" if none). */
const char* aussm_b200_last_error(void);

/* Synchronises `stream`, then returns and clears the device status word:
 * 0 = every kernel ran to completion, 1 = a kernel gave up on a bounded wait
 * for a bulk copy (its outputs are then invalid). */
int aussm_b200_device_status(aussm_stream_t stream);

/* Number of kernels this library has launched in this process so far (all
 * threads, all devices): the difference around a region counts its launches. */
unsigned long long aussm_b200_kernel_launches(void);

/* Process-wide option (one atomic word, read at the start of every operator
 * call on whatever thread makes it - framework autograd engines run backward
 * calls on threads of their own).  "window_steps": steps per
 * time window of the windowed operators (rounded up to a multiple of 64; 0 =
 * automatic, about 2 GiB of phases per window).  It decides the layout of the
 * workspace and of a kept-phase buffer, so it is meant to be set once, before
 * the calls that should see it: a kept-phase backward call refuses a buffer
 * that was written under another value, and a call given a workspace sized
 * under another value returns AUSSM_EWORKSPACE; neither computes with a wrong
 * layout.  "time_split" (default 1): 0 turns the time-axis split of under-filled
 * scans off (see aussm_b200_scan_unitary_fwd_ws); it changes workspace sizes
 * too.  Returns AUSSM_EINVAL for an unknown name. */
int aussm_b200_set_option(const char* name, int value);

/* ---- scan core: the phase tensor theta is an input ----------------------
 * The reference has no operator at this boundary (its kernels rebuild theta
 * from x and u, ssm_adaptive_unitary_forward.cu:83-110); this is the
 * memory-bound part of the path, split out so that it can be measured and
 * sharded over batch x d_inner on its own. */
int aussm_b200_scan_unitary_fwd(const float* theta, const float* u, const float* dt, const float* z,
                                const float* B_r, const float* B_theta, const float* C_r, const float* C_theta,
                                const float* Dskip, const float* h0_re, const float* h0_im, /* may be NULL (= 0) */
                                float* y, float* h1_re, float* h1_im, /* h1 may be NULL */
                                int B, int D, int N, int L, aussm_stream_t stream);

/* Time-axis split.  The scans walk time sequentially and get their parallelism
 * from the B*D channels (the reference gets it from block scans over time,
 * ssm_adaptive_unitary_forward.cu:122-144, reverse_scan.h:152-302).  When the
 * channels fill less than a quarter of the GPU, the launch is cut into equal
 * time segments per channel: an aggregate pass gives every segment's end state
 * from zero and the product of its rotations, a short chain over the segments
 * gives every segment its true initial state (backward: its end state and the
 * incoming gradient, the rotations being invertible), and the real pass then
 * runs all segments side by side.  Same results up to float32 rounding.  The
 * split needs scratch: aussm_b200_scan_unitary_fwd_ws is
 * aussm_b200_scan_unitary_fwd with a workspace of
 * aussm_b200_scan_unitary_fwd_workspace_bytes bytes (0 = this shape is not
 * split and the workspace may be NULL); the backward entry point and the drop-in
 * operators split by themselves inside the workspaces they already take. */
size_t aussm_b200_scan_unitary_fwd_workspace_bytes(int B, int D, int N, int L);
int aussm_b200_scan_unitary_fwd_ws(const float* theta, const float* u, const float* dt, const float* z,
                                   const float* B_r, const float* B_theta, const float* C_r, const float* C_theta,
                                   const float* Dskip, const float* h0_re, const float* h0_im, float* y, float* h1_re,
                                   float* h1_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                                   aussm_stream_t stream);

/* Scratch (bytes) the backward scan needs behind `workspace`. */
size_t aussm_b200_scan_unitary_bwd_workspace_bytes(int B, int D, int N, int L);

/* h1_* is the state after the last step as returned by the forward call (the
 * backward pass regenerates all earlier states from it); gh1_* its gradient
 * (NULL = 0).  dtheta may alias theta.  dh0_* may be NULL. */
int aussm_b200_scan_unitary_bwd(const float* grad_y, const float* gh1_re, const float* gh1_im, const float* theta,
                                const float* u, const float* dt, const float* z, const float* B_r,
                                const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                                const float* h1_re, const float* h1_im, float* dtheta, float* du, float* ddt,
                                float* dz, float* dB_r, float* dB_theta, float* dC_r, float* dC_theta, float* dD,
                                float* dh0_re, float* dh0_im, int B, int D, int N, int L, void* workspace,
                                size_t workspace_bytes, aussm_stream_t stream);

/* Backward scan for callers that cannot allocate device memory.  It has no
 * counterpart in the reference (whose host functions allocate their outputs
 * and temporaries through torch on every call).
 *
 * Same arguments and results as aussm_b200_scan_unitary_bwd, minus the
 * workspace: the scratch for the per-channel partial sums is a fixed array of
 * AUSSM_STATIC_SCRATCH_BYTES inside the library image.  It is meant for code
 * that runs where cudaMalloc or a framework allocator is off limits - inside a
 * serving loop that must not synchronise the device, in a plug-in that is
 * handed nothing but its input and output buffers, under a fixed memory plan -
 * and it calls no cudaMalloc, cudaFree or allocating library routine.
 *
 *  - Limit: B*D*(5*N+1)*4 bytes <= AUSSM_STATIC_SCRATCH_BYTES, otherwise
 *    AUSSM_EWORKSPACE is returned and nothing is launched.
 *  - Cost: the array is part of the library's device code.  The CUDA runtime
 *    loads device code lazily by default, so a GPU holds the 4 MiB from the
 *    first call of this function on it (from library load when
 *    CUDA_MODULE_LOADING=EAGER is set) until the process exits.
 *  - First call on a device: it makes the runtime load that code (which may
 *    reserve device memory and synchronise the device) and looks up the
 *    array's device address.  Make one warm-up call per device BEFORE the
 *    region in which allocation or synchronisation is off limits, and before
 *    starting any stream capture; every later call on that device only
 *    enqueues two kernels.  The address is cached per device ordinal for the
 *    life of the process (devices 0..63; a cudaDeviceReset invalidates it).
 *  - All calls on a device share the one array.  Each call overwrites every
 *    word it later reads, so earlier contents never matter, but two calls whose
 *    kernels overlap on the GPU (different streams) race on it: serialise them. */
#define AUSSM_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int aussm_b200_scan_unitary_bwd_static(const float* grad_y, const float* gh1_re, const float* gh1_im,
                                       const float* theta, const float* u, const float* dt, const float* z,
                                       const float* B_r, const float* B_theta, const float* C_r,
                                       const float* C_theta, const float* Dskip, const float* h1_re,
                                       const float* h1_im, float* dtheta, float* du, float* ddt, float* dz,
                                       float* dB_r, float* dB_theta, float* dC_r, float* dC_theta, float* dD,
                                       float* dh0_re, float* dh0_im, int B, int D, int N, int L,
                                       aussm_stream_t stream);

/* ---- float32-accurate tensor-core GEMM -------------------------------------
 * The contraction behind the phase projection theta = x u and its adjoints
 * (reference: the per-row loops of ssm_adaptive_unitary_forward.cu:83-110 and
 * the atomics of ssm_adaptive_unitary_backward.cu:419-490), exposed on its own.
 * C[M x N] (+)= A * B^T in the sense  C[m][n] = sum_k A(m,k) B(n,k), computed on
 * the tcgen05 tensor cores as a three-term product of FP16 hi/lo parts taken
 * after a power-of-two scaling by each tensor's largest magnitude (float32-level
 * accuracy over the whole float32 range).
 * Packed operands: x_mn_major == 0: stored (rows, K), K contiguous;
 * x_mn_major == 1: stored (K, rows), rows contiguous.  `batches` entries follow
 * each other for an operand with x_batched != 0; a non-batched operand is shared.
 * reduce_batches != 0: one C = sum over batches; else C holds `batches` M x N
 * results.  beta: 0 overwrite, 1 accumulate.  Any M, N, K and alignment: the
 * hi/lo parts are written into the workspace with 16-byte aligned rows. */
size_t aussm_b200_gemm_split3_workspace_bytes(int M, int N, int K, int batches, int a_mn_major, int a_batched,
                                              int b_mn_major, int b_batched);
int aussm_b200_gemm_split3(const float* A, int a_mn_major, int a_batched, const float* Bm, int b_mn_major,
                           int b_batched, float* C, int M, int N, int K, int batches, int reduce_batches, int beta,
                           void* workspace, size_t workspace_bytes, aussm_stream_t stream);
/* The same product on operands that are views of larger arrays: lda / ldb / ldc are the pitches of the slower
 * index in floats, x_batch_stride the distance between batch entries in floats (0 = the operand is shared by
 * all batch entries).  Same workspace size as the packed form. */
int aussm_b200_gemm_split3_strided(const float* A, int a_mn_major, long long lda, long long a_batch_stride,
                                   const float* Bm, int b_mn_major, long long ldb, long long b_batch_stride, float* C,
                                   long long ldc, long long c_batch_stride, int M, int N, int K, int batches,
                                   int reduce_batches, int beta, void* workspace, size_t workspace_bytes,
                                   aussm_stream_t stream);

/* ---- drop-in operators ---------------------------------------------------
 * aussm_b200_unitary_fwd replaces ssm_adaptive_cuda_forward_unitary
 * (ssm_adaptive_unitary_forward.cu:191-277, schema :284) and
 * aussm_b200_unitary_bwd replaces ssm_adaptive_cuda_backward_unitary
 * (ssm_adaptive_unitary_backward.cu:493-617, schema forward.cu:285): same
 * inputs, same outputs, same order.  Differences a caller sees: any L in one
 * launch sequence (the reference stops at 2048 steps per call), outputs need
 * not be zeroed, results are deterministic, nothing synchronises the device.
 * The phase tensor is never materialised for the whole sequence: the time
 * axis is processed in windows through `workspace`. */
size_t aussm_b200_unitary_workspace_bytes(int B, int D, int N, int L);

int aussm_b200_unitary_fwd(const float* u, const float* dt, const float* x, const float* x_bias, const float* B_r,
                           const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                           const float* z, const float* h0_re, const float* h0_im, float* y, float* h1_re,
                           float* h1_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                           aussm_stream_t stream);

/* h1_* (the forward call's final state) may be NULL: the state is then
 * recomputed by an extra forward sweep, as the reference's backward does
 * (ssm_adaptive_unitary_backward.cu:50-141). */
int aussm_b200_unitary_bwd(const float* grad_y, const float* gh1_re, const float* gh1_im, const float* u,
                           const float* dt, const float* x, const float* x_bias, const float* B_r,
                           const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                           const float* z, const float* h0_re, const float* h0_im, const float* h1_re,
                           const float* h1_im, float* du, float* ddt, float* dx, float* dx_bias, float* dB_r,
                           float* dB_theta, float* dC_r, float* dC_theta, float* dD, float* dz, float* dh0_re,
                           float* dh0_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                           aussm_stream_t stream);

/* The same pair with the phases kept between forward and backward (no
 * counterpart in the reference, whose backward recomputes every intermediate
 * from the 12 inputs: ssm_adaptive_unitary_backward.cu:50-141).  The forward
 * writes every window's phases into `theta_keep` (aussm_b200_unitary_keep_bytes
 * bytes, 256-byte aligned: about 4*B*D*N*L); the backward reads them instead
 * of running the projection again and overwrites them with their gradient, so
 * the buffer is consumed by one backward call.  The final state h1_* of the
 * forward call is required.  Results are bit-identical to the plain pair. */
size_t aussm_b200_unitary_keep_bytes(int B, int D, int N, int L);

int aussm_b200_unitary_fwd_keep(const float* u, const float* dt, const float* x, const float* x_bias,
                                const float* B_r, const float* B_theta, const float* C_r, const float* C_theta,
                                const float* Dskip, const float* z, const float* h0_re, const float* h0_im, float* y,
                                float* h1_re, float* h1_im, int B, int D, int N, int L, void* workspace,
                                size_t workspace_bytes, void* theta_keep, size_t keep_bytes, aussm_stream_t stream);

int aussm_b200_unitary_bwd_kept(const float* grad_y, const float* gh1_re, const float* gh1_im, const float* u,
                                const float* dt, const float* x, const float* x_bias, const float* B_r,
                                const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                                const float* z, const float* h0_re, const float* h0_im, const float* h1_re,
                                const float* h1_im, float* du, float* ddt, float* dx, float* dx_bias, float* dB_r,
                                float* dB_theta, float* dC_r, float* dC_theta, float* dD, float* dz, float* dh0_re,
                                float* dh0_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                                void* theta_keep, size_t keep_bytes, aussm_stream_t stream);

/* ---- real selective scan of the Mamba block ("S6") -------------------------
 * The reference's MambaBlock calls mamba_ssm.selective_scan_fn, a third-party
 * CUDA extension that is not part of the reference tree
 * (ai-modules/wavesAI/model/aussm.py:30, :791-802); these entry points provide
 * that operator with the call site's semantics:
 *   dlt = delta + delta_bias[i], through softplus when delta_softplus != 0
 *   h_t = exp(dlt_t A[i][j]) h_{t-1} + dlt_t Bm[b][j][t] u[b][i][t]
 *   out = (sum_j Cm[b][j][t] h_t + Dskip[i] u) * silu(z)        (Dskip, z, delta_bias may be NULL)
 * u, delta, z, out: (B, D, L); A: (D, N); Bm, Cm: (B, N, L).  L must be a
 * multiple of 4 and N <= 32.  `ckpt` (aussm_b200_selective_scan_ckpt_floats
 * floats; its layout belongs to the library) receives the state at every 16th
 * step (every 32nd for N > 16) and is what the backward pass restarts from
 * (NULL when no backward pass will follow).  dB and dC are summed
 * over the channels with float atomics (as in mamba-ssm), so they are
 * reproducible only up to rounding; everything else is deterministic. */
size_t aussm_b200_selective_scan_ckpt_floats(int B, int D, int N, int L);
size_t aussm_b200_selective_scan_bwd_workspace_bytes(int B, int D, int N, int L);
int aussm_b200_selective_scan_fwd(const float* u, const float* delta, const float* A, const float* Bm,
                                  const float* Cm, const float* Dskip, const float* z, const float* delta_bias,
                                  int delta_softplus, float* out, float* ckpt, float* last_state, int B, int D, int N,
                                  int L, aussm_stream_t stream);
int aussm_b200_selective_scan_bwd(const float* gout, const float* u, const float* delta, const float* A,
                                  const float* Bm, const float* Cm, const float* Dskip, const float* z,
                                  const float* delta_bias, int delta_softplus, const float* ckpt, float* du,
                                  float* ddelta, float* dA, float* dB, float* dC, float* dD, float* dz,
                                  float* ddelta_bias, int B, int D, int N, int L, void* workspace,
                                  size_t workspace_bytes, aussm_stream_t stream);

/* ---- general complex / positive-real scan ----------------------------------
 * The recurrence of the reference's ssm_adaptive_complex and
 * ssm_adaptive_preal kernels (csrc/cuda/ssm_adaptive_complex.cu:181-744,
 * ssm_adaptive_real.cu:115-560; compiled but never registered there):
 *   lambda_t = exp(rho_t + i theta_t),
 *   h_t = lambda_t h_{t-1} + Bc[b][j][t] dt_t silu(u_t),
 *   y_t = silu(z_t) (Dskip_i silu(u_t) + sum_j Re(Cc[b][j][t] h_t)).
 * B_re, B_im, C_re, C_im and their gradients: (B, N, L) (imaginary parts may be
 * NULL = 0: positive-real variant).  L multiple of 4, N <= 32.
 * `states` (aussm_b200_scan_complex_states_floats floats) is the state record,
 * this library's form of the reference's `hidden_states` output (real.cu:236,
 * complex.cu:324): (B, D, N, L/16 + 1) complex entries, entry k = the state
 * before step 16 k, the last entry the state after the final step.  The
 * backward pass restarts from it; `gstates` is its upstream gradient (NULL = 0).
 * dB / dC are summed over the channels with float atomics (as the reference's
 * kernels do), so they are reproducible only up to rounding.
 *
 * Scan core: the eigenvalue exponents rho, theta (B, D, N, L) are inputs
 * (either may be NULL = 0) and drho, dtheta outputs. */
size_t aussm_b200_scan_complex_states_floats(int B, int D, int N, int L);
size_t aussm_b200_scan_complex_bwd_workspace_bytes(int B, int D, int N, int L);
int aussm_b200_scan_complex_fwd(const float* rho, const float* theta, const float* u, const float* dt,
                                const float* z, const float* B_re, const float* B_im, const float* C_re,
                                const float* C_im, const float* Dskip, float* y, float* states, /* may be NULL */
                                int B, int D, int N, int L, aussm_stream_t stream);
int aussm_b200_scan_complex_bwd(const float* gy, const float* gstates, const float* rho, const float* theta,
                                const float* u, const float* dt, const float* z, const float* B_re,
                                const float* B_im, const float* C_re, const float* C_im, const float* Dskip,
                                const float* states, float* drho, float* dtheta, float* du, float* ddt, float* dz,
                                float* dB_re, float* dB_im, float* dC_re, float* dC_im, float* dD, int B, int D, int N,
                                int L, void* workspace, size_t workspace_bytes, aussm_stream_t stream);

/* Operators with the inputs of the reference's host functions:
 * aussm_b200_complex_fwd replaces ssm_adaptive_cuda_forward_complex
 * (ssm_adaptive_complex.cu:296-356) and, with has_theta == 0,
 * ssm_adaptive_cuda_forward_preal (ssm_adaptive_real.cu:211-265);
 * aussm_b200_complex_bwd replaces ssm_adaptive_cuda_backward_complex
 * (complex.cu:662-744) / ..._backward_preal (real.cu:490-560).  The exponents
 * rho = x_rho . u and theta = x_theta . u are computed inside, one time window
 * at a time through `workspace` (they are never materialised for the whole
 * sequence), and recomputed by the backward call.  x, dx: (2, D, N, D) = x_rho
 * then x_theta when has_theta != 0, (D, N, D) = x_rho otherwise.  B and C are
 * taken as real and imaginary parts (the reference's radius / angle pairs are
 * converted by the host layer). */
size_t aussm_b200_complex_workspace_bytes(int B, int D, int N, int L, int has_theta);
int aussm_b200_complex_fwd(const float* u, const float* dt, const float* x, int has_theta, const float* B_re,
                           const float* B_im, const float* C_re, const float* C_im, const float* Dskip,
                           const float* z, float* y, float* states, int B, int D, int N, int L, void* workspace,
                           size_t workspace_bytes, aussm_stream_t stream);
int aussm_b200_complex_bwd(const float* gy, const float* gstates, const float* u, const float* dt, const float* x,
                           int has_theta, const float* B_re, const float* B_im, const float* C_re, const float* C_im,
                           const float* Dskip, const float* z, const float* states, float* du, float* ddt, float* dx,
                           float* dB_re, float* dB_im, float* dC_re, float* dC_im, float* dD, float* dz, int B, int D,
                           int N, int L, void* workspace, size_t workspace_bytes, aussm_stream_t stream);

/* ---- element-wise stages of the AUSSM block, in the scan's (B, D, L) layout ----
 * What SSMauBlock does around the operator (ai-modules/wavesAI/model/aussm.py):
 * the causal depthwise convolution with bias over time (:858-864: transpose,
 * nn.Conv1d with padding K-1, cut back to L steps, transpose) and the step
 * size dt = softplus(dt_proj(.) + dt_proj.bias) (:878-880, the bias entering a
 * second time: scale = 1 adds it once to `pre`), each as one streaming pass
 * over (B, D, L) rows with no transposing copy, and their adjoints.
 *   u[b][i][t]  = bias[i] + sum_k w[i][k] xs[b][i][t - (K-1) + k]      w: (D, K), K <= AUSSM_MAX_CONV_TAPS
 *   dt[b][i][t] = softplus(pre[b][i][t] + scale * bias[i])             softplus as torch's default (threshold 20)
 * bias may be NULL.  The backward calls return the weight / bias gradients summed
 * over batch and time in a fixed order (deterministic); dt may alias pre and
 * dpre may alias ddt. */
#define AUSSM_MAX_CONV_TAPS 4
int aussm_b200_conv_pre_fwd(const float* xs, const float* w, const float* bias, float* u, int B, int D, int L, int K,
                            aussm_stream_t stream);
size_t aussm_b200_conv_pre_bwd_workspace_bytes(int B, int D);
int aussm_b200_conv_pre_bwd(const float* du, const float* xs, const float* w, float* dxs, float* dw,
                            float* dbias, /* may be NULL */
                            int B, int D, int L, int K, void* workspace, size_t workspace_bytes, aussm_stream_t stream);
int aussm_b200_softplus_bias_fwd(const float* pre, const float* bias, float scale, float* dt, int B, int D, int L,
                                 aussm_stream_t stream);
size_t aussm_b200_softplus_bias_bwd_workspace_bytes(int B, int D);
int aussm_b200_softplus_bias_bwd(const float* ddt, const float* dt, float scale, float* dpre,
                                 float* dbias, /* may be NULL */
                                 int B, int D, int L, void* workspace, size_t workspace_bytes, aussm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* AUSSM_B200_H */
