// General complex (and positive-real) diagonal selective scan: the recurrence
// of the reference's ssm_adaptive_complex / ssm_adaptive_preal kernels
// (csrc/cuda/ssm_adaptive_complex.cu:181-293, ssm_adaptive_real.cu:115-208;
// oracles extension_cpp/ops.py:233-357), with the per-element eigenvalue given
// as log-magnitude rho and phase theta:
//     lambda_t = exp(rho_t + i theta_t)
//     h_t = lambda_t h_{t-1} + Bc_jt dt_t silu(u_t)          Bc, Cc: (batch, N, L) complex
//     y_t = silu(z_t) (D_i silu(u_t) + sum_j Re(Cc_jt h_t))
// theta == nullptr and B_im == C_im == nullptr give the positive-real variant.
//
// A launch covers `L` steps that may be a window of a longer sequence: every
// pointer addresses step 0 of the window, rows keep the pitch of the tensor
// they lie in, and the state travels between launches through the state
// record (the reference's `hidden_states`, real.cu:236 / complex.cu:324).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "host_common.cuh"

namespace aussm {

constexpr int kCplxTile = 16;     // steps per tile; the forward pass records the state at every tile start

struct CplxFwdParams {
    const float* rho;         // row (b, i, j) at rho + b * lam_batch_stride + (i * N + j) * ld_lam, or nullptr (= 0)
    const float* theta;       // likewise, or nullptr (= 0)
    const float* u;           // (nch, .) rows, ld_row apart
    const float* dt;
    const float* z;
    const float* B_re;        // (batch, N, .) rows, ld_row apart
    const float* B_im;        // or nullptr
    const float* C_re;
    const float* C_im;        // or nullptr
    const float* Dskip;       // (D,)
    float* y;                 // (nch, .) rows, ld_row apart
    // State record: (nch, N, states_stride) complex entries; entry tile0 + k is the state before step 16 k of
    // this launch, entry tile0 + ntiles the state after its last step.  The launch starts from entry tile0
    // when tile0 > 0 and from zero otherwise.  nullptr: single launch from zero, nothing recorded.
    float* states;
    long long states_stride;
    int tile0;
    int nch, Dmod, N, L;
    long long ld_lam, lam_batch_stride, ld_row;
};

struct CplxBwdParams {
    const float* gy;
    const float* rho;
    const float* theta;
    const float* u;
    const float* dt;
    const float* z;
    const float* B_re;
    const float* B_im;
    const float* C_re;
    const float* C_im;
    const float* Dskip;
    const float* states;      // the forward pass's record (required)
    const float* gstates;     // gradient of the state record (same layout), or nullptr (= 0)
    long long states_stride;
    int tile0;
    float* drho;              // same addressing as rho; nullptr when rho is nullptr (may alias rho)
    float* dtheta;            // likewise
    float* du;                // direct part
    float* ddt;
    float* dz;
    float* dB_re;             // (batch, N, .): zeroed by the caller, float atomics
    float* dB_im;             // or nullptr
    float* dC_re;
    float* dC_im;             // or nullptr
    float* part_D;            // (nch,)
    const float* eta_in;      // (nch, N, 2) adjoint state handed over by the launch of the following window, or nullptr (= 0)
    float* eta_out;           // adjoint state for the launch of the preceding window, or nullptr (may alias eta_in)
    int accumulate;           // 1: add to part_D instead of overwriting it
    int nch, Dmod, N, L;
    long long ld_lam, lam_batch_stride, ld_row;
};

inline long long cplx_ntiles(long long L) { return (L + kCplxTile - 1) / kCplxTile; }

cudaError_t launch_cplx_fwd(const CplxFwdParams& p, cudaStream_t stream);
cudaError_t launch_cplx_bwd(const CplxBwdParams& p, cudaStream_t stream);
cudaError_t launch_cplx_reduce_D(const float* part_D, float* dD, int batch, int D, cudaStream_t stream);

}  // namespace aussm
