// General complex (and positive-real) diagonal selective scan: the recurrence
// of the reference's ssm_adaptive_complex / ssm_adaptive_preal kernels
// (csrc/cuda/ssm_adaptive_complex.cu:181-293, ssm_adaptive_real.cu:115-208;
// oracles extension_cpp/ops.py:233-357), with the per-element eigenvalue given
// as log-magnitude rho and phase theta:
//     lambda_t = exp(rho_t + i theta_t)
//     h_t = lambda_t h_{t-1} + Bc_jt dt_t silu(u_t)          Bc, Cc: (batch, N, L) complex
//     y_t = silu(z_t) (D_i silu(u_t) + sum_j Re(Cc_jt h_t))
// theta == nullptr and B_im == C_im == nullptr give the positive-real variant.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace aussm {

constexpr int kCplxTile = 32;     // steps per tile; the forward pass stores the state at every tile start

struct CplxFwdParams {
    const float* rho;         // (nch, N, L) or nullptr (= 0)
    const float* theta;       // (nch, N, L) or nullptr (= 0)
    const float* u;           // (nch, L)
    const float* dt;
    const float* z;
    const float* B_re;        // (batch, N, L)
    const float* B_im;        // or nullptr
    const float* C_re;
    const float* C_im;        // or nullptr
    const float* Dskip;       // (D,)
    float* y;                 // (nch, L)
    float* ckpt;              // (nch, N, ntiles, 2) or nullptr
    int nch, Dmod, N, L;
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
    const float* ckpt;
    float* drho;              // (nch, N, L) or nullptr when rho is nullptr
    float* dtheta;            // likewise
    float* du;                // direct part
    float* ddt;
    float* dz;
    float* dB_re;             // (batch, N, L): zeroed by the launcher, float atomics
    float* dB_im;             // or nullptr
    float* dC_re;
    float* dC_im;             // or nullptr
    float* part_D;            // (nch,)
    int nch, Dmod, N, L;
};

inline long long cplx_ntiles(long long L) { return (L + kCplxTile - 1) / kCplxTile; }

cudaError_t launch_cplx_fwd(const CplxFwdParams& p, cudaStream_t stream);
cudaError_t launch_cplx_bwd(const CplxBwdParams& p, cudaStream_t stream);
cudaError_t launch_cplx_reduce_D(const float* part_D, float* dD, int batch, int D, cudaStream_t stream);

}  // namespace aussm
