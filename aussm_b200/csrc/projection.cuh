// Phase projection of the drop-in operator and its two adjoints, on a time
// window [t0, t0+tl) of the sequence:
//   theta_w[b][m][t] = sum_r x[m][r] u[b][r][t0+t]            m = i*N + j
//   dx[m][r]        += sum_b sum_t dtheta_w[b][m][t] u[b][r][t0+t]
//   du[b][r][t0+t]  += sum_m x[m][r] dtheta_w[b][m][t]
// (reference: ssm_adaptive_unitary_forward.cu:83-110 builds theta row by row,
// ssm_adaptive_unitary_backward.cu:419-490 forms the adjoints with atomics.)
// These are plain dense contractions in float32 (TF32 would put 1e-3 relative
// error on every phase) and are issued as library GEMMs.
#pragma once

#include <cuda_runtime.h>

namespace aussm {

struct ProjDims {
    int B, D, N;          // batch, d_inner, states
    long long L;          // row length of u / du
    long long ldw;        // row pitch of the window workspace (floats)
    long long t0;
    int tl;
};

// returns 0 or a negative AUSSM_E* code (message set)
int proj_theta(const ProjDims& d, const float* x, const float* u, float* theta_w, cudaStream_t stream);
int proj_dx(const ProjDims& d, const float* dtheta_w, const float* u, float* dx, bool overwrite, cudaStream_t stream);
int proj_du(const ProjDims& d, const float* dtheta_w, const float* x, float* du, cudaStream_t stream);

void set_error(const char* fmt, ...);

}  // namespace aussm
