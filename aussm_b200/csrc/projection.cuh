// Phase projection of the drop-in operator and its two adjoints, on a time
// window [t0, t0+tl) of the sequence:
//   theta_w[b][m][t] = sum_r x[m][r] u[b][r][t0+t]            m = i*N + j
//   dx[m][r]        += sum_b sum_t dtheta_w[b][m][t] u[b][r][t0+t]
//   du[b][r][t0+t]  += sum_m x[m][r] dtheta_w[b][m][t]
// (reference: ssm_adaptive_unitary_forward.cu:83-110 builds theta row by row,
// ssm_adaptive_unitary_backward.cu:419-490 forms the adjoints with atomics.)
// These are dense contractions that must keep float32 accuracy (an 11-bit
// product alone would put 1e-3 relative error on every phase): they run on the
// tcgen05 kernel of gemm_split3.cu as three-term products of FP16 parts.  Any
// D and L are accepted: the FP16 parts are written into scratch rows whose
// pitch is a multiple of 16 bytes whatever the shape of the source.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "host_common.cuh"

namespace aussm {

struct ProjDims {
    int B, D;             // batch, d_inner
    long long M;          // rows of x: d_inner * states (twice that when two streams are projected at once)
    long long L;          // row length of u / du
    long long ldw;        // row pitch of the window workspace (floats; a multiple of 8)
    long long t0;
    int tl;
};

// Scratch for the FP16 hi/lo parts of the operands (caller-owned, inside the operator workspace).
struct ProjScratch {
    void* x_hi;       // (M, Dp) halves, Dp = D rounded up to 8
    void* x_lo;
    void* u_hi;       // (B, D, ldw)      window of u
    void* u_lo;
    void* dth_hi;     // (B, M, ldw)      window of dtheta
    void* dth_lo;
    float* dx_part;   // (2, M, D)        partial sums of dx when the batch is summed in two groups
    unsigned* amax;   // bit patterns of max|x|, max|u window|, max|dtheta window|
    long long Dp;
};

// bytes needed behind ProjScratch for a window pitch ldw
size_t proj_scratch_bytes(int B, int D, long long M, long long ldw);
void proj_scratch_bind(ProjScratch& s, void* base, int B, int D, long long M, long long ldw);

// returns 0 or a negative AUSSM_E* code (message set)
// Splits x (once per operator call).
int proj_begin(int D, long long M, const float* x, ProjScratch& s, cudaStream_t stream);
// FP16 parts of the current window of u (proj_theta does this itself; proj_adjoints expects it done).
int proj_split_u(const ProjDims& d, const float* u, ProjScratch& s, cudaStream_t stream);
int proj_theta(const ProjDims& d, const float* u, float* theta_w, ProjScratch& s, cudaStream_t stream);
// dx and du from dtheta_w; requires the split of u of the same window (proj_theta or proj_split_u).
// dtheta_amax_known: s.amax[2] already holds the bit pattern of max|dtheta_w| (the scan kernel produced it)
int proj_adjoints(const ProjDims& d, const float* dtheta_w, float* dx, float* du, bool overwrite_dx, ProjScratch& s,
                  cudaStream_t stream, bool dtheta_amax_known = false);

}  // namespace aussm
