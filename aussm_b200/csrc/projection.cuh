// Phase projection of the drop-in operator and its two adjoints, on a time
// window [t0, t0+tl) of the sequence:
//   theta_w[b][m][t] = sum_r x[m][r] u[b][r][t0+t]            m = i*N + j
//   dx[m][r]        += sum_b sum_t dtheta_w[b][m][t] u[b][r][t0+t]
//   du[b][r][t0+t]  += sum_m x[m][r] dtheta_w[b][m][t]
// (reference: ssm_adaptive_unitary_forward.cu:83-110 builds theta row by row,
// ssm_adaptive_unitary_backward.cu:419-490 forms the adjoints with atomics.)
// These are dense contractions that must keep float32 accuracy (TF32 alone
// would put 1e-3 relative error on every phase).  Default: the tcgen05 kernel
// of gemm_tf32x3.cu (three-term TF32 split); fallback: library SGEMM.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace aussm {

struct ProjDims {
    int B, D, N;          // batch, d_inner, states
    long long L;          // row length of u / du
    long long ldw;        // row pitch of the window workspace (floats)
    long long t0;
    int tl;
};

// Scratch for the hi/lo parts of the operands (caller-owned, inside the operator workspace); sized for TF32
// parts (one float per value and part), FP16 parts use half of it.
struct ProjScratch {
    float* x_hi;      // (D*N, D)
    float* x_lo;
    float* u_hi;      // (B, D, ldw)      window of u
    float* u_lo;
    float* dth_hi;    // (B, D*N, ldw)    window of dtheta
    float* dth_lo;
    unsigned* amax;   // FP16 parts: bit patterns of max|x|, max|u window|, max|dtheta window|
    int use_tensor_cores;   // decided once per operator call by proj_begin()
    int half;               // 1: FP16 parts (the buffers above hold halves), 0: TF32 parts
};

// floats needed behind ProjScratch for a window pitch ldw
size_t proj_scratch_floats(int B, int D, int N, long long ldw);
void proj_scratch_bind(ProjScratch& s, float* base, int B, int D, int N, long long ldw);

// Chooses the backend for this call and splits x when the tensor-core path is used.
int proj_begin(int B, int D, int N, long long L, long long ldw, const float* x, const float* u, ProjScratch& s,
               cudaStream_t stream);

// returns 0 or a negative AUSSM_E* code (message set)
// TF32 parts of the current window of u (proj_theta does this itself; proj_adjoints expects it done).
int proj_split_u(const ProjDims& d, const float* u, ProjScratch& s, cudaStream_t stream);
int proj_theta(const ProjDims& d, const float* x, const float* u, float* theta_w, ProjScratch& s,
               cudaStream_t stream);
// dx and du from dtheta_w; requires proj_theta() to have run on the same window (it leaves u's split behind)
// dtheta_amax_known: s.amax[2] already holds the bit pattern of max|dtheta_w| (the scan kernel produced it)
int proj_adjoints(const ProjDims& d, const float* dtheta_w, const float* x, const float* u, float* dx, float* du,
                  bool overwrite_dx, ProjScratch& s, cudaStream_t stream, bool dtheta_amax_known = false);

void set_error(const char* fmt, ...);
void set_gemm_backend(int mode);   // 0: tensor cores, FP16 parts when the pitches allow; 1: library SGEMM; 2: TF32 parts
int gemm_backend();

}  // namespace aussm
