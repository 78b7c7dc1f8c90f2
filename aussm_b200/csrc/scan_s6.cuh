// Real selective scan of the Mamba block ("S6"), the operator the reference
// calls as mamba_ssm.selective_scan_fn in MambaBlock.ssm_mamba
// (ai-modules/wavesAI/model/aussm.py:771-805):
//     dlt_t = softplus(delta_t + delta_bias_i)            (softplus and bias optional)
//     h_t   = exp(dlt_t A_ij) h_{t-1} + dlt_t B_jt u_t
//     y_t   = sum_j C_jt h_t + D_i u_t ;  out_t = y_t * silu(z_t)   (gate optional)
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace aussm {

constexpr int kS6Tile = 32;      // steps per tile; the forward pass stores the state at every tile start
// Channel-per-thread kernels (scan_s6_wide.cu) serve N <= kS6WideStates: 16-step tiles, record (nch, tiles, N)
constexpr int kS6WideTile = 16;
constexpr int kS6WideStates = 16;

struct S6FwdParams {
    const float* u;           // (nch, L)
    const float* delta;       // (nch, L)
    const float* A;           // (D, N)
    const float* Bm;          // (batch, N, L)
    const float* Cm;          // (batch, N, L)
    const float* Dskip;       // (D,) or nullptr
    const float* z;           // (nch, L) or nullptr
    const float* delta_bias;  // (D,) or nullptr
    float* out;               // (nch, L)
    float* ckpt;              // state at the start of every tile, or nullptr: (nch, N, tiles of 32 steps) for
                              // N > 16, (nch, tiles of 16 steps, N) for N <= 16
    float* last_state;        // (nch, N) or nullptr
    int delta_softplus;
    int nch, Dmod, N, L;
};

struct S6BwdParams {
    const float* gout;        // (nch, L)
    const float* u;
    const float* delta;
    const float* A;
    const float* Bm;
    const float* Cm;
    const float* Dskip;
    const float* z;
    const float* delta_bias;
    const float* ckpt;        // from the forward pass
    float* du;                // (nch, L)
    float* ddelta;            // (nch, L)
    float* dz;                // (nch, L) or nullptr when z is nullptr
    float* dB;                // (batch, N, L), zeroed by the launcher, accumulated with float atomics
    float* dC;
    float* part_A;            // (nch, N) per-channel partial of dA
    float* part_D;            // (nch,)
    float* part_bias;         // (nch,)
    int delta_softplus;
    int nch, Dmod, N, L;
};

struct S6ReduceParams {
    const float* part_A;
    const float* part_D;
    const float* part_bias;
    float* dA;                // (D, N)
    float* dD;                // (D,) or nullptr
    float* dbias;             // (D,) or nullptr
    int batch, D, N;
};

inline bool s6_wide(int N) { return N <= kS6WideStates; }
// tiles of the state record (its size is nch * N * tiles floats in both layouts)
inline long long s6_ntiles(long long L, int N) {
    const int t = s6_wide(N) ? kS6WideTile : kS6Tile;
    return (L + t - 1) / t;
}

cudaError_t launch_s6_fwd(const S6FwdParams& p, cudaStream_t stream);
cudaError_t launch_s6_bwd(const S6BwdParams& p, cudaStream_t stream);
cudaError_t launch_s6_reduce(const S6ReduceParams& p, cudaStream_t stream);
// N <= kS6WideStates
cudaError_t launch_s6_wide_fwd(const S6FwdParams& p, cudaStream_t stream);
cudaError_t launch_s6_wide_bwd(const S6BwdParams& p, cudaStream_t stream);

}  // namespace aussm
