// Parameter blocks and launchers of the unitary scan-core kernels.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "host_common.cuh"

namespace aussm {

// All row pointers address element t = 0 of the launch; a row is L floats
// long and rows are ld_* floats apart (so a launch can work on a window of a
// longer sequence, or on a packed workspace).
struct ScanFwdParams {
    const float* theta;        // (nch, N, L) rows, ld_theta apart
    const float* theta_bias;   // (D, N) added to every phase, or nullptr
    const float* u;            // (nch, L) rows, ld_row apart
    const float* dt;
    const float* z;
    const float* B_r;          // (N,)
    const float* B_theta;
    const float* C_r;
    const float* C_theta;
    const float* Dskip;        // (D,)
    const float* h0_re;        // (nch, N) or nullptr (= 0)
    const float* h0_im;
    float* y;                  // (nch, L) rows, ld_row apart, or nullptr (state only)
    float* h1_re;              // (nch, N) or nullptr
    float* h1_im;
    int nch;                   // batch * d_inner channels
    int Dmod;                  // d_inner (channel i = ch % Dmod)
    int N;                     // states per channel
    int L;                     // steps in this launch
    long long ld_theta;
    long long ld_row;
    int* status;               // device status word (filled in by the launcher)
};

struct ScanBwdParams {
    const float* theta;
    const float* theta_bias;
    const float* u;
    const float* dt;
    const float* z;
    const float* gy;           // upstream gradient of y, (nch, L) rows
    const float* B_r;
    const float* B_theta;
    const float* C_r;
    const float* C_theta;
    const float* Dskip;
    const float* h1_re;        // state AFTER the last step of this launch (from the forward)
    const float* h1_im;
    const float* gh1_re;       // gradient of that state, or nullptr (= 0)
    const float* gh1_im;
    float* dtheta;             // (nch, N, L) rows, ld_dtheta apart (may alias theta)
    float* du;                 // direct part only (rows ld_row apart)
    float* ddt;
    float* dz;
    float* dh0_re;             // gradient of the state before step 0, or nullptr (may alias gh1)
    float* dh0_im;
    float* h0_re;              // regenerated state before step 0, or nullptr (may alias h1)
    float* h0_im;
    float* part_bc;            // (nch, N, 4): grad of Bc (re, im), grad of Cc (re, im)
    float* part_d;             // (nch,)
    float* part_rowsum;        // (nch, N) sum over t of dtheta, or nullptr
    unsigned* dtheta_amax;     // receives (atomic max) the bit pattern of max|dtheta| of this launch, or nullptr;
                               // only with theta_bias / part_rowsum given (the drop-in pipeline)
    int accumulate;            // 1: add to the partial buffers instead of overwriting them
    int nch, Dmod, N, L;
    long long ld_theta;
    long long ld_dtheta;
    long long ld_row;
    int* status;
};

struct ReduceParams {
    const float* part_bc;
    const float* part_d;
    const float* part_rowsum;  // or nullptr
    const float* B_r;
    const float* B_theta;
    const float* C_r;
    const float* C_theta;
    float* dB_r;
    float* dB_theta;
    float* dC_r;
    float* dC_theta;
    float* dD;
    float* dx_bias;            // (D, N) or nullptr
    int batch, D, N;
};

cudaError_t launch_scan_unitary_fwd(const ScanFwdParams& p, cudaStream_t stream);
cudaError_t launch_scan_unitary_bwd(const ScanBwdParams& p, cudaStream_t stream);
cudaError_t launch_reduce_param_grads(const ReduceParams& p, cudaStream_t stream);

// floats of scratch behind part_bc / part_d / part_rowsum for a launch
inline size_t scan_bwd_partial_floats(long long nch, int N) { return (size_t)nch * (size_t)(5 * N + 1); }

}  // namespace aussm
