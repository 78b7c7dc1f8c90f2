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
    int nch;                   // batch * d_inner channels (times nseg when the time axis is split)
    int Dmod;                  // d_inner (channel i = ch % Dmod)
    int N;                     // states per channel
    int L;                     // steps in this launch (per segment when the time axis is split)
    long long ld_theta;
    long long ld_row;
    int* status;               // device status word (filled in by the launcher)
    // Time-axis split: nseg > 1 makes every channel nseg "virtual channels", one per segment of L steps; virtual
    // channel v = ch * nseg + s works on steps [s L, (s+1) L) of channel ch.  Rows are addressed through the real
    // channel and the segment; the per-channel state arrays (h0, h1, agg) are indexed by v.
    int nseg;                  // 0 or 1: no split
    // Aggregate mode (y == nullptr and agg_re != nullptr): besides the state after the segment (h1) the launch
    // returns the product of the segment's rotations, so that  h_end = h1_from_zero + agg * h_start.
    float* agg_re;             // (nch, N) or nullptr
    float* agg_im;
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
    int nseg;                  // time-axis split, as in ScanFwdParams (state and partial arrays indexed by v)
    // Adjoint-only mode (eta_only != 0): nothing but dh0 is produced - the gradient that the segment's own
    // grad_y sends to the state before it, from a zero gradient after it (gh1 is ignored).
    int eta_only;
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
    int nseg;                  // partial arrays hold nseg entries per channel (0 or 1: one)
};

cudaError_t launch_scan_unitary_fwd(const ScanFwdParams& p, cudaStream_t stream);
cudaError_t launch_scan_unitary_bwd(const ScanBwdParams& p, cudaStream_t stream);
cudaError_t launch_reduce_param_grads(const ReduceParams& p, cudaStream_t stream);

// floats of scratch behind part_bc / part_d / part_rowsum for a launch
inline size_t scan_bwd_partial_floats(long long nch, int N) { return (size_t)nch * (size_t)(5 * N + 1); }

// Time-axis split.  A launch whose channels fill less than a quarter of the GPU is cut into `nseg` equal
// segments per channel (0 or 1: not worth it, or the length does not divide).  `bwd`: for the backward kernel
// (fewer resident warps per SM).
int scan_split_segments(long long nch, int N, int L, bool bwd);
// true when the launch's pointers and pitches allow the split (16-byte aligned rows: the bulk-copy path)
bool scan_split_allowed(const ScanFwdParams& p);
bool scan_split_allowed(const ScanBwdParams& p);
// The split launches.  `p` describes the whole launch (p.nch real channels, p.L steps, nseg ignored); scratch:
// 6 (forward) / 10 (backward) * nch * nseg * N floats.  Backward: p.part_bc / part_d / part_rowsum hold nseg
// entries per channel (layout [channel][segment]) and the reduction must be told nseg.
inline size_t scan_split_fwd_scratch_floats(long long nch, int nseg, int N) { return (size_t)6 * nch * nseg * N; }
inline size_t scan_split_bwd_scratch_floats(long long nch, int nseg, int N) { return (size_t)10 * nch * nseg * N; }
cudaError_t scan_unitary_fwd_split(const ScanFwdParams& p, int nseg, float* scratch, cudaStream_t stream);
cudaError_t scan_unitary_bwd_split(const ScanBwdParams& p, int nseg, float* scratch, cudaStream_t stream);

// state after every segment from the aggregates of the forward pre-pass:  c_{s+1} = e_s + a_s c_s
//   e, a: (nch, nseg, N) pairs of arrays;  start: (nch, N) or nullptr (= 0);
//   before: (nch, nseg, N) receives c_s (the state before segment s);  final: (nch, N) receives c_nseg
cudaError_t launch_segment_states_fwd(const float* e_re, const float* e_im, const float* a_re, const float* a_im,
                                      const float* start_re, const float* start_im, float* before_re,
                                      float* before_im, float* final_re, float* final_im, long long nch, int nseg,
                                      int N, cudaStream_t stream);
// state after every segment walking back from the final state:  c_s = conj(a_s) (c_{s+1} - e_s)
//   after: (nch, nseg, N) receives c_{s+1} (the state after segment s)
//   first: (nch, N) receives c_0 (the state before the first segment), or nullptr
cudaError_t launch_segment_states_bwd(const float* e_re, const float* e_im, const float* a_re, const float* a_im,
                                      const float* final_re, const float* final_im, float* after_re, float* after_im,
                                      float* first_re, float* first_im, long long nch, int nseg, int N,
                                      cudaStream_t stream);
// adjoint state after every segment:  g_s = l_s + conj(a_s) g_{s+1}
//   l: the segments' own contributions (nch, nseg, N);  last: (nch, N) gradient of the final state or nullptr;
//   after: (nch, nseg, N) receives g_{s+1}
//   first: (nch, N) receives g_0 (the gradient of the state before the first segment), or nullptr
cudaError_t launch_segment_adjoints(const float* l_re, const float* l_im, const float* a_re, const float* a_im,
                                    const float* last_re, const float* last_im, float* after_re, float* after_im,
                                    float* first_re, float* first_im, long long nch, int nseg, int N,
                                    cudaStream_t stream);

}  // namespace aussm
