// Float32-accurate GEMM on the 5th-generation tensor cores (tcgen05, TMEM
// accumulators, TMA operand staging) by the three-term split
//     a*b ~ a_hi*b_hi + a_hi*b_lo + a_lo*b_hi
// on FP16 parts: with S the power of two that brings the tensor's largest
// magnitude to about 2^14,  hi = fp16(S a),  lo = fp16((S a - hi) 2^11).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "host_common.cuh"

namespace aussm {

// One operand, already split into its two FP16 parts by split_f16.  `mn_major == 0`: stored as [rows][K] with K
// contiguous; `mn_major == 1`: stored as [K][rows] with the row (M or N) index contiguous.  `ld` is the pitch of
// the slower index in halves (a multiple of 8), `batch_stride` the distance between batch entries (halves,
// multiple of 8, 0 for an operand shared by all batch entries).  `amax` points to the bit pattern of the
// tensor's largest magnitude on the device (the parts are scaled by a power of two derived from it).
struct SplitOperand {
    const void* hi;
    const void* lo;
    int mn_major;
    long long ld;
    long long batch_stride;
    const unsigned* amax;
};

struct GemmShape {
    int M, N, K;
    int batches;          // number of operand batch entries
    int reduce_batches;   // 0: one output per batch entry; g >= 1: the batch entries are summed in g groups of
                          // batches / g consecutive entries, one output per group (g = 1: C = sum over all)
    int beta;             // 0: overwrite C, 1: add to C
    long long ldc;        // floats; any value (rows that are not 16-byte aligned take scalar stores)
    long long c_batch_stride;
};

// Halves to reserve for one part of a split operand that holds `halves` values: rounded up to 256 bytes, with
// room for the up to 63 halves that the last copy of an MN-major operand reads past the end of its last row.
// The lo part must follow the hi part (one tensor map covers both).
inline size_t split_part_halves(size_t halves) { return (halves + 64 + 127) / 128 * 128; }

// C[m][n] (+)= sum_k A(m,k) B(n,k).  Returns 0 or a negative AUSSM_E* code.
int gemm_split3(const SplitOperand& A, const SplitOperand& B, float* C, const GemmShape& s, cudaStream_t stream);

// true when the split operands meet the alignment rules of the TMA path (pitches multiple of 8 halves, 16-byte bases)
bool gemm_split3_supported(const SplitOperand& A, const SplitOperand& B, const float* C, const GemmShape& s);

// FP16 hi/lo split of a strided 2-D float32 array (rows x cols, cols contiguous, any pitch and alignment),
// batched.  ld_dst / dst_batch_stride count halves and are multiples of 8, ld_dst >= cols rounded up to 4.
// amax is a device word that receives the bit pattern of max|src|; have_amax: *amax already holds the maximum
// (its producer computed it) and the pass over src that finds it is skipped.
int split_f16(const float* src, long long ld_src, long long src_batch_stride, void* hi, void* lo, long long ld_dst,
              long long dst_batch_stride, long long rows, long long cols, int batches, unsigned* amax,
              cudaStream_t stream, bool have_amax = false);

}  // namespace aussm
