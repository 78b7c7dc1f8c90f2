// Float32-accurate GEMM on the 5th-generation tensor cores (tcgen05, TMEM
// accumulators, TMA operand staging) by the three-term TF32 split
//     a*b ~ a_hi*b_hi + a_hi*b_lo + a_lo*b_hi,   a_hi = tf32(a), a_lo = tf32(a - a_hi).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace aussm {

// One operand, already split into its two TF32 parts.  `mn_major == 0`: stored
// as [rows][K] with K contiguous; `mn_major == 1`: stored as [K][rows] with the
// row (M or N) index contiguous.  `ld` is the pitch of the slower index in
// floats (a multiple of 4), `batch_stride` the distance between batch entries.
//
// Two kinds of parts.  amax == nullptr: TF32 parts stored as floats.  amax != nullptr: FP16 parts (hi / lo point to
// __half arrays, ld and batch_stride count halves and are multiples of 8) written by split_f16, which scales the
// tensor by a power of two derived from its largest magnitude; `amax` points to that magnitude's bit pattern on
// the device.  FP16 parts have the same 2 x 11 significant bits as TF32 parts but move half the bytes and run
// at twice the tensor-core rate.
struct SplitOperand {
    const void* hi;
    const void* lo;
    int mn_major;
    long long ld;
    long long batch_stride;
    const unsigned* amax = nullptr;
};

struct GemmShape {
    int M, N, K;
    int batches;          // number of operand batch entries
    int reduce_batches;   // 1: C = sum over batches (one output); 0: one output per batch entry
    int beta;             // 0: overwrite C, 1: add to C
    long long ldc;
    long long c_batch_stride;
};

// C (+)= A * B^T-like product described above.  Returns 0 or a negative AUSSM_E* code.
int gemm_tf32x3(const SplitOperand& A, const SplitOperand& B, float* C, const GemmShape& s, cudaStream_t stream);

// true when the shapes meet the alignment rules of the TMA path (pitches multiple of 4 floats, 16-byte bases)
bool gemm_tf32x3_supported(const SplitOperand& A, const SplitOperand& B, const float* C, const GemmShape& s);

// hi/lo split of a strided 2-D array (rows x cols, cols contiguous), batched
int split_tf32(const float* src, long long ld_src, long long src_batch_stride, float* hi, float* lo, long long ld_dst,
               long long dst_batch_stride, long long rows, long long cols, int batches, cudaStream_t stream);

// 1: clusters of two CTAs share the B tile (256 x 256 per pair); 0 (default): one CTA per 128 x 256 tile
void set_gemm_pair(int on);
// measurement only, results invalid: 1 skip the accumulator drain, 2 skip operand refills, 4 skip the MMAs
void set_gemm_probe(int bits);

// FP16 hi/lo split (see SplitOperand); amax is a device word that receives the bit pattern of max|src|
// have_amax: *amax already holds the maximum (its producer computed it): the pass over src is skipped
int split_f16(const float* src, long long ld_src, long long src_batch_stride, void* hi, void* lo, long long ld_dst,
              long long dst_batch_stride, long long rows, long long cols, int batches, unsigned* amax,
              cudaStream_t stream, bool have_amax = false);

}  // namespace aussm
