// Element-wise stages of the AUSSM block around the scan operator, in the
// scan's own (batch, channel, time) layout, so that the block needs no
// transposing copies and no separate bias / activation passes:
//
//   causal depthwise convolution + bias   u[b][i][t] = bias[i] + sum_k w[i][k] xs[b][i][t - (K-1) + k]
//       (the reference transposes to (b, d, l), calls nn.Conv1d with padding K-1, cuts the result back to l
//        steps and transposes again: ai-modules/wavesAI/model/aussm.py:858-864)
//   step size                             dt[b][i][t] = softplus(pre[b][i][t] + scale * bias[i])
//       (the reference adds dt_proj's bias a second time and applies softplus as two passes, aussm.py:878-880)
//
// and their adjoints.  All four are streaming kernels: one pass over the rows, 128-bit accesses where the rows
// are 16-byte aligned.  Sums over batch and time (weight and bias gradients) are two-stage and deterministic:
// one block per (batch entry, channel) row leaves its partial sums, a second kernel adds them over the batch.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../../include/aussm_b200.h"
#include "common.cuh"
#include "host_common.cuh"

namespace aussm {
namespace {

constexpr int KMAX = AUSSM_MAX_CONV_TAPS;
constexpr int ROW_THREADS = 256;

struct Taps {
    float w[KMAX];
};

__device__ __forceinline__ Taps load_taps(const float* w, int i, int K) {
    Taps t;
#pragma unroll
    for (int k = 0; k < KMAX; ++k) t.w[k] = k < K ? w[(long long)i * K + k] : 0.f;
    return t;
}

// ---- forward: u = conv(xs) + bias -------------------------------------------------------------
// one thread per four consecutive steps of a row
__global__ void __launch_bounds__(256) conv_pre_fwd_kernel(const float* __restrict__ xs, const float* __restrict__ w,
                                                           const float* __restrict__ bias, float* __restrict__ u,
                                                           int D, int L, int K, long long quads_per_row,
                                                           long long total_quads, int vec) {
    for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < total_quads;
         q += (long long)gridDim.x * blockDim.x) {
        const long long row = q / quads_per_row;
        const int t0 = (int)(q % quads_per_row) * 4;
        const int i = (int)(row % D);
        const float* x = xs + row * L;
        const Taps tp = load_taps(w, i, K);
        const float bv = bias ? bias[i] : 0.f;
        // window x[t0 - (KMAX-1) .. t0 + 3]
        float win[KMAX + 3];
#pragma unroll
        for (int k = 0; k < KMAX + 3; ++k) {
            const int t = t0 - (KMAX - 1) + k;
            win[k] = (t >= 0 && t < L) ? x[t] : 0.f;
        }
        float out[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float acc = bv;
            // tap k of a K-tap filter reads x[t - (K-1) + k]; with the taps right-aligned in the KMAX window
            // that is win[(KMAX - K) + k + e]
#pragma unroll
            for (int k = 0; k < KMAX; ++k) {
                const int src = (KMAX - K) + k + e;
                if (k < K) acc = fmaf(tp.w[k], win[src < KMAX + 3 ? src : 0], acc);
            }
            out[e] = acc;
        }
        float* dst = u + row * L + t0;
        if (vec && t0 + 3 < L) {
            *reinterpret_cast<float4*>(dst) = make_float4(out[0], out[1], out[2], out[3]);
        } else {
            for (int e = 0; e < 4; ++e)
                if (t0 + e < L) dst[e] = out[e];
        }
    }
}

// ---- backward: dxs = conv^T(du); per-row partial sums of dw and dbias ---------------------------
// one block per row; partial[(row) * (KMAX + 1) + k] = sum_t du[t] xs[t - (K-1) + k], [KMAX] = sum_t du[t]
__global__ void __launch_bounds__(ROW_THREADS) conv_pre_bwd_kernel(const float* __restrict__ du,
                                                                   const float* __restrict__ xs,
                                                                   const float* __restrict__ w,
                                                                   float* __restrict__ dxs,
                                                                   float* __restrict__ partial, int D, int L, int K) {
    __shared__ float red[ROW_THREADS / 32][KMAX + 1];
    const long long row = blockIdx.x;
    const int i = (int)(row % D);
    const float* g = du + row * L;
    const float* x = xs + row * L;
    float* dx = dxs + row * L;
    const Taps tp = load_taps(w, i, K);
    float acc[KMAX + 1];
#pragma unroll
    for (int k = 0; k <= KMAX; ++k) acc[k] = 0.f;
    for (int t = threadIdx.x; t < L; t += ROW_THREADS) {
        const float gt = g[t];
        // dxs[t] = sum_k w[k] du[t + (K-1) - k]
        float d = 0.f;
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            if (k < K) {
                const int tt = t + (K - 1) - k;
                if (tt < L) d = fmaf(tp.w[k], g[tt], d);
                const int ts = t - (K - 1) + k;
                if (ts >= 0) acc[k] = fmaf(gt, x[ts], acc[k]);
            }
        }
        dx[t] = d;
        acc[KMAX] += gt;
    }
#pragma unroll
    for (int k = 0; k <= KMAX; ++k) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k <= KMAX; ++k) red[warp][k] = acc[k];
    }
    __syncthreads();
    if (threadIdx.x <= KMAX) {
        float s = 0.f;
        for (int wv = 0; wv < ROW_THREADS / 32; ++wv) s += red[wv][threadIdx.x];
        partial[row * (KMAX + 1) + threadIdx.x] = s;
    }
}

// dw[i][k] = sum_b partial[b][i][k], dbias[i] = sum_b partial[b][i][KMAX]
__global__ void __launch_bounds__(256) conv_pre_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                                              float* __restrict__ dbias, int B, int D, int K) {
    const int o = blockIdx.x * 256 + threadIdx.x;
    if (o >= D * (K + 1)) return;
    const int i = o / (K + 1), k = o % (K + 1);
    const int slot = k < K ? k : KMAX;
    float s = 0.f;
    for (int b = 0; b < B; ++b) s += partial[((long long)b * D + i) * (KMAX + 1) + slot];
    if (k < K) dw[(long long)i * K + k] = s;
    else if (dbias) dbias[i] = s;
}

// ---- step size: dt = softplus(pre + scale * bias) ---------------------------------------------------
// torch.nn.functional.softplus with its defaults (beta 1, threshold 20): x above 20 passes through
__device__ __forceinline__ float softplus_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__global__ void __launch_bounds__(256) softplus_bias_fwd_kernel(const float* __restrict__ pre,
                                                                const float* __restrict__ bias, float scale,
                                                                float* __restrict__ dt, int D, int L,
                                                                long long quads_per_row, long long total_quads,
                                                                int vec) {
    for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < total_quads;
         q += (long long)gridDim.x * blockDim.x) {
        const long long row = q / quads_per_row;
        const int t0 = (int)(q % quads_per_row) * 4;
        const float bv = bias ? scale * bias[row % D] : 0.f;
        const float* src = pre + row * L + t0;
        float* dst = dt + row * L + t0;
        if (vec && t0 + 3 < L) {
            const float4 v = *reinterpret_cast<const float4*>(src);
            *reinterpret_cast<float4*>(dst) =
                make_float4(softplus_(v.x + bv), softplus_(v.y + bv), softplus_(v.z + bv), softplus_(v.w + bv));
        } else {
            for (int e = 0; e < 4; ++e)
                if (t0 + e < L) dst[e] = softplus_(src[e] + bv);
        }
    }
}

// dpre = ddt * sigmoid(pre + scale bias), with sigmoid recovered from the output: 1 - exp(-dt) (exact also
// above the threshold, where the forward passed x through and sigmoid(x) = 1 to float32 accuracy; expm1
// keeps the relative accuracy for very negative arguments, where dt is tiny);
// partial[row] = sum_t dpre
__global__ void __launch_bounds__(ROW_THREADS) softplus_bias_bwd_kernel(const float* __restrict__ ddt,
                                                                        const float* __restrict__ dt,
                                                                        float* __restrict__ dpre,
                                                                        float* __restrict__ partial, int L) {
    __shared__ float red[ROW_THREADS / 32];
    const long long row = blockIdx.x;
    const float* g = ddt + row * L;
    const float* y = dt + row * L;
    float* d = dpre + row * L;
    float acc = 0.f;
    for (int t = threadIdx.x; t < L; t += ROW_THREADS) {
        const float v = g[t] * -expm1f(-y[t]);
        d[t] = v;
        acc += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int wv = 0; wv < ROW_THREADS / 32; ++wv) s += red[wv];
        partial[row] = s;
    }
}

__global__ void __launch_bounds__(256) bias_reduce_kernel(const float* __restrict__ partial, float scale,
                                                          float* __restrict__ dbias, int B, int D) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= D) return;
    float s = 0.f;
    for (int b = 0; b < B; ++b) s += partial[(long long)b * D + i];
    dbias[i] = scale * s;
}

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int stage_dims_ok(const char* who, int B, int D, int L) {
    if (B <= 0 || D <= 0 || L <= 0 || (long long)B * D > 0x7fffffffLL) {
        set_error("%s: sizes must be positive and B*D fit 31 bits (B=%d D=%d L=%d)", who, B, D, L);
        return AUSSM_EINVAL;
    }
    return AUSSM_OK;
}

int launch_ok(const char* who) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s launch: %s", who, cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}

unsigned stream_blocks(long long items) {
    return (unsigned)std::min<long long>((items + 255) / 256, 148LL * 32);
}

}  // namespace
}  // namespace aussm

using namespace aussm;

extern "C" {

int aussm_b200_conv_pre_fwd(const float* xs, const float* w, const float* bias, float* u, int B, int D, int L, int K,
                            aussm_stream_t stream) {
    if (int rc = stage_dims_ok("conv_pre_fwd", B, D, L)) return rc;
    if (!xs || !w || !u || K < 1 || K > KMAX) {
        set_error("conv_pre_fwd: null pointer or unsupported filter length %d (1..%d)", K, KMAX);
        return AUSSM_EINVAL;
    }
    const long long qpr = ((long long)L + 3) / 4, total = qpr * B * D;
    const int vec = (L % 4 == 0 && al16(u)) ? 1 : 0;
    conv_pre_fwd_kernel<<<stream_blocks(total), 256, 0, (cudaStream_t)stream>>>(xs, w, bias, u, D, L, K, qpr, total, vec);
    count_launch();
    return launch_ok("conv_pre_fwd");
}

size_t aussm_b200_conv_pre_bwd_workspace_bytes(int B, int D) {
    if (B <= 0 || D <= 0) return 0;
    return ((size_t)B * D * (KMAX + 1) * sizeof(float) + 255) / 256 * 256;
}

int aussm_b200_conv_pre_bwd(const float* du, const float* xs, const float* w, float* dxs, float* dw, float* dbias,
                            int B, int D, int L, int K, void* workspace, size_t workspace_bytes,
                            aussm_stream_t stream_) {
    if (int rc = stage_dims_ok("conv_pre_bwd", B, D, L)) return rc;
    if (!du || !xs || !w || !dxs || !dw || K < 1 || K > KMAX) {
        set_error("conv_pre_bwd: null pointer or unsupported filter length %d (1..%d)", K, KMAX);
        return AUSSM_EINVAL;
    }
    if (!workspace || workspace_bytes < aussm_b200_conv_pre_bwd_workspace_bytes(B, D)) {
        set_error("conv_pre_bwd: workspace of %zu bytes required, got %zu", aussm_b200_conv_pre_bwd_workspace_bytes(B, D),
                  workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    float* partial = static_cast<float*>(workspace);
    conv_pre_bwd_kernel<<<(unsigned)((long long)B * D), ROW_THREADS, 0, stream>>>(du, xs, w, dxs, partial, D, L, K);
    count_launch();
    if (int rc = launch_ok("conv_pre_bwd")) return rc;
    conv_pre_reduce_kernel<<<(D * (K + 1) + 255) / 256, 256, 0, stream>>>(partial, dw, dbias, B, D, K);
    count_launch();
    return launch_ok("conv_pre_bwd reduction");
}

int aussm_b200_softplus_bias_fwd(const float* pre, const float* bias, float scale, float* dt, int B, int D, int L,
                                 aussm_stream_t stream) {
    if (int rc = stage_dims_ok("softplus_bias_fwd", B, D, L)) return rc;
    if (!pre || !dt) {
        set_error("softplus_bias_fwd: null pointer");
        return AUSSM_EINVAL;
    }
    const long long qpr = ((long long)L + 3) / 4, total = qpr * B * D;
    const int vec = (L % 4 == 0 && al16(pre) && al16(dt)) ? 1 : 0;
    softplus_bias_fwd_kernel<<<stream_blocks(total), 256, 0, (cudaStream_t)stream>>>(pre, bias, scale, dt, D, L, qpr,
                                                                                     total, vec);
    count_launch();
    return launch_ok("softplus_bias_fwd");
}

size_t aussm_b200_softplus_bias_bwd_workspace_bytes(int B, int D) {
    if (B <= 0 || D <= 0) return 0;
    return ((size_t)B * D * sizeof(float) + 255) / 256 * 256;
}

int aussm_b200_softplus_bias_bwd(const float* ddt, const float* dt, float scale, float* dpre, float* dbias, int B,
                                 int D, int L, void* workspace, size_t workspace_bytes, aussm_stream_t stream_) {
    if (int rc = stage_dims_ok("softplus_bias_bwd", B, D, L)) return rc;
    if (!ddt || !dt || !dpre) {
        set_error("softplus_bias_bwd: null pointer");
        return AUSSM_EINVAL;
    }
    if (!workspace || workspace_bytes < aussm_b200_softplus_bias_bwd_workspace_bytes(B, D)) {
        set_error("softplus_bias_bwd: workspace of %zu bytes required, got %zu",
                  aussm_b200_softplus_bias_bwd_workspace_bytes(B, D), workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    float* partial = static_cast<float*>(workspace);
    softplus_bias_bwd_kernel<<<(unsigned)((long long)B * D), ROW_THREADS, 0, stream>>>(ddt, dt, dpre, partial, L);
    count_launch();
    if (int rc = launch_ok("softplus_bias_bwd")) return rc;
    if (dbias) {
        bias_reduce_kernel<<<(D + 255) / 256, 256, 0, stream>>>(partial, scale, dbias, B, D);
        count_launch();
        return launch_ok("softplus_bias_bwd reduction");
    }
    return AUSSM_OK;
}

}  // extern "C"
