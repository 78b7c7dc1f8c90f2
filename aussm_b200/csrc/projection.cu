// Phase projection and its adjoints as three-term split GEMMs on tcgen05.
#include "projection.cuh"

#include <stdint.h>

#include <algorithm>

#include "../../include/aussm_b200.h"
#include "gemm_split3.cuh"

namespace aussm {

namespace {
size_t up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int sm_count_cached() {
    static int n = 0;
    if (n <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

// dx (+)= p0 + p1, in this order
__global__ void __launch_bounds__(256) add_groups_kernel(float* __restrict__ dx, const float* __restrict__ p0,
                                                         const float* __restrict__ p1, long long n4, int overwrite) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const float4 a = reinterpret_cast<const float4*>(p0)[i], b = reinterpret_cast<const float4*>(p1)[i];
        float4 o = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
        if (!overwrite) {
            const float4 c = reinterpret_cast<const float4*>(dx)[i];
            o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
        }
        reinterpret_cast<float4*>(dx)[i] = o;
    }
}
}  // namespace

size_t proj_scratch_bytes(int B, int D, long long M_, long long ldw) {
    const size_t M = (size_t)M_, Dp = up((size_t)D, 8);
    const size_t halves = 2 * split_part_halves(M * Dp) + 2 * split_part_halves((size_t)B * D * ldw) +
                          2 * split_part_halves((size_t)B * M * ldw);
    return halves * 2 + up(2 * M * (size_t)D * sizeof(float), 256) + 256;
}

void proj_scratch_bind(ProjScratch& s, void* base, int B, int D, long long M_, long long ldw) {
    const size_t M = (size_t)M_, Dp = up((size_t)D, 8);
    char* p = static_cast<char*>(base);
    auto take = [&](size_t halves) {
        void* r = p;
        p += split_part_halves(halves) * 2;          // every part starts 256-byte aligned
        return r;
    };
    s.x_hi = take(M * Dp);
    s.x_lo = take(M * Dp);
    s.u_hi = take((size_t)B * D * ldw);
    s.u_lo = take((size_t)B * D * ldw);
    s.dth_hi = take((size_t)B * M * ldw);
    s.dth_lo = take((size_t)B * M * ldw);
    s.dx_part = reinterpret_cast<float*>(p);
    p += up(2 * M * (size_t)D * sizeof(float), 256);
    s.amax = reinterpret_cast<unsigned*>(p);   // inside the 256 spare bytes
    s.Dp = (long long)Dp;
}

int proj_begin(int D, long long M, const float* x, ProjScratch& s, cudaStream_t stream) {
    return split_f16(x, D, 0, s.x_hi, s.x_lo, s.Dp, 0, M, D, 1, s.amax + 0, stream);
}

int proj_split_u(const ProjDims& d, const float* u, ProjScratch& s, cudaStream_t stream) {
    // rows r (D of them per batch entry), tl columns of this window
    return split_f16(u + d.t0, d.L, (long long)d.D * d.L, s.u_hi, s.u_lo, d.ldw, (long long)d.D * d.ldw, d.D, d.tl, d.B,
                     s.amax + 1, stream);
}

int proj_theta(const ProjDims& d, const float* u, float* theta_w, ProjScratch& s, cudaStream_t stream) {
    const int M = (int)d.M;
    if (int rc = proj_split_u(d, u, s, stream)) return rc;
    // theta_w[b] (M x tl) = x (M x D, K-major) * u_b (D x tl: K rows, N contiguous -> MN-major)
    const SplitOperand A = {s.x_hi, s.x_lo, 0, s.Dp, 0, s.amax + 0};
    const SplitOperand Bop = {s.u_hi, s.u_lo, 1, d.ldw, (long long)d.D * d.ldw, s.amax + 1};
    const GemmShape shape = {M, d.tl, d.D, d.B, 0, 0, d.ldw, (long long)M * d.ldw};
    return gemm_split3(A, Bop, theta_w, shape, stream);
}

int proj_adjoints(const ProjDims& d, const float* dtheta_w, float* dx, float* du, bool overwrite_dx, ProjScratch& s,
                  cudaStream_t stream, bool dtheta_amax_known) {
    const int M = (int)d.M;
    if (int rc = split_f16(dtheta_w, d.ldw, (long long)M * d.ldw, s.dth_hi, s.dth_lo, d.ldw, (long long)M * d.ldw, M,
                           d.tl, d.B, s.amax + 2, stream, dtheta_amax_known))
        return rc;
    {
        // dx (M x D) (+)= sum_b dtheta_b (M x tl, K-major) * u_b^T (u_b: D rows x tl, K-major)
        const SplitOperand A = {s.dth_hi, s.dth_lo, 0, d.ldw, (long long)M * d.ldw, s.amax + 2};
        const SplitOperand Bop = {s.u_hi, s.u_lo, 0, d.ldw, (long long)d.D * d.ldw, s.amax + 1};
        // The output has few tiles (M / 128 x D / 256: 512 for the benchmark, 3.46 waves of 148 CTAs).  When summing
        // the batch in two groups fills the last wave better, the groups' partial sums go to scratch and are added
        // in a fixed order.
        const long long tiles = ((long long)(M + 127) / 128) * ((d.D + 255) / 256), sms = sm_count_cached();
        auto fill = [&](long long n) { return (double)n / (double)(((n + sms - 1) / sms) * sms); };
        const bool two = d.B % 2 == 0 && fill(2 * tiles) > fill(tiles) + 0.05 && ((long long)M * d.D) % 4 == 0 &&
                         (reinterpret_cast<uintptr_t>(dx) & 15u) == 0;
        if (two) {
            const GemmShape shape = {M, d.D, d.tl, d.B, 2, 0, d.D, (long long)M * d.D};
            if (int rc = gemm_split3(A, Bop, s.dx_part, shape, stream)) return rc;
            const long long n4 = (long long)M * d.D / 4;
            const unsigned blocks = (unsigned)std::min<long long>((n4 + 255) / 256, 148 * 8);
            add_groups_kernel<<<blocks, 256, 0, stream>>>(dx, s.dx_part, s.dx_part + (long long)M * d.D, n4,
                                                          overwrite_dx ? 1 : 0);
            count_launch();
            if (cudaGetLastError() != cudaSuccess) {
                set_error("projection: launch of the partial-sum kernel failed");
                return AUSSM_ECUDA;
            }
        } else {
            const GemmShape shape = {M, d.D, d.tl, d.B, 1, overwrite_dx ? 0 : 1, d.D, 0};
            if (int rc = gemm_split3(A, Bop, dx, shape, stream)) return rc;
        }
    }
    {
        // du_b (D x tl) += x^T (x stored M rows x D: K rows, output-row index contiguous -> MN-major)
        //                  * dtheta_b (M x tl: K rows, N contiguous -> MN-major)
        const SplitOperand A = {s.x_hi, s.x_lo, 1, s.Dp, 0, s.amax + 0};
        const SplitOperand Bop = {s.dth_hi, s.dth_lo, 1, d.ldw, (long long)M * d.ldw, s.amax + 2};
        const GemmShape shape = {d.D, d.tl, M, d.B, 0, 1, d.L, (long long)d.D * d.L};
        return gemm_split3(A, Bop, du + d.t0, shape, stream);
    }
}

}  // namespace aussm
