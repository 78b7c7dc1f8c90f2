// Phase projection and its adjoints: tcgen05 three-term TF32 GEMMs, with the
// library SGEMM as the fallback for shapes the TMA path cannot address.
#include "projection.cuh"

#include <cublas_v2.h>
#include <stdint.h>

#include <mutex>

#include "../../include/aussm_b200.h"
#include "gemm_tf32x3.cuh"

namespace aussm {

namespace {

constexpr int kMaxDevices = 64;
cublasHandle_t g_handles[kMaxDevices] = {};
std::mutex g_handle_mutex;
int g_gemm_backend = 0;

// One cuBLAS handle per device, created on first use (this allocates; it must
// therefore happen before any stream capture).
int get_handle(cudaStream_t stream, cublasHandle_t* out) {
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("cudaGetDevice failed: %s", cudaGetErrorString(ce));
        return AUSSM_ECUDA;
    }
    {
        std::lock_guard<std::mutex> lock(g_handle_mutex);
        if (!g_handles[dev]) {
            cublasStatus_t st = cublasCreate(&g_handles[dev]);
            if (st != CUBLAS_STATUS_SUCCESS) {
                g_handles[dev] = nullptr;
                set_error("cublasCreate failed with status %d", (int)st);
                return AUSSM_ECUDA;
            }
            // float32 products and sums only: no TF32 down-conversion of the phases
            cublasSetMathMode(g_handles[dev], CUBLAS_DEFAULT_MATH);
        }
        *out = g_handles[dev];
    }
    cublasStatus_t st = cublasSetStream(*out, stream);
    if (st != CUBLAS_STATUS_SUCCESS) {
        set_error("cublasSetStream failed with status %d", (int)st);
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}

int check(cublasStatus_t st, const char* what) {
    if (st == CUBLAS_STATUS_SUCCESS) return AUSSM_OK;
    set_error("%s failed with cuBLAS status %d", what, (int)st);
    return AUSSM_ECUDA;
}

bool ok16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- library fallback: row-major C = A B issued as column-major C^T = B^T A^T ----
int lib_theta(const ProjDims& d, const float* x, const float* u, float* theta_w, cudaStream_t stream) {
    cublasHandle_t h;
    if (int rc = get_handle(stream, &h)) return rc;
    const float one = 1.f, zero = 0.f;
    const int M = d.D * d.N;
    return check(cublasSgemmStridedBatched(h, CUBLAS_OP_N, CUBLAS_OP_N, d.tl, M, d.D, &one, u + d.t0, (int)d.L,
                                           (long long)d.D * d.L, x, d.D, 0, &zero, theta_w, (int)d.ldw,
                                           (long long)M * d.ldw, d.B),
                 "phase projection GEMM");
}

int lib_dx(const ProjDims& d, const float* dtheta_w, const float* u, float* dx, bool overwrite,
           cudaStream_t stream) {
    cublasHandle_t h;
    if (int rc = get_handle(stream, &h)) return rc;
    const float one = 1.f, zero = 0.f;
    const int M = d.D * d.N;
    for (int b = 0; b < d.B; ++b) {
        const float* beta = (overwrite && b == 0) ? &zero : &one;
        int rc = check(cublasSgemm(h, CUBLAS_OP_T, CUBLAS_OP_N, d.D, M, d.tl, &one,
                                   u + (long long)b * d.D * d.L + d.t0, (int)d.L,
                                   dtheta_w + (long long)b * M * d.ldw, (int)d.ldw, beta, dx, d.D),
                       "dx GEMM");
        if (rc) return rc;
    }
    return AUSSM_OK;
}

int lib_du(const ProjDims& d, const float* dtheta_w, const float* x, float* du, cudaStream_t stream) {
    cublasHandle_t h;
    if (int rc = get_handle(stream, &h)) return rc;
    const float one = 1.f;
    const int M = d.D * d.N;
    return check(cublasSgemmStridedBatched(h, CUBLAS_OP_N, CUBLAS_OP_T, d.tl, d.D, M, &one, dtheta_w, (int)d.ldw,
                                           (long long)M * d.ldw, x, d.D, 0, &one, du + d.t0, (int)d.L,
                                           (long long)d.D * d.L, d.B),
                 "du GEMM");
}

}  // namespace

void set_gemm_backend(int mode) { g_gemm_backend = mode; }
int gemm_backend() { return g_gemm_backend; }

size_t proj_scratch_floats(int B, int D, int N, long long ldw) {
    const size_t M = (size_t)D * N;
    return 2 * M * D + 2 * (size_t)B * D * ldw + 2 * (size_t)B * M * ldw + 64;
}

void proj_scratch_bind(ProjScratch& s, float* base, int B, int D, int N, long long ldw) {
    const size_t M = (size_t)D * N;
    auto up4 = [](size_t v) { return (v + 3) / 4 * 4; };
    s.x_hi = base;
    s.x_lo = s.x_hi + up4(M * D);
    s.u_hi = s.x_lo + up4(M * D);
    s.u_lo = s.u_hi + up4((size_t)B * D * ldw);
    s.dth_hi = s.u_lo + up4((size_t)B * D * ldw);
    s.dth_lo = s.dth_hi + up4((size_t)B * M * ldw);
    s.amax = reinterpret_cast<unsigned*>(s.dth_lo + up4((size_t)B * M * ldw));   // inside the 64 spare floats
    s.use_tensor_cores = 0;
    s.half = 0;
}

int proj_begin(int B, int D, int N, long long L, long long ldw, const float* x, const float* u, ProjScratch& s,
               cudaStream_t stream) {
    (void)B;
    s.use_tensor_cores = 0;
    // TMA needs 16-byte aligned rows everywhere: x rows (D floats), u rows (L floats), window rows (ldw floats)
    const bool aligned = (D % 4 == 0) && (L % 4 == 0) && (ldw % 4 == 0) && ok16(x) && ok16(u) && ok16(s.x_hi);
    if (g_gemm_backend == 1 || !aligned) return AUSSM_OK;
    SplitOperand probe = {s.x_hi, s.x_lo, 0, D, 0};
    GemmShape shape = {D * N, 4, D, 1, 0, 0, ldw, 0};
    if (!gemm_tf32x3_supported(probe, probe, s.x_hi, shape)) return AUSSM_OK;
    // FP16 parts need 16-byte rows of halves: pitches that are multiples of 8
    s.half = (g_gemm_backend == 0 && D % 8 == 0 && ldw % 8 == 0) ? 1 : 0;
    if (s.half) {
        if (int rc = split_f16(x, D, 0, s.x_hi, s.x_lo, D, 0, (long long)D * N, D, 1, s.amax + 0, stream)) return rc;
    } else {
        if (int rc = split_tf32(x, D, 0, s.x_hi, s.x_lo, D, 0, (long long)D * N, D, 1, stream)) return rc;
    }
    s.use_tensor_cores = 1;
    return AUSSM_OK;
}

int proj_split_u(const ProjDims& d, const float* u, ProjScratch& s, cudaStream_t stream) {
    if (!s.use_tensor_cores) return AUSSM_OK;
    // split this window of u: rows r (D of them per batch entry), tl columns
    if (s.half)
        return split_f16(u + d.t0, d.L, (long long)d.D * d.L, s.u_hi, s.u_lo, d.ldw, (long long)d.D * d.ldw, d.D, d.tl,
                         d.B, s.amax + 1, stream);
    return split_tf32(u + d.t0, d.L, (long long)d.D * d.L, s.u_hi, s.u_lo, d.ldw, (long long)d.D * d.ldw, d.D, d.tl,
                      d.B, stream);
}

int proj_theta(const ProjDims& d, const float* x, const float* u, float* theta_w, ProjScratch& s,
               cudaStream_t stream) {
    if (!s.use_tensor_cores) return lib_theta(d, x, u, theta_w, stream);
    const int M = d.D * d.N;
    if (int rc = proj_split_u(d, u, s, stream)) return rc;
    // theta_w[b] (M x tl) = x (M x D, K-major) * u_b (D x tl: K rows, N contiguous -> MN-major)
    const SplitOperand A = {s.x_hi, s.x_lo, 0, d.D, 0, s.half ? s.amax + 0 : nullptr};
    const SplitOperand Bop = {s.u_hi, s.u_lo, 1, d.ldw, (long long)d.D * d.ldw, s.half ? s.amax + 1 : nullptr};
    const GemmShape shape = {M, d.tl, d.D, d.B, 0, 0, d.ldw, (long long)M * d.ldw};
    return gemm_tf32x3(A, Bop, theta_w, shape, stream);
}

int proj_adjoints(const ProjDims& d, const float* dtheta_w, const float* x, const float* u, float* dx, float* du,
                  bool overwrite_dx, ProjScratch& s, cudaStream_t stream, bool dtheta_amax_known) {
    if (!s.use_tensor_cores) {
        if (int rc = lib_dx(d, dtheta_w, u, dx, overwrite_dx, stream)) return rc;
        return lib_du(d, dtheta_w, x, du, stream);
    }
    const int M = d.D * d.N;
    if (s.half) {
        if (int rc = split_f16(dtheta_w, d.ldw, (long long)M * d.ldw, s.dth_hi, s.dth_lo, d.ldw, (long long)M * d.ldw,
                               M, d.tl, d.B, s.amax + 2, stream, dtheta_amax_known))
            return rc;
    } else if (int rc = split_tf32(dtheta_w, d.ldw, (long long)M * d.ldw, s.dth_hi, s.dth_lo, d.ldw,
                                   (long long)M * d.ldw, M, d.tl, d.B, stream)) {
        return rc;
    }
    const unsigned* ax = s.half ? s.amax + 0 : nullptr;
    const unsigned* au = s.half ? s.amax + 1 : nullptr;
    const unsigned* ad = s.half ? s.amax + 2 : nullptr;
    {
        // dx (M x D) (+)= sum_b dtheta_b (M x tl, K-major) * u_b^T (u_b: D rows x tl, K-major)
        const SplitOperand A = {s.dth_hi, s.dth_lo, 0, d.ldw, (long long)M * d.ldw, ad};
        const SplitOperand Bop = {s.u_hi, s.u_lo, 0, d.ldw, (long long)d.D * d.ldw, au};
        const GemmShape shape = {M, d.D, d.tl, d.B, 1, overwrite_dx ? 0 : 1, d.D, 0};
        if (int rc = gemm_tf32x3(A, Bop, dx, shape, stream)) return rc;
    }
    {
        // du_b (D x tl) += x^T (x stored M rows x D: K rows, output-row index contiguous -> MN-major)
        //                  * dtheta_b (M x tl: K rows, N contiguous -> MN-major)
        const SplitOperand A = {s.x_hi, s.x_lo, 1, d.D, 0, ax};
        const SplitOperand Bop = {s.dth_hi, s.dth_lo, 1, d.ldw, (long long)M * d.ldw, ad};
        const GemmShape shape = {d.D, d.tl, M, d.B, 0, 1, d.L, (long long)d.D * d.L};
        return gemm_tf32x3(A, Bop, du + d.t0, shape, stream);
    }
}

}  // namespace aussm
