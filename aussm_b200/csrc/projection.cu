// Library-GEMM implementation of the phase projection and its adjoints.
#include "projection.cuh"

#include <cublas_v2.h>

#include <mutex>

#include "../../include/aussm_b200.h"

namespace aussm {

namespace {

constexpr int kMaxDevices = 64;
cublasHandle_t g_handles[kMaxDevices] = {};
std::mutex g_handle_mutex;

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

}  // namespace

// Row-major C = A B is issued as column-major C^T = B^T A^T.
int proj_theta(const ProjDims& d, const float* x, const float* u, float* theta_w, cudaStream_t stream) {
    cublasHandle_t h;
    if (int rc = get_handle(stream, &h)) return rc;
    const float one = 1.f, zero = 0.f;
    const int M = d.D * d.N;
    return check(cublasSgemmStridedBatched(h, CUBLAS_OP_N, CUBLAS_OP_N, d.tl, M, d.D, &one, u + d.t0, (int)d.L,
                                           (long long)d.D * d.L, x, d.D, 0, &zero, theta_w, (int)d.ldw,
                                           (long long)M * d.ldw, d.B),
                 "phase projection GEMM");
}

int proj_dx(const ProjDims& d, const float* dtheta_w, const float* u, float* dx, bool overwrite,
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

int proj_du(const ProjDims& d, const float* dtheta_w, const float* x, float* du, cudaStream_t stream) {
    cublasHandle_t h;
    if (int rc = get_handle(stream, &h)) return rc;
    const float one = 1.f;
    const int M = d.D * d.N;
    return check(cublasSgemmStridedBatched(h, CUBLAS_OP_N, CUBLAS_OP_T, d.tl, d.D, M, &one, dtheta_w, (int)d.ldw,
                                           (long long)M * d.ldw, x, d.D, 0, &one, du + d.t0, (int)d.L,
                                           (long long)d.D * d.L, d.B),
                 "du GEMM");
}

}  // namespace aussm
