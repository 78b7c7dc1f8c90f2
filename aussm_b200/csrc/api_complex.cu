// extern "C" entry points of the complex / positive-real scan (see include/aussm_b200.h).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aussm_b200.h"
#include "host_common.cuh"
#include "scan_complex.cuh"

using namespace aussm;

namespace {

bool al16c(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int cplx_check(const char* who, int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) {
        set_error("%s: sizes must be positive (B=%d D=%d N=%d L=%d)", who, B, D, N, L);
        return AUSSM_EINVAL;
    }
    if (N > 32) {
        set_error("%s: N=%d states per channel, at most 32 are supported", who, N);
        return AUSSM_EINVAL;
    }
    if (L % 4 != 0) {
        set_error("%s: L=%d must be a multiple of 4 (pad the time axis with zeros)", who, L);
        return AUSSM_EINVAL;
    }
    if ((long long)B * D > 0x7fffffffLL) {
        set_error("%s: B*D exceeds the 32-bit channel count", who);
        return AUSSM_EINVAL;
    }
    return AUSSM_OK;
}

}  // namespace

extern "C" {

size_t aussm_b200_scan_complex_ckpt_floats(int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) return 0;
    return 2 * (size_t)B * D * N * (size_t)cplx_ntiles(L);
}

size_t aussm_b200_scan_complex_bwd_workspace_bytes(int B, int D, int N, int L) {
    (void)N; (void)L;
    if (B <= 0 || D <= 0) return 0;
    return ((size_t)B * D * sizeof(float) + 255) / 256 * 256;
}

int aussm_b200_scan_complex_fwd(const float* rho, const float* theta, const float* u, const float* dt,
                                const float* z, const float* B_re, const float* B_im, const float* C_re,
                                const float* C_im, const float* Dskip, float* y, float* ckpt, int B, int D, int N,
                                int L, aussm_stream_t stream) {
    if (int rc = cplx_check("scan_complex_fwd", B, D, N, L)) return rc;
    if (!u || !dt || !z || !B_re || !C_re || !Dskip || !y) {
        set_error("scan_complex_fwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if (!al16c(rho) || !al16c(theta) || !al16c(u) || !al16c(dt) || !al16c(z) || !al16c(B_re) || !al16c(B_im) ||
        !al16c(C_re) || !al16c(C_im) || !al16c(y)) {
        set_error("scan_complex_fwd: time-major tensors must be 16-byte aligned");
        return AUSSM_EINVAL;
    }
    CplxFwdParams p = {};
    p.rho = rho; p.theta = theta; p.u = u; p.dt = dt; p.z = z; p.B_re = B_re; p.B_im = B_im; p.C_re = C_re;
    p.C_im = C_im; p.Dskip = Dskip; p.y = y; p.ckpt = ckpt; p.nch = B * D; p.Dmod = D; p.N = N; p.L = L;
    cudaError_t e = launch_cplx_fwd(p, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        set_error("scan_complex_fwd launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}

int aussm_b200_scan_complex_bwd(const float* gy, const float* rho, const float* theta, const float* u,
                                const float* dt, const float* z, const float* B_re, const float* B_im,
                                const float* C_re, const float* C_im, const float* Dskip, const float* ckpt,
                                float* drho, float* dtheta, float* du, float* ddt, float* dz, float* dB_re,
                                float* dB_im, float* dC_re, float* dC_im, float* dD, int B, int D, int N, int L,
                                void* workspace, size_t workspace_bytes, aussm_stream_t stream_) {
    if (int rc = cplx_check("scan_complex_bwd", B, D, N, L)) return rc;
    if (!gy || !u || !dt || !z || !B_re || !C_re || !Dskip || !ckpt || !du || !ddt || !dz || !dB_re || !dC_re ||
        !dD || (rho && !drho) || (theta && !dtheta) || (B_im && !dB_im) || (C_im && !dC_im)) {
        set_error("scan_complex_bwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if (!al16c(gy) || !al16c(rho) || !al16c(theta) || !al16c(u) || !al16c(dt) || !al16c(z) || !al16c(B_re) ||
        !al16c(B_im) || !al16c(C_re) || !al16c(C_im) || !al16c(drho) || !al16c(dtheta) || !al16c(du) ||
        !al16c(ddt) || !al16c(dz) || !al16c(dB_re) || !al16c(dB_im) || !al16c(dC_re) || !al16c(dC_im)) {
        set_error("scan_complex_bwd: time-major tensors must be 16-byte aligned");
        return AUSSM_EINVAL;
    }
    const size_t need = aussm_b200_scan_complex_bwd_workspace_bytes(B, D, N, L);
    if (!workspace || workspace_bytes < need) {
        set_error("scan_complex_bwd: workspace of %zu bytes required, got %zu", need, workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    const size_t bnl = (size_t)B * N * L * sizeof(float);
    cudaError_t e = cudaMemsetAsync(dB_re, 0, bnl, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(dC_re, 0, bnl, stream);
    if (e == cudaSuccess && B_im) e = cudaMemsetAsync(dB_im, 0, bnl, stream);
    if (e == cudaSuccess && C_im) e = cudaMemsetAsync(dC_im, 0, bnl, stream);
    if (e != cudaSuccess) {
        set_error("scan_complex_bwd: clearing dB/dC: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    CplxBwdParams p = {};
    p.gy = gy; p.rho = rho; p.theta = theta; p.u = u; p.dt = dt; p.z = z; p.B_re = B_re; p.B_im = B_im;
    p.C_re = C_re; p.C_im = C_im; p.Dskip = Dskip; p.ckpt = ckpt; p.drho = drho; p.dtheta = dtheta; p.du = du;
    p.ddt = ddt; p.dz = dz; p.dB_re = dB_re; p.dB_im = B_im ? dB_im : nullptr; p.dC_re = dC_re;
    p.dC_im = C_im ? dC_im : nullptr; p.part_D = static_cast<float*>(workspace);
    p.nch = B * D; p.Dmod = D; p.N = N; p.L = L;
    e = launch_cplx_bwd(p, stream);
    if (e == cudaSuccess) e = launch_cplx_reduce_D(p.part_D, dD, B, D, stream);
    if (e != cudaSuccess) {
        set_error("scan_complex_bwd launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}

}  // extern "C"
