// extern "C" entry points of the complex / positive-real scan (see include/aussm_b200.h): the scan core on a
// given eigenvalue exponent, and the operators with the reference's host-function inputs (projection + scan),
// which process the time axis in windows through a caller-owned workspace.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../../include/aussm_b200.h"
#include "host_common.cuh"
#include "projection.cuh"
#include "scan_complex.cuh"

using namespace aussm;

namespace {

bool al16c(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

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

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return AUSSM_ECUDA;
}

// ---- workspace layout of the windowed operators ----
struct CPlan {
    long long M;         // projected rows per batch entry: D*N (positive real) or 2*D*N (rho rows, then theta rows)
    int window;
    long long ldw;
    size_t off_lam, off_eta, off_part, off_proj, total;
};

CPlan make_cplan(int B, int D, int N, int L, int streams) {
    CPlan p;
    p.M = (long long)streams * D * N;
    long long w;
    const int opt = window_steps_option();
    if (opt > 0) {
        w = ((long long)opt + 63) / 64 * 64;
    } else {
        // about 2 GiB of eigenvalue exponents per window, at least 64 and at most 16384 steps
        w = ((1LL << 29) / ((long long)B * p.M)) / 64 * 64;
        w = std::max(64LL, std::min(16384LL, w));
    }
    if (w >= L) w = ((long long)L + 7) / 8 * 8;       // one window: any multiple of 4 steps
    p.window = (int)std::min<long long>(w, L);
    p.ldw = w;
    size_t off = 0;
    p.off_lam = off;
    off = align_up(off + (size_t)B * p.M * p.ldw * 4, 256);
    p.off_eta = off;
    off = align_up(off + (size_t)B * D * N * 2 * 4, 256);
    p.off_part = off;
    off = align_up(off + (size_t)B * D * 4, 256);
    p.off_proj = off;
    off = align_up(off + proj_scratch_bytes(B, D, p.M, p.ldw), 256);
    p.total = off;
    return p;
}

}  // namespace

extern "C" {

size_t aussm_b200_scan_complex_states_floats(int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) return 0;
    return 2 * (size_t)B * D * N * (size_t)(cplx_ntiles(L) + 1);
}

size_t aussm_b200_scan_complex_bwd_workspace_bytes(int B, int D, int N, int L) {
    (void)N; (void)L;
    if (B <= 0 || D <= 0) return 0;
    return ((size_t)B * D * sizeof(float) + 255) / 256 * 256;
}

int aussm_b200_scan_complex_fwd(const float* rho, const float* theta, const float* u, const float* dt,
                                const float* z, const float* B_re, const float* B_im, const float* C_re,
                                const float* C_im, const float* Dskip, float* y, float* states, int B, int D, int N,
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
    p.C_im = C_im; p.Dskip = Dskip; p.y = y; p.states = states; p.states_stride = cplx_ntiles(L) + 1; p.tile0 = 0;
    p.nch = B * D; p.Dmod = D; p.N = N; p.L = L;
    p.ld_lam = L; p.lam_batch_stride = (long long)D * N * L; p.ld_row = L;
    cudaError_t e = launch_cplx_fwd(p, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "scan_complex_fwd launch");
    return AUSSM_OK;
}

int aussm_b200_scan_complex_bwd(const float* gy, const float* gstates, const float* rho, const float* theta,
                                const float* u, const float* dt, const float* z, const float* B_re,
                                const float* B_im, const float* C_re, const float* C_im, const float* Dskip,
                                const float* states, float* drho, float* dtheta, float* du, float* ddt, float* dz,
                                float* dB_re, float* dB_im, float* dC_re, float* dC_im, float* dD, int B, int D, int N,
                                int L, void* workspace, size_t workspace_bytes, aussm_stream_t stream_) {
    if (int rc = cplx_check("scan_complex_bwd", B, D, N, L)) return rc;
    if (!gy || !u || !dt || !z || !B_re || !C_re || !Dskip || !states || !du || !ddt || !dz || !dB_re || !dC_re ||
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
    if (e != cudaSuccess) return cuda_fail(e, "scan_complex_bwd: clearing dB/dC");
    CplxBwdParams p = {};
    p.gy = gy; p.rho = rho; p.theta = theta; p.u = u; p.dt = dt; p.z = z; p.B_re = B_re; p.B_im = B_im;
    p.C_re = C_re; p.C_im = C_im; p.Dskip = Dskip; p.states = states; p.gstates = gstates;
    p.states_stride = cplx_ntiles(L) + 1; p.tile0 = 0;
    p.drho = drho; p.dtheta = dtheta; p.du = du; p.ddt = ddt; p.dz = dz; p.dB_re = dB_re;
    p.dB_im = B_im ? dB_im : nullptr; p.dC_re = dC_re; p.dC_im = C_im ? dC_im : nullptr;
    p.part_D = static_cast<float*>(workspace); p.eta_in = nullptr; p.eta_out = nullptr; p.accumulate = 0;
    p.nch = B * D; p.Dmod = D; p.N = N; p.L = L;
    p.ld_lam = L; p.lam_batch_stride = (long long)D * N * L; p.ld_row = L;
    e = launch_cplx_bwd(p, stream);
    if (e == cudaSuccess) e = launch_cplx_reduce_D(p.part_D, dD, B, D, stream);
    if (e != cudaSuccess) return cuda_fail(e, "scan_complex_bwd launch");
    return AUSSM_OK;
}

// ---- operators with the reference's inputs: projection x . u per window, then the scan ----
size_t aussm_b200_complex_workspace_bytes(int B, int D, int N, int L, int has_theta) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) return 0;
    return make_cplan(B, D, N, L, has_theta ? 2 : 1).total;
}

int aussm_b200_complex_fwd(const float* u, const float* dt, const float* x, int has_theta, const float* B_re,
                           const float* B_im, const float* C_re, const float* C_im, const float* Dskip,
                           const float* z, float* y, float* states, int B, int D, int N, int L, void* workspace,
                           size_t workspace_bytes, aussm_stream_t stream_) {
    if (int rc = cplx_check("complex_fwd", B, D, N, L)) return rc;
    if (!u || !dt || !x || !B_re || !C_re || !Dskip || !z || !y || !states) {
        set_error("complex_fwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if (!al16c(u) || !al16c(dt) || !al16c(z) || !al16c(B_re) || !al16c(B_im) || !al16c(C_re) || !al16c(C_im) ||
        !al16c(y)) {
        set_error("complex_fwd: time-major tensors must be 16-byte aligned");
        return AUSSM_EINVAL;
    }
    const int streams = has_theta ? 2 : 1;
    const CPlan pl = make_cplan(B, D, N, L, streams);
    if (!workspace || workspace_bytes < pl.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) {
        set_error("complex_fwd: workspace of %zu bytes (256-byte aligned) required, got %zu", pl.total, workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    char* ws = static_cast<char*>(workspace);
    float* lam = reinterpret_cast<float*>(ws + pl.off_lam);
    ProjScratch ps;
    proj_scratch_bind(ps, ws + pl.off_proj, B, D, pl.M, pl.ldw);
    if (int rc = proj_begin(D, pl.M, x, ps, stream)) return rc;
    const long long DN = (long long)D * N;
    const int nwin = (L + pl.window - 1) / pl.window;
    for (int w = 0; w < nwin; ++w) {
        const long long t0 = (long long)w * pl.window;
        const int tl = (int)std::min<long long>(pl.window, L - t0);
        const ProjDims pd = {B, D, pl.M, L, pl.ldw, t0, tl};
        if (int rc = proj_theta(pd, u, lam, ps, stream)) return rc;
        CplxFwdParams p = {};
        p.rho = lam; p.theta = has_theta ? lam + DN * pl.ldw : nullptr;
        p.u = u + t0; p.dt = dt + t0; p.z = z + t0;
        p.B_re = B_re + t0; p.B_im = B_im ? B_im + t0 : nullptr; p.C_re = C_re + t0; p.C_im = C_im ? C_im + t0 : nullptr;
        p.Dskip = Dskip; p.y = y + t0; p.states = states; p.states_stride = cplx_ntiles(L) + 1;
        p.tile0 = (int)(t0 / kCplxTile);
        p.nch = B * D; p.Dmod = D; p.N = N; p.L = tl;
        p.ld_lam = pl.ldw; p.lam_batch_stride = pl.M * pl.ldw; p.ld_row = L;
        cudaError_t e = launch_cplx_fwd(p, stream);
        if (e != cudaSuccess) return cuda_fail(e, "complex_fwd launch");
    }
    return AUSSM_OK;
}

int aussm_b200_complex_bwd(const float* gy, const float* gstates, const float* u, const float* dt, const float* x,
                           int has_theta, const float* B_re, const float* B_im, const float* C_re, const float* C_im,
                           const float* Dskip, const float* z, const float* states, float* du, float* ddt, float* dx,
                           float* dB_re, float* dB_im, float* dC_re, float* dC_im, float* dD, float* dz, int B, int D,
                           int N, int L, void* workspace, size_t workspace_bytes, aussm_stream_t stream_) {
    if (int rc = cplx_check("complex_bwd", B, D, N, L)) return rc;
    if (!gy || !u || !dt || !x || !B_re || !C_re || !Dskip || !z || !states || !du || !ddt || !dx || !dB_re ||
        !dC_re || !dD || !dz || (B_im && !dB_im) || (C_im && !dC_im)) {
        set_error("complex_bwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if (!al16c(gy) || !al16c(u) || !al16c(dt) || !al16c(z) || !al16c(B_re) || !al16c(B_im) || !al16c(C_re) ||
        !al16c(C_im) || !al16c(du) || !al16c(ddt) || !al16c(dz) || !al16c(dB_re) || !al16c(dB_im) || !al16c(dC_re) ||
        !al16c(dC_im)) {
        set_error("complex_bwd: time-major tensors must be 16-byte aligned");
        return AUSSM_EINVAL;
    }
    const int streams = has_theta ? 2 : 1;
    const CPlan pl = make_cplan(B, D, N, L, streams);
    if (!workspace || workspace_bytes < pl.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) {
        set_error("complex_bwd: workspace of %zu bytes (256-byte aligned) required, got %zu", pl.total, workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    char* ws = static_cast<char*>(workspace);
    float* lam = reinterpret_cast<float*>(ws + pl.off_lam);
    float* eta = reinterpret_cast<float*>(ws + pl.off_eta);
    float* part_D = reinterpret_cast<float*>(ws + pl.off_part);
    const size_t bnl = (size_t)B * N * L * sizeof(float);
    cudaError_t e = cudaMemsetAsync(dB_re, 0, bnl, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(dC_re, 0, bnl, stream);
    if (e == cudaSuccess && B_im) e = cudaMemsetAsync(dB_im, 0, bnl, stream);
    if (e == cudaSuccess && C_im) e = cudaMemsetAsync(dC_im, 0, bnl, stream);
    if (e != cudaSuccess) return cuda_fail(e, "complex_bwd: clearing dB/dC");
    ProjScratch ps;
    proj_scratch_bind(ps, ws + pl.off_proj, B, D, pl.M, pl.ldw);
    if (int rc = proj_begin(D, pl.M, x, ps, stream)) return rc;
    const long long DN = (long long)D * N;
    const int nwin = (L + pl.window - 1) / pl.window;
    for (int w = nwin - 1; w >= 0; --w) {
        const long long t0 = (long long)w * pl.window;
        const int tl = (int)std::min<long long>(pl.window, L - t0);
        const bool first = (w == nwin - 1);             // first processed = last in time
        const ProjDims pd = {B, D, pl.M, L, pl.ldw, t0, tl};
        if (int rc = proj_theta(pd, u, lam, ps, stream)) return rc;     // recompute this window's exponents
        CplxBwdParams p = {};
        p.gy = gy + t0; p.rho = lam; p.theta = has_theta ? lam + DN * pl.ldw : nullptr;
        p.u = u + t0; p.dt = dt + t0; p.z = z + t0;
        p.B_re = B_re + t0; p.B_im = B_im ? B_im + t0 : nullptr; p.C_re = C_re + t0; p.C_im = C_im ? C_im + t0 : nullptr;
        p.Dskip = Dskip; p.states = states; p.gstates = gstates; p.states_stride = cplx_ntiles(L) + 1;
        p.tile0 = (int)(t0 / kCplxTile);
        p.drho = lam; p.dtheta = has_theta ? lam + DN * pl.ldw : nullptr;      // gradients replace the exponents
        p.du = du + t0; p.ddt = ddt + t0; p.dz = dz + t0;
        p.dB_re = dB_re + t0; p.dB_im = B_im ? dB_im + t0 : nullptr; p.dC_re = dC_re + t0;
        p.dC_im = C_im ? dC_im + t0 : nullptr;
        p.part_D = part_D; p.eta_in = first ? nullptr : eta; p.eta_out = (w > 0) ? eta : nullptr;
        p.accumulate = first ? 0 : 1;
        p.nch = B * D; p.Dmod = D; p.N = N; p.L = tl;
        p.ld_lam = pl.ldw; p.lam_batch_stride = pl.M * pl.ldw; p.ld_row = L;
        e = launch_cplx_bwd(p, stream);
        if (e != cudaSuccess) return cuda_fail(e, "complex_bwd launch");
        // dx (+)= d[rho; theta] u^T and du += x^T d[rho; theta]; the scan wrote only the direct part of du
        if (int rc = proj_adjoints(pd, lam, dx, du, first, ps, stream)) return rc;
    }
    e = launch_cplx_reduce_D(part_D, dD, B, D, stream);
    if (e != cudaSuccess) return cuda_fail(e, "complex_bwd reduction launch");
    return AUSSM_OK;
}

}  // extern "C"
