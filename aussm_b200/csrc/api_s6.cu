// extern "C" entry points of the real selective scan (see include/aussm_b200.h).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aussm_b200.h"
#include "host_common.cuh"
#include "scan_s6.cuh"

using namespace aussm;

namespace {

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int s6_check(const char* who, int B, int D, int N, int L) {
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

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

extern "C" {

size_t aussm_b200_selective_scan_ckpt_floats(int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) return 0;
    return (size_t)B * D * N * (size_t)s6_ntiles(L, N);
}

size_t aussm_b200_selective_scan_bwd_workspace_bytes(int B, int D, int N, int L) {
    (void)L;
    if (B <= 0 || D <= 0 || N <= 0) return 0;
    return up256(((size_t)B * D * N + 2 * (size_t)B * D) * sizeof(float));
}

int aussm_b200_selective_scan_fwd(const float* u, const float* delta, const float* A, const float* Bm,
                                  const float* Cm, const float* Dskip, const float* z, const float* delta_bias,
                                  int delta_softplus, float* out, float* ckpt, float* last_state, int B, int D, int N,
                                  int L, aussm_stream_t stream) {
    if (int rc = s6_check("selective_scan_fwd", B, D, N, L)) return rc;
    if (!u || !delta || !A || !Bm || !Cm || !out) {
        set_error("selective_scan_fwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if (!al16(u) || !al16(delta) || !al16(Bm) || !al16(Cm) || !al16(out) || (z && !al16(z))) {
        set_error("selective_scan_fwd: u, delta, B, C, z and out must be 16-byte aligned");
        return AUSSM_EINVAL;
    }
    S6FwdParams p = {};
    p.u = u; p.delta = delta; p.A = A; p.Bm = Bm; p.Cm = Cm; p.Dskip = Dskip; p.z = z; p.delta_bias = delta_bias;
    p.out = out; p.ckpt = ckpt; p.last_state = last_state; p.delta_softplus = delta_softplus;
    p.nch = B * D; p.Dmod = D; p.N = N; p.L = L;
    cudaError_t e = s6_wide(N) ? launch_s6_wide_fwd(p, (cudaStream_t)stream) : launch_s6_fwd(p, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        set_error("selective_scan_fwd launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}

int aussm_b200_selective_scan_bwd(const float* gout, const float* u, const float* delta, const float* A,
                                  const float* Bm, const float* Cm, const float* Dskip, const float* z,
                                  const float* delta_bias, int delta_softplus, const float* ckpt, float* du,
                                  float* ddelta, float* dA, float* dB, float* dC, float* dD, float* dz,
                                  float* ddelta_bias, int B, int D, int N, int L, void* workspace,
                                  size_t workspace_bytes, aussm_stream_t stream_) {
    if (int rc = s6_check("selective_scan_bwd", B, D, N, L)) return rc;
    if (!gout || !u || !delta || !A || !Bm || !Cm || !ckpt || !du || !ddelta || !dA || !dB || !dC || (z && !dz)) {
        set_error("selective_scan_bwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if (!al16(gout) || !al16(u) || !al16(delta) || !al16(Bm) || !al16(Cm) || !al16(du) || !al16(ddelta) ||
        !al16(dB) || !al16(dC) || (z && (!al16(z) || !al16(dz)))) {
        set_error("selective_scan_bwd: time-major tensors must be 16-byte aligned");
        return AUSSM_EINVAL;
    }
    const size_t need = aussm_b200_selective_scan_bwd_workspace_bytes(B, D, N, L);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15u)) {
        set_error("selective_scan_bwd: workspace of %zu bytes required, got %zu", need, workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    const long long nch = (long long)B * D;
    float* part_A = static_cast<float*>(workspace);
    float* part_D = part_A + nch * N;
    float* part_bias = part_D + nch;
    // dB and dC are accumulated with atomics: they start from zero
    cudaError_t e = cudaMemsetAsync(dB, 0, (size_t)B * N * L * sizeof(float), stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(dC, 0, (size_t)B * N * L * sizeof(float), stream);
    if (e != cudaSuccess) {
        set_error("selective_scan_bwd: clearing dB/dC: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    S6BwdParams p = {};
    p.gout = gout; p.u = u; p.delta = delta; p.A = A; p.Bm = Bm; p.Cm = Cm; p.Dskip = Dskip; p.z = z;
    p.delta_bias = delta_bias; p.ckpt = ckpt; p.du = du; p.ddelta = ddelta; p.dz = dz; p.dB = dB; p.dC = dC;
    p.part_A = part_A; p.part_D = part_D; p.part_bias = part_bias; p.delta_softplus = delta_softplus;
    p.nch = (int)nch; p.Dmod = D; p.N = N; p.L = L;
    e = s6_wide(N) ? launch_s6_wide_bwd(p, stream) : launch_s6_bwd(p, stream);
    if (e != cudaSuccess) {
        set_error("selective_scan_bwd launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    S6ReduceParams r = {part_A, part_D, part_bias, dA, dD, ddelta_bias, B, D, N};
    e = launch_s6_reduce(r, stream);
    if (e != cudaSuccess) {
        set_error("selective_scan_bwd reduction launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}

}  // extern "C"
