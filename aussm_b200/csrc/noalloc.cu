// A backward scan entry point for callers that must not allocate.
//
// The backward scan needs scratch memory for its per-channel partial sums
// (gradients of B, C and D before the fixed-order reduction).  The regular
// entry point takes that scratch from the caller, who usually gets it from
// cudaMalloc or from a framework allocator.  Some callers cannot do either at
// the point where they run the operator: code that executes inside a region
// where device allocation is forbidden or would synchronise (a latency-critical
// serving loop, a callback that runs while another library holds the
// allocator's lock, a plug-in host that hands out only the input and output
// buffers), or a runtime with a fixed memory plan that has no spare buffer to
// lend.  For them the scratch lives in a file-scope device array that is part
// of the library's device code and is never freed, so the call itself performs
// no cudaMalloc, no cudaFree and no allocating library routine.  The runtime
// loads device code lazily: the first call on a device makes it load this
// module (the array comes into being then, which may reserve memory and
// synchronise the device), so callers make one warm-up call per device before
// the region where that is off limits.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/aussm_b200.h"
#include "host_common.cuh"
#include "scan_unitary.cuh"

namespace aussm {
namespace {

// 4 MiB per GPU on which the entry point has run (or that loaded the library eagerly), held until the process exits.
constexpr size_t kStaticScratchFloats = (size_t)AUSSM_STATIC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// In host code `g_static_scratch` is only a handle for the runtime, not a
// device address.  The real address is looked up once per device, with that
// device current, and remembered.
int static_scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        set_error("scan_unitary_bwd_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("scan_unitary_bwd_static: device ordinal %d is outside the %d devices this entry point keeps an "
                  "address for", dev, kMaxDevices);
        return AUSSM_EINVAL;
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("scan_unitary_bwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return AUSSM_ECUDA;
        }
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return AUSSM_OK;
}

}  // namespace
}  // namespace aussm

using namespace aussm;

extern "C" int aussm_b200_scan_unitary_bwd_static(
    const float* grad_y, const float* gh1_re, const float* gh1_im, const float* theta, const float* u,
    const float* dt, const float* z, const float* B_r, const float* B_theta, const float* C_r, const float* C_theta,
    const float* Dskip, const float* h1_re, const float* h1_im, float* dtheta, float* du, float* ddt, float* dz,
    float* dB_r, float* dB_theta, float* dC_r, float* dC_theta, float* dD, float* dh0_re, float* dh0_im, int B, int D,
    int N, int L, aussm_stream_t stream) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0 || N > AUSSM_MAX_STATES) {
        set_error("scan_unitary_bwd_static: bad sizes (B=%d D=%d N=%d L=%d, N <= %d)", B, D, N, L, AUSSM_MAX_STATES);
        return AUSSM_EINVAL;
    }
    if (!grad_y || !theta || !u || !dt || !z || !B_r || !B_theta || !C_r || !C_theta || !Dskip || !h1_re ||
        !h1_im || !dtheta || !du || !ddt || !dz || !dB_r || !dB_theta || !dC_r || !dC_theta || !dD) {
        set_error("scan_unitary_bwd_static: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if ((gh1_re == nullptr) != (gh1_im == nullptr) || (dh0_re == nullptr) != (dh0_im == nullptr)) {
        set_error("scan_unitary_bwd_static: real and imaginary state pointers must be given together");
        return AUSSM_EINVAL;
    }
    const long long nch = (long long)B * D;
    const size_t need = scan_bwd_partial_floats(nch, N);     // nch * (5N + 1) floats; the row sums are not used here
    if (nch > 0x7fffffffLL || need > kStaticScratchFloats) {
        set_error("scan_unitary_bwd_static: B*D*(5*N+1) = %zu floats of scratch needed, the built-in array holds %zu "
                  "(%d bytes); use aussm_b200_scan_unitary_bwd with a caller-owned workspace for this size",
                  need, kStaticScratchFloats, (int)AUSSM_STATIC_SCRATCH_BYTES);
        return AUSSM_EWORKSPACE;
    }
    float* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;

    // Every launch overwrites all nch*N*4 + nch partials it later reads (accumulate = 0), so nothing in the
    // shared array has to start at zero and stale contents of an earlier call cannot leak into this one.
    float* part_bc = scratch;
    float* part_d = part_bc + nch * N * 4;
    ScanBwdParams p = {};
    p.theta = theta; p.theta_bias = nullptr; p.u = u; p.dt = dt; p.z = z; p.gy = grad_y;
    p.B_r = B_r; p.B_theta = B_theta; p.C_r = C_r; p.C_theta = C_theta; p.Dskip = Dskip;
    p.h1_re = h1_re; p.h1_im = h1_im; p.gh1_re = gh1_re; p.gh1_im = gh1_im;
    p.dtheta = dtheta; p.du = du; p.ddt = ddt; p.dz = dz; p.dh0_re = dh0_re; p.dh0_im = dh0_im;
    p.h0_re = nullptr; p.h0_im = nullptr;
    p.part_bc = part_bc; p.part_d = part_d; p.part_rowsum = nullptr; p.accumulate = 0;
    p.nch = (int)nch; p.Dmod = D; p.N = N; p.L = L; p.ld_theta = L; p.ld_dtheta = L; p.ld_row = L;
    cudaError_t e = launch_scan_unitary_bwd(p, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        set_error("scan_unitary_bwd_static: backward launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    ReduceParams r = {};
    r.part_bc = part_bc; r.part_d = part_d; r.part_rowsum = nullptr;
    r.B_r = B_r; r.B_theta = B_theta; r.C_r = C_r; r.C_theta = C_theta;
    r.dB_r = dB_r; r.dB_theta = dB_theta; r.dC_r = dC_r; r.dC_theta = dC_theta; r.dD = dD; r.dx_bias = nullptr;
    r.batch = B; r.D = D; r.N = N;
    e = launch_reduce_param_grads(r, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        set_error("scan_unitary_bwd_static: reduction launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}
