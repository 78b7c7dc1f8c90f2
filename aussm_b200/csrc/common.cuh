// Shared device helpers of the sm_100a selective-scan kernels: bulk (TMA)
// copies with mbarrier completion, bounded waits, activations, and a
// float32-accurate sine/cosine.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace aussm {

// ---------------------------------------------------------------------------
// Status word.  A kernel that gives up on a bounded wait records why here and
// returns; the host reads and clears it with aussm_b200_device_status().  Kernels
// receive its address as a parameter (device_status_ptr()).
// ---------------------------------------------------------------------------
enum : int {
    kStatusOk = 0,
    kStatusBarrierTimeout = 1,   // a bulk copy never signalled its mbarrier
};

// ---------------------------------------------------------------------------
// Shared-memory addresses, mbarriers, bulk copies (cp.async.bulk = the TMA
// engine without a tensor map: contiguous bytes, 16-byte aligned both sides).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders this thread's earlier generic-proxy accesses to shared memory before
// later async-proxy (bulk copy) accesses to the same addresses.
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: try_wait itself blocks for a hardware-defined slice, so the
// iteration limit below is seconds of wall time, never reached by a healthy
// copy.  Returns false (after recording the reason) instead of spinning on.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicExch(status, kStatusBarrierTimeout);
    return false;
}

__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem),
                 "r"(smem_addr(src_smem)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until at most N of this thread's committed bulk groups still READ
// their shared-memory source (the buffer may then be overwritten).
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// Activations (the reference's sigmoid / silu / d_silu,
// csrc/cuda/ssm_adaptive_commons.h:92-112, in float32).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }

// returns silu(x) and writes d silu / dx
__device__ __forceinline__ float silu_and_grad(float x, float& grad) {
    float s = sigmoidf_(x);
    grad = s * fmaf(x, 1.0f - s, 1.0f);
    return x * s;
}

// ---------------------------------------------------------------------------
// Sine and cosine of an arbitrary float32 angle, both to about 1e-7 absolute.
//
// The recurrence multiplies the state by exp(i*theta) once per step, so the
// error of this function is paid L times and a biased error would grow
// linearly with the sequence length; the special-function unit's sin/cos
// (2^-21 absolute) is therefore not used by default.  Method: quadrant
// k = round(theta * 2/pi) through the 1.5*2^23 rounding constant (the integer
// lands in the low mantissa bits), two-term Cody-Waite reduction with fused
// multiply-adds, then odd/even polynomials of degree 7/6 on |r| <= pi/4 whose
// coefficients were fitted (weighted least squares on Chebyshev nodes) to
// 2e-9 / 1e-10 before rounding.  Measured over 2e6 angles in [-20, 20]: max
// error 9e-8 (sin and cos), mean phase bias 3e-12, |sin^2+cos^2-1| <= 1.6e-7.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void sincos_accurate(float theta, float& sn, float& cs) {
    const float kMagic = 12582912.0f;            // 1.5 * 2^23
    float kf = fmaf(theta, 0.63661977236758134f, kMagic);
    int q = __float_as_int(kf);
    kf -= kMagic;
    float r = fmaf(kf, -1.5707963705062866f, theta);
    r = fmaf(kf, 4.371138828673793e-08f, r);
    float z = r * r;
    float ps = fmaf(fmaf(-0.00019495567539706826f, z, 0.008331977762281895f), z, -0.16666650772094727f);
    float s = fmaf(ps * z, r, r);
    float pc = fmaf(fmaf(2.4438379114144482e-05f, z, -0.0013887366512790322f), z, 0.04166664555668831f);
    float c = fmaf(pc, z * z, fmaf(-0.5f, z, 1.0f));
    // quadrant fix-up: odd k swaps, bit 1 of k (resp. k+1) flips the sign
    float s1 = (q & 1) ? c : s;
    float c1 = (q & 1) ? s : c;
    sn = __int_as_float(__float_as_int(s1) ^ ((q << 30) & 0x80000000));
    cs = __int_as_float(__float_as_int(c1) ^ (((q + 1) << 30) & 0x80000000));
}

// Special-function-unit variant (2^-21.4 absolute on [-pi, pi]); kept for
// measurement, selected at compile time by the kernels' FAST_TRIG parameter.
__device__ __forceinline__ void sincos_fast(float theta, float& sn, float& cs) {
    float k = rintf(theta * 0.15915494309189535f);
    float r = fmaf(k, -6.2831854820251465f, theta);
    r = fmaf(k, 1.7484555314695172e-07f, r);
    sn = __sinf(r);
    cs = __cosf(r);
}

template <bool FAST>
__device__ __forceinline__ void sincos_sel(float theta, float& sn, float& cs) {
    if (FAST) sincos_fast(theta, sn, cs);
    else sincos_accurate(theta, sn, cs);
}

__device__ __forceinline__ float4 ld_shared_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st_shared_f4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

}  // namespace aussm
