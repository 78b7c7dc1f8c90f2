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
// Special-function-unit exponential and reciprocal in their flush-to-zero forms (one instruction each, no
// range fix-up, about 2 ulp): 1 + 2^(-x log2 e) is at least 1, so nothing near the subnormal range is inverted,
// and an exponential that underflows to zero gives sigmoid = 1 exactly as it should.
__device__ __forceinline__ float ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_ftz(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float sigmoidf_(float x) { return rcp_ftz(1.0f + ex2_ftz(-1.4426950408889634f * x)); }

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
// (2^-21 absolute) is therefore not used by default.  Method: k =
// round(theta/pi) through the 1.5*2^23 rounding constant (the integer lands
// in the low mantissa bits), two-term Cody-Waite reduction with fused
// multiply-adds to |r| <= pi/2, odd/even polynomials of degree 9/10 in r, and
// a sign flip of both results for odd k (one shift, two xors - no quadrant
// swap).  The coefficients were fitted by weighted least squares on Chebyshev
// nodes (4.6e-9 / 2.4e-10 before rounding) and then nudged by single ulps so
// that sin^2+cos^2-1 has mean -8e-10 (a norm bias would make |h| drift).
// Measured in float32 over 4e5 angles: max error 1.0e-7 (sin), 8.3e-8 (cos),
// mean phase error -4e-11.
//
// sincos2 evaluates two angles at once with the packed float32x2
// instructions of sm_100 (one issue slot per two fused multiply-adds).
// ---------------------------------------------------------------------------
#define AUSSM_INV_PI 0.31830987334251404f
#define AUSSM_PI_HI 3.1415927410125732f
#define AUSSM_PI_LO -8.742277657347586e-08f
#define AUSSM_S0 -0.16666656732559204f
#define AUSSM_S1 0.008333015255630016f
#define AUSSM_S2 -0.00019806601630989462f
#define AUSSM_S3 2.6000245725299465e-06f
#define AUSSM_C1 0.04166664183139801f
#define AUSSM_C2 -0.0013888401445001364f
#define AUSSM_C3 2.476187000866048e-05f
#define AUSSM_C4 -2.607681608424173e-07f
#define AUSSM_MAGIC 12582912.0f   /* 1.5 * 2^23 */

__device__ __forceinline__ void sincos_accurate(float theta, float& sn, float& cs) {
    float kf = fmaf(theta, AUSSM_INV_PI, AUSSM_MAGIC);
    const int sign = __float_as_int(kf) << 31;     // odd k: flip both signs
    kf -= AUSSM_MAGIC;
    float r = fmaf(kf, -AUSSM_PI_HI, theta);
    r = fmaf(kf, -AUSSM_PI_LO, r);
    const float z = r * r;
    const float ps = fmaf(fmaf(fmaf(AUSSM_S3, z, AUSSM_S2), z, AUSSM_S1), z, AUSSM_S0);
    const float s = fmaf(ps * z, r, r);
    const float pc = fmaf(fmaf(fmaf(fmaf(AUSSM_C4, z, AUSSM_C3), z, AUSSM_C2), z, AUSSM_C1), z, -0.5f);
    const float c = fmaf(pc, z, 1.0f);
    sn = __int_as_float(__float_as_int(s) ^ sign);
    cs = __int_as_float(__float_as_int(c) ^ sign);
}

__device__ __forceinline__ float2 f2(float a) { return make_float2(a, a); }

__device__ __forceinline__ void sincos2_accurate(float2 theta, float2& sn, float2& cs) {
    float2 kf = __ffma2_rn(theta, f2(AUSSM_INV_PI), f2(AUSSM_MAGIC));
    const int sx = __float_as_int(kf.x) << 31, sy = __float_as_int(kf.y) << 31;
    kf = __fadd2_rn(kf, f2(-AUSSM_MAGIC));
    float2 r = __ffma2_rn(kf, f2(-AUSSM_PI_HI), theta);
    r = __ffma2_rn(kf, f2(-AUSSM_PI_LO), r);
    const float2 z = __fmul2_rn(r, r);
    float2 ps = __ffma2_rn(f2(AUSSM_S3), z, f2(AUSSM_S2));
    ps = __ffma2_rn(ps, z, f2(AUSSM_S1));
    ps = __ffma2_rn(ps, z, f2(AUSSM_S0));
    const float2 s = __ffma2_rn(__fmul2_rn(ps, z), r, r);
    float2 pc = __ffma2_rn(f2(AUSSM_C4), z, f2(AUSSM_C3));
    pc = __ffma2_rn(pc, z, f2(AUSSM_C2));
    pc = __ffma2_rn(pc, z, f2(AUSSM_C1));
    pc = __ffma2_rn(pc, z, f2(-0.5f));
    const float2 c = __ffma2_rn(pc, z, f2(1.0f));
    sn = make_float2(__int_as_float(__float_as_int(s.x) ^ sx), __int_as_float(__float_as_int(s.y) ^ sy));
    cs = make_float2(__int_as_float(__float_as_int(c.x) ^ sx), __int_as_float(__float_as_int(c.y) ^ sy));
}

// four angles -> four (sin, cos) pairs
__device__ __forceinline__ void sincos4(const float (&th)[4], float (&sn)[4], float (&cs)[4]) {
    float2 s01, c01, s23, c23;
    sincos2_accurate(make_float2(th[0], th[1]), s01, c01);
    sincos2_accurate(make_float2(th[2], th[3]), s23, c23);
    sn[0] = s01.x; sn[1] = s01.y; sn[2] = s23.x; sn[3] = s23.y;
    cs[0] = c01.x; cs[1] = c01.y; cs[2] = c23.x; cs[3] = c23.y;
}

// ---------------------------------------------------------------------------
// Asynchronous 16-byte global->shared copies (coalesced: consecutive lanes
// fetch consecutive 16-byte pieces of a row), grouped per thread.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst_smem)), "l"(src_gmem) : "memory");
}
// same copy with the destination given as a 32-bit shared-window address (lets base + immediate fold)
__device__ __forceinline__ void cp_async16_s(uint32_t dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// shared-memory vector access of 1, 2 or 4 floats
template <int VW> struct Vec;
template <> struct Vec<1> {
    float v[1];
    __device__ __forceinline__ void ld(const float* p) { v[0] = *p; }
    __device__ __forceinline__ void st(float* p) const { *p = v[0]; }
    __device__ __forceinline__ void add(const Vec<1>& o) { v[0] += o.v[0]; }
};
template <> struct Vec<2> {
    float v[2];
    __device__ __forceinline__ void ld(const float* p) { float2 t = *reinterpret_cast<const float2*>(p); v[0] = t.x; v[1] = t.y; }
    __device__ __forceinline__ void st(float* p) const { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
    __device__ __forceinline__ void add(const Vec<2>& o) {       // one packed add
        const float2 r = __fadd2_rn(make_float2(v[0], v[1]), make_float2(o.v[0], o.v[1]));
        v[0] = r.x; v[1] = r.y;
    }
};
template <> struct Vec<4> {
    float v[4];
    __device__ __forceinline__ void ld(const float* p) { float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    __device__ __forceinline__ void st(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
    __device__ __forceinline__ void add(const Vec<4>& o) {       // two packed adds
        const float2 a = __fadd2_rn(make_float2(v[0], v[1]), make_float2(o.v[0], o.v[1]));
        const float2 b = __fadd2_rn(make_float2(v[2], v[3]), make_float2(o.v[2], o.v[3]));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
};

__device__ __forceinline__ float4 ld_shared_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st_shared_f4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

}  // namespace aussm
