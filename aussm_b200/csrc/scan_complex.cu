// General complex / positive-real diagonal selective scan for sm_100a.
//
// Same decomposition as scan_unitary.cu and scan_s6.cu: one thread per state
// and channel, sequential in time; one independent warp per 32/NL channels of
// one batch entry; 32-step tiles staged by coalesced 16-byte asynchronous
// copies in a two-stage ring.  A thread consumes its own rho and theta rows
// (like the unitary scan) and the B_j, C_j rows of its batch entry (like the
// S6 scan).  |lambda| != 1, so the recurrence is not reversible: the forward
// kernel stores the state at every tile start, the backward kernel recomputes
// a tile's states from there and walks it in reverse.  drho / dtheta are
// written in place of rho / theta in the stage and leave with coalesced
// stores; dB and dC (sums over the channels of a batch entry) use shuffles and
// vector float atomics, as the reference's kernels do (ssm_adaptive_complex.cu).
#include "scan_complex.cuh"

#include <stdint.h>

#include "common.cuh"
#include "host_common.cuh"

namespace aussm {
namespace {

constexpr int T = kCplxTile;
constexpr int TP = T + 4;
constexpr int STAGES = 2;
constexpr float kLog2e = 1.4426950408889634f;

template <int NL_, bool BWD_>
struct CCfg {
    static constexpr int NL = NL_;
    static constexpr int CPW = 32 / NL;
    static constexpr int AUX = BWD_ ? 4 : 3;                      // u, dt, z [, gy]
    static constexpr int OWN_ROWS = 64;                           // rho rows then theta rows, one per lane
    static constexpr int BC_ROWS = 4 * NL;                        // B_re, B_im, C_re, C_im
    static constexpr int STAGE_FLOATS = (OWN_ROWS + BC_ROWS) * TP + CPW * AUX * T;
    // not staged.  forward: s row + p tile.  backward: s, w rows + h_prev (re, im), E and P tiles
    static constexpr int ROWS = BWD_ ? 2 : 1;
    static constexpr int TILES = BWD_ ? 4 : 1;
    static constexpr int SCRATCH_FLOATS = CPW * ROWS * T + TILES * 32 * TP;
    static constexpr int WARP_FLOATS = STAGES * STAGE_FLOATS + SCRATCH_FLOATS;
    static constexpr size_t SMEM_BYTES = (size_t)WARP_FLOATS * sizeof(float);
    static constexpr int NCH_OWN = OWN_ROWS * (T / 4) / 32;       // 16
    static constexpr int NCH_BC = BC_ROWS * (T / 4) / 32;         // NL
    static constexpr int NCH_AUX = (CPW * AUX * (T / 4) + 31) / 32;
    static constexpr int EPL = CPW * T / 32;
    static constexpr int VW = EPL < 4 ? EPL : 4;
    static constexpr int ITERS = EPL / VW;
};

// per-lane sources of the 16-byte pieces of one tile (at step 0); nullptr = nothing to copy
template <class C>
struct CMap {
    const float* own_ptr[C::NCH_OWN];
    const float* bc_ptr[C::NCH_BC];
    const float* aux_ptr[C::NCH_AUX];

    __device__ __forceinline__ void init(int lane, int nvalid, int N, long long L, const float* rho,
                                         const float* theta, const float* const* bc_src, long long ch0,
                                         const float* const* aux_src) {
#pragma unroll
        for (int i = 0; i < C::NCH_OWN; ++i) {
            const int id = i * 32 + lane;
            const int row = id / (T / 4), col = id % (T / 4);
            const int w = row % 32;                                // the lane that owns the row
            const int c = w / C::NL, j = w % C::NL;
            const float* base = row < 32 ? rho : theta;
            const bool ok = c < nvalid && j < N;
            own_ptr[i] = base ? base + ((ch0 + (ok ? c : 0)) * N + (ok ? j : 0)) * L + col * 4 : nullptr;
        }
#pragma unroll
        for (int i = 0; i < C::NCH_BC; ++i) {
            const int id = i * 32 + lane;
            const int row = id / (T / 4), col = id % (T / 4);
            const int which = row / C::NL, j = row % C::NL;
            const float* base = bc_src[which];
            bc_ptr[i] = base ? base + (long long)(j < N ? j : 0) * L + col * 4 : nullptr;
        }
#pragma unroll
        for (int i = 0; i < C::NCH_AUX; ++i) {
            const int id = i * 32 + lane;
            const int row = id / (T / 4), col = id % (T / 4);
            aux_ptr[i] = nullptr;
            if (row < C::CPW * C::AUX) {
                const int cc = row / C::AUX, a = row % C::AUX;
                aux_ptr[i] = aux_src[a] + (ch0 + (cc < nvalid ? cc : 0)) * L + col * 4;
            }
        }
    }

    __device__ __forceinline__ void issue(float* stage, long long t0, int tlen, int lane) const {
        float* bc = stage + C::OWN_ROWS * TP;
        float* aux = bc + C::BC_ROWS * TP;
#pragma unroll
        for (int i = 0; i < C::NCH_OWN; ++i) {
            const int id = i * 32 + lane;
            const int row = id / (T / 4), col = id % (T / 4);
            if (own_ptr[i] != nullptr && col * 4 < tlen) cp_async16(stage + row * TP + col * 4, own_ptr[i] + t0);
        }
#pragma unroll
        for (int i = 0; i < C::NCH_BC; ++i) {
            const int id = i * 32 + lane;
            const int row = id / (T / 4), col = id % (T / 4);
            if (bc_ptr[i] != nullptr && col * 4 < tlen) cp_async16(bc + row * TP + col * 4, bc_ptr[i] + t0);
        }
#pragma unroll
        for (int i = 0; i < C::NCH_AUX; ++i) {
            const int id = i * 32 + lane;
            const int row = id / (T / 4), col = id % (T / 4);
            if (aux_ptr[i] != nullptr && col * 4 < tlen) cp_async16(aux + row * T + col * 4, aux_ptr[i] + t0);
        }
        cp_async_commit();
    }
};

// rows that are never copied (null inputs) must read as zero
template <class C>
__device__ __forceinline__ void zero_stages(float* smem, int lane) {
    for (int s = 0; s < STAGES; ++s) {
        float* st = smem + s * C::STAGE_FLOATS;
        for (int i = lane; i < (C::OWN_ROWS + C::BC_ROWS) * TP; i += 32) st[i] = 0.f;
    }
    __syncwarp();
}

// lambda = exp(rho + i theta) for four steps
__device__ __forceinline__ void lambda4(const float4 r4, const float4 t4, float (&lr)[4], float (&li)[4]) {
    const float tv[4] = {t4.x, t4.y, t4.z, t4.w};
    const float rv[4] = {r4.x, r4.y, r4.z, r4.w};
    float sn[4], cs[4];
    sincos4(tv, sn, cs);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float m = exp2f(rv[e] * kLog2e);
        lr[e] = m * cs[e];
        li[e] = m * sn[e];
    }
}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
template <int NL>
__global__ void __launch_bounds__(32) cplx_fwd_kernel(const CplxFwdParams p) {
    using C = CCfg<NL, false>;
    constexpr int CPW = C::CPW, AUX = C::AUX, VW = C::VW;
    extern __shared__ __align__(128) float smem[];
    const int lane = threadIdx.x;
    const int tasks_per_batch = (p.Dmod + CPW - 1) / CPW;
    const int b = blockIdx.x / tasks_per_batch, tw = blockIdx.x % tasks_per_batch;
    const int i0 = tw * CPW;
    const int nvalid = min(CPW, p.Dmod - i0);
    const long long ch0 = (long long)b * p.Dmod + i0;
    const int c = lane / NL, j = lane % NL;
    const bool act = c < nvalid && j < p.N;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;
    const long long ch = ch0 + c;

    float* srow = smem + STAGES * C::STAGE_FLOATS;          // [CPW][T]: s = dt silu(u)
    float* pt = srow + CPW * C::ROWS * T;                   // [32][TP]
    zero_stages<C>(smem, lane);

    float hr = 0.f, hi = 0.f;
    float dval[C::ITERS];
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int cc = ((lane + 32 * it) * VW) / T;
        dval[it] = (cc < nvalid && p.Dskip) ? p.Dskip[i0 + cc] : 0.f;
    }
    const long long bo = (long long)b * N * L;
    const float* bc_src[4] = {p.B_re + bo, p.B_im ? p.B_im + bo : nullptr, p.C_re + bo, p.C_im ? p.C_im + bo : nullptr};
    const float* aux_src[AUX] = {p.u, p.dt, p.z};
    CMap<C> map;
    map.init(lane, nvalid, N, L, p.rho, p.theta, bc_src, ch0, aux_src);
    for (int s = 0; s < STAGES; ++s) {
        if (s < ntiles) map.issue(smem + s * C::STAGE_FLOATS, (long long)s * T, min(T, L - s * T), lane);
        else cp_async_commit();
    }

    for (int tile = 0; tile < ntiles; ++tile) {
        float* st = smem + (tile % STAGES) * C::STAGE_FLOATS;
        float* bc = st + C::OWN_ROWS * TP;
        float* aux = bc + C::BC_ROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        const int nq = tlen >> 2;
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        if (act && p.ckpt) {
            float2* ck = reinterpret_cast<float2*>(p.ckpt) + (ch * N + j) * ntiles + tile;
            *ck = make_float2(hr, hi);
        }
#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (t < tlen) {
                Vec<VW> u, d;
                u.ld(aux + (cc * AUX + 0) * T + t);
                d.ld(aux + (cc * AUX + 1) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) d.v[e] *= siluf_(u.v[e]);
                d.st(srow + cc * T + t);
            }
        }
        __syncwarp();

        for (int q = 0; q < nq; ++q) {
            const float4 s4 = ld_shared_f4(srow + c * T + 4 * q);
            const float4 br4 = ld_shared_f4(bc + (0 * NL + j) * TP + 4 * q);
            const float4 bi4 = ld_shared_f4(bc + (1 * NL + j) * TP + 4 * q);
            const float4 cr4 = ld_shared_f4(bc + (2 * NL + j) * TP + 4 * q);
            const float4 ci4 = ld_shared_f4(bc + (3 * NL + j) * TP + 4 * q);
            float lr[4], li[4];
            lambda4(ld_shared_f4(st + lane * TP + 4 * q), ld_shared_f4(st + (32 + lane) * TP + 4 * q), lr, li);
            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
            const float brv[4] = {br4.x, br4.y, br4.z, br4.w}, biv[4] = {bi4.x, bi4.y, bi4.z, bi4.w};
            const float crv[4] = {cr4.x, cr4.y, cr4.z, cr4.w}, civ[4] = {ci4.x, ci4.y, ci4.z, ci4.w};
            float pv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float nr = fmaf(lr[e], hr, fmaf(-li[e], hi, sv[e] * brv[e]));
                const float ni = fmaf(lr[e], hi, fmaf(li[e], hr, sv[e] * biv[e]));
                hr = nr;
                hi = ni;
                pv[e] = act ? fmaf(crv[e], nr, -civ[e] * ni) : 0.f;
            }
            st_shared_f4(pt + lane * TP + 4 * q, make_float4(pv[0], pv[1], pv[2], pv[3]));
        }
        __syncwarp();

#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (t < tlen && cc < nvalid) {
                Vec<VW> acc, u, z;
#pragma unroll
                for (int e = 0; e < VW; ++e) acc.v[e] = 0.f;
#pragma unroll
                for (int r = 0; r < NL; ++r) {
                    Vec<VW> v;
                    v.ld(pt + (cc * NL + r) * TP + t);
#pragma unroll
                    for (int e = 0; e < VW; ++e) acc.v[e] += v.v[e];
                }
                u.ld(aux + (cc * AUX + 0) * T + t);
                z.ld(aux + (cc * AUX + 2) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e)
                    acc.v[e] = siluf_(z.v[e]) * fmaf(dval[it], siluf_(u.v[e]), acc.v[e]);
                acc.st(p.y + (ch0 + cc) * L + t0 + t);
            }
        }
        __syncwarp();
        const int nt = tile + STAGES;
        if (nt < ntiles) map.issue(st, (long long)nt * T, min(T, L - nt * T), lane);
        else cp_async_commit();
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------
__device__ __forceinline__ void red_add_v4c(float* addr, const float (&v)[4]) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]),
                 "f"(v[3])
                 : "memory");
}

template <int NL>
__global__ void __launch_bounds__(32) cplx_bwd_kernel(const CplxBwdParams p) {
    using C = CCfg<NL, true>;
    constexpr int CPW = C::CPW, AUX = C::AUX, VW = C::VW;
    extern __shared__ __align__(128) float smem[];
    const int lane = threadIdx.x;
    const int tasks_per_batch = (p.Dmod + CPW - 1) / CPW;
    const int b = blockIdx.x / tasks_per_batch, tw = blockIdx.x % tasks_per_batch;
    const int i0 = tw * CPW;
    const int nvalid = min(CPW, p.Dmod - i0);
    const long long ch0 = (long long)b * p.Dmod + i0;
    const int c = lane / NL, j = lane % NL;
    const bool act = c < nvalid && j < p.N;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;
    const long long ch = ch0 + c;
    const bool has_rho = p.rho != nullptr, has_theta = p.theta != nullptr;

    float* rows = smem + STAGES * C::STAGE_FLOATS;          // [CPW][2][T]: s, w
    float* hpr = rows + CPW * C::ROWS * T;                  // [32][TP] Re h_{t-1}
    float* hpi = hpr + 32 * TP;                             // [32][TP] Im h_{t-1}
    float* et = hpi + 32 * TP;                              // [32][TP] Re(conj(eta) B)
    float* pt = et + 32 * TP;                               // [32][TP] Re(C h)
    zero_stages<C>(smem, lane);

    float er = 0.f, ei = 0.f;       // conj(lambda_{t+1}) eta_{t+1}
    float dval[C::ITERS], dD_acc[C::ITERS];
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int cc = ((lane + 32 * it) * VW) / T;
        dval[it] = (cc < nvalid && p.Dskip) ? p.Dskip[i0 + cc] : 0.f;
        dD_acc[it] = 0.f;
    }
    const long long bo = (long long)b * N * L;
    const float* bc_src[4] = {p.B_re + bo, p.B_im ? p.B_im + bo : nullptr, p.C_re + bo, p.C_im ? p.C_im + bo : nullptr};
    const float* aux_src[AUX] = {p.u, p.dt, p.z, p.gy};
    CMap<C> map;
    map.init(lane, nvalid, N, L, p.rho, p.theta, bc_src, ch0, aux_src);
    for (int r = 0; r < STAGES; ++r) {
        const int tile = ntiles - 1 - r;
        if (tile >= 0) map.issue(smem + r * C::STAGE_FLOATS, (long long)tile * T, min(T, L - tile * T), lane);
        else cp_async_commit();
    }
    const float2* ck = reinterpret_cast<const float2*>(p.ckpt) + (act ? (ch * N + j) * ntiles : 0);
    float2 h_next = act ? ck[ntiles - 1] : make_float2(0.f, 0.f);
    const long long own_row = (ch * N + j) * (long long)L;

    for (int r = 0; r < ntiles; ++r) {
        const int tile = ntiles - 1 - r;
        float* st = smem + (r % STAGES) * C::STAGE_FLOATS;
        float* bc = st + C::OWN_ROWS * TP;
        float* aux = bc + C::BC_ROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        const int nq = tlen >> 2;
        float hr = h_next.x, hi = h_next.y;
        if (tile > 0 && act) h_next = ck[tile - 1];
        cp_async_wait<STAGES - 1>();
        __syncwarp();

#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (t < tlen) {
                Vec<VW> u, d, z, g;
                u.ld(aux + (cc * AUX + 0) * T + t);
                d.ld(aux + (cc * AUX + 1) * T + t);
                z.ld(aux + (cc * AUX + 2) * T + t);
                g.ld(aux + (cc * AUX + 3) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    d.v[e] *= siluf_(u.v[e]);
                    g.v[e] *= siluf_(z.v[e]);
                }
                d.st(rows + (cc * 2 + 0) * T + t);
                g.st(rows + (cc * 2 + 1) * T + t);
            }
        }
        __syncwarp();

        // recompute the tile's states; keep the state before each step
        for (int q = 0; q < nq; ++q) {
            const float4 s4 = ld_shared_f4(rows + (c * 2 + 0) * T + 4 * q);
            const float4 br4 = ld_shared_f4(bc + (0 * NL + j) * TP + 4 * q);
            const float4 bi4 = ld_shared_f4(bc + (1 * NL + j) * TP + 4 * q);
            float lr[4], li[4];
            lambda4(ld_shared_f4(st + lane * TP + 4 * q), ld_shared_f4(st + (32 + lane) * TP + 4 * q), lr, li);
            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
            const float brv[4] = {br4.x, br4.y, br4.z, br4.w}, biv[4] = {bi4.x, bi4.y, bi4.z, bi4.w};
            float pr[4], pi[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                pr[e] = hr;
                pi[e] = hi;
                const float nr = fmaf(lr[e], hr, fmaf(-li[e], hi, sv[e] * brv[e]));
                const float ni = fmaf(lr[e], hi, fmaf(li[e], hr, sv[e] * biv[e]));
                hr = nr;
                hi = ni;
            }
            st_shared_f4(hpr + lane * TP + 4 * q, make_float4(pr[0], pr[1], pr[2], pr[3]));
            st_shared_f4(hpi + lane * TP + 4 * q, make_float4(pi[0], pi[1], pi[2], pi[3]));
        }

        // reverse pass
        for (int q = nq - 1; q >= 0; --q) {
            const float4 s4 = ld_shared_f4(rows + (c * 2 + 0) * T + 4 * q);
            const float4 w4 = ld_shared_f4(rows + (c * 2 + 1) * T + 4 * q);
            const float4 br4 = ld_shared_f4(bc + (0 * NL + j) * TP + 4 * q);
            const float4 bi4 = ld_shared_f4(bc + (1 * NL + j) * TP + 4 * q);
            const float4 cr4 = ld_shared_f4(bc + (2 * NL + j) * TP + 4 * q);
            const float4 ci4 = ld_shared_f4(bc + (3 * NL + j) * TP + 4 * q);
            const float4 pr4 = ld_shared_f4(hpr + lane * TP + 4 * q);
            const float4 pi4 = ld_shared_f4(hpi + lane * TP + 4 * q);
            float lr[4], li[4];
            lambda4(ld_shared_f4(st + lane * TP + 4 * q), ld_shared_f4(st + (32 + lane) * TP + 4 * q), lr, li);
            const float sv[4] = {s4.x, s4.y, s4.z, s4.w}, wv[4] = {w4.x, w4.y, w4.z, w4.w};
            const float brv[4] = {br4.x, br4.y, br4.z, br4.w}, biv[4] = {bi4.x, bi4.y, bi4.z, bi4.w};
            const float crv[4] = {cr4.x, cr4.y, cr4.z, cr4.w}, civ[4] = {ci4.x, ci4.y, ci4.z, ci4.w};
            const float prv[4] = {pr4.x, pr4.y, pr4.z, pr4.w}, piv[4] = {pi4.x, pi4.y, pi4.z, pi4.w};
            float dr[4], dth[4], E[4], P[4], gBr[4], gBi[4], gCr[4], gCi[4];
#pragma unroll
            for (int e = 3; e >= 0; --e) {
                // a = lambda h_{t-1};  h_t = a + s B
                const float ar = fmaf(lr[e], prv[e], -li[e] * piv[e]);
                const float ai = fmaf(lr[e], piv[e], li[e] * prv[e]);
                const float htr = fmaf(sv[e], brv[e], ar), hti = fmaf(sv[e], biv[e], ai);
                // eta_t = carry + conj(C) w
                const float nr = fmaf(crv[e], wv[e], er), ni = fmaf(-civ[e], wv[e], ei);
                dr[e] = fmaf(nr, ar, ni * ai);            // Re(conj(eta) a)
                dth[e] = fmaf(ni, ar, -nr * ai);          // -Im(conj(eta) a)
                E[e] = act ? fmaf(nr, brv[e], ni * biv[e]) : 0.f;
                P[e] = act ? fmaf(crv[e], htr, -civ[e] * hti) : 0.f;
                gBr[e] = act ? nr * sv[e] : 0.f;
                gBi[e] = act ? ni * sv[e] : 0.f;
                gCr[e] = act ? wv[e] * htr : 0.f;
                gCi[e] = act ? -wv[e] * hti : 0.f;
                er = fmaf(lr[e], nr, li[e] * ni);         // conj(lambda) eta
                ei = fmaf(lr[e], ni, -li[e] * nr);
            }
            if (has_rho) st_shared_f4(st + lane * TP + 4 * q, make_float4(dr[0], dr[1], dr[2], dr[3]));
            if (has_theta) st_shared_f4(st + (32 + lane) * TP + 4 * q, make_float4(dth[0], dth[1], dth[2], dth[3]));
            st_shared_f4(et + lane * TP + 4 * q, make_float4(E[0], E[1], E[2], E[3]));
            st_shared_f4(pt + lane * TP + 4 * q, make_float4(P[0], P[1], P[2], P[3]));
#pragma unroll
            for (int off = NL; off < 32; off <<= 1) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    gBr[e] += __shfl_xor_sync(0xffffffffu, gBr[e], off);
                    gBi[e] += __shfl_xor_sync(0xffffffffu, gBi[e], off);
                    gCr[e] += __shfl_xor_sync(0xffffffffu, gCr[e], off);
                    gCi[e] += __shfl_xor_sync(0xffffffffu, gCi[e], off);
                }
            }
            if (c == 0 && j < N) {
                const long long o = bo + (long long)j * L + t0 + 4 * q;
                red_add_v4c(p.dB_re + o, gBr);
                red_add_v4c(p.dC_re + o, gCr);
                if (p.dB_im) red_add_v4c(p.dB_im + o, gBi);
                if (p.dC_im) red_add_v4c(p.dC_im + o, gCi);
            }
        }
        __syncwarp();

#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (t < tlen && cc < nvalid) {
                Vec<VW> SE, SP, u, d, z, g, du, ddt, dz;
#pragma unroll
                for (int e = 0; e < VW; ++e) SE.v[e] = SP.v[e] = 0.f;
#pragma unroll
                for (int rr = 0; rr < NL; ++rr) {
                    Vec<VW> a, bb;
                    a.ld(et + (cc * NL + rr) * TP + t);
                    bb.ld(pt + (cc * NL + rr) * TP + t);
#pragma unroll
                    for (int e = 0; e < VW; ++e) { SE.v[e] += a.v[e]; SP.v[e] += bb.v[e]; }
                }
                u.ld(aux + (cc * AUX + 0) * T + t);
                d.ld(aux + (cc * AUX + 1) * T + t);
                z.ld(aux + (cc * AUX + 2) * T + t);
                g.ld(aux + (cc * AUX + 3) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    float gu, gz;
                    const float v = silu_and_grad(u.v[e], gu);
                    const float gg = silu_and_grad(z.v[e], gz);
                    const float w = g.v[e] * gg;
                    dz.v[e] = g.v[e] * fmaf(dval[it], v, SP.v[e]) * gz;
                    ddt.v[e] = SE.v[e] * v;
                    du.v[e] = fmaf(SE.v[e], d.v[e], w * dval[it]) * gu;
                    dD_acc[it] = fmaf(w, v, dD_acc[it]);
                }
                const long long off = (ch0 + cc) * L + t0 + t;
                du.st(p.du + off);
                ddt.st(p.ddt + off);
                dz.st(p.dz + off);
            }
        }
        __syncwarp();
        // drho / dtheta leave the stage (each lane stores pieces of real rows only)
#pragma unroll
        for (int i = 0; i < C::NCH_OWN; ++i) {
            const int id = i * 32 + lane;
            const int row = id / (T / 4), col = id % (T / 4);
            const int w = row % 32;
            const int rc = w / NL, rj = w % NL;
            float* base = row < 32 ? p.drho : p.dtheta;
            const bool on = row < 32 ? has_rho : has_theta;
            if (on && base && rc < nvalid && rj < N && col * 4 < tlen)
                *reinterpret_cast<float4*>(base + ((ch0 + rc) * N + rj) * (long long)L + t0 + col * 4) =
                    ld_shared_f4(st + row * TP + col * 4);
        }
        __syncwarp();
        const int nr = r + STAGES;
        if (nr < ntiles) {
            const int nt = ntiles - 1 - nr;
            map.issue(st, (long long)nt * T, min(T, L - nt * T), lane);
        } else {
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
    (void)own_row;

    __syncwarp();
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) et[lane + 32 * it] = dD_acc[it];
    __syncwarp();
    if (lane < nvalid) {
        float aD = 0.f;
        for (int idx = 0; idx < 32 * C::ITERS; ++idx)
            if ((idx * VW) / T == lane) aD += et[idx];
        p.part_D[ch0 + lane] = aD;
    }
}

__global__ void __launch_bounds__(256) cplx_reduce_D_kernel(const float* part_D, float* dD, int batch, int D) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= D) return;
    float acc = 0.f;
    for (int b = 0; b < batch; ++b) acc += part_D[(long long)b * D + i];
    dD[i] = acc;
}

template <int NL, bool BWD, class Kern, class Params>
cudaError_t launch_nl(Kern kern, const Params& p, cudaStream_t stream) {
    using C = CCfg<NL, BWD>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long blocks = (long long)(p.nch / p.Dmod) * ((p.Dmod + C::CPW - 1) / C::CPW);
    kern<<<(unsigned)blocks, 32, C::SMEM_BYTES, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_cplx_fwd(const CplxFwdParams& p, cudaStream_t stream) {
    if (p.nch <= 0 || p.L <= 0) return cudaSuccess;
    if (p.N <= 4) return launch_nl<4, false>(cplx_fwd_kernel<4>, p, stream);
    if (p.N <= 8) return launch_nl<8, false>(cplx_fwd_kernel<8>, p, stream);
    if (p.N <= 16) return launch_nl<16, false>(cplx_fwd_kernel<16>, p, stream);
    if (p.N <= 32) return launch_nl<32, false>(cplx_fwd_kernel<32>, p, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_cplx_bwd(const CplxBwdParams& p, cudaStream_t stream) {
    if (p.nch <= 0 || p.L <= 0) return cudaSuccess;
    if (p.N <= 4) return launch_nl<4, true>(cplx_bwd_kernel<4>, p, stream);
    if (p.N <= 8) return launch_nl<8, true>(cplx_bwd_kernel<8>, p, stream);
    if (p.N <= 16) return launch_nl<16, true>(cplx_bwd_kernel<16>, p, stream);
    if (p.N <= 32) return launch_nl<32, true>(cplx_bwd_kernel<32>, p, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_cplx_reduce_D(const float* part_D, float* dD, int batch, int D, cudaStream_t stream) {
    cplx_reduce_D_kernel<<<(D + 255) / 256, 256, 0, stream>>>(part_D, dD, batch, D);
    count_launch();
    return cudaGetLastError();
}

}  // namespace aussm
