// General complex / positive-real diagonal selective scan for sm_100a.
//
// Same decomposition as scan_unitary.cu and scan_s6.cu: one thread per state
// and channel, sequential in time; one warp per 32/NL channels of one batch
// entry; 16-step tiles staged by coalesced 16-byte asynchronous copies in a
// two-stage ring.  A thread consumes its own rho and theta rows (like the
// unitary scan) and the B_j, C_j rows of its batch entry (like the S6 scan).
// The B / C rows are the same for every channel of a batch entry, so the warps
// of a block (all of one batch entry) share one copy of them: each warp fetches
// its share, two block barriers per tile make the copy visible and protect it
// from being refilled early.  |lambda| != 1, so the recurrence is not reversible: the forward
// kernel records the state at every tile start, the backward kernel recomputes
// a tile's states from there and walks it in reverse.
//
// Shared memory is what limits the number of resident warps (each state keeps
// two streams in flight), so the tiles are short (16 steps) and every cell is
// used several times: the backward kernel's recomputing pass keeps lambda and
// the state before each step of the tile in registers (the reverse pass then
// needs no second exponential and sine / cosine, and no shared-memory round
// trip: the shared-memory pipe is the busiest unit of this kernel); the reverse
// pass writes drho / dtheta over the rho / theta cells, which leave with
// coalesced stores.  dB and dC (sums over the channels of a
// batch entry) use shuffles and vector float atomics, as the reference's
// kernels do (ssm_adaptive_complex.cu:358-660).
#include "scan_complex.cuh"

#include <stdint.h>

#include "common.cuh"

namespace aussm {
namespace {

constexpr int T = kCplxTile;
constexpr int TP = T + 4;
constexpr int STAGES = 2;
constexpr int NQ = T / 4;
constexpr float kLog2e = 1.4426950408889634f;

constexpr int cmaxi(int a, int b) { return a > b ? a : b; }
constexpr int cmini(int a, int b) { return a < b ? a : b; }

template <int NL_, bool BWD_, bool REAL_ = false>
struct CCfg {
    static constexpr int NL = NL_;
    static constexpr int CPW = 32 / NL;
    // warps per block: in the forward kernel they share the B / C tiles of their batch entry (measured 2.55
    // against 2.75 ms at batch 8 x 2048 channels x 4096 steps).  The backward kernel, and few states per channel
    // (small tiles anyway), keep one-warp blocks: with six warps sharing the tiles it measured 9.85 against 9.15
    // ms - its warps drift apart (atomics, long reverse pass) and wait for each other at the two barriers.
    static constexpr int WARPS = (NL >= 8 && !BWD_) ? 4 : 1;
    static constexpr int AUX = BWD_ ? 4 : 3;                      // u, dt, z [, gy]
    static constexpr bool REAL = REAL_;                           // no theta rows, no imaginary B / C rows
    static constexpr int OWN_ROWS = REAL_ ? 32 : 64;              // rho rows then theta rows, one per lane
    static constexpr int BC_ROWS = (REAL_ ? 2 : 4) * NL;          // B_re, B_im, C_re, C_im (real: B_re, C_re)
    static constexpr int CROW = REAL_ ? 1 : 2;                    // block of the tile that holds C_re
    static constexpr int STAGE_FLOATS = OWN_ROWS * TP + CPW * AUX * T;      // per warp
    static constexpr int BC_FLOATS = BC_ROWS * TP;                          // per block
    // not staged.  forward: s row + p tile.  backward: s, w, d silu(u)/du rows + the tiles of the two column sums
    static constexpr int ROWS = BWD_ ? 3 : 1;
    static constexpr int TILES = BWD_ ? 2 : 1;
    static constexpr int SCRATCH_FLOATS = CPW * ROWS * T + TILES * 32 * TP;
    static constexpr int WARP_FLOATS = STAGES * STAGE_FLOATS + SCRATCH_FLOATS;
    static constexpr size_t SMEM_BYTES = (size_t)(STAGES * BC_FLOATS + WARPS * WARP_FLOATS) * sizeof(float);
    static constexpr int NCH_OWN = OWN_ROWS * NQ / 32;
    static constexpr int NCH_BC = (BC_ROWS * NQ + 32 * WARPS - 1) / (32 * WARPS);   // this warp's share
    static constexpr int NCH_AUX = (CPW * AUX * NQ + 31) / 32;
    // per-(channel, step) passes: CPW * T elements over 32 lanes
    static constexpr int ELEMS = CPW * T;
    static constexpr int VW = cmaxi(1, cmini(4, ELEMS / 32));
    static constexpr int ITERS = cmaxi(1, ELEMS / (32 * VW));
};

// per-lane sources of the 16-byte pieces of one tile (at step 0 of the launch); nullptr = nothing to copy
template <class C>
struct CMap {
    const float* own_ptr[C::NCH_OWN];
    const float* bc_ptr[C::NCH_BC];
    const float* aux_ptr[C::NCH_AUX];

    __device__ __forceinline__ void init(int lane, int warp, int nvalid, int N, const float* rho_b,
                                         const float* theta_b, long long ld_lam, int i0, const float* const* bc_src,
                                         const float* const* aux_src, long long ch0, long long ld_row) {
#pragma unroll
        for (int i = 0; i < C::NCH_OWN; ++i) {
            const int id = i * 32 + lane;
            const int row = id / NQ, col = id % NQ;
            const int w = row % 32;                                // the lane that owns the row
            const int c = w / C::NL, j = w % C::NL;
            const float* base = row < 32 ? rho_b : theta_b;        // rows of this batch entry
            const bool ok = c < nvalid && j < N;
            own_ptr[i] = base ? base + ((long long)(i0 + (ok ? c : 0)) * N + (ok ? j : 0)) * ld_lam + col * 4 : nullptr;
        }
#pragma unroll
        for (int i = 0; i < C::NCH_BC; ++i) {
            const int id = (i * C::WARPS + warp) * 32 + lane;      // piece of the block's B / C tile
            const int row = id / NQ, col = id % NQ;
            bc_ptr[i] = nullptr;
            if (row < C::BC_ROWS) {
                const int which = (C::REAL ? 2 : 1) * (row / C::NL), j = row % C::NL;
                const float* base = bc_src[which];
                bc_ptr[i] = base ? base + (long long)(j < N ? j : 0) * ld_row + col * 4 : nullptr;
            }
        }
#pragma unroll
        for (int i = 0; i < C::NCH_AUX; ++i) {
            const int id = i * 32 + lane;
            const int row = id / NQ, col = id % NQ;
            aux_ptr[i] = nullptr;
            if (row < C::CPW * C::AUX) {
                const int cc = row / C::AUX, a = row % C::AUX;
                aux_ptr[i] = aux_src[a] + (ch0 + (cc < nvalid ? cc : 0)) * ld_row + col * 4;
            }
        }
    }

    // stage: this warp's rows; bc: the block's B / C tile of the same stage
    __device__ __forceinline__ void issue(float* stage, float* bc, long long t0, int tlen, int lane, int warp) const {
        float* aux = stage + C::OWN_ROWS * TP;
        const int col = lane % NQ, r0 = lane / NQ;                 // piece i of this lane: row i * (32 / NQ) + r0
        constexpr int RPI = 32 / NQ;
        if (col * 4 < tlen) {
#pragma unroll
            for (int i = 0; i < C::NCH_OWN; ++i)
                if (own_ptr[i] != nullptr) cp_async16(stage + (i * RPI + r0) * TP + col * 4, own_ptr[i] + t0);
#pragma unroll
            for (int i = 0; i < C::NCH_BC; ++i)
                if (bc_ptr[i] != nullptr)
                    cp_async16(bc + ((i * C::WARPS + warp) * RPI + r0) * TP + col * 4, bc_ptr[i] + t0);
#pragma unroll
            for (int i = 0; i < C::NCH_AUX; ++i)
                if (aux_ptr[i] != nullptr) cp_async16(aux + (i * RPI + r0) * T + col * 4, aux_ptr[i] + t0);
        }
        cp_async_commit();
    }
};

// rows that are never copied (null inputs) must read as zero
template <class C>
__device__ __forceinline__ void zero_stages(float* bc_ring, float* wsm, int lane) {
    for (int i = threadIdx.x; i < STAGES * C::BC_FLOATS; i += C::WARPS * 32) bc_ring[i] = 0.f;
    for (int s = 0; s < STAGES; ++s) {
        float* st = wsm + s * C::STAGE_FLOATS;
        for (int i = lane; i < C::OWN_ROWS * TP; i += 32) st[i] = 0.f;
    }
    if (C::WARPS > 1) __syncthreads(); else __syncwarp();
}

template <class C>
__device__ __forceinline__ void block_sync() {
    if (C::WARPS > 1) __syncthreads(); else __syncwarp();
}

// lambda = exp(rho + i theta) for four steps
__device__ __forceinline__ void lambda4(const float4 r4, const float4 t4, float (&lr)[4], float (&li)[4]) {
    const float tv[4] = {t4.x, t4.y, t4.z, t4.w};
    const float rv[4] = {r4.x, r4.y, r4.z, r4.w};
    float sn[4], cs[4];
    sincos4(tv, sn, cs);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float m = ex2_ftz(rv[e] * kLog2e);
        lr[e] = m * cs[e];
        li[e] = m * sn[e];
    }
}

#define AUSSM_F4(v) {(v).x, (v).y, (v).z, (v).w}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
// REAL: no angle stream and real B, C - the state, the multiplier and every product are real (the positive-real
// operator); the imaginary halves of the arithmetic and the sine / cosine are compiled out.
template <int NL, bool REAL>
__global__ void __launch_bounds__(CCfg<NL, false>::WARPS * 32) cplx_fwd_kernel(const CplxFwdParams p) {
    using C = CCfg<NL, false, REAL>;
    constexpr int CPW = C::CPW, AUX = C::AUX, VW = C::VW;
    extern __shared__ __align__(128) float smem_all[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // a block = WARPS consecutive tasks (32/NL channels each) of one batch entry; a warp beyond the last task
    // shadows it (it takes part in the copies of the shared tile and in the barriers, and stores nothing)
    const int tasks_per_batch = (p.Dmod + CPW - 1) / CPW;
    const int blocks_per_batch = (tasks_per_batch + C::WARPS - 1) / C::WARPS;
    const int b = blockIdx.x / blocks_per_batch;
    const int tw_raw = (blockIdx.x % blocks_per_batch) * C::WARPS + warp;
    const int tw = min(tw_raw, tasks_per_batch - 1);
    const int i0 = tw * CPW;
    const int nvalid = tw_raw < tasks_per_batch ? min(CPW, p.Dmod - i0) : 0;
    const long long ch0 = (long long)b * p.Dmod + i0;
    float* bc_ring = smem_all;
    float* smem = smem_all + STAGES * C::BC_FLOATS + warp * C::WARP_FLOATS;
    const int c = lane / NL, j = lane % NL;
    const bool act = c < nvalid && j < p.N;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;
    const long long ch = ch0 + c;

    float* srow = smem + STAGES * C::STAGE_FLOATS;          // [CPW][T]: s = dt silu(u)
    float* pt = srow + CPW * C::ROWS * T;                   // [32][TP]
    zero_stages<C>(bc_ring, smem, lane);

    float2* rec = (p.states && act) ? reinterpret_cast<float2*>(p.states) + (ch * N + j) * p.states_stride + p.tile0
                                    : nullptr;
    float hr = 0.f, hi = 0.f;
    if (rec && p.tile0 > 0) {
        const float2 h0 = rec[0];
        hr = h0.x;
        hi = h0.y;
    }
    float dval[C::ITERS];
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int cc = ((lane + 32 * it) * VW) / T;
        dval[it] = (cc < nvalid && p.Dskip) ? p.Dskip[i0 + cc] : 0.f;
    }
    const long long bo = (long long)b * N * p.ld_row;
    const float* bc_src[4] = {p.B_re + bo, p.B_im ? p.B_im + bo : nullptr, p.C_re + bo, p.C_im ? p.C_im + bo : nullptr};
    const float* aux_src[AUX] = {p.u, p.dt, p.z};
    const long long lam_b = (long long)b * p.lam_batch_stride;
    CMap<C> map;
    map.init(lane, warp, nvalid, N, p.rho ? p.rho + lam_b : nullptr, p.theta ? p.theta + lam_b : nullptr, p.ld_lam,
             i0, bc_src, aux_src, ch0, p.ld_row);
    for (int s = 0; s < STAGES; ++s) {
        if (s < ntiles)
            map.issue(smem + s * C::STAGE_FLOATS, bc_ring + s * C::BC_FLOATS, (long long)s * T, min(T, L - s * T), lane,
                      warp);
        else cp_async_commit();
    }

    for (int tile = 0; tile < ntiles; ++tile) {
        float* st = smem + (tile % STAGES) * C::STAGE_FLOATS;
        float* bc = bc_ring + (tile % STAGES) * C::BC_FLOATS;
        float* aux = st + C::OWN_ROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        cp_async_wait<STAGES - 1>();
        block_sync<C>();                                    // every warp's share of the B / C tile has landed
        if (rec) rec[tile] = make_float2(hr, hi);
        // pre-pass: silu(u) replaces u, s = dt silu(u)
#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (e0 < C::ELEMS && t < tlen) {
                Vec<VW> u, d;
                u.ld(aux + (cc * AUX + 0) * T + t);
                d.ld(aux + (cc * AUX + 1) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    u.v[e] = siluf_(u.v[e]);
                    d.v[e] *= u.v[e];
                }
                u.st(aux + (cc * AUX + 0) * T + t);
                d.st(srow + cc * T + t);
            }
        }
        __syncwarp();

        auto quad = [&](const int q) {
            const float4 s4 = ld_shared_f4(srow + c * T + 4 * q);
            const float4 br4 = ld_shared_f4(bc + (0 * NL + j) * TP + 4 * q);
            const float4 cr4 = ld_shared_f4(bc + (C::CROW * NL + j) * TP + 4 * q);
            const float sv[4] = AUSSM_F4(s4);
            const float brv[4] = AUSSM_F4(br4), crv[4] = AUSSM_F4(cr4);
            float pv[4];
            if (REAL) {
                const float4 r4 = ld_shared_f4(st + lane * TP + 4 * q);
                const float rv[4] = AUSSM_F4(r4);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    hr = fmaf(ex2_ftz(rv[e] * kLog2e), hr, sv[e] * brv[e]);
                    pv[e] = act ? crv[e] * hr : 0.f;
                }
            } else {
                const float4 bi4 = ld_shared_f4(bc + (1 * NL + j) * TP + 4 * q);
                const float4 ci4 = ld_shared_f4(bc + (3 * NL + j) * TP + 4 * q);
                float lr[4], li[4];
                lambda4(ld_shared_f4(st + lane * TP + 4 * q), ld_shared_f4(st + (32 + lane) * TP + 4 * q), lr, li);
                const float biv[4] = AUSSM_F4(bi4), civ[4] = AUSSM_F4(ci4);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float nr = fmaf(lr[e], hr, fmaf(-li[e], hi, sv[e] * brv[e]));
                    const float ni = fmaf(lr[e], hi, fmaf(li[e], hr, sv[e] * biv[e]));
                    hr = nr;
                    hi = ni;
                    pv[e] = act ? fmaf(crv[e], nr, -civ[e] * ni) : 0.f;
                }
            }
            st_shared_f4(pt + lane * TP + 4 * q, make_float4(pv[0], pv[1], pv[2], pv[3]));
        };
        if (tlen == T) {
#pragma unroll
            for (int q = 0; q < NQ; ++q) quad(q);
        } else {
            for (int q = 0; q < (tlen >> 2); ++q) quad(q);
        }
        __syncwarp();

#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (e0 < C::ELEMS && t < tlen && cc < nvalid) {
                Vec<VW> acc, v, z;
                acc.ld(pt + cc * NL * TP + t);
#pragma unroll
                for (int r = 1; r < NL; ++r) {
                    Vec<VW> a;
                    a.ld(pt + (cc * NL + r) * TP + t);
                    acc.add(a);
                }
                v.ld(aux + (cc * AUX + 0) * T + t);          // silu(u), left by the pre-pass
                z.ld(aux + (cc * AUX + 2) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) acc.v[e] = siluf_(z.v[e]) * fmaf(dval[it], v.v[e], acc.v[e]);
                acc.st(p.y + (ch0 + cc) * p.ld_row + t0 + t);
            }
        }
        block_sync<C>();                                    // nobody reads this stage's B / C tile any more
        const int nt = tile + STAGES;
        if (nt < ntiles) map.issue(st, bc, (long long)nt * T, min(T, L - nt * T), lane, warp);
        else cp_async_commit();
    }
    cp_async_wait<0>();
    if (rec) rec[ntiles] = make_float2(hr, hi);
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------
__device__ __forceinline__ void red_add_v4c(float* addr, const float (&v)[4]) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]),
                 "f"(v[3])
                 : "memory");
}

template <int NL, bool REAL>
__global__ void __launch_bounds__(CCfg<NL, true>::WARPS * 32)
cplx_bwd_kernel(const CplxBwdParams p) {
    using C = CCfg<NL, true, REAL>;
    constexpr int CPW = C::CPW, AUX = C::AUX, VW = C::VW;
    extern __shared__ __align__(128) float smem_all[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tasks_per_batch = (p.Dmod + CPW - 1) / CPW;
    const int blocks_per_batch = (tasks_per_batch + C::WARPS - 1) / C::WARPS;
    const int b = blockIdx.x / blocks_per_batch;
    const int tw_raw = (blockIdx.x % blocks_per_batch) * C::WARPS + warp;
    const int tw = min(tw_raw, tasks_per_batch - 1);          // warps beyond the last task shadow it
    const int i0 = tw * CPW;
    const int nvalid = tw_raw < tasks_per_batch ? min(CPW, p.Dmod - i0) : 0;
    const long long ch0 = (long long)b * p.Dmod + i0;
    float* bc_ring = smem_all;
    float* smem = smem_all + STAGES * C::BC_FLOATS + warp * C::WARP_FLOATS;
    const int c = lane / NL, j = lane % NL;
    const bool act = c < nvalid && j < p.N;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;
    const long long ch = ch0 + c;
    const bool has_rho = p.rho != nullptr, has_theta = p.theta != nullptr;

    float* rows = smem + STAGES * C::STAGE_FLOATS;          // [CPW][3][T]: s, w, d silu(u)/du
    float* et = rows + CPW * C::ROWS * T;                   // [32][TP] Re(conj(eta) B)
    float* pt = et + 32 * TP;                               // [32][TP] Re(C h)
    zero_stages<C>(bc_ring, smem, lane);

    const long long rec_off = (ch * N + j) * p.states_stride + p.tile0;
    const float2* rec = reinterpret_cast<const float2*>(p.states) + (act ? rec_off : 0);
    const float2* grec = (p.gstates && act) ? reinterpret_cast<const float2*>(p.gstates) + rec_off : nullptr;
    float er = 0.f, ei = 0.f;       // conj(lambda_{t+1}) eta_{t+1}: the gradient that reaches h_t from later steps
    if (act) {
        if (p.eta_in) {
            const float2 e0 = reinterpret_cast<const float2*>(p.eta_in)[ch * N + j];
            er = e0.x;
            ei = e0.y;
        } else if (grec) {            // last window: the gradient of the recorded final state enters here
            const float2 g = grec[ntiles];
            er = g.x;
            ei = g.y;
        }
    }
    float dval[C::ITERS], dD_acc[C::ITERS];
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int cc = ((lane + 32 * it) * VW) / T;
        dval[it] = (cc < nvalid && p.Dskip) ? p.Dskip[i0 + cc] : 0.f;
        dD_acc[it] = 0.f;
    }
    const long long bo = (long long)b * N * p.ld_row;
    const float* bc_src[4] = {p.B_re + bo, p.B_im ? p.B_im + bo : nullptr, p.C_re + bo, p.C_im ? p.C_im + bo : nullptr};
    const float* aux_src[AUX] = {p.u, p.dt, p.z, p.gy};
    const long long lam_b = (long long)b * p.lam_batch_stride;
    CMap<C> map;
    map.init(lane, warp, nvalid, N, has_rho ? p.rho + lam_b : nullptr, has_theta ? p.theta + lam_b : nullptr,
             p.ld_lam, i0, bc_src, aux_src, ch0, p.ld_row);
    for (int r = 0; r < STAGES; ++r) {
        const int tile = ntiles - 1 - r;
        if (tile >= 0)
            map.issue(smem + r * C::STAGE_FLOATS, bc_ring + r * C::BC_FLOATS, (long long)tile * T,
                      min(T, L - tile * T), lane, warp);
        else cp_async_commit();
    }
    float2 h_next = act ? rec[ntiles - 1] : make_float2(0.f, 0.f);

    for (int r = 0; r < ntiles; ++r) {
        const int tile = ntiles - 1 - r;
        float* st = smem + (r % STAGES) * C::STAGE_FLOATS;
        float* bc = bc_ring + (r % STAGES) * C::BC_FLOATS;
        float* aux = st + C::OWN_ROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        const int nq = tlen >> 2;
        float hr = h_next.x, hi = h_next.y;                 // state before the tile's first step
        if (tile > 0 && act) h_next = rec[tile - 1];
        cp_async_wait<STAGES - 1>();
        block_sync<C>();                                    // every warp's share of the B / C tile has landed

        // pre-pass: every activation once.  s = dt silu(u) and w = gy silu(z) feed the scan; silu(u) and
        // d silu(z)/dz replace the u and z cells, d silu(u)/du gets a row of its own.
#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (e0 < C::ELEMS && t < tlen) {
                Vec<VW> u, d, z, g, gu;
                u.ld(aux + (cc * AUX + 0) * T + t);
                d.ld(aux + (cc * AUX + 1) * T + t);
                z.ld(aux + (cc * AUX + 2) * T + t);
                g.ld(aux + (cc * AUX + 3) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    float gz;
                    u.v[e] = silu_and_grad(u.v[e], gu.v[e]);
                    d.v[e] *= u.v[e];
                    g.v[e] *= silu_and_grad(z.v[e], gz);
                    z.v[e] = gz;
                }
                u.st(aux + (cc * AUX + 0) * T + t);
                z.st(aux + (cc * AUX + 2) * T + t);
                d.st(rows + (cc * 3 + 0) * T + t);
                g.st(rows + (cc * 3 + 1) * T + t);
                gu.st(rows + (cc * 3 + 2) * T + t);
            }
        }
        __syncwarp();

        // recompute the tile's states: lambda replaces (rho, theta) in the stage, the state before each step
        // stays in registers (the quads of a tile are unrolled, so the arrays are indexed statically)
        float hpr[T], hpi[REAL ? 1 : T];
        float lmr[T], lmi[REAL ? 1 : T];                      // lambda of every step of the tile
        auto recompute = [&](const int q) {
            const float4 s4 = ld_shared_f4(rows + (c * 3 + 0) * T + 4 * q);
            const float4 br4 = ld_shared_f4(bc + (0 * NL + j) * TP + 4 * q);
            const float sv[4] = AUSSM_F4(s4);
            const float brv[4] = AUSSM_F4(br4);
            if (REAL) {
                const float4 r4 = ld_shared_f4(st + lane * TP + 4 * q);
                const float rv[4] = AUSSM_F4(r4);
                float lr[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    lr[e] = ex2_ftz(rv[e] * kLog2e);
                    hpr[4 * q + e] = hr;
                    lmr[4 * q + e] = lr[e];
                    hr = fmaf(lr[e], hr, sv[e] * brv[e]);
                }
                return;
            }
            const float4 bi4 = ld_shared_f4(bc + (1 * NL + j) * TP + 4 * q);
            float lr[4], li[4];
            lambda4(ld_shared_f4(st + lane * TP + 4 * q), ld_shared_f4(st + (32 + lane) * TP + 4 * q), lr, li);
            const float biv[4] = AUSSM_F4(bi4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                hpr[4 * q + e] = hr;
                hpi[REAL ? 0 : 4 * q + e] = hi;
                lmr[4 * q + e] = lr[e];
                lmi[REAL ? 0 : 4 * q + e] = li[e];
                const float nr = fmaf(lr[e], hr, fmaf(-li[e], hi, sv[e] * brv[e]));
                const float ni = fmaf(lr[e], hi, fmaf(li[e], hr, sv[e] * biv[e]));
                hr = nr;
                hi = ni;
            }
        };
        // reverse pass of the real operator: eta, lambda, the states and every product are real
        auto reverse_real = [&](const int q) {
            const float4 s4 = ld_shared_f4(rows + (c * 3 + 0) * T + 4 * q);
            const float4 w4 = ld_shared_f4(rows + (c * 3 + 1) * T + 4 * q);
            const float4 br4 = ld_shared_f4(bc + (0 * NL + j) * TP + 4 * q);
            const float4 cr4 = ld_shared_f4(bc + (C::CROW * NL + j) * TP + 4 * q);
            const float sv[4] = AUSSM_F4(s4), wv[4] = AUSSM_F4(w4);
            const float brv[4] = AUSSM_F4(br4), crv[4] = AUSSM_F4(cr4);
            const float lr[4] = {lmr[4 * q], lmr[4 * q + 1], lmr[4 * q + 2], lmr[4 * q + 3]};
            const float prv[4] = {hpr[4 * q], hpr[4 * q + 1], hpr[4 * q + 2], hpr[4 * q + 3]};
            float dr[4], E[4], P[4], gBr[4], gCr[4];
#pragma unroll
            for (int e = 3; e >= 0; --e) {
                const float ar = lr[e] * prv[e];                  // a = lambda h_{t-1};  h_t = a + s B
                const float htr = fmaf(sv[e], brv[e], ar);
                const float nr = fmaf(crv[e], wv[e], er);         // eta_t = carry + C w
                dr[e] = nr * ar;
                E[e] = act ? nr * brv[e] : 0.f;
                P[e] = act ? crv[e] * htr : 0.f;
                gBr[e] = act ? nr * sv[e] : 0.f;
                gCr[e] = act ? wv[e] * htr : 0.f;
                er = lr[e] * nr;
            }
            st_shared_f4(st + lane * TP + 4 * q, make_float4(dr[0], dr[1], dr[2], dr[3]));
            st_shared_f4(et + lane * TP + 4 * q, make_float4(E[0], E[1], E[2], E[3]));
            st_shared_f4(pt + lane * TP + 4 * q, make_float4(P[0], P[1], P[2], P[3]));
#pragma unroll
            for (int off = NL; off < 32; off <<= 1) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    gBr[e] += __shfl_xor_sync(0xffffffffu, gBr[e], off);
                    gCr[e] += __shfl_xor_sync(0xffffffffu, gCr[e], off);
                }
            }
            if (c == 0 && j < N && nvalid > 0) {
                const long long o = bo + (long long)j * p.ld_row + t0 + 4 * q;
                red_add_v4c(p.dB_re + o, gBr);
                red_add_v4c(p.dC_re + o, gCr);
            }
        };
        // reverse pass
        auto reverse = [&](const int q) {
            const float4 s4 = ld_shared_f4(rows + (c * 3 + 0) * T + 4 * q);
            const float4 w4 = ld_shared_f4(rows + (c * 3 + 1) * T + 4 * q);
            const float4 br4 = ld_shared_f4(bc + (0 * NL + j) * TP + 4 * q);
            const float4 bi4 = ld_shared_f4(bc + (1 * NL + j) * TP + 4 * q);
            const float4 cr4 = ld_shared_f4(bc + (C::CROW * NL + j) * TP + 4 * q);
            const float4 ci4 = ld_shared_f4(bc + (3 * NL + j) * TP + 4 * q);

            const float sv[4] = AUSSM_F4(s4), wv[4] = AUSSM_F4(w4);
            const float brv[4] = AUSSM_F4(br4), biv[4] = AUSSM_F4(bi4);
            const float crv[4] = AUSSM_F4(cr4), civ[4] = AUSSM_F4(ci4);
            const float lr[4] = {lmr[4 * q], lmr[4 * q + 1], lmr[4 * q + 2], lmr[4 * q + 3]};
            const float li[4] = {lmi[REAL ? 0 : 4 * q], lmi[REAL ? 0 : 4 * q + 1], lmi[REAL ? 0 : 4 * q + 2],
                                 lmi[REAL ? 0 : 4 * q + 3]};
            const float prv[4] = {hpr[4 * q], hpr[4 * q + 1], hpr[4 * q + 2], hpr[4 * q + 3]};
            const float piv[4] = {hpi[REAL ? 0 : 4 * q], hpi[REAL ? 0 : 4 * q + 1], hpi[REAL ? 0 : 4 * q + 2],
                                  hpi[REAL ? 0 : 4 * q + 3]};
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
            // cells of a missing stream go back to zero (they are never copied again)
            st_shared_f4(st + lane * TP + 4 * q, has_rho ? make_float4(dr[0], dr[1], dr[2], dr[3])
                                                         : make_float4(0.f, 0.f, 0.f, 0.f));
            st_shared_f4(st + (32 + lane) * TP + 4 * q, has_theta ? make_float4(dth[0], dth[1], dth[2], dth[3])
                                                                  : make_float4(0.f, 0.f, 0.f, 0.f));
            st_shared_f4(et + lane * TP + 4 * q, make_float4(E[0], E[1], E[2], E[3]));
            st_shared_f4(pt + lane * TP + 4 * q, make_float4(P[0], P[1], P[2], P[3]));
#pragma unroll
            for (int off = NL; off < 32; off <<= 1) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    gBr[e] += __shfl_xor_sync(0xffffffffu, gBr[e], off);
                    gCr[e] += __shfl_xor_sync(0xffffffffu, gCr[e], off);
                }
                if (p.dB_im) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) gBi[e] += __shfl_xor_sync(0xffffffffu, gBi[e], off);
                }
                if (p.dC_im) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) gCi[e] += __shfl_xor_sync(0xffffffffu, gCi[e], off);
                }
            }
            if (c == 0 && j < N && nvalid > 0) {
                const long long o = bo + (long long)j * p.ld_row + t0 + 4 * q;
                red_add_v4c(p.dB_re + o, gBr);
                red_add_v4c(p.dC_re + o, gCr);
                if (p.dB_im) red_add_v4c(p.dB_im + o, gBi);
                if (p.dC_im) red_add_v4c(p.dC_im + o, gCi);
            }
        };
#pragma unroll
        for (int q = 0; q < NQ; ++q)
            if (q < nq) recompute(q);
#pragma unroll
        for (int q = NQ - 1; q >= 0; --q) {
            if (q < nq) {
                if (REAL) reverse_real(q);
                else reverse(q);
            }
        }
        // the gradient of the recorded state at this tile's start joins the carry
        if (grec) {
            const float2 g = grec[tile];
            er += g.x;
            ei += g.y;
        }
        __syncwarp();

        // post-pass: du, ddt, dz for one channel and VW steps per lane
#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (e0 < C::ELEMS && t < tlen && cc < nvalid) {
                Vec<VW> SE, SP, v, d, gz, g, w, gu, du, ddt, dz;
                SE.ld(et + cc * NL * TP + t);
                SP.ld(pt + cc * NL * TP + t);
#pragma unroll
                for (int rr = 1; rr < NL; ++rr) {
                    Vec<VW> a, bb;
                    a.ld(et + (cc * NL + rr) * TP + t);
                    bb.ld(pt + (cc * NL + rr) * TP + t);
                    SE.add(a);
                    SP.add(bb);
                }
                v.ld(aux + (cc * AUX + 0) * T + t);           // silu(u)
                d.ld(aux + (cc * AUX + 1) * T + t);
                gz.ld(aux + (cc * AUX + 2) * T + t);          // d silu(z)/dz
                g.ld(aux + (cc * AUX + 3) * T + t);
                w.ld(rows + (cc * 3 + 1) * T + t);            // gy silu(z)
                gu.ld(rows + (cc * 3 + 2) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    dz.v[e] = g.v[e] * fmaf(dval[it], v.v[e], SP.v[e]) * gz.v[e];
                    ddt.v[e] = SE.v[e] * v.v[e];
                    du.v[e] = fmaf(SE.v[e], d.v[e], w.v[e] * dval[it]) * gu.v[e];
                    dD_acc[it] = fmaf(w.v[e], v.v[e], dD_acc[it]);
                }
                const long long off = (ch0 + cc) * p.ld_row + t0 + t;
                du.st(p.du + off);
                ddt.st(p.ddt + off);
                dz.st(p.dz + off);
            }
        }
        // drho / dtheta leave the stage (each lane stores pieces of real rows only)
        {
            const int col = lane % NQ, r0 = lane / NQ;
            constexpr int RPI = 32 / NQ;
#pragma unroll
            for (int i = 0; i < C::NCH_OWN; ++i) {
                const int row = i * RPI + r0;
                const int w = row % 32;
                const int rc = w / NL, rj = w % NL;
                float* base = row < 32 ? p.drho : p.dtheta;
                const bool on = row < 32 ? has_rho : has_theta;
                if (on && base && rc < nvalid && rj < N && col * 4 < tlen)
                    *reinterpret_cast<float4*>(base + lam_b + ((long long)(i0 + rc) * N + rj) * p.ld_lam + t0 + col * 4) =
                        ld_shared_f4(st + row * TP + col * 4);
            }
        }
        block_sync<C>();                                    // nobody reads this stage's B / C tile any more
        const int nr = r + STAGES;
        if (nr < ntiles) {
            const int nt = ntiles - 1 - nr;
            map.issue(st, bc, (long long)nt * T, min(T, L - nt * T), lane, warp);
        } else {
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
    if (act && p.eta_out) reinterpret_cast<float2*>(p.eta_out)[ch * N + j] = make_float2(er, ei);

    __syncwarp();
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) et[lane + 32 * it] = dD_acc[it];
    __syncwarp();
    if (lane < nvalid) {
        float aD = 0.f;
        for (int idx = 0; idx < 32 * C::ITERS; ++idx)
            if (idx * VW < C::ELEMS && (idx * VW) / T == lane) aD += et[idx];
        p.part_D[ch0 + lane] = aD + (p.accumulate ? p.part_D[ch0 + lane] : 0.f);
    }
}

__global__ void __launch_bounds__(256) cplx_reduce_D_kernel(const float* part_D, float* dD, int batch, int D) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= D) return;
    float acc = 0.f;
    for (int b = 0; b < batch; ++b) acc += part_D[(long long)b * D + i];
    dD[i] = acc;
}

template <int NL, bool BWD, bool REAL, class Kern, class Params>
cudaError_t launch_nl(Kern kern, const Params& p, cudaStream_t stream) {
    using C = CCfg<NL, BWD, REAL>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long tasks = (p.Dmod + C::CPW - 1) / C::CPW;
    const long long blocks = (long long)(p.nch / p.Dmod) * ((tasks + C::WARPS - 1) / C::WARPS);
    kern<<<(unsigned)blocks, C::WARPS * 32, C::SMEM_BYTES, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_cplx_fwd(const CplxFwdParams& p, cudaStream_t stream) {
    if (p.nch <= 0 || p.L <= 0) return cudaSuccess;
    if (!p.theta && !p.B_im && !p.C_im) {          // everything real
        if (p.N <= 4) return launch_nl<4, false, true>(cplx_fwd_kernel<4, true>, p, stream);
        if (p.N <= 8) return launch_nl<8, false, true>(cplx_fwd_kernel<8, true>, p, stream);
        if (p.N <= 16) return launch_nl<16, false, true>(cplx_fwd_kernel<16, true>, p, stream);
        if (p.N <= 32) return launch_nl<32, false, true>(cplx_fwd_kernel<32, true>, p, stream);
        return cudaErrorInvalidValue;
    }
    if (p.N <= 4) return launch_nl<4, false, false>(cplx_fwd_kernel<4, false>, p, stream);
    if (p.N <= 8) return launch_nl<8, false, false>(cplx_fwd_kernel<8, false>, p, stream);
    if (p.N <= 16) return launch_nl<16, false, false>(cplx_fwd_kernel<16, false>, p, stream);
    if (p.N <= 32) return launch_nl<32, false, false>(cplx_fwd_kernel<32, false>, p, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_cplx_bwd(const CplxBwdParams& p, cudaStream_t stream) {
    if (p.nch <= 0 || p.L <= 0) return cudaSuccess;
    if (!p.theta && !p.B_im && !p.C_im && !p.dB_im && !p.dC_im) {
        if (p.N <= 4) return launch_nl<4, true, true>(cplx_bwd_kernel<4, true>, p, stream);
        if (p.N <= 8) return launch_nl<8, true, true>(cplx_bwd_kernel<8, true>, p, stream);
        if (p.N <= 16) return launch_nl<16, true, true>(cplx_bwd_kernel<16, true>, p, stream);
        if (p.N <= 32) return launch_nl<32, true, true>(cplx_bwd_kernel<32, true>, p, stream);
        return cudaErrorInvalidValue;
    }
    if (p.N <= 4) return launch_nl<4, true, false>(cplx_bwd_kernel<4, false>, p, stream);
    if (p.N <= 8) return launch_nl<8, true, false>(cplx_bwd_kernel<8, false>, p, stream);
    if (p.N <= 16) return launch_nl<16, true, false>(cplx_bwd_kernel<16, false>, p, stream);
    if (p.N <= 32) return launch_nl<32, true, false>(cplx_bwd_kernel<32, false>, p, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_cplx_reduce_D(const float* part_D, float* dD, int batch, int D, cudaStream_t stream) {
    cplx_reduce_D_kernel<<<(D + 255) / 256, 256, 0, stream>>>(part_D, dD, batch, D);
    count_launch();
    return cudaGetLastError();
}

}  // namespace aussm
