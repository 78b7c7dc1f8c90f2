// Unitary selective-scan core for sm_100a: forward and backward kernels.
//
// Operator (per channel ch = (b, i), state j, step t), theta given:
//     h_t = exp(i*theta_t) h_{t-1} + Bc_j s_t,   s_t = dt_t * silu(u_t)
//     y_t = silu(z_t) * (D_i silu(u_t) + sum_j Re(Cc_j h_t))
// It replaces the scan part of the reference kernels
// csrc/cuda/ssm_adaptive_unitary_forward.cu:112-187 and
// csrc/cuda/ssm_adaptive_unitary_backward.cu:143-417 (the phase projection,
// forward.cu:83-110 / backward.cu:419-490, is a separate contraction).
//
// Work decomposition.  One thread owns SPT states of one channel and walks
// the time axis sequentially, so the recurrence costs four fused
// multiply-adds per step and needs no scan tree.  A warp owns 32/NL channels
// (NL lanes per channel) and is independent of every other warp: it has its
// own ring of shared-memory stages and the kernels contain no block-wide
// barrier.  The theta rows of a warp (contiguous in time in HBM, one row per
// state) are staged with 16-byte asynchronous copies, consecutive lanes
// fetching consecutive pieces of a row (fully coalesced 128-bit loads), into
// rows padded by 16 bytes so that the per-thread 128-bit shared loads of a
// quarter-warp hit disjoint banks.  Sums over the states of a channel go
// through the same tile: every thread overwrites the four phases it has just
// consumed with its four contributions, and after the tile the lanes switch
// roles (one lane = one channel and a few consecutive steps) to add the NL
// rows and emit y with coalesced vector stores.
//
// Lanes whose state or channel does not exist (N < NL*SPT, or the last warp
// of the grid) shadow a valid row: they load and process real data with a
// zero output weight and store nothing, so the inner loops carry no
// predicates.
//
// State normalisation: with Bc != 0 the kernels carry h/Bc instead of h, so
// that the input term is the real number s_t (two multiply-adds less per
// step) and the output projection uses the single constant M = Cc*Bc.
//
// Backward: because |exp(i*theta)| = 1 the recurrence is reversible,
// h_{t-1} = exp(-i*theta_t)(h_t - Bc s_t); the kernel starts from the final
// state that the forward pass returned and walks time backwards, regenerating
// the states while it runs the adjoint recurrence
//     eta_t = conj(Cc) w_t + exp(-i*theta_{t+1}) eta_{t+1},   w_t = gy_t silu(z_t)
// so nothing but the inputs and the final state is ever stored.  dtheta is
// written in place of theta in the stage and leaves with coalesced stores.
#include "common.cuh"
#include "scan_unitary.cuh"

namespace aussm {

__device__ int g_device_status = 0;

int* device_status_ptr() {
    int* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_device_status) != cudaSuccess) return nullptr;
    return ptr;
}

cudaError_t read_and_clear_device_status(cudaStream_t stream, int* value) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    e = cudaMemcpyFromSymbol(value, g_device_status, sizeof(int));
    if (e != cudaSuccess) return e;
    if (*value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    }
    return e;
}

namespace {

constexpr int cmin(int a, int b) { return a < b ? a : b; }

// Shape of one warp's work.  NL lanes per channel, SPT states per thread,
// T steps per stage, TS steps per backward sub-block, AUX per-channel rows.
template <int NL_, int SPT_, int T_, int TS_, int STAGES_, int WARPS_, int AUX_, bool BWD_>
struct Cfg {
    static constexpr int NL = NL_, SPT = SPT_, T = T_, TS = TS_, STAGES = STAGES_, WARPS = WARPS_, AUX = AUX_;
    static constexpr int CPW = 32 / NL;                 // channels per warp
    static constexpr int TP = T + 4;                    // padded row pitch (floats)
    static constexpr int TSP = TS + 4;
    static constexpr int NROWS = 32 * SPT;
    static constexpr int STAGE_FLOATS = NROWS * TP + CPW * AUX * T;
    // backward only, not staged: two column-sum tiles and the s / w / silu'(u) rows of a sub-block
    static constexpr int SCRATCH_FLOATS = BWD_ ? 2 * 32 * TSP + CPW * 3 * TS : 0;
    static constexpr int WARP_FLOATS = STAGES * STAGE_FLOATS + SCRATCH_FLOATS;
    static constexpr size_t SMEM_BYTES = (size_t)WARPS * WARP_FLOATS * sizeof(float);
    // asynchronous-copy instructions per lane and tile
    static constexpr int CHUNKS_PER_ROW = T / 4;
    static constexpr int NCH_THETA = NROWS * CHUNKS_PER_ROW / 32;
    static constexpr int NCH_AUX = (CPW * AUX * CHUNKS_PER_ROW + 31) / 32;
    // per-(channel, step) passes: every lane owns VW consecutive steps of one channel
    static constexpr int EPL = CPW * TS / 32;           // elements per lane and sub-block
    static constexpr int VW = cmin(4, EPL);
    static constexpr int ITERS = EPL / VW;
    static_assert(T % TS == 0 && T % 4 == 0 && TS % 4 == 0, "tile shape");
    static_assert((NROWS * CHUNKS_PER_ROW) % 32 == 0, "theta chunks must fill whole warps");
    static_assert(CPW * TS >= 32 && (CPW * TS) % 32 == 0, "pass mapping");
};

template <int NL, int SPT, int T, int STAGES, int WARPS>
using FwdCfg = Cfg<NL, SPT, T, T, STAGES, WARPS, 3, false>;     // aux rows: u, dt (becomes s), z
template <int NL, int SPT, int T, int TS, int STAGES, int WARPS>
using BwdCfg = Cfg<NL, SPT, T, TS, STAGES, WARPS, 4, true>;     // aux rows: u, dt, z, gy

struct StateConsts {
    float mr, mi;      // M: projection constant (Cc*Bc normalised, Cc otherwise)
    float br, bi;      // Bc
    float kr, ki;      // state scale kappa (Bc normalised, 1 otherwise)
    float bias;        // phase offset
    bool act;
};

__device__ __forceinline__ void load_state_consts(StateConsts& sc, bool act, int j, int i, int N,
                                                  const float* B_r, const float* B_theta, const float* C_r,
                                                  const float* C_theta, const float* theta_bias, bool& norm_ok) {
    sc.act = act;
    sc.mr = sc.mi = sc.br = sc.bi = 0.f;
    sc.kr = 1.f;
    sc.ki = 0.f;
    sc.bias = 0.f;
    norm_ok = true;
    if (!act) return;
    float brad = B_r[j], bth = B_theta[j], crad = C_r[j], cth = C_theta[j];
    float sb, cb, scc, ccc;
    sincosf(bth, &sb, &cb);
    sincosf(cth, &scc, &ccc);
    sc.br = brad * cb;
    sc.bi = brad * sb;
    sc.mr = crad * ccc;   // Cc for now
    sc.mi = crad * scc;
    sc.bias = theta_bias ? theta_bias[(size_t)i * N + j] : 0.f;
    norm_ok = fabsf(brad) >= 1e-12f;
}

// switch the constants of an active state to the normalised representation
__device__ __forceinline__ void normalise_consts(StateConsts& sc, float& ccr, float& cci) {
    ccr = sc.mr;
    cci = sc.mi;
    if (!sc.act) return;
    sc.kr = sc.br;
    sc.ki = sc.bi;
    float mr = ccr * sc.br - cci * sc.bi;
    float mi = ccr * sc.bi + cci * sc.br;
    sc.mr = mr;
    sc.mi = mi;
}

// (ar + i ai) / (kr + i ki), scaled to stay in range for tiny |k|
__device__ __forceinline__ void cdiv(float ar, float ai, float kr, float ki, float& qr, float& qi) {
    float inv = rsqrtf(kr * kr + ki * ki);
    float ur = kr * inv, ui = ki * inv;     // unit vector of k
    float tr = ar * inv, ti = ai * inv;     // a / |k|
    qr = tr * ur + ti * ui;                 // times conj(unit)
    qi = ti * ur - tr * ui;
}

// Where the rows of a (virtual) channel start.  Without a time-axis split channel v owns rows v; with nseg
// segments virtual channel v = ch * nseg + s owns steps [s L, (s+1) L) of the rows of channel ch.
struct SegMap {
    int nseg, N;
    long long seg_len, ld_theta, ld_row;
    __device__ __forceinline__ long long chan(long long v) const { return nseg <= 1 ? v : v / nseg; }
    // offset (floats) of the per-channel rows (u, dt, z, y, ...)
    __device__ __forceinline__ long long row(long long v) const {
        return nseg <= 1 ? v * ld_row : (v / nseg) * ld_row + (v % nseg) * seg_len;
    }
    // offset (floats) of the theta row of state 0
    __device__ __forceinline__ long long theta(long long v) const {
        return nseg <= 1 ? v * N * ld_theta : (v / nseg) * N * ld_theta + (v % nseg) * seg_len;
    }
};
template <class P>
__device__ __forceinline__ SegMap seg_map(const P& p) {
    return SegMap{p.nseg, p.N, (long long)p.L, p.ld_theta, p.ld_row};
}

// ---------------------------------------------------------------------------
// Tile movement
// ---------------------------------------------------------------------------
// shared-memory slot of state j of warp-channel c
template <int NL>
__device__ __forceinline__ int slot_of(int c, int j) {
    return (j / NL) * 32 + c * NL + (j % NL);
}

// Where a warp's rows live in global memory, as seen by one lane: the source
// of every 16-byte piece this lane copies per tile (at step 0 of the launch).
template <class C>
struct TileMap {
    unsigned theta_off[C::NCH_THETA];     // byte offset from the warp's first theta row (32 bits: base + offset addressing)
    const float* aux_ptr[C::NCH_AUX];     // per-channel rows (nullptr: this lane has no piece)

    __device__ __forceinline__ void init(int lane, int nvalid, int N, const SegMap& sm, long long ch0,
                                         const float* const* aux_src) {
        const long long base0 = sm.theta(ch0);
#pragma unroll
        for (int i = 0; i < C::NCH_THETA; ++i) {
            const int id = i * 32 + lane;
            const int slot = id / C::CHUNKS_PER_ROW, col = id % C::CHUNKS_PER_ROW;
            const int k = slot / 32, w = slot % 32;
            const int c = w / C::NL, j = (w % C::NL) + k * C::NL;
            const bool ok = c < nvalid && j < N;
            // missing rows shadow the warp's first row
            const long long row = ok ? (sm.theta(ch0 + c) - base0) + (long long)j * sm.ld_theta : 0;
            theta_off[i] = (unsigned)((row + col * 4) * (long long)sizeof(float));
        }
#pragma unroll
        for (int i = 0; i < C::NCH_AUX; ++i) {
            const int id = i * 32 + lane;
            const int row = id / C::CHUNKS_PER_ROW, col = id % C::CHUNKS_PER_ROW;
            aux_ptr[i] = nullptr;
            if (row < C::CPW * C::AUX) {
                const int cc = row / C::AUX, a = row % C::AUX;
                const long long ch = ch0 + (cc < nvalid ? cc : 0);
                aux_ptr[i] = aux_src[a] + sm.row(ch) + col * 4;
            }
        }
    }

    // queue the asynchronous copies of one tile and close the group (FULL: a whole tile, no per-piece bound check).
    // Piece i of a lane lands at a compile-time distance from the lane's first piece, so every destination is
    // one register plus an immediate.
    template <bool FULL>
    __device__ __forceinline__ void issue_t(float* stage, const float* theta_t0, long long t0, int tlen,
                                            int lane) const {
        constexpr int CPR = C::CHUNKS_PER_ROW, RPI = 32 / CPR;       // rows covered by one warp-wide instruction
        static_assert(32 % CPR == 0, "pieces per row must divide the warp");
        const int col = lane % CPR;
        const uint32_t dst0 = smem_addr(stage) + (uint32_t)(((lane / CPR) * C::TP + col * 4) * sizeof(float));
#pragma unroll
        for (int i = 0; i < C::NCH_THETA; ++i) {
            if (FULL || col * 4 < tlen)
                cp_async16_s(dst0 + (uint32_t)(i * RPI * C::TP * sizeof(float)),
                             reinterpret_cast<const char*>(theta_t0) + theta_off[i]);
        }
        const uint32_t aux0 = smem_addr(stage) +
                              (uint32_t)((C::NROWS * C::TP + (lane / CPR) * C::T + col * 4) * sizeof(float));
#pragma unroll
        for (int i = 0; i < C::NCH_AUX; ++i) {
            if (aux_ptr[i] != nullptr && (FULL || col * 4 < tlen))
                cp_async16_s(aux0 + (uint32_t)(i * RPI * C::T * sizeof(float)), aux_ptr[i] + t0);
        }
        cp_async_commit();
    }
    __device__ __forceinline__ void issue(float* stage, const float* theta_warp, long long t0, int tlen,
                                          int lane) const {
        if (tlen == C::T) issue_t<true>(stage, theta_warp + t0, t0, tlen, lane);
        else issue_t<false>(stage, theta_warp + t0, t0, tlen, lane);
    }
};

// Plain tile load for launches whose rows are not 16-byte aligned: coalesced
// along time, zero-filled up to a quad, missing rows shadow row 0.
template <class C>
__device__ __forceinline__ void plain_load_tile(float* stage, const float* theta_warp, long long ld_theta,
                                                const float* const* aux_src, long long ld_row, long long ch0,
                                                int nvalid, int N, long long t0, int tlen, int lane) {
    float* aux = stage + C::NROWS * C::TP;
    const int tq = (tlen + 3) & ~3;
    for (int slot = 0; slot < C::NROWS; ++slot) {
        const int k = slot / 32, w = slot % 32;
        const int c = w / C::NL, j = (w % C::NL) + k * C::NL;
        const long long row = (c < nvalid && j < N) ? (long long)c * N + j : 0;
        const float* src = theta_warp + row * ld_theta + t0;
        float* dst = stage + slot * C::TP;
        for (int t = lane; t < tq; t += 32) dst[t] = t < tlen ? src[t] : 0.f;
    }
    for (int row = 0; row < C::CPW * C::AUX; ++row) {
        const int cc = row / C::AUX, a = row % C::AUX;
        const float* src = aux_src[a] + (ch0 + (cc < nvalid ? cc : 0)) * ld_row + t0;
        float* dst = aux + row * C::T;
        for (int t = lane; t < tq; t += 32) dst[t] = t < tlen ? src[t] : 0.f;
    }
    __syncwarp();
}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
// AGG: aggregate mode of the time-axis split - no output row; besides the state, the product of the segment's
// rotations is carried (as a unit complex number, like the state itself) and returned.
template <class C, bool ASYNC, bool NORM, bool BIAS, bool AGG>
__device__ __forceinline__ void fwd_warp(const ScanFwdParams& p, float* wsm, long long ch0, int nvalid, int lane,
                                         StateConsts (&sc)[C::SPT]) {
    constexpr int NL = C::NL, SPT = C::SPT, T = C::T, TP = C::TP, STAGES = C::STAGES, AUX = C::AUX, VW = C::VW;
    const int c = lane / NL, jl = lane % NL;
    const long long ch = ch0 + c;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;
    const SegMap sm = seg_map(p);
    const float* theta_warp = p.theta + sm.theta(ch0);
    const float* aux_src[AUX] = {p.u, p.dt, p.z};
    float ar[SPT], ai[SPT];     // product of the rotations so far (aggregate mode)
#pragma unroll
    for (int k = 0; k < SPT; ++k) { ar[k] = 1.f; ai[k] = 0.f; }

    float hr[SPT], hi[SPT];
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        const int j = jl + k * NL;
        hr[k] = hi[k] = 0.f;
        if (sc[k].act) {
            float ar = p.h0_re ? p.h0_re[ch * N + j] : 0.f;
            float ai = p.h0_im ? p.h0_im[ch * N + j] : 0.f;
            if (NORM) cdiv(ar, ai, sc[k].kr, sc[k].ki, hr[k], hi[k]);
            else { hr[k] = ar; hi[k] = ai; }
        }
    }
    // skip weight and output row of the channel each per-(channel, step) item of this lane belongs to
    float dval[C::ITERS];
    long long ybase[C::ITERS];
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int cc = ((lane + 32 * it) * VW) / T;
        dval[it] = cc < nvalid ? p.Dskip[sm.chan(ch0 + cc) % p.Dmod] : 0.f;
        ybase[it] = sm.row(ch0 + (cc < nvalid ? cc : 0));
    }

    TileMap<C> map;
    if (ASYNC) {
        map.init(lane, nvalid, N, sm, ch0, aux_src);
        for (int s = 0; s < STAGES; ++s) {
            if (s < ntiles)
                map.issue(wsm + s * C::STAGE_FLOATS, theta_warp, (long long)s * T, min(T, L - s * T), lane);
            else
                cp_async_commit();
        }
    }

    for (int tile = 0; tile < ntiles; ++tile) {
        const int stage = ASYNC ? tile % STAGES : 0;
        float* th = wsm + stage * C::STAGE_FLOATS;
        float* aux = th + C::NROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        const int nq = (tlen + 3) >> 2;
        if (ASYNC) {
            cp_async_wait<STAGES - 1>();
            __syncwarp();
        } else {
            plain_load_tile<C>(th, theta_warp, p.ld_theta, aux_src, p.ld_row, ch0, nvalid, N, t0, tlen, lane);
        }

        // pre-pass: v = silu(u) over the u row, s = dt * v over the dt row
#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (t < tlen) {
                Vec<VW> u, d;
                u.ld(aux + (cc * AUX + 0) * T + t);
                d.ld(aux + (cc * AUX + 1) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) {
                    u.v[e] = siluf_(u.v[e]);
                    d.v[e] *= u.v[e];
                }
                u.st(aux + (cc * AUX + 0) * T + t);      // the u row now holds silu(u) for the post-pass
                d.st(aux + (cc * AUX + 1) * T + t);
            }
        }
        __syncwarp();

        // scan: SPT states per thread, four steps per shared-memory access
        const float* srow = aux + (c * AUX + 1) * T;
        auto quad = [&](const int q) {
            const float4 s4 = ld_shared_f4(srow + 4 * q);
            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
            float pacc[4];
#pragma unroll
            for (int k = 0; k < SPT; ++k) {
                const float4 t4 = ld_shared_f4(th + (k * 32 + lane) * TP + 4 * q);
                float tv[4] = {t4.x, t4.y, t4.z, t4.w};
                if (BIAS) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) tv[e] += sc[k].bias;
                }
                float sn[4], cs[4];
                sincos4(tv, sn, cs);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (!ASYNC && 4 * q + e >= tlen) {           // ragged tail (plain path only)
                        if (k == 0) pacc[e] = 0.f;
                        continue;
                    }
                    float nr, ni;
                    if (NORM) {
                        nr = fmaf(cs[e], hr[k], fmaf(-sn[e], hi[k], sv[e]));
                        ni = fmaf(cs[e], hi[k], sn[e] * hr[k]);
                    } else {
                        nr = fmaf(cs[e], hr[k], fmaf(-sn[e], hi[k], sc[k].br * sv[e]));
                        ni = fmaf(cs[e], hi[k], fmaf(sn[e], hr[k], sc[k].bi * sv[e]));
                    }
                    hr[k] = nr;
                    hi[k] = ni;
                    if (AGG) {
                        const float qr = fmaf(cs[e], ar[k], -sn[e] * ai[k]);
                        ai[k] = fmaf(cs[e], ai[k], sn[e] * ar[k]);
                        ar[k] = qr;
                    } else {
                        pacc[e] = (k == 0) ? fmaf(sc[k].mr, nr, -sc[k].mi * ni)
                                           : fmaf(sc[k].mr, nr, fmaf(-sc[k].mi, ni, pacc[e]));
                    }
                }
            }
            if (!AGG) st_shared_f4(th + lane * TP + 4 * q, make_float4(pacc[0], pacc[1], pacc[2], pacc[3]));
        };
        if (ASYNC && tlen == T) {
#pragma unroll
            for (int q = 0; q < T / 4; ++q) quad(q);
        } else {
            for (int q = 0; q < nq; ++q) quad(q);
        }
        __syncwarp();

        // post-pass: one lane = one channel and VW steps
        if (!AGG && p.y) {
#pragma unroll
            for (int it = 0; it < C::ITERS; ++it) {
                const int e0 = (lane + 32 * it) * VW;
                const int cc = e0 / T, t = e0 % T;
                if (t < tlen && cc < nvalid) {
                    Vec<VW> acc, u, z;
                    acc.ld(th + cc * NL * TP + t);
#pragma unroll
                    for (int r = 1; r < NL; ++r) {
                        Vec<VW> v;
                        v.ld(th + (cc * NL + r) * TP + t);
                        acc.add(v);
                    }
                    u.ld(aux + (cc * AUX + 0) * T + t);      // silu(u), left by the pre-pass
                    z.ld(aux + (cc * AUX + 2) * T + t);
#pragma unroll
                    for (int e = 0; e < VW; ++e) acc.v[e] = siluf_(z.v[e]) * fmaf(dval[it], u.v[e], acc.v[e]);
                    float* dst = p.y + ybase[it] + t0 + t;
                    if (ASYNC) {
                        acc.st(dst);      // global pointers take the same vector stores
                    } else {
                        for (int e = 0; e < VW; ++e)
                            if (t + e < tlen) dst[e] = acc.v[e];
                    }
                }
            }
        }
        __syncwarp();
        if (ASYNC) {
            const int nt = tile + STAGES;
            if (nt < ntiles) map.issue(th, theta_warp, (long long)nt * T, min(T, L - nt * T), lane);
            else cp_async_commit();
        }
    }
    if (ASYNC) cp_async_wait<0>();

#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        if (sc[k].act && p.h1_re) {
            const int j = jl + k * NL;
            float orr = hr[k], oi = hi[k];
            if (NORM) {
                orr = sc[k].kr * hr[k] - sc[k].ki * hi[k];
                oi = sc[k].kr * hi[k] + sc[k].ki * hr[k];
            }
            p.h1_re[ch * N + j] = orr;
            p.h1_im[ch * N + j] = oi;
        }
        if (AGG && sc[k].act && p.agg_re) {
            const int j = jl + k * NL;
            p.agg_re[ch * N + j] = ar[k];
            p.agg_im[ch * N + j] = ai[k];
        }
    }
}

template <class C, bool ASYNC, bool BIAS, bool AGG>
__global__ void __launch_bounds__(C::WARPS * 32) scan_unitary_fwd_kernel(const ScanFwdParams p) {
    extern __shared__ __align__(128) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long ch0 = ((long long)blockIdx.x * C::WARPS + warp) * C::CPW;
    if (ch0 >= p.nch) return;   // warps never meet at a block barrier
    const int nvalid = (int)min((long long)C::CPW, (long long)p.nch - ch0);
    float* wsm = smem + (size_t)warp * C::WARP_FLOATS;
    const int c = lane / C::NL, jl = lane % C::NL;
    const int i = (int)(seg_map(p).chan(ch0 + min(c, nvalid - 1)) % p.Dmod);
    StateConsts sc[C::SPT];
    bool ok = true;
#pragma unroll
    for (int k = 0; k < C::SPT; ++k) {
        const int j = jl + k * C::NL;
        bool okk;
        load_state_consts(sc[k], c < nvalid && j < p.N, j, i, p.N, p.B_r, p.B_theta, p.C_r, p.C_theta,
                          BIAS ? p.theta_bias : nullptr, okk);
        ok = ok && okk;
    }
    if (__all_sync(0xffffffffu, ok)) {
#pragma unroll
        for (int k = 0; k < C::SPT; ++k) {
            float a, b;
            normalise_consts(sc[k], a, b);
        }
        fwd_warp<C, ASYNC, true, BIAS, AGG>(p, wsm, ch0, nvalid, lane, sc);
    } else {
        fwd_warp<C, ASYNC, false, BIAS, AGG>(p, wsm, ch0, nvalid, lane, sc);
    }
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------
template <class C, bool ASYNC, bool NORM, bool BIAS>
__device__ __forceinline__ void bwd_warp(const ScanBwdParams& p, float* wsm, long long ch0, int nvalid, int lane,
                                         StateConsts (&sc)[C::SPT], const float (&ccr)[C::SPT],
                                         const float (&cci)[C::SPT]) {
    constexpr int NL = C::NL, SPT = C::SPT, T = C::T, TS = C::TS, TP = C::TP, TSP = C::TSP, STAGES = C::STAGES,
                  AUX = C::AUX, VW = C::VW;
    const int c = lane / NL, jl = lane % NL;
    const long long ch = ch0 + c;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;
    const SegMap sm = seg_map(p);
    const float* theta_warp = p.theta + sm.theta(ch0);
    float* dtheta_warp = p.dtheta + sm.theta(ch0);              // launcher guarantees equal pitches

    float* scratch = wsm + STAGES * C::STAGE_FLOATS;
    float* pt = scratch;                    // [32][TSP] projections, summed over a thread's states
    float* et = pt + 32 * TSP;              // [32][TSP] Re(eta)
    float* sw = et + 32 * TSP;              // [CPW][3][TS]: s row, w row, d silu(u)/du row

    float hr[SPT], hi[SPT];     // state h_t (normalised), walking backwards
    float er[SPT], ei[SPT];     // exp(-i theta_{t+1}) eta_{t+1}
    float gmr[SPT], gmi[SPT];   // sum_t w_t conj(h_t)
    float sbr[SPT], sbi[SPT];   // sum_t eta_t s_t              (general representation only)
    float amax = 0.f;           // max |dtheta| seen by this thread (drop-in pipeline: spares the GEMM's own pass)
    float rsum[SPT];            // sum_t dtheta_t
    float hlr[SPT], hli[SPT];   // conj(h_{L-1}) . gh   (boundary term of the Bc gradient)
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        const int j = jl + k * NL;
        hr[k] = hi[k] = er[k] = ei[k] = gmr[k] = gmi[k] = sbr[k] = sbi[k] = rsum[k] = hlr[k] = hli[k] = 0.f;
        if (sc[k].act) {
            const float ar = p.h1_re[ch * N + j], ai = p.h1_im[ch * N + j];
            const float gr = p.gh1_re ? p.gh1_re[ch * N + j] : 0.f;
            const float gi = p.gh1_im ? p.gh1_im[ch * N + j] : 0.f;
            if (NORM) {
                cdiv(ar, ai, sc[k].kr, sc[k].ki, hr[k], hi[k]);
                // gradient w.r.t. the normalised state: conj(kappa) * gh
                er[k] = sc[k].kr * gr + sc[k].ki * gi;
                ei[k] = sc[k].kr * gi - sc[k].ki * gr;
                // conj(h~_{L-1}) * gh
                hlr[k] = hr[k] * gr + hi[k] * gi;
                hli[k] = hr[k] * gi - hi[k] * gr;
            } else {
                hr[k] = ar; hi[k] = ai; er[k] = gr; ei[k] = gi;
            }
        }
    }
    float dval[C::ITERS], dacc[C::ITERS];
    long long obase[C::ITERS];
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int cc = ((lane + 32 * it) * VW) / TS;
        dval[it] = cc < nvalid ? p.Dskip[sm.chan(ch0 + cc) % p.Dmod] : 0.f;
        dacc[it] = 0.f;
        obase[it] = sm.row(ch0 + (cc < nvalid ? cc : 0));
    }
    const float* aux_src[AUX] = {p.u, p.dt, p.z, p.gy};

    // r counts tiles in processing order (last tile first)
    TileMap<C> map;
    if (ASYNC) {
        map.init(lane, nvalid, N, sm, ch0, aux_src);
        for (int r = 0; r < STAGES; ++r) {
            const int tile = ntiles - 1 - r;
            if (tile >= 0)
                map.issue(wsm + r * C::STAGE_FLOATS, theta_warp, (long long)tile * T, min(T, L - tile * T), lane);
            else
                cp_async_commit();
        }
    }

    for (int r = 0; r < ntiles; ++r) {
        const int tile = ntiles - 1 - r;
        const int stage = ASYNC ? r % STAGES : 0;
        float* th = wsm + stage * C::STAGE_FLOATS;
        float* aux = th + C::NROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        if (ASYNC) {
            cp_async_wait<STAGES - 1>();
            __syncwarp();
        } else {
            plain_load_tile<C>(th, theta_warp, p.ld_theta, aux_src, p.ld_row, ch0, nvalid, N, t0, tlen, lane);
        }

        const int nsb = (tlen + TS - 1) / TS;
        for (int sb = nsb - 1; sb >= 0; --sb) {
            const int sbeg = sb * TS;                       // first step of the sub-block in the tile
            const int slen = min(TS, tlen - sbeg);
            const int nq = (slen + 3) >> 2;

            // pre-pass: every activation of the sub-block once.  s = dt silu(u), w = gy silu(z) feed the scan;
            // silu(u) and d silu(z)/dz replace the u and z rows, d silu(u)/du gets a row of its own.
#pragma unroll
            for (int it = 0; it < C::ITERS; ++it) {
                const int e0 = (lane + 32 * it) * VW;
                const int cc = e0 / TS, t = e0 % TS;
                if (t < slen) {
                    const int o = sbeg + t;
                    Vec<VW> u, d, z, g, gu;
                    u.ld(aux + (cc * AUX + 0) * T + o);
                    d.ld(aux + (cc * AUX + 1) * T + o);
                    z.ld(aux + (cc * AUX + 2) * T + o);
                    g.ld(aux + (cc * AUX + 3) * T + o);
#pragma unroll
                    for (int e = 0; e < VW; ++e) {
                        float gz;
                        u.v[e] = silu_and_grad(u.v[e], gu.v[e]);
                        d.v[e] *= u.v[e];
                        g.v[e] *= silu_and_grad(z.v[e], gz);
                        z.v[e] = gz;
                    }
                    u.st(aux + (cc * AUX + 0) * T + o);
                    z.st(aux + (cc * AUX + 2) * T + o);
                    d.st(sw + (cc * 3 + 0) * TS + t);
                    g.st(sw + (cc * 3 + 1) * TS + t);
                    gu.st(sw + (cc * 3 + 2) * TS + t);
                }
            }
            __syncwarp();

            // reverse scan
            auto quad = [&](const int q) {
                const float4 s4 = ld_shared_f4(sw + (c * 3 + 0) * TS + 4 * q);
                const float4 w4 = ld_shared_f4(sw + (c * 3 + 1) * TS + 4 * q);
                const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
                const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
                float pacc[4], eacc[4];
#pragma unroll
                for (int k = 0; k < SPT; ++k) {
                    float* cell = th + (k * 32 + lane) * TP + sbeg + 4 * q;
                    const float4 t4 = ld_shared_f4(cell);
                    float tv[4] = {t4.x, t4.y, t4.z, t4.w};
                    if (BIAS) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) tv[e] += sc[k].bias;
                    }
                    float sn[4], cs[4];
                    sincos4(tv, sn, cs);
                    float dth[4];
#pragma unroll
                    for (int e = 3; e >= 0; --e) {
                        if (!ASYNC && 4 * q + e >= slen) {
                            dth[e] = 0.f;
                            if (k == 0) { pacc[e] = 0.f; eacc[e] = 0.f; }
                            continue;
                        }
                        const float w = wv[e], s = sv[e];
                        // eta_t = carry + conj(M) w
                        const float nr = fmaf(sc[k].mr, w, er[k]);
                        const float ni = fmaf(-sc[k].mi, w, ei[k]);
                        // a = h_t - beta s  (= exp(i theta_t) h_{t-1})
                        float ar, ai;
                        if (NORM) { ar = hr[k] - s; ai = hi[k]; }
                        else { ar = fmaf(-sc[k].br, s, hr[k]); ai = fmaf(-sc[k].bi, s, hi[k]); }
                        // dtheta_t = -Im(conj(eta) a)
                        const float d = fmaf(ni, ar, -nr * ai);
                        dth[e] = d;
                        if (BIAS) { rsum[k] += d; amax = fmaxf(amax, fabsf(d)); }
                        const float pv = fmaf(sc[k].mr, hr[k], -sc[k].mi * hi[k]);
                        // gradient of the real drive s_t: Re(conj(eta) beta)
                        const float ev = NORM ? nr : fmaf(nr, sc[k].br, ni * sc[k].bi);
                        pacc[e] = (k == 0) ? pv : pacc[e] + pv;
                        eacc[e] = (k == 0) ? ev : eacc[e] + ev;
                        gmr[k] = fmaf(w, hr[k], gmr[k]);
                        gmi[k] = fmaf(-w, hi[k], gmi[k]);
                        if (!NORM) { sbr[k] = fmaf(nr, s, sbr[k]); sbi[k] = fmaf(ni, s, sbi[k]); }
                        // step back: h_{t-1} = conj(lambda) a ; carry = conj(lambda) eta
                        hr[k] = fmaf(cs[e], ar, sn[e] * ai);
                        hi[k] = fmaf(cs[e], ai, -sn[e] * ar);
                        er[k] = fmaf(cs[e], nr, sn[e] * ni);
                        ei[k] = fmaf(cs[e], ni, -sn[e] * nr);
                    }
                    st_shared_f4(cell, make_float4(dth[0], dth[1], dth[2], dth[3]));
                }
                st_shared_f4(pt + lane * TSP + 4 * q, make_float4(pacc[0], pacc[1], pacc[2], pacc[3]));
                st_shared_f4(et + lane * TSP + 4 * q, make_float4(eacc[0], eacc[1], eacc[2], eacc[3]));
            };
            if (ASYNC && slen == TS) {
#pragma unroll
                for (int q = TS / 4 - 1; q >= 0; --q) quad(q);
            } else {
                for (int q = nq - 1; q >= 0; --q) quad(q);
            }
            __syncwarp();

            // post-pass: du, ddt, dz for one channel and VW steps per lane
#pragma unroll
            for (int it = 0; it < C::ITERS; ++it) {
                const int e0 = (lane + 32 * it) * VW;
                const int cc = e0 / TS, t = e0 % TS;
                if (t < slen && cc < nvalid) {
                    Vec<VW> P, E, v, d, gz, g, w, gu, du, ddt, dz;
                    P.ld(pt + cc * NL * TSP + t);
                    E.ld(et + cc * NL * TSP + t);
#pragma unroll
                    for (int rr = 1; rr < NL; ++rr) {
                        Vec<VW> a, b;
                        a.ld(pt + (cc * NL + rr) * TSP + t);
                        b.ld(et + (cc * NL + rr) * TSP + t);
                        P.add(a);
                        E.add(b);
                    }
                    const int o = sbeg + t;
                    v.ld(aux + (cc * AUX + 0) * T + o);       // silu(u)
                    d.ld(aux + (cc * AUX + 1) * T + o);
                    gz.ld(aux + (cc * AUX + 2) * T + o);      // d silu(z)/dz
                    g.ld(aux + (cc * AUX + 3) * T + o);
                    w.ld(sw + (cc * 3 + 1) * TS + t);         // gy silu(z)
                    gu.ld(sw + (cc * 3 + 2) * TS + t);
                    const float dv = dval[it];
#pragma unroll
                    for (int e = 0; e < VW; ++e) {
                        dz.v[e] = g.v[e] * fmaf(dv, v.v[e], P.v[e]) * gz.v[e];
                        ddt.v[e] = E.v[e] * v.v[e];
                        du.v[e] = fmaf(E.v[e], d.v[e], w.v[e] * dv) * gu.v[e];
                        if (ASYNC || t + e < slen) dacc[it] = fmaf(w.v[e], v.v[e], dacc[it]);
                    }
                    const long long off = obase[it] + t0 + o;
                    if (ASYNC) {
                        du.st(p.du + off);
                        ddt.st(p.ddt + off);
                        dz.st(p.dz + off);
                    } else {
                        for (int e = 0; e < VW; ++e) {
                            if (t + e < slen) {
                                p.du[off + e] = du.v[e];
                                p.ddt[off + e] = ddt.v[e];
                                p.dz[off + e] = dz.v[e];
                            }
                        }
                    }
                }
            }
            __syncwarp();
        }

        // dtheta leaves the stage: coalesced 16-byte stores, same piece-to-lane map as the loads
        if (ASYNC) {
            constexpr int CPR = C::CHUNKS_PER_ROW, RPI = 32 / CPR;
            const int col = lane % CPR;
            const float* src0 = th + (lane / CPR) * TP + col * 4;
            float* dst0 = dtheta_warp + t0;
            if (nvalid == C::CPW && N == NL * SPT && tlen == T) {      // whole tile, every row real: no per-piece test
#pragma unroll
                for (int i = 0; i < C::NCH_THETA; ++i)
                    *reinterpret_cast<float4*>(reinterpret_cast<char*>(dst0) + map.theta_off[i]) =
                            ld_shared_f4(src0 + i * RPI * TP);
            } else {
#pragma unroll
                for (int i = 0; i < C::NCH_THETA; ++i) {
                    const int slot = i * RPI + lane / CPR;
                    const int k = slot / 32, w = slot % 32;
                    const bool real_row = (w / NL) < nvalid && ((w % NL) + k * NL) < N;
                    if (real_row && col * 4 < tlen)
                        *reinterpret_cast<float4*>(reinterpret_cast<char*>(dst0) + map.theta_off[i]) =
                            ld_shared_f4(src0 + i * RPI * TP);
                }
            }
            __syncwarp();
            const int nr = r + STAGES;
            if (nr < ntiles) {
                const int nt = ntiles - 1 - nr;
                map.issue(th, theta_warp, (long long)nt * T, min(T, L - nt * T), lane);
            } else {
                cp_async_commit();
            }
        } else {
            for (int cc = 0; cc < nvalid; ++cc)
                for (int j = 0; j < N; ++j) {
                    float* dst = dtheta_warp + ((long long)cc * N + j) * p.ld_theta + t0;
                    const float* src = th + slot_of<NL>(cc, j) * TP;
                    for (int t = lane; t < tlen; t += 32) dst[t] = src[t];
                }
            __syncwarp();
        }
    }
    if (ASYNC) cp_async_wait<0>();

    // ---- per-(channel, state) results ----
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        if (!sc[k].act) continue;
        const int j = jl + k * NL;
        const long long o = ch * N + j;
        float dbr, dbi, dcr, dci, d0r, d0i, s0r, s0i;
        if (NORM) {
            const float kr = sc[k].kr, ki = sc[k].ki;
            // dCc = conj(Bc) G_M
            dcr = kr * gmr[k] + ki * gmi[k];
            dci = kr * gmi[k] - ki * gmr[k];
            // dBc = conj(Cc) G_M + conj(h~_{L-1}) gh - conj(h~_{-1} / Bc) carry
            float qr, qi;
            cdiv(hr[k], hi[k], kr, ki, qr, qi);
            dbr = ccr[k] * gmr[k] + cci[k] * gmi[k] + hlr[k] - (qr * er[k] + qi * ei[k]);
            dbi = ccr[k] * gmi[k] - cci[k] * gmr[k] + hli[k] - (qr * ei[k] - qi * er[k]);
            // dh0 = carry / conj(Bc) ;  h0 = Bc h~_{-1}
            cdiv(er[k], ei[k], kr, -ki, d0r, d0i);
            s0r = kr * hr[k] - ki * hi[k];
            s0i = kr * hi[k] + ki * hr[k];
        } else {
            dcr = gmr[k]; dci = gmi[k]; dbr = sbr[k]; dbi = sbi[k];
            d0r = er[k]; d0i = ei[k]; s0r = hr[k]; s0i = hi[k];
        }
        float4* pb = reinterpret_cast<float4*>(p.part_bc) + o;
        if (p.accumulate) {
            const float4 old = *pb;
            dbr += old.x; dbi += old.y; dcr += old.z; dci += old.w;
        }
        *pb = make_float4(dbr, dbi, dcr, dci);
        if (BIAS && p.part_rowsum) p.part_rowsum[o] = rsum[k] + (p.accumulate ? p.part_rowsum[o] : 0.f);
        if (p.dh0_re) { p.dh0_re[o] = d0r; p.dh0_im[o] = d0i; }
        if (p.h0_re) { p.h0_re[o] = s0r; p.h0_im[o] = s0i; }
    }
    if (BIAS && p.dtheta_amax) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0 && amax > 0.f) atomicMax(p.dtheta_amax, __float_as_uint(fminf(amax, 3.0e38f)));
    }
    // dD: add the lanes' partial sums channel by channel through the scratch tile
    __syncwarp();
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) pt[lane + 32 * it] = dacc[it];
    __syncwarp();
    if (lane < nvalid) {
        // item idx covers elements [idx*VW, idx*VW+VW) of the CPW*TS block: channel = idx*VW/TS
        float acc = 0.f;
        for (int idx = 0; idx < 32 * C::ITERS; ++idx)
            if ((idx * VW) / TS == lane) acc += pt[idx];
        const long long o = ch0 + lane;
        p.part_d[o] = acc + (p.accumulate ? p.part_d[o] : 0.f);
    }
}

template <class C, bool ASYNC, bool BIAS>
__global__ void __launch_bounds__(C::WARPS * 32) scan_unitary_bwd_kernel(const ScanBwdParams p) {
    extern __shared__ __align__(128) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long ch0 = ((long long)blockIdx.x * C::WARPS + warp) * C::CPW;
    if (ch0 >= p.nch) return;
    const int nvalid = (int)min((long long)C::CPW, (long long)p.nch - ch0);
    float* wsm = smem + (size_t)warp * C::WARP_FLOATS;
    const int c = lane / C::NL, jl = lane % C::NL;
    const int i = (int)(seg_map(p).chan(ch0 + min(c, nvalid - 1)) % p.Dmod);
    StateConsts sc[C::SPT];
    float ccr[C::SPT], cci[C::SPT];
    bool ok = true;
#pragma unroll
    for (int k = 0; k < C::SPT; ++k) {
        const int j = jl + k * C::NL;
        bool okk;
        load_state_consts(sc[k], c < nvalid && j < p.N, j, i, p.N, p.B_r, p.B_theta, p.C_r, p.C_theta,
                          BIAS ? p.theta_bias : nullptr, okk);
        ccr[k] = sc[k].mr;
        cci[k] = sc[k].mi;
        ok = ok && okk;
    }
    if (__all_sync(0xffffffffu, ok)) {
#pragma unroll
        for (int k = 0; k < C::SPT; ++k) normalise_consts(sc[k], ccr[k], cci[k]);
        bwd_warp<C, ASYNC, true, BIAS>(p, wsm, ch0, nvalid, lane, sc, ccr, cci);
    } else {
        bwd_warp<C, ASYNC, false, BIAS>(p, wsm, ch0, nvalid, lane, sc, ccr, cci);
    }
}

// ---------------------------------------------------------------------------
// Adjoint-only reverse pass (time-axis split): for every (virtual) channel the gradient that the segment's own
// grad_y sends to the state before the segment, from a zero gradient after it:
//     e <- conj(lambda_t) (e + conj(Cc) w_t),  t = L-1 .. 0,   w_t = gy_t silu(z_t)
// (general representation, no state regeneration, nothing else produced).
// ---------------------------------------------------------------------------
template <class C, bool BIAS>
__global__ void __launch_bounds__(C::WARPS * 32) scan_unitary_eta_kernel(const ScanBwdParams p) {
    constexpr int NL = C::NL, SPT = C::SPT, T = C::T, TP = C::TP, STAGES = C::STAGES, AUX = C::AUX, VW = C::VW;
    extern __shared__ __align__(128) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long ch0 = ((long long)blockIdx.x * C::WARPS + warp) * C::CPW;
    if (ch0 >= p.nch) return;
    const int nvalid = (int)min((long long)C::CPW, (long long)p.nch - ch0);
    float* wsm = smem + (size_t)warp * C::WARP_FLOATS;
    const int c = lane / NL, jl = lane % NL;
    const SegMap sm = seg_map(p);
    const int i = (int)(sm.chan(ch0 + min(c, nvalid - 1)) % p.Dmod);
    const long long ch = ch0 + c;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;
    StateConsts sc[SPT];
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        bool okk;
        load_state_consts(sc[k], c < nvalid && jl + k * NL < N, jl + k * NL, i, N, p.B_r, p.B_theta, p.C_r, p.C_theta,
                          BIAS ? p.theta_bias : nullptr, okk);      // mr, mi hold Cc
    }
    const float* theta_warp = p.theta + sm.theta(ch0);
    const float* aux_src[AUX] = {p.u, p.dt, p.z, p.gy};
    float er[SPT], ei[SPT];
#pragma unroll
    for (int k = 0; k < SPT; ++k) er[k] = ei[k] = 0.f;
    TileMap<C> map;
    map.init(lane, nvalid, N, sm, ch0, aux_src);
    for (int r = 0; r < STAGES; ++r) {
        const int tile = ntiles - 1 - r;
        if (tile >= 0) map.issue(wsm + r * C::STAGE_FLOATS, theta_warp, (long long)tile * T, min(T, L - tile * T), lane);
        else cp_async_commit();
    }
    for (int r = 0; r < ntiles; ++r) {
        const int tile = ntiles - 1 - r;
        float* th = wsm + (r % STAGES) * C::STAGE_FLOATS;
        float* aux = th + C::NROWS * TP;
        const int tlen = min(T, L - tile * T);
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        // pre-pass: w = gy silu(z) replaces gy
#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int e0 = (lane + 32 * it) * VW;
            const int cc = e0 / T, t = e0 % T;
            if (t < tlen) {
                Vec<VW> z, g;
                z.ld(aux + (cc * AUX + 2) * T + t);
                g.ld(aux + (cc * AUX + 3) * T + t);
#pragma unroll
                for (int e = 0; e < VW; ++e) g.v[e] *= siluf_(z.v[e]);
                g.st(aux + (cc * AUX + 3) * T + t);
            }
        }
        __syncwarp();
        const float* wrow = aux + (c * AUX + 3) * T;
        for (int q = (tlen >> 2) - 1; q >= 0; --q) {
            const float4 w4 = ld_shared_f4(wrow + 4 * q);
            const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int k = 0; k < SPT; ++k) {
                const float4 t4 = ld_shared_f4(th + (k * 32 + lane) * TP + 4 * q);
                float tv[4] = {t4.x, t4.y, t4.z, t4.w};
                if (BIAS) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) tv[e] += sc[k].bias;
                }
                float sn[4], cs[4];
                sincos4(tv, sn, cs);
#pragma unroll
                for (int e = 3; e >= 0; --e) {
                    const float nr = fmaf(sc[k].mr, wv[e], er[k]);
                    const float ni = fmaf(-sc[k].mi, wv[e], ei[k]);
                    er[k] = fmaf(cs[e], nr, sn[e] * ni);
                    ei[k] = fmaf(cs[e], ni, -sn[e] * nr);
                }
            }
        }
        __syncwarp();
        const int nr2 = r + STAGES;
        if (nr2 < ntiles) {
            const int nt = ntiles - 1 - nr2;
            map.issue(th, theta_warp, (long long)nt * T, min(T, L - nt * T), lane);
        } else {
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        if (sc[k].act) {
            const long long o = ch * N + jl + k * NL;
            p.dh0_re[o] = er[k];
            p.dh0_im[o] = ei[k];
        }
    }
}

// ---------------------------------------------------------------------------
// Segment chains of the time-axis split: one thread per (channel, state) walks the nseg segments.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) segment_states_fwd_kernel(const float* e_re, const float* e_im,
                                                                 const float* a_re, const float* a_im,
                                                                 const float* start_re, const float* start_im,
                                                                 float* before_re, float* before_im, float* final_re,
                                                                 float* final_im, long long total, int nseg, int N) {
    const long long id = (long long)blockIdx.x * 256 + threadIdx.x;      // ch * N + j
    if (id >= total) return;
    const long long ch = id / N, j = id % N;
    float cr = start_re ? start_re[id] : 0.f, ci = start_im ? start_im[id] : 0.f;
    for (int s = 0; s < nseg; ++s) {
        const long long o = (ch * nseg + s) * N + j;
        before_re[o] = cr;
        before_im[o] = ci;
        const float ar = a_re[o], ai = a_im[o];
        const float nr = fmaf(ar, cr, fmaf(-ai, ci, e_re[o]));
        ci = fmaf(ar, ci, fmaf(ai, cr, e_im[o]));
        cr = nr;
    }
    if (final_re) { final_re[id] = cr; final_im[id] = ci; }
}

__global__ void __launch_bounds__(256) segment_states_bwd_kernel(const float* e_re, const float* e_im,
                                                                 const float* a_re, const float* a_im,
                                                                 const float* final_re, const float* final_im,
                                                                 float* after_re, float* after_im, float* first_re,
                                                                 float* first_im, long long total, int nseg, int N) {
    const long long id = (long long)blockIdx.x * 256 + threadIdx.x;
    if (id >= total) return;
    const long long ch = id / N, j = id % N;
    float cr = final_re[id], ci = final_im[id];
    for (int s = nseg - 1; s >= 0; --s) {
        const long long o = (ch * nseg + s) * N + j;
        after_re[o] = cr;
        after_im[o] = ci;
        // the rotations have modulus one: the state before the segment is conj(a) (c - e)
        const float dr = cr - e_re[o], di = ci - e_im[o];
        const float ar = a_re[o], ai = a_im[o];
        cr = fmaf(ar, dr, ai * di);
        ci = fmaf(ar, di, -ai * dr);
    }
    if (first_re) { first_re[id] = cr; first_im[id] = ci; }
}

__global__ void __launch_bounds__(256) segment_adjoints_kernel(const float* l_re, const float* l_im, const float* a_re,
                                                               const float* a_im, const float* last_re,
                                                               const float* last_im, float* after_re, float* after_im,
                                                               float* first_re, float* first_im, long long total,
                                                               int nseg, int N) {
    const long long id = (long long)blockIdx.x * 256 + threadIdx.x;
    if (id >= total) return;
    const long long ch = id / N, j = id % N;
    float gr = last_re ? last_re[id] : 0.f, gi = last_im ? last_im[id] : 0.f;
    for (int s = nseg - 1; s >= 0; --s) {
        const long long o = (ch * nseg + s) * N + j;
        after_re[o] = gr;
        after_im[o] = gi;
        const float ar = a_re[o], ai = a_im[o];
        const float nr = fmaf(ar, gr, fmaf(ai, gi, l_re[o]));          // l + conj(a) g
        gi = fmaf(ar, gi, fmaf(-ai, gr, l_im[o]));
        gr = nr;
    }
    if (first_re) { first_re[id] = gr; first_im[id] = gi; }
}

// ---------------------------------------------------------------------------
// Second stage: fixed-order sums of the per-channel partials (deterministic)
// and the polar chain rule  dr = Re(conj(G) e^{i phi}),  dphi = -Im(conj(G) w).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) reduce_param_grads_kernel(const ReduceParams p) {
    __shared__ float4 red[256];
    const int tid = threadIdx.x;
    const int nseg = p.nseg > 1 ? p.nseg : 1;               // partial arrays: nseg entries per channel
    const long long nch = (long long)p.batch * p.D * nseg;
    if (blockIdx.x < p.N) {
        const int j = blockIdx.x;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (long long ch = tid; ch < nch; ch += 256) {
            const float4 v = reinterpret_cast<const float4*>(p.part_bc)[ch * p.N + j];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        red[tid] = acc;
        __syncthreads();
        for (int s = 128; s > 0; s >>= 1) {
            if (tid < s) {
                float4 a = red[tid], b = red[tid + s];
                red[tid] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
            }
            __syncthreads();
        }
        if (tid == 0) {
            const float4 g = red[0];
            float sb, cb, sc_, cc_;
            sincosf(p.B_theta[j], &sb, &cb);
            sincosf(p.C_theta[j], &sc_, &cc_);
            const float br = p.B_r[j], cr = p.C_r[j];
            p.dB_r[j] = g.x * cb + g.y * sb;
            p.dB_theta[j] = br * (g.y * cb - g.x * sb);
            p.dC_r[j] = g.z * cc_ + g.w * sc_;
            p.dC_theta[j] = cr * (g.w * cc_ - g.z * sc_);
        }
        return;
    }
    // remaining blocks: dD (D values) then dx_bias (D*N values), one thread per output
    const long long o = (long long)(blockIdx.x - p.N) * 256 + tid;
    if (o < p.D) {
        float acc = 0.f;
        for (int b = 0; b < p.batch; ++b)
            for (int sg = 0; sg < nseg; ++sg) acc += p.part_d[((long long)b * p.D + o) * nseg + sg];
        p.dD[o] = acc;
    } else if (p.dx_bias && o - p.D < (long long)p.D * p.N) {
        const long long e = o - p.D;
        const long long i = e / p.N, j = e % p.N;
        float acc = 0.f;
        for (int b = 0; b < p.batch; ++b)
            for (int sg = 0; sg < nseg; ++sg)
                acc += p.part_rowsum[(((long long)b * p.D + i) * nseg + sg) * p.N + j];
        p.dx_bias[e] = acc;
    }
}

// ---------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <class C, bool ASYNC, bool BIAS, bool AGG>
cudaError_t launch_fwd_cfg(const ScanFwdParams& p, cudaStream_t stream) {
    auto kern = scan_unitary_fwd_kernel<C, ASYNC, BIAS, AGG>;
    const size_t smem = C::SMEM_BYTES;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const long long tasks = ((long long)p.nch + C::CPW - 1) / C::CPW;
    const long long blocks = (tasks + C::WARPS - 1) / C::WARPS;
    kern<<<(unsigned)blocks, C::WARPS * 32, smem, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

template <class C, bool ASYNC, bool BIAS>
cudaError_t launch_bwd_cfg(const ScanBwdParams& p, cudaStream_t stream) {
    auto kern = scan_unitary_bwd_kernel<C, ASYNC, BIAS>;
    const size_t smem = C::SMEM_BYTES;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const long long tasks = ((long long)p.nch + C::CPW - 1) / C::CPW;
    const long long blocks = (tasks + C::WARPS - 1) / C::WARPS;
    kern<<<(unsigned)blocks, C::WARPS * 32, smem, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

// Runtime properties -> template parameters.  The plain (unaligned) path is instantiated with the phase
// offset always on, to keep the build small.
template <class C>
cudaError_t launch_fwd_sel(const ScanFwdParams& p, bool async, cudaStream_t s) {
    const bool bias = p.theta_bias != nullptr;
    if (!async) return p.nseg > 1 || p.agg_re ? cudaErrorInvalidValue : launch_fwd_cfg<C, false, true, false>(p, s);
    if (p.agg_re != nullptr && p.y == nullptr)
        return bias ? launch_fwd_cfg<C, true, true, true>(p, s) : launch_fwd_cfg<C, true, false, true>(p, s);
    return bias ? launch_fwd_cfg<C, true, true, false>(p, s) : launch_fwd_cfg<C, true, false, false>(p, s);
}

template <class C, bool BIAS>
cudaError_t launch_eta_cfg(const ScanBwdParams& p, cudaStream_t stream) {
    auto kern = scan_unitary_eta_kernel<C, BIAS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long tasks = ((long long)p.nch + C::CPW - 1) / C::CPW;
    const long long blocks = (tasks + C::WARPS - 1) / C::WARPS;
    kern<<<(unsigned)blocks, C::WARPS * 32, C::SMEM_BYTES, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

// the adjoint-only pass stages (u, dt, z, gy) like the backward kernel but keeps no column-sum tiles
template <int NL, int SPT, int T, int STAGES, int WARPS>
using EtaCfg = Cfg<NL, SPT, T, T, STAGES, WARPS, 4, false>;

template <class C>
cudaError_t launch_bwd_sel(const ScanBwdParams& p, bool async, cudaStream_t s) {
    const bool bias = p.theta_bias != nullptr || p.part_rowsum != nullptr;
    if (!async) return p.nseg > 1 ? cudaErrorInvalidValue : launch_bwd_cfg<C, false, true>(p, s);
    return bias ? launch_bwd_cfg<C, true, true>(p, s) : launch_bwd_cfg<C, true, false>(p, s);
}

// a warp's rows must be addressable with 32-bit byte offsets from its first row
inline bool offsets_fit(long long ld, int rows_per_warp) { return ld * (long long)rows_per_warp < (1LL << 29); }

}  // namespace

// Tile shapes per state count.  <lanes per channel, states per thread, tile
// steps, [sub-block,] stages, warps per block>.
cudaError_t launch_scan_unitary_fwd(const ScanFwdParams& p_, cudaStream_t stream) {
    if (p_.nch <= 0 || p_.L <= 0) return cudaSuccess;
    ScanFwdParams p = p_;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorInvalidSymbol;
    const bool async = (p.L % 4 == 0) && (p.ld_theta % 4 == 0) && (p.ld_row % 4 == 0) && aligned16(p.theta) &&
                       aligned16(p.u) && aligned16(p.dt) && aligned16(p.z) && (p.y == nullptr || aligned16(p.y)) &&
                       offsets_fit(p.ld_theta, 128);
    const int N = p.N;
    if (N <= 4) return launch_fwd_sel<FwdCfg<4, 1, 32, 2, 4>>(p, async, stream);
    if (N <= 8) return launch_fwd_sel<FwdCfg<8, 1, 32, 2, 4>>(p, async, stream);
    if (N <= 16) return launch_fwd_sel<FwdCfg<16, 1, 32, 2, 4>>(p, async, stream);
    if (N <= 32) return launch_fwd_sel<FwdCfg<32, 1, 32, 2, 4>>(p, async, stream);
    if (N <= 64) return launch_fwd_sel<FwdCfg<32, 2, 32, 2, 4>>(p, async, stream);
    if (N <= 128) return launch_fwd_sel<FwdCfg<32, 4, 32, 2, 2>>(p, async, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_scan_unitary_bwd(const ScanBwdParams& p_, cudaStream_t stream) {
    if (p_.nch <= 0 || p_.L <= 0) return cudaSuccess;
    ScanBwdParams p = p_;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorInvalidSymbol;
    if (p.ld_dtheta != p.ld_theta) return cudaErrorInvalidValue;
    const bool async = (p.L % 4 == 0) && (p.ld_theta % 4 == 0) && (p.ld_row % 4 == 0) && aligned16(p.theta) &&
                       aligned16(p.dtheta) && aligned16(p.u) && aligned16(p.dt) && aligned16(p.z) &&
                       aligned16(p.gy) && aligned16(p.du) && aligned16(p.ddt) && aligned16(p.dz) &&
                       offsets_fit(p.ld_theta, 128);
    const int N = p.N;
    if (p.eta_only) {
        if (!async || !p.dh0_re) return cudaErrorInvalidValue;
        const bool bias = p.theta_bias != nullptr;
#define AUSSM_ETA(...) (bias ? launch_eta_cfg<__VA_ARGS__, true>(p, stream) : launch_eta_cfg<__VA_ARGS__, false>(p, stream))
        if (N <= 4) return AUSSM_ETA(EtaCfg<4, 1, 32, 2, 4>);
        if (N <= 8) return AUSSM_ETA(EtaCfg<8, 1, 32, 2, 4>);
        if (N <= 16) return AUSSM_ETA(EtaCfg<16, 1, 32, 2, 4>);
        if (N <= 32) return AUSSM_ETA(EtaCfg<32, 1, 32, 2, 4>);
        if (N <= 64) return AUSSM_ETA(EtaCfg<32, 2, 32, 2, 4>);
        if (N <= 128) return AUSSM_ETA(EtaCfg<32, 4, 32, 2, 2>);
#undef AUSSM_ETA
        return cudaErrorInvalidValue;
    }
    if (N <= 4) return launch_bwd_sel<BwdCfg<4, 1, 32, 32, 2, 2>>(p, async, stream);
    if (N <= 8) return launch_bwd_sel<BwdCfg<8, 1, 32, 32, 2, 2>>(p, async, stream);
    // one-warp blocks: a finished warp is replaced at once (measured 9.55 ms against 10.2 ms with two-warp blocks)
    if (N <= 16) return launch_bwd_sel<BwdCfg<16, 1, 32, 32, 2, 1>>(p, async, stream);
    if (N <= 32) return launch_bwd_sel<BwdCfg<32, 1, 32, 32, 2, 2>>(p, async, stream);
    if (N <= 64) return launch_bwd_sel<BwdCfg<32, 2, 32, 32, 2, 2>>(p, async, stream);
    if (N <= 128) return launch_bwd_sel<BwdCfg<32, 4, 32, 32, 2, 2>>(p, async, stream);
    return cudaErrorInvalidValue;
}

int scan_split_segments(long long nch, int N, int L, bool bwd) {
    if (nch <= 0 || L <= 0 || N <= 0 || N > 128 || !time_split_option()) return 1;
    // warps the launch has and warps the GPU holds (148 SMs; 20 resident forward warps per SM, 10 backward:
    // shared memory limits both)
    const int nl = N <= 4 ? 4 : N <= 8 ? 8 : N <= 16 ? 16 : 32;
    const long long warps = (nch + (32 / nl) - 1) / (32 / nl);
    const long long slots = 148LL * (bwd ? 10 : 20);
    // a split doubles the work (an aggregate pass before the real one), and an SM with a third of its warps
    // resident is already more than half busy, so it pays only when the launch fills less than a quarter
    if (warps * 4 > slots) return 1;
    int best = 1;
    for (int s = 2; s <= 64; s *= 2) {
        if (L % s != 0 || (L / s) % 32 != 0 || L / s < 256) break;
        best = s;
        if (warps * s >= slots) break;
    }
    return best;
}

namespace {
unsigned seg_blocks(long long total) { return (unsigned)((total + 255) / 256); }
}  // namespace

cudaError_t launch_segment_states_fwd(const float* e_re, const float* e_im, const float* a_re, const float* a_im,
                                      const float* start_re, const float* start_im, float* before_re,
                                      float* before_im, float* final_re, float* final_im, long long nch, int nseg,
                                      int N, cudaStream_t stream) {
    const long long total = nch * N;
    segment_states_fwd_kernel<<<seg_blocks(total), 256, 0, stream>>>(e_re, e_im, a_re, a_im, start_re, start_im,
                                                                      before_re, before_im, final_re, final_im, total,
                                                                      nseg, N);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_segment_states_bwd(const float* e_re, const float* e_im, const float* a_re, const float* a_im,
                                      const float* final_re, const float* final_im, float* after_re, float* after_im,
                                      float* first_re, float* first_im, long long nch, int nseg, int N,
                                      cudaStream_t stream) {
    const long long total = nch * N;
    segment_states_bwd_kernel<<<seg_blocks(total), 256, 0, stream>>>(e_re, e_im, a_re, a_im, final_re, final_im,
                                                                      after_re, after_im, first_re, first_im, total,
                                                                      nseg, N);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_segment_adjoints(const float* l_re, const float* l_im, const float* a_re, const float* a_im,
                                    const float* last_re, const float* last_im, float* after_re, float* after_im,
                                    float* first_re, float* first_im, long long nch, int nseg, int N,
                                    cudaStream_t stream) {
    const long long total = nch * N;
    segment_adjoints_kernel<<<seg_blocks(total), 256, 0, stream>>>(l_re, l_im, a_re, a_im, last_re, last_im, after_re,
                                                                    after_im, first_re, first_im, total, nseg, N);
    count_launch();
    return cudaGetLastError();
}

bool scan_split_allowed(const ScanFwdParams& p) {
    return (p.L % 4 == 0) && (p.ld_theta % 4 == 0) && (p.ld_row % 4 == 0) && aligned16(p.theta) && aligned16(p.u) &&
           aligned16(p.dt) && aligned16(p.z) && (p.y == nullptr || aligned16(p.y)) && offsets_fit(p.ld_theta, 128);
}

bool scan_split_allowed(const ScanBwdParams& p) {
    return (p.L % 4 == 0) && (p.ld_theta % 4 == 0) && (p.ld_row % 4 == 0) && p.ld_dtheta == p.ld_theta &&
           aligned16(p.theta) && aligned16(p.dtheta) && aligned16(p.u) && aligned16(p.dt) && aligned16(p.z) &&
           aligned16(p.gy) && aligned16(p.du) && aligned16(p.ddt) && aligned16(p.dz) && offsets_fit(p.ld_theta, 128);
}

// Forward with the time axis cut into nseg segments per channel: (A) every segment from a zero state, without
// output: its end state e and the product a of its rotations; (B) the chain c_{s+1} = e_s + a_s c_s gives the
// state before every segment; (C) the real pass, every segment from its true initial state.
cudaError_t scan_unitary_fwd_split(const ScanFwdParams& p, int nseg, float* scratch, cudaStream_t stream) {
    const long long V = (long long)p.nch * nseg, VN = V * p.N;
    float *e_re = scratch, *e_im = e_re + VN, *a_re = e_im + VN, *a_im = a_re + VN, *b_re = a_im + VN,
          *b_im = b_re + VN;
    ScanFwdParams q = p;
    q.nch = (int)V; q.L = p.L / nseg; q.nseg = nseg;
    q.y = nullptr; q.h0_re = q.h0_im = nullptr; q.h1_re = e_re; q.h1_im = e_im; q.agg_re = a_re; q.agg_im = a_im;
    cudaError_t err = launch_scan_unitary_fwd(q, stream);
    if (err != cudaSuccess) return err;
    err = launch_segment_states_fwd(e_re, e_im, a_re, a_im, p.h0_re, p.h0_im, b_re, b_im, p.h1_re, p.h1_im, p.nch, nseg,
                                    p.N, stream);
    if (err != cudaSuccess) return err;
    if (!p.y) return cudaSuccess;                       // state-only call: the chain already gave the final state
    q.y = p.y; q.h0_re = b_re; q.h0_im = b_im; q.h1_re = q.h1_im = nullptr; q.agg_re = q.agg_im = nullptr;
    return launch_scan_unitary_fwd(q, stream);
}

// Backward with the same cut: (A) the forward aggregates again; (B) the state after every segment, walking
// back from the final state (the rotations are invertible); (C) every segment's own contribution to the
// gradient of the state before it; (D) the chain g_s = l_s + conj(a_s) g_{s+1} gives the gradient after every
// segment; (E) the real backward pass, every segment with its true end state and incoming gradient.
cudaError_t scan_unitary_bwd_split(const ScanBwdParams& p, int nseg, float* scratch, cudaStream_t stream) {
    const long long V = (long long)p.nch * nseg, VN = V * p.N;
    float *e_re = scratch, *e_im = e_re + VN, *a_re = e_im + VN, *a_im = a_re + VN, *s_re = a_im + VN,
          *s_im = s_re + VN, *l_re = s_im + VN, *l_im = l_re + VN, *g_re = l_im + VN, *g_im = g_re + VN;
    ScanFwdParams f = {};
    f.theta = p.theta; f.theta_bias = p.theta_bias; f.u = p.u; f.dt = p.dt; f.z = p.z;
    f.B_r = p.B_r; f.B_theta = p.B_theta; f.C_r = p.C_r; f.C_theta = p.C_theta; f.Dskip = p.Dskip;
    f.h1_re = e_re; f.h1_im = e_im; f.agg_re = a_re; f.agg_im = a_im;
    f.nch = (int)V; f.Dmod = p.Dmod; f.N = p.N; f.L = p.L / nseg; f.ld_theta = p.ld_theta; f.ld_row = p.ld_row;
    f.nseg = nseg;
    cudaError_t err = launch_scan_unitary_fwd(f, stream);
    if (err != cudaSuccess) return err;
    err = launch_segment_states_bwd(e_re, e_im, a_re, a_im, p.h1_re, p.h1_im, s_re, s_im, p.h0_re, p.h0_im, p.nch, nseg,
                                    p.N, stream);
    if (err != cudaSuccess) return err;
    ScanBwdParams q = p;
    q.nch = (int)V; q.L = p.L / nseg; q.nseg = nseg;
    q.eta_only = 1; q.dh0_re = l_re; q.dh0_im = l_im;
    err = launch_scan_unitary_bwd(q, stream);
    if (err != cudaSuccess) return err;
    err = launch_segment_adjoints(l_re, l_im, a_re, a_im, p.gh1_re, p.gh1_im, g_re, g_im, p.dh0_re, p.dh0_im, p.nch,
                                  nseg, p.N, stream);
    if (err != cudaSuccess) return err;
    q.eta_only = 0;
    q.h1_re = s_re; q.h1_im = s_im; q.gh1_re = g_re; q.gh1_im = g_im;
    q.dh0_re = q.dh0_im = nullptr; q.h0_re = q.h0_im = nullptr;
    return launch_scan_unitary_bwd(q, stream);
}

cudaError_t launch_reduce_param_grads(const ReduceParams& p, cudaStream_t stream) {
    const long long tail = (long long)p.D + (p.dx_bias ? (long long)p.D * p.N : 0);
    const unsigned blocks = (unsigned)(p.N + (tail + 255) / 256);
    reduce_param_grads_kernel<<<blocks, 256, 0, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace aussm
