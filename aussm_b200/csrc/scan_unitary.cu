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
// Work decomposition: one thread owns SPT states of one channel and walks the
// time axis sequentially, so the recurrence costs four fused multiply-adds
// per step and needs no scan tree.  A warp owns 32/NL channels (NL lanes per
// channel) and is completely independent of every other warp: it has its own
// ring of shared-memory stages and its own mbarriers, and the kernel contains
// no block-wide barrier.  The theta rows of a warp (contiguous in time in
// HBM, but one row per state) are staged by bulk copies (TMA engine), each
// lane fetching the rows it will consume, into rows padded by 16 bytes so
// that the per-thread 128-bit shared loads of a quarter-warp hit disjoint
// banks.  Sums over the states of a channel go through the same tile: every
// thread overwrites the four phases it has just consumed with its four
// contributions, and after the tile the lanes switch roles (one lane = one
// channel and four consecutive steps) to add the NL rows and emit y with
// 128-bit coalesced stores.
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
// written in place of theta in the stage and leaves by a bulk store.
#include "common.cuh"
#include "scan_unitary.cuh"

namespace aussm {

__device__ int g_device_status = 0;

ScanOptions& scan_options() {
    static ScanOptions o = {0, 0, 0};
    return o;
}

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

template <int NL_, int SPT_, int T_, int STAGES_, int WARPS_>
struct FwdCfg {
    static constexpr int NL = NL_, SPT = SPT_, T = T_, STAGES = STAGES_, WARPS = WARPS_;
    static constexpr int CPW = 32 / NL;                 // channels per warp
    static constexpr int TP = T + 4;                    // padded row pitch (floats)
    static constexpr int NROWS = 32 * SPT;
    static constexpr int AUX = 3;                       // u, dt (becomes s), z
    static constexpr int STAGE_FLOATS = NROWS * TP + CPW * AUX * T;
    static constexpr int WARP_FLOATS = STAGES * STAGE_FLOATS;
    static constexpr size_t SMEM_BYTES = (size_t)WARPS * WARP_FLOATS * sizeof(float);
    static constexpr int NIDX = CPW * (T / 4);          // (channel, quad) items of a tile
    static constexpr int ITERS = (NIDX + 31) / 32;
};

template <int NL_, int SPT_, int T_, int TS_, int STAGES_, int WARPS_>
struct BwdCfg {
    static constexpr int NL = NL_, SPT = SPT_, T = T_, TS = TS_, STAGES = STAGES_, WARPS = WARPS_;
    static constexpr int CPW = 32 / NL;
    static constexpr int TP = T + 4;
    static constexpr int TSP = TS + 4;
    static constexpr int NROWS = 32 * SPT;
    static constexpr int AUX = 4;                       // u, dt, z, gy
    static constexpr int STAGE_FLOATS = NROWS * TP + CPW * AUX * T;
    // per warp, not staged: two column-sum tiles and the s / w rows of a sub-block
    static constexpr int SCRATCH_FLOATS = 2 * 32 * TSP + CPW * 2 * TS;
    static constexpr int WARP_FLOATS = STAGES * STAGE_FLOATS + SCRATCH_FLOATS;
    static constexpr size_t SMEM_BYTES = (size_t)WARPS * WARP_FLOATS * sizeof(float);
    static constexpr int NIDX = CPW * (TS / 4);
    static constexpr int ITERS = (NIDX + 31) / 32;
    static_assert(T % TS == 0, "sub-block must divide the tile");
};

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

// ---------------------------------------------------------------------------
// Tile movement
// ---------------------------------------------------------------------------
// shared-memory slot of state j of warp-channel c
template <int NL>
__device__ __forceinline__ int slot_of(int c, int j) {
    return (j / NL) * 32 + c * NL + (j % NL);
}

// Plain (no TMA) tile load: coalesced along time, zero-filled up to a quad.
template <int NL, int TP, int T, int AUX>
__device__ __forceinline__ void plain_load_tile(float* th, float* aux, const float* theta, long long ld_theta,
                                                const float* const* aux_src, long long ld_row, long long ch0,
                                                int nvalid, int N, long long t0, int tlen, int lane) {
    const int tq = (tlen + 3) & ~3;
    for (int c = 0; c < nvalid; ++c) {
        for (int j = 0; j < N; ++j) {
            const float* src = theta + ((ch0 + c) * N + j) * ld_theta + t0;
            float* dst = th + slot_of<NL>(c, j) * TP;
            for (int t = lane; t < tq; t += 32) dst[t] = t < tlen ? src[t] : 0.f;
        }
        for (int a = 0; a < AUX; ++a) {
            const float* src = aux_src[a] + (ch0 + c) * ld_row + t0;
            float* dst = aux + (c * AUX + a) * T;
            for (int t = lane; t < tq; t += 32) dst[t] = t < tlen ? src[t] : 0.f;
        }
    }
    __syncwarp();
}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
template <class C, bool BULK, bool FAST, bool NORM>
__device__ __forceinline__ void fwd_warp(const ScanFwdParams& p, float* wsm, uint64_t* wbar, long long ch0,
                                         int nvalid, int lane, StateConsts (&sc)[C::SPT]) {
    constexpr int NL = C::NL, SPT = C::SPT, T = C::T, TP = C::TP, STAGES = C::STAGES, CPW = C::CPW, AUX = C::AUX;
    const int c = lane / NL, jl = lane % NL;
    const long long ch = ch0 + c;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;

    float hr[SPT], hi[SPT];
    const float* rowp[SPT];
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        const int j = jl + k * NL;
        hr[k] = hi[k] = 0.f;
        rowp[k] = p.theta;
        if (sc[k].act) {
            rowp[k] = p.theta + (ch * N + j) * p.ld_theta;
            float ar = p.h0_re ? p.h0_re[ch * N + j] : 0.f;
            float ai = p.h0_im ? p.h0_im[ch * N + j] : 0.f;
            if (NORM) cdiv(ar, ai, sc[k].kr, sc[k].ki, hr[k], hi[k]);
            else { hr[k] = ar; hi[k] = ai; }
        }
    }
    // D of the channel each post-pass item of this lane belongs to
    float dval[C::ITERS];
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int idx = lane + 32 * it;
        const int cc = idx / (T / 4);
        dval[it] = (idx < C::NIDX && cc < nvalid) ? p.Dskip[(ch0 + cc) % p.Dmod] : 0.f;
    }
    const float* aux_src[AUX] = {p.u, p.dt, p.z};

    auto issue = [&](int tile, int stage) {
        float* th = wsm + stage * C::STAGE_FLOATS;
        float* aux = th + C::NROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        const uint32_t bytes = (uint32_t)tlen * 4u;
        if (lane == 0) mbar_arrive_expect_tx(&wbar[stage], (uint32_t)(nvalid * (N + AUX)) * bytes);
        __syncwarp();
#pragma unroll
        for (int k = 0; k < SPT; ++k)
            if (sc[k].act) bulk_g2s(th + (k * 32 + lane) * TP, rowp[k] + t0, bytes, &wbar[stage]);
        if (lane < nvalid * AUX) {
            const int cc = lane / AUX, a = lane % AUX;
            bulk_g2s(aux + (cc * AUX + a) * T, aux_src[a] + (ch0 + cc) * p.ld_row + t0, bytes, &wbar[stage]);
        }
    };

    if (BULK) {
        for (int s = 0; s < STAGES && s < ntiles; ++s) issue(s, s);
    }

    for (int tile = 0; tile < ntiles; ++tile) {
        const int stage = BULK ? tile % STAGES : 0;
        float* th = wsm + stage * C::STAGE_FLOATS;
        float* aux = th + C::NROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        const int nq = (tlen + 3) >> 2;
        if (BULK) {
            if (!mbar_wait_bounded(&wbar[stage], (uint32_t)(tile / STAGES) & 1u, p.status)) return;
        } else {
            plain_load_tile<NL, TP, T, AUX>(th, aux, p.theta, p.ld_theta, aux_src, p.ld_row, ch0, nvalid, N, t0,
                                            tlen, lane);
        }

        // pre-pass: s = dt * silu(u) over the dt row
#pragma unroll
        for (int it = 0; it < C::ITERS; ++it) {
            const int idx = lane + 32 * it;
            const int cc = idx / (T / 4), q = idx % (T / 4);
            if (idx < C::NIDX && cc < nvalid && q < nq) {
                float4 u4 = ld_shared_f4(aux + (cc * AUX + 0) * T + 4 * q);
                float4 d4 = ld_shared_f4(aux + (cc * AUX + 1) * T + 4 * q);
                d4.x *= siluf_(u4.x); d4.y *= siluf_(u4.y); d4.z *= siluf_(u4.z); d4.w *= siluf_(u4.w);
                st_shared_f4(aux + (cc * AUX + 1) * T + 4 * q, d4);
            }
        }
        __syncwarp();

        // scan: SPT states per thread, four steps per shared-memory access
        const float* srow = aux + (c * AUX + 1) * T;
        for (int q = 0; q < nq; ++q) {
            const float4 s4 = ld_shared_f4(srow + 4 * q);
            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
            float pacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < SPT; ++k) {
                float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (sc[k].act) t4 = ld_shared_f4(th + (k * 32 + lane) * TP + 4 * q);
                const float tv[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (!BULK && 4 * q + e >= tlen) continue;   // ragged tail (plain path only)
                    float sn, cs;
                    sincos_sel<FAST>(tv[e] + sc[k].bias, sn, cs);
                    float nr, ni;
                    if (NORM) {
                        nr = fmaf(cs, hr[k], fmaf(-sn, hi[k], sv[e]));
                        ni = fmaf(cs, hi[k], sn * hr[k]);
                    } else {
                        nr = fmaf(cs, hr[k], fmaf(-sn, hi[k], sc[k].br * sv[e]));
                        ni = fmaf(cs, hi[k], fmaf(sn, hr[k], sc[k].bi * sv[e]));
                    }
                    hr[k] = nr;
                    hi[k] = ni;
                    pacc[e] += fmaf(sc[k].mr, nr, -sc[k].mi * ni);
                }
            }
            st_shared_f4(th + lane * TP + 4 * q, make_float4(pacc[0], pacc[1], pacc[2], pacc[3]));
        }
        __syncwarp();

        // post-pass: one lane = one channel and four steps
        if (p.y) {
#pragma unroll
            for (int it = 0; it < C::ITERS; ++it) {
                const int idx = lane + 32 * it;
                const int cc = idx / (T / 4), q = idx % (T / 4);
                if (idx < C::NIDX && cc < nvalid && q < nq) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int r = 0; r < NL; ++r) {
                        float4 v = ld_shared_f4(th + (cc * NL + r) * TP + 4 * q);
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                    const float4 u4 = ld_shared_f4(aux + (cc * AUX + 0) * T + 4 * q);
                    const float4 z4 = ld_shared_f4(aux + (cc * AUX + 2) * T + 4 * q);
                    const float dv = dval[it];
                    float4 y4;
                    y4.x = siluf_(z4.x) * fmaf(dv, siluf_(u4.x), acc.x);
                    y4.y = siluf_(z4.y) * fmaf(dv, siluf_(u4.y), acc.y);
                    y4.z = siluf_(z4.z) * fmaf(dv, siluf_(u4.z), acc.z);
                    y4.w = siluf_(z4.w) * fmaf(dv, siluf_(u4.w), acc.w);
                    float* dst = p.y + (ch0 + cc) * p.ld_row + t0 + 4 * q;
                    if (BULK) {
                        *reinterpret_cast<float4*>(dst) = y4;
                    } else {
                        const float yv[4] = {y4.x, y4.y, y4.z, y4.w};
                        for (int e = 0; e < 4; ++e)
                            if (4 * q + e < tlen) dst[e] = yv[e];
                    }
                }
            }
        }
        __syncwarp();
        if (BULK && tile + STAGES < ntiles) {
            fence_proxy_async();
            issue(tile + STAGES, stage);
        }
    }

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
    }
}

template <class C, bool BULK, bool FAST>
__global__ void __launch_bounds__(C::WARPS * 32) scan_unitary_fwd_kernel(const ScanFwdParams p) {
    extern __shared__ __align__(128) float smem[];
    __shared__ uint64_t bars[C::WARPS * C::STAGES];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long ch0 = ((long long)blockIdx.x * C::WARPS + warp) * C::CPW;
    if (ch0 >= p.nch) return;   // warps never meet at a block barrier
    const int nvalid = (int)min((long long)C::CPW, (long long)p.nch - ch0);
    float* wsm = smem + (size_t)warp * C::WARP_FLOATS;
    uint64_t* wbar = bars + warp * C::STAGES;
    if (BULK) {
        if (lane == 0) {
            for (int s = 0; s < C::STAGES; ++s) mbar_init(&wbar[s], 1);
            fence_mbar_init();
            fence_proxy_async();
        }
        __syncwarp();
    }
    const int c = lane / C::NL, jl = lane % C::NL;
    const int i = (int)((ch0 + min(c, nvalid - 1)) % p.Dmod);
    StateConsts sc[C::SPT];
    bool ok = true;
#pragma unroll
    for (int k = 0; k < C::SPT; ++k) {
        const int j = jl + k * C::NL;
        bool okk;
        load_state_consts(sc[k], c < nvalid && j < p.N, j, i, p.N, p.B_r, p.B_theta, p.C_r, p.C_theta,
                          p.theta_bias, okk);
        ok = ok && okk;
    }
    if (__all_sync(0xffffffffu, ok)) {
#pragma unroll
        for (int k = 0; k < C::SPT; ++k) {
            float a, b;
            normalise_consts(sc[k], a, b);
        }
        fwd_warp<C, BULK, FAST, true>(p, wsm, wbar, ch0, nvalid, lane, sc);
    } else {
        fwd_warp<C, BULK, FAST, false>(p, wsm, wbar, ch0, nvalid, lane, sc);
    }
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------
template <class C, bool BULK, bool FAST, bool NORM>
__device__ __forceinline__ void bwd_warp(const ScanBwdParams& p, float* wsm, uint64_t* wbar, long long ch0,
                                         int nvalid, int lane, StateConsts (&sc)[C::SPT],
                                         const float (&ccr)[C::SPT], const float (&cci)[C::SPT]) {
    constexpr int NL = C::NL, SPT = C::SPT, T = C::T, TS = C::TS, TP = C::TP, TSP = C::TSP, STAGES = C::STAGES,
                  CPW = C::CPW, AUX = C::AUX;
    const int c = lane / NL, jl = lane % NL;
    const long long ch = ch0 + c;
    const int N = p.N, L = p.L;
    const int ntiles = (L + T - 1) / T;

    float* scratch = wsm + STAGES * C::STAGE_FLOATS;
    float* pt = scratch;                    // [32][TSP] projections, summed over a thread's states
    float* et = pt + 32 * TSP;              // [32][TSP] Re(eta)
    float* sw = et + 32 * TSP;              // [CPW][2][TS]: s row, w row

    float hr[SPT], hi[SPT];     // state h_t (normalised), walking backwards
    float er[SPT], ei[SPT];     // exp(-i theta_{t+1}) eta_{t+1}
    float gmr[SPT], gmi[SPT];   // sum_t w_t conj(h_t)
    float sbr[SPT], sbi[SPT];   // sum_t eta_t s_t              (general representation only)
    float rsum[SPT];            // sum_t dtheta_t
    float hlr[SPT], hli[SPT];   // conj(h_{L-1}) . gh   (boundary term of the Bc gradient)
    const float* rowp[SPT];
    float* drowp[SPT];
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        const int j = jl + k * NL;
        hr[k] = hi[k] = er[k] = ei[k] = gmr[k] = gmi[k] = sbr[k] = sbi[k] = rsum[k] = hlr[k] = hli[k] = 0.f;
        rowp[k] = p.theta;
        drowp[k] = p.dtheta;
        if (sc[k].act) {
            rowp[k] = p.theta + (ch * N + j) * p.ld_theta;
            drowp[k] = p.dtheta + (ch * N + j) * p.ld_dtheta;
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
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int idx = lane + 32 * it;
        const int cc = idx / (TS / 4);
        dval[it] = (idx < C::NIDX && cc < nvalid) ? p.Dskip[(ch0 + cc) % p.Dmod] : 0.f;
        dacc[it] = 0.f;
    }
    const float* aux_src[AUX] = {p.u, p.dt, p.z, p.gy};

    auto issue = [&](int tile, int stage) {
        float* th = wsm + stage * C::STAGE_FLOATS;
        float* aux = th + C::NROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        const uint32_t bytes = (uint32_t)tlen * 4u;
        if (lane == 0) mbar_arrive_expect_tx(&wbar[stage], (uint32_t)(nvalid * (N + AUX)) * bytes);
        __syncwarp();
#pragma unroll
        for (int k = 0; k < SPT; ++k)
            if (sc[k].act) bulk_g2s(th + (k * 32 + lane) * TP, rowp[k] + t0, bytes, &wbar[stage]);
        if (lane < nvalid * AUX) {
            const int cc = lane / AUX, a = lane % AUX;
            bulk_g2s(aux + (cc * AUX + a) * T, aux_src[a] + (ch0 + cc) * p.ld_row + t0, bytes, &wbar[stage]);
        }
    };

    // r counts tiles in processing order (last tile first)
    if (BULK) {
        for (int r = 0; r < STAGES && r < ntiles; ++r) issue(ntiles - 1 - r, r);
    }

    for (int r = 0; r < ntiles; ++r) {
        const int tile = ntiles - 1 - r;
        const int stage = BULK ? r % STAGES : 0;
        float* th = wsm + stage * C::STAGE_FLOATS;
        float* aux = th + C::NROWS * TP;
        const long long t0 = (long long)tile * T;
        const int tlen = min(T, L - (int)t0);
        if (BULK) {
            if (!mbar_wait_bounded(&wbar[stage], (uint32_t)(r / STAGES) & 1u, p.status)) break;
        } else {
            plain_load_tile<NL, TP, T, AUX>(th, aux, p.theta, p.ld_theta, aux_src, p.ld_row, ch0, nvalid, N, t0,
                                            tlen, lane);
        }

        const int nsb = (tlen + TS - 1) / TS;
        for (int sb = nsb - 1; sb >= 0; --sb) {
            const int sbeg = sb * TS;                       // first step of the sub-block in the tile
            const int slen = min(TS, tlen - sbeg);
            const int nq = (slen + 3) >> 2;
            const int qoff = sbeg >> 2;                     // quad offset inside the tile

            // pre-pass: s = dt silu(u), w = gy silu(z)
#pragma unroll
            for (int it = 0; it < C::ITERS; ++it) {
                const int idx = lane + 32 * it;
                const int cc = idx / (TS / 4), q = idx % (TS / 4);
                if (idx < C::NIDX && cc < nvalid && q < nq) {
                    const int o = 4 * (qoff + q);
                    const float4 u4 = ld_shared_f4(aux + (cc * AUX + 0) * T + o);
                    const float4 d4 = ld_shared_f4(aux + (cc * AUX + 1) * T + o);
                    const float4 z4 = ld_shared_f4(aux + (cc * AUX + 2) * T + o);
                    const float4 g4 = ld_shared_f4(aux + (cc * AUX + 3) * T + o);
                    st_shared_f4(sw + (cc * 2 + 0) * TS + 4 * q,
                                 make_float4(d4.x * siluf_(u4.x), d4.y * siluf_(u4.y), d4.z * siluf_(u4.z),
                                             d4.w * siluf_(u4.w)));
                    st_shared_f4(sw + (cc * 2 + 1) * TS + 4 * q,
                                 make_float4(g4.x * siluf_(z4.x), g4.y * siluf_(z4.y), g4.z * siluf_(z4.z),
                                             g4.w * siluf_(z4.w)));
                }
            }
            __syncwarp();

            // reverse scan
            for (int q = nq - 1; q >= 0; --q) {
                const float4 s4 = ld_shared_f4(sw + (c * 2 + 0) * TS + 4 * q);
                const float4 w4 = ld_shared_f4(sw + (c * 2 + 1) * TS + 4 * q);
                const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
                const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
                float pacc[4] = {0.f, 0.f, 0.f, 0.f};
                float eacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < SPT; ++k) {
                    float* cell = th + (k * 32 + lane) * TP + 4 * (qoff + q);
                    float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (sc[k].act) t4 = ld_shared_f4(cell);
                    const float tv[4] = {t4.x, t4.y, t4.z, t4.w};
                    float dth[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int e = 3; e >= 0; --e) {
                        if (!BULK && 4 * q + e >= slen) continue;
                        float sn, cs;
                        sincos_sel<FAST>(tv[e] + sc[k].bias, sn, cs);
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
                        rsum[k] += d;
                        pacc[e] += fmaf(sc[k].mr, hr[k], -sc[k].mi * hi[k]);
                        // gradient of the real drive s_t: Re(conj(eta) beta)
                        if (NORM) eacc[e] += nr;
                        else eacc[e] += fmaf(nr, sc[k].br, ni * sc[k].bi);
                        gmr[k] = fmaf(w, hr[k], gmr[k]);
                        gmi[k] = fmaf(-w, hi[k], gmi[k]);
                        if (!NORM) { sbr[k] = fmaf(nr, s, sbr[k]); sbi[k] = fmaf(ni, s, sbi[k]); }
                        // step back: h_{t-1} = conj(lambda) a ; carry = conj(lambda) eta
                        hr[k] = fmaf(cs, ar, sn * ai);
                        hi[k] = fmaf(cs, ai, -sn * ar);
                        er[k] = fmaf(cs, nr, sn * ni);
                        ei[k] = fmaf(cs, ni, -sn * nr);
                    }
                    if (sc[k].act) st_shared_f4(cell, make_float4(dth[0], dth[1], dth[2], dth[3]));
                }
                st_shared_f4(pt + lane * TSP + 4 * q, make_float4(pacc[0], pacc[1], pacc[2], pacc[3]));
                st_shared_f4(et + lane * TSP + 4 * q, make_float4(eacc[0], eacc[1], eacc[2], eacc[3]));
            }
            __syncwarp();

            // post-pass: du, ddt, dz for one channel and four steps per lane
#pragma unroll
            for (int it = 0; it < C::ITERS; ++it) {
                const int idx = lane + 32 * it;
                const int cc = idx / (TS / 4), q = idx % (TS / 4);
                if (idx < C::NIDX && cc < nvalid && q < nq) {
                    float4 P = make_float4(0.f, 0.f, 0.f, 0.f), E = P;
#pragma unroll
                    for (int rr = 0; rr < NL; ++rr) {
                        const float4 a = ld_shared_f4(pt + (cc * NL + rr) * TSP + 4 * q);
                        const float4 b = ld_shared_f4(et + (cc * NL + rr) * TSP + 4 * q);
                        P.x += a.x; P.y += a.y; P.z += a.z; P.w += a.w;
                        E.x += b.x; E.y += b.y; E.z += b.z; E.w += b.w;
                    }
                    const int o = 4 * (qoff + q);
                    const float4 u4 = ld_shared_f4(aux + (cc * AUX + 0) * T + o);
                    const float4 d4 = ld_shared_f4(aux + (cc * AUX + 1) * T + o);
                    const float4 z4 = ld_shared_f4(aux + (cc * AUX + 2) * T + o);
                    const float4 g4 = ld_shared_f4(aux + (cc * AUX + 3) * T + o);
                    const float uv[4] = {u4.x, u4.y, u4.z, u4.w}, dtv[4] = {d4.x, d4.y, d4.z, d4.w};
                    const float zv[4] = {z4.x, z4.y, z4.z, z4.w}, gv[4] = {g4.x, g4.y, g4.z, g4.w};
                    const float Pv[4] = {P.x, P.y, P.z, P.w}, Ev[4] = {E.x, E.y, E.z, E.w};
                    float duv[4], ddtv[4], dzv[4];
                    const float dv = dval[it];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float gu, gz;
                        const float v = silu_and_grad(uv[e], gu);
                        const float g = silu_and_grad(zv[e], gz);
                        const float w = gv[e] * g;
                        dzv[e] = gv[e] * fmaf(dv, v, Pv[e]) * gz;
                        ddtv[e] = Ev[e] * v;
                        duv[e] = fmaf(Ev[e], dtv[e], w * dv) * gu;
                        if (BULK || 4 * q + e < slen) dacc[it] = fmaf(w, v, dacc[it]);
                    }
                    const long long off = (ch0 + cc) * p.ld_row + t0 + o;
                    if (BULK) {
                        *reinterpret_cast<float4*>(p.du + off) = make_float4(duv[0], duv[1], duv[2], duv[3]);
                        *reinterpret_cast<float4*>(p.ddt + off) = make_float4(ddtv[0], ddtv[1], ddtv[2], ddtv[3]);
                        *reinterpret_cast<float4*>(p.dz + off) = make_float4(dzv[0], dzv[1], dzv[2], dzv[3]);
                    } else {
                        for (int e = 0; e < 4; ++e) {
                            if (4 * q + e < slen) {
                                p.du[off + e] = duv[e];
                                p.ddt[off + e] = ddtv[e];
                                p.dz[off + e] = dzv[e];
                            }
                        }
                    }
                }
            }
            __syncwarp();
        }

        // dtheta leaves the stage
        if (BULK) {
            fence_proxy_async();
            const uint32_t bytes = (uint32_t)tlen * 4u;
#pragma unroll
            for (int k = 0; k < SPT; ++k)
                if (sc[k].act) bulk_s2g(drowp[k] + t0, th + (k * 32 + lane) * TP, bytes);
            bulk_commit();
            // refill the stage used one tile ago: its store must have finished reading
            if (r >= 1 && r - 1 + STAGES < ntiles) {
                bulk_wait_read<1>();
                __syncwarp();
                issue(ntiles - 1 - (r - 1 + STAGES), (r - 1) % STAGES);
            }
        } else {
            for (int cc = 0; cc < nvalid; ++cc)
                for (int j = 0; j < N; ++j) {
                    float* dst = p.dtheta + ((ch0 + cc) * N + j) * p.ld_dtheta + t0;
                    const float* src = th + slot_of<NL>(cc, j) * TP;
                    for (int t = lane; t < tlen; t += 32) dst[t] = src[t];
                }
            __syncwarp();
        }
    }
    if (BULK) bulk_wait_all<0>();

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
        if (p.part_rowsum) p.part_rowsum[o] = rsum[k] + (p.accumulate ? p.part_rowsum[o] : 0.f);
        if (p.dh0_re) { p.dh0_re[o] = d0r; p.dh0_im[o] = d0i; }
        if (p.h0_re) { p.h0_re[o] = s0r; p.h0_im[o] = s0i; }
    }
    // dD: add the lanes' partial sums channel by channel through the scratch tile
    __syncwarp();
#pragma unroll
    for (int it = 0; it < C::ITERS; ++it) {
        const int idx = lane + 32 * it;
        if (idx < C::NIDX) pt[idx] = dacc[it];
    }
    __syncwarp();
    if (lane < nvalid) {
        float acc = 0.f;
        for (int q = 0; q < TS / 4; ++q) acc += pt[lane * (TS / 4) + q];
        const long long o = ch0 + lane;
        p.part_d[o] = acc + (p.accumulate ? p.part_d[o] : 0.f);
    }
}

template <class C, bool BULK, bool FAST>
__global__ void __launch_bounds__(C::WARPS * 32) scan_unitary_bwd_kernel(const ScanBwdParams p) {
    extern __shared__ __align__(128) float smem[];
    __shared__ uint64_t bars[C::WARPS * C::STAGES];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long ch0 = ((long long)blockIdx.x * C::WARPS + warp) * C::CPW;
    if (ch0 >= p.nch) return;
    const int nvalid = (int)min((long long)C::CPW, (long long)p.nch - ch0);
    float* wsm = smem + (size_t)warp * C::WARP_FLOATS;
    uint64_t* wbar = bars + warp * C::STAGES;
    if (BULK) {
        if (lane == 0) {
            for (int s = 0; s < C::STAGES; ++s) mbar_init(&wbar[s], 1);
            fence_mbar_init();
            fence_proxy_async();
        }
        __syncwarp();
    }
    const int c = lane / C::NL, jl = lane % C::NL;
    const int i = (int)((ch0 + min(c, nvalid - 1)) % p.Dmod);
    StateConsts sc[C::SPT];
    float ccr[C::SPT], cci[C::SPT];
    bool ok = true;
#pragma unroll
    for (int k = 0; k < C::SPT; ++k) {
        const int j = jl + k * C::NL;
        bool okk;
        load_state_consts(sc[k], c < nvalid && j < p.N, j, i, p.N, p.B_r, p.B_theta, p.C_r, p.C_theta,
                          p.theta_bias, okk);
        ccr[k] = sc[k].mr;
        cci[k] = sc[k].mi;
        ok = ok && okk;
    }
    if (__all_sync(0xffffffffu, ok)) {
#pragma unroll
        for (int k = 0; k < C::SPT; ++k) normalise_consts(sc[k], ccr[k], cci[k]);
        bwd_warp<C, BULK, FAST, true>(p, wsm, wbar, ch0, nvalid, lane, sc, ccr, cci);
    } else {
        bwd_warp<C, BULK, FAST, false>(p, wsm, wbar, ch0, nvalid, lane, sc, ccr, cci);
    }
}

// ---------------------------------------------------------------------------
// Second stage: fixed-order sums of the per-channel partials (deterministic)
// and the polar chain rule  dr = Re(conj(G) e^{i phi}),  dphi = -Im(conj(G) w).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) reduce_param_grads_kernel(const ReduceParams p) {
    __shared__ float4 red[256];
    const int tid = threadIdx.x;
    const long long nch = (long long)p.batch * p.D;
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
        for (int b = 0; b < p.batch; ++b) acc += p.part_d[(long long)b * p.D + o];
        p.dD[o] = acc;
    } else if (p.dx_bias && o - p.D < (long long)p.D * p.N) {
        const long long e = o - p.D;
        float acc = 0.f;
        for (int b = 0; b < p.batch; ++b) acc += p.part_rowsum[(long long)b * p.D * p.N + e];
        p.dx_bias[e] = acc;
    }
}

// ---------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <class C, bool BULK, bool FAST>
cudaError_t launch_fwd_cfg(const ScanFwdParams& p, cudaStream_t stream) {
    auto kern = scan_unitary_fwd_kernel<C, BULK, FAST>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long tasks = ((long long)p.nch + C::CPW - 1) / C::CPW;
    const long long blocks = (tasks + C::WARPS - 1) / C::WARPS;
    kern<<<(unsigned)blocks, C::WARPS * 32, C::SMEM_BYTES, stream>>>(p);
    return cudaGetLastError();
}

template <class C, bool BULK, bool FAST>
cudaError_t launch_bwd_cfg(const ScanBwdParams& p, cudaStream_t stream) {
    auto kern = scan_unitary_bwd_kernel<C, BULK, FAST>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long tasks = ((long long)p.nch + C::CPW - 1) / C::CPW;
    const long long blocks = (tasks + C::WARPS - 1) / C::WARPS;
    kern<<<(unsigned)blocks, C::WARPS * 32, C::SMEM_BYTES, stream>>>(p);
    return cudaGetLastError();
}

template <class C>
cudaError_t launch_fwd_sel(const ScanFwdParams& p, bool bulk, bool fast, cudaStream_t s) {
    if (bulk) return fast ? launch_fwd_cfg<C, true, true>(p, s) : launch_fwd_cfg<C, true, false>(p, s);
    return fast ? launch_fwd_cfg<C, false, true>(p, s) : launch_fwd_cfg<C, false, false>(p, s);
}

template <class C>
cudaError_t launch_bwd_sel(const ScanBwdParams& p, bool bulk, bool fast, cudaStream_t s) {
    if (bulk) return fast ? launch_bwd_cfg<C, true, true>(p, s) : launch_bwd_cfg<C, true, false>(p, s);
    return fast ? launch_bwd_cfg<C, false, true>(p, s) : launch_bwd_cfg<C, false, false>(p, s);
}

}  // namespace

// Tile shapes per state count.  <lanes per channel, states per thread, tile
// steps, [sub-block,] stages, warps per block>.
cudaError_t launch_scan_unitary_fwd(const ScanFwdParams& p_, cudaStream_t stream) {
    if (p_.nch <= 0 || p_.L <= 0) return cudaSuccess;
    ScanFwdParams p = p_;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorInvalidSymbol;
    const ScanOptions& o = scan_options();
    const bool bulk = !o.force_plain && (p.L % 4 == 0) && (p.ld_theta % 4 == 0) && (p.ld_row % 4 == 0) &&
                      aligned16(p.theta) && aligned16(p.u) && aligned16(p.dt) && aligned16(p.z) &&
                      (p.y == nullptr || aligned16(p.y));
    const bool fast = o.fast_trig != 0;
    const int N = p.N;
    if (N <= 4) return launch_fwd_sel<FwdCfg<4, 1, 32, 3, 4>>(p, bulk, fast, stream);
    if (N <= 8) return launch_fwd_sel<FwdCfg<8, 1, 64, 3, 3>>(p, bulk, fast, stream);
    if (N <= 16) {
        if (o.variant == 1) return launch_fwd_sel<FwdCfg<8, 2, 64, 3, 3>>(p, bulk, fast, stream);
        if (o.variant == 2) return launch_fwd_sel<FwdCfg<16, 1, 128, 3, 3>>(p, bulk, fast, stream);
        if (o.variant == 3) return launch_fwd_sel<FwdCfg<16, 1, 32, 4, 5>>(p, bulk, fast, stream);
        return launch_fwd_sel<FwdCfg<16, 1, 64, 3, 3>>(p, bulk, fast, stream);
    }
    if (N <= 32) return launch_fwd_sel<FwdCfg<32, 1, 64, 3, 3>>(p, bulk, fast, stream);
    if (N <= 64) return launch_fwd_sel<FwdCfg<32, 2, 32, 3, 3>>(p, bulk, fast, stream);
    if (N <= 128) return launch_fwd_sel<FwdCfg<32, 4, 32, 3, 2>>(p, bulk, fast, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_scan_unitary_bwd(const ScanBwdParams& p_, cudaStream_t stream) {
    if (p_.nch <= 0 || p_.L <= 0) return cudaSuccess;
    ScanBwdParams p = p_;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorInvalidSymbol;
    const ScanOptions& o = scan_options();
    const bool bulk = !o.force_plain && (p.L % 4 == 0) && (p.ld_theta % 4 == 0) && (p.ld_dtheta % 4 == 0) &&
                      (p.ld_row % 4 == 0) && aligned16(p.theta) && aligned16(p.dtheta) && aligned16(p.u) &&
                      aligned16(p.dt) && aligned16(p.z) && aligned16(p.gy) && aligned16(p.du) &&
                      aligned16(p.ddt) && aligned16(p.dz);
    const bool fast = o.fast_trig != 0;
    const int N = p.N;
    if (N <= 4) return launch_bwd_sel<BwdCfg<4, 1, 32, 32, 3, 3>>(p, bulk, fast, stream);
    if (N <= 8) return launch_bwd_sel<BwdCfg<8, 1, 64, 32, 3, 2>>(p, bulk, fast, stream);
    if (N <= 16) {
        if (o.variant == 1) return launch_bwd_sel<BwdCfg<8, 2, 64, 32, 3, 3>>(p, bulk, fast, stream);
        if (o.variant == 2) return launch_bwd_sel<BwdCfg<16, 1, 128, 32, 3, 3>>(p, bulk, fast, stream);
        if (o.variant == 3) return launch_bwd_sel<BwdCfg<16, 1, 32, 32, 4, 3>>(p, bulk, fast, stream);
        return launch_bwd_sel<BwdCfg<16, 1, 64, 32, 3, 5>>(p, bulk, fast, stream);
    }
    if (N <= 32) return launch_bwd_sel<BwdCfg<32, 1, 64, 32, 3, 5>>(p, bulk, fast, stream);
    if (N <= 64) return launch_bwd_sel<BwdCfg<32, 2, 32, 32, 3, 4>>(p, bulk, fast, stream);
    if (N <= 128) return launch_bwd_sel<BwdCfg<32, 4, 32, 32, 3, 2>>(p, bulk, fast, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_reduce_param_grads(const ReduceParams& p, cudaStream_t stream) {
    const long long tail = (long long)p.D + (p.dx_bias ? (long long)p.D * p.N : 0);
    const unsigned blocks = (unsigned)(p.N + (tail + 255) / 256);
    reduce_param_grads_kernel<<<blocks, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace aussm
