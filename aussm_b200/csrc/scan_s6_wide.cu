// Real selective scan ("S6") for sm_100a, several-states-per-thread kernels for up to 16 states per channel.
//
// The S6 recurrence has a constant A, so unlike the unitary and complex scans it streams no per-state exponent:
// per (b, i, t) it moves 16 bytes forward and 28 backward for N states of arithmetic, and what has to be cheap is
// the arithmetic.  Here a channel is owned by LPC lanes (1, 2 or 4), each keeping NS / LPC of its states in
// registers (thread k of a channel owns states k, k + LPC, ...); a warp (one-warp blocks) owns 32 / LPC channels
// of ONE batch entry and walks time sequentially in 16-step tiles staged by coalesced 16-byte asynchronous copies
// through a two-stage ring:
//   * B_j(t), C_j(t) are the same for every channel of a batch entry: the lanes that own the same states read the
//     same shared-memory address (one wavefront per distinct address, and the LPC addresses of an instruction
//     fall into disjoint banks), against one wavefront per 2 channels in the thread-per-state kernels of
//     scan_s6.cu, whose bound is the shared-memory pipe;
//   * the sum over states is a chain in the thread plus log2(LPC) shuffles: no column-sum tiles;
//   * what depends on the channel and the step only (softplus, the gate and its derivative) is evaluated once per
//     tile by a pass in which the lanes of a channel share the tile's steps;
//   * dB and dC (sums over the channels of a batch entry) are added across the warp's channels through a padded
//     shared-memory tile and leave as one vector atomic per state and four steps.
// LPC is chosen per launch: one lane per channel is the cheapest per step, but a problem with few channels then has
// too few warps to hide the latency of its dependent chains (one warp per scheduler issues every third cycle).
// The recurrence contracts, so it cannot be run backwards: the forward kernel records the N states at every tile
// start, (channel, tile, state) with the states contiguous; the backward kernel recomputes a tile from there, keeping
// the states at every fourth step in shared memory, and then walks the tile's four-step groups in reverse, each
// group recomputed once more, state by state, with the state before every step held in registers.
//
// Same operator, arguments and gradients as scan_s6.cu (mamba_ssm.selective_scan_fn as called by
// MambaBlock.ssm_mamba, ai-modules/wavesAI/model/aussm.py:771-805); that file serves 16 < N <= 32.
#include <stdint.h>

#include "common.cuh"
#include "host_common.cuh"
#include "scan_s6.cuh"

namespace aussm {
namespace {

constexpr int WT = kS6WideTile;          // steps per tile = checkpoint interval
constexpr int WTP = WT + 4;              // row pitch: a quarter-warp's 128-bit reads of eight rows hit disjoint banks
constexpr int NQ = WT / 4;
constexpr int WSTAGES = 2;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int NS_, int LPC_, bool BWD_>
struct WCfg {
    static constexpr int NS = NS_, LPC = LPC_;
    static constexpr int SPT = NS / LPC;                              // states per thread
    static constexpr int CPW = 32 / LPC;                              // channels per warp
    static constexpr int AUX = BWD_ ? 4 : 3;                          // u, delta, z [, gout]
    static constexpr int BC_FLOATS = 2 * NS * WTP;                    // B rows then C rows
    static constexpr int AUX_FLOATS = CPW * WTP;                      // one array: a row per channel
    static constexpr int STAGE_FLOATS = BC_FLOATS + AUX * AUX_FLOATS;
    // backward only: this thread's states at every fourth step [NQ][SPT][32]; channel-sum tile of four steps each,
    // [2 NS rows][CPW + 1] (pitch odd: the row-per-lane reads hit disjoint banks)
    static constexpr int SUB_FLOATS = BWD_ ? NQ * SPT * 32 : 0;
    static constexpr int RED_PITCH = CPW + 1;
    static constexpr int RED_FLOATS = BWD_ ? 2 * NS * RED_PITCH * 4 : 0;
    static constexpr size_t SMEM_BYTES = (size_t)(WSTAGES * STAGE_FLOATS + SUB_FLOATS + RED_FLOATS) * sizeof(float);
    static constexpr int BC_PIECES = (2 * NS * NQ + 31) / 32;         // 16-byte pieces per lane
    static constexpr int ROW_PIECES = (CPW * NQ + 31) / 32;           // per array
    static constexpr int PRE_STEPS = WT / LPC;                        // steps per lane in the per-channel passes
    static_assert(NS % LPC == 0 && PRE_STEPS % 4 == 0, "shape");
};

// Tile movement.  Piece id = i * 32 + lane -> row id / NQ, 16-byte column id % NQ.
template <class C>
struct WMap {
    long long row_off[C::ROW_PIECES];      // offset (floats) of this lane's pieces in a (nch, L) array, step 0
    const float* bc_ptr[C::BC_PIECES];     // nullptr: nothing to copy (state beyond N)
    int nvalid;

    __device__ __forceinline__ void init(int lane, int nvalid_, int N, long long L, const float* Bb, const float* Cb,
                                         long long ch0) {
        nvalid = nvalid_;
#pragma unroll
        for (int i = 0; i < C::ROW_PIECES; ++i) {
            const int id = i * 32 + lane;
            const int row = id / NQ, col = id % NQ;
            row_off[i] = (ch0 + min(row, nvalid - 1)) * L + col * 4;       // rows beyond the last channel shadow it
        }
#pragma unroll
        for (int i = 0; i < C::BC_PIECES; ++i) {
            const int id = i * 32 + lane;
            const int row = id / NQ, col = id % NQ;
            bc_ptr[i] = nullptr;
            if (row < 2 * C::NS) {
                const int j = row % C::NS;
                if (j < N) bc_ptr[i] = (row < C::NS ? Bb : Cb) + (long long)j * L + col * 4;
            }
        }
    }

    __device__ __forceinline__ void issue(float* stage, const float* const* aux_src, long long t0, int tlen,
                                          int lane) const {
        const int col = lane % NQ;
        if (col * 4 < tlen) {
#pragma unroll
            for (int i = 0; i < C::BC_PIECES; ++i) {
                const int id = i * 32 + lane;
                if (bc_ptr[i] != nullptr) cp_async16(stage + (id / NQ) * WTP + col * 4, bc_ptr[i] + t0);
            }
#pragma unroll
            for (int a = 0; a < C::AUX; ++a) {
                if (aux_src[a] == nullptr) continue;
                float* dst = stage + C::BC_FLOATS + a * C::AUX_FLOATS;
#pragma unroll
                for (int i = 0; i < C::ROW_PIECES; ++i) {
                    const int id = i * 32 + lane;
                    if (id / NQ < C::CPW) cp_async16(dst + (id / NQ) * WTP + col * 4, aux_src[a] + row_off[i] + t0);
                }
            }
        }
        cp_async_commit();
    }

    // coalesced store of one array's rows (real channels only) from the stage
    __device__ __forceinline__ void store(const float* src_rows, float* dst, long long t0, int tlen, int lane) const {
        const int col = lane % NQ;
        if (col * 4 >= tlen) return;
#pragma unroll
        for (int i = 0; i < C::ROW_PIECES; ++i) {
            const int row = (i * 32 + lane) / NQ;
            if (row < nvalid && row < C::CPW)
                *reinterpret_cast<float4*>(dst + row_off[i] + t0) = ld_shared_f4(src_rows + row * WTP + col * 4);
        }
    }
};

__device__ __forceinline__ float softplus_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// sum over the LPC lanes of a channel (they are adjacent)
template <int LPC>
__device__ __forceinline__ float channel_sum(float v) {
#pragma unroll
    for (int o = 1; o < LPC; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

#define AUSSM_F4(v) {(v).x, (v).y, (v).z, (v).w}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
template <int NS, int LPC>
__global__ void __launch_bounds__(32) s6w_fwd_kernel(const S6FwdParams p) {
    using C = WCfg<NS, LPC, false>;
    constexpr int SPT = C::SPT, CPW = C::CPW;
    extern __shared__ __align__(128) float smem[];
    const int lane = threadIdx.x;
    const int c = lane / LPC, k = lane % LPC;
    const int tasks_per_batch = (p.Dmod + CPW - 1) / CPW;
    const int b = blockIdx.x / tasks_per_batch, i0 = (blockIdx.x % tasks_per_batch) * CPW;
    const int nvalid = min(CPW, p.Dmod - i0);
    const bool act = c < nvalid;
    const int i = i0 + min(c, nvalid - 1);
    const long long ch0 = (long long)b * p.Dmod + i0, ch = (long long)b * p.Dmod + i;
    const int N = p.N, L = p.L;
    const int ntiles = (L + WT - 1) / WT;

    float A2[SPT], h[SPT];
#pragma unroll
    for (int jj = 0; jj < SPT; ++jj) {
        const int j = jj * LPC + k;
        A2[jj] = j < N ? p.A[(long long)i * N + j] * kLog2e : 0.f;
        h[jj] = 0.f;
    }
    const float dskip = p.Dskip ? p.Dskip[i] : 0.f;
    const float bias = p.delta_bias ? p.delta_bias[i] : 0.f;
    const bool softplus = p.delta_softplus != 0, gate = p.z != nullptr;

    // rows of states beyond N are never copied: they must read as zero (B = C = 0 keeps such a state at zero)
    for (int x = lane; x < WSTAGES * C::STAGE_FLOATS; x += 32) smem[x] = 0.f;
    __syncwarp();

    const float* aux_src[C::AUX] = {p.u, p.delta, p.z};
    WMap<C> map;
    map.init(lane, nvalid, N, L, p.Bm + (long long)b * N * L, p.Cm + (long long)b * N * L, ch0);
    for (int s = 0; s < WSTAGES; ++s) {
        if (s < ntiles) map.issue(smem + s * C::STAGE_FLOATS, aux_src, (long long)s * WT, min(WT, L - s * WT), lane);
        else cp_async_commit();
    }
    float* ck = p.ckpt ? p.ckpt + ch * ntiles * N : nullptr;

    for (int tile = 0; tile < ntiles; ++tile) {
        float* st = smem + (tile % WSTAGES) * C::STAGE_FLOATS;
        float* urow = st + C::BC_FLOATS + c * WTP;
        float* drow = urow + C::AUX_FLOATS;
        float* zrow = drow + C::AUX_FLOATS;
        const long long t0 = (long long)tile * WT;
        const int tlen = min(WT, L - (int)t0);
        cp_async_wait<WSTAGES - 1>();
        __syncwarp();
        if (ck && act) {
#pragma unroll
            for (int jj = 0; jj < SPT; ++jj)
                if (jj * LPC + k < N) ck[(long long)tile * N + jj * LPC + k] = h[jj];
        }
        // per-channel pass: lane k of a channel takes steps [k PRE_STEPS, (k + 1) PRE_STEPS): the delta cells
        // receive dlt = softplus(delta + bias), the z cells silu(z)
#pragma unroll
        for (int x = 0; x < C::PRE_STEPS; x += 4) {
            const int t = k * C::PRE_STEPS + x;
            const float4 d4 = ld_shared_f4(drow + t);
            float dv[4] = AUSSM_F4(d4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                dv[e] += bias;
                if (softplus) dv[e] = softplus_(dv[e]);
            }
            st_shared_f4(drow + t, make_float4(dv[0], dv[1], dv[2], dv[3]));
            if (gate) {
                const float4 z4 = ld_shared_f4(zrow + t);
                st_shared_f4(zrow + t, make_float4(siluf_(z4.x), siluf_(z4.y), siluf_(z4.z), siluf_(z4.w)));
            }
        }
        __syncwarp();
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            if (4 * q >= tlen) break;
            const float4 u4 = ld_shared_f4(urow + 4 * q), d4 = ld_shared_f4(drow + 4 * q);
            const float uv[4] = AUSSM_F4(u4), dlt[4] = AUSSM_F4(d4);
            float s[4], y[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[e] = dlt[e] * uv[e];
                y[e] = 0.f;
            }
#pragma unroll
            for (int jj = 0; jj < SPT; ++jj) {
                const int j = jj * LPC + k;
                const float4 b4 = ld_shared_f4(st + j * WTP + 4 * q);               // one address per value of k
                const float4 c4 = ld_shared_f4(st + (NS + j) * WTP + 4 * q);
                const float bv[4] = AUSSM_F4(b4), cv[4] = AUSSM_F4(c4);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    h[jj] = fmaf(ex2_ftz(dlt[e] * A2[jj]), h[jj], s[e] * bv[e]);
                    y[e] = fmaf(cv[e], h[jj], y[e]);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = fmaf(dskip, uv[e], channel_sum<LPC>(y[e]));
            if (gate) {
                const float4 z4 = ld_shared_f4(zrow + 4 * q);                       // silu(z)
                y[0] *= z4.x; y[1] *= z4.y; y[2] *= z4.z; y[3] *= z4.w;
            }
            __syncwarp();                       // every lane of the channel has read the u cells
            if (k == 0) st_shared_f4(urow + 4 * q, make_float4(y[0], y[1], y[2], y[3]));   // they now hold the output
        }
        __syncwarp();
        map.store(st + C::BC_FLOATS, p.out, t0, tlen, lane);
        __syncwarp();
        const int nt = tile + WSTAGES;
        if (nt < ntiles) map.issue(st, aux_src, (long long)nt * WT, min(WT, L - nt * WT), lane);
        else cp_async_commit();
    }
    cp_async_wait<0>();
    if (act && p.last_state) {
#pragma unroll
        for (int jj = 0; jj < SPT; ++jj)
            if (jj * LPC + k < N) p.last_state[ch * N + jj * LPC + k] = h[jj];
    }
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------
__device__ __forceinline__ void red_add_v4w(float* addr, const float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

template <int NS, int LPC>
__global__ void __launch_bounds__(32) s6w_bwd_kernel(const S6BwdParams p) {
    using C = WCfg<NS, LPC, true>;
    constexpr int SPT = C::SPT, CPW = C::CPW, RP = C::RED_PITCH;
    extern __shared__ __align__(128) float smem[];
    const int lane = threadIdx.x;
    const int c = lane / LPC, k = lane % LPC;
    const int tasks_per_batch = (p.Dmod + CPW - 1) / CPW;
    const int b = blockIdx.x / tasks_per_batch, i0 = (blockIdx.x % tasks_per_batch) * CPW;
    const int nvalid = min(CPW, p.Dmod - i0);
    const bool act = c < nvalid;
    const int i = i0 + min(c, nvalid - 1);
    const long long ch0 = (long long)b * p.Dmod + i0, ch = (long long)b * p.Dmod + i;
    const int N = p.N, L = p.L;
    const int ntiles = (L + WT - 1) / WT;

    float* sub = smem + WSTAGES * C::STAGE_FLOATS;          // [NQ][SPT][32]
    float* red = sub + C::SUB_FLOATS;                       // [2 NS][RP] float4: gB rows, then gC rows

    float A2[SPT], eps[SPT], dA[SPT];
#pragma unroll
    for (int jj = 0; jj < SPT; ++jj) {
        const int j = jj * LPC + k;
        A2[jj] = j < N ? p.A[(long long)i * N + j] * kLog2e : 0.f;
        eps[jj] = 0.f;       // a_{t+1} eta_{t+1}
        dA[jj] = 0.f;
    }
    const float dskip = p.Dskip ? p.Dskip[i] : 0.f;
    const float bias = p.delta_bias ? p.delta_bias[i] : 0.f;
    const bool softplus = p.delta_softplus != 0, gate = p.z != nullptr;
    float dD_acc = 0.f, db_acc = 0.f;

    for (int x = lane; x < WSTAGES * C::STAGE_FLOATS; x += 32) smem[x] = 0.f;
    __syncwarp();

    const float* aux_src[C::AUX] = {p.u, p.delta, p.z, p.gout};
    WMap<C> map;
    map.init(lane, nvalid, N, L, p.Bm + (long long)b * N * L, p.Cm + (long long)b * N * L, ch0);
    for (int r = 0; r < WSTAGES; ++r) {
        const int tile = ntiles - 1 - r;
        if (tile >= 0)
            map.issue(smem + r * C::STAGE_FLOATS, aux_src, (long long)tile * WT, min(WT, L - tile * WT), lane);
        else cp_async_commit();
    }
    const float* ck = p.ckpt + ch * ntiles * N;
    float hn[SPT];                                          // state at the start of the tile taken next
#pragma unroll
    for (int jj = 0; jj < SPT; ++jj)
        hn[jj] = jj * LPC + k < N ? ck[(long long)(ntiles - 1) * N + jj * LPC + k] : 0.f;
    // lane r of the channel-sum pass owns row r of the tile: dB of state r (r < NS) or dC of state r - NS
    const int rj = lane % NS;
    float* red_dst = (lane < NS ? p.dB : p.dC) + ((long long)b * N + min(rj, N - 1)) * L;
    const bool red_on = lane < 2 * NS && rj < N;

    for (int r = 0; r < ntiles; ++r) {
        const int tile = ntiles - 1 - r;
        float* st = smem + (r % WSTAGES) * C::STAGE_FLOATS;
        float* urow = st + C::BC_FLOATS + c * WTP;
        float* drow = urow + C::AUX_FLOATS;
        float* zrow = drow + C::AUX_FLOATS;
        float* grow = zrow + C::AUX_FLOATS;
        const long long t0 = (long long)tile * WT;
        const int tlen = min(WT, L - (int)t0);
        const int nq = tlen >> 2;
        float h[SPT];
#pragma unroll
        for (int jj = 0; jj < SPT; ++jj) h[jj] = hn[jj];
        if (tile > 0) {
#pragma unroll
            for (int jj = 0; jj < SPT; ++jj)
                hn[jj] = jj * LPC + k < N ? ck[(long long)(tile - 1) * N + jj * LPC + k] : 0.f;
        }
        cp_async_wait<WSTAGES - 1>();
        __syncwarp();

        // per-channel pass (lane k of a channel: steps [k PRE_STEPS, (k + 1) PRE_STEPS)):
        //   delta cells <- dlt = softplus(delta + bias);  gout cells <- w = gout silu(z);  z cells <- gout silu'(z)
#pragma unroll
        for (int x = 0; x < C::PRE_STEPS; x += 4) {
            const int t = k * C::PRE_STEPS + x;
            const float4 d4 = ld_shared_f4(drow + t);
            float dv[4] = AUSSM_F4(d4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                dv[e] += bias;
                if (softplus) dv[e] = softplus_(dv[e]);
            }
            st_shared_f4(drow + t, make_float4(dv[0], dv[1], dv[2], dv[3]));
            const float4 g4 = ld_shared_f4(grow + t);
            float gv[4] = AUSSM_F4(g4);
            if (gate) {
                const float4 z4 = ld_shared_f4(zrow + t);
                const float zv[4] = AUSSM_F4(z4);
                float zz[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float gz;
                    const float sz = silu_and_grad(zv[e], gz);
                    zz[e] = gv[e] * gz;
                    gv[e] *= sz;
                }
                st_shared_f4(zrow + t, make_float4(zz[0], zz[1], zz[2], zz[3]));
            }
            if (!act) gv[0] = gv[1] = gv[2] = gv[3] = 0.f;            // a shadow channel adds nothing to dB / dC
            st_shared_f4(grow + t, make_float4(gv[0], gv[1], gv[2], gv[3]));
        }
        __syncwarp();

        // first pass: this thread's states at the start of every four-step group
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            if (q >= nq) break;
#pragma unroll
            for (int jj = 0; jj < SPT; ++jj) sub[(q * SPT + jj) * 32 + lane] = h[jj];
            if (q + 1 >= nq) break;                                   // the last group's end state is not needed
            const float4 u4 = ld_shared_f4(urow + 4 * q), d4 = ld_shared_f4(drow + 4 * q);
            const float uv[4] = AUSSM_F4(u4), dlt[4] = AUSSM_F4(d4);
            const float s[4] = {dlt[0] * uv[0], dlt[1] * uv[1], dlt[2] * uv[2], dlt[3] * uv[3]};
#pragma unroll
            for (int jj = 0; jj < SPT; ++jj) {
                const float4 b4 = ld_shared_f4(st + (jj * LPC + k) * WTP + 4 * q);
                const float bv[4] = AUSSM_F4(b4);
#pragma unroll
                for (int e = 0; e < 4; ++e) h[jj] = fmaf(ex2_ftz(dlt[e] * A2[jj]), h[jj], s[e] * bv[e]);
            }
        }

        // second pass: the groups in reverse
#pragma unroll 1
        for (int q = nq - 1; q >= 0; --q) {
            const float4 u4 = ld_shared_f4(urow + 4 * q), d4 = ld_shared_f4(drow + 4 * q);
            const float4 w4 = ld_shared_f4(grow + 4 * q);
            const float uv[4] = AUSSM_F4(u4), dlt[4] = AUSSM_F4(d4), w[4] = AUSSM_F4(w4);
            float s[4], SQ[4], SY[4], SP[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[e] = dlt[e] * uv[e];
                SQ[e] = SY[e] = SP[e] = 0.f;
            }
#pragma unroll
            for (int jj = 0; jj < SPT; ++jj) {
                const int j = jj * LPC + k;
                const float4 b4 = ld_shared_f4(st + j * WTP + 4 * q);
                const float4 c4 = ld_shared_f4(st + (NS + j) * WTP + 4 * q);
                const float bv[4] = AUSSM_F4(b4), cv[4] = AUSSM_F4(c4);
                float hp[4], av[4], gB[4], gC[4];
                float hj = sub[(q * SPT + jj) * 32 + lane];
#pragma unroll
                for (int e = 0; e < 4; ++e) {          // the state BEFORE each step of the group
                    hp[e] = hj;
                    av[e] = ex2_ftz(dlt[e] * A2[jj]);
                    hj = fmaf(av[e], hj, s[e] * bv[e]);
                }
#pragma unroll
                for (int e = 3; e >= 0; --e) {
                    const float ht = fmaf(av[e], hp[e], s[e] * bv[e]);       // h_t
                    const float g = fmaf(cv[e], w[e], eps[jj]);              // eta_t
                    const float qa = g * hp[e] * av[e];                      // eta_t h_{t-1} a_t
                    dA[jj] = fmaf(qa, dlt[e], dA[jj]);
                    SQ[e] = fmaf(qa, A2[jj], SQ[e]);                         // times ln 2 below
                    SY[e] = fmaf(g, bv[e], SY[e]);
                    SP[e] = fmaf(cv[e], ht, SP[e]);
                    gB[e] = g * s[e];
                    gC[e] = w[e] * ht;
                    eps[jj] = av[e] * g;
                }
                st_shared_f4(red + (j * RP + c) * 4, make_float4(gB[0], gB[1], gB[2], gB[3]));
                st_shared_f4(red + ((NS + j) * RP + c) * 4, make_float4(gC[0], gC[1], gC[2], gC[3]));
            }
            __syncwarp();
            // dB, dC: lane r adds row r over the warp's channels, one vector atomic per state and group
            if (lane < 2 * NS) {
                float4 acc = ld_shared_f4(red + (lane * RP) * 4);
#pragma unroll
                for (int l = 1; l < CPW; ++l) {
                    const float4 v = ld_shared_f4(red + (lane * RP + l) * 4);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                if (red_on) red_add_v4w(red_dst + t0 + 4 * q, acc);
            }
            // the channel's d delta, du, dz of the group replace delta, u, z in the stage
            float dd[4], du[4], dz[4];
            const float4 zz4 = gate ? ld_shared_f4(zrow + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);   // gout silu'(z)
            const float zz[4] = AUSSM_F4(zz4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float sy = channel_sum<LPC>(SY[e]), sq = channel_sum<LPC>(SQ[e]);
                float ddl = fmaf(uv[e], sy, sq * kLn2);
                if (softplus) ddl *= -expm1f(-dlt[e]);                // softplus'(x) = sigmoid(x) = 1 - exp(-softplus(x))
                dd[e] = ddl;
                du[e] = fmaf(dlt[e], sy, w[e] * dskip);
                if (gate) dz[e] = zz[e] * fmaf(dskip, uv[e], channel_sum<LPC>(SP[e]));
                db_acc += ddl;
                dD_acc = fmaf(w[e], uv[e], dD_acc);
            }
            __syncwarp();                       // every lane of the channel has read this group's cells
            if (k == 0) {
                st_shared_f4(urow + 4 * q, make_float4(du[0], du[1], du[2], du[3]));
                st_shared_f4(drow + 4 * q, make_float4(dd[0], dd[1], dd[2], dd[3]));
                if (gate) st_shared_f4(zrow + 4 * q, make_float4(dz[0], dz[1], dz[2], dz[3]));
            }
        }
        __syncwarp();
        map.store(st + C::BC_FLOATS, p.du, t0, tlen, lane);
        map.store(st + C::BC_FLOATS + C::AUX_FLOATS, p.ddelta, t0, tlen, lane);
        if (gate) map.store(st + C::BC_FLOATS + 2 * C::AUX_FLOATS, p.dz, t0, tlen, lane);
        __syncwarp();
        const int nr = r + WSTAGES;
        if (nr < ntiles) {
            const int nt = ntiles - 1 - nr;
            map.issue(st, aux_src, (long long)nt * WT, min(WT, L - nt * WT), lane);
        } else {
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
    if (act) {
#pragma unroll
        for (int jj = 0; jj < SPT; ++jj)
            if (jj * LPC + k < N) p.part_A[ch * N + jj * LPC + k] = dA[jj];
        if (k == 0) {
            p.part_D[ch] = dD_acc;
            p.part_bias[ch] = db_acc;
        }
    }
}

// Lanes per channel for a launch.  Forward: one is the cheapest per step; more when the channels alone give too few
// warps (about three per scheduler hide the latencies of the dependent chains).  Backward: two measured best at
// every size tried (batch 8 x 2048 channels x 4096 steps: 2.75 / 2.32 / 3.37 ms with 1 / 2 / 4 lanes; batch 32 x
// 4096 x 1024: 4.83 / 4.14 / 4.64 ms) - one lane per channel needs every register there is, four repeat the
// per-channel work of a group four times; four only when even two give less than one warp per scheduler.
int lanes_per_channel(long long batches, int D, int NS, bool bwd) {
    static int sms = 0;                                     // the GPUs of a box are alike
    if (sms <= 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            sms = n;
        else
            sms = 148;
    }
    auto warps = [&](int lpc) { return batches * ((D + 32 / lpc - 1) / (32 / lpc)); };
    if (bwd) return warps(2) < 4LL * sms ? 4 : 2;
    int lpc = 1;
    while (lpc < 4 && lpc * 2 <= NS && warps(lpc) < 12LL * sms) lpc *= 2;
    return lpc;
}

template <int NS, int LPC>
cudaError_t launch_w_fwd(const S6FwdParams& p, cudaStream_t stream) {
    using C = WCfg<NS, LPC, false>;
    auto kern = s6w_fwd_kernel<NS, LPC>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long blocks = (long long)(p.nch / p.Dmod) * ((p.Dmod + C::CPW - 1) / C::CPW);
    kern<<<(unsigned)blocks, 32, C::SMEM_BYTES, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

template <int NS, int LPC>
cudaError_t launch_w_bwd(const S6BwdParams& p, cudaStream_t stream) {
    using C = WCfg<NS, LPC, true>;
    auto kern = s6w_bwd_kernel<NS, LPC>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long blocks = (long long)(p.nch / p.Dmod) * ((p.Dmod + C::CPW - 1) / C::CPW);
    kern<<<(unsigned)blocks, 32, C::SMEM_BYTES, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

template <int NS>
cudaError_t launch_w_fwd_ns(const S6FwdParams& p, cudaStream_t stream) {
    switch (lanes_per_channel(p.nch / p.Dmod, p.Dmod, NS, false)) {
        case 4: return launch_w_fwd<NS, 4>(p, stream);
        case 2: return launch_w_fwd<NS, 2>(p, stream);
        default: return launch_w_fwd<NS, 1>(p, stream);
    }
}

template <int NS>
cudaError_t launch_w_bwd_ns(const S6BwdParams& p, cudaStream_t stream) {
    if (lanes_per_channel(p.nch / p.Dmod, p.Dmod, NS, true) == 4) return launch_w_bwd<NS, 4>(p, stream);
    return launch_w_bwd<NS, 2>(p, stream);
}

}  // namespace

cudaError_t launch_s6_wide_fwd(const S6FwdParams& p, cudaStream_t stream) {
    if (p.nch <= 0 || p.L <= 0) return cudaSuccess;
    if (p.N <= 4) return launch_w_fwd_ns<4>(p, stream);
    if (p.N <= 8) return launch_w_fwd_ns<8>(p, stream);
    if (p.N <= 16) return launch_w_fwd_ns<16>(p, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_s6_wide_bwd(const S6BwdParams& p, cudaStream_t stream) {
    if (p.nch <= 0 || p.L <= 0) return cudaSuccess;
    if (p.N <= 4) return launch_w_bwd_ns<4>(p, stream);
    if (p.N <= 8) return launch_w_bwd_ns<8>(p, stream);
    if (p.N <= 16) return launch_w_bwd_ns<16>(p, stream);
    return cudaErrorInvalidValue;
}

}  // namespace aussm
