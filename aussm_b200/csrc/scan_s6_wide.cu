// Real selective scan ("S6") for sm_100a, channel-per-thread kernels for up to 16 states per channel.
//
// The S6 recurrence has a constant A, so unlike the unitary and complex scans it streams no per-state exponent:
// per (b, i, t) it moves 16 bytes forward and 28 backward for N states of arithmetic, and what has to be cheap is
// the arithmetic.  Here one THREAD owns one channel and keeps all of its N states in registers; a warp (one-warp
// blocks) owns 32 channels of ONE batch entry and walks time sequentially in 16-step tiles staged by coalesced
// 16-byte asynchronous copies through a two-stage ring:
//   * B_j(t), C_j(t) are the same for every channel of a batch entry: all 32 lanes read the same shared-memory
//     address (one wavefront serves 32 channels), against one wavefront per 2 channels in the thread-per-state
//     kernels of scan_s6.cu, whose bound is the shared-memory pipe;
//   * the sum over states stays in the thread: no column-sum tiles, no second pass;
//   * dB and dC (sums over the channels of a batch entry) are added across the 32 lanes through a padded
//     shared-memory tile and leave as ONE vector atomic per state and four steps per warp of 32 channels
//     (thread-per-state: one per state, four steps and 2 channels).
// The recurrence contracts, so it cannot be run backwards: the forward kernel records the N states at every tile
// start, (channel, tile, state) with the states contiguous; the backward kernel recomputes a tile from there, keeping
// the states at every fourth step in shared memory, and then walks the tile's four-step groups in reverse, each
// group recomputed once more with the state before every step held in registers.
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

template <int NS_, bool BWD_>
struct WCfg {
    static constexpr int NS = NS_;
    static constexpr int AUX = BWD_ ? 4 : 3;                          // u, delta, z [, gout]
    static constexpr int BC_FLOATS = 2 * NS * WTP;                    // B rows then C rows
    static constexpr int AUX_FLOATS = 32 * WTP;                       // one array: a row per channel
    static constexpr int STAGE_FLOATS = BC_FLOATS + AUX * AUX_FLOATS;
    // backward only: states at every fourth step [NQ][NS][32]; lane-sum tile [2 NS][33] of four steps each
    static constexpr int SUB_FLOATS = BWD_ ? NQ * NS * 32 : 0;
    static constexpr int RED_FLOATS = BWD_ ? 2 * NS * 33 * 4 : 0;
    static constexpr size_t SMEM_BYTES = (size_t)(WSTAGES * STAGE_FLOATS + SUB_FLOATS + RED_FLOATS) * sizeof(float);
    static constexpr int BC_PIECES = (2 * NS * NQ + 31) / 32;         // 16-byte pieces per lane
    static constexpr int ROW_PIECES = 32 * NQ / 32;                   // per array
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
                    cp_async16(dst + (id / NQ) * WTP + col * 4, aux_src[a] + row_off[i] + t0);
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
            if (row < nvalid)
                *reinterpret_cast<float4*>(dst + row_off[i] + t0) = ld_shared_f4(src_rows + row * WTP + col * 4);
        }
    }
};

__device__ __forceinline__ float softplus_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

#define AUSSM_F4(v) {(v).x, (v).y, (v).z, (v).w}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
template <int NS>
__global__ void __launch_bounds__(32) s6w_fwd_kernel(const S6FwdParams p) {
    using C = WCfg<NS, false>;
    extern __shared__ __align__(128) float smem[];
    const int lane = threadIdx.x;
    const int tasks_per_batch = (p.Dmod + 31) / 32;
    const int b = blockIdx.x / tasks_per_batch, i0 = (blockIdx.x % tasks_per_batch) * 32;
    const int nvalid = min(32, p.Dmod - i0);
    const bool act = lane < nvalid;
    const int i = i0 + min(lane, nvalid - 1);
    const long long ch0 = (long long)b * p.Dmod + i0, ch = (long long)b * p.Dmod + i;
    const int N = p.N, L = p.L;
    const int ntiles = (L + WT - 1) / WT;

    float A2[NS], h[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        A2[j] = j < N ? p.A[(long long)i * N + j] * kLog2e : 0.f;
        h[j] = 0.f;
    }
    const float dskip = p.Dskip ? p.Dskip[i] : 0.f;
    const float bias = p.delta_bias ? p.delta_bias[i] : 0.f;
    const bool softplus = p.delta_softplus != 0, gate = p.z != nullptr;

    // rows of states beyond N are never copied: they must read as zero (B = C = 0 keeps such a state at zero)
    for (int k = lane; k < WSTAGES * C::STAGE_FLOATS; k += 32) smem[k] = 0.f;
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
        float* urow = st + C::BC_FLOATS + lane * WTP;
        const float* drow = urow + C::AUX_FLOATS;
        const float* zrow = drow + C::AUX_FLOATS;
        const long long t0 = (long long)tile * WT;
        const int tlen = min(WT, L - (int)t0);
        cp_async_wait<WSTAGES - 1>();
        __syncwarp();
        if (ck && act) {
#pragma unroll
            for (int j = 0; j < NS; ++j)
                if (j < N) ck[(long long)tile * N + j] = h[j];
        }
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            if (4 * q >= tlen) break;
            const float4 u4 = ld_shared_f4(urow + 4 * q), d4 = ld_shared_f4(drow + 4 * q);
            const float uv[4] = AUSSM_F4(u4), dr[4] = AUSSM_F4(d4);
            float dlt[4], s[4], y[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x = dr[e] + bias;
                dlt[e] = softplus ? softplus_(x) : x;
                s[e] = dlt[e] * uv[e];
                y[e] = dskip * uv[e];
            }
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                const float4 b4 = ld_shared_f4(st + j * WTP + 4 * q);               // same address in every lane
                const float4 c4 = ld_shared_f4(st + (NS + j) * WTP + 4 * q);
                const float bv[4] = AUSSM_F4(b4), cv[4] = AUSSM_F4(c4);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    h[j] = fmaf(ex2_ftz(dlt[e] * A2[j]), h[j], s[e] * bv[e]);
                    y[e] = fmaf(cv[e], h[j], y[e]);
                }
            }
            if (gate) {
                const float4 z4 = ld_shared_f4(zrow + 4 * q);
                const float zv[4] = AUSSM_F4(z4);
#pragma unroll
                for (int e = 0; e < 4; ++e) y[e] *= siluf_(zv[e]);
            }
            st_shared_f4(urow + 4 * q, make_float4(y[0], y[1], y[2], y[3]));        // the u cells now hold the output
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
        for (int j = 0; j < NS; ++j)
            if (j < N) p.last_state[ch * N + j] = h[j];
    }
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------
__device__ __forceinline__ void red_add_v4w(float* addr, const float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

template <int NS>
__global__ void __launch_bounds__(32) s6w_bwd_kernel(const S6BwdParams p) {
    using C = WCfg<NS, true>;
    extern __shared__ __align__(128) float smem[];
    const int lane = threadIdx.x;
    const int tasks_per_batch = (p.Dmod + 31) / 32;
    const int b = blockIdx.x / tasks_per_batch, i0 = (blockIdx.x % tasks_per_batch) * 32;
    const int nvalid = min(32, p.Dmod - i0);
    const bool act = lane < nvalid;
    const int i = i0 + min(lane, nvalid - 1);
    const long long ch0 = (long long)b * p.Dmod + i0, ch = (long long)b * p.Dmod + i;
    const int N = p.N, L = p.L;
    const int ntiles = (L + WT - 1) / WT;

    float* sub = smem + WSTAGES * C::STAGE_FLOATS;          // [NQ][NS][32]
    float* red = sub + C::SUB_FLOATS;                       // [2 NS][33] float4: gB rows, then gC rows

    float A2[NS], eps[NS], dA[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        A2[j] = j < N ? p.A[(long long)i * N + j] * kLog2e : 0.f;
        eps[j] = 0.f;       // a_{t+1} eta_{t+1}
        dA[j] = 0.f;
    }
    const float dskip = p.Dskip ? p.Dskip[i] : 0.f;
    const float bias = p.delta_bias ? p.delta_bias[i] : 0.f;
    const bool softplus = p.delta_softplus != 0, gate = p.z != nullptr;
    float dD_acc = 0.f, db_acc = 0.f;

    for (int k = lane; k < WSTAGES * C::STAGE_FLOATS; k += 32) smem[k] = 0.f;
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
    float hn[NS];                                           // state at the start of the tile taken next
#pragma unroll
    for (int j = 0; j < NS; ++j) hn[j] = j < N ? ck[(long long)(ntiles - 1) * N + j] : 0.f;
    // lane k of the lane-sum pass owns row k of the tile: dB of state k (k < NS) or dC of state k - NS
    const int rj = lane % NS;
    float* red_dst = (lane < NS ? p.dB : p.dC) + ((long long)b * N + min(rj, N - 1)) * L;
    const bool red_on = lane < 2 * NS && rj < N;

    for (int r = 0; r < ntiles; ++r) {
        const int tile = ntiles - 1 - r;
        float* st = smem + (r % WSTAGES) * C::STAGE_FLOATS;
        float* urow = st + C::BC_FLOATS + lane * WTP;
        float* drow = urow + C::AUX_FLOATS;
        float* zrow = drow + C::AUX_FLOATS;
        const float* grow = zrow + C::AUX_FLOATS;
        const long long t0 = (long long)tile * WT;
        const int tlen = min(WT, L - (int)t0);
        const int nq = tlen >> 2;
        float h[NS];
#pragma unroll
        for (int j = 0; j < NS; ++j) h[j] = hn[j];
        if (tile > 0) {
#pragma unroll
            for (int j = 0; j < NS; ++j) hn[j] = j < N ? ck[(long long)(tile - 1) * N + j] : 0.f;
        }
        cp_async_wait<WSTAGES - 1>();
        __syncwarp();

        // first pass: the states at the start of every four-step group
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            if (q >= nq) break;
#pragma unroll
            for (int j = 0; j < NS; ++j) sub[(q * NS + j) * 32 + lane] = h[j];
            if (q + 1 >= nq) break;                                   // the last group's end state is not needed
            const float4 u4 = ld_shared_f4(urow + 4 * q), d4 = ld_shared_f4(drow + 4 * q);
            const float uv[4] = AUSSM_F4(u4), dr[4] = AUSSM_F4(d4);
            float dlt[4], s[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x = dr[e] + bias;
                dlt[e] = softplus ? softplus_(x) : x;
                s[e] = dlt[e] * uv[e];
            }
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                const float4 b4 = ld_shared_f4(st + j * WTP + 4 * q);
                const float bv[4] = AUSSM_F4(b4);
#pragma unroll
                for (int e = 0; e < 4; ++e) h[j] = fmaf(ex2_ftz(dlt[e] * A2[j]), h[j], s[e] * bv[e]);
            }
        }

        // second pass: the groups in reverse
#pragma unroll 1
        for (int q = nq - 1; q >= 0; --q) {
            const float4 u4 = ld_shared_f4(urow + 4 * q), d4 = ld_shared_f4(drow + 4 * q);
            const float4 g4 = ld_shared_f4(grow + 4 * q);
            const float uv[4] = AUSSM_F4(u4), dr[4] = AUSSM_F4(d4), gv[4] = AUSSM_F4(g4);
            float zv[4] = {0.f, 0.f, 0.f, 0.f};
            if (gate) {
                const float4 z4 = ld_shared_f4(zrow + 4 * q);
                zv[0] = z4.x; zv[1] = z4.y; zv[2] = z4.z; zv[3] = z4.w;
            }
            float dlt[4], s[4], w[4], gz[4], SQ[4], SY[4], SP[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x = dr[e] + bias;
                dlt[e] = softplus ? softplus_(x) : x;
                s[e] = dlt[e] * uv[e];
                gz[e] = 0.f;
                w[e] = gate ? gv[e] * silu_and_grad(zv[e], gz[e]) : gv[e];
                if (!act) w[e] = 0.f;                 // a shadow lane adds nothing to dB / dC
                SQ[e] = SY[e] = SP[e] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                const float4 b4 = ld_shared_f4(st + j * WTP + 4 * q);
                const float4 c4 = ld_shared_f4(st + (NS + j) * WTP + 4 * q);
                const float bv[4] = AUSSM_F4(b4), cv[4] = AUSSM_F4(c4);
                float hp[4], av[4], gB[4], gC[4];
                float hj = sub[(q * NS + j) * 32 + lane];
#pragma unroll
                for (int e = 0; e < 4; ++e) {          // the state BEFORE each step of the group
                    hp[e] = hj;
                    av[e] = ex2_ftz(dlt[e] * A2[j]);
                    hj = fmaf(av[e], hj, s[e] * bv[e]);
                }
#pragma unroll
                for (int e = 3; e >= 0; --e) {
                    const float ht = fmaf(av[e], hp[e], s[e] * bv[e]);       // h_t
                    const float g = fmaf(cv[e], w[e], eps[j]);               // eta_t
                    const float qa = g * hp[e] * av[e];                      // eta_t h_{t-1} a_t
                    dA[j] = fmaf(qa, dlt[e], dA[j]);
                    SQ[e] = fmaf(qa, A2[j], SQ[e]);                          // times ln 2 below
                    SY[e] = fmaf(g, bv[e], SY[e]);
                    SP[e] = fmaf(cv[e], ht, SP[e]);
                    gB[e] = g * s[e];
                    gC[e] = w[e] * ht;
                    eps[j] = av[e] * g;
                }
                st_shared_f4(red + (j * 33 + lane) * 4, make_float4(gB[0], gB[1], gB[2], gB[3]));
                st_shared_f4(red + ((NS + j) * 33 + lane) * 4, make_float4(gC[0], gC[1], gC[2], gC[3]));
            }
            __syncwarp();
            // dB, dC: lane k adds row k over the 32 channels, one vector atomic per state and group
            if (lane < 2 * NS) {
                float4 acc = ld_shared_f4(red + (lane * 33) * 4);
#pragma unroll 8
                for (int l = 1; l < 32; ++l) {
                    const float4 v = ld_shared_f4(red + (lane * 33 + l) * 4);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                if (red_on) red_add_v4w(red_dst + t0 + 4 * q, acc);
            }
            // this lane's channel: d delta, du, dz of the group replace delta, u, z in the stage
            float dd[4], du[4], dz[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float ddl = fmaf(uv[e], SY[e], SQ[e] * kLn2);
                if (softplus) ddl *= sigmoidf_(dr[e] + bias);
                dd[e] = ddl;
                du[e] = fmaf(dlt[e], SY[e], w[e] * dskip);
                dz[e] = gv[e] * fmaf(dskip, uv[e], SP[e]) * gz[e];
                db_acc += ddl;
                dD_acc = fmaf(w[e], uv[e], dD_acc);
            }
            st_shared_f4(urow + 4 * q, make_float4(du[0], du[1], du[2], du[3]));
            st_shared_f4(drow + 4 * q, make_float4(dd[0], dd[1], dd[2], dd[3]));
            if (gate) st_shared_f4(zrow + 4 * q, make_float4(dz[0], dz[1], dz[2], dz[3]));
            __syncwarp();                                             // the lane-sum tile is free again
        }
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
        for (int j = 0; j < NS; ++j)
            if (j < N) p.part_A[ch * N + j] = dA[j];
        p.part_D[ch] = dD_acc;
        p.part_bias[ch] = db_acc;
    }
}

template <int NS>
cudaError_t launch_w_fwd(const S6FwdParams& p, cudaStream_t stream) {
    using C = WCfg<NS, false>;
    auto kern = s6w_fwd_kernel<NS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long blocks = (long long)(p.nch / p.Dmod) * ((p.Dmod + 31) / 32);
    kern<<<(unsigned)blocks, 32, C::SMEM_BYTES, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

template <int NS>
cudaError_t launch_w_bwd(const S6BwdParams& p, cudaStream_t stream) {
    using C = WCfg<NS, true>;
    auto kern = s6w_bwd_kernel<NS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const long long blocks = (long long)(p.nch / p.Dmod) * ((p.Dmod + 31) / 32);
    kern<<<(unsigned)blocks, 32, C::SMEM_BYTES, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_s6_wide_fwd(const S6FwdParams& p, cudaStream_t stream) {
    if (p.nch <= 0 || p.L <= 0) return cudaSuccess;
    if (p.N <= 4) return launch_w_fwd<4>(p, stream);
    if (p.N <= 8) return launch_w_fwd<8>(p, stream);
    if (p.N <= 16) return launch_w_fwd<16>(p, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_s6_wide_bwd(const S6BwdParams& p, cudaStream_t stream) {
    if (p.nch <= 0 || p.L <= 0) return cudaSuccess;
    if (p.N <= 4) return launch_w_bwd<4>(p, stream);
    if (p.N <= 8) return launch_w_bwd<8>(p, stream);
    if (p.N <= 16) return launch_w_bwd<16>(p, stream);
    return cudaErrorInvalidValue;
}

}  // namespace aussm
