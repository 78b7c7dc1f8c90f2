// tcgen05 / TMEM / TMA implementation of the float32-accurate GEMM used by the
// phase projection theta = x u and its two adjoints (replaces the d^2 inner
// loops of csrc/cuda/ssm_adaptive_unitary_forward.cu:83-110 and the atomics of
// ssm_adaptive_unitary_backward.cu:419-490 of the reference).
//
// Arithmetic: the three-term split  a*b ~ a_hi*b_hi + a_hi*b_lo + a_lo*b_hi  on
// FP16 parts.  split_f16 scales a tensor by the power of two S that brings its
// largest magnitude to about 2^14 and stores hi = fp16(S a), lo = fp16((S a -
// hi) 2^11): 2 x 11 significant bits over the whole float32 exponent range.
// The power-of-two scales come off exactly in the epilogue.
//
// One persistent CTA per SM walks 128 x 256 tiles of C.  Roles: warp 0 = TMA
// producer, warp 1 = MMA issuer (one lane; the warp also owns the 512-column
// TMEM allocation), warps 2-5 / 6-9 = accumulate/epilogue of the tile's left /
// right 128 columns (TMEM -> registers -> shared-memory transpose -> global).
// Per K block of 64 values and 128-column half of the tile the issuer runs, for
// each of the four K = 16 slices, one N = 256 tcgen05.mma  a_hi x [b_hi | b_lo]
// (accumulators [main | cross]) and one N = 128 tcgen05.mma  a_lo x b_hi  (cross).
//
// Shared-memory operand tiles use the 128-byte swizzle the TMA engine writes and
// the MMA descriptors expect.  K-major operand (K contiguous in memory): rows
// of 64 halves, 8-row groups 1024 B apart.  MN-major operand (row index
// contiguous): TMA boxes of 64 K-rows x 64 row-elements (8 KB) placed 8192 B
// apart along the row index, groups of 8 K-rows 1024 B apart inside a box.
//
// Every wait on an mbarrier is bounded; a wait that runs out records the reason
// in the device status word, and the CTA still frees its tensor memory.
#include "gemm_split3.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <algorithm>
#include <mutex>
#include <type_traits>

#include "../../include/aussm_b200.h"
#include "common.cuh"
#include "host_common.cuh"

namespace aussm {
namespace {

constexpr int BM = 128, BN = 256;
constexpr int BK = 64;                               // K values per block
constexpr int KROW_BYTES = BK * 2;                   // a K-major row of a block: one swizzle row (128 or 64 bytes)
constexpr int MNBOX = 64;                            // row elements per MN-major TMA box (128-byte swizzle rows)
constexpr int MNBOX_BYTES = MNBOX * 2 * BK;          // 4 KB: BK rows of 128 bytes
constexpr int STAGES = BK == 64 ? 2 : 4;
constexpr int A_TILE_BYTES = BM * BK * 2;            // one part of the A tile: 8 KB
constexpr int B_HALF_BYTES = 128 * BK * 2;           // one part of one 128-column half: 8 KB
constexpr int STAGE_BYTES = 2 * A_TILE_BYTES + 4 * B_HALF_BYTES;   // hi + lo of both operands: 48 KB
// Epilogue staging: every accumulate warp turns its 32 x 32 blocks through shared memory (pitch 33 floats, free
// of bank conflicts both ways) so that C leaves - and, with beta, enters - as whole 128-byte row pieces.
constexpr int EPI_PITCH = 33;
constexpr int EPI_WARP_FLOATS = 32 * EPI_PITCH;
constexpr int EPI_WARPS = 8;                         // per column half one warp for each TMEM lane quarter
constexpr int EPI_BYTES = EPI_WARPS * EPI_WARP_FLOATS * 4;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + EPI_BYTES;    // + slack for 1024-byte alignment
// Tensor-memory accumulation truncates instead of rounding, so a long K loop drifts (measured 3.5e-5 relative
// at K = 4096).  The K loop is therefore cut into chunks of 64 K values: each chunk accumulates from zero in
// tensor memory and the epilogue warps add the finished chunk into float32 registers (round-to-nearest).  The
// hi*hi products and the two small cross terms go to separate accumulators (adding the tiny terms must not
// cost the big sum extra truncations).  The 512 columns hold such a pair for each 128-column half of the tile,
// and the halves take turns: while the tensor core works on one half of a chunk, the epilogue warps drain the
// other.
// FP16 parts: the scaled low part is stored times 2^LO_SHIFT (see split_f16_kernel)
constexpr int LO_SHIFT = 11;
constexpr int MMA_N = 128;                           // the tile's two column halves take turns (see below)
constexpr int TMEM_COLS = 2 * BN;                    // 512: per column half a main and a cross accumulator
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);

struct GemmKernelParams {
    float* C;
    long long ldc;
    long long c_batch_stride;
    int M, N, K;
    int kbatches;      // batch entries summed inside the K loop (1 when batches are independent)
    int a_batched;     // 0: operand shared by all batch entries (batch coordinate 0)
    int b_batched;
    int beta;
    int* status;
    const unsigned* amax_a;   // FP16 parts: bit patterns of max|a|, max|b| (the parts are scaled by a power of two)
    const unsigned* amax_b;
    int c_vec;                // 1: C rows are 16-byte aligned (vector stores), 0: scalar stores
    int tiles_m, tiles_n, ntiles;   // one-CTA kernel: a CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...
};

// Power-of-two scale that brings a tensor whose largest magnitude has the bit pattern `maxbits` to about 2^14
// (FP16 overflows at 65504), and its exact inverse.
__host__ __device__ __forceinline__ int scale_exponent(unsigned maxbits) {
    const int e = (int)((maxbits >> 23) & 0xffu) - 127;      // floor(log2(max)); -127 for zero / subnormal
    int k = 14 - e;
    if (k > 100) k = 100;
    if (k < -100) k = -100;
    return k;
}
__device__ __forceinline__ float pow2f(int k) { return __uint_as_float((unsigned)(127 + k) << 23); }

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_addr(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_addr(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// One copy = both parts (hi then lo) of 128 rows of an operand for one K block: 16 KB.
template <int MN_MAJOR>
__device__ __forceinline__ void load_rows128(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int row0, int k0,
                                             int batch) {
    if (MN_MAJOR) tma_load_5d(smem_dst, map, bar, 0, k0, row0 / MNBOX, 0, batch);
    else tma_load_4d(smem_dst, map, bar, k0, row0, 0, batch);
}

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_holder, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_holder)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// streaming store: the line is not read again, so it should be the first to leave the L2
__device__ __forceinline__ void st_global_cs_f4(float* dst, const float4& v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// arrives on the mbarrier when all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}

// two 16-column loads of this warp's 32 lanes in flight, one wait
__device__ __forceinline__ void tmem_ld16_pair(uint32_t ta, uint32_t tb, float (&va)[16], float (&vb)[16]) {
    uint32_t r[16], q[16];
#define AUSSM_LD16(R, T)                                                                                          \
    asm volatile(                                                                                                 \
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "                                                                 \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"                          \
        : "=r"(R[0]), "=r"(R[1]), "=r"(R[2]), "=r"(R[3]), "=r"(R[4]), "=r"(R[5]), "=r"(R[6]), "=r"(R[7]),        \
          "=r"(R[8]), "=r"(R[9]), "=r"(R[10]), "=r"(R[11]), "=r"(R[12]), "=r"(R[13]), "=r"(R[14]), "=r"(R[15])   \
        : "r"(T)                                                                                                  \
        : "memory")
    AUSSM_LD16(r, ta);
    AUSSM_LD16(q, tb);
#undef AUSSM_LD16
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        va[i] = __uint_as_float(r[i]);
        vb[i] = __uint_as_float(q[i]);
    }
}

// Shared-memory matrix descriptors (64 bit): start address >> 4 in bits 0-13,
// leading byte offset >> 4 in bits 16-29, stride byte offset >> 4 in bits
// 32-45, descriptor version 1 in bits 46-47, 128-byte swizzle (2) in bits 61-63.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint64_t layout_type) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (layout_type << 61);
}

// descriptor of the kk-th slice (16 FP16 values of K) of an operand tile
template <int MN_MAJOR>
__device__ __forceinline__ uint64_t operand_desc(uint32_t tile_saddr, int kk) {
    if (MN_MAJOR) {
        // MN-major, 128-byte swizzle (type 2): TMA boxes of BK K-rows x 64 row-elements (4 KB) placed 4096 B
        // apart along the row index, groups of 8 K-rows 1024 B apart; a K = 16 slice is two groups
        return smem_desc(tile_saddr + kk * 2048, MNBOX_BYTES, 1024, 2);
    }
    // K-major, 64-byte swizzle (type 4): rows of 64 B (32 halves of K), 8-row groups 512 B apart; a K = 16
    // slice starts 32 B further into the row
    return smem_desc(tile_saddr + kk * 32, 16, 8 * KROW_BYTES, KROW_BYTES == 128 ? 2 : 4);
}

// Accumulation chunks.  A chunk is KC consecutive K blocks accumulated in tensor memory before the epilogue warps
// add it to their float32 registers.  The chunks of the tile's two column halves are offset by KC/2 blocks, so the
// halves never finish a chunk at the same K block: the half that starts a new chunk is issued second and its
// drain hides behind the other half's MMAs.  The first chunk of half 1 is KC + KC/2 blocks long (not KC/2): at
// the start of a tile the warps that drain are still storing the previous tile.
__device__ __forceinline__ bool half_starts(int h, int it, int kc) {
    return it == 0 || (h ? ((it % kc) == kc / 2 && it > kc / 2) : (it % kc) == 0);
}
__device__ __forceinline__ bool half_ends(int h, int it, int total, int kc) {
    return it == total - 1 || half_starts(h, it + 1, kc);
}
__device__ __forceinline__ int first_half(int it, int kc) { return (it > 0 && half_starts(0, it, kc)) ? 1 : 0; }

// Instruction descriptor of kind::f16 with float32 accumulate: c_format = 1 (bits 4-5), a/b format F16 = 0
// (bits 7-9, 10-12), a/b major (bits 15, 16), N >> 3 (bits 17-22), M >> 4 (bits 24-28).
template <int A_MN, int B_MN>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
    return (1u << 4) | ((uint32_t)A_MN << 15) | ((uint32_t)B_MN << 16) | ((uint32_t)(MMA_N >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_split3_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                   const GemmKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_holder;
    __shared__ int failed;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Persistent CTA: tile t -> (row block fastest, then column block, then independent batch entry), so that CTAs
    // running side by side share a B tile in L2.  Barrier phases, stage indices and chunk counters run on across
    // tiles: the copies and MMAs of the next tile start while the epilogue warps still store the previous one.
    const int tiles_mn = p.tiles_m * p.tiles_n;
    constexpr int CHUNK_KB = 256 / BK;                         // K blocks per accumulation chunk (256 values)
    const int kblocks = (p.K + BK - 1) / BK;
    const int total = kblocks * p.kbatches;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(&acc_full[h], 1);
            mbar_init(&acc_empty[h], EPI_WARPS / 2);
        }
        failed = 0;
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(&tmem_holder, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_holder;

    if (warp == 0) {
        // ---- TMA producer.  A stage is three copies: each tensor map covers both parts of its operand, and one
        // copy brings the hi and lo rows of 128 rows (the A tile; a 128-column half of the B tile).  clock64
        // stamps around the refill of a stage: the issuing warp is held 600-1000 cycles for the 96 KB of a stage
        // whether they go as ten copies or as three, from one lane or from several, and the data is complete
        // about 1500 cycles later - the refill of one stage takes longer than the 1536 tensor-core cycles of the
        // other, so the kernel runs at the rate the stage data arrives (about 42 bytes per cycle and SM) ----
        int g = 0;                                       // K blocks copied by this CTA so far
        bool okp = true;
        for (int t = blockIdx.x; t < p.ntiles && okp; t += gridDim.x) {
        const int zb = t / tiles_mn, m0 = ((t % tiles_mn) % p.tiles_m) * BM, n0 = ((t % tiles_mn) / p.tiles_m) * BN;
        for (int it = 0; it < total; ++it, ++g) {
            const int s = g % STAGES;
            const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
            bool w = true;
            if (lane == 0) {
                w = mbar_wait_bounded(&empty_bar[s], ph ^ 1u, p.status);
                if (!w) failed = 1;
                else mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
            }
            w = __shfl_sync(0xffffffffu, w, 0);          // also orders the copies after the arming of the barrier
            if (!w) { okp = false; break; }
            const int kb = it % kblocks;
            const int batch = zb * p.kbatches + it / kblocks;
            const int ba = p.a_batched ? batch : 0, bb = p.b_batched ? batch : 0;
            uint8_t* st = smem + s * STAGE_BYTES;
            const int k0 = kb * BK;
            // the A tile [a_hi | a_lo], then per 128-column half [b_hi | b_lo] (one N = 256 descriptor covers a half)
            if (lane == 0) load_rows128<A_MN>(st, &mapA, &full_bar[s], m0, k0, ba);
            else if (lane < 3)
                load_rows128<B_MN>(st + 2 * A_TILE_BYTES + (lane - 1) * 2 * B_HALF_BYTES, &mapB, &full_bar[s],
                                   n0 + (lane - 1) * MMA_N, k0, bb);
        }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer: per chunk of CHUNK_KB K-blocks, column half 0 then column half 1 ----
            constexpr uint32_t idesc = instr_desc<A_MN, B_MN>();                        // N = 128
            constexpr uint32_t idesc2 = idesc + ((uint32_t)(MMA_N >> 3) << 17);               // N = 256
            bool ok = true;
            int ch[2] = {0, 0};                       // chunks finished per column half
            int g = 0;                                // K blocks consumed so far
            for (int t = blockIdx.x; t < p.ntiles && ok; t += gridDim.x)
            for (int it = 0; it < total && ok; ++it, ++g) {
                const int s = g % STAGES;
                if (!mbar_wait_bounded(&full_bar[s], (uint32_t)(g / STAGES) & 1u, p.status)) { failed = 1; ok = false; break; }
                tc_fence_after();
                const uint32_t st = smem_addr(smem + s * STAGE_BYTES);
                const uint32_t a_hi = st, a_lo = st + A_TILE_BYTES;
                const int first = first_half(it, CHUNK_KB);
                for (int q = 0; q < 2 && ok; ++q) {
                    const int h = q == 0 ? first : 1 - first;
                    const bool starts = half_starts(h, it, CHUNK_KB);
                    if (starts) {
                        // the epilogue warps have taken this half's previous chunk out of tensor memory
                        if (!mbar_wait_bounded(&acc_empty[h], ((uint32_t)ch[h] & 1u) ^ 1u, p.status)) { failed = 1; ok = false; break; }
                        tc_fence_after();
                    }
                    const uint32_t acc_main = tmem_base + (uint32_t)(h * 2 * MMA_N), acc_cross = acc_main + MMA_N;
                    // [b_hi | b_lo] of this half are adjacent: a_hi meets both in one N = 256 instruction whose
                    // output columns are [main | cross] (one read of a_hi instead of two), then a_lo * b_hi
                    const uint32_t b_hi = st + 2 * A_TILE_BYTES + h * 2 * B_HALF_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        const uint64_t ah = operand_desc<A_MN>(a_hi, kk), al = operand_desc<A_MN>(a_lo, kk);
                        const uint64_t bh = operand_desc<B_MN>(b_hi, kk);
                        const uint32_t acc_flag = (starts && kk == 0) ? 0u : 1u;
                        umma_f16(acc_main, ah, bh, idesc2, acc_flag);
                        umma_f16(acc_cross, al, bh, idesc, 1u);
                    }
                    if (half_ends(h, it, total, CHUNK_KB)) {
                        umma_commit(&acc_full[h]);          // chunk of this half complete
                        ++ch[h];
                    }
                }
                umma_commit(&empty_bar[s]);                 // frees the stage when these MMAs have read it
            }
        }
    } else {
        // ---- accumulate + epilogue: warps 2..9; TMEM lane quarter = warp % 4, column half = (warp - 2) / 4.
        // The warps of a half depend on nothing the other half does: they store their half of a finished tile
        // while the tensor core works on the next one, and only have to be back when the first chunk of their
        // half of that tile is complete (four K blocks later for half 0, six for half 1).
        const int quarter = warp & 3;
        const int h = (warp - 2) >> 2;
        float acc[MMA_N];                        // scaled units (FP16 parts): the scales come off once, at the end
        const float cross_scale = pow2f(-LO_SHIFT);
        bool ok = true;
        int chn = 0;                                     // chunks drained
        // exact power-of-two scales, applied one after the other (read once: under the load of the operand
        // copies a global read takes thousands of cycles)
        const float ua = pow2f(-scale_exponent(*p.amax_a)), ub = pow2f(-scale_exponent(*p.amax_b));
        float* stg = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES) + (warp - 2) * EPI_WARP_FLOATS;
        const int rsub = lane >> 3, c4 = (lane & 7) * 4;           // coalesced phase: 4 rows x 8 quads per instruction
        const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(h * 2 * MMA_N);
        for (int t = blockIdx.x; t < p.ntiles; t += gridDim.x) {
            const int zb = t / tiles_mn, m0 = ((t % tiles_mn) % p.tiles_m) * BM, n0 = ((t % tiles_mn) / p.tiles_m) * BN;
#pragma unroll
            for (int i = 0; i < MMA_N; ++i) acc[i] = 0.f;
            for (int it = 0; it < total; ++it) {
                if (!half_ends(h, it, total, CHUNK_KB)) continue;
                // a chunk of this half is complete: add it to the registers and hand the columns back
                if (ok) ok = mbar_wait_bounded(&acc_full[h], (uint32_t)chn & 1u, p.status);
                tc_fence_after();
                if (ok) {
#pragma unroll
                    for (int part = 0; part < MMA_N / 16; ++part) {
                        float vm[16], vc[16];
                        tmem_ld16_pair(t0 + part * 16, t0 + MMA_N + part * 16, vm, vc);   // hi*hi ; hi*lo + lo*hi
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            acc[part * 16 + i] = fmaf(vc[i], cross_scale, acc[part * 16 + i] + vm[i]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[h]);            // the issuer may start this half's next chunk
                ++chn;
            }
            // The 32 x 32 blocks of the warp turn through the staging tile: lane = row on the way in, 4 rows x 128
            // bytes per instruction on the way out.
            if (ok && !failed) {
                float* cbase = p.C + (long long)zb * p.c_batch_stride;
#pragma unroll
                for (int blk = 0; blk < MMA_N / 32; ++blk) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) stg[lane * EPI_PITCH + c] = (acc[blk * 32 + c] * ua) * ub;
                    __syncwarp();
                    const int col = n0 + h * MMA_N + blk * 32 + c4;
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int rr = 4 * k + rsub;
                        const int row = m0 + quarter * 32 + rr;
                        const float* sp = stg + rr * EPI_PITCH + c4;
                        float4 o = make_float4(sp[0], sp[1], sp[2], sp[3]);
                        if (row < p.M) {
                            float* dst = cbase + (long long)row * p.ldc + col;
                            if (p.c_vec && col + 3 < p.N) {
                                if (p.beta) {
                                    const float4 cin = *reinterpret_cast<const float4*>(dst);
                                    o.x += cin.x; o.y += cin.y; o.z += cin.z; o.w += cin.w;
                                }
                                st_global_cs_f4(dst, o);           // written once, not read again by this kernel
                            } else {
                                if (col + 0 < p.N) dst[0] = o.x + (p.beta ? dst[0] : 0.f);
                                if (col + 1 < p.N) dst[1] = o.y + (p.beta ? dst[1] : 0.f);
                                if (col + 2 < p.N) dst[2] = o.z + (p.beta ? dst[2] : 0.f);
                                if (col + 3 < p.N) dst[3] = o.w + (p.beta ? dst[3] : 0.f);
                            }
                        }
                    }
                    __syncwarp();
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- hi/lo split ----------------------------------------------------------
// FP16 parts.  With S = 2^k the power of two that brings max|src| to about 2^14:
//   hi = fp16(S a),  lo = fp16((S a - hi) 2^LO_SHIFT)
// hi carries the first 11 significant bits and lo the next 11 (stored scaled up so that it stays in FP16's
// normal range); a*b ~ (hi_a hi_b + (hi_a lo_b + lo_a hi_b) 2^-LO_SHIFT) / (S_a S_b).
//
// Both passes walk the source four columns per thread.  VEC: rows of the source are 16-byte aligned and whole
// quads (one 128-bit load per thread); otherwise scalar loads with a bound check per column.  The destination
// pitch is always a multiple of 8 halves, so every thread stores its four halves as one 8-byte word; columns
// between `cols` and the pitch receive zeros (the tensor maps never read them).
template <bool VEC>
__device__ __forceinline__ float4 load_quad(const float* row, long long c, long long cols) {
    if (VEC) return *reinterpret_cast<const float4*>(row + c);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c + 0 < cols) v.x = row[c + 0];
    if (c + 1 < cols) v.y = row[c + 1];
    if (c + 2 < cols) v.z = row[c + 2];
    if (c + 3 < cols) v.w = row[c + 3];
    return v;
}

template <bool VEC>
__global__ void __launch_bounds__(256) absmax_kernel(const float* __restrict__ src, long long ld_src,
                                                     long long src_bs, long long rows, long long cols,
                                                     unsigned* __restrict__ amax) {
    const long long b = blockIdx.z;
    const long long cols4 = (cols + 3) / 4;
    const long long total = rows * cols4;
    float m = 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols4, c = (i % cols4) * 4;
        const float4 v = load_quad<VEC>(src + b * src_bs + r * ld_src, c, cols);
        m = fmaxf(fmaxf(fmaxf(m, fabsf(v.x)), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // non-negative floats order like their bit patterns; NaN / inf would only spoil a result that is spoilt anyway
    if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(amax, __float_as_uint(fminf(m, 3.0e38f)));
}

template <bool VEC>
__global__ void __launch_bounds__(256) split_f16_kernel(const float* __restrict__ src, long long ld_src,
                                                        long long src_bs, __half* __restrict__ hi,
                                                        __half* __restrict__ lo, long long ld_dst, long long dst_bs,
                                                        long long rows, long long cols,
                                                        const unsigned* __restrict__ amax) {
    const long long b = blockIdx.z;
    const long long cols4 = (cols + 3) / 4;
    const long long total = rows * cols4;
    const float S = pow2f(scale_exponent(*amax));
    const float up = pow2f(LO_SHIFT);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols4, c = (i % cols4) * 4;
        const float4 v = load_quad<VEC>(src + b * src_bs + r * ld_src, c, cols);
        const float a[4] = {v.x * S, v.y * S, v.z * S, v.w * S};
        __half h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            h[e] = __float2half_rn(a[e]);
            l[e] = __float2half_rn((a[e] - __half2float(h[e])) * up);
        }
        uint2 ph, pl;
        ph.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
        ph.y = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
        pl.x = (uint32_t)__half_as_ushort(l[0]) | ((uint32_t)__half_as_ushort(l[1]) << 16);
        pl.y = (uint32_t)__half_as_ushort(l[2]) | ((uint32_t)__half_as_ushort(l[3]) << 16);
        *reinterpret_cast<uint2*>(hi + b * dst_bs + r * ld_dst + c) = ph;
        *reinterpret_cast<uint2*>(lo + b * dst_bs + r * ld_dst + c) = pl;
    }
}

// ---- host side --------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Tensor map of a split operand (halves), both parts.  `part_stride` is the distance from the hi to the lo part
// in bytes.  K-major: dims (K, rows, part, batch), box (BK, 128, 2, 1), 64-byte swizzle.  MN-major: dims (64, K,
// rows / 64, part, batch), box (64, BK, 2, 2, 1), 128-byte swizzle: the row index is cut into the 64-element
// boxes the MMA descriptors expect, so one copy fills two boxes of each part.  Out-of-range K rows and boxes read
// as zero; the last box of an MN-major operand may reach up to 63 elements past `rows` (into the next row, or
// into the slack that split_part_halves() leaves behind the last row) - those values meet only rows or columns
// of C that are never stored.
int make_map(CUtensorMap* map, const void* base, long long part_stride, int mn_major, long long rows, long long K,
             long long ld, long long batch_stride, int batches) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return AUSSM_ECUDA;
    }
    if (part_stride <= 0 || part_stride % 16) {
        set_error("gemm_split3: the lo part must follow the hi part at a multiple of 16 bytes (distance %lld)",
                  part_stride);
        return AUSSM_EINVAL;
    }
    cuuint64_t dims[5], strides[4];
    cuuint32_t box[5], estr[5] = {1, 1, 1, 1, 1};
    const cuuint64_t esize = 2;
    const cuuint64_t bstride = (cuuint64_t)(batches > 1 ? batch_stride : 8) * esize;   // unused when batches == 1
    int rank;
    if (mn_major) {
        rank = 5;
        dims[0] = MNBOX; dims[1] = (cuuint64_t)K; dims[2] = (cuuint64_t)((rows + MNBOX - 1) / MNBOX); dims[3] = 2;
        dims[4] = (cuuint64_t)batches;
        box[0] = MNBOX; box[1] = BK; box[2] = 128 / MNBOX; box[3] = 2; box[4] = 1;
        strides[0] = (cuuint64_t)ld * esize; strides[1] = MNBOX * esize; strides[2] = (cuuint64_t)part_stride;
        strides[3] = bstride;
    } else {
        rank = 4;
        dims[0] = (cuuint64_t)K; dims[1] = (cuuint64_t)rows; dims[2] = 2; dims[3] = (cuuint64_t)batches;
        box[0] = BK; box[1] = 128; box[2] = 2; box[3] = 1;
        strides[0] = (cuuint64_t)ld * esize; strides[1] = (cuuint64_t)part_stride; strides[2] = bstride;
    }
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    (mn_major || KROW_BYTES == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d (rows=%lld K=%lld ld=%lld batches=%d mn_major=%d)", (int)r,
                  rows, K, ld, batches, mn_major);
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}

template <int A_MN, int B_MN>
int launch(const CUtensorMap* maps, const GemmKernelParams& kp, dim3 grid, cudaStream_t stream) {
    auto kern = gemm_split3_kernel<A_MN, B_MN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) {
        set_error("gemm_split3: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(maps[0], maps[1], kp);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("gemm_split3 launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    count_launch();
    return AUSSM_OK;
}

bool ok16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// SM count of the current device (cached per device ordinal)
int sm_count() {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices] = {};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
    return n;
}

}  // namespace

bool gemm_split3_supported(const SplitOperand& A, const SplitOperand& B, const float* C, const GemmShape& s) {
    if (s.M <= 0 || s.N <= 0 || s.K <= 0 || s.batches <= 0 || !C) return false;
    if (s.reduce_batches < 0 || (s.reduce_batches > 0 && s.batches % s.reduce_batches)) return false;
    if (!A.amax || !B.amax) return false;
    // the parts are rows of halves whose pitch is a multiple of 16 bytes (split_f16 writes them that way)
    if (A.ld % 8 || B.ld % 8 || A.batch_stride % 8 || B.batch_stride % 8) return false;
    if (!ok16(A.hi) || !ok16(A.lo) || !ok16(B.hi) || !ok16(B.lo)) return false;
    return encode_fn() != nullptr;
}

int gemm_split3(const SplitOperand& A, const SplitOperand& B, float* C, const GemmShape& s, cudaStream_t stream) {
    if (!gemm_split3_supported(A, B, C, s)) {
        set_error("gemm_split3: unsupported shape or alignment of the split operands (M=%d N=%d K=%d)", s.M, s.N, s.K);
        return AUSSM_EINVAL;
    }
    alignas(64) CUtensorMap maps[2];
    const int ab = A.batch_stride != 0 ? s.batches : 1, bb = B.batch_stride != 0 ? s.batches : 1;
    const long long a_ps = static_cast<const char*>(A.lo) - static_cast<const char*>(A.hi);
    const long long b_ps = static_cast<const char*>(B.lo) - static_cast<const char*>(B.hi);
    if (int rc = make_map(&maps[0], A.hi, a_ps, A.mn_major, s.M, s.K, A.ld, A.batch_stride, ab)) return rc;
    if (int rc = make_map(&maps[1], B.hi, b_ps, B.mn_major, s.N, s.K, B.ld, B.batch_stride, bb)) return rc;
    GemmKernelParams kp;
    kp.C = C; kp.ldc = s.ldc; kp.c_batch_stride = s.c_batch_stride;
    kp.M = s.M; kp.N = s.N; kp.K = s.K;
    kp.kbatches = s.reduce_batches ? s.batches / s.reduce_batches : 1;
    kp.beta = s.beta;
    kp.a_batched = A.batch_stride != 0;
    kp.b_batched = B.batch_stride != 0;
    kp.amax_a = A.amax;
    kp.amax_b = B.amax;
    kp.c_vec = (ok16(C) && s.ldc % 4 == 0 && s.c_batch_stride % 4 == 0) ? 1 : 0;
    kp.status = device_status_ptr();
    if (!kp.status) {
        set_error("gemm_split3: device status word unavailable");
        return AUSSM_ECUDA;
    }
    kp.tiles_m = (s.M + BM - 1) / BM;
    kp.tiles_n = (s.N + BN - 1) / BN;
    kp.ntiles = kp.tiles_m * kp.tiles_n * (s.reduce_batches ? s.reduce_batches : s.batches);
    const dim3 grid((unsigned)std::min(kp.ntiles, sm_count()), 1, 1);     // one persistent CTA per SM
    if (A.mn_major) return B.mn_major ? launch<1, 1>(maps, kp, grid, stream) : launch<1, 0>(maps, kp, grid, stream);
    return B.mn_major ? launch<0, 1>(maps, kp, grid, stream) : launch<0, 0>(maps, kp, grid, stream);
}

int split_f16(const float* src, long long ld_src, long long src_batch_stride, void* hi, void* lo, long long ld_dst,
              long long dst_batch_stride, long long rows, long long cols, int batches, unsigned* amax,
              cudaStream_t stream, bool have_amax) {
    if (ld_dst % 8 || dst_batch_stride % 8 || ld_dst < (cols + 3) / 4 * 4 || !ok16(hi) || !ok16(lo) || !amax) {
        set_error("split_f16: destination rows must be 16-byte aligned and hold whole quads (cols=%lld ld_dst=%lld)",
                  cols, ld_dst);
        return AUSSM_EINVAL;
    }
    const long long total = rows * ((cols + 3) / 4);
    if (total <= 0 || batches <= 0) return AUSSM_OK;
    const bool vec = cols % 4 == 0 && ld_src % 4 == 0 && src_batch_stride % 4 == 0 && ok16(src);
    cudaError_t e = have_amax ? cudaSuccess : cudaMemsetAsync(amax, 0, sizeof(unsigned), stream);
    if (e == cudaSuccess) {
        const unsigned blocks = (unsigned)std::min<long long>((total + 255) / 256, 148 * 8);
        const dim3 g1(blocks, 1, batches), g2(std::min<unsigned>(blocks * 2, 148 * 16), 1, batches);
        if (!have_amax) {
            if (vec) absmax_kernel<true><<<g1, 256, 0, stream>>>(src, ld_src, src_batch_stride, rows, cols, amax);
            else absmax_kernel<false><<<g1, 256, 0, stream>>>(src, ld_src, src_batch_stride, rows, cols, amax);
            count_launch();
        }
        __half* h = static_cast<__half*>(hi);
        __half* l = static_cast<__half*>(lo);
        if (vec)
            split_f16_kernel<true><<<g2, 256, 0, stream>>>(src, ld_src, src_batch_stride, h, l, ld_dst,
                                                            dst_batch_stride, rows, cols, amax);
        else
            split_f16_kernel<false><<<g2, 256, 0, stream>>>(src, ld_src, src_batch_stride, h, l, ld_dst,
                                                             dst_batch_stride, rows, cols, amax);
        count_launch();
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_error("split_f16 launch: %s", cudaGetErrorString(e));
        return AUSSM_ECUDA;
    }
    return AUSSM_OK;
}

}  // namespace aussm
