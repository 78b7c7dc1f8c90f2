// extern "C" entry points of libaussm_b200.so (see include/aussm_b200.h) and
// the windowed pipeline of the drop-in operators.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>

#include "../../include/aussm_b200.h"
#include "gemm_split3.cuh"
#include "projection.cuh"
#include "scan_unitary.cuh"

namespace aussm {

namespace {
thread_local std::string t_last_error;
std::atomic<int> g_window_steps{0};    // option "window_steps" (0 = automatic); process-wide, see the header
std::atomic<int> g_time_split{1};      // option "time_split" (1 = cut under-filled scans into time segments)
std::atomic<unsigned long long> g_launches{0};
}  // namespace

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }
int window_steps_option() { return g_window_steps.load(std::memory_order_relaxed); }
int time_split_option() { return g_time_split.load(std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_last_error = buf;
}

namespace {

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return AUSSM_ECUDA;
}

bool dims_ok(int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) {
        set_error("sizes must be positive (B=%d D=%d N=%d L=%d)", B, D, N, L);
        return false;
    }
    if (N > AUSSM_MAX_STATES) {
        set_error("N=%d states per channel exceeds the supported maximum of %d", N, AUSSM_MAX_STATES);
        return false;
    }
    if ((long long)B * D > 0x7fffffffLL) {
        set_error("B*D=%lld channels exceed the 32-bit channel count", (long long)B * D);
        return false;
    }
    return true;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- workspace layout of the drop-in pipeline ----
struct Plan {
    long long rows;      // B*D*N
    int window;          // steps per window
    long long ldw;       // row pitch of the window (floats)
    size_t off_theta, off_h, off_gh, off_part, off_proj, off_split, total;   // byte offsets
    int nseg_fwd, nseg_bwd;   // time-axis split of the scans inside a window (1: none)
};

Plan make_plan(int B, int D, int N, int L, int window_steps = window_steps_option()) {
    Plan p;
    p.rows = (long long)B * D * N;
    const long long Lp = ((long long)L + 7) / 8 * 8;
    long long w;
    if (window_steps > 0) {
        w = ((long long)window_steps + 63) / 64 * 64;
    } else {
        // about 2 GiB of phases per window, at least 64 and at most 16384 steps (longer windows: fewer, better
        // filled launches; measured 138 -> 132 ms on the end-to-end benchmark step against 4096-step windows)
        w = ((1LL << 29) / p.rows) / 64 * 64;
        w = std::max(64LL, std::min(16384LL, w));
    }
    if (w >= Lp) w = Lp;
    p.window = (int)w;
    p.ldw = w;
    size_t off = 0;
    p.off_theta = off;
    off = align_up(off + (size_t)p.rows * p.ldw * 4, 256);
    p.off_h = off;       // re, im
    off = align_up(off + (size_t)p.rows * 2 * 4, 256);
    p.off_gh = off;      // re, im
    off = align_up(off + (size_t)p.rows * 2 * 4, 256);
    // Few channels (small batch x d_inner) leave most of the GPU idle in a scan that is sequential in time:
    // the scans of a window are then cut into segments (only when all windows have the same length, so that
    // the per-segment partial sums of the backward pass line up from window to window).
    const long long nch = (long long)B * D;
    const bool equal_windows = (L % p.window) == 0;
    p.nseg_fwd = equal_windows ? scan_split_segments(nch, N, p.window, false) : 1;
    p.nseg_bwd = equal_windows ? scan_split_segments(nch, N, p.window, true) : 1;
    p.off_part = off;
    off = align_up(off + scan_bwd_partial_floats(nch * p.nseg_bwd, N) * 4, 256);
    p.off_proj = off;    // FP16 hi/lo parts of x, of the u window and of the dtheta window
    off = align_up(off + proj_scratch_bytes(B, D, (long long)D * N, p.ldw), 256);
    p.off_split = off;
    const size_t split_floats = std::max(p.nseg_fwd > 1 ? scan_split_fwd_scratch_floats(nch, p.nseg_fwd, N) : 0,
                                         p.nseg_bwd > 1 ? scan_split_bwd_scratch_floats(nch, p.nseg_bwd, N) : 0);
    off = align_up(off + split_floats * 4, 256);
    p.total = off;
    return p;
}

// The layout of a kept-phase buffer (window length and row pitch) follows from the plan of the forward call,
// which depends on the "window_steps" option.  The forward call notes the layout it used under
// the buffer's address (host side, no device traffic); the backward call refuses a buffer that it finds noted
// with another layout, so a changed option between the two calls is an error instead of wrong gradients.
struct KeepLayout {
    int window;
    long long ldw, rows;
};
std::mutex g_keep_mutex;
std::unordered_map<const void*, KeepLayout> g_keep_layouts;

size_t keep_bytes_of(const Plan& pl, int L) {
    const size_t nwin = (size_t)((L + pl.window - 1) / pl.window);
    return align_up(nwin * (size_t)pl.rows * pl.ldw * sizeof(float), 256);
}

void keep_note_layout(const void* keep, const Plan& pl) {
    std::lock_guard<std::mutex> lock(g_keep_mutex);
    g_keep_layouts[keep] = KeepLayout{pl.window, pl.ldw, pl.rows};
}

// consumes the note (the backward call overwrites the phases: a buffer serves one backward call)
int keep_check_layout(const void* keep, const Plan& pl) {
    std::lock_guard<std::mutex> lock(g_keep_mutex);
    auto it = g_keep_layouts.find(keep);
    if (it == g_keep_layouts.end()) return AUSSM_OK;        // written by another process image or already consumed
    const KeepLayout k = it->second;
    g_keep_layouts.erase(it);
    if (k.window != pl.window || k.ldw != pl.ldw || k.rows != pl.rows) {
        set_error("unitary_bwd_kept: the phase buffer was written with another layout (window %d, pitch %lld) than "
                  "this call uses (window %d, pitch %lld): the window_steps option changed between forward and "
                  "backward", k.window, k.ldw, pl.window, pl.ldw);
        return AUSSM_EINVAL;
    }
    return AUSSM_OK;
}

bool keep_ok(const char* who, const void* keep, size_t keep_bytes, const Plan& pl, int L) {
    if (!keep) return true;
    const size_t need = keep_bytes_of(pl, L);
    if (keep_bytes < need || (reinterpret_cast<uintptr_t>(keep) & 255u)) {
        set_error("%s: phase buffer of %zu bytes (256-byte aligned) required, got %zu", who, need, keep_bytes);
        return false;
    }
    return true;
}

struct OpArgs {
    const float *u, *dt, *x, *x_bias, *B_r, *B_theta, *C_r, *C_theta, *Dskip, *z;
    int B, D, N, L;
};

// Forward over all windows.  y == nullptr: state only.  The final state goes
// to (out_re, out_im), which may be the workspace pair itself.
// keep != nullptr: every window's phases go to their own slice of keep
// (window w at keep + w * rows * ldw) instead of the one window of the workspace.
int run_unitary_fwd(const OpArgs& a, const float* h0_re, const float* h0_im, float* y, float* out_re,
                    float* out_im, char* ws, const Plan& pl, ProjScratch& ps, cudaStream_t stream,
                    float* keep = nullptr) {
    float* theta_w = reinterpret_cast<float*>(ws + pl.off_theta);
    float* cur_re = reinterpret_cast<float*>(ws + pl.off_h);
    float* cur_im = cur_re + pl.rows;
    const int nwin = (a.L + pl.window - 1) / pl.window;
    for (int w = 0; w < nwin; ++w) {
        const long long t0 = (long long)w * pl.window;
        const int tl = (int)std::min<long long>(pl.window, a.L - t0);
        const ProjDims pd = {a.B, a.D, (long long)a.D * a.N, a.L, pl.ldw, t0, tl};
        if (keep) theta_w = keep + (size_t)w * pl.rows * pl.ldw;
        if (int rc = proj_theta(pd, a.u, theta_w, ps, stream)) return rc;
        const bool last = (w == nwin - 1);
        ScanFwdParams sp = {};
        sp.theta = theta_w;
        sp.theta_bias = a.x_bias;
        sp.u = a.u + t0;
        sp.dt = a.dt + t0;
        sp.z = a.z + t0;
        sp.B_r = a.B_r; sp.B_theta = a.B_theta; sp.C_r = a.C_r; sp.C_theta = a.C_theta; sp.Dskip = a.Dskip;
        sp.h0_re = (w == 0) ? h0_re : cur_re;
        sp.h0_im = (w == 0) ? h0_im : cur_im;
        sp.y = y ? y + t0 : nullptr;
        sp.h1_re = last ? out_re : cur_re;
        sp.h1_im = last ? out_im : cur_im;
        sp.nch = a.B * a.D; sp.Dmod = a.D; sp.N = a.N; sp.L = tl;
        sp.ld_theta = pl.ldw;
        sp.ld_row = a.L;
        cudaError_t e;
        if (pl.nseg_fwd > 1 && scan_split_allowed(sp))
            e = scan_unitary_fwd_split(sp, pl.nseg_fwd, reinterpret_cast<float*>(ws + pl.off_split), stream);
        else
            e = launch_scan_unitary_fwd(sp, stream);
        if (e != cudaSuccess) return cuda_fail(e, "unitary scan forward launch");
    }
    return AUSSM_OK;
}

}  // namespace
}  // namespace aussm

using namespace aussm;

extern "C" {

int aussm_b200_version(void) { return 100; }

const char* aussm_b200_last_error(void) { return t_last_error.c_str(); }

int aussm_b200_device_status(aussm_stream_t stream) {
    int v = 0;
    cudaError_t e = read_and_clear_device_status((cudaStream_t)stream, &v);
    if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
    if (v != 0) set_error("a kernel gave up waiting for a bulk copy (device status %d)", v);
    return v;
}

unsigned long long aussm_b200_kernel_launches(void) { return launch_count(); }

int aussm_b200_set_option(const char* name, int value) {
    if (!name) return AUSSM_EINVAL;
    if (!strcmp(name, "window_steps")) {
        g_window_steps.store(value > 0 ? value : 0, std::memory_order_relaxed);
        return AUSSM_OK;
    }
    if (!strcmp(name, "time_split")) {
        g_time_split.store(value != 0 ? 1 : 0, std::memory_order_relaxed);
        return AUSSM_OK;
    }
    set_error("unknown option '%s'", name);
    return AUSSM_EINVAL;
}

int aussm_b200_scan_unitary_fwd(const float* theta, const float* u, const float* dt, const float* z,
                                const float* B_r, const float* B_theta, const float* C_r, const float* C_theta,
                                const float* Dskip, const float* h0_re, const float* h0_im, float* y, float* h1_re,
                                float* h1_im, int B, int D, int N, int L, aussm_stream_t stream) {
    if (!dims_ok(B, D, N, L)) return AUSSM_EINVAL;
    if (!theta || !u || !dt || !z || !B_r || !B_theta || !C_r || !C_theta || !Dskip || !y) {
        set_error("scan_unitary_fwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if ((h0_re == nullptr) != (h0_im == nullptr) || (h1_re == nullptr) != (h1_im == nullptr)) {
        set_error("scan_unitary_fwd: real and imaginary state pointers must be given together");
        return AUSSM_EINVAL;
    }
    ScanFwdParams p = {};
    p.theta = theta; p.theta_bias = nullptr; p.u = u; p.dt = dt; p.z = z;
    p.B_r = B_r; p.B_theta = B_theta; p.C_r = C_r; p.C_theta = C_theta; p.Dskip = Dskip;
    p.h0_re = h0_re; p.h0_im = h0_im; p.y = y; p.h1_re = h1_re; p.h1_im = h1_im;
    p.nch = B * D; p.Dmod = D; p.N = N; p.L = L; p.ld_theta = L; p.ld_row = L;
    cudaError_t e = launch_scan_unitary_fwd(p, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "unitary scan forward launch");
    return AUSSM_OK;
}

size_t aussm_b200_scan_unitary_fwd_workspace_bytes(int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) return 0;
    const int nseg = scan_split_segments((long long)B * D, N, L, false);
    return nseg > 1 ? align_up(scan_split_fwd_scratch_floats((long long)B * D, nseg, N) * sizeof(float), 256) : 0;
}

int aussm_b200_scan_unitary_fwd_ws(const float* theta, const float* u, const float* dt, const float* z,
                                   const float* B_r, const float* B_theta, const float* C_r, const float* C_theta,
                                   const float* Dskip, const float* h0_re, const float* h0_im, float* y, float* h1_re,
                                   float* h1_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                                   aussm_stream_t stream) {
    const size_t need = aussm_b200_scan_unitary_fwd_workspace_bytes(B, D, N, L);
    if (need == 0)
        return aussm_b200_scan_unitary_fwd(theta, u, dt, z, B_r, B_theta, C_r, C_theta, Dskip, h0_re, h0_im, y, h1_re,
                                           h1_im, B, D, N, L, stream);
    if (!dims_ok(B, D, N, L)) return AUSSM_EINVAL;
    if (!theta || !u || !dt || !z || !B_r || !B_theta || !C_r || !C_theta || !Dskip || !y) {
        set_error("scan_unitary_fwd_ws: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if ((h0_re == nullptr) != (h0_im == nullptr) || (h1_re == nullptr) != (h1_im == nullptr)) {
        set_error("scan_unitary_fwd_ws: real and imaginary state pointers must be given together");
        return AUSSM_EINVAL;
    }
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15u)) {
        set_error("scan_unitary_fwd_ws: workspace of %zu bytes (16-byte aligned) required, got %zu", need,
                  workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    ScanFwdParams p = {};
    p.theta = theta; p.theta_bias = nullptr; p.u = u; p.dt = dt; p.z = z;
    p.B_r = B_r; p.B_theta = B_theta; p.C_r = C_r; p.C_theta = C_theta; p.Dskip = Dskip;
    p.h0_re = h0_re; p.h0_im = h0_im; p.y = y; p.h1_re = h1_re; p.h1_im = h1_im;
    p.nch = B * D; p.Dmod = D; p.N = N; p.L = L; p.ld_theta = L; p.ld_row = L;
    const int nseg = scan_split_segments((long long)B * D, N, L, false);
    cudaError_t e = scan_split_allowed(p) ? scan_unitary_fwd_split(p, nseg, static_cast<float*>(workspace),
                                                                   (cudaStream_t)stream)
                                          : launch_scan_unitary_fwd(p, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "unitary scan forward launch");
    return AUSSM_OK;
}

// backward workspace: the per-channel partial sums (one set per segment when the time axis is split), then
// the scratch of the split
namespace {
int bwd_segments(int B, int D, int N, int L) { return scan_split_segments((long long)B * D, N, L, true); }
}  // namespace

size_t aussm_b200_scan_unitary_bwd_workspace_bytes(int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0) return 0;
    const long long nch = (long long)B * D;
    const int nseg = L > 0 ? bwd_segments(B, D, N, L) : 1;
    size_t bytes = align_up(scan_bwd_partial_floats(nch * nseg, N) * sizeof(float), 256);
    if (nseg > 1) bytes += align_up(scan_split_bwd_scratch_floats(nch, nseg, N) * sizeof(float), 256);
    return bytes;
}

int aussm_b200_scan_unitary_bwd(const float* grad_y, const float* gh1_re, const float* gh1_im, const float* theta,
                                const float* u, const float* dt, const float* z, const float* B_r,
                                const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                                const float* h1_re, const float* h1_im, float* dtheta, float* du, float* ddt,
                                float* dz, float* dB_r, float* dB_theta, float* dC_r, float* dC_theta, float* dD,
                                float* dh0_re, float* dh0_im, int B, int D, int N, int L, void* workspace,
                                size_t workspace_bytes, aussm_stream_t stream) {
    if (!dims_ok(B, D, N, L)) return AUSSM_EINVAL;
    if (!grad_y || !theta || !u || !dt || !z || !B_r || !B_theta || !C_r || !C_theta || !Dskip || !h1_re ||
        !h1_im || !dtheta || !du || !ddt || !dz || !dB_r || !dB_theta || !dC_r || !dC_theta || !dD) {
        set_error("scan_unitary_bwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if ((gh1_re == nullptr) != (gh1_im == nullptr) || (dh0_re == nullptr) != (dh0_im == nullptr)) {
        set_error("scan_unitary_bwd: real and imaginary state pointers must be given together");
        return AUSSM_EINVAL;
    }
    const size_t need = aussm_b200_scan_unitary_bwd_workspace_bytes(B, D, N, L);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15u)) {
        set_error("scan_unitary_bwd: workspace of %zu bytes (16-byte aligned) required, got %zu", need,
                  workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    const long long nch = (long long)B * D;
    ScanBwdParams p = {};
    p.theta = theta; p.dtheta = dtheta; p.u = u; p.dt = dt; p.z = z; p.gy = grad_y; p.du = du; p.ddt = ddt; p.dz = dz;
    p.L = L; p.ld_theta = L; p.ld_dtheta = L; p.ld_row = L;
    int nseg = bwd_segments(B, D, N, L);
    if (nseg > 1 && !scan_split_allowed(p)) nseg = 1;
    float* part_bc = static_cast<float*>(workspace);
    float* part_d = part_bc + nch * nseg * N * 4;
    float* split_scratch = reinterpret_cast<float*>(
        static_cast<char*>(workspace) + align_up(scan_bwd_partial_floats(nch * bwd_segments(B, D, N, L), N) * sizeof(float), 256));
    p.theta = theta; p.theta_bias = nullptr; p.u = u; p.dt = dt; p.z = z; p.gy = grad_y;
    p.B_r = B_r; p.B_theta = B_theta; p.C_r = C_r; p.C_theta = C_theta; p.Dskip = Dskip;
    p.h1_re = h1_re; p.h1_im = h1_im; p.gh1_re = gh1_re; p.gh1_im = gh1_im;
    p.dtheta = dtheta; p.du = du; p.ddt = ddt; p.dz = dz; p.dh0_re = dh0_re; p.dh0_im = dh0_im;
    p.h0_re = nullptr; p.h0_im = nullptr;
    p.part_bc = part_bc; p.part_d = part_d; p.part_rowsum = nullptr; p.accumulate = 0;
    p.nch = (int)nch; p.Dmod = D; p.N = N; p.L = L; p.ld_theta = L; p.ld_dtheta = L; p.ld_row = L;
    cudaError_t e = nseg > 1 ? scan_unitary_bwd_split(p, nseg, split_scratch, (cudaStream_t)stream)
                             : launch_scan_unitary_bwd(p, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "unitary scan backward launch");
    ReduceParams r = {};
    r.part_bc = part_bc; r.part_d = part_d; r.part_rowsum = nullptr;
    r.B_r = B_r; r.B_theta = B_theta; r.C_r = C_r; r.C_theta = C_theta;
    r.dB_r = dB_r; r.dB_theta = dB_theta; r.dC_r = dC_r; r.dC_theta = dC_theta; r.dD = dD; r.dx_bias = nullptr;
    r.batch = B; r.D = D; r.N = N; r.nseg = nseg;
    e = launch_reduce_param_grads(r, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "parameter-gradient reduction launch");
    return AUSSM_OK;
}

// packed operands: K-major = (rows, K) with K contiguous; MN-major = (K, rows) with rows contiguous
namespace {
struct PackedDims { long long rows, cols, pitch; };
PackedDims packed_dims(int mn_major, int rows_mn, int K) {
    PackedDims p;
    p.rows = mn_major ? K : rows_mn;
    p.cols = mn_major ? rows_mn : K;
    p.pitch = (p.cols + 7) / 8 * 8;         // halves: rows of the FP16 parts start 16-byte aligned
    return p;
}
}  // namespace

size_t aussm_b200_gemm_split3_workspace_bytes(int M, int N, int K, int batches, int a_mn_major, int a_batched,
                                              int b_mn_major, int b_batched) {
    if (M <= 0 || N <= 0 || K <= 0 || batches <= 0) return 0;
    const PackedDims a = packed_dims(a_mn_major, M, K), b = packed_dims(b_mn_major, N, K);
    const size_t na = split_part_halves((size_t)a.rows * a.pitch * (a_batched ? batches : 1));
    const size_t nb = split_part_halves((size_t)b.rows * b.pitch * (b_batched ? batches : 1));
    return 2 * (na + nb) * 2 + 1024;
}

int aussm_b200_gemm_split3_strided(const float* A, int a_mn_major, long long lda, long long a_batch_stride,
                                   const float* Bm, int b_mn_major, long long ldb, long long b_batch_stride, float* C,
                                   long long ldc, long long c_batch_stride, int M, int N, int K, int batches,
                                   int reduce_batches, int beta, void* workspace, size_t workspace_bytes,
                                   aussm_stream_t stream_) {
    if (!A || !Bm || !C || M <= 0 || N <= 0 || K <= 0 || batches <= 0) {
        set_error("gemm_split3: null pointer or non-positive size");
        return AUSSM_EINVAL;
    }
    const int a_batched = a_batch_stride != 0, b_batched = b_batch_stride != 0;
    const size_t need = aussm_b200_gemm_split3_workspace_bytes(M, N, K, batches, a_mn_major, a_batched, b_mn_major,
                                                               b_batched);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u)) {
        set_error("gemm_split3: workspace of %zu bytes (256-byte aligned) required, got %zu", need, workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    const PackedDims a = packed_dims(a_mn_major, M, K), b = packed_dims(b_mn_major, N, K);
    if (lda < a.cols || ldb < b.cols || ldc < N) {
        set_error("gemm_split3: a pitch is shorter than its row (lda=%lld ldb=%lld ldc=%lld)", lda, ldb, ldc);
        return AUSSM_EINVAL;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    const int na = a_batched ? batches : 1, nb = b_batched ? batches : 1;
    const size_t a_halves = split_part_halves((size_t)a.rows * a.pitch * na);
    const size_t b_halves = split_part_halves((size_t)b.rows * b.pitch * nb);
    char* w = static_cast<char*>(workspace);
    void* a_hi = w;
    void* a_lo = w + a_halves * 2;
    void* b_hi = w + a_halves * 4;
    void* b_lo = w + a_halves * 4 + b_halves * 2;
    unsigned* amax = reinterpret_cast<unsigned*>(w + a_halves * 4 + b_halves * 4);   // in the spare 1 KiB
    if (int rc = split_f16(A, lda, a_batch_stride, a_hi, a_lo, a.pitch, a.rows * a.pitch, a.rows, a.cols, na,
                           amax + 0, stream))
        return rc;
    if (int rc = split_f16(Bm, ldb, b_batch_stride, b_hi, b_lo, b.pitch, b.rows * b.pitch, b.rows, b.cols, nb,
                           amax + 1, stream))
        return rc;
    const SplitOperand sa = {a_hi, a_lo, a_mn_major, a.pitch, a_batched ? a.rows * a.pitch : 0, amax + 0};
    const SplitOperand sb = {b_hi, b_lo, b_mn_major, b.pitch, b_batched ? b.rows * b.pitch : 0, amax + 1};
    const GemmShape shape = {M, N, K, batches, reduce_batches ? 1 : 0, beta, ldc, reduce_batches ? 0 : c_batch_stride};
    return gemm_split3(sa, sb, C, shape, stream);
}

int aussm_b200_gemm_split3(const float* A, int a_mn_major, int a_batched, const float* Bm, int b_mn_major,
                           int b_batched, float* C, int M, int N, int K, int batches, int reduce_batches, int beta,
                           void* workspace, size_t workspace_bytes, aussm_stream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) {
        set_error("gemm_split3: null pointer or non-positive size");
        return AUSSM_EINVAL;
    }
    const PackedDims a = packed_dims(a_mn_major, M, K), b = packed_dims(b_mn_major, N, K);
    return aussm_b200_gemm_split3_strided(A, a_mn_major, a.cols, a_batched ? a.rows * a.cols : 0, Bm, b_mn_major, b.cols,
                                          b_batched ? b.rows * b.cols : 0, C, N, (long long)M * N, M, N, K, batches,
                                          reduce_batches, beta, workspace, workspace_bytes, stream);
}

size_t aussm_b200_unitary_workspace_bytes(int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) return 0;
    return make_plan(B, D, N, L).total;
}

static int unitary_fwd_impl(const float* u, const float* dt, const float* x, const float* x_bias, const float* B_r,
                            const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                            const float* z, const float* h0_re, const float* h0_im, float* y, float* h1_re,
                            float* h1_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                            aussm_stream_t stream, void* keep, size_t keep_bytes) {
    if (!dims_ok(B, D, N, L)) return AUSSM_EINVAL;
    if (!u || !dt || !x || !x_bias || !B_r || !B_theta || !C_r || !C_theta || !Dskip || !z || !y) {
        set_error("unitary_fwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if ((h0_re == nullptr) != (h0_im == nullptr) || (h1_re == nullptr) != (h1_im == nullptr)) {
        set_error("unitary_fwd: real and imaginary state pointers must be given together");
        return AUSSM_EINVAL;
    }
    const Plan pl = make_plan(B, D, N, L);
    if (!workspace || workspace_bytes < pl.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) {
        set_error("unitary_fwd: workspace of %zu bytes (256-byte aligned) required, got %zu", pl.total,
                  workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    if (!keep_ok("unitary_fwd_keep", keep, keep_bytes, pl, L)) return AUSSM_EWORKSPACE;
    char* ws = static_cast<char*>(workspace);
    float* cur_re = reinterpret_cast<float*>(ws + pl.off_h);
    const OpArgs a = {u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, Dskip, z, B, D, N, L};
    ProjScratch ps;
    proj_scratch_bind(ps, ws + pl.off_proj, B, D, (long long)D * N, pl.ldw);
    if (int rc = proj_begin(D, (long long)D * N, x, ps, (cudaStream_t)stream)) return rc;
    if (keep) keep_note_layout(keep, pl);
    return run_unitary_fwd(a, h0_re, h0_im, y, h1_re ? h1_re : cur_re, h1_im ? h1_im : cur_re + pl.rows, ws, pl, ps,
                           (cudaStream_t)stream, static_cast<float*>(keep));
}

int aussm_b200_unitary_fwd(const float* u, const float* dt, const float* x, const float* x_bias, const float* B_r,
                           const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                           const float* z, const float* h0_re, const float* h0_im, float* y, float* h1_re,
                           float* h1_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                           aussm_stream_t stream) {
    return unitary_fwd_impl(u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, Dskip, z, h0_re, h0_im, y, h1_re, h1_im, B,
                            D, N, L, workspace, workspace_bytes, stream, nullptr, 0);
}

size_t aussm_b200_unitary_keep_bytes(int B, int D, int N, int L) {
    if (B <= 0 || D <= 0 || N <= 0 || L <= 0) return 0;
    return keep_bytes_of(make_plan(B, D, N, L), L);
}

int aussm_b200_unitary_fwd_keep(const float* u, const float* dt, const float* x, const float* x_bias,
                                const float* B_r, const float* B_theta, const float* C_r, const float* C_theta,
                                const float* Dskip, const float* z, const float* h0_re, const float* h0_im, float* y,
                                float* h1_re, float* h1_im, int B, int D, int N, int L, void* workspace,
                                size_t workspace_bytes, void* theta_keep, size_t keep_bytes, aussm_stream_t stream) {
    if (!theta_keep) {
        set_error("unitary_fwd_keep: null phase buffer");
        return AUSSM_EINVAL;
    }
    return unitary_fwd_impl(u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, Dskip, z, h0_re, h0_im, y, h1_re, h1_im, B,
                            D, N, L, workspace, workspace_bytes, stream, theta_keep, keep_bytes);
}

static int unitary_bwd_impl(const float* grad_y, const float* gh1_re, const float* gh1_im, const float* u,
                            const float* dt, const float* x, const float* x_bias, const float* B_r,
                            const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                            const float* z, const float* h0_re, const float* h0_im, const float* h1_re,
                            const float* h1_im, float* du, float* ddt, float* dx, float* dx_bias, float* dB_r,
                            float* dB_theta, float* dC_r, float* dC_theta, float* dD, float* dz, float* dh0_re,
                            float* dh0_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                            aussm_stream_t stream_, void* keep_buf, size_t keep_bytes) {
    if (!dims_ok(B, D, N, L)) return AUSSM_EINVAL;
    if (!grad_y || !u || !dt || !x || !x_bias || !B_r || !B_theta || !C_r || !C_theta || !Dskip || !z || !du ||
        !ddt || !dx || !dx_bias || !dB_r || !dB_theta || !dC_r || !dC_theta || !dD || !dz) {
        set_error("unitary_bwd: null input or output pointer");
        return AUSSM_EINVAL;
    }
    if ((gh1_re == nullptr) != (gh1_im == nullptr) || (dh0_re == nullptr) != (dh0_im == nullptr) ||
        (h0_re == nullptr) != (h0_im == nullptr) || (h1_re == nullptr) != (h1_im == nullptr)) {
        set_error("unitary_bwd: real and imaginary state pointers must be given together");
        return AUSSM_EINVAL;
    }
    const Plan pl = make_plan(B, D, N, L);
    if (!workspace || workspace_bytes < pl.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) {
        set_error("unitary_bwd: workspace of %zu bytes (256-byte aligned) required, got %zu", pl.total,
                  workspace_bytes);
        return AUSSM_EWORKSPACE;
    }
    if (!keep_ok("unitary_bwd_kept", keep_buf, keep_bytes, pl, L)) return AUSSM_EWORKSPACE;
    float* keep = static_cast<float*>(keep_buf);
    if (keep && !h1_re) {
        set_error("unitary_bwd_kept: the final state of the forward call is required with kept phases");
        return AUSSM_EINVAL;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    char* ws = static_cast<char*>(workspace);
    float* theta_w = reinterpret_cast<float*>(ws + pl.off_theta);
    float* cur_re = reinterpret_cast<float*>(ws + pl.off_h);
    float* cur_im = cur_re + pl.rows;
    float* g_re = reinterpret_cast<float*>(ws + pl.off_gh);
    float* g_im = g_re + pl.rows;
    const long long nch = (long long)B * D;
    // time-axis split of the backward scans: decided once per call (the partial sums of all windows share one
    // layout); it needs the bulk-copy path, i.e. 16-byte aligned rows
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    const bool rows_aligned = (L % 4 == 0) && al16(u) && al16(dt) && al16(z) && al16(grad_y) && al16(du) && al16(ddt) &&
                              al16(dz);
    const int nseg_b = (pl.nseg_bwd > 1 && rows_aligned) ? pl.nseg_bwd : 1;
    const long long nvirt = nch * nseg_b;
    float* part_bc = reinterpret_cast<float*>(ws + pl.off_part);
    float* part_d = part_bc + nvirt * N * 4;
    float* part_rowsum = part_d + nvirt;
    const OpArgs a = {u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, Dskip, z, B, D, N, L};
    if (keep_buf) {
        if (int rc = keep_check_layout(keep_buf, pl)) return rc;
    }
    ProjScratch ps;
    proj_scratch_bind(ps, ws + pl.off_proj, B, D, (long long)D * N, pl.ldw);
    if (int rc = proj_begin(D, (long long)D * N, x, ps, stream)) return rc;

    // final state: given by the caller, or recomputed by a state-only forward sweep
    const float* hend_re = h1_re;
    const float* hend_im = h1_im;
    if (!h1_re) {
        if (int rc = run_unitary_fwd(a, h0_re, h0_im, nullptr, cur_re, cur_im, ws, pl, ps, stream)) return rc;
        hend_re = cur_re;
        hend_im = cur_im;
    }

    const int nwin = (L + pl.window - 1) / pl.window;
    for (int w = nwin - 1; w >= 0; --w) {
        const long long t0 = (long long)w * pl.window;
        const int tl = (int)std::min<long long>(pl.window, L - t0);
        const bool first = (w == nwin - 1);   // first processed = last in time
        const bool final_ = (w == 0);
        const ProjDims pd = {B, D, (long long)D * N, L, pl.ldw, t0, tl};
        if (keep) {
            theta_w = keep + (size_t)w * pl.rows * pl.ldw;    // phases of the forward call; dtheta replaces them
            if (int rc = proj_split_u(pd, u, ps, stream)) return rc;
        } else if (int rc = proj_theta(pd, u, theta_w, ps, stream)) {
            return rc;
        }
        ScanBwdParams p = {};
        p.theta = theta_w; p.theta_bias = x_bias;
        p.u = u + t0; p.dt = dt + t0; p.z = z + t0; p.gy = grad_y + t0;
        p.B_r = B_r; p.B_theta = B_theta; p.C_r = C_r; p.C_theta = C_theta; p.Dskip = Dskip;
        p.h1_re = first ? hend_re : cur_re;
        p.h1_im = first ? hend_im : cur_im;
        p.gh1_re = first ? gh1_re : g_re;
        p.gh1_im = first ? gh1_im : g_im;
        p.dtheta = theta_w;
        p.du = du + t0; p.ddt = ddt + t0; p.dz = dz + t0;
        p.dh0_re = final_ ? dh0_re : g_re;
        p.dh0_im = final_ ? dh0_im : g_im;
        p.h0_re = final_ ? nullptr : cur_re;
        p.h0_im = final_ ? nullptr : cur_im;
        p.part_bc = part_bc; p.part_d = part_d; p.part_rowsum = part_rowsum;
        p.accumulate = first ? 0 : 1;
        p.nch = (int)nch; p.Dmod = D; p.N = N; p.L = tl;
        p.ld_theta = pl.ldw; p.ld_dtheta = pl.ldw; p.ld_row = L;
        // the scan leaves max|dtheta| of the window behind for the FP16 split of the adjoint GEMMs
        cudaError_t em = cudaMemsetAsync(ps.amax + 2, 0, sizeof(unsigned), stream);
        if (em != cudaSuccess) return cuda_fail(em, "clearing the dtheta maximum");
        p.dtheta_amax = ps.amax + 2;
        cudaError_t e;
        if (nseg_b > 1) {
            if (!scan_split_allowed(p)) {
                set_error("unitary_bwd: window rows lost their 16-byte alignment (t0=%lld)", t0);
                return AUSSM_EINVAL;
            }
            e = scan_unitary_bwd_split(p, nseg_b, reinterpret_cast<float*>(ws + pl.off_split), stream);
        } else {
            e = launch_scan_unitary_bwd(p, stream);
        }
        if (e != cudaSuccess) return cuda_fail(e, "unitary scan backward launch");
        if (int rc = proj_adjoints(pd, theta_w, dx, du, first, ps, stream, true)) return rc;
    }
    ReduceParams r = {};
    r.part_bc = part_bc; r.part_d = part_d; r.part_rowsum = part_rowsum;
    r.B_r = B_r; r.B_theta = B_theta; r.C_r = C_r; r.C_theta = C_theta;
    r.dB_r = dB_r; r.dB_theta = dB_theta; r.dC_r = dC_r; r.dC_theta = dC_theta; r.dD = dD; r.dx_bias = dx_bias;
    r.batch = B; r.D = D; r.N = N; r.nseg = nseg_b;
    cudaError_t e = launch_reduce_param_grads(r, stream);
    if (e != cudaSuccess) return cuda_fail(e, "parameter-gradient reduction launch");
    return AUSSM_OK;
}

int aussm_b200_unitary_bwd(const float* grad_y, const float* gh1_re, const float* gh1_im, const float* u,
                           const float* dt, const float* x, const float* x_bias, const float* B_r,
                           const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                           const float* z, const float* h0_re, const float* h0_im, const float* h1_re,
                           const float* h1_im, float* du, float* ddt, float* dx, float* dx_bias, float* dB_r,
                           float* dB_theta, float* dC_r, float* dC_theta, float* dD, float* dz, float* dh0_re,
                           float* dh0_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                           aussm_stream_t stream) {
    return unitary_bwd_impl(grad_y, gh1_re, gh1_im, u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, Dskip, z, h0_re,
                            h0_im, h1_re, h1_im, du, ddt, dx, dx_bias, dB_r, dB_theta, dC_r, dC_theta, dD, dz, dh0_re,
                            dh0_im, B, D, N, L, workspace, workspace_bytes, stream, nullptr, 0);
}

int aussm_b200_unitary_bwd_kept(const float* grad_y, const float* gh1_re, const float* gh1_im, const float* u,
                                const float* dt, const float* x, const float* x_bias, const float* B_r,
                                const float* B_theta, const float* C_r, const float* C_theta, const float* Dskip,
                                const float* z, const float* h0_re, const float* h0_im, const float* h1_re,
                                const float* h1_im, float* du, float* ddt, float* dx, float* dx_bias, float* dB_r,
                                float* dB_theta, float* dC_r, float* dC_theta, float* dD, float* dz, float* dh0_re,
                                float* dh0_im, int B, int D, int N, int L, void* workspace, size_t workspace_bytes,
                                void* theta_keep, size_t keep_bytes, aussm_stream_t stream) {
    if (!theta_keep) {
        set_error("unitary_bwd_kept: null phase buffer");
        return AUSSM_EINVAL;
    }
    return unitary_bwd_impl(grad_y, gh1_re, gh1_im, u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, Dskip, z, h0_re,
                            h0_im, h1_re, h1_im, du, ddt, dx, dx_bias, dB_r, dB_theta, dC_r, dC_theta, dD, dz, dh0_re,
                            dh0_im, B, D, N, L, workspace, workspace_bytes, stream, theta_keep, keep_bytes);
}

}  // extern "C"
