"""The allocation-free backward entry point, `aussm_b200_scan_unitary_bwd_static`.

Who needs it: callers that may not (or cannot) obtain device memory when they run the operator - a
serving loop that must not trigger a synchronising cudaMalloc, a plug-in that is handed only its input
and output buffers, a runtime with a fixed memory plan.  The regular entry point makes them supply a
workspace; this one keeps its scratch in a fixed array inside the library.

The test calls it through the C ABI and compares every output with the regular entry point on the same
inputs, for two calls in a row on different data (the array is shared between calls and keeps the
previous call's contents, which must not leak into the next result), and checks that sizes beyond the
built-in array are refused.  This file is collected last on purpose.
"""
import pytest
import torch

from aussm_b200 import _lib
from tests.helpers import scan_core_inputs

pytestmark = pytest.mark.gpu

STATIC_BYTES = 4 * 1024 * 1024


def _run_both(seed, b, d, n, l):
    lib = _lib.load()
    inp = {k: v.cuda() for k, v in scan_core_inputs(seed, b, d, n, l).items()}
    P = lambda t: t.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    # forward through the regular entry point to get the final state the backward pass starts from
    y = torch.empty_like(inp["u"])
    h_re = torch.empty(b, d, n, device="cuda")
    h_im = torch.empty_like(h_re)
    rc = lib.aussm_b200_scan_unitary_fwd(P(inp["theta"]), P(inp["u"]), P(inp["dt"]), P(inp["z"]), P(inp["B_r"]),
                                         P(inp["B_theta"]), P(inp["C_r"]), P(inp["C_theta"]), P(inp["D"]),
                                         P(inp["h0_re"]), P(inp["h0_im"]), P(y), P(h_re), P(h_im), b, d, n, l, stream)
    _lib.check(rc, "forward")

    def outputs():
        return dict(dtheta=torch.full_like(inp["theta"], float("nan")), du=torch.full_like(y, float("nan")),
                    ddt=torch.full_like(y, float("nan")), dz=torch.full_like(y, float("nan")),
                    dB_r=torch.full((n,), float("nan"), device="cuda"), dB_t=torch.full((n,), float("nan"), device="cuda"),
                    dC_r=torch.full((n,), float("nan"), device="cuda"), dC_t=torch.full((n,), float("nan"), device="cuda"),
                    dD=torch.full((d,), float("nan"), device="cuda"), dh_re=torch.full_like(h_re, float("nan")),
                    dh_im=torch.full_like(h_re, float("nan")))

    def common(o):
        return [P(inp["gy"]), P(inp["gh_re"]), P(inp["gh_im"]), P(inp["theta"]), P(inp["u"]), P(inp["dt"]),
                P(inp["z"]), P(inp["B_r"]), P(inp["B_theta"]), P(inp["C_r"]), P(inp["C_theta"]), P(inp["D"]),
                P(h_re), P(h_im), P(o["dtheta"]), P(o["du"]), P(o["ddt"]), P(o["dz"]), P(o["dB_r"]), P(o["dB_t"]),
                P(o["dC_r"]), P(o["dC_t"]), P(o["dD"]), P(o["dh_re"]), P(o["dh_im"]), b, d, n, l]

    ref = outputs()
    # The regular entry point may cut a launch with few channels into time segments (other kernels, other
    # rounding); the static one never does.  Compare like with like: the split is off for the reference call.
    _lib.set_option("time_split", 0)
    try:
        ws = torch.empty(lib.aussm_b200_scan_unitary_bwd_workspace_bytes(b, d, n, l), dtype=torch.uint8, device="cuda")
        _lib.check(lib.aussm_b200_scan_unitary_bwd(*common(ref), P(ws), ws.numel(), stream), "regular backward")
    finally:
        _lib.set_option("time_split", 1)
    got = outputs()
    _lib.check(lib.aussm_b200_scan_unitary_bwd_static(*common(got), stream), "static backward")
    torch.cuda.synchronize()
    return ref, got


def test_static_scratch_variant_matches_regular_entry_point_twice():
    # second call: other data and a smaller problem, so most of the array still holds the first call's partials
    for seed, shape in ((41, (3, 40, 16, 512)), (42, (2, 9, 8, 260))):
        ref, got = _run_both(seed, *shape)
        for k in ref:
            assert torch.isfinite(got[k]).all(), k
            # same kernels, same reduction order: the results agree to the last bit; the tolerance of the
            # parity tests (relative 1e-3 for gradients) is far looser than what is asserted here
            torch.testing.assert_close(got[k], ref[k], rtol=1e-6, atol=1e-7, msg=lambda m, k=k: f"{k}: {m}")


def test_static_scratch_variant_rejects_sizes_beyond_its_array():
    lib = _lib.load()
    b, d, n, l = 16, 1024, 16, 64            # 16384 channels * 81 floats * 4 B = 5.3 MB > 4 MiB
    assert b * d * (5 * n + 1) * 4 > STATIC_BYTES
    t = torch.zeros(16, device="cuda")
    rc = lib.aussm_b200_scan_unitary_bwd_static(*([t.data_ptr()] * 25), b, d, n, l, None)
    assert rc == -2
    msg = lib.aussm_b200_last_error().decode()
    assert "scratch" in msg and "aussm_b200_scan_unitary_bwd" in msg
    assert lib.aussm_b200_scan_unitary_bwd_static(*([None] * 25), 1, 1, 1, 4, None) == -1
