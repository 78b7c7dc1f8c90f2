"""The tcgen05 three-term split GEMM (FP16 parts by default, TF32 parts as option or when a pitch is not a
multiple of 8) against a float64 product (through the C ABI)."""
import pytest
import torch

import aussm_b200
from aussm_b200 import _lib

pytestmark = pytest.mark.gpu


def _gemm(A, a_mn, a_b, B, b_mn, b_b, C, M, N, K, batches, reduce, beta):
    lib = _lib.load()
    nbytes = lib.aussm_b200_gemm_tf32x3_workspace_bytes(M, N, K, batches, a_b, b_b)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    rc = lib.aussm_b200_gemm_tf32x3(A.data_ptr(), a_mn, a_b, B.data_ptr(), b_mn, b_b, C.data_ptr(), M, N, K, batches,
                                    reduce, beta, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "gemm_tf32x3")
    assert aussm_b200.device_status() == 0


def _operand(rows, K, mn_major, batches, gen):
    """logical (batches, rows, K) float32 tensor and its packed storage"""
    logical = torch.randn(batches, rows, K, generator=gen)
    packed = logical.transpose(1, 2).contiguous() if mn_major else logical.contiguous()
    return logical, packed.cuda()


CASES = [
    # M, N, K, batches, a_batched, b_batched, reduce
    (128, 256, 32, 1, 0, 0, 0),
    (128, 256, 128, 1, 0, 0, 0),
    (256, 512, 96, 1, 0, 0, 0),
    (200, 300, 100, 1, 0, 0, 0),      # tails in M, N and K
    (64, 36, 1024, 1, 0, 0, 0),
    (384, 260, 64, 3, 0, 1, 0),       # shared A, batched B, one output per batch (theta = x u_b)
    (320, 128, 72, 3, 1, 1, 1),       # reduction over the batch (dx)
    (132, 200, 256, 2, 0, 1, 0),      # du-like
]


@pytest.fixture(params=["f16", "tf32", "f16-pair", "tf32-pair"])
def parts(request):
    """gemm_backend 0: FP16 parts where every pitch is a multiple of 8; 2: TF32 parts always;
    gemm_pair 0: one CTA per tile (default), 1: two-CTA tiles (tcgen05.mma.cta_group::2)"""
    _lib.set_option("gemm_backend", 0 if request.param.startswith("f16") else 2)
    _lib.set_option("gemm_pair", 1 if request.param.endswith("pair") else 0)
    yield request.param
    _lib.set_option("gemm_backend", 0)
    _lib.set_option("gemm_pair", 0)


@pytest.mark.parametrize("majors", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("case", CASES)
def test_gemm_matches_float64(case, majors, parts):
    M, N, K, batches, a_b, b_b, reduce = case
    a_mn, b_mn = majors
    if (a_mn and M % 4) or (b_mn and N % 4) or K % 4:
        pytest.skip("row length not a multiple of 4 floats")
    gen = torch.Generator().manual_seed(M * 7 + N * 3 + K + batches + a_mn * 2 + b_mn)
    A_log, A = _operand(M, K, a_mn, batches if a_b else 1, gen)
    B_log, Bm = _operand(N, K, b_mn, batches if b_b else 1, gen)
    prod = torch.einsum("bmk,bnk->bmn", A_log.double().expand(batches, M, K), B_log.double().expand(batches, N, K))
    ref = prod.sum(0, keepdim=True) if reduce else prod
    nout = 1 if reduce else batches
    for beta in (0, 1):
        C0 = torch.randn(nout, M, N, generator=gen)
        C = C0.clone().cuda()
        _gemm(A, a_mn, a_b, Bm, b_mn, b_b, C, M, N, K, batches, reduce, beta)
        want = ref + (C0.double() if beta else 0)
        err = (C.cpu().double() - want).abs().max().item()
        scale = want.abs().max().item()
        # float32-level accuracy: the three-term split drops only products of two low parts (2^-22 relative)
        assert err <= 3e-6 * scale, f"beta={beta}: max error {err:.3e} on scale {scale:.3e}"


def test_large_k_accuracy_is_float32_like(parts):
    M, N, K = 256, 256, 4096
    gen = torch.Generator().manual_seed(1)
    A = torch.randn(M, K, generator=gen)
    B = torch.randn(N, K, generator=gen)
    C = torch.empty(M, N, device="cuda")
    _gemm(A.cuda(), 0, 0, B.cuda(), 0, 0, C, M, N, K, 1, 0, 0)
    want = A.double() @ B.double().T
    err_tc = (C.cpu().double() - want).abs().max().item()
    err_fp32 = ((A.cuda() @ B.cuda().T).cpu().double() - want).abs().max().item()
    print(f"K=4096: {parts} parts max error {err_tc:.3e}, float32 matmul {err_fp32:.3e}")
    assert err_tc <= 4 * err_fp32 + 1e-4


@pytest.mark.parametrize("scales", [(1e-20, 1e15), (3e7, 2e-9), (1.0, 1.0)])
def test_f16_parts_keep_accuracy_over_the_float32_range(scales):
    """The FP16 parts are taken after a power-of-two scaling by the tensor's largest magnitude, so tensors far
    outside FP16's own range, and entries 1e6 times smaller than the largest one, keep float32-like accuracy."""
    M, N, K = 128, 256, 512
    gen = torch.Generator().manual_seed(5)
    A = torch.randn(M, K, generator=gen) * scales[0]
    B = torch.randn(N, K, generator=gen) * scales[1]
    A[::3] *= 1e-6                                # rows far below the tensor's maximum
    B[:, ::5] *= 1e-4
    C = torch.empty(M, N, device="cuda")
    _lib.set_option("gemm_backend", 0)
    _gemm(A.cuda(), 0, 0, B.cuda(), 0, 0, C, M, N, K, 1, 0, 0)
    want = A.double() @ B.double().T
    got = C.cpu().double()
    # row-wise scale: every output row is judged against its own magnitude
    row_scale = (A.double().abs() @ B.double().abs().T).clamp_min(1e-300)
    rel = ((got - want).abs() / row_scale).max().item()
    ref = (((A.cuda() @ B.cuda().T).cpu().double() - want).abs() / row_scale).max().item()
    print(f"scales {scales}: f16 parts {rel:.3e}, float32 matmul {ref:.3e} (relative to sum |a||b|)")
    assert rel <= 5e-7
