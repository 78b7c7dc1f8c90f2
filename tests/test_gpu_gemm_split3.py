"""The tcgen05 three-term split GEMM (FP16 hi/lo parts) against a float64 product, through the C ABI."""
import pytest
import torch

import aussm_b200
from aussm_b200 import _lib

pytestmark = pytest.mark.gpu


def _gemm(A, a_mn, a_b, B, b_mn, b_b, C, M, N, K, batches, reduce, beta):
    lib = _lib.load()
    nbytes = lib.aussm_b200_gemm_split3_workspace_bytes(M, N, K, batches, a_mn, a_b, b_mn, b_b)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    rc = lib.aussm_b200_gemm_split3(A.data_ptr(), a_mn, a_b, B.data_ptr(), b_mn, b_b, C.data_ptr(), M, N, K, batches,
                                    reduce, beta, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "gemm_split3")
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
    (130, 75, 37, 2, 0, 1, 0),        # nothing a multiple of 4: scalar split loads, scalar stores of C
    (61, 259, 129, 3, 1, 1, 1),
    (7, 5, 3, 1, 0, 0, 0),
]


@pytest.mark.parametrize("majors", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("case", CASES)
def test_gemm_matches_float64(case, majors):
    M, N, K, batches, a_b, b_b, reduce = case
    a_mn, b_mn = majors
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


def test_large_k_accuracy_is_float32_like():
    M, N, K = 256, 256, 4096
    gen = torch.Generator().manual_seed(1)
    A = torch.randn(M, K, generator=gen)
    B = torch.randn(N, K, generator=gen)
    C = torch.empty(M, N, device="cuda")
    _gemm(A.cuda(), 0, 0, B.cuda(), 0, 0, C, M, N, K, 1, 0, 0)
    want = A.double() @ B.double().T
    err_tc = (C.cpu().double() - want).abs().max().item()
    err_fp32 = ((A.cuda() @ B.cuda().T).cpu().double() - want).abs().max().item()
    print(f"K=4096: split GEMM max error {err_tc:.3e}, float32 matmul {err_fp32:.3e}")
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
    _gemm(A.cuda(), 0, 0, B.cuda(), 0, 0, C, M, N, K, 1, 0, 0)
    want = A.double() @ B.double().T
    got = C.cpu().double()
    # row-wise scale: every output row is judged against its own magnitude
    row_scale = (A.double().abs() @ B.double().abs().T).clamp_min(1e-300)
    rel = ((got - want).abs() / row_scale).max().item()
    ref = (((A.cuda() @ B.cuda().T).cpu().double() - want).abs() / row_scale).max().item()
    print(f"scales {scales}: f16 parts {rel:.3e}, float32 matmul {ref:.3e} (relative to sum |a||b|)")
    assert rel <= 5e-7


def test_misaligned_base_pointers_take_the_scalar_paths():
    """Operands and output that start 4 bytes into a buffer (not 16-byte aligned)."""
    M, N, K = 96, 88, 72
    gen = torch.Generator().manual_seed(9)
    A = torch.randn(M, K, generator=gen)
    B = torch.randn(N, K, generator=gen)
    Ad = torch.empty(M * K + 1, device="cuda")[1:].view(M, K).copy_(A)
    Bd = torch.empty(N * K + 1, device="cuda")[1:].view(N, K).copy_(B)
    Cd = torch.zeros(M * N + 1, device="cuda")[1:].view(M, N)
    assert Ad.data_ptr() % 16 and Cd.data_ptr() % 16
    _gemm(Ad, 0, 0, Bd, 0, 0, Cd, M, N, K, 1, 0, 0)
    want = A.double() @ B.double().T
    err = (Cd.cpu().double() - want).abs().max().item()
    assert err <= 3e-6 * want.abs().max().item()


def test_launch_counter_counts_this_librarys_kernels():
    lib = _lib.load()
    A = torch.randn(64, 64, device="cuda")
    C = torch.empty(64, 64, device="cuda")
    before = lib.aussm_b200_kernel_launches()
    _gemm(A, 0, 0, A, 0, 0, C, 64, 64, 64, 1, 0, 0)
    # two maximum passes, two split passes, one GEMM
    assert lib.aussm_b200_kernel_launches() - before == 5
