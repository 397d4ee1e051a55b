"""The tcgen05 matrix product against a 64-bit product of the same bfloat16
operands: ragged sizes in every dimension, both output types, all epilogues,
and the verdict of its bounded waits."""

import math

import pytest
import torch

import plain_gemma2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _native():
    from strata_inference_b200.kernels import native
    native.require_device(torch.device(DEV))
    return native


def _rel(got, ref):
    got, ref = got.detach().double().cpu(), ref.double().cpu()
    return (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)


SHAPES = [(1, 128, 64), (8, 16, 8), (33, 200, 72), (64, 2304, 2048), (100, 300, 96),
          (129, 1000, 200), (300, 520, 1000), (1024, 384, 2304),
          # more tiles than pairs of SMs: every pair walks several, through both accumulators
          (2048, 9216, 512), (513, 5000, 136)]


@pytest.mark.parametrize("R,N,K", SHAPES)
def test_gemm_tcgen05_plain_product(R, N, K):
    n = _native()
    g = torch.Generator().manual_seed(R * 7 + N)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    out32 = torch.full((R, N), float("nan"), dtype=torch.float32, device=DEV)
    n.gemm_tcgen05(x.to(DEV), w.to(DEV), out32)
    assert n.gemm_tcgen05_error() == 0
    assert _rel(out32, ref) <= 2e-5
    out16 = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    n.gemm_tcgen05(x.to(DEV), w.to(DEV), out16)
    assert n.gemm_tcgen05_error() == 0
    assert _rel(out16, ref) <= 1e-2


@pytest.mark.parametrize("R,N,K", [(5, 64, 64), (70, 320, 96), (300, 2048, 256), (700, 9232, 128)])
def test_gemm_tcgen05_epilogues(R, N, K):
    n = _native()
    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    capped = torch.empty(R, N, dtype=torch.float32, device=DEV)
    n.gemm_tcgen05(x.to(DEV), w.to(DEV), capped, n.EPI_SOFTCAP, 0.7)
    assert _rel(capped, 0.7 * torch.tanh(ref / 0.7)) <= 2e-5
    gated = torch.empty(R, N // 2, dtype=torch.bfloat16, device=DEV)
    n.gemm_tcgen05(x.to(DEV), w.to(DEV), gated, n.EPI_GEGLU)
    y = ref.view(R, N // 16, 2, 8)
    assert _rel(gated, (plain.gelu_tanh(y[:, :, 0]) * y[:, :, 1]).reshape(R, N // 2)) <= 1e-2
    assert n.gemm_tcgen05_error() == 0


def test_gemm_tcgen05_takes_a_view_with_a_row_stride():
    n = _native()
    g = torch.Generator().manual_seed(3)
    big = torch.randn(50, 256, generator=g).to(torch.bfloat16).to(DEV)
    x = big[:, 64:192]                       # 128 columns, rows 256 apart
    w = (torch.randn(96, 128, generator=g) / 11).to(torch.bfloat16)
    out = torch.empty(50, 96, dtype=torch.float32, device=DEV)
    n.gemm_tcgen05(x, w.to(DEV), out)
    assert _rel(out, x.double().cpu() @ w.double().T) <= 2e-5
    assert n.gemm_tcgen05_error() == 0
    with pytest.raises(n.KernelError, match="multiples of 8"):
        n.gemm_tcgen05(big[:, :60], w[:, :60].contiguous().to(DEV), out)
