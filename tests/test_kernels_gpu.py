"""Each kernel alone against a plain float32 torch restatement of the same operation, at sizes
other than the engine's: odd widths, tails, head sizes in steps of 16."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _bf16(t):
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 4096, 2304), (5, 200, 72), (16, 2304, 2048), (33, 1000, 328),
                                   (64, 512, 9216), (100, 130, 8), (256, 256, 256), (300, 384, 520),
                                   (777, 2304, 576)])
def test_gemm_tcgen05_against_float32(M, N, K):
    from glint_b200 import ops_tensor
    torch.manual_seed(M * 7 + N)
    a = _bf16(torch.randn(M, K, device=DEV))
    w = _bf16(torch.randn(N, K, device=DEV) * 0.1)
    want = a.float() @ w.float().T
    out = torch.full((M, N), float("nan"), device=DEV)
    ops_tensor.gemm(a, w, out)
    torch.cuda.synchronize()
    err = (out - want).abs().max().item()
    assert err <= 2e-3 * max(1.0, want.abs().max().item()), (M, N, K, err)


@pytest.mark.parametrize("splits", [1, 2, 3, 7])
def test_gemm_split_k_is_deterministic_and_equal(splits):
    from glint_b200 import ops_tensor
    torch.manual_seed(0)
    a = _bf16(torch.randn(9, 1544, device=DEV))
    w = _bf16(torch.randn(300, 1544, device=DEV) * 0.1)
    want = a.float() @ w.float().T
    outs = []
    for _ in range(3):
        out = torch.empty(9, 300, device=DEV)
        ops_tensor.gemm(a, w, out, force_splits=splits)
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert (outs[0] - want).abs().max().item() <= 2e-3 * want.abs().max().item()


def test_gemm_rows_do_not_depend_on_the_batch():
    from glint_b200 import ops_tensor
    torch.manual_seed(1)
    a = _bf16(torch.randn(70, 1024, device=DEV))
    w = _bf16(torch.randn(2304, 1024, device=DEV) * 0.1)
    whole = torch.empty(70, 2304, device=DEV)
    ops_tensor.gemm(a, w, whole, force_splits=1)
    for lo, hi in [(0, 1), (3, 12), (13, 70)]:
        part = torch.empty(hi - lo, 2304, device=DEV)
        ops_tensor.gemm(a[lo:hi].contiguous(), w, part, force_splits=1)
        assert torch.equal(part, whole[lo:hi]), (lo, hi)


def test_gemm_soft_cap_and_bf16_output():
    from glint_b200 import ops_tensor
    torch.manual_seed(2)
    a = _bf16(torch.randn(20, 256, device=DEV))
    w = _bf16(torch.randn(1000, 256, device=DEV))
    want = 30.0 * torch.tanh((a.float() @ w.float().T) / 30.0)
    out = torch.empty(20, 1000, device=DEV)
    ops_tensor.gemm(a, w, out, cap=30.0)
    assert (out - want).abs().max().item() < 5e-3
    out16 = torch.empty(20, 1000, device=DEV, dtype=torch.bfloat16)
    ops_tensor.gemm(a, w, out16, cap=30.0)
    assert (out16.float() - want).abs().max().item() < 0.15


@pytest.mark.parametrize("M,I,K,act", [(7, 320, 96, "gelu_tanh"), (130, 9216, 2304, "gelu_tanh"), (40, 200, 136, "silu")])
def test_gemm_gated_against_float32(M, I, K, act):
    from glint_b200 import ops_tensor
    torch.manual_seed(3)
    a = _bf16(torch.randn(M, K, device=DEV))
    w = _bf16(torch.randn(2 * I, K, device=DEV) * 0.1)
    g, u = a.float() @ w[:I].float().T, a.float() @ w[I:].float().T
    actf = (lambda x: 0.5 * x * (1 + torch.tanh(0.7978846 * (x + 0.044715 * x ** 3)))) if act == "gelu_tanh" \
        else (lambda x: x * torch.sigmoid(x))
    want = actf(g) * u
    out = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    ops_tensor.gemm_gated(a, w, out, act)
    torch.cuda.synchronize()
    err = (out.float() - want).abs().max().item()
    assert err <= 1e-2 * max(1.0, want.abs().max().item()), err
