"""tcgen05 GEMM against fp32 matmul: K-major and MN-major operands, edge tiles, split-K, accumulation."""
import pytest
import torch

from lbi_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check(c, want, k):
    err = (c.float() - want).abs().max().item()
    scale = want.abs().max().item() + 1e-6
    assert err <= 2e-2 * scale + 1e-3, f"max err {err:.3e} vs scale {scale:.3e} (K={k})"
    assert ops.ext().kernel_status(c) == 0, "a bounded wait inside the GEMM ran out"


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (300, 200, 136), (1024, 1024, 1024), (4096, 128, 512), (130, 72, 8)])
def test_gemm_k_major(m, n, k):
    torch.manual_seed(0)
    a = torch.randn(m, k, device=DEV).bfloat16()
    b = torch.randn(n, k, device=DEV).bfloat16()
    want = a.float() @ b.float().t()
    _check(ops.ext().gemm(a, b), want, k)
    _check(ops.ext().gemm(a, b, out_fp32=True), want, k)


@pytest.mark.parametrize("m,n,k", [(256, 512, 320), (300, 192, 1000)])
def test_gemm_b_mn_major(m, n, k):
    """dgrad form: dx = dy @ W with W stored [K(out), N(in)]."""
    torch.manual_seed(1)
    dy = torch.randn(m, k, device=DEV).bfloat16()
    w = torch.randn(k, n, device=DEV).bfloat16()
    _check(ops.ext().gemm(dy, w, b_t=True), dy.float() @ w.float(), k)


@pytest.mark.parametrize("rows,out_f,in_f,splits", [(512, 256, 512, 1), (4096, 128, 320, 4), (1000, 192, 64, 3)])
def test_gemm_wgrad_form(rows, out_f, in_f, splits):
    """wgrad form: dW = dy^T @ x, both operands read with the reduction index outermost; split-K and accumulate."""
    torch.manual_seed(2)
    dy = torch.randn(rows, out_f, device=DEV).bfloat16()
    x = torch.randn(rows, in_f, device=DEV).bfloat16()
    want = dy.float().t() @ x.float()
    _check(ops.ext().gemm(dy, x, a_t=True, b_t=True, out_fp32=True, splits=splits), want, rows)
    acc = torch.ones(out_f, in_f, device=DEV)
    ops.ext().gemm(dy, x, a_t=True, b_t=True, out_fp32=True, accumulate_into=acc, splits=splits)
    _check(acc, want + 1.0, rows)


def test_gemm_strided_views():
    torch.manual_seed(3)
    big = torch.randn(512, 3 * 256, device=DEV).bfloat16()
    a = big[:, 256:512]  # row stride 768
    b = torch.randn(320, 256, device=DEV).bfloat16()
    _check(ops.ext().gemm(a, b), a.float() @ b.float().t(), 256)


def test_linear_helpers_use_native_gemm():
    torch.manual_seed(4)
    x = torch.randn(1024, 512, device=DEV).bfloat16()
    w = torch.randn(768, 512, device=DEV).bfloat16()
    before = ops.dispatch.KERNEL_LAUNCHES["count"]
    y = ops.linear_fwd(x, w)
    dy = torch.randn(1024, 768, device=DEV).bfloat16()
    dx = ops.linear_dgrad(dy, w)
    dw = ops.linear_wgrad(dy, x)
    assert ops.dispatch.KERNEL_LAUNCHES["count"] - before == 3
    _check(y, x.float() @ w.float().t(), 512)
    _check(dx, dy.float() @ w.float(), 768)
    _check(dw, dy.float().t() @ x.float(), 1024)
