"""Mamba-2 SSD chunk-scan kernels against the fp64 token-by-token recurrence and the chunked PyTorch form."""
import pytest
import torch

from lbi_b200 import ops
from lbi_b200.backbones.mamba2.ssd import ssd_chunk_scan, ssd_recurrent_reference
from lbi_b200.ops.ssd import ssd_chunk_scan_cuda, ssd_cuda_supported

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(b, l, h, g, n, seed=0):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(b, l, h, 64, device=DEV, generator=gen).bfloat16()
    dt = torch.rand(b, l, h, device=DEV, generator=gen) * 0.1 + 0.005
    A = -(torch.rand(h, device=DEV, generator=gen) * 4 + 0.5)
    B = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.5).bfloat16()
    C = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.5).bfloat16()
    D = torch.randn(h, device=DEV, generator=gen)
    return x, dt, A, B, C, D


@pytest.mark.parametrize("b,l,h,g,n", [(1, 128, 2, 1, 64), (2, 256, 4, 1, 64), (1, 384, 4, 2, 128), (2, 200, 2, 1, 128), (1, 1024, 8, 1, 64)])
def test_ssd_kernels_match_recurrence(b, l, h, g, n):
    x, dt, A, B, C, D = _inputs(b, l, h, g, n, seed=l)
    assert ssd_cuda_supported(x, B)
    y, final = ssd_chunk_scan_cuda(x, dt, A, B, C, D=D, return_final_state=True)
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(x) == 0, "a bounded wait inside the SSD kernels ran out"
    want, want_final = ssd_recurrent_reference(x, dt, A, B, C, D=D)
    scale = want.abs().max().item()
    assert (y.double() - want).abs().max().item() <= 2e-2 * scale + 1e-3
    assert (final.double() - want_final).abs().max().item() <= 2e-2 * want_final.abs().max().item() + 1e-3
    torch_y = ssd_chunk_scan(x, dt, A, B, C, chunk_size=128, D=D)
    assert (y.float() - torch_y.float()).abs().max().item() <= 2e-2 * scale + 1e-3


def test_ssd_initial_state_and_gradients():
    x, dt, A, B, C, D = _inputs(1, 256, 2, 1, 64, seed=7)
    init = torch.randn(1, 2, 64, 64, device=DEV) * 0.1
    y, final = ssd_chunk_scan_cuda(x, dt, A, B, C, D=D, initial_state=init, return_final_state=True)
    want, want_final = ssd_recurrent_reference(x, dt, A, B, C, D=D, initial_state=init)
    assert (y.double() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3
    assert (final.double() - want_final).abs().max().item() <= 2e-2 * want_final.abs().max().item() + 1e-3
    # gradients flow through the recompute backward and agree with the pure PyTorch path
    xs, dts = x.float().requires_grad_(True), dt.clone().requires_grad_(True)
    ssd_chunk_scan_cuda(xs, dts, A, B.float(), C.float(), D=D).float().square().sum().backward()
    xr, dtr = x.float().requires_grad_(True), dt.clone().requires_grad_(True)
    ssd_chunk_scan(xr, dtr, A, B.float(), C.float(), chunk_size=128, D=D).float().square().sum().backward()
    assert torch.allclose(xs.grad, xr.grad, rtol=5e-2, atol=5e-2 * xr.grad.abs().max().item())
    assert torch.allclose(dts.grad, dtr.grad, rtol=5e-2, atol=5e-2 * dtr.grad.abs().max().item())


@pytest.mark.parametrize("b,l,h,g", [(1, 128, 2, 1), (2, 320, 4, 2), (1, 1024, 4, 1)])
def test_siso_kernels_match_recurrence(b, l, h, g):
    from lbi_b200.backbones.mamba3.siso import mamba3_siso_chunked, mamba3_siso_recurrent_reference
    from lbi_b200.ops.ssd import mamba3_siso_cuda, siso_cuda_supported

    gen = torch.Generator(device=DEV).manual_seed(l + h)
    n, s = 128, 32
    Q = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.3).bfloat16()
    K = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.3).bfloat16()
    V = torch.randn(b, l, h, 64, device=DEV, generator=gen).bfloat16()
    DT = torch.rand(b, h, l, device=DEV, generator=gen) * 0.1 + 0.005
    ADT = -DT * (torch.rand(b, h, l, device=DEV, generator=gen) * 4 + 0.5)
    Trap = torch.randn(b, h, l, device=DEV, generator=gen)
    Qb = torch.randn(h, n, device=DEV, generator=gen) * 0.2
    Kb = torch.randn(h, n, device=DEV, generator=gen) * 0.2
    Angles = torch.randn(b, l, h, s, device=DEV, generator=gen)
    D = torch.randn(h, device=DEV, generator=gen)
    Z = torch.randn(b, l, h, 64, device=DEV, generator=gen).bfloat16()
    assert siso_cuda_supported(V, Q)
    y = mamba3_siso_cuda(Q, K, V, ADT, DT, Trap, Qb, Kb, Angles, D, Z=Z)
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(V) == 0, "a bounded wait inside the SISO kernels ran out"
    want = mamba3_siso_recurrent_reference(Q, K, V, ADT, DT, Trap, Qb, Kb, Angles, D=D, Z=Z)
    scale = want.abs().max().item()
    assert (y.double() - want).abs().max().item() <= 3e-2 * scale + 1e-3
    torch_y = mamba3_siso_chunked(Q, K, V, ADT, DT, Trap, Qb, Kb, Angles, D=D, Z=Z, chunk_size=64)
    assert (y.float() - torch_y.float()).abs().max().item() <= 3e-2 * scale + 1e-3
