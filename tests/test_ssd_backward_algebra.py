"""The SSD backward as three role-permuted scans (ops/ssd.py::ssd_backward), checked on CPU.

The scan operator is stated token by token in fp32 (``scan_generic_torch``, the oracle of the CUDA kernels); with it in
place of the kernels every gradient must agree with autograd through the fp64 recurrence, padding included.
"""
import pytest
import torch

from lbi_b200.backbones.mamba2.ssd import ssd_recurrent_reference
from lbi_b200.ops.ssd import TorchScans, scan_generic_torch, ssd_backward


@pytest.mark.parametrize("n,g,with_state,seqlen", [(128, 1, True, 40), (64, 2, False, 33), (128, 2, True, 130)])
def test_role_permuted_backward_matches_autograd(n, g, with_state, seqlen):
    torch.manual_seed(seqlen)
    b, h, p = 2, 4, 64
    dd = torch.double
    x = torch.randn(b, seqlen, h, p, dtype=dd, requires_grad=True)
    dt = (torch.rand(b, seqlen, h, dtype=dd) * 0.5 + 0.05).requires_grad_(True)
    A = (-torch.rand(h, dtype=dd) - 0.2).requires_grad_(True)
    B = torch.randn(b, seqlen, g, n, dtype=dd, requires_grad=True)
    C = torch.randn(b, seqlen, g, n, dtype=dd, requires_grad=True)
    D = torch.randn(h, dtype=dd, requires_grad=True)
    init = torch.randn(b, h, p, n, dtype=dd, requires_grad=True) if with_state else None
    y, fin = ssd_recurrent_reference(x, dt, A, B, C, D, init)
    gy, gfin = torch.randn_like(y), torch.randn_like(fin)
    leaves = [x, dt, A, B, C, D] + ([init] if with_state else [])
    want = torch.autograd.grad([y, fin], leaves, [gy, gfin])
    f = lambda t: None if t is None else t.detach().float()  # noqa: E731
    got = ssd_backward(f(x), f(dt), f(A), f(B), f(C), f(D), f(init), f(fin), f(gy), f(gfin), ops=TorchScans)
    for name, a_, w_ in zip(("dx", "ddt", "dA", "dB", "dC", "dD", "dinit"), got, want):
        assert a_.shape == w_.shape, name
        err = (a_.double() - w_).norm().item() / w_.norm().item()
        assert err < 2e-5, f"{name}: {err:.2e}"


def test_scan_oracle_strict_and_per_head_layouts():
    torch.manual_seed(0)
    b, l, h, n = 1, 9, 2, 128
    v, bk, cq = torch.randn(b, l, h, 64), torch.randn(b, l, h, n), torch.randn(b, l, h, n)
    a = -torch.rand(b, l, h)
    init = torch.randn(b, h, 64, n)
    y0, f0 = scan_generic_torch(v, bk, cq, a, None, init, strict=True)
    y1, f1 = scan_generic_torch(v, bk, cq, a, None, init.transpose(2, 3).contiguous(), strict=True, per_head=True)
    assert torch.allclose(y0, y1, atol=1e-4) and torch.allclose(f0, f1.transpose(2, 3), atol=1e-4)
    # strict: token t does not see its own (v_t, bk_t)
    want0 = torch.einsum("bhpn,bhn->bhp", init * torch.exp(a[:, 0])[..., None, None], cq[:, 0])
    assert torch.allclose(y0[:, 0], want0, atol=1e-5)


def test_siso_backward_from_permuted_strict_scans_matches_autograd():
    from lbi_b200.backbones.mamba3.siso import _prepare, mamba3_siso_recurrent_reference
    from lbi_b200.ops.ssd import siso_core_backward

    torch.manual_seed(1)
    b, l, h, g, n, p, n_angles = 2, 37, 4, 2, 128, 64, 32
    dd = torch.double
    Q, K = (torch.randn(b, l, g, n, dtype=dd, requires_grad=True) for _ in range(2))
    V = torch.randn(b, l, h, p, dtype=dd, requires_grad=True)
    DT = (torch.rand(b, h, l, dtype=dd) * 0.3 + 0.05).requires_grad_(True)
    ADT = (-(torch.rand(b, h, l, dtype=dd) * 0.3)).requires_grad_(True)
    Trap = torch.randn(b, h, l, dtype=dd, requires_grad=True)
    Qb, Kb = (torch.randn(h, n, dtype=dd, requires_grad=True) for _ in range(2))
    Ang = torch.randn(b, l, h, n_angles, dtype=dd, requires_grad=True)
    D = torch.randn(h, dtype=dd, requires_grad=True)
    leaves = [Q, K, V, ADT, DT, Trap, Qb, Kb, Ang, D]
    y = mamba3_siso_recurrent_reference(*leaves[:9], D=D)
    gy = torch.randn_like(y)
    want = torch.autograd.grad(y, leaves, gy)

    f = [t.detach().float() for t in leaves]
    pre = [t.requires_grad_(True) for t in (f[0], f[1], f[3], f[4], f[5], f[6], f[7], f[8])]
    Qr, Kr, adt, qk = _prepare(pre[0], pre[1], f[2], pre[2], pre[3], pre[4], pre[5], pre[6], pre[7], torch.float32)
    skip = qk.detach() + f[9][None, None]
    dQr, dKr, dadt, dskip, dV = siso_core_backward(Qr.detach(), Kr.detach(), adt.detach(), skip, f[2], gy.float(), ops=TorchScans)
    gr = torch.autograd.grad([Qr, Kr, adt, qk], pre, [dQr, dKr, dadt, dskip])
    got = [gr[0], gr[1], dV, gr[2], gr[3], gr[4], gr[5], gr[6], gr[7], dskip.sum((0, 1))]
    for name, a_, w_ in zip("Q K V ADT DT Trap Q_bias K_bias Angles D".split(), got, want):
        err = (a_.double() - w_).norm().item() / w_.norm().item()
        assert err < 2e-5, f"{name}: {err:.2e}"
