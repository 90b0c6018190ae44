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
    # gradients through the kernel backward agree with the pure PyTorch path
    xs, dts = x.float().requires_grad_(True), dt.clone().requires_grad_(True)
    ssd_chunk_scan_cuda(xs, dts, A, B.float(), C.float(), D=D).float().square().sum().backward()
    xr, dtr = x.float().requires_grad_(True), dt.clone().requires_grad_(True)
    ssd_chunk_scan(xr, dtr, A, B.float(), C.float(), chunk_size=128, D=D).float().square().sum().backward()
    assert torch.allclose(xs.grad, xr.grad, rtol=5e-2, atol=5e-2 * xr.grad.abs().max().item())
    assert torch.allclose(dts.grad, dtr.grad, rtol=5e-2, atol=5e-2 * dtr.grad.abs().max().item())


@pytest.mark.parametrize("strict,per_head,n", [(False, False, 64), (True, False, 128), (True, True, 128), (False, True, 128)])
def test_generic_scan_matches_its_oracle(strict, per_head, n):
    from lbi_b200.ops.ssd import scan_generic, scan_generic_torch

    b, l, h = 2, 384, 4
    g = h if per_head else 2
    gen = torch.Generator(device=DEV).manual_seed(11)
    v = torch.randn(b, l, h, 64, device=DEV, generator=gen).bfloat16()
    bk = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.3).bfloat16()
    cq = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.3).bfloat16()
    a = -(torch.rand(b, l, h, device=DEV, generator=gen) * 0.2)
    w = torch.rand(b, l, h, device=DEV, generator=gen) + 0.5
    init = torch.randn(b, h, n, 64, device=DEV, generator=gen) if per_head else torch.randn(b, h, 64, n, device=DEV, generator=gen)
    y, fin, _ = scan_generic(v, bk, cq, a, w, init, strict=strict, per_head=per_head)
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(v) == 0
    assert y.dtype == torch.float32
    want, want_fin = scan_generic_torch(v, bk, cq, a, w, init, strict=strict, per_head=per_head)
    assert (y - want).norm().item() <= 1e-2 * want.norm().item()
    assert (fin - want_fin).norm().item() <= 1e-2 * want_fin.norm().item()


@pytest.mark.parametrize("per_head,n,with_states", [(False, 64, True), (False, 128, False), (True, 128, True)])
def test_decay_gradient_kernel_matches_its_definition(per_head, n, with_states):
    from lbi_b200.ops.ssd import _shift_reverse, decay_grad, decay_grad_torch, scan_generic

    b, l, h = 2, 384, 4
    g = h if per_head else 2
    gen = torch.Generator(device=DEV).manual_seed(23 + n)
    v = torch.randn(b, l, h, 64, device=DEV, generator=gen).bfloat16()
    gy = torch.randn(b, l, h, 64, device=DEV, generator=gen).bfloat16()
    bk = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.3).bfloat16()
    cq = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.3).bfloat16()
    a = -(torch.rand(b, l, h, device=DEV, generator=gen) * 0.2)
    w = None if per_head else torch.rand(b, l, h, device=DEV, generator=gen) + 0.5
    shape = (b, h, n, 64) if per_head else (b, h, 64, n)
    init = torch.randn(shape, device=DEV, generator=gen).bfloat16().float() if with_states else None
    gfin = torch.randn(shape, device=DEV, generator=gen).bfloat16().float() if with_states else None
    fwd_states = scan_generic(v, bk, cq, a, w, init, strict=per_head, per_head=per_head)[2]
    rev_states = scan_generic(gy.flip(1), cq.flip(1), bk.flip(1), _shift_reverse(a), None, gfin, strict=per_head, per_head=per_head)[2]
    da = decay_grad(v, gy, bk, cq, a, w, states_in=fwd_states, states_cot_rev=rev_states, per_head=per_head)
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(v) == 0
    want = decay_grad_torch(v, gy, bk, cq, a, w, per_head=per_head, init=init, gfinal=gfin)
    assert da.shape == want.shape
    assert (da - want).norm().item() <= 1e-2 * want.norm().item()
    # sums that weight every token alike (what dA is made of) keep the accuracy: no accumulated cancellation
    assert abs((da.sum() - want.sum()).item()) <= 1e-2 * want.abs().sum().item() / l ** 0.5 + 1e-3 * abs(want.sum().item())


@pytest.mark.parametrize("b,l,h,g,n,with_state", [(2, 256, 4, 1, 128, True), (1, 200, 4, 2, 64, False), (1, 512, 8, 2, 128, False),
                                                   (2, 128, 2, 1, 64, True)])
def test_ssd_backward_kernels_match_autograd_of_the_recurrence(b, l, h, g, n, with_state):
    """Every gradient of the role-permuted kernel backward against fp64 autograd through the token recurrence."""
    x, dt, A, B, C, D = _inputs(b, l, h, g, n, seed=3 * l + n)
    init = torch.randn(b, h, 64, n, device=DEV) * 0.2 if with_state else None
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, dt, A, B, C, D)] + ([init.clone().requires_grad_(True)] if with_state else [])
    y, final = ssd_chunk_scan_cuda(*leaves[:5], D=leaves[5], initial_state=leaves[6] if with_state else None, return_final_state=True)
    gy = torch.randn_like(y)
    gfin = torch.randn_like(final) * (1.0 if with_state else 0.0)
    got = torch.autograd.grad([y, final], leaves, [gy, gfin])
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(x) == 0
    ref_leaves = [t.detach().double().requires_grad_(True) for t in leaves]
    ry, rfin = ssd_recurrent_reference(*ref_leaves[:5], D=ref_leaves[5], initial_state=ref_leaves[6] if with_state else None)
    want = torch.autograd.grad([ry, rfin], ref_leaves, [gy.double(), gfin.double()])
    for name, a_, w_ in zip(("dx", "ddt", "dA", "dB", "dC", "dD", "dinit"), got, want):
        err = (a_.double() - w_).norm().item() / max(w_.norm().item(), 1e-12)
        assert err <= 2.5e-2, f"{name}: relative error {err:.3e}"


@pytest.mark.parametrize("b,l,h,g,n", [(1, 200, 4, 2, 64), (2, 256, 4, 1, 128), (1, 512, 8, 2, 128)])
def test_ssd_autograd_takes_the_fused_backward_when_no_state_crosses_the_sequence(b, l, h, g, n):
    """Only y is used (no initial state, final state unused): the autograd Function routes to the fused chunk backward; every
    gradient against fp64 autograd through the token recurrence."""
    x, dt, A, B, C, D = _inputs(b, l, h, g, n, seed=5 * l + n)
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, dt, A, B, C, D)]
    y = ssd_chunk_scan_cuda(*leaves[:5], D=leaves[5])
    gy = torch.randn_like(y)
    got = torch.autograd.grad(y, leaves, gy)
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(x) == 0
    ref_leaves = [t.detach().double().requires_grad_(True) for t in leaves]
    ry, _ = ssd_recurrent_reference(*ref_leaves[:5], D=ref_leaves[5], initial_state=None)
    want = torch.autograd.grad(ry, ref_leaves, gy.double())
    for name, a_, w_ in zip(("dx", "ddt", "dA", "dB", "dC", "dD"), got, want):
        err = (a_.double() - w_).norm().item() / max(w_.norm().item(), 1e-12)
        assert err <= 3e-2, f"{name}: relative error {err:.3e}"


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


@pytest.mark.parametrize("b,l,h,g", [(1, 256, 2, 1), (2, 200, 4, 2)])
def test_siso_backward_kernels_match_autograd_of_the_recurrence(b, l, h, g):
    from lbi_b200.backbones.mamba3.siso import mamba3_siso_recurrent_reference
    from lbi_b200.ops.ssd import mamba3_siso_cuda

    gen = torch.Generator(device=DEV).manual_seed(5 * l + h)
    n, s = 128, 32
    Q = torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.3
    K = torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.3
    V = torch.randn(b, l, h, 64, device=DEV, generator=gen)
    DT = torch.rand(b, h, l, device=DEV, generator=gen) * 0.1 + 0.005
    ADT = -DT * (torch.rand(b, h, l, device=DEV, generator=gen) * 4 + 0.5)
    Trap = torch.randn(b, h, l, device=DEV, generator=gen)
    Qb = torch.randn(h, n, device=DEV, generator=gen) * 0.2
    Kb = torch.randn(h, n, device=DEV, generator=gen) * 0.2
    Angles = torch.randn(b, l, h, s, device=DEV, generator=gen)
    D = torch.randn(h, device=DEV, generator=gen)
    leaves = [t.requires_grad_(True) for t in (Q, K, V, ADT, DT, Trap, Qb, Kb, Angles, D)]
    y = mamba3_siso_cuda(*leaves)
    gy = torch.randn_like(y)
    got = torch.autograd.grad(y, leaves, gy)
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(V) == 0
    ref = [t.detach().double().requires_grad_(True) for t in leaves]
    want = torch.autograd.grad(mamba3_siso_recurrent_reference(*ref[:9], D=ref[9]), ref, gy.double())
    for name, a_, w_ in zip("Q K V ADT DT Trap Q_bias K_bias Angles D".split(), got, want):
        err = (a_.double() - w_).norm().item() / max(w_.norm().item(), 1e-12)
        assert err <= 3e-2, f"{name}: relative error {err:.3e}"


@pytest.mark.parametrize("dtype,g,n_angles", [(torch.float32, 2, 32), (torch.bfloat16, 1, 64), (torch.float32, 4, 5)])
def test_siso_preprocessing_kernels_match_the_pytorch_form(dtype, g, n_angles):
    """Forward and every gradient of the wide preprocessing (bias, qk dot, rotary turn, trapezoid scale) against autograd
    through the PyTorch form in fp64."""
    from lbi_b200.backbones.mamba3.siso import _WidePrepFunction, _rotate_pairs

    b, l, h, n = 2, 77, 4, 128
    gen = torch.Generator(device=DEV).manual_seed(17 + n_angles)
    Q = torch.randn(b, l, g, n, device=DEV, generator=gen).to(dtype)
    K = torch.randn(b, l, g, n, device=DEV, generator=gen).to(dtype)
    Qb, Kb = torch.randn(h, n, device=DEV, generator=gen) * 0.3, torch.randn(h, n, device=DEV, generator=gen) * 0.3
    theta = torch.rand(b, l, h, n_angles, device=DEV, generator=gen) * 6.28
    gamma = torch.rand(b, l, h, device=DEV, generator=gen) + 0.1
    scale = torch.rand(b, l, h, device=DEV, generator=gen) + 0.1
    leaves = [t.clone().requires_grad_(True) for t in (Q, K, Qb, Kb, theta, gamma, scale)]
    qr, kr, qk = _WidePrepFunction.apply(*leaves)
    gq, gk, gd = torch.randn(b, l, h, n, device=DEV, generator=gen), torch.randn(b, l, h, n, device=DEV, generator=gen), \
        torch.randn(b, l, h, device=DEV, generator=gen)
    # cotangents go in as fp32 through the kernel entry point (autograd would round them to the bf16 outputs' dtype)
    got = ops.ext().siso_prep_bwd(Q.contiguous(), K.contiguous(), Qb, Kb, theta, gamma, scale, gq, gk, gd)
    ref = [t.detach().double().requires_grad_(True) for t in (Q, K, Qb, Kb, theta, gamma, scale)]
    rep = h // g
    Qh = ref[0].repeat_interleave(rep, dim=2) + ref[2][None, None]
    Kh = ref[1].repeat_interleave(rep, dim=2) + ref[3][None, None]
    want_qk = ref[5] * (Qh * Kh).sum(-1)
    want_qr = _rotate_pairs(Qh, ref[4])
    want_kr = _rotate_pairs(Kh, ref[4]) * ref[6].unsqueeze(-1)
    want = torch.autograd.grad([want_qr, want_kr, want_qk], ref, [gq.double(), gk.double(), gd.double()])
    assert qr.dtype == torch.bfloat16 and (qr.double() - want_qr).abs().max().item() <= 2e-2 * want_qr.abs().max().item()
    assert (kr.double() - want_kr).abs().max().item() <= 2e-2 * want_kr.abs().max().item()
    assert (qk.double() - want_qk).abs().max().item() <= 1e-4 * want_qk.abs().max().item()
    for name, a_, w_ in zip("dQ dK dQ_bias dK_bias dtheta dgamma dscale".split(), got, want):
        err = (a_.double() - w_).norm().item() / w_.norm().item()
        assert err <= 2e-4, f"{name}: {err:.2e}"
    # dKr handed over as the reversed scan leaves it: time-reversed and padded to a multiple of the chunk
    pad = 128 - l % 128
    gk_rev = torch.nn.functional.pad(gk, (0, 0, 0, 0, 0, pad)).flip(1).contiguous()
    again = ops.ext().siso_prep_bwd(Q.contiguous(), K.contiguous(), Qb, Kb, theta, gamma, scale, gq, gk_rev, gd, True)
    for a_, b_ in zip(got, again):
        assert torch.allclose(a_, b_, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("backbone,d_state", [("mamba2", 64), ("mamba3", 128)])
def test_mamba_lbi_model_trains_through_the_kernels(backbone, d_state, monkeypatch):
    """An LBI model with a Mamba backbone on the GPU under bf16 autocast: the kernel path and the PyTorch path give the
    same loss and the same scan-engine gradients (the backward of the kernels is the role-permuted scans)."""
    import torch.nn.functional as F

    from lbi_b200.backbones import BackboneSpec
    from lbi_b200.backward import ScanADEngine
    from lbi_b200.interfaces import VectorMLPInterface
    from lbi_b200.models import LBILanguageModel
    from lbi_b200.ops import ssd as ops_ssd

    torch.manual_seed(0)
    spec = BackboneSpec(name=backbone, dim=128, layers=2, d_state=d_state, headdim=64, expand=2, d_conv=4, chunk_size=64)
    iface = VectorMLPInterface(feature_dim=128, num_regions=2, interface_width=8, interface_map_hidden_dim=32)
    model = LBILanguageModel(vocab_size=256, layers_per_region=1, backbone_spec=spec, interface=iface).to(DEV)
    g = torch.Generator().manual_seed(1)
    ids, tgt = torch.randint(0, 256, (2, 256), generator=g).to(DEV), torch.randint(0, 256, (2, 256), generator=g).to(DEV)

    def run(enabled):
        monkeypatch.setattr(ops_ssd, "ENABLED", enabled)
        model.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, cache = model.forward_with_cache(ids, detach_states=True)
        loss = F.cross_entropy(logits.float().reshape(-1, 256), tgt.reshape(-1))
        res = ScanADEngine(state_jacobian_mode="recompute", state_jacobian_basis_chunk=4).backward(model=model, loss=loss, cache=cache)
        return loss.detach(), {k: (None if v is None else v.detach().clone()) for k, v in res.grad_map.items()}

    launches0 = ops.dispatch.KERNEL_LAUNCHES["count"]
    loss_k, grads_k = run(True)
    assert ops.dispatch.KERNEL_LAUNCHES["count"] > launches0, "the Mamba mixer did not reach the CUDA kernels"
    assert ops.ext().kernel_status(ids.float()) == 0
    loss_t, grads_t = run(False)
    assert abs(float(loss_k) - float(loss_t)) < 2e-2
    for name, gt in grads_t.items():
        if gt is None:
            continue
        gk = grads_k[name]
        denom = gt.float().norm().item() + 1e-6
        assert (gk.float() - gt.float()).norm().item() / denom < 0.15, name


def _rel(a, b):
    return float((a.double() - b.double()).abs().max() / (b.double().abs().max() + 1e-9))


@pytest.mark.parametrize("per_head,n,g,l", [(True, 128, 4, 384), (False, 128, 2, 256), (False, 64, 1, 384), (True, 128, 4, 200)])
def test_fused_chunk_backward_matches_the_dense_definition(per_head, n, g, l):
    """One fused kernel per (direction, chunk, head) against the O(l^2) fp32 definition, with the forward operands shared by
    two stacked cotangent directions (the forward tensors are read with batch index b % 2)."""
    from lbi_b200.ops import ssd

    b, h, reps = 2, 4, 2
    gen = torch.Generator(device=DEV).manual_seed(11 + l)
    v = torch.randn(b, l, h, 64, device=DEV, generator=gen).bfloat16()
    bk = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.4).bfloat16()
    cq = (torch.randn(b, l, g, n, device=DEV, generator=gen) * 0.4).bfloat16()
    a = -(torch.rand(b, l, h, device=DEV, generator=gen) * 0.08 + 0.002)
    gy = torch.randn(reps * b, l, h, 64, device=DEV, generator=gen).bfloat16()
    if per_head:   # the Mamba-3 form: strict mask, per-head operands, per-token skip, no weight
        skip = torch.randn(b, l, h, device=DEV, generator=gen)
        _, _, states = ssd.scan_generic(torch.nn.functional.pad(v, (0, 0, 0, 0, 0, (-l) % 128)),
                                        torch.nn.functional.pad(bk, (0, 0, 0, 0, 0, (-l) % 128)),
                                        torch.nn.functional.pad(cq, (0, 0, 0, 0, 0, (-l) % 128)),
                                        torch.nn.functional.pad(a, (0, 0, 0, (-l) % 128)), None, None, strict=True, per_head=True)
        dv, dcq, dbk, da, dskip = ssd.chunk_backward(v, gy, bk, cq, a, None, skip, states, per_head=True, strict=True, dv_bf16=True,
                                                     dn_bf16=False)
        want = ssd.siso_core_backward_dense(cq, bk, a, skip, v, gy)   # (dQr, dKr, dadt, dskip, dV)
        got = (dcq, dbk, da, dskip, dv)
        names = ("dcq", "dbk", "da", "dskip", "dv")
    else:          # the Mamba-2 form: inclusive mask, grouped operands, weight dt
        dt = torch.rand(b, l, h, device=DEV, generator=gen) * 0.1 + 0.01
        A = -(torch.rand(h, device=DEV, generator=gen) * 2 + 0.3)
        a = dt * A
        pad = (-l) % 128
        P = torch.nn.functional.pad
        _, _, states = ssd.scan_generic(P(v, (0, 0, 0, 0, 0, pad)), P(bk, (0, 0, 0, 0, 0, pad)), P(cq, (0, 0, 0, 0, 0, pad)),
                                        P(a, (0, 0, 0, pad)), P(dt, (0, 0, 0, pad)), None)
        dx, ddt, dA, dB, dC, dD = ssd.ssd_backward_fused(v, dt, A, bk, cq, None, gy, states)
        want = ssd.ssd_backward_dense(v, dt, A, bk, cq, None, gy)[:5]
        got = (dx, ddt, dA, dB, dC)
        names = ("dx", "ddt", "dA", "dB", "dC")
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(v) == 0, "a bounded wait inside the fused backward ran out"
    for name, x, y in zip(names, got, want):
        assert x.shape == y.shape, (name, x.shape, y.shape)
        assert _rel(x.float(), y) < 3e-2, f"{name}: relative error {_rel(x.float(), y):.3e}"


def test_mamba3_small_tensor_kernels_match_pytorch():
    """Softplus / trapezoid weights / rotary phase (forward) and their pullback for stacked directions, kernel vs the
    PyTorch statement evaluated on the CPU."""
    from lbi_b200.ops import mamba as mops

    b, l, h, s, reps = 2, 300, 6, 32, 3
    gen = torch.Generator().manual_seed(5)
    dd_dt, dd_a, trap = (torch.randn(b * l, h, generator=gen) for _ in range(3))
    angles = torch.randn(b * l, s, generator=gen)
    bias = torch.randn(h, generator=gen) * 0.5 - 2.0
    want = mops.siso_small_fwd(dd_dt, dd_a, trap, angles, bias, 1e-4, b, l)
    got = mops.siso_small_fwd(dd_dt.cuda(), dd_a.cuda(), trap.cuda(), angles.cuda(), bias.cuda(), 1e-4, b, l)
    for name in ("dt", "a", "sig", "adt", "gamma", "scale", "tanh_angle", "sp_dt", "sp_a", "a_live"):
        assert torch.allclose(getattr(got, name).cpu(), getattr(want, name), atol=1e-5, rtol=1e-4), name
    # the phase is compared on the circle (a value just below 2 pi and one just above 0 are the same angle)
    diff = (got.theta.cpu() - want.theta + torch.pi) % (2 * torch.pi) - torch.pi
    assert diff.abs().max() < 2e-3
    cots = [torch.randn(reps * b, l, h, generator=gen) for _ in range(3)]
    dtheta = torch.randn(reps * b, l, h, s, generator=gen)
    want_b = mops.siso_small_bwd(want, cots[0], dtheta, cots[1], cots[2])
    got_b = mops.siso_small_bwd(got, cots[0].cuda(), dtheta.cuda(), cots[1].cuda(), cots[2].cuda())
    for name, x, y in zip(("d_dd_dt", "d_dd_a", "d_trap", "d_angles"), got_b, want_b):
        assert _rel(x.float().cpu(), y) < 1e-3, f"{name}: {_rel(x.float().cpu(), y):.3e}"
    got_bf = mops.siso_small_bwd(got, cots[0].cuda(), dtheta.cuda(), cots[1].cuda(), cots[2].cuda(), out_dtype=torch.bfloat16)
    assert got_bf[0].dtype == torch.bfloat16 and _rel(got_bf[3].float().cpu(), want_b[3]) < 2e-2


def test_gate_kernels_match_pytorch():
    from lbi_b200.ops import mamba as mops

    gen = torch.Generator().manual_seed(9)
    y, z = torch.randn(70, 192, generator=gen).bfloat16(), torch.randn(70, 192, generator=gen).bfloat16()
    dyg = torch.randn(3 * 70, 192, generator=gen).bfloat16()
    assert _rel(mops.gate_silu_fwd(y.cuda(), z.cuda()).float().cpu(), mops.gate_silu_fwd(y, z).float()) < 1e-2
    dy, dz = mops.gate_silu_bwd(dyg.cuda(), y.cuda(), z.cuda())
    wy, wz = mops.gate_silu_bwd(dyg, y, z)
    assert _rel(dy.float().cpu(), wy.float()) < 1e-2 and _rel(dz.float().cpu(), wz.float()) < 1e-2
