"""Numerics of every sm_100a kernel against its fp32 PyTorch statement (all tests need a GPU)."""
import math

import pytest
import torch

from lbi_b200 import ops
from lbi_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    bound = atol + rtol * b.abs()
    assert bool((err <= bound).all()), f"{what}: max err {err.max().item():.3e}, max ref {b.abs().max().item():.3e}"


def test_extension_loaded():
    assert ops.native_available(), "lbi_b200._C must be built in-tree and loadable on a GPU box"


@pytest.mark.parametrize("rows,dim,with_stream", [(300, 256, True), (64, 1024, False), (17, 4096, True)])
def test_add_rmsnorm_fwd_bwd(rows, dim, with_stream):
    torch.manual_seed(0)
    branch = torch.randn(rows, dim, device=DEV).bfloat16()
    stream = torch.randn(rows, dim, device=DEV) if with_stream else None
    w = torch.rand(dim, device=DEV) + 0.5
    n1, s1, r1 = ops.add_rmsnorm_fwd(branch, stream, w, 1e-5, torch.bfloat16)
    n0, s0, r0 = ref.add_rmsnorm_fwd(branch, stream, w, 1e-5, torch.bfloat16)
    _close(s1, s0, 1e-6, 1e-6, "stream")
    _close(r1, r0, 1e-5, 1e-5, "rstd")
    _close(n1, n0, 2e-2, 1e-2, "normed")
    for reps in (1, 3):
        g = torch.randn(reps * rows, dim, device=DEV).bfloat16()
        d_in = torch.randn(reps * rows, dim, device=DEV)
        got = ops.rmsnorm_bwd(g, s0, r0, w, d_in.clone())
        want = ref.rmsnorm_bwd(g, s0, r0, w, d_in)
        _close(got, want, 1e-4, 1e-4, "rmsnorm_bwd")
    g = torch.randn(rows, dim, device=DEV).bfloat16()
    _close(ops.rmsnorm_wgrad(g, s0, r0), ref.rmsnorm_wgrad(g, s0, r0), 1e-3, 1e-4, "rmsnorm_wgrad")


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope(interleaved):
    from lbi_b200.backbones.transformer.rope import rope_tables

    torch.manual_seed(1)
    heads, kv, hd, t, b = 4, 2, 64, 96, 3
    qkv = torch.randn(b * t, (heads + 2 * kv) * hd, device=DEV).bfloat16()
    cos, sin = rope_tables(t, hd, 10000.0, torch.device(DEV))
    want = ref.rope_qkv(qkv, cos, sin, heads, kv, hd, t, interleaved, False)
    got = ops.rope_qkv(qkv.clone(), cos, sin, heads, kv, hd, t, interleaved, False)
    _close(got, want, 2e-2, 1e-2, "rope")
    back = ops.rope_qkv(got.clone(), cos, sin, heads, kv, hd, t, interleaved, True)
    _close(back, qkv, 5e-2, 2e-2, "rope inverse")


def test_swiglu():
    torch.manual_seed(2)
    u = torch.randn(200, 2 * 384, device=DEV).bfloat16()
    _close(ops.swiglu_fwd(u), ref.swiglu_fwd(u), 2e-2, 1e-2, "swiglu_fwd")
    da = torch.randn(3 * 200, 384, device=DEV).bfloat16()
    _close(ops.swiglu_bwd(da, u), ref.swiglu_bwd(da, u), 3e-2, 2e-2, "swiglu_bwd")


def test_interface_glue_and_embedding():
    torch.manual_seed(3)
    b, t, d, v = 3, 200, 256, 500
    canvas = torch.randn(b * t, d, device=DEV).bfloat16()
    cond = torch.randn(b, d, device=DEV)
    _close(ops.add_condition(canvas, cond, t), ref.add_condition(canvas, cond, t), 2e-2, 1e-2, "add_condition")
    rows = torch.randn(b * t, d, device=DEV)
    _close(ops.mean_pool_tokens(rows, b, t), ref.mean_pool_tokens(rows, b, t), 1e-5, 1e-5, "mean_pool")
    _close(ops.sum_tokens(rows.bfloat16(), b, t), ref.sum_tokens(rows.bfloat16(), b, t), 1e-3, 1e-4, "sum_tokens")
    table = torch.randn(v, d, device=DEV)
    ids = torch.randint(0, v, (b, t), device=DEV)
    _close(ops.embedding_fwd(ids, table, torch.bfloat16), ref.embedding_fwd(ids, table, torch.bfloat16), 0, 0, "embedding")
    g = torch.randn(b * t, d, device=DEV)
    got = ops.embedding_scatter_add(torch.zeros(v, d, device=DEV), ids, g)
    want = ref.embedding_scatter_add(torch.zeros(v, d, device=DEV), ids, g)
    _close(got, want, 1e-4, 1e-5, "embedding_scatter_add")
    x = torch.randn(130, 70, device=DEV).bfloat16()
    assert torch.equal(ops.transpose_2d(x), x.t().contiguous())


def test_causal_conv():
    torch.manual_seed(4)
    b, t, c, w = 2, 50, 64, 4
    x = torch.randn(b * t, c, device=DEV).bfloat16()
    weight = torch.randn(c, w, device=DEV)
    bias = torch.randn(c, device=DEV)
    _close(ops.causal_conv_fwd(x, weight, bias, b, t), ref.causal_conv_fwd(x, weight, bias, b, t), 3e-2, 2e-2, "conv fwd")
    dy = torch.randn(3 * b * t, c, device=DEV).bfloat16()
    _close(ops.causal_conv_dgrad(dy, weight, b, t), ref.causal_conv_dgrad(dy, weight, b, t), 3e-2, 2e-2, "conv dgrad")
    one = dy[: b * t].contiguous()
    before = ops.dispatch.KERNEL_LAUNCHES["count"]
    dw, db = ops.causal_conv_wgrad(one, x, w, b, t)
    assert ops.dispatch.KERNEL_LAUNCHES["count"] == before + 1, "the conv weight-gradient kernel did not run"
    want_dw, want_db = ref.causal_conv_wgrad(one, x, w, b, t)
    _close(dw, want_dw, 2e-2 * float(want_dw.abs().max()), 2e-2, "conv wgrad")
    _close(db, want_db, 2e-2 * float(want_db.abs().max()), 2e-2, "conv bias grad")


@pytest.mark.parametrize("b,k,r", [(1, 1, 1), (2, 3, 8), (3, 8, 64), (2, 5, 100), (1, 16, 128), (2, 8, 256)])
def test_suffix_scans(b, k, r):
    torch.manual_seed(5)
    mats = torch.randn(b, k, r, r, device=DEV) / math.sqrt(r)
    got = ops.suffix_scan_pullbacks(mats)
    want = ref.suffix_scan_pullbacks(mats)
    _close(got, want, 2e-5, 1e-5, "suffix_scan")
    offs = torch.randn(b, k, r, device=DEV)
    seed = torch.randn(b, r, device=DEV)
    _close(ops.affine_suffix_scan(mats, offs, seed), ref.affine_suffix_scan(mats, offs, seed), 2e-5, 1e-5, "affine scan")
    _close(ops.affine_suffix_scan(mats, offs, None), ref.affine_suffix_scan(mats, offs, None), 2e-5, 1e-5, "affine scan")
    # two identical launches must agree bit for bit (no atomics in the scans)
    assert torch.equal(got, ops.suffix_scan_pullbacks(mats))


def test_suffix_scan_low_precision_inputs_promote():
    torch.manual_seed(6)
    mats = (torch.randn(2, 4, 16, 16, device=DEV) / 4).bfloat16()
    out = ops.suffix_scan_pullbacks(mats)
    assert out.dtype == torch.float32
    _close(out, ref.suffix_scan_pullbacks(mats), 1e-4, 1e-4)


def test_adamw_and_sumsq():
    torch.manual_seed(7)
    n = 100_003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    shadow = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    p0, m0, v0 = p.clone(), m.clone(), v.clone()
    sumsq = torch.zeros(1, device=DEV)
    ops.ext().sumsq_(g, sumsq)
    _close(sumsq, g.square().sum().reshape(1), 1e-1, 1e-5, "sumsq")
    for step in (1, 2):
        ops.ext().adamw_step_(p, g, m, v, shadow, 1e-2, 0.9, 0.999, 1e-8, 0.1, step, 1.0, sumsq, 1.0)
        scale = torch.clamp(1.0 / (sumsq.sqrt() + 1e-6), max=1.0)
        ref.adamw_step(p0, g, m0, v0, 1e-2, 0.9, 0.999, 1e-8, 0.1, step, scale)
    _close(p, p0, 1e-5, 1e-5, "adamw params")
    _close(shadow, p0.bfloat16(), 1e-2, 1e-2, "adamw shadow")


def test_ce_fwd_bwd():
    torch.manual_seed(8)
    rows, vocab = 37, 1024
    logits = (torch.randn(rows, vocab, device=DEV) * 3).bfloat16()
    targets = torch.randint(0, vocab, (rows,), device=DEV)
    targets[5] = -1
    want_loss = torch.nn.functional.cross_entropy(logits.float(), targets, ignore_index=-1, reduction="sum") * 0.25
    lf = logits.float().requires_grad_(True)
    (torch.nn.functional.cross_entropy(lf, targets, ignore_index=-1, reduction="sum") * 0.25).backward()
    loss = torch.zeros(1, device=DEV)
    work = logits.clone()
    ops.ext().ce_fwd_bwd_(work, targets, loss, 0.25)
    _close(loss, want_loss.reshape(1), 1e-2, 1e-4, "ce loss")
    _close(work, lf.grad, 2e-3, 2e-2, "ce grad")


def test_matrix_norms_kernel_matches_linalg():
    g = torch.Generator(device="cuda").manual_seed(11)
    mats = torch.randn(3, 5, 96, 96, device="cuda", generator=g) / 96 ** 0.5
    mats[0, 0] = torch.eye(96, device="cuda") * 0.5          # degenerate spectrum
    mats[0, 1] = 0.0                                         # zero matrix
    spec, frob = ops.ext().matrix_norms(mats, 128)
    want_spec = torch.linalg.matrix_norm(mats, ord=2)
    want_frob = torch.linalg.matrix_norm(mats, ord="fro")
    assert torch.allclose(frob, want_frob, rtol=1e-4, atol=1e-6)
    assert torch.allclose(spec, want_spec, rtol=2e-2, atol=1e-6)
    assert (spec <= want_spec * (1 + 1e-4) + 1e-6).all()     # power iteration never overshoots


@pytest.mark.parametrize("hidden,activation", [(0, "silu"), (192, "silu"), (256, "gelu")])
def test_interface_jacobian_kernels_match_the_einsum_forms(hidden, activation):
    """J^T and J of an interface head and of LayerNorm over a basis: kernels (no graph) against the PyTorch forms
    (taken with a graph attached, which routes around the kernels) and against each other by <g, J t> = <J^T g, t>."""
    from lbi_b200.interfaces import vector_mlp as vm

    torch.manual_seed(hidden + 3)
    bsz, p, din, dout = 3, 37, 160, 96
    head = vm.VectorMLPHead(din, dout, hidden_dim=hidden, activation=activation).to(DEV)
    norm = torch.nn.LayerNorm(dout).to(DEV)
    with torch.no_grad():
        norm.weight.uniform_(0.5, 1.5)
    x = torch.randn(bsz, din, device=DEV)
    s = torch.randn(bsz, dout, device=DEV)
    g = torch.randn(bsz, p, dout, device=DEV)
    t = torch.randn(bsz, p, din, device=DEV)
    before = ops.dispatch.KERNEL_LAUNCHES["count"]
    with torch.no_grad():
        jt_g, j_t = vm.head_input_jacobian_t(head, x, g), vm.head_input_jacobian(head, x, t)
        ln_t, ln_f = vm.layer_norm_input_jacobian_t(norm, s, g), vm.layer_norm_input_jacobian(norm, s, g)
    # with a hidden layer each head Jacobian also runs the skinny forward kernel for the activation slope
    assert ops.dispatch.KERNEL_LAUNCHES["count"] == before + 4 + (2 if hidden else 0), "the Jacobian kernels did not run"
    gg, tt = g.clone().requires_grad_(True), t.clone().requires_grad_(True)      # graph attached -> PyTorch forms
    _close(jt_g, vm.head_input_jacobian_t(head, x, gg).detach(), 1e-4, 1e-4, "head J^T")
    _close(j_t, vm.head_input_jacobian(head, x, tt).detach(), 1e-4, 1e-4, "head J")
    _close(ln_t, vm.layer_norm_input_jacobian_t(norm, s, gg).detach(), 1e-4, 1e-4, "layernorm J^T")
    _close(ln_f, vm.layer_norm_input_jacobian(norm, s, gg).detach(), 1e-4, 1e-4, "layernorm J")
    lhs, rhs = (g * j_t).sum(-1), (jt_g * t).sum(-1)
    _close(lhs, rhs, 1e-3, 1e-3, "adjoint identity")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("gated,norm_before_gate,group", [(True, False, None), (True, True, 64), (False, True, None), (True, True, None)])
def test_gated_rmsnorm_kernels_match_the_pytorch_form(dtype, gated, norm_before_gate, group):
    """Forward and every gradient (x, gate, weight) of the gated / grouped RMSNorm kernels against fp32 autograd."""
    from lbi_b200.backbones.norms import gated_rms_norm, rms_norm_reference

    torch.manual_seed(5)
    rows, dim = 3 * 67, 256
    x = torch.randn(3, 67, dim, device=DEV).to(dtype)
    z = torch.randn(3, 67, dim, device=DEV).to(dtype) if gated else None
    w = (torch.rand(dim, device=DEV) + 0.5)
    gy = torch.randn(3, 67, dim, device=DEV).to(dtype)
    leaves = [t.clone().requires_grad_(True) for t in ([x, z, w] if gated else [x, w])]
    before = ops.dispatch.KERNEL_LAUNCHES["count"]
    y = gated_rms_norm(leaves[0], leaves[-1], eps=1e-5, z=leaves[1] if gated else None, norm_before_gate=norm_before_gate, group_size=group)
    got = torch.autograd.grad(y, leaves, gy)
    assert ops.dispatch.KERNEL_LAUNCHES["count"] == before + 2, "the gated RMSNorm kernels did not run"
    ref = [t.detach().float().requires_grad_(True) for t in leaves]
    ry = rms_norm_reference(ref[0], ref[-1], eps=1e-5, z=ref[1] if gated else None, norm_before_gate=norm_before_gate, group_size=group)
    want = torch.autograd.grad(ry, ref, gy.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    _close(y, ry.detach(), tol, tol, "gated rmsnorm y")
    for name, a_, w_ in zip(("dx", "dz", "dw") if gated else ("dx", "dw"), got, want):
        err = (a_.float() - w_).norm().item() / w_.norm().item()
        assert err <= (1e-2 if dtype == torch.bfloat16 else 1e-5), f"{name}: {err:.2e}"


@pytest.mark.parametrize("dim,gate_first", [(3072, True), (3072, False), (1536, True)])
def test_wide_group_gated_rmsnorm_backward_matches_the_pytorch_form(dim, gate_first):
    """One group of thousands of channels per row (the Mamba-2 shape) takes the block-per-row backward kernel: stacked
    directions sharing the forward tensors, with and without the weight gradient, against the fp32 PyTorch statement."""
    from lbi_b200.ops import mamba as mops

    torch.manual_seed(2)
    n, reps = 37, 3
    x = torch.randn(n, dim, device=DEV).bfloat16()
    z = torch.randn(n, dim, device=DEV).bfloat16()
    w = torch.rand(dim, device=DEV) + 0.5
    y, rstd = mops.gated_rmsnorm_fwd(x, z, w, 1e-5, dim, gate_first)
    for r, want_dw in ((reps, False), (1, True)):
        dy = torch.randn(r * n, dim, device=DEV).bfloat16()
        before = ops.dispatch.KERNEL_LAUNCHES["count"]
        got = mops.gated_rmsnorm_bwd(dy, x, z, w, rstd, dim, gate_first, want_dweight=want_dw)
        assert ops.dispatch.KERNEL_LAUNCHES["count"] == before + 1
        want = mops.gated_rmsnorm_bwd(dy.float().cpu(), x.float().cpu(), z.float().cpu(), w.cpu(), rstd.cpu(), dim, gate_first,
                                      want_dweight=want_dw)
        for name, a_, w_ in zip(("dx", "dz", "dw"), got, want):
            if w_ is None:
                continue
            err = (a_.float().cpu() - w_.float()).norm().item() / w_.float().norm().item()
            assert err <= 1e-2, f"{name}: {err:.2e}"


def test_softplus_dt_kernel_matches_pytorch_on_a_strided_slice():
    """The Mamba-2 step size from a column range of a wider bf16 matrix (no copy), with and without the limits."""
    from lbi_b200.ops import mamba as mops

    torch.manual_seed(7)
    proj = (torch.randn(333, 200, device=DEV) * 2).bfloat16()
    raw = proj[:, 152:]                                  # 48 heads, row stride 200
    bias = torch.randn(48, device=DEV)
    for lo, hi in ((0.0, float("inf")), (0.05, 1.5)):
        before = ops.dispatch.KERNEL_LAUNCHES["count"]
        dt, slope = mops.softplus_dt_fwd(raw, bias, lo, hi)
        assert ops.dispatch.KERNEL_LAUNCHES["count"] == before + 1
        want_dt, want_slope = mops.softplus_dt_fwd(raw.float().cpu(), bias.cpu(), lo, hi)
        _close(dt.cpu(), want_dt, 1e-5, 1e-5, "dt")
        raw_dt = torch.nn.functional.softplus(raw.float().cpu() + bias.cpu())
        clear = ((raw_dt - lo).abs() > 1e-4) & ((raw_dt - hi).abs() > 1e-4)      # a value on a limit may fall on either side
        _close(slope.cpu()[clear], want_slope[clear], 1e-5, 1e-5, "slope")


def test_mamba2_conv_silu_kernels_match_pytorch():
    """Depthwise causal conv + SiLU over the x | B | C slice: forward (split outputs), input cotangent for stacked directions
    written into a column range of a wider buffer, and the weight / bias gradient."""
    from lbi_b200.ops import mamba as mops

    b, l, parts, width, reps = 2, 200, (128, 64, 64), 4, 3
    ch = sum(parts)
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(b * l, ch, generator=gen).bfloat16()
    w = torch.randn(ch, width, generator=gen) * 0.5
    bias = torch.randn(ch, generator=gen) * 0.1
    pre_c, parts_c = mops.conv_silu_fwd(x, w, bias, b, l, parts)
    pre_g, parts_g = mops.conv_silu_fwd(x.cuda(), w.cuda(), bias.cuda(), b, l, parts)
    assert torch.allclose(pre_g.float().cpu(), pre_c.float(), atol=3e-2, rtol=3e-2)
    for a, c in zip(parts_g, parts_c):
        assert a.is_contiguous() and torch.allclose(a.float().cpu(), c.float(), atol=3e-2, rtol=3e-2)
    d_parts = [torch.randn(reps * b * l, p, generator=gen) for p in parts]
    d_parts[0] = d_parts[0].bfloat16()                       # dx arrives in bf16, dB / dC in fp32
    out_c = torch.zeros(reps * b * l, 64 + ch + 8).bfloat16()
    out_g = torch.zeros_like(out_c).cuda()
    mops.conv_silu_bwd(d_parts, pre_c, w, b, l, out_c, 64)
    mops.conv_silu_bwd([d.cuda() for d in d_parts], pre_g, w.cuda(), b, l, out_g, 64)
    assert torch.equal(out_g[:, :64].cpu(), out_c[:, :64]) and torch.equal(out_g[:, 64 + ch:].cpu(), out_c[:, 64 + ch:])
    err = (out_g.float().cpu() - out_c.float()).abs().max().item()
    assert err <= 3e-2 * out_c.float().abs().max().item() + 1e-2
    one = [d[: b * l] for d in d_parts]
    dw_c, db_c = mops.conv_silu_wgrad(one, pre_c, x, width, b, l)
    dw_g, db_g = mops.conv_silu_wgrad([d.cuda() for d in one], pre_g, x.cuda(), width, b, l)
    assert torch.allclose(dw_g.cpu(), dw_c, atol=3e-2 * dw_c.abs().max().item(), rtol=3e-2)
    assert torch.allclose(db_g.cpu(), db_c, atol=3e-2 * db_c.abs().max().item(), rtol=3e-2)


@pytest.mark.parametrize("hidden,act", [(0, "silu"), (48, "silu"), (48, "gelu")])
def test_interface_head_forward_and_parameter_vjp_kernels(hidden, act):
    """The skinny fp32 linear kernels behind the interface maps: forward with cached pre-activations and the closed-form
    parameter VJP against autograd on the same head."""
    from lbi_b200.interfaces.vector_mlp import VectorMLPHead, head_forward_cached, head_parameter_vjp

    torch.manual_seed(0)
    head = VectorMLPHead(40, 24, hidden, act).cuda()
    x = torch.randn(3, 40, device="cuda")
    g = torch.randn(3, 24, device="cuda")
    xr = x.clone().requires_grad_(True)
    y_ref = head(xr)
    grads_ref = torch.autograd.grad(y_ref, [xr, *head.parameters()], g)
    sink = {id(p): torch.zeros_like(p) for p in head.parameters()}
    with torch.no_grad():
        before = ops.dispatch.KERNEL_LAUNCHES["count"]
        y, cache = head_forward_cached(head, x)
        gx = head_parameter_vjp(head, cache, g, lambda p: sink[id(p)], want_input=True)
        assert ops.dispatch.KERNEL_LAUNCHES["count"] > before, "the skinny linear kernels did not run"
    assert torch.allclose(y, y_ref.detach(), atol=1e-5, rtol=1e-5)
    assert torch.allclose(gx, grads_ref[0], atol=1e-5, rtol=1e-4)
    for p, want in zip(head.parameters(), grads_ref[1:]):
        assert torch.allclose(sink[id(p)], want, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("batch,dim,hidden,width", [(4, 1024, 1024, 128), (2, 256, 64, 16), (12, 256, 64, 16), (3, 256, 0, 16)])
def test_interface_update_handoff_kernel_matches_the_module(batch, dim, hidden, width):
    """The fused interface update (hidden units spread over the grid for batch <= 8, one CTA per row otherwise, single-layer
    maps) without a peer: state, pre-norm state and delta against the PyTorch module."""
    from lbi_b200.interfaces import VectorMLPInterface

    torch.manual_seed(0)
    iface = VectorMLPInterface(feature_dim=dim, num_regions=2, interface_width=width, interface_map_hidden_dim=hidden).cuda()
    with torch.no_grad():
        iface.update_scale.uniform_(0.2, 0.8)
    state, pooled = torch.randn(batch, width, device="cuda"), torch.randn(batch, dim, device="cuda")
    with torch.no_grad():
        want = iface.update_from_pooled(state, pooled, 1)
    enc, norm = iface.encoders[1], iface.norms[1]
    first, second = enc.layers()
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):   # the ticket counter must come back to zero
        delta, pre, out = ops.ext().interface_update_handoff(
            state, pooled, first.weight.detach(), None if first.bias is None else first.bias.detach(),
            None if second is None else second.weight.detach(), None if (second is None or second.bias is None) else second.bias.detach(),
            iface.update_scale.detach()[1:2], norm.weight.detach(), norm.bias.detach(), float(norm.eps),
            0 if iface.activation == "silu" else 1, 0, 0, 0, counter)
        assert int(counter) == 0
        torch.testing.assert_close(out, want.state, atol=2e-4, rtol=2e-4)
        torch.testing.assert_close(pre, want.diagnostics["pre_norm_state"], atol=2e-4, rtol=2e-4)
        torch.testing.assert_close(delta, want.diagnostics["delta_state"], atol=2e-4, rtol=2e-4)


def test_tail_shapes_under_the_bounds_checking_debug_build():
    """The debug extension (-DLBI_BOUNDS_CHECK: index checks that record a site code and skip the access, never trap) on
    shapes that reach the tail paths of the conv / scan-glue kernels: no violation may be recorded.  Runs in a child process
    because the extension is chosen at import time."""
    import os
    import subprocess
    import sys

    from lbi_b200.build import _ext_path

    if not _ext_path("_Cdbg").exists():
        pytest.skip("debug extension not built (python -m lbi_b200.build --bounds-check)")
    code = r"""
import torch
from lbi_b200 import ops
from lbi_b200.ops import mamba as mops
assert ops.ext().BOUNDS_CHECK
g = torch.Generator(device="cuda").manual_seed(0)
for b, l, width in ((1, 37, 4), (3, 129, 2), (2, 200, 4)):
    parts = (64, 24, 24)
    ch = sum(parts)
    x = torch.randn(b * l, ch, device="cuda", generator=g).bfloat16()
    w = torch.randn(ch, width, device="cuda", generator=g)
    pre, acts = mops.conv_silu_fwd(x, w, None, b, l, parts)
    d = [torch.randn(2 * b * l, p, device="cuda", generator=g).bfloat16() for p in parts]
    out = torch.zeros(2 * b * l, ch + 8, device="cuda").bfloat16()
    mops.conv_silu_bwd(d, pre, w, b, l, out, 8)
    mops.conv_silu_wgrad([t[: b * l] for t in d], pre, x, width, b, l)
    y = ops.causal_conv_fwd(x, w, None, b, l)
    ops.causal_conv_dgrad(y, w, b, l)
    small = mops.siso_small_fwd(*(torch.randn(b * l, 5, device="cuda", generator=g) for _ in range(3)),
                                torch.randn(b * l, 7, device="cuda", generator=g), torch.randn(5, device="cuda", generator=g), 1e-4, b, l)
    mops.siso_small_bwd(small, *(torch.randn(2 * b, l, 5, device="cuda", generator=g) for _ in range(1)),
                        torch.randn(2 * b, l, 5, 7, device="cuda", generator=g),
                        *(torch.randn(2 * b, l, 5, device="cuda", generator=g) for _ in range(2)))
ids = torch.tensor([3, 99999, 5], device="cuda")
table = torch.randn(16, 8, device="cuda")
rows = ops.embedding_fwd(ids, table, torch.bfloat16)
torch.cuda.synchronize()
assert float(rows[1].abs().sum()) == 0.0 and ops.ext().kernel_status(table) == 81   # bad id: recorded, row zeroed
print("violations", ops.ext().bounds_violations())
"""
    env = dict(os.environ, LBI_B200_DEBUG_EXT="1")
    proc = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600,
                          cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "violations [0, 0]" in proc.stdout, proc.stdout
