"""Component-level checks: closed-form interface pullbacks vs autograd, Jacobian providers vs one-step VJPs,
cache contents, state ablations, backbone smoke, Mamba scans vs token recurrences, structured Transformer lowering."""
import pytest
import torch
import torch.nn.functional as F

from lbi_b200.backbones import BackboneSpec, build_backbone_stack
from lbi_b200.backbones.mamba2.ssd import ssd_chunk_scan, ssd_recurrent_reference
from lbi_b200.backbones.mamba3 import Mamba3Block
from lbi_b200.backbones.mamba3.siso import mamba3_siso_chunked, mamba3_siso_recurrent_reference
from lbi_b200.backends import TorchAutogradTransformerLowering
from lbi_b200.backward import build_interface_pullback_provider
from lbi_b200.interfaces import VectorMLPInterface
from lbi_b200.interfaces.vector_mlp import (
    VectorMLPHead, broadcast_condition_jacobian_t, head_input_jacobian, head_input_jacobian_t, layer_norm_input_jacobian,
    layer_norm_input_jacobian_t, mean_pool_jacobian_t,
)
from lbi_b200.models import LBILanguageModel


def lbi_model(backbone="transformer", axis="depth", k=2, **kw):
    torch.manual_seed(0)
    spec = BackboneSpec(name=backbone, dim=32, layers=4, n_heads=4, d_conv=4, d_state=16, headdim=16, chunk_size=8, **kw)
    iface = VectorMLPInterface(feature_dim=32, num_regions=k, interface_width=8, interface_map_hidden_dim=16)
    return LBILanguageModel(vocab_size=50, layers_per_region=4 // k, backbone_spec=spec, interface=iface, region_axis=axis,
                            num_sequence_regions=k)


@pytest.mark.parametrize("hidden,act", [(0, "silu"), (12, "silu"), (12, "gelu")])
def test_head_pullbacks_match_autograd(hidden, act):
    torch.manual_seed(1)
    head = VectorMLPHead(10, 6, hidden_dim=hidden, activation=act)
    x = torch.randn(3, 10, requires_grad=True)
    g = torch.randn(3, 4, 6)
    want = torch.stack([torch.autograd.grad(head(x), x, g[:, p], retain_graph=True)[0] for p in range(4)], dim=1)
    assert torch.allclose(head_input_jacobian_t(head, x.detach(), g), want, atol=1e-6, rtol=1e-5)
    t = torch.randn(3, 4, 10)
    fwd = torch.stack([torch.autograd.functional.jvp(head, x.detach(), t[:, p])[1] for p in range(4)], dim=1)
    assert torch.allclose(head_input_jacobian(head, x.detach(), t), fwd, atol=1e-6, rtol=1e-5)


def test_layer_norm_pullbacks_match_autograd():
    torch.manual_seed(2)
    norm = torch.nn.LayerNorm(8)
    with torch.no_grad():
        norm.weight.uniform_(0.5, 1.5)
        norm.bias.normal_()
    x = torch.randn(3, 8, requires_grad=True)
    g = torch.randn(3, 5, 8)
    want = torch.stack([torch.autograd.grad(norm(x), x, g[:, p], retain_graph=True)[0] for p in range(5)], dim=1)
    assert torch.allclose(layer_norm_input_jacobian_t(norm, x.detach(), g), want, atol=1e-6, rtol=1e-5)
    fwd = torch.stack([torch.autograd.functional.jvp(norm, x.detach(), g[:, p])[1] for p in range(5)], dim=1)
    assert torch.allclose(layer_norm_input_jacobian(norm, x.detach(), g), fwd, atol=1e-6, rtol=1e-5)


def test_pool_and_broadcast_pullbacks():
    g = torch.randn(2, 3, 7)
    spread = mean_pool_jacobian_t(g, 5)
    assert spread.shape == (2, 3, 5, 7) and torch.allclose(spread.sum(dim=2), g, atol=1e-6)
    assert torch.allclose(broadcast_condition_jacobian_t(spread), g, atol=1e-6)
    with pytest.raises(ValueError):
        mean_pool_jacobian_t(g, 0)


@pytest.mark.parametrize("axis,k", [("depth", 2), ("sequence", 4)])
def test_providers_agree_with_one_step_vjp(axis, k):
    model = lbi_model(axis=axis, k=k)
    ids = torch.randint(0, 50, (2, 24))
    _, cache = model.forward_with_cache(ids, detach_states=True)
    jac = {m: build_interface_pullback_provider(m, basis_chunk=c).materialize_state_jacobian_t(model=model, cache=cache)
           for m, c in (("graph", 1), ("recompute", 1), ("recompute", 3), ("recompute", 8), ("structured", 3), ("forward", 1))
           for m in [m]}
    for region in range(k):
        base = jac["graph"][region]
        for mode, mats in jac.items():
            assert torch.allclose(mats[region], base, atol=1e-5, rtol=1e-4), mode
        g = torch.randn(2, 8)
        (vjp,) = torch.autograd.grad(cache["states"][region + 1], cache["state_inputs"][region], g, retain_graph=True)
        assert torch.allclose(torch.einsum("bij,bj->bi", base, g), vjp, atol=1e-5)


def test_structured_transition_hooks_match_materialised_jacobian():
    model = lbi_model()
    ids = torch.randint(0, 50, (2, 16))
    _, cache = model.forward_with_cache(ids, detach_states=True)
    rc = cache["region_caches"][0]
    eye = torch.eye(8).unsqueeze(0).expand(2, 8, 8)
    upd = model.interface.apply_update_jacobian_t_to_region_output(region_cache=rc, state_out_cotangent_basis=eye)
    g_in = model.region_backend.input_pullback_basis(cache=rc.backend_cache, output_cotangent_basis=upd["g_region_output"])
    out = model.interface.apply_region_transition_jacobian_t(region_cache=rc, state_out_cotangent_basis=eye,
                                                             region_input_cotangent_basis=g_in)
    want = build_interface_pullback_provider("graph").materialize_state_jacobian_t(model=model, cache=cache, regions=[0])[0]
    assert torch.allclose(out["g_state_input_total"].transpose(1, 2), want, atol=1e-5, rtol=1e-4)


def test_cache_contents_and_ablations():
    model = lbi_model()
    ids = torch.randint(0, 50, (2, 16))
    logits, cache = model.forward_with_cache(ids)
    assert logits.shape == (2, 16, 50) and len(cache["states"]) == 3 and len(cache["region_caches"]) == 2
    rc = cache["region_caches"][1]
    assert rc.layer_range == (2, 4) and rc.region_input.shape == (2, 16, 32) and rc.state_out is cache["states"][2]
    for key in ("pooled_features", "delta_state", "update_scale", "pre_norm_state"):
        assert key in rc.interface_step.diagnostics
    model.eval()
    with torch.no_grad():
        base = model(ids)
        zero, _ = model.forward_with_cache(ids, message_ablation="zero_all")
        g = torch.Generator().manual_seed(0)
        noisy, _ = model.forward_with_cache(ids, message_ablation="noise", message_noise_std=1.0, ablation_generator=g)
        same, _ = model.forward_with_cache(ids, message_ablation="mask", message_mask_keep_prob=1.0)
    assert not torch.allclose(zero, base) and not torch.allclose(noisy, base) and torch.allclose(same, base)
    with pytest.raises(ValueError):
        model.forward_with_cache(ids, message_ablation="shuffle")


@pytest.mark.parametrize("name", ["transformer", "mamba2", "mamba3", "hybrid"])
def test_backbone_smoke_and_range_composition(name):
    torch.manual_seed(3)
    lt = ("mamba2", "transformer", "mamba3", "transformer") if name == "hybrid" else ()
    spec = BackboneSpec(name=name, dim=32, layers=4, n_heads=4, n_kv_heads=2, d_state=16, headdim=16, chunk_size=8, layer_types=lt)
    stack = build_backbone_stack(spec)
    x = torch.randn(2, 20, 32)
    y = stack(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    y.sum().backward()
    assert all(p.grad is not None for p in stack.parameters())


def test_causality_of_every_backbone():
    for name in ("transformer", "mamba2", "mamba3"):
        torch.manual_seed(4)
        stack = build_backbone_stack(BackboneSpec(name=name, dim=32, layers=2, n_heads=4, d_state=16, headdim=16, chunk_size=8))
        x = torch.randn(1, 24, 32)
        x2 = x.clone()
        x2[:, 15:] += 1.0
        with torch.no_grad():
            assert torch.allclose(stack(x)[:, :15], stack(x2)[:, :15], atol=1e-5), name


def test_ssd_chunk_scan_matches_recurrence():
    torch.manual_seed(5)
    b, l, h, p, g, n = 2, 37, 4, 8, 2, 16
    x, dt, A = torch.randn(b, l, h, p), torch.rand(b, l, h) * 0.5 + 0.01, -torch.rand(h) - 0.1
    B, C, D = torch.randn(b, l, g, n), torch.randn(b, l, g, n), torch.randn(h)
    want, final = ssd_recurrent_reference(x, dt, A, B, C, D)
    for chunk in (4, 8, 64):
        got, state = ssd_chunk_scan(x, dt, A, B, C, chunk, D, return_final_state=True)
        assert torch.allclose(got.double(), want, atol=1e-4, rtol=1e-4)
        assert torch.allclose(state.double(), final, atol=1e-4, rtol=1e-4)


def test_mamba3_siso_matches_recurrence_and_block_pullback():
    torch.manual_seed(6)
    b, l, h, p, n = 2, 29, 4, 8, 16
    Q, K, V, Z = torch.randn(b, l, 1, n), torch.randn(b, l, 1, n), torch.randn(b, l, h, p), torch.randn(b, l, h, p)
    DT = torch.rand(b, h, l) * 0.5 + 0.01
    ADT, Trap = -DT * (torch.rand(b, h, l) + 0.1), torch.randn(b, h, l)
    qb, kb, ang, D = torch.randn(h, n), torch.randn(h, n), torch.randn(b, l, h, n // 4), torch.randn(h)
    want = mamba3_siso_recurrent_reference(Q, K, V, ADT, DT, Trap, qb, kb, ang, D, Z)
    for chunk in (8, 16):
        got = mamba3_siso_chunked(Q, K, V, ADT, DT, Trap, qb, kb, ang, D, Z, chunk_size=chunk)
        assert torch.allclose(got.double(), want, atol=2e-4, rtol=1e-4)
    block = Mamba3Block(32, d_state=16, headdim=16, chunk_size=8)
    x = torch.randn(2, 12, 32, requires_grad=True)
    basis = torch.randn(2, 3, 12, 32)
    got = block.input_pullback_matrix(x.detach(), basis)
    branch, stream = block(x)
    want = torch.stack([torch.autograd.grad(branch + stream, x, basis[:, i], retain_graph=True)[0] for i in range(3)], dim=1)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("outproj_norm", [False, True])
def test_mamba3_decode_steps_reproduce_the_full_sequence(outproj_norm):
    from lbi_b200.backbones.mamba3.mixer import Mamba3

    torch.manual_seed(11)
    mixer = Mamba3(d_model=32, d_state=16, expand=2, headdim=16, chunk_size=8, is_outproj_norm=outproj_norm)
    u = torch.randn(2, 21, 32)
    with torch.no_grad():
        want = mixer(u)
    states = mixer.allocate_inference_cache(2, 21)
    assert [tuple(t.shape) for t in states] == [(2, 4, 4), (2, 4, 16, 16), (2, 1, 4, 16), (2, 4, 16)]
    assert states[0].dtype == states[1].dtype == torch.float32
    got = torch.stack([mixer.step(u[:, t], *states) for t in range(21)], dim=1)
    assert torch.allclose(got, want, atol=2e-6, rtol=1e-5)
    assert mixer.step(u[:, :1], *mixer.allocate_inference_cache(2, 1)).shape == (2, 1, 32)
    assert float(states[1].abs().sum()) > 0 and float(states[0].max()) < 2 * torch.pi
    with pytest.raises(NotImplementedError):
        mixer(u, inference_params=object())
    packed, _ = mixer.forward_with_cache(u[:1], cu_seqlens=torch.tensor([0, 8, 21]))
    with torch.no_grad():
        assert torch.allclose(packed[:, :8], mixer(u[:1, :8]), atol=2e-6) and torch.allclose(packed[:, 8:], mixer(u[:1, 8:]), atol=2e-6)


def test_mamba3_prefill_then_decode_and_state_carrying_combined_op():
    from lbi_b200.backbones.mamba3.mamba3 import Mamba3
    from lbi_b200.backbones.mamba3.siso import angle_dt, mamba3_siso_combined

    torch.manual_seed(14)
    mixer = Mamba3(d_model=32, d_state=16, expand=2, headdim=16, chunk_size=8)
    u = torch.randn(2, 30, 32)
    with torch.no_grad():
        want = mixer(u)
    states = mixer.allocate_inference_cache(2, 30)
    pieces = [mixer.prefill(u[:, :11], *states), mixer.prefill(u[:, 11:19], *states)]
    pieces.append(torch.stack([mixer.step(u[:, t], *states) for t in range(19, 30)], dim=1))
    assert torch.allclose(torch.cat(pieces, dim=1), want, atol=3e-6, rtol=1e-5)

    b, l, h, p, n, cut = 2, 37, 4, 8, 16, 15
    Q, K, V, Z = torch.randn(b, l, 1, n), torch.randn(b, l, 1, n), torch.randn(b, l, h, p), torch.randn(b, l, h, p)
    DT = torch.rand(b, h, l) * 0.5 + 0.01
    ADT, Trap = -DT * (torch.rand(b, h, l) + 0.1), torch.randn(b, h, l)
    qb, kb, ang, D = torch.randn(h, n), torch.randn(h, n), torch.randn(b, l, h, n // 4), torch.randn(h)
    oracle = mamba3_siso_recurrent_reference(Q, K, V, ADT, DT, Trap, qb, kb, ang, D, Z)
    cutargs = lambda a, z: (Q[:, a:z], K[:, a:z], V[:, a:z], ADT[..., a:z], DT[..., a:z], Trap[..., a:z], qb, kb, ang[:, a:z], D, Z[:, a:z])  # noqa: E731
    y1, *carry = mamba3_siso_combined(*cutargs(0, cut), chunk_size=8, return_final_states=True)
    y2, *end = mamba3_siso_combined(*cutargs(cut, l), Input_States=tuple(carry), chunk_size=8, return_final_states=True)
    assert torch.allclose(torch.cat([y1, y2], dim=1).double(), oracle, atol=2e-4, rtol=1e-4)
    _, *whole = mamba3_siso_combined(*cutargs(0, l), chunk_size=16, return_final_states=True)
    for a, c in zip(whole, end):
        assert torch.allclose(a, c, atol=1e-5)
    assert torch.allclose(mamba3_siso_combined(*cutargs(0, l)).double(), oracle, atol=2e-4, rtol=1e-4)
    theta, last = angle_dt(ang, DT, return_output_state=True)
    assert theta.shape == (b, l, h, n // 4) and torch.equal(last, whole[0]) and float(theta.min()) >= 0
    # one packed row of two sequences: each evaluated on its own, states per sequence
    cu = torch.tensor([0, cut, l])
    row = lambda t: t[:1]  # noqa: E731
    packed_args = (row(Q), row(K), row(V), row(ADT), row(DT), row(Trap), qb, kb, row(ang), D, row(Z))
    yp, *sp = mamba3_siso_combined(*packed_args, chunk_size=8, return_final_states=True, cu_seqlens=cu)
    first = mamba3_siso_combined(row(Q)[:, :cut], row(K)[:, :cut], row(V)[:, :cut], row(ADT)[..., :cut], row(DT)[..., :cut],
                                 row(Trap)[..., :cut], qb, kb, row(ang)[:, :cut], D, row(Z)[:, :cut], chunk_size=8,
                                 return_final_states=True)
    assert torch.equal(yp[:, :cut], first[0]) and all(t.shape[0] == 2 for t in sp) and torch.equal(sp[1][0], first[2][0])
    theta_p, last_p = angle_dt(row(ang), row(DT), return_output_state=True, cu_seqlens=cu)
    assert torch.equal(last_p, sp[0]) and torch.equal(theta_p[:, :cut], angle_dt(row(ang)[:, :cut], row(DT)[..., :cut]))
    with pytest.raises(ValueError):
        mamba3_siso_combined(*cutargs(0, l), cu_seqlens=cu)  # two rows cannot be one packed row


def test_mamba2_op_level_entries_match_the_module_and_the_token_loop():
    from lbi_b200.backbones.mamba2.mamba2_simple import Mamba2Simple
    from lbi_b200.backbones.mamba2.ops import mamba_chunk_scan_combined, mamba_split_conv1d_scan_combined, ssd_selective_scan

    torch.manual_seed(15)
    mixer = Mamba2Simple(32, d_state=16, headdim=16, chunk_size=8, learnable_init_states=True)
    with torch.no_grad():
        mixer.init_states.normal_()
    u = torch.randn(2, 20, 32)
    packed = torch.tensor([[0] * 7 + [1] * 13, [0] * 20])
    for seq_idx in (None, packed):
        got = mamba_split_conv1d_scan_combined(
            mixer.in_proj(u), mixer.conv1d.weight.squeeze(1), mixer.conv1d.bias, mixer.dt_bias, -torch.exp(mixer.A_log), mixer.D, 8,
            initial_states=mixer.init_states.unsqueeze(0).expand(2, -1, -1, -1), seq_idx=seq_idx, rmsnorm_weight=mixer.norm.weight,
            rmsnorm_eps=mixer.norm.eps, outproj_weight=mixer.out_proj.weight, outproj_bias=mixer.out_proj.bias, headdim=16,
            ngroups=1, norm_before_gate=False)
        assert torch.allclose(got, mixer(u, seq_idx=seq_idx), atol=1e-6)
    b, l, h, p, n = 2, 19, 4, 8, 16
    x, dt, A = torch.randn(b, l, h, p), torch.randn(b, l, h), -torch.rand(h) - 0.1
    B, C, D2, z, bias = torch.randn(b, l, 2, n), torch.randn(b, l, 2, n), torch.randn(h, p), torch.randn(b, l, h, p), torch.randn(h)
    kw = dict(D=D2, z=z, dt_bias=bias, dt_softplus=True, dt_limit=(0.01, 0.5))
    y, final = mamba_chunk_scan_combined(x, dt, A, B, C, 8, return_final_states=True, **kw)
    assert final.shape == (b, h, p, n) and torch.allclose(y, ssd_selective_scan(x, dt, A, B, C, **kw), atol=1e-4, rtol=1e-4)
    y_next = mamba_chunk_scan_combined(x, dt, A, B, C, 8, initial_states=final, **kw)
    both = mamba_chunk_scan_combined(torch.cat([x, x], 1), torch.cat([dt, dt], 1), A, torch.cat([B, B], 1), torch.cat([C, C], 1), 8,
                                     D=D2, z=torch.cat([z, z], 1), dt_bias=bias, dt_softplus=True, dt_limit=(0.01, 0.5))
    assert torch.allclose(both[:, l:], y_next, atol=1e-4, rtol=1e-4)
    cu, ids = torch.tensor([0, 7, l]), torch.cat([torch.zeros(7), torch.ones(l - 7)])[None].long()
    y_p, final_p, per_seq = mamba_chunk_scan_combined(x[:1], dt[:1], A, B[:1], C[:1], 8, seq_idx=ids, cu_seqlens=cu,
                                                      return_final_states=True, return_varlen_states=True)
    y_a, final_a = mamba_chunk_scan_combined(x[:1, :7], dt[:1, :7], A, B[:1, :7], C[:1, :7], 8, return_final_states=True)
    assert per_seq.shape == (2, h, p, n) and torch.equal(per_seq[0], final_a[0]) and torch.equal(per_seq[1], final_p[0])
    assert torch.equal(y_p[:, :7], y_a)
    with pytest.raises(ValueError):
        mamba_chunk_scan_combined(x, dt, A, B, C, 8, return_varlen_states=True)


def test_functional_norms_against_the_written_out_formula():
    from lbi_b200.backbones.norms import LayerNormGated, layernorm_fn, rms_norm_ref, rmsnorm_fn

    torch.manual_seed(16)
    x, z, w, bias = torch.randn(3, 5, 16), torch.randn(3, 5, 16), torch.randn(16), torch.randn(16)

    def written_out(b, gate, group, before, rms):
        t = x * F.silu(gate) if (gate is not None and not before) else x
        g = t.unflatten(-1, (-1, group or 16))
        g = g if rms else g - g.mean(-1, keepdim=True)
        out = (g * torch.rsqrt(g.square().mean(-1, keepdim=True) + 1e-5)).flatten(-2) * w
        out = out if b is None else out + b
        return out * F.silu(gate) if (gate is not None and before) else out

    for group in (None, 8):
        for before in (True, False):
            for gate in (None, z):
                for b in (None, bias):
                    kw = dict(z=gate, eps=1e-5, group_size=group, norm_before_gate=before)
                    assert torch.allclose(rms_norm_ref(x, w, b, **kw), written_out(b, gate, group, before, True), atol=1e-5)
                    assert torch.allclose(rmsnorm_fn(x, w, b, **kw), written_out(b, gate, group, before, True), atol=1e-5)
                    assert torch.allclose(layernorm_fn(x, w, b, **kw), written_out(b, gate, group, before, False), atol=1e-5)
                    assert torch.equal(layernorm_fn(x, w, b, is_rms_norm=True, **kw), rmsnorm_fn(x, w, b, **kw))
    module = LayerNormGated(16, group_size=8)
    assert torch.allclose(module(x, z), layernorm_fn(x, module.weight, module.bias, z=z, eps=1e-5, group_size=8), atol=1e-6)


def test_kernel_entry_points_under_the_module_paths_of_the_reference():
    from lbi_b200.backends.backbone_stack import BackboneStackRegionBackend
    from lbi_b200.backends.transformer_cuda import CudaTransformerLowering
    from lbi_b200.cuda.interface import suffix_scan_pullbacks
    from lbi_b200.cuda.mamba3 import state_mixer_input_pullback_basis
    from lbi_b200.cuda.transformer import attention_input_pullback_basis

    torch.manual_seed(17)
    mats = torch.randn(2, 3, 4, 4)
    suffix = suffix_scan_pullbacks(mats)
    assert suffix.shape == (2, 4, 4, 4) and torch.allclose(suffix[:, 0], mats[:, 0] @ mats[:, 1] @ mats[:, 2], atol=1e-5)
    q, k, v, do = torch.randn(1, 2, 8, 4), torch.randn(1, 2, 8, 4), torch.randn(1, 2, 8, 4), torch.randn(1, 3, 2, 8, 4)
    ref_style = attention_input_pullback_basis(q, k, v, do, softmax_scale=0.5, causal=True, use_cuda=True, kernel_mode="fa2_mma_pblock4")
    own_style = attention_input_pullback_basis(q, k, v, do, scale=0.5, kernel_mode="dense")
    lowered = CudaTransformerLowering().attention_input_pullback_basis(q=q, k=k, v=v, output_cotangent_basis=do, softmax_scale=0.5,
                                                                       kernel_mode="fa2_mma_pblock4")
    qg = q.clone().requires_grad_(True)
    out = F.scaled_dot_product_attention(qg, k, v, is_causal=True, scale=0.5)
    (want,) = torch.autograd.grad(out, qg, do[:, 1])
    assert torch.allclose(ref_style[0][:, 1], want, atol=1e-5)
    assert all(torch.equal(a, c) and torch.equal(a, d) for a, c, d in zip(ref_style, own_style, lowered))
    block = Mamba3Block(32, d_state=16, headdim=16, chunk_size=8)
    u, basis = torch.randn(2, 6, 32), torch.randn(2, 2, 6, 32)
    assert torch.equal(state_mixer_input_pullback_basis(block.mixer, u, basis), block.mixer.input_pullback_matrix(u, basis))
    spec = BackboneSpec(name="mamba2", dim=32, layers=2, d_state=16, headdim=16, chunk_size=8)
    first = BackboneStackRegionBackend(backbone_spec=spec, region_ranges=[(0, 1), (1, 2)])
    shared = BackboneStackRegionBackend(backbone=first.backbone, region_ranges=[(0, 2)])
    assert shared.backbone is first.backbone and shared.count_parameters() == first.count_parameters()
    with pytest.raises(ValueError):
        BackboneStackRegionBackend(region_ranges=[(0, 1)])
    with pytest.raises(ValueError):
        BackboneStackRegionBackend(backbone_spec=spec, region_ranges=[])


def test_mamba3_pullbacks_in_the_cache_form_of_the_reference():
    torch.manual_seed(12)
    block = Mamba3Block(32, d_state=16, headdim=16, chunk_size=8)
    hidden, stream_in = torch.randn(2, 12, 32, requires_grad=True), torch.randn(2, 12, 32, requires_grad=True)
    basis, basis_stream = torch.randn(2, 3, 12, 32), torch.randn(2, 3, 12, 32)
    out, stream_out, cache = block.forward_with_cache(hidden, stream_in)
    assert cache.residual_output is stream_out and cache.norm_input is cache.normed and cache.mixer_cache is cache.mixer
    assert cache.hidden_input is hidden and cache.residual_input is stream_in and cache.hidden_output is out
    g_hidden, g_stream = block.input_pullback_matrix(cache, basis, basis_stream)
    for i in range(3):
        want_h, want_s = torch.autograd.grad([out, stream_out], [hidden, stream_in], [basis[:, i], basis_stream[:, i]],
                                             retain_graph=True)
        assert torch.allclose(g_hidden[:, i], want_h, atol=1e-5, rtol=1e-4)
        assert torch.allclose(g_stream[:, i], want_s, atol=1e-5, rtol=1e-4)
    _, _, first = block.forward_with_cache(hidden.detach())
    g_only, none = block.input_pullback_matrix(cache=first, g_hidden_out=basis)
    assert none is None and g_only.shape == basis.shape
    mixer_in = torch.randn(2, 12, 32, requires_grad=True)
    mixer_out, mixer_cache = block.mixer.forward_with_cache(mixer_in)
    got = block.mixer.input_pullback_matrix(cache=mixer_cache, g_out=basis)
    want = torch.stack([torch.autograd.grad(mixer_out, mixer_in, basis[:, i], retain_graph=True)[0] for i in range(3)], dim=1)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)
    with pytest.raises(ValueError):
        block.mixer.input_pullback_matrix(mixer_cache, basis[:, :, :5])


def test_mamba2_packed_sequences_initial_states_and_conv_init():
    from lbi_b200.backbones.mamba2.mixer import Mamba2Simple

    torch.manual_seed(13)
    mixer = Mamba2Simple(32, d_state=16, headdim=16, chunk_size=8, conv_init=0.3, learnable_init_states=True)
    assert float(mixer.conv1d.weight.detach().abs().max()) <= 0.3 and mixer.init_states.shape == (4, 16, 16)
    with torch.no_grad():
        mixer.init_states.normal_()
    u = torch.randn(2, 20, 32)
    seq_idx = torch.tensor([[0] * 7 + [1] * 13, [0] * 20])
    packed = mixer(u, seq_idx=seq_idx)
    assert torch.equal(packed[0, :7], mixer(u[:1, :7])[0]) and torch.equal(packed[1], mixer(u[1:])[0])
    plain = Mamba2Simple(32, d_state=16, headdim=16, chunk_size=8)
    plain.load_state_dict({k: v for k, v in mixer.state_dict().items() if k != "init_states"})
    assert torch.allclose(packed[0, 7:], plain(u[:1, 7:])[0], atol=1e-6)           # later sequences start from a zero state
    assert not torch.allclose(packed[0, :7], plain(u[:1, :7])[0], atol=1e-4)       # the first one from the learnt state
    packed.sum().backward()
    assert float(mixer.init_states.grad.abs().sum()) > 0
    with pytest.raises(ValueError):
        Mamba2Simple(32, d_state=16, headdim=16, activation="relu")
    with pytest.raises(ValueError):
        mixer(u, seq_idx=seq_idx[:, :5])


@pytest.mark.parametrize("d_conv,kv", [(0, 4), (4, 2)])
def test_structured_transformer_lowering_matches_autograd_lowering(d_conv, kv):
    torch.manual_seed(7)
    spec = BackboneSpec(name="transformer", dim=32, layers=2, n_heads=4, n_kv_heads=kv, d_conv=d_conv)
    iface = VectorMLPInterface(feature_dim=32, num_regions=1, interface_width=4)
    model = LBILanguageModel(vocab_size=20, layers_per_region=2, backbone_spec=spec, interface=iface)
    backend = model.region_backend
    x = torch.randn(2, 10, 32)
    with torch.no_grad():
        out, cache = backend.forward_region(region_input=x, region_index=0)
    with torch.enable_grad():
        ref_out = backend.backbone.forward_range(x, 0, 2)
    assert torch.allclose(out, ref_out, atol=1e-5, rtol=1e-4)
    oracle = TorchAutogradTransformerLowering()
    basis = torch.randn(2, 3, 10, 32)
    assert torch.allclose(backend.input_pullback_basis(cache=cache, output_cotangent_basis=basis),
                          oracle.input_pullback_basis(backend=backend, cache=cache, output_cotangent_basis=basis), atol=1e-5, rtol=1e-4)
    ct = torch.randn(2, 10, 32)
    got, want = backend.parameter_vjp(cache=cache, output_cotangent=ct), oracle.parameter_vjp(backend=backend, cache=cache, output_cotangent=ct)
    assert set(got) == set(want)
    for name in want:
        assert torch.allclose(got[name].reshape(want[name].shape), want[name], atol=1e-5, rtol=1e-4), name


@pytest.mark.parametrize("backbone", ["transformer", "mamba2"])
def test_recomputes_run_under_the_autocast_state_of_the_forward(backbone):
    """A forward under autocast records that state; the Jacobian provider's recompute and the backend's pullback /
    parameter VJP restore it (a recompute at another precision would take other code paths than the forward did)."""
    model = lbi_model(backbone=backbone, axis="sequence", k=2)
    ids = torch.randint(0, 50, (2, 16))
    with torch.autocast("cpu", dtype=torch.bfloat16):
        _, cache = model.forward_with_cache(ids, detach_states=True)
    assert cache["autocast"] == ("cpu", torch.bfloat16)
    assert all(rc.backend_cache.autocast == ("cpu", torch.bfloat16) for rc in cache["region_caches"])
    seen = []
    inner = model.region_backend.backbone.forward_range

    def spy(*a, **kw):
        seen.append(torch.is_autocast_enabled("cpu") and torch.get_autocast_dtype("cpu") == torch.bfloat16)
        return inner(*a, **kw)

    model.region_backend.backbone.forward_range = spy
    try:
        assert not torch.is_autocast_enabled("cpu")
        build_interface_pullback_provider("recompute", basis_chunk=4).materialize_state_jacobian_t(model=model, cache=cache)
        rc = cache["region_caches"][0].backend_cache
        model.region_backend.parameter_vjp(cache=rc, output_cotangent=torch.randn(2, 8, 32))
        if backbone != "transformer":
            model.region_backend.input_pullback_basis(cache=rc, output_cotangent_basis=torch.randn(2, 3, 8, 32))
    finally:
        model.region_backend.backbone.forward_range = inner
    assert seen and all(seen)
    _, plain = model.forward_with_cache(ids, detach_states=True)
    assert plain["autocast"] is None


def test_backbone_spec_validation_and_reference_lm():
    from lbi_b200.backbones.general import ReferenceLM, infer_message_hidden_dim

    with pytest.raises(ValueError, match="hybrid layer_types must be drawn from"):
        BackboneSpec(name="hybrid", dim=32, layers=2, d_state=8, d_conv=4, expand=2, headdim=8, n_heads=4,
                     layer_types=("unsupported", "transformer")).validate()
    with pytest.raises(ValueError):
        BackboneSpec(name="hybrid", dim=32, layers=3, d_state=16, headdim=16, n_heads=4, layer_types=("mamba2", "transformer")).validate()
    with pytest.raises(ValueError):
        BackboneSpec(name="transformer", dim=30, layers=2, n_heads=4).validate()
    spec = BackboneSpec(name="mamba2", dim=16, layers=2, d_state=4, d_conv=4, expand=2, headdim=8, ngroups=1, chunk_size=16,
                        use_mem_eff_path=True)
    model = ReferenceLM(vocab_size=64, backbone_spec=spec)
    assert len(model.blocks) == 2 and type(model.blocks[0]).__name__ == "Mamba2Block"
    logits = model(torch.randint(0, 64, (2, 12)))
    assert logits.shape == (2, 12, 64) and torch.isfinite(logits).all()
    assert infer_message_hidden_dim(spec, 0) == 16 and infer_message_hidden_dim(spec, 24) == 24
    with pytest.raises(ValueError):
        infer_message_hidden_dim(spec, -1)
