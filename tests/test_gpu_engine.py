"""FastLBIEngine on a B200 (bf16 kernels) against dense autograd of the same model in fp32 on the CPU."""
import copy

import pytest
import torch
import torch.nn.functional as F

from lbi_b200.backbones import BackboneSpec
from lbi_b200.backward import AutogradEngine
from lbi_b200.interfaces import VectorMLPInterface
from lbi_b200.models import LBILanguageModel
from lbi_b200.parallel import FastLBIEngine

pytestmark = pytest.mark.gpu


def _model(axis, k, tie):
    torch.manual_seed(0)
    spec = BackboneSpec(name="transformer", dim=256, layers=4, n_heads=4, d_conv=0, d_intermediate=512)
    iface = VectorMLPInterface(feature_dim=256, num_regions=k, interface_width=16, interface_map_hidden_dim=64)
    return LBILanguageModel(vocab_size=1024, layers_per_region=4 // k if axis == "depth" else 1, backbone_spec=spec,
                            interface=iface, region_axis=axis, num_sequence_regions=k, tie_embeddings=tie)


@pytest.mark.parametrize("axis,tie", [("sequence", True), ("depth", False)])
def test_engine_grad_parity_bf16(axis, tie):
    k = 2
    cpu_model = _model(axis, k, tie)
    gpu_model = copy.deepcopy(cpu_model).cuda()
    torch.manual_seed(1)
    ids = torch.randint(0, 1024, (2, 512))
    tgt = torch.randint(0, 1024, (2, 512))
    logits = cpu_model(ids)
    loss = F.cross_entropy(logits.float().reshape(-1, 1024), tgt.reshape(-1))
    want = AutogradEngine().backward(model=cpu_model, loss=loss).grad_map
    engine = FastLBIEngine(gpu_model, lr=1e-3, basis_chunk=8)
    res = engine.backward(ids.cuda(), tgt.cuda())
    assert abs(float(res.loss) - float(loss.detach())) < 5e-3 * max(1.0, abs(float(loss.detach())))
    got = engine.named_grads()
    worst = 0.0
    for name, ref in want.items():
        if ref is None:
            continue
        g = got[name].float().cpu()
        rel = float((g - ref).norm() / (ref.norm() + 1e-12))
        worst = max(worst, rel)
        # the reference's bf16 parity bar is elementwise allclose(atol=5e-2, rtol=5e-2); rel-L2 guards against a
        # gradient that is small everywhere but wrong
        assert torch.allclose(g, ref, atol=5e-2, rtol=5e-2), f"{name}: max abs err {float((g - ref).abs().max()):.3e}"
        # a gradient that is tiny as a whole (a two-element scale whose norm is 1e-4) is noise in bf16: the state cotangent it is
        # a dot product with carries 1e-2 relative rounding, and the elementwise bar above already covers it
        assert rel < 1.5e-1 or float(ref.norm()) < 1e-3, f"{name}: rel-L2 {rel:.3e}"
    before = [p.detach().clone() for p in gpu_model.parameters()]
    out = engine.step(ids.cuda(), tgt.cuda())
    assert torch.isfinite(out)
    assert any(not torch.equal(a, b) for a, b in zip(before, gpu_model.parameters()))


def _mamba_model(kind, k=2):
    torch.manual_seed(0)
    kw = dict(dim=256, layers=2, d_state=128, headdim=64, expand=2, d_conv=4, chunk_size=128)
    if kind == "hybrid":
        spec = BackboneSpec(name="hybrid", layer_types=("mamba3", "transformer"), n_heads=4, d_intermediate=512, **{**kw, "d_conv": 0})
    else:
        spec = BackboneSpec(name=kind, **kw)
    iface = VectorMLPInterface(feature_dim=256, num_regions=k, interface_width=16, interface_map_hidden_dim=64)
    return LBILanguageModel(vocab_size=1024, layers_per_region=1, backbone_spec=spec, interface=iface, region_axis="sequence",
                            num_sequence_regions=k, tie_embeddings=True)


@pytest.mark.parametrize("kind", ["mamba3", "mamba2", "hybrid"])
def test_mamba_engine_grad_parity_bf16(kind):
    """The closed-form Mamba lowering on the sm_100a kernels (bf16) against dense autograd in fp32 on the CPU, at the
    reference's bf16 parity bar for Mamba-3 / hybrid models (atol = rtol = 5e-2, loss 5e-3)."""
    cpu_model = _mamba_model(kind)
    gpu_model = copy.deepcopy(cpu_model).cuda()
    torch.manual_seed(1)
    ids, tgt = torch.randint(0, 1024, (2, 512)), torch.randint(0, 1024, (2, 512))
    logits = cpu_model(ids)
    loss = F.cross_entropy(logits.float().reshape(-1, 1024), tgt.reshape(-1))
    want = AutogradEngine().backward(model=cpu_model, loss=loss).grad_map
    engine = FastLBIEngine(gpu_model, lr=1e-3, basis_chunk=8)
    res = engine.backward(ids.cuda(), tgt.cuda())
    from lbi_b200 import ops

    assert ops.ext().kernel_status(res.loss) == 0
    assert abs(float(res.loss) - float(loss.detach())) < 5e-3 * max(1.0, abs(float(loss.detach())))
    got = engine.named_grads()
    for name, ref in want.items():
        if ref is None:
            continue
        g = got[name].float().cpu()
        rel = float((g - ref).norm() / (ref.norm() + 1e-12))
        assert torch.allclose(g, ref, atol=5e-2, rtol=5e-2), f"{name}: max abs err {float((g - ref).abs().max()):.3e}"
        # a gradient that is tiny as a whole (a two-element scale whose norm is 1e-4) is noise in bf16: the state cotangent it is
        # a dot product with carries 1e-2 relative rounding, and the elementwise bar above already covers it
        assert rel < 1.5e-1 or float(ref.norm()) < 1e-3, f"{name}: rel-L2 {rel:.3e}"
    out = engine.step(ids.cuda(), tgt.cuda())
    assert torch.isfinite(out)


@pytest.mark.parametrize("config", ["tiny", "mamba-tiny"])
def test_bench_paths_run_on_tiny_configs(config):
    """bench.py's training path (the region-parallel engine, every backbone) on tiny shapes: finite loss, kernels
    launched, no bounded wait ran out, end-to-end figure present."""
    import argparse
    import math
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench

    args = argparse.Namespace(config=config, gpus=1, steps=1, warmup=1, basis_chunk=8, no_e2e=False, profile_ops=False, comm="auto",
                              impl="ours", jacobian_mode="recompute", engine="fast", recompute_forward="auto", variant="lbi")
    out = bench.run_ours(args)
    assert math.isfinite(out["final_loss"]) and out["value"] > 0
    assert out["gpu_launches"] > 0 and out["kernel_status"] == 0
    assert out["e2e"]["value"] > 0 and out["e2e"]["h2d_bytes_per_step"] > 0


@pytest.mark.parametrize("kind", ["transformer", "transformer-qkv-conv", "mamba3", "mamba2", "hybrid"])
def test_engine_step_never_leaves_the_kernels_in_strict_mode(kind):
    """With strict mode on, any route to PyTorch / cuBLAS / flash_attn for a CUDA bf16 tensor raises: a full training step
    of every backbone must pass, and the fallback counters must stay empty."""
    from lbi_b200 import ops

    if kind == "transformer":
        model = _model("sequence", 2, True)
    elif kind == "transformer-qkv-conv":   # the reference's Transformer always has the depthwise conv on qkv (d_conv >= 1)
        torch.manual_seed(0)
        spec = BackboneSpec(name="transformer", dim=256, layers=2, n_heads=4, d_conv=4, d_intermediate=512)
        iface = VectorMLPInterface(feature_dim=256, num_regions=2, interface_width=16, interface_map_hidden_dim=64)
        model = LBILanguageModel(vocab_size=1024, layers_per_region=1, backbone_spec=spec, interface=iface, region_axis="sequence",
                                 num_sequence_regions=2, tie_embeddings=True)
    else:
        model = _mamba_model(kind)
    model = model.cuda()
    prev = ops.dispatch.set_strict(True)
    ops.dispatch.FALLBACKS.clear()
    try:
        engine = FastLBIEngine(model, lr=1e-3, basis_chunk=8)
        ids, tgt = torch.randint(0, 1024, (2, 512), device="cuda"), torch.randint(0, 1024, (2, 512), device="cuda")
        loss = engine.step(ids, tgt)
        assert torch.isfinite(loss)
    finally:
        ops.dispatch.set_strict(prev)
    assert ops.dispatch.FALLBACKS == {}


def test_strict_mode_refuses_a_library_route():
    from lbi_b200 import ops

    x = torch.randn(64, 100, device="cuda").bfloat16()      # K = 100 is not a multiple of 8: no kernel route
    w = torch.randn(32, 100, device="cuda").bfloat16()
    prev = ops.dispatch.set_strict(True)
    try:
        with pytest.raises(RuntimeError, match="strict mode"):
            ops.linear_fwd(x, w)
        ops.dispatch.set_strict(False)
        ops.dispatch.FALLBACKS.clear()
        ops.linear_fwd(x, w)
        assert ops.dispatch.FALLBACKS.get("linear_fwd") == 1
    finally:
        ops.dispatch.set_strict(prev)
        ops.dispatch.FALLBACKS.clear()


@pytest.mark.parametrize("kind", ["transformer", "mamba2"])
def test_engine_grad_parity_at_headline_interface_width(kind):
    """A 2-layer slice with the headline interface shape: 8 sequence regions, interface width 128, basis blocks of 16 (so the
    loss cotangent rides as the lone 17th direction of the last block) against dense autograd in fp32 on the CPU."""
    torch.manual_seed(0)
    if kind == "transformer":
        spec = BackboneSpec(name="transformer", dim=256, layers=2, n_heads=4, d_conv=0, d_intermediate=512)
    else:
        spec = BackboneSpec(name="mamba2", dim=256, layers=2, d_state=128, headdim=64, expand=2, d_conv=4, chunk_size=128)
    iface = VectorMLPInterface(feature_dim=256, num_regions=8, interface_width=128, interface_map_hidden_dim=256)
    cpu_model = LBILanguageModel(vocab_size=1024, layers_per_region=1, backbone_spec=spec, interface=iface, region_axis="sequence",
                                 num_sequence_regions=8, tie_embeddings=True)
    gpu_model = copy.deepcopy(cpu_model).cuda()
    torch.manual_seed(1)
    ids, tgt = torch.randint(0, 1024, (2, 1024)), torch.randint(0, 1024, (2, 1024))
    loss = F.cross_entropy(cpu_model(ids).float().reshape(-1, 1024), tgt.reshape(-1))
    want = AutogradEngine().backward(model=cpu_model, loss=loss).grad_map
    engine = FastLBIEngine(gpu_model, lr=1e-3, basis_chunk=16)
    res = engine.backward(ids.cuda(), tgt.cuda())
    from lbi_b200 import ops

    assert ops.ext().kernel_status(res.loss) == 0
    assert abs(float(res.loss) - float(loss.detach())) < 5e-3 * max(1.0, abs(float(loss.detach())))
    got = engine.named_grads()
    for name, ref in want.items():
        if ref is None:
            continue
        g = got[name].float().cpu()
        rel = float((g - ref).norm() / (ref.norm() + 1e-12))
        assert torch.allclose(g, ref, atol=5e-2, rtol=5e-2), f"{name}: max abs err {float((g - ref).abs().max()):.3e}"
        # a gradient that is tiny as a whole (a two-element scale whose norm is 1e-4) is noise in bf16: the state cotangent it is
        # a dot product with carries 1e-2 relative rounding, and the elementwise bar above already covers it
        assert rel < 1.5e-1 or float(ref.norm()) < 1e-3, f"{name}: rel-L2 {rel:.3e}"
