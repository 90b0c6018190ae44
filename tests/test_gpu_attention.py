"""Attention input pullback over a basis: tcgen05 kernel and the library loop against the dense fp32 formula."""
import math

import pytest
import torch

from lbi_b200 import ops
from lbi_b200.ops import reference as ref
from lbi_b200.ops.attention import attention_input_pullback_basis

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(b, h, t, dh, p, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    q, k, v = (torch.randn(b, h, t, dh, device=DEV, generator=g).bfloat16() for _ in range(3))
    do = torch.randn(b, p, h, t, dh, device=DEV, generator=g).bfloat16()
    return q, k, v, do


def _check(got, want, what):
    for name, a, w in zip(("dQ", "dK", "dV"), got, want):
        err = (a.float() - w).abs().max().item()
        scale = w.abs().max().item()
        assert err <= 3e-2 * scale + 1e-3, f"{what} {name}: max err {err:.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("b,h,t,p", [(1, 1, 128, 1), (2, 2, 256, 4), (1, 3, 384, 5), (2, 1, 512, 7), (1, 2, 1024, 3)])
def test_tcgen05_pullback_matches_dense(b, h, t, p):
    q, k, v, do = _inputs(b, h, t, 64, p)
    scale = 1.0 / math.sqrt(64)
    want = ref.attention_input_pullback_dense(q, k, v, do, scale, True)
    got = attention_input_pullback_basis(q, k, v, do, scale=scale, causal=True, kernel_mode="tcgen05_pblock")
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(q) == 0, "a bounded wait inside the attention kernels ran out"
    _check(got, want, "tcgen05")


def test_library_loop_matches_dense():
    q, k, v, do = _inputs(2, 2, 256, 64, 3, seed=1)
    scale = 0.2
    want = ref.attention_input_pullback_dense(q, k, v, do, scale, True)
    got = attention_input_pullback_basis(q, k, v, do, scale=scale, causal=True, kernel_mode="fa2_loop")
    _check(got, want, "fa2_loop")


def test_dense_mode_and_cpu_path_agree():
    q, k, v, do = _inputs(1, 2, 64, 32, 2, seed=2)
    want = ref.attention_input_pullback_dense(q.float().cpu(), k.float().cpu(), v.float().cpu(), do.float().cpu(), 0.3, True)
    got = attention_input_pullback_basis(q, k, v, do, scale=0.3, causal=True, kernel_mode="dense")
    for a, w in zip(got, want):
        assert (a.float().cpu() - w).abs().max().item() <= 3e-2 * w.abs().max().item() + 1e-3


def test_tcgen05_pullback_is_deterministic():
    q, k, v, do = _inputs(1, 2, 256, 64, 4, seed=3)
    a = attention_input_pullback_basis(q, k, v, do, causal=True, kernel_mode="tcgen05_pblock")
    b = attention_input_pullback_basis(q, k, v, do, causal=True, kernel_mode="tcgen05_pblock")
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("b,h,t", [(1, 1, 128), (2, 2, 256), (1, 3, 384), (2, 1, 640), (1, 2, 2048)])
def test_tcgen05_forward_matches_fp32_attention(b, h, t):
    from lbi_b200.ops.attention import flash_forward_packed

    g = torch.Generator(device=DEV).manual_seed(t)
    qkv = torch.randn(b * t, 3 * h * 64, device=DEV, generator=g).bfloat16()
    scale = 1.0 / math.sqrt(64)
    out, lse = flash_forward_packed(qkv, b, t, h, h, 64, scale, kernel_mode="tcgen05")
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(qkv) == 0, "a bounded wait inside the attention forward kernel ran out"
    q, k, v = (x.reshape(b, t, h, 64).permute(0, 2, 1, 3).float() for x in qkv.split(h * 64, dim=1))
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * scale
    s = s.masked_fill(torch.ones(t, t, device=DEV, dtype=torch.bool).triu(1), float("-inf"))
    want_lse = torch.logsumexp(s, dim=-1)
    want = torch.einsum("bhqk,bhkd->bhqd", torch.softmax(s, dim=-1), v).permute(0, 2, 1, 3).reshape(b * t, h * 64)
    assert (lse - want_lse).abs().max().item() < 2e-3
    assert (out.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3
    lib_out, lib_lse = flash_forward_packed(qkv, b, t, h, h, 64, scale, kernel_mode="fa2")
    assert (lib_out.float() - out.float()).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3
    assert (lib_lse - lse).abs().max().item() < 2e-3


@pytest.mark.parametrize("interleaved", [False, True])
def test_pullback_epilogue_rotates_dq_dk_back(interleaved):
    from lbi_b200.backbones.transformer.rope import rope_tables
    from lbi_b200.ops.attention import flash_forward_packed, pullback_packed

    b, h, t, p = 2, 3, 384, 5
    g = torch.Generator(device=DEV).manual_seed(9)
    qkv = torch.randn(b * t, 3 * h * 64, device=DEV, generator=g).bfloat16()
    do = torch.randn(p * b * t, h * 64, device=DEV, generator=g).bfloat16()
    scale = 0.125
    o, lse = flash_forward_packed(qkv, b, t, h, h, 64, scale)
    cos, sin = rope_tables(t, 64, 10000.0, torch.device(DEV))
    plain = pullback_packed(do, qkv, o, lse, b, t, h, h, 64, scale, kernel_mode="tcgen05_pblock")
    want = ops.rope_qkv(plain.clone(), cos, sin, h, h, 64, t, interleaved, inverse=True)
    got = pullback_packed(do, qkv, o, lse, b, t, h, h, 64, scale, kernel_mode="tcgen05_pblock", rope=(cos, sin, interleaved))
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(qkv) == 0
    tol = 2e-2 * want.float().abs().max().item()
    assert (got.float() - want.float()).abs().max().item() <= tol
    # dv is not rotated
    assert torch.equal(got[:, 2 * h * 64 :], plain[:, 2 * h * 64 :])


@pytest.mark.parametrize("heads,kv_heads", [(8, 4), (4, 1)])
def test_grouped_kv_heads_run_on_the_tcgen05_kernels(heads, kv_heads):
    """Grouped-query attention (the paper's canonical Transformer is 8 heads / 4 kv heads): forward and the basis pullback
    go through the expand / reduce kernels around the tcgen05 kernels and match the library path on the packed layout."""
    from lbi_b200.ops.attention import flash_forward_packed, pullback_packed

    b, t, p = 2, 256, 3
    g = torch.Generator(device=DEV).manual_seed(heads)
    qkv = torch.randn(b * t, (heads + 2 * kv_heads) * 64, device=DEV, generator=g).bfloat16()
    do = torch.randn(p * b * t, heads * 64, device=DEV, generator=g).bfloat16()
    scale = 0.125
    prev = ops.dispatch.set_strict(True)
    try:
        before = ops.dispatch.KERNEL_LAUNCHES["count"]
        o, lse = flash_forward_packed(qkv, b, t, heads, kv_heads, 64, scale)
        got = pullback_packed(do, qkv, o, lse, b, t, heads, kv_heads, 64, scale)
        assert ops.dispatch.KERNEL_LAUNCHES["count"] - before >= 6
    finally:
        ops.dispatch.set_strict(prev)
    o_lib, lse_lib = flash_forward_packed(qkv, b, t, heads, kv_heads, 64, scale, kernel_mode="fa2")
    want = pullback_packed(do, qkv, o_lib, lse_lib, b, t, heads, kv_heads, 64, scale, kernel_mode="fa2_loop")
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(qkv) == 0
    assert got.shape == want.shape == (p * b * t, (heads + 2 * kv_heads) * 64)
    assert (o.float() - o_lib.float()).abs().max().item() <= 2e-2 * o_lib.float().abs().max().item() + 1e-3
    assert (got.float() - want.float()).abs().max().item() <= 3e-2 * want.float().abs().max().item() + 1e-3


@pytest.mark.parametrize("t,p", [(256, 4), (512, 3)])
def test_fp16_runs_on_the_tcgen05_kernels(t, p):
    """fp16 (the reference kernel's only dtype, tolerance 2e-2 for its fused fp16 path) through the public basis-pullback entry
    point against the O(T^2) fp32 formula."""
    from lbi_b200.ops.attention import attention_input_pullback_basis

    b, h = 2, 2
    g = torch.Generator(device=DEV).manual_seed(t + p)
    q, k, v = (torch.randn(b, h, t, 64, device=DEV, generator=g).half() for _ in range(3))
    do = torch.randn(b, p, h, t, 64, device=DEV, generator=g).half()
    prev = ops.dispatch.set_strict(True)
    try:
        got = attention_input_pullback_basis(q, k, v, do, causal=True, kernel_mode="tcgen05_pblock")
    finally:
        ops.dispatch.set_strict(prev)
    torch.cuda.synchronize()
    assert ops.ext().kernel_status(q) == 0
    want = attention_input_pullback_basis(q.float(), k.float(), v.float(), do.float(), causal=True, kernel_mode="dense")
    for name, a, w in zip(("dQ", "dK", "dV"), got, want):
        assert a.dtype == torch.float16
        err = (a.float() - w).abs().max().item()
        assert err <= 2e-2 * w.abs().max().item() + 2e-3, f"{name}: {err:.3e}"
