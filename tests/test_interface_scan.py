"""Suffix scans of interface Jacobians against a sequential product (CPU statements; the CUDA kernels are
checked against the same statements in test_gpu_kernels.py)."""
import pytest
import torch

from lbi_b200 import ops
from lbi_b200.backward import (
    compose_suffix_jacobian_t, propagate_state_adjoint_affine, propagate_state_adjoint_by_chain,
    propagate_state_adjoint_from_last_region_input, propagate_state_adjoint_with_jacobian_scan,
)


def _manual(mats):
    b, k, r, _ = mats.shape
    out = [torch.eye(r).expand(b, r, r).clone()]
    for idx in range(k - 1, -1, -1):
        out.append(mats[:, idx].float() @ out[-1])
    return torch.stack(out[::-1], dim=1)


def _atol(k, r):
    if r >= 256:
        return 0.7
    if r >= 128:
        return 0.25
    return 3e-2 if (k >= 8 or r >= 16) else 2e-5


@pytest.mark.parametrize("b,k,r", [(1, 1, 1), (2, 1, 4), (1, 2, 2), (3, 5, 8), (1, 8, 16), (1, 16, 64)])
def test_suffix_scan_matches_sequential_product(b, k, r):
    torch.manual_seed(0)
    mats = torch.randn(b, k, r, r) / max(1.0, r ** 0.5)
    keep = mats.clone()
    out = ops.suffix_scan_pullbacks(mats)
    assert out.shape == (b, k + 1, r, r) and out.dtype == torch.float32
    assert torch.allclose(out, _manual(mats), atol=_atol(k, r), rtol=1e-5)
    assert torch.equal(mats, keep), "input must not be modified"
    assert torch.equal(out[:, k], torch.eye(r).expand(b, r, r))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_low_precision_inputs_give_fp32(dtype):
    torch.manual_seed(1)
    mats = (torch.randn(2, 4, 8, 8) / 3).to(dtype)
    out = ops.suffix_scan_pullbacks(mats)
    assert out.dtype == torch.float32
    assert torch.allclose(out, _manual(mats), atol=0.2, rtol=5e-3)


def test_order_of_noncommuting_factors():
    a = torch.tensor([[1.0, 2.0], [0.0, 1.0]])
    b = torch.tensor([[1.0, 0.0], [3.0, 1.0]])
    out = ops.suffix_scan_pullbacks(torch.stack([a, b]).unsqueeze(0))
    assert torch.allclose(out[0, 0], a @ b)
    assert torch.allclose(out[0, 1], b)
    assert not torch.allclose(out[0, 0], b @ a)


def test_propagation_helpers_agree():
    torch.manual_seed(2)
    bsz, k, r = 2, 5, 6
    jac = [torch.randn(bsz, r, r) / 3 for _ in range(k)]
    top = torch.randn(bsz, r)
    g = propagate_state_adjoint_with_jacobian_scan(jac, top)
    cur, manual = top, [top]
    for m in reversed(jac):
        cur = torch.einsum("bij,bj->bi", m, cur)
        manual.append(cur)
    for a, b in zip(g, manual[::-1]):
        assert torch.allclose(a, b, atol=1e-5)
    # seeding at the input state of the last region ignores the last Jacobian
    g2 = propagate_state_adjoint_from_last_region_input(jac, top)
    assert len(g2) == k and torch.allclose(g2[-1], top)
    suffix = compose_suffix_jacobian_t(jac[:-1])
    assert torch.allclose(g2[0], torch.einsum("bij,bj->bi", suffix[0], top), atol=1e-5)


def test_affine_scan_matches_chain():
    torch.manual_seed(3)
    bsz, k, r = 3, 6, 5
    jac = [torch.randn(bsz, r, r) / 2 for _ in range(k - 1)]
    off = [torch.randn(bsz, r) for _ in range(k)]
    a = propagate_state_adjoint_affine(jac, off)
    b = propagate_state_adjoint_by_chain(jac, off)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=1e-5)
    assert torch.allclose(propagate_state_adjoint_affine([], off[:1])[0], off[0])
