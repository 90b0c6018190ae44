"""Property tests (hypothesis) of the host-side planning code: region cuts, rank placement, the flat parameter layout and the
suffix-scan helpers.  Every property is one the engine relies on without checking it at run time."""
import pytest
import torch
from torch import nn

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

from lbi_b200.backward.suffix_scan import (compose_suffix_jacobian_t, propagate_state_adjoint_affine,  # noqa: E402
                                           propagate_state_adjoint_by_chain, propagate_state_adjoint_with_jacobian_scan)
from lbi_b200.models.region_plan import RegionPlacement, RegionPlan, build_region_ranges, split_tokens  # noqa: E402
from lbi_b200.parallel.flat import FlatParams  # noqa: E402

FAST = settings(max_examples=60, deadline=None)


@FAST
@given(layers=st.integers(1, 200), per=st.integers(1, 50))
def test_depth_ranges_tile_the_stack(layers, per):
    ranges = build_region_ranges(layers, per)
    assert ranges[0][0] == 0 and ranges[-1][1] == layers
    assert all(a[1] == b[0] for a, b in zip(ranges[:-1], ranges[1:]))
    assert all(0 < e - s <= per for s, e in ranges) and all(e - s == per for s, e in ranges[:-1])
    plan = RegionPlan.depth(layers, per)
    assert plan.num_regions == len(ranges) and plan.token_ranges(17) == [(0, 17)] * plan.num_regions
    assert [plan.region_has_loss(k) for k in range(plan.num_regions)] == [False] * (plan.num_regions - 1) + [True]


@FAST
@given(data=st.data())
def test_token_spans_tile_the_sequence_and_differ_by_at_most_one(data):
    regions = data.draw(st.integers(1, 64))
    seq_len = data.draw(st.integers(regions, 5000))
    spans = split_tokens(seq_len, regions)
    sizes = [e - s for s, e in spans]
    assert spans[0][0] == 0 and spans[-1][1] == seq_len and all(a[1] == b[0] for a, b in zip(spans[:-1], spans[1:]))
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    plan = RegionPlan.sequence(3, regions)
    assert plan.token_ranges(seq_len) == spans and plan.shares_backbone_parameters and all(plan.region_has_loss(k) for k in range(regions))


@FAST
@given(per=st.integers(1, 16), world=st.integers(1, 16))
def test_placement_is_contiguous_and_balanced(per, world):
    place = RegionPlacement(per * world, world)
    owners = [place.owner(k) for k in range(per * world)]
    assert owners == sorted(owners) and all(owners.count(r) == per for r in range(world))
    assert all(list(place.regions_of(r)) == [k for k, o in enumerate(owners) if o == r] for r in range(world))
    if world > 1:
        with pytest.raises(ValueError):
            RegionPlacement(per * world + 1, world)


@FAST
@given(shapes=st.lists(st.lists(st.integers(1, 9), min_size=1, max_size=3), min_size=1, max_size=6), world=st.integers(1, 8),
       align=st.sampled_from([1, 8, 64]))
def test_flat_layout_slots_are_aligned_disjoint_and_alias_the_parameters(shapes, world, align):
    model = nn.ParameterList([nn.Parameter(torch.randn(*s)) for s in shapes])
    before = [p.detach().clone() for p in model]
    flat = FlatParams(model, world_size=world, shadow_dtype=None, align=align)
    slots = sorted(flat.slots.values(), key=lambda s: s.offset)
    assert all(s.offset % align == 0 for s in slots) and all(a.offset + a.numel <= b.offset for a, b in zip(slots[:-1], slots[1:]))
    assert flat.total % (align * world) == 0 and flat.shard * world == flat.total and slots[-1].offset + slots[-1].numel <= flat.total
    for p, old in zip(model, before):
        assert torch.equal(p.detach(), old) and p.data_ptr() == flat.view(flat.params, flat.name_of(p)).data_ptr()
    with torch.no_grad():
        flat.params.mul_(2.0)  # the parameters are views: an update of the flat buffer is an update of the model
    assert all(torch.equal(p.detach(), 2.0 * old) for p, old in zip(model, before))
    assert float(flat.grads.abs().sum()) == 0.0 and set(flat.grad_map()) == set(flat.slots)


@FAST
@given(k=st.integers(1, 6), r=st.integers(1, 5), b=st.integers(1, 3), seed=st.integers(0, 10_000))
def test_suffix_products_and_affine_recursion_agree_with_the_chain(k, r, b, seed):
    g = torch.Generator().manual_seed(seed)
    mats = [torch.randn(b, r, r, generator=g, dtype=torch.float64) * 0.7 for _ in range(k)]
    suffix = compose_suffix_jacobian_t(mats)
    assert len(suffix) == k + 1 and torch.allclose(suffix[-1], torch.eye(r, dtype=suffix[-1].dtype).expand(b, r, r))
    for i in range(k):  # S_i = A_i^T S_{i+1}
        assert torch.allclose(suffix[i].double(), mats[i] @ suffix[i + 1].double(), atol=1e-5, rtol=1e-5)
    top = torch.randn(b, r, generator=g, dtype=torch.float64)
    states = propagate_state_adjoint_with_jacobian_scan(mats, top)
    assert len(states) == k + 1 and torch.allclose(states[-1].double(), top)
    for i in range(k):
        assert torch.allclose(states[i].double(), torch.einsum("bij,bj->bi", mats[i], states[i + 1].double()), atol=1e-5, rtol=1e-5)
    offsets = [torch.randn(b, r, generator=g, dtype=torch.float64) for _ in range(k + 1)]
    scanned, chained = propagate_state_adjoint_affine(mats, offsets), propagate_state_adjoint_by_chain(mats, offsets)
    assert len(scanned) == len(chained) == k + 1
    for a, c in zip(scanned, chained):
        assert torch.allclose(a.double(), c.double(), atol=1e-4, rtol=1e-4)


@settings(max_examples=25, deadline=None)
@given(lines=st.lists(st.text(alphabet="abcde é", min_size=1, max_size=30), min_size=1, max_size=12),
       shard_tokens=st.integers(1, 40), seq_len=st.integers(1, 6))
def test_shard_writer_and_sampler_round_trip(tmp_path_factory, lines, shard_tokens, seq_len):
    """Whatever the text and the shard size, the shards concatenate to the token stream and every sampled window is a contiguous
    piece of one shard."""
    import json

    import numpy as np

    from lbi_b200.data.bpe_tokenizer import ByteBPETokenizer
    from lbi_b200.data.pretokenize_corpus import write_shards
    from lbi_b200.data.token_shards import TokenShardCorpus, sample_batch_token_shards

    root = tmp_path_factory.mktemp("shards")
    text = root / "t.txt"
    text.write_text("\n".join(lines) + "\n", encoding="utf-8")
    tok = ByteBPETokenizer(merges=[], token_bytes={i: bytes([i]) for i in range(256)})  # no merges: one token per byte
    manifest = write_shards("train", text, tok, root / "out", shard_tokens)
    meta = json.loads(manifest.read_text())
    joined = np.concatenate([np.fromfile(root / "out" / s["path"], dtype=np.int32) for s in meta["shards"]])
    assert meta["num_tokens_total"] == len(joined) and joined.tolist() == list(text.read_bytes())
    corpus = TokenShardCorpus(manifest)
    longest = max(s["num_tokens"] for s in meta["shards"])
    gen = torch.Generator().manual_seed(0)
    if longest < seq_len + 1:
        with pytest.raises(ValueError):
            sample_batch_token_shards(corpus, batch_size=2, seq_len=seq_len, generator=gen, device=torch.device("cpu"))
        return
    x, y = sample_batch_token_shards(corpus, batch_size=4, seq_len=seq_len, generator=gen, device=torch.device("cpu"))
    assert x.shape == y.shape == (4, seq_len) and torch.equal(x[:, 1:], y[:, :-1])
    shards = [np.fromfile(root / "out" / s["path"], dtype=np.int32).tolist() for s in meta["shards"]]
    for row_x, row_y in zip(x.tolist(), y.tolist()):
        window = row_x + row_y[-1:]
        assert any(window == sh[i : i + seq_len + 1] for sh in shards for i in range(len(sh) - seq_len))
