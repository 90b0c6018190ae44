"""Decode throughput of a sequence-axis LBI model: cached steps against re-evaluating the span prefix.

    python -m lbi_b200.benchmarks.time_decode [--backbone transformer] [--dim 256] [--layers 4] [--regions 4] [--total-len 512]
                                              [--new-tokens 128] [--batch 1] [--device cpu|cuda]

Prints one JSON line: tokens / s of ``generate`` in both modes and their ratio, plus the bytes of decode state alive at the end
(one region span of per-block state and the interface state, whatever the sequence length).  Wall-clock timing around a
synchronised device; random-init weights, random prompt.
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from ..backbones import BackboneSpec
from ..inference import IncrementalLBIDecoder, generate
from ..interfaces import VectorMLPInterface
from ..models import LBILanguageModel


def build_model(backbone: str, dim: int, layers: int, regions: int, vocab: int, device: torch.device) -> LBILanguageModel:
    extra = dict(n_heads=max(1, dim // 64), d_conv=0) if backbone == "transformer" else dict(d_state=64, headdim=64, chunk_size=64, d_conv=4)
    spec = BackboneSpec(name=backbone, dim=dim, layers=layers, **extra)
    iface = VectorMLPInterface(feature_dim=dim, num_regions=regions, interface_width=64, interface_map_hidden_dim=dim)
    return LBILanguageModel(vocab_size=vocab, layers_per_region=1, backbone_spec=spec, interface=iface, region_axis="sequence",
                            num_sequence_regions=regions, tie_embeddings=True).to(device).eval()


def state_bytes(decoder: IncrementalLBIDecoder) -> int:
    def walk(obj) -> int:
        if isinstance(obj, torch.Tensor):
            return obj.numel() * obj.element_size()
        if isinstance(obj, dict):
            return sum(walk(v) for v in obj.values())
        if isinstance(obj, (list, tuple)):
            return sum(walk(v) for v in obj)
        return 0

    return walk(decoder._block_states) + walk(decoder.state) + walk(decoder._span_tokens) + walk(decoder._feature_sum)


def timed_generate(model, prompt, new_tokens: int, total_len: int, use_cache: bool) -> float:
    if prompt.is_cuda:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    generate(model, prompt, new_tokens, total_len=total_len, use_cache=use_cache)
    if prompt.is_cuda:
        torch.cuda.synchronize()
    return new_tokens * prompt.shape[0] / (time.perf_counter() - t0)


def main(argv: list[str] | None = None) -> dict:
    p = argparse.ArgumentParser(description="Decode throughput: cached steps vs span recomputation")
    p.add_argument("--backbone", choices=("transformer", "mamba2", "mamba3"), default="transformer")
    p.add_argument("--dim", type=int, default=256)
    p.add_argument("--layers", type=int, default=4)
    p.add_argument("--regions", type=int, default=4)
    p.add_argument("--total-len", type=int, default=512)
    p.add_argument("--prompt-len", type=int, default=16)
    p.add_argument("--new-tokens", type=int, default=128)
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--vocab", type=int, default=1024)
    p.add_argument("--device", choices=("cpu", "cuda"), default="cuda" if torch.cuda.is_available() else "cpu")
    ns = p.parse_args(argv)
    device = torch.device(ns.device)
    torch.manual_seed(0)
    model = build_model(ns.backbone, ns.dim, ns.layers, ns.regions, ns.vocab, device)
    prompt = torch.randint(0, ns.vocab, (ns.batch, ns.prompt_len), device=device)
    timed_generate(model, prompt, min(8, ns.new_tokens), ns.total_len, True)  # warm-up
    cached = timed_generate(model, prompt, ns.new_tokens, ns.total_len, True)
    recompute = timed_generate(model, prompt, ns.new_tokens, ns.total_len, False)
    decoder = IncrementalLBIDecoder(model, ns.total_len, use_cache=True)
    decoder.append(torch.randint(0, ns.vocab, (ns.batch, ns.prompt_len + ns.new_tokens), device=device))
    out = {"backbone": ns.backbone, "dim": ns.dim, "layers": ns.layers, "regions": ns.regions, "total_len": ns.total_len,
           "new_tokens": ns.new_tokens, "batch": ns.batch, "device": ns.device, "cached_tokens_per_s": cached,
           "recompute_tokens_per_s": recompute, "speedup": cached / recompute, "decode_state_bytes": state_bytes(decoder)}
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
