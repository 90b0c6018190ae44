"""Translate LBI-1 state dicts (``embedding``, ``blocks``, ``norm``, ``lm_head``, ``input_to_message``,
``message_to_hidden``, ``hidden_to_message``, ``message_norm``, ``message_alpha``) into the owned LBI-2 schema
(reference legacy/lbi1_checkpoint.py:9-42).  Duplicate keys that collapse onto one target (``backbone.blocks.*`` and
``blocks.*``) must carry equal tensors."""
from __future__ import annotations

from collections import OrderedDict
from collections.abc import Mapping

import torch

_PREFIX_MIGRATIONS = (
    ("embedding.", "canvas.embedding."),
    ("norm.", "readout.norm."),
    ("lm_head.", "readout.lm_head."),
    ("backbone.", "region_backend.backbone."),
    ("blocks.", "region_backend.backbone.blocks."),
    ("input_to_message.", "interface.initial_encoder."),
    ("message_to_hidden.", "interface.decoders."),
    ("hidden_to_message.", "interface.encoders."),
    ("message_norm.", "interface.norms."),
)
_LBI1_MARKERS = ("input_to_message.", "message_to_hidden.", "hidden_to_message.", "message_norm.", "message_alpha")


def is_lbi1_state_dict(state_dict: Mapping[str, torch.Tensor]) -> bool:
    keys = [str(k) for k in state_dict]
    return any(k.startswith(_LBI1_MARKERS) for k in keys) and not any(k.startswith("interface.") for k in keys)


def migrate_lbi1_state_key(key: str) -> str:
    if key == "message_alpha":
        return "interface.update_scale"
    for old, new in _PREFIX_MIGRATIONS:
        if key.startswith(old):
            return new + key[len(old):]
    return key


def migrate_lbi1_state_dict(state_dict: Mapping[str, torch.Tensor], *, tie_embeddings: bool | None = None) -> "OrderedDict[str, torch.Tensor]":
    """Returns a dict that loads strictly into ``LBILanguageModel``.

    ``tie_embeddings=True`` drops ``readout.lm_head.weight``: LBI-1 stores the tied head as a second copy of the
    embedding, while the owned model has no such parameter.  With ``None`` the copy is dropped when it equals the
    embedding."""
    out: OrderedDict[str, torch.Tensor] = OrderedDict()
    for key, value in state_dict.items():
        new_key = migrate_lbi1_state_key(key)
        if new_key in out:
            if torch.equal(out[new_key], value):
                continue
            raise ValueError(f"LBI-1 migration produced duplicate key with different value: {new_key}")
        out[new_key] = value
    head, emb = out.get("readout.lm_head.weight"), out.get("canvas.embedding.weight")
    if head is not None and emb is not None:
        tied = tie_embeddings if tie_embeddings is not None else (head.shape == emb.shape and torch.equal(head, emb))
        if tied:
            del out["readout.lm_head.weight"]
    return out
