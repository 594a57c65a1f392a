"""Checkpoints in the reference's interchange format plus expert-parallel shard conversion.

Format (reference ``tests/test_checkpoint.py:41-46``): ``torch.save({"model": state_dict,
"opt": optimizer.state_dict(), "gen": generator_state})``.  The canonical (unsharded) key set is
the reference's: ``tok.weight``, per block ``n1``, ``n2``, ``attn.wqkv.weight``, ``attn.wo.weight``,
dense ``ffn.w13.weight`` / ``ffn.w2.weight``, MoE ``ffn.w13[E,D,2d]``, ``ffn.w2[E,d,D]``,
``ffn.router.weight``, ``ffn.router.bias`` (persistent: the aux-loss-free balancing state),
``ffn.shared.w13.weight`` / ``ffn.shared.w2.weight``, then ``nf`` and ``head.weight``.

Expert-parallel runs hold ``w13[epr, ...]`` / ``w2[epr, ...]`` per rank (rank r owns experts
``[r*epr, (r+1)*epr)``, reference ``terrace/ep_dist.py:90``).  ``shard_state_dict`` /
``merge_state_dicts`` convert between the canonical dict and per-rank shards.
"""
from __future__ import annotations

import torch

EXPERT_KEYS = (".ffn.w13", ".ffn.w2", ".ffn.tier0.w13", ".ffn.tier0.w2", ".ffn.tier1.w13",
               ".ffn.tier1.w2")


def save_checkpoint(path, model, optimizer=None, generator=None, extra: dict | None = None):
    blob = {"model": model.state_dict()}
    if optimizer is not None:
        blob["opt"] = optimizer.state_dict()
    if generator is not None:
        blob["gen"] = generator.get_state()
    if extra:
        blob.update(extra)
    torch.save(blob, path)


def load_checkpoint(path, model, optimizer=None, generator=None, map_location="cpu",
                    strict: bool = True) -> dict:
    blob = torch.load(path, map_location=map_location, weights_only=False)
    model.load_state_dict(blob["model"], strict=strict)
    if optimizer is not None and "opt" in blob:
        optimizer.load_state_dict(blob["opt"])
    if generator is not None and "gen" in blob:
        generator.set_state(blob["gen"])
    return blob


def _is_expert_key(key: str) -> bool:
    return any(key.endswith(s) for s in EXPERT_KEYS)


def shard_state_dict(state: dict, rank: int, world: int) -> dict:
    """Canonical state dict -> the dict rank ``rank`` of an EP group of ``world`` loads: routed
    expert tensors are sliced along the expert dimension, everything else is replicated."""
    out = {}
    for key, val in state.items():
        if _is_expert_key(key) and val.dim() == 3:
            E = val.shape[0]
            if E % world:
                raise ValueError(f"{key}: {E} experts do not divide over {world} ranks")
            epr = E // world
            out[key] = val[rank * epr:(rank + 1) * epr].clone()
        else:
            out[key] = val
    return out


def merge_state_dicts(shards: list) -> dict:
    """Per-rank EP shards (rank order) -> canonical state dict.  Replicated tensors are taken
    from rank 0 after checking that all ranks agree."""
    first = shards[0]
    out = {}
    for key, val in first.items():
        if _is_expert_key(key) and val.dim() == 3:
            out[key] = torch.cat([s[key] for s in shards], dim=0)
        else:
            for r, s in enumerate(shards[1:], 1):
                if not torch.equal(s[key], val):
                    raise ValueError(f"replicated tensor {key} differs between rank 0 and {r}")
            out[key] = val
    return out
