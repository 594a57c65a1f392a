"""Data-parallel gradient synchronisation for the replicated (non-expert) parameters.

In an expert-parallel job every rank holds the same attention, router, shared-expert, embedding
and head weights but different tokens, so their gradients are averaged over the ranks after the
backward pass; the routed-expert weights are sharded, each rank owns its experts alone, and
their gradients already hold the contributions of every rank's tokens (they arrived through the
dispatch), so they are left alone.

``DPGradSync`` flattens the replicated gradients into a few large buckets (one NCCL call each:
on NVSwitch the cost of an all-reduce is launch latency plus bytes over the in-switch reduction,
not a per-link cost, so buckets are sized for few launches) and all-reduces them on a side
stream so that the copy-back overlaps the optimizer's work on earlier buckets.

The reference has no data-parallel training loop (its only train step is single-device,
``tests/test_checkpoint.py:16-23``); this is new here, for the multi-GPU decoder benchmark.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

EXPERT_PARAM_SUFFIXES = (".w13", ".w2")


def is_expert_sharded(name: str, module_types: dict) -> bool:
    """True for the routed-expert weights of an expert-parallel layer."""
    owner = name.rsplit(".", 1)[0]
    return name.endswith(EXPERT_PARAM_SUFFIXES) and module_types.get(owner) == "EPTerracedMoE"


class DPGradSync:
    def __init__(self, model: torch.nn.Module, bucket_mb: float = 256.0, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        types = {n: type(m).__name__ for n, m in model.named_modules()}
        self.replicated = [(n, p) for n, p in model.named_parameters()
                           if p.requires_grad and not is_expert_sharded(n, types)]
        self.sharded = [(n, p) for n, p in model.named_parameters()
                        if p.requires_grad and is_expert_sharded(n, types)]
        self.buckets, cur, cur_bytes = [], [], 0
        limit = int(bucket_mb * 1024 * 1024)
        for _, p in self.replicated:
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > limit or cur[0].dtype != p.dtype):
                self.buckets.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
        if cur:
            self.buckets.append(cur)
        self.calls = 0

    def sync(self) -> None:
        """Average the replicated gradients over the ranks (no-op on one rank)."""
        if self.world == 1:
            return
        for bucket in self.buckets:
            grads = [p.grad for p in bucket if p.grad is not None]
            if not grads:
                continue
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat, group=self.group)
            flat.div_(self.world)
            self.calls += 1
            off = 0
            for g in grads:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g))
                off += n
