"""Residency measurement: the two numbers the memory verdict of ``sim/codesign.py`` assumes.

    python -m terracemoe_simulator_b200.bench.residency --layers 4 8 --batch 1 2 --seq 4096

``codesign.residency`` adds expert weights and optimizer state (arithmetic) to two quantities that
are not arithmetic: the activation bytes a training step keeps per token and layer, and the share
of device memory lost to the allocator, the CUDA context, communication buffers and fragmentation.
Until they are measured every fit / does-not-fit verdict carries ``ASSUMED`` in its tag.

Protocol.  Run the decoder training step of ``bench/train_step.py`` at several (layers, tokens)
points; at each record the peak bytes the tensor allocator handed out, the peak it reserved, and
what the device reports as used (which also counts the context and the peer-memory arenas that
are allocated outside the tensor allocator).  Then

    peak_allocated - static = a * tokens * layers + b * tokens + c          (least squares)

with ``static`` the parameter, gradient and optimizer bytes, gives ``a``, the activation bytes per
token and layer (``b`` collects embeddings, logits and the loss, ``c`` the workspace), and

    overhead_frac = max over points of (device_used - peak_allocated) / capacity

gives the second.  ``fit_profile`` is plain arithmetic and is tested on a CPU; ``measure_point``
needs a CUDA device unless a probe is injected.

The reference describes this protocol and never ran it (``docs/11-residency-measurement.md``,
``sim/codesign.py:140-176``).
"""
from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict, dataclass


@dataclass
class Sample:
    layers: int
    tokens: int                 # tokens per step on this device
    static_bytes: float         # parameters + gradients + optimizer state
    peak_allocated: float       # tensor allocator, peak over the step
    peak_reserved: float        # tensor allocator, reserved from the driver
    device_used: float          # what the device reports as in use (context and arenas included)


def fit_profile(samples, capacity_bytes: float, name: str = "measured", recompute: str = "none"):
    """Least-squares fit of the activation model and the overhead share.  Needs at least three
    samples that vary both ``layers`` and ``tokens``.  Returns ``(MemoryProfile, details)``."""
    import numpy as np
    from ..sim.codesign import MemoryProfile
    if len(samples) < 3:
        raise ValueError("need at least three (layers, tokens) points")
    if len({s.layers for s in samples}) < 2 or len({s.tokens for s in samples}) < 2:
        raise ValueError("the points must vary both the layer count and the token count")
    A = np.array([[s.tokens * s.layers, s.tokens, 1.0] for s in samples], dtype=np.float64)
    y = np.array([s.peak_allocated - s.static_bytes for s in samples], dtype=np.float64)
    scale = A.max(axis=0)
    coef, *_ = np.linalg.lstsq(A / scale, y, rcond=None)
    a, b, c = (coef / scale).tolist()
    pred = A @ np.array([a, b, c])
    rel = float(np.max(np.abs(pred - y) / np.maximum(np.abs(y), 1.0)))
    overhead = max((s.device_used - s.peak_allocated) / capacity_bytes for s in samples)
    prof = MemoryProfile(name=name, activation_bytes_per_token_layer=max(a, 0.0),
                         overhead_frac=max(overhead, 0.0), recompute=recompute, measured=True,
                         source=f"{len(samples)} training-step points, worst fit residual "
                                f"{100 * rel:.1f} %")
    return prof, {"per_token_layer": a, "per_token": b, "constant": c, "worst_residual": rel,
                  "overhead_frac": overhead}


def _cuda_probe(device):
    import torch

    def reset():
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)

    def read():
        torch.cuda.synchronize(device)
        free, total = torch.cuda.mem_get_info(device)
        return {"peak_allocated": torch.cuda.max_memory_allocated(device),
                "peak_reserved": torch.cuda.max_memory_reserved(device),
                "device_used": total - free}
    return reset, read


def measure_point(layers: int, batch: int, seq: int, *, device, dim=2048, heads=16, experts=64,
                  d_expert=1024, d_shared=1024, groups=4, top_k=4, top_groups=2, vocab=32000,
                  backend="native", steps=3, probe=None, ce_chunk=0) -> Sample:
    """One (layers, tokens) point: build the decoder, run ``steps`` optimizer steps, read the peaks
    of the last one.  ``probe = (reset, read)`` replaces the CUDA counters (tests)."""
    import torch
    from ..models import ModelArgs, TerraceLM
    dev = torch.device(device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    args = ModelArgs(vocab=vocab, dim=dim, n_layers=layers, n_heads=heads, seq_len=seq,
                     n_experts=experts, n_groups=groups, top_k=top_k, top_groups=top_groups,
                     d_expert=d_expert, d_shared=d_shared, n_shared=1, dense_first=1,
                     expert_backend=backend, ce_chunk=ce_chunk)
    torch.manual_seed(0)
    model = TerraceLM(args).to(device=dev, dtype=dtype)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True if dev.type == "cuda" else None)
    reset, read = probe if probe is not None else _cuda_probe(dev)
    tok = torch.randint(0, vocab, (batch, seq + 1), device=dev)
    stats = None
    for i in range(steps):
        if i == steps - 1:
            reset()
        opt.zero_grad(set_to_none=True)
        loss, _ = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        if i == steps - 1:
            stats = read()
    n_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    state = sum(t.numel() * t.element_size() for st in opt.state.values() for t in st.values()
                if torch.is_tensor(t))
    # gradients are freed by zero_grad(set_to_none=True) and reallocated inside the step: they
    # belong to the step's peak and to ``static`` alike
    static = n_bytes * 2 + state
    del model, opt, loss
    if dev.type == "cuda":
        torch.cuda.empty_cache()
    return Sample(layers=layers, tokens=batch * seq, static_bytes=float(static),
                  peak_allocated=float(stats["peak_allocated"]),
                  peak_reserved=float(stats["peak_reserved"]),
                  device_used=float(stats["device_used"]))


def main(argv=None) -> int:
    import torch
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--layers", type=int, nargs="+", default=[4, 8])
    ap.add_argument("--batch", type=int, nargs="+", default=[1, 2])
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--d-expert", type=int, default=1024)
    ap.add_argument("--backend", default="native", choices=["native", "grouped", "loop"])
    ap.add_argument("--capacity-gb", type=float, default=180.0)
    ns = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print(json.dumps({"unavailable": "needs a CUDA device; fit_profile() runs anywhere"}))
        return 0
    dev = torch.device("cuda", torch.cuda.current_device())
    samples = [measure_point(L, b, ns.seq, device=dev, dim=ns.dim, experts=ns.experts,
                             d_expert=ns.d_expert, backend=ns.backend)
               for L in ns.layers for b in ns.batch]
    prof, details = fit_profile(samples, ns.capacity_gb * 1e9)
    print(json.dumps({"profile": asdict(prof), "fit": details,
                      "samples": [asdict(s) for s in samples]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
