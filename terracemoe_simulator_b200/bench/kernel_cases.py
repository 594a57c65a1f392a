"""Small single-kernel workloads for profiling (``ncu``) and for quick roofline numbers.

    python -m terracemoe_simulator_b200.bench.kernel_cases <case> [--iters N] [--full]

Every case allocates a few hundred MB at most (inputs larger than the 126 MB L2, so DRAM
figures are meaningful), launches its kernel ``--iters`` times after one warm-up and prints the
CUDA-event time with the achieved fraction of the measured peaks (``MEASURED_PEAKS.json`` at
the repository root when present).  ``--full`` switches to the shapes of the single-MoE-layer
benchmark (24576 rows, d_model 4096, 64 experts of hidden 1408).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

CASES = ("gemm_fwd", "gemm_swiglu", "gemm_dgrad", "gemm_wgrad", "gemm_scatter", "rmsnorm",
         "rmsnorm_bwd", "route", "route_fused", "scatter", "combine", "combine_bwd", "swiglu_bwd",
         "attn_fwd", "attn_bwd", "ep_layer",
         "k1_arrival", "k2_pack", "rope_split", "rope_merge", "route_bwd", "passthrough",
         "gemm_swiglu_bwd")


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "of measured"
    except (OSError, KeyError):
        return 6650.0, 1590.0, "of fallback"


def _time(fn, iters):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=CASES)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--full", action="store_true")
    ap.add_argument("--library", action="store_true",
                    help="attention cases: time torch's scaled_dot_product_attention instead")
    ap.add_argument("--pad", type=int, default=0,
                    help="declare the groups padded to this multiple (64 lets the weight-gradient "
                         "GEMM use CTA pairs)")
    args = ap.parse_args(argv)
    from terracemoe_simulator_b200 import ops
    if not ops.custom_ops_enabled():
        raise SystemExit("native library not loaded")
    lib = torch.ops.terrace
    dev = "cuda"
    torch.manual_seed(0)
    if args.full:
        E, rows, H, d, T, k = 64, 24576, 4096, 1408, 4096, 6
    else:
        E, rows, H, d, T, k = 8, 8192, 4096, 1408, 2048, 4
    cnt = torch.full((E,), rows // E, dtype=torch.int32, device=dev)
    st = torch.cumsum(cnt, 0, dtype=torch.int32) - cnt
    bf = torch.bfloat16
    hbm, tf, tag = _peaks()
    flops = bytes_ = 0
    extra = {}
    if args.case in ("gemm_fwd", "gemm_swiglu"):
        X = torch.randn(rows, H, device=dev, dtype=bf)
        W = torch.randn(E, H, 2 * d, device=dev, dtype=bf) * H ** -0.5
        epi = 1 if args.case == "gemm_swiglu" else 0
        fn = lambda: lib.grouped_gemm(X, W, st, cnt, 0, epi, epi == 1, 0, args.pad)
        flops = 2 * rows * H * 2 * d
    elif args.case == "gemm_dgrad":
        dY = torch.randn(rows, 2 * d, device=dev, dtype=bf)
        W = torch.randn(E, H, 2 * d, device=dev, dtype=bf) * H ** -0.5
        fn = lambda: lib.grouped_gemm(dY, W, st, cnt, 1, 0, False, 0, args.pad)
        flops = 2 * rows * H * 2 * d
    elif args.case == "gemm_swiglu_bwd":
        # d(act) = dOut @ W2^T with the SwiGLU backward in the epilogue (d[gate | up] written
        # directly), against the two launches it replaces (plain dgrad GEMM + swiglu_bwd)
        dout = torch.randn(rows, H, device=dev, dtype=bf)
        W2 = torch.randn(E, d, H, device=dev, dtype=bf) * d ** -0.5
        h13 = torch.randn(rows, 2 * d, device=dev, dtype=bf)
        dh13 = torch.empty_like(h13)
        fn = lambda: lib.grouped_gemm_ex(dout, W2, dh13, h13, st, cnt, 1, 3, None, 0, 0, 0, 0,
                                         args.pad)

        def unfused():
            dact, _ = lib.grouped_gemm(dout, W2, st, cnt, 1, 0, False, 0, args.pad)
            return lib.swiglu_bwd(h13, dact[:rows])
        extra["unfused_ms"] = round(_time(unfused, args.iters), 4)
        flops = 2 * rows * H * d
    elif args.case == "gemm_scatter":
        # the scattering epilogue on one GPU: rows leave through a random permutation into a local
        # buffer; checked once against the plain kernel followed by the same permutation
        A = torch.randn(rows, d, device=dev, dtype=bf)
        W = torch.randn(E, d, H, device=dev, dtype=bf) * d ** -0.5
        perm = torch.randperm(rows, device=dev)
        row_map = perm.to(torch.int32)                       # source 0, slot perm[r]
        ret = torch.zeros(rows, H, device=dev, dtype=bf)
        base = torch.tensor([ret.data_ptr()], dtype=torch.int64, device=dev)
        fn = lambda: lib.grouped_gemm_scatter(A, W, st, cnt, 0, row_map, base, rows)
        fn()
        plain = lib.grouped_gemm(A, W, st, cnt, 0, 0, False, 0, args.pad)
        plain = plain[0] if isinstance(plain, (tuple, list)) else plain
        want = torch.zeros_like(ret)
        want[perm] = plain[:rows]
        torch.cuda.synchronize()
        if not torch.equal(ret, want):
            raise SystemExit("gemm_scatter: rows differ from the plain kernel's, max |diff| %g"
                             % (ret.float() - want.float()).abs().max().item())
        flops = 2 * rows * d * H
    elif args.case == "gemm_wgrad":
        X = torch.randn(rows, H, device=dev, dtype=bf)
        dY = torch.randn(rows, 2 * d, device=dev, dtype=bf)
        fn = lambda: lib.grouped_wgrad(X, dY, st, cnt, 0, args.pad)
        flops = 2 * rows * H * 2 * d
    elif args.case in ("attn_fwd", "attn_bwd"):
        # small: 2 x 16 heads x 2048 x 128; --full: the decoder benchmark's 8 x 16 x 4096 x 128
        B_, H_, S_, D_ = (8, 16, 4096, 128) if args.full else (2, 16, 2048, 128)
        q, k_, v = (torch.randn(B_, H_, S_, D_, device=dev, dtype=bf) for _ in range(3))
        causal_flops = 4 * B_ * H_ * S_ * S_ * D_ / 2
        if args.case == "attn_fwd":
            fn = lambda: lib.attn_fwd(q, k_, v, True, D_ ** -0.5)
            flops = causal_flops
        else:
            o, lse = lib.attn_fwd(q, k_, v, True, D_ ** -0.5)
            go = torch.randn_like(o)
            fn = lambda: lib.attn_bwd(q, k_, v, o, go, lse, True, D_ ** -0.5)
            flops = 2.5 * causal_flops
        if args.library:
            import torch.nn.functional as F
            if args.case == "attn_fwd":
                fn = lambda: F.scaled_dot_product_attention(q, k_, v, is_causal=True)
            else:
                qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k_, v))
                oo = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True)
                fn = lambda: torch.autograd.grad(oo, (qq, kk, vv), go, retain_graph=True)
    elif args.case in ("rmsnorm", "rmsnorm_bwd"):
        x = torch.randn(rows * 2, H, device=dev, dtype=bf)
        w = torch.ones(H, device=dev, dtype=bf)
        if args.case == "rmsnorm":
            fn = lambda: lib.rmsnorm_fwd(x, w, 1e-5)
            bytes_ = 2 * x.numel() * 2
        else:
            _, rstd = lib.rmsnorm_fwd(x, w, 1e-5)
            dy = torch.randn_like(x)
            fn = lambda: lib.rmsnorm_bwd(x, w, dy, rstd)
            bytes_ = 3 * x.numel() * 2
    elif args.case == "route_fused":
        # the router GEMM with the selection in its epilogue: x is read once, nothing else moves
        Tr = T * 8
        x = torch.randn(Tr, H, device=dev, dtype=bf)
        w = torch.randn(64, H, device=dev, dtype=bf) * H ** -0.5
        bias = torch.zeros(64, device=dev)
        fn = lambda: lib.route_fused(x, w, bias, 4, 6, 2, 2)
        bytes_ = x.numel() * 2 + w.numel() * 2
    elif args.case == "ep_layer":
        # the fused expert-parallel layer at world 1: every peer-memory kernel of the one-hop path
        # (plan, push, arrival-gated GEMMs, scattering epilogue, signal, combine) on one GPU
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29911")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        from terracemoe_simulator_b200.parallel import fused as fz
        from terracemoe_simulator_b200.routing import TRouteConfig, t_route
        Ee = 64 if args.full else 16
        cfg = TRouteConfig(Ee, 4, k if args.full else 4, 2)
        ctx = fz.FusedEPContext(cfg, H, d, T, world=1, rank=0, rpn=1, device=torch.device(dev, 0),
                                overlap=not args.library)
        x = torch.randn(T, H, device=dev, dtype=bf).requires_grad_(True)
        w13 = (torch.randn(Ee, H, 2 * d, device=dev, dtype=bf) * H ** -0.5).requires_grad_(True)
        w2 = (torch.randn(Ee, d, H, device=dev, dtype=bf) * d ** -0.5).requires_grad_(True)
        idx, gates, _ = t_route(torch.rand(T, Ee, device=dev), torch.zeros(Ee, device=dev), cfg)
        gy = torch.randn(T, H, device=dev, dtype=bf)

        def fn():
            y = fz.fused_moe_forward(ctx, x, idx, gates, w13, w2, mode="one_hop")
            y.backward(gy)
        flops = 3 * 2 * 3 * T * cfg.top_k * H * d
    elif args.case == "passthrough":
        x = torch.randn(rows, H, device=dev, dtype=bf)
        fn = lambda: lib.passthrough(x)
        bytes_ = 2 * x.numel() * 2
    elif args.case in ("rope_split", "rope_merge"):
        # [B, S, 3 * heads * 128] projection output <-> three [B, heads, S, 128] tensors
        B_, S_, nh, hd = (8, 4096, 16, 128) if args.full else (2, 4096, 16, 128)
        qkv = torch.randn(B_, S_, 3 * nh * hd, device=dev, dtype=bf)
        ang = torch.outer(torch.arange(S_, device=dev, dtype=torch.float32),
                          10000.0 ** (-torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd))
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        if args.case == "rope_split":
            fn = lambda: lib.rope_split(qkv, cos, sin, nh)
        else:
            q_, k__, v_ = lib.rope_split(qkv, cos, sin, nh)
            fn = lambda: lib.rope_merge(q_, k__, v_, cos, sin)
        bytes_ = 2 * qkv.numel() * 2
    elif args.case == "route_bwd":
        Tr = T * 8
        logits = torch.randn(Tr, 64, device=dev)
        idx_, gates_, _, _, aff = lib.route_select(logits, torch.zeros(64, device=dev), 4, 6, 2, 2)
        dg = torch.randn_like(gates_)
        fn = lambda: lib.route_select_bwd(dg, gates_, aff, idx_, 64)
        bytes_ = Tr * 64 * 4 + 4 * Tr * 6 * 4
    elif args.case == "k2_pack":
        # the contract op of the send side: 8 ranks in groups of 2, 64 experts, k = 6, M = 2
        world_, rpn_, M_, q_ = 8, 2, 2, 3
        per = 64 // (world_ // rpn_)
        g = torch.Generator().manual_seed(3)
        grp = torch.stack([torch.randperm(world_ // rpn_, generator=g)[:M_] for _ in range(T)])
        pick = torch.stack([torch.cat([gr * per + torch.randperm(per, generator=g)[:q_]
                                       for gr in row]) for row in grp]).to(dev)
        x = torch.randn(T, H, device=dev, dtype=bf)
        gates_ = torch.rand(T, M_ * q_, device=dev, dtype=bf)
        fn = lambda: lib.k2_pack(x, pick, gates_, world_, 64, rpn_, M_)
        bytes_ = (T + T * M_) * H * 2
    elif args.case == "k1_arrival":
        # the contract op of the arrival side: R rows, each feeding q of this group's 16 experts
        R_, q_, epr_, rpn_ = T * 2, 3, 8, 2
        g = torch.Generator().manual_seed(4)
        rslot = torch.stack([torch.randperm(epr_ * rpn_, generator=g)[:q_].sort().values
                             for _ in range(R_)]).to(dev)
        rx = torch.randn(R_, H, device=dev, dtype=bf)
        rgate = torch.rand(R_, q_, device=dev, dtype=bf)
        fn = lambda: lib.k1_arrival(rx, rslot, rgate, q_, epr_, rpn_, 0)
        bytes_ = (R_ + R_ * q_) * H * 2
    elif args.case == "route":
        logits = torch.randn(T * 8, 64, device=dev)
        bias = torch.zeros(64, device=dev)
        fn = lambda: lib.route_select(logits, bias, 4, 6, 2, 2)
        bytes_ = logits.numel() * 4
    elif args.case in ("scatter", "combine", "combine_bwd"):
        x = torch.randn(T, H, device=dev, dtype=bf)
        idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)])
        es, gs, cols, pos, s0, c0 = lib.moe_plan(idx, torch.rand(T, k, device=dev), E, 1)
        xs = lib.moe_scatter_rows(x, pos, T * k)
        if args.case == "scatter":
            fn = lambda: lib.moe_scatter_rows(x, pos, T * k)
            bytes_ = (T + T * k) * H * 2
        elif args.case == "combine":
            fn = lambda: lib.moe_combine(xs, pos, es, gs, E)
            bytes_ = (T + T * k) * H * 2
        else:
            fn = lambda: lib.moe_combine_bwd(x, xs, pos, gs, True)
            bytes_ = (T + 2 * T * k) * H * 2
    else:
        h13 = torch.randn(rows, 2 * d, device=dev, dtype=bf)
        dact = torch.randn(rows, d, device=dev, dtype=bf)
        fn = lambda: lib.swiglu_bwd(h13, dact)
        bytes_ = rows * d * 2 * 5
    ms = _time(fn, args.iters)
    line = {"case": args.case, "full": args.full, "pad": args.pad, "library": args.library,
            "pair_policy": os.environ.get("TERRACE_GEMM_PAIR", "auto"), "ms": round(ms, 4)}
    if flops:
        line["tflops"] = round(flops / ms / 1e9, 1)
        line["frac_of_bf16_peak"] = round(flops / ms / 1e9 / tf, 3)
    if bytes_:
        line["gbs"] = round(bytes_ / ms / 1e6, 1)
        line["frac_of_hbm_peak"] = round(bytes_ / ms / 1e6 / hbm, 3)
    line.update(extra)
    line["peaks"] = tag
    line["status"] = ops.take_status()
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
