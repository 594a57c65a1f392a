"""tcgen05 attention kernels against a plain fp32 PyTorch reference (forward and all gradients)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(q, k, v, causal):
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    s = (qf @ kf.transpose(-1, -2)) * q.shape[-1] ** -0.5
    if causal:
        S = q.shape[-2]
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=q.device), 1), float("-inf"))
    o = torch.softmax(s, dim=-1) @ vf
    return o, (qf, kf, vf), torch.logsumexp(s, dim=-1)


def _close(a, b, tol=2e-2):
    scale = b.abs().max().item() + 1e-6
    torch.testing.assert_close(a.float(), b.float(), rtol=tol, atol=tol * scale)


@pytest.mark.parametrize("B,H,S,D", [(2, 3, 256, 64), (1, 2, 384, 128), (1, 1, 128, 128),
                                     (2, 2, 1024, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_fwd_bwd(native_ops, B, H, S, D, causal):
    torch.manual_seed(0)
    q, k, v = (torch.randn(B, H, S, D, device=DEV).bfloat16().requires_grad_(True) for _ in range(3))
    o = native_ops.attention(q, k, v, causal=causal)
    go = torch.randn_like(o)
    o.backward(go)
    ro, (qf, kf, vf), rlse = _ref(q, k, v, causal)
    ro.backward(go.float())
    assert native_ops.take_status() == 0
    _close(o, ro)
    _close(q.grad, qf.grad)
    _close(k.grad, kf.grad)
    _close(v.grad, vf.grad)
    _, lse = torch.ops.terrace.attn_fwd(q.detach(), k.detach(), v.detach(), causal, D ** -0.5)
    torch.testing.assert_close(lse, rlse, rtol=1e-2, atol=1e-2)


def test_attention_is_deterministic(native_ops):
    torch.manual_seed(1)
    q, k, v = (torch.randn(1, 4, 512, 128, device=DEV).bfloat16().requires_grad_(True) for _ in range(3))
    outs = []
    for _ in range(2):
        for t in (q, k, v):
            t.grad = None
        o = native_ops.attention(q, k, v)
        o.backward(torch.ones_like(o))
        outs.append([o.detach().clone()] + [t.grad.clone() for t in (q, k, v)])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_decoder_attention_uses_native_kernel(native_ops):
    from terracemoe_simulator_b200.models import ModelArgs, TerraceLM
    from terracemoe_simulator_b200.ops import native
    torch.manual_seed(0)
    a = ModelArgs(vocab=128, dim=256, n_layers=2, n_heads=4, seq_len=128, n_experts=8, n_groups=4,
                  top_k=2, top_groups=2, d_expert=64, d_shared=64, expert_backend="native")
    model = TerraceLM(a).to(DEV, torch.bfloat16)
    tok = torch.randint(0, 128, (2, 129), device=DEV)
    before = native.LIVE["attention"]
    loss, _ = model(tok[:, :-1], tok[:, 1:])
    loss.backward()
    assert native.LIVE["attention"] == before + 2 and torch.isfinite(loss)
    assert native_ops.take_status() == 0


@pytest.mark.parametrize("S", [77, 200, 129])
def test_causal_attention_of_any_length(native_ops, S):
    """Lengths that are not a multiple of 128 are padded behind the causal mask: exact result."""
    torch.manual_seed(2)
    q, k, v = (torch.randn(2, 2, S, 64, device=DEV).bfloat16().requires_grad_(True) for _ in range(3))
    o = native_ops.attention(q, k, v, causal=True)
    assert o.shape == q.shape
    go = torch.randn_like(o)
    o.backward(go)
    ro, (qf, kf, vf), _ = _ref(q, k, v, True)
    ro.backward(go.float())
    _close(o, ro)
    _close(q.grad, qf.grad)
    _close(k.grad, kf.grad)
    _close(v.grad, vf.grad)
    with pytest.raises(ValueError):
        native_ops.attention(q, k, v, causal=False)
    assert native_ops.take_status() == 0
