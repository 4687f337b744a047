"""Mixture-of-experts block on the GPU kernels against a plain fp32 PyTorch restatement (no kernel of this library on
the reference side): router softmax / top-k / renormalisation, per-expert SwiGLU MLP, weighted combine, auxiliary
load-balancing loss, and the gradients of all four parameter groups."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle(x, rw, gu, dn, k, norm, idx):
    """fp32 PyTorch on the bf16-rounded inputs. `idx` [T, k]: the experts the kernel path chose (a token whose k-th and
    (k+1)-th probabilities differ by less than the bf16 rounding of the logits may legitimately pick either); the
    caller checks separately that this choice agrees with the fp32 top-k for nearly all tokens."""
    T, H = x.shape
    E, I2, _ = gu.shape
    I = I2 // 2
    logits = x @ rw.t()
    probs = torch.softmax(logits, -1)
    top_idx = probs.topk(k, -1).indices
    w = probs.gather(-1, idx)
    if norm:
        w = w / w.sum(-1, keepdim=True)
    y = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = x[tok] @ gu[e].t()
        a = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
        y.index_add_(0, tok, (a @ dn[e].t()) * w[tok, slot][:, None])
    f = torch.zeros(E, device=x.device).scatter_add_(0, idx.reshape(-1), torch.ones(T * k, device=x.device)) / T
    aux = E * (f * probs.mean(0)).sum()
    return y, aux, top_idx


@pytest.mark.parametrize("grouped", [True, False])
@pytest.mark.parametrize("T,H,I,E,k,norm", [(300, 128, 128, 8, 2, True), (1000, 256, 192, 16, 4, True),
                                            (130, 128, 64, 4, 1, False)])
def test_moe_block_matches_fp32_pytorch(T, H, I, E, k, norm, grouped):
    from openrlhf_b200.models import moe
    from openrlhf_b200.ops import _lib

    torch.manual_seed(0)
    x = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    rw = (torch.randn(E, H, device="cuda") * 0.3).to(torch.bfloat16).requires_grad_()
    gu = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    dn = (torch.randn(E, H, I, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    if grouped:
        y, aux = moe.moe_forward_grouped(x, rw, gu, dn, k, norm)
    else:
        y, aux = moe.moe_forward(x, rw, gu, dn, k, norm, expert_range=(0, E))
    g = torch.randn(T, H, device="cuda")
    ((y.float() * g).sum() + 0.1 * aux).backward()
    _lib.check_status()

    with torch.no_grad():
        _, idx_k, _ = moe.router_topk(x.detach(), rw.detach(), k, norm)
    ref_in = [t.detach().float().requires_grad_() for t in (x, rw, gu, dn)]
    yr, auxr, idx_r = _oracle(*ref_in, k, norm, idx_k)
    ((yr * g).sum() + 0.1 * auxr).backward()
    same = (idx_k.sort(-1).values == idx_r.sort(-1).values).all(-1)
    assert same.float().mean().item() > 0.97
    rel = lambda a, b: ((a - b).norm() / b.norm().clamp_min(1e-6)).item()
    assert rel(y.float(), yr) < 2e-2
    assert abs(aux.item() - auxr.item()) < 2e-2 * abs(auxr.item()) + 1e-3
    for name, t, r in zip(("dx", "drouter", "dgate_up", "ddown"), (x, rw, gu, dn), ref_in):
        assert rel(t.grad.float(), r.grad) < 4e-2, (name, rel(t.grad.float(), r.grad))
