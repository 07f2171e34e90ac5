"""Fused model-side kernels against fp32 PyTorch formulations of the same ops."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _close(a, b, tol):
    a, b = a.float(), b.float()
    err = (a - b).norm() / b.norm().clamp_min(1e-12)
    assert err.item() < tol, err.item()


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 6e-3), (torch.float32, 2e-6)])
@pytest.mark.parametrize("shape", [(4, 96, 1024), (3, 1001)])
@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_swiglu_forward_backward(dtype, tol, shape, act):
    from dmuon_b200.ops import model_ops

    fused = model_ops.swiglu if act == "silu" else model_ops.geglu
    plain = model_ops.swiglu_reference if act == "silu" else model_ops.geglu_reference

    torch.manual_seed(0)
    g = torch.randn(shape, device=_dev()).mul_(2).to(dtype).requires_grad_()
    u = torch.randn(shape, device=_dev()).to(dtype).requires_grad_()
    d = torch.randn(shape, device=_dev()).to(dtype)
    out = fused(g, u)
    out.backward(d)
    gf, uf = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    ref = plain(gf, uf)
    ref.backward(d.float())
    _close(out, ref, tol)
    _close(g.grad, gf.grad, tol)
    _close(u.grad, uf.grad, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 6e-3), (torch.float32, 2e-6)])
def test_rope_in_place_matches_reference_and_its_gradient(dtype, tol):
    from dmuon_b200.models.llama import rope_tables
    from dmuon_b200.ops import model_ops

    torch.manual_seed(1)
    b, s, hq, hk, d = 2, 96, 4, 2, 64
    cos, sin = rope_tables(s, d, 10000.0, _dev())
    x = torch.randn(b, s, 32, device=_dev(), dtype=dtype, requires_grad=True)
    wq = torch.randn(hq * d, 32, device=_dev(), dtype=dtype, requires_grad=True)
    wk = torch.randn(hk * d, 32, device=_dev(), dtype=dtype, requires_grad=True)

    def run(fused):
        q, k = F.linear(x, wq), F.linear(x, wk)
        q0, k0 = q.detach().clone(), k.detach().clone()
        if fused:
            q, k = model_ops.rope_qk_(q, k, cos, sin, d)
        else:
            q = model_ops.rope_reference(q.float().view(b, s, hq, d), cos, sin).view(b, s, -1)
            k = model_ops.rope_reference(k.float().view(b, s, hk, d), cos, sin).view(b, s, -1)
        wgt_q = torch.linspace(-1, 1, hq * d, device=_dev())
        wgt_k = torch.linspace(1, -1, hk * d, device=_dev())
        loss = (q.float() * wgt_q).sum() + (k.float() * wgt_k).pow(2).sum()
        grads = torch.autograd.grad(loss, (x, wq, wk))
        return q.detach(), k.detach(), grads, q0, k0

    from dmuon_b200.ops.multi_tensor import launch_count

    before = launch_count()
    qf, kf, gf, q0, k0 = run(True)
    assert launch_count() - before == 2          # one launch forward, one backward: the kernel ran, not the fallback
    qr, kr, gr, _, _ = run(False)
    _close(qf, qr, tol)
    _close(kf, kr, tol)
    for a, r in zip(gf, gr):
        _close(a, r, 4 * tol)
    # a rotation: norms of every head vector are preserved
    _close(qf.float().view(b, s, hq, d).norm(dim=-1), q0.float().view(b, s, hq, d).norm(dim=-1), tol)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 8e-3), (torch.float32, 1e-5)])
@pytest.mark.parametrize("rows,vocab", [(37, 1000), (5, 128256), (16, 4099)])
def test_softmax_xent_in_place(dtype, tol, rows, vocab):
    from dmuon_b200.ops import model_ops

    torch.manual_seed(2)
    logits = torch.randn(rows, vocab, device=_dev()).mul_(3).to(dtype)
    labels = torch.randint(0, vocab, (rows,), device=_dev())
    labels[1] = -1                                   # ignored row
    ref_in = logits.detach().float().requires_grad_()
    ref_rows = F.cross_entropy(ref_in, labels, ignore_index=-1, reduction="none")
    ref_rows.sum().backward()
    work = logits.clone()
    row_loss = model_ops.softmax_xent_(work, labels, 1.0)
    assert torch.allclose(row_loss, ref_rows, rtol=1e-4, atol=1e-4)
    assert row_loss[1].item() == 0.0 and work[1].float().abs().max().item() == 0.0
    _close(work, ref_in.grad, tol)


def test_linear_cross_entropy_matches_autograd():
    from dmuon_b200.ops import model_ops

    torch.manual_seed(3)
    rows, dm, vocab = 300, 64, 777
    h = torch.randn(rows, dm, device=_dev()).to(torch.bfloat16).requires_grad_()
    w = torch.randn(vocab, dm, device=_dev()).mul_(0.2).to(torch.bfloat16).requires_grad_()
    y = torch.randint(0, vocab, (rows,), device=_dev())
    y[::7] = -100
    loss = model_ops.linear_cross_entropy(h, w, y, chunk=128)
    (loss * 2.0).backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = F.cross_entropy(F.linear(hf, wf), y, ignore_index=-100)
    (ref * 2.0).backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * abs(ref.item())
    _close(h.grad, hf.grad, 2e-2)
    _close(w.grad, wf.grad, 2e-2)


def test_llama_fused_ops_match_plain_formulation():
    from dmuon_b200.models import llama

    cfg = llama.LlamaConfig.tiny(loss_chunk=64)
    torch.manual_seed(4)
    model = llama.LlamaModel(cfg).to(_dev(), torch.bfloat16)
    ids = torch.randint(0, cfg.vocab_size, (2, 129), device=_dev())
    from dmuon_b200.ops.multi_tensor import launch_count

    res = {}
    for fused in (True, False):
        llama.FUSED_OPS = fused
        try:
            model.zero_grad()
            before = launch_count()
            loss = model(ids[:, :-1], ids[:, 1:])
            loss.backward()
            # per layer: rotary + SwiGLU, forward and backward; plus one cross-entropy launch per chunk
            assert launch_count() - before == (4 * cfg.n_layers + 4 if fused else 0)
            res[fused] = (loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters()})
        finally:
            llama.FUSED_OPS = True
    assert abs(res[True][0] - res[False][0]) < 2e-2
    for n, g in res[False][1].items():
        _close(res[True][1][n], g, 5e-2)
