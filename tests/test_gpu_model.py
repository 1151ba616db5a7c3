"""End-to-end checks of the CUDA path against the CPU fp32 oracle path (same package, PyTorch ops)."""
import pytest
import torch

from util import assert_close

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda", 0)


def test_xent_kernel_and_linear_ce():
    from context_parallelism_b200.ops import xent
    torch.manual_seed(0)
    N, d, V, Vp = 700, 256, 1000, 1024
    x = (torch.randn(N, d, device=dev()) * 0.5).bfloat16().requires_grad_()
    w = torch.zeros(Vp, d, device=dev())
    w[:V] = torch.randn(V, d, device=dev()) * 0.1
    w = w.bfloat16().requires_grad_()
    tg = torch.randint(0, V, (N,), device=dev())
    tg[5] = -100
    scale = 1.0 / N
    loss = xent.linear_cross_entropy(x, w, tg, scale, V)
    loss.backward(torch.tensor(scale, device=dev()))
    X, W = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    want = xent.linear_cross_entropy(X.cpu(), W.cpu(), tg.cpu(), scale, V)
    X2, W2 = x.detach().float().cpu().requires_grad_(), w.detach().float().cpu().requires_grad_()
    want = xent.linear_cross_entropy(X2, W2, tg.cpu(), scale, V)
    want.backward(torch.tensor(scale))
    assert abs(float(loss) - float(want)) / float(want) < 2e-3
    assert_close(x.grad.float().cpu(), X2.grad, cos=0.999, name="dx")
    assert_close(w.grad.float().cpu(), W2.grad, cos=0.999, name="dw")
    nll = xent.per_token_nll(x.detach(), w.detach(), tg.clamp(min=0), V)
    wn = xent.per_token_nll(X2.detach(), W2.detach(), tg.clamp(min=0).cpu(), V)
    assert_close(nll.cpu(), wn, cos=0.9999, name="nll")


def test_adamw_matches_torch():
    from context_parallelism_b200.ops.optim import AdamW, FlatParams
    torch.manual_seed(1)
    ps = [torch.nn.Parameter(torch.randn(64, 32, device=dev())), torch.nn.Parameter(torch.randn(48, device=dev()))]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    flat = FlatParams([("a", ps[0]), ("b", ps[1])], bf16_matrices=True)
    opt = AdamW(flat, 1e-2, (0.9, 0.95), 1e-8, 0.1)
    topt = torch.optim.AdamW([{"params": [ref[0]], "weight_decay": 0.1}, {"params": [ref[1]], "weight_decay": 0.0}],
                             lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for _ in range(5):
        gs = [torch.randn_like(r) for r in ref]
        for p, r, g in zip(ps, ref, gs):
            p.main_grad.copy_(g)
            r.grad = g.clone()
        torch.nn.utils.clip_grad_norm_(ref, 1.0)
        topt.step()
        norm = opt.step(1e-2, 1.0)
    m = flat.named_master()
    assert_close(m["a"], ref[0].detach(), cos=0.999999, rel=1e-4, name="matrix")
    assert_close(m["b"], ref[1].detach(), cos=0.999999, rel=1e-4, name="vector")
    assert ps[0].dtype == torch.bfloat16
    assert_close(ps[0].float(), ref[0].detach(), cos=0.9999, name="bf16 copy")


@pytest.mark.parametrize("family", ["llama", "gpt2"])
@pytest.mark.parametrize("recompute", ["none", "selective"])
def test_model_step_matches_cpu_oracle(family, recompute):
    """Same weights, same batch: loss and a few updated weights of the bf16 CUDA path follow the fp32 CPU path."""
    from context_parallelism_b200.config import Config
    from context_parallelism_b200.engine import TrainEngine
    kw = dict(n_embd=256, n_layer=2, n_head=4, head_dim=64, vocab_size=1000, T=384, B=2, max_steps=20, warmup_steps=1,
              checkpointing=False, recompute=recompute)
    if family == "llama":
        kw.update(n_kv_head=2, ffn_hidden=512)
    else:
        kw.update(n_kv_head=4, ffn_hidden=1024, weight_tying=True)
    cfg = Config.from_env(family, 1, env={}).replace(**kw)
    gpu = TrainEngine(cfg.replace(dtype="bf16"), dev())
    cpu = TrainEngine(cfg.replace(dtype="fp32"), torch.device("cpu"))
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab_size, (cfg.B, cfg.T + 1), generator=g)
    lg, lc = [], []
    for s in range(4):
        lg.append(float(gpu.train_step(tok[:, :-1].to(dev()), tok[:, 1:].to(dev()))))
        lc.append(float(cpu.train_step(tok[:, :-1], tok[:, 1:])))
    gpu.check_kernels()
    for a, b in zip(lg, lc):
        assert abs(a - b) / b < 2e-2, (lg, lc)
    assert lg[-1] < lg[0]
    ng, nc = float(gpu.last_grad_norm), float(cpu.last_grad_norm)
    assert abs(ng - nc) / nc < 0.1, (ng, nc)


def test_recompute_grads_identical():
    """Activation recomputation must not change any gradient nor leave gradients outside the flat buffer."""
    from context_parallelism_b200.config import Config
    from context_parallelism_b200.engine import TrainEngine
    kw = dict(n_embd=256, n_layer=2, n_head=4, head_dim=64, vocab_size=1000, T=384, B=2, max_steps=20, warmup_steps=1,
              checkpointing=False, n_kv_head=2, ffn_hidden=512)
    tok = torch.randint(0, 1000, (2, 385), generator=torch.Generator().manual_seed(3)).to(dev())
    grads = {}
    for rc in ("none", "selective"):
        eng = TrainEngine(Config.from_env("llama", 1, env={}).replace(**kw, recompute=rc), dev())
        eng.forward_backward(tok[:, :-1], tok[:, 1:])
        assert all(p.grad is None for p in eng.model.parameters())
        grads[rc] = eng.flat.grad.clone()
    assert float(grads["none"].norm()) > 0
    assert_close(grads["selective"], grads["none"], cos=0.99999, name="flat grads")
