"""End to end on a small Llama-shaped module: build_param_groups(model, preset) -> Adafactor8Bit -> a few training
steps on the GPU for every preset (the call sequence of the reference's README).  No oracle here: the test checks
that every route runs on the CUDA path, that the loss goes down and that the states are the ones the route asks for."""
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


class Block(nn.Module):
    def __init__(self, h, kv, mlp):
        super().__init__()
        self.input_layernorm = nn.LayerNorm(h)
        self.self_attn = nn.Module()
        self.self_attn.q_proj = nn.Linear(h, h, bias=False)
        self.self_attn.k_proj = nn.Linear(h, kv, bias=False)
        self.self_attn.v_proj = nn.Linear(h, kv, bias=False)
        self.self_attn.o_proj = nn.Linear(h, h, bias=False)
        self.mlp = nn.Module()
        self.mlp.gate_proj = nn.Linear(h, mlp, bias=False)
        self.mlp.up_proj = nn.Linear(h, mlp, bias=False)
        self.mlp.down_proj = nn.Linear(mlp, h, bias=False)
        self.kv = kv

    def forward(self, x):
        y = self.input_layernorm(x)
        a = self.self_attn
        q, k, v = a.q_proj(y), a.k_proj(y), a.v_proj(y)
        rep = q.shape[-1] // self.kv
        att = torch.softmax(q @ k.repeat(1, 1, rep).transpose(1, 2) / q.shape[-1] ** 0.5, dim=-1)
        x = x + a.o_proj(att @ v.repeat(1, 1, rep))
        m = self.mlp
        return x + m.down_proj(torch.nn.functional.silu(m.gate_proj(x)) * m.up_proj(x))


class Tiny(nn.Module):
    def __init__(self, vocab=512, h=128, kv=64, mlp=256, layers=2):
        super().__init__()
        self.model = nn.Module()
        self.model.embed_tokens = nn.Embedding(vocab, h)
        self.model.layers = nn.ModuleList([Block(h, kv, mlp) for _ in range(layers)])
        self.model.norm = nn.LayerNorm(h)
        self.lm_head = nn.Linear(h, vocab, bias=False)

    def forward(self, ids):
        x = self.model.embed_tokens(ids)
        for blk in self.model.layers:
            x = blk(x)
        return self.lm_head(self.model.norm(x))


@pytest.mark.parametrize("preset,extra", [
    ("adamw", {}), ("rmsprop", {}), ("sgd", dict(lr=5e-2)), ("adafactor", {}), ("came", {}),
    ("apollo", dict(apollo_rank=16)), ("adamw", dict(grouping="G0", m_quant_type="uf4", v_quant_type="al16")),
    ("adamw", dict(bf16=True, stochastic_round_writeback=True)), ("apollo", dict(bf16=True, apollo_rank=16, stochastic_round_writeback=True)),
    ("came", dict(bf16=True)), ("adamw", dict(enable_fira_for_adafactor=True, lag_norm=True)),
    ("adamw", dict(f16=True, stochastic_round_writeback=True)), ("adafactor", dict(f16=True)), ("came", dict(f16=True)),
])
def test_preset_trains_on_gpu(preset, extra):
    from adafactor8bit import Adafactor8Bit, build_param_groups
    torch.manual_seed(0)
    model = Tiny().cuda()
    extra = dict(extra)
    if extra.pop("bf16", False):
        model = model.bfloat16()
    if extra.pop("f16", False):
        model = model.half()
    kw = {k: extra.pop(k) for k in list(extra) if k in ("grouping", "apollo_rank")}
    lr = extra.pop("lr", 2e-3)
    groups = build_param_groups(model, preset, **kw)
    opt = Adafactor8Bit(groups, lr=lr, min_8bit_size=1024, **extra)       # state formats are constructor options
    ids = torch.randint(0, 512, (8, 32), device="cuda")
    losses = []
    for _ in range(6):
        logits = model(ids)
        loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 512), ids[:, 1:].reshape(-1))
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert all(torch.isfinite(p).all() for p in model.parameters())
    assert losses[-1] < losses[0], (preset, losses)
    states = [opt.state[p] for p in model.parameters()]
    assert all(st["step"] == 6 for st in states)
    if preset == "apollo":
        assert any("apollo_seed" in st for st in states) and any("variance_q" in st or "variance" in st for st in states)
    if preset in ("adafactor", "came"):
        assert any("row_var_q" in st or "row_var" in st for st in states)
    if preset == "came":
        assert any("conf_row_q" in st or "conf_row" in st for st in states)


def test_lr_scheduler_and_tensor_lr():
    """The learning rate is read from the group at every step: a torch scheduler, a manual edit and a 0-d tensor
    give the same run."""
    from adafactor8bit import Adafactor8Bit
    torch.manual_seed(1)
    w0 = torch.randn(96, 160, device="cuda") * 0.02
    grads = [torch.randn(96, 160, device="cuda") * 1e-3 for _ in range(4)]
    hp = dict(beta1=0.9, beta2=0.999, beta2_decay=None, factored=False, relative_step=False, scale_parameter=False,
              scale_weight_decay=False, d=0.0, eps=(1e-8, 1e-3), weight_decay=0.01, min_8bit_size=1)
    outs = []
    for mode in ("scheduler", "manual", "tensor"):
        p = torch.nn.Parameter(w0.clone())
        opt = Adafactor8Bit([p], lr=1e-3, **hp)
        sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda e: 0.5 ** e) if mode == "scheduler" else None
        for t, g in enumerate(grads):
            if mode == "manual":
                opt.param_groups[0]["lr"] = 1e-3 * 0.5 ** t
            if mode == "tensor":
                opt.param_groups[0]["lr"] = torch.tensor(1e-3 * 0.5 ** t, device="cuda", dtype=torch.float64)
            p.grad = g.clone()
            opt.step()
            if sched is not None:
                sched.step()
        outs.append(p.detach().clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("hp", [dict(beta1=0.9, beta2=0.999, beta2_decay=None, factored=False, relative_step=False,
                                     scale_parameter=False, d=0.0, eps=(1e-8, 1e-3), lr=1e-3),
                                dict()], ids=["adamw", "adafactor"])
def test_non_contiguous_parameter(hp):
    """A transposed (non-contiguous) parameter is stepped like its contiguous twin."""
    from adafactor8bit import Adafactor8Bit
    torch.manual_seed(2)
    base = torch.randn(160, 96, device="cuda") * 0.02
    a = torch.nn.Parameter(base.t())                      # shape (96, 160), strides (1, 96)
    b = torch.nn.Parameter(base.t().contiguous())
    assert not a.is_contiguous() and b.is_contiguous()
    oa, ob = Adafactor8Bit([a], min_8bit_size=1, **hp), Adafactor8Bit([b], min_8bit_size=1, **hp)
    for t in range(3):
        g = torch.randn(160, 96, device="cuda") * 1e-3
        a.grad, b.grad = g.t(), g.t().contiguous()
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    assert not a.is_contiguous() and torch.equal(a.detach(), b.detach())
