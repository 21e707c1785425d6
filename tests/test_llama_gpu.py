"""Llama-shaped decoder (RMSNorm, RoPE, SwiGLU, grouped-query attention) on the GPU kernels vs a PyTorch fp32 oracle."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


class OracleLlamaBlock(torch.nn.Module):
    def __init__(self, d, h, hk, dh, dff):
        super().__init__()
        self.ln_attn = torch.nn.Module(); self.ln_attn.weight = torch.nn.Parameter(torch.ones(d))
        self.ln_ff = torch.nn.Module(); self.ln_ff.weight = torch.nn.Parameter(torch.ones(d))
        self.attn = torch.nn.Module()
        self.attn.project_qkv = torch.nn.Linear(d, (h + 2 * hk) * dh, bias=False)
        self.attn.project_out = torch.nn.Linear(h * dh, d, bias=False)
        self.ff = torch.nn.Module()
        self.ff.w_gate_up = torch.nn.Linear(d, 2 * dff, bias=False)
        self.ff.w_out = torch.nn.Linear(dff, d, bias=False)
        self.h, self.hk, self.dh, self.dff = h, hk, dh, dff

    @staticmethod
    def rms(x, w, eps=1e-5):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def forward(self, x):
        from bmtrain_b200.ops.elementwise import _rope_tables, _rope_apply

        b, s, _ = x.shape
        g = self.h // self.hk
        qkv = self.attn.project_qkv(self.rms(x, self.ln_attn.weight)).view(b, s, self.hk, g + 2, self.dh)
        q = qkv[:, :, :, :g].reshape(b, s, self.h, self.dh)
        k, v = qkv[:, :, :, g], qkv[:, :, :, g + 1]
        cos, sin = _rope_tables(s, self.dh, 10000.0, x.device)
        q, k = _rope_apply(q, cos, sin, False), _rope_apply(k, cos, sin, False)
        k = k.repeat_interleave(g, dim=2); v = v.repeat_interleave(g, dim=2)
        sc = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(self.dh)
        sc = sc.masked_fill(~torch.ones(s, s, dtype=torch.bool, device=x.device).tril(), float("-inf"))
        o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), v).reshape(b, s, self.h * self.dh)
        x = x + self.attn.project_out(o)
        gu = self.ff.w_gate_up(self.rms(x, self.ln_ff.weight))
        return x + self.ff.w_out(torch.nn.functional.silu(gu[..., :self.dff]) * gu[..., self.dff:])


def test_llama_block_matches_oracle(bmt_gpu):
    bmt = bmt_gpu
    torch.manual_seed(21)
    d, h, hk, dh, dff, b, s = 256, 8, 2, 32, 512, 2, 96
    ref = OracleLlamaBlock(d, h, hk, dh, dff)
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.05)
        ref.ln_attn.weight.add_(1.0); ref.ln_ff.weight.add_(1.0)
    blk = bmt.models.LlamaBlock(d, h, hk, dh, dff, dtype=torch.bfloat16)
    blk.load_state_dict(ref.state_dict())
    x = torch.randn(b, s, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = blk(x)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr = x.detach().float().cpu().requires_grad_()
    yr = ref(xr)
    yr.backward(gy.float().cpu())

    def rel(a, b_):
        return ((a.float().cpu() - b_).abs().max() / (b_.abs().max() + 1e-6)).item()

    assert rel(y, yr) < 4e-2 and rel(x.grad, xr.grad) < 5e-2
    mine = dict(blk.named_parameters())
    for name, p in ref.named_parameters():
        assert rel(mine[name].grad.view(p.shape), p.grad) < 5e-2, name


def test_llama_model_trains(bmt_gpu):
    """A small Llama-shaped model in ZeRO blocks: loss decreases over a few Adam steps on a fixed batch."""
    bmt = bmt_gpu
    torch.manual_seed(22)
    model = bmt.models.Llama(num_layers=2, vocab_size=512, dim_model=256, num_heads=8, num_kv_heads=4, dim_ff=512, dtype=torch.bfloat16)
    bmt.init_parameters(model)
    opt = bmt.optim.AdamOptimizer(model.parameters(), lr=2e-3)
    om = bmt.optim.OptimManager(loss_scale=None)
    om.add_optimizer(opt)
    loss_fn = bmt.loss.FusedCrossEntropy()
    ids = torch.randint(0, 512, (4, 65), device="cuda")
    losses = []
    for _ in range(8):
        logits = model(ids[:, :-1].contiguous())
        loss = loss_fn(logits.view(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
        om.zero_grad(); om.backward(loss); om.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.5, losses
