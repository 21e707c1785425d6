"""End-to-end training contract on one GPU (the intent of the reference's ``tests/test_training.py:386-510`` and
``tests/test_model_wrapper.py:174-216``): the same small GPT trained through different wrappers and optimizers ends in
the same place as a plain PyTorch fp32 run, and the asynchronous offloaded optimizer is bit-identical to its
synchronous form, skipped (overflow) steps included."""
import os

import pytest
import torch

from oracle import OracleGPT

pytestmark = pytest.mark.gpu

CFG = dict(num_layers=2, vocab_size=512, dim_model=128, dim_head=32, num_heads=4, dim_ff=256, max_distance=64)
B, S = 2, 64


def _batches(n, seed=5):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, CFG["vocab_size"], (B, S + 1), generator=gen) for _ in range(n)]


def _oracle():
    return OracleGPT(CFG["num_layers"], CFG["vocab_size"], CFG["dim_model"], CFG["dim_head"], CFG["num_heads"], CFG["dim_ff"],
                     CFG["max_distance"], bias=True)


def _train(bmt, model, optimizer, batches, loss_scale, dtype):
    om = bmt.optim.OptimManager(loss_scale=loss_scale, loss_scale_steps=4)
    om.add_optimizer(optimizer)
    loss_fn = bmt.loss.FusedCrossEntropy(ignore_index=-100)
    pos = torch.arange(S, device="cuda")[None].expand(B, -1).contiguous()
    mask = torch.ones(B, S, dtype=torch.bool, device="cuda")
    losses, scales = [], []
    for ids in batches:
        ids = ids.cuda()
        logits = model(ids[:, :-1].contiguous(), pos, mask)
        loss = loss_fn(logits.view(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
        om.zero_grad()
        om.backward(loss)
        om.step()
        losses.append(float(loss.detach()))
        scales.append(om.loss_scale)
    bmt.synchronize()
    return losses, scales


def _full_state(model):
    return {k: v.detach().float().cpu() for k, v in model.state_dict().items()}


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_async_offload_is_bit_identical_to_sync(bmt_gpu, dtype, monkeypatch):
    """Same model, same data: queued updates (with and without stepping ahead during backward) against the blocking
    loop.  The initial loss scale is far too high, so the first steps overflow and are skipped: a result that was
    computed ahead of such a step must leave no trace."""
    bmt = bmt_gpu
    batches = _batches(14)
    outcomes = []
    stats = []
    for mode in ("sync", "async", "async_no_ahead"):
        monkeypatch.setenv("BMT_OFFLOAD_ASYNC", "0" if mode == "sync" else "1")
        monkeypatch.setenv("BMT_OFFLOAD_AHEAD_GB", "0" if mode == "async_no_ahead" else "4")
        torch.manual_seed(3)
        model = bmt.models.GPT(**CFG, bias=True, dtype=dtype)
        bmt.init_parameters(model)
        if outcomes:
            model.load_state_dict(first_init)
        else:
            first_init = {k: v.clone() for k, v in model.state_dict().items()}
        opt = bmt.optim.AdamOffloadOptimizer(model.parameters(), lr=2e-3, weight_decay=1e-2)
        losses, scales = _train(bmt, model, opt, batches, loss_scale=2.0 ** 22 if dtype == torch.float16 else 1024.0, dtype=dtype)
        sd = opt.state_dict()
        outcomes.append((losses, scales, _full_state(model), sd))
        stats.append(dict(opt.stats))
    ref_losses, ref_scales, ref_params, ref_sd = outcomes[0]
    if dtype == torch.float16:
        assert ref_scales[0] < 2.0 ** 22, "the test is meant to see skipped steps"
    assert stats[1]["ahead_adopted"] > 0, stats
    assert stats[2]["ahead_adopted"] == 0, stats
    for losses, scales, params, sd in outcomes[1:]:
        assert scales == ref_scales
        assert losses == ref_losses
        for k in ref_params:
            assert torch.equal(params[k], ref_params[k]), k
        for i in ref_sd["state"]:
            for key in ("exp_avg", "exp_avg_sq", "_param_fp32"):
                assert torch.equal(sd["state"][i][key], ref_sd["state"][i][key]), (i, key)
            assert sd["state"][i]["step"] == ref_sd["state"][i]["step"]


def _oracle_run(batches, steps_lr=2e-3):
    torch.manual_seed(3)
    ref = _oracle()
    with torch.no_grad():
        for name, p in ref.named_parameters():   # small weights: a well-conditioned problem, losses near log(vocab)
            if p.dim() > 1:
                p.normal_(0, 0.05)
    init = {k: v.clone() for k, v in ref.state_dict().items()}
    opt = torch.optim.AdamW(ref.parameters(), lr=steps_lr, weight_decay=1e-2)
    pos = torch.arange(S)[None].expand(B, -1)
    mask = torch.ones(B, S, dtype=torch.bool)
    losses = []
    for ids in batches:
        logits = ref(ids[:, :-1], pos, mask)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return init, losses, {k: v.detach().clone() for k, v in ref.state_dict().items()}


@pytest.mark.parametrize("form", ["blocklist", "wrapper"])
@pytest.mark.parametrize("optim", ["adam", "offload"])
def test_training_matches_fp32_oracle(bmt_gpu, form, optim):
    """20 steps in fp16 with dynamic loss scaling, {TransformerBlockList model, BMTrainModelWrapper around a plain torch
    model} x {AdamOptimizer, AdamOffloadOptimizer}, against AdamW on the fp32 PyTorch model: same loss curve and the
    same parameter statistics within half-precision tolerance."""
    bmt = bmt_gpu
    batches = _batches(20, seed=9)
    init, ref_losses, ref_final = _oracle_run(batches)
    if form == "blocklist":
        model = bmt.models.GPT(**CFG, bias=True, dtype=torch.float16)
        bmt.init_parameters(model)
        model.load_state_dict(init)
    else:
        plain = _oracle()
        plain.load_state_dict(init)
        model = bmt.BMTrainModelWrapper(plain.half())
        assert isinstance(model.transformers, bmt.TransformerBlockList)
    cls = bmt.optim.AdamOptimizer if optim == "adam" else bmt.optim.AdamOffloadOptimizer
    opt = cls(model.parameters(), lr=2e-3, weight_decay=1e-2)
    losses, _ = _train(bmt, model, opt, batches, loss_scale=2.0 ** 14, dtype=torch.float16)
    assert abs(losses[0] - ref_losses[0]) < 2e-2
    assert abs(losses[-1] - ref_losses[-1]) < 0.1, (losses[-1], ref_losses[-1])
    assert losses[-1] < losses[0]
    final = _full_state(model)
    for k, r in ref_final.items():
        g = final[k]
        assert g.shape == r.shape, k
        # Adam moves every entry by about lr per step whatever the size of its gradient, so a single entry whose gradient
        # is rounding noise in fp16 can end up to steps * lr = 0.04 away: the extremes get that tolerance
        for stat, tol in ((torch.std, 1e-2), (torch.mean, 1e-2), (torch.max, 4e-2), (torch.min, 4e-2)):
            if r.numel() > 1:
                assert abs(float(stat(g)) - float(stat(r))) < tol, (k, stat.__name__)


def test_wrapped_model_logits_equal_plain_model(bmt_gpu):
    """A wrapped fp16 model computes what the plain fp16 PyTorch model computes (same kernels are not used by the two,
    so equality is up to half-precision rounding of the individual ops)."""
    bmt = bmt_gpu
    torch.manual_seed(17)
    plain = _oracle()
    state = {k: v.clone() for k, v in plain.state_dict().items()}
    ids = _batches(1)[0][:, :-1]
    pos = torch.arange(S)[None].expand(B, -1)
    mask = torch.ones(B, S, dtype=torch.bool)
    want = plain(ids, pos, mask)
    twin = _oracle()
    twin.load_state_dict(state)
    model = bmt.BMTrainModelWrapper(twin.half())
    got = model(ids.cuda(), pos.cuda(), mask.cuda()).float().cpu()
    assert (got - want).abs().max().item() < 3e-2 * max(1.0, want.abs().max().item())
