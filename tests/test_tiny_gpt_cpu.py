"""Tiny GPT (2 pre-LN blocks, d256, 4x64 heads, FFN 1024, vocab 10240, seq 128, fp32) trained for 10 Adam
steps on CPU ranks through Block(zero_level=3) / TransformerBlockList, against a plain PyTorch model."""
import pytest
import torch

from dist_utils import run_distributed

CFG = dict(num_layers=2, vocab=10240, d=256, dh=64, h=4, dff=1024, max_distance=128)


def _data(step, batch=2, seq=128, vocab=10240):
    g = torch.Generator().manual_seed(1234 + step)
    ids = torch.randint(0, vocab, (batch, seq + 1), generator=g)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def _oracle_run(world, steps):
    """Single-process reference: the global batch is the concatenation of every rank's batch."""
    from oracle import OracleGPT

    torch.manual_seed(0)
    model = OracleGPT(CFG["num_layers"], CFG["vocab"], CFG["d"], CFG["dh"], CFG["h"], CFG["dff"], CFG["max_distance"])
    return model


def body_train(steps=10, zero_level=3, use_checkpoint=True):
    import bmtrain_b200 as bmt
    from oracle import OracleGPT

    rank, world = bmt.rank(), bmt.world_size()
    model = bmt.models.GPT(CFG["num_layers"], CFG["vocab"], CFG["d"], CFG["dh"], CFG["h"], CFG["dff"],
                           CFG["max_distance"], dtype=torch.float32, zero_level=zero_level, use_checkpoint=use_checkpoint)
    # oracle with identical weights: N(0, 0.02) drawn once on every rank with the same seed
    torch.manual_seed(42)
    ref = OracleGPT(CFG["num_layers"], CFG["vocab"], CFG["d"], CFG["dh"], CFG["h"], CFG["dff"], CFG["max_distance"])
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.02)
    missing = model.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys

    opt = bmt.optim.AdamOptimizer(model.parameters(), lr=1e-3)
    ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-3)
    om = bmt.optim.OptimManager(loss_scale=None)
    om.add_optimizer(opt)
    loss_fn = torch.nn.CrossEntropyLoss()

    for step in range(steps):
        # every rank draws its own batch; the oracle sees all of them
        batches = [_data(step * world + r) for r in range(world)]
        ids, labels = batches[rank]
        pos = torch.arange(ids.shape[1])[None].expand_as(ids).contiguous()
        mask = torch.ones_like(ids, dtype=torch.bool)
        logits = model(ids, pos, mask)
        loss = loss_fn(logits.view(-1, logits.shape[-1]), labels.view(-1))
        gl = bmt.sum_loss(loss.detach())
        om.zero_grad()
        om.backward(loss)
        om.step()

        ref_opt.zero_grad()
        ref_loss = 0
        for r in range(world):
            rids, rlabels = batches[r]
            rl = loss_fn(ref(rids, pos, mask).view(-1, CFG["vocab"]), rlabels.view(-1)) / world
            rl.backward()
            ref_loss += rl.item()
        ref_opt.step()
        assert abs(gl.item() - ref_loss) < 2e-4 * max(1.0, abs(ref_loss)), (step, gl.item(), ref_loss)

    # final parameters agree with the single-process run
    sd = {}
    from bmtrain_b200.store import _save_to_rank0
    sd = _save_to_rank0(model)
    if rank == 0:
        for k, v in ref.state_dict().items():
            assert torch.allclose(sd[k].float(), v, atol=2e-4, rtol=1e-3), k


@pytest.mark.parametrize("world", [1, 2])
def test_tiny_gpt_zero3(world):
    run_distributed("test_tiny_gpt_cpu", "body_train", world, steps=10, zero_level=3, use_checkpoint=True)


def test_tiny_gpt_zero2_nocheckpoint():
    run_distributed("test_tiny_gpt_cpu", "body_train", 2, steps=3, zero_level=2, use_checkpoint=False)


def test_example_script_runs_on_cpu(tmp_path):
    """The example training loop end to end on one CPU process (tiny model): inspect tables, timing line, checkpoint."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ckpt = tmp_path / "model.pt"
    env = dict(os.environ, BMT_DEVICE="cpu", BMT_QUIET="1", MASTER_PORT="29873")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE"):
        env.pop(k, None)
    out = subprocess.run([sys.executable, os.path.join(root, "examples", "train_gpt.py"), "--layers", "2", "--dim", "64", "--heads", "4",
                          "--ffn", "128", "--vocab", "256", "--seq", "32", "--iters", "3", "--inspect-every", "2", "--save", str(ckpt)],
                         capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "| Iter:      2 |" in out.stdout and "transformers.1.ff.w_out.weight" in out.stdout
    import torch

    state = torch.load(ckpt, map_location="cpu")
    assert state["transformers.0.attn.project_qkv.weight"].shape == (192, 64)
