"""GPT pre-training loop on synthetic tokens: the counterpart of the reference's ``example/train.py``.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_gpt.py
    python examples/train_gpt.py --layers 2 --dim 128 --heads 4 --ffn 256 --iters 20        # one process, any device

Same ingredients as the reference script: variable-length random sequences with the padding masked out of the loss,
``AdamOffloadOptimizer`` + ``Noam`` warm-up + ``OptimManager`` with dynamic loss scaling, activations recorded for
``inspect`` every ``--inspect-every`` iterations, gathered checkpoint at the end.  Differences: the layout is a command
line option (``--tp``, ``--pp``) instead of being edited in the source, timing uses ``StepTimer`` (device time, maximum
over ranks) instead of ``time.time``.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bmtrain_b200 as bmt  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--dim", type=int, default=2560)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=10240)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--iters", type=int, default=1000)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--optimizer", default="offload", choices=["offload", "adam"])
    ap.add_argument("--inspect-every", type=int, default=100)
    ap.add_argument("--save", default="")
    args = ap.parse_args()

    kw = dict(pipe_size=args.pp, num_micro_batches=args.pp) if args.pp > 1 else {}
    bmt.init_distributed(seed=0, tp_size=args.tp, **kw)
    cuda = bmt.config["device"].type == "cuda"
    dtype = torch.half if cuda else torch.float32
    model = bmt.models.GPT(args.layers, args.vocab, args.dim, args.dim // args.heads, args.heads, args.ffn, args.seq,
                           bias=True, dtype=dtype)
    bmt.init_parameters(model)
    bmt.print_rank("Model memory")
    if cuda:
        bmt.print_rank(torch.cuda.memory_summary(abbreviated=True))
    bmt.synchronize()

    # every data-parallel rank draws its own batch of random length sequences; padding is masked and ignored by the loss
    dev = bmt.config["device"]
    torch.manual_seed(1000 + bmt.rank() // args.tp)
    lengths = torch.randint(args.seq // 4, args.seq + 1, (args.batch,))
    tokens = torch.randint(0, args.vocab, (args.batch, args.seq + 1))
    position = torch.arange(args.seq + 1)[None]
    valid = position < lengths[:, None]
    targets = torch.where(valid[:, 1:], tokens[:, 1:], torch.full_like(tokens[:, 1:], -100))
    inputs, pos, mask = tokens[:, :-1].to(dev), position[:, :-1].expand(args.batch, -1).contiguous().to(dev), valid[:, :-1].to(dev)
    targets = targets.to(dev)
    if args.tp > 1:
        targets = targets.t().contiguous()  # tensor-parallel models work sequence-first

    loss_func = bmt.loss.FusedCrossEntropy(ignore_index=-100, parallel=args.tp > 1)
    opt_cls = bmt.optim.AdamOffloadOptimizer if args.optimizer == "offload" else bmt.optim.AdamOptimizer
    optimizer = opt_cls(model.parameters(), weight_decay=1e-2)
    lr_scheduler = bmt.lr_scheduler.Noam(optimizer, start_lr=1e-3, warmup_iter=40, end_iter=args.iters, num_iter=0)
    optim_manager = bmt.optim.OptimManager(loss_scale=2 ** 20 if dtype == torch.half else None)
    optim_manager.add_optimizer(optimizer, lr_scheduler)
    bmt.synchronize()

    timer = bmt.utils.StepTimer()
    avg_loss = bmt.utils.AverageRecorder()
    for iteration in range(args.iters):
        inspecting = args.inspect_every > 0 and iteration % args.inspect_every == 0
        with timer.phase("forward"):
            with bmt.inspect.inspect_tensor() as inspector:
                logits = model(inputs, pos, mask)
                loss = loss_func(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1))
                global_loss = bmt.sum_loss(loss).item()
        with timer.phase("backward"):
            optim_manager.zero_grad()
            optim_manager.backward(loss)
        if inspecting:
            bmt.print_rank(bmt.inspect.format_summary(inspector.get_summary()))
            bmt.print_rank(bmt.inspect.format_summary(bmt.inspect.inspect_model(model, "*")))
        with timer.phase("optimizer"):
            optim_manager.step()
        ms = timer.finish_step()
        avg_loss.record(global_loss)
        bmt.print_rank("| Iter: {:6d} | loss: {:.4f} average_loss: {:.4f} | lr: {:.4e} scale: {:10.4f} | fwd {:.1f} bwd {:.1f} opt {:.1f} ms".format(
            iteration, global_loss, avg_loss.value, lr_scheduler.current_lr, optim_manager.loss_scale or 1.0,
            ms["forward"], ms["backward"], ms["optimizer"]))
    if args.save:
        bmt.save(model, args.save)
    bmt.shutdown()


if __name__ == "__main__":
    main()
