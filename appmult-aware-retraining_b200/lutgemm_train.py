"""Data-parallel AppMult-aware training launcher (one process per GPU, NCCL):

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 lutgemm_train.py \\
        [--lut-file FILE] [--bits 7] [--batch 256] [--steps 100] [--lr 0.01] [--ste] [--conv-impl fused]

What the reference's single-GPU loop does per step (micronet+/app_train.py:23-36: forward, cross-entropy,
backward, optimizer step) with the batch sharded over the ranks and the parameter gradients averaged by
bucketed all-reduce.  Without --lut-file the benchmark's synthetic multiplier is used; data is synthetic
(N(0,1) images of the CIFAR shape, uniform labels) because no dataset ships with this repository - plug a
DataLoader with a DistributedSampler into `batches` for real data.  Observer statistics (activation /
weight ranges) stay per rank, like the per-GPU batch-norm statistics."""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

import self_ops
from lutgemm_dp import OverlappedGradReducer
from lutgemm_layers import prepare
from lutgemm_luts import synthetic_multiplier, window_difference_gradients
from lutgemm_models import MODELS


def install_tables(device, bits: int, lut_file: str | None) -> None:
    if lut_file:
        self_ops.init_lookup_tables(device, lut_file, bits)
    else:
        fp = synthetic_multiplier(bits, seed=0)
        ga, gb = window_difference_gradients(fp, max(1, (1 << bits) // 16))
        self_ops.set_lookup_tables(device, fp, ga, gb, bits)


def build(device, bits: int, conv_impl: str = "layer", use_ste: bool = False, lr: float = 0.01, model_name: str = "resnet18"):
    torch.manual_seed(0)  # identical initial weights on every rank
    ctor, _, classes = MODELS[model_name]
    model = ctor(classes).to(device)
    prepare(model, a_bits=bits, w_bits=bits, use_ste_gradient=use_ste, conv_impl=conv_impl)
    model = model.to(memory_format=torch.channels_last).train()
    opt = torch.optim.SGD(model.parameters(), lr=lr, momentum=0.9)
    return model, opt


def train_step(model, opt, reducer, images, labels):
    """One step: forward, cross-entropy, backward with the bucketed gradient all-reduce launched from hooks
    while backward runs (`reducer`: an OverlappedGradReducer over the model's parameters), optimizer step."""
    reducer.zero_grad()
    loss = F.cross_entropy(model(images), labels)
    loss.backward()
    reducer.finish()
    opt.step()
    return loss


@torch.no_grad()
def evaluate(model, batches):
    """Top-1 accuracy over (images, labels) batches, without building autograd graphs (the reference's test loop
    runs with gradients enabled, micronet+/app_train.py:39-85); observers are frozen by eval()."""
    was_training = model.training
    model.eval()
    correct = total = 0
    for images, labels in batches:
        correct += int((model(images).argmax(dim=1) == labels).sum())
        total += labels.numel()
    model.train(was_training)
    return correct / max(1, total)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=sorted(MODELS), default="resnet18")
    ap.add_argument("--lut-file", default=None)
    ap.add_argument("--bits", type=int, default=7, choices=[4, 6, 7, 8])
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--ste", action="store_true", help="straight-through backward instead of the gradient tables")
    ap.add_argument("--conv-impl", choices=["layer", "fused", "unfold"], default="layer")
    ap.add_argument("--eval-batches", type=int, default=0, help="synthetic batches to evaluate after training")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    device = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}")
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    install_tables(device, args.bits, args.lut_file)
    model, opt = build(device, args.bits, args.conv_impl, args.ste, args.lr, args.model)
    _, image_shape, classes = MODELS[args.model]
    reducer = OverlappedGradReducer(model.parameters())
    g = torch.Generator().manual_seed(100 + rank)
    t0 = time.time()
    for step in range(args.steps):
        images = torch.randn(args.batch, *image_shape, generator=g).pin_memory().to(device, non_blocking=True)
        labels = torch.randint(0, classes, (args.batch,), generator=g).pin_memory().to(device, non_blocking=True)
        loss = train_step(model, opt, reducer, images, labels)
        if rank == 0 and (step % 10 == 0 or step == args.steps - 1):
            print(f"step {step:4d}  loss {loss.item():.4f}  {world * args.batch * (step + 1) / (time.time() - t0):.0f} img/s",
                  flush=True)
    if args.eval_batches:
        data = [(torch.randn(args.batch, *image_shape, generator=g).to(device),
                 torch.randint(0, classes, (args.batch,), generator=g).to(device)) for _ in range(args.eval_batches)]
        acc = evaluate(model, data)
        if rank == 0:
            print(f"eval accuracy on {args.eval_batches} synthetic batches: {acc:.4f}", flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
