"""Train a small CNN on MNIST-shaped data with ``cast_model`` + ``FlashAdamW``.

    python examples/train_mnist.py --master-weight-bits 24 --gradient-release
    python examples/train_mnist.py --data /path/to/mnist.npz      # real digits, if you have them

Counterpart of the reference's ``examples/train_mnist.py``: bf16 parameters with
24-bit master weights, 8-bit optimizer states, a cosine schedule, optional
gradient release, and an fp32 checkpoint round trip at the end that must not
change the accuracy.  Without ``--data`` a synthetic, learnable 10-class image
problem of the same shape is generated (no download is attempted).
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from flashoptim_b200 import FlashAdamW, cast_model, enable_gradient_release  # noqa: E402


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 16, 3, padding=1)
        self.conv2 = nn.Conv2d(16, 32, 3, padding=1)
        self.fc1 = nn.Linear(32 * 7 * 7, 128)
        self.fc2 = nn.Linear(128, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        return self.fc2(F.relu(self.fc1(x.flatten(1))))


def load_data(path, n_train=8192, n_test=2048, seed=0):
    if path:
        d = np.load(path)
        xtr, ytr, xte, yte = d["x_train"], d["y_train"], d["x_test"], d["y_test"]
        f = lambda a: torch.from_numpy(a).float().div(255.0).sub(0.1307).div(0.3081).unsqueeze(1)
        return f(xtr), torch.from_numpy(ytr).long(), f(xte), torch.from_numpy(yte).long()
    g = torch.Generator().manual_seed(seed)
    protos = torch.randn(10, 1, 28, 28, generator=g)

    def make(n):
        y = torch.randint(0, 10, (n,), generator=g)
        return protos[y] + 0.8 * torch.randn(n, 1, 28, 28, generator=g), y

    xtr, ytr = make(n_train)
    xte, yte = make(n_test)
    return xtr, ytr, xte, yte


@torch.no_grad()
def accuracy(model, x, y, dtype, bs=512):
    model.eval()
    hit = 0
    for i in range(0, len(x), bs):
        hit += (model(x[i:i + bs].to(dtype)).argmax(1) == y[i:i + bs]).sum().item()
    model.train()
    return hit / len(x)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default=None, help=".npz with x_train/y_train/x_test/y_test")
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--batch-size", type=int, default=128)
    ap.add_argument("--lr", type=float, default=2e-3)
    ap.add_argument("--weight-decay", type=float, default=1e-2)
    ap.add_argument("--master-weight-bits", default="24", choices=["24", "32", "none"])
    ap.add_argument("--no-quantize", action="store_true")
    ap.add_argument("--gradient-release", action="store_true")
    ap.add_argument("--compress-state-dict", action="store_true")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()

    dev = torch.device(args.device)
    torch.manual_seed(0)
    xtr, ytr, xte, yte = (t.to(dev) for t in load_data(args.data))
    model = Net().to(dev)
    cast_model(model, torch.bfloat16)
    mwb = None if args.master_weight_bits == "none" else int(args.master_weight_bits)
    opt = FlashAdamW(model.parameters(), lr=args.lr, weight_decay=args.weight_decay, master_weight_bits=mwb,
                     quantize=not args.no_quantize, compress_state_dict=args.compress_state_dict)
    steps = args.epochs * (len(xtr) // args.batch_size)
    sched = torch.optim.lr_scheduler.CosineAnnealingLR(opt, T_max=steps)
    handle = enable_gradient_release(model, opt) if args.gradient_release else None
    print(opt)
    step = 0
    for epoch in range(args.epochs):
        perm = torch.randperm(len(xtr), device=dev)
        for i in range(0, len(xtr) - args.batch_size + 1, args.batch_size):
            idx = perm[i:i + args.batch_size]
            loss = F.cross_entropy(model(xtr[idx].to(torch.bfloat16)).float(), ytr[idx])
            loss.backward()
            if handle is None:
                opt.step()
                opt.zero_grad()
            sched.step()
            step += 1
            if step % 50 == 0:
                print(f"epoch {epoch} step {step}/{steps} loss {loss.item():.4f} lr {sched.get_last_lr()[0]:.2e}")
        print(f"epoch {epoch}: test accuracy {accuracy(model, xte, yte, torch.bfloat16):.4f}")
    acc = accuracy(model, xte, yte, torch.bfloat16)

    # fp32 export -> fresh bf16 model + optimizer -> import: accuracy must not move
    if handle is not None:
        handle.remove()
    fp32_sd = opt.get_fp32_model_state_dict(model)
    model2 = Net().to(dev)
    cast_model(model2, torch.bfloat16)
    opt2 = FlashAdamW(model2.parameters(), lr=args.lr, master_weight_bits=mwb)
    for p in model2.parameters():  # create optimizer state (incl. correction codes)
        p.grad = torch.zeros_like(p)
    for g in opt2.param_groups:
        g["lr"] = 0.0
    opt2.step()
    opt2.set_fp32_model_state_dict(model2, fp32_sd)
    acc2 = accuracy(model2, xte, yte, torch.bfloat16)
    print(f"final accuracy {acc:.4f}; after fp32 checkpoint round trip {acc2:.4f}")
    assert abs(acc - acc2) < 5e-3, "fp32 round trip changed the model"


if __name__ == "__main__":
    main()
