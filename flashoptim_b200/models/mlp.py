"""784 -> 256 -> ReLU -> 10 classifier: the smallest end-to-end configuration (the model of the
reference's only example, ``examples/train_mnist.py``)."""

from __future__ import annotations

import torch.nn as nn


def make_mlp(d_in: int = 784, d_hidden: int = 256, d_out: int = 10) -> nn.Sequential:
    return nn.Sequential(nn.Linear(d_in, d_hidden), nn.ReLU(), nn.Linear(d_hidden, d_out))
