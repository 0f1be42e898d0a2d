"""Plain fp32 PyTorch optimizers used as ground truth where ``torch.optim`` lacks
the exact weight-decay semantics (decoupled SGD, Lion, ``decouple_lr``).

Same role as the reference's ``test/reference.py``; written independently from
the update rules (AdamW, Lion and SGD as published; momentum starts at zero and
dampening applies from the first step, which is what the library implements).
"""

from __future__ import annotations

import torch


class _Base(torch.optim.Optimizer):
    def __init__(self, params, defaults, decouple_lr=False):
        defaults = dict(defaults)
        defaults["initial_lr"] = defaults["lr"]
        super().__init__(params, defaults)
        self.decouple_lr = decouple_lr

    def _decay_factor(self, group):
        wd = group["weight_decay"]
        if self.decouple_lr:
            return wd * group["lr"] / group["initial_lr"]
        return wd * group["lr"]


class ReferenceAdamW(_Base):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, decouple_lr=False,
                 decoupled=True):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay), decouple_lr)
        self.decoupled = decoupled

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                g = p.grad.float()
                w = p.float()
                if not self.decoupled:
                    g = g + group["weight_decay"] * w
                st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                if self.decoupled:
                    w = w * (1 - self._decay_factor(group))
                mhat = st["exp_avg"] / (1 - b1 ** st["step"])
                vhat = st["exp_avg_sq"] / (1 - b2 ** st["step"])
                w = w - group["lr"] * mhat / (vhat.sqrt() + group["eps"])
                p.copy_(w.to(p.dtype))


class ReferenceLion(_Base):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.99), weight_decay=0.0, decouple_lr=False):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay), decouple_lr)

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                g = p.grad.float()
                w = p.float()
                u = torch.sign(st["exp_avg"] * b1 + g * (1 - b1))
                st["exp_avg"].mul_(b2).add_(g, alpha=1 - b2)
                w = w * (1 - self._decay_factor(group)) - group["lr"] * u
                p.copy_(w.to(p.dtype))


class ReferenceSGD(_Base):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False,
                 decoupled=False, decouple_lr=False):
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening,
                                      weight_decay=weight_decay), decouple_lr)
        self.nesterov = nesterov
        self.decoupled = decoupled

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            mu = group["momentum"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                g = p.grad.float()
                w = p.float()
                if not self.decoupled:
                    g = g + group["weight_decay"] * w
                else:
                    w = w * (1 - self._decay_factor(group))
                if mu > 0:
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                    buf = st["momentum_buffer"]
                    buf.mul_(mu).add_(g, alpha=1 - group["dampening"])
                    upd = g + mu * buf if self.nesterov else buf
                else:
                    upd = g
                w = w - group["lr"] * upd
                p.copy_(w.to(p.dtype))
