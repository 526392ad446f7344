"""AdamW / Adam over all flat shards in one multi-tensor launch.

The trainable tensors of a run are the flat weight shards (fp32) and the flat
input-feature shard (bf16 on the device).  Parameters that are not fp32 get an
fp32 master copy in the optimizer state; the update is computed in fp32 on the
master and written back to the parameter in its own dtype.  On CUDA all
tensors are updated by a single kernel launch (``csrc/kernels/adam.cu``); on
CPU the same arithmetic runs in torch.

The reference trains with ``torch.optim.AdamW`` over the model parameters plus
the input features (reference: examples/train.py:155-159).
"""

from __future__ import annotations

from typing import Iterable

import torch

from .ops import reference


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 3e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, decoupled: bool = True):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled=decoupled)
        super().__init__(params, defaults)

    def _init_state(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            acc = torch.float64 if p.dtype == torch.float64 else torch.float32
            st["exp_avg"] = torch.zeros_like(p, dtype=acc)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=acc)
            st["master"] = p.detach().float().clone() if p.dtype not in (torch.float32, torch.float64) else None
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            ps, gs, ms, vs, ws = [], [], [], [], []
            step = None
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._init_state(p)
                st["step"] += 1
                step = st["step"]
                ps.append(p.data)
                gs.append(p.grad.data)
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
                ws.append(st["master"])
            if not ps:
                continue
            b1, b2 = group["betas"]
            args = (ps, gs, ms, vs, ws, step, group["lr"], b1, b2, group["eps"],
                    group["weight_decay"], group["decoupled"])
            if ps[0].is_cuda:
                from .ops import cuda as opc

                opc.adam_step(*args)
            else:
                reference.adam_step(*args)
        return loss


# same update rule, L2 regularisation folded into the gradient
def FusedAdam(params, **kw):
    kw.setdefault("decoupled", False)
    return FusedAdamW(params, **kw)
