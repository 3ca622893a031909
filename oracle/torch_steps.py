"""PyTorch-on-CPU restatement of one optimizer step.  TEST INFRASTRUCTURE ONLY.

Follows the reference's own pure-torch checkers: ``_reference_sgd_step`` and
``_reference_adamw_step`` (``tests/test_correctness.py:27-55``: materialise ``dY^T X``, then the
textbook update with in-place torch ops) and its int8 quantiser (``:170-180``).  Also the plain
baseline of the single-linear configuration: torch autograd + ``torch.optim.AdamW`` on CPU.
Everything here runs on CPU tensors; it is the tolerance-level oracle and the timed CPU baseline.
"""

from __future__ import annotations

import torch


def grad_weight(grad_output: torch.Tensor, input: torch.Tensor) -> torch.Tensor:
    """``dW = dY^T X`` in fp32 (bf16 operands are widened first: products are then exact)."""
    return grad_output.float().t() @ input.float()


def sgd_step(grad_output, input, weight, lr, weight_decay):
    """Returns W' = W (1 - lr wd) - lr dW as fp32."""
    w = weight.float().clone()
    w.mul_(1.0 - lr * weight_decay)
    w.add_(grad_weight(grad_output, input), alpha=-lr)
    return w


def adamw_step(grad_output, input, weight, m, v, lr, beta1, beta2, eps, weight_decay, step):
    """Returns (W', m', v') as fp32 tensors; inputs are not modified."""
    g = grad_weight(grad_output, input)
    return adamw_from_grad(g, weight, m, v, lr, beta1, beta2, eps, weight_decay, step)


def adamw_from_grad(g, weight, m, v, lr, beta1, beta2, eps, weight_decay, step):
    m_new = m.float().clone().mul_(beta1).add_(g, alpha=1 - beta1)
    v_new = v.float().clone().mul_(beta2).add_(g.square(), alpha=1 - beta2)
    m_hat = m_new / (1.0 - beta1 ** step)
    v_hat = v_new / (1.0 - beta2 ** step)
    w = weight.float().clone()
    w.mul_(1.0 - lr * weight_decay)
    w.add_(m_hat / (v_hat.sqrt() + eps), alpha=-lr)
    return w, m_new, v_new


def int8_quantise(x: torch.Tensor, qblock: int = 64):
    """Per-(row, qblock) absmax quantiser: scale = absmax/127 + 1e-12, code = round(x/scale)."""
    V, H = x.shape
    xb = x.float().reshape(V, H // qblock, qblock)
    scale = xb.abs().amax(dim=2) / 127.0 + 1e-12
    q = (xb / scale[:, :, None]).round().clamp(-127, 127).to(torch.int8).reshape(V, H)
    return q, scale


def int8_dequantise(q: torch.Tensor, scale: torch.Tensor, qblock: int = 64):
    V, H = q.shape
    return (q.float().reshape(V, H // qblock, qblock) * scale[:, :, None]).reshape(V, H)


def sgd_momentum_step(g, weight, buf, lr, momentum, weight_decay, nesterov):
    """Momentum buffer of torch.optim.SGD (dampening 0) with the reference's decoupled decay."""
    b = buf.float() * momentum + g
    u = g + momentum * b if nesterov else b
    w = weight.float() * (1.0 - lr * weight_decay) - lr * u
    return w, b


def lion_step(g, weight, m, lr, beta1, beta2, weight_decay):
    c = beta1 * m.float() + (1 - beta1) * g
    w = weight.float() * (1.0 - lr * weight_decay) - lr * torch.sign(c)
    m_new = beta2 * m.float() + (1 - beta2) * g
    return w, m_new


class TorchAdamWLinear:
    """Vanilla baseline: one bias-free ``nn.Linear`` trained by autograd + ``torch.optim.AdamW`` on
    CPU, fed the upstream gradient dY directly (``Y.backward(dY)``)."""

    def __init__(self, weight: torch.Tensor, lr, betas, eps, weight_decay):
        self.weight = torch.nn.Parameter(weight.detach().float().clone())
        self.opt = torch.optim.AdamW([self.weight], lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)

    def step(self, x: torch.Tensor, dy: torch.Tensor):
        self.opt.zero_grad(set_to_none=True)
        y = torch.nn.functional.linear(x.float(), self.weight)
        y.backward(dy.float())
        self.opt.step()
        return self.weight.detach()
