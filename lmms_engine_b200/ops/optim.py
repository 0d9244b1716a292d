"""Flat-buffer optimizer kernels: AdamW, Muon momentum/update, EMA, grad-norm and clip.

Everything that decides whether and how much to update (clip coefficient, non-finite
skip flag) stays in device memory, so an optimizer step costs no host round trip.  The
reference does the same work with ``torch.optim.AdamW``
(src/lmms_engine/train/fsdp2/fsdp2_trainer.py:202-209), foreach clipping with ``.item()``
syncs (src/lmms_engine/utils/fsdp2_utils.py:235-315) and per-parameter EMA
(src/lmms_engine/utils/ema_utils.py:97-101).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _cuda


def _is_fp32(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 1
    if t.dtype == torch.bfloat16:
        return 0
    raise TypeError(f"unsupported dtype {t.dtype}")


def adamw_step(p32, p16, m, v, g, *, lr, beta1, beta2, eps, wd, step, gscale=None, skip=None) -> None:
    """One AdamW step over flat buffers (fp32 master ``p32``, optional bf16 mirror ``p16``)."""
    bc1 = 1.0 - beta1**step
    bc2 = 1.0 - beta2**step
    if p32.is_cuda:
        _cuda.call(
            "b200_adamw", p32.data_ptr(), _cuda.ptr(p16), m.data_ptr(), v.data_ptr(), g.data_ptr(), _is_fp32(g),
            p32.numel(), float(lr), float(beta1), float(beta2), float(eps), float(wd), float(bc1), float(bc2),
            _cuda.ptr(gscale), _cuda.ptr(skip), _cuda.stream(),
        )
        return
    if skip is not None and int(skip.item()) != 0:
        return
    gf = g.float() * (gscale.item() if gscale is not None else 1.0)
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    p32.mul_(1 - lr * wd)
    p32.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(eps), value=-lr)
    if p16 is not None:
        p16.copy_(p32)


def muon_momentum(mom, g, out, sumsq, *, beta: float, nesterov: bool, gscale=None, eps: float = 1e-7) -> None:
    """``mom = beta*mom + (1-beta)*g``; ``out = bf16(u / (||u||_F + eps))`` with the Nesterov blend."""
    if mom.is_cuda:
        _cuda.call(
            "b200_muon_momentum", mom.data_ptr(), g.data_ptr(), _is_fp32(g), out.data_ptr(), sumsq.data_ptr(),
            mom.numel(), float(beta), int(nesterov), _cuda.ptr(gscale), float(eps), _cuda.stream(),
        )
        return
    gf = g.float() * (gscale.item() if gscale is not None else 1.0)
    mom.mul_(beta).add_(gf, alpha=1 - beta)
    u = gf + beta * (mom - gf) if nesterov else mom
    ub = u.to(out.dtype).float()
    sumsq.fill_(float((ub * ub).sum()))
    out.copy_((ub / (ub.norm() + eps)).to(out.dtype))


def muon_update(p32, p16, o, *, lr: float, wd: float, scale: float, skip=None) -> None:
    if p32.is_cuda:
        _cuda.call(
            "b200_muon_update", p32.data_ptr(), _cuda.ptr(p16), o.data_ptr(), p32.numel(), float(lr), float(wd),
            float(scale), _cuda.ptr(skip), _cuda.stream(),
        )
        return
    if skip is not None and int(skip.item()) != 0:
        return
    p32.mul_(1 - lr * wd).add_(o.float(), alpha=-lr * scale)
    if p16 is not None:
        p16.copy_(p32)


def ema_update(ema: torch.Tensor, p: torch.Tensor, decay: float) -> None:
    if ema.is_cuda:
        _cuda.call("b200_ema", ema.data_ptr(), p.data_ptr(), _is_fp32(p), ema.numel(), float(decay), _cuda.stream())
    else:
        ema.mul_(decay).add_(p.float(), alpha=1 - decay)


_scratch = {}


def _partials(device) -> torch.Tensor:
    key = (device.type, device.index)
    t = _scratch.get(key)
    if t is None:
        n = _cuda.fn("b200_num_partials")()
        t = torch.empty(n, dtype=torch.float32, device=device)
        _scratch[key] = t
    return t


def sumsq_(g: torch.Tensor, out: torch.Tensor, accumulate: bool) -> None:
    """``out[0] (+)= sum(g^2)`` (deterministic two-stage reduction on CUDA)."""
    if g.is_cuda:
        _cuda.call(
            "b200_sumsq", g.data_ptr(), _is_fp32(g), g.numel(), _partials(g.device).data_ptr(), out.data_ptr(),
            int(accumulate), _cuda.stream(),
        )
    else:
        s = g.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s


def clip_coef(sumsq, norm_out, coef_out, skip_out, max_norm: float) -> None:
    """norm = sqrt(sumsq); coef = min(1, max_norm/(norm+1e-6)); skip = !isfinite(norm), or a kernel
    of this device has raised the status word since it was last read (a bounded wait that ran out
    leaves the step's gradients incomplete: such a step must not update the weights)."""
    if sumsq.is_cuda:
        _cuda.call(
            "b200_clip_coef", sumsq.data_ptr(), norm_out.data_ptr(), coef_out.data_ptr(), skip_out.data_ptr(),
            float(max_norm), _cuda.status_word(sumsq.device).data_ptr(), _cuda.stream(),
        )
        return
    norm = float(sumsq.item()) ** 0.5 if sumsq.item() >= 0 else float("nan")
    finite = math.isfinite(norm)
    norm_out.fill_(norm)
    skip_out.fill_(0 if finite else 1)
    coef_out.fill_(min(1.0, max_norm / (norm + 1e-6)) if (finite and max_norm > 0) else 1.0)


def scale_(g: torch.Tensor, coef: torch.Tensor) -> None:
    if g.is_cuda:
        _cuda.call("b200_scale", g.data_ptr(), _is_fp32(g), g.numel(), coef.data_ptr(), _cuda.stream())
    else:
        g.mul_(coef.item())
