"""Norms.  RMSNorm: y = x / sqrt(mean(x^2) + eps) * weight, statistics in float32
(crates/cuda-kernels/csrc/misc/norm.cu:221-300).  The gain is held in float32.
With ``one_plus`` the checkpoint stores the gain around zero and the norm multiplies by
1 + weight; the sum is formed once at load, in float32.

Dynamic Tanh stands where a norm stands but forms no mean and no variance: y = tanh(alpha * x) * weight + bias, element
by element, with a stored scalar alpha and a stored bias vector ("<name>.alpha", "<name>.b" beside the weight).  It has no
per-row factor, so it cannot be deferred into the product that follows (``deferred()`` is None)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

from .. import ops
from .base import Norm, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class RmsNormSpec:
    weight_name: str
    size: int
    eps: float
    one_plus: bool = False          # the stored weight is the gain minus one
    kind: ClassVar[str] = "rmsnorm"


class RmsNorm(Norm):
    def __init__(self, spec: RmsNormSpec):
        self.spec = spec
        self.eps = spec.eps
        self.weight = None

    def weight_decls(self):
        return (WeightDecl(self.spec.weight_name, (self.spec.size,), init="around_zero" if self.spec.one_plus else "gain"),)

    def load(self, tensors, dtype, device):
        w = tensors[self.spec.weight_name].to(device=device, dtype=torch.float32)
        self.weight = (w + 1.0 if self.spec.one_plus else w).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * 4

    def scratch_elements_per_token(self):
        return self.spec.size

    def deferred(self):
        return self.weight, self.eps

    def apply(self, resid, delta, rows, out, write_resid: bool):
        """out = norm(resid (+ delta)) on all rows or on ``rows``; see ops.rmsnorm."""
        ops.rmsnorm(resid, delta, rows, self.weight, self.eps, out, write_resid)
        return out

    def add_normed(self, resid, branch, copy):
        """resid += norm(branch) (the norm on a branch's output); ``copy`` gets the new residual in its own type;
        see ops.branch_norm_add."""
        ops.branch_norm_add(resid, branch, self.weight, self.eps, copy)

    def apply_after(self, resid, branch, post, out) -> bool:
        """resid += post(branch), then out = this norm of the new residual, in one kernel; False (nothing done) when
        ``post`` is no RMS norm with a weight."""
        if not isinstance(post, RmsNorm):
            return False
        ops.branch_norm_add_norm(resid, branch, post.weight, post.eps, self.weight, self.eps, out)
        return True


register_part(RmsNormSpec.kind, RmsNorm)


@dataclass(frozen=True)
class DynTanhSpec:
    weight_name: str                # the bias is weight_name + bias_suffix, the scalar weight_name + alpha_suffix
    size: int
    bias_suffix: str = ".b"
    alpha_suffix: str = ".alpha"
    kind: ClassVar[str] = "dyn_tanh"


class DynTanh(Norm):
    eps = 0.0

    def __init__(self, spec: DynTanhSpec):
        self.spec = spec
        self.weight = self.bias = None
        self.alpha = 1.0

    def weight_decls(self):
        s = self.spec
        return (WeightDecl(s.weight_name, (s.size,), init="gain"), WeightDecl(s.weight_name + s.bias_suffix, (s.size,), init="around_zero"),
                WeightDecl(s.weight_name + s.alpha_suffix, (), init="gain"))

    def load(self, tensors, dtype, device):
        s = self.spec
        self.weight = tensors[s.weight_name].to(device=device, dtype=torch.float32).contiguous()
        self.bias = tensors[s.weight_name + s.bias_suffix].to(device=device, dtype=torch.float32).contiguous()
        self.alpha = float(tensors[s.weight_name + s.alpha_suffix].to(torch.float32).item())

    def weight_bytes(self):
        return self.weight.numel() * 8

    def scratch_elements_per_token(self):
        return self.spec.size

    def apply(self, resid, delta, rows, out, write_resid: bool):
        ops.dyt_norm(resid, delta, rows, self.weight, self.bias, self.alpha, out, write_resid)
        return out


register_part(DynTanhSpec.kind, DynTanh)
