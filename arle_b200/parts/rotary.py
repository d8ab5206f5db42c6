"""Rotary position encoding over the first ``rotary_dim`` elements of a head:
inv_freq_i = theta^(-2i/rotary_dim) / divide_by (divide_by 1 unless positions are scaled linearly), angle = position * inv_freq_i
(infer/src/weight_loader.rs:955-989).  ``pairing`` says which two elements turn
together: "half" pairs element i with i + rotary_dim/2 (Qwen3), "interleaved" pairs
element 2i with 2i + 1.  The reference tabulates cos and
sin of every position in bfloat16; here the kernels evaluate sincosf of the float32
angle of the positions they meet (for prompt portions once per step, into a table
that the step's layers share), so there is no limit on the position."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

from .base import PositionEncoding
from .registry import register_part


@dataclass(frozen=True)
class RotarySpec:
    rotary_dim: int
    theta: float
    pairing: str = "half"
    divide_by: float = 1.0          # linear scaling of positions: every frequency is divided by this
    kind: ClassVar[str] = "rotary"


class Rotary(PositionEncoding):
    def __init__(self, spec: RotarySpec):
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        if spec.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing must be 'half' or 'interleaved', got {spec.pairing!r}")
        if not spec.divide_by > 0:
            raise ValueError(f"rotary divide_by must be positive, got {spec.divide_by}")
        self.spec = spec
        self.inv_freq = None

    def load(self, tensors, dtype, device):
        i = torch.arange(self.spec.rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.spec.theta, dtype=torch.float64), -2.0 * i / self.spec.rotary_dim) / self.spec.divide_by
        self.inv_freq = inv.to(torch.float32).to(device)

    def rotary(self):
        return self.inv_freq, self.spec.rotary_dim

    @property
    def pairing(self) -> str:
        return self.spec.pairing


register_part(RotarySpec.kind, Rotary)
