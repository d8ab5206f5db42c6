"""Linear attention with one constant decay per head (lightning attention).

    q = silu(W_q x), k = silu(W_k x)   per head [dim];   v = silu(W_v x)   per head [vdim]
    S_t = decay_h * S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t            (S: dim x vdim per head, float32, from zero)
    y = W_o ( rmsnorm(o over all heads at once) * weight * sigmoid(W_g x) )

No positions, no softmax, no cache that grows: what a request keeps is the heads' memories, one float32 row per request
slot that the cache manager zeroes when a request gets the slot.  The four input projections are one packed product;
the silu of q, k and v is applied by the scan as it stages them; the recurrence is the package's scalar-decay scan with the
decays as one number per head; the norm over all heads, its weight and the gate are one kernel.  ``decay`` are the heads'
constants (usually in (0, 1]); nothing else scales q.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import Mixer, StateNeed, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class ConstantDecayAttentionSpec:
    prefix: str
    hidden_size: int
    num_heads: int
    key_dim: int                    # per head, of q and k
    value_dim: int                  # per head
    decay: Tuple[float, ...]        # one per head
    norm_eps: float
    activation: str = "silu"        # on q, k and v ("none": as projected)
    q_scale: float = 1.0
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    kind: ClassVar[str] = "constant_decay_attention"


DEFAULT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("o", "o"), ("norm", "norm"))


class ConstantDecayAttention(Mixer):
    def __init__(self, spec: ConstantDecayAttentionSpec):
        if min(spec.num_heads, spec.key_dim, spec.value_dim) <= 0 or spec.key_dim > 512:
            raise ValueError("constant-decay attention: heads, key_dim (at most 512) and value_dim must be positive")
        if len(spec.decay) != spec.num_heads or not all(0.0 <= float(d) < float("inf") for d in spec.decay):
            raise ValueError(f"constant-decay attention: one decay (not negative) per head, got {len(spec.decay)} for {spec.num_heads} heads")
        if spec.activation not in ("silu", "none"):
            raise ValueError(f"constant-decay attention: activation {spec.activation!r} (silu, none)")
        self.spec = spec
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        self.dqk = spec.num_heads * spec.key_dim
        self.inner = spec.num_heads * spec.value_dim
        self.w_in = self.w_o = self.norm = self.decay = None

    def _name(self, role: str) -> str:
        return self.spec.prefix + self.names[role]

    def weight_decls(self):
        s = self.spec
        return (WeightDecl(self._name("q"), (self.dqk, s.hidden_size)), WeightDecl(self._name("k"), (self.dqk, s.hidden_size)),
                WeightDecl(self._name("v"), (self.inner, s.hidden_size)), WeightDecl(self._name("gate"), (self.inner, s.hidden_size)),
                WeightDecl(self._name("o"), (s.hidden_size, self.inner)), WeightDecl(self._name("norm"), (self.inner,), init="gain"))

    def load(self, tensors, dtype, device):
        def kept(*ts):
            return dtype if dtype == torch.bfloat16 else (torch.float32 if any(t.dtype == torch.float32 for t in ts) else torch.bfloat16)

        main = [tensors[self._name(n)] for n in ("q", "k", "v", "gate")]
        self.w_in = torch.cat([m.to(device=device, dtype=kept(*main)) for m in main], dim=0).contiguous()
        o = tensors[self._name("o")]
        self.w_o = o.to(device=device, dtype=kept(o)).contiguous()
        self.norm = tensors[self._name("norm")].to(device=device, dtype=torch.float32).contiguous()
        self.decay = torch.tensor([float(d) for d in self.spec.decay], dtype=torch.float64).to(torch.float32).to(device)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def scratch_elements_per_token(self):
        return 2 * self.dqk + 6 * self.inner + self.spec.hidden_size

    def state_need(self):
        n = self.spec.num_heads * self.spec.value_dim * self.spec.key_dim
        return StateNeed((-(-n // 4) * 4,), torch.float32)

    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T = x.shape[0]
        H, dqk, inner = s.num_heads, self.dqk, self.inner
        proj = ctx.ws.get("lightning_in", (T, 2 * dqk + 2 * inner), x.dtype)                # q | k | v | gate
        ops.gemm(x, self.w_in, proj)
        o = ctx.ws.get("lightning_o", (T, H, s.value_dim), torch.float32)
        ops.decay_scan(proj[:, :dqk], proj[:, dqk: 2 * dqk], proj[:, 2 * dqk: 2 * dqk + inner], self.decay, None, state, ctx.q_indptr,
                       ctx.state_slots, o, H, H, s.key_dim, s.value_dim, False, s.q_scale, act=s.activation)
        gated = ctx.ws.get("lightning_gated", (T, inner), x.dtype)
        # one norm over all heads at once: a single "head" as wide as the row
        ops.gla_out(o.view(T, inner), proj[:, 2 * dqk + inner:], self.norm, s.norm_eps, 1.0, gated, 1, inner, gate_act="sigmoid")
        out = ctx.ws.get("lightning_out", (T, s.hidden_size), x.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


register_part(ConstantDecayAttentionSpec.kind, ConstantDecayAttention)
