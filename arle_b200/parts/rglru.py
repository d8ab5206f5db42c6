"""The recurrent block with a real-gated linear recurrent unit (RG-LRU), as a mixer.

Two branches of ``width`` channels read the input h: y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x), a causal
convolution per channel (``conv_taps`` taps, the last one the current token's, zeros before a request's first token, a bias,
no activation).  u is cut into ``blocks`` equal parts; in part b, with square matrices [out, in],

    r = sigmoid(W_ra[b] u_b + b_ra[b]),  i = sigmoid(W_ri[b] u_b + b_ri[b]),
    log a = -decay_constant * r * softplus(lam),  a = exp(log a),
    S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t          (S = 0 before the first token, which is no special case)

and the output is W_o (S * y).  The state (S, float32, and the convolution's last taps - 1 inputs) lives in the request's
state slot.  The gates, the decay and the recurrence are float32 in both precisions: the block-diagonal product that
forms the gates' sums reads u in the activation type and leaves its float32 sums as they are.  W_y and W_x are one packed
product; the two gate matrices of a block are one matrix [2 * bs, bs], so the gates' sums are one block-diagonal product.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import Mixer, StateNeed, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class RgLruSpec:
    prefix: str
    hidden_size: int
    width: int
    blocks: int
    conv_taps: int
    decay_constant: float = 8.0
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    kind: ClassVar[str] = "rglru"


DEFAULT_NAMES = (("y", "y"), ("y_bias", "y.b"), ("x", "x"), ("x_bias", "x.b"), ("conv", "conv"), ("conv_bias", "conv.b"),
                 ("ra", "ra"), ("ra_bias", "ra.b"), ("ri", "ri"), ("ri_bias", "ri.b"), ("lam", "lam"), ("o", "o"))


class RgLru(Mixer):
    def __init__(self, spec: RgLruSpec):
        if min(spec.width, spec.blocks, spec.conv_taps) <= 0 or spec.width % spec.blocks:
            raise ValueError("rglru: width, blocks and conv_taps must be positive and width a multiple of blocks")
        self.spec = spec
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        self.bs = spec.width // spec.blocks
        self.w_yx = self.w_o = self.w_gates = None
        self.y_bias = self.x_bias = self.conv = self.conv_bias = self.ra_bias = self.ri_bias = self.lam = None

    def _name(self, role: str) -> str:
        return self.spec.prefix + self.names[role]

    def weight_decls(self):
        s, bs = self.spec, self.bs
        return (WeightDecl(self._name("y"), (s.width, s.hidden_size)), WeightDecl(self._name("y_bias"), (s.width,), init="around_zero"),
                WeightDecl(self._name("x"), (s.width, s.hidden_size)), WeightDecl(self._name("x_bias"), (s.width,), init="around_zero"),
                WeightDecl(self._name("conv"), (s.width, s.conv_taps), init="around_zero"),
                WeightDecl(self._name("conv_bias"), (s.width,), init="around_zero"),
                WeightDecl(self._name("ra"), (s.blocks, bs, bs)), WeightDecl(self._name("ra_bias"), (s.blocks, bs), init="around_zero"),
                WeightDecl(self._name("ri"), (s.blocks, bs, bs)), WeightDecl(self._name("ri_bias"), (s.blocks, bs), init="around_zero"),
                WeightDecl(self._name("lam"), (s.width,), init="around_zero"), WeightDecl(self._name("o"), (s.hidden_size, s.width)))

    def load(self, tensors, dtype, device):
        def kept(*ts):
            return dtype if dtype == torch.bfloat16 else (torch.float32 if any(t.dtype == torch.float32 for t in ts) else torch.bfloat16)

        y, x, o = (tensors[self._name(n)] for n in ("y", "x", "o"))
        self.w_yx = torch.cat([y.to(device=device, dtype=kept(y, x)), x.to(device=device, dtype=kept(y, x))], dim=0).contiguous()
        self.w_o = o.to(device=device, dtype=kept(o)).contiguous()
        ra, ri = tensors[self._name("ra")], tensors[self._name("ri")]
        self.w_gates = torch.cat([ra, ri], dim=1).to(device=device, dtype=kept(ra, ri)).contiguous()     # [blocks, 2 * bs, bs]
        self.y_bias, self.x_bias, self.conv, self.conv_bias, self.lam = (
            tensors[self._name(n)].to(device=device, dtype=torch.float32).contiguous() for n in ("y_bias", "x_bias", "conv", "conv_bias", "lam"))
        self.ra_bias, self.ri_bias = (tensors[self._name(n)].to(device=device, dtype=torch.float32).reshape(-1).contiguous()
                                      for n in ("ra_bias", "ri_bias"))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_yx, self.w_o, self.w_gates))

    def scratch_elements_per_token(self):
        return 10 * self.spec.width + self.spec.hidden_size

    def state_need(self):
        n = self.spec.width * self.spec.conv_taps            # the states, then taps - 1 inputs a channel
        return StateNeed((-(-n // 4) * 4,), torch.float32)

    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T, W = x.shape[0], s.width
        yx = ctx.ws.get("lru_yx", (T, 2 * W), x.dtype)
        ops.gemm(x, self.w_yx, yx)
        u = ctx.ws.get("lru_u", (T, W), x.dtype)
        ops.causal_conv(yx[:, W:], self.x_bias, self.conv, self.conv_bias, "none", state, W, ctx.q_indptr, ctx.row_of_token,
                        ctx.state_slots, u)
        z = ctx.ws.get("lru_z", (T, 2 * W), torch.float32)
        ops.gemm_heads(u.view(T, s.blocks, self.bs), self.w_gates, z.view(T, s.blocks, 2 * self.bs))
        gated = ctx.ws.get("lru_out", (T, W), x.dtype)
        ops.rglru_scan(z, u, yx[:, :W], self.ra_bias, self.ri_bias, self.lam, self.y_bias, s.decay_constant, state, ctx.q_indptr,
                       ctx.state_slots, gated, s.blocks, ctx.max_q_len)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


register_part(RgLruSpec.kind, RgLru)
