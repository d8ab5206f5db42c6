"""The gated delta rule as a mixer: a matrix memory per head that forgets by a scalar decay and is corrected towards the
value of the current key.

q = W_q h and k = W_k h have ``num_kq_heads`` heads of ``key_dim``, v = W_v h has ``num_heads`` heads of ``value_dim`` (head h
reads q/k head h // (num_heads / num_kq_heads)); no biases.  Each of q, k, v passes a causal convolution per channel
(``conv_taps`` taps, the last one the current token's, no bias, zeros before a request's first token) and silu.  q and k
become unit vectors per head, x / sqrt(sum x^2 + unit_eps), and q is multiplied by key_dim^(-1/2).  Per head, with
beta = sigmoid(W_b h) and g = exp(-exp(A_log) * softplus(W_a h + dt_bias)):

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (S: key_dim x value_dim)

so the read-out sees the current token's write.  o is divided by its root mean square per head (``norm_eps``), multiplied
by a weight of size value_dim that the heads share and by silu(W_g h), and goes through the output projection.  The state
(S, float32, and the convolutions' last taps - 1 inputs) lives in the request's state slot.  beta, the decay and the
recurrence are float32 in both precisions: the rows of W_b and W_a are a product of their own whose sums stay float32.
q, k, v and the gate are one packed product, and one convolution runs over q | k | v.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import Mixer, StateNeed, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class GatedDeltaRuleSpec:
    prefix: str
    hidden_size: int
    num_heads: int
    num_kq_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    unit_eps: float = 1e-6
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    kind: ClassVar[str] = "gated_delta_rule"


DEFAULT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("q_conv", "q.conv"), ("k_conv", "k.conv"), ("v_conv", "v.conv"), ("beta", "b"),
                 ("a", "a"), ("a_log", "A_log"), ("dt_bias", "dt_bias"), ("gate", "g"), ("norm", "norm"), ("o", "o"))


class GatedDeltaRule(Mixer):
    def __init__(self, spec: GatedDeltaRuleSpec):
        if min(spec.num_heads, spec.num_kq_heads, spec.key_dim, spec.value_dim, spec.conv_taps) <= 0 or spec.num_heads % spec.num_kq_heads:
            raise ValueError("gated delta rule: sizes must be positive and num_heads a multiple of num_kq_heads")
        if spec.key_dim > 512:
            raise ValueError(f"gated delta rule: key_dim {spec.key_dim} not supported (at most 512)")
        self.spec = spec
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        self.dqk = spec.num_kq_heads * spec.key_dim
        self.inner = spec.num_heads * spec.value_dim
        self.channels = 2 * self.dqk + self.inner               # what the convolution runs over: q | k | v
        self.conv_offset = spec.num_heads * spec.value_dim * spec.key_dim
        self.w_in = self.w_gates = self.w_o = self.conv = self.a_log = self.dt_bias = self.norm = None

    def _name(self, role: str) -> str:
        return self.spec.prefix + self.names[role]

    def weight_decls(self):
        s, H = self.spec, self.spec.num_heads
        return (WeightDecl(self._name("q"), (self.dqk, s.hidden_size)), WeightDecl(self._name("q_conv"), (self.dqk, s.conv_taps), init="around_zero"),
                WeightDecl(self._name("k"), (self.dqk, s.hidden_size)), WeightDecl(self._name("k_conv"), (self.dqk, s.conv_taps), init="around_zero"),
                WeightDecl(self._name("v"), (self.inner, s.hidden_size)), WeightDecl(self._name("v_conv"), (self.inner, s.conv_taps), init="around_zero"),
                WeightDecl(self._name("beta"), (H, s.hidden_size)), WeightDecl(self._name("a_log"), (H,), init="around_zero"),
                WeightDecl(self._name("norm"), (s.value_dim,), init="gain"), WeightDecl(self._name("a"), (H, s.hidden_size)),
                WeightDecl(self._name("dt_bias"), (H,), init="around_zero"), WeightDecl(self._name("gate"), (self.inner, s.hidden_size)),
                WeightDecl(self._name("o"), (s.hidden_size, self.inner)))

    def load(self, tensors, dtype, device):
        def kept(*ts):
            return dtype if dtype == torch.bfloat16 else (torch.float32 if any(t.dtype == torch.float32 for t in ts) else torch.bfloat16)

        main = [tensors[self._name(n)] for n in ("q", "k", "v", "gate")]
        self.w_in = torch.cat([m.to(device=device, dtype=kept(*main)) for m in main], dim=0).contiguous()
        small = [tensors[self._name(n)] for n in ("beta", "a")]
        self.w_gates = torch.cat([m.to(device=device, dtype=kept(*small)) for m in small], dim=0).contiguous()       # [2H, hidden]
        o = tensors[self._name("o")]
        self.w_o = o.to(device=device, dtype=kept(o)).contiguous()
        self.conv = torch.cat([tensors[self._name(n)].to(device=device, dtype=torch.float32) for n in ("q_conv", "k_conv", "v_conv")],
                              dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm = (tensors[self._name(n)].to(device=device, dtype=torch.float32).contiguous()
                                               for n in ("a_log", "dt_bias", "norm"))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_gates, self.w_o))

    def scratch_elements_per_token(self):
        return 2 * (self.channels + self.inner) + 4 * self.inner + 8 * self.spec.num_heads + self.spec.hidden_size

    def state_need(self):
        n = self.conv_offset + self.channels * (self.spec.conv_taps - 1)
        return StateNeed((-(-n // 4) * 4,), torch.float32)

    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T = x.shape[0]
        H, dqk, inner, C = s.num_heads, self.dqk, self.inner, self.channels
        proj = ctx.ws.get("delta_in", (T, C + inner), x.dtype)                     # q | k | v | gate
        ops.gemm(x, self.w_in, proj)
        pre = ctx.ws.get("delta_pre", (T, 2 * H), torch.float32)
        ops.gemm(x, self.w_gates, pre)
        qkv = ctx.ws.get("delta_conv", (T, C), x.dtype)
        ops.causal_conv(proj[:, :C], None, self.conv, None, "silu", state, self.conv_offset, ctx.q_indptr, ctx.row_of_token,
                        ctx.state_slots, qkv)
        beta, decay = (ctx.ws.get(n, (T, H), torch.float32) for n in ("delta_beta", "delta_decay"))
        ops.delta_gates(pre, self.a_log, self.dt_bias, beta, decay)
        o = ctx.ws.get("delta_o", (T, H, s.value_dim), torch.float32)
        ops.delta_scan(qkv[:, :dqk], qkv[:, dqk: 2 * dqk], qkv[:, 2 * dqk:], beta, decay, state, ctx.q_indptr, ctx.state_slots, o,
                       H, s.num_kq_heads, s.key_dim, s.value_dim, float(s.key_dim) ** -0.5, s.unit_eps)
        gated = ctx.ws.get("delta_gated", (T, inner), x.dtype)
        ops.gla_out(o.view(T, inner), proj[:, C:], self.norm, s.norm_eps, 1.0, gated, H, s.value_dim)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


register_part(GatedDeltaRuleSpec.kind, GatedDeltaRule)
