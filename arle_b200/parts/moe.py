"""A feed-forward of routed experts.

Every token runs ``top`` of ``num_experts`` small gated feed-forwards (down(act(gate x) * up x), no biases) and adds their
outputs with weights.  Router: z = W_router x in float32; scores s = sigmoid(z); the choice goes by s + correction (a stored
vector), the weights are s * route_scale of the chosen, not renormalised.  The experts stand in ``groups`` equal groups of
neighbours; a group's score is the sum of its two largest choice scores and only experts of the ``keep`` best groups can be
chosen.  An optional shared expert (a gated feed-forward of its own size) runs for every token and is added, times
sigmoid(w_sg . x), one number per token, when it has such a gate.

Variants, each a field of the spec: ``scores`` "softmax" takes the scores as a softmax over all experts; "softmax_chosen"
chooses the experts with the largest router sums and weights them by the softmax over the chosen sums alone; ``group_score``
"max" scores a group by its largest choice score alone; ``activation`` "clamped_glu" makes an expert
down(g * sigmoid(act_alpha * g) * (u + 1)) with g = min(gate x, act_limit) and u = up x clamped to +-act_limit.

The step's (token, choice) pairs are sorted by expert on the device and the experts' products run as grouped tiles over
the sorted places, so nothing depends on the host knowing how many tokens an expert got (a decode step stays capturable).
The shared gate's row rides in the router's product.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import FeedForward, WeightDecl
from .registry import build_part, register_part


@dataclass(frozen=True)
class RoutedExpertsSpec:
    prefix: str
    hidden_size: int
    num_experts: int
    top: int
    expert_ff: int
    groups: int = 1
    keep: int = 1
    route_scale: float = 1.0
    correction: bool = True          # a stored vector added to the scores for the choice only
    shared: Optional[object] = None  # a feed-forward spec that runs for every token
    shared_gate: bool = False        # the shared expert's output times sigmoid(w . x)
    activation: str = "silu"
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    scores: str = "sigmoid"          # or "softmax" (over all experts), or "softmax_chosen" (the largest sums win, softmax over them alone)
    group_score: str = "top2_sum"    # or "max"
    act_limit: Optional[float] = None    # of the "clamped_glu" activation
    act_alpha: float = 1.702
    kind: ClassVar[str] = "routed_experts"


DEFAULT_NAMES = (("router", "router"), ("correction", "correction"), ("expert", "e{}."), ("gate", "gate"), ("up", "up"),
                 ("down", "down"), ("shared_gate", "shared.sg"))


class RoutedExperts(FeedForward):
    def __init__(self, spec: RoutedExpertsSpec):
        E, per = spec.num_experts, spec.num_experts // max(spec.groups, 1)
        if min(E, spec.top, spec.expert_ff, spec.groups, spec.keep) <= 0 or E % spec.groups or spec.keep > spec.groups:
            raise ValueError("routed experts: experts must split into the groups, of which at most all are kept")
        if spec.top > spec.keep * per or E > 1024:
            raise ValueError("routed experts: more experts chosen than the kept groups hold, or more than 1,024 experts")
        if spec.activation not in ops.ACTIVATIONS and spec.activation != "clamped_glu":
            raise ValueError(f"routed experts: activation {spec.activation!r}")
        if spec.activation == "clamped_glu" and not (spec.act_limit is not None and spec.act_limit > 0):
            raise ValueError("routed experts: the clamped activation needs a positive act_limit")
        if spec.scores not in ("sigmoid", "softmax", "softmax_chosen") or spec.group_score not in ("top2_sum", "max"):
            raise ValueError(f"routed experts: scores {spec.scores!r} / group_score {spec.group_score!r} not known")
        if spec.shared_gate and spec.shared is None:
            raise ValueError("routed experts: a shared gate needs a shared expert")
        self.spec = spec
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        self.shared = build_part(spec.shared) if spec.shared is not None else None
        self.w_router = self.correction = self.w_gate_up = self.w_down = None

    def _name(self, role: str, expert: int = None) -> str:
        if expert is None:
            return self.spec.prefix + self.names[role]
        return self.spec.prefix + self.names["expert"].format(expert) + self.names[role]

    def weight_decls(self):
        s = self.spec
        decls = [WeightDecl(self._name("router"), (s.num_experts, s.hidden_size))]
        if s.correction:
            decls.append(WeightDecl(self._name("correction"), (s.num_experts,), init="around_zero"))
        for e in range(s.num_experts):
            decls += [WeightDecl(self._name("gate", e), (s.expert_ff, s.hidden_size)), WeightDecl(self._name("up", e), (s.expert_ff, s.hidden_size)),
                      WeightDecl(self._name("down", e), (s.hidden_size, s.expert_ff))]
        if self.shared is not None:
            decls += list(self.shared.weight_decls())
        if s.shared_gate:
            decls.append(WeightDecl(self._name("shared_gate"), (1, s.hidden_size)))
        return tuple(decls)

    def load(self, tensors, dtype, device):
        s = self.spec

        def kept(ts):
            return dtype if dtype == torch.bfloat16 else (torch.float32 if any(t.dtype == torch.float32 for t in ts) else torch.bfloat16)

        rows = [tensors[self._name("router")]] + ([tensors[self._name("shared_gate")]] if s.shared_gate else [])
        self.w_router = torch.cat([r.to(device=device, dtype=kept(rows)) for r in rows], dim=0).contiguous()
        if s.correction:
            self.correction = tensors[self._name("correction")].to(device=device, dtype=torch.float32).contiguous()
        gu, dn = [], []
        for e in range(s.num_experts):
            g, u, d = (tensors[self._name(n, e)] for n in ("gate", "up", "down"))
            gu.append(torch.stack([g, u], dim=1).reshape(2 * s.expert_ff, s.hidden_size))      # rows 2i, 2i + 1: gate_i, up_i
            dn.append(d)
        self.w_gate_up = torch.stack(gu).to(device=device, dtype=kept(gu)).contiguous()
        self.w_down = torch.stack(dn).to(device=device, dtype=kept(dn)).contiguous()
        if self.shared is not None:
            self.shared.load(tensors, dtype, device)

    def weight_bytes(self):
        """What a step of many tokens reads: every expert."""
        n = sum(t.numel() * t.element_size() for t in (self.w_router, self.w_gate_up, self.w_down))
        return n + (self.shared.weight_bytes() if self.shared is not None else 0)

    def scratch_elements_per_token(self):
        s = self.spec
        return s.top * (3 * s.expert_ff + s.hidden_size) + 2 * s.hidden_size + 4 * (s.num_experts + s.groups + 1) + (
            self.shared.scratch_elements_per_token() if self.shared is not None else 0)

    def forward(self, x, ctx, sink=None):
        s = self.spec
        T = x.shape[0]
        E, top, ff = s.num_experts, s.top, s.expert_ff
        pairs = T * top
        z = ctx.ws.get("moe_z", (T, self.w_router.shape[0]), torch.float32)
        ops.gemm(x, self.w_router, z)
        ids = ctx.ws.get("moe_ids", (T, top), torch.int32)
        weights = ctx.ws.get("moe_weights", (T, top), torch.float32)
        ops.moe_select(z, self.correction, ctx.ws.get("moe_scratch", (T, E + s.groups), torch.float32), E, top, s.groups, s.keep,
                       s.route_scale, ids, weights, scores=s.scores, group_score=s.group_score)
        plan = ctx.ws.get("moe_plan", (ops.moe_plan_size(E, pairs),), torch.int32)
        place_of_pair = ctx.ws.get("moe_place", (pairs,), torch.int32)
        row_of_place = ctx.ws.get("moe_row", (pairs,), torch.int32)
        ops.moe_plan(ids, E, plan, place_of_pair, row_of_place)
        gu = ctx.ws.get("moe_gate_up", (pairs, 2 * ff), x.dtype)
        ops.moe_gemm(x, row_of_place, self.w_gate_up, gu, plan, E)
        act = ctx.ws.get("moe_act", (pairs, ff), x.dtype)
        if s.activation == "clamped_glu":
            ops.clamped_glu(gu, act, s.act_limit, s.act_alpha)
        else:
            ops.act_mul(gu, act, s.activation)
        y = ctx.ws.get("moe_y", (pairs, s.hidden_size), x.dtype)
        ops.moe_gemm(act, None, self.w_down, y, plan, E)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        out = ctx.ws.get("moe_out", (T, s.hidden_size), x.dtype)
        ops.moe_combine(y, place_of_pair, weights, shared, z[:, E] if s.shared_gate else None, out)
        return out


register_part(RoutedExpertsSpec.kind, RoutedExperts)
