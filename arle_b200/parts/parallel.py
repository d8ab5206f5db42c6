"""Parts that stand side by side.

``ParallelMixer``: several mixers read the same input and their outputs are added with fixed
weights, y = sum_i scale_i * mixer_i(x).  When every member can stop before its output
projection (``Mixer.pre_output_width``), each writes scale_i times that projection's input
into its columns of one buffer and ONE product with the members' output matrices side by side
gives y (the mixer then offers the same protocol itself); otherwise every member runs whole and
the outputs are summed by a kernel.  At most one member may keep a paged cache (the model hands a
schedule entry one cache layer); members that keep a state per request share one row per request slot,
each its own columns of it.

``combine="normed"``: y = sum_i scale_i * rmsnorm(mixer_i(x)) * w_i, every member's output normed over the
model width with a stored weight of its own (``norm_names``) before the sum: the members run whole and one
kernel norms and adds them.

``ParallelBlock``: x <- x + (mixer(n) + ff(n)) with n = norm(x): one norm, both branches read its
output; the feed-forward may be absent.  When mixer and feed-forward can both stop before their
last product, the block runs ONE output product over [mixer's columns | feed-forward's columns];
in a decode step of few rows that product adds into the residual itself and leaves the next
block's norm behind (``ops.ResidualSink``), and the next block's first products apply the norm's
factor (``ops.ScaledRows``): no norm kernel and no residual kernel between the blocks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import Block, Mixer, StateNeed, WeightDecl
from .registry import build_part, register_part


def _side_by_side(weights, widths):
    """The matrices [hidden, width_i] side by side, every one starting on a column that is a multiple of 8
    (16 bytes in bfloat16).  Returns (matrix, start columns)."""
    mats, at, col = [], [], 0
    for wo, w in zip(weights, widths):
        at.append(col)
        mats.append(wo)
        pad = -w % 8
        if pad:
            mats.append(torch.zeros((wo.shape[0], pad), dtype=wo.dtype, device=wo.device))
        col += w + pad
    wt = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
    return torch.cat([m.to(wt) for m in mats], dim=1).contiguous(), at


@dataclass(frozen=True)
class ParallelMixerSpec:
    members: Tuple[object, ...]     # mixer specs
    scales: Tuple[float, ...]       # one per member
    hidden_size: int
    combine: str = "sum"            # "sum": y = sum scale_i mixer_i(x); "normed": each output RMS-normed with its weight first
    norm_names: Tuple[str, ...] = ()   # "normed": the members' norm weights, full tensor names
    norm_eps: float = 0.0
    kind: ClassVar[str] = "parallel_mixer"


class ParallelMixer(Mixer):
    def __init__(self, spec: ParallelMixerSpec):
        if not spec.members or len(spec.members) != len(spec.scales):
            raise ValueError("a parallel mixer needs members and one scale for each")
        self.spec = spec
        self.members = [build_part(m) for m in spec.members]
        self.with_cache = [i for i, m in enumerate(self.members) if m.cache_need() is not None]
        self.with_state = [i for i, m in enumerate(self.members) if m.state_need() is not None]
        if len(self.with_cache) > 1:
            raise ValueError("a parallel mixer takes at most one member with a paged cache")
        if spec.combine not in ("sum", "normed") or (spec.combine == "normed" and len(spec.norm_names) != len(spec.members)):
            raise ValueError("a parallel mixer combines by 'sum' or 'normed', the latter with one norm weight's name per member")
        if spec.combine == "normed" and len(spec.members) > 4:
            raise ValueError("a parallel mixer norms and adds at most four members")
        # members with a state: each gets its columns of one float32 row per request slot
        self.state_at = {}
        at = 0
        for i in self.with_state:
            need = self.members[i].state_need()
            if len(self.with_state) > 1 and (need.dtype != torch.float32 or len(need.shape) != 1):
                raise ValueError("members of a parallel mixer that share a state row need flat float32 states")
            n = int(need.shape[0]) if len(need.shape) == 1 else 0
            self.state_at[i] = (at, n)
            at += -(-n // 4) * 4
        self.state_width = at
        self.norm_weights = None
        widths = [m.pre_output_width() for m in self.members]
        self.shared_output = spec.combine == "sum" and all(w is not None for w in widths)
        self.widths = widths if self.shared_output else None
        self.w_o = None
        self.at = None
        self.padded = False

    def weight_decls(self):
        own = tuple(WeightDecl(n, (self.spec.hidden_size,), init="gain") for n in self.spec.norm_names) if self.spec.combine == "normed" else ()
        return tuple(d for m in self.members for d in m.weight_decls()) + own

    def load(self, tensors, dtype, device):
        for m in self.members:
            m.load(tensors, dtype, device)
        if self.spec.combine == "normed":
            self.norm_weights = [tensors[n].to(device=device, dtype=torch.float32).contiguous() for n in self.spec.norm_names]
        if self.shared_output:
            self.w_o, self.at = _side_by_side([m.output_weight() for m in self.members], self.widths)
            self.padded = any(-w % 8 for w in self.widths)

    def weight_bytes(self):
        return sum(m.weight_bytes() for m in self.members)

    def scratch_elements_per_token(self):
        return sum(m.scratch_elements_per_token() for m in self.members) + (self.w_o.shape[1] if self.w_o is not None else 0)

    def cache_need(self):
        return self.members[self.with_cache[0]].cache_need() if self.with_cache else None

    def state_need(self):
        if not self.with_state:
            return None
        if len(self.with_state) == 1:
            return self.members[self.with_state[0]].state_need()
        return StateNeed((self.state_width,), torch.float32)

    def takes_scaled_rows(self, num_rows):
        return self.shared_output and all(m.takes_scaled_rows(num_rows) for m in self.members)

    def can_sink(self, num_rows):
        return self.shared_output and ops.fused_gemm_shape_ok(num_rows, self.w_o)

    def _args(self, i, cache, state):
        st = None
        if i in self.with_state:
            at, n = self.state_at[i]
            st = state if len(self.with_state) == 1 else state[:, at: at + n]
        return (cache if i in self.with_cache else None, st)

    # the mixer up to its one output product
    def pre_output_width(self):
        return self.w_o.shape[1] if self.shared_output and self.w_o is not None else (
            sum(w + -w % 8 for w in self.widths) if self.shared_output else None)

    def output_weight(self):
        return self.w_o

    def forward_pre(self, x, ctx, cache, state, into, scale):
        if self.padded:
            into.zero_()
        for i, (m, w) in enumerate(zip(self.members, self.widths)):
            c, st = self._args(i, cache, state)
            m.forward_pre(x, ctx, c, st, into[:, self.at[i]: self.at[i] + w], scale * self.spec.scales[i])

    def forward(self, x, ctx, cache, state, sink=None):
        T = x.shape[0]
        H = self.spec.hidden_size
        if self.shared_output:
            cat = ctx.ws.get("parallel_pre", (T, self.w_o.shape[1]), x.dtype)
            self.forward_pre(x, ctx, cache, state, cat, 1.0)
            out = ctx.ws.get("mixer_out", (T, H), x.dtype)
            return None if ops.gemm(cat, self.w_o, out, sink=sink) else out
        if self.spec.combine == "normed":
            outs = []
            for i, m in enumerate(self.members):
                c, st = self._args(i, cache, state)
                y = m.forward(x, ctx, c, st)
                if any(y.data_ptr() == o.data_ptr() for o in outs):
                    raise RuntimeError("parallel mixer: two members returned the same buffer; their outputs must live side by side")
                outs.append(y)
            out = ctx.ws.get("parallel_out", (T, H), x.dtype)
            ops.normed_sum(outs, None, self.norm_weights, self.spec.scales, self.spec.norm_eps, out)
            return out
        total = None
        for i, m in enumerate(self.members):
            c, st = self._args(i, cache, state)
            y = m.forward(x, ctx, c, st)
            acc = ctx.ws.get(f"parallel_sum_{i & 1}", (T, H), x.dtype)
            if total is None:
                ops.weighted_sum(y, self.spec.scales[i], y, 0.0, acc)
            else:
                ops.weighted_sum(total, 1.0, y, self.spec.scales[i], acc)
            total = acc
        return total


@dataclass(frozen=True)
class ParallelBlockSpec:
    norm: object
    mixer: object
    ffn: Optional[object]           # None: the block has no feed-forward
    kind: ClassVar[str] = "parallel_block"


class ParallelBlock(Block):
    def __init__(self, spec: ParallelBlockSpec):
        self.spec = spec
        self.norm = build_part(spec.norm)
        self.mixer = build_part(spec.mixer)
        self.ffn = build_part(spec.ffn) if spec.ffn is not None else None
        self._parts = tuple(p for p in (self.norm, self.mixer, self.ffn) if p is not None)
        self.one_product = self.mixer.pre_output_width() is not None and (self.ffn is None or self.ffn.pre_output_width() is not None)
        self.w_out = None
        self.at = None
        self.padded = False

    def weight_decls(self):
        return tuple(d for p in self._parts for d in p.weight_decls())

    def load(self, tensors, dtype, device):
        for p in self._parts:
            p.load(tensors, dtype, device)
        if self.one_product:
            branches = [self.mixer] + ([self.ffn] if self.ffn is not None else [])
            widths = [b.pre_output_width() for b in branches]
            self.w_out, self.at = _side_by_side([b.output_weight() for b in branches], widths)
            self.widths = widths
            self.padded = any(-w % 8 for w in widths)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self._parts)

    def scratch_elements_per_token(self):
        return sum(p.scratch_elements_per_token() for p in self._parts) + (self.w_out.shape[1] if self.w_out is not None else 0)

    def entry(self):
        return self.norm, self

    def takes_scaled_rows(self, num_rows):
        """Asked by the block before this one: can every first product of this block apply the norm's factor itself?"""
        return (self.one_product and self.mixer.takes_scaled_rows(num_rows)
                and (self.ffn is None or self.ffn.takes_scaled_rows(num_rows)))

    def forward(self, stream, ctx, cache, state):
        n = stream.normed(self.norm, "normed_a")
        if not self.one_product:
            stream.add(self.mixer.forward(n, ctx, cache, state))
            if self.ffn is not None:
                stream.add(self.ffn.forward(n, ctx))
            return
        T = ctx.num_tokens
        pre = ctx.ws.get("block_pre", (T, self.w_out.shape[1]), n.dtype)
        if self.padded:
            pre.zero_()
        self.mixer.forward_pre(n, ctx, cache, state, pre[:, : self.widths[0]], 1.0)
        if self.ffn is not None:
            self.ffn.forward_pre(n, ctx, pre[:, self.at[1]: self.at[1] + self.widths[1]])
        nxt = stream.next_entry
        sink = None
        if nxt is not None and ops.fused_gemm_shape_ok(T, self.w_out):
            # every reader of this block's normed rows has run by now: their buffer can take the next block's
            sink = stream.sink_for(nxt[0], nxt[1], "normed_a")
        out = ctx.ws.get("block_out", (T, stream.resid.shape[1]), n.dtype)
        stream.add(None if ops.gemm(pre, self.w_out, out, sink=sink) else out)


register_part(ParallelMixerSpec.kind, ParallelMixer)
register_part(ParallelBlockSpec.kind, ParallelBlock)
