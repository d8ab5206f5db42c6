"""Pre-norm block: x <- x + mixer(norm(x)); x <- x + ffn(norm(x)) (the second half is absent when the spec names no
feed-forward)
(infer/src/model/qwen3/prefill.rs:618-776).  The block never touches the residual
itself: it hands branch outputs to the ``ResidualStream``, which folds each into
the 32-bit residual inside the kernel of the next norm, the fusion cklxx/arle's
decode path uses (infer/src/model/qwen3/batch_decode.rs:2422-2452)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

from .base import Block
from .registry import build_part, register_part


@dataclass(frozen=True)
class PreNormBlockSpec:
    mixer_norm: object
    mixer: object
    ffn_norm: object = None         # None together with ffn: the block is its mixer half alone
    ffn: object = None
    kind: ClassVar[str] = "prenorm_block"


class PreNormBlock(Block):
    def __init__(self, spec: PreNormBlockSpec):
        self.spec = spec
        self.mixer_norm = build_part(spec.mixer_norm)
        self.mixer = build_part(spec.mixer)
        if (spec.ffn is None) != (spec.ffn_norm is None):
            raise ValueError("a pre-norm block has a feed-forward and its norm, or neither")
        self.ffn_norm = build_part(spec.ffn_norm) if spec.ffn_norm is not None else None
        self.ffn = build_part(spec.ffn) if spec.ffn is not None else None
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def weight_decls(self):
        return tuple(d for p in self._parts for d in p.weight_decls())

    def load(self, tensors, dtype, device):
        for p in self._parts:
            p.load(tensors, dtype, device)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self._parts)

    def scratch_elements_per_token(self):
        # the two normalised inputs and the larger of the two branches' buffers
        if self.ffn is None:
            return self.mixer_norm.scratch_elements_per_token() + self.mixer.scratch_elements_per_token()
        return (self.mixer_norm.scratch_elements_per_token() + self.ffn_norm.scratch_elements_per_token()
                + max(self.mixer.scratch_elements_per_token(), self.ffn.scratch_elements_per_token()))

    def entry(self):
        return self.mixer_norm, self.mixer

    def forward(self, stream, ctx, cache, state):
        T = ctx.num_tokens
        h = stream.normed(self.mixer_norm, "normed_a")
        if self.ffn is None:
            nxt = stream.next_entry
            sink = stream.sink_for(nxt[0], nxt[1], "normed_a") if nxt is not None and self.mixer.can_sink(T) else None
            stream.add(self.mixer.forward(h, ctx, cache, state, sink=sink) if sink is not None else self.mixer.forward(h, ctx, cache, state))
            return
        # where a branch's last product can add into the residual and leave the next norm's input behind,
        # and that norm's reader can apply the norm's factor itself, the norm between them is no kernel
        sink = stream.sink_for(self.ffn_norm, self.ffn, "normed_b") if self.mixer.can_sink(T) else None
        if sink is not None:
            stream.add(self.mixer.forward(h, ctx, cache, state, sink=sink))
        else:
            stream.add(self.mixer.forward(h, ctx, cache, state))
        h = stream.normed(self.ffn_norm, "normed_b")
        nxt = stream.next_entry
        sink = stream.sink_for(nxt[0], nxt[1], "normed_a") if nxt is not None and self.ffn.can_sink(T) else None
        if sink is not None:
            stream.add(self.ffn.forward(h, ctx, sink=sink))
        else:
            stream.add(self.ffn.forward(h, ctx))


register_part(PreNormBlockSpec.kind, PreNormBlock)


@dataclass(frozen=True)
class OutputNormBlockSpec:
    """x <- x + norm(mixer(x)); x <- x + norm(ffn(x)): the norms stand on the sublayers' outputs, the sublayers read the
    residual as it is (the second half is absent when the spec names no feed-forward)."""
    mixer_norm: object
    mixer: object
    ffn_norm: object = None
    ffn: object = None
    kind: ClassVar[str] = "outnorm_block"


class OutputNormBlock(Block):
    """The norm needs ``add_normed(resid, branch, copy)`` (``RmsNorm`` has it): the branch's norm, the sum into the 32-bit
    residual and the rounded copy that the next sublayer reads are one kernel."""

    def __init__(self, spec: OutputNormBlockSpec):
        self.spec = spec
        self.mixer_norm = build_part(spec.mixer_norm)
        self.mixer = build_part(spec.mixer)
        if (spec.ffn is None) != (spec.ffn_norm is None):
            raise ValueError("a block has a feed-forward and its norm, or neither")
        self.ffn_norm = build_part(spec.ffn_norm) if spec.ffn_norm is not None else None
        self.ffn = build_part(spec.ffn) if spec.ffn is not None else None
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError(f"norm {type(n).__name__} cannot stand on a branch's output (no add_normed)")

    def weight_decls(self):
        return tuple(d for p in self._parts for d in p.weight_decls())

    def load(self, tensors, dtype, device):
        for p in self._parts:
            p.load(tensors, dtype, device)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self._parts)

    def scratch_elements_per_token(self):
        width = self.mixer_norm.scratch_elements_per_token()
        return 2 * width + max(self.mixer.scratch_elements_per_token(), self.ffn.scratch_elements_per_token() if self.ffn is not None else 0)

    def forward(self, stream, ctx, cache, state):
        h = stream.plain("plain_a")
        stream.add_normed(self.mixer_norm, self.mixer.forward(h, ctx, cache, state), "plain_b")
        if self.ffn is not None:
            h = stream.plain("plain_b")
            stream.add_normed(self.ffn_norm, self.ffn.forward(h, ctx), "plain_a")


register_part(OutputNormBlockSpec.kind, OutputNormBlock)


@dataclass(frozen=True)
class SandwichBlockSpec:
    """x <- x + post(mixer(pre(x))); x <- x + post'(ffn(pre'(x))): a norm on every sublayer's input AND on its output (the
    second half is absent when the spec names no feed-forward)."""
    mixer_norm: object
    mixer: object
    mixer_post_norm: object
    ffn_norm: object = None
    ffn: object = None
    ffn_post_norm: object = None
    kind: ClassVar[str] = "sandwich_block"


class SandwichBlock(Block):
    """A sublayer's output norm, the sum into the 32-bit residual and the next sublayer's input norm are one kernel
    (``ResidualStream.add_normed_before_norm``): the stream keeps the branch until the next ``normed(...)``."""

    def __init__(self, spec: SandwichBlockSpec):
        self.spec = spec
        given = [spec.ffn is not None, spec.ffn_norm is not None, spec.ffn_post_norm is not None]
        if any(given) != all(given):
            raise ValueError("a block has a feed-forward with both of its norms, or none of the three")
        self.mixer_norm = build_part(spec.mixer_norm)
        self.mixer = build_part(spec.mixer)
        self.mixer_post_norm = build_part(spec.mixer_post_norm)
        self.ffn_norm = build_part(spec.ffn_norm) if spec.ffn is not None else None
        self.ffn = build_part(spec.ffn) if spec.ffn is not None else None
        self.ffn_post_norm = build_part(spec.ffn_post_norm) if spec.ffn is not None else None
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.ffn_norm, self.ffn, self.ffn_post_norm)
                            if p is not None)
        for n in (self.mixer_post_norm, self.ffn_post_norm):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError(f"norm {type(n).__name__} cannot stand on a branch's output (no add_normed)")

    def weight_decls(self):
        return tuple(d for p in self._parts for d in p.weight_decls())

    def load(self, tensors, dtype, device):
        for p in self._parts:
            p.load(tensors, dtype, device)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self._parts)

    def scratch_elements_per_token(self):
        width = self.mixer_norm.scratch_elements_per_token()
        return 2 * width + max(self.mixer.scratch_elements_per_token(), self.ffn.scratch_elements_per_token() if self.ffn is not None else 0)

    def forward(self, stream, ctx, cache, state):
        h = stream.normed(self.mixer_norm, "normed_a")
        stream.add_normed_before_norm(self.mixer_post_norm, self.mixer.forward(h, ctx, cache, state))
        if self.ffn is not None:
            h = stream.normed(self.ffn_norm, "normed_b")
            stream.add_normed_before_norm(self.ffn_post_norm, self.ffn.forward(h, ctx))


register_part(SandwichBlockSpec.kind, SandwichBlock)
