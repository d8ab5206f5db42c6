"""Typed configuration of the Lasupel architecture, read from ``config.json``.

A Lasupel model is a list of layers (``layers``) whose norms stand on the sublayers' OUTPUTS: x <- x + norm1(mixer(x)), then
x <- x + norm2(ff(x)); the sublayers read x as it is.  The norms are RMS norms with a weight.  A layer's ``type`` names its
mixer:

* ``attention``: grouped-query attention with a sliding window (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
  ``mask.size``, ``rot.base``, ``rot.dims``): rotation of the first ``rot.dims`` numbers of a head, then q and k brought to
  unit root mean square per head without a weight, a softmax with one more term (a sink of score 0 without a value) in
  its denominator.  With ``kv_from: j`` the layer has no key and value projections and reads layer j's cache;
* ``rglru``: the recurrent block with a real-gated linear recurrent unit (``width``, ``blocks``, ``conv``);
* ``delta``: the gated delta rule (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``).

``mlp`` is null, ``{"kind": "dense", "ff"}`` (silu-gated) or ``{"kind": "moe", "expert": {"ff", "limit"}, "router":
{"experts", "top", "groups": {"count", "keep"}}}``: softmax scores over all experts, a group scored by its best expert, the
scores of the chosen as weights, experts with clamped inputs.  Around the layers: ``vocab``, ``width``, ``embedding.scale``,
``norm.eps``; the model's norm ``final.norm`` and the output projection ``head``.  Optional keys this engine adds:
``max_position`` (default 1,048,576: the design has no position limit), ``bos_token_id``, ``eos_token_id``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional, Tuple

from .kolodra import _get, _pos_int
from .model_spec import ModelSpec, ScheduleEntry
from .qwen3 import ConfigError

MIXER_TYPES = ("attention", "rglru", "delta")
SINK_SCORE = 0.0            # the score of the softmax's extra term
LRU_DECAY = 8.0             # log a = -LRU_DECAY * r * softplus(lam)
EXPERT_ALPHA = 1.702        # an expert's gate is g * sigmoid(EXPERT_ALPHA * g)
UNIT_EPS = 1e-6             # under the root when the delta rule's q and k are brought to unit length


@dataclass(frozen=True)
class LasupelMlp:
    kind: str                       # "dense" or "moe"
    ff: int                         # dense: its size; moe: an expert's
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    limit: float = 0.0


@dataclass(frozen=True)
class LasupelLayer:
    type: str
    mixer: Tuple[Tuple[str, object], ...]     # the mixer's sizes and constants, by the names in the module's docstring
    mlp: Optional[LasupelMlp]

    def m(self, key: str):
        return dict(self.mixer)[key]


def _under(where: str, fn, d: dict, path: str, *a):
    try:
        return fn(d, path, *a)
    except ConfigError as e:
        raise ConfigError(str(e).replace("'", f"'{where}.", 1)) from None


def _mixer(kind: str, m: dict, w: str) -> Tuple[Tuple[str, object], ...]:
    w = w + ".mixer"

    def fail(msg):
        raise ConfigError(f"config.json: {w}: {msg}")

    def pos(path):
        return _under(w, _pos_int, m, path)

    def num(path):
        return float(_under(w, _get, m, path))

    if kind == "attention":
        out = {k: pos(k) for k in ("heads", "kv_heads", "dim", "vdim")}
        if out["heads"] % out["kv_heads"]:
            fail(f"'heads' ({out['heads']}) must be a multiple of 'kv_heads' ({out['kv_heads']})")
        out["scale"] = num("scale")
        out["window"] = pos("mask.size") if m.get("mask") is not None else None
        rot = m.get("rot")
        out["rot_dims"] = _under(w, _get, m, "rot.dims", int) if rot is not None else 0
        out["rot_base"] = num("rot.base") if out["rot_dims"] else 1.0
        if out["rot_dims"] < 0 or out["rot_dims"] % 2 or out["rot_dims"] > out["dim"]:
            fail(f"'rot.dims' = {out['rot_dims']} must be even and at most dim ({out['dim']})")
        if out["rot_dims"] and not out["rot_base"] > 0:
            fail("'rot.base' must be positive")
        src = m.get("kv_from")
        if src is not None and (isinstance(src, bool) or not isinstance(src, int)):
            fail(f"'kv_from' = {src!r} must be a layer's number")
        out["kv_from"] = src
    elif kind == "rglru":
        out = {"width": pos("width"), "blocks": pos("blocks"), "conv": pos("conv")}
        if out["width"] % out["blocks"]:
            fail(f"'width' ({out['width']}) must be a multiple of 'blocks' ({out['blocks']})")
    else:
        out = {k: pos(k) for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
        if out["heads"] % out["kv_heads"]:
            fail(f"'heads' ({out['heads']}) must be a multiple of 'kv_heads' ({out['kv_heads']})")
    return tuple(sorted(out.items(), key=lambda kv: kv[0]))


def _mlp(mlp, w: str) -> Optional[LasupelMlp]:
    if mlp is None:
        return None
    w = w + ".mlp"
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {w}.kind = {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} (dense, moe or null)")
    if mlp["kind"] == "dense":
        return LasupelMlp("dense", _under(w, _pos_int, mlp, "ff"))
    experts, top = _under(w, _pos_int, mlp, "router.experts"), _under(w, _pos_int, mlp, "router.top")
    groups = mlp["router"].get("groups")
    count, keep = (_under(w, _pos_int, mlp, "router.groups.count"), _under(w, _pos_int, mlp, "router.groups.keep")) if groups is not None else (1, 1)
    if experts % count or keep > count or top > keep * (experts // count):
        raise ConfigError(f"config.json: {w}.router: {experts} experts do not split into {count} groups of which {keep} are kept "
                          f"and hold the {top} chosen")
    limit = float(_under(w, _get, mlp, "expert.limit"))
    if not limit > 0:
        raise ConfigError(f"config.json: '{w}.expert.limit' must be positive")
    return LasupelMlp("moe", _under(w, _pos_int, mlp, "expert.ff"), experts, top, count, keep, limit)


@dataclass(frozen=True)
class LasupelConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[LasupelLayer, ...]
    max_position: int = 1 << 20
    bos_token_id: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()

    architecture = "Lasupel"

    @classmethod
    def from_dict(cls, d: dict) -> "LasupelConfig":
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {w} must be an object")
            if e.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: {w}.type = {e.get('type')!r} (this design has {', '.join(MIXER_TYPES)})")
            if not isinstance(e.get("mixer"), dict):
                raise ConfigError(f"config.json: {w}.mixer must be an object")
            layers.append(LasupelLayer(e["type"], _mixer(e["type"], e["mixer"], w), _mlp(e.get("mlp"), w)))
        for i, l in enumerate(layers):
            if l.type != "attention" or l.m("kv_from") is None:
                continue
            j = l.m("kv_from")
            if not 0 <= j < i or layers[j].type != "attention" or layers[j].m("kv_from") is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {j} names no earlier attention layer with keys of its own")
            same = ("kv_heads", "heads", "dim", "vdim", "rot_dims", "rot_base")
            if any(l.m(k) != layers[j].m(k) for k in same):
                raise ConfigError(f"config.json: layers[{i}] reads layer {j}'s keys and values but its head counts, sizes or rotation differ")
        eps = float(_get(d, "norm.eps"))
        if not eps > 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        eos = d.get("eos_token_id")
        stops = (eos,) if isinstance(eos, int) and not isinstance(eos, bool) else tuple(int(x) for x in eos) if isinstance(eos, list) else ()
        return cls(vocab=_pos_int(d, "vocab"), width=_pos_int(d, "width"),
                   embedding_scale=float(_get(d, "embedding.scale")) if "embedding" in d else 1.0, norm_eps=eps, layers=tuple(layers),
                   max_position=_pos_int(d, "max_position") if "max_position" in d else 1 << 20,
                   bos_token_id=d.get("bos_token_id") if isinstance(d.get("bos_token_id"), int) else None, stop_token_ids=stops)

    @classmethod
    def from_dir(cls, model_dir: str) -> "LasupelConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    # ------------------------------------------------------------------- spec
    def _kept_window(self, i: int) -> Optional[int]:
        """What layer i's cache must keep: the longest window among the layer and the layers that read its keys
        (None when one of them sees everything)."""
        windows = [self.layers[i].m("window")] + [l.m("window") for l in self.layers if l.type == "attention" and l.m("kv_from") == i]
        return None if any(w is None for w in windows) else max(windows)

    def _mixer_spec(self, i: int, l: LasupelLayer, p: str):
        from ..parts.attention import AttentionSpec
        from ..parts.delta_rule import GatedDeltaRuleSpec
        from ..parts.rglru import RgLruSpec
        from ..parts.rotary import RotarySpec

        if l.type == "attention":
            own = l.m("kv_from") is None
            kept = self._kept_window(i if own else l.m("kv_from"))
            return AttentionSpec(
                prefix=p, hidden_size=self.width, num_heads=l.m("heads"), num_kv_heads=l.m("kv_heads"), head_dim=l.m("dim"),
                scale=l.m("scale"), qk_norm_eps=self.norm_eps,
                position=RotarySpec(rotary_dim=l.m("rot_dims"), theta=l.m("rot_base"), pairing="half") if l.m("rot_dims") else None,
                window=l.m("window"), qk_norm="head_after_rotation", names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")),
                qk_norm_weight=False, value_dim=l.m("vdim"), sink=SINK_SCORE,
                cache_window=kept if l.m("window") is not None and kept != l.m("window") else None, own_keys=own)
        if l.type == "rglru":
            return RgLruSpec(prefix=p, hidden_size=self.width, width=l.m("width"), blocks=l.m("blocks"), conv_taps=l.m("conv"),
                             decay_constant=LRU_DECAY)
        return GatedDeltaRuleSpec(prefix=p, hidden_size=self.width, num_heads=l.m("heads"), num_kq_heads=l.m("kv_heads"),
                                  key_dim=l.m("dim"), value_dim=l.m("vdim"), conv_taps=l.m("conv"), norm_eps=self.norm_eps,
                                  unit_eps=UNIT_EPS)

    def _mlp_spec(self, mlp: LasupelMlp, p: str):
        from ..parts.mlp import GatedMlpSpec
        from ..parts.moe import RoutedExpertsSpec

        if mlp.kind == "dense":
            return GatedMlpSpec(prefix=p, hidden_size=self.width, intermediate_size=mlp.ff, activation="silu", names=("gate", "up", "down"))
        return RoutedExpertsSpec(prefix=p, hidden_size=self.width, num_experts=mlp.experts, top=mlp.top, expert_ff=mlp.ff,
                                 groups=mlp.groups, keep=mlp.keep, route_scale=1.0, correction=False, shared=None, shared_gate=False,
                                 activation="clamped_glu", scores="softmax", group_score="max", act_limit=mlp.limit,
                                 act_alpha=EXPERT_ALPHA)

    def to_model_spec(self) -> ModelSpec:
        from ..parts.block import OutputNormBlockSpec
        from ..parts.norm import RmsNormSpec

        blocks, schedule, ignored = [], [], []
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            if l.mlp is None:               # a layer without a feed-forward has no use for a second norm, should one be stored
                ignored.append(p + "norm2")
            blocks.append(OutputNormBlockSpec(
                mixer_norm=RmsNormSpec(p + "norm1", self.width, self.norm_eps), mixer=self._mixer_spec(i, l, p + "mix."),
                ffn_norm=RmsNormSpec(p + "norm2", self.width, self.norm_eps) if l.mlp is not None else None,
                ffn=self._mlp_spec(l.mlp, p + "mlp.") if l.mlp is not None else None))
            schedule.append(ScheduleEntry(i, keys_of=l.m("kv_from") if l.type == "attention" else None))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=tuple(schedule), final_norm=RmsNormSpec("final.norm", self.width, self.norm_eps), embed_name="embed",
            head_name="head", max_position=self.max_position, stop_token_ids=self.stop_token_ids, bos_token_id=self.bos_token_id,
            ignored_tensors=tuple(ignored), embed_scale=self.embedding_scale)
