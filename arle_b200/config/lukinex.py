"""Typed configuration of the Lukinex architecture, read from ``config.json``.

A Lukinex model is a list of layers (``layers``) that norm every sublayer's input AND its output:
x <- x + norm1b(mixer(norm1(x))), then x <- x + norm2b(ff(norm2(x))), all four RMS norms with a weight.  A layer's ``type``
names its mixer:

* ``attention``: grouped-query attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``) without biases; q and k are
  RMS-normed per head with a weight shared by the heads, then the first ``rot.dims`` numbers of a head are rotated
  (half-split pairs, ``rot.base``, every frequency divided by ``rot.scaling.factor``); a sliding window ``mask.size`` that
  keeps the first ``mask.keep_first`` tokens visible at their true positions;
* ``latent_attention``: attention without positions whose cache holds one normed latent of ``kv_rank`` numbers per token;
  queries go through a normed latent of ``q_rank`` numbers; keys (``dim`` per head) and values (``vdim`` per head) are rebuilt
  per head from the cached latent; every earlier token is visible.  With ``kv_from: j`` the layer has no down-projection and
  reads layer j's latents with its own key and value maps;
* ``parallel``: two mixers side by side on the same input, each output RMS-normed over the model width with a weight of its
  own, the result half their sum.  ``left``: an attention with biases in all four projections, a short causal convolution
  (``conv`` taps) on q, k and v right after the projection, rotation, scores capped by ``softcap * tanh(score / softcap)``, the
  same window with kept first tokens.  ``right``: linear attention with one constant ``decay`` per head, silu on q, k and v,
  an RMS norm over all heads at once and a sigmoid gate.

``mlp`` is null or ``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}, "shared": {"ff", "limit"}}``: the
``top`` experts with the largest router sums, weighted by the softmax over those sums alone; experts with clamped inputs,
down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate x, limit), u = clamp(up x, +-limit); a shared expert of the same form
(``shared``, optional) runs for every token and is added.  Around the layers: ``vocab``, ``width``, ``norm.eps``; the model's norm
``final.norm`` and the output projection ``head``.  Optional keys this engine adds: ``max_position`` (default 1,048,576: the
design has no position limit), ``bos_token_id``, ``eos_token_id``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional, Tuple

from .kolodra import _get, _pos_int
from .lasupel import _under
from .model_spec import ModelSpec, ScheduleEntry
from .qwen3 import ConfigError

MIXER_TYPES = ("attention", "latent_attention", "parallel")
EXPERT_ALPHA = 1.702        # an expert's gate is g * sigmoid(EXPERT_ALPHA * g)
PARALLEL_SHARE = 0.5        # the parallel mixer's result is this times the sum of its two normed outputs


@dataclass(frozen=True)
class LukinexMlp:
    ff: int                         # an expert's size
    limit: float
    experts: int
    top: int
    shared_ff: int = 0              # 0: no shared expert
    shared_limit: float = 0.0


@dataclass(frozen=True)
class LukinexLayer:
    type: str
    mixer: Tuple[Tuple[str, object], ...]     # the mixer's sizes and constants (for "parallel": left.* and right.*)
    mlp: Optional[LukinexMlp]

    def m(self, key: str):
        return dict(self.mixer)[key]


def _attention_keys(m: dict, w: str, prefix: str = "", left: bool = False) -> dict:
    def fail(msg):
        raise ConfigError(f"config.json: {w}: {msg}")

    out = {k: _under(w, _pos_int, m, k) for k in ("heads", "kv_heads", "dim", "vdim")}
    if out["heads"] % out["kv_heads"]:
        fail(f"'heads' ({out['heads']}) must be a multiple of 'kv_heads' ({out['kv_heads']})")
    if out["dim"] > 256 or out["vdim"] > 256:
        fail(f"'dim' = {out['dim']} and 'vdim' = {out['vdim']} may be at most 256")
    out["scale"] = float(_under(w, _get, m, "scale"))
    mask = m.get("mask")
    out["window"] = _under(w, _pos_int, m, "mask.size") if mask is not None else None
    keep = mask.get("keep_first", 0) if mask is not None else 0
    if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
        fail(f"'mask.keep_first' = {keep!r} must be a count of tokens")
    out["keep_first"] = keep
    rot = m.get("rot")
    out["rot_dims"] = _under(w, _get, m, "rot.dims", int) if rot is not None else 0
    out["rot_base"] = float(_under(w, _get, m, "rot.base")) if out["rot_dims"] else 1.0
    out["rot_divide"] = float(_under(w, _get, m, "rot.scaling.factor")) if rot is not None and rot.get("scaling") is not None else 1.0
    if out["rot_dims"] < 0 or out["rot_dims"] % 2 or out["rot_dims"] > out["dim"]:
        fail(f"'rot.dims' = {out['rot_dims']} must be even and at most dim ({out['dim']})")
    if out["rot_dims"] and not (out["rot_base"] > 0 and out["rot_divide"] > 0):
        fail("'rot.base' and 'rot.scaling.factor' must be positive")
    cap = m.get("softcap")
    if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or not float(cap) > 0):
        fail(f"'softcap' = {cap!r} must be positive")
    out["softcap"] = float(cap) if cap is not None else None
    if left:
        conv = m.get("conv", 0)
        if isinstance(conv, bool) or not isinstance(conv, int) or conv < 0:
            fail(f"'conv' = {conv!r} must be a number of taps")
        out["conv"] = conv
    return {prefix + k: v for k, v in out.items()}


def _mixer(kind: str, m: dict, w: str) -> Tuple[Tuple[str, object], ...]:
    w = w + ".mixer"

    def fail(msg):
        raise ConfigError(f"config.json: {w}: {msg}")

    if kind == "attention":
        out = _attention_keys(m, w)
    elif kind == "latent_attention":
        out = {k: _under(w, _pos_int, m, k) for k in ("heads", "dim", "vdim", "kv_rank", "q_rank")}
        if out["kv_rank"] > 512:
            fail(f"'kv_rank' = {out['kv_rank']} (at most 512)")
        out["scale"] = float(_under(w, _get, m, "scale"))
        src = m.get("kv_from")
        if src is not None and (isinstance(src, bool) or not isinstance(src, int)):
            fail(f"'kv_from' = {src!r} must be a layer's number")
        out["kv_from"] = src
    else:
        for side in ("left", "right"):
            if not isinstance(m.get(side), dict):
                fail(f"'{side}' must be an object")
        out = _attention_keys(m["left"], w + ".left", "left.", left=True)
        r, wr = m["right"], w + ".right"
        out.update({"right." + k: _under(wr, _pos_int, r, k) for k in ("heads", "dim", "vdim")})
        decay = r.get("decay")
        if (not isinstance(decay, list) or len(decay) != out["right.heads"]
                or not all(isinstance(d, (int, float)) and not isinstance(d, bool) and 0.0 <= d < float("inf") for d in decay)):
            raise ConfigError(f"config.json: {wr}.decay must list one number (not negative) for each of the {out['right.heads']} heads")
        out["right.decay"] = tuple(float(d) for d in decay)
    return tuple(sorted(out.items(), key=lambda kv: kv[0]))


def _mlp(mlp, w: str) -> Optional[LukinexMlp]:
    if mlp is None:
        return None
    w = w + ".mlp"
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {w}.kind = {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} (moe or null)")
    experts, top = _under(w, _pos_int, mlp, "router.experts"), _under(w, _pos_int, mlp, "router.top")
    if top > experts:
        raise ConfigError(f"config.json: {w}.router: {top} experts cannot be chosen among {experts}")
    limit = float(_under(w, _get, mlp, "expert.limit"))
    shared = mlp.get("shared")
    s_ff, s_limit = (_under(w, _pos_int, mlp, "shared.ff"), float(_under(w, _get, mlp, "shared.limit"))) if shared is not None else (0, 0.0)
    if not limit > 0 or (shared is not None and not s_limit > 0):
        raise ConfigError(f"config.json: '{w}.expert.limit' and '{w}.shared.limit' must be positive")
    return LukinexMlp(_under(w, _pos_int, mlp, "expert.ff"), limit, experts, top, s_ff, s_limit)


@dataclass(frozen=True)
class LukinexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[LukinexLayer, ...]
    max_position: int = 1 << 20
    bos_token_id: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()

    architecture = "Lukinex"

    @classmethod
    def from_dict(cls, d: dict) -> "LukinexConfig":
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
            layers.append(LukinexLayer(e["type"], _mixer(e["type"], e["mixer"], w), _mlp(e.get("mlp"), w)))
        for i, l in enumerate(layers):
            if l.type != "latent_attention" or l.m("kv_from") is None:
                continue
            j = l.m("kv_from")
            if not 0 <= j < i or layers[j].type != "latent_attention" or layers[j].m("kv_from") is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {j} names no earlier latent-attention layer with latents of its own")
            if l.m("kv_rank") != layers[j].m("kv_rank"):
                raise ConfigError(f"config.json: layers[{i}] reads layer {j}'s latents but their kv_rank differ")
        eps = float(_get(d, "norm.eps"))
        if not eps > 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        eos = d.get("eos_token_id")
        stops = (eos,) if isinstance(eos, int) and not isinstance(eos, bool) else tuple(int(x) for x in eos) if isinstance(eos, list) else ()
        return cls(vocab=_pos_int(d, "vocab"), width=_pos_int(d, "width"), norm_eps=eps, layers=tuple(layers),
                   max_position=_pos_int(d, "max_position") if "max_position" in d else 1 << 20,
                   bos_token_id=d.get("bos_token_id") if isinstance(d.get("bos_token_id"), int) else None, stop_token_ids=stops)

    @classmethod
    def from_dir(cls, model_dir: str) -> "LukinexConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    # ------------------------------------------------------------------- spec
    def _attention_spec(self, l: LukinexLayer, p: str, side: str = ""):
        from ..parts.attention import AttentionSpec
        from ..parts.rotary import RotarySpec

        def m(key):
            return l.m(side + key)

        left = bool(side)
        return AttentionSpec(
            prefix=p, hidden_size=self.width, num_heads=m("heads"), num_kv_heads=m("kv_heads"), head_dim=m("dim"), scale=m("scale"),
            qk_norm_eps=None if left else self.norm_eps,
            position=RotarySpec(rotary_dim=m("rot_dims"), theta=m("rot_base"), pairing="half", divide_by=m("rot_divide")) if m("rot_dims") else None,
            window=m("window"), qk_norm="head", names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"), ("k_norm", "k.norm")),
            value_dim=m("vdim"), keep_first=m("keep_first") if m("window") is not None else 0, softcap=m("softcap"),
            bias=left, conv_taps=m("conv") if left else 0)

    def _mixer_spec(self, l: LukinexLayer, p: str):
        from ..parts.latent_attention import LatentAttentionSpec
        from ..parts.lightning import ConstantDecayAttentionSpec
        from ..parts.parallel import ParallelMixerSpec

        if l.type == "attention":
            return self._attention_spec(l, p)
        if l.type == "latent_attention":
            return LatentAttentionSpec(prefix=p, hidden_size=self.width, num_heads=l.m("heads"), nope_dim=l.m("dim"), rope_dim=0,
                                       value_dim=l.m("vdim"), kv_rank=l.m("kv_rank"), scale=l.m("scale"), norm_eps=self.norm_eps,
                                       position=None, window=None, q_rank=l.m("q_rank"), own_latent=l.m("kv_from") is None)
        right = ConstantDecayAttentionSpec(prefix=p + "right.", hidden_size=self.width, num_heads=l.m("right.heads"), key_dim=l.m("right.dim"),
                                           value_dim=l.m("right.vdim"), decay=l.m("right.decay"), norm_eps=self.norm_eps, activation="silu")
        return ParallelMixerSpec(members=(self._attention_spec(l, p + "left.", "left."), right), scales=(PARALLEL_SHARE, PARALLEL_SHARE),
                                 hidden_size=self.width, combine="normed", norm_names=(p + "left.out", p + "right.out"),
                                 norm_eps=self.norm_eps)

    def _mlp_spec(self, mlp: LukinexMlp, p: str):
        from ..parts.mlp import GatedMlpSpec
        from ..parts.moe import RoutedExpertsSpec

        shared = GatedMlpSpec(prefix=p + "shared.", hidden_size=self.width, intermediate_size=mlp.shared_ff, activation="clamped_glu",
                              names=("gate", "up", "down"), act_limit=mlp.shared_limit, act_alpha=EXPERT_ALPHA) if mlp.shared_ff else None
        return RoutedExpertsSpec(prefix=p, hidden_size=self.width, num_experts=mlp.experts, top=mlp.top, expert_ff=mlp.ff, groups=1, keep=1,
                                 route_scale=1.0, correction=False, shared=shared, shared_gate=False, activation="clamped_glu",
                                 scores="softmax_chosen", act_limit=mlp.limit, act_alpha=EXPERT_ALPHA)

    def to_model_spec(self) -> ModelSpec:
        from ..parts.block import SandwichBlockSpec
        from ..parts.norm import RmsNormSpec

        blocks, schedule, ignored = [], [], []
        for i, l in enumerate(self.layers):
            p = f"l{i}."

            def norm(name):
                return RmsNormSpec(p + name, self.width, self.norm_eps)

            if l.mlp is None:               # a layer without a feed-forward has no use for its norms, should they be stored
                ignored += [p + "norm2", p + "norm2b"]
            blocks.append(SandwichBlockSpec(
                mixer_norm=norm("norm1"), mixer=self._mixer_spec(l, p + "mix."), mixer_post_norm=norm("norm1b"),
                ffn_norm=norm("norm2") if l.mlp is not None else None, ffn=self._mlp_spec(l.mlp, p + "mlp.") if l.mlp is not None else None,
                ffn_post_norm=norm("norm2b") if l.mlp is not None else None))
            schedule.append(ScheduleEntry(i, keys_of=l.m("kv_from") if l.type == "latent_attention" else None))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=tuple(schedule), final_norm=RmsNormSpec("final.norm", self.width, self.norm_eps), embed_name="embed",
            head_name="head", max_position=self.max_position, stop_token_ids=self.stop_token_ids, bos_token_id=self.bos_token_id,
            ignored_tensors=tuple(ignored))
