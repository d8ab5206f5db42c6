"""Grouped-query attention over the paged cache, with an optional RMSNorm of q and k
(per head, or over the whole projected row), an optional rotary position encoding, an
optional key window, values that are projected or are the keys as projected, and an
optional sigmoid gate per head on the output.

Order of operations (infer/src/model/qwen3/prefill.rs:652-722): q/k/v projections
without bias -> per-head norm of q and k -> rotation -> k, v into the cache ->
causal attention, query head h reading kv head h // (num_heads / num_kv_heads)
-> output projection.  The three input projections are packed into one matrix at
load, so a step runs one product for them.

Variants, each a field of the spec: ``qk_norm`` "row" norms q (and k) over all heads at once
with a weight of the row's size; ``values`` "keys" has no value projection, the value of a key
is its row of W_k x before norm and rotation (kept in the cache's second stream);
``head_gate`` multiplies head h's output by sigmoid(W_g x)_h before the output projection
(W_g's rows ride in the packed input projection); the position encoding's ``pairing`` chooses
which elements turn together.  ``names`` gives the tensors' names after the prefix.

``qk_norm`` "head_after_rotation" rotates first and norms after (per head; ``qk_norm_weight`` False: x / rms(x) without a
stored weight); ``value_dim`` gives values another width than keys; ``sink`` adds a term exp(sink) without a value to the
softmax's denominator; ``cache_window`` is what the cache keeps when other runs read this run's keys through wider windows
than its own.

The general form (any of ``keep_first``, ``softcap``, ``bias``, ``conv_taps``, or a per-head norm before the rotation with
values of another width): ``keep_first`` keeps the first tokens of a sequence visible after the window has passed them (at
their true positions); ``softcap`` turns a score s into softcap * tanh(s / softcap); ``bias`` adds stored biases in the q, k, v
and output projections (tensor name + ``bias_suffix``); ``conv_taps`` runs a short causal convolution over time on every
channel of q, k and v right after the projection (weights [channels, taps] under tensor name + ``conv_suffix``, zeros
before a sequence's start; the last taps - 1 projected rows of a request are its state).  Its order is projection (+ bias)
-> convolution -> per-head norm -> rotation -> cache -> attention -> output projection (+ bias).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import CacheNeed, Mixer, StateNeed, WeightDecl
from .registry import build_part, register_part


@dataclass(frozen=True)
class AttentionSpec:
    prefix: str                     # e.g. "model.layers.3.self_attn."
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qk_norm_eps: Optional[float]    # None: no per-head norm
    position: Optional[object]      # a position-encoding spec or None
    window: Optional[int] = None    # None: all keys; W: keys p-W+1 .. p
    qk_norm: str = "head"           # "head": per head, weight [head_dim]; "row": over all heads, weight [heads*head_dim]
    values: str = "projected"       # "projected": W_v x; "keys": the keys as projected
    head_gate: bool = False         # head h's output times sigmoid(W_g x)_h
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    qk_norm_weight: bool = True     # False: the per-head norm has no stored weight
    value_dim: Optional[int] = None  # None: head_dim
    sink: Optional[float] = None    # score of a sink without a value in the softmax's denominator
    cache_window: Optional[int] = None   # what the cache keeps (None: ``window``); at least ``window``
    own_keys: bool = True           # False: no key and value projections; every run reads another run's cache
    keep_first: int = 0             # with a window: the first tokens stay visible
    softcap: Optional[float] = None  # scores <- softcap * tanh(scores / softcap)
    bias: bool = False              # biases in the q, k, v and output projections
    conv_taps: int = 0              # a short causal convolution on q, k and v (0: none)
    bias_suffix: str = ".b"
    conv_suffix: str = ".conv"
    kind: ClassVar[str] = "attention"


DEFAULT_NAMES = (("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"), ("o", "o_proj.weight"),
                 ("q_norm", "q_norm.weight"), ("k_norm", "k_norm.weight"), ("gate", "g_proj.weight"))


class Attention(Mixer):
    def __init__(self, spec: AttentionSpec):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim > 256 or spec.head_dim <= 0:
            raise ValueError(f"head_dim {spec.head_dim} not supported (at most 256)")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("window must be positive")
        if spec.qk_norm not in ("head", "row", "head_after_rotation") or spec.values not in ("projected", "keys"):
            raise ValueError(f"attention: qk_norm {spec.qk_norm!r} / values {spec.values!r} not known")
        self.vd = spec.head_dim if spec.value_dim is None else spec.value_dim
        if not 0 < self.vd <= 256:
            raise ValueError(f"attention: value_dim {self.vd} not supported (1 to 256)")
        if spec.cache_window is not None and (spec.window is None or spec.cache_window < spec.window):
            raise ValueError("attention: cache_window goes with a window and is at least as long")
        if spec.keep_first < 0 or spec.conv_taps < 0 or (spec.softcap is not None and not spec.softcap > 0):
            raise ValueError("attention: keep_first and conv_taps cannot be negative, softcap must be positive")
        self.spec = spec
        self.own_keys = spec.own_keys
        self.general_form = bool(spec.keep_first or spec.softcap is not None or spec.bias or spec.conv_taps
                                 or (spec.qk_norm == "head" and (self.vd != spec.head_dim or spec.head_dim % 2)))
        if spec.head_dim % 2 and not self.general_form:
            raise ValueError(f"head_dim {spec.head_dim} not supported by this form of attention (even sizes only)")
        if self.general_form and (spec.qk_norm != "head" or spec.values != "projected" or spec.head_gate or spec.sink is not None
                                  or not spec.own_keys or not spec.qk_norm_weight):
            raise ValueError("attention: kept first tokens, capped scores, biases and the convolution go with a per-head norm before "
                             "the rotation (or none), projected values, keys of its own, no gate and no sink")
        # rotation first and norm after it, values of another width, a sink: the later form, with kernels of its own
        self.post_form = spec.qk_norm == "head_after_rotation"
        if self.post_form and (spec.values != "projected" or spec.head_gate):
            raise ValueError("attention: a norm after the rotation goes with projected values and no gate")
        if not self.post_form and not self.general_form and (self.vd != spec.head_dim or spec.sink is not None or not spec.qk_norm_weight or not spec.own_keys):
            raise ValueError("attention: value_dim, sink, a norm without weight and a run without keys of its own need qk_norm 'head_after_rotation'")
        self.position = build_part(spec.position) if spec.position is not None else None
        self.pairing = getattr(self.position, "pairing", "half")
        # the form the first kernels of this package were written for; everything else takes the general preparation
        if (self.post_form or self.general_form) and self.pairing != "half":
            raise ValueError("attention: a norm after the rotation, and the general form, go with half-split rotation")
        self.plain_form = (spec.qk_norm == "head" and spec.values == "projected" and not spec.head_gate
                           and self.pairing == "half")
        if not self.plain_form and spec.qk_norm == "head" and spec.qk_norm_eps is not None:
            raise ValueError("attention: a per-head q/k norm goes with half-split rotation, projected values and no gate")
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None
        self.gate_at = None             # column of the packed projection where the gate numbers start
        self.b_qkv = self.b_o = self.w_conv = None
        self.channels = spec.num_heads * spec.head_dim + spec.num_kv_heads * (spec.head_dim + self.vd)   # q | k | v

    # ---------------------------------------------------------------- weights
    def _name(self, role: str) -> str:
        return self.spec.prefix + self.names[role]

    def weight_decls(self):
        s = self.spec
        dq, dkv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        if self.general_form:
            rows = {"q": dq, "k": dkv, "v": s.num_kv_heads * self.vd}
            decls = [WeightDecl(self._name(r), (n, s.hidden_size)) for r, n in rows.items()]
            decls.append(WeightDecl(self._name("o"), (s.hidden_size, s.num_heads * self.vd)))
            if s.bias:
                decls += [WeightDecl(self._name(r) + s.bias_suffix, (n,), init="around_zero") for r, n in rows.items()]
                decls.append(WeightDecl(self._name("o") + s.bias_suffix, (s.hidden_size,), init="around_zero"))
            if s.conv_taps:
                decls += [WeightDecl(self._name(r) + s.conv_suffix, (n, s.conv_taps), init="around_zero") for r, n in rows.items()]
            if s.qk_norm_eps is not None:
                decls += [WeightDecl(self._name("q_norm"), (s.head_dim,), init="gain"), WeightDecl(self._name("k_norm"), (s.head_dim,), init="gain")]
            return tuple(decls)
        if self.post_form:
            decls = [WeightDecl(self._name("q"), (dq, s.hidden_size))]
            if self.own_keys:
                decls += [WeightDecl(self._name("k"), (dkv, s.hidden_size)), WeightDecl(self._name("v"), (s.num_kv_heads * self.vd, s.hidden_size))]
            decls.append(WeightDecl(self._name("o"), (s.hidden_size, s.num_heads * self.vd)))
            if s.qk_norm_eps is not None and s.qk_norm_weight:
                decls.append(WeightDecl(self._name("q_norm"), (s.head_dim,), init="gain"))
                if self.own_keys:
                    decls.append(WeightDecl(self._name("k_norm"), (s.head_dim,), init="gain"))
            return tuple(decls)
        decls = [WeightDecl(self._name("q"), (dq, s.hidden_size)), WeightDecl(self._name("k"), (dkv, s.hidden_size))]
        if s.values == "projected":
            decls.append(WeightDecl(self._name("v"), (dkv, s.hidden_size)))
        decls.append(WeightDecl(self._name("o"), (s.hidden_size, dq)))
        if s.qk_norm_eps is not None:
            nq_, nk_ = ((s.head_dim,), (s.head_dim,)) if s.qk_norm == "head" else ((dq,), (dkv,))
            decls += [WeightDecl(self._name("q_norm"), nq_, init="gain"), WeightDecl(self._name("k_norm"), nk_, init="gain")]
        if s.head_gate:
            decls.append(WeightDecl(self._name("gate"), (s.num_heads, s.hidden_size)))
        return tuple(decls)

    def load(self, tensors, dtype, device):
        s = self.spec
        roles = ("q", "k", "v") if s.values == "projected" else ("q", "k")
        if self.post_form and not self.own_keys:
            roles = ("q",)
        mats = [tensors[self._name(n)] for n in roles]
        if s.head_gate:
            self.gate_at = sum(m.shape[0] for m in mats)
            mats.append(tensors[self._name("gate")])
            pad = -sum(m.shape[0] for m in mats) % 8       # rows of the packed output start on 16-byte boundaries
            if pad:
                mats.append(torch.zeros((pad, s.hidden_size), dtype=mats[0].dtype))
        wt = dtype if dtype == torch.bfloat16 else (torch.float32 if any(m.dtype == torch.float32 for m in mats) else torch.bfloat16)
        self.w_qkv = torch.cat([m.to(device=device, dtype=wt) for m in mats], dim=0).contiguous()
        o = tensors[self._name("o")]
        self.w_o = o.to(device=device, dtype=dtype if dtype == torch.bfloat16 else o.dtype).contiguous()
        if s.qk_norm_eps is not None and s.qk_norm_weight:
            self.q_norm = tensors[self._name("q_norm")].to(device=device, dtype=torch.float32).contiguous()
            if self.own_keys:
                self.k_norm = tensors[self._name("k_norm")].to(device=device, dtype=torch.float32).contiguous()
        if self.position is not None:
            self.position.load(tensors, dtype, device)
        if s.bias:
            self.b_qkv = torch.cat([tensors[self._name(r) + s.bias_suffix].to(device=device, dtype=torch.float32) for r in ("q", "k", "v")]).contiguous()
            self.b_o = tensors[self._name("o") + s.bias_suffix].to(device=device, dtype=torch.float32).contiguous()
        if s.conv_taps:
            self.w_conv = torch.cat([tensors[self._name(r) + s.conv_suffix].to(device=device, dtype=torch.float32) for r in ("q", "k", "v")],
                                    dim=0).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def scratch_elements_per_token(self):
        s = self.spec
        return (3 * s.num_heads + 2 * s.num_kv_heads) * max(s.head_dim, self.vd) + s.hidden_size + 8

    # ------------------------------------------------------------------ cache
    def cache_need(self):
        s = self.spec
        window = s.cache_window if s.cache_window is not None else s.window
        keep = s.keep_first if window is not None else 0
        if self.vd != s.head_dim:
            return CacheNeed(streams=((s.num_kv_heads, s.head_dim), (s.num_kv_heads, self.vd)), window=window, keep_first=keep)
        return CacheNeed(s.num_kv_heads, s.head_dim, window, keep_first=keep)

    def state_need(self):
        """The convolution's memory: a request's last taps - 1 projected rows of q | k | v, float32."""
        if self.spec.conv_taps > 1:
            n = self.channels * (self.spec.conv_taps - 1)
            return StateNeed((-(-n // 4) * 4,), torch.float32)
        return None

    def takes_scaled_rows(self, num_rows):
        return not self.post_form and not self.general_form and ops.fused_gemm_shape_ok(num_rows, self.w_qkv)

    def can_sink(self, num_rows):
        return not self.post_form and not self.general_form and ops.fused_gemm_shape_ok(num_rows, self.w_o)

    def _angles(self, qkv, ctx, inv_freq, rdim, general=False):
        """Cosines and sines of the step's positions, evaluated once for all layers that rotate by the same
        frequencies (kept in the step's memo under the encoding's description).  The general preparation takes the
        table for any head size and any number of tokens."""
        if not rdim or not (general or ops.attention_prep_takes_angles(qkv, self.spec.head_dim, rdim)):
            return None
        key = ("rotary_angles", getattr(self.position, "spec", None) or id(self.position))
        angles = ctx.memo.get(key)
        if angles is None:
            angles = ctx.ws.get(f"rotary_angles_{len(ctx.memo)}", (qkv.shape[0], rdim // 2, 2), torch.float32)
            ops.rotary_angles(ctx.positions, inv_freq, angles)
            ctx.memo[key] = angles
        return angles

    # ------------------------------------------------- rotation first, norm after it
    def _forward_post(self, x, ctx, cache):
        s = self.spec
        T = x.shape[0]
        nq, nkv, hd, vd = s.num_heads, s.num_kv_heads, s.head_dim, self.vd
        rot = self.position.rotary() if self.position is not None else None
        inv_freq, rdim = rot if rot is not None else (None, 0)
        if cache.writable != self.own_keys:
            raise RuntimeError("attention: a run without key and value projections must read another run's cache, and only such a run")
        kv = nkv if cache.writable else 0
        proj = ctx.ws.get("qkv", (T, self.w_qkv.shape[0]), x.dtype)
        ops.gemm(x, self.w_qkv, proj)
        ops.attention_prep_post(proj, ctx.positions, cache.slot_mapping if kv else None, self.q_norm, self.k_norm if kv else None,
                                s.qk_norm_eps, inv_freq, rdim, cache.k if kv else None, cache.v if kv else None, nq, kv, hd, vd,
                                cache.page_size)
        attn = ctx.ws.get("attn_out", (T, nq * vd), x.dtype)
        ops.paged_attention(proj[:, : nq * hd], attn, cache.k, cache.v, ctx.positions, ctx.row_of_token, cache.block_table,
                            nq, nkv, hd, cache.page_size, s.scale, s.window, batch=ctx, vd=vd, sink=s.sink)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        ops.gemm(attn, self.w_o, out)
        return out

    # ------------------------------------------------- biases, convolution, kept first tokens, capped scores
    def _forward_general(self, x, ctx, cache, state):
        s = self.spec
        T = x.shape[0]
        nq, nkv, hd, vd = s.num_heads, s.num_kv_heads, s.head_dim, self.vd
        rot = self.position.rotary() if self.position is not None else None
        inv_freq, rdim = rot if rot is not None else (None, 0)
        if not cache.writable:
            raise RuntimeError("attention: this form keeps keys of its own")
        proj = ctx.ws.get("qkv", (T, self.channels), x.dtype)
        ops.gemm(x, self.w_qkv, proj)
        if s.conv_taps:
            # the biases ride into the convolution as its input bias: added to a request's rows, not to the zeros before them
            conv = ctx.ws.get("qkv_conv", (T, self.channels), x.dtype)
            ops.causal_conv(proj, self.b_qkv, self.w_conv, None, "none", state if s.conv_taps > 1 else ctx.ws.get("conv_none", (ctx.cache.max_slots, 4), torch.float32),
                            0, ctx.q_indptr, ctx.row_of_token, ctx.state_slots, conv)
            proj = conv
        elif s.bias:
            ops.bias_add(proj, self.b_qkv)
        if vd == hd and hd % 2 == 0:
            ops.attention_prep(proj, ctx.positions, cache.slot_mapping, self.q_norm, self.k_norm, s.qk_norm_eps or 0.0, inv_freq, rdim,
                               cache.k, cache.v, nq, nkv, hd, cache.page_size, angles=self._angles(proj, ctx, inv_freq, rdim))
        else:
            ops.attention_prep_post(proj, ctx.positions, cache.slot_mapping, self.q_norm, self.k_norm, s.qk_norm_eps, inv_freq, rdim,
                                    cache.k, cache.v, nq, nkv, hd, vd, cache.page_size, norm_first=True)
        attn = ctx.ws.get("attn_out", (T, nq * vd), x.dtype)
        ops.paged_attention(proj[:, : nq * hd], attn, cache.k, cache.v, ctx.positions, ctx.row_of_token, cache.block_table,
                            nq, nkv, hd, cache.page_size, s.scale, s.window, batch=ctx, vd=vd, keep_first=s.keep_first, softcap=s.softcap)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        ops.gemm(attn, self.w_o, out)
        if s.bias:
            ops.bias_add(out, self.b_o)
        return out

    # ------------------------------------------------- the general form, up to the output projection
    def pre_output_width(self):
        return None if self.general_form else self.spec.num_heads * self.vd

    def output_weight(self):
        return self.w_o

    def _attend(self, x, ctx, cache):
        """Projection, preparation, cache store and attention of any form, kernel by kernel.  Returns the
        heads' outputs [T, heads*head_dim] and the packed projection (whose gate columns the caller reads)."""
        s = self.spec
        T = x.shape[0]
        nq, nkv, hd = s.num_heads, s.num_kv_heads, s.head_dim
        rot = self.position.rotary() if self.position is not None else None
        inv_freq, rdim = rot if rot is not None else (None, 0)
        eps = s.qk_norm_eps if s.qk_norm_eps is not None else 0.0
        proj = ctx.ws.get("qkv", (T, self.w_qkv.shape[0]), x.dtype)
        ops.gemm(x, self.w_qkv, proj)
        kv = nkv if cache.writable else 0          # a run that reads another run's cache stores nothing
        if self.plain_form:
            ops.attention_prep(proj, ctx.positions, cache.slot_mapping if kv else None, self.q_norm, self.k_norm if kv else None,
                               eps, inv_freq, rdim, cache.k if kv else None, cache.v if kv else None, nq, kv, hd,
                               cache.page_size, angles=self._angles(proj, ctx, inv_freq, rdim) if kv else None)
        else:
            ops.attention_prep_row(proj, ctx.positions, cache.slot_mapping if kv else None, self.q_norm,
                                   self.k_norm if kv else None, eps, inv_freq, rdim, self.pairing, s.values == "keys",
                                   cache.k if kv else None, cache.v if kv else None, nq, kv, hd, cache.page_size,
                                   angles=self._angles(proj, ctx, inv_freq, rdim, general=True))
        attn = ctx.ws.get("attn_out", (T, nq * hd), x.dtype)
        ops.paged_attention(proj[:, : nq * hd], attn, cache.k, cache.v, ctx.positions, ctx.row_of_token,
                            cache.block_table, nq, nkv, hd, cache.page_size, s.scale, s.window, batch=ctx)
        return attn, proj

    def forward_pre(self, x, ctx, cache, state, into, scale):
        s = self.spec
        attn, proj = self._attend(x, ctx, cache)
        gate = proj[:, self.gate_at: self.gate_at + s.num_heads] if s.head_gate else None
        ops.head_gate(attn, gate, scale, into, s.num_heads, s.head_dim)

    # ---------------------------------------------------------------- forward
    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T = x.shape[0]
        if self.general_form:
            return self._forward_general(x, ctx, cache, state)
        if self.post_form:
            return self._forward_post(x, ctx, cache)
        if not self.plain_form:
            attn, proj = self._attend(x, ctx, cache)
            if s.head_gate:
                gated = ctx.ws.get("attn_gated", tuple(attn.shape), x.dtype)
                ops.head_gate(attn, proj[:, self.gate_at: self.gate_at + s.num_heads], 1.0, gated, s.num_heads, s.head_dim)
                attn = gated
            out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
            return None if ops.gemm(attn, self.w_o, out, sink=sink) else out
        nq, nkv, hd = s.num_heads, s.num_kv_heads, s.head_dim
        rot = self.position.rotary() if self.position is not None else None
        inv_freq, rdim = rot if rot is not None else (None, 0)
        eps = s.qk_norm_eps if s.qk_norm_eps is not None else 0.0
        attn = ctx.ws.get("attn_out", (T, nq * hd), x.dtype)
        if cache.writable:
            qkv = ctx.ws.get("qkv", (T, (nq + 2 * nkv) * hd), x.dtype)
            ops.gemm(x, self.w_qkv, qkv)
            if ops.fused_decode_supported(qkv, ctx, cache.k.dtype, nq, nkv, hd, cache.page_size, rdim):
                # a step of decoded tokens only: norm, rotation, cache store and attention in one launch
                ops.decode_attention_with_prep(qkv, attn, cache.k, cache.v, cache.slot_mapping, self.q_norm, self.k_norm, eps,
                                               inv_freq if rdim else None, cache.block_table, nq, nkv, hd, cache.page_size,
                                               s.scale, s.window, ctx)
                out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
                return None if ops.gemm(attn, self.w_o, out, sink=sink) else out
            ops.attention_prep(qkv, ctx.positions, cache.slot_mapping, self.q_norm, self.k_norm, eps, inv_freq, rdim,
                               cache.k, cache.v, nq, nkv, hd, cache.page_size, angles=self._angles(qkv, ctx, inv_freq, rdim))
        else:
            qkv = ctx.ws.get("q_only", (T, nq * hd), x.dtype)
            ops.gemm(x, self.w_qkv[: nq * hd], qkv)
            ops.attention_prep(qkv, ctx.positions, None, self.q_norm, None, eps, inv_freq, rdim, None, None, nq, 0, hd,
                               cache.page_size, angles=self._angles(qkv, ctx, inv_freq, rdim))
        ops.paged_attention(qkv[:, : nq * hd], attn, cache.k, cache.v, ctx.positions, ctx.row_of_token,
                            cache.block_table, nq, nkv, hd, cache.page_size, s.scale, s.window, batch=ctx)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        if ops.gemm(attn, self.w_o, out, sink=sink):
            return None                       # summed into the residual by the product itself
        return out


register_part(AttentionSpec.kind, Attention)
