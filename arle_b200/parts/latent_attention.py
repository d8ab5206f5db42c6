"""Attention whose cache holds one latent vector per token instead of keys and values per head.

    q = W_q x                       per head [dn unrotated | dr rotated]
    W_dkv x = [c_raw | k_rot_raw]   rank + dr numbers; c = rmsnorm(c_raw) * weight, k_rot = rotate(k_rot_raw)
    head h:  k_h = [W_uk[h] c | k_rot],  v_h = W_uv[h] c
    score = (q_nope . W_uk[h] c + rotate(q_rot) . k_rot) * scale;  softmax over the visible keys;  out = W_o [heads' sums]

Only c and k_rot are cached: one record of rank + dr numbers per token, one stream of one head in the paged
cache.  The keys and values are never built.  Since q_nope . (W_uk[h] c) = (W_uk[h]^T q_nope) . c, the heads' key
maps are folded into the queries (one small product per head), every head then attends over the same records with
keys [c | k_rot] and values c, and W_uv[h] is applied to the head's weighted sum of latents afterwards.  The
position encoding is the rotary part's (pairing "half"); it turns the first ``rotary_dim`` of the dr numbers.
A ``window`` keeps the last ``window`` positions visible (itself included) and lets older pages go back.

``q_rank``: the queries go through a latent of their own, c_q = rmsnorm(W_dq x) * weight, q = W_uq c_q (tensors ``dq``,
``dq.norm``, ``uq`` instead of ``q``).  ``own_latent`` False: the layer has no W_dkv and no latent norm; it reads the
records another layer stored (the schedule names that layer) with its own key and value maps, queries and window.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import CacheNeed, Mixer, WeightDecl
from .registry import build_part, register_part


@dataclass(frozen=True)
class LatentAttentionSpec:
    prefix: str
    hidden_size: int
    num_heads: int
    nope_dim: int                   # unrotated query/key numbers per head
    rope_dim: int                   # rotated query/key numbers per head (the key's are shared by the heads)
    value_dim: int                  # per head
    kv_rank: int                    # size of the latent
    scale: float
    norm_eps: float                 # of the latent's RMSNorm
    position: Optional[object]      # a rotary spec (its rotary_dim <= rope_dim) or None
    window: Optional[int] = None
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    q_rank: Optional[int] = None    # size of the queries' latent (None: q = W_q x)
    own_latent: bool = True         # False: no down-projection of its own; every run reads another run's records
    kind: ClassVar[str] = "latent_attention"


DEFAULT_NAMES = (("q", "q"), ("dkv", "dkv"), ("latent_norm", "dkv.norm"), ("uk", "uk"), ("uv", "uv"), ("o", "o"), ("dq", "dq"),
                 ("q_latent_norm", "dq.norm"), ("uq", "uq"))


class LatentAttention(Mixer):
    def __init__(self, spec: LatentAttentionSpec):
        if min(spec.num_heads, spec.value_dim, spec.kv_rank) <= 0 or spec.nope_dim < 0 or spec.rope_dim < 0 or spec.nope_dim + spec.rope_dim <= 0:
            raise ValueError("latent attention: heads, value_dim and kv_rank must be positive, nope_dim + rope_dim too")
        if spec.kv_rank > 512:
            raise ValueError(f"latent attention: kv_rank {spec.kv_rank} not supported (at most 512)")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("window must be positive")
        self.spec = spec
        self.position = build_part(spec.position) if spec.position is not None else None
        if self.position is not None and (getattr(self.position, "pairing", "half") != "half"
                                          or self.position.spec.rotary_dim > spec.rope_dim):
            raise ValueError("latent attention: the rotation pairs element i with i + dims/2 and turns at most rope_dim numbers")
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        if spec.q_rank is not None and spec.q_rank <= 0:
            raise ValueError("latent attention: q_rank must be positive")
        self.q_width = spec.num_heads * (spec.nope_dim + spec.rope_dim)
        self.record = spec.kv_rank + spec.rope_dim
        self.first = spec.q_rank if spec.q_rank is not None else self.q_width      # rows of the first product that belong to the queries
        self.rows = -(-(self.first + (self.record if spec.own_latent else 0)) // 8) * 8
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.latent_norm = self.w_uq = self.q_latent_norm = None

    def _name(self, role: str) -> str:
        return self.spec.prefix + self.names[role]

    # ---------------------------------------------------------------- weights
    def weight_decls(self):
        s = self.spec
        if s.q_rank is not None:
            decls = [WeightDecl(self._name("dq"), (s.q_rank, s.hidden_size)), WeightDecl(self._name("q_latent_norm"), (s.q_rank,), init="gain"),
                     WeightDecl(self._name("uq"), (self.q_width, s.q_rank))]
        else:
            decls = [WeightDecl(self._name("q"), (self.q_width, s.hidden_size))]
        if s.own_latent:
            decls += [WeightDecl(self._name("dkv"), (self.record, s.hidden_size)), WeightDecl(self._name("latent_norm"), (s.kv_rank,), init="gain")]
        return tuple(decls) + (WeightDecl(self._name("uk"), (s.num_heads * s.nope_dim, s.kv_rank)),
                               WeightDecl(self._name("uv"), (s.num_heads * s.value_dim, s.kv_rank)),
                               WeightDecl(self._name("o"), (s.hidden_size, s.num_heads * s.value_dim)))

    def load(self, tensors, dtype, device):
        s = self.spec
        mats = [tensors[self._name("dq" if s.q_rank is not None else "q")]] + ([tensors[self._name("dkv")]] if s.own_latent else [])
        pad = self.rows - sum(m.shape[0] for m in mats)
        if pad:
            mats.append(torch.zeros((pad, s.hidden_size), dtype=mats[0].dtype))

        def kept(ts):
            return dtype if dtype == torch.bfloat16 else (torch.float32 if any(t.dtype == torch.float32 for t in ts) else torch.bfloat16)

        self.w_in = torch.cat([m.to(device=device, dtype=kept(mats)) for m in mats], dim=0).contiguous()
        uk, uv, o = (tensors[self._name(n)] for n in ("uk", "uv", "o"))
        # head h's key map transposed: [rank, nope_dim], the matrix that folds it into the head's query
        self.w_uk_t = uk.to(device=device, dtype=kept([uk])).view(s.num_heads, s.nope_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = uv.to(device=device, dtype=kept([uv])).view(s.num_heads, s.value_dim, s.kv_rank).contiguous()
        self.w_o = o.to(device=device, dtype=kept([o])).contiguous()
        if s.own_latent:
            self.latent_norm = tensors[self._name("latent_norm")].to(device=device, dtype=torch.float32).contiguous()
        if s.q_rank is not None:
            uq = tensors[self._name("uq")]
            self.w_uq = uq.to(device=device, dtype=kept([uq])).contiguous()
            self.q_latent_norm = tensors[self._name("q_latent_norm")].to(device=device, dtype=torch.float32).contiguous()
        if self.position is not None:
            self.position.load(tensors, dtype, device)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_uk_t, self.w_uv, self.w_o, self.w_uq) if t is not None)

    def scratch_elements_per_token(self):
        s = self.spec
        return self.rows + s.num_heads * (self.record + s.kv_rank + s.value_dim) + s.hidden_size + (self.first + self.q_width if s.q_rank else 0)

    # ------------------------------------------------------------------ cache
    def cache_need(self):
        return CacheNeed(window=self.spec.window, streams=((1, self.record),))

    def can_sink(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_o)

    # ---------------------------------------------------------------- forward
    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T = x.shape[0]
        H, dn, dr, rank = s.num_heads, s.nope_dim, s.rope_dim, s.kv_rank
        rot = self.position.rotary() if self.position is not None else None
        inv_freq, rdim = rot if rot is not None else (None, 0)
        if cache.writable and not s.own_latent:
            raise RuntimeError("latent attention: a layer without a down-projection must read another run's records")
        proj = ctx.ws.get("latent_in", (T, self.rows), x.dtype)
        ops.gemm(x, self.w_in, proj)
        if s.q_rank is not None:
            cq = ctx.ws.get("latent_cq", (T, s.q_rank), x.dtype)
            ops.rms_rows(proj[:, : s.q_rank], self.q_latent_norm, s.norm_eps, cq)
            q = ctx.ws.get("latent_q_up", (T, self.q_width), x.dtype)
            ops.gemm(cq, self.w_uq, q)
        else:
            q = proj[:, : self.q_width]
        q_abs = ctx.ws.get("latent_q", (T, H, self.record), x.dtype)
        records = cache.streams[0]
        stores = cache.writable and s.own_latent
        if stores or dr:
            ops.latent_prep(q, proj[:, self.first: self.first + self.record] if s.own_latent else None, ctx.positions, cache.slot_mapping,
                            self.latent_norm, s.norm_eps, inv_freq, rdim, records if stores else None, q_abs, H, dn, dr, rank)
        if dn:
            ops.gemm_heads(q.unflatten(1, (H, dn + dr))[:, :, :dn], self.w_uk_t, q_abs[:, :, :rank])
        else:
            q_abs[:, :, :rank].zero_()
        o_lat = ctx.ws.get("latent_o", (T, H, rank), x.dtype)
        ops.latent_attention(q_abs, o_lat, records, ctx.positions, ctx.row_of_token, cache.block_table, rank, cache.page_size,
                             s.scale, s.window, batch=ctx)
        heads_out = ctx.ws.get("attn_out", (T, H, s.value_dim), x.dtype)
        ops.gemm_heads(o_lat, self.w_uv, heads_out)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        return None if ops.gemm(heads_out.view(T, H * s.value_dim), self.w_o, out, sink=sink) else out


register_part(LatentAttentionSpec.kind, LatentAttention)
