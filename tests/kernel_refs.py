"""Plain torch statements of each CUDA kernel of the package, one function per
kernel with the kernel's own signature (see ``arle_b200/ops/__init__.py``).

Two uses: the GPU tests compare every kernel alone against its function here, at
sizes other than the engine's; and the CPU tests put these functions in the place
of the kernels (fixture ``cpu_kernels`` in conftest.py) so that everything around
the kernels (cache manager, block tables, step function, scheduler) runs and is
compared with the plain model without a GPU.  They are test code only: the
package itself has no CPU path.
"""
from __future__ import annotations

import math

import torch

F32 = torch.float32


def embedding(ids, table, out, err=None, last_token=None, slot_of_token=None, scale=1.0):
    ids = ids.long()
    if last_token is not None:
        ids = torch.where(ids < 0, last_token[slot_of_token.long()].long(), ids)
    out.copy_(table[ids].to(F32) * scale)


def rmsnorm(resid, delta, rows, weight, eps, out, write_resid):
    idx = rows.long() if rows is not None else torch.arange(resid.shape[0], device=resid.device)
    x = resid[idx].to(F32)
    if delta is not None:
        x = x + delta[idx].to(F32)
    if write_resid:
        resid[idx] = x
    inv = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    out.copy_((x * inv * weight).to(out.dtype))


def residual_add(resid, delta):
    resid += delta.to(F32)


def gemm(x, w, out, sink=None):
    """``sink`` is never taken here (the parts are told so by ``fused_gemm_shape_ok``): False."""
    out.copy_((x.to(F32) @ w.to(F32).t()).to(out.dtype))
    return False


def fused_gemm_shape_ok(rows, w, gated=False):
    return False


def fused_decode_supported(*args, **kwargs):
    return False


def attention_prep_takes_angles(*args, **kwargs):
    return False


def attention_prep(qkv, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim, k_cache, v_cache,
                   nq, nkv, hd, page_size, angles=None):
    T = qkv.shape[0]
    heads = qkv[:, : (nq + 2 * nkv) * hd].view(T, nq + 2 * nkv, hd)

    def norm_rope(x, w):
        x = x.to(F32)
        if w is not None:
            x = x * (1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)) * w
        if rotary_dim:
            half = rotary_dim // 2
            ang = positions.to(F32)[:, None] * inv_freq[None, :]
            cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            lo, hi = x[..., :half], x[..., half:rotary_dim]
            x = torch.cat([lo * cos - hi * sin, lo * sin + hi * cos, x[..., rotary_dim:]], dim=-1)
        return x

    q = norm_rope(heads[:, :nq], q_weight)
    heads[:, :nq] = q.to(qkv.dtype)
    if nkv:
        k = norm_rope(heads[:, nq:nq + nkv], k_weight).to(qkv.dtype)
        v = heads[:, nq + nkv:]
        keep = slot_mapping >= 0
        page = (slot_mapping[keep] // page_size).long()
        off = (slot_mapping[keep] % page_size).long()
        k_cache[page, :, off] = k[keep]
        v_cache[page, :, off] = v[keep]


def paged_attention(q, out, k_cache, v_cache, positions, row_of_token, block_table, nq, nkv, hd, page_size, scale,
                    window, batch=None, vd=None, sink=None, keep_first=0, softcap=None):
    T = q.shape[0]
    g = nq // nkv
    vd = hd if vd is None else vd
    for t in range(T):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        js = torch.cat([torch.arange(0, min(int(keep_first or 0), lo)), torch.arange(lo, p + 1)])
        pages = block_table[int(row_of_token[t]), js // page_size].long()
        offs = js % page_size
        k = k_cache[pages, :, offs].to(F32)          # [n, nkv, hd]
        v = v_cache[pages, :, offs].to(F32)
        qt = q[t].view(nq, hd).to(F32)
        for h in range(nq):
            s = (k[:, h // g] @ qt[h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if sink is None:
                pr = torch.softmax(s, dim=0)
            else:                                            # one more term in the denominator, without a value
                pr = torch.softmax(torch.cat([s, torch.tensor([float(sink)])]), dim=0)[:-1]
            out[t, h * vd:(h + 1) * vd] = (pr @ v[:, h // g]).to(out.dtype)


def silu_mul(gate_up, out):
    g, u = gate_up[:, 0::2].to(F32), gate_up[:, 1::2].to(F32)          # rows 2i, 2i + 1 of the packed weight: gate_i, up_i
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def gemm_silu_mul(x, w, gate_up, out):
    gemm(x, w, gate_up)
    silu_mul(gate_up, out)


def argmax(logits, scratch, out, scatter=None, last_token=None):
    out[: logits.shape[0]] = torch.argmax(logits, dim=1).to(out.dtype)      # torch returns the first maximal index
    if scatter is not None:
        last_token[scatter[: logits.shape[0]].long()] = out[: logits.shape[0]]


def scatter_tokens(tokens, scatter, last_token):
    last_token[scatter.long()] = tokens[: scatter.numel()]


def sample(logits, temperature, top_k, top_p, min_p, uniform, scratch, out):
    R, V = logits.shape
    for r in range(R):
        x = logits[r].to(F32)
        t = float(temperature[r]) if temperature is not None else 0.0
        k = int(top_k[r]) if top_k is not None else -1
        if not t > 0 or k == 1:
            out[r] = int(torch.argmax(x))          # torch returns the first maximal index
            continue
        p = torch.softmax(x / t, dim=0)
        mp = float(min_p[r])
        if mp > 0:
            p = torch.where(p >= mp * p.max(), p, torch.zeros_like(p))
            p = p / p.sum()
        if 0 < k < V:
            kth = torch.sort(p, descending=True).values[k - 1]
            p = torch.where(p >= kth, p, torch.zeros_like(p))
            p = p / p.sum()
        tp = float(top_p[r])
        if tp < 1:
            sp = torch.sort(p, descending=True).values
            n = int((torch.cumsum(sp, 0) < tp).sum()) + 1
            thr = sp[min(n, V) - 1]
            p = torch.where(p >= thr, p, torch.zeros_like(p))
            p = p / p.sum()
        c = torch.cumsum(p, 0)
        target = float(uniform[r]) * float(c[-1])
        hit = torch.nonzero(c > target)
        out[r] = int(hit[0]) if hit.numel() else int(torch.nonzero(p > 0)[-1])


ACTS = {"silu": lambda g: g / (1.0 + torch.exp(-g)),
        "gelu_tanh": lambda g: 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))}


def act_mul(gate_up, out, activation):
    g, u = gate_up[:, 0::2].to(F32), gate_up[:, 1::2].to(F32)
    out.copy_((ACTS[activation](g) * u).to(out.dtype))


def gemm_act_mul(x, w, gate_up, out, activation="silu"):
    gemm(x, w, gate_up)
    act_mul(gate_up, out, activation)


def attention_prep_row(qk, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim, pairing, values_are_keys,
                       k_cache, v_cache, nq, nkv, hd, page_size, angles=None):
    T = qk.shape[0]

    def norm_rope(x, w, heads):
        x = x.to(F32)
        if w is not None:
            x = x * (1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)) * w
        x = x.view(T, heads, hd).clone()
        if rotary_dim:
            ang = positions.to(F32)[:, None] * inv_freq[None, :]
            cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            if pairing == "half":
                a, b = x[..., : rotary_dim // 2].clone(), x[..., rotary_dim // 2: rotary_dim].clone()
                x[..., : rotary_dim // 2], x[..., rotary_dim // 2: rotary_dim] = a * cos - b * sin, b * cos + a * sin
            else:
                a, b = x[..., 0:rotary_dim:2].clone(), x[..., 1:rotary_dim:2].clone()
                x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2] = a * cos - b * sin, b * cos + a * sin
        return x

    raw_k = qk[:, nq * hd:(nq + nkv) * hd].clone().view(T, nkv, hd) if nkv else None
    q = norm_rope(qk[:, : nq * hd], q_weight, nq)
    if nkv:
        k = norm_rope(qk[:, nq * hd:(nq + nkv) * hd], k_weight, nkv).to(qk.dtype)
        v = raw_k if values_are_keys else qk[:, (nq + nkv) * hd:(nq + 2 * nkv) * hd].view(T, nkv, hd)
        keep = slot_mapping >= 0
        page = (slot_mapping[keep] // page_size).long()
        off = (slot_mapping[keep] % page_size).long()
        k_cache[page, :, off] = k[keep]
        v_cache[page, :, off] = v[keep]
    qk[:, : nq * hd] = q.reshape(T, nq * hd).to(qk.dtype)


def head_gate(x, gate, scale, out, heads, hd):
    T = x.shape[0]
    y = x.to(F32).view(T, heads, hd)
    if gate is not None:
        y = y * (1.0 / (1.0 + torch.exp(-gate.to(F32))))[:, :, None]
    out.copy_((y * scale).reshape(T, heads * hd).to(out.dtype))


def weighted_sum(x, a, y, b, out):
    out.copy_((a * x.to(F32) + b * y.to(F32)).to(out.dtype))


def logit_cap(logits, cap):
    logits.copy_(cap * torch.tanh(logits / cap))


def gla_decay(low, w2t, bias, tau, alpha):
    z = low.to(F32) @ w2t
    if bias is not None:
        z = z + bias
    alpha.copy_(torch.exp(-torch.nn.functional.softplus(-z) / tau))


def gla_scan(q, k, v, alpha, state, q_indptr, state_slots, out, heads, dim, vdim, q_scale, max_q_len):
    for r in range(state_slots.numel()):
        S = state[int(state_slots[r])]                                   # [heads, vdim, dim]
        for t in range(int(q_indptr[r]), int(q_indptr[r + 1])):
            qt = q[t].to(F32).view(heads, dim) * q_scale
            kt, vt, at = k[t].to(F32).view(heads, dim), v[t].to(F32).view(heads, vdim), alpha[t].view(heads, dim)
            S.copy_(S * at[:, None, :] + vt[:, :, None] * kt[:, None, :])
            out[t] = torch.einsum("hvd,hd->hv", S, qt).reshape(-1)


def gla_out(o, gate, weight, eps, scale, out, heads, vdim, gate_act="silu"):
    T = o.shape[0]
    y = o.view(T, heads, vdim)
    y = y * (1.0 / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps))
    if weight is not None:
        y = y * weight
    y = y.reshape(T, heads * vdim)
    if gate is not None:
        g = gate.to(F32)
        y = y * ((g if gate_act == "silu" else 1.0) / (1.0 + torch.exp(-g)))
    out.copy_((y * scale).to(out.dtype))


def rotary_angles(positions, inv_freq, out):
    ang = positions.to(F32)[:, None] * inv_freq[None, :]
    out.copy_(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))


# ---------------------------------------------------------------- Dynamic Tanh
def dyt_norm(resid, delta, rows, weight, bias, alpha, out, write_resid):
    idx = rows.long() if rows is not None else torch.arange(resid.shape[0], device=resid.device)
    x = resid[idx].to(F32)
    if delta is not None:
        x = x + delta[idx].to(F32)
        if write_resid:
            resid[idx] = x
    y = torch.tanh(alpha * x) * weight
    out.copy_((y + bias if bias is not None else y).to(out.dtype))


# ---------------------------------------------------------------- attention over latent vectors
def gemm_heads(x, w, out):
    out.copy_(torch.einsum("mhk,hnk->mhn", x.to(F32), w.to(F32)).to(out.dtype))


def _turn_half(x, pos, inv_freq, dims):
    """x [T, ..., D]: the first ``dims`` elements turn, i with i + dims/2."""
    if not dims:
        return x
    half = dims // 2
    ang = pos.to(F32)[:, None] * inv_freq[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s_ = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s_, v * c + u * s_, x[..., dims:]], dim=-1)


def latent_prep(q, dkv, positions, slot_mapping, c_weight, eps, inv_freq, rot_dims, cache, q_abs, heads, dn, dr, rank):
    T = q.shape[0]
    if cache is not None:
        kv = dkv[:, : rank + dr].to(F32)
        c = kv[:, :rank]
        c = c * (1.0 / torch.sqrt((c * c).mean(dim=-1, keepdim=True) + eps)) * c_weight
        rec = torch.cat([c, _turn_half(kv[:, rank:], positions, inv_freq, rot_dims)], dim=-1).to(cache.dtype)
        page_size = cache.shape[2]
        sm = slot_mapping.long()
        cache[sm // page_size, 0, sm % page_size] = rec
    qr = q[:, : heads * (dn + dr)].to(F32).view(T, heads, dn + dr)[:, :, dn:]
    q_abs[:, :, rank:] = _turn_half(qr, positions, inv_freq, rot_dims).to(q_abs.dtype)


def latent_attention(q_abs, out, cache, positions, row_of_token, block_table, rank, page_size, scale, window, batch=None):
    T, H, kd = q_abs.shape
    for t in range(T):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        js = torch.arange(lo, p + 1)
        pages = block_table[int(row_of_token[t]), js // page_size].long()
        rec = cache[pages, 0, js % page_size].to(F32)          # [n, kd]
        pr = torch.softmax((q_abs[t].to(F32) @ rec.t()) * scale, dim=-1)
        out[t] = (pr @ rec[:, :rank]).to(out.dtype)


# ---------------------------------------------------------------- matrix memories with a scalar decay
def decay_scan(q, k, v, a, b, state, q_indptr, state_slots, out, heads, kq_heads, dim, vdim, ones_column, q_scale, act="none"):
    vcols = vdim + int(bool(ones_column))
    rep = heads // kq_heads
    T = v.shape[0]
    if a.dim() == 1:                                # one decay (and one input weight) a head for all tokens
        a = a[None, :].expand(T, heads)
        b = torch.ones(T, heads) if b is None else b[None, :].expand(T, heads)
    if act == "silu":
        q, k, v = (x.to(F32) / (1.0 + torch.exp(-x.to(F32))) for x in (q, k, v))
    for r in range(state_slots.numel()):
        S = state[int(state_slots[r]), : heads * vcols * dim].view(heads, vcols, dim)
        for t in range(int(q_indptr[r]), int(q_indptr[r + 1])):
            qt = q[t].to(F32).view(kq_heads, dim).repeat_interleave(rep, dim=0) * q_scale
            kt = k[t].to(F32).view(kq_heads, dim).repeat_interleave(rep, dim=0)
            vt = v[t].to(F32).view(heads, vdim)
            if ones_column:
                vt = torch.cat([vt, torch.ones(heads, 1)], dim=1)
            S.copy_(S * a[t][:, None, None] + (b[t][:, None] * vt)[:, :, None] * kt[:, None, :])
            out[t] = torch.einsum("hvd,hd->hv", S, qt)


def mlstm_gates(pre, bias_i, bias_f, cap, q_indptr, state_slots, state, m_offset, a, b, floor):
    H = pre.shape[1] // 2
    gi = cap * torch.tanh((pre[:, :H] + bias_i) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((pre[:, H:] + bias_f) / cap))
    for r in range(state_slots.numel()):
        m = state[int(state_slots[r]), m_offset: m_offset + H]
        for t in range(int(q_indptr[r]), int(q_indptr[r + 1])):
            m_new = torch.maximum(gf[t] + m, gi[t])
            a[t] = torch.exp(gf[t] + m - m_new)
            b[t] = torch.exp(gi[t] - m_new)
            floor[t] = torch.exp(-m_new)
            m.copy_(m_new)


def mlstm_out(num, floor, gate, weight, eps, out, heads, vdim):
    T = num.shape[0]
    o = num[:, :, :vdim] / (torch.maximum(num[:, :, vdim].abs(), floor) + 1e-6)[:, :, None]
    o = o * (1.0 / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps))
    o = o.reshape(T, heads * vdim) * weight * torch.sigmoid(gate.to(F32))
    out.copy_(o.to(out.dtype))


def ssm_gates(dt_raw, dt_bias, a_log, a, b):
    dt = torch.nn.functional.softplus(dt_raw + dt_bias)
    a.copy_(torch.exp(-torch.exp(a_log) * dt))
    b.copy_(dt)


def conv_silu(x, weight, bias, state, conv_offset, q_indptr, row_of_token, state_slots, out):
    C, taps = weight.shape
    for r in range(state_slots.numel()):
        beg, end = int(q_indptr[r]), int(q_indptr[r + 1])
        hist = state[int(state_slots[r]), conv_offset: conv_offset + C * (taps - 1)].view(C, taps - 1)
        seq = torch.cat([hist.t(), x[beg:end].to(F32)], dim=0)               # [taps - 1 + n, C]
        acc = bias[None, :].repeat(end - beg, 1) if bias is not None else torch.zeros(end - beg, C)
        for j in range(taps):
            acc = acc + seq[j: j + end - beg] * weight[:, j][None, :]
        out[beg:end] = (acc / (1.0 + torch.exp(-acc))).to(out.dtype)
        if taps > 1:
            hist.copy_(seq[seq.shape[0] - (taps - 1):].t())


def gated_group_norm(y, x, skip, vdim, z, weight, eps, out, parts):
    T, inner = y.shape
    v = y
    if skip is not None:
        v = v + skip.repeat_interleave(vdim)[None, :] * x.to(F32)
    g = z.to(F32)
    v = (v * (g / (1.0 + torch.exp(-g)))).view(T, parts, inner // parts)
    v = v * (1.0 / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps))
    out.copy_((v.reshape(T, inner) * weight).to(out.dtype))


# ---------------------------------------------------------------- routed experts
def moe_select(z, correction, scratch, experts, top, groups, keep, scale, ids, weights, scores="sigmoid", group_score="top2_sum"):
    if scores == "softmax_chosen":
        s_ = z[:, :experts].clone()
    else:
        s_ = torch.sigmoid(z[:, :experts]) if scores == "sigmoid" else torch.softmax(z[:, :experts], dim=-1)
    ch = s_ + correction if correction is not None else s_.clone()
    per = experts // groups
    g = ch.view(-1, groups, per)
    gs = g.topk(min(2, per) if group_score == "top2_sum" else 1, dim=-1).values.sum(-1)
    kept = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, gs.topk(keep, dim=-1).indices, True)
    ch = torch.where(kept[:, :, None].expand(-1, -1, per).reshape(-1, experts), ch, torch.full_like(ch, -math.inf))
    pick = torch.sort(ch, dim=-1, descending=True, stable=True).indices[:, :top]       # ties go to the lower index
    ids.copy_(pick.to(torch.int32))
    weights.copy_((torch.softmax(s_.gather(1, pick), dim=-1) if scores == "softmax_chosen" else s_.gather(1, pick)) * scale)


def moe_plan_size(experts, pairs):
    return experts + 2 + 3 * (pairs // 64 + experts + 1)


def moe_plan(ids, experts, plan, place_of_pair, row_of_place):
    T, top = ids.shape
    flat = ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    place_of_pair[order] = torch.arange(T * top, dtype=torch.int32)
    row_of_place[: T * top] = (order // top).to(torch.int32)
    counts = torch.bincount(flat, minlength=experts)
    plan[:experts] = (torch.cumsum(counts, 0) - counts).to(torch.int32)
    plan[experts] = T * top
    plan[experts + 1] = -1                      # no tiles: the plain statement of the grouped product reads the runs


def moe_gemm(x, rows, w, out, plan, experts):
    pairs = out.shape[0]
    bounds = plan[: experts + 1].tolist()
    for e in range(experts):
        lo, hi = bounds[e], bounds[e + 1]
        if hi > lo:
            src = x[rows[lo:hi].long()] if rows is not None else x[lo:hi]
            out[lo:hi] = (src.to(F32) @ w[e].to(F32).t()).to(out.dtype)


def moe_combine(y, place_of_pair, weights, shared, gate, out):
    T, top = weights.shape
    acc = (weights[:, :, None] * y[place_of_pair[: T * top].long()].to(F32).view(T, top, -1)).sum(1)
    if shared is not None:
        acc = acc + (torch.sigmoid(gate)[:, None] if gate is not None else 1.0) * shared.to(F32)
    out.copy_(acc.to(out.dtype))


# ---------------------------------------------------------------- parts of further designs
def clamped_glu(gate_up, out, limit, alpha):
    g = gate_up[:, 0::2].to(F32).clamp(max=limit)
    u = gate_up[:, 1::2].to(F32).clamp(min=-limit, max=limit)
    out.copy_((g * torch.sigmoid(alpha * g) * (u + 1.0)).to(out.dtype))


def branch_norm_add(resid, branch, weight, eps, copy):
    if branch is not None:
        b = branch.to(F32)
        resid += b / torch.sqrt((b * b).mean(-1, keepdim=True) + eps) * weight
    if copy is not None:
        copy.copy_(resid.to(copy.dtype))


def branch_norm_add_norm(resid, branch, weight, eps, next_weight, next_eps, out):
    b = branch.to(F32)
    resid += b / torch.sqrt((b * b).mean(-1, keepdim=True) + eps) * weight
    out.copy_((resid / torch.sqrt((resid * resid).mean(-1, keepdim=True) + next_eps) * next_weight).to(out.dtype))


def rms_rows(x, weight, eps, out):
    y = x.to(F32)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    out.copy_((y * weight if weight is not None else y).to(out.dtype))


def normed_sum(xs, biases, weights, scales, eps, out):
    total = 0.0
    for i, x in enumerate(xs):
        y = x.to(F32) + (biases[i] if biases is not None and biases[i] is not None else 0.0)
        total = total + scales[i] * (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)) * weights[i]
    out.copy_(total.to(out.dtype))


def bias_add(x, bias):
    x.copy_((x.to(F32) + bias).to(x.dtype))


def attention_prep_post(qkv, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim, k_cache, v_cache,
                        nq, nkv, hd, vd, page_size, norm_first=False):
    T = qkv.shape[0]
    pos = positions.to(F32)

    def prepared(x, weight):                         # x [T, heads, hd]
        x = x.to(F32).clone()
        if norm_first:
            if eps is not None:
                x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
                x = x * weight if weight is not None else x
            return _turn_half(x, pos, inv_freq, rotary_dim) if rotary_dim else x
        if rotary_dim:
            x = _turn_half(x, pos, inv_freq, rotary_dim)
        if eps is not None:
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
        return x * weight if weight is not None else x

    q = prepared(qkv[:, : nq * hd].view(T, nq, hd), q_weight)
    qkv[:, : nq * hd] = q.reshape(T, nq * hd).to(qkv.dtype)
    if nkv:
        k = prepared(qkv[:, nq * hd: (nq + nkv) * hd].view(T, nkv, hd), k_weight).to(qkv.dtype)
        v = qkv[:, (nq + nkv) * hd: (nq + nkv) * hd + nkv * vd].view(T, nkv, vd)
        keep = slot_mapping >= 0
        page, off = (slot_mapping[keep] // page_size).long(), (slot_mapping[keep] % page_size).long()
        k_cache[page, :, off] = k[keep]
        v_cache[page, :, off] = v[keep]


def causal_conv(x, in_bias, weight, out_bias, act, state, conv_offset, q_indptr, row_of_token, state_slots, out):
    C, taps = weight.shape
    for r in range(state_slots.numel()):
        beg, end = int(q_indptr[r]), int(q_indptr[r + 1])
        if end == beg:
            continue
        hist = state[int(state_slots[r]), conv_offset: conv_offset + C * (taps - 1)].view(C, taps - 1)
        xin = x[beg:end].to(F32) + (in_bias[None, :] if in_bias is not None else 0.0)
        seq = torch.cat([hist.t(), xin], dim=0)                               # [taps - 1 + n, C]
        acc = out_bias[None, :].repeat(end - beg, 1) if out_bias is not None else torch.zeros(end - beg, C)
        for j in range(taps):
            acc = acc + seq[j: j + end - beg] * weight[:, j][None, :]
        out[beg:end] = (acc / (1.0 + torch.exp(-acc)) if act == "silu" else acc).to(out.dtype)
        if taps > 1:
            hist.copy_(seq[seq.shape[0] - (taps - 1):].t())


def rglru_scan(z, u, y, bias_r, bias_i, lam, y_bias, c_decay, state, q_indptr, state_slots, out, blocks, max_q_len):
    T, width = u.shape
    bs = width // blocks
    zz = z.view(T, blocks, 2, bs)
    rg = torch.sigmoid(zz[:, :, 0].reshape(T, width) + bias_r)
    ig = torch.sigmoid(zz[:, :, 1].reshape(T, width) + bias_i)
    log_a = -c_decay * rg * torch.nn.functional.softplus(lam)
    a = torch.exp(log_a)
    b = torch.sqrt(-torch.expm1(2.0 * log_a)) * ig * u.to(F32)
    yy = y.to(F32) + (y_bias if y_bias is not None else 0.0)
    yy = 0.5 * yy * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (yy + 0.044715 * yy ** 3)))
    for r in range(state_slots.numel()):
        S = state[int(state_slots[r]), :width]
        for t in range(int(q_indptr[r]), int(q_indptr[r + 1])):
            S.copy_(a[t] * S + b[t])
            out[t] = (S * yy[t]).to(out.dtype)


def delta_gates(pre, a_log, dt_bias, beta, decay):
    H = beta.shape[1]
    beta.copy_(torch.sigmoid(pre[:, :H]))
    decay.copy_(torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(pre[:, H: 2 * H] + dt_bias)))


def delta_scan(q, k, v, beta, decay, state, q_indptr, state_slots, out, heads, kq_heads, dim, vdim, q_scale, unit_eps):
    T = v.shape[0]
    qq, kk = q.to(F32).view(T, kq_heads, dim), k.to(F32).view(T, kq_heads, dim)
    qq = qq / torch.sqrt((qq * qq).sum(-1, keepdim=True) + unit_eps) * q_scale
    kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + unit_eps)
    vv = v.to(F32).view(T, heads, vdim)
    rep = heads // kq_heads
    for r in range(state_slots.numel()):
        S = state[int(state_slots[r]), : heads * vdim * dim].view(heads, vdim, dim)         # a head's memory transposed
        for t in range(int(q_indptr[r]), int(q_indptr[r + 1])):
            for h in range(heads):
                g = h // rep
                Sh = S[h] * decay[t, h]
                u = beta[t, h] * (vv[t, h] - Sh @ kk[t, g])
                Sh = Sh + torch.outer(u, kk[t, g])
                S[h] = Sh
                out[t, h] = Sh @ qq[t, g]


ALL = ("rotary_angles", "embedding", "rmsnorm", "residual_add", "gemm", "fused_gemm_shape_ok", "fused_decode_supported", "attention_prep_takes_angles", "attention_prep", "paged_attention", "silu_mul", "gemm_silu_mul", "argmax", "scatter_tokens", "sample",
       "act_mul", "gemm_act_mul", "attention_prep_row", "head_gate", "weighted_sum", "logit_cap", "gla_decay", "gla_scan", "gla_out",
       "dyt_norm", "gemm_heads", "latent_prep", "latent_attention", "decay_scan", "mlstm_gates", "mlstm_out", "ssm_gates", "conv_silu",
       "gated_group_norm", "moe_select", "moe_plan_size", "moe_plan", "moe_gemm", "moe_combine", "clamped_glu", "branch_norm_add",
       "attention_prep_post", "causal_conv", "rglru_scan", "delta_gates", "delta_scan", "branch_norm_add_norm", "rms_rows", "normed_sum",
       "bias_add")
