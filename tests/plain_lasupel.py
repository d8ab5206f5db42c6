"""A plain, slow implementation of the Lasupel design: float64 torch on the CPU, whole sequences,
no cache, no batching, one function per mechanism.  It shares no code with the package's model
path; the tests compare the engine with it.

A model is (config dict in the form of config.json, {tensor name: tensor}).  ``forward`` returns
the logits of every position and, on request, the residual after every layer.  ``rnd`` is applied to
every stored activation (identity by default; rounding to bfloat16 gives the tests the size of what
rounding alone does).

A layer adds the NORMED output of each sublayer: x <- x + n1(mixer(x)), x <- x + n2(ff(x)); the
sublayers read x as it is.  Notation: h is a sublayer's input [T, width]; positions count from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def _ident(x):
    return x


def round_bf16(x):
    return x.to(torch.float32).to(torch.bfloat16).to(F64)


def lin(W, x):
    """Rows of x through a matrix stored [out, in]."""
    return x @ W.to(F64).t()


# ----------------------------------------------------------------------------- small functions
def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotate_first_dims(x, pos, base, dims):
    """x [T, heads, D]; of the first ``dims`` numbers of a head, number i turns with number i + dims/2 by the
    angle pos * base^(-2i/dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    ang = (pos.to(F64)[:, None] * freq[None, :])[:, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def causal_conv(x, taps, bias=None):
    """x [T, C]; taps [C, K], the last column the current token's; zeros before the sequence."""
    T, C = x.shape
    K = taps.shape[1]
    xp = torch.cat([torch.zeros(K - 1, C, dtype=F64), x], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(K):
        y = y + xp[j: j + T] * taps.to(F64)[:, j][None, :]
    return y if bias is None else y + bias.to(F64)[None, :]


# ----------------------------------------------------------------------------- mixers
def attention_keys_values(h, W, p, m, eps, rnd=_ident):
    """Keys as a cache holds them (rotated, then brought to unit RMS per head) and values."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    k = rnd(lin(W[p + "k"], h)).view(T, G, d)
    v = rnd(lin(W[p + "v"], h)).view(T, G, dv)
    k = rnd(rms_unit(rotate_first_dims(k, pos, m["rot"]["base"], m["rot"]["dims"]), eps))
    return k, v


def attention(h, W, p, m, eps, kv, rnd=_ident):
    """Sliding-window attention whose softmax has one more term in its denominator, a sink of score 0
    without a value.  ``kv``: (keys, values) of this layer or of the layer it reads them from."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rnd(lin(W[p + "q"], h)).view(T, H, d)
    q = rnd(rms_unit(rotate_first_dims(q, pos, m["rot"]["base"], m["rot"]["dims"]), eps))
    k, v = kv
    rep = H // G
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        lo = max(0, t - m["mask"]["size"] + 1)
        for hh in range(H):
            g = hh // rep
            s = (k[lo: t + 1, g] @ q[t, hh]) * m["scale"]
            e = torch.exp(s)
            w = e / (1.0 + e.sum())
            out[t, hh] = w @ v[lo: t + 1, g]
    return rnd(lin(W[p + "o"], rnd(out.reshape(T, H * dv))))


def rglru(h, W, p, m, rnd=_ident):
    """The recurrent block with a real-gated linear recurrent unit."""
    T = h.shape[0]
    width, nb = m["width"], m["blocks"]
    y = rnd(gelu_tanh(lin(W[p + "y"], h) + W[p + "y.b"].to(F64)))
    xin = rnd(lin(W[p + "x"], h) + W[p + "x.b"].to(F64))
    u = rnd(causal_conv(xin, W[p + "conv"], W[p + "conv.b"]))
    bs = width // nb
    ub = u.view(T, nb, bs)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ra"].to(F64), ub) + W[p + "ra.b"].to(F64)[None]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ri"].to(F64), ub) + W[p + "ri.b"].to(F64)[None]).reshape(T, width)
    log_a = -8.0 * r * softplus(W[p + "lam"].to(F64))[None, :]
    a = torch.exp(log_a)
    gate = torch.sqrt(1.0 - a * a)
    S = torch.zeros(width, dtype=F64)
    out = torch.zeros(T, width, dtype=F64)
    for t in range(T):
        S = a[t] * S + gate[t] * i[t] * u[t]
        out[t] = S
    return rnd(lin(W[p + "o"], rnd(out * y)))


def delta_rule(h, W, p, m, eps, rnd=_ident):
    """The gated delta rule: a matrix state per head that forgets by a decay and is corrected towards the
    value of the current key."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rnd(silu(causal_conv(rnd(lin(W[p + "q"], h)), W[p + "q.conv"]))).view(T, G, d)
    k = rnd(silu(causal_conv(rnd(lin(W[p + "k"], h)), W[p + "k.conv"]))).view(T, G, d)
    v = rnd(silu(causal_conv(rnd(lin(W[p + "v"], h)), W[p + "v.conv"]))).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(W[p + "b"], h))
    decay = torch.exp(-torch.exp(W[p + "A_log"].to(F64))[None, :] * softplus(lin(W[p + "a"], h) + W[p + "dt_bias"].to(F64)[None, :]))
    gate = rnd(silu(lin(W[p + "g"], h))).view(T, H, dv)
    rep = H // G
    o = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        g = hh // rep
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.t() @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hh] = S.t() @ q[t, g]
    o = rms_unit(o, eps) * W[p + "norm"].to(F64)[None, None, :] * gate
    return rnd(lin(W[p + "o"], rnd(o.reshape(T, H * dv))))


# ----------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, p, rnd=_ident):
    return rnd(lin(W[p + "down"], rnd(silu(lin(W[p + "gate"], h)) * lin(W[p + "up"], h))))


def route(z, top, count, keep):
    """z [T, E] router logits.  Returns (indices [T, top], weights [T, top]): softmax scores, a group's score
    its largest, only the ``keep`` best groups stay eligible, the ``top`` largest eligible scores are chosen and
    are the weights as they are."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1)
    per = E // count
    gs = s.view(T, count, per).max(-1).values
    kept = torch.zeros(T, count, dtype=torch.bool)
    kept.scatter_(1, gs.topk(keep, dim=-1).indices, True)
    eligible = kept[:, :, None].expand(T, count, per).reshape(T, E)
    masked = torch.where(eligible, s, torch.full_like(s, -1.0))
    idx = masked.topk(top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def expert_ff(h, W, p, limit, rnd=_ident):
    g = torch.clamp(lin(W[p + "gate"], h), max=limit)
    u = torch.clamp(lin(W[p + "up"], h), min=-limit, max=limit)
    return rnd(lin(W[p + "down"], rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0))))


def moe_ff(h, W, p, mlp, rnd=_ident):
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = lin(W[p + "router"], h).to(torch.float32).to(F64)
    idx, wts = route(z, r["top"], groups["count"], groups["keep"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(r["top"]):
            e = int(idx[t, c])
            out[t] = out[t] + wts[t, c] * expert_ff(h[t: t + 1], W, f"{p}e{e}.", mlp["expert"]["limit"], rnd)[0]
    return rnd(out)


# ----------------------------------------------------------------------------- the model
def forward(cfg, W, tokens, rnd=_ident, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = rnd(x)
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(h, W, p, m, eps, rnd)
            branch = attention(h, W, p, m, eps, kept[i if m.get("kv_from") is None else m["kv_from"]], rnd)
        elif layer["type"] == "rglru":
            branch = rglru(h, W, p, m, rnd)
        elif layer["type"] == "delta":
            branch = delta_rule(h, W, p, m, eps, rnd)
        else:
            raise ValueError(layer["type"])
        x = x + rms_unit(branch, eps) * W[f"l{i}.norm1"].to(F64)
        if layer.get("mlp") is not None:
            h = rnd(x)
            ff = dense_ff(h, W, f"l{i}.mlp.", rnd) if layer["mlp"]["kind"] == "dense" else moe_ff(h, W, f"l{i}.mlp.", layer["mlp"], rnd)
            x = x + rms_unit(ff, eps) * W[f"l{i}.norm2"].to(F64)
        if layers_out is not None:
            layers_out.append(x.clone())
    final = rnd(rms_unit(x, eps) * W["final.norm"].to(F64))
    return lin(W["head"], final)


def generate_greedy(cfg, W, prompt, steps):
    toks = list(prompt)
    for _ in range(steps):
        toks.append(int(forward(cfg, W, toks)[-1].argmax()))
    return toks[len(prompt):]
