"""A plain, slow implementation of the Lukinex design: float64 torch on the CPU, whole sequences,
no cache, no batching, one function per mechanism.  It shares no code with the package's model
path; the tests compare the engine with it.

A model is (config dict in the form of config.json, {tensor name: tensor}).  ``forward`` returns
the logits of every position and, on request, the residual after every layer.  ``rnd`` is applied to
every stored activation (identity by default; rounding to bfloat16 gives the tests the size of what
rounding alone does).

A layer norms before AND after each sublayer: x <- x + n1b(mixer(n1(x))), x <- x + n2b(ff(n2(x))).
Notation: h is a sublayer's input [T, width]; positions count from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
EXPERT_ALPHA = 1.702


def _ident(x):
    return x


def round_bf16(x):
    return x.to(torch.float32).to(torch.bfloat16).to(F64)


def lin(W, x, b=None):
    """Rows of x through a matrix stored [out, in], plus a bias."""
    y = x @ W.to(F64).t()
    return y if b is None else y + b.to(F64)


# ----------------------------------------------------------------------------- small functions
def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.to(F64)


def silu(z):
    return z * torch.sigmoid(z)


def rotate_first_dims(x, pos, base, dims, divide_by=1.0):
    """x [T, heads, D]; of the first ``dims`` numbers of a head, number i turns with number i + dims/2 by the
    angle pos * base^(-2i/dims) / divide_by; the rest pass."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims) / divide_by
    ang = (pos.to(F64)[:, None] * freq[None, :])[:, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T, window=None, keep_first=0):
    """[T, T] bool: query i sees key j when j <= i and (i - j < window or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see = see & ((i - j < window) | (j < keep_first))
    return see


def softmax_attention(q, k, v, scale, see, softcap=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; query head h reads key head h // (H / G).  Returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].t()) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~see, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    w = w.to(F64)
    padded = torch.cat([torch.zeros((taps - 1, u.shape[1]), dtype=F64), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j: j + T] * w[:, j]
    return y


def constant_decay_memory(q, k, v, decay):
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, from S = 0.  q, k [T, H, D], v [T, H, Dv]."""
    T, H, D = q.shape
    out = torch.zeros((T, H, v.shape[-1]), dtype=F64)
    for h in range(H):
        S = torch.zeros((D, v.shape[-1]), dtype=F64)
        for t in range(T):
            S = float(decay[h]) * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.t() @ q[t, h]
    return out


# ----------------------------------------------------------------------------- mixers
def grouped_attention(h, W, p, m, eps, rnd=_ident):
    """The 'attention' mixer: per-head norm of q and k with a shared weight, rotation with divided frequencies, a window
    that keeps the first tokens."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rnd(lin(W[p + "q"], h)).view(T, H, D)
    k = rnd(lin(W[p + "k"], h)).view(T, G, D)
    v = rnd(lin(W[p + "v"], h)).view(T, G, Dv)
    q = rms_norm(q, W[p + "q.norm"], eps)
    k = rms_norm(k, W[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot is not None:
        div = float(rot["scaling"]["factor"]) if rot.get("scaling") is not None else 1.0
        q, k = (rotate_first_dims(t, pos, rot["base"], rot["dims"], div) for t in (q, k))
    q, k = rnd(q), rnd(k)
    mask = m.get("mask")
    see = visible(T, mask["size"], mask.get("keep_first", 0)) if mask is not None else visible(T)
    o = rnd(softmax_attention(q, k, v, m["scale"], see))
    return lin(W[p + "o"], o.reshape(T, H * Dv))


def biased_conv_attention(h, W, p, m, rnd=_ident):
    """The left member of the 'parallel' mixer: biases, a short convolution on q, k, v, rotation, capped scores."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q, k, v = (rnd(lin(W[p + n], h, W[p + n + ".b"])) for n in ("q", "k", "v"))
    if m.get("conv"):
        q, k, v = (rnd(short_conv(t, W[p + n + ".conv"])) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, Dv)
    rot = m.get("rot")
    if rot is not None:
        div = float(rot["scaling"]["factor"]) if rot.get("scaling") is not None else 1.0
        q, k = (rotate_first_dims(t, pos, rot["base"], rot["dims"], div) for t in (q, k))
    q, k = rnd(q), rnd(k)
    mask = m.get("mask")
    see = visible(T, mask["size"], mask.get("keep_first", 0)) if mask is not None else visible(T)
    o = rnd(softmax_attention(q, k, v, m["scale"], see, m.get("softcap")))
    return lin(W[p + "o"], o.reshape(T, H * Dv), W[p + "o.b"])


def lightning_attention(h, W, p, m, eps, rnd=_ident):
    """The right member: silu on q, k, v, a memory per head with a constant decay, a norm over all heads at once, a
    sigmoid gate."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = rnd(silu(lin(W[p + "q"], h))).view(T, H, D)
    k = rnd(silu(lin(W[p + "k"], h))).view(T, H, D)
    v = rnd(silu(lin(W[p + "v"], h))).view(T, H, Dv)
    o = constant_decay_memory(q, k, v, m["decay"]).reshape(T, H * Dv)
    o = rnd(rms_norm(o, W[p + "norm"], eps) * torch.sigmoid(lin(W[p + "g"], h)))
    return lin(W[p + "o"], o)


def parallel_mixer(h, W, p, m, eps, rnd=_ident):
    left = rnd(biased_conv_attention(h, W, p + "left.", m["left"], rnd))
    right = rnd(lightning_attention(h, W, p + "right.", m["right"], eps, rnd))
    return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))


def latent_of(h, W, p, eps, rnd=_ident):
    """What a latent-attention layer with keys of its own caches per token."""
    return rnd(rms_norm(rnd(lin(W[p + "dkv"], h)), W[p + "dkv.norm"], eps))


def latent_attention(h, W, p, m, eps, c, rnd=_ident):
    """Queries through a latent of their own; keys and values per head from the cached latent ``c``; no positions; causal."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    cq = rnd(rms_norm(rnd(lin(W[p + "dq"], h)), W[p + "dq.norm"], eps))
    q = rnd(lin(W[p + "uq"], cq)).view(T, H, D)
    k = lin(W[p + "uk"], c).view(T, H, D)
    v = lin(W[p + "uv"], c).view(T, H, Dv)
    o = rnd(softmax_attention(q, k, v, m["scale"], visible(T)))
    return lin(W[p + "o"], o.reshape(T, H * Dv))


# ----------------------------------------------------------------------------- feed-forward
def clamped_expert(h, W, p, limit, rnd=_ident):
    g = torch.clamp(lin(W[p + "gate"], h), max=limit)
    u = torch.clamp(lin(W[p + "up"], h), min=-limit, max=limit)
    return lin(W[p + "down"], rnd(g * torch.sigmoid(EXPERT_ALPHA * g) * (u + 1.0)))


def route(z, top):
    """The ``top`` largest logits of each row (ties to the lower index) and the softmax over them alone."""
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), dim=-1)


def moe_ff(h, W, p, mlp, rnd=_ident):
    T = h.shape[0]
    top = mlp["router"]["top"]
    ids, wts = route(lin(W[p + "router"], h), top)
    out = torch.zeros((T, W[p + "e0.down"].shape[0]), dtype=F64)
    for t in range(T):
        for c in range(top):
            e = int(ids[t, c])
            out[t] += wts[t, c] * rnd(clamped_expert(h[t: t + 1], W, f"{p}e{e}.", mlp["expert"]["limit"], rnd))[0]
    if mlp.get("shared") is not None:
        out = out + rnd(clamped_expert(h, W, p + "shared.", mlp["shared"]["limit"], rnd))
    return out


# ----------------------------------------------------------------------------- the model
def forward(cfg, W, tokens, rnd=_ident, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = rnd(rms_norm(x, W[f"l{i}.norm1"], eps))
        if layer["type"] == "attention":
            branch = grouped_attention(h, W, p, m, eps, rnd)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, W, p, eps, rnd)
            branch = latent_attention(h, W, p, m, eps, latents[i if src is None else src], rnd)
        elif layer["type"] == "parallel":
            branch = parallel_mixer(h, W, p, m, eps, rnd)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(rnd(branch), W[f"l{i}.norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rnd(rms_norm(x, W[f"l{i}.norm2"], eps))
            x = x + rms_norm(rnd(moe_ff(h, W, f"l{i}.mlp.", layer["mlp"], rnd)), W[f"l{i}.norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    final = rnd(rms_norm(x, W["final.norm"], eps))
    return lin(W["head"], final)


def generate_greedy(cfg, W, prompt, steps):
    toks = list(prompt)
    for _ in range(steps):
        toks.append(int(forward(cfg, W, toks)[-1].argmax()))
    return toks[len(prompt):]
