"""Tiny Lukinex configurations for the tests.  Between them they vary every size and option of the design: the three
mixers in several orders (a parallel layer first, a latent layer first, two parallel layers), latent layers that read an
earlier layer's latents (with other head counts and sizes than the owner's), layers without a feed-forward, experts with and
without a shared expert, one expert chosen, several, and all of them, grouped, single and full key heads, rotation of a part
of a head, of all of it and of none, with and without divided frequencies, value widths below, at and above the key width,
windows of one token, of a few (not a multiple of the page) and longer than any test sequence, no window at all, kept first
tokens fewer than a page, more than a page, more than the window, and none, one to five convolution taps and none, with and
without capped scores, one decay head and several with decays from 0.3 to 1, and (K3) sizes that reach the kernels' wider
paths."""
import json
import os
import tempfile

from arle_b200.weights import write_random_model


def attn(heads, kv_heads, dim, vdim, scale, window=None, keep_first=0, rot_dims=0, base=10000.0, factor=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return {"type": "attention", "mixer": m}


def latent(heads, dim, vdim, kv_rank, q_rank, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def parallel(left, right):
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def left(heads, kv_heads, dim, vdim, scale, window=None, keep_first=0, rot_dims=0, base=10000.0, conv=0, softcap=None, factor=None):
    m = attn(heads, kv_heads, dim, vdim, scale, window, keep_first, rot_dims, base, factor)["mixer"]
    if conv:
        m["conv"] = conv
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(mixer, mlp):
    return json.loads(json.dumps({"type": mixer["type"], "mixer": mixer["mixer"], "mlp": mlp}))      # no two layers share an object


def model(vocab, width, eps, layers):
    return {"architecture": "Lukinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


TINY_K1 = model(211, 64, 1e-5, [
    layer(attn(4, 2, 16, 24, 0.2, window=7, keep_first=3, rot_dims=8, factor=4.0), moe(6, 2, 40, 1.2, shared=(24, 0.8))),
    layer(latent(3, 8, 12, 20, 28, 0.3), moe(5, 3, 16, 0.9)),
    layer(latent(2, 16, 8, 20, 12, 0.25, kv_from=1), None),                   # reads layer 1's latents with other heads and sizes
    layer(parallel(left(4, 2, 12, 20, 0.3, window=9, keep_first=2, rot_dims=12, conv=3, softcap=5.0), right(3, 8, 12, (0.6, 0.9, 0.999))),
          moe(6, 2, 40, 1.5, shared=(48, 2.0)))])
# K2: the values that a model may happen to make equal or 1 are all different or all 1 here; a parallel layer first; kept
# first tokens beyond the window's length and over more than a page; no window, no rotation, no convolution, no cap
TINY_K2 = model(157, 48, 2e-6, [
    layer(parallel(left(6, 6, 8, 4, 0.4, window=1, keep_first=0, rot_dims=0, conv=1, softcap=None), right(1, 20, 8, (1.0,))), moe(3, 1, 24, 2.0)),
    layer(attn(1, 1, 12, 40, 0.3, rot_dims=12, base=500.0), moe(4, 4, 16, 0.5, shared=(8, 0.7))),
    layer(latent(5, 4, 6, 36, 8, 0.5), None),
    layer(parallel(left(2, 1, 20, 28, 0.2, window=5, keep_first=11, rot_dims=4, conv=5, softcap=2.0, factor=1.5), right(5, 4, 6, (0.3, 0.5, 0.8, 0.95, 1.0))),
          None),
    layer(attn(6, 2, 9, 4, 0.5, window=1000, keep_first=4, rot_dims=6, factor=3.3), moe(8, 5, 12, 1.0)),      # an odd head size
    layer(latent(1, 24, 16, 36, 40, 0.2, kv_from=2), moe(2, 2, 20, 3.0, shared=(32, 1.0))),
    layer(parallel(left(3, 1, 16, 16, 0.25, conv=2), right(2, 12, 20, (0.97, 0.7))), moe(4, 2, 28, 1.1))])
# K3: wider: heads of 64 and 128 with values as wide as keys, a latent of 128, aligned rows
TINY_K3 = model(512, 256, 3e-6, [
    layer(attn(8, 2, 64, 64, 0.125, window=48, keep_first=5, rot_dims=32, base=50000.0, factor=2.5), moe(16, 4, 96, 1.25, shared=(128, 2.0))),
    layer(latent(8, 32, 64, 128, 96, 0.17), moe(8, 2, 128, 3.0)),
    layer(parallel(left(4, 1, 128, 128, 0.09, window=40, keep_first=20, rot_dims=128, conv=4, softcap=30.0), right(4, 64, 64, (0.7, 0.9, 0.97, 0.999))),
          moe(8, 2, 64, 1.0, shared=(256, 1.5))),
    layer(latent(4, 64, 32, 128, 160, 0.125, kv_from=1), None),
    layer(attn(2, 1, 128, 128, 0.09, window=33, keep_first=17, rot_dims=64), None)])
# A: attention alone (a window of 6 that keeps 3 tokens) and P: the parallel mixer alone (a window of 7 that keeps 2), for the
# tests that sharpen them; F: a window longer than any test sequence and a latent layer; S: the states with little else
TINY_A = model(180, 64, 1e-5, [layer(attn(2, 1, 16, 16, 0.25, window=6, keep_first=3, rot_dims=8), moe(4, 2, 32, 1.0))])
TINY_P = model(180, 64, 1e-5, [layer(parallel(left(2, 1, 16, 12, 0.25, window=7, keep_first=2, rot_dims=16, conv=3, softcap=50.0),
                                              right(2, 8, 8, (0.9, 0.5))), None)])
TINY_F = model(180, 64, 1e-5, [layer(attn(2, 2, 16, 12, 0.25, window=4000, keep_first=1, rot_dims=16), moe(4, 2, 32, 1.0, shared=(16, 1.0))),
                               layer(latent(2, 16, 8, 24, 16, 0.25), None)])
TINY_S = model(180, 64, 1e-5, [layer(parallel(left(2, 1, 8, 8, 0.3, window=5, keep_first=1, rot_dims=8, conv=4, softcap=10.0), right(2, 16, 12, (0.999, 1.0))),
                                     moe(3, 2, 24, 1.0)),
                               layer(parallel(left(1, 1, 8, 12, 0.3, window=3, conv=2), right(3, 8, 4, (0.5, 0.9, 0.99))), None)])
CONFIGS = {"K1": TINY_K1, "K2": TINY_K2, "K3": TINY_K3, "A": TINY_A, "P": TINY_P, "F": TINY_F, "S": TINY_S}
INIT = {"K1": dict(sigma=0.12, gain_jitter=0.3), "K2": dict(sigma=0.14, gain_jitter=0.3), "K3": dict(sigma=0.06, gain_jitter=0.3),
        "A": dict(sigma=0.12, gain_jitter=0.3), "P": dict(sigma=0.12, gain_jitter=0.3), "F": dict(sigma=0.12, gain_jitter=0.3),
        "S": dict(sigma=0.12, gain_jitter=0.3)}
PAGE_SIZES = {"K1": 4, "K2": 8, "K3": 16, "A": 4, "P": 4, "F": 16, "S": 8}


def make_model_dir(name: str, seed: int = 0, root: str = None, **init) -> str:
    root = root or tempfile.mkdtemp(prefix=f"arle_tiny_{name}_")
    kw = dict(INIT[name])
    kw.update(init)
    return write_random_model(os.path.join(root, name), CONFIGS[name], seed, **kw)


def read_model(d: str):
    """(config dict, weights by name in float64) for the plain implementation."""
    import torch
    from safetensors.torch import load_file

    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.to(torch.float64) for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
