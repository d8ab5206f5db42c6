"""Tiny Lasupel configurations for the tests.  Between them they vary every size and option of the design: the three
mixers in several orders, layers that read an earlier layer's keys and values (through a window of their own, shorter or
longer than the owner's), layers without a feed-forward, dense and routed feed-forwards, one group and as many groups as
experts, one expert chosen and several, grouped, single and full key heads, rotation of a part of a head, of all of it and
of none, value widths below, at and above the key width, windows of one token, of a few (not a multiple of the page) and
longer than any test sequence, one and several gate blocks, two to five convolution taps, and (L3) sizes that reach the
kernels' wider paths."""
import json
import os
import tempfile

from arle_b200.weights import write_random_model


def attn(heads, kv_heads, dim, vdim, window, scale, rot_dims, base=10000.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, count, keep, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def layer(mixer, mlp):
    return json.loads(json.dumps({"type": mixer["type"], "mixer": mixer["mixer"], "mlp": mlp}))      # no two layers share an object


def model(vocab, width, eps, embed_scale, layers):
    return {"architecture": "Lasupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": layers}


TINY_L1 = model(211, 64, 1e-5, 1.5, [
    layer(attn(4, 2, 16, 24, 7, 0.2, 8), dense(96)),
    layer(rglru(48, 3, 3), moe(6, 2, 3, 2, 40, 1.2)),
    layer(attn(4, 2, 16, 24, 11, 0.3, 8, kv_from=0), None),                 # reads layer 0's cache through a longer window
    layer(delta(4, 2, 8, 12, 4), moe(6, 2, 3, 2, 40, 0.8))])
# L2: the values that a model may happen to make equal or 1 are all different or all 1 here
TINY_L2 = model(157, 48, 2e-6, 1.0, [
    layer(delta(3, 3, 20, 8, 2), moe(3, 1, 1, 1, 24, 2.0)),
    layer(attn(1, 1, 12, 40, 1000, 0.3, 12, 500.0), dense(80)),
    layer(rglru(40, 1, 5), None),
    layer(attn(6, 2, 8, 4, 1, 0.5, 0), moe(8, 4, 8, 5, 16, 0.5)),
    layer(attn(1, 1, 12, 40, 5, 0.4, 12, 500.0, kv_from=1), dense(32)),      # a shorter window than the owner's
    layer(delta(2, 1, 40, 24, 3), dense(64)),
    layer(rglru(56, 7, 2), moe(4, 2, 2, 2, 20, 1.0))])
# L3: wider: head 64 and 128, gate blocks of 64, state columns past one block, aligned rows
TINY_L3 = model(512, 256, 3e-6, 0.75, [
    layer(attn(8, 2, 64, 64, 48, 0.125, 32, 50000.0), moe(16, 4, 4, 2, 96, 1.25)),
    layer(rglru(256, 4, 4), dense(512)),
    layer(attn(8, 2, 64, 64, 20, 0.125, 32, 50000.0, kv_from=0), dense(256)),
    layer(delta(8, 4, 64, 128, 4), moe(8, 2, 1, 1, 128, 3.0)),
    layer(attn(2, 1, 128, 128, 33, 0.09, 128), None),
    layer(delta(2, 2, 160, 32, 4), None)])
# A: attention alone (windows of 6 and 13; the second layer reads the first one's keys), for the tests that sharpen it;
# F: a window longer than any test sequence; S: the recurrent mixers with little else; R: no paged cache at all
TINY_A = model(180, 64, 1e-5, 1.0, [layer(attn(2, 1, 16, 16, 6, 0.25, 8), dense(64)), layer(attn(2, 1, 16, 16, 13, 0.3, 8, kv_from=0), None)])
TINY_F = model(180, 64, 1e-5, 1.0, [layer(attn(2, 2, 16, 12, 4000, 0.25, 16), dense(64)), layer(rglru(32, 2, 4), None)])
TINY_S = model(180, 64, 1e-5, 1.0, [layer(rglru(48, 2, 4), dense(64)), layer(delta(2, 1, 16, 12, 4), None),
                                    layer(attn(2, 1, 8, 8, 5, 0.3, 8), None)])
TINY_R = model(200, 48, 1e-5, 1.0, [layer(rglru(32, 4, 3), dense(32)), layer(delta(2, 2, 8, 8, 3), None)])
CONFIGS = {"R": TINY_R, "L1": TINY_L1, "L2": TINY_L2, "L3": TINY_L3, "A": TINY_A, "F": TINY_F, "S": TINY_S}
INIT = {"R": dict(sigma=0.2, gain_jitter=0.3), "L1": dict(sigma=0.12, gain_jitter=0.3), "L2": dict(sigma=0.14, gain_jitter=0.3),
        "L3": dict(sigma=0.06, gain_jitter=0.3), "A": dict(sigma=0.12, gain_jitter=0.3), "F": dict(sigma=0.12, gain_jitter=0.3),
        "S": dict(sigma=0.12, gain_jitter=0.3)}
PAGE_SIZES = {"R": 16, "L1": 4, "L2": 8, "L3": 16, "A": 4, "F": 16, "S": 8}


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
