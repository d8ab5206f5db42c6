"""Lukinex on the GPU against the plain implementation (``plain_lukinex``): every new or widened kernel alone at sizes of no
model (kept first keys and capped scores in the paged attention kernels, the norm before the rotation, the memory with a
constant decay per head continuing from states in permuted slots, the norm over all heads with a sigmoid gate, routing by a
softmax over the chosen, the fused norms around the residual, the normed sum of side-by-side outputs), the engine under
every cutting in float32 and bfloat16 on tiny configurations, the first tokens of a sequence and prompts that end on page
borders, keys just inside and just outside a window and the kept first tokens made to decide the logits (sharpened
attention), a far key deciding the logits through the latent attention, far tokens living on in the memories (decays next to
one), long decoding while window pages turn over and first pages stay, a request that starts again, greedy generation
through the public entry point with CUDA graphs and preemption, and the replay tool and the command line as subprocesses."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kernel_refs
import plain_lukinex as plain
import traces
from arle_b200 import Engine, ops
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.sampling import SamplingParams
from arle_b200.weights import SafetensorsFile, write_safetensors
from tiny_lukinex import CONFIGS, PAGE_SIZES, make_model_dir, read_model

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
# error of a logits row as a fraction of the spread of the plain model's logits: float32 rounding through a few layers.
# In bfloat16 the engine's worst position may be off by 4.5 times what the plain model's worst is off by when every
# activation it stores is rounded to bfloat16: two ways of rounding the same sums differ by more than either differs
# from the exact result.
REL = {torch.float32: 5e-4, torch.bfloat16: 1e-2}
LENGTHS = {"K1": [1, 5, 12, 23, 70, 130, 33], "K2": [2, 17, 40, 96, 64, 31], "K3": [3, 66, 150, 64, 40, 97], "S": [2, 33, 80, 17, 64],
           "A": [3, 50, 64, 29], "P": [1, 40, 33, 7, 70]}
_cache, _rounding = {}, {}


def rounding_cost(cfg, w, toks, exact) -> float:
    return (plain.forward(cfg, w, toks, rnd=plain.round_bf16) - exact).abs().max().item()


def model_and_oracle(name, tmp_path_factory):
    if name not in _cache:
        d = make_model_dir(name, seed=21, root=str(tmp_path_factory.mktemp(f"tiny{name}")))
        cfg, w = read_model(d)
        reqs = traces.make_requests(cfg["vocab"], LENGTHS[name], seed=6)
        oracle = {r: plain.forward(cfg, w, t) for r, t in reqs.items()}
        _cache[name] = (d, cfg, w, reqs, oracle)
        _rounding[id(oracle)] = max(rounding_cost(cfg, w, t, oracle[r]) for r, t in reqs.items())
    return _cache[name]


def assert_close(got, want, dtype, what="", rounding=0.0):
    err = (got.double().cpu() - want).abs().max(dim=-1).values
    tol = REL[dtype] * float(want.std())
    if dtype == torch.bfloat16:
        tol = max(tol, 4.5 * rounding)
    assert err.max().item() <= tol, f"{what}: first wrong position {int((err > tol).nonzero()[0])}, error {err.max().item():.3g}, tolerance {tol:.3g}"


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def _both(fn, args, outs, kwargs=None):
    """Runs ``fn`` of ops on the GPU and of kernel_refs on the CPU on copies of the same arguments; returns the named outputs."""
    def on(a, dev):
        if isinstance(a, torch.Tensor):
            return a.to(dev) if dev else a.clone()
        if isinstance(a, (list, tuple)) and a and all(isinstance(x, torch.Tensor) or x is None for x in a):
            return [None if x is None else (x.to(dev) if dev else x.clone()) for x in a]
        return a
    cpu = [on(a, None) for a in args]
    gpu = [on(a, DEV) for a in args]
    getattr(ops, fn)(*gpu, **(kwargs or {}))
    getattr(kernel_refs, fn)(*cpu, **(kwargs or {}))
    torch.cuda.synchronize()
    return [(gpu[i].float().cpu(), cpu[i].float()) for i in outs]


def _rows(g, starts, lens, ps, extra_pages=5):
    """Rows in scattered pages: positions, row of token, block table, slots of the step's tokens, q_indptr."""
    need = [-(-(s + n) // ps) for s, n in zip(starts, lens)]
    pages = sum(need) + extra_pages
    perm = torch.randperm(pages, generator=g)[: sum(need)].to(torch.int32)
    bt = torch.full((len(lens), max(need)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(need):
        bt[r, :n] = perm[at: at + n]
        at += n
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(torch.int32)
    row = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to(torch.int32)
    slots = (bt[row.long(), (pos // ps).long()] * ps + pos % ps).to(torch.int32)
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    return pages, bt, pos, row, slots, indptr


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nq,nkv,hd,vd,window,keep,cap,ps", [(4, 2, 16, 24, 7, 3, None, 4), (1, 1, 12, 40, 5, 11, 2.0, 8), (6, 2, 8, 4, 1, 0, 0.5, 16),
                                                            (3, 1, 48, 48, 33, 20, 20.0, 16), (2, 2, 80, 32, 0, 6, 5.0, 4), (5, 5, 20, 20, 40, 17, None, 16)])
def test_attention_with_kept_first_keys_and_capped_scores(dtype, nq, nkv, hd, vd, window, keep, cap, ps):
    """The general kernel: rows that start at 0, in the middle of the kept tokens, just past them and far past them, in pages of
    their own; the pages that a window has passed and that hold no kept token are poisoned, so a kernel that looked there shows."""
    g = torch.Generator().manual_seed(hd + vd + window)
    starts, lens = [0, 2, keep + 1, 60, 119], [70, 9, 31, 1, 12]
    pages, bt, pos, row, slots, _ = _rows(g, starts, lens, ps)
    T = int(pos.numel())
    q = torch.randn(T, nq * hd, generator=g).to(dtype)
    kc = torch.randn(pages, nkv, ps, hd, generator=g).to(dtype)
    vc = torch.randn(pages, nkv, ps, vd, generator=g).to(dtype)
    if window:
        for r, (s, n) in enumerate(zip(starts, lens)):
            for p in range(-(-keep // ps), max(0, s - window + 1) // ps):       # no query of the row sees these pages
                kc[bt[r, p]] = 1e4
                vc[bt[r, p]] = float("nan")
    out = torch.zeros(T, nq * vd, dtype=dtype)
    kw = dict(vd=vd, keep_first=keep, softcap=cap)
    (got, want), = _both("paged_attention", [q, out, kc, vc, pos, row, bt, nq, nkv, hd, ps, 0.3, window or None], [1], kw)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nq,nkv,hd,vd,rdim,ps,norm", [(4, 2, 16, 24, 8, 4, True), (1, 1, 12, 40, 12, 8, True), (6, 6, 8, 4, 0, 16, False),
                                                       (3, 1, 48, 20, 48, 16, False), (2, 1, 130, 64, 64, 16, True)])
def test_preparation_with_the_norm_before_the_rotation(dtype, nq, nkv, hd, vd, rdim, ps, norm):
    g = torch.Generator().manual_seed(hd)
    pages, bt, pos, row, slots, _ = _rows(g, [0, 13, 200], [9, 4, 1], ps)
    T = int(pos.numel())
    qkv = torch.randn(T, nq * hd + nkv * (hd + vd) + 3, generator=g).to(dtype)[:, : nq * hd + nkv * (hd + vd)]
    wq, wk = (torch.rand(hd, generator=g) + 0.5 for _ in range(2))
    inv = torch.pow(torch.tensor(300.0), -torch.arange(rdim // 2) * 2.0 / max(rdim, 1)).float() / 1.5
    kc, vc = torch.zeros(pages, nkv, ps, hd, dtype=dtype), torch.zeros(pages, nkv, ps, vd, dtype=dtype)
    args = [qkv, pos, slots, wq if norm else None, wk if norm else None, 1e-5 if norm else None, inv if rdim else None, rdim, kc, vc, nq, nkv, hd, vd, ps]
    for got, want in _both("attention_prep_post", args, [0, 8, 9], dict(norm_first=True)):
        torch.testing.assert_close(got, want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("H,dim,vdim,lens", [(3, 8, 12, [1, 5, 40]), (1, 20, 8, [18, 1, 2]), (4, 64, 64, [33, 1, 9]), (5, 4, 6, [1, 1, 1]),
                                             (2, 160, 32, [70, 3]), (4, 32, 32, [300])])
def test_constant_decay_memory_kernel(dtype, H, dim, vdim, lens):
    """Rows of unequal length that continue from memories in permuted slots; silu inside the scan; decays from 0.3 to 1."""
    g = torch.Generator().manual_seed(dim + vdim)
    T, R = sum(lens), len(lens)
    q, k, v = (torch.randn(T, n, generator=g).to(dtype) for n in (H * dim, H * dim, H * vdim))
    decay = torch.linspace(0.3, 1.0, H) if H > 1 else torch.tensor([0.999])
    state = torch.randn(R + 2, H * vdim * dim + 8, generator=g) * 0.5
    slots = torch.randperm(R + 2, generator=g)[:R].to(torch.int32)
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    out = torch.zeros(T, H, vdim)
    args = [q, k, v, decay, None, state, indptr, slots, out, H, H, dim, vdim, False, 1.0]
    res = _both("decay_scan", args, [8, 5], dict(act="silu"))
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=5e-2)
    for got, want in res:
        torch.testing.assert_close(got, want, **tol)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_norm_over_all_heads_with_a_sigmoid_gate_and_the_small_row_kernels(dtype):
    g = torch.Generator().manual_seed(3)
    for T, n in ((5, 36), (3, 128), (70, 1000), (2, 4100)):
        o = torch.randn(T, n, generator=g)
        gate = torch.randn(T, n + 8, generator=g).to(dtype)[:, 4: n + 4]
        wt = torch.rand(n, generator=g) + 0.5
        out = torch.zeros(T, n + 4, dtype=dtype)[:, :n]
        (got, want), = _both("gla_out", [o, gate, wt, 1e-5, 1.0, out, 1, n], [5], dict(gate_act="sigmoid"))
        torch.testing.assert_close(got, want, **_tol(dtype))
        x = torch.randn(T, n + 6, generator=g)[:, 2: n + 2]
        for xin in (x, x.to(dtype)):
            (got, want), = _both("rms_rows", [xin, wt, 2e-6, torch.zeros(T, n + 8, dtype=dtype)[:, 8:]], [3])
            torch.testing.assert_close(got, want, **_tol(dtype))
        y = torch.randn(T, n, generator=g).to(dtype)
        (got, want), = _both("bias_add", [y, wt], [0])
        torch.testing.assert_close(got, want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("T,H", [(1, 48), (7, 64), (33, 1000), (3, 4096), (5, 130)])
def test_fused_norms_around_the_residual_and_the_normed_sum(dtype, T, H):
    g = torch.Generator().manual_seed(H)
    resid = torch.randn(T, H, generator=g) * 3
    branch = (torch.randn(T, H + 8, generator=g) * 0.2).to(dtype)[:, :H]
    w1, w2 = (torch.rand(H, generator=g) + 0.5 for _ in range(2))
    out = torch.zeros(T, H, dtype=dtype)
    for got, want in _both("branch_norm_add_norm", [resid, branch, w1, 1e-5, w2, 3e-6, out], [0, 6]):
        torch.testing.assert_close(got, want, **_tol(dtype))
    xs = [(torch.randn(T, H, generator=g) * s).to(dtype) for s in (0.1, 4.0, 1.0)]
    ws = [torch.rand(H, generator=g) + 0.5 for _ in range(3)]
    bs = [torch.randn(H, generator=g), None, torch.randn(H, generator=g) * 0.1]
    for n in (1, 2, 3):
        (got, want), = _both("normed_sum", [xs[:n], bs[:n], ws[:n], (0.5, 0.25, 2.0)[:n], 1e-5, torch.zeros(T, H, dtype=dtype)], [5])
        torch.testing.assert_close(got, want, **_tol(dtype))
    (got, want), = _both("normed_sum", [xs[:2], None, ws[:2], (0.5, 0.5), 1e-5, torch.zeros(T, H, dtype=dtype)], [5])
    torch.testing.assert_close(got, want, **_tol(dtype))


def test_routing_by_a_softmax_over_the_chosen():
    g = torch.Generator().manual_seed(5)
    for T, E, top in ((9, 12, 2), (70, 5, 5), (3, 64, 1), (130, 7, 3)):
        z = torch.randn(T, E + 3, generator=g)[:, :E] * 2
        z[0, :2] = z[0].max() + 1.0                          # a tie at the top: the lower index first
        ids, wts = torch.zeros(T, top, dtype=torch.int32), torch.zeros(T, top)
        res = _both("moe_select", [z, None, torch.zeros(T, E + 1), E, top, 1, 1, 1.0, ids, wts], [8, 9], dict(scores="softmax_chosen"))
        assert torch.equal(res[0][0], res[0][1]) and res[0][0][0, 0] == 0 and (top == 1 or res[0][0][0, 1] == 1)
        torch.testing.assert_close(res[1][0], res[1][1], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(res[1][0].sum(-1), torch.ones(T), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("cap", [None, 3.0])
@pytest.mark.parametrize("nq,nkv,hd,ps,window,keep", [(8, 2, 128, 16, 37, 20), (4, 1, 64, 16, 33, 5), (2, 2, 64, 32, 300, 100), (12, 4, 128, 8, 64, 64),
                                                       (4, 4, 64, 16, 40, 0), (4, 2, 128, 16, None, 7), (2, 1, 128, 32, 100, 290), (4, 2, 128, 16, 150, 129),
                                                       (2, 2, 128, 16, 20, 600)])
def test_kept_first_keys_and_capped_scores_in_the_tensor_core_attention_kernels(nq, nkv, hd, ps, window, keep, cap):
    """Prompts on mma.sync and on tcgen05 (kept keys over one, two and several of its 128-key tiles, reaching into the window's
    first tile, and beyond a whole short request) and decoding with split keys (one split and several), with requests shorter than what is kept,
    shorter than the window, and far longer than both: each against the plain statement, which differs from the attention
    without the kept keys, and from the one without the cap, by far more than the tolerance.  The pages that no query can
    see hold poison."""
    import math

    from test_kernels_gpu import _fast_setup

    scale = 4.0 / math.sqrt(hd)

    def want(q, kc, vc, pos, rows, bt, keep_, cap_):
        exp = torch.empty(q.shape[0], nq * hd, dtype=torch.bfloat16)
        kernel_refs.paged_attention(q.cpu(), exp, kc.cpu(), vc.cpu(), pos.cpu(), rows.cpu(), bt.cpu(), nq, nkv, hd, ps, scale, window,
                                    keep_first=keep_, softcap=cap_)
        return exp.float()

    def poison(kc, vc, bt, lens, q_lens):
        if not window:
            return
        for r, (n, ql) in enumerate(zip(lens, q_lens)):
            for p in range(-(-keep // ps), max(0, n - ql - window + 1) // ps):
                kc[bt[r, p]] = 1e3
                vc[bt[r, p]] = float("nan")

    lens, q_lens = [130, 300, 128, 129, 9, 700], [130, 2, 128, 3, 1, 333]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=6)
    poison(kc, vc, bt, lens, q_lens)
    exp = want(q, kc, vc, pos, rows, bt, keep, cap)
    if window and keep:
        assert (exp - want(q, kc, vc, pos, rows, bt, 0, cap)).abs().max() > 0.05
    if cap:
        assert (exp - want(q, kc, vc, pos, rows, bt, keep, None)).abs().max() > 0.05
    for fn in ([ops.paged_attention_prefill_tc] if hd == 128 and ps % 16 == 0 else []) + [ops.paged_attention_prefill]:
        out = torch.zeros(q.shape[0], nq * hd, dtype=torch.bfloat16, device=DEV)
        fn(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, scale, window, max(q_lens), keep_first=keep, softcap=cap)
        ops.check_errors(DEV)
        torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)
    lens = [1, 63, 64, 65, 700, 2049, 17, keep + 1, (window or 50) + keep]
    R = len(lens)
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, [1] * R, seed=3)
    poison(kc, vc, bt, lens, [1] * R)
    exp = want(q, kc, vc, pos, rows, bt, keep, cap)
    for splits in (1, 2, 5):
        out = torch.zeros(R, nq * hd, dtype=torch.bfloat16, device=DEV)
        po, pml = torch.zeros(R * nq * splits * hd, device=DEV), torch.zeros(R * nq * splits * 2, device=DEV)
        ops.paged_attention_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, scale, window, splits, po, pml,
                                   torch.zeros(R * nkv, dtype=torch.int32, device=DEV), keep_first=keep, softcap=cap)
        torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)


# ------------------------------------------------------------------ the engine under every cutting
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("name", ["K1", "K2", "K3", "S"])
def test_cuttings(name, cut, dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    steps = traces.mixed(reqs, seed=4) if cut == "mixed" else getattr(traces, cut)(reqs)
    ps = PAGE_SIZES[name]
    runner = ModelRunner(load_model(d, dtype, DEV), ps, max(1, traces.peak_tokens(steps) // ps), 4, device=DEV)
    got = traces.run_trace(runner, steps)
    ops.check_errors(DEV)
    runner.cache.check()
    assert runner.cache.num_free_slots == 4 and all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups)
    for r, want in oracle.items():
        assert_close(got[r], want, dtype, f"{name} {cut}: request {r}", _rounding[id(oracle)])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_other_page_sizes_and_the_plain_kernel_set(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("K3", tmp_path_factory)
    steps = traces.mixed(reqs, seed=9)
    for ps, ks in ((32, "fast"), (64, "fast"), (16, "plain")):
        runner = ModelRunner(load_model(d, dtype, DEV), ps, max(1, -(-traces.peak_tokens(steps) // ps)), 4, device=DEV, kernel_set=ks)
        got = traces.run_trace(runner, steps)
        for r, want in oracle.items():
            assert_close(got[r], want, dtype, f"pages of {ps}, {ks} kernels, request {r}", _rounding[id(oracle)])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["K1", "K2", "S"])
def test_first_tokens_and_page_borders(name, dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    ps = PAGE_SIZES[name]
    runner = ModelRunner(load_model(d, dtype, DEV), ps, 64, 3, device=DEV)
    toks = [7, 7, 3, 150, 1]
    want = plain.forward(cfg, w, toks)
    rc = _rounding[id(oracle)]
    one_by_one = torch.cat([runner.step([StepEntry("a", [t], (0,))]).clone() for t in toks])
    together = runner.step([StepEntry("b", toks, range(5))]).clone()
    assert_close(one_by_one, want, dtype, "one by one", rc)
    assert_close(together, want, dtype, "together", rc)
    runner.end_request("a"), runner.end_request("b")
    # prompts that end exactly on a page border, one before and one after, then two decoded tokens
    long = traces.make_requests(cfg["vocab"], [4 * ps + 3], seed=2)["r0"]
    want = plain.forward(cfg, w, long)
    for n in (ps - 1, ps, ps + 1, 2 * ps, 4 * ps):
        got = [runner.step([StepEntry("c", long[:n], range(n))]).clone()]
        got += [runner.step([StepEntry("c", [long[n + i]], (0,))]).clone() for i in range(2)]
        assert_close(torch.cat(got), want[: n + 2], dtype, f"prompt of {n}", rc)
        runner.end_request("c")


def _changed(name, tmp_path, change, length, edit_config=None):
    """A tiny model with some tensors (and configuration values) changed: (folder, config, weights, tokens, the plain logits,
    what rounding costs)."""
    d = make_model_dir(name, seed=9, root=str(tmp_path))
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    change(t)
    write_safetensors(path, t)
    cfg, w = read_model(d)
    if edit_config is not None:
        edit_config(cfg)
        with open(os.path.join(d, "config.json"), "w") as fh:
            json.dump(cfg, fh)
    toks = traces.make_requests(cfg["vocab"], [length], seed=3)["r0"]
    want = plain.forward(cfg, w, toks)
    return d, cfg, w, toks, want, rounding_cost(cfg, w, toks, want)


def _run_cut(d, dtype, ps, toks, sizes):
    runner = ModelRunner(load_model(d, dtype, DEV), ps, -(-(len(toks) + 64) // ps), 2, device=DEV)
    got, at = [], 0
    for n in sizes:
        got.append(runner.step([StepEntry("r", toks[at:at + n], range(n))]).clone())
        at += n
    assert at == len(toks)
    return torch.cat(got)


def _scale(t, name, f):
    t[name] = (t[name].float() * f).to(torch.bfloat16)


CUTS_90 = ((90,), (40, 1, 1, 5, 2, 13, 6, 7) + (1,) * 15, (2,) * 10 + (3, 4, 12, 13, 14) + (1,) * 24)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["A", "P"])
def test_keys_at_the_windows_edges_and_the_kept_tokens_decide_the_logits(name, dtype, tmp_path):
    """Random weights make attention nearly uniform, which hides a window that is one token off.  The score scale is raised
    until the softmax picks single keys (A: a window of 6 that keeps 3 tokens; P: the parallel mixer's attention side, a
    window of 7 that keeps 2, scores capped at 4, the other side's share scaled down).  The plain model with the window one
    longer or one shorter, with one kept token more or fewer, or (P) without the cap is far from the plain model at several
    positions, so such a fault would show; the engine is not, in prompts cut at every kind of place and in decoding."""
    def edit(cfg):
        if name == "A":
            cfg["layers"][0]["mixer"]["scale"] = 2.5
        else:
            cfg["layers"][0]["mixer"]["left"].update(scale=6.0, softcap=4.0)

    def side(cfg):
        return cfg["layers"][0]["mixer"] if name == "A" else cfg["layers"][0]["mixer"]["left"]

    change = (lambda t: None) if name == "A" else (lambda t: _scale(t, "l0.mix.right.out", 0.05))
    d, cfg, w, toks, want, rc = _changed(name, tmp_path, change, 90, edit)
    tol = max(REL[dtype] * float(want.std()), 4.5 * rc if dtype == torch.bfloat16 else 0.0)
    for key in ("size", "keep_first"):
        for delta in (1, -1):
            off = copy.deepcopy(cfg)
            side(off)["mask"][key] += delta
            wrong = (plain.forward(off, w, toks) - want).abs().max(dim=-1).values
            assert (wrong > 3 * tol).sum() >= 2, f"{key} off by {delta} would not show"
    if name == "P":
        off = copy.deepcopy(cfg)
        side(off).pop("softcap")
        assert ((plain.forward(off, w, toks) - want).abs().max(dim=-1).values > 3 * tol).sum() >= 2, "scores without the cap would not show"
    for sizes in CUTS_90:
        assert_close(_run_cut(d, dtype, PAGE_SIZES[name], toks, sizes), want, dtype, f"cut {sizes[:4]}", rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_key_decides_the_logits_through_the_latents(dtype, tmp_path):
    """A latent attention that sees every earlier token, sharpened, 330 tokens over many pages: late logits depend on single far
    tokens through the cached latents alone (the first layer's mixer is scaled down by its output norm's weight)."""
    d, cfg, w, toks, want, rc = _changed("F", tmp_path, lambda t: _scale(t, "l0.norm1b", 0.05), 330,
                                         lambda cfg: cfg["layers"][1]["mixer"].update(scale=5.0))
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab"]
    effect = (plain.forward(cfg, w, moved)[200:] - want[200:]).abs().max().item() / float(want.std())
    assert effect > 1e-2, "the sharpened layer does not look far back"
    assert_close(_run_cut(d, dtype, PAGE_SIZES["F"], toks, (130, 1, 1, 64, 2, 99, 1, 1) + (1,) * 31), want, dtype, "far", rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_token_lives_on_in_the_memories(dtype, tmp_path):
    """Decays of 0.999 and 1: the memories keep what the first tokens wrote for hundreds of steps; the attention sides'
    shares are scaled down.  A memory that is lost, reset or mixed up between steps shows."""
    def change(t):
        _scale(t, "l0.mix.left.out", 0.02)
        _scale(t, "l1.mix.left.out", 0.02)
    d, cfg, w, toks, want, rc = _changed("S", tmp_path, change, 250)
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab"]
    effect = (plain.forward(cfg, w, moved)[200:] - want[200:]).abs().max().item() / float(want.std())
    assert effect > 1e-2, "the memories do not remember far tokens"
    assert_close(_run_cut(d, dtype, PAGE_SIZES["S"], toks, (100, 1, 1, 64, 2, 49, 1, 1) + (1,) * 31), want, dtype, "state", rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_keeps_cache_and_states_exact(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("K1", tmp_path_factory)
    toks = traces.make_requests(cfg["vocab"], [320], seed=8)["r0"]
    want = plain.forward(cfg, w, toks)
    runner = ModelRunner(load_model(d, dtype, DEV), 4, 80, 2, device=DEV)         # pages of four: the windows' pages turn over, the first stay
    got = [runner.step([StepEntry("r", toks[:20], range(20))]).clone()]
    got += [runner.step([StepEntry("r", [t], (0,))]).clone() for t in toks[20:]]
    held = [g.pool.num_pages - g.pool.num_free for g in runner.cache.groups]
    assert held == [3, 80, 3]                    # a first page and the two pages under the window; every latent
    assert_close(torch.cat(got), want, dtype, "300 decoded tokens", rounding_cost(cfg, w, toks, want))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_request_that_starts_again(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("S", tmp_path_factory)
    steps = traces.preempted(reqs)
    ps = PAGE_SIZES["S"]
    runner = ModelRunner(load_model(d, dtype, DEV), ps, traces.peak_tokens(steps) // ps, 3, device=DEV)
    for rid, pos, row in traces.run_trace_by_position(runner, steps):
        assert_close(row[None], oracle[rid][pos][None], dtype, f"{rid} at {pos}", _rounding[id(oracle)])


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("graph", [True, False], ids=["graphs", "eager"])
@pytest.mark.parametrize("name", ["F", "K1", "S"])
def test_greedy_generation_equals_plain_model_f32(name, graph, tmp_path):
    d = make_model_dir(name, seed=3, root=str(tmp_path), sigma=0.3)
    cfg, w = read_model(d)
    prompts = [[5, 17, 3, 150, 9, 1, 1, 44, 102, 7, 7], [42] * 19, [7], list(range(20, 61))]
    ref = [plain.generate_greedy(cfg, w, p, 12) for p in prompts]
    assert all(len(set(r)) >= 3 for r in ref), "the continuation is too uniform to test anything"
    ps = PAGE_SIZES[name]
    for pages in (256 // ps, 112 // ps):                     # plenty; and (for the long window) so few that a request is preempted
        eng = Engine(d, dtype="float32", device=DEV, page_size=ps, num_pages=pages, num_slots=3, chunked_prefill_size=16,
                     max_num_batched_tokens=32, cuda_graph=graph)
        outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
        assert [o.token_ids for o in outs] == ref, f"{pages} pages"
        assert not graph or eng.runner.graph_steps > 0
        eng.runner.cache.check()


def test_greedy_generation_bf16_stays_on_the_plain_models_best(tmp_path):
    """bfloat16 through the engine with CUDA graphs: every generated token is, for the plain model, the best token or within
    what rounding costs of it; and a captured step gives the tokens the same step gives when it is launched kernel by kernel."""
    d = make_model_dir("S", seed=3, root=str(tmp_path), sigma=0.2)
    cfg, w = read_model(d)
    prompts = [traces.make_requests(cfg["vocab"], [n], seed=n)["r0"] for n in (40, 3, 90, 9, 77)]
    eng = Engine(d, dtype="bfloat16", device=DEV, page_size=16, num_pages=40, num_slots=4)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    assert eng.runner.graph_steps > 0
    for p, o in zip(prompts, outs):
        toks = list(p) + o.token_ids
        lg = plain.forward(cfg, w, toks[:-1])
        slack = max(0.06 * float(lg.std()), 3 * rounding_cost(cfg, w, toks[:-1], lg))
        for i in range(len(p) - 1, len(toks) - 1):
            assert lg[i][toks[i + 1]] >= lg[i].max() - slack, (len(p), i)
    d = make_model_dir("K3", seed=3, root=str(tmp_path))
    prompts = [traces.make_requests(512, [n], seed=n)["r0"] for n in (40, 3, 90, 9)]
    tokens = []
    for graph in (True, False):
        eng = Engine(d, dtype="bfloat16", device=DEV, page_size=16, num_pages=40, num_slots=4, cuda_graph=graph)
        tokens.append([o.token_ids for o in eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))])
        assert (eng.runner.graph_steps > 0) == graph
    assert tokens[0] == tokens[1]


# ------------------------------------------------------------------ the tools
def test_replay_tool_and_command_line(tmp_path_factory, tmp_path):
    d, cfg, w, reqs, oracle = model_and_oracle("K2", tmp_path_factory)
    steps = traces.mixed(reqs, seed=11)
    out_dir = str(tmp_path / "out")
    p = subprocess.Popen([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out_dir, "--max-tokens",
                          str(traces.peak_tokens(steps))], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=ROOT)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            assert p.stdout.readline().strip() == f"done {s['step']}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    at = {r: 0 for r in reqs}
    for s in steps:
        rows = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        k = 0
        for e in s["entries"]:
            n = len(e["want"])
            assert_close(torch.from_numpy(rows[k:k + n].copy()), oracle[e["id"]][at[e["id"]]: at[e["id"]] + n], torch.float32, e["id"])
            at[e["id"]] += n
            k += n
    ref = plain.generate_greedy(cfg, w, [5, 6, 7, 8], 6)
    r = subprocess.run([sys.executable, "-m", "arle_b200", "--model-path", d, "--dtype", "float32", "--max-tokens", "6", "--ignore-eos",
                        "--num-slots", "2", "--num-pages", "16", "run", "--prompt", "5 6 7 8", "--json"], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout)["outputs"][0]["token_ids"] == ref
