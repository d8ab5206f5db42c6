"""Lasupel on the GPU against the plain implementation (``plain_lasupel``): every new kernel alone at sizes of no model
(rows of unequal length that continue from states in permuted slots, windows and page borders, values wider and narrower
than keys, the sink, routing on made-up scores), the engine under every cutting in float32 and bfloat16 on tiny
configurations, the first tokens of a sequence and prompts that end on page borders, keys just inside and just outside
a window and far keys made to decide the logits (sharpened attention), far tokens living on in the recurrent states (decays
next to one), long decoding, a request that starts again, greedy generation through the public entry point with CUDA
graphs and preemption, and the replay tool and the command line as subprocesses."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kernel_refs
import plain_lasupel as plain
import traces
from arle_b200 import Engine, ops
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.sampling import SamplingParams
from arle_b200.weights import SafetensorsFile, write_safetensors
from tiny_lasupel import CONFIGS, PAGE_SIZES, make_model_dir, read_model

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
LENGTHS = {"L1": [1, 5, 12, 23, 70, 130, 33], "L2": [2, 17, 40, 96, 64, 31], "L3": [3, 66, 150, 64, 40, 97], "S": [2, 33, 80, 17, 64],
           "A": [3, 50, 64, 29], "R": [1, 40, 33, 7, 70]}
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
    cpu = [a.clone() if isinstance(a, torch.Tensor) else a for a in args]
    gpu = [a.to(DEV) if isinstance(a, torch.Tensor) else a for a in args]
    getattr(ops, fn)(*gpu, **(kwargs or {}))
    getattr(kernel_refs, fn)(*cpu, **(kwargs or {}))
    torch.cuda.synchronize()
    return [(gpu[i].float().cpu(), cpu[i].float()) for i in outs]


def _rows(g, starts, lens, ps, extra_pages=5):
    """Three rows in scattered pages: positions, row of token, block table, slots of the step's tokens, q_indptr."""
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
def test_branch_norm_add_kernel(dtype):
    g = torch.Generator().manual_seed(0)
    for H in (48, 51, 100, 256, 4096):
        resid = torch.randn(7, H, generator=g) * 3
        branch = (torch.randn(7, H + 8, generator=g) * 5).to(dtype)[:, :H]                 # a view of wider rows
        w = torch.rand(H, generator=g) + 0.5
        copy_ = torch.zeros(7, H, dtype=dtype)
        for (a, c) in _both("branch_norm_add", [resid, branch, w, 1e-5, copy_], [0, 4]):
            torch.testing.assert_close(a, c, **_tol(dtype))
        for (a, c) in _both("branch_norm_add", [resid, None, None, 0.0, copy_], [0, 4]):    # the copy alone
            torch.testing.assert_close(a, c, **_tol(dtype))
        for (a, c) in _both("branch_norm_add", [resid, branch, w, 1e-5, None], [0]):
            torch.testing.assert_close(a, c, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nq,nkv,hd,vd,rdim,window,ps,sink", [(4, 2, 16, 24, 8, 7, 4, 0.0), (1, 1, 12, 40, 12, 0, 8, 0.0), (6, 2, 8, 4, 0, 1, 16, 0.0),
                                                                (8, 2, 64, 64, 32, 48, 16, 0.0), (2, 1, 128, 128, 128, 33, 16, 0.7),
                                                                (6, 3, 96, 256, 40, 300, 32, None), (3, 3, 256, 8, 64, 129, 8, -1.5)])
def test_preparation_and_attention_with_sink_and_value_width(dtype, nq, nkv, hd, vd, rdim, window, ps, sink):
    """Three rows of unequal length in scattered pages: a portion that continues a request, a decoded token far into its
    request, a fresh prompt.  Rotation first, then the norm without a weight (and with one); keys of width hd and values
    of width vd in caches of their own shapes; the softmax with the sink's term."""
    g = torch.Generator().manual_seed(nq * 7 + hd)
    starts, lens = [37, 700, 0], [23, 1, 41]
    T = sum(lens)
    pages, bt, pos, row, slots, _ = _rows(g, starts, lens, ps)
    qkv = torch.randn(T, nq * hd + nkv * (hd + vd) + 3, generator=g).to(dtype)
    inv = (10000.0 ** (-2.0 * torch.arange(rdim // 2, dtype=torch.float64) / max(rdim, 1))).float()
    kc, vc = (torch.randn(pages, nkv, ps, hd, generator=g) * 0.7).to(dtype), (torch.randn(pages, nkv, ps, vd, generator=g) * 0.7).to(dtype)
    for qw, kw, eps in ((None, None, 1e-5), (torch.rand(hd, generator=g) + 0.5, torch.rand(hd, generator=g) + 0.5, 1e-6), (None, None, None)):
        res = _both("attention_prep_post", [qkv, pos, slots, qw, kw, eps, inv if rdim else None, rdim, kc, vc, nq, nkv, hd, vd, ps], [0, 8, 9])
        for (a, c) in res:
            torch.testing.assert_close(a, c, **_tol(dtype))
    (qa, qc), (ka, kcc), (va, vcc) = res[0], res[1], res[2]
    only_q = qkv[:, : nq * hd].clone()
    for (a, c) in _both("attention_prep_post", [only_q, pos, None, None, None, 1e-5, inv if rdim else None, rdim, None, None, nq, 0, hd, vd, ps], [0]):
        torch.testing.assert_close(a, c, **_tol(dtype))
    # attention over what the reference left in the caches (unit-RMS keys from the first pass would make all scores tiny)
    q = (qc[:, : nq * hd] * 2.0).to(dtype)
    out = torch.zeros(T, nq * vd, dtype=dtype)
    for (a, c) in _both("paged_attention", [q, out, kcc.to(dtype), vcc.to(dtype), pos, row, bt, nq, nkv, hd, ps, 0.4 * hd ** -0.5, window or None],
                        [1], dict(vd=vd, sink=sink)):
        torch.testing.assert_close(a, c, **_tol(dtype))
    if sink is not None:           # the sink takes weight: the rows' weights sum to less than one, so outputs shrink against the usual softmax
        plain_out = torch.zeros(T, nq * vd, dtype=dtype)
        kernel_refs.paged_attention(q, plain_out, kcc.to(dtype), vcc.to(dtype), pos, row, bt, nq, nkv, hd, ps, 0.4 * hd ** -0.5, window or None, vd=vd)
        assert (plain_out.float() - c).abs().max() > 1e-2


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("C,taps,out_f32,pad,at", [(48, 3, True, 5, 2), (130, 4, False, 5, 2), (7, 2, True, 5, 2), (256, 5, False, 5, 2),
                                                     (33, 1, True, 5, 2), (48, 3, True, 16, 8), (256, 4, False, 24, 16), (1032, 2, False, 8, 0),
                                                     (8, 1, True, 8, 8)])
def test_causal_conv_kernel(dtype, C, taps, out_f32, pad, at):
    """Rows shorter than the taps reach back into the state; a second call continues from the state the first one left; an
    input bias is added to the request's tokens and not to the zeros before them.  The channels are views into wider rows,
    at odd places and on 16-byte boundaries."""
    g = torch.Generator().manual_seed(C)
    lens = [1, 2, 9, 1, 30]
    T = sum(lens)
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    row = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to(torch.int32)
    slots = torch.tensor([4, 0, 6, 2, 5], dtype=torch.int32)
    off = 11
    state = torch.zeros(8, off + C * max(taps - 1, 0) + 3)
    state[:, :off] = 7.0
    w, ib, ob = torch.randn(C, taps, generator=g), torch.randn(C, generator=g), torch.randn(C, generator=g)
    for act, in_bias, out_bias in (("none", ib, ob), ("silu", None, None), ("silu", ib, None)):
        st_gpu, st_cpu = state.clone().to(DEV), state.clone()
        for call in range(2):
            wide = torch.randn(T, C + pad, generator=g).to(dtype)
            x = wide[:, at: at + C]
            out = torch.zeros(T, C, dtype=torch.float32 if out_f32 else dtype)
            gpu_out = out.to(DEV)
            ops.causal_conv(wide.to(DEV)[:, at: at + C], in_bias.to(DEV) if in_bias is not None else None, w.to(DEV), out_bias.to(DEV) if out_bias is not None else None,
                            act, st_gpu, off, indptr.to(DEV), row.to(DEV), slots.to(DEV), gpu_out)
            kernel_refs.causal_conv(x, in_bias, w, out_bias, act, st_cpu, off, indptr, row, slots, out)
            torch.testing.assert_close(gpu_out.float().cpu(), out.float(), **_tol(dtype))
            torch.testing.assert_close(st_gpu.cpu(), st_cpu, **_tol(torch.float32))
        assert (st_cpu[[1, 3, 7]] == state[[1, 3, 7]]).all() and (st_cpu[:, :off] == 7.0).all()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width,blocks,lens", [(48, 3, [1, 5, 70]), (40, 1, [300, 1, 2]), (256, 4, [33, 1, 9, 1]), (56, 7, [1, 1, 1]), (72, 2, [256, 257, 700, 3])])
def test_rglru_scan_kernel(dtype, width, blocks, lens):
    """Rows of unequal length from states in permuted slots; long rows run in segments whose states are chained; a second
    call continues.  Some decays are next to one (lam far below zero) so that a lost state would show."""
    g = torch.Generator().manual_seed(width)
    T = sum(lens)
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    slots = torch.randperm(6, generator=g)[: len(lens)].to(torch.int32)
    lam = torch.randn(width, generator=g)
    lam[::3] = -9.0
    br, bi, yb = torch.randn(width, generator=g), torch.randn(width, generator=g), torch.randn(width, generator=g) * 0.2
    state = torch.randn(6, width + 9, generator=g)
    st_gpu, st_cpu = state.clone().to(DEV), state.double()                 # the statement runs in float64
    for call in range(2):
        z, u = torch.randn(T, 2 * width, generator=g), torch.randn(T, width, generator=g).to(dtype)
        y = torch.randn(T, width + 3, generator=g).to(dtype)[:, :width]
        out = torch.zeros(T, width, dtype=torch.float64)
        gpu_out = torch.zeros(T, width, dtype=dtype, device=DEV)
        ops.rglru_scan(z.to(DEV), u.to(DEV), y.to(DEV), br.to(DEV), bi.to(DEV), lam.to(DEV), yb.to(DEV), 8.0, st_gpu, indptr.to(DEV),
                       slots.to(DEV), gpu_out, blocks, max(lens))
        kernel_refs.rglru_scan(z.double(), u, y, br.double(), bi.double(), lam.double(), yb.double(), 8.0, st_cpu, indptr, slots, out, blocks, max(lens))
        torch.testing.assert_close(gpu_out.double().cpu(), out, **_tol(dtype))
        torch.testing.assert_close(st_gpu.double().cpu(), st_cpu, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("kernels", ["fast", "plain"])
@pytest.mark.parametrize("M,blocks,bs", [(1, 3, 16), (70, 4, 64), (9, 7, 8), (260, 2, 136), (5, 1, 40)])
def test_gate_sums_of_bfloat16_rows_stay_float32(M, blocks, bs, kernels):
    """The block-diagonal product behind the RG-LRU's gates reads bfloat16 rows and matrices and leaves its float32 sums
    unrounded: against float64, far closer than a bfloat16 rounding of the result would be."""
    g = torch.Generator().manual_seed(M + bs)
    u = torch.randn(M, blocks * bs, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(blocks, 2 * bs, bs, generator=g) * bs ** -0.5).to(torch.bfloat16).to(DEV)
    z = torch.zeros(M, 2 * blocks * bs, dtype=torch.float32, device=DEV)
    with ops.use_kernel_set(kernels):
        ops.gemm_heads(u.view(M, blocks, bs), w, z.view(M, blocks, 2 * bs))
    want = torch.einsum("mhk,hnk->mhn", u.double().cpu().view(M, blocks, bs), w.double().cpu()).reshape(M, -1)
    torch.testing.assert_close(z.double().cpu(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("H,G,dim,vdim,lens", [(4, 2, 8, 12, [1, 5, 40]), (3, 3, 20, 8, [18, 1, 2]), (8, 4, 64, 128, [33, 1, 9]),
                                               (2, 2, 160, 32, [1, 20, 1]), (2, 1, 300, 70, [3, 1, 17]), (4, 2, 128, 128, [40, 1, 1]),
                                               (40, 20, 32, 96, [1, 1, 19, 1, 1, 1]), (2, 1, 100, 33, [50])])
def test_delta_rule_kernels(dtype, H, G, dim, vdim, lens):
    g = torch.Generator().manual_seed(H * 5 + dim)
    T = sum(lens)
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    slots = torch.randperm(7, generator=g)[: len(lens)].to(torch.int32)
    pre = torch.randn(T, 2 * H + 3, generator=g)
    a_log, dtb = torch.randn(H, generator=g) * 0.5 - 1.0, torch.randn(H, generator=g)
    beta, decay = torch.zeros(T, H), torch.zeros(T, H)
    res = _both("delta_gates", [pre, a_log, dtb, beta, decay], [3, 4])
    for (a, c) in res:
        torch.testing.assert_close(a, c, rtol=1e-5, atol=1e-6)
    beta, decay = res[0][1], res[1][1]
    state = torch.randn(7, H * vdim * dim + 6, generator=g) * 0.3
    st_gpu, st_cpu = state.clone().to(DEV), state.clone()
    for call in range(2):
        q, k = torch.randn(T, G * dim + 4, generator=g).to(dtype)[:, : G * dim], torch.randn(T, G * dim, generator=g).to(dtype)
        v = torch.randn(T, H * vdim, generator=g).to(dtype)
        out = torch.zeros(T, H, vdim)
        gpu_out = out.to(DEV)
        ops.delta_scan(q.to(DEV), k.to(DEV), v.to(DEV), beta.to(DEV), decay.to(DEV), st_gpu, indptr.to(DEV), slots.to(DEV), gpu_out, H, G, dim,
                       vdim, dim ** -0.5, 1e-6)
        kernel_refs.delta_scan(q, k, v, beta, decay, st_cpu, indptr, slots, out, H, G, dim, vdim, dim ** -0.5, 1e-6)
        torch.testing.assert_close(gpu_out.cpu(), out, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(st_gpu.cpu(), st_cpu, rtol=1e-4, atol=1e-4)


def test_routing_and_clamped_experts_kernels():
    """The selection on made-up scores (a group counts by its best expert alone; the weights are the softmax scores) and at
    random against the plain rules; the clamped gate on values around its limits."""
    s = torch.tensor([[0.05, 0.30, 0.17, 0.16, 0.18, 0.01, 0.02, 0.11]])
    z = torch.log(s).to(DEV)
    ids, wts = torch.zeros(1, 3, dtype=torch.int32, device=DEV), torch.zeros(1, 3, device=DEV)
    ops.moe_select(z, None, torch.zeros(1, 12, device=DEV), 8, 3, 4, 2, 1.0, ids, wts, scores="softmax", group_score="max")
    assert sorted(ids[0].tolist()) == [0, 1, 4] and abs(float(wts.sum()) - 0.53) < 1e-5
    ops.moe_select(z, None, torch.zeros(1, 12, device=DEV), 8, 3, 4, 2, 1.0, ids, wts, scores="softmax", group_score="top2_sum")
    assert sorted(ids[0].tolist()) == [1, 2, 3]                                           # by two-best sums group 1 beats group 2
    g = torch.Generator().manual_seed(3)
    for E, top, count, keep in ((6, 2, 3, 2), (8, 4, 8, 5), (16, 3, 2, 1), (3, 1, 1, 1), (64, 6, 8, 3)):
        zz = torch.randn(50, E + 2, generator=g) * 2
        ids, wts = torch.zeros(50, top, dtype=torch.int32), torch.zeros(50, top)
        (ia, ic), (wa, wc) = _both("moe_select", [zz, None, torch.zeros(50, E + count), E, top, count, keep, 1.0, ids, wts], [8, 9],
                                   dict(scores="softmax", group_score="max"))
        want_i, want_w = plain.route(zz[:, :E].double(), top, count, keep)
        assert (ia.sort(-1).values == ic.sort(-1).values).all() and (ia.sort(-1).values.long() == want_i.sort(-1).values).all()
        torch.testing.assert_close(wa.sort(-1).values, want_w.float().sort(-1).values, rtol=1e-5, atol=1e-6)
    for dtype in DTYPES:
        for inter, wide in ((40, 44), (37, 41), (256, 256)):          # four results a thread, and one
            gu = (torch.randn(9, 2 * inter, generator=g) * 2).to(dtype)
            out_gpu = torch.zeros(9, wide, dtype=dtype, device=DEV)
            ops.clamped_glu(gu.to(DEV), out_gpu[:, :inter], 1.3, 1.702)
            gate, up = gu[:, 0::2].double().clamp(max=1.3), gu[:, 1::2].double().clamp(-1.3, 1.3)
            torch.testing.assert_close(out_gpu[:, :inter].double().cpu(), gate * torch.sigmoid(1.702 * gate) * (up + 1), **_tol(dtype))
            assert float(out_gpu[:, inter:].abs().sum()) == 0.0
            c = torch.zeros(9, inter, dtype=dtype)
            kernel_refs.clamped_glu(gu, c, 1.3, 1.702)
            torch.testing.assert_close(out_gpu[:, :inter].float().cpu(), c.float(), **_tol(dtype))


@pytest.mark.parametrize("sink", [0.0, 1.5, -2.0])
@pytest.mark.parametrize("nq,nkv,hd,ps,window", [(8, 2, 128, 16, None), (12, 4, 128, 16, 37), (4, 1, 64, 16, 33), (2, 2, 64, 32, 300)])
def test_the_sink_in_the_tensor_core_attention_kernels(nq, nkv, hd, ps, window, sink):
    """The sink is one more term at the end of every fast kernel's sums (prompts on mma.sync and on tcgen05, decoding with
    split keys and streaming, with and without pieces to merge): each against the plain statement, which differs from the
    usual softmax by far more than the tolerance."""
    import math

    from test_kernels_gpu import _fast_setup

    scale = 2.0 / math.sqrt(hd)

    def want(q, kc, vc, pos, rows, bt, sink_):
        exp = torch.empty(q.shape[0], nq * hd, dtype=torch.bfloat16)
        kernel_refs.paged_attention(q.cpu(), exp, kc.cpu(), vc.cpu(), pos.cpu(), rows.cpu(), bt.cpu(), nq, nkv, hd, ps, scale, window, sink=sink_)
        return exp.float()

    lens, q_lens = [130, 300, 128, 129, 9, 700], [130, 2, 128, 3, 1, 333]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=6)
    exp = want(q, kc, vc, pos, rows, bt, sink)
    assert (exp - want(q, kc, vc, pos, rows, bt, None)).abs().max() > 0.05
    for fn in ([ops.paged_attention_prefill_tc] if hd == 128 else []) + [ops.paged_attention_prefill]:
        out = torch.zeros(q.shape[0], nq * hd, dtype=torch.bfloat16, device=DEV)
        fn(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, scale, window, max(q_lens), sink=sink)
        ops.check_errors(DEV)
        torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)
    lens = [1, 63, 64, 65, 700, 2049, 17]
    R = len(lens)
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, [1] * R, seed=3)
    exp = want(q, kc, vc, pos, rows, bt, sink)
    for splits in (1, 5):
        out = torch.zeros(R, nq * hd, dtype=torch.bfloat16, device=DEV)
        po, pml = torch.zeros(R * nq * splits * hd, device=DEV), torch.zeros(R * nq * splits * 2, device=DEV)
        ops.paged_attention_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, scale, window, splits, po, pml,
                                   torch.zeros(R * nkv, dtype=torch.int32, device=DEV), sink=sink)
        torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)
    for ctas in (3, 148):
        slots = (ctas + R * nkv) * (nq // nkv)
        out = torch.zeros(R, nq * hd, dtype=torch.bfloat16, device=DEV)
        ops.paged_attention_decode_stream(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, scale, window, torch.zeros(slots * hd, device=DEV),
                                          torch.zeros(slots * 2, device=DEV), torch.zeros(R * nkv, dtype=torch.int32, device=DEV), ctas, sink=sink)
        ops.check_errors(DEV)
        torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)


# ------------------------------------------------------------------ the engine
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("name", ["L1", "L2", "L3", "R"])
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
    d, cfg, w, reqs, oracle = model_and_oracle("L3", tmp_path_factory)
    steps = traces.mixed(reqs, seed=9)
    for ps, ks in ((32, "fast"), (64, "fast"), (16, "plain")):
        runner = ModelRunner(load_model(d, dtype, DEV), ps, max(1, -(-traces.peak_tokens(steps) // ps)), 4, device=DEV, kernel_set=ks)
        got = traces.run_trace(runner, steps)
        for r, want in oracle.items():
            assert_close(got[r], want, dtype, f"pages of {ps}, {ks} kernels, request {r}", _rounding[id(oracle)])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["L1", "L2", "S"])
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


def _changed(name, tmp_path, change, length):
    """A tiny model with some tensors changed: (folder, config, weights, tokens, the plain logits, what rounding costs)."""
    d = make_model_dir(name, seed=9, root=str(tmp_path))
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    change(t)
    write_safetensors(path, t)
    cfg, w = read_model(d)
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


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("which,score_scale", [(0, 40.0), (1, 40.0)])
def test_keys_at_the_windows_edges_decide_the_logits(which, score_scale, dtype, tmp_path):
    """Random weights make attention nearly uniform, which hides a window that is one token off.  Queries and keys have unit
    root mean square here whatever their matrices, so one layer's score scale is raised instead until its softmax picks
    single keys (windows of 6 and 13, the second over the first layer's keys: the picked key is the oldest visible one every
    few positions).  The plain model with that window one longer or one shorter is far from the plain model at several
    positions, so such a fault would show; the engine is not, in prompts cut at every kind of place and in decoding."""
    d, cfg, w, toks, want, rc = _changed("A", tmp_path, lambda t: None, 90)
    cfg["layers"][which]["mixer"]["scale"] = score_scale / 16
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    want = plain.forward(cfg, w, toks)
    rc = rounding_cost(cfg, w, toks, want)
    tol = max(REL[dtype] * float(want.std()), 4.5 * rc if dtype == torch.bfloat16 else 0.0)
    for delta in (1, -1):
        off = copy.deepcopy(cfg)
        off["layers"][which]["mixer"]["mask"]["size"] += delta
        wrong = (plain.forward(off, w, toks) - want).abs().max(dim=-1).values
        assert (wrong > 3 * tol).sum() >= 2, "a window that is one off would not show"
    nosink = (_no_sink_forward(cfg, w, toks) - want).abs().max(dim=-1).values
    assert (nosink > 3 * tol).sum() >= 1, "a softmax without the sink's term would not show"
    for sizes in ((90,), (40, 1, 1, 5, 2, 13, 6, 7) + (1,) * 15, (2,) * 10 + (3, 4, 12, 13, 14) + (1,) * 24):
        assert_close(_run_cut(d, dtype, PAGE_SIZES["A"], toks, sizes), want, dtype, f"cut {sizes[:4]}", rc)


def _no_sink_forward(cfg, w, toks):
    """The plain model with the usual softmax in its attention (what an engine that left the sink out would compute)."""
    real = plain.attention

    def usual(h, W, p, m, eps, kv, rnd=plain._ident):
        T, H, G, dv = h.shape[0], m["heads"], m["kv_heads"], m["vdim"]
        q = plain.rms_unit(plain.rotate_first_dims(plain.lin(W[p + "q"], h).view(T, H, m["dim"]), torch.arange(T), m["rot"]["base"], m["rot"]["dims"]), eps)
        k, v = kv
        out = torch.zeros(T, H, dv, dtype=torch.float64)
        for t in range(T):
            lo = max(0, t - m["mask"]["size"] + 1)
            for hh in range(H):
                g = hh // (H // G)
                out[t, hh] = torch.softmax((k[lo: t + 1, g] @ q[t, hh]) * m["scale"], 0) @ v[lo: t + 1, g]
        return plain.lin(W[p + "o"], out.reshape(T, H * dv))

    plain.attention = usual
    try:
        return plain.forward(cfg, w, toks)
    finally:
        plain.attention = real


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_key_decides_the_logits(dtype, tmp_path):
    """A window longer than the sequence, a sharpened softmax, 330 tokens over many pages: late logits depend on single far
    tokens through the attention alone (the recurrent layer's branch is scaled down by its output norm's weight)."""
    d, cfg, w, toks, want, rc = _changed("F", tmp_path, lambda t: _scale(t, "l1.norm1", 0.05), 330)
    cfg["layers"][0]["mixer"]["scale"] = 2.0
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    want = plain.forward(cfg, w, toks)
    rc = rounding_cost(cfg, w, toks, want)
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab"]
    effect = (plain.forward(cfg, w, moved)[200:] - want[200:]).abs().max().item() / float(want.std())
    assert effect > 1e-2, "the sharpened layer does not look far back"
    assert_close(_run_cut(d, dtype, PAGE_SIZES["F"], toks, (130, 1, 1, 64, 2, 99, 1, 1) + (1,) * 31), want, dtype, "far", rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_token_lives_on_in_the_states(dtype, tmp_path):
    """Decays next to one (lam and A_log far below zero) and small write strengths: the states keep what the first tokens
    wrote for hundreds of steps; the attention layer's branch is scaled down.  A state that is lost, reset or mixed up
    between steps shows."""
    def change(t):
        t["l0.mix.lam"] = torch.full_like(t["l0.mix.lam"], -9.0)
        t["l1.mix.A_log"] = torch.full_like(t["l1.mix.A_log"], -7.0)
        t["l1.mix.b"] = torch.zeros_like(t["l1.mix.b"])
        _scale(t, "l2.norm1", 0.02)
    d, cfg, w, toks, want, rc = _changed("S", tmp_path, change, 250)
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab"]
    effect = (plain.forward(cfg, w, moved)[200:] - want[200:]).abs().max().item() / float(want.std())
    assert effect > 1e-2, "the states do not remember far tokens"
    assert_close(_run_cut(d, dtype, PAGE_SIZES["S"], toks, (100, 1, 1, 64, 2, 49, 1, 1) + (1,) * 31), want, dtype, "state", rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_keeps_cache_and_states_exact(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("L1", tmp_path_factory)
    toks = traces.make_requests(cfg["vocab"], [320], seed=8)["r0"]
    want = plain.forward(cfg, w, toks)
    runner = ModelRunner(load_model(d, dtype, DEV), 4, 10, 2, device=DEV)         # ten pages of four: the window's pages turn over
    got = [runner.step([StepEntry("r", toks[:20], range(20))]).clone()]
    got += [runner.step([StepEntry("r", [t], (0,))]).clone() for t in toks[20:]]
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
@pytest.mark.parametrize("name", ["F", "L1", "R"])
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
    d = make_model_dir("L3", seed=3, root=str(tmp_path))
    prompts = [traces.make_requests(512, [n], seed=n)["r0"] for n in (40, 3, 90, 9)]
    tokens = []
    for graph in (True, False):
        eng = Engine(d, dtype="bfloat16", device=DEV, page_size=16, num_pages=40, num_slots=4, cuda_graph=graph)
        tokens.append([o.token_ids for o in eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))])
        assert (eng.runner.graph_steps > 0) == graph
    assert tokens[0] == tokens[1]


# ------------------------------------------------------------------ the tools
def test_replay_tool_and_command_line(tmp_path_factory, tmp_path):
    d, cfg, w, reqs, oracle = model_and_oracle("L2", tmp_path_factory)
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
