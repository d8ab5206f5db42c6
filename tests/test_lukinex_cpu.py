"""Lukinex without a GPU: the configuration reader and what it refuses, the model as the registry builds it (latent layers
that read another layer's latents, a cache that keeps a request's first pages, two states in one row), the plain
implementation's own checks (each mechanism against its sum written out or on made-up inputs), and the engine around the
kernels (cache pages, state slots, step function, scheduler) under every way of cutting the work, with the kernels
replaced by their torch statements."""
import copy
import math

import pytest
import torch

import plain_lukinex as plain
import traces
from arle_b200 import Engine
from arle_b200.cache import CacheManager
from arle_b200.config import ConfigError, LukinexConfig, config_from_dict
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.parts import CacheNeed, build_model
from arle_b200.sampling import SamplingParams
from tiny_lukinex import CONFIGS, PAGE_SIZES, make_model_dir, read_model

LENGTHS = {"K1": [1, 5, 12, 23, 70, 33], "K2": [2, 17, 40, 64, 9, 31], "S": [3, 30, 11, 2, 45], "P": [1, 20, 33, 7]}
F64 = torch.float64
_cache = {}


def model_and_oracle(name, tmp_path_factory):
    if name not in _cache:
        d = make_model_dir(name, seed=21, root=str(tmp_path_factory.mktemp(f"tiny{name}")))
        cfg, w = read_model(d)
        reqs = traces.make_requests(cfg["vocab"], LENGTHS[name], seed=6)
        _cache[name] = (d, cfg, w, reqs, {r: plain.forward(cfg, w, t) for r, t in reqs.items()})
    return _cache[name]


# ------------------------------------------------------------------ configuration
def test_registry_finds_the_architecture_and_reads_every_size():
    cfg = config_from_dict(CONFIGS["K1"])
    assert isinstance(cfg, LukinexConfig) and [l.type for l in cfg.layers] == ["attention", "latent_attention", "latent_attention", "parallel"]
    a, lat, reader, par = cfg.layers
    assert (a.m("window"), a.m("keep_first"), a.m("vdim"), a.m("rot_dims"), a.m("rot_divide")) == (7, 3, 24, 8, 4.0)
    assert reader.m("kv_from") == 1 and lat.m("kv_from") is None and reader.mlp is None and (lat.m("q_rank"), lat.m("kv_rank")) == (28, 20)
    assert (par.m("left.conv"), par.m("left.softcap"), par.m("left.keep_first"), par.m("right.decay")) == (3, 5.0, 2, (0.6, 0.9, 0.999))
    assert (a.mlp.experts, a.mlp.top, a.mlp.limit, a.mlp.shared_ff, a.mlp.shared_limit) == (6, 2, 1.2, 24, 0.8) and lat.mlp.shared_ff == 0
    assert cfg.norm_eps == 1e-5
    k2 = config_from_dict(CONFIGS["K2"])
    assert k2.layers[1].m("window") is None and k2.layers[1].m("rot_divide") == 1.0 and k2.layers[0].m("left.softcap") is None


def test_model_spec_shares_latents_keeps_first_pages_and_packs_two_states():
    spec = config_from_dict(CONFIGS["K1"]).to_model_spec()
    assert [e.keys_of for e in spec.schedule] == [None, None, 1, None]
    model = build_model(spec)
    assert model.entry_cache_layer == [0, 1, 1, 2] and len(model.state_needs) == 1
    needs = model.cache_needs
    assert needs[0].arrays() == ((2, 16), (2, 24)) and (needs[0].window, needs[0].keep_first) == (7, 3)
    assert needs[1].arrays() == ((1, 20),) and needs[1].window is None
    assert needs[2].arrays() == ((2, 12), (2, 20)) and (needs[2].window, needs[2].keep_first) == (9, 2)
    # the convolution's two rows of q | k | v (4*12 + 2*12 + 2*20 = 112 channels) and three memories of 8 x 12
    conv, mem = 112 * 2, 3 * 8 * 12
    assert model.state_needs[0].shape == (conv + mem,)
    names = {d.name for d in model.weight_decls()}
    assert {"l0.mix.q.norm", "l0.mix.k.norm", "l0.norm1b", "l0.norm2b", "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uq", "l1.mix.dkv", "l1.mix.dkv.norm",
            "l2.mix.uk", "l2.mix.uv", "l3.mix.left.q.b", "l3.mix.left.o.b", "l3.mix.left.v.conv", "l3.mix.right.g", "l3.mix.right.norm",
            "l3.mix.left.out", "l3.mix.right.out", "l0.mlp.shared.down", "l0.mlp.e5.up", "l0.mlp.router", "final.norm", "head", "embed"} <= names
    assert not any(n.startswith(("l2.mix.dkv", "l2.mlp", "l2.norm2", "l1.mlp.shared", "l0.mix.q.b", "l1.mix.q")) for n in names)
    k2 = build_model(config_from_dict(CONFIGS["K2"]).to_model_spec())
    assert len(k2.state_needs) == 3 and k2.state_needs[0].shape == (1 * 8 * 20,)       # one tap: the convolution keeps nothing


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="rglru"), "type"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=24), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0), "factor"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "heads"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][3]["mixer"]["right"].update(decay=[0.5, 0.5]), "decay"),
    (lambda c: c["layers"][3]["mixer"]["right"].update(decay=[0.5, 0.5, -0.1]), "decay"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=-2.0), "softcap"),
    (lambda c: c["layers"][3]["mixer"]["left"].update(softcap=0.0), "softcap"),
    (lambda c: c["layers"][3]["mixer"].pop("left"), "left"),
    (lambda c: c["layers"][0].update(mlp={"kind": "dense", "ff": 8}), "mlp"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "chosen"),
    (lambda c: c["layers"][1]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_the_key(change, match):
    c = copy.deepcopy(CONFIGS["K1"])
    change(c)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(c)


# ------------------------------------------------------------ the plain implementation
def _rand(g, *shape):
    return torch.randn(*shape, generator=g, dtype=F64)


def test_plain_constant_decay_memory_equals_its_sum_written_out():
    """o_t = sum_(s <= t) decay^(t - s) (q_t . k_s) v_s per head."""
    g = torch.Generator().manual_seed(0)
    T, H, D, Dv = 9, 3, 5, 4
    q, k, v = _rand(g, T, H, D), _rand(g, T, H, D), _rand(g, T, H, Dv)
    decay = [0.5, 0.93, 1.0]
    got = plain.constant_decay_memory(q, k, v, decay)
    for h in range(H):
        for t in range(T):
            want = sum(decay[h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert torch.allclose(got[t, h], want, atol=1e-12)


def test_plain_convolution_mask_cap_and_rotation_on_made_up_inputs():
    g = torch.Generator().manual_seed(1)
    u, w = _rand(g, 6, 3), _rand(g, 3, 4)
    y = plain.short_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0]) and torch.allclose(y[4], w[:, 0] * u[1] + w[:, 1] * u[2] + w[:, 2] * u[3] + w[:, 3] * u[4])
    see = plain.visible(12, 4, 2)
    assert see[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9] and see[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert plain.visible(5, 2, 9)[4].all() and plain.visible(5)[4].all() and not plain.visible(5)[2, 3]
    # a cap bounds every score: with a cap of 0.1 all weights are within e^0.2 of each other however large q . k is
    q, k, v = 50 * _rand(g, 7, 1, 4), _rand(g, 7, 1, 4), torch.eye(7, dtype=F64)[:, None, :]
    p = plain.softmax_attention(q, k, v, 1.0, plain.visible(7), softcap=0.1)[6, 0]
    assert p.max() / p.min() <= math.exp(0.2) + 1e-9
    # rotation: dims / 2 pairs (i, i + dims / 2), the rest pass; divided frequencies are positions divided
    x = _rand(g, 5, 2, 8)
    r = plain.rotate_first_dims(x, torch.arange(5), 100.0, 4)
    assert torch.equal(r[..., 4:], x[..., 4:]) and torch.allclose(r[0], x[0])
    a = 3 * 100.0 ** (-2 * 1 / 4)
    assert torch.allclose(r[3, 1, 1], x[3, 1, 1] * math.cos(a) - x[3, 1, 3] * math.sin(a))
    assert torch.allclose(plain.rotate_first_dims(x, torch.arange(5) * 2, 100.0, 4, divide_by=2.0), r)


def test_plain_routing_and_experts_on_made_up_scores():
    z = torch.tensor([[0.1, 2.0, -1.0, 2.0, 1.5]], dtype=F64)
    ids, wts = plain.route(z, 3)
    assert ids[0].tolist() == [1, 3, 4]                        # ties go to the lower index
    e = torch.exp(torch.tensor([2.0, 2.0, 1.5], dtype=F64))
    assert torch.allclose(wts[0], e / e.sum()) and abs(float(wts.sum()) - 1) < 1e-12
    x = torch.tensor([[3.0, -2.0, 0.5]], dtype=F64)
    W = {"e.gate": torch.eye(3, dtype=F64), "e.up": torch.eye(3, dtype=F64), "e.down": torch.eye(3, dtype=F64)}
    gg, uu = torch.tensor([1.5, -2.0, 0.5], dtype=F64), torch.tensor([1.5, -1.5, 0.5], dtype=F64)   # the gate is capped from above only
    assert torch.allclose(plain.clamped_expert(x, W, "e.", 1.5)[0], gg * torch.sigmoid(1.702 * gg) * (uu + 1))


def test_plain_kept_tokens_shared_latents_and_causality(tmp_path):
    d = make_model_dir("A", seed=5, root=str(tmp_path))
    cfg, w = read_model(d)
    toks = traces.make_requests(cfg["vocab"], [40], seed=1)["r0"]
    base = plain.forward(cfg, w, toks)
    # one layer, a window of 6 that keeps 3 tokens: position 20 sees 0..2 and 15..20
    for j, reaches in ((2, True), (3, False), (14, False), (15, True)):
        moved = list(toks)
        moved[j] = (moved[j] + 1) % cfg["vocab"]
        diff = (plain.forward(cfg, w, moved)[20] - base[20]).abs().max().item()
        assert (diff > 1e-9) == reaches, (j, diff)
    assert (plain.forward(cfg, w, toks[:25]) - base[:25]).abs().max() < 1e-12          # causal
    d = make_model_dir("K1", seed=5, root=str(tmp_path))
    cfg, w = read_model(d)
    toks = traces.make_requests(cfg["vocab"], [12], seed=1)["r0"]
    lo = []
    plain.forward(cfg, w, toks, layers_out=lo)
    # layer 2 has no down-projection: give it one that is layer 1's and a config without kv_from, and nothing changes
    # only if it reads what layer 1 read, which it does not (its input is another layer's): so the outputs differ
    own = copy.deepcopy(cfg)
    own["layers"][2]["mixer"].pop("kv_from")
    w2 = dict(w, **{"l2.mix.dkv": w["l1.mix.dkv"], "l2.mix.dkv.norm": w["l1.mix.dkv.norm"]})
    assert (plain.forward(own, w2, toks) - plain.forward(cfg, w, toks)).abs().max() > 1e-6


# ------------------------------------------------------------------ the cache manager
def test_kept_first_pages_stay_while_the_windows_pages_go_back():
    need = CacheNeed(2, 8, window=6, keep_first=5)
    cm = CacheManager([need, CacheNeed(2, 8, window=6)], [], page_size=4, num_pages=12, max_slots=2, max_tokens_per_request=200, dtype=torch.float32,
                      device="cpu")
    assert len(cm.groups) == 2 and [g.kept_pages for g in cm.groups] == [2, 0]
    cm.add_request("a")
    for _ in range(10):
        cm.append([("a", 4)])
        cm.release_passed("a")
        cm.check()
    kept, plain_window = cm.groups
    assert kept.table[0, :2].tolist() == [0, 1] and (kept.table[0, 2:8] == -1).all() and (kept.table[0, 8:10] >= 0).all()
    assert (plain_window.table[0, :8] == -1).all()
    assert [g.pool.num_pages - g.pool.num_free for g in cm.groups] == [4, 2]
    cm.free_request("a")
    cm.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in cm.groups)
    # a request shorter than what is kept, and one that is truncated back into its kept pages
    cm.add_request("b")
    cm.append([("b", 3)])
    cm.release_passed("b")
    cm.append([("b", 30)])
    cm.truncate("b", 3)
    cm.check()
    cm.free_request("b")
    assert all(g.pool.num_free == g.pool.num_pages for g in cm.groups)


# ------------------------------------------------------------------ the engine on the CPU
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("name", ["K1", "K2", "P"])
def test_cuttings_cpu(name, cut, tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    steps = traces.mixed(reqs, seed=4) if cut == "mixed" else getattr(traces, cut)(reqs)
    ps = PAGE_SIZES[name]
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), ps, max(1, traces.peak_tokens(steps) // ps), 4, device="cpu")
    got = traces.run_trace(runner, steps)
    runner.cache.check()
    assert runner.cache.num_free_slots == 4 and all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups)
    for r, want in oracle.items():
        err = (got[r].double() - want).abs().max().item()
        assert err < 5e-4 * float(want.std()), f"{name} {cut}: request {r}, error {err:.3g}"


def test_window_pages_go_back_and_first_pages_stay_while_the_request_lives(tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle("K1", tmp_path_factory)
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), 4, 40, 2, device="cpu")
    toks = reqs["r4"]
    runner.step([StepEntry("a", toks[:50], ())])
    held = [g.pool.num_pages - g.pool.num_free for g in runner.cache.groups]
    # windows of 7 and 9 keep the pages from token 44 and 42 on (two and three pages) beside one first page each; the
    # latents keep all 13
    assert held == [3, 13, 4]
    lg = runner.step([StepEntry("a", toks[50:], range(20))])
    assert (lg.double() - oracle["r4"][50:]).abs().max() < 5e-4 * float(oracle["r4"].std())


def test_a_request_that_starts_again_starts_from_empty_states(tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle("S", tmp_path_factory)
    steps = traces.preempted(reqs)
    ps = PAGE_SIZES["S"]
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), ps, traces.peak_tokens(steps) // ps, 3, device="cpu")
    seen = 0
    for rid, pos, row in traces.run_trace_by_position(runner, steps):
        assert (row.double() - oracle[rid][pos]).abs().max() < 5e-4 * float(oracle[rid].std()), (rid, pos)
        seen += 1
    assert seen > sum(len(t) for t in reqs.values())          # the victim's first half came out twice


@pytest.mark.parametrize("pages", [64, 14])
def test_greedy_generation_through_the_engine_and_scheduler(pages, tmp_path_factory, cpu_kernels):
    """The public entry point: prompts of unequal length, portions of eight tokens, and (with 14 pages) so few pages that a
    request is preempted and recomputed, cache, state and all (a model whose window is longer than the requests, so that
    no page goes back early)."""
    d = make_model_dir("F", seed=3, root=str(tmp_path_factory.mktemp("gen")), sigma=0.3)
    cfg, w = read_model(d)
    prompts = [[5, 17, 3, 150, 9, 1, 1, 44, 102, 7, 7], [42] * 19, [7]]
    ref = [plain.generate_greedy(cfg, w, p, 10) for p in prompts]
    assert all(len(set(r)) >= 3 for r in ref), "the continuation is too uniform to test anything"
    eng = Engine(d, dtype="float32", device="cpu", page_size=4, num_pages=pages, num_slots=3, chunked_prefill_size=8,
                 max_num_batched_tokens=16, cuda_graph=False)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == ref
    if pages == 14:
        assert sum(o.preemptions for o in outs) > 0
    eng.runner.cache.check()


def test_generation_with_states_and_kept_pages(tmp_path_factory, cpu_kernels):
    d = make_model_dir("S", seed=3, root=str(tmp_path_factory.mktemp("gen")), sigma=0.3)
    cfg, w = read_model(d)
    prompts = [[5, 6, 7, 8], [9] * 12, [3], [100, 2, 50]]
    eng = Engine(d, dtype="float32", device="cpu", page_size=4, num_pages=12, num_slots=2, chunked_prefill_size=8,
                 max_num_batched_tokens=16, cuda_graph=False)
    assert len(eng.runner.cache.groups) == 2 and len(eng.runner.cache.states) == 2
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert [o.token_ids for o in outs] == [plain.generate_greedy(cfg, w, p, 6) for p in prompts]
