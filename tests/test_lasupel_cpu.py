"""Lasupel without a GPU: the configuration reader and what it refuses, the model as the registry builds it (layers that
read another layer's cache, states of their own), the plain implementation's own checks (each recurrence against its sum
written out, the routing rules on made-up scores, the window and the sink), and the engine around the kernels (cache
pages, state slots, step function, scheduler) under every way of cutting the work, with the kernels replaced by their
torch statements."""
import copy
import math

import pytest
import torch

import plain_lasupel as plain
import traces
from arle_b200 import Engine
from arle_b200.config import ConfigError, LasupelConfig, config_from_dict
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.parts import build_model
from arle_b200.sampling import SamplingParams
from tiny_lasupel import CONFIGS, PAGE_SIZES, make_model_dir, read_model

LENGTHS = {"L1": [1, 5, 12, 23, 70, 33], "L2": [2, 17, 40, 64, 9, 31], "S": [3, 30, 11, 2, 45], "R": [1, 20, 33, 7]}
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
    cfg = config_from_dict(CONFIGS["L1"])
    assert isinstance(cfg, LasupelConfig) and [l.type for l in cfg.layers] == ["attention", "rglru", "attention", "delta"]
    assert cfg.layers[2].m("kv_from") == 0 and cfg.layers[0].m("kv_from") is None and cfg.layers[2].mlp is None
    assert cfg.layers[0].m("window") == 7 and cfg.layers[0].m("vdim") == 24 and cfg.layers[0].m("rot_dims") == 8
    assert cfg.layers[1].m("blocks") == 3 and cfg.layers[1].m("conv") == 3 and cfg.layers[3].m("conv") == 4
    assert cfg.layers[1].mlp.experts == 6 and cfg.layers[1].mlp.keep == 2 and cfg.layers[1].mlp.limit == 1.2 and cfg.layers[3].mlp.limit == 0.8
    assert cfg.embedding_scale == 1.5 and cfg.norm_eps == 1e-5


def test_model_spec_gives_readers_their_owners_cache_and_the_longest_window():
    spec = config_from_dict(CONFIGS["L1"]).to_model_spec()
    assert [e.keys_of for e in spec.schedule] == [None, None, 0, None]
    model = build_model(spec)
    assert len(model.cache_needs) == 1 and len(model.state_needs) == 2
    assert model.cache_needs[0].arrays() == ((2, 16), (2, 24)) and model.cache_needs[0].window == 11       # the reader's window is longer
    assert model.entry_cache_layer == [0, None, 0, None]
    names = {d.name for d in model.weight_decls()}
    assert {"l0.mix.k", "l0.mix.v", "l2.mix.q", "l2.mix.o", "l1.mix.ra.b", "l1.mix.conv.b", "l3.mix.q.conv", "l3.mix.A_log", "l3.mix.norm",
            "l1.mlp.e5.down", "l1.mlp.router", "final.norm", "head", "embed"} <= names
    assert not any(n.startswith(("l2.mix.k", "l2.mix.v", "l2.mlp", "l2.norm2")) or n.endswith(("q_norm", "correction")) for n in names)
    spec = config_from_dict(CONFIGS["L2"]).to_model_spec()
    model = build_model(spec)
    windows = sorted((n.window, n.arrays()) for n in model.cache_needs)
    assert windows == [(1, ((2, 8), (2, 4))), (1000, ((1, 12), (1, 40)))]                                 # the reader's shorter window changes nothing
    assert config_from_dict(CONFIGS["R"]).to_model_spec() and not build_model(config_from_dict(CONFIGS["R"]).to_model_spec()).cache_needs


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="latent"), "type"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=1), "differ"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(base=500.0), "differ"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "heads"),
    (lambda c: c["layers"][1]["mixer"].update(blocks=5), "blocks"),
    (lambda c: c["layers"][3]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][3]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0].update(mlp={"kind": "sparse", "ff": 8}), "mlp"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "chosen"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_the_key(change, match):
    c = copy.deepcopy(CONFIGS["L1"])
    change(c)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(c)


# ------------------------------------------------------------ the plain implementation
def _rand(g, *shape):
    return torch.randn(*shape, generator=g, dtype=F64)


def test_plain_rglru_equals_its_sum_written_out():
    """S_t = sum_s (a_(s+1) .. a_t) sqrt(1 - a_s^2) i_s u_s with the gates of every token from its own convolved input."""
    g = torch.Generator().manual_seed(0)
    T, D, width, nb, taps = 9, 10, 12, 3, 3
    bs = width // nb
    W = {"p.y": _rand(g, width, D), "p.y.b": _rand(g, width), "p.x": _rand(g, width, D), "p.x.b": _rand(g, width), "p.conv": _rand(g, width, taps),
         "p.conv.b": _rand(g, width), "p.ra": _rand(g, nb, bs, bs), "p.ra.b": _rand(g, nb, bs), "p.ri": _rand(g, nb, bs, bs),
         "p.ri.b": _rand(g, nb, bs), "p.lam": _rand(g, width), "p.o": torch.eye(width, dtype=F64)}
    h = _rand(g, T, D)
    got = plain.rglru(h, W, "p.", {"width": width, "blocks": nb, "conv": taps})
    xin = h @ W["p.x"].T + W["p.x.b"]
    u = torch.zeros(T, width, dtype=F64)
    for t in range(T):
        for j in range(taps):
            if t - (taps - 1) + j >= 0:
                u[t] += W["p.conv"][:, j] * xin[t - (taps - 1) + j]
    u = u + W["p.conv.b"]
    r, i = torch.zeros(T, width, dtype=F64), torch.zeros(T, width, dtype=F64)
    for b in range(nb):
        sl = slice(b * bs, (b + 1) * bs)
        r[:, sl] = torch.sigmoid(u[:, sl] @ W["p.ra"][b].T + W["p.ra.b"][b])
        i[:, sl] = torch.sigmoid(u[:, sl] @ W["p.ri"][b].T + W["p.ri.b"][b])
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(W["p.lam"]))
    y = h @ W["p.y"].T + W["p.y.b"]
    y = 0.5 * y * (1 + torch.tanh(math.sqrt(2 / math.pi) * (y + 0.044715 * y ** 3)))
    want = torch.zeros(T, width, dtype=F64)
    for t in range(T):
        for s in range(t + 1):
            want[t] += a[s + 1: t + 1].prod(0) * torch.sqrt(1 - a[s] ** 2) * i[s] * u[s]
    assert (got - want * y).abs().max() < 1e-9


def test_plain_delta_rule_equals_its_recurrence_in_the_other_form():
    """S_t = g_t S_(t-1) (I - beta_t k_t k_t^T)-wise: S_t = g_t S_(t-1) - beta_t k_t (g_t S_(t-1)^T k_t)^T + beta_t k_t v_t^T."""
    g = torch.Generator().manual_seed(1)
    T, D, H, G, dk, dv, taps = 8, 9, 4, 2, 5, 3, 3
    W = {"p.q": _rand(g, G * dk, D), "p.k": _rand(g, G * dk, D), "p.v": _rand(g, H * dv, D), "p.q.conv": _rand(g, G * dk, taps),
         "p.k.conv": _rand(g, G * dk, taps), "p.v.conv": _rand(g, H * dv, taps), "p.b": _rand(g, H, D), "p.a": _rand(g, H, D),
         "p.A_log": _rand(g, H) * 0.3, "p.dt_bias": _rand(g, H), "p.g": _rand(g, H * dv, D), "p.norm": torch.rand(dv, generator=g, dtype=F64) + 0.5,
         "p.o": torch.eye(H * dv, dtype=F64)}
    h = _rand(g, T, D)
    got = plain.delta_rule(h, W, "p.", {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "conv": taps}, 1e-6)

    def conv_silu(x, taps_w):
        out = torch.zeros_like(x)
        for t in range(T):
            for j in range(taps):
                if t - (taps - 1) + j >= 0:
                    out[t] += taps_w[:, j] * x[t - (taps - 1) + j]
        return out * torch.sigmoid(out)

    q = conv_silu(h @ W["p.q"].T, W["p.q.conv"]).view(T, G, dk)
    k = conv_silu(h @ W["p.k"].T, W["p.k.conv"]).view(T, G, dk)
    v = conv_silu(h @ W["p.v"].T, W["p.v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(dk)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W["p.b"].T)
    dec = torch.exp(-torch.exp(W["p.A_log"]) * torch.nn.functional.softplus(h @ W["p.a"].T + W["p.dt_bias"]))
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            kt = k[t, a // (H // G)]
            S = dec[t, a] * (torch.eye(dk, dtype=F64) - beta[t, a] * torch.outer(kt, kt)) @ S + beta[t, a] * torch.outer(kt, v[t, a])
            o[t, a] = S.T @ q[t, a // (H // G)]
    gate = (h @ W["p.g"].T).view(T, H, dv)
    want = plain.rms_unit(o, 1e-6) * W["p.norm"] * (gate * torch.sigmoid(gate))
    assert (got - want.reshape(T, H * dv)).abs().max() < 1e-9


def test_plain_routing_rules_on_made_up_scores():
    """Eight experts in four pairs: a group counts by its best expert alone (not by its two best), experts outside the kept
    groups are never chosen however large, and the weights are the softmax scores as they are (they do not sum to one)."""
    s = torch.tensor([[0.05, 0.30, 0.17, 0.16, 0.18, 0.01, 0.02, 0.11]], dtype=F64)       # sums to one: its own softmax
    idx, wts = plain.route(torch.log(s), 3, 4, 2)
    # group scores 0.30, 0.17, 0.18, 0.11: groups 0 and 2 are kept (by two-best sums, 0.33 of group 1 would beat group 2's 0.19)
    assert sorted(idx[0].tolist()) == [0, 1, 4]
    assert torch.allclose(wts[0].sort().values, torch.tensor([0.05, 0.18, 0.30], dtype=F64))
    idx, wts = plain.route(torch.log(s), 2, 1, 1)
    assert sorted(idx[0].tolist()) == [1, 4]
    x = torch.tensor([[3.0, -2.0, 0.5]], dtype=F64)
    W = {"e.gate": torch.eye(3, dtype=F64), "e.up": torch.eye(3, dtype=F64), "e.down": torch.eye(3, dtype=F64)}
    g, u = torch.tensor([1.5, -2.0, 0.5], dtype=F64), torch.tensor([1.5, -1.5, 0.5], dtype=F64)   # the gate is capped from above only
    assert torch.allclose(plain.expert_ff(x, W, "e.", 1.5)[0], g * torch.sigmoid(1.702 * g) * (u + 1))


def test_plain_window_sink_and_shared_keys(tmp_path):
    d = make_model_dir("A", seed=5, root=str(tmp_path))
    cfg, w = read_model(d)
    toks = traces.make_requests(cfg["vocab"], [40], seed=1)["r0"]
    base = plain.forward(cfg, w, toks)
    # the second layer's keys and values are the first layer's, which come from the embeddings alone: position 20 sees
    # tokens 8 to 20 through the second window (13) and nothing older (windows that chain would reach 17 back)
    for back, reaches in ((13, False), (12, True)):
        moved = list(toks)
        moved[20 - back] = (moved[20 - back] + 1) % cfg["vocab"]
        diff = (plain.forward(cfg, w, moved)[20] - base[20]).abs().max().item()
        assert (diff > 1e-9) == reaches, (back, diff)
    assert (plain.forward(cfg, w, toks[:25]) - base[:25]).abs().max() < 1e-12          # causal
    # the sink: a single key of score 0 gets weight 1/2, so the first token's attention output is half its value
    g = torch.Generator().manual_seed(2)
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 0.0, "mask": {"size": 8}, "rot": {"base": 10.0, "dims": 2}}
    W = {"p.q": _rand(g, 4, 5), "p.k": _rand(g, 4, 5), "p.v": _rand(g, 3, 5), "p.o": torch.eye(3, dtype=F64)}
    h = _rand(g, 6, 5)
    out = plain.attention(h, W, "p.", m, 1e-6, plain.attention_keys_values(h, W, "p.", m, 1e-6))
    v = h @ W["p.v"].T
    for t in range(6):
        assert torch.allclose(out[t], v[: t + 1].sum(0) / (t + 2))
    k, _ = plain.attention_keys_values(h, W, "p.", m, 1e-6)
    assert torch.allclose((k * k).mean(-1), torch.ones(6, 1, dtype=F64), atol=1e-4)     # unit root mean square after the rotation


# ------------------------------------------------------------------ the engine on the CPU
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("name", ["L1", "L2", "R"])
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


def test_window_pages_go_back_while_the_request_lives(tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle("L1", tmp_path_factory)
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), 4, 40, 2, device="cpu")
    toks = reqs["r4"]
    runner.step([StepEntry("a", toks[:50], ())])
    held = [g.pool.num_pages - g.pool.num_free for g in runner.cache.groups]
    assert held == [3]                      # the longer of the two windows (11): the pages of the last 10 tokens (40..49), not all 13
    lg = runner.step([StepEntry("a", toks[50:], range(20))])
    assert (lg.double() - oracle["r4"][50:]).abs().max() < 5e-4 * float(oracle["r4"].std())


def test_a_request_that_starts_again_starts_from_an_empty_state(tmp_path_factory, cpu_kernels):
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


def test_generation_with_a_model_that_keeps_no_paged_cache(tmp_path_factory, cpu_kernels):
    """Recurrent mixers only: the cache manager has state slots and no page group; the scheduler admits by slots alone."""
    d = make_model_dir("R", seed=3, root=str(tmp_path_factory.mktemp("gen")), sigma=0.3)
    cfg, w = read_model(d)
    prompts = [[5, 6, 7, 8], [9] * 12, [3], [100, 2, 50]]
    eng = Engine(d, dtype="float32", device="cpu", page_size=4, num_pages=8, num_slots=2, chunked_prefill_size=8,
                 max_num_batched_tokens=16, cuda_graph=False)
    assert not eng.runner.cache.groups and len(eng.runner.cache.states) == 2
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert [o.token_ids for o in outs] == [plain.generate_greedy(cfg, w, p, 6) for p in prompts]
