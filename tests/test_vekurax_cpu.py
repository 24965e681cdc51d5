"""Host-side parts of the Vekurax design: its configuration reader and model description, the cache manager's windows that
keep the first tokens, caches of mixers that keep several things, and the plain implementation's own consistency."""

import json

import pytest
import torch

import plain_vekurax as pv
from tiny_models import random_tokens
from tiny_vekurax import CONFIGS_V, config_json, make_weights, tensor_shapes


def test_model_description_from_config_json():
    from mini_sglang_b200.config import ConfigError, architecture_of
    from mini_sglang_b200.parts.model import expected_tensors
    for name, cfg in CONFIGS_V.items():
        raw = config_json(cfg)
        arch = architecture_of(raw)
        assert arch.name == "Vekurax"
        spec = arch.build_spec(arch.config_cls.from_dict(raw))
        spec.validate()
        # one run per listed layer, each with a cache id of its own; layers that run another's weights own no tensors
        assert [r.cache for r in spec.schedule] == list(range(len(cfg["layers"])))
        owners = [i for i, l in enumerate(cfg["layers"]) if "weights_of" not in l]
        assert len(spec.layers) == len(owners)
        for i, (run, layer) in enumerate(zip(spec.schedule, cfg["layers"])):
            assert spec.layers[run.layer].prefix == f"l{layer.get('weights_of', i)}"
        want = tensor_shapes(cfg)
        got = {n: d for n, d in expected_tensors(spec).items() if not d.optional}
        assert set(got) == set(want)
        for n, d in got.items():
            assert len(d.shape) == len(want[n]) and all(a in (-1, b) for a, b in zip(d.shape, want[n])), n
    raw = config_json(CONFIGS_V["VA"])
    bad = json.loads(json.dumps(raw))
    bad["layers"][2]["weights_of"] = 9
    with pytest.raises(ConfigError):
        architecture_of(bad).config_cls.from_dict(bad)
    bad = json.loads(json.dumps(raw))
    bad["layers"][0]["type"] = "serial"
    with pytest.raises(ConfigError):
        architecture_of(bad).config_cls.from_dict(bad)
    bad = json.loads(json.dumps(raw))
    bad["layers"][0]["mixer"]["left"]["vdim"] = 7
    with pytest.raises(ConfigError):
        arch = architecture_of(bad)
        arch.build_spec(arch.config_cls.from_dict(bad))
    chain = json.loads(json.dumps(raw))
    chain["layers"][3]["weights_of"] = 2           # layer 2 runs layer 1's weights: so does layer 3
    arch = architecture_of(chain)
    spec = arch.build_spec(arch.config_cls.from_dict(chain))
    assert spec.schedule[3].layer == spec.schedule[1].layer


def test_cache_needs_of_a_pair_of_mixers():
    from mini_sglang_b200.cache import CacheManager, PagedKVNeed, StateNeed
    from mini_sglang_b200.config import architecture_of
    from mini_sglang_b200.parts import BuildEnv, DecoderModel
    raw = config_json(CONFIGS_V["VA"])
    arch = architecture_of(raw)
    model = DecoderModel(arch.build_spec(arch.config_cls.from_dict(raw)), BuildEnv(torch.bfloat16, torch.device("cpu")))
    needs = model.cache_needs()
    assert sorted(needs) == [(c, k) for c in range(4) for k in range(3)]
    assert needs[(0, 0)] == PagedKVNeed(3, 24, 9, q_heads=6, keep_first=3, library="mixers", even_cut=False)
    assert needs[(1, 0)].window == 5 and needs[(1, 0)].keep_first == 0
    assert needs[(0, 1)] == StateNeed((2, 6 * 24 + 3 * 24), "compute") and needs[(0, 2)] == StateNeed((3, 12, 20), "float32")
    mgr = CacheManager(needs, page_size=4, num_pages=40, max_reqs=3, max_context_len=512)
    # runs 0 and 3 share a kind of window, runs 1 and 2 the other: two groups with pools of their own
    assert sorted(sorted(g.cache_ids) for g in mgr.groups) == [[(0, 0), (3, 0)], [(1, 0), (2, 0)]]
    assert len(mgr.state_ids) == 8


def test_windows_give_pages_back_but_never_the_first_tokens():
    from mini_sglang_b200.cache import CacheManager, PagedKVNeed
    P = 4
    mgr = CacheManager({0: PagedKVNeed(1, 8, window=6, keep_first=5), 1: PagedKVNeed(1, 8, window=6, keep_first=0)},
                       page_size=P, num_pages=64, max_reqs=2, max_context_len=400, max_step_tokens=400)
    kept = next(g for g in mgr.groups if g.keep_first == 5)
    plain_window = next(g for g in mgr.groups if g.keep_first == 0)
    assert kept.keep_pages == 2 and plain_window.keep_pages == 0
    gi = mgr.groups.index(kept)
    s = mgr.open()
    first_pages = None
    for step, n in enumerate([3, 9, 1, 1, 30, 2, 1, 1, 1, 50]):
        mgr.reserve(s, n)
        mgr.commit(s, n)
        L = int(mgr.length[s])
        row = kept.table[s]
        if first_pages is None and L >= 8:
            first_pages = [int(row[0]), int(row[1])]
        if first_pages:
            assert [int(row[0]), int(row[1])] == first_pages and all(kept.pool.is_held(p) for p in first_pages)
        # every page that the next query's window or the kept tokens touch is there; everything between is given back
        lo = max(0, L - 6 + 1)
        for page in range(-(-L // P)):
            needed = page < 2 or page >= lo // P
            assert (row[page] != 0) == needed, (step, L, page)
        assert len(mgr.owned_pages(s, gi)) == kept.pool.in_use
        # the window without kept tokens holds only the window's pages
        assert plain_window.pool.in_use == -(-L // P) - lo // P
    mgr.close(s)
    assert kept.pool.in_use == 0 and plain_window.pool.in_use == 0
    mgr.check_idle()
    # the pages come round again
    s = mgr.open()
    mgr.reserve(s, 64 * P - 4)
    mgr.close(s)
    mgr.check_idle()


def test_plain_token_by_token_recurrence_equals_its_closed_form():
    """The plain linear attention against the sum it stands for, o_t = sum_{s<=t} decay^(t-s) (q_t . k_s) v_s, and the plain
    convolution against a direct sum; both catch an off-by-one in the plain implementation itself."""
    g = torch.Generator().manual_seed(0)
    T, E = 11, 16
    c = {"heads": 2, "dim": 3, "vdim": 5, "decay": [0.5, 0.9]}
    w = {"r.q": torch.randn(6, E, generator=g), "r.k": torch.randn(6, E, generator=g), "r.v": torch.randn(10, E, generator=g),
         "r.g": torch.randn(10, E, generator=g), "r.o": torch.eye(10), "r.norm": torch.ones(10)}
    w = {k: v.double() for k, v in w.items()}
    u = torch.randn(T, E, generator=g).double()
    got = pv.right_attention(u, w, "r", c, 1e-6)
    silu = torch.nn.functional.silu
    q, k, v = silu(u @ w["r.q"].T).view(T, 2, 3), silu(u @ w["r.k"].T).view(T, 2, 3), silu(u @ w["r.v"].T).view(T, 2, 5)
    o = torch.zeros(T, 2, 5, dtype=torch.float64)
    for h in range(2):
        for t in range(T):
            for s in range(t + 1):
                o[t, h] += c["decay"][h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h]
    want = pv.rms_scale(o.reshape(T, 10), w["r.norm"], 1e-6) * torch.sigmoid(u @ w["r.g"].T)
    torch.testing.assert_close(got, want)
    x, taps = torch.randn(T, 4, generator=g).double(), torch.randn(4, 3, generator=g).double()
    y = pv.short_causal_conv(x, taps)
    for t in range(T):
        for ch in range(4):
            direct = sum(taps[ch, j] * x[t - 2 + j, ch] for j in range(3) if t - 2 + j >= 0)
            assert abs(float(y[t, ch]) - float(direct)) < 1e-12
    assert [pv.distance_bucket(n, 8, 64) for n in (0, 3, 4, 7, 8, 15, 16, 63, 64, 500)] == [0, 3, 4, 4, 5, 5, 6, 7, 7, 7]


def test_plain_sequence_is_causal_and_runs_shared_weights():
    cfg = config_json(CONFIGS_V["VA"])
    w = make_weights(CONFIGS_V["VA"], 3)
    toks = random_tokens(20, cfg["vocab"], 1)
    full = pv.forward_sequence(cfg, w, toks)
    part = pv.forward_sequence(cfg, w, toks[:12])
    torch.testing.assert_close(full[:12], part)
    streams = []
    pv.forward_sequence(cfg, w, toks, streams=streams)
    assert len(streams) == len(cfg["layers"])


def test_a_window_or_kept_token_one_off_would_show():
    """The bound of the model-level comparisons on the GPU (an rms error of 2.5 % of a row's rms in bfloat16) can fail: the plain
    implementation with the window one token wider or narrower, or one kept token more or fewer, moves every row behind the
    window by at least twice that."""
    cfg = config_json(CONFIGS_V["VA"])
    w = make_weights(CONFIGS_V["VA"], 3)
    toks = random_tokens(60, cfg["vocab"], 9)
    base = pv.forward_sequence(cfg, w, toks).float()
    for key, delta in (("size", 1), ("size", -1), ("keep_first", -1), ("keep_first", 1)):
        other = json.loads(json.dumps(cfg))
        for layer in other["layers"]:
            if layer["mixer"]["left"]["mask"][key] + delta >= 0:
                layer["mixer"]["left"]["mask"][key] += delta
        moved = pv.forward_sequence(other, w, toks).float()
        err = (moved - base).pow(2).mean(1).sqrt() / base.pow(2).mean(1).sqrt()
        assert float(err[20:].min()) > 0.045, (key, delta, float(err[20:].min()))
