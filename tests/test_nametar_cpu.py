"""Nametar without a GPU: the configuration reader and the model description against the tiny configurations, the plain
implementation's mechanisms against closed forms, the frequency scaling of the rotary part, and what the model-level
bounds of the GPU tests can tell apart."""

import copy
import math

import pytest
import torch

import plain_nametar as pn
from tiny_models import random_tokens
from tiny_nametar import CONFIGS_N, config_json, make_weights, tensor_shapes


@pytest.mark.parametrize("name", sorted(CONFIGS_N))
def test_description_declares_the_checkpoints_tensors(name):
    from mini_sglang_b200.config import architecture_of
    from mini_sglang_b200.parts.model import expected_tensors
    raw = config_json(CONFIGS_N[name])
    arch = architecture_of(raw)
    assert arch.name == "Nametar"
    spec = arch.build_spec(arch.config_cls.from_dict(raw))
    spec.validate()
    want = tensor_shapes(CONFIGS_N[name])
    got = expected_tensors(spec)
    assert set(got) == set(want)
    for k, decl in got.items():
        assert len(decl.shape) == len(want[k]) and all(a in (-1, b) for a, b in zip(decl.shape, want[k])), (k, decl.shape, want[k])
    assert [l.block for l in spec.layers] == ["sandwich_residual"] * len(raw["layers"])
    for l, entry in zip(spec.layers, raw["layers"]):
        assert (l.feed_forward is None) == (entry["mlp"] is None)
        assert (l.position is not None) == bool(entry["mixer"].get("rot_dim"))
        if entry["type"] != "gla":
            assert l.mixer["window"] == (entry["mixer"].get("mask") or {}).get("size")


def test_configuration_refusals():
    from mini_sglang_b200.config import ConfigError, architecture_of
    raw = config_json(CONFIGS_N["NA"])
    arch = architecture_of(raw)
    for change in (lambda c: c["layers"][0].__setitem__("type", "something"),
                   lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"),
                   lambda c: c["layers"][0]["mixer"].pop("kv_rank"),
                   lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 10),
                   lambda c: c.pop("width")):
        bad = copy.deepcopy(raw)
        change(bad)
        with pytest.raises(ConfigError):
            arch.build_spec(arch.config_cls.from_dict(bad))


def test_frequencies_of_the_rotary_part():
    from mini_sglang_b200.parts.rope import yarn_frequencies
    for dims, base, sc in ((16, 10000.0, {"factor": 2.0, "original": 1024, "fast": 32.0, "slow": 1.0}),
                           (8, 50.0, None), (32, 500000.0, {"factor": 8.0, "original": 4096, "fast": 4.0, "slow": 0.5}),
                           (4, 100.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})):
        f, mag = yarn_frequencies(dims, base, sc)
        want, wmag = pn.rotary_frequencies(dims, base, sc)
        torch.testing.assert_close(f, want, rtol=1e-12, atol=0)
        assert abs(mag - wmag) < 1e-12
        plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        if sc is None:
            torch.testing.assert_close(f, plain)
        else:
            assert (f <= plain + 1e-15).all() and (f >= plain / sc["factor"] - 1e-15).all()
            assert float(f[0]) == 1.0                       # the fastest pair turns too often within `original` to be slowed


def test_plain_mechanisms_against_closed_forms():
    # a rotation by position p composed with one by position -p is the identity times mag^2; norms are preserved up to mag
    freq, mag = pn.rotary_frequencies(8, 100.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})
    v = torch.randn(12, dtype=torch.float64)
    w = pn.rotate(v, 7, freq, mag, 8)
    torch.testing.assert_close(w[8:], v[8:])
    torch.testing.assert_close(w[:8].norm(), v[:8].norm() * mag)
    torch.testing.assert_close(pn.rotate(w, -7, freq, mag, 8)[:8], v[:8] * mag * mag)
    # the score of two rotated vectors depends on the distance only
    a, b = torch.randn(8, dtype=torch.float64), torch.randn(8, dtype=torch.float64)
    s1 = pn.rotate(a, 10, freq, 1.0, 8) @ pn.rotate(b, 4, freq, 1.0, 8)
    s2 = pn.rotate(a, 106, freq, 1.0, 8) @ pn.rotate(b, 100, freq, 1.0, 8)
    assert abs(float(s1 - s2)) < 1e-4           # float32 angles
    # the linear attention with alpha = 1 (z large) is a plain running sum; with alpha = 0 it sees the current token only
    E, H, dk, dv, T = 6, 1, 3, 2, 5
    g = torch.Generator().manual_seed(0)
    W = {"q": torch.randn(dk, E, generator=g), "k": torch.randn(dk, E, generator=g), "v": torch.randn(dv, E, generator=g),
         "g": torch.randn(dv, E, generator=g), "o": torch.eye(E)[:, :dv], "norm": torch.ones(dv), "a1": torch.zeros(2, E),
         "a2": torch.zeros(dk, 2)}
    W = {k: t.double() for k, t in W.items()}
    h = torch.randn(T, E, generator=g).double()
    m = {"heads": H, "dim": dk, "vdim": dv, "tau": 2.0}
    for bias, keep in ((60.0, 1.0), (-2000.0, 0.0)):
        W["a2.b"] = torch.full((dk,), bias, dtype=torch.float64)
        got = pn.gated_linear_attention(W, "", m, h, 0.0)
        q, k, v = h @ W["q"].T * dk ** -0.5, h @ W["k"].T, h @ W["v"].T
        o = torch.stack([sum((q[t] @ k[j]) * v[j] for j in range(t + 1) if keep or j == t) for t in range(T)])
        want = (pn.rms_scale(o, None, 0.0) * pn.silu(h @ W["g"].T)) @ W["o"].T
        torch.testing.assert_close(got, want)
    assert pn.visible(9, 1, 9) and not pn.visible(9, 0, 9) and pn.visible(9, 0, None) and not pn.visible(3, 4, None)


def _bound_would_catch(name, mutate, n, from_pos):
    cfg, W = config_json(CONFIGS_N[name]), make_weights(CONFIGS_N[name], 3)
    toks = random_tokens(n, cfg["vocab"], 5)
    a = pn.forward_sequence(cfg, W, toks)
    b = pn.forward_sequence(cfg, W, toks, mutate=mutate)
    scale = a.pow(2).mean(-1).sqrt()
    rel = (a - b).pow(2).mean(-1).sqrt() / scale
    return rel[from_pos:]


def test_the_model_level_bound_tells_a_wrong_window_or_decay_apart():
    """The GPU tests accept a bfloat16 row whose error is below 3 % of the row's rms.  A window one token wider, a rotation
    at a position one off, a decay taken with another tau or a missing residual factor move the rows by more."""
    def wider(cfg):
        c = copy.deepcopy(cfg)
        c["layers"][0]["mixer"]["mask"]["size"] += 1
        return c
    assert float(_bound_would_catch("NA", wider, 30, 12).median()) > 0.05

    def other_tau(cfg):
        c = copy.deepcopy(cfg)
        c["layers"][1]["mixer"]["tau"] *= 2.0
        return c
    assert float(_bound_would_catch("NA", other_tau, 30, 5).median()) > 0.04

    def no_scaling(cfg):
        c = copy.deepcopy(cfg)
        c["layers"][0]["mixer"]["rot"].pop("scaling")
        return c
    assert float(_bound_would_catch("NA", no_scaling, 30, 5).median()) > 0.05

    def wider_b(cfg):
        c = copy.deepcopy(cfg)
        c["layers"][2]["mixer"]["mask"]["size"] += 1
        return c
    assert float(_bound_would_catch("NB", wider_b, 30, 6).median()) > 0.08

    def other_tau_b(cfg):
        c = copy.deepcopy(cfg)
        c["layers"][0]["mixer"]["tau"] *= 2.0
        return c
    assert float(_bound_would_catch("NB", other_tau_b, 30, 6).median()) > 0.08

    def unit_mult(cfg):
        c = copy.deepcopy(cfg)
        c["residual_mult"] = 1.0
        return c
    assert float(_bound_would_catch("NA", unit_mult, 12, 0).median()) > 0.05
