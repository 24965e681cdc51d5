"""The Vekurax parts and the whole model in the engine against the plain implementation (tests/plain_vekurax.py).

Kernels one by one with inputs made so that a fault shows (one key whose score stands out: far away, just inside and
just outside the window, the last kept first token and the one after it), then the model through the step function:
whole prompts, token by token, in portions down to two tokens, mixed batches on a pool so small that pages and request
slots are used again, long decoding past every window, and greedy generation through the engine's entry point.
"""

import functools
import json
import math
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_vekurax as pv
from helpers import assert_row_close, play
from tiny_models import random_tokens, write_model_dir
from tiny_vekurax import CONFIGS_V, config_json, make_weights

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEED = {"VA": 3, "VB": 4, "VC": 5}
PAGE = {"VA": 4, "VB": 1, "VC": 16}
_tmp = tempfile.TemporaryDirectory(prefix="msgl_vekurax_")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@functools.lru_cache(None)
def weights(name):
    return make_weights(CONFIGS_V[name], SEED[name])


@functools.lru_cache(None)
def model_dir(name):
    return write_model_dir(os.path.join(_tmp.name, name), config_json(CONFIGS_V[name]), weights(name))


@functools.lru_cache(None)
def plain(name, tokens):
    with torch.no_grad():
        return pv.forward_sequence(config_json(CONFIGS_V[name]), weights(name), list(tokens)).float()


def runner(name, dtype, num_pages, max_reqs=4, page_size=None, graphs=True):
    from mini_sglang_b200.engine.step import ModelRunner
    return ModelRunner.from_model_dir(model_dir(name), dtype=dtype, page_size=page_size or PAGE[name], num_pages=num_pages,
                                      max_reqs=max_reqs, max_context_len=4096, use_cuda_graph=graphs)


# bfloat16: a layer of this design rounds to 8 mantissa bits at more places than a plain attention layer (what leaves the
# convolution, the normed q and k, both mixers' gated outputs, the activation), and a run of the layer list twice doubles them:
# the rounding noise of the logits is up to about 1.7 % of a row's rms at these small widths.  The bound is 2.5 %; a window one
# token off or one kept token fewer moves every row behind the window by 5 % or more (tests/test_vekurax_cpu.py).
BF16_RMS_FRACTION_V = 0.025


def row_close(row, want, dtype):
    if dtype == "float32":
        return assert_row_close(row, want, dtype)
    row, want = row.float(), want.float()
    assert torch.isfinite(row).all(), "logits are not finite"
    err = row - want
    scale = want.pow(2).mean().sqrt().item()
    rms, worst = err.pow(2).mean().sqrt().item(), err.abs().max().item()
    assert rms <= BF16_RMS_FRACTION_V * scale, f"rms error {rms:.4g} is {rms / scale:.2%} of the row's rms {scale:.4g}"
    assert worst <= 6.0 * BF16_RMS_FRACTION_V * scale, f"largest error {worst:.4g} is {worst / scale:.2%} of the row's rms {scale:.4g}"


def compare(name, dtype, got, seqs):
    assert got
    for (rid, pos), row in sorted(got.items()):
        want = plain(name, tuple(seqs[rid]))[pos]
        try:
            row_close(row, want, dtype)
        except AssertionError as e:
            raise AssertionError(f"request {rid!r} position {pos} ({dtype}, {name}): {e}") from None


def poison(r):
    """Whatever a page or a state row held before must not be read: fill the caches with NaN (state rows are zeroed when a
    request is opened)."""
    for k, v in r.storage.kv.values():
        k.fill_(float("nan"))
        v.fill_(float("nan"))
    for s in r.storage.state.values():
        s.fill_(float("nan"))


# ---------------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_dynamic_tanh_norm(dtype):
    from mini_sglang_b200 import ops
    g = torch.Generator().manual_seed(0)
    H, T = 70, 9
    res, x = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g)
    w, b, alpha = 1 + 0.1 * torch.randn(H, generator=g), 0.1 * torch.randn(H, generator=g), 0.61
    want = pv.dynamic_tanh((res + x).double(), torch.tensor(alpha).double(), w.double(), b.double()).float()
    res_d = res.cuda()
    y = ops.dyntanh(w.cuda(), b.cuda(), alpha, x=x.cuda(), residual=res_d, residual_out=res_d, out_dtype=DT[dtype])
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(y.float().cpu(), want, **tol)
    torch.testing.assert_close(res_d.cpu(), res + x)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32).cuda()
    y2 = ops.dyntanh(w.cuda(), b.cuda(), alpha, residual=res_d, rows=rows, out_dtype=DT[dtype])
    torch.testing.assert_close(y2.float().cpu(), want[[7, 0, 3]], **tol)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gated_activation_and_rms_gate(act):
    from mini_sglang_b200 import ops
    g = torch.Generator().manual_seed(1)
    T, I = 5, 37
    packed = (3 * torch.randn(T, 2 * I + 3, generator=g)).cuda()
    out = torch.zeros(T, I + 5).cuda()
    ops.gated_act(packed[:, 1:1 + I], packed[:, 2 + I:2 + 2 * I], out[:, 2:2 + I], ops.ACT_GELU_TANH if act == "gelu_tanh" else ops.ACT_SILU)
    a, u = packed[:, 1:1 + I].double().cpu(), packed[:, 2 + I:2 + 2 * I].double().cpu()
    want = (pv.gelu_tanh(a) if act == "gelu_tanh" else torch.nn.functional.silu(a)) * u
    torch.testing.assert_close(out[:, 2:2 + I].cpu(), want.float(), rtol=1e-5, atol=1e-5)
    assert float(out[:, :2].abs().sum()) == 0 and float(out[:, 2 + I:].abs().sum()) == 0
    x, w = torch.randn(T, I, generator=g), 1 + 0.1 * torch.randn(I, generator=g)
    o2 = torch.zeros(T, I + 4).cuda()
    ops.rms_gate(x.cuda(), w.cuda(), 1e-3, packed[:, 1:1 + I], o2[:, 4:], 0.7)
    want2 = pv.rms_scale(x.double(), w.double(), 1e-3) * torch.sigmoid(a) * 0.7
    torch.testing.assert_close(o2[:, 4:].cpu(), want2.float(), rtol=1e-5, atol=1e-5)


def test_distance_buckets_equal_the_plain_ones():
    from mini_sglang_b200.parts.window_attention import distance_buckets
    for rows, far in ((24, 300), (10, 37), (2, 5), (15, 200), (16, 256), (1, 9), (64, 1000)):
        n = int(far) + 40
        got = distance_buckets(rows, far, n).tolist()
        want = [pv.distance_bucket(k, rows, far) if rows > 1 else 0 for k in range(n)]
        assert got == want, (rows, far)
        assert all(b == rows - 1 for b in got[int(far):])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,cuts", [(4, (1, 2, 1, 5, 3, 11)), (2, (7, 1, 1, 14)), (1, (23,)), (5, (2, 2, 2, 2, 15)),
                                       (4, (3, 1, 1, 1, 1, 1, 1, 3)), (3, (1,) * 9), (6, (1,) * 8)])
@pytest.mark.parametrize("pad", [3, 0, 2])          # columns beside q and k in the packed rows: one, eight or two channels a thread
def test_convolution_norm_and_cache_write_in_portions(dtype, taps, cuts, pad):
    """Two requests fed in different portions in the same steps: the convolution continues from each request's own state,
    and the cache receives the normed keys and the un-normed keys as values at the given slots."""
    from mini_sglang_b200 import ops
    g = torch.Generator().manual_seed(taps)
    H, G, d, P = 4, 2, 12, 4
    Cq, Ck, T = H * d, G * d, sum(cuts)
    dt = DT[dtype]
    rnd = lambda *s: torch.randn(*s, generator=g).to(dt).float()          # noqa: E731
    u = {r: rnd(T, Cq + Ck + pad) for r in (0, 1)}                          # packed rows: q | k | something else
    qt, kt = 0.6 * torch.randn(Cq, taps, generator=g), 0.6 * torch.randn(Ck, taps, generator=g)
    qn, kn = 1 + 0.1 * torch.randn(Cq, generator=g), 1 + 0.1 * torch.randn(Ck, generator=g)
    eps = 1e-5
    state = torch.full((3, taps - 1, Cq + Ck), float("nan"), dtype=dt).cuda()
    state[1:].zero_()
    n_pages = 2 * (-(-T // P))
    kc = torch.full((n_pages + 1, G, P, d), float("nan"), dtype=dt).cuda()
    vc = kc.clone()
    perm = torch.randperm(n_pages, generator=g) + 1
    loc = {r: [int(perm[r * (n_pages // 2) + p // P]) * P + p % P for p in range(T)] for r in (0, 1)}
    got_q = {0: [], 1: []}
    at = {0: 0, 1: 0}
    order = {0: list(cuts), 1: list(reversed(cuts))}
    while order[0] or order[1]:
        reqs = [r for r in (1, 0) if order[r]]
        ns = [order[r].pop(0) for r in reqs]
        x = torch.cat([u[r][at[r]:at[r] + n] for r, n in zip(reqs, ns)]).to(dt).cuda()
        q_start = torch.tensor(np.concatenate(([0], np.cumsum(ns))), dtype=torch.int32).cuda()
        token_req = torch.tensor(sum(([i] * n for i, n in enumerate(ns)), []), dtype=torch.int32).cuda()
        slots = torch.tensor([r + 1 for r in reqs], dtype=torch.int32).cuda()
        out_loc = torch.tensor(sum((loc[r][at[r]:at[r] + n] for r, n in zip(reqs, ns)), []), dtype=torch.int32).cuda()
        q = ops.conv_norm_kvwrite(x[:, :Cq], x[:, Cq:Cq + Ck], n_kv=G, head_dim=d, q_taps=qt.t().contiguous().cuda(), k_taps=kt.t().contiguous().cuda(),
                                  q_norm=qn.cuda(),
                                  k_norm=kn.cuda(), eps=eps, state=state, token_req=token_req, q_start=q_start, slots=slots,
                                  out_loc=out_loc, k_cache=kc, v_cache=vc, page_size=P, one_token=all(n == 1 for n in ns))
        o = 0
        for r, n in zip(reqs, ns):
            got_q[r].append(q[o:o + n].float().cpu())
            o += n
            at[r] += n
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)
    for r in (0, 1):
        yq = pv.short_causal_conv(u[r][:, :Cq].double(), qt.double())
        yk = pv.short_causal_conv(u[r][:, Cq:Cq + Ck].double(), kt.double())
        torch.testing.assert_close(torch.cat(got_q[r]), pv.rms_scale(yq, qn.double(), eps).float(), **tol)
        idx = torch.tensor(loc[r])
        k_got = kc.float().cpu().permute(0, 2, 1, 3).reshape(-1, G * d)[idx]
        v_got = vc.float().cpu().permute(0, 2, 1, 3).reshape(-1, G * d)[idx]
        torch.testing.assert_close(k_got, pv.rms_scale(yk, kn.double(), eps).float(), **tol)
        torch.testing.assert_close(v_got, yk.float(), **tol)


def _window_case(dtype, *, H, G, d, P, window, keep_first, rows, far, ctx, n_new, spike_at, seed):
    """One request with `ctx` cached tokens and `n_new` new ones.  Queries and keys are small random vectors except
    that every query and the key at distance `spike_at[0]` from the last query (or, given as ("abs", j), the key at
    position j) share a large component: that key takes nearly all the weight wherever the mask lets it be seen."""
    from mini_sglang_b200 import ops
    from mini_sglang_b200.parts.window_attention import distance_buckets
    g = torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    L = ctx + n_new
    q = (0.3 * torch.randn(n_new, H, d, generator=g))
    k = (0.3 * torch.randn(L, G, d, generator=g))
    v = torch.randn(L, G, d, generator=g)
    j_star = spike_at[1] if spike_at[0] == "abs" else L - 1 - spike_at[0]
    q[:, :, 0] += 6.0
    if 0 <= j_star < L:
        k[j_star, :, 0] += 6.0
    q, k, v = q.to(dt).float(), k.to(dt).float(), v.to(dt).float()
    rel = torch.randn(rows, H, generator=g)
    gate = torch.randn(n_new, H, generator=g).to(dt).float()
    scale = 0.5
    # plain: every query by itself over the keys it may see
    want = torch.zeros(n_new, H, d, dtype=torch.float64)
    bucket = torch.tensor([pv.distance_bucket(n, rows, far) if rows > 1 else 0 for n in range(L)])
    qd_, kd_, vd_ = q.double(), k.double(), v.double()
    for t in range(n_new):
        i = ctx + t
        js = torch.tensor([j for j in range(i + 1) if pv.visible(i, j, window, keep_first)])
        for h in range(H):
            kvh = h // (H // G)
            sc_ = (kd_[js, kvh] @ qd_[t, h]) * scale + rel[bucket[i - js], h].double()
            a = torch.softmax(sc_, 0)
            want[t, h] = (a[:, None] * vd_[js, kvh]).sum(0) * torch.sigmoid(gate[t, h].double()) * 1.25
    # engine kernel over a paged cache with shuffled pages
    n_pages = -(-L // P)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages] + 1
    kc = torch.full((n_pages + 4, G, P, d), float("nan"), dtype=dt)
    vc = kc.clone()
    for p in range(L):
        kc[perm[p // P], :, p % P] = k[p].to(dt)
        vc[perm[p // P], :, p % P] = v[p].to(dt)
    n_dist = int(math.ceil(far)) + 1 if rows > 1 else 1
    bias = rel[distance_buckets(rows, far, n_dist)].t().contiguous()
    packed = torch.zeros(n_new, H + 3, dtype=dt)
    packed[:, 2:2 + H] = gate.to(dt)
    out = torch.zeros(n_new, H * d + 8, dtype=dt).cuda()
    ops.window_attention(q.to(dt).cuda(), out[:, 8:], kc.cuda(), vc.cuda(), q_start=torch.tensor([0, n_new], dtype=torch.int32).cuda(),
                         kv_len=torch.tensor([L], dtype=torch.int32).cuda(), block_table=perm.to(torch.int32)[None].contiguous().cuda(),
                         n_kv=G, page_size=P, window=window, keep_first=keep_first, scale=scale,
                         q_lens=None if n_new == 1 else [n_new], bias=bias.cuda(), gate=packed.cuda()[:, 2:2 + H], out_scale=1.25)
    got = out[:, 8:].float().cpu().view(n_new, H, d)
    assert torch.isfinite(got).all()
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(got, want.float(), **tol)
    if ops.window_bias_supported(d, dt, H // G):
        # the same through the mma kernels of the paged attention launch: the prefill kernel, and for a few tokens the decode
        # kernel, whole and with the keys cut into pieces (the kept tokens then ride with the first piece)
        bias_log2 = (bias * math.log2(math.e)).contiguous().cuda()
        ungated = (want / torch.sigmoid(gate.double())[:, :, None] / 1.25).float()
        qd, kd, vd = q.to(dt).cuda(), kc.cuda(), vc.cuda()
        common = dict(q_start=torch.tensor([0, n_new], dtype=torch.int32).cuda(), kv_len=torch.tensor([L], dtype=torch.int32).cuda(),
                      block_table=perm.to(torch.int32)[None].contiguous().cuda(), n_kv=G, page_size=P, window=window, scale=scale,
                      uniform_decode=n_new == 1, keep_first=keep_first, bias_log2=bias_log2)
        runs = [(ops.VARIANT_MMA_ROWS, 1)]
        if n_new <= ops.attention_tile_tokens(ops.VARIANT_MMA_DECODE, H // G, d):
            runs += [(ops.VARIANT_MMA_DECODE, 1), (ops.VARIANT_MMA_DECODE, 3)]
        for variant, ns in runs:
            o = torch.full((n_new, H, d), float("nan"), dtype=dt).cuda()
            part_o = torch.empty(ns * n_new * H * d, dtype=torch.float32).cuda() if ns > 1 else None
            part_ml = torch.empty(ns * n_new * H * 2, dtype=torch.float32).cuda() if ns > 1 else None
            nsplit = torch.tensor([ns], dtype=torch.int32).cuda() if ns > 1 else None
            qt = ops.attention_tile_tokens(variant, H // G, d)
            ops.attention(qd, o, kd, vd, nsplit=nsplit, part_o=part_o, part_ml=part_ml, max_split=ns, qlen_min=1, qlen_max=1 << 30,
                          variant=variant, grid_x=-(-n_new // qt), **common)
            if ns > 1:
                ops.attention_combine(part_o, part_ml, None if n_new == 1 else torch.zeros(n_new, dtype=torch.int32).cuda(), nsplit, o, ns)
            assert torch.isfinite(o).all(), (variant, ns)
            torch.testing.assert_close(o.float().cpu(), ungated, rtol=3e-2, atol=3e-2, msg=lambda m: f"variant {variant}, {ns} pieces: {m}")
        if ops.tc_supported(d, dt, H // G) and n_new > ops.attention_tile_tokens(ops.VARIANT_MMA_DECODE, H // G, d):
            # and through the tcgen05 prefill kernel (head size 128)
            o = torch.full((n_new, H, d), float("nan"), dtype=dt).cuda()
            done = ops.attention_tc(qd, o, kd, vd, q_start=common["q_start"], kv_len=common["kv_len"], block_table=common["block_table"],
                                    n_kv=G, page_size=P, window=window, scale=scale, qlen_min=1, qlen_max=1 << 30, q_lens=[n_new],
                                    keep_first=keep_first, bias_log2=bias_log2)
            ops.check_kernel_status()
            if done:
                assert torch.isfinite(o).all()
                torch.testing.assert_close(o.float().cpu(), ungated, rtol=3e-2, atol=3e-2, msg=lambda m: f"tcgen05 kernel: {m}")
            else:
                assert P < 8 or P & (P - 1), "the tcgen05 kernel refused a page size that TMA fetches"
    return want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_new", [1, 13])
@pytest.mark.parametrize("d", [24, 32])
def test_window_attention_sees_exactly_the_window_and_the_kept_tokens(dtype, n_new, d):
    """A key that would take all the weight sits just inside the window, just outside it, on the last kept first token, on
    the first token that is not kept, far behind, and at page borders; for a prompt's portion and for a decoded token."""
    geo = dict(H=6, G=3, d=d, P=4, window=9, keep_first=3, rows=10, far=37, ctx=150)
    wants = {}
    for name, spike in (("inside", (8,)), ("outside", (9,)), ("far", (140,)), ("kept", ("abs", 2)), ("not kept", ("abs", 3)),
                        ("first", ("abs", 0)), ("page border", (4,)), ("self", (0,)), ("none", ("abs", -1))):
        wants[name] = _window_case(dtype, n_new=n_new, spike_at=spike, seed=11, **geo)
    # the cases are told apart by the result: seeing or not seeing that key changes the output grossly
    last = {k: w[-1] for k, w in wants.items()}
    assert (last["inside"] - last["outside"]).abs().max() > 0.3
    assert (last["kept"] - last["not kept"]).abs().max() > 0.3
    assert (last["far"] - last["none"]).abs().max() < 1e-6          # a far key outside both is never seen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_attention_other_geometries(dtype):
    # sixteen heads on one kv head, head size 64, the window wider than the context, kept tokens inside it
    _window_case(dtype, H=16, G=1, d=64, P=16, window=300, keep_first=7, rows=15, far=200, ctx=70, n_new=9, spike_at=(40,), seed=1)
    # one head per kv head, a window of one token, a table of two rows, pages of one token
    _window_case(dtype, H=3, G=3, d=16, P=1, window=1, keep_first=4, rows=2, far=5, ctx=40, n_new=5, spike_at=("abs", 3), seed=2)
    # no kept tokens, head size above 128, nothing cached before the portion (the first tokens of a sequence)
    _window_case(dtype, H=2, G=2, d=160, P=8, window=33, keep_first=0, rows=20, far=130, ctx=0, n_new=70, spike_at=(32,), seed=3)
    _window_case(dtype, H=2, G=1, d=40, P=4, window=5, keep_first=17, rows=8, far=64, ctx=0, n_new=2, spike_at=(1,), seed=4)
    # decoding the second token of a sequence; decoding with the window's far edge on a page border
    _window_case(dtype, H=4, G=2, d=32, P=4, window=8, keep_first=2, rows=8, far=64, ctx=1, n_new=1, spike_at=(1,), seed=5)
    _window_case(dtype, H=4, G=2, d=32, P=4, window=8, keep_first=2, rows=8, far=64, ctx=31, n_new=1, spike_at=(7,), seed=6)
    # head size 128 (the tcgen05 prefill kernel): kept tokens in a tile of their own, the window's edge, the first tokens of a
    # sequence (no tile before the window), a window wider than the context, one kv head for eight query heads
    for spike in (("abs", 69), (199,), ("abs", 70), (200,)):
        _window_case(dtype, H=8, G=2, d=128, P=16, window=200, keep_first=70, rows=24, far=300, ctx=700, n_new=200, spike_at=spike, seed=9)
    _window_case(dtype, H=4, G=2, d=128, P=16, window=150, keep_first=5, rows=24, far=100, ctx=0, n_new=400, spike_at=(149,), seed=10)
    _window_case(dtype, H=8, G=1, d=128, P=32, window=1000, keep_first=9, rows=16, far=300, ctx=100, n_new=150, spike_at=(120,), seed=11)
    _window_case(dtype, H=2, G=2, d=128, P=8, window=130, keep_first=140, rows=6, far=50, ctx=300, n_new=260, spike_at=("abs", 139), seed=12)
    # a window of several key tiles with kept tokens far before it: a decoded token, a short run and a long portion
    for n_new in (1, 3, 90):
        _window_case(dtype, H=8, G=2, d=96, P=16, window=200, keep_first=70, rows=24, far=300, ctx=700, n_new=n_new, spike_at=("abs", 69), seed=7)
        _window_case(dtype, H=8, G=2, d=96, P=16, window=200, keep_first=70, rows=24, far=300, ctx=700, n_new=n_new, spike_at=(199,), seed=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decaying_linear_attention_in_portions_and_batches(dtype):
    """Three requests with states of their own, fed in different portions in shared steps (a long decode among them),
    against the recurrence written out; decays down to 0.3 and up to 1."""
    from mini_sglang_b200 import ops
    g = torch.Generator().manual_seed(7)
    heads, dk, dv = 3, 12, 20
    decay = [0.3, 0.97, 1.0]
    dt = DT[dtype]
    lens = {0: 90, 1: 37, 2: 64}
    Nk, Nv = heads * dk, heads * dv
    u = {r: torch.randn(n, 2 * Nk + Nv + 5, generator=g).to(dt).float() for r, n in lens.items()}
    cuts = {0: [1] * 90, 1: [30, 2, 2, 3], 2: [5, 40, 1, 1, 17]}
    state = torch.full((5, heads, dk, dv), float("nan")).cuda()
    state[1:4].zero_()
    at = {r: 0 for r in lens}
    got = {r: [] for r in lens}
    while any(cuts.values()):
        reqs = [r for r in (2, 0, 1) if cuts[r]]
        ns = [cuts[r].pop(0) for r in reqs]
        x = torch.cat([u[r][at[r]:at[r] + n] for r, n in zip(reqs, ns)]).to(dt).cuda()
        q_start = torch.tensor(np.concatenate(([0], np.cumsum(ns))), dtype=torch.int32).cuda()
        slots = torch.tensor([r + 1 for r in reqs], dtype=torch.int32).cuda()
        o = ops.decay_attention(x[:, 2:2 + Nk], x[:, 2 + Nk:2 + 2 * Nk], x[:, 2 + 2 * Nk:2 + 2 * Nk + Nv], heads=heads,
                                decay=torch.tensor(decay).cuda(), state=state, q_start=q_start, slots=slots)
        k = 0
        for r, n in zip(reqs, ns):
            got[r].append(o[k:k + n].cpu())
            k += n
            at[r] += n
    silu = torch.nn.functional.silu
    for r, n in lens.items():
        q = silu(u[r][:, 2:2 + Nk].double()).view(n, heads, dk)
        k = silu(u[r][:, 2 + Nk:2 + 2 * Nk].double()).view(n, heads, dk)
        v = silu(u[r][:, 2 + 2 * Nk:2 + 2 * Nk + Nv].double()).view(n, heads, dv)
        want = torch.zeros(n, heads, dv, dtype=torch.float64)
        for h in range(heads):
            S = torch.zeros(dk, dv, dtype=torch.float64)
            for t in range(n):
                S = decay[h] * S + k[t, h][:, None] * v[t, h][None, :]
                want[t, h] = S.T @ q[t, h]
        torch.testing.assert_close(torch.cat(got[r]), want.view(n, Nv).float(), rtol=2e-5, atol=2e-5)


# ---------------------------------------------------------------------------------------------------------------------
# the model through the step function
# ---------------------------------------------------------------------------------------------------------------------
LENGTHS = {"VA": 61, "VB": 40, "VC": 75}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["VA", "VB", "VC"])
def test_whole_prompt_token_by_token_and_in_portions(name, dtype):
    """The same sequence three ways: one step; five tokens and then one token a step (through the CUDA graph); portions of
    changing sizes down to two tokens.  Every position against the plain implementation."""
    V = CONFIGS_V[name]["vocab"]
    n = LENGTHS[name]
    toks = random_tokens(n, V, 100 + n)
    seqs = {"w": toks, "d": toks, "p": toks}
    r = runner(name, dtype, num_pages=3 * (-(-n // PAGE[name])) + 8)
    poison(r)
    got = play(r, [{"entries": [("w", toks, list(range(n)))], "end": ["w"]}])
    compare(name, dtype, got, seqs)
    steps = [{"entries": [("d", toks[:5], list(range(5)))]}] + [{"entries": [("d", [t], [0])]} for t in toks[5:]]
    got = play(r, steps)
    assert r.last_step_used_graph
    compare(name, dtype, got, seqs)
    sizes, at, steps = [2, 3, 7, 2, 16, 1, 1, 2, 5, 2, 9], 0, []
    while at < n:
        c = min(sizes[len(steps) % len(sizes)], n - at)
        steps.append({"entries": [("p", toks[at:at + c], list(range(c)))]})
        at += c
    got = play(r, steps)
    compare(name, dtype, got, seqs)
    assert len(got) == n
    r.mgr.check_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["VA", "VC"])
def test_mixed_batches_on_a_small_pool(name, dtype):
    """Five requests of unequal lengths through two request slots and a pool that holds little more than the two longest:
    portions of one beside single tokens of another; pages, block-table rows and state rows are used again, and what
    they held before (NaN at the start) must never be read."""
    V = CONFIGS_V[name]["vocab"]
    P = PAGE[name]
    lens = {"a": 50, "b": 23, "c": 1, "d": 66, "e": 34}
    seqs = {k: random_tokens(n, V, 7 + n) for k, n in lens.items()}
    r = runner(name, dtype, num_pages=-(-66 // P) + -(-50 // P) + 1, max_reqs=2)
    poison(r)
    a, b, c, d, e = (seqs[k] for k in "abcde")
    steps = [
        {"entries": [("a", a[:17], [0, 16]), ("b", b[:2], [1])]},
        {"entries": [("b", b[2:3], [0]), ("a", a[17:40], [5, 22])]},
        {"entries": [("a", a[40:41], [0]), ("b", b[3:23], list(range(20)))], "end": ["b"]},
        {"entries": [("c", c, [0]), ("a", a[41:42], [0])], "end": ["c"]},
        {"entries": [("a", a[42:43], [0]), ("d", d[:30], [29])]},
        {"entries": [("d", d[30:60], [0, 29]), ("a", a[43:50], list(range(7)))], "end": ["a"]},
        {"entries": [("d", d[60:61], [0]), ("e", e[:9], [8])]},
        {"entries": [("e", e[9:11], [0, 1]), ("d", d[61:62], [0])]},
    ] + [{"entries": [("d", d[62 + i:63 + i], [0]), ("e", e[11 + i:12 + i], [0])]} for i in range(4)] + [
        {"entries": [("e", e[15:34], [18])], "end": ["d", "e"]},
    ]
    got = play(r, steps)
    compare(name, dtype, got, seqs)
    r.mgr.check_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_every_window(dtype):
    """Two requests decode together for 140 steps through the CUDA graph: the window leaves the prompt, pages behind it are
    given back while the first tokens' pages stay, and the linear attention's state carries everything."""
    name = "VA"
    V = CONFIGS_V[name]["vocab"]
    P = PAGE[name]
    a, b = random_tokens(150, V, 1), random_tokens(160, V, 2)
    seqs = {"a": a, "b": b}
    r = runner(name, dtype, num_pages=24, max_reqs=2)
    poison(r)
    steps = [{"entries": [("a", a[:10], [9]), ("b", b[:20], [19])]}]
    steps += [{"entries": [("a", [a[10 + i]], [0]), ("b", [b[20 + i]], [0])]} for i in range(140)]
    got = play(r, steps)
    assert r.last_step_used_graph
    compare(name, dtype, got, seqs)
    # 310 tokens went through a pool of 24 pages of 4: the window gave pages back, the kept first tokens' page stayed
    assert r.mgr.groups[0].keep_pages == 1
    r.mgr.check_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype):
    """Engine.generate with the scheduler: prompts of unequal lengths, portions of at most 16 tokens, a small pool."""
    from mini_sglang_b200 import Engine, EngineArgs
    name = "VA"
    cfg = config_json(CONFIGS_V[name])
    prompts = [random_tokens(n, cfg["vocab"], 50 + n) for n in (5, 33, 18)]
    eng = Engine(EngineArgs(model=model_dir(name), dtype=dtype, page_size=4, num_pages=48, max_num_reqs=3, random_seed=0,
                            chunk_size=16, max_context_len=256, log_level="WARNING"))
    outs = eng.generate(input_ids=prompts, sampling_params={"temperature": 0.0, "max_new_tokens": 12, "ignore_eos": True})
    for p, o in zip(prompts, outs):
        got = o["token_ids"]
        assert len(got) == 12
        if dtype == "float32":
            assert got == pv.greedy_generate(cfg, weights(name), p, 12)
        else:
            toks = list(p)
            for t in got:           # bfloat16 may take another of two nearly equal logits
                row = pv.forward_sequence(cfg, weights(name), toks)[-1]
                assert float(row.max() - row[t]) < 0.05 * float(row.std()) + 0.05
                toks.append(t)
    eng.scheduler.check_idle_invariants()


def test_trace_replay_program(tmp_path):
    name = "VB"
    V = CONFIGS_V[name]["vocab"]
    a, b = random_tokens(37, V, 1), random_tokens(21, V, 2)
    lines = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[20:35], "want": []}, {"id": "b", "tokens": b[:21], "want": [20]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[35:36], "want": [0]}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[36:37], "want": [0]}], "end": ["a"]},
    ]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir(name), "--dtype", dtype,
                               "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(l) for l in lines) + "\n",
                              capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(4)]
        ra, rb = plain(name, tuple(a)), plain(name, tuple(b))
        rd = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V))        # noqa: E731
        for got, want in ((rd(0), ra[[0, 19]]), (rd(1), rb[[20]]), (rd(2), ra[[35]]), (rd(3), ra[[36]])):
            assert got.shape == want.shape
            for g_row, w_row in zip(got, want):
                row_close(g_row, w_row, dtype)
