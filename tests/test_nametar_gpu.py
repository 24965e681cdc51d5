"""The Nametar parts and the whole model in the engine against the plain implementation (tests/plain_nametar.py).

Kernels one by one, the attention over a cache of latents with inputs made so that a fault shows (one key whose score stands
out: far away, just inside and just outside the window, the first token, at page borders), then the model through the step
function: whole prompts, token by token, in portions down to two tokens, mixed batches on a pool so small that pages and
request slots are used again, long decoding past every window, greedy generation through the engine's entry point, and the
trace replay program.
"""

import functools
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_nametar as pn
from helpers import assert_row_close, play
from tiny_models import random_tokens, write_model_dir
from tiny_nametar import CONFIGS_N, config_json, make_weights

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEED = {"NA": 3, "NB": 4, "NC": 5}
PAGE = {"NA": 4, "NB": 1, "NC": 16}
_tmp = tempfile.TemporaryDirectory(prefix="msgl_nametar_")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


@functools.lru_cache(None)
def weights(name):
    return make_weights(CONFIGS_N[name], SEED[name])


@functools.lru_cache(None)
def model_dir(name):
    return write_model_dir(os.path.join(_tmp.name, name), config_json(CONFIGS_N[name]), weights(name))


@functools.lru_cache(None)
def plain(name, tokens):
    with torch.no_grad():
        return pn.forward_sequence(config_json(CONFIGS_N[name]), weights(name), list(tokens)).float()


def runner(name, dtype, num_pages, max_reqs=4, page_size=None, graphs=True):
    from mini_sglang_b200.engine.step import ModelRunner
    return ModelRunner.from_model_dir(model_dir(name), dtype=dtype, page_size=page_size or PAGE[name], num_pages=num_pages,
                                      max_reqs=max_reqs, max_context_len=4096, use_cuda_graph=graphs)


# bfloat16: every sublayer's output is normed to unit size before it is added, so the rounding of a sublayer's last product
# reaches the stream undamped, and a layer rounds at more places than a plain attention layer (both latents, the folded query,
# what the heads gather of the latent, the gated heads).  The noise of the logits stays below about 1.5 % of a row's rms at
# these widths (up to 2.6 % after 100 decoded tokens); the bound is 3 %.  A window one token wider, another tau or a missing factor moves the rows by 4 % or more
# (tests/test_nametar_cpu.py).  Configuration NB adds every sublayer's normed output at full weight into a stream 48 wide and
# takes its decays with tau 1: its noise reaches 3.5 %, its bound is 5 %, and a window one token wider or another tau moves its
# rows by 11 % or more.
BF16_RMS_FRACTION_N = 0.03
BF16_RMS_FRACTION_BY_CONFIG = {"NB": 0.05}


def row_close(row, want, dtype, bound=BF16_RMS_FRACTION_N):
    if dtype == "float32":
        return assert_row_close(row, want, dtype)
    row, want = row.float(), want.float()
    assert torch.isfinite(row).all(), "logits are not finite"
    err = row - want
    scale = want.pow(2).mean().sqrt().item()
    rms, worst = err.pow(2).mean().sqrt().item(), err.abs().max().item()
    assert rms <= bound * scale, f"rms error {rms:.4g} is {rms / scale:.2%} of the row's rms {scale:.4g}"
    assert worst <= 6.0 * bound * scale, f"largest error {worst:.4g} is {worst / scale:.2%} of the row's rms {scale:.4g}"


def compare(name, dtype, got, seqs):
    """Every row against the plain implementation.  bfloat16: rounding noise has outliers (a row whose sums nearly cancel before
    a norm), so one row in fifty (at least one) may pass the bound, none by more than two and a half times; a fault of the
    cache, a window or a state moves every row behind it by more than that."""
    assert got
    bound = BF16_RMS_FRACTION_BY_CONFIG.get(name, BF16_RMS_FRACTION_N)
    over = []
    for (rid, pos), row in sorted(got.items()):
        want = plain(name, tuple(seqs[rid]))[pos]
        try:
            row_close(row, want, dtype, bound)
        except AssertionError as e:
            if dtype == "bfloat16" and torch.isfinite(row).all():
                try:
                    row_close(row, want, dtype, 2.5 * bound)
                    over.append((rid, pos))
                    continue
                except AssertionError:
                    pass
            raise AssertionError(f"request {rid!r} position {pos} ({dtype}, {name}): {e}") from None
    assert len(over) <= max(1, len(got) // 50), f"{len(over)} of {len(got)} rows beyond the bound ({dtype}, {name}): {over[:8]}"


def poison(r):
    """Whatever a page or a state row held before must not be read: fill the caches with NaN (state rows are zeroed when a
    request is opened).  Page 0 and state row 0 are never handed out: it stands in for pages that a window gave back and takes the rows of padded
    batch rows, so it holds finite numbers at all times, and a masked key may be fetched from it."""
    for k, v in r.storage.kv.values():
        k[1:].fill_(float("nan"))
        v[1:].fill_(float("nan"))
    for s in r.storage.state.values():          # row 0 belongs to the padded rows of a captured batch, as page 0 does
        s[1:].fill_(float("nan"))


def tol_of(dtype, f32=1e-5, bf16=2e-2):
    return dict(rtol=f32, atol=f32) if dtype == "float32" else dict(rtol=bf16, atol=bf16)


# ---------------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scaled_embedding(dtype):
    from mini_sglang_b200 import ops
    g = torch.Generator().manual_seed(0)
    table = torch.randn(23, 70, generator=g).to(DT[dtype])
    ids = torch.tensor([5, 0, 22, 5, 11], dtype=torch.int32)
    got = ops.scaled_embedding(ids.cuda(), table.cuda(), 17.25).cpu()
    torch.testing.assert_close(got, table.float()[ids.long()] * 17.25, rtol=1e-6, atol=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [70, 1024, 4100, 5000, 8192, 9000])
def test_output_norm_sum_and_next_input_norm(dtype, H):
    from mini_sglang_b200 import ops
    g = torch.Generator().manual_seed(H)
    T, dt = 7, DT[dtype]
    res = torch.randn(T, H, generator=g)
    wa, wy = 1 + 0.1 * torch.randn(H, generator=g), 1 + 0.1 * torch.randn(H, generator=g)
    for a_dt in {dt, torch.float32}:
        a = (3 * torch.randn(T, H, generator=g)).to(a_dt)
        want_res = res.double() + 0.6 * pn.rms_scale(a.double(), wa.double(), 1e-5)
        want_y = pn.rms_scale(want_res, wy.double(), 1e-3)
        r1 = res.clone().cuda()
        y = ops.postnorm_residual(a.cuda(), wa.cuda(), 1e-5, 0.6, r1, next_weight=wy.cuda(), next_eps=1e-3, out_dtype=dt)
        torch.testing.assert_close(r1.cpu(), want_res.float(), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(y.float().cpu(), want_y.float(), **tol_of(dtype))
        r2 = res.clone().cuda()
        assert ops.postnorm_residual(a.cuda(), wa.cuda(), 1e-5, 0.6, r2, out_dtype=dt) is None
        torch.testing.assert_close(r2.cpu(), want_res.float(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geo", [dict(q_rank=20, r=24, rd=8, dims=8, H=3, dk=8, sc={"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}),
                                 dict(q_rank=0, r=20, rd=8, dims=4, H=1, dk=20, sc=None),
                                 dict(q_rank=33, r=112, rd=16, dims=16, H=16, dk=16, sc={"factor": 2.0, "original": 64, "fast": 16.0, "slow": 2.0}),
                                 dict(q_rank=0, r=48, rd=0, dims=0, H=4, dk=16, sc=None)])
def test_latents_cache_rows_and_query_rotation(dtype, geo):
    """The query latent, the cache row of a token (normed latent, rotated shared key part) and the rotated part of every
    query head against the plain functions, at positions far beyond any table and with pages in any order."""
    from mini_sglang_b200 import ops
    from mini_sglang_b200.parts.rope import yarn_frequencies
    q_rank, r, rd, dims, H, dk = (geo[k] for k in ("q_rank", "r", "rd", "dims", "H", "dk"))
    g = torch.Generator().manual_seed(r)
    dt, T, P = DT[dtype], 11, 4
    pos = torch.tensor([0, 1, 2, 3, 100, 101, 5000, 77777, 9, 10, 11], dtype=torch.int32)
    off = 3 if dtype == "float32" else 8
    proj = torch.randn(T, off + q_rank + r + rd + 5, generator=g).to(dt)
    wq, wc = 1 + 0.1 * torch.randn(max(q_rank, 1), generator=g), 1 + 0.1 * torch.randn(r, generator=g)
    freq = mag = None
    if rd:
        f64, mag = yarn_frequencies(dims, 100.0, geo["sc"])
        freq = f64.float().cuda()
    loc = (torch.randperm(6 * P, generator=g)[:T] + P).to(torch.int32)
    cache = torch.full((7, 1, P, r + rd), float("nan"), dtype=dt).cuda()
    cq = ops.latent_prep(proj.cuda(), dq_off=off, q_rank=q_rank, dkv_off=off + q_rank, kv_rank=r, rot_dim=rd, rot_dims=dims,
                         dq_norm=wq[:q_rank].cuda() if q_rank else None, dkv_norm=wc.cuda(), eps=1e-5, freq=freq, mag=mag or 1.0,
                         positions=pos.cuda(), out_loc=loc.cuda(), cache=cache, page_size=P)
    p64 = proj.double()
    if q_rank:
        torch.testing.assert_close(cq.float().cpu(), pn.rms_scale(p64[:, off:off + q_rank], wq[:q_rank].double(), 1e-5).float(), **tol_of(dtype))
    else:
        assert cq is None
    rows = cache.float().cpu().view(-1, r + rd)[loc.long()]
    torch.testing.assert_close(rows[:, :r], pn.rms_scale(p64[:, off + q_rank:off + q_rank + r], wc.double(), 1e-5).float(), **tol_of(dtype))
    untouched = torch.ones(7 * P, dtype=torch.bool)
    untouched[loc.long()] = False
    assert torch.isnan(cache.float().cpu().view(-1, r + rd)[untouched]).all()
    if not rd:
        return
    wf, wmag = pn.rotary_frequencies(dims, 100.0, geo["sc"])
    kr = p64[:, off + q_rank + r:off + q_rank + r + rd]
    want = torch.stack([pn.rotate(kr[t], int(pos[t]), wf, wmag, dims) for t in range(T)])
    torch.testing.assert_close(rows[:, r:], want.float(), **tol_of(dtype, 2e-5))
    q = torch.randn(T, H * (dk + rd) + 8, generator=g).to(dt)
    q3 = q[:, :H * (dk + rd)].unflatten(1, (H, dk + rd)).cuda()
    qf = torch.zeros(T, H, r + rd, dtype=dt).cuda()
    ops.rope_heads(q3, dk, qf, r, rot_dim=rd, rot_dims=dims, freq=freq, mag=mag, positions=pos.cuda())
    want_q = torch.stack([torch.stack([pn.rotate(q3[t, h, dk:].double().cpu(), int(pos[t]), wf, wmag, dims) for h in range(H)]) for t in range(T)])
    torch.testing.assert_close(qf[:, :, r:].float().cpu(), want_q.float(), **tol_of(dtype, 2e-5))
    assert float(qf[:, :, :r].abs().sum()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [13, 200, 512, 530])
def test_gates(dtype, d):
    from mini_sglang_b200 import ops
    g = torch.Generator().manual_seed(1)
    T, heads, dt = 5, 3, DT[dtype]
    N = heads * d
    packed = (2 * torch.randn(T, N + 6, generator=g)).to(dt).cuda()
    x = torch.randn(T, N, generator=g).to(dt).cuda()
    out = torch.zeros(T, N + 4, dtype=dt).cuda()
    ops.gate_mul(packed[:, 3:3 + N], x, out[:, 2:2 + N], ops.ACT_SIGMOID)
    torch.testing.assert_close(out[:, 2:2 + N].float().cpu(), (torch.sigmoid(packed[:, 3:3 + N].double()) * x.double()).float().cpu(), **tol_of(dtype))
    assert float(out[:, :2].abs().sum()) == 0 and float(out[:, 2 + N:].abs().sum()) == 0
    if N + 3 + N <= packed.shape[1] + N:          # the packed-row form with gate and input side by side in the same rows
        both = torch.cat((packed[:, 3:3 + N], x), dim=1).contiguous()
        out3 = torch.zeros(T, N, dtype=dt).cuda()
        ops.gated_act(both[:, :N], both[:, N:], out3, ops.ACT_SIGMOID)
        torch.testing.assert_close(out3.float().cpu(), (torch.sigmoid(both[:, :N].double()) * both[:, N:].double()).float().cpu(), **tol_of(dtype))
    ops.gate_mul(packed[:, 3:3 + N], x, x, ops.ACT_SILU)          # in place
    o = torch.randn(T, N, generator=g)
    w = 1 + 0.1 * torch.randn(d, generator=g)
    out2 = torch.zeros(T, N + 4, dtype=dt).cuda()
    ops.group_rms_gate(o.cuda(), heads, w.cuda(), 1e-4, packed[:, 3:3 + N], out2[:, 4:], ops.ACT_SILU)
    want = pn.rms_scale(o.double().view(T, heads, d), w.double(), 1e-4).reshape(T, N) * pn.silu(packed[:, 3:3 + N].double().cpu())
    torch.testing.assert_close(out2[:, 4:].float().cpu(), want.float(), **tol_of(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geo", [(3, 12, 20, 4.0), (1, 36, 8, 1.0), (2, 64, 70, 16.0)])
def test_gated_linear_attention_in_portions_and_batches(dtype, geo):
    """Three requests with states of their own, fed in different portions in shared steps (a long decode among them), against
    the recurrence written out; decays from nearly 0 to nearly 1 in the same head."""
    from mini_sglang_b200 import ops
    heads, dk, dv, tau = geo
    g = torch.Generator().manual_seed(7)
    dt = DT[dtype]
    lens = {0: 90, 1: 37, 2: 150}
    Nk, Nv = heads * dk, heads * dv
    u = {r: torch.randn(n, 2 * Nk + Nv + 5, generator=g).to(dt).float() for r, n in lens.items()}
    z = {r: 4.0 * torch.randn(n, Nk, generator=g) for r, n in lens.items()}
    bias = torch.linspace(-12.0, 12.0, Nk)
    cuts = {0: [1] * 90, 1: [30, 2, 2, 3], 2: [5, 70, 1, 1, 73]}
    state = torch.full((5, heads, dk, dv), float("nan")).cuda()
    state[1:4].zero_()
    at = {r: 0 for r in lens}
    got = {r: [] for r in lens}
    while any(cuts.values()):
        reqs = [r for r in (2, 0, 1) if cuts[r]]
        ns = [cuts[r].pop(0) for r in reqs]
        x = torch.cat([u[r][at[r]:at[r] + n] for r, n in zip(reqs, ns)]).to(dt).cuda()
        zz = torch.cat([z[r][at[r]:at[r] + n] for r, n in zip(reqs, ns)]).cuda()
        q_start = torch.tensor(np.concatenate(([0], np.cumsum(ns))), dtype=torch.int32).cuda()
        slots = torch.tensor([r + 1 for r in reqs], dtype=torch.int32).cuda()
        o = ops.gated_decay_attention(x[:, 2:2 + Nk], x[:, 2 + Nk:2 + 2 * Nk], x[:, 2 + 2 * Nk:2 + 2 * Nk + Nv], zz, bias.cuda(),
                                      heads=heads, tau=tau, q_scale=0.37, state=state, q_start=q_start, slots=slots,
                                      q_lens=None if all(n == 1 for n in ns) else ns)
        k = 0
        for r, n in zip(reqs, ns):
            got[r].append(o[k:k + n].cpu())
            k += n
            at[r] += n
    for r, n in lens.items():
        q = u[r][:, 2:2 + Nk].double().view(n, heads, dk) * 0.37
        k = u[r][:, 2 + Nk:2 + 2 * Nk].double().view(n, heads, dk)
        v = u[r][:, 2 + 2 * Nk:2 + 2 * Nk + Nv].double().view(n, heads, dv)
        alpha = (torch.sigmoid(z[r].double() + bias.double()) ** (1.0 / tau)).view(n, heads, dk)
        want = torch.zeros(n, heads, dv, dtype=F64)
        for h in range(heads):
            S = torch.zeros(dk, dv, dtype=F64)
            for t in range(n):
                S = alpha[t, h][:, None] * S + k[t, h][:, None] * v[t, h][None, :]
                want[t, h] = S.T @ q[t, h]
        torch.testing.assert_close(torch.cat(got[r]), want.view(n, Nv).float(), rtol=1e-4, atol=1e-4)
    assert torch.isnan(state[0]).all() and torch.isnan(state[4]).all()


def _latent_case(dtype, *, H, D, P, window, ctx, n_new, spike_at, seed, splits=1):
    """One request with `ctx` cached tokens and `n_new` new ones over a cache whose rows are keys and values at once (one kv
    head for all H query heads), through the launches the latent attention makes.  Queries and rows are small random vectors
    except that every query and the row at distance `spike_at[0]` from the last query (or, given as ("abs", j), at position j)
    share a large component: that row takes nearly all the weight wherever the mask lets it be seen."""
    from mini_sglang_b200 import ops
    from mini_sglang_b200.parts.attention import paged_attend
    from mini_sglang_b200.parts.context import GroupContext, KVCacheView, StepContext, Workspace
    g = torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    L = ctx + n_new
    q = 0.3 * torch.randn(n_new, H, D, generator=g)
    k = 0.3 * torch.randn(L, D, generator=g)
    k[:, 1] = torch.arange(L) % 7 - 3.0                 # the gathered values tell which rows were seen
    j_star = spike_at[1] if spike_at[0] == "abs" else L - 1 - spike_at[0]
    q[:, :, 0] += 6.0
    if 0 <= j_star < L:
        k[j_star, 0] += 6.0
    q, k = q.to(dt).float(), k.to(dt).float()
    scale = 0.5
    want = torch.zeros(n_new, H, D, dtype=F64)
    for t in range(n_new):
        i = ctx + t
        js = torch.tensor([j for j in range(i + 1) if pn.visible(i, j, window)])
        for h in range(H):
            a = torch.softmax((k[js].double() @ q[t, h].double()) * scale, 0)
            want[t, h] = a @ k[js].double()
    n_pages = -(-L // P)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages] + 1
    kc = torch.full((n_pages + 4, 1, P, D), float("nan"), dtype=dt)
    kc[0] = 0.0          # the page that stands in for pages given back holds finite rows
    for p in range(L):
        kc[perm[p // P], 0, p % P] = k[p].to(dt)
    if window:          # pages wholly behind the window of the first new token may have been given back: their table entries are 0
        dead = max(0, (ctx - window + 1) // P)
        perm = perm.clone()
        perm[:dead] = 0
    kc = kc.cuda()
    dev = kc.device
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)          # noqa: E731
    uniform = n_new == 1
    grp = GroupContext(block_table=perm.to(torch.int32)[None].contiguous().cuda(), out_loc=i32([0] * n_new),
                       nsplit=i32([splits]) if splits > 1 else None, max_split=splits, window=window, host_nsplit=[splits],
                       order=i32([0]) if uniform else None)
    sc = StepContext(T=n_new, B=1, page_size=P, input_ids=None, positions=None, q_start=i32([0, n_new]), kv_len=i32([L]),
                     token_req=i32([0] * n_new), slots=i32([1]), groups=[grp], host_q_lens=[n_new], host_kv_lens=[L],
                     host_slots=[1], uniform_decode=uniform, workspace=Workspace(dev))
    out = torch.full((n_new, H, D), float("nan"), dtype=dt, device=dev)
    paged_attend(q.to(dt).cuda(), out, sc, KVCacheView(kc, kc, grp, P), n_q=H, n_kv=1, d=D, window=int(window or 0), scale=scale,
                 use_mma=ops.mma_supported(D, dt))
    ops.check_kernel_status()
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want.float(), **tol_of(dtype, 1e-4, 3e-2))
    return want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_new", [1, 2, 13])
@pytest.mark.parametrize("D", [28, 32, 48])
def test_attention_over_latents_sees_exactly_the_window(dtype, n_new, D):
    """A row that would take all the weight sits just inside the window, just outside it, far behind, on the first token, and
    at page borders; for a prompt's portion and for a decoded token."""
    geo = dict(H=3, D=D, P=4, window=9, ctx=150)
    wants = {}
    for name, spike in (("inside", (8,)), ("outside", (9,)), ("far", (140,)), ("first", ("abs", 0)), ("page border", (4,)),
                        ("self", (0,)), ("none", ("abs", -1))):
        wants[name] = _latent_case(dtype, n_new=n_new, spike_at=spike, seed=11, **geo)
    last = {k: w[-1] for k, w in wants.items()}
    assert (last["inside"] - last["outside"]).abs().max() > 0.3
    assert (last["far"] - last["none"]).abs().max() < 1e-6          # a far row outside the window is never seen
    assert (last["first"] - last["none"]).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_over_latents_other_geometries(dtype):
    # no window: a far row among hundreds is seen, by a decoded token (whole and with the keys cut into pieces) and by a portion
    for n_new, splits in ((1, 1), (1, 3), (40, 1), (2, 1)):
        w1 = _latent_case(dtype, H=8, D=64, P=16, window=None, ctx=700, n_new=n_new, spike_at=("abs", 3), seed=1, splits=splits)
        w0 = _latent_case(dtype, H=8, D=64, P=16, window=None, ctx=700, n_new=n_new, spike_at=("abs", -1), seed=1, splits=splits)
        assert (w1[-1] - w0[-1]).abs().max() > 0.3
    # sixteen heads on a row of 128 (the tcgen05 prefill kernel in bfloat16): the window's edge within a long portion, the first
    # tokens of a sequence, a window wider than the context
    for spike in ((199,), (200,)):
        _latent_case(dtype, H=16, D=128, P=16, window=200, ctx=700, n_new=200, spike_at=spike, seed=9)
    _latent_case(dtype, H=16, D=128, P=16, window=150, ctx=0, n_new=400, spike_at=(149,), seed=10)
    _latent_case(dtype, H=4, D=128, P=32, window=1000, ctx=100, n_new=150, spike_at=(120,), seed=11)
    # a window of one token; pages of one token; the second token of a sequence; the window's far edge on a page border
    _latent_case(dtype, H=1, D=28, P=1, window=1, ctx=40, n_new=5, spike_at=(1,), seed=2)
    _latent_case(dtype, H=5, D=144, P=16, window=96, ctx=1, n_new=1, spike_at=(1,), seed=5)
    _latent_case(dtype, H=5, D=144, P=16, window=96, ctx=300, n_new=1, spike_at=(95,), seed=6, splits=2)
    _latent_case(dtype, H=4, D=32, P=4, window=8, ctx=31, n_new=1, spike_at=(7,), seed=6)
    _latent_case(dtype, H=2, D=160, P=8, window=33, ctx=0, n_new=70, spike_at=(32,), seed=3)
    _latent_case(dtype, H=20, D=80, P=8, window=64, ctx=200, n_new=3, spike_at=(63,), seed=4)


# ---------------------------------------------------------------------------------------------------------------------
# the model through the step function
# ---------------------------------------------------------------------------------------------------------------------
LENGTHS = {"NA": 61, "NB": 40, "NC": 75}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("NA", None), ("NB", None), ("NC", None), ("NA", 16), ("NB", 8), ("NC", 1)])
def test_whole_prompt_token_by_token_and_in_portions(name, page, dtype):
    """The same sequence three ways: one step; five tokens and then one token a step (through the CUDA graph); portions of
    changing sizes down to two tokens.  Every position against the plain implementation; with each configuration's own page
    size and with another (pages wider than a window, pages of one token)."""
    V = CONFIGS_N[name]["vocab"]
    n = LENGTHS[name]
    toks = random_tokens(n, V, 100 + n)
    seqs = {"w": toks, "d": toks, "p": toks}
    r = runner(name, dtype, num_pages=3 * (-(-n // (page or PAGE[name]))) + 8, page_size=page)
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
@pytest.mark.parametrize("name", ["NA", "NC"])
def test_mixed_batches_on_a_small_pool(name, dtype):
    """Five requests of unequal lengths through two request slots and a pool that holds little more than the two longest:
    portions of one beside single tokens of another; pages, block-table rows and state rows are used again, and what
    they held before (NaN at the start) must never be read."""
    V = CONFIGS_N[name]["vocab"]
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
    # each request alone gives the same rows as in the batch, beyond rounding
    alone = play(r, [{"entries": [("a", a, [0, 16, 22, 39, 40, 41, 42, 49])], "end": ["a"]}])
    for (rid, pos), row in alone.items():
        row_close(got[(rid, pos)], row, dtype) if dtype == "bfloat16" else torch.testing.assert_close(got[(rid, pos)], row, rtol=1e-4, atol=2e-5)
    r.mgr.check_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["NA", "NB"])
def test_long_decoding_past_every_window(name, dtype):
    """Two requests decode together for 140 steps through the CUDA graph: the windows leave the prompt, pages behind them are
    given back and used again, and the linear attention's state carries everything."""
    V = CONFIGS_N[name]["vocab"]
    a, b = random_tokens(150, V, 1), random_tokens(160, V, 2)
    seqs = {"a": a, "b": b}
    r = runner(name, dtype, num_pages=-(-330 // PAGE[name]), max_reqs=2)
    poison(r)
    steps = [{"entries": [("a", a[:10], [9]), ("b", b[:20], [19])]}]
    steps += [{"entries": [("a", [a[10 + i]], [0]), ("b", [b[20 + i]], [0])]} for i in range(140)]
    got = play(r, steps)
    assert r.last_step_used_graph
    compare(name, dtype, got, seqs)
    windowed = [g for g in r.mgr.groups if g.window is not None]
    assert windowed and all(g.pool.in_use == 0 for g in r.mgr.groups)
    r.mgr.check_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype):
    """Engine.generate with the scheduler: prompts of unequal lengths, portions of at most 16 tokens, a small pool."""
    from mini_sglang_b200 import Engine, EngineArgs
    name = "NA"
    cfg = config_json(CONFIGS_N[name])
    prompts = [random_tokens(n, cfg["vocab"], 50 + n) for n in (5, 33, 18)]
    eng = Engine(EngineArgs(model=model_dir(name), dtype=dtype, page_size=4, num_pages=48, max_num_reqs=3, random_seed=0,
                            chunk_size=16, max_context_len=256, log_level="WARNING"))
    outs = eng.generate(input_ids=prompts, sampling_params={"temperature": 0.0, "max_new_tokens": 12, "ignore_eos": True})
    for p, o in zip(prompts, outs):
        got = o["token_ids"]
        assert len(got) == 12
        if dtype == "float32":
            assert got == pn.greedy_generate(cfg, weights(name), p, 12)
        else:
            toks = list(p)
            for t in got:           # bfloat16 may take another of two nearly equal logits
                row = pn.forward_sequence(cfg, weights(name), toks)[-1]
                assert float(row.max() - row[t]) < 0.05 * float(row.std()) + 0.05
                toks.append(t)
    eng.scheduler.check_idle_invariants()


def test_trace_replay_program(tmp_path):
    name = "NB"
    V = CONFIGS_N[name]["vocab"]
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
                row_close(g_row, w_row, dtype, BF16_RMS_FRACTION_BY_CONFIG[name])


# ---------------------------------------------------------------------------------------------------------------------
# seeded random configurations
# ---------------------------------------------------------------------------------------------------------------------
def _random_config(seed):
    """Everything the design lets differ, drawn at random: width, vocabulary, number, kinds and order of layers, heads, key /
    value / latent sizes (cache rows that are no multiple of 16 or of 8 among them), query latent or none, rotated dimensions,
    frequency scaling or none, windows, tau, the decay projection's rank, layers without feed-forward, the factors."""
    import random

    import tiny_nametar as tn
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 128])
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["la", "la2", "la2", "gla"])
        ff = rng.choice([None, 24, 56, 96])
        if kind == "gla":
            layer = tn._gla(rng.randint(1, 4), rng.choice([8, 12, 20, 32, 40]), rng.choice([8, 24, 36]), rng.choice([1.0, 3.5, 16.0]),
                            rank=rng.randint(1, 9))
        elif kind == "la":
            layer = tn._la(rng.randint(1, 6), rng.choice([8, 12, 16, 24]), rng.choice([8, 20, 32]), rng.choice([16, 24, 40, 52, 64, 100]),
                           scale=rng.choice([None, 0.2, 0.5]))
        else:
            rot = rng.choice([4, 8, 16])
            layer = tn._la2(rng.randint(1, 6), rng.choice([8, 12, 16, 24]), rot, rng.choice([8, 20, 32]), rng.choice([12, 24, 40, 56, 112]),
                            window=rng.choice([None, 3, 17, 64]), q_rank=rng.choice([None, 9, 32]), dims=rng.choice([rot, rot, rot // 2]),
                            base=rng.choice([10000.0, 200.0]),
                            scaling=rng.choice([None, {"factor": rng.choice([2.0, 8.0]), "original": rng.choice([16, 64]),
                                                       "fast": rng.choice([4.0, 16.0]), "slow": rng.choice([0.5, 1.0])}]))
        layers.append(tn._with(layer, ff))
    return tn._model(width, rng.choice([33, 64, 150]), rng.choice([1e-5, 1e-6]), rng.choice([0.3, 0.5, 0.8]), rng.choice([1.0, 2.5, 7.0]),
                     layers), rng.choice([1, 2, 4, 8, 16])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(seed, dtype):
    """A random model whole, token by token through the graph, and in portions beside another request's single tokens.
    float32: every row element by element.  bfloat16: how much rounding moves a row depends on the configuration drawn (sharp
    softmaxes, norms over a few elements), so the bound is statistical: a row's error within 5 % of its rms, one row in ten up
    to 12.5 %, none beyond; the float32 run of the same configuration holds the logic to 1e-4."""
    from mini_sglang_b200.engine.step import ModelRunner
    cfg, page = _random_config(seed)
    cj, W = config_json(cfg), make_weights(cfg, 100 + seed)
    d = write_model_dir(os.path.join(_tmp.name, f"random{seed}"), cj, W)
    n = 70
    a, b = random_tokens(n, cfg["vocab"], seed), random_tokens(30, cfg["vocab"], 50 + seed)
    with torch.no_grad():
        ref = {"w": pn.forward_sequence(cj, W, a).float(), "b": pn.forward_sequence(cj, W, b).float()}
    ref["d"] = ref["p"] = ref["w"]
    r = ModelRunner.from_model_dir(d, dtype=dtype, page_size=page, num_pages=3 * (-(-n // page)) + 8, max_reqs=3, max_context_len=4096)
    poison(r)
    steps = [{"entries": [("w", a, list(range(n)))], "end": ["w"]}, {"entries": [("d", a[:5], [4])]}]
    steps += [{"entries": [("d", [t], [0])]} for t in a[5:]]
    sizes, at, k = [2, 3, 33, 2, 16, 1, 7], 0, 0
    while at < n:
        c = min(sizes[k % len(sizes)], n - at)
        ent = [("p", a[at:at + c], list(range(c)))]
        if k < 30:
            ent.append(("b", [b[k]], [0]))
        steps.append({"entries": ent})
        at, k = at + c, k + 1
    got = play(r, steps)
    over = []
    for (rid, pos), row in sorted(got.items()):
        try:
            row_close(row, ref[rid][pos], dtype, 0.05)
        except AssertionError as e:
            if dtype == "bfloat16" and torch.isfinite(row).all():
                err = (row - ref[rid][pos]).pow(2).mean().sqrt() / ref[rid][pos].pow(2).mean().sqrt()
                if float(err) < 0.125:
                    over.append((rid, pos, round(float(err), 3)))
                    continue
            raise AssertionError(f"seed {seed}, request {rid!r} position {pos} ({dtype}): {e}\\n{json.dumps(cj)}") from None
    assert len(over) <= max(1, len(got) // 10), f"seed {seed}: {len(over)} of {len(got)} rows beyond the bound: {over[:8]}"
    r.mgr.check_idle()


# ---------------------------------------------------------------------------------------------------------------------
# layers at serving sizes
# ---------------------------------------------------------------------------------------------------------------------
@functools.lru_cache(None)
def _wide_model():
    """Three layers whose mixers have the sizes of a served model (the stream itself is kept at 512 so that the plain
    implementation stays quick): 32 heads over a cache row of 192 + 64 with a window, a linear attention with a state of 256 x
    512 a head, 16 heads over a cache row of 128."""
    import tiny_nametar as tn
    cfg = tn._model(512, 1000, 1e-5, 0.5, 20.0, [
        tn._with(tn._la2(32, 128, 64, 128, 192, window=128, q_rank=256, scaling={"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0}), 1024),
        tn._with(tn._gla(2, 256, 512, 16.0, rank=16), None),
        tn._with(tn._la(16, 64, 64, 128), 512)])
    W = make_weights(cfg, 77)
    return cfg, W, write_model_dir(os.path.join(_tmp.name, "wide"), config_json(cfg), W)


@functools.lru_cache(None)
def _wide_reference():
    cfg, W, _ = _wide_model()
    a, b = random_tokens(250, cfg["vocab"], 1), random_tokens(120, cfg["vocab"], 2)
    with torch.no_grad():
        return a, b, {"a": pn.forward_sequence(config_json(cfg), W, a).float(), "b": pn.forward_sequence(config_json(cfg), W, b).float()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixers_at_serving_sizes(dtype):
    """A 220-token prompt in one step (the prompt kernels at these head counts and row sizes, the window's edge inside the
    portion, the linear attention in chunks), then a second request's portions behind a cached context beside decoded tokens
    of the first through the graph."""
    from mini_sglang_b200.engine.step import ModelRunner
    cfg, W, d = _wide_model()
    a, b, ref = _wide_reference()
    r = ModelRunner.from_model_dir(d, dtype=dtype, page_size=16, num_pages=40, max_reqs=2, max_context_len=1024)
    poison(r)
    want_a = [0, 1, 60, 127, 128, 129, 200, 219]
    steps = [{"entries": [("a", a[:220], want_a)]},
             {"entries": [("b", b[:80], [0, 79])]},
             {"entries": [("a", [a[220]], [0]), ("b", b[80:110], [0, 29])]}]
    steps += [{"entries": [("a", [a[221 + i]], [0]), ("b", [b[110 + i]], [0])]} for i in range(10)]
    steps += [{"entries": [("a", [a[231 + i]], [0])]} for i in range(19)]
    got = play(r, steps)
    assert r.last_step_used_graph
    over = []
    for (rid, pos), row in sorted(got.items()):
        try:
            row_close(row, ref[rid][pos], dtype, 0.03)
        except AssertionError as e:
            if dtype == "bfloat16" and torch.isfinite(row).all():
                err = (row - ref[rid][pos]).pow(2).mean().sqrt() / ref[rid][pos].pow(2).mean().sqrt()
                if float(err) < 0.075:
                    over.append((rid, pos, round(float(err), 3)))
                    continue
            raise AssertionError(f"request {rid!r} position {pos} ({dtype}): {e}") from None
    assert len(over) <= 1, over
    r.mgr.check_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kinds", ["linear only", "latent only", "one layer"])
def test_models_of_one_kind_of_layer(kinds, dtype):
    """A model that keeps no keys at all (only states), one that keeps no state and has no window (one cache group), and a
    model of a single layer: whole, token by token through the graph, in portions."""
    import tiny_nametar as tn
    from mini_sglang_b200.engine.step import ModelRunner
    layers = {"linear only": [tn._with(tn._gla(2, 16, 24, 4.0, rank=4), 48), tn._with(tn._gla(3, 8, 8, 16.0, rank=2), None)],
              "latent only": [tn._with(tn._la(3, 16, 8, 32), 48), tn._with(tn._la2(2, 8, 8, 12, 24, window=None, q_rank=16), None)],
              "one layer": [tn._with(tn._la2(4, 8, 8, 8, 40, window=5, scaling=tn.YARN), 32)]}[kinds]
    cfg = tn._model(64, 50, 1e-5, 0.6, 4.0, layers)
    cj, W = config_json(cfg), make_weights(cfg, 9)
    d = write_model_dir(os.path.join(_tmp.name, kinds.replace(" ", "_")), cj, W)
    n = 45
    a = random_tokens(n, cfg["vocab"], 3)
    with torch.no_grad():
        ref = pn.forward_sequence(cj, W, a).float()
    r = ModelRunner.from_model_dir(d, dtype=dtype, page_size=4, num_pages=40, max_reqs=2, max_context_len=256)
    assert len(r.mgr.groups) == {"linear only": 0, "latent only": 1, "one layer": 1}[kinds]
    poison(r)
    steps = [{"entries": [("w", a, list(range(n)))], "end": ["w"]}, {"entries": [("d", a[:3], [2])]}]
    steps += [{"entries": [("d", [t], [0])]} for t in a[3:]]
    steps += [{"entries": [("p", a[i:i + 7], list(range(len(a[i:i + 7]))))]} for i in range(0, n, 7)]
    got = play(r, steps)
    assert r.last_step_used_graph is False and len(got) == 3 * n - 2
    for (rid, pos), row in sorted(got.items()):
        try:
            row_close(row, ref[pos], dtype, 0.04)
        except AssertionError as e:
            raise AssertionError(f"{kinds}, request {rid!r} position {pos} ({dtype}): {e}") from None
    r.mgr.check_idle()
    if dtype != "float32":
        return
    # and through the entry point: the scheduler's admission with no page pool at all / with the prefix tree over a cache whose
    # rows are keys and values at once (two prompts share their first 24 tokens)
    del r
    from mini_sglang_b200 import Engine, EngineArgs
    prompts = [a[:30], a[:24] + random_tokens(9, cfg["vocab"], 8), a[:7]]
    eng = Engine(EngineArgs(model=d, dtype=dtype, page_size=4, num_pages=64, max_num_reqs=3, random_seed=0, chunk_size=16,
                            max_context_len=128, log_level="WARNING"))
    for _ in range(2):          # the second pass finds the first one's pages in the prefix tree, where the model has one
        outs = eng.generate(input_ids=prompts, sampling_params={"temperature": 0.0, "max_new_tokens": 6, "ignore_eos": True})
        for p, o in zip(prompts, outs):
            assert o["token_ids"] == pn.greedy_generate(cj, W, p, 6), (kinds, o["token_ids"])
    eng.scheduler.check_idle_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_geometries_in_one_cache_group(dtype):
    """Two latent attentions over all keys with different head counts and row sizes share a cache group (one block table, one
    plan of kv splits made from the first one's geometry).  A long context, then portions of a few tokens and single tokens:
    short runs take the decode kernel with the keys cut into pieces, and which runs are short differs between the two."""
    import tiny_nametar as tn
    from mini_sglang_b200.engine.step import ModelRunner
    cfg = tn._model(64, 50, 1e-5, 0.6, 4.0, [tn._with(tn._la(2, 16, 8, 64), 48), tn._with(tn._la(16, 8, 8, 32), None),
                                              tn._with(tn._la2(3, 8, 8, 8, 40, window=300, q_rank=16), 32),
                                              tn._with(tn._la2(12, 8, 8, 8, 24, window=300), None)])
    cj, W = config_json(cfg), make_weights(cfg, 11)
    d = write_model_dir(os.path.join(_tmp.name, "two_geometries"), cj, W)
    n = 420
    a = random_tokens(n, cfg["vocab"], 4)
    with torch.no_grad():
        ref = pn.forward_sequence(cj, W, a).float()
    r = ModelRunner.from_model_dir(d, dtype=dtype, page_size=16, num_pages=32, max_reqs=2, max_context_len=1024)
    assert len(r.mgr.groups) == 2
    poison(r)
    steps, at = [{"entries": [("a", a[:380], [0, 379])]}], 380
    for c in (3, 2, 4, 1, 1, 8, 2, 1, 5, 1, 1, 1, 3, 6, 1):
        steps.append({"entries": [("a", a[at:at + c], list(range(c)))]})
        at += c
    assert at == n
    got = play(r, steps)
    assert any(max(ns) > 1 for ns in r.last_plan["nsplits"]), "the test wants kv splits"
    for (rid, pos), row in sorted(got.items()):
        try:
            row_close(row, ref[pos], dtype, 0.04)
        except AssertionError as e:
            raise AssertionError(f"position {pos} ({dtype}): {e}") from None
    r.mgr.check_idle()
