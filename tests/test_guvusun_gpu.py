"""Guvusun on the GPU against the plain float64 restatement in oracle/guvusun.py: every mechanism alone, then whole models through the
runner (portions, decoding, batches, reused blocks and slots) and greedy generation through LLMEngine.  Configurations are small and made
here; sizes that one model might happen to make equal (value size == unrotated size, one group kept, heads a multiple of the kernel's
group, top == 2, every layer with a feed-forward) differ between them."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import candle_vllm_b200 as pkg
from candle_vllm_b200 import seq_ops as ops, synthetic as S
from candle_vllm_b200.engine import LLMEngine, ModelRunner
from candle_vllm_b200.guvusun import GuvusunConfig, GuvusunModel
from candle_vllm_b200.inputs import prepare_step
from candle_vllm_b200.mixers import LatentAttentionMixer, RoutedExperts, TokenSideInput
from oracle import guvusun as G

pytestmark = pytest.mark.gpu
DEV = "cuda"
F64 = torch.float64
YARN = dict(factor=4.0, original=128, fast=16.0, slow=1.0)


def dev(t, dt=torch.float32):
    return t.to(dt).to(DEV).contiguous()


def batch_of(entries, block_size=64):
    return ops.StepBatch.from_host(prepare_step(entries, block_size), DEV)


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().to(F64), want.detach().cpu().to(F64)
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err < tol, f"{what}: max-err/max = {err:.3e} (tolerance {tol})"


def _portions(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append((at, n)); at += n; i += 1
    return out


# ----------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ----------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bigram_embedding_carries_the_previous_token(dtype):
    """rows of three sequences in portions down to one token; the previous token crosses step borders through the slot state, slots are
    handed over dirty, and a sequence's first token takes the extra row whatever the slot held"""
    g = torch.Generator().manual_seed(0)
    V, D, bg = 70, 36, dict(buckets=13, mul_prev=31, mul_cur=7)
    tab, big, nw = torch.randn(V, D, generator=g).to(torch.bfloat16), torch.randn(14, D, generator=g).to(torch.bfloat16), torch.ones(D)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (19, 1, 8)]
    state = torch.full((3, 1), 55, dtype=torch.int32, device=DEV)            # dirty slots
    plans = [[3, 1, 1, 5, 2, 7], [1], [2, 2, 1, 3]]
    slots = [2, 0, 1]
    got = [[] for _ in seqs]
    fed, step = [0, 0, 0], 0
    while any(f < len(s) for f, s in zip(fed, seqs)):
        entries, who = [], []
        for i, s in enumerate(seqs):
            if fed[i] < len(s) and (step + i) % 3 != 2:                 # a request may sit a step out
                n = min(plans[i][step % len(plans[i])], len(s) - fed[i])
                entries.append(dict(tokens=s[fed[i]:fed[i] + n], start=fed[i], block_table=[0, 1], state_slot=slots[i], want=[]))
                who.append((i, n))
        step += 1
        if not entries:
            continue
        out = ops.embedding_bigram(tab.to(dtype).to(DEV), big.to(dtype).to(DEV), batch_of(entries), state, bg["buckets"], bg["mul_prev"], bg["mul_cur"])
        at = 0
        for i, n in who:
            got[i].append(out[at:at + n]); at += n; fed[i] += n
    for i, s in enumerate(seqs):
        rows = torch.tensor(G.bigram_rows(s, **bg))
        assert rows[0] == bg["buckets"] and (len(s) == 1 or int(rows[1:].max()) < bg["buckets"])
        close(torch.cat(got[i]), tab.to(F64)[torch.tensor(s)] + big.to(F64)[rows], 1e-6, f"sequence {i}")
    # a slot that changes hands: the new owner's first token ignores what is there, its second sees its own first
    e = [dict(tokens=[5, 9], start=0, block_table=[0], state_slot=2, want=[])]
    out = ops.embedding_bigram(tab.to(dtype).to(DEV), big.to(dtype).to(DEV), batch_of(e), state, bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    close(out, tab.to(F64)[torch.tensor([5, 9])] + big.to(F64)[torch.tensor(G.bigram_rows([5, 9], **bg))], 1e-6, "reused slot")
    assert int(state[2, 0]) == 9


@pytest.mark.parametrize("n", [5, 96, 321, 1030])
def test_norm_after_the_sum_and_added_norm(n):
    g = torch.Generator().manual_seed(n)
    x, y, w = torch.randn(7, n, generator=g) * 3, torch.randn(7, n + 3, generator=g), 1 + torch.randn(n, generator=g) * 0.3
    for alpha in (2.0, 0.5, 1.0):
        xd, o16 = dev(x), torch.empty(7, n, dtype=torch.bfloat16, device=DEV)
        ops.residual_rms_norm(xd, dev(y)[:, :n], dev(w), alpha, 1e-6, True, o16)
        want = G.rms(alpha * x.to(F64) + y[:, :n].to(F64), 1e-6) * w.to(F64)
        close(xd, want, 2e-6, f"norm(alpha x + y), alpha {alpha}")
        close(o16, want, 6e-3, "its 16-bit copy")
    xd = dev(x)
    ops.residual_rms_norm(xd, None, dev(w), 1.0, 1e-5, True)
    close(xd, G.rms(x.to(F64), 1e-5) * w.to(F64), 2e-6, "no sublayer output")
    xd = dev(x)
    ops.residual_rms_norm(xd, dev(y)[:, :n], dev(w), 1.0, 1e-6, False)
    close(xd, x.to(F64) + G.rms(y[:, :n].to(F64), 1e-6) * w.to(F64), 2e-6, "x + norm(y)")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 2e-2)])
def test_token_side_input(dtype, tol):
    g = torch.Generator().manual_seed(1)
    V, D, dim, layers, li = 40, 72, 10, 3, 1
    table = torch.randn(V, dim * layers, generator=g).to(torch.bfloat16)
    w = dict(gate=(torch.randn(dim, D, generator=g) * D ** -0.5).to(torch.bfloat16), proj=(torch.randn(D, dim, generator=g) * dim ** -0.5).to(torch.bfloat16),
             norm=(0.5 + torch.randn(D, generator=g) * 0.1).to(torch.bfloat16))
    toks = torch.randint(0, V, (21,), generator=g).tolist()
    x = torch.randn(21, D, generator=g)
    if dtype == torch.bfloat16:
        x = x.to(torch.bfloat16).float()
    side = TokenSideInput({k: v.to(DEV) for k, v in w.items()}, table.to(dtype).to(DEV), li * dim, dim, 1e-6, dtype)
    xd = dev(x)
    o16 = torch.empty(21, D, dtype=torch.bfloat16, device=DEV) if dtype == torch.bfloat16 else None
    b = batch_of([dict(tokens=toks, start=0, block_table=[0], state_slot=0, want=[])])
    side.forward(xd, dev(x, dtype), b, o16)
    close(xd, G.token_side(x.to(F64), toks, table, li, dim, w, 1e-6), tol, "token side input")


ROUTES = [  # N, top, groups, keep
    (18, 2, 3, 1), (12, 3, 4, 2), (9, 1, 3, 3), (40, 6, 8, 3), (7, 7, 0, 0), (33, 4, 0, 0), (64, 8, 64, 9), (6, 2, 3, 1),
]


@pytest.mark.parametrize("N,top,groups,keep", ROUTES)
def test_router_choice(N, top, groups, keep):
    """choice scores are softmax + correction with corrections that make every choice score NEGATIVE (a masked group must count as
    -inf, not 0), weights are the plain softmax of the chosen"""
    g = torch.Generator().manual_seed(N * 7 + top)
    T, D = 50, 24
    h = torch.randn(T, D, generator=g)
    wr = torch.randn(N, D, generator=g) * 3 * D ** -0.5
    corr = torch.randn(N, generator=g) * 0.2 - 1.5
    r = dict(top=top, scale=1.8)
    if groups:
        r["groups"] = dict(count=groups, keep=keep)
    ids_w, w_w = G.route(h.to(F64), wr, corr, r)
    ids, wts = ops.moe_route(ops.linear(dev(h), dev(wr)), dev(corr), top, groups, keep, 1.8)
    ids, wts = ids.cpu().long(), wts.cpu().to(F64)
    for t in range(T):
        assert sorted(ids[t].tolist()) == sorted(ids_w[t].tolist()), f"token {t}: {ids[t].tolist()} vs {ids_w[t].tolist()}"
        got = dict(zip(ids[t].tolist(), wts[t].tolist()))
        for e, a in zip(ids_w[t].tolist(), w_w[t].tolist()):
            assert abs(got[e] - a) < 1e-5 * 1.8
    # without a correction the choice follows the softmax itself
    ids2, _ = ops.moe_route(ops.linear(dev(h), dev(wr)), None, top, groups, keep, 1.0)
    ids_w2, _ = G.route(h.to(F64), wr, None, r)
    assert all(sorted(a) == sorted(b) for a, b in zip(ids2.cpu().tolist(), ids_w2.tolist()))


@pytest.mark.parametrize("E,I,top,ff,D,groups", [(6, 2, 2, 40, 72, (2, 1)), (5, 0, 3, 17, 52, None), (0, 4, 2, 0, 40, None), (3, 5, 4, 64, 64, (4, 3)), (1, 1, 1, 8, 24, None)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-6), (torch.bfloat16, 3e-2)])
def test_routed_experts(E, I, top, ff, D, groups, dtype, tol):
    cfg = S.guvusun_config(D, 30, [S.guvusun_layer(2, 8, 4, 8, 16, experts=E, ff=ff, top=top, identity=I, groups=groups, router_scale=1.7)])
    w = {k[len("l0.mlp."):]: v for k, v in S.guvusun_weights(cfg, E + I).items() if k.startswith("l0.mlp.")}
    g = torch.Generator().manual_seed(3)
    x = torch.randn(37, D, generator=g).to(torch.bfloat16).float()
    mlp = RoutedExperts({k: v.to(DEV) for k, v in w.items()}, E, I, top, 1.7, dtype, groups=groups[0] if groups else 0, keep=groups[1] if groups else 0)
    close(mlp.forward(dev(x, dtype), dev(x)), G.moe(x.to(F64), w, cfg["layers"][0]["mlp"]), tol, "routed experts")


@pytest.mark.parametrize("tile", [128, 32, 64])
@pytest.mark.parametrize("n,k,G", [(64, 64, 3), (40, 72, 5), (300, 128, 2), (24, 200, 4)])
def test_grouped_product_on_the_tensor_core_gemm(n, k, G, tile):
    """rows in tiles of 128 (or 32 / 64: the form for few rows per matrix, weights on the 128-row side of the MMA), every tile multiplying the
    matrix its entry names (in any order, with skipped tiles), against float64 on the same bf16 operands; rows of skipped tiles stay as they were"""
    g = torch.Generator().manual_seed(n + k)
    tiles = [1, -1, 0, G - 1, 1, -1, 0]
    m = tile * len(tiles)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(G, n, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 6e-3)):
        out = torch.full((m, n + 8), 3.0, dtype=dt, device=DEV)
        ops.linear_grouped(x.to(DEV), w.to(DEV), torch.tensor(tiles, dtype=torch.int32, device=DEV), out, tile)
        for i, e in enumerate(tiles):
            rows = slice(tile * i, tile * i + tile)
            if e < 0:
                assert float((out[rows].float() - 3.0).abs().max()) == 0.0
            else:
                close(out[rows, :n], x[rows].to(F64) @ w[e].to(F64).T, tol, f"tile {i} -> matrix {e}")
                assert float((out[rows, n:].float() - 3.0).abs().max()) == 0.0


def test_pairs_sorted_by_expert():
    g = torch.Generator().manual_seed(0)
    E, T, top = 5, 333, 3
    ids = torch.randint(0, E + 2, (T, top), generator=g).to(torch.int32)           # ids E, E + 1 are identity choices
    ids[ids == 3] = 4                                                              # an expert nobody chose
    flat = ids.reshape(-1)
    for tile in (128, 32, 1):
        pair_row, row_pair, tile_group = (t.cpu() for t in ops.moe_sorted_rows(ids.to(DEV), E, tile))
        assert row_pair.shape[0] % tile == 0 and tile_group.shape[0] == row_pair.shape[0] // tile
        for p in range(T * top):
            r = int(pair_row[p])
            if flat[p] >= E:
                assert r == -1
            else:
                assert int(row_pair[r]) == p and int(tile_group[r // tile]) == int(flat[p])
        assert int((row_pair >= 0).sum()) == int((flat < E).sum())
        assert 3 not in tile_group.tolist()


def _mixer_case(H, dn, dr, dv, R, D, scaling, seed=0, **kw):
    cfg = S.guvusun_config(D, 30, [S.guvusun_layer(H, dn, dr, dv, R, scaling=scaling, **kw)])
    w = {k[len("l0.mix."):]: v for k, v in S.guvusun_weights(cfg, seed).items() if k.startswith("l0.mix.")}
    return cfg["layers"][0]["mixer"], w


def _run_mixer(mix, h, sizes, tables, nblocks, dtype, cache=None):
    """one sequence in portions through the mixer; returns (output rows, cache)"""
    R, dr = mix.R, mix.dr
    if cache is None:
        cache = (torch.full((nblocks, 64, 1, R), 7.0, dtype=dtype, device=DEV), torch.full((nblocks, 64, 1, max(dr, 1)), 7.0, dtype=dtype, device=DEV))
    outs = []
    for at, n in _portions(h.shape[0], sizes):
        b = batch_of([dict(tokens=[0] * n, start=at, block_table=tables, state_slot=0, want=[])])
        outs.append(mix.forward(dev(h[at:at + n], dtype), b, cache))
    return torch.cat(outs), cache


MIXERS = [  # H, dn, dr, dv, R, D, scaling
    (3, 24, 8, 40, 72, 48, YARN), (8, 16, 16, 16, 96, 64, None), (9, 8, 4, 12, 33, 40, YARN), (1, 40, 2, 8, 130, 32, None), (12, 12, 6, 20, 260, 56, YARN),
]


@pytest.mark.parametrize("H,dn,dr,dv,R,D,scaling", MIXERS)
@pytest.mark.parametrize("sizes", [[300], [1], [2], [37, 1, 1, 64, 5]])
def test_latent_attention_with_loud_keys(H, dn, dr, dv, R, D, scaling, sizes):
    """the mixer alone over scattered blocks; some tokens are made LOUD (their shared rotated key part, which is not normed, is scaled up), at
    the first positions, on both sides of block borders and far back, so a missed or wrongly seen key changes the output by far more than the
    tolerance; the positions next to a loud key check the causal edge in prompts and in decoding"""
    m, w = _mixer_case(H, dn, dr, dv, R, D, scaling)
    g = torch.Generator().manual_seed(H)
    T = 300
    h = torch.randn(T, D, generator=g)
    for j, s in ((0, 25.0), (2, -25.0), (63, 30.0), (64, -30.0), (65, 20.0), (127, -20.0), (128, 25.0), (190, 30.0), (255, -30.0), (256, 30.0)):
        h[j] *= s
    want, _ = G.latent_attention(h.to(F64), w, m, 1e-6)
    mix = LatentAttentionMixer({k: v.to(DEV) for k, v in w.items()}, H, dn, dr, dv, R, m["scale"], 1e-6, torch.float32, rot=m["rot"], max_pos=64)
    got, _ = _run_mixer(mix, h, sizes, [5, 2, 7, 0, 3], 8, torch.float32)
    close(got, want, 2e-5, "latent attention")
    # the loud keys matter: without the key at 190 the rows after it change by far more than the tolerance
    h2 = h.clone(); h2[190] /= 30.0
    other, _ = G.latent_attention(h2.to(F64), w, m, 1e-6)
    assert float((other[200:250] - want[200:250]).abs().max()) > 1e-2 * float(want.abs().max())


def test_latent_attention_sink_gate_and_shared_cache():
    H, dn, dr, dv, R, D = 4, 16, 8, 24, 40, 48
    m, w = _mixer_case(H, dn, dr, dv, R, D, YARN, seed=3)
    g = torch.Generator().manual_seed(1)
    h = torch.randn(150, D, generator=g)
    mk = lambda ww, **kw: LatentAttentionMixer({k: v.to(DEV) for k, v in ww.items()}, H, dn, dr, dv, R, m["scale"], 1e-6, torch.float32, rot=m["rot"], **kw)
    # a large sink takes nearly all the weight of the first rows; a missing sink tensor means no sink at all; no gate tensor, no gate
    for variant in ("big sink", "no sink", "no gate"):
        ww = dict(w)
        if variant == "big sink":
            ww["sink"] = torch.tensor([6.0, -3.0, 0.0, 9.0]).to(torch.bfloat16)
        elif variant == "no sink":
            ww.pop("sink")
        else:
            ww.pop("g")
        want, _ = G.latent_attention(h.to(F64), ww, m, 1e-6)
        got, _ = _run_mixer(mk(ww), h, [70, 1, 1, 30], [1, 0, 2], 3, torch.float32)
        close(got, want, 2e-5, variant)
    # a second mixer without a latent projection reads the cache the first one wrote (its own queries, up-projections, sink and gate)
    m2, w2 = _mixer_case(H + 1, dn - 4, dr, dv + 8, R, D, YARN, seed=4, kv_from=0)
    assert "dkv" not in w2
    _, kept = G.latent_attention(h.to(F64), w, m, 1e-6)
    h_next = torch.randn(150, D, generator=g)
    want2, _ = G.latent_attention(h_next.to(F64), w2, m2, 1e-6, shared=kept)
    first = mk(w)
    second = LatentAttentionMixer({k: v.to(DEV) for k, v in w2.items()}, H + 1, dn - 4, dr, dv + 8, R, m2["scale"], 1e-6, torch.float32, rot=m2["rot"], shared=True)
    cache, outs = None, []
    for at, n in _portions(150, [40, 1, 2, 64]):
        b = batch_of([dict(tokens=[0] * n, start=at, block_table=[2, 0, 1], state_slot=0, want=[])])
        if cache is None:
            cache = (torch.zeros((3, 64, 1, R), device=DEV), torch.zeros((3, 64, 1, dr), device=DEV))
        first.forward(dev(h[at:at + n]), b, cache)
        outs.append(second.forward(dev(h_next[at:at + n]), b, cache))
    close(torch.cat(outs), want2, 2e-5, "shared latent cache")


def test_latent_attention_window_parameter():
    """the kernel's window argument (unused by Guvusun, there for other designs): position i sees j with i - j < window"""
    H, dn, dr, dv, R, D = 2, 8, 4, 8, 24, 32
    m, w = _mixer_case(H, dn, dr, dv, R, D, None)
    g = torch.Generator().manual_seed(2)
    h = torch.randn(100, D, generator=g)
    h[40] *= 30.0
    mix = LatentAttentionMixer({k: v.to(DEV) for k, v in w.items()}, H, dn, dr, dv, R, m["scale"], 1e-6, torch.float32, rot=m["rot"], window=17)
    got, _ = _run_mixer(mix, h, [50, 1, 1, 1, 1, 1, 1, 1, 1, 9], [0, 1], 2, torch.float32)
    full, _ = G.latent_attention(h.to(F64), w, m, 1e-6)
    close(got[:17], full[:17], 2e-5, "inside the first window")
    # rows 41..56 still see the loud key at 40, row 57 is the first that does not: compare with the oracle run on the window alone
    for i in (56, 57, 80):
        lo = i - 16
        c, kr = G.latent_kv(h.to(F64), w["dkv"], w["dkv.norm"], R, dr, m["rot"], 1e-6)
        q = (h[i].to(F64) @ w["q"].to(F64).T).reshape(H, dn + dr)
        cos, sin = G.rotary_angles(100, dr, m["rot"]["base"], None)
        qr = G.rotate_half(q[None, :, dn:], cos[i:i + 1], sin[i:i + 1])[0]
        kn = (c[lo:i + 1] @ w["uk"].to(F64).T).reshape(-1, H, dn)
        v = (c[lo:i + 1] @ w["uv"].to(F64).T).reshape(-1, H, dv)
        s = (torch.einsum("hd,jhd->hj", q[:, :dn], kn) + torch.einsum("hd,jd->hj", qr, kr[lo:i + 1])) * m["scale"]
        sink = w["sink"].to(F64)[:, None]
        mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
        p = torch.exp(s - mx) / (torch.exp(s - mx).sum(-1, keepdim=True) + torch.exp(sink - mx))
        o = torch.einsum("hj,jhd->hd", p, v) * torch.sigmoid(h[i].to(F64) @ w["g"].to(F64).T)[:, None]
        close(got[i], o.reshape(-1) @ w["o"].to(F64).T, 2e-5, f"row {i}")


# ----------------------------------------------------------------------------------------------------------------------
# whole models
# ----------------------------------------------------------------------------------------------------------------------
CONFIGS = {
    # three layers, the last on the first one's cache; groups, identity experts, bigram, side input
    "shared": S.guvusun_config(96, 160, [S.guvusun_layer(6, 24, 8, 16, 48, experts=6, ff=40, top=2, identity=2, groups=(4, 2), router_scale=1.8, scaling=YARN),
                                         S.guvusun_layer(3, 16, 16, 40, 72, experts=4, ff=24, top=3, router_scale=1.0),
                                         S.guvusun_layer(5, 12, 8, 20, 48, experts=3, ff=32, top=1, identity=3, groups=(2, 1), kv_from=0, scaling=YARN)],
                               alpha=1.6, bigram=dict(buckets=251, mul_prev=113, mul_cur=29), side_dim=12),
    # no bigram, no side input, a layer without feed-forward, no groups, alpha below one, one head, latent wider than 128
    "plain": S.guvusun_config(72, 97, [S.guvusun_layer(1, 32, 4, 24, 136), S.guvusun_layer(4, 8, 8, 8, 24, experts=5, ff=48, top=2, router_scale=1.3)], alpha=0.7,
                              eps=1e-5),
    # odd sizes everywhere (no 8-element alignment), two layers sharing the cache of layer 1, only identity experts in one layer
    "odd": S.guvusun_config(52, 61, [S.guvusun_layer(2, 10, 6, 14, 20, experts=3, ff=18, top=2, identity=1),
                                     S.guvusun_layer(9, 6, 2, 10, 34, identity=3, top=2, router_scale=0.8),
                                     S.guvusun_layer(3, 14, 2, 6, 34, experts=2, ff=44, top=2, kv_from=1),
                                     S.guvusun_layer(2, 4, 2, 22, 34, experts=7, ff=10, top=4, identity=1, groups=(4, 2), kv_from=1)],
                            alpha=3.0, bigram=dict(buckets=7, mul_prev=3, mul_cur=5), side_dim=5),
}
_CACHE = {}
TOL = {torch.float32: 2e-4, torch.bfloat16: 8e-2}


def model_and_oracle(name, dtype, n_tokens, seed=0):
    cfg = CONFIGS[name]
    key = (name, seed)
    if key not in _CACHE:
        w = S.guvusun_weights(cfg, seed)
        toks = torch.randint(0, cfg["vocab"], (300,), generator=torch.Generator().manual_seed(seed + 1)).tolist()
        _CACHE[key] = (w, toks, G.forward(cfg, w, toks))
    w, toks, ref = _CACHE[key]
    model = GuvusunModel(GuvusunConfig.from_dict(cfg), w, dtype=dtype, block_size=64, max_pos=128, device=DEV)
    return model, toks[:n_tokens], ref[:n_tokens]


def run_schedule(runner, seq_id, toks, sizes):
    runner.admit(seq_id)
    out = []
    for at, n in _portions(len(toks), sizes):
        out.append(runner.execute([dict(seq_id=seq_id, tokens=toks[at:at + n], want=list(range(n)))]))
    runner.release(seq_id)
    return torch.cat(out)


def row_errors(got, want):
    """per position: rms over the vocabulary of the centred difference, relative to the rms of the reference logits"""
    d = got.detach().cpu().to(F64) - want
    d = d - d.mean(-1, keepdim=True)
    return torch.sqrt((d * d).mean(-1)) / torch.sqrt((want * want).mean())


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_the_oracle(name):
    model, toks, ref = model_and_oracle(name, torch.float32, 230)
    runner = ModelRunner(model, 8, 2, 64)
    trace = []
    runner.admit(0)
    got = runner.execute([dict(seq_id=0, tokens=toks, want=list(range(len(toks))))], hidden_trace=trace)
    close(got, ref, TOL[torch.float32], f"{name} logits")
    want_trace = []
    G.forward(CONFIGS[name], _CACHE[(name, 0)][0], toks, want_trace)
    assert len(trace) == len(want_trace) == len(CONFIGS[name]["layers"])
    for i, (a, b) in enumerate(zip(trace, want_trace)):
        close(a, b, 1e-4, f"{name} stream after layer {i}")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_bf16_stays_within_rounding(name):
    """bf16 operands may flip a router's near-tie at a few positions, so the bound is on the typical position, with a loose cap on all"""
    model, toks, ref = model_and_oracle(name, torch.bfloat16, 230)
    runner = ModelRunner(model, 8, 2, 64)
    whole = run_schedule(runner, 0, toks, [230])
    parts = run_schedule(runner, 1, toks, [37, 2, 1, 1, 64])
    for got in (whole, parts):
        e = row_errors(got, ref)
        assert float(e.median()) < 0.03 and float(e.quantile(0.9)) < 0.08, (float(e.median()), float(e.quantile(0.9)))


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("sizes", [[1], [2], [3, 2, 7], [64, 1, 1, 5], [39, 1, 41, 2, 63]])
def test_portions_and_decoding_match_the_whole_prompt(name, sizes):
    model, toks, ref = model_and_oracle(name, torch.float32, 200)
    runner = ModelRunner(model, 4, 1, 64)
    close(run_schedule(runner, 5, toks, sizes), ref, TOL[torch.float32], f"{name} portions {sizes}")


@pytest.mark.parametrize("name", ["shared", "odd"])
def test_unequal_batches_match_each_request_alone(name):
    """Requests of different lengths advance together, portions of some beside single tokens of others; the pool is smaller than the sum of
    all requests, so blocks and slots of finished requests go to later ones (the previous-token slot is handed over dirty)."""
    cfg = CONFIGS[name]
    w = S.guvusun_weights(cfg, 0)
    model = GuvusunModel(GuvusunConfig.from_dict(cfg), w, dtype=torch.float32, block_size=64, max_pos=512, device=DEV)
    g = torch.Generator().manual_seed(9)
    lens = [130, 7, 64, 201, 65, 1, 90]
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    refs = [G.forward(cfg, w, s) for s in seqs]
    runner = ModelRunner(model, 9, 3, 64)
    plans = [[64, 1, 1, 30, 2, 1], [2, 1], [63, 1], [100, 3, 1, 1, 50, 2], [64, 1], [1], [1, 1, 1, 80, 2]]
    waiting, live, got = list(range(len(seqs))), {}, {i: [] for i in range(len(seqs))}
    guard = 0
    while waiting or live:
        guard += 1
        assert guard < 500
        while waiting and runner.state.pool.num_free() > 0 and runner.can_admit(lens[waiting[0]], sum(-(-lens[i] // 64) - len(runner.blocks.tables.get(i, ())) for i in live)):
            i = waiting.pop(0)
            runner.admit(i)
            live[i] = [0, 0]
        entries = []
        for i, (fed, pi) in live.items():
            n = min(plans[i][pi % len(plans[i])] if pi < len(plans[i]) else 1, lens[i] - fed)
            entries.append(dict(seq_id=i, tokens=seqs[i][fed:fed + n], want=list(range(n))))
        out = runner.execute(entries)
        at = 0
        for e in entries:
            i, n = e["seq_id"], len(e["tokens"])
            got[i].append(out[at:at + n]); at += n
            live[i][0] += n; live[i][1] += 1
        for i in [i for i, (fed, _) in live.items() if fed == lens[i]]:
            runner.release(i); del live[i]
    for i in range(len(seqs)):
        close(torch.cat(got[i]), refs[i], TOL[torch.float32], f"{name} request {i} in a batch")
    runner.blocks.check_invariants()
    assert runner.blocks.num_free_gpu_blocks() == 9 and runner.state.pool.num_free() == 3


def test_long_decoding_across_blocks():
    model, toks, ref = model_and_oracle("plain", torch.float32, 300)
    runner = ModelRunner(model, 5, 1, 64)
    runner.admit(0)
    got = [runner.execute([dict(seq_id=0, tokens=toks[:20], want=list(range(20)))])]
    for t in range(20, 300):
        got.append(runner.execute([dict(seq_id=0, tokens=[toks[t]], want=[0])]))
    close(torch.cat(got), ref, TOL[torch.float32], "280 decoded tokens")


def test_first_tokens_and_single_token_requests():
    model, toks, ref = model_and_oracle("shared", torch.float32, 230)
    runner = ModelRunner(model, 4, 2, 64)
    for n in (1, 2, 3):
        runner.admit(n)
        close(runner.execute([dict(seq_id=n, tokens=toks[:n], want=list(range(n)))]), ref[:n], TOL[torch.float32], f"first {n} tokens")
        runner.release(n)


def test_many_rows_take_the_tensor_core_routes():
    """a bf16 step with hundreds of rows and 8-aligned sizes: the expert products and the latent up-projections run as grouped products on
    the tensor-core GEMM; the same rows in steps of a few tokens run on the streaming kernels; both stay within rounding of the oracle and
    of each other"""
    cfg = S.guvusun_config(128, 200, [S.guvusun_layer(4, 64, 16, 32, 64, experts=6, ff=64, top=2, identity=2, groups=(2, 1), router_scale=2.0, scaling=YARN),
                                      S.guvusun_layer(8, 16, 16, 24, 64, experts=3, ff=128, top=2, kv_from=0, scaling=YARN)],
                           bigram=dict(buckets=101, mul_prev=11, mul_cur=3), side_dim=8)
    w = S.guvusun_weights(cfg, 2)
    toks = torch.randint(0, 200, (420,), generator=torch.Generator().manual_seed(4)).tolist()
    ref = G.forward(cfg, w, toks)
    model = GuvusunModel(GuvusunConfig.from_dict(cfg), w, dtype=torch.bfloat16, block_size=64, max_pos=512, device=DEV)
    runner = ModelRunner(model, 14, 2, 64)
    big = run_schedule(runner, 0, toks, [420])
    mid = run_schedule(runner, 1, toks, [300, 1, 119])
    small = run_schedule(runner, 2, toks, [9, 1, 30])
    for got in (big, mid, small):
        e = row_errors(got, ref)
        assert float(e.median()) < 0.03 and float(e.quantile(0.9)) < 0.08, (float(e.median()), float(e.quantile(0.9)))
    e = row_errors(big, small.detach().cpu().to(F64))
    assert float(e.median()) < 0.03


def test_single_token_steps_on_the_split_kv_latent_kernel():
    """latent 512 + rotated 64 in bf16 with 64-token blocks: steps of 16 and more rows (single tokens and rows of prompts alike) run on the split-KV
    tensor-core kernel of the latent cache, whose merge takes the sink; contexts on both sides of its 256-key runs and of block borders, scattered
    blocks, decoded side by side"""
    cfg = S.guvusun_config(128, 150, [S.guvusun_layer(4, 64, 64, 32, 512, experts=4, ff=64, top=2, identity=1, scaling=YARN),
                                      S.guvusun_layer(3, 64, 64, 40, 512, kv_from=0, scaling=YARN)], bigram=dict(buckets=31, mul_prev=7, mul_cur=3))
    w = S.guvusun_weights(cfg, 5)
    w["l0.mix.sink"] = torch.tensor([4.0, -2.0, 1.0, 7.0]).to(torch.bfloat16)          # sinks that visibly take weight
    model = GuvusunModel(GuvusunConfig.from_dict(cfg), w, dtype=torch.bfloat16, block_size=64, max_pos=512, device=DEV)
    assert model.layers[0].mixer.decode_kernel and model.layers[1].mixer.decode_kernel
    g = torch.Generator().manual_seed(6)
    lens = [1, 2, 63, 64, 65, 127, 128, 129, 250, 255, 256, 257, 300, 17, 200, 90, 5]
    steps = 4
    seqs = [torch.randint(0, 150, (n + steps,), generator=g).tolist() for n in lens]
    refs = [G.forward(cfg, w, s) for s in seqs]
    runner = ModelRunner(model, 60, len(lens), 64)
    got = [[] for _ in lens]
    for i in reversed(range(len(lens))):                                                # admitted in reverse: tables are not in sequence order
        runner.admit(i)
        out = runner.execute([dict(seq_id=i, tokens=seqs[i][:lens[i]], want=list(range(lens[i])))])
        if lens[i] >= 16:                                                               # rows of prompts take the same kernel, each with its own context length
            e = row_errors(out, refs[i][:lens[i]])
            # (a bf16 router may flip a near-tie on a single row: the bound is on the typical row and on the share of far-off rows)
            assert float(e.median()) < 0.03 and float((e > 0.1).float().mean()) < 0.03, (i, float(e.median()), float(e.max()))
    for k in range(steps):
        out = runner.execute([dict(seq_id=i, tokens=[seqs[i][lens[i] + k]], want=[0]) for i in range(len(lens))])
        for i in range(len(lens)):
            got[i].append(out[i:i + 1])
    errs = torch.cat([row_errors(torch.cat(got[i]), refs[i][lens[i]:]) for i in range(len(lens))])
    assert float(errs.median()) < 0.03 and float(errs.quantile(0.9)) < 0.08 and float((errs > 0.1).float().mean()) < 0.05, (float(errs.median()), float(errs.max()))
    # without the sink the same rows move by far more than rounding: the merge does take it
    w2 = dict(w); w2["l0.mix.sink"] = torch.full((4,), -30.0).to(torch.bfloat16)
    other = torch.cat([row_errors(torch.cat(got[i]), G.forward(cfg, w2, seqs[i])[lens[i]:]) for i in (3, 8)])
    assert float(other.median()) > 3 * float(errs.median())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_engine(dtype, tmp_path):
    """checkpoint on disk -> registry -> LLMEngine (scheduler, chunked prefill, sampler) against the oracle's greedy continuation"""
    from candle_vllm_b200.safetensors_io import save_file
    cfg = CONFIGS["shared"]
    w = S.guvusun_weights(cfg, 4)
    save_file(w, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (70, 3, 33, 1, 129)]
    eng = LLMEngine.from_pretrained(str(tmp_path), dtype=dtype, num_blocks=7, max_num_seqs=2, prefill_chunk=48, max_batch_tokens=64, max_model_len=256)
    assert type(eng.model).__name__ == "GuvusunModel"
    outs = eng.generate(prompts, pkg.SamplingParams(max_tokens=6))
    assert eng.runner.blocks.num_free_gpu_blocks() == 7 and eng.runner.state.pool.num_free() == 2
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        if dtype == torch.float32:
            assert o == G.greedy(cfg, w, p, 6)
        else:
            assert all(0 <= t < cfg["vocab"] for t in o)


def test_graph_replay_of_decode_steps_matches_eager():
    cfg = CONFIGS["shared"]
    w = S.guvusun_weights(cfg, 0)
    model = GuvusunModel(GuvusunConfig.from_dict(cfg), w, dtype=torch.float32, block_size=64, max_pos=64, device=DEV)      # tables must grow
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (100, 140)]
    refs = [G.forward(cfg, w, s) for s in seqs]
    runner = ModelRunner(model, 6, 2, 64, decode_graphs=True)
    got = [[], []]
    runner.admit(0); runner.admit(1)
    out = runner.execute([dict(seq_id=0, tokens=seqs[0][:50], want=list(range(50))), dict(seq_id=1, tokens=seqs[1][:61], want=list(range(61)))])
    got[0].append(out[:50]); got[1].append(out[50:])
    fed = [50, 61]
    while fed[0] < 100 or fed[1] < 140:
        live = [i for i in (0, 1) if fed[i] < len(seqs[i])]
        out = runner.execute([dict(seq_id=i, tokens=[seqs[i][fed[i]]], want=[0]) for i in live]).clone()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1]); fed[i] += 1
    assert 1 in runner._graphs
    for i in (0, 1):
        close(torch.cat(got[i]), refs[i], TOL[torch.float32], f"graph replay, request {i}")


def test_command_line_and_trace_runner(tmp_path):
    """the two programs a user starts, as child processes on a checkpoint on disk"""
    from candle_vllm_b200.safetensors_io import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CONFIGS["odd"]
    w = S.guvusun_weights(cfg, 1)
    save_file(w, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "candle_vllm_b200", "generate", "--model", str(tmp_path), "--dtype", "float32", "--prompt-ids", "5,6,7,8", "--max-new-tokens", "5"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    assert json.loads(r.stdout.strip().splitlines()[-1])["output"] == G.greedy(cfg, w, [5, 6, 7, 8], 5)
    a, b = list(range(3, 43)), [9, 8, 7]
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:30], want=[0, 29]), dict(id="b", tokens=b[:1], want=[0])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[30:], want=[9]), dict(id="b", tokens=b[1:2], want=[])], end=["a"]),
             dict(step=2, entries=[dict(id="b", tokens=b[2:], want=[0]), dict(id="c", tokens=a[:2], want=[1])], end=[])]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ra, rb = G.forward(cfg, w, a), G.forward(cfg, w, b)
    V = cfg["vocab"]
    s0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
    close(s0, torch.stack([ra[0], ra[29], rb[0]]), TOL[torch.float32], "step 0")
    s1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V))
    close(s1, ra[39:40], TOL[torch.float32], "step 1")
    s2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
    close(s2, torch.stack([rb[2], ra[1]]), TOL[torch.float32], "step 2")
