"""Gobesun on the GPU against the plain float64 restatement in oracle/gobesun.py: every mechanism alone, then whole models through the
runner (portions, decode, batches, reused blocks and slots) and greedy generation through LLMEngine.  Configurations are small and
made here; none of the values that one model might happen to make equal (heads == kv_heads, dim == vdim, chunk == block size,
taps == 4, one pass) is left equal everywhere."""
import math

import numpy as np
import pytest
import torch

import candle_vllm_b200 as pkg
from candle_vllm_b200 import seq_ops as ops, synthetic as S
from candle_vllm_b200.engine import LLMEngine, ModelRunner
from candle_vllm_b200.gobesun import GobesunConfig, GobesunModel
from candle_vllm_b200.inputs import prepare_step
from candle_vllm_b200.mixers import yarn_rotary_tables
from oracle import gobesun as G

pytestmark = pytest.mark.gpu
DEV = "cuda"
F64 = torch.float64


def dev(t, dt=torch.float32):
    return t.to(dt).to(DEV).contiguous()


def batch_of(entries, block_size=64):
    return ops.StepBatch.from_host(prepare_step(entries, block_size), DEV)


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().to(F64), want.detach().cpu().to(F64)
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err < tol, f"{what}: max-err/max = {err:.3e} (tolerance {tol})"


# ----------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ----------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [5, 96, 321, 1030])
def test_rms_norm_variants(n):
    g = torch.Generator().manual_seed(n)
    x, w, r = torch.randn(7, n, generator=g) * 3, torch.randn(n, generator=g) * 0.3, torch.randn(7, n, generator=g)
    want = G.norm_zero_centred(x.to(F64), w.to(F64), 1e-6)
    close(ops.rms_norm_ex(dev(x), dev(w), 1e-6, 1.0, torch.float32), want, 2e-6, "offset weight")
    close(ops.rms_norm_ex(dev(x), dev(w), 1e-6, 0.0, torch.float32), G.rms(x.to(F64), 1e-6) * w.to(F64), 2e-6, "plain weight")
    res = dev(r)
    ops.rms_norm_ex(dev(x), dev(w), 1e-6, 1.0, torch.float32, residual=res, out=res)
    close(res, r.to(F64) + want, 2e-6, "closing norm, in place")
    idx = torch.tensor([6, 0, 3], dtype=torch.int32)
    close(ops.rms_norm_ex(dev(x), dev(w), 1e-6, 1.0, torch.float32, row_index=idx.to(DEV)), want[idx.long()], 2e-6, "gathered rows")
    close(ops.rms_norm_ex(dev(x), dev(w), 1e-6, 1.0, torch.bfloat16), want, 6e-3, "bf16 out")


def test_gelu_embedding():
    g = torch.Generator().manual_seed(0)
    gu = torch.randn(9, 2 * 37, generator=g) * 2
    close(ops.gelu_tanh_mul(dev(gu), torch.float32), G.gelu_tanh(gu[:, :37].to(F64)) * gu[:, 37:].to(F64), 2e-6, "gelu_tanh_mul")
    tab = torch.randn(50, 33, generator=g).to(torch.bfloat16)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    close(ops.embedding_scaled(tab.to(DEV), ids.to(DEV), 5.5), tab.to(F64)[ids.long()] * 5.5, 1e-6, "bf16 table")
    close(ops.embedding_scaled(dev(tab), ids.to(DEV), 5.5), tab.to(F64)[ids.long()] * 5.5, 1e-6, "f32 table")


@pytest.mark.parametrize("m,n,k", [(1, 4, 320), (3, 130, 72), (23, 6, 96), (70, 257, 100), (200, 64, 328), (600, 48, 64)])
def test_linear_f32out(m, n, k):
    g = torch.Generator().manual_seed(m * n)
    x, w = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g) * k ** -0.5
    close(ops.linear(dev(x), dev(w)), x.to(F64) @ w.to(F64).T, 3e-6, "f32")
    xb, wb = x.to(torch.bfloat16), w.to(torch.bfloat16)
    close(ops.linear(xb.to(DEV), wb.to(DEV)), xb.to(F64) @ wb.to(F64).T, 2e-5, "bf16 operands, f32 accumulation")
    # a strided view of a wider buffer (how the mixers read slices of their fused projection)
    wide = torch.randn(m, k + 24, generator=g)
    close(ops.linear(dev(wide)[:, 8:8 + k], dev(w)), wide[:, 8:8 + k].to(F64) @ w.to(F64).T, 3e-6, "strided f32")


def _portions(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append((at, n)); at += n; i += 1
    return out


@pytest.mark.parametrize("taps,sizes", [(4, [50]), (4, [1]), (3, [2, 1, 5]), (2, [3, 2]), (5, [2, 7, 1, 1, 11])])
def test_short_convolution_carries_its_inputs(taps, sizes):
    g = torch.Generator().manual_seed(taps)
    T, Cn = 50, 70
    x, w = torch.randn(T, Cn + 10, generator=g), torch.randn(Cn, taps, generator=g)
    want = G.silu(G.short_conv(x[:, :Cn].to(F64), w.to(F64)))
    state = torch.full((3, taps - 1, Cn), 7.0, device=DEV)       # dirty slots: a new sequence must not see them
    xd, got = dev(x), []
    for at, n in _portions(T, sizes):
        b = batch_of([dict(tokens=[0] * n, start=at, block_table=[0], state_slot=2, want=[])])
        got.append(ops.causal_conv_silu(xd[at:at + n, :Cn], dev(w), state, b))
    close(torch.cat(got), want, 2e-6, f"taps {taps} portions {sizes}")


def _delta_case(H, Gk, dk, dv, T, seed):
    """random inputs of the rule and the plain recurrence over them"""
    g = torch.Generator().manual_seed(seed)
    Cn = 2 * Gk * dk + H * dv
    qkv = torch.randn(T, Cn, generator=g)
    proj = torch.randn(T, 2 * H + 3, generator=g) * 2
    A_log, dt_bias = torch.rand(H, generator=g) * 4 - 4, torch.rand(H, generator=g) * 3 - 4
    A_log[0] = -8.0                                          # one head that forgets very slowly: early tokens still count at the end
    q = G.unit(qkv[:, :Gk * dk].to(F64).view(T, Gk, dk)) * dk ** -0.5
    k = G.unit(qkv[:, Gk * dk:2 * Gk * dk].to(F64).view(T, Gk, dk))
    v = qkv[:, 2 * Gk * dk:].to(F64).view(T, H, dv)
    rep = H // Gk
    beta = torch.sigmoid(proj[:, 1:1 + H].to(F64))
    decay = torch.exp(-torch.exp(A_log.to(F64)) * torch.nn.functional.softplus(proj[:, 2 + H:2 + 2 * H].to(F64) + dt_bias.to(F64)))
    want = G.delta_recurrence(q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1), v, beta, decay).reshape(T, H * dv)
    return qkv, proj, A_log, dt_bias, want


@pytest.mark.parametrize("kernel", ["token", "tiled", "step"])
@pytest.mark.parametrize("H,Gk,dk,dv", [(4, 2, 64, 32), (2, 2, 32, 16), (3, 1, 128, 80), (4, 4, 48, 24), (2, 1, 200, 40), (2, 1, 30, 17), (2, 2, 300, 20)])
def test_gated_delta_rule(H, Gk, dk, dv, kernel):
    """the kernels of the rule, alone: token by token; over tiles of 16 tokens; one token per entry (portions of one row only)"""
    if kernel == "tiled" and dk > 128:
        pytest.skip("the tiled kernel takes key sizes up to 128")
    T = 90 if kernel != "step" else 40
    qkv, proj, A_log, dt_bias, want = _delta_case(H, Gk, dk, dv, T, dk + dv)
    for sizes in ([T], [1], [2, 3, 1, 17], [16], [33, 15, 32, 7]) if kernel != "step" else ([1],):
        state = torch.full((2, H, dv, dk), 3.0, device=DEV)
        got = []
        for at, n in _portions(T, sizes):
            b = batch_of([dict(tokens=[0] * n, start=at, block_table=[0, 1], state_slot=1, want=[])])
            got.append(ops.gated_delta_rule(dev(qkv)[at:at + n], dev(proj)[at:at + n], 1, 2 + H, dev(A_log), dev(dt_bias), state, b, H, Gk, dk, dv, kernel=kernel))
        close(torch.cat(got), want[:T], 5e-6, f"portions {sizes}")


@pytest.mark.parametrize("kernel", ["token", "tiled", None])
def test_gated_delta_rule_unequal_entries(kernel):
    """Several sequences in one step, portions of unequal length beside single tokens, each continuing from its own slot: every one
    comes out as it does alone.  With kernel = None the tiled, the single-token and again the tiled kernel run in turn and hand the state on."""
    H, Gk, dk, dv = 4, 2, 40, 24
    lens = [37, 1, 16, 5, 70]
    cases = [_delta_case(H, Gk, dk, dv, n + 9, 100 + i) for i, n in enumerate(lens)]
    state = torch.full((len(lens) + 1, H, dv, dk), -2.0, device=DEV)
    A_log, dt_bias = cases[0][2], cases[0][3]                # one model: the same per-head constants for every sequence
    outs = [[] for _ in lens]
    for step, take in enumerate((lambda n: n, lambda n: 1, lambda n: 8)):
        rows_q, rows_p, entries, spans = [], [], [], []
        for i, n in enumerate(lens):
            at = 0 if step == 0 else (n if step == 1 else n + 1)
            m = take(n)
            rows_q.append(cases[i][0][at:at + m]); rows_p.append(cases[i][1][at:at + m])
            entries.append(dict(tokens=[0] * m, start=at, block_table=[0, 1], state_slot=len(lens) - i, want=[]))
            spans.append(m)
        b = batch_of(entries)
        got = ops.gated_delta_rule(dev(torch.cat(rows_q)), dev(torch.cat(rows_p)), 1, 2 + H, dev(A_log), dev(dt_bias), state, b, H, Gk, dk, dv,
                                   kernel=kernel)
        for i, piece in enumerate(torch.split(got, spans)):
            outs[i].append(piece)
    for i, n in enumerate(lens):
        qkv, proj, _, _, _ = cases[i]
        # the oracle with this test's shared constants
        q = G.unit(qkv[:, :Gk * dk].to(F64).view(-1, Gk, dk)) * dk ** -0.5
        k = G.unit(qkv[:, Gk * dk:2 * Gk * dk].to(F64).view(-1, Gk, dk))
        v = qkv[:, 2 * Gk * dk:].to(F64).view(-1, H, dv)
        beta = torch.sigmoid(proj[:, 1:1 + H].to(F64))
        decay = torch.exp(-torch.exp(A_log.to(F64)) * torch.nn.functional.softplus(proj[:, 2 + H:2 + 2 * H].to(F64) + dt_bias.to(F64)))
        ref = G.delta_recurrence(q.repeat_interleave(H // Gk, 1), k.repeat_interleave(H // Gk, 1), v, beta, decay).reshape(-1, H * dv)
        close(torch.cat(outs[i]), ref, 5e-6, f"entry {i} ({n} rows, then 1, then 8)")


def test_gated_rms_norm():
    g = torch.Generator().manual_seed(3)
    T, H, dv = 11, 3, 40
    o, gate, w = torch.randn(T, H * dv, generator=g), torch.randn(T, H * dv + 5, generator=g), torch.randn(dv, generator=g)
    want = (G.rms(o.to(F64).view(T, H, dv), 1e-5) * w.to(F64) * G.silu(gate[:, 5:].to(F64)).view(T, H, dv)).reshape(T, H * dv)
    close(ops.gated_rms_norm(dev(o), dev(gate)[:, 5:], dev(w), H, dv, 1e-5, torch.float32), want, 2e-6, "gated norm")


@pytest.mark.parametrize("scaling", [None, dict(factor=4.0, original=2048, fast=32.0, slow=1.0), dict(factor=8.0, original=512, fast=16.0, slow=2.0)])
def test_rotary_tables(scaling):
    rot = dict(dims=24, base=50000.0)
    if scaling:
        rot["scaling"] = scaling
    cos, sin = yarn_rotary_tables(24, 50000.0, 700, scaling, DEV)
    wc, ws = G.rotary_angles(rot, torch.arange(700))
    close(cos, wc, 1e-6, "cos"); close(sin, ws, 1e-6, "sin")


def _attention_case(H, Gk, dk, dv, chunk, T, rot_dims, seed, cache_dtype=torch.float32, bs=16):
    """q / k / v rows of one sequence at positions 0..T-1, the product's result through the paged cache in portions, the oracle's."""
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(T, H * dk + Gk * dk + Gk * dv, generator=g)
    qn, kn = 1 + 0.3 * torch.randn(H * dk, generator=g), 1 + 0.3 * torch.randn(Gk * dk, generator=g)
    return g, qkv, qn, kn


@pytest.mark.parametrize("H,Gk,dk,dv,chunk,rot_dims", [(4, 4, 64, 64, 96, 32), (6, 2, 32, 48, 40, 32), (2, 1, 80, 16, 7, 10), (3, 3, 16, 100, 0, 0)])
def test_attention_norm_rotation_cache_and_chunk_mask(H, Gk, dk, dv, chunk, rot_dims):
    T, bs, eps, scale = 150, 16, 1e-6, 0.17
    g, qkv, qn, kn = _attention_case(H, Gk, dk, dv, chunk, T, rot_dims, seed=H * dk)
    rot = dict(dims=rot_dims, base=1e4, scaling=dict(factor=4.0, original=64, fast=8.0, slow=1.0)) if rot_dims else None
    pos = torch.arange(T)
    q = (G.rms(qkv[:, :H * dk].to(F64), eps) * qn.to(F64)).view(T, H, dk)
    k = (G.rms(qkv[:, H * dk:(H + Gk) * dk].to(F64), eps) * kn.to(F64)).view(T, Gk, dk)
    v = qkv[:, (H + Gk) * dk:].to(F64).view(T, Gk, dv)
    cos = sin = None
    if rot:
        wc, ws = G.rotary_angles(rot, pos)
        q, k = G.rotate(q, wc, ws, rot_dims), G.rotate(k, wc, ws, rot_dims)
        cos, sin = yarn_rotary_tables(rot_dims, 1e4, T, rot["scaling"], DEV)
    want = G.masked_attention(q, k, v, scale, dict(size=chunk) if chunk else None, pos).reshape(T, H * dv)
    nb = -(-T // bs)
    table = list(np.random.default_rng(1).permutation(nb + 3)[:nb])          # scattered physical blocks
    for sizes in ([T], [1], [2, 5, 1, 31]):
        kc = torch.full((nb + 3, bs, Gk, dk), 9.0, device=DEV)
        vc = torch.full((nb + 3, bs, Gk, dv), 9.0, device=DEV)
        got = []
        for at, n in _portions(T, sizes):
            b = batch_of([dict(tokens=[0] * n, start=at, block_table=table, state_slot=-1, want=[])], bs)
            qq = ops.qk_norm_rope_cache(dev(qkv)[at:at + n], dev(qn), dev(kn), cos, sin, b, kc, vc, H, Gk, dk, dv, rot_dims, eps)
            got.append(ops.paged_attention_varlen(qq, kc, vc, b, H, Gk, dk, dv, bs, scale, chunk, 0, torch.float32))
        close(torch.cat(got), want, 5e-6, f"portions {sizes}")


@pytest.mark.parametrize("chunk,bs,tc", [(96, 64, False), (40, 16, False), (64, 64, False), (96, 64, True), (40, 64, True), (64, 64, True), (130, 64, True)])
def test_attention_edges_show_a_key_one_off(chunk, bs, tc):
    """One key per probe is made to dominate (its score stands far above the rest).  Queries at the first position of a chunk must not
    see the key just before them; queries at the last position of a chunk must see the chunk's first key; both across page borders."""
    H = Gk = 1
    dk, dv, T = (128, 128, 3 * chunk + 5) if tc else (8, 4, 3 * chunk + 5)      # tc: the shapes the tensor-core kernel takes (bf16 cache and q)
    cdt, tol = (torch.bfloat16, 1e-2) if tc else (torch.float32, 1e-5)
    g = torch.Generator().manual_seed(chunk)
    q = torch.randn(T, 1, dk, generator=g) * 0.1
    k = torch.randn(T, 1, dk, generator=g) * 0.1
    v = torch.randn(T, 1, dv, generator=g)
    mark = torch.zeros(dk); mark[0] = 1.0
    probes = []
    for c in (1, 2, 3):
        first, last_prev = c * chunk, c * chunk - 1
        k[last_prev, 0] = 40 * mark; v[last_prev, 0] = 100.0           # loud key just outside the next chunk
        q[first, 0] = 40 * mark
        probes.append(first)
        if first + chunk - 1 < T:
            q[first + chunk - 1, 0] = -40 * mark                         # looks for the chunk's first key, far back inside the chunk
            k[first, 0] = -40 * mark + k[first, 0] * 0; v[first, 0] = -50.0
            probes.append(first + chunk - 1)
    pos = torch.arange(T)
    q, k, v = (x.to(cdt).float() for x in (q, k, v))
    want = G.masked_attention(q.to(F64), k.to(F64), v.to(F64), 1.0, dict(size=chunk), pos).reshape(T, dv)
    assert all(abs(float(want[p, 0])) < 60 for p in probes if p % chunk == 0)        # the loud outside key is not in the answer
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1)
    nb = -(-T // bs)
    for sizes in ([T], [1], [chunk - 1, 2, 1], [bs, 3]):
        kc, vc = torch.zeros((nb, bs, 1, dk), device=DEV, dtype=cdt), torch.zeros((nb, bs, 1, dv), device=DEV, dtype=cdt)
        got = []
        for at, n in _portions(T, sizes):
            b = batch_of([dict(tokens=[0] * n, start=at, block_table=list(range(nb)), state_slot=-1, want=[])], bs)
            qq = ops.qk_norm_rope_cache(dev(qkv)[at:at + n], None, None, None, None, b, kc, vc, 1, 1, dk, dv, 0, 1e-6, cdt)
            got.append(ops.paged_attention_varlen(qq, kc, vc, b, 1, 1, dk, dv, bs, 1.0, chunk, 0, cdt))
        close(torch.cat(got), want, tol, f"chunk {chunk} portions {sizes}")


@pytest.mark.parametrize("chunk", [96, 64, 200, 33, 0])
def test_tensor_core_attention_path(chunk):
    """bf16 q / cache / out with 128-wide heads and 64-token blocks runs on the tensor-core kernel: random rows, grouped heads, scattered
    blocks, two requests of unequal progress in one step"""
    H, Gk, dk, bs, scale = 4, 2, 128, 64, 0.09
    g = torch.Generator().manual_seed(chunk)
    lens = (300, 131)
    data, wants = [], []
    for T in lens:
        q, k, v = (torch.randn(T, n, dk, generator=g).to(torch.bfloat16).float() for n in (H, Gk, Gk))
        data.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1))
        wants.append(G.masked_attention(q.to(F64), k.to(F64), v.to(F64), scale, dict(size=chunk) if chunk else None, torch.arange(T)).reshape(T, -1))
    nb = 8
    perm = list(np.random.default_rng(2).permutation(nb))
    tables = [perm[:5], perm[5:]]
    kc = torch.zeros((nb, bs, Gk, dk), device=DEV, dtype=torch.bfloat16); vc = torch.zeros_like(kc)
    plans = [[70, 1, 1, 64, 100, 1, 63], [1, 2, 64, 1, 1, 30, 32]]
    fed, got, step = [0, 0], [[], []], 0
    while fed[0] < lens[0] or fed[1] < lens[1]:
        ent, ns = [], []
        for i in (0, 1):
            n = min(plans[i][step % 7], lens[i] - fed[i])
            ns.append(n)
            if n:
                ent.append(dict(tokens=[0] * n, start=fed[i], block_table=tables[i], state_slot=-1, want=[]))
        b = batch_of(ent, bs)
        rows = torch.cat([data[i][fed[i]:fed[i] + ns[i]] for i in (0, 1)])
        qq = ops.qk_norm_rope_cache(dev(rows), None, None, None, None, b, kc, vc, H, Gk, dk, dk, 0, 1e-6, torch.bfloat16)
        out = ops.paged_attention_varlen(qq, kc, vc, b, H, Gk, dk, dk, bs, scale, chunk, 0, torch.bfloat16)
        at = 0
        for i in (0, 1):
            got[i].append(out[at:at + ns[i]]); at += ns[i]; fed[i] += ns[i]
        step += 1
    for i in (0, 1):
        close(torch.cat(got[i]), wants[i], 1.5e-2, f"chunk {chunk} request {i}")


def test_sliding_window_parameter():
    """The same kernel with a window instead of a chunk (for designs that use one): key j is seen iff 0 <= i - j < window."""
    T, dk, dv, win, bs = 70, 16, 8, 9, 16
    g = torch.Generator().manual_seed(5)
    q, k, v = torch.randn(T, 2, dk, generator=g), torch.randn(T, 1, dk, generator=g), torch.randn(T, 1, dv, generator=g)
    want = torch.zeros(T, 2, dv, dtype=F64)
    for i in range(T):
        lo = max(0, i - win + 1)
        for h in range(2):
            s = torch.softmax((k[lo:i + 1, 0].to(F64) @ q[i, h].to(F64)) * 0.3, 0)
            want[i, h] = s @ v[lo:i + 1, 0].to(F64)
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1)
    nb = -(-T // bs)
    kc, vc = torch.zeros((nb, bs, 1, dk), device=DEV), torch.zeros((nb, bs, 1, dv), device=DEV)
    b = batch_of([dict(tokens=[0] * T, start=0, block_table=list(range(nb)), state_slot=-1, want=[])], bs)
    qq = ops.qk_norm_rope_cache(dev(qkv), None, None, None, None, b, kc, vc, 2, 1, dk, dv, 0, 1e-6)
    close(ops.paged_attention_varlen(qq, kc, vc, b, 2, 1, dk, dv, bs, 0.3, 0, win, torch.float32), want.reshape(T, -1), 5e-6, "window")


# ----------------------------------------------------------------------------------------------------------------------
# whole models through the runner
# ----------------------------------------------------------------------------------------------------------------------
YARN = dict(factor=4.0, original=128, fast=16.0, slow=1.0)
CONFIGS = {
    # looped span of an attention + a recurrent layer, then a recurrent layer with a feed-forward; chunk smaller than a block
    "loop2": S.gobesun_config(96, 160, [S.gobesun_attention_layer(6, 3, 32, 24, 40, 16, ff=128, scaling=YARN, scale=0.21),
                                        S.gobesun_delta_layer(4, 2, 48, 24, conv=3),
                                        S.gobesun_delta_layer(2, 2, 32, 40, conv=4, ff=72)], loop=dict(start=0, stop=2, times=2)),
    # recurrent first, attention without scaling and with full-head rotation, chunk larger than a block, no loop entry at all
    "plain": S.gobesun_config(72, 97, [S.gobesun_delta_layer(3, 1, 64, 16, conv=2, ff=80),
                                       S.gobesun_attention_layer(2, 1, 24, 56, 100, 24),
                                       S.gobesun_attention_layer(4, 4, 16, 16, 33, 8, ff=64, scaling=dict(factor=2.0, original=64, fast=4.0, slow=0.5))]),
    # the whole model looped three times, one head everywhere
    "tiny": S.gobesun_config(40, 50, [S.gobesun_delta_layer(1, 1, 128, 32, conv=5), S.gobesun_attention_layer(1, 1, 40, 8, 64, 40, ff=48)],
                             loop=dict(start=0, stop=2, times=3)),
}
# attention heads of 128 with 64-token blocks: in bf16 this is the tensor-core attention path
CONFIGS["wide"] = S.gobesun_config(64, 80, [S.gobesun_attention_layer(2, 1, 128, 128, 96, 64, scaling=YARN), S.gobesun_delta_layer(2, 1, 32, 32, conv=4, ff=96)],
                                   loop=dict(start=0, stop=1, times=2))
# the same with chunks that start on block borders: single-token steps in bf16 then run on the split-KV decode kernel
CONFIGS["wide64"] = S.gobesun_config(64, 80, [S.gobesun_delta_layer(2, 2, 64, 16, conv=3), S.gobesun_attention_layer(4, 2, 128, 128, 128, 32, ff=96)],
                                     loop=dict(start=1, stop=2, times=2))
# degenerate sizes: a 1-tap convolution (no carried inputs), rotation of the whole head without scaling, one pass of a one-layer loop,
# odd width / vocabulary / ff (no 8-element alignment anywhere), only recurrent + one attention layer without feed-forward
CONFIGS["odd"] = S.gobesun_config(52, 61, [S.gobesun_delta_layer(2, 1, 20, 12, conv=1, ff=44), S.gobesun_attention_layer(3, 3, 12, 20, 50, 12)],
                                  loop=dict(start=1, stop=2, times=1), eps=1e-5, embedding_scale=3.0)
CONFIGS["plain"].pop("loop")
_CACHE = {}


def model_and_oracle(name, dtype, n_tokens, seed=0):
    cfg = CONFIGS[name]
    key = (name, seed)
    if key not in _CACHE:
        w = S.gobesun_weights(cfg, seed)
        toks = torch.randint(0, cfg["vocab"], (300,), generator=torch.Generator().manual_seed(seed + 1)).tolist()
        _CACHE[key] = (w, toks, G.forward(cfg, w, toks))
    w, toks, ref = _CACHE[key]
    assert len(toks) >= n_tokens
    model = GobesunModel(GobesunConfig.from_dict(cfg), w, dtype=dtype, block_size=64, max_pos=512, device=DEV)
    return model, toks[:n_tokens], ref[:n_tokens]


def run_schedule(runner, seq_id, toks, sizes, want_all=True):
    """feeds toks in portions; returns logits of every position"""
    runner.admit(seq_id)
    out = []
    for at, n in _portions(len(toks), sizes):
        out.append(runner.execute([dict(seq_id=seq_id, tokens=toks[at:at + n], want=list(range(n)))]))
    runner.release(seq_id)
    return torch.cat(out)


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_matches_the_oracle(name, dtype):
    model, toks, ref = model_and_oracle(name, dtype, 230)
    runner = ModelRunner(model, 8, 2, 64)
    trace = []
    runner.admit(0)
    got = runner.execute([dict(seq_id=0, tokens=toks, want=list(range(len(toks))))], hidden_trace=trace)
    close(got, ref, TOL[dtype], f"{name} logits")
    if dtype == torch.float32:
        want_trace = []
        G.forward(CONFIGS[name], _CACHE[(name, 0)][0], toks, want_trace)
        assert len(trace) == len(want_trace) == len(model.runs)
        for i, (a, b) in enumerate(zip(trace, want_trace)):
            close(a, b, 1e-4, f"{name} residual after run {i}")


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("sizes", [[1], [2], [3, 2, 7], [64, 1, 1, 5], [39, 1, 41, 2, 63]])
def test_portions_and_decoding_match_the_whole_prompt(name, sizes):
    model, toks, ref = model_and_oracle(name, torch.float32, 230)
    runner = ModelRunner(model, 4, 1, 64)
    close(run_schedule(runner, 5, toks, sizes), ref, TOL[torch.float32], f"{name} portions {sizes}")


def test_portions_in_bf16_stay_within_rounding():
    model, toks, ref = model_and_oracle("loop2", torch.bfloat16, 200)
    runner = ModelRunner(model, 4, 1, 64)
    whole = run_schedule(runner, 0, toks, [200])
    parts = run_schedule(runner, 1, toks, [37, 2, 1, 1, 64])
    close(parts, ref, TOL[torch.bfloat16], "bf16 portions")
    close(parts, whole, 3e-2, "bf16 portions against the whole prompt")


@pytest.mark.parametrize("name", ["wide", "wide64"])
def test_bf16_decoding_on_the_tensor_core_attention_paths(name):
    """128-wide heads in bf16: prompt portions and mixed steps use the tensor-core prefill kernel, steps of single tokens the split-KV
    decode kernel when chunks start on block borders; two requests decode side by side across chunk and block edges"""
    cfg = CONFIGS[name]
    w = S.gobesun_weights(cfg, 0)
    model = GobesunModel(GobesunConfig.from_dict(cfg), w, dtype=torch.bfloat16, block_size=64, max_pos=512, device=DEV)
    g = torch.Generator().manual_seed(5)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (300, 270)]
    refs = [G.forward(cfg, w, s) for s in seqs]
    runner = ModelRunner(model, 10, 2, 64)
    runner.admit(0); runner.admit(1)
    got = [[], []]
    out = runner.execute([dict(seq_id=0, tokens=seqs[0][:100], want=list(range(100))), dict(seq_id=1, tokens=seqs[1][:1], want=[0])])
    got[0].append(out[:100]); got[1].append(out[100:])
    fed = [100, 1]
    while fed[0] < 300 or fed[1] < 270:
        live = [i for i in (0, 1) if fed[i] < len(seqs[i])]
        out = runner.execute([dict(seq_id=i, tokens=[seqs[i][fed[i]]], want=[0]) for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1]); fed[i] += 1
    for i in (0, 1):
        close(torch.cat(got[i]), refs[i], TOL[torch.bfloat16], f"{name} request {i}")


@pytest.mark.parametrize("name", ["loop2", "plain"])
def test_unequal_batches_match_each_request_alone(name):
    """Four requests of different lengths advance together, portions of some beside single tokens of others; the pool is smaller than the
    sum of all requests, so blocks and slots of finished requests go to later ones (slots are handed over dirty)."""
    cfg = CONFIGS[name]
    w = S.gobesun_weights(cfg, 0)
    model = GobesunModel(GobesunConfig.from_dict(cfg), w, dtype=torch.float32, block_size=64, max_pos=512, device=DEV)
    g = torch.Generator().manual_seed(9)
    lens = [130, 7, 64, 201, 65, 1, 90]
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    refs = [G.forward(cfg, w, s) for s in seqs]
    runner = ModelRunner(model, 9, 3, 64)            # 9 blocks, 3 slots: not everything fits at once
    plans = [[64, 1, 1, 30, 2, 1], [2, 1], [63, 1], [100, 3, 1, 1, 50, 2], [64, 1], [1], [1, 1, 1, 80, 2]]
    waiting, live, got = list(range(len(seqs))), {}, {i: [] for i in range(len(seqs))}
    guard = 0
    while waiting or live:
        guard += 1
        assert guard < 500
        while waiting and runner.state.pool.num_free() > 0 and runner.can_admit(lens[waiting[0]], sum(-(-lens[i] // 64) - len(runner.blocks.tables.get(i, ())) for i in live)):
            i = waiting.pop(0)
            runner.admit(i)
            live[i] = [0, 0]                         # tokens fed, index into its plan
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


def test_long_decoding_across_chunks_and_blocks():
    model, toks, ref = model_and_oracle("tiny", torch.float32, 300)
    runner = ModelRunner(model, 5, 1, 64)
    runner.admit(0)
    got = [runner.execute([dict(seq_id=0, tokens=toks[:20], want=list(range(20)))])]
    for t in range(20, 300):
        got.append(runner.execute([dict(seq_id=0, tokens=[toks[t]], want=[0])]))
    close(torch.cat(got), ref, TOL[torch.float32], "280 decoded tokens")


def test_first_tokens_and_single_token_requests():
    model, toks, ref = model_and_oracle("loop2", torch.float32, 230)
    runner = ModelRunner(model, 4, 2, 64)
    for n in (1, 2, 3):
        runner.admit(n)
        close(runner.execute([dict(seq_id=n, tokens=toks[:n], want=list(range(n)))]), ref[:n], TOL[torch.float32], f"first {n} tokens")
        runner.release(n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_engine(dtype, tmp_path):
    """checkpoint on disk -> registry -> LLMEngine (scheduler, chunked prefill, sampler) against the oracle's greedy continuation"""
    import json
    from candle_vllm_b200.safetensors_io import save_file
    cfg = CONFIGS["plain"]
    w = S.gobesun_weights(cfg, 4)
    save_file(w, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (70, 3, 33, 1, 129)]
    eng = LLMEngine.from_pretrained(str(tmp_path), dtype=dtype, num_blocks=7, max_num_seqs=2, prefill_chunk=48, max_batch_tokens=64, max_model_len=256)
    outs = eng.generate(prompts, pkg.SamplingParams(max_tokens=6))
    assert eng.runner.blocks.num_free_gpu_blocks() == 7 and eng.runner.state.pool.num_free() == 2
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        if dtype == torch.float32:
            assert o == G.greedy(cfg, w, p, 6)
        else:       # bf16 may flip a near-tie: every produced token must be within rounding of the oracle's best at its place
            ids = list(p)
            for t in o:
                lg = G.forward(cfg, w, ids)[-1]
                assert float(lg.max() - lg[t]) < 0.05 * float(lg.abs().max())
                ids.append(t)


def test_sampling_with_temperature_is_seeded(tmp_path):
    cfg = CONFIGS["tiny"]
    model = GobesunModel(GobesunConfig.from_dict(cfg), S.gobesun_weights(cfg, 1), dtype=torch.float32, device=DEV)
    outs = []
    for _ in range(2):
        eng = LLMEngine(model, num_blocks=4, max_num_seqs=2)
        outs.append(eng.generate([[1, 2, 3], [4, 5]], pkg.SamplingParams(temperature=0.9, top_k=12, top_p=0.9, max_tokens=8, seed=11)))
    assert outs[0] == outs[1] and all(0 <= t < cfg["vocab"] for o in outs[0] for t in o)


def test_graph_replay_of_decode_steps_matches_eager():
    """steps of single tokens through captured CUDA graphs (two batch sizes, growing tables) against the eager path and the oracle"""
    cfg = CONFIGS["loop2"]
    w = S.gobesun_weights(cfg, 0)
    model = GobesunModel(GobesunConfig.from_dict(cfg), w, dtype=torch.float32, block_size=64, max_pos=64, device=DEV)      # tables must grow
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
    assert 1 in runner._graphs            # (the two-entry graph was dropped when the rotary tables grew, and captured again while needed)
    for i in (0, 1):
        close(torch.cat(got[i]), refs[i], TOL[torch.float32], f"graph replay, request {i}")


def test_command_line_and_trace_runner(tmp_path):
    """the two programs a user starts, as child processes on a checkpoint on disk: `generate` against the oracle's greedy continuation,
    `bin/trace_run` fed two steps (a portion of one request beside the first token of another, then single tokens; the first request ends)
    against the oracle's logits"""
    import json, os, subprocess, sys
    from candle_vllm_b200.safetensors_io import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CONFIGS["plain"]
    w = S.gobesun_weights(cfg, 7)
    save_file(w, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    prompt = [5, 9, 2, 44, 17, 3]
    r = subprocess.run([sys.executable, "-m", "candle_vllm_b200", "generate", "--model", str(tmp_path), "--dtype", "float32", "--prompt-ids",
                        ",".join(map(str, prompt)), "--max-new-tokens", "5"], capture_output=True, text=True, env=env, cwd=root, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["output"] == G.greedy(cfg, w, prompt, 5)

    a, b = list(range(1, 71)), [7, 8, 9]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:69], "want": [0, 68]}, {"id": "b", "tokens": b[:1], "want": [0]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[69:], "want": [0]}, {"id": "b", "tokens": b[1:2], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": b[2:], "want": [0]}, {"id": "c", "tokens": a[:2], "want": [1]}], "end": ["b", "c"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "192"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, env=env, cwd=root, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ra, rb = G.forward(cfg, w, a), G.forward(cfg, w, b)
    V = cfg["vocab"]
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", np.float32).reshape(-1, V))
    close(got0, torch.stack([ra[0], ra[68], rb[0]]), TOL[torch.float32], "step 0")
    close(torch.from_numpy(np.fromfile(out / "1.f32", np.float32).reshape(-1, V)), ra[69:70], TOL[torch.float32], "step 1")
    close(torch.from_numpy(np.fromfile(out / "2.f32", np.float32).reshape(-1, V)), torch.stack([rb[2], ra[1]]), TOL[torch.float32], "step 2")
