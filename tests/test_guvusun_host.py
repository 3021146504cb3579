"""Host-side pieces of Guvusun on the CPU: configuration checks, the registry entry, typed state slots, and properties of the float64
restatement that the GPU tests lean on (so that a fault there is not taken for a fault of the product)."""
import copy

import pytest
import torch

from candle_vllm_b200 import synthetic as S
from candle_vllm_b200._lib import BackendError
from candle_vllm_b200.guvusun import GuvusunConfig
from candle_vllm_b200.registry import registered
from candle_vllm_b200.state_cache import StateCache
from oracle import guvusun as G

CFG = S.guvusun_config(48, 60, [S.guvusun_layer(3, 8, 4, 12, 20, experts=4, ff=16, top=2, identity=2, groups=(3, 2)),
                                S.guvusun_layer(2, 6, 4, 8, 20, experts=2, ff=8, top=1, kv_from=0)],
                       bigram=dict(buckets=11, mul_prev=5, mul_cur=3), side_dim=6)


def test_registered_and_config_roundtrip():
    assert "Guvusun" in registered()
    c = GuvusunConfig.from_dict(copy.deepcopy(CFG))
    assert (c.vocab, c.width, c.alpha, c.side_dim) == (60, 48, 1.5, 6) and c.bigram["buckets"] == 11


@pytest.mark.parametrize("edit,needle", [
    (lambda d: d["layers"][0].update(type="other"), "unknown mixer"),
    (lambda d: d["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
    (lambda d: d["layers"][1]["mixer"].update(kv_rank=24), "must equal"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "feed-forward kind"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=2), "rotation spans"),
    (lambda d: d["layers"][0]["mixer"].pop("vdim"), "lacks"),
    (lambda d: d.pop("width"), "lacks"),
])
def test_config_faults_are_named(edit, needle):
    d = copy.deepcopy(CFG)
    edit(d)
    with pytest.raises(BackendError, match=needle):
        GuvusunConfig.from_dict(d)


def test_typed_state_slots():
    st = StateCache([(((1,), torch.int32),), ((2, 3), (4,))], 3, device="cpu")
    assert st.tensors[0][0].dtype == torch.int32 and st.tensors[0][0].shape == (4, 1)
    assert st.tensors[1][0].dtype == torch.float32 and st.tensors[1][1].shape == (4, 4)
    assert st.bytes_per_slot() == 4 + 24 + 16


def test_oracle_router_properties():
    g = torch.Generator().manual_seed(0)
    h = torch.randn(40, 16, generator=g, dtype=torch.float64)
    wr = torch.randn(12, 16, generator=g) * 0.8
    corr = torch.randn(12, generator=g) * 0.3 - 1.0
    r = dict(top=3, scale=2.0, groups=dict(count=4, keep=2))
    ids, ws = G.route(h, wr, corr, r)
    assert torch.allclose(ws.sum(-1), torch.full((40,), 2.0, dtype=torch.float64))
    s = torch.softmax(h @ wr.double().T, -1)
    pick = s + corr.double()
    for t in range(40):
        groups = sorted(range(4), key=lambda k: -float(pick[t, 3 * k:3 * k + 3].max()))[:2]
        assert all(int(e) // 3 in groups for e in ids[t])
        allowed = [e for e in range(12) if e // 3 in groups]
        assert sorted(ids[t].tolist()) == sorted(sorted(allowed, key=lambda e: -float(pick[t, e]))[:3])


def test_oracle_bigram_rows_and_sink():
    assert G.bigram_rows([4, 9, 9], 11, 5, 3) == [11, (4 * 5 + 9 * 3) % 11, (9 * 5 + 9 * 3) % 11]
    # the sink only takes weight away: with a huge sink the mixer's output vanishes, with none the first row attends fully to itself
    w = {k[len("l0.mix."):]: v for k, v in S.guvusun_weights(CFG, 0).items() if k.startswith("l0.mix.")}
    m = CFG["layers"][0]["mixer"]
    h = torch.randn(5, 48, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    big = dict(w, sink=torch.full((3,), 40.0))
    assert float(G.latent_attention(h, big, m, 1e-6)[0].abs().max()) < 1e-9
    none = {k: v for k, v in w.items() if k not in ("sink", "g")}
    c, _ = G.latent_kv(h[:1], w["dkv"], w["dkv.norm"], 20, 4, m["rot"], 1e-6)
    v0 = (c @ w["uv"].double().T) @ w["o"].double().T
    assert torch.allclose(G.latent_attention(h, none, m, 1e-6)[0][0], v0[0], atol=1e-9)


def test_oracle_whole_model_is_causal():
    w = S.guvusun_weights(CFG, 0)
    toks = list(range(1, 30))
    a = G.forward(CFG, w, toks)
    b = G.forward(CFG, w, toks[:17] + [59] * 12)
    assert torch.allclose(a[:17], b[:17], atol=1e-12) and not torch.allclose(a[17:], b[17:], atol=1e-3)
