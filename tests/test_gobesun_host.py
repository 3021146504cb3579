"""CPU tests of the host side that serves ragged-step models: step metadata, state slots, incremental block tables, the scheduler's
admission and batching, the checkpoint reader, the registry, the sampler and the Gobesun configuration."""
import json

import numpy as np
import pytest
import torch

import candle_vllm_b200 as pkg
from candle_vllm_b200 import synthetic as S
from candle_vllm_b200.block_manager import BlockManager
from candle_vllm_b200.engine import Request, Scheduler
from candle_vllm_b200.gobesun import GobesunConfig
from candle_vllm_b200.inputs import prepare_step
from candle_vllm_b200.mixers import yarn_rotary_tables
from candle_vllm_b200.registry import architecture_of, load_model, registered
from candle_vllm_b200.safetensors_io import load_file, read_header, save_file
from candle_vllm_b200.sampling import SamplingParams, sample_host
from candle_vllm_b200.state_cache import SlotPool
from oracle import gobesun as G


def test_prepare_step_layout():
    p = prepare_step([dict(tokens=[7, 8, 9], start=62, block_table=[5, 2], state_slot=3, want=[2]),
                      dict(tokens=[4], start=0, block_table=[9], state_slot=0, want=[0]),
                      dict(tokens=[1, 1], start=10, block_table=[4], state_slot=1, want=[])], 64)
    assert p["tokens"].tolist() == [7, 8, 9, 4, 1, 1]
    assert p["positions"].tolist() == [62, 63, 64, 0, 10, 11]
    assert p["token_seq"].tolist() == [0, 0, 0, 1, 2, 2]
    assert p["slot_mapping"].tolist() == [5 * 64 + 62, 5 * 64 + 63, 2 * 64, 9 * 64, 4 * 64 + 10, 4 * 64 + 11]
    assert p["cu_seqlens"].tolist() == [0, 3, 4, 6] and p["seq_slots"].tolist() == [3, 0, 1] and p["seq_start"].tolist() == [62, 0, 10]
    assert p["block_tables"].tolist() == [[5, 2], [9, 0], [4, 0]] and p["want_rows"].tolist() == [2, 3] and p["max_position"] == 64
    with pytest.raises(pkg.BackendError):
        prepare_step([dict(tokens=[1, 2], start=63, block_table=[0], state_slot=0, want=[])], 64)       # table too short
    with pytest.raises(pkg.BackendError):
        prepare_step([dict(tokens=[1], start=0, block_table=[0], state_slot=0, want=[1])], 64)


def test_slot_pool_hands_slots_on():
    sp = SlotPool(2)
    assert sp.acquire(10) == 0 and sp.acquire(11) == 1 and sp.acquire(10) == 0
    with pytest.raises(pkg.BackendError):
        sp.acquire(12)
    sp.release(10)
    assert sp.num_free() == 1 and sp.acquire(12) == 0 and not sp.has(10)


def test_block_tables_grow_by_exact_need_and_are_reused():
    bm = BlockManager(64, 3, 0)
    assert bm.grow_to(1, 64) == [0] and bm.blocks_to_hold(1, 64) == 0 and bm.blocks_to_hold(1, 65) == 1
    assert bm.grow_to(1, 65) == [0, 1] and bm.grow_to(2, 1) == [2]
    with pytest.raises(pkg.BackendError):
        bm.grow_to(2, 65)
    bm.free_table(1)
    assert bm.grow_to(2, 128) == [2, 0]
    bm.free_table(2); bm.check_invariants()
    assert bm.num_free_gpu_blocks() == 3


class _FakeRunner:
    """what Scheduler needs of ModelRunner, without a device"""

    def __init__(self, blocks, slots):
        from candle_vllm_b200.state_cache import SlotPool as SP
        self.block_size, self.blocks = 64, BlockManager(64, blocks, 0)
        self.state = type("S", (), {"pool": SP(slots)})()

    def admit(self, i):
        self.state.pool.acquire(i)

    def release(self, i):
        self.blocks.free_table(i); self.state.pool.release(i)


def test_scheduler_admission_chunks_and_mixed_steps():
    run = _FakeRunner(blocks=4, slots=2)
    sch = Scheduler(run, max_batch_tokens=50, max_num_seqs=2, prefill_chunk=40)
    a, b, c = (Request(i, list(range(n)), SamplingParams(max_tokens=4)) for i, n in ((0, 100), (1, 30), (2, 10)))
    for r in (a, b, c):
        sch.add(r)
    with pytest.raises(pkg.BackendError):
        sch.add(Request(3, list(range(300)), SamplingParams(max_tokens=4)))        # can never fit 4 blocks
    e = sch.schedule()                    # a (2 blocks reserved) and b (1 block) run; c waits for a slot
    assert [(x["seq_id"], len(x["tokens"]), x["want"]) for x in e] == [(0, 40, []), (1, 10, [])]
    for x in e:
        run.blocks.grow_to(x["seq_id"], x["request"].computed + len(x["tokens"])); x["request"].computed += len(x["tokens"])
    e = sch.schedule()
    assert [(x["seq_id"], len(x["tokens"]), x["want"]) for x in e] == [(0, 40, []), (1, 10, [])]
    for x in e:
        x["request"].computed += len(x["tokens"])
    e = sch.schedule()
    assert [(x["seq_id"], len(x["tokens"]), x["want"]) for x in e] == [(0, 20, [19]), (1, 10, [9])]
    for x in e:
        x["request"].computed += len(x["tokens"]); x["request"].output.append(5)
    e = sch.schedule()                    # both decode now: one token each, the fresh output token
    assert [(x["seq_id"], x["tokens"], x["want"]) for x in e] == [(0, [5], [0]), (1, [5], [0])]
    sch.finish(b)
    e = sch.schedule()                    # c takes b's slot and starts beside a's decode
    assert [(x["seq_id"], len(x["tokens"])) for x in e] == [(0, 1), (2, 10)] and e[1]["want"] == [9]


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int32), "d": torch.randn(2, 2, 2)}
    path = str(tmp_path / "x.safetensors")
    save_file(t, path)
    meta, base = read_header(path)
    assert meta["a"]["dtype"] == "BF16" and meta["a"]["shape"] == [3, 5] and base % 8 == 0
    back = load_file(path)
    assert set(back) == set(t) and all(back[k].dtype == t[k].dtype and torch.equal(back[k], t[k]) for k in t)
    with open(path, "r+b") as f:
        f.write((1 << 40).to_bytes(8, "little"))
    with pytest.raises(pkg.BackendError):
        read_header(path)


def test_registry_picks_the_class_by_config(tmp_path):
    assert "Gobesun" in registered()
    assert architecture_of({"architecture": "Gobesun"}) == "Gobesun" and architecture_of({"architectures": ["X"]}) == "X"
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(pkg.BackendError):
        load_model(str(tmp_path))


def test_registry_loads_a_dense_llama_checkpoint(tmp_path):
    """the other family goes through the same door: HF-style names -> the layout the decode engine takes"""
    D, ff, V, H, G, hd = 32, 48, 40, 2, 1, 16
    t = {"model.embed_tokens.weight": torch.randn(V, D), "model.norm.weight": torch.ones(D), "lm_head.weight": torch.randn(V, D)}
    p = "model.layers.0."
    t.update({p + "input_layernorm.weight": torch.ones(D), p + "post_attention_layernorm.weight": torch.ones(D),
              p + "self_attn.q_proj.weight": torch.randn(H * hd, D), p + "self_attn.k_proj.weight": torch.randn(G * hd, D),
              p + "self_attn.v_proj.weight": torch.randn(G * hd, D), p + "self_attn.o_proj.weight": torch.randn(D, H * hd),
              p + "mlp.gate_proj.weight": torch.randn(ff, D), p + "mlp.up_proj.weight": torch.randn(ff, D), p + "mlp.down_proj.weight": torch.randn(D, ff)})
    save_file({k: v.to(torch.bfloat16) for k, v in t.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(dict(architectures=["LlamaForCausalLM"], hidden_size=D, num_hidden_layers=1, num_attention_heads=H,
                                                          num_key_value_heads=G, intermediate_size=ff, vocab_size=V, rms_norm_eps=1e-6, rope_theta=5e5)))
    ck = load_model(str(tmp_path), device="cpu")
    assert ck.cfg.head_dim == hd and ck.cfg.num_kv_heads == G and ck.cfg.ffn == ff and ck.cfg.rope_theta == 5e5
    L = ck.weights["layers"][0]
    assert L["w1"].shape == (ff, D) and L["w2"].shape == (D, ff) and L["wq"].dtype == torch.bfloat16 and ck.weights["tok_embeddings"].dtype == torch.float32
    assert torch.equal(L["w3"], t[p + "mlp.up_proj.weight"].to(torch.bfloat16))


def test_config_layer_runs_and_validation():
    L = [S.gobesun_delta_layer(2, 1, 32, 16), S.gobesun_attention_layer(2, 2, 16, 16, 32, 8), S.gobesun_delta_layer(2, 2, 32, 16)]
    assert GobesunConfig.from_dict(S.gobesun_config(32, 40, L, loop=dict(start=1, stop=3, times=2))).layer_runs() == [0, 1, 2, 1, 2]
    assert GobesunConfig.from_dict(S.gobesun_config(32, 40, L, loop=dict(start=0, stop=1, times=3))).layer_runs() == [0, 0, 0, 1, 2]
    c = S.gobesun_config(32, 40, L); c.pop("loop")
    assert GobesunConfig.from_dict(c).layer_runs() == [0, 1, 2] == G.layer_order(c)
    bad = S.gobesun_config(32, 40, [dict(type="conv", mixer={}, mlp=None)])
    with pytest.raises(pkg.BackendError):
        GobesunConfig.from_dict(bad)


def test_rotary_tables_on_cpu_match_the_oracle():
    sc = dict(factor=4.0, original=2048, fast=32.0, slow=1.0)
    cos, sin = yarn_rotary_tables(32, 1e6, 300, sc, "cpu")
    wc, ws = G.rotary_angles(dict(dims=32, base=1e6, scaling=sc), torch.arange(300))
    assert float((cos - wc).abs().max()) < 1e-6 and float((sin - ws).abs().max()) < 1e-6
    cos2, _ = yarn_rotary_tables(32, 1e6, 300, None, "cpu")
    assert float((cos2[:, 0] - torch.cos(torch.arange(300.0))).abs().max()) < 1e-5        # unscaled: frequency 0 is 1 rad / position


def test_host_sampler():
    rng = np.random.default_rng(0)
    z = np.array([0.0, 5.0, 4.9, -3.0], np.float32)
    assert all(sample_host(z, SamplingParams(temperature=1.0, top_k=1), rng) == 1 for _ in range(5))
    picks = {sample_host(z, SamplingParams(temperature=1.0, top_k=2), rng) for _ in range(200)}
    assert picks == {1, 2}
    picks = {sample_host(z, SamplingParams(temperature=1.0, top_p=0.3), rng) for _ in range(50)}
    assert picks == {1}
    assert SamplingParams().greedy and not SamplingParams(temperature=0.7).greedy


def test_oracle_is_causal_and_chunked():
    """the plain restatement itself: a later token never changes earlier logits; a token in the next chunk does not see the previous one
    through attention"""
    cfg = S.gobesun_config(32, 30, [S.gobesun_attention_layer(2, 1, 16, 8, 4, 8)])
    w = S.gobesun_weights(cfg, 0)
    a = G.forward(cfg, w, [1, 2, 3, 4, 5, 6])
    b = G.forward(cfg, w, [1, 2, 3, 4, 5, 6, 7])
    assert torch.allclose(a, b[:6])
    c = G.forward(cfg, w, [9, 9, 9, 9, 5, 6])          # other tokens in chunk 0: positions 4, 5 (chunk 1) see none of them
    assert torch.allclose(a[4:], c[4:])
