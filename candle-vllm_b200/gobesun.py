"""Gobesun: a decoder whose layers mix the sequence either with a gated delta rule (recurrent, f32 state per sequence) or with
chunk-masked grouped-query attention (paged KV cache), each sublayer wrapped in an RMS norm before and after, a span of layers
optionally run several times in a row with the same weights (every pass with its own cache / state), scaled embeddings and an
untied head.  Everything size- or constant-like comes from ``config.json``:

  architecture, vocab, width, embedding.scale, norm.eps,
  layers[i] = {type: "delta" | "attention", mixer: {...}, mlp: null | {kind: "dense", ff}},
  loop = {start, stop, times}

Tensor names: embed, l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.*, l<i>.mlp.{gate, up, down}, final.norm, head.
The model object holds weights only; caches and state are allocated by the engine from ``cache_plan()`` and handed to ``forward``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ._lib import BackendError, require_device
from . import seq_ops as ops
from .mixers import GatedDeltaMixer, GatedMlp, PagedAttentionMixer
from .seq_ops import StepBatch


@dataclass
class GobesunConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: List[dict]
    loop: Optional[dict] = None
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict) -> "GobesunConfig":
        try:
            cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), embedding_scale=float(d.get("embedding", {}).get("scale", 1.0)),
                      eps=float(d["norm"]["eps"]), layers=list(d["layers"]), loop=d.get("loop") or None, raw=d)
        except KeyError as e:
            raise BackendError(f"Gobesun config lacks {e}")
        for i, L in enumerate(cfg.layers):
            if L.get("type") not in ("delta", "attention"):
                raise BackendError(f"layer {i}: unknown mixer type {L.get('type')!r}")
            if L.get("mlp") and L["mlp"].get("kind", "dense") != "dense":
                raise BackendError(f"layer {i}: unknown feed-forward kind {L['mlp'].get('kind')!r}")
        if cfg.loop:
            a, b, t = int(cfg.loop["start"]), int(cfg.loop["stop"]), int(cfg.loop["times"])
            if not (0 <= a <= b <= len(cfg.layers)) or t < 1:
                raise BackendError(f"bad loop {cfg.loop}")
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "GobesunConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def layer_runs(self) -> List[int]:
        """layer index of every layer run, in execution order"""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, t = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
        return list(range(a)) + list(range(a, b)) * t + list(range(b, n))


class _Layer:
    def __init__(self, cfg: GobesunConfig, i: int, w: Dict[str, torch.Tensor], dtype: torch.dtype, block_size: int, max_pos: int):
        L, p = cfg.layers[i], f"l{i}."
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
        m = L["mixer"]
        f32 = lambda name: w[p + name].float().contiguous()
        self.norm1, self.norm1b = f32("norm1"), f32("norm1b")
        if L["type"] == "delta":
            self.mixer = GatedDeltaMixer(sub(p + "mix."), int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"]), cfg.eps, dtype)
        else:
            mask = m.get("mask") or {}
            self.mixer = PagedAttentionMixer(sub(p + "mix."), int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]), cfg.eps,
                                             dtype, rot=m.get("rot") or None, chunk=int(mask.get("size", 0)), window=0, block_size=block_size,
                                             max_pos=max_pos)
        self.mlp = None
        if L.get("mlp"):
            self.mlp = GatedMlp(sub(p + "mlp."), dtype)
            self.norm2, self.norm2b = f32("norm2"), f32("norm2b")


class GobesunModel:
    architecture = "Gobesun"

    def __init__(self, cfg: GobesunConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16, block_size: int = 64,
                 max_pos: int = 4096, device="cuda"):
        require_device()
        if dtype not in (torch.bfloat16, torch.float32):
            raise BackendError("Gobesun runs in bfloat16 or float32")
        self.cfg, self.dtype, self.block_size, self.device = cfg, dtype, block_size, torch.device(device)
        w = {k: v.to(self.device) for k, v in weights.items()}
        self.embed = w["embed"].to(dtype).contiguous()
        self.head = w["head"].to(dtype).contiguous()
        self.final_norm = w["final.norm"].float().contiguous()
        self.layers = [_Layer(cfg, i, w, dtype, block_size, max_pos) for i in range(len(cfg.layers))]
        self.runs = cfg.layer_runs()
        # cache index of every run: its position among the runs of the same kind
        self.run_cache, nkv, nst = [], 0, 0
        for li in self.runs:
            if self.layers[li].mixer.kind == "kv":
                self.run_cache.append(("kv", nkv)); nkv += 1
            else:
                self.run_cache.append(("state", nst)); nst += 1
        self.vocab = cfg.vocab

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, **kw) -> "GobesunModel":
        from .safetensors_io import load_file
        cfg = GobesunConfig.from_json(os.path.join(path, "config.json"))
        return cls(cfg, load_file(os.path.join(path, "model.safetensors")), dtype=dtype, **kw)

    def ensure_positions(self, max_pos: int) -> bool:
        """grow the rotary tables (outside any graph capture) to cover positions below ``max_pos``; True if a table moved"""
        moved = False
        for L in self.layers:
            if L.mixer.kind == "kv" and L.mixer.rot and L.mixer.cos.shape[0] < max_pos:
                L.mixer.ensure_positions(max(2 * L.mixer.cos.shape[0], max_pos))
                moved = True
        return moved

    def cache_plan(self) -> dict:
        """What the engine allocates: one (kv heads, key size, value size) per attention run, one tuple of per-slot state shapes per
        recurrent run, in run order."""
        kv = [self.layers[li].mixer.cache_shape() for li in self.runs if self.layers[li].mixer.kind == "kv"]
        st = [self.layers[li].mixer.state_shapes() for li in self.runs if self.layers[li].mixer.kind == "state"]
        return dict(kv_layers=kv, state_layers=st)

    def forward(self, batch: StepBatch, kv_cache, state_cache, hidden_trace: Optional[list] = None) -> Optional[torch.Tensor]:
        """Runs the step's rows through every layer run, advancing caches and state; returns f32 logits [R, vocab] of the wanted rows
        (None when nothing is wanted)."""
        cfg, dt = self.cfg, self.dtype
        x = ops.embedding_scaled(self.embed, batch.tokens, cfg.embedding_scale)
        for li, (kind, ci) in zip(self.runs, self.run_cache):
            L = self.layers[li]
            h = ops.rms_norm_ex(x, L.norm1, cfg.eps, 1.0, dt)
            y = L.mixer.forward(h, batch, kv_cache[ci] if kind == "kv" else state_cache[ci])
            ops.rms_norm_ex(y, L.norm1b, cfg.eps, 1.0, torch.float32, residual=x, out=x)
            if L.mlp is not None:
                h = ops.rms_norm_ex(x, L.norm2, cfg.eps, 1.0, dt)
                y = L.mlp.forward(h)
                ops.rms_norm_ex(y, L.norm2b, cfg.eps, 1.0, torch.float32, residual=x, out=x)
            if hidden_trace is not None:
                hidden_trace.append(x.clone())
        if batch.num_want == 0:
            return None
        hn = ops.rms_norm_ex(x, self.final_norm, cfg.eps, 1.0, dt, row_index=batch.want_rows)
        return ops.linear(hn, self.head)
