"""Guvusun: a decoder with "norm after the sum" layers (x <- norm(alpha x + sublayer(x))), latent attention (a low-rank latent and one shared
rotated key part are all the cache holds; softmax with a per-head sink; sigmoid head gates; a layer may attend over an earlier layer's cache),
a routed mixture of experts as feed-forward (group-limited top-k, choice-only correction, identity experts), a hashed bigram embedding
added to the token embedding, and a per-layer token embedding gated by the stream after every feed-forward.  Everything size- or
constant-like comes from ``config.json``:

  architecture, vocab, width, norm.eps, postln_alpha, embedding.bigram = {buckets, mul_prev, mul_cur}, token_side = {dim},
  layers[i] = {type: "latent_attention", mixer: {heads, dim, rot_dim, vdim, kv_rank, scale, rot: {base, dims, scaling}, kv_from},
               mlp: null | {kind: "moe", expert: {ff}, router: {experts, identity, top, scale, groups: {count, keep}}}}

Tensor names: embed, bigram, embed.norm, side.embed, l<i>.norm1 / norm2, l<i>.mix.{q, dkv, dkv.norm, uk, uv, sink, g, o},
l<i>.mlp.{router, correction, e<j>.gate / up / down}, l<i>.side.{gate, proj, norm}, final.norm, head.
The model object holds weights only; the latent cache and the previous-token state are allocated by the engine from ``cache_plan()``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ._lib import BackendError, require_device
from . import seq_ops as ops
from .mixers import LatentAttentionMixer, RoutedExperts, TokenSideInput
from .seq_ops import StepBatch


@dataclass
class GuvusunConfig:
    vocab: int
    width: int
    eps: float
    alpha: float
    layers: List[dict]
    bigram: Optional[dict] = None
    side_dim: int = 0
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict) -> "GuvusunConfig":
        try:
            cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]), alpha=float(d.get("postln_alpha", 1.0)),
                      layers=list(d["layers"]), bigram=(d.get("embedding") or {}).get("bigram") or None,
                      side_dim=int((d.get("token_side") or {}).get("dim", 0)), raw=d)
            for i, L in enumerate(cfg.layers):
                if L.get("type") != "latent_attention":
                    raise BackendError(f"layer {i}: unknown mixer type {L.get('type')!r}")
                m = L["mixer"]
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"):
                    m[key]
                rot = m.get("rot")
                if rot and int(rot.get("dims", m["rot_dim"])) != int(m["rot_dim"]):
                    raise BackendError(f"layer {i}: the rotation spans {rot['dims']} entries, the rotated part has {m['rot_dim']}")
                src = m.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not 0 <= src < i or cfg.layers[src]["mixer"].get("kv_from") is not None:
                        raise BackendError(f"layer {i}: kv_from {src} must name an earlier layer with a cache of its own")
                    sm = cfg.layers[src]["mixer"]
                    if (int(sm["kv_rank"]), int(sm["rot_dim"])) != (int(m["kv_rank"]), int(m["rot_dim"])) or sm.get("rot") != m.get("rot"):
                        raise BackendError(f"layer {i}: latent size, rotated size and rotation must equal those of layer {src}")
                mlp = L.get("mlp")
                if mlp:
                    if mlp.get("kind") != "moe":
                        raise BackendError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
                    mlp["router"]["experts"], mlp["router"]["top"]
            if cfg.bigram:
                for key in ("buckets", "mul_prev", "mul_cur"):
                    cfg.bigram[key]
        except KeyError as e:
            raise BackendError(f"Guvusun config lacks {e}")
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "GuvusunConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))


class _Layer:
    def __init__(self, cfg: GuvusunConfig, i: int, w: Dict[str, torch.Tensor], side_table, dtype: torch.dtype, block_size: int, max_pos: int):
        L, p = cfg.layers[i], f"l{i}."
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
        m = L["mixer"]
        self.kv_from = None if m.get("kv_from") is None else int(m["kv_from"])
        self.norm1 = w[p + "norm1"].float().contiguous()
        self.mixer = LatentAttentionMixer(sub(p + "mix."), int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]), float(m["scale"]),
                                          cfg.eps, dtype, rot=m.get("rot") or None, shared=self.kv_from is not None, block_size=block_size, max_pos=max_pos)
        self.mlp = None
        self.norm2 = w[p + "norm2"].float().contiguous() if p + "norm2" in w else None
        if L.get("mlp"):
            r = L["mlp"]["router"]
            g = r.get("groups") or {}
            self.mlp = RoutedExperts(sub(p + "mlp."), int(r["experts"]), int(r.get("identity", 0)), int(r["top"]), float(r.get("scale", 1.0)), dtype,
                                     groups=int(g.get("count", 0)), keep=int(g.get("keep", 0)))
            if self.mlp.E and self.mlp.ff != int(L["mlp"]["expert"]["ff"]):
                raise BackendError(f"layer {i}: expert tensors have ff {self.mlp.ff}, the config says {L['mlp']['expert']['ff']}")
            if self.norm2 is None:
                raise BackendError(f"layer {i}: a feed-forward without norm2")
        self.side = TokenSideInput(sub(p + "side."), side_table, i * cfg.side_dim, cfg.side_dim, cfg.eps, dtype) if cfg.side_dim else None


class GuvusunModel:
    architecture = "Guvusun"

    def __init__(self, cfg: GuvusunConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16, block_size: int = 64,
                 max_pos: int = 4096, device="cuda"):
        require_device()
        if dtype not in (torch.bfloat16, torch.float32):
            raise BackendError("Guvusun runs in bfloat16 or float32")
        self.cfg, self.dtype, self.block_size, self.device = cfg, dtype, block_size, torch.device(device)
        w = {k: v.to(self.device) for k, v in weights.items()}
        self.embed = w["embed"].to(dtype).contiguous()
        self.bigram = w["bigram"].to(dtype).contiguous() if cfg.bigram else None
        self.embed_norm = w["embed.norm"].float().contiguous()
        self.head = w["head"].to(dtype).contiguous()
        self.final_norm = w["final.norm"].float().contiguous()
        side_table = w["side.embed"].to(dtype).contiguous() if cfg.side_dim else None
        if side_table is not None and side_table.shape[1] != len(cfg.layers) * cfg.side_dim:
            raise BackendError(f"side.embed has {side_table.shape[1]} columns, expected {len(cfg.layers)} x {cfg.side_dim}")
        self.layers = [_Layer(cfg, i, w, side_table, dtype, block_size, max_pos) for i in range(len(cfg.layers))]
        # cache index of every layer: layers with a latent projection of their own get a cache in layer order, the others use their source's
        self.layer_cache, n = [], 0
        for L in self.layers:
            if L.kv_from is None:
                self.layer_cache.append(n); n += 1
            else:
                self.layer_cache.append(self.layer_cache[L.kv_from])
        self.vocab = cfg.vocab

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, **kw) -> "GuvusunModel":
        from .safetensors_io import load_file
        cfg = GuvusunConfig.from_json(os.path.join(path, "config.json"))
        return cls(cfg, load_file(os.path.join(path, "model.safetensors")), dtype=dtype, **kw)

    def ensure_positions(self, max_pos: int) -> bool:
        """grow the rotary tables (outside any graph capture) to cover positions below ``max_pos``; True if a table moved"""
        moved = False
        for L in self.layers:
            if L.mixer.cos is not None and L.mixer.cos.shape[0] < max_pos:
                L.mixer.ensure_positions(max(2 * L.mixer.cos.shape[0], max_pos))
                moved = True
        return moved

    def cache_plan(self) -> dict:
        """What the engine allocates: one (1, latent size, rotated size) per layer that writes a latent cache, and one i32 per state slot for the
        sequence's last token (what the bigram hash of the next step's first row needs)."""
        kv = [L.mixer.cache_shape() for L in self.layers if L.kv_from is None]
        return dict(kv_layers=kv, state_layers=[(((1,), torch.int32),)] if self.bigram is not None else [])

    def forward(self, batch: StepBatch, kv_cache, state_cache, hidden_trace: Optional[list] = None) -> Optional[torch.Tensor]:
        """Runs the step's rows through every layer, advancing the caches and the previous-token state; returns f32 logits [R, vocab] of the wanted
        rows (None when nothing is wanted)."""
        cfg, dt = self.cfg, self.dtype
        bg = cfg.bigram or {}
        x = ops.embedding_bigram(self.embed, self.bigram, batch, state_cache[0][0] if self.bigram is not None else None, int(bg.get("buckets", 0)),
                                 int(bg.get("mul_prev", 0)), int(bg.get("mul_cur", 0)))
        x16 = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if dt == torch.bfloat16 else None
        h = x if x16 is None else x16                      # what the sublayers read: the stream itself, in the compute dtype
        ops.residual_rms_norm(x, None, self.embed_norm, 1.0, cfg.eps, True, x16)
        for L, ci in zip(self.layers, self.layer_cache):
            y = L.mixer.forward(h, batch, kv_cache[ci])
            ops.residual_rms_norm(x, y, L.norm1, cfg.alpha, cfg.eps, True, x16)
            if L.norm2 is not None:
                y = L.mlp.forward(h, x) if L.mlp is not None else None
                ops.residual_rms_norm(x, y, L.norm2, cfg.alpha, cfg.eps, True, x16)
            if L.side is not None:
                L.side.forward(x, h, batch, x16)
            if hidden_trace is not None:
                hidden_trace.append(x.clone())
        if batch.num_want == 0:
            return None
        hn = ops.rms_norm_ex(x, self.final_norm, cfg.eps, 0.0, dt, row_index=batch.want_rows)
        return ops.linear(hn, self.head)
