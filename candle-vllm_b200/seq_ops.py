"""Operator wrappers for ragged-step models: the C entry points that serve portions of prompts beside single decoded tokens in one
launch (include/b200_backend.h: linear_f32out ... paged_attention_varlen).  Same conventions as ``backend.py``: torch tensors are
device memory and stream plumbing only, every op is one hand-written kernel launch on the current stream, errors raise
``BackendError``; nothing here allocates on the host or synchronises, so a step can be captured into a CUDA graph.

``StepBatch`` is the device-side description of one step that ``inputs.prepare_step`` builds on the host.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ._lib import BackendError, check, lib
from .backend import DType, _ptr, _stream

_B200 = {torch.float32: DType.F32, torch.bfloat16: DType.BF16}


def _tag(dt: torch.dtype) -> int:
    try:
        return _B200[dt]
    except KeyError:
        raise BackendError(f"ragged-step ops take f32 / bf16, not {dt}")


@dataclass
class StepBatch:
    """One step on the device (all i32 unless said): T rows, B entries, R wanted rows."""
    tokens: torch.Tensor          # [T]
    positions: torch.Tensor       # [T] position of each row in its sequence
    token_seq: torch.Tensor       # [T] entry that owns the row
    slot_mapping: torch.Tensor    # [T] i64, flat cache slot = block * block_size + offset
    cu_seqlens: torch.Tensor      # [B + 1] rows
    cu_seqlens_k: torch.Tensor    # [B + 1] context lengths (start + rows), cumulative
    seq_slots: torch.Tensor       # [B] state slot of each entry's sequence
    seq_start: torch.Tensor       # [B] position of each entry's first row (0 = new sequence)
    block_tables: torch.Tensor    # [B, W]
    want_rows: torch.Tensor       # [R] rows whose logits are returned
    num_tokens: int = 0
    num_seqs: int = 0
    num_want: int = 0
    max_position: int = 0
    pure_decode: bool = False     # every entry brings exactly one token
    max_rows: int = 1             # the most rows any entry brings

    @classmethod
    def from_host(cls, prep: dict, device="cuda") -> "StepBatch":
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dt)).to(device, non_blocking=True)
        return cls(tokens=t(prep["tokens"], np.int32), positions=t(prep["positions"], np.int32), token_seq=t(prep["token_seq"], np.int32),
                   slot_mapping=t(prep["slot_mapping"], np.int64), cu_seqlens=t(prep["cu_seqlens"], np.int32), cu_seqlens_k=t(prep["cu_seqlens_k"], np.int32),
                   seq_slots=t(prep["seq_slots"], np.int32), seq_start=t(prep["seq_start"], np.int32),
                   block_tables=t(prep["block_tables"], np.int32), want_rows=t(prep["want_rows"], np.int32),
                   num_tokens=len(prep["tokens"]), num_seqs=len(prep["seq_slots"]), num_want=len(prep["want_rows"]),
                   max_position=int(prep["max_position"]), pure_decode=len(prep["tokens"]) == len(prep["seq_slots"]),
                   max_rows=int(np.diff(np.asarray(prep["cu_seqlens"], np.int64)).max()) if len(prep["seq_slots"]) else 1)


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [m, k] (rows may be strided) . weight [n, k]^T -> f32 [m, n]; both operands f32 (true 32-bit product) or both bf16."""
    if x.dtype != weight.dtype or x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1 or not weight.is_contiguous():
        raise BackendError(f"linear: x {tuple(x.shape)} {x.dtype} vs weight {tuple(weight.shape)} {weight.dtype}")
    m, k = x.shape
    n = weight.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    lib().linear_f32out(_ptr(x), _ptr(weight), _ptr(out), C.c_int32(m), C.c_int32(n), C.c_int32(k), C.c_int64(x.stride(0) if m > 1 else max(k, x.stride(0))),
                        C.c_int64(out.stride(0) if m > 1 else max(n, out.stride(0))), C.c_int32(_tag(x.dtype)), _stream(x.device))
    check("linear")
    return out


def rms_norm_ex(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float, out_dtype: torch.dtype, residual: Optional[torch.Tensor] = None,
                row_index: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS norm of f32 rows times (offset + weight); with ``residual`` the result is added to it (pass out=residual for in place);
    ``row_index`` (i32) selects the rows to normalise."""
    n = x.shape[-1]
    rows = x.shape[0] if row_index is None else row_index.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or x.stride(-1) != 1:
        raise BackendError("rms_norm_ex: x and weight are f32")
    if out is None:
        out = torch.empty((rows, n), dtype=out_dtype, device=x.device)
    lib().rms_norm_ex(_ptr(x), _ptr(weight), _ptr(out), _ptr(residual), _ptr(row_index), C.c_int32(rows), C.c_int32(n), C.c_int64(x.stride(0) if x.shape[0] > 1 else n),
                      C.c_float(eps), C.c_float(offset), C.c_int32(_tag(out.dtype)), _stream(x.device))
    check("rms_norm_ex")
    return out


def gelu_tanh_mul(gate_up: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    rows, two_ff = gate_up.shape
    ff = two_ff // 2
    out = torch.empty((rows, ff), dtype=out_dtype, device=gate_up.device)
    lib().gelu_tanh_mul(_ptr(gate_up), _ptr(out), C.c_int64(rows), C.c_int32(ff), C.c_int64(gate_up.stride(0) if rows > 1 else two_ff),
                        C.c_int32(_tag(out_dtype)), _stream(gate_up.device))
    check("gelu_tanh_mul")
    return out


def embedding_scaled(table: torch.Tensor, ids: torch.Tensor, scale: float) -> torch.Tensor:
    vocab, dim = table.shape
    out = torch.empty((ids.shape[0], dim), dtype=torch.float32, device=table.device)
    lib().embedding_scaled(_ptr(table), _ptr(ids), _ptr(out), C.c_int32(ids.shape[0]), C.c_int32(dim), C.c_int32(vocab), C.c_float(scale),
                           C.c_int32(_tag(table.dtype)), _stream(table.device))
    check("embedding_scaled")
    return out


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor, conv_state: torch.Tensor, batch: StepBatch) -> torch.Tensor:
    """x: f32 view [T, C] of the fused projection (row stride allowed); taps f32 [C, K]; conv_state f32 [slots, K-1, C], advanced in place."""
    T, Cn = x.shape
    K = taps.shape[1]
    if T > 65535:
        raise BackendError("causal_conv_silu: at most 65535 rows per step")
    y = torch.empty((T, Cn), dtype=torch.float32, device=x.device)
    lib().causal_conv_silu(_ptr(x), C.c_int64(x.stride(0) if T > 1 else max(Cn, x.stride(0))), _ptr(taps), _ptr(conv_state), _ptr(y), _ptr(batch.token_seq),
                           _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(T), C.c_int32(batch.num_seqs), C.c_int32(Cn),
                           C.c_int32(K), _stream(x.device))
    check("causal_conv_silu")
    return y


TILED_DELTA_MIN_ROWS = 8      # steps in which some entry brings at least this many rows take the tiled form of the rule


def gated_delta_rule(qkv: torch.Tensor, proj: torch.Tensor, off_b: int, off_a: int, A_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor,
                     batch: StepBatch, heads: int, kv_heads: int, dk: int, dv: int, kernel: Optional[str] = None) -> torch.Tensor:
    """qkv f32 [T, G dk | G dk | H dv]; b / a read from columns off_b.. / off_a.. of ``proj``; state f32 [slots, H, dv, dk] advanced in place.
    Three kernels compute the same rule: "step" (every entry brings one token: one pass over the state, nothing staged), "tiled" (over
    tiles of 16 tokens, for portions of prompts; key sizes up to 128) and "token" (token by token, any step).  ``kernel`` forces one;
    None chooses by the step's shape."""
    T = qkv.shape[0]
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=qkv.device)
    ld_proj = C.c_int64(proj.stride(0) if T > 1 else proj.shape[1])
    if kernel is None:
        kernel = "step" if batch.pure_decode else "tiled" if (dk <= 128 and batch.max_rows >= TILED_DELTA_MIN_ROWS) else "token"
    if kernel == "step":
        if T != batch.num_seqs:
            raise BackendError("gated_delta_rule: the single-token kernel takes one row per entry")
        lib().gated_delta_rule_step(_ptr(qkv), _ptr(proj), ld_proj, C.c_int32(off_b), C.c_int32(off_a), _ptr(A_log), _ptr(dt_bias), _ptr(state), _ptr(out),
                                    _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(batch.num_seqs), C.c_int32(heads), C.c_int32(kv_heads),
                                    C.c_int32(dk), C.c_int32(dv), _stream(qkv.device))
        check("gated_delta_rule_step")
    elif kernel == "tiled":
        scratch = torch.empty((T * (2 * kv_heads * dk + 35 * heads),), dtype=torch.float32, device=qkv.device)
        lib().gated_delta_rule_tiled(_ptr(qkv), _ptr(proj), ld_proj, C.c_int32(off_b), C.c_int32(off_a), _ptr(A_log), _ptr(dt_bias), _ptr(state), _ptr(out),
                                     _ptr(scratch), _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start), C.c_int32(T),
                                     C.c_int32(batch.num_seqs), C.c_int32(batch.max_rows), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk),
                                     C.c_int32(dv), _stream(qkv.device))
        check("gated_delta_rule_tiled")
    elif kernel == "token":
        lib().gated_delta_rule(_ptr(qkv), _ptr(proj), ld_proj, C.c_int32(off_b), C.c_int32(off_a), _ptr(A_log),
                               _ptr(dt_bias), _ptr(state), _ptr(out), _ptr(batch.cu_seqlens), _ptr(batch.seq_slots), _ptr(batch.seq_start),
                               C.c_int32(batch.num_seqs), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk), C.c_int32(dv), _stream(qkv.device))
        check("gated_delta_rule")
    else:
        raise BackendError(f"gated_delta_rule: unknown kernel {kernel!r}")
    return out


def gated_rms_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, heads: int, dv: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    T = o.shape[0]
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=o.device)
    lib().gated_rms_norm(_ptr(o), _ptr(gate), C.c_int64(gate.stride(0) if T > 1 else max(heads * dv, gate.stride(0))), _ptr(weight), _ptr(out), C.c_int32(T),
                         C.c_int32(heads), C.c_int32(dv), C.c_float(eps), C.c_int32(_tag(out_dtype)), _stream(o.device))
    check("gated_rms_norm")
    return out


def qk_norm_rope_cache(qkv: torch.Tensor, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                       sin: Optional[torch.Tensor], batch: StepBatch, k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int, kv_heads: int, dk: int,
                       dv: int, rot_dims: int, eps: float, q_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    T = qkv.shape[0]
    if cos is not None and batch.max_position >= cos.shape[0]:
        raise BackendError(f"position {batch.max_position} is outside the rotary table ({cos.shape[0]} rows)")
    q = torch.empty((T, heads * dk), dtype=q_dtype, device=qkv.device)
    lib().qk_norm_rope_cache(_ptr(qkv), C.c_int64(qkv.stride(0) if T > 1 else qkv.shape[1]), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin),
                             C.c_int32(0 if cos is None else cos.shape[0]), _ptr(batch.positions), _ptr(batch.slot_mapping), _ptr(q), _ptr(k_cache),
                             _ptr(v_cache), C.c_int32(T), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk), C.c_int32(dv), C.c_int32(rot_dims),
                             C.c_float(eps), C.c_int32(_tag(k_cache.dtype)), C.c_int32(_tag(q_dtype)), _stream(qkv.device))
    check("qk_norm_rope_cache")
    return q


def paged_attention_varlen(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: StepBatch, heads: int, kv_heads: int, dk: int, dv: int,
                           block_size: int, scale: float, chunk: int, window: int, out_dtype: torch.dtype) -> torch.Tensor:
    T = q.shape[0]
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=q.device)
    lib().paged_attention_varlen(_ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(batch.block_tables), C.c_int32(batch.block_tables.shape[1]),
                                 _ptr(batch.token_seq), _ptr(batch.positions), _ptr(batch.cu_seqlens), _ptr(batch.cu_seqlens_k), C.c_int32(batch.num_seqs),
                                 C.c_int32(T), C.c_int32(heads), C.c_int32(kv_heads), C.c_int32(dk), C.c_int32(dv), C.c_int32(block_size), C.c_float(scale),
                                 C.c_int32(chunk), C.c_int32(window), C.c_int32(_tag(q.dtype)), C.c_int32(_tag(k_cache.dtype)), C.c_int32(_tag(out_dtype)),
                                 _stream(q.device))
    check("paged_attention_varlen")
    return out


def paged_attention_decode_chunked(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: StepBatch, heads: int, kv_heads: int, hd: int,
                                   block_size: int, scale: float, chunk: int, scratch: dict) -> torch.Tensor:
    """A step of single tokens under a chunk mask with chunk % block_size == 0, on the split-KV decode kernel of ``PagedAttention``: the
    block tables are viewed from each sequence's chunk start (``chunk_decode_view``).  q bf16 [B, H * hd]; ``scratch`` keeps the view
    and the kernel's workspace between calls (allocated on first use, so call once before capturing a graph)."""
    B = q.shape[0]
    width = chunk // block_size
    key = (B, width)
    if key not in scratch:
        need = lib().paged_attention_decode_workspace_bytes(C.c_int32(B), C.c_int32(heads), C.c_int32(hd), C.c_int32(width), C.c_int32(block_size))
        scratch[key] = (torch.zeros((B, width), dtype=torch.int32, device=q.device), torch.zeros(B, dtype=torch.int32, device=q.device),
                        torch.zeros(int(need), dtype=torch.uint8, device=q.device))
    tables, ctx, ws = scratch[key]
    out = torch.empty((B, heads * hd), dtype=q.dtype, device=q.device)
    L = lib()
    L.chunk_decode_view(_ptr(batch.block_tables), C.c_int32(batch.block_tables.shape[1]), _ptr(batch.positions), _ptr(tables), _ptr(ctx), C.c_int32(B),
                        C.c_int32(width), C.c_int32(block_size), C.c_int32(chunk), _stream(q.device))
    L.paged_attention_decode(_ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(tables), _ptr(ctx), C.c_int32(B), C.c_int32(heads), C.c_int32(kv_heads),
                             C.c_int32(hd), C.c_int32(block_size), C.c_int32(width), C.c_int64(k_cache.shape[0]), C.c_float(scale), C.c_float(0.0),
                             C.c_int32(0), C.c_int32(_tag(q.dtype)), C.c_int32(_tag(k_cache.dtype)), C.c_int32(0), C.c_int32(_tag(q.dtype)), _ptr(ws),
                             C.c_size_t(ws.numel()), _stream(q.device))
    check("paged_attention_decode_chunked")
    return out
