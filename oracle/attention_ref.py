"""TEST INFRASTRUCTURE ONLY — CPU restatement (torch, ATen op-for-op) of the reference's attention path.

The reference is Rust on tch-rs, a 1:1 binding over ATen, so every function below issues the same
ATen operators in the same order and dtypes as the cited Rust.  It cannot be compiled here (no
cargo/rustc), and the reference holds no golden vectors for this path, so this restatement is
PARITY UNPINNED against reference outputs; it is pinned only against itself through the reference's
own equivalence tests (batched == serial, cached multi-token == serial steps) re-expressed in
``tests/``.  Reference pins libtorch 2.10.0 (Dockerfile:6); this container has torch 2.11.0.

Only ``tests/``, ``__graft_entry__.smoke`` and ``bench.py``'s CPU-baseline leg may import this module.
Citations are paths inside the reference project.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

CHUNK = 1024  # llama.rs:1032, qwen3_5.rs:1012


# --------------------------------------------------------------------------- RoPE
def rope_tables(dim: int, base: float, n_pos: int, dtype: torch.dtype):
    """sin/cos tables [n_pos, dim/2]; fp32 compute, cast to `dtype` (runtime/rope.rs:100-122)."""
    half = dim // 2
    positions = torch.arange(half, dtype=torch.float32)
    exponents = positions * 2.0 / float(dim)
    base_t = torch.full((half,), float(base), dtype=torch.float32)
    inv_freq = base_t.pow(-exponents)
    pos = torch.arange(n_pos, dtype=torch.float32)
    angles = pos.unsqueeze(-1).matmul(inv_freq.unsqueeze(0))
    return angles.sin().to(dtype), angles.cos().to(dtype)


def apply_rope(x: torch.Tensor, sin: torch.Tensor, cos: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
    """Half-split rotation in the tensor's own dtype (runtime/rope.rs:185-248).

    x: [..., seq, heads, dim]; sin/cos: tables [n_pos, dim/2]; position_ids: int64 [seq].
    Each `*`, `-`, `+` is a separate op in x.dtype (three roundings per output element in bf16).
    """
    half = x.shape[-1] // 2
    s = sin.index_select(0, position_ids).unsqueeze(1)
    c = cos.index_select(0, position_ids).unsqueeze(1)
    while s.dim() < x.dim():
        s = s.unsqueeze(0)
        c = c.unsqueeze(0)
    x1 = x.narrow(-1, 0, half)
    x2 = x.narrow(-1, half, half)
    s = s.expand_as(x1)
    c = c.expand_as(x1)
    x1r = x1 * c - x2 * s
    x2r = x1 * s + x2 * c
    return torch.cat([x1r, x2r], -1)


def apply_partial_rope(x, sin, cos, position_ids, rotary_dim: int):
    """Rotate x[..., :rotary_dim], pass the rest through (architectures/qwen3_5.rs:978-990)."""
    if rotary_dim <= 0:
        return x
    rot = apply_rope(x.narrow(-1, 0, rotary_dim), sin, cos, position_ids)
    return torch.cat([rot, x.narrow(-1, rotary_dim, x.shape[-1] - rotary_dim)], -1)


# --------------------------------------------------------------------------- Llama attention
def expand_kv_for_gqa(kv: torch.Tensor, n_heads: int) -> torch.Tensor:
    """[B,L,Hkv,D] -> [B,L,Hq,D]; q head h uses kv head h // (Hq/Hkv) (architectures/llama.rs:847-872)."""
    b, l, hkv, d = kv.shape
    rep = n_heads // hkv
    if rep == 1:
        return kv
    return kv.unsqueeze(3).expand(b, l, hkv, rep, d).reshape(b, l, n_heads, d)


def compute_attention_masked(q, k, v, attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """architectures/llama.rs:1023-1119.  q [B,q,H,D], k/v [B,L,H,D] (already GQA-expanded).

    Returns [B,H,q,D] in q.dtype.  fp32 scores, -10000 causal fill, fp32 softmax, fp32 P@V.
    """
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(float(d))
    scale = float(torch.tensor(scale, dtype=torch.float32))  # `scale` is an f32 widened to f64 (:1034,1068)
    orig = q.dtype
    qh = q.transpose(1, 2).contiguous()
    kt = k.transpose(1, 2).transpose(2, 3).contiguous()
    vh = v.transpose(1, 2).contiguous()
    if orig != torch.float32:
        qh, kt, vh = qh.float(), kt.float(), vh.float()
    if attn_mask is not None and attn_mask.dtype != torch.float32:
        attn_mask = attn_mask.float()
    q_len, k_len = qh.shape[2], kt.shape[3]
    single = attn_mask is not None or q_len <= CHUNK
    if single:
        scores = qh.matmul(kt) * scale
        if attn_mask is not None:
            scores = scores + attn_mask
        elif q_len > 1:
            mask = torch.ones(q_len, k_len, dtype=torch.float32).tril(k_len - q_len)
            mask = mask.unsqueeze(0).unsqueeze(0).expand_as(scores)
            scores = scores.masked_fill(mask.eq(0.0), -10000.0)
        out = scores.softmax(-1, dtype=torch.float32).matmul(vh)
    else:
        outs = []
        start = 0
        while start < q_len:
            cur = min(q_len - start, CHUNK)
            scores = qh.narrow(2, start, cur).matmul(kt) * scale
            mask = torch.ones(cur, k_len, dtype=torch.float32).tril(k_len - q_len + start)
            mask = mask.unsqueeze(0).unsqueeze(0).expand_as(scores)
            scores = scores.masked_fill(mask.eq(0.0), -10000.0)
            outs.append(scores.softmax(-1, dtype=torch.float32).matmul(vh))
            start += cur
        out = torch.cat(outs, 2)
    return out.to(orig) if orig != torch.float32 else out


def batched_decode_mask(start_positions: Sequence[int], q_len: int) -> torch.Tensor:
    """Additive mask [B,1,q,kv_max] with 0 / -1e9 (architectures/llama.rs:2540-2572)."""
    kv_lens = [sp + q_len for sp in start_positions]
    kv_max = max(kv_lens) if kv_lens else 0
    mask = torch.zeros(len(start_positions), 1, q_len, kv_max, dtype=torch.float32)
    cols = torch.arange(kv_max, dtype=torch.int64)
    for r, sp in enumerate(start_positions):
        for i in range(q_len):
            valid = cols.le(sp + i).logical_and(cols.lt(kv_lens[r]))
            mask[r, 0, i].copy_(valid.logical_not().to(torch.float32) * -1.0e9)
    return mask


def llama_attention_core(q, k_full, v_full, n_heads: int) -> torch.Tensor:
    """GQA expand + attention + transpose back, as LlamaAttention::forward does between the cache
    read and o_proj (architectures/llama.rs:618-650).  Returns [B, q, Hq*D]."""
    ke = expand_kv_for_gqa(k_full, n_heads)
    ve = expand_kv_for_gqa(v_full, n_heads)
    out = compute_attention_masked(q, ke, ve)
    b, h, ql, d = out.shape
    return out.transpose(1, 2).contiguous().reshape(b, ql, h * d)


def llama_batched_decode(q, row_keys, row_values, start_positions, n_heads: int) -> torch.Tensor:
    """LlamaAttention::forward_batched between the per-row cache reads and o_proj
    (architectures/llama.rs:787-832): right-pad each row's KV with zeros to kv_max, stack,
    GQA-expand, one masked attention.  q: [B, q_len, Hq, D]; row_keys[r]: [1, L_r, Hkv, D]."""
    q_len = q.shape[1]
    kv_lens = [t.shape[1] for t in row_keys]
    kv_max = max(kv_lens)

    def pad(t, length):
        if length == kv_max:
            return t
        shape = list(t.shape)
        shape[1] = kv_max - length
        return torch.cat([t, torch.zeros(shape, dtype=t.dtype)], 1)

    k_st = torch.cat([pad(t, l) for t, l in zip(row_keys, kv_lens)], 0)
    v_st = torch.cat([pad(t, l) for t, l in zip(row_values, kv_lens)], 0)
    mask = batched_decode_mask(list(start_positions), q_len)
    out = compute_attention_masked(q, expand_kv_for_gqa(k_st, n_heads), expand_kv_for_gqa(v_st, n_heads), mask)
    b, h, ql, d = out.shape
    return out.transpose(1, 2).contiguous().reshape(b, ql, h * d)


# --------------------------------------------------------------------------- Qwen3.5 gated full attention
def qk_norm(x: torch.Tensor, weight_f32: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head RMS norm with (1 + w), fp32 inside (architectures/qwen3_5.rs:1077-1091)."""
    shape = x.shape
    flat = x.reshape(-1, shape[-1])
    f = flat.float()
    mean_sq = (f * f).mean(dim=-1, keepdim=True, dtype=torch.float32)
    rrms = (mean_sq + float(eps)).rsqrt()
    normed = f * rrms
    return (normed * (weight_f32.reshape(1, -1) + 1.0)).to(x.dtype).reshape(shape)


def qwen_gated_attention_core(query, gate, k_full, v_full, n_heads: int) -> torch.Tensor:
    """Qwen3_5FullAttention::forward between the cache read and o_proj
    (architectures/qwen3_5.rs:999-1059).  query, gate: [B,q,Hq,D]; k_full, v_full: [B,L,Hkv,D].

    fp32 scores and softmax; P cast to the model dtype, P@V in the model dtype; times sigmoid(gate).
    Returns [B*q, Hq*D]."""
    dtype = query.dtype
    b, ql, nh, hd = query.shape
    groups = nh // k_full.shape[2]
    k_exp = k_full.repeat_interleave(groups, dim=2)
    v_exp = v_full.repeat_interleave(groups, dim=2)
    scale = 1.0 / math.sqrt(float(hd))
    q_p = query.permute(0, 2, 1, 3).float().contiguous()
    k_p = k_exp.permute(0, 2, 3, 1).float().contiguous()
    v_p = v_exp.permute(0, 2, 1, 3).float().contiguous()
    kv_len = k_p.shape[3]
    if ql <= CHUNK:
        scores = q_p.matmul(k_p) * scale
        if ql > 1:
            mask = torch.ones(ql, kv_len, dtype=torch.float32).tril(kv_len - ql)
            mask = mask.unsqueeze(0).unsqueeze(0).expand_as(scores)
            scores = scores.masked_fill(mask.eq(0.0), -10000.0)
        attn = scores.softmax(-1, dtype=torch.float32).to(dtype)
        ctx = attn.matmul(v_p.to(dtype))
    else:
        v_d = v_p.to(dtype)
        outs = []
        start = 0
        while start < ql:
            cur = min(ql - start, CHUNK)
            scores = q_p.narrow(2, start, cur).matmul(k_p) * scale
            mask = torch.ones(cur, kv_len, dtype=torch.float32).tril(kv_len - ql + start)
            mask = mask.unsqueeze(0).unsqueeze(0).expand_as(scores)
            scores = scores.masked_fill(mask.eq(0.0), -10000.0)
            outs.append(scores.softmax(-1, dtype=torch.float32).to(dtype).matmul(v_d))
            start += cur
        ctx = torch.cat(outs, 2)
    ctx = ctx.permute(0, 2, 1, 3).contiguous()
    ctx_flat = ctx.reshape(b * ql, nh * hd)
    gate_flat = gate.reshape(b * ql, nh * hd).sigmoid()
    return ctx_flat * gate_flat


# --------------------------------------------------------------------------- fp32 recomputation
def attention_fp32(q, k, v, causal_offset: Optional[int] = None, kv_lens: Optional[Sequence[int]] = None):
    """The tolerance anchor named by the acceptance rule: exact-softmax attention in fp32.

    q [B,ql,Hq,D], k/v [B,L,Hkv,D] (any dtype, widened to fp32); query row i may see keys
    j <= causal_offset + i (default L - ql) and j < kv_lens[b].  Returns fp32 [B,ql,Hq,D]."""
    b, ql, hq, d = q.shape
    l, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().repeat_interleave(g, dim=2).permute(0, 2, 1, 3)
    vf = v.float().repeat_interleave(g, dim=2).permute(0, 2, 1, 3)
    out = torch.empty(b, hq, ql, d, dtype=torch.float32)
    off = (l - ql) if causal_offset is None else causal_offset
    cols = torch.arange(l)
    for bi in range(b):
        lim = l if kv_lens is None else int(kv_lens[bi])
        for start in range(0, ql, CHUNK):
            cur = min(CHUNK, ql - start)
            s = qf[bi, :, start:start + cur].matmul(kf[bi].transpose(-1, -2)) / math.sqrt(d)
            rows = torch.arange(start, start + cur).unsqueeze(-1)
            bad = (cols.unsqueeze(0) > rows + off) | (cols.unsqueeze(0) >= lim)
            s = s.masked_fill(bad.unsqueeze(0), float("-inf"))
            out[bi, :, start:start + cur] = s.softmax(-1).matmul(vf[bi])
    return out.permute(0, 2, 1, 3).contiguous()
