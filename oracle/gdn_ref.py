"""TEST INFRASTRUCTURE ONLY — CPU restatement (torch, ATen op-for-op) of the reference's gated-DeltaNet core.

Follows architectures/qwen3_5.rs: l2_normalize (:331-335), chunked_delta_rule (:342-498), the
recurrent decode step (:725-751), the gate arithmetic (:681-701) and RMSNormGated (:305-313).
PARITY UNPINNED against reference outputs (the Rust cannot be built here and the reference holds
no fixture for this path); the restatement is cross-checked in tests against the independent
implementations shipped in `transformers` (models/qwen3_5/modeling_qwen3_5.py), which the
reference names as the function it translated (qwen3_5.rs:337).

Only ``tests/``, ``__graft_entry__.smoke`` and ``bench.py``'s CPU-baseline leg may import this module.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

CHUNK_SIZE = 64  # qwen3_5.rs:351


def l2_normalize(x: torch.Tensor) -> torch.Tensor:
    """x / max(||x||_2, 1e-3) over the last dim (qwen3_5.rs:331-335)."""
    norm = x.norm(p=2.0, dim=-1, keepdim=True)
    return x / norm.clamp_min(1e-3)


def gdn_gates(a_in: torch.Tensor, b_in: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor):
    """g = -exp(A_log) * softplus(a + dt_bias) (fp32), beta = sigmoid(b) (qwen3_5.rs:687-701)."""
    g = (-a_log.float().exp()) * torch.nn.functional.softplus(a_in.float() + dt_bias.float())
    beta = b_in.float().sigmoid()
    return g, beta


def rmsnorm_gated(x: torch.Tensor, gate: torch.Tensor, weight_f32: torch.Tensor, eps: float) -> torch.Tensor:
    """norm(x) * w * silu(gate), fp32 inside, cast to x.dtype (qwen3_5.rs:305-313)."""
    orig = x.dtype
    xf = x.float()
    mean_sq = (xf * xf).mean(dim=-1, keepdim=True, dtype=torch.float32)
    rrms = (mean_sq + float(eps)).rsqrt()
    normed = xf * rrms
    g = torch.nn.functional.silu(gate.float())
    return (normed * weight_f32 * g).to(orig)


def gdn_prologue(mixed_qkv: torch.Tensor, conv_weight: torch.Tensor, conv_state: Optional[torch.Tensor], a_in: torch.Tensor,
                 b_in: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, n_k_heads: int, head_k_dim: int,
                 n_v_heads: int, head_v_dim: int):
    """GatedDeltaNetLayer::forward between the input projection and the delta rule (qwen3_5.rs:627-701), same ATen
    operators in the same order and dtypes: depthwise causal conv1d (kernel ks, left context = conv_state or zeros) in
    the model dtype, SiLU, split into q | k | v, q and k to fp32 and L2-normalised, q * 1/sqrt(head_k_dim), v to fp32,
    g and beta in fp32.

    mixed_qkv [B,T,conv_dim] and conv_weight [conv_dim,1,ks] in the model dtype; conv_state [B,conv_dim,ks-1] or None.
    Returns (q [B,T,nk,hk], k, v [B,T,nv,hv], g [B,T,nv], beta [B,T,nv], new_conv_state [B,conv_dim,ks-1]).

    The reference keeps fewer than ks-1 frames after a first call shorter than ks-1 tokens (:650-651) and then cannot
    run the next call; here the state always has ks-1 frames (zeros in front), which is the same wherever the
    reference runs."""
    bsz, seq, conv_dim = mixed_qkv.shape
    ks = conv_weight.shape[-1]
    x_t = mixed_qkv.permute(0, 2, 1)
    if conv_state is None:
        conv_state = torch.zeros(bsz, conv_dim, ks - 1, dtype=mixed_qkv.dtype)
    padded = torch.cat([conv_state, x_t], dim=2)
    new_state = padded.narrow(2, padded.shape[2] - (ks - 1), ks - 1).contiguous()
    conv_out = torch.nn.functional.conv1d(padded, conv_weight, None, stride=1, padding=0, dilation=1, groups=conv_dim)
    conv_out = torch.nn.functional.silu(conv_out).permute(0, 2, 1)
    key_dim, val_dim = n_k_heads * head_k_dim, n_v_heads * head_v_dim
    q = conv_out.narrow(2, 0, key_dim).reshape(bsz, seq, n_k_heads, head_k_dim)
    k = conv_out.narrow(2, key_dim, key_dim).reshape(bsz, seq, n_k_heads, head_k_dim)
    v = conv_out.narrow(2, 2 * key_dim, val_dim).reshape(bsz, seq, n_v_heads, head_v_dim)
    q = l2_normalize(q.float()) * (1.0 / float(head_k_dim) ** 0.5)
    k = l2_normalize(k.float())
    g, beta = gdn_gates(a_in, b_in, a_log, dt_bias)
    return q, k, v.float(), g, beta, new_state


def recurrent_step(q_t, k_t, v_t, g_t, b_t, state) -> Tuple[torch.Tensor, torch.Tensor]:
    """One decode step (qwen3_5.rs:725-751).

    q_t,k_t [B,nv,hk] (already L2-normalised, q scaled, heads expanded), v_t [B,nv,hv],
    g_t,b_t [B,nv], state [B,nv,hk,hv] fp32.  Returns (out [B,nv,hv], new state)."""
    batch, nv, hk = k_t.shape
    hv = v_t.shape[-1]
    decay = g_t.exp().reshape(batch, nv, 1, 1)
    state = state * decay
    kv_mem = k_t.reshape(batch * nv, 1, hk).bmm(state.reshape(batch * nv, hk, hv)).reshape(batch, nv, hv)
    delta = (v_t - kv_mem) * b_t.unsqueeze(-1)
    state = state.reshape(batch, nv, hk, hv) + k_t.unsqueeze(-1) * delta.unsqueeze(-2)
    out = q_t.reshape(batch * nv, 1, hk).bmm(state.reshape(batch * nv, hk, hv)).reshape(batch, nv, hv)
    return out, state


def recurrent_sequence(q, k, v, g, beta, initial_state: Optional[torch.Tensor] = None):
    """The same recurrence applied token by token over [B,nv,T,*] inputs (reference for chunked)."""
    b, nv, t, hk = q.shape
    hv = v.shape[-1]
    state = initial_state.float().clone() if initial_state is not None else torch.zeros(b, nv, hk, hv)
    outs = []
    for i in range(t):
        o, state = recurrent_step(q[:, :, i], k[:, :, i], v[:, :, i], g[:, :, i], beta[:, :, i], state)
        outs.append(o)
    return torch.stack(outs, 2), state


def chunked_delta_rule(q, k, v, g, beta, initial_state: Optional[torch.Tensor] = None):
    """Chunked prefill (qwen3_5.rs:342-498).  q,k [B,nv,T,hk], v [B,nv,T,hv], g,beta [B,nv,T], all fp32.

    Returns (out [B,nv,T,hv], final state [B,nv,hk,hv])."""
    c = CHUNK_SIZE
    batch, nv, seq, hk = q.shape
    hv = v.shape[3]
    pad = (c - seq % c) % c
    seq_p = seq + pad

    def padded(t, extra):
        if pad == 0:
            return t
        shape = (batch, nv, pad) if extra == 0 else (batch, nv, pad, extra)
        return torch.cat([t, torch.zeros(shape, dtype=torch.float32)], 2)

    q, k, v, g, beta = padded(q, hk), padded(k, hk), padded(v, hv), padded(g, 0), padded(beta, 0)
    v_beta = v * beta.unsqueeze(-1)
    k_beta = k * beta.unsqueeze(-1)
    nc = seq_p // c
    q = q.reshape(batch, nv, nc, c, hk)
    k = k.reshape(batch, nv, nc, c, hk)
    v = v.reshape(batch, nv, nc, c, hv)
    k_beta = k_beta.reshape(batch, nv, nc, c, hk)
    v_beta = v_beta.reshape(batch, nv, nc, c, hv)
    g = g.reshape(batch, nv, nc, c).cumsum(-1, dtype=torch.float32)
    decay_mask = (g.unsqueeze(-1) - g.unsqueeze(-2)).exp().tril(0)   # exp first, then tril (:396-400)
    mask0 = torch.ones(c, c, dtype=torch.bool).triu(0)
    mask1 = torch.ones(c, c, dtype=torch.bool).triu(1)
    attn0 = -(k_beta.matmul(k.transpose(-1, -2)) * decay_mask).masked_fill(mask0, 0.0)
    rows = [attn0.narrow(-2, 0, 1).squeeze(-2)]
    for i in range(1, c):                                            # forward substitution (:423-442)
        a_row = attn0.narrow(-2, i, 1).narrow(-1, 0, i).squeeze(-2)
        sub = torch.stack(rows, -2).narrow(-1, 0, i)
        correction = a_row.unsqueeze(-2).matmul(sub).squeeze(-2)
        corrected = a_row + correction
        zeros = torch.zeros(batch, nv, nc, c - i, dtype=torch.float32)
        rows.append(torch.cat([corrected, zeros], -1))
    attn = torch.stack(rows, -2) + torch.eye(c, dtype=torch.float32)
    value_t = attn.matmul(v_beta)
    k_cumdecay = attn.matmul(k_beta * g.exp().unsqueeze(-1))
    state = initial_state.float() if initial_state is not None else torch.zeros(batch, nv, hk, hv)
    chunks = []
    for i in range(nc):
        q_i, k_i, v_i = q.select(2, i), k.select(2, i), value_t.select(2, i)
        g_i, dm_i, kcd_i = g.select(2, i), decay_mask.select(2, i), k_cumdecay.select(2, i)
        attn_inner = (q_i.matmul(k_i.transpose(-1, -2)) * dm_i).masked_fill(mask1, 0.0)
        v_new = v_i - kcd_i.matmul(state)
        attn_inter = (q_i * g_i.exp().unsqueeze(-1)).matmul(state)
        chunks.append(attn_inter + attn_inner.matmul(v_new))
        g_last = g_i.narrow(-1, c - 1, 1)
        decay = g_last.exp().unsqueeze(-1)
        g_diff = (g_last - g_i).exp().unsqueeze(-1)
        state = state * decay + (k_i * g_diff).transpose(-1, -2).matmul(v_new)
    out = torch.stack(chunks, 2).reshape(batch, nv, seq_p, hv).narrow(2, 0, seq).contiguous()
    return out, state
