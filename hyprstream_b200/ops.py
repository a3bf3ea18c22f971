"""Thin functional wrappers over the C ABI: torch tensors supply device memory and the stream, nothing else.

Every function launches on torch's current CUDA stream and returns without synchronising.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence, Tuple

import torch

from . import ffi
from .ffi import KVView, check, lib

_DTYPES = {torch.bfloat16: ffi.DTYPE_BF16, torch.float16: ffi.DTYPE_F16, torch.float32: ffi.DTYPE_F32}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("hyprstream_b200 ops take CUDA tensors; there is no CPU path")
        if t is not None and not t.is_contiguous():
            raise ValueError("hyprstream_b200 ops take contiguous tensors")


def n_code_bytes(kind: int, n: int) -> int:
    return n if kind == ffi.KV_INT8 else (n + 1) // 2


def quantize_blockwise(x: torch.Tensor, kind: int, block: int = 64, scale_dtype: int = ffi.SCALE_F32
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """QuantizedTensor::from_tensor (kv_cache.rs:741-865): flat blockwise quantisation -> (codes u8, absmax)."""
    _need_cuda(x)
    n = x.numel()
    nb = (n + block - 1) // block
    # code buffers are allocated in whole 8-byte words (the kernel stores 8 codes at a time)
    codes = torch.empty((n_code_bytes(kind, n) + 7) // 8 * 8, dtype=torch.uint8, device=x.device)
    absmax = torch.empty(nb, dtype=torch.float16 if scale_dtype == ffi.SCALE_F16 else torch.float32, device=x.device)
    check(lib.hs_quantize_blockwise(kind, _ptr(x), _DTYPES[x.dtype], n, block, scale_dtype, _ptr(codes), _ptr(absmax), _stream()))
    return codes[: n_code_bytes(kind, n)], absmax


def dequantize_blockwise(codes: torch.Tensor, absmax: torch.Tensor, kind: int, n: int, block: int = 64,
                         dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """QuantizedTensor::to_tensor (kv_cache.rs:871-957)."""
    _need_cuda(codes, absmax)
    out = torch.empty(n, dtype=dtype, device=codes.device)
    sd = ffi.SCALE_F16 if absmax.dtype == torch.float16 else ffi.SCALE_F32
    check(lib.hs_dequantize_blockwise(kind, _ptr(codes), _ptr(absmax), n, block, sd, _ptr(out), _DTYPES[dtype], _stream()))
    return out


def rope_apply(x: torch.Tensor, sin: torch.Tensor, cos: torch.Tensor, positions: torch.Tensor,
               rotary_dim: Optional[int] = None) -> torch.Tensor:
    """RoPE::apply_rotary_pos_emb (rope.rs:206-248) on x [rows, heads, dim] bf16 with int32 positions [rows]."""
    _need_cuda(x, sin, cos, positions)
    rows, heads, dim = x.shape
    rd = dim if rotary_dim is None else rotary_dim
    out = torch.empty_like(x)
    check(lib.hs_rope_apply(_ptr(x), _ptr(out), _ptr(sin), _ptr(cos), _ptr(positions), rows, heads, dim, rd,
                            sin.shape[0], _stream()))
    return out


def qk_norm_rope(x: torch.Tensor, n_heads: int, head_dim: int, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                 weight_plus_one: bool = True, sin: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                 positions: Optional[torch.Tensor] = None, rotary_dim: int = 0, with_gate: bool = False):
    """Per-head RMS norm + partial RoPE (+ gate split) of a projection output (qwen3_5.rs:963-990,1077-1091).

    x bf16 [n_tokens, n_heads * head_dim] (or [n_tokens, n_heads * 2 * head_dim] with ``with_gate``: per head the query
    half then the gate half).  Returns bf16 [n_tokens, n_heads, head_dim], and the gate of the same shape with
    ``with_gate``."""
    _need_cuda(x, norm_weight, sin, cos, positions)
    n_tokens = x.shape[0]
    per_head = head_dim * (2 if with_gate else 1)
    if x.dim() != 2 or x.shape[1] != n_heads * per_head or not x.is_contiguous():
        raise ValueError("qk_norm_rope: x must be contiguous [n_tokens, n_heads * head_dim (* 2 with the gate)]")
    out = torch.empty(n_tokens, n_heads, head_dim, dtype=torch.bfloat16, device=x.device)
    gate = torch.empty_like(out) if with_gate else None
    check(lib.hs_qk_norm_rope(_ptr(x), n_heads * per_head, per_head, _ptr(out), _ptr(gate), _ptr(norm_weight), float(eps),
                              1 if weight_plus_one else 0, _ptr(sin), _ptr(cos), _ptr(positions),
                              0 if sin is None else sin.shape[0], rotary_dim, n_tokens, n_heads, head_dim, _stream()))
    return (out, gate) if with_gate else out


def kv_quantize_write(view: KVView, k_new: torch.Tensor, v_new: torch.Tensor, dst_pos: Optional[torch.Tensor],
                      sin: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                      rotary_dim: int = 0) -> None:
    """LayerKVCache::update (kv_cache.rs:1275-1496) into device-resident (quantised) storage."""
    _need_cuda(k_new, v_new, dst_pos, sin, cos)
    n_seqs, n_tokens = k_new.shape[0], k_new.shape[1]
    check(lib.hs_kv_quantize_write(ctypes.byref(view), _ptr(k_new), _ptr(v_new), n_seqs, n_tokens, _ptr(dst_pos),
                                   _ptr(sin), _ptr(cos), rotary_dim, 0 if sin is None else sin.shape[0], _stream()))


def kv_norm_rope_quantize_write(view: KVView, k_proj: torch.Tensor, v_new: torch.Tensor, dst_pos: Optional[torch.Tensor], norm_weight: torch.Tensor,
                                eps: float = 1e-6, weight_plus_one: bool = True, sin: Optional[torch.Tensor] = None,
                                cos: Optional[torch.Tensor] = None, rotary_dim: int = 0, want_keys: bool = False) -> Optional[torch.Tensor]:
    """K's per-head RMS norm + (partial) RoPE + cache update in one pass (qwen3_5.rs:971-999): k_proj is the raw k projection
    [n_seqs, n_tokens, Hkv, D]; what is stored equals hs_qk_norm_rope followed by hs_kv_quantize_write, bit for bit.
    With ``want_keys`` the normed, rotated keys come back in bf16 (for a prompt's own attention)."""
    _need_cuda(k_proj, v_new, dst_pos, norm_weight, sin, cos)
    n_seqs, n_tokens = k_proj.shape[0], k_proj.shape[1]
    k_out = torch.empty_like(k_proj) if want_keys else None
    check(lib.hs_kv_norm_rope_quantize_write(ctypes.byref(view), _ptr(k_proj), _ptr(v_new), n_seqs, n_tokens, _ptr(dst_pos), _ptr(norm_weight),
                                             float(eps), 1 if weight_plus_one else 0, _ptr(sin), _ptr(cos), rotary_dim,
                                             0 if sin is None else sin.shape[0], _ptr(k_out), _stream()))
    return k_out


def kv_gather_dequantize(view: KVView, seq_lens: torch.Tensor, out_tokens: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """LayerKVCache::get (kv_cache.rs:1499-1643): bf16 [n_seqs, out_tokens, Hkv, D], zero past each length."""
    _need_cuda(seq_lens)
    n = seq_lens.numel()
    shape = (n, out_tokens, view.n_kv_heads, view.head_dim)
    k = torch.empty(shape, dtype=torch.bfloat16, device=seq_lens.device)
    v = torch.empty(shape, dtype=torch.bfloat16, device=seq_lens.device)
    check(lib.hs_kv_gather_dequantize(ctypes.byref(view), _ptr(seq_lens), n, out_tokens, _ptr(k), _ptr(v), _stream()))
    return k, v


_workspaces: dict = {}


def decode_workspace(n_seqs: int, n_q_heads: int, head_dim: int, device: torch.device) -> torch.Tensor:
    need = lib.hs_attn_decode_workspace_bytes(n_seqs, n_q_heads, head_dim)
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def decode_attention(q: torch.Tensor, view: KVView, seq_lens: torch.Tensor, softmax_scale: Optional[float] = None,
                     gate: Optional[torch.Tensor] = None, shard: bool = False, out: Optional[torch.Tensor] = None,
                     workspace: Optional[torch.Tensor] = None, shard_out=None):
    """Fused decode attention (llama.rs:605-640,710-844,1023-1119; qwen3_5.rs:992-1059).

    q bf16 [n_seqs, Hq, D], seq_lens int32 [n_seqs].  Returns bf16 [n_seqs, Hq, D], or with
    ``shard=True`` the fp32 pair (o [n_seqs, Hq, D], lse [n_seqs, Hq]) of a KV-length shard (written into the
    pair ``shard_out`` when given)."""
    _need_cuda(q, seq_lens, gate)
    n_seqs, hq, d = q.shape
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    ws = decode_workspace(n_seqs, hq, d, q.device) if workspace is None else workspace
    if shard:
        if shard_out is not None:
            o, lse = shard_out
            _need_cuda(o, lse)
            if o.dtype != torch.float32 or lse.dtype != torch.float32 or o.numel() != n_seqs * hq * d or lse.numel() != n_seqs * hq:
                raise ValueError("decode_attention: shard_out must be fp32 (o [n_seqs, Hq, D], lse [n_seqs, Hq])")
        else:
            o = torch.empty(n_seqs, hq, d, dtype=torch.float32, device=q.device)
            lse = torch.empty(n_seqs, hq, dtype=torch.float32, device=q.device)
        check(lib.hs_attn_decode(_ptr(q), ctypes.byref(view), _ptr(seq_lens), n_seqs, hq, scale, None, None, _ptr(ws),
                                 ws.numel(), _ptr(o), _ptr(lse), _stream()))
        return o, lse
    if out is None:
        out = torch.empty_like(q)
    check(lib.hs_attn_decode(_ptr(q), ctypes.byref(view), _ptr(seq_lens), n_seqs, hq, scale, _ptr(out), _ptr(gate), _ptr(ws),
                             ws.numel(), None, None, _stream()))
    return out


def decode_append(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, view: KVView, dst_pos: Optional[torch.Tensor], seq_lens: torch.Tensor,
                  softmax_scale: Optional[float] = None, sin: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                  rotary_dim: int = 0, gate: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Cache update of one new token per sequence + decode attention as one call (hs_attn_decode_append; llama.rs:598-640): the
    new token of sequence s goes to ``dst_pos[s]``, or with ``dst_pos=None`` to ``seq_lens[s] - 1`` - then, on an int8 cache, the
    attention kernel writes it itself (one launch per step).
    q bf16 [n_seqs, Hq, D]; k_new, v_new bf16 [n_seqs, 1, Hkv, D]; dst_pos, seq_lens int32 [n_seqs]."""
    _need_cuda(q, k_new, v_new, dst_pos, seq_lens, sin, cos, gate)
    n_seqs, hq, d = q.shape
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    ws = decode_workspace(n_seqs, hq, d, q.device) if workspace is None else workspace
    if out is None:
        out = torch.empty_like(q)
    check(lib.hs_attn_decode_append(_ptr(q), _ptr(k_new), _ptr(v_new), ctypes.byref(view), _ptr(dst_pos), _ptr(seq_lens), n_seqs, hq, scale,
                                    _ptr(sin), _ptr(cos), rotary_dim, 0 if sin is None else sin.shape[0], _ptr(out), _ptr(gate), _ptr(ws),
                                    ws.numel(), _stream()))
    return out


class DecodeStep:
    """One decode step of a batch as one C-ABI call (hs_attn_decode_step): the step's q, new K and new V travel from one
    pinned host buffer in one copy, the new token is quantised into the caches, the batch is attended, and the result
    comes back into a pinned host buffer.  Mirrors the reference engine's one-forward-per-step loop
    (torch_engine.rs:3719-3731).  Fill ``q_host`` / ``k_host`` / ``v_host`` (views of the pinned input buffer), call
    ``run()``, read ``out_host``."""

    def __init__(self, view: KVView, n_seqs: int, n_q_heads: int, device: torch.device, softmax_scale: Optional[float] = None):
        self.view, self.n_seqs, self.hq = view, n_seqs, n_q_heads
        hkv, d = view.n_kv_heads, view.head_dim
        self.scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
        sizes = [n_seqs * n_q_heads * d, n_seqs * hkv * d, n_seqs * hkv * d]
        self.host_in = torch.empty(sum(sizes), dtype=torch.bfloat16).pin_memory()
        self.q_host, self.k_host, self.v_host = (t.view(n_seqs, h, d) for t, h in zip(self.host_in.split(sizes), (n_q_heads, hkv, hkv)))
        self.dev_in = torch.empty(sum(sizes), dtype=torch.bfloat16, device=device)
        self.dev_out = torch.empty(n_seqs, n_q_heads, d, dtype=torch.bfloat16, device=device)
        self.out_host = torch.empty(n_seqs, n_q_heads, d, dtype=torch.bfloat16).pin_memory()
        self.ws = decode_workspace(n_seqs, n_q_heads, d, device)
        self.h2d_bytes, self.d2h_bytes = self.host_in.numel() * 2, self.out_host.numel() * 2

    def run(self, dst_pos: Optional[torch.Tensor], seq_lens: torch.Tensor, sin: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
            rotary_dim: int = 0, sync: bool = True) -> torch.Tensor:
        check(lib.hs_attn_decode_step(ctypes.byref(self.view), self.host_in.data_ptr(), self.dev_in.data_ptr(), _ptr(dst_pos), _ptr(seq_lens),
                                      self.n_seqs, self.hq, self.scale, _ptr(sin), _ptr(cos), rotary_dim, 0 if sin is None else sin.shape[0],
                                      self.dev_out.data_ptr(), self.out_host.data_ptr(), self.ws.data_ptr(), self.ws.numel(),
                                      ffi.STEP_SYNC if sync else 0, _stream()))
        return self.out_host


def merge_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LSE merge of partials: o_parts fp32 [P, n_seqs, Hq, D], lse_parts fp32 [P, n_seqs, Hq] -> bf16 [n_seqs, Hq, D]."""
    _need_cuda(o_parts, lse_parts, gate)
    p, n_seqs, hq, d = o_parts.shape
    out = torch.empty(n_seqs, hq, d, dtype=torch.bfloat16, device=o_parts.device)
    check(lib.hs_attn_merge_partials(_ptr(o_parts), _ptr(lse_parts), p, n_seqs * hq, d, _ptr(out), _ptr(gate), _stream()))
    return out


def merge_gathered(msgs: torch.Tensor, n_parts: int, n_seqs: int, hq: int, d: int, out: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LSE merge of `n_parts` all-gathered shard messages, in place: msgs is flat fp32, part p = [o (n_seqs*Hq*D) | lse
    (n_seqs*Hq)] at offset p * n_seqs*Hq*(D+1).  Returns bf16 [n_seqs, Hq, D]."""
    _need_cuda(msgs, gate, out)
    rows = n_seqs * hq
    stride = rows * (d + 1)
    if msgs.dtype != torch.float32 or msgs.numel() < n_parts * stride:
        raise ValueError("merge_gathered: msgs must hold n_parts fp32 messages of n_seqs*Hq*(D+1) floats")
    if out is None:
        out = torch.empty(n_seqs, hq, d, dtype=torch.bfloat16, device=msgs.device)
    base = msgs.data_ptr()
    check(lib.hs_attn_merge_partials_strided(base, base + rows * d * 4, n_parts, stride, stride, rows, d, _ptr(out), _ptr(gate), _stream()))
    return out


def gdn_recurrent(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                  state: torch.Tensor) -> torch.Tensor:
    """Recurrent gated delta rule (qwen3_5.rs:725-751) over [B, T, heads, dim] fp32 inputs; `state`
    [B, nv, hk, hv] fp32 is updated in place.  Returns out [B, T, nv, hv] fp32."""
    _need_cuda(q, k, v, g, beta, state)
    b, t, nk, hk = q.shape
    nv, hv = v.shape[2], v.shape[3]
    out = torch.empty(b, t, nv, hv, dtype=torch.float32, device=q.device)
    check(lib.hs_gdn_recurrent(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(state), _ptr(out), b, t, nk, nv, hk, hv,
                               _stream()))
    return out


def gdn_chunk_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                      state: torch.Tensor) -> torch.Tensor:
    """chunked_delta_rule (qwen3_5.rs:342-498) on the tensor cores: same arguments as gdn_recurrent, bf16 operand
    rounding inside (results within ~1e-3 of the fp32 rule); `state` is updated in place."""
    _need_cuda(q, k, v, g, beta, state)
    b, t, nk, hk = q.shape
    nv, hv = v.shape[2], v.shape[3]
    out = torch.empty(b, t, nv, hv, dtype=torch.float32, device=q.device)
    check(lib.hs_gdn_chunk_prefill(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(state), _ptr(out), b, t, nk, nv, hk, hv,
                                   _stream()))
    return out


def gdn_prologue(mixed_qkv: torch.Tensor, conv_weight: torch.Tensor, conv_state: torch.Tensor, has_state: bool, a_in: torch.Tensor,
                 b_in: torch.Tensor, neg_a_exp: torch.Tensor, dt_bias: torch.Tensor, n_k_heads: int, n_v_heads: int,
                 head_k_dim: int = 128, head_v_dim: int = 128):
    """conv1d + SiLU + split + L2 norm + gates of GatedDeltaNetLayer::forward (qwen3_5.rs:627-701).

    mixed_qkv bf16 [B, T, conv_dim]; conv_weight bf16 [conv_dim, 1, ks] or [conv_dim, ks]; conv_state bf16
    [B, conv_dim, ks-1], read when ``has_state`` and always replaced; a_in, b_in bf16 [B, T, nv]; neg_a_exp, dt_bias
    fp32 [nv].  Returns fp32 (q [B,T,nk,hk], k, v [B,T,nv,hv], g [B,T,nv], beta [B,T,nv])."""
    _need_cuda(mixed_qkv, conv_weight, conv_state, a_in, b_in, neg_a_exp, dt_bias)
    b, t, _ = mixed_qkv.shape
    ks = conv_weight.shape[-1]
    dev = mixed_qkv.device
    q = torch.empty(b, t, n_k_heads, head_k_dim, dtype=torch.float32, device=dev)
    k = torch.empty_like(q)
    v = torch.empty(b, t, n_v_heads, head_v_dim, dtype=torch.float32, device=dev)
    g = torch.empty(b, t, n_v_heads, dtype=torch.float32, device=dev)
    beta = torch.empty_like(g)
    check(lib.hs_gdn_prologue(_ptr(mixed_qkv), _ptr(conv_weight), _ptr(conv_state), 1 if has_state else 0, _ptr(a_in), _ptr(b_in),
                              _ptr(neg_a_exp), _ptr(dt_bias), _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), b, t, n_k_heads,
                              n_v_heads, head_k_dim, head_v_dim, ks, _stream()))
    return q, k, v, g, beta


def gdn_epilogue(o: torch.Tensor, z: torch.Tensor, norm_weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNormGated (qwen3_5.rs:305-313): o fp32 [..., hv], z bf16 same shape, norm_weight fp32 [hv] -> bf16 [..., hv]."""
    _need_cuda(o, z, norm_weight)
    hv = o.shape[-1]
    y = torch.empty(o.shape, dtype=torch.bfloat16, device=o.device)
    check(lib.hs_gdn_epilogue(_ptr(o), _ptr(z), _ptr(norm_weight), float(eps), _ptr(y), o.numel() // hv, hv, _stream()))
    return y


class GdnLayer:
    """The weights of one gated-DeltaNet layer that its elementwise steps use, and the batched layer call
    (hs_gdn_layer_forward: conv1d + SiLU + split + L2 norm + gates -> delta rule -> RMSNormGated; qwen3_5.rs:606-802
    between in_proj and out_proj)."""

    def __init__(self, conv_weight: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, norm_weight: torch.Tensor, n_k_heads: int,
                 n_v_heads: int, head_k_dim: int = 128, head_v_dim: int = 128, norm_eps: float = 1e-6):
        _need_cuda(conv_weight, a_log, dt_bias, norm_weight)
        self.conv_weight = conv_weight.reshape(conv_weight.shape[0], -1).contiguous()
        self.neg_a_exp = (-a_log.float().exp()).contiguous()
        self.dt_bias, self.norm_weight = dt_bias.float().contiguous(), norm_weight.float().contiguous()
        self.nk, self.nv, self.hk, self.hv = n_k_heads, n_v_heads, head_k_dim, head_v_dim
        self.params = ffi.GdnLayerParams(self.conv_weight.data_ptr(), self.neg_a_exp.data_ptr(), self.dt_bias.data_ptr(), self.norm_weight.data_ptr(),
                                         float(norm_eps), n_k_heads, n_v_heads, head_k_dim, head_v_dim, self.conv_weight.shape[1])

    def new_states(self, n_seqs: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """(conv_state bf16 [B, conv_dim, ks-1], rec_state f32 [B, nv, hk, hv]), one row per sequence."""
        conv_dim = (2 * self.nk * self.hk) + self.nv * self.hv
        return (torch.zeros(n_seqs, conv_dim, self.conv_weight.shape[1] - 1, dtype=torch.bfloat16, device=device),
                torch.zeros(n_seqs, self.nv, self.hk, self.hv, dtype=torch.float32, device=device))

    def workspace_bytes(self, n_seqs: int, n_tokens: int) -> int:
        return max(int(lib.hs_gdn_layer_workspace_bytes(ctypes.byref(self.params), n_seqs, n_tokens)), 256)

    def workspace(self, n_seqs: int, n_tokens: int, device) -> torch.Tensor:
        return torch.empty(self.workspace_bytes(n_seqs, n_tokens), dtype=torch.uint8, device=device)

    def forward(self, mixed_qkv: torch.Tensor, z: torch.Tensor, a_in: torch.Tensor, b_in: torch.Tensor, conv_state: torch.Tensor,
                rec_state: torch.Tensor, has_state: bool, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """mixed_qkv bf16 [B, T, conv_dim]; z bf16 [B, T, nv, hv]; a_in, b_in bf16 [B, T, nv]; states updated in place.
        Returns y bf16 [B, T, nv, hv]."""
        _need_cuda(mixed_qkv, z, a_in, b_in, conv_state, rec_state)
        b, t = mixed_qkv.shape[0], mixed_qkv.shape[1]
        ws = self.workspace(b, t, mixed_qkv.device) if workspace is None else workspace
        y = torch.empty(b, t, self.nv, self.hv, dtype=torch.bfloat16, device=mixed_qkv.device)
        check(lib.hs_gdn_layer_forward(ctypes.byref(self.params), _ptr(mixed_qkv), _ptr(z), _ptr(a_in), _ptr(b_in), _ptr(conv_state), _ptr(rec_state),
                                       1 if has_state else 0, b, t, _ptr(y), _ptr(ws), ws.numel(), _stream()))
        return y


class QwenAttnLayer:
    """Qwen3.5 gated full attention between its projections (hs_qwen_attn_layer_forward; qwen3_5.rs:902-1075): QK-norm
    with (1 + w), partial RoPE, gate split, cache update, decode or prompt attention, output gate."""

    def __init__(self, q_norm_weight: torch.Tensor, k_norm_weight: torch.Tensor, sin: torch.Tensor, cos: torch.Tensor, rotary_dim: int,
                 n_q_heads: int, n_kv_heads: int, head_dim: int, norm_eps: float = 1e-6, softmax_scale: Optional[float] = None):
        _need_cuda(q_norm_weight, k_norm_weight, sin, cos)
        self.qw, self.kw, self.sin, self.cos = q_norm_weight.float().contiguous(), k_norm_weight.float().contiguous(), sin, cos
        self.hq, self.hkv, self.d = n_q_heads, n_kv_heads, head_dim
        scale = 1.0 / math.sqrt(head_dim) if softmax_scale is None else softmax_scale
        self.params = ffi.QwenAttnParams(self.qw.data_ptr(), self.kw.data_ptr(), float(norm_eps), sin.data_ptr(), cos.data_ptr(), sin.shape[0],
                                         rotary_dim, n_q_heads, n_kv_heads, head_dim, float(scale))

    def workspace_bytes(self, n_seqs: int, n_tokens: int) -> int:
        return max(int(lib.hs_qwen_attn_layer_workspace_bytes(ctypes.byref(self.params), n_seqs, n_tokens)), 256)

    def workspace(self, n_seqs: int, n_tokens: int, device) -> torch.Tensor:
        return torch.empty(self.workspace_bytes(n_seqs, n_tokens), dtype=torch.uint8, device=device)

    def forward(self, q_proj: torch.Tensor, k_proj: torch.Tensor, v_proj: torch.Tensor, view: KVView, positions: torch.Tensor,
                dst_pos: torch.Tensor, seq_lens: Optional[torch.Tensor], n_seqs: int, n_tokens: int,
                workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """q_proj bf16 [B*T, Hq*2*D]; k_proj bf16 [B*T, Hkv*D]; v_proj bf16 [B, T, Hkv, D]; positions int32 [B*T]; dst_pos,
        seq_lens int32 [B].  Returns bf16 [B, T, Hq, D]."""
        _need_cuda(q_proj, k_proj, v_proj, positions, dst_pos, seq_lens)
        ws = self.workspace(n_seqs, n_tokens, q_proj.device) if workspace is None else workspace
        out = torch.empty(n_seqs, n_tokens, self.hq, self.d, dtype=torch.bfloat16, device=q_proj.device)
        check(lib.hs_qwen_attn_layer_forward(ctypes.byref(self.params), _ptr(q_proj), _ptr(k_proj), _ptr(v_proj), ctypes.byref(view), _ptr(positions),
                                             _ptr(dst_pos), _ptr(seq_lens), n_seqs, n_tokens, _ptr(out), _ptr(ws), ws.numel(), _stream()))
        return out


def qwen_block_forward(gdn_layers: Sequence[GdnLayer], gdn_inputs: Sequence[tuple], attn: Optional[QwenAttnLayer], attn_inputs: Optional[tuple],
                       has_state: bool, n_seqs: int, n_tokens: int, device, workspace: Optional[torch.Tensor] = None):
    """hs_qwen_block_forward: the DeltaNet layers of a block, then its full-attention layer, in one call.

    gdn_inputs[i] = (mixed_qkv, z, a_in, b_in, conv_state, rec_state); attn_inputs = (q_proj, k_proj, v_proj, view, positions,
    dst_pos, seq_lens).  Returns ([y_i bf16 [B, T, nv, hv]], out bf16 [B, T, Hq, D] or None)."""
    n = len(gdn_layers)
    params = (ffi.GdnLayerParams * max(n, 1))(*[l.params for l in gdn_layers])
    ys, ios = [], (ffi.GdnLayerIO * max(n, 1))()
    for i, (layer, inp) in enumerate(zip(gdn_layers, gdn_inputs)):
        _need_cuda(*inp)
        y = torch.empty(n_seqs, n_tokens, layer.nv, layer.hv, dtype=torch.bfloat16, device=device)
        ys.append(y)
        ios[i] = ffi.GdnLayerIO(*[_ptr(t) for t in inp], _ptr(y))
    out, ap, aio = None, None, None
    if attn is not None:
        q_proj, k_proj, v_proj, view, positions, dst_pos, seq_lens = attn_inputs
        _need_cuda(q_proj, k_proj, v_proj, positions, dst_pos, seq_lens)
        out = torch.empty(n_seqs, n_tokens, attn.hq, attn.d, dtype=torch.bfloat16, device=device)
        ap = ctypes.byref(attn.params)
        aio = ffi.QwenAttnIO(_ptr(q_proj), _ptr(k_proj), _ptr(v_proj), ctypes.addressof(view), _ptr(positions), _ptr(dst_pos), _ptr(seq_lens), _ptr(out))
    need = lib.hs_qwen_block_workspace_bytes(params, n, ap, n_seqs, n_tokens)
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device=device) if workspace is None else workspace
    check(lib.hs_qwen_block_forward(params, ios, n, ap, None if aio is None else ctypes.byref(aio), 1 if has_state else 0, n_seqs, n_tokens,
                                    _ptr(ws), ws.numel(), _stream()))
    return ys, out


def prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: Optional[float] = None,
                      gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal GQA prefill (llama.rs:1023-1119; qwen3_5.rs:1012-1059 with `gate`).

    q bf16 [B, q_len, Hq, D]; k, v bf16 [B, kv_len, Hkv, D], kv_len >= q_len.  Returns bf16 [B, q_len, Hq, D]."""
    _need_cuda(q, k, v, gate)
    b, ql, hq, d = q.shape
    kl, hkv = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    out = torch.empty_like(q)
    check(lib.hs_attn_prefill_causal(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(gate), b, ql, kl, hq, hkv, d, scale, _stream()))
    return out
