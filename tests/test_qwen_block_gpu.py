"""GPU parity of the batched Qwen3.5 layer-level entry points (hs_gdn_layer_forward, hs_qwen_attn_layer_forward,
hs_qwen_block_forward) against the CPU oracle's chained layer functions (ATen restatements of
architectures/qwen3_5.rs:606-802 and :902-1075) at reduced size, and batched == serial: every row of a batch equals the
unbatched call on that sequence (the property the reference tests for its batched Llama path, llama.rs:3658-3711)."""
import math

import pytest
import torch

from oracle import attention_ref as ar
from oracle import gdn_ref as gr
from oracle import quant_ref as qr
from tests.util import assert_close_attn, no_device_error

pytestmark = pytest.mark.gpu

NK, NV, HD, KS = 2, 4, 128, 4
CONV_DIM = (2 * NK + NV) * HD
HQ, HKV, D, RD = 16, 2, 256, 64


def _gdn_weights(seed):
    g = torch.Generator().manual_seed(seed)
    return ((torch.randn(CONV_DIM, 1, KS, generator=g) * 0.5).bfloat16(), torch.randn(NV, generator=g) * 0.3, torch.randn(NV, generator=g) * 0.3,
            1.0 + 0.1 * torch.randn(HD, generator=g))


def _gdn_inputs(b, t, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(b, t, CONV_DIM, generator=g).bfloat16(), torch.randn(b, t, NV, HD, generator=g).bfloat16(),
            torch.randn(b, t, NV, generator=g).bfloat16(), torch.randn(b, t, NV, generator=g).bfloat16())


def _oracle_gdn_layer(w, a_log, dt_bias, nw, x, z, a, bb, conv, rec):
    q, k, v, g, beta, conv = gr.gdn_prologue(x, w, conv, a, bb, a_log, dt_bias, NK, HD, NV, HD)
    r = NV // NK
    qh = q.repeat_interleave(r, dim=2).permute(0, 2, 1, 3).contiguous()
    kh = k.repeat_interleave(r, dim=2).permute(0, 2, 1, 3).contiguous()
    fn = gr.chunked_delta_rule if x.shape[1] > 1 else gr.recurrent_sequence
    o, rec = fn(qh, kh, v.permute(0, 2, 1, 3).contiguous(), g.permute(0, 2, 1).contiguous(), beta.permute(0, 2, 1).contiguous(), rec)
    return gr.rmsnorm_gated(o.permute(0, 2, 1, 3), z, nw, 1e-6), conv, rec


def test_gdn_layer_prompt_then_decode_matches_oracle_and_serial(cuda):
    from hyprstream_b200 import ops

    b, t = 3, 70
    w, a_log, dt_bias, nw = _gdn_weights(1)
    layer = ops.GdnLayer(w.to(cuda), a_log.to(cuda), dt_bias.to(cuda), nw.to(cuda), NK, NV)
    x, z, a, bb = _gdn_inputs(b, t + 2, seed=2)
    conv, rec = layer.new_states(b, cuda)
    conv_ref = rec_ref = None
    ys, ys_ref = [], []
    for i, (lo, hi) in enumerate(((0, t), (t, t + 1), (t + 1, t + 2))):
        sl = [u[:, lo:hi].contiguous() for u in (x, z, a, bb)]
        ys.append(layer.forward(*[u.to(cuda) for u in sl], conv, rec, has_state=i > 0))
        yr, conv_ref, rec_ref = _oracle_gdn_layer(w, a_log, dt_bias, nw, *sl, conv_ref, rec_ref)
        ys_ref.append(yr)
    torch.cuda.synchronize()
    y, y_ref = torch.cat(ys, 1).cpu().float(), torch.cat(ys_ref, 1).float()
    diff = (y - y_ref).abs()
    # the prompt runs through the tensor-core chunked rule (bf16 operands: within 2e-2 / 2e-3 of the fp32 rule on outputs of
    # unit scale); RMSNormGated then divides a row by its rms and multiplies by silu(z), so the bound carries to y relative to
    # the row's scale
    scale = y_ref.abs().amax(dim=-1, keepdim=True).clamp_min(1.0)
    assert torch.all(diff <= 2e-2 * scale) and diff.mean().item() <= 2e-3, (diff.max().item(), diff.mean().item())
    assert (rec.cpu() - rec_ref).abs().max().item() <= 2e-2 * max(1.0, rec_ref.abs().max().item())
    assert torch.equal(conv.cpu(), conv_ref)
    # batched == serial: every row alone gives the same outputs and states
    for r in range(b):
        c1, r1 = layer.new_states(1, cuda)
        outs = []
        for i, (lo, hi) in enumerate(((0, t), (t, t + 1), (t + 1, t + 2))):
            sl = [u[r:r + 1, lo:hi].contiguous().to(cuda) for u in (x, z, a, bb)]
            outs.append(layer.forward(*sl, c1, r1, has_state=i > 0))
        torch.cuda.synchronize()
        assert torch.equal(torch.cat(outs, 1)[0], torch.cat(ys, 1)[r]), f"row {r}"
        assert torch.equal(r1[0], rec[r]) and torch.equal(c1[0], conv[r])
    no_device_error()


def test_gdn_layer_prompt_equals_the_three_boundary_calls_bit_for_bit(cuda):
    """The layer entry hands q, k, v from its prologue to the chunked rule as bf16; the rule rounds q and k to bf16 itself and v is
    a bf16 value already, so the entry must equal hs_gdn_prologue (fp32 tensors) -> hs_gdn_chunk_prefill -> hs_gdn_epilogue exactly,
    output and both states; a ragged token count (tail chunk) and a continued prompt (carried states) included."""
    from hyprstream_b200 import ops

    b = 2
    w, a_log, dt_bias, nw = _gdn_weights(5)
    layer = ops.GdnLayer(w.to(cuda), a_log.to(cuda), dt_bias.to(cuda), nw.to(cuda), NK, NV)
    x, z, a, bb = [u.to(cuda) for u in _gdn_inputs(b, 150, seed=6)]
    conv, rec = layer.new_states(b, cuda)
    conv2, rec2 = layer.new_states(b, cuda)
    for i, (lo, hi) in enumerate(((0, 83), (83, 150))):
        sl = [u[:, lo:hi].contiguous() for u in (x, z, a, bb)]
        y = layer.forward(*sl, conv, rec, has_state=i > 0)
        q, k, v, g, beta = ops.gdn_prologue(sl[0], layer.conv_weight, conv2, i > 0, sl[2], sl[3], layer.neg_a_exp, layer.dt_bias, NK, NV)
        o = ops.gdn_chunk_prefill(q, k, v, g, beta, rec2)
        y2 = ops.gdn_epilogue(o, sl[1], layer.norm_weight)
        torch.cuda.synchronize()
        assert torch.equal(y, y2) and torch.equal(rec, rec2) and torch.equal(conv, conv2), i
    no_device_error()


def test_gdn_layer_decode_step_equals_the_three_boundary_calls_bit_for_bit(cuda):
    """A decode step of the layer entry is one kernel (conv, gates, recurrent rule, RMSNormGated) plus the conv_state shift; it
    must equal hs_gdn_prologue -> hs_gdn_recurrent -> hs_gdn_epilogue exactly - output, recurrent state and conv state - for a
    sequence's very first token (no carried state) and for later ones."""
    from hyprstream_b200 import ops

    b = 5
    w, a_log, dt_bias, nw = _gdn_weights(7)
    layer = ops.GdnLayer(w.to(cuda), a_log.to(cuda), dt_bias.to(cuda), nw.to(cuda), NK, NV)
    x, z, a, bb = [u.to(cuda) for u in _gdn_inputs(b, 6, seed=8)]
    conv, rec = layer.new_states(b, cuda)
    conv2, rec2 = layer.new_states(b, cuda)
    rec.fill_(7.0)  # a state that is being started is cleared by the entry
    for t in range(6):
        sl = [u[:, t:t + 1].contiguous() for u in (x, z, a, bb)]
        y = layer.forward(*sl, conv, rec, has_state=t > 0)
        q, k, v, g, beta = ops.gdn_prologue(sl[0], layer.conv_weight, conv2, t > 0, sl[2], sl[3], layer.neg_a_exp, layer.dt_bias, NK, NV)
        o = ops.gdn_recurrent(q, k, v, g, beta, rec2)
        y2 = ops.gdn_epilogue(o, sl[1], layer.norm_weight)
        torch.cuda.synchronize()
        assert torch.equal(y, y2) and torch.equal(rec, rec2) and torch.equal(conv, conv2), t
    no_device_error()


def _attn_case(cuda, b, t, seed):
    from hyprstream_b200 import kv_cache as kc

    g = torch.Generator().manual_seed(seed)
    qw, kw = 0.1 * torch.randn(D, generator=g), 0.1 * torch.randn(D, generator=g)
    sin, cos = ar.rope_tables(RD, 10000.0, 256, torch.bfloat16)
    caches = [kc.LayerKVCache(1024, kc.KVQuantType.INT8, HKV, D, cuda, block=128, scale_dtype=1) for _ in range(b)]
    for c in caches:
        c._ensure_capacity(t + 8)
    view, keep = kc.make_view(caches)
    return g, qw, kw, sin, cos, caches, view, keep


def _oracle_attn(qw, kw, sin, cos, q_proj, k_proj, v_proj, positions, k_hist, v_hist, b, t):
    """Qwen3_5FullAttention::forward between projections, over the dequantised history (+ the new tokens quantised)."""
    x = q_proj.reshape(b * t, HQ, 2 * D)
    query = ar.apply_partial_rope(ar.qk_norm(x[..., :D], qw, 1e-6).unsqueeze(0), sin, cos, positions, RD)[0].reshape(b, t, HQ, D)
    gate = x[..., D:].reshape(b, t, HQ, D)
    k_rot = ar.apply_partial_rope(ar.qk_norm(k_proj.reshape(b * t, HKV, D), kw, 1e-6).unsqueeze(0), sin, cos, positions, RD)[0].reshape(b, t, HKV, D)
    outs = []
    for r in range(b):
        new = []
        for src in (k_rot[r:r + 1], v_proj[r:r + 1]):
            oc, oa = qr.quantize(src.float().numpy(), qr.INT8, 128, True)
            new.append(torch.from_numpy(qr.dequantize(oc, oa, qr.INT8, src.numel(), 128)).bfloat16().reshape(src.shape))
        k_hist[r] = new[0] if k_hist[r] is None else torch.cat([k_hist[r], new[0]], 1)
        v_hist[r] = new[1] if v_hist[r] is None else torch.cat([v_hist[r], new[1]], 1)
        if t == 1:   # decode attends the cache (quantised precision)
            kf, vf = k_hist[r], v_hist[r]
        else:        # the prompt attends the K/V it has just produced, in bf16 (what an unquantised reference cache hands back,
                     # qwen3_5.rs:992-1003; a quantised one would hand back the dequantised values: inside the tolerance)
            kf, vf = k_rot[r:r + 1], v_proj[r:r + 1]
        outs.append(ar.qwen_gated_attention_core(query[r:r + 1], gate[r:r + 1], kf, vf, HQ).reshape(t, HQ, D))
    return torch.stack(outs)


def test_attn_layer_prompt_then_ragged_decode_matches_oracle_and_serial(cuda):
    from hyprstream_b200 import kv_cache as kc, ops

    b, t = 3, 33
    g, qw, kw, sin, cos, caches, view, keep = _attn_case(cuda, b, t, seed=5)
    layer = ops.QwenAttnLayer(qw.to(cuda), kw.to(cuda), sin.to(cuda), cos.to(cuda), RD, HQ, HKV, D)
    k_hist, v_hist = [None] * b, [None] * b
    pos0 = torch.zeros(b, dtype=torch.int32, device=cuda)
    steps = [(t, torch.arange(t).repeat(b), pos0)]
    for s in range(2):
        steps.append((1, torch.full((b,), t + s), torch.full((b,), t + s, dtype=torch.int32, device=cuda)))
    got, ref, inputs = [], [], []
    for n_tok, positions, dst in steps:
        q_proj = torch.randn(b * n_tok, HQ * 2 * D, generator=g).bfloat16()
        k_proj = torch.randn(b * n_tok, HKV * D, generator=g).bfloat16()
        v_proj = torch.randn(b, n_tok, HKV, D, generator=g).bfloat16()
        inputs.append((q_proj, k_proj, v_proj))
        out = layer.forward(q_proj.to(cuda), k_proj.to(cuda), v_proj.to(cuda), view, positions.int().to(cuda), dst, dst + 1, b, n_tok)
        torch.cuda.synchronize()
        got.append(out.cpu())
        ref.append(_oracle_attn(qw, kw, sin, cos, q_proj, k_proj, v_proj, positions, k_hist, v_hist, b, n_tok))
    for i, (o, r) in enumerate(zip(got, ref)):
        assert_close_attn(o, r.float(), f"step {i}")
    # batched == serial: row 1 alone, through its own cache
    c1 = kc.LayerKVCache(1024, kc.KVQuantType.INT8, HKV, D, cuda, block=128, scale_dtype=1)
    c1._ensure_capacity(t + 8)
    v1, k1 = kc.make_view([c1])
    r = 1
    for (n_tok, positions, dst), (q_proj, k_proj, v_proj), full in zip(steps, inputs, got):
        rows = slice(r * n_tok, (r + 1) * n_tok)
        o = layer.forward(q_proj[rows].contiguous().to(cuda), k_proj[rows].contiguous().to(cuda), v_proj[r:r + 1].contiguous().to(cuda), v1,
                          positions[rows].int().contiguous().to(cuda), dst[r:r + 1].contiguous(), dst[r:r + 1] + 1, 1, n_tok)
        torch.cuda.synchronize()
        assert (o[0].cpu().float() - full[r].float()).abs().max().item() <= 8e-3, "batched row differs from the unbatched call"
    no_device_error()


def test_block_forward_equals_its_layers(cuda):
    """hs_qwen_block_forward (3 DeltaNet layers + 1 full-attention layer, one call) == the layer calls one by one, for a
    prompt and for a decode step."""
    from hyprstream_b200 import kv_cache as kc, ops

    b, t = 2, 40
    gdn = []
    for i in range(3):
        w, a_log, dt_bias, nw = _gdn_weights(10 + i)
        gdn.append(ops.GdnLayer(w.to(cuda), a_log.to(cuda), dt_bias.to(cuda), nw.to(cuda), NK, NV))
    g, qw, kw, sin, cos, caches_a, view_a, keep_a = _attn_case(cuda, b, t, seed=7)
    _, _, _, _, _, caches_b, view_b, keep_b = _attn_case(cuda, b, t, seed=7)
    attn = ops.QwenAttnLayer(qw.to(cuda), kw.to(cuda), sin.to(cuda), cos.to(cuda), RD, HQ, HKV, D)
    states_a = [l.new_states(b, cuda) for l in gdn]
    states_b = [l.new_states(b, cuda) for l in gdn]
    for step, n_tok in enumerate((t, 1)):
        gin = [tuple(u.to(cuda) for u in _gdn_inputs(b, n_tok, seed=20 + 10 * step + i)) for i in range(3)]
        q_proj = torch.randn(b * n_tok, HQ * 2 * D, generator=g).bfloat16().to(cuda)
        k_proj = torch.randn(b * n_tok, HKV * D, generator=g).bfloat16().to(cuda)
        v_proj = torch.randn(b, n_tok, HKV, D, generator=g).bfloat16().to(cuda)
        start = 0 if step == 0 else t
        positions = (torch.arange(n_tok) + start).repeat(b).int().to(cuda)
        dst = torch.full((b,), start, dtype=torch.int32, device=cuda)
        ys, out = ops.qwen_block_forward(gdn, [gin[i] + states_a[i] for i in range(3)], attn, (q_proj, k_proj, v_proj, view_a, positions, dst, dst + 1),
                                         step > 0, b, n_tok, cuda)
        ys2 = [gdn[i].forward(*gin[i], *states_b[i], has_state=step > 0) for i in range(3)]
        out2 = attn.forward(q_proj, k_proj, v_proj, view_b, positions, dst, dst + 1, b, n_tok)
        torch.cuda.synchronize()
        for y, y2 in zip(ys, ys2):
            assert torch.equal(y, y2)
        assert torch.equal(out, out2)
        for (ca, ra), (cb, rb) in zip(states_a, states_b):
            assert torch.equal(ca, cb) and torch.equal(ra, rb)
    no_device_error()
