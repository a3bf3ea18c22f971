"""GPU parity: gated-DeltaNet recurrent kernel against the CPU oracle (ATen restatement of
architectures/qwen3_5.rs:342-498,725-751) and the committed fixture from the independent implementation."""
import os

import numpy as np
import pytest
import torch

from oracle import gdn_ref as gr
from tests.util import GOLD, no_device_error

pytestmark = pytest.mark.gpu

STATE_REL_TOL = 1e-4   # fp32 state: <= 1e-4 relative to its largest magnitude
OUT_ABS_TOL = 1e-4     # fp32 outputs of an fp32 rule


def _inputs(b, t, nk, nv, hk, hv, seed):
    g_ = torch.Generator().manual_seed(seed)
    q = gr.l2_normalize(torch.randn(b, t, nk, hk, generator=g_)) * hk ** -0.5
    k = gr.l2_normalize(torch.randn(b, t, nk, hk, generator=g_))
    v = torch.randn(b, t, nv, hv, generator=g_)
    g = torch.nn.functional.logsigmoid(torch.randn(b, t, nv, generator=g_))   # decay in (0,1): config 5
    beta = torch.sigmoid(torch.randn(b, t, nv, generator=g_))
    s0 = torch.randn(b, nv, hk, hv, generator=g_) * 0.1
    return q, k, v, g, beta, s0


def _oracle(q, k, v, g, beta, s0, chunked):
    """The oracle takes [B, nv, T, d] with k/q heads already repeated (qwen3_5.rs:704-720)."""
    r = v.shape[2] // q.shape[2]
    qh = q.repeat_interleave(r, dim=2).permute(0, 2, 1, 3).contiguous()
    kh = k.repeat_interleave(r, dim=2).permute(0, 2, 1, 3).contiguous()
    vh = v.permute(0, 2, 1, 3).contiguous()
    gh, bh = g.permute(0, 2, 1).contiguous(), beta.permute(0, 2, 1).contiguous()
    fn = gr.chunked_delta_rule if chunked else gr.recurrent_sequence
    o, s = fn(qh, kh, vh, gh, bh, s0)
    return o.permute(0, 2, 1, 3).contiguous(), s


def _check(out, state, o_ref, s_ref, what):
    od = (out.cpu() - o_ref).abs().max().item()
    sd = (state.cpu() - s_ref).abs().max().item() / max(s_ref.abs().max().item(), 1e-6)
    assert od <= OUT_ABS_TOL, f"{what}: out max-abs {od:.3g}"
    assert sd <= STATE_REL_TOL, f"{what}: state rel {sd:.3g}"


@pytest.mark.parametrize("t", [1, 2, 63, 64, 65, 200])
@pytest.mark.parametrize("nk,nv,hk", [(2, 4, 128), (2, 2, 64)])
def test_recurrent_matches_oracle(cuda, t, nk, nv, hk):
    from hyprstream_b200 import ops

    q, k, v, g, beta, s0 = _inputs(2, t, nk, nv, hk, 128, seed=t + nk)
    state = s0.clone().to(cuda)
    out = ops.gdn_recurrent(*(x.to(cuda) for x in (q, k, v, g, beta)), state)
    torch.cuda.synchronize()
    o_rec, s_rec = _oracle(q, k, v, g, beta, s0, chunked=False)
    _check(out, state, o_rec, s_rec, f"T={t} vs recurrent oracle")
    if t > 1:  # the reference's prefill branch (chunked_delta_rule) is the same recurrence
        o_ch, s_ch = _oracle(q, k, v, g, beta, s0, chunked=True)
        _check(out, state, o_ch, s_ch, f"T={t} vs chunked oracle")


def test_matches_independent_implementation_fixture(cuda):
    from hyprstream_b200 import ops

    f = np.load(os.path.join(GOLD, "gdn_hf.npz"))
    q, k, v, g, beta, s0 = (torch.from_numpy(f[n]) for n in ("q", "k", "v", "g", "beta", "s0"))
    tr = lambda x: x.transpose(1, 2).contiguous()
    qs = q * q.shape[-1] ** -0.5
    state = s0.clone().to(cuda)
    out = ops.gdn_recurrent(tr(qs).to(cuda), tr(k).to(cuda), tr(v).to(cuda), tr(g).to(cuda), tr(beta).to(cuda), state)
    torch.cuda.synchronize()
    _check(out, state, torch.from_numpy(f["out_chunk"]).transpose(1, 2), torch.from_numpy(f["state_chunk"]), "HF chunk")
    _check(out, state, torch.from_numpy(f["out_rec"]).transpose(1, 2), torch.from_numpy(f["state_rec"]), "HF recurrent")


def test_decode_steps_equal_one_multi_token_call(cuda):
    """256 single-token decode steps == one 256-token call (state carried in place), config-5 head geometry."""
    from hyprstream_b200 import ops

    q, k, v, g, beta, s0 = _inputs(3, 256, 16, 32, 128, 128, seed=5)
    dev = [x.to(cuda) for x in (q, k, v, g, beta)]
    s_a = s0.clone().to(cuda)
    out_a = ops.gdn_recurrent(*dev, s_a)
    s_b = s0.clone().to(cuda)
    outs = [ops.gdn_recurrent(*(x[:, i:i + 1].contiguous() for x in dev), s_b) for i in range(256)]
    torch.cuda.synchronize()
    # the single-token and the multi-token kernels sum in different orders: equal to fp32 round-off, not bit for bit
    assert (torch.cat(outs, 1) - out_a).abs().max().item() <= 1e-5
    assert (s_a - s_b).abs().max().item() <= 1e-5 * max(1.0, s_a.abs().max().item())


def test_rejects_unsupported_geometry(cuda):
    from hyprstream_b200 import ffi

    x = torch.zeros(16, device=cuda)
    p = x.data_ptr()
    assert ffi.lib.hs_gdn_recurrent(p, p, p, p, p, p, p, 1, 1, 2, 4, 96, 128, None) == ffi.HS_ERR_UNSUPPORTED
    assert ffi.lib.hs_gdn_recurrent(p, p, p, p, p, p, p, 1, 1, 3, 4, 128, 128, None) == ffi.HS_ERR_ARG
    assert ffi.lib.hs_gdn_recurrent(None, p, p, p, p, p, p, 1, 1, 2, 4, 128, 128, None) == ffi.HS_ERR_ARG


CHUNK_MAX_TOL, CHUNK_MEAN_TOL = 2e-2, 2e-3   # the path's stated tolerance against an fp32 recomputation


@pytest.mark.parametrize("t", [1, 15, 16, 17, 64, 200, 1000])
def test_chunk_prefill_matches_oracle_and_fp32_kernel(cuda, t):
    """hs_gdn_chunk_prefill (tensor cores, bf16 operands) against the oracle's chunked_delta_rule (fp32, chunk 64) and
    the fp32 recurrent kernel: outputs and final state, from a non-zero initial state."""
    from hyprstream_b200 import ops

    q, k, v, g, beta, s0 = _inputs(2, t, 2, 4, 128, 128, seed=100 + t)
    state = s0.clone().to(cuda)
    out = ops.gdn_chunk_prefill(*(x.to(cuda) for x in (q, k, v, g, beta)), state)
    state32 = s0.clone().to(cuda)
    out32 = ops.gdn_recurrent(*(x.to(cuda) for x in (q, k, v, g, beta)), state32)
    torch.cuda.synchronize()
    o_ref, s_ref = _oracle(q, k, v, g, beta, s0, chunked=t > 1)
    for ref_o, ref_s, what in ((o_ref, s_ref, "oracle"), (out32.cpu(), state32.cpu(), "fp32 kernel")):
        d = (out.cpu() - ref_o).abs()
        assert d.max().item() <= CHUNK_MAX_TOL and d.mean().item() <= CHUNK_MEAN_TOL, f"T={t} vs {what}: max {d.max().item():.3g} mean {d.mean().item():.3g}"
        sd = (state.cpu() - ref_s).abs().max().item() / max(ref_s.abs().max().item(), 1e-6)
        assert sd <= 1e-2, f"T={t} state vs {what}: rel {sd:.3g}"


def test_chunk_prefill_whole_head_and_half_head_ctas_agree(cuda):
    """The chunk kernel gives a head to one CTA, or - when the launch would leave most SMs idle - its two column halves to two
    CTAs.  A value column's arithmetic is the same either way: a small batch (half heads) must equal, row for row, the same
    sequences inside a batch large enough for whole-head CTAs; the large batch is also checked against the fp32 kernel."""
    from hyprstream_b200 import ops

    b, t, nk, nv = 6, 150, 8, 16  # 96 heads: whole-head CTAs on a 148-SM part; the first sequence alone: half-head CTAs
    q, k, v, g, beta, s0 = _inputs(b, t, nk, nv, 128, 128, seed=77)
    dev = [x.to(cuda) for x in (q, k, v, g, beta)]
    state = s0.clone().to(cuda)
    out = ops.gdn_chunk_prefill(*dev, state)
    state1 = s0[:1].clone().to(cuda)
    out1 = ops.gdn_chunk_prefill(*(x[:1].contiguous() for x in dev), state1)
    state32 = s0.clone().to(cuda)
    out32 = ops.gdn_recurrent(*dev, state32)
    torch.cuda.synchronize()
    assert torch.equal(out[:1], out1) and torch.equal(state[:1], state1)
    d = (out - out32).abs()
    assert d.max().item() <= CHUNK_MAX_TOL and d.mean().item() <= CHUNK_MEAN_TOL, (d.max().item(), d.mean().item())
    no_device_error()


def test_chunk_prefill_long_run_stays_close(cuda):
    """8192 tokens: the bf16 operand rounding does not accumulate in the fp32 state."""
    from hyprstream_b200 import ops

    q, k, v, g, beta, s0 = _inputs(1, 8192, 2, 2, 128, 128, seed=77)
    dev = [x.to(cuda) for x in (q, k, v, g, beta)]
    state, state32 = s0.clone().to(cuda), s0.clone().to(cuda)
    out = ops.gdn_chunk_prefill(*dev, state)
    out32 = ops.gdn_recurrent(*dev, state32)
    torch.cuda.synchronize()
    d = (out - out32).abs()
    assert d.max().item() <= CHUNK_MAX_TOL and d.mean().item() <= CHUNK_MEAN_TOL, f"max {d.max().item():.3g} mean {d.mean().item():.3g}"
    tail = d[:, -256:]
    assert tail.mean().item() <= 2 * d[:, :256].mean().item() + 1e-4, "error grows along the sequence"
    assert (state - state32).abs().max().item() <= 1e-2 * state32.abs().max().item()


def test_chunk_prefill_extreme_decay(cuda):
    """Decays down to e^-30 per token and beta at its ends: nothing overflows, results match the fp32 kernel."""
    from hyprstream_b200 import ops

    q, k, v, g, beta, s0 = _inputs(1, 100, 2, 2, 128, 128, seed=5)
    g = g * 0.0 - torch.tensor([0.0, 30.0]).repeat(50).reshape(1, 100, 1)
    beta = torch.where(torch.arange(100).reshape(1, 100, 1) % 3 == 0, torch.ones_like(beta), beta * 0.0)
    dev = [x.to(cuda) for x in (q, k, v, g.expand_as(beta).contiguous(), beta)]
    state, state32 = s0.clone().to(cuda), s0.clone().to(cuda)
    out = ops.gdn_chunk_prefill(*dev, state)
    out32 = ops.gdn_recurrent(*dev, state32)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and torch.isfinite(state).all()
    d = (out - out32).abs()
    assert d.max().item() <= CHUNK_MAX_TOL and d.mean().item() <= CHUNK_MEAN_TOL
