"""GPU parity: gated-DeltaNet recurrent kernel against the CPU oracle (ATen restatement of
architectures/qwen3_5.rs:342-498,725-751) and the committed fixture from the independent implementation."""
import os

import numpy as np
import pytest
import torch

from oracle import gdn_ref as gr
from tests.util import GOLD

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
