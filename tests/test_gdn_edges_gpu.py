"""GPU parity: the elementwise steps either side of the gated-DeltaNet rule (conv1d + SiLU + split + L2 norm + gates;
RMSNormGated) against the CPU oracle (ATen restatement of architectures/qwen3_5.rs:305-313,627-701), alone and chained
with the rule as GatedDeltaNetLayer::forward chains them."""
import pytest
import torch

from oracle import gdn_ref as gr
from tests.util import no_device_error

pytestmark = pytest.mark.gpu

NK, NV, HD, KS = 2, 4, 128, 4
CONV_DIM = (2 * NK + NV) * HD


def _layer_inputs(b, t, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(b, t, CONV_DIM, generator=g).bfloat16()
    w = (torch.randn(CONV_DIM, 1, KS, generator=g) * 0.5).bfloat16()
    a = torch.randn(b, t, NV, generator=g).bfloat16()
    bb = torch.randn(b, t, NV, generator=g).bfloat16()
    a_log = torch.randn(NV, generator=g) * 0.3
    dt_bias = torch.randn(NV, generator=g) * 0.3
    return x, w, a, bb, a_log, dt_bias


def _close(mine, ref, what):
    """The conv sum and SiLU are rounded to bf16 in the reference; an fp32 summation-order difference can flip such a
    rounding by one bf16 step (2^-8 relative) on isolated elements, which then shows in every element of that head
    through the norm.  Nearly all elements agree to fp32 round-off; none may differ by more than a bf16 step."""
    mine, ref = mine.cpu().float(), ref.float()
    diff = (mine - ref).abs()
    assert torch.all(diff <= 1e-5 + 8e-3 * ref.abs()), f"{what}: max diff {diff.max().item():.3g}"
    assert (diff <= 1e-6 + 1e-5 * ref.abs()).float().mean().item() >= 0.98, f"{what}: too many elements off by a bf16 step"


def _run_prologue(cuda, x, w, state, has_state, a, bb, a_log, dt_bias):
    from hyprstream_b200 import ops

    st = state.clone().to(cuda)
    outs = ops.gdn_prologue(x.to(cuda), w.to(cuda), st, has_state, a.to(cuda), bb.to(cuda), (-a_log.exp()).to(cuda), dt_bias.to(cuda), NK, NV)
    torch.cuda.synchronize()
    return outs, st


@pytest.mark.parametrize("t", [1, 2, 3, 31, 32, 33, 100])
@pytest.mark.parametrize("has_state", [False, True])
def test_prologue_matches_oracle(cuda, t, has_state):
    x, w, a, bb, a_log, dt_bias = _layer_inputs(2, t, seed=t)
    state = torch.randn(2, CONV_DIM, KS - 1, generator=torch.Generator().manual_seed(99)).bfloat16()
    ref = gr.gdn_prologue(x, w, state if has_state else None, a, bb, a_log, dt_bias, NK, HD, NV, HD)
    (q, k, v, g, beta), st = _run_prologue(cuda, x, w, state, has_state, a, bb, a_log, dt_bias)
    for mine, r, name in ((q, ref[0], "q"), (k, ref[1], "k"), (v, ref[2], "v")):
        _close(mine, r, f"T={t} {name}")
    assert (g.cpu() - ref[3]).abs().max().item() <= 1e-5 and (beta.cpu() - ref[4]).abs().max().item() <= 1e-6
    assert torch.equal(st.cpu(), ref[5]), "conv state"
    no_device_error()


def test_prologue_two_calls_equal_one(cuda):
    """Carrying conv_state across calls (prefill, then decode steps) equals one call over all tokens, bit for bit."""
    x, w, a, bb, a_log, dt_bias = _layer_inputs(1, 70, seed=5)
    zero = torch.zeros(1, CONV_DIM, KS - 1).bfloat16()
    (q, k, v, g, beta), st = _run_prologue(cuda, x, w, zero, False, a, bb, a_log, dt_bias)
    (q1, k1, v1, g1, b1), s1 = _run_prologue(cuda, x[:, :68], w, zero, False, a[:, :68], bb[:, :68], a_log, dt_bias)
    parts = [(q1, k1, v1)]
    for i in (68, 69):  # two single-token decode steps
        (qi, ki, vi, gi, bi), s1 = _run_prologue(cuda, x[:, i:i + 1], w, s1.cpu(), True, a[:, i:i + 1], bb[:, i:i + 1], a_log, dt_bias)
        parts.append((qi, ki, vi))
    for j, full in enumerate((q, k, v)):
        assert torch.equal(torch.cat([p[j] for p in parts], dim=1), full)
    assert torch.equal(s1, st)


@pytest.mark.parametrize("rows", [1, 15, 16, 17, 1000])
def test_epilogue_matches_oracle(cuda, rows):
    from hyprstream_b200 import ops

    g = torch.Generator().manual_seed(rows)
    o = torch.randn(rows, HD, generator=g)
    z = torch.randn(rows, HD, generator=g).bfloat16()
    w = 1.0 + 0.1 * torch.randn(HD, generator=g)
    y = ops.gdn_epilogue(o.to(cuda), z.to(cuda), w.to(cuda), 1e-6)
    torch.cuda.synchronize()
    ref = gr.rmsnorm_gated(o, z, w, 1e-6)  # fp32 in, fp32 out; the layer then casts to the model dtype (qwen3_5.rs:782)
    diff = (y.cpu().float() - ref).abs()
    assert torch.all(diff <= 1e-6 + 2 ** -8 * ref.abs()), f"max diff {diff.max().item():.3g}"  # one bf16 rounding


def test_layer_chain_prefill_then_decode(cuda):
    """prologue -> delta rule -> RMSNormGated over a 100-token prompt and 3 decode steps, states carried, against the
    oracle's chain (its chunked rule for the prompt, its recurrent step for decode: qwen3_5.rs:725-769)."""
    from hyprstream_b200 import ops

    b, t = 2, 100
    x, w, a, bb, a_log, dt_bias = _layer_inputs(b, t + 3, seed=11)
    gen = torch.Generator().manual_seed(12)
    z = torch.randn(b, t + 3, NV, HD, generator=gen).bfloat16()
    nw = 1.0 + 0.1 * torch.randn(HD, generator=gen)
    # oracle
    conv_ref, rec_ref, ys_ref = None, None, []
    for lo, hi in ((0, t), (t, t + 1), (t + 1, t + 2), (t + 2, t + 3)):
        q, k, v, g, beta, conv_ref = gr.gdn_prologue(x[:, lo:hi], w, conv_ref, a[:, lo:hi], bb[:, lo:hi], a_log, dt_bias, NK, HD, NV, HD)
        r = NV // NK
        qh = q.repeat_interleave(r, dim=2).permute(0, 2, 1, 3).contiguous()
        kh = k.repeat_interleave(r, dim=2).permute(0, 2, 1, 3).contiguous()
        fn = gr.chunked_delta_rule if hi - lo > 1 else gr.recurrent_sequence
        o, rec_ref = fn(qh, kh, v.permute(0, 2, 1, 3).contiguous(), g.permute(0, 2, 1).contiguous(), beta.permute(0, 2, 1).contiguous(), rec_ref)
        ys_ref.append(gr.rmsnorm_gated(o.permute(0, 2, 1, 3), z[:, lo:hi], nw, 1e-6))
    y_ref = torch.cat(ys_ref, dim=1)
    # kernels
    conv = torch.zeros(b, CONV_DIM, KS - 1, dtype=torch.bfloat16, device=cuda)
    rec = torch.zeros(b, NV, HD, HD, dtype=torch.float32, device=cuda)
    ys = []
    for i, (lo, hi) in enumerate(((0, t), (t, t + 1), (t + 1, t + 2), (t + 2, t + 3))):
        q, k, v, g, beta = ops.gdn_prologue(x[:, lo:hi].contiguous().to(cuda), w.to(cuda), conv, i > 0, a[:, lo:hi].contiguous().to(cuda),
                                            bb[:, lo:hi].contiguous().to(cuda), (-a_log.exp()).to(cuda), dt_bias.to(cuda), NK, NV)
        o = ops.gdn_recurrent(q, k, v, g, beta, rec)
        ys.append(ops.gdn_epilogue(o, z[:, lo:hi].contiguous().to(cuda), nw.to(cuda), 1e-6))
    torch.cuda.synchronize()
    y = torch.cat(ys, dim=1).cpu().float()
    diff = (y - y_ref).abs()
    # y is bf16 and a flipped bf16 rounding upstream moves isolated outputs by a step or two of their own size
    assert torch.all(diff <= 2e-2 + 2 ** -7 * y_ref.abs()) and diff.mean().item() <= 2e-3, f"max {diff.max().item():.3g} mean {diff.mean().item():.3g}"
    assert (rec.cpu() - rec_ref).abs().max().item() <= 2e-2 * max(1.0, rec_ref.abs().max().item())
    assert torch.equal(conv.cpu(), conv_ref)
    no_device_error()
