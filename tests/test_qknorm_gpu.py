"""GPU parity: per-head RMS norm + partial RoPE + gate split (hs_qk_norm_rope) against the CPU oracle's restatement of
architectures/qwen3_5.rs:963-990,1077-1091 and runtime/rope.rs:206-248."""
import pytest
import torch

from oracle import attention_ref as ar
from tests.util import no_device_error

pytestmark = pytest.mark.gpu


def _bf16_step_close(mine, ref, what):
    """The norm is computed in fp32 and rounded once to bf16; a different summation order can flip that rounding on
    isolated elements, and the rotation then mixes such an element into its partner: nearly all outputs are equal bit
    for bit, none differs by more than about two bf16 steps of the row's scale."""
    mine, ref = mine.cpu().float(), ref.float()
    diff = (mine - ref).abs()
    scale = ref.abs().amax(dim=-1, keepdim=True)
    assert torch.all(diff <= 2 ** -6 * scale + 1e-6), f"{what}: max diff {diff.max().item():.3g}"
    assert (diff == 0).float().mean().item() >= 0.98, f"{what}: only {(diff == 0).float().mean().item():.4f} of the elements equal"


@pytest.mark.parametrize("nh,hd,rd,plus_one", [(16, 256, 64, True), (2, 256, 64, True), (32, 128, 128, False), (8, 64, 32, True)])
def test_norm_rope_gate_matches_oracle(cuda, nh, hd, rd, plus_one):
    from hyprstream_b200 import ops

    t = 37
    g = torch.Generator().manual_seed(nh + hd)
    x = torch.randn(t, nh, 2 * hd, generator=g).bfloat16()        # the doubled q projection: query | gate per head
    w = 0.1 * torch.randn(hd, generator=g)
    sin, cos = ar.rope_tables(rd, 10000.0, 200, torch.bfloat16)
    pos = torch.randint(0, 200, (t,), generator=g)
    query, gate = x[..., :hd], x[..., hd:]
    normed = ar.qk_norm(query, w if plus_one else w - 1.0, 1e-6)   # the oracle multiplies by (1 + w)
    ref = ar.apply_partial_rope(normed.unsqueeze(0), sin, cos, pos, rd)[0]
    out, gate_out = ops.qk_norm_rope(x.reshape(t, -1).to(cuda), nh, hd, (w if plus_one else w).to(cuda), 1e-6, plus_one, sin.to(cuda),
                                     cos.to(cuda), pos.int().to(cuda), rd, with_gate=True)
    torch.cuda.synchronize()
    if not plus_one:
        ref = ar.apply_partial_rope(ar.qk_norm(query, w - 1.0, 1e-6).unsqueeze(0), sin, cos, pos, rd)[0]
    _bf16_step_close(out, ref, "norm + rope")
    assert torch.equal(gate_out.cpu(), gate.contiguous())
    no_device_error()


def test_rope_only_equals_rope_apply_and_k_path(cuda):
    """No norm weight: the rotation alone, bit for bit the stand-alone RoPE kernel; dense k input (no gate)."""
    from hyprstream_b200 import ops

    t, nh, hd, rd = 50, 2, 256, 64
    g = torch.Generator().manual_seed(3)
    k = torch.randn(t, nh, hd, generator=g).bfloat16().to(cuda)
    sin, cos = ar.rope_tables(rd, 10000.0, 128, torch.bfloat16)
    pos = torch.arange(t, dtype=torch.int32, device=cuda)
    a = ops.qk_norm_rope(k.reshape(t, -1), nh, hd, None, sin=sin.to(cuda), cos=cos.to(cuda), positions=pos, rotary_dim=rd)
    b = ops.rope_apply(k, sin.to(cuda), cos.to(cuda), pos, rotary_dim=rd)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    w = 0.05 * torch.randn(hd, generator=g)
    kn = ops.qk_norm_rope(k.reshape(t, -1), nh, hd, w.to(cuda), 1e-6, True, sin.to(cuda), cos.to(cuda), pos, rd)
    ref = ar.apply_partial_rope(ar.qk_norm(k.cpu(), w, 1e-6).unsqueeze(0), sin, cos, pos.cpu().long(), rd)[0]
    _bf16_step_close(kn, ref, "k norm + rope")
    no_device_error()


def test_position_outside_table_is_recorded(cuda):
    from hyprstream_b200 import ffi, ops

    t, nh, hd, rd = 4, 2, 128, 64
    x = torch.randn(t, nh * hd).bfloat16().to(cuda)
    sin, cos = ar.rope_tables(rd, 10000.0, 16, torch.bfloat16)
    pos = torch.tensor([0, 5, 16, 3], dtype=torch.int32, device=cuda)  # 16 is one past the table
    out = ops.qk_norm_rope(x, nh, hd, None, sin=sin.to(cuda), cos=cos.to(cuda), positions=pos, rotary_dim=rd)
    torch.cuda.synchronize()
    assert ffi.take_device_error() & ffi.DEVERR_ROPE_RANGE
    assert torch.equal(out[2].cpu(), x[2].reshape(nh, hd).cpu())  # left unrotated


@pytest.mark.parametrize("kind,block,sdt,hkv,d,rd,t,paged", [(1, 128, 1, 2, 256, 64, 5, False), (1, 128, 1, 2, 256, 64, 300, False),
                                                              (2, 64, 1, 8, 128, 128, 70, False), (1, 64, 0, 8, 128, 128, 260, True),
                                                              (0, 64, 0, 2, 256, 64, 40, False)])
def test_fused_norm_rope_cache_write_equals_the_two_kernel_route(cuda, kind, block, sdt, hkv, d, rd, t, paged):
    """hs_kv_norm_rope_quantize_write (K normed, rotated, quantised and stored in one pass) against hs_qk_norm_rope followed
    by hs_kv_quantize_write: the same stored codes and scales and the same bf16 keys, bit for bit; short and long writes
    (8 and 16 elements per thread), cache positions that do not start at 0, contiguous and paged storage."""
    from hyprstream_b200 import kv_cache as kc, ops

    b = 2
    g = torch.Generator().manual_seed(t + d)
    k_proj = torch.randn(b, t, hkv, d, generator=g).bfloat16().to(cuda)
    v = torch.randn(b, t, hkv, d, generator=g).bfloat16().to(cuda)
    w = (0.1 * torch.randn(d, generator=g)).to(cuda)
    sin, cos = (x.to(cuda) for x in ar.rope_tables(rd, 10000.0, 512, torch.bfloat16))
    start = torch.tensor([0, 37], dtype=torch.int32, device=cuda)

    def caches():
        if paged:
            pool = kc.BlockPool(8, hkv, d, cuda, kind=kind, block=block, scale_dtype=sdt)
            cs = [kc.LayerKVCache.new_paged(2048, pool, owner=i) for i in range(b)]
        else:
            cs = [kc.LayerKVCache(2048, kc.KVQuantType(kind), hkv, d, cuda, block=block, scale_dtype=sdt) for _ in range(b)]
        for c in cs:
            c._ensure_capacity(37 + t)
        return cs

    ca, cb = caches(), caches()
    va, keep_a = kc.make_view(ca)
    vb, keep_b = kc.make_view(cb)
    k_fused = ops.kv_norm_rope_quantize_write(va, k_proj, v, start, w, 1e-6, True, sin, cos, rd, want_keys=True)
    positions = (start[:, None] + torch.arange(t, dtype=torch.int32, device=cuda)[None, :]).reshape(-1).contiguous()
    k_two = ops.qk_norm_rope(k_proj.reshape(b * t, -1), hkv, d, w, 1e-6, True, sin, cos, positions, rd).view(b, t, hkv, d)
    ops.kv_quantize_write(vb, k_two, v, start)
    torch.cuda.synchronize()
    assert torch.equal(k_fused, k_two)
    for i, (x, y) in enumerate(zip(ca, cb)):
        x.seq_pos = y.seq_pos = int(start[i]) + t
        for u, w_ in zip(x.snapshot(), y.snapshot()):
            if u is not None:
                lo = int(start[i])
                assert torch.equal(u[lo:].view(torch.uint8), w_[lo:].view(torch.uint8)), f"sequence {i}"
    no_device_error()
