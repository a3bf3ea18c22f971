"""GPU parity of the multi-GPU partition of prefill and of the gated-DeltaNet layers: the units `partition_units`
deals out - (sequence, head group) - computed one by one give exactly the unpartitioned result, so N GPUs that each take
their units need no exchange (causal prefill is independent per (sequence, kv head), llama.rs:776-781; the DeltaNet
state per (sequence, value head), qwen3_5.rs:697-699)."""
import pytest
import torch

from tests.util import no_device_error

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,hq,hkv,d", [(2, 32, 8, 128), (8, 32, 8, 128), (8, 16, 2, 256)])
def test_prefill_units_equal_unpartitioned(cuda, world, hq, hkv, d):
    from hyprstream_b200 import ops
    from hyprstream_b200.sharded import partition_units

    b, t = 2, 300
    g = torch.Generator(device=cuda).manual_seed(1)
    q = torch.randn(b, t, hq, d, device=cuda, generator=g).bfloat16()
    k = torch.randn(b, t, hkv, d, device=cuda, generator=g).bfloat16()
    v = torch.randn(b, t, hkv, d, device=cuda, generator=g).bfloat16()
    full = ops.prefill_attention(q, k, v)
    out = torch.zeros_like(full)
    grp = hq // hkv
    for rank_units in partition_units(b, hkv, world):
        for (s, lo, hi) in rank_units:
            o = ops.prefill_attention(q[s:s + 1, :, lo * grp:hi * grp].contiguous(), k[s:s + 1, :, lo:hi].contiguous(), v[s:s + 1, :, lo:hi].contiguous())
            out[s, :, lo * grp:hi * grp] = o[0]
    torch.cuda.synchronize()
    assert torch.equal(out, full)
    no_device_error()


@pytest.mark.parametrize("world", [2, 8])
def test_deltanet_units_equal_unpartitioned(cuda, world):
    from hyprstream_b200 import ops
    from hyprstream_b200.sharded import partition_units

    b, t, nk, nv, d = 2, 100, 4, 8, 128
    g = torch.Generator(device=cuda).manual_seed(2)
    q = torch.nn.functional.normalize(torch.randn(b, t, nk, d, device=cuda, generator=g), dim=-1) * d ** -0.5
    k = torch.nn.functional.normalize(torch.randn(b, t, nk, d, device=cuda, generator=g), dim=-1)
    v = torch.randn(b, t, nv, d, device=cuda, generator=g)
    gl = torch.nn.functional.logsigmoid(torch.randn(b, t, nv, device=cuda, generator=g))
    beta = torch.sigmoid(torch.randn(b, t, nv, device=cuda, generator=g))
    for fn in (ops.gdn_chunk_prefill, ops.gdn_recurrent):
        st_full = torch.zeros(b, nv, d, d, device=cuda)
        full = fn(q, k, v, gl, beta, st_full)
        out, st = torch.zeros_like(full), torch.zeros_like(st_full)
        groups = 4  # head groups per sequence: a group is 1 k head and its 2 v heads
        for rank_units in partition_units(b, groups, world):
            for (s, lo, hi) in rank_units:
                k0, k1, v0, v1 = lo * nk // groups, hi * nk // groups, lo * nv // groups, hi * nv // groups
                s_loc = torch.zeros(1, v1 - v0, d, d, device=cuda)
                o = fn(q[s:s + 1, :, k0:k1].contiguous(), k[s:s + 1, :, k0:k1].contiguous(), v[s:s + 1, :, v0:v1].contiguous(),
                       gl[s:s + 1, :, v0:v1].contiguous(), beta[s:s + 1, :, v0:v1].contiguous(), s_loc)
                out[s, :, v0:v1] = o[0]
                st[s, v0:v1] = s_loc[0]
        torch.cuda.synchronize()
        assert torch.equal(out, full) and torch.equal(st, st_full), fn.__name__
    no_device_error()
