"""CPU tests of the KV-length sharding host logic: shard geometry, message packing, and the all-gather + log-sum-exp
merge on a world_size-2 gloo group (the GPU path replaces the two CPU helpers below by the kernels)."""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hyprstream_b200 import sharded


def test_shard_bounds_cover_and_align():
    for length in (0, 1, 255, 256, 257, 131072, 131072 + 17):
        for n in (1, 2, 3, 4, 8):
            b = sharded.shard_bounds(length, n)
            assert len(b) == n and b[0][0] == 0 and b[-1][1] == length
            for (s0, e0), (s1, e1) in zip(b[:-1], b[1:]):
                assert e0 == s1 and s0 <= e0
            assert all(s % 256 == 0 for s, _ in b if s < length)
            sizes = [e - s for s, e in b]
            assert max(sizes) - min(sizes) <= 256 + 255
    assert sharded.shard_bounds(131072, 8) == [(i * 16384, (i + 1) * 16384) for i in range(8)]
    with pytest.raises(ValueError):
        sharded.shard_bounds(10, 0)


def test_pack_unpack_roundtrip():
    o, lse = torch.randn(4, 32, 128), torch.randn(4, 32)
    msgs = torch.stack([sharded.pack_partial(o, lse), sharded.pack_partial(o * 2, lse - 1)])
    o2, l2 = sharded.unpack_partials(msgs)
    assert torch.equal(o2[0], o) and torch.equal(l2[1], lse - 1) and o2.is_contiguous() and l2.is_contiguous()
    assert msgs[0].numel() * 4 == 4 * 32 * 129 * 4  # the 66,048-byte message of config 3


def _partial(q, k, v):
    """fp32 shard attention -> (o normalised, lse); an empty shard yields lse = -inf."""
    b, hq, d = q.shape
    g = hq // k.shape[2]
    if k.shape[1] == 0:
        return torch.zeros(b, hq, d), torch.full((b, hq), float("-inf"))
    kf = k.float().repeat_interleave(g, dim=2).permute(0, 2, 1, 3)
    vf = v.float().repeat_interleave(g, dim=2).permute(0, 2, 1, 3)
    s = torch.einsum("bhd,bhld->bhl", q.float(), kf) / math.sqrt(d)
    lse = torch.logsumexp(s, dim=-1)
    return torch.einsum("bhl,bhld->bhd", (s - lse.unsqueeze(-1)).exp(), vf), lse


def _merge(o_parts, lse_parts):
    m = lse_parts.max(dim=0).values
    w = (lse_parts - m).exp()
    w = torch.where(torch.isinf(lse_parts), torch.zeros_like(w), w)
    return (w.unsqueeze(-1) * o_parts).sum(0) / w.sum(0).unsqueeze(-1)


def _worker(rank, world, port, length, q, k, v, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        s, e = sharded.shard_bounds(length, world)[rank]
        o, lse = _partial(q, k[:, s:e], v[:, s:e])
        o_parts, lse_parts = sharded.all_gather_partials(o, lse)
        ret[rank] = _merge(o_parts, lse_parts)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("length", [700, 200])  # 200 tokens < 2 pages: rank 1's shard is empty
def test_two_rank_gloo_sharded_decode_equals_unsharded(length):
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 8, 64), torch.randn(2, length, 2, 64), torch.randn(2, length, 2, 64)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, length, q, k, v, ret), nprocs=2, join=True)
    full, _ = _partial(q, k, v)
    assert torch.allclose(ret[0], full, rtol=1e-5, atol=1e-5)
    assert torch.equal(ret[0], ret[1])  # every rank ends with the same result


def test_balance_sequences_equalises_token_sums():
    """The batched-decode partition: equal counts per rank, near-equal cached-token sums, deterministic, a permutation."""
    import numpy as np

    from hyprstream_b200.sharded import balance_sequences

    rng = np.random.default_rng(7)
    for n_ranks in (1, 2, 4, 8):
        lens = [int(x) for x in rng.integers(512, 8193, size=32 * n_ranks)]
        parts = balance_sequences(lens, n_ranks)
        assert parts == balance_sequences(lens, n_ranks)
        assert sorted(i for p in parts for i in p) == list(range(len(lens)))
        assert all(len(p) == 32 for p in parts)
        sums = [sum(lens[i] for i in p) for p in parts]
        assert max(sums) - min(sums) <= 0.01 * max(sums)
    import pytest

    with pytest.raises(ValueError):
        balance_sequences([1, 2, 3], 2)
