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


def test_partition_units_covers_every_unit_once():
    """Prefill / DeltaNet partition: sequences first, head groups only when there are more ranks than sequences."""
    from hyprstream_b200.sharded import partition_units

    for n_seqs, n_groups, n_ranks in [(8, 8, 1), (8, 8, 2), (8, 8, 8), (4, 2, 8), (4, 32, 8), (4, 2, 2), (4, 2, 4), (4, 1, 8), (3, 4, 8), (64, 1, 8)]:
        parts = partition_units(n_seqs, n_groups, n_ranks)
        assert len(parts) == n_ranks
        units = sorted((s, g) for p in parts for (s, lo, hi) in p for g in range(lo, hi))
        assert units == [(s, g) for s in range(n_seqs) for g in range(n_groups)], (n_seqs, n_groups, n_ranks)
        assert parts == partition_units(n_seqs, n_groups, n_ranks)
        widths = {hi - lo for p in parts for (_, lo, hi) in p}
        assert len(widths) == 1  # every unit of a run has the same head width: one kernel shape per rank
    assert partition_units(8, 8, 8) == [[(i, 0, 8)] for i in range(8)]                       # prefill 8 x 8192 on 8 GPUs: a sequence each
    assert partition_units(4, 2, 8) == [[(i // 2, i % 2, i % 2 + 1)] for i in range(8)]    # the 4 x 32768 block: (sequence, head half)
    with pytest.raises(ValueError):
        partition_units(0, 1, 1)


def _gdn_worker(rank, world, port, q, k, v, g, beta, ret):
    """Each rank runs the oracle's recurrence on its (sequence, value-head range) units only; one all-gather of the
    outputs shows that the union is the unpartitioned result (no data-path exchange is needed to compute it)."""
    from oracle import gdn_ref as gr

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, nv = v.shape[0], v.shape[1]
        r = nv // k.shape[1]
        out = torch.zeros_like(v)
        for (s, lo, hi) in sharded.partition_units(b, 2, world)[rank]:  # two head groups per sequence
            h0, h1 = lo * nv // 2, hi * nv // 2
            qh = q[s:s + 1].repeat_interleave(r, dim=1)[:, h0:h1]
            kh = k[s:s + 1].repeat_interleave(r, dim=1)[:, h0:h1]
            o, _ = gr.recurrent_sequence(qh, kh, v[s:s + 1, h0:h1], g[s:s + 1, h0:h1], beta[s:s + 1, h0:h1], None)
            out[s, h0:h1] = o[0]
        dist.all_reduce(out)  # disjoint supports: the sum is the union
        ret[rank] = out
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_deltanet_partition_equals_unpartitioned():
    from oracle import gdn_ref as gr

    torch.manual_seed(1)
    b, nk, nv, t, d = 1, 2, 4, 12, 16   # one sequence, two ranks: the value heads are cut in halves
    q = torch.nn.functional.normalize(torch.randn(b, nk, t, d), dim=-1) * d ** -0.5
    k = torch.nn.functional.normalize(torch.randn(b, nk, t, d), dim=-1)
    v = torch.randn(b, nv, t, d)
    g = torch.nn.functional.logsigmoid(torch.randn(b, nv, t))
    beta = torch.sigmoid(torch.randn(b, nv, t))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_gdn_worker, args=(2, port, q, k, v, g, beta, ret), nprocs=2, join=True)
    r = nv // nk
    full, _ = gr.recurrent_sequence(q.repeat_interleave(r, dim=1), k.repeat_interleave(r, dim=1), v, g, beta, None)
    assert torch.allclose(ret[0], full, rtol=1e-6, atol=1e-6) and torch.equal(ret[0], ret[1])


def test_exchange_handles_two_rank_gloo():
    """Host set-up of the one-launch sharded decode: every rank ends with all ranks' handles in rank order."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_handles_worker, args=(2, port, ret), nprocs=2, join=True)
    want = bytes([7] * 64) + bytes([8] * 64)
    assert ret[0] == want and ret[1] == want


def _handles_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = sharded.exchange_handles(bytes([7 + rank] * 64))
    finally:
        dist.destroy_process_group()
