"""KV-length sharding of one long context across the GPUs of a node (long-context decode: batch 4, 131072 tokens).

The reference has no collectives (its multi-GPU story is replicas and a layer split); this is
new design.  Each rank owns a contiguous, page-aligned slice of every sequence's KV cache, runs the
ordinary decode kernel over its slice with the shard outputs (normalised fp32 o and natural-log lse per
(sequence, head)), all-gathers the 66 KB pair over NCCL, and merges with the log-sum-exp kernel:
m = max lse_i; w_i = exp(lse_i - m); o = sum w_i o_i / sum w_i.  q is replicated.  No other exchange exists
on this path, so the NCCL all-gather (latency-bound at this size) is the only collective.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

PAGE_TOKENS = 256  # shard boundaries fall on the reference's page size (kv_cache.rs:477)


def shard_bounds(length: int, n_shards: int, page: int = PAGE_TOKENS) -> List[Tuple[int, int]]:
    """[start, end) token ranges of `n_shards` contiguous shards of a context of `length` tokens.

    Boundaries are multiples of `page`; pages are dealt as evenly as possible, earlier shards take the
    remainder, trailing shards may be empty when there are fewer pages than shards."""
    if length < 0 or n_shards <= 0 or page <= 0:
        raise ValueError("shard_bounds: length >= 0, n_shards > 0, page > 0 required")
    n_pages = (length + page - 1) // page
    base, rem = divmod(n_pages, n_shards)
    out, start = [], 0
    for i in range(n_shards):
        pages = base + (1 if i < rem else 0)
        end = min(length, start + pages * page)
        out.append((start, end))
        start = end
    return out


def balance_sequences(lengths: Sequence[int], n_ranks: int) -> List[List[int]]:
    """Deal sequences (by index) to `n_ranks` GPUs for batched decode: the same number of sequences per rank (the batch
    per GPU is fixed) and cached-token sums as equal as a longest-first greedy makes them, since a decode step costs its
    rank the sum of its context lengths.  Deterministic; returns the index lists, rank by rank.

    Sequences are independent on this path (each has its own cache, architectures/llama.rs:776-781), so the
    assignment is free and needs no collective."""
    n = len(lengths)
    if n_ranks <= 0 or n % n_ranks != 0:
        raise ValueError("balance_sequences: the number of sequences must be a positive multiple of n_ranks")
    per_rank = n // n_ranks
    order = sorted(range(n), key=lambda i: (-lengths[i], i))
    sums, out = [0] * n_ranks, [[] for _ in range(n_ranks)]
    for i in order:
        r = min((r for r in range(n_ranks) if len(out[r]) < per_rank), key=lambda r: (sums[r], r))
        out[r].append(i)
        sums[r] += lengths[i]
    return [sorted(ix) for ix in out]


def partition_units(n_seqs: int, n_head_groups: int, n_ranks: int) -> List[List[Tuple[int, int, int]]]:
    """Deal the independent units of prefill and of the gated-DeltaNet layers to `n_ranks` GPUs with no data-path
    collective: causal prefill is independent per (sequence, kv head) (architectures/llama.rs:776-781: every sequence
    has its own cache; query heads travel with their kv head) and the DeltaNet state per (sequence, value head)
    (qwen3_5.rs:697-699).  Sequences are dealt first; only when there are more ranks than sequences is a sequence's head
    range cut, into equal contiguous groups.

    Returns, rank by rank, a list of (sequence, head_group_begin, head_group_end) with `n_head_groups` groups per
    sequence; every (sequence, group) appears exactly once.  A rank may get nothing when the units do not divide."""
    if n_seqs <= 0 or n_head_groups <= 0 or n_ranks <= 0:
        raise ValueError("partition_units: positive counts required")
    out: List[List[Tuple[int, int, int]]] = [[] for _ in range(n_ranks)]
    if n_ranks <= n_seqs:
        for s in range(n_seqs):
            out[s % n_ranks].append((s, 0, n_head_groups))
        return out
    per_seq = max(1, min(n_head_groups, n_ranks // n_seqs))  # ranks that share one sequence
    while n_head_groups % per_seq != 0:
        per_seq -= 1
    width = n_head_groups // per_seq
    for s in range(n_seqs):
        for j in range(per_seq):
            r = s * per_seq + j
            if r < n_ranks:
                out[r].append((s, j * width, (j + 1) * width))
            else:  # more units than ranks after rounding: wrap around
                out[r % n_ranks].append((s, j * width, (j + 1) * width))
    return out


def pack_partial(o: torch.Tensor, lse: torch.Tensor) -> torch.Tensor:
    """(o [B,Hq,D], lse [B,Hq]) -> one [B,Hq,D+1] fp32 message, so a step is a single all-gather."""
    return torch.cat([o, lse.unsqueeze(-1)], dim=-1).contiguous()


def unpack_partials(msgs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[P,B,Hq,D+1] -> (o_parts [P,B,Hq,D], lse_parts [P,B,Hq]), contiguous."""
    return msgs[..., :-1].contiguous(), msgs[..., -1].contiguous()


def all_gather_partials(o: torch.Tensor, lse: torch.Tensor, group: Optional[dist.ProcessGroup] = None
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gather every rank's (o, lse); works on any backend (NCCL on GPUs, gloo in the CPU tests)."""
    world = dist.get_world_size(group)
    msg = pack_partial(o, lse)
    buf = torch.empty(world * msg.numel(), dtype=msg.dtype, device=msg.device)  # flat: the form every backend accepts
    dist.all_gather_into_tensor(buf, msg.reshape(-1), group=group)
    return unpack_partials(buf.reshape((world,) + tuple(msg.shape)))


class ShardedDecoder:
    """Decode over a KV-length-sharded cache with nothing allocated or repacked per step.

    The local decode writes its shard result straight into one flat fp32 message [o (B*Hq*D) | lse (B*Hq)]; one
    all-gather brings every rank's message into `gathered`; the merge kernel reads the parts where they landed
    (hs_attn_merge_partials_strided).  Per step: one decode launch, one collective, one merge launch."""

    def __init__(self, n_seqs: int, n_q_heads: int, head_dim: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        from . import ops

        self.n_seqs, self.hq, self.d, self.group = n_seqs, n_q_heads, head_dim, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        rows = n_seqs * n_q_heads
        self.msg = torch.empty(rows * (head_dim + 1), dtype=torch.float32, device=device)
        self.o = self.msg[:rows * head_dim].view(n_seqs, n_q_heads, head_dim)
        self.lse = self.msg[rows * head_dim:].view(n_seqs, n_q_heads)
        self.gathered = torch.empty(self.world * self.msg.numel(), dtype=torch.float32, device=device)
        self.out = torch.empty(n_seqs, n_q_heads, head_dim, dtype=torch.bfloat16, device=device)
        self.ws = ops.decode_workspace(n_seqs, n_q_heads, head_dim, device)

    def step(self, q: torch.Tensor, local_view, local_lens: torch.Tensor, softmax_scale: Optional[float] = None,
             gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        from . import ops

        ops.decode_attention(q, local_view, local_lens, softmax_scale=softmax_scale, shard=True, shard_out=(self.o, self.lse),
                             workspace=self.ws)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.msg, group=self.group)
            src = self.gathered
        else:
            src = self.msg
        return ops.merge_gathered(src, self.world, self.n_seqs, self.hq, self.d, out=self.out, gate=gate)


def exchange_handles(handle: bytes, group: Optional[dist.ProcessGroup] = None) -> bytes:
    """All-gather one fixed-size byte string per rank (a CUDA IPC handle) over any backend; returns them concatenated
    in rank order.  Host set-up of FusedShardedDecoder, once per process."""
    world = dist.get_world_size(group)
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    mine = torch.frombuffer(bytearray(handle), dtype=torch.uint8).to(dev)
    buf = torch.empty(world * len(handle), dtype=torch.uint8, device=dev)
    dist.all_gather_into_tensor(buf, mine, group=group)
    return bytes(buf.cpu().numpy().tobytes())


class FusedShardedDecoder:
    """KV-length-sharded decode as ONE launch per GPU and step (hs_attn_decode_sharded): the decode kernel stores its
    shard's (o, lse) into every rank's inbox over NVLink, waits - bounded - for the others' and merges.  The process
    group is used once, at set-up, to exchange the inboxes' IPC handles; no collective runs per step.  Every rank must
    call ``step`` the same number of times."""

    def __init__(self, n_seqs: int, n_q_heads: int, head_dim: int, device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 wait_ms: Optional[int] = None):
        import ctypes

        from . import ffi, ops

        self.n_seqs, self.hq, self.d = n_seqs, n_q_heads, head_dim
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._h = ctypes.c_void_p()
        with torch.cuda.device(device):
            ffi.check(ffi.lib.hs_shard_group_create(self.rank, self.world, n_seqs, n_q_heads, head_dim, ctypes.byref(self._h)))
            if self.world > 1:
                hb = ffi.lib.hs_shard_group_handle_bytes()
                mine = ctypes.create_string_buffer(hb)
                ffi.check(ffi.lib.hs_shard_group_export(self._h, mine))
                handles = exchange_handles(mine.raw, group)
                ffi.check(ffi.lib.hs_shard_group_connect(self._h, handles))
            if wait_ms is not None:
                ffi.check(ffi.lib.hs_shard_group_set_wait_ms(self._h, wait_ms))
        self.out = torch.empty(n_seqs, n_q_heads, head_dim, dtype=torch.bfloat16, device=device)
        self.ws = ops.decode_workspace(n_seqs, n_q_heads, head_dim, device)

    def step(self, q: torch.Tensor, local_view, local_lens: torch.Tensor, softmax_scale: Optional[float] = None,
             gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        import ctypes
        import math

        from . import ffi

        scale = 1.0 / math.sqrt(self.d) if softmax_scale is None else softmax_scale
        ffi.check(ffi.lib.hs_attn_decode_sharded(self._h, q.data_ptr(), ctypes.byref(local_view), local_lens.data_ptr(), self.n_seqs, self.hq,
                                                 scale, self.out.data_ptr(), None if gate is None else gate.data_ptr(), self.ws.data_ptr(),
                                                 self.ws.numel(), 0, torch.cuda.current_stream().cuda_stream))
        return self.out

    def __del__(self):
        if getattr(self, "_h", None):
            from . import ffi

            ffi.lib.hs_shard_group_destroy(self._h)
            self._h = None


def sharded_decode(q: torch.Tensor, local_view, local_lens: torch.Tensor, softmax_scale: Optional[float] = None,
                   gate: Optional[torch.Tensor] = None, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Decode attention over a KV-length-sharded cache: local shard -> all-gather -> LSE merge.

    `local_view`/`local_lens` describe this rank's slice (lengths may be 0: such a shard contributes lse = -inf).
    Every rank returns the same bf16 [B, Hq, D]."""
    from . import ops

    o, lse = ops.decode_attention(q, local_view, local_lens, softmax_scale=softmax_scale, shard=True)
    o_parts, lse_parts = all_gather_partials(o, lse, group)
    return ops.merge_partials(o_parts, lse_parts, gate=gate)
