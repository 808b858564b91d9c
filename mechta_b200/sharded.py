"""Sequence sharding of one long context over the ranks of a torch.distributed job (one process per GPU),
and placement of independent sessions on GPUs.

The reference runs on one GPU; it already splits attention over blocks of positions inside the GPU and merges
un-normalised partials [m, l, O] by log-sum-exp (ops.wgsl:523-538). A rank is treated as one more level of that
split: it owns the contiguous rows [rank * L / n, (rank + 1) * L / n), computes the record of the step over its
rows, the records are exchanged (an all-gather of 66 KB per rank) and every rank merges them.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import kv


def shard_range(context: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous equal chunks; `context / world` must be a multiple of 64 (the attention tile)."""
    per = context // world
    if per * world != context or per % 64 != 0:
        raise ValueError(f"context {context} does not split into {world} shards of a multiple of 64 rows")
    return rank * per, per


def gather_records(rec: torch.Tensor, recs: torch.Tensor, group=None) -> None:
    """All-gather of the per-rank records [64][258] into recs [world][64][258] (rank order = shard order)."""
    dist.all_gather_into_tensor(recs.view(-1), rec.view(-1), group=group)


class ShardPlan:
    """Which rows a rank holds and who owns a position; no device needed."""

    def __init__(self, context: int, world: int, rank: int):
        self.context, self.world, self.rank = kv.check_ctx(context), world, rank
        self.first, self.per = shard_range(self.context, world, rank)

    def owner_of(self, pos: int) -> int:
        return min(pos // self.per, self.world - 1)

    def rows_of_append(self, pos: int, ntok: int) -> range:
        """The positions of an append at `pos` that this rank stores."""
        lo, hi = max(pos, self.first), min(pos + ntok, self.first + self.per)
        return range(lo, max(lo, hi))


class ShardedKvCache:
    """This rank's shard of a sequence-sharded KV cache plus the exchange step of its attention.

    `group` is a torch.distributed process group (NCCL on GPUs; gloo works for CPU-side tests of the
    bookkeeping). Every rank makes the same calls with the same arguments (q, k, v are replicated: they come
    from the token's hidden state, which every rank holds).
    """

    def __init__(self, ctx: kv.KvContext, fmt: kv.KvFormat, n_layers: int, context: int, group=None, exchange: str = "p2p"):
        """exchange = "p2p": the attention kernel pushes its record into every rank's mailbox (CUDA IPC, NVLink
        stores); "nccl": all-gather of the records through torch.distributed, then the merge kernel."""
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.plan = ShardPlan(context, self.world, self.rank)
        self.first, self.per = self.plan.first, self.plan.per
        self.ctx = ctx
        self.cache = kv.KvCache(ctx, fmt, n_layers, context, shard_first=self.first,
                                shard_tokens=self.per if self.world > 1 else 0)
        dev = f"cuda:{ctx.device}"
        self.recs = torch.empty(self.world, 64, 258, device=dev)  # gathered records, one per rank
        self.rec = torch.empty(64, 258, device=dev)
        self.exchange = None
        if exchange == "p2p" and self.world > 1:
            def gather(mine: bytes):
                got = [None] * self.world
                dist.all_gather_object(got, mine, group=group)
                return got
            self.exchange = kv.KvExchange(ctx, self.rank, self.world, gather)

    def owner_of(self, pos: int) -> int:
        return self.plan.owner_of(pos)

    def append_layers(self, pos, k, v, tab):
        """Every rank calls this; only rows inside the rank's shard are written (appends go to the owner)."""
        self.cache.append_layers(pos, k, v, tab)

    def append(self, layer, pos, k, v, tab):
        self.cache.append(layer, pos, k, v, tab)

    def truncate(self, new_len: int):
        self.cache.truncate(min(new_len, len(self.cache)))

    def attn_verify(self, layer: int, first_pos: int, pos: int, q: torch.Tensor, out: torch.Tensor) -> None:
        """Local record -> all-gather over NVLink -> log-sum-exp merge on every rank."""
        if self.world == 1:
            self.cache.attn_verify(layer, first_pos, pos, q, out)
            return
        if self.exchange is not None:
            self.exchange.attn_verify(self.cache, layer, first_pos, pos, q, out)
            return
        self.cache.attn_verify_partial(layer, first_pos, pos, q, self.rec)
        gather_records(self.rec, self.recs, self.group)
        self.ctx.combine_shards(self.recs, q.shape[0], out)

    def close(self):
        if self.exchange is not None:
            self.exchange.close()
        self.cache.close()


def place_sessions(kv_bytes: list[int], n_gpus: int) -> list[list[int]]:
    """Greedy longest-processing-time placement of sessions on GPUs, balanced by KV bytes.
    Returns, per GPU, the indices of its sessions."""
    order = sorted(range(len(kv_bytes)), key=lambda i: -kv_bytes[i])
    load = [0] * n_gpus
    out: list[list[int]] = [[] for _ in range(n_gpus)]
    for i in order:
        g = min(range(n_gpus), key=lambda j: (load[j], j))
        out[g].append(i)
        load[g] += kv_bytes[i]
    return out
