"""Host-side helpers for tensor parallelism (one process per GPU of one node).

The library shards the weights itself (``pi_ctx_create_tp``); the host only has
to (1) agree on the sharding plan, (2) ship rank 0's 128-byte NCCL id to the
other ranks, (3) give every rank the same block tables.  The reference has no
multi-device code; the split follows the usual Megatron layout: q/k/v/gate/up
split by output rows (whole heads / FFN rows per rank), o/down split by input
columns with one all-reduce each, LM head split over the vocabulary.
"""
from __future__ import annotations

from dataclasses import dataclass

from .loader import LlamaConfig


@dataclass
class ShardPlan:
    tp: int
    rank: int
    heads: range          # query heads owned by this rank
    kv_heads: range       # KV heads owned (their K/V live in this rank's pool only)
    ffn_rows: range       # gate/up rows == down-projection input columns
    vocab_rows: range     # LM-head rows


def shard_plan(cfg: LlamaConfig, rank: int, tp: int) -> ShardPlan:
    """Validate ``tp`` for this model and return what ``rank`` owns."""
    if tp not in (1, 2, 4, 8) or not 0 <= rank < tp:
        raise ValueError(f"tensor-parallel rank {rank} of {tp} (tp must be 1, 2, 4 or 8)")
    for name, n in (("num_key_value_heads", cfg.num_key_value_heads), ("num_attention_heads", cfg.num_attention_heads),
                    ("intermediate_size", cfg.intermediate_size), ("vocab_size", cfg.vocab_size)):
        if n % tp:
            raise ValueError(f"{name}={n} does not split over {tp} ranks")

    def part(n):
        return range(rank * n // tp, (rank + 1) * n // tp)

    return ShardPlan(tp, rank, part(cfg.num_attention_heads), part(cfg.num_key_value_heads),
                     part(cfg.intermediate_size), part(cfg.vocab_size))


def exchange_unique_id(make_id, dist) -> bytes:
    """Rank 0 calls ``make_id()`` (-> 128 bytes); every rank returns the same bytes.
    ``dist`` is ``torch.distributed`` with an initialised process group (any backend)."""
    import torch

    rank = dist.get_rank()
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        raw = make_id()
        if len(raw) != 128:
            raise ValueError("the NCCL unique id is 128 bytes")
        buf = torch.tensor(list(raw), dtype=torch.uint8)
    if dist.get_backend() == "nccl":
        buf = buf.cuda()
    dist.broadcast(buf, src=0)
    return bytes(buf.cpu().tolist())


def enable_peer_exchange(ctx, max_floats: int, dist) -> None:
    """Set up the peer-memory path for the exchange after the row-split projections: every rank exports a handle
    to its buffers (``max_floats`` = max batch rows x hidden size), the handles are all-gathered over ``dist``
    (``torch.distributed``, any backend) and imported.  Without this call the NCCL all-reduce is used."""
    import torch

    mine = torch.tensor(list(ctx.tp_peer_export(max_floats)), dtype=torch.uint8)
    if dist.get_backend() == "nccl":
        mine = mine.cuda()
    everyone = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(everyone, mine)
    ctx.tp_peer_import([bytes(t.cpu().tolist()) for t in everyone])
