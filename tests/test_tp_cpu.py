"""Tensor-parallel host logic on CPU ranks (gloo, world size 2): the plan covers
every head/row exactly once, the NCCL id reaches every rank, and the split the
library uses - whole rows quantised first, column-split q/k/v/gate/up, row-split
o/down with whole-row scales, partial sums all-reduced - reproduces the unsharded
int8 projection (checked with the oracle's int8 matvec on the shards)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from oracle import pi_oracle as orc
    from paged_infer_b200.loader import LlamaConfig
    from paged_infer_b200.tp import exchange_unique_id, shard_plan

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ident = exchange_unique_id(lambda: bytes(range(128)), dist)
        assert ident == bytes(range(128))
        cfg = LlamaConfig(hidden_size=256, num_hidden_layers=1, num_attention_heads=8, num_key_value_heads=2,
                          intermediate_size=384, vocab_size=64)
        plan = shard_plan(cfg, rank, world)
        rng = np.random.default_rng(0)                       # same weights on every rank
        w_up = (rng.standard_normal((384, 256)) * 0.02).astype(np.float32)     # column split (rows)
        w_down = (rng.standard_normal((256, 384)) * 0.02).astype(np.float32)   # row split (input columns)
        x = rng.standard_normal(256).astype(np.float32)
        q_up, s_up = orc.quantize_rows_i8(w_up, 384, 256)
        q_dn, s_dn = orc.quantize_rows_i8(w_down, 256, 384)   # FULL rows quantised, then sliced
        rows = plan.ffn_rows
        h_local = orc.matvec_i8(x, q_up[rows.start:rows.stop], s_up[rows.start:rows.stop])
        partial = orc.matvec_i8(h_local, np.ascontiguousarray(q_dn[:, rows.start:rows.stop]), s_dn)
        t = torch.from_numpy(partial.copy())
        dist.all_reduce(t)                                    # the one exchange of a row-split projection
        h_full = orc.matvec_i8(x, q_up, s_up)
        want = orc.matvec_i8(h_full, q_dn, s_dn)
        err = float(np.abs(t.numpy() - want).max())
        gathered = [None] * world
        dist.all_gather_object(gathered, (list(plan.heads), list(plan.kv_heads), list(plan.ffn_rows), list(plan.vocab_rows)))
        if rank == 0:
            for i, n in enumerate((8, 2, 384, 64)):
                assert sorted(sum((g[i] for g in gathered), [])) == list(range(n))
            out.put(("ok", err))
    except Exception as e:  # noqa: BLE001
        if rank == 0:
            out.put(("fail", repr(e)))
        raise
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_agree_on_plan_id_and_split_numerics(oracle):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    status, val = out.get(timeout=120)
    for p in procs:
        p.join(60)
    assert status == "ok", val
    assert val < 1e-5, val   # only the order of the partial sums differs


def test_plan_rejects_what_does_not_split():
    from paged_infer_b200.loader import LlamaConfig
    from paged_infer_b200.tp import shard_plan
    tiny = LlamaConfig()  # TinyLlama: 4 KV heads
    assert list(shard_plan(tiny, 3, 4).kv_heads) == [3]
    with pytest.raises(ValueError):
        shard_plan(tiny, 0, 8)
    with pytest.raises(ValueError):
        shard_plan(tiny, 2, 2)
    with pytest.raises(ValueError):
        shard_plan(tiny, 0, 3)
