"""Tensor parallelism on two GPUs of one box (skipped where fewer are visible):
each rank keeps its shard of the int8 weights and of the KV pool, the row-split
projections are followed by one NCCL all-reduce, and the logits must agree with
the single-GPU run of the same model within 1e-4 (only the summation order of the
partial sums differs) and with the CPU oracle within 1e-3.  The same with the
exchange done by the library's own kernels over peer memory instead of NCCL: the
row-split projection pushes its partial sums into every rank's buffer from its epilogue
(plain peer stores) and one kernel per exchange waits for the arrival flags and adds
them up with the residual folded in ("peer-push"), or that kernel fetches the peers'
partial sums itself with P2P loads ("peer-pull").  Two geometries: head_dim
64 with kv_group 4, and the Llama-3 / Llama-2-70B one - head_dim 128, kv_group 4,
ONE KV head per rank.  On a single GPU: a peer that never delivers its partial
sums makes the bounded wait run out, the call reports PI_ERR_TIMEOUT and the
context stays usable (no kernel traps or spins for ever)."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BLOCK = 16


GEOMETRIES = {
    "hd64": dict(layers=2, hidden=512, heads=8, kv_heads=2, inter=1408, vocab=1000),
    "hd128-one-kv-head-per-rank": dict(layers=2, hidden=1024, heads=8, kv_heads=2, inter=3584, vocab=1024),
}


def _worker(rank, world, port, out, peer, geom):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from oracle import pi_oracle as orc
    from paged_infer_b200 import api
    from paged_infer_b200.tp import enable_peer_exchange, exchange_unique_id
    from test_gpu_model import kv_floats, small_llama

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ident = exchange_unique_id(api.nccl_unique_id, dist)
        ctx = api.Context(rank, rank=rank, tp=world, nccl_id=ident)
        if peer:
            enable_peer_exchange(ctx, 64 * GEOMETRIES[geom]["hidden"], dist)       # max batch rows x hidden
            if peer == "pull":   # the exchange kernel fetches the peers' partial sums itself (default: the projections push them)
                ctx.set_option(api._lib.PI_OPT_TP_PUSH, 0)
        cfg, om, gm = small_llama(ctx, orc, 9, **GEOMETRIES[geom])   # 8 heads / 2 KV heads -> one KV head per rank
        rng = np.random.default_rng(9)
        B, nblocks = 6, 8
        lens = [int(x) for x in rng.integers(5, 100, B)]
        tables = [[b * nblocks + i for i in range(nblocks)] for b in range(B)]
        kv = api.KvCache(ctx, gm.kv_layout(B * nblocks, BLOCK))
        assert kv.layout.num_kv_heads == cfg.num_key_value_heads // world
        prompts = [rng.integers(0, cfg.vocab_size, n).astype(np.uint32) for n in lens]
        last = [gm.prefill_batched(p, 0, t, kv, 16) for p, t in zip(prompts, tables)]
        tok = [int(np.argmax(l)) for l in last]
        logits, ids = gm.decode_batch_into(tok, lens, tables, kv, want_argmax=True)
        multi = gm.decode_multi(tok, lens, tables, kv, 5)             # overwrites position lens[b] with the same values
        if rank == 0:
            # the same model on one GPU, and on the CPU oracle
            c1 = api.Context(0)
            _, _, g1 = small_llama(c1, orc, 9, **GEOMETRIES[geom])
            kv1 = api.KvCache(c1, g1.kv_layout(B * nblocks, BLOCK))
            okv = np.zeros(kv_floats(cfg, B * nblocks), np.float32)
            for p, t in zip(prompts, tables):
                g1.prefill_batched(p, 0, t, kv1, 16)
                om.prefill_batched(p, 0, t, okv, BLOCK, 16)
            l1, i1 = g1.decode_batch_into(tok, lens, tables, kv1, want_argmax=True)
            m1 = g1.decode_multi(tok, lens, tables, kv1, 5)
            lo = om.decode_batch(tok, lens, tables, okv, BLOCK)
            out.put(("ok", float(np.abs(logits - l1).max()), float(np.abs(logits - lo).max()),
                     ids.tolist() == i1.tolist(), multi.tolist() == m1.tolist()))
        dist.barrier()
    except Exception as e:  # noqa: BLE001
        if rank == 0:
            out.put(("fail", repr(e)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("geom", list(GEOMETRIES))
@pytest.mark.parametrize("peer", [False, "push", "pull"], ids=["nccl", "peer-push", "peer-pull"])
def test_tp2_matches_single_gpu_and_oracle(peer, geom):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29700 + os.getpid() % 2000 + 3 * list(GEOMETRIES).index(geom)
    procs = [ctx.Process(target=_worker, args=(r, 2, port + [False, "push", "pull"].index(peer), out, peer, geom)) for r in range(2)]
    for p in procs:
        p.start()
    res = out.get(timeout=600)
    for p in procs:
        p.join(120)
    assert res[0] == "ok", res
    _, d_single, d_oracle, same_ids, same_multi = res
    assert d_single < 1e-4 and d_oracle < 1e-3 and same_ids and same_multi, res


def test_a_peer_that_never_delivers_ends_in_a_timeout_not_a_hang():
    """Rank 0 of a two-rank group whose second rank's buffer exists (a second context on the same GPU) but whose
    owner never runs a step: nothing ever raises the arrival flag.  With the wait budget lowered, the exchange
    kernel gives up, skips the add and returns; the next synchronising call reports PI_ERR_TIMEOUT; the context
    still computes afterwards, and the peer path is retired so that no later step trusts the out-of-step slots.
    Only the waiting side runs: there is no second kernel on this GPU that the first one waits for."""
    import torch

    from paged_infer_b200 import _lib, api

    c0 = api.Context(0, rank=0, tp=2)        # no NCCL id: the peer-memory exchange is the only one
    c1 = api.Context(0, rank=1, tp=2)
    rows, cols = 8, 512
    c0.tp_peer_export(rows * cols)
    c1.tp_peer_export(rows * cols)
    c0.tp_peer_import_pointers([c0.tp_peer_base(), c1.tp_peer_base()])
    c0.set_option(_lib.PI_OPT_PEER_SPIN_LIMIT, 2000)
    x = torch.ones(rows, cols, device="cuda")
    part = torch.full((rows, cols), 2.0, device="cuda")
    torch.cuda.synchronize()
    c0.tp_exchange_add(part, x, rows, cols)
    with pytest.raises(api.PiError) as err:
        c0.synchronize()
    assert err.value.status == _lib.PI_ERR_TIMEOUT and "peer" in err.value.message
    assert bool((x == 1.0).all())                              # the add was skipped, not done with missing terms
    c0.synchronize()                                           # the error word was cleared: the context works on
    q = np.ones((64, 256), np.int8)
    lin = api.Projection.int8(c0, q, np.full(64, 0.5, np.float32))
    got = lin.apply_batched(np.ones((2, 256), np.float32))
    assert np.array_equal(got, np.full((2, 64), 128.0, np.float32))
    with pytest.raises(api.PiError, match="no NCCL communicator"):
        c0.tp_exchange_add(part, x, rows, cols)                # the peer path is retired after a timeout
    lin.close()
    c0.close()
    c1.close()
