"""The multi-rank host logic on CPU: shard plan, gather order of the records and the merge, with world_size 2 and 4
gloo ranks. The records themselves come from the oracle here (there is no GPU); on GPUs they come from
mkv_attn_verify_partial, which tests/test_gpu_kv.py checks against the same oracle records."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mechta_b200 import sharded, synth


def test_shard_plan_and_owner():
    for world in (1, 2, 4, 8):
        covered = []
        for r in range(world):
            p = sharded.ShardPlan(262144, world, r)
            assert p.per == 262144 // world and p.first == r * p.per
            covered.append((p.first, p.first + p.per))
            assert p.owner_of(p.first) == r and p.owner_of(p.first + p.per - 1) == r
        assert covered[0][0] == 0 and covered[-1][1] == 262144
        assert all(covered[i][1] == covered[i + 1][0] for i in range(world - 1))
    p = sharded.ShardPlan(8192, 4, 1)
    assert list(p.rows_of_append(2046, 4)) == [2048, 2049]  # an append that straddles two shards
    assert list(p.rows_of_append(100, 4)) == [] and list(p.rows_of_append(4094, 4)) == [4094, 4095]
    with pytest.raises(ValueError):
        sharded.shard_range(4096, 3, 0)  # does not split evenly
    with pytest.raises(ValueError):
        sharded.shard_range(5120, 32, 0)  # 160 rows per shard: not a multiple of the 64-row tile

def test_place_sessions_balances_kv_bytes():
    lens = synth.session_lengths(3, 32)
    byts = [int(n) * 2048 * 10 for n in lens]
    place = sharded.place_sessions(byts, 8)
    assert sorted(i for g in place for i in g) == list(range(32))
    loads = [sum(byts[i] for i in g) for g in place]
    assert max(loads) / (sum(loads) / 8) < 1.15  # greedy longest-first is within a few percent here
    assert sharded.place_sessions([5, 1, 1], 2) == [[0], [1, 2]]


def _rank_main(rank, world, port, total, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle
    fmt, pos = 1, total - 4
    plan = sharded.ShardPlan(total, world, rank)
    # every rank sees every append and keeps its own rows, as ShardedKvCache.append_layers does
    kc, vc = oracle.new_cache(fmt, plan.per), oracle.new_cache(fmt, plan.per)
    for p0 in range(0, total, 512):
        k, v = synth.normal(9, synth.S_K, p0, (512, 2, 256)), synth.normal(9, synth.S_V, p0, (512, 2, 256))
        tab = oracle.rope_tables(p0, 512)
        rows = plan.rows_of_append(p0, 512)
        if len(rows):
            a, b = rows[0] - p0, rows[-1] + 1 - p0
            oracle.append(fmt, kc, vc, rows[0] - plan.first, k[a:b], v[a:b], tab[a:b])
    q = synth.normal(9, synth.S_Q, 0, (4, 16, 256))
    rec = torch.from_numpy(oracle.attn_shard_partial(fmt, kc, vc, plan.first, plan.first, plan.first + plan.per, 0, pos, q))
    recs = torch.empty(world, 64, 258)
    sharded.gather_records(rec, recs)
    out = oracle.combine_shards(recs.numpy()).reshape(4, 16, 256)
    if rank == world - 1:
        np.save(ret, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_step_over_gloo_equals_unsharded(world, tmp_path, oracle):
    total = 4096
    ret = str(tmp_path / "out.npy")
    port = 29000 + (os.getpid() + world) % 2000
    mp.spawn(_rank_main, args=(world, port, total, ret), nprocs=world, join=True)
    got = np.load(ret)
    kc, vc = oracle.new_cache(1, total), oracle.new_cache(1, total)
    for p0 in range(0, total, 512):
        oracle.append(1, kc, vc, p0, synth.normal(9, synth.S_K, p0, (512, 2, 256)), synth.normal(9, synth.S_V, p0, (512, 2, 256)),
                      oracle.rope_tables(p0, 512))
    want = oracle.attn_ref_f32(1, kc, vc, 0, total - 4, synth.normal(9, synth.S_Q, 0, (4, 16, 256)))
    assert oracle.max_rel(got, want) < 2e-6
