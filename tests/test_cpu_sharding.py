"""Multi-rank host logic on CPU (gloo, world_size 2 and 3): batch sharding by sequence + gather reproduces the
single-rank result exactly.  The per-rank compute stands in with the CPU oracle (the product kernels need a GPU);
what is under test is the sharding and the collective plumbing, and the property that makes sharding exact."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hydra_b200.parallel import gather_rows, shard_batch, shard_bounds


def test_shard_bounds_cover_every_row_once():
    for n in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _worker(rank: int, world: int, port: int, tmp: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import hydra_oracle as O
        torch.set_num_threads(1)
        cfg = O.HydraConfig(vocab_size=64, dim=128, n_mor_blocks=3, recursions_per_block=2, n_heads=2, n_kv_heads=1,
                            max_seq_len=24, mod_capacity=0.75)
        w = O.init_params(cfg, seed=0, perturb=True)
        ids = torch.randint(0, 64, (5, 24), generator=torch.Generator().manual_seed(1))   # 5 rows: uneven shards
        mine = shard_batch(ids, rank, world)
        local = O.model_forward(mine, w, cfg)[:, -1, :] if mine.shape[0] else torch.zeros(0, 64)
        full = gather_rows(local, ids.shape[0])
        if rank == 0:
            ref = O.model_forward(ids, w, cfg)[:, -1, :]
            torch.save({"full": full, "ref": ref}, tmp)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_forward_plus_gather_equals_single_rank(world, tmp_path):
    port = 29500 + (os.getpid() % 2000) + world
    out = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    r = torch.load(out)
    assert r["full"].shape == r["ref"].shape
    assert torch.allclose(r["full"], r["ref"], atol=1e-6, rtol=0), "sharding by sequence must not change any row"
