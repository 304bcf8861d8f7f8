"""The N > 1 path on CPU: two gloo ranks shard the environments contiguously, run their
shard with no data-path collective, and the pieces put together equal the single-rank result
to float32 rounding (environments are independent).  The arithmetic here is the CPU oracle; the
point of the test is the sharding and reduction logic that bench.py uses on GPUs."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import boost_and_broadside_b200 as bnb
        from boost_and_broadside_b200 import sharding
        from boost_and_broadside_b200 import workloads as W
        from oracle import trunk_oracle as O

        torch.set_num_threads(2)
        torch.manual_seed(0)
        trunk = bnb.YemongTrunk(W.rl_config()).eval()
        P = O.split_trunk_state_dict(trunk.state_dict())
        results = {}
        # uniform step
        w = W.c2(n_envs=37, seed=11)
        s = sharding.shard_workload(w, rank, world)
        results["c2"] = O.trunk_step(s.x, s.alive, s.hidden, P, 4, "fp32")
        # uniform step with bullet tokens: the bullets follow their environments
        w = W.c2b(n_envs=11, seed=14, bullets_per_env=9)
        s = sharding.shard_workload(w, rank, world)
        assert s.bullets.shape[0] == s.x.shape[0] == s.bullet_mask.shape[0]
        results["c2b"] = O.trunk_step(s.x, s.alive, s.hidden, P, 4, "fp32", s.bullets, s.bullet_mask)
        # sequence with done flags
        w = W.c4(n_envs=5, timesteps=4, seed=12)
        s = sharding.shard_workload(w, rank, world)
        results["c4"] = O.trunk_sequence(s.x, s.alive, s.hidden, s.done, P, 4, "fp32")
        # ragged
        w = W.c5(n_envs=21, seed=13, max_tokens=20)
        s = sharding.shard_workload(w, rank, world)
        results["c5"] = O.trunk_step_ragged(s.x, s.alive, s.hidden, s.n_tokens.tolist(), s.n_ships.tolist(), P, 4, "fp32")
        torch.save(results, os.path.join(out_dir, f"rank{rank}.pt"))
        # reduction used for the timing: every rank must see the slowest rank's time
        t = sharding.max_over_ranks(10.0 + rank)
        assert t == 10.0 + world - 1
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_env_shard_ranges():
    from boost_and_broadside_b200.sharding import env_shard

    for n, world in ((16384, 8), (37, 2), (5, 4), (3, 8)):
        ranges = [env_shard(n, r, world) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        sizes = [hi - lo for lo, hi in ranges]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        env_shard(4, 2, 2)


# The shards run the same float32 arithmetic on smaller batches: the CPU matmul blocks its sums
# differently for a different batch size, so the comparison is to float32 rounding of O(1)
# activations, not to the bit.
SHARD_ATOL = 5e-5


def test_two_ranks_reproduce_the_single_rank_result(tmp_path):
    import boost_and_broadside_b200 as bnb
    from boost_and_broadside_b200 import workloads as W
    from oracle import trunk_oracle as O

    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.start_processes(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]

    torch.set_num_threads(4)
    torch.manual_seed(0)
    trunk = bnb.YemongTrunk(W.rl_config()).eval()
    P = O.split_trunk_state_dict(trunk.state_dict())

    w = W.c2(n_envs=37, seed=11)
    y, h = O.trunk_step(w.x, w.alive, w.hidden, P, 4, "fp32")
    assert torch.allclose(torch.cat([p["c2"][0] for p in parts]), y, atol=SHARD_ATOL)
    assert torch.allclose(torch.cat([p["c2"][1] for p in parts], dim=1), h, atol=SHARD_ATOL)

    w = W.c2b(n_envs=11, seed=14, bullets_per_env=9)
    y, h = O.trunk_step(w.x, w.alive, w.hidden, P, 4, "fp32", w.bullets, w.bullet_mask)
    assert torch.allclose(torch.cat([p["c2b"][0] for p in parts]), y, atol=SHARD_ATOL)
    assert torch.allclose(torch.cat([p["c2b"][1] for p in parts], dim=1), h, atol=SHARD_ATOL)

    w = W.c4(n_envs=5, timesteps=4, seed=12)
    y, h = O.trunk_sequence(w.x, w.alive, w.hidden, w.done, P, 4, "fp32")
    assert torch.allclose(torch.cat([p["c4"][0] for p in parts], dim=1), y, atol=SHARD_ATOL)
    assert torch.allclose(torch.cat([p["c4"][1] for p in parts], dim=1), h, atol=SHARD_ATOL)

    w = W.c5(n_envs=21, seed=13, max_tokens=20)
    y, h = O.trunk_step_ragged(w.x, w.alive, w.hidden, w.n_tokens.tolist(), w.n_ships.tolist(), P, 4, "fp32")
    assert torch.allclose(torch.cat([p["c5"][0] for p in parts]), y, atol=SHARD_ATOL)
    assert torch.allclose(torch.cat([p["c5"][1] for p in parts], dim=1), h, atol=SHARD_ATOL)
