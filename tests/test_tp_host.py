"""CPU tests of the tensor-parallel host logic: shard arithmetic, and the communicator-id exchange run as
world_size-2 `gloo` ranks (the same code path `bench.py` takes under torchrun, with a fake id maker)."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_shards_tile_every_tensor_exactly_once(pkg, tp):
    from oneiron_luminal_b200 import tp as T
    d = pkg.CONFIGS["llama3_8b_q8"]
    T.validate(d, tp)
    for slot in ("q", "k", "v", "o", "gate", "up", "down", "lm_head", "embed", "attn_norm"):
        n, k = T.full_shape(d, slot)
        seen = set()
        for r in range(tp):
            s = T.shard_of(d, slot, tp, r)
            cell = (s["row0"], s["rows"], s["col0"], s["cols"])
            if slot in T.ROW_SHARDED + T.COL_SHARDED:
                assert cell not in seen
            seen.add(cell)
        rows = sum(c[1] for c in seen) if slot in T.ROW_SHARDED else n
        cols = sum(c[3] for c in seen) if slot in T.COL_SHARDED else k
        assert (rows, cols) == (n, k)
    # whole heads per rank, whole Q8_0 blocks per K-shard
    assert T.shard_of(d, "q", tp, 0)["rows"] % d.head_dim == 0
    assert T.shard_of(d, "down", tp, tp - 1)["cols"] % 32 == 0


def test_validate_rejects_uneven_splits(pkg):
    from oneiron_luminal_b200 import tp as T
    d = pkg.CONFIGS["llama3_8b_q8"]
    with pytest.raises(ValueError):
        T.validate(d, 3)
    with pytest.raises(ValueError):
        T.validate(d, 16)     # 8 KV heads
    with pytest.raises(ValueError):
        T.shard_of(d, "q", 2, 2)


def test_unique_id_exchange_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        from __graft_entry__ import load_package
        pkg = load_package()
        from oneiron_luminal_b200 import tp as T
        dist.init_process_group("gloo")
        rank = dist.get_rank()
        calls = []
        def make():
            calls.append(1)
            return bytes((7 * i + 3) % 256 for i in range(128))
        got = T.exchange_unique_id(dist, rank, make)
        assert got == bytes((7 * i + 3) % 256 for i in range(128)), got[:8]
        assert len(calls) == (1 if rank == 0 else 0)          # only rank 0 makes the id
        # the peer-memory handles travel the same way: every rank ends with all handles in rank order
        hs = T.exchange_peer_handles(dist, dist.get_world_size(), bytes([rank + 1]) * 64)
        assert hs == [bytes([1]) * 64, bytes([2]) * 64], [h[:2] for h in hs]
        d = pkg.CONFIGS["llama3_8b_q8"]
        s = T.shard_of(d, "down", dist.get_world_size(), rank)
        assert s["col0"] == rank * d.ffn // 2 and s["cols"] == d.ffn // 2
        dist.barrier()
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29617")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29617", str(script)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stdout[-3000:]
    assert r.stdout.count("ok") == 2


def test_expert_parallel_host_helpers(pkg):
    """Which experts a rank holds, and which models / group sizes are refused (no GPU needed)."""
    from oneiron_luminal_b200 import tp as T
    d = pkg.CONFIGS["gpt_oss_20b_q8"]
    assert list(T.local_experts(d, 8, 3)) == [12, 13, 14, 15]
    assert list(T.local_experts(d, 1, 0)) == list(range(32))
    with pytest.raises(ValueError):
        T.validate_ep(d, 5)                                  # 32 experts over 5 ranks
    with pytest.raises(ValueError):
        T.validate_ep(pkg.CONFIGS["llama3_8b_q8"], 2)        # no experts
    with pytest.raises(ValueError):
        T.local_experts(d, 4, 4)


def test_expert_parallel_group_two_gloo_ranks(tmp_path):
    """The group handshake an expert-parallel run makes (communicator id to every rank, every rank its own block of experts),
    as two gloo ranks on CPU."""
    script = tmp_path / "ep_worker.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        from __graft_entry__ import load_package
        pkg = load_package()
        from oneiron_luminal_b200 import tp as T
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        d = pkg.CONFIGS["small_oss"]
        T.validate_ep(d, world)
        uid = T.exchange_unique_id(dist, rank, lambda: bytes(range(128)))
        assert uid == bytes(range(128))
        mine = list(T.local_experts(d, world, rank))
        got = [None] * world
        dist.all_gather_object(got, mine)
        assert sorted(sum(got, [])) == list(range(d.n_experts))            # every expert on exactly one rank
        shard = d.copy(ep_size=world, ep_rank=rank)
        assert (shard.ep_size, shard.ep_rank, shard.tp_size) == (world, rank, 1)
        dist.barrier()
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29619")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29619", str(script)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stdout[-3000:]
    assert r.stdout.count("ok") == 2
