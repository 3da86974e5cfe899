"""World-size-2 (and 3) CPU runs of the sharding host logic over gloo; the kernel is replaced by the oracle."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from general_ai_compiler_b200.distributed import dcn_units, query_block, unit_block  # noqa: E402


def test_partitions_are_balanced_and_cover():
    for total in (0, 1, 7, 10000, 10001):
        for world in (1, 2, 3, 4, 8):
            blocks = [unit_block(total, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
            sizes = [e - b for b, e in blocks]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        unit_block(10, 2, 2)
    assert query_block(10000, 8, 3) == (3750, 5000)


def test_dcn_units_keep_every_rank_busy():
    for world in (1, 2, 4, 8):
        units = dcn_units(6, 58, world)
        assert len(units) % world == 0 or world == 1
        covered = sorted((n, r) for n, r0, r1 in units for r in range(r0, r1))
        assert covered == [(n, r) for n in range(6) for r in range(58)]
    assert dcn_units(6, 58, 2) == [(n, 0, 58) for n in range(6)]       # cameras divide evenly: whole cameras
    assert len(dcn_units(6, 58, 4)) == 12 and len(dcn_units(6, 58, 8)) == 24


def test_dcn_rank_pieces_cover_once_and_balance():
    from general_ai_compiler_b200.distributed import dcn_rank_pieces

    for cameras, rows in ((6, 58), (6, 29), (3, 19), (1, 7)):
        for world in (1, 2, 3, 4, 8):
            per_rank = [dcn_rank_pieces(cameras, rows, world, r) for r in range(world)]
            covered = sorted((n, r) for pieces in per_rank for n0, n1, r0, r1 in pieces
                             for n in range(n0, n1) for r in range(r0, r1))
            assert covered == [(n, r) for n in range(cameras) for r in range(rows)], (cameras, rows, world)
            for pieces in per_rank:
                assert all(isinstance(v, int) for p in pieces for v in p)
                # an image range longer than one camera always spans whole planes
                assert all((n1 - n0 == 1) or (r0 == 0 and r1 == rows) for n0, n1, r0, r1 in pieces)
    load = [sum((n1 - n0) * (r1 - r0) for n0, n1, r0, r1 in dcn_rank_pieces(6, 58, 8, r)) for r in range(8)]
    assert max(load) - min(load) <= 6                                     # rows; the camera split leaves two ranks idle
    assert dcn_rank_pieces(6, 58, 2, 1) == [(3, 6, 0, 58)]


def test_dcn_pixel_blocks_are_contiguous_and_tile_aligned():
    from general_ai_compiler_b200.distributed import dcn_pixel_block

    for cameras, plane in ((6, 5800), (6, 1450), (3, 513), (1, 7)):
        for world in (1, 2, 3, 4, 8):
            blocks = [dcn_pixel_block(cameras, plane, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == cameras * plane
            assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:])) and all(a <= b for a, b in blocks)
            assert all(b[0] % 128 == 0 or b[0] == cameras * plane for b in blocks)
            sizes = [b[1] - b[0] for b in blocks]
            assert max(sizes) - min(sizes) <= 2 * 128


def test_head_shards_concatenate_to_the_whole_output():
    from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
    from general_ai_compiler_b200.distributed import head_shard
    from oracle import msda_c

    w = WORKLOADS["base_sca"].with_queries(23)
    x = make_workload_inputs(w)
    whole = msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
    for world in (1, 2, 3, 8):
        parts = []
        for rank in range(world):
            v, l, a, (h0, h1) = head_shard(x["value"], x["sampling_locations"], x["attention_weights"], world, rank)
            assert v.shape[2] == h1 - h0 and v.flags.c_contiguous and l.flags.c_contiguous
            if h1 > h0:
                parts.append(msda_c(v, l, a, w.spatial_shapes))
        assert np.array_equal(np.concatenate(parts, axis=2), whole)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, tmp: str) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
        from general_ai_compiler_b200.distributed import broadcast_value, sharded_msda
        from oracle import msda_c

        w = WORKLOADS["base_sca"].with_queries(101)
        x = make_workload_inputs(w)
        value = torch.from_numpy(x["value"]) if rank == 0 else torch.zeros(x["value"].shape)
        ms = broadcast_value(value, src=0)
        assert ms >= 0 and torch.equal(value, torch.from_numpy(x["value"]))

        def compute(v, l, a, shapes):      # stand-in for the CUDA kernel on a CPU-only box
            return torch.from_numpy(msda_c(v.numpy(), l.numpy(), a.numpy(), shapes))

        loc, attn = torch.from_numpy(x["sampling_locations"]), torch.from_numpy(x["attention_weights"])
        block = sharded_msda(value, loc, attn, w.spatial_shapes, compute=compute)
        q0, q1 = query_block(101, world, rank)
        assert block.shape[1] == q1 - q0
        full = sharded_msda(value, loc, attn, w.spatial_shapes, gather=True, compute=compute)
        whole = msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
        assert np.array_equal(full.numpy(), whole)
        assert np.array_equal(block.numpy(), whole[:, q0:q1])
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_query_sharded_msda_over_gloo(world, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == [f"ok{r}" for r in range(world)]


def _sharded_value_worker(rank: int, world: int, port: int, tmp: str) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
        from general_ai_compiler_b200.distributed import ShardedMsda, sharded_msda
        from oracle import msda_c

        # S = 30825 does not divide by 2 or 3 evenly for every level mix; 37 queries leave ragged blocks
        w = WORKLOADS["base_sca"].with_queries(37)
        x = make_workload_inputs(w)
        whole = msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)

        def compute(v, l, a, shapes, out):          # stand-in for the CUDA kernel on a CPU-only box
            out.copy_(torch.from_numpy(msda_c(v.float().numpy(), l.numpy(), a.numpy(), shapes)))

        for replicate in ("all_gather", "broadcast"):
            runner = ShardedMsda(batch=w.batch, spatial_shapes=w.spatial_shapes, queries=w.queries, heads=w.heads,
                                 head_dim=w.head_dim, points=w.points, device="cpu", replicate=replicate, compute=compute)
            assert runner.rows * world >= runner.S and (runner.q0, runner.q1) == query_block(37, world, rank)
            runner.load_host(x["value"], x["sampling_locations"], x["attention_weights"])
            if replicate == "broadcast":
                runner.set_broadcast_source(x["value"])
            # a rank uploads only its rows of value: 1/world of it (rounded up) instead of all of it
            assert runner.host["value_shard"].shape[1] == -(-w.spatial_size // world)
            if replicate == "all_gather":
                out = runner.step()                                   # end to end from the host staging buffers
                assert np.array_equal(out.numpy(), whole[:, runner.q0:runner.q1])
                # every rank now holds the whole value, assembled from the shards, in its own memory
                assert np.array_equal(runner.slabs[:, : runner.S].numpy(), x["value"])
            runner.out.zero_()
            runner.upload()
            runner.step_resident()
            assert np.array_equal(runner.out.numpy(), whole[:, runner.q0:runner.q1]), replicate
        # bf16 on the wire: the gathered slabs are the rounded value, the result is the oracle on that value
        runner = ShardedMsda(batch=w.batch, spatial_shapes=w.spatial_shapes, queries=w.queries, heads=w.heads,
                             head_dim=w.head_dim, points=w.points, device="cpu", value_storage="bfloat16", compute=compute)
        runner.load_host(x["value"], x["sampling_locations"], x["attention_weights"])
        out = runner.step()
        rounded = torch.from_numpy(x["value"]).to(torch.bfloat16).float().numpy()
        want = msda_c(rounded, x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
        assert np.array_equal(out.numpy(), want[:, runner.q0:runner.q1])
        assert runner.wire_bytes_in == (world - 1) * w.batch * runner.rows * w.heads * w.head_dim * 2

        # sharded_msda given a rank-local slice of a stated global query count
        loc, attn = torch.from_numpy(x["sampling_locations"]), torch.from_numpy(x["attention_weights"])
        q0, q1 = query_block(37, world, rank)

        def compute3(v, l, a, shapes):
            return torch.from_numpy(msda_c(v.numpy(), l.numpy(), a.numpy(), shapes))

        full = sharded_msda(torch.from_numpy(x["value"]), loc[:, q0:q1].contiguous(), attn[:, q0:q1].contiguous(),
                            w.spatial_shapes, gather=True, compute=compute3, total_queries=37)
        assert np.array_equal(full.numpy(), whole)
        with pytest.raises(ValueError):
            sharded_msda(torch.from_numpy(x["value"]), loc, attn, w.spatial_shapes, compute=compute3, total_queries=37 * 5)
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_value_arrives_sharded_and_is_all_gathered(world, tmp_path):
    mp.spawn(_sharded_value_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == [f"ok{r}" for r in range(world)]
