"""Two-GPU checks of the sharded MSDA runner (skipped on a box with one GPU): the value assembled by NCCL
all-gather and by copy-engine peer copies gives, on every rank, the oracle's result for that rank's query block."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, tmp: str) -> None:
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    from general_ai_compiler_b200.distributed import ShardedMsda, nccl_high_priority_options

    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device, pg_options=nccl_high_priority_options())
    log = open(Path(tmp, f"log{rank}.txt"), "w")

    def note(*what):
        print(*what, file=log, flush=True)

    try:
        from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
        from oracle import msda_c

        w = WORKLOADS["base_sca"].with_queries(203)
        x = make_workload_inputs(w)
        whole = msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
        rounded = torch.from_numpy(x["value"]).to(torch.bfloat16).float().numpy()
        whole16 = msda_c(rounded, x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
        for replicate, storage in (("all_gather", "float32"), ("peer_copy", "float32"), ("peer_copy", "bfloat16")):
            note("case", replicate, storage)
            runner = ShardedMsda(batch=w.batch, spatial_shapes=w.spatial_shapes, queries=w.queries, heads=w.heads,
                                 head_dim=w.head_dim, points=w.points, device=device, replicate=replicate, value_storage=storage)
            note("constructed")
            runner.load_host(x["value"], x["sampling_locations"], x["attention_weights"])
            runner.upload()
            want = (whole if storage == "float32" else whole16)[:, runner.q0:runner.q1]
            for attempt in range(3):                       # repeated steps reuse the barriers' step counters
                runner.out.zero_()
                runner.step_resident()
                torch.cuda.synchronize()
                note("step", attempt, "status", None if runner.peers is None else int(runner.peers.status.item()))
                got = runner.out.cpu().numpy()
                assert float(np.abs(got - want).max()) <= 1e-4, (replicate, storage, attempt)
            if storage == "float32":
                assert np.array_equal(runner.slabs[:, : runner.S].cpu().numpy(), x["value"])
            replay = runner.capture_resident()
            note("captured", replay is not None)
            if replay is not None:
                runner.out.zero_()
                replay()
                replay()
                torch.cuda.synchronize()
                assert float(np.abs(runner.out.cpu().numpy() - want).max()) <= 1e-4, (replicate, storage, "graph")
            if runner.peers is not None:
                runner.peers.check()
            if replicate == "all_gather":
                out = runner.step()                             # the host-buffer step, end to end
                assert float(np.abs(out.numpy() - whole[:, runner.q0:runner.q1]).max()) <= 1e-4
            runner.close()
        Path(tmp, f"ok{rank}").write_text("ok")
        dist.destroy_process_group()
    except BaseException:
        # leave at once: a rank that waited for its peers in a collective tear-down would hang the other one
        import traceback

        note(traceback.format_exc())
        log.close()
        os._exit(1)


def test_value_replication_by_collective_and_by_copy_engines(tmp_path):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    try:
        mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    finally:
        for p in sorted(tmp_path.glob("log*.txt")):
            print(p.name, p.read_text())
    assert sorted(p.name for p in tmp_path.glob("ok*")) == ["ok0", "ok1"]
