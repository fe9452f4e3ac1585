"""The multi-GPU path on CPU: two gloo ranks each take their row shard of a graph, evaluate it with the
oracle, and the shards assembled in rank order equal the unsharded result; constants are identical
on every rank after the broadcast. This covers the partitioner and the bench's sharding logic
without GPUs (the device path is covered by the -m gpu tests and bench.py --gpus N)."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, graph: str, dims: str, batch_dim: str, out_dir: str):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    import minicompiler_b200 as mc
    from oracle import reference_cpu as oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    path = mc.graph_path(graph)
    full_dims = {k: int(v) for k, v in (kv.split("=") for kv in dims.split(","))}
    shard, row_offset, rows = mc.shard_dims(path, dims, batch_dim, rank, world)
    shard_dims = {k: int(v) for k, v in (kv.split("=") for kv in shard.split(","))}
    g = oracle.parse_mcg_file(path, shard_dims)
    whole = oracle.parse_mcg_file(path, full_dims)

    # one broadcast replicates the constants (here: checks that they were identical to begin with)
    consts = np.concatenate([np.zeros(1, dtype=np.float32)] + [n.value.reshape(-1) for n in g.nodes if n.op == "const"])
    t = torch.from_numpy(consts.copy())
    dist.broadcast(t, src=0)
    assert np.array_equal(t.numpy(), consts)

    # every rank slices its rows out of the same seeded full-batch input
    x_full = oracle.make_random_inputs(whole, 1)[0]
    x = x_full[row_offset:row_offset + rows]
    y = oracle.evaluate_f32(g, [x])[0].reshape(rows, -1)

    gathered = [torch.empty_like(torch.from_numpy(y)) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(y))
    if rank == 0:
        assembled = np.concatenate([p.numpy() for p in gathered], axis=0)
        want = oracle.evaluate_f32(whole, [x_full])[0].reshape(assembled.shape)
        np.save(os.path.join(out_dir, "max_err.npy"), np.array([float(np.max(np.abs(assembled - want)))]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("graph,dims,batch_dim", [("c5_mlp_stack", "B=32,D=64", "B"), ("c3_ffn", "T=16,D=32,H=64", "T"),
                                                  ("x1_softmax", "M=16,N=96", "M")])
def test_row_shards_assemble_to_the_unsharded_result(tmp_path, graph, dims, batch_dim):
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, graph, dims, batch_dim, str(tmp_path)), nprocs=2, join=True)
    err = float(np.load(tmp_path / "max_err.npy")[0])
    # row sharding changes no arithmetic except the BLAS blocking of the matmuls
    assert err <= 1e-5
