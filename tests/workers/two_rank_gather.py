"""Worker of tests/test_gpu_two_ranks.py: one rank of a 2-GPU run (started by torch.distributed.run).

Each rank compiles the MLP stack for its share of the rows (mc_shard_dims), takes rank 0's constants through the
library's own NCCL broadcast (mc_replicate_constants), runs its rows, and assembles the whole output on its device
with mc_gather_output. Every rank prints one line saying whether its rows and the gathered tensor equal, bit for
bit, what the unsharded graph gives on the same GPU."""

import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import minicompiler_b200 as mc  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")  # carries the 128-byte unique id only
    uid = [mc.Communicator.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    comm = mc.Communicator(world, rank, uid[0], local, timeout_s=60.0)
    path = mc.graph_path("c5_mlp_stack")
    dims = {"B": 1024, "D": 256}
    x = np.random.default_rng(5).standard_normal((1024, 256), dtype=np.float32)
    shard, first, rows = mc.shard_dims(path, dims, "B", rank, world)
    options = {"device": local, "matmul": "tensor_core_f16"}
    with mc.CompiledGraph(path, dims=shard, options=options) as exe:
        if rank != 0:
            # a rank whose constants are wrong before the broadcast must be right after it
            ptr, nbytes = exe.constants_region()
            torch.cuda.synchronize()
            junk = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
            assert mc.lib().mcd_copy_d2d(ptr, junk.data_ptr(), nbytes, None) == 0
            torch.cuda.synchronize()
        exe.replicate_constants(comm, root=0)
        exe.upload([x[first:first + rows]])
        exe.enqueue()
        mine = exe.download()[0]
        dst = torch.full((1024 * 256,), float("nan"), dtype=torch.float32, device="cuda")
        exe.gather_output(0, comm, dst.data_ptr())
        gathered = dst.cpu().numpy()
    with mc.CompiledGraph(path, dims=dims, options=options) as whole_exe:
        whole = whole_exe.run([x])[0]
    own = np.array_equal(mine, whole.reshape(1024, 256)[first:first + rows].reshape(-1))
    print(f"rank {rank} own_rows_equal={own} gathered_equal={np.array_equal(gathered, whole)}", flush=True)
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
