"""Two ranks on two GPUs (NCCL): every rank runs its rows of one seeded global batch through the CUDA op with no
collective on the data path; NCCL only gathers the results, which must equal the single-GPU run of the whole batch.
Skipped on a machine with fewer than two GPUs.  NVLS is switched off: the test needs plain NCCL only."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import linearnexus_b200 as L
    from linearnexus_b200 import ops
    from linearnexus_b200.shard import gather_outputs, shard_inputs, unit_range
    from linearnexus_b200.synthetic import make_rows
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, H, T = 3, 2, 320            # uneven cut: 2 rows on rank 0, 1 on rank 1
        whole = make_rows("gated", 0, B, H, T, 128, 128, seed=31, io_dtype=torch.bfloat16, h0_std=0.02)
        mine, mode = shard_inputs(whole, world, rank)
        cu = {k: (None if v is None else v.contiguous().to(dev)) for k, v in mine.items()}
        o, hT = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
        ops.check_device_status(dev)
        sizes = [unit_range(B, world, r)[1] - unit_range(B, world, r)[0] for r in range(world)]
        o_all = gather_outputs(o.contiguous(), sizes)
        h_all = gather_outputs(hT.contiguous(), sizes)
        if rank == 0:
            w = {k: (None if v is None else v.to(dev)) for k, v in whole.items()}
            ro, rh = L.gated_delta_rule_chunkwise(w["q"], w["k"], w["v"], w["g"], w["beta"], initial_state=w["h0"])
            queue.put((mode, bool(torch.equal(o_all, ro)), bool(torch.equal(h_all, rh))))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpus_shard_run_and_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    mode, same_o, same_h = q.get(timeout=10)
    assert mode == "batch" and same_o and same_h   # a unit's result does not depend on which GPU ran it
