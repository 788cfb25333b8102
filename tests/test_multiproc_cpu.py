"""World-size-2 test (gloo, CPU) of the multi-GPU host logic: unit sharding, independent per-rank
work with no data-path collective, gather for checking.  The per-rank compute here is the CPU
oracle (tests may use it); on GPUs the same shards go to the CUDA ops."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from linearnexus_b200.shard import gather_outputs, shard_inputs, unit_range
from oracle import delta_rule_oracle as O


def test_unit_range_covers_everything():
    for n in (1, 7, 8, 128, 130):
        for world in (1, 2, 3, 8):
            got = [unit_range(n, world, r) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            sizes = [hi - lo for lo, hi in got]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        unit_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, H, result_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        inp = O.make_inputs("gated", B, H, 48, 16, 16, seed=21, h0_std=0.1)
        shard, mode = shard_inputs(inp, world, rank)
        o, hT = O.gated_delta_rule_chunkwise(shard["q"], shard["k"], shard["v"], shard["g"], shard["beta"],
                                             initial_state=shard["h0"], chunk_size=16)
        n_units = B if mode == "batch" else B * H
        sizes = [unit_range(n_units, world, r)[1] - unit_range(n_units, world, r)[0] for r in range(world)]
        o_all = gather_outputs(o, sizes)
        h_all = gather_outputs(hT, sizes)
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)   # the benchmark's max-over-ranks timing reduction
        if rank == 0:
            ro, rh = O.gated_delta_rule_chunkwise(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"],
                                                  initial_state=inp["h0"], chunk_size=16)
            if mode == "unit":
                ro, rh = ro.reshape(B * H, 1, *ro.shape[2:]), rh.reshape(B * H, 1, *rh.shape[2:])
            result_queue.put((mode, float((o_all - ro).abs().max()), float((h_all - rh).abs().max()), float(t)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,H,mode", [(4, 2, "batch"), (1, 6, "unit")])
def test_two_ranks_shard_and_gather(B, H, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, B, H, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got_mode, eo, eh, tmax = q.get(timeout=10)
    assert got_mode == mode
    assert eo < 1e-6 and eh < 1e-6
    assert tmax == 2.0


def test_rows_built_per_rank_equal_the_cut_of_the_global_batch():
    """The benchmark builds only a rank's rows of the global batch; that must be what shard_inputs cuts out of it."""
    from linearnexus_b200.synthetic import make_rows
    whole = make_rows("gated", 0, 4, 2, 24, 8, 8, seed=11, h0_std=0.1)
    for world in (2, 4):
        for rank in range(world):
            cut, mode = shard_inputs(whole, world, rank)
            lo, hi = unit_range(4, world, rank)
            mine = make_rows("gated", lo, hi, 2, 24, 8, 8, seed=11, h0_std=0.1)
            assert mode == "batch"
            for name in whole:
                assert torch.equal(cut[name], mine[name]), name
    assert make_rows("delta", 0, 1, 2, 8, 4, 4, seed=1)["g"] is None
