"""torch-collectives API on CPU tensors over gloo, world_size 2: all_reduce(sum), reduce_scatter and
all_gather on fp32 tensors of 1, 4097 and 1,048,576 elements (values ~N(0,1), seed 0 per rank),
checked against torch.distributed."""
import pytest
import torch

from mp_util import free_port, run_ranks

SIZES = [1, 4097, 1048576]


def _rank(rank, world, port):
    import torch.distributed as dist
    from ooverlap_b200 import Communicator
    from ooverlap_b200.utils.partition import partition
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    comm = Communicator()
    assert comm.is_cpu and comm.world == world and comm.rank == rank
    report = []
    for n in SIZES:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(n, generator=g, dtype=torch.float32) * (rank + 1)
        # all_reduce
        want = x.clone()
        dist.all_reduce(want)
        got = comm.all_reduce(x.clone())
        report.append(("ar", n, float((got - want).abs().max())))
        # reduce_scatter (uneven partitions: base + 1 for the first ranks)
        b, e = partition(n, world, rank)
        full = x.clone()
        dist.all_reduce(full)
        got = comm.reduce_scatter(x.clone())
        assert got.numel() == e - b
        report.append(("rs", n, float((got - full[b:e]).abs().max()) if e > b else 0.0))
        out = torch.empty(e - b)
        comm.reduce_scatter(x.clone(), out=out)
        report.append(("rs_out", n, float((out - full[b:e]).abs().max()) if e > b else 0.0))
        # all_gather (even shards, against dist.all_gather)
        shard = x[: max(1, n // world)].clone()
        parts = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(parts, shard)
        got = comm.all_gather(shard)
        report.append(("ag", n, float((got - torch.cat(parts)).abs().max())))
        # all_gather with uneven shards
        mine = x[b:e].clone()
        got = comm.all_gather(mine, total=n)
        ref = [torch.randn(n, generator=torch.Generator().manual_seed(0)) * (r + 1) for r in range(world)]
        want = torch.cat([ref[r][slice(*partition(n, world, r))] for r in range(world)])
        report.append(("ag_uneven", n, float((got - want).abs().max())))
    # min / max and 16-bit dtypes go through the same path
    y = torch.tensor([float(rank), -float(rank), 3.0])
    assert comm.all_reduce(y.clone(), "max").tolist() == [float(world - 1), 0.0, 3.0]
    assert comm.all_reduce(y.clone(), "min").tolist() == [0.0, -float(world - 1), 3.0]
    h = torch.full((5,), 1.5, dtype=torch.bfloat16)
    assert comm.all_reduce(h).tolist() == [1.5 * world] * 5
    # host-side exchange of a few integers per rank (what the autotuner agrees through)
    assert comm.host_all_gather([rank, 7 - rank]) == [[r, 7 - r] for r in range(world)]
    assert comm.status_ok()
    # all-to-all: slice j of every rank's [world, 3, 5] tensor goes to rank j
    t = torch.arange(world * 15, dtype=torch.float32).view(world, 3, 5) + 1000 * rank
    got = comm.all_to_all(t)
    want = torch.stack([torch.arange(world * 15, dtype=torch.float32).view(world, 3, 5)[rank] + 1000 * r for r in range(world)])
    report.append(("a2a", 15, float((got - want).abs().max())))
    comm.barrier()
    dist.destroy_process_group()
    return report


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_gloo_collectives(world):
    res = run_ranks(_rank, world, (free_port(),), timeout=180)
    assert len(res) == world
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok", val
        for name, n, err in val:
            assert err <= 1e-5, (name, n, err)


def test_cpu_communicator_needs_process_group():
    from ooverlap_b200 import Communicator
    with pytest.raises(RuntimeError):
        Communicator()


def test_unsupported_dtype_and_op():
    from ooverlap_b200.utils.dtypes import dtype_code, op_code
    with pytest.raises(TypeError):
        dtype_code(torch.int32)
    with pytest.raises(ValueError):
        op_code("prod")
