"""All-to-all kernel with the ranks emulated as block rows of one cooperative launch, and across real GPUs when
there are several.  Oracle: index arithmetic on the host (the kernel moves bytes, it does no arithmetic)."""
import uuid

import pytest
import torch

from mp_util import run_ranks

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype,per", [(torch.bfloat16, 8), (torch.bfloat16, 4097), (torch.float32, 1), (torch.float16, 65536 + 24),
                                       (torch.float32, 300000)])
def test_all_to_all_emulated(world, dtype, per):
    from ooverlap_b200 import EmulatedGroup
    g = EmulatedGroup(world, heap_bytes=64 << 20)
    try:
        esize = torch.empty(0, dtype=dtype).element_size()
        off = g.alloc(world * per * esize + 64)
        src = torch.empty(world, world, per, device="cuda", dtype=dtype)  # [sender, destination, per]
        for s in range(world):
            for d in range(world):
                src[s, d] = (torch.arange(per, device="cuda") % 251 + 1000 * s + 10 * d).to(dtype)
        for r in range(world):
            g.view(off, (world, per), dtype, r).fill_(-1)
        for it in range(2):  # twice: the barriers' epochs carry over
            g.all_to_all(off, per, dtype, src, max_ctas=3)
            g.check_status()
            torch.cuda.synchronize()
            for d in range(world):
                got = g.view(off, (world, per), dtype, d)
                assert torch.equal(got, src[:, d]), (world, dtype, per, d, it)
        g.free(off)
    finally:
        g.close()


def _rank_a2a(rank, world, key):
    from ooverlap_b200 import Communicator
    torch.cuda.set_device(rank)
    comm = Communicator(list(range(world)), rank, key, heap_bytes=128 << 20)
    bad = []
    for shape, dtype in (((world, 3, 5), torch.float32), ((world, 4096, 64), torch.bfloat16), ((world, 1), torch.float16)):
        n = 1
        for s in shape[1:]:
            n *= s
        x = ((torch.arange(world * n, device="cuda") % 199).view(shape) + 1000 * rank).to(dtype)
        for it in range(2):
            y = comm.all_to_all(x)
            torch.cuda.synchronize()
            want = torch.stack([((torch.arange(world * n, device="cuda") % 199).view(shape)[rank] + 1000 * r).to(dtype)
                                for r in range(world)])
            if not torch.equal(y, want):
                bad.append((shape, str(dtype), it))
    comm.check_status()
    comm.barrier()
    comm.close()
    return bad


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_all_to_all_across_gpus():
    world = min(torch.cuda.device_count(), 8)
    res = run_ranks(_rank_a2a, world, ("a2a_" + uuid.uuid4().hex[:10],), timeout=300)
    assert len(res) == world, res
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok" and not val, val
