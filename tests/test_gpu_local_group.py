"""One process drives every GPU of the box through LocalGroup: collectives and a fused GEMM->AllReduce against PyTorch
references computed on the host."""
import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                 reason="needs at least 2 GPUs")]


def _world():
    return min(torch.cuda.device_count(), 8)


def test_collectives_from_one_process():
    from ooverlap_b200 import LocalGroup
    world = _world()
    with LocalGroup(list(range(world)), heap_bytes=256 << 20) as g:
        assert g.world == world and all(c.rank == r for r, c in enumerate(g.comms))
        for n in (1024, 65536 + 8, 4 << 20):
            n = n // world * world
            host = [(torch.rand(n, generator=torch.Generator().manual_seed(31 * r + n)) * 2 - 1).bfloat16() for r in range(world)]
            total = sum(h.float() for h in host)
            xs = g.empty((n,), torch.bfloat16)
            for r in range(world):
                xs[r].copy_(host[r])
            g.synchronize()
            # reduce-scatter of a registered tensor leaves the result in the rank's own partition of it
            rs = g.reduce_scatter(xs)
            g.check_status()
            per = n // world
            for r in range(world):
                assert (rs[r].float().cpu() - total[r * per:(r + 1) * per]).abs().max().item() <= 0.05 * world, (n, r)
                xs[r].copy_(host[r])
            g.synchronize()
            ag = g.all_gather([x[:per] for x in xs])
            g.check_status()
            want = torch.cat([h[:per] for h in host])
            for r in range(world):
                assert torch.equal(ag[r].cpu(), want), (n, r)
            ys = g.all_reduce(xs)
            g.check_status()
            for r in range(world):
                assert (ys[r].float().cpu() - total).abs().max().item() <= 0.05 * world, (n, r)
                assert torch.equal(ys[r].cpu(), ys[0].cpu())
            g.free(xs)
        g.barrier()


@pytest.mark.parametrize("kernel", ["pair", "one_sm"])
def test_fused_gemm_all_reduce_from_one_process(kernel):
    from ooverlap_b200 import LocalGroup
    from ooverlap_b200.ops import GemmAllReduce
    world = _world()
    M, N, K = 1024, 2048, 512
    with LocalGroup(list(range(world)), heap_bytes=512 << 20) as g:
        a_host = [torch.randn(M, K, generator=torch.Generator().manual_seed(r)).half() for r in range(world)]
        b_host = [(torch.randn(N, K, generator=torch.Generator().manual_seed(100 + r)) / (K * world) ** 0.5).half()
                  for r in range(world)]
        want = sum(a.float() @ b.float().t() for a, b in zip(a_host, b_host))
        a = [a_host[r].to(f"cuda:{g.devices[r]}") for r in range(world)]
        b = [b_host[r].to(f"cuda:{g.devices[r]}") for r in range(world)]
        ops = g.each(lambda r, c: GemmAllReduce(c, M, N, torch.float16, strategy="fused", kernel=kernel, comm_ctas=8))
        g.synchronize()
        for _ in range(3):
            outs = g.each(lambda r, c: ops[r](a[r], b[r]))
            g.check_status()
            for r in range(world):
                got = outs[r].float().cpu()
                assert (got - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item()), r
        g.each(lambda r, c: ops[r].release())
