"""One process per GPU with the real ``Communicator`` (symmetric heap over VMM file descriptors, NVLS multicast
where the driver grants it).  Needs at least two GPUs; skipped otherwise.  Oracle: PyTorch fp32 on the host."""
import os
import uuid

import pytest
import torch

from mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return min(n, 8)


needs_multi = pytest.mark.skipif(_world() < 2, reason="needs at least 2 GPUs")


def _inputs(world, n, dtype, seed):
    return [(torch.rand(n, generator=torch.Generator().manual_seed(seed * 31 + r)) * 2 - 1).to(dtype)
            for r in range(world)]


def _rank_collectives(rank, world, key, flags_env):
    import os
    os.environ.update(flags_env)
    from ooverlap_b200 import Communicator, _lib
    from ooverlap_b200.utils.partition import partition
    torch.cuda.set_device(rank)
    comm = Communicator(list(range(world)), rank, key, heap_bytes=256 << 20)
    report = {"nvls": comm.nvls, "memory_kind": comm.info.memory_kind, "checks": []}

    def check(name, got, want, tol):
        err = (got.float().cpu() - want.float()).abs().max().item() if want.numel() else 0.0
        report["checks"].append((name, err, tol))

    ar_algos = [_lib.AR_TWOSHOT_P2P] + ([_lib.AR_TWOSHOT_NVLS] if comm.nvls else [])
    os_algos = [_lib.AR_ONESHOT_P2P] + ([_lib.AR_ONESHOT_NVLS] if comm.nvls else [])
    for dtype, tol in ((torch.bfloat16, 1e-2 * world), (torch.float16, 1e-2 * world), (torch.float32, 1e-5 * world)):
        for n in (1, 7, 4097, (1 << 20) + 8):
            xs = _inputs(world, n, dtype, n)
            want = torch.stack([x.float() for x in xs]).sum(0)
            buf = comm.empty((n,), dtype)
            for algo in ar_algos:
                buf.copy_(xs[rank].cuda())
                comm.all_reduce(buf, algo=algo)
                check(f"ar_inplace algo{algo} {dtype} {n}", buf, want, tol)
            for algo in os_algos:
                buf.copy_(xs[rank].cuda())
                out = torch.empty(n, dtype=dtype, device="cuda")
                comm.all_reduce_out(buf, out, algo=algo)
                check(f"ar_oneshot algo{algo} {dtype} {n}", out, want, tol)
            # policy-selected, unregistered input (copied into the cached scratch)
            got = comm.all_reduce(xs[rank].cuda())
            check(f"ar_auto {dtype} {n}", got, want, tol)
            # reduce-scatter: in place and into a separate tensor, both algorithms
            b, e = partition(n, world, rank)
            for algo in [_lib.RS_P2P] + ([_lib.RS_NVLS] if comm.nvls else []):
                buf.copy_(xs[rank].cuda())
                got = comm.reduce_scatter(buf, algo=algo)
                check(f"rs algo{algo} {dtype} {n}", got, want[b:e], tol)
            out = torch.empty(e - b, dtype=dtype, device="cuda")
            comm.reduce_scatter(xs[rank].cuda(), out=out)
            check(f"rs_out {dtype} {n}", out, want[b:e], tol)
            # all-gather (uneven shards)
            full = torch.cat([xs[r][slice(*partition(n, world, r))] for r in range(world)])
            for algo in [_lib.AG_PUSH_P2P] + ([_lib.AG_PUSH_NVLS] if comm.nvls else []):
                got = comm.all_gather(xs[rank][b:e].cuda(), total=n, algo=algo)
                check(f"ag algo{algo} {dtype} {n}", got, full, 0.0)
            torch.cuda.synchronize()
            comm.check_status()
    # min / max
    x = torch.tensor([float(rank), -float(rank), 0.5], device="cuda")
    check("max", comm.all_reduce(x.clone(), "max"), torch.tensor([world - 1.0, 0.0, 0.5]), 0.0)
    check("min", comm.all_reduce(x.clone(), "min"), torch.tensor([0.0, 1.0 - world, 0.5]), 0.0)
    # slot pools: zero-copy producer -> all-reduce, ring wraps
    comm.init_round_robin_slots(torch.bfloat16, 1 << 20, 3)
    for it in range(5):
        slot = comm.acquire_all_reduce_slot((64, 128))
        slot.fill_(float(rank + it))
        got = comm.all_reduce_preloaded_slot(slot)
        check(f"slot {it}", got, torch.full((64, 128), float(sum(r + it for r in range(world)))), 1e-2 * world)
    got = comm.all_reduce_round_robin(torch.full((10,), 2.0, dtype=torch.bfloat16, device="cuda"))
    check("rr", got, torch.full((10,), 2.0 * world), 1e-2)
    # small tensors take the one-barrier push kernel (pieces in its own staging area, result in the slot); the ring of
    # three wraps twice,
    # odd sizes exercise the element tail and a misaligned view the element-wise local path
    for it in range(7):
        for n in (1, 8, 4097, 32768):
            xs = _inputs(world, n + 1, torch.bfloat16, 1000 * it + n)
            x = xs[rank].cuda()[1:] if it % 2 else xs[rank].cuda()[:n]
            ref = torch.stack([(t[1:] if it % 2 else t[:n]).float() for t in xs]).sum(0)
            got = comm.all_reduce_push(x)
            assert got is not None
            check(f"push {it} {n}", got, ref, 1e-2 * world)
    assert comm.all_reduce_push(torch.zeros(1 << 19, dtype=torch.bfloat16, device="cuda")) is None  # 1 MiB: too large
    comm.init_all_gather_slots(torch.bfloat16, 1 << 20, 2)
    got = comm.all_gather_round_robin(torch.full((4, 8), float(rank), dtype=torch.bfloat16, device="cuda"))
    check("ag_rr", got, torch.arange(world).float().repeat_interleave(4).unsqueeze(1).expand(-1, 8), 0.0)
    # torch-allocated tensor registered through legacy IPC (base + offset inside the caching allocator's block)
    try:
        big = torch.zeros(1 << 16, device="cuda")
        view = big[1000:1000 + 4096]
        view.fill_(rank + 1.0)
        comm.all_reduce_inplace(view)
        check("ipc_inplace", view, torch.full((4096,), float(sum(r + 1 for r in range(world)))), 1e-5 * world)
        report["ipc"] = "ok"
    except _lib.OobError as e:  # e.g. expandable segments: reported, not fatal
        report["ipc"] = f"unsupported: {e}"
    torch.cuda.synchronize()
    comm.check_status()
    comm.barrier()
    comm.close()
    return report


@needs_multi
@pytest.mark.parametrize("nvls", [True, False])
def test_collectives_all_algorithms(nvls):
    world = _world()
    env = {} if nvls else {"OOB_DISABLE_NVLS": "1"}
    res = run_ranks(_rank_collectives, world, ("mp_" + uuid.uuid4().hex[:10], env), timeout=600)
    assert len(res) == world, res
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok", val
        if not nvls:
            assert not val["nvls"]
        bad = [(n, e, t) for n, e, t in val["checks"] if not e <= t]
        assert not bad, bad[:10]
    print("nvls:", res[0][1]["nvls"], "memory kind:", res[0][1]["memory_kind"], "ipc:", res[0][1].get("ipc"))


def _rank_fused(rank, world, key):
    from ooverlap_b200 import Communicator
    from ooverlap_b200.ops import (AllGatherGemm, GemmAllReduce, GemmReduceScatterNorm, fused_allreduce_rmsnorm,
                                   fused_reduce_scatter_rmsnorm)
    torch.cuda.set_device(rank)
    comm = Communicator(list(range(world)), rank, key, heap_bytes=512 << 20)
    dt = torch.bfloat16
    out = []

    def gen(shape, seed, scale=1.0):
        return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).to(dt)

    # fused all-reduce + residual + RMSNorm (one-shot for few tokens, two-shot for many)
    hidden, eps = 4096, 1e-6
    w = (1 + 0.02 * torch.randn(hidden, generator=torch.Generator().manual_seed(5))).to(dt)
    for rows in (4, 512):
        xs = [gen((rows, hidden), 100 + r) for r in range(world)]
        res = gen((rows, hidden), 99)
        x = comm.empty((rows, hidden), dt)
        x.copy_(xs[rank].cuda())
        y, ro = fused_allreduce_rmsnorm(comm, x, w.cuda(), eps, res.cuda())
        s = (torch.stack([t.float() for t in xs]).sum(0) + res.float()).to(dt).float()
        want = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        out.append((f"ar_norm {rows}", (y.float().cpu() - want).abs().max().item(), 6e-2))
        # through NVLS the switch rounds the sum of the partials once before the residual is added, so the
        # error scales with the operands (which may cancel), not with the result
        sx = torch.stack([t.float() for t in xs]).sum(0)
        allow = (sx.abs() + res.float().abs()) * 2 ** -6
        out.append((f"ar_norm_res {rows}", ((ro.float().cpu() - s).abs() - allow).max().item(), 1e-2))
        # sequence-parallel form
        b, e = rows * rank // world, rows * (rank + 1) // world
        if rows % world == 0:
            x.copy_(xs[rank].cuda())
            y2, _ = fused_reduce_scatter_rmsnorm(comm, x, w.cuda(), eps, res[b:e].cuda())
            out.append((f"rs_norm {rows}", (y2.float().cpu() - want[b:e]).abs().max().item(), 6e-2))
    # fused GEMM ops: both kernels (CTA pairs with in-place reduction; one-SM with pushed partial tiles), every data
    # path (peer loads/stores, through the switch), a small shape and one with several waves of tiles per rank
    nvls_variants = [0, 1, 2] if comm.nvls else [0]
    for (M, N, K) in ((128 * world * 2, 1024, 512), (256 * world * 2, 4096, 256)):
        a = [gen((M, K), 200 + r) for r in range(world)]
        bw = [gen((N, K), 300 + r, (K * world) ** -0.5) for r in range(world)]
        want = sum(a[r].float() @ bw[r].float().t() for r in range(world))
        tol_c = 3e-2 * max(1, want.abs().max().item())
        for kernel in ("pair", "one_sm"):
            for variant in nvls_variants:
                if kernel == "pair" and variant == 2:
                    continue  # the pair kernel has one path through the switch
                op = GemmAllReduce(comm, M, N, dt, comm_ctas=8, use_nvls=variant, strategy="fused", kernel=kernel)
                for it in range(3):
                    c = op(a[rank].cuda(), bw[rank].cuda())
                    torch.cuda.synchronize()
                    out.append((f"gemm_ar {kernel} nvls{variant} M{M} {it}", (c.float().cpu() - want).abs().max().item(), tol_c))
                    c.zero_()
                    comm.barrier()  # nobody starts the next call while a peer still zeroes its output
                op.release()
        for strat in ("auto", "unfused"):
            op = GemmAllReduce(comm, M, N, dt, strategy=strat)
            c = op(a[rank].cuda(), bw[rank].cuda())
            torch.cuda.synchronize()
            out.append((f"gemm_ar {strat} M{M}", (c.float().cpu() - want).abs().max().item(), tol_c))
            op.release()
        if M != 128 * world * 2:
            # decided at the first call: every candidate is checked and timed on these operands, all ranks agree
            op = GemmAllReduce(comm, M, N, dt, strategy="autotune")
            for it in range(2):
                c = op(a[rank].cuda(), bw[rank].cuda())
                torch.cuda.synchronize()
                out.append((f"gemm_ar autotune {it}", (c.float().cpu() - want).abs().max().item(), tol_c))
            assert op.strategy in ("fused", "unfused") and op.tuning and any(t["us"] for t in op.tuning)
            op.release()
        if M == 128 * world * 2:
            # slabs of rows: GEMM on the caller's stream, all-reduce of each slab on a side stream
            op = GemmAllReduce(comm, M, N, dt, strategy="chunked", chunks=2)
            for it in range(3):
                c = op(a[rank].cuda(), bw[rank].cuda())
                torch.cuda.synchronize()
                out.append((f"gemm_ar chunked {it}", (c.float().cpu() - want).abs().max().item(), tol_c))
                c.zero_()
                torch.cuda.synchronize()
                comm.barrier()
            op.release()
        wn = (1 + 0.02 * torch.randn(N, generator=torch.Generator().manual_seed(6))).to(dt)
        res = gen((M, N), 400)
        rows = M // world
        s = (want + res.float()).to(dt).float()
        wanty = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * wn.float()
        a_full = gen((M, K), 500)
        wantc = a_full.float() @ bw[rank].float().t()
        for kernel in ("pair", "one_sm"):
            for variant in ([0, 1] if comm.nvls else [0]):
                rs = GemmReduceScatterNorm(comm, M, N, dt, eps=eps, comm_ctas=8, use_nvls=variant, kernel=kernel)
                for it in range(2):
                    y, ro = rs(a[rank].cuda(), bw[rank].cuda(), wn.cuda(), res[rank * rows:(rank + 1) * rows].cuda())
                    torch.cuda.synchronize()
                    out.append((f"gemm_rs_norm {kernel} nvls{variant} M{M} {it}",
                                (y.float().cpu() - wanty[rank * rows:(rank + 1) * rows]).abs().max().item(), 8e-2))
                    # the switch rounds the sum of the partials before the residual is added: allow for that
                    allow = (want[rank * rows:(rank + 1) * rows].abs() + res[rank * rows:(rank + 1) * rows].float().abs()) * 2 ** -6
                    out.append((f"gemm_rs_res {kernel} nvls{variant} M{M} {it}",
                                ((ro.float().cpu() - s[rank * rows:(rank + 1) * rows]).abs() - allow).max().item(), 1e-2))
                ag = AllGatherGemm(comm, M, K, dt, comm_ctas=8, use_nvls=variant, kernel=kernel)
                for it in range(2):
                    c = ag(a_full[rank * rows:(rank + 1) * rows].cuda(), bw[rank].cuda())
                    torch.cuda.synchronize()
                    out.append((f"ag_gemm {kernel} nvls{variant} M{M} {it}", (c.float().cpu() - wantc).abs().max().item(),
                                3e-2 * max(1, wantc.abs().max().item())))
                    comm.barrier()
                ag.release()
                rs.release()
    comm.check_status()
    comm.barrier()
    nv = comm.nvls
    comm.close()
    return nv, out


@needs_multi
def test_fused_ops_across_gpus():
    world = _world()
    res = run_ranks(_rank_fused, world, ("mf_" + uuid.uuid4().hex[:10],), timeout=600)
    assert len(res) == world, res
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok", val
        bad = [(n, e, t) for n, e, t in val[1] if not e <= t]
        assert not bad, bad


def _rank_absent_peer(rank, world, key):
    """Failure detection without faulting a GPU: the last rank sits out one collective (it is between steps,
    nothing of its own in flight).  The others' kernels give up after the wait budget, return, and the host
    reads who was missing; after a collective recover() the group works again.  NVLS is off here."""
    import os
    os.environ["OOB_DISABLE_NVLS"] = "1"
    from ooverlap_b200 import Communicator, DeviceTimeout, _lib
    torch.cuda.set_device(rank)
    comm = Communicator(list(range(world)), rank, key, heap_bytes=64 << 20)
    buf = comm.empty((1024,), torch.float32)
    buf.fill_(1.0)
    comm.all_reduce(buf, algo=_lib.AR_TWOSHOT_P2P)  # generous default budget: first launches load the kernels
    torch.cuda.synchronize()
    comm.check_status()
    ok_before = buf[0].item() == world
    comm.set_timeout_ms(500)
    comm.barrier()
    detected = None
    if rank != world - 1:
        buf.fill_(1.0)
        comm.all_reduce(buf, algo=_lib.AR_TWOSHOT_P2P)  # the last rank never joins this one
        torch.cuda.synchronize()  # returns: the kernel's wait is bounded
        try:
            comm.check_status()
        except DeviceTimeout as e:
            detected = str(e)
    comm.recover()  # collective, host side
    comm.set_timeout_ms(10000)
    comm.barrier()
    buf.fill_(2.0)
    comm.all_reduce(buf, algo=_lib.AR_TWOSHOT_P2P)
    torch.cuda.synchronize()
    comm.check_status()
    ok_after = buf[0].item() == 2.0 * world
    comm.barrier()
    comm.close()
    return ok_before, detected, ok_after


@needs_multi
def test_absent_peer_is_detected_and_recovered():
    world = min(_world(), 4)
    res = run_ranks(_rank_absent_peer, world, ("ma_" + uuid.uuid4().hex[:10],), timeout=300)
    assert len(res) == world, res
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok", val
        ok_before, detected, ok_after = val
        assert ok_before and ok_after
        if r != world - 1:
            assert detected is not None and f"peer {world - 1}" in detected


def _rank_recover_then_flag_in_data(rank, world, key):
    """recover() restarts the call numbers of the flag-in-data all-reduce, so it has to zero the cells as well: the
    third call before the recovery is a long message, the third call after it too, and the two calls in between are
    short, so without the zeroing the long one would find its own number in cells that nobody has written since."""
    import os
    os.environ["OOB_DISABLE_NVLS"] = "1"
    from ooverlap_b200 import Communicator
    torch.cuda.set_device(rank)
    comm = Communicator(list(range(world)), rank, key, heap_bytes=64 << 20)
    comm.init_round_robin_slots(torch.bfloat16, 1 << 20, 4)
    results = []

    def calls(scale):
        for n in (256, 256, 16384):
            x = torch.full((n,), scale * (rank + 1), device="cuda", dtype=torch.bfloat16)
            got = comm.all_reduce_push(x)
            torch.cuda.synchronize()
            results.append(bool((got.float() == scale * world * (world + 1) / 2).all().item()))

    calls(1.0)
    comm.check_status()
    comm.recover()
    calls(2.0)
    comm.check_status()
    comm.barrier()
    comm.close()
    return results


@needs_multi
def test_recover_zeroes_the_flag_in_data_cells():
    world = min(_world(), 4)
    res = run_ranks(_rank_recover_then_flag_in_data, world, ("mr_" + uuid.uuid4().hex[:10],), timeout=300)
    assert len(res) == world, res
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok", val
        assert all(val), val


def _rank_llama(rank, world, key, port, cfg_name="TINY"):
    import os
    import torch.distributed as dist
    from ooverlap_b200 import Communicator, models
    from ooverlap_b200.models import LlamaTP
    TINY = getattr(models, cfg_name)
    torch.cuda.set_device(rank)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    comm = Communicator(list(range(world)), rank, key, heap_bytes=256 << 20)
    comm.init_round_robin_slots(torch.bfloat16, 1 << 20, 4)
    ours = LlamaTP(TINY, comm, rank=rank, world=world, backend="ours", max_batch=4, max_len=64, seed=5)
    ref = LlamaTP(TINY, None, rank=rank, world=world, backend="nccl", max_batch=4, max_len=64, seed=5)
    prompts = torch.randint(0, TINY.vocab, (4, 16), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    with torch.no_grad():
        h1 = ours.forward(prompts, 0)
        h2 = ref.forward(prompts, 0)
    cos = torch.nn.functional.cosine_similarity(h1.float(), h2.float(), dim=-1).min().item()
    t_graph = ours.generate(prompts, 8, use_graph=True)
    t_eager = ours.generate(prompts, 8, use_graph=False)
    same = bool(torch.equal(t_graph, t_eager))
    # every rank must have produced the same tokens
    gathered = [torch.empty_like(t_graph) for _ in range(world)]
    dist.all_gather(gathered, t_graph)
    agree = all(torch.equal(g, gathered[0]) for g in gathered)
    comm.check_status()
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return cos, same, agree


@needs_multi
@pytest.mark.parametrize("cfg_name", ["TINY", "TINY128"])  # head size 64 (SDPA decode) and 128 (decode-attention kernel)
def test_llama_tensor_parallel_matches_nccl_backend(cfg_name):
    from mp_util import free_port
    world = 2
    res = run_ranks(_rank_llama, world, ("ml_" + uuid.uuid4().hex[:10], free_port(), cfg_name), timeout=600)
    assert len(res) == world, res
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok", val
        cos, same, agree = val
        assert cos > 0.99 and same and agree


def _rank_llama_prefill_chunks(rank, world, key, port):
    """Prefill with the row-parallel projections cut into slabs (GEMM of slab i overlapped with the all-reduce + norm
    of slab i - 1 on a side stream) against the same model without slabs."""
    import torch.distributed as dist
    from ooverlap_b200 import Communicator
    from ooverlap_b200.models import TINY128, LlamaTP
    torch.cuda.set_device(rank)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    comm = Communicator(list(range(world)), rank, key, heap_bytes=512 << 20)
    comm.init_round_robin_slots(torch.bfloat16, 1 << 20, 4)
    os.environ["OOB_PREFILL_CHUNKS"] = "1"
    plain = LlamaTP(TINY128, comm, rank=rank, world=world, backend="ours", max_batch=2, max_len=1100, seed=5)
    os.environ["OOB_PREFILL_CHUNKS"], os.environ["OOB_PREFILL_CHUNK_MIN_ROWS"] = "2", "1024"
    slabs = LlamaTP(TINY128, comm, rank=rank, world=world, backend="ours", max_batch=2, max_len=1100, seed=5)
    assert slabs.prefill_chunks == 2 and plain.prefill_chunks == 1
    prompts = torch.randint(0, TINY128.vocab, (2, 1024), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    with torch.no_grad():
        h1 = plain.forward(prompts, 0).clone()
        h2 = slabs.forward(prompts, 0).clone()
    torch.cuda.synchronize()
    cos = torch.nn.functional.cosine_similarity(h1.float(), h2.float(), dim=-1).min().item()
    err = (h1.float() - h2.float()).abs().max().item()
    comm.check_status()
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return cos, err


@needs_multi
def test_llama_prefill_in_slabs_matches_unchunked():
    from mp_util import free_port
    world = 2
    res = run_ranks(_rank_llama_prefill_chunks, world, ("mp_" + uuid.uuid4().hex[:10], free_port()), timeout=600)
    assert len(res) == world, res
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok", val
        cos, err = val
        assert cos > 0.999 and err < 0.1, val
