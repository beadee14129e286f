"""Multi-rank collective kernels on ONE GPU: all ranks of the group are block rows of a single cooperative
launch, so flags, barriers and peer loads/stores run exactly as across GPUs.  Oracle: PyTorch fp32."""
import pytest
import torch

from ooverlap_b200 import _lib

pytestmark = pytest.mark.gpu

SIZES = [1, 7, 8, 4097, 65536 + 24]
TOL = {torch.float16: 1e-2, torch.bfloat16: 1e-2, torch.float32: 1e-5}


@pytest.fixture(scope="module", params=[2, 4, 8])
def group(request):
    from ooverlap_b200 import EmulatedGroup
    g = EmulatedGroup(request.param, heap_bytes=64 << 20)
    yield g
    g.close()


def _fill(group, off, n, dtype, seed):
    xs = []
    for r in range(group.world):
        g = torch.Generator(device="cuda").manual_seed(seed * 100 + r)
        x = (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype)
        group.view(off, (n,), dtype, r).copy_(x)
        xs.append(x)
    return xs


def _reduce(xs, op):
    st = torch.stack([x.float() for x in xs])
    return {"sum": st.sum(0), "min": st.min(0).values, "max": st.max(0).values}[op]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("n", SIZES)
def test_all_reduce_one_shot(group, n, dtype):
    off = group.alloc(n * 4 + 64)
    xs = _fill(group, off, n, dtype, n)
    out = torch.zeros(group.world, n, device="cuda", dtype=dtype)
    group.all_reduce(off, n, dtype, algo=_lib.AR_ONESHOT_P2P, out_local=out)
    group.check_status()
    want = _reduce(xs, "sum")
    for r in range(group.world):
        assert (out[r].float() - want).abs().max().item() <= TOL[dtype] * group.world
        assert torch.equal(out[r], out[0])  # fixed rank order: every rank gets the same bits
    group.free(off)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", SIZES)
def test_all_reduce_two_shot_in_place(group, n, dtype):
    off = group.alloc(n * 4 + 64)
    xs = _fill(group, off, n, dtype, n + 1)
    group.all_reduce(off, n, dtype, algo=_lib.AR_TWOSHOT_P2P, out_off=off, max_ctas=3)
    group.check_status()
    want = _reduce(xs, "sum")
    for r in range(group.world):
        got = group.view(off, (n,), dtype, r)
        assert (got.float() - want).abs().max().item() <= TOL[dtype] * group.world
    group.free(off)


@pytest.mark.parametrize("op", ["min", "max"])
def test_all_reduce_min_max(group, op):
    n = 4097
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        off = group.alloc(n * 4 + 64)
        xs = _fill(group, off, n, dtype, 5)
        out_off = group.alloc(n * 4 + 64)
        group.all_reduce(off, n, dtype, op, algo=_lib.AR_TWOSHOT_P2P, out_off=out_off)
        group.check_status()
        want = _reduce(xs, op)
        for r in range(group.world):
            assert torch.equal(group.view(out_off, (n,), dtype, r).float(), want)
            assert torch.equal(group.view(off, (n,), dtype, r), xs[r])  # out of place: input untouched
        group.free(off)
        group.free(out_off)


def test_back_to_back_calls_reuse_flags(group):
    n, dtype = 1024, torch.bfloat16
    off = group.alloc(n * 2)
    for it in range(20):
        xs = _fill(group, off, n, dtype, 1000 + it)
        out = torch.empty(group.world, n, device="cuda", dtype=dtype)
        group.all_reduce(off, n, dtype, algo=_lib.AR_ONESHOT_P2P, out_local=out, max_ctas=1 + it % 3)
        assert (out[0].float() - _reduce(xs, "sum")).abs().max().item() <= 1e-2 * group.world
    group.check_status()
    group.free(off)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", SIZES)
def test_reduce_scatter(group, n, dtype):
    from ooverlap_b200.utils.partition import max_shard, partition
    off = group.alloc(n * 4 + 64)
    xs = _fill(group, off, n, dtype, n + 2)
    out = torch.zeros(group.world, max_shard(n, group.world), device="cuda", dtype=dtype)
    group.reduce_scatter(off, n, dtype, out)
    group.check_status()
    want = _reduce(xs, "sum")
    for r in range(group.world):
        b, e = partition(n, group.world, r)
        if e > b:
            assert (out[r, : e - b].float() - want[b:e]).abs().max().item() <= TOL[dtype] * group.world
    group.free(off)


@pytest.mark.parametrize("algo", [_lib.AG_PUSH_P2P, _lib.AG_PULL_P2P])
@pytest.mark.parametrize("n", SIZES)
def test_all_gather(group, n, algo):
    from ooverlap_b200.utils.partition import max_shard, partition
    dtype = torch.bfloat16
    w = group.world
    shard = max_shard(n, w)
    full = torch.randn(n, device="cuda").to(dtype)
    if algo == _lib.AG_PUSH_P2P:
        src = torch.zeros(w, shard, device="cuda", dtype=dtype)
        for r in range(w):
            b, e = partition(n, w, r)
            src[r, : e - b] = full[b:e]
        off = group.alloc(n * 2 + 64)
        for r in range(w):
            group.view(off, (n,), dtype, r).zero_()
        group.all_gather(off, n, dtype, src_local=src, algo=algo)
        group.check_status()
        for r in range(w):
            assert torch.equal(group.view(off, (n,), dtype, r), full)
    else:
        off = group.alloc(shard * 2 + 64)
        for r in range(w):
            b, e = partition(n, w, r)
            group.view(off, (shard,), dtype, r)[: e - b] = full[b:e]
        dst = torch.zeros(w, n, device="cuda", dtype=dtype)
        group.all_gather(off, n, dtype, dst_local=dst, algo=algo)
        group.check_status()
        for r in range(w):
            assert torch.equal(dst[r], full)
    group.free(off)


def test_bounded_wait_reports_and_recovers():
    """A wait on a flag that nothing sets runs out after the configured budget, the kernel returns, the host
    reads who waited for what, and the communicator works again after recover()."""
    from ooverlap_b200 import DeviceTimeout, EmulatedGroup
    g = EmulatedGroup(2, heap_bytes=8 << 20, timeout_ms=200)
    g.bounded_wait_selftest()
    st = g.status()
    assert st.code == 2 and st.where == 99 and st.expected == 1 and st.observed == 0
    with pytest.raises(DeviceTimeout):
        g.check_status()
    off = g.alloc(1024)
    with pytest.raises(DeviceTimeout):  # poisoned until recovered
        g.all_reduce(off, 16, torch.float32, algo=_lib.AR_TWOSHOT_P2P, out_off=off)
    g.recover()
    for r in range(2):
        g.view(off, (16,), torch.float32, r).fill_(r + 1.0)
    g.all_reduce(off, 16, torch.float32, algo=_lib.AR_TWOSHOT_P2P, out_off=off)
    g.check_status()
    assert g.view(off, (16,), torch.float32, 1).tolist() == [3.0] * 16
    g.close()


def test_heap_allocator_reuses_freed_blocks():
    from ooverlap_b200 import EmulatedGroup, OobError
    g = EmulatedGroup(2, heap_bytes=4 << 20)
    a = g.alloc(1 << 20)
    b = g.alloc(1 << 20)
    assert b >= a + (1 << 20)
    g.free(a)
    c = g.alloc(512 << 10)
    assert c == a
    with pytest.raises(OobError):
        g.alloc(64 << 20)
    with pytest.raises(OobError):
        g.free(12345)
    g.close()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("n", [1, 7, 8, 4096, 4097, 65536 + 24])
@pytest.mark.parametrize("op", ["sum", "max"])
def test_all_reduce_push_one_barrier(group, n, dtype, op):
    """Every rank pushes its unregistered input into its piece of a staging area on all ranks, one barrier, local sum in
    rank order.  Odd counts make the ranks' rows start off a 16-byte boundary (element-wise local accesses) while the
    staging pieces stay aligned.  The same staging area serves five calls in a row: it holds two sets of pieces and the
    kernel alternates between them by a call counter kept on the device."""
    esize = torch.empty((), dtype=dtype).element_size()
    piece = (n * esize + 255) // 256 * 256
    stages = [group.alloc(2 * group.world * piece)]
    for it in range(5):
        gen = torch.Generator(device="cuda").manual_seed(n * 10 + it)
        x = (torch.rand(group.world, n, device="cuda", generator=gen) * 2 - 1).to(dtype)
        out = torch.zeros_like(x)
        group.all_reduce_push(stages[0], piece, x, out, op, max_ctas=3 if it % 2 else 2)
        group.check_status()
        want = _reduce(list(x), op)
        for r in range(group.world):
            assert (out[r].float() - want).abs().max().item() <= TOL[dtype] * group.world, (it, r)
            assert torch.equal(out[r], out[0])
    for s in reversed(stages):
        group.free(s)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("n", [1, 2, 7, 8, 4096, 4097, 32768])
@pytest.mark.parametrize("op", ["sum", "max"])
def test_all_reduce_flag_in_data(group, n, dtype, op):
    """No barrier: every rank stores 8-byte cells of data + call number into its piece on all ranks, receivers spin on
    the cells.  The same zeroed staging area serves six calls in a row (two sets of cells, alternated by the call
    counter on the device); odd counts leave half a word at the end."""
    esize = torch.empty((), dtype=dtype).element_size()
    words = (n * esize + 3) // 4
    piece = (8 * words + 255) // 256 * 256
    stage = group.alloc(2 * group.world * piece)
    for r in range(group.world):
        group.view(stage, (2 * group.world * piece,), torch.uint8, r).zero_()
    torch.cuda.synchronize()
    for it in range(6):
        gen = torch.Generator(device="cuda").manual_seed(n * 10 + it)
        x = (torch.rand(group.world, n, device="cuda", generator=gen) * 2 - 1).to(dtype)
        out = torch.zeros_like(x)
        group.all_reduce_ll(stage, piece, x, out, op, max_ctas=3 if it % 2 else 1)
        group.check_status()
        want = _reduce(list(x), op)
        for r in range(group.world):
            assert (out[r].float() - want).abs().max().item() <= TOL[dtype] * group.world, (it, r)
            assert torch.equal(out[r], out[0])
    group.free(stage)
