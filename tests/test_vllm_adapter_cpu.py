"""vLLM backend hook: environment handling, eligibility rules and data flow, with a fake communicator
(no GPU, no vLLM engine)."""
import pytest
import torch

from ooverlap_b200.parallel import vllm_adapter as va


class FakeComm:
    """Stands in for Communicator: 'reduces' by multiplying with the world size, gathers by repetition."""

    def __init__(self, world=4, rank=1):
        self.world, self.rank, self.device, self.nvls = world, rank, 0, False
        self.calls = []
        self.closed = False

    def init_round_robin_slots(self, dtype, cap, n):
        self.calls.append(("rr", dtype, cap, n))

    def init_all_gather_slots(self, dtype, cap, n):
        self.calls.append(("ag", dtype, cap, n))

    def all_reduce_round_robin(self, x):
        self.calls.append(("ar", tuple(x.shape)))
        return x * self.world

    def all_gather_round_robin(self, shard):
        self.calls.append(("gather", tuple(shard.shape)))
        return torch.cat([shard + r for r in range(self.world)], dim=0)

    def close(self):
        self.closed = True


@pytest.fixture
def adapter(monkeypatch):
    monkeypatch.setenv("VLLM_OOVERLAP_RR_DTYPE", "fp32")
    monkeypatch.setenv("VLLM_OOVERLAP_AG_DTYPE", "fp32")
    monkeypatch.setenv("VLLM_OOVERLAP_RR_SLOTS", "5")
    monkeypatch.setenv("VLLM_OOVERLAP_RR_CAPACITY_BYTES", "4096")
    a = va.OoverlapAllReduce(communicator=FakeComm())
    a.device = torch.device("cpu")  # the fake lives on the CPU
    return a


def test_pools_follow_environment(adapter):
    assert not adapter.disabled
    assert ("rr", torch.float32, 4096, 5) in adapter.comm.calls
    assert ("ag", torch.float32, 64 << 20, 4) in adapter.comm.calls


def test_eligibility_rules(adapter, monkeypatch):
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    ok = torch.zeros(8, 16)
    assert adapter.should_custom_ar(ok)
    assert not adapter.should_custom_ar(torch.zeros(8, 16, dtype=torch.float16))      # wrong dtype
    assert not adapter.should_custom_ar(torch.zeros(64, 64))                           # larger than a slot
    assert not adapter.should_custom_ar(torch.zeros(8, 16).t())                        # not contiguous
    assert not adapter.should_custom_ar(torch.zeros(3))                                # not a multiple of 16 bytes
    assert adapter.custom_all_reduce(torch.zeros(64, 64)) is None                      # caller falls back
    out = adapter.custom_all_reduce(torch.ones(8, 16))
    assert torch.equal(out, torch.full((8, 16), 4.0))
    with adapter.capture():
        assert adapter._IS_CAPTURING
    assert not adapter._IS_CAPTURING


@pytest.mark.parametrize("dim", [0, 1, -1, 2])
def test_all_gather_any_dim(adapter, monkeypatch, dim):
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    x = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)
    got = adapter.all_gather(x, dim)
    want = torch.cat([x + r for r in range(4)], dim=dim)
    assert torch.equal(got, want)


def test_disabled_for_single_rank_and_after_close():
    a = va.OoverlapAllReduce(communicator=FakeComm(world=1, rank=0))
    assert a.disabled and a.custom_all_reduce(torch.zeros(4)) is None
    b = va.OoverlapAllReduce(communicator=FakeComm())
    comm = b.comm
    b.close()
    assert b.disabled and comm.closed


def test_forced_backend_switch(monkeypatch):
    monkeypatch.delenv("VLLM_FORCE_ALLREDUCE_BACKEND", raising=False)
    assert va.forced_backend() == "auto"
    assert va.install() is False
    monkeypatch.setenv("VLLM_FORCE_ALLREDUCE_BACKEND", "OOVERLAP")
    assert va.forced_backend() == "ooverlap"
    monkeypatch.setenv("VLLM_FORCE_ALLREDUCE_BACKEND", "bogus")
    with pytest.raises(ValueError):
        va.forced_backend()
    monkeypatch.setenv("VLLM_OOVERLAP_RR_DTYPE", "int8")
    with pytest.raises(ValueError):
        va.OoverlapAllReduce(communicator=FakeComm())


def test_short_broker_key():
    key = va.short_broker_key("a/b:c" * 40)
    assert len(key) <= 48 and key.startswith("vllm_") and "/" not in key and ":" not in key


def test_install_patches_vllm_communicator(monkeypatch):
    """With the backend forced, CudaCommunicator gets an OoverlapAllReduce as ca_comm and the other fast paths
    are switched off (vLLM's own classes are replaced by stand-ins; no GPU is touched)."""
    cc = pytest.importorskip("vllm.distributed.device_communicators.cuda_communicator")
    monkeypatch.setenv("VLLM_FORCE_ALLREDUCE_BACKEND", "ooverlap")
    monkeypatch.setattr(va, "_installed", False)
    built = {}

    class FakeBackend(va.OoverlapAllReduce):
        def __init__(self, group=None, device=None, **kw):
            built["args"] = (group, device)
            self.disabled = False

        def all_gather(self, inp, dim=-1):
            return "gathered"

        def close(self):
            built["closed"] = True

    monkeypatch.setattr(va, "OoverlapAllReduce", FakeBackend)
    orig_init, orig_ag, orig_destroy = cc.CudaCommunicator.__init__, cc.CudaCommunicator.all_gather, cc.CudaCommunicator.destroy

    def fake_init(self, *a, **k):
        self.world_size, self.cpu_group, self.device = 2, "cpu-group", "cuda:0"
        self.ca_comm, self.qr_comm, self.fi_ar_comm, self.symm_mem_comm = "vllm-ca", None, None, "symm"

    monkeypatch.setattr(cc.CudaCommunicator, "__init__", fake_init)
    monkeypatch.setattr(cc.CudaCommunicator, "destroy", lambda self: built.setdefault("orig_destroy", True))
    try:
        assert va.install() is True
        c = cc.CudaCommunicator()
        assert isinstance(c.ca_comm, FakeBackend) and built["args"] == ("cpu-group", "cuda:0")
        assert c.symm_mem_comm is None
        assert c.all_gather(torch.zeros(2), 0) == "gathered"
        c.destroy()
        assert built.get("closed") and built.get("orig_destroy")
    finally:
        cc.CudaCommunicator.__init__, cc.CudaCommunicator.all_gather, cc.CudaCommunicator.destroy = orig_init, orig_ag, orig_destroy
        va._installed = False


def test_row_parallel_eligibility_and_custom_op():
    """The direct-slot row-parallel path is taken only for bias-free, unquantised, reduced layers whose result fits
    a slot; the torch custom op dispatches to the registered backend and has a shape-only (fake) implementation."""

    class UnquantizedLinearMethod:  # same class NAME as vLLM's; the check is by name
        pass

    class Layer:
        reduce_results, tp_size, input_is_parallel, bias, return_bias = True, 2, True, None, False
        quant_method = UnquantizedLinearMethod()
        weight = torch.zeros(16, 8, dtype=torch.bfloat16)

    class Backend(va.OoverlapAllReduce):
        def __init__(self):
            self.disabled, self.rr_dtype, self.rr_capacity = False, torch.bfloat16, 1 << 20
            self.calls = 0

        def row_parallel(self, x, weight):
            self.calls += 1
            return (x.float() @ weight.float().t()).to(x.dtype) * 2  # stand-in for GEMM + 2-rank all-reduce

    b = Backend()
    x = torch.ones(4, 8, dtype=torch.bfloat16)
    # CPU tensors are never eligible (the kernels need CUDA memory) ...
    assert not va.row_parallel_eligible(Layer(), x, b)
    # ... every other condition is checked on a meta-free stand-in that claims to be on the GPU
    class CudaLike:
        def __init__(self, t):
            self._t = t
            self.dtype, self.shape, self.is_cuda = t.dtype, t.shape, True

        def numel(self):
            return self._t.numel()

        def is_contiguous(self):
            return True

        def element_size(self):
            return self._t.element_size()

    xc = CudaLike(x)
    assert va.row_parallel_eligible(Layer(), xc, b)
    for attr, val in (("reduce_results", False), ("tp_size", 1), ("input_is_parallel", False), ("bias", torch.zeros(16))):
        layer = Layer()
        setattr(layer, attr, val)
        assert not va.row_parallel_eligible(layer, xc, b), attr
    quant = Layer()
    quant.quant_method = object()
    assert not va.row_parallel_eligible(quant, xc, b)
    small = Backend()
    small.rr_capacity = 16
    assert not va.row_parallel_eligible(Layer(), xc, small)
    assert not va.row_parallel_eligible(Layer(), xc, "vllm-ca")
    # the custom op: real dispatch and fake (meta) shape inference
    va._row_parallel_backend = b
    try:
        out = torch.ops.ooverlap_b200.row_parallel_linear(x, Layer.weight)
        assert out.shape == (4, 16) and b.calls == 1
        meta = torch.ops.ooverlap_b200.row_parallel_linear(x.to("meta"), Layer.weight.to("meta"))
        assert meta.shape == (4, 16) and meta.device.type == "meta"
        va._row_parallel_backend = None
        with pytest.raises(RuntimeError):
            torch.ops.ooverlap_b200.row_parallel_linear(x, Layer.weight)
    finally:
        va._row_parallel_backend = None


def test_row_parallel_patch_falls_back_to_vllm(monkeypatch):
    """With VLLM_OOVERLAP_ROW_PARALLEL the patched RowParallelLinear.forward defers to vLLM's own forward for any
    call that is not eligible (here: no tensor-parallel group exists)."""
    vl = pytest.importorskip("vllm.model_executor.layers.linear")
    orig = vl.RowParallelLinear.forward
    seen = {}
    monkeypatch.setattr(vl.RowParallelLinear, "forward", lambda self, x: seen.setdefault("orig", x))
    try:
        assert va._patch_row_parallel_linear()

        class L:
            reduce_results, tp_size, input_is_parallel, bias, return_bias = True, 2, True, None, False

        out = vl.RowParallelLinear.forward(L(), torch.ones(2, 8))
        assert out is seen["orig"]
    finally:
        vl.RowParallelLinear.forward = orig


def test_forced_all_reduce_serves_or_raises(adapter, monkeypatch):
    """A forced backend serves every all-reduce or raises (no silent fall-through); tensors larger than a slot go
    through the ring in pieces; with VLLM_OOVERLAP_STRICT=0 the rest is counted and handed on."""
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))

    class Host:  # stands in for vLLM's CudaCommunicator
        ca_comm = adapter
        pynccl_comm = None

    def original(self, t):
        return "vllm-chain"

    small = torch.ones(8, 16)
    assert torch.equal(va.forced_all_reduce(Host(), small, "ooverlap", original), small * 4)
    big = torch.ones(64, 64)  # 16 KiB against 4 KiB slots: four pieces of 16 rows
    out = va.forced_all_reduce(Host(), big, "ooverlap", original)
    assert torch.equal(out, big * 4) and out.data_ptr() != big.data_ptr()
    assert adapter.stats() == {"served": 1, "served_in_pieces": 1, "declined": {}}
    assert [c for c in adapter.comm.calls if c[0] == "ar"][-4:] == [("ar", (16, 64))] * 4
    wrong = torch.ones(8, 16, dtype=torch.float16)
    monkeypatch.setenv("VLLM_OOVERLAP_STRICT", "1")
    with pytest.raises(RuntimeError, match="cannot be served"):
        va.forced_all_reduce(Host(), wrong, "ooverlap", original)
    monkeypatch.setenv("VLLM_OOVERLAP_STRICT", "0")
    assert va.forced_all_reduce(Host(), wrong, "ooverlap", original) == "vllm-chain"
    assert sum(adapter.stats()["declined"].values()) == 2
    # the comparison arms raise as well when their backend is missing
    with pytest.raises(RuntimeError, match="pynccl"):
        va.forced_all_reduce(Host(), small, "pynccl", original)

    class NoBackend:
        ca_comm = None

    with pytest.raises(RuntimeError):
        va.forced_all_reduce(NoBackend(), small, "ooverlap", original)
    with pytest.raises(RuntimeError, match="custom"):
        va.forced_all_reduce(NoBackend(), small, "custom", original)

    class Pynccl:
        disabled = False

        def all_reduce(self, t):
            return t + 1

    class Host2:
        ca_comm = None
        pynccl_comm = Pynccl()

    assert torch.equal(va.forced_all_reduce(Host2(), small, "pynccl", original), small + 1)


def test_stats_file_written_at_close(adapter, monkeypatch, tmp_path):
    import json
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    path = tmp_path / "stats.jsonl"
    monkeypatch.setenv("VLLM_OOVERLAP_STATS_FILE", str(path))
    adapter.custom_all_reduce(torch.ones(8, 16))
    adapter.custom_all_reduce(torch.ones(3))
    adapter.close()
    rec = json.loads(path.read_text().strip())
    assert rec["served"] == 1 and rec["declined"] == {"size is not a multiple of 16 bytes": 1} and rec["world"] == 4
