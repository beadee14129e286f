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
