"""HostPipeline: inputs prefetched from pinned host memory and results read back one step late must be the data of
the right step, whatever the overlap."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pipeline_delivers_every_step_in_order():
    from ooverlap_b200.utils.hostio import HostPipeline
    steps, rows, cols = 12, 2048, 1024
    host = [torch.full((rows, cols), float(i + 1), dtype=torch.float16).pin_memory() for i in range(steps)]
    back = [torch.empty(cols, dtype=torch.float16).pin_memory() for _ in range(2)]
    io = HostPipeline({"x": (rows, cols)}, torch.float16, depth=2)
    out = torch.empty(rows, cols, dtype=torch.float16, device="cuda")
    got, pending = [], None
    io.feed({"x": host[0]})
    for i in range(steps):
        dev = io.take()
        if i + 1 < steps:
            io.feed({"x": host[i + 1]})
        torch.mul(dev["x"], 2.0, out=out)      # the step's "kernel"; overwrites the same output every step
        for _ in range(20):                    # keep the stream busy so that copies really overlap
            out.add_(0.0)
        io.done()
        fut = io.read_back(out[0], back[i & 1])
        if pending is not None:
            got.append(float(pending.wait()[0]))
        pending = fut
    got.append(float(pending.wait()[0]))
    assert got == [2.0 * (i + 1) for i in range(steps)]
    assert io.h2d_bytes == steps * rows * cols * 2 and io.d2h_bytes == steps * cols * 2


def test_pipeline_guards():
    from ooverlap_b200.utils.hostio import HostPipeline
    io = HostPipeline({"x": (4, 4)}, torch.float32, depth=2)
    x = torch.zeros(4, 4).pin_memory()
    with pytest.raises(RuntimeError):
        io.take()
    with pytest.raises(ValueError):
        io.feed({"x": torch.zeros(4, 4)})      # not pinned
    io.feed({"x": x})
    io.feed({"x": x})
    with pytest.raises(RuntimeError):
        io.feed({"x": x})                      # both buffers in use
    with pytest.raises(RuntimeError):
        io.done()                              # nothing taken yet
    io.take()
    io.done()
    io.feed({"x": x})
    with pytest.raises(ValueError):
        HostPipeline({"x": (4, 4)}, torch.float32, depth=1)
    torch.cuda.synchronize()
