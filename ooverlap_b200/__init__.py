"""ooverlap_b200 — Blackwell-native intra-node collectives and GEMM/collective overlap.

Public surface:

* :class:`Communicator` — ``all_reduce`` / ``reduce_scatter`` / ``all_gather`` on
  registered buffers, slot pools, CPU (gloo) fallback.
* :mod:`ooverlap_b200.ops` — tcgen05 GEMM, fused GEMM->AllReduce,
  GEMM->ReduceScatter+residual+RMSNorm, AllGather->GEMM, fused
  AllReduce+residual+RMSNorm.
* :mod:`ooverlap_b200.parallel` — tensor-parallel linear layers and the vLLM
  custom-all-reduce hook.
* :mod:`ooverlap_b200.models` — a Llama-architecture tensor-parallel model used
  by the serving benchmark.
"""
from . import _lib  # noqa: F401
from ._lib import DeviceTimeout, OobError  # noqa: F401
from .comm import Communicator, SlotPool  # noqa: F401
from .emulated import EmulatedGroup  # noqa: F401

__version__ = "0.2.0"


def build(force: bool = False):
    """Compile the native library for sm_100a (no-op when the in-tree binary is current)."""
    from . import _build
    return _build.build(force=force)


def topology(run_probes: bool = False) -> dict:
    """Topology of the visible GPUs as a dict (see ``lib/oob_topology`` for the CLI)."""
    import ctypes
    import json
    buf = ctypes.create_string_buffer(1 << 20)
    _lib.check(_lib.lib().oob_topology_json(buf, len(buf), 1 if run_probes else 0))
    return json.loads(buf.value.decode())
