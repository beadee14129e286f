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
from .local_group import LocalGroup  # noqa: F401

__version__ = "0.2.0"


def build(force: bool = False):
    """Compile the native library for sm_100a (no-op when the in-tree binary is current)."""
    from . import _build
    return _build.build(force=force)


def topology(run_probes: bool = False, *, devices=None, enable_peer: bool = True, atomic_probe: bool = True,
             copy_probe: bool = True, multimem_probe: bool = True, bulk_probe: bool = True, require_peer: bool = False,
             text: bool = False):
    """Topology of the visible GPUs (or of ``devices``) as a dict, or as a table when ``text`` is set (the CLI
    ``lib/oob_topology`` prints the same).  ``run_probes`` runs the live probes: per directed pair a remote store / load,
    a remote atomic, a bulk store from shared memory and a timed peer copy, and over all devices a multimem store / add / in-switch sum; the keyword
    switches take single probes out (``enable_peer=False``: peer access is never switched on, so no per-pair probe
    runs).  ``require_peer`` raises ``OobError`` when a pair has no peer access."""
    import ctypes
    import json
    flags = _lib.TOPO_PROBES if run_probes else 0
    flags |= 0 if enable_peer else _lib.TOPO_NO_ENABLE_PEER
    flags |= 0 if atomic_probe else _lib.TOPO_NO_ATOMIC_PROBE
    flags |= 0 if copy_probe else _lib.TOPO_NO_COPY_PROBE
    flags |= 0 if multimem_probe else _lib.TOPO_NO_MULTIMEM_PROBE
    flags |= 0 if bulk_probe else _lib.TOPO_NO_BULK_PROBE
    flags |= _lib.TOPO_REQUIRE_PEER if require_peer else 0
    flags |= _lib.TOPO_TEXT if text else 0
    devs = [int(d) for d in devices] if devices else []
    arr = (ctypes.c_int * len(devs))(*devs) if devs else None
    buf = ctypes.create_string_buffer(1 << 20)
    _lib.check(_lib.lib().oob_topology_describe(buf, len(buf), flags, arr, len(devs)))
    out = buf.value.decode()
    return out if text else json.loads(out)
