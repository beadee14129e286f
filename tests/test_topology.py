"""Topology document and its CLI.  On a machine without GPUs the document is empty but well formed; on GPUs the live
probes (remote ld/st, remote atomic, timed peer copy, multimem over all devices) must all pass."""
import json
import os
import subprocess

import pytest
import torch

import ooverlap_b200 as oob
from ooverlap_b200 import _lib

CLI = os.path.join(os.path.dirname(oob.__file__), "lib", "oob_topology")
HAS_GPU = torch.cuda.is_available()


def _cli(*args):
    return subprocess.run([CLI, *args], capture_output=True, text=True, timeout=300)


def test_cli_switches_parse():
    assert _cli("--help").returncode == 0
    bad = _cli("--bogus")
    assert bad.returncode == 2 and "unknown option" in bad.stderr
    r = _cli("--json", "--no-probe", "--no-enable-peer", "--no-atomic-probe", "--no-copy-probe", "--no-multimem-probe",
             "--no-bulk-probe", "--no-tma-probe", "--no-shm")
    assert r.returncode == 0, r.stderr
    doc = json.loads(r.stdout)
    assert doc["device_count"] == len(doc["devices"]) and doc["probe_multimem"] == -1
    assert all(l["probe_ldst"] == -1 and l["copy_gbs"] == 0 for l in doc["links"])


def test_unknown_device_is_an_error():
    with pytest.raises(_lib.OobError):
        oob.topology(devices=[63])
    r = _cli("--no-probe", "63")
    assert r.returncode == 1 and "not visible" in r.stderr


@pytest.mark.skipif(HAS_GPU, reason="the empty document is what a machine without GPUs reports")
def test_document_without_gpus():
    doc = oob.topology()
    assert doc == {"devices": [], "links": [], "all_pairs_nvlink": False, "all_pairs_p2p": False, "probe_multimem": -1,
                   "probe_multimem_note": "not run", "device_count": 0}
    assert "0 device(s)" in oob.topology(text=True)
    assert _cli("--require-peer", "--no-probe").returncode == 0  # nothing to require between zero devices


@pytest.mark.gpu
def test_probes_pass_on_every_pair():
    n = torch.cuda.device_count()
    doc = oob.topology(run_probes=True)
    assert doc["device_count"] == n and len(doc["links"]) == n * (n - 1)
    for d in doc["devices"]:
        assert d["cc"] == "10.0" and d["sms"] >= 100 and d["memory_bytes"] > (100 << 30)
    for l in doc["links"]:
        assert l["p2p"] == 1 and l["kind"] == "nvlink", l
        assert l["probe_ldst"] == 1 and l["probe_atomic"] == 1 and l["probe_bulk_store"] == 1 and l["copy_gbs"] > 100.0, l
    if n >= 2:
        assert doc["all_pairs_nvlink"] and doc["all_pairs_p2p"]
        assert doc["probe_multimem"] == 1, doc["probe_multimem_note"]
        text = oob.topology(run_probes=True, copy_probe=False, text=True)
        assert "multimem probe: ok" in text and "nvlink" in text
        assert _cli("--require-peer", "--no-copy-probe").returncode == 0
    else:
        assert doc["probe_multimem"] == -1 and "two or more" in doc["probe_multimem_note"]
    # single switches: without the atomic probe the column stays "not run"
    doc = oob.topology(run_probes=True, atomic_probe=False, copy_probe=False, multimem_probe=False, devices=list(range(min(n, 2))))
    assert all(l["probe_atomic"] == -1 and l["probe_ldst"] == 1 for l in doc["links"])
    doc = oob.topology(run_probes=True, enable_peer=False, multimem_probe=False)
    assert all(l["probe_ldst"] == -1 for l in doc["links"])
