"""Host-side placement helpers of the host-buffer path (no GPU needed): the CPU list of a PCIe
slot is parsed from a fake sysfs tree, and binding is a no-op when the topology is unknown."""
from __future__ import annotations

import os
from types import SimpleNamespace

import pytest

from fhob import hostmem


def test_cpulist_parsing():
    assert hostmem._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert hostmem._parse_cpulist("5") == {5}
    assert hostmem._parse_cpulist("") == set()


def _fake_device(monkeypatch, tmp_path, cpulist, node):
    bdf = "0000:53:00.0"
    dev_dir = tmp_path / bdf
    dev_dir.mkdir()
    (dev_dir / "local_cpulist").write_text(cpulist)
    (dev_dir / "numa_node").write_text(f"{node}\n")
    props = SimpleNamespace(pci_domain_id=0, pci_bus_id=0x53, pci_device_id=0)
    monkeypatch.setattr(hostmem.torch.cuda, "get_device_properties", lambda device: props)
    return bdf


def test_device_topology_is_read_from_sysfs(monkeypatch, tmp_path):
    bdf = _fake_device(monkeypatch, tmp_path, "0-1,4\n", 1)
    info = hostmem.device_local_cpus(0, sysfs=str(tmp_path))
    assert info == dict(pci=bdf, numa_node=1, cpus={0, 1, 4})
    assert hostmem.device_local_cpus(0, sysfs=str(tmp_path / "missing")) is None


def test_binding_narrows_the_affinity_and_restores_it(monkeypatch, tmp_path):
    before = os.sched_getaffinity(0)
    if len(before) < 2:
        pytest.skip("needs two allowed CPUs")
    keep = sorted(before)[:1]
    _fake_device(monkeypatch, tmp_path, ",".join(map(str, keep)), 0)
    real = hostmem.device_local_cpus
    monkeypatch.setattr(hostmem, "device_local_cpus", lambda device: real(device, sysfs=str(tmp_path)))
    with hostmem.near_device(0) as rec:
        assert rec["bound"] and rec["cpus"] == 1 and rec["numa_node"] == 0
        assert os.sched_getaffinity(0) == set(keep)
    assert os.sched_getaffinity(0) == before


def test_binding_is_a_no_op_without_topology(monkeypatch):
    monkeypatch.setattr(hostmem, "device_local_cpus", lambda device: None)
    before = os.sched_getaffinity(0)
    with hostmem.near_device(0) as rec:
        assert rec == dict(bound=False)
        assert os.sched_getaffinity(0) == before


def test_head_ranges_of_the_host_buffer_path():
    """Ranges cover every head once, in order; there are at least four when there are that many
    heads; no range is larger than the requested bytes allow (one head at least); and the last
    range is cut into a half and two quarters so that the un-overlapped tail is short."""
    from fhob import ops
    for bh in (1, 2, 3, 4, 5, 7, 16, 63, 64, 512, 1025):
        for head_bytes, range_bytes in ((1 << 20, 192 << 20), (12 << 20, 192 << 20), (300 << 20, 192 << 20), (1, 1)):
            b = ops._host_ranges(bh, head_bytes, range_bytes)
            assert b[0] == 0 and b[-1] == bh
            sizes = [hi - lo for lo, hi in zip(b, b[1:])]
            assert all(s > 0 for s in sizes), (bh, head_bytes, sizes)
            assert len(sizes) >= min(bh, 4)
            per_range = max(1, range_bytes // head_bytes)
            assert max(sizes) <= per_range + 1           # even split of bh over ceil(bh / per_range) ranges
            if len(sizes) >= 6 and sizes[0] >= 4:
                assert sizes[-1] <= sizes[0] // 4 + 1 and sizes[-2] <= sizes[0] // 4 + 1
    # the 512-head cross-attention job: 12.6 MB of input per head -> 15 heads per range
    b = ops._host_ranges(512, 12599296, 192 << 20)
    sizes = [hi - lo for lo, hi in zip(b, b[1:])]
    assert max(sizes) <= 15 and sizes[-3:] == [9, 3, 3] and sum(sizes) == 512
