"""Host-memory placement helpers against a fake sysfs tree and fake system calls."""

import os
from unittest import mock

from ep_xpress_b200.utils import numa


def make_sysfs(tmp_path, node_of_device=1):
    device = tmp_path / "bus/pci/devices/0000:1b:00.0"
    device.mkdir(parents=True)
    (device / "numa_node").write_text(f"{node_of_device}\n")
    for node, cpus in ((0, "0-3,8-11"), (1, "4-7,12-15")):
        directory = tmp_path / f"devices/system/node/node{node}"
        directory.mkdir(parents=True)
        (directory / "cpulist").write_text(cpus + "\n")
    return str(tmp_path)


def test_cpu_list_and_pci_address():
    assert numa.parse_cpu_list("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert numa.parse_cpu_list("") == []
    assert numa.pci_address(0, 0x1B, 0) == "0000:1b:00.0"


def test_node_lookup_and_missing_information(tmp_path):
    sysfs = make_sysfs(tmp_path)
    assert numa.node_of_pci_device("0000:1b:00.0", sysfs) == 1
    assert numa.node_of_pci_device("0000:ff:00.0", sysfs) == -1
    assert numa.node_of_pci_device(None, sysfs) == -1
    assert numa.node_cpus(1, sysfs) == [4, 5, 6, 7, 12, 13, 14, 15] and numa.node_cpus(7, sysfs) == []


def test_binding_stays_inside_the_current_affinity_mask(tmp_path):
    sysfs = make_sysfs(tmp_path)
    calls = []
    record = numa.bind_to_node(1, sysfs, set_affinity=lambda pid, cpus: calls.append((pid, list(cpus))),
                               get_affinity=lambda pid: {0, 1, 4, 5, 12}, prefer=lambda node: True)
    assert calls == [(0, [4, 5, 12])]
    assert record == {"node": 1, "bound": True, "cpus": 3, "memory_policy": True}


def test_binding_degrades_to_a_recorded_no_op(tmp_path):
    sysfs = make_sysfs(tmp_path)
    untouched = lambda *a: (_ for _ in ()).throw(AssertionError("must not be called"))   # noqa: E731
    assert numa.bind_to_node(-1, sysfs, set_affinity=untouched)["bound"] is False
    outside = numa.bind_to_node(0, sysfs, set_affinity=untouched, get_affinity=lambda pid: {4, 5})
    assert outside["bound"] is False and "affinity mask" in outside["reason"]

    def refuse(pid, cpus):
        raise PermissionError("no")
    refused = numa.bind_to_node(0, sysfs, set_affinity=refuse, get_affinity=lambda pid: {0, 1})
    assert refused["bound"] is False and "sched_setaffinity failed" in refused["reason"]


def test_pages_by_node_picks_the_containing_mapping(tmp_path):
    maps = tmp_path / "numa_maps"
    maps.write_text("7f0000000000 default anon=16 dirty=16 N0=16 kernelpagesize_kB=4\n"
                    "7f0000100000 prefer:1 file=/dev/zero mapped=4096 N0=96 N1=4000 kernelpagesize_kB=4\n"
                    "7f0000900000 default anon=1 N0=1\n")
    assert numa.pages_by_node(0x7F0000100000, str(maps)) == {0: 96, 1: 4000}
    assert numa.pages_by_node(0x7F0000100000 + 4096 * 10, str(maps)) == {0: 96, 1: 4000}
    assert numa.pages_by_node(0x1000, str(maps)) == {}
    assert numa.pages_by_node(0x1000, str(tmp_path / "missing")) == {}


def test_prefer_node_never_raises():
    assert numa.prefer_node(-1) is False
    assert numa.prefer_node(0) in (True, False)        # allowed or refused, depending on the sandbox
    assert isinstance(os.sched_getaffinity(0), set)


class FakeNvml:
    def __init__(self, mask, fail=False):
        self.mask, self.fail, self.asked = mask, fail, None

    def nvmlInit(self):
        if self.fail:
            raise RuntimeError("no driver")

    def nvmlDeviceGetHandleByPciBusId(self, address):
        self.asked = address
        return "handle"

    def nvmlDeviceGetCpuAffinity(self, handle, words):
        return (self.mask + [0] * words)[:words]


def test_driver_topology_is_the_fallback_when_sysfs_is_hidden():
    nvml = FakeNvml([0b1111 << 4, 0b1])                       # CPUs 4..7 and 64
    with mock.patch.object(os, "cpu_count", lambda: 128):       # two mask words
        assert numa.nvml_cpu_affinity("0000:1b:00.0", nvml) == [4, 5, 6, 7, 64]
    assert nvml.asked == b"0000:1b:00.0"
    assert numa.nvml_cpu_affinity(None, nvml) == []
    assert numa.nvml_cpu_affinity("0000:1b:00.0", FakeNvml([], fail=True)) == []
    calls = []
    record = numa.bind_to_cpus([4, 5, 6, 7, 64], set_affinity=lambda pid, cpus: calls.append(list(cpus)),
                               get_affinity=lambda pid: set(range(0, 8)))
    assert calls == [[4, 5, 6, 7]] and record["bound"] and record["cpus"] == 4 and record["source"] == "nvml"
    nothing = numa.bind_to_cpus([], set_affinity=lambda *a: calls.append("never"), get_affinity=lambda pid: {0})
    assert not nothing["bound"] and "never" not in calls
