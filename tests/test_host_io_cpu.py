"""Host-side helpers of the host<->device plumbing that need no GPU."""
import os

import pytest


def test_chunk_schedule_covers_the_layer_on_16_element_boundaries():
    from slideformer_b200.host_io import chunk_schedule
    for n in (0, 5, 4 << 20, 218_112_000, (64 << 20) + 7, 100_000_003):
        pieces = chunk_schedule(n, 16 << 20, 4 << 20)
        pos = 0
        for a, b in pieces:
            assert a == pos and b > a
            assert a % 16 == 0
            pos = b
        assert pos == n
    with pytest.raises(ValueError):
        chunk_schedule(100, 24, 8)


def test_numa_cpus_from_a_fake_sysfs(tmp_path):
    from slideformer_b200.numa import _parse_cpulist, numa_cpus_of_pci
    assert _parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("16-31\n")
    assert numa_cpus_of_pci("0000:1b:00.0", str(tmp_path)) == set(range(16, 32))
    (dev / "numa_node").write_text("-1\n")                       # the kernel's "unknown"
    assert numa_cpus_of_pci("0000:1b:00.0", str(tmp_path)) is None
    assert numa_cpus_of_pci("0000:ff:00.0", str(tmp_path)) is None


def test_numa_local_restores_the_cpu_mask():
    from slideformer_b200.host_io import numa_local
    before = os.sched_getaffinity(0)
    with numa_local("cuda:0"):     # no GPU here: the body runs where it is
        pass
    assert os.sched_getaffinity(0) == before
