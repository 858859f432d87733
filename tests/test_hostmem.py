"""Host placement helpers (llm720_b200/hostmem.py) against a fake sysfs tree: which cores and memory node
belong to a GPU, how ranks that share a core list split it, and that nothing breaks when the topology is
not visible.  No GPU needed; the binding itself is exercised on the calling process and undone."""
import os

from llm720_b200 import hostmem


def _fake_sysfs(tmp_path, addr, cpulist, node):
    d = tmp_path / addr
    d.mkdir(parents=True)
    (d / "local_cpulist").write_text(cpulist + "\n")
    (d / "numa_node").write_text(str(node) + "\n")
    return str(tmp_path)


def test_cpulist_parsing_and_rank_shares():
    assert hostmem._parse_cpulist("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]
    cpus = list(range(32))
    shares = [hostmem.slice_for_rank(cpus, r, 8) for r in range(8)]
    assert all(len(s) == 4 for s in shares)
    assert sorted(c for s in shares for c in s) == cpus            # disjoint and complete
    assert hostmem.slice_for_rank(cpus, 0, 1) == cpus
    assert hostmem.slice_for_rank([0, 1], 3, 8) == [0, 1]          # fewer cores than ranks: no split


def test_locality_from_sysfs(tmp_path, monkeypatch):
    root = _fake_sysfs(tmp_path, "0000:1b:00.0", "0-3", 1)
    monkeypatch.setattr(hostmem, "pci_address", lambda i: "0000:1b:00.0")
    info = hostmem.gpu_locality(0, root)
    assert info == {"pci": "0000:1b:00.0", "numa_node": 1, "cpus": [0, 1, 2, 3]}
    root2 = _fake_sysfs(tmp_path / "b", "0000:1c:00.0", "", -1)     # a host that exposes nothing
    monkeypatch.setattr(hostmem, "pci_address", lambda i: "0000:1c:00.0")
    assert hostmem.gpu_locality(0, root2) == {"pci": "0000:1c:00.0", "numa_node": None, "cpus": []}
    monkeypatch.setattr(hostmem, "pci_address", lambda i: None)
    assert hostmem.gpu_locality(0, root)["cpus"] == []


def test_binding_restricts_to_local_cores_and_is_reversible(tmp_path, monkeypatch):
    before = os.sched_getaffinity(0)
    allowed = sorted(before)
    local = allowed[: max(1, len(allowed) // 2)]
    root = _fake_sysfs(tmp_path, "0000:1b:00.0", ",".join(str(c) for c in local), -1)
    monkeypatch.setattr(hostmem, "pci_address", lambda i: "0000:1b:00.0")
    try:
        done = hostmem.bind_process_to_gpu(0, 0, 1, root)
        assert sorted(os.sched_getaffinity(0)) == local
        assert done["cpus_bound"] is not None and done["mempolicy"] is False
        # no topology: the allowed set is split among the ranks of the host instead
        os.sched_setaffinity(0, before)
        monkeypatch.setattr(hostmem, "pci_address", lambda i: None)
        hostmem.bind_process_to_gpu(0, 1, 2, root)
        if len(allowed) >= 2:
            assert sorted(os.sched_getaffinity(0)) == allowed[len(allowed) // 2: 2 * (len(allowed) // 2)]
    finally:
        os.sched_setaffinity(0, before)
