"""Host-side pieces of bench.py that need no GPU: a multi-GPU run's ranks keep their threads next to their GPU
(the affinity comes from a fake NVML here), and the workload descriptions of the two arms agree."""
import os
import sys
import types

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402
from qubivex_b200 import workload as wl  # noqa: E402


def _fake_nvml(mask_words):
    m = types.ModuleType("pynvml")
    m.nvmlInit = lambda: None
    m.nvmlDeviceGetHandleByPciBusId = lambda bus: ("by-bus", bus)
    m.nvmlDeviceGetHandleByIndex = lambda i: ("by-index", i)
    m.nvmlDeviceGetCpuAffinity = lambda h, n: list(mask_words)[:n] + [0] * max(0, n - len(mask_words))
    m.NVML_AFFINITY_SCOPE_NODE = 0
    m.nvmlDeviceGetMemoryAffinity = lambda h, n, scope: [0]          # no node reported: the policy stays
    return m


def test_a_rank_binds_to_the_allowed_cores_next_to_its_gpu(monkeypatch):
    allowed = {0, 1, 2, 3, 8, 9}
    bound = {}
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(allowed))
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cores: bound.update(cores=set(cores)))
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml([0b1100001100]))   # cores 2, 3, 8, 9 next to the GPU
    said = bench.bind_near_gpu(0)
    assert bound["cores"] == {2, 3, 8, 9} and said.startswith("4 of 6") and "memory policy unchanged (no node reported)" in said


def test_nothing_is_bound_when_the_gpus_cores_are_not_allowed_or_are_all_of_them(monkeypatch):
    calls = []
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: {0, 1})
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cores: calls.append(cores))
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml([0b110000]))       # cores 4, 5: none allowed here
    assert bench.bind_near_gpu(0).startswith("cores unchanged")
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml([0b11]))           # exactly the allowed ones
    assert bench.bind_near_gpu(0).startswith("cores unchanged")
    assert calls == []


def test_no_nvml_leaves_the_run_unbound(monkeypatch):
    broken = types.ModuleType("pynvml")

    def boom():
        raise RuntimeError("no driver")
    broken.nvmlInit = boom
    monkeypatch.setitem(sys.modules, "pynvml", broken)
    assert bench.bind_near_gpu(3) == "unchanged (RuntimeError)"


def test_both_arms_describe_the_workload_with_the_same_keys():
    c = bench.config_of(wl.C2, wl.C2.layers)
    assert c["workload"] == wl.C2.name and c["layers"] == 48 and c["batch_per_gpu"] == 64
    assert set(c) >= {"workload", "layers", "batch_per_gpu", "heads", "kv_heads", "head_dim", "block_tokens", "context", "partition", "l2"}


def test_the_memory_policy_prefers_the_gpus_node_or_says_why_not():
    import ctypes
    fake = _fake_nvml([0b1])
    fake.nvmlDeviceGetMemoryAffinity = lambda h, n, scope: [0b1]     # node 0: every machine has it
    said = bench.prefer_memory_near_gpu(fake, "handle")
    try:
        assert said == "memory preferred on node 0" or said.startswith("memory policy unchanged (set_mempolicy: errno")
    finally:
        if os.uname().machine == "x86_64":
            ctypes.CDLL(None).syscall(238, 0, None, 0)               # back to the default policy
