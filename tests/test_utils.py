"""Shared utilities: logger, metrics, step gate, device lock, ledger, the CPU face."""
import os

import pytest
import torch

from owl_engine_b200.utils import device, log, metrics, stepgate, testkit


def test_logger_filters_and_ring(tmp_path, capsys):
    L = log.Logger()
    L.configure(level="info", tags_allow=["store"], tags_deny=["store.noisy"], path=str(tmp_path / "l.log"), max_mb=0)
    L.emit("info", "store.evict", "a")
    L.emit("debug", "store.evict", "b")
    L.emit("info", "store.noisy.x", "c")
    L.emit("error", "engine", "d")
    assert [l.split("] ")[1] for l in L.tail()] == ["a"]
    L.set_level("debug"); L.set_tags([])
    L.emit("debug", "engine", "e")
    assert L.tail()[-1].endswith("e") and "a" in open(tmp_path / "l.log").read()


def test_metrics_tree_and_dumps():
    M = metrics.Metrics()
    with M.timer("pump"):
        with M.timer("pump.schedule"):
            pass
        with M.timer("pump.decode"):
            M.count("tokens", 3)
    snap = M.snapshot()
    assert snap["timers"]["pump.decode"]["parent"] == "pump" and snap["counters"]["tokens"] == 3
    assert M.tree()["roots"][0]["tag"] == "pump" and len(M.tree()["roots"][0]["children"]) == 2
    assert "pump.schedule" in M.dump_csv() and "timers" in M.dump_json()
    M.set_level("off")
    with M.timer("x"):
        pass
    assert "x" not in M.snapshot()["timers"]


def test_stepgate_single_step():
    import threading
    G = stepgate.StepGate()
    G.configure("single")
    hits = []
    t = threading.Thread(target=lambda: (G.checkpoint("a"), hits.append(1), G.checkpoint("b"), hits.append(2)))
    t.start()
    import time
    time.sleep(0.1)
    assert hits == [] and G.status()["parked_at"] == "a"
    G.step(); time.sleep(0.2)
    assert hits == [1]
    G.configure("off"); t.join(2)
    assert hits == [1, 2]


class FakeNvml:
    class _Pci:
        def __init__(self, b): self.busId = b
    class _Mem:
        total = 180 << 30
    def nvmlInit(self): pass
    def nvmlDeviceGetCount(self): return 2
    def nvmlDeviceGetHandleByIndex(self, i): return i
    def nvmlDeviceGetUUID(self, h): return f"GPU-aaaa-{h}"
    def nvmlDeviceGetPciInfo(self, h): return self._Pci(f"00000000:{h+1:02x}:00.0")
    def nvmlDeviceGetName(self, h): return "NVIDIA B200"
    def nvmlDeviceGetMemoryInfo(self, h): return self._Mem()


def test_device_selection_and_lock(tmp_path):
    devs = device.enumerate_devices(FakeNvml())
    assert [d.index for d in device.resolve(["GPU-AAAA-1", "find:b200"], devs)] == [1, 0]
    assert device.resolve(["02:00.0"], devs)[0].index == 1
    with pytest.raises(LookupError):
        device.resolve(["GPU-nope"], devs)
    a = device.GpuLock("u1", str(tmp_path)); a.acquire()
    open(a.path, "w").write("999999999")          # pretend a dead process holds it
    b = device.GpuLock("u1", str(tmp_path)); b.acquire(); b.release()
    open(a.path, "w").write(str(os.getppid()))    # a live foreign pid
    with pytest.raises(RuntimeError):
        device.GpuLock("u1", str(tmp_path)).acquire()


def test_testkit():
    r1, r2 = testkit.SplitMix64(7), testkit.SplitMix64(7)
    assert r1.next_u64() == r2.next_u64() and 0 <= r1.uniform() < 1
    rep = testkit.allclose(torch.tensor([1.0, 2.0]), torch.tensor([1.0, 2.1]), rtol=1e-3)
    assert not rep.ok and rep.worst_index == (1,) and "MISMATCH" in str(rep)


def test_kernel_registry_matches_sources_and_bindings():
    from owl_engine_b200.ops import registry as R

    assert R.cross_check() == []
    assert {k.entry for k in R.admit("gemm")} == {"owl_w4a16_gemm_tc", "owl_f16_gemm_tc", "owl_f16_gemm_persist",
                                                     "owl_f16_gemm_ag", "owl_f16_gemm_rs", "owl_e4m3_gemm",
                                                     "owl_f16_gemm_persist_f16out", "owl_nvfp4_gemm"}
    assert all("tcgen05" in k.gen for k in R.admit("gemm"))


def test_cpu_face_ledger_limits_and_capture_gate():
    import pytest
    import torch
    from owl_engine_b200.utils.cpuface import (CaptureUnsupported, CaptureViolation, CpuFace, MockLimits, OutOfMemory)

    dev = CpuFace(MockLimits(vram_bytes=4096, poison_uninit=True))
    a = dev.alloc((256,), owner="engine", klass="kv")          # 1 KiB
    b = dev.alloc((256,), owner="engine", klass="state")
    assert torch.isnan(dev.tensor(a)).all() and dev.ledger()[("engine", "kv")] == 1024
    with pytest.raises(OutOfMemory):
        dev.alloc((1024,), owner="engine", klass="kv")
    dev.register("axpy", lambda x, y, alpha=1.0: y.add_(alpha * x))
    dev.memset(a, 1.0); dev.memset(b, 0.0)
    dev.graph_begin()
    dev.launch("axpy", a, b, alpha=2.0)
    with pytest.raises(CaptureViolation):
        dev.free(a)
    g = dev.graph_end()
    dev.graph_launch(g)
    assert torch.allclose(dev.tensor(b), torch.full((256,), 4.0))       # once at capture, once at replay
    dev.free(a)
    assert dev.used == 1024 and dev.peak == 2048
    null = CpuFace(MockLimits(null_kernels=True, graph_capture=False))
    null.register("axpy", lambda x, y, alpha=1.0: y.add_(x))
    h = null.alloc((4,)); null.memset(h, 3.0)
    null.launch("axpy", h, h)
    assert null.launch_log == ["axpy"] and torch.allclose(null.tensor(h), torch.full((4,), 3.0))
    with pytest.raises(CaptureUnsupported):
        null.graph_begin()
