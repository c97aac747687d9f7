"""Tensor-parallel planning on the host: shard rules, peer classification against a fake NVML, the host relay over gloo."""
def test_peer_classification_limits_and_plan():
    """Reference rules (crates/backends/cuda/src/comm/peer.rs): P2P + both BAR1 wide -> static, both narrow -> window with
    the smaller aperture minus the reserve, mixed or no P2P -> refused; NVLink pairs bypass the aperture."""
    import pytest
    from owl_engine_b200.parallel import peer as P

    wide = P.PeerCaps("GPU-a", 32 << 30, True)
    wide2 = P.PeerCaps("GPU-b", 16 << 30, True)
    narrow = P.PeerCaps("GPU-c", 256 << 20, True)
    narrow2 = P.PeerCaps("GPU-d", 256 << 20, True)
    nop2p = P.PeerCaps("GPU-e", 32 << 30, False)
    b200 = [P.PeerCaps(f"GPU-n{i}", 256 << 30, True, nvlink=True) for i in range(8)]
    assert P.classify(wide, wide2) == "static" and P.per_alloc_limit("static", wide, wide2) == 192 << 20
    assert P.classify(narrow, narrow2) == "window" and P.per_alloc_limit("window", narrow, narrow2) == 192 << 20
    tiny = P.PeerCaps("GPU-f", 128 << 20, True)
    assert P.per_alloc_limit("window", narrow, tiny) == (128 - 64) << 20
    assert P.classify(wide, narrow) == "rejected" and P.classify(wide, nop2p) == "rejected"
    assert P.PeerPlan.plan(b200, 64 << 20).mechanism == "nvlink"
    assert P.PeerPlan.plan([wide, wide2], 64 << 20) == P.PeerPlan("static", 192 << 20, 64 << 20)
    with pytest.raises(P.PeerRejected):
        P.PeerPlan.plan([wide, wide2], 256 << 20)                 # over the per-allocation limit: refused, not shrunk
    with pytest.raises(P.PeerRejected):
        P.PeerPlan.plan([wide, wide2, narrow], 1 << 20)

    class FakeNvml:
        NVML_P2P_CAPS_INDEX_READ, NVML_P2P_STATUS_OK, NVML_NVLINK_MAX_LINKS = 0, 0, 2

        class _B:
            bar1Total = 256 << 30
        def nvmlInit(self): pass
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetBAR1MemoryInfo(self, h): return self._B()
        def nvmlDeviceGetP2PStatus(self, a, b, idx): return 0
        def nvmlDeviceGetNvLinkState(self, h, l): return 1
        def nvmlDeviceGetUUID(self, h): return f"GPU-{h}".encode()
    caps = P.probe([0, 1], FakeNvml())
    assert [c.uuid for c in caps] == ["GPU-0", "GPU-1"] and all(c.nvlink and c.p2p_supported for c in caps)


def _relay_worker(rank, world, port, q):
    import os
    import torch
    import torch.distributed as dist
    from owl_engine_b200.parallel.peer import HostRelay

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    relay = HostRelay(dist.group.WORLD)
    t = torch.full((4, 8), float(rank + 1))
    relay.allreduce_(t)
    q.put((rank, t.sum().item()))
    dist.barrier()
    dist.destroy_process_group()


def test_host_relay_allreduce_between_two_cpu_ranks():
    import socket
    import torch.multiprocessing as mp

    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_relay_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res == [(0, 96.0), (1, 96.0)]


def test_27b_shards_meet_the_kernel_alignments_at_2_4_8_ranks():
    """Per-rank shapes of the 27B preset at every supported world size: record widths (k multiples of 128), GEMM tile widths and
    whole head groups, which the weight-streaming and tcgen05 kernels require; kv heads are replicated past 4 ranks."""
    from owl_engine_b200.models.spec import qwen_27b

    full = qwen_27b()
    for world in (2, 4, 8):
        for rank in (0, world - 1):
            sp = full.sharded(rank, world)
            assert sp.tp_world == world and sp.tp_rank == rank and sp.hidden == full.hidden
            assert sp.inter * world == full.inter and sp.inter % 128 == 0            # down-proj k, gate/up rows
            assert sp.hq * world == full.hq and sp.hq % sp.hkv == 0 and sp.hq // sp.hkv <= 8
            assert sp.hkv == max(1, full.hkv // world) and sp.kv_replicas == max(1, world // full.hkv)
            assert (sp.hq * sp.hd) % 128 == 0                                       # o-proj k
            assert sp.nk * world == full.nk and sp.nv * world == full.nv and sp.nv % sp.nk == 0
            assert sp.value_dim % 128 == 0 and (sp.conv_dim + sp.value_dim) % 16 == 0
