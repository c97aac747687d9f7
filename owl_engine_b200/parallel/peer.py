"""Peer capability classification, the per-allocation limit and the peer plan of a tensor-parallel group, plus the host-relay
fallback transport.

``classify`` decides, from facts probed once at boot (NVLink state, P2P support, BAR1 size), how two GPUs may map each other's
memory:

* ``"nvlink"``   both GPUs reach each other over NVLink / NVSwitch: symmetric (VMM) memory, no BAR1 window involved
                 (the B200 case; not present in the reference, which targets PCIe consumer cards);
* ``"static"``   PCIe P2P with both BAR1 apertures >= 2 GiB: static mapping, allocations capped at 192 MiB each;
* ``"window"``   PCIe P2P with both apertures narrow: each allocation <= min(smaller BAR1 - 64 MiB, 192 MiB);
* ``"rejected"`` no P2P on either side, or one wide and one narrow aperture (mixed pairs are refused, not degraded).

``PeerPlan.plan`` applies that to every pair of a group and refuses a staging size above the limit instead of shrinking it.
``HostRelay`` is the transport for rejected groups (``tp_comm = "host"``): payloads cross through pinned host memory and a
``gloo`` all-reduce; it cannot be captured in a CUDA graph, so the runner steps eagerly on it.

Reference counterpart: ``crates/backends/cuda/src/comm/peer.rs:33-110`` (classification, limits, plan),
``crates/backends/cuda/src/server/host.rs:1-82`` and ``crates/models/src/interpreters/eval.rs:1218-1323`` (host relay).
"""
from __future__ import annotations

from dataclasses import dataclass

PEER_ALLOC_HARD_CAP = 192 << 20
WINDOW_BAR1_RESERVE = 64 << 20
STATIC_BAR1_MIN = 2 << 30


class PeerRejected(RuntimeError):
    pass


@dataclass(frozen=True)
class PeerCaps:
    uuid: str
    bar1_bytes: int
    p2p_supported: bool
    nvlink: bool = False           # an active NVLink path to the peers of its group

    @property
    def wide_bar1(self) -> bool:
        return self.bar1_bytes >= STATIC_BAR1_MIN


def classify(a: PeerCaps, b: PeerCaps) -> str:
    if a.nvlink and b.nvlink:
        return "nvlink"
    if not (a.p2p_supported and b.p2p_supported):
        return "rejected"
    if a.wide_bar1 and b.wide_bar1:
        return "static"
    if not a.wide_bar1 and not b.wide_bar1:
        return "window"
    return "rejected"


def per_alloc_limit(mechanism: str, a: PeerCaps, b: PeerCaps) -> int:
    if mechanism == "nvlink":
        return 1 << 62                       # bounded by the VRAM budget, not by an aperture
    if mechanism == "static":
        return PEER_ALLOC_HARD_CAP
    if mechanism == "window":
        return min(max(0, min(a.bar1_bytes, b.bar1_bytes) - WINDOW_BAR1_RESERVE), PEER_ALLOC_HARD_CAP)
    return 0


@dataclass(frozen=True)
class PeerPlan:
    mechanism: str
    per_alloc_limit: int
    staging_bytes: int

    @classmethod
    def plan(cls, caps: list[PeerCaps], staging_bytes: int) -> "PeerPlan":
        """One mechanism for the whole group (every pair must agree) and the tightest limit; raises ``PeerRejected`` with
        the offending pair instead of degrading silently."""
        mech, limit = None, 1 << 62
        for i, a in enumerate(caps):
            for b in caps[i + 1:]:
                m = classify(a, b)
                if m == "rejected" or (mech is not None and m != mech):
                    raise PeerRejected(f"peer pair refused: {a.uuid} (bar1 {a.bar1_bytes >> 20} MiB, p2p {a.p2p_supported}, "
                                       f"nvlink {a.nvlink}) x {b.uuid} (bar1 {b.bar1_bytes >> 20} MiB, p2p {b.p2p_supported}, "
                                       f"nvlink {b.nvlink}): {m if mech is None or m == 'rejected' else 'mixed ' + mech + '/' + m}")
                mech = m
                limit = min(limit, per_alloc_limit(m, a, b))
        if mech is None:
            raise PeerRejected("a peer plan needs at least two GPUs")
        if staging_bytes > limit:
            raise PeerRejected(f"staging of {staging_bytes} bytes exceeds the per-allocation limit {limit} of mechanism {mech}")
        return cls(mech, limit, staging_bytes)


def probe(indices: list[int], nvml=None) -> list[PeerCaps]:
    """Read the facts from NVML (``nvml``: the ``pynvml`` module or a fake with the same calls)."""
    if nvml is None:
        import pynvml as nvml
    nvml.nvmlInit()
    hs = [nvml.nvmlDeviceGetHandleByIndex(i) for i in indices]
    out = []
    for i, h in enumerate(hs):
        bar1 = int(nvml.nvmlDeviceGetBAR1MemoryInfo(h).bar1Total)
        others = [o for j, o in enumerate(hs) if j != i]
        p2p = all(nvml.nvmlDeviceGetP2PStatus(h, o, nvml.NVML_P2P_CAPS_INDEX_READ) == nvml.NVML_P2P_STATUS_OK for o in others)
        link = False
        try:
            link = any(nvml.nvmlDeviceGetNvLinkState(h, l) for l in range(getattr(nvml, "NVML_NVLINK_MAX_LINKS", 18)))
        except Exception:
            link = False
        uuid = nvml.nvmlDeviceGetUUID(h)
        out.append(PeerCaps(uuid.decode() if isinstance(uuid, bytes) else uuid, bar1, p2p, bool(link)))
    return out


class HostRelay:
    """All-reduce through host memory: device payloads are staged in pinned host buffers, summed with a ``gloo``
    all-reduce and copied back. Works for CPU tensors as is (that is how it is tested without GPUs)."""

    capturable = False

    def __init__(self, group=None):
        import torch.distributed as dist

        self.group = group if group is not None else dist.new_group(backend="gloo")
        self._stage: dict = {}

    def allreduce_(self, t) -> None:
        import torch
        import torch.distributed as dist

        if not t.is_cuda:
            dist.all_reduce(t, group=self.group)
            return
        key = (t.dtype, t.numel())
        buf = self._stage.get(key)
        if buf is None:
            buf = torch.empty(t.numel(), dtype=torch.float32).pin_memory()      # gloo sums fp32; the payload is 16-bit
            self._stage[key] = buf
        buf.copy_(t.reshape(-1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        dist.all_reduce(buf, group=self.group)
        t.reshape(-1).copy_(buf, non_blocking=True)
