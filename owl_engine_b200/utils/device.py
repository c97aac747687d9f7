"""Declarative GPU selection and per-GPU lock files.

A profile names devices by UUID (``GPU-...``), PCI bus id (``0000:1b:00.0``), a name substring
(``find:B200``) or, as a last resort on single-tenant boxes, a CUDA index. ``resolve`` maps each
selector to a CUDA ordinal using NVML facts; ``GpuLock`` takes a UUID-named lock file with
stale-pid cleanup so two engine processes never share a device by accident.

Reference counterpart: ``crates/shared/src/device.rs`` (``{bdf, find_name, uuid}``) and
``gpu_lock.rs``. Only reads device properties; never changes clocks, power limits or modes.
"""
from __future__ import annotations

import errno
import os
import tempfile
from dataclasses import dataclass


@dataclass
class DeviceFacts:
    index: int
    uuid: str
    bdf: str
    name: str
    total_bytes: int


def enumerate_devices(nvml=None) -> list[DeviceFacts]:
    """Device facts through NVML (``nvml`` may be a fake with the same call surface for tests)."""
    if nvml is None:
        import pynvml as nvml
    nvml.nvmlInit()
    out = []
    for i in range(nvml.nvmlDeviceGetCount()):
        h = nvml.nvmlDeviceGetHandleByIndex(i)
        def s(x): return x.decode() if isinstance(x, bytes) else x
        pci = nvml.nvmlDeviceGetPciInfo(h)
        out.append(DeviceFacts(i, s(nvml.nvmlDeviceGetUUID(h)), s(pci.busId).lower(), s(nvml.nvmlDeviceGetName(h)),
                               int(nvml.nvmlDeviceGetMemoryInfo(h).total)))
    return out


def resolve(selectors: list[str], devices: list[DeviceFacts]) -> list[DeviceFacts]:
    picked = []
    for sel in selectors:
        s = sel.strip()
        match = None
        for d in devices:
            if d in picked:
                continue
            if s.upper().startswith("GPU-") and d.uuid.upper() == s.upper():
                match = d
            elif ":" in s and not s.startswith("find:") and d.bdf.endswith(s.lower()):
                match = d
            elif s.startswith("find:") and s[5:].lower() in d.name.lower():
                match = d
            elif s.isdigit() and d.index == int(s):
                match = d
            if match:
                break
        if match is None:
            raise LookupError(f"no free device matches selector {sel!r}")
        picked.append(match)
    return picked


class GpuLock:
    """``<dir>/owl-b200-<uuid>.lock`` holding the owner's pid; stale locks (dead pid) are taken over."""

    def __init__(self, uuid: str, directory: str | None = None):
        self.path = os.path.join(directory or tempfile.gettempdir(), f"owl-b200-{uuid}.lock")
        self.held = False

    def acquire(self) -> None:
        for _ in range(2):
            try:
                fd = os.open(self.path, os.O_CREAT | os.O_EXCL | os.O_WRONLY, 0o644)
                os.write(fd, str(os.getpid()).encode())
                os.close(fd)
                self.held = True
                return
            except FileExistsError:
                try:
                    pid = int(open(self.path).read().strip() or "0")
                except (OSError, ValueError):
                    pid = 0
                if pid and _alive(pid) and pid != os.getpid():
                    raise RuntimeError(f"GPU is locked by pid {pid} ({self.path})") from None
                try:
                    os.unlink(self.path)      # stale
                except FileNotFoundError:
                    pass
        raise RuntimeError(f"could not take {self.path}")

    def release(self) -> None:
        if self.held:
            try:
                os.unlink(self.path)
            except FileNotFoundError:
                pass
            self.held = False

    def __enter__(self):
        self.acquire()
        return self

    def __exit__(self, *a):
        self.release()


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
        return True
    except OSError as e:
        return e.errno == errno.EPERM
