"""KvStore: Python face of the native block ledger (``csrc/host/store_core.cpp``).

Content-addressed chains: ``chain(tokens)`` hashes every full block with its parent's hash, so a
prefix shared between requests maps to the same nodes. ``match`` finds the longest cached prefix
(and pins the device pages it returns), ``publish`` indexes freshly written blocks, ``evict``
plans leaf-LRU victims (drop or demote). All of it is host bookkeeping; the engine performs the
copies at step boundaries.

Reference counterpart: ``crates/store/src/kv/*.rs`` and ``id.rs`` (block = 32 tokens there; here the
block is the KV page, 16 tokens by default).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int8, c_int32, c_uint64, c_void_p

import numpy as np

from .. import _native

DEVICE, HOST, DISK = 0, 1, 2
_lib = None


def lib():
    global _lib
    if _lib is None:
        l = _native.host()
        l.owl_kv_new.restype = c_void_p
        l.owl_kv_new.argtypes = [c_int, c_int]
        l.owl_kv_free.argtypes = [c_void_p]
        l.owl_kv_hash.restype = c_uint64
        l.owl_kv_hash.argtypes = [c_uint64, c_void_p, c_int, c_uint64]
        l.owl_kv_chain.argtypes = [c_void_p, c_int, c_int, c_uint64, c_void_p, c_void_p]
        l.owl_kv_free_pages.argtypes = [c_void_p]
        l.owl_kv_alloc.argtypes = [c_void_p, c_int, c_void_p]
        l.owl_kv_ref.argtypes = [c_void_p, c_void_p, c_int]
        l.owl_kv_unref.argtypes = [c_void_p, c_void_p, c_int]
        l.owl_kv_refcount.argtypes = [c_void_p, c_int]
        l.owl_kv_match.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        l.owl_kv_publish.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_uint64, c_void_p]
        l.owl_kv_evict.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int]
        l.owl_kv_set_carrier.argtypes = [c_void_p, c_uint64, c_int, c_int]
        l.owl_kv_forget.argtypes = [c_void_p, c_uint64]
        l.owl_kv_adopt.argtypes = [c_void_p, c_uint64, c_uint64, c_int, c_int, c_uint64]
        l.owl_kv_node.argtypes = [c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p]
        l.owl_kv_stats.argtypes = [c_void_p, c_void_p]
        l.owl_kv_list.argtypes = [c_void_p, c_int, c_void_p, c_int]
        l.owl_kv_set_policy.argtypes = [c_void_p, ctypes.c_double]
        l.owl_kv_set_policy.restype = None
        _lib = l
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(c_void_p)


class KvStore:
    def __init__(self, n_pages: int, block_tokens: int = 16):
        self.n_pages, self.block_tokens = n_pages, block_tokens
        self.h = lib().owl_kv_new(n_pages, block_tokens)

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.owl_kv_free(self.h)
            self.h = None

    def set_policy(self, policy: str) -> None:
        """Victim order of ``evict``: ``"lru"`` (least recently used leaf), ``"lrfu"`` or ``"lrfu:<lambda>"`` (combined
        recency / frequency: every use adds 1 to a block's value, which halves every ``1 / lambda`` uses of the store;
        default lambda 0.05)."""
        name, _, arg = policy.partition(":")
        if name == "lru" and not arg:
            lam = -1.0
        elif name == "lrfu":
            lam = float(arg) if arg else 0.05
            if lam < 0:
                raise ValueError(f"evict_policy {policy!r}: lambda must be >= 0")
        else:
            raise ValueError(f"evict_policy {policy!r}: expected lru, lrfu or lrfu:<lambda>")
        self.policy = policy
        lib().owl_kv_set_policy(self.h, lam)

    # -- hashing -----------------------------------------------------------------------------
    def chain(self, tokens, root: int = 0, tags=None) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        nb = len(t) // self.block_tokens
        out = np.zeros(nb, dtype=np.uint64)
        tg = np.ascontiguousarray(tags, dtype=np.uint64) if tags is not None else None
        lib().owl_kv_chain(_p(t), len(t), self.block_tokens, root, _p(tg) if tg is not None else None, _p(out))
        return out

    # -- pages -------------------------------------------------------------------------------
    @property
    def free_pages(self) -> int:
        return lib().owl_kv_free_pages(self.h)

    def alloc(self, n: int) -> list[int] | None:
        out = np.zeros(max(n, 1), dtype=np.int32)
        return out[:n].tolist() if n == 0 or lib().owl_kv_alloc(self.h, n, _p(out)) == n else None

    def ref(self, pages) -> None:
        a = np.ascontiguousarray(pages, dtype=np.int32)
        lib().owl_kv_ref(self.h, _p(a), len(a))

    def unref(self, pages) -> None:
        a = np.ascontiguousarray(pages, dtype=np.int32)
        if len(a):
            lib().owl_kv_unref(self.h, _p(a), len(a))

    def refcount(self, page: int) -> int:
        return lib().owl_kv_refcount(self.h, page)

    # -- tree --------------------------------------------------------------------------------
    def match(self, hashes: np.ndarray):
        """Returns (n_matched, pages, carriers); device pages in the result are pinned (ref +1)."""
        n = len(hashes)
        pages, carr = np.zeros(max(n, 1), dtype=np.int32), np.zeros(max(n, 1), dtype=np.int8)
        m = lib().owl_kv_match(self.h, _p(np.ascontiguousarray(hashes, dtype=np.uint64)), n, _p(pages), _p(carr)) if n else 0
        return m, pages[:m].tolist(), carr[:m].tolist()

    def publish(self, hashes: np.ndarray, pages, root: int = 0, tags=None) -> int:
        hs = np.ascontiguousarray(hashes, dtype=np.uint64)
        pg = np.ascontiguousarray(pages, dtype=np.int32)
        assert len(hs) == len(pg)
        tg = np.ascontiguousarray(tags, dtype=np.uint64) if tags is not None else None
        return lib().owl_kv_publish(self.h, _p(hs), _p(pg), len(hs), root, _p(tg) if tg is not None else None) if len(hs) else 0

    def evict(self, need_free: int, demote: bool = False, max_victims: int = 4096):
        """Victims (pages, hashes) so that ``need_free`` pages are free; may return fewer."""
        pages, hs = np.zeros(max_victims, dtype=np.int32), np.zeros(max_victims, dtype=np.uint64)
        n = lib().owl_kv_evict(self.h, need_free, 1 if demote else 0, _p(pages), _p(hs), max_victims)
        return pages[:n].tolist(), hs[:n].tolist()

    def set_carrier(self, h: int, carrier: int, slot: int) -> None:
        if lib().owl_kv_set_carrier(self.h, h, carrier, slot) != 0:
            raise KeyError(h)

    def adopt(self, h: int, parent: int, carrier: int, slot: int = 0, tag: int = 0) -> bool:
        """Insert a node that lives on the host (carrier 1, ``slot``) or on disk (carrier 2): restart adoption."""
        return lib().owl_kv_adopt(self.h, h, parent, carrier, slot, tag) == 1

    def forget(self, h: int) -> bool:
        return lib().owl_kv_forget(self.h, h) == 0

    def node(self, h: int):
        page, carr = c_int32(), c_int8()
        tag, parent = c_uint64(), c_uint64()
        if lib().owl_kv_node(self.h, h, ctypes.byref(page), ctypes.byref(carr), ctypes.byref(tag), ctypes.byref(parent)):
            return None
        return {"page": page.value, "carrier": carr.value, "tag": tag.value, "parent": parent.value}

    def stats(self) -> dict:
        out = np.zeros(8, dtype=np.uint64)
        lib().owl_kv_stats(self.h, _p(out))
        k = ["nodes", "device_nodes", "free_pages", "lookups", "hits", "evictions", "published", "lru_len"]
        return dict(zip(k, map(int, out)))

    def list(self, carrier: int = -1) -> list[int]:
        n = lib().owl_kv_list(self.h, carrier, None, 0)
        out = np.zeros(max(n, 1), dtype=np.uint64)
        lib().owl_kv_list(self.h, carrier, _p(out), n)
        return out[:n].tolist()
