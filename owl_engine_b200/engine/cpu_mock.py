"""The engine on the CPU face: every host-side mechanism of ``Engine`` / ``RunningEngine`` (page accounting, prefix tree,
snapshots, tiers, admission, parked sessions, budget refusals) running without a GPU over a stand-in model.

``Engine(cfg, device="cpu")`` builds a real ``StatePool`` on host tensors and, instead of ``HybridRunner``, a ``NullRunner``:
the same step interface (packed input buffer, block table, ``capture(b, t).replay()``, ``prefill_chunk_forward``), whose
"model" is a checksum recurrence that is cheap and fully determined by the tokens consumed:

    state' = (state * 31 + token + position) mod 2^31           (kept in the sequence's GDN state row)
    next   = (state' + sum of the KV marks of the visible pages) mod vocab

and whose "KV write" stores one mark per token in the paged pool. A continuation therefore depends on the recurrent state row AND
on every page of the context being the right page: a sequence resumed from a prefix hit, from a snapshot restored out of a
lower tier, or after a leave-gap deletion produces the same tokens as the uninterrupted run only if the host logic moved the
right bytes. ``MockLimits`` (``utils/cpuface.py``) supplies the injected limits: ``vram_bytes`` becomes an enforcing ledger, so
a pool that does not fit is refused at boot with the ledger's message.

Reference counterpart: ``crates/engine/tests/cpu_mock_smoke.rs:1-106`` (engine boot on the CPU backend with ``MockLimits``),
``crates/backends/cpu/src/face.rs``.
"""
from __future__ import annotations

import torch

from ..models import hybrid as H
from ..utils.cpuface import MockLimits
from ..utils.ledger import DeviceLedger

PAGE = 16
MOD = 1 << 31


def ledger_from(limits: MockLimits) -> DeviceLedger:
    """An enforcing ledger of the CPU face whose whole budget is ``limits.vram_bytes``."""
    return DeviceLedger("cpu", total_bytes=int(limits.vram_bytes), budget_frac=1.0, reserve_bytes=0, enforce=True)


class _Replay:
    def __init__(self, runner, b: int, t: int):
        self.r, self.b, self.t = runner, b, t

    def replay(self) -> None:
        self.r.step_forward(H.StepLayout(self.b, self.t))


class _Fold:
    """Stand-in for the captured fold graphs: replays the recurrent-state update of the first rows of the last step."""

    def __init__(self, runner, b: int, t: int, batched: bool):
        self.r, self.b, self.t, self.batched = runner, b, t, batched

    def replay(self) -> None:
        r = self.r
        for i in range(self.b):
            slot = int(r.fold_slots[i]) if self.batched else int(r.fold_slot[0])
            n = int(r.fold_tlen[i]) if self.batched else self.t
            if slot < 0:
                continue
            for tok, pos in r._saved.get(i, [])[:n]:
                r._set_state(slot, (r._state(slot) * 31 + tok + pos) % (1 << 23))
                r.launches += 1


class NullRunner:
    """Stand-in for ``HybridRunner`` on host tensors (see the module docstring for its arithmetic)."""
    MAX_ROWS = H.HybridRunner.MAX_ROWS

    def __init__(self, spec, pool, *, max_seqs: int, max_blocks: int, limits: MockLimits | None = None):
        self.spec, self.pool, self.device = spec, pool, pool.device
        self.max_seqs, self.max_blocks = max_seqs, max_blocks
        self.limits = limits or MockLimits()
        m = self.MAX_ROWS
        self.inp = torch.zeros(8 * m, dtype=torch.int32)
        self.out_tok = torch.zeros(m, dtype=torch.int32)
        self.block_table = torch.zeros(max_seqs, max_blocks, dtype=torch.int32)
        self.h = torch.zeros(m, spec.hidden, dtype=torch.bfloat16)
        self.graphs: dict = {}
        self.uniform_rows = True
        self.gdn_save = self.taps = self.tap_sink = None
        self._saved: dict = {}        # batch index -> [(token, position)] of the last step (what a fold replays)
        self.fold_slot = torch.full((1,), -1, dtype=torch.int32)
        self.fold_slots = torch.full((m,), -1, dtype=torch.int32)
        self.fold_tlen = torch.zeros(m, dtype=torch.int32)
        self.decode_gemv, self.act_bits, self.vocab_split = "null", 15, False
        self.launches = 0

    # -- the stand-in model -----------------------------------------------------------------------------------------
    def _state(self, slot: int) -> int:
        return int(self.pool.conv_state[0, slot, 0, 0].item())

    def _set_state(self, slot: int, v: int) -> None:
        self.pool.conv_state[0, slot, 0, 0] = float(v % (1 << 23))          # exact in fp32
        self.pool.rec_state[0, slot].view(-1)[0] = float(v % (1 << 23))

    def _mark(self, row: int, pos: int, tok: int) -> None:
        page = int(self.block_table[row, pos // PAGE])
        self.pool.k_pool[0, page, pos % PAGE].view(-1)[0] = (tok * 7 + pos) % 251
        self.pool.v_pool[0, page, pos % PAGE].view(-1)[0] = (tok + 3) % 251

    def _context_sum(self, row: int, n: int) -> int:
        if n <= 0:
            return 0
        pages = self.block_table[row, :(n + PAGE - 1) // PAGE].long()
        marks = self.pool.k_pool[0, pages, :, 0, 0].reshape(-1)[:n].long() + self.pool.v_pool[0, pages, :, 0, 0].reshape(-1)[:n].long()
        return int(marks.sum())

    def _consume(self, row: int, slot: int, pos: int, tok: int) -> int:
        """One token at ``pos``: KV mark, state update; returns the token that follows."""
        self.launches += 1
        if self.limits.null_kernels:
            return 0
        self._mark(row, pos, tok)
        st = (self._state(slot) * 31 + tok + pos) % (1 << 23)
        self._set_state(slot, st)
        return (st + self._context_sum(row, pos + 1)) % self.spec.vocab

    # -- step interface ---------------------------------------------------------------------------------------------
    def views(self, lay):
        v = self.inp
        return {"ids": v[lay.ids:lay.ids + lay.m], "pos3": v[lay.pos3:lay.pos3 + 3 * lay.m], "kv_slot": v[lay.kv_slot:lay.kv_slot + lay.m],
                "ctx": v[lay.ctx:lay.ctx + lay.b], "gslot": v[lay.gslot:lay.gslot + lay.b], "bt_row": v[lay.bt_row:lay.bt_row + lay.b]}

    def step_forward(self, lay, **_) -> None:
        v = self.views(lay)
        for i in range(lay.b):
            slot, row, ctx = int(v["gslot"][i]), int(v["bt_row"][i]), int(v["ctx"][i])
            if slot < 0:
                continue
            self._saved[i] = []
            for j in range(lay.t):
                pos = ctx - lay.t + j
                self._saved[i].append((int(v["ids"][i * lay.t + j]), pos))
                self.out_tok[i * lay.t + j] = self._consume(row, slot, pos, int(v["ids"][i * lay.t + j]))

    def capture(self, b: int, t: int = 1, *, ctx_hint: int = 2048, advance: bool = False, sample: bool = True):
        if not self.limits.graph_capture:
            from ..utils.cpuface import CaptureUnsupported

            raise CaptureUnsupported("graph capture is switched off on this face")
        key = (b, t)
        g = self.graphs.get(key)
        if g is None:
            g = self.graphs[key] = _Replay(self, b, t)
        return g

    # speculative decoding: the verify step keeps its rows (above), a fold replays the accepted ones on the restored state
    def enable_gdn_save(self) -> None:
        if self.gdn_save is None:
            self.gdn_save = True
            self.graphs.clear()

    def capture_fold(self, t: int):
        return self.graphs.setdefault(("fold", t), _Fold(self, 1, t, False))

    def capture_fold_batch(self, b: int, t: int):
        return self.graphs.setdefault(("foldb", b, t), _Fold(self, b, t, True))

    def prefill_chunk_forward(self, ids, pos0: int, seq_row: int, slot: int, want_logits: bool = True, embeds=None, pos3=None,
                              snap=None):
        nxt = 0
        for i, tok in enumerate(ids.tolist()):
            if snap is not None and i == snap[0]:
                self.pool.copy_slot(slot, snap[1])
            nxt = self._consume(seq_row, slot, pos0 + i, tok)
        return torch.tensor([nxt], dtype=torch.int32)
