"""Engine core: one rank's model runner plus the page / slot bookkeeping and the host-fed step.

``Engine`` is what the serving layers (scheduler, RunningEngine, HTTP server) and ``bench.py``
drive. A step is host-fed: the step inputs (token ids, positions, KV slots, context lengths,
GDN rows, block-table rows) are written into one pinned host buffer, copied to the device with
a single asynchronous copy, the captured CUDA graph of that (batch, rows) shape is replayed, and
the sampled tokens come back through one small device-to-host copy -- the only blocking point
of a step, as in the reference (charter A3; ``crates/engine/src/exec/phases.rs:963-1124``).

Reference counterpart: ``Engine::new/on/run`` + ``boot_rank`` (``crates/engine/src/engine.rs:1152-
2774``), the executor phases (``exec/phases.rs``) and the graph fleet (``graph/graph_fleet.rs``).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..models import hybrid as H
from ..models.spec import ModelSpec, PRESETS
from ..ops import kernels as K

PAGE = H.PAGE


@dataclass
class EngineConfig:
    model: str = "qwen3.8-27b"
    quant: str = "w4a16"           # weight format of the random-init / loaded checkpoint
    group: int = 128
    lm_head_int8: bool = False
    n_pages: int = 4096            # KV pool pages (16 tokens each) per rank
    n_slots: int = 8               # GDN state rows (= concurrency ceiling, like gdn_slots)
    max_seqs: int = 8
    max_seq: int = 8192
    prefill_chunk: int = 2048
    pdl: bool = True
    prefill_gemm: str = "tc"
    seed: int = 0
    n_layers: int | None = None    # override (tests / smoke)


@dataclass
class Sequence:
    sid: int
    row: int                       # block-table row
    slot: int                      # GDN state row
    tokens: list = field(default_factory=list)    # all tokens so far (prompt + generated)
    n_cached: int = 0              # tokens whose KV / GDN state is materialised
    pages: list = field(default_factory=list)


class Engine:
    def __init__(self, cfg: EngineConfig, *, spec: ModelSpec | None = None, weights: H.HybridWeights | None = None,
                 comm=None, device=None):
        self.cfg = cfg
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        full = spec or PRESETS[cfg.model]()
        if cfg.n_layers is not None:
            from dataclasses import replace
            full = replace(full, n_layers=cfg.n_layers)
        self.full_spec = full
        self.comm = comm
        world = comm.world if comm is not None else 1
        rank = comm.rank if comm is not None else 0
        self.spec = full.sharded(rank, world) if world > 1 and full.tp_world == 1 else full
        self.weights = weights or H.random_weights(self.spec, self.device, group=cfg.group, seed=cfg.seed + rank * 7919,
                                                   lm_head_int8=cfg.lm_head_int8)
        self.pool = H.StatePool(self.spec, self.device, cfg.n_pages, cfg.n_slots)
        self.max_blocks = (cfg.max_seq + PAGE - 1) // PAGE
        self.runner = H.HybridRunner(self.spec, self.weights, self.pool, max_seqs=cfg.max_seqs,
                                     max_blocks=self.max_blocks, prefill_chunk=cfg.prefill_chunk, comm=comm,
                                     pdl=cfg.pdl, prefill_gemm=cfg.prefill_gemm)
        self.free_pages = list(range(cfg.n_pages - 1, -1, -1))
        self.free_rows = list(range(cfg.max_seqs - 1, -1, -1))
        self.free_slots = list(range(cfg.n_slots - 1, -1, -1))
        self.seqs: dict[int, Sequence] = {}
        self._next_sid = 0
        # pinned staging for the host-fed step
        self.h_inp = torch.zeros(self.runner.inp.numel(), dtype=torch.int32).pin_memory()
        self.h_tok = torch.zeros(H.HybridRunner.MAX_ROWS, dtype=torch.int32).pin_memory()
        self.h_inp_np = self.h_inp.numpy()
        self.h_tok_np = self.h_tok.numpy()
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.stream = torch.cuda.current_stream(self.device)

    # -- sequences ----------------------------------------------------------------------------
    def add_sequence(self, prompt: list[int]) -> int:
        if not self.free_rows or not self.free_slots:
            raise RuntimeError("no free sequence row / GDN slot (concurrency ceiling reached)")
        sid = self._next_sid
        self._next_sid += 1
        seq = Sequence(sid, self.free_rows.pop(), self.free_slots.pop(), list(prompt))
        self.pool.reset_slot(seq.slot)
        self.seqs[sid] = seq
        return sid

    def free_sequence(self, sid: int) -> None:
        seq = self.seqs.pop(sid)
        self.free_pages.extend(seq.pages)
        self.free_rows.append(seq.row)
        self.free_slots.append(seq.slot)

    def _ensure_pages(self, seq: Sequence, n_tokens: int) -> None:
        need = (n_tokens + PAGE - 1) // PAGE
        if need > self.max_blocks:
            raise RuntimeError(f"sequence longer than max_seq ({n_tokens} tokens)")
        if need > len(seq.pages):
            add = need - len(seq.pages)
            if add > len(self.free_pages):
                raise RuntimeError("KV pool exhausted")
            new = [self.free_pages.pop() for _ in range(add)]
            start = len(seq.pages)
            seq.pages.extend(new)
            self.runner.block_table[seq.row, start:start + add] = torch.tensor(new, dtype=torch.int32,
                                                                                 device=self.device)

    # -- prefill ------------------------------------------------------------------------------
    def prefill(self, sid: int) -> int:
        """Feed every not-yet-cached prompt token; returns the first generated token."""
        seq = self.seqs[sid]
        n = len(seq.tokens)
        self._ensure_pages(seq, n + 1)
        ids = torch.tensor(seq.tokens[seq.n_cached:], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        tok = None
        pos = seq.n_cached
        chunk = self.cfg.prefill_chunk
        for s in range(0, ids.shape[0], chunk):
            part = ids[s:s + chunk]
            last = s + chunk >= ids.shape[0]
            tok = self.runner.prefill_chunk_forward(part, pos, seq.row, seq.slot, want_logits=last)
            pos += part.shape[0]
        seq.n_cached = n
        t = int(tok.item())
        seq.tokens.append(t)
        return t

    # -- host-fed decode step -----------------------------------------------------------------
    def decode_step(self, sids: list[int]) -> list[int]:
        """One token for each listed sequence (their last token is the step input)."""
        b = len(sids)
        lay = H.StepLayout(b, 1)
        hi = self.h_inp_np
        ctx_max = 0
        for i, sid in enumerate(sids):
            seq = self.seqs[sid]
            pos = seq.n_cached
            self._ensure_pages(seq, pos + 1)
            hi[lay.ids + i] = seq.tokens[-1]
            hi[lay.pos3 + i] = pos
            hi[lay.pos3 + b + i] = pos
            hi[lay.pos3 + 2 * b + i] = pos
            hi[lay.kv_slot + i] = seq.pages[pos // PAGE] * PAGE + pos % PAGE
            hi[lay.ctx + i] = pos + 1
            hi[lay.gslot + i] = seq.slot
            hi[lay.bt_row + i] = seq.row
            ctx_max = max(ctx_max, pos + 1)
        graph = self.runner.capture(b, 1, ctx_hint=self._ctx_bucket(ctx_max))
        n = lay.size
        self.runner.inp[:n].copy_(self.h_inp[:n], non_blocking=True)
        graph.replay()
        self.h_tok[:b].copy_(self.runner.out_tok[:b], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.h2d_bytes += n * 4
        self.d2h_bytes += b * 4
        out = []
        for i, sid in enumerate(sids):
            seq = self.seqs[sid]
            t = int(self.h_tok_np[i])
            seq.n_cached += 1
            seq.tokens.append(t)
            out.append(t)
        return out

    @staticmethod
    def _ctx_bucket(ctx: int) -> int:
        """Context-length bucket that picks the split-KV factor of the captured graph."""
        b = 512
        while b < ctx:
            b *= 2
        return b

    # -- public convenience -------------------------------------------------------------------
    def generate(self, prompt: list[int], max_new_tokens: int, eos: int | None = None) -> list[int]:
        """Greedy generation for one prompt (the call a user of the library makes)."""
        sid = self.add_sequence(prompt)
        try:
            out = [self.prefill(sid)]
            while len(out) < max_new_tokens and (eos is None or out[-1] != eos):
                out.append(self.decode_step([sid])[0])
            return out
        finally:
            self.free_sequence(sid)
