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

import numpy as np
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
    n_snap_rows: int = 2           # extra state rows that hold prefix-boundary snapshots
    spec_rows: int = 1             # scratch state rows of speculative verify steps (= sequences per batched verify)
    host_cache_mb: int = 0         # pinned-host KV tier (0 = off)
    pinned_segment_mb: int = 256   # the host tier's pinned memory is allocated in segments of this size
    disk_cache_mb: int = 0         # disk KV tier behind the host tier (0 = off)
    disk_dir: str = ""             # directory of the disk tier (block files + restart index)
    max_seqs: int = 8
    max_seq: int = 8192
    prefill_chunk: int = 2048
    pdl: bool = True
    prefill_gemm: str = "tc"
    act_bits: int = 15             # decode activations: 15-bit fixed point, or 8 (the W4A8 decode arm, `[model] quant = "w4a8"`)
    decode_gemv: str = "fma"       # W4 decode arm: "fma" (one-token steps on the half-precision FMA projection with fused norm /
                                   # residual / activation; other row counts on the integer arm), "dp4a" (integer arm only) or
                                   # "tc" (tcgen05 streaming kernel, block-major records)
    seed: int = 0
    n_layers: int | None = None    # override (tests / smoke)
    snap_cut: bool = False         # cut a separate chunk at the prompt's last block boundary instead of snapshotting inside a chunk
    kv_dtype: str = "fp8"          # KV pool format: "fp8" (e4m3), "int8" (per token, per head scales), "bf16" / "f16" (16-bit)
    kvmem_budget: int = 0          # tokens of KV a decode step may attend to (0 = everything): longer contexts attend to a
                                   # view of sink + recent + best-scoring blocks, re-selected at every block boundary
    kvmem_sink: int = 2
    kvmem_recent: int = 4
    kvmem_query_tokens: int = 1    # the newest queries (one per decode step) a block is scored against; the score is their maximum
    kvmem_recall_every: int = 1    # blocks written between two selections (the blocks written in between join the view as recent)
    recall_mode: str = "sync"      # recall of demoted prefix blocks: "sync" (host and disk), "host" (host only), "resident" (none)
    workspace_reserve_mb: int = 3072   # n_pages = 0: device memory the boot plan leaves for graphs, prefill workspace, scratch
    vocab_split: bool = True       # tensor parallel: each rank holds vocab / world lm_head rows and the winners are merged
    attn_splits: int = 0           # split-KV factor of decode attention (0 = from the context length)
    cuda_graph: bool = True        # False: steps launch their kernels eagerly (debugging; slower)
    rope_yarn: tuple = None        # (factor, original_max, beta_fast, beta_slow, attention_factor): YaRN context extension
    prefix_cache: bool = True      # False: nothing is looked up in or published to the prefix tree, no snapshots are taken
    no_reclaim: bool = False       # diagnostic: cached blocks are never evicted under pressure (requests that do not fit fail)
    evict_policy: str = "lru"      # victim order of the prefix tree's leaves: "lru", "lrfu" or "lrfu:<lambda>"
    # recurrent-state snapshot policy (store/snap_policy.py)
    msg_open_ids: tuple = ()       # token ids of the chat format's message-open marker; () = no message-boundary snapshots
    snap_msg_min_gap: int = 2048   # tokens between kept message boundaries (the first and the newest `recent` are always kept)
    snap_msg_recent: int = 4
    snap_decode_stride: int = 0    # pages of generated text between rolling snapshots (0 = generation takes none)
    snap_spec_rollback: bool = False   # speculative rounds that step over a page boundary roll back and save it (two extra folds)
    snap_session_cap: int = 0      # snapshots one session may hold over all tiers (0 = unbounded)
    snap_structural_reserve: int = 4
    snap_host_mb: int = 0          # host memory for snapshots whose state row was recycled
    snap_disk_mb: int = 0          # disk budget of snapshot files (needs the disk tier); 0 = only checkpoints write them


@dataclass
class Sequence:
    sid: int
    row: int                       # block-table row
    slot: int                      # GDN state row
    tokens: list = field(default_factory=list)    # all tokens so far (prompt + generated)
    n_cached: int = 0              # tokens whose KV / GDN state is materialised
    pages: list = field(default_factory=list)     # device pages, one reference each held by the sequence
    n_prompt: int = 0
    reused: int = 0                # prompt tokens served from the prefix cache
    chain: object = None           # block hashes of the prompt (numpy uint64)
    meank: object = None           # KV selection: block means of de-rotated keys (last full-attention layer), float [blocks, hkv, hd]
    meank_n: int = 0               # blocks indexed so far
    view: list = None              # block indices of the current view (ascending, ends with the block being written)
    view_at: int = 0               # block index at which the view was last selected
    q_ring: object = None          # KV selection: the newest queries of this sequence, bf16 [window, hq, hd] (ring by step)
    q_ring_pos: object = None      # their rope positions, int32 [window]
    q_ring_n: int = 0              # queries recorded so far
    tokens_epoch: int = 0          # bumped by every edit of ``tokens`` other than an append (host-side caches of the history key on it)
    gap_from: int = None           # first token index after which the KV is carried memory (leave-gap deletions); None = exact
    images: list = field(default_factory=list)    # [(first token index, merged embeddings [n, H], fingerprint)]
    pos3: object = None            # multimodal (t, h, w) position ids of the prompt, int32 [3, n_prompt] (None = text only)
    rope_delta: int = 0            # rope position of a decode token = its cache index + rope_delta
    snap_points: dict = field(default_factory=dict)   # page-aligned prompt position -> (class, rank) of the snapshot to take there
    session: str = None            # whose snapshots these are (per-session cap)
    tail_hash: int = None          # prefix hash of this sequence's rolling generation-phase snapshot


class Engine:
    def __init__(self, cfg: EngineConfig, *, spec: ModelSpec | None = None, weights: H.HybridWeights | None = None,
                 comm=None, device=None, ledger=None, limits=None):
        """``device="cpu"`` boots the engine on the CPU face (``engine/cpu_mock.py``): every host-side mechanism runs over a
        stand-in model, ``limits`` (``utils.cpuface.MockLimits``) injects the capacity and capture limits."""
        from ..store.kv import KvStore
        from ..store.rel import Rel
        from ..store.state import StateStore
        from ..store.tiers import HostTier, Mover, page_bytes
        from ..utils.ledger import ledger_for

        self.cfg = cfg
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.mock = self.device.type == "cpu"
        if self.mock and ledger is None and limits is not None and limits.vram_bytes:
            from .cpu_mock import ledger_from

            ledger = ledger_from(limits)
        full = spec or PRESETS[cfg.model]()
        if cfg.n_layers is not None:
            from dataclasses import replace
            full = replace(full, n_layers=cfg.n_layers)
        if cfg.rope_yarn and cfg.rope_yarn[0] > 1.0:
            from dataclasses import replace
            full = replace(full, rope_yarn=tuple(cfg.rope_yarn))
        self.full_spec = full
        self.ledger = ledger if ledger is not None else ledger_for(self.device)
        self.comm = comm
        world = comm.world if comm is not None else 1
        rank = comm.rank if comm is not None else 0
        self.spec = full.sharded(rank, world) if world > 1 and full.tp_world == 1 else full
        if self.mock and weights is None:
            from types import SimpleNamespace

            weights = SimpleNamespace(embed=None, vocab_offset=0, layers=[])
        self.weights = weights or H.random_weights(self.spec, self.device, group=cfg.group, seed=cfg.seed + rank * 7919,
                                                   lm_head_int8=cfg.lm_head_int8,
                                                   layout="block" if cfg.decode_gemv == "tc" else "slice",
                                                   vocab_split=cfg.vocab_split,
                                                   quant="nvfp4" if cfg.quant == "nvfp4" else "w4a16")
        self.ledger.track_tree("weights", "weights", self.weights)
        n_rows = cfg.n_slots + cfg.n_snap_rows + max(1, cfg.spec_rows)
        if cfg.n_pages <= 0:
            cfg.n_pages = self._plan_pages(cfg, n_rows)
        self.ledger.check("kv pool + gdn state", cfg.n_pages * H.StatePool.bytes_per_page(self.spec, cfg.kv_dtype)
                          + n_rows * H.StatePool.bytes_per_slot(self.spec))
        # GDN rows: one per sequence slot, the prefix-snapshot rows, and the scratch rows for speculative rollback
        self.pool = H.StatePool(self.spec, self.device, cfg.n_pages, n_rows, kv_dtype=cfg.kv_dtype)
        for nm in ("k_pool", "v_pool", "k_scale", "v_scale"):
            if getattr(self.pool, nm, None) is not None:
                self.ledger.track("pool." + nm, "kv pool", getattr(self.pool, nm))
        self.ledger.track("pool.conv_state", "gdn state", self.pool.conv_state)
        self.ledger.track("pool.rec_state", "gdn state", self.pool.rec_state)
        self.spec_row = cfg.n_slots + cfg.n_snap_rows
        self.max_blocks = (cfg.max_seq + PAGE - 1) // PAGE
        if self.mock:
            from .cpu_mock import NullRunner

            self.runner = NullRunner(self.spec, self.pool, max_seqs=cfg.max_seqs * (2 if cfg.kvmem_budget else 1),
                                     max_blocks=self.max_blocks, limits=limits)
        else:
            self.runner = H.HybridRunner(self.spec, self.weights, self.pool, max_seqs=cfg.max_seqs * (2 if cfg.kvmem_budget else 1),
                                         max_blocks=self.max_blocks, prefill_chunk=cfg.prefill_chunk, comm=comm,
                                         pdl=cfg.pdl, prefill_gemm=cfg.prefill_gemm)
        self.runner.decode_gemv = cfg.decode_gemv
        if cfg.attn_splits:
            self.runner.attn_splits = cfg.attn_splits
        self.runner.use_graphs = cfg.cuda_graph
        if cfg.act_bits != 15:
            assert cfg.act_bits == 8, "act_bits is 15 or 8"
            self.runner.act_bits = 8
        self.ledger.track_tree("runner", "workspace", {k: v for k, v in vars(self.runner).items() if k not in ("w", "pool", "comm")})
        if comm is not None and getattr(comm, "symm", None) is not None:
            self.ledger.track("symmetric workspace", "symmetric", comm.symm.buf)
        self.kv = KvStore(cfg.n_pages, PAGE)
        from ..store.snap_policy import SessionCap

        self.states = StateStore(cfg.n_slots, cfg.n_snap_rows, cap=SessionCap(cfg.snap_session_cap, cfg.snap_structural_reserve))
        if cfg.evict_policy != "lru":
            self.kv.set_policy(cfg.evict_policy)
        self.host = HostTier(page_bytes(self.pool), cfg.host_cache_mb << 20, segment_bytes=cfg.pinned_segment_mb << 20) \
            if cfg.host_cache_mb else None
        self.mover = Mover(self.pool, self.host) if self.host else None
        self.disk = None
        if cfg.disk_cache_mb and cfg.disk_dir and self.host is not None:
            from ..store.tiers import DiskTier

            self.disk = DiskTier(cfg.disk_dir, page_bytes(self.pool), cfg.disk_cache_mb << 20,
                                 state_capacity=(cfg.snap_disk_mb << 20) if cfg.snap_disk_mb else None)
        elif cfg.snap_disk_mb:
            raise ValueError("snap_disk_mb needs the disk tier (host_cache_mb, disk_cache_mb and disk_dir)")
        # every move between the device pool, the host tier and the disk tier goes through the relocation facade
        self.rel = Rel(self.kv, self.states, self.pool, self.host, self.mover, self.disk, PAGE,
                       snap_host_bytes=cfg.snap_host_mb << 20, no_reclaim=cfg.no_reclaim)
        self.adopted = self.rel.adopt() if self.disk is not None else {"blocks": 0, "states": 0}
        self._last_rows: dict = {}
        self.free_rows = list(range(cfg.max_seqs - 1, -1, -1))
        self.seqs: dict[int, Sequence] = {}
        self._next_sid = 0
        # pinned staging for the host-fed step
        pin = (lambda t: t) if self.mock else (lambda t: t.pin_memory())
        self.h_inp = pin(torch.zeros(self.runner.inp.numel(), dtype=torch.int32))
        self.h_tok = pin(torch.zeros(H.HybridRunner.MAX_ROWS, dtype=torch.int32))
        self.h_inp_np = self.h_inp.numpy()
        self.h_tok_np = self.h_tok.numpy()
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.prefix_hits = self.prefix_lookups = 0
        self.last_recall: dict = {}
        self.recall_modes: dict = {}

    # counters that used to live on the engine (kept for callers and tests)
    @property
    def spilled(self) -> int:
        return self.rel.spilled

    @property
    def recalled(self) -> int:
        return self.rel.recalled

    @property
    def host_slot_of(self) -> dict:
        return self.rel.host_slot_of

    def _plan_pages(self, cfg: EngineConfig, n_rows: int) -> int:
        """``n_pages = 0``: the KV pool takes what the declared budget leaves after the weights (already on the device and
        in the ledger), the recurrent-state rows and the workspace reserve; the boot refuses when that is not enough for
        one sequence of ``max_seq`` tokens."""
        from ..store.budget import BudgetError, MemoryPlan

        led = self.ledger
        plan = MemoryPlan(total=led._total(), budget_frac=led.budget_frac, reserve=led.reserve, weights=led.used(),
                          gdn_rows=n_rows * H.StatePool.bytes_per_slot(self.spec), workspace=cfg.workspace_reserve_mb << 20,
                          page_bytes=H.StatePool.bytes_per_page(self.spec, cfg.kv_dtype))
        plan.check(min_pages=(cfg.max_seq + PAGE - 1) // PAGE + 8)
        cap = ((cfg.max_seq + PAGE - 1) // PAGE + 8) * max(cfg.n_slots, 1) * 2        # no point in more than every slot twice over
        self.memory_plan = plan
        if plan.kv_pages <= 0:
            raise BudgetError("no room for a KV pool")
        return int(min(plan.kv_pages, cap))

    def checkpoint(self, include_device: bool = True, budget_bytes: int | None = None) -> dict:
        """Write the cached prefix blocks and their state snapshots through to the disk tier and save the restart index
        (called in beats of ``budget_bytes`` while the server is idle, and whole at shutdown)."""
        return self.rel.checkpoint(include_device, budget_bytes)

    def relieve(self) -> int:
        """Watermark relief between steps (``store/rel.py``): demote cold prefix blocks before an admission needs the room."""
        return self.rel.relieve()

    def close(self) -> None:
        """Orderly end: checkpoint when a disk tier is configured, stop its writer."""
        if self.disk is not None:
            self.rel.checkpoint()
            self.disk.close()

    # -- pages ----------------------------------------------------------------------------------
    def _alloc_pages(self, n: int) -> list[int]:
        """Pages from the pool; under pressure the prefix tree gives up leaf-LRU blocks (demoted to the
        pinned-host tier when one is configured, dropped otherwise)."""
        got = self.kv.alloc(n)
        if got is not None:
            return got
        self.rel.make_room(n)
        got = self.kv.alloc(n)
        if got is None:
            raise RuntimeError("KV pool exhausted")
        return got

    def _mover_sync(self) -> None:
        if self.mover is not None:
            self.mover.sync()

    def _ensure_pages(self, seq: Sequence, n_tokens: int) -> None:
        need = (n_tokens + PAGE - 1) // PAGE
        if need > self.max_blocks:
            raise RuntimeError(f"sequence longer than max_seq ({n_tokens} tokens)")
        if need > len(seq.pages):
            new = self._alloc_pages(need - len(seq.pages))
            start = len(seq.pages)
            seq.pages.extend(new)
            self.runner.block_table[seq.row, start:start + len(new)] = torch.tensor(new, dtype=torch.int32,
                                                                                      device=self.device)

    # -- sequences ------------------------------------------------------------------------------
    def _hash_tokens(self, seq_or_tokens, images=None) -> list[int]:
        """Tokens as seen by the prefix cache: every image-pad run is replaced by values derived from the
        image's content fingerprint, so two prompts share a cached block only if they show the same pixels."""
        toks = list(seq_or_tokens)
        for first, emb, fp in images or []:
            for j in range(emb.shape[0]):
                if first + j < len(toks):
                    toks[first + j] = ((fp >> (8 * (j % 8))) ^ (j * 0x9E3779B1)) & 0x7FFFFFFF
        return toks

    def add_sequence(self, prompt: list[int], reuse: bool = True, images: list | None = None,
                     image_pad_id: int | None = None, session: str | None = None, snap_extra: list | None = None) -> int:
        """Start a sequence. With ``reuse`` the longest cached prefix for which a GDN snapshot exists
        is adopted: its KV pages are shared (pinned) and the snapshot is copied into the new row.

        ``images``: ``[(merged embeddings [n_i, hidden], (t, gh, gw), fingerprint)]`` in prompt order
        (``models.vision``); their rows replace the ``image_pad_id`` tokens and the prompt gets
        (t, h, w) position ids. ``session`` tags the sequence's snapshots (per-session cap); ``snap_extra``: further
        page-aligned prompt positions worth a snapshot (the start of a segment the client may drop later)."""
        reuse = reuse and self.cfg.prefix_cache
        if not self.free_rows:
            raise RuntimeError("no free sequence row")
        sid = self._next_sid
        slot = self.states.borrow(sid)
        if slot is None:
            raise RuntimeError("no free GDN state row (concurrency ceiling reached)")
        self._next_sid += 1
        seq = Sequence(sid, self.free_rows.pop(), slot, list(prompt), n_prompt=len(prompt), session=session)
        self.pool.reset_slot(slot)
        if images:
            from ..models.vision import mrope_positions

            merge = 2
            seq.pos3, nxt = mrope_positions(list(prompt), image_pad_id, [g for _, g, _ in images], merge)
            seq.rope_delta = nxt - len(prompt)
            i = 0
            for emb, grid, fp in images:
                while prompt[i] != image_pad_id:
                    i += 1
                seq.images.append((i, emb, fp))
                i += emb.shape[0]
        usable = (len(prompt) - 1) // PAGE * PAGE             # at least one token is always prefilled
        seq.chain = self.kv.chain(self._hash_tokens(prompt, seq.images)[:usable]) if reuse and usable else None
        self._plan_snapshots(seq, snap_extra)
        if seq.chain is not None and len(seq.chain):
            self.prefix_lookups += 1
            m, pages, carriers = self.kv.match(seq.chain)
            snap = self.rel.find_snapshot(seq.chain[:m]) if m else None
            keep = snap.n_tokens // PAGE if snap else 0
            keep0 = keep

            def one_page():
                try:
                    return self._alloc_pages(1)[0]              # may push other cold blocks down a tier
                except RuntimeError:
                    return None
            keep, promoted = self.rel.promote(seq.chain, keep, pages, carriers, one_page, mode=self.cfg.recall_mode) \
                if any(c != 0 for c in carriers[:keep]) else (keep, set())
            if keep < keep0:
                # the recurrent state must match the KV prefix: fall back to the longest snapshot inside what is resident
                snap = self.rel.find_snapshot(seq.chain[:keep]) if keep else None
                keep = snap.n_tokens // PAGE if snap else 0
            self.kv.unref([p for j, (p, c) in enumerate(zip(pages[:m], carriers[:m])) if j >= keep and (c == 0 or j in promoted)])
            if keep:
                seq.pages = pages[:keep]
                self.runner.block_table[seq.row, :keep] = torch.tensor(seq.pages, dtype=torch.int32, device=self.device)
                self.pool.copy_slot(snap.row, slot)
                seq.n_cached = seq.reused = keep * PAGE
                self.prefix_hits += 1
            # the recall report: "exact" = KV blocks and a recurrent state of the same point were both found; "context_only"
            # = blocks matched but no state snapshot lies inside them (a hybrid model cannot resume from KV alone); "miss"
            self.last_recall = {"mode": "exact" if keep else ("context_only" if m else "miss"), "prompt_blocks": len(seq.chain),
                                "matched_blocks": m, "used_blocks": keep, "promoted_blocks": len(promoted),
                                "from_lower_tiers": sum(1 for c in carriers[:keep0] if c != 0),
                                "snapshot_tokens": snap.n_tokens if (snap is not None and keep) else 0}
            self.recall_modes[self.last_recall["mode"]] = self.recall_modes.get(self.last_recall["mode"], 0) + 1
        self.seqs[sid] = seq
        return sid

    def _plan_snapshots(self, seq: Sequence, extra: list | None = None) -> None:
        """Prompt positions at which the recurrent state is saved while this prompt is prefilled: the kept message
        boundaries with their eviction classes, caller-named extra points, and the prompt's last page boundary."""
        from ..store import snap_policy as P

        seq.snap_points = {}
        if seq.chain is None or not len(seq.chain):
            return
        usable = len(seq.chain) * PAGE
        cfg = self.cfg
        if cfg.msg_open_ids:
            pts = [p for p in P.message_points(seq.tokens[:seq.n_prompt], cfg.msg_open_ids, PAGE, cfg.snap_msg_min_gap,
                                               cfg.snap_msg_recent) if p <= usable]
            seq.snap_points.update(zip(pts, P.classify(pts, seq.n_prompt, cfg.snap_msg_recent)))
        for p in extra or ():
            if 0 < p <= usable and p % PAGE == 0:
                seq.snap_points.setdefault(int(p), ("extra", 0))
        seq.snap_points[usable] = ("durable", 0)

    def _hash_slice(self, seq: Sequence, lo: int, hi: int) -> list:
        """``_hash_tokens`` of tokens [lo, hi) only (the generation phase extends a chain block by block)."""
        toks = list(seq.tokens[lo:hi])
        for first, emb, fp in seq.images or []:
            for j in range(max(first, lo) - first, min(first + emb.shape[0], hi) - first):
                toks[first + j - lo] = ((fp >> (8 * (j % 8))) ^ (j * 0x9E3779B1)) & 0x7FFFFFFF
        return toks

    def _tail_snapshot(self, seq: Sequence, pos_before: int) -> None:
        """Generation advanced the sequence from ``pos_before`` to ``seq.n_cached`` cached tokens and its state row holds
        the state after exactly ``n_cached`` tokens: when that is a page boundary on the configured stride, save it as the
        sequence's rolling snapshot (the previous one is released), keyed like the blocks ``free_sequence`` will publish."""
        from ..store.snap_policy import decode_boundary

        if seq.gap_from is not None or not self.cfg.prefix_cache:
            return
        if seq.chain is None:
            seq.chain = np.zeros(0, dtype=np.uint64)          # a prompt shorter than a page: the chain starts with the answer
        b = decode_boundary(pos_before, seq.n_cached, PAGE, self.cfg.snap_decode_stride)
        if b is None or b != seq.n_cached:
            return
        have = len(seq.chain)
        if have < b // PAGE:
            more = self.kv.chain(self._hash_slice(seq, have * PAGE, b), root=int(seq.chain[-1]) if have else 0)
            seq.chain = np.concatenate([seq.chain, more])
        h = int(seq.chain[b // PAGE - 1])
        old = seq.tail_hash
        row = self.states.snapshot(h, b, "tail", session=seq.session)
        if row is None:
            return
        self.pool.copy_slot(seq.slot, row)
        if old is not None and old != h and old in self.states.snaps and self.states.snaps[old].klass == "tail":
            self.states.forget(old)
        seq.tail_hash = h

    def snapshot_now(self, sid: int, klass: str = "dense") -> bool:
        """Save the sequence's recurrent state as it stands, when it stands on a page boundary inside the prompt's chain
        (a turn cancelled between two prefill chunks: the blocks it wrote are published, and with this snapshot the retry
        resumes behind them instead of recomputing the prompt). Returns whether a snapshot was taken."""
        seq = self.seqs.get(sid)
        if seq is None or seq.chain is None or seq.gap_from is not None or not self.cfg.prefix_cache:
            return False
        n = seq.n_cached
        if n < PAGE or n % PAGE or n // PAGE > len(seq.chain) or n <= seq.reused:
            return False
        h = int(seq.chain[n // PAGE - 1])
        if h in self.states.snaps:
            return False
        row = self.states.snapshot(h, n, klass, session=seq.session)
        if row is None:
            return False
        self.pool.copy_slot(seq.slot, row)
        return True

    def free_sequence(self, sid: int, publish: bool = True) -> None:
        """End a sequence: index its full blocks in the prefix tree (the tree takes its own
        references) and give pages, row and state row back."""
        seq = self.seqs.pop(sid)
        if publish and self.cfg.prefix_cache and seq.n_cached >= PAGE:
            exact = seq.n_cached if seq.gap_from is None else min(seq.n_cached, seq.gap_from)
            nb = min(exact // PAGE, len(seq.pages))
            hashed = self._hash_tokens(seq.tokens, seq.images)[:nb * PAGE]
            chain = self.kv.chain(hashed)
            self.kv.publish(chain, seq.pages[:nb])
            if self.disk is not None:
                self.rel.note_published(chain, hashed)
        self.kv.unref(seq.pages)
        self.free_rows.append(seq.row)
        self.states.give_back(sid)

    # -- live-sequence surgery (agent sessions) --------------------------------------------------
    def drop_ranges(self, sid: int, ranges: list) -> int:
        """Leave-gap deletion on a live sequence: unlink the pages of the page-aligned token ranges ``[lo, hi)`` (all inside
        the cached part). Survivors keep their KV and their rotary positions; the position ledger keeps the hole
        (``rope_delta`` grows by the removed length, so new tokens continue from the old maximum position + 1). Returns the
        number of tokens removed. What precedes the first range stays content-addressable; what follows it is carried
        memory and is no longer published to the prefix tree (``engine/img_evict.py`` has the host-side rules)."""
        from .img_evict import page_map

        seq = self.seqs[sid]
        ranges = sorted(ranges)
        assert all(lo % PAGE == 0 and hi % PAGE == 0 and 0 <= lo < hi <= seq.n_cached for lo, hi in ranges)
        keep = page_map(len(seq.pages) * PAGE, ranges, PAGE)
        gone = [p for i, p in enumerate(seq.pages) if i not in set(keep)]
        seq.pages = [seq.pages[i] for i in keep]
        self.kv.unref(gone)
        row = torch.zeros(self.max_blocks, dtype=torch.int32)
        row[:len(seq.pages)] = torch.tensor(seq.pages, dtype=torch.int32)
        self.runner.block_table[seq.row].copy_(row.to(self.device))
        removed = 0
        for lo, hi in reversed(ranges):
            del seq.tokens[lo:hi]
            removed += hi - lo
        seq.tokens_epoch += 1
        if seq.pos3 is not None:
            keep_tok = torch.ones(seq.pos3.shape[1], dtype=torch.bool)
            for lo, hi in ranges:
                keep_tok[lo:hi] = False
            seq.pos3 = seq.pos3[:, keep_tok]
        shifted = []
        for first, emb, fp in seq.images:
            if any(lo <= first < hi for lo, hi in ranges):
                continue
            shifted.append((first - sum(hi - lo for lo, hi in ranges if hi <= first), emb, fp))
        seq.images = shifted
        seq.n_cached -= removed
        seq.n_prompt = max(0, seq.n_prompt - removed)
        seq.rope_delta += removed
        seq.gap_from = min(ranges[0][0], seq.gap_from if seq.gap_from is not None else ranges[0][0])
        seq.chain = None
        seq.meank_n, seq.view = min(seq.meank_n, ranges[0][0] // PAGE), None
        return removed

    def extend_sequence(self, sid: int, new_tokens: list, images: list | None = None, image_pad_id: int | None = None) -> int:
        """Continue a live sequence with more prompt tokens (the next turn of an agent session on its parked sequence): the
        not-yet-cached tail (the last sampled token and ``new_tokens``, new images included) is prefilled from the sequence's
        current position; returns the next token."""
        self.append_tokens(sid, new_tokens, images, image_pad_id)
        return self.prefill(sid)

    def _pos3_cover(self, seq, upto: int) -> None:
        """The (t, h, w) position ledger covers the prompt it was built for; tokens after it (sampled ones, appended text)
        sit at cache index + ``rope_delta`` in all three components."""
        n = seq.pos3.shape[1]
        if n < upto:
            ext = torch.arange(n + seq.rope_delta, upto + seq.rope_delta, dtype=torch.int32).repeat(3, 1)
            seq.pos3 = torch.cat([seq.pos3, ext], 1)

    def append_tokens(self, sid: int, new_tokens: list, images: list | None = None, image_pad_id: int | None = None) -> None:
        """More prompt for a live sequence, without running it. ``images`` (same triples as ``add_sequence``) belong to the
        image-pad runs inside ``new_tokens``: their (t, h, w) blocks start at the sequence's next position."""
        seq = self.seqs[sid]
        new_tokens = [int(t) for t in new_tokens]
        base = len(seq.tokens)
        if images:
            from ..models.vision import mrope_positions

            if seq.pos3 is None:
                seq.pos3 = torch.zeros(3, 0, dtype=torch.int32)
            self._pos3_cover(seq, base)
            p0 = base + seq.rope_delta
            pos, nxt = mrope_positions(new_tokens, image_pad_id, [g for _, g, _ in images], 2)
            seq.pos3 = torch.cat([seq.pos3, pos + p0], 1)
            i = 0
            for emb, grid, fp in images:
                while new_tokens[i] != image_pad_id:
                    i += 1
                seq.images.append((base + i, emb, fp))
                i += emb.shape[0]
            seq.rope_delta = p0 + nxt - (base + len(new_tokens))
        seq.tokens.extend(new_tokens)
        seq.n_prompt = len(seq.tokens)
        if seq.gap_from is None:
            usable = (seq.n_prompt - 1) // PAGE * PAGE        # the longer prompt has its own block identities
            seq.chain = self.kv.chain(self._hash_tokens(seq.tokens, seq.images)[:usable]) if usable and self.cfg.prefix_cache else None
            self._plan_snapshots(seq)
            seq.snap_points = {p: c for p, c in seq.snap_points.items() if p > seq.n_cached}

    # -- prefill ------------------------------------------------------------------------------
    def prefill_range(self, sid: int, start: int, end: int, want_token: bool):
        """Feed prompt tokens [start, end) (start == tokens already cached). A GDN snapshot is taken when
        ``end`` is the last block boundary of the prompt, so later requests can reuse the prefix."""
        seq = self.seqs[sid]
        assert start == seq.n_cached and end <= seq.n_prompt
        self._ensure_pages(seq, end + 1)
        ids = torch.tensor(seq.tokens[start:end], dtype=torch.int32)
        if not self.mock:
            ids = ids.pin_memory().to(self.device, non_blocking=True)
        embeds = pos3 = None
        if seq.images:
            # text rows from the embedding table, image rows from the vision tower's merged embeddings
            embeds = torch.empty(end - start, self.spec.hidden, dtype=torch.bfloat16, device=self.device)
            K.embed(ids, self.weights.embed, embeds, end - start)
            for first, emb, _ in seq.images:
                lo, hi = max(first, start), min(first + emb.shape[0], end)
                if lo < hi:
                    embeds[lo - start:hi - start] = emb[lo - first:hi - first].to(self.device, torch.bfloat16)
            self._pos3_cover(seq, end)
            pos3 = seq.pos3[:, start:end].to(self.device)
        elif seq.rope_delta:
            # positions after a leave-gap deletion: cache index + the removed length
            pos3 = torch.arange(start + seq.rope_delta, end + seq.rope_delta, dtype=torch.int32, device=self.device).repeat(3, 1)
        pts = [p for p in seq.snap_points if start < p <= end and p > seq.reused] if seq.chain is not None else []
        inside = [p for p in pts if p < end]
        snap = None
        if inside:
            # a snapshot point lies inside this chunk: the runner leaves the GDN state of that point in the snapshot row
            # (one per chunk: `prefill_plan` cuts so that a chunk holds at most one inside and one at its end)
            p = max(inside)
            row = self.states.snapshot(int(seq.chain[p // PAGE - 1]), p, *seq.snap_points[p], session=seq.session)
            if row is not None:
                snap = (p - start, row)
        tok = self.runner.prefill_chunk_forward(ids, start, seq.row, seq.slot, want_logits=want_token, embeds=embeds,
                                                pos3=pos3, snap=snap)
        seq.n_cached = end
        if end in pts:
            row = self.states.snapshot(int(seq.chain[end // PAGE - 1]), end, *seq.snap_points[end], session=seq.session)
            if row is not None:
                self.pool.copy_slot(seq.slot, row)
        for p in pts:
            if seq.snap_points[p][0] == "durable":
                self.states.supersede(seq.chain[:p // PAGE], p)       # this conversation's earlier anchors become fork points
        if want_token:
            t = int(tok.item())
            seq.tokens.append(t)
            return t
        return None

    def prefill_plan(self, sid: int) -> list[tuple[int, int]]:
        """Chunk boundaries for the rest of the prompt: multiples of prefill_chunk. The GDN snapshot at the last block
        boundary is taken inside the chunk that contains it (``snap`` of the runner), so no few-row tail chunk is cut
        off; ``cfg.snap_cut`` restores the separate cut."""
        seq = self.seqs[sid]
        n, c = seq.n_prompt, self.cfg.prefill_chunk
        boundary = (n - 1) // PAGE * PAGE
        pts = sorted(p for p in seq.snap_points if p > max(seq.n_cached, seq.reused)) if seq.chain is not None else []
        out, lo = [], seq.n_cached
        while lo < n:
            hi = min(lo + c, n)
            inside = [p for p in pts if lo < p < hi]
            if len(inside) > 1:
                hi = inside[1]             # one point inside the chunk (saved by the runner) and one at its end (saved after it)
            if self.cfg.snap_cut and lo < boundary < hi:
                hi = boundary
            out.append((lo, hi))
            lo = hi
        return out

    def prefill(self, sid: int) -> int:
        """Feed every not-yet-cached prompt token; returns the first generated token."""
        tok = None
        plan = self.prefill_plan(sid)
        for i, (lo, hi) in enumerate(plan):
            tok = self.prefill_range(sid, lo, hi, want_token=i + 1 == len(plan))
        return tok

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
            hi[lay.pos3 + i] = pos + seq.rope_delta
            hi[lay.pos3 + b + i] = pos + seq.rope_delta
            hi[lay.pos3 + 2 * b + i] = pos + seq.rope_delta
            hi[lay.kv_slot + i] = seq.pages[pos // PAGE] * PAGE + pos % PAGE
            hi[lay.ctx + i] = pos + 1
            hi[lay.gslot + i] = seq.slot
            hi[lay.bt_row + i] = seq.row
            if self.cfg.kvmem_budget and pos + 1 > self.cfg.kvmem_budget:
                n_view = self._kvmem_view(seq, pos)
                hi[lay.ctx + i] = (n_view - 1) * PAGE + pos % PAGE + 1
                hi[lay.bt_row + i] = seq.row + self.cfg.max_seqs
            ctx_max = max(ctx_max, int(hi[lay.ctx + i]))
        graph = self.runner.capture(b, 1, ctx_hint=self._ctx_bucket(ctx_max))
        self._last_rows = {sid: i for i, sid in enumerate(sids)}     # whose query sits in which row of runner.q_rope
        n = lay.size
        self.runner.inp[:n].copy_(self.h_inp[:n], non_blocking=True)
        graph.replay()
        self.h_tok[:b].copy_(self.runner.out_tok[:b], non_blocking=True)
        if self.cfg.kvmem_budget and self.cfg.kvmem_query_tokens > 1 and not self.mock:
            self._record_queries(sids)
        if not self.mock:
            torch.cuda.current_stream().synchronize()
        self.h2d_bytes += n * 4
        self.d2h_bytes += b * 4
        self._check_status()
        out = []
        for i, sid in enumerate(sids):
            seq = self.seqs[sid]
            t = int(self.h_tok_np[i])
            seq.n_cached += 1
            seq.tokens.append(t)
            out.append(t)
            if self.cfg.snap_decode_stride and seq.n_cached % PAGE == 0:
                self._tail_snapshot(seq, seq.n_cached - 1)
        return out

    STATUS_EVERY = 16      # steps between reads of the kernels' bounded-wait status words on a tensor-parallel rank

    def _check_status(self, force: bool = False) -> None:
        """Read the native library's bounded-wait status words at the step's existing host sync point. A kernel whose wait
        for a copy, an MMA or a peer flag ran out finishes on stale data, so the tokens of such a step must not be emitted:
        the step raises, its turns fail, and under tensor parallelism the rank leaves the hand-written collectives for the
        library arm (every rank runs the same check on the same step count, so they switch together). Single-GPU steps
        check every ``STATUS_EVERY`` x 8 steps (only copy / MMA waits exist there), tensor-parallel ones every
        ``STATUS_EVERY``."""
        if self.mock:
            return
        self._status_tick = getattr(self, "_status_tick", 0) + 1
        every = self.STATUS_EVERY * (1 if self.comm is not None else 8)
        if not force and self._status_tick % every:
            return
        bad = {k: v for k, v in K.all_status().items() if v}
        if not bad:
            return
        if self.comm is not None and getattr(self.comm, "symm", None) is not None:
            self.comm.symm, self.comm.mode = None, "nccl"
            self.runner.graphs.clear()
        raise RuntimeError(f"a bounded wait ran out inside a kernel ({bad}): the step's output is discarded")

    def _record_queries(self, sids: list) -> None:
        """Keep this step's rotated query of every long sequence in its ring (what the next block selection scores with)."""
        W, sp = self.cfg.kvmem_query_tokens, self.spec
        for i, sid in enumerate(sids):
            seq = self.seqs[sid]
            if seq.n_cached + 1 <= self.cfg.kvmem_budget:
                continue
            if seq.q_ring is None:
                seq.q_ring = torch.zeros(W, sp.hq, sp.hd, dtype=torch.bfloat16, device=self.device)
                seq.q_ring_pos = torch.zeros(W, dtype=torch.int32, device=self.device)
            j = seq.q_ring_n % W
            seq.q_ring[j].copy_(self.runner.q_rope[i].view(sp.hq, sp.hd))
            seq.q_ring_pos[j] = seq.n_cached + seq.rope_delta
            seq.q_ring_n += 1

    def set_last_token(self, sid: int, tok: int) -> None:
        """Replace the sequence's newest token (the host sampled something other than the device's argmax). The next
        step reads it as its input, so under tensor parallelism this call is mirrored to every rank."""
        self.seqs[sid].tokens[-1] = int(tok)
        self.seqs[sid].tokens_epoch += 1

    def _kvmem_view(self, seq: Sequence, pos: int) -> int:
        """Bounded attention view of a long sequence: sink blocks + recent blocks + the best-scoring blocks of the rest,
        re-selected whenever the write position enters a new block. The index (block means of de-rotated keys of the last
        full-attention layer) grows incrementally; blocks are scored on the GPU against the sequence's query of the previous
        step. The view's page table lives in a second block-table row of the sequence. Returns the number of view blocks."""
        from ..store import select as S

        cur = pos // PAGE                                  # block being written
        if seq.view is not None and seq.view[-1] == cur:
            return len(seq.view)
        sp, run, dev = self.spec, self.runner, self.device
        if seq.view is not None and cur - seq.view_at < self.cfg.kvmem_recall_every and seq.view[-1] == cur - 1:
            # between two selections the block just entered joins the view as it is (one more recent block)
            seq.view = seq.view + [cur]
            row = seq.row + self.cfg.max_seqs
            run.block_table[row, len(seq.view) - 1] = seq.pages[cur]
            return len(seq.view)
        fi = sp.n_full - 1
        if seq.meank is None:
            seq.meank = torch.zeros(self.max_blocks, sp.hkv, sp.hd, dtype=torch.float32, device=dev)
        if seq.meank_n < cur:                              # index the blocks completed since the last selection
            ids = torch.arange(seq.meank_n, cur, dtype=torch.int32, device=dev)
            pages = torch.tensor(seq.pages[seq.meank_n:cur], dtype=torch.int32, device=dev)
            S.mean_k_blocks_gpu(self.pool.k_pool[fi], pages, ids * PAGE + seq.rope_delta, torch.full_like(ids, PAGE), run.inv_freq,
                                sp.rotary_dim, seq.meank[seq.meank_n:cur],
                                k_scale=None if self.pool.k_scale is None else self.pool.k_scale[fi])
            seq.meank_n = cur
        budget_blocks = max(self.cfg.kvmem_sink + self.cfg.kvmem_recent + 1, self.cfg.kvmem_budget // PAGE)
        q_row = self._last_rows.get(seq.sid, -1)
        if seq.q_ring is not None and seq.q_ring_n and cur > 0:
            # the window of newest queries (one per decode step, kept by `decode_step`)
            n = min(seq.q_ring_n, seq.q_ring.shape[0])
            scores = S.score_blocks_gpu(seq.q_ring[:n], seq.q_ring_pos[:n], seq.meank[:cur], run.inv_freq, sp.rotary_dim).cpu()
        elif q_row >= 0 and cur > 0:
            qpos = torch.tensor([pos - 1 + seq.rope_delta], dtype=torch.int32, device=dev)
            scores = S.score_blocks_gpu(run.q_rope[q_row:q_row + 1], qpos, seq.meank[:cur], run.inv_freq, sp.rotary_dim).cpu()
        else:
            scores = torch.zeros(max(cur, 1))
        scores = torch.cat([scores[:cur], torch.zeros(1)])          # the block being written is always "recent"
        seq.view = S.select(scores, cur + 1, budget_blocks, self.cfg.kvmem_sink, self.cfg.kvmem_recent)
        seq.view_at = cur
        row = seq.row + self.cfg.max_seqs
        run.block_table[row, :len(seq.view)] = torch.tensor([seq.pages[b] for b in seq.view], dtype=torch.int32, device=dev)
        return len(seq.view)

    def pool_keys(self, sid: int, layer: int | None = None) -> torch.Tensor:
        """The cached keys of a sequence as float ``[n_cached, hkv, hd]`` (rotated, as the attention kernels read them), read
        from the paged pool of one full-attention layer (default: the last, the one the KV-selection index is built on)."""
        seq = self.seqs[sid]
        fi = self.spec.n_full - 1 if layer is None else layer
        n = seq.n_cached
        pages = torch.tensor(seq.pages[:(n + PAGE - 1) // PAGE], dtype=torch.long, device=self.device)
        raw = self.pool.k_pool[fi][pages]                                  # [pages, 16, hkv, hd]
        if raw.dtype == torch.float16:
            k = raw.float()
        elif self.pool.k_scale is not None:
            k = raw.view(torch.int8).float() * self.pool.k_scale[fi][pages][..., None]
        else:
            k = raw.view(torch.float8_e4m3fn).float()
        return k.reshape(-1, k.shape[-2], k.shape[-1])[:n]

    def coverage_probe(self, sid: int, ks=(1, 2, 4, 8, 16, 32)) -> dict:
        """How much of the true attention mass of the sequence's newest queries lies in the blocks the Mean-K index scores
        highest (``store/coverage.py``). Queries: the sequence's query window when KV selection keeps one, else the query of
        its last decode step. Read-only; runs on the host."""
        from ..store import coverage as C

        seq = self.seqs[sid]
        if seq.q_ring is not None and seq.q_ring_n:
            n = min(seq.q_ring_n, seq.q_ring.shape[0])
            q, qpos = seq.q_ring[:n].float().cpu(), seq.q_ring_pos[:n].cpu()
        else:
            row = self._last_rows.get(sid)
            if row is None:
                raise RuntimeError("coverage probe: the sequence has no decode step yet (no query to probe with)")
            q = self.runner.q_rope[row:row + 1].float().cpu()
            qpos = torch.tensor([seq.n_cached - 1 + seq.rope_delta])
        k = self.pool_keys(sid).cpu()
        if seq.rope_delta:
            raise RuntimeError("coverage probe: sequences with shifted positions (images, leave-gap deletions) are not supported")
        return C.probe(q, qpos, k, self.runner.inv_freq.cpu(), self.spec.rotary_dim, PAGE, ks)

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
