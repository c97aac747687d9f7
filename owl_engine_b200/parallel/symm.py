"""Symmetric (peer-mapped) workspace of one tensor-parallel rank and the fused collectives on it.

Allocation and the address exchange use ``torch.distributed._symmetric_memory`` (CUDA VMM
allocation + handle exchange between the rank processes, NVLS multicast binding when the fabric
offers it) -- that is plumbing. Everything that moves data is our own kernel (``csrc/comm.cu``):
peers' buffers are read with plain NVLink P2P loads or ``multimem.ld_reduce`` through NVSwitch.

Workspace layout (identical on every rank, so an offset is valid on all peers):

    flags      : uint32[FLAG_SLOTS][8]          sequence numbers written by peers
    part_a/b   : bf16[MAX_ROWS][hidden]         partial sums of the two row-parallel call sites
    exch       : uint2[MAX_ROWS][8]             vocab-split argmax exchange
    big        : bf16[big_elems]                prefill-size all-reduce payload
    push_a/b   : bf16[world][MAX_ROWS][hidden]  slots the peers' GEMV epilogues write their partial sums into
    push_flags : uint32[2][8]                   sequence numbers published by the peers' GEMVs
    push_ll    : uint2[2][8][hidden/2]          one-token exchange of the FMA projections: (two bf16 sums, exchange number) words
    pf_slots   : bf16[world][max_local*128][hidden]  prefill reduce-scatter slots (partial sums of this rank's row tiles)
    pf_x       : 16-bit[pf_rows][hidden]        prefill all-gather target (normalised rows from every owner)
    pf_flags   : uint32[2][world][max_local]    reduce-scatter / all-gather sequence flags per row tile

Reference counterpart: VMM peer grant + staging header (``crates/backends/cuda/src/vmm.rs``,
``comm/ar.rs:38-175``), generalised from 2 threads in one process to 2/4/8 processes.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import kernels as K

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
K.register("owl_ar_residual_norm", [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, ctypes.c_uint,
                                    _I, _P])
K.register("owl_w4a16_skinny_push", [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P])
K.register("owl_push_residual_norm", [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, ctypes.c_uint, _P, _I, _P, _I, _P])
K.register("owl_w4_fma_tp", [_P, _P, _P, _P, _I, _I, _I, _F, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I,
                             ctypes.c_uint, _I, _I, _P])
K.register("owl_ar_inplace", [_P, _P, _P, _P, ctypes.c_longlong, _I, _I, _I, _I, ctypes.c_uint, _P])
K.register("owl_argmax_merge", [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, ctypes.c_uint, _I, _P])
K.register("owl_comm_wait_probe", [_P, ctypes.c_uint, ctypes.c_uint, _P, _P])
_U = ctypes.c_uint
K.register("owl_f16_gemm_ag", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P, _U, _I, _I, _U, _P])
K.register("owl_f16_gemm_rs", [_P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _U, _I, _I, _I, _P])
K.register("owl_rs_norm_ag", [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _U, _U, _F, _I, _I, _U, _P])

FLAG_SLOTS = 128
MAX_ROWS = 32
SPIN_LIMIT = 1 << 22          # polls (each ~100 ns once backing off): a couple of hundred ms


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class PrefillPipe:
    """Sequence-parallel prefill plumbing of one rank: GEMM + reduce-scatter, owner-side sum + residual + RMSNorm +
    all-gather, and the column-parallel GEMM that consumes the gathered rows tile by tile.

    Token rows are cut into 128-row tiles; tile j is owned by rank ``j % world`` (its local tile ``j // world``). The
    residual stream of a chunk lives only on the owners (``h``, local). All buffers are passed in, so a world of one
    (plain device tensors) exercises the same kernels and flags on a single GPU."""

    TILE = 128

    def __init__(self, rank: int, world: int, hidden: int, rows: int, *, slots, x_bytes, rs_flags, ag_flags, x_ptrs, slot_ptrs,
                 rs_flag_ptrs, ag_flag_ptrs, device):
        self.rank, self.world, self.hidden, self.rows = rank, world, hidden, rows
        self.max_local = self.max_local_for(rows, world)
        self.slots, self.x_bytes, self.rs_flags, self.ag_flags = slots, x_bytes, rs_flags, ag_flags
        self.x_ptrs, self.slot_ptrs = _ptr_array(x_ptrs), _ptr_array(slot_ptrs)
        self.rs_flag_ptrs, self.ag_flag_ptrs = _ptr_array(rs_flag_ptrs), _ptr_array(ag_flag_ptrs)
        self.h = torch.zeros(self.max_local * self.TILE, hidden, dtype=torch.bfloat16, device=device)
        self.rs_done = torch.zeros((rows + self.TILE - 1) // self.TILE, dtype=torch.int32, device=device)
        self.rows_done = torch.zeros(self.max_local, dtype=torch.int32, device=device)
        self.rs_seq = self.ag_seq = 0
        self.device = device

    @classmethod
    def max_local_for(cls, rows: int, world: int) -> int:
        tiles = (rows + cls.TILE - 1) // cls.TILE
        return (tiles + world - 1) // world

    @classmethod
    def local(cls, hidden: int, rows: int, device) -> "PrefillPipe":
        """A world of one on plain device memory (single-GPU tests of the protocol)."""
        ml = cls.max_local_for(rows, 1)
        slots = torch.zeros(ml * cls.TILE, hidden, dtype=torch.bfloat16, device=device)
        xb = torch.zeros(rows * hidden * 2, dtype=torch.uint8, device=device)
        rf = torch.zeros(ml, dtype=torch.int32, device=device)
        af = torch.zeros(ml, dtype=torch.int32, device=device)
        return cls(0, 1, hidden, rows, slots=slots, x_bytes=xb, rs_flags=rf, ag_flags=af, x_ptrs=[xb.data_ptr()],
                   slot_ptrs=[slots.data_ptr()], rs_flag_ptrs=[rf.data_ptr()], ag_flag_ptrs=[af.data_ptr()], device=device)

    def x(self, t: int, dtype) -> torch.Tensor:
        """This rank's copy of the gathered activation rows."""
        return self.x_bytes[:t * self.hidden * 2].view(dtype).view(t, self.hidden)

    def own_rows(self, t: int) -> torch.Tensor:
        """Global row numbers of the rows this rank owns, in local order (padded tiles clipped to t)."""
        tiles = (t + self.TILE - 1) // self.TILE
        if self.rank >= tiles:                                # a chunk with fewer row tiles than ranks: nothing to own
            return torch.empty(0, dtype=torch.int64, device=self.device)
        mine = torch.arange(self.rank, tiles, self.world)
        rows = (mine[:, None] * self.TILE + torch.arange(self.TILE)[None]).reshape(-1)
        return rows.to(self.device)

    def local_row(self, row: int) -> tuple[int, int]:
        """(owner rank, local row) of a global token row."""
        j = row // self.TILE
        return j % self.world, (j // self.world) * self.TILE + row % self.TILE

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, t: int) -> None:
        """Partial sums of ``x[:t] @ w^T`` go to the owners' slots (row-parallel GEMM + reduce-scatter)."""
        assert x.dtype == w.dtype and w.shape[0] == self.hidden and t <= self.rows
        self.rs_seq += 1
        K.call("owl_f16_gemm_rs", K.ptr(x), x.stride(0), K.ptr(w), w.stride(0), t, w.shape[0], x.shape[1], self.hidden,
               1 if x.dtype == torch.bfloat16 else 0, self.slot_ptrs, self.rs_flag_ptrs, K.ptr(self.rs_done), self.rs_seq,
               self.rank, self.world, self.max_local, K.stream())

    def reduce_norm_gather(self, t: int, norm_w, *, out_dtype=torch.float16, eps: float = 1e-6, seed: bool = False,
                           one_plus_w: bool = True) -> None:
        """Owner side: residual rows += slots (unless ``seed``), then normalised rows to every rank (unless ``norm_w`` is
        None, which only updates the residual)."""
        if norm_w is not None:
            self.ag_seq += 1
        K.call("owl_rs_norm_ag", K.ptr(self.slots), K.ptr(self.rs_flags), K.ptr(self.h), K.ptr(norm_w), self.x_ptrs,
               self.ag_flag_ptrs, K.ptr(self.rows_done), t, self.hidden, self.rank, self.world, self.max_local,
               0 if seed else self.world, self.rs_seq, self.ag_seq, eps, int(one_plus_w), int(out_dtype == torch.float16),
               SPIN_LIMIT, K.stream())

    def gemm_ag(self, w: torch.Tensor, out: torch.Tensor, t: int) -> torch.Tensor:
        """``out[:t] = gathered_x[:t] @ w^T``, starting on the row tiles that have arrived."""
        x = self.x(t, w.dtype)
        K.call("owl_f16_gemm_ag", K.ptr(x), x.stride(0), K.ptr(w), w.stride(0), K.ptr(out), t, w.shape[0], self.hidden,
               out.stride(0), 1 if w.dtype == torch.bfloat16 else 0, K.ptr(self.ag_flags), self.ag_seq, self.world,
               self.max_local, SPIN_LIMIT, K.stream())
        return out


class LocalSplit:
    """The push / pull pairing of the one-token projections on ONE GPU (no peers): a row-parallel projection with few row
    tiles is cut into ``kparts`` k parts whose partial sums land in slots of a plain device buffer, and the next
    column-parallel projection adds them in its prologue. Same kernels, flags and sequence numbers as the tensor-parallel
    form with a world of one, so a single GPU exercises the protocol."""

    def __init__(self, device, hidden: int, kparts: int = 4):
        self.rank, self.world, self.device, self.hidden, self.kparts = 0, 1, device, hidden, kparts
        from ..utils.ledger import ledger_for

        led = ledger_for(device)
        self.buf = led.alloc("k-split slots", "workspace", (2, 8, MAX_ROWS, hidden), torch.bfloat16, zero=True)
        self.flags = torch.zeros(2, 8, dtype=torch.int32, device=device)
        self.push_slots = [self.buf[0], self.buf[1]]
        self.push_flags_local = [self.flags[0], self.flags[1]]
        self.push_dst = [_ptr_array([self.buf[w].data_ptr()]) for w in range(2)]
        self.push_flag = [_ptr_array([self.flags[w].data_ptr()]) for w in range(2)]
        self.push_count = torch.zeros(2, dtype=torch.int32, device=device)
        self.push_seq = torch.zeros(2, dtype=torch.int32, device=device)
        self.push_counters = torch.zeros(2, MAX_ROWS, dtype=torch.int32, device=device)
        self.ll = led.alloc("k-split words", "workspace", (2, 8, hidden // 2, 2), torch.int32, zero=True)
        self.push_ll_local = [self.ll[0], self.ll[1]]
        self.push_ll = [_ptr_array([self.ll[w].data_ptr()]) for w in range(2)]
        self.pull_count = torch.zeros(2, dtype=torch.int32, device=device)


class SymmetricWorkspace:
    def __init__(self, rank: int, world: int, device, group=None, hidden: int = 5120, big_elems: int = 2048 * 5120,
                 use_multimem: bool = False):
        import torch.distributed._symmetric_memory as symm_mem

        self.rank, self.world, self.device, self.hidden = rank, world, device, hidden
        self.off_flags = 0
        self.off_a = FLAG_SLOTS * 8 * 4
        self.off_b = self.off_a + MAX_ROWS * hidden * 2
        self.off_exch = self.off_b + MAX_ROWS * hidden * 2
        self.off_big = (self.off_exch + MAX_ROWS * 8 * 8 + 255) // 256 * 256
        self.big_elems = big_elems
        self.off_push = (self.off_big + big_elems * 2 + 255) // 256 * 256
        self.kparts = 1          # k parts of the one-token row-parallel projections (ranks x parts <= 8; one: whole tiles)
        push_bytes = 8 * MAX_ROWS * hidden * 2
        self.off_pflags = self.off_push + 2 * push_bytes
        pf_rows = big_elems // hidden
        ml = PrefillPipe.max_local_for(pf_rows, world)
        self.off_ll = (self.off_pflags + 2 * 8 * 4 + 255) // 256 * 256
        ll_bytes = 8 * (hidden // 2) * 8
        self.off_pf_slots = (self.off_ll + 2 * ll_bytes + 255) // 256 * 256
        pf_slot_bytes = world * ml * PrefillPipe.TILE * hidden * 2
        self.off_pf_x = self.off_pf_slots + pf_slot_bytes
        self.off_pf_flags = self.off_pf_x + pf_rows * hidden * 2
        nbytes = self.off_pf_flags + 2 * world * ml * 4
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        gname = (group or dist.group.WORLD).group_name
        self.handle = symm_mem.rendezvous(self.buf, gname)
        torch.cuda.synchronize()
        dist.barrier(group=group)
        base = [int(p) for p in self.handle.buffer_ptrs]
        self.flag_ptrs = _ptr_array([b + self.off_flags for b in base])
        self.a_ptrs = _ptr_array([b + self.off_a for b in base])
        self.b_ptrs = _ptr_array([b + self.off_b for b in base])
        self.exch_ptrs = _ptr_array([b + self.off_exch for b in base])
        self.big_ptrs = _ptr_array([b + self.off_big for b in base])
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0) if use_multimem else 0
        self.mc_a = mc + self.off_a if mc else None
        self.mc_b = mc + self.off_b if mc else None
        self.part_a = self.buf[self.off_a:self.off_b].view(torch.bfloat16).view(MAX_ROWS, hidden)
        self.part_b = self.buf[self.off_b:self.off_exch].view(torch.bfloat16).view(MAX_ROWS, hidden)
        self.big = self.buf[self.off_big:self.off_big + big_elems * 2].view(torch.bfloat16)
        self.push_dst = [_ptr_array([b + self.off_push + w * push_bytes for b in base]) for w in range(2)]
        self.push_flag = [_ptr_array([b + self.off_pflags + w * 32 for b in base]) for w in range(2)]
        self.push_slots = [self.buf[self.off_push + w * push_bytes:self.off_push + (w + 1) * push_bytes] for w in range(2)]
        self.push_flags_local = [self.buf[self.off_pflags + w * 32:self.off_pflags + (w + 1) * 32] for w in range(2)]
        self.push_count = torch.zeros(2, dtype=torch.int32, device=device)
        self.push_seq = torch.zeros(2, dtype=torch.int32, device=device)
        self.push_counters = torch.zeros(2, MAX_ROWS, dtype=torch.int32, device=device)
        self.push_ll = [_ptr_array([b + self.off_ll + w * ll_bytes for b in base]) for w in range(2)]
        self.push_ll_local = [self.buf[self.off_ll + w * ll_bytes:self.off_ll + (w + 1) * ll_bytes] for w in range(2)]
        self.pull_count = torch.zeros(2, dtype=torch.int32, device=device)
        fl = world * ml * 4
        self.prefill = PrefillPipe(
            rank, world, hidden, pf_rows, device=device,
            slots=self.buf[self.off_pf_slots:self.off_pf_x].view(torch.bfloat16),
            x_bytes=self.buf[self.off_pf_x:self.off_pf_flags],
            rs_flags=self.buf[self.off_pf_flags:self.off_pf_flags + fl], ag_flags=self.buf[self.off_pf_flags + fl:self.off_pf_flags + 2 * fl],
            x_ptrs=[b + self.off_pf_x for b in base], slot_ptrs=[b + self.off_pf_slots for b in base],
            rs_flag_ptrs=[b + self.off_pf_flags for b in base], ag_flag_ptrs=[b + self.off_pf_flags + fl for b in base]) if pf_rows >= 128 else None
        self.counters = torch.zeros(FLAG_SLOTS, dtype=torch.int32, device=device)
        self.scratch = torch.empty(big_elems, dtype=torch.bfloat16, device=device)

    # slots 0..31: part_a rows, 32..63: part_b rows, 64: argmax merge, 65..: big all-reduce CTAs
    def ar_residual_norm(self, which: int, h, m: int, norm_w, *, normed=None, xpack=None, xs=None, group: int = 128,
                         eps: float = 1e-6, pdl: bool = False) -> None:
        ptrs, mc, slot0 = (self.a_ptrs, self.mc_a, 0) if which == 0 else (self.b_ptrs, self.mc_b, 32)
        K.call("owl_ar_residual_norm", ptrs, mc, self.flag_ptrs, K.ptr(self.counters), K.ptr(h), K.ptr(norm_w),
               K.ptr(normed), K.ptr(xpack), K.ptr(xs), m, self.hidden, group, self.rank, self.world, slot0, eps, 1,
               SPIN_LIMIT, int(pdl), K.stream())

    def gemv_push(self, which: int, w, xpack, xs, m: int, *, pdl: bool = False, force_mma: bool = False) -> None:
        """Row-parallel W4 GEMV whose epilogue writes the partial sums into every rank's slot buffer (fused
        GEMV + all-gather of partials over NVLink); pair with ``push_residual_norm``."""
        assert w.layout == "slice"
        K.call("owl_w4a16_skinny_push", K.ptr(w.records), K.ptr(xpack), K.ptr(xs), self.push_dst[which], self.push_flag[which],
               K.ptr(self.push_count[which:]), K.ptr(self.push_seq[which:]), m, w.n, w.k, self.hidden, w.group, self.rank,
               self.world, MAX_ROWS, int(force_mma), int(pdl), K.stream())

    def push_residual_norm(self, which: int, h, m: int, norm_w, *, normed=None, xpack=None, xs=None, group: int = 128,
                           eps: float = 1e-6, pdl: bool = False, fma: bool = False) -> None:
        """Consumer of ``gemv_push`` / ``fma_push``: waits until every rank's flag reached the sequence number the LOCAL
        producer of this call site published last (one number series per call site, whichever producer or consumer kernel
        a step uses), then residual + norm. ``fma``: the producer was ``fma_push`` (one row; the slots are the 8-byte words
        [rank][k part] of that exchange, which carry their own number, and this kernel advances the call site's word)."""
        K.call("owl_push_residual_norm", K.ptr(self.push_slots[which]), K.ptr(self.push_flags_local[which]),
               K.ptr(self.push_counters[which]), K.ptr(h), K.ptr(norm_w), K.ptr(normed), K.ptr(xpack), K.ptr(xs), m,
               self.hidden, group, self.world, MAX_ROWS, eps, 1, SPIN_LIMIT,
               K.ptr(self.push_seq[which:]), self.kparts if fma else 1, K.ptr(self.push_ll_local[which]) if fma else None,
               int(pdl), K.stream())

    # -- one-token projections on the FMA arm with the collective inside (csrc/gemv_fma.cu) ------------------------------
    def fma_push(self, which: int, w, x, *, pdl: bool = False, groups_per_cta: int = 0) -> None:
        """Row-parallel projection of one token: the partial sums go straight into slot [rank] of every rank's word buffer,
        each 8-byte word carrying two sums and the number of this exchange (no flag, no fence)."""
        assert w.n == self.hidden
        K.call("owl_w4_fma_tp", K.ptr(w.records), K.ptr(x), None, None, w.n, w.k, 0, 0.0, 1, 1, self.push_ll[which],
               K.ptr(self.push_seq[which:]), None, None, None, None, None, 0, self.rank, self.world, self.kparts, SPIN_LIMIT,
               groups_per_cta, int(pdl), K.stream())

    def fma_pull(self, which: int, w, h_in, h_out, norm_w, out, *, epi: int = 0, eps: float = 1e-6, ab_w=None, ab_out=None,
                 ab_rows: int = 0, pdl: bool = False, groups_per_cta: int = 0) -> None:
        """Column-parallel projection of one token that first completes the all-reduce of call site ``which``:
        ``h_out = h_in + sum of the ranks' slots`` (stored by one CTA), ``out = epilogue(W . rmsnorm(h_out))``."""
        assert w.k == self.hidden
        K.call("owl_w4_fma_tp", K.ptr(w.records), K.ptr(h_in), K.ptr(norm_w), K.ptr(out), w.n, w.k, epi, eps, 1, 0, None,
               K.ptr(self.push_seq[which:]), K.ptr(self.push_ll_local[which]), K.ptr(self.pull_count[which:]),
               K.ptr(h_out), K.ptr(ab_w), K.ptr(ab_out), ab_rows, self.rank, self.world, self.kparts, SPIN_LIMIT,
               groups_per_cta, int(pdl), K.stream())

    def partial(self, which: int) -> torch.Tensor:
        return self.part_a if which == 0 else self.part_b

    def argmax_merge(self, local_val, local_idx, out_idx, rows: int, pdl: bool = False) -> None:
        K.call("owl_argmax_merge", self.exch_ptrs, self.flag_ptrs, K.ptr(self.counters), K.ptr(local_val),
               K.ptr(local_idx), K.ptr(out_idx), rows, self.rank, self.world, 64, SPIN_LIMIT, int(pdl), K.stream())

    def can_reduce(self, y: torch.Tensor) -> bool:
        return y.dtype == torch.bfloat16 and y.is_contiguous() and y.numel() <= self.big_elems and y.numel() % 8 == 0

    def allreduce_(self, y: torch.Tensor) -> None:
        """In-place sum over ranks of a contiguous bf16 tensor (copied through the symmetric area)."""
        n = y.numel()
        self.big[:n].copy_(y.view(-1))
        K.call("owl_ar_inplace", self.big_ptrs, self.flag_ptrs, K.ptr(self.counters), K.ptr(self.scratch), n, self.rank,
               self.world, 65, 48, SPIN_LIMIT, K.stream())
        y.view(-1).copy_(self.big[:n])

    @staticmethod
    def status() -> int:
        f = K.fn("owl_comm_status")
        f.argtypes = []
        return f()


# the world-of-one form shares the launch wrappers
LocalSplit.fma_push = SymmetricWorkspace.fma_push
LocalSplit.fma_pull = SymmetricWorkspace.fma_pull
LocalSplit.push_residual_norm = SymmetricWorkspace.push_residual_norm
