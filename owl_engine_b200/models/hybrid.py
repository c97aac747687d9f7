"""GPU runner of the hybrid model: device weights in kernel layouts, the state pool (paged fp8
KV + GDN rows), the decode / verify step as a capturable kernel sequence, chunked prefill.

One ``HybridRunner`` lives in each rank's process. With ``spec.tp_world > 1`` the row-parallel
projections (o_proj / out_proj / down_proj) hand their partial sums to ``comm`` (see
``owl_engine_b200.parallel``), which reduces them across ranks fused with the residual add.

Reference counterpart: the model backbone (``crates/models/src/model.rs``), decoder layer
(``layers/decoder.rs:80-100``), executor device halves (``crates/engine/src/exec/phases.rs``) and
the state pool (``crates/engine/src/mem/state.rs``). The reference's TensorOps interpreter is
not reproduced: the step is a fixed launch sequence recorded into a CUDA graph.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch

from ..ops import kernels as K
from ..ops import quant as Q
from ..ops import reference as R
from .spec import ModelSpec, mrope_section_map

PAGE = 16


# ---------------------------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------------------------
@dataclass
class LayerWeights:
    kind: str
    ln1: torch.Tensor
    ln2: torch.Tensor
    gate_up: object
    down: object
    # gdn
    qkvz: object = None
    ab: object = None               # DenseSkinny [pad16(2*nv), H]: in_proj_a rows then in_proj_b rows
    ab_dense: torch.Tensor = None   # same rows as plain bf16 [pad16(2*nv), H] for the prefill GEMM
    conv_w: torch.Tensor = None
    a_log: torch.Tensor = None
    dt_bias: torch.Tensor = None
    gamma: torch.Tensor = None
    out_proj: object = None
    # full
    qkv: object = None
    q_norm: torch.Tensor = None
    k_norm: torch.Tensor = None
    o_proj: object = None


@dataclass
class HybridWeights:
    spec: ModelSpec
    embed: torch.Tensor
    final_norm: torch.Tensor
    lm_head: object                  # DenseSkinny (bf16 or int8 records), [V or vocab shard, H]
    layers: list
    group: int
    vocab_offset: int = 0

    @property
    def layout(self) -> str:
        """Record layout of the W4 weights: "slice" (legacy streaming kernels) or "block" (tcgen05 streaming kernel)."""
        return self.layers[0].gate_up.layout if self.layers else "slice"

    def nbytes(self) -> int:
        n = self.embed.numel() * 2 + self.lm_head.nbytes
        for l in self.layers:
            for w in (l.gate_up, l.down, l.qkvz, l.out_proj, l.qkv, l.o_proj, l.ab):
                if w is not None:
                    n += w.nbytes
        return n

    def streamed_bytes(self) -> int:
        """Bytes one decode step must read from HBM (everything but the embedding table)."""
        return self.nbytes() - self.embed.numel() * 2


def _pad16_rows(w: torch.Tensor) -> torch.Tensor:
    n = w.shape[0]
    if n % 16 == 0:
        return w
    return torch.cat([w, torch.zeros(16 - n % 16, w.shape[1], dtype=w.dtype, device=w.device)])


def weights_from_dense(spec: ModelSpec, dense: dict, device, group: int = 128, lm_head_int8: bool = False, layout: str = "slice",
                       vocab_split: bool = False, quant: str = "w4a16"):
    """Build device weights from HF-named dense tensors (full, unsharded model; ``spec`` may be
    a TP shard, in which case rows / columns are cut with ``parallel.plan``). Returns
    ``(HybridWeights, dense_equiv)`` where ``dense_equiv`` holds the dequantised weights under
    the same HF names, i.e. exactly what the kernels compute with (for the CPU oracle)."""
    from ..parallel.plan import shard_dense_for_rank

    dense = shard_dense_for_rank(spec, dense)
    equiv = dict(dense)

    def w4(name_or_tensor, names=None):
        w = name_or_tensor.float()
        if quant == "nvfp4":
            from ..formats import nvfp4

            q4 = nvfp4.quantize(w)
            deq = nvfp4.dequantize(q4)
            off = 0
            for nm, rows in names or []:
                equiv[nm] = deq[off:off + rows]
                off += rows
            return Q.NvFp4Linear(q4.codes.to(device), q4.scales.to(device), q4.global_scale, w.shape[0], w.shape[1], group)
        c = Q.quantize_w4(w, group)
        if names:
            deq = c.dequant()
            off = 0
            for nm, rows in names:
                equiv[nm] = deq[off:off + rows]
                off += rows
        return Q.pack_skinny(c, layout).to(device)

    bf = lambda t: t.to(torch.bfloat16).to(device)
    f32 = lambda t: t.float().to(device)
    layers = []
    for i in range(spec.n_layers):
        p = f"model.layers.{i}."
        m = p + "mlp."
        gu = Q.interleave_gate_up(dense[m + "gate_proj.weight"].float(), dense[m + "up_proj.weight"].float())
        if quant == "nvfp4":
            from ..formats import nvfp4

            qgu = nvfp4.quantize(gu)
            gu_dev = Q.NvFp4Linear(qgu.codes.to(device), qgu.scales.to(device), qgu.global_scale, gu.shape[0], gu.shape[1], group)
            gu_deq = nvfp4.dequantize(qgu)
        else:
            cgu = Q.quantize_w4(gu, group)
            gu_dev, gu_deq = Q.pack_skinny(cgu, layout).to(device), cgu.dequant()
        ge, ue = Q.deinterleave_gate_up(gu_deq.t())
        equiv[m + "gate_proj.weight"], equiv[m + "up_proj.weight"] = ge.t().contiguous(), ue.t().contiguous()
        lw = LayerWeights(kind="full" if spec.is_full(i) else "gdn", ln1=bf(dense[p + "input_layernorm.weight"]),
                          ln2=bf(dense[p + "post_attention_layernorm.weight"]), gate_up=gu_dev,
                          down=w4(dense[m + "down_proj.weight"], [(m + "down_proj.weight", spec.hidden)]))
        if lw.kind == "gdn":
            a = p + "linear_attn."
            qkvz = torch.cat([dense[a + "in_proj_qkv.weight"], dense[a + "in_proj_z.weight"]]).float()
            lw.qkvz = w4(qkvz, [(a + "in_proj_qkv.weight", spec.conv_dim), (a + "in_proj_z.weight", spec.value_dim)])
            ab = torch.cat([dense[a + "in_proj_a.weight"], dense[a + "in_proj_b.weight"]]).to(torch.bfloat16)
            equiv[a + "in_proj_a.weight"], equiv[a + "in_proj_b.weight"] = ab[:spec.nv].float(), ab[spec.nv:].float()
            lw.ab_dense = _pad16_rows(ab).to(device)
            lw.ab = Q.dense_skinny(lw.ab_dense, device)
            lw.conv_w = f32(dense[a + "conv1d.weight"].reshape(spec.conv_dim, spec.conv_k))
            lw.a_log, lw.dt_bias = f32(dense[a + "A_log"]), f32(dense[a + "dt_bias"])
            lw.gamma = f32(dense[a + "norm.weight"])
            lw.out_proj = w4(dense[a + "out_proj.weight"], [(a + "out_proj.weight", spec.hidden)])
        else:
            a = p + "self_attn."
            qkv = torch.cat([dense[a + "q_proj.weight"], dense[a + "k_proj.weight"], dense[a + "v_proj.weight"]]).float()
            lw.qkv = w4(qkv, [(a + "q_proj.weight", 2 * spec.hq * spec.hd), (a + "k_proj.weight", spec.hkv * spec.hd),
                              (a + "v_proj.weight", spec.hkv * spec.hd)])
            lw.q_norm, lw.k_norm = bf(dense[a + "q_norm.weight"]), bf(dense[a + "k_norm.weight"])
            lw.o_proj = w4(dense[a + "o_proj.weight"], [(a + "o_proj.weight", spec.hidden)])
        for nm in ("input_layernorm.weight", "post_attention_layernorm.weight"):
            equiv[p + nm] = dense[p + nm].to(torch.bfloat16).float()
        layers.append(lw)
    emb = dense["model.embed_tokens.weight"].to(torch.bfloat16)
    head = emb if spec.tied else dense["lm_head.weight"].to(torch.bfloat16)
    equiv["model.embed_tokens.weight"] = emb.float()
    equiv["model.norm.weight"] = dense["model.norm.weight"].to(torch.bfloat16).float()
    hw = HybridWeights(spec=spec, embed=emb.to(device), final_norm=bf(dense["model.norm.weight"]), lm_head=None,
                       layers=layers, group=group)
    if vocab_split and spec.tp_world > 1 and spec.vocab % (16 * spec.tp_world) == 0:
        vrows = spec.vocab // spec.tp_world
        hw.vocab_offset = spec.tp_rank * vrows
        head_dev = head[hw.vocab_offset:hw.vocab_offset + vrows].contiguous()
    else:
        head_dev = head
    hw.lm_head = Q.dense_skinny(head_dev.to(device), device, int8=lm_head_int8)
    if lm_head_int8:
        q8, s8 = Q.quantize_w8_rows(head.float())
        equiv["lm_head.weight"] = q8.float() * s8[:, None]
    else:
        equiv["lm_head.weight"] = head.float()
    return hw, equiv


def random_weights(spec: ModelSpec, device, group: int = 128, seed: int = 0, lm_head_int8: bool = False, layout: str = "slice",
                   std: float = 0.02, vocab_split: bool = True, quant: str = "w4a16") -> HybridWeights:
    """Random-init weights generated directly in the device layouts (benchmarks: no dense copy)."""
    if quant == "nvfp4":
        class _Q4:                      # same call shape as Q.random_skinny, NVFP4 storage
            @staticmethod
            def random_skinny(n, k, group, device, std, seed, layout):
                return Q.random_nvfp4(n, k, device, std, seed, group)
        return _random_weights(spec, device, group, seed, lm_head_int8, "nvfp4", std, vocab_split, _Q4)
    return _random_weights(spec, device, group, seed, lm_head_int8, layout, std, vocab_split, Q)


def _random_weights(spec, device, group, seed, lm_head_int8, layout, std, vocab_split, QW) -> HybridWeights:
    gen = torch.Generator(device=device).manual_seed(seed)
    rnd = lambda *s: (torch.randn(*s, device=device, generator=gen) * std)
    H = spec.hidden
    layers = []
    sd = seed * 100003
    for i in range(spec.n_layers):
        sd += 17
        lw = LayerWeights(kind="full" if spec.is_full(i) else "gdn", ln1=rnd(H).to(torch.bfloat16),
                          ln2=rnd(H).to(torch.bfloat16),
                          gate_up=QW.random_skinny(2 * spec.inter, H, group, device, std, sd + 1, layout),
                          down=QW.random_skinny(H, spec.inter, group, device, std, sd + 2, layout))
        if lw.kind == "gdn":
            lw.qkvz = QW.random_skinny(spec.conv_dim + spec.value_dim, H, group, device, std, sd + 3, layout)
            lw.ab_dense = _pad16_rows(rnd(2 * spec.nv, H).to(torch.bfloat16))
            lw.ab = Q.dense_skinny(lw.ab_dense, device)
            lw.conv_w = (torch.randn(spec.conv_dim, spec.conv_k, device=device, generator=gen) * 0.2)
            lw.a_log = torch.log(torch.empty(spec.nv, device=device).uniform_(1.0, 16.0, generator=gen))
            lw.dt_bias = torch.ones(spec.nv, device=device)
            lw.gamma = torch.ones(spec.vd, device=device)
            lw.out_proj = QW.random_skinny(H, spec.value_dim, group, device, std, sd + 4, layout)
        else:
            lw.qkv = QW.random_skinny(2 * spec.hq * spec.hd + 2 * spec.hkv * spec.hd, H, group, device, std, sd + 5, layout)
            lw.q_norm, lw.k_norm = rnd(spec.hd).to(torch.bfloat16), rnd(spec.hd).to(torch.bfloat16)
            lw.o_proj = QW.random_skinny(H, spec.hq * spec.hd, group, device, std, sd + 6, layout)
        layers.append(lw)
    emb = rnd(spec.vocab, H).to(torch.bfloat16)
    hw = HybridWeights(spec=spec, embed=emb, final_norm=torch.zeros(H, dtype=torch.bfloat16, device=device),
                       lm_head=None, layers=layers, group=group)
    # vocab-split head: each TP rank holds V / world rows and the winners are merged across ranks
    vrows = spec.vocab
    if vocab_split and spec.tp_world > 1 and spec.vocab % (16 * spec.tp_world) == 0:
        vrows = spec.vocab // spec.tp_world
        hw.vocab_offset = spec.tp_rank * vrows
    if lm_head_int8:
        q8 = torch.randint(-127, 128, (vrows, H), device=device, dtype=torch.int8, generator=gen)
        hw.lm_head = Q.DenseSkinny(Q.pack_dense_int8(q8), vrows, H, "int8", torch.full((vrows,), std / 40.0, device=device))
    else:
        head = emb if spec.tied else rnd(spec.vocab, H).to(torch.bfloat16)
        hw.lm_head = Q.dense_skinny(head[hw.vocab_offset:hw.vocab_offset + vrows].contiguous(), device)
    return hw


# ---------------------------------------------------------------------------------------------
# state pool
# ---------------------------------------------------------------------------------------------
class StatePool:
    """Device state: paged fp8 KV (``[layer][page][16][hkv][hd]`` e4m3, zero-initialised so that
    masked slots never hold NaN encodings), GDN convolution history and recurrent state rows."""

    def __init__(self, spec: ModelSpec, device, n_pages: int, n_slots: int, ledger=None, kv_dtype: str = "fp8"):
        """``kv_dtype`` "fp8": e4m3 values (no scales); "int8": int8 values with one fp32 scale per (token, kv head) in
        ``k_scale`` / ``v_scale`` (the reference's int8 KV family, crates/kernels/cu/attn int8 kernels)."""
        assert kv_dtype in ("fp8", "int8", "bf16", "f16")
        self.spec, self.device, self.n_pages, self.n_slots, self.kv_dtype = spec, device, n_pages, n_slots, kv_dtype
        nf, ng = spec.n_full, spec.n_gdn
        # "bf16" / "f16": a 16-bit pool of fp16 words that hold the bf16-rounded K / V values (exact inside the fp16 range,
        # clamped outside), which the attention kernel feeds to the fp16 MMA as stored; the kernels tell the pools apart by dtype
        pdt = torch.float16 if kv_dtype in ("bf16", "f16") else torch.uint8
        self.k_pool = torch.zeros(nf, n_pages, PAGE, spec.hkv, spec.hd, dtype=pdt, device=device)
        self.v_pool = torch.zeros(nf, n_pages, PAGE, spec.hkv, spec.hd, dtype=pdt, device=device)
        self.k_scale = self.v_scale = None
        if kv_dtype == "int8":
            self.k_scale = torch.zeros(nf, n_pages, PAGE, spec.hkv, dtype=torch.float32, device=device)
            self.v_scale = torch.zeros(nf, n_pages, PAGE, spec.hkv, dtype=torch.float32, device=device)
        self.conv_state = torch.zeros(ng, n_slots, spec.conv_dim, spec.conv_k - 1, dtype=torch.float32, device=device)
        self.rec_state = torch.zeros(ng, n_slots, spec.nv, spec.kd, spec.vd, dtype=torch.float32, device=device)
        if ledger is not None:
            ledger.record("kv_pool", "pool", self.k_pool.numel() * self.k_pool.element_size() * 2)
            ledger.record("gdn_state", "pool", self.conv_state.numel() * 4 + self.rec_state.numel() * 4)

    @staticmethod
    def bytes_per_page(spec: ModelSpec, kv_dtype: str = "fp8") -> int:
        return spec.n_full * 2 * PAGE * spec.hkv * spec.hd * (2 if kv_dtype in ("bf16", "f16") else 1)

    @staticmethod
    def bytes_per_slot(spec: ModelSpec) -> int:
        return spec.gdn_state_bytes()

    def scales(self, layer: int):
        """(k_scale, v_scale) of one full-attention layer for the int8 pool, None for the e4m3 pool."""
        return None if self.k_scale is None else (self.k_scale[layer], self.v_scale[layer])

    def reset_slot(self, slot: int) -> None:
        self.conv_state[:, slot].zero_()
        self.rec_state[:, slot].zero_()

    def copy_slot(self, src: int, dst: int) -> None:
        """Snapshot / restore of a GDN row (speculative rollback, prefix-boundary snapshots)."""
        self.conv_state[:, dst].copy_(self.conv_state[:, src])
        self.rec_state[:, dst].copy_(self.rec_state[:, src])


# ---------------------------------------------------------------------------------------------
# runner
# ---------------------------------------------------------------------------------------------
class StepLayout:
    """Offsets (int32 elements) of the packed per-step input buffer for B sequences x T rows."""

    def __init__(self, b: int, t: int):
        m = b * t
        self.b, self.t, self.m = b, t, m
        self.ids, self.pos3, self.kv_slot = 0, m, 4 * m
        self.ctx, self.gslot, self.bt_row = 5 * m, 5 * m + b, 5 * m + 2 * b
        self.size = 5 * m + 3 * b


class _CapturedStep:
    """A captured CUDA graph with its manifest: the native launches the capture recorded, and how often it was replayed.
    A replay is invisible to the host-side launch ring (the graph launches its kernels itself), so this is what attributes
    device work to entries when steps run from graphs."""

    def __init__(self, graph, launches: list):
        self.graph, self.launches, self.replays = graph, launches, 0

    def replay(self) -> None:
        self.replays += 1
        self.graph.replay()


class _EagerStep:
    """Stands in for a captured graph when steps run eagerly: ``replay()`` launches the kernel sequence directly."""

    def __init__(self, fn):
        self.fn = fn

    def replay(self) -> None:
        self.fn()


class HybridRunner:
    MAX_ROWS = 32

    def __init__(self, spec: ModelSpec, weights: HybridWeights, pool: StatePool, *, max_seqs: int = 32,
                 max_blocks: int = 1024, prefill_chunk: int = 2048, comm=None, pdl: bool = True,
                 attn_splits: int = 0, prefill_gemm: str = "tc"):
        self.spec, self.w, self.pool, self.comm = spec, weights, pool, comm
        self.device = pool.device
        self.max_seqs, self.max_blocks, self.prefill_chunk = max_seqs, max_blocks, prefill_chunk
        self.pdl = pdl
        # row projection + residual + next norm in one launch (128 fewer launches per 27B step). Off by default: measured
        # 195.9 against 212.4 tok/s on one B200; the one CTA that normalises after the last arrival sits on the critical
        # path, while the separate norm kernel's launch is hidden by programmatic dependent launch
        self.fuse_norm = os.environ.get("OWL_FUSE_NORM", "0") == "1"
        self._norm_count = None
        self._attn_ws = None         # scratch of the GEMM-form prefill attention
        # decode activations: 15-bit fixed point (exact for bf16 inputs up to rounding at 2^-14 of the group maximum), or 8
        # bits per group (the W4A8 decode arm: half the integer products per weight byte)
        self.act_bits = int(os.environ.get("OWL_ACT_BITS", "15"))
        # L2 prefetch of the next projection's weights on a side branch of the step graph (MB per projection, 0 = off) and
        # where the branch forks: "before" the current projection (concurrent with it) or "after" it (in the gap that follows)
        self.l2_prefetch_mb = float(os.environ.get("OWL_L2_PREFETCH_MB", "0"))
        self.l2_prefetch_at = os.environ.get("OWL_L2_PREFETCH_AT", "after")
        self._pf_rec = None          # warm-up pass of a capture: the weight tensors in launch order
        self._pf_play = None         # capture pass: (schedule, side stream, capture stream)
        self._pf_i = 0
        self.prefill_gemm = prefill_gemm
        self.G = weights.group
        dev, H, M = self.device, spec.hidden, self.MAX_ROWS
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
        self.tiles = weights.layout == "block"      # decode GEMVs on the tcgen05 streaming kernel
        self.tc_ws = K.StreamTcWorkspace(dev, max_n=max(2 * spec.inter, spec.conv_dim + spec.value_dim, 4096)) if self.tiles else None
        # ActPack: 2 bytes per k in the row layout; the tile layout needs a little more (scale pairs ride along)
        f16 = lambda m_, k_: torch.zeros(max(m_ * 2 * k_, ((m_ + 7) // 8) * K.act_tile_bytes(k_, weights.group)),
                                         dtype=torch.uint8, device=dev)
        f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
        G = self.G
        self.block_table = torch.zeros(max_seqs, max_blocks, dtype=torch.int32, device=dev)
        self.inp = torch.zeros(8 * M + 3 * max_seqs, dtype=torch.int32, device=dev)
        self.h = bf(M, H)
        self.xn = bf(M, H)
        self.xp_h, self.xs_h = f16(M, H), f32(M, H // G, 2)
        self.partial = bf(M, H)
        qkvz_n = spec.conv_dim + spec.value_dim
        self.qkvz_out = bf(M, qkvz_n)
        self.ldab = ((2 * spec.nv + 15) // 16) * 16
        self.ab_out = bf(M, self.ldab)
        self.xp_v, self.xs_v = f16(M, spec.value_dim), f32(M, spec.value_dim // G, 2)
        self.qkv_n = 2 * spec.hq * spec.hd + 2 * spec.hkv * spec.hd
        self.qkv_out = bf(M, self.qkv_n)
        self.q_rope = bf(M, spec.hq, spec.hd)
        self.attn_splits = attn_splits
        self.use_graphs = True          # False: every step, fold and verify launches its kernels eagerly (debugging)
        self.max_splits = 64
        self.part_o = f32(M * spec.hq * self.max_splits * spec.hd)
        self.part_ml = f32(M * spec.hq * self.max_splits * 2)
        self.xp_a, self.xs_a = f16(M, spec.hq * spec.hd), f32(M, spec.hq * spec.hd // G, 2)
        self.act = bf(M, spec.inter)
        self.side = torch.cuda.Stream(device=dev)   # forked branch for the small a/b projection
        self.xp_i, self.xs_i = f16(M, spec.inter), f32(M, spec.inter // G, 2)
        self.vocab_local = weights.lm_head.n
        self.logits = bf(M, self.vocab_local)
        self.am_parts = 64
        self.am_val, self.am_idx = f32(M * self.am_parts), torch.zeros(M * self.am_parts, dtype=torch.int32, device=dev)
        self.out_tok = torch.zeros(M, dtype=torch.int32, device=dev)
        self.loc_val, self.loc_idx = f32(M), torch.zeros(M, dtype=torch.int32, device=dev)
        self.vocab_split = self.vocab_local != spec.vocab
        self.inv_freq = R.rope_inv_freq(spec.rotary_dim, spec.rope_theta).to(dev)
        yarn_scale = 1.0
        if getattr(spec, "rope_yarn", None):
            y_factor, y_orig, y_fast, y_slow, y_att = spec.rope_yarn
            inv, yarn_scale = R.rope_yarn(spec.rotary_dim, spec.rope_theta, y_factor, y_orig or spec.max_position, y_fast, y_slow, y_att)
            self.inv_freq = inv.to(dev)
        self.section = torch.tensor(mrope_section_map(spec), dtype=torch.uint8, device=dev)
        self.rope_scale = yarn_scale
        self.scale = 1.0 / math.sqrt(spec.hd)
        self.graphs: dict = {}
        self._pf = None   # lazily allocated prefill workspace
        self.taps: dict | None = None   # layer -> bf16 [M,H] buffers filled during decode/prefill for draft heads
        self._x16 = self._gu16 = None   # bf16 staging of the NVFP4 GEMV arm (allocated on first use)
        self._x16h = self._y16 = self._xq8 = None   # fp16 / e4m3 activations and bf16 outputs of the batched dense-GEMM arm
        self.tap_sink = None            # callable(pos0, t, {layer: [t, H]}) called after every prefill chunk when taps are on
        self.pre_hook = None            # callable(m): rewrites self.h after the embedding (draft heads mix in the target's hidden)
        self.uniform_rows = False       # per-row arithmetic independent of the number of rows in the step (speculative
                                        # verify must reproduce plain decoding bit for bit): one GEMV arm for 1..8 rows,
                                        # KV splits aligned to positions instead of to the row's length
        self.pf_pipe = None             # explicit prefill pipe (parallel/symm.PrefillPipe); default: the communicator's
        self.sp_prefill = True          # tensor-parallel prefill through the GEMM-fused reduce-scatter / all-gather path
        self.gdn_save = None            # (qkvz [n_gdn, M, nq], ab [n_gdn, M, ldab]): GDN inputs of the last step, kept for fold()
        # one-token steps: "fma" = the half-precision FMA projection with the norm / residual / activation glue folded in
        # (5 launches per GDN layer, 7 per attention layer); "dp4a" = the integer arm with separate norm and pack launches
        self.decode_gemv = "fma"
        self.mix = bf(M, max(spec.value_dim, spec.hq * spec.hd))   # mixer output (GDN / attention) of the fused one-token path
        self.h_alt = bf(M, H)           # second residual-stream buffer of the one-token path with split projections
        # one GPU: k parts of the projections into the hidden size (0 = off). Off by default: measured 161 against 234 tok/s on
        # the 27B step (a part of a tile is one to four records per warp, so the per-unit reduction dominates)
        self.ksplit = int(os.environ.get("OWL_FMA_KSPLIT", "0"))
        self._local_split = None

    # -- step inputs -------------------------------------------------------------------------
    def views(self, lay: StepLayout):
        i = self.inp
        return dict(ids=i[lay.ids:lay.ids + lay.m], pos3=i[lay.pos3:lay.pos3 + 3 * lay.m],
                    kv_slot=i[lay.kv_slot:lay.kv_slot + lay.m], ctx=i[lay.ctx:lay.ctx + lay.b],
                    gslot=i[lay.gslot:lay.gslot + lay.b], bt_row=i[lay.bt_row:lay.bt_row + lay.b])

    # -- building blocks ---------------------------------------------------------------------
    def _grp(self) -> int:
        """``group`` argument for the ActPack producers: the tile layout when the tcgen05 streaming kernel consumes it."""
        g = (self.G | K.ACT_TILES) if self.tiles else self.G
        return g | K.ACT_A8 if self.act_bits == 8 else g

    def _pf_hook(self, w, after: bool) -> None:
        """Weight-stream bookkeeping around a projection: the warm-up pass of a capture records the weight tensors in launch
        order; the capture pass forks a side branch that prefetches the front of the NEXT projection's weights into L2 (the
        last projection of a step prefetches the first one of the next step)."""
        if self._pf_rec is not None:
            if not after:
                self._pf_rec.append(getattr(w, "records", None))
            return
        if self._pf_play is None:
            return
        if not after:
            self._pf_cur, self._pf_i = self._pf_i, self._pf_i + 1
        if after != (self.l2_prefetch_at == "after"):
            return
        sched, side, cur = self._pf_play
        nxt = sched[(self._pf_cur + 1) % len(sched)]
        if nxt is None:
            return
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            K.l2_prefetch(nxt, int(self.l2_prefetch_mb * (1 << 20)))

    def _gemv(self, w, xp, xs, out, m: int, *, residual=None, epi: int = K.EPI_STORE, ldo=None, pdl: bool = False) -> None:
        """out[m] = W x on the weight-streaming kernel that matches the weight's record layout."""
        self._pf_hook(w, False)
        self._gemv_inner(w, xp, xs, out, m, residual=residual, epi=epi, ldo=ldo, pdl=pdl)
        self._pf_hook(w, True)

    def _gemv_inner(self, w, xp, xs, out, m: int, *, residual=None, epi: int = K.EPI_STORE, ldo=None, pdl: bool = False) -> None:
        if w.layout == "nvfp4":
            self._gemv_nvfp4(w, xp, xs, out, m, residual, epi, ldo)
            return
        # (not under uniform_rows: a speculating engine needs the same arithmetic for every row count, and the dense product
        # rounds differently from the integer arm that plain steps of a few rows use)
        if m >= self.BATCH_GEMM_FROM and self.prefill_gemm in ("tcr", "tc8r") and w.layout == "slice" and w.k % 128 == 0 \
                and epi in (K.EPI_STORE, K.EPI_RESIDUAL, K.EPI_SILU_MUL) and not self.uniform_rows:
            self._gemv_dense16(w, xp, xs, out, m, residual, epi, ldo)
            return
        if w.layout != "block":
            K.w4a16_skinny(w, xp, xs, out, m, residual=residual, epi=epi, ldo=ldo, pdl=pdl,
                           force_mma=self.uniform_rows and m == 1,
                           a8=self.act_bits == 8 and epi in (K.EPI_STORE, K.EPI_RESIDUAL, K.EPI_SILU_MUL, K.EPI_F32))
            return
        tb = K.act_tile_bytes(w.k, w.group)
        for r0 in range(0, m, 8):       # 8 tokens per pass (one activation tile buffer each)
            rows = min(8, m - r0)
            K.w4a16_stream_tc(w, xp.view(-1)[(r0 // 8) * tb:], out[r0:], rows, self.tc_ws,
                              residual=None if residual is None else residual[r0:], epi=epi,
                              ldo=ldo if ldo is not None else out.shape[-1], pdl=pdl)

    BATCH_GEMM_FROM = 24   # rows from which a batched step multiplies the resident dense weight copy on the tcgen05 GEMM

    def _gemv_dense16(self, w, xp, xs, out, m: int, residual, epi: int, ldo) -> None:
        """Wide batched steps (16+ rows) with a resident dense copy of the weights (``prefill_gemm = "tcr"``: fp16, 4x the
        int4 bytes; ``"tc8r"``: e4m3 rows, 2x, activations quantised per token): the integer weight-streaming arms run on
        warp-level MMA and grow linearly with the row count from 8 rows on, while the persistent tcgen05 GEMM streams the
        dense matrix once for all rows."""
        from ..ops import gemm_tc, linear

        sp = self.spec
        if self._x16h is None:
            kmax = max(sp.hidden, sp.inter, sp.value_dim, sp.hq * sp.hd)
            nmax = max(2 * sp.inter, sp.conv_dim + sp.value_dim, self.qkv_n, sp.hidden)
            self._x16h = torch.empty(self.MAX_ROWS, kmax, dtype=torch.float16, device=self.device)
            self._y16 = torch.empty(self.MAX_ROWS * nmax, dtype=torch.bfloat16, device=self.device)
        x = self._x16h[:m, :w.k]
        K.act_unpack(xp, xs, x, m, w.k, self.G)
        direct = epi == K.EPI_STORE
        ld = (ldo if ldo is not None else out.shape[-1]) if direct else w.n
        y = (out.view(-1)[:m * ld] if direct and out.is_contiguous() and (ldo is None or ldo == out.shape[-1]) else self._y16[:m * ld]).view(m, ld)
        if self.prefill_gemm == "tc8r":
            wq, sw = linear.w4_e4m3(w, self.device)
            if self._xq8 is None:
                self._xq8 = (torch.empty(self.MAX_ROWS * self._x16h.shape[1], dtype=torch.uint8, device=self.device),
                             torch.empty(self.MAX_ROWS, dtype=torch.float32, device=self.device))
            xq, sx = gemm_tc.quant_e4m3_rows(x, self._xq8[0][:m * w.k].view(m, w.k), self._xq8[1][:m])
            gemm_tc.e4m3_gemm(xq, sx, wq, sw, y)
        else:
            gemm_tc.f16_gemm(x, linear.w4_dense(w, torch.float16, self.device, resident=True), y, force_persist=True)
        if epi == K.EPI_RESIDUAL:
            K.add_rows(residual, y, out, m, w.n)
        elif epi == K.EPI_SILU_MUL:
            K.silu_mul(y, m, w.n // 2, out=out, pdl=False)
        elif y.data_ptr() != out.data_ptr():
            out[:m, :w.n].copy_(y[:, :w.n])

    def _gemv_nvfp4(self, w, xp, xs, out, m: int, residual, epi: int, ldo) -> None:
        """NVFP4 weights as stored in the checkpoint (e2m1 codes + e4m3 block scales): the activations come back from
        ActPack to bf16 (15 bits of fixed point: nothing is lost on the way to bf16), the streaming dequant GEMV runs 8 rows
        per pass, and the gate / up activation is the stand-alone kernel."""
        sp = self.spec
        if self._x16 is None:
            kmax = max(sp.hidden, sp.inter, sp.value_dim, sp.hq * sp.hd)
            self._x16 = torch.empty(self.MAX_ROWS, kmax, dtype=torch.bfloat16, device=self.device)
            self._gu16 = torch.empty(self.MAX_ROWS, 2 * sp.inter, dtype=torch.bfloat16, device=self.device)
        x = self._x16[:, :w.k]
        K.act_unpack(xp, xs, x, m, w.k, self.G)
        dst = self._gu16 if epi == K.EPI_SILU_MUL else (out if ldo is None else out.view(-1)[:out.shape[0] * ldo].view(out.shape[0], ldo))
        for r0 in range(0, m, 8):
            rows = min(8, m - r0)
            K.nvfp4_linear_gemv(w, x[r0:], dst[r0:], rows, residual=residual[r0:] if epi == K.EPI_RESIDUAL else None)
        if epi == K.EPI_SILU_MUL:
            K.silu_mul(self._gu16, m, w.n // 2, out=out, pdl=False)
        elif epi not in (K.EPI_STORE, K.EPI_RESIDUAL):
            raise ValueError(f"NVFP4 arm: epilogue {epi} is not built")

    def _norm(self, m: int, w, *, want_xn: bool, want_pack: bool = True) -> None:
        sp = self.spec
        K.rmsnorm_pack(self.h, w, normed=self.xn if want_xn else None, xpack=self.xp_h if want_pack else None,
                       xs=self.xs_h if want_pack else None, m=m, k=sp.hidden, group=self._grp(), eps=sp.eps, pdl=self.pdl)

    def _row_parallel(self, which: int, w, xp, xs, m: int, next_norm, *, want_xn: bool, want_pack: bool = True) -> None:
        """h += W x for a row-parallel projection, then x_next = rmsnorm(h) * (1 + next_norm).

        TP=1: residual fused into the GEMV epilogue, then the norm kernel. TP>1 (fused arm): the
        GEMV writes its partial sums into the symmetric buffer `which` (mixer / MLP alternate) and one
        kernel does all-reduce + residual + norm + pack. TP>1 (nccl arm): library all-reduce."""
        sp = self.spec
        symm = getattr(self.comm, "symm", None) if self.comm is not None else None
        if self.comm is None or sp.tp_world == 1:
            if self.fuse_norm and w.layout == "slice" and w.n == sp.hidden and m < self.BATCH_GEMM_FROM and (want_xn or want_pack):
                # projection + residual + the next block's norm in one launch: the last CTA to finish normalises the rows
                if self._norm_count is None:
                    self._norm_count = torch.zeros(1, dtype=torch.int32, device=self.device)
                K.w4a16_skinny_norm(w, xp, xs, self.h, next_norm, self._norm_count, m, normed=self.xn if want_xn else None,
                                    norm_pack=self.xp_h if want_pack else None, norm_xs=self.xs_h if want_pack else None,
                                    group=self._grp(), eps=sp.eps, pdl=self.pdl, force_mma=self.uniform_rows and m == 1)
                return
            self._gemv(w, xp, xs, self.h, m, residual=self.h, epi=K.EPI_RESIDUAL, pdl=self.pdl)
            self._norm(m, next_norm, want_xn=want_xn, want_pack=want_pack)
        elif symm is not None and getattr(self.comm, "mode", "") == "push" and w.layout == "slice" and w.n == sp.hidden:
            # fused arm: the GEMV's epilogue writes its partial sums into every rank's slots over NVLink while the
            # rest of the matrix is still streaming; the consumer waits for the peers' sequence numbers and reduces
            # local memory only
            symm.gemv_push(which, w, xp, xs, m, pdl=self.pdl, force_mma=self.uniform_rows and m == 1)
            symm.push_residual_norm(which, self.h, m, next_norm, normed=self.xn if want_xn else None,
                                    xpack=self.xp_h if want_pack else None, xs=self.xs_h if want_pack else None,
                                    group=self._grp(), eps=sp.eps, pdl=self.pdl)
        elif symm is not None:
            self._gemv(w, xp, xs, symm.partial(which), m, pdl=self.pdl)
            symm.ar_residual_norm(which, self.h, m, next_norm, normed=self.xn if want_xn else None,
                                  xpack=self.xp_h if want_pack else None, xs=self.xs_h if want_pack else None,
                                  group=self._grp(), eps=sp.eps, pdl=self.pdl)
        else:
            self._gemv(w, xp, xs, self.partial, m, pdl=self.pdl)
            self.comm.allreduce_add_residual(self.partial, self.h, m)
            self._norm(m, next_norm, want_xn=want_xn, want_pack=want_pack)

    def _mlp(self, lw: LayerWeights, m: int, next_norm, *, want_xn: bool, want_pack: bool = True) -> None:
        sp = self.spec
        # silu(gate)*up is written as bf16 and packed by a small kernel: the fused pack epilogue
        # (EPI_SILU_PACK) needs 16 row tiles per CTA, which leaves too few CTAs at this size
        self._gemv(lw.gate_up, self.xp_h, self.xs_h, self.act, m, epi=K.EPI_SILU_MUL, ldo=sp.inter, pdl=self.pdl)
        K.act_pack(self.act, self.xp_i, self.xs_i, m, sp.inter, self._grp(), pdl=self.pdl)
        self._row_parallel(1, lw.down, self.xp_i, self.xs_i, m, next_norm, want_xn=want_xn, want_pack=want_pack)

    def _gdn(self, lw: LayerWeights, li: int, lay: StepLayout, v: dict) -> None:
        sp, m = self.spec, lay.m
        # fork: the tiny dense a/b projection runs beside the big qkvz stream
        main = torch.cuda.current_stream()
        # a speculative verify step keeps every layer's GDN inputs so that fold() can replay a prefix
        qo, ao = (self.qkvz_out, self.ab_out) if self.gdn_save is None else (self.gdn_save[0][li], self.gdn_save[1][li])
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            K.dense_skinny(lw.ab, self.xn, ao, m, pdl=False)
        self._gemv(lw.qkvz, self.xp_h, self.xs_h, qo, m, pdl=False)
        main.wait_stream(self.side)
        K.gdn_decode(qo, qo.shape[1], ao, self.ldab, lw.conv_w, lw.a_log, lw.dt_bias,
                     lw.gamma, self.pool.conv_state[li], self.pool.rec_state[li], v["gslot"], xpack=self.xp_v,
                     xs=self.xs_v, batch=lay.b, t=lay.t, nk=sp.nk, nv=sp.nv, group=self._grp(), eps=sp.eps, pdl=False)
        self._row_parallel(0, lw.out_proj, self.xp_v, self.xs_v, m, lw.ln2, want_xn=False)

    def _pick_splits(self, b: int, ctx_hint: int) -> int:
        if self.attn_splits:
            return self.attn_splits
        pages = max(1, (ctx_hint + PAGE - 1) // PAGE)
        if self.uniform_rows:
            b = 8        # a speculating engine: the split of the keys (and with it the order of the partial sums) must not
                         # depend on how many sequences share the step, or batched verify rows round differently from plain ones
        want = max(1, (2 * 148) // max(1, b * self.spec.hkv))
        return max(1, min(self.max_splits, want, (pages + 3) // 4))

    def _full(self, lw: LayerWeights, li: int, lay: StepLayout, v: dict, splits: int, ctx_hint: int = 0) -> None:
        sp, m = self.spec, lay.m
        self._gemv(lw.qkv, self.xp_h, self.xs_h, self.qkv_out, m, pdl=self.pdl)
        qn = 2 * sp.hq * sp.hd
        kraw = self.qkv_out[:, qn:]
        vraw = self.qkv_out[:, qn + sp.hkv * sp.hd:]
        K.qknorm_rope_insert(self.qkv_out, self.qkv_n, kraw, self.qkv_n, vraw, self.qkv_n, lw.q_norm, lw.k_norm,
                             v["pos3"], self.inv_freq, self.section, v["kv_slot"], self.q_rope, self.pool.k_pool[li],
                             self.pool.v_pool[li], m, sp.hq, sp.hkv, sp.hd, sp.rotary_dim, sp.eps, self.rope_scale,
                             pdl=self.pdl, scales=self.pool.scales(li))
        K.paged_attn(self.q_rope, self.pool.k_pool[li], self.pool.v_pool[li], self.block_table, v["bt_row"], v["ctx"],
                     self.part_o, self.part_ml, lay.b, lay.t, sp.hq, sp.hkv, sp.hd, self.max_blocks, splits, self.scale,
                     pdl=self.pdl, scales=self.pool.scales(li),
                     per_pages=((ctx_hint + PAGE - 1) // PAGE + splits - 1) // splits if self.uniform_rows and ctx_hint else 0)
        K.attn_reduce(self.part_o, self.part_ml, splits, self.qkv_out, self.qkv_n, m, sp.hq, xpack=self.xp_a,
                      xs=self.xs_a, group=self._grp(), pdl=self.pdl)
        self._row_parallel(0, lw.o_proj, self.xp_a, self.xs_a, m, lw.ln2, want_xn=False)

    def _head(self, m: int, sample: bool = True) -> None:
        """lm_head over ``self.xn`` (the final norm is produced by the last row-parallel step) and the
        greedy sample; with a vocab-split head the per-rank winners are merged across ranks."""
        w = self.w
        self._pf_hook(w.lm_head, False)
        K.dense_skinny(w.lm_head, self.xn, self.logits, m, pdl=self.pdl)
        self._pf_hook(w.lm_head, True)
        if not sample:
            return
        symm = getattr(self.comm, "symm", None) if self.comm is not None else None
        if self.vocab_split and symm is not None:
            K.argmax(self.logits, m, self.vocab_local, self.vocab_local, self.am_val, self.am_idx, self.am_parts,
                     self.loc_idx, w.vocab_offset, pdl=self.pdl, out_val=self.loc_val)
            symm.argmax_merge(self.loc_val, self.loc_idx, self.out_tok, m, pdl=self.pdl)
        else:
            K.argmax(self.logits, m, self.vocab_local, self.vocab_local, self.am_val, self.am_idx, self.am_parts,
                     self.out_tok, w.vocab_offset, pdl=self.pdl)

    # -- one-token step on the FMA arm -----------------------------------------------------------
    def _fma_ok(self, lay: StepLayout) -> bool:
        """The fused one-token path applies: one row, slice-major group-128 int4 weights, 15-bit-equivalent activations, and no
        mode that needs row-count-independent arithmetic (speculative verify reproduces plain decoding bit for bit on the
        integer arm). Under tensor parallelism it needs the symmetric workspace (the collective lives inside the
        projections) and no hidden-state taps (the residual stream is only materialised inside the next projection)."""
        w0 = self.w.layers[0].gate_up if self.w.layers else None
        if not (self.decode_gemv == "fma" and lay.m == 1 and not self.uniform_rows and self.act_bits == 15
                and getattr(w0, "layout", "") == "slice" and getattr(w0, "group", 0) == 128):
            return False
        if self.comm is None or self.spec.tp_world == 1:
            return True
        return getattr(self.comm, "symm", None) is not None and self.taps is None and self.spec.hidden // 8 <= 1024

    def _step_forward_fma(self, lay: StepLayout, v: dict, splits: int, ctx_hint: int) -> None:
        """Layers of a one-token step with every projection on the FMA arm: the RMSNorm is the prologue of the column
        projections, the residual add / silu * up their epilogue, the GDN a / b rows ride in the qkvz launch.

        Tensor parallel: a row-parallel projection stores its partial sums into every rank's slot buffer while it streams
        (``fma_push``), and the next column-parallel projection waits for the ranks' flags, adds the slots to the residual
        stream and normalises in its own prologue (``fma_pull``): the all-reduce costs no launch of its own. The residual
        stream alternates between two buffers, because the CTA that stores the new row must not overwrite what the other
        CTAs of the same launch still read."""
        sp, pdl = self.spec, self.pdl
        symm = getattr(self.comm, "symm", None) if (self.comm is not None and sp.tp_world > 1) else None
        if symm is None and self.ksplit and self.taps is None and sp.hidden // 8 <= 1024:
            # one GPU: the projections into the hidden size have few row tiles; cut their k range into parts that land in
            # local slots (the same push / pull kernels with a world of one)
            if self._local_split is None:
                from ..parallel.symm import LocalSplit

                self._local_split = LocalSplit(self.device, sp.hidden, kparts=self.ksplit)
            symm = self._local_split
        st = {"cur": self.h, "alt": self.h_alt, "pending": None}
        if symm is not None and (2 * len(self.w.layers) - 1) % 2 == 1:
            # an odd number of buffer swaps follows: start in the alternate buffer so that the step ends in self.h
            self.h_alt[:1].copy_(self.h[:1])
            st["cur"], st["alt"] = self.h_alt, self.h
        mix, act = self.mix[0], self.act[0]

        def col(w, out, norm_w, epi=K.EPI_STORE, **ab):
            if st["pending"] is None:
                K.w4_fma(w, st["cur"][0], out, norm_w=norm_w, epi=epi, eps=sp.eps, pdl=pdl, **ab)
                return
            symm.fma_pull(st["pending"], w, st["cur"][0], st["alt"][0], norm_w, out, epi=epi, eps=sp.eps, pdl=pdl, **ab)
            st["cur"], st["alt"], st["pending"] = st["alt"], st["cur"], None

        def row(which, w, x):
            if symm is None:
                K.w4_fma(w, x, st["cur"][0], residual=st["cur"][0], epi=K.EPI_RESIDUAL, pdl=pdl)
            else:
                symm.fma_push(which, w, x, pdl=pdl)
                st["pending"] = which

        fi = gi = 0
        for i, lw in enumerate(self.w.layers):
            if lw.kind == "gdn":
                qo, ao = (self.qkvz_out, self.ab_out) if self.gdn_save is None else (self.gdn_save[0][gi], self.gdn_save[1][gi])
                col(lw.qkvz, qo[0], lw.ln1, ab_w=lw.ab_dense, ab_out=ao[0], ab_rows=lw.ab_dense.shape[0])
                K.gdn_decode(qo, qo.shape[1], ao, self.ldab, lw.conv_w, lw.a_log, lw.dt_bias, lw.gamma,
                             self.pool.conv_state[gi], self.pool.rec_state[gi], v["gslot"], out=self.mix, batch=lay.b, t=lay.t,
                             nk=sp.nk, nv=sp.nv, group=self.G, eps=sp.eps, pdl=pdl)
                row(0, lw.out_proj, mix)
                gi += 1
            else:
                col(lw.qkv, self.qkv_out[0], lw.ln1)
                qn = 2 * sp.hq * sp.hd
                kraw, vraw = self.qkv_out[:, qn:], self.qkv_out[:, qn + sp.hkv * sp.hd:]
                K.qknorm_rope_insert(self.qkv_out, self.qkv_n, kraw, self.qkv_n, vraw, self.qkv_n, lw.q_norm, lw.k_norm,
                                     v["pos3"], self.inv_freq, self.section, v["kv_slot"], self.q_rope, self.pool.k_pool[fi],
                                     self.pool.v_pool[fi], 1, sp.hq, sp.hkv, sp.hd, sp.rotary_dim, sp.eps, self.rope_scale,
                                     pdl=pdl, scales=self.pool.scales(fi))
                K.paged_attn(self.q_rope, self.pool.k_pool[fi], self.pool.v_pool[fi], self.block_table, v["bt_row"], v["ctx"],
                             self.part_o, self.part_ml, lay.b, lay.t, sp.hq, sp.hkv, sp.hd, self.max_blocks, splits, self.scale,
                             pdl=pdl, scales=self.pool.scales(fi))
                K.attn_reduce(self.part_o, self.part_ml, splits, self.qkv_out, self.qkv_n, 1, sp.hq, out=self.mix,
                              group=self.G, pdl=pdl)
                row(0, lw.o_proj, mix)
                fi += 1
            col(lw.gate_up, act, lw.ln2, epi=K.EPI_SILU_MUL)
            row(1, lw.down, act)
            if self.taps is not None and i in self.taps:
                self.taps[i][:1].copy_(self.h[:1])
        if st["pending"] is not None:
            assert st["cur"] is self.h
            symm.push_residual_norm(st["pending"], self.h, 1, self.w.final_norm, normed=self.xn, group=self.G, eps=sp.eps, pdl=pdl,
                                    fma=True)
        else:
            self._norm(1, self.w.final_norm, want_xn=True, want_pack=False)

    # -- decode / verify step ------------------------------------------------------------------
    def step_forward(self, lay: StepLayout, *, ctx_hint: int = 2048, advance: bool = False, sample: bool = True) -> None:
        """One forward over ``lay.m`` rows whose inputs sit in ``self.inp``. Capturable."""
        v = self.views(lay)
        m = lay.m
        splits = self._pick_splits(lay.b, ctx_hint)
        K.embed(v["ids"], self.w.embed, self.h, m, pdl=False)
        if self.pre_hook is not None:
            self.pre_hook(m)
        layers = self.w.layers
        if self._fma_ok(lay):
            self._step_forward_fma(lay, v, splits, ctx_hint)
            layers = ()
        else:
            self._norm(m, layers[0].ln1, want_xn=layers[0].kind == "gdn")
        fi = gi = 0
        for i, lw in enumerate(layers):
            if lw.kind == "gdn":
                self._gdn(lw, gi, lay, v)
                gi += 1
            else:
                self._full(lw, fi, lay, v, splits, ctx_hint)
                fi += 1
            last = i + 1 == len(layers)
            nxt_w = self.w.final_norm if last else layers[i + 1].ln1
            self._mlp(lw, m, nxt_w, want_xn=last or layers[i + 1].kind == "gdn", want_pack=not last)
            if self.taps is not None and i in self.taps:
                self.taps[i][:m].copy_(self.h[:m])
        self._head(m, sample)
        if advance:
            assert lay.t == 1
            K.decode_advance(self.inp, self.out_tok, self.block_table, self.max_blocks, lay.b, pdl=self.pdl)

    def enable_gdn_save(self) -> None:
        """Allocate the per-layer GDN input buffers that a verify step fills and fold() replays."""
        if self.gdn_save is None:
            sp, ng = self.spec, self.spec.n_layers - self.spec.n_full
            self.gdn_save = (torch.zeros(ng, self.MAX_ROWS, sp.conv_dim + sp.value_dim, dtype=torch.bfloat16, device=self.device),
                             torch.zeros(ng, self.MAX_ROWS, self.ldab, dtype=torch.bfloat16, device=self.device))
            self.graphs.clear()     # captured graphs point at the old buffers

    def fold(self, gslot: torch.Tensor, t: int) -> None:
        """Advance the GDN state of one sequence over the first ``t`` rows of the last (saved)
        step: the recurrent state update only, no outputs. After a speculative verify the caller
        restores the pre-verify state and folds the accepted prefix, so the state equals what
        plain decoding of those tokens would have produced. Capturable; ``gslot`` int32 [1]."""
        sp = self.spec
        qs, as_ = self.gdn_save
        gi = 0
        for lw in self.w.layers:
            if lw.kind != "gdn":
                continue
            K.gdn_decode(qs[gi], qs.shape[2], as_[gi], self.ldab, lw.conv_w, lw.a_log, lw.dt_bias, lw.gamma,
                         self.pool.conv_state[gi], self.pool.rec_state[gi], gslot, batch=1, t=t, nk=sp.nk, nv=sp.nv,
                         group=self.G, eps=sp.eps, pdl=False)
            gi += 1

    def fold_batch(self, b: int, t: int) -> None:
        """``fold`` for the ``b`` sequences of the last (b, t) step at once: sequence i (GDN slot ``fold_slots[i]``) advances
        over its first ``fold_tlen[i]`` rows; a slot < 0 or a length 0 leaves that sequence alone. Capturable."""
        sp = self.spec
        qs, as_ = self.gdn_save
        gi = 0
        for lw in self.w.layers:
            if lw.kind != "gdn":
                continue
            K.gdn_decode(qs[gi], qs.shape[2], as_[gi], self.ldab, lw.conv_w, lw.a_log, lw.dt_bias, lw.gamma,
                         self.pool.conv_state[gi], self.pool.rec_state[gi], self.fold_slots, batch=b, t=t, nk=sp.nk, nv=sp.nv,
                         group=self.G, eps=sp.eps, pdl=False, tlen=self.fold_tlen)
            gi += 1

    def capture_fold_batch(self, b: int, t: int):
        """CUDA graph of fold_batch(b, t) reading ``self.fold_slots`` / ``self.fold_tlen`` (int32 [MAX_ROWS])."""
        key = ("foldb", b, t)
        g = self.graphs.get(key)
        if g is None:
            if not hasattr(self, "fold_slots"):
                self.fold_slots = torch.full((self.MAX_ROWS,), -1, dtype=torch.int32, device=self.device)
                self.fold_tlen = torch.zeros(self.MAX_ROWS, dtype=torch.int32, device=self.device)
            if not self.use_graphs:
                g = self.graphs[key] = _EagerStep(lambda: self.fold_batch(b, t))
                return g
            stream = torch.cuda.Stream(device=self.device)
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                saved = (self.fold_slots.clone(), self.fold_tlen.clone())
                self.fold_slots.fill_(-1)
                self.fold_batch(b, t)                  # warm-up on inert slots
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    self.fold_batch(b, t)
                self.fold_slots.copy_(saved[0])
                self.fold_tlen.copy_(saved[1])
            torch.cuda.current_stream().wait_stream(stream)
            self.graphs[key] = g
        return g

    def capture_fold(self, t: int):
        """CUDA graph of fold(t) reading the GDN slot from ``self.fold_slot``."""
        key = ("fold", t)
        g = self.graphs.get(key)
        if g is None:
            if not hasattr(self, "fold_slot"):
                self.fold_slot = torch.full((1,), -1, dtype=torch.int32, device=self.device)
            if not self.use_graphs:
                g = self.graphs[key] = _EagerStep(lambda: self.fold(self.fold_slot, t))
                return g
            stream = torch.cuda.Stream(device=self.device)
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                saved = self.fold_slot.clone()
                self.fold_slot.fill_(-1)
                self.fold(self.fold_slot, t)           # warm-up on an inert slot
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    self.fold(self.fold_slot, t)
                self.fold_slot.copy_(saved)
            torch.cuda.current_stream().wait_stream(stream)
            self.graphs[key] = g
        return g

    def capture(self, b: int, t: int = 1, *, ctx_hint: int = 2048, advance: bool = False, sample: bool = True):
        """Capture (once) and return the CUDA graph of a (b, t) step."""
        key = (b, t, self._pick_splits(b, ctx_hint), advance, sample, ctx_hint if self.uniform_rows else 0)
        g = self.graphs.get(key)
        if g is not None:
            return g
        lay = StepLayout(b, t)
        if not self.use_graphs or (self.comm is not None and not getattr(self.comm, "capturable", True)):
            # graphs switched off (`[cuda] graph = false`), or a transport that crosses the host (relay fallback) and cannot
            # be captured: the "graph" is the eager step
            self.graphs[key] = _EagerStep(lambda: self.step_forward(lay, ctx_hint=ctx_hint, advance=advance, sample=sample))
            return self.graphs[key]
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            # warm-up outside capture writes state; callers capture before real traffic or accept
            # that rows with gdn slot -1 / kv slot -1 are inert. Here inputs are forced inert.
            saved = self.inp.clone()
            v = self.views(lay)
            v["gslot"].fill_(-1)
            v["kv_slot"].fill_(-1)
            v["ctx"].fill_(1)
            v["bt_row"].zero_()
            prefetch = self.l2_prefetch_mb > 0 and b * t < self.BATCH_GEMM_FROM
            self._pf_rec = [] if prefetch else None
            self.step_forward(lay, ctx_hint=ctx_hint, advance=False, sample=sample)
            sched, self._pf_rec = self._pf_rec, None
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            mark = K.launch_seq()
            with torch.cuda.graph(graph, stream=stream):
                if prefetch and sched:
                    side = torch.cuda.Stream(device=self.device)
                    self._pf_play, self._pf_i = (sched, side, stream), 0
                try:
                    self.step_forward(lay, ctx_hint=ctx_hint, advance=advance, sample=sample)
                finally:
                    if self._pf_play is not None:
                        stream.wait_stream(self._pf_play[1])       # join the prefetch branch before the capture ends
                        self._pf_play = None
            self.inp.copy_(saved)
        torch.cuda.current_stream().wait_stream(stream)
        self.graphs[key] = _CapturedStep(graph, K.launches_since(mark))
        return self.graphs[key]

    def graph_manifest(self) -> list[dict]:
        """Per captured step graph: its key, how often it was replayed, and the native entries one replay launches (with
        their multiplicity), so that device work is attributable to entries although replays bypass the launch ring."""
        out = []
        for key, g in self.graphs.items():
            if isinstance(g, _CapturedStep):
                counts: dict = {}
                for name in g.launches:
                    counts[name] = counts.get(name, 0) + 1
                out.append({"key": [str(k) for k in key] if isinstance(key, tuple) else str(key), "replays": g.replays,
                            "launches_per_replay": len(g.launches), "entries": counts})
        return out

    # -- prefill ---------------------------------------------------------------------------------
    def _prefill_ws(self, t: int):
        if self._pf is not None and self._pf["t"] >= t:
            return self._pf
        sp, dev = self.spec, self.device
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=dev)
        # GEMM inputs are fp16 on the tcgen05 arm (exact int4 dequant), bf16 on the baseline arm
        xd = torch.float16 if self.prefill_gemm != "baseline" else torch.bfloat16
        xa = lambda *s: torch.empty(*s, dtype=xd, device=dev)
        widest = max(2 * sp.inter, sp.conv_dim + sp.value_dim, self.qkv_n)
        ws = dict(t=t, h=bf(t, sp.hidden), x=xa(t, sp.hidden), wide=bf(t, widest), act=xa(t, sp.inter),
                  conv=bf(t, sp.conv_dim), mix=xa(t, max(sp.value_dim, sp.hq * sp.hd)), ab=bf(t, self.ldab),
                  q=bf(t + 8, sp.hq, sp.hd), y=bf(t, sp.hidden),
                  part_o=torch.empty((t + 8) * sp.hq * sp.hd, dtype=torch.float32, device=dev),
                  part_ml=torch.empty((t + 8) * sp.hq * 2, dtype=torch.float32, device=dev),
                  pos3=torch.zeros(3, t, dtype=torch.int32, device=dev),
                  kv_slot=torch.zeros(t, dtype=torch.int32, device=dev),
                  ctx=torch.zeros(t // 8 + 2, dtype=torch.int32, device=dev),
                  bt_row=torch.zeros(t // 8 + 2, dtype=torch.int32, device=dev),
                  ids=torch.zeros(t, dtype=torch.int32, device=dev))
        self._pf = ws
        return ws

    def _gemm(self, w, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[T, N] = x[T, K] @ dequant(w)^T for a prefill chunk."""
        from ..ops import linear

        if w.layout == "nvfp4":
            return linear.nvfp4_gemm(w, x, out, arm=self.prefill_gemm)
        return linear.w4_gemm(w, x, out, arm=self.prefill_gemm)

    def _gdn_prefill(self, lw, gi: int, wide, nq: int, ab, conv, mix, t: int, gdn_slot: int, use_state: bool, snap) -> None:
        """Convolution + delta-rule scan of one GDN layer over the chunk's rows. With ``snap = (rows, state_row)`` the
        scan stops after ``rows`` rows, the layer's convolution history and recurrent state are copied to ``state_row``
        (the prefix snapshot at a block boundary inside the chunk) and the remaining rows follow."""
        sp, pool = self.spec, self.pool
        parts = [(0, t)] if snap is None else [(0, snap[0]), (snap[0], t)]
        for a, b in parts:
            st = use_state or a > 0
            K.gdn_conv_fwd(wide[a:], nq, lw.conv_w, pool.conv_state[gi], gdn_slot, conv[a:], b - a, sp.nk, sp.nv, st)
            K.gdn_scan(conv[a:], wide[a:, sp.conv_dim:], nq, ab[a:], self.ldab, lw.a_log, lw.dt_bias, lw.gamma,
                       pool.rec_state[gi], gdn_slot, mix[a:], b - a, sp.nk, sp.nv, st, sp.eps)
            if snap is not None and b == snap[0]:
                pool.conv_state[gi, snap[1]].copy_(pool.conv_state[gi, gdn_slot])
                pool.rec_state[gi, snap[1]].copy_(pool.rec_state[gi, gdn_slot])

    def prefill_chunk_forward(self, ids: torch.Tensor, pos0: int, seq_row: int, gdn_slot: int, *,
                              pos3: torch.Tensor | None = None, want_logits: bool = True,
                              embeds: torch.Tensor | None = None, snap: tuple | None = None):
        """Run one prefill chunk (eager). ``ids`` int32 [T] on device; KV pages for positions
        pos0..pos0+T-1 must already be in ``block_table[seq_row]``. Returns the argmax token of
        the last row when ``want_logits``. ``snap = (rows, state_row)``: also leave the GDN state after the first
        ``rows`` rows of the chunk in ``state_row`` (0 < rows < T)."""
        from ..ops import linear

        sp, pool = self.spec, self.pool
        t = ids.shape[0]
        pipe = self._pipe()
        if pipe is not None and t >= self.SP_FROM and t <= pipe.rows and self.prefill_gemm in ("tc", "tcr") and self.taps is None \
                and self.w.layout != "nvfp4":
            return self._prefill_chunk_sp(pipe, ids, pos0, seq_row, gdn_slot, pos3, want_logits, embeds, snap)
        ws = self._prefill_ws(max(t, 16))
        h, x = ws["h"][:t], ws["x"][:t]
        if pos3 is None:
            p = torch.arange(pos0, pos0 + t, dtype=torch.int32, device=self.device)
            ws["pos3"][:, :t] = p[None]
        else:
            ws["pos3"][:, :t] = pos3
        pos3_v = ws["pos3"][:, :t].contiguous()
        tpos = torch.arange(pos0, pos0 + t, device=self.device)
        pages = self.block_table[seq_row, (tpos // PAGE).long()]
        kv_slot = (pages * PAGE + (tpos % PAGE).int()).int()
        # query groups of 8 rows (+ a tail group)
        ng, tail = t // 8, t % 8
        if ng:
            ws["ctx"][:ng] = pos0 + 8 * torch.arange(1, ng + 1, dtype=torch.int32, device=self.device)
            ws["bt_row"][:ng] = seq_row
        if tail:
            ws["ctx"][ng] = pos0 + t
            ws["bt_row"][ng] = seq_row
        if embeds is None:
            K.embed(ids, self.w.embed, h, t)
        else:
            h.copy_(embeds)
        fi = gi = 0
        use_state = pos0 > 0
        for i, lw in enumerate(self.w.layers):
            K.rmsnorm_pack(h, lw.ln1, normed=x, m=t, k=sp.hidden, group=self.G, eps=sp.eps)
            if lw.kind == "gdn":
                nq = sp.conv_dim + sp.value_dim
                wide = ws["wide"].view(-1)[:t * nq].view(t, nq)
                self._gemm(lw.qkvz, x, wide)
                ab = ws["ab"][:t]
                linear.dense_gemm(x, lw.ab_dense, ab, arm="baseline" if self.prefill_gemm == "baseline" else "tc")
                mix = ws["mix"].view(-1)[:t * sp.value_dim].view(t, sp.value_dim)
                self._gdn_prefill(lw, gi, wide, nq, ab, ws["conv"][:t], mix, t, gdn_slot, use_state, snap)
                self._gemm(lw.out_proj, mix, ws["y"][:t])
                gi += 1
            else:
                wide = ws["wide"].view(-1)[:t * self.qkv_n].view(t, self.qkv_n)
                self._gemm(lw.qkv, x, wide)
                qn = 2 * sp.hq * sp.hd
                K.qknorm_rope_insert(wide, self.qkv_n, wide[:, qn:], self.qkv_n, wide[:, qn + sp.hkv * sp.hd:],
                                     self.qkv_n, lw.q_norm, lw.k_norm, pos3_v, self.inv_freq, self.section, kv_slot,
                                     ws["q"], pool.k_pool[fi], pool.v_pool[fi], t, sp.hq, sp.hkv, sp.hd, sp.rotary_dim,
                                     sp.eps, self.rope_scale, scales=pool.scales(fi))
                mix = ws["mix"].view(-1)[:t * sp.hq * sp.hd].view(t, sp.hq * sp.hd)
                self._prefill_attention(ws, pool, fi, wide, mix, t, pos0, seq_row, ng, tail)
                self._gemm(lw.o_proj, mix, ws["y"][:t])
                fi += 1
            if self.comm is not None and sp.tp_world > 1:
                self.comm.allreduce_prefill(ws["y"][:t])
            K.rmsnorm_pack(h, lw.ln2, delta=ws["y"][:t], out_h=h, normed=x, m=t, k=sp.hidden, group=self.G, eps=sp.eps)
            gu = ws["wide"].view(-1)[:t * 2 * sp.inter].view(t, 2 * sp.inter)
            self._gemm(lw.gate_up, x, gu)
            K.silu_mul(gu, t, sp.inter, out=ws["act"][:t], group=self.G)
            self._gemm(lw.down, ws["act"][:t], ws["y"][:t])
            if self.comm is not None and sp.tp_world > 1:
                self.comm.allreduce_prefill(ws["y"][:t])
            h.add_(ws["y"][:t])
            if self.taps is not None and i in self.taps and "prefill" in self.taps:
                self.taps["prefill"][i] = h.clone()
        if self.taps is not None and self.tap_sink is not None and "prefill" in self.taps:
            self.tap_sink(pos0, t, self.taps["prefill"])
        if not want_logits:
            return None
        self.h[:1].copy_(h[t - 1:t])
        self._norm(1, self.w.final_norm, want_xn=True, want_pack=False)
        self._head(1, sample=True)
        return self.out_tok[:1]

    SP_FROM = 256       # tokens per chunk from which the sequence-parallel fused path is used under tensor parallelism

    # keys from which a prefill chunk's attention runs as tcgen05 GEMMs (0: never)
    ATTN_GEMM_FROM = int(os.environ.get("OWL_ATTN_GEMM_FROM", "2048"))

    def _prefill_attention(self, ws, pool, fi: int, wide, mix, t: int, pos0: int, seq_row: int, ng: int, tail: int) -> None:
        """Causal attention of a prefill chunk over the sequence's pages. Short contexts: the fused warp-level kernel (8 query
        rows per group). Long contexts: gather the pages once, S = Q K^T and O = P V as tcgen05 GEMMs with a causal softmax
        between them (``K.attn_gemm_prefill``): the fused kernel's tensor path tops out near 60 TFLOP/s of attention work."""
        sp = self.spec
        ctx = pos0 + t
        if self.ATTN_GEMM_FROM and ctx >= self.ATTN_GEMM_FROM and t >= 32 and sp.hd == 256:
            aw = self._attn_ws
            if aw is None or aw["t"] < t or aw["ctx"] < ctx:
                cap = max(ctx, 2 * (aw["ctx"] if aw else 0), 8192)
                self._attn_ws = aw = K.attn_gemm_ws(self.device, max(t, aw["t"] if aw else 0), cap, sp.hq, sp.hkv, sp.hd)
            K.attn_gemm_prefill(ws["q"], pool.k_pool[fi], pool.v_pool[fi], pool.scales(fi), self.block_table[seq_row], pos0, t,
                                sp.hq, sp.hkv, sp.hd, self.scale, aw, wide, self.qkv_n, mix)
            return
        if ng:
            K.paged_attn(ws["q"], pool.k_pool[fi], pool.v_pool[fi], self.block_table, ws["bt_row"], ws["ctx"],
                         ws["part_o"], ws["part_ml"], ng, 8, sp.hq, sp.hkv, sp.hd, self.max_blocks, 1, self.scale,
                         scales=pool.scales(fi))
        if tail:
            off = ng * 8
            K.paged_attn(ws["q"][off:], pool.k_pool[fi], pool.v_pool[fi], self.block_table, ws["bt_row"][ng:],
                         ws["ctx"][ng:], ws["part_o"][off * sp.hq * sp.hd:], ws["part_ml"][off * sp.hq * 2:], 1,
                         tail, sp.hq, sp.hkv, sp.hd, self.max_blocks, 1, self.scale, scales=pool.scales(fi))
        K.attn_reduce(ws["part_o"], ws["part_ml"], 1, wide, self.qkv_n, t, sp.hq, out=mix, group=self.G)

    def _pipe(self):
        """The prefill pipe of the tensor-parallel communicator (or one set explicitly, e.g. a world of one)."""
        if self.pf_pipe is not None:
            return self.pf_pipe
        symm = getattr(self.comm, "symm", None) if self.comm is not None else None
        if symm is None or self.spec.tp_world == 1 or not self.sp_prefill:
            return None
        return getattr(symm, "prefill", None)

    def _prefill_chunk_sp(self, pipe, ids, pos0: int, seq_row: int, gdn_slot: int, pos3, want_logits: bool, embeds, snap=None):
        """Tensor-parallel prefill chunk with the collectives inside the GEMMs: every row-parallel projection is a
        tcgen05 GEMM whose epilogue scatters its partial row tiles to their owner ranks over NVLink; the owner adds
        them to its share of the residual stream, normalises and stores the result into every rank's activation buffer;
        the next column-parallel GEMM starts on the row tiles that have arrived. The residual stream of the chunk is
        sharded by 128-row tiles over the ranks (sequence parallel) and never gathered.

        Reference counterpart: all-reduce injection after every row-parallel node followed by a separate
        fused_add_rmsnorm launch (crates/models/src/interpreters/eval.rs:1154-1419); no GEMM / collective overlap there."""
        from ..ops import linear

        sp, pool, dev = self.spec, self.pool, self.device
        t = ids.shape[0]
        ws = self._prefill_ws(t)
        xd = torch.float16
        dense = lambda w: linear.w4_dense(w, xd, dev, resident=self.prefill_gemm == "tcr")
        if pos3 is None:
            ws["pos3"][:, :t] = torch.arange(pos0, pos0 + t, dtype=torch.int32, device=dev)[None]
        else:
            ws["pos3"][:, :t] = pos3
        pos3_v = ws["pos3"][:, :t].contiguous()
        tpos = torch.arange(pos0, pos0 + t, device=dev)
        pages = self.block_table[seq_row, (tpos // PAGE).long()]
        kv_slot = (pages * PAGE + (tpos % PAGE).int()).int()
        ng, tail = t // 8, t % 8
        if ng:
            ws["ctx"][:ng] = pos0 + 8 * torch.arange(1, ng + 1, dtype=torch.int32, device=dev)
            ws["bt_row"][:ng] = seq_row
        if tail:
            ws["ctx"][ng] = pos0 + t
            ws["bt_row"][ng] = seq_row
        own = pipe.own_rows(t).clamp(max=t - 1)
        if own.numel():
            if embeds is None:
                K.embed(ids[own].contiguous(), self.w.embed, pipe.h, own.numel())
            else:
                pipe.h[:own.numel()].copy_(embeds[own])
        layers = self.w.layers
        pipe.reduce_norm_gather(t, layers[0].ln1, out_dtype=xd, eps=sp.eps, seed=True)
        fi = gi = 0
        use_state = pos0 > 0
        for i, lw in enumerate(layers):
            x = pipe.x(t, xd)
            if lw.kind == "gdn":
                nq = sp.conv_dim + sp.value_dim
                wide = ws["wide"].view(-1)[:t * nq].view(t, nq)
                pipe.gemm_ag(dense(lw.qkvz), wide, t)
                ab = ws["ab"][:t]
                linear.dense_gemm(x, lw.ab_dense, ab, arm="tc")        # after the gathering GEMM: all rows are here
                mix = ws["mix"].view(-1)[:t * sp.value_dim].view(t, sp.value_dim)
                self._gdn_prefill(lw, gi, wide, nq, ab, ws["conv"][:t], mix, t, gdn_slot, use_state, snap)
                pipe.gemm_rs(mix, dense(lw.out_proj), t)
                gi += 1
            else:
                wide = ws["wide"].view(-1)[:t * self.qkv_n].view(t, self.qkv_n)
                pipe.gemm_ag(dense(lw.qkv), wide, t)
                qn = 2 * sp.hq * sp.hd
                K.qknorm_rope_insert(wide, self.qkv_n, wide[:, qn:], self.qkv_n, wide[:, qn + sp.hkv * sp.hd:],
                                     self.qkv_n, lw.q_norm, lw.k_norm, pos3_v, self.inv_freq, self.section, kv_slot,
                                     ws["q"], pool.k_pool[fi], pool.v_pool[fi], t, sp.hq, sp.hkv, sp.hd, sp.rotary_dim,
                                     sp.eps, self.rope_scale, scales=pool.scales(fi))
                mix = ws["mix"].view(-1)[:t * sp.hq * sp.hd].view(t, sp.hq * sp.hd)
                self._prefill_attention(ws, pool, fi, wide, mix, t, pos0, seq_row, ng, tail)
                pipe.gemm_rs(mix, dense(lw.o_proj), t)
                fi += 1
            pipe.reduce_norm_gather(t, lw.ln2, out_dtype=xd, eps=sp.eps)
            gu = ws["wide"].view(-1)[:t * 2 * sp.inter].view(t, 2 * sp.inter)
            pipe.gemm_ag(dense(lw.gate_up), gu, t)
            K.silu_mul(gu, t, sp.inter, out=ws["act"][:t], group=self.G)
            pipe.gemm_rs(ws["act"][:t], dense(lw.down), t)
            pipe.reduce_norm_gather(t, layers[i + 1].ln1 if i + 1 < len(layers) else None, out_dtype=xd, eps=sp.eps)
        if not want_logits:
            return None
        owner, lrow = pipe.local_row(t - 1)
        if pipe.rank == owner:
            self.h[:1].copy_(pipe.h[lrow:lrow + 1])
        else:
            self.h[:1].zero_()
        if pipe.world > 1:
            self.comm.allreduce_prefill(self.h[:1])             # the other ranks hold zeros: a broadcast of the last row
        self._norm(1, self.w.final_norm, want_xn=True, want_pack=False)
        self._head(1, sample=True)
        return self.out_tok[:1]

    def last_hidden(self) -> torch.Tensor:
        return self.h
