"""Multi-token-prediction (MTP) draft head.

One gated-attention decoder layer that shares the target's embedding table and lm_head:

    x_q  = fc_e . norm_e(embed(tok_{q+1})) + fc_h . norm_h(hidden_q)      (fc = [fc_e | fc_h] : 2H -> H)
    y_q  = decoder_layer(x_q)   (own paged KV at index q, same page ids as the target)
    draft_{q+2} = argmax lm_head(norm(y_q))

``absorb`` feeds rows whose target hidden is known (the rows a verify step accepted, or a prefill
chunk); its last row yields the first draft of the next round. ``chain`` continues from the
head's own hidden for the remaining drafts, entirely on the device (self-feeding steps).
The head is a one-layer ``HybridRunner`` whose ``pre_hook`` mixes the hidden in, so it runs on the
same kernels, CUDA graphs and TP collectives as the target.

Reference counterpart: ``crates/models/src/layers/mtp.rs:1-20``, ``crates/engine/src/exec/draft.rs``
(MTP chain), ``exec/mtp_window.rs``.
"""
from __future__ import annotations

from dataclasses import replace

import torch

from ..ops import kernels as K
from ..ops import quant as Q
from . import hybrid as H


class MtpHead:
    def __init__(self, target: H.HybridRunner, *, seed: int = 1, std: float = 0.02, weights: dict | None = None,
                 kv_dtype: str | None = None):
        """``kv_dtype``: format of the head's own KV pool (``"bf16"`` or ``"fp8"``, half the memory; None = the target
        pool's format). ``weights`` (optional): dense tensors ``fc`` [H, 2H], ``norm_e``, ``norm_h``, ``norm`` [H] and the
        HF-named tensors of one full-attention layer under ``layers.0.*``; random-init otherwise."""
        self.target = target
        spec = replace(target.spec, n_layers=1, full_every=1)
        dev, Hd = target.device, spec.hidden
        layout = target.w.layout
        if weights is None:
            hw = H.random_weights(replace(spec, vocab=16), dev, group=target.G, seed=seed, std=std, layout=layout)
            g = torch.Generator(device=dev).manual_seed(seed + 77)
            fc = torch.randn(Hd, 2 * Hd, device=dev, generator=g) * std
            # start close to "copy the hidden": the head then predicts from the target's own features
            fc[:, Hd:] += torch.eye(Hd, device=dev)
            norm_e = norm_h = torch.zeros(Hd, device=dev)
        else:
            dense = {k: v for k, v in weights.items() if k.startswith("model.layers.0.") or k.startswith("layers.0.")}
            dense = {("model." + k if not k.startswith("model.") else k): v for k, v in dense.items()}
            dense.update({"model.embed_tokens.weight": torch.zeros(16, Hd), "model.norm.weight": weights["norm"],
                          "lm_head.weight": torch.zeros(16, Hd)})
            hw, _ = H.weights_from_dense(replace(spec, vocab=16), dense, dev, group=target.G, layout=layout)
            fc, norm_e, norm_h = weights["fc"].to(dev), weights["norm_e"].to(dev), weights["norm_h"].to(dev)
        hw.spec, hw.embed, hw.lm_head, hw.vocab_offset = spec, target.w.embed, target.w.lm_head, target.w.vocab_offset
        self.fc_e = Q.dense_skinny(fc[:, :Hd].contiguous().to(torch.bfloat16), dev)
        self.fc_h = Q.dense_skinny(fc[:, Hd:].contiguous().to(torch.bfloat16), dev)
        self.fc_dense = fc.to(torch.bfloat16)
        self.norm_e, self.norm_h = norm_e.to(torch.bfloat16), norm_h.to(torch.bfloat16)
        self.pool = H.StatePool(spec, dev, target.pool.n_pages, 1, kv_dtype=kv_dtype or getattr(target.pool, "kv_dtype", "fp8"))
        self.runner = H.HybridRunner(spec, hw, self.pool, max_seqs=target.max_seqs, max_blocks=target.max_blocks,
                                     prefill_chunk=target.prefill_chunk, comm=target.comm, pdl=target.pdl,
                                     prefill_gemm=target.prefill_gemm)
        self.runner.block_table = target.block_table          # same page ids as the target
        M = self.runner.MAX_ROWS
        self.hid_in = torch.zeros(M, Hd, dtype=torch.bfloat16, device=dev)
        self.e_n = torch.zeros(M, Hd, dtype=torch.bfloat16, device=dev)
        self.h_n = torch.zeros(M, Hd, dtype=torch.bfloat16, device=dev)
        self.drafts = torch.zeros(M, dtype=torch.int32, device=dev)
        self.runner.pre_hook = self._mix
        self._chains: dict = {}

    # x = fc_e . norm_e(embed) + fc_h . norm_h(hidden); runs inside the runner's step (capturable)
    def _mix(self, m: int) -> None:
        r, sp = self.runner, self.runner.spec
        K.rmsnorm_pack(r.h, self.norm_e, normed=self.e_n, m=m, k=sp.hidden, group=r.G, eps=sp.eps)
        K.rmsnorm_pack(self.hid_in, self.norm_h, normed=self.h_n, m=m, k=sp.hidden, group=r.G, eps=sp.eps)
        K.dense_skinny(self.fc_e, self.e_n, r.h, m)
        K.dense_skinny(self.fc_h, self.h_n, r.h, m, residual=r.h, epi=K.EPI_RESIDUAL)

    # -- rows with a known target hidden --------------------------------------------------------
    def absorb(self, next_ids: list[int], hiddens: torch.Tensor, q0: int, seq_row: int, pages: list[int]) -> None:
        """Rows q0 .. q0+T-1 (T <= 8): ``next_ids[i]`` = token at position q0+i+1, ``hiddens[i]`` = target hidden
        at position q0+i. Leaves the first draft in ``runner.out_tok[T-1]`` and the head's hidden in ``runner.h[T-1]``."""
        r, t = self.runner, len(next_ids)
        lay = H.StepLayout(1, t)
        v = r.views(lay)
        dev = r.device
        pos = torch.arange(q0, q0 + t, dtype=torch.int32, device=dev)
        v["ids"].copy_(torch.tensor(next_ids, dtype=torch.int32, device=dev))
        v["pos3"].copy_(pos.repeat(3))
        pg = torch.tensor([pages[(q0 + i) // H.PAGE] for i in range(t)], dtype=torch.int32, device=dev)
        v["kv_slot"].copy_(pg * H.PAGE + pos % H.PAGE)
        v["ctx"].fill_(q0 + t)
        v["gslot"].fill_(0)          # no GDN layer in the head; a non-negative slot marks the row as live
        v["bt_row"].fill_(seq_row)
        self.hid_in[:t].copy_(hiddens[:t])
        r.capture(1, t, ctx_hint=_bucket(q0 + t)).replay()
        self._last = (t, q0 + t, seq_row)

    def absorb_prefill(self, ids_next: torch.Tensor, hiddens: torch.Tensor, q0: int, seq_row: int) -> None:
        """Prefill-sized absorb (prompt chunk): GEMM path, fills the head's KV for positions q0 .. q0+T-1."""
        r, sp = self.runner, self.runner.spec
        t = ids_next.shape[0]
        e = torch.empty(t, sp.hidden, dtype=torch.bfloat16, device=r.device)
        K.embed(ids_next, r.w.embed, e, t)
        en, hn = torch.empty_like(e), torch.empty_like(e)
        K.rmsnorm_pack(e, self.norm_e, normed=en, m=t, k=sp.hidden, group=r.G, eps=sp.eps)
        K.rmsnorm_pack(hiddens.contiguous(), self.norm_h, normed=hn, m=t, k=sp.hidden, group=r.G, eps=sp.eps)
        x0 = torch.cat([en, hn], dim=1) @ self.fc_dense.t()          # library GEMM: off the hot path
        r.prefill_chunk_forward(ids_next, q0, seq_row, 0, want_logits=False, embeds=x0)

    # -- the head's own continuation -------------------------------------------------------------
    def chain(self, k: int) -> torch.Tensor:
        """After ``absorb``: ``k`` drafts (int32 [k] on the device). Draft 0 is the absorb step's
        prediction; drafts 1.. come from self-feeding single-row steps."""
        t, q, seq_row = self._last
        r = self.runner
        self.drafts[0:1].copy_(r.out_tok[t - 1:t])
        if k > 1:
            lay = H.StepLayout(1, 1)
            v = r.views(lay)
            # step input: the draft just produced, at the next position, with the head's own hidden
            v["ids"].copy_(r.out_tok[t - 1:t])
            v["pos3"].fill_(q)
            v["kv_slot"].copy_(r.block_table[seq_row, q // H.PAGE:q // H.PAGE + 1] * H.PAGE + q % H.PAGE)
            v["ctx"].fill_(q + 1)
            v["gslot"].fill_(0)
            v["bt_row"].fill_(seq_row)
            self.hid_in[:1].copy_(r.h[t - 1:t])
            g = self._chain_graph(_bucket(q + k))
            for i in range(1, k):
                g.replay()
                self.drafts[i:i + 1].copy_(r.out_tok[:1])
        return self.drafts[:k]

    def _chain_graph(self, ctx_hint: int):
        """One self-feeding step: forward, then next ids / position / kv slot from the sampled token
        (decode_advance) and the new hidden as the next step's hidden input."""
        r = self.runner
        key = r._pick_splits(1, ctx_hint)
        g = self._chains.get(key)
        if g is None:
            lay = H.StepLayout(1, 1)
            stream = torch.cuda.Stream(device=r.device)
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                saved, saved_h = r.inp.clone(), self.hid_in.clone()
                v = r.views(lay)
                v["gslot"].fill_(-1); v["kv_slot"].fill_(-1); v["ctx"].fill_(1); v["bt_row"].zero_()
                def body():
                    r.step_forward(lay, ctx_hint=ctx_hint, advance=True)
                    self.hid_in[:1].copy_(r.h[:1])
                body()
                stream.synchronize()
                r.inp.copy_(saved)
                v["gslot"].fill_(-1); v["kv_slot"].fill_(-1); v["ctx"].fill_(1); v["bt_row"].zero_()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    body()
                r.inp.copy_(saved)
                self.hid_in.copy_(saved_h)
            torch.cuda.current_stream().wait_stream(stream)
            self._chains[key] = g
        return g


def _bucket(ctx: int) -> int:
    b = 512
    while b < ctx:
        b *= 2
    return b
