"""awq-forge: offline conversion of a dense (bf16 / fp16 / fp8 + scale) checkpoint into int4 weights in
the compressed-tensors layout the loader reads (``weight_packed`` / ``weight_scale`` / ``weight_zero_point``,
asymmetric, group 32 or 128).

Two modes:

* ``rtn``   round-to-nearest per group (no data needed);
* ``awq``   activation-aware scaling: for each linear layer a per-input-channel scale ``s = mean|x|^alpha`` is
            searched over ``alpha`` in a grid to minimise the output error ``|| W x - Q(W * s) (x / s) ||`` on
            calibration activations; the scale is folded into the weight before quantisation and its inverse
            is written next to it (``<name>.input_scale_inv``) for the producer of the activations to absorb.

``python -m owl_engine_b200.forge.awq --src DIR --dst DIR [--group 32] [--mode rtn] [--skip lm_head ...]``

Reference counterpart: ``tools/awq-forge/`` (FP8/BF16 -> AWQ INT4 converter, ``convert_rtn_g32.py``).
"""
from __future__ import annotations

import argparse
import json
import shutil
from pathlib import Path

import torch

from ..formats import awq as A
from ..formats import safetensors as ST
from ..ops import quant as Q

QUANT_SUFFIXES = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "gate_proj.weight", "up_proj.weight",
                  "down_proj.weight", "in_proj_qkvz.weight", "in_proj_qkv.weight", "in_proj_z.weight", "out_proj.weight")


def wants_quant(name: str, skip: list[str]) -> bool:
    return name.endswith(QUANT_SUFFIXES) and not any(s in name for s in skip)


def dense_of(name: str, tensors) -> torch.Tensor:
    """fp32 view of a source weight; fp8 weights come with ``<name>_scale_inv`` (per 128 x 128 block) or a scalar scale."""
    w = tensors[name]
    if w.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        w = w.float()
        sname = name.replace(".weight", ".weight_scale_inv")
        if sname in tensors:
            s = tensors[sname].float()
            if s.numel() == 1:
                w = w * s
            else:
                w = w * s.repeat_interleave(128, 0)[:w.shape[0]].repeat_interleave(128, 1)[:, :w.shape[1]]
        return w
    return w.float()


def search_awq_scale(w: torch.Tensor, x: torch.Tensor, group: int, grid: int = 11) -> torch.Tensor:
    """Per-input-channel scale minimising the layer's output error on calibration rows ``x`` [T, K]."""
    act = x.abs().mean(0).clamp_min(1e-5)
    ref = x @ w.t()
    best, best_err = torch.ones_like(act), float("inf")
    for i in range(grid):
        alpha = i / (grid - 1)
        s = act.pow(alpha)
        s = s / (s.max() * s.min()).sqrt()
        deq = Q.quantize_w4(w * s[None], group).dequant() / s[None]
        err = float((x @ deq.t() - ref).pow(2).mean())
        if err < best_err:
            best, best_err = s, err
    return best


def convert(src: str | Path, dst: str | Path, group: int = 32, mode: str = "rtn", skip: list[str] | None = None,
            calib: dict | None = None) -> dict:
    """Convert every shard of ``src`` into ``dst``. ``calib``: layer name -> activations [T, K] for ``mode='awq'``.
    Returns a summary (tensor counts, bytes before / after)."""
    src, dst = Path(src), Path(dst)
    dst.mkdir(parents=True, exist_ok=True)
    skip = skip if skip is not None else ["lm_head", "embed", "mtp", "visual"]
    sd = ST.SafeDir(src)
    names = list(sd.keys())
    tensors = {n: sd.get(n) for n in names}
    out, n_q, before, after = {}, 0, 0, 0
    for n in names:
        t = tensors[n]
        before += t.numel() * t.element_size()
        if n.endswith("_scale_inv"):
            continue
        if t.dim() == 2 and wants_quant(n, skip) and t.shape[1] % group == 0:
            w = dense_of(n, tensors)
            prefix = n[:-len(".weight")]
            if mode == "awq" and calib and prefix in calib:
                s = search_awq_scale(w, calib[prefix].float(), group)
                w = w * s[None]
                out[prefix + ".input_scale_inv"] = (1.0 / s).to(torch.bfloat16)
            out.update(A.to_compressed_tensors(Q.quantize_w4(w, group), prefix))
            n_q += 1
        else:
            out[n] = dense_of(n, tensors).to(torch.bfloat16) if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else t
    for v in out.values():
        after += v.numel() * v.element_size()
    ST.save_file(out, dst / "model.safetensors", metadata={"format": "pt"})
    cfg_p = src / "config.json"
    cfg = json.loads(cfg_p.read_text()) if cfg_p.exists() else {}
    cfg["quantization_config"] = {"quant_method": "compressed-tensors", "format": "pack-quantized",
                                  "config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": group, "symmetric": False,
                                                                            "strategy": "group", "type": "int"}}},
                                  "ignore": skip}
    (dst / "config.json").write_text(json.dumps(cfg, indent=1))
    for extra in ("tokenizer.json", "tokenizer_config.json", "chat_template.jinja", "generation_config.json"):
        if (src / extra).exists():
            shutil.copy(src / extra, dst / extra)
    return {"tensors": len(names), "quantized": n_q, "bytes_before": before, "bytes_after": after}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="awq-forge")
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--group", type=int, default=32, choices=[32, 128])
    ap.add_argument("--mode", default="rtn", choices=["rtn", "awq"])
    ap.add_argument("--skip", nargs="*")
    a = ap.parse_args(argv)
    print(json.dumps(convert(a.src, a.dst, a.group, a.mode, a.skip)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
