"""Kernel registry: one table row per exported launcher of the native CUDA library.

Every row names the entry symbol, its source file, the op family, whether the launch may be recorded
into a CUDA graph (no host synchronisation, no allocation, fixed launch geometry for fixed shapes),
whether the result is bit-reproducible run to run, and the instruction generation the kernel is
written for. ``cross_check`` parses the ``OWL_API`` declarations of the ``.cu`` sources and verifies
that (a) every exported symbol has a row and every row an exported symbol, (b) the ctypes signature
registered in ``ops.kernels`` has as many parameters as the C declaration. The unit tests run it, so a
launcher cannot change its argument list without the binding noticing.

Reference counterpart: ``crates/kernels/src/{spec,registry,cu_sig}.rs`` (KernelSpec table and the
``.cu`` signature cross-check), ``admit.rs`` (per-architecture admission: here one architecture).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from pathlib import Path

CSRC = Path(__file__).resolve().parents[1] / "csrc"
ARCH = "sm_100a"


@dataclass(frozen=True)
class KernelSpec:
    entry: str
    src: str
    family: str
    capture: bool = True          # safe inside CUDA graph capture
    deterministic: bool = True
    gen: str = "simt"             # simt | mma.sync | dp4a | tcgen05 | tma | p2p


_T = [
    # weight streaming / GEMM
    KernelSpec("owl_w4a16_skinny", "gemv.cu", "gemv", gen="dp4a+mma.sync+bulk-copy"),
    KernelSpec("owl_w4a16_skinny_norm", "gemv.cu", "gemv", gen="dp4a+mma.sync+bulk-copy"),
    KernelSpec("owl_w4a16_skinny_a8", "gemv.cu", "gemv", gen="dp4a+mma.sync+bulk-copy"),
    KernelSpec("owl_bf16_skinny", "gemv.cu", "gemv", gen="mma.sync+bulk-copy"),
    KernelSpec("owl_w8a16_skinny", "gemv.cu", "gemv", gen="mma.sync+bulk-copy"),
    KernelSpec("owl_skinny_status", "gemv.cu", "status", capture=False),
    KernelSpec("owl_w4_fma", "gemv_fma.cu", "gemv", gen="hfma2+bulk-copy"),
    KernelSpec("owl_w4_fma_tp", "gemv_fma.cu", "gemv", gen="hfma2+bulk-copy+p2p"),
    KernelSpec("owl_fma_status", "gemv_fma.cu", "status", capture=False),
    KernelSpec("owl_w4a16_stream_tc", "gemv_tc.cu", "gemv", gen="tcgen05+tmem+bulk-copy"),
    KernelSpec("owl_stream_tc_status", "gemv_tc.cu", "status", capture=False),
    KernelSpec("owl_w4a16_gemm_tc", "gemm_tc.cu", "gemm", gen="tcgen05+tmem+tma"),
    KernelSpec("owl_f16_gemm_tc", "gemm_tc.cu", "gemm", gen="tcgen05+tmem+tma"),
    KernelSpec("owl_gemm_status", "gemm_tc.cu", "status", capture=False),
    KernelSpec("owl_f16_gemm_persist", "gemm_dense.cu", "gemm", gen="tcgen05+tmem+tma"),
    KernelSpec("owl_f16_gemm_persist_f16out", "gemm_dense.cu", "gemm", gen="tcgen05+tmem+tma"),
    KernelSpec("owl_f16_gemm_ag", "gemm_dense.cu", "gemm", gen="tcgen05+tmem+tma+p2p"),
    KernelSpec("owl_f16_gemm_rs", "gemm_dense.cu", "gemm", gen="tcgen05+tmem+tma+p2p"),
    KernelSpec("owl_e4m3_gemm", "gemm_dense.cu", "gemm", gen="tcgen05+tmem+tma"),
    KernelSpec("owl_gemm_dense_status", "gemm_dense.cu", "status", capture=False),
    KernelSpec("owl_gemm_dense_set_scratch", "gemm_dense.cu", "status", capture=False),
    KernelSpec("owl_nvfp4_gemm", "gemm_nvfp4.cu", "gemm", gen="tcgen05.block_scale+tmem+tma"),
    KernelSpec("owl_nvfp4_quant_rows", "gemm_nvfp4.cu", "quant"),
    KernelSpec("owl_gemm_nvfp4_status", "gemm_nvfp4.cu", "status", capture=False),
    KernelSpec("owl_attn_tc", "attn_tc.cu", "attn", gen="tcgen05+tmem+tma"),
    KernelSpec("owl_attn_tc_status", "attn_tc.cu", "status", capture=False),
    KernelSpec("owl_vis_layernorm", "vision.cu", "vision"),
    KernelSpec("owl_vis_bias_act", "vision.cu", "vision"),
    KernelSpec("owl_vis_pos_embed", "vision.cu", "vision"),
    KernelSpec("owl_vis_rope", "vision.cu", "vision"),
    KernelSpec("owl_vis_attn", "vision.cu", "vision", gen="mma.sync"),
    KernelSpec("owl_w4_dequant", "dequant.cu", "load"),
    KernelSpec("owl_quant_e4m3_rows", "dequant.cu", "load"),
    KernelSpec("owl_kv_pages_gather", "kvmove.cu", "store"),
    KernelSpec("owl_kv_pages_scatter", "kvmove.cu", "store"),
    KernelSpec("owl_mean_k_block", "kvmem.cu", "select"),
    KernelSpec("owl_mean_k_block_fmt", "kvmem.cu", "select"),
    KernelSpec("owl_kvscore", "kvmem.cu", "select"),
    KernelSpec("owl_kvscore_softmax", "kvmem.cu", "select"),
    KernelSpec("owl_dflash_conv", "dflash.cu", "draft"),
    KernelSpec("owl_dflash_norm_rope", "dflash.cu", "draft"),
    KernelSpec("owl_dflash_nc_attn", "dflash.cu", "draft"),
    KernelSpec("owl_dflash_select", "dflash.cu", "draft"),
    KernelSpec("owl_nvfp4_gemv", "lowbit.cu", "gemv"),
    KernelSpec("owl_nvfp4_gemv_res", "lowbit.cu", "gemv"),
    KernelSpec("owl_nvfp4_gemv_rows", "lowbit.cu", "gemv"),
    KernelSpec("owl_nvfp4_dequant_rows", "lowbit.cu", "load"),
    KernelSpec("owl_act_unpack", "lowbit.cu", "elem"),
    KernelSpec("owl_add_rows", "lowbit.cu", "elem"),
    KernelSpec("owl_nvfp4_dequant", "lowbit.cu", "load"),
    KernelSpec("owl_nvfp4_quant_act", "lowbit.cu", "quant"),
    KernelSpec("owl_gguf_dequant", "lowbit.cu", "load"),
    KernelSpec("owl_gguf_set_grids", "lowbit.cu", "load", capture=False),
    KernelSpec("owl_gguf_gemv", "lowbit.cu", "gemv"),
    # elementwise / norms / sampling
    KernelSpec("owl_rmsnorm_pack", "elem.cu", "norm"),
    KernelSpec("owl_act_pack", "elem.cu", "quant"),
    KernelSpec("owl_silu_mul", "elem.cu", "act"),
    KernelSpec("owl_sigmoid_gate", "elem.cu", "act"),
    KernelSpec("owl_embed", "elem.cu", "embed"),
    KernelSpec("owl_argmax", "elem.cu", "sample"),
    KernelSpec("owl_argmax_noalloc", "elem.cu", "sample"),
    KernelSpec("owl_decode_advance", "elem.cu", "step"),
    KernelSpec("owl_topk", "sample.cu", "sample"),
    KernelSpec("owl_topk_merge", "sample.cu", "sample"),
    # GDN
    KernelSpec("owl_gdn_decode", "gdn.cu", "gdn", gen="simt+cluster-dsmem"),
    KernelSpec("owl_gdn_conv_fwd", "gdn.cu", "gdn"),
    KernelSpec("owl_gdn_scan", "gdn.cu", "gdn"),
    KernelSpec("owl_gdn_scan_split", "gdn.cu", "gdn", gen="simt+cp.async"),
    KernelSpec("owl_gdn_norm_gate", "gdn.cu", "gdn"),
    KernelSpec("owl_gdn_chunk_scan", "gdn_chunk.cu", "gdn", gen="mma.sync+cp.async"),
    KernelSpec("owl_gdn_chunk_work_bytes", "gdn_chunk.cu", "status", capture=False),
    KernelSpec("owl_l2_prefetch", "prefetch.cu", "elem", gen="bulk-prefetch"),
    # attention / KV
    KernelSpec("owl_qknorm_rope_insert", "attn.cu", "attn"),
    KernelSpec("owl_paged_attn", "attn.cu", "attn", gen="mma.sync"),
    KernelSpec("owl_qknorm_rope_insert_i8", "attn.cu", "attn"),
    KernelSpec("owl_paged_attn_i8", "attn.cu", "attn", gen="mma.sync"),
    KernelSpec("owl_qknorm_rope_insert_f16", "attn.cu", "attn"),
    KernelSpec("owl_paged_attn_f16", "attn.cu", "attn", gen="mma.sync"),
    KernelSpec("owl_attn_reduce", "attn.cu", "attn"),
    KernelSpec("owl_kv_gather", "attn_gemm.cu", "attn"),
    KernelSpec("owl_causal_softmax", "attn_gemm.cu", "attn"),
    KernelSpec("owl_attn_gate", "attn_gemm.cu", "attn"),
    KernelSpec("owl_q_group", "attn_gemm.cu", "attn"),
    # collectives over peer memory
    KernelSpec("owl_ar_residual_norm", "comm.cu", "comm", gen="p2p+multimem"),
    KernelSpec("owl_ar_inplace", "comm.cu", "comm", gen="p2p+multimem"),
    KernelSpec("owl_push_residual_norm", "comm.cu", "comm", gen="p2p"),
    KernelSpec("owl_rs_norm_ag", "comm.cu", "comm", gen="p2p"),
    KernelSpec("owl_w4a16_skinny_push", "gemv.cu", "gemv", gen="dp4a+mma.sync+bulk-copy+p2p"),
    KernelSpec("owl_argmax_merge", "comm.cu", "comm", gen="p2p"),
    KernelSpec("owl_comm_wait_probe", "comm.cu", "comm", gen="p2p"),
    KernelSpec("owl_comm_status", "comm.cu", "status", capture=False),
]
TABLE = {k.entry: k for k in _T}

_DECL = re.compile(r"OWL_API\s+int\s+(owl_\w+)\s*\(([^)]*)\)", re.S)


def declared() -> dict[str, tuple[str, int]]:
    """entry -> (source file, parameter count) from the OWL_API declarations under csrc/."""
    out = {}
    for f in sorted(CSRC.glob("*.cu")):
        text = re.sub(r"#ifdef OWL_VT_TRACE.*?#endif", "", f.read_text(), flags=re.S)   # tuning-only exports are not built
        for name, args in _DECL.findall(text):
            args = args.strip()
            n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
            out[name] = (f.name, n)
    return out


def cross_check() -> list[str]:
    """Mismatches between the sources, this table and the ctypes signatures (empty = consistent)."""
    from . import kernels as K
    from . import gemm_tc, nvfp4_tc  # noqa: F401  (register their signatures)
    from ..models import dflash2, vision  # noqa: F401

    vision._bind_vision(K)
    from ..parallel import symm  # noqa: F401
    from ..store import select

    select._K()
    K.register("owl_argmax_noalloc", [K._P, K._I, K._I, K._I, K._P, K._I, K._P])     # bound by its own test through the C symbol

    problems = []
    decl = declared()
    for name, (src, n) in decl.items():
        row = TABLE.get(name)
        if row is None:
            problems.append(f"{name} ({src}) is exported but has no registry row")
            continue
        if row.src != src:
            problems.append(f"{name}: registry says {row.src}, declared in {src}")
        sig = K._SIGS.get(name)
        if sig is not None and len(sig) != n:
            problems.append(f"{name}: ctypes signature has {len(sig)} parameters, the C declaration {n}")
        if sig is None and n > 0:
            # without argtypes ctypes passes Python ints as 32-bit C ints: a device pointer would be cut in half
            problems.append(f"{name}: {n} parameters but no ctypes signature registered")
    for name in TABLE:
        if name not in decl:
            problems.append(f"{name}: registry row without an exported symbol")
    return problems


def admit(family: str) -> list[KernelSpec]:
    """Kernels of a family that this build admits (one architecture: everything in the table)."""
    return [k for k in _T if k.family == family]
