"""Model specification for the Qwen3.5 / Qwen3.8 hybrid family (3 Gated-DeltaNet layers : 1
gated full-attention layer), its presets and tensor-parallel sharding of the head counts.

Reference counterpart: ``crates/models/src/formats/qwen35.rs:489-544`` (presets) and
``crates/models/src/model.rs:55-140`` (``ModelSpec::sharded``).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace


@dataclass(frozen=True)
class ModelSpec:
    name: str
    vocab: int
    hidden: int
    inter: int
    n_layers: int
    # full attention
    hq: int
    hkv: int
    hd: int
    rotary_dim: int
    rope_theta: float
    # gated delta net
    nk: int
    kd: int
    nv: int
    vd: int
    conv_k: int = 4
    full_every: int = 4            # layer i is full attention when (i + 1) % full_every == 0
    eps: float = 1e-6
    tied: bool = False
    mrope_section: tuple = (11, 11, 10)
    max_position: int = 262144     # context length the checkpoint was trained for (YaRN's original_max when the profile gives 0)
    rope_yarn: tuple = None        # (factor, original_max, beta_fast, beta_slow, attention_factor) or None = plain rope
    # tensor parallel view (filled by ``sharded``)
    tp_rank: int = 0
    tp_world: int = 1
    kv_replicas: int = 1           # > 1 when world > hkv: several ranks hold the same kv head

    def is_full(self, layer: int) -> bool:
        return (layer + 1) % self.full_every == 0

    @property
    def layer_types(self) -> list[str]:
        return ["full" if self.is_full(i) else "gdn" for i in range(self.n_layers)]

    @property
    def key_dim(self) -> int:
        return self.nk * self.kd

    @property
    def value_dim(self) -> int:
        return self.nv * self.vd

    @property
    def conv_dim(self) -> int:
        return 2 * self.key_dim + self.value_dim

    @property
    def n_full(self) -> int:
        return sum(1 for i in range(self.n_layers) if self.is_full(i))

    @property
    def n_gdn(self) -> int:
        return self.n_layers - self.n_full

    def kv_bytes_per_token(self, kv_elem_bytes: int = 1) -> int:
        return self.n_full * 2 * self.hkv * self.hd * kv_elem_bytes

    def gdn_state_bytes(self) -> int:
        return self.n_gdn * (self.nv * self.kd * self.vd * 4 + self.conv_dim * (self.conv_k - 1) * 4)

    def sharded(self, rank: int, world: int) -> "ModelSpec":
        """Per-rank view: intermediate size, attention heads and GDN heads are cut; hidden and
        vocab are not. With more ranks than kv heads, kv heads are replicated."""
        if world == 1:
            return self
        assert self.inter % world == 0 and self.hq % world == 0 and self.nk % world == 0 and self.nv % world == 0, \
            f"tp world {world} does not divide the head counts of {self.name}"
        if self.hkv % world == 0:
            hkv, rep = self.hkv // world, 1
        else:
            assert world % self.hkv == 0
            hkv, rep = 1, world // self.hkv
        return replace(self, inter=self.inter // world, hq=self.hq // world, hkv=hkv, nk=self.nk // world,
                       nv=self.nv // world, tp_rank=rank, tp_world=world, kv_replicas=rep)


def tiny_hybrid() -> ModelSpec:
    """The CPU reference-numerics configuration (24 layers, hidden 1024)."""
    return ModelSpec(name="tiny-hybrid", vocab=151936, hidden=1024, inter=3584, n_layers=24, hq=8, hkv=2, hd=128,
                     rotary_dim=32, rope_theta=1e7, nk=16, kd=128, nv=16, vd=128)


def qwen_27b() -> ModelSpec:
    """27B hybrid with the benchmark vocabulary (151936)."""
    return ModelSpec(name="qwen3.8-27b", vocab=151936, hidden=5120, inter=17408, n_layers=64, hq=24, hkv=4, hd=256,
                     rotary_dim=64, rope_theta=1e7, nk=16, kd=128, nv=48, vd=128)


def test_hybrid(n_layers: int = 4, hidden: int = 256, vocab: int = 512, mult: int = 1) -> ModelSpec:
    """A few-layer model with the 27B head geometry (hd 256, GVA 3:1) for kernel / engine tests. ``mult`` multiplies every
    head count (2: divisible by a tensor-parallel world of 4, with 2 kv heads replicated over pairs of ranks)."""
    return ModelSpec(name="test-hybrid", vocab=vocab, hidden=hidden, inter=2 * hidden, n_layers=n_layers, hq=6 * mult, hkv=mult,
                     hd=256, rotary_dim=64, rope_theta=1e7, nk=2 * mult, kd=128, nv=6 * mult, vd=128)


PRESETS = {
    "tiny-hybrid": tiny_hybrid,
    "qwen3.8-27b": qwen_27b,
    "test-hybrid": test_hybrid,
    "qwen3.5-0.8b": lambda: ModelSpec(name="qwen3.5-0.8b", vocab=248320, hidden=1024, inter=3584, n_layers=24, hq=8,
                                      hkv=2, hd=256, rotary_dim=64, rope_theta=1e7, nk=16, kd=128, nv=16, vd=128,
                                      tied=True),
    "qwen3.8-27b-full-vocab": lambda: replace(qwen_27b(), name="qwen3.8-27b-full-vocab", vocab=248320),
}


def mrope_section_map(spec: ModelSpec):
    """Per rotary frequency j the position stream it follows (0=T, 1=H, 2=W), interleaved
    ``THWTHW...TT`` as in HF ``apply_interleaved_mrope``."""
    half = spec.rotary_dim // 2
    sec = []
    for j in range(half):
        s = 0
        if j % 3 == 1 and j < spec.mrope_section[1] * 3:
            s = 1
        elif j % 3 == 2 and j < spec.mrope_section[2] * 3:
            s = 2
        sec.append(s)
    return sec
