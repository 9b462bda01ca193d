"""Model configuration for the UV-50M rollout-decode path.

Field names and defaults follow the reference's ``MathConfig`` (ultraviolet/model.py:28-161) so that a config dict
saved by the reference loads here unchanged.  Only the attention-only architecture is executable in this package: the
optional mixers (conv / GDN), MUDD residual mixing and the hashed bigram table are off in the ``uv-50m-alpha``
preset (docs/math_arch.md:41-42) and are rejected by :func:`MathConfig.check_decode_supported`.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, fields


@dataclass
class MathConfig:
    vocab_size: int = 32768
    d_model: int = 512
    n_layers: int = 16
    n_heads: int = 4
    n_kv_heads: int = 1
    head_dim: int = 128
    d_ff: int = 0
    window: int = 1024
    global_every: int = 4
    global_layers: list | None = None
    rope_frac: float = 0.5
    rope_base: float = 1024.0
    global_rope: bool = False
    attn_scale: float = 0.0
    ve_every: int = 3
    ve_gate_channels: int = 12
    attn_gate_channels: int = 128
    xsa: bool = False
    xsa_eps: float = 1e-4
    mudd: bool = False
    mudd_inter: int = 32
    local_mixer: str = "attn"
    conv_layers: list | None = None
    conv_kernel: int = 4
    gdn_heads: int = 0
    gdn_dk: int = 64
    gdn_dv: int = 128
    softcap: tuple = (23.0, 5.0, 7.5)
    init_std_embed: float = 0.02
    init_std_ve: float = 0.1
    ve_block_pos: list | None = None
    bigram_rows: int = 0
    bigram_dim: int = 0
    bigram_lambda_init: float = 0.1

    def __post_init__(self):
        if not self.d_ff:
            self.d_ff = int(round(2.6 * self.d_model / 64) * 64)
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if not self.attn_scale:
            self.attn_scale = 1.13 / math.sqrt(self.head_dim)
        self.softcap = tuple(float(v) for v in self.softcap)
        if self.global_layers is not None:
            self.global_layers = sorted(int(x) for x in self.global_layers)
        if self.ve_block_pos is not None:
            self.ve_block_pos = sorted(int(x) for x in self.ve_block_pos)

    # ---- layer pattern (ultraviolet/model.py:90-107)
    def is_global(self, l: int) -> bool:
        if self.global_layers is not None:
            return l in self.global_layers
        return self.global_every > 0 and l % self.global_every == self.global_every - 1

    def mixer(self, l: int) -> str:
        if self.is_global(l):
            return "attn"
        if self.conv_layers and l in self.conv_layers:
            return "conv"
        return self.local_mixer

    def has_ve(self, l: int) -> bool:
        if self.ve_block_pos is not None:
            return l % self.global_every in self.ve_block_pos
        return self.ve_every > 0 and l % self.ve_every == 1 % self.ve_every

    @property
    def group(self) -> int:
        return self.n_heads // self.n_kv_heads

    @property
    def rope_pairs(self) -> int:
        return int(self.head_dim * self.rope_frac) // 2

    @property
    def gate_channels(self) -> int:
        return min(self.attn_gate_channels, self.d_model)

    def to_dict(self) -> dict:
        return asdict(self)

    def check_decode_supported(self) -> None:
        """Raise if the config needs a component outside the int8-KV attention decode path."""
        bad = []
        if self.mudd:
            bad.append("mudd")
        if self.bigram_rows:
            bad.append("bigram_rows")
        if any(self.mixer(l) != "attn" for l in range(self.n_layers)):
            bad.append("non-attention mixers")
        if self.global_rope:
            bad.append("global_rope")
        if self.head_dim not in (16, 32, 64, 128):
            bad.append(f"head_dim {self.head_dim}")
        if self.group > 16:
            bad.append(f"group size {self.group} > 16")
        if bad:
            raise NotImplementedError("ultraviolet_b200 decode path does not cover: " + ", ".join(bad))

    def param_counts(self) -> dict:
        d, hd = self.d_model, self.head_dim
        attn = d * hd * (2 * self.n_heads + 2 * self.n_kv_heads)
        nonemb = self.n_layers * (attn + 3 * d * self.d_ff)
        embed = self.vocab_size * d
        ve = self.vocab_size * self.n_kv_heads * hd if any(self.has_ve(l) for l in range(self.n_layers)) else 0
        return {"non_embedding": nonemb, "embedding_tied": embed, "value_embedding": ve,
                "total_with_tied_embed": nonemb + embed, "total_incl_ve": nonemb + embed + ve}


# Presets used on this path (ultraviolet/model.py:164-181): the production model and the reference tests' tiny model.
PRESETS: dict[str, dict] = {
    "uv-50m-alpha": dict(d_model=640, n_layers=10, n_heads=8, n_kv_heads=1, head_dim=64, d_ff=1664, global_every=5,
                         window=256, xsa=True),
    "tiny": dict(vocab_size=512, d_model=64, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                 window=8, global_every=2, attn_gate_channels=16, ve_gate_channels=4),
}


def make_config(name: str, **over) -> MathConfig:
    kw = dict(PRESETS[name])
    kw.update({k: v for k, v in over.items() if v is not None})
    return MathConfig(**kw)


def config_from(obj) -> MathConfig:
    """Build a MathConfig from a reference ``MathConfig`` instance, a dict, or one of ours."""
    if isinstance(obj, MathConfig):
        return obj
    src = obj if isinstance(obj, dict) else {f.name: getattr(obj, f.name) for f in fields(MathConfig)
                                             if hasattr(obj, f.name)}
    names = {f.name for f in fields(MathConfig)}
    return MathConfig(**{k: v for k, v in src.items() if k in names})
