"""MathLM parameter container and inference entry points for the UV-50M rollout-decode path.

``MathLM`` here holds exactly the parameters of the reference's ``MathLM`` (ultraviolet/model.py:609-640) under the
same names, created and initialised in the same order, so that

* ``torch.manual_seed(s); MathLM(cfg)`` gives bit-identical random-init weights to the reference, and
* ``load_state_dict`` accepts a reference checkpoint unchanged.

It has no training forward.  Inference goes through the B200 decode engine (``ultraviolet_b200.engine``): the methods
``new_state`` / ``prefill`` / ``decode_step`` / ``logits`` / ``fuse_for_inference`` keep the reference's signatures
(model.py:824-1008) so ``DecodeRunner``, ``generate``, ``generate_continuous`` and ``StreamGen`` callers are unchanged.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
from torch import Tensor

from .config import MathConfig, config_from, make_config, PRESETS  # noqa: F401


def _scalar(v: float) -> nn.Parameter:
    return nn.Parameter(torch.tensor(float(v)))


class Attention(nn.Module):
    """Parameters of one attention mixer (model.py:265-287)."""

    kind = "attn"

    def __init__(self, cfg: MathConfig, l: int):
        super().__init__()
        d, hd, H, K = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        self.l, self.H, self.K, self.G, self.hd = l, H, K, H // K, hd
        self.is_global = cfg.is_global(l)
        self.rope = (not self.is_global) or cfg.global_rope
        self.has_ve = cfg.has_ve(l)
        self.wq = nn.Parameter(torch.empty(H * hd, d))
        self.wk = nn.Parameter(torch.empty(K * hd, d))
        self.wv = nn.Parameter(torch.empty(K * hd, d))
        self.wo = nn.Parameter(torch.zeros(d, H * hd))
        self.qkv_scale = _scalar(1.0)
        self.o_scale = _scalar(1.0)
        if self.has_ve:
            self.ve_gate = nn.Parameter(torch.zeros(K, cfg.ve_gate_channels))
        self.gate_ch = cfg.gate_channels
        if self.gate_ch:
            self.attn_gate = nn.Parameter(torch.zeros(H, self.gate_ch))
        if cfg.xsa:
            self.xsa_alpha = nn.Parameter(torch.zeros(H))

    def reset_parameters(self):
        bound = math.sqrt(3) * 0.5 / math.sqrt(self.wq.size(1))
        for w in (self.wq, self.wk, self.wv):
            nn.init.uniform_(w, -bound, bound)
        nn.init.zeros_(self.wo)


class MLP(nn.Module):
    """SwiGLU parameters (model.py:368-382)."""

    def __init__(self, cfg: MathConfig):
        super().__init__()
        d, f = cfg.d_model, cfg.d_ff
        self.w_gate = nn.Parameter(torch.empty(f, d))
        self.w_up = nn.Parameter(torch.empty(f, d))
        self.w_down = nn.Parameter(torch.zeros(d, f))

    def reset_parameters(self):
        bound = math.sqrt(3) * 0.5 / math.sqrt(self.w_gate.size(1))
        nn.init.uniform_(self.w_gate, -bound, bound)
        nn.init.uniform_(self.w_up, -bound, bound)
        nn.init.zeros_(self.w_down)


class Block(nn.Module):
    def __init__(self, cfg: MathConfig, l: int):
        super().__init__()
        self.attn = Attention(cfg, l)
        self.mlp = MLP(cfg)
        self.resid_attn = _scalar(1.0)
        self.post_attn = _scalar(1.0)
        self.resid_mlp = _scalar(1.0)
        self.post_mlp = _scalar(1.0)


class MathLM(nn.Module):
    # Decode implementation switches kept from the reference (model.py:849-851).  On this package every kernel state is
    # the int8 (or 16-bit) slot cache read by the sm_100a kernels; there is no SDPA decode path to fall back to.
    decode_impl = "kernel-int8"
    decode_backend = "b200"
    decode_num_splits = None
    prefill_chunk_tokens = 65536

    def __init__(self, cfg: MathConfig):
        super().__init__()
        cfg = config_from(cfg)
        cfg.check_decode_supported()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.use_ve = any(cfg.has_ve(l) for l in range(cfg.n_layers))
        if self.use_ve:
            self.value_embed = nn.Embedding(cfg.vocab_size, cfg.n_kv_heads * cfg.head_dim)
        self.blocks = nn.ModuleList([Block(cfg, l) for l in range(cfg.n_layers)])
        self._engine = None
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.normal_(self.embed.weight, std=self.cfg.init_std_embed)
        if self.use_ve:
            nn.init.normal_(self.value_embed.weight, std=self.cfg.init_std_ve)
        for b in self.blocks:
            b.attn.reset_parameters()
            b.mlp.reset_parameters()

    # ---- inference API (signatures of model.py:824-1008); bodies live in engine.py
    def fuse_for_inference(self, dtype=torch.bfloat16):
        from .engine import DecodeEngine
        self.eval()
        self._engine = DecodeEngine.from_model(self, dtype)
        return self

    @property
    def engine(self):
        if self._engine is None:
            raise RuntimeError("call fuse_for_inference(dtype) before decoding")
        return self._engine

    def resolve_decode_impl(self, dtype, device) -> str:
        impl = self.decode_impl
        return "kernel-int8" if impl == "auto" else impl

    def new_state(self, batch: int, max_len: int, dtype=None, device=None, ring_extra: int = 0):
        from .fast_decode import KernelDecodeState
        eng = self.engine
        impl = self.resolve_decode_impl(dtype or eng.dtype, device or eng.device)
        if not impl.startswith("kernel-"):
            raise NotImplementedError(f"decode_impl {impl!r}: only the kernel KV states exist in ultraviolet_b200")
        return KernelDecodeState(self.cfg, batch, max_len, dtype or eng.dtype, device or eng.device,
                                 kv_dtype=impl.split("-")[1], ring_extra=ring_extra)

    @torch.no_grad()
    def prefill(self, idx: Tensor, starts: Tensor, st, rows: Tensor | None = None) -> Tensor:
        from .fast_decode import prefill_fast
        return prefill_fast(self, idx, starts, st, rows)

    @torch.no_grad()
    def decode_step(self, tok: Tensor, st, g_len: int, skip_attn: bool = False) -> Tensor:
        from .fast_decode import decode_step_fast
        return decode_step_fast(self, tok, st, g_len, skip_attn, self.decode_num_splits, self.decode_backend)

    def logits(self, h: Tensor) -> Tensor:
        return self.engine.logits(h)
