"""Decode engine: fused inference weights in one pointer-stable arena + the per-step kernel sequence.

The arena plays the role of the reference's ``_fused`` dictionaries (Attention.fuse / MLP.fuse, ultraviolet/model.py:
289-300, :384-386): per layer ``wqkv = cat(wq, wk, wv) * qkv_scale``, ``wo * o_scale``, ``gu = cat(w_gate, w_up)``,
``down``, the gates, ``tanh(xsa_alpha)`` and the four residual lambdas, plus the (tied) embedding and the value
embedding.  Everything of activation dtype lives in ONE flat tensor so that a weight refresh is an in-place write (or
one NCCL broadcast) and every captured CUDA graph keeps reading the same addresses -- the contract of
``sync_weights_inplace`` (scripts/rl_stream.py:23-36).

One decode step (``step``) is the kernel sequence of ``decode_step_fast`` (ultraviolet/kernels/fast_decode.py:272-334):
per layer  GEMM(qkv) -> uv_qkv_post (VE gate, QK norm, RoPE, int8 append) -> uv_decode_attn (+XSA, head gate)
-> GEMM(wo) -> uv_resid_norm -> GEMM(gate|up) -> uv_swiglu -> GEMM(down) -> uv_resid_norm, then the tied LM head and
uv_sample.  GEMMs are plain library calls (cuBLAS through torch.mm into preallocated outputs); everything else is
libuvdecode.  Nothing here allocates after warm-up, so the whole step captures into one CUDA graph.
"""
from __future__ import annotations

import ctypes as C
import os

import torch
from torch import Tensor

from . import _lib
from .config import MathConfig
from .kernels._util import DTYPE_CODE, stream_ptr
from .kernels.decode_attn import attn_launch, default_splits, workspace_for


def _align(n: int, a: int = 128) -> int:
    return (n + a - 1) // a * a


class DecodeEngine:
    def __init__(self, cfg: MathConfig, dtype: torch.dtype, device):
        cfg.check_decode_supported()
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("decode engine computes in float16 or bfloat16")
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("ultraviolet_b200 decodes on CUDA devices only (there is no CPU path)")
        d, hd, H, K, f = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff
        self.use_ve = any(cfg.has_ve(l) for l in range(cfg.n_layers))
        # ---- arena layout (element offsets, 128-element aligned so every matrix starts on a 256-byte boundary)
        shapes = [("embed", (cfg.vocab_size, d))]
        if self.use_ve:
            shapes.append(("value_embed", (cfg.vocab_size, K * hd)))
        for l in range(cfg.n_layers):
            shapes += [(f"l{l}.wqkv", ((H + 2 * K) * hd, d)), (f"l{l}.wo", (d, H * hd)), (f"l{l}.gu", (2 * f, d)),
                       (f"l{l}.down", (d, f))]
            if cfg.has_ve(l):
                shapes.append((f"l{l}.ve_gate", (K, cfg.ve_gate_channels)))
            if cfg.gate_channels:
                shapes.append((f"l{l}.attn_gate", (H, cfg.gate_channels)))
        off, self.layout = 0, {}
        for name, shp in shapes:
            n = 1
            for s in shp:
                n *= s
            self.layout[name] = (off, shp)
            off = _align(off + n)
        self.arena = torch.zeros(off, dtype=dtype, device=self.device)
        # fp32 side arena: per layer 4 lambdas (rounded to dtype) + tanh(xsa_alpha) (H) ; then rope inv_freq
        self.n32_layer = 4 + H
        self.arena32 = torch.zeros(cfg.n_layers * self.n32_layer + max(cfg.rope_pairs, 1), dtype=torch.float32,
                                   device=self.device)
        self.w = {name: self.arena[o:o + torch.Size(shp).numel()].view(shp) for name, (o, shp) in self.layout.items()}
        self.lambdas = [self.arena32[l * self.n32_layer:l * self.n32_layer + 4] for l in range(cfg.n_layers)]
        self.xsa = [self.arena32[l * self.n32_layer + 4:(l + 1) * self.n32_layer] for l in range(cfg.n_layers)]
        self.inv_freq = self.arena32[cfg.n_layers * self.n32_layer:][:cfg.rope_pairs]
        # Rotary.inv_freq (model.py:203-204): (1 / base) ** linspace(0, 1, n_pairs), fp32
        if cfg.rope_pairs:
            self.inv_freq.copy_((1.0 / cfg.rope_base) ** torch.linspace(0, 1, cfg.rope_pairs, dtype=torch.float32))
        self._scratch: dict[int, dict] = {}
        self.version = 0
        # GEMMs with fused epilogues (csrc/gemm_fused.cu).  Correct, but measured SLOWER than cuBLAS + the separate row
        # kernels on B200 at decode batch sizes (per pair 8-20 us against 6-8 us: four warps of straight-line code per
        # SM stall on instruction fetch and on the serial MMA chain), so the path is opt-in: UVDECODE_FUSED_GEMM=1.
        self.fused_gemm_ok = (hd == 64 and d % 80 == 0 and d // 80 <= 8 and f % 64 == 0 and d % 64 == 0
                              and (H * hd) % 64 == 0)
        self.fused_gemm = os.environ.get("UVDECODE_FUSED_GEMM", "0") == "1" and self.fused_gemm_ok
        # uv_qkv_attn: one launch for the QKV post-processing + cache append + attention of a layer.  Opt-in: results
        # are bit-identical, but inside the decode step the one launch measured ~1 us per layer SLOWER than the two
        # (four warps per row do serially what uv_qkv_post spreads over ten, and the longer kernel pays more cold
        # instruction fetch), although it is ~0.5 us faster when timed back to back in isolation.
        self.qkv_in_attn = os.environ.get("UVDECODE_QKV_IN_ATTN", "0") == "1"
        # cos / sin of pos * inv_freq once per step (uv_embed_norm_rope) instead of in every layer's q / k rotation
        self.rope_table = os.environ.get("UVDECODE_ROPE_TABLE", "1") != "0"
        # attention output gates computed by uv_qkv_post (they depend on xn only) instead of in the attention epilogue
        self.gate_pre = os.environ.get("UVDECODE_GATE_PRE", "1") != "0"
        # GEMMs on this library's own tcgen05 kernels with the row kernels in their epilogues and the RMS norms
        # deferred into the consuming GEMM (csrc/gemm_sw.cu): 5 launches per layer instead of 9.  bf16 only, shapes of
        # the uv-50m family (head_dim 64, every GEMM dimension a multiple of 64 / 128).  UVDECODE_TC_GEMM=0 turns it
        # off (library GEMMs + row kernels).
        self.tc_gemm_ok = (dtype == torch.bfloat16 and hd == 64 and d % 128 == 0 and (H * hd) % 64 == 0
                           and f % 64 == 0 and (H + 2 * K) % 2 == 0 and d // 128 <= 32
                           and (cfg.rope_pairs == 0 or self.rope_table))
        self.tc_gemm = os.environ.get("UVDECODE_TC_GEMM", "0") == "1" and self.tc_gemm_ok
        self.tc_hints = {k: tuple(int(v) for v in os.environ.get(f"UVDECODE_TC_{k.upper()}", d_).split(","))
                         for k, d_ in (("qkv", "0,0"), ("wo", "0,0"), ("gu", "0,0"), ("down", "0,0"))}
        # Folded residual stream (default): the step carries y = x / s_l, s_l the running product of the residual
        # lambdas, so that  h = l0 x + l1 a  becomes  y += a'  with l1 / s folded into wo (and into w_down for the MLP
        # branch) when the weights are fused.  Every consumer of the stream is an RMS norm, which does not see the
        # scale, and the norm itself is deferred into the kernel that follows the consuming GEMM (uv_qkv_post_args
        # with xn_raw, uv_swiglu_rs).  The two residual + norm launches of a layer disappear: the residual add is
        # the GEMM's own accumulate (C += A . B), 7 launches per layer instead of 9.  UVDECODE_FOLD=0: the
        # reference's literal op order (separate uv_resid_norm launches).
        self.fold = (os.environ.get("UVDECODE_FOLD", "1") != "0" and not self.fused_gemm and not self.tc_gemm
                     and not self.qkv_in_attn and d % 8 == 0)
        # Folded step only: the QKV projection and everything uv_qkv_post does in ONE launch of this library's tcgen05
        # kernel (uv_gemm_sw_qkv with self-computed row sums of squares) instead of library GEMM + uv_qkv_post_args.
        # "1": with the PDL attribute on that launch, "nopdl": without, "0": off.
        self.sw_qkv = os.environ.get("UVDECODE_SW_QKV", "0")
        if not (self.fold and self.tc_gemm_ok and d // 64 <= 12):
            self.sw_qkv = "0"
        self.n_sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        _lib.lib()

    # ------------------------------------------------------------------------------------------------ weights
    @classmethod
    def from_model(cls, model, dtype=torch.bfloat16) -> "DecodeEngine":
        from .config import config_from
        dev = model.embed.weight.device
        eng = cls(config_from(model.cfg), dtype, dev)
        eng.load_from(model)
        return eng

    @torch.no_grad()
    def load_from(self, model) -> None:
        """(Re)compute every fused weight from the model's parameters INTO the existing arena (same formulas and
        rounding as Attention.fuse / MLP.fuse; pointers never change)."""
        cfg, dt, w = self.cfg, self.dtype, self.w
        w["embed"].copy_(model.embed.weight)
        if self.use_ve:
            w["value_embed"].copy_(model.value_embed.weight)
        scale = 1.0   # s_l: the residual stream the kernels carry is x / s_l (folded mode)
        for l, blk in enumerate(model.blocks):
            at, mlp = blk.attn, blk.mlp
            w[f"l{l}.wqkv"].copy_((torch.cat([at.wq, at.wk, at.wv]) * at.qkv_scale).to(dt))
            lam_h = [float(v.detach().to(dt).float()) for v in (blk.resid_attn, blk.post_attn, blk.resid_mlp,
                                                                 blk.post_mlp)]
            if self.fold:
                if min(abs(lam_h[0]), abs(lam_h[2])) < 2.0 ** -6:
                    raise ValueError(f"layer {l}: a residual lambda is ~0, the folded residual stream cannot "
                                     "represent it; set UVDECODE_FOLD=0")
                scale *= lam_h[0]
                w[f"l{l}.wo"].copy_((at.wo.float() * float(at.o_scale) * (lam_h[1] / scale)).to(dt))
                scale *= lam_h[2]
                w[f"l{l}.down"].copy_((mlp.w_down.float() * (lam_h[3] / scale)).to(dt))
                lim = 2.0 ** (24 if dt == torch.bfloat16 else 6)   # fp16 has 5 exponent bits: keep y near x
                if not (1.0 / lim < abs(scale) < lim):
                    raise ValueError("the product of the residual lambdas leaves the range the folded residual "
                                     "stream keeps in half precision; set UVDECODE_FOLD=0")
            else:
                w[f"l{l}.wo"].copy_((at.wo * at.o_scale).to(dt))
                w[f"l{l}.down"].copy_(mlp.w_down.to(dt))
            w[f"l{l}.gu"].copy_(torch.cat([mlp.w_gate, mlp.w_up]).to(dt))
            if cfg.has_ve(l):
                w[f"l{l}.ve_gate"].copy_(at.ve_gate.to(dt))
            if cfg.gate_channels:
                w[f"l{l}.attn_gate"].copy_(at.attn_gate.to(dt))
            lam = torch.stack([blk.resid_attn, blk.post_attn, blk.resid_mlp, blk.post_mlp]).detach()
            self.lambdas[l].copy_(lam.to(dt).float())  # Block.finish casts each scalar to the activation dtype
            if cfg.xsa:
                self.xsa[l].copy_(torch.tanh(at.xsa_alpha.detach().float()))
        self.version += 1

    def nbytes(self) -> int:
        return self.arena.numel() * self.arena.element_size() + self.arena32.numel() * 4

    # ------------------------------------------------------------------------------------------------ scratch
    BIG_ROWS = 2048  # batches above this (packed prompt prefill) share bucketed buffers instead of one set per size

    def scratch(self, B: int, tag: str = "") -> dict:
        """The buffers of a B-row trunk call.  tag names a second, independent family of buffers for calls that may
        run beside the untagged ones on another stream (admission passes next to decode steps)."""
        if B > self.BIG_ROWS:
            # prefill batches come in every size: one allocation per 4096-row bucket, handed out as [:B] views
            cap = (B + 4095) // 4096 * 4096
            big = self._scratch.get((cap, tag) if tag else cap) or self.scratch_exact(cap, tag)
            return {k: (v[:B] if isinstance(v, Tensor) and v.dim() >= 1 and v.size(0) == cap and k not in
                        ("flags", "status", "oob") else v) for k, v in big.items()}
        return self.scratch_exact(B, tag)

    def scratch_exact(self, B: int, tag: str = "") -> dict:
        key = (B, tag) if tag else B
        s = self._scratch.get(key)
        if s is None:
            cfg, dt, dev = self.cfg, self.dtype, self.device
            d, hd, H, K, f = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff
            e = lambda *shape: torch.empty(*shape, dtype=dt, device=dev)
            s = dict(x=e(B, d), xn=e(B, d), qkv=e(B, (H + 2 * K) * hd), z=e(B, H * hd), a=e(B, d), h=e(B, d),
                     hn=e(B, d), gu=e(B, 2 * f), act=e(B, f), m=e(B, d),
                     tok=torch.zeros(B, dtype=torch.int64, device=dev),
                     logp=torch.zeros(B, dtype=torch.float32, device=dev),
                     counters=torch.zeros(B * K, dtype=torch.int32, device=dev),
                     flags=torch.zeros(2, dtype=torch.int32, device=dev),
                     rope_cs=torch.zeros(B, 2 * max(cfg.rope_pairs, 1), dtype=torch.float32, device=dev),
                     gate=torch.zeros(B, H, dtype=torch.float32, device=dev), ws={},
                     ss_x=torch.zeros(max(d // 128, 1), B, dtype=torch.float32, device=dev),
                     ss_h=torch.zeros(max(d // 128, 1), B, dtype=torch.float32, device=dev))
            # device words the kernels raise on silent failures: [0] attention status (bit 0: a bulk copy did not
            # land in time, outputs of that launch are undefined), [1] count of skipped out-of-range KV writes
            s["status"], s["oob"] = s["flags"][0:1], s["flags"][1:2]
            self._scratch[key] = s
        return s

    def device_status(self, B: int | None = None) -> dict:
        """The failure words of the scratch set of batch size B (default: all sets), one small D2H each."""
        out = {"attn_status": 0, "kv_oob": 0}
        for b, s in self._scratch.items():
            if B is None or b == B or (isinstance(b, tuple) and b[0] == B):
                st, oob = s["flags"].tolist()
                out["attn_status"] |= st
                out["kv_oob"] += oob
        return out

    def check_status(self, B: int | None = None) -> dict:
        """Raise if a kernel of this engine flagged a silent failure since the words were last cleared: outputs of
        a launch whose attention status bit is set are undefined, and a skipped KV write corrupts later tokens."""
        d = self.device_status(B)
        if d["attn_status"] or d["kv_oob"]:
            for b, s in self._scratch.items():
                if B is None or b == B or (isinstance(b, tuple) and b[0] == B):
                    s["flags"].zero_()
            raise _lib.UvError(f"decode kernels reported a device-side failure: attention status word "
                               f"{d['attn_status']:#x} (bit 0 = a cache tile copy timed out), {d['kv_oob']} KV "
                               "cache writes skipped as out of range; tokens produced since the last check are invalid")
        return d

    def launches_per_step(self) -> int:
        """Kernel launches of one trunk + head call (the sampler is one more)."""
        n = self.cfg.n_layers
        if self.tc_gemm:
            return 1 + 5 * n + 2
        if self.fused_gemm:
            return 1 + 5 * n + 1
        if self.fold:
            return 1 + (6 if self.sw_qkv != "0" else 7) * n + 2
        return 1 + (8 if self.qkv_in_attn else 9) * n + 1

    def _workspace(self, s: dict, B: int, splits: int) -> Tensor | None:
        if splits <= 1:
            return None
        ws = s["ws"].get(splits)
        if ws is None:
            cfg = self.cfg
            ws = s["ws"][splits] = workspace_for(B, cfg.n_kv_heads, cfg.group, cfg.head_dim, splits, self.device)
        return ws

    # ------------------------------------------------------------------------------------------------ one step
    def trunk(self, tok: Tensor, st, pos: Tensor, starts: Tensor, g_len: int | None = None,
              num_splits: dict | None = None, row_map: Tensor | None = None, skip_attn: bool = False,
              packed: dict | None = None, scratch_tag: str = "") -> Tensor:
        """One token for every batch entry: writes K/V at `pos` and returns the final normed hidden (B, d) (a view
        of engine scratch, overwritten by the next call).  pos/starts are batch-indexed (B,) int64; row_map
        optionally maps batch entries to cache rows.

        packed (prompt prefill): the batch entries are the tokens of whole prompts packed back to back --
        dict(cu=int32 (n + 1,) first row of each prompt, tile_cu=int32 (n + 1,) first 16-token tile of each prompt,
        n_seq, max_tiles, last_pos=int64 (B,) last position of the entry's prompt).  Attention then runs over the
        unquantised keys / values of the batch itself (uv_prefill_attn) instead of the cache, and ring caches keep
        only the newest positions of each prompt."""
        cfg, lib, dt = self.cfg, _lib.lib(), DTYPE_CODE[self.dtype]
        B = tok.size(0)
        s = self.scratch(B, scratch_tag)
        d, hd, H, K, f = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff
        sp = stream_ptr(self.device)
        w = self.w
        ns = num_splits or {}
        rm = row_map.data_ptr() if row_map is not None else None
        fused = self.fused_gemm and packed is None
        qkv_in_attn = self.qkv_in_attn and packed is None
        fold = self.fold
        if self.tc_gemm and not fused and not qkv_in_attn and B <= self.BIG_ROWS:
            return self._trunk_tc(tok, st, pos, starts, g_len, ns, rm, row_map, skip_attn, packed)
        with torch.cuda.device(self.device):
            use_table = self.rope_table and not fused and cfg.rope_pairs > 0
            if use_table:  # one cos / sin table per step instead of cosf / sinf in every layer's prologue
                _lib.check(lib.uv_embed_norm_rope(tok.data_ptr(), w["embed"].data_ptr(), dt, cfg.vocab_size, d,
                                                  s["x"].data_ptr(), s["xn"].data_ptr(), B, pos.data_ptr(),
                                                  self.inv_freq.data_ptr(), cfg.rope_pairs, s["rope_cs"].data_ptr(),
                                                  sp), "uv_embed_norm_rope")
            else:
                _lib.check(lib.uv_embed_norm(tok.data_ptr(), w["embed"].data_ptr(), dt, cfg.vocab_size, d,
                                             s["x"].data_ptr(), s["xn"].data_ptr(), B, sp), "uv_embed_norm")
            x, xn, h, hn = s["x"], s["xn"], s["h"], s["hn"]
            qkv3 = s["qkv"].view(B, H + 2 * K, hd)
            q, v_cur = qkv3[:, :H], qkv3[:, H + K:]
            z3 = s["z"].view(B, H, hd)
            for l in range(cfg.n_layers):
                glob = cfg.is_global(l)
                kc, vc, ks, vs = st.k[l], st.v[l], st.k_scale[l], st.v_scale[l]
                S = kc.size(2)
                ve_gate = w[f"l{l}.ve_gate"].data_ptr() if cfg.has_ve(l) else None
                pre = gate_vals = None
                rope = (not glob) or cfg.global_rope
                post_args = (tok.data_ptr(), w["value_embed"].data_ptr() if self.use_ve else None, ve_gate,
                             self.inv_freq.data_ptr() if rope and cfg.rope_pairs else None, pos.data_ptr(),
                             kc.data_ptr(), vc.data_ptr(), ks.data_ptr(), vs.data_ptr(), rm, s["oob"].data_ptr(), dt,
                             cfg.vocab_size, B, H, K, hd, d, S, kc.stride(1) // hd, int(not glob),
                             cfg.ve_gate_channels, cfg.rope_pairs, sp)
                if fused:
                    _lib.check(lib.uv_gemm_qkv(xn.data_ptr(), d, w[f"l{l}.wqkv"].data_ptr(), s["qkv"].data_ptr(),
                                               *post_args), "uv_gemm_qkv")
                else:
                    gin = x if fold else xn   # folded: the GEMM reads the un-normalised stream, uv_qkv_post norms
                    sw_qkv = (fold and self.sw_qkv != "0" and packed is None and not qkv_in_attn and B <= 1024
                              and (use_table or not (rope and cfg.rope_pairs)))
                    if not sw_qkv:
                        torch.mm(gin, w[f"l{l}.wqkv"].t(), out=s["qkv"])
                    qa = _lib.QkvArgs()
                    (qa.qkv, qa.xn, qa.tok, qa.value_embed, qa.ve_gate, qa.inv_freq, qa.pos, qa.k_cache,
                     qa.v_cache, qa.k_scale, qa.v_scale, qa.row_map, qa.oob_count, qa.dtype, qa.vocab,
                     qa.B, qa.H, qa.K, qa.hd, qa.d, qa.S, qa.S_alloc, qa.ring, qa.ve_ch,
                     qa.n_pairs) = (s["qkv"].data_ptr(), gin.data_ptr(), *post_args[:-1])
                    qa.xn_raw = int(fold)
                    qa.rope_cs = s["rope_cs"].data_ptr() if use_table else None
                    if packed is not None:
                        qa.last_pos = packed["last_pos"].data_ptr()
                    if qkv_in_attn:  # the attention launch below does uv_qkv_post's work in its prologue
                        pre = qa
                    else:
                        if cfg.gate_channels and (self.gate_pre or packed is not None or fold):  # depend on xn only:
                            qa.gate_w = w[f"l{l}.attn_gate"].data_ptr()  # computed off the attention kernel's tail
                            qa.gate_out, qa.gate_ch = s["gate"].data_ptr(), cfg.gate_channels
                            gate_vals = s["gate"]
                        if sw_qkv:
                            _lib.check(lib.uv_gemm_sw_qkv(gin.data_ptr(), d, w[f"l{l}.wqkv"].data_ptr(), C.byref(qa),
                                                          None, -1 if self.sw_qkv == "nopdl" else 0, 0,
                                                          self.tc_hints["qkv"][0], self.tc_hints["qkv"][1],
                                                          s["status"].data_ptr(), sp), "uv_gemm_sw_qkv")
                        else:
                            _lib.check(lib.uv_qkv_post_args(C.byref(qa), sp), "uv_qkv_post")
                if glob:
                    ctx = min(g_len or S, S)
                    splits = ns.get("global") or default_splits(B * K, ctx, self.device)
                    window, ring = 0, False
                else:
                    splits = ns.get("local") or default_splits(B * K, S, self.device)
                    window, ring = cfg.window, True
                if packed is not None and not skip_attn:
                    self._prefill_attn(s, packed, l, gate_vals, sp)
                elif skip_attn:
                    # the reference's A/B profiling switch (fast_decode.py:312-313): the step timed without its
                    # attention kernel -- the "attention output" is the query itself (no XSA, no head gate: both live
                    # in the attention kernel's epilogue here).  Outputs are meaningless by design.
                    z3.copy_(q)
                    if pre is not None:  # the fused launch would also have done the QKV post-processing
                        _lib.check(lib.uv_qkv_post_args(C.byref(pre), sp), "uv_qkv_post")
                else:
                    attn_launch(q, kc, vc, pos, starts, cfg.attn_scale, window, ring, ks, vs, splits, z3,
                                self._workspace(s, B, splits), v_cur=v_cur,
                                xsa_alpha=self.xsa[l] if cfg.xsa else None, xsa_eps=cfg.xsa_eps,
                                gate_x=xn if cfg.gate_channels else None,
                                gate_w=w[f"l{l}.attn_gate"] if cfg.gate_channels else None,
                                counters=s["counters"], status=s["status"], row_map=row_map, pre=pre,
                                gate_vals=gate_vals)
                lam = self.lambdas[l]
                if fused:
                    _lib.check(lib.uv_gemm_resid_norm(s["z"].data_ptr(), H * hd, w[f"l{l}.wo"].data_ptr(), H * hd,
                                                      x.data_ptr(), lam.data_ptr(), h.data_ptr(), hn.data_ptr(), dt,
                                                      B, d, sp), "uv_gemm_resid_norm")
                    _lib.check(lib.uv_gemm_swiglu(hn.data_ptr(), d, w[f"l{l}.gu"].data_ptr(), s["act"].data_ptr(),
                                                  dt, B, d, f, sp), "uv_gemm_swiglu")
                    _lib.check(lib.uv_gemm_resid_norm(s["act"].data_ptr(), f, w[f"l{l}.down"].data_ptr(), f,
                                                      h.data_ptr(), lam[2:].data_ptr(), x.data_ptr(), xn.data_ptr(),
                                                      dt, B, d, sp), "uv_gemm_resid_norm")
                    continue
                if fold:
                    x.addmm_(s["z"], w[f"l{l}.wo"].t())                       # y += z . wo'^T  (lambdas folded in)
                    torch.mm(x, w[f"l{l}.gu"].t(), out=s["gu"])
                    _lib.check(lib.uv_swiglu_rs(s["gu"].data_ptr(), x.data_ptr(), dt, d, f, s["act"].data_ptr(), B,
                                                sp), "uv_swiglu_rs")
                    x.addmm_(s["act"], w[f"l{l}.down"].t())                   # y += act . down'^T
                    continue
                torch.mm(s["z"], w[f"l{l}.wo"].t(), out=s["a"])
                _lib.check(lib.uv_resid_norm(x.data_ptr(), s["a"].data_ptr(), lam.data_ptr(), dt, d, h.data_ptr(),
                                             hn.data_ptr(), B, sp), "uv_resid_norm")
                torch.mm(hn, w[f"l{l}.gu"].t(), out=s["gu"])
                _lib.check(lib.uv_swiglu(s["gu"].data_ptr(), dt, f, s["act"].data_ptr(), B, sp), "uv_swiglu")
                torch.mm(s["act"], w[f"l{l}.down"].t(), out=s["m"])
                _lib.check(lib.uv_resid_norm(h.data_ptr(), s["m"].data_ptr(), lam[2:].data_ptr(), dt, d,
                                             x.data_ptr(), xn.data_ptr(), B, sp), "uv_resid_norm")
            if fold:  # the final norm (fast_decode.py:332-334): h = 1 * y + 0 * y is y itself, hn its RMS norm
                _lib.check(lib.uv_resid_norm(x.data_ptr(), x.data_ptr(), self._unit_lambdas().data_ptr(), dt, d,
                                             h.data_ptr(), xn.data_ptr(), B, sp), "uv_resid_norm")
        return xn  # rms_norm of the last residual stream == the final norm (fast_decode.py:332-334)

    def _trunk_tc(self, tok, st, pos, starts, g_len, ns, rm, row_map, skip_attn, packed) -> Tensor:
        """The step on the tensor-core GEMM path: per layer  uv_gemm_sw_qkv -> attention -> uv_gemm_sw_resid (wo) ->
        uv_gemm_sw_swiglu -> uv_gemm_sw_resid (down); the residual stream stays un-normalised and every consumer
        applies the RMS norm to its own result (per-tile sums of squares travel in ss_x / ss_h)."""
        cfg, lib, dt = self.cfg, _lib.lib(), DTYPE_CODE[self.dtype]
        B = tok.size(0)
        s = self.scratch(B)
        d, hd, H, K, f = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff
        sp = stream_ptr(self.device)
        w = self.w
        parts = d // 128
        x, h, xn = s["x"], s["h"], s["xn"]
        ss_x, ss_h = s["ss_x"], s["ss_h"]
        ss_ld = ss_x.stride(0)
        status = s["status"].data_ptr()
        qkv3 = s["qkv"].view(B, H + 2 * K, hd)
        q, v_cur = qkv3[:, :H], qkv3[:, H + K:]
        z3 = s["z"].view(B, H, hd)
        hq, hw, hg, hdn = (self.tc_hints[k] for k in ("qkv", "wo", "gu", "down"))
        with torch.cuda.device(self.device):
            _lib.check(lib.uv_embed_norm_ss(tok.data_ptr(), w["embed"].data_ptr(), dt, cfg.vocab_size, d,
                                            x.data_ptr(), None, B, pos.data_ptr(), self.inv_freq.data_ptr(),
                                            cfg.rope_pairs, s["rope_cs"].data_ptr() if cfg.rope_pairs else None,
                                            ss_x.data_ptr(), parts, ss_ld, sp), "uv_embed_norm_ss")
            for l in range(cfg.n_layers):
                glob = cfg.is_global(l)
                kc, vc, ks, vs = st.k[l], st.v[l], st.k_scale[l], st.v_scale[l]
                S = kc.size(2)
                rope = ((not glob) or cfg.global_rope) and cfg.rope_pairs > 0
                qa = _lib.QkvArgs()
                qa.qkv, qa.tok, qa.pos = s["qkv"].data_ptr(), tok.data_ptr(), pos.data_ptr()
                if self.use_ve and cfg.has_ve(l):
                    qa.value_embed, qa.ve_gate = w["value_embed"].data_ptr(), w[f"l{l}.ve_gate"].data_ptr()
                if rope:
                    qa.inv_freq, qa.rope_cs = self.inv_freq.data_ptr(), s["rope_cs"].data_ptr()
                qa.k_cache, qa.v_cache, qa.k_scale, qa.v_scale = kc.data_ptr(), vc.data_ptr(), ks.data_ptr(), vs.data_ptr()
                qa.row_map, qa.oob_count, qa.dtype, qa.vocab = rm, s["oob"].data_ptr(), dt, cfg.vocab_size
                qa.B, qa.H, qa.K, qa.hd, qa.d, qa.S, qa.S_alloc = B, H, K, hd, d, S, kc.stride(1) // hd
                qa.ring, qa.ve_ch, qa.n_pairs = int(not glob), cfg.ve_gate_channels, cfg.rope_pairs
                gate_vals = None
                if cfg.gate_channels:
                    qa.gate_w, qa.gate_out, qa.gate_ch = w[f"l{l}.attn_gate"].data_ptr(), s["gate"].data_ptr(), \
                        cfg.gate_channels
                    gate_vals = s["gate"]
                if packed is not None:
                    qa.last_pos = packed["last_pos"].data_ptr()
                _lib.check(lib.uv_gemm_sw_qkv(x.data_ptr(), d, w[f"l{l}.wqkv"].data_ptr(), C.byref(qa),
                                              ss_x.data_ptr(), parts, ss_ld, hq[0], hq[1], status, sp),
                           "uv_gemm_sw_qkv")
                if skip_attn:
                    z3.copy_(q)
                elif packed is not None:
                    self._prefill_attn(s, packed, l, gate_vals, sp)
                else:
                    if glob:
                        splits = ns.get("global") or default_splits(B * K, min(g_len or S, S), self.device)
                        window, ring = 0, False
                    else:
                        splits = ns.get("local") or default_splits(B * K, S, self.device)
                        window, ring = cfg.window, True
                    attn_launch(q, kc, vc, pos, starts, cfg.attn_scale, window, ring, ks, vs, splits, z3,
                                self._workspace(s, B, splits), v_cur=v_cur,
                                xsa_alpha=self.xsa[l] if cfg.xsa else None, xsa_eps=cfg.xsa_eps,
                                counters=s["counters"], status=s["status"], row_map=row_map, gate_vals=gate_vals)
                lam = self.lambdas[l]
                _lib.check(lib.uv_gemm_sw_resid(s["z"].data_ptr(), H * hd, w[f"l{l}.wo"].data_ptr(), x.data_ptr(),
                                                lam.data_ptr(), h.data_ptr(), d, ss_h.data_ptr(), ss_ld, dt, B, d,
                                                H * hd, hw[0], hw[1], status, sp), "uv_gemm_sw_resid")
                _lib.check(lib.uv_gemm_sw_swiglu(h.data_ptr(), d, w[f"l{l}.gu"].data_ptr(), s["act"].data_ptr(), dt,
                                                 B, d, f, ss_h.data_ptr(), parts, ss_ld, hg[0], status, sp),
                           "uv_gemm_sw_swiglu")
                _lib.check(lib.uv_gemm_sw_resid(s["act"].data_ptr(), f, w[f"l{l}.down"].data_ptr(), h.data_ptr(),
                                                lam[2:].data_ptr(), x.data_ptr(), d, ss_x.data_ptr(), ss_ld, dt, B, d,
                                                f, hdn[0], hdn[1], status, sp), "uv_gemm_sw_resid")
            # the final norm (fast_decode.py:332-334) for the head: h = 1 * x + 0 * x is x itself, hn its RMS norm
            _lib.check(lib.uv_resid_norm(x.data_ptr(), x.data_ptr(), self._unit_lambdas().data_ptr(), dt, d,
                                         h.data_ptr(), xn.data_ptr(), B, sp), "uv_resid_norm")
        return xn

    def _unit_lambdas(self) -> Tensor:
        if not hasattr(self, "_unit_lam"):
            self._unit_lam = torch.tensor([1.0, 0.0], dtype=torch.float32, device=self.device)
        return self._unit_lam

    def _prefill_attn(self, s, packed, l, gate_vals, sp) -> None:
        cfg, lib = self.cfg, _lib.lib()
        pa = _lib.PrefillAttnArgs()
        pa.qkv, pa.dtype, pa.ld = s["qkv"].data_ptr(), DTYPE_CODE[self.dtype], s["qkv"].stride(0)
        pa.cu_seqlens, pa.tile_cu = packed["cu"].data_ptr(), packed["tile_cu"].data_ptr()
        pa.n_seq, pa.max_tiles = int(packed["n_seq"]), int(packed["max_tiles"])
        pa.out, pa.ldo = s["z"].data_ptr(), s["z"].stride(0)
        pa.H, pa.K, pa.hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        pa.window = 0 if cfg.is_global(l) else cfg.window
        pa.scale = cfg.attn_scale
        if cfg.xsa:
            pa.xsa_alpha, pa.xsa_eps = self.xsa[l].data_ptr(), cfg.xsa_eps
        if gate_vals is not None:
            pa.gate_vals = gate_vals.data_ptr()
        elif cfg.gate_channels:
            raise RuntimeError("packed prefill needs the precomputed head gates")
        _lib.check(lib.uv_prefill_attn(C.byref(pa), sp), "uv_prefill_attn")

    def head(self, hfin: Tensor) -> Tensor:
        """Raw tied-head output (B, V) in the activation dtype (the GEMM of MathLM.logits, model.py:826)."""
        out = self.head_buffer(hfin.size(0))
        torch.mm(hfin, self.w["embed"].t(), out=out)
        return out

    def head_buffer(self, B: int) -> Tensor:
        """(B, V) buffer of the raw head output (allocated on first use: packed prefill batches never need it)."""
        s = self.scratch(B)
        if "head" not in s:
            s["head"] = torch.empty(B, self.cfg.vocab_size, dtype=self.dtype, device=self.device)
        return s["head"]

    def logits(self, h: Tensor) -> Tensor:
        """MathLM.logits (model.py:824-827): fp32 softcapped logits, for API callers that want the full matrix."""
        a, b, c = self.cfg.softcap
        z = torch.mm(h.to(self.dtype), self.w["embed"].t()).float()
        return a * torch.sigmoid((z + b) / c)

    def sample(self, head: Tensor, temperature: float, top_p: float = 1.0, u: Tensor | None = None, seed: int = 0,
               row_keys: Tensor | None = None, steps: Tensor | None = None, tok_out: Tensor | None = None,
               logp_out: Tensor | None = None, precapped: bool = False, inc_a: Tensor | None = None,
               inc_b: Tensor | None = None, top_k: int = 0):
        """uv_sample_topk on (B, V) head output; returns (tok int64 (B,), logp fp32 (B,)) in engine scratch unless
        output tensors are given."""
        B, V = head.shape
        s = self.scratch(B)
        tok_out = s["tok"] if tok_out is None else tok_out
        logp_out = s["logp"] if logp_out is None else logp_out
        a, b, c = self.cfg.softcap
        p = lambda t: None if t is None else t.data_ptr()
        with torch.cuda.device(self.device):
            rc = _lib.lib().uv_sample_topk(head.data_ptr(), DTYPE_CODE[head.dtype], head.stride(0), B, V,
                                           int(precapped), a, b, c, float(temperature), int(top_k or 0), float(top_p),
                                           p(u), C.c_uint64(seed & (2**64 - 1)), p(row_keys), p(steps),
                                           tok_out.data_ptr(), logp_out.data_ptr(), p(inc_a), p(inc_b),
                                           stream_ptr(self.device))
        _lib.check(rc, "uv_sample_topk")
        return tok_out, logp_out
