"""Oracle (test infrastructure): fp32 numpy restatement of the reference's int8-KV decode path for MathLM.

Follows, function by function:
  fuse_weights        Attention.fuse / MLP.fuse                    ultraviolet/model.py:289-300, :384-386
  rms_norm            F.rms_norm(x, (d,)) with eps=None            ultraviolet/model.py:190-191
  rope_cos_sin        Rotary.cos_sin                               ultraviolet/model.py:198-216
  apply_rope          apply_rope (half-split pairing)              ultraviolet/model.py:219-226
  new_state           KernelDecodeState (int8)                     ultraviolet/kernels/fast_decode.py:21-57
  decode_step         decode_step_fast                             ultraviolet/kernels/fast_decode.py:272-334
  prefill             prefill_fast + MathLM.trunk (dense masks)    fast_decode.py:70-114, model.py:742-822
  logits              MathLM.logits                                ultraviolet/model.py:824-827
  sample_greedy       sample(T <= 0)                               ultraviolet/model.py:1194-1199
  top_p_keep          sample(top_p < 1) kept set                   ultraviolet/model.py:1203-1208
  fused_sample_ref    fused_sample_ref                             ultraviolet/kernels/fused_sample.py:81-91
  left_pad            _left_pad                                    ultraviolet/model.py:1214-1221
  generate            generate                                     ultraviolet/model.py:1228-1263
  generate_continuous generate_continuous                          ultraviolet/model.py:1266-1354

Weights are a dict of fp32 numpy arrays keyed by the reference's parameter names ("blocks.3.attn.wq", ...).  The
config object only needs the reference's MathConfig attributes.  All arithmetic is fp32 (the reference's CPU path
with an fp32 model); ``round_to`` lets the caller round fused weights to bf16/fp16 exactly as ``fuse(dtype)`` does.
"""
from __future__ import annotations

import numpy as np

from .attn import decode_attention_ref
from .kv import kv_write, kv_write_rows

F32_EPS = np.float32(1.1920929e-07)  # torch.finfo(float32).eps: F.rms_norm's default eps in fp32 opmath


# ------------------------------------------------------------------------------------------------ rounding helpers
def round_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest-even bfloat16, returned as fp32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    out = ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def round_fp16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


ROUNDERS = {"fp32": lambda a: np.asarray(a, dtype=np.float32), "bf16": round_bf16, "fp16": round_fp16}


# ------------------------------------------------------------------------------------------------ weights
def fuse_weights(params: dict, cfg, round_to: str = "fp32") -> dict:
    """model.py:289-300 (Attention.fuse), :384-386 (MLP.fuse), for every layer, plus the tensors decode reads
    directly.  ``params`` holds the model's parameters already cast to the compute dtype (as fp32 arrays)."""
    rnd = ROUNDERS[round_to]
    f32 = lambda a: np.asarray(a, dtype=np.float32)
    W = {"embed": f32(params["embed.weight"]), "layers": []}
    if "value_embed.weight" in params:
        W["value_embed"] = f32(params["value_embed.weight"])
    for l in range(cfg.n_layers):
        p = lambda n: f32(params[f"blocks.{l}.{n}"])
        L = {"wqkv": rnd(np.concatenate([p("attn.wq"), p("attn.wk"), p("attn.wv")]) * p("attn.qkv_scale")),
             "wo": rnd(p("attn.wo") * p("attn.o_scale")),
             "gu": rnd(np.concatenate([p("mlp.w_gate"), p("mlp.w_up")])),
             "down": rnd(p("mlp.w_down")),
             "lambdas": np.array([rnd(p("resid_attn")), rnd(p("post_attn")), rnd(p("resid_mlp")),
                                  rnd(p("post_mlp"))], dtype=np.float32)}
        if cfg.has_ve(l):
            L["ve_gate"] = rnd(p("attn.ve_gate"))
        if min(cfg.attn_gate_channels, cfg.d_model):
            L["attn_gate"] = rnd(p("attn.attn_gate"))
        if cfg.xsa:
            L["xsa"] = np.tanh(p("attn.xsa_alpha")).astype(np.float32)
        W["layers"].append(L)
    return W


# ------------------------------------------------------------------------------------------------ elementwise pieces
def rms_norm(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    ms = np.mean(x * x, axis=-1, keepdims=True, dtype=np.float32)
    return x * (np.float32(1.0) / np.sqrt(ms + F32_EPS))


def rope_inv_freq(cfg) -> np.ndarray:
    n = int(cfg.head_dim * cfg.rope_frac) // 2
    return (np.float32(1.0 / cfg.rope_base) ** np.linspace(0, 1, n, dtype=np.float32)).astype(np.float32)


def rope_cos_sin(cfg, pos: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    th = np.asarray(pos).astype(np.float32)[..., None] * rope_inv_freq(cfg)
    return np.cos(th).astype(np.float32), np.sin(th).astype(np.float32)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x (..., H, hd); cos/sin broadcastable to (..., 1, n_pairs)."""
    n = cos.shape[-1]
    if n == 0:
        return x
    c, s = cos[..., None, :], sin[..., None, :]
    x1, x2, rest = x[..., :n], x[..., n:2 * n], x[..., 2 * n:]
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c, rest], axis=-1)


def _sigmoid(x):
    return np.float32(1.0) / (np.float32(1.0) + np.exp(-x.astype(np.float32)))


def logits(W: dict, cfg, h: np.ndarray) -> np.ndarray:
    a, b, c = (np.float32(v) for v in cfg.softcap)
    z = h.astype(np.float32) @ W["embed"].T
    return a * _sigmoid((z + b) / c)


def _qkv(L: dict, cfg, l: int, xn, ve, cos, sin):
    """Attention.qkv (model.py:302-320).  xn (N, d); ve (N, K, hd) or None; cos/sin (N, n_pairs)."""
    H, K, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    N = xn.shape[0]
    qkv = xn @ L["wqkv"].T
    q = qkv[:, :H * hd].reshape(N, H, hd)
    k = qkv[:, H * hd:(H + K) * hd].reshape(N, K, hd)
    v = qkv[:, (H + K) * hd:].reshape(N, K, hd)
    if cfg.has_ve(l) and ve is not None:
        gw = L["ve_gate"]
        g = np.float32(2.0) * _sigmoid(xn[:, :gw.shape[-1]] @ gw.T)  # (N, K)
        v = v + g[..., None] * ve
    q, k = rms_norm(q), rms_norm(k)
    if not cfg.is_global(l) or cfg.global_rope:
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    return q, k, v


def _post(L: dict, cfg, z, xn, v):
    """Attention.post (model.py:322-335).  z (N, H, hd) attention output; v (N, K, hd) current-token values."""
    N = z.shape[0]
    H, K, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    G = H // K
    if cfg.xsa:
        a = L["xsa"].reshape(1, K, G, 1)
        zg = z.reshape(N, K, G, hd).astype(np.float32)
        nrm = np.sqrt(np.sum(v * v, axis=-1, keepdims=True, dtype=np.float32))
        vd = (v / np.maximum(nrm, np.float32(cfg.xsa_eps)))[:, :, None, :]
        proj = np.sum(zg * vd, axis=-1, keepdims=True, dtype=np.float32)
        z = (zg - a * proj * vd).reshape(N, H, hd)
    gch = min(cfg.attn_gate_channels, cfg.d_model)
    if gch:
        g = np.float32(2.0) * _sigmoid(xn[:, :gch] @ L["attn_gate"].T)  # (N, H)
        z = z * g[..., None]
    return z.reshape(N, H * hd) @ L["wo"].T


def _finish(L: dict, base, a):
    """Block.finish (model.py:567-571) with the fused MLP (model.py:388-391)."""
    ra, pa, rm, pm = L["lambdas"]
    h = ra * base + pa * a
    gu = rms_norm(h) @ L["gu"].T
    f = gu.shape[-1] // 2
    g, u = gu[:, :f], gu[:, f:]
    m = (g * _sigmoid(g) * u) @ L["down"].T
    return rm * h + pm * m


# ------------------------------------------------------------------------------------------------ state
class State:
    """fast_decode.py:21-57 for kv_dtype == "int8" (attention-only configs)."""

    def __init__(self, cfg, B: int, max_len: int):
        self.cfg, self.B, self.max_len = cfg, B, max_len
        self.local_len = min(cfg.window, max_len)
        K, hd = cfg.n_kv_heads, cfg.head_dim
        self.k, self.v, self.k_scale, self.v_scale = [], [], [], []
        for l in range(cfg.n_layers):
            S = max_len if cfg.is_global(l) else self.local_len
            self.k.append(np.zeros((B, K, S, hd), np.int8))
            self.v.append(np.zeros((B, K, S, hd), np.int8))
            self.k_scale.append(np.zeros((B, K, S), np.float16))
            self.v_scale.append(np.zeros((B, K, S), np.float16))
        self.pos = np.zeros(B, np.int64)
        self.starts = np.zeros(B, np.int64)


def decode_step(W: dict, cfg, tok: np.ndarray, st: State, return_hidden: bool = False) -> np.ndarray:
    """fast_decode.py:272-334: feed tok (B,) at each row's position st.pos; returns (B, V) softcapped logits (or the
    final normed hidden) and advances st.pos."""
    B = tok.shape[0]
    K, hd, H = cfg.n_kv_heads, cfg.head_dim, cfg.n_heads
    p = st.pos.copy()
    cos, sin = rope_cos_sin(cfg, p)
    ve = W["value_embed"][tok].reshape(B, K, hd) if "value_embed" in W else None
    x = rms_norm(W["embed"][tok])
    Wl = st.local_len
    bk = np.arange(B)[:, None] * K + np.arange(K)[None, :]
    gidx = (bk * st.max_len + p[:, None]).reshape(-1)
    lidx = (bk * Wl + np.remainder(p[:, None], Wl)).reshape(-1)
    for l, L in enumerate(W["layers"]):
        xn = rms_norm(x)
        q, k, v = _qkv(L, cfg, l, xn, ve, cos, sin)
        glob = cfg.is_global(l)
        ix = gidx if glob else lidx
        kv_write(st.k[l], st.k_scale[l], ix, k)
        kv_write(st.v[l], st.v_scale[l], ix, v)
        z = decode_attention_ref(q, st.k[l], st.v[l], p, st.starts, cfg.attn_scale,
                                 window=0 if glob else cfg.window, ring=not glob,
                                 k_scale=st.k_scale[l], v_scale=st.v_scale[l])
        x = _finish(L, x, _post(L, cfg, z, xn, v))
    st.pos += 1
    h = rms_norm(x)
    return h if return_hidden else logits(W, cfg, h)


def left_pad(prompts, pad_id: int = 0):
    """model.py:1214-1221."""
    T = max(len(p) for p in prompts)
    idx = np.full((len(prompts), T), pad_id, np.int64)
    starts = np.zeros(len(prompts), np.int64)
    for b, p in enumerate(prompts):
        idx[b, T - len(p):] = np.asarray(p, np.int64)
        starts[b] = T - len(p)
    return idx, starts


def _masked_attention(q, k, v, mask, scale, G):
    """SDPA with a boolean mask (model.py:361-363): q (n, T, H, hd), k/v (n, T, K, hd), mask (n, T, T)."""
    n, T, H, hd = q.shape
    K = k.shape[2]
    qg = q.reshape(n, T, K, G, hd)
    s = np.einsum("nikgd,njkd->nkgij", qg, k, optimize=True) * np.float32(scale)
    s = np.where(mask[:, None, None], s, -np.inf).astype(np.float32)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    w = e / e.sum(-1, keepdims=True)
    return np.einsum("nkgij,njkd->nikgd", w, v, optimize=True).reshape(n, T, H, hd)


def prefill(W: dict, cfg, idx: np.ndarray, starts: np.ndarray, st: State, rows=None) -> np.ndarray:
    """fast_decode.py:70-114 over MathLM.trunk with key_valid masks (model.py:742-822).  idx (n, T) left-padded.
    Writes the int8 cache of `rows`, sets their pos = T / starts, returns last-position logits (n, V)."""
    n, T = idx.shape
    assert T <= st.max_len
    K, hd = cfg.n_kv_heads, cfg.head_dim
    G = cfg.n_heads // K
    ar = np.arange(T)
    key_valid = ar[None, :] >= starts[:, None]
    cos, sin = rope_cos_sin(cfg, ar)
    ve = W["value_embed"][idx].reshape(n * T, K, hd) if "value_embed" in W else None
    cosn, sinn = np.tile(cos, (n, 1)), np.tile(sin, (n, 1))
    causal = ar[:, None] >= ar[None, :]
    local = causal & ((ar[:, None] - ar[None, :]) < cfg.window)
    eye = np.eye(T, dtype=bool)
    masks = {True: (causal[None] & key_valid[:, None, :]) | eye[None],
             False: (local[None] & key_valid[:, None, :]) | eye[None]}
    x = rms_norm(W["embed"][idx]).reshape(n * T, -1)
    full = rows is None
    if full:
        assert n == st.B
        rows = np.arange(n)
    rows = np.asarray(rows)
    for l, L in enumerate(W["layers"]):
        xn = rms_norm(x)
        q, k, v = _qkv(L, cfg, l, xn, ve, cosn, sinn)
        glob = cfg.is_global(l)
        z = _masked_attention(q.reshape(n, T, -1, hd), k.reshape(n, T, K, hd), v.reshape(n, T, K, hd),
                              masks[glob], cfg.attn_scale, G)
        x = _finish(L, x, _post(L, cfg, z.reshape(n * T, -1, hd), xn, v))
        kt = k.reshape(n, T, K, hd).transpose(0, 2, 1, 3)
        vt = v.reshape(n, T, K, hd).transpose(0, 2, 1, 3)
        for cache, sc, new in ((st.k[l], st.k_scale[l], kt), (st.v[l], st.v_scale[l], vt)):
            S = cache.shape[2]
            if glob:
                kv_write_rows(cache, sc, new, slice(0, T), None if full else rows)
            else:
                lo = max(0, T - S)
                kv_write_rows(cache, sc, new[:, :, lo:], np.arange(lo, T) % S, None if full else rows)
    st.starts[rows] = starts
    st.pos[rows] = T
    h = rms_norm(x).reshape(n, T, -1)[:, -1]
    return logits(W, cfg, h)


# ------------------------------------------------------------------------------------------------ samplers
def sample_greedy(lg: np.ndarray) -> np.ndarray:
    return np.argmax(lg, axis=-1).astype(np.int64)


def log_prob_of(lg: np.ndarray, tok: np.ndarray, temperature: float) -> np.ndarray:
    """Behaviour log-prob log softmax(logits / T)[tok] (model.py:1160-1169, rl_stream.py:119): untruncated."""
    z = lg.astype(np.float32) / np.float32(temperature)
    m = z.max(-1, keepdims=True)
    lse = (m[:, 0] + np.log(np.exp(z - m).sum(-1, dtype=np.float32))).astype(np.float32)
    return z[np.arange(z.shape[0]), tok] - lse


def top_p_keep(lg: np.ndarray, temperature: float, top_p: float) -> np.ndarray:
    """model.py:1203-1208: boolean mask of the tokens that survive nucleus truncation (ties with the cut kept)."""
    z = lg.astype(np.float32) / np.float32(temperature)
    zs = -np.sort(-z, axis=-1)
    e = np.exp(zs - zs[:, :1])
    ps = e / e.sum(-1, keepdims=True)
    keep = (np.cumsum(ps, axis=-1, dtype=np.float32) - ps) < np.float32(top_p)
    cut = np.where(keep, zs, np.inf).min(-1, keepdims=True)
    return z >= cut


def fused_sample_ref(x: np.ndarray, u: np.ndarray, softcap, temperature: float = 1.0):
    """fused_sample.py:81-91.  x (B, V) raw head output, u (B,) uniforms in [0, 1) -> (tokens, log-probs)."""
    a, b, c = (np.float32(v) for v in softcap)
    z = a * _sigmoid((x.astype(np.float32) + b) / c)
    e = np.exp((z - a) / np.float32(temperature)).astype(np.float32)
    cs = np.cumsum(e, axis=-1, dtype=np.float32)
    S = cs[:, -1]
    target = (np.float32(1.0) - u.astype(np.float32)) * S
    tok = np.array([np.searchsorted(cs[i], target[i], side="left") for i in range(x.shape[0])], np.int64)
    tok = np.minimum(tok, x.shape[1] - 1)
    lp = (z[np.arange(x.shape[0]), tok] - a) / np.float32(temperature) - np.log(S)
    return tok, lp.astype(np.float32)


# ------------------------------------------------------------------------------------------------ generation
def generate(W: dict, cfg, prompts, max_new: int, eos_id=None, pad_id: int = 0, max_len=None):
    """model.py:1228-1263 with temperature 0 (greedy)."""
    B = len(prompts)
    idx, starts = left_pad(prompts, pad_id)
    max_len = max_len or (idx.shape[1] + max_new)
    st = State(cfg, B, max_len)
    tok = sample_greedy(prefill(W, cfg, idx, starts, st))
    out = [tok.copy()]
    for _ in range(max_new - 1):
        if st.pos.max() >= max_len:
            break
        tok = sample_greedy(decode_step(W, cfg, tok, st))
        out.append(tok.copy())
    res = []
    for row in np.stack(out, 1).tolist():
        if eos_id is not None and eos_id in row:
            row = row[:row.index(eos_id) + 1]
        res.append(row)
    return res


def generate_continuous(W: dict, cfg, prompts, max_new: int, batch: int, eos_id=None, pad_id: int = 0,
                        check_every: int = 16, target_lens=None):
    """model.py:1266-1354 with temperature 0: slots harvested every check_every steps, finished rows refilled by a
    left-padded prefill of just those rows, idle rows parked at position 0.  Completions in prompt order."""
    n = len(prompts)
    B = min(batch, n)
    max_len = max(len(p) for p in prompts) + max_new + check_every
    st = State(cfg, B, max_len)
    buf = np.zeros((B, max_new + check_every), np.int64)
    cnt = np.zeros(B, np.int64)
    slot_item = [-1] * B
    limit = np.zeros(B, np.int64)
    host_cnt = np.zeros(B, np.int64)
    results = [None] * n
    nxt = 0
    tok = np.zeros(B, np.int64)

    def refill(rows):
        nonlocal nxt
        rows = rows[:max(0, n - nxt)]
        if not rows:
            return
        items = list(range(nxt, nxt + len(rows)))
        nxt += len(rows)
        idx, starts = left_pad([prompts[i] for i in items], pad_id)
        rt = np.asarray(rows)
        buf[rt] = -1
        first = sample_greedy(prefill(W, cfg, idx, starts, st, rows=rt))
        tok[rt] = first
        buf[rt, 0] = first
        cnt[rt] = 1
        for r, i in zip(rows, items):
            slot_item[r] = i
            limit[r] = min(max_new, target_lens[i]) if target_lens is not None else max_new
            host_cnt[r] = 1

    refill(list(range(B)))
    while any(s >= 0 for s in slot_item):
        for _ in range(check_every):
            tok = sample_greedy(decode_step(W, cfg, tok, st))
            buf[np.arange(B), cnt] = tok
            cnt = np.minimum(cnt + 1, buf.shape[1] - 1)
        host_cnt += check_every
        done = []
        for r in range(B):
            if slot_item[r] < 0:
                continue
            hit = eos_id is not None and bool((buf[r] == eos_id).any())
            if host_cnt[r] >= limit[r] or hit:
                row = buf[r, :min(host_cnt[r], limit[r])].tolist()
                if eos_id is not None and eos_id in row:
                    row = row[:row.index(eos_id) + 1]
                results[slot_item[r]] = row
                slot_item[r] = -1
                done.append(r)
        if done:
            refill(done)
            idle = [r for r in done if slot_item[r] < 0]
            if idle:
                st.pos[idle] = 0
                st.starts[idle] = 0
    return results
