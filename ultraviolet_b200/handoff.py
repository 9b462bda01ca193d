"""Device-resident hand-off of finished rollouts to the trainer.

The reference moves every rollout to the host as Python lists / numpy arrays (``StreamGen.chunk``,
scripts/rl_stream.py:119-147), and its trainer packs them into fixed-size token micro-batches on the host before
copying them back to the GPU (``build_packed``, ultraviolet/perf.py:55-95; ``Trainer.step``, scripts/rl_grpo.py:
230-302).  Here the payload never leaves the device: ``GpuScheduler.harvest_packed(with_prompts=True)`` returns flat
device tensors (prompt tokens, generated tokens, behaviour log-probs, per-rollout offsets), and
``build_packed_device`` lays them out as the trainer's micro-batches with index arithmetic on the GPU.  Only the
rollout LENGTHS (one small D2H) go to the host, where the bin packing -- a few hundred integers -- is planned.

Micro-batch layout (the contract of perf.py:55-95): each sequence contributes its first len - 1 tokens as inputs
``x`` and the shifted tokens as targets ``y`` (-1 on prompt positions: only generated tokens are trained on), its
advantage on every position (``A``), its behaviour log-probs on the target positions (``OL``), positions restarting at
every sequence (``pos``) and the segment boundaries ``cu``; the unused tail is cut into pad segments of at most
seg_max tokens so that every position lies in a segment a varlen kernel visits; ``tgt`` lists the target positions.
"""
from __future__ import annotations

import numpy as np
import torch


def pack_bins(lens, budget: int) -> list[list[int]]:
    """First-fit decreasing (same plan as perf.py:38-52): indices grouped so that a group's lengths sum to <= budget."""
    order = sorted(range(len(lens)), key=lambda i: -int(lens[i]))
    bins: list[list[int]] = []
    room: list[int] = []
    for i in order:
        L = int(lens[i])
        if L > budget:
            raise ValueError(f"a sequence of {L} tokens does not fit a micro-batch of {budget}")
        for j in range(len(bins)):
            if room[j] >= L:
                bins[j].append(i)
                room[j] -= L
                break
        else:
            bins.append([i])
            room.append(budget - L)
    return bins


@torch.no_grad()
def build_packed_device(p: dict, adv, budget: int, pad_id: int, seg_max: int = 512) -> list[dict]:
    """p: the dict of ``harvest_packed(with_prompts=True)``; adv: one advantage per rollout (sequence, array or tensor,
    in p's order).  Returns one dict per micro-batch with DEVICE tensors x (1, budget) int64, y (1, budget) int64,
    A, OL (1, budget) fp32, pos (budget,) int64, cu (S + 1,) int32, tgt (n_t,) int64 and the int max_seqlen."""
    dev = p["tokens"].device
    n = len(p["metas"])
    off_o = p["offsets"].to(torch.int64)                 # generated tokens of rollout i: [off_o[i], off_o[i + 1])
    off_p = p["prompt_offsets"].to(torch.int64)          # prompt tokens likewise
    host = torch.stack([off_p[1:] - off_p[:-1], off_o[1:] - off_o[:-1]]).cpu().numpy()    # the one D2H: 2n integers
    plen, olen = host[0], host[1]
    seq = plen + olen - 1                                 # inputs per sequence: every token but the last
    adv_d = torch.as_tensor(np.asarray(adv, dtype=np.float32) if not torch.is_tensor(adv) else adv,
                            dtype=torch.float32, device=dev)
    out = []
    for b in pack_bins(seq.tolist(), budget):
        b = sorted(b)
        ids = torch.as_tensor(b, dtype=torch.int64, device=dev)
        L = torch.as_tensor(seq[b], dtype=torch.int64, device=dev)
        s = torch.as_tensor(plen[b], dtype=torch.int64, device=dev)
        start = torch.cumsum(L, 0) - L                    # first micro-batch position of each sequence
        used = int(seq[b].sum())
        which = torch.repeat_interleave(torch.arange(len(b), device=dev), L, output_size=used)   # sequence of a position
        j = torch.arange(used, device=dev) - start[which]                                     # index inside it
        sq, po, oo = s[which], off_p[ids][which], off_o[ids][which]
        # token j of a sequence is prompt[j] for j < s, else generated[j - s]
        tok_at = lambda k: torch.where(k < sq, p["prompt_tokens"][(po + k).clamp_(max=p["prompt_tokens"].numel() - 1)],
                                       p["tokens"][(oo + (k - sq).clamp_(min=0)).clamp_(max=p["tokens"].numel() - 1)]
                                       ).to(torch.int64)
        x = torch.full((budget,), pad_id, dtype=torch.int64, device=dev)
        y = torch.full((budget,), -1, dtype=torch.int64, device=dev)
        A = torch.zeros(budget, dtype=torch.float32, device=dev)
        OL = torch.zeros(budget, dtype=torch.float32, device=dev)
        pos = torch.zeros(budget, dtype=torch.int64, device=dev)
        x[:used] = tok_at(j)
        is_t = j >= sq - 1                                # position j predicts token j + 1, a generated one
        y[:used] = torch.where(is_t, tok_at(j + 1), y[:used])
        A[:used] = adv_d[ids][which]
        lp_i = (oo + (j - (sq - 1)).clamp_(min=0)).clamp_(max=p["logp"].numel() - 1)
        OL[:used] = torch.where(is_t, p["logp"][lp_i], OL[:used])
        pos[:used] = j
        cu = np.concatenate([[0], np.cumsum(seq[b])]).tolist()
        ms, o = int(seq[b].max()), used
        while o < budget:                                 # pad segments: every position belongs to some segment
            k = min(seg_max, budget - o)
            pos[o:o + k] = torch.arange(k, device=dev)
            o += k
            cu.append(o)
        ms = max(ms, min(seg_max, budget))
        out.append({"x": x[None], "y": y[None], "A": A[None], "OL": OL[None], "pos": pos,
                    "cu": torch.as_tensor(cu, dtype=torch.int32, device=dev), "max_seqlen": ms,
                    "tgt": torch.nonzero(y != -1).squeeze(1), "requests": [p["metas"][i] for i in b]})
    return out
