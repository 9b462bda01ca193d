"""CPU oracle for the UV-50M rollout-decode path.  TEST INFRASTRUCTURE ONLY.

This package restates, in numpy, the reference's own CPU-runnable implementation of the path (quantiser, cache
writes, fp32 decode-attention reference, one int8-KV decode step of the model, left-padded prefill, softcap head,
samplers and the continuous-batching output contract).  Every function cites the reference file:line it follows.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference itself (CPU, fp32) and stores its
outputs on seeded inputs under ``tests/golden/*.npz``; ``tests/test_oracle_golden.py`` checks this restatement
against those files (int8 bytes / fp16 scales / token streams exactly, floating point to 1e-4 or tighter).

Nothing under ``ultraviolet_b200/`` imports this package.  Only ``tests/``, ``__graft_entry__.smoke()`` and
``bench.py``'s CPU-baseline legs may use it, and only as the checker or as the timed CPU baseline.
"""
from .kv import dequantize_kv, kv_write, kv_write_rows, quantize_kv  # noqa: F401
from .attn import decode_attention_ref, attention_key_counts  # noqa: F401
