/*
 * uvdecode.h -- C ABI of libuvdecode.so: the UV-50M rollout-decode hot path as hand-written sm_100a CUDA kernels.
 *
 * The reference (hliuson/ultraviolet) is pure Python and has no FFI; its one native boundary on this path is the
 * NVRTC launch `torch.cuda._compile_kernel(...)(grid, block, args=[...])` (ultraviolet/kernels/decode_attn_cuda.py:
 * 300-305).  Each entry point below replaces one reference Python function (cited per function) and is what a
 * ctypes / cffi binding on the reference side would call.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name starts with "h_"; the library never allocates, frees or
 *     synchronises; all work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy default
 *     stream), so every call is CUDA-graph capturable;
 *   - return value: 0 on success, a negative UV_ERR_* code on an argument error (nothing is launched), or
 *     UV_ERR_CUDA with the CUDA error retrievable through uv_last_cuda_error();
 *   - dtype codes: UV_F32 / UV_F16 / UV_BF16 / UV_I8;
 *   - strides are in ELEMENTS of the tensor they describe; the innermost (head_dim) dimension is contiguous;
 *   - no global mutable state apart from a per-thread last-error slot: calls are re-entrant per device/stream.
 */
#ifndef UVDECODE_H_
#define UVDECODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UV_ABI_VERSION 2

enum { UV_F32 = 0, UV_F16 = 1, UV_BF16 = 2, UV_I8 = 3 };

enum {
  UV_OK = 0,
  UV_ERR_ARG = -1,        /* null pointer / negative size / unsupported combination */
  UV_ERR_DTYPE = -2,      /* dtype code not supported by this entry point */
  UV_ERR_SHAPE = -3,      /* head_dim / group size / vocabulary outside the compiled set */
  UV_ERR_ALIGN = -4,      /* pointer or stride alignment requirement not met */
  UV_ERR_WORKSPACE = -5,  /* workspace missing or too small */
  UV_ERR_CUDA = -6,       /* a CUDA runtime call failed; see uv_last_cuda_error() */
  UV_ERR_STATIC_LIMIT = -7 /* problem larger than the built-in scratch of uv_decode_attn_static */
};

int uv_abi_version(void);
const char* uv_error_string(int code);
int uv_last_cuda_error(void); /* cudaError_t of the last UV_ERR_CUDA on this host thread */

/* ---------------------------------------------------------------------------------------------------------------
 * (b) KV quantise + append.  Replaces quantize_kv + kv_write (ultraviolet/kernels/kv_quant.py:12-36) and the two
 * kv_write calls per layer of decode_step_fast (ultraviolet/kernels/fast_decode.py:316-317).
 *
 * Quantiser (bit-exact with kv_quant.py:12-19): scale16 = fp16_rne(max|x| / 127) (fp32 division); q = clamp(
 * rint(x / max(float(scale16), 1e-30)), -127, 127) with a true fp32 division and round-half-even.
 *
 * uv_kv_quant_scatter: n_rows vectors x[i] (hd elements, row stride x_stride) are quantised and written to row
 * flat_idx[i] of the flat (rows, hd) int8 view `cache` and element flat_idx[i] of `scale` (fp16 bits).
 * flat_idx == NULL means the identity (plain quantize_kv into contiguous outputs).  n_cache_rows bounds flat_idx;
 * out-of-range indices are skipped and counted in *oob_count (optional device int, may be NULL).
 */
int uv_kv_quant_scatter(const void* x, int x_dtype, int64_t x_stride, int64_t n_rows, int hd,
                        int8_t* cache, uint16_t* scale, const int64_t* flat_idx, int64_t n_cache_rows,
                        int* oob_count, void* stream);

/* uv_kv_append: the decode-time form.  For every slot-row b < B and kv head h < KH, quantise k_new[b,h,:] and
 * v_new[b,h,:] and store them at cache slot (ring ? pos[b] % S : pos[b]) of row (b*KH + h) in caches laid out
 * (B, KH, S, hd) int8 / (B, KH, S) fp16 (kv_quant.py:3-4).  Rows whose slot falls outside [0, S) are skipped and
 * counted in *oob_count.  k_new / v_new: (B, KH, hd) with row strides in elements between consecutive (b, h). */
int uv_kv_append(const void* k_new, const void* v_new, int dtype, int64_t k_stride, int64_t v_stride,
                 int8_t* k_cache, int8_t* v_cache, uint16_t* k_scale, uint16_t* v_scale,
                 const int64_t* pos, int B, int KH, int hd, int S, int ring, int* oob_count, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * (c) Split-K single-query decode attention over the slot-indexed cache.  Replaces decode_attention / _launch /
 * _split_kernel / _combine_kernel (ultraviolet/kernels/decode_attn.py:24-230) and decode_attn_cuda.launch
 * (ultraviolet/kernels/decode_attn_cuda.py:273-309).
 *
 * Row b attends to the keys at absolute positions lo_b..pos_b, lo_b = max(starts_b, pos_b - window + 1, 0)
 * (window 0 = unlimited); position t lives in slot t % S when ring, else slot t.  Query head h*G+g uses kv head h.
 * out[b, h*G+g, :] = softmax_t(scale * q.K_t * ks_t) . (V_t * vs_t).
 *
 * Optional fused epilogue (Attention.post up to the output projection, ultraviolet/model.py:322-333), applied
 * when the pointers are non-NULL: XSA  z -= xsa_alpha[head] * (z . vhat) * vhat with vhat = v_cur / max(|v_cur|,
 * xsa_eps) from the CURRENT token's unquantised v, then the head gate z *= 2*sigmoid(gate_x[b, :gate_ch] .
 * gate_w[head, :gate_ch]).
 */
typedef struct uv_attn_args {
  const void* q;          /* (B, H, hd) */
  int q_dtype;            /* UV_F16 | UV_BF16 */
  int64_t sqb, sqh;
  const void* k_cache;    /* (B, KH, S, hd) */
  const void* v_cache;
  int kv_dtype;           /* UV_I8 (with scales) */
  int64_t skb, skh, sks, svb, svh, svs;
  const uint16_t* k_scale; /* (B, KH, S) fp16 bits */
  const uint16_t* v_scale;
  int64_t ssb, ssh, stb, sth;
  const int64_t* pos;     /* (B,) position of the newest key (already in the cache) */
  const int64_t* starts;  /* (B,) first valid position */
  const int64_t* row_map; /* optional (B,): cache row read by batch entry b (default b); lets a sub-batch address
                             rows of a larger cache, as prefill(rows=...) does (fast_decode.py:70-114) */
  void* out;              /* (B, H, hd) in q_dtype */
  int64_t sob, soh;
  int B, H, KH, hd, S;
  int S_alloc;            /* slots allocated per (b, kv head) row, 0 = S.  A linear (non-ring) cache whose rows are
                             allocated to a multiple of 8 slots takes the TMA path even when S itself is not; a ring
                             takes it when S is a multiple of 8 */
  int window, ring;
  float scale;
  int num_splits;         /* >= 1.  2..8 splits of a row run as one thread-block cluster and merge through distributed
                             shared memory; more than 8 merge through workspace */
  void* workspace;        /* uv_decode_attn_workspace_bytes() bytes, 16-byte aligned */
  size_t workspace_bytes;
  int* counters;          /* optional, B*KH ints, all zero on entry (left zero on exit): when given and num_splits > 1,
                             the split CTA that arrives last merges the partials (one launch instead of two); two
                             launches that overlap on the GPU must not share one counters array */
  int* status;            /* optional device word: bit 0 is set if a bulk copy did not land within 200 ms (the row's
                             output is then undefined); never cleared by the library */
  /* fused epilogue, all optional */
  const void* v_cur;      /* (B, KH, hd) q_dtype with batch / head strides v_cur_sb / v_cur_sh (elements) */
  int64_t v_cur_sb, v_cur_sh;
  const float* xsa_alpha; /* (H,) fp32, already tanh'ed (Attention.fuse, model.py:298-299) */
  float xsa_eps;
  const void* gate_x;     /* (B, >= gate_ch) q_dtype, row stride gate_x_stride */
  int64_t gate_x_stride;
  const void* gate_w;     /* (H, gate_ch) q_dtype contiguous */
  int gate_ch;
  const float* gate_vals; /* optional (B, H) fp32: the gates themselves, as uv_qkv_post_args writes them (gate_out);
                             when set, gate_x / gate_w are not read */
} uv_attn_args;

size_t uv_decode_attn_workspace_bytes(int B, int KH, int G, int hd, int num_splits);
/* Split count for (B*KH) cache rows of at most ctx keys on a device with n_sm SMs (role of default_splits,
 * decode_attn.py:121-129): every CTA resident in one wave (4 per SM), at least two 128-key tiles per split, and at
 * most 8 splits (the cluster merge) unless the batch is so small that 8 per row leave most SMs idle. */
int uv_default_splits(int n_bk, int ctx, int n_sm);
/* A row whose key range is empty (starts[b] > pos[b], or pos[b] < 0) attends to nothing: its output is all zeros
 * (the reference's softmax over an empty set is NaN there; the case does not occur on the decode path, where the
 * current token's key is always in range).  Such rows do not affect the others. */
int uv_decode_attn(const uv_attn_args* args, void* stream);
/* Which copy path uv_decode_attn takes for these arguments: 1 = bulk-copy (TMA) tiles (linear rows allocated to a
 * multiple of 8 slots, or a ring whose length is a multiple of 8; 16-byte aligned rows and scale rows), 0 = the
 * two-stage cp.async path that every other geometry takes; negative = argument error.  Launches nothing.  (The
 * reference picks its backend the same way, from tensor metadata: decode_attn_cuda.supported, decode_attn_cuda.py:
 * 262-268.) */
int uv_decode_attn_uses_bulk(const uv_attn_args* args);

/* uv_decode_attn_static: the same attention, for hosts that cannot allocate device memory.  (No counterpart in the
 * reference: its Python op allocates split partials with torch.empty on every call.)
 *
 * Who needs it: an embedding runtime that owns no CUDA allocator (a service calling this library over FFI whose HBM
 * is already reserved in full for the KV cache), or a serving loop that is not allowed to call cudaMalloc on its
 * latency path because device allocation synchronises the whole GPU.  Such callers still pass q, the caches, pos /
 * starts and out; args->workspace, workspace_bytes and counters are IGNORED.  The split partials and the arrival
 * counters live in a device array built into the library: 4 MiB of partials and 4096 cache rows (B*KH), held by
 * every GPU that loads the library until the process exits.  Larger problems -- uv_decode_attn_workspace_bytes(...)
 * above 4 MiB or B*KH above 4096 -- are rejected with UV_ERR_STATIC_LIMIT and nothing is launched.
 *
 * The first call on a device looks the array's device address up (cudaGetSymbolAddress, cached per device); make
 * that first call outside any stream capture.  All calls share the one array, which keeps the previous call's
 * contents: the counters are cleared on `stream` before each launch, the partials are fully rewritten before they
 * are read.  Two calls whose kernels can overlap on the GPU (different streams, no dependency) race on the array
 * and produce undefined output; serialise them.  The function calls no cudaMalloc / cudaFree and no allocating
 * library routine. */
int uv_decode_attn_static(const uv_attn_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * (d) Row-wise fused kernels of one decode step (the elementwise chain of decode_step_fast, ultraviolet/kernels/
 * fast_decode.py:272-334, between its GEMMs).  dtype = UV_F16 | UV_BF16 activations; every result is rounded to
 * dtype where the reference's half-precision torch ops round.
 *
 * uv_embed_norm: x = rms_norm(embed[tok]); xn = rms_norm(x)            (fast_decode.py:284, :303)
 * uv_qkv_post:   in place on the packed QKV GEMM output qkv (B, (H+2K)*hd): value-embedding gate
 *                v += 2*sigmoid(xn[:, :ve_ch] . ve_gate) * value_embed[tok] (when ve_gate != NULL), per-head RMS norm
 *                of q and k, partial RoPE with angles pos * inv_freq (when inv_freq != NULL; pairs j <-> j + n_pairs),
 *                then K and V quantised and appended to the int8 cache at slot pos (ring: pos % S) when k_cache !=
 *                NULL (Attention.qkv, ultraviolet/model.py:302-320; kv_write, kv_quant.py:26-36); row_map as in
 *                uv_attn_args (cache row of batch entry b); S_alloc (0 = S) = slots allocated per cache row
 * uv_resid_norm: h = lambdas[0]*x + lambdas[1]*a; hn = rms_norm(h)     (Block.finish, model.py:567-571)
 * uv_swiglu:     act = silu(gu[:, :f]) * gu[:, f:]                     (MLP.forward, model.py:388-391)
 */
int uv_embed_norm(const int64_t* tok, const void* embed, int dtype, int64_t vocab, int d, void* x, void* xn, int B,
                  void* stream);
/* uv_embed_norm that also writes the step's RoPE table rope_cs (B, 2*n_pairs) fp32: cos(pos*inv_freq[j]) for j <
 * n_pairs, then the sines, each rounded to dtype (the cos / sin operands of apply_rope, fast_decode.py:286-290). */
int uv_embed_norm_rope(const int64_t* tok, const void* embed, int dtype, int64_t vocab, int d, void* x, void* xn,
                       int B, const int64_t* pos, const float* inv_freq, int n_pairs, float* rope_cs, void* stream);
/* The same kernel for the tensor-core GEMM path: also writes the sum of squares of every x row as ss_out (ss_parts,
 * ss_ld) fp32 (the whole sum in part 0, zeros in the rest), the form uv_gemm_sw* take as ss_in; xn may then be NULL. */
int uv_embed_norm_ss(const int64_t* tok, const void* embed, int dtype, int64_t vocab, int d, void* x, void* xn, int B,
                     const int64_t* pos, const float* inv_freq, int n_pairs, float* rope_cs, float* ss_out,
                     int ss_parts, int ss_ld, void* stream);
int uv_qkv_post(void* qkv, const void* xn, const int64_t* tok, const void* value_embed, const void* ve_gate,
                const float* inv_freq, const int64_t* pos, int8_t* k_cache, int8_t* v_cache, uint16_t* k_scale,
                uint16_t* v_scale, const int64_t* row_map, int* oob_count, int dtype, int64_t vocab, int B, int H, int K,
                int hd, int d, int S, int S_alloc, int ring, int ve_ch, int n_pairs, void* stream);
int uv_resid_norm(const void* x, const void* a, const float* lambdas, int dtype, int d, void* h, void* hn, int B,
                  void* stream);
int uv_swiglu(const void* gu, int dtype, int f, void* act, int B, void* stream);
/* uv_swiglu with the deferred RMS norm: gu = h . [Wg ; Wu]^T computed on the UN-normalised rows h (B, d); the kernel
 * forms rs = rsqrt(mean(h[b]^2) + 2^-23) and returns act = silu(g * rs) * (u * rs) (MLP.forward on rms_norm(h),
 * ultraviolet/model.py:388-391, :567-571). */
int uv_swiglu_rs(const void* gu, const void* h, int dtype, int d, int f, void* act, int B, void* stream);

/* uv_qkv_attn: uv_qkv_post followed by uv_decode_attn on the same rows, as ONE launch.  The attention CTAs do the
 * per-head post-processing of their row in their prologue, while the bulk copies of the older cache tiles are already
 * in flight; the split that owns position pos appends the new key / value and only then copies that tile.  Both
 * argument blocks must describe the same step: same B / H / K / hd / S / ring, the same pos, row_map, cache and scale
 * pointers; attn->q = qkv, attn->v_cur = the value slots of qkv; cache rows contiguous with S_alloc slots.  The
 * one-launch form needs the bulk-copy path, arrival counters for more than 8 splits and, on layers with RoPE, the
 * rope_cs table; otherwise the function runs the two launches itself.  qkv is left unmodified by the one-launch form and post-processed in place by the
 * two-launch form: callers must not read it afterwards. */
typedef struct uv_qkv_args { /* the parameters of uv_qkv_post, by name */
  void* qkv;
  const void* xn;
  const int64_t* tok;
  const void* value_embed;
  const void* ve_gate;
  const float* inv_freq;
  const int64_t* pos;
  int8_t* k_cache;
  int8_t* v_cache;
  uint16_t* k_scale;
  uint16_t* v_scale;
  const int64_t* row_map;
  int* oob_count;
  int dtype;
  int64_t vocab;
  int B, H, K, hd, d, S, S_alloc, ring, ve_ch, n_pairs;
  const float* rope_cs;   /* optional (B, 2*n_pairs) table from uv_embed_norm_rope for these pos: read instead of
                             evaluating cos / sin in every layer (same values bit for bit) */
  const void* gate_w;     /* optional, uv_qkv_post_args only: (H, gate_ch) attention output gate weights; the kernel */
  float* gate_out;        /* also writes gate_out (B, H) = 2*sigmoid(xn[b, :gate_ch] . gate_w[head]) for the */
  int gate_ch;            /* attention launch that follows (uv_attn_args.gate_vals) */
  const int64_t* last_pos; /* optional (B,), packed prefill: the last position of batch entry b's sequence in THIS
                             launch.  A ring cache then keeps only the newest S positions of a sequence (entries with
                             pos + S <= last_pos are not written), as _write_kv_layers does (ultraviolet/kernels/
                             fast_decode.py:166-207), so that no two rows of one launch write the same slot */
  int xn_raw;              /* uv_qkv_post_args only.  1: xn holds the UN-normalised residual rows and qkv the projection
                             of those rows; the kernel forms rs = rsqrt(mean(xn[b]^2) + 2^-23) itself, scales the
                             projection by it and reads rms_norm(xn) on the fly for the gates (deferred RMS norm: the
                             step then needs no separate norm kernel in front of the QKV GEMM) */
} uv_qkv_args;
int uv_qkv_attn(const uv_qkv_args* qkv, const uv_attn_args* attn, void* stream);
/* uv_qkv_post with its parameters by name; with rope_cs set the rotation reads the step's table. */
int uv_qkv_post_args(const uv_qkv_args* qkv, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * (f1) Packed variable-length prefill attention.  Replaces the attention of the reference's prompt prefill: SDPA
 * over the left-padded batch in prefill_fast (ultraviolet/kernels/fast_decode.py:70-114) and varlen_attention over
 * the packed batch in _prefill_packed (fast_decode.py:117-163, ultraviolet/kernels/varlen_attn.py:38-92).
 *
 * qkv (M, (H + 2K) * hd) holds the post-processed rows of ALL prompts of a refill batch back to back (q heads, then
 * k heads, then v heads, as uv_qkv_post leaves them: normalised / rotated q and k, v with its value embedding).
 * cu_seqlens (n_seq + 1) int32: first row of every sequence; tile_cu (n_seq + 1) int32: tile_cu[s] = sum over
 * s' < s of ceil(len_s' / 16) (the kernel works in 16-token query tiles; max_tiles >= tile_cu[n_seq] is the grid,
 * blocks beyond the last tile exit, so both arrays may be built on the device).  Token i of a sequence attends to
 * tokens max(0, i - window + 1) .. i of the same sequence (window 0 = unlimited) with the UNQUANTISED keys / values
 * of the chunk; out (M, H * hd) gets softmax(scale * q.K^T) V per query head, followed by the optional epilogue of
 * uv_attn_args (XSA with the token's own v, then gate_vals (M, H)).  hd in {16, 32, 64, 128}, H / K <= 16. */
typedef struct uv_prefill_attn_args {
  const void* qkv;
  int dtype;              /* UV_F16 | UV_BF16 */
  int64_t ld;             /* row stride of qkv in elements (ld * 2 bytes a multiple of 16) */
  const int32_t* cu_seqlens;
  const int32_t* tile_cu;
  int n_seq, max_tiles;
  void* out;
  int64_t ldo;
  int H, K, hd, window;
  float scale;
  const float* xsa_alpha; /* (H,) fp32, already tanh'ed, or NULL */
  float xsa_eps;
  const float* gate_vals; /* (M, H) fp32 or NULL */
} uv_prefill_attn_args;
int uv_prefill_attn(const uv_prefill_attn_args* args, void* stream);

/* GEMMs of the decode step with the row-wise kernels above fused into their epilogues (hand-written mma.sync
 * mainloop; same results as library GEMM + the separate kernel up to the summation order of the fp32 accumulation).
 * Activations (B, K) row-major with row stride ld*, weights (N, K) row-major contiguous, K % 64 == 0.
 *   uv_gemm_qkv:        qkv = xn . wqkv^T followed by everything uv_qkv_post does (head_dim 64 only)
 *   uv_gemm_swiglu:     act = silu(hn . Wg^T) * (hn . Wu^T), w_gu = [Wg ; Wu] (2f, d), f % 32 == 0
 *   uv_gemm_resid_norm: h = lambdas[0]*x + lambdas[1]*(a . w^T), hn = rms_norm(h); d % 80 == 0 and d <= 640 (the d
 *                       columns are split over a thread-block cluster of d/80 CTAs whose row sums meet in
 *                       distributed shared memory) */
int uv_gemm_qkv(const void* xn, int64_t ldx, const void* wqkv, void* qkv, const int64_t* tok, const void* value_embed,
                const void* ve_gate, const float* inv_freq, const int64_t* pos, int8_t* k_cache, int8_t* v_cache,
                uint16_t* k_scale, uint16_t* v_scale, const int64_t* row_map, int* oob_count, int dtype, int64_t vocab,
                int B, int H, int KH, int hd, int d, int S, int S_alloc, int ring, int ve_ch, int n_pairs, void* stream);
int uv_gemm_swiglu(const void* hn, int64_t ldh, const void* w_gu, void* act, int dtype, int B, int d, int f,
                   void* stream);
int uv_gemm_resid_norm(const void* a, int64_t lda, const void* w, int K, const void* x, const float* lambdas, void* h,
                       void* hn, int dtype, int B, int d, void* stream);

/* Decode-step GEMMs on the tcgen05 tensor cores with the row-wise kernels fused into their epilogues (the default
 * GEMM path of the engine for bf16 models whose shapes fit: head_dim 64, K % 64 == 0, N % 128 == 0).  They replace the
 * library GEMMs of decode_step_fast (ultraviolet/kernels/fast_decode.py:303-330: the fused wqkv / wo / gate|up / down
 * matmuls of Attention.qkv, Attention.post, MLP.forward and Block.finish, ultraviolet/model.py:302-335, :388-391,
 * :567-571) together with the elementwise ops between them.
 *
 * Tiling: 128 weight rows per CTA on the TMEM lanes, a tile of bn batch rows as the MMA's N (bn_hint 32 / 64 / 128,
 * 0 = automatic); ks_hint splits K over a thread-block cluster (0 = automatic, <= 8) with the partials summed
 * through distributed shared memory.  Weights are requested before griddepcontrol.wait, activations after it.
 *
 * Deferred RMS norm: ss_in (ss_parts, ss_ld) fp32 holds per-feature-tile sums of squares of the INPUT rows (written
 * by uv_gemm_sw_resid or uv_embed_norm_ss); the kernel multiplies row b of its result by
 * rsqrt(sum_j ss_in[j][b] / K + 2^-23), i.e. it computes rms_norm(x) . w^T from the un-normalised x.  ss_in = NULL:
 * no scaling.
 *   uv_gemm_sw         c (M, N) = [rms_norm](x) . w^T                                   (building block)
 *   uv_gemm_sw_qkv     the QKV projection + everything uv_qkv_post_args does (args->xn is ignored: the gates read
 *                      x scaled on the fly; args->rope_cs is required on RoPE layers).  ss_in = NULL here means
 *                      "nobody left sums of squares behind": the kernel forms sum(x[b]^2) itself from the
 *                      activation tiles it stages (all K blocks of a CTA must fit its stage ring, else
 *                      UV_ERR_SHAPE) and the launch carries the programmatic-dependent-launch attribute so that
 *                      its weight tiles are requested while the previous kernel drains (ss_parts = -1: without it)
 *   uv_gemm_sw_swiglu  act (M, f) = silu(g) * u, [g | u] = rms_norm(h) . w_gu^T, w_gu = [Wg ; Wu] (2f, K), f % 64 == 0
 *   uv_gemm_sw_resid   h = lambdas[0] * x + lambdas[1] * (a . w^T) (each product and the sum rounded, Block.finish)
 *                      and ss_out[tile][b] = sum over the tile's 128 features of h[b]^2 (N / 128 tiles)
 * status (optional device word): bit 2 is set when a bounded wait ran out (outputs then undefined). */
int uv_gemm_sw(const void* x, int64_t ldx, const void* w, void* c, int64_t ldc, int dtype, int M, int N, int K,
               const float* ss_in, int ss_parts, int ss_ld, int bn_hint, int ks_hint, int* status, void* stream);
int uv_gemm_sw_qkv(const void* x, int64_t ldx, const void* wqkv, const uv_qkv_args* args, const float* ss_in,
                   int ss_parts, int ss_ld, int bn_hint, int ks_hint, int* status, void* stream);
int uv_gemm_sw_swiglu(const void* h, int64_t ldh, const void* w_gu, void* act, int dtype, int M, int K, int f,
                      const float* ss_in, int ss_parts, int ss_ld, int bn_hint, int* status, void* stream);
int uv_gemm_sw_resid(const void* a, int64_t lda, const void* w, const void* x, const float* lambdas, void* h,
                     int64_t ldh, float* ss_out, int ss_out_ld, int dtype, int M, int N, int K, int bn_hint,
                     int ks_hint, int* status, void* stream);

/* uv_sample: softcap + token draw + behaviour log-prob per row of the LM-head output x (B, V), V % 256 == 0.
 * Replaces fused_sample (ultraviolet/kernels/fused_sample.py:68-78) and sample + the log-prob gather
 * (ultraviolet/model.py:1160-1169, :1194-1211).  precapped = 0: x is the raw head output and z = a*sigmoid((x+b)/c)
 * is applied here; precapped = 1: x already holds logits z (cap_* ignored).  temperature <= 0: argmax (first index
 * on ties), logp reported at T = 1.  temperature > 0: inverse-CDF draw of softmax(z / T) restricted to the top_p
 * nucleus (top_p >= 1: none), with one uniform per row taken from u (B,) or, when u == NULL, from Philox4x32-10 with
 * key = seed and counter = (steps[row], row_keys[row]).  logp = log softmax(z / T)[token] over the FULL vocabulary.
 * inc_a / inc_b (optional, (B,) int64): counters advanced by one per row after the draw -- the decode step passes
 * the cache positions and the Philox step counters here instead of launching two more kernels. */
int uv_sample(const void* x, int x_dtype, int64_t x_stride, int B, int V, int precapped, float cap_a, float cap_b,
              float cap_c, float temperature, float top_p, const float* u, uint64_t seed, const int64_t* row_keys,
              const int64_t* steps, int64_t* tok_out, float* logp_out, int64_t* inc_a, int64_t* inc_b, void* stream);
/* uv_sample_topk: uv_sample with the top_k filter of sample() (ultraviolet/model.py:1201-1203) applied before the
 * nucleus: only the top_k largest logits of a row (ties with the k-th kept) can be drawn, and top_p then acts on
 * that renormalised set.  top_k = 0: no limit (uv_sample is this call with top_k = 0).  logp stays the log-softmax
 * over the full vocabulary. */
int uv_sample_topk(const void* x, int x_dtype, int64_t x_stride, int B, int V, int precapped, float cap_a, float cap_b,
                   float cap_c, float temperature, int top_k, float top_p, const float* u, uint64_t seed,
                   const int64_t* row_keys, const int64_t* steps, int64_t* tok_out, float* logp_out, int64_t* inc_a,
                   int64_t* inc_b, void* stream);

/* GEMM on the tcgen05 tensor cores with TMEM accumulators and TMA operand tiles (bf16 only; K % 64 == 0; A (M, K)
 * row stride lda, W (N, K) row stride ldw, 16-byte aligned rows).  The tensor maps are encoded on the host at every
 * call (driver entry point cuTensorMapEncodeTiled): nothing is cached, nothing is allocated.
 *   uv_gemm_tc:        C (M, N) = A . W^T, N % 64 == 0
 *   uv_gemm_tc_swiglu: act (M, f) = silu(A . Wg^T) * (A . Wu^T) with w_gu = [Wg ; Wu] (2f, K) contiguous, f % 32 == 0;
 *                      same rounding points as library GEMM + uv_swiglu
 * status: optional device word, bit 2 is set if a bounded wait inside the kernel ran out (output then undefined). */
int uv_gemm_tc(const void* a, int64_t lda, const void* w, int64_t ldw, void* c, int64_t ldc, int dtype, int M, int N,
               int K, int* status, void* stream);
int uv_gemm_tc_swiglu(const void* a, int64_t lda, const void* w_gu, void* act, int dtype, int M, int K, int f,
                      int* status, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * (a) GPU-resident continuous-batching scheduler.  Replaces the host loops of StreamGen.chunk / _refill / _park
 * (scripts/rl_stream.py:76-147) and generate_continuous (ultraviolet/model.py:1266-1354): one single-CTA kernel per
 * decode step, no host round trip.  All arrays are device memory owned by the caller; rings are addressed by
 * absolute indices modulo their capacity.
 *
 * uv_sched_step, run after the sampler of every step: for each slot with a request, either feed the next prompt
 * token (prefill as decode; the sample is discarded) or append (samp_tok, samp_lp) to the request's output range and
 * retire it on EOS (eos >= 0), on reaching limit[r] tokens (force_eos: the last allowed token is replaced by EOS,
 * the "stop length" of synthetic benchmarks) or when the cache row is full (status bit 1).  Retired requests get
 * out_len[r] and are pushed to fin_ring; free slots then take the next queued requests in slot order (ranks by
 * block prefix sum) with cur_tok = first prompt token, pos = starts = 0, row_key = key[r], step_ctr = 0,
 * start_version[r] = ctl[3]; slots left without work are parked at pos 0 with cur_tok = pad.
 *
 * uv_sched_enqueue(n): the host has copied prompt_len / limit / key of n new requests to ring entries
 * [tail, tail+n) and their tokens back to back at absolute token offset ctl[7]; the kernel assigns prompt_off and
 * out_off by prefix sum (each request owns limit[r] output slots), clears out_len and publishes tail += n.
 *
 * ctl (int64[16]): [0] head  [1] tail  [2] finished count  [3] weight version (host-written)  [4] active slots
 *                  [5] status bits  [6] steps run  [7] prompt-token tail  [8] output-slot tail
 *                  [9] tokens generated so far  [10] active slots summed over steps (occupancy = [10] / ([6] * B))
 *                  [11] packed prefill rows used by uv_sched_admit passes  [12] admission passes run
 */
typedef struct uv_sched_args {
  int* req; int* fed; int* gen;                 /* per slot (B,) */
  int64_t* cur_tok; int64_t* pos; int64_t* starts; int64_t* row_key; int64_t* step_ctr;
  const int64_t* samp_tok; const float* samp_lp; /* sampler output of the step just run (B,) */
  int64_t* prompt_off; int* prompt_len; int* limit; int64_t* key; int64_t* out_off; int* out_len;
  int* start_version;                            /* request rings (q_cap,) */
  const int* tokens;                             /* prompt-token ring (tok_cap,) */
  int* out_tok; float* out_lp;                   /* output rings (out_cap,) */
  int* fin_ring;                                 /* (q_cap,) */
  int64_t* ctl;                                  /* (16,) */
  int B, q_cap;
  int64_t tok_cap, out_cap;
  int eos, pad, force_eos;
  int64_t max_len;
  /* Prefill lanes (0 = off).  cur_tok / pos / starts then have B + lanes entries and row_map (B + lanes,) names the
   * cache row of every batch row of the decode step ([0, B): the identity).  A slot still feeding its prompt gets up
   * to lane_chunk - 1 lane rows per step, which carry its next prompt tokens at consecutive positions of its cache
   * row while its own row moves to the last token of the chunk: a prompt of P tokens takes about P / lane_chunk
   * steps.  Idle lanes are parked on cache row B (one spare row).  A chunk never crosses position ring_len - 1 (the
   * length of the shortest ring cache), where a wrapped write would overwrite keys the chunk still reads. */
  int64_t* row_map;
  int lanes, lane_chunk;
  int64_t ring_len;
  /* 1: uv_sched_step only retires (freed slots are parked); queued requests enter through uv_sched_admit passes */
  int no_admit;
  /* 1 (needs no_admit = 1, lanes = 0, row_map (B,) initialised to the identity, B <= 4096): a step that retires
   * something moves the live slots down to batch rows [0, active), keeping their order; row_map[b] stays the cache
   * row of batch row b (a permutation of [0, B); uv_sched_admit hands it to the packed prefill), so the caller can
   * run the decode step on the first n >= active rows only.  Request outputs do not depend on it. */
  int compact;
  /* Deferred admission (all optional, no_admit mode).  step_row (B,) is the cache row the decode step should use
   * for batch row b: row_map[b] while the slot is live, the spare row B otherwise (pass it to uv_decode_attn /
   * uv_qkv_post as their row_map), so that parked rows never write into a cache row an admission pass is filling.
   * With ctl[14] (defer) = 1, uv_sched_admit leaves the admitted requests in the pend_* arrays (B,) instead of the
   * slot state; uv_sched_commit, launched after that pass's prefill, makes them live.  The caller sets ctl[13]
   * (in flight) = 1 on the step's stream before it launches such a pass on another stream: the step kernel then
   * does not compact and notes the owed compaction in ctl[15]. */
  int64_t* step_row;
  int* pend_req; int* pend_fed;
  int64_t* pend_tok; int64_t* pend_pos; int64_t* pend_key;
} uv_sched_args;

int uv_sched_step(const uv_sched_args* args, void* stream);

/* uv_sched_admit: one admission pass of the no_admit mode -- the device-side counterpart of StreamGen._refill's
 * batched prefill (scripts/rl_stream.py:76-101; packed form: ultraviolet/kernels/fast_decode.py:210-269).  Queued
 * requests, in queue order, take the free slots, in slot order, while their prompts fit `cap` packed rows (the
 * admitted set is a prefix of the queue).  A request of P prompt tokens contributes tokens 0 .. P - 2 as packed rows
 * (tok / pos / row / last_pos, the inputs of one packed prefill pass: uv_prefill_attn with cu / tile_cu as its
 * cu_seqlens / tile_cu over n_seq = B sequences, unused entries empty) and its slot is left with the last prompt
 * token at position P - 1 for the next decode step.  Unused rows carry the pad token on cache row B (a spare row the
 * caller allocates).  ctl[0] (head) advances by the number admitted; ctl[11] accumulates the rows used. */
typedef struct uv_sched_admit_args {
  int64_t* tok; int64_t* pos; int64_t* row; int64_t* last_pos;   /* (cap,) */
  int32_t* cu; int32_t* tile_cu;                                 /* (B + 1,) */
  int cap;
  int reserved_;
} uv_sched_admit_args;
int uv_sched_admit(const uv_sched_args* args, const uv_sched_admit_args* pass, void* stream);
/* uv_sched_commit: the slots a deferred admission pass filled (pend_req[s] >= 0) go live; clears ctl[13] / ctl[14],
 * sets ctl[15].  Order it after the pass's prefill kernels. */
int uv_sched_commit(const uv_sched_args* args, void* stream);
int uv_sched_enqueue(const uv_sched_args* args, int n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* UVDECODE_H_ */
