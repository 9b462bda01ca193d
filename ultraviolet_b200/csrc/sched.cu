// GPU-resident continuous-batching scheduler: after every decode step one small kernel retires finished
// sequences (EOS, per-request token limit, cache full), appends the sampled token / log-prob to the request's
// output range, admits queued requests into the freed slots (free-slot ranks by block prefix sum) and sets each
// slot's next input token and cache position.  The host never takes part in a step: it appends requests to the
// device queue and harvests finished ones whenever it likes.
//
// It reproduces the per-request output contract of the reference's host schedulers (StreamGen.chunk,
// scripts/rl_stream.py:103-147; generate_continuous, ultraviolet/model.py:1266-1354): generated tokens up to and
// including the first EOS, at most `limit` of them (limit = min(max_new, target_len)), one behaviour log-prob per
// token, the weight version at admission.  A newly admitted request is prefilled by feeding its prompt through the
// decode step one token per step (sampling output ignored until the last prompt token), starting at position 0.
//
// Queue layout (rings addressed by absolute, monotonically increasing indices):
//   requests  index r -> r % q_cap : prompt_off, prompt_len, limit, key, out_off, out_len, start_version
//   prompt tokens        absolute offset % tok_cap        (packed back to back; offsets by prefix sum at enqueue)
//   outputs              absolute offset % out_cap        (each request owns `limit` slots; offsets by prefix sum)
#include <string.h>

#include "common.cuh"

namespace uv {

constexpr int SCHED_THREADS = 1024;

struct SchedParams {
  // per slot
  int* req;            // request index or -1
  int* fed;            // prompt tokens fed so far (including the one in cur_tok)
  int* gen;            // tokens generated so far
  int64_t* cur_tok;    // next input token of the slot (the decode step's tok vector)
  int64_t* pos;        // cache position cur_tok is written at
  int64_t* starts;     // first valid position (always 0 in this frame)
  int64_t* row_key;    // Philox key of the sequence in the slot
  int64_t* step_ctr;   // Philox counter = index of the token being generated
  // sampler output of the step just run
  const int64_t* samp_tok;
  const float* samp_lp;
  // request rings
  int64_t* prompt_off;
  int* prompt_len;
  int* limit;
  int64_t* key;
  int64_t* out_off;
  int* out_len;        // -1 until finished
  int* start_version;
  const int* tokens;
  int* out_tok;
  float* out_lp;
  int* fin_ring;       // request indices in finishing order (ring of q_cap)
  // control words: [0] head (next request to admit) [1] tail (requests enqueued) [2] finished count
  //                [3] weight version [4] active slots after this step [5] status bits [6] steps run
  //                [7] prompt-token tail [8] output-slot tail [9] tokens generated [10] sum of active slots per step
  int64_t* ctl;
  int B, q_cap;
  int64_t tok_cap, out_cap;
  int eos, pad, force_eos;
  int64_t max_len;
  // prefill lanes: rows [B, B + lanes) of cur_tok / pos / starts / row_map are extra batch rows of the decode step.
  // A slot that is still feeding its prompt gets up to lane_chunk - 1 of them per step: the lanes carry the next
  // prompt tokens at consecutive positions of the slot's cache row (row_map = slot) and the slot's own row moves to
  // the last token of the chunk, so a prompt of P tokens takes P / lane_chunk steps instead of P.  Idle lanes are
  // parked on cache row B (one spare row the caller allocates).
  int64_t* row_map;    // (B + lanes,) cache row of every batch row; [0, B) is the identity
  int lanes, lane_chunk;
  int64_t ring_len;    // length of the shortest ring cache: a chunk never wraps it (a wrapped write would destroy
                       // keys that the chunk's earlier positions still attend to)
  // 1: the step kernel only retires; freed slots are parked and queued requests wait for an admission pass
  // (sched_admit_kernel + packed prefill) that the host launches between steps
  int no_admit;
  // 1 (with no_admit): after a step that retired something, the live slots are moved down so that they occupy
  // batch rows [0, active) in their old order.  A slot's cache row moves with it through row_map, which stays a
  // permutation of [0, B) (the rows of retired slots go to the tail); outputs and Philox streams are addressed by
  // request, not by slot, so nothing a request produces depends on the move.  The host can then run the decode
  // step on the first n >= active batch rows only.
  int compact;
  // Deferred admission (optional; no_admit mode): an admission pass may run BESIDE the decode steps, on another
  // stream.  It then writes the admitted requests into the pend_* arrays instead of the slot state (ctl[DEFER] = 1),
  // and uv_sched_commit makes them live once the pass's prefill has finished.  While a pass is in flight
  // (ctl[INFLIGHT]) the step kernel does not compact -- the pass has chosen slots and cache rows -- and remembers
  // in ctl[DIRTY] that it owes a compaction.  step_row (B,) is what the decode step uses as the cache row of batch
  // row b: row_map[b] while the slot is live, the spare row B otherwise, so that the parked rows of a step never
  // write into a cache row that a pass is filling.
  int64_t* step_row;
  int* pend_req;       // (B,) request waiting in slot s for its commit, or -1
  int* pend_fed;
  int64_t* pend_tok;
  int64_t* pend_pos;
  int64_t* pend_key;
};

constexpr int COMPACT_MAX_SLOTS = 4096;  // the new row_map is staged in shared memory

// One admission pass: packed prefill inputs for the requests it admits.
struct AdmitParams {
  int64_t* tok;        // (cap,) token of every packed row
  int64_t* pos;        // (cap,) its position inside its prompt
  int64_t* row;        // (cap,) its cache row (the slot); unused rows point at the spare row B
  int64_t* last_pos;   // (cap,) last prefilled position of its prompt
  int* cu;             // (B + 1,) first packed row of the q-th admitted request (unused entries = rows used)
  int* tile_cu;        // (B + 1,) first 16-token tile likewise
  int cap;             // packed rows available in this pass
  int reserved_;
};

enum { CTL_HEAD = 0, CTL_TAIL, CTL_FIN, CTL_VERSION, CTL_ACTIVE, CTL_STATUS, CTL_STEPS, CTL_TOK_TAIL, CTL_OUT_TAIL,
       CTL_GENERATED, CTL_SLOT_STEPS, CTL_PREFILL_ROWS, CTL_ADMIT_PASSES, CTL_INFLIGHT, CTL_DEFER, CTL_DIRTY };

__device__ __forceinline__ int block_excl_scan(int v, int* warp_tot, int tid, int& total) {
  const int lane = tid & 31, warp = tid >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int base = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < SCHED_THREADS / 32; ++w) {
    const int t = warp_tot[w];
    if (w < warp) base += t;
    tot += t;
  }
  total = tot;
  return base + incl - v;
}

// The same scan over three counters at once, packed 20 bits each into one 64-bit word (a chunk holds at most
// SCHED_THREADS = 2^10 ones per counter): one pass through the barriers instead of three.
__device__ __forceinline__ unsigned long long pack3(int a, int b, int c) {
  return (unsigned long long)a | ((unsigned long long)b << 20) | ((unsigned long long)c << 40);
}
__device__ __forceinline__ int field(unsigned long long v, int i) { return (int)((v >> (20 * i)) & 0xfffffull); }
__device__ __forceinline__ unsigned long long block_excl_scan3(unsigned long long v, unsigned long long* warp_tot,
                                                               int tid, unsigned long long& total) {
  const int lane = tid & 31, warp = tid >> 5;
  unsigned long long incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  // every warp scans the 32 warp totals itself: lane w holds the total of warp w
  unsigned long long wt = warp_tot[lane], wincl = wt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, wincl, o);
    if (lane >= o) wincl += t;
  }
  total = __shfl_sync(0xffffffffu, wincl, 31);
  const unsigned long long base = __shfl_sync(0xffffffffu, wincl - wt, warp);
  return base + incl - v;
}

__global__ void __launch_bounds__(SCHED_THREADS) sched_step_kernel(const __grid_constant__ SchedParams P) {
  __shared__ int warp_tot[SCHED_THREADS / 32];
  __shared__ unsigned long long warp_tot3[SCHED_THREADS / 32];
  static_assert(SCHED_THREADS == 1024, "block_excl_scan3 scans the warp totals with one warp: 32 warps");
  const int tid = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  const int64_t head0 = P.ctl[CTL_HEAD], tail = P.ctl[CTL_TAIL];
  const int version = (int)P.ctl[CTL_VERSION];
  int64_t head = head0;
  const int64_t fin0 = P.ctl[CTL_FIN];
  int64_t fin_base = fin0;
  const bool inflight = P.ctl[CTL_INFLIGHT] != 0, dirty = P.ctl[CTL_DIRTY] != 0;
  int active = 0, generated = 0;
  for (int base = 0; base < P.B; base += SCHED_THREADS) {  // uniform trip count: every thread joins every scan
    const int s = base + tid;
    const bool in = s < P.B;
    int freed = 0, finished = 0, fin_req = -1, emitted = 0;
    if (in) {
      const int r = P.req[s];
      if (r < 0) {
        freed = 1;
      } else {
        const int ri = r % P.q_cap;
        const int f = P.fed[s];
        if (f < P.prompt_len[ri]) {  // still prefilling: next prompt token, the sample is discarded
          P.cur_tok[s] = P.tokens[(P.prompt_off[ri] + f) % P.tok_cap];
          P.fed[s] = f + 1;
          P.pos[s] += 1;
        } else {
          int g = P.gen[s];
          const int lim = P.limit[ri];
          int64_t t = P.samp_tok[s];
          if (P.force_eos && g + 1 >= lim) t = P.eos;
          const int64_t o = (P.out_off[ri] + g) % P.out_cap;
          P.out_tok[o] = (int)t;
          P.out_lp[o] = P.samp_lp[s];
          ++g;
          emitted = 1;
          const bool full = P.pos[s] + 1 >= P.max_len;
          if ((P.eos >= 0 && t == P.eos) || g >= lim || full) {
            P.out_len[ri] = g;
            finished = 1, fin_req = r;
            if (full && g < lim)
              atomicOr(reinterpret_cast<unsigned long long*>(P.ctl + CTL_STATUS), 2ull);  // cut short: cache full
            if (P.step_row) P.step_row[s] = P.B;  // from the next step on this batch row works on the spare cache row
            P.req[s] = -1;
            freed = 1;
          } else {
            P.gen[s] = g;
            P.cur_tok[s] = t;
            P.pos[s] += 1;
            P.step_ctr[s] = g;
          }
        }
      }
    }
    // ---- one packed scan: finished requests enter the ring in slot order (deterministic harvest order), emitted
    //      tokens are only counted, freed slots get their rank among the chunk's free slots
    unsigned long long tot3;
    const unsigned long long pre3 = block_excl_scan3(pack3(finished, emitted, freed), warp_tot3, tid, tot3);
    const int frank = field(pre3, 0), total_fin = field(tot3, 0);
    if (finished) P.fin_ring[(fin_base + frank) % P.q_cap] = fin_req;
    fin_base += total_fin;
    generated += field(tot3, 1);
    // ---- admit queued requests into the free slots of this chunk, in slot order
    const int rank = field(pre3, 2), total_free = field(tot3, 2);
    const int64_t avail = P.no_admit ? 0 : tail - head;
    if (in && freed) {
      if (rank < avail) {
        const int64_t r = head + rank;
        const int ri = (int)(r % P.q_cap);
        P.req[s] = (int)r;
        P.fed[s] = 1;
        P.gen[s] = 0;
        P.cur_tok[s] = P.tokens[P.prompt_off[ri] % P.tok_cap];
        P.pos[s] = 0;
        P.starts[s] = 0;
        P.row_key[s] = P.key[ri];
        P.step_ctr[s] = 0;
        P.start_version[ri] = version;
        if (P.step_row) P.step_row[s] = P.row_map ? P.row_map[s] : (int64_t)s;
      } else {  // nothing queued: park the slot at position 0 so it never overruns the cache (model.py:1345-1350)
        P.cur_tok[s] = P.pad;
        P.pos[s] = 0;
        P.starts[s] = 0;
      }
    }
    const int admitted = total_free < avail ? total_free : (int)avail;
    head += admitted;
    // slots of this chunk that hold a request after the step: the ones that kept theirs plus the admissions
    const int n_in = P.B - base < SCHED_THREADS ? P.B - base : SCHED_THREADS;
    active += n_in - total_free + admitted;
  }
  // ---- compaction (see SchedParams::compact): stable partition of the slots into live ones, then free ones
  const bool owes = fin_base != fin0 || dirty;
  if (P.compact && owes && inflight && tid == 0) P.ctl[CTL_DIRTY] = 1;  // a pass holds slots and rows: later
  if (P.compact && owes && !inflight) {  // uniform: every thread has the same totals and flags
    __shared__ int rm_new[COMPACT_MAX_SLOTS];
    int live_before = 0;
    for (int base = 0; base < P.B; base += SCHED_THREADS) {
      const int s = base + tid;
      const bool in = s < P.B;
      const int r = in ? P.req[s] : -1;
      const bool live = r >= 0;
      int fed = 0, gen = 0, rm = 0;
      int64_t ct = 0, po = 0, sta = 0, rk = 0, sc = 0;
      if (in) rm = (int)P.row_map[s];
      if (live) fed = P.fed[s], gen = P.gen[s], ct = P.cur_tok[s], po = P.pos[s], sta = P.starts[s],
                rk = P.row_key[s], sc = P.step_ctr[s];
      int total;
      const int rank = block_excl_scan(live ? 1 : 0, warp_tot, tid, total);  // its barriers order reads before writes
      if (in) {
        // live slots only ever move down (dst <= s), onto slots of this or an earlier chunk, all read by now
        const int dst = live ? live_before + rank : active + (s - live_before - rank);
        rm_new[dst] = rm;
        if (live && dst != s) {
          P.req[dst] = r, P.fed[dst] = fed, P.gen[dst] = gen, P.cur_tok[dst] = ct, P.pos[dst] = po;
          P.starts[dst] = sta, P.row_key[dst] = rk, P.step_ctr[dst] = sc;
        }
      }
      live_before += total;
    }
    __syncthreads();
    for (int s = tid; s < P.B; s += SCHED_THREADS) {
      P.row_map[s] = rm_new[s];
      if (P.step_row) P.step_row[s] = s < active ? (int64_t)rm_new[s] : (int64_t)P.B;
      if (s >= active) P.req[s] = -1, P.cur_tok[s] = P.pad, P.pos[s] = 0, P.starts[s] = 0;
    }
    if (tid == 0) P.ctl[CTL_DIRTY] = 0;
  }
  // ---- prefill lanes (see SchedParams): hand out the lane rows in slot order by prefix sum
  if (P.lanes > 0) {
    int used = 0;
    for (int base = 0; base < P.B; base += SCHED_THREADS) {
      const int s = base + tid;
      int want = 0, f = 0, ri = 0;
      int64_t p = 0;
      if (s < P.B && P.req[s] >= 0) {
        ri = P.req[s] % P.q_cap;
        f = P.fed[s];                                  // prompt tokens handed out so far (cur_tok is token f - 1)
        p = P.pos[s];
        const int64_t rem = (int64_t)P.prompt_len[ri] - f;  // prompt tokens after cur_tok
        const int64_t room = P.ring_len - 1 - p;       // the chunk's last position must not wrap the ring
        int64_t w = rem < P.lane_chunk - 1 ? rem : P.lane_chunk - 1;
        if (w > room) w = room;
        want = w > 0 ? (int)w : 0;
      }
      int total;
      const int off = block_excl_scan(want, warp_tot, tid, total);
      int grant = want;
      if (used + off >= P.lanes) grant = 0;
      else if (used + off + want > P.lanes) grant = P.lanes - used - off;
      if (grant > 0) {
        const int64_t toff = P.prompt_off[ri];
        for (int j = 0; j < grant; ++j) {              // lanes: tokens f-1 .. f+grant-2 at positions p .. p+grant-1
          const int lane = P.B + used + off + j;
          P.cur_tok[lane] = j == 0 ? P.cur_tok[s] : (int64_t)P.tokens[(toff + f + j - 1) % P.tok_cap];
          P.pos[lane] = p + j;
          P.starts[lane] = 0;
          P.row_map[lane] = s;
        }
        P.cur_tok[s] = P.tokens[(toff + f + grant - 1) % P.tok_cap];  // the slot's row: last token of the chunk
        P.pos[s] = p + grant;
        P.fed[s] = f + grant;
      }
      used = used + total < P.lanes ? used + total : P.lanes;
    }
    for (int l = used + tid; l < P.lanes; l += SCHED_THREADS) {  // idle lanes: the spare cache row, position 0
      P.cur_tok[P.B + l] = P.pad;
      P.pos[P.B + l] = 0;
      P.starts[P.B + l] = 0;
      P.row_map[P.B + l] = P.B;
    }
  }
  if (tid == 0) {
    if (!P.no_admit) P.ctl[CTL_HEAD] = head;  // (no_admit: only admission passes move the head, possibly meanwhile)
    __threadfence();  // ring entries and out_len before the count that publishes them
    P.ctl[CTL_FIN] = fin_base;
    P.ctl[CTL_ACTIVE] = active;
    P.ctl[CTL_STEPS] += 1;
    P.ctl[CTL_GENERATED] += generated;
    P.ctl[CTL_SLOT_STEPS] += active;
  }
}

// Admission pass (no_admit mode): queued requests, in queue order, take the free slots, in slot order, as long as
// their prompts fit the pass's packed rows.  A request of P prompt tokens contributes its first P - 1 tokens as
// packed rows (positions 0 .. P - 2 of its slot's cache row; the packed trunk that follows prefills them in one
// pass) and its slot is left holding the LAST prompt token at position P - 1, which the next decode step consumes
// like any other token -- the sampler's output of that step is generated token 0.  The admitted set is always a
// prefix of the queue: request k is taken iff the prompts of requests 0 .. k fit together.
__global__ void __launch_bounds__(SCHED_THREADS) sched_admit_kernel(const __grid_constant__ SchedParams P,
                                                                    const __grid_constant__ AdmitParams A) {
  __shared__ unsigned long long warp_tot3[SCHED_THREADS / 32];
  const int tid = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  const int64_t head = P.ctl[CTL_HEAD], tail = P.ctl[CTL_TAIL];
  const int version = (int)P.ctl[CTL_VERSION];
  const bool defer = P.pend_req != nullptr && P.ctl[CTL_DEFER] != 0;
  int nseq = 0, rows = 0, tiles = 0;
  bool stop = false;
  for (int base = 0; base < P.B; base += SCHED_THREADS) {  // uniform trip count and uniform `stop`
    const int s = base + tid;
    const bool freed = s < P.B && P.req[s] < 0 && !(P.pend_req != nullptr && P.pend_req[s] >= 0);
    unsigned long long tot;
    // (1) rank among the chunk's free slots -> candidate request
    const unsigned long long pre_a = block_excl_scan3(pack3(freed ? 1 : 0, 0, 0), warp_tot3, tid, tot);
    const int rank = field(pre_a, 0);
    const int64_t r = head + nseq + rank;
    const bool has = !stop && freed && r < tail;
    const int ri = has ? (int)(r % P.q_cap) : 0;
    const int plen = has ? P.prompt_len[ri] : 0;
    const int w = has ? plen - 1 : 0;
    // (2) does the queue prefix up to this request fit?  (inclusive prefix sums are monotone: the set is a prefix)
    const unsigned long long pre_b = block_excl_scan3(pack3(w, has ? 1 : 0, 0), warp_tot3, tid, tot);
    const bool ok = has && rows + field(pre_b, 0) + w <= A.cap;
    const int n_has = field(tot, 1);
    // (3) offsets of the admitted ones
    const unsigned long long pre_c = block_excl_scan3(pack3(ok ? w : 0, ok ? (w + 15) / 16 : 0, ok ? 1 : 0), warp_tot3,
                                                      tid, tot);
    if (ok) {
      const int q = nseq + field(pre_c, 2), row0 = rows + field(pre_c, 0);
      A.cu[q] = row0;
      A.tile_cu[q] = tiles + field(pre_c, 1);
      const int64_t toff = P.prompt_off[ri];
      for (int j = 0; j < w; ++j) {
        A.tok[row0 + j] = P.tokens[(toff + j) % P.tok_cap];
        A.pos[row0 + j] = j;
        A.row[row0 + j] = P.row_map ? P.row_map[s] : (int64_t)s;  // the slot's cache row
        A.last_pos[row0 + j] = w - 1;
      }
      if (defer) {  // the slot goes live at uv_sched_commit, after this pass's prefill
        P.pend_fed[s] = plen;
        P.pend_tok[s] = P.tokens[(toff + plen - 1) % P.tok_cap];
        P.pend_pos[s] = plen - 1;
        P.pend_key[s] = P.key[ri];
        P.pend_req[s] = (int)r;
      } else {
        P.req[s] = (int)r;
        P.fed[s] = plen;
        P.gen[s] = 0;
        P.cur_tok[s] = P.tokens[(toff + plen - 1) % P.tok_cap];
        P.pos[s] = plen - 1;
        P.starts[s] = 0;
        P.row_key[s] = P.key[ri];
        P.step_ctr[s] = 0;
        if (P.step_row) P.step_row[s] = P.row_map ? P.row_map[s] : (int64_t)s;
      }
      P.start_version[ri] = version;
    }
    rows += field(tot, 0);
    tiles += field(tot, 1);
    const int n_ok = field(tot, 2);
    nseq += n_ok;
    if (n_ok < n_has) stop = true;  // the next request does not fit: later (shorter) ones must not overtake it
  }
  // unused sequence entries and packed rows
  for (int q = nseq + tid; q <= P.B; q += SCHED_THREADS) {
    A.cu[q] = rows;
    A.tile_cu[q] = tiles;
  }
  for (int i = rows + tid; i < A.cap; i += SCHED_THREADS) {
    A.tok[i] = P.pad;
    A.pos[i] = 0;
    A.row[i] = P.B;      // the spare cache row
    A.last_pos[i] = 0;
  }
  if (tid == 0) {
    P.ctl[CTL_HEAD] = head + nseq;
    P.ctl[CTL_PREFILL_ROWS] += rows;
    P.ctl[CTL_ADMIT_PASSES] += 1;
  }
}

// Deferred admission, second half: the slots a deferred pass filled go live (their prefill is complete: the caller
// orders this launch after the pass), the in-flight mark is cleared and the step kernel is told that it owes a
// compaction.
__global__ void __launch_bounds__(SCHED_THREADS) sched_commit_kernel(const __grid_constant__ SchedParams P) {
  for (int s = threadIdx.x; s < P.B; s += SCHED_THREADS) {
    const int r = P.pend_req[s];
    if (r < 0) continue;
    P.req[s] = r;
    P.fed[s] = P.pend_fed[s];
    P.gen[s] = 0;
    P.cur_tok[s] = P.pend_tok[s];
    P.pos[s] = P.pend_pos[s];
    P.starts[s] = 0;
    P.row_key[s] = P.pend_key[s];
    P.step_ctr[s] = 0;
    if (P.step_row) P.step_row[s] = P.row_map ? P.row_map[s] : (int64_t)s;
    P.pend_req[s] = -1;
  }
  if (threadIdx.x == 0) {
    P.ctl[CTL_INFLIGHT] = 0;
    P.ctl[CTL_DEFER] = 0;
    P.ctl[CTL_DIRTY] = 1;
  }
}

// Append n requests whose prompt_len / limit / key entries and prompt tokens the host has already copied into the
// rings at [tail, tail + n) and [tok_tail, tok_tail + sum(len)): computes their prompt and output offsets by prefix
// sum, clears out_len, then publishes the new tail.
__global__ void __launch_bounds__(SCHED_THREADS) sched_enqueue_kernel(const __grid_constant__ SchedParams P, int n) {
  __shared__ int warp_tot[SCHED_THREADS / 32];
  const int tid = threadIdx.x;
  const int64_t tail = P.ctl[CTL_TAIL];
  int64_t tok_base = P.ctl[CTL_TOK_TAIL], out_base = P.ctl[CTL_OUT_TAIL];
  for (int base = 0; base < n; base += SCHED_THREADS) {
    const int i = base + tid;
    const bool in = i < n;
    const int ri = in ? (int)((tail + i) % P.q_cap) : 0;
    const int len = in ? P.prompt_len[ri] : 0;
    const int lim = in ? P.limit[ri] : 0;
    int tot_len, tot_lim;
    const int off_len = block_excl_scan(len, warp_tot, tid, tot_len);
    const int off_lim = block_excl_scan(lim, warp_tot, tid, tot_lim);
    if (in) {
      P.prompt_off[ri] = tok_base + off_len;
      P.out_off[ri] = out_base + off_lim;
      P.out_len[ri] = -1;
    }
    tok_base += tot_len;
    out_base += tot_lim;
  }
  __syncthreads();
  if (tid == 0) {
    P.ctl[CTL_TOK_TAIL] = tok_base;
    P.ctl[CTL_OUT_TAIL] = out_base;
    __threadfence();
    P.ctl[CTL_TAIL] = tail + n;
  }
}

}  // namespace uv

extern "C" int uv_sched_step(const uv_sched_args* a, void* stream) {
  using namespace uv;
  if (!a) return UV_ERR_ARG;
  if (a->B < 1 || a->q_cap < 1 || a->tok_cap < 1 || a->out_cap < 1 || a->max_len < 1) return UV_ERR_ARG;
  if (!a->req || !a->fed || !a->gen || !a->cur_tok || !a->pos || !a->starts || !a->row_key || !a->step_ctr ||
      !a->samp_tok || !a->samp_lp || !a->prompt_off || !a->prompt_len || !a->limit || !a->key || !a->out_off ||
      !a->out_len || !a->start_version || !a->tokens || !a->out_tok || !a->out_lp || !a->fin_ring || !a->ctl)
    return UV_ERR_ARG;
  if (a->lanes < 0 || (a->lanes > 0 && (!a->row_map || a->lane_chunk < 2 || a->ring_len < 1))) return UV_ERR_ARG;
  if (a->compact && (!a->row_map || a->lanes > 0 || !a->no_admit || a->B > COMPACT_MAX_SLOTS)) return UV_ERR_ARG;
  SchedParams P;
  static_assert(sizeof(SchedParams) == sizeof(uv_sched_args), "uv_sched_args mirrors SchedParams");
  memcpy(&P, a, sizeof(P));
  launch_pdl(sched_step_kernel, dim3(1), dim3(SCHED_THREADS), 0, static_cast<cudaStream_t>(stream), P);
  return check_launch();
}

extern "C" int uv_sched_admit(const uv_sched_args* a, const uv_sched_admit_args* p, void* stream) {
  using namespace uv;
  if (!a || !p) return UV_ERR_ARG;
  if (a->B < 1 || a->q_cap < 1 || a->tok_cap < 1) return UV_ERR_ARG;
  if (!a->req || !a->fed || !a->gen || !a->cur_tok || !a->pos || !a->starts || !a->row_key || !a->step_ctr ||
      !a->prompt_off || !a->prompt_len || !a->key || !a->start_version || !a->tokens || !a->ctl)
    return UV_ERR_ARG;
  if (!p->tok || !p->pos || !p->row || !p->last_pos || !p->cu || !p->tile_cu || p->cap < 0) return UV_ERR_ARG;
  SchedParams P;
  AdmitParams A;
  static_assert(sizeof(AdmitParams) == sizeof(uv_sched_admit_args), "uv_sched_admit_args mirrors AdmitParams");
  memcpy(&P, a, sizeof(P));
  memcpy(&A, p, sizeof(A));
  launch_pdl(sched_admit_kernel, dim3(1), dim3(SCHED_THREADS), 0, static_cast<cudaStream_t>(stream), P, A);
  return check_launch();
}

extern "C" int uv_sched_enqueue(const uv_sched_args* a, int n, void* stream) {
  using namespace uv;
  if (!a || n < 0) return UV_ERR_ARG;
  if (n == 0) return UV_OK;
  if (n > a->q_cap) return UV_ERR_ARG;
  if (!a->prompt_off || !a->prompt_len || !a->limit || !a->out_off || !a->out_len || !a->ctl) return UV_ERR_ARG;
  SchedParams P;
  memcpy(&P, a, sizeof(P));
  sched_enqueue_kernel<<<1, SCHED_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(P, n);
  return check_launch();
}

extern "C" int uv_sched_commit(const uv_sched_args* a, void* stream) {
  using namespace uv;
  if (!a || a->B < 1) return UV_ERR_ARG;
  if (!a->pend_req || !a->pend_fed || !a->pend_tok || !a->pend_pos || !a->pend_key || !a->req || !a->ctl)
    return UV_ERR_ARG;
  SchedParams P;
  memcpy(&P, a, sizeof(P));
  sched_commit_kernel<<<1, SCHED_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(P);
  return check_launch();
}
