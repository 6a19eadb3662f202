// Block selection: per-row rules on a score tensor -> packed keep bits, then Block-Union KV
// selection (OR over the chunk's Q-blocks, OR over the GQA group) and compaction into the
// per-KV-head block table.  Integer/byte work, HBM- and launch-bound: coalesced loads, warp
// ballots for bit packing, popcount prefix scans for compaction; no host synchronisation, every
// output is sized by capacity.
#include "ca_common.cuh"

#include <mutex>

namespace ca {
namespace select {

constexpr int kRowThreads = 256;

#ifdef CA_SELECT_PROFILE
// Development build: cycle stamps of one CTA's phases (thread 0 of team 0 of CTA 0).
__device__ long long g_sel_prof[32];
#define SEL_MARK(team_is_first, tid, k) \
  if (blockIdx.x == 0 && (team_is_first) && (tid) == 0) g_sel_prof[k] = clock64();
#define SEL_MARK_ANY0(k) \
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) g_sel_prof[k] = clock64();
#else
#define SEL_MARK(team_is_first, tid, k)
#define SEL_MARK_ANY0(k)
#endif
constexpr int kMaxKb = 8192;  // key blocks per row supported by the row kernels (512K tokens at bs 64)

__device__ __forceinline__ float load_score(const void* base, long long off, int dtype) {
  if (dtype == CA_DTYPE_F32) return reinterpret_cast<const float*>(base)[off];
  if (dtype == CA_DTYPE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off]);
  return __half2float(reinterpret_cast<const __half*>(base)[off]);
}

// Monotone map float -> uint32 (larger float -> larger key); -0 and +0 differ but compare adjacent.
__device__ __forceinline__ uint32_t order_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct RowArgs {
  const void* score;  // [B,H,Qb,Kb] by strides; dtype f32/bf16/f16, or uint8 when rule == MASK
  long long s_b, s_h, s_q, s_k;
  int score_dtype;
  const float* score_max;  // optional f32, score's strides: the rule sees score[j] * 2^(score_max[j] - row max of score_max)
  const uint8_t* valid;  // optional bool [B,1|H,Qb,Kb] by strides; NULL = block-causal j <= Pb + i
  long long v_b, v_h, v_q, v_k;
  uint32_t* bits;  // [B,H,Qb,W]
  float* prob_out; // optional fp32 [B,H,Qb,Kb] contiguous: the row after softmax / masking
  int B, H, Qb, Kb, Pb, W;
  int rule;
  int softmax;     // apply a masked softmax to the row before the rule
  float threshold; // THRESHOLD: keep s > threshold.  CUMMASS: tau
  const float* threshold_ptr;  // optional device value(s) replacing `threshold`: element b * threshold_stride
  long long threshold_stride;
  float alpha;     // ALPHA_ROWMAX: keep s >= alpha * rowmax
  int topk_k;      // TOPK: absolute k when > 0 ...
  int topk_num, topk_den;  // ... else k = max(1, (num * n_valid + den/2) / den)
  int min_budget;  // ALPHA_ROWMAX: also keep the top min_budget entries
  int sink, local; // forced blocks: j < sink, and 0 <= (Pb+i) - j < local
  int rows_voting; // rows i >= rows_voting produce no bits (FlashPrefill last_n_block)
  // Fused Block-Union (optional, fuse != 0): every row CTA stores its words (`bits`, the caller's or a scratch
  // area: plain stores - OR-ing them into one word array with atomics made 64 CTAs queue on every address)
  // and takes a ticket; the CTA that takes the last ticket of a KV-head row ORs that row's G * Qb word rows,
  // compacts them into the block table and leaves the ticket zeroed for the next call.
  int fuse;
  int G;                 // query heads per KV head (H = Hkv * G)
  uint32_t* tickets;     // [B*Hkv], zero on entry, left zero
  int keep_recent, block_size, page_size, idx_stride;
  int32_t* block_idx;
  int32_t* counts;
  int32_t* cache_seqlens;
  int32_t* pages_per_row;
};

// A team is a warp-aligned group of `nt` threads of a CTA that works on one row and synchronises on its own
// named barrier: the row kernels run one team per CTA (barrier 0 = the whole CTA), the fused score + rule
// kernel runs one team per query head of a KV head side by side.
struct Team {
  int tid;  // thread index inside the team
  int nt;   // threads in the team (a multiple of 32, <= kRowThreads)
  int bar;  // named barrier of the team
};
__device__ __forceinline__ void team_sync(const Team& t) { asm volatile("bar.sync %0, %1;" ::"r"(t.bar), "r"(t.nt) : "memory"); }

// Per-team scratch in shared memory.
struct TeamShared {
  float red[kRowThreads / 32];
  int hist[256];
  int warp_sums[kRowThreads / 32];
  int cut, total, nvalid;
  uint32_t prefix;
  int remaining, last_bin_count;
};

// Exclusive team-wide prefix sum of one int per thread.
__device__ __forceinline__ int block_exclusive_scan(const Team& tm, int v, int* warp_sums, int* total) {
  const int lane = tm.tid & 31, warp = tm.tid >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += n;
  }
  if (lane == 31) warp_sums[warp] = inc;
  team_sync(tm);
  if (warp == 0) {
    int w = lane < (tm.nt / 32) ? warp_sums[lane] : 0;
    int winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, winc, d);
      if (lane >= d) winc += n;
    }
    if (lane < (tm.nt / 32)) warp_sums[lane] = winc - w;
    if (lane == 31) *total = winc;
  }
  team_sync(tm);
  int r = warp_sums[warp] + inc - v;
  team_sync(tm);
  return r;
}

__device__ __forceinline__ float block_reduce_max(const Team& tm, float v, float* scratch) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  if ((tm.tid & 31) == 0) scratch[tm.tid >> 5] = v;
  team_sync(tm);
  float r = scratch[0];
  for (int w = 1; w < tm.nt / 32; ++w) r = fmaxf(r, scratch[w]);
  team_sync(tm);
  return r;
}

// Deterministic block sum: fixed tree inside the warp, then warps added in order.
__device__ __forceinline__ float block_reduce_sum(const Team& tm, float v, float* scratch) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  if ((tm.tid & 31) == 0) scratch[tm.tid >> 5] = v;
  team_sync(tm);
  float r = 0.f;
  for (int w = 0; w < tm.nt / 32; ++w) r += scratch[w];
  team_sync(tm);
  return r;
}

// Marks the k largest entries of s[0..n) (ties -> lower index) in keep[] (1 byte per entry).
// Radix select over the monotone keys, 8 bits per pass, then an ordered pass for the ties.
// EPT > 0: n <= EPT * tm.nt and every thread keeps its EPT keys in registers across the passes (the key is
// computed once and a pass costs a compare, a shift and one shared-memory atomic per entry - the rule is bound
// by instruction issue: 512 rows x 2048 entries x every instruction of the pass loops); EPT == 0: any n, keys
// re-read from shared memory in every pass.
template <int EPT>
__device__ void topk_mark_impl(const Team& tm, const float* s, int n, int k, uint8_t* keep, TeamShared* ts) {
  int* hist = ts->hist;
  int* warp_sums = ts->warp_sums;
  if (k >= n) {
    for (int j = tm.tid; j < n; j += tm.nt) keep[j] = 1;
    team_sync(tm);
    return;
  }
  uint32_t key[EPT > 0 ? EPT : 1];
  if (EPT > 0) {
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const int j = tm.tid + e * tm.nt;
      key[e] = j < n ? order_key(s[j]) : 0u;
    }
  }
  if (tm.tid == 0) {
    ts->prefix = 0;
    ts->remaining = k;
  }
  team_sync(tm);
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tm.tid; i < 256; i += tm.nt) hist[i] = 0;
    team_sync(tm);
    const uint32_t prefix = ts->prefix;
    const uint32_t mask_hi = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    if (EPT > 0) {
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        if (tm.tid + e * tm.nt < n && (key[e] & mask_hi) == prefix) atomicAdd(&hist[(key[e] >> shift) & 255u], 1);
      }
    } else {
      for (int j = tm.tid; j < n; j += tm.nt) {
        const uint32_t kj = order_key(s[j]);
        if ((kj & mask_hi) == prefix) atomicAdd(&hist[(kj >> shift) & 255u], 1);
      }
    }
    team_sync(tm);
    if (tm.tid < 32) {
      // warp 0 finds the bin that holds the rem-th largest key: lane l owns bins 255-8l .. 248-8l
      const int lane = tm.tid;
      const int rem = ts->remaining;
      int mine = 0;
#pragma unroll
      for (int u = 0; u < 8; ++u) mine += hist[255 - 8 * lane - u];
      int inc = mine;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int nb = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += nb;
      }
      const uint32_t hit = __ballot_sync(0xffffffffu, inc >= rem);
      const int owner = hit ? __ffs(hit) - 1 : 31;
      if (lane == owner) {
        int left = rem - (inc - mine);  // still wanted inside this lane's eight bins
        int bin = 255 - 8 * lane;
        for (int u = 0; u < 7; ++u) {
          if (hist[bin] >= left) break;
          left -= hist[bin];
          --bin;
        }
        ts->prefix = prefix | (static_cast<uint32_t>(bin) << shift);
        ts->remaining = left;  // entries still wanted among those equal to the chosen digit
        ts->last_bin_count = hist[bin];
      }
    }
    team_sync(tm);
    // every key that shares the prefix found so far is wanted: the lower digits cannot change the answer (with
    // 2048 distinct scores the chosen bin holds a single key after two or three of the four passes)
    if (ts->remaining == ts->last_bin_count) break;
  }
  const uint32_t kth = ts->prefix;
  const int want_equal = ts->remaining;
  if (want_equal == ts->last_bin_count) {
    // every key equal to the k-th is wanted: no tie to break
    if (EPT > 0) {
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        const int j = tm.tid + e * tm.nt;
        if (j < n) keep[j] = key[e] >= kth;
      }
    } else {
      for (int j = tm.tid; j < n; j += tm.nt) keep[j] = order_key(s[j]) >= kth;
    }
    team_sync(tm);
    return;
  }
  // ordered pass: keys above kth are kept, keys equal to kth are kept in index order
  int taken = 0;
  for (int base = 0; base < n; base += tm.nt) {
    const int j = base + tm.tid;
    const uint32_t kj = j < n ? order_key(s[j]) : 0u;
    const int eq = (j < n && kj == kth) ? 1 : 0;
    const int pos = block_exclusive_scan(tm, eq, warp_sums, &ts->total);
    if (j < n) keep[j] = (kj > kth) || (eq && (taken + pos) < want_equal);
    taken += ts->total;
    team_sync(tm);
  }
}

__device__ void topk_mark(const Team& tm, const float* s, int n, int k, uint8_t* keep, TeamShared* ts) {
  const int per_thread = (n + tm.nt - 1) / tm.nt;
  if (per_thread <= 8) {
    topk_mark_impl<8>(tm, s, n, k, keep, ts);
  } else if (per_thread <= 16) {
    topk_mark_impl<16>(tm, s, n, k, keep, ts);
  } else if (per_thread <= 32) {
    topk_mark_impl<32>(tm, s, n, k, keep, ts);
  } else {
    topk_mark_impl<0>(tm, s, n, k, keep, ts);
  }
}

// Sorts comp[0..n2) ascending (n2 a power of two), bitonic network in shared memory.
__device__ void bitonic_sort(const Team& tm, unsigned long long* comp, int n2) {
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tm.tid; t < (n2 >> 1); t += tm.nt) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool asc = (lo & size) == 0;
        const unsigned long long x = comp[lo], y = comp[hi];
        if ((x > y) == asc) {
          comp[lo] = y;
          comp[hi] = x;
        }
      }
      team_sync(tm);
    }
  }
}

// Compacts one KV-head row: `words` (shared memory, W words, bit j%32 of word j/32 = key block j kept by
// some query head / Q-block) -> ascending past block ids, -1 padded, count, seqlen, pages.  Columns
// j >= Kb - keep_recent are forced on first; only past columns (j < Pb) enter the table.  All threads of
// the CTA call it.
__device__ void compact_row(const Team& tm, uint32_t* words, int W, int Kb, int Pb, int Qb, int keep_recent, int block_size, int page_size,
                            int32_t* idx_row, int idx_stride, int row, int32_t* counts, int32_t* cache_seqlens,
                            int32_t* pages_per_row, uint8_t* keep_kv_row, int* warp_sums, int* sh_total) {
  int running = 0;
  for (int wbase = 0; wbase < W; wbase += tm.nt) {
    const int w = wbase + tm.tid;
    uint32_t word = 0;
    if (w < W) {
      word = words[w];
      const int j0 = w * 32;
      // forced recent columns; bits beyond Kb cleared
      const int first_recent = Kb - keep_recent;
      if (j0 + 32 > first_recent) word |= first_recent <= j0 ? 0xffffffffu : (0xffffffffu << (first_recent - j0));
      if (j0 + 32 > Kb) word &= Kb <= j0 ? 0u : (0xffffffffu >> (j0 + 32 - Kb));
      if (keep_kv_row) {
        for (int t = 0; t < 32 && j0 + t < Kb; ++t) keep_kv_row[j0 + t] = ((word >> t) & 1u) || (j0 + t >= Pb);
      }
      // keep past columns only
      if (j0 + 32 > Pb) word = j0 >= Pb ? 0u : (word & ((1u << (Pb - j0)) - 1u));
    }
    const int pc = __popc(word);
    const int off = running + block_exclusive_scan(tm, pc, warp_sums, sh_total);
    int o = off;
    while (word) {
      const int t = __ffs(word) - 1;
      word &= word - 1;
      if (o < idx_stride) idx_row[o] = w * 32 + t;
      ++o;
    }
    running += *sh_total;
    team_sync(tm);
  }
  const int count = running < idx_stride ? running : idx_stride;
  for (int o = count + tm.tid; o < idx_stride; o += tm.nt) idx_row[o] = -1;
  if (tm.tid == 0) {
    counts[row] = count;
    const int seqlen = (count + Qb) * block_size;
    if (cache_seqlens) cache_seqlens[row] = seqlen;
    if (pages_per_row) pages_per_row[row] = (seqlen + page_size - 1) / page_size;
  }
}

// One row (b, h, i) of the rule, by one team: scores -> (softmax) -> rule -> forced blocks -> packed bits, which
// go to a.bits (if given) and, with a.fuse, are ORed into the KV-head row's union words.  `row_smem` holds
// s[Kb] f32, keep[Kb], flag[Kb] and, for the cumulative-mass rule, the sort keys.  With `preloaded` the raw
// scores of the row are already in s[] (the fused score + rule kernel) instead of in a.score.
__device__ void select_row(const RowArgs& a, const Team& tm, TeamShared* ts, unsigned char* row_smem, int b, int h, int i,
                           bool preloaded) {
  float* s = reinterpret_cast<float*>(row_smem);                     // [Kb]
  uint8_t* keep = reinterpret_cast<uint8_t*>(s + a.Kb);               // [Kb]
  uint8_t* flag = keep + a.Kb;                                        // [Kb] scratch flags
  unsigned long long* comp =
      reinterpret_cast<unsigned long long*>(row_smem + ((a.Kb * 6 + 15) / 16) * 16);  // cummass only
  const int diag = a.Pb + i;  // last causally valid key block of this row
  uint32_t* bits_row = a.bits ? a.bits + ((static_cast<long long>(b) * a.H + h) * a.Qb + i) * a.W : nullptr;
  const int kv_row = a.fuse ? b * (a.H / a.G) + h / a.G : 0;
  SEL_MARK(tm.bar <= 1, tm.tid, 4);
  const bool voting = i < a.rows_voting;
  if (!voting) {
    if (a.bits) for (int w = tm.tid; w < a.W; w += tm.nt) bits_row[w] = 0u;
    return;
  }
  {
  const long long s_off = b * a.s_b + h * a.s_h + i * a.s_q;
  const long long v_off = a.valid ? (b * a.v_b + h * a.v_h + i * a.v_q) : 0;

  // ---- load the row; invalid entries become -inf.  Eight entries per thread and round, every load issued
  // before the first store (the loop used to pay one memory latency per entry) ----
  float exp_max = -INFINITY;  // with score_max: the row's largest exponent
  if (a.score_max) {
    float m = -INFINITY;
    for (int j = tm.tid; j < a.Kb; j += tm.nt) m = fmaxf(m, __ldg(a.score_max + s_off + j * a.s_k));
    exp_max = block_reduce_max(tm, m, ts->red);
  }
  for (int base = 0; base < a.Kb; base += tm.nt * 8) {
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = base + u * tm.nt + tm.tid;
      x[u] = 0.f;
      if (j < a.Kb) {
        if (preloaded) {
          x[u] = s[j];  // left there by the caller (only entries with j <= diag are meaningful)
        } else if (a.rule == CA_RULE_MASK) {
          x[u] = reinterpret_cast<const uint8_t*>(a.score)[s_off + j * a.s_k] ? 1.f : 0.f;
        } else {
          x[u] = load_score(a.score, s_off + j * a.s_k, a.score_dtype);
          if (a.score_max) {
            const float e = __ldg(a.score_max + s_off + j * a.s_k);
            x[u] = e == -INFINITY ? 0.f : x[u] * exp2f(e - exp_max);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = base + u * tm.nt + tm.tid;
      if (j < a.Kb) {
        const bool ok = a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
        s[j] = ok ? x[u] : -INFINITY;
        keep[j] = 0;
      }
    }
  }
  team_sync(tm);

  if (a.softmax) {
    float m = -INFINITY;
    for (int j = tm.tid; j < a.Kb; j += tm.nt) m = fmaxf(m, s[j]);
    m = block_reduce_max(tm, m, ts->red);
    float sum = 0.f;
    for (int j = tm.tid; j < a.Kb; j += tm.nt) {
      const float e = s[j] == -INFINITY ? 0.f : expf(s[j] - m);
      s[j] = e;
      sum += e;
    }
    sum = block_reduce_sum(tm, sum, ts->red);
    const float inv = sum > 0.f ? 1.0f / sum : 0.f;
    for (int j = tm.tid; j < a.Kb; j += tm.nt) {
      const bool ok = a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
      s[j] = ok ? s[j] * inv : -INFINITY;
    }
    team_sync(tm);
  }
  if (a.prob_out) {
    float* prow = a.prob_out + ((static_cast<long long>(b) * a.H + h) * a.Qb + i) * a.Kb;
    for (int j = tm.tid; j < a.Kb; j += tm.nt) prow[j] = s[j] == -INFINITY ? 0.f : s[j];
  }

  SEL_MARK(tm.bar <= 1, tm.tid, 5);
  // ---- the rule ----
  const float thr = a.threshold_ptr ? __ldg(a.threshold_ptr + b * a.threshold_stride) : a.threshold;
  if (a.rule == CA_RULE_THRESHOLD) {
    for (int j = tm.tid; j < a.Kb; j += tm.nt) keep[j] = s[j] > thr;  // -inf never passes
  } else if (a.rule == CA_RULE_MASK) {
    for (int j = tm.tid; j < a.Kb; j += tm.nt) keep[j] = s[j] > 0.5f;
  } else if (a.rule == CA_RULE_ALPHA_ROWMAX) {
    // non-finite or acausal entries count as 0 for the maximum and are never selected by score
    // (the reference zero-fills them before taking the maximum and the top-k)
    float m = 0.f;
    for (int j = tm.tid; j < a.Kb; j += tm.nt) {
      const float x = s[j];
      const bool fin = (x == x) && fabsf(x) != INFINITY && j <= diag;
      flag[j] = fin;
      s[j] = fin ? x : 0.f;
      m = fmaxf(m, s[j]);
    }
    m = block_reduce_max(tm, m, ts->red);
    if (a.min_budget > 0) {
      topk_mark(tm, s, a.Kb, a.min_budget < a.Kb ? a.min_budget : a.Kb, keep, ts);
      team_sync(tm);
    }
    for (int j = tm.tid; j < a.Kb; j += tm.nt) keep[j] = keep[j] || (flag[j] && s[j] >= m * a.alpha);
  } else if (a.rule == CA_RULE_TOPK) {
    // valid entries are a prefix for the block-causal case; with an explicit mask they are counted
    int n_valid = diag + 1 < a.Kb ? diag + 1 : a.Kb;
    if (a.valid) {
      int cnt = 0;
      for (int j = tm.tid; j < a.Kb; j += tm.nt) cnt += a.valid[v_off + j * a.v_k] != 0;
      block_exclusive_scan(tm, cnt, ts->warp_sums, &ts->nvalid);
      n_valid = ts->nvalid;
    }
    int k = a.topk_k > 0 ? a.topk_k
                         : static_cast<int>((static_cast<long long>(a.topk_num) * n_valid + a.topk_den / 2) / a.topk_den);
    if (k < 1) k = 1;
    if (k > n_valid) k = n_valid;
    // invalid entries are -inf and sort last, so taking k <= n_valid never reaches them
    if (k > 0) topk_mark(tm, s, a.Kb, k, keep, ts);
  } else if (a.rule == CA_RULE_CUMMASS) {
    int n2 = 1;
    while (n2 < a.Kb) n2 <<= 1;
    for (int j = tm.tid; j < n2; j += tm.nt) {
      // descending by value, ascending by index; invalid (-inf) and padding sort last
      const uint32_t key = j < a.Kb ? order_key(s[j] == -INFINITY ? -1.0f : s[j]) : 0u;
      comp[j] = (static_cast<unsigned long long>(~key) << 32) | static_cast<uint32_t>(j);
    }
    team_sync(tm);
    bitonic_sort(tm, comp, n2);
    if (tm.tid == 0) {
      // sequential fp32 prefix sum in sorted order; keep the shortest prefix with mass >= tau
      float acc = 0.f;
      int cut = a.Kb;
      for (int r = 0; r < a.Kb; ++r) {
        const int j = static_cast<int>(comp[r] & 0xffffffffu);
        const float p = s[j] == -INFINITY ? 0.f : s[j];
        acc = __fadd_rn(acc, p);
        if (acc >= thr) {
          cut = r + 1;
          break;
        }
      }
      ts->cut = cut;
    }
    team_sync(tm);
    const int cut = ts->cut;
    for (int r = tm.tid; r < cut; r += tm.nt) {
      const int j = static_cast<int>(comp[r] & 0xffffffffu);
      keep[j] = s[j] != -INFINITY;
    }
  }
  team_sync(tm);

  SEL_MARK(tm.bar <= 1, tm.tid, 6);
  // ---- forced blocks, validity, bit packing: a thread packs eight consecutive entries into a byte, four
  // neighbouring lanes put their bytes together into a word (one pass over the row instead of a ballot per
  // 32 entries and iteration: the iterations' shared-memory reads and ballots ran one after the other) ----
  for (int base = 0; base < a.W * 32; base += tm.nt * 8) {
    const int j0 = base + tm.tid * 8;
    uint32_t byte = 0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = j0 + u;
      if (j < a.Kb) {
        const bool ok = a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
        const int d = diag - j;
        const bool forced = d >= 0 && (j < a.sink || d < a.local);
        if ((keep[j] || forced) && ok) byte |= 1u << u;
      }
    }
    uint32_t word = byte << (8 * (tm.tid & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if ((tm.tid & 3) == 0 && (j0 >> 5) < a.W) {
      if (bits_row) bits_row[j0 >> 5] = word;
    }
  }
  }
}

__global__ void __launch_bounds__(kRowThreads, 4) select_rows_kernel(const RowArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ TeamShared ts;
  __shared__ int sh_last;
  const Team tm{static_cast<int>(threadIdx.x), kRowThreads, 0};
  const int i = blockIdx.x % a.Qb;
  const int h = (blockIdx.x / a.Qb) % a.H;
  const int b = blockIdx.x / (a.Qb * a.H);
  SEL_MARK(true, tm.tid, 0);
  select_row(a, tm, &ts, dyn_smem, b, h, i, false);
  SEL_MARK(true, tm.tid, 7);
  if (!a.fuse) return;
  const int kv_row = b * (a.H / a.G) + h / a.G;
  // ---- fused Block-Union: the last row CTA of this KV-head row builds the table.  Nobody waits: a CTA
  // publishes its words, takes a ticket and leaves unless the ticket is the last one. ----
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(&a.tickets[kv_row], 1u);
    sh_last = ticket == static_cast<unsigned int>(a.G * a.Qb - 1) ? 1 : 0;
  }
  __syncthreads();
  SEL_MARK(true, tm.tid, 9);
  if (!sh_last) return;
  __threadfence();
  uint32_t* words = reinterpret_cast<uint32_t*>(dyn_smem);  // the row's score scratch is free now
  for (int w = threadIdx.x; w < a.W; w += kRowThreads) words[w] = 0u;
  if (threadIdx.x == 0) a.tickets[kv_row] = 0u;  // left clean for the next call
  __syncthreads();
  {
    // OR of the KV head's G * Qb word rows (contiguous: heads h0..h0+G-1, every Q-block), read past L1
    const uint32_t* src = a.bits + ((static_cast<long long>(b) * a.H + (h / a.G) * a.G) * a.Qb) * a.W;
    const int n_words = a.G * a.Qb * a.W;
    if (a.W % 4 == 0) {
      for (int e = threadIdx.x * 4; e < n_words; e += kRowThreads * 4) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + e));
        const int w = e % a.W;
        if (v.x) atomicOr(&words[w], v.x);
        if (v.y) atomicOr(&words[w + 1], v.y);
        if (v.z) atomicOr(&words[w + 2], v.z);
        if (v.w) atomicOr(&words[w + 3], v.w);
      }
    } else {
      for (int e = threadIdx.x; e < n_words; e += kRowThreads) {
        const uint32_t v = __ldcg(src + e);
        if (v) atomicOr(&words[e % a.W], v);
      }
    }
  }
  __syncthreads();
  compact_row(tm, words, a.W, a.Kb, a.Pb, a.Qb, a.keep_recent, a.block_size, a.page_size,
              a.block_idx + static_cast<long long>(kv_row) * a.idx_stride, a.idx_stride, kv_row, a.counts, a.cache_seqlens,
              a.pages_per_row, nullptr, ts.warp_sums, &ts.cut);
}

constexpr int kGsTileKeys = 128;
constexpr int kGsHalfBytes = kGsTileKeys * 128;  // [128 key blocks][64 x 16-bit], 128-byte swizzle
constexpr int kGsTileBytes = 2 * kGsHalfBytes;

__device__ __forceinline__ uint16_t to16(float x, int dtype) {
  if (dtype == CA_DTYPE_BF16) {
    const __nv_bfloat16 h = __float2bfloat16_rn(x);
    return *reinterpret_cast<const uint16_t*>(&h);
  }
  const __half h = __float2half_rn(x);
  return *reinterpret_cast<const uint16_t*>(&h);
}
__device__ __forceinline__ float from16(uint16_t v, int dtype) {
  if (dtype == CA_DTYPE_BF16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
  return __half2float(*reinterpret_cast<const __half*>(&v));
}

// ------------------------------------------------------------------------------------------
// Gate logits of a whole chunk on the tensor core.
// One CTA per (key tile of 128 blocks, group of 16 query rows, cache head, batch), a query row being a
// (Q-block, query head) pair of the cache head: D[128 key blocks][32] = K_tile . Q^T, the 32 columns holding
// the 16 rows rounded to the cache's 16-bit type and then their rounding remainders (hi + lo restores the f32
// query to 2^-16).  Eight tcgen05.mma (M 128, N 32, K 16) per CTA; the key blocks are the TMEM lanes, a thread
// of the four collecting warps owns one and writes its 16 logits row by row, 32 lanes to 128 consecutive bytes.
// A key tile is fetched once per row group (4 times at 16 Q-blocks x 4 heads: 16 MB from L2 in all).
// Measured and dropped: (1) CUDA-core forms (a thread, or a half-warp with packed f32x2 FMAs and a halving
// shuffle reduction, per key block): 27 600 - 50 000 cycles per CTA of four rows, bound first by the L1 tag
// stage (128-bit loads 256 bytes apart across a warp), then by issue slots.  (2) One launch for scores + rule +
// table, a CTA per (KV head, Q-block) with N = 16 columns and the rule run by teams of the same CTA: correct
// and bit-identical, but every Q-block re-read the head's cache from L2 (TMA delivered a 32 KB tile per
// 1 100 - 1 400 cycles) and eight N = 16 MMAs took as long again: 41 us against 47 us for the two launches it
// replaced.  (3) All rows of a cache head as the columns of one CTA (N = 128, 128 CTAs of 5 warps): 18 000
// instructions per CTA for the query tile and the 64 stores per thread at 8 % occupancy, 15.6 us.
struct GateTcArgs {
  const void* q;  // [B,Qb,Hq,128] by strides
  long long q_b, q_blk, q_h;
  int q_dtype;
  float* out;     // [B,Hq,Qb,Kb] contiguous
  int B, Hq, Hk, G, Qb, Kb, Pb;
  int n_rows;     // Qb * G query rows per cache head
  int n_groups;   // ceil(n_rows / 16)
  float scale, masked_value;
  uint32_t idesc;
  unsigned long long wait_limit_ns;
};

struct GateTcShared {
  uint64_t k_full, t_full;
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kGtRows = 16;                 // query rows per CTA
constexpr int kGtCols = 2 * kGtRows;        // MMA N: hi and lo
constexpr int kGtQHalfBytes = kGtCols * 128;
constexpr int kGtThreads = 160;             // 4 collecting warps + the TMA / MMA warp

template <int KDT>
__device__ __forceinline__ uint32_t pack16x2(float x0, float x1) {
  if (KDT == CA_DTYPE_BF16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __half2 h = __floats2half2_rn(x0, x1);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <int KDT>
__device__ __forceinline__ float2 unpack16x2(uint32_t v) {
  if (KDT == CA_DTYPE_BF16) return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

template <int KDT>
__global__ void __launch_bounds__(kGtThreads) gate_scores_tc_kernel(const __grid_constant__ CUtensorMap k_map, const GateTcArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ uint8_t gt_smem_raw[];
  __shared__ GateTcShared sh;
  const uint32_t smem_base = (ptx::smem_u32(gt_smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = gt_smem_raw + (smem_base - ptx::smem_u32(gt_smem_raw));
  // layout: K tile (two swizzled halves) | Q tile (two swizzled halves of 32 rows)
  const uint32_t k_smem = smem_base;
  uint8_t* q_tile = smem_aligned + kGsTileBytes;
  const uint32_t q_smem = smem_base + kGsTileBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x / a.n_groups, group = blockIdx.x % a.n_groups;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int row0 = group * kGtRows;  // first query row (i * G + g) of this CTA
  volatile int* abort_flag = &sh.abort_flag;

  if (tid == 0) {
    ptx::mbar_init(ptx::smem_u32(&sh.k_full), 1);
    ptx::mbar_init(ptx::smem_u32(&sh.t_full), 1);
    sh.abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 4) {
    ptx::tmem_alloc(ptx::smem_u32(&sh.tmem_base), kGtCols);
    ptx::tmem_relinquish();
  }
  __syncthreads();
  SEL_MARK_ANY0(16);
  if (warp == 4 && lane == 0) {
    // the key tile is on its way while the other warps build the Q tile
    ptx::mbar_expect_tx(ptx::smem_u32(&sh.k_full), kGsTileBytes);
    for (int h = 0; h < 2; ++h)
      ptx::tma_load_4d(k_smem + h * kGsHalfBytes, &k_map, ptx::smem_u32(&sh.k_full), h * 64, hk, tile * kGsTileKeys, b);
  }
  // Q tile: column n < 16 = query row row0 + n rounded to 16 bits, column 16 + n = what the rounding dropped.
  // An item is 8 channels of one query row: 256 items, at most two per thread, loads first.
  {
    float v[2][8];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int e = tid + u * kGtThreads;
      const int rr = row0 + (e >> 4), piece = e & 15;
#pragma unroll
      for (int c = 0; c < 8; ++c) v[u][c] = 0.f;
      if (e < kGtRows * 16 && rr < a.n_rows) {
        const int i = rr / a.G, g = rr - i * a.G;
        const long long off = b * a.q_b + i * a.q_blk + static_cast<long long>(hk * a.G + g) * a.q_h + piece * 8;
        if (a.q_dtype == CA_DTYPE_F32) {
          const float4 x0 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.q) + off));
          const float4 x1 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.q) + off + 4));
          v[u][0] = x0.x, v[u][1] = x0.y, v[u][2] = x0.z, v[u][3] = x0.w, v[u][4] = x1.x, v[u][5] = x1.y, v[u][6] = x1.z, v[u][7] = x1.w;
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) v[u][c] = load_score(a.q, off + c, a.q_dtype);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int e = tid + u * kGtThreads;
      if (e < kGtRows * 16) {
        const int n = e >> 4, piece = e & 15;
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          hi[c] = pack16x2<KDT>(v[u][2 * c], v[u][2 * c + 1]);
          const float2 back = unpack16x2<KDT>(hi[c]);
          lo[c] = pack16x2<KDT>(v[u][2 * c] - back.x, v[u][2 * c + 1] - back.y);
        }
        const int half = piece >> 3, chunk = piece & 7;
        const int nl = kGtRows + n;
        *reinterpret_cast<uint4*>(q_tile + half * kGtQHalfBytes + (n >> 3) * 1024 + (n & 7) * 128 + ((chunk ^ (n & 7)) << 4)) =
            make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(q_tile + half * kGtQHalfBytes + (nl >> 3) * 1024 + (nl & 7) * 128 + ((chunk ^ (nl & 7)) << 4)) =
            make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
    }
  }
  SEL_MARK_ANY0(17);
  ptx::fence_proxy_async_smem();  // the tensor core reads the tile through the async proxy
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sh.tmem_base;
  bool ok = true;
  if (warp == 4) {
    if (lane == 0) {
      ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh.k_full), 0, abort_flag, a.wait_limit_ns);
      if (ok) {
        ptx::tc_fence_after();
        const uint64_t k_desc0 = ptx::make_smem_desc_sw128(k_smem, 0, 1024);
        const uint64_t q_desc0 = ptx::make_smem_desc_sw128(q_smem, 0, 1024);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // A: key blocks (K-major), B: query rows (K-major); channel half k>>2, 32-byte step inside the swizzled row
          const uint64_t ko = static_cast<uint64_t>(((k >> 2) * kGsHalfBytes + (k & 3) * 32) >> 4);
          const uint64_t qo = static_cast<uint64_t>(((k >> 2) * kGtQHalfBytes + (k & 3) * 32) >> 4);
          ptx::mma_ss(tmem, k_desc0 + ko, q_desc0 + qo, a.idesc, k > 0 ? 1u : 0u);
        }
        ptx::tc_commit(ptx::smem_u32(&sh.t_full));
      }
    }
  } else {
    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh.t_full), 0, abort_flag, a.wait_limit_ns);
    ok = __all_sync(0xffffffffu, ok);
    SEL_MARK_ANY0(18);
    if (ok) {
      ptx::tc_fence_after();
      const int j = tile * kGsTileKeys + tid;  // this thread's key block
      uint32_t acc[32];
      ptx::tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16), acc);
      ptx::tc_wait_ld();
      if (j < a.Kb) {
        const long long head_stride = static_cast<long long>(a.Qb) * a.Kb;
        int i = row0 / a.G, g = row0 - i * a.G;
        float* dst = a.out + (static_cast<long long>(b) * a.Hq + hk * a.G + g) * head_stride + static_cast<long long>(i) * a.Kb + j;
#pragma unroll
        for (int u = 0; u < kGtRows; ++u) {
          if (row0 + u < a.n_rows) {
            const float dot = __uint_as_float(acc[u]) + __uint_as_float(acc[kGtRows + u]);
            *dst = j <= a.Pb + i ? dot * a.scale : a.masked_value;
            // next row: next head of the same Q-block, or head 0 of the next Q-block
            if (++g == a.G) {
              g = 0, ++i;
              dst += a.Kb - static_cast<long long>(a.G - 1) * head_stride;
            } else {
              dst += head_stride;
            }
          }
        }
      }
    }
  }
  SEL_MARK_ANY0(19);
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    if (lane == 0 && sh.abort_flag) {
      // after an expired wait: give the copy and the MMAs that may still be in flight 200 us to land
      const uint64_t t0 = ptx::globaltimer_ns();
      while (ptx::globaltimer_ns() - t0 < 200000ull) {
      }
    }
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kGtCols);
  }
}

struct UnionArgs {
  const uint32_t* bits;   // [B,Hin,Qin,W] packed keep bits, or NULL
  const uint8_t* mask;    // [B,Hin,Qin,Kb] bool by strides, used when bits == NULL
  long long m_b, m_h, m_q, m_k;
  int B, Hin, Qin, Hkv, G;  // Hin = Hkv*G (G = 1 when the input is already per KV head)
  int Kb, Pb, Qb, W;
  int keep_recent;          // past columns j >= Kb - keep_recent are forced on (Seer keep_recent_blocks)
  int block_size, page_size;
  int32_t* block_idx;       // [R, idx_stride] ascending past ids, -1 padded
  int idx_stride;
  int32_t* counts;          // [R]
  int32_t* cache_seqlens;   // optional [R] = (count + Qb) * bs
  int32_t* pages_per_row;   // optional [R] = ceil(cache_seqlens / page_size)
  uint8_t* keep_kv;         // optional bool [B,Hkv,Kb]: union with every chunk column on
};

__global__ void __launch_bounds__(kRowThreads) union_table_kernel(const UnionArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  __shared__ int warp_sums[kRowThreads / 32];
  __shared__ int sh_total;
  const int row = blockIdx.x;
  const int b = row / a.Hkv, hkv = row % a.Hkv;
  int32_t* idx_row = a.block_idx + static_cast<long long>(row) * a.idx_stride;
  // phase 1: OR over the group's heads and the Q rows, all threads sharing the (head, row, word) items
  __shared__ uint32_t words[kMaxKb / 32];
  for (int w = threadIdx.x; w < a.W; w += kRowThreads) words[w] = 0u;
  __syncthreads();
  const int items = a.G * a.Qin * a.W;
#pragma unroll 4
  for (int e = threadIdx.x; e < items; e += kRowThreads) {
    const int w = e % a.W, gi = e / a.W;
    const int h = hkv * a.G + gi / a.Qin, i = gi % a.Qin;
    uint32_t word = 0;
    if (a.bits) {
      word = a.bits[((static_cast<long long>(b) * a.Hin + h) * a.Qin + i) * a.W + w];
    } else {
      const uint8_t* m = a.mask + b * a.m_b + h * a.m_h + i * a.m_q;
      const int j0 = w * 32;
      const int n = a.Kb - j0 < 32 ? a.Kb - j0 : 32;
      for (int t = 0; t < n; ++t) word |= (m[(j0 + t) * a.m_k] ? 1u : 0u) << t;
    }
    if (word) atomicOr(&words[w], word);
  }
  __syncthreads();
  const Team tm{static_cast<int>(threadIdx.x), kRowThreads, 0};
  compact_row(tm, words, a.W, a.Kb, a.Pb, a.Qb, a.keep_recent, a.block_size, a.page_size, idx_row, a.idx_stride, row, a.counts,
              a.cache_seqlens, a.pages_per_row, a.keep_kv ? a.keep_kv + static_cast<long long>(row) * a.Kb : nullptr, warp_sums,
              &sh_total);
}

// Exclusive prefix over rows of pages_per_row -> page_offsets[R+1]; block_table[row,slot] =
// page_offsets[row] + slot for slot < pages_per_row[row] (else 0).  One CTA; R is small.
__global__ void __launch_bounds__(kRowThreads) paged_metadata_kernel(const int32_t* pages_per_row, int R,
                                                                     int32_t* page_offsets, int32_t* block_table,
                                                                     int max_pages) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  __shared__ int warp_sums[kRowThreads / 32];
  __shared__ int sh_total;
  int running = 0;
  const Team tm{static_cast<int>(threadIdx.x), kRowThreads, 0};
  for (int base = 0; base < R; base += kRowThreads) {
    const int r = base + threadIdx.x;
    const int v = r < R ? pages_per_row[r] : 0;
    const int off = running + block_exclusive_scan(tm, v, warp_sums, &sh_total);
    if (r < R) page_offsets[r] = off;
    running += sh_total;
    __syncthreads();
  }
  if (threadIdx.x == 0) page_offsets[R] = running;
  __syncthreads();
  if (block_table) {
    for (long long e = threadIdx.x; e < static_cast<long long>(R) * max_pages; e += kRowThreads) {
      const int r = static_cast<int>(e / max_pages), slot = static_cast<int>(e % max_pages);
      block_table[e] = slot < pages_per_row[r] ? page_offsets[r] + slot : 0;
    }
  }
}

}  // namespace select
}  // namespace ca

namespace ca {

// ca_gate_scores on the tensor core (declared in ca_score.cu): 128 gate channels, a 16-bit key-block cache and at
// most 128 query rows (Q-blocks x heads) per cache head.  CA_ERR_UNSUPPORTED for other shapes (the caller then
// takes the CUDA-core kernels).
int launch_gate_scores_tc(const ca_gate_score_params* g, cudaStream_t stream) {
  using namespace select;
  const bool k16 = g->k_dtype == CA_DTYPE_BF16 || g->k_dtype == CA_DTYPE_F16;
  if (g->C != 128 || !k16 || g->Hk <= 0 || g->Hq % g->Hk != 0) return CA_ERR_UNSUPPORTED;
  const int G = g->Hq / g->Hk;
  const int n_rows = g->Qb * G;
  if (g->k_stride_b % 8 != 0 || g->k_stride_blk % 8 != 0 || g->k_stride_h % 8 != 0 || reinterpret_cast<uintptr_t>(g->k) % 16 != 0)
    return CA_ERR_UNSUPPORTED;
  DeviceInfo dev;
  int rc = get_device_info(&dev);
  if (rc != CA_OK) return rc;
  if (dev.cc_major != 10) return CA_ERR_UNSUPPORTED;
  tensor_map_encode_fn enc = get_tensor_map_encoder();
  if (!enc) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const CUtensorMapDataType dt = g->k_dtype == CA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap k_map;
  {
    // (channel, cache head, key block, batch); the box is 128 key blocks x 64 channels of one head
    const cuuint32_t ones[4] = {1, 1, 1, 1};
    const cuuint64_t dims[4] = {128, (cuuint64_t)g->Hk, (cuuint64_t)g->Kb, (cuuint64_t)g->B};
    const cuuint64_t strides[3] = {(cuuint64_t)g->k_stride_h * 2, (cuuint64_t)g->k_stride_blk * 2, (cuuint64_t)g->k_stride_b * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)kGsTileKeys, 1};
    CUresult res = enc(&k_map, dt, 4, const_cast<void*>(g->k), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled(key-block cache) failed with CUresult %d", (int)res);
  }
  GateTcArgs a;
  a.q = g->q, a.q_b = g->q_stride_b, a.q_blk = g->q_stride_blk, a.q_h = g->q_stride_h;
  a.q_dtype = g->q_dtype;
  a.out = g->out;
  a.B = g->B, a.Hq = g->Hq, a.Hk = g->Hk, a.G = G, a.Qb = g->Qb, a.Kb = g->Kb, a.Pb = g->Pb;
  a.n_rows = n_rows;
  a.n_groups = ceil_div(n_rows, kGtRows);
  a.scale = g->scale, a.masked_value = g->masked_value;
  a.idesc = ptx::make_idesc_f16(g->k_dtype == CA_DTYPE_BF16 ? 1u : 0u, kGsTileKeys, kGtCols, 0, 0);
  a.wait_limit_ns = 2000000000ull;
  const size_t smem = 1024 + kGsTileBytes + 2 * kGtQHalfBytes;
  const long long ctas_x = static_cast<long long>(ceil_div(g->Kb, kGsTileKeys)) * a.n_groups;
  if (ctas_x > 0x7fffffffLL) return CA_ERR_UNSUPPORTED;
  const dim3 grid(static_cast<unsigned>(ctas_x), g->Hk, g->B);
  if (g->k_dtype == CA_DTYPE_BF16) {
    launch_kernel_as(true, gate_scores_tc_kernel<CA_DTYPE_BF16>, grid, dim3(kGtThreads), smem, stream, k_map, a);
  } else {
    launch_kernel_as(true, gate_scores_tc_kernel<CA_DTYPE_F16>, grid, dim3(kGtThreads), smem, stream, k_map, a);
  }
  CA_LAUNCH_CHECK("gate_scores_tc_kernel");
  return CA_OK;
}

}  // namespace ca

extern "C" {

// Validates a row-selection request, fills the kernel arguments and returns the dynamic shared memory it
// needs (the opt-in attribute is raised once per device when a row is longer than 8K blocks' worth).
static int fill_row_args(const ca_select_params* p, ca::select::RowArgs* out, size_t* smem_out, bool bits_required) {
  using namespace ca;
  using namespace ca::select;
  CA_REQUIRE(p != nullptr, "params is null");
  CA_REQUIRE(p->score && (p->bits || !bits_required), "score and bits must be non-null");
  CA_REQUIRE(p->B > 0 && p->H > 0 && p->Qb > 0 && p->Kb > 0, "B, H, Qb, Kb must be positive");
  CA_REQUIRE(p->Kb <= kMaxKb, "Kb %d exceeds the supported maximum %d", p->Kb, kMaxKb);
  CA_REQUIRE(p->Pb >= 0 && p->Pb + p->Qb <= p->Kb + p->Qb, "Pb out of range");
  CA_REQUIRE(p->rule >= CA_RULE_THRESHOLD && p->rule <= CA_RULE_MASK, "unknown rule %d", p->rule);
  CA_REQUIRE(p->rule == CA_RULE_MASK || p->score_dtype == CA_DTYPE_F32 || p->score_dtype == CA_DTYPE_BF16 ||
                 p->score_dtype == CA_DTYPE_F16,
             "score dtype must be f32, bf16 or f16");
  if (p->rule == CA_RULE_TOPK) CA_REQUIRE(p->topk_k > 0 || (p->topk_num >= 0 && p->topk_den > 0), "top-k needs k or num/den");
  CA_REQUIRE(p->score_max == nullptr || (p->score_dtype == CA_DTYPE_F32 && p->softmax == 0 && p->rule != CA_RULE_MASK),
             "score_max needs f32 scores, no softmax and a rule on scores");
  RowArgs a;
  a.score = p->score;
  a.s_b = p->score_stride_b, a.s_h = p->score_stride_h, a.s_q = p->score_stride_q, a.s_k = p->score_stride_k;
  a.score_dtype = p->score_dtype;
  a.score_max = p->score_max;
  a.valid = static_cast<const uint8_t*>(p->valid);
  a.v_b = p->valid_stride_b, a.v_h = p->valid_stride_h, a.v_q = p->valid_stride_q, a.v_k = p->valid_stride_k;
  a.bits = static_cast<uint32_t*>(p->bits);
  a.prob_out = p->prob_out;
  a.B = p->B, a.H = p->H, a.Qb = p->Qb, a.Kb = p->Kb, a.Pb = p->Pb;
  a.W = (p->Kb + 31) / 32;
  a.rule = p->rule;
  a.softmax = p->softmax;
  a.threshold = p->threshold;
  a.threshold_ptr = p->threshold_ptr;
  a.threshold_stride = p->threshold_stride_b;
  a.alpha = p->alpha;
  a.topk_k = p->topk_k, a.topk_num = p->topk_num, a.topk_den = p->topk_den;
  a.min_budget = p->min_budget;
  a.sink = p->sink, a.local = p->local;
  a.rows_voting = p->rows_voting > 0 ? p->rows_voting : p->Qb;
  a.fuse = 0, a.G = 1;
  a.tickets = nullptr;
  a.keep_recent = 0, a.block_size = 0, a.page_size = 0, a.idx_stride = 0;
  a.block_idx = nullptr, a.counts = nullptr, a.cache_seqlens = nullptr, a.pages_per_row = nullptr;
  size_t smem = ((static_cast<size_t>(p->Kb) * 6 + 15) / 16) * 16;
  if (p->rule == CA_RULE_CUMMASS) {
    size_t n2 = 1;
    while (n2 < static_cast<size_t>(p->Kb)) n2 <<= 1;
    smem += n2 * 8;
  }
  if (smem > 48 * 1024) {
    // a per-device function attribute: raised once per device to the largest size the kernel can be asked for
    static std::mutex mu;
    static bool done[64] = {};
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != CA_OK) return rc;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[dev.ordinal]) {
      const int max_smem = ((kMaxKb * 6 + 15) / 16) * 16 + kMaxKb * 8;
      CA_CUDA(cudaFuncSetAttribute(select_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      done[dev.ordinal] = true;
    }
  }
  *out = a;
  *smem_out = smem;
  return CA_OK;
}

int ca_select_rows(const ca_select_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::select;
  RowArgs a;
  size_t smem = 0;
  int rc = fill_row_args(p, &a, &smem, true);
  if (rc != CA_OK) return rc;
  launch_kernel(select_rows_kernel, dim3(p->B * p->H * p->Qb), dim3(kRowThreads), smem, static_cast<cudaStream_t>(stream_), a);
  CA_LAUNCH_CHECK("select_rows_kernel");
  return CA_OK;
}

#ifdef CA_SELECT_PROFILE
int ca_debug_select_profile(long long* out32) {
  return cudaMemcpyFromSymbol(out32, ca::select::g_sel_prof, 32 * sizeof(long long)) == cudaSuccess ? 0 : -3;
}
#endif

int ca_select_union_scratch_bytes(int B, int H, int Hkv, int Qb, int Kb, size_t* bytes_out) {
  using namespace ca;
  CA_REQUIRE(bytes_out != nullptr, "bytes_out is null");
  CA_REQUIRE(B > 0 && H > 0 && Hkv > 0 && Qb > 0 && Kb > 0, "B, H, Hkv, Qb, Kb must be positive");
  // tickets (one word per KV-head row, rounded to 16 bytes), then the rows' packed bits for callers that do not keep them
  const size_t tickets = ((static_cast<size_t>(B) * Hkv + 3) / 4) * 4;
  *bytes_out = (tickets + static_cast<size_t>(B) * H * Qb * ((Kb + 31) / 32)) * sizeof(uint32_t);
  return CA_OK;
}

// The fused rule + union + table request: validates both halves and fills the row kernel's arguments.
static int fill_fused_args(const ca_select_params* p, const ca_union_params* u, void* scratch, size_t scratch_bytes,
                           ca::select::RowArgs* out, size_t* smem_out) {
  using namespace ca;
  using namespace ca::select;
  RowArgs a;
  size_t smem = 0;
  int rc = fill_row_args(p, &a, &smem, false);
  if (rc != CA_OK) return rc;
  CA_REQUIRE(u != nullptr, "union params is null");
  CA_REQUIRE(u->block_idx && u->counts, "block_idx and counts must be non-null");
  CA_REQUIRE(u->B == p->B && u->Kb == p->Kb && u->Pb == p->Pb, "selection and union must agree on B, Kb and Pb");
  CA_REQUIRE(u->Hkv > 0 && u->G > 0 && u->Hkv * u->G == p->H, "Hkv * G (%d * %d) must equal the selection's head count %d", u->Hkv,
             u->G, p->H);
  CA_REQUIRE(u->Qin == p->Qb, "the union takes every Q-block row of the selection (Qin %d, Qb %d)", u->Qin, p->Qb);
  CA_REQUIRE(u->Pb <= u->Kb && u->Kb - u->Pb == p->Qb, "Kb - Pb must equal the chunk's Q-block count");
  CA_REQUIRE(u->idx_stride >= (u->Pb > 0 ? u->Pb : 1), "block_idx capacity %d is smaller than the past block count %d",
             u->idx_stride, u->Pb);
  CA_REQUIRE(u->block_size > 0 && u->page_size > 0, "block_size and page_size must be positive");
  CA_REQUIRE(u->keep_kv == nullptr && u->bits == nullptr && u->mask == nullptr,
             "the fused form takes its input from the selection; keep_kv is not produced");
  size_t need = 0;
  ca_select_union_scratch_bytes(u->B, p->H, u->Hkv, p->Qb, u->Kb, &need);
  const size_t ticket_words = ((static_cast<size_t>(u->B) * u->Hkv + 3) / 4) * 4;
  if (p->bits != nullptr) need = ticket_words * sizeof(uint32_t);  // the caller's bits serve as the rows' word store
  CA_REQUIRE(scratch != nullptr && reinterpret_cast<uintptr_t>(scratch) % 16 == 0, "scratch must be a 16-byte aligned device pointer");
  if (scratch_bytes < need) return fail(CA_ERR_CAPACITY, "scratch holds %zu bytes, %zu are needed", scratch_bytes, need);
  a.fuse = 1, a.G = u->G;
  a.tickets = static_cast<uint32_t*>(scratch);
  if (a.bits == nullptr) a.bits = a.tickets + ticket_words;
  a.keep_recent = u->keep_recent, a.block_size = u->block_size, a.page_size = u->page_size, a.idx_stride = u->idx_stride;
  a.block_idx = u->block_idx, a.counts = u->counts, a.cache_seqlens = u->cache_seqlens, a.pages_per_row = u->pages_per_row;
  *out = a;
  *smem_out = smem;
  return CA_OK;
}

int ca_select_union_table(const ca_select_params* p, const ca_union_params* u, void* scratch, size_t scratch_bytes,
                          ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::select;
  RowArgs a;
  size_t smem = 0;
  int rc = fill_fused_args(p, u, scratch, scratch_bytes, &a, &smem);
  if (rc != CA_OK) return rc;
  launch_kernel_as(true, select_rows_kernel, dim3(p->B * p->H * p->Qb), dim3(kRowThreads), smem, static_cast<cudaStream_t>(stream_), a);
  CA_LAUNCH_CHECK("select_rows_kernel");
  return CA_OK;
}


int ca_gate_score_select(const ca_gate_score_params* g, const ca_select_params* p, const ca_union_params* u, void* scratch,
                         size_t scratch_bytes, int write_scores, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::select;
  CA_REQUIRE(g != nullptr && p != nullptr && u != nullptr, "params are null");
  CA_REQUIRE(g->q && g->k && g->out, "q, k and the score buffer must be non-null");
  CA_REQUIRE(p->score == g->out && p->score_dtype == CA_DTYPE_F32 && p->score_stride_k == 1 && p->score_stride_q == g->Kb &&
                 p->score_stride_h == static_cast<int64_t>(g->Qb) * g->Kb && p->score_stride_b == p->score_stride_h * g->Hq,
             "the selection must read the gate's contiguous fp32 score buffer");
  CA_REQUIRE(p->B == g->B && p->H == g->Hq && p->Qb == g->Qb && p->Kb == g->Kb && p->Pb == g->Pb, "scores and selection disagree on sizes");
  RowArgs a;
  size_t row_smem = 0;
  int rc = fill_fused_args(p, u, scratch, scratch_bytes, &a, &row_smem);
  if (rc != CA_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  (void)write_scores;  // the logits always pass through score->out
  rc = ca_gate_scores(g, stream_);
  if (rc != CA_OK) return rc;
  launch_kernel_as(true, select_rows_kernel, dim3(p->B * p->H * p->Qb), dim3(kRowThreads), row_smem, stream, a);
  CA_LAUNCH_CHECK("select_rows_kernel");
  return CA_OK;
}

int ca_union_table(const ca_union_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::select;
  CA_REQUIRE(p != nullptr, "params is null");
  CA_REQUIRE((p->bits != nullptr) != (p->mask != nullptr), "exactly one of bits and mask must be given");
  CA_REQUIRE(p->block_idx && p->counts, "block_idx and counts must be non-null");
  CA_REQUIRE(p->B > 0 && p->Hkv > 0 && p->G > 0 && p->Qin > 0 && p->Kb > 0, "B, Hkv, G, Qin, Kb must be positive");
  CA_REQUIRE(p->Pb >= 0 && p->Pb <= p->Kb, "Pb (%d) must lie in [0, Kb=%d]", p->Pb, p->Kb);
  CA_REQUIRE(p->idx_stride >= (p->Pb > 0 ? p->Pb : 1), "block_idx capacity %d is smaller than the past block count %d",
             p->idx_stride, p->Pb);
  CA_REQUIRE(p->block_size > 0 && p->page_size > 0, "block_size and page_size must be positive");
  UnionArgs a;
  a.bits = static_cast<const uint32_t*>(p->bits);
  a.mask = static_cast<const uint8_t*>(p->mask);
  a.m_b = p->mask_stride_b, a.m_h = p->mask_stride_h, a.m_q = p->mask_stride_q, a.m_k = p->mask_stride_k;
  a.B = p->B, a.Hkv = p->Hkv, a.G = p->G, a.Hin = p->Hkv * p->G, a.Qin = p->Qin;
  a.Kb = p->Kb, a.Pb = p->Pb, a.Qb = p->Kb - p->Pb;
  a.W = (p->Kb + 31) / 32;
  a.keep_recent = p->keep_recent;
  a.block_size = p->block_size, a.page_size = p->page_size;
  a.block_idx = p->block_idx, a.idx_stride = p->idx_stride, a.counts = p->counts;
  a.cache_seqlens = p->cache_seqlens, a.pages_per_row = p->pages_per_row;
  a.keep_kv = static_cast<uint8_t*>(p->keep_kv);
  launch_kernel(union_table_kernel, dim3(p->B * p->Hkv), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream_), a);
  CA_LAUNCH_CHECK("union_table_kernel");
  return CA_OK;
}

int ca_paged_metadata(const int32_t* pages_per_row, int rows, int32_t* page_offsets, int32_t* block_table,
                      int max_pages, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::select;
  CA_REQUIRE(pages_per_row && page_offsets, "pages_per_row and page_offsets must be non-null");
  CA_REQUIRE(rows > 0, "rows must be positive");
  CA_REQUIRE(block_table == nullptr || max_pages > 0, "max_pages must be positive with a block_table");
  launch_kernel(paged_metadata_kernel, dim3(1), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream_), pages_per_row, rows, page_offsets,
                                                                                    block_table, max_pages);
  CA_LAUNCH_CHECK("paged_metadata_kernel");
  return CA_OK;
}

}  // extern "C"
