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
  // Fused Block-Union (optional, fuse != 0): every row CTA ORs its words into the KV-head row's word
  // array in global memory and takes a ticket; the CTA that takes the last ticket of a KV-head row
  // compacts that row into the block table and leaves the words and the ticket zeroed for the next call.
  int fuse;
  int G;                 // query heads per KV head (H = Hkv * G)
  uint32_t* union_words; // [B*Hkv, W], zero on entry
  uint32_t* tickets;     // [B*Hkv], zero on entry
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
__device__ void topk_mark(const Team& tm, const float* s, int n, int k, uint8_t* keep, TeamShared* ts) {
  int* hist = ts->hist;
  int* warp_sums = ts->warp_sums;
  if (k >= n) {
    for (int j = tm.tid; j < n; j += tm.nt) keep[j] = 1;
    team_sync(tm);
    return;
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
    for (int j = tm.tid; j < n; j += tm.nt) {
      const uint32_t key = order_key(s[j]);
      if ((key & mask_hi) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
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
  }
  const uint32_t kth = ts->prefix;
  const int want_equal = ts->remaining;
  if (want_equal == ts->last_bin_count) {
    // every key equal to the k-th is wanted: no tie to break
    for (int j = tm.tid; j < n; j += tm.nt) keep[j] = order_key(s[j]) >= kth;
    team_sync(tm);
    return;
  }
  // ordered pass: keys above kth are kept, keys equal to kth are kept in index order
  int taken = 0;
  for (int base = 0; base < n; base += tm.nt) {
    const int j = base + tm.tid;
    const uint32_t key = j < n ? order_key(s[j]) : 0u;
    const int eq = (j < n && key == kth) ? 1 : 0;
    const int pos = block_exclusive_scan(tm, eq, warp_sums, &ts->total);
    if (j < n) keep[j] = (key > kth) || (eq && (taken + pos) < want_equal);
    taken += ts->total;
    team_sync(tm);
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
  const bool voting = i < a.rows_voting;
  if (!voting) {
    if (a.bits) for (int w = tm.tid; w < a.W; w += tm.nt) bits_row[w] = 0u;
    return;
  }
  {
  const long long s_off = b * a.s_b + h * a.s_h + i * a.s_q;
  const long long v_off = a.valid ? (b * a.v_b + h * a.v_h + i * a.v_q) : 0;

  // ---- load the row; invalid entries become -inf ----
  for (int j = tm.tid; j < a.Kb; j += tm.nt) {
    const bool ok = a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
    float x;
    if (preloaded) {
      x = s[j];  // left there by the caller (only entries with j <= diag are meaningful)
    } else if (a.rule == CA_RULE_MASK) {
      x = reinterpret_cast<const uint8_t*>(a.score)[s_off + j * a.s_k] ? 1.f : 0.f;
    } else {
      x = load_score(a.score, s_off + j * a.s_k, a.score_dtype);
    }
    s[j] = ok ? x : -INFINITY;
    keep[j] = 0;
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
    // valid entries are a prefix for the block-causal case; in general count them
    int cnt = 0;
    for (int j = tm.tid; j < a.Kb; j += tm.nt) cnt += a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
    block_exclusive_scan(tm, cnt, ts->warp_sums, &ts->nvalid);
    const int n_valid = ts->nvalid;
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

  // ---- forced blocks, validity, bit packing ----
  for (int base = 0; base < a.W * 32; base += tm.nt) {
    const int j = base + tm.tid;
    bool k = false;
    if (j < a.Kb) {
      const bool ok = a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
      const int d = diag - j;
      const bool forced = d >= 0 && (j < a.sink || d < a.local);
      k = (keep[j] || forced) && ok;
    }
    const uint32_t word = __ballot_sync(0xffffffffu, k);
    if ((tm.tid & 31) == 0 && (j >> 5) < a.W) {
      if (bits_row) bits_row[j >> 5] = word;
      if (a.fuse && word) atomicOr(&a.union_words[static_cast<long long>(kv_row) * a.W + (j >> 5)], word);
    }
  }
  }
}

__global__ void __launch_bounds__(kRowThreads) select_rows_kernel(const RowArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ TeamShared ts;
  __shared__ int sh_last;
  const Team tm{static_cast<int>(threadIdx.x), kRowThreads, 0};
  const int i = blockIdx.x % a.Qb;
  const int h = (blockIdx.x / a.Qb) % a.H;
  const int b = blockIdx.x / (a.Qb * a.H);
  select_row(a, tm, &ts, dyn_smem, b, h, i, false);
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
  if (!sh_last) return;
  __threadfence();
  uint32_t* words = reinterpret_cast<uint32_t*>(dyn_smem);  // the row's score scratch is free now
  uint32_t* gw = a.union_words + static_cast<long long>(kv_row) * a.W;
  for (int w = threadIdx.x; w < a.W; w += kRowThreads) {
    words[w] = __ldcg(&gw[w]);
    gw[w] = 0u;  // left clean for the next call
  }
  if (threadIdx.x == 0) a.tickets[kv_row] = 0u;
  __syncthreads();
  compact_row(tm, words, a.W, a.Kb, a.Pb, a.Qb, a.keep_recent, a.block_size, a.page_size,
              a.block_idx + static_cast<long long>(kv_row) * a.idx_stride, a.idx_stride, kv_row, a.counts, a.cache_seqlens,
              a.pages_per_row, nullptr, ts.warp_sums, &ts.cut);
}

// ------------------------------------------------------------------------------------------
// Gate scores + row rule + Block-Union + table in ONE launch.
// One CTA per (batch, KV head, Q-block): G teams of 128 threads, one per query head of the KV head.  All
// threads first compute the G rows of gate logits against the KV head's key-block cache - a thread owns a key
// block, fetches its 128 channels with sixteen 128-bit loads issued back to back and accumulates the G dot
// products in the channel order of gate_scores3_kernel, so the logits equal the stand-alone kernel's bit for
// bit - straight into the rows' shared memory.  Then every team runs the rule on its row (select_row), ORs its
// bits into the KV-head row's words, and the CTA takes ONE ticket; the CTA with the last ticket of a KV-head
// row compacts it.  The 4 MB of logits (128K context) never travel to memory and back, three launches
// become one, and the key-block cache is read once per Q-block from L2.
struct GateSelArgs {
  RowArgs row;  // row.score is unused
  const void* q;  // [B,Qb,Hq,128] by strides
  long long q_b, q_blk, q_h;
  int q_dtype;
  const void* k;  // [B,Kb,Hkv,128] by strides, 16-bit
  long long k_b, k_blk, k_h;
  float scale, masked_value;
  float* score_out;  // optional [B,Hq,Qb,Kb] contiguous: the logits as gate_scores writes them
  int row_bytes;     // shared memory per row
};

constexpr int kFusedTeam = 128;

__device__ __forceinline__ void widen8_16(const uint4& raw, int dtype, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (dtype == CA_DTYPE_BF16) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      v[2 * i] = __low2float(h);
      v[2 * i + 1] = __high2float(h);
    }
  }
}

template <int KDT, int G>
__global__ void __launch_bounds__(G* kFusedTeam) gate_select_kernel(const GateSelArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ TeamShared ts[G];
  __shared__ int sh_last;
  constexpr int T = G * kFusedTeam;
  const RowArgs& r = a.row;
  const int tid = threadIdx.x;
  const int Hkv = r.H / G;
  const int i = blockIdx.x % r.Qb;
  const int hk = (blockIdx.x / r.Qb) % Hkv;
  const int b = blockIdx.x / (r.Qb * Hkv);
  float* qs = reinterpret_cast<float*>(dyn_smem);  // [G][128]
  unsigned char* rows = dyn_smem + G * 128 * sizeof(float);
  for (int e = tid; e < G * 128; e += T) {
    const int g = e >> 7, c = e & 127;
    qs[e] = load_score(a.q, b * a.q_b + i * a.q_blk + static_cast<long long>(hk * G + g) * a.q_h + c, a.q_dtype);
  }
  __syncthreads();
  const int diag = r.Pb + i;
  const int jmax = r.valid ? r.Kb - 1 : diag;  // with an explicit validity mask every column may count
  for (int j = tid; j <= jmax; j += T) {
    const uint16_t* kp = reinterpret_cast<const uint16_t*>(a.k) + b * a.k_b + static_cast<long long>(j) * a.k_blk + hk * a.k_h;
    uint4 raw[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) raw[u] = __ldg(reinterpret_cast<const uint4*>(kp + u * 8));
    float acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) acc[g] = 0.f;
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      float kv[8];
      widen8_16(raw[u], KDT, kv);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float4 q0 = *reinterpret_cast<const float4*>(&qs[g * 128 + u * 8]);
        const float4 q1 = *reinterpret_cast<const float4*>(&qs[g * 128 + u * 8 + 4]);
        acc[g] = fmaf(q0.x, kv[0], acc[g]);
        acc[g] = fmaf(q0.y, kv[1], acc[g]);
        acc[g] = fmaf(q0.z, kv[2], acc[g]);
        acc[g] = fmaf(q0.w, kv[3], acc[g]);
        acc[g] = fmaf(q1.x, kv[4], acc[g]);
        acc[g] = fmaf(q1.y, kv[5], acc[g]);
        acc[g] = fmaf(q1.z, kv[6], acc[g]);
        acc[g] = fmaf(q1.w, kv[7], acc[g]);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float v = j <= diag ? acc[g] * a.scale : a.masked_value;
      reinterpret_cast<float*>(rows + static_cast<size_t>(g) * a.row_bytes)[j] = v;
      if (a.score_out) a.score_out[((static_cast<long long>(b) * r.H + hk * G + g) * r.Qb + i) * r.Kb + j] = v;
    }
  }
  if (a.score_out) {
    for (int e = tid; e < G * (r.Kb - 1 - jmax); e += T) {
      const int g = e / (r.Kb - 1 - jmax), j = jmax + 1 + e % (r.Kb - 1 - jmax);
      a.score_out[((static_cast<long long>(b) * r.H + hk * G + g) * r.Qb + i) * r.Kb + j] = a.masked_value;
    }
  }
  __syncthreads();
  {
    const int g = tid / kFusedTeam;
    const Team tm{tid % kFusedTeam, kFusedTeam, 1 + g};
    select_row(r, tm, &ts[g], rows + static_cast<size_t>(g) * a.row_bytes, b, hk * G + g, i, true);
  }
  // ---- Block-Union: one ticket per CTA; the last CTA of the KV-head row builds its table ----
  const int kv_row = b * Hkv + hk;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int ticket = atomicAdd(&r.tickets[kv_row], 1u);
    sh_last = ticket == static_cast<unsigned int>(r.Qb - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!sh_last) return;
  __threadfence();
  constexpr int kTail = T < kRowThreads ? T : kRowThreads;
  if (tid >= kTail) return;
  const Team tm{tid, kTail, 1};
  uint32_t* words = reinterpret_cast<uint32_t*>(rows);  // the rows' scratch is free now
  uint32_t* gw = r.union_words + static_cast<long long>(kv_row) * r.W;
  for (int w = tid; w < r.W; w += kTail) {
    words[w] = __ldcg(&gw[w]);
    gw[w] = 0u;  // left clean for the next call
  }
  if (tid == 0) r.tickets[kv_row] = 0u;
  team_sync(tm);
  compact_row(tm, words, r.W, r.Kb, r.Pb, r.Qb, r.keep_recent, r.block_size, r.page_size,
              r.block_idx + static_cast<long long>(kv_row) * r.idx_stride, r.idx_stride, kv_row, r.counts, r.cache_seqlens,
              r.pages_per_row, nullptr, ts[0].warp_sums, &ts[0].cut);
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

namespace {
template <int KDT, int G>
int launch_gate_select(const ca::select::GateSelArgs& a, size_t smem, int ctas, int device, cudaStream_t stream) {
  using namespace ca;
  using namespace ca::select;
  static std::mutex mu;
  static bool done[64] = {};
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!done[device]) {
      CA_CUDA(cudaFuncSetAttribute(gate_select_kernel<KDT, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      done[device] = true;
    }
  }
  launch_kernel(gate_select_kernel<KDT, G>, dim3(ctas), dim3(G * kFusedTeam), smem, stream, a);
  CA_LAUNCH_CHECK("gate_select_kernel");
  return CA_OK;
}
}  // namespace

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
  RowArgs a;
  a.score = p->score;
  a.s_b = p->score_stride_b, a.s_h = p->score_stride_h, a.s_q = p->score_stride_q, a.s_k = p->score_stride_k;
  a.score_dtype = p->score_dtype;
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
  a.union_words = nullptr, a.tickets = nullptr;
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

int ca_select_union_scratch_bytes(int B, int Hkv, int Kb, size_t* bytes_out) {
  using namespace ca;
  CA_REQUIRE(bytes_out != nullptr, "bytes_out is null");
  CA_REQUIRE(B > 0 && Hkv > 0 && Kb > 0, "B, Hkv, Kb must be positive");
  const size_t rows = static_cast<size_t>(B) * Hkv;
  *bytes_out = (rows * ((Kb + 31) / 32) + rows) * sizeof(uint32_t);
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
  ca_select_union_scratch_bytes(u->B, u->Hkv, u->Kb, &need);
  CA_REQUIRE(scratch != nullptr && reinterpret_cast<uintptr_t>(scratch) % 4 == 0, "scratch must be a 4-byte aligned device pointer");
  if (scratch_bytes < need) return fail(CA_ERR_CAPACITY, "scratch holds %zu bytes, %zu are needed", scratch_bytes, need);
  a.fuse = 1, a.G = u->G;
  a.union_words = static_cast<uint32_t*>(scratch);
  a.tickets = a.union_words + static_cast<size_t>(u->B) * u->Hkv * a.W;
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
  launch_kernel(select_rows_kernel, dim3(p->B * p->H * p->Qb), dim3(kRowThreads), smem, static_cast<cudaStream_t>(stream_), a);
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
  const int G = u->G;
  const bool k16 = g->k_dtype == CA_DTYPE_BF16 || g->k_dtype == CA_DTYPE_F16;
  const size_t smem = static_cast<size_t>(G) * 128 * sizeof(float) + static_cast<size_t>(G) * row_smem;
  const bool fused = g->C == 128 && k16 && g->Hk == u->Hkv && (G == 1 || G == 2 || G == 4) && p->rule != CA_RULE_MASK &&
                     smem <= 200 * 1024 && g->k_stride_blk % 8 == 0 && g->k_stride_h % 8 == 0 && g->k_stride_b % 8 == 0 &&
                     reinterpret_cast<uintptr_t>(g->k) % 16 == 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!fused) {
    // shapes the one-launch form does not cover: the two kernels it stands for
    rc = ca_gate_scores(g, stream_);
    if (rc != CA_OK) return rc;
    launch_kernel(select_rows_kernel, dim3(p->B * p->H * p->Qb), dim3(kRowThreads), row_smem, stream, a);
    CA_LAUNCH_CHECK("select_rows_kernel");
    return CA_OK;
  }
  DeviceInfo dev;
  rc = get_device_info(&dev);
  if (rc != CA_OK) return rc;
  GateSelArgs ga;
  ga.row = a;
  ga.q = g->q, ga.q_b = g->q_stride_b, ga.q_blk = g->q_stride_blk, ga.q_h = g->q_stride_h, ga.q_dtype = g->q_dtype;
  ga.k = g->k, ga.k_b = g->k_stride_b, ga.k_blk = g->k_stride_blk, ga.k_h = g->k_stride_h;
  ga.scale = g->scale, ga.masked_value = g->masked_value;
  ga.score_out = write_scores ? g->out : nullptr;
  ga.row_bytes = static_cast<int>(row_smem);
  const int ctas = p->B * u->Hkv * p->Qb;
  const bool bf = g->k_dtype == CA_DTYPE_BF16;
  if (G == 1) return bf ? launch_gate_select<CA_DTYPE_BF16, 1>(ga, smem, ctas, dev.ordinal, stream) : launch_gate_select<CA_DTYPE_F16, 1>(ga, smem, ctas, dev.ordinal, stream);
  if (G == 2) return bf ? launch_gate_select<CA_DTYPE_BF16, 2>(ga, smem, ctas, dev.ordinal, stream) : launch_gate_select<CA_DTYPE_F16, 2>(ga, smem, ctas, dev.ordinal, stream);
  return bf ? launch_gate_select<CA_DTYPE_BF16, 4>(ga, smem, ctas, dev.ordinal, stream) : launch_gate_select<CA_DTYPE_F16, 4>(ga, smem, ctas, dev.ordinal, stream);
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
