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

// Exclusive block-wide prefix sum of one int per thread (kRowThreads threads).
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += n;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (kRowThreads / 32) ? warp_sums[lane] : 0;
    int winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, winc, d);
      if (lane >= d) winc += n;
    }
    if (lane < (kRowThreads / 32)) warp_sums[lane] = winc - w;
    if (lane == 31) *total = winc;
  }
  __syncthreads();
  int r = warp_sums[warp] + inc - v;
  __syncthreads();
  return r;
}

__device__ __forceinline__ float block_reduce_max(float v, float* scratch) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < kRowThreads / 32; ++w) r = fmaxf(r, scratch[w]);
  __syncthreads();
  return r;
}

// Deterministic block sum: fixed tree inside the warp, then warps added in order.
__device__ __forceinline__ float block_reduce_sum(float v, float* scratch) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int w = 0; w < kRowThreads / 32; ++w) r += scratch[w];
  __syncthreads();
  return r;
}

// Marks the k largest entries of s[0..n) (ties -> lower index) in keep[] (1 byte per entry).
// Radix select over the monotone keys, 8 bits per pass, then an ordered pass for the ties.
__device__ void topk_mark(const float* s, int n, int k, uint8_t* keep, int* hist, int* warp_sums) {
  __shared__ uint32_t sh_prefix;
  __shared__ int sh_remaining, sh_total, sh_last_bin_count;
  if (k >= n) {
    for (int j = threadIdx.x; j < n; j += kRowThreads) keep[j] = 1;
    __syncthreads();
    return;
  }
  if (threadIdx.x == 0) {
    sh_prefix = 0;
    sh_remaining = k;
  }
  __syncthreads();
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kRowThreads) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = sh_prefix;
    const uint32_t mask_hi = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int j = threadIdx.x; j < n; j += kRowThreads) {
      const uint32_t key = order_key(s[j]);
      if ((key & mask_hi) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // warp 0 finds the bin that holds the rem-th largest key: lane l owns bins 255-8l .. 248-8l
      const int lane = threadIdx.x;
      const int rem = sh_remaining;
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
        sh_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
        sh_remaining = left;  // entries still wanted among those equal to the chosen digit
        sh_last_bin_count = hist[bin];
      }
    }
    __syncthreads();
  }
  const uint32_t kth = sh_prefix;
  const int want_equal = sh_remaining;
  if (want_equal == sh_last_bin_count) {
    // every key equal to the k-th is wanted: no tie to break
    for (int j = threadIdx.x; j < n; j += kRowThreads) keep[j] = order_key(s[j]) >= kth;
    __syncthreads();
    return;
  }
  // ordered pass: keys above kth are kept, keys equal to kth are kept in index order
  int taken = 0;
  for (int base = 0; base < n; base += kRowThreads) {
    const int j = base + threadIdx.x;
    const uint32_t key = j < n ? order_key(s[j]) : 0u;
    const int eq = (j < n && key == kth) ? 1 : 0;
    const int pos = block_exclusive_scan(eq, warp_sums, &sh_total);
    if (j < n) keep[j] = (key > kth) || (eq && (taken + pos) < want_equal);
    taken += sh_total;
    __syncthreads();
  }
}

// Sorts comp[0..n2) ascending (n2 a power of two), bitonic network in shared memory.
__device__ void bitonic_sort(unsigned long long* comp, int n2) {
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (n2 >> 1); t += kRowThreads) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool asc = (lo & size) == 0;
        const unsigned long long x = comp[lo], y = comp[hi];
        if ((x > y) == asc) {
          comp[lo] = y;
          comp[hi] = x;
        }
      }
      __syncthreads();
    }
  }
}

// Compacts one KV-head row: `words` (shared memory, W words, bit j%32 of word j/32 = key block j kept by
// some query head / Q-block) -> ascending past block ids, -1 padded, count, seqlen, pages.  Columns
// j >= Kb - keep_recent are forced on first; only past columns (j < Pb) enter the table.  All threads of
// the CTA call it.
__device__ void compact_row(uint32_t* words, int W, int Kb, int Pb, int Qb, int keep_recent, int block_size, int page_size,
                            int32_t* idx_row, int idx_stride, int row, int32_t* counts, int32_t* cache_seqlens,
                            int32_t* pages_per_row, uint8_t* keep_kv_row, int* warp_sums, int* sh_total) {
  int running = 0;
  for (int wbase = 0; wbase < W; wbase += kRowThreads) {
    const int w = wbase + threadIdx.x;
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
    const int off = running + block_exclusive_scan(pc, warp_sums, sh_total);
    int o = off;
    while (word) {
      const int t = __ffs(word) - 1;
      word &= word - 1;
      if (o < idx_stride) idx_row[o] = w * 32 + t;
      ++o;
    }
    running += *sh_total;
    __syncthreads();
  }
  const int count = running < idx_stride ? running : idx_stride;
  for (int o = count + threadIdx.x; o < idx_stride; o += kRowThreads) idx_row[o] = -1;
  if (threadIdx.x == 0) {
    counts[row] = count;
    const int seqlen = (count + Qb) * block_size;
    if (cache_seqlens) cache_seqlens[row] = seqlen;
    if (pages_per_row) pages_per_row[row] = (seqlen + page_size - 1) / page_size;
  }
}

__global__ void __launch_bounds__(kRowThreads) select_rows_kernel(const RowArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ unsigned char dyn_smem[];
  float* s = reinterpret_cast<float*>(dyn_smem);                    // [Kb]
  uint8_t* keep = reinterpret_cast<uint8_t*>(s + a.Kb);              // [Kb]
  uint8_t* flag = keep + a.Kb;                                       // [Kb] scratch flags
  unsigned long long* comp =
      reinterpret_cast<unsigned long long*>(dyn_smem + ((a.Kb * 6 + 15) / 16) * 16);  // cummass only
  __shared__ float red[kRowThreads / 32];
  __shared__ int hist[256];
  __shared__ int warp_sums[kRowThreads / 32];
  __shared__ int sh_cut;

  const int i = blockIdx.x % a.Qb;
  const int h = (blockIdx.x / a.Qb) % a.H;
  const int b = blockIdx.x / (a.Qb * a.H);
  const int diag = a.Pb + i;  // last causally valid key block of this row
  uint32_t* bits_row = a.bits ? a.bits + ((static_cast<long long>(b) * a.H + h) * a.Qb + i) * a.W : nullptr;
  const int kv_row = a.fuse ? b * (a.H / a.G) + h / a.G : 0;

  const bool voting = i < a.rows_voting;
  if (!voting) {
    if (a.bits) for (int w = threadIdx.x; w < a.W; w += kRowThreads) bits_row[w] = 0u;
    if (!a.fuse) return;
  }
  if (voting) {
  const long long s_off = b * a.s_b + h * a.s_h + i * a.s_q;
  const long long v_off = a.valid ? (b * a.v_b + h * a.v_h + i * a.v_q) : 0;

  // ---- load the row; invalid entries become -inf ----
  for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) {
    const bool ok = a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
    float x;
    if (a.rule == CA_RULE_MASK) {
      x = reinterpret_cast<const uint8_t*>(a.score)[s_off + j * a.s_k] ? 1.f : 0.f;
    } else {
      x = load_score(a.score, s_off + j * a.s_k, a.score_dtype);
    }
    s[j] = ok ? x : -INFINITY;
    keep[j] = 0;
  }
  __syncthreads();

  if (a.softmax) {
    float m = -INFINITY;
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) m = fmaxf(m, s[j]);
    m = block_reduce_max(m, red);
    float sum = 0.f;
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) {
      const float e = s[j] == -INFINITY ? 0.f : expf(s[j] - m);
      s[j] = e;
      sum += e;
    }
    sum = block_reduce_sum(sum, red);
    const float inv = sum > 0.f ? 1.0f / sum : 0.f;
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) {
      const bool ok = a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
      s[j] = ok ? s[j] * inv : -INFINITY;
    }
    __syncthreads();
  }
  if (a.prob_out) {
    float* prow = a.prob_out + ((static_cast<long long>(b) * a.H + h) * a.Qb + i) * a.Kb;
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) prow[j] = s[j] == -INFINITY ? 0.f : s[j];
  }

  // ---- the rule ----
  const float thr = a.threshold_ptr ? __ldg(a.threshold_ptr + b * a.threshold_stride) : a.threshold;
  if (a.rule == CA_RULE_THRESHOLD) {
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) keep[j] = s[j] > thr;  // -inf never passes
  } else if (a.rule == CA_RULE_MASK) {
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) keep[j] = s[j] > 0.5f;
  } else if (a.rule == CA_RULE_ALPHA_ROWMAX) {
    // non-finite or acausal entries count as 0 for the maximum and are never selected by score
    // (the reference zero-fills them before taking the maximum and the top-k)
    float m = 0.f;
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) {
      const float x = s[j];
      const bool fin = (x == x) && fabsf(x) != INFINITY && j <= diag;
      flag[j] = fin;
      s[j] = fin ? x : 0.f;
      m = fmaxf(m, s[j]);
    }
    m = block_reduce_max(m, red);
    if (a.min_budget > 0) {
      topk_mark(s, a.Kb, a.min_budget < a.Kb ? a.min_budget : a.Kb, keep, hist, warp_sums);
      __syncthreads();
    }
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) keep[j] = keep[j] || (flag[j] && s[j] >= m * a.alpha);
  } else if (a.rule == CA_RULE_TOPK) {
    // valid entries are a prefix for the block-causal case; in general count them
    int cnt = 0;
    for (int j = threadIdx.x; j < a.Kb; j += kRowThreads) cnt += a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
    __shared__ int sh_nvalid;
    block_exclusive_scan(cnt, warp_sums, &sh_nvalid);
    const int n_valid = sh_nvalid;
    int k = a.topk_k > 0 ? a.topk_k
                         : static_cast<int>((static_cast<long long>(a.topk_num) * n_valid + a.topk_den / 2) / a.topk_den);
    if (k < 1) k = 1;
    if (k > n_valid) k = n_valid;
    // invalid entries are -inf and sort last, so taking k <= n_valid never reaches them
    if (k > 0) topk_mark(s, a.Kb, k, keep, hist, warp_sums);
  } else if (a.rule == CA_RULE_CUMMASS) {
    int n2 = 1;
    while (n2 < a.Kb) n2 <<= 1;
    for (int j = threadIdx.x; j < n2; j += kRowThreads) {
      // descending by value, ascending by index; invalid (-inf) and padding sort last
      const uint32_t key = j < a.Kb ? order_key(s[j] == -INFINITY ? -1.0f : s[j]) : 0u;
      comp[j] = (static_cast<unsigned long long>(~key) << 32) | static_cast<uint32_t>(j);
    }
    __syncthreads();
    bitonic_sort(comp, n2);
    if (threadIdx.x == 0) {
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
      sh_cut = cut;
    }
    __syncthreads();
    const int cut = sh_cut;
    for (int r = threadIdx.x; r < cut; r += kRowThreads) {
      const int j = static_cast<int>(comp[r] & 0xffffffffu);
      keep[j] = s[j] != -INFINITY;
    }
  }
  __syncthreads();

  // ---- forced blocks, validity, bit packing ----
  for (int base = 0; base < a.W * 32; base += kRowThreads) {
    const int j = base + threadIdx.x;
    bool k = false;
    if (j < a.Kb) {
      const bool ok = a.valid ? (a.valid[v_off + j * a.v_k] != 0) : (j <= diag);
      const int d = diag - j;
      const bool forced = d >= 0 && (j < a.sink || d < a.local);
      k = (keep[j] || forced) && ok;
    }
    const uint32_t word = __ballot_sync(0xffffffffu, k);
    if ((threadIdx.x & 31) == 0 && (j >> 5) < a.W) {
      if (bits_row) bits_row[j >> 5] = word;
      if (a.fuse && word) atomicOr(&a.union_words[static_cast<long long>(kv_row) * a.W + (j >> 5)], word);
    }
  }
  }  // voting
  if (!a.fuse) return;
  // ---- fused Block-Union: the last row CTA of this KV-head row builds the table.  Nobody waits: a CTA
  // publishes its words, takes a ticket and leaves unless the ticket is the last one. ----
  __shared__ int sh_last;
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
  compact_row(words, a.W, a.Kb, a.Pb, a.Qb, a.keep_recent, a.block_size, a.page_size,
              a.block_idx + static_cast<long long>(kv_row) * a.idx_stride, a.idx_stride, kv_row, a.counts, a.cache_seqlens,
              a.pages_per_row, nullptr, warp_sums, &sh_cut);
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
  compact_row(words, a.W, a.Kb, a.Pb, a.Qb, a.keep_recent, a.block_size, a.page_size, idx_row, a.idx_stride, row, a.counts,
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
  for (int base = 0; base < R; base += kRowThreads) {
    const int r = base + threadIdx.x;
    const int v = r < R ? pages_per_row[r] : 0;
    const int off = running + block_exclusive_scan(v, warp_sums, &sh_total);
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

int ca_select_union_table(const ca_select_params* p, const ca_union_params* u, void* scratch, size_t scratch_bytes,
                          ca_stream_t stream_) {
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
  launch_kernel(select_rows_kernel, dim3(p->B * p->H * p->Qb), dim3(kRowThreads), smem, static_cast<cudaStream_t>(stream_), a);
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
