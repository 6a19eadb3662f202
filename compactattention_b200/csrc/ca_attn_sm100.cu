// Block-table-indexed dense causal attention for sm_100a: tcgen05 MMA with TMEM accumulators,
// TMA loads whose page coordinate comes from the per-KV-head block table.
//
// Work unit = one KV-head row (b, hkv) and a pair of 128-row query tiles ("A" and "B").  A query
// tile stacks the G query heads of the KV head along M: tile row i is (token i / G, head i % G),
// so one K/V stage feeds G heads.  K/V are consumed in 128-token steps = two 64-token sub-blocks,
// each fetched by its own TMA box at (page, token offset) resolved from the block table and the
// optional page table.  Selected past blocks are fully visible; the chunk's own blocks follow in
// order and are causally masked (bottom-right aligned), which is what
// compact_attn/kernels/varlen/indexed_dense_prefill_direct_triton.py:155-241 computes.
//
// Scheduling: a persistent grid of one CTA per SM.  The KV steps of all units are laid end to end
// and cut into equal spans, one per CTA ("stream-K"), so the SMs stay balanced whatever the
// per-row block counts are and however few rows a tensor-parallel rank owns.  A unit that falls
// entirely inside one span is written straight to the output; a unit cut by a span boundary
// leaves per-segment partials (unnormalised O, running max, running sum) in the workspace and a
// small combine kernel merges them.  Without a workspace the spans snap to unit boundaries.
//
// Warp roles (384 threads): warps 0-3 softmax of tile A, warps 4-7 softmax of tile B (thread =
// TMEM lane = tile row), warp 8 lane 0 issues every tcgen05.mma, warp 9 issues every TMA, warps
// 10-11 idle.  The third warpgroup gives its registers to the softmax warpgroups (setmaxnreg),
// which hold a whole 128-column S row per thread.
// TMEM (512 columns): S_A | S_B | O_A | O_B, 128 fp32 columns each; P (16-bit) overwrites the
// first 64 columns of its S and feeds the P.V MMA straight from TMEM.
// MMA order S_A0 S_B0 { PV_A(j) S_A(j+1) PV_B(j) S_B(j+1) } so one tile's softmax overlaps the
// other tile's MMAs.  Every wait is bounded; on expiry the CTA raises CA_STATUS_TIMEOUT, drains
// what it issued, frees TMEM and returns.
#include "ca_common.cuh"

#include <mutex>

namespace ca {
namespace attn {

constexpr int kThreads = 384;  // three warpgroups: softmax A, softmax B, {MMA, TMA, 2 idle warps}
constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kHeadDim = 128;
constexpr int kSub = 64;               // tokens per TMA box / sub-block
constexpr int kHalfBytes = 128 * 128;  // one [128 rows][64 x 16-bit] swizzled half tile
constexpr int kTileBytes = 2 * kHalfBytes;
constexpr int kBoxBytes = kSub * 128;  // one [64 tokens][64 x 16-bit] box
constexpr int kStages = 4;
constexpr int kTmemCols = 512;
constexpr int kMaxRows = 1024;  // (batch x kv heads) rows per launch
constexpr int kMaxSegs = 64;    // segments planned per batch
constexpr float kRescaleThreshold = 8.0f;  // log2 units; lazy accumulator rescale
constexpr int kMinSpanSteps = 8;           // shortest span worth a CTA of its own when units are cut
#ifndef CA_ATTN_MIN_UNIT_STEPS
#define CA_ATTN_MIN_UNIT_STEPS 24
#endif
// (units of 27-30 KV steps: 44 us cut against 66 us whole, so the threshold must stay below that;
// units of ~6 steps: 22 us whole against 45 us cut)
constexpr int kMinUnitStepsToCut = CA_ATTN_MIN_UNIT_STEPS;  // average KV steps per unit below which units stay whole
// Measured on B200 (sustained 300-launch loop, 128K context, 20 % density): handing P to the MMA warp
// in two halves 434 us, in one piece 450 us; packed fp32 pairs for the scale and the row sum 421 us.
// A polynomial exp2 on the FMA pipe for part of the exponentials (2 / 4 / 6 of every 16 pairs) took
// 486 / 499 / 518 us against 485 us without: with the softmax warps of both tiles on every scheduler
// the added instructions cost more than the MUFU operations they replace, so there is none.
#ifndef CA_ATTN_P_PARTS
#define CA_ATTN_P_PARTS 2
#endif
#ifndef CA_ATTN_PROFILE
#define CA_ATTN_PROFILE 0
#endif
#ifndef CA_ATTN_MERGE_DEPENDENT
// The merge kernel is enqueued as a programmatic dependent of the attention kernel (it waits with
// griddepcontrol.wait before reading anything): its CTAs are resident when the last attention CTA
// leaves.  Measured: 90.8 -> 88.2 us (one KV head), 134.4 -> 131.1 us (two), 32.9 -> 30.8 us (a small
// shape whose units stay whole); 0 restores a plain launch.
#define CA_ATTN_MERGE_DEPENDENT 1
#endif
static_assert(CA_ATTN_P_PARTS == 1 || CA_ATTN_P_PARTS == 2, "P is handed over in one or two pieces");
constexpr int kPParts = CA_ATTN_P_PARTS;  // P is handed to the MMA warp in this many pieces so P.V overlaps the softmax

// Optional cycle accounting (development builds only, -DCA_ATTN_PROFILE=1): one thread of each role
// adds the clock cycles between consecutive marks to per-CTA counters.
#if CA_ATTN_PROFILE
__device__ long long g_prof[160][32];
#define CA_PROF_DECL long long prof_t = clock64(); long long prof_acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
#define CA_PROF(i) { const long long prof_n = clock64(); prof_acc[i] += prof_n - prof_t; prof_t = prof_n; }
#define CA_PROF_FLUSH(base) { for (int prof_i = 0; prof_i < 10; ++prof_i) g_prof[blockIdx.x][(base) + prof_i] = prof_acc[prof_i]; }
#else
#define CA_PROF_DECL
#define CA_PROF(i) {}
#define CA_PROF_FLUSH(base) {}
#endif

// Partial results of one segment of a split unit.
constexpr int kPartialOFloats = 2 * kTileM * kHeadDim;  // [tile][col/4][row][4]
constexpr int kPartialMLFloats = 2 * kTileM * 2;        // [tile][row][m, l]

struct SegDesc {  // one per workspace slot
  int unit;       // row * n_pairs + pair, or -1 when the slot is unused
  int j0, j1;     // KV-step range of the segment inside the unit
  int n_iter;     // KV steps of the whole unit
};

struct Segment {
  int row, pair;
  int j0, j1;
  int n_sub, n_past_sub;
  int slot;  // workspace slot of a partial segment, -1: whole unit, written to the output
  int pad;
};

struct KernelArgs {
  int Q, G, Hkv, B;
  int tpt;          // query tokens per 128-row tile = 128 / G
  int n_pairs;      // tile pairs per row
  int past_blocks;  // Pb
  int spb;          // 64-token sub-blocks per block
  int block_size;
  int past_tokens;  // tokens before the chunk region (a multiple of block_size)
  int q_off;        // tokens of the chunk region that precede the first query (0 unless a dense launch has an unaligned past)
  int page_size, pages_per_seq, num_pages;
  const int32_t* block_idx;
  int block_idx_stride;
  const int32_t* counts;
  const int32_t* page_table;
  void* out;
  long long o_stride_b, o_stride_t, o_stride_h;
  float* lse;
  float scale_log2;
  int32_t* status;
  uint32_t idesc_qk, idesc_pv;
  unsigned long long wait_limit_ns;
  // K/V tensor-map dimensions 1..3 are ordered by ascending stride at encode time; these give the
  // coordinate slot (0..2) of the token, page and head coordinates.
  int slot_tok, slot_page, slot_head;
  int kv_head_div;     // block-table rows per KV head (1 unless per-query-head / sub-group tables)
  int split;           // 1: spans may cut units (needs the workspace)
  int max_cut_steps;   // > 0: units longer than this many KV steps on average stay whole
  SegDesc* descs;      // [2 * gridDim.x]
  float* part_ml;      // [2 * gridDim.x][kPartialMLFloats]
  float* part_o;       // [2 * gridDim.x][kPartialOFloats]
};

struct Shared {
  uint64_t q_full[2];
  uint64_t ring_full[kStages];
  uint64_t ring_empty[kStages];
  uint64_t s_full[2];
  uint64_t p_part[2][4];  // [tile][piece]; the last piece in use completes P
  uint64_t o_done;
  uint64_t o_free[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  int n_segs;
  int more;            // another batch of segments follows
  long long next_x;    // linear KV-step index where the next batch starts
  int row_count[kMaxRows];
  long long row_prefix[kMaxRows + 1];
  Segment segs[kMaxSegs];
};

constexpr int kSmemBytes = 2 * kTileBytes + kStages * kTileBytes + 1024 /*align*/ + static_cast<int>(sizeof(Shared));

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Number of visible columns (0..64) of 64-token sub-block u for chunk token t.
__device__ __forceinline__ int visible_cols(int u, int n_sub, int n_past_sub, int t) {
  // t counts from the start of the chunk region (query token index + q_off)
  if (u >= n_sub) return 0;
  if (u < n_past_sub) return kSub;
  int lim = t - (u - n_past_sub) * kSub + 1;
  return lim < 0 ? 0 : (lim > kSub ? kSub : lim);
}

// 64-token sub-blocks of the chunk that tile pair `pair` can see.
__device__ __forceinline__ int chunk_subs(const KernelArgs& a, int pair) {
  int t_last = (2 * pair + 2) * a.tpt - 1;
  if (t_last > a.Q - 1) t_last = a.Q - 1;
  return (t_last + a.q_off) / kSub + 1;
}
__device__ __forceinline__ int unit_iters(const KernelArgs& a, int count, int pair) {
  return (count * a.spb + chunk_subs(a, pair) + 1) >> 1;
}

// Plans up to kMaxSegs segments of this CTA's span starting at linear step x (thread 0 only).
__device__ void plan_segments(const KernelArgs& a, Shared* sh, long long x, long long span_begin, long long span_end,
                              int R) {
  int n = 0;
  // row containing x: largest r with row_prefix[r] <= x
  int lo = 0, hi = R;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sh->row_prefix[mid] <= x) lo = mid; else hi = mid;
  }
  int row = lo;
  long long acc = sh->row_prefix[row];
  int pair = 0;
  while (x < span_end && n < kMaxSegs && row < R) {
    const int count = sh->row_count[row];
    const int ni = unit_iters(a, count, pair);
    if (x >= acc + ni) {  // unit lies before x: walk on
      acc += ni;
      if (++pair == a.n_pairs) pair = 0, ++row;
      continue;
    }
    Segment s;
    s.row = row, s.pair = pair;
    s.j0 = static_cast<int>(x - acc);
    const long long rem = span_end - acc;
    s.j1 = rem < ni ? static_cast<int>(rem) : ni;
    s.n_past_sub = count * a.spb;
    s.n_sub = s.n_past_sub + chunk_subs(a, pair);
    const bool partial = !(s.j0 == 0 && s.j1 == ni);
    s.slot = partial ? static_cast<int>(2 * blockIdx.x + (x == span_begin ? 0 : 1)) : -1;
    s.pad = 0;
    if (partial) {
      SegDesc d;
      d.unit = row * a.n_pairs + pair, d.j0 = s.j0, d.j1 = s.j1, d.n_iter = ni;
      a.descs[s.slot] = d;
    }
    sh->segs[n++] = s;
    x = acc + s.j1;
  }
  sh->n_segs = n;
  sh->next_x = x;
  sh->more = (x < span_end && row < R) ? 1 : 0;
}

// P = exp2(S*sc + neg_m) for one 128-column row held in registers: packs to 16 bit, stores the four
// 32-column chunks over S in TMEM, signals the MMA warp after each of the kPParts pieces.  The scale
// and the row sum use packed fp32 pairs.  Returns the row sum of P.
template <typename T>
__device__ __forceinline__ float exp_pack_store(const uint32_t (&sv)[128], float sc, float neg_m, uint32_t tS,
                                                uint32_t p_part_bar) {
  float2 l2 = make_float2(0.f, 0.f);
  const float2 sc2 = make_float2(sc, sc);
  const float2 nm2 = make_float2(neg_m, neg_m);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[c * 32 + i]), __uint_as_float(sv[c * 32 + i + 1])), sc2, nm2);
      float2 pr;
      pr.x = ptx::ex2(x.x);
      pr.y = ptx::ex2(x.y);
      l2 = __fadd2_rn(l2, pr);
      pk[i >> 1] = pack2<T>(pr.x, pr.y);
    }
    ptx::tmem_st16(tS + c * 16, pk);
    if ((c + 1) % (4 / kPParts) == 0) {
      // a piece of P is in TMEM: let the MMA warp run P.V on it (the last piece completes P)
      ptx::tc_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(p_part_bar + static_cast<uint32_t>(((c + 1) / (4 / kPParts) - 1) * sizeof(uint64_t)));
    }
  }
  return l2.x + l2.y;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    attn_compact_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map, const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;                      // Q_A, Q_B
  const uint32_t ring_smem = smem_base + 2 * kTileBytes;  // kStages slots
  Shared* sh = reinterpret_cast<Shared*>(smem_aligned + 2 * kTileBytes + kStages * kTileBytes);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int R = a.B * a.Hkv;
  volatile int* abort_flag = &sh->abort_flag;
  const uint64_t limit = a.wait_limit_ns;
  bool bad_index = false;

#if CA_ATTN_PROFILE
  const long long prof_kernel_t0 = clock64();
#endif
  // ---- on-chip set-up first: it needs nothing from global memory, so under a programmatic
  // dependent launch it overlaps the tail of the previous kernel (the table builder) ----
  ptx::grid_launch_dependents();
  if (tid == 0) {
    sh->row_prefix[0] = 0;
    sh->abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&sh->q_full[0]), 1);
    ptx::mbar_init(ptx::smem_u32(&sh->q_full[1]), 1);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&sh->ring_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sh->ring_empty[s]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(&sh->s_full[0]), 1);
    ptx::mbar_init(ptx::smem_u32(&sh->s_full[1]), 1);
    for (int q = 0; q < 4; ++q) {
      ptx::mbar_init(ptx::smem_u32(&sh->p_part[0][q]), 128);
      ptx::mbar_init(ptx::smem_u32(&sh->p_part[1][q]), 128);
    }
    ptx::mbar_init(ptx::smem_u32(&sh->o_done), 1);
    ptx::mbar_init(ptx::smem_u32(&sh->o_free[0]), 128);
    ptx::mbar_init(ptx::smem_u32(&sh->o_free[1]), 128);
    ptx::mbar_init(ptx::smem_u32(&sh->drain), 1);
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 8) {
    ptx::tmem_alloc(ptx::smem_u32(&sh->tmem_base), kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == 9 && lane == 0) {
    ptx::tma_prefetch_desc(&q_map);
    ptx::tma_prefetch_desc(&k_map);
    ptx::tma_prefetch_desc(&v_map);
  }
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this

  // ---- per-row KV-step totals and their prefix (every CTA; a few thousand integer operations) ----
  for (int r = tid; r < R; r += kThreads) {
    int count = a.past_blocks;
    if (a.block_idx != nullptr) {
      count = a.counts[r];
      const int cap = a.block_idx_stride < a.past_blocks ? a.block_idx_stride : a.past_blocks;
      if (count < 0 || count > cap) {
        bad_index = true;
        count = count < 0 ? 0 : cap;
      }
    }
    sh->row_count[r] = count;
    long long tot = 0;
    for (int p = 0; p < a.n_pairs; ++p) tot += unit_iters(a, count, p);
    sh->row_prefix[r + 1] = tot;  // turned into a prefix below
  }
  if (tid == 0 && a.descs) {
    SegDesc none;
    none.unit = -1, none.j0 = 0, none.j1 = 0, none.n_iter = 0;
    a.descs[2 * blockIdx.x] = none;
    a.descs[2 * blockIdx.x + 1] = none;
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  long long span_begin = 0, span_end = 0;
  if (tid == 0) {
    for (int r = 0; r < R; ++r) sh->row_prefix[r + 1] += sh->row_prefix[r];
    const long long total = sh->row_prefix[R];
    long long nc = gridDim.x;
    const long long c = blockIdx.x;
    const long long n_units_all = static_cast<long long>(R) * a.n_pairs;
    // Cutting units pays only when a unit is long: measured on B200, units of ~6 KV steps ran 2x
    // slower cut (partials + the merge) than whole (45 vs 22 us), units of ~50 steps 20 % faster.
    const bool cut = a.split && total >= n_units_all * kMinUnitStepsToCut &&
                     (a.max_cut_steps <= 0 || total <= n_units_all * a.max_cut_steps);
    if (cut) {
      // A span costs a prologue, an epilogue and (when it cuts a unit) 128 KB of partials, about
      // as much as kMinSpanSteps KV steps: with little work, fewer CTAs take longer spans and the
      // others leave at once.
      const long long by_work = total / kMinSpanSteps;
      const long long cap = by_work > n_units_all ? by_work : n_units_all;
      if (cap < nc) nc = cap;
      if (c < nc) {
        span_begin = total * c / nc;
        span_end = total * (c + 1) / nc;
      }
    } else {
      // whole units only: equal unit counts per CTA
      const long long nu = static_cast<long long>(R) * a.n_pairs;
      auto unit_start = [&](long long u) -> long long {
        if (u >= nu) return total;
        const int r = static_cast<int>(u / a.n_pairs), p = static_cast<int>(u % a.n_pairs);
        long long s = sh->row_prefix[r];
        for (int q = 0; q < p; ++q) s += unit_iters(a, sh->row_count[r], q);
        return s;
      };
      span_begin = unit_start(nu * c / nc);
      span_end = unit_start(nu * (c + 1) / nc);
    }
    sh->next_x = span_begin;
    sh->more = span_end > span_begin ? 1 : 0;
    sh->n_segs = 0;
  }
  __syncthreads();

#if CA_ATTN_PROFILE
  if (tid == 0) g_prof[blockIdx.x][30] = clock64() - prof_kernel_t0;  // prologue
#endif
  // role state that lives across segments
  int ring_n = 0;        // ring entries issued (loader) / consumed (MMA)
  uint32_t it = 0;       // KV steps processed so far: parity of s_full / p_part
  uint32_t seg_seq = 0;  // segments processed so far: parity of q_full / o_done / o_free
  bool ok = true;

  // The producer warpgroup hands registers to the softmax warpgroups.  The pool is what the CTA got
  // at launch, 384 threads x 168 registers = 64512, so 2 x 128 x 208 + 128 x 88 = 64512 fits it
  // exactly; asking for more would block the second setmaxnreg.inc forever.  Each side keeps its
  // own copy of the batch loop so the raised budget applies to the softmax code; both sides
  // execute the same sequence of CTA-wide barriers.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    while (true) {
      __syncthreads();  // thread 0 (softmax side) has planned the next batch
      const int n_segs = sh->n_segs;
      if (n_segs == 0) break;
      if (warp == 9) {
        // =============================== TMA producer ===============================
        for (int si = 0; si < n_segs && ok; ++si) {
          const Segment sg = sh->segs[si];
          const int b = sg.row / a.Hkv, hkv = sg.row % a.Hkv;
          if (lane == 0) {
            // Q smem is free once every MMA of the previous segment has completed
            if (seg_seq > 0) ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh->o_done), (seg_seq - 1) & 1, abort_flag, limit);
            if (ok) {
              const uint32_t q_bytes = 2u * 128u * static_cast<uint32_t>(a.G * a.tpt);
              for (int tile = 0; tile < 2; ++tile) {
                const uint32_t bar = ptx::smem_u32(&sh->q_full[tile]);
                ptx::mbar_expect_tx(bar, q_bytes);
                for (int h = 0; h < 2; ++h) {
                  ptx::tma_load_5d(q_smem + tile * kTileBytes + h * kHalfBytes, &q_map, bar, h * 64, 0, hkv,
                                   (2 * sg.pair + tile) * a.tpt, b);
                }
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          for (int base = 2 * sg.j0; base < 2 * sg.j1 && ok; base += 32) {
            // every lane resolves one sub-block of this batch of 32
            const int u = base + lane;
            int page = 0, off = 0;
            if (u < sg.n_sub) {
              int tok;
              if (u < sg.n_past_sub) {
                const int bi = u / a.spb;
                int blk = a.block_idx ? a.block_idx[static_cast<long long>(sg.row) * a.block_idx_stride + bi] : bi;
                if (blk < 0 || blk >= a.past_blocks) {
                  bad_index = true;
                  blk = blk < 0 ? 0 : a.past_blocks - 1;
                }
                tok = blk * a.block_size + (u - bi * a.spb) * kSub;
              } else {
                tok = a.past_tokens + (u - sg.n_past_sub) * kSub;
              }
              const int lp = tok / a.page_size;
              off = tok - lp * a.page_size;
              if (a.page_table) {
                page = (lp < a.pages_per_seq) ? a.page_table[static_cast<long long>(b) * a.pages_per_seq + lp] : -1;
                if (page < 0 || page >= a.num_pages) {
                  bad_index = true;
                  page = 0;
                }
              } else {
                page = b * a.pages_per_seq + lp;  // beyond the tensor: TMA zero-fills
              }
            }
            for (int i = 0; i < 16 && ok; ++i) {
              const int j = (base >> 1) + i;
              if (j >= sg.j1) break;
              const int p0 = __shfl_sync(0xffffffffu, page, 2 * i);
              const int o0 = __shfl_sync(0xffffffffu, off, 2 * i);
              const int p1 = __shfl_sync(0xffffffffu, page, 2 * i + 1);
              const int o1 = __shfl_sync(0xffffffffu, off, 2 * i + 1);
              const bool two = (2 * j + 1) < sg.n_sub;
              if (lane == 0) {
                for (int kv = 0; kv < 2 && ok; ++kv, ++ring_n) {
                  const int slot = ring_n % kStages;
                  const uint32_t phase = (ring_n / kStages) & 1;
                  ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh->ring_empty[slot]), phase ^ 1u, abort_flag, limit);
                  if (!ok) break;
                  const uint32_t bar = ptx::smem_u32(&sh->ring_full[slot]);
                  const CUtensorMap* map = kv == 0 ? &k_map : &v_map;
                  const uint32_t dst = ring_smem + slot * kTileBytes;
                  ptx::mbar_expect_tx(bar, two ? 4u * kBoxBytes : 2u * kBoxBytes);
                  int c0[3], c1[3];
                  c0[a.slot_tok] = o0, c0[a.slot_page] = p0, c0[a.slot_head] = hkv / a.kv_head_div;
                  c1[a.slot_tok] = o1, c1[a.slot_page] = p1, c1[a.slot_head] = hkv / a.kv_head_div;
                  for (int h = 0; h < 2; ++h) {
                    ptx::tma_load_4d(dst + h * kHalfBytes, map, bar, h * 64, c0[0], c0[1], c0[2]);
                    if (two) ptx::tma_load_4d(dst + h * kHalfBytes + kBoxBytes, map, bar, h * 64, c1[0], c1[1], c1[2]);
                  }
                }
              }
              ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
          }
          ++seg_seq;
        }
      } else if (warp == 8) {
        // =============================== MMA issuer ===============================
        if (lane == 0) {
          const uint32_t tS[2] = {tmem + 0u, tmem + 128u};
          const uint32_t tO[2] = {tmem + 256u, tmem + 384u};
          // Descriptors: one base per operand buffer, then a constant added per MMA (the start address
          // sits in the low 14 bits in 16-byte units and never carries), so the single issuing thread
          // spends two adds per instruction instead of rebuilding descriptors.
          const uint64_t q_desc[2] = {ptx::make_smem_desc_sw128(q_smem, 0, 1024),
                                      ptx::make_smem_desc_sw128(q_smem + kTileBytes, 0, 1024)};
          const uint64_t k_desc0 = ptx::make_smem_desc_sw128(ring_smem, 0, 1024);
          const uint64_t v_desc0 = ptx::make_smem_desc_sw128(ring_smem, kHalfBytes, 1024);
          const uint32_t idesc_qk = a.idesc_qk, idesc_pv = a.idesc_pv;
          auto issue_s = [&](int tile, int slot) {
            const uint64_t qd = q_desc[tile];
            const uint64_t kd = k_desc0 + static_cast<uint64_t>(slot * (kTileBytes >> 4));
  #pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint64_t o = static_cast<uint64_t>(((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4);
              ptx::mma_ss(tS[tile], qd + o, kd + o, idesc_qk, k > 0 ? 1u : 0u);
            }
          };
          // k-steps [k0, k1) of O += P.V; kN compile-time so the loop unrolls
          auto issue_pv = [&](int tile, int slot, int k0, int k1, bool first) {
            const uint64_t vd = v_desc0 + static_cast<uint64_t>(slot * (kTileBytes >> 4));
  #pragma unroll
            for (int k = 0; k < 8; ++k) {
              if (k >= k0 && k < k1) {
                ptx::mma_ts(tO[tile], tS[tile] + k * 8, vd + static_cast<uint64_t>(k * (2048 >> 4)), idesc_pv,
                            (first && k == 0) ? 0u : 1u);
              }
            }
          };
          auto wait = [&](uint64_t* bar, uint32_t parity) {
            if (ok) ok = ptx::mbar_wait_bounded(ptx::smem_u32(bar), parity, abort_flag, limit);
            return ok;
          };
          CA_PROF_DECL
          for (int si = 0; si < n_segs && ok; ++si) {
            const Segment sg = sh->segs[si];
            const uint32_t qpar = seg_seq & 1;
            {
              const int slot = ring_n % kStages;
              const uint32_t phase = (ring_n / kStages) & 1;
              if (!(wait(&sh->q_full[0], qpar) && wait(&sh->q_full[1], qpar) && wait(&sh->ring_full[slot], phase))) break;
              ptx::tc_fence_after();
              issue_s(0, slot);
              ptx::tc_commit(ptx::smem_u32(&sh->s_full[0]));
              issue_s(1, slot);
              ptx::tc_commit(ptx::smem_u32(&sh->s_full[1]));
              ptx::tc_commit(ptx::smem_u32(&sh->ring_empty[slot]));
              ++ring_n;
            }
            for (int j = sg.j0; j < sg.j1 && ok; ++j, ++it) {
              const int v_slot = ring_n % kStages;
              const uint32_t v_phase = (ring_n / kStages) & 1;
              ++ring_n;
              const bool more = (j + 1) < sg.j1;
              const int k_slot = ring_n % kStages;
              const uint32_t k_phase = (ring_n / kStages) & 1;
              if (more) ++ring_n;
              const int ksteps = ((2 * j + 1) < sg.n_sub) ? 8 : 4;
              const bool first = j == sg.j0;
              CA_PROF(0)
              if (!wait(&sh->ring_full[v_slot], v_phase)) break;
              CA_PROF(1)
              // P arrives in pieces so P.V starts while the softmax still works
              for (int q = 0; q < kPParts && ok; ++q) {
                if (q > 0) CA_PROF(0)
                if (!wait(&sh->p_part[0][q], it & 1)) break;
                CA_PROF(2 + q)
                // the accumulator is free once the previous segment's epilogue has read it
                if (q == 0 && first && seg_seq > 0 && !wait(&sh->o_free[0], (seg_seq - 1) & 1)) break;
                ptx::tc_fence_after();
                const int k1 = (q + 1) * (8 / kPParts);
                issue_pv(0, v_slot, q * (8 / kPParts), k1 < ksteps ? k1 : ksteps, first);
              }
              if (!ok) break;
              CA_PROF(0)
              if (more) {
                if (!wait(&sh->ring_full[k_slot], k_phase)) break;
                CA_PROF(4)
                ptx::tc_fence_after();
                issue_s(0, k_slot);
                ptx::tc_commit(ptx::smem_u32(&sh->s_full[0]));
              }
              for (int q = 0; q < kPParts && ok; ++q) {
                CA_PROF(0)
                if (!wait(&sh->p_part[1][q], it & 1)) break;
                CA_PROF(5 + q)
                // the accumulator is free once the previous segment's epilogue has read it
                if (q == 0 && first && seg_seq > 0 && !wait(&sh->o_free[1], (seg_seq - 1) & 1)) break;
                ptx::tc_fence_after();
                const int k1 = (q + 1) * (8 / kPParts);
                issue_pv(1, v_slot, q * (8 / kPParts), k1 < ksteps ? k1 : ksteps, first);
              }
              if (!ok) break;
              ptx::tc_commit(ptx::smem_u32(&sh->ring_empty[v_slot]));
              if (more) {
                issue_s(1, k_slot);
                ptx::tc_commit(ptx::smem_u32(&sh->s_full[1]));
                ptx::tc_commit(ptx::smem_u32(&sh->ring_empty[k_slot]));
              }
            }
            if (ok) ptx::tc_commit(ptx::smem_u32(&sh->o_done));
            ++seg_seq;
            CA_PROF(7)
          }
          CA_PROF_FLUSH(0)
        }
      }
      ok = __syncthreads_and(ok ? 1 : 0) != 0;  // all roles finished this batch (or aborted)
      if (!ok) break;
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    while (true) {
      if (tid == 0 && sh->more) plan_segments(a, sh, sh->next_x, span_begin, span_end, R);
      else if (tid == 0) sh->n_segs = 0;
      __syncthreads();
      const int n_segs = sh->n_segs;
      if (n_segs == 0) break;
      {
        // =============================== softmax + epilogue ===============================
        const int tile = warp >> 2;  // 0: A, 1: B
        const int r = tid & 127;     // tile row = TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + lane_base + tile * 128u;
        const uint32_t tO = tmem + lane_base + 256u + tile * 128u;
        const float sc = a.scale_log2;
        uint32_t v[32];
        CA_PROF_DECL
        for (int si = 0; si < n_segs && ok; ++si) {
          const Segment sg = sh->segs[si];
          const int b = sg.row / a.Hkv, hkv = sg.row % a.Hkv;
          const int t = (2 * sg.pair + tile) * a.tpt + r / a.G;  // chunk token of this row
          const int g = r % a.G;
          float m_run = -INFINITY;
          float l_run = 0.f;
          for (int j = sg.j0; j < sg.j1; ++j, ++it) {
            CA_PROF(0)
            ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh->s_full[tile]), it & 1, abort_flag, limit);
            ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the collective TMEM ops
            if (!ok) break;
            CA_PROF(1)
            ptx::tc_fence_after();
            const bool masked = (2 * j + 1) >= sg.n_past_sub;  // a chunk or tail sub-block is in this step
            int lim0 = kSub, lim1 = kSub;
            if (masked) {
              lim0 = visible_cols(2 * j, sg.n_sub, sg.n_past_sub, t + a.q_off);
              lim1 = visible_cols(2 * j + 1, sg.n_sub, sg.n_past_sub, t + a.q_off);
            }
            // the whole S row (128 fp32) comes into registers with one wait
            uint32_t sv[128];
            ptx::tmem_ld32_row<0>(tS + 0, sv);
            ptx::tmem_ld32_row<32>(tS + 32, sv);
            ptx::tmem_ld32_row<64>(tS + 64, sv);
            ptx::tmem_ld32_row<96>(tS + 96, sv);
            ptx::tc_wait_ld();
            CA_PROF(2)
            if (masked) {
  #pragma unroll
              for (int i = 0; i < 128; ++i) {
                const int lim = i < 64 ? lim0 : lim1;
                if ((i & 63) >= lim) sv[i] = 0xff800000u;  // -inf
              }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
  #pragma unroll
            for (int i = 0; i < 128; i += 4) {
              mx0 = fmaxf(mx0, __uint_as_float(sv[i]));
              mx1 = fmaxf(mx1, __uint_as_float(sv[i + 1]));
              mx2 = fmaxf(mx2, __uint_as_float(sv[i + 2]));
              mx3 = fmaxf(mx3, __uint_as_float(sv[i + 3]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            // lazy rescale of the running accumulator
            const float m_new = fmaxf(m_run, mx);
            const bool need = m_new > m_run && (m_run == -INFINITY || (m_new - m_run) * sc > kRescaleThreshold);
            if (__any_sync(0xffffffffu, need)) {
              const float alpha = need ? (m_run == -INFINITY ? 0.f : ptx::ex2((m_run - m_new) * sc)) : 1.0f;
              if (j > sg.j0) {
  #pragma unroll
                for (int c = 0; c < 4; ++c) {
                  ptx::tmem_ld32(tO + c * 32, v);
                  ptx::tc_wait_ld();
  #pragma unroll
                  for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                  ptx::tmem_st32(tO + c * 32, v);
                }
                ptx::tc_wait_st();
              }
              l_run *= alpha;
              if (need) m_run = m_new;
            }
            // P = exp2(S*sc - m*sc) -> 16-bit, written over S.  Masked entries are -inf -> 0; a row
            // that has seen nothing yet (m = -inf) produces zeros.
            const float neg_m = m_run == -INFINITY ? 0.f : -m_run * sc;
            const uint32_t half_bar = ptx::smem_u32(&sh->p_part[tile][0]);
            CA_PROF(3)
            l_run += exp_pack_store<T>(sv, sc, neg_m, tS, half_bar);
            CA_PROF(4)

          }
          if (ok) ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh->o_done), seg_seq & 1, abort_flag, limit);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
          const bool live = (r < a.tpt * a.G) && (t < a.Q);
          if (sg.slot < 0) {
            // whole unit: normalise and write the output rows
            const float inv_l = 1.0f / l_run;
            T* orow = reinterpret_cast<T*>(a.out) + b * a.o_stride_b + static_cast<long long>(t) * a.o_stride_t +
                      static_cast<long long>(hkv * a.G + g) * a.o_stride_h;
  #pragma unroll
            for (int c = 0; c < 4; ++c) {
              ptx::tmem_ld32(tO + c * 32, v);
              ptx::tc_wait_ld();
              if (live) {
  #pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  uint4 w;
                  w.x = pack2<T>(__uint_as_float(v[i + 0]) * inv_l, __uint_as_float(v[i + 1]) * inv_l);
                  w.y = pack2<T>(__uint_as_float(v[i + 2]) * inv_l, __uint_as_float(v[i + 3]) * inv_l);
                  w.z = pack2<T>(__uint_as_float(v[i + 4]) * inv_l, __uint_as_float(v[i + 5]) * inv_l);
                  w.w = pack2<T>(__uint_as_float(v[i + 6]) * inv_l, __uint_as_float(v[i + 7]) * inv_l);
                  *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
                }
              }
            }
            if (live && a.lse) {
              a.lse[(static_cast<long long>(b) * (a.Hkv * a.G) + hkv * a.G + g) * a.Q + t] =
                  0.6931471805599453f * (m_run * sc + log2f(l_run));
            }
          } else {
            // segment of a split unit: unnormalised accumulator, running max and sum to the workspace
            float* po = a.part_o + static_cast<long long>(sg.slot) * kPartialOFloats + tile * (kTileM * kHeadDim);
            float* pml = a.part_ml + static_cast<long long>(sg.slot) * kPartialMLFloats + (tile * kTileM + r) * 2;
  #pragma unroll
            for (int c = 0; c < 4; ++c) {
              ptx::tmem_ld32(tO + c * 32, v);
              ptx::tc_wait_ld();
  #pragma unroll
              for (int i = 0; i < 32; i += 4) {
                const int c4 = (c * 32 + i) >> 2;
                *reinterpret_cast<uint4*>(po + (static_cast<long long>(c4) * kTileM + r) * 4) =
                    make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
              }
            }
            pml[0] = m_run;
            pml[1] = l_run;
          }
          // the accumulator may be overwritten by the next segment
          ptx::tc_fence_before();
          ptx::mbar_arrive(ptx::smem_u32(&sh->o_free[tile]));
          ++seg_seq;
          CA_PROF(5)
        }
        if ((tid & 127) == 0) CA_PROF_FLUSH(10 + 10 * tile)
      }
      ok = __syncthreads_and(ok ? 1 : 0) != 0;  // all roles finished this batch (or aborted)
      if (!ok) break;
    }
  }

  // ---- teardown: every thread arrives here on every path ----
  if (sh->abort_flag) {
    if (warp == 9 && lane == 0) {
      // drain: give copies already issued a bounded chance to land before the CTA exits
      for (int e = (ring_n > kStages ? ring_n - kStages : 0); e < ring_n; ++e) {
        int dummy = 0;
        ptx::mbar_wait_bounded(ptx::smem_u32(&sh->ring_full[e % kStages]), (e / kStages) & 1, &dummy, 100000000ull);
      }
    }
    if (warp == 8 && lane == 0) {
      // drain the tensor pipe (bounded) before TMEM is released
      ptx::tc_commit(ptx::smem_u32(&sh->drain));
      int dummy = 0;
      ptx::mbar_wait_bounded(ptx::smem_u32(&sh->drain), 0, &dummy, 100000000ull);
    }
  }
  if (bad_index && a.status) atomicOr(a.status, CA_STATUS_BAD_INDEX);
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && sh->abort_flag && a.status) atomicOr(a.status, CA_STATUS_TIMEOUT);
#if CA_ATTN_PROFILE
  if (tid == 0) g_prof[blockIdx.x][31] = clock64() - prof_kernel_t0;  // whole kernel
#endif
}

// Merges the segments of every split unit.  One CTA per (attention CTA, tile, 16-column part);
// the CTAs whose slot holds the first segment of a unit (j0 == 0) walk the following CTAs' head
// slots until the unit is complete.  Thread = tile row.  The per-segment weights are computed once
// and kept in shared memory; the loads of the partial accumulators of different segments are
// independent, so several are in flight per thread.  (The first form of this kernel, one CTA per
// (slot, tile) with the weights recomputed inside the column loop, took 70-80 us for the 16 units
// of a tensor-parallel rank with one KV head - longer than the attention kernel itself.)
#ifndef CA_ATTN_COMBINE_PARTS
#define CA_ATTN_COMBINE_PARTS 8
#endif
// Measured (us, attention + merge): 1 KV head 95.3 / 87.4 / 85.4 with 4 / 8 / 16 parts, 4 KV heads
// 229.5 / 227 / 235, a small shape with whole units 30.4 / 30.8 / 32.9: 8 is the balanced choice.
constexpr int kCombineParts = CA_ATTN_COMBINE_PARTS;    // column parts per tile (16 must be divisible by it)
constexpr int kCombineC8 = kHeadDim / 8 / kCombineParts;  // 8-column groups per part
constexpr int kCombineMaxChain = 32;                    // segments whose weights are cached in shared memory

template <typename T>
__global__ void __launch_bounds__(kTileM) attn_combine_kernel(const KernelArgs a, int n_slots) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  __shared__ int chain_sh[256];
  __shared__ float w_sh[kCombineMaxChain][kTileM];
  // blockIdx.x = attention CTA; at most one of its two slots holds the first segment of a cut unit
  // (slot 0 when a unit starts exactly at the span's start, else slot 1)
  const int tile = blockIdx.y, part = blockIdx.z, r = threadIdx.x;
  int slot = 2 * blockIdx.x;
  SegDesc first = a.descs[slot];
  if (first.unit < 0 || first.j0 != 0) {
    slot += 1;
    first = a.descs[slot];
    if (first.unit < 0 || first.j0 != 0) return;
  }
  // chain of slots: this one, then the head slots (even) of the following CTAs
  // (CTAs whose span is empty leave their slots unused and are skipped)
  __shared__ int n_sh;
  __shared__ SegDesc cand_sh[2 * kTileM];
  // the head slots of the following CTAs, fetched by all threads at once (a one-thread walk over
  // global memory costs a dependent load per segment)
  for (int i = r; i < 2 * kTileM; i += kTileM) {
    const int s = (slot / 2 + 1 + i) * 2;
    SegDesc d;
    d.unit = -1, d.j0 = 0, d.j1 = 0, d.n_iter = 0;
    if (s < n_slots) d = a.descs[s];
    cand_sh[i] = d;
  }
  __syncthreads();
  if (r == 0) {
    int n = 0;
    chain_sh[n++] = slot;
    int reached = first.j1;
    for (int i = 0; i < 2 * kTileM && reached < first.n_iter && n < 256; ++i) {
      const SegDesc d = cand_sh[i];
      if (d.unit < 0) continue;
      if (d.unit != first.unit || d.j0 != reached) break;
      chain_sh[n++] = (slot / 2 + 1 + i) * 2;
      reached = d.j1;
    }
    n_sh = reached == first.n_iter ? n : -1;
  }
  __syncthreads();
  const int n = n_sh;
  if (n < 0) {
    if (r == 0 && part == 0 && a.status) atomicOr(a.status, CA_STATUS_BAD_INDEX);
    return;
  }
  const int row = first.unit / a.n_pairs, pair = first.unit % a.n_pairs;
  const int b = row / a.Hkv, hkv = row % a.Hkv;
  const int t = (2 * pair + tile) * a.tpt + r / a.G;
  const int g = r % a.G;
  const bool live = (r < a.tpt * a.G) && (t < a.Q);
  const float sc = a.scale_log2;
  auto ml_of = [&](int i) { return a.part_ml + static_cast<long long>(chain_sh[i]) * kPartialMLFloats + (tile * kTileM + r) * 2; };
  float m = -INFINITY;
#pragma unroll 8
  for (int i = 0; i < n; ++i) m = fmaxf(m, __ldg(ml_of(i)));
  float l = 0.f;
#pragma unroll 8
  for (int i = 0; i < n; ++i) {
    const float2 ml = __ldg(reinterpret_cast<const float2*>(ml_of(i)));
    const float w = ml.x == -INFINITY ? 0.f : ptx::ex2((ml.x - m) * sc);
    if (i < kCombineMaxChain) w_sh[i][r] = w;
    l += ml.y * w;
  }
  const float inv_l = 1.0f / l;
  auto weight = [&](int i) {
    if (i < kCombineMaxChain) return w_sh[i][r];  // written by this very thread
    const float ms = ml_of(i)[0];
    return ms == -INFINITY ? 0.f : ptx::ex2((ms - m) * sc);
  };
  T* orow = reinterpret_cast<T*>(a.out) + b * a.o_stride_b + static_cast<long long>(t) * a.o_stride_t +
            static_cast<long long>(hkv * a.G + g) * a.o_stride_h;
#pragma unroll
  for (int cc = 0; cc < kCombineC8; ++cc) {
    const int c8 = part * kCombineC8 + cc;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int i = 0; i < n; ++i) {
      const float w = weight(i);
      const float* po = a.part_o + static_cast<long long>(chain_sh[i]) * kPartialOFloats + tile * (kTileM * kHeadDim);
      const float4 x0 = *reinterpret_cast<const float4*>(po + (static_cast<long long>(2 * c8) * kTileM + r) * 4);
      const float4 x1 = *reinterpret_cast<const float4*>(po + (static_cast<long long>(2 * c8 + 1) * kTileM + r) * 4);
      acc[0] += w * x0.x, acc[1] += w * x0.y, acc[2] += w * x0.z, acc[3] += w * x0.w;
      acc[4] += w * x1.x, acc[5] += w * x1.y, acc[6] += w * x1.z, acc[7] += w * x1.w;
    }
    if (live) {
      uint4 w;
      w.x = pack2<T>(acc[0] * inv_l, acc[1] * inv_l);
      w.y = pack2<T>(acc[2] * inv_l, acc[3] * inv_l);
      w.z = pack2<T>(acc[4] * inv_l, acc[5] * inv_l);
      w.w = pack2<T>(acc[6] * inv_l, acc[7] * inv_l);
      *reinterpret_cast<uint4*>(orow + c8 * 8) = w;
    }
  }
  if (live && part == 0 && a.lse) {
    a.lse[(static_cast<long long>(b) * (a.Hkv * a.G) + hkv * a.G + g) * a.Q + t] = 0.6931471805599453f * (m * sc + log2f(l));
  }
}

static int encode_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims,
                      const cuuint64_t* strides_bytes, const cuuint32_t* box, const char* what) {
  tensor_map_encode_fn enc = get_tensor_map_encoder();
  if (!enc) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  CUresult res = enc(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides_bytes, box,
                     elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)res);
  return CA_OK;
}

static int validate(const ca_attn_params* p) {
  CA_REQUIRE(p != nullptr, "params is null");
  CA_REQUIRE(p->q && p->out && p->kv.k && p->kv.v, "q, out, kv.k and kv.v must be non-null");
  CA_REQUIRE(p->D == kHeadDim, "head dim must be 128, got %d", p->D);
  CA_REQUIRE(p->dtype == CA_DTYPE_BF16 || p->dtype == CA_DTYPE_F16, "dtype must be bf16 or f16");
  CA_REQUIRE(p->B > 0 && p->Q > 0 && p->Hq > 0 && p->Hkv > 0, "B, Q, Hq, Hkv must be positive");
  CA_REQUIRE(p->Hq % p->Hkv == 0, "Hq (%d) must be a multiple of Hkv (%d)", p->Hq, p->Hkv);
  CA_REQUIRE(p->kv.head_div >= 0 && (p->kv.head_div <= 1 || p->Hkv % p->kv.head_div == 0),
             "kv.head_div (%d) must divide the number of block-table rows per batch entry (Hkv = %d)", p->kv.head_div, p->Hkv);
  CA_REQUIRE(p->Hq / p->Hkv <= 128, "GQA group larger than 128 is not supported");
  CA_REQUIRE(static_cast<long long>(p->B) * p->Hkv <= kMaxRows, "more than %d (batch x kv head) rows are not supported", kMaxRows);
  CA_REQUIRE(p->block_size > 0 && p->block_size % kSub == 0, "block_size must be a positive multiple of 64");
  CA_REQUIRE(p->kv_len >= p->Q, "kv_len (%d) must be >= Q (%d)", p->kv_len, p->Q);
  CA_REQUIRE((p->kv_len - p->Q) % p->block_size == 0 || p->block_idx == nullptr,
             "with a block table the past length (kv_len - Q = %d) must be a multiple of block_size (%d)", p->kv_len - p->Q,
             p->block_size);
  CA_REQUIRE(p->kv.page_size > 0 && (p->kv.page_size % kSub == 0 || p->kv.pages_per_seq == 1),
             "page_size must be a positive multiple of 64 (any length when a sequence is one page)");
  CA_REQUIRE(p->kv.num_pages > 0 && p->kv.pages_per_seq > 0, "num_pages and pages_per_seq must be positive");
  CA_REQUIRE((long long)p->kv.pages_per_seq * p->kv.page_size >= p->kv_len,
             "pages_per_seq*page_size (%lld) does not cover kv_len (%d)",
             (long long)p->kv.pages_per_seq * p->kv.page_size, p->kv_len);
  CA_REQUIRE(p->kv.page_stride % 8 == 0 && p->kv.token_stride % 8 == 0 && p->kv.head_stride % 8 == 0,
             "kv strides must be multiples of 8 elements (16 bytes)");
  CA_REQUIRE(p->q_stride_b % 8 == 0 && p->q_stride_t % 8 == 0 && p->q_stride_h % 8 == 0,
             "q strides must be multiples of 8 elements (16 bytes)");
  CA_REQUIRE(p->o_stride_b % 8 == 0 && p->o_stride_t % 8 == 0 && p->o_stride_h % 8 == 0,
             "out strides must be multiples of 8 elements (16 bytes)");
  CA_REQUIRE((reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->out) |
              reinterpret_cast<uintptr_t>(p->kv.k) | reinterpret_cast<uintptr_t>(p->kv.v)) % 16 == 0,
             "q, out, k, v must be 16-byte aligned");
  if (p->block_idx) {
    CA_REQUIRE(p->counts != nullptr, "counts is required with block_idx");
    CA_REQUIRE(p->block_idx_stride > 0 || p->kv_len == p->Q, "block_idx_stride must be positive");
  }
  CA_REQUIRE(p->workspace == nullptr || reinterpret_cast<uintptr_t>(p->workspace) % 256 == 0,
             "workspace must be 256-byte aligned");
  return CA_OK;
}

// Workspace layout for a grid of nc CTAs: descriptors, then (max, sum) pairs, then accumulators.
static size_t desc_bytes(int nc) { return ((static_cast<size_t>(2) * nc * sizeof(SegDesc) + 255) / 256) * 256; }
static size_t ml_bytes(int nc) { return static_cast<size_t>(2) * nc * kPartialMLFloats * sizeof(float); }
static size_t o_bytes(int nc) { return static_cast<size_t>(2) * nc * kPartialOFloats * sizeof(float); }
static size_t workspace_bytes_for(int nc) { return desc_bytes(nc) + ml_bytes(nc) + o_bytes(nc); }


// ---- scratch for callers that cannot allocate -------------------------------------------------
// Room for the split-unit partials of a grid of up to kStaticMaxCtas CTAs (a B200 has 148 SMs):
// 160 * 2 slots * (128 KiB accumulator + 2 KiB max/sum) + descriptors = 41.6 MiB, resident on every
// GPU that loads the library until the process exits.
constexpr int kStaticMaxCtas = 160;
constexpr size_t kStaticScratchBytes =
    ((2 * kStaticMaxCtas * sizeof(SegDesc) + 255) / 256) * 256 +
    static_cast<size_t>(2) * kStaticMaxCtas * (kPartialMLFloats + kPartialOFloats) * sizeof(float);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device.  In host code the array's name is only
// a stand-in for the symbol, not a pointer a kernel can use, so the address is asked from the
// runtime once per device (with that device current) and remembered.
static int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = 0;
  CA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(CA_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      return fail(CA_ERR_CUDA, "cudaGetSymbolAddress(static attention scratch) failed: %s", cudaGetErrorString(err));
    }
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return CA_OK;
}

}  // namespace attn
}  // namespace ca

extern "C" {

int ca_attn_workspace_bytes(const ca_attn_params* p, size_t* bytes_out) {
  using namespace ca;
  CA_REQUIRE(bytes_out != nullptr, "bytes_out is null");
  int rc = attn::validate(p);
  if (rc != CA_OK) return rc;
  DeviceInfo dev;
  rc = get_device_info(&dev);
  if (rc != CA_OK) return rc;
  *bytes_out = attn::workspace_bytes_for(dev.sm_count);
  return CA_OK;
}

int ca_attn_compact(const ca_attn_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::attn;
  int rc = validate(p);
  if (rc != CA_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  DeviceInfo dev;
  rc = get_device_info(&dev);
  if (rc != CA_OK) return rc;
  if (dev.cc_major != 10) return fail(CA_ERR_UNSUPPORTED, "this library targets sm_100a; device is sm_%d%d", dev.cc_major, dev.cc_minor);

  const int G = p->Hq / p->Hkv;
  const int tpt = kTileM / G;
  const int n_mtiles = ceil_div(p->Q, tpt);
  const int n_pairs = ceil_div(n_mtiles, 2);
  const CUtensorMapDataType dt = p->dtype == CA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;

  CUtensorMap q_map, k_map, v_map;
  int slot_tok = 0, slot_page = 1, slot_head = 2;
  {
    // (d, g, hkv, token, batch): the box walks g fastest, then tokens, so tile row = token*G + g
    cuuint64_t dims[5] = {(cuuint64_t)kHeadDim, (cuuint64_t)G, (cuuint64_t)p->Hkv, (cuuint64_t)p->Q, (cuuint64_t)p->B};
    cuuint64_t strides[4] = {(cuuint64_t)p->q_stride_h * 2, (cuuint64_t)p->q_stride_h * G * 2,
                             (cuuint64_t)p->q_stride_t * 2, (cuuint64_t)p->q_stride_b * 2};
    cuuint32_t box[5] = {64, (cuuint32_t)G, 1, (cuuint32_t)tpt, 1};
    rc = encode_map(&q_map, dt, 5, p->q, dims, strides, box, "q");
    if (rc != CA_OK) return rc;
  }
  {
    // roles: 0 token-in-page, 1 page, 2 head; outer dimensions sorted by ascending stride
    const cuuint64_t role_dim[3] = {(cuuint64_t)p->kv.page_size, (cuuint64_t)p->kv.num_pages,
                                    (cuuint64_t)(p->Hkv / (p->kv.head_div > 1 ? p->kv.head_div : 1))};
    const cuuint64_t role_stride[3] = {(cuuint64_t)p->kv.token_stride * 2, (cuuint64_t)p->kv.page_stride * 2,
                                       (cuuint64_t)p->kv.head_stride * 2};
    const cuuint32_t role_box[3] = {64, 1, 1};
    int order[3] = {0, 1, 2};
    for (int i = 0; i < 3; ++i)
      for (int j = i + 1; j < 3; ++j)
        if (role_stride[order[j]] < role_stride[order[i]]) { int t = order[i]; order[i] = order[j]; order[j] = t; }
    cuuint64_t dims[4] = {(cuuint64_t)kHeadDim, 0, 0, 0};
    cuuint64_t strides[3];
    cuuint32_t box[4] = {64, 0, 0, 0};
    int slot_of_role[3];
    for (int i = 0; i < 3; ++i) {
      dims[i + 1] = role_dim[order[i]];
      strides[i] = role_stride[order[i]];
      box[i + 1] = role_box[order[i]];
      slot_of_role[order[i]] = i;
    }
    slot_tok = slot_of_role[0], slot_page = slot_of_role[1], slot_head = slot_of_role[2];
    rc = encode_map(&k_map, dt, 4, p->kv.k, dims, strides, box, "k");
    if (rc != CA_OK) return rc;
    rc = encode_map(&v_map, dt, 4, p->kv.v, dims, strides, box, "v");
    if (rc != CA_OK) return rc;
  }

  KernelArgs a;
  a.Q = p->Q;
  a.G = G;
  a.Hkv = p->Hkv;
  a.B = p->B;
  a.tpt = tpt;
  a.n_pairs = n_pairs;
  a.block_size = p->block_size;
  // a dense launch whose past is not a block multiple treats the remainder as the head of the chunk region
  a.q_off = (p->kv_len - p->Q) % p->block_size;
  a.past_tokens = p->kv_len - p->Q - a.q_off;
  a.past_blocks = a.past_tokens / p->block_size;
  a.spb = p->block_size / kSub;
  a.page_size = p->kv.page_size;
  a.pages_per_seq = p->kv.pages_per_seq;
  a.num_pages = p->kv.num_pages;
  a.block_idx = p->block_idx;
  a.block_idx_stride = p->block_idx_stride;
  a.counts = p->counts;
  a.page_table = p->kv.page_table;
  a.out = p->out;
  a.o_stride_b = p->o_stride_b;
  a.o_stride_t = p->o_stride_t;
  a.o_stride_h = p->o_stride_h;
  a.lse = p->lse;
  a.scale_log2 = p->softmax_scale * 1.4426950408889634f;
  a.status = p->status;
  const uint32_t fmt = p->dtype == CA_DTYPE_BF16 ? 1u : 0u;
  a.idesc_qk = ptx::make_idesc_f16(fmt, kTileM, kTileN, 0, 0);
  a.idesc_pv = ptx::make_idesc_f16(fmt, kTileM, kHeadDim, 0, 1);
  a.wait_limit_ns = 2000000000ull;
  a.kv_head_div = p->kv.head_div > 1 ? p->kv.head_div : 1;
  a.slot_tok = slot_tok;
  a.slot_page = slot_page;
  a.slot_head = slot_head;

  // persistent grid: one CTA per SM, never more CTAs than units when units cannot be cut
  const long long n_units = static_cast<long long>(p->B) * p->Hkv * n_pairs;
  int grid = dev.sm_count;
  // Cutting units costs partial traffic and a combine launch; it pays when whole units would leave SMs
  // idle (few rows per rank under tensor parallelism, a nearly empty last wave) or unevenly loaded (the
  // rows of a block table differ in length).  Measured on B200, 128 units on 148 SMs, 128K context:
  // with ~460 selected blocks per row (236 KV steps per unit) whole units 503 us, cut 450 us in a short
  // run and 516 vs 512 us in a seconds-long loop (the board then holds a lower clock with every SM busy);
  // dense attention of the same shape (1028 steps per unit, 2 ms per launch) 1923 us whole, 2028 us cut.
  // So a launch that already fills more than 80 % of a wave is cut only while its units are short.
  // 16 units (one KV head of a tensor-parallel rank): 442 us whole, 91 us cut.
  // (CA_ATTN_SPLIT_PERCENT overrides the 90 % threshold in development builds.)
  const long long waves = (n_units + dev.sm_count - 1) / dev.sm_count;
#ifdef CA_ATTN_SPLIT_PERCENT
  const bool want_split = n_units * 100 < waves * dev.sm_count * CA_ATTN_SPLIT_PERCENT;
#else
  const bool want_split = n_units * 100 < waves * dev.sm_count * 90;
#endif
  a.max_cut_steps = n_units * 100 >= waves * dev.sm_count * 80 ? 512 : 0;
  const bool can_split = p->workspace != nullptr && p->workspace_bytes >= workspace_bytes_for(grid);
  a.split = (want_split && can_split) ? 1 : 0;
  if (!a.split && n_units < grid) grid = static_cast<int>(n_units);
  a.descs = nullptr, a.part_ml = nullptr, a.part_o = nullptr;
  if (a.split) {
    uint8_t* ws = static_cast<uint8_t*>(p->workspace);
    a.descs = reinterpret_cast<SegDesc*>(ws);
    a.part_ml = reinterpret_cast<float*>(ws + desc_bytes(grid));
    a.part_o = reinterpret_cast<float*>(ws + desc_bytes(grid) + ml_bytes(grid));
  }

  // the opt-in shared-memory size is a per-device function attribute: set once per device and type
  // (the call costs a few microseconds of host time, which short contexts notice)
  {
    static std::mutex mu;
    static bool done[2][64] = {};
    const int ti = p->dtype == CA_DTYPE_BF16 ? 0 : 1;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[ti][dev.ordinal]) {
      if (ti == 0) {
        CA_CUDA(cudaFuncSetAttribute(attn_compact_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      } else {
        CA_CUDA(cudaFuncSetAttribute(attn_compact_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      }
      done[ti][dev.ordinal] = true;
    }
  }
  if (p->dtype == CA_DTYPE_BF16) {
    // a programmatic dependent launch: barrier set-up, TMEM allocation and descriptor prefetch overlap the tail of
    // the table builder; the kernel waits (griddepcontrol.wait) before it reads anything from global memory
    launch_kernel_as(true, attn_compact_kernel<__nv_bfloat16>, dim3(grid), dim3(kThreads), kSmemBytes, stream, q_map, k_map, v_map, a);
  } else {
    launch_kernel_as(true, attn_compact_kernel<__half>, dim3(grid), dim3(kThreads), kSmemBytes, stream, q_map, k_map, v_map, a);
  }
  CA_LAUNCH_CHECK("attn_compact_kernel");
  if (a.split) {
    if (p->dtype == CA_DTYPE_BF16) {
      launch_kernel_as(CA_ATTN_MERGE_DEPENDENT != 0, attn_combine_kernel<__nv_bfloat16>, dim3(grid, 2, kCombineParts), dim3(kTileM), 0, stream, a, 2 * grid);
    } else {
      launch_kernel_as(CA_ATTN_MERGE_DEPENDENT != 0, attn_combine_kernel<__half>, dim3(grid, 2, kCombineParts), dim3(kTileM), 0, stream, a, 2 * grid);
    }
    CA_LAUNCH_CHECK("attn_combine_kernel");
  }
  return CA_OK;
}

int ca_attn_compact_static_scratch(const ca_attn_params* p, ca_stream_t stream) {
  using namespace ca;
  using namespace ca::attn;
  int rc = validate(p);
  if (rc != CA_OK) return rc;
  DeviceInfo dev;
  rc = get_device_info(&dev);
  if (rc != CA_OK) return rc;
  const size_t need = workspace_bytes_for(dev.sm_count);
  if (need > kStaticScratchBytes) {
    return fail(CA_ERR_CAPACITY,
                "this device has %d SMs and needs %zu bytes of attention scratch; the built-in scratch holds %zu bytes "
                "(up to %d SMs): use ca_attn_compact with a caller-provided workspace",
                dev.sm_count, need, kStaticScratchBytes, kStaticMaxCtas);
  }
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);  // first call on a device looks the address up
  if (rc != CA_OK) return rc;
  ca_attn_params q = *p;
  q.workspace = scratch;
  q.workspace_bytes = kStaticScratchBytes;
  return ca_attn_compact(&q, stream);
}

}  // extern "C"

#if CA_ATTN_PROFILE
// Development builds only: copies the cycle counters of the last launch to the host.
extern "C" int ca_debug_attn_profile(long long* dst) {
  return cudaMemcpyFromSymbol(dst, ca::attn::g_prof, sizeof(long long) * 160 * 32) == cudaSuccess ? 0 : -3;
}
#endif
