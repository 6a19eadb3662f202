// Row-parallel output projection fused with the tensor-parallel reduction, over peer memory.
//
// Under KV-head tensor parallelism every rank holds the attention output of its own heads,
// A_r [M, K_r], and the matching input columns of the output projection, W_r [N, K_r]; the layer
// output is sum_r A_r . W_r^T on every rank.  The reference runs a library GEMM and then an NCCL
// all-reduce whose wait it can defer (compact_attn/prefill_sparse/llama/modeling_llama_seerattn.py:111-120,
// modeling_llama_flashprefill_compactattn.py:37-41, 321-322).  Here the sum travels inside the kernels:
//
//   1. oproj_gemm_kernel   tcgen05 GEMM, one CTA per 128 x 256 output tile: TMA loads of A and W from this
//      GPU's own memory into a 4-stage ring, 128x256x16 MMAs into a TMEM accumulator, and an epilogue that
//      lays the 16-bit partial tile down in shared memory and sends it with bulk copies (512 bytes per row)
//      into the staging buffer of the rank(s) that reduce the tile - peer-mapped memory - then fences and
//      bumps that tile's arrival counter there.
//   2. oproj_reduce_kernel four CTAs per tile: wait (bounded) until all `world` partials of the tile have
//      arrived, sum them in fp32, store the finished 16-bit tile.  Launched programmatically behind the GEMM
//      without a grid-dependency wait, so its CTAs are seated while the GEMM still runs.
//   3. oproj_wait_kernel   (two-shot only) one thread: waits (bounded) until this rank's output holds all tiles.
//
// Two exchange forms.  Two-shot (any world): tile t is reduced by rank t % world, which then stores the result
// into EVERY rank's output and bumps every rank's count of finished tiles - the traffic of a reduce-scatter
// plus an all-gather, (world-1)/world of the output each way.  One-shot (two ranks, the default there): every
// partial tile goes to both ranks and each rank reduces all tiles into its own output - the same bytes over
// NVLink on two ranks, but one exchange and one chain of signalling latencies instead of two and no final
// wait.  Its staging buffer is used in halves by alternate calls: a rank one call ahead writes the other
// half, and it cannot get two calls ahead because its own reduction waits for the slower rank's tiles.
//
// No TMA load ever touches another GPU's memory and nothing uses cluster multicast.  Counters only grow
// (targets are multiples of per-row-block call counts kept by the host), so nothing has to be reset between
// calls and M may change from call to call.  A wait that runs out sets CA_STATUS_TIMEOUT and the kernel
// returns; the output is then invalid but the context stays usable.
//
// Measured and rejected: computing the tile as two passes over K (128 columns each) so that the first half
// travels while the second is computed - the two passes load A twice and 128-column passes need 128 bytes per
// clock and SM from L2, more than it delivers: the GEMM alone went from 16.4 to 28.2 us (M 1024, K 2048).
#include "ca_common.cuh"

#include <mutex>
#include <type_traits>

namespace ca {
namespace oproj {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;   // 16 KB
constexpr int kWBytes = kBN * kBK * 2;   // 32 KB
constexpr int kStageBytes = kABytes + kWBytes;
constexpr int kThreads = 192;            // warp 0 TMA, warp 1 MMA (+ TMEM alloc), warps 2-5 epilogue
constexpr int kMaxWorld = 8;
constexpr int kTileElems = kBM * kBN;
constexpr int kMaxRowTiles = 128;        // rows per call <= 128 * 128

struct GemmArgs {
  int M, N, K;
  int tiles_n, n_tiles;
  int world, rank, tiles_per_owner;
  int one_shot;                      // 1: every tile goes to every rank (no broadcast afterwards)
  int via_switch;                    // 1: every tile stays in this rank's own staging buffer (slot = tile); the owner
                                     //    sums the ranks' copies with multimem.ld_reduce through the NVLink switch
  int slot_tiles;                    // tiles per source rank in a staging buffer (two-shot: tiles_per_owner; one-shot: n_tiles)
  long long buf_off_elems;           // one-shot: offset of this call's half of the double-buffered staging area
  void* stage[kMaxWorld];            // every rank's staging buffer: [src][tile slot][128][256] 16-bit
  uint32_t* tile_counters[kMaxWorld];
  void* out_local;                   // world == 1: the output itself
  long long out_stride_m;
  uint32_t idesc;
  unsigned long long wait_limit_ns;
  int32_t* status;
};

// Where a partial tile goes and who is told.  Data: rank `data_rank(di)`, element offset `data_off`; signals:
// rank `signal_rank(si)`, counter `signal_slot`.
struct TileRoute {
  int n_data, n_signal, owner, signal_slot;
  long long data_off;
  int rank, world, one_shot, via_switch;
  __device__ __forceinline__ int data_rank(int di) const {
    return via_switch ? rank : (one_shot ? (rank + 1 + di) % world : owner);   // one exchange: the peers first, this rank last
  }
  __device__ __forceinline__ int signal_rank(int si) const { return one_shot ? (rank + 1 + si) % world : owner; }
};
__device__ __forceinline__ TileRoute route_tile(const GemmArgs& a, int tile) {
  TileRoute r;
  r.rank = a.rank, r.world = a.world, r.one_shot = a.one_shot, r.via_switch = a.via_switch;
  r.owner = a.world > 1 ? tile % a.world : 0;
  r.n_data = (a.world > 1 && a.one_shot) ? a.world : 1;
  r.n_signal = r.n_data;
  r.signal_slot = a.one_shot ? tile : (a.world > 1 ? tile / a.world : 0);
  r.data_off = a.via_switch ? static_cast<long long>(tile) * kTileElems
                            : a.buf_off_elems + (static_cast<long long>(a.rank) * a.slot_tiles + r.signal_slot) * kTileElems;
  return r;
}

struct Shared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kSmemBytes = kStages * kStageBytes + 1024 + static_cast<int>(sizeof(Shared));

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// Untiled bulk copy shared -> global (both addresses 16-byte aligned, size a multiple of 16 bytes); the
// destination may be peer-mapped memory.  Completion is tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Polls *p until it reaches `target` (counters only grow; compared as a signed difference so a wrap is
// harmless) or the time limit passes.
__device__ bool wait_counter(const uint32_t* p, uint32_t target, uint64_t limit_ns) {
  if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  while (true) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return true;
    if (ptx::globaltimer_ns() - t0 > limit_ns) return false;
    __nanosleep(200);
  }
}

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
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    oproj_gemm_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map, const GemmArgs a) {
  ptx::grid_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  Shared* sh = reinterpret_cast<Shared*>(smem_aligned + kStages * kStageBytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &sh->abort_flag;
  const uint64_t limit = a.wait_limit_ns;
  if (tid == 0) {
    sh->abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&sh->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sh->empty[s]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(&sh->acc_full), 1);
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&sh->tmem_base), kBN);
    ptx::tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    ptx::tma_prefetch_desc(&a_map);
    ptx::tma_prefetch_desc(&w_map);
  }
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  const int tile = blockIdx.x;
  const int tm = tile / a.tiles_n, tn = tile % a.tiles_n;
  const int k_steps = a.K / kBK;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      for (int ks = 0; ks < k_steps && ok; ++ks) {
        const int s = ks % kStages;
        const uint32_t phase = (ks / kStages) & 1;
        ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh->empty[s]), phase ^ 1u, abort_flag, limit);
        if (!ok) break;
        const uint32_t bar = ptx::smem_u32(&sh->full[s]);
        const uint32_t dst = smem_base + s * kStageBytes;
        ptx::mbar_expect_tx(bar, kStageBytes);
        tma_load_2d(dst, &a_map, bar, ks * kBK, tm * kBM);
        tma_load_2d(dst + kABytes, &w_map, bar, ks * kBK, tn * kBN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int ks = 0; ks < k_steps && ok; ++ks) {
        const int s = ks % kStages;
        const uint32_t phase = (ks / kStages) & 1;
        ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh->full[s]), phase, abort_flag, limit);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint64_t ad = ptx::make_smem_desc_sw128(smem_base + s * kStageBytes, 0, 1024);
        const uint64_t wd = ptx::make_smem_desc_sw128(smem_base + s * kStageBytes + kABytes, 0, 1024);
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k) {
          ptx::mma_ss(tmem, ad + static_cast<uint64_t>((k * 32) >> 4), wd + static_cast<uint64_t>((k * 32) >> 4), a.idesc,
                      (ks > 0 || k > 0) ? 1u : 0u);
        }
        ptx::tc_commit(ptx::smem_u32(&sh->empty[s]));
      }
      if (ok) ptx::tc_commit(ptx::smem_u32(&sh->acc_full));
    }
  } else {
    // epilogue: thread = tile row (TMEM lane).  The 16-bit row is laid down in shared memory (the ring is idle
    // by now: every load has landed and every MMA has read its operands; rows padded by 16 bytes so that the
    // 16-byte pieces of 8 neighbouring rows fall into different banks) and leaves as one 512-byte bulk copy per
    // row and destination.  A thread-per-row store straight from registers sends 16-byte pieces 512 bytes
    // apart, which over NVLink cost ~4x the time of the whole GEMM.
    const int quad = warp & 3;
    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh->acc_full), 0, abort_flag, limit);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      ptx::tc_fence_after();
      const TileRoute route = route_tile(a, tile);
      constexpr int kRowPitch = kBN * 2 + 16;
      uint8_t* my_row = smem_aligned + (quad * 32 + lane) * kRowPitch;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 2
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t v[32];
        ptx::tmem_ld32(taddr + c * 32, v);
        ptx::tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 w;
          w.x = pack2<T>(__uint_as_float(v[i + 0]), __uint_as_float(v[i + 1]));
          w.y = pack2<T>(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
          w.z = pack2<T>(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
          w.w = pack2<T>(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
          *reinterpret_cast<uint4*>(my_row + (c * 32 + i) * 2) = w;
        }
      }
      ptx::fence_proxy_async_smem();   // this thread's row is visible to the bulk-copy engine
      const int row = tm * kBM + quad * 32 + lane;
      if (row < a.M) {
        for (int di = 0; di < route.n_data; ++di) {
          T* dst;
          if (a.world > 1) {
            dst = reinterpret_cast<T*>(a.stage[route.data_rank(di)]) + route.data_off + static_cast<long long>(quad * 32 + lane) * kBN;
          } else {
            dst = reinterpret_cast<T*>(a.out_local) + static_cast<long long>(row) * a.out_stride_m + tn * kBN;
          }
          bulk_store(dst, ptx::smem_u32(my_row), kBN * 2);
        }
        bulk_commit();
        bulk_wait_all();   // the copies have been performed (not merely read out of shared memory)
      }
      if (a.world > 1) {
        // the partial tile is out: make it visible system-wide, then tell its reader(s)
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid >= 64 && tid < 64 + route.n_signal) red_add_release_sys(a.tile_counters[route.signal_rank(tid - 64)] + route.signal_slot, 1u);
      }
    }
  }
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  if (sh->abort_flag && warp == 1 && lane == 0) {
    // drain the tensor pipe (bounded) before TMEM is released
    ptx::tc_commit(ptx::smem_u32(&sh->acc_full));
    int dummy = 0;
    ptx::mbar_wait_bounded(ptx::smem_u32(&sh->acc_full), 1, &dummy, 100000000ull);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kBN);
  }
  if (tid == 0 && sh->abort_flag && a.status) atomicOr(a.status, CA_STATUS_TIMEOUT);
}

// The exchange without the GEMM: `src` already holds this rank's partial [M, N] (a_stride_m elements between
// rows) and is pushed tile by tile exactly as the GEMM's epilogue would push it.  One CTA per 128 x 256 tile,
// 256 threads, 16 bytes per thread and step (a warp covers one 512-byte tile row), all loads of a pass issued
// before its stores.
template <typename T>
__global__ void __launch_bounds__(256) oproj_push_kernel(const T* __restrict__ src, long long src_stride_m, const GemmArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  const int tile = blockIdx.x;
  const int tm = tile / a.tiles_n, tn = tile % a.tiles_n;
  const TileRoute route = route_tile(a, tile);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_live = min(kBM, a.M - tm * kBM);
  const T* tile_src = src + static_cast<long long>(tm * kBM) * src_stride_m + tn * kBN + lane * 8;
  for (int r0 = warp; r0 < rows_live; r0 += 8 * 8) {   // 8 warps, 8 rows each per pass
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = r0 + u * 8;
      v[u] = r < rows_live ? *reinterpret_cast<const uint4*>(tile_src + static_cast<long long>(r) * src_stride_m) : make_uint4(0u, 0u, 0u, 0u);
    }
    for (int di = 0; di < route.n_data; ++di) {
      T* dst = reinterpret_cast<T*>(a.stage[route.data_rank(di)]) + route.data_off + lane * 8;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int r = r0 + u * 8;
        if (r < rows_live) *reinterpret_cast<uint4*>(dst + static_cast<long long>(r) * kBN) = v[u];
      }
    }
  }
  // the partial tile is out: make it visible system-wide, then tell its reader(s)
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < route.n_signal) red_add_release_sys(a.tile_counters[route.signal_rank(threadIdx.x)] + route.signal_slot, 1u);
}

struct ReduceArgs {
  int M, N, tiles_n, n_tiles, world, rank, tiles_per_owner;
  int one_shot, slot_tiles;            // as in GemmArgs
  int split;                           // CTAs per tile: 4, 8, 16 or 32
  long long buf_off_elems;
  uint32_t row_target[kMaxRowTiles];   // arrivals expected at a tile of row tile tm once this call's partials are in
  const void* stage_local;             // this rank's staging buffer
  const uint32_t* tile_counters_local;
  void* out[kMaxWorld];                // every rank's output [M, N]
  long long out_stride_m;
  uint32_t* done_counters[kMaxWorld];
  unsigned long long wait_limit_ns;
  int32_t* status;
};

constexpr int kMaxReduceSplit = 32;  // a tile's 128 rows go to 4, 8, 16 or 32 CTAs: enough CTAs to fill the GPU when a
                                     // rank owns few tiles; a finished part counts kMaxReduceSplit / split, so a
                                     // finished tile always adds kMaxReduceSplit to the ranks' done counters

// `split` CTAs per tile this rank reduces: sum of the `world` staged partials -> every rank's output.
template <typename T>
__global__ void __launch_bounds__(256) oproj_reduce_kernel(const ReduceArgs a) {
  // Launched programmatically behind the GEMM and deliberately without a grid-dependency wait: everything this
  // kernel reads is guarded by a tile counter (release by the producer, acquire here), so its CTAs may take
  // their seats while the GEMM's CTAs are still computing and reduce each tile the moment its partials land.
  // The GEMM itself is a plain launch, so nothing of an earlier call or of the producer of A is overtaken.
  ptx::grid_launch_dependents();
  __shared__ int sh_ok;
  const int lt = blockIdx.x / a.split, part = blockIdx.x % a.split;   // lt: tile slot and counter on this rank
  const int tile = a.one_shot ? lt : lt * a.world + a.rank;
  if (tile >= a.n_tiles) return;
  if (threadIdx.x == 0) {
    sh_ok = wait_counter(a.tile_counters_local + lt, a.row_target[tile / a.tiles_n], a.wait_limit_ns) ? 1 : 0;
    if (!sh_ok && a.status) atomicOr(a.status, CA_STATUS_TIMEOUT);
  }
  __syncthreads();
  const bool ok = sh_ok != 0;
  if (ok) {
    const int tm = tile / a.tiles_n, tn = tile % a.tiles_n;
    const T* base = reinterpret_cast<const T*>(a.stage_local) + a.buf_off_elems + static_cast<long long>(lt) * kTileElems;
    const long long src_stride = static_cast<long long>(a.slot_tiles) * kTileElems;
    const int d0 = a.one_shot ? a.rank : 0, d1 = a.one_shot ? a.rank + 1 : a.world;   // one-shot: only this rank's output
    // 8 elements (16 bytes) per thread and step; a row of the tile is 32 such groups
    const int part_groups = kTileElems / 8 / a.split;
    for (int e = part * part_groups + threadIdx.x; e < (part + 1) * part_groups; e += 256) {
      const int r = e / (kBN / 8), c8 = e % (kBN / 8);
      if (tm * kBM + r >= a.M) break;  // rows are visited in order: the rest lies beyond M too
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < a.world; ++s) {
        // L2 loads: the partials arrived from other GPUs, a line cached in L1 by an earlier call would be stale.
        // (Unrolling the loop to the rank count so that all loads are in flight together, and splitting a tile
        // over 16 CTAs instead of 4 when a rank owns few tiles, both measured slower at 8 GPUs: 22 against 17 us.)
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(base + s * src_stride + static_cast<long long>(e) * 8));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack2<T>(w[i]);
          acc[2 * i] += f.x, acc[2 * i + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack2<T>(acc[0], acc[1]), o.y = pack2<T>(acc[2], acc[3]), o.z = pack2<T>(acc[4], acc[5]), o.w = pack2<T>(acc[6], acc[7]);
      const long long off = static_cast<long long>(tm * kBM + r) * a.out_stride_m + tn * kBN + c8 * 8;
      for (int d = d0; d < d1; ++d) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.out[d]) + off) = o;
    }
    if (!a.one_shot) __threadfence_system();
  }
  if (a.one_shot) return;   // nothing left another rank waits for
  __syncthreads();
  // the finished tile is in every rank's output: every rank's count of delivered tiles moves on.  (After a
  // timeout nothing is counted: the other ranks' final waits then run out too and report it.)
  if (threadIdx.x < a.world && ok) red_add_release_sys(a.done_counters[threadIdx.x], static_cast<uint32_t>(kMaxReduceSplit / a.split));
}

// The reduction through the NVLink switch: every rank left its partial tile in its OWN staging buffer (slot =
// tile) and told the tile's owner; the owner reads the sum of all ranks' copies with multimem.ld_reduce on the
// multicast address of the staging buffers (the switch adds, fp32 accumulation) and stores the finished tile to
// every rank's output with one multimem.st on the multicast address of the outputs.  Each rank sends its partial
// once and receives the result once; the owner moves 1/world of the data instead of all of it twice.
// Measured at 4 GPUs (1024 x 4096 bf16): correct, but 59.4 us for the sum alone against 52.4 us for the
// reduce-scatter + all-gather form over peer stores and 46.8 us for NCCL - each thread has one 16-byte
// multimem.ld_reduce in flight and the round trip through the switch is long; it is therefore only taken when
// asked for (mode 3).
template <typename T>
__global__ void __launch_bounds__(256) oproj_reduce_switch_kernel(const ReduceArgs a, const void* stage_mc, void* out_mc) {
  ptx::grid_launch_dependents();
  __shared__ int sh_ok;
  const int lt = blockIdx.x / a.split, part = blockIdx.x % a.split;
  const int tile = lt * a.world + a.rank;
  if (tile >= a.n_tiles) return;
  if (threadIdx.x == 0) {
    sh_ok = wait_counter(a.tile_counters_local + lt, a.row_target[tile / a.tiles_n], a.wait_limit_ns) ? 1 : 0;
    if (!sh_ok && a.status) atomicOr(a.status, CA_STATUS_TIMEOUT);
  }
  __syncthreads();
  const bool ok = sh_ok != 0;
  if (ok) {
    const int tm = tile / a.tiles_n, tn = tile % a.tiles_n;
    const T* src = reinterpret_cast<const T*>(stage_mc) + static_cast<long long>(tile) * kTileElems;
    const int part_groups = kTileElems / 8 / a.split;
    for (int e = part * part_groups + threadIdx.x; e < (part + 1) * part_groups; e += 256) {
      const int r = e / (kBN / 8), c8 = e % (kBN / 8);
      if (tm * kBM + r >= a.M) break;
      uint4 v;
      if (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(src + static_cast<long long>(e) * 8)
                     : "memory");
      } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(src + static_cast<long long>(e) * 8)
                     : "memory");
      }
      T* dst = reinterpret_cast<T*>(out_mc) + static_cast<long long>(tm * kBM + r) * a.out_stride_m + tn * kBN + c8 * 8;
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                   : "memory");
    }
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x < a.world && ok) red_add_release_sys(a.done_counters[threadIdx.x], static_cast<uint32_t>(kMaxReduceSplit / a.split));
}

__global__ void oproj_wait_kernel(const uint32_t* done_local, uint32_t target, unsigned long long limit_ns, int32_t* status) {
  // no grid-dependency wait either: the counter is the dependency.  Whatever follows on the stream is a plain
  // launch, so it still waits for this kernel and the two before it.
  if (threadIdx.x == 0 && !wait_counter(done_local, target, limit_ns) && status) atomicOr(status, CA_STATUS_TIMEOUT);
}

static int encode_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer, uint64_t stride_bytes,
                     uint32_t box_inner, uint32_t box_outer, const char* what) {
  tensor_map_encode_fn enc = get_tensor_map_encoder();
  if (!enc) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem[2] = {1, 1};
  CUresult res = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)res);
  return CA_OK;
}

}  // namespace oproj
}  // namespace ca

extern "C" {

int ca_oproj_scratch_bytes(int M_max, int N, int world, size_t* stage_bytes, size_t* counter_bytes) {
  using namespace ca;
  using namespace ca::oproj;
  CA_REQUIRE(stage_bytes && counter_bytes, "output pointers are null");
  CA_REQUIRE(M_max > 0 && N > 0 && N % kBN == 0 && world >= 1 && world <= kMaxWorld, "M_max, N (multiple of %d), world (1..%d)", kBN,
             kMaxWorld);
  const long long n_tiles = static_cast<long long>(ceil_div(M_max, kBM)) * (N / kBN);
  const long long per_owner = (n_tiles + world - 1) / world;
  // two-shot: [src][owned tile]; one-shot (sized for up to four ranks): two halves of [src][tile], used by alternate calls
  const long long slots = world <= 4 ? 2 * n_tiles : per_owner;   // up to four ranks may ask for the one-exchange form
  *stage_bytes = world > 1 ? static_cast<size_t>(world) * slots * kTileElems * 2 : 0;
  *counter_bytes = (static_cast<size_t>(n_tiles) + 1) * sizeof(uint32_t);  // per tile slot, then the finished-tile count
  return CA_OK;
}

int ca_oproj_tile_count(int M, int N) {
  using namespace ca::oproj;
  return (M > 0 && N > 0) ? ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN) : 0;
}

int ca_oproj_allreduce(const ca_oproj_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::oproj;
  CA_REQUIRE(p != nullptr, "params is null");
  CA_REQUIRE(p->a, "a must be non-null");
  const bool reduce_only = p->w == nullptr;  // a is the partial [M, N] itself
  CA_REQUIRE(!reduce_only || p->world > 1, "without w there is nothing to do on one rank");
  CA_REQUIRE(p->dtype == CA_DTYPE_BF16 || p->dtype == CA_DTYPE_F16, "dtype must be bf16 or f16");
  CA_REQUIRE(p->M > 0 && p->N > 0 && (reduce_only || p->K > 0), "M, N, K must be positive");
  CA_REQUIRE(p->N % kBN == 0, "N (%d) must be a multiple of %d", p->N, kBN);
  CA_REQUIRE(reduce_only || p->K % kBK == 0, "K (%d) must be a multiple of %d", p->K, kBK);
  CA_REQUIRE(p->a_stride_m % 8 == 0 && (reduce_only || p->w_stride_n % 8 == 0) && p->out_stride_m % 8 == 0,
             "strides must be multiples of 8 elements");
  CA_REQUIRE((reinterpret_cast<uintptr_t>(p->a) | reinterpret_cast<uintptr_t>(p->w)) % 16 == 0, "a and w must be 16-byte aligned");
  CA_REQUIRE(!reduce_only || p->a_stride_m >= p->N, "without w, a is the partial [M, N]: its row stride must cover N");
  CA_REQUIRE(p->world >= 1 && p->world <= kMaxWorld && p->rank >= 0 && p->rank < p->world, "world (1..%d) / rank out of range", kMaxWorld);
  CA_REQUIRE(p->out != nullptr, "out pointer list is null");
  for (int r = 0; r < p->world; ++r) {
    CA_REQUIRE(p->out[r] != nullptr && reinterpret_cast<uintptr_t>(p->out[r]) % 16 == 0, "out[%d] must be a 16-byte aligned pointer", r);
    if (p->world > 1) {
      CA_REQUIRE(p->stage && p->tile_counters && p->done_counters && p->stage[r] && p->tile_counters[r] && p->done_counters[r],
                 "stage, tile_counters and done_counters of rank %d must be given", r);
    }
  }
  CA_REQUIRE(p->world == 1 || p->epoch > 0, "epoch counts calls from 1");
  CA_REQUIRE(ceil_div(p->M, kBM) <= kMaxRowTiles, "M (%d) exceeds %d rows per call", p->M, kMaxRowTiles * kBM);
  CA_REQUIRE(p->mode >= 0 && p->mode <= 3, "mode must be 0 (auto), 1 (two-shot), 2 (one-shot) or 3 (through the switch)");
  const bool have_mc = p->stage_mc != nullptr && p->out_mc != nullptr;
  CA_REQUIRE(p->mode != 3 || (have_mc && p->world > 1), "mode 3 needs the multicast addresses of the staging and output buffers");
  const bool one_shot = p->world > 1 && (p->mode == 2 || (p->mode == 0 && p->world == 2));
  // mode 0 never picks the switch: at 4 GPUs it measured slower than the peer-store forms (see the kernel's comment)
  const bool via_switch = p->world > 1 && p->mode == 3;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  DeviceInfo dev;
  int rc = get_device_info(&dev);
  if (rc != CA_OK) return rc;
  if (dev.cc_major != 10) return fail(CA_ERR_UNSUPPORTED, "this library targets sm_100a; device is sm_%d%d", dev.cc_major, dev.cc_minor);
  const CUtensorMapDataType dt = p->dtype == CA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap a_map, w_map;
  if (!reduce_only) {
    rc = encode_2d(&a_map, dt, p->a, p->K, p->M, static_cast<uint64_t>(p->a_stride_m) * 2, kBK, kBM, "a");
    if (rc != CA_OK) return rc;
    rc = encode_2d(&w_map, dt, p->w, p->K, p->N, static_cast<uint64_t>(p->w_stride_n) * 2, kBK, kBN, "w");
    if (rc != CA_OK) return rc;
  }
  GemmArgs g;
  g.M = p->M, g.N = p->N, g.K = p->K;
  g.tiles_n = p->N / kBN;
  g.n_tiles = ceil_div(p->M, kBM) * g.tiles_n;
  g.world = p->world, g.rank = p->rank;
  g.tiles_per_owner = ceil_div(g.n_tiles, p->world);
  g.one_shot = one_shot ? 1 : 0;
  g.via_switch = via_switch ? 1 : 0;
  g.slot_tiles = one_shot ? g.n_tiles : g.tiles_per_owner;
  g.buf_off_elems = 0;
  if (p->world > 1) {
    const size_t need = via_switch ? static_cast<size_t>(g.n_tiles) * kTileElems * 2
                                   : static_cast<size_t>(p->world) * g.slot_tiles * kTileElems * 2 * (one_shot ? 2 : 1);
    CA_REQUIRE(p->stage_bytes >= need, "staging buffers of %zu bytes are too small for this call (%zu)", p->stage_bytes, need);
    // one-shot: alternate calls use alternate halves, so a rank that is one call ahead never overwrites what a
    // slower rank still reads (it cannot get two calls ahead: its own reduction waits for the slower rank's tiles)
    if (one_shot && (p->epoch & 1u)) g.buf_off_elems = static_cast<long long>(p->stage_bytes / 4 / 8) * 8;
  }
  for (int r = 0; r < kMaxWorld; ++r) {
    g.stage[r] = (p->world > 1 && r < p->world) ? p->stage[r] : nullptr;
    g.tile_counters[r] = (p->world > 1 && r < p->world) ? p->tile_counters[r] : nullptr;
  }
  g.out_local = p->out[p->rank];
  g.out_stride_m = p->out_stride_m;
  g.idesc = ptx::make_idesc_f16(p->dtype == CA_DTYPE_BF16 ? 1u : 0u, kBM, kBN, 0, 0);
  g.wait_limit_ns = p->wait_limit_ns ? p->wait_limit_ns : 2000000000ull;
  g.status = p->status;
  {
    static std::mutex mu;
    static bool done[2][64] = {};
    const int ti = p->dtype == CA_DTYPE_BF16 ? 0 : 1;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[ti][dev.ordinal]) {
      if (ti == 0) {
        CA_CUDA(cudaFuncSetAttribute(oproj_gemm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      } else {
        CA_CUDA(cudaFuncSetAttribute(oproj_gemm_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      }
      done[ti][dev.ordinal] = true;
    }
  }
  const uint32_t phases = p->phases ? p->phases : 7u;
  if ((phases & 1u) && reduce_only) {
    // both 16-bit types move as bits
    launch_kernel(oproj_push_kernel<uint16_t>, dim3(g.n_tiles), dim3(256), 0, stream, static_cast<const uint16_t*>(p->a),
                  static_cast<long long>(p->a_stride_m), g);
    CA_LAUNCH_CHECK("oproj_push_kernel");
  } else if (phases & 1u) {
    if (p->dtype == CA_DTYPE_BF16) {
      launch_kernel(oproj_gemm_kernel<__nv_bfloat16>, dim3(g.n_tiles), dim3(kThreads), kSmemBytes, stream, a_map, w_map, g);
    } else {
      launch_kernel(oproj_gemm_kernel<__half>, dim3(g.n_tiles), dim3(kThreads), kSmemBytes, stream, a_map, w_map, g);
    }
    CA_LAUNCH_CHECK("oproj_gemm_kernel");
  }
  if (p->world == 1) return CA_OK;
  ReduceArgs r;
  r.M = p->M, r.N = p->N, r.tiles_n = g.tiles_n, r.n_tiles = g.n_tiles, r.world = p->world, r.rank = p->rank;
  r.tiles_per_owner = g.tiles_per_owner;
  r.one_shot = g.one_shot, r.slot_tiles = g.slot_tiles, r.buf_off_elems = g.buf_off_elems;
  r.split = 4;   // 4, 8, 16 and 32 all work (a finished part counts kMaxReduceSplit / split); 4 measured best
  for (int tm = 0; tm < kMaxRowTiles; ++tm) {
    const uint32_t calls = (p->row_epochs && tm < ceil_div(p->M, kBM)) ? p->row_epochs[tm] : p->epoch;
    r.row_target[tm] = calls * static_cast<uint32_t>(p->world);
  }
  r.stage_local = p->stage[p->rank];
  r.tile_counters_local = p->tile_counters[p->rank];
  for (int d = 0; d < kMaxWorld; ++d) {
    r.out[d] = d < p->world ? p->out[d] : nullptr;
    r.done_counters[d] = d < p->world ? p->done_counters[d] : nullptr;
  }
  r.out_stride_m = p->out_stride_m;
  r.wait_limit_ns = g.wait_limit_ns;
  r.status = p->status;
  if (phases & 2u) {
    const dim3 grid(g.slot_tiles * r.split);
    const bool bf = p->dtype == CA_DTYPE_BF16;
    if (via_switch) {
      if (bf) launch_kernel_as(true, oproj_reduce_switch_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, r, static_cast<const void*>(p->stage_mc), p->out_mc);
      else launch_kernel_as(true, oproj_reduce_switch_kernel<__half>, grid, dim3(256), 0, stream, r, static_cast<const void*>(p->stage_mc), p->out_mc);
    } else {
      if (bf) launch_kernel_as(true, oproj_reduce_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, r);
      else launch_kernel_as(true, oproj_reduce_kernel<__half>, grid, dim3(256), 0, stream, r);
    }
    CA_LAUNCH_CHECK("oproj_reduce_kernel");
  }
  if ((phases & 4u) && !one_shot) {
    const uint32_t done_tiles = p->done_tiles_total ? p->done_tiles_total : p->epoch * static_cast<uint32_t>(g.n_tiles);
    launch_kernel_as(true, oproj_wait_kernel, dim3(1), dim3(32), 0, stream, static_cast<const uint32_t*>(p->done_counters[p->rank]),
                     done_tiles * static_cast<uint32_t>(kMaxReduceSplit), static_cast<unsigned long long>(g.wait_limit_ns),
                     p->status);
    CA_LAUNCH_CHECK("oproj_wait_kernel");
  }
  return CA_OK;
}

}  // extern "C"
