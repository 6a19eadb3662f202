// Training-free (FlashPrefill) block score on the sm_100a tensor cores.
//
// For q-block i, query head h and key block j the reference's Triton kernel
// (compact_attn/flashprefill_vendor/flashprefill_native_forward.py:98-207) computes
//   S[t, j] = (q_t . meanK_j) * D^-0.5 * log2(e)   over the tokens t of the q-block,
//   max[j] = max_t S,  score[j] = sum_t 2^(S - max[j]),   tokens counted iff P + t >= (j+1)*bs - 1.
// Here the product is taken transposed, S^T = meanK_tile [128 key blocks x D] . Q^T [D x tokens], so
// a key block is a TMEM lane: every thread of the epilogue owns one key block and reduces over its
// own columns (tokens) without any shuffle.  The G query heads of a KV head share the meanK operand:
// one CTA handles (batch, kv head, q-block), loads the q-block's tokens of all G heads once, and
// walks the visible key-block tiles with a 2-stage TMA ring and a double-buffered TMEM accumulator
// (2 x 256 columns), so the MMAs of the next tile overlap the reductions of the current one.
// One warp issues TMA and tcgen05.mma (lane 0); two warpgroups reduce, one per accumulator buffer,
// so every scheduler has two reduction warps to interleave.  A thread takes a head's whole row of
// tokens into registers with one TMEM read, masks it only on the diagonal tiles (-inf entries
// contribute exp2(-inf) = 0 to the sum, so the sum needs no select), and uses packed fp32 pairs
// for the scale and the sum.  Every wait is bounded.
#include "ca_common.cuh"

namespace ca {
namespace fpscore {

constexpr int kThreads = 288;       // 2 x 4 reduction warps + 1 producer warp
constexpr int kProducerWarp = 8;
constexpr int kTileKeys = 128;      // key blocks per tile = UMMA M
constexpr int kD = 128;
constexpr int kHalfBytesK = kTileKeys * 128;  // one [128 key blocks][64 x 16-bit] swizzled half
constexpr int kKTileBytes = 2 * kHalfBytesK;
constexpr int kMaxCols = 256;       // tokens x heads per MMA pass (UMMA N)

struct Args {
  int B, Q, Hq, Hkv, G, Kb, Qb, bs, P;
  int heads_per_pass, passes;
  float sm_scale;  // D^-0.5 * log2(e)
  float* score;    // [B,Qb,Kb,Hq]
  float* mx;
  uint32_t idesc_base;  // instruction descriptor without the N field
  unsigned long long wait_limit_ns;
  int32_t* status;
};

struct Shared {
  uint64_t q_full;
  uint64_t k_full[2];
  uint64_t k_empty[2];
  uint64_t t_full[2];
  uint64_t t_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// max_t S and sum_t 2^((S - max) * scale) over one head's kBs token columns of this thread's key
// block.  Columns outside [c_min, c_max) are not counted; `all_counted` (warp-uniform) skips the mask.
template <int kBs>
__device__ __forceinline__ void reduce_row(uint32_t taddr, float scale, int c_min, int c_max, bool all_counted,
                                           float& m_scaled, float& p_sum) {
  uint32_t v[128];
  ptx::tmem_ld32_row<0>(taddr, v);
  ptx::tmem_ld32_row<32>(taddr + 32, v);
  if (kBs == 128) {
    ptx::tmem_ld32_row<64>(taddr + 64, v);
    ptx::tmem_ld32_row<96>(taddr + 96, v);
  }
  ptx::tc_wait_ld();
  if (!all_counted) {
#pragma unroll
    for (int c = 0; c < kBs; ++c)
      if (c < c_min || c >= c_max) v[c] = 0xff800000u;  // -inf
  }
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int c = 0; c < kBs; c += 8) {
    m0 = fmaxf(m0, fmaxf(__uint_as_float(v[c + 0]), __uint_as_float(v[c + 1])));
    m1 = fmaxf(m1, fmaxf(__uint_as_float(v[c + 2]), __uint_as_float(v[c + 3])));
    m2 = fmaxf(m2, fmaxf(__uint_as_float(v[c + 4]), __uint_as_float(v[c + 5])));
    m3 = fmaxf(m3, fmaxf(__uint_as_float(v[c + 6]), __uint_as_float(v[c + 7])));
  }
  const float m = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
  m_scaled = m * scale;
  const float neg = m == -INFINITY ? 0.f : -m_scaled;
  const float2 sc2 = make_float2(scale, scale), neg2 = make_float2(neg, neg);
  float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
  for (int c = 0; c < kBs; c += 4) {
    float2 x0 = __ffma2_rn(make_float2(__uint_as_float(v[c + 0]), __uint_as_float(v[c + 1])), sc2, neg2);
    float2 x1 = __ffma2_rn(make_float2(__uint_as_float(v[c + 2]), __uint_as_float(v[c + 3])), sc2, neg2);
    x0.x = ptx::ex2(x0.x), x0.y = ptx::ex2(x0.y);
    x1.x = ptx::ex2(x1.x), x1.y = ptx::ex2(x1.y);
    acc0 = __fadd2_rn(acc0, x0);
    acc1 = __fadd2_rn(acc1, x1);
  }
  p_sum = m == -INFINITY ? -INFINITY : (acc0.x + acc0.y) + (acc1.x + acc1.y);
}

__global__ void __launch_bounds__(kThreads, 1)
    fp_score_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map, const Args a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  // layout: K stage 0 | K stage 1 | Q half 0 [G*bs rows][64] | Q half 1 | barriers
  const int q_rows = a.G * a.bs;
  const uint32_t k_smem = smem_base;
  const uint32_t q_smem = smem_base + 2 * kKTileBytes;
  const uint32_t q_half_bytes = static_cast<uint32_t>(q_rows) * 128u;
  Shared* sh = reinterpret_cast<Shared*>(smem_aligned + 2 * kKTileBytes + 2 * q_half_bytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int i = blockIdx.x;                       // q-block
  const int hkv = blockIdx.y, b = blockIdx.z;
  volatile int* abort_flag = &sh->abort_flag;
  const uint64_t limit = a.wait_limit_ns;

  // key blocks this q-block can see: j with (j+1)*bs - 1 <= P + last token of the q-block
  const int t_end = min((i + 1) * a.bs, a.Q);     // one past the q-block's last token
  const long long last_abs = static_cast<long long>(a.P) + t_end - 1;
  int vis_blocks = static_cast<int>((last_abs + 1) / a.bs);
  if (vis_blocks > a.Kb) vis_blocks = a.Kb;
  const int n_tiles = (vis_blocks + kTileKeys - 1) / kTileKeys;
  const int n_work = n_tiles * a.passes;          // (tile, head pass) items, pass fastest

  if (tid == 0) {
    ptx::mbar_init(ptx::smem_u32(&sh->q_full), 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(ptx::smem_u32(&sh->k_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sh->k_empty[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sh->t_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sh->t_empty[s]), 128);
    }
    sh->abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == kProducerWarp) {
    ptx::tmem_alloc(ptx::smem_u32(&sh->tmem_base), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  // invisible key blocks keep the reference's -inf initialisation
  {
    float* sc = a.score + ((static_cast<long long>(b) * a.Qb + i) * a.Kb) * a.Hq + hkv * a.G;
    float* mx = a.mx + ((static_cast<long long>(b) * a.Qb + i) * a.Kb) * a.Hq + hkv * a.G;
    const int first = n_tiles * kTileKeys;
    for (long long e = static_cast<long long>(first) * a.G + tid; e < static_cast<long long>(a.Kb) * a.G; e += kThreads) {
      const long long j = e / a.G, g = e % a.G;
      sc[j * a.Hq + g] = -INFINITY;
      mx[j * a.Hq + g] = -INFINITY;
    }
  }

  bool ok = true;
  if (warp == kProducerWarp) {
    // =============================== TMA + MMA issuer ===============================
    if (lane == 0 && n_work > 0) {
      auto wait = [&](uint64_t* bar, uint32_t parity) {
        if (ok) ok = ptx::mbar_wait_bounded(ptx::smem_u32(bar), parity, abort_flag, limit);
        return ok;
      };
      // the q-block's tokens of all G heads: one box per (head, d-half)
      ptx::mbar_expect_tx(ptx::smem_u32(&sh->q_full), 2u * q_half_bytes);
      for (int g = 0; g < a.G; ++g)
        for (int h = 0; h < 2; ++h)
          ptx::tma_load_4d(q_smem + h * q_half_bytes + g * a.bs * 128, &q_map, ptx::smem_u32(&sh->q_full), h * 64,
                           hkv * a.G + g, i * a.bs, b);
      auto load_k = [&](int tile) {
        const int s = tile & 1;
        if (tile >= 2 && !wait(&sh->k_empty[s], ((tile >> 1) - 1) & 1)) return;
        ptx::mbar_expect_tx(ptx::smem_u32(&sh->k_full[s]), kKTileBytes);
        for (int h = 0; h < 2; ++h)
          ptx::tma_load_4d(k_smem + s * kKTileBytes + h * kHalfBytesK, &k_map, ptx::smem_u32(&sh->k_full[s]), h * 64, hkv,
                           tile * kTileKeys, b);
      };
      load_k(0);
      wait(&sh->q_full, 0);
      const uint64_t k_desc0 = ptx::make_smem_desc_sw128(k_smem, 0, 1024);
      const uint64_t q_desc0 = ptx::make_smem_desc_sw128(q_smem, 0, 1024);
      for (int w = 0; w < n_work && ok; ++w) {
        const int tile = w / a.passes, pass = w % a.passes;
        const int s = tile & 1, buf = w & 1;
        if (pass == 0) {
          if (tile + 1 < n_tiles) load_k(tile + 1);  // prefetch the next key tile
          if (!wait(&sh->k_full[s], (tile >> 1) & 1)) break;
        }
        if (w >= 2 && !wait(&sh->t_empty[buf], ((w >> 1) - 1) & 1)) break;
        ptx::tc_fence_after();
        const int h0 = pass * a.heads_per_pass;
        const int nh = min(a.heads_per_pass, a.G - h0);
        const uint32_t idesc = a.idesc_base | (static_cast<uint32_t>((nh * a.bs) >> 3) << 17);
        const uint64_t kd = k_desc0 + static_cast<uint64_t>(s * (kKTileBytes >> 4));
        const uint64_t qd = q_desc0 + static_cast<uint64_t>((h0 * a.bs * 128) >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // A: key blocks (K-major), B: tokens (K-major); d-half k>>2, 32-byte step inside the swizzled row
          const uint64_t ko = static_cast<uint64_t>(((k >> 2) * kHalfBytesK + (k & 3) * 32) >> 4);
          const uint64_t qo = static_cast<uint64_t>(((k >> 2) * q_half_bytes + (k & 3) * 32) >> 4);
          ptx::mma_ss(tmem + buf * kMaxCols, kd + ko, qd + qo, idesc, k > 0 ? 1u : 0u);
        }
        ptx::tc_commit(ptx::smem_u32(&sh->t_full[buf]));
        if (pass == a.passes - 1) ptx::tc_commit(ptx::smem_u32(&sh->k_empty[s]));
      }
    }
  } else {
    // =============================== reduction over tokens ===============================
    // warpgroup g owns accumulator buffer g and the work items of its parity
    const int wg = warp >> 2;
    const int row = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int c_max = t_end - i * a.bs;  // one past the last real token of the q-block
    for (int w = wg; w < n_work; w += 2) {
      const int tile = w / a.passes, pass = w % a.passes;
      const int buf = wg;
      ok = ptx::mbar_wait_bounded(ptx::smem_u32(&sh->t_full[buf]), (w >> 1) & 1, abort_flag, limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      const int j = tile * kTileKeys + row;  // this thread's key block
      const int h0 = pass * a.heads_per_pass;
      const int nh = min(a.heads_per_pass, a.G - h0);
      // token t of the q-block is counted iff P + t >= (j+1)*bs - 1  <=>  t >= (j+1)*bs - 1 - P
      const long long t_min_ll = static_cast<long long>(j + 1) * a.bs - 1 - a.P - static_cast<long long>(i) * a.bs;
      const int c_min = t_min_ll < 0 ? 0 : (t_min_ll > a.bs ? a.bs : static_cast<int>(t_min_ll));  // first counted column
      const bool all_counted = __all_sync(0xffffffffu, c_min == 0 && c_max == a.bs);
      float res_p[4], res_m[4];
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) {
        if (hh < nh) {  // warp-uniform
          const uint32_t taddr = tmem + lane_base + buf * kMaxCols + hh * a.bs;
          if (a.bs == 64) reduce_row<64>(taddr, a.sm_scale, c_min, c_max, all_counted, res_m[hh], res_p[hh]);
          else reduce_row<128>(taddr, a.sm_scale, c_min, c_max, all_counted, res_m[hh], res_p[hh]);
        }
      }
      // the accumulator buffer is free as soon as its rows are in registers
      ptx::tc_fence_before();
      ptx::mbar_arrive(ptx::smem_u32(&sh->t_empty[buf]));
      if (j < a.Kb) {
        const long long o = ((static_cast<long long>(b) * a.Qb + i) * a.Kb + j) * a.Hq + hkv * a.G + h0;
        if (nh == 4 && (o & 3) == 0) {
          *reinterpret_cast<float4*>(a.score + o) = make_float4(res_p[0], res_p[1], res_p[2], res_p[3]);
          *reinterpret_cast<float4*>(a.mx + o) = make_float4(res_m[0], res_m[1], res_m[2], res_m[3]);
        } else {
#pragma unroll
          for (int hh = 0; hh < 4; ++hh) {
            if (hh < nh) a.score[o + hh] = res_p[hh], a.mx[o + hh] = res_m[hh];
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) {
    if (lane == 0 && sh->abort_flag) {
      // after an expired wait: give the few copies and MMAs that may still be in flight 200 us to
      // land before shared memory and TMEM are released
      const uint64_t t0 = ptx::globaltimer_ns();
      while (ptx::globaltimer_ns() - t0 < 200000ull) {
      }
    }
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && sh->abort_flag && a.status) atomicOr(a.status, CA_STATUS_TIMEOUT);
}

}  // namespace fpscore

// Launches the tensor-core block score; returns CA_ERR_UNSUPPORTED when the shape does not fit it
// (the caller then uses the CUDA-core kernel).
int launch_fp_score_sm100(const ca_flashprefill_score_params* p, cudaStream_t stream) {
  using namespace fpscore;
  const int G = p->Hq / p->Hkv;
  const int bs = p->block_size;
  if (p->D != kD || (bs != 64 && bs != 128) || p->q_dtype != p->k_dtype ||
      (p->q_dtype != CA_DTYPE_BF16 && p->q_dtype != CA_DTYPE_F16))
    return CA_ERR_UNSUPPORTED;
  const size_t smem = 2 * kKTileBytes + 2 * static_cast<size_t>(G) * bs * 128 + 1024 + sizeof(Shared);
  DeviceInfo dev;
  int rc = get_device_info(&dev);
  if (rc != CA_OK) return rc;
  if (dev.cc_major != 10 || smem > static_cast<size_t>(dev.smem_optin)) return CA_ERR_UNSUPPORTED;
  if ((p->q_stride_b | p->q_stride_t | p->q_stride_h | p->k_stride_b | p->k_stride_blk | p->k_stride_h) % 8 != 0 ||
      (reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->mean_k)) % 16 != 0)
    return CA_ERR_UNSUPPORTED;
  tensor_map_encode_fn enc = get_tensor_map_encoder();
  if (!enc) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const CUtensorMapDataType dt = p->q_dtype == CA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint32_t ones[4] = {1, 1, 1, 1};
  CUtensorMap q_map, k_map;
  {
    // (d, head, token, batch); the box is one head's bs tokens x 64 channels
    const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)p->Hq, (cuuint64_t)p->Q, (cuuint64_t)p->B};
    const cuuint64_t strides[3] = {(cuuint64_t)p->q_stride_h * 2, (cuuint64_t)p->q_stride_t * 2, (cuuint64_t)p->q_stride_b * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)bs, 1};
    CUresult res = enc(&q_map, dt, 4, const_cast<void*>(p->q), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled(q) failed with CUresult %d", (int)res);
  }
  {
    // (d, kv head, key block, batch); the box is 128 key blocks x 64 channels of one head
    const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)p->Hkv, (cuuint64_t)p->Kb, (cuuint64_t)p->B};
    const cuuint64_t strides[3] = {(cuuint64_t)p->k_stride_h * 2, (cuuint64_t)p->k_stride_blk * 2, (cuuint64_t)p->k_stride_b * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)kTileKeys, 1};
    CUresult res = enc(&k_map, dt, 4, const_cast<void*>(p->mean_k), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled(mean_k) failed with CUresult %d", (int)res);
  }
  Args a;
  a.B = p->B, a.Q = p->Q, a.Hq = p->Hq, a.Hkv = p->Hkv, a.G = G, a.Kb = p->Kb, a.bs = bs;
  a.Qb = ceil_div(p->Q, bs);
  a.P = p->kv_len - p->Q;
  a.heads_per_pass = kMaxCols / bs;
  a.passes = ceil_div(G, a.heads_per_pass);
  a.sm_scale = (1.0f / sqrtf(static_cast<float>(kD))) * 1.4426950408889634f;
  a.score = p->score_raw, a.mx = p->max_raw;
  a.idesc_base = ptx::make_idesc_f16(p->q_dtype == CA_DTYPE_BF16 ? 1u : 0u, kTileKeys, 0, 0, 0);
  a.wait_limit_ns = 2000000000ull;
  a.status = nullptr;
  CA_CUDA(cudaFuncSetAttribute(fp_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  launch_kernel(fp_score_kernel, dim3(a.Qb, p->Hkv, p->B), dim3(kThreads), smem, stream, q_map, k_map, a);
  CA_LAUNCH_CHECK("fp_score_kernel");
  return CA_OK;
}

}  // namespace ca
