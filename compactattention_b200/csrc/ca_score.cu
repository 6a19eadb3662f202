// Block scoring for the two selectors.
//   learned gate (SeerAttention AttnGate): block pooling (max / min / avg) of the chunk's Q and K,
//     per-head linear projection, block RoPE, append to the gate's K-block cache, then
//     logits = q_block . k_block * scale for every cached key block;
//   training-free (FlashPrefill): per-block mean of K, per-token Q x mean-K block score with
//     per-block max / sum-exp2, and the row normalisation.
// All of it is small, HBM/launch-bound work on CUDA cores: 128-bit loads, fp32 accumulation,
// warp-shuffle reductions.
#include "ca_common.cuh"

namespace ca {
namespace score {

__device__ __forceinline__ float load_elem(const void* base, long long off, int dtype) {
  if (dtype == CA_DTYPE_F32) return reinterpret_cast<const float*>(base)[off];
  if (dtype == CA_DTYPE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off]);
  return __half2float(reinterpret_cast<const __half*>(base)[off]);
}
__device__ __forceinline__ void store_elem(void* base, long long off, int dtype, float v) {
  if (dtype == CA_DTYPE_F32) reinterpret_cast<float*>(base)[off] = v;
  else if (dtype == CA_DTYPE_BF16) reinterpret_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(base)[off] = __float2half_rn(v);
}
// 8 consecutive elements starting at off (16-byte aligned for 16-bit types, 32-byte for f32).
__device__ __forceinline__ void load8(const void* base, long long off, int dtype, float (&v)[8]) {
  if (dtype == CA_DTYPE_F32) {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + off);
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
}

// Compile-time-typed variant: a batch of these unrolls into straight-line loads whose latencies overlap.
template <int DT>
__device__ __forceinline__ void load8_t(const void* base, long long off, float (&v)[8]) {
  if (DT == CA_DTYPE_F32) {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + off);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (DT == CA_DTYPE_BF16) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        v[2 * i] = __low2float(h);
        v[2 * i + 1] = __high2float(h);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Block pooling: x [B,L,H,D] -> out [B, blocks, H, nk*D] at block offset, channel order max|min|avg
// ------------------------------------------------------------------------------------------
struct PoolArgs {
  const void* x;
  long long x_b, x_t, x_h;
  int x_dtype;
  void* out;
  long long o_b, o_blk, o_h;
  int o_dtype;
  int out_block_offset;
  int B, L, H, D, bs;
  int kinds;  // bit 0 max, bit 1 min, bit 2 avg
};

constexpr int kPoolThreads = 128;

__global__ void __launch_bounds__(kPoolThreads) pool_blocks_kernel(const PoolArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  // thread = (token phase, 8-dim group); D/8 groups, kPoolThreads/(D/8) phases
  extern __shared__ float pool_smem[];  // [3][phases][D]
  const int groups = a.D / 8;
  const int phases = kPoolThreads / groups;
  const int grp = threadIdx.x % groups, ph = threadIdx.x / groups;
  const int blk = blockIdx.x;
  const int h = blockIdx.y % a.H, b = blockIdx.y / a.H;
  const int t0 = blk * a.bs;
  const int t1 = min(t0 + a.bs, a.L);
  float mx[8], mn[8], sm[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mx[i] = -INFINITY, mn[i] = INFINITY, sm[i] = 0.f;
  if (ph < phases) {
    for (int t = t0 + ph; t < t1; t += phases) {
      float v[8];
      load8(a.x, b * a.x_b + t * a.x_t + h * a.x_h + grp * 8, a.x_dtype, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx[i] = fmaxf(mx[i], v[i]), mn[i] = fminf(mn[i], v[i]), sm[i] += v[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      pool_smem[(0 * phases + ph) * a.D + grp * 8 + i] = mx[i];
      pool_smem[(1 * phases + ph) * a.D + grp * 8 + i] = mn[i];
      pool_smem[(2 * phases + ph) * a.D + grp * 8 + i] = sm[i];
    }
  }
  __syncthreads();
  const float inv_cnt = 1.0f / static_cast<float>(t1 - t0);
  const long long obase = b * a.o_b + static_cast<long long>(a.out_block_offset + blk) * a.o_blk + h * a.o_h;
  for (int d = threadIdx.x; d < a.D; d += kPoolThreads) {
    float rmx = -INFINITY, rmn = INFINITY, rsm = 0.f;
    for (int p = 0; p < phases; ++p) {
      rmx = fmaxf(rmx, pool_smem[(0 * phases + p) * a.D + d]);
      rmn = fminf(rmn, pool_smem[(1 * phases + p) * a.D + d]);
      rsm += pool_smem[(2 * phases + p) * a.D + d];
    }
    int c = 0;
    if (a.kinds & 1) store_elem(a.out, obase + (c++) * a.D + d, a.o_dtype, rmx);
    if (a.kinds & 2) store_elem(a.out, obase + (c++) * a.D + d, a.o_dtype, rmn);
    if (a.kinds & 4) store_elem(a.out, obase + (c++) * a.D + d, a.o_dtype, rsm * inv_cnt);
  }
}

// ------------------------------------------------------------------------------------------
// Per-head linear + block RoPE + append: x [B,nb,Hin,Cin] (f32) * W [Hout,Cin,Cout] -> out
// ------------------------------------------------------------------------------------------
struct ProjArgs {
  const float* x;  // pooled blocks, contiguous [B, nb, Hin, Cin]
  const void* w;   // [Hout, Cin, Cout] contiguous or NULL (identity, Cin == Cout, Hout == Hin)
  int w_dtype;
  const float* cos;  // optional [Bc, nb, Cout] (Bc = 1 or B), half-rotation tables; NULL = no RoPE
  const float* sin;
  int rope_batch;    // Bc
  void* out;
  long long o_b, o_blk, o_h;
  int o_dtype;
  int out_block_offset;
  int B, nb, Hin, Hout, Cin, Cout;
};

constexpr int kProjBlocks = 8;  // blocks handled per CTA
constexpr int kProjSlices = 4;  // the Cin reduction is split over this many thread slices

// blockDim = (min(Cout,128), kProjSlices).  Weight loads are issued eight at a time so their
// latencies overlap; slice partial sums meet in shared memory.
__global__ void __launch_bounds__(128 * kProjSlices) proj_rope_kernel(const ProjArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ float proj_smem[];  // x tile [kProjBlocks][Cin], partials [kProjSlices][kProjBlocks][Cout]
  float* xs = proj_smem;
  float* ys = proj_smem + kProjBlocks * a.Cin;
  const int tid = threadIdx.y * blockDim.x + threadIdx.x;
  const int nthreads = blockDim.x * blockDim.y;
  const int blk0 = blockIdx.x * kProjBlocks;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hin = h / (a.Hout / a.Hin);  // kv head repeated up to the weight's head count
  const int nblk = min(kProjBlocks, a.nb - blk0);
  for (int e = tid; e < kProjBlocks * a.Cin; e += nthreads) {
    const int r = e / a.Cin, c = e % a.Cin;
    xs[e] = r < nblk ? a.x[((static_cast<long long>(b) * a.nb + blk0 + r) * a.Hin + hin) * a.Cin + c] : 0.f;
  }
  __syncthreads();
  const int slice = threadIdx.y;
  const int c_per = (a.Cin + kProjSlices - 1) / kProjSlices;
  const int c_lo = slice * c_per, c_hi = min(a.Cin, c_lo + c_per);
  for (int o = threadIdx.x; o < a.Cout; o += blockDim.x) {
    float acc[kProjBlocks];
#pragma unroll
    for (int r = 0; r < kProjBlocks; ++r) acc[r] = 0.f;
    if (a.w) {
      const long long wbase = static_cast<long long>(h) * a.Cin * a.Cout + o;
      for (int c0 = c_lo; c0 < c_hi; c0 += 8) {
        float w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = (c0 + u < c_hi) ? load_elem(a.w, wbase + static_cast<long long>(c0 + u) * a.Cout, a.w_dtype) : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int c = min(c0 + u, a.Cin - 1);
#pragma unroll
          for (int r = 0; r < kProjBlocks; ++r) acc[r] = fmaf(xs[r * a.Cin + c], w[u], acc[r]);
        }
      }
    } else if (slice == 0) {
#pragma unroll
      for (int r = 0; r < kProjBlocks; ++r) acc[r] = xs[r * a.Cin + o];
    }
#pragma unroll
    for (int r = 0; r < kProjBlocks; ++r) ys[(slice * kProjBlocks + r) * a.Cout + o] = acc[r];
  }
  __syncthreads();
  // fold the slices into slice 0
  for (int e = tid; e < kProjBlocks * a.Cout; e += nthreads) {
    float y = ys[e];
    for (int sidx = 1; sidx < kProjSlices; ++sidx) y += ys[sidx * kProjBlocks * a.Cout + e];
    ys[e] = y;
  }
  __syncthreads();
  const int half = a.Cout / 2;
  for (int e = tid; e < nblk * a.Cout; e += nthreads) {
    const int r = e / a.Cout, o = e % a.Cout;
    float y = ys[r * a.Cout + o];
    if (a.cos) {
      const long long ro = ((a.rope_batch > 1 ? static_cast<long long>(b) : 0) * a.nb + blk0 + r) * a.Cout + o;
      const float rot = o < half ? -ys[r * a.Cout + o + half] : ys[r * a.Cout + o - half];
      y = y * a.cos[ro] + rot * a.sin[ro];
    }
    store_elem(a.out, b * a.o_b + static_cast<long long>(a.out_block_offset + blk0 + r) * a.o_blk + h * a.o_h + o,
               a.o_dtype, y);
  }
}

// ------------------------------------------------------------------------------------------
// Gate logits: q_blocks [B,Qb,Hq,C] . k_blocks [B,Kb,Hk,C] * scale -> [B,Hq,Qb,Kb] f32
// ------------------------------------------------------------------------------------------
struct GateArgs {
  const void* q;
  long long q_b, q_blk, q_h;
  int q_dtype;
  const void* k;
  long long k_b, k_blk, k_h;
  int k_dtype;
  float* out;  // [B,Hq,Qb,Kb] contiguous
  int B, Hq, Hk, Qb, Kb, Pb, C;
  float scale;
  float masked_value;  // written where j > Pb + i (the reference fills finfo.min)
};

constexpr int kGateThreads = 128;
constexpr int kGateRows = 16;  // q-blocks accumulated per pass

// Widen 8 packed 16-bit elements (KDT: CA_DTYPE_BF16 / CA_DTYPE_F16) to f32.
template <int KDT>
__device__ __forceinline__ void widen8(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (KDT == CA_DTYPE_BF16) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      v[2 * i] = __low2float(h);
      v[2 * i + 1] = __high2float(h);
    }
  }
}

// Thread = key block j; the chunk's q-block rows sit in shared memory (broadcast reads).  The key
// block's channels are fetched 64 at a time as straight-line 128-bit loads so their latencies
// overlap, then widened to f32.
template <int KDT>
__global__ void __launch_bounds__(kGateThreads) gate_scores_kernel(const GateArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ float gate_smem[];  // q rows [Qb][C]
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hk);
  for (int e = threadIdx.x * 8; e < a.Qb * a.C; e += kGateThreads * 8) {
    const int i = e / a.C, c = e % a.C;
    float v[8];
    load8(a.q, b * a.q_b + i * a.q_blk + h * a.q_h + c, a.q_dtype, v);
#pragma unroll
    for (int u = 0; u < 8; ++u) gate_smem[e + u] = v[u];
  }
  __syncthreads();
  const int j = blockIdx.x * kGateThreads + threadIdx.x;
  if (j >= a.Kb) return;
  const long long kbase = b * a.k_b + static_cast<long long>(j) * a.k_blk + hk * a.k_h;
  float* orow = a.out + ((static_cast<long long>(b) * a.Hq + h) * a.Qb) * a.Kb + j;
  for (int i0 = 0; i0 < a.Qb; i0 += kGateRows) {
    float acc[kGateRows];
#pragma unroll
    for (int r = 0; r < kGateRows; ++r) acc[r] = 0.f;
    const int rows = min(kGateRows, a.Qb - i0);
    for (int c0 = 0; c0 < a.C; c0 += 64) {
      float kv[8][8];
      if (KDT == CA_DTYPE_F32) {
        const float* kp = reinterpret_cast<const float*>(a.k) + kbase + c0;
        float4 raw[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) raw[u] = (c0 + u * 4 < a.C) ? *reinterpret_cast<const float4*>(kp + u * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          kv[u][0] = raw[2 * u].x, kv[u][1] = raw[2 * u].y, kv[u][2] = raw[2 * u].z, kv[u][3] = raw[2 * u].w;
          kv[u][4] = raw[2 * u + 1].x, kv[u][5] = raw[2 * u + 1].y, kv[u][6] = raw[2 * u + 1].z, kv[u][7] = raw[2 * u + 1].w;
        }
      } else {
        const uint16_t* kp = reinterpret_cast<const uint16_t*>(a.k) + kbase + c0;
        uint4 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) raw[u] = (c0 + u * 8 < a.C) ? *reinterpret_cast<const uint4*>(kp + u * 8) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < 8; ++u) widen8<KDT>(raw[u], kv[u]);
      }
      const int cn = min(64, a.C - c0);
#pragma unroll
      for (int r = 0; r < kGateRows; ++r) {
        if (r < rows) {
          const float* qrow = &gate_smem[(i0 + r) * a.C + c0];
          float sum = acc[r];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (u * 8 < cn) {
              const float4 q0 = *reinterpret_cast<const float4*>(qrow + u * 8);
              const float4 q1 = *reinterpret_cast<const float4*>(qrow + u * 8 + 4);
              sum += q0.x * kv[u][0] + q0.y * kv[u][1] + q0.z * kv[u][2] + q0.w * kv[u][3] + q1.x * kv[u][4] +
                     q1.y * kv[u][5] + q1.z * kv[u][6] + q1.w * kv[u][7];
            }
          }
          acc[r] = sum;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kGateRows; ++r) {
      const int i = i0 + r;
      if (i < a.Qb) orow[static_cast<long long>(i) * a.Kb] = (j <= a.Pb + i) ? acc[r] * a.scale : a.masked_value;
    }
  }
}

// Lean variant for C % 32 == 0: a thread owns two key blocks (j and j + 128) so every broadcast
// read of a q value from shared memory feeds two FMAs; q rows are zero-padded to a multiple of 16
// so the inner loops carry no predicates.
template <int KDT>
__device__ __forceinline__ void load_k32(const void* base, long long off, float (&v)[32]) {
  if (KDT == CA_DTYPE_F32) {
    const float* kp = reinterpret_cast<const float*>(base) + off;
    float4 raw[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const float4*>(kp + u * 4);
#pragma unroll
    for (int u = 0; u < 8; ++u) v[4 * u] = raw[u].x, v[4 * u + 1] = raw[u].y, v[4 * u + 2] = raw[u].z, v[4 * u + 3] = raw[u].w;
  } else {
    const uint16_t* kp = reinterpret_cast<const uint16_t*>(base) + off;
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) raw[u] = *reinterpret_cast<const uint4*>(kp + u * 8);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float t[8];
      widen8<KDT>(raw[u], t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[8 * u + i] = t[i];
    }
  }
}

template <int KDT>
__global__ void __launch_bounds__(kGateThreads) gate_scores2_kernel(const GateArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ float gate_smem[];  // q rows [ceil16(Qb)][C], zero padded
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hk);
  const int q_pad = ((a.Qb + kGateRows - 1) / kGateRows) * kGateRows;
  for (int e = threadIdx.x * 8; e < q_pad * a.C; e += kGateThreads * 8) {
    const int i = e / a.C, c = e % a.C;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (i < a.Qb) load8(a.q, b * a.q_b + i * a.q_blk + h * a.q_h + c, a.q_dtype, v);
#pragma unroll
    for (int u = 0; u < 8; ++u) gate_smem[e + u] = v[u];
  }
  __syncthreads();
  const int j0 = blockIdx.x * (2 * kGateThreads) + threadIdx.x;
  const int j1 = j0 + kGateThreads;
  if (j0 >= a.Kb) return;
  const int j1c = j1 < a.Kb ? j1 : a.Kb - 1;  // clamped address; its result is not stored
  const long long k0 = b * a.k_b + static_cast<long long>(j0) * a.k_blk + hk * a.k_h;
  const long long k1 = b * a.k_b + static_cast<long long>(j1c) * a.k_blk + hk * a.k_h;
  float* obase = a.out + ((static_cast<long long>(b) * a.Hq + h) * a.Qb) * a.Kb;
  for (int i0 = 0; i0 < a.Qb; i0 += kGateRows) {
    float acc0[kGateRows], acc1[kGateRows];
#pragma unroll
    for (int r = 0; r < kGateRows; ++r) acc0[r] = 0.f, acc1[r] = 0.f;
    for (int c0 = 0; c0 < a.C; c0 += 32) {
      float kv0[32], kv1[32];
      load_k32<KDT>(a.k, k0 + c0, kv0);
      load_k32<KDT>(a.k, k1 + c0, kv1);
#pragma unroll
      for (int r = 0; r < kGateRows; ++r) {
        const float* qrow = &gate_smem[(i0 + r) * a.C + c0];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float4 q4 = *reinterpret_cast<const float4*>(qrow + u * 4);
          acc0[r] = fmaf(q4.x, kv0[4 * u], acc0[r]);
          acc1[r] = fmaf(q4.x, kv1[4 * u], acc1[r]);
          acc0[r] = fmaf(q4.y, kv0[4 * u + 1], acc0[r]);
          acc1[r] = fmaf(q4.y, kv1[4 * u + 1], acc1[r]);
          acc0[r] = fmaf(q4.z, kv0[4 * u + 2], acc0[r]);
          acc1[r] = fmaf(q4.z, kv1[4 * u + 2], acc1[r]);
          acc0[r] = fmaf(q4.w, kv0[4 * u + 3], acc0[r]);
          acc1[r] = fmaf(q4.w, kv1[4 * u + 3], acc1[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kGateRows; ++r) {
      const int i = i0 + r;
      if (i < a.Qb) {
        obase[static_cast<long long>(i) * a.Kb + j0] = (j0 <= a.Pb + i) ? acc0[r] * a.scale : a.masked_value;
        if (j1 < a.Kb) obase[static_cast<long long>(i) * a.Kb + j1] = (j1 <= a.Pb + i) ? acc1[r] * a.scale : a.masked_value;
      }
    }
  }
}

// Variant for 16-bit key blocks with C == 128 and Qb <= 16 (the learned gate's usual shape): a thread
// owns ONE key block and fetches all of its 128 channels as sixteen 128-bit loads issued back to back,
// so the row costs one memory latency instead of four; half as much work per thread gives twice the
// CTAs of the two-blocks-per-thread form (latency-bound: 20.4 us -> see profiles/ for the figure).
template <int KDT>
__global__ void __launch_bounds__(kGateThreads) gate_scores3_kernel(const GateArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ float gate_smem[];  // q rows [16][128], zero padded
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hk);
  const int j = blockIdx.x * kGateThreads + threadIdx.x;
  const int jc = j < a.Kb ? j : a.Kb - 1;
  // the key block's loads go out first; the q rows are staged while they are in flight
  const uint16_t* kp = reinterpret_cast<const uint16_t*>(a.k) + b * a.k_b + static_cast<long long>(jc) * a.k_blk + hk * a.k_h;
  uint4 raw[16];
#pragma unroll
  for (int u = 0; u < 16; ++u) raw[u] = __ldg(reinterpret_cast<const uint4*>(kp + u * 8));
  for (int e = threadIdx.x * 8; e < kGateRows * 128; e += kGateThreads * 8) {
    const int i = e / 128, c = e % 128;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (i < a.Qb) load8(a.q, b * a.q_b + i * a.q_blk + h * a.q_h + c, a.q_dtype, v);
#pragma unroll
    for (int u = 0; u < 8; ++u) gate_smem[e + u] = v[u];
  }
  __syncthreads();
  if (j >= a.Kb) return;
  float acc[kGateRows];
#pragma unroll
  for (int r = 0; r < kGateRows; ++r) acc[r] = 0.f;
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    float kv[8];
    widen8<KDT>(raw[u], kv);
#pragma unroll
    for (int r = 0; r < kGateRows; ++r) {
      const float4 q0 = *reinterpret_cast<const float4*>(&gate_smem[r * 128 + u * 8]);
      const float4 q1 = *reinterpret_cast<const float4*>(&gate_smem[r * 128 + u * 8 + 4]);
      acc[r] = fmaf(q0.x, kv[0], acc[r]);
      acc[r] = fmaf(q0.y, kv[1], acc[r]);
      acc[r] = fmaf(q0.z, kv[2], acc[r]);
      acc[r] = fmaf(q0.w, kv[3], acc[r]);
      acc[r] = fmaf(q1.x, kv[4], acc[r]);
      acc[r] = fmaf(q1.y, kv[5], acc[r]);
      acc[r] = fmaf(q1.z, kv[6], acc[r]);
      acc[r] = fmaf(q1.w, kv[7], acc[r]);
    }
  }
  float* obase = a.out + ((static_cast<long long>(b) * a.Hq + h) * a.Qb) * a.Kb;
#pragma unroll
  for (int r = 0; r < kGateRows; ++r) {
    if (r < a.Qb) obase[static_cast<long long>(r) * a.Kb + j] = (j <= a.Pb + r) ? acc[r] * a.scale : a.masked_value;
  }
}

// ------------------------------------------------------------------------------------------
// FlashPrefill block score: for q-block i, head h, key block j:
//   S[t,j] = (q_t . meanK_j) * D^-0.5 * log2e over tokens t of the q-block with P + t >= (j+1)*bs - 1
//   max[i,j,h] = max_t S, score[i,j,h] = sum_t 2^(S - max); -inf where no token qualifies.
// ------------------------------------------------------------------------------------------
struct FpScoreArgs {
  const void* q;  // [B,Q,Hq,D]
  long long q_b, q_t, q_h;
  int q_dtype;
  const void* mk;  // mean-K [B,Kb,Hkv,D]
  long long k_b, k_blk, k_h;
  int k_dtype;
  float* score;  // [B,Qb,Kb,Hq]
  float* mx;     // [B,Qb,Kb,Hq]
  int B, Q, Hq, Hkv, D, Kb, Qb, bs, P;
  float sm_scale;  // D^-0.5 * log2e
};

constexpr int kFpThreads = 256;
constexpr int kFpTile = 64;  // tokens per pass and key blocks per CTA

__global__ void __launch_bounds__(kFpThreads) flashprefill_score_kernel(const FpScoreArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  // shared: key tile [64][D+1], query tile [64][D+1], S tile [64][65]
  extern __shared__ float fp_smem[];
  const int ld = a.D + 1;
  float* ks = fp_smem;
  float* qs = ks + kFpTile * ld;
  float* ss = qs + kFpTile * ld;
  const int jt = blockIdx.x, i = blockIdx.y;
  const int h = blockIdx.z % a.Hq, b = blockIdx.z / a.Hq;
  const int hkv = h / (a.Hq / a.Hkv);
  const int j0 = jt * kFpTile;
  float* sc_out = a.score + ((static_cast<long long>(b) * a.Qb + i) * a.Kb) * a.Hq + h;
  float* mx_out = a.mx + ((static_cast<long long>(b) * a.Qb + i) * a.Kb) * a.Hq + h;
  // key blocks whose last token lies beyond the q-block's last token are never visible
  const int q_last_abs = a.P + min((i + 1) * a.bs, a.Q) - 1;
  if (static_cast<long long>(j0 + 1) * a.bs - 1 > q_last_abs) {
    for (int jj = threadIdx.x; jj < kFpTile && j0 + jj < a.Kb; jj += kFpThreads) {
      sc_out[static_cast<long long>(j0 + jj) * a.Hq] = -INFINITY;
      mx_out[static_cast<long long>(j0 + jj) * a.Hq] = -INFINITY;
    }
    return;
  }
  for (int e = threadIdx.x; e < kFpTile * a.D; e += kFpThreads) {
    const int r = e / a.D, c = e % a.D;
    ks[r * ld + c] = (j0 + r < a.Kb) ? load_elem(a.mk, b * a.k_b + static_cast<long long>(j0 + r) * a.k_blk + hkv * a.k_h + c, a.k_dtype) : 0.f;
  }
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16x16 threads, 4x4 outputs each
  float run_m = -INFINITY, run_p = 0.f;  // threads 0..63 own key block j0 + threadIdx.x
  for (int t0 = i * a.bs; t0 < min((i + 1) * a.bs, a.Q); t0 += kFpTile) {
    __syncthreads();
    for (int e = threadIdx.x; e < kFpTile * a.D; e += kFpThreads) {
      const int r = e / a.D, c = e % a.D;
      qs[r * ld + c] = (t0 + r < a.Q && t0 + r < (i + 1) * a.bs)
                           ? load_elem(a.q, b * a.q_b + static_cast<long long>(t0 + r) * a.q_t + h * a.q_h + c, a.q_dtype)
                           : 0.f;
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
    for (int d = 0; d < a.D; ++d) {
      float qv[4], kv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) qv[r] = qs[(ty * 4 + r) * ld + d];
#pragma unroll
      for (int c = 0; c < 4; ++c) kv[c] = ks[(tx * 4 + c) * ld + d];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(qv[r], kv[c], acc[r][c]);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int t = t0 + ty * 4 + r, j = j0 + tx * 4 + c;
        const bool vis = t < a.Q && t < (i + 1) * a.bs && j < a.Kb &&
                         (static_cast<long long>(a.P) + t >= static_cast<long long>(j + 1) * a.bs - 1);
        ss[(ty * 4 + r) * (kFpTile + 1) + tx * 4 + c] = vis ? acc[r][c] * a.sm_scale : -INFINITY;
      }
    __syncthreads();
    if (threadIdx.x < kFpTile) {
      float m = run_m;
      for (int r = 0; r < kFpTile; ++r) m = fmaxf(m, ss[r * (kFpTile + 1) + threadIdx.x]);
      if (m != -INFINITY) {
        float p = run_p * exp2f(run_m - m);
        for (int r = 0; r < kFpTile; ++r) {
          const float s = ss[r * (kFpTile + 1) + threadIdx.x];
          p += s == -INFINITY ? 0.f : exp2f(s - m);
        }
        run_m = m, run_p = p;
      }
    }
  }
  if (threadIdx.x < kFpTile && j0 + threadIdx.x < a.Kb) {
    const long long o = static_cast<long long>(j0 + threadIdx.x) * a.Hq;
    sc_out[o] = run_m == -INFINITY ? -INFINITY : run_p;
    mx_out[o] = run_m;
  }
}

// normalize_scores: per (b, i, h) over key blocks j:
//   w_j = 2^(max_j - max_j' max), out_j = score_j * w_j / (sum_j score_j * w_j + 1e-9); 0 where max = -inf.
__global__ void __launch_bounds__(256) flashprefill_normalize_kernel(const float* score, const float* mx, float* out,
                                                                     int Kb, int Hq) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  // one CTA per (b, i); thread -> head tid % Hq, key phase tid / Hq
  extern __shared__ float nz_smem[];  // [phases][Hq]
  const long long base = static_cast<long long>(blockIdx.x) * Kb * Hq;
  const int h = threadIdx.x % Hq, ph = threadIdx.x / Hq;
  const int phases = blockDim.x / Hq;
  float m = -INFINITY;
  if (ph < phases)
    for (int j = ph; j < Kb; j += phases) m = fmaxf(m, mx[base + static_cast<long long>(j) * Hq + h]);
  if (ph < phases) nz_smem[ph * Hq + h] = m;
  __syncthreads();
  m = -INFINITY;
  for (int p = 0; p < phases; ++p) m = fmaxf(m, nz_smem[p * Hq + h]);
  __syncthreads();
  float sum = 0.f;
  if (ph < phases)
    for (int j = ph; j < Kb; j += phases) {
      const long long o = base + static_cast<long long>(j) * Hq + h;
      const float mj = mx[o];
      sum += mj == -INFINITY ? 0.f : score[o] * exp2f(mj - m);
    }
  if (ph < phases) nz_smem[ph * Hq + h] = sum;
  __syncthreads();
  sum = 0.f;
  for (int p = 0; p < phases; ++p) sum += nz_smem[p * Hq + h];
  const float inv = 1.0f / (sum + 1e-9f);
  if (ph < phases)
    for (int j = ph; j < Kb; j += phases) {
      const long long o = base + static_cast<long long>(j) * Hq + h;
      const float mj = mx[o];
      out[o] = mj == -INFINITY ? 0.f : score[o] * exp2f(mj - m) * inv;
    }
}

// The same normalisation with enough CTAs to fill the GPU: one CTA per (b, i, group of 4 query
// heads), thread = key-block phase, the 4 heads of a key block move as one 16-byte vector.
// (The one-CTA-per-(b, i) form above runs 16 CTAs for a 1024-token chunk and took longer than the
// tensor-core score kernel it follows.)
__global__ void __launch_bounds__(256) flashprefill_normalize4_kernel(const float* score, const float* mx, float* out,
                                                                      int Kb, int Hq) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  __shared__ float4 red[8];
  const long long base = static_cast<long long>(blockIdx.x) * Kb * Hq + blockIdx.y * 4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto block_reduce = [&](float4 v, bool is_max) -> float4 {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float4 w;
      w.x = __shfl_xor_sync(0xffffffffu, v.x, o), w.y = __shfl_xor_sync(0xffffffffu, v.y, o);
      w.z = __shfl_xor_sync(0xffffffffu, v.z, o), w.w = __shfl_xor_sync(0xffffffffu, v.w, o);
      if (is_max) v = make_float4(fmaxf(v.x, w.x), fmaxf(v.y, w.y), fmaxf(v.z, w.z), fmaxf(v.w, w.w));
      else v = make_float4(v.x + w.x, v.y + w.y, v.z + w.z, v.w + w.w);
    }
    __syncthreads();  // red is reused
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float4 r = red[0];
    for (int w = 1; w < 8; ++w) {
      const float4 t = red[w];
      if (is_max) r = make_float4(fmaxf(r.x, t.x), fmaxf(r.y, t.y), fmaxf(r.z, t.z), fmaxf(r.w, t.w));
      else r = make_float4(r.x + t.x, r.y + t.y, r.z + t.z, r.w + t.w);
    }
    return r;
  };
  float4 m = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
  for (int j = tid; j < Kb; j += 256) {
    const float4 v = *reinterpret_cast<const float4*>(mx + base + static_cast<long long>(j) * Hq);
    m = make_float4(fmaxf(m.x, v.x), fmaxf(m.y, v.y), fmaxf(m.z, v.z), fmaxf(m.w, v.w));
  }
  m = block_reduce(m, true);
  auto weigh = [](float sc, float mj, float mm) { return mj == -INFINITY ? 0.f : sc * exp2f(mj - mm); };
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = tid; j < Kb; j += 256) {
    const long long o = base + static_cast<long long>(j) * Hq;
    const float4 mj = *reinterpret_cast<const float4*>(mx + o);
    const float4 sc = *reinterpret_cast<const float4*>(score + o);
    sum.x += weigh(sc.x, mj.x, m.x), sum.y += weigh(sc.y, mj.y, m.y);
    sum.z += weigh(sc.z, mj.z, m.z), sum.w += weigh(sc.w, mj.w, m.w);
  }
  sum = block_reduce(sum, false);
  const float4 inv = make_float4(1.0f / (sum.x + 1e-9f), 1.0f / (sum.y + 1e-9f), 1.0f / (sum.z + 1e-9f), 1.0f / (sum.w + 1e-9f));
  for (int j = tid; j < Kb; j += 256) {
    const long long o = base + static_cast<long long>(j) * Hq;
    const float4 mj = *reinterpret_cast<const float4*>(mx + o);
    const float4 sc = *reinterpret_cast<const float4*>(score + o);
    *reinterpret_cast<float4*>(out + o) = make_float4(weigh(sc.x, mj.x, m.x) * inv.x, weigh(sc.y, mj.y, m.y) * inv.y,
                                                      weigh(sc.z, mj.z, m.z) * inv.z, weigh(sc.w, mj.w, m.w) * inv.w);
  }
}

// ------------------------------------------------------------------------------------------
// Fused gate preparation for one chunk: block pooling of Q and K, per-head projection, block RoPE,
// Q blocks to their buffer and K blocks appended to the gate cache -- one launch.
// One CTA per (block, job head): job heads 0..Hq-1 are the query side, the rest the key side
// (one per head of the key weight, pooling the KV head it belongs to).
// ------------------------------------------------------------------------------------------
struct PrepSide {
  const void* x;  // [B, L, H, D] tokens
  long long x_b, x_t, x_h;
  int x_dtype;
  int H;          // heads of x
  int kinds;      // pooling kinds
  const void* w;  // [Hw, nk*D, C] or NULL (identity: nk*D == C, Hw == H)
  int w_dtype;
  int Hw;         // heads of the weight (= output heads)
  const float* cos;  // [Bc, nb, C] or NULL
  const float* sin;
  int rope_batch;
  void* out;      // [B, >= off + nb, Hw, C] by strides
  long long o_b, o_blk, o_h;
  int o_dtype;
  int out_block_offset;
};
struct PrepArgs {
  PrepSide q, k;
  int B, L, D, C, bs, nb;
};

constexpr int kPrepThreads = 128;

template <int XDT, int WDT>
__global__ void __launch_bounds__(kPrepThreads) gate_prepare_kernel(const PrepArgs a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ float prep_smem[];  // partials [3][phases][D], pooled [3*D], y [C]
  const bool is_q = static_cast<int>(blockIdx.y) < a.q.Hw;
  const PrepSide& sd = is_q ? a.q : a.k;
  const int hw = is_q ? blockIdx.y : blockIdx.y - a.q.Hw;  // output / weight head
  const int hx = hw / (sd.Hw / sd.H);                      // token head it pools
  const int blk = blockIdx.x, b = blockIdx.z;
  const int groups = a.D / 8;
  const int phases = kPrepThreads / groups;
  float* part = prep_smem;
  float* pooled = part + 3 * phases * a.D;
  float* y = pooled + 3 * a.D;
  const int grp = threadIdx.x % groups, ph = threadIdx.x / groups;
  const int t0 = blk * a.bs, t1 = min(t0 + a.bs, a.L);
  float mx[8], mn[8], sm[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mx[i] = -INFINITY, mn[i] = INFINITY, sm[i] = 0.f;
  if (ph < phases) {
    // eight token rows per round, all loads issued before the arithmetic
    for (int tb = t0 + ph; tb < t1; tb += phases * 8) {
      float v[8][8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int t = min(tb + u * phases, t1 - 1);  // clamped rows repeat a token: harmless for max/min, skipped for the sum
        load8_t<XDT>(sd.x, b * sd.x_b + static_cast<long long>(t) * sd.x_t + hx * sd.x_h + grp * 8, v[u]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool real = tb + u * phases < t1;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          mx[i] = fmaxf(mx[i], v[u][i]), mn[i] = fminf(mn[i], v[u][i]);
          sm[i] += real ? v[u][i] : 0.f;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      part[(0 * phases + ph) * a.D + grp * 8 + i] = mx[i];
      part[(1 * phases + ph) * a.D + grp * 8 + i] = mn[i];
      part[(2 * phases + ph) * a.D + grp * 8 + i] = sm[i];
    }
  }
  __syncthreads();
  const float inv_cnt = 1.0f / static_cast<float>(t1 - t0);
  int n_kinds = 0;
  for (int d = threadIdx.x; d < a.D; d += kPrepThreads) {
    float rmx = -INFINITY, rmn = INFINITY, rsm = 0.f;
    for (int p = 0; p < phases; ++p) {
      rmx = fmaxf(rmx, part[(0 * phases + p) * a.D + d]);
      rmn = fminf(rmn, part[(1 * phases + p) * a.D + d]);
      rsm += part[(2 * phases + p) * a.D + d];
    }
    int c = 0;
    if (sd.kinds & 1) pooled[(c++) * a.D + d] = rmx;
    if (sd.kinds & 2) pooled[(c++) * a.D + d] = rmn;
    if (sd.kinds & 4) pooled[(c++) * a.D + d] = rsm * inv_cnt;
  }
  n_kinds = ((sd.kinds & 1) ? 1 : 0) + ((sd.kinds & 2) ? 1 : 0) + ((sd.kinds & 4) ? 1 : 0);
  const int Cin = n_kinds * a.D;
  __syncthreads();
  if (sd.w) {
    // Thread = (8 output channels, input-channel phase): every load is a 128-bit piece of a weight row
    // and a whole round of loads is issued before any arithmetic, so the round costs one latency.
    const int ogroups = a.C / 8;                   // 16-byte groups per weight row
    const int cphases = kPrepThreads / ogroups;    // input channels covered per load round
    const int og = threadIdx.x % ogroups, cp = threadIdx.x / ogroups;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (cp < cphases) {
      const long long wbase = static_cast<long long>(hw) * Cin * a.C + og * 8;
      for (int c0 = cp; c0 < Cin; c0 += cphases * 8) {
        float w[8][8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int c = c0 + u * cphases;
          if (c < Cin) {
            load8_t<WDT>(sd.w, wbase + static_cast<long long>(c) * a.C, w[u]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) w[u][i] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float xv = pooled[min(c0 + u * cphases, Cin - 1)];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = fmaf(xv, w[u][i], acc[i]);
        }
      }
      // partial sums of the input-channel phases meet in shared memory (reusing the pooling scratch)
#pragma unroll
      for (int i = 0; i < 8; ++i) part[cp * a.C + og * 8 + i] = acc[i];
    }
    __syncthreads();
    for (int o = threadIdx.x; o < a.C; o += kPrepThreads) {
      float sum = 0.f;
      for (int q = 0; q < cphases; ++q) sum += part[q * a.C + o];
      y[o] = sum;
    }
  } else {
    for (int o = threadIdx.x; o < a.C; o += kPrepThreads) y[o] = pooled[o];
  }
  __syncthreads();
  const int half = a.C / 2;
  for (int o = threadIdx.x; o < a.C; o += kPrepThreads) {
    float v = y[o];
    if (sd.cos) {
      const long long ro = ((sd.rope_batch > 1 ? static_cast<long long>(b) : 0) * a.nb + blk) * a.C + o;
      const float rot = o < half ? -y[o + half] : y[o - half];
      v = v * sd.cos[ro] + rot * sd.sin[ro];
    }
    store_elem(sd.out, b * sd.o_b + static_cast<long long>(sd.out_block_offset + blk) * sd.o_blk + hw * sd.o_h + o, sd.o_dtype, v);
  }
}

static bool dtype_ok(int dt) { return dt == CA_DTYPE_F32 || dt == CA_DTYPE_BF16 || dt == CA_DTYPE_F16; }

}  // namespace score
}  // namespace ca

namespace ca {
int launch_fp_score_sm100(const ca_flashprefill_score_params* p, cudaStream_t stream);  // ca_fpscore_sm100.cu
int launch_gate_scores_tc(const ca_gate_score_params* g, cudaStream_t stream);            // ca_select.cu
}

extern "C" {

int ca_pool_blocks(const ca_pool_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::score;
  CA_REQUIRE(p != nullptr && p->x && p->out, "params, x and out must be non-null");
  CA_REQUIRE(dtype_ok(p->x_dtype) && dtype_ok(p->out_dtype), "unsupported dtype");
  CA_REQUIRE(p->B > 0 && p->L > 0 && p->H > 0 && p->block_size > 0, "B, L, H, block_size must be positive");
  CA_REQUIRE(p->D > 0 && p->D % 8 == 0 && p->D <= 1024 && kPoolThreads % (p->D / 8) == 0,
             "D must be a multiple of 8 with D/8 dividing %d", kPoolThreads);
  CA_REQUIRE(p->kinds > 0 && p->kinds < 8, "kinds must be a non-empty subset of max|min|avg");
  CA_REQUIRE(p->x_stride_b % 8 == 0 && p->x_stride_t % 8 == 0 && p->x_stride_h % 8 == 0,
             "x strides must be multiples of 8 elements");
  CA_REQUIRE(reinterpret_cast<uintptr_t>(p->x) % 32 == 0 || (p->x_dtype != CA_DTYPE_F32 && reinterpret_cast<uintptr_t>(p->x) % 16 == 0),
             "x must be 16-byte aligned (32-byte for f32)");
  PoolArgs a;
  a.x = p->x, a.x_b = p->x_stride_b, a.x_t = p->x_stride_t, a.x_h = p->x_stride_h, a.x_dtype = p->x_dtype;
  a.out = p->out, a.o_b = p->out_stride_b, a.o_blk = p->out_stride_blk, a.o_h = p->out_stride_h, a.o_dtype = p->out_dtype;
  a.out_block_offset = p->out_block_offset;
  a.B = p->B, a.L = p->L, a.H = p->H, a.D = p->D, a.bs = p->block_size, a.kinds = p->kinds;
  const int nb = ceil_div(p->L, p->block_size);
  const int phases = kPoolThreads / (p->D / 8);
  const size_t smem = static_cast<size_t>(3) * phases * p->D * sizeof(float);
  launch_kernel(pool_blocks_kernel, dim3(nb, p->B * p->H), dim3(kPoolThreads), smem, static_cast<cudaStream_t>(stream_), a);
  CA_LAUNCH_CHECK("pool_blocks_kernel");
  return CA_OK;
}

int ca_gate_prepare(const ca_gate_prepare_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::score;
  CA_REQUIRE(p != nullptr, "params is null");
  CA_REQUIRE(p->B > 0 && p->L > 0 && p->block_size > 0, "B, L, block_size must be positive");
  CA_REQUIRE(p->D > 0 && p->D % 8 == 0 && p->D <= 1024 && kPrepThreads % (p->D / 8) == 0,
             "D must be a multiple of 8 with D/8 dividing %d", kPrepThreads);
  CA_REQUIRE(p->C >= 8 && p->C % 8 == 0 && p->C <= 1024 && kPrepThreads % (p->C / 8) == 0,
             "C must be a multiple of 8 with C/8 dividing %d", kPrepThreads);
  const ca_gate_side* sides[2] = {&p->q, &p->k};
  PrepArgs a;
  PrepSide* out_sides[2] = {&a.q, &a.k};
  for (int i = 0; i < 2; ++i) {
    const ca_gate_side* sd = sides[i];
    CA_REQUIRE(sd->x && sd->out, "token tensor and output of both sides must be non-null");
    CA_REQUIRE(dtype_ok(sd->x_dtype) && dtype_ok(sd->out_dtype), "unsupported dtype");
    CA_REQUIRE(sd->H > 0 && sd->Hw > 0 && sd->Hw % sd->H == 0, "weight heads must be a multiple of token heads");
    CA_REQUIRE(sd->kinds > 0 && sd->kinds < 8, "kinds must be a non-empty subset of max|min|avg");
    const int nk = ((sd->kinds & 1) ? 1 : 0) + ((sd->kinds & 2) ? 1 : 0) + ((sd->kinds & 4) ? 1 : 0);
    CA_REQUIRE(sd->w != nullptr || (nk * p->D == p->C && sd->Hw == sd->H), "identity projection needs nk*D == C and Hw == H");
    CA_REQUIRE(sd->w == nullptr || dtype_ok(sd->w_dtype), "unsupported weight dtype");
    CA_REQUIRE((sd->cos == nullptr) == (sd->sin == nullptr), "cos and sin must be given together");
    CA_REQUIRE(sd->cos == nullptr || sd->rope_batch == 1 || sd->rope_batch == p->B, "rope_batch must be 1 or B");
    CA_REQUIRE(sd->x_stride_b % 8 == 0 && sd->x_stride_t % 8 == 0 && sd->x_stride_h % 8 == 0, "token strides must be multiples of 8 elements");
    PrepSide* o = out_sides[i];
    o->x = sd->x, o->x_b = sd->x_stride_b, o->x_t = sd->x_stride_t, o->x_h = sd->x_stride_h, o->x_dtype = sd->x_dtype;
    o->H = sd->H, o->kinds = sd->kinds, o->w = sd->w, o->w_dtype = sd->w_dtype, o->Hw = sd->Hw;
    o->cos = sd->cos, o->sin = sd->sin, o->rope_batch = sd->rope_batch;
    o->out = sd->out, o->o_b = sd->out_stride_b, o->o_blk = sd->out_stride_blk, o->o_h = sd->out_stride_h;
    o->o_dtype = sd->out_dtype, o->out_block_offset = sd->out_block_offset;
  }
  a.B = p->B, a.L = p->L, a.D = p->D, a.C = p->C, a.bs = p->block_size;
  a.nb = ceil_div(p->L, p->block_size);
  const int phases = kPrepThreads / (p->D / 8);
  const size_t smem = (static_cast<size_t>(3) * phases * p->D + 3 * p->D + p->C) * sizeof(float);
  CA_REQUIRE(smem <= 48 * 1024, "D and C too large for the gate preparation kernel");
  CA_REQUIRE(p->q.x_dtype == p->k.x_dtype, "q and k tokens must share a dtype");
  const int wdt = p->k.w ? p->k.w_dtype : (p->q.w ? p->q.w_dtype : p->q.x_dtype);
  CA_REQUIRE((p->q.w == nullptr || p->q.w_dtype == wdt) && (p->k.w == nullptr || p->k.w_dtype == wdt), "q and k weights must share a dtype");
  const dim3 grid(a.nb, p->q.Hw + p->k.Hw, p->B);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
#define CA_PREP_CASE(XD, WD)                                                            \
  if (p->q.x_dtype == XD && wdt == WD) {                                                \
    launch_kernel_as(true, gate_prepare_kernel<XD, WD>, dim3(grid), dim3(kPrepThreads), smem, stream, a);     \
  } else
  CA_PREP_CASE(CA_DTYPE_BF16, CA_DTYPE_BF16)
  CA_PREP_CASE(CA_DTYPE_BF16, CA_DTYPE_F32)
  CA_PREP_CASE(CA_DTYPE_F16, CA_DTYPE_F16)
  CA_PREP_CASE(CA_DTYPE_F16, CA_DTYPE_F32)
  CA_PREP_CASE(CA_DTYPE_F32, CA_DTYPE_F32)
  CA_PREP_CASE(CA_DTYPE_F32, CA_DTYPE_BF16)
  CA_PREP_CASE(CA_DTYPE_F32, CA_DTYPE_F16)
  CA_PREP_CASE(CA_DTYPE_BF16, CA_DTYPE_F16)
  CA_PREP_CASE(CA_DTYPE_F16, CA_DTYPE_BF16)
  { return fail(CA_ERR_UNSUPPORTED, "unsupported dtype combination"); }
#undef CA_PREP_CASE
  CA_LAUNCH_CHECK("gate_prepare_kernel");
  return CA_OK;
}

int ca_gate_project(const ca_project_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::score;
  CA_REQUIRE(p != nullptr && p->x && p->out, "params, x and out must be non-null");
  CA_REQUIRE(p->B > 0 && p->nb > 0 && p->Hin > 0 && p->Hout > 0 && p->Cin > 0 && p->Cout > 0, "sizes must be positive");
  CA_REQUIRE(p->Hout % p->Hin == 0, "Hout (%d) must be a multiple of Hin (%d)", p->Hout, p->Hin);
  CA_REQUIRE(p->w != nullptr || (p->Cin == p->Cout), "identity projection needs Cin == Cout");
  CA_REQUIRE(p->w == nullptr || dtype_ok(p->w_dtype), "unsupported weight dtype");
  CA_REQUIRE(dtype_ok(p->out_dtype), "unsupported out dtype");
  CA_REQUIRE((p->cos == nullptr) == (p->sin == nullptr), "cos and sin must be given together");
  CA_REQUIRE(p->cos == nullptr || (p->Cout % 2 == 0 && (p->rope_batch == 1 || p->rope_batch == p->B)),
             "RoPE needs an even Cout and rope_batch in {1, B}");
  ProjArgs a;
  a.x = p->x, a.w = p->w, a.w_dtype = p->w_dtype, a.cos = p->cos, a.sin = p->sin, a.rope_batch = p->rope_batch;
  a.out = p->out, a.o_b = p->out_stride_b, a.o_blk = p->out_stride_blk, a.o_h = p->out_stride_h, a.o_dtype = p->out_dtype;
  a.out_block_offset = p->out_block_offset;
  a.B = p->B, a.nb = p->nb, a.Hin = p->Hin, a.Hout = p->Hout, a.Cin = p->Cin, a.Cout = p->Cout;
  const size_t smem = static_cast<size_t>(kProjBlocks) * (p->Cin + kProjSlices * p->Cout) * sizeof(float);
  CA_REQUIRE(smem <= 48 * 1024, "Cin + Cout too large");
  const dim3 threads(p->Cout >= 128 ? 128 : (p->Cout >= 64 ? 64 : 32), kProjSlices);
  launch_kernel(proj_rope_kernel, dim3(ceil_div(p->nb, kProjBlocks), p->Hout, p->B), dim3(threads), smem, static_cast<cudaStream_t>(stream_), a);
  CA_LAUNCH_CHECK("proj_rope_kernel");
  return CA_OK;
}

int ca_gate_scores(const ca_gate_score_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::score;
  CA_REQUIRE(p != nullptr && p->q && p->k && p->out, "params, q, k and out must be non-null");
  CA_REQUIRE(dtype_ok(p->q_dtype) && dtype_ok(p->k_dtype), "unsupported dtype");
  CA_REQUIRE(p->B > 0 && p->Hq > 0 && p->Hk > 0 && p->Qb > 0 && p->Kb > 0, "sizes must be positive");
  CA_REQUIRE(p->Hq % p->Hk == 0, "Hq must be a multiple of Hk");
  CA_REQUIRE(p->C > 0 && p->C % 8 == 0, "channel count must be a multiple of 8");
  CA_REQUIRE(p->k_stride_b % 8 == 0 && p->k_stride_blk % 8 == 0 && p->k_stride_h % 8 == 0,
             "k strides must be multiples of 8 elements");
  CA_REQUIRE(p->q_stride_b % 8 == 0 && p->q_stride_blk % 8 == 0 && p->q_stride_h % 8 == 0,
             "q strides must be multiples of 8 elements");
  CA_REQUIRE(p->Pb >= 0 && p->Pb + p->Qb >= 1, "Pb out of range");
  GateArgs a;
  a.q = p->q, a.q_b = p->q_stride_b, a.q_blk = p->q_stride_blk, a.q_h = p->q_stride_h, a.q_dtype = p->q_dtype;
  a.k = p->k, a.k_b = p->k_stride_b, a.k_blk = p->k_stride_blk, a.k_h = p->k_stride_h, a.k_dtype = p->k_dtype;
  a.out = p->out;
  a.B = p->B, a.Hq = p->Hq, a.Hk = p->Hk, a.Qb = p->Qb, a.Kb = p->Kb, a.Pb = p->Pb, a.C = p->C;
  a.scale = p->scale;
  a.masked_value = p->masked_value;
  const size_t smem = static_cast<size_t>(p->Qb) * p->C * sizeof(float);
  CA_REQUIRE(smem <= 160 * 1024, "Qb * C too large for the gate score kernel");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  {
    // the learned gate's usual shape: the tensor-core form, the same arithmetic as the fused score + rule launch
    const int rc_tc = launch_gate_scores_tc(p, stream);
    if (rc_tc != CA_ERR_UNSUPPORTED) return rc_tc;
  }
  if (p->C == 128 && p->Qb <= kGateRows && (p->k_dtype == CA_DTYPE_BF16 || p->k_dtype == CA_DTYPE_F16)) {
    const dim3 grid3(ceil_div(p->Kb, kGateThreads), p->Hq, p->B);
    const size_t smem3 = static_cast<size_t>(kGateRows) * 128 * sizeof(float);
    if (p->k_dtype == CA_DTYPE_BF16) {
      launch_kernel(gate_scores3_kernel<CA_DTYPE_BF16>, dim3(grid3), dim3(kGateThreads), smem3, stream, a);
    } else {
      launch_kernel(gate_scores3_kernel<CA_DTYPE_F16>, dim3(grid3), dim3(kGateThreads), smem3, stream, a);
    }
    CA_LAUNCH_CHECK("gate_scores3_kernel");
    return CA_OK;
  }
  if (p->C % 32 == 0) {
    const int q_pad = ceil_div(p->Qb, kGateRows) * kGateRows;
    const size_t smem2 = static_cast<size_t>(q_pad) * p->C * sizeof(float);
    CA_REQUIRE(smem2 <= 160 * 1024, "Qb * C too large for the gate score kernel");
    const dim3 grid2(ceil_div(p->Kb, 2 * kGateThreads), p->Hq, p->B);
    if (p->k_dtype == CA_DTYPE_BF16) {
      if (smem2 > 48 * 1024) CA_CUDA(cudaFuncSetAttribute(gate_scores2_kernel<CA_DTYPE_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem2)));
      launch_kernel(gate_scores2_kernel<CA_DTYPE_BF16>, dim3(grid2), dim3(kGateThreads), smem2, stream, a);
    } else if (p->k_dtype == CA_DTYPE_F16) {
      if (smem2 > 48 * 1024) CA_CUDA(cudaFuncSetAttribute(gate_scores2_kernel<CA_DTYPE_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem2)));
      launch_kernel(gate_scores2_kernel<CA_DTYPE_F16>, dim3(grid2), dim3(kGateThreads), smem2, stream, a);
    } else {
      if (smem2 > 48 * 1024) CA_CUDA(cudaFuncSetAttribute(gate_scores2_kernel<CA_DTYPE_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem2)));
      launch_kernel(gate_scores2_kernel<CA_DTYPE_F32>, dim3(grid2), dim3(kGateThreads), smem2, stream, a);
    }
    CA_LAUNCH_CHECK("gate_scores2_kernel");
    return CA_OK;
  }
  const dim3 grid(ceil_div(p->Kb, kGateThreads), p->Hq, p->B);
  if (p->k_dtype == CA_DTYPE_BF16) {
    if (smem > 48 * 1024) CA_CUDA(cudaFuncSetAttribute(gate_scores_kernel<CA_DTYPE_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    launch_kernel(gate_scores_kernel<CA_DTYPE_BF16>, dim3(grid), dim3(kGateThreads), smem, stream, a);
  } else if (p->k_dtype == CA_DTYPE_F16) {
    if (smem > 48 * 1024) CA_CUDA(cudaFuncSetAttribute(gate_scores_kernel<CA_DTYPE_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    launch_kernel(gate_scores_kernel<CA_DTYPE_F16>, dim3(grid), dim3(kGateThreads), smem, stream, a);
  } else {
    if (smem > 48 * 1024) CA_CUDA(cudaFuncSetAttribute(gate_scores_kernel<CA_DTYPE_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    launch_kernel(gate_scores_kernel<CA_DTYPE_F32>, dim3(grid), dim3(kGateThreads), smem, stream, a);
  }
  CA_LAUNCH_CHECK("gate_scores_kernel");
  return CA_OK;
}

int ca_flashprefill_score(const ca_flashprefill_score_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::score;
  CA_REQUIRE(p != nullptr && p->q && p->mean_k && p->score_raw && p->max_raw, "params, q, mean_k, score_raw, max_raw must be non-null");
  CA_REQUIRE(dtype_ok(p->q_dtype) && dtype_ok(p->k_dtype), "unsupported dtype");
  CA_REQUIRE(p->B > 0 && p->Q > 0 && p->Hq > 0 && p->Hkv > 0 && p->Kb > 0 && p->block_size > 0, "sizes must be positive");
  CA_REQUIRE(p->Hq % p->Hkv == 0, "Hq must be a multiple of Hkv");
  CA_REQUIRE(p->D == 128 || p->D == 64, "head dim must be 64 or 128");
  CA_REQUIRE(p->kv_len >= p->Q, "kv_len must be >= Q");
  CA_REQUIRE(p->Hq <= 256, "Hq larger than 256 is not supported");
  FpScoreArgs a;
  a.q = p->q, a.q_b = p->q_stride_b, a.q_t = p->q_stride_t, a.q_h = p->q_stride_h, a.q_dtype = p->q_dtype;
  a.mk = p->mean_k, a.k_b = p->k_stride_b, a.k_blk = p->k_stride_blk, a.k_h = p->k_stride_h, a.k_dtype = p->k_dtype;
  a.score = p->score_raw, a.mx = p->max_raw;
  a.B = p->B, a.Q = p->Q, a.Hq = p->Hq, a.Hkv = p->Hkv, a.D = p->D, a.Kb = p->Kb, a.bs = p->block_size;
  a.Qb = ceil_div(p->Q, p->block_size);
  a.P = p->kv_len - p->Q;
  a.sm_scale = (1.0f / sqrtf(static_cast<float>(p->D))) * 1.4426950408889634f;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // 16-bit inputs with d = 128 and block 64/128 run on the tensor cores; everything else (fp32
  // inputs, other shapes) on the CUDA-core kernel below
  const int rc_tc = launch_fp_score_sm100(p, stream);
  if (rc_tc != CA_OK && rc_tc != CA_ERR_UNSUPPORTED) return rc_tc;
  if (rc_tc == CA_ERR_UNSUPPORTED) {
    const size_t smem = (static_cast<size_t>(2) * kFpTile * (p->D + 1) + kFpTile * (kFpTile + 1)) * sizeof(float);
    CA_CUDA(cudaFuncSetAttribute(flashprefill_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    launch_kernel(flashprefill_score_kernel, dim3(ceil_div(p->Kb, kFpTile), a.Qb, p->B * p->Hq), dim3(kFpThreads), smem, stream, a);
    CA_LAUNCH_CHECK("flashprefill_score_kernel");
  }
  if (p->score_norm) {
    const int threads = 256;
    const size_t nsmem = static_cast<size_t>(threads / p->Hq) * p->Hq * sizeof(float);
    const bool vec4 = p->Hq % 4 == 0 && ((reinterpret_cast<uintptr_t>(p->score_raw) | reinterpret_cast<uintptr_t>(p->max_raw) |
                                          reinterpret_cast<uintptr_t>(p->score_norm)) & 15u) == 0;
    // (a plain launch: as a programmatic dependent of the score kernel the pair measured 98 us instead
    // of 52 us at block 64 / 128K, although the same change helps the attention merge kernel)
    if (vec4) {
      launch_kernel(flashprefill_normalize4_kernel, dim3(p->B * a.Qb, p->Hq / 4), dim3(256), 0, stream, p->score_raw, p->max_raw,
                    p->score_norm, p->Kb, p->Hq);
    } else {
      launch_kernel(flashprefill_normalize_kernel, dim3(p->B * a.Qb), dim3(threads), nsmem, stream, p->score_raw, p->max_raw,
                    p->score_norm, p->Kb, p->Hq);
    }
    CA_LAUNCH_CHECK("flashprefill_normalize_kernel");
  }
  return CA_OK;
}

}  // extern "C"
