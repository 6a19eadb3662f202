// Chunk append for a paged KV cache, fused with RoPE and the mean-K pooling of the training-free
// selector.  One pass over the chunk's q/k/v: q -> RoPE -> q_out, k -> RoPE -> cache pages (and
// the per-block mean of the rotated keys), v -> cache pages.  HBM-bound: every element is read
// once and written once; the reference spends a torch kernel per elementwise step and then
// re-concatenates the whole layer cache (DynamicCache.update through the _do_kv_cache_update hook,
// compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py:518-536).
//
// RoPE is the half-rotation form of compact_attn/modules/common.py:49-75,
//   out = (x * cos) + (rotate_half(x) * sin),
// evaluated the way torch evaluates it: each product and the sum are rounded separately, in the
// tensors' 16-bit type when the tables are 16-bit and in fp32 when the tables are fp32, so the
// result is bit-identical to the reference expression.
#include "ca_common.cuh"

namespace ca {
namespace append {

constexpr int kThreads = 128;

struct Tensor4 {  // [B, Q, H, D] with element strides, D contiguous
  const void* p;
  long long sb, st, sh;
};

struct Args {
  Tensor4 q, k, v;
  void* q_out;
  long long qo_b, qo_t, qo_h;
  const void* cos;
  const void* sin;
  long long cs_b, cs_t;  // cs_b == 0: one table for every batch entry
  int rope_f32;          // tables are fp32 (else the tensors' 16-bit type)
  void* k_pages;
  void* v_pages;
  long long page_stride, token_stride, head_stride;
  int page_size, num_pages, pages_per_seq;
  const int32_t* page_table;
  void* mean_k;  // optional [B, blocks, Hkv, D]
  long long mk_b, mk_blk, mk_h;
  int B, Q, Hq, Hkv, D;
  int position, block_size;
  int is_bf16;
  int32_t* status;
};

template <typename T>
__device__ __forceinline__ float to_f(T x);
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T from_f(float x);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

union Vec8 {
  uint4 u;
  __nv_bfloat16 b[8];
  __half h[8];
};

template <typename T>
__device__ __forceinline__ T& elem(Vec8& v, int i);
template <>
__device__ __forceinline__ __nv_bfloat16& elem<__nv_bfloat16>(Vec8& v, int i) { return v.b[i]; }
template <>
__device__ __forceinline__ __half& elem<__half>(Vec8& v, int i) { return v.h[i]; }

// Rotates one (lo, hi) pair of 8-element groups: lo = x[d..d+7], hi = x[d+D/2 .. d+D/2+7].
// kF32: tables fp32 -> fp32 products and sum, one rounding to T at the end.
// else: tables in T -> each product rounded to T, then the sum rounded to T (torch's 16-bit ops).
template <typename T, bool kF32>
__device__ __forceinline__ void rope8(Vec8& lo, Vec8& hi, const void* cos, const void* sin, long long cs_off, int half) {
  float c_lo[8], s_lo[8], c_hi[8], s_hi[8];
  if (kF32) {
    const float* c = static_cast<const float*>(cos) + cs_off;
    const float* s = static_cast<const float*>(sin) + cs_off;
    const float4 a0 = *reinterpret_cast<const float4*>(c), a1 = *reinterpret_cast<const float4*>(c + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(c + half), b1 = *reinterpret_cast<const float4*>(c + half + 4);
    const float4 e0 = *reinterpret_cast<const float4*>(s), e1 = *reinterpret_cast<const float4*>(s + 4);
    const float4 f0 = *reinterpret_cast<const float4*>(s + half), f1 = *reinterpret_cast<const float4*>(s + half + 4);
    c_lo[0] = a0.x, c_lo[1] = a0.y, c_lo[2] = a0.z, c_lo[3] = a0.w, c_lo[4] = a1.x, c_lo[5] = a1.y, c_lo[6] = a1.z, c_lo[7] = a1.w;
    c_hi[0] = b0.x, c_hi[1] = b0.y, c_hi[2] = b0.z, c_hi[3] = b0.w, c_hi[4] = b1.x, c_hi[5] = b1.y, c_hi[6] = b1.z, c_hi[7] = b1.w;
    s_lo[0] = e0.x, s_lo[1] = e0.y, s_lo[2] = e0.z, s_lo[3] = e0.w, s_lo[4] = e1.x, s_lo[5] = e1.y, s_lo[6] = e1.z, s_lo[7] = e1.w;
    s_hi[0] = f0.x, s_hi[1] = f0.y, s_hi[2] = f0.z, s_hi[3] = f0.w, s_hi[4] = f1.x, s_hi[5] = f1.y, s_hi[6] = f1.z, s_hi[7] = f1.w;
  } else {
    const T* c = static_cast<const T*>(cos) + cs_off;
    const T* s = static_cast<const T*>(sin) + cs_off;
    Vec8 a, b, e, f;
    a.u = *reinterpret_cast<const uint4*>(c), b.u = *reinterpret_cast<const uint4*>(c + half);
    e.u = *reinterpret_cast<const uint4*>(s), f.u = *reinterpret_cast<const uint4*>(s + half);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      c_lo[i] = to_f(elem<T>(a, i)), c_hi[i] = to_f(elem<T>(b, i));
      s_lo[i] = to_f(elem<T>(e, i)), s_hi[i] = to_f(elem<T>(f, i));
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float x_lo = to_f(elem<T>(lo, i)), x_hi = to_f(elem<T>(hi, i));
    // rotate_half(x) = [-x_hi, x_lo]
    float o_lo, o_hi;
    if (kF32) {
      o_lo = __fadd_rn(__fmul_rn(x_lo, c_lo[i]), __fmul_rn(-x_hi, s_lo[i]));
      o_hi = __fadd_rn(__fmul_rn(x_hi, c_hi[i]), __fmul_rn(x_lo, s_hi[i]));
    } else {
      const float p0 = to_f(from_f<T>(__fmul_rn(x_lo, c_lo[i]))), p1 = to_f(from_f<T>(__fmul_rn(-x_hi, s_lo[i])));
      const float p2 = to_f(from_f<T>(__fmul_rn(x_hi, c_hi[i]))), p3 = to_f(from_f<T>(__fmul_rn(x_lo, s_hi[i])));
      o_lo = __fadd_rn(p0, p1);
      o_hi = __fadd_rn(p2, p3);
    }
    elem<T>(lo, i) = from_f<T>(o_lo);
    elem<T>(hi, i) = from_f<T>(o_hi);
  }
}

// grid: (chunk blocks, Hq + 2*Hkv head slots, B).  A CTA moves one block_size-token block of one
// head: slot < Hq -> q head, next Hkv -> k head, last Hkv -> v head.  Thread = (token phase,
// 8-element group of the low half); it also handles the matching group of the high half.
template <typename T, bool kF32>
__global__ void __launch_bounds__(kThreads) rope_append_kernel(const Args a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  extern __shared__ float mk_smem[];  // [phases][D] partial sums of the rotated keys
  const int half = a.D / 2;
  const int groups = half / 8;               // threads per token row
  const int phases = kThreads / groups;      // token rows per pass
  const int grp = threadIdx.x % groups, ph = threadIdx.x / groups;
  const int blk = blockIdx.x, slot = blockIdx.y, b = blockIdx.z;
  const int t0 = blk * a.block_size;
  const int t1 = min(t0 + a.block_size, a.Q);
  const int d = grp * 8;
  const bool is_q = slot < a.Hq;
  const bool is_k = !is_q && slot < a.Hq + a.Hkv;
  const int h = is_q ? slot : (is_k ? slot - a.Hq : slot - a.Hq - a.Hkv);
  const Tensor4 src = is_q ? a.q : (is_k ? a.k : a.v);
  if (src.p == nullptr) return;  // q is optional
  float sum_lo[8], sum_hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sum_lo[i] = 0.f, sum_hi[i] = 0.f;
  bool bad = false;
  if (ph < phases) {
    for (int t = t0 + ph; t < t1; t += phases) {
      const T* x = static_cast<const T*>(src.p) + b * src.sb + static_cast<long long>(t) * src.st + h * src.sh;
      Vec8 lo, hi;
      lo.u = *reinterpret_cast<const uint4*>(x + d);
      hi.u = *reinterpret_cast<const uint4*>(x + half + d);
      if (is_q || is_k) rope8<T, kF32>(lo, hi, a.cos, a.sin, b * a.cs_b + static_cast<long long>(t) * a.cs_t + d, half);
      T* dst;
      if (is_q) {
        dst = static_cast<T*>(a.q_out) + b * a.qo_b + static_cast<long long>(t) * a.qo_t + h * a.qo_h;
      } else {
        const int tok = a.position + t;
        const int lp = tok / a.page_size, off = tok - lp * a.page_size;
        int page = a.page_table ? a.page_table[static_cast<long long>(b) * a.pages_per_seq + lp] : b * a.pages_per_seq + lp;
        if (page < 0 || page >= a.num_pages) {
          bad = true;  // reported through the status word; the token is skipped, nothing is written out of range
          continue;
        }
        dst = static_cast<T*>(is_k ? a.k_pages : a.v_pages) + page * a.page_stride + off * a.token_stride + h * a.head_stride;
      }
      *reinterpret_cast<uint4*>(dst + d) = lo.u;
      *reinterpret_cast<uint4*>(dst + half + d) = hi.u;
      if (is_k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sum_lo[i] += to_f(elem<T>(lo, i)), sum_hi[i] += to_f(elem<T>(hi, i));
      }
    }
  }
  if (bad && a.status) atomicOr(a.status, CA_STATUS_BAD_INDEX);
  if (!is_k || a.mean_k == nullptr) return;  // uniform per CTA
  // mean of the rotated keys of this block: token phases summed in order 0..phases-1
  if (ph < phases) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      mk_smem[ph * a.D + d + i] = sum_lo[i];
      mk_smem[ph * a.D + half + d + i] = sum_hi[i];
    }
  }
  __syncthreads();
  const float inv = 1.0f / static_cast<float>(t1 - t0);
  T* mk = static_cast<T*>(a.mean_k) + b * a.mk_b + static_cast<long long>(a.position / a.block_size + blk) * a.mk_blk + h * a.mk_h;
  for (int e = threadIdx.x; e < a.D; e += kThreads) {
    float s = 0.f;
    for (int p = 0; p < phases; ++p) s += mk_smem[p * a.D + e];
    mk[e] = from_f<T>(s * inv);
  }
}

}  // namespace append
}  // namespace ca

extern "C" int ca_rope_append(const ca_rope_append_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::append;
  CA_REQUIRE(p != nullptr, "params is null");
  CA_REQUIRE(p->B > 0 && p->Q > 0 && p->Hkv > 0 && p->Hq >= 0, "B, Q, Hkv must be positive");
  CA_REQUIRE(p->dtype == CA_DTYPE_BF16 || p->dtype == CA_DTYPE_F16, "q/k/v must be bf16 or f16");
  CA_REQUIRE(p->D >= 16 && p->D % 16 == 0 && p->D <= 512 && kThreads % (p->D / 16) == 0,
             "D must be a multiple of 16, at most 512, with D/16 dividing %d", kThreads);
  CA_REQUIRE(p->k && p->v && p->cache.k && p->cache.v, "k, v and the cache pages must be non-null");
  CA_REQUIRE((p->q == nullptr) == (p->q_out == nullptr), "q and q_out must be given together");
  CA_REQUIRE(p->q != nullptr || p->Hq == 0, "Hq must be 0 without q");
  CA_REQUIRE(p->cos && p->sin, "cos and sin must be non-null");
  CA_REQUIRE(p->rope_dtype == p->dtype || p->rope_dtype == CA_DTYPE_F32, "cos/sin must be fp32 or the tensors' type");
  CA_REQUIRE(p->block_size > 0 && p->position >= 0, "block_size must be positive and position non-negative");
  CA_REQUIRE(p->mean_k == nullptr || p->position % p->block_size == 0, "mean_k needs a chunk that starts on a block boundary");
  const ca_kv_layout& c = p->cache;
  CA_REQUIRE(c.page_size > 0 && c.pages_per_seq > 0 && c.num_pages > 0, "cache layout must be positive");
  CA_REQUIRE(c.head_div <= 1, "cache.head_div is read by ca_attn_compact only");
  CA_REQUIRE(static_cast<long long>(p->position) + p->Q <= static_cast<long long>(c.pages_per_seq) * c.page_size,
             "chunk does not fit in the cache (position %d + Q %d > %lld tokens)", p->position, p->Q,
             static_cast<long long>(c.pages_per_seq) * c.page_size);
  const long long strides[] = {p->q_stride_b, p->q_stride_t, p->q_stride_h, p->qo_stride_b, p->qo_stride_t, p->qo_stride_h,
                               p->k_stride_b, p->k_stride_t, p->k_stride_h, p->v_stride_b, p->v_stride_t, p->v_stride_h,
                               p->cs_stride_b, p->cs_stride_t, c.page_stride, c.token_stride, c.head_stride,
                               p->mk_stride_b, p->mk_stride_blk, p->mk_stride_h};
  for (long long s : strides) CA_REQUIRE(s % 8 == 0, "every stride must be a multiple of 8 elements (16-byte vector access)");
  const void* ptrs[] = {p->q, p->q_out, p->k, p->v, p->cos, p->sin, c.k, c.v, p->mean_k};
  for (const void* q : ptrs) CA_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15u) == 0, "every tensor must be 16-byte aligned");

  Args a;
  a.q = Tensor4{p->q, p->q_stride_b, p->q_stride_t, p->q_stride_h};
  a.k = Tensor4{p->k, p->k_stride_b, p->k_stride_t, p->k_stride_h};
  a.v = Tensor4{p->v, p->v_stride_b, p->v_stride_t, p->v_stride_h};
  a.q_out = p->q_out, a.qo_b = p->qo_stride_b, a.qo_t = p->qo_stride_t, a.qo_h = p->qo_stride_h;
  a.cos = p->cos, a.sin = p->sin, a.cs_b = p->cs_stride_b, a.cs_t = p->cs_stride_t;
  a.rope_f32 = p->rope_dtype == CA_DTYPE_F32;
  a.k_pages = const_cast<void*>(c.k), a.v_pages = const_cast<void*>(c.v);
  a.page_stride = c.page_stride, a.token_stride = c.token_stride, a.head_stride = c.head_stride;
  a.page_size = c.page_size, a.num_pages = c.num_pages, a.pages_per_seq = c.pages_per_seq, a.page_table = c.page_table;
  a.mean_k = p->mean_k, a.mk_b = p->mk_stride_b, a.mk_blk = p->mk_stride_blk, a.mk_h = p->mk_stride_h;
  a.B = p->B, a.Q = p->Q, a.Hq = p->Hq, a.Hkv = p->Hkv, a.D = p->D;
  a.position = p->position, a.block_size = p->block_size;
  a.is_bf16 = p->dtype == CA_DTYPE_BF16;
  a.status = p->status;

  const int nb = ceil_div(p->Q, p->block_size);
  const int phases = kThreads / (p->D / 16);
  const size_t smem = static_cast<size_t>(phases) * p->D * sizeof(float);
  const dim3 grid(nb, p->Hq + 2 * p->Hkv, p->B);
  CA_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "too many heads or batch entries for one launch");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a.is_bf16) {
    if (a.rope_f32) launch_kernel(rope_append_kernel<__nv_bfloat16, true>, dim3(grid), dim3(kThreads), smem, stream, a);
    else launch_kernel(rope_append_kernel<__nv_bfloat16, false>, dim3(grid), dim3(kThreads), smem, stream, a);
  } else {
    if (a.rope_f32) launch_kernel(rope_append_kernel<__half, true>, dim3(grid), dim3(kThreads), smem, stream, a);
    else launch_kernel(rope_append_kernel<__half, false>, dim3(grid), dim3(kThreads), smem, stream, a);
  }
  CA_LAUNCH_CHECK("rope_append_kernel");
  return CA_OK;
}
