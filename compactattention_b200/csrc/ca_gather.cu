// Compact KV gather (cache fill): copies each row's selected past blocks, then the chunk's own
// blocks, from the source cache (paged or contiguous) into a compact paged cache.
// Pure byte movement, HBM-bound: a persistent grid walks exactly the selected (row, rank)
// work items (the counts stay on the device), 128-bit loads and stores, one 64-token sub-block of
// K and of V per item so every warp instruction moves full 512-byte token rows.
#include "ca_common.cuh"

namespace ca {
namespace gather {

constexpr int kThreads = 256;
constexpr int kSub = 64;
constexpr int kMaxRows = 1024;

struct Args {
  const uint16_t* k;
  const uint16_t* v;
  long long page_stride, token_stride, head_stride;
  int page_size, num_pages, pages_per_seq;
  const int32_t* page_table;
  const int32_t* block_idx;
  int idx_stride;
  const int32_t* counts;
  const int32_t* page_offsets;  // optional [R+1] in destination pages
  long long dst_row_stride_tokens;  // used when page_offsets == NULL
  uint16_t* k_dst;
  uint16_t* v_dst;
  int dst_page_size;
  int B, Hkv, D, R;
  int past_blocks, past_tokens, cur_sub, spb, block_size;
  int32_t* status;
};

__global__ void __launch_bounds__(kThreads) gather_kv_kernel(const Args a) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // nothing in global memory is touched before this
  __shared__ int prefix[kMaxRows + 1];  // exclusive prefix of sub-block items per row
  __shared__ int warp_sums[kThreads / 32];
  // prefix over rows (R <= kMaxRows), recomputed by every CTA: a few hundred integer adds
  int running = 0;
  for (int base = 0; base < a.R; base += kThreads) {
    const int r = base + threadIdx.x;
    int c = 0;
    if (r < a.R) {
      c = a.counts[r];
      c = c < 0 ? 0 : (c > a.past_blocks ? a.past_blocks : c);
      c = c * a.spb + a.cur_sub;
    }
    int inc = c;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += n;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    int woff = 0;
    for (int w = 0; w < warp; ++w) woff += warp_sums[w];
    if (r < a.R) prefix[r] = running + woff + inc - c;
    int tot = 0;
    for (int w = 0; w < kThreads / 32; ++w) tot += warp_sums[w];
    running += tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) prefix[a.R] = running;
  __syncthreads();
  const int total = prefix[a.R];
  const int chunks = a.D / 8;               // 16-byte chunks per token row
  const int tok_per_pass = kThreads / chunks;
  const int ch = threadIdx.x % chunks, tp = threadIdx.x / chunks;

  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    // owner row: largest r with prefix[r] <= item
    int lo = 0, hi = a.R;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid] <= item) lo = mid; else hi = mid;
    }
    const int row = lo;
    const int u = item - prefix[row];  // sub-block rank inside the row's compact sequence
    const int b = row / a.Hkv, hkv = row % a.Hkv;
    int cnt = a.counts[row];
    cnt = cnt < 0 ? 0 : (cnt > a.past_blocks ? a.past_blocks : cnt);
    const int n_past_sub = cnt * a.spb;
    int tok;
    if (u < n_past_sub) {
      const int bi = u / a.spb;
      int blk = a.block_idx[static_cast<long long>(row) * a.idx_stride + bi];
      if (blk < 0 || blk >= a.past_blocks) {
        if (threadIdx.x == 0 && a.status) atomicOr(a.status, CA_STATUS_BAD_INDEX);
        blk = blk < 0 ? 0 : a.past_blocks - 1;
      }
      tok = blk * a.block_size + (u - bi * a.spb) * kSub;
    } else {
      tok = a.past_tokens + (u - n_past_sub) * kSub;
    }
    const int lp = tok / a.page_size;
    const int off = tok - lp * a.page_size;
    int page = a.page_table ? a.page_table[static_cast<long long>(b) * a.pages_per_seq + lp] : b * a.pages_per_seq + lp;
    if (page < 0 || page >= a.num_pages) {
      if (threadIdx.x == 0 && a.status) atomicOr(a.status, CA_STATUS_BAD_INDEX);
      page = 0;
    }
    const long long src = page * a.page_stride + static_cast<long long>(off) * a.token_stride + hkv * a.head_stride;
    const long long dst_tok = (a.page_offsets ? static_cast<long long>(a.page_offsets[row]) * a.dst_page_size
                                              : static_cast<long long>(row) * a.dst_row_stride_tokens) +
                              static_cast<long long>(u) * kSub;
    uint4 kreg[4], vreg[4];
    for (int t0 = 0; t0 < kSub; t0 += 4 * tok_per_pass) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int t = t0 + q * tok_per_pass + tp;
        if (t < kSub) {
          kreg[q] = *reinterpret_cast<const uint4*>(a.k + src + static_cast<long long>(t) * a.token_stride + ch * 8);
          vreg[q] = *reinterpret_cast<const uint4*>(a.v + src + static_cast<long long>(t) * a.token_stride + ch * 8);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int t = t0 + q * tok_per_pass + tp;
        if (t < kSub) {
          *reinterpret_cast<uint4*>(a.k_dst + (dst_tok + t) * a.D + ch * 8) = kreg[q];
          *reinterpret_cast<uint4*>(a.v_dst + (dst_tok + t) * a.D + ch * 8) = vreg[q];
        }
      }
    }
  }
}

}  // namespace gather
}  // namespace ca

extern "C" {

int ca_gather_kv(const ca_gather_params* p, ca_stream_t stream_) {
  using namespace ca;
  using namespace ca::gather;
  CA_REQUIRE(p != nullptr, "params is null");
  CA_REQUIRE(p->kv.head_div <= 1, "kv.head_div is read by ca_attn_compact only");
  CA_REQUIRE(p->kv.k && p->kv.v && p->k_dst && p->v_dst, "kv.k, kv.v, k_dst and v_dst must be non-null");
  CA_REQUIRE(p->block_idx && p->counts, "block_idx and counts must be non-null");
  CA_REQUIRE(p->dtype == CA_DTYPE_BF16 || p->dtype == CA_DTYPE_F16, "dtype must be bf16 or f16");
  CA_REQUIRE(p->B > 0 && p->Hkv > 0 && p->Q > 0, "B, Hkv, Q must be positive");
  CA_REQUIRE(p->B * p->Hkv <= kMaxRows, "more than %d rows are not supported", kMaxRows);
  CA_REQUIRE(p->D > 0 && p->D % 8 == 0 && kThreads % (p->D / 8) == 0, "D must be a multiple of 8 with D/8 dividing %d", kThreads);
  CA_REQUIRE(p->block_size > 0 && p->block_size % kSub == 0, "block_size must be a positive multiple of 64");
  CA_REQUIRE(p->kv_len >= p->Q && (p->kv_len - p->Q) % p->block_size == 0 && p->Q % kSub == 0,
             "past length must be a multiple of block_size and Q a multiple of 64");
  CA_REQUIRE(p->kv.page_size > 0 && p->kv.page_size % kSub == 0, "source page_size must be a positive multiple of 64");
  CA_REQUIRE(p->kv.page_stride % 8 == 0 && p->kv.token_stride % 8 == 0 && p->kv.head_stride % 8 == 0,
             "kv strides must be multiples of 8 elements");
  CA_REQUIRE(p->page_offsets != nullptr || p->dst_row_stride_tokens > 0, "page_offsets or dst_row_stride_tokens is required");
  CA_REQUIRE(p->dst_page_size > 0, "dst_page_size must be positive");
  DeviceInfo dev;
  int rc = get_device_info(&dev);
  if (rc != CA_OK) return rc;
  Args a;
  a.k = static_cast<const uint16_t*>(p->kv.k), a.v = static_cast<const uint16_t*>(p->kv.v);
  a.page_stride = p->kv.page_stride, a.token_stride = p->kv.token_stride, a.head_stride = p->kv.head_stride;
  a.page_size = p->kv.page_size, a.num_pages = p->kv.num_pages, a.pages_per_seq = p->kv.pages_per_seq;
  a.page_table = p->kv.page_table;
  a.block_idx = p->block_idx, a.idx_stride = p->block_idx_stride, a.counts = p->counts;
  a.page_offsets = p->page_offsets;
  a.dst_row_stride_tokens = p->dst_row_stride_tokens;
  a.k_dst = static_cast<uint16_t*>(p->k_dst), a.v_dst = static_cast<uint16_t*>(p->v_dst);
  a.dst_page_size = p->dst_page_size;
  a.B = p->B, a.Hkv = p->Hkv, a.D = p->D, a.R = p->B * p->Hkv;
  a.past_tokens = p->kv_len - p->Q;
  a.past_blocks = a.past_tokens / p->block_size;
  a.cur_sub = p->Q / kSub;
  a.spb = p->block_size / kSub;
  a.block_size = p->block_size;
  a.status = p->status;
  // persistent grid: a multiple of the SM count, 8 CTAs of 256 threads per SM
  const int grid = dev.sm_count * 8;
  launch_kernel(gather_kv_kernel, dim3(grid), dim3(kThreads), 0, static_cast<cudaStream_t>(stream_), a);
  CA_LAUNCH_CHECK("gather_kv_kernel");
  return CA_OK;
}

}  // extern "C"
