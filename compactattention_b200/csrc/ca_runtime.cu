// Host-side runtime shared by every entry point: thread-local error text, launch accounting,
// driver entry-point resolution and cached device properties.
#include "ca_common.cuh"

#include <mutex>

namespace ca {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

std::atomic<int>& programmatic_launch_flag() {
  static std::atomic<int> flag{0};
  return flag;
}

std::atomic<long long>& launch_counter() {
  static std::atomic<long long> counter{0};
  return counter;
}

tensor_map_encode_fn get_tensor_map_encoder() {
  static std::once_flag once;
  static tensor_map_encode_fn fn = nullptr;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (err == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<tensor_map_encode_fn>(sym);
    }
  });
  return fn;
}

int get_device_info(DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  static bool have[64] = {false};
  int dev = 0;
  CA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(CA_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceInfo info;
    info.ordinal = dev;
    CA_CUDA(cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev));
    CA_CUDA(cudaDeviceGetAttribute(&info.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    CA_CUDA(cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    CA_CUDA(cudaDeviceGetAttribute(&info.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    cache[dev] = info;
    have[dev] = true;
  }
  *out = cache[dev];
  return CA_OK;
}

// One CTA waits, with the bounded wait every tcgen05 / TMA kernel of the library uses, on a barrier nothing
// ever arrives on: the wait must end after `limit_ns` with the abort flag set, and the kernel must return.
__global__ void selftest_bounded_wait_kernel(unsigned long long limit_ns, int32_t* status, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::mbar_fence_init();
  }
  __syncthreads();
  const uint64_t t0 = ptx::globaltimer_ns();
  // every thread waits like the roles of a kernel do; the first to pass the limit raises the flag, the others see it
  const bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0, &abort_flag, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (waited_ns) *waited_ns = ptx::globaltimer_ns() - t0;
    if (!ok && abort_flag && status) atomicOr(status, CA_STATUS_TIMEOUT);
  }
}

}  // namespace ca

extern "C" {

int ca_selftest_bounded_wait(uint64_t limit_ns, int32_t* status, uint64_t* waited_ns, ca_stream_t stream) {
  using namespace ca;
  CA_REQUIRE(status != nullptr, "status must be non-null");
  CA_REQUIRE(limit_ns > 0 && limit_ns <= 1000000000ull, "limit_ns must lie in (0, 1 s]");
  launch_kernel(selftest_bounded_wait_kernel, dim3(1), dim3(128), 0, static_cast<cudaStream_t>(stream),
                static_cast<unsigned long long>(limit_ns), status, reinterpret_cast<unsigned long long*>(waited_ns));
  CA_LAUNCH_CHECK("selftest_bounded_wait_kernel");
  return CA_OK;
}

const char* ca_last_error(void) { return ca::last_error_buffer(); }

int ca_abi_version(void) { return 2; }

int ca_chunk_step(const ca_chunk_step_params* p, ca_stream_t stream) {
  using namespace ca;
  CA_REQUIRE(p != nullptr, "params is null");
  int rc = CA_OK;
  if (p->append.k != nullptr && (rc = ca_rope_append(&p->append, stream)) != CA_OK) return rc;
  if (p->prepare.q.x != nullptr && (rc = ca_gate_prepare(&p->prepare, stream)) != CA_OK) return rc;
  // gate scores feeding a fused rule + table: one launch for the three stages
  const bool score_select = p->score.q != nullptr && p->union_scratch != nullptr && p->select.score != nullptr &&
                            p->select.score == p->score.out && p->fp_score.q == nullptr;
  if (score_select) {
    if ((rc = ca_gate_score_select(&p->score, &p->select, &p->table, p->union_scratch, p->union_scratch_bytes, p->write_scores,
                                   stream)) != CA_OK)
      return rc;
  }
  if (!score_select && p->score.q != nullptr && (rc = ca_gate_scores(&p->score, stream)) != CA_OK) return rc;
  if (p->fp_score.q != nullptr && (rc = ca_flashprefill_score(&p->fp_score, stream)) != CA_OK) return rc;
  if (!score_select && p->select.score != nullptr) {
    if (p->union_scratch != nullptr) {
      if ((rc = ca_select_union_table(&p->select, &p->table, p->union_scratch, p->union_scratch_bytes, stream)) != CA_OK) return rc;
    } else {
      if ((rc = ca_select_rows(&p->select, stream)) != CA_OK) return rc;
      if ((rc = ca_union_table(&p->table, stream)) != CA_OK) return rc;
    }
  }
  if (p->attn.q != nullptr && (rc = ca_attn_compact(&p->attn, stream)) != CA_OK) return rc;
  return CA_OK;
}

int ca_set_programmatic_launch(int enabled) {
  return ca::programmatic_launch_flag().exchange(enabled != 0 ? 1 : 0, std::memory_order_relaxed);
}

int64_t ca_launch_count(void) { return ca::launch_counter().load(std::memory_order_relaxed); }

}  // extern "C"
