// The hop between pipeline stages over peer memory (NVLink): the sender's kernel stores the
// activations straight into the next GPU's inbox and raises a flag there; the receiver's stream
// holds a one-thread kernel that waits (bounded) for that flag. Flags only ever grow (message
// number + 1), so nothing is reset and a late reader cannot mistake an old value for a new one.
// The reference moves the same tensor with an HTTP POST per hop
// (deserve_worker/engine/pipeline/processor.py:218-224).
#include <algorithm>

#include "common.cuh"

namespace dsv {
namespace {

constexpr int kPushThreads = 256;

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
  return t;
}

// Once a wait of this hop has given up, the link is out of step: later pushes and credits of the
// same process are dropped (nothing is credited for a message that never came, no buffer is
// overwritten on the strength of a credit that never came) until the host has read the status.
__device__ __forceinline__ bool link_broken(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status) == ST_WAIT_TIMEOUT;
}

// dst (peer or local memory) <- src, 16 bytes per thread and step; the CTA that finishes last
// publishes `value` in *flag. `arrivals` is a local counter that returns to zero.
__global__ void __launch_bounds__(kPushThreads)
push_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t n_vec, int32_t* flag, int32_t value,
            unsigned int* arrivals, const int* status) {
  if (link_broken(status)) return;
  for (int64_t i = (int64_t)blockIdx.x * kPushThreads + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * kPushThreads)
    dst[i] = src[i];
  __threadfence_system();  // this thread's stores are visible to the peer before anything that follows
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int seen = atomicAdd(arrivals, 1u);
    if (seen == gridDim.x - 1) {
      *arrivals = 0;
      __threadfence_system();
      st_release_sys(flag, value);
    }
  }
}

__global__ void signal_kernel(int32_t* flag, int32_t value, const int* status) {
  if (link_broken(status)) return;
  __threadfence_system();
  st_release_sys(flag, value);
}

// One thread polls until *flag >= value; gives up once timeout_ns of the global timer have passed
// (and, as a second bound that does not depend on the timer, after 2^31 polls) and records
// ST_WAIT_TIMEOUT.
__global__ void wait_kernel(const int32_t* flag, int32_t value, long long timeout_ns, int* status) {
  if (link_broken(status)) return;  // an earlier wait already gave up: do not sit out another full timeout
  const unsigned long long t0 = global_ns();
  for (long long i = 0; i < (1ll << 31); ++i) {
    if (ld_acquire_sys(flag) >= value) return;
    if (i > 64) {
      __nanosleep(200);
      if ((i & 15) == 0 && global_ns() - t0 > (unsigned long long)timeout_ns) break;
    }
  }
  record_status(status, ST_WAIT_TIMEOUT);
}

}  // namespace
}  // namespace dsv

extern "C" {

int dsv_peer_push(void* dst, const void* src, int64_t bytes, int32_t* flag, int32_t value, uint32_t* arrivals,
                  int sm_count, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dst && src && flag && arrivals, "peer_push: null pointer argument");
  DSV_REQUIRE(bytes > 0 && bytes % 16 == 0 && aligned16(dst) && aligned16(src),
              "peer_push: %lld bytes / pointers must be multiples of 16", (long long)bytes);
  if (sm_count <= 0) sm_count = 148;
  const int64_t n_vec = bytes / 16;
  const int grid = (int)std::min<int64_t>((n_vec + kPushThreads - 1) / kPushThreads, (int64_t)sm_count * 2);
  push_kernel<<<grid, kPushThreads, 0, (cudaStream_t)stream>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src),
                                                               n_vec, flag, value, arrivals, device_status_ptr());
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

int dsv_peer_signal(int32_t* flag, int32_t value, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(flag != nullptr, "peer_signal: null flag");
  signal_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag, value, device_status_ptr());
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

int dsv_peer_wait(const int32_t* flag, int32_t value, int64_t timeout_ns, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(flag != nullptr, "peer_wait: null flag");
  DSV_REQUIRE(timeout_ns > 0 && timeout_ns <= 600ll * 1000000000ll,
              "peer_wait: timeout_ns must be in (0, 600 s] (every wait is bounded)");
  wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag, value, (long long)timeout_ns, device_status_ptr());
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

}  // extern "C"
