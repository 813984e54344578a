// Library-level entry points of libdeserve_kv.so: version, error string,
// device info and the device status word that kernels' self-checks write.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace dsv {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

// One status word per device image of this library.
__device__ int g_device_status = 0;

namespace {
constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices] = {nullptr};
std::mutex g_status_mutex;
}  // namespace

int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

}  // namespace dsv

extern "C" {

int dsv_version(void) { return DSV_VERSION; }

const char* dsv_last_error(void) { return dsv::error_buffer(); }

int dsv_device_info(int* sm_count, int* cc_major, int* cc_minor) {
  DSV_REQUIRE(sm_count && cc_major && cc_minor, "dsv_device_info: null output pointer");
  int dev = 0;
  DSV_CUDA(cudaGetDevice(&dev));
  DSV_CUDA(cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, dev));
  DSV_CUDA(cudaDeviceGetAttribute(cc_major, cudaDevAttrComputeCapabilityMajor, dev));
  DSV_CUDA(cudaDeviceGetAttribute(cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
  return DSV_OK;
}

int dsv_read_device_status(int* status) {
  DSV_REQUIRE(status != nullptr, "dsv_read_device_status: null output pointer");
  int* p = dsv::device_status_ptr();
  if (p == nullptr) return dsv::fail(DSV_E_CUDA, "device status word unavailable");
  DSV_CUDA(cudaDeviceSynchronize());
  DSV_CUDA(cudaMemcpy(status, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) {
    DSV_CUDA(cudaMemset(p, 0, sizeof(int)));
  }
  return DSV_OK;
}

}  // extern "C"
