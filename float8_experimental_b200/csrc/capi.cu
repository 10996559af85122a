// Status strings, device checks and per-thread CUDA error text for the C ABI.
#include <mutex>
#include <string>

#include "common.cuh"

namespace f8b200 {

static thread_local std::string t_last_error;

int record_cuda_error(cudaError_t e) {
  if (e == cudaSuccess) return F8B200_OK;
  t_last_error = std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e);
  return F8B200_ERR_LAUNCH;
}

namespace {
struct DeviceInfo {
  int major = -1;
  int sms = 0;
};
DeviceInfo g_info[kMaxDevices];
std::mutex g_per_device_mutex;
std::mutex g_info_mutex;

const DeviceInfo* current_info() {
  int dev = 0;
  if (record_cuda_error(cudaGetDevice(&dev)) != F8B200_OK || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_info_mutex);
  DeviceInfo& d = g_info[dev];
  if (d.major < 0) {
    int major = 0, sms = 0;
    if (record_cuda_error(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != F8B200_OK) return nullptr;
    if (record_cuda_error(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != F8B200_OK) return nullptr;
    d.major = major;
    d.sms = sms;
  }
  return &d;
}
}  // namespace

int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}
void per_device_lock() { g_per_device_mutex.lock(); }
void per_device_unlock() { g_per_device_mutex.unlock(); }

int sm_count() {
  const DeviceInfo* d = current_info();
  return (d != nullptr && d->sms > 0) ? d->sms : 148;
}

}  // namespace f8b200

extern "C" const char* f8b200_status_string(int status) {
  switch (status) {
    case F8B200_OK: return "ok";
    case F8B200_ERR_BAD_ARG: return "bad argument (null pointer, negative size or unknown enum)";
    case F8B200_ERR_ALIGNMENT: return "pointer or leading dimension is not sufficiently aligned";
    case F8B200_ERR_ARCH: return "current CUDA device is not compute capability 10.x (B200)";
    case F8B200_ERR_LAUNCH: return "CUDA error at launch (see f8b200_last_cuda_error)";
    case F8B200_ERR_DRIVER: return "tensor-map encode failed or driver entry point missing";
    case F8B200_ERR_UNSUPPORTED: return "request not supported by the kernels";
    case F8B200_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    default: return "unknown status";
  }
}

extern "C" int f8b200_device_check(void) {
  const f8b200::DeviceInfo* d = f8b200::current_info();
  if (d == nullptr) return F8B200_ERR_LAUNCH;
  return d->major == 10 ? F8B200_OK : F8B200_ERR_ARCH;
}

extern "C" const char* f8b200_last_cuda_error(void) { return f8b200::t_last_error.c_str(); }
