// Host-side helpers shared by the launch wrappers: per-device cached properties and
// once-per-device set-up (function attributes such as the dynamic shared-memory opt-in belong
// to one device, so a process that drives several GPUs must repeat them on each).
#pragma once
#include <cuda_runtime.h>

namespace tb200 {

constexpr int MAX_DEVICES = 64;

inline int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
  return dev;
}

// Number of SMs of the current device (148 on a B200), queried once per device.
inline int sm_count() {
  static int sms[MAX_DEVICES] = {0};
  const int dev = current_device();
  if (dev < 0) return 148;
  if (sms[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    sms[dev] = v;
  }
  return sms[dev];
}

// `static OncePerDevice once; if (once.need()) { ...; once.done(); }`
struct OncePerDevice {
  bool flags[MAX_DEVICES] = {false};
  bool need() const {
    const int dev = current_device();
    return dev < 0 || !flags[dev];
  }
  void done() {
    const int dev = current_device();
    if (dev >= 0) flags[dev] = true;
  }
};

}  // namespace tb200
