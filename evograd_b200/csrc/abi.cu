// Library-wide services behind the C ABI: error text, tunables, device facts,
// and two small utility kernels.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "evg_common.cuh"

namespace evg {

namespace {
thread_local char g_error[512] = "";
std::mutex g_tune_mutex;
std::map<std::string, int>& tune_map() {
  static std::map<std::string, int> m;
  return m;
}
const char* const kTuneKeys[] = {
    "rows.force_generic",       "norm_bwd.blocks_per_sm", "swiglu.blocks_per_sm",
    "rope.blocks_per_sm",       "softmax_fwd.group",      "softmax_fwd.vpt",
    "softmax_fwd.threads",      "softmax_bwd.group",      "softmax_bwd.vpt",
    "softmax_bwd.threads",      "layernorm_fwd.group",    "layernorm_fwd.vpt",
    "layernorm_fwd.threads",    "layernorm_bwd.group",    "layernorm_bwd.vpt",
    "layernorm_bwd.threads",    "rmsnorm_fwd.group",      "rmsnorm_fwd.vpt",
    "rmsnorm_fwd.threads",      "rmsnorm_bwd.group",      "rmsnorm_bwd.vpt",
    "rmsnorm_bwd.threads",      "rope.generic",           "norm_bwd.no_ring",
    "norm_bwd.stages",         "norm_bwd.ring_threads",      "attention.wait_limit",
    "softmax.no_cluster",       "softmax.cluster",        "softmax.cluster_stages", "softmax.cluster_threads", "evoattention.no_stage", "evoattention.no_tc",
    "attention.two_kernel_bwd", "norm_bwd.tile_ring", "norm_bwd.no_pdl", "norm_bwd.narrow_colreduce",
};
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return fail(EVG_ELAUNCH, "%s: %s (%s)", what, cudaGetErrorName(err), cudaGetErrorString(err));
  return EVG_OK;
}

namespace {
StatusReader g_status_readers[16];
int g_status_reader_count = 0;
}  // namespace

void register_device_status(StatusReader reader) {
  if (g_status_reader_count < 16) g_status_readers[g_status_reader_count++] = reader;
}

int tune(const char* key) {
  std::lock_guard<std::mutex> lock(g_tune_mutex);
  auto& m = tune_map();
  auto it = m.find(key);
  return it == m.end() ? 0 : it->second;
}

const DeviceInfo& device_info() {
  static thread_local DeviceInfo cache[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  DeviceInfo& d = cache[dev];
  if (d.device != dev) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
      d.device = dev;
      d.sm_count = prop.multiProcessorCount;
      d.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
      d.l2_bytes = (size_t)prop.l2CacheSize;
    } else {
      cudaGetLastError();
      d.sm_count = 148;
      d.max_smem_optin = 227 * 1024;
      d.l2_bytes = 126u << 20;
    }
  }
  return d;
}

namespace {

template <typename T>
__global__ void cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<T>(src[i]);
}

__global__ void flush_kernel(uint4* __restrict__ buf, int64_t nvec, uint32_t tag) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x)
    buf[i] = make_uint4(tag, tag, tag, tag);
}

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_abi_version(void) { return EVG_ABI_VERSION; }
extern "C" const char* evg_last_error(void) { return g_error; }
extern "C" int evg_built_for_sm(void) { return 100; }

extern "C" int evg_tune_set(const char* key, int value) {
  if (!key) return fail(EVG_ENULL, "tune_set: null key");
  bool known = false;
  for (const char* k : kTuneKeys) known = known || strcmp(k, key) == 0;
  if (!known) return fail(EVG_EUNSUPPORTED, "tune_set: unknown key '%s'", key);
  std::lock_guard<std::mutex> lock(g_tune_mutex);
  if (value == 0) tune_map().erase(key);
  else tune_map()[key] = value;
  return EVG_OK;
}

extern "C" int evg_tune_get(const char* key) { return key ? tune(key) : 0; }

extern "C" int evg_cast_from_f32(const float* src, void* dst, int64_t n, int dtype, void* stream) {
  if (!src || !dst) return fail(EVG_ENULL, "cast_from_f32: null pointer argument");
  if (n < 0) return fail(EVG_EBADSHAPE, "cast_from_f32: n=%lld", (long long)n);
  if (n == 0) return EVG_OK;
  return EVG_DISPATCH_DTYPE(dtype, [&] {
    int64_t blocks = (n + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    cast_from_f32_kernel<T><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(src, (T*)dst, n);
    return check_launch("cast_from_f32");
  });
}

extern "C" int evg_flush_l2(void* buffer, int64_t bytes, void* stream) {
  if (!buffer) return fail(EVG_ENULL, "flush_l2: null buffer");
  if (bytes < 16 || !aligned16(buffer))
    return fail(EVG_EALIGN, "flush_l2: need a 16-byte aligned buffer of at least 16 bytes");
  static uint32_t tag = 0;
  flush_kernel<<<device_info().sm_count * 4, 512, 0, (cudaStream_t)stream>>>((uint4*)buffer,
                                                                            bytes / 16, ++tag);
  return check_launch("flush_l2");
}

extern "C" int evg_device_status(int reset) {
  if (cudaDeviceSynchronize() != cudaSuccess) {
    const cudaError_t err = cudaGetLastError();
    return fail(EVG_ELAUNCH, "device_status: %s", cudaGetErrorString(err));
  }
  int first = 0;
  for (int i = 0; i < g_status_reader_count; ++i) {
    const int code = g_status_readers[i](reset);
    if (code != 0 && first == 0) first = code;
  }
  if (first < 0) return fail(EVG_ELAUNCH, "device_status: cannot read a status word");
  if (first != 0)
    return fail(EVG_ETIMEOUT, "a bounded device-side wait gave up (wait id %d)", first);
  return EVG_OK;
}
