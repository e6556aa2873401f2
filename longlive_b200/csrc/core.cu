// Library-wide plumbing: error strings, device status word, cached device properties.
#include <atomic>
#include <cstring>
#include <mutex>

#include <cstdlib>

#include "common.cuh"

namespace llnv {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return LLNV_E_CUDA;
}

static constexpr int kMaxDevices = 64;
static unsigned int* g_status[kMaxDevices] = {};
static int g_sms[kMaxDevices] = {};
static std::mutex g_mu;

unsigned int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_status[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, sizeof(unsigned int) * 4) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(unsigned int) * 4) != cudaSuccess) return nullptr;
    g_status[dev] = p;
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

namespace {
std::atomic<unsigned long long> g_launches{0};
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

namespace {
thread_local int g_amax_accumulate = 0;
int g_pdl = -1;                        // -1: not decided yet (environment LLNV_PDL=1 turns it on; default off)
}

bool amax_accumulate(int which) { return (g_amax_accumulate & which) != 0; }

bool pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("LLNV_PDL");
    g_pdl = (e && e[0] == '1') ? 1 : 0;
  }
  return g_pdl != 0;
}

}  // namespace llnv

extern "C" int llnv_set_pdl(int on) {
  const int before = llnv::pdl_enabled() ? 1 : 0;
  llnv::g_pdl = on ? 1 : 0;
  return before;
}

extern "C" int llnv_set_amax_accumulate(int on) {
  const int before = llnv::g_amax_accumulate;
  llnv::g_amax_accumulate = on & 3;
  return before;
}

extern "C" int llnv_version(void) { return 2; }

extern "C" unsigned long long llnv_launch_count(void) { return llnv::g_launches.load(std::memory_order_relaxed); }

extern "C" int llnv_init_device(void) {
  if (!llnv::device_status_word()) {
    llnv::set_error("llnv_init_device: could not allocate the device status word");
    return LLNV_E_CUDA;
  }
  llnv::sm_count();
  return LLNV_OK;
}

extern "C" const char* llnv_last_error(void) { return llnv::g_err; }

extern "C" int llnv_check_status(llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  unsigned int* w = llnv::device_status_word();
  if (!w) {
    llnv::set_error("llnv_check_status: no status word on this device");
    return LLNV_E_CUDA;
  }
  unsigned int host[4] = {0, 0, 0, 0};
  LLNV_CUDA(cudaMemcpyAsync(host, w, sizeof(host), cudaMemcpyDeviceToHost, stream));
  LLNV_CUDA(cudaStreamSynchronize(stream));
  if (host[0] != 0) {
    LLNV_CUDA(cudaMemsetAsync(w, 0, sizeof(host), stream));
    llnv::set_error("device-side bounded wait gave up: code=%u where=%u block=%u iter=%u", host[0], host[1], host[2], host[3]);
    return LLNV_E_TIMEOUT;
  }
  return LLNV_OK;
}
