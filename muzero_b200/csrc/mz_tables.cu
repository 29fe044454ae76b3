// Error text, version, and the per-device lookup tables of the compander.
#include <cmath>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "mz_common.cuh"

static thread_local char g_error[512] = "";

int mz_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

extern "C" int mz_version(void) { return 100; }

extern "C" int mz_last_error(char* buf, int len) {
  if (!buf || len <= 0) return (int)strlen(g_error);
  strncpy(buf, g_error, (size_t)len - 1);
  buf[len - 1] = 0;
  return (int)strlen(buf);
}

// Checked build: the record the guarded accesses write (current device).  Synchronizes the device.
#ifdef MZ_BOUNDS
__device__ MzBoundsRecord g_mz_bounds = {0ull, 0ll, 0ll, 0, 0};
#endif
extern "C" long long mz_bounds_violations(long long* first_index, long long* first_extent, int* first_site, int reset) {
#ifdef MZ_BOUNDS
  MzBoundsRecord r;
  if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpyFromSymbol(&r, g_mz_bounds, sizeof(r)) != cudaSuccess) {
    mz_fail(MZ_ERR_CUDA, "reading the bounds record failed: %s", cudaGetErrorString(cudaGetLastError()));
    return -2;
  }
  if (first_index) *first_index = r.index;
  if (first_extent) *first_extent = r.extent;
  if (first_site) *first_site = r.site;
  if (reset) {
    const MzBoundsRecord zero = {0ull, 0ll, 0ll, 0, 0};
    cudaMemcpyToSymbol(g_mz_bounds, &zero, sizeof(zero));
  }
  return (long long)r.count;
#else
  (void)first_index; (void)first_extent; (void)first_site; (void)reset;
  return -1;   // not a checked build
#endif
}

// ---------------------------------------------------------------------------
namespace {
std::mutex g_mu;
// (device, bits, alpha bits) -> device table
std::map<std::tuple<int, int, uint32_t>, float*> g_expand;
// (device, dtype, alpha bits) -> (device table, entries)
std::map<std::tuple<int, int, uint32_t>, std::pair<uint16_t*, int>> g_compand;

uint32_t fbits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float round_to(int dt, float v) {
  if (dt == MZ_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dt == MZ_F16) return __half2float(__float2half_rn(v));
  return v;
}
uint16_t bits_of(int dt, float v) {
  if (dt == MZ_BF16) { __nv_bfloat16 b = __float2bfloat16_rn(v); uint16_t u; memcpy(&u, &b, 2); return u; }
  __half h = __float2half_rn(v); uint16_t u; memcpy(&u, &h, 2); return u;
}
float value_of(int dt, uint16_t u) {
  if (dt == MZ_BF16) { uint32_t w = ((uint32_t)u) << 16; float f; memcpy(&f, &w, 4); return f; }
  __half h; memcpy(&h, &u, 2); return __half2float(h);
}

void build_expand_host(int bits, float alpha, std::vector<float>& t) {
  const int tw = 1 << bits;
  t.assign((size_t)tw * tw, 0.0f);
  const float lb = (float)log1p((double)alpha);
  for (int den = 0; den < tw; ++den) {
    const float d = (float)(den < 1 ? 1 : den);
    for (int num = 0; num < tw; ++num) {
      float frac = (float)num / d;
      frac = frac < 0.f ? 0.f : (frac > 1.f ? 1.f : frac);
      const float arg = frac * lb;
      const float e = (float)expm1((double)arg);
      t[(size_t)den * tw + num] = e / alpha;
    }
  }
}

int upload_expand(int dev, int bits, float alpha, const float* host) {
  const size_t n = (size_t)1 << (2 * bits);
  auto key = std::make_tuple(dev, bits, fbits(alpha));
  float* d = nullptr;
  auto it = g_expand.find(key);
  if (it != g_expand.end()) d = it->second;
  else MZ_CUDA(cudaMalloc(&d, n * sizeof(float)));
  MZ_CUDA(cudaMemcpy(d, host, n * sizeof(float), cudaMemcpyHostToDevice));
  g_expand[key] = d;
  return MZ_OK;
}
}  // namespace

extern "C" int mz_set_expand_table(int bits, float alpha, const float* host_table) {
  MZ_REQUIRE(bits >= 1 && bits <= 8, "bits must be 1..8, got %d", bits);
  MZ_REQUIRE(host_table != nullptr, "host_table is NULL");
  MZ_REQUIRE(alpha > 0.f, "alpha must be > 0");
  int dev = 0;
  MZ_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  return upload_expand(dev, bits, alpha, host_table);
}

int mz_get_expand_table(int bits, float alpha, const float** dev_table) {
  int dev = 0;
  MZ_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  auto key = std::make_tuple(dev, bits, fbits(alpha));
  auto it = g_expand.find(key);
  if (it == g_expand.end()) {
    std::vector<float> host;
    build_expand_host(bits, alpha, host);
    int rc = upload_expand(dev, bits, alpha, host.data());
    if (rc != MZ_OK) return rc;
    it = g_expand.find(key);
  }
  *dev_table = it->second;
  return MZ_OK;
}

int mz_get_compand_table(int dtype, float alpha, const uint16_t** dev_table, int* n_entries) {
  int dev = 0;
  MZ_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  auto key = std::make_tuple(dev, dtype, fbits(alpha));
  auto it = g_compand.find(key);
  if (it == g_compand.end()) {
    const int n = (int)bits_of(dtype, 1.0f) + 1;  // every value in [0,1]
    std::vector<uint16_t> host((size_t)n);
    const float lb = (float)log1p((double)alpha);
    for (int i = 0; i < n; ++i) {
      const float p = value_of(dtype, (uint16_t)i);
      const float ap = round_to(dtype, alpha * p);
      const float l = round_to(dtype, (float)log1p((double)ap));
      host[(size_t)i] = bits_of(dtype, l / lb);
    }
    uint16_t* d = nullptr;
    MZ_CUDA(cudaMalloc(&d, (size_t)n * sizeof(uint16_t)));
    MZ_CUDA(cudaMemcpy(d, host.data(), (size_t)n * sizeof(uint16_t), cudaMemcpyHostToDevice));
    it = g_compand.emplace(key, std::make_pair(d, n)).first;
  }
  *dev_table = it->second.first;
  *n_entries = it->second.second;
  return MZ_OK;
}
