// mz_decode_attention_static: decode attention whose scratch lives in a static device array,
// for callers that may not allocate device memory.
#include <mutex>

#include "mz_decode.cuh"

int mz_decode_plan_info(const mz_decode_args* args, size_t* ws_bytes, int* needs_tables);

// The scratch itself.  In host code this name is only a stand-in for the symbol: it is not a
// device address and must never be handed to a kernel; the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[MZ_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the array on the current device (looked up once per device).
int scratch_address(void** out) {
  int dev = 0;
  MZ_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return mz_fail(MZ_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return mz_fail(MZ_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return MZ_OK;
}
}  // namespace

extern "C" int mz_decode_attention_static(const mz_decode_args* args, void* stream) {
  MZ_RANGE("mz_decode_attention_static");
  MZ_REQUIRE(args != nullptr, "args is NULL");
  size_t need = 0;
  int needs_tables = 0;
  int rc = mz_decode_plan_info(args, &need, &needs_tables);
  if (rc) return rc;
  if (needs_tables)
    return mz_fail(MZ_ERR_UNSUPPORTED,
                   "this shape runs on the shape-generic kernel, whose lookup tables are allocated on first use; "
                   "mz_decode_attention_static serves head_dim 128, group 32/64/128, 1/2/4/8 query heads per kv head");
  if (need > (size_t)MZ_STATIC_SCRATCH_BYTES)
    return mz_fail(MZ_ERR_WORKSPACE, "request needs %zu bytes of scratch, the static array holds %u; lower `splits` or the batch",
                   need, (unsigned)MZ_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  if ((rc = scratch_address(&scratch))) return rc;
  mz_decode_args local = *args;
  local.workspace = scratch;
  local.workspace_bytes = MZ_STATIC_SCRATCH_BYTES;
  return mz_decode_attention(&local, stream);
}
