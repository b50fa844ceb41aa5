// Host-side helpers shared by all kernels: driver entry point for tensor-map encoding, a small
// tensor-map cache, the launch counter and the library-wide device error word.
#include "tc05.cuh"

#include <mutex>
#include <unordered_map>
#include <string.h>

namespace pb {

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_encodeTiled>(p);
    }
  });
  return fn;
}

struct TmapKey {
  const void* ptr;
  uint64_t d[3];
  uint64_t pitch[2];
  uint32_t box[3];
  int elem_bytes;
  int swizzle;
  bool operator==(const TmapKey& o) const { return memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return h;
  }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
static std::mutex g_tmap_mu;

static int encode_cached(CUtensorMap* tm, const void* ptr, int elem_bytes, int rank, const uint64_t* dims,
                         const uint64_t* pitch_elems, const uint32_t* box, int swizzle128) {
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.ptr = ptr;
  key.elem_bytes = elem_bytes;
  key.swizzle = swizzle128;
  for (int i = 0; i < rank; ++i) {
    key.d[i] = dims[i];
    key.box[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) key.pitch[i] = pitch_elems[i];
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *tm = it->second;
      return 0;
    }
  }
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return -1;
  // The encoder is a driver-API call and needs a context bound to the calling thread.  A thread that has only ever
  // been told "device 0" (autograd's backward thread on the first GPU: frameworks skip cudaSetDevice when the
  // target is already the current device) has none until its first runtime call, and the encoder then answers
  // CUDA_ERROR_INVALID_CONTEXT.  cudaFree(0) binds the primary context; once per thread.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(0);
    context_bound = true;
  }
  cuuint64_t gdim[3];
  cuuint64_t gstride[2];
  cuuint32_t bx[3];
  cuuint32_t estr[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) gstride[i] = pitch_elems[i] * (uint64_t)elem_bytes;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  CUresult r = enc(tm, dt, (cuuint32_t)rank, const_cast<void*>(ptr), gdim, gstride, bx, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return (int)r;
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    if (g_tmap_cache.size() > 8192) g_tmap_cache.clear();
    g_tmap_cache.emplace(key, *tm);
  }
  return 0;
}

int make_tmap_2d(CUtensorMap* tm, const void* ptr, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t pitch_elems, uint32_t box_inner, uint32_t box_outer, int swizzle128) {
  uint64_t dims[2] = {inner, outer};
  uint64_t pitch[1] = {pitch_elems};
  uint32_t box[2] = {box_inner, box_outer};
  return encode_cached(tm, ptr, elem_bytes, 2, dims, pitch, box, swizzle128);
}

int make_tmap_bf16_2d(CUtensorMap* tm, const void* ptr, uint64_t inner, uint64_t outer, uint64_t pitch_elems,
                      uint32_t box_inner, uint32_t box_outer) {
  return make_tmap_2d(tm, ptr, 2, inner, outer, pitch_elems, box_inner, box_outer, 1);
}

int make_tmap_bf16_3d(CUtensorMap* tm, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1_elems,
                      uint64_t pitch2_elems, uint32_t box0, uint32_t box1, uint32_t box2) {
  uint64_t dims[3] = {d0, d1, d2};
  uint64_t pitch[2] = {pitch1_elems, pitch2_elems};
  uint32_t box[3] = {box0, box1, box2};
  return encode_cached(tm, ptr, 2, 3, dims, pitch, box, 1);
}

}  // namespace pb

// ---------------------------------------------------------------- exported utilities
static long long g_launch_count = 0;

extern "C" {

// Number of kernels this library has launched since load (or since the last reset).
long long pb_launch_count() { return g_launch_count; }
void pb_launch_count_reset() { g_launch_count = 0; }
void pb_count_launch(int n) { g_launch_count += n; }

// Limit of the peer-flag waits in SM cycles (about 3 s by default: a peer may lag by a whole schedule action).
static long long g_peer_wait_cycles = 6000000000LL;
long long pb_peer_wait_cycles() { return g_peer_wait_cycles; }
// `ms` milliseconds at a nominal 2 GHz SM clock; a lower clock only makes the wait longer.  ms <= 0 restores the default.
void pb_set_peer_wait_ms(double ms) { g_peer_wait_cycles = ms > 0 ? (long long)(ms * 2.0e6) : 6000000000LL; }

// Debug build (-DPB_BOUNDS_CHECK): the error word that out-of-range indices are reported to (see dbgcheck.cuh).
static int* g_debug_err = nullptr;
int* pb_debug_err_ptr() { return g_debug_err; }
void pb_set_debug_err_ptr(int* dev_ptr) { g_debug_err = dev_ptr; }
int pb_bounds_check_enabled() {
#ifdef PB_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

int pb_device_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}

const char* pb_last_cuda_error() { return cudaGetErrorString(cudaGetLastError()); }

}  // extern "C"
