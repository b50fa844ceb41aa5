// Device-side primitives for kernels that talk to other GPUs through peer-mapped memory:
// system-scope flag signalling with bounded waits, and an intra-GPU grid barrier.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pbp {

constexpr long long kPeerWaitCycles = 6000000000LL;  // ~3 s of SM clock: peers may legitimately lag by a whole action

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Spins until *p >= target (system scope). Returns false (and sets *err) when `limit` SM cycles have passed, or as
// soon as another wait of this GPU has already reported an error.
__device__ __forceinline__ bool wait_flag_sys(const int* p, int target, int* err, int err_code,
                                              long long limit = kPeerWaitCycles) {
  if (ld_acquire_sys(p) >= target) return true;
  const long long t0 = clock64();
  while (true) {
    for (int i = 0; i < 64; ++i) {
      if (ld_acquire_sys(p) >= target) return true;
      __nanosleep(100);
    }
    if (*reinterpret_cast<volatile int*>(err) != 0) return false;
    if (clock64() - t0 > limit) {
      atomicExch(err, err_code);
      return false;
    }
  }
}
__device__ __forceinline__ bool wait_flag_gpu(const int* p, int target, int* err, int err_code,
                                              long long limit = kPeerWaitCycles) {
  if (ld_acquire_gpu(p) >= target) return true;
  const long long t0 = clock64();
  while (true) {
    for (int i = 0; i < 64; ++i) {
      if (ld_acquire_gpu(p) >= target) return true;
      __nanosleep(40);
    }
    if (*reinterpret_cast<volatile int*>(err) != 0) return false;
    if (clock64() - t0 > limit) {
      atomicExch(err, err_code);
      return false;
    }
  }
}

// Barrier over all CTAs of a grid whose CTAs are co-resident. `counter` only ever grows; the caller passes the
// value it must reach (calls so far * gridDim.x). Returns false on timeout.
__device__ __forceinline__ bool grid_barrier(int* counter, int target, int* err, int err_code,
                                             long long limit = kPeerWaitCycles) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1);
    ok = wait_flag_gpu(counter, target, err, err_code, limit);
  }
  ok = __syncthreads_and(ok);
  return ok;
}

}  // namespace pbp

// Host side (common.cu): the limit that launchers hand to the waits above, in SM cycles.  pb_set_peer_wait_ms
// changes it for the whole library (tests use a few milliseconds to let a wait run out on purpose).
extern "C" long long pb_peer_wait_cycles();
