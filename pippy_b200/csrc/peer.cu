// Peer (symmetric) memory: plain cudaMalloc allocations exported with CUDA IPC so that every rank of a node can map
// every other rank's buffer and kernels can load/store it directly over NVLink.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "peer.cuh"

extern "C" void pb_count_launch(int n);

namespace pbpeer {

using namespace pbp;
constexpr int MAX_RANKS = 8;
constexpr int THREADS = 512;
constexpr int UNROLL = 4;

struct GatherParams {
  const uint4* src[MAX_RANKS];  // every rank's shard (peer mapped), `vecs` 16-byte vectors each
  int* flags[MAX_RANKS];        // every rank's flag block: [0, W) "shard ready", [W, 2W) "done reading"
  uint4* dst;                   // local [W * vecs]
  int* counter;                 // local arrival counter, zeroed before the launch
  int* err;
  long long vecs;
  long long wait_cycles;
  int rank, world, epoch;
};

// All-gather over peer memory: every rank pulls the other ranks' shards with plain vector loads over NVLink (its own
// shard is copied locally).  The shards must stay untouched until every rank has passed the closing handshake.
__global__ void __launch_bounds__(THREADS) peer_allgather_kernel(GatherParams p) {
  const int W = p.world;
  if (blockIdx.x == 0 && (int)threadIdx.x < W) st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);
  bool ok = true;
  if ((int)threadIdx.x < W) ok = wait_flag_sys(p.flags[p.rank] + threadIdx.x, p.epoch, p.err, 3, p.wait_cycles);
  if (!__syncthreads_and(ok)) return;
  const long long tid = blockIdx.x * (long long)THREADS + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * THREADS;
  for (int q = 0; q < W; ++q) {
    const int r = (p.rank + q) % W;  // own shard first, then the peers round-robin
    const uint4* src = p.src[r];
    uint4* dst = p.dst + (long long)r * p.vecs;
    for (long long i0 = tid; i0 < p.vecs; i0 += nthreads * UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (i0 + u * nthreads < p.vecs) v[u] = src[i0 + u * nthreads];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (i0 + u * nthreads < p.vecs) dst[i0 + u * nthreads] = v[u];
    }
  }
  // the last CTA to finish tells every peer that this rank no longer reads their shards
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.counter, 1) + 1 == (int)gridDim.x) ? 1 : 0;
  __syncthreads();
  if (s_last) {
    if ((int)threadIdx.x < W) st_release_sys(p.flags[threadIdx.x] + W + p.rank, p.epoch);
    ok = true;
    if ((int)threadIdx.x < W) ok = wait_flag_sys(p.flags[p.rank] + W + threadIdx.x, p.epoch, p.err, 3, p.wait_cycles);
    __syncthreads_and(ok);
  }
}

}  // namespace pbpeer

extern "C" {

// Allocates `bytes` of zeroed device memory. Returns 0 on success.
int pb_peer_alloc(unsigned long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*out, 0, bytes);
  return (int)e;
}

int pb_peer_free(void* p) { return (int)cudaFree(p); }

// Writes the 64-byte IPC handle of allocation `p` to `handle_out`.
int pb_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

int pb_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}

int pb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

int pb_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

// dst[W * bytes] = concatenation of every rank's `bytes`-long shard.  src / flags: host arrays of `world` device
// pointers (peer mapped; this rank's own included); flags[r] is int[2 * world], zero-initialised once; `epoch` grows
// by one per call on every rank.  bytes % 16 == 0.  The kernel returns on this rank only after every rank has
// finished reading this rank's shard, so the caller may overwrite it right after.
int pb_peer_allgather(void* dst, void** src, int** flags, int* counter, int* err, long long bytes, int rank,
                      int world, int epoch, int ctas, void* stream_) {
  using namespace pbpeer;
  if (world < 1 || world > MAX_RANKS || bytes <= 0 || bytes % 16 != 0 || rank < 0 || rank >= world) return -1;
  GatherParams p;
  for (int i = 0; i < world; ++i) {
    p.src[i] = reinterpret_cast<const uint4*>(src[i]);
    p.flags[i] = flags[i];
  }
  p.dst = reinterpret_cast<uint4*>(dst);
  p.counter = counter;
  p.err = err;
  p.vecs = bytes / 16;
  p.wait_cycles = pb_peer_wait_cycles();
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  long long want = (p.vecs + (long long)THREADS * UNROLL - 1) / ((long long)THREADS * UNROLL);
  int grid = (int)(want < ctas ? want : ctas);
  if (grid < 1) grid = 1;
  peer_allgather_kernel<<<grid, THREADS, 0, stream>>>(p);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

// Same-process "peers" (several devices driven by one process, used by tests): enable direct access.
int pb_enable_peer_access(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return (int)e;
}

}  // extern "C"
