// Data-parallel gradient all-reduce fused with the cast and the 1/(microbatches * replicas) scale, over NVLink
// peer memory (one kernel, no NCCL):
//
//   phase 0  every rank casts its fp32 gradient bucket * scale to bf16 into its staging buffer (the wire format)
//   phase 1  rank r owns slice r of the bucket: it loads that slice from every peer's staging buffer (P2P loads),
//            adds its own fp32 values, writes the fp32 sum into its own gradient buffer and stores the bf16 sum
//            into every peer's staging buffer (P2P stores)
//   phase 2  every rank converts the slices it does not own from staging back to fp32
//
// Ranks synchronise with epoch-numbered flags in each other's memory (st.release.sys / ld.acquire.sys, bounded
// waits); CTAs of one GPU synchronise with a counter barrier (the grid is sized to be co-resident).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "peer.cuh"

extern "C" void pb_count_launch(int n);

namespace pbd {

using namespace pbp;

constexpr int MAX_RANKS = 8;
constexpr int THREADS = 512;
constexpr int UNROLL = 4;  // independent 8-element groups per thread and loop trip: the passes are latency-bound otherwise

struct Params {
  float* grad;                        // local fp32 gradients [n]
  __nv_bfloat16* staging[MAX_RANKS];  // every rank's staging buffer [n] (index = rank; own included)
  int* flags[MAX_RANKS];              // every rank's flag block: [0..W) ready, [W..2W) done
  int* local_counter;                 // grid barrier counter (local)
  int* err;
  long long n;
  float scale;
  int rank, world;
  int epoch;          // grows by 1 per call
  int barrier_base;   // local_counter value before this call
};

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

__global__ void __launch_bounds__(THREADS) dp_allreduce_kernel(Params p) {
  const long long nvec = p.n / 8;  // 8 elements per 16-byte bf16 vector
  const long long tid = blockIdx.x * (long long)THREADS + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * THREADS;
  const int W = p.world;
  __nv_bfloat16* my_stage = p.staging[p.rank];
  int bar = p.barrier_base;

  // ---- phase 0: cast + scale into the wire buffer
  for (long long i0 = tid; i0 < nvec; i0 += nthreads * UNROLL) {
    float4 a[UNROLL], b[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * nthreads;
      if (i < nvec) {
        a[u] = reinterpret_cast<const float4*>(p.grad)[2 * i];
        b[u] = reinterpret_cast<const float4*>(p.grad)[2 * i + 1];
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * nthreads;
      if (i >= nvec) continue;
      float f[8] = {a[u].x * p.scale, a[u].y * p.scale, a[u].z * p.scale, a[u].w * p.scale,
                    b[u].x * p.scale, b[u].y * p.scale, b[u].z * p.scale, b[u].w * p.scale};
      reinterpret_cast<uint4*>(my_stage)[i] = pack8(f);
    }
  }
  __threadfence_system();
  bar += gridDim.x;
  if (!grid_barrier(p.local_counter, bar, p.err, 3)) return;
  if (blockIdx.x == 0 && threadIdx.x < W) st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);  // "ready"
  bool ok = true;
  if (threadIdx.x < W) ok = wait_flag_sys(p.flags[p.rank] + threadIdx.x, p.epoch, p.err, 3);
  if (!__syncthreads_and(ok)) return;

  // ---- phase 1: reduce the slice this rank owns, publish the sum to everyone
  const long long per = (nvec + W - 1) / W;
  const long long lo = per * p.rank;
  const long long hi = (lo + per < nvec) ? lo + per : nvec;
  for (long long i0 = lo + tid; i0 < hi; i0 += nthreads * UNROLL) {
    float acc[UNROLL][8];
    // own fp32 values and, peer by peer, UNROLL remote vectors in flight at once (a peer load takes microseconds)
    {
      float4 a[UNROLL], b[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < hi) {
          a[u] = reinterpret_cast<const float4*>(p.grad)[2 * i];
          b[u] = reinterpret_cast<const float4*>(p.grad)[2 * i + 1];
        } else {
          a[u] = b[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        acc[u][0] = a[u].x * p.scale; acc[u][1] = a[u].y * p.scale; acc[u][2] = a[u].z * p.scale;
        acc[u][3] = a[u].w * p.scale; acc[u][4] = b[u].x * p.scale; acc[u][5] = b[u].y * p.scale;
        acc[u][6] = b[u].z * p.scale; acc[u][7] = b[u].w * p.scale;
      }
    }
    for (int q = 1; q < W; ++q) {
      const uint4* src = reinterpret_cast<const uint4*>(p.staging[(p.rank + q) % W]);
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * nthreads;
        v[u] = (i < hi) ? src[i] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        float f[8];
        unpack8(v[u], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[u][j] += f[j];
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * nthreads;
      if (i >= hi) continue;
      reinterpret_cast<float4*>(p.grad)[2 * i] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
      reinterpret_cast<float4*>(p.grad)[2 * i + 1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
      const uint4 packed = pack8(acc[u]);
      for (int q = 1; q < W; ++q) reinterpret_cast<uint4*>(p.staging[(p.rank + q) % W])[i] = packed;
    }
  }
  __threadfence_system();
  bar += gridDim.x;
  if (!grid_barrier(p.local_counter, bar, p.err, 3)) return;
  if (blockIdx.x == 0 && threadIdx.x < W) st_release_sys(p.flags[threadIdx.x] + W + p.rank, p.epoch);  // "done"
  ok = true;
  if (threadIdx.x < W) ok = wait_flag_sys(p.flags[p.rank] + W + threadIdx.x, p.epoch, p.err, 3);
  if (!__syncthreads_and(ok)) return;

  // ---- phase 2: slices owned by the others are now complete in my staging buffer
  for (long long i0 = tid; i0 < nvec; i0 += nthreads * UNROLL) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * nthreads;
      if (i < nvec && !(i >= lo && i < hi)) v[u] = reinterpret_cast<const uint4*>(my_stage)[i];
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * nthreads;
      if (i >= nvec || (i >= lo && i < hi)) continue;
      float f[8];
      unpack8(v[u], f);
      reinterpret_cast<float4*>(p.grad)[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
      reinterpret_cast<float4*>(p.grad)[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
}

}  // namespace pbd

extern "C" {

// grad: local fp32 [n] (n % 8 == 0). staging/flags: arrays of `world` device pointers (this rank's own included) to
// bf16[n] and int[2*world] peer-mapped buffers. counter: local int (zero-initialised once); the caller passes its
// current value in `barrier_base` and adds 2 * grid (returned through *grid_out) afterwards.
int pb_dp_allreduce(float* grad, void** staging, int** flags, int* counter, int* err, long long n, float scale,
                    int rank, int world, int epoch, int barrier_base, int max_ctas, int* grid_out, void* stream_) {
  using namespace pbd;
  if (world < 1 || world > MAX_RANKS || n % 8 != 0) return -1;
  Params p;
  p.grad = grad;
  for (int i = 0; i < world; ++i) {
    p.staging[i] = reinterpret_cast<__nv_bfloat16*>(staging[i]);
    p.flags[i] = flags[i];
  }
  p.local_counter = counter;
  p.err = err;
  p.n = n;
  p.scale = scale;
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  p.barrier_base = barrier_base;
  long long want = (n / 8 + THREADS - 1) / THREADS;
  int grid = (int)(want < max_ctas ? want : max_ctas);
  if (grid < 1) grid = 1;
  *grid_out = grid;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  dp_allreduce_kernel<<<grid, THREADS, 0, stream>>>(p);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // extern "C"
