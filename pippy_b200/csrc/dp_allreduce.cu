// Data-parallel gradient all-reduce fused with the cast and the 1/(microbatches * replicas) scale, over NVLink
// peer memory (one kernel, no NCCL).  Rank r owns slice r of the bucket.
//
//   pass A   every rank casts the slices it does NOT own (fp32 gradient * scale -> bf16) into its staging buffer,
//            the wire format its peers will read.  Its own slice is never cast: pass B reads it in fp32.
//   pass B   the owner of a slice loads that slice from every peer's staging buffer (P2P loads), adds its own fp32
//            values, rounds the sum to bf16 ONCE, stores that bf16 sum into every peer's staging buffer (P2P
//            stores, over the values it has just read) and writes the same rounded value, widened to fp32, into
//            its own gradient buffer.  Every replica therefore ends with bit-identical gradients.
//   pass C   every rank widens the slices it does not own from staging back to fp32.
//
// Each gradient element is read and written twice locally (three times in a cast-everything-first design) and
// crosses NVLink once in each direction as bf16.
//
// Ranks synchronise with epoch-numbered flags in each other's memory (st.release.sys / ld.acquire.sys, bounded
// waits).  Inside one GPU there is no grid barrier: the last CTA to finish a pass (an arrival counter) publishes
// the flag, and every CTA waits for the peers' flags on its own, so the kernel makes progress even when some of its
// CTAs only become resident after others have finished (it shares the GPU with persistent GEMM kernels).
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
constexpr int ERR_PEER = 3;

struct Params {
  float* grad;                        // local fp32 gradients [n]
  __nv_bfloat16* staging[MAX_RANKS];  // every rank's staging buffer [n] (index = rank; own included)
  int* flags[MAX_RANKS];              // every rank's flag block: [0..W) ready, [W..2W) done
  int* local_counter;                 // two arrival counters (local), one per pass; zeroed before every launch
  int* err;
  long long n;
  long long wait_cycles;
  float scale;
  int rank, world;
  int epoch;          // grows by 1 per call
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

// The CTA's writes become visible system-wide, then it counts itself in; the CTA that completes the count
// publishes `epoch` at flags[q][slot] of every rank q.
__device__ __forceinline__ void arrive_and_publish(const Params& p, int* counter, int slot_base) {
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = (atomicAdd(counter, 1) + 1 == (int)gridDim.x) ? 1 : 0;
  }
  __syncthreads();
  if (s_last && threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + slot_base + p.rank, p.epoch);
  }
}

// Every CTA waits until all ranks have published `epoch` in this rank's flag block.
__device__ __forceinline__ bool wait_all_ranks(const Params& p, int slot_base) {
  bool ok = true;
  if (threadIdx.x < p.world)
    ok = wait_flag_sys(p.flags[p.rank] + slot_base + threadIdx.x, p.epoch, p.err, ERR_PEER, p.wait_cycles);
  return __syncthreads_and(ok);
}

__global__ void __launch_bounds__(THREADS) dp_allreduce_kernel(Params p) {
  const long long nvec = p.n / 8;  // 8 elements per 16-byte bf16 vector
  const long long tid = blockIdx.x * (long long)THREADS + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * THREADS;
  const int W = p.world;
  __nv_bfloat16* my_stage = p.staging[p.rank];
  const long long per = (nvec + W - 1) / W;
  const long long lo = per * p.rank < nvec ? per * p.rank : nvec;
  const long long hi = (lo + per < nvec) ? lo + per : nvec;
  const long long n_other = nvec - (hi - lo);
  // position j in [0, n_other) of the vectors this rank does not own -> vector index
  auto other = [&](long long j) { return j < lo ? j : j + (hi - lo); };

  // ---- pass A: cast + scale the slices the peers will read
  for (long long j0 = tid; j0 < n_other; j0 += nthreads * UNROLL) {
    float4 a[UNROLL], b[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long j = j0 + u * nthreads;
      if (j < n_other) {
        const long long i = other(j);
        a[u] = reinterpret_cast<const float4*>(p.grad)[2 * i];
        b[u] = reinterpret_cast<const float4*>(p.grad)[2 * i + 1];
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long j = j0 + u * nthreads;
      if (j >= n_other) continue;
      float f[8] = {a[u].x * p.scale, a[u].y * p.scale, a[u].z * p.scale, a[u].w * p.scale,
                    b[u].x * p.scale, b[u].y * p.scale, b[u].z * p.scale, b[u].w * p.scale};
      reinterpret_cast<uint4*>(my_stage)[other(j)] = pack8(f);
    }
  }
  arrive_and_publish(p, p.local_counter, 0);  // "ready"
  if (!wait_all_ranks(p, 0)) return;

  // ---- pass B: reduce the slice this rank owns, publish the rounded sum to everyone
  for (long long i0 = lo + tid; i0 < hi; i0 += nthreads * UNROLL) {
    float acc[UNROLL][8];
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
    // peer by peer, UNROLL remote vectors in flight at once (a peer load takes microseconds)
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
      const uint4 packed = pack8(acc[u]);
      float r[8];
      unpack8(packed, r);  // what the peers will hold
      reinterpret_cast<float4*>(p.grad)[2 * i] = make_float4(r[0], r[1], r[2], r[3]);
      reinterpret_cast<float4*>(p.grad)[2 * i + 1] = make_float4(r[4], r[5], r[6], r[7]);
      for (int q = 1; q < W; ++q) reinterpret_cast<uint4*>(p.staging[(p.rank + q) % W])[i] = packed;
    }
  }
  arrive_and_publish(p, p.local_counter + 1, W);  // "done"
  if (!wait_all_ranks(p, W)) return;

  // ---- pass C: slices owned by the others are now complete in my staging buffer
  for (long long j0 = tid; j0 < n_other; j0 += nthreads * UNROLL) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long j = j0 + u * nthreads;
      if (j < n_other) v[u] = reinterpret_cast<const uint4*>(my_stage)[other(j)];
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long j = j0 + u * nthreads;
      if (j >= n_other) continue;
      const long long i = other(j);
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
// bf16[n] and int[2*world] peer-mapped buffers. counter: two local ints, cleared here on the stream before the
// launch (so a call that gave up half way cannot disturb the next one).  `epoch` must grow from call to call.  A
// peer that never arrives makes the waits run out after pb_peer_wait_cycles(): the kernel then returns with the
// device error word set to 3 and the gradients of this call undefined; the context stays usable.
int pb_dp_allreduce(float* grad, void** staging, int** flags, int* counter, int* err, long long n, float scale,
                    int rank, int world, int epoch, int max_ctas, int* grid_out, void* stream_) {
  using namespace pbd;
  if (world < 1 || world > MAX_RANKS || n % 8 != 0 || rank < 0 || rank >= world) return -1;
  Params p;
  p.grad = grad;
  for (int i = 0; i < world; ++i) {
    p.staging[i] = reinterpret_cast<__nv_bfloat16*>(staging[i]);
    p.flags[i] = flags[i];
  }
  p.local_counter = counter;
  p.err = err;
  p.n = n;
  p.wait_cycles = pb_peer_wait_cycles();
  p.scale = scale;
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  long long want = (n / 8 + (long long)THREADS * UNROLL - 1) / ((long long)THREADS * UNROLL);
  int grid = (int)(want < max_ctas ? want : max_ctas);
  if (grid < 1) grid = 1;
  *grid_out = grid;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemsetAsync(counter, 0, 2 * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  dp_allreduce_kernel<<<grid, THREADS, 0, stream>>>(p);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // extern "C"
