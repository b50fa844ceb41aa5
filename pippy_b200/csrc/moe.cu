// Expert-parallel MoE data movement over NVLink peer memory.
//
//   moe_slots     : position of every (token, k) assignment inside its expert's group (atomic histogram)
//   moe_dispatch  : permute + all-to-all in one kernel: each assignment's token row (optionally scaled) is stored
//                   straight into the owning rank's expert-grouped receive buffer (P2P stores)
//   moe_combine   : all-to-all + un-permute + weighted top-k sum in one kernel: each token pulls its k expert rows
//                   from the ranks that computed them (P2P loads), fp32 accumulate; can keep the pulled rows
//   moe_rowdot    : dots[t, k] = <dy[t], rows[t, k]>  (gradient of the router weights)
//
// Ranks synchronise with epoch flags in each other's memory (bounded waits), CTAs of a rank with a counter barrier.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "peer.cuh"

extern "C" void pb_count_launch(int n);

namespace pbmoe {

using namespace pbp;
constexpr int MAX_RANKS = 8;
constexpr int THREADS = 256;
constexpr int UNROLL = 4;   // 16-byte vectors a lane keeps in flight per source row
constexpr int MAX_TOPK = 4;

struct Comm {
  int* flags[MAX_RANKS];  // every rank's flag block: [0,W) phase A, [W,2W) phase B
  int* counter;           // local grid-barrier counter (zeroed before launch)
  int* err;
  int rank, world, epoch;
};

__global__ void moe_slots_kernel(const int* __restrict__ expert, int* __restrict__ counts, int* __restrict__ slot,
                                 int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) slot[i] = atomicAdd(&counts[expert[i]], 1);
}

__device__ __forceinline__ bool handshake(const Comm& c, int phase) {
  // announce phase to every peer, then wait until every peer announced it
  if (blockIdx.x == 0 && (int)threadIdx.x < c.world && (int)threadIdx.x != c.rank)
    st_release_sys(c.flags[threadIdx.x] + phase * c.world + c.rank, c.epoch);
  bool ok = true;
  if ((int)threadIdx.x < c.world && (int)threadIdx.x != c.rank)
    ok = wait_flag_sys(c.flags[c.rank] + phase * c.world + threadIdx.x, c.epoch, c.err, 3);
  return __syncthreads_and(ok);
}

// x: [T, H] bf16; expert/slot: [T*k]; dst_base[e]: first row of this rank's block inside expert e's group on its
// owner; recv[r]: every rank's receive buffer [rows, H]; scale: optional [T*k] fp32.
__global__ void __launch_bounds__(THREADS) moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const int* __restrict__ expert,
                                                               const int* __restrict__ slot,
                                                               const int* __restrict__ dst_base,
                                                               const float* __restrict__ scale,
                                                               __nv_bfloat16* const* __restrict__ recv_ptrs, int T,
                                                               int k, int H, int experts_per_rank, Comm c) {
  __shared__ __nv_bfloat16* s_recv[MAX_RANKS];
  if (threadIdx.x < MAX_RANKS) s_recv[threadIdx.x] = threadIdx.x < c.world ? recv_ptrs[threadIdx.x] : nullptr;
  __syncthreads();
  if (!handshake(c, 0)) return;  // every peer's receive buffer is free
  const int warps_per_block = THREADS / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vec = H / 8;
  const long long n = (long long)T * k;
  for (long long a = blockIdx.x * warps_per_block + warp; a < n; a += (long long)gridDim.x * warps_per_block) {
    const int e = expert[a];
    const int d = e / experts_per_rank;
    const long long row = (long long)dst_base[e] + slot[a];
    const uint4* src = reinterpret_cast<const uint4*>(x + (a / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(s_recv[d] + row * H);
    const float s = scale ? scale[a] : 1.f;
    // four independent 16-byte loads per lane before the first store: the copy is latency-bound otherwise
    for (int v0 = lane; v0 < vec; v0 += 32 * UNROLL) {
      uint4 u[UNROLL];
#pragma unroll
      for (int i = 0; i < UNROLL; ++i)
        if (v0 + i * 32 < vec) u[i] = __ldg(src + v0 + i * 32);
#pragma unroll
      for (int i = 0; i < UNROLL; ++i) {
        if (v0 + i * 32 >= vec) continue;
        if (scale) {
          __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u[i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(b[j]);
            b[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
          }
        }
        dst[v0 + i * 32] = u[i];
      }
    }
  }
  __threadfence_system();
  if (!grid_barrier(c.counter, (int)gridDim.x, c.err, 3)) return;
  handshake(c, 1);  // everything destined to me has landed when every peer reports "pushed"
}

// out[t] = sum_k w[t,k] * y[d(t,k)][row(t,k)]; rowmap: [T*k] row inside the owner's buffer; optional save [T*k, H].
__global__ void __launch_bounds__(THREADS) moe_combine_kernel(__nv_bfloat16* __restrict__ out,
                                                              const int* __restrict__ expert,
                                                              const int* __restrict__ slot,
                                                              const int* __restrict__ dst_base,
                                                              const float* __restrict__ weight,
                                                              __nv_bfloat16* const* __restrict__ y_ptrs,
                                                              __nv_bfloat16* __restrict__ save, int T, int k, int H,
                                                              int experts_per_rank, Comm c) {
  __shared__ __nv_bfloat16* s_y[MAX_RANKS];
  if (threadIdx.x < MAX_RANKS) s_y[threadIdx.x] = threadIdx.x < c.world ? y_ptrs[threadIdx.x] : nullptr;
  __syncthreads();
  if (!handshake(c, 0)) return;  // every peer's expert outputs are complete
  const int warps_per_block = THREADS / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vec = H / 8;
  for (long long t = blockIdx.x * warps_per_block + warp; t < T; t += (long long)gridDim.x * warps_per_block) {
    // the k source rows of this token: looked up once, not once per vector
    const uint4* rows[MAX_TOPK];
    float w[MAX_TOPK];
#pragma unroll
    for (int j = 0; j < MAX_TOPK; ++j) {
      if (j < k) {
        const long long a = t * k + j;
        const int e = expert[a];
        rows[j] = reinterpret_cast<const uint4*>(s_y[e / experts_per_rank] + ((long long)dst_base[e] + slot[a]) * H);
        w[j] = weight ? weight[a] : 1.f;
      }
    }
    // peer loads take microseconds: every lane issues k * UNROLL of them before it touches the first result
    for (int v0 = lane; v0 < vec; v0 += 32 * UNROLL) {
      uint4 u[MAX_TOPK][UNROLL];
#pragma unroll
      for (int j = 0; j < MAX_TOPK; ++j)
#pragma unroll
        for (int i = 0; i < UNROLL; ++i)
          if (j < k && v0 + i * 32 < vec) u[j][i] = rows[j][v0 + i * 32];
#pragma unroll
      for (int i = 0; i < UNROLL; ++i) {
        if (v0 + i * 32 >= vec) continue;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < MAX_TOPK; ++j) {
          if (j >= k) continue;
          if (save) reinterpret_cast<uint4*>(save + (t * k + j) * H)[v0 + i * 32] = u[j][i];
          const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u[j][i]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(b[q]);
            acc[2 * q] += w[j] * f.x;
            acc[2 * q + 1] += w[j] * f.y;
          }
        }
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int q = 0; q < 4; ++q) ob[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
        reinterpret_cast<uint4*>(out + t * H)[v0 + i * 32] = o;
      }
    }
  }
  if (!grid_barrier(c.counter, (int)gridDim.x, c.err, 3)) return;
  handshake(c, 1);  // peers may reuse their output buffers once everybody has finished reading
}

__global__ void moe_rowdot_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ rows,
                                  float* __restrict__ dots, int T, int k, int H) {
  const long long a = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (a >= (long long)T * k) return;
  const uint4* p = reinterpret_cast<const uint4*>(dy + (a / k) * H);
  const uint4* q = reinterpret_cast<const uint4*>(rows + a * H);
  float acc = 0.f;
  for (int v = lane; v < H / 8; v += 32) {
    const uint4 u = p[v], w = q[v];
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
    const __nv_bfloat162* d = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(b[j]), g = __bfloat1622float2(d[j]);
      acc += f.x * g.x + f.y * g.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dots[a] = acc;
}

static Comm make_comm(int** flags, int* counter, int* err, int rank, int world, int epoch) {
  Comm c;
  for (int i = 0; i < MAX_RANKS; ++i) c.flags[i] = i < world ? flags[i] : nullptr;
  c.counter = counter;
  c.err = err;
  c.rank = rank;
  c.world = world;
  c.epoch = epoch;
  return c;
}

}  // namespace pbmoe

extern "C" {

int pb_moe_slots(const int* expert, int* counts, int* slot, int n, int n_experts, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemsetAsync(counts, 0, n_experts * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  pbmoe::moe_slots_kernel<<<(n + 255) / 256, 256, 0, stream>>>(expert, counts, slot, n);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

// recv_ptrs_dev / y_ptrs_dev: device arrays of `world` pointers. counter: local int, zeroed here.
int pb_moe_dispatch(const void* x, const int* expert, const int* slot, const int* dst_base, const float* scale,
                    void* recv_ptrs_dev, int T, int k, int H, int experts_per_rank, int** flags, int* counter,
                    int* err, int rank, int world, int epoch, int ctas, void* stream_) {
  using namespace pbmoe;
  if (H % 8 != 0 || world > MAX_RANKS) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  moe_dispatch_kernel<<<ctas, THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), expert, slot, dst_base,
                                                    scale, reinterpret_cast<__nv_bfloat16* const*>(recv_ptrs_dev), T,
                                                    k, H, experts_per_rank,
                                                    make_comm(flags, counter, err, rank, world, epoch));
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_moe_combine(void* out, const int* expert, const int* slot, const int* dst_base, const float* weight,
                   void* y_ptrs_dev, void* save, int T, int k, int H, int experts_per_rank, int** flags,
                   int* counter, int* err, int rank, int world, int epoch, int ctas, void* stream_) {
  using namespace pbmoe;
  if (H % 8 != 0 || world > MAX_RANKS || k > MAX_TOPK) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  moe_combine_kernel<<<ctas, THREADS, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(out), expert, slot, dst_base,
                                                   weight, reinterpret_cast<__nv_bfloat16* const*>(y_ptrs_dev),
                                                   reinterpret_cast<__nv_bfloat16*>(save), T, k, H, experts_per_rank,
                                                   make_comm(flags, counter, err, rank, world, epoch));
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_moe_rowdot(const void* dy, const void* rows, float* dots, int T, int k, int H, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const long long threads = (long long)T * k * 32;
  pbmoe::moe_rowdot_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(rows), dots, T, k, H);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // extern "C"
