// Expert-parallel MoE data movement over NVLink peer memory.
//
//   moe_route     : softmax over the router logits, top-k, normalised weights, load-balance statistics and the
//                   position of every (token, k) assignment inside its expert's group, in token order (no atomics:
//                   the order, and with it the summation order of the expert weight gradients, is reproducible)
//   moe_route_bwd : gradient of the router logits from the gradients of the top-k weights and of the aux loss
//   moe_dispatch  : count exchange + permute + all-to-all in one kernel: the ranks tell each other how many rows
//                   they hold per expert, every rank derives the layout of every receive buffer from that (expert
//                   groups start on multiples of 256 rows), and each assignment's token row (optionally scaled) is
//                   stored straight into the owning rank's expert-grouped receive buffer (P2P stores).  Sizes never
//                   visit the host: the receiver gets its group table in device memory for the grouped GEMM.
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
  long long wait_cycles;
  int rank, world, epoch;
};

constexpr int MAX_EXPERTS = 16;
constexpr int ROUTE_THREADS = 256;

// One thread per token.  logits: [T, ld] bf16.  Outputs: probs [T, E] fp32, topi / topw [T, k] (weights normalised
// over the selected k), pos [T*k] = rank of the assignment among this CTA's assignments to the same expert (token
// order), cta_counts / cta_psum [gridDim.x, E] = this CTA's assignments per expert and sums of probabilities.
__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_kernel(const __nv_bfloat16* __restrict__ logits, int ld,
                                                                  int T, int E, int k, float* __restrict__ probs,
                                                                  int* __restrict__ topi, float* __restrict__ topw,
                                                                  int* __restrict__ pos, int* __restrict__ cta_counts,
                                                                  float* __restrict__ cta_psum) {
  __shared__ int s_wcnt[ROUTE_THREADS / 32][MAX_EXPERTS];
  __shared__ float s_wsum[ROUTE_THREADS / 32][MAX_EXPERTS];
  const int t = blockIdx.x * ROUTE_THREADS + threadIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool live = t < T;
  float p[MAX_EXPERTS];
  int sel[MAX_TOPK];
  unsigned chosen = 0;
  if (live) {
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) {
      p[e] = e < E ? __bfloat162float(logits[(long long)t * ld + e]) : -INFINITY;
      mx = fmaxf(mx, p[e]);
    }
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) {
      p[e] = e < E ? __expf(p[e] - mx) : 0.f;
      sum += p[e];
    }
    const float inv = 1.f / sum;
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) {
      p[e] *= inv;
      if (e < E) probs[(long long)t * E + e] = p[e];
    }
    float wsum = 0.f;
    float w[MAX_TOPK];
#pragma unroll
    for (int j = 0; j < MAX_TOPK; ++j) {
      if (j >= k) continue;
      int best = 0;
      float bv = -1.f;
#pragma unroll
      for (int e = 0; e < MAX_EXPERTS; ++e)
        if (e < E && !((chosen >> e) & 1u) && p[e] > bv) {  // ties go to the lower index, as torch.topk does
          bv = p[e];
          best = e;
        }
      chosen |= 1u << best;
      sel[j] = best;
      w[j] = bv;
      wsum += bv;
    }
#pragma unroll
    for (int j = 0; j < MAX_TOPK; ++j)
      if (j < k) {
        topi[(long long)t * k + j] = sel[j];
        topw[(long long)t * k + j] = w[j] / wsum;
      }
  } else {
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) p[e] = 0.f;
  }
  // per expert: how many tokens of this warp chose it, and which of them come before this token
  int rank_in_warp[MAX_EXPERTS];
#pragma unroll
  for (int e = 0; e < MAX_EXPERTS; ++e) {
    if (e >= E) continue;
    const unsigned m = __ballot_sync(0xffffffffu, (chosen >> e) & 1u);
    rank_in_warp[e] = __popc(m & ((1u << lane) - 1u));
    float v = p[e];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) {
      s_wcnt[warp][e] = __popc(m);
      s_wsum[warp][e] = v;
    }
  }
  __syncthreads();
  if (live) {
#pragma unroll
    for (int j = 0; j < MAX_TOPK; ++j) {
      if (j >= k) continue;
      int base = 0;
      int r = 0;
#pragma unroll
      for (int e = 0; e < MAX_EXPERTS; ++e)
        if (e == sel[j]) r = rank_in_warp[e];
      for (int w2 = 0; w2 < warp; ++w2) base += s_wcnt[w2][sel[j]];
      pos[(long long)t * k + j] = base + r;
    }
  }
  if (threadIdx.x < E) {
    int c = 0;
    float ps = 0.f;
    for (int w2 = 0; w2 < ROUTE_THREADS / 32; ++w2) {
      c += s_wcnt[w2][threadIdx.x];
      ps += s_wsum[w2][threadIdx.x];
    }
    cta_counts[blockIdx.x * E + threadIdx.x] = c;
    cta_psum[blockIdx.x * E + threadIdx.x] = ps;
  }
}

// One CTA: prefix over the route kernel's CTAs (in order), totals, the load-balance loss, final positions.
//   counts[e] = assignments to e; share[e] = counts[e] / (T k); aux = E * sum_e share[e] * mean_t probs[t, e]
__global__ void __launch_bounds__(1024) moe_route_finish_kernel(int* __restrict__ cta_counts,
                                                                const float* __restrict__ cta_psum, int n_cta, int T,
                                                                int E, int k, const int* __restrict__ topi,
                                                                int* __restrict__ pos, int* __restrict__ counts,
                                                                float* __restrict__ share, float* __restrict__ aux) {
  __shared__ float s_term[MAX_EXPERTS];
  if (threadIdx.x < E) {
    const int e = threadIdx.x;
    int run = 0;
    float ps = 0.f;
    for (int c = 0; c < n_cta; ++c) {
      const int v = cta_counts[c * E + e];
      cta_counts[c * E + e] = run;  // becomes the CTA's base
      run += v;
      ps += cta_psum[c * E + e];
    }
    counts[e] = run;
    const float sh = (float)run / (float)((long long)T * k);
    share[e] = sh;
    s_term[e] = sh * (ps / (float)T);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int e = 0; e < E; ++e) a += s_term[e];
    *aux = a * (float)E;
  }
  const long long n = (long long)T * k;
  for (long long a = threadIdx.x; a < n; a += blockDim.x)
    pos[a] += cta_counts[(int)((a / k) / ROUTE_THREADS) * E + topi[a]];
}

// dlogits[t, :] from g_w [T, k] (gradient of the normalised top-k weights) and *g_aux (gradient of the aux loss).
__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_bwd_kernel(const float* __restrict__ probs,
                                                                      const int* __restrict__ topi,
                                                                      const float* __restrict__ topw,
                                                                      const float* __restrict__ g_w,
                                                                      const float* __restrict__ g_aux,
                                                                      const float* __restrict__ share, int T, int E,
                                                                      int k, __nv_bfloat16* __restrict__ dlogits,
                                                                      int ld) {
  const int t = blockIdx.x * ROUTE_THREADS + threadIdx.x;
  if (t >= T) return;
  float p[MAX_EXPERTS], dp[MAX_EXPERTS];
  const float ga = g_aux ? *g_aux : 0.f;
#pragma unroll
  for (int e = 0; e < MAX_EXPERTS; ++e) {
    p[e] = e < E ? probs[(long long)t * E + e] : 0.f;
    dp[e] = e < E ? ga * (float)E * share[e] / (float)T : 0.f;
  }
  if (g_w) {
    float s = 0.f, gdotw = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_TOPK; ++j)
      if (j < k) {
        const int e = topi[(long long)t * k + j];
#pragma unroll
        for (int q = 0; q < MAX_EXPERTS; ++q)
          if (q == e) s += p[q];
        gdotw += g_w[(long long)t * k + j] * topw[(long long)t * k + j];
      }
    const float inv_s = 1.f / s;
#pragma unroll
    for (int j = 0; j < MAX_TOPK; ++j)
      if (j < k) {
        const int e = topi[(long long)t * k + j];
        const float g = (g_w[(long long)t * k + j] - gdotw) * inv_s;
#pragma unroll
        for (int q = 0; q < MAX_EXPERTS; ++q)
          if (q == e) dp[q] += g;
      }
  }
  float dot = 0.f;
#pragma unroll
  for (int e = 0; e < MAX_EXPERTS; ++e) dot += dp[e] * p[e];
#pragma unroll
  for (int e = 0; e < MAX_EXPERTS; ++e)
    if (e < ld) dlogits[(long long)t * ld + e] = __float2bfloat16(e < E ? p[e] * (dp[e] - dot) : 0.f);
  for (int e = MAX_EXPERTS; e < ld; ++e) dlogits[(long long)t * ld + e] = __float2bfloat16(0.f);  // padding columns
}

__device__ __forceinline__ bool handshake(const Comm& c, int phase) {
  // announce phase to every peer, then wait until every peer announced it
  if (blockIdx.x == 0 && (int)threadIdx.x < c.world && (int)threadIdx.x != c.rank)
    st_release_sys(c.flags[threadIdx.x] + phase * c.world + c.rank, c.epoch);
  bool ok = true;
  if ((int)threadIdx.x < c.world && (int)threadIdx.x != c.rank)
    ok = wait_flag_sys(c.flags[c.rank] + phase * c.world + threadIdx.x, c.epoch, c.err, 3, c.wait_cycles);
  return __syncthreads_and(ok);
}

constexpr int ERR_CAPACITY = 4;

// x: [T, H] bf16; expert/slot: [T*k]; counts: this rank's assignments per expert [E]; cnt[r]: every rank's [W, E]
// count table (row s = what rank s holds); recv[r]: every rank's receive buffer [cap_rows, H]; scale: optional [T*k]
// fp32.  Outputs on this rank: dst_base[e] = first row of this rank's block inside expert e's group on its owner
// (what the combine needs), group_rows / group_start [experts_per_rank] = the layout of this rank's own receive
// buffer (what the grouped GEMM needs), rows_used = where the last group's padding ends.
__global__ void __launch_bounds__(THREADS) moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const int* __restrict__ expert,
                                                               const int* __restrict__ slot,
                                                               const int* __restrict__ counts,
                                                               const float* __restrict__ scale,
                                                               __nv_bfloat16* const* __restrict__ recv_ptrs,
                                                               int* const* __restrict__ cnt_ptrs, int T, int k, int H,
                                                               int E, int experts_per_rank, int cap_rows,
                                                               int* __restrict__ dst_base_out,
                                                               int* __restrict__ group_rows_out,
                                                               int* __restrict__ group_start_out,
                                                               int* __restrict__ rows_used_out, Comm c) {
  __shared__ __nv_bfloat16* s_recv[MAX_RANKS];
  __shared__ int s_cnt[MAX_RANKS][MAX_EXPERTS];
  __shared__ int s_total[MAX_EXPERTS], s_base[MAX_EXPERTS];
  const int W = c.world;
  if (threadIdx.x < MAX_RANKS) s_recv[threadIdx.x] = (int)threadIdx.x < W ? recv_ptrs[threadIdx.x] : nullptr;
  // phase 0: "my receive buffer is free, and this is how many rows I hold for each expert"
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < W * E; i += THREADS) {
      const int q = i / E, e = i % E;
      cnt_ptrs[q][c.rank * E + e] = counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < W) st_release_sys(c.flags[threadIdx.x] + c.rank, c.epoch);
  }
  bool ok = true;
  if ((int)threadIdx.x < W) ok = wait_flag_sys(c.flags[c.rank] + threadIdx.x, c.epoch, c.err, 3, c.wait_cycles);
  if (!__syncthreads_and(ok)) return;
  {
    const int* mine = cnt_ptrs[c.rank];
    for (int i = threadIdx.x; i < W * E; i += THREADS) s_cnt[i / E][i % E] = mine[i];
  }
  __syncthreads();
  if ((int)threadIdx.x < E) {
    int tot = 0;
    for (int s_ = 0; s_ < W; ++s_) tot += s_cnt[s_][threadIdx.x];
    s_total[threadIdx.x] = tot;
  }
  __syncthreads();
  if ((int)threadIdx.x < E) {
    const int e = threadIdx.x, d = e / experts_per_rank;
    int start = 0;
    for (int h = d * experts_per_rank; h < e; ++h) start += (s_total[h] + 255) / 256 * 256;
    int before = 0;
    for (int s_ = 0; s_ < c.rank; ++s_) before += s_cnt[s_][e];
    s_base[e] = start + before;
    if (start + s_total[e] > cap_rows) atomicExch(c.err, ERR_CAPACITY);  // rows past the capacity are dropped below
    if (blockIdx.x == 0) {
      dst_base_out[e] = start + before;
      if (d == c.rank) {
        group_rows_out[e - d * experts_per_rank] = min(s_total[e], max(cap_rows - start, 0));
        group_start_out[e - d * experts_per_rank] = min(start, cap_rows / 256 * 256);
        // rows of this rank's buffer that hold a group or its padding: what element-wise kernels have to touch
        if (e == (d + 1) * experts_per_rank - 1) *rows_used_out = min(start + (s_total[e] + 255) / 256 * 256, cap_rows);
      }
    }
  }
  __syncthreads();
  const int warps_per_block = THREADS / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vec = H / 8;
  const long long n = (long long)T * k;
  for (long long a = blockIdx.x * warps_per_block + warp; a < n; a += (long long)gridDim.x * warps_per_block) {
    const int e = expert[a];
    const int d = e / experts_per_rank;
    const long long row = (long long)s_base[e] + slot[a];
    if (row >= cap_rows) continue;
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
  if (!grid_barrier(c.counter, (int)gridDim.x, c.err, 3, c.wait_cycles)) return;
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
                                                              int experts_per_rank, int cap_rows, Comm c) {
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
        long long row = (long long)dst_base[e] + slot[a];
        w[j] = weight ? weight[a] : 1.f;
        if (row >= cap_rows) {  // the dispatch dropped this row (receive buffer full, error word set): contributes 0
          row = 0;
          w[j] = 0.f;
        }
        rows[j] = reinterpret_cast<const uint4*>(s_y[e / experts_per_rank] + row * H);
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
  if (!grid_barrier(c.counter, (int)gridDim.x, c.err, 3, c.wait_cycles)) return;
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
  c.wait_cycles = pb_peer_wait_cycles();
  c.rank = rank;
  c.world = world;
  c.epoch = epoch;
  return c;
}

}  // namespace pbmoe

extern "C" {

// Router: logits [T, ld] bf16 -> probs [T, E], topi / topw [T, k], slot [T*k] (position inside the expert's group of
// this rank's assignments, token order), counts [E], share [E], aux (scalar).  scratch_i: int[n_cta * E],
// scratch_f: float[n_cta * E] with n_cta = ceil(T / 256).  E <= 16, k <= 4.
int pb_moe_route(const void* logits, int ld, int T, int E, int k, float* probs, int* topi, float* topw, int* slot,
                 int* counts, float* share, float* aux, int* scratch_i, float* scratch_f, void* stream_) {
  using namespace pbmoe;
  if (E < 1 || E > MAX_EXPERTS || k < 1 || k > MAX_TOPK || k > E || ld < E || T < 1) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int n_cta = (T + ROUTE_THREADS - 1) / ROUTE_THREADS;
  moe_route_kernel<<<n_cta, ROUTE_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, T, E, k,
                                                        probs, topi, topw, slot, scratch_i, scratch_f);
  moe_route_finish_kernel<<<1, 1024, 0, stream>>>(scratch_i, scratch_f, n_cta, T, E, k, topi, slot, counts, share,
                                                  aux);
  pb_count_launch(2);
  return (int)cudaGetLastError();
}

// g_w: [T, k] fp32 or null; g_aux: device scalar or null.
int pb_moe_route_bwd(const float* probs, const int* topi, const float* topw, const float* g_w, const float* g_aux,
                     const float* share, int T, int E, int k, void* dlogits, int ld, void* stream_) {
  using namespace pbmoe;
  if (E < 1 || E > MAX_EXPERTS || k < 1 || k > MAX_TOPK || ld < E) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  moe_route_bwd_kernel<<<(T + ROUTE_THREADS - 1) / ROUTE_THREADS, ROUTE_THREADS, 0, stream>>>(
      probs, topi, topw, g_w, g_aux, share, T, E, k, reinterpret_cast<__nv_bfloat16*>(dlogits), ld);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

// recv_ptrs_dev / cnt_ptrs_dev / y_ptrs_dev: device arrays of `world` pointers. counter: local int, zeroed here.
// A receive buffer that would overflow `cap_rows` sets the device error word to 4 and drops the rows beyond it.
int pb_moe_dispatch(const void* x, const int* expert, const int* slot, const int* counts, const float* scale,
                    void* recv_ptrs_dev, void* cnt_ptrs_dev, int T, int k, int H, int E, int experts_per_rank,
                    int cap_rows, int* dst_base_out, int* group_rows_out, int* group_start_out, int* rows_used_out,
                    int** flags, int* counter, int* err, int rank, int world, int epoch, int ctas, void* stream_) {
  using namespace pbmoe;
  if (H % 8 != 0 || world > MAX_RANKS || E > MAX_EXPERTS || E % world != 0 || experts_per_rank * world != E) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  moe_dispatch_kernel<<<ctas, THREADS, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), expert, slot, counts, scale,
      reinterpret_cast<__nv_bfloat16* const*>(recv_ptrs_dev), reinterpret_cast<int* const*>(cnt_ptrs_dev), T, k, H, E,
      experts_per_rank, cap_rows, dst_base_out, group_rows_out, group_start_out, rows_used_out,
      make_comm(flags, counter, err, rank, world, epoch));
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_moe_combine(void* out, const int* expert, const int* slot, const int* dst_base, const float* weight,
                   void* y_ptrs_dev, void* save, int T, int k, int H, int experts_per_rank, int cap_rows, int** flags,
                   int* counter, int* err, int rank, int world, int epoch, int ctas, void* stream_) {
  using namespace pbmoe;
  if (H % 8 != 0 || world > MAX_RANKS || k > MAX_TOPK) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  moe_combine_kernel<<<ctas, THREADS, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(out), expert, slot, dst_base,
                                                   weight, reinterpret_cast<__nv_bfloat16* const*>(y_ptrs_dev),
                                                   reinterpret_cast<__nv_bfloat16*>(save), T, k, H, experts_per_rank,
                                                   cap_rows, make_comm(flags, counter, err, rank, world, epoch));
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
