// Fused softmax cross-entropy over bf16 logits: one pass computes the per-row loss and overwrites the logits
// with (softmax - onehot) * row_scale, so no fp32 [T, V] tensor and no separate backward kernel exist.
// One CTA per row; the row (V up to a few hundred thousand) is read twice, the second time from L2.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "dbgcheck.cuh"

extern "C" void pb_count_launch(int n);

namespace pbx {

constexpr int THREADS = 512;

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

// logits: [T, ld] bf16, first V columns are classes (ld >= V, ld % 8 == 0; columns >= V are padding and get
// zero gradient).  targets: int64 [T], ignore_index rows contribute nothing.  loss_rows: fp32 [T].
// On exit dlogits (which may alias logits) holds grad_scale * (softmax - onehot).
__global__ void __launch_bounds__(THREADS) xent_fwd_bwd_kernel(const __nv_bfloat16* logits, __nv_bfloat16* dlogits,
                                                               const long long* __restrict__ targets,
                                                               float* __restrict__ loss_rows, int V, long long ld,
                                                               float grad_scale, long long ignore_index
                                                               PB_DBG_PARAMS) {
  __shared__ float red_m[THREADS / 32];
  __shared__ float red_s[THREADS / 32];
  __shared__ float bc[2];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  __nv_bfloat16* dr = dlogits + row * ld;
  long long tgt = targets[row];
  if (tgt != ignore_index && !PB_DBG_IN_RANGE(tgt)) tgt = ignore_index;  // debug build: reported, row skipped
  const int nvec = V / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  float m = -CUDART_INF_F, s = 0.f;
  for (int c = threadIdx.x; c < nvec; c += THREADS) {
    float v[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[c], v);
    float cm = v[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, v[j]);
    const float nm = fmaxf(m, cm);
    float add = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) add += __expf(v[j] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += THREADS) {  // ragged tail
    const float v = __bfloat162float(lr[c]);
    const float nm = fmaxf(m, v);
    s = s * __expf(m - nm) + __expf(v - nm);
    m = nm;
  }
  // block combine of (m, s)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (nm == -CUDART_INF_F) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  if (lane == 0) {
    red_m[warp] = m;
    red_s[warp] = s;
  }
  __syncthreads();
  if (warp == 0) {
    m = lane < THREADS / 32 ? red_m[lane] : -CUDART_INF_F;
    s = lane < THREADS / 32 ? red_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (nm == -CUDART_INF_F) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
    }
    if (lane == 0) {
      bc[0] = m;
      bc[1] = s;
    }
  }
  __syncthreads();
  m = bc[0];
  s = bc[1];
  const float lse = m + __logf(s);
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
  if (threadIdx.x == 0) loss_rows[row] = ignored ? 0.f : (lse - __bfloat162float(lr[tgt]));
  __syncthreads();  // the target logit was read before anything is overwritten
  const float gs = ignored ? 0.f : grad_scale;
  const float inv = 1.f / s;
  for (int c = threadIdx.x; c < nvec; c += THREADS) {
    float v[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[c], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(v[j] - m) * inv;
      if ((long long)c * 8 + j == tgt) p -= 1.f;
      v[j] = p * gs;
    }
    reinterpret_cast<uint4*>(dr)[c] = pack8(v);
  }
  for (int c = nvec * 8 + threadIdx.x; c < ld; c += THREADS) {
    float p = 0.f;
    if (c < V) {
      p = __expf(__bfloat162float(lr[c]) - m) * inv;
      if (c == tgt) p -= 1.f;
    }
    dr[c] = __float2bfloat16(p * gs);
  }
}

}  // namespace pbx

extern "C" {

int pb_xent_fwd_bwd(const void* logits, void* dlogits, const long long* targets, float* loss_rows, long long T, int V, long long ld,
                    float grad_scale, long long ignore_index, void* stream_) {
  using namespace pbx;
  if (ld % 8 != 0 || ld < V) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  xent_fwd_bwd_kernel<<<(unsigned)T, THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits),
                                                           reinterpret_cast<__nv_bfloat16*>(dlogits), targets,
                                                           loss_rows, V, ld, grad_scale, ignore_index PB_DBG_ARGS(V));
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // extern "C"
