// RMSNorm and LayerNorm, forward and backward, bf16 activations with fp32 statistics.
//
// Forward: one CTA per group of rows, each row held in registers (16-byte loads), one pass.
// Backward: a persistent grid walks the rows; every thread keeps its slice of the weight (and bias)
// gradient in registers and writes one partial row per CTA to a scratch buffer [grid, H] which a
// second kernel folds.  dx is produced in the same pass.
#include <cuda_bf16.h>
#include <mutex>
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" void pb_count_launch(int n);

namespace pbn {

constexpr int THREADS = 256;
constexpr int MAX_VEC = 4;  // up to 4 x 8 bf16 per thread -> H <= 8192

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

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

// kLayer = false: RMSNorm (y = x * rstd * w);  true: LayerNorm (y = (x - mean) * rstd * w + b)
template <bool kLayer, int NV>
__global__ void __launch_bounds__(THREADS) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           const __nv_bfloat16* __restrict__ b,
                                                           __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
                                                           float* __restrict__ rstd_out, int T, int H, float eps) {
  __shared__ float red[THREADS / 32];
  const int nvec = H / 8;  // 16-byte vectors per row
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    float v[NV][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < nvec) {
        unpack8(xr[c], v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s += v[i][j];
          ss += v[i][j] * v[i][j];
        }
      }
    }
    float mean = 0.f;
    if (kLayer) {
      mean = block_sum(s, red) / H;
      // second moment around the mean, from registers
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float d = v[i][j] - mean;
            sq += d * d;
          }
        }
      }
      ss = sq;
    }
    const float var = block_sum(ss, red) / H;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (kLayer) mean_out[row] = mean;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < nvec) {
        float wv[8], o[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(w) + c), wv);
        if (kLayer) {
          float bv[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(b) + c), bv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * wv[j] + bv[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
        }
        yr[c] = pack8(o);
      }
    }
  }
}

// dx and per-CTA partial dw (and db). partial: [gridDim.x, 2, H] fp32 (db half unused for RMSNorm).
// dres (optional, [T, H]): a gradient that reached x on another path (the residual branch); it is added to dx here
// instead of by a separate elementwise kernel.
template <bool kLayer, int NV, bool kRes>
__global__ void __launch_bounds__(THREADS) norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                           const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           const float* __restrict__ mean_in,
                                                           const float* __restrict__ rstd_in,
                                                           const __nv_bfloat16* __restrict__ dres,
                                                           __nv_bfloat16* __restrict__ dx, float* __restrict__ partial,
                                                           int T, int H) {
  __shared__ float red[THREADS / 32];
  const int nvec = H / 8;
  float dw_acc[NV][8], db_acc[NV][8], wv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dw_acc[i][j] = 0.f;
      db_acc[i][j] = 0.f;
      wv[i][j] = 0.f;
    }
    if (c < nvec) unpack8(__ldg(reinterpret_cast<const uint4*>(w) + c), wv[i]);
  }
  // The next row's loads are issued before this row's reductions: the block-wide sums wait at barriers, and
  // without loads in flight across them the kernel ran at half of the copy bandwidth.
  uint4 xq[NV], gq[NV], rq[NV];
  float rstd_next = 0.f, mean_next = 0.f;
  auto fetch = [&](int row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    const uint4* rr = kRes ? reinterpret_cast<const uint4*>(dres + (size_t)row * H) : nullptr;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < nvec) {
        xq[i] = xr[c];
        gq[i] = gr[c];
        if (kRes) rq[i] = rr[c];
      }
    }
    rstd_next = rstd_in[row];
    if (kLayer) mean_next = mean_in[row];
  };
  if ((int)blockIdx.x < T) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_next;
    const float mean = kLayer ? mean_next : 0.f;
    float xh[NV][8], g[NV][8];
    uint4 rcur[NV];
    float s1 = 0.f, s2 = 0.f;  // sum(g*w*xhat), sum(g*w)
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < nvec) {
        unpack8(xq[i], xh[i]);
        unpack8(gq[i], g[i]);
        if (kRes) rcur[i] = rq[i];
      }
    }
    if (row + (int)gridDim.x < T) fetch(row + gridDim.x);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          const float gw = g[i][j] * wv[i][j];
          s1 += gw * xh[i][j];
          s2 += gw;
          dw_acc[i][j] += g[i][j] * xh[i][j];
          if (kLayer) db_acc[i][j] += g[i][j];
        }
      }
    }
    const float m1 = block_sum(s1, red) / H;
    const float m2 = kLayer ? block_sum(s2, red) / H : 0.f;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] * wv[i][j] - m2 - xh[i][j] * m1);
        if (kRes) {
          float r[8];
          unpack8(rcur[i], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        dxr[c] = pack8(o);
      }
    }
  }
  float* pw = partial + (size_t)blockIdx.x * 2 * H;
  float* pb = pw + H;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * THREADS;
    if (c < nvec) {
      float4* d0 = reinterpret_cast<float4*>(pw + c * 8);
      d0[0] = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
      d0[1] = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
      if (kLayer) {
        float4* d1 = reinterpret_cast<float4*>(pb + c * 8);
        d1[0] = make_float4(db_acc[i][0], db_acc[i][1], db_acc[i][2], db_acc[i][3]);
        d1[1] = make_float4(db_acc[i][4], db_acc[i][5], db_acc[i][6], db_acc[i][7]);
      }
    }
  }
}

// out[h] (+)= sum_p partial[p, which, h]; writes fp32 (accumulate) or bf16.  A CTA owns 32 columns; its 8 warps
// each sum every 8th partial row (four loads in flight per thread), then warp 0 adds the 8 sums in a fixed order.
constexpr int RED_COLS = 32, RED_WAYS = 8;
__global__ void __launch_bounds__(RED_COLS* RED_WAYS)
    norm_reduce_partials(const float* __restrict__ partial, int parts, int H, int which, float* out_f32,
                         __nv_bfloat16* out_bf16, int accumulate) {
  __shared__ float sums[RED_WAYS][RED_COLS];
  const int cx = threadIdx.x & (RED_COLS - 1), way = threadIdx.x / RED_COLS;
  const int h = blockIdx.x * RED_COLS + cx;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (h < H) {
    const float* src = partial + (size_t)which * H + h;
    const size_t step = (size_t)2 * H;
    int p = way;
    for (; p + 3 * RED_WAYS < parts; p += 4 * RED_WAYS) {
      s0 += src[(size_t)p * step];
      s1 += src[(size_t)(p + RED_WAYS) * step];
      s2 += src[(size_t)(p + 2 * RED_WAYS) * step];
      s3 += src[(size_t)(p + 3 * RED_WAYS) * step];
    }
    for (; p < parts; p += RED_WAYS) s0 += src[(size_t)p * step];
  }
  sums[way][cx] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (way == 0 && h < H) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < RED_WAYS; ++w) s += sums[w][cx];
    if (out_f32) out_f32[h] = accumulate ? out_f32[h] + s : s;
    else out_bf16[h] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[h]) + s : s);
  }
}

}  // namespace pbn

extern "C" {

// Number of scratch floats pb_norm_bwd needs for hidden size H.
long long pb_norm_bwd_scratch_floats(int H, int sm_count) { return (long long)sm_count * 2 * 2 * H; }

int pb_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int T, int H,
                float eps, int layer_norm, void* stream_) {
  using namespace pbn;
  if (H % 8 != 0 || H > THREADS * MAX_VEC * 8) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = T < 148 * 8 ? T : 148 * 8;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto B = reinterpret_cast<const __nv_bfloat16*>(b);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  const int nv = (H / 8 + THREADS - 1) / THREADS;
#define PB_FWD(L, NVV) norm_fwd_kernel<L, NVV><<<grid, THREADS, 0, stream>>>(X, W, B, Y, mean, rstd, T, H, eps)
  if (layer_norm) {
    if (nv <= 1) PB_FWD(true, 1); else if (nv <= 2) PB_FWD(true, 2); else PB_FWD(true, 4);
  } else {
    if (nv <= 1) PB_FWD(false, 1); else if (nv <= 2) PB_FWD(false, 2); else PB_FWD(false, 4);
  }
#undef PB_FWD
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

// dw_f32/db_f32 (fp32, accumulate) or dw_bf16/db_bf16; scratch: pb_norm_bwd_scratch_floats(H, sm_count) floats.
// dres: optional [T, H] bf16 gradient added to dx (the residual branch's gradient of the same tensor).
int pb_norm_bwd_res(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                    const void* dres, void* dx, float* dw_f32, float* db_f32, void* dw_bf16, void* db_bf16,
                    int accumulate, float* scratch, int T, int H, int layer_norm, int sm_count, void* stream_) {
  using namespace pbn;
  if (H % 8 != 0 || H > THREADS * MAX_VEC * 8) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int grid = sm_count * 2;
  if (grid > T) grid = T;
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  const int nv = (H / 8 + THREADS - 1) / THREADS;
  auto DR = reinterpret_cast<const __nv_bfloat16*>(dres);
#define PB_BWD(L, NVV)                                                                                          \
  do {                                                                                                          \
    if (DR) norm_bwd_kernel<L, NVV, true><<<grid, THREADS, 0, stream>>>(DY, X, W, mean, rstd, DR, DX, scratch, T, H); \
    else norm_bwd_kernel<L, NVV, false><<<grid, THREADS, 0, stream>>>(DY, X, W, mean, rstd, DR, DX, scratch, T, H);   \
  } while (0)
  if (layer_norm) {
    if (nv <= 1) PB_BWD(true, 1); else if (nv <= 2) PB_BWD(true, 2); else PB_BWD(true, 4);
  } else {
    if (nv <= 1) PB_BWD(false, 1); else if (nv <= 2) PB_BWD(false, 2); else PB_BWD(false, 4);
  }
#undef PB_BWD
  const int rb = (H + RED_COLS - 1) / RED_COLS, rt = RED_COLS * RED_WAYS;
  norm_reduce_partials<<<rb, rt, 0, stream>>>(scratch, grid, H, 0, dw_f32, reinterpret_cast<__nv_bfloat16*>(dw_bf16),
                                              accumulate);
  int launches = 2;
  if (layer_norm) {
    norm_reduce_partials<<<rb, rt, 0, stream>>>(scratch, grid, H, 1, db_f32,
                                                reinterpret_cast<__nv_bfloat16*>(db_bf16), accumulate);
    launches = 3;
  }
  pb_count_launch(launches);
  return (int)cudaGetLastError();
}

int pb_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                float* dw_f32, float* db_f32, void* dw_bf16, void* db_bf16, int accumulate, float* scratch, int T, int H,
                int layer_norm, int sm_count, void* stream_) {
  return pb_norm_bwd_res(dy, x, w, mean, rstd, nullptr, dx, dw_f32, db_f32, dw_bf16, db_bf16, accumulate, scratch, T, H,
                         layer_norm, sm_count, stream_);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared in no_alloc.h; the reference has no counterpart).
//
// Same math and kernels as pb_norm_bwd(layer_norm = 0), but the per-CTA partial weight gradients live in a
// file-scope device array instead of a caller-provided buffer, so the call performs no cudaMalloc/cudaFree and
// needs no allocator of any kind.
namespace pbn {
constexpr int NOALLOC_MAX_H = 8192;
constexpr int NOALLOC_MAX_CTAS = 128;
// [NOALLOC_MAX_CTAS][2][NOALLOC_MAX_H] floats = 8 MiB, resident on every device that loads this library
static __device__ __align__(256) float g_noalloc_scratch[(size_t)NOALLOC_MAX_CTAS * 2 * NOALLOC_MAX_H];
constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_scratch_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
static std::mutex g_noalloc_setup_mu;  // two host threads may make a device's first call at the same time
}  // namespace pbn

extern "C" {

int pb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_f32,
                           int accumulate, int T, int H, void* stream_) {
  using namespace pbn;
  if (T <= 0 || H <= 0 || H % 8 != 0) return -1;
  if (H > NOALLOC_MAX_H) return -2;  // beyond the built-in scratch: use pb_norm_bwd with a caller buffer instead
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return -3;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_setup_mu);
    if (g_noalloc_scratch_ptr[dev] == nullptr) {
      // first call on this device: resolve the device address of the array (its name is only a host-side handle)
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess) return (int)e;
      g_noalloc_scratch_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_noalloc_scratch_ptr[dev];
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int grid = NOALLOC_MAX_CTAS;
  if (grid > T) grid = T;
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  const int nv = (H / 8 + THREADS - 1) / THREADS;
  // every CTA overwrites its own partial row before the fold reads it, so nothing needs clearing between calls
  if (nv <= 1) norm_bwd_kernel<false, 1, false><<<grid, THREADS, 0, stream>>>(DY, X, W, nullptr, rstd, nullptr, DX, scratch, T, H);
  else if (nv <= 2) norm_bwd_kernel<false, 2, false><<<grid, THREADS, 0, stream>>>(DY, X, W, nullptr, rstd, nullptr, DX, scratch, T, H);
  else norm_bwd_kernel<false, 4, false><<<grid, THREADS, 0, stream>>>(DY, X, W, nullptr, rstd, nullptr, DX, scratch, T, H);
  norm_reduce_partials<<<(H + RED_COLS - 1) / RED_COLS, RED_COLS * RED_WAYS, 0, stream>>>(scratch, grid, H, 0, dw_f32,
                                                                                          nullptr, accumulate);
  pb_count_launch(2);
  return (int)cudaGetLastError();
}

int pb_rmsnorm_bwd_noalloc_max_hidden() { return pbn::NOALLOC_MAX_H; }

}  // extern "C"
