// Memory-bound activation kernels: RoPE (in place, forward and backward), SwiGLU and GELU(tanh) forward/backward,
// scaling, column sums for bias gradients, fp32 -> bf16 casts.  bf16 in/out, fp32 math, 16-byte accesses.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" void pb_count_launch(int n);

namespace pbe {

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

// Rotates the first `n_rot_heads` heads of every row of `qkv` [T, row_stride] in place ("rotate-half" pairing:
// element i pairs with i + D/2).  cos/sin: [S, D/2] fp32, position of row t is t % S.  sign = +1 forward, -1 backward.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cs, const float* __restrict__ sn,
                            long long T, int S, int n_rot_heads, int D, long long row_stride, float sign) {
  const int half = D / 2;
  const int vec_per_head = half / 8;
  const long long total = T * n_rot_heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int h = (int)(th % n_rot_heads);
    const long long t = th / n_rot_heads;
    const int pos = (int)(t % S);
    __nv_bfloat16* base = qkv + t * row_stride + (long long)h * D + v * 8;
    uint4 lo = *reinterpret_cast<uint4*>(base);
    uint4 hi = *reinterpret_cast<uint4*>(base + half);
    float a[8], b[8], c[8], s[8];
    unpack8(lo, a);
    unpack8(hi, b);
    const float4* cp = reinterpret_cast<const float4*>(cs + (long long)pos * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sn + (long long)pos * half + v * 8);
    float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
    float oa[8], ob[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = sign * s[j];
      oa[j] = a[j] * c[j] - b[j] * sj;
      ob[j] = b[j] * c[j] + a[j] * sj;
    }
    *reinterpret_cast<uint4*>(base) = pack8(oa);
    *reinterpret_cast<uint4*>(base + half) = pack8(ob);
  }
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// gu: [T, 2F] (gate | up) -> out [T, F] = silu(gate) * up
// row_limit (optional, device): only rows below *row_limit are processed (buffers sized for a capacity of which the
// device knows how much is in use)
// Thread layout of both SwiGLU kernels: x covers the 16-byte column vectors of a row, y strides over the rows, so
// that no index is ever divided (a flat index split by 64-bit division made these kernels instruction-bound).
__global__ void __launch_bounds__(128) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                                         __nv_bfloat16* __restrict__ out, long long T, int F,
                                                         const int* __restrict__ row_limit) {
  if (row_limit && *row_limit < T) T = *row_limit;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= F / 8) return;
  const long long step = gridDim.y;
  // two rows per trip: four 16-byte loads in flight per thread
  for (long long t = blockIdx.y; t < T; t += 2 * step) {
    const long long t1 = t + step < T ? t + step : t;
    const __nv_bfloat16* r0 = gu + t * 2 * F + v * 8;
    const __nv_bfloat16* r1 = gu + t1 * 2 * F + v * 8;
    const uint4 g0 = *reinterpret_cast<const uint4*>(r0);
    const uint4 u0 = *reinterpret_cast<const uint4*>(r0 + F);
    const uint4 g1 = *reinterpret_cast<const uint4*>(r1);
    const uint4 u1 = *reinterpret_cast<const uint4*>(r1 + F);
    float g[8], u[8], o[8];
    unpack8(g0, g);
    unpack8(u0, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_(g[j]) * u[j];
    *reinterpret_cast<uint4*>(out + t * F + v * 8) = pack8(o);
    if (t1 != t) {
      unpack8(g1, g);
      unpack8(u1, u);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_(g[j]) * u[j];
      *reinterpret_cast<uint4*>(out + t1 * F + v * 8) = pack8(o);
    }
  }
}

// dgu [T, 2F] from dout [T, F] and gu
__global__ void __launch_bounds__(128) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                                         const __nv_bfloat16* __restrict__ gu,
                                                         __nv_bfloat16* __restrict__ dgu, long long T, int F,
                                                         const int* __restrict__ row_limit) {
  if (row_limit && *row_limit < T) T = *row_limit;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= F / 8) return;
  for (long long t = blockIdx.y; t < T; t += gridDim.y) {
    const __nv_bfloat16* row = gu + t * 2 * F + v * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(row), g);
    unpack8(*reinterpret_cast<const uint4*>(row + F), u);
    unpack8(*reinterpret_cast<const uint4*>(dout + t * F + v * 8), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoidf_(g[j]);
      const float silu = g[j] * s;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
    }
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + v * 8) = pack8(dg);
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + F + v * 8) = pack8(du);
  }
}

// dx = dy * gelu'(x) (tanh approximation), elementwise over n elements (n % 8 == 0)
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                __nv_bfloat16* __restrict__ dx, long long n) {
  const long long total = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8], g[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
    unpack8(reinterpret_cast<const uint4*>(dy)[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      const float xx = a[j];
      const float u = k0 * (xx + k1 * xx * xx * xx);
      const float t = tanhf(u);
      const float du = k0 * (1.f + 3.f * k1 * xx * xx);
      o[j] = g[j] * (0.5f * (1.f + t) + 0.5f * xx * (1.f - t * t) * du);
    }
    reinterpret_cast<uint4*>(dx)[i] = pack8(o);
  }
}

__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long total = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      const float xx = a[j];
      o[j] = 0.5f * xx * (1.f + tanhf(k0 * (xx + k1 * xx * xx * xx)));
    }
    reinterpret_cast<uint4*>(y)[i] = pack8(o);
  }
}

// x *= *scale (scale read from device memory), bf16, n % 8 == 0
__global__ void scale_bf16_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ scale, long long n) {
  const float s = *scale;
  const long long total = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] *= s;
    reinterpret_cast<uint4*>(x)[i] = pack8(a);
  }
}

// out[c] (+)= sum_t x[t, c];  x bf16 [T, C] row pitch ld; one thread per column pair, rows strided over blockIdx.y,
// partial sums combined with fp32 atomics into a zeroed or accumulating fp32 buffer.
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, long long T, int C,
                              long long ld) {
  const int c2 = blockIdx.x * blockDim.x + threadIdx.x;  // column pair
  if (c2 * 2 >= C) return;
  float s0 = 0.f, s1 = 0.f;
  for (long long t = blockIdx.y; t < T; t += gridDim.y) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + t * ld + c2 * 2);
    const float2 f = __bfloat1622float2(v);
    s0 += f.x;
    s1 += f.y;
  }
  atomicAdd(out + c2 * 2, s0);
  if (c2 * 2 + 1 < C) atomicAdd(out + c2 * 2 + 1, s1);
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n,
                                        float scale) {
  const long long total = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x * scale, v.y * scale);
    __nv_bfloat162 b = __floats2bfloat162_rn(v.z * scale, v.w * scale);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    reinterpret_cast<uint2*>(y)[i] = o;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = total * 4; i < n; ++i) y[i] = __float2bfloat16(x[i] * scale);
}

// acc (fp32) += x (bf16), n % 8 == 0
__global__ void accum_bf16_into_f32_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ x, long long n) {
  const long long total = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
    float4* p = reinterpret_cast<float4*>(acc) + 2 * i;
    float4 u = p[0], w = p[1];
    u.x += a[0]; u.y += a[1]; u.z += a[2]; u.w += a[3];
    w.x += a[4]; w.y += a[5]; w.z += a[6]; w.w += a[7];
    p[0] = u;
    p[1] = w;
  }
}

static inline int grid_for(long long work_items, int threads) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = 148LL * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// x: 128-thread CTAs over the F / 8 column vectors; y: rows, about 32 CTAs per SM in all
static inline dim3 swiglu_grid(long long T, int F) {
  const int gx = (F / 8 + 127) / 128;
  long long gy = (148LL * 32 + gx - 1) / gx;
  if (gy > T) gy = T;
  if (gy < 1) gy = 1;
  return dim3((unsigned)gx, (unsigned)gy);
}

}  // namespace pbe

extern "C" {

int pb_rope(void* qkv, const float* cs, const float* sn, long long T, int S, int n_rot_heads, int D,
            long long row_stride, float sign, void* stream_) {
  using namespace pbe;
  if (D % 16 != 0 || row_stride % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const long long total = T * n_rot_heads * (D / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(qkv), cs, sn, T, S,
                                                         n_rot_heads, D, row_stride, sign);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_swiglu_fwd(const void* gu, void* out, long long T, int F, const int* row_limit, void* stream_) {
  using namespace pbe;
  if (F % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  swiglu_fwd_kernel<<<swiglu_grid(T, F), 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(gu),
                                                           reinterpret_cast<__nv_bfloat16*>(out), T, F, row_limit);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long T, int F, const int* row_limit,
                  void* stream_) {
  using namespace pbe;
  if (F % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  swiglu_bwd_kernel<<<swiglu_grid(T, F), 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
                                                           reinterpret_cast<const __nv_bfloat16*>(gu),
                                                           reinterpret_cast<__nv_bfloat16*>(dgu), T, F, row_limit);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_gelu_fwd(const void* x, void* y, long long n, void* stream_) {
  using namespace pbe;
  if (n % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                            reinterpret_cast<__nv_bfloat16*>(y), n);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, void* stream_) {
  using namespace pbe;
  if (n % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dy),
                                                            reinterpret_cast<const __nv_bfloat16*>(x),
                                                            reinterpret_cast<__nv_bfloat16*>(dx), n);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_scale_bf16(void* x, const float* scale_dev, long long n, void* stream_) {
  using namespace pbe;
  if (n % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  scale_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(x), scale_dev, n);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

// out (fp32, [C]) += column sums of x (bf16 [T, C]); caller zeroes `out` when it does not want accumulation.
int pb_colsum_bf16(const void* x, float* out, long long T, int C, long long ld, void* stream_) {
  using namespace pbe;
  if (C % 2 != 0 || ld % 2 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  dim3 grid((C / 2 + 127) / 128, (unsigned)(T < 256 ? T : 256));
  colsum_kernel<<<grid, 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), out, T, C, ld);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_cast_f32_to_bf16(const float* x, void* y, long long n, float scale, void* stream_) {
  using namespace pbe;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cast_f32_to_bf16_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, stream>>>(x, reinterpret_cast<__nv_bfloat16*>(y), n,
                                                                        scale);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_accum_bf16_into_f32(float* acc, const void* x, long long n, void* stream_) {
  using namespace pbe;
  if (n % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  accum_bf16_into_f32_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(acc, reinterpret_cast<const __nv_bfloat16*>(x),
                                                                        n);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // extern "C"
