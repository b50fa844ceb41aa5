// Fused AdamW over a flat parameter buffer: one launch updates every parameter of a stage.
// Parameters are bf16 (optionally with an fp32 master copy), gradients fp32, moments fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" void pb_count_launch(int n);

namespace pbo {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale;
};

// n % 4 == 0 handled vectorised; tail handled by thread 0.
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, float* __restrict__ master, float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, long long n, AdamArgs a, int zero_grad) {
  const long long total = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float4 gg = reinterpret_cast<float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float w[4];
    if (master) {
      const float4 t = reinterpret_cast<float4*>(master)[i];
      w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
    } else {
      const uint2 raw = reinterpret_cast<uint2*>(p)[i];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 lo = __bfloat1622float2(b[0]), hi = __bfloat1622float2(b[1]);
      w[0] = lo.x; w[1] = lo.y; w[2] = hi.x; w[3] = hi.y;
    }
    float gr[4] = {gg.x * a.grad_scale, gg.y * a.grad_scale, gg.z * a.grad_scale, gg.w * a.grad_scale};
    float m4[4] = {mm.x, mm.y, mm.z, mm.w};
    float v4[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      m4[j] = a.beta1 * m4[j] + (1.f - a.beta1) * gr[j];
      v4[j] = a.beta2 * v4[j] + (1.f - a.beta2) * gr[j] * gr[j];
      const float mh = m4[j] / a.bias_c1;
      const float vh = v4[j] / a.bias_c2;
      w[j] = w[j] * (1.f - a.lr * a.weight_decay) - a.lr * mh / (sqrtf(vh) + a.eps);
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(m4[0], m4[1], m4[2], m4[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(v4[0], v4[1], v4[2], v4[3]);
    if (master) reinterpret_cast<float4*>(master)[i] = make_float4(w[0], w[1], w[2], w[3]);
    __nv_bfloat162 o0 = __floats2bfloat162_rn(w[0], w[1]);
    __nv_bfloat162 o1 = __floats2bfloat162_rn(w[2], w[3]);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&o0);
    o.y = *reinterpret_cast<uint32_t*>(&o1);
    reinterpret_cast<uint2*>(p)[i] = o;
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long i = total * 4; i < n; ++i) {
      float w = master ? master[i] : __bfloat162float(p[i]);
      const float gr = g[i] * a.grad_scale;
      m[i] = a.beta1 * m[i] + (1.f - a.beta1) * gr;
      v[i] = a.beta2 * v[i] + (1.f - a.beta2) * gr * gr;
      w = w * (1.f - a.lr * a.weight_decay) - a.lr * (m[i] / a.bias_c1) / (sqrtf(v[i] / a.bias_c2) + a.eps);
      if (master) master[i] = w;
      p[i] = __float2bfloat16(w);
      if (zero_grad) g[i] = 0.f;
    }
  }
}

}  // namespace pbo

extern "C" {

int pb_adamw(void* p, float* master, float* g, float* m, float* v, long long n, float lr, float beta1, float beta2,
             float eps, float weight_decay, int step, float grad_scale, int zero_grad, void* stream_) {
  using namespace pbo;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AdamArgs a;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.weight_decay = weight_decay;
  a.bias_c1 = 1.f - powf(beta1, (float)step);
  a.bias_c2 = 1.f - powf(beta2, (float)step);
  a.grad_scale = grad_scale;
  long long gsz = (n / 4 + 255) / 256;
  if (gsz > 148 * 16) gsz = 148 * 16;
  if (gsz < 1) gsz = 1;
  adamw_kernel<<<(unsigned)gsz, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(p), master, g, m, v, n, a,
                                                  zero_grad);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // extern "C"
