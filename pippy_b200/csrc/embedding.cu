// Token (+ learned position) embedding gather and its scatter-add backward into an fp32 gradient table.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dbgcheck.cuh"

extern "C" void pb_count_launch(int n);

namespace pbm {

// out[t, :] = wte[ids[t], :] (+ wpe[t % S, :]);  H % 8 == 0
__global__ void embed_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ wte,
                                 const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, long long T,
                                 int H, int S PB_DBG_PARAMS) {
  const int vec = H / 8;
  const long long total = T * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int v = (int)(i % vec);
    const long long id = ids[t];
    if (!PB_DBG_IN_RANGE(id)) continue;  // debug build: a token id outside the table is reported, not read
    uint4 a = __ldg(reinterpret_cast<const uint4*>(wte + id * H) + v);
    if (wpe) {
      uint4 p = __ldg(reinterpret_cast<const uint4*>(wpe + (long long)(t % S) * H) + v);
      __nv_bfloat162* ab = reinterpret_cast<__nv_bfloat162*>(&a);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&p);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 x = __bfloat1622float2(ab[j]), y = __bfloat1622float2(pb[j]);
        ab[j] = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
      }
    }
    reinterpret_cast<uint4*>(out + t * H)[v] = a;
  }
}

// dwte[ids[t], :] += dout[t, :]  (fp32 table, vector atomics);  dwpe[t % S, :] += dout[t, :]
__global__ void embed_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                 float* __restrict__ dwte, float* __restrict__ dwpe, long long T, int H, int S
                                 PB_DBG_PARAMS) {
  const int vec = H / 4;
  const long long total = T * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int v = (int)(i % vec);
    if (!PB_DBG_IN_RANGE(ids[t])) continue;
    const uint2 raw = *reinterpret_cast<const uint2*>(dout + t * H + v * 4);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 lo = __bfloat1622float2(b[0]), hi = __bfloat1622float2(b[1]);
    const float4 g = make_float4(lo.x, lo.y, hi.x, hi.y);
    atomicAdd(reinterpret_cast<float4*>(dwte + ids[t] * H) + v, g);
    if (dwpe) atomicAdd(reinterpret_cast<float4*>(dwpe + (long long)(t % S) * H) + v, g);
  }
}

}  // namespace pbm

extern "C" {

// `vocab` (rows of wte) is only used by the debug build's bounds check.
int pb_embed_fwd(const long long* ids, const void* wte, const void* wpe, void* out, long long T, int H, int S,
                 long long vocab, void* stream_) {
  using namespace pbm;
  if (H % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  long long g = (T * (H / 8) + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  embed_fwd_kernel<<<(unsigned)g, 256, 0, stream>>>(ids, reinterpret_cast<const __nv_bfloat16*>(wte),
                                                    reinterpret_cast<const __nv_bfloat16*>(wpe),
                                                    reinterpret_cast<__nv_bfloat16*>(out), T, H, S PB_DBG_ARGS(vocab));
  (void)vocab;
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

int pb_embed_bwd(const long long* ids, const void* dout, float* dwte, float* dwpe, long long T, int H, int S,
                 long long vocab, void* stream_) {
  using namespace pbm;
  if (H % 4 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  long long g = (T * (H / 4) + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  embed_bwd_kernel<<<(unsigned)g, 256, 0, stream>>>(ids, reinterpret_cast<const __nv_bfloat16*>(dout), dwte, dwpe, T,
                                                    H, S PB_DBG_ARGS(vocab));
  (void)vocab;
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // extern "C"
