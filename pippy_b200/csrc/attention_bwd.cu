// Causal flash attention backward for sm_100a, built from the same tcgen05/TMEM/TMA pieces as the forward.
//
// Two passes share one templated kernel (no atomics, deterministic):
//   mode 0 (dK, dV): a CTA keeps one 128-row KV tile resident and streams 64-row Q/dO blocks of every query head
//                    of its KV group:  S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T (bf16, smem)  ->
//                    dV += P^T dO, dK += dS^T Q
//   mode 1 (dQ):     a CTA keeps one 128-row Q/dO tile resident and streams 64-row K/V blocks:
//                    S = Q K^T, dP = dO V^T -> dS (bf16, smem) -> dQ += dS K
// In both, TMEM lane = resident row, so each thread owns one row of the score tile.  The streamed operand tiles
// serve twice: K-major for the score GEMMs and, reinterpreted as MN-major, for the accumulation GEMMs.
// Score tiles are double-buffered in TMEM: the score GEMMs of block i+1 run while block i is in the softmax.
// A small pre-pass computes delta = rowsum(dO * O).
#include "tc05.cuh"

#include <math_constants.h>
#include <string.h>

extern "C" void pb_count_launch(int n);

namespace pbb {

using namespace pb;

struct BwdParams {
  const float* lse;    // [B, Hq, S] natural log
  const float* delta;  // [B, Hq, S]
  __nv_bfloat16* out_a;  // mode 0: dV;  mode 1: unused
  __nv_bfloat16* out_b;  // mode 0: dK;  mode 1: dQ
  long long out_stride;
  int B, S, Hq, Hkv;
  float scale, scale_log2;
  int causal;
  int* err;
};

constexpr int BR = 128;  // resident rows
constexpr int BS = 64;   // streamed rows per block
constexpr int NST = 3;   // stages of the streamed operands (TMA latency hides behind two blocks of MMAs)

template <int D, int kMode>
__global__ void __launch_bounds__(320, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
              const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2, BwdParams p) {
  constexpr int NCH = D / 64;
  constexpr int CH_A = 128 * 128;  // resident chunk: 128 rows x 128 B
  constexpr int CH_B = 64 * 128;   // streamed chunk: 64 rows x 128 B
  constexpr int RES_BYTES = NCH * CH_A;
  constexpr int STR_BYTES = NCH * CH_B;
  constexpr int PS_BYTES = 128 * 128;  // 128 rows x 64 bf16

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX1 = smem;
  uint8_t* sX2 = sX1 + RES_BYTES;
  uint8_t* sY1 = sX2 + RES_BYTES;        // NST stages
  uint8_t* sY2 = sY1 + NST * STR_BYTES;  // NST stages
  uint8_t* sP = sY2 + NST * STR_BYTES;   // 2 buffers
  uint8_t* sdS = sP + 2 * PS_BYTES;   // 2 buffers
  float* s_lse = reinterpret_cast<float*>(sdS + 2 * PS_BYTES);  // [2][64]
  float* s_delta = s_lse + 128;                             // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 128);
  uint64_t* res_full = bars;
  uint64_t* y_full = bars + 1;           // [NST]
  uint64_t* y_empty = bars + 1 + NST;    // [NST]
  uint64_t* t_full = bars + 1 + 2 * NST;  // [2]
  uint64_t* ds_ready = t_full + 2;       // [2]
  uint64_t* pds_free = ds_ready + 2;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pds_free + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int b = blockIdx.z;
  const int row_base = b * p.S;

  // ---- work decomposition
  int r0;         // first resident row (sequence index)
  int head_res;   // head of the resident tiles (kv head in mode 0, q head in mode 1)
  int hkv;
  int blk_start, nblk_per_head, n_it;
  if (kMode == 0) {
    const int kt = blockIdx.x;
    r0 = kt * BR;
    hkv = blockIdx.y;
    head_res = hkv;
    blk_start = p.causal ? (r0 / BS) : 0;
    nblk_per_head = (p.S + BS - 1) / BS - blk_start;
    n_it = G * nblk_per_head;
  } else {
    const int nqt = (p.S + BR - 1) / BR;
    const int qt = nqt - 1 - blockIdx.x;
    r0 = qt * BR;
    head_res = blockIdx.y;
    hkv = head_res / G;
    blk_start = 0;
    const int kv_end = p.causal ? min(p.S, r0 + BR) : p.S;
    nblk_per_head = (kv_end + BS - 1) / BS;
    n_it = nblk_per_head;
  }

  if (threadIdx.x == 0) {
    mbar_init(res_full, 1);
    for (int i = 0; i < NST; ++i) {
      mbar_init(&y_full[i], 1);
      mbar_init(&y_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&ds_ready[i], 256);
      mbar_init(&pds_free[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc<1>(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tT1 = tmem_base;          // 2 x 64 columns
  const uint32_t tT2 = tmem_base + 128;    // 2 x 64 columns
  const uint32_t tAccA = tmem_base + 256;  // D columns
  const uint32_t tAccB = tmem_base + 384;  // D columns

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(res_full, 2 * RES_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        tma_load_2d(sX1 + c * CH_A, &tmX1, res_full, head_res * D + c * 64, row_base + r0);
        tma_load_2d(sX2 + c * CH_A, &tmX2, res_full, head_res * D + c * 64, row_base + r0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it % NST;
        if (!mbar_wait(&y_empty[s], ((it / NST) & 1) ^ 1, abort_flag)) { ok = false; break; }
        int head_str, blk;
        if (kMode == 0) {
          head_str = hkv * G + it / nblk_per_head;
          blk = blk_start + it % nblk_per_head;
        } else {
          head_str = hkv;
          blk = it;
        }
        mbar_expect_tx(&y_full[s], 2 * STR_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sY1 + s * STR_BYTES + c * CH_B, &tmY1, &y_full[s], head_str * D + c * 64, row_base + blk * BS);
          tma_load_2d(sY2 + s * STR_BYTES + c * CH_B, &tmY2, &y_full[s], head_str * D + c * 64, row_base + blk * BS);
        }
      }
      if (!ok) atomicExch(p.err, ERR_WAIT_TIMEOUT);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_t = make_idesc_bf16(128, BS, 0, 0);
      const uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
      bool ok = true;
      auto issue_scores = [&](int it) {
        const int s = it & 1;
        const int ys = it % NST;
        const uint32_t x1 = smem_u32(sX1), x2 = smem_u32(sX2);
        const uint32_t y1 = smem_u32(sY1 + ys * STR_BYTES), y2 = smem_u32(sY2 + ys * STR_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t oa = (kk >> 2) * CH_A + (kk & 3) * 32;
          const uint32_t ob = (kk >> 2) * CH_B + (kk & 3) * 32;
          umma_ss<1>(tT1 + s * 64, make_smem_desc(x1 + oa, 16, 1024), make_smem_desc(y1 + ob, 16, 1024), idesc_t,
                     kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t oa = (kk >> 2) * CH_A + (kk & 3) * 32;
          const uint32_t ob = (kk >> 2) * CH_B + (kk & 3) * 32;
          umma_ss<1>(tT2 + s * 64, make_smem_desc(x2 + oa, 16, 1024), make_smem_desc(y2 + ob, 16, 1024), idesc_t,
                     kk != 0);
        }
        umma_commit(&t_full[s]);
      };
      ok = mbar_wait(res_full, 0, abort_flag) && (n_it == 0 || mbar_wait(&y_full[0], 0, abort_flag));
      if (ok && n_it > 0) {
        tc_fence_after_sync();
        issue_scores(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        if (it + 1 < n_it) {
          if (!mbar_wait(&y_full[(it + 1) % NST], ((it + 1) / NST) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          issue_scores(it + 1);
        }
        if (!mbar_wait(&ds_ready[s], (it >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const int ys = it % NST;
        const uint32_t y1 = smem_u32(sY1 + ys * STR_BYTES), y2 = smem_u32(sY2 + ys * STR_BYTES);
        // in mode 0 a new query head restarts nothing: dK/dV accumulate over every head of the group
        if (kMode == 0) {
          const uint32_t pa = smem_u32(sP + s * PS_BYTES);
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk)
            umma_ss<1>(tAccA, make_smem_desc(pa + kk * 32, 16, 1024), make_smem_desc(y2 + kk * 2048, CH_B, 1024),
                       idesc_acc, (it | kk) != 0);
        }
        const uint32_t da = smem_u32(sdS + s * PS_BYTES);
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          umma_ss<1>(tAccB, make_smem_desc(da + kk * 32, 16, 1024), make_smem_desc(y1 + kk * 2048, CH_B, 1024),
                     idesc_acc, (it | kk) != 0);
        umma_commit(&y_empty[ys]);
        umma_commit(&pds_free[s]);
      }
      if (!ok) atomicExch(p.err, ERR_WAIT_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------ softmax-gradient threads, one resident row each
    // 8 warps: two per TMEM lane quarter, each taking 32 of the block's 64 columns, so every scheduler has two
    // warps to switch between while one waits on TMEM or the special-function unit
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int tid = threadIdx.x - 64;  // 0..255
    const int res_idx = r0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int sw = r & 7;
    bool ok = true;
    float my_lse2 = 0.f, my_delta = 0.f;
    if (kMode == 1 && res_idx < p.S) {
      const long long off = ((long long)b * p.Hq + head_res) * p.S + res_idx;
      my_lse2 = p.lse[off] * 1.4426950408889634f;
      my_delta = p.delta[off];
    }
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      int blk;
      if (kMode == 0) {
        const int head_q = hkv * G + it / nblk_per_head;
        blk = blk_start + it % nblk_per_head;
        // column statistics of this block's 64 queries
        const int qi = blk * BS + (tid & 63);
        float val = 0.f;
        if (qi < p.S) {
          const long long off = ((long long)b * p.Hq + head_q) * p.S + qi;
          val = (tid < 64) ? p.lse[off] * 1.4426950408889634f : p.delta[off];
        }
        if (tid < 64) s_lse[s * 64 + tid] = val;
        else if (tid < 128) s_delta[s * 64 + (tid - 64)] = val;
      } else {
        blk = it;
      }
      const int c0 = blk * BS;
      bool got = mbar_wait(&t_full[s], (it >> 1) & 1, abort_flag);
      if (kMode == 0) got = !named_bar_or(1, 256, !got);  // also publishes s_lse / s_delta
      if (!got) { ok = false; break; }
      __syncwarp();
      tc_fence_after_sync();
      bool need_mask;
      if (kMode == 0) need_mask = (p.causal && (c0 < r0 + BR - 1)) || (c0 + BS > p.S) || (r0 + BR > p.S);
      else need_mask = (p.causal && (c0 + BS - 1 > r0)) || (c0 + BS > p.S) || (r0 + BR > p.S);

      uint32_t pk_p[16], pk_ds[16];  // 32 bf16 each: this warp's half of the block's columns
      {
        uint32_t t1[32], t2[32];
        tmem_ld_32x32(tT1 + s * 64 + lane_off + half * 32, t1);
        tmem_ld_32x32(tT2 + s * 64 + lane_off + half * 32, t2);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float lse4[4], dl4[4];
          if (kMode == 0) {
            const float4 a = *reinterpret_cast<const float4*>(&s_lse[s * 64 + half * 32 + e]);
            const float4 d4 = *reinterpret_cast<const float4*>(&s_delta[s * 64 + half * 32 + e]);
            lse4[0] = a.x; lse4[1] = a.y; lse4[2] = a.z; lse4[3] = a.w;
            dl4[0] = d4.x; dl4[1] = d4.y; dl4[2] = d4.z; dl4[3] = d4.w;
          } else {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              lse4[w] = my_lse2;
              dl4[w] = my_delta;
            }
          }
          float pv[4], dv[4];
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int col = half * 32 + e + w;
            float pr = exp2f(__uint_as_float(t1[e + w]) * p.scale_log2 - lse4[w]);
            if (need_mask) {
              const int str_idx = c0 + col;
              const int qi = (kMode == 0) ? str_idx : res_idx;
              const int ki = (kMode == 0) ? res_idx : str_idx;
              const bool valid = (qi < p.S) && (ki < p.S) && (!p.causal || ki <= qi);
              pr = valid ? pr : 0.f;
            }
            pv[w] = pr;
            dv[w] = pr * (__uint_as_float(t2[e + w]) - dl4[w]) * p.scale;
          }
          __nv_bfloat162 a0 = __floats2bfloat162_rn(pv[0], pv[1]), a1 = __floats2bfloat162_rn(pv[2], pv[3]);
          __nv_bfloat162 d0 = __floats2bfloat162_rn(dv[0], dv[1]), d1 = __floats2bfloat162_rn(dv[2], dv[3]);
          pk_p[e / 2] = *reinterpret_cast<uint32_t*>(&a0);
          pk_p[e / 2 + 1] = *reinterpret_cast<uint32_t*>(&a1);
          pk_ds[e / 2] = *reinterpret_cast<uint32_t*>(&d0);
          pk_ds[e / 2 + 1] = *reinterpret_cast<uint32_t*>(&d1);
        }
      }
      if (it >= 2) {
        // the accumulation GEMMs that read this P / dS buffer two blocks ago must be done
        if (!mbar_wait(&pds_free[s], ((it - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int unit = (half * 4 + u) ^ sw;
        if (kMode == 0)
          *reinterpret_cast<uint4*>(sP + s * PS_BYTES + r * 128 + unit * 16) =
              make_uint4(pk_p[u * 4], pk_p[u * 4 + 1], pk_p[u * 4 + 2], pk_p[u * 4 + 3]);
        *reinterpret_cast<uint4*>(sdS + s * PS_BYTES + r * 128 + unit * 16) =
            make_uint4(pk_ds[u * 4], pk_ds[u * 4 + 1], pk_ds[u * 4 + 2], pk_ds[u * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&ds_ready[s]);
    }
    if (ok && n_it > 0) {
      // commits complete in order, so the last block's barrier covers every accumulation GEMM
      if (!mbar_wait(&pds_free[(n_it - 1) & 1], ((n_it - 1) >> 1) & 1, abort_flag)) ok = false;
    }
    __syncwarp();
    if (ok) {
      tc_fence_after_sync();
      const bool row_ok = res_idx < p.S;
#pragma unroll 1
      for (int which = (kMode == 0 ? 0 : 1); which < 2; ++which) {
        const uint32_t tA = (which == 0 ? tAccA : tAccB) + lane_off;
        __nv_bfloat16* base = (which == 0 ? p.out_a : p.out_b);
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {
          const int c = half * (D / 64) + cc;  // each half writes its own D/2 columns
          uint32_t v[32];
          if (n_it > 0) {
            tmem_ld_32x32(tA + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0u;
          }
          if (row_ok) {
            __nv_bfloat16* dst = base + (long long)(row_base + res_idx) * p.out_stride + head_res * D + c * 32;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 w;
              __nv_bfloat162* wb = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                wb[e] = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + e * 2]), __uint_as_float(v[u * 8 + e * 2 + 1]));
              reinterpret_cast<uint4*>(dst)[u] = w;
            }
          }
        }
      }
    }
    if (!ok && lane == 0) atomicExch(p.err, ERR_WAIT_TIMEOUT);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_after_sync();
  __syncwarp();
  if (warp == 1) tmem_dealloc<1>(tmem_base, 512);
}

// delta[b, h, s] = sum_d dO * O ; one warp per (token, head)
__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                float* __restrict__ delta, int B, int S, int Hq, int D, long long do_stride,
                                long long o_stride) {
  const long long gw = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * Hq;
  if (gw >= total) return;
  const int h = (int)(gw % Hq);
  const long long t = gw / Hq;
  const __nv_bfloat16* a = dO + t * do_stride + h * D;
  const __nv_bfloat16* c = O + t * o_stride + h * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(c + i));
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const long long bb = t / S, s = t % S;
    delta[(bb * Hq + h) * S + s] = acc;
  }
}

template <int D, int kMode>
static int launch_bwd(const CUtensorMap& x1, const CUtensorMap& x2, const CUtensorMap& y1, const CUtensorMap& y2,
                      const BwdParams& p, cudaStream_t stream) {
  constexpr int NCH = D / 64;
  constexpr int SMEM = 2 * NCH * 128 * 128 + 2 * NST * NCH * 64 * 128 + 4 * 128 * 128 + 1024 + 1024 + 256;
  auto kern = fa_bwd_kernel<D, kMode>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((p.S + BR - 1) / BR, kMode == 0 ? p.Hkv : p.Hq, p.B);
  kern<<<grid, 320, SMEM, stream>>>(x1, x2, y1, y2, p);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // namespace pbb

extern "C" {

// Layouts as in pb_flash_fwd. dq/dk/dv: bf16 [B*S, dqkv_stride] with head h at columns [h*D, (h+1)*D) of each
// pointer. delta: fp32 scratch/output [B, Hq, S].
int pb_flash_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse,
                 float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv, int D, long long q_stride,
                 long long k_stride, long long v_stride, long long o_stride, long long do_stride,
                 long long dqkv_stride, float softmax_scale, int causal, int* err_dev, void* stream_) {
  using namespace pbb;
  if (D != 64 && D != 128) return -1;
  if (Hq % Hkv != 0) return -2;
  if ((q_stride % 8) || (k_stride % 8) || (v_stride % 8) || (o_stride % 8) || (do_stride % 8) || (dqkv_stride % 8))
    return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const uint64_t T = (uint64_t)B * S;
  {
    const long long warps = (long long)T * Hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    fa_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dO),
                                                              reinterpret_cast<const __nv_bfloat16*>(o), delta, B, S,
                                                              Hq, D, do_stride, o_stride);
    pb_count_launch(1);
  }
  CUtensorMap q128, q64, k128, k64, v128, v64, do128, do64;
  int r = 0;
  r |= pb::make_tmap_bf16_2d(&q128, q, (uint64_t)Hq * D, T, (uint64_t)q_stride, 64, 128);
  r |= pb::make_tmap_bf16_2d(&q64, q, (uint64_t)Hq * D, T, (uint64_t)q_stride, 64, 64);
  r |= pb::make_tmap_bf16_2d(&k128, k, (uint64_t)Hkv * D, T, (uint64_t)k_stride, 64, 128);
  r |= pb::make_tmap_bf16_2d(&k64, k, (uint64_t)Hkv * D, T, (uint64_t)k_stride, 64, 64);
  r |= pb::make_tmap_bf16_2d(&v128, v, (uint64_t)Hkv * D, T, (uint64_t)v_stride, 64, 128);
  r |= pb::make_tmap_bf16_2d(&v64, v, (uint64_t)Hkv * D, T, (uint64_t)v_stride, 64, 64);
  r |= pb::make_tmap_bf16_2d(&do128, dO, (uint64_t)Hq * D, T, (uint64_t)do_stride, 64, 128);
  r |= pb::make_tmap_bf16_2d(&do64, dO, (uint64_t)Hq * D, T, (uint64_t)do_stride, 64, 64);
  if (r) return -10;
  BwdParams p;
  memset(&p, 0, sizeof(p));
  p.lse = lse;
  p.delta = delta;
  p.out_stride = dqkv_stride;
  p.B = B;
  p.S = S;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.err = err_dev;
  int rc;
  // pass 1: dK, dV (resident K, V; streamed Q, dO)
  p.out_a = reinterpret_cast<__nv_bfloat16*>(dv);
  p.out_b = reinterpret_cast<__nv_bfloat16*>(dk);
  rc = (D == 128) ? launch_bwd<128, 0>(k128, v128, q64, do64, p, stream) : launch_bwd<64, 0>(k128, v128, q64, do64, p, stream);
  if (rc) return rc;
  // pass 2: dQ (resident Q, dO; streamed K, V)
  p.out_a = nullptr;
  p.out_b = reinterpret_cast<__nv_bfloat16*>(dq);
  rc = (D == 128) ? launch_bwd<128, 1>(q128, do128, k64, v64, p, stream) : launch_bwd<64, 1>(q128, do128, k64, v64, p, stream);
  return rc;
}

}  // extern "C"
