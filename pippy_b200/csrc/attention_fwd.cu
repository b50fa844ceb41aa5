// Causal flash attention forward for sm_100a (head_dim 64 or 128, GQA, packed or separate q/k/v).
//
// One CTA owns 128 query rows of one head.  Per 128-row KV block:
//   S = Q K^T          tcgen05.mma, both operands K-major in 128B-swizzled smem, fp32 S in TMEM
//   softmax            one thread per query row reads its S row from TMEM (no shuffles) and writes bf16 P back
//                      into TMEM over the first half of the same S buffer
//   O_j = P V          tcgen05.mma with the A operand (P) in TMEM, V is the MN-major operand straight from its
//                      TMA tile: only V crosses the shared-memory port, which is what bounds small-N MMAs
// S/P is double-buffered in TMEM, so S(j+1) runs during softmax(j) and P V(j) during softmax(j+1).  O accumulates in TMEM across KV blocks; it is only rescaled when some row's running maximum grew
// by more than 2^8 (the stale maximum keeps every probability <= 256, exact after the final division by l).
// Warp roles: 0 = TMA producer, 1 = MMA issuer (+TMEM owner), 2..9 = softmax/epilogue: two warps per TMEM lane
// quarter, each owning 64 of the block's 128 columns (row maxima are exchanged through shared memory), so every
// scheduler has two warps to alternate between.
#include "tc05.cuh"

#include <math_constants.h>
#include <string.h>

extern "C" void pb_count_launch(int n);

namespace pba {

using namespace pb;

// one MUFU instruction; arguments here are <= 8 and very negative ones flush to zero, which is what softmax wants
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct FwdParams {
  __nv_bfloat16* o;  // [T, o_stride], head h at column h * D
  long long o_stride;
  float* lse;  // [B, Hq, S] natural log
  int B, S, Hq, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  int* err;
};

constexpr int BM = 128;
constexpr int BN = 128;

template <int D>
__global__ void __launch_bounds__(320, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  constexpr int NCH = D / 64;               // 64-column chunks per operand tile
  constexpr int CHUNK_BYTES = 128 * 128;    // 128 rows x 128 B
  constexpr int TILE_BYTES = NCH * CHUNK_BYTES;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (smem != smem_raw) {
    // the launch reserves no slack for re-alignment; refuse to run rather than overrun shared memory
    if (threadIdx.x == 0) atomicExch(p.err, ERR_BAD_ARG);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;      // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;  // 2 stages
  float* s_xchg = reinterpret_cast<float*>(sV + 2 * TILE_BYTES);  // [2 buffers][2 halves][128 rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_xchg + 512);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;
  uint64_t* o_full = bars + 11;
  uint64_t* p_ready = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_q_tiles = (p.S + BM - 1) / BM;
  const int qt = num_q_tiles - 1 - blockIdx.x;  // heavy (long) rows first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = qt * BM;
  const int kv_end = p.causal ? min(p.S, q0 + BM) : p.S;
  const int nblk = (kv_end + BN - 1) / BN;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&o_full[i], 1);
      mbar_init(&p_ready[i], 256);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc<1>(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS0 = tmem_base;       // S buffers: columns [0,128) and [128,256)
  const uint32_t tO = tmem_base + 256;  // O accumulator: columns [256, 256 + D)

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) tma_load_2d(sQ + c * CHUNK_BYTES, &tmQ, q_full, h * D + c * 64, row_base + q0);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&k_full[s], TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_2d(sK + s * TILE_BYTES + c * CHUNK_BYTES, &tmK, &k_full[s], hkv * D + c * 64, row_base + j * BN);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&v_full[s], TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_2d(sV + s * TILE_BYTES + c * CHUNK_BYTES, &tmV, &v_full[s], hkv * D + c * 64, row_base + j * BN);
      }
      if (!ok) atomicExch(p.err, ERR_WAIT_TIMEOUT);
    }
  } else if (warp == 1) {
    // The whole warp walks the loop (waits included) so that control flow stays warp-uniform; one elected lane,
    // the same every time, issues the MMAs and their commits.
    {
      const uint32_t idesc_s = make_idesc_bf16(128, BN, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);
      bool ok = true;
      auto issue_s = [&](int j) {
        const int s = j & 1;
        // descriptors differ only in the start address (low 14 bits, in 16-byte units): add the step offset
        const uint64_t qd = make_smem_desc(smem_u32(sQ), 16, 1024);
        const uint64_t kd = make_smem_desc(smem_u32(sK + s * TILE_BYTES), 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = ((kk >> 2) * CHUNK_BYTES + (kk & 3) * 32) >> 4;
            umma_ss<1>(tS0 + s * 128, qd + off, kd + off, idesc_s, kk != 0);
          }
          umma_commit(&s_full[s]);
          umma_commit(&k_empty[s]);
        }
        __syncwarp();
      };
      ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&k_full[0], 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < nblk) {
          ok = __all_sync(0xffffffffu, mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag));
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(j + 1);
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&p_ready[s], ph, abort_flag) && mbar_wait(&v_full[s], ph, abort_flag));
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t vd = make_smem_desc(smem_u32(sV + s * TILE_BYTES), CHUNK_BYTES, 1024);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            // A = P: 16 bf16 of K per step = 8 TMEM columns of the S/P buffer
            umma_ts(tO, tS0 + s * 128 + kk * 8, vd + ((kk * 2048) >> 4), idesc_pv, (j | kk) != 0);
          }
          umma_commit(&o_full[s]);
          umma_commit(&v_empty[s]);
        }
        __syncwarp();
      }
      if (!ok && lane == 0) atomicExch(p.err, ERR_WAIT_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (row x column half per thread)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;  // row inside the tile == TMEM lane
    const int q_idx = q0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    float m = -CUDART_INF_F, l = 0.f;  // l: this thread's half of the row sum
    bool ok = true;

    for (int j = 0; j < nblk; ++j) {
      const int s = j & 1;
      bool got = mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag);
      __syncwarp();
      tc_fence_after_sync();
      const int k0 = j * BN;
      const int col0 = half * 64;
      const bool need_mask = (p.causal && (k0 + BN - 1 > q0)) || (k0 + BN > p.S);
      const uint32_t tS = tS0 + s * 128 + lane_off + col0;
      uint32_t v[2][32];
      tmem_ld_32x32(tS, v[0]);
      tmem_ld_32x32(tS + 32, v[1]);
      tmem_ld_wait();
      float mx = -CUDART_INF_F;
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int kv = k0 + col0 + c * 32 + e;
            const bool valid = (kv < p.S) && (!p.causal || kv <= q_idx);
            if (!valid) v[c][e] = 0xff800000u;  // -inf
            mx = fmaxf(mx, __uint_as_float(v[c][e]));
          }
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(v[c][e]));
      }
      // combine with the other half of the row
      s_xchg[(s * 2 + half) * 128 + r] = mx;
      got = !named_bar_or(1, 256, !got);
      if (!got) { ok = false; break; }
      mx = fmaxf(mx, s_xchg[(s * 2 + (half ^ 1)) * 128 + r]);
      const float m_cand = fmaxf(m, mx * p.scale_log2);
      // rescale only when some row of the warp moved its maximum by more than 2^8
      const bool grow = m_cand > m + 8.f;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_use = (m_cand == -CUDART_INF_F) ? 0.f : m_cand;
        const float alpha = exp2f(m - m_use);  // 0 on the first block (m = -inf)
        if (j > 0) {
          if (!mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          __syncwarp();
          tc_fence_after_sync();
#pragma unroll
          for (int cc = 0; cc < D / 64; ++cc) {
            const uint32_t ta = tO + lane_off + (half * (D / 64) + cc) * 32;
            uint32_t o[32];
            tmem_ld_32x32(ta, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x32(ta, o);
          }
          tmem_st_wait();
        }
        l *= alpha;
        m = m_use;
      }
      // P goes back into TMEM over columns [0, 64) of this S buffer (2 bf16 per 32-bit column).  Both warps of a
      // lane quarter have their S values in registers since before the exchange barrier above, and P V(j-2), the
      // last reader of this buffer, completed before S(j) (the tensor pipe runs its MMAs in issue order).
      float rowsum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float x0 = fast_exp2(__uint_as_float(v[e >> 4][(e & 15) * 2]) * p.scale_log2 - m);
        const float x1 = fast_exp2(__uint_as_float(v[e >> 4][(e & 15) * 2 + 1]) * p.scale_log2 - m);
        rowsum += x0 + x1;
        __nv_bfloat162 w = __floats2bfloat162_rn(x0, x1);
        pk[e] = *reinterpret_cast<uint32_t*>(&w);
      }
      tmem_st_32x32(tS0 + s * 128 + lane_off + half * 32, pk);
      tmem_st_wait();
      l += rowsum;
      tc_fence_before_sync();
      mbar_arrive(&p_ready[s]);
    }
    bool got = true;
    if (ok && nblk > 0) got = mbar_wait(&o_full[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, abort_flag);
    // total row sum = both halves
    s_xchg[half * 128 + r] = l;
    got = !named_bar_or(1, 256, !(got && ok));
    if (!got) ok = false;
    __syncwarp();
    if (ok && nblk > 0) {
      tc_fence_after_sync();
      const float l_total = l + s_xchg[(half ^ 1) * 128 + r];
      const float inv_l = 1.f / l_total;
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int c = half * (D / 64) + cc;
        uint32_t o[32];
        tmem_ld_32x32(tO + lane_off + c * 32, o);
        tmem_ld_wait();
        if (q_idx < p.S) {
          __nv_bfloat16* dst = p.o + (long long)(row_base + q_idx) * p.o_stride + h * D + c * 32;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            __nv_bfloat162* wb = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wb[e] = __floats2bfloat162_rn(__uint_as_float(o[u * 8 + e * 2]) * inv_l,
                                            __uint_as_float(o[u * 8 + e * 2 + 1]) * inv_l);
            reinterpret_cast<uint4*>(dst)[u] = w;
          }
        }
      }
      if (half == 0 && q_idx < p.S)
        p.lse[((long long)b * p.Hq + h) * p.S + q_idx] = (m + log2f(l_total)) * 0.6931471805599453f;
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

template <int D>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                      cudaStream_t stream) {
  constexpr int TILE = (D / 64) * 128 * 128;
  constexpr int SMEM = 5 * TILE + 2048 + 256;
  auto kern = fa_fwd_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((p.S + BM - 1) / BM, p.Hq, p.B);
  kern<<<grid, 320, SMEM, stream>>>(tq, tk, tv, p);
  pb_count_launch(1);
  return (int)cudaGetLastError();
}

}  // namespace pba

extern "C" {

// q/k/v: bf16, token-major: row t = b * S + s, head h at columns [h * D, (h + 1) * D) of the respective pointer,
// row pitches in elements (a packed qkv buffer passes three pointers into the same rows).
// o: [B * S, o_stride] bf16; lse: [B, Hq, S] fp32.
int pb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq, int Hkv,
                 int D, long long q_stride, long long k_stride, long long v_stride, long long o_stride,
                 float softmax_scale, int causal, int* err_dev, void* stream_) {
  using namespace pba;
  if (D != 64 && D != 128) return -1;
  if (Hq % Hkv != 0) return -2;
  if ((q_stride % 8) || (k_stride % 8) || (v_stride % 8) || (o_stride % 8)) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const uint64_t T = (uint64_t)B * S;
  CUtensorMap tq, tk, tv;
  if (pb::make_tmap_bf16_2d(&tq, q, (uint64_t)Hq * D, T, (uint64_t)q_stride, 64, 128)) return -10;
  if (pb::make_tmap_bf16_2d(&tk, k, (uint64_t)Hkv * D, T, (uint64_t)k_stride, 64, 128)) return -11;
  if (pb::make_tmap_bf16_2d(&tv, v, (uint64_t)Hkv * D, T, (uint64_t)v_stride, 64, 128)) return -12;
  FwdParams p;
  memset(&p, 0, sizeof(p));
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.o_stride = o_stride;
  p.lse = lse;
  p.B = B;
  p.S = S;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.err = err_dev;
  if (D == 128) return launch_fwd<128>(tq, tk, tv, p, stream);
  return launch_fwd<64>(tq, tk, tv, p, stream);
}

}  // extern "C"
