// Persistent bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma with
// fp32 accumulators in TMEM -> tcgen05.ld epilogue with fused bias / GELU / residual / fp32
// accumulate.  C[M,N] = sum_k A(m,k) * B(n,k).
//
// Operand layouts (runtime): each operand is either K-major (stored [rows, K], K contiguous)
// or MN-major (stored [K, rows], rows contiguous), so forward (X.W^T), dgrad (dY.W) and wgrad
// (dY^T.X) all run on the same kernel without any transposed copies.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (+TMEM owner),
// warps 2..5 = epilogue (TMEM lane quarter = warp_id % 4).  The accumulator is double-buffered
// in TMEM (2 x BN columns) so the epilogue of tile i overlaps the main loop of tile i+1.
//
// kCtaGroup == 2 pairs two CTAs of a cluster on one 256 x BN tile (tcgen05 cta_group::2): each
// CTA loads its own 128 rows of A and its own half of B; the leader CTA issues the MMAs.
#include "tc05.cuh"

#include <string.h>

extern "C" void pb_count_launch(int n);

namespace pb {

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  long long ldr;
  __nv_bfloat16* aux;  // optional pre-activation output [M, ldc] (bf16), written when act != 0
  int act;             // 0 none, 1 gelu(tanh)
  int out_fp32;        // C is float (else bf16)
  int accumulate;      // C += result (fp32 output only)
  int a_mn, b_mn;      // operand majors
  int* err;
  int num_m_tiles, num_n_tiles, num_k_blocks;
  int group_m;
};

constexpr int BK = 64;
constexpr int BM_CTA = 128;

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.f + t);
}

__device__ __forceinline__ void tile_coords(int tile, const GemmParams& p, int& tm, int& tn) {
  const int per_group = p.group_m * p.num_n_tiles;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.group_m, p.num_m_tiles - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

template <int kCtaGroup, int BN, int kStages>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  constexpr int A_BYTES = BM_CTA * BK * 2;
  constexpr int BN_CTA = BN / kCtaGroup;  // B rows loaded by this CTA
  constexpr int B_BYTES = BN_CTA * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN >= 512 ? 512 : (2 * BN <= 32 ? 32 : 2 * BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;
  uint64_t* tempty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCtaGroup == 2) ? cluster_ctarank() : 0;
  const bool leader = (cta_rank == 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4 * kCtaGroup);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) tmem_alloc<kCtaGroup>(tmem_slot, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kCtaGroup == 2) cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int unit = blockIdx.x / kCtaGroup;
  const int num_units = gridDim.x / kCtaGroup;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int nkb = p.num_k_blocks;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      const uint32_t full0_remote = (kCtaGroup == 2) ? mapa_u32(smem_u32(&full[0]), 0) : 0;
      for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
        int tm, tn;
        tile_coords(tile, p, tm, tn);
        const int m0 = tm * (BM_CTA * kCtaGroup) + cta_rank * BM_CTA;
        const int n0 = tn * BN + cta_rank * BN_CTA;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          const int k0 = kb * BK;
          if constexpr (kCtaGroup == 1) {
            mbar_expect_tx(&full[stage], STAGE_BYTES);
            if (!p.a_mn) {
              tma_load_2d(a_dst, &tmA, &full[stage], k0, m0);
            } else {
#pragma unroll
              for (int i = 0; i < BM_CTA / 64; ++i) tma_load_2d(a_dst + i * 8192, &tmA, &full[stage], m0 + i * 64, k0);
            }
            if (!p.b_mn) {
              tma_load_2d(b_dst, &tmB, &full[stage], k0, n0);
            } else {
#pragma unroll
              for (int i = 0; i < BN_CTA / 64; ++i) tma_load_2d(b_dst + i * 8192, &tmB, &full[stage], n0 + i * 64, k0);
            }
          } else {
            if (leader) mbar_expect_tx(&full[stage], STAGE_BYTES * 2);
            const uint32_t bar = full0_remote + stage * 8;
            if (!p.a_mn) {
              tma_load_2d_pair(a_dst, &tmA, bar, k0, m0);
            } else {
#pragma unroll
              for (int i = 0; i < BM_CTA / 64; ++i) tma_load_2d_pair(a_dst + i * 8192, &tmA, bar, m0 + i * 64, k0);
            }
            if (!p.b_mn) {
              tma_load_2d_pair(b_dst, &tmB, bar, k0, n0);
            } else {
#pragma unroll
              for (int i = 0; i < BN_CTA / 64; ++i) tma_load_2d_pair(b_dst + i * 8192, &tmB, bar, n0 + i * 64, k0);
            }
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) atomicExch(p.err, ERR_WAIT_TIMEOUT);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_bf16(BM_CTA * kCtaGroup, BN, p.a_mn, p.b_mn);
      // K-major: 16 k-elements = 32 B inside the swizzled row; MN-major: 16 k-rows of 128 B
      const uint32_t a_kstep = p.a_mn ? 2048 : 32;
      const uint32_t b_kstep = p.b_mn ? 2048 : 32;
      const uint32_t a_lbo = p.a_mn ? 8192 : 16;
      const uint32_t b_lbo = p.b_mn ? 8192 : 16;
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = make_smem_desc(a_addr + k * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc(b_addr + k * b_kstep, b_lbo, 1024);
            umma_ss<kCtaGroup>(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          if constexpr (kCtaGroup == 1) umma_commit(&empty[stage]);
          else umma_commit_pair(&empty[stage], 3);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if constexpr (kCtaGroup == 1) umma_commit(&tfull[acc]);
        else umma_commit_pair(&tfull[acc], 3);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      if (!ok) atomicExch(p.err, ERR_WAIT_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    const bool vec_ok = (p.ldc % 8 == 0) && (p.residual == nullptr || p.ldr % 8 == 0) &&
                        (((reinterpret_cast<uintptr_t>(p.C) | reinterpret_cast<uintptr_t>(p.residual) |
                           reinterpret_cast<uintptr_t>(p.bias) | reinterpret_cast<uintptr_t>(p.aux)) &
                          15) == 0);
    for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
      int tm, tn;
      tile_coords(tile, p, tm, tn);
      const int row = tm * (BM_CTA * kCtaGroup) + cta_rank * BM_CTA + quarter * 32 + lane;
      const int n0 = tn * BN;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      __syncwarp();
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        if (row < p.M) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          const bool full_chunk = (col0 + 32 <= p.N) && vec_ok;
          if (full_chunk) {
            if (p.bias) {
              const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 b4 = __ldg(bp + q);
                const __nv_bfloat162* bb = reinterpret_cast<const __nv_bfloat162*>(&b4);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float2 f = __bfloat1622float2(bb[e]);
                  v[q * 8 + e * 2] += f.x;
                  v[q * 8 + e * 2 + 1] += f.y;
                }
              }
            }
            if (p.act == 1) {
              if (p.aux) {
                uint4* ap = reinterpret_cast<uint4*>(p.aux + (long long)row * p.ldc + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 o;
                  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                  for (int e = 0; e < 4; ++e) ob[e] = __floats2bfloat162_rn(v[q * 8 + e * 2], v[q * 8 + e * 2 + 1]);
                  ap[q] = o;
                }
              }
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
            }
            if (p.residual) {
              const uint4* rp = reinterpret_cast<const uint4*>(p.residual + (long long)row * p.ldr + col0);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 r4 = __ldg(rp + q);
                const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&r4);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float2 f = __bfloat1622float2(rb[e]);
                  v[q * 8 + e * 2] += f.x;
                  v[q * 8 + e * 2 + 1] += f.y;
                }
              }
            }
            if (p.out_fp32) {
              float4* cp = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0);
              if (p.accumulate) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  float4 o = cp[q];
                  o.x += v[q * 4];
                  o.y += v[q * 4 + 1];
                  o.z += v[q * 4 + 2];
                  o.w += v[q * 4 + 3];
                  cp[q] = o;
                }
              } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) cp[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              }
            } else {
              uint4* cp =
                  reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) ob[e] = __floats2bfloat162_rn(v[q * 8 + e * 2], v[q * 8 + e * 2 + 1]);
                cp[q] = o;
              }
            }
          } else {
            // ragged edge: scalar path
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + j;
              if (col >= p.N) break;
              float x = v[j];
              if (p.bias) x += __bfloat162float(p.bias[col]);
              if (p.act == 1) {
                if (p.aux) p.aux[(long long)row * p.ldc + col] = __float2bfloat16(x);
                x = gelu_tanh(x);
              }
              if (p.residual) x += __bfloat162float(p.residual[(long long)row * p.ldr + col]);
              if (p.out_fp32) {
                float* cp = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col;
                *cp = p.accumulate ? (*cp + x) : x;
              } else {
                reinterpret_cast<__nv_bfloat16*>(p.C)[(long long)row * p.ldc + col] = __float2bfloat16(x);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCtaGroup == 1) mbar_arrive(&tempty[acc]);
        else mbar_arrive_cluster(&tempty[acc], 0);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (!ok && lane == 0) atomicExch(p.err, ERR_WAIT_TIMEOUT);
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies still in flight time to land before shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  __syncwarp();
  if constexpr (kCtaGroup == 2) cluster_sync_all();
  tc_fence_after_sync();
  __syncwarp();
  if (warp == 1) tmem_dealloc<kCtaGroup>(tmem_base, TMEM_COLS);
}

template <int kCtaGroup, int BN, int kStages>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams p, int sm_count,
                       cudaStream_t stream) {
  constexpr int A_BYTES = BM_CTA * BK * 2;
  constexpr int B_BYTES = (BN / kCtaGroup) * BK * 2;
  constexpr int SMEM = kStages * (A_BYTES + B_BYTES) + 1024 + 256;
  auto kern = gemm_bf16_kernel<kCtaGroup, BN, kStages>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int tile_m = BM_CTA * kCtaGroup;
  p.num_m_tiles = (p.M + tile_m - 1) / tile_m;
  p.num_n_tiles = (p.N + BN - 1) / BN;
  p.num_k_blocks = (p.K + BK - 1) / BK;
  p.group_m = kCtaGroup == 1 ? 16 : 8;
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  int units = sm_count / kCtaGroup;
  if (units > tiles) units = tiles;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(units * kCtaGroup, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtaGroup;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p);
  pb_count_launch(1);
  return (int)e;
}

}  // namespace pb

static int g_sm_reserve = 0;

extern "C" {

// Leaves `n` SMs out of the persistent GEMM grid (for communication kernels that must run beside it).
void pb_set_sm_reserve(int n) { g_sm_reserve = n < 0 ? 0 : n; }
int pb_get_sm_reserve() { return g_sm_reserve; }

// C[M,N] = A.B^T with fused epilogue.  A: a_mn ? [K, M] (ld = lda) : [M, K];  B: b_mn ? [K, N] : [N, K].
// variant: 0 = automatic, 1 = single-CTA tiles (128 x 256), 2 = CTA-pair tiles (256 x 256),
//          3 = single-CTA 128 x 128.
// Returns 0 on success, a negative value for an argument error, a positive CUDA error otherwise.
int pb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                 long long ldc, int a_mn, int b_mn, const void* bias, const void* residual, long long ldr, void* aux,
                 int act, int out_fp32, int accumulate, int variant, int* err_dev, void* stream_) {
  using namespace pb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((lda % 8) || (ldb % 8)) return -2;  // TMA needs 16-byte row pitch
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (accumulate && !out_fp32) return -4;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (variant == 0) variant = (N <= 128) ? 3 : ((M >= 1024 && N >= 256) ? 2 : 1);
  const int bn = (variant == 3) ? 128 : 256;
  const int b_rows = (variant == 2) ? bn / 2 : bn;

  CUtensorMap tmA, tmB;
  int r;
  if (!a_mn) r = make_tmap_bf16_2d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 128);
  else r = make_tmap_bf16_2d(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, 64);
  if (r) return -10;
  if (!b_mn) r = make_tmap_bf16_2d(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, (uint32_t)b_rows);
  else r = make_tmap_bf16_2d(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, 64);
  if (r) return -11;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M;
  p.N = N;
  p.K = K;
  p.C = C;
  p.ldc = ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.aux = reinterpret_cast<__nv_bfloat16*>(aux);
  p.act = act;
  p.out_fp32 = out_fp32;
  p.accumulate = accumulate;
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  p.err = err_dev;
  int sms = sm_count - g_sm_reserve;
  if (sms < 2) sms = 2;
  switch (variant) {
    case 1: return launch_gemm<1, 256, 4>(tmA, tmB, p, sms, stream);
    case 2: return launch_gemm<2, 256, 6>(tmA, tmB, p, sms, stream);
    case 3: return launch_gemm<1, 128, 6>(tmA, tmB, p, sms, stream);
    default: return -5;
  }
}

}  // extern "C"
