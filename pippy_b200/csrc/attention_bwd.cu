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
// Small-N MMAs with both operands in shared memory are bound by the shared-memory port (a 128 x 64 x 16 step reads
// 6 KB for 32 cycles of math), so every A operand that can live in TMEM does: the bf16 P^T / dS^T (dS) tiles are
// written back over the fp32 score columns they were computed from, and in the dQ pass the resident Q and dO rows
// are loaded from global memory straight into TMEM, leaving only the streamed tile on the port.
// Score tiles are double-buffered in TMEM: the score GEMMs of block i+1 run while block i is in the softmax.
// The softmax-gradient work is latency-bound (TMEM loads, barrier round trips, the proxy fence), so two groups of
// eight warps take the even and the odd blocks: each group owns one TMEM score buffer and one P/dS buffer, the
// groups drift apart in phase, and every scheduler has four warps to switch between.
// A small pre-pass computes delta = rowsum(dO * O).
#include "tc05.cuh"

#include <math_constants.h>
#include <string.h>

extern "C" void pb_count_launch(int n);

namespace pbb {

using namespace pb;

template <bool V>
struct MaskTag {
  static constexpr bool value = V;
};

// one MUFU instruction; the argument is log2 of a probability (<= 0 up to rounding), very negative ones flush to 0
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct BwdParams {
  const float* lse;    // [B, Hq, S] natural log
  const float* delta;  // [B, Hq, S]
  const __nv_bfloat16* res1;  // mode 1: Q rows (resident A operand, loaded straight into TMEM)
  const __nv_bfloat16* res2;  // mode 1: dO rows
  long long res1_stride, res2_stride;
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
constexpr int kThreads = 64 + 2 * 256;  // TMA warp, MMA warp, two softmax groups of 8 warps

template <int D, int kMode>
__global__ void __launch_bounds__(kThreads, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
              const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2, BwdParams p) {
  constexpr int NCH = D / 64;
  constexpr int CH_A = 128 * 128;  // resident chunk: 128 rows x 128 B
  constexpr int CH_B = 64 * 128;   // streamed chunk: 64 rows x 128 B
  constexpr int RES_BYTES = NCH * CH_A;
  constexpr int STR_BYTES = NCH * CH_B;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (smem != smem_raw) {
    // the launch reserves no slack for re-alignment; refuse to run rather than overrun shared memory
    if (threadIdx.x == 0) atomicExch(p.err, ERR_BAD_ARG);
    return;
  }
  uint8_t* sX1 = smem;
  uint8_t* sX2 = sX1 + RES_BYTES;
  uint8_t* sY1 = sX2 + RES_BYTES;        // NST stages
  uint8_t* sY2 = sY1 + NST * STR_BYTES;  // NST stages
  float* s_lse = reinterpret_cast<float*>(sY2 + NST * STR_BYTES);  // [2 groups][2 buffers][64]
  float* s_delta = s_lse + 256;                             // [2 groups][2 buffers][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 256);
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
    mbar_init(res_full, kMode == 0 ? 1 : 256);
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
  const uint32_t tAccA = tmem_base + 256;  // D columns (mode 0 only)
  const uint32_t tAccB = tmem_base + 384;  // D columns
  const uint32_t tRes1 = tmem_base + 256;  // mode 1: Q as bf16 pairs, D / 2 columns
  const uint32_t tRes2 = tmem_base + 320;  // mode 1: dO as bf16 pairs, D / 2 columns

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      if (kMode == 0) {
        mbar_expect_tx(res_full, 2 * RES_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sX1 + c * CH_A, &tmX1, res_full, head_res * D + c * 64, row_base + r0);
          tma_load_2d(sX2 + c * CH_A, &tmX2, res_full, head_res * D + c * 64, row_base + r0);
        }
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
    // The whole warp walks the loop (waits included) so that control flow stays warp-uniform; one elected lane,
    // the same every time, issues the MMAs and their commits.
    {
      const uint32_t idesc_t = make_idesc_bf16(128, BS, 0, 0);
      const uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
      bool ok = true;
      auto issue_scores = [&](int it) {
        const int s = it & 1;
        const int ys = it % NST;
        // descriptors differ only in the start address (low 14 bits, in 16-byte units): add the step offset
        const uint64_t x1 = make_smem_desc(smem_u32(sX1), 16, 1024), x2 = make_smem_desc(smem_u32(sX2), 16, 1024);
        const uint64_t y1 = make_smem_desc(smem_u32(sY1 + ys * STR_BYTES), 16, 1024);
        const uint64_t y2 = make_smem_desc(smem_u32(sY2 + ys * STR_BYTES), 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t oa = ((kk >> 2) * CH_A + (kk & 3) * 32) >> 4;
            const uint32_t ob = ((kk >> 2) * CH_B + (kk & 3) * 32) >> 4;
            if (kMode == 0) umma_ss<1>(tT1 + s * 64, x1 + oa, y1 + ob, idesc_t, kk != 0);
            else umma_ts(tT1 + s * 64, tRes1 + kk * 8, y1 + ob, idesc_t, kk != 0);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t oa = ((kk >> 2) * CH_A + (kk & 3) * 32) >> 4;
            const uint32_t ob = ((kk >> 2) * CH_B + (kk & 3) * 32) >> 4;
            if (kMode == 0) umma_ss<1>(tT2 + s * 64, x2 + oa, y2 + ob, idesc_t, kk != 0);
            else umma_ts(tT2 + s * 64, tRes2 + kk * 8, y2 + ob, idesc_t, kk != 0);
          }
        umma_commit(&t_full[s]);
        }
        __syncwarp();
      };
      ok = mbar_wait(res_full, 0, abort_flag) && (n_it == 0 || mbar_wait(&y_full[0], 0, abort_flag));
      ok = __all_sync(0xffffffffu, ok);
      if (ok && n_it > 0) {
        tc_fence_after_sync();
        issue_scores(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        if (it + 1 < n_it) {
          ok = __all_sync(0xffffffffu, mbar_wait(&y_full[(it + 1) % NST], ((it + 1) / NST) & 1, abort_flag));
          if (!ok) break;
          tc_fence_after_sync();
          issue_scores(it + 1);
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&ds_ready[s], (it >> 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after_sync();
        const int ys = it % NST;
        // the streamed tiles again, now as MN-major B operands (64-wide chunks CH_B apart, 16 k-rows per step)
        const uint64_t y1 = make_smem_desc(smem_u32(sY1 + ys * STR_BYTES), CH_B, 1024);
        const uint64_t y2 = make_smem_desc(smem_u32(sY2 + ys * STR_BYTES), CH_B, 1024);
        // A operands from TMEM: the softmax threads wrote bf16 pairs over the score columns; the 16 query
        // (mode 0) / key (mode 1) indices of step kk sit in 8 columns at (kk >> 1) * 32 + (kk & 1) * 8.
        // In mode 0 a new query head restarts nothing: dK/dV accumulate over every head of the group.
        if (elect_one()) {
          if (kMode == 0) {
#pragma unroll
            for (int kk = 0; kk < BS / 16; ++kk)
              umma_ts(tAccA, tT1 + s * 64 + (kk >> 1) * 32 + (kk & 1) * 8, y2 + ((kk * 2048) >> 4), idesc_acc,
                      (it | kk) != 0);
#pragma unroll
            for (int kk = 0; kk < BS / 16; ++kk)
              umma_ts(tAccB, tT2 + s * 64 + (kk >> 1) * 32 + (kk & 1) * 8, y1 + ((kk * 2048) >> 4), idesc_acc,
                      (it | kk) != 0);
          } else {
#pragma unroll
            for (int kk = 0; kk < BS / 16; ++kk)
              umma_ts(tAccB, tT1 + s * 64 + (kk >> 1) * 32 + (kk & 1) * 8, y1 + ((kk * 2048) >> 4), idesc_acc,
                      (it | kk) != 0);
          }
        umma_commit(&y_empty[ys]);
        umma_commit(&pds_free[s]);
        }
        __syncwarp();
      }
      if (!ok && lane == 0) atomicExch(p.err, ERR_WAIT_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------ softmax-gradient threads, one resident row each
    // Two groups of 8 warps; group g takes the blocks with (it & 1) == g, i.e. always score buffer g and P/dS
    // buffer g.  Inside a group there are two warps per TMEM lane quarter, each taking 32 of the block's 64 columns.
    const int sw_warp = warp - 2;          // 0..15
    const int group = sw_warp >> 3;        // 0..1
    const int half = (sw_warp >> 2) & 1;   // column half of the block
    const int quarter = warp & 3;          // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;
    const int gtid = (threadIdx.x - 64) & 255;  // index inside the group
    const int res_idx = r0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int s = group;
    bool ok = true;
    float my_lse2 = 0.f, my_delta = 0.f;
    if (kMode == 1 && res_idx < p.S) {
      const long long off = ((long long)b * p.Hq + head_res) * p.S + res_idx;
      my_lse2 = p.lse[off] * 1.4426950408889634f;
      my_delta = p.delta[off];
    }
    // mode 0: the statistics of a block's 64 queries are fetched one block of this group ahead, so that the global
    // load is not on the critical path of the block that needs it
    auto load_stat = [&](int it2) -> float {
      float val = 0.f;
      if (gtid < 128 && it2 < n_it) {
        const int head_q = hkv * G + it2 / nblk_per_head;
        const int qi = (blk_start + it2 % nblk_per_head) * BS + (gtid & 63);
        if (qi < p.S) {
          const long long off = ((long long)b * p.Hq + head_q) * p.S + qi;
          val = (gtid < 64) ? p.lse[off] * 1.4426950408889634f : p.delta[off];
        }
      }
      return val;
    };
    float stat_next = 0.f;
    if (kMode == 0) stat_next = load_stat(group);
    if (kMode == 1 && group == 0) {
      // resident A operands: this thread's row of Q (half 0) or dO (half 1), two bf16 per TMEM column
      const __nv_bfloat16* src = (half == 0 ? p.res1 : p.res2) +
                                 (long long)(row_base + res_idx) * (half == 0 ? p.res1_stride : p.res2_stride) +
                                 head_res * D;
      const uint32_t dst = (half == 0 ? tRes1 : tRes2) + lane_off;
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t w[32];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          uint4 x = make_uint4(0u, 0u, 0u, 0u);
          if (res_idx < p.S) x = __ldg(reinterpret_cast<const uint4*>(src + c * 64) + u);
          w[u * 4] = x.x; w[u * 4 + 1] = x.y; w[u * 4 + 2] = x.z; w[u * 4 + 3] = x.w;
        }
        tmem_st_32x32(dst + c * 32, w);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(res_full);
    }

    for (int it = group; it < n_it; it += 2) {
      const int sb = (it >> 1) & 1;
      const float* lse_buf = s_lse + (group * 2 + sb) * 64;
      const float* dl_buf = s_delta + (group * 2 + sb) * 64;
      int blk;
      if (kMode == 0) {
        blk = blk_start + it % nblk_per_head;
        if (gtid < 64) s_lse[(group * 2 + sb) * 64 + gtid] = stat_next;
        else if (gtid < 128) s_delta[(group * 2 + sb) * 64 + (gtid - 64)] = stat_next;
        stat_next = load_stat(it + 2);
      } else {
        blk = it;
      }
      const int c0 = blk * BS;
      bool got = mbar_wait(&t_full[s], (it >> 1) & 1, abort_flag);
      // (the accumulation GEMMs that read this group's P / dS columns one group-iteration ago ran before the score
      // GEMMs that t_full just reported: the tensor pipe executes its MMAs in issue order)
      // the group leaves the loop together (a thread that gave up must not leave the others at the barrier);
      // the barrier also publishes the group's s_lse / s_delta
      if (kMode == 0) got = !named_bar_or(1 + group, 256, !got);
      if (!got) { ok = false; break; }
      __syncwarp();
      tc_fence_after_sync();
      bool need_mask;
      if (kMode == 0) need_mask = (p.causal && (c0 < r0 + BR - 1)) || (c0 + BS > p.S) || (r0 + BR > p.S);
      else need_mask = (p.causal && (c0 + BS - 1 > r0)) || (c0 + BS > p.S) || (r0 + BR > p.S);

      // 16 columns at a time: load S and dP, form P and dS' = P * (dP - delta) (the softmax scale is applied once
      // to the accumulated dQ / dK in the epilogue), write the bf16 pairs back over the same columns.  A small live
      // set leaves the scheduler room to overlap the exponentials of one element with the arithmetic of others.
      const uint32_t ta = s * 64 + lane_off + half * 32;
      // The masked variant (diagonal and ragged blocks only) is a separate instantiation: a per-element test of a
      // run-time flag costs a branch per element, which serialises the otherwise independent elements.
      auto do_block = [&](auto masked) {
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t t1[16], t2[16];
          tmem_ld_32x16(tT1 + ta + ch * 16, t1);
          tmem_ld_32x16(tT2 + ta + ch * 16, t2);
          tmem_ld_wait();
          uint32_t pk_p[8], pk_ds[8];  // 16 bf16 each
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            float lse2[2], dl2[2];
            if (kMode == 0) {
              const float2 a = *reinterpret_cast<const float2*>(&lse_buf[half * 32 + ch * 16 + e]);
              const float2 d2 = *reinterpret_cast<const float2*>(&dl_buf[half * 32 + ch * 16 + e]);
              lse2[0] = a.x; lse2[1] = a.y;
              dl2[0] = d2.x; dl2[1] = d2.y;
            } else {
              lse2[0] = lse2[1] = my_lse2;
              dl2[0] = dl2[1] = my_delta;
            }
            float pv[2], dv[2];
#pragma unroll
            for (int w = 0; w < 2; ++w) {
              float pr = fast_exp2(__uint_as_float(t1[e + w]) * p.scale_log2 - lse2[w]);
              if constexpr (decltype(masked)::value) {
                const int str_idx = c0 + half * 32 + ch * 16 + e + w;
                const int qi = (kMode == 0) ? str_idx : res_idx;
                const int ki = (kMode == 0) ? res_idx : str_idx;
                const bool valid = (qi < p.S) && (ki < p.S) && (!p.causal || ki <= qi);
                pr = valid ? pr : 0.f;
              }
              pv[w] = pr;
              dv[w] = pr * (__uint_as_float(t2[e + w]) - dl2[w]);
            }
            __nv_bfloat162 a0 = __floats2bfloat162_rn(pv[0], pv[1]);
            __nv_bfloat162 d0 = __floats2bfloat162_rn(dv[0], dv[1]);
            pk_p[e / 2] = *reinterpret_cast<uint32_t*>(&a0);
            pk_ds[e / 2] = *reinterpret_cast<uint32_t*>(&d0);
          }
          // back into TMEM over this thread's own score columns: 16 values = 8 columns at half * 32 + ch * 8
          if (kMode == 0) tmem_st_32x8(tT1 + ta + ch * 8, pk_p);
          tmem_st_32x8((kMode == 0 ? tT2 : tT1) + ta + ch * 8, pk_ds);
        }
      };
      if (need_mask) do_block(MaskTag<true>{});
      else do_block(MaskTag<false>{});
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&ds_ready[s]);
    }
    if (ok && n_it > 0 && group == ((n_it - 1) & 1)) {
      // commits complete in order, so the last block's barrier covers every accumulation GEMM.  Only the group
      // that owns the last block has followed every phase of that barrier; a parity wait by the other group could
      // be satisfied by an older phase, so it learns of the completion through the barrier below instead.
      if (!mbar_wait(&pds_free[group], ((n_it - 1) >> 1) & 1, abort_flag)) ok = false;
    }
    if (named_bar_or(3, 512, !ok)) ok = false;
    __syncwarp();
    if (ok) {
      tc_fence_after_sync();
      const bool row_ok = res_idx < p.S;
      constexpr int EC = D / 4;        // accumulator columns per warp: four warps share a lane quarter
      const int sub = sw_warp >> 2;    // 0..3
#pragma unroll 1
      for (int which = (kMode == 0 ? 0 : 1); which < 2; ++which) {
        const uint32_t tA = (which == 0 ? tAccA : tAccB) + lane_off + sub * EC;
        __nv_bfloat16* base = (which == 0 ? p.out_a : p.out_b);
        const float out_scale = (which == 0) ? 1.f : p.scale;  // dV is exact; dK / dQ carry the softmax scale
        uint32_t v[EC];
        if (n_it > 0) {
          if constexpr (EC == 32) tmem_ld_32x32(tA, v);
          else tmem_ld_32x16(tA, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < EC; ++e) v[e] = 0u;
        }
        if (row_ok) {
          __nv_bfloat16* dst = base + (long long)(row_base + res_idx) * p.out_stride + head_res * D + sub * EC;
#pragma unroll
          for (int u = 0; u < EC / 8; ++u) {
            uint4 w;
            __nv_bfloat162* wb = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wb[e] = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + e * 2]) * out_scale,
                                            __uint_as_float(v[u * 8 + e * 2 + 1]) * out_scale);
            reinterpret_cast<uint4*>(dst)[u] = w;
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

// delta[b, h, s] = sum_d dO * O.  D / 8 lanes share one (token, head) row with one 16-byte load each from dO and O;
// every lane group takes kRows consecutive rows so that 2 * kRows loads are in flight per lane.  Rows are split into
// (token, head) and tokens into (batch, position) once per thread and then stepped: a division per row made the
// one-warp-per-row version of this kernel instruction-bound.
template <int D, int kRows>
__global__ void __launch_bounds__(256) fa_delta_kernel(const __nv_bfloat16* __restrict__ dO,
                                                       const __nv_bfloat16* __restrict__ O, float* __restrict__ delta,
                                                       int total, int S, int Hq, long long do_stride,
                                                       long long o_stride) {
  constexpr int LPR = D / 8;  // lanes per row: 16 (D = 128) or 8 (D = 64)
  const int sub = threadIdx.x % LPR;
  const unsigned group = (blockIdx.x * blockDim.x + threadIdx.x) / LPR;
  const unsigned first = group * kRows;  // the launcher keeps total + 256 * kRows below 2^31
  int t = (int)(first / (unsigned)Hq), h = (int)(first - (unsigned)t * Hq);
  int bb = t / S, s = t - bb * S;
  const int h0 = h, bb0 = bb, s0 = s;
  uint4 a[kRows], c[kRows];
  {
    long long tt = t;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      if (first + r < (unsigned)total) {
        a[r] = *reinterpret_cast<const uint4*>(dO + tt * do_stride + h * D + sub * 8);
        c[r] = *reinterpret_cast<const uint4*>(O + tt * o_stride + h * D + sub * 8);
      } else {
        a[r] = make_uint4(0, 0, 0, 0);
        c[r] = make_uint4(0, 0, 0, 0);
      }
      if (++h == Hq) {
        h = 0;
        ++tt;
      }
    }
  }
  h = h0, bb = bb0, s = s0;
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&a[r]);
    const __nv_bfloat162* y = reinterpret_cast<const __nv_bfloat162*>(&c[r]);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 xf = __bfloat1622float2(x[i]), yf = __bfloat1622float2(y[i]);
      acc += xf.x * yf.x + xf.y * yf.y;
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (sub == 0 && first + r < (unsigned)total) delta[((long long)bb * Hq + h) * S + s] = acc;
    if (++h == Hq) {
      h = 0;
      if (++s == S) {
        s = 0;
        ++bb;
      }
    }
  }
}

template <int D, int kMode>
static int launch_bwd(const CUtensorMap& x1, const CUtensorMap& x2, const CUtensorMap& y1, const CUtensorMap& y2,
                      const BwdParams& p, cudaStream_t stream) {
  constexpr int NCH = D / 64;
  constexpr int SMEM = 2 * NCH * 128 * 128 + 2 * NST * NCH * 64 * 128 + 2048 + 256;
  auto kern = fa_bwd_kernel<D, kMode>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((p.S + BR - 1) / BR, kMode == 0 ? p.Hkv : p.Hq, p.B);
  kern<<<grid, kThreads, SMEM, stream>>>(x1, x2, y1, y2, p);
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
  if ((reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(o)) & 15) return -3;  // 16-byte loads below
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const uint64_t T = (uint64_t)B * S;
  {
    constexpr int kRows = 4;
    const long long rows = (long long)T * Hq;
    if (rows > 0x7fffffffLL - 256 * kRows) return -4;  // the delta kernel indexes rows with 32 bits
    const int lpr = D / 8;
    const long long threads_needed = (rows + kRows - 1) / kRows * lpr;
    const unsigned blocks = (unsigned)((threads_needed + 255) / 256);
    auto DO = reinterpret_cast<const __nv_bfloat16*>(dO);
    auto OO = reinterpret_cast<const __nv_bfloat16*>(o);
    if (D == 128)
      fa_delta_kernel<128, kRows><<<blocks, 256, 0, stream>>>(DO, OO, delta, (int)rows, S, Hq, do_stride, o_stride);
    else
      fa_delta_kernel<64, kRows><<<blocks, 256, 0, stream>>>(DO, OO, delta, (int)rows, S, Hq, do_stride, o_stride);
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
  p.res1 = reinterpret_cast<const __nv_bfloat16*>(q);
  p.res2 = reinterpret_cast<const __nv_bfloat16*>(dO);
  p.res1_stride = q_stride;
  p.res2_stride = do_stride;
  rc = (D == 128) ? launch_bwd<128, 1>(q128, do128, k64, v64, p, stream) : launch_bwd<64, 1>(q128, do128, k64, v64, p, stream);
  return rc;
}

}  // extern "C"
