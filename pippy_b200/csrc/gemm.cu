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
#include "peer.cuh"

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
  // ---- fused tensor-parallel modes (0 = plain GEMM)
  //   1: all-gather -> GEMM.  A is the row-wise concatenation of `world` shards of `chunk_rows` rows; this rank's
  //      shard is read in place (tmA), the others from a local gathered copy (tmA2) that copy CTAs of this same
  //      grid fill from the peers' shards while GEMM CTAs already work on the rows that have arrived.
  //   2: GEMM -> reduce-scatter.  Output rows are owned chunk-wise by the ranks; tiles of a foreign chunk are stored
  //      straight into the owner's staging slot (P2P stores), the own chunk into `C`; when everything has been
  //      sent the grid reduces own partial + received partials into `rs_out`.
  int fused;
  int rank, world, chunk_rows;
  long long lda_elems;  // row pitch (elements) of the shards and of the gathered buffer
  int m_rot;         // rotation of the M-tile order (tiles): own chunk first (mode 1) / last (mode 2)
  int gemm_ctas;     // CTAs running the GEMM roles; the rest of the grid copies (mode 1)
  int epoch;
  int* tile_flags;   // local [num_m_tiles]: rows of that M tile have landed in the gathered buffer (mode 1)
  int* counters;     // local scratch, zeroed before launch: [0] grid barrier, [1 + peer] copy CTAs done with peer
  int* flags[8];     // every rank's flag block (peer mapped): [0,W) ready, [W,2W) done / sent
  const __nv_bfloat16* peer_src[8];  // mode 1: every rank's shard [chunk_rows, K] (row pitch lda)
  __nv_bfloat16* gathered;           // mode 1: local [world * chunk_rows, K] (row pitch lda)
  __nv_bfloat16* rs_staging[8];      // mode 2: every rank's staging [world, chunk_rows, N]
  __nv_bfloat16* rs_out;             // mode 2: local result [chunk_rows, N] (row pitch ldc)
  const __nv_bfloat16* rs_residual;  // mode 2: optional [chunk_rows, N] added in the final reduce
  // ---- grouped modes (0 = plain GEMM): the rows of one operand dimension belong to `n_groups` groups (the
  // experts of a mixture-of-experts layer) whose sizes are only known on the device.  Group g occupies rows
  // [group_start[g], group_start[g] + group_rows[g]); every group_start is a multiple of 256.
  //   1: the M rows of A and C are grouped; each group multiplies its own B: a K-major B is the row-wise stack of
  //      the groups' [b_group_stride, K] matrices, an MN-major B the stack of their [b_group_stride (= K), N]
  //      matrices.  Only tiles that hold rows of a group run; output rows of such a tile beyond the group's end
  //      are written as zeros, so that a later contraction over the rows can run to the next multiple of 64.
  //   2: the contraction dimension is grouped (both operands MN-major, stored [rows, M] and [rows, N]); group g
  //      writes (or accumulates into) its own C block at C + g * c_group_stride elements.  The contraction of a
  //      group runs over whole 64-row blocks: rows between the group's end and the next multiple of 64 must be
  //      zero in one operand and finite in the other.
  int grouped;
  int n_groups;
  const int* group_rows;
  const int* group_start;
  int b_group_stride;
  long long c_group_stride;
};

constexpr int MAX_GROUPS = 8;

// Group table in shared memory, built by every CTA from the device-side sizes.
struct GroupTable {
  int prefix[MAX_GROUPS + 1];  // mode 1: M tiles before group g
  int start[MAX_GROUPS];
  int rows[MAX_GROUPS];
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

__device__ __forceinline__ void tile_coords(int tile, const GemmParams& p, int num_m_tiles, int& tm, int& tn) {
  const int per_group = p.group_m * p.num_n_tiles;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.group_m, num_m_tiles - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
  if (p.fused == 1) {
    tm += p.m_rot;
    if (tm >= p.num_m_tiles) tm -= p.num_m_tiles;
  } else if (p.fused == 2) {
    // reduce-scatter: walk the owners round-robin, one tile group at a time, starting with the next rank, so the
    // stores to each peer are spread over the whole kernel instead of bursting at its start
    const int tiles_per_chunk = p.num_m_tiles / p.world;
    if (tiles_per_chunk % p.group_m == 0) {
      const int grp = tm / p.group_m, within = tm % p.group_m;
      const int chunk = (p.rank + 1 + grp) % p.world;
      tm = chunk * tiles_per_chunk + (grp / p.world) * p.group_m + within;
    } else {
      tm += p.m_rot;
      if (tm >= p.num_m_tiles) tm -= p.num_m_tiles;
    }
  }
}

template <int kCtaGroup, int BN, int kStages>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, GemmParams p) {
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
  GroupTable* gt = reinterpret_cast<GroupTable*>(smem + kStages * STAGE_BYTES + 152);  // 100 bytes of the 256
  static_assert((2 * kStages + 4) * 8 + 8 <= 152, "barriers overlap the group table");
  uint8_t* sEpi = smem + kStages * STAGE_BYTES + 256;  // 4 epilogue warps x 32 rows x (128 + 16) bytes

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
    if (p.grouped) {
      int acc_tiles = 0;
      for (int g = 0; g < MAX_GROUPS; ++g) {
        const int rows = g < p.n_groups ? p.group_rows[g] : 0;
        gt->prefix[g] = acc_tiles;
        gt->start[g] = g < p.n_groups ? p.group_start[g] : 0;
        gt->rows[g] = rows;
        acc_tiles += (rows + BM_CTA * kCtaGroup - 1) / (BM_CTA * kCtaGroup);
      }
      gt->prefix[MAX_GROUPS] = acc_tiles;
    }
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
  const int num_units = (p.fused == 1 ? p.gemm_ctas : (int)gridDim.x) / kCtaGroup;
  const bool copy_cta = (p.fused == 1) && ((int)blockIdx.x >= p.gemm_ctas);
  // grouped mode 1 only knows its M tiles now; mode 2 runs the full [M, N] tile grid once per group
  const int num_m_tiles = (p.grouped == 1) ? gt->prefix[MAX_GROUPS] : p.num_m_tiles;
  const int tiles_per_group = num_m_tiles * p.num_n_tiles;
  const int num_tiles = (p.grouped == 2) ? tiles_per_group * p.n_groups : tiles_per_group;
  constexpr int TILE_M_ALL = BM_CTA * kCtaGroup;
  // Where a tile lives.  Every role calls this with the same arguments, so all agree on the rows, the group and
  // the contraction range (kb0 <= kb < kb1; an empty range means the tile is skipped by everybody).
  auto locate = [&](int tile, int& tn, int& row0, int& m_limit, int& grp, int& kb0, int& kb1) {
    int tm;
    grp = 0;
    kb0 = 0;
    kb1 = p.num_k_blocks;
    if (p.grouped == 2) {
      grp = tile / tiles_per_group;
      tile -= grp * tiles_per_group;
      kb0 = gt->start[grp] / BK;
      kb1 = (gt->start[grp] + gt->rows[grp] + BK - 1) / BK;
      if (gt->rows[grp] == 0) kb1 = kb0;
    }
    tile_coords(tile, p, num_m_tiles, tm, tn);
    row0 = tm * TILE_M_ALL;
    m_limit = p.M;
    if (p.grouped == 1) {
      while (grp + 1 < MAX_GROUPS && tm >= gt->prefix[grp + 1]) ++grp;
      row0 = gt->start[grp] + (tm - gt->prefix[grp]) * TILE_M_ALL;
      m_limit = min(p.M, gt->start[grp] + gt->rows[grp]);
    }
  };

  if (copy_cta) {
    // ------------------------------------------------------------ all-gather copy role (mode 1)
    using namespace pbp;
    const int n_copy = (int)gridDim.x - p.gemm_ctas;
    const int me = (int)blockIdx.x - p.gemm_ctas;
    const int W = p.world;
    constexpr int TILE_M = BM_CTA * kCtaGroup;
    const int blocks_per_chunk = (p.chunk_rows + TILE_M - 1) / TILE_M;
    __shared__ int s_ok;
    uint32_t copy_issue = 0, copy_done = 0;
    if (me == 0 && threadIdx.x < W && (int)threadIdx.x != p.rank)
      st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);  // my shard is complete (stream order)
    for (int q = 1; q < W; ++q) {
      const int peer = (p.rank + q) % W;
      if (threadIdx.x == 0) s_ok = wait_flag_sys(p.flags[p.rank] + peer, p.epoch, p.err, ERR_PEER_TIMEOUT) ? 1 : 0;
      __syncthreads();
      if (!s_ok) break;
      const __nv_bfloat16* src = p.peer_src[peer];
      // One thread streams the rows through a ring of shared-memory slots with bulk copies (peer -> smem -> local):
      // up to kStages pieces of 32 KiB are in flight per copy CTA, enough to cover the NVLink round trip.
      if (threadIdx.x == 0) {
        constexpr uint32_t PIECE = 32768;
        bool good = true;
        for (int blk = me; blk < blocks_per_chunk && good; blk += n_copy) {
          const int r0 = blk * TILE_M;
          const int rows = min(TILE_M, p.chunk_rows - r0);
          const long long bytes_total = (long long)rows * p.lda_elems * 2;
          const char* gsrc = reinterpret_cast<const char*>(src + (long long)r0 * p.lda_elems);
          char* gdst = reinterpret_cast<char*>(p.gathered + ((long long)peer * p.chunk_rows + r0) * p.lda_elems);
          const int n_pieces = (int)((bytes_total + PIECE - 1) / PIECE);
          int issued = 0, stored = 0;
          while (stored < n_pieces) {
            while (issued < n_pieces && issued - stored < kStages) {
              const uint32_t slot = copy_issue % kStages;
              const long long off = (long long)issued * PIECE;
              const uint32_t nb = (uint32_t)min((long long)PIECE, bytes_total - off);
              mbar_expect_tx(&full[slot], nb);
              bulk_load(smem + slot * PIECE, gsrc + off, nb, &full[slot]);
              ++copy_issue;
              ++issued;
            }
            const uint32_t slot = copy_done % kStages;
            if (!mbar_wait(&full[slot], (copy_done / kStages) & 1, abort_flag)) {
              good = false;
              atomicExch(p.err, ERR_WAIT_TIMEOUT);
              break;
            }
            const long long off = (long long)stored * PIECE;
            const uint32_t nb = (uint32_t)min((long long)PIECE, bytes_total - off);
            bulk_store(gdst + off, smem + slot * PIECE, nb);
            tma_store_commit();
            tma_store_wait_read<0>();  // the slot may be refilled once the store has read it
            ++copy_done;
            ++stored;
          }
          if (!good) break;
          tma_store_wait<0>();  // rows are in local memory
          __threadfence();
          st_release_gpu(p.tile_flags + (peer * p.chunk_rows + r0) / TILE_M, p.epoch);
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        // the last copy CTA to finish with this peer tells it that its shard may be overwritten
        __threadfence();
        if (atomicAdd(p.counters + 1 + peer, 1) == n_copy - 1) st_release_sys(p.flags[peer] + W + p.rank, p.epoch);
      }
    }
    if (me == 0) {
      // do not return before every peer has finished reading my shard
      bool ok = true;
      if (threadIdx.x < W && (int)threadIdx.x != p.rank)
        ok = wait_flag_sys(p.flags[p.rank] + W + threadIdx.x, p.epoch, p.err, ERR_PEER_TIMEOUT);
      __syncthreads_and(ok);
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      const uint32_t full0_remote = (kCtaGroup == 2) ? mapa_u32(smem_u32(&full[0]), 0) : 0;
      for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
        int tn, row0, m_limit, grp, kb0, kb1;
        locate(tile, tn, row0, m_limit, grp, kb0, kb1);
        const int tm = row0 / TILE_M_ALL;  // fused modes only (never grouped)
        int m0 = row0 + cta_rank * BM_CTA;
        const int n0 = tn * BN + cta_rank * BN_CTA;
        // a grouped-M GEMM reads group `grp`'s own B: a row offset for a K-major B, a k offset for an MN-major one
        const int bn_off = (p.grouped == 1 && !p.b_mn) ? grp * p.b_group_stride : 0;
        const int bk_off = (p.grouped == 1 && p.b_mn) ? grp * p.b_group_stride : 0;
        const CUtensorMap* tma_a = &tmA;
        if (p.fused == 1) {
          const int chunk = (tm * (BM_CTA * kCtaGroup)) / p.chunk_rows;
          if (chunk == p.rank) {
            m0 -= chunk * p.chunk_rows;  // own shard, read in place
          } else {
            tma_a = &tmA2;
            if (!pbp::wait_flag_gpu(p.tile_flags + tm, p.epoch, p.err, ERR_PEER_TIMEOUT)) {
              ok = false;
              break;
            }
            asm volatile("fence.proxy.async.global;" ::: "memory");  // copied rows -> visible to the TMA engine
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
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
              tma_load_2d(a_dst, tma_a, &full[stage], k0, m0);
            } else {
#pragma unroll
              for (int i = 0; i < BM_CTA / 64; ++i) tma_load_2d(a_dst + i * 8192, tma_a, &full[stage], m0 + i * 64, k0);
            }
            if (!p.b_mn) {
              tma_load_2d(b_dst, &tmB, &full[stage], k0, n0 + bn_off);
            } else {
#pragma unroll
              for (int i = 0; i < BN_CTA / 64; ++i)
                tma_load_2d(b_dst + i * 8192, &tmB, &full[stage], n0 + i * 64, k0 + bk_off);
            }
          } else {
            if (leader) mbar_expect_tx(&full[stage], STAGE_BYTES * 2);
            const uint32_t bar = full0_remote + stage * 8;
            if (!p.a_mn) {
              tma_load_2d_pair(a_dst, tma_a, bar, k0, m0);
            } else {
#pragma unroll
              for (int i = 0; i < BM_CTA / 64; ++i) tma_load_2d_pair(a_dst + i * 8192, tma_a, bar, m0 + i * 64, k0);
            }
            if (!p.b_mn) {
              tma_load_2d_pair(b_dst, &tmB, bar, k0, n0 + bn_off);
            } else {
#pragma unroll
              for (int i = 0; i < BN_CTA / 64; ++i)
                tma_load_2d_pair(b_dst + i * 8192, &tmB, bar, n0 + i * 64, k0 + bk_off);
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
        int tn_, row0_, ml_, grp_, kb0, kb1;
        locate(tile, tn_, row0_, ml_, grp_, kb0, kb1);
        if (kb1 <= kb0) continue;  // empty group: no accumulator is produced, the epilogue skips the tile too
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
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
            umma_ss<kCtaGroup>(d_tmem, da, db, idesc, (kb != kb0) || (k != 0));
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
    uint32_t peer_ready_mask = 0;
    bool ok = true;
    if (p.fused == 2 && blockIdx.x == 0 && warp == 2 && lane < p.world && lane != p.rank)
      pbp::st_release_sys(p.flags[lane] + p.rank, p.epoch);  // "my previous reduce is over": peers may write to me
    const bool vec_ok = (p.ldc % 8 == 0) && (p.residual == nullptr || p.ldr % 8 == 0) &&
                        (((reinterpret_cast<uintptr_t>(p.C) | reinterpret_cast<uintptr_t>(p.residual) |
                           reinterpret_cast<uintptr_t>(p.bias) | reinterpret_cast<uintptr_t>(p.aux)) &
                          15) == 0);
    for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
      int tn, row0, m_limit, grp, kb0, kb1;
      locate(tile, tn, row0, m_limit, grp, kb0, kb1);
      if (kb1 <= kb0) continue;
      const int tm = row0 / TILE_M_ALL;  // fused modes only
      int row = row0 + cta_rank * BM_CTA + quarter * 32 + lane;
      const int n0 = tn * BN;
      void* c_base = p.C;
      if (p.grouped == 2)
        c_base = p.out_fp32 ? static_cast<void*>(reinterpret_cast<float*>(p.C) + grp * p.c_group_stride)
                            : static_cast<void*>(reinterpret_cast<__nv_bfloat16*>(p.C) + grp * p.c_group_stride);
      // grouped M: rows of this tile past the group's end are written as zeros (bf16 outputs)
      const bool zero_tail = (p.grouped == 1) && !p.out_fp32 && row >= m_limit && row < p.M;
      bool peer_tile = false;
      if (p.fused == 2) {
        const int chunk = (tm * (BM_CTA * kCtaGroup)) / p.chunk_rows;
        m_limit = (row < p.M) ? p.chunk_rows : 0;
        row -= chunk * p.chunk_rows;
        if (chunk != p.rank) {
          c_base = p.rs_staging[chunk] + (long long)p.rank * p.chunk_rows * p.ldc;  // my slot in the owner's staging
          // Tiles that leave over NVLink go out as whole 128-byte row pieces: a lane owns a row, so its direct
          // stores are 16-byte pieces 32 rows apart, which use a fraction of the link; two 32-column chunks are
          // staged in shared memory and written back with 8 lanes per row instead.
          peer_tile = vec_ok && !p.out_fp32 && (n0 + BN <= p.N) && (p.M % 32 == 0) && p.bias == nullptr &&
                      p.act == 0 && p.residual == nullptr;
          if (!(peer_ready_mask & (1u << chunk))) {
            // the owner must have finished reducing the previous call's partials before they are overwritten
            bool rdy = true;
            if (lane == 0) rdy = pbp::wait_flag_sys(p.flags[p.rank] + chunk, p.epoch, p.err, ERR_PEER_TIMEOUT);
            rdy = __shfl_sync(0xffffffffu, rdy, 0);
            if (!rdy) {
              ok = false;
              break;
            }
            peer_ready_mask |= 1u << chunk;
          }
        }
      }
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
        if (zero_tail) {
          __nv_bfloat16* zp = reinterpret_cast<__nv_bfloat16*>(c_base) + (long long)row * p.ldc + col0;
          if (col0 + 32 <= p.N && vec_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(zp)[q] = make_uint4(0u, 0u, 0u, 0u);
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) zp[j] = __float2bfloat16(0.f);
          }
        }
        if (row < m_limit) {
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
              float4* cp = reinterpret_cast<float4*>(reinterpret_cast<float*>(c_base) + (long long)row * p.ldc + col0);
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
                  peer_tile
                      ? reinterpret_cast<uint4*>(sEpi + ((warp - 2) * 32 + lane) * 144 + (c & 1) * 64)
                      : reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(c_base) + (long long)row * p.ldc +
                                                 col0);
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
                float* cp = reinterpret_cast<float*>(c_base) + (long long)row * p.ldc + col;
                *cp = p.accumulate ? (*cp + x) : x;
              } else {
                reinterpret_cast<__nv_bfloat16*>(c_base)[(long long)row * p.ldc + col] = __float2bfloat16(x);
              }
            }
          }
        }
        if (peer_tile && (c & 1)) {
          // 32 rows x 128 bytes staged by this warp: piece i = q * 32 + lane is bytes [16 * (i % 8), +16) of row i / 8
          __syncwarp();
          const int row_w = row - lane;  // first row of this warp's block, relative to the owner's chunk
          const uint8_t* stage = sEpi + (warp - 2) * 32 * 144;
          __nv_bfloat16* dst0 = reinterpret_cast<__nv_bfloat16*>(c_base) + n0 + (c - 1) * 32;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int i = q * 32 + lane;
            const int rr = i >> 3, part = i & 7;
            if (row_w + rr < m_limit && row_w + rr >= 0) {
              const uint4 val = *reinterpret_cast<const uint4*>(stage + rr * 144 + part * 16);
              *reinterpret_cast<uint4*>(dst0 + (long long)(row_w + rr) * p.ldc + part * 8) = val;
            }
          }
          __syncwarp();
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

  if (p.fused == 2) {
    // ------------------------------------------------------------ reduce-scatter tail: sum what arrived
    using namespace pbp;
    const int W = p.world;
    __threadfence_system();
    if (!grid_barrier(p.counters, (int)gridDim.x, p.err, ERR_PEER_TIMEOUT)) return;
    if (blockIdx.x == 0 && (int)threadIdx.x < W && (int)threadIdx.x != p.rank)
      st_release_sys(p.flags[threadIdx.x] + W + p.rank, p.epoch);  // everything I owed you has been stored
    bool ok = true;
    if ((int)threadIdx.x < W && (int)threadIdx.x != p.rank)
      ok = wait_flag_sys(p.flags[p.rank] + W + threadIdx.x, p.epoch, p.err, ERR_PEER_TIMEOUT);
    if (!__syncthreads_and(ok)) return;
    const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(p.C);
    const __nv_bfloat16* stag = p.rs_staging[p.rank];
    const int vec_per_row = p.N / 8;
    const long long total = (long long)p.chunk_rows * vec_per_row;
    // Four output vectors per thread and trip, all their loads issued before the first use: with one vector in
    // flight per thread this pass ran at a fraction of the HBM rate.
    constexpr int RU = 4;
    const long long nthr = (long long)gridDim.x * blockDim.x;
    auto add8 = [](float* accv, const uint4& u) {
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(b2[e]);
        accv[2 * e] += f.x;
        accv[2 * e + 1] += f.y;
      }
    };
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < total; i0 += nthr * RU) {
      long long off[RU];
      uint4 own[RU], res[RU];
#pragma unroll
      for (int u = 0; u < RU; ++u) {
        const long long i = i0 + u * nthr;
        off[u] = -1;
        if (i < total) {
          off[u] = (i / vec_per_row) * p.ldc + (i % vec_per_row) * 8;
          own[u] = *reinterpret_cast<const uint4*>(mine + off[u]);
          if (p.rs_residual) res[u] = *reinterpret_cast<const uint4*>(p.rs_residual + off[u]);
        }
      }
      float accv[RU][8];
#pragma unroll
      for (int u = 0; u < RU; ++u) {
#pragma unroll
        for (int e = 0; e < 8; ++e) accv[u][e] = 0.f;
        if (off[u] >= 0) {
          add8(accv[u], own[u]);
          if (p.rs_residual) add8(accv[u], res[u]);
        }
      }
      for (int src = 0; src < W; ++src) {
        if (src == p.rank) continue;
        const __nv_bfloat16* base = stag + (long long)src * p.chunk_rows * p.ldc;
        uint4 v[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u)
          if (off[u] >= 0) v[u] = *reinterpret_cast<const uint4*>(base + off[u]);
#pragma unroll
        for (int u = 0; u < RU; ++u)
          if (off[u] >= 0) add8(accv[u], v[u]);
      }
#pragma unroll
      for (int u = 0; u < RU; ++u) {
        if (off[u] < 0) continue;
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) ob[e] = __floats2bfloat162_rn(accv[u][2 * e], accv[u][2 * e + 1]);
        *reinterpret_cast<uint4*>(p.rs_out + off[u]) = o;
      }
    }
  }
}

// Tile order knob: output tiles are walked in bands of `group_m` row tiles, row-fastest inside a band (0 = default).
static int g_group_m = 0;

template <int kCtaGroup, int BN, int kStages>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams p, int sm_count,
                       cudaStream_t stream, const CUtensorMap* tmA2 = nullptr, int copy_ctas = 0,
                       int tile_multiplier = 1) {
  constexpr int A_BYTES = BM_CTA * BK * 2;
  constexpr int B_BYTES = (BN / kCtaGroup) * BK * 2;
  constexpr int SMEM = kStages * (A_BYTES + B_BYTES) + 1024 + 256 + 4 * 32 * 144;
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
  if (g_group_m > 0 && !p.fused) p.group_m = g_group_m;
  // grouped M: up to one partial tile per group on top of the dense count (p.M is the buffers' row capacity)
  const int tiles = (p.num_m_tiles + (p.grouped == 1 ? p.n_groups : 0)) * p.num_n_tiles * tile_multiplier;
  int units = (sm_count - copy_ctas) / kCtaGroup;
  if (units > tiles) units = tiles;
  if (units < 1) units = 1;
  if (p.fused) {
    const int tiles_per_chunk = p.chunk_rows / tile_m;
    // own chunk first when gathering (its rows need no transfer), last when scattering (foreign tiles leave early)
    p.m_rot = (p.fused == 1 ? p.rank : (p.rank + 1) % p.world) * tiles_per_chunk;
    p.gemm_ctas = units * kCtaGroup;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(units * kCtaGroup + (p.fused == 1 ? copy_ctas : 0), 1, 1);
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmA2 ? *tmA2 : tmA, p);
  pb_count_launch(1);
  return (int)e;
}

}  // namespace pb

static int g_sm_reserve = 0;

extern "C" {

// Leaves `n` SMs out of the persistent GEMM grid (for communication kernels that must run beside it).
void pb_set_sm_reserve(int n) { g_sm_reserve = n < 0 ? 0 : n; }
int pb_get_sm_reserve() { return g_sm_reserve; }

// Rows of output tiles per band of the tile order of the plain and grouped GEMMs (0 restores the default).
void pb_set_gemm_group_m(int n) { pb::g_group_m = n < 0 ? 0 : n; }

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
  if (r) return -1000 - r;  // tensor map of A refused: -1000 - CUresult (or +1 when the encoder is missing)
  if (!b_mn) r = make_tmap_bf16_2d(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, (uint32_t)b_rows);
  else r = make_tmap_bf16_2d(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, 64);
  if (r) return -2000 - r;  // tensor map of B refused

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


// Grouped GEMMs of a mixture-of-experts layer: ONE launch covers all local experts, and the group sizes stay on the
// device (group_rows / group_start: int[n_groups] in device memory, group_start[g] a multiple of 256).
//   mode 1 (rows grouped):  C[r, :] = A[r, :] . B_g^T for the rows r of group g.  A: [M, K] K-major, M = the row
//       capacity of the buffers.  B: b_mn ? the groups' [K, N] matrices stacked to [n_groups * K, N]
//                                         : the groups' [N, K] matrices stacked to [n_groups * N, K].
//       C: [M, N] bf16.  Rows of a computed tile beyond its group's end are set to zero; tiles without rows of any
//       group are not computed and their part of C is left untouched.  b_mn needs K % 64 == 0.
//   mode 2 (contraction grouped):  C_g[M, N] (+)= sum over the rows r of group g of A[r, m] * B[r, n].
//       A: [rows, M], B: [rows, N] (both MN-major), C: n_groups stacked [M, N] blocks (fp32 accumulate or bf16).
//       Rows from a group's end to the next multiple of 64 take part: they must be zero in A or in B and finite in
//       the other (mode 1 outputs satisfy this).
int pb_gemm_grouped(int mode, const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                    long long ldb, long long ldc, int b_mn, int n_groups, const int* group_rows,
                    const int* group_start, int out_fp32, int accumulate, int* err_dev, void* stream_) {
  using namespace pb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (mode != 1 && mode != 2) return -1;
  if (M <= 0 || N <= 0 || K <= 0 || n_groups < 1 || n_groups > MAX_GROUPS) return -1;
  if ((lda % 8) || (ldb % 8) || (ldc % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (accumulate && !out_fp32) return -4;
  if (mode == 1 && (out_fp32 || (b_mn && K % 64 != 0))) return -6;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tmA, tmB;
  int r;
  if (mode == 1) {
    r = make_tmap_bf16_2d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 128);
    if (r) return -10;
    if (!b_mn) r = make_tmap_bf16_2d(&tmB, B, (uint64_t)K, (uint64_t)n_groups * N, (uint64_t)ldb, 64, 128);
    else r = make_tmap_bf16_2d(&tmB, B, (uint64_t)N, (uint64_t)n_groups * K, (uint64_t)ldb, 64, 64);
    if (r) return -11;
  } else {
    r = make_tmap_bf16_2d(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, 64);
    if (r) return -10;
    r = make_tmap_bf16_2d(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, 64);
    if (r) return -11;
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M;
  p.N = N;
  p.K = K;
  p.C = C;
  p.ldc = ldc;
  p.out_fp32 = out_fp32;
  p.accumulate = accumulate;
  p.a_mn = mode == 2;
  p.b_mn = mode == 2 ? 1 : b_mn;
  p.err = err_dev;
  p.grouped = mode;
  p.n_groups = n_groups;
  p.group_rows = group_rows;
  p.group_start = group_start;
  p.b_group_stride = b_mn ? K : N;
  p.c_group_stride = (long long)M * ldc;
  int sms = sm_count - g_sm_reserve;
  if (sms < 2) sms = 2;
  return launch_gemm<2, 256, 6>(tmA, tmB, p, sms, stream, nullptr, 0, mode == 2 ? n_groups : 1);
}


// Tensor-parallel fused GEMMs over peer memory (CTA-pair tiles, 256 x 256).
//   mode 1 (all-gather -> GEMM):  C[world*chunk_rows, N] = concat_r(shard_r)[.., K] . B^T.  `a_local` is this rank's
//       shard, `peer_src[r]` every rank's shard (peer mapped), `gathered` a local [world*chunk_rows, K] buffer.
//   mode 2 (GEMM -> reduce-scatter): partial = A[world*chunk_rows, K] . B^T; rank r ends up with
//       rs_out[chunk_rows, N] = sum over ranks of their partial rows [r*chunk_rows, (r+1)*chunk_rows) (+ residual).
//       `C` is local scratch [chunk_rows, N]; `rs_staging[r]` every rank's [world, chunk_rows, N] staging buffer.
// chunk_rows must be a multiple of 256; K, N multiples of 8; flags[r]: every rank's int[2*world] block;
// tile_flags: local int[world*chunk_rows/256]; counters: local int[16]. All flag memory starts at zero and `epoch`
// grows by one per call on every rank.
int pb_gemm_tp_fused(int mode, const void* a_local, const void* B, void* C, int N, int K, long long lda,
                     long long ldb, long long ldc, int b_mn, int rank, int world, int chunk_rows, int epoch,
                     void** peer_src, void* gathered, void** rs_staging, void* rs_out, const void* rs_residual,
                     int** flags, int* tile_flags, int* counters, int copy_ctas, int* err_dev, void* stream_) {
  using namespace pb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (mode != 1 && mode != 2) return -1;
  if (world < 2 || world > 8 || chunk_rows % 256 != 0) return -2;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8) || (K % 8)) return -3;
  if (mode == 1 && lda != K) return -4;  // shards are streamed as contiguous byte ranges
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const int M = world * chunk_rows;
  CUtensorMap tmA, tmA2, tmB;
  if (mode == 1) {
    if (make_tmap_bf16_2d(&tmA, a_local, (uint64_t)K, (uint64_t)chunk_rows, (uint64_t)lda, 64, 128)) return -10;
    if (make_tmap_bf16_2d(&tmA2, gathered, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 128)) return -10;
  } else {
    if (make_tmap_bf16_2d(&tmA, a_local, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 128)) return -10;
    tmA2 = tmA;
  }
  int r;
  if (!b_mn) r = make_tmap_bf16_2d(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 128);
  else r = make_tmap_bf16_2d(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, 64);
  if (r) return -11;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M;
  p.N = N;
  p.K = K;
  p.C = C;
  p.ldc = ldc;
  p.b_mn = b_mn;
  p.err = err_dev;
  p.fused = mode;
  p.rank = rank;
  p.world = world;
  p.chunk_rows = chunk_rows;
  p.lda_elems = lda;
  p.epoch = epoch;
  p.tile_flags = tile_flags;
  p.counters = counters;
  for (int i = 0; i < world; ++i) {
    p.flags[i] = flags[i];
    if (peer_src) p.peer_src[i] = reinterpret_cast<const __nv_bfloat16*>(peer_src[i]);
    if (rs_staging) p.rs_staging[i] = reinterpret_cast<__nv_bfloat16*>(rs_staging[i]);
  }
  p.gathered = reinterpret_cast<__nv_bfloat16*>(gathered);
  p.rs_out = reinterpret_cast<__nv_bfloat16*>(rs_out);
  p.rs_residual = reinterpret_cast<const __nv_bfloat16*>(rs_residual);
  cudaError_t e = cudaMemsetAsync(counters, 0, 16 * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  int sms = sm_count - g_sm_reserve;
  if (copy_ctas < 2) copy_ctas = 2;
  copy_ctas &= ~1;
  // every CTA of this grid waits on others of the same grid: it must be fully resident
  return launch_gemm<2, 256, 6>(tmA, tmB, p, sms, stream, &tmA2, mode == 1 ? copy_ctas : 0);
}

}  // extern "C"
