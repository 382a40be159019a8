// Dense block-scaled NVFP4 GEMM on CTA pairs (tcgen05 cta_group::2).  Included by gemm_nvfp4.cu
// (one translation unit, so both kernels share the sticky device status word).
//
// Two CTAs on neighbouring SMs own one 256 x 256 output tile: CTA r of the pair
// holds rows [128r, 128r+128) of the A tile and rows [128r, 128r+128) of the B
// tile (its half of the output columns' operand) in its own shared memory, and
// the leader (r = 0) issues 256 x 256 x 64 MMAs that read both halves.  Per
// k-block each SM then pulls 16 KB of A, 16 KB of B and 6 KB of scales from L2
// instead of 16 + 32 + 6, which is what bounds the single-CTA kernel.  No load
// is multicast: each CTA loads what it holds.
//
// Hand-over: both CTAs' TMA loads credit the leader's "full" barrier (the leader
// arms it for the bytes of both); the leader's tcgen05.commit releases the stage
// in both CTAs and publishes the accumulator to both epilogues; epilogue warps of
// both CTAs arrive on the leader's "accumulator free" barrier.  Every wait is
// bounded; the kernel ends with a hardware cluster barrier so neither CTA exits
// while its peer may still touch its shared memory or barriers.
#pragma once

#include "gemm_common.cuh"

#include <cstdlib>
#include <type_traits>

namespace hb200 {
namespace pair {

using namespace sm100;

constexpr int kThreads2 = 640;  // producer, MMA issuer, scale copier, one idle warp, sixteen epilogue warps
constexpr int kTileN = 256;
constexpr int kStages2 = 5;
constexpr int kABytes2 = kBlockM * kBlockKBytes;          // 16 KB: this CTA's 128 rows of A
constexpr int kBBytes2 = 128 * kBlockKBytes;              // 16 KB: this CTA's half of B
constexpr int kSfaBytes2 = kAtomsPerStage * kAtomBytes;   // 2 KB
constexpr int kSfbBytes2 = 2 * kAtomsPerStage * kAtomBytes;  // 4 KB: scales of all 256 B rows
constexpr int kBOff2 = kABytes2;
constexpr int kSfaOff2 = kBOff2 + kBBytes2;
constexpr int kSfbOff2 = kSfaOff2 + kSfaBytes2;
constexpr int kStageBytes2 = kSfbOff2 + kSfbBytes2;       // 38912, a multiple of 1024
constexpr int kOutStageBytes = 16 * 2048;                 // one 32-row x 64-byte box per epilogue warp
constexpr int kSfCols2 = kAtomsPerStage * 4 * 3;          // 48 scale columns per stage
constexpr int kSfBase2 = kTileN;                          // after the 256 accumulator columns
static_assert(kStageBytes2 % 1024 == 0, "stage must keep 1024-byte alignment");
static_assert(kSfBase2 + kStages2 * kSfCols2 <= 512, "tensor memory budget exceeded");

// named barrier of the four epilogue warps (128 threads) that share lane quarter q; barrier 0 is __syncthreads'
__device__ __forceinline__ void quarter_bar(int q) { asm volatile("bar.sync %0, 128;" : : "r"(q + 1) : "memory"); }
// the same barrier with a vote: true when `mine` holds in all 128 threads (a warp that gave up a bounded wait
// takes the other three out of the loop with it instead of leaving them at the barrier)
__device__ __forceinline__ bool quarter_bar_all(int q, bool mine) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, o;\n\tsetp.ne.u32 p, %2, 0;\n\tbar.red.and.pred o, %1, 128, p;\n\tselp.u32 %0, 1, 0, o;\n\t}"
      : "=r"(r)
      : "r"(q + 1), "r"(uint32_t(mine))
      : "memory");
  return r != 0;
}

struct PairArgs {
  void* out;
  int64_t ldc;
  int m, n, k;
  float alpha;
  int m_tiles, n_tiles;  // 256 x 256 tiles
  // Tensor-parallel form: every tile row (512 contiguous bytes) is written to the same place of every rank's
  // buffer with bulk copies from shared memory; stores only, nothing is ever loaded from peer memory.
  int n_dst;
  void* dst[8];  // the [m, ldc] buffers, peers in ring order from the next rank, this rank's own last; the tile columns start at column col0
  int col0;
  // Grouped form (tile_info != nullptr): the rows of A are laid out group after group, every group padded to a
  // multiple of 256 rows; tile_info[t] = (group, valid rows) of 128-row tile t, so entries 2j and 2j+1 describe
  // 256-row tile j.  B is [groups * n, K/2] with the groups' scale tiles back to back.
  const int2* tile_info;
  const float* row_scale;    // optional fp32 factor per row of A
  const float* group_alpha;  // optional fp32 factor per group
  // SiLU-mul epilogue (grouped bf16 only): the 256 columns of a tile are 128 gate columns followed by the 128 up
  // columns of the same outputs; the kernel writes y = bf16(silu(gate) * up) [rows, n / 2] with leading dimension
  // ldc and folds every row's max |y| into row_amax (fp32 bits, compared as integers).
  float* row_amax;
};

constexpr int kBand = 32;  // row tiles per band of the dense tile order (8192 rows: 16384 x 8192 x 8192 went from 450 to 385 us)

struct PairTile {
  int m_blk, n_blk, group;
  bool valid;
};

__device__ __forceinline__ PairTile decode_pair_tile(const PairArgs& g, int tile) {
  PairTile t;
  if (g.tile_info != nullptr) {
    // all column tiles of a 256-row tile run back to back: its group's weights stay in L2
    t.m_blk = tile / g.n_tiles;
    t.n_blk = tile - t.m_blk * g.n_tiles;
    const int2 ti = g.tile_info[2 * t.m_blk];
    t.group = ti.x;
    t.valid = ti.x >= 0 && ti.y > 0;
  } else {
    // bands of kBand row tiles; inside a band the row tile runs fastest, then the column tile: the 74 pairs that work
    // at the same time share a few row tiles of A and a few column tiles of B, which stay in L2
    const int per_band = kBand * g.n_tiles;
    const int b = tile / per_band, r = tile - b * per_band;
    const int rows_here = min(kBand, g.m_tiles - b * kBand);
    t.n_blk = r / rows_here;
    t.m_blk = b * kBand + (r - t.n_blk * rows_here);
    t.group = 0;
    t.valid = true;
  }
  return t;
}

// TP: the tensor-parallel form (every tile also goes to the peers).  It trades one stage of the operand ring
// for output staging boxes twice as wide, so that a store over NVLink writes 128 contiguous bytes per row.
template <typename OutT, bool TP, bool SILU = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                       const __grid_constant__ CUtensorMap tmap_out, const PairArgs g) {
  constexpr int kS = TP ? kStages2 - 1 : kStages2;
  // staging: one 32-row x 64-byte box per epilogue warp, or (TP) one 32-row x 512-byte box per lane quarter
  // whose rows are padded to 528 bytes so that the 32 lanes of a warp spread over all banks
  constexpr int kBoxBytes = 2048;
  constexpr int kRowPitchTp = 528;
  constexpr int kOutBytes = TP ? 4 * 32 * kRowPitchTp : 16 * kBoxBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_out = smem + kS * kStageBytes2;  // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + ((kOutBytes + 127) / 128) * 128);
  uint64_t* full_bar = bars;                 // used in the leader only
  uint64_t* empty_bar = bars + kS;     // one set per CTA
  uint64_t* sf_full_bar = bars + 2 * kS;   // scales of a stage are in tensor memory (leader only)
  uint64_t* tmem_full_bar = bars + 3 * kS;
  uint64_t* tmem_empty_bar = tmem_full_bar + 1;  // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int col_tiles = (g.k / 16 + 3) / 4;
  const int num_kb = (col_tiles + kAtomsPerStage - 1) / kAtomsPerStage;
  const int num_tiles = g.m_tiles * g.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kS; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);   // the leader's producer arms it; bytes come from both CTAs
      mbar_init(smem_u32(&empty_bar[s]), 1);  // the leader's commit, multicast to both CTAs
      mbar_init(smem_u32(&sf_full_bar[s]), 1);
    }
    mbar_init(smem_u32(tmem_full_bar), 1);
    mbar_init(smem_u32(tmem_empty_bar), 32);  // sixteen epilogue warps in each CTA
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before anything remote happens
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    uint32_t it = 0;
    bool ok = true;
    const uint32_t stage_bytes = kABytes2 + kBBytes2 + kSfaBytes2 + kSfbBytes2;
    const int n_row_tiles = (g.n + 127) / 128;  // 128-row scale tiles of one group of B
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const PairTile t = decode_pair_tile(g, tile);
      if (!t.valid) continue;
      const int m_blk = t.m_blk, n_blk = t.n_blk;
      const int a_row = m_blk * 256 + int(rank) * 128;
      const int b_row = t.group * g.n + n_blk * kTileN + int(rank) * 128;
      const int sfb_tile = t.group * n_row_tiles + n_blk * 2;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kS;
        const uint32_t ph = (it / kS) & 1;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag)) { ok = false; break; }
        uint8_t* st = smem + s * kStageBytes2;
        const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);  // always the leader's barrier
        if (elect_one()) {
          if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[s]), 2 * stage_bytes);
          tma_load_2d_pair(smem_u32(st), &tmap_a, kb * kBlockKBytes, a_row, bar);
          tma_load_2d_pair(smem_u32(st + kBOff2), &tmap_b, kb * kBlockKBytes, b_row, bar);
          // scale atoms: row = atom index = row_tile * col_tiles + column tile
          tma_load_2d_pair(smem_u32(st + kSfaOff2), &tmap_sfa, 0, (a_row / 128) * col_tiles + kb * kAtomsPerStage, bar);
          tma_load_2d_pair(smem_u32(st + kSfbOff2), &tmap_sfb, 0, sfb_tile * col_tiles + kb * kAtomsPerStage, bar);
          tma_load_2d_pair(smem_u32(st + kSfbOff2 + kSfaBytes2), &tmap_sfb, 0,
                           (sfb_tile + 1) * col_tiles + kb * kAtomsPerStage, bar);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (leader only)
    if (leader) {
      constexpr uint32_t idesc = make_idesc_mxf4nvf4(256, kTileN);
      bool ok = true;
      uint32_t it = 0, tc = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!decode_pair_tile(g, tile).valid) continue;
        const uint32_t tcur = tc++;
        if (!mbar_wait(smem_u32(tmem_empty_bar), (tcur & 1) ^ 1, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kS;
          const uint32_t ph = (it / kS) & 1;
          if (!mbar_wait(smem_u32(&sf_full_bar[s]), ph, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
          uint8_t* st = smem + s * kStageBytes2;
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + kBOff2);
          const uint32_t sf_col = tmem_base + kSfBase2 + s * kSfCols2;
          if (elect_one()) {
            for (int a = 0; a < atoms; ++a) {
              const uint64_t adesc = make_smem_desc(a_addr + a * 32, 16, 1024, kSwizzle128B);
              const uint64_t bdesc = make_smem_desc(b_addr + a * 32, 16, 1024, kSwizzle128B);
              mma_mxf4nvf4_pair(tmem_base, adesc, bdesc, idesc, (kb | a) != 0 ? 1u : 0u, sf_col + a * 4,
                                sf_col + 16 + a * 8);
            }
            tcgen05_commit_pair(smem_u32(&empty_bar[s]), 3);  // stage free in both CTAs
          }
          __syncwarp();
        }
        if (ok && elect_one()) tcgen05_commit_pair(smem_u32(tmem_full_bar), 3);
        __syncwarp();
      }
    }
  } else if (warp == 2) {
    // ---------------------------------------------------------- scale copier (leader only)
    // A separate issue stream: the copies of stage s+1 run beside the MMAs of stage s instead of
    // queueing in front of them.  Every stage has its own scale columns in tensor memory.
    if (leader) {
      bool ok = true;
      uint32_t it = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!decode_pair_tile(g, tile).valid) continue;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kS;
          const uint32_t ph = (it / kS) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
          uint8_t* st = smem + s * kStageBytes2;
          const uint32_t sfa_addr = smem_u32(st + kSfaOff2), sfb_addr = smem_u32(st + kSfbOff2);
          const uint32_t sf_col = tmem_base + kSfBase2 + s * kSfCols2;
          if (elect_one()) {
            for (int a = 0; a < atoms; ++a) {
              tcgen05_cp_32x128b_warpx4_pair(sf_col + a * 4, make_smem_desc(sfa_addr + a * kAtomBytes, 0, 128, kSwizzleNone));
              tcgen05_cp_32x128b_warpx4_pair(sf_col + 16 + a * 8,
                                             make_smem_desc(sfb_addr + a * kAtomBytes, 0, 128, kSwizzleNone));
              tcgen05_cp_32x128b_warpx4_pair(sf_col + 16 + a * 8 + 4,
                                             make_smem_desc(sfb_addr + kSfaBytes2 + a * kAtomBytes, 0, 128, kSwizzleNone));
            }
            tcgen05_commit_pair_local(smem_u32(&sf_full_bar[s]));
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 3) {
    // idle: keeps the epilogue warps' lane-quarter mapping (warp % 4) aligned
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    // Sixteen warps: warp w reads lane quarter w % 4 (the only one it may) and the 64 columns
    // [(w - 4) / 4 * 64, +64).  Each warp pulls its whole share into registers with two loads and hands the
    // accumulator back at once; conversion and the TMA stores happen off the MMA's critical path.
    const int quarter = warp & 3, cgroup = (warp - 4) >> 2;
    OutT* out = static_cast<OutT*>(g.out);
    const bool vec_ok = (g.ldc * sizeof(OutT)) % 16 == 0 && (reinterpret_cast<uintptr_t>(g.out) % 16) == 0;
    const uint32_t free_bar = map_to_cta(smem_u32(tmem_empty_bar), 0);
    uint8_t* box = stage_out + (warp - 4) * kBoxBytes;
    uint32_t tc = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const PairTile t = decode_pair_tile(g, tile);
      if (!t.valid) continue;
      const int m_blk = t.m_blk, n_blk = t.n_blk;
      const uint32_t tcur = tc++;
      const bool have = mbar_wait(smem_u32(tmem_full_bar), tcur & 1, abort_flag);
      if constexpr (!TP) {
        if (!have) { ok = false; break; }
      }
      tcgen05_fence_after();
      const int row0 = m_blk * 256 + int(rank) * 128 + quarter * 32;
      const int row = row0 + lane;
      float alpha = g.alpha;
      if (g.group_alpha != nullptr) alpha *= g.group_alpha[t.group];
      if (g.row_scale != nullptr && row < g.m) alpha *= g.row_scale[row];
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + cgroup * 64;
      uint32_t r[2][32];
      if constexpr (SILU) {
        // 32 gate columns and the 32 up columns of the same outputs
        const uint32_t tbase = tmem_base + (uint32_t(quarter * 32) << 16);
        tmem_ld_32x32b_x32(tbase + cgroup * 32, r[0]);
        tmem_ld_32x32b_x32(tbase + 128 + cgroup * 32, r[1]);
      } else {
        tmem_ld_32x32b_x32(taddr, r[0]);
        tmem_ld_32x32b_x32(taddr + 32, r[1]);
      }
      tmem_ld_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(free_bar);
      const int col = n_blk * kTileN + cgroup * 64;
      if constexpr (SILU) {
        const int valid_rows = g.tile_info[2 * m_blk + int(rank)].y;  // of this CTA's 128 rows
        if (quarter * 32 + lane < valid_rows) {
          uint32_t packed[16];
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float y[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // gate and up rounded to bf16 first, as a bf16 activation pipeline holds them
              const float gv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[0][2 * j + h]) * alpha));
              const float uv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[1][2 * j + h]) * alpha));
              y[h] = __fmul_rn(__fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv))), uv);
            }
            const __nv_bfloat162 pk = __floats2bfloat162_rn(y[0], y[1]);
            packed[j] = *reinterpret_cast<const uint32_t*>(&pk);
            amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(packed[j] << 16)), fabsf(__uint_as_float(packed[j] & 0xffff0000u))));
          }
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(g.out) + int64_t(row) * g.ldc + n_blk * 128 + cgroup * 32;
          if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {  // 32 bytes per store: whole sectors
            const uint32_t lo[8] = {packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6], packed[7]};
            const uint32_t hi[8] = {packed[8], packed[9], packed[10], packed[11], packed[12], packed[13], packed[14], packed[15]};
            stg_v8(dst, lo);
            stg_v8(dst + 16, hi);
          } else {
#pragma unroll
            for (int v = 0; v < 4; ++v)
              *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
          }
          atomicMax(reinterpret_cast<int*>(g.row_amax + row), __float_as_int(amax));
        }
      } else if constexpr (sizeof(OutT) == 2 && TP) {
        // The four warps of a lane quarter fill one box of 32 rows x 256 columns; its first warp then sends every
        // row, 512 contiguous bytes, to this rank and to every peer with one bulk copy per destination.
        uint8_t* qbox = stage_out + quarter * (32 * kRowPitchTp);
        if (cgroup == 0) bulk_wait_group_read0();  // each lane waits for the copies it issued for the last tile
        if (!quarter_bar_all(quarter, have)) { ok = false; break; }  // the box is free (or a wait ran out)
        uint8_t* rowp = qbox + lane * kRowPitchTp + cgroup * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lo = __uint_as_float(r[h][v * 8 + 2 * j]) * alpha;
              const float hi = __uint_as_float(r[h][v * 8 + 2 * j + 1]) * alpha;
              if constexpr (std::is_same<OutT, __half>::value) {
                p[j] = h2_as_u32(__floats2half2_rn(lo, hi));
              } else {
                const __nv_bfloat162 hh = __floats2bfloat162_rn(lo, hi);
                p[j] = *reinterpret_cast<const uint32_t*>(&hh);
              }
            }
            *reinterpret_cast<uint4*>(rowp + (h * 4 + v) * 16) = make_uint4(p[0], p[1], p[2], p[3]);
          }
        }
        fence_proxy_async_smem();
        quarter_bar(quarter);  // the box is complete
        if (cgroup == 0) {
          const int tile_col = n_blk * kTileN;
          if (row < g.m && tile_col < g.n) {
            const uint32_t bytes = uint32_t(min(kTileN, g.n - tile_col)) * 2u;
            const int64_t off = int64_t(row) * g.ldc + g.col0 + tile_col;
            for (int d = 0; d < g.n_dst; ++d)
              bulk_store(static_cast<OutT*>(g.dst[d]) + off, smem_u32(qbox + lane * kRowPitchTp), bytes);
          }
          bulk_commit_group();
        }
      } else if constexpr (sizeof(OutT) == 2) {
        // two boxes of 32 columns (64 bytes per row, 64-byte swizzle) through this warp's staging buffer
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (lane == 0) bulk_wait_group_read0();
          __syncwarp();
          uint8_t* rowp = box + lane * 64;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lo = __uint_as_float(r[h][v * 8 + 2 * j]) * alpha;
              const float hi = __uint_as_float(r[h][v * 8 + 2 * j + 1]) * alpha;
              if constexpr (std::is_same<OutT, __half>::value) {
                p[j] = h2_as_u32(__floats2half2_rn(lo, hi));
              } else {
                const __nv_bfloat162 hh = __floats2bfloat162_rn(lo, hi);
                p[j] = *reinterpret_cast<const uint32_t*>(&hh);
              }
            }
            // 64-byte swizzle: 16-byte chunk index xor bits 1..2 of the row
            *reinterpret_cast<uint4*>(rowp + ((v ^ ((lane >> 1) & 3)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_out, col + h * 32, row0, smem_u32(box));
            bulk_commit_group();
          }
        }
      } else {
        if (row < g.m && col < g.n)
          store_row_chunk<OutT>(out + int64_t(row) * g.ldc + col, r[0], alpha, g.n - col, vec_ok);
        if (row < g.m && col + 32 < g.n)
          store_row_chunk<OutT>(out + int64_t(row) * g.ldc + col + 32, r[1], alpha, g.n - col - 32, vec_ok);
      }
    }
    // peers read the result right after the barrier kernel that follows: wait for the writes themselves
    if constexpr (TP) {
      if (cgroup == 0) bulk_wait_group0();
    } else {
      if (lane == 0) bulk_wait_group_read0();
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer is done with this CTA's shared memory, barriers and tensor memory
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicMin(&g_device_status, HB200_ERR_DEVICE_TIMEOUT);
}

// Dense GEMM on CTA pairs; returns HB200_ERR_UNSUPPORTED for shapes it does not take
// (the caller then uses the single-CTA kernel).
struct PeerOut {
  int64_t n_total = 0;  // columns of the gathered output (0: not tensor parallel)
  int64_t col0 = 0;
  int n_peers = 0;
  void* ptr[7] = {};
};

inline int launch_gemm_pair(const void* a, const void* b, const void* sfa, const void* sfb, void* out, int64_t m, int64_t n,
                     int64_t k, int64_t ldc, float alpha, int out_dtype, cudaStream_t stream,
                     const PeerOut& peers = PeerOut()) {
  if (m < 256 || n < 256 || (k % 32) != 0) return HB200_ERR_UNSUPPORTED;
  const bool tp = peers.n_total > 0;
  if (tp && (out_dtype == 2 || (n % 8) != 0 || (peers.col0 % 8) != 0)) return HB200_ERR_UNSUPPORTED;
  CUtensorMap ta, tb, tsa, tsb;
  const int64_t col_tiles = (k / 16 + 3) / 4;
  if (!make_operand_map(&ta, a, m, k / 2, 128) || !make_operand_map(&tb, b, n, k / 2, 128)) return HB200_ERR_CUDA;
  if (!make_scale_map(&tsa, sfa, ceil_div64(m, 128) * col_tiles) ||
      !make_scale_map(&tsb, sfb, ceil_div64(n, 128) * col_tiles))
    return HB200_ERR_CUDA;
  CUtensorMap tout;
  if (out_dtype != 2) {
    if ((ldc % 8) != 0 || reinterpret_cast<uintptr_t>(out) % 16) return HB200_ERR_UNSUPPORTED;
    if (tp) {
      tout = ta;  // the tensor-parallel epilogue writes rows with bulk copies, not through a map
    } else if (!make_output_map16(&tout, out, m, n, ldc, out_dtype == 0)) {
      return HB200_ERR_CUDA;
    }
  } else {
    tout = ta;  // unused by the fp32 epilogue
  }
  PairArgs g{out, ldc, int(m), int(n), int(k), alpha, int(ceil_div64(m, 256)), int(ceil_div64(n, 256)), 0, {}, 0,
             nullptr, nullptr, nullptr, nullptr};
  if (tp) {
    g.col0 = int(peers.col0);
    // the copies over NVLink are issued first, the local one last
    for (int i = 0; i < peers.n_peers; ++i) g.dst[g.n_dst++] = peers.ptr[i];
    g.dst[g.n_dst++] = out;
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = g.m_tiles * g.n_tiles;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  constexpr size_t smem = size_t(kStages2) * kStageBytes2 + kOutStageBytes + (3 * kStages2 + 2) * 8 + 16 + 1024;
  constexpr size_t smem_tp = size_t(kStages2 - 1) * kStageBytes2 + 4 * 32 * 528 + 128 + (3 * kStages2 + 2) * 8 + 16 + 1024;
  static_assert(smem <= 232448 && smem_tp <= 232448, "shared memory budget exceeded");
#define HB200_PAIR(T, TPV, SMEM)                                                                              \
  do {                                                                                                        \
    auto kernel = nvfp4_gemm_pair_kernel<T, TPV>;                                                             \
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM)) != cudaSuccess)  \
      return HB200_ERR_CUDA;                                                                                  \
    kernel<<<2 * pairs, kThreads2, SMEM, stream>>>(ta, tb, tsa, tsb, tout, g);                            \
  } while (0)
  if (tp) {
    if (out_dtype == 0) HB200_PAIR(__nv_bfloat16, true, smem_tp);
    else HB200_PAIR(__half, true, smem_tp);
  } else {
    if (out_dtype == 0) HB200_PAIR(__nv_bfloat16, false, smem);
    else if (out_dtype == 1) HB200_PAIR(__half, false, smem);
    else HB200_PAIR(float, false, smem);
  }
#undef HB200_PAIR
  return launch_status();
}

// Grouped GEMM on CTA pairs: rows of A group after group, every group padded to a multiple of 256 rows
// (max_m_tiles counts 128-row tiles and is even); bf16 or fp16 out.  HB200_ERR_UNSUPPORTED for shapes it
// does not take.
inline int launch_grouped_pair(const void* a, const void* b, const void* sfa, const void* sfb, void* out,
                               const int32_t* tile_info, int64_t max_m_tiles, int64_t n, int64_t k, int64_t groups,
                               int64_t ldc, const float* row_scale, const float* group_alpha, float alpha,
                               int out_dtype, cudaStream_t stream, float* row_amax = nullptr) {
  if ((max_m_tiles % 2) != 0 || (n % 256) != 0 || (k % 32) != 0 || out_dtype == 2 || (ldc % 8) != 0 ||
      reinterpret_cast<uintptr_t>(out) % 16 || (row_amax != nullptr && out_dtype != 0))
    return HB200_ERR_UNSUPPORTED;
  const int64_t m = max_m_tiles * 128;
  CUtensorMap ta, tb, tsa, tsb, tout;
  const int64_t col_tiles = (k / 16 + 3) / 4;
  if (!make_operand_map(&ta, a, m, k / 2, 128) || !make_operand_map(&tb, b, n * groups, k / 2, 128)) return HB200_ERR_CUDA;
  if (!make_scale_map(&tsa, sfa, max_m_tiles * col_tiles) || !make_scale_map(&tsb, sfb, (n / 128) * groups * col_tiles))
    return HB200_ERR_CUDA;
  if (row_amax != nullptr) {
    tout = ta;  // the SiLU-mul epilogue stores rows directly
  } else if (!make_output_map16(&tout, out, m, n, ldc, out_dtype == 0)) {
    return HB200_ERR_CUDA;
  }
  PairArgs g{out, ldc, int(m), int(n), int(k), alpha, int(max_m_tiles / 2), int(n / 256), 0, {}, 0,
             reinterpret_cast<const int2*>(tile_info), row_scale, group_alpha, row_amax};
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = g.m_tiles * g.n_tiles;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  if (pairs == 0) return HB200_OK;
  constexpr size_t smem = size_t(kStages2) * kStageBytes2 + kOutStageBytes + (3 * kStages2 + 2) * 8 + 16 + 1024;
  if (row_amax != nullptr) {
    auto kernel = nvfp4_gemm_pair_kernel<__nv_bfloat16, false, true>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
    kernel<<<2 * pairs, kThreads2, smem, stream>>>(ta, tb, tsa, tsb, tout, g);
  } else if (out_dtype == 0) {
    auto kernel = nvfp4_gemm_pair_kernel<__nv_bfloat16, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
    kernel<<<2 * pairs, kThreads2, smem, stream>>>(ta, tb, tsa, tsb, tout, g);
  } else {
    auto kernel = nvfp4_gemm_pair_kernel<__half, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
    kernel<<<2 * pairs, kThreads2, smem, stream>>>(ta, tb, tsa, tsb, tout, g);
  }
  return launch_status();
}

}  // namespace pair
}  // namespace hb200
