// Block-scaled NVFP4 GEMM for sm_100a:  D[M,N] = alpha * (A[M,K] . B[N,K]^T)
// with both operands packed e2m1 (K-major) and one e4m3 scale per 16 K-elements
// in the SWIZZLE_32_4_4 layout.
//
// One persistent CTA per SM, warps with fixed roles:
//   warp 0   producer : TMA loads of the A and B tiles (128-byte swizzled rows of
//                       256 K-elements) and plain bulk copies of the scale tiles
//                       (the swizzled global layout is already the 128x4 atom the
//                       tensor core wants, 512 contiguous bytes per 64 K-elements)
//   warp 1   MMA      : tcgen05.mma.kind::mxf4nvf4.block_scale accumulates
//                       128 x BLOCK_N x 64 per instruction into tensor memory
//   warp 2   copier   : tcgen05.cp moves the scale atoms of a stage to that stage's own
//                       tensor-memory columns, as a separate issue stream so the copies
//                       run beside the MMAs of earlier stages
//   warps 4-7 epilogue: tcgen05.ld of the fp32 accumulator, * alpha, convert, store
// Stages of the shared-memory ring and of the accumulator ring are handed over
// with mbarriers; every wait is bounded and a timeout ends the kernel with an
// error status instead of hanging.  No cluster multicast is used anywhere.
#include "common.cuh"
#include "tcgen05.cuh"
#include "gemm_common.cuh"

#include <cstdlib>
#include <mutex>
#include <type_traits>

namespace hb200 {

__device__ int g_device_status = 0;

}  // namespace hb200

#include "gemm_nvfp4_2cta.cuh"

namespace hb200 {

namespace {

using namespace sm100;

constexpr int kGemmThreads = 640;  // producer, MMA issuer, scale copier, idle, sixteen epilogue warps
constexpr int kTmemCols = 512;

struct GemmArgs {
  const uint8_t* sfa;  // swizzled scales of A, logical [M, K/16]
  const uint8_t* sfb;  // swizzled scales of B, logical [N, K/16] (per group when grouped)
  void* out;           // [M, N] row-major, leading dimension ldc elements
  int64_t ldc;
  int m, n, k;         // m counts the (padded) rows of A and of the output
  float alpha;
  int m_tiles, n_tiles;
  // Grouped mode (tile_info != nullptr): the rows of A are laid out group after
  // group, every group padded to a multiple of 128 rows; tile_info[t] = (group,
  // valid rows) of 128-row tile t, group < 0 for tiles past the last group.  B is
  // [groups * n, K/2] with one scale buffer of sfb_group_stride bytes per group.
  const int2* tile_info;
  int64_t sfb_group_stride;
  const float* row_scale;    // optional fp32 factor per row of A
  const float* group_alpha;  // optional fp32 factor per group
  // SiLU-mul epilogue (grouped bf16 only, BLOCK_N = 256): the 256 columns of a tile are 128 gate columns
  // followed by the 128 up columns of the same outputs; the kernel writes y = bf16(silu(gate) * up)
  // [rows, n / 2] and folds every row's max |y| into row_amax (fp32 bits, compared as integers).
  float* row_amax;
};

struct Tile {
  int m_blk, n_blk, group, rows;
  bool valid;
};

__device__ __forceinline__ Tile decode_tile(const GemmArgs& g, int tile) {
  Tile t;
  if (g.tile_info != nullptr) {
    // all column tiles of a 128-row tile run back to back: its group's weights stay in L2
    t.m_blk = tile / g.n_tiles;
    t.n_blk = tile - t.m_blk * g.n_tiles;
    const int2 ti = g.tile_info[t.m_blk];
    t.group = ti.x;
    t.rows = ti.y;
    t.valid = ti.x >= 0 && ti.y > 0;
  } else {
    t.m_blk = tile % g.m_tiles;
    t.n_blk = tile / g.m_tiles;
    t.group = 0;
    t.rows = min(kBlockM, g.m - t.m_blk * kBlockM);
    t.valid = true;
  }
  return t;
}

template <int BLOCK_N>
struct StageLayout {
  static constexpr int kNB = (BLOCK_N + 127) / 128;  // 128-row scale atoms along N
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = BLOCK_N * kBlockKBytes;
  static constexpr int kSfaBytes = kAtomsPerStage * kAtomBytes;
  static constexpr int kSfbBytes = kNB * kAtomsPerStage * kAtomBytes;
  static constexpr int kBOff = kABytes;
  static constexpr int kSfaOff = kBOff + ((kBBytes + 1023) / 1024) * 1024;
  static constexpr int kSfbOff = kSfaOff + kSfaBytes;
  static constexpr int kBytes = ((kSfbOff + kSfbBytes + 1023) / 1024) * 1024;
  // tensor memory: accumulator ring, then one set of scale columns per shared-memory stage
  static constexpr int kSfCols = kAtomsPerStage * 4 * (1 + kNB);
  static constexpr int kSfaColOff = 0;                       // inside a stage's scale columns
  static constexpr int kSfbColOff = kAtomsPerStage * 4;
  template <int STAGES>
  static constexpr int acc_stages() { return (2 * BLOCK_N + STAGES * kSfCols <= kTmemCols) ? 2 : 1; }
};

template <int BLOCK_N, int STAGES, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const GemmArgs g) {
  using L = StageLayout<BLOCK_N>;
  constexpr int ACC = L::template acc_stages<STAGES>();
  constexpr int kSfBase = ACC * BLOCK_N;
  static_assert(kSfBase + STAGES * L::kSfCols <= kTmemCols, "tensor memory budget exceeded");
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles need 1024-byte aligned bases
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * L::kBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* sf_full_bar = bars + 2 * STAGES;  // a stage's scales have reached tensor memory
  uint64_t* tmem_full_bar = bars + 3 * STAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col_tiles = (g.k / 16 + 3) / 4;                     // 64-element scale atoms along K
  const int num_kb = (col_tiles + kAtomsPerStage - 1) / kAtomsPerStage;
  const int num_tiles = g.m_tiles * g.n_tiles;
  const int n_row_tiles = (g.n + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&sf_full_bar[s]), 1);
    }
    for (int a = 0; a < ACC; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 16);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    // the whole warp walks the schedule; one elected lane issues the copies
    {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Tile t = decode_tile(g, tile);
        if (!t.valid) continue;
        const int m_blk = t.m_blk, n_blk = t.n_blk;
        const int b_row0 = t.group * g.n + n_blk * BLOCK_N;
        const uint8_t* sfb_base = g.sfb + int64_t(t.group) * g.sfb_group_stride;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag)) { ok = false; break; }
          const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
          int sfb_tiles = 0;
#pragma unroll
          for (int nb = 0; nb < L::kNB; ++nb)
            if ((n_blk * BLOCK_N) / 128 + nb < n_row_tiles) ++sfb_tiles;
          const uint32_t bytes = L::kABytes + L::kBBytes + uint32_t(atoms) * kAtomBytes * (1 + sfb_tiles);
          const uint32_t bar = smem_u32(&full_bar[s]);
          uint8_t* st = smem + s * L::kBytes;
          if (elect_one()) {
            mbar_arrive_expect_tx(bar, bytes);
            tma_load_2d(smem_u32(st), &tmap_a, kb * kBlockKBytes, m_blk * kBlockM, bar);
            tma_load_2d(smem_u32(st + L::kBOff), &tmap_b, kb * kBlockKBytes, b_row0, bar);
            bulk_load(smem_u32(st + L::kSfaOff),
                      g.sfa + (int64_t(m_blk) * col_tiles + kb * kAtomsPerStage) * kAtomBytes, atoms * kAtomBytes,
                      bar);
#pragma unroll
            for (int nb = 0; nb < L::kNB; ++nb) {
              const int rt = (n_blk * BLOCK_N) / 128 + nb;
              if (rt < n_row_tiles)
                bulk_load(smem_u32(st + L::kSfbOff + nb * kAtomsPerStage * kAtomBytes),
                          sfb_base + (int64_t(rt) * col_tiles + kb * kAtomsPerStage) * kAtomBytes, atoms * kAtomBytes,
                          bar);
            }
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // The whole warp walks the schedule and waits; one elected lane issues.
    {
      constexpr uint32_t idesc = make_idesc_mxf4nvf4(kBlockM, BLOCK_N);
      uint32_t it = 0, tc = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!decode_tile(g, tile).valid) continue;
        const int acc = tc % ACC;
        const uint32_t acc_ph = (tc / ACC) & 1;
        ++tc;
        if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_ph ^ 1, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&sf_full_bar[s]), ph, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
          uint8_t* st = smem + s * L::kBytes;
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + L::kBOff);
          const uint32_t sf_col = tmem_base + kSfBase + s * L::kSfCols;
          if (elect_one()) {
            for (int a = 0; a < atoms; ++a) {
              // 64 K-elements = 32 bytes further along the 128-byte swizzled row
              const uint64_t adesc = make_smem_desc(a_addr + a * 32, 16, 1024, kSwizzle128B);
              const uint64_t bdesc = make_smem_desc(b_addr + a * 32, 16, 1024, kSwizzle128B);
              mma_mxf4nvf4(tmem_d, adesc, bdesc, idesc, (kb | a) != 0 ? 1u : 0u, sf_col + L::kSfaColOff + a * 4,
                           sf_col + L::kSfbColOff + a * L::kNB * 4);
            }
            tcgen05_commit(smem_u32(&empty_bar[s]));  // stage reusable once these MMAs have read it
          }
          __syncwarp();
        }
        if (ok && elect_one()) tcgen05_commit(smem_u32(&tmem_full_bar[acc]));
        __syncwarp();
      }
    }
  } else if (warp == 2) {
    // -------------------------------------------------------- scale copier
    // Its own issue stream: the scale atoms of a stage go to that stage's tensor-memory columns while
    // the MMAs of earlier stages run, instead of queueing in front of them.
    {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!decode_tile(g, tile).valid) continue;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
          uint8_t* st = smem + s * L::kBytes;
          const uint32_t sfa_addr = smem_u32(st + L::kSfaOff), sfb_addr = smem_u32(st + L::kSfbOff);
          const uint32_t sf_col = tmem_base + kSfBase + s * L::kSfCols;
          if (elect_one()) {
            for (int a = 0; a < atoms; ++a) {
              tcgen05_cp_32x128b_warpx4(sf_col + L::kSfaColOff + a * 4,
                                        make_smem_desc(sfa_addr + a * kAtomBytes, 0, 128, kSwizzleNone));
#pragma unroll
              for (int nb = 0; nb < L::kNB; ++nb)
                tcgen05_cp_32x128b_warpx4(
                    sf_col + L::kSfbColOff + (a * L::kNB + nb) * 4,
                    make_smem_desc(sfb_addr + (nb * kAtomsPerStage + a) * kAtomBytes, 0, 128, kSwizzleNone));
            }
            tcgen05_commit(smem_u32(&sf_full_bar[s]));
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 3) {
    // idle: keeps the epilogue warps' lane-quarter mapping (warp % 4) aligned with warps 4..7
  } else {
    // ------------------------------------------------------------ epilogue
    // Sixteen warps: warp w reads lane quarter w % 4 (the only one it may) and a quarter of the tile's
    // columns.  A warp pulls its share of the accumulator into registers and hands the accumulator back
    // at once; scaling, conversion and the stores then run beside the next tile's MMAs.
    const int quarter = warp & 3, cgroup = (warp - 4) >> 2;
    constexpr int CW = BLOCK_N / 4;  // columns per warp
    OutT* out = static_cast<OutT*>(g.out);
    const bool vec_ok = (g.ldc * sizeof(OutT)) % 16 == 0 && (reinterpret_cast<uintptr_t>(g.out) % 16) == 0;
    uint32_t tc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const Tile t = decode_tile(g, tile);
      if (!t.valid) continue;
      const int m_blk = t.m_blk, n_blk = t.n_blk;
      const int acc = tc % ACC;
      const uint32_t acc_ph = (tc / ACC) & 1;
      ++tc;
      if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_ph, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const int row_in_tile = quarter * 32 + lane;
      const int row = m_blk * kBlockM + row_in_tile;
      const bool row_ok = row_in_tile < t.rows;
      float alpha = g.alpha;
      if (g.group_alpha != nullptr) alpha *= g.group_alpha[t.group];
      if (g.row_scale != nullptr && row_ok) alpha *= g.row_scale[row];
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BLOCK_N + cgroup * CW;
      if constexpr (CW >= 32) {
        uint32_t r[CW / 32][32];
        bool silu = false;
        if constexpr (BLOCK_N == 256 && std::is_same<OutT, __nv_bfloat16>::value) silu = g.row_amax != nullptr;
        if (silu) {
          // 32 gate columns and the 32 up columns of the same outputs
          const uint32_t tbase = taddr - cgroup * CW;
          tmem_ld_32x32b_x32(tbase + cgroup * 32, r[0]);
          tmem_ld_32x32b_x32(tbase + 128 + cgroup * 32, r[CW / 32 - 1]);
        } else {
#pragma unroll
          for (int c = 0; c < CW / 32; ++c) tmem_ld_32x32b_x32(taddr + c * 32, r[c]);
        }
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        if constexpr (BLOCK_N == 256 && std::is_same<OutT, __nv_bfloat16>::value) {
          if (silu) {
            if (row_ok) {
              uint32_t packed[16];
              float amax = 0.f;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float y[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  // gate and up rounded to bf16 first, as a bf16 activation pipeline holds them
                  const float gv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[0][2 * j + h]) * alpha));
                  const float uv =
                      __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[CW / 32 - 1][2 * j + h]) * alpha));
                  y[h] = __fmul_rn(__fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv))), uv);
                }
                const __nv_bfloat162 p = __floats2bfloat162_rn(y[0], y[1]);
                packed[j] = *reinterpret_cast<const uint32_t*>(&p);
                amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(packed[j] << 16)),
                                         fabsf(__uint_as_float(packed[j] & 0xffff0000u))));
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
                  *reinterpret_cast<uint4*>(dst + v * 8) =
                      make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
              }
              atomicMax(reinterpret_cast<int*>(g.row_amax + row), __float_as_int(amax));
            }
            continue;
          }
        }
#pragma unroll
        for (int c = 0; c < CW / 32; ++c) {
          const int col = n_blk * BLOCK_N + cgroup * CW + c * 32;
          if (row_ok && col < g.n)
            store_row_chunk<OutT>(out + int64_t(row) * g.ldc + col, r[c], alpha, g.n - col, vec_ok);
        }
      } else {
        uint32_t r8[8];
        if (cgroup * CW < BLOCK_N) tmem_ld_32x32b_x8(taddr, r8);
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        const int col = n_blk * BLOCK_N + cgroup * CW;
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < CW && col + j < g.n) {
              const float v = __uint_as_float(r8[j]) * alpha;
              if constexpr (sizeof(OutT) == 4) out[int64_t(row) * g.ldc + col + j] = v;
              else if constexpr (std::is_same<OutT, __half>::value) out[int64_t(row) * g.ldc + col + j] = __float2half_rn(v);
              else out[int64_t(row) * g.ldc + col + j] = __float2bfloat16_rn(v);
            }
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicMin(&g_device_status, HB200_ERR_DEVICE_TIMEOUT);
}

// ----------------------------------------------------------------- host side
int sm_count_gemm() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n > 0 ? n : 148;
}

template <int BLOCK_N, int STAGES, typename OutT>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs g, cudaStream_t stream) {
  using L = StageLayout<BLOCK_N>;
  constexpr size_t smem = size_t(STAGES) * L::kBytes + (3 * STAGES + 4) * 8 + 16 + 1024;
  static_assert(smem <= 232448, "shared memory budget exceeded");
  auto kernel = nvfp4_gemm_kernel<BLOCK_N, STAGES, OutT>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
    return HB200_ERR_CUDA;
  if (g.tile_info == nullptr) g.m_tiles = (g.m + kBlockM - 1) / kBlockM;  // grouped: set by the caller
  g.n_tiles = (g.n + BLOCK_N - 1) / BLOCK_N;
  const int tiles = g.m_tiles * g.n_tiles;
  const int grid = tiles < sm_count_gemm() ? tiles : sm_count_gemm();
  kernel<<<grid, kGemmThreads, smem, stream>>>(ta, tb, g);
  return launch_status();
}

template <typename OutT>
int dispatch_gemm(const void* a, const void* b, GemmArgs g, int groups, cudaStream_t stream) {
  CUtensorMap ta, tb;
  // (128-wide tiles with two accumulator stages were tried for the short-K second MoE GEMM: 435 against 393 us;
  // the extra operand traffic costs more than the overlapped epilogue brings)
  const int block_n = g.n > 128 ? 256 : 128;
  if (!make_operand_map(&ta, a, g.m, g.k / 2, kBlockM)) return HB200_ERR_CUDA;
  if (!make_operand_map(&tb, b, int64_t(g.n) * groups, g.k / 2, block_n)) return HB200_ERR_CUDA;
  if (block_n == 256) return launch_gemm<256, 4, OutT>(ta, tb, g, stream);
  return launch_gemm<128, 6, OutT>(ta, tb, g, stream);
}

}  // namespace
}  // namespace hb200

extern "C" int hb200_nvfp4_scaled_matmul(const void* a_packed, const void* b_packed, const void* scale_a,
                                         const void* scale_b, void* out, int64_t m, int64_t n, int64_t k,
                                         int64_t ldc, float alpha, int out_dtype, void* stream) {
  using namespace hb200;
  if (!a_packed || !b_packed || !scale_a || !scale_b || !out) return HB200_ERR_INVALID_ARGUMENT;
  if (m < 0 || n < 0 || k < 0 || ldc < n || out_dtype < 0 || out_dtype > 2) return HB200_ERR_INVALID_ARGUMENT;
  if ((k % 16) != 0) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a_packed) % 16 || reinterpret_cast<uintptr_t>(b_packed) % 16 ||
      reinterpret_cast<uintptr_t>(scale_a) % 16 || reinterpret_cast<uintptr_t>(scale_b) % 16)
    return HB200_ERR_INVALID_ARGUMENT;
  if (m == 0 || n == 0) return HB200_OK;
  if ((k % 32) != 0) return HB200_ERR_UNSUPPORTED;  // TMA needs 16-byte row pitch
  if (m > 0x7fffff00 || n > 0x7fffff00 || k > 0x7fffff00) return HB200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t elt = out_dtype == 2 ? 4 : 2;
  if (k == 0) {
    return cudaMemset2DAsync(out, size_t(ldc) * elt, 0, size_t(n) * elt, size_t(m), s) == cudaSuccess ? HB200_OK
                                                                                                      : HB200_ERR_CUDA;
  }
  {
    const int rc = pair::launch_gemm_pair(a_packed, b_packed, scale_a, scale_b, out, m, n, k, ldc, alpha, out_dtype, s);
    if (rc != HB200_ERR_UNSUPPORTED) return rc;
  }
  GemmArgs g{static_cast<const uint8_t*>(scale_a), static_cast<const uint8_t*>(scale_b), out, ldc,
             int(m), int(n), int(k), alpha, 0, 0, nullptr, 0, nullptr, nullptr, nullptr};
  switch (out_dtype) {
    case 0: return dispatch_gemm<__nv_bfloat16>(a_packed, b_packed, g, 1, s);
    case 1: return dispatch_gemm<__half>(a_packed, b_packed, g, 1, s);
    default: return dispatch_gemm<float>(a_packed, b_packed, g, 1, s);
  }
}

// Column-parallel form: this rank computes columns [col0, col0 + n) of the [m, n_total] result and writes them
// into the buffer of every rank (out_ptrs[0..world), peer-mapped pointers of one symmetric allocation; entry
// `rank` is this rank's own).  Every copy, local and remote, is a bulk copy of a 512-byte tile row out of a
// shared-memory staging box; nothing is loaded from peer memory.  Follow with hb200_peer_barrier before any rank reads its buffer.
extern "C" int hb200_nvfp4_scaled_matmul_tp(const void* a_packed, const void* b_packed, const void* scale_a,
                                            const void* scale_b, void* const* out_ptrs, int64_t world, int64_t rank,
                                            int64_t m, int64_t n, int64_t k, int64_t n_total, int64_t col0,
                                            float alpha, int out_dtype, void* stream) {
  using namespace hb200;
  if (!a_packed || !b_packed || !scale_a || !scale_b || !out_ptrs) return HB200_ERR_INVALID_ARGUMENT;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return HB200_ERR_INVALID_ARGUMENT;
  if (m < 0 || n < 0 || k < 0 || col0 < 0 || col0 + n > n_total || out_dtype < 0 || out_dtype > 1)
    return HB200_ERR_INVALID_ARGUMENT;
  if ((k % 16) != 0) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a_packed) % 16 || reinterpret_cast<uintptr_t>(b_packed) % 16 ||
      reinterpret_cast<uintptr_t>(scale_a) % 16 || reinterpret_cast<uintptr_t>(scale_b) % 16)
    return HB200_ERR_INVALID_ARGUMENT;
  pair::PeerOut peers;
  peers.n_total = n_total;
  peers.col0 = col0;
  for (int i = 0; i < world; ++i)
    if (!out_ptrs[i] || reinterpret_cast<uintptr_t>(out_ptrs[i]) % 16) return HB200_ERR_INVALID_ARGUMENT;
  // peers in ring order starting at the next rank: at any moment every rank then pushes to a different destination
  for (int i = 1; i < world; ++i) peers.ptr[peers.n_peers++] = out_ptrs[(rank + i) % world];
  if (m == 0 || n == 0) return HB200_OK;
  if (k == 0 || (k % 32) != 0 || (n_total % 8) != 0) return HB200_ERR_UNSUPPORTED;
  if (m > 0x7fffff00 || n_total > 0x7fffff00 || k > 0x7fffff00) return HB200_ERR_UNSUPPORTED;
  return pair::launch_gemm_pair(a_packed, b_packed, scale_a, scale_b, out_ptrs[rank], m, n, k, n_total, alpha,
                                out_dtype, static_cast<cudaStream_t>(stream), peers);
}

extern "C" int hb200_nvfp4_grouped_matmul(const void* a_packed, const void* b_packed, const void* scale_a,
                                          const void* scale_b, void* out, const int32_t* tile_info,
                                          int64_t max_m_tiles, int64_t n, int64_t k, int64_t groups, int64_t ldc,
                                          const float* row_scale, const float* group_alpha, float alpha,
                                          int out_dtype, void* stream) {
  using namespace hb200;
  if (!a_packed || !b_packed || !scale_a || !scale_b || !out || !tile_info) return HB200_ERR_INVALID_ARGUMENT;
  if (max_m_tiles < 0 || n < 0 || k <= 0 || groups <= 0 || ldc < n || out_dtype < 0 || out_dtype > 2)
    return HB200_ERR_INVALID_ARGUMENT;
  if ((k % 16) != 0) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a_packed) % 16 || reinterpret_cast<uintptr_t>(b_packed) % 16 ||
      reinterpret_cast<uintptr_t>(scale_a) % 16 || reinterpret_cast<uintptr_t>(scale_b) % 16 ||
      reinterpret_cast<uintptr_t>(tile_info) % 8)
    return HB200_ERR_INVALID_ARGUMENT;
  if (max_m_tiles == 0 || n == 0) return HB200_OK;
  if ((k % 32) != 0) return HB200_ERR_UNSUPPORTED;
  if (max_m_tiles * 128 > 0x7fffff00 || n * groups > 0x7fffff00 || k > 0x7fffff00) return HB200_ERR_UNSUPPORTED;
  const int64_t sfb_stride = round_up64(n, 128) * round_up64(k / 16, 4);
  GemmArgs g{static_cast<const uint8_t*>(scale_a), static_cast<const uint8_t*>(scale_b), out, ldc,
             int(max_m_tiles * 128), int(n), int(k), alpha, int(max_m_tiles), 0,
             reinterpret_cast<const int2*>(tile_info), sfb_stride, row_scale, group_alpha, nullptr};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (out_dtype) {
    case 0: return dispatch_gemm<__nv_bfloat16>(a_packed, b_packed, g, int(groups), s);
    case 1: return dispatch_gemm<__half>(a_packed, b_packed, g, int(groups), s);
    default: return dispatch_gemm<float>(a_packed, b_packed, g, int(groups), s);
  }
}

// hb200_nvfp4_grouped_matmul for a row layout whose groups are padded to multiples of 256 rows
// (hb200_moe_build_schedule_256): runs on CTA pairs with 256 x 256 tiles, which halves the weight-tile traffic
// per CTA; falls back to the 128-row kernel for shapes the pair kernel does not take (N % 256 != 0, fp32 out).
extern "C" int hb200_nvfp4_grouped_matmul_256(const void* a_packed, const void* b_packed, const void* scale_a,
                                              const void* scale_b, void* out, const int32_t* tile_info,
                                              int64_t max_m_tiles, int64_t n, int64_t k, int64_t groups, int64_t ldc,
                                              const float* row_scale, const float* group_alpha, float alpha,
                                              int out_dtype, void* stream) {
  using namespace hb200;
  if (!a_packed || !b_packed || !scale_a || !scale_b || !out || !tile_info) return HB200_ERR_INVALID_ARGUMENT;
  if (max_m_tiles < 0 || (max_m_tiles % 2) != 0 || n < 0 || k <= 0 || groups <= 0 || ldc < n || out_dtype < 0 ||
      out_dtype > 2 || (k % 16) != 0)
    return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a_packed) % 16 || reinterpret_cast<uintptr_t>(b_packed) % 16 ||
      reinterpret_cast<uintptr_t>(scale_a) % 16 || reinterpret_cast<uintptr_t>(scale_b) % 16 ||
      reinterpret_cast<uintptr_t>(tile_info) % 8)
    return HB200_ERR_INVALID_ARGUMENT;
  if (max_m_tiles == 0 || n == 0) return HB200_OK;
  if (max_m_tiles * 128 <= 0x7fffff00 && n * groups <= 0x7fffff00 && k <= 0x7fffff00) {
    const int rc = pair::launch_grouped_pair(a_packed, b_packed, scale_a, scale_b, out, tile_info, max_m_tiles, n, k,
                                             groups, ldc, row_scale, group_alpha, alpha, out_dtype,
                                             static_cast<cudaStream_t>(stream));
    if (rc != HB200_ERR_UNSUPPORTED) return rc;
  }
  return hb200_nvfp4_grouped_matmul(a_packed, b_packed, scale_a, scale_b, out, tile_info, max_m_tiles, n, k, groups,
                                    ldc, row_scale, group_alpha, alpha, out_dtype, stream);
}

// The first expert GEMM of an NVFP4 MoE layer with SiLU-mul in the epilogue.  The weight rows are gate/up
// interleaved in blocks of 128 (rows [256 j, 256 j + 128) = gate outputs [128 j, 128 j + 128), the next 128
// rows the up rows of the same outputs), n counts all of them; y = bf16(silu(gate) * up) is written to
// y_out [rows, n / 2] (leading dimension ldy) and row_amax[r] receives max |y[r, :]| (cleared here first,
// on the stream).  Same value, bit for bit, as hb200_nvfp4_grouped_matmul followed by the SiLU-mul of
// hb200_nvfp4_quantize_rows.  No counterpart in the reference (its MoE example is a bf16 top-1 GEMM,
// examples/moe_matmul_ogs.py:31-85); the gate-first convention is silu_and_mul_per_block_quant's.
extern "C" int hb200_nvfp4_grouped_matmul_silu(const void* a_packed, const void* b_packed, const void* scale_a,
                                               const void* scale_b, void* y_out, float* row_amax,
                                               const int32_t* tile_info, int64_t max_m_tiles, int64_t n, int64_t k,
                                               int64_t groups, int64_t ldy, const float* row_scale,
                                               const float* group_alpha, float alpha, void* stream) {
  using namespace hb200;
  if (!a_packed || !b_packed || !scale_a || !scale_b || !y_out || !row_amax || !tile_info)
    return HB200_ERR_INVALID_ARGUMENT;
  if (max_m_tiles < 0 || n <= 0 || k <= 0 || groups <= 0 || (n % 256) != 0 || ldy < n / 2 || (ldy % 8) != 0)
    return HB200_ERR_INVALID_ARGUMENT;
  if ((k % 16) != 0) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a_packed) % 16 || reinterpret_cast<uintptr_t>(b_packed) % 16 ||
      reinterpret_cast<uintptr_t>(scale_a) % 16 || reinterpret_cast<uintptr_t>(scale_b) % 16 ||
      reinterpret_cast<uintptr_t>(tile_info) % 8 || reinterpret_cast<uintptr_t>(y_out) % 16)
    return HB200_ERR_INVALID_ARGUMENT;
  if (max_m_tiles == 0) return HB200_OK;
  if ((k % 32) != 0) return HB200_ERR_UNSUPPORTED;
  if (max_m_tiles * 128 > 0x7fffff00 || n * groups > 0x7fffff00 || k > 0x7fffff00) return HB200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(row_amax, 0, size_t(max_m_tiles) * 128 * sizeof(float), s) != cudaSuccess) return HB200_ERR_CUDA;
  const int64_t sfb_stride = round_up64(n, 128) * round_up64(k / 16, 4);
  GemmArgs g{static_cast<const uint8_t*>(scale_a), static_cast<const uint8_t*>(scale_b), y_out, ldy,
             int(max_m_tiles * 128), int(n), int(k), alpha, int(max_m_tiles), 0,
             reinterpret_cast<const int2*>(tile_info), sfb_stride, row_scale, group_alpha, row_amax};
  return dispatch_gemm<__nv_bfloat16>(a_packed, b_packed, g, int(groups), s);
}

// hb200_nvfp4_grouped_matmul_silu for a row layout whose groups are padded to multiples of 256 rows
// (hb200_moe_build_schedule_256): 256 x 256 tiles on CTA pairs, the same epilogue, the same values bit for bit;
// falls back to the 128-row kernel for shapes the pair kernel does not take.
extern "C" int hb200_nvfp4_grouped_matmul_silu_256(const void* a_packed, const void* b_packed, const void* scale_a,
                                                   const void* scale_b, void* y_out, float* row_amax,
                                                   const int32_t* tile_info, int64_t max_m_tiles, int64_t n, int64_t k,
                                                   int64_t groups, int64_t ldy, const float* row_scale,
                                                   const float* group_alpha, float alpha, void* stream) {
  using namespace hb200;
  const bool pair_ok = a_packed && b_packed && scale_a && scale_b && y_out && row_amax && tile_info && max_m_tiles > 0 &&
                       (max_m_tiles % 2) == 0 && n > 0 && (n % 256) == 0 && k > 0 && (k % 32) == 0 && groups > 0 &&
                       ldy >= n / 2 && (ldy % 8) == 0 && max_m_tiles * 128 <= 0x7fffff00 && n * groups <= 0x7fffff00 &&
                       k <= 0x7fffff00 && reinterpret_cast<uintptr_t>(a_packed) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(b_packed) % 16 == 0 && reinterpret_cast<uintptr_t>(scale_a) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(scale_b) % 16 == 0 && reinterpret_cast<uintptr_t>(tile_info) % 8 == 0 &&
                       reinterpret_cast<uintptr_t>(y_out) % 16 == 0;
  if (pair_ok) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(row_amax, 0, size_t(max_m_tiles) * 128 * sizeof(float), s) != cudaSuccess) return HB200_ERR_CUDA;
    const int rc = pair::launch_grouped_pair(a_packed, b_packed, scale_a, scale_b, y_out, tile_info, max_m_tiles, n, k,
                                             groups, ldy, row_scale, group_alpha, alpha, 0, s, row_amax);
    if (rc != HB200_ERR_UNSUPPORTED) return rc;
  }
  return hb200_nvfp4_grouped_matmul_silu(a_packed, b_packed, scale_a, scale_b, y_out, row_amax, tile_info, max_m_tiles,
                                         n, k, groups, ldy, row_scale, group_alpha, alpha, stream);
}

// Reads (and optionally clears) the sticky device status set by kernels whose
// bounded waits ran out.  Synchronises the device.
namespace hb200 {
int f16_device_status(int reset);
int peer_device_status(int reset);
int gemv_tc_device_status(int reset);
int fp8_device_status(int reset);
int dense_device_status(int reset);
int dense_set_wait_budget(long long cycles);
int f16_set_wait_budget(long long cycles);
int peer_set_wait_budget(long long cycles);
int gemv_tc_set_wait_budget(long long cycles);
int fp8_set_wait_budget(long long cycles);

namespace {
// One CTA whose thread 0 waits, with the bounded wait every pipeline here uses, on an mbarrier that nothing
// ever completes: the wait runs out, the kernel records the sticky timeout status and returns.
__global__ void bounded_wait_selftest_kernel() {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    sm100::mbar_init(sm100::smem_u32(&bar), 1);
    sm100::fence_barrier_init();
    if (!sm100::mbar_wait(sm100::smem_u32(&bar), 0, &abort_flag)) atomicMin(&g_device_status, HB200_ERR_DEVICE_TIMEOUT);
  }
}
}  // namespace
}  // namespace hb200

// Sets the budget, in SM clock cycles, of every bounded device-side wait of the library (mbarrier waits of the
// tcgen05 pipelines, the flag wait of hb200_peer_barrier) on the current device; the default is 4e9 cycles,
// about two seconds.  Synchronous (a copy to device variables); not for use while kernels are in flight.
extern "C" int hb200_set_wait_budget_cycles(int64_t cycles) {
  using namespace hb200;
  if (cycles <= 0) return HB200_ERR_INVALID_ARGUMENT;
  if (!sm100::set_wait_budget_cycles(cycles)) return HB200_ERR_CUDA;
  int rc = f16_set_wait_budget(cycles);
  if (rc == HB200_OK) rc = peer_set_wait_budget(cycles);
  if (rc == HB200_OK) rc = gemv_tc_set_wait_budget(cycles);
  if (rc == HB200_OK) rc = fp8_set_wait_budget(cycles);
  if (rc == HB200_OK) rc = dense_set_wait_budget(cycles);
  return rc;
}

// Launches a one-CTA kernel whose bounded wait cannot be satisfied (an mbarrier nothing arrives on), to check
// the expiry path: after it, hb200_device_status reads HB200_ERR_DEVICE_TIMEOUT until reset.  It runs for one wait
// budget, so shorten the budget first.
extern "C" int hb200_selftest_bounded_wait(void* stream) {
  hb200::bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>();
  return hb200::launch_status();
}

extern "C" int hb200_device_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, hb200::g_device_status, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  if (reset && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(hb200::g_device_status, &zero, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  }
  const int w = hb200::f16_device_status(reset);
  const int p = hb200::peer_device_status(reset);
  const int t = hb200::gemv_tc_device_status(reset);
  const int f = hb200::fp8_device_status(reset);
  const int d = hb200::dense_device_status(reset);
  return v != 0 ? v : (w != 0 ? w : (p != 0 ? p : (t != 0 ? t : (f != 0 ? f : d))));
}
