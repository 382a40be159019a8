// Dense 8-bit GEMM on CTA pairs (tcgen05 cta_group::2, kind::f8f6f4 or kind::i8) for the prefill shapes of
// scaled_mm (pretuned_kernels/scaled_mm/scaled_mm.py:18-84).  Included by gemm_fp8.cu (one translation unit, so
// both kernels share the sticky device status word).
//
//   c[m, n] = cast(scale_b[n] * (scale_a[m] * acc[m, n])) + bias[n],   acc = a[m, :] . b[n, :]
//
// Unlike the decode kernel, the activations ride the tensor core's M side: two CTAs on neighbouring SMs own one
// 256 x 256 output tile, CTA r of the pair holds rows [128 r, 128 r + 128) of the a tile and of the b tile, and
// the leader issues 256 x 256 x 32 MMAs that read both halves: per 128 bytes of K every SM pulls 16 KB of a and
// 16 KB of b from L2 for 128 x 256 outputs.  Without block scales the 512 columns of tensor memory hold two
// accumulators, so the epilogue of a tile (scales, cast, bias, staged through shared memory into TMA stores) runs
// beside the next tile's MMAs.  No load is multicast; every wait is bounded; the kernel ends with a hardware
// cluster barrier so neither CTA exits while its peer may still touch its shared memory or barriers.
#pragma once

#include "gemm_common.cuh"

#include <type_traits>

namespace hb200 {
namespace dense_pair {

using namespace sm100;

constexpr int kThreads = 640;  // producer, MMA issuer, two idle warps, sixteen epilogue warps
constexpr int kTile = 256;
constexpr int kStages = 6;
constexpr int kHalfBytes = 128 * 128;          // this CTA's 128 rows of a (or of b) x 128 bytes of K
constexpr int kStageBytes = 2 * kHalfBytes;    // 32 KB
constexpr int kBoxBytes = 2048;                // one 32-row x 64-byte output box per epilogue warp
constexpr int kAcc = 2;
constexpr size_t kSmemBytes = size_t(kStages) * kStageBytes + 16 * kBoxBytes + (2 * kStages + 2 * kAcc) * 8 + 16 + 1024;
static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");

struct Args {
  void* out;
  int64_t ldc;
  const float* scale_a;  // [M] or [1]
  const float* scale_b;  // [N] or [1]
  const void* bias;      // [N] in the output type, or nullptr
  int m, n, k_bytes;
  int scale_a_per_row, scale_b_per_col;
  int m_tiles, n_tiles;
  int band;  // row tiles per band of the tile order
};

__device__ __forceinline__ void mma_pair_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_pair_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Tile order: bands of `band` row tiles; inside a band the row tile runs fastest, then the column tile.  The 74
// pairs that work at the same time then share a few row tiles of a and a few column tiles of b, which stay in L2.
__device__ __forceinline__ void decode_tile(const Args& g, int tile, int& m_blk, int& n_blk) {
  const int per_band = g.band * g.n_tiles;
  const int b = tile / per_band, r = tile - b * per_band;
  const int rows_here = min(g.band, g.m_tiles - b * g.band);
  n_blk = r / rows_here;
  m_blk = b * g.band + (r - n_blk * rows_here);
}

template <typename T> __device__ __forceinline__ T cast_out(float v);
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(float v) { return v; }

// format: 0 = e4m3, 1 = e5m2, 2 = int8 (int32 accumulator, converted to fp32 once)
template <typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
dense_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_out, const Args g, const int format) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_out = smem + kStages * kStageBytes;  // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + 16 * kBoxBytes);
  uint64_t* full_bar = bars;                   // used in the leader only
  uint64_t* empty_bar = bars + kStages;        // one set per CTA
  uint64_t* tmem_full_bar = bars + 2 * kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + kAcc;  // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + kAcc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_kb = (g.k_bytes + 127) / 128;
  const int num_tiles = g.m_tiles * g.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);   // the leader's producer arms it; bytes come from both CTAs
      mbar_init(smem_u32(&empty_bar[s]), 1);  // the leader's commit, sent to both CTAs
    }
    for (int a = 0; a < kAcc; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 32);  // sixteen epilogue warps in each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
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
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int m_blk, n_blk;
      decode_tile(g, tile, m_blk, n_blk);
      const int a_row = m_blk * kTile + int(rank) * 128;
      const int b_row = n_blk * kTile + int(rank) * 128;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kStages;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
        uint8_t* st = smem + s * kStageBytes;
        const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);  // always the leader's barrier
        if (elect_one()) {
          if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[s]), 2 * kStageBytes);
          tma_load_2d_pair(smem_u32(st), &tmap_a, kb * 128, a_row, bar);
          tma_load_2d_pair(smem_u32(st + kHalfBytes), &tmap_b, kb * 128, b_row, bar);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (leader only)
    if (leader) {
      const bool is_int = format == 2;
      // fp32 (or int32) accumulator at bits 4-5, operand formats at bits 7-9 and 10-12, N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t idesc = (is_int ? ((2u << 4) | (1u << 7) | (1u << 10))
                                     : ((1u << 4) | (uint32_t(format) << 7) | (uint32_t(format) << 10))) |
                             (uint32_t(kTile >> 3) << 17) | (uint32_t(256 >> 4) << 24);
      bool ok = true;
      uint32_t it = 0, tc = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tc) {
        const int acc = tc % kAcc;
        if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), ((tc / kAcc) & 1) ^ 1, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kTile;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(smem_u32(&full_bar[s]), (it / kStages) & 1, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          uint8_t* st = smem + s * kStageBytes;
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + kHalfBytes);
          const int k_left = g.k_bytes - kb * 128;
          const int steps = k_left >= 128 ? 4 : (k_left + 31) / 32;  // K tail: TMA zero-fills past K
          if (elect_one()) {
            for (int a = 0; a < steps; ++a) {
              const uint64_t adesc = make_smem_desc(a_addr + a * 32, 16, 1024, kSwizzle128B);
              const uint64_t bdesc = make_smem_desc(b_addr + a * 32, 16, 1024, kSwizzle128B);
              if (is_int) mma_pair_i8(tmem_d, adesc, bdesc, idesc, (kb | a) != 0 ? 1u : 0u);
              else mma_pair_f8(tmem_d, adesc, bdesc, idesc, (kb | a) != 0 ? 1u : 0u);
            }
            tcgen05_commit_pair(smem_u32(&empty_bar[s]), 3);  // stage free in both CTAs
          }
          __syncwarp();
        }
        if (ok && elect_one()) tcgen05_commit_pair(smem_u32(&tmem_full_bar[acc]), 3);
        __syncwarp();
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (both CTAs)
    // Sixteen warps: warp w reads lane quarter w % 4 (the only one it may) and the 64 columns [(w - 4) / 4 * 64, +64)
    // into registers with two loads, hands the accumulator back, then scales, casts, adds the bias and stores.
    const int quarter = warp & 3, cgroup = (warp - 4) >> 2;
    const bool is_int = format == 2;
    OutT* out = static_cast<OutT*>(g.out);
    const OutT* bias = static_cast<const OutT*>(g.bias);
    uint8_t* box = stage_out + (warp - 4) * kBoxBytes;
    const float sa_all = g.scale_a[0], sb_all = g.scale_b[0];
    uint32_t tc = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tc) {
      int m_blk, n_blk;
      decode_tile(g, tile, m_blk, n_blk);
      const int acc = tc % kAcc;
      const int row0 = m_blk * kTile + int(rank) * 128 + quarter * 32;
      const int row = row0 + lane;
      const int col = n_blk * kTile + cgroup * 64;
      // this row's scale and the columns' scales and biases (lane l keeps columns col + l and col + 32 + l) are
      // fetched before the wait
      const float sa = g.scale_a_per_row ? (row < g.m ? g.scale_a[row] : 0.f) : sa_all;
      float sb_l[2], bias_l[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = col + h * 32 + lane;
        sb_l[h] = g.scale_b_per_col ? (c < g.n ? g.scale_b[c] : 0.f) : sb_all;
        bias_l[h] = (bias != nullptr && c < g.n) ? widen(bias[c]) : 0.f;
      }
      if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), (tc / kAcc) & 1, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * kTile + cgroup * 64;
      uint32_t r[2][32];
      tmem_ld_32x32b_x32(taddr, r[0]);
      tmem_ld_32x32b_x32(taddr + 32, r[1]);
      tmem_ld_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        OutT o[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float v = is_int ? __int2float_rn(int(r[h][j])) : __uint_as_float(r[h][j]);
          const float sb = __shfl_sync(0xffffffffu, sb_l[h], j);
          o[j] = cast_out<OutT>(sb * (sa * v));
          if (bias != nullptr) o[j] = cast_out<OutT>(widen(o[j]) + __shfl_sync(0xffffffffu, bias_l[h], j));
        }
        if constexpr (sizeof(OutT) == 2) {
          // a box of 32 rows x 32 columns (64 bytes per row, 64-byte swizzle) through this warp's staging buffer
          if (lane == 0) bulk_wait_group_read0();
          __syncwarp();
          uint8_t* rowp = box + lane * 64;
          const uint32_t* p = reinterpret_cast<const uint32_t*>(o);
#pragma unroll
          for (int v = 0; v < 4; ++v)  // 16-byte chunk index xor bits 1..2 of the row
            *reinterpret_cast<uint4*>(rowp + ((v ^ ((lane >> 1) & 3)) << 4)) =
                make_uint4(p[4 * v], p[4 * v + 1], p[4 * v + 2], p[4 * v + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < g.m && col + h * 32 < g.n) {
            tma_store_2d(&tmap_out, col + h * 32, row0, smem_u32(box));  // rows and columns past the edge are clipped
            bulk_commit_group();
          }
        } else {
          if (row < g.m) {
            float* dst = reinterpret_cast<float*>(out) + int64_t(row) * g.ldc + col + h * 32;
            const int valid = g.n - (col + h * 32);
            if (valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                *reinterpret_cast<float4*>(dst + 4 * v) = make_float4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < valid) dst[j] = o[j];
            }
          }
        }
      }
    }
    if constexpr (sizeof(OutT) == 2) {
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
  if (threadIdx.x == 0 && *abort_flag) atomicMin(&g_device_status_fp8, HB200_ERR_DEVICE_TIMEOUT);
}

// K-major byte matrix [rows, K] with a row pitch of `pitch` bytes; box = 128 bytes x 128 rows, 128-byte swizzle.
inline bool make_byte_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t pitch) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(pitch)};
  const cuuint32_t box[2] = {128, 128};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns HB200_ERR_UNSUPPORTED for what the kernel does not take (the caller then uses the decode kernel).
inline int launch(const void* a, const void* b, void* c, const float* scale_a, const float* scale_b, const void* bias,
                  int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int scale_a_per_row,
                  int scale_b_per_col, int format, int out_dtype, int sms, cudaStream_t stream) {
  if (m < 256 || n < 256) return HB200_ERR_UNSUPPORTED;
  if (out_dtype != 2 && ((ldc % 8) != 0 || reinterpret_cast<uintptr_t>(c) % 16)) return HB200_ERR_UNSUPPORTED;
  CUtensorMap ta, tb, tout;
  if (!make_byte_map(&ta, a, m, k, lda) || !make_byte_map(&tb, b, n, k, ldb)) return HB200_ERR_CUDA;
  if (out_dtype == 2) tout = ta;  // unused by the fp32 epilogue
  else if (!make_output_map16(&tout, c, m, n, ldc, out_dtype == 0)) return HB200_ERR_CUDA;
  Args g{};
  g.out = c;
  g.ldc = ldc;
  g.scale_a = scale_a;
  g.scale_b = scale_b;
  g.bias = bias;
  g.m = int(m);
  g.n = int(n);
  g.k_bytes = int(k);
  g.scale_a_per_row = scale_a_per_row != 0;
  g.scale_b_per_col = scale_b_per_col != 0;
  g.m_tiles = int((m + kTile - 1) / kTile);
  g.n_tiles = int((n + kTile - 1) / kTile);
  g.band = 8;
  const int tiles = g.m_tiles * g.n_tiles;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
#define HB200_DENSE_PAIR(T)                                                                                         \
  do {                                                                                                              \
    auto kernel = dense_pair_kernel<T>;                                                                             \
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)) != cudaSuccess)  \
      return HB200_ERR_CUDA;                                                                                        \
    kernel<<<2 * pairs, kThreads, kSmemBytes, stream>>>(ta, tb, tout, g, format);                                   \
  } while (0)
  if (out_dtype == 0) HB200_DENSE_PAIR(__nv_bfloat16);
  else if (out_dtype == 1) HB200_DENSE_PAIR(__half);
  else HB200_DENSE_PAIR(float);
#undef HB200_DENSE_PAIR
  return launch_status();
}

}  // namespace dense_pair
}  // namespace hb200
