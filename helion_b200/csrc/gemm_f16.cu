// bf16 / fp16 grouped GEMM for sm_100a (tcgen05 kind::f16, fp32 accumulate):
//   out[r, :] = A[r, :] . B[g(r)]^T     A [rows, K] and B [groups * N, K] both K-major.
// The work is a list of row tiles (group, first row, valid rows, rows to store): rows past
// "valid" count as zero on input, rows past "store" are left untouched.  This covers the
// reference's grouped GEMMs: the worklist form of grouped_gemm_deepgemm
// (pretuned_kernels/grouped_gemm_deepgemm/grouped_gemm_deepgemm.py:172-224), the sorted-token
// expert GEMM of moe_matmul_ogs (examples/moe_matmul_ogs.py:31-85) and, with one group, the
// shared-B jagged GEMM (examples/grouped_gemm.py:52-104) and a plain dense GEMM.
//
// Same structure as the NVFP4 kernel without scale factors: persistent CTAs, warp 0 TMA producer
// (A tile 128 x 64, B tile 256 x 64 elements, 128-byte swizzle, no multicast), warp 1 MMA issuer
// (128 x 256 x 16 per instruction), warps 2-5 epilogue; two accumulator stages in tensor memory so
// the epilogue of a tile overlaps the next tile's MMAs; bounded waits throughout.
#include "gemm_common.cuh"

#include <type_traits>

namespace hb200 {

__device__ int g_device_status_f16 = 0;

namespace {

using namespace sm100;

constexpr int kF16Threads = 192;
constexpr int kF16BlockN = 256;
constexpr int kF16Stages = 4;
constexpr int kF16ABytes = 128 * 128;
constexpr int kF16BBytes = kF16BlockN * 128;
constexpr int kF16StageBytes = kF16ABytes + kF16BBytes;  // 48 KB

struct F16Args {
  void* out;
  int64_t ldc;
  int n, k;
  const int4* tiles;  // (group, first row, valid rows, rows to store); group < 0 ends the list early
  int num_row_tiles, n_tiles;
};

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor of kind::f16: fp32 accumulator (bits 4-5 = 1), operand format 0 = f16 / 1 = bf16
// (bits 7-9 and 10-12), both operands K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_f16(int m, int n, bool bf16) {
  return (1u << 4) | (uint32_t(bf16 ? 1 : 0) << 7) | (uint32_t(bf16 ? 1 : 0) << 10) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

template <typename T>
__global__ void __launch_bounds__(kF16Threads, 1)
grouped_gemm_f16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const F16Args g) {
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int ACC = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kF16Stages * kF16StageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kF16Stages;
  uint64_t* tmem_full_bar = bars + 2 * kF16Stages;
  uint64_t* tmem_empty_bar = tmem_full_bar + ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (g.k + 63) / 64;
  const int num_tiles = g.num_row_tiles * g.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF16Stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < ACC; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (row tile, column tile); all column tiles of a row tile run back to back
  auto row_tile = [&](int tile) -> int4 { return g.tiles[tile / g.n_tiles]; };

  if (warp == 0) {
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int4 rt = row_tile(tile);
      if (rt.x < 0 || rt.w <= 0) continue;
      const int n_blk = tile % g.n_tiles;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kF16Stages;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / kF16Stages) & 1) ^ 1, abort_flag)) { ok = false; break; }
        const uint32_t bar = smem_u32(&full_bar[s]);
        uint8_t* st = smem + s * kF16StageBytes;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar, kF16StageBytes);
          tma_load_2d(smem_u32(st), &tmap_a, kb * 64, rt.y, bar);
          tma_load_2d(smem_u32(st + kF16ABytes), &tmap_b, kb * 64, rt.x * g.n + n_blk * kF16BlockN, bar);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc_f16(128, kF16BlockN, kBf16);
    uint32_t it = 0, tc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int4 rt = row_tile(tile);
      if (rt.x < 0 || rt.w <= 0) continue;
      const int acc = tc % ACC;
      const uint32_t acc_ph = (tc / ACC) & 1;
      ++tc;
      if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_ph ^ 1, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t tmem_d = tmem_base + acc * kF16BlockN;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kF16Stages;
        if (!mbar_wait(smem_u32(&full_bar[s]), (it / kF16Stages) & 1, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        uint8_t* st = smem + s * kF16StageBytes;
        const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + kF16ABytes);
        const int k_left = g.k - kb * 64;
        const int steps = k_left >= 64 ? 4 : (k_left + 15) / 16;  // K tail: TMA zero-fills past K
        if (elect_one()) {
          for (int a = 0; a < steps; ++a) {
            // 16 K-elements = 32 bytes further along the 128-byte swizzled row
            const uint64_t adesc = make_smem_desc(a_addr + a * 32, 16, 1024, kSwizzle128B);
            const uint64_t bdesc = make_smem_desc(b_addr + a * 32, 16, 1024, kSwizzle128B);
            mma_f16(tmem_d, adesc, bdesc, idesc, (kb | a) != 0 ? 1u : 0u);
          }
          tcgen05_commit(smem_u32(&empty_bar[s]));
        }
        __syncwarp();
      }
      if (ok && elect_one()) tcgen05_commit(smem_u32(&tmem_full_bar[acc]));
      __syncwarp();
    }
  } else {
    const int quarter = warp & 3;
    T* out = static_cast<T*>(g.out);
    const bool vec_ok = (g.ldc * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(g.out) % 16) == 0;
    uint32_t tc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int4 rt = row_tile(tile);
      if (rt.x < 0 || rt.w <= 0) continue;
      const int n_blk = tile % g.n_tiles;
      const int acc = tc % ACC;
      const uint32_t acc_ph = (tc / ACC) & 1;
      ++tc;
      if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_ph, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const int r_in = quarter * 32 + lane;
      const int64_t row = int64_t(rt.y) + r_in;
      const bool store = r_in < rt.w;
      const float keep = r_in < rt.z ? 1.0f : 0.0f;  // rows between "valid" and "store" are written as zero
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * kF16BlockN;
#pragma unroll 1
      for (int c = 0; c < kF16BlockN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n_blk * kF16BlockN + c * 32;
        if (store && col < g.n) store_row_chunk<T>(out + row * g.ldc + col, r, keep, g.n - col, vec_ok);
      }
      tcgen05_fence_before();
      mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicMin(&g_device_status_f16, HB200_ERR_DEVICE_TIMEOUT);
}

// K-major 2-byte matrix [rows, K]; box = 64 elements (128 bytes) x box_rows, 128-byte swizzle.
bool make_f16_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows, bool bf16) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(k) * 2};
  const cuuint32_t box[2] = {64, cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base),
            dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Row tiles of a jagged layout: group g owns rows [offsets[g], offsets[g+1]); one 128-row tile list entry per
// 128 rows of every group, (-1, 0, 0, 0) after the last.  One CTA.
__global__ void __launch_bounds__(256)
build_row_tiles_kernel(const int32_t* __restrict__ offsets, int groups, int4* __restrict__ tiles, int max_tiles) {
  __shared__ int32_t first_tile[1025];
  if (threadIdx.x == 0) {
    int32_t t = 0;
    for (int gidx = 0; gidx < groups; ++gidx) {
      first_tile[gidx] = t;
      const int32_t rows = max(offsets[gidx + 1] - offsets[gidx], 0);
      t += (rows + 127) / 128;
    }
    first_tile[groups] = t;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    int4 info = make_int4(-1, 0, 0, 0);
    if (t < first_tile[groups]) {
      int lo = 0, hi = groups;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (first_tile[mid] <= t) lo = mid; else hi = mid;
      }
      const int32_t local = (t - first_tile[lo]) * 128;
      const int32_t rows = min(128, offsets[lo + 1] - offsets[lo] - local);
      info = make_int4(lo, offsets[lo] + local, rows, rows);
    }
    tiles[t] = info;
  }
}

}  // namespace
}  // namespace hb200

extern "C" int hb200_grouped_gemm_f16(const void* a, const void* b, void* out, const int32_t* row_tiles,
                                      int64_t num_row_tiles, int64_t a_rows, int64_t n, int64_t k, int64_t groups,
                                      int64_t ldc, int is_bf16, void* stream) {
  using namespace hb200;
  if (!a || !b || !out || !row_tiles) return HB200_ERR_INVALID_ARGUMENT;
  if (num_row_tiles < 0 || a_rows < 0 || n < 0 || k <= 0 || groups <= 0 || ldc < n) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(b) % 16 ||
      reinterpret_cast<uintptr_t>(row_tiles) % 16)
    return HB200_ERR_INVALID_ARGUMENT;
  if (num_row_tiles == 0 || n == 0 || a_rows == 0) return HB200_OK;
  if ((k % 8) != 0) return HB200_ERR_UNSUPPORTED;  // TMA needs a 16-byte row pitch
  if (a_rows > 0x7fffff00 || n * groups > 0x7fffff00 || num_row_tiles > 0xffffff) return HB200_ERR_UNSUPPORTED;
  CUtensorMap ta, tb;
  if (!make_f16_map(&ta, a, a_rows, k, 128, is_bf16 != 0)) return HB200_ERR_CUDA;
  if (!make_f16_map(&tb, b, n * groups, k, kF16BlockN, is_bf16 != 0)) return HB200_ERR_CUDA;
  F16Args g{out, ldc, int(n), int(k), reinterpret_cast<const int4*>(row_tiles), int(num_row_tiles),
            int((n + kF16BlockN - 1) / kF16BlockN)};
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = num_row_tiles * g.n_tiles;
  const int grid = int(tiles < sms ? tiles : sms);
  constexpr size_t smem = size_t(kF16Stages) * kF16StageBytes + (2 * kF16Stages + 4) * 8 + 16 + 1024;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16) {
    auto kernel = grouped_gemm_f16_kernel<__nv_bfloat16>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
    kernel<<<grid, kF16Threads, smem, s>>>(ta, tb, g);
  } else {
    auto kernel = grouped_gemm_f16_kernel<__half>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
    kernel<<<grid, kF16Threads, smem, s>>>(ta, tb, g);
  }
  return launch_status();
}

extern "C" int hb200_build_row_tiles(const int32_t* group_offsets, int64_t groups, int32_t* row_tiles,
                                     int64_t max_tiles, void* stream) {
  using namespace hb200;
  if (!group_offsets || !row_tiles) return HB200_ERR_INVALID_ARGUMENT;
  if (groups <= 0 || groups > 1024 || max_tiles < 0 || max_tiles > 0xffffff) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(row_tiles) % 16) return HB200_ERR_INVALID_ARGUMENT;
  if (max_tiles == 0) return HB200_OK;
  build_row_tiles_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(group_offsets, int(groups),
                                                                           reinterpret_cast<int4*>(row_tiles),
                                                                           int(max_tiles));
  return launch_status();
}

namespace hb200 {
// Sticky status of this translation unit's kernels, folded into hb200_device_status().
int f16_device_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status_f16, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  if (reset && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_device_status_f16, &zero, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  }
  return v;
}
}  // namespace hb200
