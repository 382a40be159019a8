// Pieces shared by the block-scaled GEMM kernels: tile constants, the epilogue's
// row-chunk stores and the host-side TMA descriptor construction.
#pragma once

#include "common.cuh"
#include "tcgen05.cuh"

#include <mutex>

namespace hb200 {

constexpr int kBlockM = 128;
constexpr int kBlockKBytes = 128;   // one swizzle row: 256 e2m1 values
constexpr int kAtomBytes = 512;     // one 128-row x 4-scale atom (64 K-elements)
constexpr int kAtomsPerStage = 4;

// 32 consecutive fp32 accumulator columns of one row -> scaled, converted, stored (vectorised when whole and aligned).
template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* dst, const uint32_t (&r)[32], float alpha, int valid, bool vec_ok);

// 32 bytes in one instruction (sm_100 has 256-bit global stores): a whole sector per lane, half the store
// instructions of 16-byte stores.  dst must be 32-byte aligned.
__device__ __forceinline__ void stg_v8(void* dst, const uint32_t (&p)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(p[0]), "r"(p[1]), "r"(p[2]),
               "r"(p[3]), "r"(p[4]), "r"(p[5]), "r"(p[6]), "r"(p[7])
               : "memory");
}

template <>
__device__ __forceinline__ void store_row_chunk<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t (&r)[32], float alpha,
                                                               int valid, bool vec_ok) {
  if (valid >= 32 && vec_ok && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      uint32_t p[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 16 + 2 * j]) * alpha,
                                                       __uint_as_float(r[v * 16 + 2 * j + 1]) * alpha);
        p[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      stg_v8(dst + v * 16, p);
    }
  } else if (valid >= 32 && vec_ok) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint32_t p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]) * alpha,
                                                       __uint_as_float(r[v * 8 + 2 * j + 1]) * alpha);
        p[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(p[0], p[1], p[2], p[3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]) * alpha);
  }
}

template <>
__device__ __forceinline__ void store_row_chunk<__half>(__half* dst, const uint32_t (&r)[32], float alpha, int valid,
                                                        bool vec_ok) {
  if (valid >= 32 && vec_ok && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      uint32_t p[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        p[j] = h2_as_u32(__floats2half2_rn(__uint_as_float(r[v * 16 + 2 * j]) * alpha,
                                           __uint_as_float(r[v * 16 + 2 * j + 1]) * alpha));
      stg_v8(dst + v * 16, p);
    }
  } else if (valid >= 32 && vec_ok) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint32_t p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        p[j] = h2_as_u32(__floats2half2_rn(__uint_as_float(r[v * 8 + 2 * j]) * alpha,
                                           __uint_as_float(r[v * 8 + 2 * j + 1]) * alpha));
      *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(p[0], p[1], p[2], p[3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) dst[j] = __float2half_rn(__uint_as_float(r[j]) * alpha);
  }
}

template <>
__device__ __forceinline__ void store_row_chunk<float>(float* dst, const uint32_t (&r)[32], float alpha, int valid,
                                                       bool vec_ok) {
  if (valid >= 32 && vec_ok) {
#pragma unroll
    for (int v = 0; v < 8; ++v)
      *reinterpret_cast<float4*>(dst + v * 4) =
          make_float4(__uint_as_float(r[v * 4]) * alpha, __uint_as_float(r[v * 4 + 1]) * alpha,
                      __uint_as_float(r[v * 4 + 2]) * alpha, __uint_as_float(r[v * 4 + 3]) * alpha);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) dst[j] = __uint_as_float(r[j]) * alpha;
  }
}


// ------------------------------------------------------- stream-K work split
// The contiguous range of (tile, K block) units of CTA c when `total` units are dealt to `grid` CTAs.
__device__ __forceinline__ int range_start(int c, int total, int grid) { return int((int64_t(c) * total) / grid); }

__device__ __forceinline__ int owner_of(int unit, int total, int grid) {
  int c = int((int64_t(unit) * grid) / total);
  while (c + 1 < grid && range_start(c + 1, total, grid) <= unit) ++c;
  while (c > 0 && range_start(c, total, grid) > unit) --c;
  return c;
}

// The segments (tile, K blocks [kb0, kb1)) of a CTA's unit range [u_begin, u_end), in the order it works on them.
// In natural order only the first and the last can be partial tiles.  With three or more segments and a partial
// last one, that one is moved to second place: both partial tiles are then published (and, where this CTA
// arrives last, finished) while the whole tiles still stream, and the kernel's tail is a plain tile write.
struct Segments {
  int first_tile, count, kb_total, u_begin, u_end;
  bool tail_first;
  __device__ Segments(int ub, int ue, int kb) : kb_total(kb), u_begin(ub), u_end(ue) {
    first_tile = ub / kb;
    count = ue > ub ? (ue - 1) / kb - first_tile + 1 : 0;
    tail_first = count >= 3 && (ue % kb) != 0;
  }
  __device__ void get(int i, int& tile, int& kb0, int& kb1) const {
    const int j = !tail_first ? i : (i == 0 ? 0 : (i == 1 ? count - 1 : i - 1));
    tile = first_tile + j;
    kb0 = j == 0 ? u_begin - first_tile * kb_total : 0;
    kb1 = j == count - 1 ? u_end - tile * kb_total : kb_total;
  }
};

// ----------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Packed e2m1 matrix [rows, k/2 bytes] as a byte tensor; box = 128 bytes x box_rows, 128-byte swizzle.
inline bool make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k_bytes, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(k_bytes), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(k_bytes)};
  const cuuint32_t box[2] = {cuuint32_t(kBlockKBytes), cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


// Swizzled scale buffer as a [atoms, 128 x u32] tensor: one row per 512-byte atom; box = 4 atoms.
inline bool make_scale_map(CUtensorMap* map, const void* base, int64_t atoms) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {128, cuuint64_t(atoms)};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, cuuint32_t(kAtomsPerStage)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Row-major 2-byte output [rows, cols] (leading dimension ldc elements) for the epilogue's TMA stores:
// box = 32 columns (64 bytes) x 32 rows, 64-byte swizzle.
// Output boxes of 32 rows: 32 columns (64-byte rows, 64-byte swizzle) or, wide, 64 columns (128-byte rows,
// 128-byte swizzle: longer contiguous writes, which is what a store over NVLink wants).
inline bool make_output_map16(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int64_t ldc, bool is_bf16,
                              bool wide = false) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(ldc) * 2};
  const cuuint32_t box[2] = {wide ? 64u : 32u, 32};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides,
            box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, wide ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace hb200
