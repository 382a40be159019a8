// Shared device helpers for the sm_100a kernels: error codes, packed-format
// conversions (e2m1 / e4m3 / bf16), cache-hinted loads and warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/helion_b200.h"

namespace hb200 {

constexpr int kWarp = 32;

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t round_up64(int64_t a, int64_t b) { return ceil_div64(a, b) * b; }

// Flat offset of logical scale (row, col) inside the SWIZZLE_32_4_4 layout:
// 512-byte tiles of 128 rows x 4 columns, row-tile major, then column tile
// (reference: examples/nvfp4_gemv.py:68-79).
__host__ __device__ inline int64_t swizzled_scale_offset(int64_t row, int64_t col, int64_t cols) {
  const int64_t col_tiles = (cols + 3) / 4;
  return ((row / 128) * col_tiles + col / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + col % 4;
}

// Where a kernel writes its bf16 result rows: one buffer, or the same place in the buffer of every rank of a
// tensor-parallel group (peer-mapped pointers), at column col0 of rows of ld elements.
// Reduce-scatter form (scatter_rows > 0, a rank that holds a K shard): the fp32 partial of output row r goes to rank
// r / scatter_rows only, into that rank's fp32 buffer [world, batch_cap, scatter_rows] at [src_rank, b, r % scatter_rows]
// (ptr[] then hold those buffers); the owner adds the partials up in rank order (hb200_tp_reduce_partials).
struct OutSpec {
  __nv_bfloat16* ptr[8];
  int count;
  int64_t ld;
  int64_t col0;
  int64_t scatter_rows;
  int src_rank, batch_cap;
};

// One output value (row = output column index, b = activation row) as every GEMV kernel writes it.
__device__ __forceinline__ void store_out(const OutSpec& o, int b, int64_t row, float value) {
  if (o.scatter_rows > 0) {
    const int64_t owner = row / o.scatter_rows;
    float* dst = reinterpret_cast<float*>(o.ptr[owner]);
    dst[(int64_t(o.src_rank) * o.batch_cap + b) * o.scatter_rows + (row - owner * o.scatter_rows)] = value;
    return;
  }
  const __nv_bfloat16 v = __float2bfloat16_rn(value);
  for (int p = 0; p < o.count; ++p) o.ptr[p][int64_t(b) * o.ld + o.col0 + row] = v;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HB200_OK : HB200_ERR_CUDA;
}

// ---------------------------------------------------------------- conversions

// Two packed e2m1 codes (low nibble = first element) -> half2 (exact).
__device__ __forceinline__ uint32_t e2m1x2_to_h2(uint32_t byte) {
  uint32_t r;
  asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(r) : "r"(byte));
  return r;
}

// Four bytes (8 codes) of a 32-bit word -> four half2 values in element order.
__device__ __forceinline__ void e2m1x8_to_h2x4(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t"
      "}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}

// Two e4m3 bytes (low byte first) -> half2 (exact).
__device__ __forceinline__ uint32_t e4m3x2_to_h2(uint32_t two_bytes) {
  uint32_t r;
  asm("{\n\t.reg .b16 s;\n\tcvt.u16.u32 s, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, s;\n\t}" : "=r"(r) : "r"(two_bytes));
  return r;
}

__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
  uint32_t h = e4m3x2_to_h2(byte & 0xffu);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h & 0xffffu)));
}

// fp32 pair -> two e4m3 bytes, round-to-nearest-even, saturating at +-448.
// Result byte 0 = lo, byte 1 = hi.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  unsigned short r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// ---------------------------------------------------------------------- loads

// Streaming 16-byte load: read-only path, no L1 allocation (data is used once).
__device__ __forceinline__ uint4 ldg_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint2 ldg_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ void stg_stream_u4(void* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1, %2, %3, %4};"
               :
               : "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void stg_stream_u2(void* p, uint2 v) {
  asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1, %2};" : : "l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// ----------------------------------------------------------------- reductions

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace hb200
