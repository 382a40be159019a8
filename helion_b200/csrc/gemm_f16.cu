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
  int rows_total;  // rows of A and of the output: tile entries come from device data and are not trusted beyond this
  int groups;
};

// Direct mode (heterogeneous groups): every group has operands and an output of its own, with its own N and K.
// The tensor maps and the per-group extents ride in kernel parameter space; a launch takes up to kDirectGroups.
constexpr int kDirectGroups = 8;
struct DirectMaps {
  CUtensorMap a[kDirectGroups], b[kDirectGroups];
};
struct DirectGroups {
  void* out[kDirectGroups];
  int64_t ldc[kDirectGroups];
  int m[kDirectGroups], n[kDirectGroups], k[kDirectGroups];
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

// DIRECT: the operands of tile (group, ...) come through that group's own tensor maps (row coordinates are local to
// the group's matrices), its K and N are the group's, and the rows go to the group's own output.
template <typename T, bool DIRECT>
__global__ void __launch_bounds__(kF16Threads, 1)
grouped_gemm_f16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ DirectMaps dmaps, const __grid_constant__ DirectGroups dgroups,
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
  const int num_tiles = g.num_row_tiles * g.n_tiles;
  // K and N of a tile's group; a column tile past the group's N is skipped by every role alike
  auto group_k = [&](int grp) -> int { return DIRECT ? dgroups.k[grp] : g.k; };
  auto group_n = [&](int grp) -> int { return DIRECT ? dgroups.n[grp] : g.n; };
  auto skip = [&](const int4& rt, int n_blk) -> bool {
    return rt.x < 0 || rt.x >= g.groups || rt.w <= 0 || n_blk * kF16BlockN >= group_n(rt.x);
  };

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
  auto row_tile = [&](int tile) -> int4 {
    if constexpr (!DIRECT) {
      return g.tiles[tile / g.n_tiles];
    } else {
      // groups own ceil(m / 128) consecutive row tiles each (groups with nothing to do have n == 0 and own none)
      int rt = tile / g.n_tiles;
      for (int i = 0; i < g.groups; ++i) {
        const int own = dgroups.n[i] > 0 ? (dgroups.m[i] + 127) >> 7 : 0;
        if (rt < own) {
          const int rows = min(128, dgroups.m[i] - rt * 128);
          return make_int4(i, rt * 128, rows, rows);
        }
        rt -= own;
      }
      return make_int4(-1, 0, 0, 0);
    }
  };

  if (warp == 0) {
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int4 rt = row_tile(tile);
      const int n_blk = tile % g.n_tiles;
      if (skip(rt, n_blk)) continue;
      const int num_kb = (group_k(rt.x) + 63) / 64;
      const CUtensorMap* ma = DIRECT ? &dmaps.a[rt.x] : &tmap_a;
      const CUtensorMap* mb = DIRECT ? &dmaps.b[rt.x] : &tmap_b;
      const int b_row = DIRECT ? n_blk * kF16BlockN : rt.x * g.n + n_blk * kF16BlockN;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kF16Stages;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / kF16Stages) & 1) ^ 1, abort_flag)) { ok = false; break; }
        const uint32_t bar = smem_u32(&full_bar[s]);
        uint8_t* st = smem + s * kF16StageBytes;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar, kF16StageBytes);
          tma_load_2d(smem_u32(st), ma, kb * 64, rt.y, bar);
          tma_load_2d(smem_u32(st + kF16ABytes), mb, kb * 64, b_row, bar);
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
      if (skip(rt, tile % g.n_tiles)) continue;
      const int k_g = group_k(rt.x);
      const int num_kb = (k_g + 63) / 64;
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
        const int k_left = k_g - kb * 64;
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
    uint32_t tc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int4 rt = row_tile(tile);
      const int n_blk = tile % g.n_tiles;
      if (skip(rt, n_blk)) continue;
      const int acc = tc % ACC;
      const uint32_t acc_ph = (tc / ACC) & 1;
      ++tc;
      if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_ph, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const int r_in = quarter * 32 + lane;
      const int64_t row = int64_t(rt.y) + r_in;
      const int rows_total = DIRECT ? dgroups.m[rt.x] : g.rows_total;
      const int n_g = group_n(rt.x);
      const int64_t ldc = DIRECT ? dgroups.ldc[rt.x] : g.ldc;
      T* out = DIRECT ? static_cast<T*>(dgroups.out[rt.x]) : static_cast<T*>(g.out);
      const bool vec_ok = (ldc * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(out) % 16) == 0;
      const bool store = r_in < rt.w && row >= 0 && row < rows_total;  // a tile list built from bad sizes cannot write outside
      const float keep = r_in < rt.z ? 1.0f : 0.0f;  // rows between "valid" and "store" are written as zero
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * kF16BlockN;
#pragma unroll 1
      for (int c = 0; c < kF16BlockN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n_blk * kF16BlockN + c * 32;
        if (store && col < n_g) store_row_chunk<T>(out + row * ldc + col, r, keep, n_g - col, vec_ok);
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

// The same map for a matrix whose rows are `pitch` elements apart (a view into a larger allocation).
bool make_f16_map_pitched(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t pitch, int box_rows,
                          bool bf16) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(pitch) * 2};
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

// Row tiles from per-group row counts ("split sizes", device-resident, int32 or int64, element stride `stride`):
// group g owns rows [P_g, P_g + size_g) with P the raw running sum of the sizes as given, clipped to the rows that
// exist: a size is first clipped to [0, total_rows] (in 64 bits, before any narrowing), the interval then to
// [0, total_rows).  Rows no group covers get no tile.  One CTA.
template <typename SizeT>
__global__ void __launch_bounds__(256)
build_split_tiles_kernel(const SizeT* __restrict__ sizes, int64_t stride, int groups, int total_rows,
                         int4* __restrict__ tiles, int max_tiles) {
  __shared__ int32_t first_tile[1025];
  __shared__ int32_t lo_row[1024], hi_row[1024];
  if (threadIdx.x == 0) {
    long long prefix = 0;
    int32_t t = 0;
    for (int gidx = 0; gidx < groups; ++gidx) {
      const long long raw = static_cast<long long>(sizes[int64_t(gidx) * stride]);
      const long long len = raw < 0 ? 0 : (raw > total_rows ? total_rows : raw);
      long long lo = prefix, hi = prefix + len;
      lo = lo < 0 ? 0 : (lo > total_rows ? total_rows : lo);
      hi = hi < 0 ? 0 : (hi > total_rows ? total_rows : hi);
      lo_row[gidx] = int32_t(lo);
      hi_row[gidx] = int32_t(hi > lo ? hi : lo);
      first_tile[gidx] = t;
      t += (hi_row[gidx] - lo_row[gidx] + 127) / 128;
      prefix += raw;  // the raw sum: a negative size moves the groups after it back
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
      const int32_t rows = min(128, hi_row[lo] - lo_row[lo] - local);
      info = make_int4(lo, lo_row[lo] + local, rows, rows);
    }
    tiles[t] = info;
  }
}

// Row tiles of a DeepGEMM-style worklist: item i = (group, start row, valid rows, rows to store) becomes
// ceil(store / 128) tiles.  Nothing in an item is trusted: a negative group or start drops the item, store is
// clipped to the rows that exist past start, valid to store; tiles past max_tiles are dropped.  One CTA.
__global__ void __launch_bounds__(256)
build_worklist_tiles_kernel(const int4* __restrict__ items, int num_items, int total_rows, int4* __restrict__ tiles,
                            int max_tiles) {
  extern __shared__ int32_t first_tile[];  // [num_items + 1]
  auto store_rows = [&](const int4 it) -> int32_t {
    if (it.x < 0 || it.y < 0 || it.y >= total_rows) return 0;
    return max(0, min(it.w, total_rows - it.y));
  };
  if (threadIdx.x == 0) {
    int32_t t = 0;
    for (int i = 0; i < num_items; ++i) {
      first_tile[i] = t;
      t += (store_rows(items[i]) + 127) / 128;
    }
    first_tile[num_items] = t;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    int4 info = make_int4(-1, 0, 0, 0);
    if (t < first_tile[num_items]) {
      int lo = 0, hi = num_items;  // last item with first_tile <= t (items without tiles share a value)
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (first_tile[mid] <= t) lo = mid; else hi = mid;
      }
      const int4 it = items[lo];
      const int32_t local = (t - first_tile[lo]) * 128;
      const int32_t store = store_rows(it);
      const int32_t valid = max(0, min(it.z, store));
      info = make_int4(it.x, it.y + local, max(0, min(128, valid - local)), min(128, store - local));
    }
    tiles[t] = info;
  }
}

}  // namespace
}  // namespace hb200

// Tile list (the row_tiles argument of hb200_grouped_gemm_f16) for a worklist [items, 4] of
// (group, start row, valid rows, rows to store) as grouped_gemm_deepgemm takes it
// (pretuned_kernels/grouped_gemm_deepgemm/grouped_gemm_deepgemm.py:172-224), built on the device without a
// host read: ceil(total_rows / 128) + items entries always suffice for items whose row ranges do not overlap.
extern "C" int hb200_build_worklist_tiles(const int32_t* worklist, int64_t items, int64_t total_rows,
                                          int32_t* row_tiles, int64_t max_tiles, void* stream) {
  using namespace hb200;
  if (!row_tiles || (items > 0 && !worklist)) return HB200_ERR_INVALID_ARGUMENT;
  if (items < 0 || items > 8192 || total_rows < 0 || total_rows > 0x7fffff00 || max_tiles < 0 || max_tiles > 0xffffff)
    return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(row_tiles) % 16 || reinterpret_cast<uintptr_t>(worklist) % 16)
    return HB200_ERR_INVALID_ARGUMENT;
  if (max_tiles == 0) return HB200_OK;
  build_worklist_tiles_kernel<<<1, 256, size_t(items + 1) * 4, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int4*>(worklist), int(items), int(total_rows), reinterpret_cast<int4*>(row_tiles),
      int(max_tiles));
  return launch_status();
}

// Tile list from device-resident per-group row counts (the "device split sizes" of the reference's grouped
// tcgen05 kernels, test/test_cute_grouped_gemm_split_sizes.py:620-745): sizes are int64 (sizes_are_i64 != 0) or
// int32 with an element stride; oversized, negative and beyond-int32 entries are clipped as that test pins them,
// never trusted.  groups <= 1024; max_tiles >= ceil(total_rows / 128) + groups suffices for sizes that do not
// make groups overlap (tiles past max_tiles are dropped).
extern "C" int hb200_build_split_tiles(const void* split_sizes, int sizes_are_i64, int64_t stride, int64_t groups,
                                       int64_t total_rows, int32_t* row_tiles, int64_t max_tiles, void* stream) {
  using namespace hb200;
  if (!split_sizes || !row_tiles) return HB200_ERR_INVALID_ARGUMENT;
  if (groups <= 0 || groups > 1024 || stride <= 0 || total_rows < 0 || total_rows > 0x7fffff00 || max_tiles < 0 ||
      max_tiles > 0xffffff)
    return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(row_tiles) % 16 || reinterpret_cast<uintptr_t>(split_sizes) % (sizes_are_i64 ? 8 : 4))
    return HB200_ERR_INVALID_ARGUMENT;
  if (max_tiles == 0) return HB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (sizes_are_i64)
    build_split_tiles_kernel<long long><<<1, 256, 0, s>>>(static_cast<const long long*>(split_sizes), stride, int(groups),
                                                         int(total_rows), reinterpret_cast<int4*>(row_tiles), int(max_tiles));
  else
    build_split_tiles_kernel<int32_t><<<1, 256, 0, s>>>(static_cast<const int32_t*>(split_sizes), stride, int(groups),
                                                       int(total_rows), reinterpret_cast<int4*>(row_tiles), int(max_tiles));
  return launch_status();
}

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
            int((n + kF16BlockN - 1) / kF16BlockN), int(a_rows), int(groups)};
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = num_row_tiles * g.n_tiles;
  const int grid = int(tiles < sms ? tiles : sms);
  constexpr size_t smem = size_t(kF16Stages) * kF16StageBytes + (2 * kF16Stages + 4) * 8 + 16 + 1024;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const DirectMaps no_maps{};
  const DirectGroups no_groups{};
  if (is_bf16) {
    auto kernel = grouped_gemm_f16_kernel<__nv_bfloat16, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
    kernel<<<grid, kF16Threads, smem, s>>>(ta, tb, no_maps, no_groups, g);
  } else {
    auto kernel = grouped_gemm_f16_kernel<__half, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
    kernel<<<grid, kF16Threads, smem, s>>>(ta, tb, no_maps, no_groups, g);
  }
  return launch_status();
}

// Direct mode of the reference's grouped GEMM (pretuned_kernels/grouped_gemm/grouped_gemm.py:213-327): group i is an
// NT GEMM of its own, out_i[m_i, n_i] = A_i[m_i, k_i] . B_i[n_i, k_i]^T, with operands and output anywhere in
// device memory (the reference passes a device table of pointers and strides; here the host arrays those tables
// were built from).  All pointer / size arrays are HOST arrays of `groups` entries; lda / ldb / ldc are row pitches in
// elements (unit stride along K and N).  One launch per eight groups.  k_i % 8 == 0, bases 16-byte aligned.
extern "C" int hb200_grouped_gemm_f16_direct(const void* const* a_ptrs, const void* const* b_ptrs, void* const* out_ptrs,
                                             const int64_t* m, const int64_t* n, const int64_t* k, const int64_t* lda,
                                             const int64_t* ldb, const int64_t* ldc, int64_t groups, int is_bf16,
                                             void* stream) {
  using namespace hb200;
  if (!a_ptrs || !b_ptrs || !out_ptrs || !m || !n || !k || !lda || !ldb || !ldc || groups < 0) return HB200_ERR_INVALID_ARGUMENT;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  constexpr size_t smem = size_t(kF16Stages) * kF16StageBytes + (2 * kF16Stages + 4) * 8 + 16 + 1024;
  for (int64_t g0 = 0; g0 < groups; g0 += kDirectGroups) {
    const int cnt = int(groups - g0 < kDirectGroups ? groups - g0 : kDirectGroups);
    DirectMaps maps{};
    DirectGroups dg{};
    int64_t row_tiles = 0, max_n = 0;
    for (int i = 0; i < cnt; ++i) {
      const int64_t gi = g0 + i;
      if (m[gi] < 0 || n[gi] < 0 || k[gi] < 0 || lda[gi] < k[gi] || ldb[gi] < k[gi] || ldc[gi] < n[gi]) return HB200_ERR_INVALID_ARGUMENT;
      if (m[gi] > 0x7fffff00 || n[gi] > 0x7fffff00 || k[gi] > 0x7fffff00) return HB200_ERR_UNSUPPORTED;
      dg.m[i] = int(m[gi]); dg.n[i] = int(n[gi]); dg.k[i] = int(k[gi]);
      dg.out[i] = out_ptrs[gi]; dg.ldc[i] = ldc[gi];
      if (m[gi] == 0 || n[gi] == 0 || k[gi] == 0) { dg.n[i] = 0; continue; }  // nothing to do (k == 0 leaves out untouched)
      if (!a_ptrs[gi] || !b_ptrs[gi] || !out_ptrs[gi]) return HB200_ERR_INVALID_ARGUMENT;
      if ((k[gi] % 8) != 0 || (lda[gi] % 8) != 0 || (ldb[gi] % 8) != 0) return HB200_ERR_UNSUPPORTED;  // 16-byte row pitch for TMA
      if (reinterpret_cast<uintptr_t>(a_ptrs[gi]) % 16 || reinterpret_cast<uintptr_t>(b_ptrs[gi]) % 16) return HB200_ERR_UNSUPPORTED;
      if (!make_f16_map_pitched(&maps.a[i], a_ptrs[gi], m[gi], k[gi], lda[gi], 128, is_bf16 != 0)) return HB200_ERR_CUDA;
      if (!make_f16_map_pitched(&maps.b[i], b_ptrs[gi], n[gi], k[gi], ldb[gi], kF16BlockN, is_bf16 != 0)) return HB200_ERR_CUDA;
      row_tiles += ceil_div64(m[gi], 128);
      if (n[gi] > max_n) max_n = n[gi];
    }
    if (row_tiles == 0 || max_n == 0) continue;
    if (row_tiles > 0xffffff) return HB200_ERR_UNSUPPORTED;
    // no tile list in this mode: the kernel derives (group, first row) of a row tile from the groups' row counts
    F16Args g{nullptr, 0, 0, 0, nullptr, int(row_tiles), int(ceil_div64(max_n, kF16BlockN)), 0, cnt};
    const int64_t tiles = row_tiles * g.n_tiles;
    const int grid = int(tiles < sms ? tiles : sms);
    if (is_bf16) {
      auto kernel = grouped_gemm_f16_kernel<__nv_bfloat16, true>;
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
      kernel<<<grid, kF16Threads, smem, s>>>(maps.a[0], maps.b[0], maps, dg, g);
    } else {
      auto kernel = grouped_gemm_f16_kernel<__half, true>;
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
      kernel<<<grid, kF16Threads, smem, s>>>(maps.a[0], maps.b[0], maps, dg, g);
    }
    if (launch_status() != HB200_OK) return HB200_ERR_CUDA;
  }
  return HB200_OK;
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
// Wait budget of this translation unit's bounded mbarrier waits (see hb200_set_wait_budget_cycles).
int f16_set_wait_budget(long long cycles) { return sm100::set_wait_budget_cycles(cycles) ? HB200_OK : HB200_ERR_CUDA; }

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
