// Row-wise scaled FP8 matrix multiply for sm_100a (tcgen05 kind::f8f6f4, fp32 accumulate; for int8 operands
// kind::i8 with an int32 accumulator that is converted to fp32 once, after the whole K range is summed):
//   c[m, n] = cast(scale_a[m] * acc[m, n] * scale_b[n]) + bias[n],   acc = a[m, :] . b[:, n]
// a [M, K] row-major, b [K, N] with unit stride along K (the weight stored [N, K]); scales per tensor or per
// row / column; the bias is added after the cast, in the output type.  This is the operator of
// pretuned_kernels/scaled_mm/scaled_mm.py:18-84.
//
// The shapes that operator is tuned on are decode shapes (16 or 64 tokens against weights of 4 to 262 MB), so
// the kernel streams the WEIGHT through the tensor core's M side: a tile is 128 weight rows by up to 256 tokens
// and the accumulator holds c transposed (lane = n, column = m).  One SM streams about 1/148 of the HBM
// bandwidth, so the work must cover the SMs whatever the tile count; three forms, chosen on the host:
//  * cluster form (few tiles): one thread-block cluster of 2, 4 or 8 CTAs per tile, the K range split across
//    them, the partial sums exchanged through distributed shared memory (see the kernel's comment);
//  * whole tiles, one per CTA, when there is nearly one tile per SM;
//  * stream-K otherwise, one CTA per SM: every CTA takes the same number of whole tiles, and the tiles left over
//    are dealt as (tile, K block) units in contiguous ranges of equal length, worked on first.  A tile whose K
//    range is shared has each of its CTAs write an fp32 partial to the workspace; the last to arrive (an acq_rel
//    counter per tile) adds them in K order and finishes the tile.
// In every form partial sums are added in a fixed order: results do not depend on timing.  Large M runs through the
// same kernel, 256 tokens per tile.
//
// CTAs of 192 threads: warp 0 TMA producer (weights 128 x 128 bytes, tokens cols x 128 bytes, 128-byte swizzle,
// no multicast; the first ring of loads goes out during set-up), warp 1 MMA issuer (128 x cols x 32 per
// instruction), warps 2-5 epilogue (scales, cast, bias; 32 x 16 blocks turned round in shared memory so that c
// is written in 16-byte pieces); two accumulators in tensor memory; every wait bounded.
#include "gemm_common.cuh"

#include <mutex>
#include <type_traits>

namespace hb200 {

__device__ int g_device_status_fp8 = 0;


// CTA-pair kernel for prefill shapes (gemm_dense.cu)
int dense_pair_scaled_mm(const void* a, const void* b, void* c, const float* scale_a, const float* scale_b,
                         const void* bias, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                         int scale_a_per_row, int scale_b_per_col, int format, int out_dtype, cudaStream_t stream);

namespace {

using namespace sm100;

constexpr int kFp8Threads = 192;
constexpr int kFp8WBytes = 128 * 128;   // one stage of weights: 128 rows x 128 K-bytes
constexpr int kFp8MaxCols = 256;        // tokens per tile
constexpr int kFp8MaxStages = 10;
constexpr int kFp8CounterBytes = 16384; // arrival counters at the start of the workspace
constexpr int kFp8MaxTiles = kFp8CounterBytes / 4;
constexpr int kFp8MinUnits = 4;         // K blocks per CTA below which more CTAs only add partial sums
constexpr int kPairMinTokens = 384;     // from here on the CTA-pair kernel (activations on the M side) takes over

struct Fp8Args {
  void* out;
  int64_t ldc;
  const float* scale_a;  // [M] or [1]
  const float* scale_b;  // [N] or [1]
  const void* bias;      // [N] in the output type, or nullptr
  float* partials;       // two slots per CTA of [cols][128] fp32
  unsigned int* counters;  // arrivals per tile; zero whenever no call is in flight
  int m, n, k;
  int scale_a_per_row, scale_b_per_col;
  int n_tiles, m_chunks, cols;  // cols = tokens per tile, a multiple of 16
  int num_kb;                   // K blocks of 128 elements per tile
  int whole_tiles;
  int vec_ok;  // 16-byte stores into c are possible
  int cluster;  // CTAs per tile in the cluster form, 0 otherwise
  int stages, stage_bytes;
};

__device__ __forceinline__ void mma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor of kind::f8f6f4: fp32 accumulator (bits 4-5 = 1), operand format at bits 7-9 and 10-12
// (0 = e4m3, 1 = e5m2), both operands K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_f8(int m, int n, int format) {
  return (1u << 4) | (uint32_t(format) << 7) | (uint32_t(format) << 10) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

// The integer form (int8 x int8 -> int32, pretuned_kernels/scaled_mm/scaled_mm.py:53): kind::i8, the accumulator
// holds int32 (bits 4-5 = 2), operand format 1 = signed 8-bit; the same shapes, strides and K per instruction.
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Accumulator words travel as float registers whatever they hold (fp32, or the bits of an int32 in the integer
// form): `wide` turns one into the fp32 value the scales multiply, `add_acc` adds two partial sums of a tile.
__device__ __forceinline__ float wide(float v, bool is_int) { return is_int ? __int2float_rn(__float_as_int(v)) : v; }
__device__ __forceinline__ float add_acc(float a, float b, bool is_int) {
  return is_int ? __int_as_float(__float_as_int(a) + __float_as_int(b)) : a + b;
}

__device__ __forceinline__ void fp8_epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Arrival on a tile's counter: releases what the CTA's threads wrote before the barrier they passed on the way
// here, and acquires what earlier arrivers released, for the threads that pass the next barrier.
__device__ __forceinline__ unsigned int arrive_acq_rel(unsigned int* counter) {
  unsigned int old;
  asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  return old;
}

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
__device__ __forceinline__ float as_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float as_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float as_float(float v) { return v; }

__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

// CLUSTER: the small-problem form.  One tile per thread-block cluster, its K range split over the cluster's CTAs.
// Every CTA owns the tile's columns c with c % CLUSTER == its rank; each CTA stores its fp32 partial of a column into the owner's
// shared memory (distributed shared memory: remote stores, nothing waits on them), and after one cluster
// barrier every owner adds up its columns from local shared memory in rank order.  No workspace, no counters,
// no trip through L2.
// CLUSTER: CTAs per tile (2, 4 or 8) in the cluster form, 0 otherwise.  INT8: int8 operands (format 2), int32 accumulation.
template <typename OutT, int CLUSTER, bool INT8>
__global__ void __launch_bounds__(kFp8Threads, 1)
fp8_scaled_mm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                     const Fp8Args g, const int format) {
  constexpr int ACC = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + g.stages * g.stage_bytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kFp8MaxStages;
  uint64_t* tmem_full_bar = bars + 2 * kFp8MaxStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* fix = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [0] last arriver? [1] first owner [2] last owner
  uint8_t* turn_base = reinterpret_cast<uint8_t*>(bars) + 256;  // 2 KB per epilogue warp
  float* stash = reinterpret_cast<float*>(turn_base + 4 * 2048);  // CLUSTER: [rank][column of mine][128] partials

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = g.stages;
  const int KB = g.num_kb;
  const int total = g.n_tiles * g.m_chunks * KB, grid = int(gridDim.x), cta = int(blockIdx.x);
  // Stream-K form: every CTA first gets the same number of whole tiles (tile cta + i * grid); only the tiles left
  // over are dealt as (tile, K block) ranges, and a CTA works on its share of those first, so that what it does
  // last is a plain tile and the sums of shared tiles are finished while everybody still streams.
  const int tiles_all = g.n_tiles * g.m_chunks;
  const int whole_each = (CLUSTER > 0 || g.whole_tiles) ? 0 : tiles_all / int(gridDim.x);
  const int rest_base = whole_each * int(gridDim.x);  // first tile of the shared remainder
  int u_begin, u_end;
  if constexpr (CLUSTER > 0) {
    const int rank = int(cluster_ctarank()), tile = cta / CLUSTER;
    u_begin = tile * KB + range_start(rank, KB, CLUSTER);
    u_end = tile * KB + range_start(rank + 1, KB, CLUSTER);
  } else {
    // beyond the counters' reach (thousands of tiles) whole tiles are dealt instead: nothing is shared then
    const int rest_total = (tiles_all - rest_base) * KB;
    u_begin = g.whole_tiles ? range_start(cta, total / KB, grid) * KB : range_start(cta, rest_total, grid);
    u_end = g.whole_tiles ? range_start(cta + 1, total / KB, grid) * KB : range_start(cta + 1, rest_total, grid);
  }
  const Segments segs(u_begin, u_end, KB);
  const int rest_total = (tiles_all - rest_base) * KB;  // units of the remainder (ranges above are within it)
  const int work_count = segs.count + whole_each;
  // i-th piece of work of this CTA: the remainder's segments, then the whole tiles
  auto work = [&](int i, int& tile, int& kb0, int& kb1) {
    if (i < segs.count) {
      segs.get(i, tile, kb0, kb1);
      tile += rest_base;
    } else {
      tile = cta + (i - segs.count) * grid;
      kb0 = 0;
      kb1 = KB;
    }
  };
  const int acc_stride = g.cols < 32 ? 32 : g.cols;

  // one stage of (tile, K block): the stage's barrier is told the bytes, both boxes are requested.  The weights do
  // not depend on the kernel before this one on the stream, the tokens may: `part` 1 requests the weights only
  // (and arms the barrier for both), 2 the tokens only, 3 both.
  auto issue = [&](int s, int tile, int kb, int part) {
    const uint32_t bar = smem_u32(&full_bar[s]);
    uint8_t* st = smem + s * g.stage_bytes;
    if (part & 1) {
      mbar_arrive_expect_tx(bar, uint32_t(kFp8WBytes + g.cols * 128));
      tma_load_2d(smem_u32(st), &tmap_w, kb * 128, (tile / g.m_chunks) * 128, bar);
    }
    if (part & 2) tma_load_2d(smem_u32(st + kFp8WBytes), &tmap_x, kb * 128, (tile % g.m_chunks) * g.cols, bar);
  };
  // the first ring of loads, requested before the main loop
  auto first_ring = [&](int part) {
    int it = 0;
    for (int i = 0; i < work_count && it < stages; ++i) {
      int tile, kb0, kb1;
      work(i, tile, kb0, kb1);
      for (int kb = kb0; kb < kb1 && it < stages; ++kb, ++it) issue(it, tile, kb, part);
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < ACC; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    // The ring is empty: the weights of its first round are requested now, while tensor memory is still being set
    // up and (when this kernel was launched as a programmatic dependent) while the kernel before it still runs.
    first_ring(1);
  }
  // two accumulators of acc_stride columns; the allocation is a power of two of at least 32 columns
  uint32_t tmem_cols = 32;
  while (tmem_cols < uint32_t(ACC * acc_stride)) tmem_cols *= 2;
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), tmem_cols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: kernels queued behind this one may be scheduled from now on (every CTA of this
  // grid is resident once all have got here, so they only take what this grid frees), and everything below that
  // touches memory another kernel may have written, or writes memory another kernel may still read, waits for the
  // kernel before this one to complete.  Both are no-ops in an ordinary launch.
  if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) first_ring(2);  // the tokens of the first round
  // CLUSTER: a CTA's shared memory may be written by its peers only once it runs.  Everybody arrives here;
  // the wait for the others sits in front of the first remote store, behind the whole main loop.
  bool peers_running = false;
  if constexpr (CLUSTER > 0) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

  // CLUSTER: what the final reduction needs from global memory is fetched now, long before it is used
  const int c_rank = CLUSTER > 0 ? int(cluster_ctarank()) : 0, c_tile = CLUSTER > 0 ? cta / CLUSTER : 0;
  const int per = CLUSTER > 0 ? g.cols / CLUSTER : 0;
  const int c_r_in = (warp & 3) * 32 + lane;
  const int c_n_idx = (c_tile / g.m_chunks) * 128 + c_r_in, c_m0 = (c_tile % g.m_chunks) * g.cols + c_rank;
  const bool c_active = CLUSTER > 0 && warp >= 2 && c_n_idx < g.n;
  const float c_sb = c_active ? g.scale_b[g.scale_b_per_col ? c_n_idx : 0] : 0.f;
  const float c_bias = (c_active && g.bias) ? as_float(static_cast<const OutT*>(g.bias)[c_n_idx]) : 0.f;
  const float c_sa_all = c_active ? g.scale_a[0] : 0.f;

  if (warp == 0) {
    uint32_t it = 0;
    bool ok = true;
    for (int i = 0; i < work_count && ok; ++i) {
      int tile, kb0, kb1;
      work(i, tile, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        if (it < uint32_t(stages)) continue;  // requested during set-up
        const int s = it % stages;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / stages) & 1) ^ 1, abort_flag)) { ok = false; break; }
        if (elect_one()) issue(s, tile, kb, 3);
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    constexpr bool is_int = INT8;
    const uint32_t idesc = is_int ? make_idesc_i8(128, g.cols) : make_idesc_f8(128, g.cols, format);
    uint32_t it = 0, sc = 0;
    bool ok = true;
    for (int i = 0; i < work_count && ok; ++i, ++sc) {
      int tile, kb0, kb1;
      work(i, tile, kb0, kb1);
      const int acc = sc % ACC;
      if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), ((sc / ACC) & 1) ^ 1, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t tmem_d = tmem_base + acc * acc_stride;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % stages;
        if (!mbar_wait(smem_u32(&full_bar[s]), (it / stages) & 1, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        uint8_t* st = smem + s * g.stage_bytes;
        const uint32_t w_addr = smem_u32(st), x_addr = smem_u32(st + kFp8WBytes);
        const int k_left = g.k - kb * 128;
        const int steps = k_left >= 128 ? 4 : (k_left + 31) / 32;  // K tail: TMA zero-fills past K
        if (elect_one()) {
          for (int a = 0; a < steps; ++a) {
            // 32 K-elements = 32 bytes further along the 128-byte swizzled row
            const uint64_t wdesc = make_smem_desc(w_addr + a * 32, 16, 1024, kSwizzle128B);
            const uint64_t xdesc = make_smem_desc(x_addr + a * 32, 16, 1024, kSwizzle128B);
            if (is_int) mma_i8(tmem_d, wdesc, xdesc, idesc, (kb != kb0 || a != 0) ? 1u : 0u);
            else mma_f8(tmem_d, wdesc, xdesc, idesc, (kb != kb0 || a != 0) ? 1u : 0u);
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
    constexpr bool is_int = INT8;
    const int r_in = quarter * 32 + lane;  // weight row inside the tile = accumulator lane
    OutT* out = static_cast<OutT*>(g.out);
    const OutT* bias = static_cast<const OutT*>(g.bias);
    const float sa_all = g.scale_a[0], sb_all = g.scale_b[0];
    const int first_tile = rest_base + u_begin / KB;
    const int64_t slot_floats = int64_t(g.cols) * 128;
    uint32_t sc = 0;
    bool ok = true;
    for (int i = 0; i < work_count && ok; ++i, ++sc) {
      int tile, kb0, kb1;
      work(i, tile, kb0, kb1);
      const int n_blk = tile / g.m_chunks, m_blk = tile % g.m_chunks;
      const int acc = sc % ACC;
      // this row's scale and bias are fetched before the wait, not after it
      const int n_idx = n_blk * 128 + r_in;
      const bool n_ok = n_idx < g.n;
      const int m0 = m_blk * g.cols;
      const float sb = g.scale_b_per_col ? (n_ok ? g.scale_b[n_idx] : 0.f) : sb_all;
      const float bias_n = (bias && n_ok) ? as_float(bias[n_idx]) : 0.f;
      if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), (sc / ACC) & 1, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * acc_stride;
      const bool whole = kb0 == 0 && kb1 == KB;
      float* slot = g.partials + int64_t(2 * cta + (tile == first_tile ? 0 : 1)) * slot_floats;

      // 16 accumulator columns (tokens m0 + c0 ...) of this thread's weight row.  Where alignment allows the
      // warp's 32 x 16 block is turned round in shared memory and leaves as 16-byte pieces of output rows.
      const bool vec_tile = g.vec_ok && n_blk * 128 + 128 <= g.n;
      auto finalize = [&](const float (&v)[16], int c0) {
        if (vec_tile) {
          constexpr int VEC = 16 / int(sizeof(OutT)), SEGS = 32 / VEC;
          OutT* turn = reinterpret_cast<OutT*>(turn_base + (warp - 2) * 2048);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m_idx = m0 + c0 + j;
            const float sa = g.scale_a_per_row ? (m_idx < g.m ? __ldg(g.scale_a + m_idx) : 0.f) : sa_all;
            OutT o = from_float<OutT>(__fmul_rn(sb, __fmul_rn(sa, wide(v[j], is_int))));
            if (bias) o = from_float<OutT>(__fadd_rn(as_float(o), bias_n));
            turn[j * 32 + lane] = o;
          }
          __syncwarp();
#pragma unroll
          for (int pass = 0; pass < SEGS / 2; ++pass) {
            const int idx = pass * 32 + lane, row = idx / SEGS, seg = idx % SEGS;
            const int m_idx = m0 + c0 + row;
            if (m_idx < g.m) {
              const uint4 val = *reinterpret_cast<const uint4*>(turn + row * 32 + seg * VEC);
              *reinterpret_cast<uint4*>(out + int64_t(m_idx) * g.ldc + n_blk * 128 + quarter * 32 + seg * VEC) = val;
            }
          }
          __syncwarp();
          return;
        }
        if (!n_ok) return;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m_idx = m0 + c0 + j;
          if (m_idx < g.m) {
            const float sa = g.scale_a_per_row ? __ldg(g.scale_a + m_idx) : sa_all;
            OutT o = from_float<OutT>(__fmul_rn(sb, __fmul_rn(sa, wide(v[j], is_int))));
            if (bias) o = from_float<OutT>(__fadd_rn(as_float(o), bias_n));
            out[int64_t(m_idx) * g.ldc + n_idx] = o;
          }
        }
      };

#pragma unroll 1
      for (int c0 = 0; c0 < g.cols; c0 += 16) {
        float v[16];
        {
          uint32_t r0[8], r1[8];
          tmem_ld_32x32b_x8(taddr + c0, r0);
          tmem_ld_32x32b_x8(taddr + c0 + 8, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[j] = __uint_as_float(r0[j]);
            v[8 + j] = __uint_as_float(r1[j]);
          }
        }
        if (c0 + 16 >= g.cols) {  // everything is in registers: hand the accumulator back
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        }
        if constexpr (CLUSTER > 0) {
          if (!peers_running) {
            asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
            peers_running = true;
          }
          // column c belongs to rank c % CLUSTER, which keeps it as its column c / CLUSTER of this rank's block
          const int per = g.cols / CLUSTER, rank = int(cluster_ctarank());
          uint32_t owner_base[CLUSTER];
#pragma unroll
          for (int q = 0; q < CLUSTER; ++q)
            owner_base[q] = map_to_cta(smem_u32(stash + (rank * per + c0 / CLUSTER) * 128 + r_in), uint32_t(q));
#pragma unroll
          for (int j = 0; j < 16; ++j) st_cluster_f32(owner_base[j % CLUSTER] + uint32_t(j / CLUSTER) * 512u, v[j]);
        } else if (whole) {
          finalize(v, c0);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) __stcg(slot + (c0 + j) * 128 + r_in, v[j]);
        }
      }
      if (CLUSTER > 0 || whole) continue;

      // a tile shared with other CTAs: publish the partial, the last arriver finishes the tile
      fp8_epilogue_bar();
      if (r_in == 0) {
        const int rt = tile - rest_base;  // the tile's index in the remainder
        const int c_first = owner_of(rt * KB, rest_total, grid), c_last = owner_of(rt * KB + KB - 1, rest_total, grid);
        const unsigned int seen = arrive_acq_rel(&g.counters[rt]);
        fix[0] = seen + 1u == unsigned(c_last - c_first + 1);
        fix[1] = c_first;
        fix[2] = c_last;
      }
      fp8_epilogue_bar();
      const bool last = fix[0] != 0;
      const int c_first = fix[1], c_last = fix[2];
      fp8_epilogue_bar();  // fix[] may be rewritten by the next shared tile
      if (!last) continue;
      // ascending K: a fixed summation order; four pieces' loads of a whole chunk of columns in flight at a time
      auto reduce = [&](auto width) {
        constexpr int CW = decltype(width)::value;
#pragma unroll 1
        for (int c0 = 0; c0 < g.cols; c0 += CW) {
          float v[CW];
#pragma unroll
          for (int j = 0; j < CW; ++j) v[j] = 0.f;
          for (int c = c_first; c <= c_last; c += 4) {
            float t[4][CW];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int cq = c + q;
              if (cq <= c_last) {
                const int c_tile0 = rest_base + range_start(cq, rest_total, grid) / KB;
                const float* src = g.partials + int64_t(2 * cq + (tile == c_tile0 ? 0 : 1)) * slot_floats;
#pragma unroll
                for (int j = 0; j < CW; ++j) t[q][j] = __ldcg(src + (c0 + j) * 128 + r_in);
              } else {
#pragma unroll
                for (int j = 0; j < CW; ++j) t[q][j] = 0.f;
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
#pragma unroll
              for (int j = 0; j < CW; ++j) v[j] = add_acc(v[j], t[q][j], is_int);
            }
          }
#pragma unroll
          for (int h = 0; h < CW / 16; ++h) finalize(reinterpret_cast<const float(&)[16]>(v[h * 16]), c0 + h * 16);
        }
      };
      if (g.cols % 32 == 0) reduce(std::integral_constant<int, 32>{}); else reduce(std::integral_constant<int, 16>{});
      if (r_in == 0) g.counters[tile - rest_base] = 0u;
    }
  }

  if constexpr (CLUSTER > 0) {
    if (!peers_running) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    if (warp >= 2 && segs.count == 0) {  // no K blocks for this rank: its partials are zero
      for (int c = 0; c < g.cols; ++c)
        st_cluster_f32(map_to_cta(smem_u32(stash + (c_rank * per + c / CLUSTER) * 128 + c_r_in), uint32_t(c % CLUSTER)), 0.f);
    }
    __syncwarp();
    // Every thread of every CTA of the cluster gets here (all waits above are bounded).  The barrier orders the
    // remote stores before the loads below; after it nobody touches another CTA's shared memory again, so a
    // CTA may leave as soon as it has written its columns.
    cluster_sync_all();
    if (c_active) {
      OutT* out = static_cast<OutT*>(g.out) + c_n_idx;
      const bool bias = g.bias != nullptr;
      const float* mine = stash + c_r_in;
#pragma unroll 4
      for (int i = 0; i < per; ++i) {  // my i-th column is the tile's column i * CLUSTER + rank
        float t[CLUSTER];
#pragma unroll
        for (int q = 0; q < CLUSTER; ++q) t[q] = mine[(q * per + i) * 128];
        float v = t[0];
#pragma unroll
        for (int q = 1; q < CLUSTER; ++q) v = add_acc(v, t[q], INT8);  // rank order = ascending K: a fixed summation order
        const int m_idx = c_m0 + i * CLUSTER;
        if (m_idx < g.m) {
          const float sa = g.scale_a_per_row ? __ldg(g.scale_a + m_idx) : c_sa_all;
          OutT o = from_float<OutT>(__fmul_rn(c_sb, __fmul_rn(sa, wide(v, INT8))));
          if (bias) o = from_float<OutT>(__fadd_rn(as_float(o), c_bias));
          out[int64_t(m_idx) * g.ldc] = o;
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicMin(&g_device_status_fp8, HB200_ERR_DEVICE_TIMEOUT);
}

// K-major byte matrix [rows, K] with a row pitch of `pitch` bytes; box = 128 bytes x box_rows, 128-byte swizzle.
bool make_fp8_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t pitch, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(pitch)};
  const cuuint32_t box[2] = {128, cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Fp8Plan {
  int n_tiles, m_chunks, cols, num_kb, stages, stage_bytes, grid, whole_tiles, cluster;
  int64_t workspace_bytes;
};

// How many clusters of `size` CTAs (one CTA per SM) the device runs at the same time; asked once per device and size.
int max_active_clusters(int size) {
  static std::mutex mu;
  static int cached[64][9] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || size < 1 || size > 8) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev][size] == 0) {
    auto kernel = size == 8 ? fp8_scaled_mm_kernel<__nv_bfloat16, 8, false>
                  : size == 4 ? fp8_scaled_mm_kernel<__nv_bfloat16, 4, false> : fp8_scaled_mm_kernel<__nv_bfloat16, 2, false>;
    const size_t smem = 200 * 1024;
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(size) * 64, 1, 1);
    cfg.blockDim = dim3(kFp8Threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = unsigned(size);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess)
      n = 0;
    cached[dev][size] = n > 0 ? n : -1;
  }
  return cached[dev][size] > 0 ? cached[dev][size] : 0;
}

bool make_fp8_plan(int64_t m, int64_t n, int64_t k, int sms, Fp8Plan* out) {
  Fp8Plan p{};
  p.n_tiles = int((n + 127) / 128);
  p.m_chunks = int((m + kFp8MaxCols - 1) / kFp8MaxCols);
  p.cols = m >= kFp8MaxCols ? kFp8MaxCols : int((m + 15) / 16 * 16);
  p.num_kb = int((k + 127) / 128);
  const int64_t tiles = int64_t(p.n_tiles) * p.m_chunks;
  const int64_t total = tiles * p.num_kb;
  if (total > 0x7fffffff) return false;
  p.whole_tiles = tiles > kFp8MaxTiles;
  // one CTA per SM, fewer when that would leave a CTA under a handful of K blocks (but never fewer than tiles)
  int64_t grid = total / kFp8MinUnits;
  if (grid < tiles) grid = tiles;
  if (grid > sms) grid = sms;
  if (grid < 1) grid = 1;
  p.grid = int(grid);
  p.stage_bytes = kFp8WBytes + ((p.cols * 128 + 1023) / 1024) * 1024;
  const int fit = (232448 - 256 - 4 * 2048 - 1024) / p.stage_bytes;
  p.stages = fit > kFp8MaxStages ? kFp8MaxStages : fit;
  // Small problems (a decode GEMM against a weight of a few megabytes) are latency-bound: one cluster per tile.
  p.cluster = 0;
  if (p.m_chunks == 1 && p.cols <= 64) {
    for (int size = 8; size >= 2; size /= 2) {
      if (tiles * size <= sms && p.num_kb >= 2 * size && tiles <= max_active_clusters(size)) { p.cluster = size; break; }
    }
    // A large weight is worth a cluster only if the clusters cover most of the GPU: one SM streams about 1/148
    // of the HBM bandwidth, so idle SMs cost more there than the trip through L2 that stream-K takes.
    if (n * k > (int64_t(32) << 20) && tiles * p.cluster * 4 < int64_t(sms) * 3) p.cluster = 0;
  }
  // Nearly one tile per SM: whole tiles, one per CTA, beat sharing the last few through the workspace.
  if (!p.cluster && tiles <= sms && tiles * 5 >= int64_t(sms) * 3) {
    p.whole_tiles = 1;
    p.grid = int(tiles);
  }
  if (p.cluster) {
    const int per_cta = (p.num_kb + p.cluster - 1) / p.cluster;
    const int fit_with_partial = (232448 - 256 - 4 * 2048 - 1024 - p.cols * 512) / p.stage_bytes;
    if (p.stages > fit_with_partial) p.stages = fit_with_partial;
    if (p.stages > per_cta) p.stages = per_cta;
    p.grid = int(tiles) * p.cluster;
    p.workspace_bytes = 0;
    *out = p;
    return true;
  }
  // tiles are shared between CTAs only when the ranges do not end on tile boundaries
  // stream-K: every CTA takes tiles / grid whole tiles, the rest is dealt in (tile, K block) ranges
  const int64_t rest_total = (tiles >= p.grid ? tiles % p.grid : tiles) * p.num_kb;
  const bool shared = !p.whole_tiles && rest_total > 0 &&
                      ((rest_total % p.grid) != 0 || ((rest_total / p.grid) % p.num_kb) != 0);
  p.workspace_bytes = shared ? kFp8CounterBytes + int64_t(2) * p.grid * p.cols * 128 * 4 : 0;
  *out = p;
  return true;
}

int device_sms() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

template <typename OutT, bool INT8>
int launch_fp8_kind(const CUtensorMap& tw, const CUtensorMap& tx, const Fp8Args& g, const Fp8Plan& p, int format,
                    cudaStream_t s) {
  if (p.cluster) {
    auto kernel = p.cluster == 8 ? fp8_scaled_mm_kernel<OutT, 8, INT8>
                  : p.cluster == 4 ? fp8_scaled_mm_kernel<OutT, 4, INT8> : fp8_scaled_mm_kernel<OutT, 2, INT8>;
    const size_t smem = size_t(p.stages) * p.stage_bytes + 256 + 4 * 2048 + size_t(p.cols) * 512 + 1024;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(p.grid), 1, 1);
    cfg.blockDim = dim3(kFp8Threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = unsigned(p.cluster);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (cudaLaunchKernelEx(&cfg, kernel, tw, tx, g, format) != cudaSuccess) return HB200_ERR_CUDA;
    return HB200_OK;
  }
  // launched as a programmatic dependent of whatever precedes it on the stream: resident early, its first weights
  // on their way, waiting (griddepcontrol.wait) for that kernel's completion before anything else
  auto kernel = fp8_scaled_mm_kernel<OutT, 0, INT8>;
  const size_t smem = size_t(p.stages) * p.stage_bytes + 256 + 4 * 2048 + 1024;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return HB200_ERR_CUDA;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(p.grid), 1, 1);
  cfg.blockDim = dim3(kFp8Threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, tw, tx, g, format) != cudaSuccess) return HB200_ERR_CUDA;
  return HB200_OK;
}

template <typename OutT>
int launch_fp8(const CUtensorMap& tw, const CUtensorMap& tx, const Fp8Args& g, const Fp8Plan& p, int format,
               cudaStream_t s) {
  return format == 2 ? launch_fp8_kind<OutT, true>(tw, tx, g, p, format, s)
                     : launch_fp8_kind<OutT, false>(tw, tx, g, p, format, s);
}

}  // namespace
}  // namespace hb200

extern "C" int64_t hb200_fp8_scaled_mm_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  using namespace hb200;
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  Fp8Plan p;
  return make_fp8_plan(m, n, k, device_sms(), &p) ? p.workspace_bytes : 0;
}

extern "C" int hb200_fp8_scaled_mm(const void* a, const void* b, void* c, const float* scale_a, const float* scale_b,
                                   const void* bias, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                                   int64_t ldc, int scale_a_per_row, int scale_b_per_col, int fp8_format,
                                   int out_dtype, void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace hb200;
  if (!a || !b || !c || !scale_a || !scale_b) return HB200_ERR_INVALID_ARGUMENT;
  if (m <= 0 || n <= 0 || k <= 0 || lda < k || ldb < k || ldc < n) return HB200_ERR_INVALID_ARGUMENT;
  if (fp8_format < 0 || fp8_format > 2) return HB200_ERR_INVALID_ARGUMENT;
  if (out_dtype < 0 || out_dtype > 2) return HB200_ERR_INVALID_ARGUMENT;
  // TMA: 16-byte aligned bases and row pitches
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(b) % 16 || (lda % 16) != 0 || (ldb % 16) != 0)
    return HB200_ERR_UNSUPPORTED;
  if (m > 0x7fffff00 || n > 0x7fffff00 || k > 0x7fffff00) return HB200_ERR_UNSUPPORTED;
  // prefill shapes: 256 x 256 tiles on CTA pairs, activations on the M side (no workspace)
  if (m >= kPairMinTokens) {
    const int rc = dense_pair_scaled_mm(a, b, c, scale_a, scale_b, bias, m, n, k, lda, ldb, ldc, scale_a_per_row,
                                        scale_b_per_col, fp8_format, out_dtype, static_cast<cudaStream_t>(stream));
    if (rc != HB200_ERR_UNSUPPORTED) return rc;
  }
  Fp8Plan p;
  if (!make_fp8_plan(m, n, k, device_sms(), &p)) return HB200_ERR_UNSUPPORTED;
  if (p.workspace_bytes > 0) {
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 16) return HB200_ERR_WORKSPACE;
    if (workspace_bytes < p.workspace_bytes) return HB200_ERR_WORKSPACE;
  }
  CUtensorMap tw, tx;
  if (!make_fp8_map(&tw, b, n, k, ldb, 128)) return HB200_ERR_CUDA;
  if (!make_fp8_map(&tx, a, m, k, lda, p.cols)) return HB200_ERR_CUDA;
  Fp8Args g{};
  g.out = c;
  g.ldc = ldc;
  g.scale_a = scale_a;
  g.scale_b = scale_b;
  g.bias = bias;
  g.counters = static_cast<unsigned int*>(workspace);
  g.partials = p.workspace_bytes > 0
                   ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kFp8CounterBytes) : nullptr;
  g.m = int(m);
  g.n = int(n);
  g.k = int(k);
  g.scale_a_per_row = scale_a_per_row != 0;
  g.scale_b_per_col = scale_b_per_col != 0;
  g.n_tiles = p.n_tiles;
  g.m_chunks = p.m_chunks;
  g.cols = p.cols;
  g.num_kb = p.num_kb;
  g.whole_tiles = p.whole_tiles;
  g.cluster = p.cluster;
  g.vec_ok = reinterpret_cast<uintptr_t>(c) % 16 == 0 && (ldc * (out_dtype == 2 ? 4 : 2)) % 16 == 0;
  g.stages = p.stages;
  g.stage_bytes = p.stage_bytes;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == 0) return launch_fp8<__nv_bfloat16>(tw, tx, g, p, fp8_format, s);
  if (out_dtype == 1) return launch_fp8<__half>(tw, tx, g, p, fp8_format, s);
  return launch_fp8<float>(tw, tx, g, p, fp8_format, s);
}

namespace hb200 {
// Wait budget of this translation unit's bounded mbarrier waits (see hb200_set_wait_budget_cycles).
int fp8_set_wait_budget(long long cycles) { return sm100::set_wait_budget_cycles(cycles) ? HB200_OK : HB200_ERR_CUDA; }

// Sticky status of this translation unit's kernels, folded into hb200_device_status().
int fp8_device_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status_fp8, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  if (reset && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_device_status_fp8, &zero, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  }
  return v;
}
}  // namespace hb200
