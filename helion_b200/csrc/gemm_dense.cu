// Dense GEMM on CTA pairs (tcgen05 cta_group::2; kind::f8f6f4, kind::i8 or kind::f16) with two accumulators in
// tensor memory, and its two fused compute + collective forms over peer memory.
//
//   c[m, n] = cast(scale_b[n] * (scale_a[m] * acc[m, n])) + bias[n],   acc = a[m, :] . b[n, :]
//
// Serves the prefill shapes of scaled_mm (pretuned_kernels/scaled_mm/scaled_mm.py:18-84; FP8 and int8) and, in
// bf16 / fp16 with unit scales, the GEMMs of the reference's distributed examples.  Two CTAs on neighbouring SMs own
// one 256 x 256 output tile: CTA r of the pair holds rows [128 r, 128 r + 128) of the a tile and of the b tile, and
// the leader issues 256 x 256 MMAs over 32 bytes of K that read both halves: per 128 bytes of K every SM pulls
// 16 KB of a and 16 KB of b from L2 for 128 x 256 outputs.  The 512 columns of tensor memory hold two accumulators,
// so the epilogue of a tile (scales, cast, bias, staged through shared memory into TMA stores) runs beside the next
// tile's MMAs.  No load is multicast; every wait is bounded; the kernel ends with a hardware cluster barrier so
// neither CTA exits while its peer may still touch its shared memory or barriers.
//
// MODE 1, all-gather + matmul (examples/distributed/all_gather_matmul.py:36-141): every rank holds rows_local rows
// of a; c = gathered a . b.  The two warps of every CTA that have no role in the GEMM do the gather: each copies its
// slice of every chunk of this rank's shard into every peer's gather buffer (16-byte loads from local memory, 16-byte
// stores to peer memory, several in flight per lane; peers in ring order) and, when its stores of a chunk to a
// destination are done, adds one arrival to that chunk's progress counter there (a system-scope release
// reduction); the local copy of the shard comes last.  Spread over all SMs the copy needs no SM of its own and is
// not held back by what a single SM can keep in flight towards a peer.  The GEMM takes the tiles in the order the
// chunks arrive (own rows first, read from the shard itself, then the ring backwards); before the first load of a
// peer chunk's rows the producer warp waits (system-scope acquire, bounded) until the counter shows all arrivals of
// this call.  Counters only grow: call number s (1, 2, ...) expects s arrivals from every pushing warp, so nothing is
// reset between calls; the caller orders calls with a barrier, since a rank may not overwrite a peer's gather buffer
// while the peer still reads it.  A pushing warp never waits for anything remote, and all CTAs of the grid are
// resident at once (one per SM), so ranks cannot deadlock one another.
//
// MODE 2, matmul + reduce-scatter (examples/distributed/matmul_reduce_scatter.py:37-115): every rank holds a K
// shard; the tile rows [d R, d R + R) of its partial product, rounded to the output type as the reference rounds
// them, go straight from the epilogue into slot `rank` of rank d's receive buffer [world, R, N] with TMA stores
// (remote ranks first, the own slot last).  A barrier kernel and hb200_reduce_slots (sum over the slots in rank
// order, fp32) finish the reduce-scatter; nothing is ever loaded from peer memory.
#include "gemm_common.cuh"

#include <type_traits>

namespace hb200 {

__device__ int g_device_status_dense = 0;
__device__ float g_unit_scale = 1.0f;

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
  // MODE 1 (all-gather + matmul)
  const uint8_t* shard;  // this rank's rows of a, contiguous [rows_local, k_bytes]
  uint8_t* gather[8];    // every rank's gather buffer [world * rows_local, k_bytes], contiguous, as mapped here
  uint32_t* progress[8]; // every rank's arrival counters [world * splits]
  int rank, world, splits, rows_local;
  uint32_t arrivals;     // what a counter shows once a chunk of this call has landed
  int push;              // the kernel's own warps do the gather (else somebody else fills the buffer and the counters)
  // MODE 2 (matmul + reduce-scatter)
  int rows_per_dest;     // R: rows [d R, d R + R) of the product belong to rank d
};

constexpr int kPushUnroll = 8;  // 16-byte loads a lane of a pushing warp keeps in flight

struct OutMaps {
  // MODE 2: rank d's receive buffer [world * R, N]; otherwise dest[0] is c.  MODE 1: dest[1] maps this rank's shard
  // of a (an operand, not an output: the slot is free there).
  CUtensorMap dest[8];
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

__device__ __forceinline__ void mma_pair_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Tile order: bands of `band` row tiles; inside a band the row tile runs fastest, then the column tile.  The 74
// pairs that work at the same time then share a few row tiles of a and a few column tiles of b, which stay in L2.
__device__ __forceinline__ void decode_banded(int tile, int m_tiles, int n_tiles, int band, int& m_blk, int& n_blk) {
  const int per_band = band * n_tiles;
  const int b = tile / per_band, r = tile - b * per_band;
  const int rows_here = min(band, m_tiles - b * band);
  n_blk = r / rows_here;
  m_blk = b * band + (r - n_blk * rows_here);
}

// MODE 1: the row tiles of one source rank after the other, in the order their chunks arrive (own rows, then the
// ring backwards: rank r pushes to r + 1 first, so what arrives first here comes from rank - 1).  MODE 2: the row
// tiles of one destination rank after the other, the next rank's first, the own rows last.
template <int MODE>
__device__ __forceinline__ void decode_tile(const Args& g, int tile, int& m_blk, int& n_blk) {
  if constexpr (MODE == 0) {
    decode_banded(tile, g.m_tiles, g.n_tiles, g.band, m_blk, n_blk);
  } else {
    const int per_rank = g.m_tiles / g.world;  // row tiles per source (MODE 1) or destination (MODE 2) rank
    const int pos = tile / (per_rank * g.n_tiles), r = tile - pos * per_rank * g.n_tiles;
    const int who = MODE == 1 ? (g.rank - pos + g.world) % g.world : (g.rank + 1 + pos) % g.world;
    int m_local;
    decode_banded(r, per_rank, g.n_tiles, min(g.band, per_rank), m_local, n_blk);
    m_blk = who * per_rank + m_local;
  }
}

template <typename T> __device__ __forceinline__ T cast_out(float v);
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(float v) { return v; }

// format: 0 = e4m3, 1 = e5m2, 2 = int8 (int32 accumulator, converted to fp32 once), 3 = fp16, 4 = bf16
template <typename OutT, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
dense_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ OutMaps omaps, const Args g, const int format) {
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
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
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
    int seen_chunk = -1;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int m_blk, n_blk;
      decode_tile<MODE>(g, tile, m_blk, n_blk);
      const int a_row = m_blk * kTile + int(rank) * 128;
      const int b_row = n_blk * kTile + int(rank) * 128;
      if constexpr (MODE == 1) {
        // rows of chunk (source rank, split): wait until every push CTA of the source has delivered its part
        const int rows_chunk = g.rows_local / g.splits;
        const int chunk = (m_blk * kTile) / rows_chunk;  // = source * splits + split
        if (chunk / g.splits != g.rank && chunk != seen_chunk) {
          const uint32_t* counter = g.progress[g.rank] + chunk;
          const long long t0 = clock64();
          while (int32_t(ld_acquire_sys(counter) - g.arrivals) < 0) {
            if (*abort_flag || clock64() - t0 > *const_cast<volatile long long*>(&g_wait_budget_cycles)) {
              *abort_flag = 1;
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_proxy_async_all();  // the TMA loads below read what the acquire made visible
          seen_chunk = chunk;
        }
      }
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kStages;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
        uint8_t* st = smem + s * kStageBytes;
        const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);  // always the leader's barrier
        if (elect_one()) {
          if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[s]), 2 * kStageBytes);
          if (MODE == 1 && a_row / g.rows_local == g.rank)  // own rows: straight from the shard
            tma_load_2d_pair(smem_u32(st), &omaps.dest[1], kb * 128, a_row - g.rank * g.rows_local, bar);
          else
            tma_load_2d_pair(smem_u32(st), &tmap_a, kb * 128, a_row, bar);
          tma_load_2d_pair(smem_u32(st + kHalfBytes), &tmap_b, kb * 128, b_row, bar);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (leader only)
    if (leader) {
      const bool is_int = format == 2, is_f16 = format >= 3;
      // fp32 (or int32) accumulator at bits 4-5, operand formats at bits 7-9 and 10-12 (kind::f8f6f4: 0 e4m3, 1 e5m2;
      // kind::i8: 1 signed; kind::f16: 0 fp16, 1 bf16), N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t fmt = is_f16 ? uint32_t(format - 3) : uint32_t(format);
      const uint32_t idesc = (is_int ? ((2u << 4) | (1u << 7) | (1u << 10)) : ((1u << 4) | (fmt << 7) | (fmt << 10))) |
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
              else if (is_f16) mma_pair_f16(tmem_d, adesc, bdesc, idesc, (kb | a) != 0 ? 1u : 0u);
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
  } else if (warp < 4) {
    // ------------------------------------------------------------ all-gather push (warps 2 and 3 of every CTA)
    if (MODE == 1 && g.push) {
      const int pw = int(blockIdx.x) * 2 + (warp - 2), n_pw = int(gridDim.x) * 2;
      const int64_t chunk_bytes = int64_t(g.rows_local / g.splits) * g.k_bytes;  // a multiple of 16
      const int64_t part0 = (chunk_bytes / 16 * pw / n_pw) * 16, part1 = (chunk_bytes / 16 * (pw + 1) / n_pw) * 16;
      auto copy_part = [&](const uint8_t* src, uint8_t* dst) {
        for (int64_t off = part0 + lane * 16; off < part1; off += 32 * 16 * kPushUnroll) {
          uint4 v[kPushUnroll];
#pragma unroll
          for (int u = 0; u < kPushUnroll; ++u) {
            const int64_t o = off + int64_t(u) * 32 * 16;
            if (o < part1)
              asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + o));
          }
#pragma unroll
          for (int u = 0; u < kPushUnroll; ++u) {
            const int64_t o = off + int64_t(u) * 32 * 16;
            if (o < part1)
              asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + o), "r"(v[u].x), "r"(v[u].y), "r"(v[u].z), "r"(v[u].w) : "memory");
          }
        }
      };
      const int64_t my_rows_off = int64_t(g.rank) * g.rows_local * g.k_bytes;
      for (int c = 0; c < g.splits; ++c) {
        for (int step = 1; step < g.world; ++step) {
          const int d = (g.rank + step) % g.world;  // the ring, the next rank first
          copy_part(g.shard + int64_t(c) * chunk_bytes, g.gather[d] + my_rows_off + int64_t(c) * chunk_bytes);
          __threadfence_system();  // every lane's stores, before the arrival that lane 0 publishes
          __syncwarp();
          if (lane == 0) red_release_sys_add(g.progress[d] + g.rank * g.splits + c, 1u);
        }
      }
      // this rank's own copy of its rows comes last: its tiles read the shard itself
      for (int c = 0; c < g.splits; ++c)
        copy_part(g.shard + int64_t(c) * chunk_bytes, g.gather[g.rank] + my_rows_off + int64_t(c) * chunk_bytes);
    }
  } else {
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
      decode_tile<MODE>(g, tile, m_blk, n_blk);
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
          o[j] = cast_out<OutT>(__fmul_rn(sb, __fmul_rn(sa, v)));  // no contraction with the bias add below
          if (bias != nullptr) o[j] = cast_out<OutT>(__fadd_rn(widen(o[j]), __shfl_sync(0xffffffffu, bias_l[h], j)));
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
            if constexpr (MODE == 2) {
              // slot `rank` of the receive buffer of the rank that owns these rows
              const int d = row0 / g.rows_per_dest;
              tma_store_2d(&omaps.dest[d], col + h * 32, g.rank * g.rows_per_dest + (row0 - d * g.rows_per_dest), smem_u32(box));
            } else {
              tma_store_2d(&omaps.dest[0], col + h * 32, row0, smem_u32(box));  // rows and columns past the edge are clipped
            }
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
      // MODE 2: peers read the slots right after the barrier kernel that follows: wait for the writes themselves
      if (lane == 0) {
        if constexpr (MODE == 2) bulk_wait_group0(); else bulk_wait_group_read0();
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer is done with this CTA's shared memory, barriers and tensor memory
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicMin(&g_device_status_dense, HB200_ERR_DEVICE_TIMEOUT);
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

int device_sms() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

const float* unit_scale() {
  void* p = nullptr;
  return cudaGetSymbolAddress(&p, g_unit_scale) == cudaSuccess ? static_cast<const float*>(p) : nullptr;
}

template <typename OutT, int MODE>
int launch_kernel(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& om, const Args& g, int format, int pairs,
                  cudaStream_t stream) {
  auto kernel = dense_pair_kernel<OutT, MODE>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)) != cudaSuccess)
    return HB200_ERR_CUDA;
  kernel<<<2 * pairs, kThreads, kSmemBytes, stream>>>(ta, tb, om, g, format);
  return launch_status();
}

void fill_shape(Args& g, int64_t m, int64_t n, int64_t k_bytes) {
  g.m = int(m);
  g.n = int(n);
  g.k_bytes = int(k_bytes);
  g.m_tiles = int((m + kTile - 1) / kTile);
  g.n_tiles = int((n + kTile - 1) / kTile);
  g.band = 16;
}

}  // namespace dense_pair

// scaled_mm on CTA pairs.  Returns HB200_ERR_UNSUPPORTED for what the kernel does not take (the caller then uses
// the decode kernel).  k counts bytes of K (= elements for the 8-bit formats).
int dense_pair_scaled_mm(const void* a, const void* b, void* c, const float* scale_a, const float* scale_b,
                         const void* bias, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                         int scale_a_per_row, int scale_b_per_col, int format, int out_dtype, cudaStream_t stream) {
  using namespace dense_pair;
  if (m < 256 || n < 256) return HB200_ERR_UNSUPPORTED;
  if (out_dtype != 2 && ((ldc % 8) != 0 || reinterpret_cast<uintptr_t>(c) % 16)) return HB200_ERR_UNSUPPORTED;
  CUtensorMap ta, tb;
  OutMaps om{};
  if (!make_byte_map(&ta, a, m, k, lda) || !make_byte_map(&tb, b, n, k, ldb)) return HB200_ERR_CUDA;
  if (out_dtype != 2 && !make_output_map16(&om.dest[0], c, m, n, ldc, out_dtype == 0)) return HB200_ERR_CUDA;
  Args g{};
  g.out = c;
  g.ldc = ldc;
  g.scale_a = scale_a;
  g.scale_b = scale_b;
  g.bias = bias;
  g.scale_a_per_row = scale_a_per_row != 0;
  g.scale_b_per_col = scale_b_per_col != 0;
  fill_shape(g, m, n, k);
  const int sms = device_sms(), tiles = g.m_tiles * g.n_tiles;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  if (out_dtype == 0) return launch_kernel<__nv_bfloat16, 0>(ta, tb, om, g, format, pairs, stream);
  if (out_dtype == 1) return launch_kernel<__half, 0>(ta, tb, om, g, format, pairs, stream);
  return launch_kernel<float, 0>(ta, tb, om, g, format, pairs, stream);
}

int dense_set_wait_budget(long long cycles) { return sm100::set_wait_budget_cycles(cycles) ? HB200_OK : HB200_ERR_CUDA; }

int dense_device_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status_dense, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  if (reset && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_device_status_dense, &zero, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  }
  return v;
}

namespace {

// out[r, c] = cast(sum over slots s, ascending, of fp32(slots[s, r, c])): the second half of the reduce-scatter
template <typename T>
__global__ void __launch_bounds__(256)
reduce_slots_kernel(const T* __restrict__ slots, T* __restrict__ out, int world, int64_t rows, int64_t cols, int64_t ld_out) {
  const int64_t vecs = rows * cols / 8, slot_vecs = vecs;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += int64_t(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < world; ++s) {
      const uint4 v = reinterpret_cast<const uint4*>(slots)[int64_t(s) * slot_vecs + i];
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += dense_pair::widen(e[j]);
    }
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = dense_pair::cast_out<T>(acc[j]);
    const int64_t r = (i * 8) / cols, c = i * 8 - r * cols;
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = *reinterpret_cast<const uint4*>(o);
  }
}

}  // namespace
}  // namespace hb200

extern "C" int hb200_dense_matmul(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int64_t lda,
                                  int64_t ldb, int64_t ldc, int is_bf16, void* stream) {
  using namespace hb200;
  if (!a || !b || !c || m <= 0 || n <= 0 || k <= 0 || lda < k || ldb < k || ldc < n) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(b) % 16 || (lda % 8) != 0 || (ldb % 8) != 0)
    return HB200_ERR_UNSUPPORTED;
  if (m > 0x3fffff00 || n > 0x3fffff00 || k > 0x3fffff00) return HB200_ERR_UNSUPPORTED;
  const float* one = dense_pair::unit_scale();
  if (!one) return HB200_ERR_CUDA;
  return dense_pair_scaled_mm(a, b, c, one, one, nullptr, m, n, 2 * k, 2 * lda, 2 * ldb, ldc, 0, 0, is_bf16 ? 4 : 3,
                              is_bf16 ? 0 : 1, static_cast<cudaStream_t>(stream));
}

extern "C" int hb200_ag_matmul(const void* a_shard, void* const* gather_ptrs, void* const* progress_ptrs, const void* b,
                               void* c, int64_t rows_local, int64_t n, int64_t k, int64_t ldb, int64_t ldc, int64_t world,
                               int64_t rank, int64_t splits, uint32_t call_number, int push, int is_bf16, void* stream) {
  using namespace hb200;
  using namespace hb200::dense_pair;
  if (!a_shard || !gather_ptrs || !progress_ptrs || !b || !c) return HB200_ERR_INVALID_ARGUMENT;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || splits < 1 || rows_local <= 0 || n <= 0 || k <= 0 ||
      ldb < k || ldc < n || call_number == 0)
    return HB200_ERR_INVALID_ARGUMENT;
  // a pair tile lies inside one chunk; rows move as 16-byte pieces; the output goes out through TMA stores
  if ((rows_local % splits) != 0 || ((rows_local / splits) % 256) != 0 || (k % 8) != 0 || (ldb % 8) != 0 ||
      (ldc % 8) != 0 || n < 256 || reinterpret_cast<uintptr_t>(a_shard) % 16 || reinterpret_cast<uintptr_t>(b) % 16 ||
      reinterpret_cast<uintptr_t>(c) % 16)
    return HB200_ERR_UNSUPPORTED;
  const int64_t m = rows_local * world;
  if (m > 0x3fffff00 || n > 0x3fffff00 || k > 0x3fffff00 || world * splits > 4096) return HB200_ERR_UNSUPPORTED;
  const int sms = device_sms();
  Args g{};
  for (int i = 0; i < world; ++i) {
    if (!push && i != rank) continue;  // only this rank's own buffer and counters are touched
    if (!gather_ptrs[i] || !progress_ptrs[i] || reinterpret_cast<uintptr_t>(gather_ptrs[i]) % 16 ||
        reinterpret_cast<uintptr_t>(progress_ptrs[i]) % 4)
      return HB200_ERR_INVALID_ARGUMENT;
    g.gather[i] = static_cast<uint8_t*>(gather_ptrs[i]);
    g.progress[i] = static_cast<uint32_t*>(progress_ptrs[i]);
  }
  const float* one = unit_scale();
  if (!one) return HB200_ERR_CUDA;
  CUtensorMap ta, tb;
  OutMaps om{};
  if (!make_byte_map(&ta, gather_ptrs[rank], m, 2 * k, 2 * k) || !make_byte_map(&tb, b, n, 2 * k, 2 * ldb)) return HB200_ERR_CUDA;
  if (!make_output_map16(&om.dest[0], c, m, n, ldc, is_bf16 != 0)) return HB200_ERR_CUDA;
  if (!make_byte_map(&om.dest[1], a_shard, rows_local, 2 * k, 2 * k)) return HB200_ERR_CUDA;
  g.out = c;
  g.ldc = ldc;
  g.scale_a = one;
  g.scale_b = one;
  fill_shape(g, m, n, 2 * k);
  g.shard = static_cast<const uint8_t*>(a_shard);
  g.rank = int(rank);
  g.world = int(world);
  g.splits = int(splits);
  g.rows_local = int(rows_local);
  const int tiles = g.m_tiles * g.n_tiles;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  g.push = push != 0;
  // pushed by the kernels: two pushing warps in each of the 2 * pairs CTAs, on every rank alike, one arrival each per
  // call; filled from outside: whoever fills a chunk then writes the call number into its counter
  g.arrivals = push ? uint32_t(4 * pairs) * call_number : call_number;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int format = is_bf16 ? 4 : 3;
  if (is_bf16) return launch_kernel<__nv_bfloat16, 1>(ta, tb, om, g, format, pairs, s);
  return launch_kernel<__half, 1>(ta, tb, om, g, format, pairs, s);
}

extern "C" int hb200_matmul_rs(const void* a, const void* b, void* const* recv_ptrs, int64_t m, int64_t n, int64_t k,
                               int64_t lda, int64_t ldb, int64_t world, int64_t rank, int is_bf16, void* stream) {
  using namespace hb200;
  using namespace hb200::dense_pair;
  if (!a || !b || !recv_ptrs || world < 1 || world > 8 || rank < 0 || rank >= world || m <= 0 || n <= 0 || k <= 0 ||
      lda < k || ldb < k)
    return HB200_ERR_INVALID_ARGUMENT;
  if ((m % (256 * world)) != 0 || (n % 8) != 0 || n < 256 || (lda % 8) != 0 || (ldb % 8) != 0 ||
      reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(b) % 16)
    return HB200_ERR_UNSUPPORTED;
  if (m > 0x3fffff00 || n > 0x3fffff00 || k > 0x3fffff00) return HB200_ERR_UNSUPPORTED;
  const float* one = unit_scale();
  if (!one) return HB200_ERR_CUDA;
  CUtensorMap ta, tb;
  OutMaps om{};
  if (!make_byte_map(&ta, a, m, 2 * k, 2 * lda) || !make_byte_map(&tb, b, n, 2 * k, 2 * ldb)) return HB200_ERR_CUDA;
  for (int i = 0; i < world; ++i) {
    if (!recv_ptrs[i] || reinterpret_cast<uintptr_t>(recv_ptrs[i]) % 16) return HB200_ERR_INVALID_ARGUMENT;
    if (!make_output_map16(&om.dest[i], recv_ptrs[i], m, n, n, is_bf16 != 0)) return HB200_ERR_CUDA;
  }
  Args g{};
  g.out = recv_ptrs[rank];
  g.ldc = n;
  g.scale_a = one;
  g.scale_b = one;
  fill_shape(g, m, n, 2 * k);
  g.rank = int(rank);
  g.world = int(world);
  g.rows_per_dest = int(m / world);
  const int sms = device_sms(), tiles = g.m_tiles * g.n_tiles;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16) return launch_kernel<__nv_bfloat16, 2>(ta, tb, om, g, 4, pairs, s);
  return launch_kernel<__half, 2>(ta, tb, om, g, 3, pairs, s);
}

extern "C" int hb200_reduce_slots(const void* slots, void* out, int64_t world, int64_t rows, int64_t cols, int64_t ld_out,
                                  int is_bf16, void* stream) {
  using namespace hb200;
  if (!slots || !out || world < 1 || world > 8 || rows < 0 || cols < 0 || ld_out < cols) return HB200_ERR_INVALID_ARGUMENT;
  if ((cols % 8) != 0 || (ld_out % 8) != 0 || reinterpret_cast<uintptr_t>(slots) % 16 || reinterpret_cast<uintptr_t>(out) % 16)
    return HB200_ERR_UNSUPPORTED;
  const int64_t vecs = rows * cols / 8;
  if (vecs == 0) return HB200_OK;
  const int64_t need = (vecs + 255) / 256;
  const int grid = int(need < 1184 ? need : 1184);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    reduce_slots_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(slots),
                                                           static_cast<__nv_bfloat16*>(out), int(world), rows, cols, ld_out);
  else
    reduce_slots_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(slots), static_cast<__half*>(out),
                                                    int(world), rows, cols, ld_out);
  return launch_status();
}
