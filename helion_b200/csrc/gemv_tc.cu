// Tensor-core NVFP4 GEMV / decode-batch skinny GEMM for sm_100a.
//
// The SIMT GEMV has to decode every weight byte (one cvt.rn.f16x2.e2m1x2 per byte, a 16-lane pipe), which
// caps it well below HBM bandwidth.  tcgen05.mma.kind::mxf4nvf4 consumes the packed codes and the e4m3
// block scales as they lie in memory, so here the weights are never decoded by a thread: they ride the M
// side of the MMA (128 weight rows per tile, TMA straight from the K-major weight into 128-byte swizzled
// shared memory, scale atoms copied to tensor memory), and the activations ride the N side.
//
// Activations are bf16 in the reference operator, and the tensor core wants e2m1 on both sides.  Each
// activation row is therefore expanded into TERMS NVFP4 rows whose sum reproduces it: term t quantises
// the residual left by terms 0..t-1 with 16-element e4m3 block scales and a power-of-two global factor
// (so every term dequantises exactly in fp32 and the residual is exact).  A term removes at least a
// factor of about six from the block's residual; four terms leave |error| < 1e-3 of the block maximum,
// far below the bf16 rounding of the output (4e-3) -- the GPU tests bound the output error against the
// fp32 reference.  The columns of one MMA are the batch x TERMS term rows; the epilogue multiplies each
// column by its term's global factor, sums the terms and writes bf16.  With activations that already are
// NVFP4 (the fp4in operator) TERMS is 1 and nothing is approximated.
//
// Work split ("stream-K"): the (row tile, 256-element K block) pairs are numbered tile-major and cut into
// one contiguous range per CTA, so every SM streams the same number of weight bytes whatever the shape.
// A CTA that owns a whole tile writes it out itself.  A tile cut between CTAs is finished by whichever of
// them arrives last: every owner stores its fp32 partial to its own workspace slot, fences, and bumps the
// tile's arrival counter; the last one adds the partials in K order (a fixed order: results do not depend
// on timing) and resets the counter.  Nobody waits for anybody.
//
// Warp roles as in the block-scaled GEMM: 0 TMA producer, 1 MMA issuer, 2 scale copier, 4-7 epilogue.
// Every mbarrier wait is bounded; a timeout raises the sticky device status instead of hanging.
#include "common.cuh"
#include "tcgen05.cuh"
#include "gemm_common.cuh"

#include <mutex>

namespace hb200 {

__device__ int g_device_status_gemv_tc = 0;

namespace {

using namespace sm100;

constexpr int kTcThreads = 256;
constexpr int kTcTmemCols = 512;
constexpr int kExpandThreads = 256;  // one 16-element block per thread
constexpr int kMaxRowTiles = 4096;   // arrival counters reserved in the workspace: N <= 524288

struct TcArgs {
  const uint8_t* sfa;      // swizzled weight scales, logical [N, K/16]
  const uint8_t* sfb;      // swizzled scales of the activation terms: one 128-row tile, [cols, K/16]
  const float* col_scale;  // fp32 factor per MMA column (term), nullptr = 1
  float* partials;         // two slots per CTA of [NCOLS][128] fp32
  unsigned int* counters;  // arrivals per 128-row tile; zero whenever no call is in flight
  OutSpec out;             // [batch, n] bf16 (one buffer, or one per tensor-parallel rank)
  int n, k, batch;
  int row_tiles, num_kb;   // 128-row tiles; 256-element K blocks per tile
  float alpha;
};

template <int NCOLS>
struct TcLayout {
  static constexpr int kABytes = kBlockM * kBlockKBytes;   // 16 KB of weights
  static constexpr int kBBytes = NCOLS * kBlockKBytes;     // the activation terms of the same K block
  static constexpr int kSfBytes = kAtomsPerStage * kAtomBytes;
  static constexpr int kBOff = kABytes;
  static constexpr int kSfaOff = kBOff + ((kBBytes + 1023) / 1024) * 1024;
  static constexpr int kSfbOff = kSfaOff + kSfBytes;
  static constexpr int kBytes = ((kSfbOff + kSfBytes + 1023) / 1024) * 1024;
  static constexpr int kStagesFit = (232448 - 3072) / kBytes;
  static constexpr int kStages = kStagesFit > 10 ? 10 : kStagesFit;
  static constexpr int kAccStride = NCOLS < 32 ? 32 : NCOLS;
  static constexpr int kSfBase = 2 * kAccStride;           // two accumulators, then per-stage scale columns
  static constexpr int kSfCols = kAtomsPerStage * 4 * 2;
  static_assert(kSfBase + kStages * kSfCols <= kTcTmemCols, "tensor memory budget exceeded");
  static constexpr size_t kSmem = size_t(kStages) * kBytes + (3 * kStages + 4) * 8 + 64 + 1024;
};

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Arrival on a tile's counter: releases what the CTA's threads wrote before the barrier they passed on the way
// here, and acquires what earlier arrivers released, for the threads that pass the next barrier.
__device__ __forceinline__ unsigned int arrive_acq_rel(unsigned int* counter) {
  unsigned int old;
  asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  return old;
}

template <int NCOLS, int TERMS>
__global__ void __launch_bounds__(kTcThreads, 1)
nvfp4_gemv_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                     const TcArgs g) {
  using L = TcLayout<NCOLS>;
  constexpr int STAGES = L::kStages;
  constexpr int CH = NCOLS < 32 ? NCOLS : 32;  // accumulator columns handled at a time by an epilogue thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * L::kBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* sf_full_bar = bars + 2 * STAGES;
  uint64_t* tmem_full_bar = bars + 3 * STAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* fix = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [0] last arriver? [1] first owner [2] last owner

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col_tiles = (g.k / 16 + 3) / 4;
  const int KB = g.num_kb;
  const int total = g.row_tiles * KB, grid = int(gridDim.x), cta = int(blockIdx.x);
  const int u_begin = range_start(cta, total, grid), u_end = range_start(cta + 1, total, grid);
  const Segments segs(u_begin, u_end, KB);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&sf_full_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTcTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Kernels queued behind this one as programmatic dependents (the next call's expansion and, behind it, its
  // GEMV) may be scheduled from now on.  They become eligible only once every CTA of this grid has got here,
  // i.e. is resident, so they can only take what this grid's CTAs free when they exit; and they wait for
  // this grid's completion (griddepcontrol.wait) before they touch anything it uses.
  if (threadIdx.x == 0) griddep_launch_dependents();

  // activation terms and their scales of K block kb into stage s (the stage's barrier already expects the bytes)
  auto issue_x = [&](uint32_t s, int kb) {
    const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
    const uint32_t bar = smem_u32(&full_bar[s]);
    uint8_t* st = smem + s * L::kBytes;
    tma_load_2d(smem_u32(st + L::kBOff), &tmap_x, kb * kBlockKBytes, 0, bar);
    bulk_load(smem_u32(st + L::kSfbOff), g.sfb + int64_t(kb) * kAtomsPerStage * kAtomBytes, atoms * kAtomBytes, bar);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    // The weights do not depend on the kernel before this one, the activation terms do: when launched as a
    // programmatic dependent of the expansion kernel, the first ring of weight tiles is requested at once
    // and only the activation tiles wait for the expansion to finish (griddepcontrol.wait is a no-op in an
    // ordinary launch).
    uint32_t it = 0;
    bool ok = true;
    bool dependency_met = false;
    // the activation tiles of the first `limit` iterations, whose weights were requested before the wait
    auto issue_deferred_x = [&](uint32_t limit) {
      uint32_t j = 0;
      for (int i = 0; i < segs.count && j < limit; ++i) {
        int tile, kb0, kb1;
        segs.get(i, tile, kb0, kb1);
        for (int kb = kb0; kb < kb1 && j < limit; ++kb, ++j) issue_x(j, kb);
      }
    };
    for (int i = 0; i < segs.count && ok; ++i) {
      int tile, kb0, kb1;
      segs.get(i, tile, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!dependency_met && it == uint32_t(STAGES)) {
          // every stage of the ring holds its weights: now wait for the activations and request them
          griddep_wait();
          dependency_met = true;
          if (elect_one()) issue_deferred_x(uint32_t(STAGES));
          __syncwarp();
        }
        if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag)) { ok = false; break; }
        const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
        const uint32_t bytes = L::kABytes + L::kBBytes + 2u * uint32_t(atoms) * kAtomBytes;
        const uint32_t bar = smem_u32(&full_bar[s]);
        uint8_t* st = smem + s * L::kBytes;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar, bytes);
          tma_load_2d(smem_u32(st), &tmap_w, kb * kBlockKBytes, tile * kBlockM, bar);
          bulk_load(smem_u32(st + L::kSfaOff), g.sfa + (int64_t(tile) * col_tiles + kb * kAtomsPerStage) * kAtomBytes,
                    atoms * kAtomBytes, bar);
          if (dependency_met) issue_x(uint32_t(s), kb);
        }
        __syncwarp();
      }
    }
    if (!dependency_met && ok) {  // fewer K blocks than stages: nothing was deferred past the loop's end
      griddep_wait();
      if (elect_one()) issue_deferred_x(it);
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = make_idesc_mxf4nvf4(kBlockM, NCOLS);
    uint32_t it = 0, sc = 0;
    bool ok = true;
    for (int i = 0; i < segs.count && ok; ++i, ++sc) {
      int tile, kb0, kb1;
      segs.get(i, tile, kb0, kb1);
      const int acc = sc & 1;
      const uint32_t acc_ph = (sc >> 1) & 1;
      if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_ph ^ 1, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t tmem_d = tmem_base + acc * L::kAccStride;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(smem_u32(&sf_full_bar[s]), ph, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
        uint8_t* st = smem + s * L::kBytes;
        const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + L::kBOff);
        const uint32_t sf_col = tmem_base + L::kSfBase + s * L::kSfCols;
        if (elect_one()) {
          for (int a = 0; a < atoms; ++a) {
            const uint64_t adesc = make_smem_desc(a_addr + a * 32, 16, 1024, kSwizzle128B);
            const uint64_t bdesc = make_smem_desc(b_addr + a * 32, 16, 1024, kSwizzle128B);
            mma_mxf4nvf4(tmem_d, adesc, bdesc, idesc, (kb != kb0 || a != 0) ? 1u : 0u, sf_col + a * 4,
                         sf_col + 16 + a * 4);
          }
          tcgen05_commit(smem_u32(&empty_bar[s]));
        }
        __syncwarp();
      }
      if (ok && elect_one()) tcgen05_commit(smem_u32(&tmem_full_bar[acc]));
      __syncwarp();
    }
  } else if (warp == 2) {
    // -------------------------------------------------------- scale copier
    uint32_t it = 0;
    bool ok = true;
    for (int i = 0; i < segs.count && ok; ++i) {
      int tile, kb0, kb1;
      segs.get(i, tile, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const int atoms = min(kAtomsPerStage, col_tiles - kb * kAtomsPerStage);
        uint8_t* st = smem + s * L::kBytes;
        const uint32_t sfa_addr = smem_u32(st + L::kSfaOff), sfb_addr = smem_u32(st + L::kSfbOff);
        const uint32_t sf_col = tmem_base + L::kSfBase + s * L::kSfCols;
        if (elect_one()) {
          for (int a = 0; a < atoms; ++a) {
            tcgen05_cp_32x128b_warpx4(sf_col + a * 4, make_smem_desc(sfa_addr + a * kAtomBytes, 0, 128, kSwizzleNone));
            tcgen05_cp_32x128b_warpx4(sf_col + 16 + a * 4,
                                      make_smem_desc(sfb_addr + a * kAtomBytes, 0, 128, kSwizzleNone));
          }
          tcgen05_commit(smem_u32(&sf_full_bar[s]));
        }
        __syncwarp();
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int et = row_in_tile;  // index among the 128 epilogue threads
    const int first_tile = u_begin / KB;
    uint32_t sc = 0;
    bool ok = true;

    // columns [c0, c0 + CH) of one output row: scale the terms, add them up, write bf16
    auto finalize = [&](const float (&v)[CH], int c0, int row) {
      if (row >= g.n) return;
#pragma unroll
      for (int j = 0; j < CH; j += TERMS) {
        const int b = (c0 + j) / TERMS;
        if (b < g.batch) {
          float y = 0.f;
#pragma unroll
          for (int t = 0; t < TERMS; ++t) y = fmaf(v[j + t], g.col_scale ? g.col_scale[c0 + j + t] : 1.f, y);
          store_out(g.out, b, row, y * g.alpha);
        }
      }
    };

    for (int i = 0; i < segs.count && ok; ++i, ++sc) {
      int tile, kb0, kb1;
      segs.get(i, tile, kb0, kb1);
      const int acc = sc & 1;
      const uint32_t acc_ph = (sc >> 1) & 1;
      if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_ph, abort_flag)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * L::kAccStride;
      const int row = tile * kBlockM + row_in_tile;
      const bool whole = kb0 == 0 && kb1 == KB;
      float* slot = g.partials + (int64_t(2 * cta + (tile == first_tile ? 0 : 1)) * NCOLS) * kBlockM;

#pragma unroll
      for (int c0 = 0; c0 < NCOLS; c0 += CH) {
        float v[CH];
        if constexpr (CH == 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        } else {
#pragma unroll
          for (int h = 0; h < CH / 8; ++h) {
            uint32_t r[8];
            tmem_ld_32x32b_x8(taddr + c0 + h * 8, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) v[h * 8 + j] = __uint_as_float(r[j]);
          }
        }
        if (c0 + CH >= NCOLS) {  // everything is in registers: hand the accumulator back
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        }
        if (whole) {
          finalize(v, c0, row);
        } else {
#pragma unroll
          for (int j = 0; j < CH; ++j) __stcg(slot + (c0 + j) * kBlockM + et, v[j]);
        }
      }
      if (whole) continue;

      // a tile shared with other CTAs: publish the partial, the last arriver finishes the tile
      epilogue_bar();
      if (et == 0) {
        const int c_first = owner_of(tile * KB, total, grid), c_last = owner_of(tile * KB + KB - 1, total, grid);
        const unsigned int seen = arrive_acq_rel(&g.counters[tile]);
        fix[0] = seen + 1u == unsigned(c_last - c_first + 1);
        fix[1] = c_first;
        fix[2] = c_last;
      }
      epilogue_bar();
      const bool last = fix[0] != 0;
      const int c_first = fix[1], c_last = fix[2];
      epilogue_bar();  // fix[] may be rewritten by the next shared tile
      if (!last) continue;
#pragma unroll 1
      for (int c0 = 0; c0 < NCOLS; c0 += CH) {
        float v[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j) v[j] = 0.f;
        // ascending K: a fixed summation order; two pieces' loads in flight at a time
        for (int c = c_first; c <= c_last; c += 2) {
          float t[2][CH];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int cq = c + q;
            if (cq <= c_last) {
              const int c_tile0 = range_start(cq, total, grid) / KB;
              const float* src = g.partials + (int64_t(2 * cq + (tile == c_tile0 ? 0 : 1)) * NCOLS) * kBlockM;
#pragma unroll
              for (int j = 0; j < CH; ++j) t[q][j] = __ldcg(src + (c0 + j) * kBlockM + et);
            } else {
#pragma unroll
              for (int j = 0; j < CH; ++j) t[q][j] = 0.f;
            }
          }
#pragma unroll
          for (int q = 0; q < 2; ++q) {
#pragma unroll
            for (int j = 0; j < CH; ++j) v[j] += t[q][j];
          }
        }
        finalize(v, c0, row);
      }
      if (et == 0) g.counters[tile] = 0u;
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTcTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicMin(&g_device_status_gemv_tc, HB200_ERR_DEVICE_TIMEOUT);
}

// ------------------------------------------------------------------ activation expansion
// x [batch, K] bf16 -> TERMS NVFP4 rows per activation row (row b * TERMS + t of `codes`, [cols, K/2]),
// their e4m3 block scales in one swizzled 128-row tile, and the fp32 factor of every row.
template <int TERMS>
__global__ void __launch_bounds__(kExpandThreads)
expand_terms_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ codes, uint8_t* __restrict__ sf,
                    float* __restrict__ col_scale, int k) {
  __shared__ float red[kExpandThreads / 32];
  // the GEMV that consumes the terms may start its prologue and its weight prefetch now; this kernel itself
  // must not overwrite the terms before the GEMV of the previous call (its prerequisite when launched as a
  // programmatic dependent; a no-op otherwise) has finished reading them
  griddep_launch_dependents();
  griddep_wait();
  const int b = blockIdx.y, tid = threadIdx.x;
  const __nv_bfloat16* xr = x + int64_t(b) * k;

  // the row's largest magnitude (every CTA of the row recomputes it: the row is a few tens of KB in L2)
  float m = 0.f;
#pragma unroll 4
  for (int i = tid; i < k / 8; i += kExpandThreads) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i * 8);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      m = fmaxf(m, fmaxf(fabsf(bf16_bits_to_f32(w[j] & 0xffffu)), fabsf(bf16_bits_to_f32(w[j] >> 16))));
  }
  m = warp_max(m);
  if ((tid & 31) == 0) red[tid >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int i = 1; i < kExpandThreads / 32; ++i) m = fmaxf(m, red[i]);
  // power of two g0 >= amax / (6 * 448): the first term's block scales fit e4m3
  float g0 = 1.f;
  if (m > 0.f && m < 3.0e38f) {
    int e;
    frexpf(m * (1.f / 2688.f), &e);
    g0 = ldexpf(1.f, max(-120, min(120, e)));
  }
  if (blockIdx.x == 0 && tid < TERMS) col_scale[b * TERMS + tid] = ldexpf(g0, -2 * tid);

  const int blk = blockIdx.x * kExpandThreads + tid;
  if (blk >= k / 16) return;
  float r[16];
  {
    const uint4 lo = *reinterpret_cast<const uint4*>(xr + blk * 16), hi = *reinterpret_cast<const uint4*>(xr + blk * 16 + 8);
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      r[2 * j] = bf16_bits_to_f32(w[j] & 0xffffu);
      r[2 * j + 1] = bf16_bits_to_f32(w[j] >> 16);
    }
  }
  const int64_t k_bytes = k / 2;
#pragma unroll
  for (int t = 0; t < TERMS; ++t) {
    const float g = ldexpf(g0, -2 * t);
    float bmax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) bmax = fmaxf(bmax, fabsf(r[j]));
    const uint32_t sbyte = f32x2_to_e4m3x2(bmax * (1.f / 6.f) / g, 0.f) & 0xffu;
    const float s = e4m3_to_f32(sbyte) * g;  // exact: four significant bits times a power of two
    const float inv = s > 0.f ? 1.f / s : 0.f;
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t byte;
      asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n\tcvt.u32.u8 %0, b;\n\t}"
          : "=r"(byte)
          : "f"(r[2 * j + 1] * inv), "f"(r[2 * j] * inv));
      packed[j >> 2] |= byte << (8 * (j & 3));
      const __half2 d = u32_as_h2(e2m1x2_to_h2(byte));
      r[2 * j] -= __low2float(d) * s;       // products are exact (three bits times four bits times 2^e)
      r[2 * j + 1] -= __high2float(d) * s;
    }
    const int rowi = b * TERMS + t;
    *reinterpret_cast<uint2*>(codes + int64_t(rowi) * k_bytes + int64_t(blk) * 8) = make_uint2(packed[0], packed[1]);
    uint8_t* sf_row = sf + (int64_t(blk >> 2)) * kAtomBytes + (rowi & 31) * 16 + (rowi >> 5) * 4;
    sf_row[blk & 3] = uint8_t(sbyte);
    // the scale columns that pad the last 64-element atom multiply zero codes: they must be finite (the
    // workspace is reused between shapes and may hold any bytes there, the e4m3 NaN patterns included)
    if (blk == k / 16 - 1)
      for (int c = (blk & 3) + 1; c < 4; ++c) sf_row[c] = 0;
  }
}

// ------------------------------------------------------------------ host side
int sm_count_tc() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached = n;
  }
  return cached;
}

// The expansion is launched as a programmatic dependent of whatever kernel precedes it on the stream: it is
// resident early, waits for that kernel's completion, and lets its own dependent (the GEMV) be scheduled.
int launch_expand(const __nv_bfloat16* x, uint8_t* codes, uint8_t* sf, float* col_scale, int64_t k, int64_t batch,
                  cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(ceil_div64(k / 16, kExpandThreads)), unsigned(batch), 1);
  cfg.blockDim = dim3(kExpandThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, expand_terms_kernel<4>, x, codes, sf, col_scale, int(k)) != cudaSuccess) return HB200_ERR_CUDA;
  return HB200_OK;
}

struct TcPlan {
  int ncols;          // MMA N: batch * terms rounded up to 16, 32, 64 or 128
  int grid;
  int row_tiles, num_kb;
  size_t off_counters, off_codes, off_sf, off_cs, off_partials, bytes;
};

inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

bool make_plan(int64_t n, int64_t k, int64_t batch, int terms, TcPlan* p) {
  const int64_t cols = batch * terms;
  if (cols < 1 || cols > 128) return false;
  p->ncols = cols <= 16 ? 16 : cols <= 32 ? 32 : cols <= 64 ? 64 : 128;
  p->row_tiles = int(ceil_div64(n, kBlockM));
  const int64_t col_tiles = ceil_div64(k / 16, 4);
  p->num_kb = int(ceil_div64(col_tiles, kAtomsPerStage));
  const int64_t total = int64_t(p->row_tiles) * p->num_kb;
  if (total <= 0 || total > 0x7fffffff) return false;
  const int sms = sm_count_tc();
  p->grid = int(total < sms ? total : sms);
  // The counters sit in a region of fixed size at the start of the workspace, whatever the shape: it is the
  // only part that has to be zero between calls, and no call ever puts anything else there.
  if (p->row_tiles > kMaxRowTiles) return false;
  size_t off = 0;
  p->off_counters = off; off = align256(off + size_t(kMaxRowTiles) * 4);
  p->off_codes = off;    off = align256(off + size_t(p->ncols) * size_t(k / 2));
  p->off_sf = off;       off = align256(off + size_t(col_tiles) * kAtomBytes);
  p->off_cs = off;       off = align256(off + size_t(p->ncols) * 4);
  p->off_partials = off; off = align256(off + size_t(2) * p->grid * p->ncols * kBlockM * 4);
  p->bytes = off;
  return true;
}

template <int NCOLS, int TERMS>
int launch_tc(const CUtensorMap& tw, const CUtensorMap& tx, const TcArgs& a, int grid, cudaStream_t stream) {
  using L = TcLayout<NCOLS>;
  static_assert(L::kSmem <= 232448, "shared memory budget exceeded");
  auto kernel = nvfp4_gemv_tc_kernel<NCOLS, TERMS>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(L::kSmem)) != cudaSuccess)
    return HB200_ERR_CUDA;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(grid), 1, 1);
  cfg.blockDim = dim3(kTcThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  // after the expansion kernel (TERMS > 1): start while it still runs; the kernel waits for it before it
  // touches the activation terms
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = TERMS > 1 ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kernel, tw, tx, a) != cudaSuccess) return HB200_ERR_CUDA;
  return HB200_OK;
}

template <int TERMS>
int dispatch_tc(int ncols, const CUtensorMap& tw, const CUtensorMap& tx, const TcArgs& a, int grid, cudaStream_t s) {
  switch (ncols) {
    case 16: return launch_tc<16, TERMS>(tw, tx, a, grid, s);
    case 32: return launch_tc<32, TERMS>(tw, tx, a, grid, s);
    case 64: return launch_tc<64, TERMS>(tw, tx, a, grid, s);
    default: return launch_tc<128, TERMS>(tw, tx, a, grid, s);
  }
}

// Shared tail of both operators: the activation terms are in the workspace (or at x_codes / x_sf).
int run_tc(const void* w, const void* w_scale, const uint8_t* x_codes, const uint8_t* x_sf, const float* col_scale,
           const OutSpec& out, int64_t n, int64_t k, int64_t batch, int terms, float alpha, const TcPlan& p,
           uint8_t* ws, cudaStream_t stream) {
  CUtensorMap tw, tx;
  if (!make_operand_map(&tw, w, n, k / 2, kBlockM)) return HB200_ERR_CUDA;
  if (!make_operand_map(&tx, x_codes, p.ncols, k / 2, p.ncols)) return HB200_ERR_CUDA;
  TcArgs a{};
  a.sfa = static_cast<const uint8_t*>(w_scale);
  a.sfb = x_sf;
  a.col_scale = col_scale;
  a.partials = reinterpret_cast<float*>(ws + p.off_partials);
  a.counters = reinterpret_cast<unsigned int*>(ws + p.off_counters);
  a.out = out;
  a.n = int(n);
  a.k = int(k);
  a.batch = int(batch);
  a.row_tiles = p.row_tiles;
  a.num_kb = p.num_kb;
  a.alpha = alpha;
  return terms == 1 ? dispatch_tc<1>(p.ncols, tw, tx, a, p.grid, stream) : dispatch_tc<4>(p.ncols, tw, tx, a, p.grid, stream);
}

int check_common(const void* w, const void* x, const void* ws, int64_t n, int64_t k, int64_t batch) {
  if (!w || !x || !ws) return HB200_ERR_INVALID_ARGUMENT;
  if (n <= 0 || k <= 0 || (k % 16) != 0 || batch < 1) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(w) % 16 || reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(ws) % 16)
    return HB200_ERR_INVALID_ARGUMENT;
  if ((k % 32) != 0 || batch > 32 || n > 0x7fffff00 || k > 0x7fffff00) return HB200_ERR_UNSUPPORTED;
  return HB200_OK;
}

}  // namespace

// Wait budget of this translation unit's bounded mbarrier waits (see hb200_set_wait_budget_cycles).
int gemv_tc_set_wait_budget(long long cycles) { return sm100::set_wait_budget_cycles(cycles) ? HB200_OK : HB200_ERR_CUDA; }

int builtin_scratch_clear_counters_sync();

int gemv_tc_device_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status_gemv_tc, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  if (reset && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_device_status_gemv_tc, &zero, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
    // a kernel that gave up may have left tile arrival counters non-zero: clear the built-in scratch's here
    // (caller-owned workspaces are the caller's to clear: their first hb200_nvfp4_gemv_tc_counter_bytes())
    if (builtin_scratch_clear_counters_sync() != HB200_OK) return HB200_ERR_CUDA;
  }
  return v;
}

}  // namespace hb200

// Bytes of workspace the tensor-core GEMV needs for this shape (terms = 4 for bf16 activations, 1 for
// NVFP4 activations); negative HB200_ERR_* for shapes it does not take.
extern "C" int64_t hb200_nvfp4_gemv_tc_workspace_bytes(int64_t n, int64_t k, int64_t batch, int64_t terms) {
  hb200::TcPlan p;
  if (n <= 0 || k <= 0 || (k % 32) != 0 || batch < 1 || batch > 32 || (terms != 1 && terms != 4))
    return HB200_ERR_UNSUPPORTED;
  if (!hb200::make_plan(n, k, batch, int(terms), &p)) return HB200_ERR_UNSUPPORTED;
  return int64_t(p.bytes);
}

extern "C" int hb200_nvfp4_gemv_bf16in_tc(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                                          void* const* out_ptrs, int64_t world, int64_t n, int64_t k, int64_t batch,
                                          int64_t n_total, int64_t col0, float alpha, void* workspace,
                                          int64_t workspace_bytes, void* stream) {
  using namespace hb200;
  if (!out_ptrs || !workspace || world < 1 || world > 8 || col0 < 0 || col0 + n > n_total)
    return HB200_ERR_INVALID_ARGUMENT;
  const int rc = check_common(weight_packed, x_bf16, weight_scale, n, k, batch);
  if (rc != HB200_OK) return rc;
  if (reinterpret_cast<uintptr_t>(workspace) % 256) return HB200_ERR_INVALID_ARGUMENT;
  TcPlan p;
  if (!make_plan(n, k, batch, 4, &p)) return HB200_ERR_UNSUPPORTED;
  if (workspace_bytes < int64_t(p.bytes)) return HB200_ERR_WORKSPACE;
  OutSpec o{};
  for (int i = 0; i < world; ++i) {
    if (!out_ptrs[i]) return HB200_ERR_INVALID_ARGUMENT;
    o.ptr[i] = static_cast<__nv_bfloat16*>(out_ptrs[i]);
  }
  o.count = int(world);
  o.ld = n_total;
  o.col0 = col0;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (launch_expand(static_cast<const __nv_bfloat16*>(x_bf16), ws + p.off_codes, ws + p.off_sf,
                    reinterpret_cast<float*>(ws + p.off_cs), k, batch, s) != HB200_OK)
    return HB200_ERR_CUDA;
  return run_tc(weight_packed, weight_scale, ws + p.off_codes, ws + p.off_sf, reinterpret_cast<const float*>(ws + p.off_cs),
                o, n, k, batch, 4, alpha, p, ws, s);
}

extern "C" int hb200_nvfp4_gemv_fp4in_tc(const void* weight_packed, const void* x_packed, const void* weight_scale,
                                         const void* x_scale, void* out_bf16, int64_t n, int64_t k, float alpha,
                                         void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace hb200;
  if (!out_bf16 || !x_scale || !workspace) return HB200_ERR_INVALID_ARGUMENT;
  const int rc = check_common(weight_packed, x_packed, weight_scale, n, k, 1);
  if (rc != HB200_OK) return rc;
  if (reinterpret_cast<uintptr_t>(workspace) % 256 || reinterpret_cast<uintptr_t>(x_scale) % 16)
    return HB200_ERR_INVALID_ARGUMENT;
  TcPlan p;
  if (!make_plan(n, k, 1, 1, &p)) return HB200_ERR_UNSUPPORTED;
  if (workspace_bytes < int64_t(p.bytes)) return HB200_ERR_WORKSPACE;
  OutSpec o{};
  o.ptr[0] = static_cast<__nv_bfloat16*>(out_bf16);
  o.count = 1;
  o.ld = n;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the single activation row becomes row 0 of the 16-row operand; rows 1..15 feed columns nobody reads
  if (cudaMemcpyAsync(ws + p.off_codes, x_packed, size_t(k / 2), cudaMemcpyDeviceToDevice, s) != cudaSuccess)
    return HB200_ERR_CUDA;
  return run_tc(weight_packed, weight_scale, ws + p.off_codes, static_cast<const uint8_t*>(x_scale), nullptr, o, n, k, 1, 1,
                alpha, p, ws, s);
}

// ------------------------------------------------------------------ built-in scratch
// hb200_nvfp4_gemv_bf16in_tc for callers that cannot hand over a workspace: the scratch is this array in
// the library's own device image, one per device, so the call allocates nothing, neither here nor in the
// caller.  8 MiB holds every shape with at most 8 activation rows and K <= 65536; larger requests are
// refused with HB200_ERR_SCRATCH_LIMIT.
namespace hb200 {
namespace {

constexpr size_t kBuiltinScratchBytes = size_t(8) << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

std::mutex g_builtin_mutex;
void* g_builtin_ptr[kMaxDevices] = {};  // device address of g_builtin_scratch on every device seen so far

// First call on a device (that device current): look the array's address up and clear the part that has to
// start at zero, the tile arrival counters, on the caller's stream.  Later calls only read the cached address.
int builtin_scratch(cudaStream_t stream, void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HB200_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return HB200_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_builtin_mutex);
  if (g_builtin_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_builtin_scratch) != cudaSuccess || ptr == nullptr)
      return HB200_ERR_CUDA;
    if (cudaMemsetAsync(ptr, 0, size_t(kMaxRowTiles) * 4, stream) != cudaSuccess) return HB200_ERR_CUDA;
    g_builtin_ptr[dev] = ptr;
  }
  *out = g_builtin_ptr[dev];
  return HB200_OK;
}

}  // namespace

// Clears the arrival counters of the current device's built-in scratch, if that device has used it; device-synchronous.
int builtin_scratch_clear_counters_sync() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HB200_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return HB200_OK;
  std::lock_guard<std::mutex> lock(g_builtin_mutex);
  if (g_builtin_ptr[dev] == nullptr) return HB200_OK;
  return cudaMemset(g_builtin_ptr[dev], 0, size_t(kMaxRowTiles) * 4) == cudaSuccess ? HB200_OK : HB200_ERR_CUDA;
}

}  // namespace hb200

// Re-zeroes, on `stream`, the part of the built-in scratch that must be zero between calls (the tile arrival
// counters).  Needed after a call that ended with HB200_ERR_DEVICE_TIMEOUT or after two calls overlapped on the
// device: either can leave counters non-zero, and every later call would then leave tiles unwritten.  Allocates
// nothing.  (hb200_device_status(1) does the same, synchronously, when it clears a non-zero status.)
extern "C" int hb200_nvfp4_gemv_tc_builtin_scratch_reset(void* stream) {
  using namespace hb200;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* scratch = nullptr;
  const int rs = builtin_scratch(s, &scratch);
  if (rs != HB200_OK) return rs;
  return cudaMemsetAsync(scratch, 0, size_t(kMaxRowTiles) * 4, s) == cudaSuccess ? HB200_OK : HB200_ERR_CUDA;
}

// Bytes at the start of every tensor-core GEMV workspace (caller-owned or built-in) that hold the tile arrival
// counters: the only part that must be zero when a call starts.
extern "C" int64_t hb200_nvfp4_gemv_tc_counter_bytes(void) { return int64_t(hb200::kMaxRowTiles) * 4; }

extern "C" int hb200_nvfp4_gemv_bf16in_tc_builtin_scratch(const void* weight_packed, const void* x_bf16,
                                                          const void* weight_scale, void* out_bf16, int64_t n,
                                                          int64_t k, int64_t batch, float alpha, void* stream) {
  using namespace hb200;
  if (!out_bf16) return HB200_ERR_INVALID_ARGUMENT;
  const int rc = check_common(weight_packed, x_bf16, weight_scale, n, k, batch);
  if (rc != HB200_OK) return rc;
  TcPlan p;
  if (!make_plan(n, k, batch, 4, &p)) return HB200_ERR_UNSUPPORTED;
  if (p.bytes > kBuiltinScratchBytes) return HB200_ERR_SCRATCH_LIMIT;  // more rows or a longer K than the array holds
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* scratch = nullptr;
  const int rs = builtin_scratch(s, &scratch);
  if (rs != HB200_OK) return rs;
  uint8_t* ws = static_cast<uint8_t*>(scratch);
  OutSpec o{};
  o.ptr[0] = static_cast<__nv_bfloat16*>(out_bf16);
  o.count = 1;
  o.ld = n;
  if (launch_expand(static_cast<const __nv_bfloat16*>(x_bf16), ws + p.off_codes, ws + p.off_sf,
                    reinterpret_cast<float*>(ws + p.off_cs), k, batch, s) != HB200_OK)
    return HB200_ERR_CUDA;
  return run_tc(weight_packed, weight_scale, ws + p.off_codes, ws + p.off_sf, reinterpret_cast<const float*>(ws + p.off_cs),
                o, n, k, batch, 4, alpha, p, ws, s);
}
