// NVFP4 GEMV for sm_100a: out[n] = bf16(alpha * sum_g s[n,g] * sum_i e2m1(W[n,16g+i]) * x[16g+i]).
//
// Memory-bound: each weight byte is read once with 128-bit streaming loads, the
// block scales are read in their native SWIZZLE_32_4_4 order, the activation is
// staged once per CTA in shared memory (as fp16, laid out so the inner loop's
// 128-bit shared loads are conflict free), products are exact in fp16 and the
// running sum is fp32.  K is reduced across the 8 lanes that share a row with
// warp shuffles and, when the K range is split over a thread-block cluster,
// across CTAs through distributed shared memory.
//
// Thread mapping.  A CTA owns 32 rows of one 128-row scale tile: warp w (0..7)
// owns the four rows  tile*128 + l + 32q  (l = 8*(group%4) + w, q = 0..3), which
// are exactly the rows whose scales share one 16-byte line of the swizzled
// layout.  Lane = (q = lane/8, j = lane%8); per iteration (256 K-elements) lane
// (q, j) consumes the 16 weight bytes [32j, 32j+32) of its row, i.e. two scale
// groups, so a warp request touches four full 128-byte lines of weights and four
// 16-byte pieces of scales.
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace hb200 {
namespace {

constexpr int kGemvThreads = 256;
constexpr int kIterK = 256;        // K-elements consumed by one warp iteration
constexpr int kRowsPerCta = 32;
constexpr int kMaxSplit = 8;       // portable cluster size limit
constexpr int kChunkIters = 32;    // iterations staged at once: 8192 activations = 16 KB of fp16

// 16 codes (two 32-bit words) against 16 fp16 activations held in two uint4.
__device__ __forceinline__ float dot16(uint32_t wa, uint32_t wb, const uint4& xa, const uint4& xb) {
  uint32_t ha[4], hb[4];
  e2m1x8_to_h2x4(wa, ha);
  e2m1x8_to_h2x4(wb, hb);
  __half2 a = __hmul2(u32_as_h2(ha[0]), u32_as_h2(xa.x));
  __half2 b = __hmul2(u32_as_h2(hb[0]), u32_as_h2(xb.x));
  a = __hfma2(u32_as_h2(ha[1]), u32_as_h2(xa.y), a);
  b = __hfma2(u32_as_h2(hb[1]), u32_as_h2(xb.y), b);
  a = __hfma2(u32_as_h2(ha[2]), u32_as_h2(xa.z), a);
  b = __hfma2(u32_as_h2(hb[2]), u32_as_h2(xb.z), b);
  a = __hfma2(u32_as_h2(ha[3]), u32_as_h2(xa.w), a);
  b = __hfma2(u32_as_h2(hb[3]), u32_as_h2(xb.w), b);
  const float2 fa = __half22float2(a);
  const float2 fb = __half22float2(b);
  return (fa.x + fa.y) + (fb.x + fb.y);
}

// Stage x[k_begin, k_end) into shared memory as fp16.  The range is cut into
// 16-byte chunks of 8 values; inside every block of 32 chunks (one iteration)
// logical chunk 4j+k is stored at slot 8k+j so that the eight lanes j of a row
// read eight consecutive slots.  Slots past k_end are zero.
template <bool X_FP4>
__device__ __forceinline__ void stage_x(uint4* xs, const void* x, const uint8_t* x_scale, int64_t k_begin,
                                        int64_t k_end, int n_iter) {
  const int chunks = n_iter * 32;
  for (int ci = threadIdx.x; ci < chunks; ci += kGemvThreads) {
    const int64_t k0 = k_begin + int64_t(ci) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (k0 < k_end) {  // K % 16 == 0 and k_begin % 256 == 0, so a chunk is all-in or all-out
      if constexpr (X_FP4) {
        const uint32_t codes = *reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(x) + k0 / 2);
        const int64_t g = k0 / 16;
        // logical scale shape [1, K/16]: row 0 of a 128-row tile
        const uint32_t sb = x_scale[(g / 4) * 512 + (g % 4)];
        const uint32_t sh = e4m3x2_to_h2(sb) & 0xffffu;
        const __half2 s2 = u32_as_h2(sh | (sh << 16));
        uint32_t h[4];
        e2m1x8_to_h2x4(codes, h);
        v.x = h2_as_u32(__hmul2(u32_as_h2(h[0]), s2));  // e2m1 * e4m3 has <= 6 significant bits: exact
        v.y = h2_as_u32(__hmul2(u32_as_h2(h[1]), s2));
        v.z = h2_as_u32(__hmul2(u32_as_h2(h[2]), s2));
        v.w = h2_as_u32(__hmul2(u32_as_h2(h[3]), s2));
      } else {
        const uint4 b = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + k0);
        auto cv = [](uint32_t two_bf16) {
          const float lo = bf16_bits_to_f32(two_bf16 & 0xffffu);
          const float hi = bf16_bits_to_f32(two_bf16 >> 16);
          return h2_as_u32(__floats2half2_rn(lo, hi));
        };
        v.x = cv(b.x); v.y = cv(b.y); v.z = cv(b.z); v.w = cv(b.w);
      }
    }
    const int it = ci >> 5, c = ci & 31;
    xs[it * 32 + (c & 3) * 8 + (c >> 2)] = v;
  }
}

struct GemvArgs {
  const uint8_t* w;        // [N, K/2]
  const void* x;           // bf16 [K] or packed e2m1 [K/2]
  const uint8_t* w_scale;  // swizzled [N, K/16]
  const uint8_t* x_scale;  // swizzled [1, K/16] (fp4 input only)
  OutSpec out;             // [N] (one buffer, or one per tensor-parallel rank)
  int64_t n, k;
  int iters_per_split;     // 256-element iterations handled by one CTA of the cluster
  float alpha;
};

// U: weight loads a thread keeps in flight per round.  4 for matrices that fill the machine several times over
// (four CTAs per SM); 8 for small ones, which are bound by the latency of dependent rounds, not by occupancy.
template <bool X_FP4, bool VEC16, int U>
__global__ void __launch_bounds__(kGemvThreads, U == 4 ? 4 : 2) nvfp4_gemv_kernel(const GemvArgs a) {
  extern __shared__ uint4 xs[];
  __shared__ float part[kMaxSplit][kRowsPerCta];

  cg::cluster_group cluster = cg::this_cluster();
  const int split = blockIdx.y;  // the cluster spans gridDim.y
  const int n_split = gridDim.y;

  const int64_t k_begin = int64_t(split) * a.iters_per_split * kIterK;
  const int64_t k_end = min(a.k, k_begin + int64_t(a.iters_per_split) * kIterK);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane >> 3, j = lane & 7;
  const int64_t tile = blockIdx.x >> 2;
  const int l = ((blockIdx.x & 3) << 3) + warp;
  const int64_t row = tile * 128 + l + 32 * q;
  const bool row_ok = row < a.n;
  const int64_t k_bytes = a.k >> 1;
  const int64_t groups = a.k >> 4;
  const int64_t col_tiles = (groups + 3) >> 2;
  const uint4* xp = xs + j;

  float acc = 0.f;
  if (n_split > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");  // waited for before the reduction

  // The CTA's K range is consumed in chunks of kChunkIters iterations so the
  // staged activation stays small enough for several CTAs per SM.
#pragma unroll 1
  for (int64_t c_begin = k_begin; c_begin < k_end; c_begin += int64_t(kChunkIters) * kIterK) {
    const int64_t c_end = min(k_end, c_begin + int64_t(kChunkIters) * kIterK);
    const int n_iter = int((c_end - c_begin + kIterK - 1) / kIterK);
    const uint8_t* wp = a.w + (row_ok ? row : 0) * k_bytes + (c_begin >> 1) + j * 16;
    // scale bytes of groups (2j, 2j+1) of this lane's row, inside column tile j/2 of the iteration
    const uint8_t* sp =
        a.w_scale + (tile * col_tiles + (c_begin >> 6) + (j >> 1)) * 512 + l * 16 + q * 4 + (j & 1) * 2;
    const int full_iter = row_ok ? int((c_end - c_begin) / kIterK) : 0;

    auto consume = [&](const uint4& w, uint32_t sc2, int it) {
      const uint4* xi = xp + it * 32;
      const float2 s = __half22float2(u32_as_h2(e4m3x2_to_h2(sc2)));
      const float d0 = dot16(w.x, w.y, xi[0], xi[8]);
      const float d1 = dot16(w.z, w.w, xi[16], xi[24]);
      acc = fmaf(s.x, d0, acc);
      acc = fmaf(s.y, d1, acc);
    };
    auto load_w = [&](int it) -> uint4 {
      const uint8_t* p = wp + int64_t(it) * (kIterK / 2);
      if constexpr (VEC16) {
        return ldg_stream_u4(p);
      } else {
        const uint2 lo = ldg_stream_u2(p), hi = ldg_stream_u2(p + 8);
        return make_uint4(lo.x, lo.y, hi.x, hi.y);
      }
    };
    auto load_s = [&](int it) -> uint32_t {
      return *reinterpret_cast<const unsigned short*>(sp + int64_t(it) * (4 * 512));
    };

    // The first weight and scale loads of the chunk do not depend on the staged activation: they are issued
    // before it is staged, so their latency overlaps the activation's (on a small matrix a CTA's whole share
    // is these few loads, and the two latencies in a row were a third of the kernel).
    uint4 w0[U];
    uint32_t sc0[U];
    const bool head = full_iter >= U;
    if (head) {
#pragma unroll
      for (int u = 0; u < U; ++u) { w0[u] = load_w(u); sc0[u] = load_s(u); }
    }
    if (c_begin != k_begin) __syncthreads();  // previous chunk fully consumed
    stage_x<X_FP4>(xs, a.x, a.x_scale, c_begin, c_end, n_iter);
    __syncthreads();

    int it = 0;
    if (head) {
#pragma unroll
      for (int u = 0; u < U; ++u) consume(w0[u], sc0[u], u);
      it = U;
    }
#pragma unroll 1
    for (; it + U <= full_iter; it += U) {
      uint4 w[U];
      uint32_t sc[U];
#pragma unroll
      for (int u = 0; u < U; ++u) { w[u] = load_w(it + u); sc[u] = load_s(it + u); }
#pragma unroll
      for (int u = 0; u < U; ++u) consume(w[u], sc[u], it + u);
    }
#pragma unroll 1
    for (; it < full_iter; ++it) consume(load_w(it), load_s(it), it);

    // ragged last iteration of the whole K range: per-group predicates (K % 16 == 0)
    if (row_ok && full_iter < n_iter) {
      const int64_t g0 = ((c_begin + int64_t(full_iter) * kIterK) >> 4) + 2 * j;
      const uint8_t* p = wp + int64_t(full_iter) * (kIterK / 2);
      const uint8_t* s1 = sp + int64_t(full_iter) * (4 * 512);
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      uint32_t sc = 0;
      if (g0 < groups) {
        const uint2 lo = ldg_stream_u2(p);
        w.x = lo.x; w.y = lo.y;
        sc = s1[0];
      }
      if (g0 + 1 < groups) {
        const uint2 hi = ldg_stream_u2(p + 8);
        w.z = hi.x; w.w = hi.y;
        sc |= uint32_t(s1[1]) << 8;
      }
      consume(w, sc, full_iter);
    }
  }

  // reduce over the 8 lanes of a row
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);

  if (n_split == 1) {
    if (j == 0 && row_ok) store_out(a.out, 0, row, acc * a.alpha);
    return;
  }
  // split-K: every CTA deposits its 32 partial sums in the leader's shared
  // memory.  The first barrier (arrived at when the kernel started, waited for only here, so it costs
  // nothing by now) guarantees the leader is resident before the remote store, the second publishes the stores.
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
  if (j == 0) {
    float* dst = cluster.map_shared_rank(&part[0][0], 0);
    dst[split * kRowsPerCta + warp * 4 + q] = acc;
  }
  cluster.sync();
  if (split == 0 && threadIdx.x < kRowsPerCta) {
    const int w2 = threadIdx.x >> 2, q2 = threadIdx.x & 3;
    const int64_t r = tile * 128 + ((blockIdx.x & 3) << 3) + w2 + 32 * q2;
    float s = 0.f;
    for (int i = 0; i < n_split; ++i) s += part[i][threadIdx.x];
    if (r < a.n) store_out(a.out, 0, r, s * a.alpha);
  }
}

int sm_count() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached = n;
  }
  return cached;
}

template <bool X_FP4, bool VEC16>
int launch_gemv(const GemvArgs& base, cudaStream_t stream) {
  GemvArgs a = base;
  // four CTAs cover one 128-row scale tile (rows l + 32q), so tiles are launched whole
  const int64_t row_groups = ceil_div64(a.n, 128) * 4;
  const int64_t total_iters = ceil_div64(a.k, kIterK);
  // Split K over a cluster until every SM has two CTAs, while every CTA keeps at least 4 iterations.  Measured
  // on 19 to 47 MB matrices (in-graph, microseconds for cluster sizes 1 / 2 / 4 / 8): 8192 x 4096: 9.5 / 8.6 / 10.1 /
  // 15.8; 8192 x 8192: 15.6 / 12.4 / 14.1 / 17.1; 15360 x 5120: 14.2 / 16.4 / 19.5 / 30.8: the cluster barrier and
  // the reduction through distributed shared memory cost more than the extra CTAs bring beyond that point.
  int split = 1;
  const int64_t want = int64_t(sm_count()) * 2;
  while (split < 4 && row_groups * split < want && total_iters / (split * 2) >= 4) split *= 2;

  a.iters_per_split = int(ceil_div64(total_iters, split));
  if (row_groups > 0x7fffffff) return HB200_ERR_UNSUPPORTED;
  const size_t smem = size_t(kChunkIters) * kIterK * 2;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(row_groups), unsigned(split), 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = unsigned(split);
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // small grids (at most three CTAs per SM): the deeper kernel
  const bool deep = row_groups * split <= int64_t(sm_count()) * 3 && a.iters_per_split >= 8;
  const cudaError_t rc = deep ? cudaLaunchKernelEx(&cfg, nvfp4_gemv_kernel<X_FP4, VEC16, 8>, a)
                              : cudaLaunchKernelEx(&cfg, nvfp4_gemv_kernel<X_FP4, VEC16, 4>, a);
  return rc == cudaSuccess ? HB200_OK : HB200_ERR_CUDA;
}

template <bool X_FP4>
int dispatch_gemv(const GemvArgs& a, cudaStream_t stream) {
  const bool vec16 = (a.k % 32 == 0) && (reinterpret_cast<uintptr_t>(a.w) % 16 == 0);
  return vec16 ? launch_gemv<X_FP4, true>(a, stream) : launch_gemv<X_FP4, false>(a, stream);
}

}  // namespace

int gemv_bf16in_batch1(const void* w, const void* x, const void* ws, const OutSpec& out, int64_t n, int64_t k,
                       float alpha, cudaStream_t stream) {
  GemvArgs a{static_cast<const uint8_t*>(w), x, static_cast<const uint8_t*>(ws), nullptr, out, n, k, 0, alpha};
  return dispatch_gemv<false>(a, stream);
}

}  // namespace hb200

extern "C" int hb200_nvfp4_gemv_fp4in(const void* weight_packed, const void* x_packed, const void* weight_scale,
                                      const void* x_scale, void* out_bf16, int64_t n, int64_t k, float alpha,
                                      void* stream) {
  if (!weight_packed || !x_packed || !weight_scale || !x_scale || !out_bf16) return HB200_ERR_INVALID_ARGUMENT;
  if (n < 0 || k < 0 || (k % 16) != 0) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(weight_packed) % 8 || reinterpret_cast<uintptr_t>(x_packed) % 4)
    return HB200_ERR_INVALID_ARGUMENT;
  if (n == 0) return HB200_OK;
  hb200::OutSpec o{};
  o.ptr[0] = static_cast<__nv_bfloat16*>(out_bf16);
  o.count = 1;
  o.ld = n;
  o.col0 = 0;
  hb200::GemvArgs a{static_cast<const uint8_t*>(weight_packed), x_packed,
                    static_cast<const uint8_t*>(weight_scale), static_cast<const uint8_t*>(x_scale), o, n, k, 0, alpha};
  return hb200::dispatch_gemv<true>(a, static_cast<cudaStream_t>(stream));
}
