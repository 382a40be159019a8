// Decode-batch NVFP4 "skinny GEMM": out[b, n] = bf16(alpha * sum_k x[b, k] * deq(W)[n, k]) for 1..32
// activation rows.  Still bound by the single pass over the weights, so the
// structure is the GEMV's: 128-bit streaming weight loads, native-order scale
// loads, activations staged in shared memory as fp16.  What changes is the
// arithmetic: each weight pair is decoded to fp16, multiplied by its block
// scale (e2m1 x e4m3 has at most 6 significant bits, so the product is exact in
// fp16) and fed as the A operand of warp-level m16n8k16 MMAs whose B operand is
// an 8-row slice of the batch; accumulation is fp32 inside the MMA.  The weight
// rows ride the MMA's M dimension (swap-AB), so the cost per weight byte is the
// same for every batch size up to 8 and grows by one MMA per extra 8 rows.
//
// A CTA owns one 128-row scale tile; warp w owns the 16 rows
//   m -> tile*128 + (4w + m/4) + 32*(m%4),
// lane (g = lane/4, t = lane%4) holds MMA rows g and g+8 and, per iteration of
// 128 K-elements, the 16 weight bytes [16t, 16t+16) of both rows.  The K slots
// of an MMA are filled with whatever k each lane holds (slot 2t,2t+1 <- k0,k0+1;
// slot 2t+8,2t+9 <- k0+2,k0+3 with k0 = 32t + 4i for the i-th MMA); the B
// fragment reads the same k from shared memory, so the contraction is unchanged.
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace hb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kSlabK = 128;  // K-elements per iteration
constexpr int kRows = 128;   // weight rows per CTA

__device__ __forceinline__ void mma_m16n8k16_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct BatchedArgs {
  const uint8_t* w;
  const __nv_bfloat16* x;  // [batch, K]
  const uint8_t* w_scale;
  OutSpec out;             // [batch, N] (one buffer, or one per tensor-parallel rank)
  int64_t n, k;
  int batch;
  int iters_per_split;     // 128-element iterations per CTA of the cluster
  int chunk_iters;         // iterations staged in shared memory at once
  float alpha;
};

// NT = number of 8-row batch tiles.
template <int NT, bool VEC16>
__global__ void __launch_bounds__(kThreads) nvfp4_gemv_batched_kernel(const BatchedArgs a) {
  extern __shared__ uint4 xs[];
  cg::cluster_group cluster = cg::this_cluster();
  const int split = blockIdx.y, n_split = gridDim.y;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t tile = blockIdx.x;
  const int qr = g & 3;
  const int l_a = warp * 4 + (g >> 2), l_b = l_a + 2;
  const int64_t row_a = tile * kRows + l_a + 32 * qr, row_b = tile * kRows + l_b + 32 * qr;
  const bool ok_a = row_a < a.n, ok_b = row_b < a.n;
  const int64_t k_bytes = a.k >> 1, groups = a.k >> 4, col_tiles = (groups + 3) >> 2;
  const int stride16 = a.chunk_iters * 16 + 4;  // row stride of xs in 16-byte units, == 4 (mod 8)

  const int64_t k_begin = int64_t(split) * a.iters_per_split * kSlabK;
  const int64_t k_end = min(a.k, k_begin + int64_t(a.iters_per_split) * kSlabK);

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

#pragma unroll 1
  for (int64_t c_begin = k_begin; c_begin < k_end; c_begin += int64_t(a.chunk_iters) * kSlabK) {
    const int64_t c_end = min(k_end, c_begin + int64_t(a.chunk_iters) * kSlabK);
    const int n_iter = int((c_end - c_begin + kSlabK - 1) / kSlabK);
    if (c_begin != k_begin) __syncthreads();
    // stage x[:, c_begin:c_end) as fp16: chunk 4t+k of a slab goes to slot 4k+t
    for (int ci = threadIdx.x; ci < NT * 8 * n_iter * 16; ci += kThreads) {
      const int b = ci / (n_iter * 16), c = ci - b * (n_iter * 16);
      const int64_t k0 = c_begin + int64_t(c) * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (b < a.batch && k0 < c_end) {
        const uint4 raw = *reinterpret_cast<const uint4*>(a.x + int64_t(b) * a.k + k0);
        auto cv = [](uint32_t two_bf16) {
          return h2_as_u32(__floats2half2_rn(bf16_bits_to_f32(two_bf16 & 0xffffu), bf16_bits_to_f32(two_bf16 >> 16)));
        };
        v.x = cv(raw.x); v.y = cv(raw.y); v.z = cv(raw.z); v.w = cv(raw.w);
      }
      const int it = c >> 4, cc = c & 15;
      xs[b * stride16 + it * 16 + (cc & 3) * 4 + (cc >> 2)] = v;
    }
    __syncthreads();

    const uint8_t* wpa = a.w + (ok_a ? row_a : 0) * k_bytes + (c_begin >> 1) + t * 16;
    const uint8_t* wpb = a.w + (ok_b ? row_b : 0) * k_bytes + (c_begin >> 1) + t * 16;
    const uint8_t* sbase = a.w_scale + (tile * col_tiles + (c_begin >> 6) + (t >> 1)) * 512 + qr * 4 + (t & 1) * 2;
    const uint8_t* spa = sbase + l_a * 16;
    const uint8_t* spb = sbase + l_b * 16;
    const uint4* xrow = xs + g * stride16 + t;
    const int full_iter = int((c_end - c_begin) / kSlabK);

    auto consume = [&](const uint4& wa, const uint4& wb, uint32_t sa2, uint32_t sb2, int it) {
      const uint32_t sah = e4m3x2_to_h2(sa2), sbh = e4m3x2_to_h2(sb2);
      const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w};
      const uint32_t wbv[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        // words 0,1 belong to the lane's first scale group, words 2,3 to the second
        const uint32_t sa = wi < 2 ? __byte_perm(sah, 0, 0x1010) : __byte_perm(sah, 0, 0x3232);
        const uint32_t sb = wi < 2 ? __byte_perm(sbh, 0, 0x1010) : __byte_perm(sbh, 0, 0x3232);
        uint32_t ha[4], hb[4];
        e2m1x8_to_h2x4(wav[wi], ha);
        e2m1x8_to_h2x4(wbv[wi], hb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ha[i] = h2_as_u32(__hmul2(u32_as_h2(ha[i]), u32_as_h2(sa)));
          hb[i] = h2_as_u32(__hmul2(u32_as_h2(hb[i]), u32_as_h2(sb)));
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4 xv = xrow[nt * 8 * stride16 + it * 16 + wi * 4];
          mma_m16n8k16_f16(acc[nt], ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
          mma_m16n8k16_f16(acc[nt], ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
        }
      }
    };
    auto load_w = [&](const uint8_t* base, bool ok, int it) -> uint4 {
      if (!ok) return make_uint4(0u, 0u, 0u, 0u);
      const uint8_t* p = base + int64_t(it) * (kSlabK / 2);
      if constexpr (VEC16) {
        return ldg_stream_u4(p);
      } else {
        const uint2 lo = ldg_stream_u2(p), hi = ldg_stream_u2(p + 8);
        return make_uint4(lo.x, lo.y, hi.x, hi.y);
      }
    };
    auto load_s = [&](const uint8_t* base, int it) -> uint32_t {
      return *reinterpret_cast<const unsigned short*>(base + int64_t(it) * (2 * 512));
    };

    constexpr int U = NT >= 4 ? 2 : 4;
    int it = 0;
#pragma unroll 1
    for (; it + U <= full_iter; it += U) {
      uint4 wa[U], wb[U];
      uint32_t sa[U], sb[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        wa[u] = load_w(wpa, ok_a, it + u); wb[u] = load_w(wpb, ok_b, it + u);
        sa[u] = load_s(spa, it + u); sb[u] = load_s(spb, it + u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) consume(wa[u], wb[u], sa[u], sb[u], it + u);
    }
#pragma unroll 1
    for (; it < full_iter; ++it)
      consume(load_w(wpa, ok_a, it), load_w(wpb, ok_b, it), load_s(spa, it), load_s(spb, it), it);

    if (full_iter < n_iter) {  // ragged tail of K: per-group predicates
      const int64_t g0 = ((c_begin + int64_t(full_iter) * kSlabK) >> 4) + 2 * t;
      const int64_t off = int64_t(full_iter) * (kSlabK / 2);
      const int64_t soff = int64_t(full_iter) * (2 * 512);
      uint4 wa = make_uint4(0u, 0u, 0u, 0u), wb = wa;
      uint32_t sa = 0, sb = 0;
      if (g0 < groups) {
        if (ok_a) { const uint2 v = ldg_stream_u2(wpa + off); wa.x = v.x; wa.y = v.y; }
        if (ok_b) { const uint2 v = ldg_stream_u2(wpb + off); wb.x = v.x; wb.y = v.y; }
        sa = spa[soff]; sb = spb[soff];
      }
      if (g0 + 1 < groups) {
        if (ok_a) { const uint2 v = ldg_stream_u2(wpa + off + 8); wa.z = v.x; wa.w = v.y; }
        if (ok_b) { const uint2 v = ldg_stream_u2(wpb + off + 8); wb.z = v.x; wb.w = v.y; }
        sa |= uint32_t(spa[soff + 1]) << 8; sb |= uint32_t(spb[soff + 1]) << 8;
      }
      consume(wa, wb, sa, sb, full_iter);
    }
  }

  // Split-K reduction and coalesced store through the leader CTA's shared memory:
  // buffer[split][b][local row], local row = 32q + l.
  cluster.sync();  // every CTA is done reading its staged activations
  {
    float* buf = reinterpret_cast<float*>(cluster.map_shared_rank(xs, 0)) + size_t(split) * (NT * 8 * kRows);
    const int lr_a = 32 * qr + l_a, lr_b = 32 * qr + l_b;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int b0 = nt * 8 + 2 * t;
      buf[b0 * kRows + lr_a] = acc[nt][0];
      buf[(b0 + 1) * kRows + lr_a] = acc[nt][1];
      buf[b0 * kRows + lr_b] = acc[nt][2];
      buf[(b0 + 1) * kRows + lr_b] = acc[nt][3];
    }
  }
  cluster.sync();
  if (split == 0) {
    const float* buf = reinterpret_cast<const float*>(xs);
    for (int e = threadIdx.x; e < a.batch * kRows; e += kThreads) {
      const int b = e / kRows, lr = e - b * kRows;
      const int64_t r = tile * kRows + lr;
      if (r >= a.n) continue;
      float s = 0.f;
      for (int i = 0; i < n_split; ++i) s += buf[size_t(i) * (NT * 8 * kRows) + e];
      store_out(a.out, b, r, s * a.alpha);
    }
  }
}

int sm_count_b() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached = n;
  }
  return cached;
}

template <int NT, bool VEC16>
int launch_batched(BatchedArgs a, cudaStream_t stream) {
  const int64_t tiles = ceil_div64(a.n, kRows);
  const int64_t total_iters = ceil_div64(a.k, kSlabK);
  a.chunk_iters = NT >= 4 ? 8 : 16;
  const size_t smem = size_t(NT) * 8 * (a.chunk_iters * 16 + 4) * 16;
  // the reduction buffer (split x NT*8 x 128 floats) reuses the staging area
  const int max_split = int(smem / (size_t(NT) * 8 * kRows * 4));
  int split = 1;
  const int64_t want = int64_t(sm_count_b()) * 3;
  while (split * 2 <= max_split && split < 8 && tiles * split < want && total_iters / (split * 2) >= 8) split *= 2;
  a.iters_per_split = int(ceil_div64(total_iters, split));
  if (tiles > 0x7fffffff) return HB200_ERR_UNSUPPORTED;

  auto kernel = nvfp4_gemv_batched_kernel<NT, VEC16>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
    return HB200_ERR_CUDA;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(tiles), unsigned(split), 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = unsigned(split);
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, a) != cudaSuccess) return HB200_ERR_CUDA;
  return HB200_OK;
}

template <int NT>
int dispatch_batched(const BatchedArgs& a, cudaStream_t stream) {
  const bool vec16 = (a.k % 32 == 0) && (reinterpret_cast<uintptr_t>(a.w) % 16 == 0);
  return vec16 ? launch_batched<NT, true>(a, stream) : launch_batched<NT, false>(a, stream);
}

}  // namespace

int gemv_bf16in_batch1(const void* w, const void* x, const void* ws, const OutSpec& out, int64_t n, int64_t k,
                       float alpha, cudaStream_t stream);

namespace {
int gemv_dispatch_all(const void* w, const void* x, const void* ws, const OutSpec& out, int64_t n, int64_t k,
                      int64_t batch, float alpha, bool force_mma, cudaStream_t s) {
  if (batch == 1 && !force_mma) return gemv_bf16in_batch1(w, x, ws, out, n, k, alpha, s);
  BatchedArgs a{static_cast<const uint8_t*>(w), static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(ws),
                out, n, k, int(batch), 0, 0, alpha};
  if (batch <= 8) return dispatch_batched<1>(a, s);
  if (batch <= 16) return dispatch_batched<2>(a, s);
  return dispatch_batched<4>(a, s);
}
}  // namespace

}  // namespace hb200

namespace {
int check_gemv_args(const void* w, const void* x, const void* ws, int64_t n, int64_t k, int64_t batch) {
  if (!w || !x || !ws) return HB200_ERR_INVALID_ARGUMENT;
  if (n < 0 || k < 0 || (k % 16) != 0 || batch < 0) return HB200_ERR_INVALID_ARGUMENT;
  if (batch > 32) return HB200_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(w) % 8 || reinterpret_cast<uintptr_t>(x) % 16) return HB200_ERR_INVALID_ARGUMENT;
  return HB200_OK;
}
}  // namespace

extern "C" int hb200_nvfp4_gemv_bf16in(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                                       void* out_bf16, int64_t n, int64_t k, int64_t batch, float alpha,
                                       void* stream) {
  if (!out_bf16) return HB200_ERR_INVALID_ARGUMENT;
  const int rc = check_gemv_args(weight_packed, x_bf16, weight_scale, n, k, batch);
  if (rc != HB200_OK) return rc;
  if (n == 0 || batch == 0) return HB200_OK;
  hb200::OutSpec o{};
  o.ptr[0] = static_cast<__nv_bfloat16*>(out_bf16);
  o.count = 1;
  o.ld = n;
  return hb200::gemv_dispatch_all(weight_packed, x_bf16, weight_scale, o, n, k, batch, alpha, false,
                                  static_cast<cudaStream_t>(stream));
}

// Same arithmetic as the batched kernel for a single activation row (fp32
// accumulation inside the MMA); used to cross-check the SIMT GEMV.
extern "C" int hb200_nvfp4_gemv_bf16in_mma(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                                           void* out_bf16, int64_t n, int64_t k, int64_t batch, float alpha,
                                           void* stream) {
  if (!out_bf16 || batch < 1) return HB200_ERR_INVALID_ARGUMENT;
  const int rc = check_gemv_args(weight_packed, x_bf16, weight_scale, n, k, batch);
  if (rc != HB200_OK) return rc;
  if (n == 0) return HB200_OK;
  hb200::OutSpec o{};
  o.ptr[0] = static_cast<__nv_bfloat16*>(out_bf16);
  o.count = 1;
  o.ld = n;
  return hb200::gemv_dispatch_all(weight_packed, x_bf16, weight_scale, o, n, k, batch, alpha, true,
                                  static_cast<cudaStream_t>(stream));
}

// Column-parallel form: this rank owns weight rows (output columns) [col0, col0 + n) of n_total and writes
// its slice of the result into the [batch, n_total] buffer of every rank (out_ptrs[0..world), peer-mapped
// device pointers of a symmetric allocation).  Follow with hb200_peer_barrier before reading the buffer.
extern "C" int hb200_nvfp4_gemv_bf16in_tp(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                                          void* const* out_ptrs, int64_t world, int64_t n, int64_t k, int64_t batch,
                                          int64_t n_total, int64_t col0, float alpha, void* stream) {
  if (!out_ptrs || world < 1 || world > 8 || col0 < 0 || col0 + n > n_total) return HB200_ERR_INVALID_ARGUMENT;
  const int rc = check_gemv_args(weight_packed, x_bf16, weight_scale, n, k, batch);
  if (rc != HB200_OK) return rc;
  if (n == 0 || batch == 0) return HB200_OK;
  hb200::OutSpec o{};
  for (int i = 0; i < world; ++i) {
    if (!out_ptrs[i]) return HB200_ERR_INVALID_ARGUMENT;
    o.ptr[i] = static_cast<__nv_bfloat16*>(out_ptrs[i]);
  }
  o.count = int(world);
  o.ld = n_total;
  o.col0 = col0;
  return hb200::gemv_dispatch_all(weight_packed, x_bf16, weight_scale, o, n, k, batch, alpha, false,
                                  static_cast<cudaStream_t>(stream));
}

// Row-parallel form with a fused reduce-scatter: this rank holds the K shard [N, K_local] of the weight and the
// matching columns of the activations, computes its fp32 partial of all N outputs and stores the partial of output
// column c into the buffer of the rank that owns it (c / (n / world)), at [this rank, row, c % (n / world)] of that
// rank's fp32 [world, batch, n / world] buffer (partial_ptrs[i] = rank i's buffer as mapped here).  After
// hb200_peer_barrier every rank adds up the world partials of its own columns with hb200_tp_reduce_partials.  Peer
// memory is only stored to.  The pattern of examples/distributed/matmul_reduce_scatter.py:36-120 (which exchanges
// through loads of the peers' buffers instead).  n % world == 0; runs on the SIMT (one row) / warp-MMA kernels.
extern "C" int hb200_nvfp4_gemv_bf16in_rs(const void* weight_packed, const void* x_bf16, const void* weight_scale,
                                          void* const* partial_ptrs, int64_t world, int64_t rank, int64_t n,
                                          int64_t k_local, int64_t batch, float alpha, void* stream) {
  if (!partial_ptrs || world < 1 || world > 8 || rank < 0 || rank >= world) return HB200_ERR_INVALID_ARGUMENT;
  const int rc = check_gemv_args(weight_packed, x_bf16, weight_scale, n, k_local, batch);
  if (rc != HB200_OK) return rc;
  if (n % world) return HB200_ERR_INVALID_ARGUMENT;
  if (n == 0 || batch == 0) return HB200_OK;
  hb200::OutSpec o{};
  for (int i = 0; i < world; ++i) {
    if (!partial_ptrs[i] || reinterpret_cast<uintptr_t>(partial_ptrs[i]) % 4) return HB200_ERR_INVALID_ARGUMENT;
    o.ptr[i] = static_cast<__nv_bfloat16*>(partial_ptrs[i]);
  }
  o.count = int(world);
  o.scatter_rows = n / world;
  o.src_rank = int(rank);
  o.batch_cap = int(batch);
  return hb200::gemv_dispatch_all(weight_packed, x_bf16, weight_scale, o, n, k_local, batch, alpha, false,
                                  static_cast<cudaStream_t>(stream));
}
