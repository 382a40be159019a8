// Expert-parallel bookkeeping for the NVFP4 MoE layer: the device-side tile
// schedule of the grouped GEMM (no host read of the routing result) and the
// routing-weighted combine.
#include "common.cuh"

namespace hb200 {
namespace {

// One CTA.  counts[e] tokens were routed to expert e; sorted_pairs lists the
// (token, slot) pairs (pair = token * top_k + slot) ordered by expert, stably.
//   padded_offsets[e] : first row of expert e when every expert is padded to 128 rows
//   tile_info[t]      : (expert, valid rows) of 128-row tile t, (-1, 0) past the end
//   row_of_sorted[p]  : padded row of sorted position p
//   row_of_pair[pair] : padded row of a (token, slot) pair
__global__ void __launch_bounds__(1024)
moe_schedule_kernel(const int32_t* __restrict__ counts, int experts, int32_t* __restrict__ padded_offsets,
                    int2* __restrict__ tile_info, int max_tiles, int pad_rows) {
  extern __shared__ int32_t sh[];  // offsets[experts + 1], padded[experts + 1]
  int32_t* off = sh;
  int32_t* pad = sh + experts + 1;
  if (threadIdx.x == 0) {
    int32_t o = 0, p = 0;
    for (int e = 0; e < experts; ++e) {
      off[e] = o;
      pad[e] = p;
      const int32_t c = max(counts[e], 0);
      o += c;
      p += (c + pad_rows - 1) / pad_rows * pad_rows;
    }
    off[experts] = o;
    pad[experts] = p;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) padded_offsets[e] = pad[e];
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int32_t row0 = t * 128;
    int2 info = make_int2(-1, 0);
    if (row0 < pad[experts]) {
      int lo = 0, hi = experts;  // last e with pad[e] <= row0
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pad[mid] <= row0) lo = mid; else hi = mid;
      }
      const int32_t cnt = off[lo + 1] - off[lo];
      info = make_int2(lo, max(0, min(128, cnt - (row0 - pad[lo]))));  // 0: a padding-only tile of the group
    }
    tile_info[t] = info;
  }
}

// Padded row of every sorted position / pair; every CTA rebuilds the two offset tables from the counts.
__global__ void __launch_bounds__(256)
moe_row_map_kernel(const int32_t* __restrict__ counts, int experts, const int32_t* __restrict__ sorted_pairs,
                   int pairs, int32_t* __restrict__ row_of_sorted, int32_t* __restrict__ row_of_pair, int pad_rows) {
  extern __shared__ int32_t sh[];
  int32_t* off = sh;
  int32_t* pad = sh + experts + 1;
  if (threadIdx.x == 0) {
    int32_t o = 0, q = 0;
    for (int e = 0; e < experts; ++e) {
      off[e] = o;
      pad[e] = q;
      const int32_t c = max(counts[e], 0);
      o += c;
      q += (c + pad_rows - 1) / pad_rows * pad_rows;
    }
    off[experts] = o;
    pad[experts] = q;
  }
  __syncthreads();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= pairs) return;
  if (p >= off[experts]) {  // the sorted list is shorter than `pairs` when entries were dropped (expert id out of range)
    row_of_sorted[p] = -1;
    return;
  }
  int lo = 0, hi = experts;  // last e with off[e] <= p (experts with zero tokens share an offset)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (off[mid] <= p) lo = mid; else hi = mid;
  }
  const int32_t row = pad[lo] + (p - off[lo]);
  row_of_sorted[p] = row;
  row_of_pair[sorted_pairs[p]] = row;
}

// ---- stable counting sort of the (token, slot) pairs by expert: three small launches instead of a radix sort.
constexpr int kSortThreads = 1024;

// Pass 1: every CTA counts the experts of its 1024 pairs.  block_hist is [blocks][experts].
template <typename IdxT>
__global__ void __launch_bounds__(kSortThreads)
moe_sort_hist_kernel(const IdxT* __restrict__ expert_of_pair, int pairs, int experts, int32_t* __restrict__ block_hist) {
  extern __shared__ int32_t hist[];
  for (int e = threadIdx.x; e < experts; e += kSortThreads) hist[e] = 0;
  __syncthreads();
  const int p = blockIdx.x * kSortThreads + threadIdx.x;
  if (p < pairs) {
    const int e = int(expert_of_pair[p]);
    if (e >= 0 && e < experts) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += kSortThreads) block_hist[blockIdx.x * experts + e] = hist[e];
}

// Pass 2 (one CTA): counts per expert, and block_hist turned in place into the first sorted position of every
// (block, expert) bucket: expert-major, block-minor, which is what makes the sort stable.
__global__ void __launch_bounds__(kSortThreads)
moe_sort_scan_kernel(int32_t* __restrict__ block_hist, int blocks, int experts, int32_t* __restrict__ counts) {
  extern __shared__ int32_t base[];  // [experts + 1]
  for (int e = threadIdx.x; e < experts; e += kSortThreads) {
    int32_t c = 0;
    for (int b = 0; b < blocks; ++b) c += block_hist[b * experts + e];
    counts[e] = c;
    base[e + 1] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    base[0] = 0;
    for (int e = 0; e < experts; ++e) base[e + 1] += base[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += kSortThreads) {
    int32_t run = base[e];
    for (int b = 0; b < blocks; ++b) {
      const int32_t c = block_hist[b * experts + e];
      block_hist[b * experts + e] = run;
      run += c;
    }
  }
}

// Pass 3: a pair's rank inside its (block, expert) bucket is the number of earlier threads of the block with
// the same expert: lanes before it in the warp (match + popc) plus the same expert's totals of the warps before.
template <typename IdxT>
__global__ void __launch_bounds__(kSortThreads)
moe_sort_scatter_kernel(const IdxT* __restrict__ expert_of_pair, int pairs, int experts,
                        const int32_t* __restrict__ bucket_start, int32_t* __restrict__ sorted_pairs) {
  extern __shared__ int32_t warp_cnt[];  // [32 warps][experts]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * experts; i += kSortThreads) warp_cnt[i] = 0;
  __syncthreads();
  const int p = blockIdx.x * kSortThreads + threadIdx.x;
  int e = -1;
  if (p < pairs) {
    e = int(expert_of_pair[p]);
    if (e < 0 || e >= experts) e = -1;
  }
  const unsigned same = __match_any_sync(0xffffffffu, e);
  const int before = __popc(same & ((1u << lane) - 1u));
  if (e >= 0 && before == 0) warp_cnt[warp * experts + e] = __popc(same);  // one writer per (warp, expert)
  __syncthreads();
  if (e >= 0) {
    int rank = before;
    for (int w = 0; w < warp; ++w) rank += warp_cnt[w * experts + e];
    sorted_pairs[bucket_start[blockIdx.x * experts + e] + rank] = p;
  }
}

// Copies quantised token rows into the expert-sorted padded layout: codes [*, k/2], the row's scale bytes
// (re-swizzled for the destination row) and its global scale.  A warp per destination row.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint8_t* __restrict__ codes_in, const uint8_t* __restrict__ scales_in,
                       const float* __restrict__ g_in, uint8_t* __restrict__ codes_out,
                       uint8_t* __restrict__ scales_out, float* __restrict__ g_out,
                       const int32_t* __restrict__ src_pair, int src_div, const int32_t* __restrict__ dst_row,
                       int64_t items, int64_t k) {
  const int64_t item = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const int64_t src = int64_t(src_pair[item]) / src_div, dst = dst_row[item];
  const int64_t k_bytes = k >> 1, col_tiles = ((k >> 4) + 3) >> 2;
  const uint4* ci = reinterpret_cast<const uint4*>(codes_in + src * k_bytes);
  uint4* co = reinterpret_cast<uint4*>(codes_out + dst * k_bytes);
  for (int64_t c = lane; c < (k_bytes >> 4); c += 32) co[c] = ci[c];
  // the four scales of a row inside one column tile are one aligned 32-bit word
  const int64_t so = (src >> 7) * col_tiles * 512 + (src & 31) * 16 + ((src & 127) >> 5) * 4;
  const int64_t d_o = (dst >> 7) * col_tiles * 512 + (dst & 31) * 16 + ((dst & 127) >> 5) * 4;
  for (int64_t t = lane; t < col_tiles; t += 32)
    *reinterpret_cast<uint32_t*>(scales_out + d_o + t * 512) = *reinterpret_cast<const uint32_t*>(scales_in + so + t * 512);
  if (lane == 0) g_out[dst] = g_in[src];
}

// out[t, :] = bf16(sum over the token's top_k slots, in slot order, of w * o[row_of_pair[t*top_k + s], :]) in fp32,
// w = pair_weight[t*top_k + s] or 1.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ o, int64_t ldo, const int32_t* __restrict__ row_of_pair,
                   const float* __restrict__ pair_weight, __nv_bfloat16* __restrict__ out, int64_t tokens, int top_k,
                   int64_t hidden) {
  const int64_t chunks = hidden >> 3;
  const int64_t total = tokens * chunks;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t t = total <= 0x7fffffff ? int64_t(uint32_t(i) / uint32_t(chunks)) : i / chunks, c = i - t * chunks;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < top_k; ++s) {
      const int64_t row = row_of_pair[t * top_k + s];
      const float pw = pair_weight ? pair_weight[t * top_k + s] : 1.0f;
      const uint4 v = ldg_stream_u4(o + row * ldo + c * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] = fmaf(pw, __uint_as_float(w[e] << 16), acc[2 * e]);
        acc[2 * e + 1] = fmaf(pw, __uint_as_float(w[e] & 0xffff0000u), acc[2 * e + 1]);
      }
    }
    uint32_t p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      p[e] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + t * hidden + c * 8) = make_uint4(p[0], p[1], p[2], p[3]);
  }
}

// ------------------------------------------------------------------ routing
// softmax over the experts (fp32: exp(x - max) / sum) followed by top-k, one warp per token; lane l holds experts
// l, l + 32, ...  The k winners come out in descending order, equal values by ascending expert index.
template <typename T, int VPL>
__global__ void __launch_bounds__(256) moe_route_top_k_kernel(const T* __restrict__ logits, int64_t tokens, int experts,
                                                              int top_k, float* __restrict__ weights,
                                                              int64_t* __restrict__ chosen) {
  const int lane = threadIdx.x & 31;
  const int64_t token = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (token >= tokens) return;
  const T* row = logits + token * experts;
  float v[VPL];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < experts ? float(row[e]) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    v[j] = lane + 32 * j < experts ? expf(v[j] - mx) : 0.f;
    sum += v[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
  for (int j = 0; j < VPL; ++j) v[j] = lane + 32 * j < experts ? __fdiv_rn(v[j], sum) : -1.f;  // -1: never chosen

  float my_w = 0.f;
  int my_e = 0;
  for (int r = 0; r < top_k; ++r) {
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      if (v[j] > best) {  // ascending j = ascending expert index: the first maximum stays
        best = v[j];
        best_e = lane + 32 * j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int j = 0; j < VPL; ++j)
        if (lane + 32 * j == best_e) v[j] = -1.f;
    }
    if (lane == (r & 31)) {
      my_w = best;
      my_e = best_e;
    }
    if ((r & 31) == 31 || r == top_k - 1) {  // lanes 0..(r % 32) hold results r - r % 32 ... r
      if (lane <= (r & 31)) {
        const int64_t o = token * top_k + (r - (r & 31)) + lane;
        weights[o] = my_w;
        chosen[o] = my_e;
      }
    }
  }
}

template <typename T>
int launch_route(const void* logits, int64_t tokens, int experts, int top_k, float* weights, int64_t* chosen,
                 cudaStream_t s) {
  const int64_t threads = tokens * 32;
  const int grid = int((threads + 255) / 256);
  const T* in = static_cast<const T*>(logits);
#define HB200_ROUTE(V) moe_route_top_k_kernel<T, V><<<grid, 256, 0, s>>>(in, tokens, experts, top_k, weights, chosen)
  if (experts <= 32) HB200_ROUTE(1);
  else if (experts <= 64) HB200_ROUTE(2);
  else if (experts <= 128) HB200_ROUTE(4);
  else if (experts <= 256) HB200_ROUTE(8);
  else if (experts <= 512) HB200_ROUTE(16);
  else HB200_ROUTE(32);
#undef HB200_ROUTE
  return launch_status();
}

}  // namespace
}  // namespace hb200

// Device-side replacement for the host bookkeeping of
// moe_matmul_ogs_helion_kernel_args_gen (examples/moe_matmul_ogs.py:89-124), which
// reads max_T_per_expert back to the host; nothing here synchronises.
namespace {
int build_schedule(const int32_t* counts, int64_t experts, const int32_t* sorted_pairs, int64_t pairs,
                   int32_t* padded_offsets, int32_t* tile_info, int64_t max_tiles, int32_t* row_of_sorted,
                   int32_t* row_of_pair, int pad_rows, void* stream) {
  using namespace hb200;
  if (!counts || !sorted_pairs || !padded_offsets || !tile_info || !row_of_sorted || !row_of_pair)
    return HB200_ERR_INVALID_ARGUMENT;
  if (experts <= 0 || experts > 4096 || pairs < 0 || max_tiles < 0 || pairs > 0x7fffff00 || max_tiles > 0xffffff)
    return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(tile_info) % 8) return HB200_ERR_INVALID_ARGUMENT;
  const size_t smem = size_t(2 * (experts + 1)) * sizeof(int32_t);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  moe_schedule_kernel<<<1, 1024, smem, s>>>(counts, int(experts), padded_offsets, reinterpret_cast<int2*>(tile_info),
                                           int(max_tiles), pad_rows);
  if (launch_status() != HB200_OK) return HB200_ERR_CUDA;
  if (pairs > 0)
    moe_row_map_kernel<<<unsigned(ceil_div64(pairs, 256)), 256, smem, s>>>(counts, int(experts), sorted_pairs,
                                                                          int(pairs), row_of_sorted, row_of_pair, pad_rows);
  return launch_status();
}
}  // namespace

extern "C" int hb200_moe_build_schedule(const int32_t* counts, int64_t experts, const int32_t* sorted_pairs,
                                        int64_t pairs, int32_t* padded_offsets, int32_t* tile_info,
                                        int64_t max_tiles, int32_t* row_of_sorted, int32_t* row_of_pair,
                                        void* stream) {
  return build_schedule(counts, experts, sorted_pairs, pairs, padded_offsets, tile_info, max_tiles, row_of_sorted,
                        row_of_pair, 128, stream);
}

// The same schedule with every expert padded to a multiple of 256 rows, for the CTA-pair grouped GEMM whose
// tiles are 256 rows: tile_info still has one entry per 128 rows (entries 2j and 2j+1 belong to one expert;
// the second may have 0 valid rows).  max_tiles >= ceil(pairs / 128) + 2 * experts always suffices.
extern "C" int hb200_moe_build_schedule_256(const int32_t* counts, int64_t experts, const int32_t* sorted_pairs,
                                            int64_t pairs, int32_t* padded_offsets, int32_t* tile_info,
                                            int64_t max_tiles, int32_t* row_of_sorted, int32_t* row_of_pair,
                                            void* stream) {
  if ((max_tiles % 2) != 0) return HB200_ERR_INVALID_ARGUMENT;
  return build_schedule(counts, experts, sorted_pairs, pairs, padded_offsets, tile_info, max_tiles, row_of_sorted,
                        row_of_pair, 256, stream);
}

// Copies per-token NVFP4 rows (codes, swizzled scales, global scale) into the expert-sorted padded layout:
// item i reads token src_pair[i] / src_div and writes row dst_row[i].  No reference counterpart.
extern "C" int hb200_moe_gather_rows(const void* codes_in, const void* scales_in, const float* g_in, void* codes_out,
                                     void* scales_out, float* g_out, const int32_t* src_pair, int src_div,
                                     const int32_t* dst_row, int64_t items, int64_t k, void* stream) {
  using namespace hb200;
  if (!codes_in || !scales_in || !g_in || !codes_out || !scales_out || !g_out || !src_pair || !dst_row)
    return HB200_ERR_INVALID_ARGUMENT;
  if (items < 0 || k <= 0 || (k % 32) != 0 || src_div <= 0) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(codes_in) % 16 || reinterpret_cast<uintptr_t>(codes_out) % 16 ||
      reinterpret_cast<uintptr_t>(scales_in) % 4 || reinterpret_cast<uintptr_t>(scales_out) % 4)
    return HB200_ERR_INVALID_ARGUMENT;
  if (items == 0) return HB200_OK;
  moe_gather_rows_kernel<<<unsigned(ceil_div64(items, 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(codes_in), static_cast<const uint8_t*>(scales_in), g_in,
      static_cast<uint8_t*>(codes_out), static_cast<uint8_t*>(scales_out), g_out, src_pair, src_div, dst_row, items, k);
  return launch_status();
}

// Routing-weighted combine of the expert outputs (the weights were folded into
// the rows by the down-projection's epilogue).  No reference counterpart.
extern "C" int hb200_moe_combine(const void* expert_out_bf16, int64_t ld, const int32_t* row_of_pair,
                                 const float* pair_weight, void* out_bf16, int64_t tokens, int64_t top_k,
                                 int64_t hidden, void* stream) {
  using namespace hb200;
  if (!expert_out_bf16 || !row_of_pair || !out_bf16) return HB200_ERR_INVALID_ARGUMENT;
  if (tokens < 0 || top_k <= 0 || hidden < 0 || (hidden % 8) != 0 || ld < hidden || (ld % 8) != 0)
    return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(expert_out_bf16) % 16 || reinterpret_cast<uintptr_t>(out_bf16) % 16)
    return HB200_ERR_INVALID_ARGUMENT;
  if (tokens == 0 || hidden == 0) return HB200_OK;
  const int64_t items = tokens * hidden / 8;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t need = ceil_div64(items, 256);
  const int grid = int(need < int64_t(sms) * 8 ? need : int64_t(sms) * 8);
  moe_combine_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(expert_out_bf16), ld, row_of_pair, pair_weight,
      static_cast<__nv_bfloat16*>(out_bf16), tokens, int(top_k), hidden);
  return launch_status();
}

// Stable sort of the (token, slot) pairs by expert and the per-expert counts, replacing the argsort and the
// bincount of moe_matmul_ogs_helion_kernel_args_gen (examples/moe_matmul_ogs.py:96-117) without a host read.
// expert_of_pair: int64 (idx_is_i64 != 0, what torch.topk returns) or int32, one entry per pair; entries outside
// [0, experts) are dropped.  scratch: at least ceil(pairs / 1024) * experts int32.  experts <= 1024.
extern "C" int hb200_moe_sort_pairs(const void* expert_of_pair, int idx_is_i64, int64_t pairs, int64_t experts,
                                    int32_t* sorted_pairs, int32_t* counts, int32_t* scratch, void* stream) {
  using namespace hb200;
  if (pairs < 0 || experts <= 0 || !counts) return HB200_ERR_INVALID_ARGUMENT;
  if (pairs > 0 && (!expert_of_pair || !sorted_pairs || !scratch)) return HB200_ERR_INVALID_ARGUMENT;
  if (experts > 1024 || pairs > 0x7fffffff) return HB200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = int(ceil_div64(pairs, kSortThreads));
  const int e = int(experts), np = int(pairs);
  if (blocks == 0) {
    return cudaMemsetAsync(counts, 0, size_t(e) * 4, s) == cudaSuccess ? HB200_OK : HB200_ERR_CUDA;
  }
  const size_t scatter_smem = size_t(32) * e * 4;
  if (idx_is_i64) {
    auto scatter = moe_sort_scatter_kernel<long long>;
    if (scatter_smem > 48 * 1024 &&
        cudaFuncSetAttribute(scatter, cudaFuncAttributeMaxDynamicSharedMemorySize, int(scatter_smem)) != cudaSuccess)
      return HB200_ERR_CUDA;
    moe_sort_hist_kernel<long long><<<blocks, kSortThreads, size_t(e) * 4, s>>>(
        static_cast<const long long*>(expert_of_pair), np, e, scratch);
    moe_sort_scan_kernel<<<1, kSortThreads, size_t(e + 1) * 4, s>>>(scratch, blocks, e, counts);
    scatter<<<blocks, kSortThreads, scatter_smem, s>>>(static_cast<const long long*>(expert_of_pair), np, e, scratch,
                                                       sorted_pairs);
  } else {
    auto scatter = moe_sort_scatter_kernel<int32_t>;
    if (scatter_smem > 48 * 1024 &&
        cudaFuncSetAttribute(scatter, cudaFuncAttributeMaxDynamicSharedMemorySize, int(scatter_smem)) != cudaSuccess)
      return HB200_ERR_CUDA;
    moe_sort_hist_kernel<int32_t><<<blocks, kSortThreads, size_t(e) * 4, s>>>(
        static_cast<const int32_t*>(expert_of_pair), np, e, scratch);
    moe_sort_scan_kernel<<<1, kSortThreads, size_t(e + 1) * 4, s>>>(scratch, blocks, e, counts);
    scatter<<<blocks, kSortThreads, scatter_smem, s>>>(static_cast<const int32_t*>(expert_of_pair), np, e, scratch,
                                                       sorted_pairs);
  }
  return launch_status();
}

extern "C" int hb200_moe_route_top_k(const void* logits, int logits_dtype, int64_t tokens, int64_t experts,
                                     int64_t top_k, float* weights, int64_t* chosen, void* stream) {
  using namespace hb200;
  if (tokens < 0 || experts <= 0 || experts > 1024 || top_k <= 0 || top_k > experts) return HB200_ERR_INVALID_ARGUMENT;
  if (logits_dtype < 0 || logits_dtype > 2) return HB200_ERR_INVALID_ARGUMENT;
  if (tokens == 0) return HB200_OK;
  if (!logits || !weights || !chosen) return HB200_ERR_INVALID_ARGUMENT;
  if (tokens > (int64_t(1) << 31)) return HB200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (logits_dtype == 0) return launch_route<__nv_bfloat16>(logits, tokens, int(experts), int(top_k), weights, chosen, s);
  if (logits_dtype == 1) return launch_route<__half>(logits, tokens, int(experts), int(top_k), weights, chosen, s);
  return launch_route<float>(logits, tokens, int(experts), int(top_k), weights, chosen, s);
}
