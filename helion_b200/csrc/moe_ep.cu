// Expert-parallel exchange of the NVFP4 MoE layer over peer memory: one process per GPU, rank r owns experts
// [r E/W, (r+1) E/W) and T tokens of its own.  A step is
//   dispatch : every rank pushes, for each of its (token, slot) pairs, the token's NVFP4 row (packed codes, its
//              block scales, its global scale), the pair's local expert id and routing weight into the receive
//              area of the rank that owns the expert, at slot [source][i]; the pair counts and a [T, top_k] table
//              of where every pair went follow                                              (then a peer barrier)
//   experts  : the owning rank sorts what arrived by expert, runs the two grouped GEMMs with SiLU-mul between them,
//   return   : sums, per (source rank, token), the routing-weighted bf16 output rows of that token's pairs in fp32
//              (slot order) and pushes ONE row per (token, expert rank) back to the source: fp16 values times a
//              power-of-two row scale that travels with them (11 significant bits at the bytes of bf16, so the
//              per-rank partial sums add at most 2^-12 of relative error each)            (peer barrier)
//   combine  : the source adds the rows it got from the ranks its token used, in rank order, in fp32.
// Everything that crosses NVLink is a plain store from the sending rank's kernel into the receiver's symmetric
// buffer; nothing is loaded from peer memory, nothing is multicast, no count is read on the host: the receive
// areas have a capacity that follows from the shapes alone (T * min(top_k, E/W) pairs per source).
//
// The reference has no expert-parallel operator; the pattern (push to peers, then a signal-pad barrier) is the
// one of its distributed examples (examples/distributed/all_gather_matmul.py:36-87).
#include "common.cuh"

namespace hb200 {
namespace {

struct EpShape {
  int world, rank;
  int tokens;   // T: tokens per rank
  int hidden;   // H
  int top_k;
  int experts;  // E (global)
  int e_local;  // E / world
  int cap;      // pairs one source can send to one destination: T * min(top_k, e_local)
};

// Byte offsets of the regions inside one rank's symmetric buffer.
struct EpLayout {
  int64_t codes, sf, meta, count, table, ret, ret_scale, bytes;
};

__host__ __device__ inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

__host__ __device__ inline EpLayout ep_layout(const EpShape& s) {
  EpLayout l;
  int64_t off = 0;
  l.codes = off; off = align_up(off + int64_t(s.world) * s.cap * (s.hidden / 2), 256);
  l.sf = off;    off = align_up(off + int64_t(s.world) * s.cap * (s.hidden / 16), 256);
  l.meta = off;  off = align_up(off + int64_t(s.world) * s.cap * 16, 256);
  l.count = off; off = align_up(off + int64_t(s.world) * 4, 256);
  l.table = off; off = align_up(off + int64_t(s.world) * s.tokens * s.top_k * 4, 256);
  l.ret = off;   off = align_up(off + int64_t(s.world) * s.tokens * s.hidden * 2, 256);
  l.ret_scale = off; off = align_up(off + int64_t(s.world) * s.tokens * 4, 256);
  l.bytes = off;
  return l;
}

struct EpPeers {
  uint8_t* base[8];
};

// ---- dispatch: a warp per sorted (token, slot) pair.  sorted_pairs lists the pairs by global expert (stable), so
// the pairs of destination d are the sorted positions [first[d], first[d + 1]).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint8_t* __restrict__ codes_t, const uint8_t* __restrict__ scales_t,
                   const float* __restrict__ g_t, const float* __restrict__ weights,
                   const int64_t* __restrict__ experts_of_pair, const int32_t* __restrict__ sorted_pairs,
                   const int32_t* __restrict__ counts, int32_t* __restrict__ route_local, const EpPeers peers,
                   const EpShape s, const EpLayout l) {
  __shared__ int32_t first[9];
  if (threadIdx.x == 0) {
    int32_t run = 0;
    for (int d = 0; d < s.world; ++d) {
      first[d] = run;
      for (int e = d * s.e_local; e < (d + 1) * s.e_local; ++e) run += max(counts[e], 0);
    }
    first[s.world] = run;
  }
  __syncthreads();
  const int64_t pairs = int64_t(s.tokens) * s.top_k;
  const int64_t p = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (p == 0 && lane < s.world) {
    // how many pairs this rank sent to rank `lane`
    *reinterpret_cast<int32_t*>(peers.base[lane] + l.count + int64_t(s.rank) * 4) =
        min(first[lane + 1] - first[lane], s.cap);
  }
  if (p >= pairs || p >= first[s.world]) return;  // (pairs whose expert id was out of range are not in the list)
  const int32_t pair = sorted_pairs[p];
  const int64_t e = experts_of_pair[pair];
  const int d = int(e / s.e_local);
  const int32_t idx = int32_t(p) - first[d];
  if (d < 0 || d >= s.world || idx < 0 || idx >= s.cap) return;  // cannot happen for a valid routing result
  const int64_t t = pair / s.top_k;
  const int64_t slot = int64_t(s.rank) * s.cap + idx;
  uint8_t* dst = peers.base[d];
  const int64_t k_bytes = s.hidden >> 1, col_tiles = ((s.hidden >> 4) + 3) >> 2;
  const uint4* ci = reinterpret_cast<const uint4*>(codes_t + t * k_bytes);
  uint4* co = reinterpret_cast<uint4*>(dst + l.codes + slot * k_bytes);
  for (int64_t c = lane; c < (k_bytes >> 4); c += 32) co[c] = ci[c];
  // block scales: the four scales of a row inside one column tile are one aligned 32-bit word of the swizzled
  // source; they go out row-major, one row of hidden / 16 bytes per pair
  const int64_t so = (t >> 7) * col_tiles * 512 + (t & 31) * 16 + ((t & 127) >> 5) * 4;
  uint32_t* sfo = reinterpret_cast<uint32_t*>(dst + l.sf + slot * (s.hidden >> 4));
  for (int64_t j = lane; j < (s.hidden >> 6); j += 32)
    sfo[j] = *reinterpret_cast<const uint32_t*>(scales_t + so + j * 512);
  if (lane == 0) {
    const int4 meta = make_int4(int(e - int64_t(d) * s.e_local), __float_as_int(g_t[t]), __float_as_int(weights[pair]), pair);
    *reinterpret_cast<int4*>(dst + l.meta + slot * 16) = meta;
    route_local[pair] = d * s.cap + idx;
  }
}

// Pushes this rank's [T, top_k] table of where every pair went (destination * cap + index) to every rank.
__global__ void __launch_bounds__(256)
ep_push_table_kernel(const int32_t* __restrict__ route_local, const EpPeers peers, const EpShape s, const EpLayout l) {
  const int64_t n = int64_t(s.tokens) * s.top_k;
  const int d = blockIdx.y;
  int32_t* dst = reinterpret_cast<int32_t*>(peers.base[d] + l.table) + int64_t(s.rank) * n;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    dst[i] = route_local[i];
}

// ---- expert side: the local expert of every receive slot, -1 for slots beyond what the source sent.
__global__ void __launch_bounds__(256)
ep_collect_kernel(const uint8_t* __restrict__ base, int32_t* __restrict__ expert_of_slot, const EpShape s,
                  const EpLayout l) {
  const int64_t n = int64_t(s.world) * s.cap;
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int src = int(i / s.cap);
  const int32_t have = min(max(reinterpret_cast<const int32_t*>(base + l.count)[src], 0), s.cap);
  int32_t e = -1;
  if (i - int64_t(src) * s.cap < have) {
    e = reinterpret_cast<const int4*>(base + l.meta)[i].x;
    if (e < 0 || e >= s.e_local) e = -1;
  }
  expert_of_slot[i] = e;
}

// Copies the received rows into the expert-sorted padded layout of the grouped GEMM: a warp per sorted position.
// sorted_slots[p] is the receive slot at sorted position p, row_of_sorted[p] its padded row (-1 past the end).
__global__ void __launch_bounds__(256)
ep_gather_kernel(const uint8_t* __restrict__ base, const int32_t* __restrict__ sorted_slots,
                 const int32_t* __restrict__ row_of_sorted, uint8_t* __restrict__ codes_out,
                 uint8_t* __restrict__ scales_out, float* __restrict__ g_out, float* __restrict__ w_row,
                 const EpShape s, const EpLayout l) {
  const int64_t n = int64_t(s.world) * s.cap;
  const int64_t p = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (p >= n) return;
  const int64_t dst = row_of_sorted[p];
  if (dst < 0) return;
  const int lane = threadIdx.x & 31;
  const int64_t slot = sorted_slots[p];
  const int64_t k_bytes = s.hidden >> 1, col_tiles = ((s.hidden >> 4) + 3) >> 2;
  const uint4* ci = reinterpret_cast<const uint4*>(base + l.codes + slot * k_bytes);
  uint4* co = reinterpret_cast<uint4*>(codes_out + dst * k_bytes);
  for (int64_t c = lane; c < (k_bytes >> 4); c += 32) co[c] = ci[c];
  const uint32_t* sfi = reinterpret_cast<const uint32_t*>(base + l.sf + slot * (s.hidden >> 4));
  const int64_t d_o = (dst >> 7) * col_tiles * 512 + (dst & 31) * 16 + ((dst & 127) >> 5) * 4;
  for (int64_t j = lane; j < (s.hidden >> 6); j += 32) *reinterpret_cast<uint32_t*>(scales_out + d_o + j * 512) = sfi[j];
  if (lane == 0) {
    const int4 meta = reinterpret_cast<const int4*>(base + l.meta)[slot];
    g_out[dst] = __int_as_float(meta.y);
    w_row[dst] = __int_as_float(meta.z);
  }
}

// ---- return: one CTA per (source rank, token): row = sum over the token's pairs that came to this rank, in slot
// order, of weight * o[row] in fp32; the row goes to the source's return area [this rank][token] as fp16 values
// times 2^e (e from the row's largest magnitude, so that it lands just below the fp16 maximum) with the factor
// beside it.  Rows with no pair here are not written.  hidden <= 8 * 256 * kRetChunks.
constexpr int kRetChunks = 4;  // 8-column chunks per thread: hidden <= 8192

__global__ void __launch_bounds__(256)
ep_return_kernel(const __nv_bfloat16* __restrict__ o, int64_t ldo, const int32_t* __restrict__ row_of_slot,
                 const float* __restrict__ w_row, const EpPeers peers, const uint8_t* __restrict__ base,
                 const EpShape s, const EpLayout l) {
  __shared__ float red[8];
  __shared__ int64_t rows_s[64];
  __shared__ float w_s[64];
  __shared__ int n_rows_s;
  const int64_t st = blockIdx.x;  // source * T + token
  const int src = int(st / s.tokens);
  const int64_t t = st - int64_t(src) * s.tokens;
  if (threadIdx.x == 0) {
    const int32_t* tab = reinterpret_cast<const int32_t*>(base + l.table) + st * s.top_k;
    int n = 0;
    for (int k = 0; k < s.top_k; ++k) {
      const int32_t v = tab[k];
      if (v < 0 || v / s.cap != s.rank) continue;
      const int64_t row = row_of_slot[int64_t(src) * s.cap + (v - s.rank * s.cap)];
      if (row < 0) continue;
      rows_s[n] = row;
      w_s[n] = w_row[row];
      ++n;
    }
    n_rows_s = n;
  }
  __syncthreads();
  const int n_rows = n_rows_s;
  if (n_rows == 0) return;
  const int chunks = s.hidden >> 3;
  float acc[kRetChunks][8];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < kRetChunks; ++j) {
    const int c = threadIdx.x + j * 256;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
    if (c < chunks) {
      for (int r = 0; r < n_rows; ++r) {
        const float pw = w_s[r];
        const uint4 q = ldg_stream_u4(o + rows_s[r] * ldo + c * 8);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[j][2 * e] = fmaf(pw, __uint_as_float(w[e] << 16), acc[j][2 * e]);
          acc[j][2 * e + 1] = fmaf(pw, __uint_as_float(w[e] & 0xffff0000u), acc[j][2 * e + 1]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(acc[j][e]));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  // power of two that brings the largest magnitude into [2^14, 2^15): exact to apply and to undo
  int ex = 0;
  if (amax > 0.f && amax < INFINITY) ex = 14 - (int((__float_as_uint(amax) >> 23) & 0xffu) - 127);
  ex = max(-100, min(100, ex));
  const float up = __uint_as_float(uint32_t(127 + ex) << 23), down = __uint_as_float(uint32_t(127 - ex) << 23);
  uint8_t* dst_base = peers.base[src];
  __half* dst = reinterpret_cast<__half*>(dst_base + l.ret) + (int64_t(s.rank) * s.tokens + t) * s.hidden;
#pragma unroll
  for (int j = 0; j < kRetChunks; ++j) {
    const int c = threadIdx.x + j * 256;
    if (c < chunks) {
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __half2 h = __floats2half2_rn(acc[j][2 * e] * up, acc[j][2 * e + 1] * up);
        pk[e] = *reinterpret_cast<const uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
  if (threadIdx.x == 0)
    reinterpret_cast<float*>(dst_base + l.ret_scale)[int64_t(s.rank) * s.tokens + t] = down;
}

// ---- combine on the source: out[t] = bf16(sum over the ranks the token's pairs went to, ascending, of the row
// that rank returned times its factor), fp32.
__global__ void __launch_bounds__(256)
ep_combine_kernel(const uint8_t* __restrict__ base, const int32_t* __restrict__ route_local,
                  __nv_bfloat16* __restrict__ out, const EpShape s, const EpLayout l) {
  const int64_t chunks = s.hidden >> 3;
  const int64_t total = int64_t(s.tokens) * chunks;
  const __half* ret = reinterpret_cast<const __half*>(base + l.ret);
  const float* ret_scale = reinterpret_cast<const float*>(base + l.ret_scale);
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t t = i / chunks, c = i - t * chunks;
    uint32_t used = 0;
    for (int k = 0; k < s.top_k; ++k) {
      const int32_t v = route_local[t * s.top_k + k];
      if (v >= 0) used |= 1u << (v / s.cap);
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < s.world; ++d) {
      if (!(used >> d & 1u)) continue;
      const float f = ret_scale[int64_t(d) * s.tokens + t];
      const uint4 q = ldg_stream_u4(ret + (int64_t(d) * s.tokens + t) * s.hidden + c * 8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
        acc[2 * e] = fmaf(v2.x, f, acc[2 * e]);
        acc[2 * e + 1] = fmaf(v2.y, f, acc[2 * e + 1]);
      }
    }
    uint32_t pk[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      pk[e] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + t * s.hidden + c * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
}

bool make_shape(int64_t world, int64_t rank, int64_t tokens, int64_t hidden, int64_t top_k, int64_t experts, EpShape* s) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return false;
  if (tokens <= 0 || tokens > (1 << 24) || hidden <= 0 || (hidden % 64) != 0 || hidden > (1 << 20)) return false;
  if (hidden > 8 * 256 * kRetChunks) return false;
  if (top_k <= 0 || top_k > 64 || experts <= 0 || experts > 1024 || (experts % world) != 0 || top_k > experts) return false;
  s->world = int(world);
  s->rank = int(rank);
  s->tokens = int(tokens);
  s->hidden = int(hidden);
  s->top_k = int(top_k);
  s->experts = int(experts);
  s->e_local = int(experts / world);
  const int64_t cap = tokens * (top_k < s->e_local ? top_k : s->e_local);
  if (cap * world > 0x7fffff00) return false;
  s->cap = int(cap);
  return true;
}

bool make_peers(void* const* bases, int world, EpPeers* p) {
  if (!bases) return false;
  for (int i = 0; i < world; ++i) {
    if (!bases[i] || reinterpret_cast<uintptr_t>(bases[i]) % 256) return false;
    p->base[i] = static_cast<uint8_t*>(bases[i]);
  }
  return true;
}

int grid_for(int64_t items, int per_block) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t need = ceil_div64(items, per_block);
  return int(need < int64_t(sms) * 8 ? (need > 0 ? need : 1) : int64_t(sms) * 8);
}

}  // namespace
}  // namespace hb200

// Bytes of the symmetric buffer every rank allocates (zero-filled once) for the expert-parallel exchange, and the
// number of receive slots (world * capacity) an expert rank sorts; negative HB200_ERR_* for shapes it does not take.
// hidden % 64 == 0, experts % world == 0, world <= 8.
extern "C" int64_t hb200_ep_buffer_bytes(int64_t world, int64_t tokens, int64_t hidden, int64_t top_k, int64_t experts) {
  hb200::EpShape s;
  if (!hb200::make_shape(world, 0, tokens, hidden, top_k, experts, &s)) return HB200_ERR_UNSUPPORTED;
  return hb200::ep_layout(s).bytes;
}

extern "C" int64_t hb200_ep_slots(int64_t world, int64_t tokens, int64_t hidden, int64_t top_k, int64_t experts) {
  hb200::EpShape s;
  if (!hb200::make_shape(world, 0, tokens, hidden, top_k, experts, &s)) return HB200_ERR_UNSUPPORTED;
  return int64_t(s.world) * s.cap;
}

// Dispatch: push this rank's quantised token rows to the ranks that own their experts.  codes_t [T, H/2],
// scales_t swizzled for [T, H/16], g_t [T] (hb200_nvfp4_quantize, one global scale per token); weights fp32 and
// experts int64 [T, top_k] (hb200_moe_route_top_k); sorted_pairs / counts from hb200_moe_sort_pairs over the global
// expert ids.  route_local (int32 [T * top_k], this rank's memory) receives destination * capacity + index of every
// pair.  bases[i] = rank i's exchange buffer as mapped here.  Follow with hb200_peer_barrier.
extern "C" int hb200_ep_dispatch(const void* codes_t, const void* scales_t, const float* g_t, const float* weights,
                                 const int64_t* experts_of_pair, const int32_t* sorted_pairs, const int32_t* counts,
                                 int32_t* route_local, void* const* bases, int64_t world, int64_t rank, int64_t tokens,
                                 int64_t hidden, int64_t top_k, int64_t experts, void* stream) {
  using namespace hb200;
  EpShape s;
  EpPeers peers{};
  if (!codes_t || !scales_t || !g_t || !weights || !experts_of_pair || !sorted_pairs || !counts || !route_local)
    return HB200_ERR_INVALID_ARGUMENT;
  if (!make_shape(world, rank, tokens, hidden, top_k, experts, &s)) return HB200_ERR_UNSUPPORTED;
  if (!make_peers(bases, s.world, &peers)) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(codes_t) % 16 || reinterpret_cast<uintptr_t>(scales_t) % 4) return HB200_ERR_INVALID_ARGUMENT;
  const EpLayout l = ep_layout(s);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t pairs = int64_t(s.tokens) * s.top_k;
  if (cudaMemsetAsync(route_local, 0xff, size_t(pairs) * 4, st) != cudaSuccess) return HB200_ERR_CUDA;  // -1: pair not sent
  ep_dispatch_kernel<<<unsigned(ceil_div64(pairs, 8)), 256, 0, st>>>(
      static_cast<const uint8_t*>(codes_t), static_cast<const uint8_t*>(scales_t), g_t, weights, experts_of_pair,
      sorted_pairs, counts, route_local, peers, s, l);
  if (launch_status() != HB200_OK) return HB200_ERR_CUDA;
  ep_push_table_kernel<<<dim3(unsigned(grid_for(pairs, 256) < 64 ? grid_for(pairs, 256) : 64), unsigned(s.world)), 256, 0, st>>>(
      route_local, peers, s, l);
  return launch_status();
}

// Expert side, after the barrier: expert_of_slot (int32 [world * capacity]) gets the local expert of every receive
// slot, -1 where nothing arrived; sort it with hb200_moe_sort_pairs and lay it out with hb200_moe_build_schedule.
extern "C" int hb200_ep_collect(const void* base, int32_t* expert_of_slot, int64_t world, int64_t rank, int64_t tokens,
                                int64_t hidden, int64_t top_k, int64_t experts, void* stream) {
  using namespace hb200;
  EpShape s;
  if (!base || !expert_of_slot) return HB200_ERR_INVALID_ARGUMENT;
  if (!make_shape(world, rank, tokens, hidden, top_k, experts, &s)) return HB200_ERR_UNSUPPORTED;
  const int64_t n = int64_t(s.world) * s.cap;
  ep_collect_kernel<<<unsigned(ceil_div64(n, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(base), expert_of_slot, s, ep_layout(s));
  return launch_status();
}

// Copies the received rows into the padded, expert-sorted operand of the first grouped GEMM (codes [rows, H/2],
// swizzled scales, per-row global scale) and the routing weight of every padded row (w_row).
extern "C" int hb200_ep_gather(const void* base, const int32_t* sorted_slots, const int32_t* row_of_sorted,
                               void* codes_out, void* scales_out, float* g_out, float* w_row, int64_t world,
                               int64_t rank, int64_t tokens, int64_t hidden, int64_t top_k, int64_t experts,
                               void* stream) {
  using namespace hb200;
  EpShape s;
  if (!base || !sorted_slots || !row_of_sorted || !codes_out || !scales_out || !g_out || !w_row)
    return HB200_ERR_INVALID_ARGUMENT;
  if (!make_shape(world, rank, tokens, hidden, top_k, experts, &s)) return HB200_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(codes_out) % 16 || reinterpret_cast<uintptr_t>(scales_out) % 4) return HB200_ERR_INVALID_ARGUMENT;
  const int64_t n = int64_t(s.world) * s.cap;
  ep_gather_kernel<<<unsigned(ceil_div64(n, 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(base), sorted_slots, row_of_sorted, static_cast<uint8_t*>(codes_out),
      static_cast<uint8_t*>(scales_out), g_out, w_row, s, ep_layout(s));
  return launch_status();
}

// Return: o [padded rows, H] bf16 (leading dimension ldo) are the second grouped GEMM's rows, row_of_slot the padded
// row of every receive slot, w_row the routing weight per padded row.  Stores one routing-weighted, pre-reduced
// row (fp16 values and a power-of-two factor) per (source, token) that has pairs here into the source's return
// area.  Follow with hb200_peer_barrier.
extern "C" int hb200_ep_return(const void* o_bf16, int64_t ldo, const int32_t* row_of_slot, const float* w_row,
                               void* const* bases, int64_t world, int64_t rank, int64_t tokens, int64_t hidden,
                               int64_t top_k, int64_t experts, void* stream) {
  using namespace hb200;
  EpShape s;
  EpPeers peers{};
  if (!o_bf16 || !row_of_slot || !w_row || ldo < hidden || (ldo % 8) != 0) return HB200_ERR_INVALID_ARGUMENT;
  if (!make_shape(world, rank, tokens, hidden, top_k, experts, &s)) return HB200_ERR_UNSUPPORTED;
  if (!make_peers(bases, s.world, &peers)) return HB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(o_bf16) % 16) return HB200_ERR_INVALID_ARGUMENT;
  ep_return_kernel<<<unsigned(int64_t(s.world) * s.tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o_bf16), ldo, row_of_slot, w_row, peers, peers.base[s.rank], s, ep_layout(s));
  return launch_status();
}

// Combine on the source rank, after the second barrier: out [T, H] bf16.
extern "C" int hb200_ep_combine(const void* base, const int32_t* route_local, void* out_bf16, int64_t world,
                                int64_t rank, int64_t tokens, int64_t hidden, int64_t top_k, int64_t experts,
                                void* stream) {
  using namespace hb200;
  EpShape s;
  if (!base || !route_local || !out_bf16 || reinterpret_cast<uintptr_t>(out_bf16) % 16) return HB200_ERR_INVALID_ARGUMENT;
  if (!make_shape(world, rank, tokens, hidden, top_k, experts, &s)) return HB200_ERR_UNSUPPORTED;
  const int64_t items = int64_t(s.tokens) * (s.hidden / 8);
  ep_combine_kernel<<<grid_for(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(base), route_local, static_cast<__nv_bfloat16*>(out_bf16), s, ep_layout(s));
  return launch_status();
}
