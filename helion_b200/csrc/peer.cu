// Barrier between the ranks of a tensor-parallel group, as a kernel on the caller's stream.
//
// Every rank owns a small flag array in a symmetric allocation (flags[i] is written by rank i only).  A call
// takes the next epoch from a counter in this rank's own memory, publishes it into flags[rank] of every rank
// with a system-scope release store, and waits (system-scope acquire loads) until every entry of its own
// array has reached that epoch.  Stores that kernels earlier on the stream made to peer buffers are ordered
// before the release by a system-scope fence, so after the barrier every rank may read what the others
// pushed into its buffer.  All ranks must call it the same number of times; the kernel keeps no host state,
// so a CUDA graph that contains it can be replayed.
//
// The wait is bounded (about two seconds of SM clock unless hb200_set_wait_budget_cycles changed it): on expiry the kernel records a sticky
// HB200_ERR_DEVICE_TIMEOUT, readable through hb200_device_status, and returns.
#include "common.cuh"

namespace hb200 {

__device__ int g_device_status_peer = 0;

namespace {

struct BarrierArgs {
  uint32_t* flags[8];  // flags[i]: rank i's array, as mapped into this process
  uint32_t* epoch;     // this rank's counter (local memory)
  int rank, world;
};

__device__ long long g_peer_wait_cycles = 4000000000ll;  // settable: hb200_set_wait_budget_cycles

__global__ void peer_barrier_kernel(const BarrierArgs a) {
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) {
    epoch_s = *a.epoch + 1;
    *a.epoch = epoch_s;
  }
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const int peer = threadIdx.x;
  if (peer >= a.world) return;
  __threadfence_system();
  uint32_t* remote = a.flags[peer] + a.rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" : : "l"(remote), "r"(epoch) : "memory");
  const uint32_t* mine = a.flags[a.rank] + peer;
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (int32_t(v - epoch) >= 0) break;
    if (clock64() - t0 > *const_cast<volatile long long*>(&g_peer_wait_cycles)) {
      atomicMin(&g_device_status_peer, HB200_ERR_DEVICE_TIMEOUT);
      break;
    }
    __nanosleep(64);
  }
}

}  // namespace

int peer_device_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status_peer, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  if (reset && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_device_status_peer, &zero, sizeof(int)) != cudaSuccess) return HB200_ERR_CUDA;
  }
  return v;
}

// out[b, c] = bf16(sum over ranks, ascending, of partials[rank, b, c]) in fp32.
__global__ void __launch_bounds__(256)
tp_reduce_partials_kernel(const float* __restrict__ partials, __nv_bfloat16* __restrict__ out, int world, int64_t items,
                          int64_t cols, int64_t ld_out) {
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < items; i += int64_t(gridDim.x) * blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < world; ++r) s += partials[int64_t(r) * items + i];
    const int64_t b = i / cols;
    out[b * ld_out + (i - b * cols)] = __float2bfloat16_rn(s);
  }
}

int peer_set_wait_budget(long long cycles) {
  return cudaMemcpyToSymbol(g_peer_wait_cycles, &cycles, sizeof(cycles)) == cudaSuccess ? HB200_OK : HB200_ERR_CUDA;
}

}  // namespace hb200

extern "C" int hb200_peer_barrier(void* const* flag_ptrs, int64_t world, int64_t rank, void* epoch_counter,
                                  void* stream) {
  if (!flag_ptrs || !epoch_counter || world < 1 || world > 8 || rank < 0 || rank >= world)
    return HB200_ERR_INVALID_ARGUMENT;
  hb200::BarrierArgs a{};
  for (int i = 0; i < world; ++i) {
    if (!flag_ptrs[i] || reinterpret_cast<uintptr_t>(flag_ptrs[i]) % 4) return HB200_ERR_INVALID_ARGUMENT;
    a.flags[i] = static_cast<uint32_t*>(flag_ptrs[i]);
  }
  a.epoch = static_cast<uint32_t*>(epoch_counter);
  a.rank = int(rank);
  a.world = int(world);
  hb200::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return hb200::launch_status();
}

// Second half of the fused reduce-scatter (after hb200_nvfp4_gemv_bf16in_rs and hb200_peer_barrier): adds the `world`
// fp32 partials [world, batch, cols] that the ranks stored into this rank's buffer, in rank order, and writes
// bf16 out[batch, cols] (row pitch ld_out elements).  The sum order is fixed, so results do not depend on timing.
extern "C" int hb200_tp_reduce_partials(const void* partials_f32, void* out_bf16, int64_t world, int64_t batch,
                                        int64_t cols, int64_t ld_out, void* stream) {
  if (!partials_f32 || !out_bf16 || world < 1 || world > 8 || batch < 0 || cols < 0 || ld_out < cols)
    return HB200_ERR_INVALID_ARGUMENT;
  const int64_t items = batch * cols;
  if (items == 0) return HB200_OK;
  const int64_t need = (items + 255) / 256;
  const int grid = int(need < 1184 ? need : 1184);
  hb200::tp_reduce_partials_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(partials_f32), static_cast<__nv_bfloat16*>(out_bf16), int(world), items, cols, ld_out);
  return hb200::launch_status();
}
