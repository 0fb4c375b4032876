// Routing bookkeeping: stable counting sort of top-k expert ids, per-expert inclusive offsets.
//
// Replaces torch.sort + bincount + cumsum of the reference's flatten_sort_count
// (scattermoe/parallel_experts.py:14-21). The key range is tiny (E experts), so a counting sort does it in
// two passes over the ids: per-block/per-warp histograms (warp match-any ballots, no atomics), one scan of
// the (expert-major) block histograms, and a stable scatter that recomputes the warp-local ranks.
#include <stdarg.h>

#include <mutex>

#include "smoe_common.cuh"

namespace smoe {

constexpr int SC_THREADS = 256;
constexpr int SC_WARPS = SC_THREADS / 32;
constexpr int SC_ITERS = 8;                        // 32-id steps per warp
constexpr int SC_CHUNK = SC_WARPS * 32 * SC_ITERS;  // ids per block
constexpr int SC_MAX_E = 4096;

// Pass 1 of a block: every warp counts the keys of its own contiguous run of SC_ITERS*32 ids into its
// private row of `whist` (E ints per warp) and keeps the keys in registers.
__device__ __forceinline__ void warp_histogram(const int64_t* __restrict__ ids, int64_t R, int E,
                                               int32_t* __restrict__ my_hist, int64_t warp_base, int lane,
                                               int (&keys)[SC_ITERS]) {
#pragma unroll
  for (int it = 0; it < SC_ITERS; ++it) {
    const int64_t i = warp_base + it * 32 + lane;
    int key = -1;
    if (i < R) {
      const int64_t v = ids[i];
      key = (v >= 0 && v < E) ? static_cast<int>(v) : -1;
    }
    keys[it] = key;
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (key >= 0 && lane == __ffs(peers) - 1) my_hist[key] += __popc(peers);
    __syncwarp();
  }
}

__global__ void __launch_bounds__(SC_THREADS)
sc_hist_kernel(const int64_t* __restrict__ ids, int64_t R, int E, int nblk, int32_t* __restrict__ block_hist) {
  extern __shared__ int32_t whist[];  // [SC_WARPS][E]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < SC_WARPS * E; i += SC_THREADS) whist[i] = 0;
  __syncthreads();
  int keys[SC_ITERS];
  const int64_t warp_base = static_cast<int64_t>(blockIdx.x) * SC_CHUNK + warp * (32 * SC_ITERS);
  warp_histogram(ids, R, E, whist + warp * E, warp_base, lane, keys);
  __syncthreads();
  for (int e = tid; e < E; e += SC_THREADS) {
    int s = 0;
#pragma unroll
    for (int w = 0; w < SC_WARPS; ++w) s += whist[w * E + e];
    block_hist[static_cast<int64_t>(e) * nblk + blockIdx.x] = s;
  }
}

// Exclusive scan, in place, of the expert-major block histograms (L = E*nblk ints) by ONE block, and the
// inclusive per-expert end offsets. Entry [e*nblk + b] becomes the first output position of expert e's
// ids that live in block b.
__global__ void __launch_bounds__(1024)
sc_scan_kernel(int32_t* __restrict__ hist, int L, int E, int nblk, int64_t* __restrict__ expert_offsets) {
  __shared__ int32_t warp_sums[32];
  __shared__ int32_t s_total;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int per = (L + 1023) / 1024;
  const int beg = min(tid * per, L), end = min(beg + per, L);
  int sum = 0;
  for (int i = beg; i < end; ++i) sum += hist[i];
  int inc = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += v;
  }
  if (lane == 31) warp_sums[w] = inc;
  __syncthreads();
  if (w == 0) {
    const int v = warp_sums[lane];
    int winc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += u;
    }
    warp_sums[lane] = winc - v;
    if (lane == 31) s_total = winc;
  }
  __syncthreads();
  int run = warp_sums[w] + inc - sum;
  for (int i = beg; i < end; ++i) {
    const int v = hist[i];
    hist[i] = run;
    run += v;
  }
  __syncthreads();
  for (int e = tid; e < E; e += 1024)
    expert_offsets[e] = (e + 1 < E) ? static_cast<int64_t>(hist[static_cast<int64_t>(e + 1) * nblk])
                                    : static_cast<int64_t>(s_total);
}

__global__ void __launch_bounds__(SC_THREADS)
sc_scatter_kernel(const int64_t* __restrict__ ids, int64_t R, int E, int nblk,
                  const int32_t* __restrict__ block_excl, int64_t* __restrict__ sorted_e,
                  int64_t* __restrict__ sorted_idx) {
  extern __shared__ int32_t whist[];  // [SC_WARPS][E]; counts, then running output positions
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < SC_WARPS * E; i += SC_THREADS) whist[i] = 0;
  __syncthreads();
  int keys[SC_ITERS];
  const int64_t warp_base = static_cast<int64_t>(blockIdx.x) * SC_CHUNK + warp * (32 * SC_ITERS);
  int32_t* my = whist + warp * E;
  warp_histogram(ids, R, E, my, warp_base, lane, keys);
  __syncthreads();
  for (int e = tid; e < E; e += SC_THREADS) {
    int run = block_excl[static_cast<int64_t>(e) * nblk + blockIdx.x];
#pragma unroll
    for (int w = 0; w < SC_WARPS; ++w) {
      const int c = whist[w * E + e];
      whist[w * E + e] = run;
      run += c;
    }
  }
  __syncthreads();
  const unsigned lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int it = 0; it < SC_ITERS; ++it) {
    const int key = keys[it];
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (key >= 0) {
      const int pos = my[key] + __popc(peers & lt_mask);
      sorted_e[pos] = key;
      sorted_idx[pos] = warp_base + it * 32 + lane;
    }
    __syncwarp();
    if (key >= 0 && lane == __ffs(peers) - 1) my[key] += __popc(peers);
    __syncwarp();
  }
}

__global__ void zero_offsets_kernel(int64_t* expert_offsets, int E) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < E) expert_offsets[e] = 0;
}

// Position m (0..R) is the end of every expert e with sorted[m-1] <= e < sorted[m].
__global__ void offsets_from_sorted_kernel(const int64_t* __restrict__ sorted_e, int64_t R, int E,
                                           int64_t* __restrict__ expert_offsets) {
  const int64_t m = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (m > R) return;
  int64_t cur = (m < R) ? sorted_e[m] : E;
  int64_t prev = (m > 0) ? sorted_e[m - 1] : 0;
  cur = cur < 0 ? 0 : (cur > E ? E : cur);
  prev = prev < 0 ? 0 : (prev > E ? E : prev);
  for (int64_t e = prev; e < cur; ++e) expert_offsets[e] = m;
}

// ---- the allocation-free variant ----------------------------------------------------------------------
// Scratch for smoe_sort_count_static: the per-block histograms live in this fixed array instead of a
// caller-provided workspace. Every GPU that loads the library carries these 512 KiB until the process exits.
constexpr int SC_STATIC_INTS = 128 * 1024;
static __device__ __align__(256) int32_t g_sort_scratch[SC_STATIC_INTS];

// Host code cannot pass `g_sort_scratch` to a kernel: in host code that name is a stand-in for the symbol, not
// a device address. The address is looked up once per device, with that device current, and cached.
static int static_scratch_address(int32_t** out) {
  static std::mutex mu;
  static int32_t* cached[64] = {nullptr};
  int dev = 0;
  SMOE_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64 && cached[dev]) {
    *out = cached[dev];
    return SMOE_OK;
  }
  void* ptr = nullptr;
  SMOE_CUDA(cudaGetSymbolAddress(&ptr, g_sort_scratch));
  if (ptr == nullptr) {
    set_error("sort_count_static: cudaGetSymbolAddress returned a null address");
    return SMOE_ERR_CUDA;
  }
  if (dev >= 0 && dev < 64) cached[dev] = static_cast<int32_t*>(ptr);
  *out = static_cast<int32_t*>(ptr);
  return SMOE_OK;
}

}  // namespace smoe

using namespace smoe;

extern "C" size_t smoe_sort_count_workspace_bytes(int64_t R, int32_t E) {
  if (R < 0 || E < 1) return 0;
  const int64_t nblk = cdiv64(R > 0 ? R : 1, SC_CHUNK);
  return static_cast<size_t>(nblk) * static_cast<size_t>(E) * sizeof(int32_t) + 256;
}

// The three launches of the sort. `block_hist` holds ceil(R / SC_CHUNK) * E ints; the caller has checked its size.
static int sort_count_launch(const char* who, const int64_t* expert_idxs, int64_t R, int32_t E,
                             int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, int64_t* expert_offsets,
                             int32_t* block_hist, cudaStream_t stream) {
  SMOE_CHECK_ARG(expert_offsets != nullptr, "%s: expert_offsets is null", who);
  if (R == 0) {
    zero_offsets_kernel<<<cdiv(E, 256), 256, 0, stream>>>(expert_offsets, E);
    SMOE_LAUNCH_CHECK();
    return SMOE_OK;
  }
  SMOE_CHECK_ARG(expert_idxs && sorted_expert_idxs && sorted_scattered_idxs && block_hist, "%s: null pointer", who);
  const int nblk = static_cast<int>(cdiv64(R, SC_CHUNK));
  const size_t smem = static_cast<size_t>(SC_WARPS) * E * sizeof(int32_t);
  if (smem > 48 * 1024) {
    static thread_local int configured_device = -1;
    int dev = 0;
    SMOE_CUDA(cudaGetDevice(&dev));
    if (configured_device != dev) {
      SMOE_CUDA(cudaFuncSetAttribute(sc_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     SC_WARPS * SC_MAX_E * 4));
      SMOE_CUDA(cudaFuncSetAttribute(sc_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     SC_WARPS * SC_MAX_E * 4));
      configured_device = dev;
    }
  }
  sc_hist_kernel<<<nblk, SC_THREADS, smem, stream>>>(expert_idxs, R, E, nblk, block_hist);
  SMOE_LAUNCH_CHECK();
  sc_scan_kernel<<<1, 1024, 0, stream>>>(block_hist, E * nblk, E, nblk, expert_offsets);
  SMOE_LAUNCH_CHECK();
  sc_scatter_kernel<<<nblk, SC_THREADS, smem, stream>>>(expert_idxs, R, E, nblk, block_hist,
                                                        sorted_expert_idxs, sorted_scattered_idxs);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

extern "C" int smoe_sort_count(const int64_t* expert_idxs, int64_t R, int32_t E, int64_t* sorted_expert_idxs,
                               int64_t* sorted_scattered_idxs, int64_t* expert_offsets, void* workspace,
                               size_t workspace_bytes, void* stream_) {
  SMOE_CHECK_ARG(R >= 0 && R < (int64_t(1) << 31), "sort_count: R=%lld out of range [0, 2^31)", (long long)R);
  SMOE_CHECK_ARG(E >= 1 && E <= SC_MAX_E, "sort_count: E=%d out of range [1, %d]", E, SC_MAX_E);
  if (R > 0 && (workspace == nullptr || workspace_bytes < smoe_sort_count_workspace_bytes(R, E))) {
    set_error("sort_count: workspace of %zu bytes needed, %zu given", smoe_sort_count_workspace_bytes(R, E),
              workspace_bytes);
    return SMOE_ERR_WORKSPACE;
  }
  return sort_count_launch("sort_count", expert_idxs, R, E, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
                           static_cast<int32_t*>(workspace), static_cast<cudaStream_t>(stream_));
}

extern "C" int smoe_offsets_from_sorted(const int64_t* sorted_expert_idxs, int64_t R, int32_t E,
                                        int64_t* expert_offsets, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  SMOE_CHECK_ARG(R >= 0 && R < (int64_t(1) << 31), "offsets_from_sorted: R=%lld out of range", (long long)R);
  SMOE_CHECK_ARG(E >= 1, "offsets_from_sorted: E=%d", E);
  SMOE_CHECK_ARG(expert_offsets && (R == 0 || sorted_expert_idxs), "offsets_from_sorted: null pointer");
  const int64_t n = R + 1;
  offsets_from_sorted_kernel<<<static_cast<unsigned>(cdiv64(n, 256)), 256, 0, stream>>>(sorted_expert_idxs, R, E,
                                                                                      expert_offsets);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

extern "C" int64_t smoe_sort_count_static_capacity(void) { return SC_STATIC_INTS; }

extern "C" int smoe_sort_count_static(const int64_t* expert_idxs, int64_t R, int32_t E, int64_t* sorted_expert_idxs,
                                      int64_t* sorted_scattered_idxs, int64_t* expert_offsets, void* stream) {
  SMOE_CHECK_ARG(R >= 0 && R < (int64_t(1) << 31), "sort_count_static: R=%lld out of range [0, 2^31)", (long long)R);
  SMOE_CHECK_ARG(E >= 1 && E <= SC_MAX_E, "sort_count_static: E=%d out of range [1, %d]", E, SC_MAX_E);
  const int64_t need = cdiv64(R > 0 ? R : 1, SC_CHUNK) * E;
  if (need > SC_STATIC_INTS) {
    set_error("sort_count_static: ceil(R/%d) * E = %lld exceeds the built-in scratch of %d entries (R=%lld, E=%d); "
              "use smoe_sort_count with a caller-provided workspace", SC_CHUNK, (long long)need, SC_STATIC_INTS,
              (long long)R, E);
    return SMOE_ERR_WORKSPACE;
  }
  int32_t* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  // Same kernels as smoe_sort_count, on the built-in array: its SC_STATIC_INTS entries are exactly what the capacity
  // check above admits (the caller-workspace entry point asks for 256 spare bytes that the kernels never touch).
  // The histogram pass writes every scratch entry the later passes read, so nothing left behind by an earlier
  // call needs clearing.
  return sort_count_launch("sort_count_static", expert_idxs, R, E, sorted_expert_idxs, sorted_scattered_idxs,
                           expert_offsets, scratch, static_cast<cudaStream_t>(stream));
}
