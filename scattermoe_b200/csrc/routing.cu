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

// ---- router fusion: logits -> top-k ids, gates and the block histograms of the sort, in one pass -----------------
// Replaces, for the callers of flatten_sort_count (scattermoe/utils/replace_moe.py:67-71, the reference test's
// tests/test_mlp.py:46-51, Hugging Face's top-k routers), the softmax / topk / renormalise / histogram sequence of
// separate PyTorch kernels with a (T, E) round trip through HBM between each: one warp reads a token's E logits once,
// keeps them in registers, and emits the k selected expert ids (int64, descending by logit; equal logits: lower
// expert id first), their gates (fp32) and its share of the counting sort's block histogram. Block b covers the
// slots [b * SC_CHUNK, (b + 1) * SC_CHUNK) of the flat (T, k) id tensor, exactly what sc_scan_kernel and
// sc_scatter_kernel expect from sc_hist_kernel; a token whose slots straddle two blocks is evaluated by both, each
// writing and counting only its own slots.
//   mode 0: p = softmax(logits) over all experts, gates = top-k of p (renorm: divided by their sum)
//   mode 1: gates = softmax over the k selected logits
// lse (nullable): log-sum-exp of the token's logits over all experts (what the backward of mode 0 needs).
enum { ROUTE_SOFTMAX_TOPK = 0, ROUTE_TOPK_SOFTMAX = 1 };
constexpr int ROUTE_MAX_E = 1024;
constexpr int ROUTE_MAX_K = 32;

template <typename T, int NV>
__global__ void __launch_bounds__(SC_THREADS)
route_topk_kernel(const T* __restrict__ logits, int64_t stride_t, int64_t Tn, int E, int k, int mode, int renorm,
                  int64_t* __restrict__ ids, float* __restrict__ gates, float* __restrict__ lse, int nblk,
                  int32_t* __restrict__ block_hist) {
  extern __shared__ int32_t hist[];     // [E]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int e = tid; e < E; e += SC_THREADS) hist[e] = 0;
  __syncthreads();
  const int64_t R = Tn * k;
  const int64_t s_beg = static_cast<int64_t>(blockIdx.x) * SC_CHUNK;
  const int64_t s_end = min(R, s_beg + SC_CHUNK);
  const int64_t t_beg = s_beg / k, t_end = (s_end + k - 1) / k;
  const float NEG = -INFINITY;
  for (int64_t t = t_beg + warp; t < t_end; t += SC_WARPS) {
    float v[NV];
    const T* row = logits + t * stride_t;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int e = i * 32 + lane;
      v[i] = e < E ? to_f32<T>(row[e]) : NEG;
    }
    // maximum and sum of exponentials over all experts
    float m = v[0];
#pragma unroll
    for (int i = 1; i < NV; ++i) m = fmaxf(m, v[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float ssum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) ssum += (v[i] == NEG) ? 0.f : expf(v[i] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
    if (lse && lane == 0 && t * k >= s_beg) lse[t] = m + logf(ssum);     // the block that owns the token's first slot
    // k rounds of arg-max; lane j keeps the j-th winner
    float my_val = 0.f;
    int my_id = 0;
    for (int j = 0; j < k; ++j) {
      float best = v[0];
      int bi = 0;
#pragma unroll
      for (int i = 1; i < NV; ++i)
        if (v[i] > best) { best = v[i]; bi = i; }
      int be = bi * 32 + lane;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; }
      }
      if (lane == j) { my_val = best; my_id = be; }
      if ((be & 31) == lane) {
#pragma unroll
        for (int i = 0; i < NV; ++i)
          if (i == (be >> 5)) v[i] = NEG;
      }
    }
    // gates of the k winners (lanes 0..k-1)
    const bool sel = lane < k;
    const float top = __shfl_sync(0xffffffffu, my_val, 0);
    float g = sel ? expf(my_val - (mode == ROUTE_TOPK_SOFTMAX ? top : m)) : 0.f;
    float gs = g;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gs += __shfl_xor_sync(0xffffffffu, gs, o);
    if (mode == ROUTE_TOPK_SOFTMAX) g = g / gs;
    else g = renorm ? g / gs : g / ssum;
    if (sel) {
      const int64_t slot = t * k + lane;
      if (slot >= s_beg && slot < s_end) {
        ids[slot] = my_id;
        gates[slot] = g;
        if (my_id < E) atomicAdd(&hist[my_id], 1);
      }
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += SC_THREADS) block_hist[static_cast<int64_t>(e) * nblk + blockIdx.x] = hist[e];
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

extern "C" size_t smoe_route_topk_workspace_bytes(int64_t T, int32_t k, int32_t E) {
  if (T < 0 || k < 1 || E < 1) return 0;
  return smoe_sort_count_workspace_bytes(T * k, E);
}

template <typename T>
static int route_launch(const void* logits, int64_t stride_t, int64_t Tn, int E, int k, int mode, int renorm,
                        int64_t* ids, float* gates, float* lse, int nblk, int32_t* block_hist, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(E) * sizeof(int32_t);
  const int nv = cdiv(E, 32);
#define SMOE_ROUTE_CASE(NV)                                                                                         \
  route_topk_kernel<T, NV><<<nblk, SC_THREADS, smem, stream>>>(static_cast<const T*>(logits), stride_t, Tn, E, k, mode, \
                                                               renorm, ids, gates, lse, nblk, block_hist)
  if (nv <= 1) SMOE_ROUTE_CASE(1);
  else if (nv <= 2) SMOE_ROUTE_CASE(2);
  else if (nv <= 4) SMOE_ROUTE_CASE(4);
  else if (nv <= 8) SMOE_ROUTE_CASE(8);
  else if (nv <= 16) SMOE_ROUTE_CASE(16);
  else SMOE_ROUTE_CASE(32);
#undef SMOE_ROUTE_CASE
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

extern "C" int smoe_route_topk(const void* logits, int64_t T, int32_t E, int64_t stride_t, int32_t logits_dtype,
                               int32_t k, int32_t mode, int32_t renormalize, int64_t* expert_idxs, float* gates,
                               float* lse, int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs,
                               int64_t* expert_offsets, void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  SMOE_CHECK_ARG(T >= 0 && E >= 1 && k >= 1 && k <= E, "route_topk: bad sizes T=%lld E=%d k=%d", (long long)T, E, k);
  SMOE_CHECK_ARG(T * k < (int64_t(1) << 31), "route_topk: T*k=%lld out of range [0, 2^31)", (long long)(T * k));
  SMOE_CHECK_ARG(mode == ROUTE_SOFTMAX_TOPK || mode == ROUTE_TOPK_SOFTMAX, "route_topk: unknown mode %d", mode);
  SMOE_CHECK_ARG(logits_dtype == SMOE_F32 || logits_dtype == SMOE_BF16 || logits_dtype == SMOE_F16,
                 "route_topk: unknown dtype %d", logits_dtype);
  if (E > ROUTE_MAX_E || k > ROUTE_MAX_K) return SMOE_ERR_UNSUPPORTED;     // the caller uses separate kernels
  SMOE_CHECK_ARG(expert_offsets != nullptr, "route_topk: expert_offsets is null");
  const int64_t R = T * k;
  if (R == 0) {
    zero_offsets_kernel<<<cdiv(E, 256), 256, 0, stream>>>(expert_offsets, E);
    SMOE_LAUNCH_CHECK();
    return SMOE_OK;
  }
  SMOE_CHECK_ARG(logits && expert_idxs && gates && sorted_expert_idxs && sorted_scattered_idxs, "route_topk: null pointer");
  SMOE_CHECK_ARG(stride_t >= E, "route_topk: row stride %lld smaller than E=%d", (long long)stride_t, E);
  if (workspace == nullptr || workspace_bytes < smoe_route_topk_workspace_bytes(T, k, E)) {
    set_error("route_topk: workspace of %zu bytes needed, %zu given", smoe_route_topk_workspace_bytes(T, k, E),
              workspace_bytes);
    return SMOE_ERR_WORKSPACE;
  }
  const int nblk = static_cast<int>(cdiv64(R, SC_CHUNK));
  int32_t* block_hist = static_cast<int32_t*>(workspace);
  int rc;
  switch (logits_dtype) {
    case SMOE_F32: rc = route_launch<float>(logits, stride_t, T, E, k, mode, renormalize ? 1 : 0, expert_idxs, gates, lse, nblk, block_hist, stream); break;
    case SMOE_BF16: rc = route_launch<__nv_bfloat16>(logits, stride_t, T, E, k, mode, renormalize ? 1 : 0, expert_idxs, gates, lse, nblk, block_hist, stream); break;
    default: rc = route_launch<__half>(logits, stride_t, T, E, k, mode, renormalize ? 1 : 0, expert_idxs, gates, lse, nblk, block_hist, stream); break;
  }
  if (rc != SMOE_OK) return rc;
  const size_t smem = static_cast<size_t>(SC_WARPS) * E * sizeof(int32_t);     // E <= 1024: at most 32 KB
  sc_scan_kernel<<<1, 1024, 0, stream>>>(block_hist, E * nblk, E, nblk, expert_offsets);
  SMOE_LAUNCH_CHECK();
  sc_scatter_kernel<<<nblk, SC_THREADS, smem, stream>>>(expert_idxs, R, E, nblk, block_hist, sorted_expert_idxs,
                                                        sorted_scattered_idxs);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}
