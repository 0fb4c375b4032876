// Single-token expert matvec: Y[j,:] = X[j or 0,:] . W[expert_idxs[j]]  for the k experts of one token.
//
// Replaces the reference's decode kernel _single2scatter (scattermoe/kernels/single.py:5-59). The work is a
// handful of matrix-vector products, i.e. bound by reading k weight matrices once from HBM: the kernels below
// only make those reads wide and coalesced (16-byte loads along whichever weight dimension is contiguous) and
// accumulate in fp32 (single.py:56 ACC_TYPE). Unlike the reference (no masks, sizes must be multiples of 128)
// any K and N are accepted.
#include "smoe_common.cuh"

namespace smoe {

// N-contiguous weights (E, K, N): a block owns 256 output columns of one (token, slot); its 8 warps split K.
template <typename T>
__global__ void __launch_bounds__(256)
single_ncontig_kernel(const T* __restrict__ X, int64_t sxm, int x_rows, const T* __restrict__ W, int64_t swe,
                      int64_t swk, T* __restrict__ Y, int64_t sym, const int64_t* __restrict__ expert_idxs, int E,
                      int K, int N, bool vec) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float red[8][32 * V + 1];
  const int j = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t e = expert_idxs[j];
  const int n0 = blockIdx.x * (32 * V) + lane * V;
  float acc[V];
#pragma unroll
  for (int q = 0; q < V; ++q) acc[q] = 0.f;
  if (e >= 0 && e < E) {
    const T* x = X + (x_rows == 1 ? 0 : j) * sxm;
    const T* w = W + e * swe;
    for (int kk = warp; kk < K; kk += 8) {
      const float xv = to_f32<T>(__ldg(x + kk));
      const T* wr = w + kk * swk + n0;
      if (vec && n0 + V <= N) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(wr));
        const T* pv = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = fmaf(xv, to_f32<T>(pv[q]), acc[q]);
      } else {
#pragma unroll
        for (int q = 0; q < V; ++q)
          if (n0 + q < N) acc[q] = fmaf(xv, to_f32<T>(wr[q]), acc[q]);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < V; ++q) red[warp][lane * V + q] = acc[q];
  __syncthreads();
  for (int c = threadIdx.x; c < 32 * V; c += 256) {
    float s = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) s += red[w8][c];
    const int n = blockIdx.x * (32 * V) + c;
    if (n < N) Y[j * sym + n] = from_f32<T>(s);
  }
}

// Any other layout (K-contiguous included): one warp per output column, lanes stride over K.
template <typename T>
__global__ void __launch_bounds__(256)
single_generic_kernel(const T* __restrict__ X, int64_t sxm, int64_t sxk, int x_rows, const T* __restrict__ W, int64_t swe,
                      int64_t swk, int64_t swn, T* __restrict__ Y, int64_t sym, int64_t syn,
                      const int64_t* __restrict__ expert_idxs, int E, int K, int N, bool vec) {
  constexpr int V = 16 / sizeof(T);
  const int j = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const int64_t e = expert_idxs[j];
  float acc = 0.f;
  if (e >= 0 && e < E) {
    const T* x = X + (x_rows == 1 ? 0 : j) * sxm;
    const T* w = W + e * swe + n * swn;
    if (vec) {   // swk == 1, sxk == 1, 16-byte aligned rows
      for (int kk = lane * V; kk + V <= K; kk += 32 * V) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(x + kk));
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(w + kk));
        const T* pa = reinterpret_cast<const T*>(&a);
        const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
        for (int q = 0; q < V; ++q) acc = fmaf(to_f32<T>(pa[q]), to_f32<T>(pb[q]), acc);
      }
      for (int kk = (K / V) * V + lane; kk < K; kk += 32) acc = fmaf(to_f32<T>(x[kk]), to_f32<T>(w[kk]), acc);
    } else {
      for (int kk = lane; kk < K; kk += 32) acc = fmaf(to_f32<T>(x[kk * sxk]), to_f32<T>(w[kk * swk]), acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) Y[j * sym + n * syn] = from_f32<T>(acc);
}

static bool al16s(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static int single_typed(const void* X, int64_t sxm, int64_t sxk, int x_rows, const void* W, int64_t swe, int64_t swk,
                        int64_t swn, void* Y, int64_t sym, int64_t syn, const int64_t* idx, int k, int E, int K, int N,
                        cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  if (swn == 1 && sxk == 1 && syn == 1) {
    const bool vec = al16s(W) && swk % V == 0 && swe % V == 0;
    dim3 grid(static_cast<unsigned>(cdiv(N, 32 * V)), static_cast<unsigned>(k));
    single_ncontig_kernel<T><<<grid, 256, 0, st>>>((const T*)X, sxm, x_rows, (const T*)W, swe, swk, (T*)Y, sym, idx, E, K,
                                                   N, vec);
  } else {
    const bool vec = swk == 1 && sxk == 1 && al16s(W) && al16s(X) && swn % V == 0 && swe % V == 0 && sxm % V == 0;
    dim3 grid(static_cast<unsigned>(cdiv(N, 8)), static_cast<unsigned>(k));
    single_generic_kernel<T><<<grid, 256, 0, st>>>((const T*)X, sxm, sxk, x_rows, (const T*)W, swe, swk, swn, (T*)Y, sym,
                                                   syn, idx, E, K, N, vec);
  }
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

}  // namespace smoe

using namespace smoe;

extern "C" int smoe_single2scatter(const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk, const void* W,
                                   int64_t stride_we, int64_t stride_wk, int64_t stride_wn, void* Y, int64_t stride_ym,
                                   int64_t stride_yn, const int64_t* expert_idxs, int32_t k, int32_t K, int32_t N,
                                   int32_t E, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(k >= 0 && k <= 65535 && K >= 0 && N >= 0 && E >= 1, "single2scatter: bad sizes k=%d K=%d N=%d E=%d", k, K,
                 N, E);
  // same contract as the reference's assertion (single.py:44): one input row, or one per selected expert
  SMOE_CHECK_ARG(x_rows == 1 || x_rows == k, "single2scatter: X has %lld rows, expected 1 or k=%d", (long long)x_rows, k);
  if (k == 0 || N == 0) return SMOE_OK;
  SMOE_CHECK_ARG(X && W && Y && expert_idxs, "single2scatter: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SMOE_F32: return single_typed<float>(X, stride_xm, stride_xk, (int)x_rows, W, stride_we, stride_wk, stride_wn, Y, stride_ym, stride_yn, expert_idxs, k, E, K, N, st);
    case SMOE_BF16: return single_typed<__nv_bfloat16>(X, stride_xm, stride_xk, (int)x_rows, W, stride_we, stride_wk, stride_wn, Y, stride_ym, stride_yn, expert_idxs, k, E, K, N, st);
    case SMOE_F16: return single_typed<__half>(X, stride_xm, stride_xk, (int)x_rows, W, stride_we, stride_wk, stride_wn, Y, stride_ym, stride_yn, expert_idxs, k, E, K, N, st);
  }
  set_error("single2scatter: unknown dtype %d", dtype);
  return SMOE_ERR_BAD_ARG;
}
