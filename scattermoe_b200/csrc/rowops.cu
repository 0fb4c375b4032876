// HBM-bound row kernels around the grouped GEMMs: gather-with-scale (group), gate-weighted top-k
// reduction and the gate gradient. One warp (group, gate_grad) or one block (reduce) per row, 16-byte
// vector accesses when the layout allows, scalar strided accesses otherwise.
#include "smoe_common.cuh"

namespace smoe {

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float (&f)[Vec16<T>::N]) {
  const T* p = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < Vec16<T>::N; ++i) f[i] = to_f32<T>(p[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack16(const float (&f)[Vec16<T>::N]) {
  uint4 v;
  T* p = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < Vec16<T>::N; ++i) p[i] = from_f32<T>(f[i]);
  return v;
}

// ---- group: Y[n,:] = A[idx[n]/fan_out,:] * coeff[idx[n]] ------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
group_kernel(const T* __restrict__ A, int64_t a_rows, int64_t sam, int64_t sak, const int64_t* __restrict__ idx,
             const T* __restrict__ coeff, int fan_out, T* __restrict__ Y, int64_t sym, int64_t syk, int64_t R,
             int K) {
  const int lane = threadIdx.x & 31;
  const int64_t n = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (n >= R) return;
  const int64_t slot = idx[n];
  const int64_t src = slot / fan_out;
  if (slot < 0 || src >= a_rows) return;  // malformed index: leave the row untouched
  const bool scaled = coeff != nullptr;
  const float c = scaled ? to_f32<T>(coeff[slot]) : 1.0f;
  const T* a = A + src * sam;
  T* y = Y + n * sym;
  if (VEC) {
    constexpr int V = Vec16<T>::N;
    const uint4* a4 = reinterpret_cast<const uint4*>(a);
    uint4* y4 = reinterpret_cast<uint4*>(y);
    const int nv = K / V;
    for (int i = lane; i < nv; i += 32) {
      uint4 v = __ldg(a4 + i);
      if (scaled) {
        float f[V];
        unpack16<T>(v, f);
#pragma unroll
        for (int j = 0; j < V; ++j) f[j] *= c;
        v = pack16<T>(f);
      }
      y4[i] = v;
    }
  } else {
    for (int i = lane; i < K; i += 32) {
      const T v = a[i * sak];
      y[i * syk] = scaled ? from_f32<T>(to_f32<T>(v) * c) : v;
    }
  }
}

// ---- top-k reduce: out[t,:] = sum_j gates[t,j] * Yx[t*k+j,:] --------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(128)
topk_reduce_kernel(const T* __restrict__ Yx, int64_t syxm, const T* __restrict__ gates, int64_t sgt, int64_t sgk,
                   T* __restrict__ out, int64_t som, int k, int N) {
  const int64_t t = blockIdx.x;
  const T* y0 = Yx + t * k * syxm;
  T* o = out + t * som;
  if (VEC) {
    constexpr int V = Vec16<T>::N;
    const int nv = N / V;
    for (int i = threadIdx.x; i < nv; i += 128) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      for (int j = 0; j < k; ++j) {
        const float g = gates ? to_f32<T>(gates[t * sgt + j * sgk]) : 1.0f;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(y0 + j * syxm) + i);
        float f[V];
        unpack16<T>(v, f);
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = fmaf(g, f[q], acc[q]);
      }
      reinterpret_cast<uint4*>(o)[i] = pack16<T>(acc);
    }
  } else {
    for (int i = threadIdx.x; i < N; i += 128) {
      float acc = 0.f;
      for (int j = 0; j < k; ++j) {
        const float g = gates ? to_f32<T>(gates[t * sgt + j * sgk]) : 1.0f;
        acc = fmaf(g, to_f32<T>(y0[j * syxm + i]), acc);
      }
      o[i] = from_f32<T>(acc);
    }
  }
}

// ---- gate gradient: d_gates[t,j] = <Yx[t*k+j,:], grad_out[t,:]> ------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
gate_grad_kernel(const T* __restrict__ Yx, int64_t syxm, const T* __restrict__ go, int64_t sgom,
                 T* __restrict__ dg, int64_t sdgt, int64_t sdgk, int64_t T_, int k, int N) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= T_ * k) return;
  const int64_t t = row / k;
  const int j = static_cast<int>(row - t * k);
  const T* y = Yx + row * syxm;
  const T* g = go + t * sgom;
  float acc = 0.f;
  if (VEC) {
    constexpr int V = Vec16<T>::N;
    const int nv = N / V;
    for (int i = lane; i < nv; i += 32) {
      float a[V], b[V];
      unpack16<T>(__ldg(reinterpret_cast<const uint4*>(y) + i), a);
      unpack16<T>(__ldg(reinterpret_cast<const uint4*>(g) + i), b);
#pragma unroll
      for (int q = 0; q < V; ++q) acc = fmaf(a[q], b[q], acc);
    }
  } else {
    for (int i = lane; i < N; i += 32) acc = fmaf(to_f32<T>(y[i]), to_f32<T>(g[i]), acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dg[t * sdgt + j * sdgk] = from_f32<T>(acc);
}

// ---- gate gradient from the partial sums of the fused gradient epilogue -------------------------------------
// d_gates[slot(m)] = sum over lines l of partials[l * R + m]; one thread per sorted position m.
template <typename T>
__global__ void __launch_bounds__(256)
gate_grad_partials_kernel(const float* __restrict__ partials, int lines, int64_t R, const int64_t* __restrict__ sorted_idx,
                          T* __restrict__ d_gates) {
  const int64_t m = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (m >= R) return;
  float acc = 0.f;
  for (int l = 0; l < lines; ++l) acc += partials[static_cast<int64_t>(l) * R + m];
  const int64_t slot = sorted_idx[m];
  if (slot >= 0 && slot < R) d_gates[slot] = from_f32<T>(acc);
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
int group_typed(const void* A, int64_t a_rows, int64_t sam, int64_t sak, const int64_t* idx, const void* coeff,
                int fan_out, void* Y, int64_t sym, int64_t syk, int64_t R, int K, cudaStream_t stream) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = sak == 1 && syk == 1 && K % V == 0 && sam % V == 0 && sym % V == 0 && aligned16(A) && aligned16(Y);
  const unsigned grid = static_cast<unsigned>(cdiv64(R, 8));
  if (vec)
    group_kernel<T, true><<<grid, 256, 0, stream>>>((const T*)A, a_rows, sam, sak, idx, (const T*)coeff, fan_out,
                                                    (T*)Y, sym, syk, R, K);
  else
    group_kernel<T, false><<<grid, 256, 0, stream>>>((const T*)A, a_rows, sam, sak, idx, (const T*)coeff, fan_out,
                                                     (T*)Y, sym, syk, R, K);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

template <typename T>
int topk_reduce_typed(const void* Yx, int64_t syxm, const void* gates, int64_t sgt, int64_t sgk, void* out,
                      int64_t som, int64_t T_, int k, int N, cudaStream_t stream) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = N % V == 0 && syxm % V == 0 && som % V == 0 && aligned16(Yx) && aligned16(out);
  if (vec)
    topk_reduce_kernel<T, true><<<static_cast<unsigned>(T_), 128, 0, stream>>>((const T*)Yx, syxm, (const T*)gates,
                                                                               sgt, sgk, (T*)out, som, k, N);
  else
    topk_reduce_kernel<T, false><<<static_cast<unsigned>(T_), 128, 0, stream>>>((const T*)Yx, syxm, (const T*)gates,
                                                                                sgt, sgk, (T*)out, som, k, N);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

template <typename T>
int gate_grad_typed(const void* Yx, int64_t syxm, const void* go, int64_t sgom, void* dg, int64_t sdgt, int64_t sdgk,
                    int64_t T_, int k, int N, cudaStream_t stream) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = N % V == 0 && syxm % V == 0 && sgom % V == 0 && aligned16(Yx) && aligned16(go);
  const unsigned grid = static_cast<unsigned>(cdiv64(T_ * k, 8));
  if (vec)
    gate_grad_kernel<T, true><<<grid, 256, 0, stream>>>((const T*)Yx, syxm, (const T*)go, sgom, (T*)dg, sdgt, sdgk,
                                                        T_, k, N);
  else
    gate_grad_kernel<T, false><<<grid, 256, 0, stream>>>((const T*)Yx, syxm, (const T*)go, sgom, (T*)dg, sdgt, sdgk,
                                                         T_, k, N);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

}  // namespace smoe

using namespace smoe;

#define SMOE_DISPATCH_DTYPE(dtype, FN, ...)                              \
  switch (dtype) {                                                       \
    case SMOE_F32: return FN<float>(__VA_ARGS__);                        \
    case SMOE_BF16: return FN<__nv_bfloat16>(__VA_ARGS__);               \
    case SMOE_F16: return FN<__half>(__VA_ARGS__);                       \
    default: set_error("unknown dtype %d", dtype); return SMOE_ERR_BAD_ARG; \
  }

extern "C" int smoe_group(const void* A, int64_t a_rows, int64_t stride_am, int64_t stride_ak, const int64_t* idx,
                          const void* coeff, int32_t fan_out, void* Y, int64_t stride_ym, int64_t stride_yk,
                          int64_t R, int32_t K, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(R >= 0 && K >= 0 && fan_out >= 1, "group: bad sizes R=%lld K=%d fan_out=%d", (long long)R, K, fan_out);
  if (R == 0 || K == 0) return SMOE_OK;
  SMOE_CHECK_ARG(A && Y && idx, "group: null pointer");
  SMOE_CHECK_ARG(R < (int64_t(1) << 31) * 8, "group: R too large");
  SMOE_DISPATCH_DTYPE(dtype, group_typed, A, a_rows, stride_am, stride_ak, idx, coeff, fan_out, Y, stride_ym,
                      stride_yk, R, K, static_cast<cudaStream_t>(stream));
}

extern "C" int smoe_topk_reduce(const void* Yx, int64_t stride_yxm, const void* gates, int64_t stride_gt,
                                int64_t stride_gk, void* out, int64_t stride_om, int64_t T, int32_t k, int32_t N,
                                int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(T >= 0 && k >= 1 && N >= 0, "topk_reduce: bad sizes T=%lld k=%d N=%d", (long long)T, k, N);
  if (T == 0 || N == 0) return SMOE_OK;
  SMOE_CHECK_ARG(Yx && out, "topk_reduce: null pointer");
  SMOE_CHECK_ARG(T < (int64_t(1) << 31), "topk_reduce: T too large");
  SMOE_DISPATCH_DTYPE(dtype, topk_reduce_typed, Yx, stride_yxm, gates, stride_gt, stride_gk, out, stride_om, T, k, N,
                      static_cast<cudaStream_t>(stream));
}

extern "C" int smoe_gate_grad(const void* Yx, int64_t stride_yxm, const void* grad_out, int64_t stride_gom,
                              void* d_gates, int64_t stride_dgt, int64_t stride_dgk, int64_t T, int32_t k, int32_t N,
                              int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(T >= 0 && k >= 1 && N >= 0, "gate_grad: bad sizes T=%lld k=%d N=%d", (long long)T, k, N);
  if (T == 0) return SMOE_OK;
  SMOE_CHECK_ARG(Yx && grad_out && d_gates, "gate_grad: null pointer");
  SMOE_DISPATCH_DTYPE(dtype, gate_grad_typed, Yx, stride_yxm, grad_out, stride_gom, d_gates, stride_dgt, stride_dgk, T,
                      k, N, static_cast<cudaStream_t>(stream));
}

extern "C" int smoe_gate_grad_from_partials(const float* partials, int32_t lines, int64_t R,
                                            const int64_t* sorted_scattered_idxs, void* d_gates, int32_t dtype,
                                            void* stream) {
  SMOE_CHECK_ARG(R >= 0 && lines >= 1, "gate_grad_from_partials: bad sizes R=%lld lines=%d", (long long)R, lines);
  if (R == 0) return SMOE_OK;
  SMOE_CHECK_ARG(partials && sorted_scattered_idxs && d_gates, "gate_grad_from_partials: null pointer");
  const unsigned grid = static_cast<unsigned>(cdiv64(R, 256));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SMOE_F32: gate_grad_partials_kernel<float><<<grid, 256, 0, st>>>(partials, lines, R, sorted_scattered_idxs, static_cast<float*>(d_gates)); break;
    case SMOE_BF16: gate_grad_partials_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(partials, lines, R, sorted_scattered_idxs, static_cast<__nv_bfloat16*>(d_gates)); break;
    case SMOE_F16: gate_grad_partials_kernel<__half><<<grid, 256, 0, st>>>(partials, lines, R, sorted_scattered_idxs, static_cast<__half*>(d_gates)); break;
    default: set_error("gate_grad_from_partials: unknown dtype %d", dtype); return SMOE_ERR_BAD_ARG;
  }
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}
