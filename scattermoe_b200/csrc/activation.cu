// The activation between the two expert linears, forward and backward, as single HBM-bound passes.
//
// The reference leaves this to PyTorch elementwise ops and autograd (scattermoe/mlp.py:41 and :81-87,
// scattermoe/utils/replace_moe.py:39-43 and :76-83): several kernels and temporaries per direction, and the
// backward of chunk()/strided slices materialises a full-width gradient. Here one kernel reads the
// up-projection once and writes the hidden activations; one kernel reads the up-projection and the hidden
// gradient and writes the up-projection gradient. Arithmetic in fp32, one rounding to the storage dtype.
//
// Layouts of the (rows, n_up) up-projection `U` -> (rows, F) hidden `H`:
//   PLAIN       n_up = F     H[j] = act(U[j])                                   (MLP, mlp.py:41)
//   GLU_SECOND  n_up = 2F    H[j] = act(U[F+j]) * U[j]                           (GLUMLP, mlp.py:81-87)
//   GLU_FIRST   n_up = 2F    H[j] = act(U[j]) * U[F+j]                           (granite, replace_moe.py:76-83)
//   GPT_OSS     n_up = 2F    g = min(U[2j], limit), u = clamp(U[2j+1], +-limit),
//                            H[j] = (u + 1) * g * sigmoid(alpha * g)             (gpt-oss, replace_moe.py:39-43)
#include "act_math.cuh"
#include "smoe_common.cuh"

namespace smoe {

template <typename T, int V> struct alignas(sizeof(T) * V) Pack { T v[V]; };

template <typename T, int V>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[V]) {
  if constexpr (V == 1) {
    f[0] = to_f32<T>(p[0]);
  } else {
    const Pack<T, V> pk = *reinterpret_cast<const Pack<T, V>*>(p);
#pragma unroll
    for (int i = 0; i < V; ++i) f[i] = to_f32<T>(pk.v[i]);
  }
}
template <typename T, int V>
__device__ __forceinline__ void store_vec(T* p, const float (&f)[V]) {
  if constexpr (V == 1) {
    p[0] = from_f32<T>(f[0]);
  } else {
    Pack<T, V> pk;
#pragma unroll
    for (int i = 0; i < V; ++i) pk.v[i] = from_f32<T>(f[i]);
    *reinterpret_cast<Pack<T, V>*>(p) = pk;
  }
}

// One thread per V hidden columns of one row. V = 16/sizeof(T) on the vector path, 1 otherwise.
template <typename T, int LAYOUT, int V>
__global__ void __launch_bounds__(256)
act_forward_kernel(const T* __restrict__ U, int64_t su, T* __restrict__ H, int64_t sh, int64_t rows,
                   const int64_t* __restrict__ rows_dev, int F, int act, float alpha, float limit) {
  constexpr bool FAST = sizeof(T) == 2;
  const int vec_per_row = F / V;
  if (rows_dev) rows = min(rows, *rows_dev);     // live row count known only on the device
  for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < rows * vec_per_row;
       gid += static_cast<int64_t>(gridDim.x) * blockDim.x) {
  // 32-bit division when the index fits (a 64-bit division per thread costs more than the rest of the body)
  const int64_t r = (gid >> 32) == 0 ? static_cast<int64_t>(static_cast<uint32_t>(gid) / static_cast<uint32_t>(vec_per_row))
                                     : gid / vec_per_row;
  const int j = static_cast<int>(gid - r * vec_per_row) * V;
  const T* u = U + r * su;
  float out[V];
  if (LAYOUT == LAYOUT_PLAIN) {
    float a[V];
    load_vec<T, V>(u + j, a);
    SMOE_ACT_SWITCH(act, _Pragma("unroll") for (int i = 0; i < V; ++i) out[i] = act_fwd<ACT_, FAST>(a[i]);)
  } else if (LAYOUT == LAYOUT_GPT_OSS) {
    float a[V], b[V];
    load_vec<T, V>(u + 2 * j, a);
    load_vec<T, V>(u + 2 * j + V, b);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float g0 = (2 * i < V) ? a[(2 * i) % V] : b[(2 * i) % V];
      const float u0 = (2 * i + 1 < V) ? a[(2 * i + 1) % V] : b[(2 * i + 1) % V];
      const float g = fminf(g0, limit);
      const float uc = fminf(fmaxf(u0, -limit), limit);
      out[i] = (uc + 1.0f) * (g * sigmoidf_<FAST>(alpha * g));
    }
  } else {
    float lin[V], gate[V];
    load_vec<T, V>(u + (LAYOUT == LAYOUT_GLU_SECOND ? j : F + j), lin);
    load_vec<T, V>(u + (LAYOUT == LAYOUT_GLU_SECOND ? F + j : j), gate);
    SMOE_ACT_SWITCH(act, _Pragma("unroll") for (int i = 0; i < V; ++i) out[i] = act_fwd<ACT_, FAST>(gate[i]) * lin[i];)
  }
  store_vec<T, V>(H + r * sh + j, out);
  }
}

template <typename T, int LAYOUT, int V>
__global__ void __launch_bounds__(256)
act_backward_kernel(const T* __restrict__ U, int64_t su, const T* __restrict__ DH, int64_t sdh, T* __restrict__ DU,
                    int64_t sdu, int64_t rows, const int64_t* __restrict__ rows_dev, int F, int act, float alpha,
                    float limit) {
  constexpr bool FAST = sizeof(T) == 2;
  const int vec_per_row = F / V;
  if (rows_dev) rows = min(rows, *rows_dev);
  for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < rows * vec_per_row;
       gid += static_cast<int64_t>(gridDim.x) * blockDim.x) {
  // 32-bit division when the index fits (a 64-bit division per thread costs more than the rest of the body)
  const int64_t r = (gid >> 32) == 0 ? static_cast<int64_t>(static_cast<uint32_t>(gid) / static_cast<uint32_t>(vec_per_row))
                                     : gid / vec_per_row;
  const int j = static_cast<int>(gid - r * vec_per_row) * V;
  const T* u = U + r * su;
  T* du = DU + r * sdu;
  float dh[V];
  load_vec<T, V>(DH + r * sdh + j, dh);
  if (LAYOUT == LAYOUT_PLAIN) {
    float a[V], o[V];
    load_vec<T, V>(u + j, a);
    SMOE_ACT_SWITCH(act, _Pragma("unroll") for (int i = 0; i < V; ++i) o[i] = dh[i] * act_bwd<ACT_, FAST>(a[i]);)
    store_vec<T, V>(du + j, o);
  } else if (LAYOUT == LAYOUT_GPT_OSS) {
    float a[V], b[V], oa[V], ob[V];
    load_vec<T, V>(u + 2 * j, a);
    load_vec<T, V>(u + 2 * j + V, b);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float g0 = (2 * i < V) ? a[(2 * i) % V] : b[(2 * i) % V];
      const float u0 = (2 * i + 1 < V) ? a[(2 * i + 1) % V] : b[(2 * i + 1) % V];
      const float g = fminf(g0, limit);
      const float uc = fminf(fmaxf(u0, -limit), limit);
      const float s = sigmoidf_<FAST>(alpha * g);
      const float glu = g * s;
      const float d_u = (u0 >= -limit && u0 <= limit) ? dh[i] * glu : 0.f;
      const float d_glu = dh[i] * (uc + 1.0f);
      const float d_g = (g0 <= limit) ? d_glu * (s + g * alpha * s * (1.0f - s)) : 0.f;
      if (2 * i < V) oa[(2 * i) % V] = d_g; else ob[(2 * i) % V] = d_g;
      if (2 * i + 1 < V) oa[(2 * i + 1) % V] = d_u; else ob[(2 * i + 1) % V] = d_u;
    }
    store_vec<T, V>(du + 2 * j, oa);
    store_vec<T, V>(du + 2 * j + V, ob);
  } else {
    const int lin_off = (LAYOUT == LAYOUT_GLU_SECOND) ? j : F + j;
    const int gate_off = (LAYOUT == LAYOUT_GLU_SECOND) ? F + j : j;
    float lin[V], gate[V], dl[V], dg[V];
    load_vec<T, V>(u + lin_off, lin);
    load_vec<T, V>(u + gate_off, gate);
    SMOE_ACT_SWITCH(act, _Pragma("unroll") for (int i = 0; i < V; ++i) {
      dl[i] = dh[i] * act_fwd<ACT_, FAST>(gate[i]);
      dg[i] = dh[i] * lin[i] * act_bwd<ACT_, FAST>(gate[i]);
    })
    store_vec<T, V>(du + lin_off, dl);
    store_vec<T, V>(du + gate_off, dg);
  }
  }
}

static inline bool aligned16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, int LAYOUT>
static int act_launch(bool backward, const void* U, int64_t su, const void* DH, int64_t sdh, void* OUT, int64_t so,
                      int64_t rows, const int64_t* rows_dev, int F, int act, float alpha, float limit, cudaStream_t stream) {
  constexpr int VV = 16 / sizeof(T);
  // GPT_OSS scalar path pairs columns itself (V = 1 reads u[2j], u[2j+1]); vector path needs whole vectors
  bool vec = F % VV == 0 && su % VV == 0 && so % VV == 0 && aligned16p(U) && aligned16p(OUT);
  if (backward) vec = vec && sdh % VV == 0 && aligned16p(DH);
  const int64_t work = rows * (vec ? F / VV : F);
  // with a device-side row count the host `rows` is only an upper bound: cap the grid, the kernels grid-stride
  const int64_t blocks = cdiv64(work, 256);
  const unsigned grid = static_cast<unsigned>(rows_dev && blocks > 148 * 32 ? 148 * 32 : blocks);
  if (grid == 0) return SMOE_OK;
  if (vec) {
    if (backward)
      act_backward_kernel<T, LAYOUT, VV><<<grid, 256, 0, stream>>>((const T*)U, su, (const T*)DH, sdh, (T*)OUT, so, rows,
                                                                  rows_dev, F, act, alpha, limit);
    else
      act_forward_kernel<T, LAYOUT, VV><<<grid, 256, 0, stream>>>((const T*)U, su, (T*)OUT, so, rows, rows_dev, F, act, alpha, limit);
  } else {
    if (backward)
      act_backward_kernel<T, LAYOUT, 1><<<grid, 256, 0, stream>>>((const T*)U, su, (const T*)DH, sdh, (T*)OUT, so, rows,
                                                                 rows_dev, F, act, alpha, limit);
    else
      act_forward_kernel<T, LAYOUT, 1><<<grid, 256, 0, stream>>>((const T*)U, su, (T*)OUT, so, rows, rows_dev, F, act, alpha, limit);
  }
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

template <typename T>
static int act_dispatch_layout(int layout, bool backward, const void* U, int64_t su, const void* DH, int64_t sdh,
                               void* OUT, int64_t so, int64_t rows, const int64_t* rows_dev, int F, int act, float alpha,
                               float limit, cudaStream_t stream) {
  switch (layout) {
    case LAYOUT_PLAIN: return act_launch<T, LAYOUT_PLAIN>(backward, U, su, DH, sdh, OUT, so, rows, rows_dev, F, act, alpha, limit, stream);
    case LAYOUT_GLU_SECOND: return act_launch<T, LAYOUT_GLU_SECOND>(backward, U, su, DH, sdh, OUT, so, rows, rows_dev, F, act, alpha, limit, stream);
    case LAYOUT_GLU_FIRST: return act_launch<T, LAYOUT_GLU_FIRST>(backward, U, su, DH, sdh, OUT, so, rows, rows_dev, F, act, alpha, limit, stream);
    case LAYOUT_GPT_OSS: return act_launch<T, LAYOUT_GPT_OSS>(backward, U, su, DH, sdh, OUT, so, rows, rows_dev, F, act, alpha, limit, stream);
  }
  set_error("activation: unknown layout %d", layout);
  return SMOE_ERR_BAD_ARG;
}

static int act_entry(bool backward, const void* U, int64_t su, const void* DH, int64_t sdh, void* OUT, int64_t so,
                     int64_t rows, const int64_t* rows_dev, int F, int layout, int act, float alpha, float limit,
                     int dtype, void* stream) {
  SMOE_CHECK_ARG(rows >= 0 && F >= 0, "activation: bad sizes rows=%lld F=%d", (long long)rows, F);
  SMOE_CHECK_ARG(act >= ACT_SILU && act <= ACT_IDENTITY, "activation: unknown function %d", act);
  if (rows == 0 || F == 0) return SMOE_OK;
  SMOE_CHECK_ARG(U && OUT && (!backward || DH), "activation: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SMOE_F32: return act_dispatch_layout<float>(layout, backward, U, su, DH, sdh, OUT, so, rows, rows_dev, F, act, alpha, limit, st);
    case SMOE_BF16: return act_dispatch_layout<__nv_bfloat16>(layout, backward, U, su, DH, sdh, OUT, so, rows, rows_dev, F, act, alpha, limit, st);
    case SMOE_F16: return act_dispatch_layout<__half>(layout, backward, U, su, DH, sdh, OUT, so, rows, rows_dev, F, act, alpha, limit, st);
  }
  set_error("activation: unknown dtype %d", dtype);
  return SMOE_ERR_BAD_ARG;
}

}  // namespace smoe

extern "C" int smoe_activation_forward(const void* U, int64_t stride_um, void* H, int64_t stride_hm, int64_t rows,
                                       const int64_t* rows_dev, int32_t F, int32_t layout, int32_t act, float alpha,
                                       float limit, int32_t dtype, void* stream) {
  return smoe::act_entry(false, U, stride_um, nullptr, 0, H, stride_hm, rows, rows_dev, F, layout, act, alpha, limit,
                         dtype, stream);
}

extern "C" int smoe_activation_backward(const void* U, int64_t stride_um, const void* DH, int64_t stride_dhm, void* DU,
                                        int64_t stride_dum, int64_t rows, const int64_t* rows_dev, int32_t F,
                                        int32_t layout, int32_t act, float alpha, float limit, int32_t dtype,
                                        void* stream) {
  return smoe::act_entry(true, U, stride_um, DH, stride_dhm, DU, stride_dum, rows, rows_dev, F, layout, act, alpha, limit,
                         dtype, stream);
}
