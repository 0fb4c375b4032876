// CUDA-core (fp32 FMA) grouped GEMM kernels.
//
// These serve every request the tcgen05 kernels do not: fp32 inputs (the reference test demands 1e-4 with
// TF32 off, tests/test_mlp.py:8,:83, and the tensor cores have no full-fp32 mode), and layouts whose rows
// are not 16-byte aligned (e.g. hidden size 133). They accept arbitrary element strides like the reference's
// Triton kernels (scattermoe/kernels/ops.py:165-171) and accumulate in fp32 (ops.py:180, :237).
#include "smoe_common.cuh"

namespace smoe {

constexpr int ST_BM = 64, ST_BN = 64, ST_BK = 16, ST_THREADS = 256;

// Y[out(m),:] = X[in(m),:] @ W[e(m)] + b[e(m)]. A block owns 64 consecutive positions of the sorted slot
// list and 64 output columns; it runs one K loop per expert present in its rows, with the rows of other
// experts zeroed in shared memory (same scheme as ops.py:87-107).
template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
s2s_simt_kernel(const T* __restrict__ X, int64_t x_rows, int64_t sxm, int64_t sxk, const T* __restrict__ W,
                int64_t swe, int64_t swk, int64_t swn, const T* __restrict__ bias, int64_t sbe, int64_t sbn,
                T* __restrict__ Y, int64_t sym, int64_t syn, const int64_t* __restrict__ sorted_e,
                const int64_t* __restrict__ sorted_idx, int64_t R, int K, int N, int E, int fan_out, int x_grouped,
                int y_grouped) {
  __shared__ float As[ST_BK][ST_BM + 4];
  __shared__ float Bs[ST_BK][ST_BN + 4];
  __shared__ int64_t s_in[ST_BM];
  __shared__ int64_t s_out[ST_BM];
  __shared__ int s_exp[ST_BM];

  const int tid = threadIdx.x;
  const int64_t m0 = static_cast<int64_t>(blockIdx.x) * ST_BM;
  const int n0 = blockIdx.y * ST_BN;
  if (tid < ST_BM) {
    const int64_t m = m0 + tid;
    int e = -1;
    int64_t in = 0, out = 0;
    if (m < R) {
      const int64_t ev = sorted_e[m];
      const int64_t slot = sorted_idx[m];
      in = x_grouped ? m : slot / fan_out;
      out = y_grouped ? m : slot;
      e = (ev >= 0 && ev < E && in >= 0 && in < x_rows && out >= 0 && out < R) ? static_cast<int>(ev) : -1;
    }
    s_exp[tid] = e;
    s_in[tid] = in;
    s_out[tid] = out;
  }
  __syncthreads();
  const int rows = static_cast<int>(min(static_cast<int64_t>(ST_BM), R - m0));
  int e_first = E, e_last = -1;
  for (int r = 0; r < rows; ++r) {  // tiny: 64 reads of shared memory
    const int e = s_exp[r];
    if (e >= 0) { e_first = min(e_first, e); e_last = max(e_last, e); }
  }
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const bool w_n_fast = (swn <= swk);

  for (int e = e_first; e <= e_last; ++e) {
    bool any = false;
    for (int r = 0; r < rows; ++r) any |= (s_exp[r] == e);
    if (!any) continue;
    const T* We = W + static_cast<int64_t>(e) * swe;
    for (int k0 = 0; k0 < K; k0 += ST_BK) {
#pragma unroll
      for (int i = 0; i < (ST_BM * ST_BK) / ST_THREADS; ++i) {
        const int id = tid + i * ST_THREADS;
        const int kk = id % ST_BK, r = id / ST_BK;
        float v = 0.f;
        if (s_exp[r] == e && k0 + kk < K) v = to_f32<T>(X[s_in[r] * sxm + (k0 + kk) * sxk]);
        As[kk][r] = v;
      }
#pragma unroll
      for (int i = 0; i < (ST_BN * ST_BK) / ST_THREADS; ++i) {
        const int id = tid + i * ST_THREADS;
        int kk, n;
        if (w_n_fast) { n = id % ST_BN; kk = id / ST_BN; } else { kk = id % ST_BK; n = id / ST_BK; }
        float v = 0.f;
        if (k0 + kk < K && n0 + n < N) v = to_f32<T>(We[(k0 + kk) * swk + (n0 + n) * swn]);
        Bs[kk][n] = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < ST_BK; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    const int e = s_exp[r];
    if (r >= rows || e < 0) continue;
    T* y = Y + s_out[r] * sym;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += to_f32<T>(bias[static_cast<int64_t>(e) * sbe + n * sbn]);
      y[n * syn] = from_f32<T>(v);
    }
  }
}

// DW[e][kk][n] = sum_m X[xrow(m)][kk] * DY[m][n] over expert e's rows; Db[e][n] = sum_m DY[m][n].
// Grid (K tiles, N tiles, E). Every output element is written (zeros for experts without rows).
template <typename T>
__global__ void __launch_bounds__(ST_THREADS)
wgrad_simt_kernel(const T* __restrict__ DY, int64_t sdym, int64_t sdyn, const T* __restrict__ X, int64_t x_rows,
                  int64_t sxm, int64_t sxk, const int64_t* __restrict__ offsets, const int64_t* __restrict__ gidx,
                  int fan_out, T* __restrict__ DW, int64_t sdwe, int64_t sdwk, int64_t sdwn, T* __restrict__ Db,
                  int64_t sdbe, int64_t sdbn, int64_t R, int K, int N) {
  __shared__ float Xs[ST_BK][ST_BM + 4];
  __shared__ float Ds[ST_BK][ST_BN + 4];
  __shared__ int64_t s_row[ST_BK];
  const int tid = threadIdx.x;
  const int e = blockIdx.z;
  const int k0 = blockIdx.x * ST_BM, n0 = blockIdx.y * ST_BN;
  int64_t start = e ? offsets[e - 1] : 0;
  int64_t end = offsets[e];
  start = max(static_cast<int64_t>(0), min(start, R));
  end = max(start, min(end, R));
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  float db = 0.f;
  const bool want_db = (Db != nullptr) && blockIdx.x == 0;

  for (int64_t m0 = start; m0 < end; m0 += ST_BK) {
    if (tid < ST_BK) {
      const int64_t m = m0 + tid;
      int64_t row = -1;
      if (m < end) {
        row = gidx ? gidx[m] / fan_out : m;
        if (row < 0 || row >= x_rows) row = -1;
      }
      s_row[tid] = row;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < (ST_BM * ST_BK) / ST_THREADS; ++i) {
      const int id = tid + i * ST_THREADS;
      const int kk = id % ST_BM, mm = id / ST_BM;
      const int64_t row = s_row[mm];
      float v = 0.f;
      if (row >= 0 && k0 + kk < K) v = to_f32<T>(X[row * sxm + (k0 + kk) * sxk]);
      Xs[mm][kk] = v;
    }
#pragma unroll
    for (int i = 0; i < (ST_BN * ST_BK) / ST_THREADS; ++i) {
      const int id = tid + i * ST_THREADS;
      const int n = id % ST_BN, mm = id / ST_BN;
      float v = 0.f;
      if (m0 + mm < end && n0 + n < N) v = to_f32<T>(DY[(m0 + mm) * sdym + (n0 + n) * sdyn]);
      Ds[mm][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int mm = 0; mm < ST_BK; ++mm) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = Xs[mm][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ds[mm][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (want_db && tid < ST_BN) {
#pragma unroll
      for (int mm = 0; mm < ST_BK; ++mm) db += Ds[mm][tid];
    }
    __syncthreads();
  }
  T* dw = DW + static_cast<int64_t>(e) * sdwe;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int kk = k0 + ty * 4 + i;
    if (kk >= K) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) dw[kk * sdwk + n * sdwn] = from_f32<T>(acc[i][j]);
    }
  }
  if (want_db && tid < ST_BN && n0 + tid < N) Db[static_cast<int64_t>(e) * sdbe + (n0 + tid) * sdbn] = from_f32<T>(db);
}

template <typename T>
static int s2s_simt_typed(const S2SArgs& a) {
  dim3 grid(static_cast<unsigned>(cdiv64(a.R, ST_BM)), static_cast<unsigned>(cdiv(a.N, ST_BN)));
  s2s_simt_kernel<T><<<grid, ST_THREADS, 0, a.stream>>>(
      (const T*)a.X, a.x_rows, a.sxm, a.sxk, (const T*)a.W, a.swe, a.swk, a.swn, (const T*)a.bias, a.sbe, a.sbn,
      (T*)a.Y, a.sym, a.syn, a.sorted_e, a.sorted_idx, a.R, a.K, a.N, a.E, a.fan_out, a.x_grouped, a.y_grouped);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

template <typename T>
static int wgrad_simt_typed(const WGradArgs& a) {
  dim3 grid(static_cast<unsigned>(cdiv(a.K, ST_BM)), static_cast<unsigned>(cdiv(a.N, ST_BN)),
            static_cast<unsigned>(a.E));
  wgrad_simt_kernel<T><<<grid, ST_THREADS, 0, a.stream>>>(
      (const T*)a.DY, a.sdym, a.sdyn, (const T*)a.X, a.x_rows, a.sxm, a.sxk, a.offsets, a.gather_idx, a.fan_out,
      (T*)a.DW, a.sdwe, a.sdwk, a.sdwn, (T*)a.Db, a.sdbe, a.sdbn, a.R, a.K, a.N);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

int launch_s2s_simt(const S2SArgs& a) {
  if (a.R == 0 || a.N == 0) return SMOE_OK;
  switch (a.dtype) {
    case SMOE_F32: return s2s_simt_typed<float>(a);
    case SMOE_BF16: return s2s_simt_typed<__nv_bfloat16>(a);
    case SMOE_F16: return s2s_simt_typed<__half>(a);
  }
  set_error("scatter2scatter: unknown dtype %d", a.dtype);
  return SMOE_ERR_BAD_ARG;
}

int launch_wgrad_simt(const WGradArgs& a) {
  if (a.E == 0 || a.N == 0 || a.K == 0) return SMOE_OK;
  if (a.E > 65535) { set_error("group_bwd_w: E=%d exceeds the CUDA-core kernel's grid limit 65535", a.E); return SMOE_ERR_UNSUPPORTED; }
  switch (a.dtype) {
    case SMOE_F32: return wgrad_simt_typed<float>(a);
    case SMOE_BF16: return wgrad_simt_typed<__nv_bfloat16>(a);
    case SMOE_F16: return wgrad_simt_typed<__half>(a);
  }
  set_error("group_bwd_w: unknown dtype %d", a.dtype);
  return SMOE_ERR_BAD_ARG;
}

}  // namespace smoe
