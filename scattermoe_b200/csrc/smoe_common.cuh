// Shared host/device helpers for the scattermoe_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/scattermoe_b200.h"

namespace smoe {

// ---- error reporting (thread-local message, integer status across the ABI) ----------------------
void set_error(const char* fmt, ...);
void set_last_path(int tensor_core);

#define SMOE_CHECK_ARG(cond, ...)                 \
  do {                                            \
    if (!(cond)) {                                \
      ::smoe::set_error(__VA_ARGS__);             \
      return SMOE_ERR_BAD_ARG;                    \
    }                                             \
  } while (0)

#define SMOE_CUDA(call)                                                                          \
  do {                                                                                           \
    cudaError_t err__ = (call);                                                                  \
    if (err__ != cudaSuccess) {                                                                  \
      ::smoe::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(err__), __FILE__,    \
                        __LINE__);                                                               \
      return SMOE_ERR_CUDA;                                                                      \
    }                                                                                            \
  } while (0)

#define SMOE_LAUNCH_CHECK() SMOE_CUDA(cudaGetLastError())

// Properties of the current device, cached per device ordinal.
struct DeviceInfo {
  int device;
  int sm_count;
  int cc_major;
  int cc_minor;
  int max_smem_optin;
};
int get_device_info(DeviceInfo* out);

inline int dtype_size(int dtype) { return dtype == SMOE_F32 ? 4 : 2; }

// ---- element conversion -----------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

__host__ __device__ __forceinline__ int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int cdiv(int a, int b) { return (a + b - 1) / b; }

// ---- internal launchers (one per translation unit) -----------------------------------------------
struct S2SArgs {
  const void* X; int64_t x_rows, sxm, sxk;
  const void* W; int64_t swe, swk, swn;
  const void* bias; int64_t sbe, sbn;
  void* Y; int64_t sym, syn;
  const int64_t* sorted_e; const int64_t* sorted_idx; const int64_t* offsets;
  int64_t R; int K, N, E, fan_out, x_grouped, y_grouped, dtype, flags;
  int32_t* status;
  cudaStream_t stream;
  // fused activation epilogue (tensor-core kernel only): act_layout < 0 = none, else a LAYOUT_* of act_math.cuh
  void* H = nullptr; int64_t shm = 0;
  int act_layout = -1, act = 0;
  float alpha = 0.f, limit = 0.f;
  // fused activation-gradient epilogue: U = saved up-projection (rows, n_up); Y then receives dU, N is F
  const void* U = nullptr; int64_t sum = 0;
  int act_bwd = 0;
  // per-slot gates for the fused epilogues (nullable) and the gate gradient's partial sums (act_bwd only, nullable)
  const void* row_gate = nullptr;
  float* dot_out = nullptr;
  // expert-parallel return fused into the epilogue (tensor-core kernel, plain launches only): output row m goes to
  // out_peers[rank] at the row packed in out_addr[m] instead of Y
  const int64_t* out_addr = nullptr;
  void* const* out_peers = nullptr;
  int64_t out_peer_stride = 0, out_peer_rows = 0;
  int out_world = 0, my_rank = 0;
};

struct WGradArgs {
  const void* DY; int64_t sdym, sdyn;
  const void* X; int64_t x_rows, sxm, sxk;
  const int64_t* offsets; const int64_t* gather_idx; int fan_out;
  void* DW; int64_t sdwe, sdwk, sdwn;
  void* Db; int64_t sdbe, sdbn;
  int64_t R; int K, N, E, dtype, flags;
  int32_t* status;
  cudaStream_t stream;
};

int launch_s2s_simt(const S2SArgs& a);
int launch_wgrad_simt(const WGradArgs& a);
// Tensor-core launchers return SMOE_ERR_UNSUPPORTED (without setting an error) when the arguments do
// not meet their alignment / dtype rules; the dispatcher then takes the CUDA-core kernel.
int launch_s2s_tc(const S2SArgs& a);
int launch_wgrad_tc(const WGradArgs& a);

}  // namespace smoe
