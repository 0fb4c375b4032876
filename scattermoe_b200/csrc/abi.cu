// C-ABI entry points of the GEMM-shaped calls: argument validation and the choice between the tcgen05
// kernels and the CUDA-core kernels. Declarations and the contract are in include/scattermoe_b200.h.
#include <stdarg.h>

#include <mutex>

#include "smoe_common.cuh"

namespace smoe {

static thread_local char g_last_error[512] = "";
static thread_local int g_last_path_tc = 0;

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

void set_last_path(int tensor_core) { g_last_path_tc = tensor_core; }

int get_device_info(DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  static bool have[64] = {false};
  int dev = 0;
  SMOE_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 0 || dev >= 64 || !have[dev]) {
    DeviceInfo d;
    d.device = dev;
    SMOE_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    SMOE_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    SMOE_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    SMOE_CUDA(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    if (dev < 0 || dev >= 64) { *out = d; return SMOE_OK; }
    cache[dev] = d;
    have[dev] = true;
  }
  *out = cache[dev];
  return SMOE_OK;
}

}  // namespace smoe

using namespace smoe;

extern "C" int smoe_version(void) { return SMOE_ABI_VERSION; }
extern "C" const char* smoe_last_error(void) { return g_last_error; }
extern "C" int smoe_last_path_was_tensor_core(void) { return g_last_path_tc; }

static int check_dtype(const char* who, int dtype) {
  if (dtype != SMOE_F32 && dtype != SMOE_BF16 && dtype != SMOE_F16) {
    set_error("%s: unknown dtype %d", who, dtype);
    return SMOE_ERR_BAD_ARG;
  }
  return SMOE_OK;
}

extern "C" int smoe_scatter2scatter(const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk,
                                    const void* W, int64_t stride_we, int64_t stride_wk, int64_t stride_wn,
                                    const void* bias, int64_t stride_be, int64_t stride_bn, void* Y,
                                    int64_t stride_ym, int64_t stride_yn, const int64_t* sorted_expert_idxs,
                                    const int64_t* sorted_scattered_idxs, const int64_t* expert_offsets, int64_t R,
                                    int32_t K, int32_t N, int32_t E, int32_t fan_out, int32_t x_grouped,
                                    int32_t y_grouped, int32_t dtype, int32_t flags, int32_t* status,
                                    void* stream) {
  if (int rc = check_dtype("scatter2scatter", dtype)) return rc;
  SMOE_CHECK_ARG(R >= 0 && R < (int64_t(1) << 31), "scatter2scatter: R=%lld out of range [0, 2^31)", (long long)R);
  SMOE_CHECK_ARG(K >= 0 && N >= 0 && E >= 1 && fan_out >= 1, "scatter2scatter: bad sizes K=%d N=%d E=%d fan_out=%d", K,
                 N, E, fan_out);
  // same contract as the reference's assertion `idx.size(0) == X.size(0) * k` (ops.py:124-125)
  SMOE_CHECK_ARG(x_rows * fan_out == R && (!x_grouped || fan_out == 1),
                 "scatter2scatter: %lld index entries but X has %lld rows with fan_out %d", (long long)R,
                 (long long)x_rows, fan_out);
  if (R == 0 || N == 0) return SMOE_OK;
  SMOE_CHECK_ARG(X && W && Y && sorted_expert_idxs && sorted_scattered_idxs && expert_offsets,
                 "scatter2scatter: null pointer");
  S2SArgs a{X, x_rows, stride_xm, stride_xk, W, stride_we, stride_wk, stride_wn, bias, stride_be, stride_bn,
            Y, stride_ym, stride_yn, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
            R, K, N, E, fan_out, x_grouped ? 1 : 0, y_grouped ? 1 : 0, dtype, flags,
            status, static_cast<cudaStream_t>(stream)};
  if (!(flags & SMOE_FLAG_FORCE_SIMT)) {
    const int rc = launch_s2s_tc(a);
    if (rc != SMOE_ERR_UNSUPPORTED) {
      if (rc == SMOE_OK) set_last_path(1);
      return rc;
    }
    if (flags & SMOE_FLAG_FORCE_TC) {
      set_error("scatter2scatter: no tensor-core kernel for this dtype/alignment (dtype=%d K=%d N=%d)", dtype, K, N);
      return rc;
    }
  }
  set_last_path(0);
  return launch_s2s_simt(a);
}

extern "C" int smoe_group_bwd_w(const void* DY, int64_t stride_dym, int64_t stride_dyn, const void* X,
                                int64_t x_rows, int64_t stride_xm, int64_t stride_xk,
                                const int64_t* expert_offsets, const int64_t* x_gather_idx, int32_t fan_out,
                                void* DW, int64_t stride_dwe, int64_t stride_dwk, int64_t stride_dwn, void* Db,
                                int64_t stride_dbe, int64_t stride_dbn, int64_t R, int32_t K, int32_t N, int32_t E,
                                int32_t dtype, int32_t flags, int32_t* status, void* stream) {
  if (int rc = check_dtype("group_bwd_w", dtype)) return rc;
  SMOE_CHECK_ARG(R >= 0 && R < (int64_t(1) << 31), "group_bwd_w: R=%lld out of range [0, 2^31)", (long long)R);
  SMOE_CHECK_ARG(K >= 0 && N >= 0 && E >= 1 && fan_out >= 1, "group_bwd_w: bad sizes K=%d N=%d E=%d fan_out=%d", K, N,
                 E, fan_out);
  if (K == 0 || N == 0) return SMOE_OK;
  SMOE_CHECK_ARG(DW && expert_offsets && (R == 0 || (DY && X)), "group_bwd_w: null pointer");
  SMOE_CHECK_ARG(x_gather_idx != nullptr || x_rows >= R, "group_bwd_w: grouped X has %lld rows, %lld needed",
                 (long long)x_rows, (long long)R);
  WGradArgs a{DY, stride_dym, stride_dyn, X, x_rows, stride_xm, stride_xk, expert_offsets, x_gather_idx, fan_out,
              DW, stride_dwe, stride_dwk, stride_dwn, Db, stride_dbe, stride_dbn, R, K, N, E, dtype, flags,
              status, static_cast<cudaStream_t>(stream)};
  if (!(flags & SMOE_FLAG_FORCE_SIMT)) {
    const int rc = launch_wgrad_tc(a);
    if (rc != SMOE_ERR_UNSUPPORTED) {
      if (rc == SMOE_OK) set_last_path(1);
      return rc;
    }
    if (flags & SMOE_FLAG_FORCE_TC) {
      set_error("group_bwd_w: no tensor-core kernel for this dtype/alignment (dtype=%d K=%d N=%d)", dtype, K, N);
      return rc;
    }
  }
  set_last_path(0);
  return launch_wgrad_simt(a);
}

// Up-projection with the activation fused into the epilogue of the tensor-core kernel. Returns
// SMOE_ERR_UNSUPPORTED (no error text) when the request does not fit that kernel: the caller then runs
// smoe_scatter2scatter followed by smoe_activation_forward.
extern "C" int smoe_scatter2scatter_act(const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk,
                                        const void* W, int64_t stride_we, int64_t stride_wk, int64_t stride_wn,
                                        const void* bias, int64_t stride_be, int64_t stride_bn, void* Y,
                                        int64_t stride_ym, int64_t stride_yn, void* H, int64_t stride_hm,
                                        const int64_t* sorted_expert_idxs, const int64_t* sorted_scattered_idxs,
                                        const int64_t* expert_offsets, int64_t R, int32_t K, int32_t N, int32_t E,
                                        int32_t fan_out, int32_t x_grouped, int32_t dtype, int32_t flags,
                                        int32_t act_layout, int32_t act, float alpha, float limit,
                                        const void* row_gates, int32_t* status, void* stream) {
  if (int rc = check_dtype("scatter2scatter_act", dtype)) return rc;
  SMOE_CHECK_ARG(R >= 0 && R < (int64_t(1) << 31), "scatter2scatter_act: R=%lld out of range", (long long)R);
  SMOE_CHECK_ARG(K >= 0 && N >= 0 && E >= 1 && fan_out >= 1, "scatter2scatter_act: bad sizes K=%d N=%d E=%d fan_out=%d",
                 K, N, E, fan_out);
  SMOE_CHECK_ARG(x_rows * fan_out == R && (!x_grouped || fan_out == 1),
                 "scatter2scatter_act: %lld index entries but X has %lld rows with fan_out %d", (long long)R,
                 (long long)x_rows, fan_out);
  SMOE_CHECK_ARG(act_layout >= 0 && act_layout <= 3 && act >= 0 && act <= 4, "scatter2scatter_act: layout %d / function %d",
                 act_layout, act);
  if (R == 0 || N == 0) return SMOE_OK;
  SMOE_CHECK_ARG(X && W && H && sorted_expert_idxs && sorted_scattered_idxs && expert_offsets,
                 "scatter2scatter_act: null pointer");
  if (flags & SMOE_FLAG_FORCE_SIMT) return SMOE_ERR_UNSUPPORTED;
  S2SArgs a{X, x_rows, stride_xm, stride_xk, W, stride_we, stride_wk, stride_wn, bias, stride_be, stride_bn,
            Y, stride_ym, stride_yn, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
            R, K, N, E, fan_out, x_grouped ? 1 : 0, 1, dtype, flags, status, static_cast<cudaStream_t>(stream)};
  a.H = H; a.shm = stride_hm; a.act_layout = act_layout; a.act = act; a.alpha = alpha; a.limit = limit;
  a.row_gate = row_gates;
  if (Y == nullptr) { a.sym = 8; a.syn = 1; }
  const int rc = launch_s2s_tc(a);
  if (rc == SMOE_OK) set_last_path(1);
  return rc;
}

// Input gradient of the down-projection with the activation gradient fused into the epilogue of the tensor-core
// kernel: dU = activation'(U) applied to (DY @ W), the (rows, F) hidden gradient itself never stored. Returns
// SMOE_ERR_UNSUPPORTED (no error text) when the request does not fit that kernel: the caller then runs
// smoe_scatter2scatter followed by smoe_activation_backward.
extern "C" int smoe_scatter2scatter_act_bwd(const void* DY, int64_t stride_dym, int64_t stride_dyk, const void* W,
                                            int64_t stride_we, int64_t stride_wk, int64_t stride_wn, const void* U,
                                            int64_t stride_um, void* DU, int64_t stride_dum,
                                            const int64_t* expert_offsets, int64_t R, int32_t K, int32_t F, int32_t E,
                                            int32_t dtype, int32_t flags, int32_t act_layout, int32_t act, float alpha,
                                            float limit, const void* row_gates, const int64_t* sorted_scattered_idxs,
                                            float* gate_partials, int32_t* status, void* stream) {
  if (int rc = check_dtype("scatter2scatter_act_bwd", dtype)) return rc;
  SMOE_CHECK_ARG(R >= 0 && R < (int64_t(1) << 31), "scatter2scatter_act_bwd: R=%lld out of range", (long long)R);
  SMOE_CHECK_ARG(K >= 0 && F >= 0 && E >= 1, "scatter2scatter_act_bwd: bad sizes K=%d F=%d E=%d", K, F, E);
  SMOE_CHECK_ARG(act_layout >= 0 && act_layout <= 3 && act >= 0 && act <= 4,
                 "scatter2scatter_act_bwd: layout %d / function %d", act_layout, act);
  if (R == 0 || F == 0) return SMOE_OK;
  SMOE_CHECK_ARG(DY && W && U && DU && expert_offsets, "scatter2scatter_act_bwd: null pointer");
  SMOE_CHECK_ARG((row_gates == nullptr && gate_partials == nullptr) || (row_gates && gate_partials && sorted_scattered_idxs),
                 "scatter2scatter_act_bwd: row_gates, sorted_scattered_idxs and gate_partials go together");
  if (flags & SMOE_FLAG_FORCE_SIMT) return SMOE_ERR_UNSUPPORTED;
  // rows are in expert order on both sides: without gates the index tensors are never read (the offsets stand in)
  const int64_t* slots = sorted_scattered_idxs ? sorted_scattered_idxs : expert_offsets;
  S2SArgs a{DY, R, stride_dym, stride_dyk, W, stride_we, stride_wk, stride_wn, nullptr, 0, 0,
            DU, stride_dum, 1, expert_offsets, slots, expert_offsets,
            R, K, F, E, 1, 1, 1, dtype, flags, status, static_cast<cudaStream_t>(stream)};
  a.U = U; a.sum = stride_um; a.act_layout = act_layout; a.act = act; a.alpha = alpha; a.limit = limit; a.act_bwd = 1;
  a.row_gate = row_gates; a.dot_out = gate_partials;
  const int rc = launch_s2s_tc(a);
  if (rc == SMOE_OK) set_last_path(1);
  return rc;
}

// Grouped GEMM whose epilogue returns the rows to their home ranks (the expert-parallel return direction, fused):
// what smoe_scatter2scatter (grouped in, grouped out) followed by smoe_ep_return does, without the intermediate
// result buffer and with the NVLink transfer overlapped tile by tile with the tensor-core work. Returns
// SMOE_ERR_UNSUPPORTED (no error text) when the request does not fit the tensor-core kernel: the caller then runs
// the two separate calls.
extern "C" int smoe_scatter2scatter_to_peers(const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk,
                                             const void* W, int64_t stride_we, int64_t stride_wk, int64_t stride_wn,
                                             const int64_t* expert_offsets, const int64_t* return_addr,
                                             void* const* peer_slot_bufs, int64_t peer_stride_rows, int64_t peer_rows,
                                             int32_t world, int32_t my_rank, int32_t K, int32_t N, int32_t E,
                                             int32_t dtype, int32_t flags, int32_t* status, void* stream) {
  if (int rc = check_dtype("scatter2scatter_to_peers", dtype)) return rc;
  SMOE_CHECK_ARG(x_rows >= 0 && x_rows < (int64_t(1) << 31), "scatter2scatter_to_peers: %lld rows out of range",
                 (long long)x_rows);
  SMOE_CHECK_ARG(K >= 0 && N >= 0 && E >= 1, "scatter2scatter_to_peers: bad sizes K=%d N=%d E=%d", K, N, E);
  SMOE_CHECK_ARG(world >= 1 && my_rank >= 0 && my_rank < world, "scatter2scatter_to_peers: rank %d of %d", my_rank, world);
  SMOE_CHECK_ARG(peer_rows >= 0 && peer_rows < (int64_t(1) << 40), "scatter2scatter_to_peers: peer buffer too large");
  if (x_rows == 0 || N == 0) return SMOE_OK;
  SMOE_CHECK_ARG(X && W && expert_offsets && return_addr && peer_slot_bufs, "scatter2scatter_to_peers: null pointer");
  if (flags & SMOE_FLAG_FORCE_SIMT) return SMOE_ERR_UNSUPPORTED;
  S2SArgs a{X, x_rows, stride_xm, stride_xk, W, stride_we, stride_wk, stride_wn, nullptr, 0, 0,
            nullptr, 0, 1, expert_offsets, expert_offsets, expert_offsets,
            x_rows, K, N, E, 1, 1, 1, dtype, flags, status, static_cast<cudaStream_t>(stream)};
  a.out_addr = return_addr; a.out_peers = peer_slot_bufs; a.out_peer_stride = peer_stride_rows;
  a.out_peer_rows = peer_rows; a.out_world = world; a.my_rank = my_rank;
  const int rc = launch_s2s_tc(a);
  if (rc == SMOE_OK) set_last_path(1);
  return rc;
}

// Lines of fp32 partial sums (each R long) that smoe_scatter2scatter_act_bwd writes per row when it is given gates:
// two per 256-wide tile of hidden columns (one per group of epilogue warps).
extern "C" int32_t smoe_act_bwd_partial_lines(int32_t F) { return F > 0 ? 2 * ((F + 255) / 256) : 0; }
