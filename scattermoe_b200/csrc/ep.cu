// Expert-parallel row exchange over NVLink peer memory (plain P2P loads and stores, no multicast, no flags).
//
// The reference has no multi-GPU code; these kernels replace what a NCCL all-to-all-v based expert-parallel layer
// does around the local grouped GEMMs (pack rows by destination -> all-to-all-v -> regroup by expert, and the way
// back) with ONE pass each way and no intermediate copies:
//   dispatch  every (token, slot) row is written straight into the owning rank's receive buffer at the position
//             that makes that buffer expert-grouped (all ranks know all counts, so every row's final position is
//             computable at the sender); an optional per-slot coefficient (the gate, in backward) is applied
//             on the fly. The receiver runs its grouped GEMMs on the buffer as is: no sort, no regroup copy.
//   combine   the owning rank of a token pulls the k expert-output rows from the peers' output buffers and
//             reduces them with the gate weights in registers: out[t] = sum_j g[t,j] * peer[w_j][row_j].
//   gate_grad d_gates[t,j] = <peer[w_j][row_j], grad_out[t]> with the same pulls.
// Synchronisation between the phases is the caller's (a stream-ordered barrier across the ranks); the kernels
// themselves never wait on another GPU.
#include "smoe_common.cuh"

namespace smoe {

constexpr int EP_MAX_WORLD = 16;
struct PeerPtrs { uint8_t* p[EP_MAX_WORLD]; };

__device__ __forceinline__ int64_t pack_dest(int rank, int64_t row) { return (static_cast<int64_t>(rank) << 40) | row; }
__device__ __forceinline__ int dest_rank(int64_t d) { return static_cast<int>(d >> 40); }
__device__ __forceinline__ int64_t dest_row(int64_t d) { return d & ((int64_t(1) << 40) - 1); }

template <typename T> struct V16 { static constexpr int N = 16 / sizeof(T); };

// One warp per sorted position m. Row m belongs to global expert e = sorted_e[m], owned by rank e / e_local; its
// position in the owner's buffer is dst_off[e] + (m - first position of e in this rank's sorted list).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const T* __restrict__ X, int64_t x_rows, int64_t sxm, const int64_t* __restrict__ sorted_e,
                   const int64_t* __restrict__ sorted_idx, const int64_t* __restrict__ offsets,
                   const int64_t* __restrict__ dst_off, const T* __restrict__ coeff, int fan_out, PeerPtrs peers,
                   int64_t peer_row_elems, int64_t cap_rows, int64_t* __restrict__ slot_dest, int64_t R, int K, int E,
                   int e_local, int world) {
  const int lane = threadIdx.x & 31;
  const int64_t m = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (m >= R) return;
  const int64_t e = sorted_e[m];
  const int64_t slot = sorted_idx[m];
  if (e < 0 || e >= E || slot < 0 || slot >= R) return;
  const int64_t src = slot / fan_out;
  const int rank = static_cast<int>(e / e_local);
  const int64_t seg_start = e ? offsets[e - 1] : 0;
  const int64_t row = dst_off[e] + (m - seg_start);
  if (src >= x_rows || rank >= world || row < 0 || row >= cap_rows) return;   // malformed plan: drop the row
  if (lane == 0 && slot_dest) slot_dest[slot] = pack_dest(rank, row);
  const float c = coeff ? to_f32<T>(coeff[slot]) : 1.0f;
  const T* x = X + src * sxm;
  T* y = reinterpret_cast<T*>(peers.p[rank]) + row * peer_row_elems;
  if (VEC) {
    constexpr int V = V16<T>::N;
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    uint4* y4 = reinterpret_cast<uint4*>(y);
    for (int i = lane; i < K / V; i += 32) {
      uint4 v = __ldg(x4 + i);
      if (coeff) {
        T* pv = reinterpret_cast<T*>(&v);
#pragma unroll
        for (int j = 0; j < V; ++j) pv[j] = from_f32<T>(to_f32<T>(pv[j]) * c);
      }
      y4[i] = v;
    }
  } else {
    for (int i = lane; i < K; i += 32) y[i] = coeff ? from_f32<T>(to_f32<T>(x[i]) * c) : x[i];
  }
}

// One block per token: out[t,:] = sum_j gates[t,j] * peer[rank_j][row_j,:]   (gates == nullptr: plain sum)
template <typename T, bool VEC>
__global__ void __launch_bounds__(128)
ep_combine_kernel(PeerPtrs peers, int64_t peer_row_elems, const int64_t* __restrict__ slot_dest,
                  const T* __restrict__ gates, int64_t sgt, int64_t sgk, T* __restrict__ out, int64_t som, int k, int N) {
  const int64_t t = blockIdx.x;
  T* o = out + t * som;
  constexpr int V = VEC ? V16<T>::N : 1;
  for (int i = threadIdx.x; i < N / V; i += 128) {
    float acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = 0.f;
    for (int j = 0; j < k; ++j) {
      const int64_t d = slot_dest[t * k + j];
      const float g = gates ? to_f32<T>(gates[t * sgt + j * sgk]) : 1.0f;
      const T* src = reinterpret_cast<const T*>(peers.p[dest_rank(d)]) + dest_row(d) * peer_row_elems;
      if (VEC) {
        const uint4 v = *(reinterpret_cast<const uint4*>(src) + i);
        const T* pv = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = fmaf(g, to_f32<T>(pv[q]), acc[q]);
      } else {
        acc[0] = fmaf(g, to_f32<T>(src[i]), acc[0]);
      }
    }
    if (VEC) {
      uint4 v;
      T* pv = reinterpret_cast<T*>(&v);
#pragma unroll
      for (int q = 0; q < V; ++q) pv[q] = from_f32<T>(acc[q]);
      reinterpret_cast<uint4*>(o)[i] = v;
    } else {
      o[i] = from_f32<T>(acc[0]);
    }
  }
}

// One warp per (token, slot): d_gates[t,j] = <peer row, grad_out[t,:]>
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
ep_gate_grad_kernel(PeerPtrs peers, int64_t peer_row_elems, const int64_t* __restrict__ slot_dest,
                    const T* __restrict__ go, int64_t sgom, T* __restrict__ dg, int64_t sdgt, int64_t sdgk, int64_t T_,
                    int k, int N) {
  const int lane = threadIdx.x & 31;
  const int64_t s = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (s >= T_ * k) return;
  const int64_t t = s / k;
  const int j = static_cast<int>(s - t * k);
  const int64_t d = slot_dest[s];
  const T* y = reinterpret_cast<const T*>(peers.p[dest_rank(d)]) + dest_row(d) * peer_row_elems;
  const T* g = go + t * sgom;
  float acc = 0.f;
  if (VEC) {
    constexpr int V = V16<T>::N;
    for (int i = lane; i < N / V; i += 32) {
      const uint4 a = *(reinterpret_cast<const uint4*>(y) + i);
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(g) + i);
      const T* pa = reinterpret_cast<const T*>(&a);
      const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
      for (int q = 0; q < V; ++q) acc = fmaf(to_f32<T>(pa[q]), to_f32<T>(pb[q]), acc);
    }
  } else {
    for (int i = lane; i < N; i += 32) acc = fmaf(to_f32<T>(y[i]), to_f32<T>(g[i]), acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dg[t * sdgt + j * sdgk] = from_f32<T>(acc);
}

static bool a16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int fill_peers(PeerPtrs* pp, void* const* peer_bufs, int world, const char* who, bool* all_aligned) {
  if (world < 1 || world > EP_MAX_WORLD) {
    set_error("%s: world size %d out of range [1, %d]", who, world, EP_MAX_WORLD);
    return SMOE_ERR_BAD_ARG;
  }
  *all_aligned = true;
  for (int i = 0; i < EP_MAX_WORLD; ++i) {
    pp->p[i] = i < world ? static_cast<uint8_t*>(peer_bufs[i]) : nullptr;
    if (i < world && pp->p[i] == nullptr) {
      set_error("%s: peer buffer %d is null", who, i);
      return SMOE_ERR_BAD_ARG;
    }
    if (i < world && !a16(pp->p[i])) *all_aligned = false;
  }
  return SMOE_OK;
}

template <typename T>
static int dispatch_typed(const void* X, int64_t x_rows, int64_t sxm, const int64_t* sorted_e, const int64_t* sorted_idx,
                          const int64_t* offsets, const int64_t* dst_off, const void* coeff, int fan_out,
                          const PeerPtrs& pp, bool aligned, int64_t peer_row_elems, int64_t cap_rows, int64_t* slot_dest,
                          int64_t R, int K, int E, int e_local, int world, cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = aligned && K % V == 0 && sxm % V == 0 && peer_row_elems % V == 0 && a16(X);
  const unsigned grid = static_cast<unsigned>(cdiv64(R, 8));
  if (vec)
    ep_dispatch_kernel<T, true><<<grid, 256, 0, st>>>((const T*)X, x_rows, sxm, sorted_e, sorted_idx, offsets, dst_off,
                                                      (const T*)coeff, fan_out, pp, peer_row_elems, cap_rows, slot_dest,
                                                      R, K, E, e_local, world);
  else
    ep_dispatch_kernel<T, false><<<grid, 256, 0, st>>>((const T*)X, x_rows, sxm, sorted_e, sorted_idx, offsets, dst_off,
                                                       (const T*)coeff, fan_out, pp, peer_row_elems, cap_rows, slot_dest,
                                                       R, K, E, e_local, world);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

template <typename T>
static int combine_typed(const PeerPtrs& pp, bool aligned, int64_t peer_row_elems, const int64_t* slot_dest,
                         const void* gates, int64_t sgt, int64_t sgk, void* out, int64_t som, int64_t T_, int k, int N,
                         cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = aligned && N % V == 0 && peer_row_elems % V == 0 && som % V == 0 && a16(out);
  if (vec)
    ep_combine_kernel<T, true><<<static_cast<unsigned>(T_), 128, 0, st>>>(pp, peer_row_elems, slot_dest, (const T*)gates,
                                                                          sgt, sgk, (T*)out, som, k, N);
  else
    ep_combine_kernel<T, false><<<static_cast<unsigned>(T_), 128, 0, st>>>(pp, peer_row_elems, slot_dest, (const T*)gates,
                                                                           sgt, sgk, (T*)out, som, k, N);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

template <typename T>
static int gate_grad_typed(const PeerPtrs& pp, bool aligned, int64_t peer_row_elems, const int64_t* slot_dest,
                           const void* go, int64_t sgom, void* dg, int64_t sdgt, int64_t sdgk, int64_t T_, int k, int N,
                           cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = aligned && N % V == 0 && peer_row_elems % V == 0 && sgom % V == 0 && a16(go);
  const unsigned grid = static_cast<unsigned>(cdiv64(T_ * k, 8));
  if (vec)
    ep_gate_grad_kernel<T, true><<<grid, 256, 0, st>>>(pp, peer_row_elems, slot_dest, (const T*)go, sgom, (T*)dg, sdgt,
                                                       sdgk, T_, k, N);
  else
    ep_gate_grad_kernel<T, false><<<grid, 256, 0, st>>>(pp, peer_row_elems, slot_dest, (const T*)go, sgom, (T*)dg, sdgt,
                                                        sdgk, T_, k, N);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

}  // namespace smoe

using namespace smoe;

extern "C" int smoe_ep_dispatch(const void* X, int64_t x_rows, int64_t stride_xm, const int64_t* sorted_expert_idxs,
                                const int64_t* sorted_scattered_idxs, const int64_t* expert_offsets,
                                const int64_t* dst_offsets, const void* coeff, int32_t fan_out, void* const* peer_bufs,
                                int64_t peer_stride_rows, int64_t capacity_rows, int64_t* slot_dest, int64_t R, int32_t K,
                                int32_t E, int32_t world, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(R >= 0 && K >= 0 && E >= 1 && fan_out >= 1, "ep_dispatch: bad sizes R=%lld K=%d E=%d fan_out=%d",
                 (long long)R, K, E, fan_out);
  SMOE_CHECK_ARG(world >= 1 && E % world == 0, "ep_dispatch: E=%d is not divisible by the world size %d", E, world);
  SMOE_CHECK_ARG(capacity_rows < (int64_t(1) << 40), "ep_dispatch: capacity too large");
  if (R == 0 || K == 0) return SMOE_OK;
  SMOE_CHECK_ARG(X && sorted_expert_idxs && sorted_scattered_idxs && expert_offsets && dst_offsets && peer_bufs,
                 "ep_dispatch: null pointer");
  PeerPtrs pp;
  bool aligned;
  if (int rc = fill_peers(&pp, peer_bufs, world, "ep_dispatch", &aligned)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int e_local = E / world;
  switch (dtype) {
    case SMOE_F32: return dispatch_typed<float>(X, x_rows, stride_xm, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, dst_offsets, coeff, fan_out, pp, aligned, peer_stride_rows, capacity_rows, slot_dest, R, K, E, e_local, world, st);
    case SMOE_BF16: return dispatch_typed<__nv_bfloat16>(X, x_rows, stride_xm, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, dst_offsets, coeff, fan_out, pp, aligned, peer_stride_rows, capacity_rows, slot_dest, R, K, E, e_local, world, st);
    case SMOE_F16: return dispatch_typed<__half>(X, x_rows, stride_xm, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, dst_offsets, coeff, fan_out, pp, aligned, peer_stride_rows, capacity_rows, slot_dest, R, K, E, e_local, world, st);
  }
  set_error("ep_dispatch: unknown dtype %d", dtype);
  return SMOE_ERR_BAD_ARG;
}

extern "C" int smoe_ep_combine(void* const* peer_bufs, int64_t peer_stride_rows, const int64_t* slot_dest,
                               const void* gates, int64_t stride_gt, int64_t stride_gk, void* out, int64_t stride_om,
                               int64_t T, int32_t k, int32_t N, int32_t world, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(T >= 0 && T < (int64_t(1) << 31) && k >= 1 && N >= 0, "ep_combine: bad sizes T=%lld k=%d N=%d",
                 (long long)T, k, N);
  if (T == 0 || N == 0) return SMOE_OK;
  SMOE_CHECK_ARG(peer_bufs && slot_dest && out, "ep_combine: null pointer");
  PeerPtrs pp;
  bool aligned;
  if (int rc = fill_peers(&pp, peer_bufs, world, "ep_combine", &aligned)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SMOE_F32: return combine_typed<float>(pp, aligned, peer_stride_rows, slot_dest, gates, stride_gt, stride_gk, out, stride_om, T, k, N, st);
    case SMOE_BF16: return combine_typed<__nv_bfloat16>(pp, aligned, peer_stride_rows, slot_dest, gates, stride_gt, stride_gk, out, stride_om, T, k, N, st);
    case SMOE_F16: return combine_typed<__half>(pp, aligned, peer_stride_rows, slot_dest, gates, stride_gt, stride_gk, out, stride_om, T, k, N, st);
  }
  set_error("ep_combine: unknown dtype %d", dtype);
  return SMOE_ERR_BAD_ARG;
}

extern "C" int smoe_ep_gate_grad(void* const* peer_bufs, int64_t peer_stride_rows, const int64_t* slot_dest,
                                 const void* grad_out, int64_t stride_gom, void* d_gates, int64_t stride_dgt,
                                 int64_t stride_dgk, int64_t T, int32_t k, int32_t N, int32_t world, int32_t dtype,
                                 void* stream) {
  SMOE_CHECK_ARG(T >= 0 && k >= 1 && N >= 0, "ep_gate_grad: bad sizes T=%lld k=%d N=%d", (long long)T, k, N);
  if (T == 0) return SMOE_OK;
  SMOE_CHECK_ARG(peer_bufs && slot_dest && grad_out && d_gates, "ep_gate_grad: null pointer");
  PeerPtrs pp;
  bool aligned;
  if (int rc = fill_peers(&pp, peer_bufs, world, "ep_gate_grad", &aligned)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SMOE_F32: return gate_grad_typed<float>(pp, aligned, peer_stride_rows, slot_dest, grad_out, stride_gom, d_gates, stride_dgt, stride_dgk, T, k, N, st);
    case SMOE_BF16: return gate_grad_typed<__nv_bfloat16>(pp, aligned, peer_stride_rows, slot_dest, grad_out, stride_gom, d_gates, stride_dgt, stride_dgk, T, k, N, st);
    case SMOE_F16: return gate_grad_typed<__half>(pp, aligned, peer_stride_rows, slot_dest, grad_out, stride_gom, d_gates, stride_dgt, stride_dgk, T, k, N, st);
  }
  set_error("ep_gate_grad: unknown dtype %d", dtype);
  return SMOE_ERR_BAD_ARG;
}
