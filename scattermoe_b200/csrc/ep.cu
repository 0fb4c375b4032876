// Expert-parallel row exchange over NVLink peer memory (plain P2P stores, no multicast, no flags, no waits).
//
// The reference has no multi-GPU code; these kernels replace what a NCCL all-to-all-v based expert-parallel layer
// does around the local grouped GEMMs (pack rows by destination -> all-to-all-v -> regroup by expert, and the way
// back) with ONE pass each way and no intermediate copies. Both directions PUSH (remote stores are fire-and-forget;
// a first version that pulled rows with remote loads was latency-bound and slower than NCCL at 8 GPUs):
//   dispatch  every (token, slot) row is written straight into the owning rank's receive buffer at the position
//             that makes that buffer expert-grouped (all ranks know all counts, so every row's final position is
//             computable at the sender), together with its return address (sender rank, slot); an optional
//             per-slot coefficient (the gate, in backward) is applied on the fly. The receiver runs its grouped
//             GEMMs on the buffer as is: no sort, no regroup copy.
//   return    every live row of the owner's result buffer is written to its return address: the sender's
//             slot-ordered (T*k, d) buffer, where the gate-weighted top-k sum and the gate gradient are local.
// Synchronisation between the phases is the caller's (a stream-ordered barrier across the ranks); the kernels
// themselves never wait on another GPU.
#include "ep_common.cuh"

namespace smoe {

// One warp per sorted position m. Row m belongs to global expert e = sorted_e[m], owned by rank e / e_local; its
// position in the owner's buffer is dst_off[e] + (m - first position of e in this rank's sorted list).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const T* __restrict__ X, int64_t x_rows, int64_t sxm, const int64_t* __restrict__ sorted_e,
                   const int64_t* __restrict__ sorted_idx, const int64_t* __restrict__ offsets,
                   const int64_t* __restrict__ dst_off, const T* __restrict__ coeff, int fan_out, PeerPtrs peers,
                   int64_t peer_row_elems, int64_t cap_rows, PeerPtrs ret_peers, int my_rank, int64_t R, int K, int E,
                   int e_local, int world) {
  const int lane = threadIdx.x & 31;
  int64_t m = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  // the sorted list may be shorter than R (ids outside [0, E) are not part of it): its length is the last offset
  int64_t live = offsets[E - 1];
  live = live < 0 ? 0 : (live > R ? R : live);
  if (m >= live) return;
  // Rank r starts with the rows of rank r+1's experts and wraps around: at any moment the ranks are then writing
  // to DIFFERENT owners. In plain sorted order every rank would first write to rank 0, then all to rank 1, ...:
  // eight senders into one receiver's NVLink ingress at a time.
  {
    const int first = ((my_rank + 1) % world) * e_local;
    int64_t shift = first ? offsets[first - 1] : 0;
    shift = shift < 0 ? 0 : (shift > live ? live : shift);
    m += shift;
    if (m >= live) m -= live;
  }
  const int64_t e = sorted_e[m];
  const int64_t slot = sorted_idx[m];
  if (e < 0 || e >= E || slot < 0 || slot >= R) return;
  const int64_t src = slot / fan_out;
  const int rank = static_cast<int>(e / e_local);
  const int64_t seg_start = e ? offsets[e - 1] : 0;
  const int64_t row = dst_off[e] + (m - seg_start);
  if (src >= x_rows || rank >= world || row < 0 || row >= cap_rows) return;   // malformed plan: drop the row
  if (lane == 0 && ret_peers.p[rank]) reinterpret_cast<int64_t*>(ret_peers.p[rank])[row] = pack_dest(my_rank, slot);
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

// One warp per row of the owner's result buffer; rows at or beyond the live count (a device scalar) are skipped.
// Row i goes to rank r's slot-ordered buffer at the slot recorded in ret_addr[i].
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
ep_return_kernel(const T* __restrict__ Y, int64_t sym, const int64_t* __restrict__ ret_addr,
                 const int64_t* __restrict__ live_rows, int64_t cap_rows, PeerPtrs peers, int64_t peer_row_elems,
                 int64_t peer_rows, int K, int world, int64_t row_shift_num, int64_t row_shift_den) {
  const int lane = threadIdx.x & 31;
  const int64_t live = min(cap_rows, *live_rows);
  // The buffer is ordered (local expert, sending rank): walked from row 0 every owner would be returning rows to
  // the same rank at the same time. Owner r starts r sub-segments in (live * r / (local experts * world) rows) and
  // wraps, so that the owners address different ranks at any moment (exactly so when the load is even).
  const int64_t shift = row_shift_den > 0 ? (live * row_shift_num / row_shift_den) : 0;
  // grid-stride over the live rows: the grid is sized for the device, not for the (much larger) capacity
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); j < live;
       j += static_cast<int64_t>(gridDim.x) * 8) {
    int64_t i = j + shift;
    if (i >= live) i -= live;
    const int64_t d = ret_addr[i];
    const int rank = dest_rank(d);
    const int64_t slot = dest_row(d);
    if (rank < 0 || rank >= world || slot >= peer_rows) continue;      // malformed return address: drop the row
    const T* y = Y + i * sym;
    T* o = reinterpret_cast<T*>(peers.p[rank]) + slot * peer_row_elems;
    if (VEC) {
      constexpr int V = V16<T>::N;
      const uint4* y4 = reinterpret_cast<const uint4*>(y);
      uint4* o4 = reinterpret_cast<uint4*>(o);
      for (int c = lane; c < K / V; c += 32) o4[c] = y4[c];
    } else {
      for (int c = lane; c < K; c += 32) o[c] = y[c];
    }
  }
}

// Barrier across the ranks through peer memory. Every rank owns an int32 slot per peer; rank r announces epoch
// n by storing n into slot r of every rank's array (release, system scope, after a system fence so that the
// rows this rank pushed earlier on the stream are visible first) and then waits until all of its own slots have
// reached n (acquire, system scope). Epochs only grow, so a fast peer that is already one barrier ahead is
// fine. The wait is bounded: after ~1 s of SM clocks it records (2, 100, peer, epoch) in `status` and returns, so
// a lost rank can never hang this GPU. One block of 32 threads, thread w talks to rank w. What ran on the strength of
// an expired barrier has read rows that had not arrived: callers follow their last barrier with
// smoe_status_poison on their results, so that the step yields NaNs instead of plausible numbers.
constexpr long long EP_BARRIER_LIMIT_CYCLES = 2000000000LL;

__global__ void __launch_bounds__(32)
ep_barrier_kernel(PeerPtrs flags, int my_rank, int world, int epoch, long long limit_cycles, int32_t* status) {
  const int w = threadIdx.x;
  if (w >= world) return;
  __threadfence_system();
  int* remote = reinterpret_cast<int*>(flags.p[w]) + my_rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const int* mine = reinterpret_cast<const int*>(flags.p[my_rank]) + w;
  const long long t0 = clock64();
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) break;
    if (clock64() - t0 > limit_cycles) {
      if (status && atomicCAS(status, 0, 2) == 0) {
        status[1] = 100;
        status[2] = w;
        status[3] = epoch;
      }
      break;
    }
    __nanosleep(64);
  }
}

// Where this rank's rows go and what it will hold, from every rank's expert offsets (one block; replaces a dozen
// small tensor operations between the counts all-gather and the dispatch). all_offsets is (world, E): row s = the
// inclusive per-expert ends of sender s's expert-sorted slot list. With count[s][e] the differences:
//   dst_off[e]       = (slots of all senders for the experts before e on e's owner) + (slots of senders < rank for e)
//   local_offsets[j] = inclusive ends of this rank's own experts over all senders' slots
// i.e. every owner's buffer is ordered (local expert, sender), which is what ep_dispatch_kernel fills.
__global__ void __launch_bounds__(256)
ep_plan_rows_kernel(const int64_t* __restrict__ all_offsets, int my_rank, int world, int E, int e_local,
                    int64_t* __restrict__ dst_off, int64_t* __restrict__ local_offsets) {
  extern __shared__ int64_t plan_tot[];          // E totals over the senders
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int64_t tot = 0, before = 0;
    for (int s = 0; s < world; ++s) {
      const int64_t* row = all_offsets + static_cast<int64_t>(s) * E;
      int64_t c = row[e] - (e ? row[e - 1] : 0);
      c = c < 0 ? 0 : c;
      tot += c;
      if (s < my_rank) before += c;
    }
    plan_tot[e] = tot;
    dst_off[e] = before;                         // completed below, once every total is known
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int first = (e / e_local) * e_local;
    int64_t base = 0;
    for (int j = first; j < e; ++j) base += plan_tot[j];
    dst_off[e] += base;
    if (e / e_local == my_rank) local_offsets[e - first] = base + plan_tot[e];
  }
}

template <typename T>
static int dispatch_typed(const void* X, int64_t x_rows, int64_t sxm, const int64_t* sorted_e, const int64_t* sorted_idx,
                          const int64_t* offsets, const int64_t* dst_off, const void* coeff, int fan_out,
                          const PeerPtrs& pp, bool aligned, int64_t peer_row_elems, int64_t cap_rows,
                          const PeerPtrs& ret, int my_rank, int64_t R, int K, int E, int e_local, int world,
                          cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = aligned && K % V == 0 && sxm % V == 0 && peer_row_elems % V == 0 && a16(X);
  const unsigned grid = static_cast<unsigned>(cdiv64(R, 8));
  if (vec)
    ep_dispatch_kernel<T, true><<<grid, 256, 0, st>>>((const T*)X, x_rows, sxm, sorted_e, sorted_idx, offsets, dst_off,
                                                      (const T*)coeff, fan_out, pp, peer_row_elems, cap_rows, ret, my_rank,
                                                      R, K, E, e_local, world);
  else
    ep_dispatch_kernel<T, false><<<grid, 256, 0, st>>>((const T*)X, x_rows, sxm, sorted_e, sorted_idx, offsets, dst_off,
                                                       (const T*)coeff, fan_out, pp, peer_row_elems, cap_rows, ret, my_rank,
                                                       R, K, E, e_local, world);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

template <typename T>
static int return_typed(const void* Y, int64_t sym, const int64_t* ret_addr, const int64_t* live_rows, int64_t cap_rows,
                        const PeerPtrs& pp, bool aligned, int64_t peer_row_elems, int64_t peer_rows, int K, int world,
                        int64_t shift_num, int64_t shift_den, cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = aligned && K % V == 0 && sym % V == 0 && peer_row_elems % V == 0 && a16(Y);
  const int64_t want = cdiv64(cap_rows, 8);
  const unsigned grid = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
  if (vec)
    ep_return_kernel<T, true><<<grid, 256, 0, st>>>((const T*)Y, sym, ret_addr, live_rows, cap_rows, pp, peer_row_elems,
                                                    peer_rows, K, world, shift_num, shift_den);
  else
    ep_return_kernel<T, false><<<grid, 256, 0, st>>>((const T*)Y, sym, ret_addr, live_rows, cap_rows, pp, peer_row_elems,
                                                     peer_rows, K, world, shift_num, shift_den);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

}  // namespace smoe

using namespace smoe;

extern "C" int smoe_ep_dispatch(const void* X, int64_t x_rows, int64_t stride_xm, const int64_t* sorted_expert_idxs,
                                const int64_t* sorted_scattered_idxs, const int64_t* expert_offsets,
                                const int64_t* dst_offsets, const void* coeff, int32_t fan_out, void* const* peer_bufs,
                                int64_t peer_stride_rows, int64_t capacity_rows, void* const* peer_return_addr,
                                int32_t my_rank, int64_t R, int32_t K, int32_t E, int32_t world, int32_t dtype,
                                void* stream) {
  SMOE_CHECK_ARG(R >= 0 && K >= 0 && E >= 1 && fan_out >= 1, "ep_dispatch: bad sizes R=%lld K=%d E=%d fan_out=%d",
                 (long long)R, K, E, fan_out);
  SMOE_CHECK_ARG(world >= 1 && E % world == 0, "ep_dispatch: E=%d is not divisible by the world size %d", E, world);
  SMOE_CHECK_ARG(my_rank >= 0 && my_rank < world, "ep_dispatch: rank %d outside the world of %d", my_rank, world);
  SMOE_CHECK_ARG(capacity_rows < (int64_t(1) << 40) && R < (int64_t(1) << 40), "ep_dispatch: capacity too large");
  if (R == 0 || K == 0) return SMOE_OK;
  SMOE_CHECK_ARG(X && sorted_expert_idxs && sorted_scattered_idxs && expert_offsets && dst_offsets && peer_bufs,
                 "ep_dispatch: null pointer");
  PeerPtrs pp, ret;
  bool aligned, ret_aligned;
  if (int rc = fill_peers(&pp, peer_bufs, world, "ep_dispatch", &aligned)) return rc;
  if (peer_return_addr) {
    if (int rc = fill_peers(&ret, peer_return_addr, world, "ep_dispatch", &ret_aligned)) return rc;
  } else {
    for (int i = 0; i < EP_MAX_WORLD; ++i) ret.p[i] = nullptr;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int e_local = E / world;
  switch (dtype) {
    case SMOE_F32: return dispatch_typed<float>(X, x_rows, stride_xm, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, dst_offsets, coeff, fan_out, pp, aligned, peer_stride_rows, capacity_rows, ret, my_rank, R, K, E, e_local, world, st);
    case SMOE_BF16: return dispatch_typed<__nv_bfloat16>(X, x_rows, stride_xm, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, dst_offsets, coeff, fan_out, pp, aligned, peer_stride_rows, capacity_rows, ret, my_rank, R, K, E, e_local, world, st);
    case SMOE_F16: return dispatch_typed<__half>(X, x_rows, stride_xm, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, dst_offsets, coeff, fan_out, pp, aligned, peer_stride_rows, capacity_rows, ret, my_rank, R, K, E, e_local, world, st);
  }
  set_error("ep_dispatch: unknown dtype %d", dtype);
  return SMOE_ERR_BAD_ARG;
}

extern "C" int smoe_ep_plan_rows(const int64_t* all_offsets, int32_t my_rank, int32_t world, int32_t E,
                                 int64_t* dst_offsets, int64_t* local_offsets, void* stream) {
  SMOE_CHECK_ARG(world >= 1 && world <= EP_MAX_WORLD && E >= 1 && E <= 4096 && E % world == 0,
                 "ep_plan_rows: E=%d (<= 4096), world=%d", E, world);
  SMOE_CHECK_ARG(my_rank >= 0 && my_rank < world, "ep_plan_rows: rank %d of %d", my_rank, world);
  SMOE_CHECK_ARG(all_offsets && dst_offsets && local_offsets, "ep_plan_rows: null pointer");
  ep_plan_rows_kernel<<<1, 256, static_cast<size_t>(E) * sizeof(int64_t), static_cast<cudaStream_t>(stream)>>>(
      all_offsets, my_rank, world, E, E / world, dst_offsets, local_offsets);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

extern "C" int smoe_ep_return(const void* Y, int64_t stride_ym, const int64_t* return_addr, const int64_t* live_rows,
                              int64_t capacity_rows, void* const* peer_slot_bufs, int64_t peer_stride_rows,
                              int64_t peer_rows, int32_t K, int32_t world, int32_t my_rank, int32_t local_experts,
                              int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(capacity_rows >= 0 && K >= 0, "ep_return: bad sizes rows=%lld K=%d", (long long)capacity_rows, K);
  SMOE_CHECK_ARG(my_rank >= 0 && my_rank < world && local_experts >= 1, "ep_return: rank %d of %d, %d local experts",
                 my_rank, world, local_experts);
  const int64_t shift_num = my_rank, shift_den = static_cast<int64_t>(local_experts) * world;
  if (capacity_rows == 0 || K == 0) return SMOE_OK;
  SMOE_CHECK_ARG(Y && return_addr && live_rows && peer_slot_bufs, "ep_return: null pointer");
  PeerPtrs pp;
  bool aligned;
  if (int rc = fill_peers(&pp, peer_slot_bufs, world, "ep_return", &aligned)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SMOE_F32: return return_typed<float>(Y, stride_ym, return_addr, live_rows, capacity_rows, pp, aligned, peer_stride_rows, peer_rows, K, world, shift_num, shift_den, st);
    case SMOE_BF16: return return_typed<__nv_bfloat16>(Y, stride_ym, return_addr, live_rows, capacity_rows, pp, aligned, peer_stride_rows, peer_rows, K, world, shift_num, shift_den, st);
    case SMOE_F16: return return_typed<__half>(Y, stride_ym, return_addr, live_rows, capacity_rows, pp, aligned, peer_stride_rows, peer_rows, K, world, shift_num, shift_den, st);
  }
  set_error("ep_return: unknown dtype %d", dtype);
  return SMOE_ERR_BAD_ARG;
}

extern "C" int smoe_ep_barrier(void* const* peer_flags, int32_t my_rank, int32_t world, int32_t epoch,
                               int64_t limit_cycles, int32_t* status, void* stream) {
  SMOE_CHECK_ARG(peer_flags != nullptr, "ep_barrier: null pointer");
  SMOE_CHECK_ARG(my_rank >= 0 && my_rank < world && epoch > 0, "ep_barrier: rank %d of %d, epoch %d", my_rank, world, epoch);
  PeerPtrs pp;
  bool aligned;
  if (int rc = fill_peers(&pp, peer_flags, world, "ep_barrier", &aligned)) return rc;
  SMOE_CHECK_ARG(limit_cycles >= 0, "ep_barrier: negative wait limit");
  const long long limit = limit_cycles > 0 ? static_cast<long long>(limit_cycles) : EP_BARRIER_LIMIT_CYCLES;
  ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pp, my_rank, world, epoch, limit, status);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

// Fills `buf` with 0xFF bytes (NaN in every floating-point format this library stores) if the status word says that
// a bounded wait ran out. Reads one int and returns otherwise.
__global__ void __launch_bounds__(256)
status_poison_kernel(const int32_t* __restrict__ status, uint8_t* __restrict__ buf, int64_t bytes) {
  if (status[0] == 0) return;
  int64_t head = (16 - static_cast<int64_t>(reinterpret_cast<uintptr_t>(buf) & 15)) & 15;
  head = head < bytes ? head : bytes;
  uint4* body = reinterpret_cast<uint4*>(buf + head);
  const int64_t n16 = (bytes - head) / 16;
  const uint4 ff = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    body[i] = ff;
  if (blockIdx.x == 0) {
    for (int64_t i = threadIdx.x; i < head; i += blockDim.x) buf[i] = 0xff;
    for (int64_t i = head + n16 * 16 + threadIdx.x; i < bytes; i += blockDim.x) buf[i] = 0xff;
  }
}

extern "C" int smoe_status_poison(const int32_t* status, void* buf, int64_t bytes, void* stream) {
  SMOE_CHECK_ARG(bytes >= 0, "status_poison: negative size");
  if (bytes == 0) return SMOE_OK;
  SMOE_CHECK_ARG(status && buf, "status_poison: null pointer");
  const int64_t want = cdiv64(bytes / 16 + 1, 256);
  const unsigned grid = static_cast<unsigned>(want < 148 * 4 ? want : 148 * 4);
  status_poison_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(status, static_cast<uint8_t*>(buf), bytes);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}
