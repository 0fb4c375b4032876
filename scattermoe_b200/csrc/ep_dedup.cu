// Expert-parallel exchange with every token row crossing NVLink ONCE per owning rank instead of once per (token, slot).
//
// With top-k routing over E experts on W ranks a token's k slots land on fewer than k distinct ranks (k = 8, W = 8:
// 5.25 on average; W = 2: both ranks, i.e. 2 instead of 8). The per-slot exchange (ep.cu) pushes the same token row
// to an owner once for each of its slots there, and pushes every slot's result row back. Here:
//   dispatch   the token row goes to each owning rank once (smoe_ep_dispatch over the list of distinct (token, rank)
//              pairs), together with 16 bytes per SLOT (smoe_ep_dispatch_meta: where the slot's row must appear in
//              the owner's expert-grouped buffer, which received token row it is, its gate, its return address) and
//              one small record per (token, rank) pair (smoe_ep_plan_tokens: the slots of that token at that owner);
//   expand     the owner copies received token rows into expert order in its own HBM (smoe_ep_expand): a local copy at
//              HBM speed replaces the duplicate NVLink transfers; the grouped GEMMs run on it as before;
//   combine    the owner adds up, per received token row, the (gate-weighted) result rows of that token's slots and
//              pushes ONE row back (smoe_ep_combine); the token owner adds the rows it got from the different owners
//              (smoe_ep_sum_parts).
// In backward the output gradient travels the same way (un-weighted; the owner applies the gate while expanding and
// computes the gate gradient as the dot product with the slot's saved expert output, pushing 4 bytes per slot back).
// The reference has no multi-GPU code; nothing here has a counterpart in it. Plain peer stores only; no kernel waits
// on another GPU (the barrier between phases is the caller's, smoe_ep_barrier).
#include "ep_common.cuh"

namespace smoe {

constexpr int EP_MAX_K = 16;            // slots per token the per-pair record can list
constexpr int TM_HEADER = 4;            // ints before the slot list: source rank, return row, slot count, reserved

__host__ __device__ __forceinline__ int tokmeta_ints(int k) { return ((TM_HEADER + 2 * k + 3) / 4) * 4; }

template <typename T>
__global__ void __launch_bounds__(256)
ep_plan_tokens_kernel(const int64_t* __restrict__ ids, const T* __restrict__ gates, int64_t Tn, int k,
                      const int64_t* __restrict__ pair_rank, const int64_t* __restrict__ pair_slot,
                      const int64_t* __restrict__ pair_offsets, const int64_t* __restrict__ tok_base,
                      const int64_t* __restrict__ slot_pos, const int64_t* __restrict__ offsets,
                      const int64_t* __restrict__ dst_off, int32_t* __restrict__ tok_row, int32_t* __restrict__ tok_parts,
                      PeerPtrs tokmeta, int tm_ints, int64_t cap_tok, int64_t cap_slots, int my_rank, int E, int e_local,
                      int world, int kw) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t pairs = pair_offsets[world - 1];
  pairs = pairs < 0 ? 0 : (pairs > Tn * k ? Tn * k : pairs);
  if (i >= pairs) return;
  const int64_t w64 = pair_rank[i], slot0 = pair_slot[i];
  if (w64 < 0 || w64 >= world || slot0 < 0 || slot0 >= Tn * k) return;
  const int w = static_cast<int>(w64);
  const int64_t t = slot0 / k;
  const int64_t start = w ? pair_offsets[w - 1] : 0;
  const int64_t dest_row = tok_base[w] + (i - start);
  if (dest_row < 0 || dest_row >= cap_tok) return;              // malformed plan: drop the pair
  tok_row[t * world + w] = static_cast<int32_t>(dest_row);
  int32_t rec[TM_HEADER + 2 * EP_MAX_K + 4];
  unsigned mask = 0;
  int count = 0;
  for (int j = 0; j < k; ++j) {
    const int64_t e = ids[t * k + j];
    if (e < 0 || e >= E) continue;
    const int r = static_cast<int>(e / e_local);
    mask |= 1u << r;
    if (r == w) {
      const int64_t m = slot_pos[t * k + j];
      const int64_t seg = e ? offsets[e - 1] : 0;
      const int64_t p = dst_off[e] + (m - seg);
      rec[TM_HEADER + count] = (p >= 0 && p < cap_slots) ? static_cast<int32_t>(p) : -1;
      rec[TM_HEADER + k + count] = __float_as_int(to_f32<T>(gates[t * k + j]));
      ++count;
    }
  }
  for (int j = count; j < k; ++j) { rec[TM_HEADER + j] = -1; rec[TM_HEADER + k + j] = 0; }
  const int c = __popc(mask & ((1u << w) - 1u));                // ordinal of this owner among the token's owners
  if (c == 0) tok_parts[t] = min(__popc(mask), kw);
  rec[0] = my_rank;
  rec[1] = static_cast<int32_t>(t * kw + c);
  rec[2] = count;
  rec[3] = 0;
  for (int j = TM_HEADER + 2 * k; j < tm_ints; ++j) rec[j] = 0;
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<int32_t*>(tokmeta.p[w]) + dest_row * tm_ints);
  for (int q = 0; q < tm_ints / 4; ++q)
    dst[q] = make_uint4(rec[4 * q], rec[4 * q + 1], rec[4 * q + 2], rec[4 * q + 3]);
}

// One thread per position m of this rank's expert-sorted slot list: 16 bytes to the owner, at the position the
// slot's row takes in the owner's expert-grouped buffer.
template <typename T>
__global__ void __launch_bounds__(256)
ep_dispatch_meta_kernel(const int64_t* __restrict__ sorted_e, const int64_t* __restrict__ sorted_idx,
                        const int64_t* __restrict__ offsets, const int64_t* __restrict__ dst_off,
                        const T* __restrict__ gates, const int32_t* __restrict__ tok_row, int k, PeerPtrs meta,
                        int64_t cap_slots, int my_rank, int64_t R, int E, int e_local, int world) {
  const int64_t m = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t live = offsets[E - 1];
  live = live < 0 ? 0 : (live > R ? R : live);
  if (m >= live) return;
  const int64_t e = sorted_e[m], slot = sorted_idx[m];
  if (e < 0 || e >= E || slot < 0 || slot >= R) return;
  const int w = static_cast<int>(e / e_local);
  const int64_t seg = e ? offsets[e - 1] : 0;
  const int64_t p = dst_off[e] + (m - seg);
  if (w >= world || p < 0 || p >= cap_slots) return;
  const int64_t t = slot / k;
  const uint32_t row = static_cast<uint32_t>(tok_row[t * world + w]);
  const uint32_t gbits = static_cast<uint32_t>(__float_as_int(to_f32<T>(gates[slot])));
  const unsigned long long lo = static_cast<unsigned long long>(pack_dest(my_rank, slot));
  const unsigned long long hi = static_cast<unsigned long long>(row) | (static_cast<unsigned long long>(gbits) << 32);
  ulonglong2* dst = reinterpret_cast<ulonglong2*>(meta.p[w]) + p;
  *dst = make_ulonglong2(lo, hi);
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(h[i]); f[2 * i + 1] = __high2float(h[i]); }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& v, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(h[i]); f[2 * i + 1] = __high2float(h[i]); }
}
template <typename T>
__device__ __forceinline__ uint4 pack8f(const float (&f)[8]);
template <>
__device__ __forceinline__ uint4 pack8f<__nv_bfloat16>(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
template <>
__device__ __forceinline__ uint4 pack8f<__half>(const float (&f)[8]) {
  uint4 v;
  __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// Owner side, one warp per live slot position p: out[p] = tok[row(p)] (* gate(p)); with `y` also the gate gradient
// <y[p], tok[row(p)]> (un-weighted), stored as fp32 at the slot's return address on the token owner.
template <typename T>
__global__ void __launch_bounds__(256)
ep_expand_kernel(const T* __restrict__ tok, int64_t stok, int64_t cap_tok, const ulonglong2* __restrict__ meta,
                 const int64_t* __restrict__ live_slots, int64_t cap_slots, int scale, T* __restrict__ out, int64_t sout,
                 const T* __restrict__ y, int64_t sy, PeerPtrs dgate, int64_t peer_slots, int K, int world) {
  const int lane = threadIdx.x & 31;
  const int64_t live = min(cap_slots, *live_slots);
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); p < live;
       p += static_cast<int64_t>(gridDim.x) * 8) {
    const ulonglong2 mt = meta[p];
    const int64_t row = static_cast<int64_t>(static_cast<uint32_t>(mt.y & 0xffffffffull));
    const float g = __int_as_float(static_cast<int>(mt.y >> 32));
    if (row >= cap_tok) continue;                                // malformed record: leave the row
    const uint4* src = reinterpret_cast<const uint4*>(tok + row * stok);
    uint4* dst = reinterpret_cast<uint4*>(out + p * sout);
    const uint4* yy = y ? reinterpret_cast<const uint4*>(y + p * sy) : nullptr;
    float dot = 0.f;
    for (int i = lane; i < K / 8; i += 32) {
      uint4 v = __ldg(src + i);
      if (scale || yy) {
        float f[8];
        unpack8<T>(v, f);
        if (yy) {
          float fy[8];
          unpack8<T>(__ldg(yy + i), fy);
#pragma unroll
          for (int j = 0; j < 8; ++j) dot = fmaf(f[j], fy[j], dot);
        }
        if (scale) {
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] *= g;
          v = pack8f<T>(f);
        }
      }
      dst[i] = v;
    }
    if (yy) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (lane == 0) {
        const int64_t d = static_cast<int64_t>(mt.x);
        const int rank = dest_rank(d);
        const int64_t slot = dest_row(d);
        if (rank >= 0 && rank < world && slot < peer_slots) reinterpret_cast<float*>(dgate.p[rank])[slot] = dot;
      }
    }
  }
}

// Owner side, one warp per received token row u: the (gate-weighted) sum of the result rows of that token's slots
// here, pushed to its return row on the token owner. Token rows are ordered by sending rank; owner r starts with
// the rows of rank r+1 and wraps, so that the owners address different ranks at any moment.
template <typename T>
__global__ void __launch_bounds__(256)
ep_combine_kernel(const T* __restrict__ rows, int64_t srows, int64_t cap_slots, const int32_t* __restrict__ tokmeta,
                  int tm_ints, const int64_t* __restrict__ live_tok, int64_t cap_tok, const int64_t* __restrict__ src_base,
                  int use_gates, PeerPtrs comb, int64_t scomb, int64_t peer_rows, int K, int k, int my_rank, int world) {
  const int lane = threadIdx.x & 31;
  const int64_t live = min(cap_tok, *live_tok);
  int64_t shift = src_base ? src_base[(my_rank + 1) % world] : 0;
  shift = shift < 0 ? 0 : (shift >= live ? 0 : shift);
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); j < live;
       j += static_cast<int64_t>(gridDim.x) * 8) {
    int64_t u = j + shift;
    if (u >= live) u -= live;
    const int32_t* tm = tokmeta + u * tm_ints;
    const int src = tm[0];
    const int64_t ret_row = tm[1];
    const int cnt = min(tm[2], k);
    if (src < 0 || src >= world || ret_row < 0 || ret_row >= peer_rows) continue;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(comb.p[src]) + ret_row * scomb);
    for (int i = lane; i < K / 8; i += 32) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      for (int c = 0; c < cnt; ++c) {
        const int64_t p = tm[TM_HEADER + c];
        if (p < 0 || p >= cap_slots) continue;
        const float g = use_gates ? __int_as_float(tm[TM_HEADER + k + c]) : 1.0f;
        float f[8];
        unpack8<T>(__ldg(reinterpret_cast<const uint4*>(rows + p * srows) + i), f);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = fmaf(g, f[q], acc[q]);
      }
      dst[i] = pack8f<T>(acc);
    }
  }
}

// Token owner: out[t] = sum of the parts[t] rows (t * kw + c, c < parts[t]) the owners sent back.
template <typename T>
__global__ void __launch_bounds__(128)
ep_sum_parts_kernel(const T* __restrict__ comb, int64_t scomb, const int32_t* __restrict__ parts, int kw,
                    T* __restrict__ out, int64_t sout, int K) {
  const int64_t t = blockIdx.x;
  const int n = min(max(parts[t], 0), kw);
  for (int i = threadIdx.x; i < K / 8; i += 128) {
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    for (int c = 0; c < n; ++c) {
      float f[8];
      unpack8<T>(__ldg(reinterpret_cast<const uint4*>(comb + (t * kw + c) * scomb) + i), f);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += f[q];
    }
    reinterpret_cast<uint4*>(out + t * sout)[i] = pack8f<T>(acc);
  }
}

static int check16(const char* who, int dtype, int K) {
  if (dtype != SMOE_BF16 && dtype != SMOE_F16) {
    set_error("%s: 16-bit dtypes only (got %d)", who, dtype);
    return SMOE_ERR_BAD_ARG;
  }
  if (K % 8) {
    set_error("%s: the row width %d must be a multiple of 8", who, K);
    return SMOE_ERR_BAD_ARG;
  }
  return SMOE_OK;
}

static unsigned capped_grid(int64_t units_of_8_rows) {
  const int64_t want = units_of_8_rows > 0 ? units_of_8_rows : 1;
  return static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
}

}  // namespace smoe

using namespace smoe;

extern "C" int32_t smoe_ep_tokmeta_ints(int32_t k) { return (k >= 1 && k <= EP_MAX_K) ? tokmeta_ints(k) : 0; }

extern "C" int smoe_ep_plan_tokens(const int64_t* expert_idxs, const void* gates, int64_t T, int32_t k,
                                   const int64_t* pair_rank, const int64_t* pair_slot, const int64_t* pair_offsets,
                                   const int64_t* tok_base, const int64_t* slot_pos, const int64_t* expert_offsets,
                                   const int64_t* dst_offsets, int32_t* tok_row, int32_t* tok_parts,
                                   void* const* peer_tokmeta, int64_t cap_tok, int64_t cap_slots, int32_t my_rank,
                                   int32_t E, int32_t world, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(T >= 0 && k >= 1 && k <= EP_MAX_K, "ep_plan_tokens: T=%lld, k=%d (k <= %d)", (long long)T, k, EP_MAX_K);
  SMOE_CHECK_ARG(world >= 1 && world <= EP_MAX_WORLD && E >= 1 && E % world == 0, "ep_plan_tokens: E=%d, world=%d", E, world);
  SMOE_CHECK_ARG(my_rank >= 0 && my_rank < world, "ep_plan_tokens: rank %d of %d", my_rank, world);
  SMOE_CHECK_ARG(cap_tok < (int64_t(1) << 31) && cap_slots < (int64_t(1) << 31), "ep_plan_tokens: capacity too large");
  if (int rc = check16("ep_plan_tokens", dtype, 8)) return rc;
  if (T == 0) return SMOE_OK;
  SMOE_CHECK_ARG(expert_idxs && gates && pair_rank && pair_slot && pair_offsets && tok_base && slot_pos &&
                 expert_offsets && dst_offsets && tok_row && tok_parts && peer_tokmeta, "ep_plan_tokens: null pointer");
  PeerPtrs pp;
  bool aligned;
  if (int rc = fill_peers(&pp, peer_tokmeta, world, "ep_plan_tokens", &aligned)) return rc;
  SMOE_CHECK_ARG(aligned, "ep_plan_tokens: the record buffers must be 16-byte aligned");
  const int64_t n = T * k;
  const unsigned grid = static_cast<unsigned>(cdiv64(n, 256));
  const int kw = k < world ? k : world;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SMOE_BF16)
    ep_plan_tokens_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(expert_idxs, static_cast<const __nv_bfloat16*>(gates), T, k,
        pair_rank, pair_slot, pair_offsets, tok_base, slot_pos, expert_offsets, dst_offsets, tok_row, tok_parts, pp,
        tokmeta_ints(k), cap_tok, cap_slots, my_rank, E, E / world, world, kw);
  else
    ep_plan_tokens_kernel<__half><<<grid, 256, 0, st>>>(expert_idxs, static_cast<const __half*>(gates), T, k,
        pair_rank, pair_slot, pair_offsets, tok_base, slot_pos, expert_offsets, dst_offsets, tok_row, tok_parts, pp,
        tokmeta_ints(k), cap_tok, cap_slots, my_rank, E, E / world, world, kw);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

extern "C" int smoe_ep_dispatch_meta(const int64_t* sorted_expert_idxs, const int64_t* sorted_scattered_idxs,
                                     const int64_t* expert_offsets, const int64_t* dst_offsets, const void* gates,
                                     const int32_t* tok_row, int32_t k, void* const* peer_meta, int64_t cap_slots,
                                     int32_t my_rank, int64_t R, int32_t E, int32_t world, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(R >= 0 && k >= 1 && E >= 1 && world >= 1 && E % world == 0, "ep_dispatch_meta: R=%lld k=%d E=%d world=%d",
                 (long long)R, k, E, world);
  SMOE_CHECK_ARG(my_rank >= 0 && my_rank < world, "ep_dispatch_meta: rank %d of %d", my_rank, world);
  if (int rc = check16("ep_dispatch_meta", dtype, 8)) return rc;
  if (R == 0) return SMOE_OK;
  SMOE_CHECK_ARG(sorted_expert_idxs && sorted_scattered_idxs && expert_offsets && dst_offsets && gates && tok_row &&
                 peer_meta, "ep_dispatch_meta: null pointer");
  PeerPtrs pp;
  bool aligned;
  if (int rc = fill_peers(&pp, peer_meta, world, "ep_dispatch_meta", &aligned)) return rc;
  SMOE_CHECK_ARG(aligned, "ep_dispatch_meta: the record buffers must be 16-byte aligned");
  const unsigned grid = static_cast<unsigned>(cdiv64(R, 256));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SMOE_BF16)
    ep_dispatch_meta_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
        dst_offsets, static_cast<const __nv_bfloat16*>(gates), tok_row, k, pp, cap_slots, my_rank, R, E, E / world, world);
  else
    ep_dispatch_meta_kernel<__half><<<grid, 256, 0, st>>>(sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
        dst_offsets, static_cast<const __half*>(gates), tok_row, k, pp, cap_slots, my_rank, R, E, E / world, world);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

extern "C" int smoe_ep_expand(const void* tok_rows, int64_t stride_tok, int64_t cap_tok, const void* meta,
                              const int64_t* live_slots, int64_t cap_slots, int32_t scale_by_gate, void* out,
                              int64_t stride_out, const void* y_rows, int64_t stride_y, void* const* peer_dgate,
                              int64_t peer_slots, int32_t K, int32_t world, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(cap_tok >= 0 && cap_slots >= 0 && K >= 0, "ep_expand: bad sizes");
  if (int rc = check16("ep_expand", dtype, K)) return rc;
  if (cap_slots == 0 || K == 0) return SMOE_OK;
  SMOE_CHECK_ARG(tok_rows && meta && live_slots && out, "ep_expand: null pointer");
  SMOE_CHECK_ARG(stride_tok % 8 == 0 && stride_out % 8 == 0 && a16(tok_rows) && a16(out) && a16(meta),
                 "ep_expand: rows must be 16-byte aligned");
  PeerPtrs pp;
  for (int i = 0; i < EP_MAX_WORLD; ++i) pp.p[i] = nullptr;
  if (y_rows) {
    SMOE_CHECK_ARG(peer_dgate != nullptr && stride_y % 8 == 0 && a16(y_rows), "ep_expand: gate-gradient arguments");
    bool aligned;
    if (int rc = fill_peers(&pp, peer_dgate, world, "ep_expand", &aligned)) return rc;
  }
  const unsigned grid = capped_grid(cdiv64(cap_slots, 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SMOE_BF16)
    ep_expand_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(tok_rows), stride_tok, cap_tok,
        static_cast<const ulonglong2*>(meta), live_slots, cap_slots, scale_by_gate ? 1 : 0, static_cast<__nv_bfloat16*>(out),
        stride_out, static_cast<const __nv_bfloat16*>(y_rows), stride_y, pp, peer_slots, K, world);
  else
    ep_expand_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(tok_rows), stride_tok, cap_tok,
        static_cast<const ulonglong2*>(meta), live_slots, cap_slots, scale_by_gate ? 1 : 0, static_cast<__half*>(out),
        stride_out, static_cast<const __half*>(y_rows), stride_y, pp, peer_slots, K, world);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

extern "C" int smoe_ep_combine(const void* rows, int64_t stride_rows, int64_t cap_slots, const int32_t* tokmeta,
                               const int64_t* live_tok, int64_t cap_tok, const int64_t* src_base, int32_t use_gates,
                               void* const* peer_comb, int64_t peer_stride, int64_t peer_rows, int32_t K, int32_t k,
                               int32_t my_rank, int32_t world, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(cap_tok >= 0 && cap_slots >= 0 && K >= 0 && k >= 1 && k <= EP_MAX_K, "ep_combine: bad sizes (k=%d)", k);
  SMOE_CHECK_ARG(my_rank >= 0 && my_rank < world, "ep_combine: rank %d of %d", my_rank, world);
  if (int rc = check16("ep_combine", dtype, K)) return rc;
  if (cap_tok == 0 || K == 0) return SMOE_OK;
  SMOE_CHECK_ARG(rows && tokmeta && live_tok && peer_comb, "ep_combine: null pointer");
  SMOE_CHECK_ARG(stride_rows % 8 == 0 && peer_stride % 8 == 0 && a16(rows), "ep_combine: rows must be 16-byte aligned");
  PeerPtrs pp;
  bool aligned;
  if (int rc = fill_peers(&pp, peer_comb, world, "ep_combine", &aligned)) return rc;
  SMOE_CHECK_ARG(aligned, "ep_combine: the return buffers must be 16-byte aligned");
  const unsigned grid = capped_grid(cdiv64(cap_tok, 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SMOE_BF16)
    ep_combine_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows), stride_rows, cap_slots,
        tokmeta, tokmeta_ints(k), live_tok, cap_tok, src_base, use_gates ? 1 : 0, pp, peer_stride, peer_rows, K, k, my_rank,
        world);
  else
    ep_combine_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(rows), stride_rows, cap_slots, tokmeta,
        tokmeta_ints(k), live_tok, cap_tok, src_base, use_gates ? 1 : 0, pp, peer_stride, peer_rows, K, k, my_rank, world);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

extern "C" int smoe_ep_sum_parts(const void* comb, int64_t stride_comb, const int32_t* parts, int32_t kw, void* out,
                                 int64_t stride_out, int64_t T, int32_t K, int32_t dtype, void* stream) {
  SMOE_CHECK_ARG(T >= 0 && kw >= 1 && K >= 0, "ep_sum_parts: bad sizes T=%lld kw=%d K=%d", (long long)T, kw, K);
  if (int rc = check16("ep_sum_parts", dtype, K)) return rc;
  if (T == 0 || K == 0) return SMOE_OK;
  SMOE_CHECK_ARG(comb && parts && out, "ep_sum_parts: null pointer");
  SMOE_CHECK_ARG(T < (int64_t(1) << 31) && stride_comb % 8 == 0 && stride_out % 8 == 0 && a16(comb) && a16(out),
                 "ep_sum_parts: rows must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SMOE_BF16)
    ep_sum_parts_kernel<__nv_bfloat16><<<static_cast<unsigned>(T), 128, 0, st>>>(static_cast<const __nv_bfloat16*>(comb),
        stride_comb, parts, kw, static_cast<__nv_bfloat16*>(out), stride_out, K);
  else
    ep_sum_parts_kernel<__half><<<static_cast<unsigned>(T), 128, 0, st>>>(static_cast<const __half*>(comb), stride_comb, parts,
        kw, static_cast<__half*>(out), stride_out, K);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}
