// Shared by the expert-parallel exchange kernels (ep.cu, ep_dedup.cu): the table of peer pointers a kernel receives
// by value, the (rank, row) return-address packing, and the host-side check of a caller's pointer table.
#pragma once

#include "smoe_common.cuh"

namespace smoe {

constexpr int EP_MAX_WORLD = 16;
struct PeerPtrs { uint8_t* p[EP_MAX_WORLD]; };

__device__ __forceinline__ int64_t pack_dest(int rank, int64_t row) { return (static_cast<int64_t>(rank) << 40) | row; }
__device__ __forceinline__ int dest_rank(int64_t d) { return static_cast<int>(d >> 40); }
__device__ __forceinline__ int64_t dest_row(int64_t d) { return d & ((int64_t(1) << 40) - 1); }

template <typename T> struct V16 { static constexpr int N = 16 / sizeof(T); };


static inline bool a16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static inline int fill_peers(PeerPtrs* pp, void* const* peer_bufs, int world, const char* who, bool* all_aligned) {
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

}  // namespace smoe
