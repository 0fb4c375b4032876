// tcgen05 (5th-generation tensor core) grouped GEMM with fused row gather / scatter for sm_100a.
//
//   Y[out(m), :] = X[in(m), :] @ W[e(m)] (+ bias[e(m)])      for every position m of the expert-sorted slot list
//
// replaces the reference's Triton kernel _scatter2scatter (scattermoe/kernels/ops.py:55-118). Design:
//   * persistent CTAs (one per SM) walk a tile list derived on the device from the expert offsets; a tile is
//     128 sorted positions of ONE expert x BN output columns, so no row of another expert is ever multiplied
//     (the reference instead masks rows and repeats the K loop per expert, ops.py:87-107);
//   * warp-specialised roles: one warp feeds the expert's weight tiles with TMA (3-D tensor map over
//     (inner, outer, expert), 128-byte swizzle), four warps gather the token rows with 16-byte cp.async
//     straight into the same swizzled layout (no padded or grouped copy of X exists), one thread issues
//     tcgen05.mma (128 x BN x 16, bf16/fp16 in, fp32 accumulators in tensor memory), four warps run the
//     epilogue (tcgen05.ld -> bias -> convert -> scattered or grouped row stores);
//   * the accumulator is double-buffered in tensor memory so the epilogue of one tile overlaps the MMAs of
//     the next; a STAGES-deep shared-memory ring decouples loads from MMAs;
//   * both weight orientations are native: K-contiguous (nn.Linear storage seen through .permute) and
//     N-contiguous (gpt-oss storage, and the transposed views used for the input gradient), selected by the
//     "major" bits of the UMMA descriptors.
// Every wait is bounded (ptx.cuh): a protocol bug sets the status word and the kernel returns.
#include <cuda.h>
#include <stdlib.h>

#include <mutex>

#include "act_math.cuh"
#include "ptx.cuh"
#include "ep_common.cuh"
#include "smoe_common.cuh"

namespace smoe {
namespace tc {

using namespace ptx;

constexpr int BM = 128;            // sorted positions per tile (UMMA M)
constexpr int BK = 64;             // K elements per pipeline stage: one 128-byte swizzle row of 16-bit data
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 320;   // warp 0 TMA, warp 1 MMA + TMEM, warps 2-5 row gather, warps 6-9 epilogue
constexpr int MAX_E = 1024;
constexpr int A_LAG = 2;           // cp.async groups kept in flight before a stage is published
constexpr int A_STAGE_BYTES = BM * BK * 2;

template <int BN> struct Cfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TABLE_BYTES = ((2 * (MAX_E + 1) * 4 + 15) / 16) * 16;
  static constexpr int STAGE_ROW_BYTES = 80;                       // 64 payload + 16 pad: conflict-free 16-byte accesses
  static constexpr int EPI_STAGING_BYTES = 8 * 32 * STAGE_ROW_BYTES;   // one 32-row slab per epilogue warp (up to 8)
  static constexpr int SMEM_BYTES =
      1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + BAR_BYTES + TABLE_BYTES + EPI_STAGING_BYTES;
  static_assert(SMEM_BYTES <= 232448, "over the 227 KB of shared memory a CTA can have");
};

struct S2SParams {
  const uint8_t* X; int64_t x_row_bytes; int64_t x_rows;
  const uint8_t* bias; int64_t bias_row_elems;
  uint8_t* Y; int64_t y_row_bytes;
  const int64_t* sorted_idx; const int64_t* offsets;
  int64_t R;
  int K, N, E, fan_out, x_grouped, y_grouped, is_bf16, bias_vec;
  int a_by_tma;        // X is grouped and TMA-addressable: the row tiles come by TMA, the gather warps stay idle
  // fused activation epilogue (EPI != 0): H (rows, F) receives the hidden activations, Y (nullable) the
  // up-projection itself; see act_math.cuh for layouts and functions
  uint8_t* H; int64_t h_row_bytes;
  int F, glu_first, act;
  float alpha, limit;
  // fused activation-gradient epilogue (EPI_BWD_*): U (rows, n_up) is the up-projection saved by forward; the GEMM's
  // result is the hidden gradient (N = F columns, never stored) and Y receives the (rows, n_up) gradient of U
  const uint8_t* U; int64_t u_row_bytes;
  // per-row gate (nullable; 16-bit, indexed by the row's slot = sorted_idx[m]). Forward activation epilogues write
  // hidden * gate (the gate weighting of the layer's output moves in front of the down-projection, which is linear);
  // gradient epilogues take the UN-weighted output gradient as A, scale the hidden gradient by the gate and emit the
  // gate gradient's partial dot products <dH_unweighted, hidden_unweighted> over their chunks of hidden columns:
  // dot_out[(column tile * 2 + epilogue group) * dot_stride + m], fp32.
  const uint8_t* row_gate;
  float* dot_out; int64_t dot_stride;
  int group_m;         // m-tiles per raster group (see decode_tile)
  int wide_rows;       // gradient epilogues: rows of U and of the result are read and written 32 bytes per lane (put_rows)
  // Expert-parallel return fused into the epilogue (plain launches only; out_addr nullable). Output row m is not
  // stored to Y but straight into another rank's memory over NVLink: out_addr[m] packs (rank, row) as in
  // ep_common.cuh, the row lands in out_peer.p[rank] + row * out_peer_row_bytes. Each rank also starts the m-tiles
  // of every expert m_rot_num / m_rot_den of the way in and wraps, so that the ranks address different receivers
  // at any moment (the rows of an expert are ordered by the rank they return to).
  const int64_t* out_addr; int64_t out_peer_row_bytes, out_peer_rows;
  int out_world, m_rot_num, m_rot_den;
  int out_pieces;      // 16-byte pieces of a row per store instruction of that epilogue: 8, 16, or 4 (the plain epilogue)
  PeerPtrs out_peer;
  uint32_t idesc;
  int32_t* status;
};

// Shared by all roles: offsets -> per-expert segment starts and the exclusive prefix of tiles per expert.
__device__ __forceinline__ void build_tile_table(const int64_t* __restrict__ offsets, int64_t R, int E, int units_per_mtile,
                                                 int32_t* seg_start, int32_t* tile_prefix, int tid, int nthreads) {
  constexpr int mtile_rows = BM;
  for (int e = tid; e < E; e += nthreads) {
    int64_t v = offsets[e];
    v = v < 0 ? 0 : (v > R ? R : v);
    seg_start[e + 1] = static_cast<int32_t>(v);
  }
  if (tid == 0) seg_start[0] = 0;
  __syncthreads();
  if (tid < 32) {
    const int per = (E + 31) / 32;
    const int beg = min(tid * per, E), end = min(beg + per, E);
    int sum = 0;
    for (int e = beg; e < end; ++e) {
      const int cnt = max(0, seg_start[e + 1] - seg_start[e]);
      sum += ((cnt + mtile_rows - 1) / mtile_rows) * units_per_mtile;
    }
    int inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, o);
      if (tid >= o) inc += v;
    }
    int run = inc - sum;
    for (int e = beg; e < end; ++e) {
      tile_prefix[e] = run;
      const int cnt = max(0, seg_start[e + 1] - seg_start[e]);
      run += ((cnt + mtile_rows - 1) / mtile_rows) * units_per_mtile;
    }
    if (tid == 31) tile_prefix[E] = inc;
  }
}

struct Tile { int e, m0, rows, n0; };

// Tile t of the launch -> expert, row tile, column tile. Inside one expert the m-tiles are walked in groups of
// `group_m`: all column tiles of a group before the next group, the m-tiles of the group innermost. The 148
// tiles that run at the same time then cover about group_m x 148/group_m tiles instead of a whole column of
// m-tiles x a few columns: with group_m chosen so that both footprints are alike, the operands a wave streams
// from HBM (rows x K of A plus columns x K of W) are at their minimum for the number of tiles in flight.
__device__ __forceinline__ Tile decode_tile(int t, const int32_t* tile_prefix, const int32_t* seg_start, int E, int BN,
                                            int group_m, int rot_num = 0, int rot_den = 1) {
  constexpr int mtile_rows = BM;
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_prefix[mid] <= t) lo = mid; else hi = mid;
  }
  Tile tl;
  tl.e = lo;
  const int local = t - tile_prefix[lo];
  const int cnt = seg_start[lo + 1] - seg_start[lo];
  const int m_tiles = (cnt + mtile_rows - 1) / mtile_rows;
  const int n_tiles_e = (tile_prefix[lo + 1] - tile_prefix[lo]) / m_tiles;
  const int gm = max(1, min(group_m, m_tiles));
  const int per_group = gm * n_tiles_e;
  const int grp = local / per_group;
  const int in_grp = local - grp * per_group;
  const int gw = min(gm, m_tiles - grp * gm);
  const int n_tile = in_grp / gw;
  int m_tile = grp * gm + (in_grp - n_tile * gw);
  if (rot_num > 0) {          // rotated start (rot_num < rot_den): see S2SParams::out_addr
    m_tile += static_cast<int>(static_cast<int64_t>(m_tiles) * rot_num / rot_den);
    if (m_tile >= m_tiles) m_tile -= m_tiles;
  }
  tl.m0 = seg_start[lo] + m_tile * mtile_rows;
  tl.rows = min(mtile_rows, seg_start[lo + 1] - tl.m0);
  tl.n0 = n_tile * BN;
  return tl;
}

// EPI: 0 plain linear; 1 H = act(Y); 2 gated halves, H[j] = act(gate) * lin with the halves F columns apart (a tile then
// holds 128 columns of EACH half: accumulator columns [0,128) and [128,256)); 3 gpt-oss interleaved clamped SwiGLU.
// EPI_BWD_*: the GEMM's result is the gradient of the hidden activations (N = F columns); the epilogue turns it into
// the gradient of the saved up-projection U and stores that, (rows, n_up), instead: the hidden gradient never
// reaches memory (4 plain, 5 gated halves, 6 gpt-oss interleaved).
// EPI_PEERS: plain linear whose rows are stored into other ranks' memory (S2SParams::out_addr).
enum { EPI_NONE = 0, EPI_ACT = 1, EPI_GLU_HALVES = 2, EPI_GPT_OSS = 3, EPI_BWD_PLAIN = 4, EPI_BWD_GLU = 5,
       EPI_BWD_GPT_OSS = 6, EPI_PEERS = 7 };

__device__ __forceinline__ void add_bias8(const uint8_t* brow, int col, int is_bf16, int bias_vec, float (&v)[8]) {
  if (!brow) return;
  if (bias_vec) {
    const uint4 bv = __ldg(reinterpret_cast<const uint4*>(brow + col * 2));
    const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float lo, hi;
      if (is_bf16) {
        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&bw[j]);
        lo = __low2float(h); hi = __high2float(h);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&bw[j]);
        lo = __low2float(h); hi = __high2float(h);
      }
      v[2 * j] += lo; v[2 * j + 1] += hi;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint16_t raw = __ldg(reinterpret_cast<const uint16_t*>(brow + (col + j) * 2));
      v[j] += is_bf16 ? __bfloat162float(__ushort_as_bfloat16(raw)) : __half2float(__ushort_as_half(raw));
    }
  }
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8], int is_bf16) {
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (is_bf16) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      o[j] = *reinterpret_cast<const uint32_t*>(&h);
    } else {
      const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      o[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Whole-warp call. Lane l holds NCH 16-byte pieces (8 columns each, starting at column `col0`) of ITS output row
// `rowptr` (row valid or not). The pieces go through a padded shared-memory slab so that every store instruction
// writes 32/NCH rows x NCH*16 contiguous bytes instead of 32 rows x 16 bytes: 4-8x fewer memory transactions for
// the scattered / grouped row stores of the epilogue. Columns at or beyond `col_limit` are not written.
template <int NCH>
__device__ __forceinline__ void flush_rows(uint8_t* slab, int lane, const uint4 (&mine)[NCH], uint8_t* rowptr, bool valid,
                                           int col0, int col_limit) {
  constexpr int ROW = 80;
#pragma unroll
  for (int g = 0; g < NCH; ++g) *reinterpret_cast<uint4*>(slab + lane * ROW + g * 16) = mine[g];
  __syncwarp();
  const unsigned long long mine_ptr = reinterpret_cast<unsigned long long>(rowptr);
  constexpr int ROWS_PER_STORE = 32 / NCH;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int row = i * ROWS_PER_STORE + lane / NCH;
    const int ck = lane % NCH;
    const uint4 v = *reinterpret_cast<const uint4*>(slab + row * ROW + ck * 16);
    const unsigned long long ptr = __shfl_sync(0xffffffffu, mine_ptr, row);
    const int ok = __shfl_sync(0xffffffffu, valid ? 1 : 0, row);
    const int col = col0 + ck * 8;
    if (ok && col < col_limit) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(ptr) + col * 2) = v;
  }
  __syncwarp();
}

// flush_rows for rows that leave this GPU: lane l holds NP 16-byte pieces (NP * 8 columns from `col0`) of ITS row.
// The rows pass through the same slab RP at a time (RP rows x (NP * 16 + 16) bytes fit the warp's 32 x 80 bytes), so that
// every store instruction writes 32 / NP rows x NP * 16 CONTIGUOUS bytes: whole 128-byte lines per row instead of the
// half lines of flush_rows<4>. Local stores do not care (L2 merges them); over NVLink a partial line costs a packet of
// its own.
template <int NP>
__device__ __forceinline__ void flush_rows_wide(uint8_t* slab, int lane, const uint4 (&mine)[NP], uint8_t* rowptr,
                                                bool valid, int col0, int col_limit) {
  constexpr int ROW = NP * 16 + 16;
  constexpr int RP = (NP == 8) ? 16 : 8;                 // rows per pass
  static_assert(RP * ROW <= 32 * 80, "the pass does not fit the warp's staging slab");
  constexpr int ROWS_PER_STORE = 32 / NP;
  const unsigned long long mine_ptr = reinterpret_cast<unsigned long long>(rowptr);
#pragma unroll
  for (int pass = 0; pass < 32 / RP; ++pass) {
    if (lane / RP == pass) {
#pragma unroll
      for (int g = 0; g < NP; ++g) *reinterpret_cast<uint4*>(slab + (lane % RP) * ROW + g * 16) = mine[g];
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < RP / ROWS_PER_STORE; ++i) {
      const int row = i * ROWS_PER_STORE + lane / NP;      // row of this pass
      const int ck = lane % NP;
      const uint4 v = *reinterpret_cast<const uint4*>(slab + row * ROW + ck * 16);
      const unsigned long long ptr = __shfl_sync(0xffffffffu, mine_ptr, pass * RP + row);
      const int ok = __shfl_sync(0xffffffffu, valid ? 1 : 0, pass * RP + row);
      const int col = col0 + ck * 8;
      if (ok && col < col_limit) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(ptr) + col * 2) = v;
    }
    __syncwarp();
  }
}

// NCH consecutive 16-byte pieces (NCH * 8 columns from `col0`) of every lane's own row. `direct`: two pieces at a time
// straight from registers as 32-byte stores, one full sector per lane (needs 32-byte aligned rows and col0, and a
// col_limit that is a multiple of 16); else through the staging slab (flush_rows). The direct form costs more
// store transactions but no shared-memory traffic, and shared-memory bandwidth is what the MMAs of the next tile are
// short of while an epilogue with twice the usual output (the activation gradients) runs.
template <int NCH>
__device__ __forceinline__ void put_rows(bool direct, uint8_t* slab, int lane, const uint4 (&mine)[NCH], uint8_t* rowptr,
                                         bool valid, int col0, int col_limit) {
  if (direct) {
#pragma unroll
    for (int g = 0; g < NCH; g += 2) {
      const int col = col0 + g * 8;
      if (valid && col < col_limit) st_global_256(rowptr + static_cast<int64_t>(col) * 2, mine[g], mine[g + 1]);
    }
  } else {
    flush_rows<NCH>(slab, lane, mine, rowptr, valid, col0, col_limit);
  }
}

// Plain epilogue of a launch whose rows return to their home ranks (S2SParams::out_addr): NP * 8 accumulator columns
// at a time (64: each row travels in whole 128-byte lines; 128: in pairs of lines). The two groups of epilogue warps
// take every other unit.
template <int BN, int NP>
__device__ __forceinline__ void epilogue_rows_to_peers(const S2SParams& p, int n0, uint32_t taddr, uint8_t* slab, int lane,
                                                       bool valid, uint8_t* yrow, int u_first, int u_step) {
  constexpr int UNIT = NP * 8;
#pragma unroll 1
  for (int u = u_first; u < BN / UNIT; u += u_step) {
    const int n = n0 + u * UNIT;
    if (n >= p.N) break;
    uint4 py[NP];
#pragma unroll
    for (int h = 0; h < NP / 4; ++h) {
      uint32_t acc[32];
      tmem_ld_32x32b_x32(taddr + u * UNIT + h * 32, acc);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float v[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) v[jj] = __uint_as_float(acc[g * 8 + jj]);
        py[h * 4 + g] = pack8(v, p.is_bf16);
      }
    }
    flush_rows_wide<NP>(slab, lane, py, yrow, valid, n, p.N);
  }
}

// Epilogue of one tile for one warp: lane l owns accumulator row (TMEM lane) l of the warp's quarter. Reads the BN
// accumulator columns at `taddr` 32 at a time, adds the bias, applies the fused activation (EPI) and stores the rows
// through the warp's staging slab. Every lane runs the arithmetic (rows past the segment end hold finite leftovers
// of other rows' tiles or zeros and are never stored): the stores are whole-warp operations.
template <int BN, int EPI>
__device__ __forceinline__ void epilogue_rows(const S2SParams& p, int n0, uint32_t taddr, uint8_t* slab, int lane,
                                              bool valid, uint8_t* yrow, uint8_t* hrow, const uint8_t* brow,
                                              int c_first = 0, int c_step = 1, float hscale = 1.0f) {
  constexpr int TN = (EPI == EPI_GLU_HALVES) ? BN / 2 : BN;
  const bool write_y = (EPI == EPI_NONE) || p.Y != nullptr;
  // 32-column chunks c_first, c_first + c_step, ...: with two groups of epilogue warps each takes every other chunk
  if (EPI == EPI_GLU_HALVES) {
#pragma unroll 1
    for (int c = c_first; c < TN / 32; c += c_step) {
      const int n = n0 + c * 32;            // column inside one half
      if (n >= p.F) break;
      uint32_t acc_a[32], acc_b[32];
      tmem_ld_32x32b_x32(taddr + c * 32, acc_a);
      tmem_ld_32x32b_x32(taddr + TN + c * 32, acc_b);
      tmem_ld_wait();
      uint4 pa[4], pb[4], ph[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int nn = min(n + g * 8, p.F - 8);      // clamped for the bias reads; the flush masks the columns
        float a[8], b[8], h[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          a[jj] = __uint_as_float(acc_a[g * 8 + jj]);
          b[jj] = __uint_as_float(acc_b[g * 8 + jj]);
        }
        add_bias8(brow, nn, p.is_bf16, p.bias_vec, a);
        add_bias8(brow, p.F + nn, p.is_bf16, p.bias_vec, b);
        SMOE_ACT_SWITCH(p.act, _Pragma("unroll") for (int jj = 0; jj < 8; ++jj)
          h[jj] = hscale * (p.glu_first ? act_fwd<ACT_, true>(a[jj]) * b[jj] : act_fwd<ACT_, true>(b[jj]) * a[jj]);)
        pa[g] = pack8(a, p.is_bf16);
        pb[g] = pack8(b, p.is_bf16);
        ph[g] = pack8(h, p.is_bf16);
      }
      if (write_y) {
        flush_rows<4>(slab, lane, pa, yrow, valid, n, p.F);
        flush_rows<4>(slab, lane, pb, yrow + static_cast<int64_t>(p.F) * 2, valid, n, p.F);
      }
      flush_rows<4>(slab, lane, ph, hrow, valid, n, p.F);
    }
  } else {
#pragma unroll 1
    for (int c = c_first; c < BN / 32; c += c_step) {
      const int n = n0 + c * 32;
      if (n >= p.N) break;
      uint32_t acc[32];
      tmem_ld_32x32b_x32(taddr + c * 32, acc);
      tmem_ld_wait();
      uint4 py[4];
      if (EPI == EPI_GPT_OSS) {
        uint4 ph[2];
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {           // 16 accumulator columns -> 8 hidden columns
          const int nn = min(n + gg * 16, p.N - 16);
          float v0[8], v1[8], h[8];
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            v0[jj] = __uint_as_float(acc[gg * 16 + jj]);
            v1[jj] = __uint_as_float(acc[gg * 16 + 8 + jj]);
          }
          add_bias8(brow, nn, p.is_bf16, p.bias_vec, v0);
          add_bias8(brow, nn + 8, p.is_bf16, p.bias_vec, v1);
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const float g0 = (jj < 4) ? v0[2 * jj] : v1[2 * jj - 8];
            const float u0 = (jj < 4) ? v0[2 * jj + 1] : v1[2 * jj - 7];
            const float gc = fminf(g0, p.limit);
            const float uc = fminf(fmaxf(u0, -p.limit), p.limit);
            h[jj] = hscale * (uc + 1.0f) * (gc * sigmoidf_<true>(p.alpha * gc));
          }
          py[2 * gg] = pack8(v0, p.is_bf16);
          py[2 * gg + 1] = pack8(v1, p.is_bf16);
          ph[gg] = pack8(h, p.is_bf16);
        }
        if (write_y) flush_rows<4>(slab, lane, py, yrow, valid, n, p.N);
        flush_rows<2>(slab, lane, ph, hrow, valid, n / 2, p.N / 2);
      } else {
        uint4 ph[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int nn = min(n + g * 8, p.N - 8);
          float v[8];
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) v[jj] = __uint_as_float(acc[g * 8 + jj]);
          add_bias8(brow, nn, p.is_bf16, p.bias_vec, v);
          py[g] = pack8(v, p.is_bf16);
          if (EPI == EPI_ACT) {
            float h[8];
            SMOE_ACT_SWITCH(p.act, _Pragma("unroll") for (int jj = 0; jj < 8; ++jj) h[jj] = hscale * act_fwd<ACT_, true>(v[jj]);)
            ph[g] = pack8(h, p.is_bf16);
          }
        }
        if (write_y) flush_rows<4>(slab, lane, py, yrow, valid, n, p.N);
        if (EPI == EPI_ACT) flush_rows<4>(slab, lane, ph, hrow, valid, n, p.N);
      }
    }
  }
}

// Eight 16-bit values (one 16-byte piece of a row) as floats.
__device__ __forceinline__ void cvt8(const uint4& raw, int is_bf16, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (is_bf16) {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
      v[2 * j] = __low2float(h); v[2 * j + 1] = __high2float(h);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
      v[2 * j] = __low2float(h); v[2 * j + 1] = __high2float(h);
    }
  }
}

// Epilogue of one tile of the fused "input gradient of the down-projection + activation gradient" launch. The
// accumulator holds dH = dL/d(hidden) for 128 rows x BN hidden columns starting at n0; lane l owns row l of the warp's
// quarter, reads ITS row of the saved up-projection U (`urow`) and writes the matching columns of dU (`durow`):
//   plain       dU[j]      = dH[j] * act'(U[j])
//   gated       dU[lin j]  = dH[j] * act(U[gate j]),   dU[gate j] = dH[j] * U[lin j] * act'(U[gate j])
//   gpt-oss     g = U[2j], u = U[2j+1] (clamped in forward): dU[2j+1] = dH[j] * glu(g) inside the clamp, else 0;
//               dU[2j] = dH[j] * (u_c + 1) * glu'(g) below the limit, else 0
// (the arithmetic of act_backward_kernel in activation.cu, on fp32 accumulators instead of a rounded dH).
// U does not depend on the MMAs: the pieces of a chunk are requested one chunk ahead, the first chunk's before
// `wait_acc()` (the caller's wait for the accumulator), so that their HBM latency hides behind the wait, the
// tensor-memory loads and the arithmetic of the chunk before. Returns what `wait_acc()` returned.
template <int BN, int EPI, typename WaitFn>
__device__ __forceinline__ bool epilogue_act_bwd(const S2SParams& p, int n0, uint32_t taddr, uint8_t* slab, int lane,
                                                 bool valid, uint8_t* durow, const uint8_t* urow, int c_first, int c_step,
                                                 WaitFn wait_acc, float rg, float& dot) {
  constexpr int NRAW = (EPI == EPI_BWD_PLAIN) ? 4 : 8;       // 16-byte pieces of U per 32 hidden columns
  const int F = p.N;
  const int lin_off = p.glu_first ? F : 0, gate_off = p.glu_first ? 0 : F;
  // byte offset inside the row of piece q of the chunk that starts at hidden column n (clamped to stay inside
  // the row: the flush masks what lies beyond it)
  const bool wide = p.wide_rows != 0;      // 32-byte loads and stores, two pieces at a time (host-checked alignment)
  const int last = F - (wide ? 16 : 8);    // last column a (pair of) piece(s) may start at
  auto piece_offset = [&](int n, int q) -> int64_t {
    if (EPI == EPI_BWD_PLAIN) return static_cast<int64_t>(min(n + q * 8, last)) * 2;
    if (EPI == EPI_BWD_GLU) return static_cast<int64_t>((q < 4 ? lin_off : gate_off) + min(n + (q & 3) * 8, last)) * 2;
    return static_cast<int64_t>(2 * min(n + (q >> 1) * 8, F - 8) + (q & 1) * 8) * 2;
  };
  uint4 nxt[NRAW];
  auto request = [&](int c) {
    const int n = n0 + c * 32;
    const bool live = valid && c < BN / 32 && n < F;
    if (wide) {
#pragma unroll
      for (int q = 0; q < NRAW; q += 2) {
        if (live) ld_global_nc_256(urow + piece_offset(n, q), nxt[q], nxt[q + 1]);
        else nxt[q] = nxt[q + 1] = make_uint4(0u, 0u, 0u, 0u);
      }
    } else {
#pragma unroll
      for (int q = 0; q < NRAW; ++q)
        nxt[q] = live ? __ldg(reinterpret_cast<const uint4*>(urow + piece_offset(n, q))) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  request(c_first);
  if (!wait_acc()) return false;
  tc_fence_after_sync();
#pragma unroll 1
  for (int c = c_first; c < BN / 32; c += c_step) {
    const int n = n0 + c * 32;
    if (n >= F) break;
    uint4 cur[NRAW];
#pragma unroll
    for (int q = 0; q < NRAW; ++q) cur[q] = nxt[q];
    request(c + c_step);
    uint32_t acc[32];
    tmem_ld_32x32b_x32(taddr + c * 32, acc);
    tmem_ld_wait();
    if (EPI == EPI_BWD_PLAIN) {
      uint4 pd[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float u[8], d[8];
        cvt8(cur[g], p.is_bf16, u);
        SMOE_ACT_SWITCH(p.act, _Pragma("unroll") for (int jj = 0; jj < 8; ++jj) {
          const float a0 = __uint_as_float(acc[g * 8 + jj]);
          if (p.dot_out) dot = fmaf(a0, act_fwd<ACT_, true>(u[jj]), dot);
          d[jj] = rg * a0 * act_bwd<ACT_, true>(u[jj]);
        })
        pd[g] = pack8(d, p.is_bf16);
      }
      put_rows<4>(wide, slab, lane, pd, durow, valid, n, F);
    } else if (EPI == EPI_BWD_GLU) {
      uint4 pl[4], pg[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float lin[8], gate[8], dl[8], dg[8];
        cvt8(cur[g], p.is_bf16, lin);
        cvt8(cur[4 + g], p.is_bf16, gate);
        SMOE_ACT_SWITCH(p.act, _Pragma("unroll") for (int jj = 0; jj < 8; ++jj) {
          const float a0 = __uint_as_float(acc[g * 8 + jj]);
          const float af = act_fwd<ACT_, true>(gate[jj]);
          dot = fmaf(a0, lin[jj] * af, dot);
          const float dh = rg * a0;
          dl[jj] = dh * af;
          dg[jj] = dh * lin[jj] * act_bwd<ACT_, true>(gate[jj]);
        })
        pl[g] = pack8(dl, p.is_bf16);
        pg[g] = pack8(dg, p.is_bf16);
      }
      put_rows<4>(wide, slab, lane, pl, durow + static_cast<int64_t>(lin_off) * 2, valid, n, F);
      put_rows<4>(wide, slab, lane, pg, durow + static_cast<int64_t>(gate_off) * 2, valid, n, F);
    } else {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {               // 16 hidden columns -> 32 columns of U
        uint4 po[4];
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          float u0[8], u1[8], o0[8], o1[8];
          cvt8(cur[(hh * 2 + g) * 2], p.is_bf16, u0);
          cvt8(cur[(hh * 2 + g) * 2 + 1], p.is_bf16, u1);
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const float g0 = (jj < 4) ? u0[2 * jj] : u1[2 * jj - 8];
            const float up0 = (jj < 4) ? u0[2 * jj + 1] : u1[2 * jj - 7];
            const float a0 = __uint_as_float(acc[hh * 16 + g * 8 + jj]);
            const float dh = rg * a0;
            const float gc = fminf(g0, p.limit);
            const float uc = fminf(fmaxf(up0, -p.limit), p.limit);
            const float sg = sigmoidf_<true>(p.alpha * gc);
            dot = fmaf(a0, (uc + 1.0f) * (gc * sg), dot);
            const float d_u = (up0 >= -p.limit && up0 <= p.limit) ? dh * (gc * sg) : 0.f;
            const float d_g = (g0 <= p.limit) ? dh * (uc + 1.0f) * (sg + gc * p.alpha * sg * (1.0f - sg)) : 0.f;
            if (jj < 4) { o0[2 * jj] = d_g; o0[2 * jj + 1] = d_u; }
            else { o1[2 * jj - 8] = d_g; o1[2 * jj - 7] = d_u; }
          }
          po[2 * g] = pack8(o0, p.is_bf16);
          po[2 * g + 1] = pack8(o1, p.is_bf16);
        }
        put_rows<4>(wide, slab, lane, po, durow, valid, 2 * (n + hh * 16), 2 * F);
      }
    }
  }
  return true;
}

template <int BN, bool B_KMAJOR, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
s2s_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
              const S2SParams p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + C::B_STAGE_BYTES));
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int32_t* seg_start = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(bars) + C::BAR_BYTES);
  int32_t* tile_prefix = seg_start + (MAX_E + 1);
  uint8_t* epi_staging = reinterpret_cast<uint8_t*>(bars) + C::BAR_BYTES + C::TABLE_BYTES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // columns of the output a tile advances by: with gated halves a tile owns TN = BN/2 columns of each half
  constexpr int TN = (EPI == EPI_GLU_HALVES) ? BN / 2 : BN;
  const int n_tiles = ((EPI == EPI_GLU_HALVES ? p.F : p.N) + TN - 1) / TN;
  const int num_kb = (p.K + BK - 1) / BK;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), p.a_by_tma ? 1 : 1 + 128);   // TMA thread (expect_tx) [+ 128 gather threads]
      mbar_init(empty_bar(s), 1);                         // tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);                        // tcgen05.commit
      mbar_init(tempty_bar(b), p.a_by_tma ? 256 : 128);  // epilogue threads (the idle gather warps join them)
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_w);
    if (p.a_by_tma) tma_prefetch_desc(&tmap_x);
  }
  build_tile_table(p.offsets, p.R, p.E, n_tiles, seg_start, tile_prefix, tid, NUM_THREADS);
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const int total_tiles = tile_prefix[p.E];

  if (warp == 0) {
    // ---------------- weight tiles: TMA producer -------------------------------------------------------
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Tile tl = decode_tile(t, tile_prefix, seg_start, p.E, TN, p.group_m, p.m_rot_num, p.m_rot_den);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(empty_bar(s), ph ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
        if (lane == 0) {
          mbar_arrive_expect_tx(full_bar(s), C::B_STAGE_BYTES + (p.a_by_tma ? A_STAGE_BYTES : 0));
          if (p.a_by_tma) tma_load_2d(smem_u32(sA + s * A_STAGE_BYTES), &tmap_x, full_bar(s), kb * BK, tl.m0);
          const uint32_t dst = smem_u32(sB + s * C::B_STAGE_BYTES);
          if (EPI == EPI_GLU_HALVES) {
            // weight rows of the two halves: [n0, n0+TN) and [F+n0, F+n0+TN)
            if (B_KMAJOR) {
              tma_load_3d(dst, &tmap_w, full_bar(s), kb * BK, tl.n0, tl.e);
              tma_load_3d(dst + TN * BK * 2, &tmap_w, full_bar(s), kb * BK, p.F + tl.n0, tl.e);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) {
                const int col = (j < BN / 128) ? tl.n0 + j * 64 : p.F + tl.n0 + (j - BN / 128) * 64;
                tma_load_3d(dst + j * (64 * BK * 2), &tmap_w, full_bar(s), col, kb * BK, tl.e);
              }
            }
          } else if (B_KMAJOR) {
            tma_load_3d(dst, &tmap_w, full_bar(s), kb * BK, tl.n0, tl.e);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(dst + j * (64 * BK * 2), &tmap_w, full_bar(s), tl.n0 + j * 64, kb * BK, tl.e);
          }
        }
        __syncwarp();
      }
    }
    if (!ok) {  // give copies already in flight time to land before the CTA goes away
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer -----------------------------------------------------------------------
    int it = 0, tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_iter) {
      const int buf = tile_iter & 1;
      const uint32_t tph = (tile_iter >> 1) & 1;
      if (!mbar_wait_warp(tempty_bar(buf), tph ^ 1, abort_flag, p.status, 2)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(full_bar(s), ph, abort_flag, p.status, 3)) { ok = false; break; }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * C::B_STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t adesc = make_smem_desc_sw128(a_addr + j * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_KMAJOR ? make_smem_desc_sw128(b_addr + j * (UMMA_K * 2), 16, 1024)
                                            : make_smem_desc_sw128(b_addr + j * (UMMA_K * 128), 64 * BK * 2, 1024);
            umma_f16(d_tmem, adesc, bdesc, p.idesc, (kb | j) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(tfull_bar(buf));
      __syncwarp();
    }
  } else if (warp < 6 && !p.a_by_tma) {
    // ---------------- token rows: cp.async gather into the swizzled A tile -----------------------------
    const int ptid = tid - 64;
    const int chunk = ptid & 7;          // 16-byte chunk of the 128-byte K slice
    const int row_base = ptid >> 3;      // rows row_base + 16*i
    const uint32_t dst_off = row_base * 128 + ((chunk ^ (row_base & 7)) << 4);
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Tile tl = decode_tile(t, tile_prefix, seg_start, p.E, TN, p.group_m, p.m_rot_num, p.m_rot_den);
      const uint8_t* rowptr[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = row_base + 16 * i;
        const uint8_t* ptr = nullptr;
        if (r < tl.rows) {
          const int64_t m = tl.m0 + r;
          const int64_t in = p.x_grouped ? m : p.sorted_idx[m] / p.fan_out;
          if (in >= 0 && in < p.x_rows) ptr = p.X + in * p.x_row_bytes + chunk * 16;
        }
        rowptr[i] = ptr;
      }
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(empty_bar(s), ph ^ 1, abort_flag, p.status, 4)) { ok = false; break; }
        const bool k_ok = (kb * BK + chunk * 8) < p.K;
        const uint32_t dst = smem_u32(sA + s * A_STAGE_BYTES) + dst_off;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool v = k_ok && rowptr[i] != nullptr;
          cp_async16(dst + i * 2048, v ? rowptr[i] + static_cast<int64_t>(kb) * (BK * 2) : p.X, v ? 16u : 0u);
        }
        cp_async_commit();
        if (it >= A_LAG) {
          cp_async_wait<A_LAG>();
          fence_proxy_async_smem();
          mbar_arrive(full_bar((it - A_LAG) % STAGES));
        }
      }
    }
    cp_async_wait<0>();
    fence_proxy_async_smem();
    if (ok) {
      for (int j = max(0, it - A_LAG); j < it; ++j) mbar_arrive(full_bar(j % STAGES));
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> bias -> 16-bit -> global rows ----------------------
    // Warps 6-9 always; warps 2-5 too when the rows come by TMA and there is nothing for them to gather. A warp may
    // read the tensor-memory lanes of quarter (warp % 4), so each group of four covers all 128 accumulator rows; the
    // two groups split the tile's 32-column chunks between them (even / odd).
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int r = q * 32 + lane;
    const int group = warp >= 6 ? 0 : 1;
    const int c_step = p.a_by_tma ? 2 : 1;
    int tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_iter) {
      const Tile tl = decode_tile(t, tile_prefix, seg_start, p.E, TN, p.group_m, p.m_rot_num, p.m_rot_den);
      const int buf = tile_iter & 1;
      const uint32_t tph = (tile_iter >> 1) & 1;
      bool valid = r < tl.rows;
      int64_t out_row = 0;
      if (valid) {
        const int64_t m = tl.m0 + r;
        out_row = p.y_grouped ? m : p.sorted_idx[m];
        valid = out_row >= 0 && out_row < p.R;
      }
      uint8_t* yrow = p.Y + out_row * p.y_row_bytes;
      if (EPI == EPI_PEERS) {
        // the row's home is on another rank (or this one): a malformed return address drops the row
        yrow = nullptr;
        if (valid) {
          const int64_t d = p.out_addr[tl.m0 + r];
          const int rk = dest_rank(d);
          const int64_t s = dest_row(d);
          valid = rk >= 0 && rk < p.out_world && s < p.out_peer_rows;
          if (valid) yrow = p.out_peer.p[rk] + s * p.out_peer_row_bytes;
        }
      }
      const uint8_t* brow = p.bias ? p.bias + static_cast<int64_t>(tl.e) * p.bias_row_elems * 2 : nullptr;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      uint8_t* slab = epi_staging + (group * 4 + q) * (32 * C::STAGE_ROW_BYTES);
      auto wait_acc = [&]() { return mbar_wait_warp(tfull_bar(buf), tph, abort_flag, p.status, 5); };
      float rg = 1.0f;                     // the row's gate, where the launch carries gates
      if (EPI != EPI_NONE && EPI != EPI_PEERS && p.row_gate != nullptr && valid) {
        const int64_t slot = p.sorted_idx[tl.m0 + r];
        if (slot >= 0 && slot < p.R) {
          const uint16_t raw = __ldg(reinterpret_cast<const uint16_t*>(p.row_gate) + slot);
          rg = p.is_bf16 ? __bfloat162float(__ushort_as_bfloat16(raw)) : __half2float(__ushort_as_half(raw));
        }
      }
      if constexpr (EPI >= EPI_BWD_PLAIN && EPI <= EPI_BWD_GPT_OSS) {
        // (the first pieces of the saved up-projection are requested before the wait for the accumulator)
        float dot = 0.f;
        if (!epilogue_act_bwd<BN, EPI>(p, tl.n0, taddr, slab, lane, valid, yrow, p.U + out_row * p.u_row_bytes, group,
                                       c_step, wait_acc, rg, dot)) { ok = false; break; }
        if (p.dot_out != nullptr && valid) {
          float* line = p.dot_out + static_cast<int64_t>((tl.n0 / BN) * 2 + group) * p.dot_stride + (tl.m0 + r);
          *line = dot;
          if (c_step == 1) line[p.dot_stride] = 0.f;       // one epilogue group only: the other group's line is empty
        }
      } else {
        if (!wait_acc()) { ok = false; break; }
        tc_fence_after_sync();
        if constexpr (EPI == EPI_PEERS) {
          if (p.out_pieces == 16)
            epilogue_rows_to_peers<BN, 16>(p, tl.n0, taddr, slab, lane, valid, yrow, group, c_step);
          else if (p.out_pieces == 8)
            epilogue_rows_to_peers<BN, 8>(p, tl.n0, taddr, slab, lane, valid, yrow, group, c_step);
          else
            epilogue_rows<BN, EPI_NONE>(p, tl.n0, taddr, slab, lane, valid, yrow, nullptr, nullptr, group, c_step, 1.0f);
        } else {
          uint8_t* hrow = (EPI != EPI_NONE) ? p.H + out_row * p.h_row_bytes : nullptr;
          epilogue_rows<BN, EPI>(p, tl.n0, taddr, slab, lane, valid, yrow, hrow, brow, group, c_step, rg);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(tempty_bar(buf));
    }
  }

  // ---------------- teardown ---------------------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Weight gradient: DWt[e] (N x K) = DY_e^T (N x rows_e) . X_e (rows_e x K), replacing the reference's _groupXtY
// (scattermoe/kernels/ops.py:247-366). Token rows are the contraction dimension, so both operands are fed
// "MN-major": the DY slab by TMA (2-D map over (feature, row)), the X slab by cp.async row gather, which also
// serves the still un-grouped input (row = slot / fan_out) and zero-fills the rows past the segment end, the
// only masking the ragged segments need. A tile is 128 DY features x BNW X features of one expert.
struct WGradParams {
  const uint8_t* DY; int64_t dy_row_bytes;
  const uint8_t* X; int64_t x_row_bytes; int64_t x_rows;
  uint8_t* DW; int64_t dw_e_bytes; int64_t dw_row_bytes;
  const int64_t* gather_idx; const int64_t* offsets;
  int64_t R;
  int K, N, E, fan_out, is_bf16;
  int x_by_tma;        // X is grouped and TMA-addressable: whole 64-row slabs come by TMA, ragged tails by cp.async
  int band_over_n;     // 0: bands of `band` X-feature tiles, DY-feature tiles stream through them; 1: the other way
  int band;            // band width in tiles (see the tile order in the kernel)
  uint32_t idesc;
  int32_t* status;
};

template <int BNW>
__global__ void __launch_bounds__(NUM_THREADS, 1)
wgrad_tc_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x,
                const WGradParams p) {
  using C = Cfg<BNW>;
  constexpr int STAGES = C::STAGES;
  constexpr int CPR = BNW / 8;          // 16-byte chunks per gathered row
  constexpr int RPP = 128 / CPR;        // rows covered by the 128 gather threads in one pass
  constexpr int NI = BK / RPP;          // passes per stage
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + C::B_STAGE_BYTES));
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  // go[s]: "stage s is free for the ragged tail slab", TMA lane -> gather threads (grouped X only)
  auto go_bar = [&](int s) { return bar0 + 8u * (2 * STAGES + 5 + s); };
  static_assert((3 * STAGES + 5) * 8 <= C::BAR_BYTES, "barrier area too small");
  int32_t* seg_start = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(bars) + C::BAR_BYTES);
  uint8_t* epi_staging = reinterpret_cast<uint8_t*>(bars) + C::BAR_BYTES + C::TABLE_BYTES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = (p.N + BM - 1) / BM;
  const int k_tiles = (p.K + BNW - 1) / BNW;
  const int tiles_per_e = n_tiles * k_tiles;
  const int total_tiles = p.E * tiles_per_e;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1 + 128);
      mbar_init(empty_bar(s), 1);
      mbar_init(go_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_dy);
    tma_prefetch_desc(&tmap_x);
    seg_start[0] = 0;
  }
  for (int e = tid; e < p.E; e += NUM_THREADS) {
    int64_t v = p.offsets[e];
    v = v < 0 ? 0 : (v > p.R ? p.R : v);
    seg_start[e + 1] = static_cast<int32_t>(v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  // tile t -> expert, DY-feature tile, X-feature tile and the expert's row segment. Inside one expert the tiles are
  // walked in bands: `band` tiles of ONE operand's feature dimension stay in L2 (band * tile width * rows of the
  // expert) while every tile of the other operand passes over them once, so the banded operand is read from HBM
  // once per expert and the streamed one once per band. The host picks the operand to band (the one whose whole
  // panel, or failing that the larger share of it, fits the L2 budget) and the band width.
  const int band_w = max(1, p.band);
  auto decode = [&](int t, int& e, int& n0, int& k0, int& m_beg, int& m_end) {
    e = t / tiles_per_e;
    const int rem = t - e * tiles_per_e;
    int nt, kt;
    if (p.band_over_n) {
      const int band = rem / (k_tiles * band_w);
      const int in_band = rem - band * k_tiles * band_w;
      const int bw = min(band_w, n_tiles - band * band_w);
      kt = in_band / bw;
      nt = band * band_w + (in_band - kt * bw);
    } else {
      const int band = rem / (n_tiles * band_w);
      const int in_band = rem - band * n_tiles * band_w;
      const int bw = min(band_w, k_tiles - band * band_w);
      nt = in_band / bw;
      kt = band * band_w + (in_band - nt * bw);
    }
    n0 = nt * BM;
    k0 = kt * BNW;
    m_beg = seg_start[e];
    m_end = max(m_beg, seg_start[e + 1]);
  };
  // A 64-row slab that crosses the end of the expert's segment is "ragged": both operands of it are copied with
  // cp.async, which zero-fills the rows past the end. Rows past the end are either another expert's or not
  // initialised at all; zeroing BOTH sides keeps a stray NaN/Inf there from reaching this expert's gradient.
  // Whole slabs: DY always by TMA; X by TMA unless it has to be gathered.
  auto slab_ragged = [&](int c, int m_beg, int m_end) { return m_beg + (c + 1) * BK > m_end; };
  auto slab_by_tma = [&](int c, int m_beg, int m_end) { return p.x_by_tma && !slab_ragged(c, m_beg, m_end); };

  if (warp == 0) {
    // ---------------- DY slabs: TMA producer --------------------------------------------------------------
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int e, n0, k0, m_beg, m_end;
      decode(t, e, n0, k0, m_beg, m_end);
      const int nchunks = (m_end - m_beg + BK - 1) / BK;
      for (int c = 0; c < nchunks; ++c, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(empty_bar(s), ph ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
        if (lane == 0) {
          const bool x_too = slab_by_tma(c, m_beg, m_end);
          if (slab_ragged(c, m_beg, m_end)) {
            if (p.x_by_tma) mbar_arrive(go_bar(s));   // the gather threads may now fill this stage
            mbar_arrive(full_bar(s));                  // nothing comes by TMA for this slab
          } else {
            // a slab that comes whole by TMA needs nothing from the 128 gather threads: their arrivals are made
            // here in one instruction (128 same-address arrives per slab cost the shared-memory pipe the MMAs need)
            if (x_too) mbar_arrive_count(full_bar(s), 128);
            mbar_arrive_expect_tx(full_bar(s), A_STAGE_BYTES + (x_too ? C::B_STAGE_BYTES : 0));
            const uint32_t dst = smem_u32(sA + s * A_STAGE_BYTES);
            tma_load_2d(dst, &tmap_dy, full_bar(s), n0, m_beg + c * BK);
            tma_load_2d(dst + 64 * BK * 2, &tmap_dy, full_bar(s), n0 + 64, m_beg + c * BK);
          }
          if (x_too) {
            const uint32_t dstb = smem_u32(sB + s * C::B_STAGE_BYTES);
#pragma unroll
            for (int j = 0; j < BNW / 64; ++j)
              tma_load_2d(dstb + j * (64 * BK * 2), &tmap_x, full_bar(s), k0 + j * 64, m_beg + c * BK);
          }
        }
        __syncwarp();
      }
    }
    if (!ok) {
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer --------------------------------------------------------------------------
    int it = 0, tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int e, n0, k0, m_beg, m_end;
      decode(t, e, n0, k0, m_beg, m_end);
      const int nchunks = (m_end - m_beg + BK - 1) / BK;
      if (nchunks == 0) continue;       // the epilogue writes zeros, no accumulator involved
      const int buf = tile_iter & 1;
      const uint32_t tph = (tile_iter >> 1) & 1;
      if (!mbar_wait_warp(tempty_bar(buf), tph ^ 1, abort_flag, p.status, 12)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + buf * BNW;
      for (int c = 0; c < nchunks; ++c, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(full_bar(s), ph, abort_flag, p.status, 13)) { ok = false; break; }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * C::B_STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t adesc = make_smem_desc_sw128(a_addr + j * (UMMA_K * 128), 64 * BK * 2, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(b_addr + j * (UMMA_K * 128), 64 * BK * 2, 1024);
            umma_f16(d_tmem, adesc, bdesc, p.idesc, (c | j) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(tfull_bar(buf));
      __syncwarp();
      ++tile_iter;
    }
  } else if (warp < 6 && p.x_by_tma) {
    // ---------------- grouped X: only the ragged tail slab of a tile is copied by these threads ------------
    // Whole slabs need nothing from them (the TMA lane makes their 128 arrivals in one instruction), and they do
    // not follow the ring: they wait on go[s], which the TMA lane signals once per ragged use of stage s and
    // which cannot complete a second time before all of them have arrived for the first (the MMA needs their
    // arrivals to free the stage), so its parity can never run ahead of a waiting thread.
    const int ptid = tid - 64;
    const int chunk = ptid % CPR;
    const int row_base = ptid / CPR;
    const uint32_t box_off = (chunk >> 3) * (64 * BK * 2);
    const int a_chunk = ptid & 15, a_row0 = ptid >> 4;
    uint32_t go_parity = 0;            // bit s: parity of the next go[s] phase
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int e, n0, k0, m_beg, m_end;
      decode(t, e, n0, k0, m_beg, m_end);
      const int nchunks = (m_end - m_beg + BK - 1) / BK;
      if (nchunks == 0) continue;
      const int c = nchunks - 1;
      if (slab_ragged(c, m_beg, m_end)) {
        const int s = (it + c) % STAGES;
        if (!mbar_wait_warp(go_bar(s), (go_parity >> s) & 1u, abort_flag, p.status, 16)) { ok = false; break; }
        go_parity ^= 1u << s;
        const int64_t m0 = static_cast<int64_t>(m_beg) + c * BK;
        // DY slab: 64 rows x 128 features = 1024 16-byte chunks, 8 per thread
        const bool n_ok = (n0 + a_chunk * 8) < p.N;
        const uint32_t dsta = smem_u32(sA + s * A_STAGE_BYTES) + (a_chunk >> 3) * (64 * BK * 2);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = a_row0 + 8 * i;
          const int64_t m = m0 + row;
          const bool v = n_ok && m < m_end;
          cp_async16(dsta + row * 128 + (((a_chunk & 7) ^ (row & 7)) << 4),
                     v ? p.DY + m * p.dy_row_bytes + static_cast<int64_t>(n0 + a_chunk * 8) * 2 : p.DY, v ? 16u : 0u);
        }
        // X slab: 64 rows x BNW features
        const bool k_ok = (k0 + chunk * 8) < p.K;
        const int64_t col_bytes = static_cast<int64_t>(k0 + chunk * 8) * 2;
        const uint32_t dstb = smem_u32(sB + s * C::B_STAGE_BYTES) + box_off;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          const int row = row_base + RPP * i;
          const int64_t m = m0 + row;
          const bool v = k_ok && m < m_end && m < p.x_rows;
          cp_async16(dstb + row * 128 + (((chunk & 7) ^ (row & 7)) << 4), v ? p.X + m * p.x_row_bytes + col_bytes : p.X,
                     v ? 16u : 0u);
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_proxy_async_smem();
        mbar_arrive(full_bar(s));
      }
      it += nchunks;
    }
  } else if (warp < 6) {
    // ---------------- X slabs: cp.async row gather (zero-fill past the segment end) ----------------------
    const int ptid = tid - 64;
    const int chunk = ptid % CPR;
    const int row_base = ptid / CPR;                 // rows row_base + RPP*i
    const uint32_t box_off = (chunk >> 3) * (64 * BK * 2);
    // lanes 0..15 of each warp fetch the source-row offsets the warp needs for one stage
    const int rows_per_warp_pass = 32 / CPR == 0 ? 1 : 32 / CPR;   // 1 (BNW=256) or 2 (BNW=128)
    const int wrow0 = (warp - 2) * rows_per_warp_pass;
    const int my_half = (rows_per_warp_pass == 2) ? (lane >> 4) : 0;
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int e, n0, k0, m_beg, m_end;
      decode(t, e, n0, k0, m_beg, m_end);
      const int nchunks = (m_end - m_beg + BK - 1) / BK;
      const bool k_ok = (k0 + chunk * 8) < p.K;
      const int64_t col_bytes = static_cast<int64_t>(k0 + chunk * 8) * 2;
      // Byte offset of the source row that lane l < 16 looks up for slab c (half h, pass i), -1 = zero row.
      // Looked up three slabs ahead so that the index load is off the critical path of the copies.
      auto row_offset = [&](int c) -> long long {
        long long off = -1;
        if (lane < 16 && c < nchunks) {
          const int h = (rows_per_warp_pass == 2) ? (lane >> 3) : 0;
          const int i = (rows_per_warp_pass == 2) ? (lane & 7) : lane;
          if (i < NI) {
            const int64_t m = static_cast<int64_t>(m_beg) + c * BK + wrow0 + h + RPP * i;
            if (m < m_end) {
              const int64_t row = p.gather_idx ? p.gather_idx[m] / p.fan_out : m;
              if (row >= 0 && row < p.x_rows) off = row * p.x_row_bytes;
            }
          }
        }
        return off;
      };
      long long off0 = row_offset(0), off1 = row_offset(1), off2 = row_offset(2);
      for (int c = 0; c < nchunks; ++c, ++it) {
        const long long my_off = off0;
        off0 = off1; off1 = off2; off2 = row_offset(c + 3);
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(empty_bar(s), ph ^ 1, abort_flag, p.status, 14)) { ok = false; break; }
        if (slab_ragged(c, m_beg, m_end)) {
          // DY slab of the ragged tail: 64 rows x 128 features = 1024 16-byte chunks, 8 per thread
          const int a_chunk = ptid & 15, a_row0 = ptid >> 4;
          const bool n_ok = (n0 + a_chunk * 8) < p.N;
          const uint32_t dsta = smem_u32(sA + s * A_STAGE_BYTES) + (a_chunk >> 3) * (64 * BK * 2);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = a_row0 + 8 * i;
            const int64_t m = static_cast<int64_t>(m_beg) + c * BK + row;
            const bool v = n_ok && m < m_end;
            cp_async16(dsta + row * 128 + (((a_chunk & 7) ^ (row & 7)) << 4),
                       v ? p.DY + m * p.dy_row_bytes + static_cast<int64_t>(n0 + a_chunk * 8) * 2 : p.DY, v ? 16u : 0u);
          }
        }
        if (!slab_by_tma(c, m_beg, m_end)) {
          const uint32_t dst = smem_u32(sB + s * C::B_STAGE_BYTES) + box_off;
#pragma unroll
          for (int i = 0; i < NI; ++i) {
            const int src_lane = (rows_per_warp_pass == 2) ? (my_half * 8 + i) : i;
            const long long off = __shfl_sync(0xffffffffu, my_off, src_lane);
            const bool v = k_ok && off >= 0;
            const int row = row_base + RPP * i;     // token row inside the 64-row slab
            cp_async16(dst + row * 128 + (((chunk & 7) ^ (row & 7)) << 4), v ? p.X + off + col_bytes : p.X,
                       v ? 16u : 0u);
          }
        }
        if (p.x_by_tma) {
          // not reached: grouped X takes the branch above (p.x_by_tma is uniform for the launch)
          if (slab_ragged(c, m_beg, m_end)) {
            cp_async_commit();
            cp_async_wait<0>();
            fence_proxy_async_smem();
            mbar_arrive(full_bar(s));
          }
        } else {
          cp_async_commit();
          if (it >= A_LAG) {
            cp_async_wait<A_LAG>();
            fence_proxy_async_smem();
            mbar_arrive(full_bar((it - A_LAG) % STAGES));
          }
        }
      }
    }
    cp_async_wait<0>();
    fence_proxy_async_smem();
    if (ok && !p.x_by_tma) {
      for (int j = max(0, it - A_LAG); j < it; ++j) mbar_arrive(full_bar(j % STAGES));
    }
  } else {
    // ---------------- epilogue: rows = DY features, columns = X features -----------------------------------
    const int q = warp & 3;
    const int r = q * 32 + lane;
    uint8_t* slab = epi_staging + q * (32 * C::STAGE_ROW_BYTES);
    int tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int e, n0, k0, m_beg, m_end;
      decode(t, e, n0, k0, m_beg, m_end);
      const int nchunks = (m_end - m_beg + BK - 1) / BK;
      const bool valid = (n0 + r) < p.N;
      uint8_t* drow = p.DW + static_cast<int64_t>(e) * p.dw_e_bytes + static_cast<int64_t>(n0 + r) * p.dw_row_bytes;
      if (nchunks == 0) {
        if (valid) {
          for (int kk = k0; kk < min(k0 + BNW, p.K); kk += 8)
            *reinterpret_cast<uint4*>(drow + kk * 2) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int buf = tile_iter & 1;
      const uint32_t tph = (tile_iter >> 1) & 1;
      if (!mbar_wait_warp(tfull_bar(buf), tph, abort_flag, p.status, 15)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BNW;
#pragma unroll 1
      for (int c = 0; c < BNW / 32; ++c) {
        const int kk0 = k0 + c * 32;
        if (kk0 >= p.K) break;
        uint32_t acc[32];
        tmem_ld_32x32b_x32(taddr + c * 32, acc);
        tmem_ld_wait();
        uint4 pk[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(acc[g * 8 + j]);
          pk[g] = pack8(v, p.is_bf16);
        }
        flush_rows<4>(slab, lane, pk, drow, valid, kk0, p.K);
      }
      tc_fence_before_sync();
      mbar_arrive(tempty_bar(buf));
      ++tile_iter;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// Db[e][n] = sum of DY[m][n] over expert e's rows (the bias gradient, ops.py:358-366). HBM-bound column sum:
// a block owns one expert and 64 columns, 8 row lanes x 32 column pairs, fp32 accumulation.
template <typename T2, bool IS_BF16>
__global__ void __launch_bounds__(256)
bias_grad_kernel(const uint8_t* __restrict__ DY, int64_t dy_row_bytes, const int64_t* __restrict__ offsets, int64_t R,
                 uint8_t* __restrict__ Db, int64_t sdbe, int64_t sdbn, int N) {
  __shared__ float red[8][64];
  const int e = blockIdx.y;
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int n = blockIdx.x * 64 + cx * 2;
  int64_t beg = e ? offsets[e - 1] : 0, end = offsets[e];
  beg = beg < 0 ? 0 : (beg > R ? R : beg);
  end = end < beg ? beg : (end > R ? R : end);
  float a0 = 0.f, a1 = 0.f;
  if (n < N) {
    for (int64_t m = beg + ry; m < end; m += 8) {
      const T2 v = *reinterpret_cast<const T2*>(DY + m * dy_row_bytes + n * 2);
      a0 += __low2float(v);
      a1 += __high2float(v);
    }
  }
  red[ry][cx * 2] = a0;
  red[ry][cx * 2 + 1] = a1;
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i][threadIdx.x];
    const int nn = blockIdx.x * 64 + threadIdx.x;
    if (nn < N) {
      uint16_t* out = reinterpret_cast<uint16_t*>(Db) + static_cast<int64_t>(e) * sdbe + nn * sdbn;
      if (IS_BF16) *out = __bfloat16_as_ushort(__float2bfloat16_rn(s));
      else *out = __half_as_ushort(__float2half_rn(s));
    }
  }
}

// ---- host side -----------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// rank-3 map over (inner, outer, expert) of 16-bit elements with a 128-byte swizzled box.
static bool encode_map3(CUtensorMap* map, bool bf16, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  const cuuint32_t box[3] = {box0, box1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Tuning knobs, read once: SMOE_GROUP_M (m-tiles per raster group of the grouped GEMM) and SMOE_L2_BAND_MB (bytes
// of L2 the weight gradient plans to keep one operand's band resident in). Unset: the built-in choices.
static int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  if (!v || !*v) return fallback;
  const long x = strtol(v, nullptr, 10);
  return x > 0 && x < (1 << 20) ? static_cast<int>(x) : fallback;
}

template <int BN, bool B_KMAJOR, int EPI = EPI_NONE>
static int launch_s2s_cfg(const CUtensorMap& map, const CUtensorMap& map_x, const S2SParams& p, int grid,
                          cudaStream_t stream) {
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  SMOE_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      SMOE_CUDA(cudaFuncSetAttribute(s2s_tc_kernel<BN, B_KMAJOR, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg<BN>::SMEM_BYTES));
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  s2s_tc_kernel<BN, B_KMAJOR, EPI><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(map, map_x, p);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

// rank-2 map over (feature, row) of 16-bit elements, box0 x box1 box (64 x 64 by default), 128-byte swizzle.
static bool encode_map2(CUtensorMap* map, bool bf16, const void* base, uint64_t d0, uint64_t d1,
                        uint64_t stride1_bytes, uint32_t box0 = 64, uint32_t box1 = BK) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {d0, d1};
  const cuuint64_t strides[1] = {stride1_bytes};
  const cuuint32_t box[2] = {box0, box1};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

template <int BNW>
static int launch_wgrad_cfg(const CUtensorMap& map, const CUtensorMap& map_x, const WGradParams& p, int grid,
                            cudaStream_t stream) {
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  SMOE_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      SMOE_CUDA(cudaFuncSetAttribute(wgrad_tc_kernel<BNW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg<BNW>::SMEM_BYTES));
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  wgrad_tc_kernel<BNW><<<grid, NUM_THREADS, Cfg<BNW>::SMEM_BYTES, stream>>>(map, map_x, p);
  SMOE_LAUNCH_CHECK();
  return SMOE_OK;
}

}  // namespace tc

int launch_s2s_tc(const S2SArgs& a) {
  using namespace tc;
  if (a.dtype != SMOE_BF16 && a.dtype != SMOE_F16) return SMOE_ERR_UNSUPPORTED;
  if (a.K < 8 || a.K % 8 || a.N % 8 || a.E > MAX_E) return SMOE_ERR_UNSUPPORTED;
  if (a.sxk != 1 || a.sxm % 8 || !al16(a.X)) return SMOE_ERR_UNSUPPORTED;
  const bool to_peers = a.out_addr != nullptr;
  if (!to_peers && (a.syn != 1 || a.sym % 8 || !al16(a.Y))) return SMOE_ERR_UNSUPPORTED;
  if (to_peers && (a.act_layout >= 0 || a.act_bwd || a.bias || a.N <= 128 || a.out_peers == nullptr || a.out_peer_stride % 8 ||
                   a.out_peer_stride < a.N || a.out_world < 1 || a.out_world > EP_MAX_WORLD))
    return SMOE_ERR_UNSUPPORTED;
  if (a.bias && a.sbn != 1) return SMOE_ERR_UNSUPPORTED;
  if (!al16(a.W) || a.swe % 8 || a.swe < 0) return SMOE_ERR_UNSUPPORTED;
  const bool k_major = (a.swk == 1 && a.swn % 8 == 0 && a.swn >= a.K);
  const bool n_major = (a.swn == 1 && a.swk % 8 == 0 && a.swk >= a.N);
  if (!k_major && !n_major) return SMOE_ERR_UNSUPPORTED;
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  if (di.cc_major != 10) return SMOE_ERR_UNSUPPORTED;

  const bool bf16 = a.dtype == SMOE_BF16;
  // fused activation epilogue: which kernel variant, and what it needs
  int epi = EPI_NONE, F = 0;
  if (a.act_layout >= 0 && !a.act_bwd) {
    if (a.N <= 128 || a.H == nullptr || a.shm % 8 || !al16(a.H)) return SMOE_ERR_UNSUPPORTED;
    if (a.act_layout == LAYOUT_PLAIN) { epi = EPI_ACT; F = a.N; }
    else if (a.act_layout == LAYOUT_GPT_OSS) { epi = EPI_GPT_OSS; F = a.N / 2; if (a.N % 16) return SMOE_ERR_UNSUPPORTED; }
    else { epi = EPI_GLU_HALVES; F = a.N / 2; if (a.N % 16) return SMOE_ERR_UNSUPPORTED; }
    if (a.Y && (a.syn != 1 || a.sym % 8 || !al16(a.Y))) return SMOE_ERR_UNSUPPORTED;
  }
  if (a.act_bwd) {
    // fused activation gradient: N = F hidden columns, U and Y (= dU) are (rows, n_up)
    if (a.N <= 128 || a.U == nullptr || a.sum % 8 || !al16(a.U) || !a.x_grouped || !a.y_grouped || a.bias)
      return SMOE_ERR_UNSUPPORTED;
    epi = a.act_layout == LAYOUT_PLAIN ? EPI_BWD_PLAIN : (a.act_layout == LAYOUT_GPT_OSS ? EPI_BWD_GPT_OSS : EPI_BWD_GLU);
    F = a.N;
  }
  if (to_peers) epi = EPI_PEERS;
  const int BN = a.N > 128 ? 256 : 128;
  CUtensorMap map;
  const uint64_t e_stride = (a.E > 1 ? static_cast<uint64_t>(a.swe) : static_cast<uint64_t>(a.K) * a.N) * 2;
  bool ok;
  if (k_major)
    ok = encode_map3(&map, bf16, a.W, a.K, a.N, a.E, static_cast<uint64_t>(a.swn) * 2, e_stride, BK,
                     epi == EPI_GLU_HALVES ? BN / 2 : BN);
  else
    ok = encode_map3(&map, bf16, a.W, a.N, a.K, a.E, static_cast<uint64_t>(a.swk) * 2, e_stride, 64, BK);
  if (!ok) return SMOE_ERR_UNSUPPORTED;

  S2SParams p;
  p.X = static_cast<const uint8_t*>(a.X); p.x_row_bytes = a.sxm * 2; p.x_rows = a.x_rows;
  p.bias = static_cast<const uint8_t*>(a.bias); p.bias_row_elems = a.sbe;
  p.Y = static_cast<uint8_t*>(a.Y); p.y_row_bytes = a.sym * 2;
  p.sorted_idx = a.sorted_idx; p.offsets = a.offsets; p.R = a.R;
  p.K = a.K; p.N = a.N; p.E = a.E; p.fan_out = a.fan_out; p.x_grouped = a.x_grouped; p.y_grouped = a.y_grouped;
  p.is_bf16 = bf16 ? 1 : 0;
  p.bias_vec = (a.bias && al16(a.bias) && a.sbe % 8 == 0) ? 1 : 0;
  p.idesc = make_idesc_f16(bf16, false, !k_major, BM, BN);
  p.status = a.status;
  p.H = static_cast<uint8_t*>(a.H); p.h_row_bytes = a.shm * 2;
  p.F = F; p.glu_first = a.act_layout == LAYOUT_GLU_FIRST ? 1 : 0; p.act = a.act; p.alpha = a.alpha; p.limit = a.limit;
  p.U = static_cast<const uint8_t*>(a.U); p.u_row_bytes = a.sum * 2;
  p.row_gate = static_cast<const uint8_t*>(a.row_gate);
  p.dot_out = a.dot_out; p.dot_stride = a.R;
  {
    // SMOE_EPI_DIRECT=2 keeps the staged stores (a measurement hook)
    auto al32 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31) == 0; };
    p.wide_rows = (a.act_bwd && a.N % 16 == 0 && a.sum % 16 == 0 && a.sym % 16 == 0 && al32(a.U) && al32(a.Y) &&
                   env_int("SMOE_EPI_DIRECT", 1) == 1) ? 1 : 0;
  }
  p.out_addr = a.out_addr; p.out_peer_row_bytes = a.out_peer_stride * 2; p.out_peer_rows = a.out_peer_rows;
  p.out_world = a.out_world; p.m_rot_num = 0; p.m_rot_den = 1;
  const int peer_store_bytes = to_peers ? env_int("SMOE_PEER_STORE_BYTES", 128) : 0;    // read per launch: a test hook
  p.out_pieces = peer_store_bytes >= 256 ? 16 : (peer_store_bytes >= 128 ? 8 : 4);
  for (int i = 0; i < EP_MAX_WORLD; ++i) p.out_peer.p[i] = nullptr;
  if (to_peers) {
    for (int i = 0; i < a.out_world; ++i) {
      p.out_peer.p[i] = static_cast<uint8_t*>(a.out_peers[i]);
      if (p.out_peer.p[i] == nullptr || !al16(p.out_peer.p[i])) return SMOE_ERR_UNSUPPORTED;
    }
    p.Y = nullptr; p.y_row_bytes = 0;
    if (a.my_rank > 0 && a.my_rank < a.out_world) { p.m_rot_num = a.my_rank; p.m_rot_den = a.out_world; }
  }
  // Raster (see decode_tile). While one expert's A panel (its rows x K) fits comfortably in L2, every m-tile of the
  // expert runs beside each column tile, so each weight tile is fetched from HBM once and the A panel comes from L2.
  // When the panel does not fit, both operands stream from HBM for every wave of tiles in flight and the wave is
  // shaped to minimise their sum: about sqrt(tiles in flight * tile columns / tile rows) m-tiles per group.
  static const int group_m_env = env_int("SMOE_GROUP_M", 0);
  const double a_panel_bytes = static_cast<double>(a.R) / a.E * a.K * 2.0;
  p.group_m = group_m_env ? group_m_env : (a_panel_bytes <= 48e6 ? (1 << 20) : (BN == 256 ? 16 : 12));

  CUtensorMap map_x = map;   // placeholder when the rows are gathered: the kernel then never touches it
  p.a_by_tma = (a.x_grouped && !(a.flags & SMOE_FLAG_GATHER_ROWS) && a.sxm >= a.K &&
                encode_map2(&map_x, bf16, a.X, a.K, a.x_rows, static_cast<uint64_t>(a.sxm) * 2, 64, BM)) ? 1 : 0;

  const int tile_cols = epi == EPI_GLU_HALVES ? BN / 2 : BN;

  const int64_t max_tiles = (cdiv64(a.R, BM) + a.E) * cdiv(epi == EPI_GLU_HALVES ? F : a.N, tile_cols);
  const int grid = static_cast<int>(max_tiles < di.sm_count ? max_tiles : di.sm_count);
  switch (epi) {
    case EPI_ACT:
      return k_major ? launch_s2s_cfg<256, true, EPI_ACT>(map, map_x, p, grid, a.stream)
                     : launch_s2s_cfg<256, false, EPI_ACT>(map, map_x, p, grid, a.stream);
    case EPI_GLU_HALVES:
      return k_major ? launch_s2s_cfg<256, true, EPI_GLU_HALVES>(map, map_x, p, grid, a.stream)
                     : launch_s2s_cfg<256, false, EPI_GLU_HALVES>(map, map_x, p, grid, a.stream);
    case EPI_GPT_OSS:
      return k_major ? launch_s2s_cfg<256, true, EPI_GPT_OSS>(map, map_x, p, grid, a.stream)
                     : launch_s2s_cfg<256, false, EPI_GPT_OSS>(map, map_x, p, grid, a.stream);
    case EPI_BWD_PLAIN:
      return k_major ? launch_s2s_cfg<256, true, EPI_BWD_PLAIN>(map, map_x, p, grid, a.stream)
                     : launch_s2s_cfg<256, false, EPI_BWD_PLAIN>(map, map_x, p, grid, a.stream);
    case EPI_BWD_GLU:
      return k_major ? launch_s2s_cfg<256, true, EPI_BWD_GLU>(map, map_x, p, grid, a.stream)
                     : launch_s2s_cfg<256, false, EPI_BWD_GLU>(map, map_x, p, grid, a.stream);
    case EPI_BWD_GPT_OSS:
      return k_major ? launch_s2s_cfg<256, true, EPI_BWD_GPT_OSS>(map, map_x, p, grid, a.stream)
                     : launch_s2s_cfg<256, false, EPI_BWD_GPT_OSS>(map, map_x, p, grid, a.stream);
    case EPI_PEERS:
      return k_major ? launch_s2s_cfg<256, true, EPI_PEERS>(map, map_x, p, grid, a.stream)
                     : launch_s2s_cfg<256, false, EPI_PEERS>(map, map_x, p, grid, a.stream);
    default: break;
  }
  if (BN == 256)
    return k_major ? launch_s2s_cfg<256, true>(map, map_x, p, grid, a.stream)
                   : launch_s2s_cfg<256, false>(map, map_x, p, grid, a.stream);
  return k_major ? launch_s2s_cfg<128, true>(map, map_x, p, grid, a.stream)
                 : launch_s2s_cfg<128, false>(map, map_x, p, grid, a.stream);
}

int launch_wgrad_tc(const WGradArgs& a) {
  using namespace tc;
  if (a.dtype != SMOE_BF16 && a.dtype != SMOE_F16) return SMOE_ERR_UNSUPPORTED;
  if (a.K % 8 || a.N % 8 || a.E > MAX_E || a.R == 0) return SMOE_ERR_UNSUPPORTED;
  if (a.sxk != 1 || a.sxm % 8 || !al16(a.X)) return SMOE_ERR_UNSUPPORTED;
  if (a.sdyn != 1 || a.sdym % 8 || a.sdym < a.N || !al16(a.DY)) return SMOE_ERR_UNSUPPORTED;
  if (a.sdwk != 1 || a.sdwn % 8 || a.sdwe % 8 || !al16(a.DW)) return SMOE_ERR_UNSUPPORTED;
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  if (di.cc_major != 10) return SMOE_ERR_UNSUPPORTED;
  const bool bf16 = a.dtype == SMOE_BF16;
  CUtensorMap map;
  if (!encode_map2(&map, bf16, a.DY, a.N, a.R, static_cast<uint64_t>(a.sdym) * 2)) return SMOE_ERR_UNSUPPORTED;
  const int BNW = a.K > 128 ? 256 : 128;
  CUtensorMap map_x = map;   // placeholder when X is gathered: the kernel then never touches it
  const bool x_by_tma = a.gather_idx == nullptr && a.sxm >= a.K &&
                        encode_map2(&map_x, bf16, a.X, a.K, a.x_rows, static_cast<uint64_t>(a.sxm) * 2);
  WGradParams p;
  p.DY = static_cast<const uint8_t*>(a.DY); p.dy_row_bytes = a.sdym * 2;
  p.x_by_tma = x_by_tma ? 1 : 0;
  p.X = static_cast<const uint8_t*>(a.X); p.x_row_bytes = a.sxm * 2; p.x_rows = a.x_rows;
  p.DW = static_cast<uint8_t*>(a.DW); p.dw_e_bytes = a.sdwe * 2; p.dw_row_bytes = a.sdwn * 2;
  p.gather_idx = a.gather_idx; p.offsets = a.offsets; p.R = a.R;
  p.K = a.K; p.N = a.N; p.E = a.E; p.fan_out = a.fan_out; p.is_bf16 = bf16 ? 1 : 0;
  p.idesc = make_idesc_f16(bf16, true, true, BM, BNW);
  p.status = a.status;
  {
    // Which operand's band stays in L2 (see the tile order in the kernel). The row count per expert is only
    // known on the device; the average decides. Bytes read per expert: the banded operand once, the streamed
    // one once per band.
    static const int budget_mb = env_int("SMOE_L2_BAND_MB", 40);
    const double rows = static_cast<double>(a.R) / a.E, budget = budget_mb * 1e6;
    const int n_tiles = cdiv(a.N, BM), k_tiles = cdiv(a.K, BNW);
    auto width = [&](int tiles, int tile_cols) {
      const int fit = static_cast<int>(budget / (tile_cols * rows * 2.0 + 1.0));
      const int w = fit < 1 ? 1 : (fit > tiles ? tiles : fit);
      return cdiv(tiles, cdiv(tiles, w));          // equal-sized bands
    };
    const int wn = width(n_tiles, BM), wk = width(k_tiles, BNW);
    const double dy_panel = a.N * rows * 2.0, x_panel = a.K * rows * 2.0;
    const double bytes_over_n = dy_panel + x_panel * cdiv(n_tiles, wn);
    const double bytes_over_k = x_panel + dy_panel * cdiv(k_tiles, wk);
    p.band_over_n = bytes_over_n < bytes_over_k ? 1 : 0;
    p.band = p.band_over_n ? wn : wk;
  }
  const int64_t total = static_cast<int64_t>(a.E) * cdiv(a.N, BM) * cdiv(a.K, BNW);
  const int grid = static_cast<int>(total < di.sm_count ? total : di.sm_count);
  int rc = (BNW == 256) ? launch_wgrad_cfg<256>(map, map_x, p, grid, a.stream)
                        : launch_wgrad_cfg<128>(map, map_x, p, grid, a.stream);
  if (rc != SMOE_OK) return rc;
  if (a.Db) {
    dim3 g(static_cast<unsigned>(cdiv(a.N, 64)), static_cast<unsigned>(a.E));
    if (bf16)
      bias_grad_kernel<__nv_bfloat162, true><<<g, 256, 0, a.stream>>>(static_cast<const uint8_t*>(a.DY), a.sdym * 2, a.offsets,
                                                                     a.R, static_cast<uint8_t*>(a.Db), a.sdbe, a.sdbn, a.N);
    else
      bias_grad_kernel<__half2, false><<<g, 256, 0, a.stream>>>(static_cast<const uint8_t*>(a.DY), a.sdym * 2, a.offsets, a.R,
                                                               static_cast<uint8_t*>(a.Db), a.sdbe, a.sdbn, a.N);
    SMOE_LAUNCH_CHECK();
  }
  return SMOE_OK;
}

}  // namespace smoe
