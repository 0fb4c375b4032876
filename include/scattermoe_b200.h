/*
 * scattermoe_b200 — C ABI of the B200 (sm_100a) kernels behind ScatterMoE's `ParallelLinear` path.
 *
 * Conventions (all entry points):
 *   - every pointer is a DEVICE pointer owned by the caller unless the comment says otherwise; the library
 *     never allocates, frees or synchronises; work is enqueued on `stream` (a cudaStream_t passed as void*)
 *     of the CUDA device that is current on the calling thread;
 *   - strides are in ELEMENTS, sizes in elements/rows; index tensors are int64 like the reference's;
 *   - return value: SMOE_OK (0) or one of the SMOE_ERR_* codes; `smoe_last_error()` gives the message of the
 *     last failure on the calling thread. Nothing throws, aborts or traps;
 *   - `status` (nullable) is a device int32[4] word the tensor-core kernels write if one of their bounded waits
 *     ran out: status[0] != 0 means "device timeout", status[1..3] say where. The caller reads it when it likes.
 *
 * Each declaration cites the interface of the reference project (shawntan/scattermoe) that it replaces.
 */
#ifndef SCATTERMOE_B200_H
#define SCATTERMOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMOE_ABI_VERSION 4

enum smoe_status {
  SMOE_OK = 0,
  SMOE_ERR_BAD_ARG = 1,       /* shape / pointer / enum value rejected */
  SMOE_ERR_UNSUPPORTED = 2,   /* valid request this build has no kernel for */
  SMOE_ERR_CUDA = 3,          /* a CUDA runtime/driver call failed (message has the CUDA error) */
  SMOE_ERR_WORKSPACE = 4,     /* workspace too small or missing */
  SMOE_ERR_ARCH = 5           /* current device is not sm_100 */
};

enum smoe_dtype { SMOE_F32 = 0, SMOE_BF16 = 1, SMOE_F16 = 2 };

/* flags for the GEMM entry points */
enum smoe_flags {
  SMOE_FLAG_ALLOW_TF32 = 1,   /* fp32 inputs may use reduced-precision tensor cores (ops.py:7 ALLOW_TF32) */
  SMOE_FLAG_FORCE_SIMT = 2,   /* take the CUDA-core kernel even where a tensor-core kernel exists */
  SMOE_FLAG_FORCE_TC = 4,     /* fail with SMOE_ERR_UNSUPPORTED instead of taking the CUDA-core kernel */
  SMOE_FLAG_GATHER_ROWS = 8   /* feed grouped inputs through the row-gather path too (testing / comparison) */
};

int smoe_version(void);
const char* smoe_last_error(void);
/* 1 if the last GEMM-shaped call on this thread ran on tcgen05 tensor cores, 0 if on CUDA cores. */
int smoe_last_path_was_tensor_core(void);

/* ---- routing bookkeeping ----------------------------------------------------------------------------
 * Replaces flatten_sort_count (scattermoe/parallel_experts.py:14-21): torch.sort + scattermoe::bincount
 * (:6-12) + cumsum. One stable counting sort: `sorted_expert_idxs[R]` ascending, `sorted_scattered_idxs[R]`
 * = flat slot index t*k+j of each sorted entry (ascending inside one expert), `expert_offsets[E]` =
 * inclusive cumulative counts. Ids outside [0, E) are ignored (their output slots are left untouched).
 * Limits: 0 <= R < 2^31, 1 <= E <= 4096. */
size_t smoe_sort_count_workspace_bytes(int64_t R, int32_t E);
int smoe_sort_count(const int64_t* expert_idxs, int64_t R, int32_t E,
                    int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, int64_t* expert_offsets,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Allocation-free variant of smoe_sort_count. It has no counterpart in the reference. It exists for hosts that
 * bind this C ABI directly and cannot obtain device memory at call time: servers that hand the whole HBM to
 * their own arena at start-up and forbid cudaMalloc on the request path (it synchronises the device and can fail
 * once memory is fragmented), or embedders without a device allocator at all. The caller passes only inputs
 * and outputs; the block histograms go to a 512 KiB array built into the library (one per GPU that loads it,
 * held until the process exits). Limit: ceil(R / 2048) * E <= smoe_sort_count_static_capacity() (131072), e.g.
 * R <= 2^21 slots at E = 128; larger requests return SMOE_ERR_WORKSPACE. The call performs no cudaMalloc,
 * cudaFree or other allocating call. The first call on each device looks up the array's device address (a
 * host-side set-up step, done with that device current): make that first call before any stream capture.
 * All calls on one device share the array: calls that may overlap on the GPU (different streams) race; calls
 * issued in order on one stream do not, and nothing has to be cleared between them. */
int64_t smoe_sort_count_static_capacity(void);
int smoe_sort_count_static(const int64_t* expert_idxs, int64_t R, int32_t E,
                           int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, int64_t* expert_offsets,
                           void* stream);

/* Router fusion: from the router's logits to everything flatten_sort_count returns, without the (T, E) softmax
 * round trip and the separate top-k / renormalise / histogram kernels of the callers of flatten_sort_count
 * (scattermoe/utils/replace_moe.py:67-71; the reference test, tests/test_mlp.py:46-51; Hugging Face's top-k routers).
 *   mode 0: p = softmax(logits) over all E experts, gates = the k largest p (renormalize != 0: divided by their sum)
 *   mode 1: gates = softmax over the k largest logits
 * Outputs: expert_idxs (T, k) int64, descending by logit (equal logits: lower expert id first); gates (T, k) fp32;
 * lse (T) fp32 log-sum-exp over all experts (nullable); and the three outputs of smoe_sort_count for expert_idxs.
 * logits is (T, E), row stride `stride_t` elements, inner stride 1, dtype SMOE_F32 / BF16 / F16 (arithmetic in fp32).
 * One kernel produces ids, gates and the sort's block histograms; the sort's scan and scatter kernels follow.
 * Limits: E <= 1024, k <= min(E, 32), beyond which SMOE_ERR_UNSUPPORTED is returned (no error text) and the caller
 * runs its own top-k followed by smoe_sort_count. */
size_t smoe_route_topk_workspace_bytes(int64_t T, int32_t k, int32_t E);
int smoe_route_topk(const void* logits, int64_t T, int32_t E, int64_t stride_t, int32_t logits_dtype, int32_t k,
                    int32_t mode, int32_t renormalize, int64_t* expert_idxs, float* gates, float* lse,
                    int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, int64_t* expert_offsets,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Inclusive end offsets from the sorted ids alone. The reference's kernels.ops.scatter2scatter
 * (scattermoe/kernels/ops.py:120) receives no offsets and masks rows per expert inside the kernel
 * (:81-91); this build's grouped GEMM walks expert segments, so callers that only hold the sorted ids
 * derive the offsets with this call first. */
int smoe_offsets_from_sorted(const int64_t* sorted_expert_idxs, int64_t R, int32_t E,
                             int64_t* expert_offsets, void* stream);

/* ---- grouped GEMM with fused row gather / scatter -----------------------------------------------------
 * Replaces kernels.ops.scatter2scatter (scattermoe/kernels/ops.py:120-183, kernel :55-118).
 * For sorted position m in [0, R) with expert e(m):
 *     Y[out(m), :] = X[in(m), :] @ W[e(m)] (+ bias[e(m), :])
 *     in(m)  = m if x_grouped else sorted_scattered_idxs[m] / fan_out
 *     out(m) = m if y_grouped else sorted_scattered_idxs[m]
 * X is (x_rows, K), W is (E, K, N) with arbitrary element strides (either K or N contiguous for the
 * tensor-core kernel), Y is (R, N). fp32 accumulation; Y, bias in the dtype of X and W.
 * `expert_offsets` is REQUIRED (see smoe_offsets_from_sorted). */
int smoe_scatter2scatter(const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk,
                         const void* W, int64_t stride_we, int64_t stride_wk, int64_t stride_wn,
                         const void* bias, int64_t stride_be, int64_t stride_bn,
                         void* Y, int64_t stride_ym, int64_t stride_yn,
                         const int64_t* sorted_expert_idxs, const int64_t* sorted_scattered_idxs,
                         const int64_t* expert_offsets,
                         int64_t R, int32_t K, int32_t N, int32_t E, int32_t fan_out,
                         int32_t x_grouped, int32_t y_grouped, int32_t dtype, int32_t flags,
                         int32_t* status, void* stream);

/* ---- per-expert weight gradient ---------------------------------------------------------------------
 * Replaces kernels.ops.group_bwd_W (scattermoe/kernels/ops.py:191-239, kernel :247-366).
 *     DW[e][kk][n] = sum over rows m of expert e of X[xrow(m)][kk] * DY[m][n]
 *     Db[e][n]     = sum over rows m of expert e of DY[m][n]          (Db nullable)
 * DY is (R, N) grouped. X is grouped (x_gather_idx == NULL, xrow(m) = m) or, an extension of the
 * reference, still un-grouped: xrow(m) = x_gather_idx[m] / fan_out, which removes the reference's
 * group(x) copy (scattermoe/parallel_experts.py:99). DW is addressed through its element strides
 * (the reference hands out the (E,K,N) permuted view of an (E,N,K) buffer, ops.py:192-193). Every
 * element of DW and Db is written, experts without rows get zeros: no pre-zeroing is needed. */
int smoe_group_bwd_w(const void* DY, int64_t stride_dym, int64_t stride_dyn,
                     const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk,
                     const int64_t* expert_offsets, const int64_t* x_gather_idx, int32_t fan_out,
                     void* DW, int64_t stride_dwe, int64_t stride_dwk, int64_t stride_dwn,
                     void* Db, int64_t stride_dbe, int64_t stride_dbn,
                     int64_t R, int32_t K, int32_t N, int32_t E, int32_t dtype, int32_t flags,
                     int32_t* status, void* stream);

/* ---- row gather with optional per-row scale -----------------------------------------------------------
 * Replaces kernels.ops.group (scattermoe/kernels/ops.py:377-410, kernel :417-457):
 *     Y[n, :] = A[idx[n] / fan_out, :] * coeff[idx[n]]     (coeff nullable, same dtype as A) */
int smoe_group(const void* A, int64_t a_rows, int64_t stride_am, int64_t stride_ak,
               const int64_t* idx, const void* coeff, int32_t fan_out,
               void* Y, int64_t stride_ym, int64_t stride_yk,
               int64_t R, int32_t K, int32_t dtype, void* stream);

/* ---- top-k reductions around the GEMMs ----------------------------------------------------------------
 * smoe_topk_reduce replaces `(gates.unsqueeze(1) @ output.view(T,k,N)).squeeze(1)`
 * (scattermoe/parallel_experts.py:44-46) and, with gates == NULL, `.view(T,k,K).sum(-2)` (:123):
 *     out[t, :] = sum_j gates[t, j] * Yx[t*k + j, :]        fp32 accumulation
 * smoe_gate_grad replaces `(output_expanded @ grad_out.unsqueeze(-1)).squeeze(-1)` (:79):
 *     d_gates[t, j] = <Yx[t*k + j, :], grad_out[t, :]>     fp32 accumulation */
int smoe_topk_reduce(const void* Yx, int64_t stride_yxm, const void* gates, int64_t stride_gt, int64_t stride_gk,
                     void* out, int64_t stride_om, int64_t T, int32_t k, int32_t N, int32_t dtype, void* stream);
int smoe_gate_grad(const void* Yx, int64_t stride_yxm, const void* grad_out, int64_t stride_gom,
                   void* d_gates, int64_t stride_dgt, int64_t stride_dgk,
                   int64_t T, int32_t k, int32_t N, int32_t dtype, void* stream);

/* ---- activation between the two expert linears ---------------------------------------------------------
 * Replaces the PyTorch elementwise ops + autograd of scattermoe/mlp.py:41 (MLP), :81-87 (GLUMLP),
 * scattermoe/utils/replace_moe.py:76-83 (granite) and :39-43 (gpt-oss) with one pass per direction.
 * U is the (rows, n_up) up-projection, H the (rows, F) hidden activations, inner strides 1:
 *   layout 0 PLAIN       n_up = F    H[j] = act(U[j])
 *   layout 1 GLU_SECOND  n_up = 2F   H[j] = act(U[F+j]) * U[j]
 *   layout 2 GLU_FIRST   n_up = 2F   H[j] = act(U[j]) * U[F+j]
 *   layout 3 GPT_OSS     n_up = 2F   g = min(U[2j], limit), u = clamp(U[2j+1], -limit, limit),
 *                                    H[j] = (u + 1) * g * sigmoid(alpha * g)        (act ignored)
 *   act: 0 SiLU, 1 GELU (erf), 2 GELU (tanh), 3 ReLU, 4 identity.
 * smoe_activation_backward writes DU = dL/dU (rows, n_up) from U and DH = dL/dH.
 * `rows_dev` (nullable device int64): when the live row count is only known on the device (expert-parallel
 * receive buffers sized for the worst case) only min(rows, *rows_dev) rows are processed. */
int smoe_activation_forward(const void* U, int64_t stride_um, void* H, int64_t stride_hm, int64_t rows,
                            const int64_t* rows_dev, int32_t F, int32_t layout, int32_t act, float alpha, float limit,
                            int32_t dtype, void* stream);
int smoe_activation_backward(const void* U, int64_t stride_um, const void* DH, int64_t stride_dhm, void* DU,
                             int64_t stride_dum, int64_t rows, const int64_t* rows_dev, int32_t F, int32_t layout,
                             int32_t act, float alpha, float limit, int32_t dtype, void* stream);

/* Up-projection + activation in one kernel: smoe_scatter2scatter with grouped output (y_grouped = 1) whose
 * epilogue also writes H = activation(Y) (layouts / functions as above; Y nullable when the up-projection itself
 * is not needed, e.g. inference). Fuses scattermoe/mlp.py:35-41 / :76-87 (the first expert linear and the
 * activation after it). Tensor-core kernel only: returns SMOE_ERR_UNSUPPORTED when the request does not fit it
 * (dtype, alignment, N <= 128), and the caller runs the two separate calls instead.
 * `row_gates` (nullable; the (T, k) gates, flat, in the dtype of X): H receives activation(Y) * gates[slot of the row]
 * instead. The down-projection is linear, so a layer whose hidden rows carry the gate needs no gate weighting after
 * it (scattermoe/parallel_experts.py:44-46 becomes a plain sum over the k slots); Y stays un-weighted. */
int smoe_scatter2scatter_act(const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk,
                             const void* W, int64_t stride_we, int64_t stride_wk, int64_t stride_wn,
                             const void* bias, int64_t stride_be, int64_t stride_bn,
                             void* Y, int64_t stride_ym, int64_t stride_yn, void* H, int64_t stride_hm,
                             const int64_t* sorted_expert_idxs, const int64_t* sorted_scattered_idxs,
                             const int64_t* expert_offsets, int64_t R, int32_t K, int32_t N, int32_t E,
                             int32_t fan_out, int32_t x_grouped, int32_t dtype, int32_t flags, int32_t act_layout,
                             int32_t act, float alpha, float limit, const void* row_gates, int32_t* status,
                             void* stream);

/* Input gradient of the down-projection + activation gradient in one kernel. Fuses the backward of
 * scattermoe/mlp.py:41 / :81-87 (PyTorch autograd of the activation in the reference) into the grouped GEMM that the
 * reference runs for the down-projection's input gradient (scattermoe/parallel_experts.py:110-116):
 *     dU = d activation(U) applied to dH,   dH = DY @ W    (never stored)
 * DY (R, K) and U, DU (R, n_up) are in expert order, W is (E, K, F) in element strides (the transposed view of the
 * down-projection weight), layouts / functions as for smoe_activation_backward, n_up = F (plain) or 2F.
 * Tensor-core kernel only: returns SMOE_ERR_UNSUPPORTED when the request does not fit it (dtype, alignment,
 * F <= 128); the caller then runs smoe_scatter2scatter and smoe_activation_backward.
 * With `row_gates` (nullable, as in smoe_scatter2scatter_act; then `sorted_scattered_idxs` and `gate_partials` are
 * required too) DY is the UN-weighted output gradient in expert order: the epilogue scales dH by the row's gate and
 * also writes, for the gate gradient of scattermoe/parallel_experts.py:79 (<expert output, output gradient> =
 * <hidden, dH>), the partial dot products of dH with the un-weighted hidden row over its chunks of columns:
 * gate_partials is (smoe_act_bwd_partial_lines(F), R) fp32, every entry written; smoe_gate_grad_from_partials adds
 * the lines up into d_gates[slot of row m] (T*k values in `dtype`). Deterministic: no atomics. */
int smoe_scatter2scatter_act_bwd(const void* DY, int64_t stride_dym, int64_t stride_dyk,
                                 const void* W, int64_t stride_we, int64_t stride_wk, int64_t stride_wn,
                                 const void* U, int64_t stride_um, void* DU, int64_t stride_dum,
                                 const int64_t* expert_offsets, int64_t R, int32_t K, int32_t F, int32_t E,
                                 int32_t dtype, int32_t flags, int32_t act_layout, int32_t act, float alpha,
                                 float limit, const void* row_gates, const int64_t* sorted_scattered_idxs,
                                 float* gate_partials, int32_t* status, void* stream);
int32_t smoe_act_bwd_partial_lines(int32_t F);
int smoe_gate_grad_from_partials(const float* partials, int32_t lines, int64_t R, const int64_t* sorted_scattered_idxs,
                                 void* d_gates, int32_t dtype, void* stream);

/* ---- single-token decode ---------------------------------------------------------------------------------
 * Replaces kernels.single.single2scatter (scattermoe/kernels/single.py:41-59, kernel :5-39): the k expert
 * matvecs of one token, Y[j, :] = X[j or 0, :] @ W[expert_idxs[j]]; X has 1 or k rows; any strides, any K and N
 * (the reference needs multiples of 128); fp32 accumulation. */
int smoe_single2scatter(const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk, const void* W,
                        int64_t stride_we, int64_t stride_wk, int64_t stride_wn, void* Y, int64_t stride_ym,
                        int64_t stride_yn, const int64_t* expert_idxs, int32_t k, int32_t K, int32_t N, int32_t E,
                        int32_t dtype, void* stream);

/* ---- expert-parallel row exchange over NVLink peer memory -----------------------------------------------
 * No counterpart in the reference (it has no multi-GPU code). `peer_*` arguments are HOST arrays of `world` device
 * pointers, entry w = that buffer of rank w mapped into this process (e.g. a symmetric-memory allocation); entry
 * `my_rank` is the local buffer. The calls only enqueue plain peer stores; ordering against the other ranks (a
 * barrier between phases) is the caller's. Both directions push.
 *
 * smoe_ep_dispatch: for every position m of this rank's expert-sorted slot list (global expert e, slot s):
 *     row = dst_offsets[e] + (m - first position of e);  owner = e / (E/world)
 *     peer_bufs[owner][row, :]      = X[s / fan_out, :] * coeff[s]          (coeff nullable)
 *     peer_return_addr[owner][row]  = my_rank << 40 | s                      (nullable: not recorded)
 *   `dst_offsets[e]` = first row reserved for this rank's rows of expert e in the owner's (capacity_rows,
 *   peer_stride_rows) buffer, chosen so that the owner's buffer ends up expert-grouped with no further copy.
 * smoe_ep_return: for every row i < min(capacity_rows, *live_rows) of the local (capacity_rows, K) result Y:
 *     (r, s) = return_addr[i];  peer_slot_bufs[r][s, :] = Y[i, :]           (peer buffers are (peer_rows, stride))
 * Both kernels walk their rows in an order rotated by the calling rank (dispatch: starting with the next rank's
 * experts; return: starting `my_rank` (expert, sender) sub-segments in, `local_experts` = E / world), so that at any
 * moment the ranks write to different peers instead of all to the same one. */
int smoe_ep_dispatch(const void* X, int64_t x_rows, int64_t stride_xm, const int64_t* sorted_expert_idxs,
                     const int64_t* sorted_scattered_idxs, const int64_t* expert_offsets, const int64_t* dst_offsets,
                     const void* coeff, int32_t fan_out, void* const* peer_bufs, int64_t peer_stride_rows,
                     int64_t capacity_rows, void* const* peer_return_addr, int32_t my_rank, int64_t R, int32_t K,
                     int32_t E, int32_t world, int32_t dtype, void* stream);
/* smoe_ep_plan_rows: the placement arithmetic between the all-gather of every rank's expert offsets and
 * smoe_ep_dispatch, as one small kernel. all_offsets is (world, E) int64, row s = sender s's inclusive per-expert ends
 * (its smoe_sort_count offsets). Writes dst_offsets (E,) for smoe_ep_dispatch (every owner's buffer ordered (local
 * expert, sender)) and local_offsets (E / world,), the inclusive ends of this rank's own experts in its buffer. */
int smoe_ep_plan_rows(const int64_t* all_offsets, int32_t my_rank, int32_t world, int32_t E, int64_t* dst_offsets,
                      int64_t* local_offsets, void* stream);
int smoe_ep_return(const void* Y, int64_t stride_ym, const int64_t* return_addr, const int64_t* live_rows,
                   int64_t capacity_rows, void* const* peer_slot_bufs, int64_t peer_stride_rows, int64_t peer_rows,
                   int32_t K, int32_t world, int32_t my_rank, int32_t local_experts, int32_t dtype, void* stream);
/* smoe_scatter2scatter_to_peers: the grouped GEMM of the local experts and smoe_ep_return in ONE kernel. X is the
 * owner's expert-grouped (x_rows, K) buffer (x_rows = its capacity; the live rows are those the offsets of the E
 * LOCAL experts delimit), W is (E, K, N) in element strides; for every live row i
 *     (r, s) = return_addr[i];  peer_slot_bufs[r][s, 0:N] = X[i, :] @ W[expert of row i]
 * written by the epilogue of the tcgen05 kernel with plain peer stores, whole 128-byte lines of a row per store instruction, as
 * each 128 x 256 tile finishes: the rows cross NVLink while the tensor cores work on the next tile, and the local
 * result buffer of the two-call form does not exist. Rank `my_rank` walks the row tiles of every expert starting
 * my_rank / world of the way in (the same reason as the rotation of smoe_ep_return). Tensor-core kernel only:
 * returns SMOE_ERR_UNSUPPORTED (nothing launched, no error text) when the request does not fit it (dtype, alignment);
 * the caller then runs smoe_scatter2scatter and smoe_ep_return. */
int smoe_scatter2scatter_to_peers(const void* X, int64_t x_rows, int64_t stride_xm, int64_t stride_xk,
                                  const void* W, int64_t stride_we, int64_t stride_wk, int64_t stride_wn,
                                  const int64_t* expert_offsets, const int64_t* return_addr,
                                  void* const* peer_slot_bufs, int64_t peer_stride_rows, int64_t peer_rows,
                                  int32_t world, int32_t my_rank, int32_t K, int32_t N, int32_t E, int32_t dtype,
                                  int32_t flags, int32_t* status, void* stream);
/* ---- the same exchange with every token row crossing NVLink once per owning rank (no counterpart in the reference) ----
 * A token whose k slots fall on n distinct ranks is sent n times instead of k times, and n rows come back. The caller
 * lists the distinct (token, rank) pairs in rank order (a counting sort of each token's first slot per rank) and
 * pushes the token rows with smoe_ep_dispatch over that list (E = world). The calls below carry the rest:
 *
 * smoe_ep_plan_tokens: for pair i (rank w = pair_rank[i], token t = pair_slot[i] / k), whose row lands at
 *     row(t, w) = tok_base[w] + (i - first pair of w) of owner w's token buffer: tok_row[t, w] = row(t, w),
 *     tok_parts[t] = number of owners of t, and into owner w's record buffer (smoe_ep_tokmeta_ints(k) int32 per row):
 *     [this rank, return row t*min(k,world) + ordinal of w among t's owners, n slots, 0, position[k], gate bits[k]]
 *     where position = place of each of t's slots at w in w's expert-grouped slot buffer (as in smoe_ep_dispatch) and
 *     slot_pos[s] = position of slot s in this rank's expert-sorted list.
 * smoe_ep_dispatch_meta: for every position m of the expert-sorted slot list, 16 bytes into the owner's slot record
 *     buffer at the slot's position: [this rank << 40 | slot, row(t, w) | gate bits << 32].
 * smoe_ep_expand (owner): out[p, :] = tok_rows[row(p), :] (* gate(p) if scale_by_gate) for p < *live_slots; with y_rows
 *     also peer_dgate[rank(p)][slot(p)] = <y_rows[p, :], tok_rows[row(p), :]> as fp32 (the gate gradient).
 * smoe_ep_combine (owner): for every received token row u < *live_tok with record [src, ret, n, -, pos[], gate[]]:
 *     peer_comb[src][ret, :] = sum_i (gate[i] if use_gates else 1) * rows[pos[i], :]. src_base (world + 1, nullable):
 *     first token row of each sending rank, used to start with the next rank's rows.
 * smoe_ep_sum_parts (token owner): out[t, :] = sum over c < parts[t] of comb[t*kw + c, :].
 * 16-bit dtypes, row widths multiples of 8, k <= 16. */
int32_t smoe_ep_tokmeta_ints(int32_t k);
int smoe_ep_plan_tokens(const int64_t* expert_idxs, const void* gates, int64_t T, int32_t k, const int64_t* pair_rank,
                        const int64_t* pair_slot, const int64_t* pair_offsets, const int64_t* tok_base,
                        const int64_t* slot_pos, const int64_t* expert_offsets, const int64_t* dst_offsets,
                        int32_t* tok_row, int32_t* tok_parts, void* const* peer_tokmeta, int64_t cap_tok,
                        int64_t cap_slots, int32_t my_rank, int32_t E, int32_t world, int32_t dtype, void* stream);
int smoe_ep_dispatch_meta(const int64_t* sorted_expert_idxs, const int64_t* sorted_scattered_idxs,
                          const int64_t* expert_offsets, const int64_t* dst_offsets, const void* gates,
                          const int32_t* tok_row, int32_t k, void* const* peer_meta, int64_t cap_slots, int32_t my_rank,
                          int64_t R, int32_t E, int32_t world, int32_t dtype, void* stream);
int smoe_ep_expand(const void* tok_rows, int64_t stride_tok, int64_t cap_tok, const void* meta, const int64_t* live_slots,
                   int64_t cap_slots, int32_t scale_by_gate, void* out, int64_t stride_out, const void* y_rows,
                   int64_t stride_y, void* const* peer_dgate, int64_t peer_slots, int32_t K, int32_t world, int32_t dtype,
                   void* stream);
int smoe_ep_combine(const void* rows, int64_t stride_rows, int64_t cap_slots, const int32_t* tokmeta,
                    const int64_t* live_tok, int64_t cap_tok, const int64_t* src_base, int32_t use_gates,
                    void* const* peer_comb, int64_t peer_stride, int64_t peer_rows, int32_t K, int32_t k, int32_t my_rank,
                    int32_t world, int32_t dtype, void* stream);
int smoe_ep_sum_parts(const void* comb, int64_t stride_comb, const int32_t* parts, int32_t kw, void* out,
                      int64_t stride_out, int64_t T, int32_t K, int32_t dtype, void* stream);

/* Stream-ordered barrier across the ranks through peer memory: `peer_flags[w]` is rank w's int32[world] flag array
 * (zeroed once, before the first barrier, with the ranks synchronised by other means). Call with epoch = 1, 2, 3,
 * ... in the same order on every rank. Work enqueued after it on a rank runs after everything every rank
 * enqueued before its own call with the same epoch, including its peer stores. The wait inside is bounded
 * (`limit_cycles` SM clocks, 0 = about one second): on expiry `status` gets (2, 100, silent rank, epoch) and the kernel
 * returns; the work enqueued after it then runs on rows that may not have arrived. */
int smoe_ep_barrier(void* const* peer_flags, int32_t my_rank, int32_t world, int32_t epoch, int64_t limit_cycles,
                    int32_t* status, void* stream);
/* Makes an expired wait loud: if status[0] != 0 when the kernel runs, `buf` (bytes) is filled with 0xFF bytes, which
 * read as NaN in fp32 / bf16 / fp16; otherwise nothing is written. Enqueue it on the results of a step after the
 * step's last barrier. */
int smoe_status_poison(const int32_t* status, void* buf, int64_t bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SCATTERMOE_B200_H */
