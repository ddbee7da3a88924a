/*
 * autosage_b200.h — C ABI of libautosage_b200.so (CUDA, sm_100a).
 *
 * The library is the device side of AutoSAGE's sparse hot path: CSR SpMM, CSR SDDMM, CSR row
 * softmax and the fused SDDMM -> softmax -> SpMM attention row kernel.  Every entry point takes
 * plain device pointers and sizes, launches on the stream it is given, never synchronises the
 * device, never allocates device memory and never throws.  Return value: 0 on success, a negative
 * ASG_E* code otherwise; asg_last_error_string() gives the message for the calling thread.
 *
 * Conventions shared by all entry points
 *   crow   int64[n_rows+1]  CSR row pointers (device), crow[0] may be non-zero only if col/val are
 *                           indexed by the same absolute positions
 *   col    int64[nnz]       column indices (device); every value must be < 2^31
 *   val    float32[nnz]     edge weights (device) or NULL for an all-ones matrix
 *   x,q,k,v float32 row-major dense operands with leading dimension f (device)
 *   stream a cudaStream_t passed as void* (NULL = the legacy default stream)
 *   workspace  caller-owned device scratch of at least asg_workspace_bytes(n_rows) bytes, 256-byte
 *              aligned; it holds the degree-binned row order ("plan") and the work counters of the
 *              persistent kernels.  One workspace serves one stream at a time.
 *
 * Reference interfaces replaced (paths inside the AutoSAGE repository):
 *   asg_spmm_csr          csrc/spmm_csr_vec4.cu:97-176   spmm_csr_cuda  (op autosage::spmm_csr,
 *                         csrc/spmm_binding.cpp:31-38)
 *   asg_spmm_csr_split    csrc/launcher_spmm.cu:22-72    spmm_csr_split_cuda (op
 *                         autosage::spmm_csr_split, csrc/spmm_binding.cpp:40-61), including the
 *                         row launchers csrc/spmm_rows.cu:132-157 and csrc/spmm_hub.cu:149-182
 *   asg_plan_build        csrc/launcher_spmm.cu:49-59    the per-call hub/light row split
 *   asg_sddmm_csr         csrc/sddmm_csr_op.cu:108-134   sddmm_csr
 *   asg_sddmm_csr_split   csrc/sddmm_csr_op.cu:136-187   sddmm_csr_split
 *   asg_csr_row_softmax   autosage/_auto.py:744-759      _csr_row_softmax
 *   asg_csr_attention     autosage/_auto.py:762-780      csr_attention_forward's three passes,
 *                         fused into one kernel
 */
#ifndef AUTOSAGE_B200_H_
#define AUTOSAGE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ASG_OK 0
#define ASG_EINVAL (-1)    /* bad argument (message says which) */
#define ASG_ECUDA (-2)     /* a CUDA runtime call or kernel launch failed */
#define ASG_EWORKSPACE (-3) /* workspace missing, misaligned or too small */
#define ASG_ERANGE (-4)    /* a size exceeds what the kernels index (2^31-1 rows / features) */

/* flags for the *_ex entry points */
#define ASG_FLAG_ACCUMULATE 1u /* y += A x instead of y = A x */
#define ASG_FLAG_NO_VEC4 2u    /* force the scalar kernels (AUTOSAGE_VEC4=0 in the reference) */
#define ASG_FLAG_PLAN_READY 4u /* workspace already holds a plan for this crow/threshold */
#define ASG_FLAG_NO_BULK_STAGE 8u /* hub rows: stage col/val with plain loads, not bulk copies */
#define ASG_FLAG_NO_TILE_PASSES 16u /* SDDMM: never split the feature dimension into 64-wide passes */
#define ASG_FLAG_PACK_SHORT_ROWS 32u /* SpMM: rows under 32 edges one per lane group (for very short rows) */
#define ASG_FLAG_SELFTEST_STALL 64u /* self-test of the give-up path: one wait inside the kernel is pointed at a
                                       barrier nothing arrives on, so it runs out (after 20 ms here), the
                                       status word is set and the kernel returns with part of its output
                                       unwritten; nothing faults or hangs.  asg_spmm_csr_ex: the hub staging
                                       wait, status 1.  asg_linear_bias_umma_ex (status 2) and asg_conv_fused
                                       (status 3): the MMA thread's wait before its second tile */

/* Library version: major*10000 + minor*100 + patch. */
int asg_version(void);

/* Message of the last failing call made by this thread ("" if none). */
const char* asg_last_error_string(void);

/* Bytes of workspace needed for a graph with n_rows rows (0 rows -> still a small header). */
size_t asg_workspace_bytes(int64_t n_rows);

/*
 * Degree-bin the rows of a CSR matrix into the workspace: rows with degree >= hub_threshold
 * ("hubs", processed one CTA each) come first, then the light rows (one warp each); inside each
 * class rows are ordered by descending floor(log2(degree)) and, within a bucket, by ascending row
 * id, so the result is deterministic.  hub_threshold <= 0 disables the hub class.
 * Replaces the nonzero()/cast sequence the reference runs on every call
 * (csrc/launcher_spmm.cu:49-59, csrc/sddmm_csr_op.cu:169-171) with three small kernels and no
 * host synchronisation.
 */
int asg_plan_build(const int64_t* crow, int64_t n_rows, int64_t hub_threshold, void* workspace,
                   size_t workspace_bytes, void* stream);

/*
 * Copy the plan out for inspection: order[n_rows] (int32 row ids in processing order) and
 * counts[2] = {n_hub, n_light}.  Both are device pointers; either may be NULL.
 */
int asg_plan_export(const void* workspace, int64_t n_rows, int32_t* order, int32_t* counts,
                    void* stream);

/*
 * y[n_rows, f] = A x.  Plain SpMM (reference op autosage::spmm_csr).  Chooses the feature tile and
 * hub threshold itself.  x must have at least max(col)+1 rows of f floats.
 */
int asg_spmm_csr(const int64_t* crow, const int64_t* col, const float* val, const float* x,
                 float* y, int64_t n_rows, int64_t nnz, int64_t f, void* workspace,
                 size_t workspace_bytes, void* stream);

/*
 * SpMM with the reference's three tuning knobs (op autosage::spmm_csr_split):
 *   feature_tile     64 or 128 (also 32 and 256 through this ABI): features handled per pass
 *   warps_per_block  2, 4, 8 (also 16): warps of each CTA; a hub row is shared by all of them
 *   hub_threshold    rows with degree >= threshold take the CTA-per-hub path (> 0)
 */
int asg_spmm_csr_split(const int64_t* crow, const int64_t* col, const float* val, const float* x,
                       float* y, int64_t n_rows, int64_t nnz, int64_t f, int feature_tile,
                       int warps_per_block, int64_t hub_threshold, void* workspace,
                       size_t workspace_bytes, void* stream);

/* As asg_spmm_csr_split, plus ASG_FLAG_* bits. */
int asg_spmm_csr_ex(const int64_t* crow, const int64_t* col, const float* val, const float* x,
                    float* y, int64_t n_rows, int64_t nnz, int64_t f, int feature_tile,
                    int warps_per_block, int64_t hub_threshold, unsigned flags, void* workspace,
                    size_t workspace_bytes, void* stream);

/*
 * As asg_spmm_csr_ex, but only the output columns [feature_begin, feature_begin + feature_count) are
 * computed (x and y keep their leading dimension f).  The range must start on a feature_tile boundary
 * and end on one or at f.  Used by the sharded path, which multiplies a band of feature columns as
 * soon as that band of every remote shard has arrived.  No counterpart in the reference.
 */
int asg_spmm_csr_range(const int64_t* crow, const int64_t* col, const float* val, const float* x,
                       float* y, int64_t n_rows, int64_t nnz, int64_t f, int64_t feature_begin,
                       int64_t feature_count, int feature_tile, int warps_per_block,
                       int64_t hub_threshold, unsigned flags, void* workspace,
                       size_t workspace_bytes, void* stream);

/* out[nnz]: out[e] = <q[row(e), :], k[col[e], :]>  (reference op autosage::sddmm_csr). */
int asg_sddmm_csr(const int64_t* crow, const int64_t* col, const float* q, const float* k,
                  float* out, int64_t n_rows, int64_t nnz, int64_t f, void* workspace,
                  size_t workspace_bytes, void* stream);

/* SDDMM with the reference's two knobs (op autosage::sddmm_csr_split). */
int asg_sddmm_csr_split(const int64_t* crow, const int64_t* col, const float* q, const float* k,
                        float* out, int64_t n_rows, int64_t nnz, int64_t f, int warps_per_block,
                        int64_t hub_threshold, void* workspace, size_t workspace_bytes,
                        void* stream);

/* As asg_sddmm_csr_split, plus ASG_FLAG_* bits (ACCUMULATE is not accepted). */
int asg_sddmm_csr_ex(const int64_t* crow, const int64_t* col, const float* q, const float* k,
                     float* out, int64_t n_rows, int64_t nnz, int64_t f, int warps_per_block,
                     int64_t hub_threshold, unsigned flags, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * probs[nnz] = softmax over each CSR row segment of scores[nnz]
 * (exp(s - rowmax) / sum exp(s - rowmax)); empty rows write nothing.  scores and probs may alias.
 */
int asg_csr_row_softmax(const int64_t* crow, const float* scores, float* probs, int64_t n_rows,
                        int64_t nnz, int warps_per_block, int64_t hub_threshold, unsigned flags,
                        void* workspace, size_t workspace_bytes, void* stream);

/*
 * out[n_rows, f] = softmax_row(scale * (q k^T restricted to the CSR pattern)) v, computed in one
 * pass with a running maximum and running sum per row, so scores and probabilities never reach
 * memory.  Rows without edges produce zeros.  scale = 1.0 reproduces the reference pipeline.
 */
/*
 * Workspace size with which asg_csr_attention also splits very long rows (4,096 edges or more) into
 * 1,024-edge segments that different CTAs process and the last one merges: asg_workspace_bytes(n_rows)
 * plus about 1 MB.  A workspace of only asg_workspace_bytes(n_rows) still works; such rows then stay
 * with one CTA each.
 */
size_t asg_attention_workspace_bytes(int64_t n_rows);

int asg_csr_attention(const int64_t* crow, const int64_t* col, const float* q, const float* k,
                      const float* v, float* out, int64_t n_rows, int64_t nnz, int64_t f,
                      float scale, int warps_per_block, int64_t hub_threshold, unsigned flags,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * out[rows, cols] += bias[cols] in place: the bias step of the layer's nn.Linear
 * (autosage/conv.py:55), issued after a plain matrix product.
 */
int asg_add_row_bias(float* out, const float* bias, int64_t rows, int64_t cols, void* stream);

/*
 * COO -> CSR on the device, rows keyed by row_of_edge, edges of one row in their input order:
 *   crow[r]  = number of edges with row id below r              (r = 0 .. n_rows; int64[n_rows + 1])
 *   perm     = the stable ordering of the edges by row id        (int64[n_edges]; may be null)
 *   col[i]   = col_of_edge[perm[i]]                              (int64[n_edges])
 *   val_out[i] = val_in[perm[i]]                                 (float32[n_edges]; both may be null)
 * Replaces edge_index_to_csr (autosage/utils/csr.py:6-26: stable argsort + bincount + cumsum + gather)
 * and the second argsort by which AutoSAGEConv.forward permutes edge weights (autosage/conv.py:44-45).
 * Row ids must lie in [0, n_rows); n_edges and n_rows below 2^31.  The workspace holds
 * asg_csr_build_workspace_bytes(n_edges, n_rows) bytes (about 16 bytes per edge), 256-byte aligned.
 */
size_t asg_csr_build_workspace_bytes(int64_t n_edges, int64_t n_rows);
int asg_csr_from_edges(const int64_t* row_of_edge, const int64_t* col_of_edge, const float* val_in,
                       int64_t n_edges, int64_t n_rows, int64_t* crow, int64_t* col, int64_t* perm,
                       float* val_out, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Row sample for the scheduler's probe: the rows listed in rows[n_sampled_rows] (device, int64,
 * ascending) are cut out of the CSR with every one of their edges and their column ids unchanged:
 *   out_crow[n_sampled_rows + 1]  row pointers of the sample
 *   out_col / out_val[capacity]   the rows' column and weight segments, one after the other
 *   kept[2]                       {rows kept, edges kept}: if the sampled rows hold more than `capacity`
 *                                 edges, only the leading rows that fit are copied and the remaining row
 *                                 pointers repeat the last value (empty rows), so the arrays are always a
 *                                 valid CSR of n_sampled_rows rows
 * Three small kernels and one device-wide scan, no host synchronisation; the caller reads kept[] when it
 * next synchronises.  Replaces the ATen sequence (and its .item() synchronisation) with which the
 * reference builds its probe sample, autosage/_auto.py:95-154.  The workspace holds
 * asg_row_sample_workspace_bytes(n_sampled_rows) bytes, 256-byte aligned.
 */
size_t asg_row_sample_workspace_bytes(int64_t n_sampled_rows);
int asg_csr_row_sample(const int64_t* crow, const int64_t* col, const float* val, const int64_t* rows,
                       int64_t n_sampled_rows, int64_t capacity, int64_t* out_crow, int64_t* out_col,
                       float* out_val, int64_t* kept, void* workspace, size_t workspace_bytes, void* stream);

/*
 * out[rows, out_features] = x[rows, in_features] @ weight[out_features, in_features]^T + bias:
 * the layer's nn.Linear (autosage/conv.py:55) at float32 accuracy on the tensor cores (each float32
 * operand is split into three bfloat16 pieces, the piece products are summed in float32; no TF32
 * rounding of the inputs).  bias may be null.  in_features and out_features must be multiples
 * of 4 and all pointers 16-byte aligned; x, weight and out are dense row-major.
 */
int asg_linear_bias(const float* x, const float* weight, const float* bias, float* out, int64_t rows,
                    int64_t in_features, int64_t out_features, void* stream);
/* 1 when asg_linear_bias is usable, 0 when the library was built without a CUTLASS header tree (the
 * entry point then returns ASG_EINVAL; asg_linear_bias_umma is unaffected). */
int asg_linear_available(void);

/*
 * The same product as asg_linear_bias from the hand-written tcgen05 kernel (csrc/asg_linear_umma.cu):
 * persistent CTAs, x split into bfloat16 pieces on the fly, the weight split once per call into the
 * workspace, accumulators in tensor memory, bias in the epilogue.  Replaces the nn.Linear call of
 * autosage/conv.py:55 for the sizes asg_linear_supported() accepts: in_features a multiple of 64,
 * out_features a multiple of 32 up to 256.  x and out 16-byte aligned, dense row-major.
 * The workspace holds asg_linear_workspace_bytes(in_features, out_features) bytes, 256-byte aligned; its
 * first 256 bytes are a header whose status word asg_workspace_status() reads (non-zero: a bounded wait
 * inside the kernel gave up and the output is invalid).
 */
size_t asg_linear_workspace_bytes(int64_t in_features, int64_t out_features);
int asg_linear_supported(int64_t in_features, int64_t out_features);
int asg_linear_bias_umma(const float* x, const float* weight, const float* bias, float* out, int64_t rows,
                         int64_t in_features, int64_t out_features, void* workspace, size_t workspace_bytes,
                         void* stream);
/* As asg_linear_bias_umma, plus ASG_FLAG_SELFTEST_STALL (the MMA thread's wait before its second tile
 * runs out after 20 ms: status 2, part of the output unwritten, nothing faults or hangs). */
int asg_linear_bias_umma_ex(const float* x, const float* weight, const float* bias, float* out, int64_t rows,
                            int64_t in_features, int64_t out_features, unsigned flags, void* workspace,
                            size_t workspace_bytes, void* stream);

/*
 * out[n_rows, out_features] = (A x) @ weight^T + bias, the whole forward of the reference layer
 * (autosage/conv.py:54-55: spmm_csr, then nn.Linear), with the aggregated rows kept on chip
 * (csrc/asg_conv_fused.cu).  Rows of hub_threshold edges or more are aggregated by a first launch (the
 * CTA-per-hub path, hub_warps warps per CTA) into a side buffer in the workspace; a second, persistent
 * kernel aggregates every other row of a 128-row tile in registers, writes it as bfloat16 pieces into
 * shared memory, multiplies the tile with the weight on the tensor cores (tcgen05, accumulators in tensor
 * memory, float32 accuracy as asg_linear_bias_umma) and writes only the output.
 * Accepted by asg_conv_fused_supported(): in_features 64 or 128, out_features a multiple of 32 up to 256.
 * x and out 32-byte aligned, dense row-major; val and bias may be null.  flags: ASG_FLAG_PLAN_READY (the
 * plan workspace already holds the plan of crow for hub_threshold), ASG_FLAG_NO_BULK_STAGE,
 * ASG_FLAG_SELFTEST_STALL.
 * plan_workspace: asg_workspace_bytes(n_rows) bytes; workspace:
 * asg_conv_fused_workspace_bytes(n_rows, nnz, in_features, out_features, hub_threshold) bytes, 256-byte
 * aligned, whose status word asg_workspace_status() reads (non-zero: a bounded wait gave up, the output
 * is invalid).  The workspace is sized for the worst case, min(n_rows, nnz / hub_threshold) hub rows of
 * in_features floats (the number of hub rows is known on the device only); only the rows that exist are
 * touched.  The reference has no counterpart: it runs the two steps as separate PyTorch calls.
 */
int asg_conv_fused_supported(int64_t in_features, int64_t out_features);
size_t asg_conv_fused_workspace_bytes(int64_t n_rows, int64_t nnz, int64_t in_features, int64_t out_features,
                                      int64_t hub_threshold);
int asg_conv_fused(const int64_t* crow, const int64_t* col, const float* val, const float* x, const float* weight,
                   const float* bias, float* out, int64_t n_rows, int64_t nnz, int64_t in_features,
                   int64_t out_features, int64_t hub_threshold, int hub_warps, unsigned flags, void* plan_workspace,
                   size_t plan_workspace_bytes, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Pitched device-to-device copy of `height` rows of `width_bytes` bytes (cudaMemcpy2DAsync; runs on
 * the copy engines).  Either pointer may be peer-mapped memory of another GPU.
 */
int asg_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                size_t height, void* stream);

/*
 * Stores `bytes` bytes of src into each of destinations[0 .. n_destinations) (host array of device
 * pointers, at most 7; peer-mapped memory of other GPUs is what it is meant for) from n_ctas CTAs
 * (<= 0: 32) with plain 128-bit stores, reading src once.  src and every destination 16-byte aligned,
 * bytes a multiple of 16.  The sharded path's SM-driven alternative to pulling shards with the copy
 * engines.  No counterpart in the reference (single-GPU).
 */
int asg_push_to_peers(const void* src, void* const* destinations, int n_destinations, size_t bytes, int n_ctas,
                      void* stream);

/*
 * Status word written by kernels whose bounded waits gave up (0 = none).  The word lives in the
 * workspace header; this reads it back asynchronously into *host_status (pinned or pageable host
 * memory) on the given stream.  Non-zero means the output of the launch that set it is invalid.
 */
int asg_workspace_status(const void* workspace, int32_t* host_status, void* stream);

/*
 * SpMM that allocates nothing (no counterpart in the reference, whose operators always allocate
 * through ATen).  Same arguments and results as asg_spmm_csr_split, minus the workspace: the
 * scratch (row order of the plan, work counters) is a fixed array built into the library's device
 * image, about 4.4 MB on every GPU that loads the library, kept until the process exits.
 *
 * Meant for callers that cannot obtain device memory where they call from - a host whose
 * allocator is frozen after start-up, a callback of another runtime in which cudaMalloc is
 * forbidden or would stall the device, a language binding without a device allocator.
 *
 *   - n_rows may be at most asg_static_max_rows() (1,048,576); larger graphs are rejected with
 *     ASG_ERANGE and a message naming the limit.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current); make that first call before starting any stream capture.  It is
 *     also the moment at which the CUDA runtime (lazy module loading, its default) places the
 *     library's code and this array on that GPU: the driver allocates device memory then and may
 *     synchronise the device.  Make the first call per GPU - a one-row SpMM will do - while the
 *     host is still starting up; every later call allocates nothing.
 *   - All calls on a device share the one array and each call rebuilds its contents from scratch,
 *     so nothing needs clearing between calls - but two calls that overlap on the GPU (different
 *     streams, or different host threads) race on it.  Issue them on one stream, or serialise them.
 *   - No cudaMalloc, cudaFree or other allocating routine is called.
 */
int asg_spmm_csr_split_noalloc(const int64_t* crow, const int64_t* col, const float* val,
                               const float* x, float* y, int64_t n_rows, int64_t nnz, int64_t f,
                               int feature_tile, int warps_per_block, int64_t hub_threshold,
                               void* stream);

/* Largest n_rows asg_spmm_csr_split_noalloc accepts. */
int64_t asg_static_max_rows(void);

/*
 * asg_workspace_status for the built-in scratch of asg_spmm_csr_split_noalloc: reads the status word of
 * the array on the GPU that owns device_pointer (null: the current GPU) into *host_status,
 * asynchronously on the given stream.  Non-zero: a bounded wait inside the last call's kernel gave up
 * and its output is invalid.  No counterpart in the reference.
 */
int asg_static_status(const void* device_pointer, int32_t* host_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AUTOSAGE_B200_H_ */
