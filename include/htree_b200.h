/*
 * htree_b200 — C ABI of the sm_100a implementation of htree hierarchical tree sparse attention.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle; no entry point below allocates
 * memory or keeps state between calls, work is enqueued asynchronously on `stream` of the current device, and any
 * host thread may call.  Return value: 0 on success, a negative HTREE_E_* code when an argument is rejected before
 * anything is launched, or a positive cudaError_t reported by a launch.  htree_b200_error_string() explains both.
 *
 * Tensor layouts are the reference's (skywong14/htree, src/parallel.py:874-905):
 *     q   [B, T, H,    K]      k  [B, T, H_kv, K]      v  [B, T, H_kv, V]      out [B, T, H, V]
 * all contiguous, all of one storage type `dtype`.  Tree level l (l = 0 are the leaves k, v themselves) holds
 *     layers_k[l] [B, N_l, H_kv, K],  layers_v[l] [B, N_l, H_kv, V],   N_0 = T, N_{l+1} = ceil(N_l / CR)
 * and pooling stops at the first level with N_l <= max_top_nodes (src/parallel.py:941-945).
 */
#ifndef HTREE_B200_H
#define HTREE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HTREE_B200_VERSION 3
#define HTREE_MAX_LEVELS 12

/* storage types */
#define HTREE_F32 0
#define HTREE_BF16 1
#define HTREE_F16 2

/* error codes (negative) */
#define HTREE_E_NULL (-1)        /* a required pointer is NULL */
#define HTREE_E_SHAPE (-2)       /* a size is non-positive, H % H_kv != 0, or K is odd */
#define HTREE_E_DTYPE (-3)       /* unknown storage type */
#define HTREE_E_LEVELS (-4)      /* more than HTREE_MAX_LEVELS levels, or level sizes inconsistent with T, CR */
#define HTREE_E_TOPLEVEL (-5)    /* top level longer than top_k * compression_rate */
#define HTREE_E_ROPE (-6)        /* cos/sin tables shorter than top_k * compression_rate rows */
#define HTREE_E_ALIGN (-7)       /* a pointer or row size breaks the 16-byte alignment the kernels need */
#define HTREE_E_UNSUPPORTED (-8) /* shape outside what the kernels were built for (e.g. shared memory need) */
#define HTREE_E_NODEVICE (-9)    /* no CUDA device / wrong architecture */
#define HTREE_E_WINDOW (-10)     /* query window outside the sequence, or a backward window without the window flags */
#define HTREE_E_SCRATCH (-11)    /* pooled-level accumulators exceed the library's built-in scratch array */

/* forward flags */
#define HTREE_FWD_SELECT_ONLY 1u /* rebuild the selections only: no V reads, no accumulation, out/gmax/gsum untouched */
#define HTREE_FWD_GENERIC 2u     /* force the dtype-generic fp32-arithmetic kernel even where a tensor-core kernel exists
                                    (also honoured by the backward) */
#define HTREE_FWD_TILED 8u       /* generic forward: use the tiled variant (scores not held for a whole level) even when the
                                    untiled one fits into shared memory; it is chosen automatically when it does not */
#define HTREE_PARENTS_U16 16u     /* forward and backward: the parent-list buffers hold uint16 node ids (0xFFFF = none) instead of
                                    int32 (-1 = none): half the saved-selection memory.  Needs every pooled level to have at
                                    most 65535 nodes (else HTREE_E_UNSUPPORTED).  The reference keeps int32
                                    (src/parallel.py:1044; docs/backward_derivation.md:355-372 names the cost). */
#define HTREE_FWD_NO_PIPELINE 128u /* tensor-core forward: gather operands into registers instead of streaming the blocked
                                    keys / values through shared memory (the kernels used where no blocked keys are given) */
#define HTREE_FWD_FUSED 4u       /* tensor-core forward: keep selection and accumulation in ONE kernel even when parent
                                    buffers are provided (default then: a selection kernel followed by an accumulation kernel) */

/* backward flags: a backward may be run as several calls over consecutive query windows (HtreeShape.T_q / t_offset) that share
 * the dk_levels / dv_levels accumulators, e.g. to overlap transfers of q, dO, out and dq with the kernels.  The first call
 * passes HTREE_BWD_NO_FOLD, calls in the middle HTREE_BWD_KEEP_ACCUM | HTREE_BWD_NO_FOLD, the last one HTREE_BWD_KEEP_ACCUM;
 * dq (or typed->dq) of every call covers that call's window only, dk / dv are complete after the last call.  Every call
 * of one backward must be given the same level buffers and operand copies (they select the same kernel).
 * No counterpart in the reference (its backward always runs every position, src/backward.py:941-1119). */
#define HTREE_BWD_KEEP_ACCUM 32u /* do not zero-fill dk_levels / dv_levels: they hold the sums of earlier windows */
#define HTREE_BWD_NO_FOLD 64u    /* stop after accumulating: later windows follow, dk / dv are not final yet */

/* Problem description shared by all entry points (mirrors the keyword arguments of htree_forward,
 * src/parallel.py:874-885). */
typedef struct HtreeShape {
    int32_t B, T, H, H_kv, K, V;
    int32_t compression_rate;
    int32_t top_k;          /* top_k_per_layer */
    int32_t max_top_nodes;  /* may be smaller than top_k*compression_rate; the reference asserts equality */
    int32_t dtype;          /* HTREE_F32 / HTREE_BF16 / HTREE_F16 */
    /* Query window (sequence-sharded forward calls, windowed forward / backward of the host-buffer pipeline): the call
     * computes query positions t_offset .. t_offset + T_q - 1 of the sequence, q/out/dO/dq are [B,T_q,H,*], gmax/gsum
     * [B,T_q,H] and parents [B,T_q,H_kv,top_k], while the tree levels (and dk_levels/dv_levels) still cover all T
     * positions.  T_q = 0 means the whole sequence (T_q = T, t_offset = 0).  The backward accepts a window only together
     * with HTREE_BWD_KEEP_ACCUM / HTREE_BWD_NO_FOLD.  The reference has no counterpart (it always runs every position). */
    int32_t T_q;
    int32_t t_offset;
} HtreeShape;

/* Optional per-level accumulator dump, the reference's LayerTrace (src/naive.py:13-19; filled by the harness in
 * correctness_test.py:168-347).  Arrays are indexed [level][...]: layer_max/layer_sum [L][B,T,H] fp32,
 * layer_out [L][B,T,H,V] fp32 (un-normalised).  Any pointer may be NULL. */
typedef struct HtreeTrace {
    float* layer_max;
    float* layer_sum;
    float* layer_out;
} HtreeTrace;

/* Optional gradient outputs in the storage type (`dtype` of the shape) for htree_b200_backward: dq [B,T,H,K],
 * dk [B,T,H_kv,K], dv [B,T,H_kv,V], 16-byte aligned.  The reference returns fp32 gradients and its autograd function
 * casts them afterwards (src/backward.py:1119, 1193); with this struct the cast is fused into the kernels that produce
 * the values and no fp32 dq tensor exists at all. */
typedef struct HtreeTypedGrads {
    void* dq;
    void* dk;
    void* dv;
} HtreeTypedGrads;

int htree_b200_version(void);
const char* htree_b200_error_string(int code);

/* Diagnostic: number of kernels this library has launched in the calling process so far (all threads, all devices).
 * No counterpart in the reference. */
uint64_t htree_b200_launch_count(void);

/* Number of tree levels for a sequence length, and their lengths N_l (level loop of src/parallel.py:941-945).
 * htree_b200_level_sizes writes at most `cap` entries and returns the level count (or HTREE_E_LEVELS). */
int htree_b200_num_levels(int32_t T, int32_t compression_rate, int32_t max_top_nodes);
int htree_b200_level_sizes(int32_t T, int32_t compression_rate, int32_t max_top_nodes, int32_t* sizes, int32_t cap);

/* Mean-pool tree build: replaces htree_build_kernel and its per-level launch loop (src/parallel.py:87-181, 955-976)
 * and _recompute_tree_build (src/backward.py:848-878).  layers_k[0]/layers_v[0] are the inputs k, v; levels
 * 1..L-1 are written (tail parents average only their valid children; fp32 accumulation, one rounding).
 *   layers_k_rot  NULL, or L pointers to buffers shaped like layers_k (level 0 included) that receive
 *                 K'[node] = R(node % compression_rate) K[node], the keys rotated by their child index with the
 *                 half-split RoPE of src/parallel.py:687-692, stored as IEEE half for bf16 and fp16 inputs alike
 *                 (clamped to the finite half range).  The column order inside a K' row is private to the library
 *                 (rows of 64 columns interleave 8-column pieces of the two halves).  The tensor-core forward reads K' (16-bit storage
 *                 types only; needs cos_cache/sin_cache with at least compression_rate rows, and K % 16 == 0).
 *                 Pass NULL for fp32 or when only the generic kernels are wanted.
 *   layers_k_blk  NULL, or (bf16/fp16, K = 128, compression_rate 16 only; needs layers_k_rot) L pointers to buffers of
 *                 B * ceil(N_l / 16) * H_kv * 16 * K halves (32-byte aligned) that receive K' grouped by parent in the order
 *                 in which the pipelined tensor-core forward consumes it: with them that forward streams whole parent blocks
 *                 into shared memory with asynchronous bulk copies instead of gathering rows into registers.
 *   layers_v_blk  NULL, or L pointers to buffers of B * ceil(N_l / compression_rate) * H_kv * compression_rate * V
 *                 elements of `dtype` (level 0 included; 32-byte aligned) that receive the values of every level grouped by
 *                 parent: the compression_rate children of one parent and KV head form one block whose element order is
 *                 private to the library (the order in which the lanes of the tensor-core forward consume them); rows
 *                 past the end of a level are zero.  The tensor-core forward accumulates from these blocks instead of
 *                 gathering value rows.  16-bit storage types, V in {64,128}, compression_rate 8 or 16 only. */
int htree_b200_build_tree(const HtreeShape* shape, void* const* layers_k, void* const* layers_v,
                          void* const* layers_k_rot, void* const* layers_k_blk, void* const* layers_v_blk,
                          const float* cos_cache, const float* sin_cache, void* stream);

/* K' levels alone, from tree levels that already exist (e.g. levels assembled by an all-gather in sequence-sharded
 * runs): layers_k_rot[l][node] = R(node % compression_rate) layers_k[l][node] for every level.  16-bit storage types
 * only.  Same arithmetic as the rotation inside htree_b200_build_tree; no counterpart in the reference. */
int htree_b200_rotate_keys(const HtreeShape* shape, void* const* layers_k, void* const* layers_k_rot,
                           const float* cos_cache, const float* sin_cache, void* stream);

/* The blocked values / blocked keys alone (layers_v_blk, layers_k_blk of htree_b200_build_tree), from tree levels and K' levels
 * that already exist.  No counterpart in the reference. */
int htree_b200_block_values(const HtreeShape* shape, void* const* layers_v, void* const* layers_v_blk, void* stream);
int htree_b200_block_keys(const HtreeShape* shape, void* const* layers_k_rot, void* const* layers_k_blk, void* stream);

/* Fused forward over all levels: replaces the per-level launches of htree_select_accumulate_gqa_kernel,
 * htree_bottom_accumulate_gqa_kernel, htree_merge_to_global_kernel and htree_final_normalize_kernel together with
 * the host-side state and virtual-parent initialisation (src/parallel.py:995-1134), and — with
 * HTREE_FWD_SELECT_ONLY — htree_recompute_selection_kernel / _recompute_parents (src/parallel.py:1167-1399,
 * src/backward.py:881-934).
 *   layers_k_blk  NULL or the blocked keys of htree_b200_build_tree: selects the pipelined variant of the tensor-core kernels
 *                 (status bit 16 reports a bulk copy that did not complete within the kernels' bounded waits)
 *   layers_k_rot, layers_v_blk  NULL or the K' levels and blocked values written by htree_b200_build_tree; when present
 *                 (and the shape qualifies: bf16/fp16, K == V in {64,128}, H/H_kv <= 16, compression_rate 16 or 8, and q,
 *                 every level of layers_k_rot / layers_v_blk and the tables 32-byte aligned; the backward also wants
 *                 layers_v, out and dO so) the tensor-core kernel runs, otherwise the generic fp32-arithmetic kernel
 *                 (16-byte alignment).  With HTREE_FWD_SELECT_ONLY layers_v_blk is not read and may be NULL.
 *   cos_cache, sin_cache  [n_pos, K/2] fp32 RoPE tables (src/parallel.py:983-988); n_pos >= top_k*compression_rate
 *   cos_half, sin_half    NULL, or [n_pos, K/2] IEEE half tables holding cos*scale and sin*scale: the tensor-core
 *                         kernels then rotate queries with packed half arithmetic where that does not touch the
 *                         Top-K decision (accumulation passes, backward); without them everything rotates in fp32
 *   out [B,T,H,V] in `dtype`; gmax, gsum [B,T,H] fp32 (global_max / global_sum of bwd_ctx)
 *   parents  NULL, or L pointers: parents[l] [B,T,H_kv,top_k] int32 receives the parent list CONSUMED at level l,
 *            ascending and -1 padded (per_layer_parents of bwd_ctx, src/parallel.py:1039-1044)
 *   trace    NULL or per-level accumulator dumps
 *   status   NULL or one int32 on the device, OR-ed with a non-zero code if a kernel met an out-of-range node index
 */
int htree_b200_forward(const HtreeShape* shape, const void* q, void* const* layers_k, void* const* layers_v,
                       void* const* layers_k_rot, void* const* layers_k_blk, void* const* layers_v_blk, const float* cos_cache,
                       const float* sin_cache, const void* cos_half,
                       const void* sin_half, int32_t n_pos, float scale, void* out,
                       float* gmax, float* gsum, int32_t* const* parents, const HtreeTrace* trace, int32_t* status,
                       uint32_t flags, void* stream);

/* One tree level at a time (the call surface the reference's parity harness uses, correctness_test.py:168-347):
 * htree_b200_level_forward replaces one launch of htree_select_accumulate_gqa_kernel (level > 0; src/parallel.py:537-867)
 * or of htree_bottom_accumulate_gqa_kernel (level 0; src/parallel.py:369-530): given the parent lists consumed at this
 * level it writes the level's accumulator state (layer_max/layer_sum [B,T,H], layer_out [B,T,H,V], fp32) and, above the
 * leaves, the kept nodes (next_parents [B,T,H_kv,top_k], ascending, -1 padded).  layer_k/layer_v are this level's
 * tensors [B,n_level,H_kv,*]; shape->T is the query length, shape->max_top_nodes is ignored.  fp32-arithmetic kernel.
 * htree_b200_merge_to_global / htree_b200_final_normalize replace htree_merge_to_global_kernel and
 * htree_final_normalize_kernel (src/parallel.py:248-363); rows = B*T*H. */
int htree_b200_level_forward(const HtreeShape* shape, int32_t level, int32_t n_level, const void* q, const void* layer_k,
                             const void* layer_v, const int32_t* prev_parents, const float* cos_cache,
                             const float* sin_cache, int32_t n_pos, float scale, float* layer_max, float* layer_sum,
                             float* layer_out, int32_t* next_parents, int32_t* status, void* stream);
int htree_b200_merge_to_global(const float* layer_max, const float* layer_sum, const float* layer_out, float* global_max,
                               float* global_sum, float* global_out, int64_t rows, int32_t V, void* stream);
int htree_b200_final_normalize(const float* global_out, const float* global_sum, void* out, int32_t dtype, int64_t rows,
                               int32_t V, void* stream);

/* Strided copy for callers whose tensors live in host memory (no reference counterpart): `height` rows of `width` bytes,
 * consecutive rows dpitch / spitch bytes apart, direction inferred from the pointers (pinned host memory for an
 * asynchronous copy).  htree_b200.host uses it to move one (batch, KV head) unit of q, k, v, dO and of the results. */
int htree_b200_copy_rows(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height,
                         void* stream);

/* Selector micro-benchmark (no counterpart on the operator path; the experiment of topk_test/benchmark.py:34-46):
 * `batch` independent problems, the k largest of n <= 8192 fp32 values each; pay1 [batch,n] and pay8 [batch,n,8] are
 * optional int32 payloads gathered for the winners.  method 0 = threshold search (the attention kernels' selector),
 * 1 = radix select, 2 = bitonic (n and k powers of two).  Methods 0 and 1 return the winners by ascending index,
 * method 2 by descending value; ties go to the smaller index. */
int htree_b200_topk(const float* values, const int32_t* pay1, const int32_t* pay8, int32_t batch, int32_t n, int32_t k,
                    int32_t method, float* out_val, int32_t* out_idx, int32_t* out_pay1, int32_t* out_pay8, void* stream);

/* Backward: replaces htree_backward and every kernel it launches (preprocess_delta, dq_bottom/upper,
 * build_parent_mask, dkv_bottom/upper, tree_backward; src/backward.py:45-841, 941-1119).
 *   layers_k_rot  NULL or the K' levels of htree_b200_build_tree: selects the tensor-core kernel where the shape
 *                 qualifies (bf16/fp16, K == V in {64,128}, H/H_kv <= 16, compression_rate 16 or 8), else the generic kernel
 *   out, dO [B,T,H,V] in `dtype`; gmax, gsum from the forward; parents[l] as written by the forward (required)
 *   dq [B,T,H,K] fp32 (written)
 *   dk_levels[l] [B,N_l,H_kv,K] fp32, dv_levels[l] [B,N_l,H_kv,V] fp32 for every level: zero-filled by this call,
 *   accumulated, then folded top-down by the mean-pool gradient; level 0 holds dk, dv on return and levels >= 1 are
 *   scratch (the reference's dk_layers / dv_layers, src/backward.py:979-981).
 *   typed  NULL (the reference's contract: fp32 dq, dk, dv as above), or the three outputs in the storage type: dq is
 *          then not written (it may be NULL), dk_levels[0] / dv_levels[0] still have to be provided as fp32
 *          accumulators but hold no result on return, and the finished gradients are rounded once into typed->dq/dk/dv.
 * A shape that no compiled kernel takes is refused with HTREE_E_UNSUPPORTED before anything is queued on the stream.
 */
int htree_b200_backward(const HtreeShape* shape, const void* q, void* const* layers_k, void* const* layers_v,
                        void* const* layers_k_rot, const float* cos_cache, const float* sin_cache, const void* cos_half,
                        const void* sin_half, int32_t n_pos, float scale, const void* out,
                        const void* dO, const float* gmax, const float* gsum, int32_t* const* parents, float* dq,
                        float* const* dk_levels, float* const* dv_levels, const HtreeTypedGrads* typed, int32_t* status,
                        uint32_t flags, void* stream);

/* Backward without caller-provided scratch.  No counterpart in the reference (its backward allocates its level
 * buffers with torch, src/backward.py:979-981); it exists for callers that cannot allocate device memory around
 * the call: a host program that reaches this library through a plain FFI and holds only the tensors its framework
 * passed in, or a process whose device memory is fully reserved by a framework pool, or one that must not take the
 * device-wide synchronisation of an allocation while other streams run.
 *
 * Same arguments and results as htree_b200_backward, except that only the outputs dk [B,T,H_kv,K] and
 * dv [B,T,H_kv,V] (fp32) are passed: the accumulators of the pooled levels live in an array built into the library
 * (htree_b200_static_scratch_bytes() bytes, 16 MiB, present in the memory of every GPU that loads the library until
 * the process exits).  The call allocates nothing and frees nothing.
 *   - Shapes whose pooled levels need more than that, sum over l >= 1 of B*N_l*H_kv*(K+V) floats (each level slice
 *     rounded up to 64 floats), are rejected with HTREE_E_SCRATCH before anything is launched.
 *   - The first call on a device looks up the array's device address (once per device, with that device current);
 *     make that first call outside of any stream capture.  As everywhere in this library, `stream` must belong to the
 *     device that is current in the calling thread: the address is looked up and cached for the current device.
 *   - All calls on one device share the array.  It keeps the previous call's contents; each call clears the part it
 *     uses on its own stream before use.  Two calls that overlap on the GPU (different streams, or threads without
 *     ordering between them) race on it: serialise them. */
size_t htree_b200_static_scratch_bytes(void);
int htree_b200_backward_static_scratch(const HtreeShape* shape, const void* q, void* const* layers_k,
                                       void* const* layers_v, void* const* layers_k_rot, const float* cos_cache,
                                       const float* sin_cache, const void* cos_half, const void* sin_half,
                                       int32_t n_pos, float scale, const void* out,
                                       const void* dO, const float* gmax, const float* gsum, int32_t* const* parents,
                                       float* dq, float* dk, float* dv, int32_t* status, uint32_t flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HTREE_B200_H */
