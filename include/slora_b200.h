/*
 * slora_b200 -- C ABI of the B200 (sm_100a) multi-adapter LoRA shrink/expand library.
 *
 * Every pointer named "device" is a CUDA device pointer borrowed for the duration of the call; the library
 * never takes ownership and never allocates.  All calls are asynchronous on the given stream (a cudaStream_t
 * passed as void*; NULL is the legacy default stream) and return an int status: 0 on success, a negative
 * SLORA_ERR_* code otherwise, with a human-readable message available from slora_last_error().
 * No call aborts, traps or synchronises the device, except where stated.
 *
 * Table vocabulary (the reference's InferAdapter tables, slora/server/router/model_infer/infer_adapter.py:11-39):
 *   start[a]   offset of adapter a's first entry in loc            (a_start, int64)
 *   ranks4[a]  4 * slot_rows of adapter a                          (a_len,   int64; slot_rows == LoRA rank r)
 *   loc[i]     pool row index                                      (a_loc,   int64)
 *   ids[t]     adapter slot of token t                             (req_bins / batch_req_bins, int64)
 *   scales[a]  alpha / r, same dtype as the activations            (a_scaling)
 * Projection p in {0,1,2,3} = {q,k,v,o} owns the slot  loc[start[a] + slot_rows*p .. + slot_rows).
 * Pool buffers are [pool_rows, pool_stride] elements (key_buffer[l] holds A rows, value_buffer[l] holds B rows,
 * slora/common/mem_allocator.py:229-234).
 *
 * Layout inside a slot: the slot's rows concatenated form a flat array; A is [slot_rows, h_in] row-major in it
 * and B is [h_out, slot_rows*rank_mult] row-major in it.  With pool_stride == h_in (A) / == h_out (B) and
 * rank_mult == 1 this is bit-for-bit the layout the reference kernels read
 * (slora/csrc/bgmv/bgmv_impl.cuh:34-38 and :174-179,191); other strides serve GQA and tensor-parallel shards.
 */
#ifndef SLORA_B200_H_
#define SLORA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SLORA_OK 0
#define SLORA_ERR_NULL (-1)      /* required pointer is NULL */
#define SLORA_ERR_ALIGN (-2)     /* pointer or stride not 16-byte aligned where vector access needs it */
#define SLORA_ERR_DTYPE (-3)     /* dtype is neither SLORA_F16 nor SLORA_BF16 */
#define SLORA_ERR_SHAPE (-4)     /* a feature size is not a positive multiple of 8, or a size is out of range */
#define SLORA_ERR_QKVO (-5)      /* projection index outside 0..3 */
#define SLORA_ERR_WORKSPACE (-6) /* plan workspace too small or not a plan */
#define SLORA_ERR_LAUNCH (-7)    /* CUDA reported an error at launch; message holds cudaGetErrorString */
#define SLORA_ERR_RANK (-8)      /* rank not supported by the expand path (needs 8,16,32,64 or 128) */
#define SLORA_ERR_TABLE (-9)     /* slora_validate_tables found an out-of-range entry */

#define SLORA_F16 0
#define SLORA_BF16 1

/* flags */
#define SLORA_FLAG_PDL 1u /* launch with programmatic dependent launch: the kernel may start while the previous
                             kernel on the stream drains, and prefetches adapter rows before it waits for that
                             kernel.  Safe whenever the previous kernels on the stream do not write the pool
                             buffers or the tables that this call reads. */

#define SLORA_FLAG_BIG_GROUPS 2u /* planned calls (slora_batch_lora_*, slora_lora_*_multi with a plan): some adapter
                                   has 128 or more tokens in the batch (slora_plan_big_tiles > 0, or the caller's
                                   scheduler knows): such groups are computed on the tensor cores (tcgen05) in
                                   tiles of 128 tokens by a second launch, the rest stays on the CUDA-core kernels.
                                   Without the flag everything stays on the CUDA-core kernels.  Results of the two
                                   paths differ in summation order and in the expand's rounding (the tensor-core
                                   path rounds scale * sum to the I/O type and adds it to y in that type, as the
                                   reference's kernels do). */

#define SLORA_FLAG_EXACT_ITEMS 4u /* planned calls: count each tile's work items from its adapter's rank instead of
                                    enumerating, per tile, the slots of the widest rank and skipping the empty ones.
                                    A hint about speed, never about results: worth setting when the batch's adapters
                                    differ in rank, or are all narrower than the delta buffers (slora_plan_info tells)
                                    - the CTAs' shares are then equal (measured: 15 % less time per layer on a
                                    rank-16/32/64 mix, 30 % on a rank-8..64 mix); with one rank that fills the delta
                                    buffers the plain enumeration is exact already and starts a few hundred
                                    nanoseconds sooner. */
#define SLORA_FLAG_ONLY_BIG 16u /* with SLORA_FLAG_BIG_GROUPS on a planned call: EVERY group of the plan is a big
                                  group that the tensor-core kernels serve (slora_plan_header: no small tiles, every big
                                  group's rank a power of two that divides pool_stride and fits the delta buffers), so
                                  the call's CUDA-core launch would find nothing and is left out. */
/* The plan was built by slora_plan_build_ex with this max_rank (resolved tiles: token ids, scale and pool rows of
 * every tile at an address that follows from the tile index, so a launch fetches them in one round trip instead of
 * chasing perm and the loc table).  Passing the flag for a plan built without them, or with another max_rank, is
 * harmless when the workspace is at least slora_plan_workspace_bytes_ex(T, n_adapters, max_rank) bytes: the
 * kernels check the plan's header and fall back to the tables. */
#define SLORA_FLAG_RESOLVED(max_rank) (((((unsigned)(max_rank) + 7u) >> 3) & 0x1fu) << 8)
#define SLORA_FLAG_RESOLVED_MASK (0x1fu << 8)
/* With SLORA_FLAG_BIG_GROUPS: the plan's count of 128-token tiles of big groups (slora_plan_header word 6), when the
   caller has read it, in bits 16..31 of flags.  The tensor-core launches then enumerate exactly those tiles (and
   size their K split for them) instead of the most a batch of T tokens could have.  0 = not known. */
#define SLORA_FLAG_BIG_TILES(n) (((unsigned)(n) & 0xffffu) << 16)

/* Bits of the device status word (plan header / status argument). */
#define SLORA_STATUS_BAD_ID 1      /* a token's adapter id was outside [0, n_adapters) - token skipped   */
#define SLORA_STATUS_BAD_TABLE 2   /* start/ranks4/loc entry out of range - work item skipped            */
#define SLORA_STATUS_BAD_RANK 4    /* expand met a rank outside {8,16,32,64,128} or wider than the delta
                                      buffers - work item skipped                                         */
#define SLORA_STATUS_TIMEOUT 8     /* a bounded wait for a bulk copy ran out - work item skipped          */

int slora_version(void);
const char* slora_last_error(void); /* thread-local, valid until the next failing call on this thread */

/*
 * Drop-in for the reference's one native entry point,
 *   dispatch_bgmv(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies, qkvo, lora_scales)
 *   (slora/csrc/lora_ops.cc:76-126).
 * Direction is chosen as the reference does (slora/csrc/bgmv/bgmv_impl.cuh:221,232): h_in < h_out => expand
 * (y[t,:] += scale * x[t,:r] . B), else shrink (y[t,:r] = x[t,:] . A^T, columns >= r untouched).
 * T tokens; x is [T, h_in] and y is [T, h_out], both contiguous as in the reference.
 */
int slora_dispatch_bgmv(void* y, const void* x, const void* w, const int64_t* start, const int64_t* ranks4,
                        const int64_t* loc, const int64_t* ids, int qkvo, const void* scales, int64_t T,
                        int h_in, int h_out, int64_t pool_rows, int64_t pool_stride, int64_t n_adapters,
                        int64_t loc_len, int dtype, void* stream);

/*
 * The two halves of dispatch_bgmv with explicit strides (replace bgmv_multi_lora_rank_shrink_kernel /
 * bgmv_multi_lora_rank_expand_kernel, slora/csrc/bgmv/bgmv_impl.cuh:15-149 and :153-208).
 * delta_width = number of columns of delta (the batch's maximum rank).
 */
int slora_bgmv_shrink(void* delta, const void* x, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int64_t* ids, int qkvo, int64_t T, int h_in, int64_t x_stride,
                      int64_t delta_stride, int delta_width, int64_t pool_rows, int64_t pool_stride,
                      int64_t n_adapters, int64_t loc_len, int dtype, void* stream);
int slora_bgmv_expand(void* y, const void* delta, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int64_t* ids, const void* scales, int qkvo, int64_t T,
                      int h_out, int64_t delta_stride, int delta_width, int64_t y_stride, int64_t pool_rows,
                      int64_t pool_stride, int64_t n_adapters, int64_t loc_len, int dtype, void* stream);

/*
 * Segment (prefill) variants: request i covers tokens [seg_start[i], seg_start[i]+seg_len[i]) and uses adapter
 * seg_adapter[i].  Replace lora_get_qkvo_fwd_shrink / lora_get_qkvo_fwd_expand
 * (slora/models/peft/triton_kernel/lora/lora_prefill.py:139-164 and :105-136).  seg_start/seg_len are int32
 * (the reference's b_start_loc / b_seq_len), seg_adapter int64 (req_bins).  max_seg_len bounds the grid exactly as
 * the reference's max_input_len does.
 *
 * Segments of 32 tokens or more whose adapter has 8..128 slot rows (a multiple of 8) are computed on the tensor
 * cores (tcgen05, FP32 accumulation in tensor memory) in tiles of 128 tokens, when the layout allows: for the
 * shrink pool_stride == h_in and h_in % 64 == 0; for the expand 16-byte aligned y and delta rows.  Everything else
 * of the same call runs on the CUDA-core kernels; the two launches write disjoint tokens.  Results of the two
 * paths differ in summation order only (same tolerance against the FP32 oracle).  SLORA_MMA=0 in the environment
 * keeps every segment on the CUDA-core kernels.
 */
int slora_sgmv_shrink(void* delta, const void* x, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int32_t* seg_start, const int32_t* seg_len,
                      const int64_t* seg_adapter, int n_seg, int max_seg_len, int qkvo, int64_t T, int h_in,
                      int64_t x_stride, int64_t delta_stride, int delta_width, int64_t pool_rows,
                      int64_t pool_stride, int64_t n_adapters, int64_t loc_len, int dtype, void* stream);
int slora_sgmv_expand(void* y, const void* delta, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int32_t* seg_start, const int32_t* seg_len,
                      const int64_t* seg_adapter, const void* scales, int n_seg, int max_seg_len, int qkvo,
                      int64_t T, int h_out, int64_t delta_stride, int delta_width, int64_t y_stride,
                      int64_t pool_rows, int64_t pool_stride, int64_t n_adapters, int64_t loc_len, int dtype,
                      void* stream);

/*
 * Batch plan: groups the tokens of one batch by adapter once, so that every later call of the batch (all layers,
 * all projections) reads each adapter row once per group instead of once per token.  The reference has no
 * counterpart (it re-derives everything per token in every launch, bgmv_impl.cuh:34-38); the plan plays the role
 * of req_bins / batch_req_bins built in LoraUnorderedBatchInfer.__init__ / forward
 * (slora/models/peft/lora_unordered_batch_infer.py:24-38,66).
 * The workspace is caller-owned device memory of slora_plan_workspace_bytes(T, n_adapters) bytes, 16-byte aligned.
 * slora_plan_build launches one small kernel on the stream; the plan is valid for later calls on that stream.
 * slora_plan_status copies the plan's status word back (synchronises the stream).
 */
size_t slora_plan_workspace_bytes(int64_t T, int64_t n_adapters);
/* The same with resolved tiles for adapters of rank <= max_rank (see SLORA_FLAG_RESOLVED): loc is the adapters' loc
 * table and scales their scale table (16-bit values; may be NULL), both read when the plan is built, so the plan
 * must be rebuilt when they change.  max_rank = 0 or loc = NULL: no resolved tiles. */
size_t slora_plan_workspace_bytes_ex(int64_t T, int64_t n_adapters, int max_rank);
int slora_plan_build_ex(void* workspace, size_t workspace_bytes, const int64_t* ids, int64_t T, const int64_t* start,
                        const int64_t* ranks4, const int64_t* loc, const void* scales, int64_t n_adapters,
                        int64_t loc_len, int max_rank, void* stream);
int slora_plan_build(void* workspace, size_t workspace_bytes, const int64_t* ids, int64_t T, const int64_t* start,
                     const int64_t* ranks4, int64_t n_adapters, int64_t loc_len, void* stream);
/*
 * Number of 128-token tiles of big same-adapter groups in a plan (0: SLORA_FLAG_BIG_GROUPS would only add empty
 * launches).  Reads the plan header back: synchronises `stream`.  No counterpart in the reference, which picks its
 * prefill kernels on the host from the request lengths (lora_unordered_batch_infer.py:127-130).
 */
int slora_plan_big_tiles(const void* workspace, int* n_big_out, void* stream);
/*
 * What a plan holds, for the caller's choice of flags: its 8-token tiles, its 128-token tiles of big groups (as
 * slora_plan_big_tiles) and the slot rows (rank) shared by every adapter of the batch, 0 when they differ.  Any of
 * the three pointers may be NULL.  Reads the plan header back: synchronises `stream`.
 */
int slora_plan_info(const void* workspace, int* n_tiles_out, int* n_big_out, int* uniform_rank_out, void* stream);

int slora_plan_status(const void* workspace, int* status_out, int* n_tiles_out, void* stream);
/*
 * The plan's 16 header words, for callers that choose flags from them: [1] 8-token tiles, [2] status bits, [4] tokens,
 * [5] adapters, [6] 128-token tiles of big groups, [9] the slot rows (rank) every group shares or 0, [10] 8-token tiles
 * of groups that are not big, [11] widest rank among the big groups, [12] 1 when every big group's rank is a power
 * of two.  Reads the header back: synchronises `stream`.  No counterpart in the reference.
 */
int slora_plan_header(const void* workspace, int32_t out[16], void* stream);

/*
 * Planned multi-projection calls.  nproj in 1..3 projections share the activations x (shrink) and the tables.
 * plan may be NULL, in which case ids (per-token adapter ids) must be given and every token is its own group.
 *   slora_lora_shrink_multi: delta[p][t, :r] = x[t, :] . A_{p}^T for p < nproj
 *   slora_lora_expand_multi: y[p][t, :] += scale * delta[p][t, :r_b] . B_{p}^T
 * delta element (t, k) of projection p is read at
 *   delta[p] + (k / (r_b / delta_parts)) * delta_part_stride + t * delta_stride + k % (r_b / delta_parts)
 * (delta_parts == 1: a plain [T, delta_stride] matrix; delta_parts == N: the all-gathered [N, T, r/N] buffer of an
 * N-way tensor-parallel shrink).  rank_mult: B rank = slot_rows * rank_mult (1 except under tensor parallelism).
 * These mirror _batch_lora_get_qkv / _batch_lora_get_o and _lora_get_qkv / _lora_get_o
 * (slora/models/peft/lora_unordered_batch_infer.py:254-318,428-448,321-424,451-483).
 */
int slora_lora_shrink_multi(const void* plan, const int64_t* ids, int nproj, const int* qkvo, void* const* delta,
                            int64_t delta_stride, int delta_width, const void* x, int64_t x_stride, int h_in,
                            const void* pool_a, int64_t pool_rows, int64_t pool_stride, const int64_t* start,
                            const int64_t* ranks4, const int64_t* loc, int64_t n_adapters, int64_t loc_len,
                            int64_t T, int dtype, unsigned flags, void* stream);
int slora_lora_expand_multi(const void* plan, const int64_t* ids, int nproj, const int* qkvo, void* const* y,
                            const int64_t* y_stride, const int* h_out, const void* const* delta,
                            int64_t delta_stride, int delta_width, int delta_parts, int64_t delta_part_stride,
                            int rank_mult, const void* pool_b, int64_t pool_rows, int64_t pool_stride,
                            const int64_t* start, const int64_t* ranks4, const int64_t* loc, const void* scales,
                            int64_t n_adapters, int64_t loc_len, int64_t T, int dtype, unsigned flags,
                            void* stream);

/*
 * One layer's q/k/v LoRA deltas (shrink for q,k,v then expand for q,k,v: two launches) and the o delta.
 * Counterparts of _batch_lora_get_qkv (lora_unordered_batch_infer.py:254-318) and _batch_lora_get_o (:428-448)
 * without the base torch.mm and rotary calls.  delta_* are caller scratch [T, delta_stride] like self.delta[0..2]
 * (:68-69,75-76); they need not be zeroed (only columns < r are written and read).
 */
int slora_batch_lora_qkv(const void* plan, const int64_t* ids, void* q, void* k, void* v, int64_t q_stride,
                         int64_t k_stride, int64_t v_stride, int h_out_q, int h_out_kv, const void* x,
                         int64_t x_stride, int h_in, const void* pool_a, const void* pool_b, int64_t pool_rows,
                         int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                         const void* scales, int64_t n_adapters, int64_t loc_len, void* delta_q, void* delta_k,
                         void* delta_v, int64_t delta_stride, int delta_width, int64_t T, int dtype,
                         unsigned flags, void* stream);
int slora_batch_lora_o(const void* plan, const int64_t* ids, void* o, int64_t o_stride, int h_out, const void* x,
                       int64_t x_stride, int h_in, const void* pool_a, const void* pool_b, int64_t pool_rows,
                       int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                       const void* scales, int64_t n_adapters, int64_t loc_len, void* delta, int64_t delta_stride,
                       int delta_width, int64_t T, int dtype, unsigned flags, void* stream);

/*
 * slora_batch_lora_qkv with the two steps that follow it in the reference's layer folded in: the rotary embedding of
 * q and k (rotary_emb_fwd, slora/models/peft/lora_unordered_batch_infer.py:277,298; kernel
 * slora/models/llama/triton_kernel/rotary_emb.py:8-71: out0 = x0 cos - x1 sin, out1 = x0 sin + x1 cos over the two
 * halves of every head) and the scatter of the new k and v rows into the KV pool (destindex_copy_kv,
 * slora/common/basemodel/layer_infer/template/transformer_layer_infer_template.py:50-62; kernel
 * slora/common/basemodel/triton_kernel/destindex_copy_kv.py:8-50).
 *   cos / sin: [T][head_dim / 2] in the I/O type, rows cs_stride elements apart (infer_state.position_cos / _sin).
 *   q is updated in place: q = rotary(q + lora_q(x)).
 *   k_out == NULL: k = rotary(k + lora_k(x)) and v = v + lora_v(x) in place.
 *   k_out != NULL: the results go to rows kv_rows[t] (device int64 [T]; infer_state.prefill_mem_index /
 *     decode_mem_index) of k_out and v_out, [kv_out_rows][kv_out_stride] with h_out_kv used columns (the pool's
 *     key_buffer[layer] / value_buffer[layer]); k and v themselves are only read (they hold the base projection).
 *     A token whose kv_rows entry is outside [0, kv_out_rows) is skipped with SLORA_STATUS_BAD_TABLE.
 * With head_dim == 128 and the pipelined expand both steps happen in the expand's epilogue (one pass over q, k, v
 * instead of three); otherwise (tensor-core routing of big groups, other layouts, other head sizes) the expand is
 * followed by one small launch that does them.  Values are rounded to the I/O type before the rotation, where the
 * reference stores them; the rotation itself is computed in FP32.
 */
int slora_batch_lora_qkv_rope(const void* plan, const int64_t* ids, void* q, void* k, void* v, int64_t q_stride,
                              int64_t k_stride, int64_t v_stride, int h_out_q, int h_out_kv, const void* x,
                              int64_t x_stride, int h_in, const void* pool_a, const void* pool_b, int64_t pool_rows,
                              int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                              const void* scales, int64_t n_adapters, int64_t loc_len, void* delta_q, void* delta_k,
                              void* delta_v, int64_t delta_stride, int delta_width, int64_t T, int dtype,
                              unsigned flags, void* stream, const void* cos, const void* sin, int64_t cs_stride,
                              int head_dim, const int64_t* kv_rows, void* k_out, void* v_out, int64_t kv_out_stride,
                              int64_t kv_out_rows);

/*
 * No counterpart in the reference.  The o-projection LoRA delta (same result as slora_batch_lora_o) for callers that
 * must not allocate device memory: code running inside someone else's memory budget or allocator -- a serving process
 * whose pool already owns the whole GPU, a plugin called from a real-time path that may not block on the driver's
 * allocation lock.  The batch plan and the rank-r intermediate live in an array built into the library (320 KB per
 * GPU, held from library load to process exit) instead of caller-provided workspace and delta buffers; the caller
 * passes only inputs and outputs.
 * Limits: T <= 1024 tokens, n_adapters <= 4096, max_rank a multiple of 8 up to 128; beyond them the call fails with
 * SLORA_ERR_WORKSPACE / SLORA_ERR_RANK and launches nothing.  The call never calls cudaMalloc, cudaFree or any
 * allocating routine; SLORA_FLAG_BIG_GROUPS is ignored here (that route may create a side stream at first use).
 * Its first call on a device looks up the array's device address (cudaGetSymbolAddress), which may also make the
 * CUDA runtime load the library's kernels: make that first call outside any stream capture, and before the host
 * hands the rest of the GPU's memory to its own pool.  All calls on one GPU share the array, which keeps the last
 * call's plan: calls whose kernels may overlap on the GPU (different streams without ordering) race on it; calls on
 * one stream are safe back to back.
 * The kernels' status word (SLORA_STATUS_*: a token with an adapter id outside the tables, a bad table entry, an
 * adapter wider than max_rank -- whose tokens are skipped --, a wait that ran out) lives in that array too;
 * slora_noalloc_status reads the word the latest call on the current device left (synchronises `stream`).
 */
int slora_batch_lora_o_noalloc(const int64_t* ids, void* o, int64_t o_stride, int h_out, const void* x,
                               int64_t x_stride, int h_in, const void* pool_a, const void* pool_b, int64_t pool_rows,
                               int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                               const void* scales, int64_t n_adapters, int64_t loc_len, int max_rank, int64_t T,
                               int dtype, unsigned flags, void* stream);
int slora_noalloc_status(int* status_out, void* stream);

/*
 * Debug check of the tables (the reference has none; its kernels read whatever the tables say).
 * Launches one kernel that range-checks start/ranks4/loc/ids and writes report[0] = number of bad entries,
 * report[1] = kind of the first one found (1 ids, 2 start/ranks4, 3 loc), report[2] = its index.
 * report is device memory (4 x int32).  Asynchronous; the caller reads report after synchronising.
 */
int slora_validate_tables(const int64_t* start, const int64_t* ranks4, const int64_t* loc, const int64_t* ids,
                          int64_t n_adapters, int64_t loc_len, int64_t T, int64_t pool_rows, int32_t* report,
                          void* stream);

/*
 * Tensor parallelism (no reference code: lora_adapter.py:24 asserts world_size 1; the scheme is figures/slora_tp.png):
 * after the all-gather of the rank-sharded intermediates, `gathered` holds [n_parts][nproj][T][part_width] (part g
 * starts at element g * part_stride; its row (p, t) holds rank rows [g * rs, (g + 1) * rs) of token t's adapter,
 * rs = ranks4[ids[t]] / 4 slot rows per part).  Writes plain delta rows out[p][t][g * rs + j], out being
 * [nproj][T][n_parts * part_width], the layout slora_lora_expand_multi reads with delta_parts = 1 and
 * rank_mult = n_parts.  Columns at and beyond an adapter's rank are not written.
 */
int slora_tp_regroup(void* out, const void* gathered, const int64_t* ids, const int64_t* ranks4, int n_parts,
                     int nproj, int64_t T, int part_width, int64_t part_stride, int64_t n_adapters, int dtype,
                     void* stream);

/*
 * Tensor parallelism, the exchange over peer memory (NVLink loads/stores; no reference code, see slora_tp_regroup).
 * One launch per rank replaces all-gather + slora_tp_regroup: rank `my_part` writes its [nproj][T][part_width]
 * intermediates `local` into every rank's delta buffer peer_full[g] ([2][3][full_tokens][n_parts * part_width]; the
 * caller names the half: 0 for q,k,v calls, 1 for o calls, strictly alternating) at the regrouped columns, raises
 * its flag on every rank (peer_flags[g]: int32 [2][n_parts]) and waits until the flags of all ranks for this exchange
 * have arrived on this rank.  The expand then reads peer_full[my_part] + half * 3 * full_tokens * R with
 * delta_parts = 1, rank_mult = n_parts.
 *   peer_full / peer_flags: host arrays of n_parts device pointers valid on this GPU (symmetric memory, or
 *   cudaIpc / cudaMalloc with peer access); flags start at zero.  seq_state: int32 [2] in this GPU's memory, zero at
 *   the start: exchanges completed per half, maintained by the kernel (so a captured graph can be replayed).
 *   counter: one zero-initialised int32 in this GPU's memory.  status: device status word or NULL.
 *   mode: 1 = write and signal, 2 = wait (and count the exchange as done), 3 = both (the normal call).
 *   flags: SLORA_FLAG_PDL lets the expand that follows fetch its adapter rows while the exchange is in flight.
 * The wait is bounded (about 2 s of SM clock); when it runs out SLORA_STATUS_TIMEOUT is set in *status and the
 * kernel returns, so a missing rank never hangs the GPU.  Ranks must run on different GPUs (a rank waiting for
 * another rank's launch on the same GPU may wait for a kernel that cannot start).
 */
int slora_tp_exchange(const void* local, void* const* peer_full, int32_t* const* peer_flags, int32_t* counter,
                      int32_t* status, const int64_t* ids, const int64_t* ranks4, int my_part, int n_parts, int nproj,
                      int64_t T, int64_t full_tokens, int part_width, int64_t n_adapters, int half, int32_t* seq_state,
                      int mode, int dtype, unsigned flags, void* stream);

/*
 * Tensor parallelism with a head-sharded input (the o projection after attention: each rank holds x[T, h_in / N]):
 * A is then sharded over the INPUT dimension - a rank's slot holds the [r, h_in / N] slice of A, flat, in r / N pool
 * rows - every rank computes a partial [T, r] and the partials are summed (figures/slora_tp.png; the reference has
 * no code for it).
 *   slora_lora_shrink_rows: slora_lora_shrink_multi with rank_mult A rows per slot row (rank_mult = N here, h_in the
 *     shard width; delta_width must hold r).
 *   slora_tp_allsum: all-reduce (sum) of the partials over peer memory.  Every rank copies its local [T][width] block
 *     into slot my_part of every rank's parts buffer ([n_parts][full_tokens][width]), signals and waits exactly as
 *     slora_tp_exchange does (same flags / seq_state / half / counter conventions; o calls use half 1), then a second
 *     small launch adds the n_parts slots in FP32 and writes out[T][width] in the I/O type.  width % 8 == 0.
 *     mode: 1 = write and signal, 2 = wait and sum, 3 = both (the normal call).
 */
int slora_lora_shrink_rows(const void* plan, const int64_t* ids, int nproj, const int* qkvo, void* const* delta,
                           int64_t delta_stride, int delta_width, int rank_mult, const void* x, int64_t x_stride,
                           int h_in, const void* pool_a, int64_t pool_rows, int64_t pool_stride, const int64_t* start,
                           const int64_t* ranks4, const int64_t* loc, int64_t n_adapters, int64_t loc_len, int64_t T,
                           int dtype, unsigned flags, void* stream);
int slora_tp_allsum(const void* local, void* const* peer_parts, int32_t* const* peer_flags, int32_t* counter,
                    int32_t* status, void* out, int my_part, int n_parts, int64_t T, int64_t full_tokens, int width,
                    int half, int32_t* seq_state, int mode, int dtype, unsigned flags, void* stream);

/*
 * The same exchange without a launch of its own (the pipelined kernels only; SLORA_ERR_SHAPE / SLORA_ERR_ALIGN with
 * "No suitable kernel" when the layout needs another kernel family - then use slora_lora_shrink_multi +
 * slora_tp_exchange + slora_lora_expand_multi).
 *   slora_tp_shrink_push: the planned shrink of slora_lora_shrink_multi whose reduction epilogue stores each result
 *     into every rank's delta buffer (regrouped columns) instead of a local buffer; the launch's last CTA raises this
 *     rank's flag on every rank.  part_width = columns per rank (R / n_parts).
 *   slora_tp_expand_wait: the planned expand of slora_lora_expand_multi reading this rank's delta buffer half; its
 *     producer warps wait (bounded, ~2 s) for every rank's flag after the grid-dependency wait and before the first
 *     delta row is copied - adapter rows are already streaming by then; the launch's last CTA counts the exchange
 *     as done in seq_state.
 * Buffers, flags, seq_state, half: as for slora_tp_exchange; counter: one zero-initialised int32 per entry point.
 * The two calls of one exchange must both be made (a rank that pushes must also wait).  T == 0 returns at once.
 *
 * inband != 0 (both calls of an exchange alike): no flag, no fence.  The delta buffers must start out filled with the
 * 16-bit pattern 0xffff (a NaN that no float-to-16-bit conversion produces); the shrink stores its results with
 * plain stores and signals nothing; the expand starts as soon as this rank's own shrink has finished, and a consumer
 * lane that finds the pattern among the eight delta values it is about to use re-reads them from this rank's buffer
 * until the other rank's store has landed (bounded, ~2 s, then SLORA_STATUS_TIMEOUT and zeros).  The expand's last
 * CTA refills the half it consumed with the pattern.  Only the pipelined kernels do this: a layout they do not take
 * is an error in this mode.
 * inband == 2: the same, and the expand does not wait for this rank's own shrink grid either (its values are
 * recognised like the peers'): the two calls of an exchange must follow each other on one stream, and with
 * SLORA_FLAG_PDL the expand's CTAs start as the shrink's retire (the shrink lets dependents launch only after its own
 * grid-dependency wait, so what preceded the shrink is complete before the expand reads y).
 * inband == 3: the early start over buffers of THREE parts, [3][3][full_tokens][R] (all 0xffff at the start), that
 * rotate with the exchange's number.  seq_state is then two words of this rank's device memory, zeroed once and the
 * kernels' to keep: word 0 is read by a shrink (after its grid-dependency wait) as its exchange's number e, word 1 is
 * left by that shrink for its expand, which writes e + 1 back to word 0.  The exchange works in part e % 3 on every
 * rank, and the shrink refills - spread over its CTAs, on this rank's own buffer - the part exchange e - 1 used.
 * Nothing is done at the end of an expand; `half` is ignored; every rank must make the same sequence of calls.
 */
int slora_tp_shrink_push(const void* plan, const int64_t* ids, int nproj, const int* qkvo, int part_width,
                         const void* x, int64_t x_stride, int h_in, const void* pool_a, int64_t pool_rows,
                         int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                         int64_t n_adapters, int64_t loc_len, int64_t T, void* const* peer_full,
                         int32_t* const* peer_flags, int32_t* counter, int32_t* seq_state, int my_part, int n_parts,
                         int half, int64_t full_tokens, int inband, int dtype, unsigned flags, void* stream);
int slora_tp_expand_wait(const void* plan, const int64_t* ids, int nproj, const int* qkvo, void* const* y,
                         const int64_t* y_stride, const int* h_out, const void* pool_b, int64_t pool_rows,
                         int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                         const void* scales, int64_t n_adapters, int64_t loc_len, int64_t T, void* my_full,
                         int32_t* my_flags, int32_t* counter, int32_t* seq_state, int my_part, int n_parts, int half,
                         int64_t full_tokens, int part_width, int inband, int dtype, unsigned flags, void* stream);

/*
 * Adapter load into the Unified-Paging pool: replaces the per-layer indexed copies of InferAdapter.load_lora_A /
 * load_lora_B (slora/server/router/model_infer/infer_adapter.py:41-90: two index_put launches per layer and adapter)
 * by one launch for all layers and both buffers.  key_buffers / value_buffers / src are HOST arrays of n_layers device
 * pointers: src[l] holds the adapter's [2][n_rows][row_bytes] block of layer l (w_combined: A rows, then B rows,
 * lora_layer_weight.py:215-224); row i goes to pool row loc[i] (device int64) of key_buffers[l] (A) and
 * value_buffers[l] (B), pool rows being pool_row_bytes apart.  Rows are multiples of 16 bytes.  A loc entry outside
 * [0, pool_rows) is skipped and SLORA_STATUS_BAD_TABLE is set in *status (device int32, may be NULL).
 */
int slora_pool_scatter_rows(void* const* key_buffers, void* const* value_buffers, const void* const* src, int n_layers,
                            const int64_t* loc, int64_t n_rows, int64_t row_bytes, int64_t pool_rows,
                            int64_t pool_row_bytes, int32_t* status, void* stream);

/*
 * Row allocation from the pool's free map: replaces MemoryAllocator.alloc (slora/common/mem_allocator.py:30-39: a
 * cumulative sum over the whole map, a mask and a nonzero, whose result size the host has to wait for).  mem_state is
 * the map itself (one byte per pool row, non-zero = free; a torch.bool tensor), 16-byte aligned.  The first `need`
 * free rows, in increasing order, are written to out_rows[0..need) (device int64) and marked used; nothing comes back
 * to the host, so the call is asynchronous - the caller keeps the count of free rows, as the reference does
 * (can_use_mem_size).  If the map holds fewer than `need` free rows, those it has are handed out, the remaining
 * entries are set to -1 and SLORA_STATUS_BAD_TABLE is set in *status (device int32, may be NULL).
 * workspace: slora_pool_alloc_workspace_bytes(tot_rows) bytes of device memory, contents irrelevant.
 */
size_t slora_pool_alloc_workspace_bytes(int64_t tot_rows);
int slora_pool_alloc_rows(uint8_t* mem_state, int64_t tot_rows, int64_t need, int64_t* out_rows, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream);

/*
 * MemoryAllocator.free (slora/common/mem_allocator.py:185-199): mem_state[rows[i]] = 1 for i < n.  Rows outside
 * [0, tot_rows) are skipped with SLORA_STATUS_BAD_TABLE.
 */
int slora_pool_free_rows(uint8_t* mem_state, int64_t tot_rows, const int64_t* rows, int64_t n, int32_t* status,
                         void* stream);

/*
 * Table compaction after adapters are dropped: replaces the body of InferAdapter.offload_adapters
 * (slora/server/router/model_infer/infer_adapter.py:186-250: index gathers, a cumulative sum, a Triton
 * variable-length copy and MemoryAllocator.free) by two launches.  keep[i] != 0 (device bytes) marks the adapters that
 * stay; they keep their order.  new_len / new_scaling = the kept entries, new_start = exclusive prefix sum of the kept
 * lengths, new_loc = the kept runs of a_loc back to back; every pool row of a dropped adapter is marked free in
 * mem_state (skipped when mem_state is NULL).  a_scaling / new_scaling have 2-byte elements.  The new tables are
 * separate buffers with room for n_adapters / loc_len entries; scratch holds n_adapters int64; counts (device int64[2],
 * may be NULL) receives the kept adapters and kept rows.  An adapter whose run does not fit in a_loc is neither kept
 * nor freed and sets SLORA_STATUS_BAD_TABLE.
 */
int slora_tables_compact(const int64_t* a_start, const int64_t* a_len, const int64_t* a_loc, const void* a_scaling,
                         const uint8_t* keep, int64_t n_adapters, int64_t loc_len, int64_t* new_start,
                         int64_t* new_len, int64_t* new_loc, void* new_scaling, int64_t* scratch, int64_t* counts,
                         uint8_t* mem_state, int64_t tot_rows, int32_t* status, void* stream);

/* Kernels this process has launched through the library so far, per family:
 * out[0] simple (one CTA per work item), out[1] pipelined (persistent, warp-specialised), out[2] tensor core
 * (tcgen05, long segments), out[3] plan building and table validation.  The counters only ever grow; a caller
 * that wants the launches of a region subtracts two readings.  (Accounting aid: the reference has no counterpart;
 * its kernel launches are counted by the profiler.) */
void slora_launch_counts(int64_t out[4]);

#ifdef __cplusplus
}
#endif
#endif /* SLORA_B200_H_ */
