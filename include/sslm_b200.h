/* libsslm_b200 -- the C ABI of the B200 (sm_100a) implementation of SuperSLM's
 * integer-only transformer forward pass.
 *
 * The first block re-declares, name for name and argument for argument, the verbs of the
 * reference's public ABI that lie on the forward-pass path, so that a program written
 * against the reference header links against this library unchanged. Each declaration
 * cites the reference declaration it replaces (paths inside the reference project).
 * Handles are opaque; statuses keep the reference's frozen ordinals
 * (include/superslm/sslm_abi.h:96-163).
 *
 * Differences a caller can observe, all inside the reference's contract:
 *  - model weights and KV live in GPU memory. The `buf` passed to sslm_kv_pool_create /
 *    sslm_workspace_create is still validated (non-null, size, 64-byte alignment) but is
 *    used only as the caller's reservation: device memory of the same capacity is
 *    allocated by the call (SSLM_ALLOCATION_FAILED if the device cannot provide it).
 *  - sslm_kv_block_size still returns layers*context_cap*kv_heads*head_dim*2 bytes; a
 *    pool of N blocks holds N full-length sequences, stored as 16-token pages.
 *  - the int16 KV precision is rejected at map time with SSLM_ARTIFACT_REJECTED; the
 *    Option-G header flag is ignored, as the reference's CPU ABI path ignores it
 *    (src/sslm_abi.cpp:1539, :2256 always run the legacy K landing).
 * There is no CPU fallback: every compute verb fails with SSLM_ALLOCATION_FAILED if no
 * CUDA device is usable.
 */
#ifndef SSLM_B200_H
#define SSLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- types: include/superslm/sslm_abi.h:20-46, :96-224, :250 ---------------------- */
typedef struct sslm_model_s* sslm_model;
typedef struct sslm_seq_s* sslm_seq;
typedef struct sslm_adapter_s* sslm_adapter;
typedef struct sslm_prefix_s* sslm_prefix;
typedef struct sslm_schema_s* sslm_schema;     /* owned by the model; NULL = no schema */
typedef struct sslm_kv_pool_s* sslm_kv_pool;
typedef struct sslm_workspace_s* sslm_workspace;

typedef struct sslm_config {
	int32_t max_batch;        /* max sequences in one sslm_decode_step call, >= 1 */
	int32_t max_chunk_budget; /* max tokens in one sslm_prefill call, >= 1 */
	int32_t max_layer_budget; /* in [1, num_hidden_layers] */
	uint32_t reserved;        /* must be 0 */
} sslm_config;

typedef enum sslm_status {
	SSLM_OK = 0,
	SSLM_INVALID_ARGUMENT = 1,
	SSLM_BUFFER_TOO_SMALL = 2,
	SSLM_MISALIGNED_BUFFER = 3,
	SSLM_ARTIFACT_REJECTED = 4,
	SSLM_ADAPTER_MODEL_MISMATCH = 5,
	SSLM_RESTORE_MODEL_MISMATCH = 6,
	SSLM_RESTORE_KV_MISMATCH = 7,
	SSLM_MODEL_HAS_LIVE_SEQUENCES = 8,
	SSLM_POOL_HAS_LIVE_HANDLES = 9,
	SSLM_ADAPTER_HAS_LIVE_SEQUENCES = 10,
	SSLM_ADAPTER_SWAP_MIDTOKEN_REJECTED = 11,
	SSLM_SEQ_RESET_MIDTOKEN_REJECTED = 12,
	SSLM_PREFIX_FROZEN_REJECTED = 13,
	SSLM_KV_POOL_EXHAUSTED = 14,
	SSLM_TOKEN_ID_OUT_OF_RANGE = 15,
	SSLM_CONTEXT_CAP_EXCEEDED = 16,
	SSLM_TOKEN_ID_UNMAPPED = 17,
	SSLM_SCHEMA_NOT_FOUND = 18,
	SSLM_SCHEMA_BIND_REJECTED = 19,
	SSLM_SCHEMA_SPAN_UNBOUND = 20,
	SSLM_PREFIX_SCHEMA_MISMATCH = 21,
	SSLM_RESTORE_SCHEMA_MISMATCH = 22,
	SSLM_SCHEMA_SPAN_UNREACHABLE = 23,
	SSLM_SCHEMA_UNSATISFIABLE = 24,
	SSLM_ALLOCATION_FAILED = 25,
	SSLM_NUMERIC_STEP_REFUSED = 26,
	SSLM_STATUS_NEXT_FREE
} sslm_status;

typedef enum sslm_span_kind { SSLM_SPAN_PROMPT = 0, SSLM_SPAN_SCHEMA_CONTENT = 1 } sslm_span_kind;

/* sslm_decode_step reads layer_budget only (the v1.1 four-byte prefix); the remaining
 * fields exist so that the struct has the reference's size and layout. */
typedef struct sslm_decode_params {
	int32_t layer_budget;
	uint32_t struct_size;
	int32_t mode;
	int32_t alpha_q15;
	int32_t anti_lm_max_order;
	int32_t top_k;
	int64_t q_ln2;
	int64_t q_b;
	int64_t q_c;
} sslm_decode_params;

#define SSLM_ABI_ALIGNMENT_BYTES 64u

/* every entry point below has default visibility; the rest of the library is hidden */
#if defined(__GNUC__)
#define SSLM_API __attribute__((visibility("default")))
#else
#define SSLM_API
#endif

/* ---- model: include/superslm/sslm_abi_functions_g5_comparable.inc (sslm_model_map,
 *      sslm_model_unmap); src/sslm_abi.cpp:1058-1140. The artifact bytes are copied to the
 *      device during the call; the caller may free `data` afterwards. */
SSLM_API sslm_status sslm_model_map(const void* data, size_t size, sslm_model* out);
SSLM_API sslm_status sslm_model_unmap(sslm_model model);

/* ---- sizing + pool + workspace: sslm_abi_functions.inc (sslm_kv_block_size,
 *      sslm_kv_pool_overhead_size, sslm_kv_pool_create/destroy, sslm_workspace_size,
 *      sslm_workspace_create/destroy); src/sslm_abi.cpp:852-1051 */
SSLM_API size_t sslm_kv_block_size(sslm_model model);
SSLM_API size_t sslm_kv_pool_overhead_size(sslm_model model, uint32_t block_count);
SSLM_API sslm_status sslm_kv_pool_create(sslm_model model, void* buf, size_t buf_size, uint32_t block_count,
                                sslm_kv_pool* out);
SSLM_API sslm_status sslm_kv_pool_destroy(sslm_kv_pool pool);
SSLM_API size_t sslm_workspace_size(sslm_model model, const sslm_config* config);
SSLM_API sslm_status sslm_workspace_create(sslm_model model, const sslm_config* config, void* buf,
                                  size_t buf_size, sslm_workspace* out);
SSLM_API sslm_status sslm_workspace_destroy(sslm_workspace ws);

/* ---- sequences: sslm_abi_functions_g5_comparable.inc (sslm_seq_create, sslm_seq_release,
 *      sslm_prefill, sslm_decode_step); src/sslm_abi.cpp:1695-1760, :1950-1975, :1989-2449.
 *      sslm_prefill consumes min(count, chunk_budget) tokens as ONE chunk-batched pass;
 *      sslm_decode_step advances every sequence by params->layer_budget layers and writes
 *      the greedy token, or -1 while the token is in flight, -3 for a released handle. `ws`
 *      may be NULL (an internal workspace is used). */
SSLM_API sslm_status sslm_seq_create(sslm_model model, sslm_kv_pool* pool, sslm_seq* out);
SSLM_API sslm_status sslm_seq_release(sslm_seq seq);
SSLM_API sslm_status sslm_prefill(sslm_model model, sslm_seq seq, const int32_t* tokens, int32_t count,
                         int32_t chunk_budget, sslm_span_kind kind, sslm_workspace ws,
                         int32_t* consumed);
SSLM_API sslm_status sslm_decode_step(sslm_model model, sslm_seq* seqs, int32_t n,
                             const sslm_decode_params* params, sslm_workspace ws, int32_t* out_tokens);

/* ---- adapters: sslm_abi_functions.inc (sslm_adapter_map, sslm_adapter_release,
 *      sslm_adapter_residency, sslm_seq_set_adapter); src/sslm_abi.cpp:2990-3118 */
SSLM_API sslm_status sslm_adapter_map(const void* data, size_t size, sslm_model base, sslm_adapter* out);
SSLM_API sslm_status sslm_adapter_release(sslm_adapter adapter);
SSLM_API size_t sslm_adapter_residency(sslm_adapter adapter);
SSLM_API sslm_status sslm_seq_set_adapter(sslm_seq seq, sslm_adapter adapter /* NULL = detach */);

/* ---- state export: sslm_abi_functions.inc (sslm_seq_save); src/sslm_abi.cpp:2620-2716.
 *      Writes the reference's SSB3 blob, KV block in canonical
 *      [layer][K|V][kv_head][position][head_dim] order. */
SSLM_API sslm_status sslm_seq_save(sslm_seq seq, void* buf, size_t* n);

/* ---- state import and restart: sslm_abi_functions_g5_comparable.inc (sslm_seq_restore,
 *      sslm_seq_reset); src/sslm_abi.cpp:2722-2990, :1820-1860.
 *      Restore accepts the blobs sslm_seq_save writes here AND the ones the reference's CPU
 *      library writes (SSB3, and its SSB2 predecessor), so a sequence saved on either side
 *      continues bit-exactly on the other. Validation order and statuses follow the
 *      reference: bad magic / lengths -> SSLM_INVALID_ARGUMENT, other model ->
 *      SSLM_RESTORE_MODEL_MISMATCH, other KV precision -> SSLM_RESTORE_KV_MISMATCH, any
 *      schema binding that does not resolve in this model -> SSLM_RESTORE_SCHEMA_MISMATCH, pool of
 *      another model -> SSLM_INVALID_ARGUMENT, no free block -> SSLM_KV_POOL_EXHAUSTED.
 *      A blob that carries damped-greedy history (sslm_decode_step_v2 state) is refused with
 *      SSLM_INVALID_ARGUMENT: that decode mode is not part of this library.
 *      Reset returns a sequence to the state of a freshly created one (an attached adapter
 *      stays attached); mid-token -> SSLM_SEQ_RESET_MIDTOKEN_REJECTED. */
SSLM_API sslm_status sslm_seq_restore(sslm_model model, sslm_kv_pool* pool, const void* buf, size_t n,
                                      sslm_seq* out);
SSLM_API sslm_status sslm_seq_reset(sslm_seq seq);

/* ---- shared prompt prefixes: sslm_abi_functions_g5_comparable.inc (sslm_prefix_begin,
 *      sslm_prefix_prefill, sslm_prefix_freeze, sslm_prefix_release, sslm_seq_adopt_prefix);
 *      src/sslm_abi.cpp:1584-1694, :1870-1925.
 *      A prefix holds one block credit of the pool, is prefilled like a sequence, frozen, and
 *      then adopted by any number of sequences, each of which continues as if it had prefilled
 *      the same tokens itself (same tokens, same save blobs). The reference copies the whole KV
 *      block at adoption; this library shares the prefix's full 16-token pages between the
 *      prefix and its adopters and copies only the last, partly filled page. Prefill of a frozen
 *      prefix -> SSLM_PREFIX_FROZEN_REJECTED; adopting a prefix that is not frozen, or one of
 *      another model -> SSLM_INVALID_ARGUMENT. A prefix may be released while sequences that
 *      adopted it live on. */
SSLM_API sslm_status sslm_prefix_begin(sslm_model model, sslm_kv_pool* pool, sslm_prefix* out);
SSLM_API sslm_status sslm_prefix_prefill(sslm_model model, sslm_prefix prefix, const int32_t* tokens, int32_t count,
                                         int32_t chunk_budget, sslm_span_kind kind, sslm_workspace ws,
                                         int32_t* consumed);
SSLM_API sslm_status sslm_prefix_freeze(sslm_prefix prefix);
SSLM_API sslm_status sslm_prefix_release(sslm_prefix prefix);
SSLM_API sslm_status sslm_seq_adopt_prefix(sslm_seq seq, sslm_prefix prefix);

/* ---- constrained decoding: sslm_abi_functions_g5_comparable.inc (sslm_schema_lookup,
 *      sslm_schema_count, sslm_schema_name, sslm_seq_set_schema, sslm_prefix_set_schema);
 *      src/sslm_abi.cpp:1236-1264, :1791-1818, :1646-1654, :1486-1512, :2392-2424;
 *      include/superslm/schema_masks.h (the SCM1 section).
 *      An artifact may carry decode schemas: DFAs over token ids with one vocab-bit mask page
 *      per state. A sequence bound to a schema picks each token as the arg-max over the tokens
 *      its current state allows (the mask is applied inside the vocab-head kernel) and then
 *      follows the transition; a state that allows nothing yields -2 in out_tokens and the
 *      sequence stays where it is (later steps report SSLM_ARTIFACT_REJECTED, as the
 *      reference's do). sslm_prefill with SSLM_SPAN_SCHEMA_CONTENT walks the DFA with the given
 *      tokens and stops with SSLM_SCHEMA_SPAN_UNREACHABLE at the first one the schema does not
 *      allow; SSLM_SPAN_PROMPT never moves the walk. The binding, the walk state and the count
 *      of forced tokens travel in save blobs. Binding is possible only on a fresh (or reset)
 *      sequence: otherwise SSLM_SCHEMA_BIND_REJECTED. Damped-greedy decoding
 *      (sslm_decode_step_v2) is not part of this library. */
SSLM_API sslm_status sslm_schema_lookup(sslm_model model, const char* name, sslm_schema* out);
SSLM_API size_t sslm_schema_count(sslm_model model);
SSLM_API sslm_status sslm_schema_name(sslm_model model, int32_t index, char* buf, size_t* n);
SSLM_API sslm_status sslm_seq_set_schema(sslm_seq seq, sslm_schema schema);
SSLM_API sslm_status sslm_prefix_set_schema(sslm_prefix prefix, sslm_schema schema);

/* ======================================================================================
 * Entry points below have no counterpart in the reference; they exist for device
 * selection, for the standalone linear-layer workload and for measurement.
 * ====================================================================================== */

/* CUDA device ordinal used by subsequent sslm_model_map calls of this process (default 0,
 * or the SSLM_B200_DEVICE environment variable). */
SSLM_API sslm_status sslm_b200_set_device(int ordinal);

/* One int8 linear layer with the reference's full epilogue, on host buffers:
 *   acc = x[M,K] . w[N,K]^T ; folded = ApplyWeightScaleFold(acc, fold[N,3]) ;
 *   per row: RequantChainChecked(folded, incoming = {in_scale[m]}, site constant).
 * (GemmInt8Accumulate + FunnelProjectedRow, src/matmul.cpp:466-509,
 * src/forward/forward_sites.cpp:1114-1146, :1182-1203.) Outputs that are NULL are skipped.
 * in_scales: M pairs (m, e); out_scales: M pairs; row_status: M reference
 * SslmForwardStatus ordinals (0 = Ok). use_tensor_cores: 0 forces the streaming GEMV
 * kernel, 1 lets M > 8 take the tcgen05 kernel. */
SSLM_API sslm_status sslm_b200_linear(const int8_t* x, const int8_t* w, const int32_t* fold, int32_t M,
                             int32_t N, int32_t K, const int64_t* in_scales, int64_t site_m,
                             int64_t site_e, int32_t use_tensor_cores, int32_t* out_folded,
                             int8_t* out_codes, int64_t* out_scales, int32_t* row_status);

/* The same layer with operands resident in HBM, launched `iters` times back to back on one
 * stream; returns the average device time of one launch of the GEMM/GEMV kernel plus its
 * funnel kernel in microseconds through *avg_us (CUDA events). For the benchmark. */
SSLM_API sslm_status sslm_b200_linear_bench(int32_t M, int32_t N, int32_t K, int32_t use_tensor_cores,
                                   int32_t iters, uint64_t seed, double* avg_us_gemm,
                                   double* avg_us_total);

/* Device time (ms, CUDA events on the workspace stream) of the most recent sslm_prefill or
 * sslm_decode_step that ran on `ws`, and the number of kernels launched on it so far. */
SSLM_API sslm_status sslm_b200_last_call_ms(sslm_workspace ws, float* ms, uint64_t* kernel_launches);

/* Process-wide counters of the tensor-core linear kernel: launches, times it declined a shape
 * (the streaming kernel ran instead) and the reason code of the last refusal. */
SSLM_API sslm_status sslm_b200_tc_stats(uint64_t* launches, uint64_t* refusals, int32_t* last_reason);
/* Launches of the tensor-core linear kernel per tile shape (rows x weight columns), first n of:
 * 128 x 64, 128 x 128, 256 x 64, 256 x 128. Lets a test assert which variant served a shape. */
SSLM_API sslm_status sslm_b200_tc_variant_counts(uint64_t* counts, int32_t n);

/* Attention cuts a row along its context width into slices that run as the blocks of one
 * thread-block cluster. splits = 1, 2, 4, 8 or 16 fixes the slices per kv head of later calls
 * (rounded down to a power of two, limited by the row's width); 0 restores the automatic choice.
 * Results do not depend on it. For tuning and for tests that walk every cut. */
SSLM_API sslm_status sslm_b200_set_attention_splits(int32_t splits);

/* Bisection aid (the counterpart of the reference's per-site trace hook,
 * src/forward/checked_chain_funnel.cpp:338-361). With a buffer set, every later sslm_prefill /
 * sslm_decode_step on this workspace appends one record per traced site, layer and row:
 *   { int64 position; int32 layer; int32 site; int64 scale_m; int64 scale_e; int32 n; int32 row }
 * followed by the site's n int8 codes, padded to a multiple of 8 bytes. Sites: 0 attn_norm,
 * 2 rotated q (no scale), 3 attn_ctx, 5 attn_residual, 6 mlp_norm, 9 mlp_act, 11 mlp_residual.
 * Records that do not fit are dropped. buf = NULL ends the trace; *used (optional) receives the
 * bytes the trace held when this call was made. Slow (a copy per record); results are unchanged. */
SSLM_API sslm_status sslm_b200_trace(sslm_workspace ws, void* buf, size_t capacity, size_t* used);

/* Tests only: every wait of the kernels on an mbarrier is bounded, and this makes one run out on
 * purpose. The next `launches` (0..16) launches of the tensor-core linear kernel arm the barrier of
 * their first weight tile in block 0 without requesting the tile; the wait on it gives up after its
 * poll limit (about a second), the rows of that tile end with an internal status, and the verb
 * that launched the kernel returns SSLM_ALLOCATION_FAILED like any other refusal (a prefill chunk
 * consumes nothing). Nothing faults and nothing spins without a limit; the next call works normally. */
SSLM_API sslm_status sslm_b200_debug_withhold_tc_load(int32_t launches);

/* Tests only: the device integer library's primitives evaluated ON THE DEVICE over n operand
 * tuples (host arrays a, b, c, e; three host result arrays), so that their device-only halves
 * (reciprocal / root estimates, 32-bit short forms) are held to the CPU oracle as well. `which`:
 *   0 DynamicScaleReciprocal(a)            1 ISqrt(a)            2 floor((a << 32) / b), |a| <= 127
 *   3 RequantTokenCodeWide(x = a, R = b, s = c): out0 the code, out1 / out2 the per-row coders' code
 *   4 LandingRescale(code a, m b, R c, e_a = e >> 32, e_t = low half of e): out0 value, out1 flags
 *   5 a / b (unsigned, small quotient)     6 the funnel's scalars for a one-element row of magnitude a,
 *     incoming scale (b, c), site constant (e >> 32, low half of e): out0/out1 the output scale, out2 status
 *   7 one i-exp softmax element: shifted score a, constants (q_ln2 b, q_b c, q_c e >> 32), peak = low
 *     half of e << 16: out0 value, out1 refused, out2 the value rebuilt from its (shift, remainder)
 *   8 Q15 probability floor((a << 15) / b). */
SSLM_API sslm_status sslm_b200_int_sweep(int32_t which, const int64_t* a, const int64_t* b, const int64_t* c,
                                const int64_t* e, int64_t n, int64_t* out0, int64_t* out1, int64_t* out2);

/* The vocabulary head on host buffers: logits[m, n] = sum_k x[m,k] w[n,k] (int32, no fold), and per
 * row the greedy token = the lowest index of the row's maximum (LogitsSite + NarrowRowChecked +
 * ArgmaxLowestIndexTieBreak, src/forward/forward_sites.cpp:2412-2437). out_logits ([M,N], may be
 * NULL: the kernels then keep only the running maximum, as in a decode step) and out_tokens [M].
 * use_tensor_cores as for sslm_b200_linear. For the parity sweep of the logits form. */
SSLM_API sslm_status sslm_b200_logits(const int8_t* x, const int8_t* w, int32_t M, int32_t N, int32_t K,
                             int32_t use_tensor_cores, int32_t* out_logits, int32_t* out_tokens);

/* Per-kernel-class device timing of later calls on `ws` (CUDA events around every launch;
 * slows the call slightly). Classes, in order: begin, linear q/k/v, q/k/v post, attention,
 * context funnel, linear o, residual 1, linear gate/up, activation, linear down, residual 2,
 * head, LoRA u, other. profile_read returns accumulated milliseconds and launch counts of the
 * first n classes since profiling was enabled. */
SSLM_API sslm_status sslm_b200_profile(sslm_workspace ws, int32_t enable);
SSLM_API sslm_status sslm_b200_profile_read(sslm_workspace ws, double* ms, uint64_t* launches, int32_t n);

/* Tests only: capture the full int32 logit row of every token produced by later
 * sslm_decode_step calls on `ws` into host memory ([tokens in call order][vocab]);
 * pass NULL to stop. */
SSLM_API sslm_status sslm_b200_capture_logits(sslm_workspace ws, int32_t* host_rows);

/* Bytes of HBM held by the model's weights, tables and constants. */
SSLM_API size_t sslm_b200_model_device_bytes(sslm_model model);

/* The layer of sslm_b200_linear for operands that are already in device memory, for callers
 * that may not allocate (all HBM already assigned to their own pools, or no device-wide stall
 * allowed where they call from). This entry point has no counterpart in the reference. It
 * allocates nothing on the host or the device: the only scratch the layer needs, the per-row
 * peak of the folded accumulators, lives in a fixed array inside the library's device image
 * (SSLM_B200_RESIDENT_MAX_ROWS rows). Every pointer is a device pointer on the calling
 * thread's current device; x, w and out_folded 16-byte aligned; out_folded is required
 * ([M,N] int32), out_codes / out_scales / row_status may be NULL. The work is enqueued on
 * `stream` (a cudaStream_t, NULL = the default stream) and the call returns without waiting.
 *  - M > SSLM_B200_RESIDENT_MAX_ROWS or K > 16384: SSLM_INVALID_ARGUMENT, nothing is launched.
 *  - The first call on a device also looks up the array's address (set-up): make that call
 *    before any stream capture begins.
 *  - All calls on a device share the array. It reads zero at load time and every call leaves
 *    it zero again; calls whose kernels may overlap in time (other streams or threads) race
 *    on it and must be ordered by the caller.
 * Always the streaming dp4a kernel (the tensor-core path keeps host-side caches). */
#define SSLM_B200_RESIDENT_MAX_ROWS 256
SSLM_API sslm_status sslm_b200_linear_resident(const int8_t* d_x, const int8_t* d_w, const int32_t* d_fold,
                                               int32_t M, int32_t N, int32_t K, const int64_t* d_in_scales,
                                               int64_t site_m, int64_t site_e, int32_t* d_out_folded,
                                               int8_t* d_out_codes, int64_t* d_out_scales,
                                               int32_t* d_row_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SSLM_B200_H */
