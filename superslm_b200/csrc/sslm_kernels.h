// Launch interface of the CUDA kernels (host side). Every launcher enqueues on the given
// stream and returns immediately; errors surface through cudaGetLastError at the call
// site. Nothing here allocates.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <utility>

#include "sslm_types.cuh"

namespace sslm {

// ---- programmatic dependent launch
// A step is a chain of ~285 short dependent kernels. Each is launched with the programmatic
// stream-serialization attribute: its blocks may be placed on the SMs, and run whatever does
// not depend on earlier kernels (index arithmetic, barrier and tensor-memory set-up), while
// the previous kernel is still running. Every kernel calls pdl_wait() before its first access
// to global memory -- it returns once the previous kernel has completed and its writes are
// visible -- and then pdl_release(), which lets the NEXT kernel's blocks be placed. Releasing
// only after the wait keeps the look-ahead to one kernel. A kernel launched without the
// attribute (or after a memcpy / memset) sees both calls as no-ops and plain stream order.
#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif
// SSLM_B200_PDL=0 in the environment turns the attribute off (plain stream order).
inline bool pdl_enabled() {
	static const bool on = [] {
		const char* e = getenv("SSLM_B200_PDL");
		return !(e && e[0] == '0');
	}();
	return on;
}
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = grid;
	cfg.blockDim = block;
	cfg.dynamicSmemBytes = smem;
	cfg.stream = st;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = attr;
	cfg.numAttrs = pdl_enabled() ? 1 : 0;
	return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ---- per-device one-time set-up
// cudaFuncSetAttribute and the device attributes apply to the CURRENT device only, and models may
// be mapped on several devices of one process (sslm_b200_set_device): everything a launcher sets
// up once is therefore kept per device ordinal. The set-up calls are idempotent, so two host
// threads racing through the first launch on a device at worst both make them.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
	std::atomic<unsigned char> done[kMaxDevices];
};
inline int current_device_ordinal() {
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
	return dev;
}
template <typename F>
cudaError_t once_per_device(PerDeviceOnce& o, F&& setup) {
	const int dev = current_device_ordinal();
	if (o.done[dev].load(std::memory_order_acquire)) return cudaSuccess;
	const cudaError_t e = setup();
	if (e == cudaSuccess) o.done[dev].store(1, std::memory_order_release);
	return e;
}
// multiprocessor count of the current device
inline int sm_count() {
	static std::atomic<int> cached[kMaxDevices];
	const int dev = current_device_ordinal();
	int v = cached[dev].load(std::memory_order_relaxed);
	if (v > 0) return v;
	if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v < 1) v = 148;
	cached[dev].store(v, std::memory_order_relaxed);
	return v;
}

struct RowSource { const int8_t* hidden; const Scale* scale; };  // nullptr hidden: embed rows[r].token
struct RowSink { int8_t* hidden; Scale* scale; };                // nullptr hidden: drop

// ---- per-row sites (sslm_rows.cu)
cudaError_t rows_configure(const Dims& d);
void launch_begin(const RowBatch& b, const Dims& d, const int8_t* embed, Scale c_embed,
                  const RowSource* src, const LayerDev* layer, cudaStream_t st);
void launch_rmsnorm(const RowBatch& b, const Dims& d, const int8_t* gain, Scale site, cudaStream_t st);
void launch_qkv_post(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index,
                     KvPoolDev pool, const int32_t* cos, const int32_t* sin, cudaStream_t st);
void launch_ctx_funnel(const RowBatch& b, const Dims& d, const LayerDev* layer, cudaStream_t st);
void launch_res1(const RowBatch& b, const Dims& d, const LayerDev* layer, cudaStream_t st);
void launch_res2(const RowBatch& b, const Dims& d, const LayerDev* layer, const LayerDev* next,
                 cudaStream_t st);
void launch_act(const RowBatch& b, const Dims& d, const LayerDev* layer, const int32_t* silu,
                cudaStream_t st);
void launch_scatter(const RowBatch& b, const Dims& d, const RowSink* sink, cudaStream_t st);

// ---- int8 linear layers (sslm_gemv.cu, sslm_gemm_tc.cu)
// out[m, n] = fold_n( sum_k x[m,k] * w[n,k] ) (+ LoRA delta), plus the per-row max |out|
// of each column segment, reduced into rowmax[m][slot].
struct LinearArgs {
	const int8_t* x;      // [M, K] row-major activations
	const int8_t* w;      // [N, K] row-major weights
	const int32_t* fold;  // [N, 3] or nullptr (no fold: logits)
	int M, N, K;
	void* out;            // [M, out_ld] int32, or int64 when out64
	int out_ld;
	int out64;
	unsigned long long* rowmax;  // [M][4] or nullptr
	int nseg;             // column segments (fused projections)
	int seg_end[3];       // exclusive end column of each segment
	int seg_slot[3];      // rowmax slot per segment, -1: none
	int seg_lora[3];      // LoraSlot per segment, -1: projection is never adapted
	const RowDesc* rows;  // per-row adapter pointers (may be nullptr: no LoRA at all)
	int layer;
	const int8_t* lora_u; // [M][3][kMaxLoraRank]
	// head mode: packed argmax keys instead of a stored row (out may be nullptr)
	unsigned long long* best;
	int32_t* logits;      // optional full dump [M, N]
	// head mode, constrained decoding: per row the vocab-bit mask page of the row's DFA state
	// (bit n clear = token n not allowed: its logit counts as INT32_MIN, ApplyMaskAndArgmax,
	// src/forward/forward_sites.cpp:2443-2449), or nullptr for an unconstrained row; the array
	// itself may be nullptr
	const uint8_t* const* row_mask;
	int32_t* status;      // [M] row statuses (a bounded device wait that ran out is reported here), or nullptr
	// split-K scratch of the tensor-core path (optional): partial accumulators and one
	// arrival counter per output tile. Counters are zero between launches.
	int32_t* partial;
	size_t partial_bytes;
	unsigned int* tile_counters;
	int n_tile_counters;
	int splits;           // filled in by launch_linear_tc
	int debug_withhold;   // tests only (tc_debug_withhold): block 0 never requests its first weight tile
};
// HBM-bound small-M path: bulk-copy weight streaming through a shared-memory ring, dp4a.
cudaError_t launch_linear_gemv(const LinearArgs& a, cudaStream_t st);
// tensor-core path for M > 8 rows (tcgen05 kind::i8, TMA-fed). Returns false when the
// shape is not supported by that kernel (caller then uses the GEMV path).
bool launch_linear_tc(const LinearArgs& a, cudaStream_t st);
// Tests of the bounded waits: the next `launches` tensor-core launches arm their first weight-tile
// barrier in block 0 without requesting the tile, so that the wait on it runs out (no fault, no
// endless loop: the rows of that tile end with the internal wait-timeout status).
void tc_debug_withhold(int launches);
// process-wide counters of the tensor-core path: launches, refusals, reason of the last refusal
void tc_stats(unsigned long long* launches, unsigned long long* refusals, int* last_reason);
// launches per kernel variant (tile shape) of the tensor-core path
void tc_variant_counts(unsigned long long* counts, int n);

// u = clamp127(amp_fold(A x)) for up to three projections sharing the input x
// (AddAmplifyingLoraDelta's first half, src/forward/forward_sites.cpp:1062-1080)
void launch_lora_u(const RowBatch& b, const int8_t* x, int k_in, int layer, int nproj,
                   const int* lora_slots, cudaStream_t st);

// ---- attention over the paged KV pool (sslm_attn.cu)
cudaError_t attn_configure(const Dims& d);
// slices per kv head of later attention launches (0: chosen per launch); for tuning and tests
void attn_force_splits(int splits);
// Returns true when the launch also ran the attention-context funnel (codes in b.ctx, scale in
// b.cs); otherwise b.ctxw / rowmax slot 3 are filled and launch_ctx_funnel must follow.
bool launch_attention(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index,
                      KvPoolDev pool, int max_width, int reverse_rows, cudaStream_t st, cudaError_t* err);
// gather a sequence's pages into the reference's canonical block layout
// [layer][K|V][kv_head][position][head_dim]; positions beyond `valid(layer)` are zero
void launch_kv_export(const Dims& d, KvPoolDev pool, const int32_t* pages, int context_length,
                      int layer_index, int8_t* out, cudaStream_t st);
// tests: the device integer primitives over arrays of operands (device pointers)
void launch_int_sweep(int which, const int64_t* a, const int64_t* b, const int64_t* c, const int64_t* e, long long n, int64_t* out0,
                      int64_t* out1, int64_t* out2, cudaStream_t st);
// copy page src_page to dst_page in every (layer, kv head, K|V) plane
void launch_page_copy(const Dims& d, KvPoolDev pool, int src_page, int dst_page, cudaStream_t st);
// the inverse: scatter a canonical block into the sequence's pages (valid positions only)
void launch_kv_import(const Dims& d, KvPoolDev pool, const int32_t* pages, int context_length,
                      int layer_index, const int8_t* in, cudaStream_t st);

}  // namespace sslm
