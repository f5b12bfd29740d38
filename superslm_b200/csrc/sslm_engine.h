// Host-side objects behind the sslm_* handles: a model resident in HBM, a paged KV pool,
// a workspace (device scratch + stream + pinned staging), sequences and adapters.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/sslm_b200.h"
#include "sslm_artifact.h"
#include "sslm_kernels.h"
#include "sslm_schema.h"

struct DeviceArena {
	uint8_t* base = nullptr;
	size_t size = 0, used = 0;
	void* take(size_t bytes) {
		used = (used + 255) & ~(size_t)255;
		void* p = base + used;
		used += bytes;
		return p;
	}
};

constexpr int kTcTileCounters = 1024;

struct sslm_workspace_s {
	sslm_model_s* model = nullptr;
	sslm_config config{};
	int device = 0;
	int row_cap = 0;            // rows the device scratch can hold
	cudaStream_t stream = nullptr;
	uint8_t* d_scratch = nullptr;
	size_t scratch_bytes = 0;
	// pinned host staging, row_cap entries each
	sslm::RowDesc* h_rows = nullptr;
	sslm::RowSource* h_src = nullptr;
	sslm::RowSink* h_sink = nullptr;
	int32_t* h_status = nullptr;
	int32_t* h_done = nullptr;
	unsigned long long* h_sat = nullptr;
	unsigned long long* h_best = nullptr;
	// device mirrors
	sslm::RowDesc* d_rows = nullptr;
	sslm::RowSource* d_src = nullptr;
	sslm::RowSink* d_sink = nullptr;
	// head rows of constrained sequences: the mask page of the row's DFA state (else nullptr)
	const uint8_t** h_row_mask = nullptr;   // pinned
	const uint8_t** d_row_mask = nullptr;
	// carved row buffers (base pointers for row 0)
	sslm::RowBatch base{};
	size_t wide_ld = 0;
	// split-K scratch of the tensor-core linear kernel: parked partial accumulators and one
	// arrival counter per output tile (zero between launches)
	int32_t* d_tc_partial = nullptr;
	size_t tc_partial_bytes = 0;
	unsigned int* d_tc_counters = nullptr;
	int32_t* logit_capture = nullptr;   // host buffer for full logit rows (tests), or nullptr
	int32_t* d_logits = nullptr;
	cudaEvent_t ev0 = nullptr, ev1 = nullptr;
	float last_ms = 0.f;
	uint64_t launches = 0;
	bool launch_failed = false;   // a kernel launch of the current call was refused by the runtime
	// optional per-site trace (sslm_b200_trace): host buffer that receives one record per traced
	// site, layer and row of the calls that follow
	uint8_t* trace_buf = nullptr;
	size_t trace_cap = 0, trace_used = 0;
	// optional per-kernel-class timing (sslm_b200_profile): an event before every launch
	bool profile = false;
	std::vector<cudaEvent_t> prof_events;
	std::vector<int> prof_class;
	size_t prof_used = 0;
	double prof_ms[16] = {0};
	uint64_t prof_n[16] = {0};
};

// kernel classes reported by sslm_b200_profile_read
enum ProfClass {
	kProfBegin = 0, kProfLinQkv, kProfQkvPost, kProfAttention, kProfCtxFunnel, kProfLinO, kProfRes1,
	kProfLinGateUp, kProfAct, kProfLinDown, kProfRes2, kProfHead, kProfLoraU, kProfOther, kProfClasses
};

// what sslm_schema_lookup hands out: (model, index into its schema table)
struct sslm_schema_s {
	sslm_model_s* model = nullptr;
	uint32_t index = 0;
};

struct sslm_model_s {
	int device = 0;
	sslm::Dims dims{};
	sslm::ConfigView cfg{};
	uint8_t hash[32]{};
	DeviceArena arena;
	std::vector<sslm::LayerDev> h_layers;
	sslm::LayerDev* d_layers = nullptr;
	const int8_t* d_embed = nullptr;
	const int8_t* d_head = nullptr;
	const int8_t* d_final_gain = nullptr;
	sslm::Scale c_embed{}, c_final{};
	int32_t* d_cos = nullptr;
	int32_t* d_sin = nullptr;
	int32_t* d_silu = nullptr;
	std::atomic<uint32_t> live_refs{0};
	std::mutex default_ws_mutex;
	sslm_workspace_s* default_ws = nullptr;
	size_t weight_bytes = 0;
	// decode schemas (SCM1), if the artifact carries any: the parsed table on the host (the DFA
	// walk runs there, one lookup per produced token) and every state's mask page on the device
	sslm::SchemaTable schemas;
	std::vector<sslm_schema_s> schema_handles;
	uint8_t* d_schema_pages = nullptr;
};

struct sslm_kv_pool_s {
	sslm_model_s* model = nullptr;
	uint32_t block_count = 0;
	uint32_t blocks_free = 0;
	int pages_per_block = 0;
	sslm::KvPoolDev dev{};
	std::mutex mutex;
	std::vector<int32_t> free_pages;
	// holders per page: a frozen prefix's full pages are shared, read-only, by every sequence
	// that adopted it; a page returns to the free list when its last holder lets go
	std::vector<uint32_t> page_refs;
	std::atomic<uint32_t> live_refs{0};
};

struct sslm_adapter_s {
	sslm_model_s* base = nullptr;
	size_t artifact_bytes = 0;
	DeviceArena arena;
	sslm::LoraLayerDev* d_layers = nullptr;  // [layers]
	uint32_t rank = 0;
	std::atomic<uint32_t> live_refs{0};
};

struct sslm_seq_s {
	sslm_model_s* model = nullptr;
	sslm_kv_pool_s* pool = nullptr;
	uint8_t* d_state = nullptr;     // two (hidden codes + carried scale) slots
	size_t state_stride = 0, scale_off = 0;
	int cur = 0;                    // slot holding the committed stream
	std::vector<int32_t> pages;     // page ids in position order
	int32_t* d_pages = nullptr;     // device page table, pages_per_block entries
	int64_t context_length = 0;
	uint32_t layer_index = 0;
	int32_t current_token = -1;
	bool ready_for_logits = false;
	uint64_t kv_saturation_count = 0;
	sslm_adapter_s* adapter = nullptr;
	// constrained decoding: the bound schema (or nullptr), the DFA state the next token is
	// masked by, and how many tokens were admitted through schema-content prefill spans
	sslm_schema_s* bound_schema = nullptr;
	uint32_t dfa_walk_state = sslm::kDfaWalkUnused;
	int64_t forced_token_count = 0;
	std::mutex lifecycle_mutex;

	int8_t* hidden(int slot) const { return (int8_t*)(d_state + (size_t)slot * state_stride); }
	sslm::Scale* scale(int slot) const { return (sslm::Scale*)(d_state + (size_t)slot * state_stride + scale_off); }
};

// A prefix is a sequence that can be prefilled, then frozen and adopted by sequences
// (sslm_prefix_s, src/sslm_abi.cpp:1584-1694).
struct sslm_prefix_s {
	sslm_seq_s* inner = nullptr;
	bool frozen = false;
};
