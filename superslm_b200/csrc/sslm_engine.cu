// Host side of the C ABI: artifact upload, paged KV pool, workspaces, sequences, and the
// launch schedules of sslm_prefill / sslm_decode_step. No arithmetic of the forward pass
// happens on the host; a missing or failing CUDA device surfaces as an error status.
#include "sslm_engine.h"

#include <algorithm>
#include <initializer_list>
#include <utility>
#include <cstdlib>
#include <cstring>
#include <new>
#include <unordered_set>

using namespace sslm;

namespace {

std::atomic<int> g_device{-1};
std::mutex g_seq_registry_mutex;
std::unordered_set<sslm_seq_s*> g_live_seqs;

int current_device_choice() {
	int d = g_device.load();
	if (d >= 0) return d;
	const char* env = getenv("SSLM_B200_DEVICE");
	return env ? atoi(env) : 0;
}

bool cuda_ok(cudaError_t e) { return e == cudaSuccess; }

bool is_aligned64(const void* p) { return ((uintptr_t)p % SSLM_ABI_ALIGNMENT_BYTES) == 0; }

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

sslm_status map_forward_status(int32_t st) {
	// MapForwardStatus, src/sslm_abi.cpp:1352-1370
	st = status_code(st);      // (the device packs the failing site and layer beside the code)
	if (st == kOk) return SSLM_OK;
	if (st == kSoftmaxKernelRefused) return SSLM_NUMERIC_STEP_REFUSED;
	// not a reference status: a bounded device-side wait of this implementation ran out
	if (st == kInternalWaitTimeout) return SSLM_ALLOCATION_FAILED;
	return SSLM_ARTIFACT_REJECTED;
}

Scale read_scale(const ArtifactView& v, const std::string& name, bool* ok) {
	const ConstEntry* e = v.composition(name);
	if (!e) {
		*ok = false;
		return Scale{0, 0};
	}
	return Scale{e->v[0], e->v[1]};
}

struct Upload {
	DeviceArena* arena;
	bool ok = true;
	void* put(const void* src, size_t bytes) {
		void* d = arena->take(bytes);
		if (arena->used > arena->size) {
			ok = false;
			return nullptr;
		}
		if (!cuda_ok(cudaMemcpy(d, src, bytes, cudaMemcpyHostToDevice))) ok = false;
		return d;
	}
};

}  // namespace

// ------------------------------------------------------------------------ model
extern "C" sslm_status sslm_b200_set_device(int ordinal) {
	int n = 0;
	if (!cuda_ok(cudaGetDeviceCount(&n)) || ordinal < 0 || ordinal >= n) return SSLM_INVALID_ARGUMENT;
	g_device.store(ordinal);
	return SSLM_OK;
}

extern "C" sslm_status sslm_model_map(const void* data, size_t size, sslm_model* out) {
	if (!out) return SSLM_INVALID_ARGUMENT;
	*out = nullptr;
	if (!data) return SSLM_INVALID_ARGUMENT;
	ArtifactView v;
	std::string err;
	try {
		if (!v.Open((const uint8_t*)data, size, &err)) return SSLM_ARTIFACT_REJECTED;
	} catch (const std::bad_alloc&) {
		return SSLM_ALLOCATION_FAILED;
	}
	const ConfigView& c = v.config();
	// what this implementation does not run: int16 KV, geometries outside the kernels'
	// vector widths
	if (c.kv_precision != 0) return SSLM_ARTIFACT_REJECTED;
	// Header flags bit 0 (fused wide K landing, RopeApplyPairWide) is deliberately not looked
	// at: the reference's sslm_prefill / sslm_decode_step always run the legacy landing
	// whatever the flag says (src/sslm_abi.cpp:1539 passes option_g_fused_k_landing = false,
	// :2256 calls the overload without it), and so does this library.
	if (c.hidden % 16 || c.inter % 16 || c.head_dim % 16 || c.head_dim > 128 ||
	    (128 % c.head_dim) != 0 || c.heads / c.kv_heads > 8 || c.kv_heads > 16)
		return SSLM_ARTIFACT_REJECTED;
	// int32 accumulation must be exact for the widest reduction (K * 127 * 128 < 2^31)
	if ((uint64_t)std::max(c.hidden, c.inter) > 131071) return SSLM_ARTIFACT_REJECTED;

	const int dev = current_device_choice();
	if (!cuda_ok(cudaSetDevice(dev))) return SSLM_ALLOCATION_FAILED;

	sslm_model_s* m = new (std::nothrow) sslm_model_s();
	if (!m) return SSLM_ALLOCATION_FAILED;
	m->device = dev;
	m->cfg = c;
	Dims& d = m->dims;
	d.hidden = c.hidden; d.layers = c.layers; d.heads = c.heads; d.kv_heads = c.kv_heads;
	d.head_dim = c.head_dim; d.inter = c.inter; d.vocab = c.vocab; d.context_cap = c.context_cap;
	d.kv_hidden = c.kv_heads * c.head_dim;
	d.qkv_rows = d.hidden + 2 * d.kv_hidden;
	memcpy(m->hash, v.integrity_hash(), 32);

	const size_t H = c.hidden, I = c.inter, KV = d.kv_hidden, L = c.layers;
	// arena size: weights + folds + tables + slack for 256-byte alignment of every piece
	size_t bytes = (size_t)c.vocab * H * (c.tie ? 1 : 2) + H;
	bytes += L * ((H + 2 * KV) * H + H * H + 2 * I * H + H * I + 2 * H);
	bytes += L * 12 * ((H + 2 * KV) + H + 2 * I + H + c.heads);
	bytes += L * (2 * c.kv_heads * 3 * 8 + c.kv_heads * 2 * 8);
	bytes += 2 * (size_t)c.context_cap * (c.head_dim / 2) * 4 + 1025 * 4 + L * sizeof(LayerDev);
	bytes += L * (H + 2 * KV) * 8;                       // q/k/v bias codes, when the artifact has them
	bytes += (L * 28 + 64) * 256;
	if (!cuda_ok(cudaMalloc((void**)&m->arena.base, bytes))) {
		delete m;
		return SSLM_ALLOCATION_FAILED;
	}
	m->arena.size = bytes;
	Upload up{&m->arena};

	auto fail = [&](sslm_status st) {
		cudaFree(m->arena.base);
		cudaFree(m->d_schema_pages);
		delete m;
		return st;
	};
	auto W = [&](const std::string& n, uint64_t rows, uint64_t cols) -> const TensorView* {
		const TensorView* t = v.weight(n);
		return (t && t->elem_count == rows * cols) ? t : nullptr;
	};
	auto F = [&](const std::string& n, uint64_t rows) -> const TensorView* {
		const TensorView* t = v.weight_scale(n);
		return (t && t->elem_count == rows * 3) ? t : nullptr;
	};
	// cat: upload several host pieces back to back as one device array
	auto cat = [&](std::initializer_list<std::pair<const void*, size_t>> parts) -> void* {
		size_t total = 0;
		for (auto& p : parts) total += p.second;
		uint8_t* dst = (uint8_t*)m->arena.take(total);
		if (m->arena.used > m->arena.size) { up.ok = false; return nullptr; }
		size_t off = 0;
		for (auto& p : parts) {
			if (!cuda_ok(cudaMemcpy(dst + off, p.first, p.second, cudaMemcpyHostToDevice))) up.ok = false;
			off += p.second;
		}
		return dst;
	};

	const TensorView* embed = W("embed", c.vocab, H);
	const TensorView* fgain = W("final_norm.gain", 1, H);
	if (!embed || !fgain) return fail(SSLM_ARTIFACT_REJECTED);
	m->d_embed = (const int8_t*)up.put(embed->data, embed->elem_count);
	if (c.tie) {
		m->d_head = m->d_embed;
	} else {
		const TensorView* head = W("lm_head", c.vocab, H);
		if (!head) return fail(SSLM_ARTIFACT_REJECTED);
		m->d_head = (const int8_t*)up.put(head->data, head->elem_count);
	}
	m->d_final_gain = (const int8_t*)up.put(fgain->data, H);
	bool ok = true;
	m->c_embed = read_scale(v, "embed", &ok);
	m->c_final = read_scale(v, "final_norm", &ok);
	if (!ok) return fail(SSLM_ARTIFACT_REJECTED);

	// RoPE tables: int64 Q30 in the artifact, consumed as int32 (RopeApplySite narrows them,
	// src/forward/forward_sites.cpp:753-754)
	const TensorView* cosv = v.rope("cos");
	const TensorView* sinv = v.rope("sin");
	if (!cosv || !sinv) return fail(SSLM_ARTIFACT_REJECTED);
	{
		const size_t n = (size_t)c.context_cap * (c.head_dim / 2);
		std::vector<int32_t> tmp(n);
		for (int pass = 0; pass < 2; ++pass) {
			const uint8_t* src = pass ? sinv->data : cosv->data;
			for (size_t i = 0; i < n; ++i) {
				int64_t x;
				memcpy(&x, src + 8 * i, 8);
				tmp[i] = (int32_t)x;
			}
			int32_t* dptr = (int32_t*)up.put(tmp.data(), n * 4);
			if (pass) m->d_sin = dptr; else m->d_cos = dptr;
		}
	}
	m->d_silu = (int32_t*)up.put(v.silu_table(), 1025 * 4);

	m->h_layers.resize(L);
	for (size_t l = 0; l < L; ++l) {
		const std::string p = "layer" + std::to_string(l) + ".";
		const TensorView *qw = W(p + "q_proj", H, H), *kw = W(p + "k_proj", KV, H), *vw = W(p + "v_proj", KV, H),
		                 *ow = W(p + "o_proj", H, H), *gw = W(p + "gate_proj", I, H), *uw = W(p + "up_proj", I, H),
		                 *dw = W(p + "down_proj", H, I), *ag = W(p + "attn_norm.gain", 1, H),
		                 *mg = W(p + "mlp_norm.gain", 1, H);
		const TensorView *qf = F(p + "q_proj", H), *kf = F(p + "k_proj", KV), *vf = F(p + "v_proj", KV),
		                 *of = F(p + "o_proj", H), *gf = F(p + "gate_proj", I), *uf = F(p + "up_proj", I),
		                 *df = F(p + "down_proj", H), *cf = F(p + "ctx_fold", c.heads);
		if (!qw || !kw || !vw || !ow || !gw || !uw || !dw || !ag || !mg || !qf || !kf || !vf || !of || !gf ||
		    !uf || !df || !cf)
			return fail(SSLM_ARTIFACT_REJECTED);
		LayerDev& ld = m->h_layers[l];
		ld.w_qkv = (const int8_t*)cat({{qw->data, H * H}, {kw->data, KV * H}, {vw->data, KV * H}});
		ld.w_o = (const int8_t*)up.put(ow->data, H * H);
		ld.w_gu = (const int8_t*)cat({{gw->data, I * H}, {uw->data, I * H}});
		ld.w_down = (const int8_t*)up.put(dw->data, H * I);
		ld.f_qkv = (const int32_t*)cat({{qf->data, H * 12}, {kf->data, KV * 12}, {vf->data, KV * 12}});
		ld.f_o = (const int32_t*)up.put(of->data, H * 12);
		ld.f_gu = (const int32_t*)cat({{gf->data, I * 12}, {uf->data, I * 12}});
		ld.f_down = (const int32_t*)up.put(df->data, H * 12);
		ld.f_ctx = (const int32_t*)up.put(cf->data, (size_t)c.heads * 12);
		ld.g_attn = (const int8_t*)up.put(ag->data, H);
		ld.g_mlp = (const int8_t*)up.put(mg->data, H);
		std::vector<int64_t> kr(c.kv_heads * 3), vr(c.kv_heads * 3), sk(c.kv_heads * 2);
		for (uint32_t h = 0; h < c.kv_heads; ++h) {
			const ConstEntry* ke = v.kv_recip(p + "k_head" + std::to_string(h));
			const ConstEntry* ve = v.kv_recip(p + "v_head" + std::to_string(h));
			const ConstEntry* se = v.composition(p + "softmax_khead" + std::to_string(h));
			if (!ke || !ve || !se) return fail(SSLM_ARTIFACT_REJECTED);
			for (int k = 0; k < 3; ++k) { kr[3 * h + k] = ke->v[k]; vr[3 * h + k] = ve->v[k]; }
			sk[2 * h] = se->v[0]; sk[2 * h + 1] = se->v[1];
		}
		ld.k_recip = (const int64_t*)up.put(kr.data(), kr.size() * 8);
		ld.v_recip = (const int64_t*)up.put(vr.data(), vr.size() * 8);
		ld.sm_khead = (const int64_t*)up.put(sk.data(), sk.size() * 8);
		// BIA1 (layer_marshal.h:247-253): each of the three is optional on its own
		const TensorView *qb = v.bias(p + "q_proj"), *kb = v.bias(p + "k_proj"), *vb = v.bias(p + "v_proj");
		if ((qb && qb->elem_count != H) || (kb && kb->elem_count != KV) || (vb && vb->elem_count != KV))
			return fail(SSLM_ARTIFACT_REJECTED);
		ld.b_q = qb ? (const int64_t*)up.put(qb->data, H * 8) : nullptr;
		ld.b_k = kb ? (const int64_t*)up.put(kb->data, KV * 8) : nullptr;
		ld.b_v = vb ? (const int64_t*)up.put(vb->data, KV * 8) : nullptr;
		ld.c_attn_norm = read_scale(v, p + "attn_norm", &ok);
		ld.c_q = read_scale(v, p + "q_proj", &ok);
		ld.c_o = read_scale(v, p + "o_proj", &ok);
		ld.c_ctx = read_scale(v, p + "attn_ctx", &ok);
		ld.c_attn_res = read_scale(v, p + "attn_residual", &ok);
		ld.c_mlp_norm = read_scale(v, p + "mlp_norm", &ok);
		ld.c_gate = read_scale(v, p + "gate_proj", &ok);
		ld.c_up = read_scale(v, p + "up_proj", &ok);
		ld.c_act = read_scale(v, p + "mlp_act", &ok);
		ld.c_down = read_scale(v, p + "down_proj", &ok);
		ld.c_mlp_res = read_scale(v, p + "mlp_residual", &ok);
		if (!ok) return fail(SSLM_ARTIFACT_REJECTED);
	}
	m->d_layers = (LayerDev*)up.put(m->h_layers.data(), L * sizeof(LayerDev));
	if (!up.ok) return fail(SSLM_ALLOCATION_FAILED);
	// decode schemas (src/sslm_abi.cpp:1196-1218): a malformed SCM1 section refuses the artifact
	if (v.has(kSecSchemaMasks)) {
		uint64_t ssize = 0;
		const uint8_t* sdata = v.section_data(kSecSchemaMasks, &ssize);
		bool sok = false;
		try {
			sok = sdata != nullptr && m->schemas.parse(sdata, ssize, c.vocab);
			if (sok) {
				m->schema_handles.resize(m->schemas.entries.size());
				for (size_t i = 0; i < m->schema_handles.size(); ++i) m->schema_handles[i] = sslm_schema_s{m, (uint32_t)i};
			}
		} catch (const std::bad_alloc&) {
			return fail(SSLM_ALLOCATION_FAILED);
		}
		if (!sok) return fail(SSLM_ARTIFACT_REJECTED);
		const size_t pb = m->schemas.page_bytes;
		if (!cuda_ok(cudaMalloc((void**)&m->d_schema_pages, m->schemas.total_pages() * pb))) return fail(SSLM_ALLOCATION_FAILED);
		for (const SchemaEntry& e : m->schemas.entries) {
			if (!cuda_ok(cudaMemcpy(m->d_schema_pages + e.device_page0 * pb, m->schemas.pages(e), (size_t)e.states * pb,
			                        cudaMemcpyHostToDevice))) {
				return fail(SSLM_ALLOCATION_FAILED);
			}
		}
	}
	m->weight_bytes = m->arena.used;
	if (!cuda_ok(rows_configure(d)) || !cuda_ok(attn_configure(d))) return fail(SSLM_ARTIFACT_REJECTED);
	cudaDeviceSynchronize();
	*out = m;
	return SSLM_OK;
}

static void destroy_workspace(sslm_workspace_s* ws);

extern "C" sslm_status sslm_model_unmap(sslm_model model) {
	if (!model) return SSLM_INVALID_ARGUMENT;
	if (model->live_refs.load(std::memory_order_acquire) != 0) return SSLM_MODEL_HAS_LIVE_SEQUENCES;
	cudaSetDevice(model->device);
	if (model->default_ws) destroy_workspace(model->default_ws);
	cudaFree(model->arena.base);
	cudaFree(model->d_schema_pages);
	delete model;
	return SSLM_OK;
}

extern "C" size_t sslm_b200_model_device_bytes(sslm_model model) { return model ? model->weight_bytes : 0; }

// ------------------------------------------------------------------ sizing + pool
extern "C" size_t sslm_kv_block_size(sslm_model model) {
	if (!model) return 0;
	const ConfigView& c = model->cfg;
	return (size_t)c.layers * c.context_cap * c.kv_heads * c.head_dim * 2;
}

extern "C" size_t sslm_kv_pool_overhead_size(sslm_model model, uint32_t block_count) {
	if (!model) return 0;
	return (size_t)block_count * 8 + 32;
}

extern "C" sslm_status sslm_kv_pool_create(sslm_model model, void* buf, size_t buf_size,
                                           uint32_t block_count, sslm_kv_pool* out) {
	if (!out) return SSLM_INVALID_ARGUMENT;
	*out = nullptr;
	if (!model || !buf || block_count == 0) return SSLM_INVALID_ARGUMENT;
	const size_t block = sslm_kv_block_size(model);
	if (block == 0 || block_count > SIZE_MAX / block) return SSLM_INVALID_ARGUMENT;
	const size_t required = block * block_count + sslm_kv_pool_overhead_size(model, block_count);
	if (buf_size < required) return SSLM_BUFFER_TOO_SMALL;
	if (!is_aligned64(buf)) return SSLM_MISALIGNED_BUFFER;
	if (!cuda_ok(cudaSetDevice(model->device))) return SSLM_ALLOCATION_FAILED;
	sslm_kv_pool_s* p = new (std::nothrow) sslm_kv_pool_s();
	if (!p) return SSLM_ALLOCATION_FAILED;
	const Dims& d = model->dims;
	p->model = model;
	p->block_count = block_count;
	p->blocks_free = block_count;
	p->pages_per_block = (d.context_cap + kPageTokens - 1) / kPageTokens;
	p->dev.num_pages = (int64_t)p->pages_per_block * block_count;
	const size_t bytes = (size_t)d.layers * d.kv_heads * 2 * p->dev.num_pages * kPageTokens * d.head_dim;
	if (!cuda_ok(cudaMalloc((void**)&p->dev.base, bytes))) {
		delete p;
		return SSLM_ALLOCATION_FAILED;
	}
	try {
		p->free_pages.reserve(p->dev.num_pages);
		for (int64_t i = p->dev.num_pages - 1; i >= 0; --i) p->free_pages.push_back((int32_t)i);
		p->page_refs.assign((size_t)p->dev.num_pages, 0u);
	} catch (const std::bad_alloc&) {
		cudaFree(p->dev.base);
		delete p;
		return SSLM_ALLOCATION_FAILED;
	}
	*out = p;
	return SSLM_OK;
}

extern "C" sslm_status sslm_kv_pool_destroy(sslm_kv_pool pool) {
	if (!pool) return SSLM_INVALID_ARGUMENT;
	if (pool->live_refs.load(std::memory_order_acquire) != 0) return SSLM_POOL_HAS_LIVE_HANDLES;
	cudaSetDevice(pool->model->device);
	cudaFree(pool->dev.base);
	delete pool;
	return SSLM_OK;
}

// ---------------------------------------------------------------------- workspace
namespace {

bool config_ok(const sslm_model_s* model, const sslm_config* c) {
	if (!model || !c) return false;
	if (c->max_batch < 1 || c->max_chunk_budget < 1 || c->max_layer_budget < 1) return false;
	if ((uint32_t)c->max_layer_budget > model->cfg.layers) return false;
	return c->reserved == 0;
}

// Carve the per-row buffers for `rows` rows out of one device allocation.
size_t carve(const Dims& d, int rows, uint8_t* basep, RowBatch* b, size_t* wide_ld_out, int32_t** d_logits) {
	size_t off = 0;
	auto take = [&](size_t bytes) -> uint8_t* {
		off = align_up(off, 256);
		uint8_t* p = basep ? basep + off : nullptr;
		off += bytes;
		return p;
	};
	const size_t R = rows, H = d.hidden, I = d.inter;
	const size_t wide_ld = std::max<size_t>(d.qkv_rows, 2 * I);
	b->x = (int8_t*)take(R * H);      b->xs = (Scale*)take(R * sizeof(Scale));
	b->a = (int8_t*)take(R * H);      b->as = (Scale*)take(R * sizeof(Scale));
	b->nrm = (int8_t*)take(R * H);    b->ns = (Scale*)take(R * sizeof(Scale));
	b->wide = take(R * wide_ld * 8);
	b->qrot = (int8_t*)take(R * H);
	b->ctxw = (int32_t*)take(R * H * 4);
	b->ctx = (int8_t*)take(R * H);    b->cs = (Scale*)take(R * sizeof(Scale));
	b->act = (int8_t*)take(R * I);    b->acts = (Scale*)take(R * sizeof(Scale));
	b->rowmax = (unsigned long long*)take(R * 4 * 8);
	b->smc = (SoftmaxConsts*)take(R * d.kv_heads * sizeof(SoftmaxConsts));
	b->status = (int32_t*)take(R * 4);
	b->done = (int32_t*)take(R * 4);
	b->sat = (unsigned long long*)take(R * 8);
	b->sat_layer = (uint32_t*)take(R * d.layers * 4);
	b->sat_ld = (int)d.layers;
	b->lora_u = (int8_t*)take(R * 3 * kMaxLoraRank);
	b->best = (unsigned long long*)take(R * 8);
	*d_logits = (int32_t*)take((size_t)d.vocab * 4 * std::min<size_t>(R, 64));
	*wide_ld_out = wide_ld;
	return align_up(off, 256);
}

sslm_workspace_s* create_workspace(sslm_model_s* model, const sslm_config& cfg, int rows) {
	if (!cuda_ok(cudaSetDevice(model->device))) return nullptr;
	sslm_workspace_s* w = new (std::nothrow) sslm_workspace_s();
	if (!w) return nullptr;
	w->model = model;
	w->config = cfg;
	w->device = model->device;
	w->row_cap = rows;
	RowBatch tmp{};
	size_t ld;
	int32_t* dl;
	w->scratch_bytes = carve(model->dims, rows, nullptr, &tmp, &ld, &dl);
	bool ok = cuda_ok(cudaMalloc((void**)&w->d_scratch, w->scratch_bytes));
	ok = ok && cuda_ok(cudaMemset(w->d_scratch, 0, w->scratch_bytes));
	ok = ok && cuda_ok(cudaStreamCreateWithFlags(&w->stream, cudaStreamNonBlocking));
	ok = ok && cuda_ok(cudaMallocHost((void**)&w->h_rows, rows * sizeof(RowDesc)));
	ok = ok && cuda_ok(cudaMallocHost((void**)&w->h_src, rows * sizeof(RowSource)));
	ok = ok && cuda_ok(cudaMallocHost((void**)&w->h_sink, rows * sizeof(RowSink)));
	ok = ok && cuda_ok(cudaMallocHost((void**)&w->h_status, rows * 4));
	ok = ok && cuda_ok(cudaMallocHost((void**)&w->h_done, rows * 4));
	ok = ok && cuda_ok(cudaMallocHost((void**)&w->h_sat, rows * 8));
	ok = ok && cuda_ok(cudaMallocHost((void**)&w->h_best, rows * 8));
	ok = ok && cuda_ok(cudaMalloc((void**)&w->d_rows, rows * sizeof(RowDesc)));
	ok = ok && cuda_ok(cudaMalloc((void**)&w->d_src, rows * sizeof(RowSource)));
	ok = ok && cuda_ok(cudaMalloc((void**)&w->d_sink, rows * sizeof(RowSink)));
	ok = ok && cuda_ok(cudaMallocHost((void**)&w->h_row_mask, rows * sizeof(void*)));
	ok = ok && cuda_ok(cudaMalloc((void**)&w->d_row_mask, rows * sizeof(void*)));
	ok = ok && cuda_ok(cudaEventCreate(&w->ev0)) && cuda_ok(cudaEventCreate(&w->ev1));
	if (ok && rows > 8) {
		// K slices times tiles never exceeds the SM count, and a tile is at most 256 x 64
		// accumulators, so 16 MiB holds every case the tensor-core path picks
		w->tc_partial_bytes = (size_t)16 << 20;
		ok = cuda_ok(cudaMalloc((void**)&w->d_tc_partial, w->tc_partial_bytes));
		ok = ok && cuda_ok(cudaMalloc((void**)&w->d_tc_counters, kTcTileCounters * sizeof(unsigned int)));
		ok = ok && cuda_ok(cudaMemset(w->d_tc_counters, 0, kTcTileCounters * sizeof(unsigned int)));
	}
	if (!ok) {
		destroy_workspace(w);
		return nullptr;
	}
	carve(model->dims, rows, w->d_scratch, &w->base, &w->wide_ld, &w->d_logits);
	w->base.wide_ld = (int)w->wide_ld;
	return w;
}

}  // namespace

static void destroy_workspace(sslm_workspace_s* w) {
	if (!w) return;
	cudaSetDevice(w->device);
	if (w->stream) cudaStreamSynchronize(w->stream);
	cudaFree(w->d_scratch);
	cudaFree(w->d_tc_partial);
	cudaFree(w->d_tc_counters);
	cudaFree(w->d_rows);
	cudaFree(w->d_src);
	cudaFree(w->d_sink);
	cudaFree(w->d_row_mask);
	cudaFreeHost(w->h_row_mask);
	cudaFreeHost(w->h_rows);
	cudaFreeHost(w->h_src);
	cudaFreeHost(w->h_sink);
	cudaFreeHost(w->h_status);
	cudaFreeHost(w->h_done);
	cudaFreeHost(w->h_sat);
	cudaFreeHost(w->h_best);
	if (w->ev0) cudaEventDestroy(w->ev0);
	if (w->ev1) cudaEventDestroy(w->ev1);
	for (cudaEvent_t e : w->prof_events) cudaEventDestroy(e);
	if (w->stream) cudaStreamDestroy(w->stream);
	delete w;
}

extern "C" size_t sslm_workspace_size(sslm_model model, const sslm_config* config) {
	if (!config_ok(model, config)) return 0;
	// the host-side reservation the reference's layout would need (src/sslm_abi.cpp:852-933):
	// header, per-sequence status, staged tokens, embed codes, final codes, logits rows
	const ConfigView& c = model->cfg;
	size_t n = 64;
	n = align_up(n, 64) + (size_t)config->max_batch * 8;
	n = align_up(n, 64) + (size_t)config->max_chunk_budget * 4;
	n = align_up(n, 64) + (size_t)config->max_chunk_budget * c.hidden;
	n = align_up(n, 64) + c.hidden;
	n = align_up(n, 64) + (size_t)c.vocab * 8;
	n = align_up(n, 64) + (size_t)c.vocab * 4;
	n = align_up(n, 64) + (size_t)c.vocab * 4;
	n = align_up(n, 64) + (size_t)c.hidden * 8;
	return n;
}

extern "C" sslm_status sslm_workspace_create(sslm_model model, const sslm_config* config, void* buf,
                                             size_t buf_size, sslm_workspace* out) {
	if (!out) return SSLM_INVALID_ARGUMENT;
	*out = nullptr;
	if (!config_ok(model, config) || !buf) return SSLM_INVALID_ARGUMENT;
	if (buf_size < sslm_workspace_size(model, config)) return SSLM_BUFFER_TOO_SMALL;
	if (!is_aligned64(buf)) return SSLM_MISALIGNED_BUFFER;
	const int rows = std::max(2 * config->max_batch, config->max_chunk_budget);
	sslm_workspace_s* w = create_workspace(model, *config, rows);
	if (!w) return SSLM_ALLOCATION_FAILED;
	*out = w;
	return SSLM_OK;
}

extern "C" sslm_status sslm_workspace_destroy(sslm_workspace ws) {
	if (!ws) return SSLM_INVALID_ARGUMENT;
	destroy_workspace(ws);
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_last_call_ms(sslm_workspace ws, float* ms, uint64_t* launches) {
	if (!ws) return SSLM_INVALID_ARGUMENT;
	if (ms) *ms = ws->last_ms;
	if (launches) *launches = ws->launches;
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_tc_stats(uint64_t* launches, uint64_t* refusals, int32_t* last_reason) {
	unsigned long long l = 0, r = 0;
	int why = 0;
	tc_stats(&l, &r, &why);
	if (launches) *launches = l;
	if (refusals) *refusals = r;
	if (last_reason) *last_reason = why;
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_tc_variant_counts(uint64_t* counts, int32_t n) {
	if (!counts || n < 1) return SSLM_INVALID_ARGUMENT;
	unsigned long long c[8] = {0};
	tc_variant_counts(c, 8);
	for (int i = 0; i < n; ++i) counts[i] = i < 8 ? c[i] : 0;
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_trace(sslm_workspace ws, void* buf, size_t capacity, size_t* used) {
	if (!ws) return SSLM_INVALID_ARGUMENT;
	if (used) *used = ws->trace_used;          // what the trace that ends (or continues) here holds
	if (!cuda_ok(cudaSetDevice(ws->device))) return SSLM_ALLOCATION_FAILED;
	cudaStreamSynchronize(ws->stream);
	ws->trace_buf = (uint8_t*)buf;
	ws->trace_cap = buf ? capacity : 0;
	ws->trace_used = 0;
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_debug_withhold_tc_load(int32_t launches) {
	if (launches < 0 || launches > 16) return SSLM_INVALID_ARGUMENT;
	tc_debug_withhold(launches);
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_set_attention_splits(int32_t splits) {
	if (splits < 0 || splits > 16) return SSLM_INVALID_ARGUMENT;
	attn_force_splits(splits);
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_profile(sslm_workspace ws, int32_t enable) {
	if (!ws) return SSLM_INVALID_ARGUMENT;
	ws->profile = enable != 0;
	ws->prof_used = 0;
	for (int i = 0; i < 16; ++i) { ws->prof_ms[i] = 0; ws->prof_n[i] = 0; }
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_profile_read(sslm_workspace ws, double* ms, uint64_t* launches, int32_t n) {
	if (!ws || !ms || !launches || n < 0) return SSLM_INVALID_ARGUMENT;
	for (int i = 0; i < n && i < kProfClasses; ++i) { ms[i] = ws->prof_ms[i]; launches[i] = ws->prof_n[i]; }
	return SSLM_OK;
}

extern "C" sslm_status sslm_b200_capture_logits(sslm_workspace ws, int32_t* host_rows) {
	if (!ws) return SSLM_INVALID_ARGUMENT;
	ws->logit_capture = host_rows;
	return SSLM_OK;
}

#include "sslm_engine_run.inc"
#include "sslm_engine_misc.inc"
