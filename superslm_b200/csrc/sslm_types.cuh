// Device-side data layout of a mapped model, an adapter, and one batch of rows.
//
// A "row" is one token of one sequence moving through the layers: a decode step over
// n sequences is n rows, a prefill chunk of c tokens is c rows. Every kernel works on
// a RowBatch; nothing in a kernel knows whether its rows came from prefill or decode.
#pragma once
#include <stdint.h>

#include "sslm_int.cuh"

namespace sslm {

constexpr int kPageTokens = 16;       // KV page = 16 token positions of one (layer, kv head, K|V)
constexpr int kMaxLoraRank = 64;
constexpr int kRowThreads = 256;     // block size of the per-row kernels

struct LoraProjDev {
	const int8_t* a;      // [rank, in]   lora_A
	const int8_t* b;      // [out, rank]  lora_B
	const int32_t* uf;    // [rank, 3]    (identity, mult, exponent) on u = A x
	const int32_t* df;    // [out, 3]     (identity, mult, exponent) on delta = B u
};
// projection order inside a layer's adapter record
enum LoraSlot { kLoraQ = 0, kLoraK, kLoraV, kLoraO, kLoraGate, kLoraUp, kLoraDown, kLoraSlots };
struct LoraLayerDev {
	uint32_t rank;
	uint32_t pad;
	LoraProjDev p[kLoraSlots];
};

struct LayerDev {
	const int8_t* w_qkv;   // [hidden + 2*kv_hidden, hidden]  rows: q, then k, then v
	const int8_t* w_o;     // [hidden, hidden]
	const int8_t* w_gu;    // [2*inter, hidden]               rows: gate, then up
	const int8_t* w_down;  // [hidden, inter]
	const int32_t* f_qkv;  // [rows,3] (identity, mult, shift), same row order as the weights
	const int32_t* f_o;
	const int32_t* f_gu;
	const int32_t* f_down;
	const int32_t* f_ctx;  // [heads,3]
	const int8_t* g_attn;  // [hidden] RMSNorm gains (int8, widened on use)
	const int8_t* g_mlp;
	const int64_t* k_recip;   // [kv_heads][3] (m_t, e_t, R_t)
	const int64_t* v_recip;
	const int64_t* sm_khead;  // [kv_heads][2] (m, e)
	const int64_t* b_q;       // [hidden]     q/k/v bias codes (BIA1, Q30), each nullptr when absent
	const int64_t* b_k;       // [kv_hidden]
	const int64_t* b_v;       // [kv_hidden]
	Scale c_attn_norm, c_q, c_o, c_ctx, c_attn_res, c_mlp_norm, c_gate, c_up, c_act, c_down, c_mlp_res;
};

struct Dims {
	int hidden, layers, heads, kv_heads, head_dim, inter, vocab, context_cap;
	int kv_hidden;   // kv_heads * head_dim
	int qkv_rows;    // hidden + 2*kv_hidden
};

// Paged KV pool: [layer][kv_head][K|V][page] int8 pages of 16 positions. A K page is
// [16][head_dim] (one row per position); a V page is stored transposed, [head_dim][16],
// so that 4 consecutive positions of one channel are one 32-bit word: the K-major operand
// the tensor cores want for P.V. A page id names the same slot in every (layer, kv head,
// K|V) plane, so one page table serves all layers.
struct KvPoolDev {
	int8_t* base;
	int64_t num_pages;
};
__host__ __device__ __forceinline__ int64_t kv_plane_offset(const Dims& d, const KvPoolDev& p, int layer,
                                                            int kv_head, int is_v) {
	return ((((int64_t)layer * d.kv_heads + kv_head) * 2 + is_v) * p.num_pages) *
	       (int64_t)(kPageTokens * d.head_dim);
}

struct RowDesc {
	const int32_t* pages;       // page table of the row's sequence (device)
	const LoraLayerDev* lora;   // the sequence's adapter, per-layer array, or nullptr
	int32_t pos;                // position this token occupies
	int32_t token;              // token id to embed when the row starts a token
};

// Where in the reference's program order a row was refused. A row's status word holds the
// reference status in bits 0..7, the site in bits 8..15 and the layer index + 1 in bits 16..31;
// any non-zero word means "refused". The host needs the place twice: a decode step that fails in
// a later layer of its budget has committed the layers before it (the reference commits layer by
// layer, src/forward/forward_sites.cpp:1989-2009), and when several rows of a prefill chunk fail,
// the reference reports the failure that comes first in ITS loop order (layer, stage, token).
enum Site : int32_t {
	kSiteEmbed = 0, kSiteAttnNorm, kSiteQ, kSiteKv, kSiteRope, kSiteSoftmaxConsts, kSiteSoftmax, kSiteCtx, kSiteO,
	kSiteAttnRes, kSiteMlpNorm, kSiteGate, kSiteUp, kSiteSilu, kSiteAct, kSiteDown, kSiteMlpRes, kSiteFinalNorm,
	kSiteLogits
};
__host__ __device__ __forceinline__ int32_t pack_status(int32_t st, int site, int layer) {
	return st == 0 ? 0 : (st & 0xFF) | (site << 8) | ((layer + 1) << 16);
}
__host__ __device__ __forceinline__ int32_t status_code(int32_t word) { return word & 0xFF; }

struct SoftmaxConsts {
	IExpConsts c;
	int64_t peak;
};

// All per-row working buffers of one call (device pointers into a workspace arena).
struct RowBatch {
	int m;                       // rows
	const RowDesc* rows;
	int8_t* x;  Scale* xs;       // residual stream in / out            [m, hidden]
	int8_t* a;  Scale* as;       // stream after the attention residual [m, hidden]
	int8_t* nrm; Scale* ns;      // RMSNorm output                      [m, hidden]
	void* wide;                  // projection accumulators after fold  [m, wide_ld] int32 (int64 with adapters)
	int wide_ld;
	int wide64;                  // 1: wide holds int64 (some row has an adapter)
	int8_t* qrot;                // rotated q codes                     [m, hidden]
	int32_t* ctxw;               // folded attention context            [m, hidden]
	int8_t* ctx; Scale* cs;      // attention context codes             [m, hidden]
	int8_t* act; Scale* acts;    // SwiGLU output codes                 [m, inter]
	unsigned long long* rowmax;  // [m][4] max |x| slots: 0 q/o/down, 1 gate, 2 up, 3 ctx (self-clearing)
	SoftmaxConsts* smc;          // [m][kv_heads]
	int32_t* status;             // [m] first failing site's packed status word (pack_status), 0 = ok
	int32_t* done;               // [m] layers this call completed for the row
	int layer;                   // index of the layer the current launch works on
	unsigned long long* sat;     // [m] K/V landing saturation events of this call
	uint32_t* sat_layer;         // [m][sat_ld] the same events per layer (a refused prefill chunk counts those the
	int sat_ld;                  //             reference's walk had reached); sat_ld = layers
	int8_t* lora_u;              // [m][3][kMaxLoraRank] clamped u = fold(A x) per projection slot of the current GEMM
	unsigned long long* best;    // [m] packed (logit, index) argmax key
	int32_t* logits;             // optional [m, vocab] dump, or nullptr
};

}  // namespace sslm
