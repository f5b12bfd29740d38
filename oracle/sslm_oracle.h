/* CPU oracle -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference's integer-only forward pass (the hot path
 * behind sslm_prefill / sslm_decode_step), written from the reference's algorithm
 * and checked against (a) the reference's own golden vectors and (b) the reference
 * library itself compiled from its sources (oracle/_ref). Only tests/, the smoke
 * check and the benchmark's cpu_baseline leg may call into this file; the CUDA
 * product never does.
 *
 * Parity status: PINNED -- tests/test_oracle_*.py compare every function here with
 * the reference's fixture headers (transcribed to tests/golden/) and with
 * oracle/_ref on seeded sweeps.
 *
 * Each function names the reference function it restates (path:line inside the
 * reference project).
 */
#ifndef SSLM_ORACLE_H
#define SSLM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct { int64_t m, e; } osc_scale;

/* status vocabulary: ordinals of the reference's SslmForwardStatus
 * (include/superslm/checked_chain_funnel.h:68-284) that this path can return */
enum {
	OSC_OK = 0,
	OSC_CHAIN_INPUT_OUT_OF_DOMAIN = 1,
	OSC_LOGIT_NARROWING_OVERFLOW = 2,
	OSC_IEXP_CONSTANTS_OUT_OF_DOMAIN = 3,
	OSC_CARRIED_SCALE_MANTISSA_OUT_OF_DOMAIN = 4,
	OSC_SILU_SCALE_OUT_OF_DOMAIN = 5,
	OSC_RDIVPOT_EXPONENT_OUT_OF_DOMAIN = 6,
	OSC_SOFTMAX_ROW_WIDTH_OUT_OF_DOMAIN = 7,
	OSC_TOKEN_ID_OUT_OF_RANGE = 8,
	OSC_POSITION_OVER_CAP = 9,
	OSC_KV_CAPACITY_EXHAUSTED = 11,
	OSC_SOFTMAX_KERNEL_REFUSED = 20,
	OSC_RESIDUAL_MAGNITUDE_OUT_OF_DOMAIN = 21,
	OSC_IEXP_SCALE_DERIVATION_OUT_OF_DOMAIN = 23,
	OSC_BIAS_RECONCILE_PRODUCT_OUT_OF_DOMAIN = 24
};

/* ---- scalar primitives ------------------------------------------------- */
int32_t osc_srdhm(int32_t a, int32_t b);                    /* src/intmath.cpp:230-236 */
int32_t osc_rdivpot32(int32_t x, int exponent);             /* src/intmath.cpp:245-256 */
int64_t osc_rdivpot64(int64_t x, int exponent);             /* src/intmath.cpp:258-263 */
int32_t osc_mbqm(int32_t x, int32_t mult, int shift);       /* src/intmath.cpp:265-268 */
int32_t osc_sat_lshift32(int32_t x, int shift);             /* src/intmath.cpp:270-276 */
void osc_normalize_scale(int64_t d_prime, int64_t* dn, int* s); /* src/intmath.cpp:296-301 */
int64_t osc_dyn_recip(int64_t dn);                          /* src/intmath.cpp:303-333 */
int8_t osc_requant_code_wide(int64_t x, int64_t r, int s);  /* src/intmath.cpp:476-490 */
int64_t osc_isqrt(int64_t n);                               /* src/intmath.cpp:502-524 */
int64_t osc_floor_div(int64_t a, int64_t b);                /* src/forward/forward_sites.cpp:399-408 */
void osc_rope_pair(int32_t x, int32_t y, int32_t c, int32_t s, int64_t* ox, int64_t* oy); /* src/intmath.cpp:782-792 */
int64_t osc_fold(int64_t acc, int32_t identity, int32_t mult, int32_t shift);      /* forward_sites.cpp:461-470 */
void osc_fold_matrix(const int64_t* acc, size_t m, size_t n, const int32_t* fold, int64_t* out);
/* BiasReconcileWide with q_B = 30 (src/intmath.cpp:397-418): 1 and *out = round_half_away(b * r_a / 2^(92 + e_a))
 * when the exponent is in [0,63] and the result fits int64, else 0 */
int osc_bias_reconcile(int64_t b, int64_t r_a, int64_t e_a, int64_t* out);
/* ApplyBiasReconcileRow (src/forward/forward_sites.cpp:1015-1036): status; acc untouched on refusal */
int osc_apply_bias_row(int64_t* acc, size_t n, const int64_t* bias, int64_t in_scale_m, int64_t in_scale_e);
int64_t osc_amp_fold(int64_t acc, int32_t identity, int32_t mult, int32_t exponent); /* forward_sites.cpp:472-481 */
osc_scale osc_combine(osc_scale a, osc_scale b);            /* src/forward/checked_chain_funnel.cpp:157-180 */
int64_t osc_landing_rescale(int64_t code, int64_t m_a, int64_t r_t, int64_t e_a, int64_t e_t,
                            uint64_t* sat_count, int* exceeded_int64); /* forward_sites.cpp:513-653 */
int32_t osc_silu_sigmoid_q15(const int32_t* table, int8_t code, int64_t m, int e); /* src/silu_lut.cpp:16-67 */
/* returns 0 ok, 1 bad coefficient, 2 negative shift, 3 not representable (src/intmath.cpp:702-778) */
int osc_iexp_scale_constants(int64_t m, int64_t e, int64_t* q_ln2, int64_t* q_b, int64_t* q_c);
/* IExpConstruct + IExpEvaluate (src/intmath.cpp:540-668) */
int osc_iexp(int64_t q, int64_t q_ln2, int64_t q_b, int64_t q_c, int64_t* z_out, int64_t* base_out,
             int64_t* value);
int osc_softmax_width_domain(int64_t q_b, int64_t q_c, size_t width); /* checked_chain_funnel.cpp:520-583 */
int osc_softmax_row_q15(const int64_t* scores, size_t width, int64_t q_ln2, int64_t q_b,
                        int64_t q_c, int64_t* out_probs);   /* src/intmath.cpp:796-901 */

/* ---- rows --------------------------------------------------------------- */
void osc_gemm(const int8_t* a, const int8_t* w, size_t m, size_t k, size_t n, int64_t* out); /* src/matmul.cpp:466-509 */
int osc_funnel(const int64_t* wide, size_t n, const osc_scale* incoming, size_t n_incoming,
               osc_scale site_constant, int8_t* out_codes, osc_scale* out_scale); /* checked_chain_funnel.cpp:257-364 */
int osc_rmsnorm_site(const int8_t* h, const int8_t* gain, size_t n, osc_scale c, int8_t* out,
                     osc_scale* out_scale);                 /* forward_sites.cpp:410-459 */
int osc_mlp_act_site(const int8_t* gate, osc_scale gs, const int8_t* up, osc_scale us, size_t n,
                     const int32_t* table, osc_scale c, int8_t* out, osc_scale* out_scale); /* :796-864 */
int osc_residual_site(const int8_t* branch, osc_scale bs, const int8_t* stream, osc_scale ss,
                      size_t n, osc_scale c, int8_t* out, osc_scale* out_scale); /* :871-989 */
int osc_embed_entry(int32_t token, int32_t vocab, const int8_t* embed, size_t hidden, osc_scale c,
                    int8_t* out, osc_scale* out_scale);     /* :763-787 */

/* ---- model / sequence --------------------------------------------------- */
typedef struct {
	const int8_t *a_w, *b_w;          /* lora_A [rank,in], lora_B [out,rank]; NULL = not adapted */
	const int32_t *u_fold, *d_fold;   /* [rank,3], [out,3] (identity, mult, exponent) */
} osc_lora_proj;

typedef struct {
	uint32_t rank;
	osc_lora_proj q, k, v, o, gate, up, down;
} osc_lora_layer;

typedef struct {
	const int8_t *q_w, *k_w, *v_w, *o_w, *gate_w, *up_w, *down_w;   /* [out,in] row-major */
	const int8_t *attn_gain, *mlp_gain;
	const int32_t *q_fold, *k_fold, *v_fold, *o_fold, *gate_fold, *up_fold, *down_fold; /* [out,3] */
	const int32_t *ctx_fold;                                        /* [heads,3] */
	const int64_t *k_recip, *v_recip;                               /* [kv_heads,3] (m_t,e_t,R_t) */
	const int64_t *softmax_khead;                                   /* [kv_heads,2] (m,e) */
	const int64_t *q_bias, *k_bias, *v_bias;                        /* BIA1 codes (Q30) or NULL: [hidden], [kv_hidden] x2 */
	osc_scale c_attn_norm, c_q, c_o, c_ctx, c_attn_res, c_mlp_norm, c_gate, c_up, c_act, c_down,
	    c_mlp_res;
} osc_layer;

typedef struct {
	uint32_t hidden, layers, heads, kv_heads, head_dim, inter, vocab, context_cap;
	const int8_t* embed;       /* [vocab, hidden]; also the tied head */
	const int8_t* head;        /* [vocab, hidden] */
	const int8_t* final_gain;
	osc_scale c_embed, c_final_norm;
	const int64_t *rope_cos, *rope_sin;  /* [context_cap, head_dim/2] */
	const int32_t* silu_table;           /* 1025 */
	const osc_layer* layer;              /* [layers] */
} osc_model;

typedef struct {
	int8_t* hidden_codes;      /* [hidden] */
	osc_scale hidden_scale;
	uint32_t layer_index;
	int64_t context_length;
	uint64_t kv_saturation_count;
	int8_t* kv;                /* canonical block [layer][K|V][kv_head][pos][head_dim] */
} osc_seq;

/* RunLayerLoopImpl, legacy K landing (forward_sites.cpp:1429-2014); lora may be NULL */
int osc_layer_loop(const osc_model* m, const osc_lora_layer* lora, osc_seq* s, uint32_t layer_budget);
/* PrefillWholeTokensImpl's admitted-token path: EmbedEntry per token +
 * RunLayerLoopChunkBatched (src/sslm_abi.cpp:1525-1556, forward_sites.cpp:2098-2401) */
int osc_prefill(const osc_model* m, const osc_lora_layer* lora, osc_seq* s, const int32_t* tokens,
                int32_t n);
/* final_norm + LogitsSite + argmax (src/sslm_abi.cpp:2275-2291, :2425);
 * out_logits may be NULL */
int osc_logits_argmax(const osc_model* m, const osc_seq* s, int32_t* out_logits, int32_t* out_token);
/* embed the token into the sequence's hidden state (src/sslm_abi.cpp:2231-2251) */
int osc_embed_into_seq(const osc_model* m, osc_seq* s, int32_t token);

/* per-site trace of one_layer into a caller buffer (record layout at the definition) */
void osc_trace_begin(uint8_t* buf, size_t capacity);
size_t osc_trace_end(void);

/* the primitives over arrays of operands (see sslm_oracle.c) */
void osc_sweep(int which, const int64_t* a, const int64_t* b, const int64_t* c, const int64_t* e, int64_t n,
               int64_t* out0, int64_t* out1, int64_t* out2);

#ifdef __cplusplus
}
#endif

#endif
