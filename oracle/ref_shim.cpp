// Test infrastructure, not product code.
//
// extern "C" doors onto the reference library's internal C++ functions so that
// tests can call the reference's own arithmetic through ctypes. This file adds no
// arithmetic of its own: every function forwards to the reference function named
// in its body. It is compiled together with the reference's sources (see the
// Makefile beside it) into oracle/_ref/libsslm_ref.so. The reference's public
// sslm_* C ABI (src/sslm_abi.cpp) is exported by that library as it stands.
#include <cstddef>
#include <cstdint>
#include <span>

#include "superslm/checked_chain_funnel.h"
#include "superslm/forward_sites.h"
#include "superslm/intmath.h"
#include "superslm/matmul.h"
#include "superslm/silu_lut.h"
#include "superslm/silu_lut_canonical.h"

using namespace superslm;

extern "C" {

int32_t refshim_srdhm(int32_t a, int32_t b) { return SaturatingRoundingDoublingHighMul(a, b); }
int32_t refshim_rdivpot32(int32_t x, int e) { return RoundingDivideByPOT(x, e); }
int64_t refshim_rdivpot64(int64_t x, int e) { return RoundingDivideByPOT(x, e); }
int32_t refshim_mbqm(int32_t x, int32_t m, int s) { return MultiplyByQuantizedMultiplier(x, m, s); }
int32_t refshim_sat_lshift32(int32_t x, int s) { return SaturatingLeftShift32(x, s); }
void refshim_normalize_scale(int64_t d_prime, int64_t* dn, int* s) {
	const NormalizedScale n = NormalizeScale(d_prime);
	*dn = n.dn;
	*s = n.s;
}
int64_t refshim_dyn_recip(int64_t dn) { return DynamicScaleReciprocal(dn); }
int8_t refshim_requant_code_wide(int64_t x, int64_t r, int s) { return RequantTokenCodeWide(x, r, s); }
int64_t refshim_isqrt(int64_t n) { return ISqrt(n); }
int64_t refshim_floor_div(int64_t a, int64_t b) { return FloorDivI64(a, b); }
void refshim_rope_pair(int32_t x, int32_t y, int32_t c, int32_t s, int64_t* ox, int64_t* oy) {
	const RopePair p = RopeApplyPair(x, y, c, s);
	*ox = p.x;
	*oy = p.y;
}
int64_t refshim_fold(int64_t acc, int32_t id, int32_t mult, int32_t shift) {
	return ApplyWeightScaleFold(acc, id, mult, shift);
}
int64_t refshim_amp_fold(int64_t acc, int32_t id, int32_t mult, int32_t exponent) {
	return ApplyAmplifyingWeightScaleFold(acc, id, mult, exponent);
}
void refshim_combine(int64_t am, int64_t ae, int64_t bm, int64_t be, int64_t* om, int64_t* oe) {
	const CarriedScale c = CombineCarriedScale(CarriedScale{am, ae}, CarriedScale{bm, be});
	*om = c.m;
	*oe = c.e;
}
int64_t refshim_landing_rescale(int64_t code, int64_t m_a, int64_t r_t, int64_t e_a, int64_t e_t,
                                uint64_t* sat_count, int* exceeded_int64) {
	bool ex = false;
	const int64_t r = LandingRescale(code, m_a, r_t, e_a, e_t, sat_count, &ex);
	if (exceeded_int64) *exceeded_int64 = ex ? 1 : 0;
	return r;
}
int32_t refshim_silu_sigmoid_q15(const int32_t* table, int8_t code, int64_t m, int e) {
	return SiluSigmoidQ15(table, code, m, e);
}
const int32_t* refshim_silu_canonical_table(void) { return kSiluLutCanonicalTable; }
int refshim_iexp_scale_constants(int64_t m, int64_t e, int64_t* q_ln2, int64_t* q_b, int64_t* q_c) {
	return static_cast<int>(
	    IExpScaleConstants(m, e, kIExpLn2Q, 30, kIExpBQ, 30, kIExpCaQ, 30, q_ln2, q_b, q_c));
}
void refshim_iexp_coefficients(int64_t* ln2_q, int64_t* b_q, int64_t* ca_q) {
	*ln2_q = kIExpLn2Q;
	*b_q = kIExpBQ;
	*ca_q = kIExpCaQ;
}
int refshim_softmax_width_domain(int64_t q_b, int64_t q_c, size_t width) {
	return static_cast<int>(CheckSoftmaxRowWidthDomain(q_b, q_c, width));
}
int refshim_softmax_row_q15(const int64_t* scores, size_t width, int64_t q_ln2, int64_t q_b,
                            int64_t q_c, int64_t* out_probs) {
	return SoftmaxRowQ15(scores, width, q_ln2, q_b, q_c, out_probs) ? 1 : 0;
}
void refshim_gemm(const int8_t* a, const int8_t* w, size_t m, size_t k, size_t n, int64_t* out) {
	GemmInt8Accumulate(a, w, m, k, n, out);
}
void refshim_prob_v(const int64_t* probs, const int8_t* v, size_t width, size_t hd, int64_t* out) {
	GemmProbQ15Accumulate(probs, v, width, hd, out);
}
int refshim_funnel(const int64_t* wide, size_t n, const int64_t* incoming_me, size_t n_incoming,
                   int64_t cm, int64_t ce, int8_t* out_codes, int64_t* om, int64_t* oe) {
	CarriedScale inc[4];
	for (size_t i = 0; i < n_incoming && i < 4; ++i) {
		inc[i] = CarriedScale{incoming_me[2 * i], incoming_me[2 * i + 1]};
	}
	CarriedScale out{};
	const ChainResult r = RequantChainChecked(
	    wide, n, std::span<const CarriedScale>{inc, n_incoming}, CarriedScale{cm, ce}, out_codes, &out);
	*om = out.m;
	*oe = out.e;
	return static_cast<int>(r.status);
}
int refshim_rmsnorm_site(const int8_t* h, const int32_t* g, size_t n, int64_t cm, int64_t ce,
                         int8_t* out_codes, int64_t* om, int64_t* oe) {
	CarriedScale out{};
	const SslmForwardStatus s =
	    RmsNormSite(h, g, n, CarriedScale{}, CarriedScale{cm, ce}, out_codes, &out);
	*om = out.m;
	*oe = out.e;
	return static_cast<int>(s);
}
int refshim_mlp_act_site(const int8_t* gate, int64_t gm, int64_t ge, const int8_t* up, int64_t um,
                         int64_t ue, size_t n, const int32_t* table, int64_t cm, int64_t ce,
                         int8_t* out_codes, int64_t* om, int64_t* oe) {
	CarriedScale out{};
	const SslmForwardStatus s = MlpActSite(gate, CarriedScale{gm, ge}, up, CarriedScale{um, ue}, n,
	                                        table, CarriedScale{cm, ce}, out_codes, &out);
	*om = out.m;
	*oe = out.e;
	return static_cast<int>(s);
}
int refshim_residual_site(const int8_t* branch, int64_t bm, int64_t be, const int8_t* stream,
                          int64_t sm, int64_t se, size_t n, int64_t cm, int64_t ce,
                          int8_t* out_codes, int64_t* om, int64_t* oe) {
	CarriedScale out{};
	const SslmForwardStatus s =
	    ResidualReconcileSite(branch, CarriedScale{bm, be}, stream, CarriedScale{sm, se}, n,
	                          CarriedScale{cm, ce}, out_codes, &out);
	*om = out.m;
	*oe = out.e;
	return static_cast<int>(s);
}
int refshim_narrow_row(const int64_t* wide, size_t n, int32_t* out) {
	return static_cast<int>(NarrowRowChecked(wide, n, out));
}
int32_t refshim_argmax(const int32_t* logits, size_t n) { return ArgmaxLowestIndexTieBreak(logits, n); }

}  // extern "C"
