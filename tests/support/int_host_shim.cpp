// Host build of the device integer library (sslm_int.cuh compiles for the host when
// nvcc is not the compiler), exported with C linkage so that the CPU test-suite can
// compare every function with the oracle without a GPU. Test support only.
#include "../../superslm_b200/csrc/sslm_int.cuh"
using namespace sslm;
extern "C" {
int32_t dev_srdhm(int32_t a, int32_t b) { return srdhm(a, b); }
int32_t dev_rdivpot32(int32_t x, int e) { return rdivpot32(x, e); }
int64_t dev_rdivpot64(int64_t x, int e) { return rdivpot64(x, e); }
int32_t dev_fold(int32_t a, int32_t id, int32_t m, int32_t s) { return fold(a, id, m, s); }
int32_t dev_amp_fold(int32_t a, int32_t id, int32_t m, int32_t s) { return amp_fold(a, id, m, s); }
void dev_normalize_scale(int64_t d, int64_t* dn, int* s) { normalize_scale(d, dn, s); }
int64_t dev_dyn_recip(int64_t dn) { return dyn_recip(dn); }
int8_t dev_requant_code(int64_t x, int64_t r, int s) { return requant_code(x, r, s); }
// the epilogue's fold: the plain form where it applies, fold() elsewhere; -1 in *plain when not plain
int32_t dev_fold_epilogue(int32_t acc, int32_t identity, int32_t mult, int32_t shift, int* plain, uint32_t* mag) {
	*plain = fold_is_plain(identity, mult, shift) ? 1 : 0;
	*mag = 0;
	if (!*plain) return fold(acc, identity, mult, shift);
	return fold_plain(acc, mult, shift, shift ? (uint32_t)1 << (shift - 1) : 0u, mag);
}
int8_t dev_code_of64(int64_t x, int64_t r, int s) { return code_of(x, make_coder(r, s)); }
int8_t dev_code_of32(int32_t x, int64_t r, int s) { return code_of(x, make_coder(r, s)); }
void dev_combine(int64_t am, int64_t ae, int64_t bm, int64_t be, int64_t* om, int64_t* oe) {
	Scale c = combine(Scale{am, ae}, Scale{bm, be});
	*om = c.m; *oe = c.e;
}
int dev_funnel_params(uint64_t max_abs, const int64_t* inc, int n, int64_t cm, int64_t ce,
                      int64_t* r, int* s, int64_t* om, int64_t* oe) {
	Scale in[4];
	for (int i = 0; i < n; ++i) in[i] = Scale{inc[2 * i], inc[2 * i + 1]};
	FunnelParams fp = funnel_params(max_abs, in, n, Scale{cm, ce});
	*r = fp.r; *s = fp.s; *om = fp.out.m; *oe = fp.out.e;
	return fp.status;
}
int64_t dev_floor_div(int64_t a, int64_t b) { return floor_div(a, b); }
int64_t dev_floor_div_h32(int h, int64_t root) { return floor_div_h32(h, root, 1.0 / (double)root); }
uint64_t dev_udiv_small(uint64_t n, uint64_t d) { return udiv_small_quotient(n, d, 1.0 / (double)d); }
int64_t dev_isqrt(int64_t n) { return isqrt64(n); }
int64_t dev_landing_rescale(int64_t c, int64_t m, int64_t r, int64_t ea, int64_t et, int* sat, int* ex) {
	bool s = false, e = false;
	int64_t v = landing_rescale(c, m, r, ea, et, &s, &e);
	*sat = s; *ex = e;
	return v;
}
void dev_rope_pair(int32_t x, int32_t y, int32_t c, int32_t s, int8_t* ox, int8_t* oy) {
	rope_pair_clamped(x, y, c, s, ox, oy);
}
int32_t dev_silu(const int32_t* t, int32_t code, int64_t m, int e) { return silu_sigmoid_q15(t, code, m, e); }
int dev_iexp_scale_constants(int64_t m, int64_t e, int64_t* a, int64_t* b, int64_t* c) {
	IExpConsts k{0, 0, 0};
	int st = iexp_scale_constants(m, e, &k);
	*a = k.q_ln2; *b = k.q_b; *c = k.q_c;
	return st;
}
int dev_softmax_width(int64_t qb, int64_t qc, uint64_t w, int64_t* peak) {
	return softmax_width_in_domain(qb, qc, w, peak) ? 1 : 0;
}
// 1 with *out = the bias term when the exponent gate and the int64 fit both hold, else 0
int dev_bias_reconcile(int64_t b, int64_t r_a, int64_t e_a, int64_t* out) {
	int ex = 0;
	*out = 0;
	if (!bias_exponent_in_domain(e_a, &ex)) return 0;
	return bias_reconcile(b, r_a, ex, out) ? 1 : 0;
}
int dev_bias_accumulate(int64_t acc, int64_t term, int64_t* out) { return bias_accumulate(acc, term, out) ? 1 : 0; }
int dev_iexp_element(int64_t q, int64_t ln2, int64_t b, int64_t c, int64_t peak, int64_t* v) {
	IExpConsts k{ln2, b, c};
	return iexp_element(q, k, peak, v) ? 1 : 0;
}

// dyn_recip's one-division form against the reference's operation sequence (seed, three Newton
// steps, two corrections) on normalised divisors start, start + stride, ... : mismatches found
// (the first one through *first_bad). With stride 1 and count 2^30 this is the exhaustive check.
int64_t dev_dyn_recip_sweep(int64_t start, int64_t stride, int64_t count, int64_t* first_bad) {
	int64_t bad = 0;
	for (int64_t i = 0; i < count; ++i) {
		const int64_t dn = start + i * stride;
		if (dn < ((int64_t)1 << 30) || dn >= ((int64_t)1 << 31)) break;
		if (dyn_recip(dn) != dyn_recip_sequence(dn)) {
			if (bad == 0 && first_bad) *first_bad = dn;
			++bad;
		}
	}
	return bad;
}
}
