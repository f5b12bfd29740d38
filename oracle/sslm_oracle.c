/* CPU oracle -- TEST INFRASTRUCTURE, NOT PRODUCT CODE. See sslm_oracle.h.
 *
 * Plain C11 + the compiler's 128-bit integer. Scalar, single-threaded, written for
 * clarity: one function per reference function, same operation order, so that every
 * intermediate can be compared. Right shifts of negative values are arithmetic
 * (floor) shifts on the compilers this builds with, as in the reference.
 */
#include "sslm_oracle.h"

#include <stdlib.h>
#include <string.h>

typedef __int128 s128;
typedef unsigned __int128 u128;

#define I32_MAX 2147483647
#define I32_MIN (-2147483647 - 1)

/* ---------------------------------------------------------------- primitives */

int32_t osc_srdhm(int32_t a, int32_t b) {
	int64_t ab = (int64_t)a * (int64_t)b;
	int64_t r = (ab + ((int64_t)1 << 30)) >> 31;
	return r > I32_MAX ? I32_MAX : (int32_t)r;
}

int32_t osc_rdivpot32(int32_t x, int exponent) {
	uint32_t mask = ((uint32_t)1 << exponent) - 1u;
	uint32_t rem = (uint32_t)x & mask;
	uint32_t thr = (mask >> 1) + (x < 0 ? 1u : 0u);
	return (x >> exponent) + (rem > thr ? 1 : 0);
}

int64_t osc_rdivpot64(int64_t x, int exponent) {
	uint64_t mask = ((uint64_t)1 << exponent) - 1u;
	uint64_t rem = (uint64_t)x & mask;
	uint64_t thr = (mask >> 1) + (x < 0 ? 1u : 0u);
	return (x >> exponent) + (rem > thr ? 1 : 0);
}

int32_t osc_mbqm(int32_t x, int32_t mult, int shift) {
	return osc_rdivpot32(osc_srdhm(x, mult), shift);
}

int32_t osc_sat_lshift32(int32_t x, int shift) {
	if (shift <= 0) return x;
	int64_t w = (int64_t)x << shift;
	if (w > I32_MAX) return I32_MAX;
	if (w < I32_MIN) return I32_MIN;
	return (int32_t)w;
}

void osc_normalize_scale(int64_t d_prime, int64_t* dn, int* s) {
	int p = 63 - __builtin_clzll((uint64_t)d_prime);
	*s = 30 - p;
	*dn = *s >= 0 ? (d_prime << *s) : (d_prime >> 1);
}

int64_t osc_dyn_recip(int64_t dn) {
	const int64_t c48 = (2 * ((int64_t)48 << 31) + 17) / 34;
	const int64_t c32 = (2 * ((int64_t)32 << 31) + 17) / 34;
	/* the reference forms c32*dn in int64 (it is < 2^63 on the canonical domain and
	 * wraps silently elsewhere); unsigned multiply gives the same bits without UB */
	int64_t y = c48 - ((int64_t)((uint64_t)c32 * (uint64_t)dn) >> 31);
	for (int i = 0; i < 3; ++i) {
		int64_t dn_y = (int64_t)(((s128)dn * (s128)y) >> 31);
		int64_t delta = (int64_t)((uint64_t)((int64_t)1 << 32) - (uint64_t)dn_y);
		y = (int64_t)(((s128)y * (s128)delta) >> 31);
	}
	for (int i = 0; i < 2; ++i) {
		s128 r2 = (((s128)1 << 62) - (s128)y * (s128)dn) << 1;
		if (r2 >= (s128)dn) {
			y = (int64_t)((uint64_t)y + 1u);
		} else if (r2 < -(s128)dn) {
			y = (int64_t)((uint64_t)y - 1u);
		}
	}
	return y;
}

int8_t osc_requant_code_wide(int64_t x, int64_t r, int s) {
	int exponent = 62 - s;
	uint64_t ax = x < 0 ? (~(uint64_t)x + 1u) : (uint64_t)x;
	u128 prod = (u128)ax * (uint64_t)r * 127u;
	u128 num = (prod << 1) + ((uint64_t)1 << exponent);
	uint64_t mag = (uint64_t)(num >> (exponent + 1));
	if (mag > 127u) mag = 127u;
	int32_t q = (int32_t)mag;
	return (int8_t)(x < 0 ? -q : q);
}

int64_t osc_isqrt(int64_t n) {
	int64_t rem = n, root = 0, bit = (int64_t)1 << 62;
	for (int i = 0; i < 32; ++i) {
		int64_t trial = root + bit;
		if (rem >= trial) {
			rem -= trial;
			root = (root >> 1) + bit;
		} else {
			root >>= 1;
		}
		bit >>= 2;
	}
	return root;
}

int64_t osc_floor_div(int64_t a, int64_t b) {
	int64_t q = a / b, r = a % b;
	return (r != 0 && r < 0) ? q - 1 : q;
}

void osc_rope_pair(int32_t x, int32_t y, int32_t c, int32_t s, int64_t* ox, int64_t* oy) {
	int64_t xr = (int64_t)x * c - (int64_t)y * s;
	int64_t yr = (int64_t)x * s + (int64_t)y * c;
	*ox = osc_rdivpot64(xr, 30);
	*oy = osc_rdivpot64(yr, 30);
}

int64_t osc_fold(int64_t acc, int32_t identity, int32_t mult, int32_t shift) {
	if (identity != 0) return acc;
	return (int64_t)osc_mbqm((int32_t)acc, mult, shift);
}

/* the same fold over a whole [m, n] accumulator matrix (fold triples per column), for the linear sweeps */
void osc_fold_matrix(const int64_t* acc, size_t m, size_t n, const int32_t* fold, int64_t* out) {
	for (size_t t = 0; t < m; ++t)
		for (size_t j = 0; j < n; ++j)
			out[t * n + j] = osc_fold(acc[t * n + j], fold[3 * j], fold[3 * j + 1], fold[3 * j + 2]);
}

int64_t osc_amp_fold(int64_t acc, int32_t identity, int32_t mult, int32_t exponent) {
	if (identity != 0) return acc;
	int32_t hi = osc_srdhm((int32_t)acc, mult);
	if (exponent >= 0) return (int64_t)osc_rdivpot32(hi, exponent);
	return (int64_t)osc_sat_lshift32(hi, -exponent);
}

static int64_t sat_add64(int64_t a, int64_t b) {
	int64_t out = (int64_t)((uint64_t)a + (uint64_t)b);
	if ((a >= 0) == (b >= 0) && (out >= 0) != (a >= 0)) return a >= 0 ? INT64_MAX : INT64_MIN;
	return out;
}

static int64_t sat_sub64(int64_t a, int64_t b) {
	int64_t out = (int64_t)((uint64_t)a - (uint64_t)b);
	if ((a >= 0) != (b >= 0) && (out >= 0) != (a >= 0)) return a >= 0 ? INT64_MAX : INT64_MIN;
	return out;
}

osc_scale osc_combine(osc_scale a, osc_scale b) {
	int64_t e = sat_add64(sat_add64(a.e, b.e), 31);
	int64_t m = (int64_t)osc_srdhm((int32_t)a.m, (int32_t)b.m);
	if (m < ((int64_t)1 << 30)) {
		m <<= 1;
		e -= 1;
	}
	osc_scale r = {m, e};
	return r;
}

static u128 u128_shl(u128 v, int k) { return k <= 0 ? v : (k >= 128 ? 0 : v << k); }
static u128 u128_shr(u128 v, int k) { return k <= 0 ? v : (k >= 128 ? 0 : v >> k); }

int64_t osc_landing_rescale(int64_t code, int64_t m_a, int64_t r_t, int64_t e_a, int64_t e_t,
                            uint64_t* sat_count, int* exceeded_int64) {
	const int neg = (code < 0) != (m_a < 0);
	uint64_t ac = code < 0 ? (~(uint64_t)code + 1u) : (uint64_t)code;
	uint64_t am = m_a < 0 ? (~(uint64_t)m_a + 1u) : (uint64_t)m_a;
	/* |code|*|m_a| is a full 128-bit product; the multiply by r_t keeps the low 128
	 * bits (the reference's U128MulSmall) */
	u128 mag = ((u128)ac * am) * (u128)(uint64_t)r_t;
	int64_t k = sat_sub64(62, sat_sub64(e_a, e_t));
	if (k > 4096) k = 4096;
	if (k < -4096) k = -4096;
	int over_clamp, over_i64;
	int64_t raw;
	if (k >= 0) {
		u128 q = u128_shr(mag + mag + u128_shl(1, (int)k), (int)k + 1);
		uint64_t hi = (uint64_t)(q >> 64), lo = (uint64_t)q;
		over_clamp = hi != 0 || lo > 127;
		over_i64 = hi != 0 || lo > (uint64_t)INT64_MAX;
		raw = (int64_t)lo;
	} else {
		int shift = (int)(-k);
		u128 sh = u128_shl(mag, shift);
		if (shift >= 128) {
			over_clamp = mag != 0;
			over_i64 = over_clamp;
		} else {
			int lost = u128_shr(sh, shift) != mag;
			uint64_t hi = (uint64_t)(sh >> 64), lo = (uint64_t)sh;
			over_clamp = lost || hi != 0 || lo > 127;
			over_i64 = lost || hi != 0 || lo > (uint64_t)INT64_MAX;
		}
		raw = (int64_t)(uint64_t)sh;
	}
	if (neg) raw = (int64_t)(0u - (uint64_t)raw);
	if (sat_count && (over_clamp || raw < -127 || raw > 127)) *sat_count += 1;
	if (exceeded_int64) *exceeded_int64 = over_i64;
	return raw;
}

static int64_t clamp127(int64_t v) { return v > 127 ? 127 : (v < -127 ? -127 : v); }

int32_t osc_silu_sigmoid_q15(const int32_t* table, int8_t code, int64_t m, int e) {
	int64_t term = (int64_t)code * m;
	int shift = e + 5 + 12;
	int64_t pos = shift >= 0 ? (int64_t)((uint64_t)term << shift) : osc_rdivpot64(term, -shift);
	const int64_t hi_dom = (int64_t)1024 << 12;
	pos += hi_dom / 2;
	if (pos < 0) pos = 0;
	else if (pos > hi_dom) pos = hi_dom;
	int64_t i0 = pos >> 12;
	if (i0 > 1023) i0 = 1023;
	int64_t frac = pos - (i0 << 12);
	int64_t lo = table[i0], hi = table[i0 + 1];
	return (int32_t)(lo + osc_rdivpot64(frac * (hi - lo), 12));
}

/* Q30 coefficients of the second-order i-exp polynomial
 * (include/superslm/intmath.h:518-527): ln2, b = 1.353, c/a = 0.344/0.3585 */
static void iexp_coefficients(int64_t* ln2_q, int64_t* b_q, int64_t* ca_q) {
	*ln2_q = (int64_t)(0x1.62e42fefa39efp-1 * (double)((int64_t)1 << 30));
	*b_q = (int64_t)(1.353 * (double)((int64_t)1 << 30));
	*ca_q = (int64_t)((0.344 / 0.3585) * (double)((int64_t)1 << 30));
}

int osc_iexp_scale_constants(int64_t m, int64_t e, int64_t* q_ln2, int64_t* q_b, int64_t* q_c) {
	int64_t ln2_q, b_q, ca_q;
	iexp_coefficients(&ln2_q, &b_q, &ca_q);
	int64_t sh_ln2 = sat_add64(sat_add64(30, 62), e);
	int64_t sh_b = sat_add64(sat_add64(30, 62), e);
	int64_t sh_c = sat_add64(sat_add64(30, 124), sat_add64(e, e));
	int64_t mn = sh_ln2 < sh_b ? sh_ln2 : sh_b;
	if (sh_c < mn) mn = sh_c;
	if (mn < 0) return 2;
	uint64_t rm = (uint64_t)osc_dyn_recip(m);
	u128 n_ln2 = (u128)(uint64_t)ln2_q * rm;
	u128 n_b = (u128)(uint64_t)b_q * rm;
	u128 n_c = ((u128)rm * rm) * (uint64_t)ca_q;
	u128 f_ln2 = sh_ln2 >= 128 ? 0 : n_ln2 >> (int)sh_ln2;
	u128 f_b = sh_b >= 128 ? 0 : n_b >> (int)sh_b;
	u128 f_c = sh_c >= 128 ? 0 : n_c >> (int)sh_c;
	if (f_ln2 > (u128)INT64_MAX || f_b > (u128)INT64_MAX || f_c > (u128)INT64_MAX) return 3;
	*q_ln2 = (int64_t)(uint64_t)f_ln2;
	*q_b = (int64_t)(uint64_t)f_b;
	*q_c = (int64_t)(uint64_t)f_c;
	return 0;
}

#define SOFTMAX_MAX_SAFE (((int64_t)1 << 62) >> 15)

int osc_softmax_width_domain(int64_t q_b, int64_t q_c, size_t width) {
	if (q_c < 0 || width == 0) return OSC_SOFTMAX_ROW_WIDTH_OUT_OF_DOMAIN;
	s128 m128 = (s128)q_b * q_b + q_c;
	if (m128 > (s128)SOFTMAX_MAX_SAFE) return OSC_SOFTMAX_ROW_WIDTH_OUT_OF_DOMAIN;
	int64_t m = (int64_t)m128;
	if (m != 0 && width > (size_t)(INT64_MAX / m)) return OSC_SOFTMAX_ROW_WIDTH_OUT_OF_DOMAIN;
	return OSC_OK;
}

/* IExpConstruct + IExpEvaluate for one shifted score (src/intmath.cpp:540-668).
 * returns 0 when the element is refused (bad q / q_ln2 / q_b) */
static int iexp_element(int64_t q, int64_t q_ln2, int64_t q_b, int64_t q_c, int64_t* value) {
	if (q > 0) return 0;
	if (q_ln2 < 1 || q_ln2 > INT64_MAX / 30) return 0;
	int64_t clip_lo = -(int64_t)30 * q_ln2;
	int64_t clipped = q < clip_lo ? clip_lo : q;
	int64_t z = (-clipped) / q_ln2;
	int64_t q_p = clipped + z * q_ln2;
	if (q_b < INT64_MIN - q_p) return 0;
	int64_t base = q_p + q_b;
	s128 v = (s128)base * base + q_c;
	*value = (int64_t)(v >> (int)z);
	return 1;
}

/* 0 kOk, 1 kBadQ, 2 kBadQLn2, 3 kBadQB, 4 kNotRepresentable (IExpDomain,
 * include/superslm/intmath.h:349); *value = IExpEvaluate of the construction */
int osc_iexp(int64_t q, int64_t q_ln2, int64_t q_b, int64_t q_c, int64_t* z_out, int64_t* base_out,
             int64_t* value) {
	*value = 0;
	if (q > 0) return 1;
	if (q_ln2 < 1 || q_ln2 > INT64_MAX / 30) return 2;
	int64_t clip_lo = -(int64_t)30 * q_ln2;
	int64_t clipped = q < clip_lo ? clip_lo : q;
	int64_t z = (-clipped) / q_ln2;
	int64_t q_p = clipped + z * q_ln2;
	if (q_b < INT64_MIN - q_p) return 3;
	int64_t base = q_p + q_b;
	if (z_out) *z_out = z;
	if (base_out) *base_out = base;
	s128 v = (s128)base * base + q_c;
	*value = (int64_t)(v >> (int)z);
	s128 limit = (s128)1 << (63 + (int)z);
	return (v <= limit - 1 && v >= -limit) ? 0 : 4;
}

int osc_softmax_row_q15(const int64_t* scores, size_t width, int64_t q_ln2, int64_t q_b,
                        int64_t q_c, int64_t* out_probs) {
	if (width == 0) return 1;
	s128 m128 = (s128)q_b * q_b + q_c;
	int m_usable = m128 >= 1 && m128 <= (s128)SOFTMAX_MAX_SAFE;
	int64_t m = m_usable ? (int64_t)m128 : 0;
	int64_t peak = scores[0];
	for (size_t k = 1; k < width; ++k) {
		if (scores[k] > peak) peak = scores[k];
	}
	int64_t total = 0;
	int ok = 1;
	for (size_t k = 0; k < width; ++k) {
		int64_t v;
		if (!iexp_element(scores[k] - peak, q_ln2, q_b, q_c, &v) || !m_usable || v < 0 || v > m) {
			ok = 0;
			out_probs[k] = 0;
			continue;
		}
		out_probs[k] = v;
		total += v;
	}
	int64_t denom = total > 1 ? total : 1;
	for (size_t k = 0; k < width; ++k) out_probs[k] = (out_probs[k] << 15) / denom;
	return ok;
}

/* ---------------------------------------------------------------------- rows */

void osc_gemm(const int8_t* a, const int8_t* w, size_t m, size_t k, size_t n, int64_t* out) {
	for (size_t t = 0; t < m; ++t) {
		for (size_t j = 0; j < n; ++j) {
			int64_t acc = 0;
			const int8_t* ar = a + t * k;
			const int8_t* wr = w + j * k;
			for (size_t i = 0; i < k; ++i) acc += (int64_t)ar[i] * (int64_t)wr[i];
			out[t * n + j] = acc;
		}
	}
}

static int fits_i32(int64_t v) { return v >= I32_MIN && v <= I32_MAX; }

int osc_funnel(const int64_t* wide, size_t n, const osc_scale* incoming, size_t n_incoming,
               osc_scale site_constant, int8_t* out_codes, osc_scale* out_scale) {
	for (size_t i = 0; i < n_incoming; ++i) {
		if (!fits_i32(incoming[i].m)) return OSC_CARRIED_SCALE_MANTISSA_OUT_OF_DOMAIN;
	}
	if (!fits_i32(site_constant.m)) return OSC_CARRIED_SCALE_MANTISSA_OUT_OF_DOMAIN;
	uint64_t d = 0;
	for (size_t i = 0; i < n; ++i) {
		uint64_t a = wide[i] < 0 ? (~(uint64_t)wide[i] + 1u) : (uint64_t)wide[i];
		if (a > d) d = a;
	}
	if (d < 1) d = 1;
	int64_t d_prime = d > (uint64_t)INT64_MAX ? INT64_MAX : (int64_t)d;
	if (d_prime > ((int64_t)1 << 31)) return OSC_CHAIN_INPUT_OUT_OF_DOMAIN;
	int64_t dn;
	int s;
	osc_normalize_scale(d_prime, &dn, &s);
	int64_t r = osc_dyn_recip(dn);
	osc_scale run = {0, 0};
	int have = 0;
	for (size_t i = 0; i < n_incoming + 2; ++i) {
		osc_scale next;
		if (i < n_incoming) next = incoming[i];
		else if (i == n_incoming) next = site_constant;
		else { next.m = dn; next.e = -(int64_t)s; }
		run = have ? osc_combine(run, next) : next;
		have = 1;
		if (!fits_i32(run.m)) return OSC_CARRIED_SCALE_MANTISSA_OUT_OF_DOMAIN;
	}
	for (size_t i = 0; i < n; ++i) out_codes[i] = osc_requant_code_wide(wide[i], r, s);
	*out_scale = run;
	return OSC_OK;
}

int osc_rmsnorm_site(const int8_t* h, const int8_t* gain, size_t n, osc_scale c, int8_t* out,
                     osc_scale* out_scale) {
	int64_t sumsq = 0;
	for (size_t i = 0; i < n; ++i) sumsq += (int64_t)h[i] * h[i];
	int64_t root = osc_isqrt(osc_floor_div(sumsq << 32, (int64_t)n));
	if (root < 1) root = 1;
	int64_t* wide = (int64_t*)malloc(n * sizeof(int64_t));
	for (size_t i = 0; i < n; ++i) {
		wide[i] = osc_floor_div((int64_t)h[i] * ((int64_t)1 << 32), root) * (int64_t)gain[i];
	}
	int st = osc_funnel(wide, n, NULL, 0, c, out, out_scale);
	free(wide);
	return st;
}

int osc_mlp_act_site(const int8_t* gate, osc_scale gs, const int8_t* up, osc_scale us, size_t n,
                     const int32_t* table, osc_scale c, int8_t* out, osc_scale* out_scale) {
	if (gs.m < -(((int64_t)1 << 31) - 1) || gs.m > (((int64_t)1 << 31) - 1) || gs.e < -80 || gs.e > 8) {
		return OSC_SILU_SCALE_OUT_OF_DOMAIN;
	}
	int64_t* wide = (int64_t*)malloc(n * sizeof(int64_t));
	for (size_t i = 0; i < n; ++i) {
		int32_t sig = osc_silu_sigmoid_q15(table, gate[i], gs.m, (int)gs.e);
		wide[i] = (int64_t)gate[i] * sig * (int64_t)up[i];
	}
	osc_scale inc[2] = {gs, us};
	int st = osc_funnel(wide, n, inc, 2, c, out, out_scale);
	free(wide);
	return st;
}

int osc_residual_site(const int8_t* branch, osc_scale bs, const int8_t* stream, osc_scale ss,
                      size_t n, osc_scale c, int8_t* out, osc_scale* out_scale) {
	if (!fits_i32(ss.m)) return OSC_CARRIED_SCALE_MANTISSA_OUT_OF_DOMAIN;
	int64_t r_h = osc_dyn_recip(ss.m);
	int64_t* wide = (int64_t*)calloc(n, sizeof(int64_t));
	int bad = 0;
	for (size_t i = 0; i < n; ++i) {
		int ex = 0;
		int64_t v = osc_landing_rescale(branch[i], bs.m, r_h, bs.e, ss.e, NULL, &ex);
		if (ex) { bad = 1; continue; }
		wide[i] = v + (int64_t)stream[i];
	}
	int st = bad ? OSC_RESIDUAL_MAGNITUDE_OUT_OF_DOMAIN : osc_funnel(wide, n, &ss, 1, c, out, out_scale);
	free(wide);
	return st;
}

int osc_embed_entry(int32_t token, int32_t vocab, const int8_t* embed, size_t hidden, osc_scale c,
                    int8_t* out, osc_scale* out_scale) {
	if (token < 0 || token >= vocab) return OSC_TOKEN_ID_OUT_OF_RANGE;
	int64_t* wide = (int64_t*)malloc(hidden * sizeof(int64_t));
	for (size_t i = 0; i < hidden; ++i) wide[i] = embed[(size_t)token * hidden + i];
	int st = osc_funnel(wide, hidden, NULL, 0, c, out, out_scale);
	free(wide);
	return st;
}

/* ------------------------------------------------------------ layer machinery */

/* AddAmplifyingLoraDelta (forward_sites.cpp:1051-1103) */
static void lora_delta(const int8_t* in, size_t k_in, const osc_lora_proj* p, uint32_t rank,
                       size_t n_out, int64_t* acc) {
	if (!p || !p->a_w || !p->b_w || !p->u_fold || !p->d_fold) return;
	int8_t u8[256];
	for (uint32_t r = 0; r < rank; ++r) {
		int64_t u;
		osc_gemm(in, p->a_w + (size_t)r * k_in, 1, k_in, 1, &u);
		u = osc_amp_fold(u, p->u_fold[3 * r], p->u_fold[3 * r + 1], p->u_fold[3 * r + 2]);
		u8[r] = (int8_t)clamp127(u);
	}
	for (size_t i = 0; i < n_out; ++i) {
		int64_t d;
		osc_gemm(u8, p->b_w + i * rank, 1, rank, 1, &d);
		acc[i] += osc_amp_fold(d, p->d_fold[3 * i], p->d_fold[3 * i + 1], p->d_fold[3 * i + 2]);
	}
}

/* BiasReconcileWide (src/intmath.cpp:397-418) with RoundingDivideByPOTWide (:365-378) */
int osc_bias_reconcile(int64_t b, int64_t r_a, int64_t e_a, int64_t* out) {
	*out = 0;
	if (e_a < -92 || e_a > -29) return 0;       /* 0 <= 30 + 62 + e_a <= 63 */
	const int exponent = (int)(92 + e_a);
	const s128 wide = (s128)b * (s128)r_a;
	const uint64_t mask = ((uint64_t)1 << exponent) - 1u;
	const uint64_t rem = (uint64_t)wide & mask;
	const uint64_t thr = (mask >> 1) + (wide < 0 ? 1u : 0u);
	s128 r = wide >> exponent;
	if (rem > thr) r += 1;
	*out = (int64_t)r;
	return r >= (s128)INT64_MIN && r <= (s128)INT64_MAX;
}

/* ApplyBiasReconcileRow (src/forward/forward_sites.cpp:1015-1036): exponent gate, then a
 * checking pass over every element (term fits, acc + term fits), then the add */
int osc_apply_bias_row(int64_t* acc, size_t n, const int64_t* bias, int64_t in_scale_m, int64_t in_scale_e) {
	if (in_scale_e < -92 || in_scale_e > -29) return OSC_RDIVPOT_EXPONENT_OUT_OF_DOMAIN;
	const int64_t r_a = osc_dyn_recip(in_scale_m);
	for (size_t i = 0; i < n; ++i) {
		int64_t term;
		if (!osc_bias_reconcile(bias[i], r_a, in_scale_e, &term)) return OSC_BIAS_RECONCILE_PRODUCT_OUT_OF_DOMAIN;
		int64_t sum;
		if (__builtin_add_overflow(acc[i], term, &sum)) return OSC_BIAS_RECONCILE_PRODUCT_OUT_OF_DOMAIN;
	}
	for (size_t i = 0; i < n; ++i) {
		int64_t term;
		osc_bias_reconcile(bias[i], r_a, in_scale_e, &term);
		acc[i] += term;
	}
	return OSC_OK;
}

/* ProjectAndFunnel (forward_sites.cpp:1148-1164, :1114-1146): fold, LoRA delta, bias, funnel */
static int project_funnel_bias(const int8_t* in, osc_scale in_scale, const int8_t* w, size_t k_in,
                               size_t n_out, const int32_t* fold, osc_scale c, const osc_lora_proj* lp,
                               uint32_t rank, const int64_t* bias, int8_t* out, osc_scale* out_scale) {
	int64_t* acc = (int64_t*)malloc(n_out * sizeof(int64_t));
	osc_gemm(in, w, 1, k_in, n_out, acc);
	for (size_t i = 0; i < n_out; ++i) acc[i] = osc_fold(acc[i], fold[3 * i], fold[3 * i + 1], fold[3 * i + 2]);
	lora_delta(in, k_in, lp, rank, n_out, acc);
	int st = OSC_OK;
	if (bias != NULL) st = osc_apply_bias_row(acc, n_out, bias, in_scale.m, in_scale.e);
	if (st == OSC_OK) st = osc_funnel(acc, n_out, &in_scale, 1, c, out, out_scale);
	free(acc);
	return st;
}

/* the same for the projections that never carry a bias (o, gate, up, down) */
static int project_funnel(const int8_t* in, osc_scale in_scale, const int8_t* w, size_t k_in,
                          size_t n_out, const int32_t* fold, osc_scale c, const osc_lora_proj* lp,
                          uint32_t rank, int8_t* out, osc_scale* out_scale) {
	int64_t* acc = (int64_t*)malloc(n_out * sizeof(int64_t));
	osc_gemm(in, w, 1, k_in, n_out, acc);
	for (size_t i = 0; i < n_out; ++i) acc[i] = osc_fold(acc[i], fold[3 * i], fold[3 * i + 1], fold[3 * i + 2]);
	lora_delta(in, k_in, lp, rank, n_out, acc);
	int st = osc_funnel(acc, n_out, &in_scale, 1, c, out, out_scale);
	free(acc);
	return st;
}

static int8_t* kv_row(const osc_model* m, int8_t* kv, uint32_t layer, int is_v, size_t kv_head, int64_t pos) {
	size_t half = (size_t)m->context_cap * m->kv_heads * m->head_dim;
	return kv + (size_t)layer * half * 2 + (is_v ? half : 0) +
	       kv_head * (size_t)m->context_cap * m->head_dim + (size_t)pos * m->head_dim;
}

static void rope_row(const osc_model* m, const int8_t* row, int64_t pos, int8_t* out) {
	size_t pairs = m->head_dim / 2;
	for (size_t i = 0; i < pairs; ++i) {
		int32_t c = (int32_t)m->rope_cos[(size_t)pos * pairs + i];
		int32_t s = (int32_t)m->rope_sin[(size_t)pos * pairs + i];
		int64_t x, y;
		osc_rope_pair(row[2 * i], row[2 * i + 1], c, s, &x, &y);
		out[2 * i] = (int8_t)clamp127(x);
		out[2 * i + 1] = (int8_t)clamp127(y);
	}
}

/* Per-site trace for bisection (the counterpart of the reference's trace hook,
 * src/forward/checked_chain_funnel.cpp:338-361): while a buffer is set, one_layer appends a
 * record per site: { int64 position; int32 layer; int32 site; int64 m; int64 e; int32 n;
 * int32 row (= -1 here) } followed by n codes, padded to a multiple of 8 bytes. Site numbers:
 * 0 attn_norm, 2 rotated q (no scale), 3 attn_ctx, 5 attn_residual, 6 mlp_norm, 9 mlp_act,
 * 11 mlp_residual -- the sites whose codes the CUDA path keeps in global memory. */
static uint8_t* g_trace_buf = NULL;
static size_t g_trace_cap = 0, g_trace_used = 0;
void osc_trace_begin(uint8_t* buf, size_t capacity) {
	g_trace_buf = buf;
	g_trace_cap = capacity;
	g_trace_used = 0;
}
size_t osc_trace_end(void) {
	g_trace_buf = NULL;
	return g_trace_used;
}
static void trace_emit(int64_t position, uint32_t layer, int site, const int8_t* codes, size_t n, osc_scale sc) {
	if (g_trace_buf == NULL) return;
	const size_t bytes = 40 + ((n + 7) & ~(size_t)7);
	if (g_trace_used + bytes > g_trace_cap) return;
	uint8_t* p = g_trace_buf + g_trace_used;
	int32_t l32 = (int32_t)layer, s32 = site, n32 = (int32_t)n, row = -1;
	memset(p, 0, bytes);
	memcpy(p, &position, 8);
	memcpy(p + 8, &l32, 4);
	memcpy(p + 12, &s32, 4);
	memcpy(p + 16, &sc.m, 8);
	memcpy(p + 24, &sc.e, 8);
	memcpy(p + 32, &n32, 4);
	memcpy(p + 36, &row, 4);
	memcpy(p + 40, codes, n);
	g_trace_used += bytes;
}

/* One layer for one token at `position`: steps 1-13 of RunLayerLoopImpl's body
 * (forward_sites.cpp:1685-1987). hidden/hidden_scale are the layer input; the new
 * stream is written to out_hidden/out_scale. K/V of this position are landed in kv. */
static int one_layer(const osc_model* m, const osc_lora_layer* lora, uint32_t l, int64_t position,
                     const int8_t* hidden, osc_scale hidden_scale, int8_t* kv, uint64_t* sat,
                     int8_t* out_hidden, osc_scale* out_scale) {
	const osc_layer* lw = &m->layer[l];
	const size_t H = m->hidden, I = m->inter, hd = m->head_dim, KVH = m->kv_heads;
	const size_t kvh = KVH * hd, heads = H / hd, group = heads / KVH;
	const size_t width = (size_t)position + 1;
	const uint32_t rank = lora ? lora->rank : 0;
	int st = OSC_OK;
	int8_t* buf = (int8_t*)malloc(6 * H + 3 * I);
	int8_t *normed = buf, *q = buf + H, *q_rot = buf + 2 * H, *ctx = buf + 3 * H, *o = buf + 4 * H,
	       *attn_stream = buf + 5 * H, *gate = buf + 6 * H, *up = gate + I, *act = up + I;
	int64_t* wide = (int64_t*)malloc((2 * kvh + H + 2 * width + hd) * sizeof(int64_t));
	int64_t *kacc = wide, *vacc = wide + kvh, *ctx_wide = wide + 2 * kvh, *scores = ctx_wide + H,
	        *probs = scores + width, *ctx_acc = probs + width;
	osc_scale s_n, s_q, s_ctx, s_o, s_a, s_n2, s_g, s_u, s_act, s_d;

	if ((st = osc_rmsnorm_site(hidden, lw->attn_gain, H, lw->c_attn_norm, normed, &s_n))) goto done;
	trace_emit(position, l, 0, normed, H, s_n);
	if ((st = project_funnel_bias(normed, s_n, lw->q_w, H, H, lw->q_fold, lw->c_q, lora ? &lora->q : NULL,
	                              rank, lw->q_bias, q, &s_q))) goto done;
	/* K/V projection + landing (LandTokenKVRow, forward_sites.cpp:1281-1418, legacy branch) */
	osc_gemm(normed, lw->k_w, 1, H, kvh, kacc);
	osc_gemm(normed, lw->v_w, 1, H, kvh, vacc);
	for (size_t i = 0; i < kvh; ++i) {
		kacc[i] = osc_fold(kacc[i], lw->k_fold[3 * i], lw->k_fold[3 * i + 1], lw->k_fold[3 * i + 2]);
		vacc[i] = osc_fold(vacc[i], lw->v_fold[3 * i], lw->v_fold[3 * i + 1], lw->v_fold[3 * i + 2]);
	}
	lora_delta(normed, H, lora ? &lora->k : NULL, rank, kvh, kacc);
	lora_delta(normed, H, lora ? &lora->v : NULL, rank, kvh, vacc);
	if (lw->k_bias != NULL && (st = osc_apply_bias_row(kacc, kvh, lw->k_bias, s_n.m, s_n.e))) goto done;
	if (lw->v_bias != NULL && (st = osc_apply_bias_row(vacc, kvh, lw->v_bias, s_n.m, s_n.e))) goto done;
	for (size_t h = 0; h < KVH; ++h) {
		int8_t* krow = kv_row(m, kv, l, 0, h, position);
		int8_t* vrow = kv_row(m, kv, l, 1, h, position);
		for (size_t d = 0; d < hd; ++d) {
			krow[d] = (int8_t)clamp127(osc_landing_rescale(kacc[h * hd + d], s_n.m, lw->k_recip[3 * h + 2],
			                                               s_n.e, lw->k_recip[3 * h + 1], sat, NULL));
		}
		for (size_t d = 0; d < hd; ++d) {
			vrow[d] = (int8_t)clamp127(osc_landing_rescale(vacc[h * hd + d], s_n.m, lw->v_recip[3 * h + 2],
			                                               s_n.e, lw->v_recip[3 * h + 1], sat, NULL));
		}
	}
	/* RoPE: q heads; landed K rotated in place (read, then write back) */
	for (size_t h = 0; h < heads; ++h) rope_row(m, q + h * hd, position, q_rot + h * hd);
	for (size_t h = 0; h < KVH; ++h) {
		int8_t tmp[512];
		int8_t* krow = kv_row(m, kv, l, 0, h, position);
		rope_row(m, krow, position, tmp);
		memcpy(krow, tmp, hd);
	}
	{
		const osc_scale none = {0, 0};
		trace_emit(position, l, 2, q_rot, H, none);
	}
	/* attention (forward_sites.cpp:1791-1905) */
	for (size_t h = 0; h < heads; ++h) {
		size_t kvhd = h / group;
		osc_scale kh = {lw->softmax_khead[2 * kvhd], lw->softmax_khead[2 * kvhd + 1]};
		if (!fits_i32(s_q.m) || !fits_i32(kh.m)) { st = OSC_CARRIED_SCALE_MANTISSA_OUT_OF_DOMAIN; goto done; }
		osc_scale sm = osc_combine(s_q, kh);
		if (!fits_i32(sm.m)) { st = OSC_CARRIED_SCALE_MANTISSA_OUT_OF_DOMAIN; goto done; }
		int64_t q_ln2, q_b, q_c;
		if (osc_iexp_scale_constants(sm.m, sm.e, &q_ln2, &q_b, &q_c)) {
			st = OSC_IEXP_SCALE_DERIVATION_OUT_OF_DOMAIN;
			goto done;
		}
		if ((st = osc_softmax_width_domain(q_b, q_c, width))) goto done;
		osc_gemm(q_rot + h * hd, kv_row(m, kv, l, 0, kvhd, 0), 1, hd, width, scores);
		if (!osc_softmax_row_q15(scores, width, q_ln2, q_b, q_c, probs)) {
			st = OSC_SOFTMAX_KERNEL_REFUSED;
			goto done;
		}
		const int8_t* vbase = kv_row(m, kv, l, 1, kvhd, 0);
		for (size_t d = 0; d < hd; ++d) ctx_acc[d] = 0;
		for (size_t k = 0; k < width; ++k) {
			for (size_t d = 0; d < hd; ++d) ctx_acc[d] += probs[k] * (int64_t)vbase[k * hd + d];
		}
		for (size_t d = 0; d < hd; ++d) {
			ctx_wide[h * hd + d] = osc_fold(ctx_acc[d], lw->ctx_fold[3 * h], lw->ctx_fold[3 * h + 1],
			                                lw->ctx_fold[3 * h + 2]);
		}
	}
	if ((st = osc_funnel(ctx_wide, H, NULL, 0, lw->c_ctx, ctx, &s_ctx))) goto done;
	trace_emit(position, l, 3, ctx, H, s_ctx);
	if ((st = project_funnel(ctx, s_ctx, lw->o_w, H, H, lw->o_fold, lw->c_o, lora ? &lora->o : NULL,
	                         rank, o, &s_o))) goto done;
	if ((st = osc_residual_site(o, s_o, hidden, hidden_scale, H, lw->c_attn_res, attn_stream, &s_a))) goto done;
	trace_emit(position, l, 5, attn_stream, H, s_a);
	if ((st = osc_rmsnorm_site(attn_stream, lw->mlp_gain, H, lw->c_mlp_norm, normed, &s_n2))) goto done;
	trace_emit(position, l, 6, normed, H, s_n2);
	if ((st = project_funnel(normed, s_n2, lw->gate_w, H, I, lw->gate_fold, lw->c_gate,
	                         lora ? &lora->gate : NULL, rank, gate, &s_g))) goto done;
	if ((st = project_funnel(normed, s_n2, lw->up_w, H, I, lw->up_fold, lw->c_up,
	                         lora ? &lora->up : NULL, rank, up, &s_u))) goto done;
	if ((st = osc_mlp_act_site(gate, s_g, up, s_u, I, m->silu_table, lw->c_act, act, &s_act))) goto done;
	trace_emit(position, l, 9, act, I, s_act);
	if ((st = project_funnel(act, s_act, lw->down_w, I, H, lw->down_fold, lw->c_down,
	                         lora ? &lora->down : NULL, rank, o, &s_d))) goto done;
	st = osc_residual_site(o, s_d, attn_stream, s_a, H, lw->c_mlp_res, out_hidden, out_scale);
	if (!st) trace_emit(position, l, 11, out_hidden, H, *out_scale);
done:
	free(buf);
	free(wide);
	return st;
}

int osc_layer_loop(const osc_model* m, const osc_lora_layer* lora, osc_seq* s, uint32_t layer_budget) {
	if (s->context_length < 0) return OSC_POSITION_OVER_CAP;
	if (s->context_length >= (int64_t)m->context_cap) return OSC_KV_CAPACITY_EXHAUSTED;
	int8_t* next = (int8_t*)malloc(m->hidden);
	uint32_t advanced = 0;
	int st = OSC_OK;
	while (advanced < layer_budget && s->layer_index < m->layers) {
		osc_scale ns;
		uint32_t l = s->layer_index;
		st = one_layer(m, lora ? &lora[l] : NULL, l, s->context_length, s->hidden_codes,
		               s->hidden_scale, s->kv, &s->kv_saturation_count, next, &ns);
		if (st) break;
		memcpy(s->hidden_codes, next, m->hidden);
		s->hidden_scale = ns;
		s->layer_index = l + 1;
		if (s->layer_index == m->layers) s->context_length += 1;
		++advanced;
	}
	free(next);
	return st;
}

int osc_embed_into_seq(const osc_model* m, osc_seq* s, int32_t token) {
	int st = osc_embed_entry(token, (int32_t)m->vocab, m->embed, m->hidden, m->c_embed,
	                         s->hidden_codes, &s->hidden_scale);
	if (!st) s->layer_index = 0;
	return st;
}

/* The chunk-batched loop couples tokens only through K/V of earlier positions, and
 * every row's arithmetic is independent of which rows share the call
 * (forward_sites.cpp:2175-2397, src/matmul.cpp:470-500), so it is restated here
 * token by token: each token runs all layers over the KV written so far. */
int osc_prefill(const osc_model* m, const osc_lora_layer* lora, osc_seq* s, const int32_t* tokens,
                int32_t n) {
	for (int32_t i = 0; i < n; ++i) {
		int st = osc_embed_into_seq(m, s, tokens[i]);
		if (st) return st;
		st = osc_layer_loop(m, lora, s, m->layers);
		if (st) return st;
		s->layer_index = 0;
	}
	return OSC_OK;
}

int osc_logits_argmax(const osc_model* m, const osc_seq* s, int32_t* out_logits, int32_t* out_token) {
	int8_t* fin = (int8_t*)malloc(m->hidden);
	osc_scale fs;
	int st = osc_rmsnorm_site(s->hidden_codes, m->final_gain, m->hidden, m->c_final_norm, fin, &fs);
	if (st) { free(fin); return st; }
	int64_t best_v = 0;
	int32_t best_i = 0;
	for (uint32_t v = 0; v < m->vocab; ++v) {
		int64_t acc;
		osc_gemm(fin, m->head + (size_t)v * m->hidden, 1, m->hidden, 1, &acc);
		if (acc > I32_MAX || acc < I32_MIN) { free(fin); return OSC_LOGIT_NARROWING_OVERFLOW; }
		if (out_logits) out_logits[v] = (int32_t)acc;
		if (v == 0 || acc > best_v) { best_v = acc; best_i = (int32_t)v; }
	}
	free(fin);
	*out_token = best_i;
	return OSC_OK;
}


/* The primitives over arrays of operands, one call per sweep: the CPU side of the device
 * primitive sweep (tests/test_gpu_int_sweep.py). Operand meaning per `which` is documented at
 * sslm_b200_int_sweep in include/sslm_b200.h; every case forwards to the function above that
 * restates the reference primitive. */
void osc_sweep(int which, const int64_t* a, const int64_t* b, const int64_t* c, const int64_t* e, int64_t n,
               int64_t* out0, int64_t* out1, int64_t* out2) {
	for (int64_t i = 0; i < n; ++i) {
		out0[i] = out1[i] = out2[i] = 0;
		switch (which) {
		case 0: out0[i] = osc_dyn_recip(a[i]); break;
		case 1: out0[i] = osc_isqrt(a[i]); break;
		case 2: out0[i] = osc_floor_div((int64_t)((uint64_t)a[i] << 32), b[i]); break;
		case 3: out0[i] = osc_requant_code_wide(a[i], b[i], (int)c[i]); break;
		case 4: {
			uint64_t sat = 0;
			int ex = 0;
			out0[i] = osc_landing_rescale(a[i], b[i], c[i], e[i] >> 32, (int64_t)(int32_t)(uint32_t)e[i], &sat, &ex);
			out1[i] = (int64_t)sat | ((int64_t)ex << 1);
			break;
		}
		case 5: out0[i] = (int64_t)((uint64_t)a[i] / (uint64_t)b[i]); break;
		case 6: {      /* the scalar half of the funnel on a one-element row of magnitude a */
			osc_scale inc = {b[i], c[i]}, site = {e[i] >> 32, (int64_t)(int32_t)(uint32_t)e[i]}, out = {0, 0};
			int64_t row = a[i];
			int8_t code = 0;
			out2[i] = osc_funnel(&row, 1, &inc, 1, site, &code, &out);
			out0[i] = out.m;
			out1[i] = out.e;
			break;
		}
		case 7: {      /* one softmax element: value and whether the row would be refused (peak = e) */
			int64_t v = 0;
			const int st = osc_iexp(-a[i], b[i], c[i], e[i] >> 32, 0, 0, &v);
			const int64_t peak = (int64_t)(uint32_t)e[i] | 0;      /* unused here: the caller derives the bound */
			(void)peak;
			out0[i] = v;
			out1[i] = st;
			break;
		}
		default: break;
		}
	}
}
