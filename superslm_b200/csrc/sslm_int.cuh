// Integer-only arithmetic of the SuperSLM forward pass, written for the GPU.
//
// Every function is bit-exact with the reference CPU function it names and uses
// only 32/64-bit integer operations (128-bit intermediates are carried as explicit
// {lo, hi} word pairs built from 64x64->128 multiplies), so the same source
// compiles for the device (the product) and, with SSLM_HD empty, for the host
// (a unit-test build that checks these functions against the CPU oracle without
// a GPU). No floating point is used for any value that reaches an output, except
// the reciprocal *estimates* inside the exact division helpers, whose results are
// corrected with integer arithmetic before use.
#pragma once
#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define SSLM_HD __host__ __device__ __forceinline__
#define SSLM_HD_OUTLINE inline __host__ __device__ __noinline__
#else
#define SSLM_HD inline
#define SSLM_HD_OUTLINE inline __attribute__((noinline))
#endif
// SSLM_HD_OUTLINE marks the general (rare-operand) halves of functions whose common case has a
// short exact form, and the per-row scalar derivations that a kernel calls several times. Kept
// out of line they exist once per module instead of once per call site and unrolled pass: a
// row kernel executes most of its instructions once per block, so its speed is set by how many
// instruction-cache lines it touches, and the inlined general paths made those kernels ~100 KB.

namespace sslm {

struct Scale { int64_t m, e; };

// status ordinals of the reference's SslmForwardStatus
// (include/superslm/checked_chain_funnel.h:68-284)
enum Status : int32_t {
	kOk = 0,
	kChainInputOutOfDomain = 1,
	kLogitNarrowingOverflow = 2,
	kCarriedScaleMantissaOutOfDomain = 4,
	kSiluScaleOutOfDomain = 5,
	kRoundingDivideExponentOutOfDomain = 6,
	kSoftmaxRowWidthOutOfDomain = 7,
	kTokenIdOutOfRange = 8,
	kSoftmaxKernelRefused = 20,
	kResidualMagnitudeOutOfDomain = 21,
	kIExpScaleDerivationOutOfDomain = 23,
	kBiasReconcileProductOutOfDomain = 24,
	kInternalWaitTimeout = 100,  // this implementation only: a bounded device-side wait ran out
};

// ---------------------------------------------------------------- 128-bit words
struct U128 { uint64_t lo, hi; };

SSLM_HD uint64_t umulhi64(uint64_t a, uint64_t b) {
#if defined(__CUDA_ARCH__)
	return __umul64hi(a, b);
#else
	return (uint64_t)(((unsigned __int128)a * b) >> 64);
#endif
}
SSLM_HD int clz64(uint64_t v) {
#if defined(__CUDA_ARCH__)
	return __clzll((long long)v);
#else
	return v ? __builtin_clzll(v) : 64;
#endif
}
SSLM_HD U128 umul64(uint64_t a, uint64_t b) { return U128{a * b, umulhi64(a, b)}; }
// low 128 bits of (128-bit a) * (64-bit b)
SSLM_HD U128 umul128x64(U128 a, uint64_t b) {
	U128 r = umul64(a.lo, b);
	r.hi += a.hi * b;
	return r;
}
SSLM_HD U128 uadd(U128 a, U128 b) {
	U128 r;
	r.lo = a.lo + b.lo;
	r.hi = a.hi + b.hi + (r.lo < a.lo ? 1u : 0u);
	return r;
}
SSLM_HD U128 ushl(U128 v, int k) {
	if (k <= 0) return v;
	if (k >= 128) return U128{0, 0};
	if (k >= 64) return U128{0, v.lo << (k - 64)};
	return U128{v.lo << k, (v.hi << k) | (v.lo >> (64 - k))};
}
SSLM_HD U128 ushr(U128 v, int k) {
	if (k <= 0) return v;
	if (k >= 128) return U128{0, 0};
	if (k >= 64) return U128{v.hi >> (k - 64), 0};
	return U128{(v.lo >> k) | (v.hi << (64 - k)), v.hi >> k};
}
// signed 64x64 -> 128 (two's complement words)
SSLM_HD U128 smul64(int64_t a, int64_t b) {
	U128 r = umul64((uint64_t)a, (uint64_t)b);
	if (a < 0) r.hi -= (uint64_t)b;
	if (b < 0) r.hi -= (uint64_t)a;
	return r;
}
// arithmetic shift right of a signed 128-bit value by k in [1,63], low 64 bits
SSLM_HD int64_t sshr_to_i64(U128 v, int k) {
	return (int64_t)((v.lo >> k) | (v.hi << (64 - k)));
}
SSLM_HD U128 ssub(U128 a, U128 b) {
	U128 r;
	r.lo = a.lo - b.lo;
	r.hi = a.hi - b.hi - (a.lo < b.lo ? 1u : 0u);
	return r;
}
SSLM_HD bool sge(U128 a, U128 b) {  // signed a >= b
	if ((int64_t)a.hi != (int64_t)b.hi) return (int64_t)a.hi > (int64_t)b.hi;
	return a.lo >= b.lo;
}
SSLM_HD U128 sfrom64(int64_t v) { return U128{(uint64_t)v, v < 0 ? ~0ull : 0ull}; }

// ------------------------------------------------ floating-point ESTIMATES only
// 1/x and sqrt(x) to nearly full double precision without the IEEE division / square-root
// routines (hundreds of cycles each on a path where one thread block waits on one scalar).
// Nothing that reaches an output is taken from these: every caller turns the estimate into
// an integer quotient or root and repairs it with exact integer arithmetic, so their
// accuracy only bounds how many repair steps run (none or one).
SSLM_HD double rcp_estimate(double x) {  // x >= 1
#if defined(__CUDA_ARCH__)
	double r;
	asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(r) : "d"(x));
	r = fma(r, fma(-x, r, 1.0), r);
	r = fma(r, fma(-x, r, 1.0), r);
	return r;
#else
	return 1.0 / x;
#endif
}
SSLM_HD double sqrt_estimate(double x) {  // x >= 1
#if defined(__CUDA_ARCH__)
	double y;
	asm("rsqrt.approx.ftz.f64 %0, %1;" : "=d"(y) : "d"(x));
	double s = x * y;
	const double h = 0.5 * y;
	s = fma(fma(-s, s, x), h, s);
	s = fma(fma(-s, s, x), h, s);
	return s;
#else
	return sqrt(x);
#endif
}

// ------------------------------------------------- gemmlowp-style requant prims
// SaturatingRoundingDoublingHighMul (src/intmath.cpp:230-236)
SSLM_HD int32_t srdhm(int32_t a, int32_t b) {
	int64_t r = ((int64_t)a * (int64_t)b + ((int64_t)1 << 30)) >> 31;
	return r > 2147483647ll ? 2147483647 : (int32_t)r;
}
// RoundingDivideByPOT, ties away from zero (src/intmath.cpp:245-263)
SSLM_HD int32_t rdivpot32(int32_t x, int e) {
	uint32_t mask = ((uint32_t)1 << e) - 1u;
	uint32_t rem = (uint32_t)x & mask;
	uint32_t thr = (mask >> 1) + (x < 0 ? 1u : 0u);
	return (x >> e) + (rem > thr ? 1 : 0);
}
SSLM_HD int64_t rdivpot64(int64_t x, int e) {
	uint64_t mask = ((uint64_t)1 << e) - 1u;
	uint64_t rem = (uint64_t)x & mask;
	uint64_t thr = (mask >> 1) + (x < 0 ? 1u : 0u);
	return (x >> e) + (rem > thr ? 1 : 0);
}
// ApplyWeightScaleFold on an int32 accumulator (src/forward/forward_sites.cpp:461-470)
SSLM_HD int32_t fold(int32_t acc, int32_t identity, int32_t mult, int32_t shift) {
	if (identity != 0) return acc;
	return rdivpot32(srdhm(acc, mult), shift);
}
// The same fold for the GEMM epilogue, where it runs once per output element. For a column
// that is not an identity, has 0 <= shift <= 31 and a multiplier other than INT32_MIN (the
// only operand that can saturate the doubling high multiply) the two rounding steps are
//   t = (acc * mult + 2^30) >> 31                       (no saturation possible)
//   fold = sign(t) * ((|t| + half) >> shift),  half = shift ? 2^(shift-1) : 0
// because rounding half away from zero equals the reference's mask / threshold test:
// for t >= 0 the test adds one iff the remainder >= 2^(shift-1); for t = -u it yields
// -(k+1) iff u mod 2^shift >= 2^(shift-1), else -k, with k = u >> shift. The magnitude
// (|t| + half) >> shift is also |fold|, which the row maximum wants. Other columns take fold().
SSLM_HD bool fold_is_plain(int32_t identity, int32_t mult, int32_t shift) {
	return identity == 0 && shift >= 0 && shift <= 31 && mult != (int32_t)(-2147483647 - 1);
}
SSLM_HD int32_t fold_plain(int32_t acc, int32_t mult, int32_t shift, uint32_t half, uint32_t* magnitude) {
	const int64_t p = (int64_t)acc * (int64_t)mult + ((int64_t)1 << 30);
	const int32_t t = (int32_t)(p >> 31);
	const uint32_t u = t < 0 ? 0u - (uint32_t)t : (uint32_t)t;
	const uint32_t a = (u + half) >> shift;
	*magnitude = a;
	return t < 0 ? (int32_t)(0u - a) : (int32_t)a;
}
// ApplyAmplifyingWeightScaleFold (src/forward/forward_sites.cpp:472-481) with
// SaturatingLeftShift32 (src/intmath.cpp:270-276)
SSLM_HD int32_t amp_fold(int32_t acc, int32_t identity, int32_t mult, int32_t exponent) {
	if (identity != 0) return acc;
	int32_t hi = srdhm(acc, mult);
	if (exponent >= 0) return rdivpot32(hi, exponent);
	int64_t w = (int64_t)hi << (-exponent);
	if (w > 2147483647ll) return 2147483647;
	if (w < -2147483648ll) return (int32_t)(-2147483647 - 1);
	return (int32_t)w;
}
SSLM_HD int64_t clamp127(int64_t v) { return v > 127 ? 127 : (v < -127 ? -127 : v); }

// --------------------------------------------------- dynamic-scale chain pieces
// NormalizeScale (src/intmath.cpp:296-301)
SSLM_HD void normalize_scale(int64_t d_prime, int64_t* dn, int* s) {
	int p = 63 - clz64((uint64_t)d_prime);
	*s = 30 - p;
	*dn = *s >= 0 ? (d_prime << *s) : (d_prime >> 1);
}
// DynamicScaleReciprocal (src/intmath.cpp:303-333): seed, 3 Newton steps, 2
// corrections, on the exact word sequence of the reference (it is also called on
// non-canonical mantissas, where only the operation sequence defines the result).
SSLM_HD_OUTLINE int64_t dyn_recip_sequence(int64_t dn) {
	const int64_t c48 = (2 * ((int64_t)48 << 31) + 17) / 34;
	const int64_t c32 = (2 * ((int64_t)32 << 31) + 17) / 34;
	int64_t y = c48 - ((int64_t)((uint64_t)c32 * (uint64_t)dn) >> 31);
	for (int i = 0; i < 3; ++i) {
		int64_t dn_y = sshr_to_i64(smul64(dn, y), 31);
		int64_t delta = (int64_t)(((uint64_t)1 << 32) - (uint64_t)dn_y);
		y = sshr_to_i64(smul64(y, delta), 31);
	}
	for (int i = 0; i < 2; ++i) {
		U128 res = ssub(U128{(uint64_t)1 << 62, 0}, smul64(y, dn));
		U128 r2 = U128{res.lo << 1, (res.hi << 1) | (res.lo >> 63)};
		if (sge(r2, sfrom64(dn))) {
			y = (int64_t)((uint64_t)y + 1u);
		} else if (!sge(r2, ssub(U128{0, 0}, sfrom64(dn)))) {
			y = (int64_t)((uint64_t)y - 1u);
		}
	}
	return y;
}
SSLM_HD int64_t dyn_recip(int64_t dn) {
	// On a normalised divisor (2^30 <= dn < 2^31, every funnel's case) the seed, the three
	// Newton steps and the two corrections land on round(2^62 / dn) = floor((2^62 + dn/2) / dn):
	// checked exhaustively, once, over all 2^30 such divisors against the word sequence
	// below. One division (a double estimate repaired with integers) replaces ~40 wide
	// multiplies; every other operand still takes the reference's operation sequence.
	if ((uint64_t)(dn - ((int64_t)1 << 30)) < ((uint64_t)1 << 30)) {
		const uint64_t num = ((uint64_t)1 << 62) + ((uint64_t)dn >> 1);
		uint64_t q = (uint64_t)((double)num * rcp_estimate((double)dn));
		int64_t r = (int64_t)(num - q * (uint64_t)dn);
		while (r < 0) { --q; r += dn; }
		while (r >= dn) { ++q; r -= dn; }
		return (int64_t)q;
	}
	return dyn_recip_sequence(dn);
}
// RequantTokenCodeWide (src/intmath.cpp:476-490): the 128-bit composite for any operands
SSLM_HD_OUTLINE int8_t requant_code_general(int64_t x, int64_t r, int s) {
	int exponent = 62 - s;  // [32,63]
	uint64_t ax = x < 0 ? (~(uint64_t)x + 1u) : (uint64_t)x;
	U128 prod = umul128x64(umul64(ax, (uint64_t)r), 127u);
	U128 num = uadd(U128{prod.lo << 1, (prod.hi << 1) | (prod.lo >> 63)}, U128{(uint64_t)1 << exponent, 0});
	U128 sh = ushr(num, exponent + 1);
	uint64_t mag = sh.lo > 127u ? 127u : sh.lo;
	int32_t q = (int32_t)mag;
	return (int8_t)(x < 0 ? -q : q);
}
SSLM_HD int8_t requant_code(int64_t x, int64_t r, int s) {
	int exponent = 62 - s;  // [32,63]
	uint64_t ax = x < 0 ? (~(uint64_t)x + 1u) : (uint64_t)x;
	// Everything the funnel hands over satisfies |x| <= 2^31, 2^31 < R <= 2^32; for an
	// exponent E >= 33 the composite floor((|x|*R*127 + 2^(E-1)) / 2^E) then needs 64-bit
	// words only: with P = |x|*R*127 = A*2^32 + b (0 <= b < 2^32) it equals
	// floor((A + 2^(E-33)) / 2^(E-32)), because the dropped fraction b/2^32 < 1 cannot carry
	// the sum over a multiple of the integer divisor.
	if (exponent >= 33 && ax <= ((uint64_t)1 << 31) && (uint64_t)r <= ((uint64_t)1 << 32)) {
		const uint64_t p = ax * (uint64_t)r;                                   // <= 2^63
		const uint64_t a = (p >> 32) * 127u + (((p & 0xFFFFFFFFull) * 127u) >> 32);
		uint64_t mag = (a + ((uint64_t)1 << (exponent - 33))) >> (exponent - 32);
		if (mag > 127u) mag = 127u;
		const int32_t qf = (int32_t)mag;
		return (int8_t)(x < 0 ? -qf : qf);
	}
	return requant_code_general(x, r, s);
}
// The same code with 32-bit words, for the operands a funnel hands over once its domain
// check passed: |x| <= 2^31, 2^31 < R < 2^32 and an exponent E >= 33. With p = |x| * R =
// hi * 2^32 + lo, floor(p * 127 / 2^32) = hi * 127 + floor(lo * 127 / 2^32) =: a (< 2^38), and
// the code is min(127, floor((a + 2^(E-33)) / 2^(E-32))) as derived above. Anything outside
// those ranges (R = 2^32 when the row maximum is a power of two, E = 32 when it is 1) takes
// requant_code. A Coder is per row; code_of is the per-element step.
struct Coder {
	int64_t r;
	int s;
	uint32_t r32;
	int sh;        // E - 32, in [1, 31] when narrow
	bool narrow;
};
SSLM_HD Coder make_coder(int64_t r, int s) {
	Coder c;
	c.r = r;
	c.s = s;
	c.r32 = (uint32_t)r;
	c.sh = 30 - s;
	c.narrow = (62 - s) >= 33 && (62 - s) <= 63 && r > 0 && (uint64_t)r < ((uint64_t)1 << 32);
	return c;
}
SSLM_HD uint32_t umulhi32(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
	return __umulhi(a, b);
#else
	return (uint32_t)(((uint64_t)a * b) >> 32);
#endif
}
SSLM_HD int32_t code_narrow(uint32_t ax, bool neg, const Coder& c) {
	const uint32_t hi = umulhi32(ax, c.r32), lo = ax * c.r32;
	const uint64_t a = (uint64_t)hi * 127u + umulhi32(lo, 127u);
	uint64_t mag = (a + ((uint64_t)1 << (c.sh - 1))) >> c.sh;
	if (mag > 127u) mag = 127u;
	const int32_t q = (int32_t)mag;
	return neg ? -q : q;
}
SSLM_HD int8_t code_of(int32_t x, const Coder& c) {
	if (c.narrow) return (int8_t)code_narrow(x < 0 ? 0u - (uint32_t)x : (uint32_t)x, x < 0, c);
	return requant_code_general((int64_t)x, c.r, c.s);
}
SSLM_HD int8_t code_of(int64_t x, const Coder& c) {
	const uint64_t ax = x < 0 ? (~(uint64_t)x + 1u) : (uint64_t)x;
	if (c.narrow && ax <= ((uint64_t)1 << 31)) return (int8_t)code_narrow((uint32_t)ax, x < 0, c);
	return requant_code_general(x, c.r, c.s);
}
SSLM_HD int64_t sat_add64(int64_t a, int64_t b) {
	int64_t out = (int64_t)((uint64_t)a + (uint64_t)b);
	if ((a >= 0) == (b >= 0) && (out >= 0) != (a >= 0)) return a >= 0 ? INT64_MAX : INT64_MIN;
	return out;
}
SSLM_HD int64_t sat_sub64(int64_t a, int64_t b) {
	int64_t out = (int64_t)((uint64_t)a - (uint64_t)b);
	if ((a >= 0) != (b >= 0) && (out >= 0) != (a >= 0)) return a >= 0 ? INT64_MAX : INT64_MIN;
	return out;
}
// CombineCarriedScale (src/forward/checked_chain_funnel.cpp:157-180)
SSLM_HD Scale combine(Scale a, Scale b) {
	int64_t e = sat_add64(sat_add64(a.e, b.e), 31);
	int64_t m = (int64_t)srdhm((int32_t)a.m, (int32_t)b.m);
	if (m < ((int64_t)1 << 30)) {
		m <<= 1;
		e -= 1;
	}
	return Scale{m, e};
}
SSLM_HD bool fits_i32(int64_t v) { return v >= -2147483648ll && v <= 2147483647ll; }

// The scalar half of RequantChainChecked (src/forward/checked_chain_funnel.cpp:257-336):
// given the row's max magnitude, produce (R, s) for the coder and the folded output
// scale; left-associated fold incoming[0..n), site constant, (Dn, -s), with the
// mantissa-range check after every step.
struct FunnelParams {
	int64_t r;
	int s;
	Scale out;
	int32_t status;
};
//
// The fold of the incoming scales and the site constant does not depend on the row maximum, so
// it is split off (funnel_prefold): a kernel derives it while the data it will reduce is still
// on its way, and only normalise + reciprocal + one combine (funnel_finish) follow the maximum.
struct FunnelFold {
	Scale run;            // incoming[0] (x) incoming[1] ... (x) site constant
	int32_t pre_status;   // a mantissa outside int32 before anything is folded
	int32_t fold_status;  // a folded mantissa outside int32
};
SSLM_HD FunnelFold funnel_prefold(const Scale* incoming, int n_incoming, Scale site_constant) {
	FunnelFold f;
	f.run = Scale{0, 0};
	f.pre_status = kOk;
	f.fold_status = kOk;
	for (int i = 0; i < n_incoming; ++i) {
		if (!fits_i32(incoming[i].m)) f.pre_status = kCarriedScaleMantissaOutOfDomain;
	}
	if (!fits_i32(site_constant.m)) f.pre_status = kCarriedScaleMantissaOutOfDomain;
	if (f.pre_status != kOk) return f;
	Scale run = n_incoming > 0 ? incoming[0] : site_constant;
	for (int i = 1; i < n_incoming; ++i) {
		run = combine(run, incoming[i]);
		if (!fits_i32(run.m)) f.fold_status = kCarriedScaleMantissaOutOfDomain;
	}
	if (n_incoming > 0) {
		run = combine(run, site_constant);
		if (!fits_i32(run.m)) f.fold_status = kCarriedScaleMantissaOutOfDomain;
	}
	f.run = run;
	return f;
}
SSLM_HD FunnelParams funnel_finish(uint64_t max_abs, const FunnelFold& f) {
	FunnelParams fp;
	fp.r = 0;
	fp.s = 0;
	fp.out = Scale{0, 0};
	fp.status = f.pre_status;
	if (fp.status != kOk) return fp;
	uint64_t d = max_abs < 1 ? 1 : max_abs;
	if (d > ((uint64_t)1 << 31)) {
		fp.status = kChainInputOutOfDomain;
		return fp;
	}
	int64_t dn;
	normalize_scale((int64_t)d, &dn, &fp.s);
	fp.r = dyn_recip(dn);
	fp.status = f.fold_status;
	const Scale run = combine(f.run, Scale{dn, -(int64_t)fp.s});
	if (!fits_i32(run.m)) fp.status = kCarriedScaleMantissaOutOfDomain;
	fp.out = run;
	return fp;
}
SSLM_HD FunnelParams funnel_params(uint64_t max_abs, const Scale* incoming, int n_incoming,
                                   Scale site_constant) {
	return funnel_finish(max_abs, funnel_prefold(incoming, n_incoming, site_constant));
}

// ----------------------------------------------------------- exact divisions
// floor(a / b) for b > 0 (FloorDivI64, src/forward/forward_sites.cpp:399-408)
SSLM_HD int64_t floor_div(int64_t a, int64_t b) {
	int64_t q = a / b, r = a % b;
	return (r != 0 && r < 0) ? q - 1 : q;
}
// floor((h << 32) / root) for an activation code |h| <= 127 and root >= 1: the per-element
// division of RmsNormSite. A double-precision estimate (numerator < 2^39, so the estimate is
// within one of the quotient) corrected by exact integer arithmetic, then floored toward
// minus infinity for negative h.
SSLM_HD int64_t floor_div_h32(int h, int64_t root, double inv_root) {
	const uint64_t num = (uint64_t)(h < 0 ? -h : h) << 32;
	uint64_t q = (uint64_t)((double)num * inv_root);
	int64_t r = (int64_t)(num - q * (uint64_t)root);
	while (r < 0) { --q; r += root; }
	while (r >= root) { ++q; r -= root; }
	if (h >= 0) return (int64_t)q;
	return -(int64_t)q - (r != 0 ? 1 : 0);
}
// num / den (truncating, both non-negative, den >= 1) when the quotient is known to
// be below 2^20: a double-precision estimate corrected by exact integer arithmetic.
SSLM_HD uint64_t udiv_small_quotient(uint64_t num, uint64_t den, double inv_den) {
	uint64_t q = (uint64_t)((double)num * inv_den);
	int64_t r = (int64_t)(num - q * den);
	while (r < 0) { --q; r += (int64_t)den; }
	while (r >= (int64_t)den) { ++q; r -= (int64_t)den; }
	return q;
}
// ISqrt, 32 restoring digit steps (src/intmath.cpp:502-524)
SSLM_HD int64_t isqrt64(int64_t n) {
	if (n >= 0) {
		// the digit recurrence below yields floor(sqrt(n)); so does a double-precision
		// estimate repaired with exact integer squares (the estimate is within 1)
		if (n == 0) return 0;
		uint64_t r = (uint64_t)sqrt_estimate((double)n);
		while (r * r > (uint64_t)n) --r;
		while ((r + 1) * (r + 1) <= (uint64_t)n) ++r;
		return (int64_t)r;
	}
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

// -------------------------------------------------------------- q/k/v bias (BIA1)
// C28 bias reconciliation: acc_i += round_half_away(B_i * R_a / 2^(q_B + 62 + e_a)) with
// q_B = 30, R_a = Recip(S[input].m), e_a = S[input].e (ApplyBiasReconcileRow,
// src/forward/forward_sites.cpp:1015-1036; BiasReconcileWide, src/intmath.cpp:397-418).
// The composed exponent must lie in [0, 63] (RoundingDivideByPotComposedExponentInDomain,
// src/intmath.cpp:381-395).
SSLM_HD bool bias_exponent_in_domain(int64_t e_a, int* exponent) {
	if (e_a < -92 || e_a > -29) return false;
	*exponent = (int)(92 + e_a);
	return true;
}
// false when the rounded term does not fit int64 (the reference refuses the row)
SSLM_HD_OUTLINE bool bias_reconcile(int64_t b, int64_t r_a, int exponent, int64_t* term) {
	const U128 w = smul64(b, r_a);
	const uint64_t mask = ((uint64_t)1 << exponent) - 1u;     // exponent <= 63
	const bool neg = (int64_t)w.hi < 0;
	const uint64_t rem = w.lo & mask;
	const uint64_t thr = (mask >> 1) + (neg ? 1u : 0u);
	U128 sh;                                                   // arithmetic shift right by exponent
	if (exponent == 0) {
		sh = w;
	} else {
		sh.lo = (w.lo >> exponent) | (w.hi << (64 - exponent));
		sh.hi = (uint64_t)((int64_t)w.hi >> exponent);
	}
	if (rem > thr) {
		sh.lo += 1u;
		if (sh.lo == 0u) sh.hi += 1u;
	}
	*term = (int64_t)sh.lo;
	return sh.hi == ((int64_t)sh.lo < 0 ? ~0ull : 0ull);
}
// acc + term, false on int64 overflow (CheckBiasAccumulateMagnitudeDomain,
// src/forward/checked_chain_funnel.cpp:454-482)
SSLM_HD bool bias_accumulate(int64_t acc, int64_t term, int64_t* out) {
	const uint64_t ua = (uint64_t)acc, ub = (uint64_t)term, sum = ua + ub;
	*out = (int64_t)sum;
	return !((((ua ^ ub) >> 63) == 0) && (((ua ^ sum) >> 63) != 0));
}

// ---------------------------------------------------------------- site scalars
// LandingRescale (src/forward/forward_sites.cpp:513-653):
// round_half_away((code * m_a * r_t) / 2^(62-(e_a-e_t))), exact left shift when the
// composed exponent is negative; reports "outside +-127 or lost" (the saturation
// counter's predicate) and "does not fit int64".
SSLM_HD_OUTLINE int64_t landing_rescale_general(int64_t code, int64_t m_a, int64_t r_t, int64_t k,
                                                bool* saturated, bool* exceeded_int64) {
	const bool neg = (code < 0) != (m_a < 0);
	uint64_t ac = code < 0 ? (~(uint64_t)code + 1u) : (uint64_t)code;
	uint64_t am = m_a < 0 ? (~(uint64_t)m_a + 1u) : (uint64_t)m_a;
	U128 mag = umul128x64(umul64(ac, am), (uint64_t)r_t);
	bool over_clamp, over_i64;
	int64_t raw;
	if (k >= 0) {
		U128 q = ushr(uadd(uadd(mag, mag), ushl(U128{1, 0}, (int)k)), (int)k + 1);
		over_clamp = q.hi != 0 || q.lo > 127;
		over_i64 = q.hi != 0 || q.lo > (uint64_t)INT64_MAX;
		raw = (int64_t)q.lo;
	} else {
		int shift = (int)(-k);
		U128 sh = ushl(mag, shift);
		if (shift >= 128) {
			over_clamp = (mag.lo | mag.hi) != 0;
			over_i64 = over_clamp;
		} else {
			U128 back = ushr(sh, shift);
			bool lost = back.lo != mag.lo || back.hi != mag.hi;
			over_clamp = lost || sh.hi != 0 || sh.lo > 127;
			over_i64 = lost || sh.hi != 0 || sh.lo > (uint64_t)INT64_MAX;
		}
		raw = (int64_t)sh.lo;
	}
	if (neg) raw = (int64_t)(0u - (uint64_t)raw);
	if (saturated) *saturated = over_clamp || raw < -127 || raw > 127;
	if (exceeded_int64) *exceeded_int64 = over_i64;
	return raw;
}
SSLM_HD int64_t landing_rescale(int64_t code, int64_t m_a, int64_t r_t, int64_t e_a, int64_t e_t,
                                bool* saturated, bool* exceeded_int64) {
	const bool neg = (code < 0) != (m_a < 0);
	uint64_t ac = code < 0 ? (~(uint64_t)code + 1u) : (uint64_t)code;
	uint64_t am = m_a < 0 ? (~(uint64_t)m_a + 1u) : (uint64_t)m_a;
	int64_t k = sat_sub64(62, sat_sub64(e_a, e_t));
	if (k > 4096) k = 4096;
	if (k < -4096) k = -4096;
	// The operands every in-domain call site produces (|code| <= 2^31, |m_a| < 2^31,
	// 0 < r_t <= 2^32, 33 <= k <= 94) keep the composite inside 64-bit words: with
	// P = |code|*|m_a|*r_t = A*2^32 + b the rounded quotient floor((P + 2^(k-1)) / 2^k) is
	// floor((A + 2^(k-33)) / 2^(k-32)). Anything else takes the general 128-bit route.
	if (k >= 33 && k <= 94 && ac <= ((uint64_t)1 << 31) && am < ((uint64_t)1 << 31) && r_t > 0 &&
	    (uint64_t)r_t <= ((uint64_t)1 << 32)) {
		const uint64_t p = am * (uint64_t)r_t;                                        // < 2^63
		const uint64_t a = ac * (p >> 32) + ((ac * (p & 0xFFFFFFFFull)) >> 32);       // floor(P / 2^32)
		const uint64_t qm = (a + ((uint64_t)1 << (k - 33))) >> (k - 32);
		if (saturated) *saturated = qm > 127;
		if (exceeded_int64) *exceeded_int64 = false;
		return neg ? -(int64_t)qm : (int64_t)qm;
	}
	return landing_rescale_general(code, m_a, r_t, k, saturated, exceeded_int64);
}
// RopeApplyPair + ClampRopeCode (src/intmath.cpp:782-792, forward_sites.cpp:655-661, :750-758)
SSLM_HD void rope_pair_clamped(int32_t x, int32_t y, int32_t c, int32_t s, int8_t* ox, int8_t* oy) {
	int64_t xr = (int64_t)x * c - (int64_t)y * s;
	int64_t yr = (int64_t)x * s + (int64_t)y * c;
	*ox = (int8_t)clamp127(rdivpot64(xr, 30));
	*oy = (int8_t)clamp127(rdivpot64(yr, 30));
}
// SiluSigmoidQ15 (src/silu_lut.cpp:16-67); e in [-80, 8] (checked by the caller)
SSLM_HD int32_t silu_sigmoid_q15(const int32_t* table, int32_t code, int64_t m, int e) {
	int64_t term = (int64_t)code * m;
	int shift = e + 17;
	int64_t pos = shift >= 0 ? (int64_t)((uint64_t)term << shift) : rdivpot64(term, -shift);
	const int64_t hi_dom = (int64_t)1024 << 12;
	pos += hi_dom / 2;
	if (pos < 0) pos = 0;
	else if (pos > hi_dom) pos = hi_dom;
	int64_t i0 = pos >> 12;
	if (i0 > 1023) i0 = 1023;
	int64_t frac = pos - (i0 << 12);
	int64_t lo = table[i0], hi = table[i0 + 1];
	return (int32_t)(lo + rdivpot64(frac * (hi - lo), 12));
}
SSLM_HD bool silu_scale_in_domain(Scale g) {
	const int64_t mx = ((int64_t)1 << 31) - 1;
	return g.m >= -mx && g.m <= mx && g.e >= -80 && g.e <= 8;
}

// Q30 coefficients of the i-exp polynomial: floor(ln2 * 2^30), floor(1.353 * 2^30),
// floor((0.344/0.3585) * 2^30) (include/superslm/intmath.h:518-527).
#define SSLM_IEXP_LN2_Q 744261117ll
#define SSLM_IEXP_B_Q 1452772687ll
#define SSLM_IEXP_CA_Q 1030312935ll

struct IExpConsts { int64_t q_ln2, q_b, q_c; };
// IExpScaleConstants with the production coefficients, all formats 30
// (src/intmath.cpp:702-778). 0 ok, else out of domain.
SSLM_HD_OUTLINE int iexp_scale_constants(int64_t m, int64_t e, IExpConsts* out) {
	int64_t sh_l = sat_add64(92, e);
	int64_t sh_c = sat_add64(154, sat_add64(e, e));
	int64_t mn = sh_l < sh_c ? sh_l : sh_c;
	if (mn < 0) return 2;
	uint64_t rm = (uint64_t)dyn_recip(m);
	U128 n_ln2 = umul64((uint64_t)SSLM_IEXP_LN2_Q, rm);
	U128 n_b = umul64((uint64_t)SSLM_IEXP_B_Q, rm);
	U128 n_c = umul128x64(umul64(rm, rm), (uint64_t)SSLM_IEXP_CA_Q);
	U128 f_ln2 = sh_l >= 128 ? U128{0, 0} : ushr(n_ln2, (int)sh_l);
	U128 f_b = sh_l >= 128 ? U128{0, 0} : ushr(n_b, (int)sh_l);
	U128 f_c = sh_c >= 128 ? U128{0, 0} : ushr(n_c, (int)sh_c);
	if (f_ln2.hi != 0 || f_ln2.lo > (uint64_t)INT64_MAX) return 3;
	if (f_b.hi != 0 || f_b.lo > (uint64_t)INT64_MAX) return 3;
	if (f_c.hi != 0 || f_c.lo > (uint64_t)INT64_MAX) return 3;
	out->q_ln2 = (int64_t)f_ln2.lo;
	out->q_b = (int64_t)f_b.lo;
	out->q_c = (int64_t)f_c.lo;
	return 0;
}
// largest row peak the Q15 normalisation can carry (checked_chain_funnel.h:563)
#define SSLM_SOFTMAX_MAX_SAFE (((int64_t)1 << 62) >> 15)
// CheckSoftmaxRowWidthDomain (src/forward/checked_chain_funnel.cpp:520-583)
SSLM_HD_OUTLINE bool softmax_width_in_domain(int64_t q_b, int64_t q_c, uint64_t width, int64_t* peak) {
	if (q_c < 0 || width == 0) return false;
	U128 m = uadd(smul64(q_b, q_b), U128{(uint64_t)q_c, 0});
	if (m.hi != 0 || m.lo > (uint64_t)SSLM_SOFTMAX_MAX_SAFE) return false;
	*peak = (int64_t)m.lo;
	if (m.lo != 0 && width > (uint64_t)(INT64_MAX / (int64_t)m.lo)) return false;
	return true;
}
// One softmax element: IExpConstruct + IExpEvaluate on a shifted score q <= 0 followed
// by SoftmaxRowQ15's per-element bound (src/intmath.cpp:580-668, :870-888), specialised
// to constants that passed the width gate with q_ln2 <= q_b (so |q_b| < 2^24,
// 1 <= q_ln2 < 2^24 and every intermediate fits 64 bits). Returns false when the
// reference would refuse the element.
SSLM_HD bool iexp_element(int64_t q, const IExpConsts& c, int64_t peak, int64_t* value) {
	int64_t clip_lo = -(int64_t)30 * c.q_ln2;
	int64_t clipped = q < clip_lo ? clip_lo : q;
	uint32_t z = (uint32_t)(-clipped) / (uint32_t)c.q_ln2;
	int64_t q_p = clipped + (int64_t)z * c.q_ln2;
	int64_t base = q_p + c.q_b;
	int64_t v = (base * base + c.q_c) >> z;
	*value = v;
	return peak >= 1 && v >= 0 && v <= peak;
}

}  // namespace sslm
