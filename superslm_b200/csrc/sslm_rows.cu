// Per-row sites of the integer forward pass as fused CUDA kernels: one thread block
// owns one row (one token of one sequence) and carries it through every step that
// needs only that row -- the dynamic-scale requant "funnel", RMSNorm, q/k/v
// post-processing (K/V landing, RoPE, page write, softmax constants), the residual
// reconciliation and the SwiGLU activation. All of these are HBM/latency-bound integer
// work; rows are independent, so the grid is simply the row count.
#include <cuda_runtime.h>

#include "sslm_kernels.h"

namespace sslm {

// per-row lookup tables indexed by an int8 code: 256 int64 values + 256 flag bytes
constexpr int kLutBytes = 256 * 8 + 256;

// ------------------------------------------------------------ block reductions
// Every row kernel is a chain of dependent phases, so a reduction's latency is paid in full
// each time. These cost one barrier: each warp reduces with the warp-reduce instruction and
// posts its value in one of two alternating banks of shared words, and after the barrier
// every thread folds the (at most 32) posted values itself. A bank is rewritten only two
// reductions later, i.e. after a barrier that every reader of its old contents has passed.
constexpr int kRedBank = 32;                   // one slot per warp
constexpr int kRedMisc = 2 * kRedBank;         // four more words for single values handed to the block
constexpr int kRedWords = kRedMisc + 4;
constexpr int kRedBytes = kRedWords * 8;
struct Red {
	unsigned long long* w;
	int phase;
};
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
	const uint32_t hi = (uint32_t)(v >> 32), lo = (uint32_t)v;
	const uint32_t mh = __reduce_max_sync(0xffffffffu, hi);
	const uint32_t ml = __reduce_max_sync(0xffffffffu, hi == mh ? lo : 0u);
	return ((unsigned long long)mh << 32) | ml;
}
__device__ __forceinline__ long long warp_sum_i64(long long v) {
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
	return v;
}
// Every thread gets the result. All threads of the block must call these together.
__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, Red& red) {
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
	unsigned long long* bank = red.w + red.phase * kRedBank;
	red.phase ^= 1;
	v = warp_max_u64(v);
	if (lane == 0) bank[warp] = v;
	__syncthreads();
	unsigned long long m = bank[0];
	for (int w = 1; w < nw; ++w) {
		const unsigned long long t = bank[w];
		m = t > m ? t : m;
	}
	return m;
}
// small: every thread's addend and the warp totals fit 32 bits (a cheaper warp step)
__device__ __forceinline__ long long block_sum_i64(long long v, Red& red, bool small = false) {
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
	unsigned long long* bank = red.w + red.phase * kRedBank;
	red.phase ^= 1;
	if (small) v = (long long)__reduce_add_sync(0xffffffffu, (uint32_t)v);
	else v = warp_sum_i64(v);
	if (lane == 0) bank[warp] = (unsigned long long)v;
	__syncthreads();
	long long s = (long long)bank[0];
	for (int w = 1; w < nw; ++w) s += (long long)bank[w];
	return s;
}

__device__ __forceinline__ unsigned long long abs_u64(int64_t v) {
	return v < 0 ? (~(unsigned long long)v + 1ull) : (unsigned long long)v;
}
__device__ __forceinline__ int64_t load_wide(const RowBatch& b, int row, int col) {
	const size_t i = (size_t)row * b.wide_ld + col;
	return b.wide64 ? ((const int64_t*)b.wide)[i] : (int64_t)((const int32_t*)b.wide)[i];
}
// Cooperative asynchronous 16-byte copies, global -> shared (both 16-byte aligned, bytes a
// multiple of 16), through L2. The kernels below issue all of a row's input copies back to
// back and wait once (stage_wait + a barrier), so the row pays one memory round trip instead
// of one per dependent phase, and no registers are held while the copies are in flight.
//
// Order against the previous kernel: inputs that were written at least two launches back
// (the stream row and scales of earlier sites, weights, tables) are fetched BEFORE pdl_wait(),
// while the projection that feeds this kernel is still running; what that projection writes
// (its output row, the reduced row maximum) and the row's status word are read only after
// pdl_wait(), and past the L1 (cp.async.cg / __ldcg), which may hold lines fetched earlier.
__device__ __forceinline__ void stage16(void* dst, const void* src, int bytes) {
	const char* s = (const char*)src;
	const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
#pragma unroll 1
	for (int i = threadIdx.x * 16; i < bytes; i += blockDim.x * 16)
		asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d + i), "l"(s + i) : "memory");
}
__device__ __forceinline__ void stage_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// the row of folded int32 accumulators can be staged with 16-byte copies
__device__ __forceinline__ bool wide_stageable(const RowBatch& b, int cols) {
	return !b.wide64 && (b.wide_ld & 3) == 0 && (cols & 3) == 0;
}
__device__ __forceinline__ const int32_t* wide_row32(const RowBatch& b, int row) {
	return (const int32_t*)b.wide + (size_t)row * b.wide_ld;
}
// codes of a staged int32 row, four per thread and pass (src 16-byte, dst 4-byte aligned)
__device__ __forceinline__ void code_words(const int32_t* src, int n4, const Coder& cd, int8_t* dst) {
	for (int i = threadIdx.x; i < n4; i += blockDim.x) {
		const int4 p = ((const int4*)src)[i];
		const uint32_t c0 = (uint8_t)code_of(p.x, cd);
		const uint32_t c1 = (uint8_t)code_of(p.y, cd);
		const uint32_t c2 = (uint8_t)code_of(p.z, cd);
		const uint32_t c3 = (uint8_t)code_of(p.w, cd);
		((uint32_t*)dst)[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
	}
}
// After pdl_wait(): thread 0 fetches the GEMM-reduced row maxima of slots [slot, slot + count)
// (leaving them zero for their next producer) and the row's status word into the misc words;
// they are readable after the caller's next barrier, which also completes the staged copies.
__device__ __forceinline__ void fetch_row_words(const RowBatch& b, int row, int slot, int count, Red& red) {
	if (threadIdx.x == 0) {
		for (int i = 0; i < count; ++i) {
			red.w[kRedMisc + i] = __ldcg(&b.rowmax[row * 4 + slot + i]);
			b.rowmax[row * 4 + slot + i] = 0ull;
		}
		red.w[kRedMisc + 3] = (unsigned long long)(uint32_t)__ldcg(&b.status[row]);
	}
}
__device__ __forceinline__ bool row_refused(const Red& red) { return red.w[kRedMisc + 3] != 0ull; }

// Funnel over a row staged in shared memory (RequantChainChecked,
// src/forward/checked_chain_funnel.cpp:257-364). Codes go to out_g (global) and, when
// non-null, out_s (shared). Every thread returns the same status; on failure nothing
// is written.
//
// block_code is the part after the row maximum is known to every thread (the caller's
// reduction barrier must also have made w[] visible); block_funnel takes the maximum itself.
// `fold` is the scale fold of the site, derived ahead of the maximum (funnel_prefold).
// sumsq (optional): this thread's sum of squares of the codes it wrote, for the RMSNorm that
// follows a residual site in the same kernel.
__device__ int32_t block_code(const int64_t* w, int n, unsigned long long mx, const FunnelFold& fold,
                              int8_t* out_g, int8_t* out_s, Scale* out_scale, long long* sumsq = nullptr) {
	const FunnelParams fp = funnel_finish(mx, fold);
	if (fp.status != kOk) return fp.status;
	const Coder cd = make_coder(fp.r, fp.s);
	if ((n & 3) == 0) {
		// four codes per thread and pass: word stores to global and shared memory
		int sq = 0;
		for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
			uint32_t pk = 0;
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				const int c = code_of(w[4 * i + j], cd);
				sq += c * c;
				pk |= (uint32_t)(uint8_t)c << (8 * j);
			}
			if (out_g) ((uint32_t*)out_g)[i] = pk;
			if (out_s) ((uint32_t*)out_s)[i] = pk;
		}
		if (sumsq) *sumsq = sq;
	} else {
		long long sq = 0;
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) {
			const int8_t c = code_of(w[i], cd);
			sq += (int)c * (int)c;
			if (out_g) out_g[i] = c;
			if (out_s) out_s[i] = c;
		}
		if (sumsq) *sumsq = sq;
	}
	if (threadIdx.x == 0 && out_scale) *out_scale = fp.out;
	return kOk;
}
__device__ int32_t block_funnel(const int64_t* w, int n, const Scale* incoming, int n_incoming, Scale site,
                                int8_t* out_g, int8_t* out_s, Scale* out_scale, Red& red) {
	const FunnelFold fold = funnel_prefold(incoming, n_incoming, site);
	unsigned long long mx = 0;
#pragma unroll 1
	for (int i = threadIdx.x; i < n; i += blockDim.x) {
		unsigned long long a = abs_u64(w[i]);
		mx = a > mx ? a : mx;
	}
	mx = block_max_u64(mx, red);
	return block_code(w, n, mx, fold, out_g, out_s, out_scale);
}

// RmsNormSite (src/forward/forward_sites.cpp:410-459) on codes h[n] (global or shared):
// root = max(isqrt(floor((sum h^2) << 32 / n)), 1); wide_i = floor((h_i << 32) / root) * g_i;
// funnel with no incoming scale. wide: shared int64[n].
// ss_partial (optional): this thread's share of sum h^2, already taken by whoever wrote h.
__device__ int32_t block_rmsnorm(const int8_t* h, const int8_t* gain, int n, Scale site, int64_t* wide,
                                 int8_t* out_g, Scale* out_scale, int64_t* lut, Red& red,
                                 const long long* ss_partial = nullptr) {
	// four codes per word where the rows allow it: these passes are short dependent chains,
	// and a quarter of the iterations is a quarter of the latency
	const bool vec = (n & 3) == 0 && ((((uintptr_t)h) | ((uintptr_t)gain)) & 3) == 0;
	const double inv_n = rcp_estimate((double)n);
	long long ss = 0;
	if (ss_partial != nullptr) {
		ss = *ss_partial;
	} else if (vec) {
		for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
			const uint32_t w = ((const uint32_t*)h)[i];
			const int v0 = (int8_t)w, v1 = (int8_t)(w >> 8), v2 = (int8_t)(w >> 16), v3 = (int8_t)(w >> 24);
			ss += v0 * v0 + v1 * v1 + v2 * v2 + v3 * v3;
		}
	} else {
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) {
			const int v = h[i];
			ss += v * v;
		}
	}
	ss = block_sum_i64(ss, red, n <= (1 << 20));   // 127^2 * 2^20 / warps fits 32 bits per warp
	// floor((sum << 32) / n): non-negative operands, an estimated quotient repaired exactly
	int64_t root = isqrt64((int64_t)udiv_small_quotient((uint64_t)ss << 32, (uint64_t)n, inv_n));
	if (root < 1) root = 1;
	// floor((h << 32) / root) depends only on the code: one division per code value, not per element
	const double inv_root = rcp_estimate((double)root);
	for (int t = threadIdx.x; t < 255; t += blockDim.x) lut[t] = floor_div_h32(t - 127, root, inv_root);
	__syncthreads();
	unsigned long long mx = 0;
	if (vec) {
		for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
			const uint32_t hw = ((const uint32_t*)h)[i], gw = ((const uint32_t*)gain)[i];
			int64_t v[4];
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				v[j] = lut[(int)(int8_t)(hw >> (8 * j)) + 127] * (int64_t)(int8_t)(gw >> (8 * j));
				const unsigned long long a = abs_u64(v[j]);
				mx = a > mx ? a : mx;
			}
			*(longlong2*)&wide[4 * i] = make_longlong2(v[0], v[1]);
			*(longlong2*)&wide[4 * i + 2] = make_longlong2(v[2], v[3]);
		}
	} else {
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) {
			const int64_t v = lut[(int)h[i] + 127] * (int64_t)gain[i];
			wide[i] = v;
			const unsigned long long a = abs_u64(v);
			mx = a > mx ? a : mx;
		}
	}
	mx = block_max_u64(mx, red);   // its barrier also publishes wide[]
	return block_code(wide, n, mx, funnel_prefold(nullptr, 0, site), out_g, nullptr, out_scale);
}

__device__ __forceinline__ void set_status(const RowBatch& b, int row, int32_t st, int site, int layer) {
	if (threadIdx.x == 0 && st != kOk) atomicCAS(&b.status[row], 0, pack_status(st, site, layer));
}

// ------------------------------------------------------------------- kernels
// Start of a call for each row: embed the token (EmbedEntry,
// src/forward/forward_sites.cpp:763-787) or pick up the sequence's stored mid-token
// stream, then the first layer's attention RMSNorm.
__global__ void __launch_bounds__(kRowThreads)
k_begin(RowBatch b, Dims d, const int8_t* embed, Scale c_embed, const RowSource* src,
        const LayerDev* layer) {
	pdl_wait();
	pdl_release();
	extern __shared__ __align__(16) unsigned char smem[];
	Red red{(unsigned long long*)smem, 0};
	int64_t* lut = (int64_t*)(smem + kRedBytes);
	int64_t* wide = (int64_t*)(smem + kRedBytes + kLutBytes);
	const int r = blockIdx.x, n = d.hidden;
	int8_t* x = b.x + (size_t)r * n;
	if (threadIdx.x == 0) {
		b.status[r] = 0;
		b.sat[r] = 0ull;
		b.done[r] = 0;
	}
	for (int i = threadIdx.x; i < b.sat_ld; i += blockDim.x) b.sat_layer[(size_t)r * b.sat_ld + i] = 0u;
	int32_t st = kOk;
	int site = kSiteEmbed;
	const RowSource s = src[r];
	if (s.hidden != nullptr) {
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) x[i] = s.hidden[i];
		if (threadIdx.x == 0) b.xs[r] = *s.scale;
	} else {
		const int8_t* e = embed + (size_t)b.rows[r].token * n;
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) wide[i] = e[i];
		__syncthreads();
		st = block_funnel(wide, n, nullptr, 0, c_embed, x, nullptr, &b.xs[r], red);
	}
	__syncthreads();
	if (st == kOk && layer != nullptr) {
		site = kSiteAttnNorm;
		st = block_rmsnorm(x, layer->g_attn, n, layer->c_attn_norm, wide, b.nrm + (size_t)r * n,
		                   &b.ns[r], lut, red);
	}
	set_status(b, r, st, site, b.layer);
}

// RMSNorm of the stream with the given gain (used for the final norm before the head).
__global__ void __launch_bounds__(kRowThreads)
k_rmsnorm(RowBatch b, Dims d, const int8_t* gain, Scale site) {
	pdl_wait();
	pdl_release();
	extern __shared__ __align__(16) unsigned char smem[];
	Red red{(unsigned long long*)smem, 0};
	int64_t* lut = (int64_t*)(smem + kRedBytes);
	int64_t* wide = (int64_t*)(smem + kRedBytes + kLutBytes);
	const int r = blockIdx.x, n = d.hidden;
	if (b.status[r] != 0) return;
	const int32_t st = block_rmsnorm(b.x + (size_t)r * n, gain, n, site, wide, b.nrm + (size_t)r * n,
	                                 &b.ns[r], lut, red);
	set_status(b, r, st, kSiteFinalNorm, b.layer);
}

// After the fused q/k/v projection: q funnel (ProjectAndFunnel's tail,
// forward_sites.cpp:1114-1146), K/V landing with the saturation counter (LandTokenKVRow
// :1397-1415, LandingRescale :513-653), RoPE on q and on the landed K (:1748-1787,
// RopeApplySite :663-761), the page write, and the per-kv-head softmax constants with
// their domain gates (:1806-1856).
__global__ void __launch_bounds__(kRowThreads)
k_qkv_post(RowBatch b, Dims d, const LayerDev* layer, int layer_index, KvPoolDev pool,
           const int32_t* rope_cos, const int32_t* rope_sin) {
	extern __shared__ __align__(16) unsigned char smem[];
	Red red{(unsigned long long*)smem, 0};
	int32_t* st_kv = (int32_t*)(smem + kRedBytes);             // 16 ints
	int8_t* sq = (int8_t*)(smem + kRedBytes + 64);             // hidden
	int8_t* sk = sq + d.hidden;                                // kv_hidden
	const int r = blockIdx.x, H = d.hidden, hd = d.head_dim, half = hd / 2;
	int32_t* sw = (int32_t*)(smem + kRedBytes + 64 + ((H + d.kv_hidden + 15) & ~15));   // staged q|k|v row
	int32_t* s_cos = sw + d.qkv_rows;                                                    // staged RoPE row
	int32_t* s_sin = s_cos + half;
	const bool vec = wide_stageable(b, d.qkv_rows) && (half & 3) == 0;
	// ahead of the projection: the normed row's scale (written by the previous residual site),
	// the position, its RoPE row and page, the site constant
	const LayerDev& lw = *layer;
	const Scale ns = b.ns[r];
	const Scale c_q = lw.c_q;
	const int pos = b.rows[r].pos;
	if (vec) {
		stage16(s_cos, rope_cos + (size_t)pos * half, half * 4);
		stage16(s_sin, rope_sin + (size_t)pos * half, half * 4);
	}
	const int32_t* cos_row = vec ? s_cos : rope_cos + (size_t)pos * half;   // table row = position
	const int32_t* sin_row = vec ? s_sin : rope_sin + (size_t)pos * half;
	const int page = b.rows[r].pages[pos / kPageTokens];
	const int slot = pos % kPageTokens;
	const FunnelFold fold_q = funnel_prefold(&ns, 1, c_q);
	// the landing constants (weights) of the kv head this thread's first K / V element belongs to
	int64_t k_rt0 = 0, k_et0 = 0, v_rt0 = 0, v_et0 = 0;
	if ((int)threadIdx.x < d.kv_hidden) {
		const int h0 = (int)threadIdx.x / hd;
		k_rt0 = lw.k_recip[3 * h0 + 2]; k_et0 = lw.k_recip[3 * h0 + 1];
		v_rt0 = lw.v_recip[3 * h0 + 2]; v_et0 = lw.v_recip[3 * h0 + 1];
	}
	pdl_wait();
	pdl_release();
	if (vec) stage16(sw, wide_row32(b, r), d.qkv_rows * 4);
	fetch_row_words(b, r, 0, 1, red);
	stage_wait();
	__syncthreads();
	const unsigned long long mx = red.w[kRedMisc];
	if (row_refused(red)) return;

	auto wv = [&](int i) -> int64_t { return vec ? (int64_t)sw[i] : load_wide(b, r, i); };
	// q/k/v bias (BIA1): term_i = round(B_i * Recip(S[x].m) / 2^(92 + S[x].e)) joins the folded
	// accumulator (after the LoRA delta) before the q funnel and before the K/V landing
	// (ApplyBiasReconcileRow, forward_sites.cpp:1015-1036). The exponent gate and R_a are per
	// row; a term or a sum that leaves int64 refuses the row.
	const bool any_bias = lw.b_q != nullptr || lw.b_k != nullptr || lw.b_v != nullptr;
	int bexp = 0;
	int64_t r_a = 0;
	bool bias_gate = true;
	if (any_bias) {
		r_a = dyn_recip(ns.m);
		bias_gate = bias_exponent_in_domain(ns.e, &bexp);
	}
	auto biased = [&](int64_t acc, const int64_t* bias, int i, bool* ok) -> int64_t {
		int64_t term, sum;
		const bool t_ok = bias_reconcile(bias[i], r_a, bexp, &term);
		const bool s_ok = bias_accumulate(acc, term, &sum);
		*ok = t_ok && s_ok;
		return sum;
	};
	unsigned long long mxq = mx;
	if (lw.b_q != nullptr) {
		if (!bias_gate) {
			set_status(b, r, kRoundingDivideExponentOutOfDomain, kSiteQ, b.layer);
			return;
		}
		// the row maximum the GEMM reduced does not include the bias: take it here
		unsigned long long lmx = 0;
		int bad = 0;
#pragma unroll 1
		for (int i = threadIdx.x; i < H; i += blockDim.x) {
			bool ok;
			const unsigned long long a = abs_u64(biased(wv(i), lw.b_q, i, &ok));
			if (!ok) bad = 1;
			lmx = a > lmx ? a : lmx;
		}
		bad = __syncthreads_or(bad);
		if (bad != 0) {
			set_status(b, r, kBiasReconcileProductOutOfDomain, kSiteQ, b.layer);
			return;
		}
		mxq = block_max_u64(lmx, red);
	}
	const FunnelParams fp = funnel_finish(mxq, fold_q);
	if (fp.status != kOk) {
		set_status(b, r, fp.status, kSiteQ, b.layer);
		return;
	}
	// softmax constants per kv head: sm = Combine(S[q], softmax_khead) -> C30 constants -> width gate.
	// A serial scalar derivation that needs only the q scale: the last warp's first lanes run it
	// now, while the other warps code the q row, instead of after everything else.
	const int kv_lane = (int)threadIdx.x - ((int)blockDim.x - 32);
	if (kv_lane >= 0 && kv_lane < d.kv_heads) {
		const int h = kv_lane;
		int32_t st = kOk;
		const Scale kh = Scale{lw.sm_khead[2 * h], lw.sm_khead[2 * h + 1]};
		SoftmaxConsts sc;
		sc.c = IExpConsts{0, 0, 0};
		sc.peak = 0;
		if (!fits_i32(fp.out.m) || !fits_i32(kh.m)) {
			st = kCarriedScaleMantissaOutOfDomain;
		} else {
			const Scale sm = combine(fp.out, kh);
			if (!fits_i32(sm.m)) {
				st = kCarriedScaleMantissaOutOfDomain;
			} else if (iexp_scale_constants(sm.m, sm.e, &sc.c) != 0) {
				st = kIExpScaleDerivationOutOfDomain;
			} else if (!softmax_width_in_domain(sc.c.q_b, sc.c.q_c, (uint64_t)pos + 1, &sc.peak)) {
				st = kSoftmaxRowWidthOutOfDomain;
			} else if (sc.c.q_ln2 < 1) {
				// q_ln2 == 0: every element's construction is refused by the reference
				// (IExpConstruct's q_ln2 >= 1 check) -> SoftmaxKernelRefused.
				// The attention kernel's 32-bit element form also needs q_ln2 <= q_b; that holds
				// for every constant triple iexp_scale_constants returns and needs no test here:
				// q_ln2 = floor(LN2_Q * r / 2^s) and q_b = floor(B_Q * r / 2^s) with the same
				// unsigned reciprocal r and the same shift s, and LN2_Q < B_Q, so the floors are
				// ordered the same way.
				st = kSoftmaxKernelRefused;
			}
		}
		st_kv[h] = st;
		b.smc[(size_t)r * d.kv_heads + h] = sc;
	}

	const int q_threads = blockDim.x > 32 ? (int)blockDim.x - 32 : (int)blockDim.x;   // the other warps
	if ((int)threadIdx.x < q_threads) {
		const Coder cd = make_coder(fp.r, fp.s);
		if (lw.b_q != nullptr) {
#pragma unroll 1
			for (int i = threadIdx.x; i < H; i += q_threads) {
				bool ok;
				sq[i] = code_of(biased(wv(i), lw.b_q, i, &ok), cd);
			}
		} else if (vec) {
			for (int i = threadIdx.x; i < (H >> 2); i += q_threads) {
				const int4 p = ((const int4*)sw)[i];
				const uint32_t c0 = (uint8_t)code_of(p.x, cd);
				const uint32_t c1 = (uint8_t)code_of(p.y, cd);
				const uint32_t c2 = (uint8_t)code_of(p.z, cd);
				const uint32_t c3 = (uint8_t)code_of(p.w, cd);
				((uint32_t*)sq)[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
			}
		} else {
#pragma unroll 1
			for (int i = threadIdx.x; i < H; i += q_threads) sq[i] = code_of(wv(i), cd);
		}
	}
	if ((lw.b_k != nullptr || lw.b_v != nullptr) && !bias_gate) {
		set_status(b, r, kRoundingDivideExponentOutOfDomain, kSiteKv, b.layer);
		return;
	}

	// K/V landing
	long long sat = 0;
	int kv_bad = 0;
#pragma unroll 1
	for (int i = threadIdx.x; i < d.kv_hidden; i += blockDim.x) {
		const int h = i / hd, dd = i - h * hd;
		bool s1, s2;
		int64_t kacc = wv(H + i), vacc = wv(H + d.kv_hidden + i);
		if (lw.b_k != nullptr) {
			bool ok;
			kacc = biased(kacc, lw.b_k, i, &ok);
			if (!ok) kv_bad = 1;
		}
		if (lw.b_v != nullptr) {
			bool ok;
			vacc = biased(vacc, lw.b_v, i, &ok);
			if (!ok) kv_bad = 1;
		}
		// this thread's first element uses the head constants it fetched ahead of the wait
		const bool first = i == (int)threadIdx.x;
		const int64_t k_rt = first ? k_rt0 : lw.k_recip[3 * h + 2], k_et = first ? k_et0 : lw.k_recip[3 * h + 1];
		const int64_t v_rt = first ? v_rt0 : lw.v_recip[3 * h + 2], v_et = first ? v_et0 : lw.v_recip[3 * h + 1];
		const int64_t kraw = landing_rescale(kacc, ns.m, k_rt, ns.e, k_et, &s1, nullptr);
		const int64_t vraw = landing_rescale(vacc, ns.m, v_rt, ns.e, v_et, &s2, nullptr);
		sat += (s1 ? 1 : 0) + (s2 ? 1 : 0);
		sk[i] = (int8_t)clamp127(kraw);
		// V pages are stored transposed ([head_dim][16 positions]) so that the attention
		// kernel can feed them to the tensor cores as the K-major operand of P.V
		int8_t* vdst = pool.base + kv_plane_offset(d, pool, layer_index, h, 1) +
		               ((int64_t)page * hd + dd) * kPageTokens + slot;
		*vdst = (int8_t)clamp127(vraw);
	}
	sat = block_sum_i64(sat, red, d.kv_hidden <= (1 << 20));   // also orders the sq / sk writes before the reads below
	if (lw.b_k != nullptr || lw.b_v != nullptr) {
		// (a bias term outside int64 refuses the row before anything lands, so before anything
		// could count as saturated: LandTokenKVRow, forward_sites.cpp:1281-1418)
		kv_bad = __syncthreads_or(kv_bad);
		if (kv_bad != 0) {
			set_status(b, r, kBiasReconcileProductOutOfDomain, kSiteKv, b.layer);
			return;
		}
	}
	if (threadIdx.x == 0) {
		b.sat[r] += (unsigned long long)sat;
		if (layer_index < b.sat_ld) b.sat_layer[(size_t)r * b.sat_ld + layer_index] = (uint32_t)sat;
	}

	// RoPE: interleaved pairs (2i, 2i+1), table row = position
	int8_t* qrot = b.qrot + (size_t)r * H;
	if (vec && (H & 3) == 0 && (d.kv_hidden & 3) == 0) {
		// two pairs (one word of codes) per thread and pass
		auto rope_word = [&](uint32_t w4, int pi) -> uint32_t {
			const int2 c = *(const int2*)&cos_row[pi], s = *(const int2*)&sin_row[pi];
			int8_t o0, o1, o2, o3;
			rope_pair_clamped((int8_t)w4, (int8_t)(w4 >> 8), c.x, s.x, &o0, &o1);
			rope_pair_clamped((int8_t)(w4 >> 16), (int8_t)(w4 >> 24), c.y, s.y, &o2, &o3);
			return (uint32_t)(uint8_t)o0 | ((uint32_t)(uint8_t)o1 << 8) | ((uint32_t)(uint8_t)o2 << 16) |
			       ((uint32_t)(uint8_t)o3 << 24);
		};
		for (int w = threadIdx.x; w < (H >> 2); w += blockDim.x)
			((uint32_t*)qrot)[w] = rope_word(((const uint32_t*)sq)[w], (2 * w) % half);
		for (int w = threadIdx.x; w < (d.kv_hidden >> 2); w += blockDim.x) {
			const int h = (4 * w) / hd, dd = 4 * w - h * hd;
			int8_t* kdst = pool.base + kv_plane_offset(d, pool, layer_index, h, 0) +
			               ((int64_t)page * kPageTokens + slot) * hd + dd;
			*(uint32_t*)kdst = rope_word(((const uint32_t*)sk)[w], dd / 2);
		}
	} else {
#pragma unroll 1
	for (int p = threadIdx.x; p < H / 2; p += blockDim.x) {
		const int pi = p % half;
		const int32_t c = cos_row[pi], s = sin_row[pi];
		int8_t ox, oy;
		rope_pair_clamped(sq[2 * p], sq[2 * p + 1], c, s, &ox, &oy);
		qrot[2 * p] = ox;
		qrot[2 * p + 1] = oy;
	}
#pragma unroll 1
	for (int p = threadIdx.x; p < d.kv_hidden / 2; p += blockDim.x) {
		const int h = (2 * p) / hd, dd = 2 * p - h * hd, pi = dd / 2;
		const int32_t c = cos_row[pi], s = sin_row[pi];
		int8_t ox, oy;
		rope_pair_clamped(sk[2 * p], sk[2 * p + 1], c, s, &ox, &oy);
		int8_t* kdst = pool.base + kv_plane_offset(d, pool, layer_index, h, 0) +
		               ((int64_t)page * kPageTokens + slot) * hd + dd;
		kdst[0] = ox;
		kdst[1] = oy;
	}
	}

	__syncthreads();
	if (threadIdx.x == 0) {
		if (b.xs != nullptr) { /* q scale is consumed only through smc */ }
		for (int h = 0; h < d.kv_heads; ++h) {
			if (st_kv[h] != kOk) {
				atomicCAS(&b.status[r], 0, pack_status(st_kv[h], kSiteSoftmaxConsts, b.layer));
				break;
			}
		}
	}
}

// Attention-context funnel (forward_sites.cpp:1898-1903): empty incoming, attn_ctx constant.
__global__ void __launch_bounds__(kRowThreads)
k_ctx_funnel(RowBatch b, Dims d, const LayerDev* layer) {
	extern __shared__ __align__(16) unsigned char smem[];
	Red red{(unsigned long long*)smem, 0};
	int32_t* sw = (int32_t*)(smem + kRedBytes);
	const int r = blockIdx.x, n = d.hidden;
	const bool vec = (n & 3) == 0;
	const FunnelFold fold_ctx = funnel_prefold(nullptr, 0, layer->c_ctx);
	pdl_wait();
	pdl_release();
	if (vec) stage16(sw, b.ctxw + (size_t)r * n, n * 4);
	fetch_row_words(b, r, 3, 1, red);
	stage_wait();
	__syncthreads();
	const unsigned long long mx = red.w[kRedMisc];
	if (row_refused(red)) return;
	const FunnelParams fp = funnel_finish(mx, fold_ctx);
	if (fp.status != kOk) {
		set_status(b, r, fp.status, kSiteCtx, b.layer);
		return;
	}
	int8_t* out = b.ctx + (size_t)r * n;
	const Coder cd = make_coder(fp.r, fp.s);
	if (vec) {
		for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
			const int4 p = ((const int4*)sw)[i];
			const uint32_t c0 = (uint8_t)code_of(p.x, cd);
			const uint32_t c1 = (uint8_t)code_of(p.y, cd);
			const uint32_t c2 = (uint8_t)code_of(p.z, cd);
			const uint32_t c3 = (uint8_t)code_of(p.w, cd);
			((uint32_t*)out)[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
		}
	} else {
		const int32_t* w = b.ctxw + (size_t)r * n;
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = code_of(w[i], cd);
	}
	if (threadIdx.x == 0) b.cs[r] = fp.out;
}

// Residual reconciliation (ResidualReconcileSite, forward_sites.cpp:871-989) staged in
// shared memory: wide_i = LandingRescale(branch_i, S[branch], Recip(S[stream].m), ...) + stream_i.
// `fold` = funnel_prefold(&ss, 1, site constant), which the caller derives ahead of its data.
// The branch is given either as codes (branch_s) or, with raw != nullptr, as the staged int32
// projection row together with its coder: the codes are then taken on the fly, which saves the
// separate coding pass and its barrier.
__device__ int32_t block_residual(const int8_t* branch_s, const int32_t* raw, const Coder& raw_coder, Scale bs,
                                  const int8_t* stream, Scale ss, int n, int64_t r_h, const FunnelFold& fold,
                                  int64_t* wide, int8_t* out_g, int8_t* out_s, Scale* out_scale, int64_t* lut,
                                  Red& red, long long* sumsq = nullptr) {
	// r_h = Recip(S[stream].m), also derived by the caller ahead of its data
	if (!fits_i32(ss.m)) return kCarriedScaleMantissaOutOfDomain;
	// the rescaled branch value depends only on the branch code: one LandingRescale per code value.
	// lex marks the codes whose rescaled magnitude left int64 (the site refuses a row that uses one).
	uint8_t* lex = (uint8_t*)(lut + 256);
	for (int t = threadIdx.x; t < 255; t += blockDim.x) {
		bool ex;
		lut[t] = landing_rescale((int64_t)(t - 127), bs.m, r_h, bs.e, ss.e, nullptr, &ex);
		lex[t] = ex ? 1 : 0;
	}
	__syncthreads();
	// one reduction carries both the row maximum and "some code's rescaled magnitude left
	// int64": no in-range sum has magnitude 2^64 - 1, which stands for the latter
	unsigned long long mx = 0;
	if (raw != nullptr) {
		// (the caller guarantees n % 4 == 0, raw 16-byte and stream 4-byte aligned)
		for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
			const int4 p = ((const int4*)raw)[i];
			const uint32_t sw = ((const uint32_t*)stream)[i];
			const int cs4[4] = {code_of(p.x, raw_coder), code_of(p.y, raw_coder), code_of(p.z, raw_coder),
			                    code_of(p.w, raw_coder)};
			int64_t v[4];
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				const int c = cs4[j] + 127;
				const bool ex = lex[c] != 0;
				v[j] = ex ? 0 : lut[c] + (int64_t)(int8_t)(sw >> (8 * j));
				const unsigned long long a = ex ? ~0ull : abs_u64(v[j]);
				mx = a > mx ? a : mx;
			}
			*(longlong2*)&wide[4 * i] = make_longlong2(v[0], v[1]);
			*(longlong2*)&wide[4 * i + 2] = make_longlong2(v[2], v[3]);
		}
	} else if ((n & 3) == 0 && ((((uintptr_t)branch_s) | ((uintptr_t)stream)) & 3) == 0) {
		for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
			const uint32_t bw = ((const uint32_t*)branch_s)[i], sw = ((const uint32_t*)stream)[i];
			int64_t v[4];
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				const int c = (int)(int8_t)(bw >> (8 * j)) + 127;
				const bool ex = lex[c] != 0;
				v[j] = ex ? 0 : lut[c] + (int64_t)(int8_t)(sw >> (8 * j));
				const unsigned long long a = ex ? ~0ull : abs_u64(v[j]);
				mx = a > mx ? a : mx;
			}
			*(longlong2*)&wide[4 * i] = make_longlong2(v[0], v[1]);
			*(longlong2*)&wide[4 * i + 2] = make_longlong2(v[2], v[3]);
		}
	} else {
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) {
			const int c = (int)branch_s[i] + 127;
			if (lex[c]) {
				mx = ~0ull;
				wide[i] = 0;
			} else {
				const int64_t v = lut[c] + (int64_t)stream[i];
				wide[i] = v;
				const unsigned long long a = abs_u64(v);
				mx = a > mx ? a : mx;
			}
		}
	}
	mx = block_max_u64(mx, red);   // its barrier also publishes wide[]
	if (mx == ~0ull) return kResidualMagnitudeOutOfDomain;
	return block_code(wide, n, mx, fold, out_g, out_s, out_scale, sumsq);
}

// o-projection funnel -> attention residual -> MLP RMSNorm (forward_sites.cpp:1906-1937)
__global__ void __launch_bounds__(kRowThreads, 1024 / kRowThreads)
k_res1(RowBatch b, Dims d, const LayerDev* layer) {
	extern __shared__ __align__(16) unsigned char smem[];
	Red red{(unsigned long long*)smem, 0};
	int64_t* lut = (int64_t*)(smem + kRedBytes);
	int64_t* wide = (int64_t*)(smem + kRedBytes + kLutBytes);
	int8_t* so = (int8_t*)(wide + d.hidden);
	int8_t* sa = so + d.hidden;
	int8_t* sx = sa + d.hidden;                  // staged stream row
	int8_t* sg = sx + d.hidden;                  // staged gain
	int32_t* wraw = (int32_t*)(sg + d.hidden);   // staged projection row
	const int r = blockIdx.x, n = d.hidden;
	const LayerDev& lw = *layer;
	const bool vec = wide_stageable(b, n) && (n & 15) == 0;
	// ahead of the o-projection: the stream row and its scale, the context scale (written by the
	// context funnel, which ran before that projection), the gain and the site constants
	if (vec) {
		stage16(sx, b.x + (size_t)r * n, n);
		stage16(sg, lw.g_mlp, n);
	}
	const Scale cs = b.cs[r], xs = b.xs[r];
	const Scale c_o = lw.c_o, c_res = lw.c_attn_res, c_norm = lw.c_mlp_norm;
	// ... and every scalar that needs only those: the scale folds of both funnels and the
	// stream scale's reciprocal
	const FunnelFold fold_o = funnel_prefold(&cs, 1, c_o);
	const FunnelFold fold_res = funnel_prefold(&xs, 1, c_res);
	const int64_t r_h = dyn_recip(xs.m);
	pdl_wait();
	pdl_release();
	if (vec) stage16(wraw, wide_row32(b, r), n * 4);
	fetch_row_words(b, r, 0, 1, red);
	stage_wait();
	__syncthreads();
	const unsigned long long mx = red.w[kRedMisc];
	if (row_refused(red)) return;
	const FunnelParams fp = funnel_finish(mx, fold_o);
	int32_t st = fp.status;
	int site = kSiteO;
	long long ssq = 0;
	if (st == kOk) {
		const Coder cd = make_coder(fp.r, fp.s);
		if (!vec) {
#pragma unroll 1
			for (int i = threadIdx.x; i < n; i += blockDim.x) so[i] = code_of(load_wide(b, r, i), cd);
			__syncthreads();
		}
		site = kSiteAttnRes;
		st = block_residual(so, vec ? wraw : nullptr, cd, fp.out, vec ? sx : b.x + (size_t)r * n, xs, n, r_h,
		                    fold_res, wide, b.a + (size_t)r * n, sa, &b.as[r], lut, red, &ssq);
	}
	if (st == kOk) {
		// (the norm's first barrier, in its sum, also separates the passes above from its own)
		site = kSiteMlpNorm;
		st = block_rmsnorm(sa, vec ? sg : lw.g_mlp, n, c_norm, wide, b.nrm + (size_t)r * n, &b.ns[r], lut, red, &ssq);
	}
	set_status(b, r, st, site, b.layer);
}

// down-projection funnel -> MLP residual -> (next layer's attention RMSNorm)
// (forward_sites.cpp:1968-1987, :1694-1698)
__global__ void __launch_bounds__(kRowThreads, 1024 / kRowThreads)
k_res2(RowBatch b, Dims d, const LayerDev* layer, const LayerDev* next_layer) {
	extern __shared__ __align__(16) unsigned char smem[];
	Red red{(unsigned long long*)smem, 0};
	int64_t* lut = (int64_t*)(smem + kRedBytes);
	int64_t* wide = (int64_t*)(smem + kRedBytes + kLutBytes);
	int8_t* sd = (int8_t*)(wide + d.hidden);
	int8_t* sx = sd + d.hidden;
	int8_t* sa = sx + d.hidden;                  // staged stream row (after the attention residual)
	int8_t* sg = sa + d.hidden;                  // staged gain of the next layer
	int32_t* wraw = (int32_t*)(sg + d.hidden);   // staged projection row
	const int r = blockIdx.x, n = d.hidden;
	const LayerDev& lw = *layer;
	const bool vec = wide_stageable(b, n) && (n & 15) == 0;
	// ahead of the down-projection: the stream row after the attention residual and its scale,
	// the activation scale (written before that projection ran), the next gain, the constants
	if (vec) {
		stage16(sa, b.a + (size_t)r * n, n);
		if (next_layer != nullptr) stage16(sg, next_layer->g_attn, n);
	}
	const Scale as = b.acts[r], rs = b.as[r];
	const Scale c_down = lw.c_down, c_res = lw.c_mlp_res;
	Scale c_norm = Scale{0, 0};
	if (next_layer != nullptr) c_norm = next_layer->c_attn_norm;
	const FunnelFold fold_down = funnel_prefold(&as, 1, c_down);
	const FunnelFold fold_res = funnel_prefold(&rs, 1, c_res);
	const int64_t r_h = dyn_recip(rs.m);
	pdl_wait();
	pdl_release();
	if (vec) stage16(wraw, wide_row32(b, r), n * 4);
	fetch_row_words(b, r, 0, 1, red);
	stage_wait();
	__syncthreads();
	const unsigned long long mx = red.w[kRedMisc];
	if (row_refused(red)) return;
	const FunnelParams fp = funnel_finish(mx, fold_down);
	int32_t st = fp.status;
	int site = kSiteDown, site_layer = b.layer;
	long long ssq = 0;
	if (st == kOk) {
		const Coder cd = make_coder(fp.r, fp.s);
		if (!vec) {
#pragma unroll 1
			for (int i = threadIdx.x; i < n; i += blockDim.x) sd[i] = code_of(load_wide(b, r, i), cd);
			__syncthreads();
		}
		site = kSiteMlpRes;
		st = block_residual(sd, vec ? wraw : nullptr, cd, fp.out, vec ? sa : b.a + (size_t)r * n, rs, n, r_h,
		                    fold_res, wide, b.x + (size_t)r * n, sx, &b.xs[r], lut, red, &ssq);
	}
	if (st == kOk) {
		// the layer is complete for this row: x / xs hold its stream, whatever the next layer does
		if (threadIdx.x == 0) b.done[r] += 1;
		if (next_layer != nullptr) {
			site = kSiteAttnNorm;
			site_layer = b.layer + 1;
			st = block_rmsnorm(sx, vec ? sg : next_layer->g_attn, n, c_norm, wide,
			                   b.nrm + (size_t)r * n, &b.ns[r], lut, red, &ssq);
		}
	}
	set_status(b, r, st, site, site_layer);
}

// The activation row is the longest a row kernel walks (intermediate width, three codes per
// element), and its passes are bound by instruction issue: the row's coders are checked once
// and the passes below are compiled for the 32-bit coder and for the general one.
template <bool NARROW>
__device__ __forceinline__ int code_sel(int32_t x, const Coder& c) {
	if (NARROW) return code_narrow(x < 0 ? 0u - (uint32_t)x : (uint32_t)x, x < 0, c);
	return (int)requant_code_general((int64_t)x, c.r, c.s);
}
// wide[] holds the gate row on entry and g * sigmoid(g) * u on exit; returns this thread's
// largest product magnitude
template <bool NARROW>
__device__ __forceinline__ uint32_t act_products(int32_t* wide, const int32_t* urow, const int32_t* gsil, int n4,
                                                 const Coder& cg, const Coder& cu) {
	uint32_t lmax = 0;
#pragma unroll 2
	for (int i = threadIdx.x; i < n4; i += blockDim.x) {
		const int4 gv = ((const int4*)wide)[i], uv = ((const int4*)urow)[i];
		const int gs[4] = {gv.x, gv.y, gv.z, gv.w}, us[4] = {uv.x, uv.y, uv.z, uv.w};
		int pr[4];
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const int g = code_sel<NARROW>(gs[j], cg);
			const int u = code_sel<NARROW>(us[j], cu);
			pr[j] = gsil[g + 127] * u;
			const uint32_t a = pr[j] < 0 ? 0u - (uint32_t)pr[j] : (uint32_t)pr[j];
			lmax = a > lmax ? a : lmax;
		}
		((int4*)wide)[i] = make_int4(pr[0], pr[1], pr[2], pr[3]);
	}
	return lmax;
}
template <bool NARROW>
__device__ __forceinline__ void code_row4(const int32_t* wide, int n4, const Coder& c, int8_t* out) {
#pragma unroll 2
	for (int i = threadIdx.x; i < n4; i += blockDim.x) {
		const int4 p = ((const int4*)wide)[i];
		const uint32_t c0 = (uint8_t)code_sel<NARROW>(p.x, c);
		const uint32_t c1 = (uint8_t)code_sel<NARROW>(p.y, c);
		const uint32_t c2 = (uint8_t)code_sel<NARROW>(p.z, c);
		const uint32_t c3 = (uint8_t)code_sel<NARROW>(p.w, c);
		((uint32_t*)out)[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
	}
}

// gate / up funnels -> SwiGLU activation site (MlpActSite, forward_sites.cpp:796-864)
__global__ void __launch_bounds__(kRowThreads, 1024 / kRowThreads)
k_act(RowBatch b, Dims d, const LayerDev* layer, const int32_t* silu_table) {
	extern __shared__ __align__(16) unsigned char smem[];
	Red red{(unsigned long long*)smem, 0};
	int32_t* gsil = (int32_t*)(smem + kRedBytes);      // g * sigmoid(g) for the 255 gate codes, this row's scale
	int32_t* wide = gsil + 256;                         // inter: the gate row, then the products in place
	int32_t* urow = wide + d.inter;                     // inter: the up row
	const int r = blockIdx.x, n = d.inter;
	const bool vec = !b.wide64 && (n & 3) == 0 && (b.wide_ld & 3) == 0;
	// ahead of the gate/up projection: the normed row's scale (written by the residual site
	// before that projection ran) and the site constants
	const LayerDev& lw = *layer;
	const Scale ns = b.ns[r];
	const Scale c_gate = lw.c_gate, c_up = lw.c_up, c_act = lw.c_act;
	const FunnelFold fold_g = funnel_prefold(&ns, 1, c_gate), fold_u = funnel_prefold(&ns, 1, c_up);
	pdl_wait();
	pdl_release();
	if (vec) {
		// the whole gate | up row lands in shared memory while the scalar derivations below run
		const int32_t* gp = (const int32_t*)b.wide + (size_t)r * b.wide_ld;
		stage16(wide, gp, n * 4);
		stage16(urow, gp + n, n * 4);
	}
	fetch_row_words(b, r, 1, 2, red);
	__syncthreads();
	const unsigned long long mxg = red.w[kRedMisc], mxu = red.w[kRedMisc + 1];
	if (row_refused(red)) {
		stage_wait();
		return;
	}
	const FunnelParams fg = funnel_finish(mxg, fold_g);
	const FunnelParams fu = funnel_finish(mxu, fold_u);
	int32_t st = fg.status != kOk ? fg.status : fu.status;
	int site = fg.status != kOk ? kSiteGate : kSiteUp;
	if (st == kOk && !silu_scale_in_domain(fg.out)) {
		st = kSiluScaleOutOfDomain;
		site = kSiteSilu;
	}
	if (st != kOk) {
		stage_wait();
		set_status(b, r, st, site, b.layer);
		return;
	}
	const int ge = (int)fg.out.e;
	// the sigmoid depends only on the gate code and the row's gate scale: 255 evaluations per
	// row instead of one per element
	for (int t = threadIdx.x; t < 255; t += blockDim.x) {
		const int g = t - 127;
		gsil[t] = g * silu_sigmoid_q15(silu_table, g, fg.out.m, ge);
	}
	stage_wait();
	__syncthreads();
	// products g * sigmoid(g) * u, |.| <= 127 * 2^15 * 127 < 2^29, left in shared memory
	// with their running maximum so that the funnel below needs no second pass for it
	const Scale inc[2] = {fg.out, fu.out};
	const FunnelFold fold_act = funnel_prefold(inc, 2, c_act);   // ahead of the maximum it will meet
	uint32_t lmax = 0;
	if (vec) {
		const Coder cg = make_coder(fg.r, fg.s), cu = make_coder(fu.r, fu.s);
		lmax = (cg.narrow && cu.narrow) ? act_products<true>(wide, urow, gsil, n >> 2, cg, cu)
		                                : act_products<false>(wide, urow, gsil, n >> 2, cg, cu);
	} else {
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) {
			const int g = requant_code(load_wide(b, r, i), fg.r, fg.s);
			const int u = requant_code(load_wide(b, r, n + i), fu.r, fu.s);
			const int p = gsil[g + 127] * u;
			wide[i] = p;
			const uint32_t a = p < 0 ? 0u - (uint32_t)p : (uint32_t)p;
			lmax = a > lmax ? a : lmax;
		}
	}
	const unsigned long long mx = block_max_u64((unsigned long long)lmax, red);
	const FunnelParams fp = funnel_finish(mx, fold_act);
	if (fp.status != kOk) {
		set_status(b, r, fp.status, kSiteAct, b.layer);
		return;
	}
	int8_t* out = b.act + (size_t)r * n;
	if ((n & 3) == 0) {
		const Coder ca = make_coder(fp.r, fp.s);
		if (ca.narrow) code_row4<true>(wide, n >> 2, ca, out);
		else code_row4<false>(wide, n >> 2, ca, out);
	} else {
#pragma unroll 1
		for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = requant_code((int64_t)wide[i], fp.r, fp.s);
	}
	if (threadIdx.x == 0) b.acts[r] = fp.out;
}

// End of a call: hand each row's stream back to its sequence (or nowhere).
__global__ void __launch_bounds__(kRowThreads)
k_scatter(RowBatch b, Dims d, const RowSink* sink) {
	pdl_wait();
	pdl_release();
	const int r = blockIdx.x, n = d.hidden;
	const RowSink s = sink[r];
	if (s.hidden == nullptr || b.status[r] != 0) return;
	const int8_t* x = b.x + (size_t)r * n;
#pragma unroll 1
	for (int i = threadIdx.x; i < n; i += blockDim.x) s.hidden[i] = x[i];
	if (threadIdx.x == 0) *s.scale = b.xs[r];
}

// ------------------------------------------------------------------ launchers
// Threads per row block. A row kernel derives its scalar chains (scale folds, reciprocals, roots) in
// every thread, so that no phase waits for a broadcast: right for a decode batch, whose time is the
// length of that chain. A prefill chunk has hundreds of rows and is bound by instruction issue
// instead, where fewer threads per row mean fewer redundant copies of those chains (the residual
// sites of a 1024-row chunk take 0.85 ms instead of 1.03 ms per pass over the 1.5B shape's layers).
static int row_threads(int rows) {
	static const int big = [] {
		const char* e = getenv("SSLM_B200_ROW_THREADS_BIG");      // tuning: 64, 128 or 256
		const int v = e ? atoi(e) : 128;
		return (v == 64 || v == 128 || v == 256) ? v : 128;
	}();
	static const int min_rows = [] {
		const char* e = getenv("SSLM_B200_ROW_THREADS_MIN_ROWS");      // tuning: batch size from which `big` applies
		return e ? atoi(e) : 512;
	}();
	return rows >= min_rows ? big : kRowThreads;
}
static size_t smem_wide(const Dims& d) { return kRedBytes + kLutBytes + (size_t)d.hidden * 8; }
// reductions, the int64 staging row, four code rows and the staged int32 projection row
static size_t res_smem_bytes(const Dims& d) { return kRedBytes + kLutBytes + (size_t)d.hidden * 16; }

void launch_begin(const RowBatch& b, const Dims& d, const int8_t* embed, Scale c_embed,
                  const RowSource* src, const LayerDev* layer, cudaStream_t st) {
	launch_pdl(k_begin, dim3(b.m), dim3(kRowThreads), smem_wide(d), st, b, d, embed, c_embed, src, layer);
}
void launch_rmsnorm(const RowBatch& b, const Dims& d, const int8_t* gain, Scale site, cudaStream_t st) {
	launch_pdl(k_rmsnorm, dim3(b.m), dim3(kRowThreads), smem_wide(d), st, b, d, gain, site);
}
void launch_qkv_post(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index,
                     KvPoolDev pool, const int32_t* cos, const int32_t* sin, cudaStream_t st) {
	const size_t sm = kRedBytes + 64 + (size_t)((d.hidden + d.kv_hidden + 15) & ~15) +
	                  (size_t)(d.qkv_rows + d.head_dim) * 4;
	launch_pdl(k_qkv_post, dim3(b.m), dim3(row_threads(b.m)), sm, st, b, d, layer, layer_index, pool, cos, sin);
}
void launch_ctx_funnel(const RowBatch& b, const Dims& d, const LayerDev* layer, cudaStream_t st) {
	launch_pdl(k_ctx_funnel, dim3(b.m), dim3(row_threads(b.m)), kRedBytes + (size_t)d.hidden * 4, st, b, d, layer);
}
void launch_res1(const RowBatch& b, const Dims& d, const LayerDev* layer, cudaStream_t st) {
	launch_pdl(k_res1, dim3(b.m), dim3(row_threads(b.m)), res_smem_bytes(d), st, b, d, layer);
}
void launch_res2(const RowBatch& b, const Dims& d, const LayerDev* layer, const LayerDev* next,
                 cudaStream_t st) {
	launch_pdl(k_res2, dim3(b.m), dim3(row_threads(b.m)), res_smem_bytes(d), st, b, d, layer, next);
}
size_t act_smem_bytes(const Dims& d) { return kRedBytes + 256 * 4 + (size_t)d.inter * 8; }
cudaError_t rows_configure(const Dims& d) {
	cudaError_t e = cudaFuncSetAttribute(k_act, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)act_smem_bytes(d));
	if (e != cudaSuccess) return e;
	// Every kernel of a step asks for the same (largest) shared-memory carve-out as the
	// tensor-core GEMM between them, so consecutive launches never make the SMs re-split
	// their L1 / shared memory.
	const void* all[] = {(const void*)k_begin, (const void*)k_rmsnorm, (const void*)k_qkv_post, (const void*)k_ctx_funnel,
	                     (const void*)k_res1,  (const void*)k_res2,    (const void*)k_act,      (const void*)k_scatter};
	for (const void* f : all) {
		e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
		if (e != cudaSuccess) return e;
	}
	const int res = (int)res_smem_bytes(d);
	if (res > 227 * 1024) return cudaErrorInvalidConfiguration;
	e = cudaFuncSetAttribute(k_res1, cudaFuncAttributeMaxDynamicSharedMemorySize, res);
	if (e != cudaSuccess) return e;
	return cudaFuncSetAttribute(k_res2, cudaFuncAttributeMaxDynamicSharedMemorySize, res);
}
void launch_act(const RowBatch& b, const Dims& d, const LayerDev* layer, const int32_t* silu,
                cudaStream_t st) {
	launch_pdl(k_act, dim3(b.m), dim3(kRowThreads), act_smem_bytes(d), st, b, d, layer, silu);
}
void launch_scatter(const RowBatch& b, const Dims& d, const RowSink* sink, cudaStream_t st) {
	launch_pdl(k_scatter, dim3(b.m), dim3(kRowThreads), 0, st, b, d, sink);
}

}  // namespace sslm
