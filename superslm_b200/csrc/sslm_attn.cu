// Integer i-exp softmax attention over the paged int8 KV pool, staged through shared
// memory, with both contractions on the tensor cores (mma.sync m16n8k32, exact int32
// accumulation). One block of head_dim/16 warps owns one (row, kv head) and serves every q head
// of the GQA group from one pass over the K and V pages, so each K / V byte of the
// sequence leaves HBM once per kv head.
//
//   stage 1  scores[g][k] = q_rot[g] . K[k]      A = the group's q rows (heads in the M
//            dimension), B = 8 K rows per MMA straight from the page (16-byte loads; the
//            head-dim order inside an MMA is permuted identically on both operands)
//   stage 2  e_k = second-order integer exp of (score - max); total; p_k = (e_k << 15) /
//            total (SoftmaxRowQ15); p_k is split into two u8 planes, p = 256 ph + pl
//   stage 3  ctx[g][d] = sum_k p_k V[k][d]       A = pl / ph (u8), B = transposed V page
//            words (4 positions of one channel per register), two MMAs per plane, then
//            ctx = acc_l + 256 acc_h, the per-head fold and the row max for the funnel
//
// Every reduction is an integer max or add, so the result does not depend on the order in
// which lanes, warps or blocks contribute. Restates the attention block of RunLayerLoopImpl
// (src/forward/forward_sites.cpp:1858-1897), SoftmaxRowQ15 (src/intmath.cpp:796-901) and
// GemmProbQ15Accumulate (src/matmul.cpp:522-538).
#include <cuda_runtime.h>

#include "sslm_kernels.h"

namespace sslm {

// threads per block = 2 * head_dim: one warp per pair of 8-channel blocks of P.V
constexpr int kAttnMaxWarps = 8;

// One softmax element for constants that passed the gates of k_qkv_post (1 <= q_ln2 <= q_b
// < 2^24, q_c >= 0): the value iexp_element() computes, on 32-bit words. dq = max - score
// (0 <= dq < 2^32). z = floor(x / q_ln2) comes from a float estimate repaired with the
// exact remainder.
struct IExpFast {
	uint32_t ln2, clip;     // q_ln2, 30 * q_ln2
	int32_t qb;
	int64_t qc, peak;
	float inv_ln2;
};
__device__ __forceinline__ IExpFast iexp_fast_prepare(const SoftmaxConsts& k) {
	IExpFast f;
	f.ln2 = (uint32_t)k.c.q_ln2;
	f.clip = 30u * f.ln2;
	f.qb = (int32_t)k.c.q_b;
	f.qc = k.c.q_c;
	f.peak = k.peak;
	f.inv_ln2 = 1.0f / (float)f.ln2;
	return f;
}
// *parts = (z << 24) | rem with x = z * q_ln2 + rem (rem < q_ln2 < 2^24, z <= 30): the second
// softmax pass rebuilds the element from it (iexp_from_parts) instead of dividing again.
__device__ __forceinline__ bool iexp_fast(uint32_t dq, const IExpFast& f, int64_t* value, uint32_t* parts) {
	const uint32_t x = dq < f.clip ? dq : f.clip;
	int32_t z = (int32_t)((float)x * f.inv_ln2);
	int32_t rem = (int32_t)(x - (uint32_t)z * f.ln2);
	if (rem < 0) { --z; rem += (int32_t)f.ln2; }
	if (rem >= (int32_t)f.ln2) { ++z; rem -= (int32_t)f.ln2; }
	const int32_t base = f.qb - rem;
	const int64_t v = ((int64_t)base * (int64_t)base + f.qc) >> z;
	*value = v;
	*parts = ((uint32_t)z << 24) | (uint32_t)rem;
	return f.peak >= 1 && v >= 0 && v <= f.peak;
}
__device__ __forceinline__ int64_t iexp_from_parts(uint32_t parts, const IExpFast& f) {
	const int32_t base = f.qb - (int32_t)(parts & 0xFFFFFFu);
	return ((int64_t)base * (int64_t)base + f.qc) >> (parts >> 24);
}
// floor((e << 15) / tot) for 0 <= e <= tot, tot >= 1: float estimate (within 1), exact repair
__device__ __forceinline__ uint32_t prob_q15(int64_t e, unsigned long long tot, float rinv) {
	const unsigned long long num = (unsigned long long)e << 15;
	unsigned long long p = (unsigned long long)((float)e * rinv);
	if (p > 32768ull) p = 32768ull;
	while (p * tot > num) --p;
	while (num - p * tot >= tot) ++p;
	return (uint32_t)p;
}

// D += A(16x32, row) * B(32x8, col); rows 8..15 of A are always zero here (a1 = a3 = 0)
__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
	asm volatile(
	    "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
	    : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
	    : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
	asm volatile(
	    "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
	    : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
	    : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// The HD/16 words of a head-dim row that lane column c (= lane & 3) feeds to the HD/32
// score MMAs: MMA j takes words 2j (k slots 4c..4c+3) and 2j+1 (k slots 16+4c..). Any
// assignment of head-dim bytes to k slots is valid as long as q and K use the same one.
// (Plain loads, not the read-only path: q and the newest K / V rows were written by the kernel
// just before this one, which may still have been running when this block was placed.)
template <int HD>
__device__ __forceinline__ void load_row_words(const int8_t* row, int c, uint32_t (&w)[HD / 16]) {
	if constexpr (HD == 32) {
		const int2 x = *(const int2*)(row + c * 8);
		w[0] = (uint32_t)x.x; w[1] = (uint32_t)x.y;
	} else if constexpr (HD == 128) {
		// one 32-byte load per lane: the four lanes of a position cover its 128-byte row, and a
		// warp's load covers eight whole lines (rows are 128-byte aligned in the pages and in q)
		asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
		             : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
		             : "l"(row + c * 32)
		             : "memory");
	} else {
		const int4 x = *(const int4*)(row + c * 16);
		w[0] = (uint32_t)x.x; w[1] = (uint32_t)x.y; w[2] = (uint32_t)x.z; w[3] = (uint32_t)x.w;
		if constexpr (HD == 128) {
			const int4 y = *(const int4*)(row + 64 + c * 16);
			w[4] = (uint32_t)y.x; w[5] = (uint32_t)y.y; w[6] = (uint32_t)y.z; w[7] = (uint32_t)y.w;
		}
	}
}

struct AttnSmem {
	int64_t* pbase;       // [wp/16] byte offset of each page inside a plane
	int32_t* sc;          // [G][wp] scores
	uint8_t* pl;          // [G][wp] low byte of the Q15 probability
	uint8_t* ph;          // [G][wp] high byte
	unsigned long long* red;   // [8 heads][warps] partials
	int* flag;            // [4] single values handed to the whole block
};
__host__ __device__ inline size_t attn_smem_bytes(int group, int wp) {
	return (size_t)wp / 16 * 8 + (size_t)group * wp * 6 + 8 * kAttnMaxWarps * 8 + 16;
}
__device__ __forceinline__ AttnSmem carve(unsigned char* smem, int group, int wp) {
	AttnSmem s;
	s.pbase = (int64_t*)smem;
	s.sc = (int32_t*)(smem + (size_t)wp / 16 * 8);
	s.pl = (uint8_t*)(s.sc + (size_t)group * wp);
	s.ph = s.pl + (size_t)group * wp;
	s.red = (unsigned long long*)(s.ph + (size_t)group * wp);
	s.flag = (int*)(s.red + 8 * kAttnMaxWarps);
	return s;
}
// ask for the line at p to be brought into L2; nothing waits for it
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// HD = head_dim (32, 64 or 128); wp = padded width, a multiple of 64
template <int HD>
__global__ void __launch_bounds__(2 * HD, HD == 128 ? 4 : 8)
k_attention(RowBatch b, Dims d, const LayerDev* layer, int layer_index, KvPoolDev pool, int wp, int reverse_rows) {
	extern __shared__ __align__(16) unsigned char smem[];
	// blocks start in index order: with reverse_rows the last (widest) rows of a prefill chunk go first
	const int r = reverse_rows ? (int)gridDim.y - 1 - (int)blockIdx.y : (int)blockIdx.y, kvh = blockIdx.x;
	constexpr int kAttnThreads = 2 * HD, kAttnWarps = kAttnThreads / 32;
	const int G = d.heads / d.kv_heads;
	const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
	const int g = lane >> 2, c = lane & 3;
	const AttnSmem s = carve(smem, G, wp);
	// Ahead of the kernel that lands this step's K / V rows (it may still be running): the row
	// descriptor and the page table were uploaded before the step's first launch, and every K / V
	// row but the newest was written by earlier steps. So the page offsets are staged now, and
	// the old K rows are asked into L2 while that kernel, which moves little data, finishes.
	const int width = b.rows[r].pos + 1;
	const int w64 = (width + 63) & ~63;
	const int8_t* kplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 0);
	const int8_t* vplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 1);
	const int npages = (width + kPageTokens - 1) / kPageTokens;
	{
		const int32_t* pages = b.rows[r].pages;
		for (int j = t; j < npages; j += kAttnThreads) s.pbase[j] = (int64_t)pages[j] * (kPageTokens * HD);
	}
	int32_t fi = 1, fm = 0, fs = 0;                // this lane's head: the context fold (weights)
	if (g < G) {
		const int32_t* f = layer->f_ctx + 3 * (kvh * G + g);
		fi = f[0]; fm = f[1]; fs = f[2];
	}
	__syncthreads();
	constexpr int kRowsPerLine = 128 / HD;
	for (int pos = t * kRowsPerLine; pos < width - 1; pos += kAttnThreads * kRowsPerLine)
		prefetch_l2(kplane + s.pbase[pos >> 4] + (pos & 15) * HD);
	pdl_wait();
	pdl_release();
	// one thread reads the row's status for everybody: the block of the row's other kv head may
	// refuse the row at any moment, and the threads here must agree on leaving
	if (t == 0) *s.flag = __ldcg(&b.status[r]);
	const SoftmaxConsts smc = b.smc[(size_t)r * d.kv_heads + kvh];   // wanted after the scores; asked for now
	__syncthreads();
	if (*s.flag != 0) return;

	// ---- stage 1: scores, 8 positions per MMA group, groups dealt round-robin to the warps
	{
		constexpr int NW = HD / 16;
		uint32_t qw[NW];
#pragma unroll
		for (int j = 0; j < NW; ++j) qw[j] = 0;
		if (g < G) load_row_words<HD>(b.qrot + (size_t)r * d.hidden + (size_t)(kvh * G + g) * HD, c, qw);
		const int nblk = (width + 7) >> 3;
		constexpr int U = 4;
		for (int blk0 = warp * U; blk0 < nblk; blk0 += kAttnWarps * U) {
			uint32_t kw[U][NW];
#pragma unroll
			for (int u = 0; u < U; ++u) {
				const int pos = (blk0 + u) * 8 + g;
#pragma unroll
				for (int j = 0; j < NW; ++j) kw[u][j] = 0;
				if (pos < width)
					load_row_words<HD>(kplane + s.pbase[pos >> 4] + (pos & 15) * HD, c, kw[u]);
			}
#pragma unroll
			for (int u = 0; u < U; ++u) {
				int acc[4] = {0, 0, 0, 0};
#pragma unroll
				for (int j = 0; j < NW / 2; ++j) mma_s8s8(acc, qw[2 * j], qw[2 * j + 1], kw[u][2 * j], kw[u][2 * j + 1]);
				const int k = (blk0 + u) * 8 + c * 2;
				if (g < G && blk0 + u < nblk) *(int2*)&s.sc[(size_t)g * wp + k] = make_int2(acc[0], acc[1]);
			}
		}
	}
	__syncthreads();

	// the softmax below moves no data: ask for this row's V pages (16 lines each) meanwhile
	for (int ln = t; ln < npages * (kPageTokens * HD / 128); ln += kAttnThreads)
		prefetch_l2(vplane + s.pbase[ln / (kPageTokens * HD / 128)] + (ln % (kPageTokens * HD / 128)) * 128);

	// ---- stage 2: softmax. Each thread takes 4 consecutive positions of every head.
	const IExpFast fx = iexp_fast_prepare(smc);
	int mx[8];
#pragma unroll
	for (int h = 0; h < 8; ++h) mx[h] = INT32_MIN;
	for (int k4 = t * 4; k4 < width; k4 += kAttnThreads * 4) {
#pragma unroll
		for (int h = 0; h < 8; ++h) {
			if (h < G) {
				const int4 v = *(const int4*)&s.sc[(size_t)h * wp + k4];
				int m = v.x;
				if (k4 + 1 < width) m = max(m, v.y);
				if (k4 + 2 < width) m = max(m, v.z);
				if (k4 + 3 < width) m = max(m, v.w);
				mx[h] = max(mx[h], m);
			}
		}
	}
	int* redi = (int*)s.red;
#pragma unroll
	for (int h = 0; h < 8; ++h) {
		if (h < G) {
			mx[h] = __reduce_max_sync(0xffffffffu, mx[h]);
			if (lane == 0) redi[h * kAttnWarps + warp] = mx[h];
		}
	}
	__syncthreads();
#pragma unroll
	for (int h = 0; h < 8; ++h) {
		int m = redi[h * kAttnWarps];
#pragma unroll
		for (int w = 1; w < kAttnWarps; ++w) m = max(m, redi[h * kAttnWarps + w]);
		mx[h] = m;
	}
	__syncthreads();

	unsigned long long tot[8];
#pragma unroll
	for (int h = 0; h < 8; ++h) tot[h] = 0;
	bool bad = false;
	for (int k4 = t * 4; k4 < width; k4 += kAttnThreads * 4) {
#pragma unroll
		for (int h = 0; h < 8; ++h) {
			if (h < G) {
				const int4 v = *(const int4*)&s.sc[(size_t)h * wp + k4];
				const int sv[4] = {v.x, v.y, v.z, v.w};
				uint32_t parts[4];
#pragma unroll
				for (int j = 0; j < 4; ++j) {
					int64_t e;
					const bool ok = iexp_fast((uint32_t)mx[h] - (uint32_t)sv[j], fx, &e, &parts[j]);
					if (k4 + j < width) {
						tot[h] += ok ? (unsigned long long)e : 0ull;
						bad |= !ok;
					}
				}
				// the score has done its work: its place now holds the element's (shift, remainder),
				// which this same thread reads back in the probability pass
				*(int4*)&s.sc[(size_t)h * wp + k4] = make_int4((int)parts[0], (int)parts[1], (int)parts[2], (int)parts[3]);
			}
		}
	}
#pragma unroll
	for (int h = 0; h < 8; ++h) {
		if (h < G) {
			// a thread's partial is below 2^62; three 24-bit limbs (the top one 16 bits) add up
			// across the warp without leaving 32 bits, one warp-reduce instruction each
			const uint32_t l0 = __reduce_add_sync(0xffffffffu, (uint32_t)tot[h] & 0xFFFFFFu);
			const uint32_t l1 = __reduce_add_sync(0xffffffffu, (uint32_t)(tot[h] >> 24) & 0xFFFFFFu);
			const uint32_t l2 = __reduce_add_sync(0xffffffffu, (uint32_t)(tot[h] >> 48));
			if (lane == 0)
				s.red[h * kAttnWarps + warp] = (unsigned long long)l0 + ((unsigned long long)l1 << 24) + ((unsigned long long)l2 << 48);
		}
	}
	if (__syncthreads_or(bad ? 1 : 0)) {
		// the reference refuses the row (SoftmaxKernelRefusedAfterGateAccepted)
		if (t == 0) atomicCAS(&b.status[r], 0, pack_status(kSoftmaxKernelRefused, kSiteSoftmax, b.layer));
		return;
	}
	float inv[8];
#pragma unroll
	for (int h = 0; h < 8; ++h) {
		unsigned long long x = 0;
#pragma unroll
		for (int w = 0; w < kAttnWarps; ++w) x += s.red[h * kAttnWarps + w];
		tot[h] = x > 1ull ? x : 1ull;
		inv[h] = 32768.0f / (float)tot[h];
	}
	// probabilities, zero beyond the width up to the next multiple of 64 (stage 3 reads whole pages)
	for (int k4 = t * 4; k4 < w64; k4 += kAttnThreads * 4) {
#pragma unroll
		for (int h = 0; h < 8; ++h) {
			if (h < G) {
				const int4 v = *(const int4*)&s.sc[(size_t)h * wp + k4];
				const int sv[4] = {v.x, v.y, v.z, v.w};
				uint32_t lo = 0, hi = 0;
#pragma unroll
				for (int j = 0; j < 4; ++j) {
					if (k4 + j < width) {
						const int64_t e = iexp_from_parts((uint32_t)sv[j], fx);
						const uint32_t p = prob_q15(e, tot[h], inv[h]);
						lo |= (p & 0xffu) << (8 * j);
						hi |= (p >> 8) << (8 * j);
					}
				}
				*(uint32_t*)&s.pl[(size_t)h * wp + k4] = lo;
				*(uint32_t*)&s.ph[(size_t)h * wp + k4] = hi;
			}
		}
	}
	__syncthreads();

	// ---- stage 3: ctx = P V. Lane column c owns page 4*grp + c of each 64-position group;
	// its 16-byte row of the transposed page feeds two MMAs (positions 0..7 and 8..15).
	constexpr int NDB = 2;            // 8-channel blocks per warp
	int accl[NDB][4], acch[NDB][4];
#pragma unroll
	for (int i = 0; i < NDB; ++i)
#pragma unroll
		for (int j = 0; j < 4; ++j) accl[i][j] = acch[i][j] = 0;
	const int ngrp = w64 >> 6;
	constexpr int UG = 2;
	for (int grp0 = 0; grp0 < ngrp; grp0 += UG) {
		int4 vv[UG][NDB];
		int4 al[UG], ah[UG];
#pragma unroll
		for (int u = 0; u < UG; ++u) {
			const int page = (grp0 + u) * 4 + c;
			const bool live = page * kPageTokens < width;
			al[u] = ah[u] = make_int4(0, 0, 0, 0);
			if (g < G && live) {
				al[u] = *(const int4*)&s.pl[(size_t)g * wp + page * kPageTokens];
				ah[u] = *(const int4*)&s.ph[(size_t)g * wp + page * kPageTokens];
			}
#pragma unroll
			for (int i = 0; i < NDB; ++i) {
				vv[u][i] = make_int4(0, 0, 0, 0);
				if (live) {
					const int ch = (warp * NDB + i) * 8 + g;
					vv[u][i] = *(const int4*)(vplane + s.pbase[page] + ch * kPageTokens);
				}
			}
		}
#pragma unroll
		for (int u = 0; u < UG; ++u) {
#pragma unroll
			for (int i = 0; i < NDB; ++i) {
				const int4 v = vv[u][i];
				mma_u8s8(accl[i], (uint32_t)al[u].x, (uint32_t)al[u].y, (uint32_t)v.x, (uint32_t)v.y);
				mma_u8s8(accl[i], (uint32_t)al[u].z, (uint32_t)al[u].w, (uint32_t)v.z, (uint32_t)v.w);
				mma_u8s8(acch[i], (uint32_t)ah[u].x, (uint32_t)ah[u].y, (uint32_t)v.x, (uint32_t)v.y);
				mma_u8s8(acch[i], (uint32_t)ah[u].z, (uint32_t)ah[u].w, (uint32_t)v.z, (uint32_t)v.w);
			}
		}
	}
	// per-head context fold (forward_sites.cpp:1889-1896), store, row max for the funnel
	uint32_t lmax = 0;
	if (g < G) {
		const int head = kvh * G + g;
#pragma unroll
		for (int i = 0; i < NDB; ++i) {
			int2 o;
			o.x = fold(accl[i][0] + 256 * acch[i][0], fi, fm, fs);
			o.y = fold(accl[i][1] + 256 * acch[i][1], fi, fm, fs);
			const int ch = (warp * NDB + i) * 8 + c * 2;
			*(int2*)(b.ctxw + (size_t)r * d.hidden + (size_t)head * HD + ch) = o;
			const uint32_t ax = o.x < 0 ? 0u - (uint32_t)o.x : (uint32_t)o.x;
			const uint32_t ay = o.y < 0 ? 0u - (uint32_t)o.y : (uint32_t)o.y;
			lmax = max(lmax, max(ax, ay));
		}
	}
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) lmax = max(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
	if (lane == 0 && lmax) atomicMax(&b.rowmax[(size_t)r * 4 + 3], (unsigned long long)lmax);
}

static int pad_width(int w) { return (w + 63) / 64 * 64; }
template <int HD>
static void launch_attn(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index, KvPoolDev pool,
                        int wp, size_t sm, int reverse_rows, cudaStream_t st) {
	launch_pdl(k_attention<HD>, dim3(d.kv_heads, b.m), dim3(2 * HD), sm, st, b, d, layer, layer_index, pool, wp, reverse_rows);
}

cudaError_t attn_configure(const Dims& d) {
	const int group = d.heads / d.kv_heads;
	if (group < 1 || group > 8 || d.heads % d.kv_heads != 0) return cudaErrorInvalidConfiguration;
	const size_t need = attn_smem_bytes(group, pad_width(d.context_cap));
	if (need > 227 * 1024) return cudaErrorInvalidConfiguration;
	const int n = (int)need;
	const void* f = nullptr;
	if (d.head_dim == 128) f = (const void*)k_attention<128>;
	else if (d.head_dim == 64) f = (const void*)k_attention<64>;
	else if (d.head_dim == 32) f = (const void*)k_attention<32>;
	else return cudaErrorInvalidConfiguration;
	cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, n);
	if (e != cudaSuccess) return e;
	// same carve-out as the kernels around it (see rows_configure)
	return cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

void launch_attention(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index,
                      KvPoolDev pool, int max_width, int reverse_rows, cudaStream_t st) {
	const int wp = pad_width(max_width);
	const size_t sm = attn_smem_bytes(d.heads / d.kv_heads, wp);
	if (d.head_dim == 128) launch_attn<128>(b, d, layer, layer_index, pool, wp, sm, reverse_rows, st);
	else if (d.head_dim == 64) launch_attn<64>(b, d, layer, layer_index, pool, wp, sm, reverse_rows, st);
	else launch_attn<32>(b, d, layer, layer_index, pool, wp, sm, reverse_rows, st);
}

// ------------------------------------------------------------ canonical KV export
// Writes the sequence's K and V in the reference's save layout, [layer][K|V][kv head]
// [context_cap][head_dim] with zeros past the valid positions, undoing the paging and the
// V-page transposition.
__global__ void k_kv_export(Dims d, KvPoolDev pool, const int32_t* pages, int context_length,
                            int layer_index, int8_t* out) {
	const int hd = d.head_dim, vec = hd / 16;
	const int64_t per_plane = (int64_t)d.context_cap * vec;
	const int64_t total = (int64_t)d.layers * 2 * d.kv_heads * per_plane;
	for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
	     i += (int64_t)gridDim.x * blockDim.x) {
		const int64_t plane = i / per_plane, within = i - plane * per_plane;
		const int pos = (int)(within / vec), v = (int)(within % vec);
		const int kvh = (int)(plane % d.kv_heads);
		const int is_v = (int)((plane / d.kv_heads) % 2);
		const int layer = (int)(plane / (2 * d.kv_heads));
		// layers already run for the token in flight hold one more position
		const int valid = context_length + (layer < layer_index ? 1 : 0);
		int4 val = make_int4(0, 0, 0, 0);
		if (pos < valid) {
			const int8_t* src = pool.base + kv_plane_offset(d, pool, layer, kvh, is_v) +
			                    (int64_t)pages[pos / kPageTokens] * (kPageTokens * hd);
			const int slot = pos % kPageTokens;
			if (!is_v) {
				val = *((const int4*)(src + slot * hd) + v);
			} else {
				uint32_t w[4] = {0, 0, 0, 0};
				for (int j = 0; j < 16; ++j)
					w[j >> 2] |= (uint32_t)(uint8_t)src[(v * 16 + j) * kPageTokens + slot] << (8 * (j & 3));
				val = make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]);
			}
		}
		((int4*)out)[i] = val;
	}
}

void launch_kv_export(const Dims& d, KvPoolDev pool, const int32_t* pages, int context_length,
                      int layer_index, int8_t* out, cudaStream_t st) {
	k_kv_export<<<148 * 4, 256, 0, st>>>(d, pool, pages, context_length, layer_index, out);
}

// The inverse: scatter a canonical block (a save blob's K/V) into the sequence's pages.
// Only the valid positions are written; everything else in the pages is never read.
__global__ void k_kv_import(Dims d, KvPoolDev pool, const int32_t* pages, int context_length,
                            int layer_index, const int8_t* in) {
	const int hd = d.head_dim, vec = hd / 16;
	const int64_t per_plane = (int64_t)d.context_cap * vec;
	const int64_t total = (int64_t)d.layers * 2 * d.kv_heads * per_plane;
	for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
	     i += (int64_t)gridDim.x * blockDim.x) {
		const int64_t plane = i / per_plane, within = i - plane * per_plane;
		const int pos = (int)(within / vec), v = (int)(within % vec);
		const int kvh = (int)(plane % d.kv_heads);
		const int is_v = (int)((plane / d.kv_heads) % 2);
		const int layer = (int)(plane / (2 * d.kv_heads));
		const int valid = context_length + (layer < layer_index ? 1 : 0);
		if (pos >= valid) continue;
		const int4 val = ((const int4*)in)[i];
		int8_t* dst = pool.base + kv_plane_offset(d, pool, layer, kvh, is_v) +
		              (int64_t)pages[pos / kPageTokens] * (kPageTokens * hd);
		const int slot = pos % kPageTokens;
		if (!is_v) {
			*((int4*)(dst + slot * hd) + v) = val;
		} else {
			const uint32_t w[4] = {(uint32_t)val.x, (uint32_t)val.y, (uint32_t)val.z, (uint32_t)val.w};
			for (int j = 0; j < 16; ++j)
				dst[(v * 16 + j) * kPageTokens + slot] = (int8_t)((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
		}
	}
}

// Copy one page id to another in every (layer, kv head, K|V) plane: the private copy a
// sequence takes of an adopted prefix's last, partly filled page.
__global__ void k_page_copy(Dims d, KvPoolDev pool, int src_page, int dst_page) {
	const int64_t page_bytes = (int64_t)kPageTokens * d.head_dim;
	const int64_t plane_stride = pool.num_pages * page_bytes;
	int8_t* plane = pool.base + (int64_t)blockIdx.x * plane_stride;
	const int4* src = (const int4*)(plane + (int64_t)src_page * page_bytes);
	int4* dst = (int4*)(plane + (int64_t)dst_page * page_bytes);
	for (int i = threadIdx.x; i < (int)(page_bytes / 16); i += blockDim.x) dst[i] = src[i];
}
void launch_page_copy(const Dims& d, KvPoolDev pool, int src_page, int dst_page, cudaStream_t st) {
	k_page_copy<<<d.layers * d.kv_heads * 2, 128, 0, st>>>(d, pool, src_page, dst_page);
}

void launch_kv_import(const Dims& d, KvPoolDev pool, const int32_t* pages, int context_length,
                      int layer_index, const int8_t* in, cudaStream_t st) {
	k_kv_import<<<148 * 4, 256, 0, st>>>(d, pool, pages, context_length, layer_index, in);
}

}  // namespace sslm
