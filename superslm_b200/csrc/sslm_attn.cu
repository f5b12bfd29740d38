// Integer i-exp softmax attention over the paged int8 KV pool, staged through shared
// memory, with both contractions on the tensor cores (mma.sync m16n8k32, exact int32
// accumulation). A row (one token's q heads over positions 0..pos) is cut by kv head and along
// the context width; a block of head_dim/16 warps owns one slice of one kv head and serves every
// q head of the GQA group from one pass over its K and V pages, so each K / V byte of the
// sequence leaves HBM once per kv head. The blocks of a row form a thread-block cluster and
// exchange maxima, sums and partial contexts through distributed shared memory (k_attention).
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

#include <atomic>

#include "sslm_kernels.h"

namespace sslm {

// threads per block = 2 * head_dim: one warp per pair of 8-channel blocks of P.V
constexpr int kAttnMaxWarps = 8;

// One softmax element for constants that passed the gates of k_qkv_post (1 <= q_ln2 <= q_b
// < 2^24, q_c >= 0, peak = q_b^2 + q_c within the width gate): the value iexp_element()
// computes, on 32-bit words and without a branch. dq = max - score (0 <= dq < 2^32).
// z = floor(x / q_ln2) comes from a float estimate (within 1) repaired with the exact remainder.
//
// The reference also refuses an element whose value leaves [0, peak] (SoftmaxRowQ15's per-element
// bound, src/intmath.cpp:870-888). Under the gates above that cannot happen, so the kernels carry
// no such test: 0 <= rem < q_ln2 <= q_b gives 1 <= base = q_b - rem <= q_b, hence
// 0 <= (base^2 + q_c) >> z <= q_b^2 + q_c = peak (and peak >= 1 because q_b >= 1).
struct IExpFast {
	uint32_t ln2, clip;     // q_ln2, 30 * q_ln2
	int32_t qb;
	int64_t qc;
	float inv_ln2;
};
__device__ __forceinline__ IExpFast iexp_fast_prepare(const SoftmaxConsts& k) {
	IExpFast f;
	f.ln2 = (uint32_t)k.c.q_ln2;
	f.clip = 30u * f.ln2;
	f.qb = (int32_t)k.c.q_b;
	f.qc = k.c.q_c;
	f.inv_ln2 = 1.0f / (float)f.ln2;
	return f;
}
// *parts = (z << 24) | rem with x = z * q_ln2 + rem (rem < q_ln2 < 2^24, z <= 30): the second
// softmax pass rebuilds the element from it (iexp_from_parts) instead of dividing again.
constexpr uint32_t kPartsOfZero = 63u << 24;      // parts that rebuild to the value 0 (shift by 63)
__device__ __forceinline__ int64_t iexp_fast(uint32_t dq, const IExpFast& f, uint32_t* parts) {
	const uint32_t x = min(dq, f.clip);
	int32_t z = __float2int_rz(__uint2float_rn(x) * f.inv_ln2);
	int32_t rem = (int32_t)(x - (uint32_t)z * f.ln2);
	const int32_t adj = rem < 0 ? -1 : (rem >= (int32_t)f.ln2 ? 1 : 0);
	z += adj;
	rem -= adj * (int32_t)f.ln2;
	const int32_t base = f.qb - rem;
	*parts = ((uint32_t)z << 24) | (uint32_t)rem;
	return ((int64_t)base * (int64_t)base + f.qc) >> z;
}
__device__ __forceinline__ int64_t iexp_from_parts(uint32_t parts, const IExpFast& f) {
	const int32_t base = f.qb - (int32_t)(parts & 0xFFFFFFu);
	return ((int64_t)base * (int64_t)base + f.qc) >> (parts >> 24);
}
// floor((e << 15) / tot) for 0 <= e <= min(tot, 2^47), 1 <= tot < 2^63, rinv = 32768 / tot in
// float: the float quotient is within 2^-6 of the true one, so its floor is off by at most one
// either way, and one signed remainder settles it (|e * 2^15 - p * tot| < 2 * tot stays inside
// 64 bits because e * 2^15 <= 2^62).
__device__ __forceinline__ uint32_t prob_q15(int64_t e, unsigned long long tot, float rinv) {
	const unsigned long long num = (unsigned long long)e << 15;
	uint32_t p = min(__float2uint_rz(__ll2float_rn(e) * rinv), 32768u);
	const long long r = (long long)(num - (unsigned long long)p * tot);
	p -= r < 0 ? 1u : 0u;
	p += r >= (long long)tot ? 1u : 0u;
	return p;
}
// bytes 0 (low plane) or 1 (high plane) of four probabilities, packed into one word
__device__ __forceinline__ uint32_t pack_plane(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3, int byte) {
	const uint32_t sel = byte ? 0x0051u : 0x0040u;
	return __byte_perm(__byte_perm(p0, p1, sel), __byte_perm(p2, p3, sel), 0x5410u);
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

// ---- thread-block cluster helpers (distributed shared memory)
__device__ __forceinline__ uint32_t cluster_rank() {
	uint32_t r;
	asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
	return r;
}
// the address, in the cluster's shared window, of `local` (a shared-memory address of this
// block) inside the block of rank `rank`
__device__ __forceinline__ uint32_t peer_addr(const void* local, uint32_t rank) {
	uint32_t a = (uint32_t)__cvta_generic_to_shared(local), out;
	asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(a), "r"(rank));
	return out;
}
__device__ __forceinline__ uint32_t peer_ld32(uint32_t addr) {
	uint32_t v;
	asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
	return v;
}
__device__ __forceinline__ unsigned long long peer_ld64(uint32_t addr) {
	unsigned long long v;
	asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
	return v;
}
// Hardware barrier over all threads of all blocks of the cluster: everything written to shared
// memory before it is visible to every block after it. Every block of a cluster executes every
// barrier of the kernel (no early return), so nothing can wait for a block that left.
__device__ __forceinline__ void cluster_sync_all() {
	asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
	asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// What one block keeps in shared memory. `cp` = positions a block can hold (a multiple of 64).
struct AttnSmem {
	int64_t* pbase;       // [cp/16] byte offset of each of the block's pages inside a plane
	int32_t* sc;          // [G][cp] scores, later (shift, remainder) of each element
	uint8_t* pl;          // [G][cp] low byte of the Q15 probability
	uint8_t* ph;          // [G][cp] high byte
	unsigned long long* red;   // [8 heads][warps] partials inside the block
	// what the other blocks of the cluster read (one block = one slice of one kv head's row):
	int32_t* x_max;       // [8] largest score per head in this slice
	unsigned long long* x_sum;   // [8] sum of the slice's exponentials per head
	int32_t* x_ctx;       // [8][HD] this slice's share of P.V per head
	uint32_t* x_flags;    // [0] the slice met an element the reference refuses, [1] largest folded |ctx| of the
	                      //     channels this block reduced, [2] this block sits the row out
	// local copies of what the exchanges fetched (a few threads read the peers, everybody reads these)
	int32_t* l_max;       // [8] row maximum per head
	unsigned long long* l_sum;   // [8] row total per head
	uint32_t* l_misc;     // [0] some block refused the row, [1] largest folded |ctx| of the row
	int32_t* l_fold;      // [8][3] context fold (identity, multiplier, shift) of this kv head's q heads
};
__host__ __device__ inline size_t attn_smem_bytes(int group, int cp, int hd) {
	return (size_t)cp / 16 * 8 + (size_t)group * cp * 6 + 8 * kAttnMaxWarps * 8 + 8 * 4 + 8 * 8 + (size_t)8 * hd * 4 + 16 +
	       8 * 8 + 8 * 4 + 8 + 24 * 4;
}
__device__ __forceinline__ AttnSmem carve(unsigned char* smem, int group, int cp, int hd) {
	AttnSmem s;
	s.pbase = (int64_t*)smem;
	s.sc = (int32_t*)(smem + (size_t)cp / 16 * 8);
	s.pl = (uint8_t*)(s.sc + (size_t)group * cp);
	s.ph = s.pl + (size_t)group * cp;
	s.red = (unsigned long long*)(s.ph + (size_t)group * cp);
	s.x_sum = s.red + 8 * kAttnMaxWarps;
	s.x_max = (int32_t*)(s.x_sum + 8);
	s.x_ctx = s.x_max + 8;
	s.x_flags = (uint32_t*)(s.x_ctx + 8 * hd);
	s.l_sum = (unsigned long long*)(s.x_flags + 4);
	s.l_max = (int32_t*)(s.l_sum + 8);
	s.l_misc = (uint32_t*)(s.l_max + 8);
	s.l_fold = (int32_t*)(s.l_misc + 2);
	return s;
}
// ask for the line at p to be brought into L2; nothing waits for it
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// One attention row = one token of one sequence, all its q heads over the positions 0..pos.
// The row is cut two ways: by kv head (a block serves the q heads of one GQA group, so K and V
// bytes are read once per kv head) and along the context width into `splits` slices of
// `slice_len(width)` positions. The blocks of a row -- kv_heads x splits of them when
// `whole_row`, else the `splits` of one kv head -- form one thread-block cluster and meet three
// times through distributed shared memory, which is what the exact integer softmax needs
// (SoftmaxRowQ15 is not mergeable online: an element's exponential depends on the row maximum
// through floor divisions):
//   1  scores of the slice (tensor cores), slice maximum per head      -> exchange: row maximum
//   2  e_k per element, slice sum per head, refusal flag               -> exchange: row total
//   3  p_k = (e_k << 15) / total, the slice's share of P.V (tensor cores) -> exchange: the shares
//      are added per channel (integer adds: any order), then folded per head
// and, when the cluster holds the whole row, a fourth time for the attention-context funnel
// (forward_sites.cpp:1898-1903): largest folded magnitude of the row -> codes and carried scale,
// so that no separate funnel kernel runs. HD = head_dim (32, 64 or 128); threads = 2 * HD.
template <int HD>
__global__ void __launch_bounds__(2 * HD, HD == 128 ? 4 : 8)
k_attention(RowBatch b, Dims d, const LayerDev* layer, int layer_index, KvPoolDev pool, int cp, int splits, int whole_row,
            int reverse_rows) {
	extern __shared__ __align__(16) unsigned char smem[];
	// blocks start in index order: with reverse_rows the last (widest) rows of a prefill chunk go first
	const int r = reverse_rows ? (int)gridDim.y - 1 - (int)blockIdx.y : (int)blockIdx.y;
	const int kvh = (int)blockIdx.x / splits, split = (int)blockIdx.x % splits;
	constexpr int kAttnThreads = 2 * HD, kAttnWarps = kAttnThreads / 32;
	const int G = d.heads / d.kv_heads;
	const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
	const int g = lane >> 2, c = lane & 3;
	const AttnSmem s = carve(smem, G, cp, HD);
	const uint32_t my_rank = cluster_rank();
	const uint32_t kv_rank0 = my_rank - (uint32_t)split;     // rank of this kv head's first slice
	const uint32_t cluster_blocks = whole_row ? (uint32_t)(d.kv_heads * splits) : (uint32_t)splits;
	// Ahead of the kernel that lands this step's K / V rows (it may still be running): the row
	// descriptor and the page table were uploaded before the step's first launch, and every K / V
	// row but the newest was written by earlier steps. So the page offsets are staged now, and
	// the slice's old K rows are asked into L2 while that kernel, which moves little data, finishes.
	const int width = b.rows[r].pos + 1;
	// slice length: the row's width over the slices, rounded up to whole 64-position groups
	const int slen = ((width + splits - 1) / splits + 63) & ~63;
	const int p0 = split * slen;                                   // first position of this slice
	const int n = max(0, min(slen, width - p0));                   // positions in it
	const int n64 = (n + 63) & ~63;
	const int8_t* kplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 0);
	const int8_t* vplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 1);
	const int npages = (n + kPageTokens - 1) / kPageTokens;
	{
		// entries beyond the slice's last page, up to the 64-position group stage 3 reads, repeat
		// that page: their probabilities are zero, so any readable V words will do
		const int32_t* pages = b.rows[r].pages + p0 / kPageTokens;
		for (int j = t; j < (n64 >> 4); j += kAttnThreads)
			s.pbase[j] = (int64_t)pages[min(j, npages - 1)] * (kPageTokens * HD);
	}
	const FunnelFold fold_ctx = funnel_prefold(nullptr, 0, layer->c_ctx);
	if (t < 3 * G) s.l_fold[t] = layer->f_ctx[3 * kvh * G + t];      // (weights: ahead of the wait)
	__syncthreads();
	constexpr int kRowsPerLine = 128 / HD;
	for (int pos = t * kRowsPerLine; pos < n - (p0 + n == width ? 1 : 0); pos += kAttnThreads * kRowsPerLine)
		prefetch_l2(kplane + s.pbase[pos >> 4] + (pos & 15) * HD);
	pdl_wait();
	pdl_release();
	// A row that an earlier site refused is sat out: no loads, zero contributions, but every
	// barrier. One thread reads the word for the block; blocks of a cluster may see different
	// words (another block can refuse the row while this one runs), which is harmless: a refused
	// row's outputs are never used.
	if (t == 0) s.x_flags[2] = __ldcg(&b.status[r]) != 0 ? 1u : 0u;
	if (t < 8) {
		s.x_max[t] = INT32_MIN;
		s.x_sum[t] = 0ull;
		s.l_max[t] = INT32_MIN;
		s.l_sum[t] = 0ull;
	}
	if (t == 8) s.x_flags[0] = 0u;
	if (t == 9) s.x_flags[1] = 0u;
	const SoftmaxConsts smc = b.smc[(size_t)r * d.kv_heads + kvh];   // wanted after the scores; asked for now
	__syncthreads();
	const bool live = s.x_flags[2] == 0u;
	// A row that is one slice of one kv head has nobody to meet: the block keeps everything local
	// (and may leave early).
	const bool solo = splits == 1 && !whole_row;
	if (solo && !live) return;

	// ---- stage 1: scores, 8 positions per MMA group, groups dealt round-robin to the warps, and the
	// slice's maximum per head on the way. Lanes beyond the slice's end read its last position again
	// (no predicated loads); their columns are stored as INT32_MIN, which the maximum ignores.
	int32_t* const s_max = solo ? s.l_max : s.x_max;
	unsigned long long* const s_sum = solo ? s.l_sum : s.x_sum;
	if (live) {
		constexpr int NW = HD / 16;
		uint32_t qw[NW];
		load_row_words<HD>(b.qrot + (size_t)r * d.hidden + (size_t)(kvh * G + min(g, G - 1)) * HD, c, qw);
		const int nblk = (n + 7) >> 3;
		constexpr int U = 4;
		int rmax = INT32_MIN;
		for (int blk0 = warp * U; blk0 < nblk; blk0 += kAttnWarps * U) {
			uint32_t kw[U][NW];
#pragma unroll
			for (int u = 0; u < U; ++u) {
				const int pos = min((blk0 + u) * 8 + g, n - 1);
				load_row_words<HD>(kplane + s.pbase[pos >> 4] + (pos & 15) * HD, c, kw[u]);
			}
#pragma unroll
			for (int u = 0; u < U; ++u) {
				int acc[4] = {0, 0, 0, 0};
#pragma unroll
				for (int j = 0; j < NW / 2; ++j) mma_s8s8(acc, qw[2 * j], qw[2 * j + 1], kw[u][2 * j], kw[u][2 * j + 1]);
				const int k = (blk0 + u) * 8 + c * 2;
				if (g < G && blk0 + u < nblk) {
					const int v0 = k < n ? acc[0] : INT32_MIN, v1 = k + 1 < n ? acc[1] : INT32_MIN;
					*(int2*)&s.sc[(size_t)g * cp + k] = make_int2(v0, v1);
					rmax = max(rmax, max(v0, v1));
				}
			}
		}
		rmax = max(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
		rmax = max(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
		if (c == 0 && g < G && rmax != INT32_MIN) atomicMax(&s_max[g], rmax);
	}
	__syncthreads();

	// the softmax below moves no data: ask for this slice's V pages (16 lines each) meanwhile
	if (live)
		for (int ln = t; ln < npages * (kPageTokens * HD / 128); ln += kAttnThreads)
			prefetch_l2(vplane + s.pbase[ln / (kPageTokens * HD / 128)] + (ln % (kPageTokens * HD / 128)) * 128);

	if (!solo) {
		cluster_sync_all();      // ---- exchange 1: every slice's maxima are up
		// (one thread per head fetches the peers' values; reading them from every thread would put
		// thousands of remote loads on the cluster's shared-memory network)
		if (t < G) {
			int m = INT32_MIN;
			for (int j = 0; j < splits; ++j) m = max(m, (int)peer_ld32(peer_addr(&s.x_max[t], kv_rank0 + (uint32_t)j)));
			s.l_max[t] = m;
		}
		__syncthreads();
	}

	// ---- stage 2: softmax. The work is dealt to the warps as (head, 128-position chunk) pairs, so
	// that every warp is busy whatever the width; a lane takes 4 consecutive positions. First the
	// exponentials and their sum per head; the score's place then holds the element's
	// (shift, remainder), which the probability pass rebuilds it from.
	const IExpFast fx = iexp_fast_prepare(smc);
	const int nchunk = (n64 + 127) >> 7;
	if (live) {
#pragma unroll 1
		for (int pr = warp; pr < G * nchunk; pr += kAttnWarps) {
			const int h = pr / nchunk, k4 = (pr - h * nchunk) * 128 + lane * 4;
			unsigned long long tot = 0;
			if (k4 < n) {
				int32_t* row = s.sc + (size_t)h * cp;
				const uint32_t m = (uint32_t)s.l_max[h];
				const int4 v = *(const int4*)&row[k4];
				uint32_t q0, q1, q2, q3;
				const int64_t e0 = iexp_fast(m - (uint32_t)v.x, fx, &q0);
				int64_t e1 = iexp_fast(m - (uint32_t)v.y, fx, &q1);
				int64_t e2 = iexp_fast(m - (uint32_t)v.z, fx, &q2);
				int64_t e3 = iexp_fast(m - (uint32_t)v.w, fx, &q3);
				if (k4 + 3 >= n) {       // the row's last group: positions beyond its end count for nothing
					if (k4 + 1 >= n) { e1 = 0; q1 = kPartsOfZero; }
					if (k4 + 2 >= n) { e2 = 0; q2 = kPartsOfZero; }
					e3 = 0; q3 = kPartsOfZero;
				}
				tot = (unsigned long long)(e0 + e1) + (unsigned long long)(e2 + e3);
				*(int4*)&row[k4] = make_int4((int)q0, (int)q1, (int)q2, (int)q3);
			}
			// a lane's partial is below 2^50; three 24-bit limbs add up across the warp without
			// leaving 32 bits, one warp-reduce instruction each
			const uint32_t l0 = __reduce_add_sync(0xffffffffu, (uint32_t)tot & 0xFFFFFFu);
			const uint32_t l1 = __reduce_add_sync(0xffffffffu, (uint32_t)(tot >> 24) & 0xFFFFFFu);
			const uint32_t l2 = __reduce_add_sync(0xffffffffu, (uint32_t)(tot >> 48));
			if (lane == 0) atomicAdd(&s_sum[h], (unsigned long long)l0 + ((unsigned long long)l1 << 24) + ((unsigned long long)l2 << 48));
		}
	}
	if (solo) {
		__syncthreads();
	} else {
		cluster_sync_all();      // ---- exchange 2: every slice's sums are up
		if (t < G) {
			unsigned long long x = 0;
			for (int j = 0; j < splits; ++j) x += peer_ld64(peer_addr(&s.x_sum[t], kv_rank0 + (uint32_t)j));
			s.l_sum[t] = x;
		}
		__syncthreads();
	}
	const bool work = live;
	// probabilities as two u8 planes, zero beyond the slice up to the next multiple of 64 (stage 3
	// reads whole 64-position groups)
	if (work) {
		const int n4 = (n + 3) & ~3;
#pragma unroll 1
		for (int pr = warp; pr < G * nchunk; pr += kAttnWarps) {
			const int h = pr / nchunk, k4 = (pr - h * nchunk) * 128 + lane * 4;
			if (k4 < n4) {
				const unsigned long long x = s.l_sum[h];
				const unsigned long long tot = x > 1ull ? x : 1ull;
				const float inv = 32768.0f / (float)tot;
				const int4 v = *(const int4*)&s.sc[(size_t)h * cp + k4];
				const uint32_t p0 = prob_q15(iexp_from_parts((uint32_t)v.x, fx), tot, inv);
				const uint32_t p1 = prob_q15(iexp_from_parts((uint32_t)v.y, fx), tot, inv);
				const uint32_t p2 = prob_q15(iexp_from_parts((uint32_t)v.z, fx), tot, inv);
				const uint32_t p3 = prob_q15(iexp_from_parts((uint32_t)v.w, fx), tot, inv);
				*(uint32_t*)&s.pl[(size_t)h * cp + k4] = pack_plane(p0, p1, p2, p3, 0);
				*(uint32_t*)&s.ph[(size_t)h * cp + k4] = pack_plane(p0, p1, p2, p3, 1);
			} else if (k4 < n64) {
				*(uint32_t*)&s.pl[(size_t)h * cp + k4] = 0u;
				*(uint32_t*)&s.ph[(size_t)h * cp + k4] = 0u;
			}
		}
	}
	__syncthreads();

	// ---- stage 3: the slice's share of ctx = P V. Lane column c owns page 4*grp + c of each
	// 64-position group; its 16-byte row of the transposed page feeds two MMAs (positions 0..7 and
	// 8..15). Nothing is predicated: the page table and the planes are padded to whole groups, and
	// lanes of MMA rows beyond the group's heads read head 0's probabilities (their output rows are
	// never stored).
	constexpr int NDB = 2;            // 8-channel blocks per warp
	int accl[NDB][4], acch[NDB][4];
#pragma unroll
	for (int i = 0; i < NDB; ++i)
#pragma unroll
		for (int j = 0; j < 4; ++j) accl[i][j] = acch[i][j] = 0;
	if (work) {
		const int ngrp = n64 >> 6;
		const uint8_t* pl = s.pl + (size_t)(g < G ? g : 0) * cp + c * kPageTokens;
		const uint8_t* ph = s.ph + (size_t)(g < G ? g : 0) * cp + c * kPageTokens;
		const int8_t* vch = vplane + (warp * NDB * 8 + g) * kPageTokens;
		// UG groups' V words are requested before the first of them is used
		constexpr int UG = 4;
		auto group = [&](int grp, const int4 (&vv)[NDB]) {
			const int4 al = *(const int4*)(pl + grp * 64);
			const int4 ah = *(const int4*)(ph + grp * 64);
#pragma unroll
			for (int i = 0; i < NDB; ++i) {
				const int4 v = vv[i];
				mma_u8s8(accl[i], (uint32_t)al.x, (uint32_t)al.y, (uint32_t)v.x, (uint32_t)v.y);
				mma_u8s8(accl[i], (uint32_t)al.z, (uint32_t)al.w, (uint32_t)v.z, (uint32_t)v.w);
				mma_u8s8(acch[i], (uint32_t)ah.x, (uint32_t)ah.y, (uint32_t)v.x, (uint32_t)v.y);
				mma_u8s8(acch[i], (uint32_t)ah.z, (uint32_t)ah.w, (uint32_t)v.z, (uint32_t)v.w);
			}
		};
		int grp0 = 0;
		for (; grp0 + UG <= ngrp; grp0 += UG) {
			int4 vv[UG][NDB];
#pragma unroll
			for (int u = 0; u < UG; ++u) {
				const int64_t pb = s.pbase[(grp0 + u) * 4 + c];
#pragma unroll
				for (int i = 0; i < NDB; ++i) vv[u][i] = *(const int4*)(vch + pb + i * 8 * kPageTokens);
			}
#pragma unroll
			for (int u = 0; u < UG; ++u) group(grp0 + u, vv[u]);
		}
		for (; grp0 < ngrp; ++grp0) {
			int4 vv[NDB];
			const int64_t pb = s.pbase[grp0 * 4 + c];
#pragma unroll
			for (int i = 0; i < NDB; ++i) vv[i] = *(const int4*)(vch + pb + i * 8 * kPageTokens);
			group(grp0, vv);
		}
	}
	if (solo) {
		// per-head context fold (forward_sites.cpp:1889-1896), store, row maximum for the funnel
		uint32_t smax = 0;
		if (g < G) {
			const int head = kvh * G + g;
			const int32_t fi = s.l_fold[3 * g], fm = s.l_fold[3 * g + 1], fs = s.l_fold[3 * g + 2];
#pragma unroll
			for (int i = 0; i < NDB; ++i) {
				int2 o;
				o.x = fold(accl[i][0] + 256 * acch[i][0], fi, fm, fs);
				o.y = fold(accl[i][1] + 256 * acch[i][1], fi, fm, fs);
				const int ch = (warp * NDB + i) * 8 + c * 2;
				*(int2*)(b.ctxw + (size_t)r * d.hidden + (size_t)head * HD + ch) = o;
				const uint32_t ax = o.x < 0 ? 0u - (uint32_t)o.x : (uint32_t)o.x;
				const uint32_t ay = o.y < 0 ? 0u - (uint32_t)o.y : (uint32_t)o.y;
				smax = max(smax, max(ax, ay));
			}
		}
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) smax = max(smax, __shfl_xor_sync(0xffffffffu, smax, o));
		if (lane == 0 && smax) atomicMax(&b.rowmax[(size_t)r * 4 + 3], (unsigned long long)smax);
		return;
	}
	// the slice's share, [head][channel], for the block that reduces that channel
	if (g < G) {
#pragma unroll
		for (int i = 0; i < NDB; ++i) {
			const int ch = (warp * NDB + i) * 8 + c * 2;
			*(int2*)&s.x_ctx[g * HD + ch] = make_int2(accl[i][0] + 256 * acch[i][0], accl[i][1] + 256 * acch[i][1]);
		}
	}
	cluster_sync_all();      // ---- exchange 3: every slice's share of P.V is up

	// Slice `split` of a kv head reduces channels [split * HD / splits, ...) of each of its heads:
	// add the shares, per-head context fold (forward_sites.cpp:1889-1896), row maximum.
	const int per = (HD + splits - 1) / splits;                    // channels per block
	const int ch0 = split * per, nch = max(0, min(per, HD - ch0));
	// element e of this block = (head e / nch, channel ch0 + e % nch); at most G * HD <= 2 * threads * ... per block
	uint32_t lmax = 0;
	constexpr int kMaxMine = 4;                                   // G * per <= 8 * HD = 4 * threads
	int32_t mine[kMaxMine];
#pragma unroll
	for (int q = 0; q < kMaxMine; ++q) {
		mine[q] = 0;
		const int e = q * kAttnThreads + t;
		if (e < G * nch) {
			const int h = e / nch, ch = ch0 + e - h * nch;
			int32_t sum = 0;
			for (int j = 0; j < splits; ++j) sum += (int32_t)peer_ld32(peer_addr(&s.x_ctx[h * HD + ch], kv_rank0 + (uint32_t)j));
			const int32_t o = fold(sum, s.l_fold[3 * h], s.l_fold[3 * h + 1], s.l_fold[3 * h + 2]);
			mine[q] = o;
			lmax = max(lmax, o < 0 ? 0u - (uint32_t)o : (uint32_t)o);
			if (!whole_row && work) b.ctxw[(size_t)r * d.hidden + (size_t)(kvh * G + h) * HD + ch] = o;
		}
	}
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) lmax = max(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
	if (!whole_row) {
		if (lane == 0 && lmax && work) atomicMax(&b.rowmax[(size_t)r * 4 + 3], (unsigned long long)lmax);
		cluster_sync_all();  // nobody leaves while its shared memory may still be read
		return;
	}
	// ---- the cluster holds the whole row: its funnel runs here
	if (lane == 0 && lmax) atomicMax(&s.x_flags[1], lmax);
	cluster_sync_all();      // ---- exchange 4: every block's largest folded magnitude is up
	if (t == 0) {
		uint32_t v = 0;
		for (uint32_t j = 0; j < cluster_blocks; ++j) v = max(v, peer_ld32(peer_addr(&s.x_flags[1], j)));
		s.l_misc[1] = v;
	}
	__syncthreads();
	const uint32_t rowmx = s.l_misc[1];
	const FunnelParams fp = funnel_finish((unsigned long long)rowmx, fold_ctx);
	if (work) {
		if (fp.status != kOk) {
			if (my_rank == 0 && t == 0) atomicCAS(&b.status[r], 0, pack_status(fp.status, kSiteCtx, b.layer));
		} else {
			const Coder cd = make_coder(fp.r, fp.s);
#pragma unroll
			for (int q = 0; q < kMaxMine; ++q) {
				const int e = q * kAttnThreads + t;
				if (e < G * nch) {
					const int h = e / nch, ch = ch0 + e - h * nch;
					b.ctx[(size_t)r * d.hidden + (size_t)(kvh * G + h) * HD + ch] = code_of(mine[q], cd);
				}
			}
			if (my_rank == 0 && t == 0) b.cs[r] = fp.out;
		}
	}
	cluster_sync_all();      // nobody leaves while its shared memory may still be read
}

// ------------------------------------------------------------ prefill: query-tiled attention
// The rows of a prefill chunk are consecutive positions of ONE sequence, so neighbouring tokens
// read almost the same K / V prefix. A block takes a tile of TQ consecutive tokens of one kv head
// -- TQ * G = up to 64 query rows (token, q head), four 16-row MMA blocks -- and walks the prefix
// in steps of 64 positions staged in shared memory (cp.async, double buffered): every K / V byte
// is fetched once per tile instead of once per token. The exact integer softmax needs the row
// maximum before any exponential and the row total before any probability, so the prefix is
// walked three times: (1) scores -> row maxima, (2) scores -> exponentials -> row totals,
// (3) scores -> probabilities -> P.V. Scores are recomputed each time (tensor-core work, cheap
// beside the integer softmax); nothing of size rows x width is ever stored. The causal limit is
// per row: token i of the tile sees positions <= pos0 + i.
// Warp w works on MMA block w / 2 (16 query rows) and on half w % 2 of each 64-position step
// (scores) respectively half w % 2 of the channels (P.V).
constexpr int kTileRows = 64;
constexpr int kTileKeys = 64;
constexpr int kTileThreads = 256;
constexpr int kTilePStride = 80;      // bytes per row of the probability planes (64 + padding against bank conflicts)

__device__ __forceinline__ void mma_s8s8_full(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
	asm volatile(
	    "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
	    : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
	    : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8_full(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
	asm volatile(
	    "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
	    : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
	    : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int HD>
struct TileSmem {
	static constexpr int kKStride = HD + 16;                       // bytes per staged K row (padding against bank conflicts)
	static constexpr size_t kK = (size_t)2 * kTileKeys * kKStride;
	static constexpr size_t kV = (size_t)2 * kTileKeys * HD;
	static constexpr size_t kP = (size_t)2 * kTileRows * kTilePStride;
	static constexpr size_t kFx = (size_t)kTileRows * sizeof(IExpFast);
	static constexpr size_t kMisc = (size_t)kTileRows * (4 + 2 * 4 + 2 * 8) + 8 * 3 * 4 + 64;
	static constexpr size_t kBytes = kK + kV + kP + kFx + kMisc;
};

template <int HD>
__global__ void __launch_bounds__(kTileThreads, 2)
k_attention_tile(RowBatch b, Dims d, const LayerDev* layer, int layer_index, KvPoolDev pool, int tq) {
	using L = TileSmem<HD>;
	constexpr int KS = HD / 32;          // MMA steps along the head dimension
	constexpr int NGW = HD / 16;         // 8-channel groups a warp owns in P.V
	extern __shared__ __align__(16) unsigned char smem[];
	int8_t* Ks = (int8_t*)smem;
	int8_t* Vs = (int8_t*)(smem + L::kK);
	uint8_t* Pl = (uint8_t*)(smem + L::kK + L::kV);
	uint8_t* Ph = Pl + (size_t)kTileRows * kTilePStride;
	IExpFast* fxs = (IExpFast*)(smem + L::kK + L::kV + L::kP);
	unsigned long long* wsum = (unsigned long long*)(fxs + kTileRows);      // [2][64]
	int32_t* wmax = (int32_t*)(wsum + 2 * kTileRows);                        // [2][64]
	int32_t* tok_ok = wmax + 2 * kTileRows;                                  // [64] 1: the token takes part
	int32_t* l_fold = tok_ok + kTileRows;                                    // [8][3]

	const int kvh = blockIdx.x;
	const int tile = (int)gridDim.y - 1 - (int)blockIdx.y;      // the last (widest) tiles start first
	const int G = d.heads / d.kv_heads;
	const int r0 = tile * tq, nt = min(tq, b.m - r0);
	const int t = threadIdx.x, warp = t >> 5, lane = t & 31, g = lane >> 2, c = lane & 3;
	const int mb = warp >> 1, ph = warp & 1;
	// this lane's two query rows (token, head)
	const int rho_a = mb * 16 + g, rho_b = rho_a + 8;
	const int tok_a = rho_a / G, tok_b = rho_b / G;
	const int head_a = rho_a - tok_a * G, head_b = rho_b - tok_b * G;
	// uploaded before the step's first launch: the tile's first position and the sequence's page table
	const int pos0 = b.rows[r0].pos;
	const int32_t* pages = b.rows[r0].pages;
	const int width = pos0 + nt;
	const int nblk = (width + kTileKeys - 1) / kTileKeys;
	const int8_t* kplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 0);
	const int8_t* vplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 1);
	if (t < 3 * G) l_fold[t] = layer->f_ctx[3 * kvh * G + t];
	pdl_wait();
	pdl_release();
	if (t < kTileRows) {
		int okv = 0;
		if (t < nt) {
			okv = __ldcg(&b.status[r0 + t]) == 0 ? 1 : 0;
			fxs[t] = iexp_fast_prepare(b.smc[(size_t)(r0 + t) * d.kv_heads + kvh]);
		}
		tok_ok[t] = okv;
	}
	__syncthreads();
	const bool in_a = tok_a < nt && tok_ok[tok_a] != 0, in_b = tok_b < nt && tok_ok[tok_b] != 0;
	const int lim_a = in_a ? pos0 + tok_a : -1, lim_b = in_b ? pos0 + tok_b : -1;    // last position each row sees
	// q fragments (A operand) of this warp's MMA block, kept in registers for all three walks
	uint32_t qa[KS][4];
	{
		const int8_t* qpa = b.qrot + (size_t)(r0 + (in_a ? tok_a : 0)) * d.hidden + (size_t)(kvh * G + head_a) * HD;
		const int8_t* qpb = b.qrot + (size_t)(r0 + (in_b ? tok_b : 0)) * d.hidden + (size_t)(kvh * G + head_b) * HD;
#pragma unroll
		for (int ks = 0; ks < KS; ++ks) {
			qa[ks][0] = in_a ? *(const uint32_t*)(qpa + 32 * ks + 4 * c) : 0u;
			qa[ks][1] = in_b ? *(const uint32_t*)(qpb + 32 * ks + 4 * c) : 0u;
			qa[ks][2] = in_a ? *(const uint32_t*)(qpa + 32 * ks + 16 + 4 * c) : 0u;
			qa[ks][3] = in_b ? *(const uint32_t*)(qpb + 32 * ks + 16 + 4 * c) : 0u;
		}
	}
	const IExpFast fa = fxs[in_a ? tok_a : 0], fb = fxs[in_b ? tok_b : 0];

	// stage step `blk` of the prefix: K rows (and V pages) of positions blk * 64 ...; positions
	// beyond the tile's width are left as they are (their scores are masked, their probabilities zero)
	auto load_block = [&](int stage, int blk, bool with_v) {
		int8_t* kd = Ks + (size_t)stage * kTileKeys * L::kKStride;
		for (int idx = t; idx < kTileKeys * (HD / 16); idx += kTileThreads) {
			const int row = idx / (HD / 16), piece = idx - row * (HD / 16);
			const int pos = blk * kTileKeys + row;
			if (pos < width)
				cp_async16(kd + (size_t)row * L::kKStride + piece * 16,
				           kplane + (int64_t)pages[pos >> 4] * (kPageTokens * HD) + (pos & 15) * HD + piece * 16);
		}
		if (with_v) {
			int8_t* vd = Vs + (size_t)stage * kTileKeys * HD;
			for (int idx = t; idx < 4 * HD; idx += kTileThreads) {
				const int pg = idx / HD, piece = idx - pg * HD;
				const int page = blk * 4 + pg;
				if (page * kPageTokens < width)
					cp_async16(vd + (size_t)pg * HD * kPageTokens + piece * 16,
					           vplane + (int64_t)pages[page] * (kPageTokens * HD) + piece * 16);
			}
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	// scores of this warp's 16 rows x 32 positions of the staged step
	auto scores = [&](int stage, int (&acc)[4][4]) {
		const int8_t* kd = Ks + (size_t)stage * kTileKeys * L::kKStride;
#pragma unroll
		for (int j = 0; j < 4; ++j) {
#pragma unroll
			for (int q = 0; q < 4; ++q) acc[j][q] = 0;
			const int8_t* krow = kd + (size_t)(32 * ph + 8 * j + g) * L::kKStride;
#pragma unroll
			for (int ks = 0; ks < KS; ++ks) {
				const uint32_t b0 = *(const uint32_t*)(krow + 32 * ks + 4 * c);
				const uint32_t b1 = *(const uint32_t*)(krow + 32 * ks + 16 + 4 * c);
				mma_s8s8_full(acc[j], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
			}
		}
	};
	// walk the prefix: `body(stage, blk)` runs with step blk staged; the next step loads meanwhile
	auto walk = [&](bool with_v, auto&& body) {
		load_block(0, 0, with_v);
		for (int blk = 0; blk < nblk; ++blk) {
			const int stage = blk & 1;
			if (blk + 1 < nblk) {
				load_block(stage ^ 1, blk + 1, with_v);
				asm volatile("cp.async.wait_group 1;" ::: "memory");
			} else {
				asm volatile("cp.async.wait_group 0;" ::: "memory");
			}
			__syncthreads();
			body(stage, blk);
			__syncthreads();      // the stage (and the probability planes) may be overwritten
		}
	};

	// ---- walk 1: row maxima
	int mx_a = INT32_MIN, mx_b = INT32_MIN;
	walk(false, [&](int stage, int blk) {
		int acc[4][4];
		scores(stage, acc);
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const int k0 = blk * kTileKeys + 32 * ph + 8 * j + 2 * c;
			if (k0 <= lim_a) mx_a = max(mx_a, acc[j][0]);
			if (k0 + 1 <= lim_a) mx_a = max(mx_a, acc[j][1]);
			if (k0 <= lim_b) mx_b = max(mx_b, acc[j][2]);
			if (k0 + 1 <= lim_b) mx_b = max(mx_b, acc[j][3]);
		}
	});
	mx_a = max(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
	mx_a = max(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
	mx_b = max(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
	mx_b = max(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
	if (c == 0) {
		wmax[ph * kTileRows + rho_a] = mx_a;
		wmax[ph * kTileRows + rho_b] = mx_b;
	}
	__syncthreads();
	mx_a = max(wmax[rho_a], wmax[kTileRows + rho_a]);
	mx_b = max(wmax[rho_b], wmax[kTileRows + rho_b]);

	// ---- walk 2: exponentials and row totals (elements beyond a row's causal limit are computed
	// and dropped by a select: no branch in the element code)
	unsigned long long sum_a = 0, sum_b = 0;
	walk(false, [&](int stage, int blk) {
		int acc[4][4];
		scores(stage, acc);
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const int k0 = blk * kTileKeys + 32 * ph + 8 * j + 2 * c;
#pragma unroll
			for (int q = 0; q < 2; ++q) {
				uint32_t parts;
				const int64_t ea = iexp_fast((uint32_t)mx_a - (uint32_t)acc[j][q], fa, &parts);
				const int64_t eb = iexp_fast((uint32_t)mx_b - (uint32_t)acc[j][2 + q], fb, &parts);
				sum_a += k0 + q <= lim_a ? (unsigned long long)ea : 0ull;
				sum_b += k0 + q <= lim_b ? (unsigned long long)eb : 0ull;
			}
		}
	});
	sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
	sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
	sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
	sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
	if (c == 0) {
		wsum[ph * kTileRows + rho_a] = sum_a;
		wsum[ph * kTileRows + rho_b] = sum_b;
	}
	__syncthreads();
	sum_a = wsum[rho_a] + wsum[kTileRows + rho_a];
	sum_b = wsum[rho_b] + wsum[kTileRows + rho_b];
	const unsigned long long tot_a = sum_a > 1ull ? sum_a : 1ull, tot_b = sum_b > 1ull ? sum_b : 1ull;
	const float inv_a = 32768.0f / (float)tot_a, inv_b = 32768.0f / (float)tot_b;
	const bool go_a = in_a, go_b = in_b;

	// ---- walk 3: probabilities and P.V
	int accl[NGW][4], acch[NGW][4];
#pragma unroll
	for (int i = 0; i < NGW; ++i)
#pragma unroll
		for (int q = 0; q < 4; ++q) accl[i][q] = acch[i][q] = 0;
	walk(true, [&](int stage, int blk) {
		int acc[4][4];
		scores(stage, acc);
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const int col = 32 * ph + 8 * j + 2 * c;
			const int k0 = blk * kTileKeys + col;
			uint32_t pa[2], pb[2];
#pragma unroll
			for (int q = 0; q < 2; ++q) {
				uint32_t parts;
				const uint32_t va = prob_q15(iexp_fast((uint32_t)mx_a - (uint32_t)acc[j][q], fa, &parts), tot_a, inv_a);
				const uint32_t vb = prob_q15(iexp_fast((uint32_t)mx_b - (uint32_t)acc[j][2 + q], fb, &parts), tot_b, inv_b);
				pa[q] = k0 + q <= lim_a ? va : 0u;
				pb[q] = k0 + q <= lim_b ? vb : 0u;
			}
			*(uint16_t*)(Pl + (size_t)rho_a * kTilePStride + col) = (uint16_t)((pa[0] & 0xffu) | ((pa[1] & 0xffu) << 8));
			*(uint16_t*)(Ph + (size_t)rho_a * kTilePStride + col) = (uint16_t)((pa[0] >> 8) | ((pa[1] >> 8) << 8));
			*(uint16_t*)(Pl + (size_t)rho_b * kTilePStride + col) = (uint16_t)((pb[0] & 0xffu) | ((pb[1] & 0xffu) << 8));
			*(uint16_t*)(Ph + (size_t)rho_b * kTilePStride + col) = (uint16_t)((pb[0] >> 8) | ((pb[1] >> 8) << 8));
		}
		// the two warps of an MMA block wrote its rows' 64 probabilities between them
		asm volatile("bar.sync %0, 64;" ::"r"(1 + mb) : "memory");
		const int8_t* vd = Vs + (size_t)stage * kTileKeys * HD;
#pragma unroll
		for (int ks = 0; ks < 2; ++ks) {
			const uint8_t* la = Pl + (size_t)rho_a * kTilePStride + 32 * ks + 4 * c;
			const uint8_t* lb = Pl + (size_t)rho_b * kTilePStride + 32 * ks + 4 * c;
			const uint8_t* ha = Ph + (size_t)rho_a * kTilePStride + 32 * ks + 4 * c;
			const uint8_t* hb = Ph + (size_t)rho_b * kTilePStride + 32 * ks + 4 * c;
			const uint32_t l0 = *(const uint32_t*)la, l1 = *(const uint32_t*)lb, l2 = *(const uint32_t*)(la + 16), l3 = *(const uint32_t*)(lb + 16);
			const uint32_t h0 = *(const uint32_t*)ha, h1 = *(const uint32_t*)hb, h2 = *(const uint32_t*)(ha + 16), h3 = *(const uint32_t*)(hb + 16);
#pragma unroll
			for (int i = 0; i < NGW; ++i) {
				const int ch = 8 * (ph * NGW + i) + g;
				const uint32_t b0 = *(const uint32_t*)(vd + (size_t)(2 * ks) * HD * kPageTokens + ch * kPageTokens + 4 * c);
				const uint32_t b1 = *(const uint32_t*)(vd + (size_t)(2 * ks + 1) * HD * kPageTokens + ch * kPageTokens + 4 * c);
				mma_u8s8_full(accl[i], l0, l1, l2, l3, b0, b1);
				mma_u8s8_full(acch[i], h0, h1, h2, h3, b0, b1);
			}
		}
	});

	// ---- per-head context fold (forward_sites.cpp:1889-1896), store, row maximum for the funnel
	uint32_t lm_a = 0, lm_b = 0;
#pragma unroll
	for (int i = 0; i < NGW; ++i) {
		const int ch = 8 * (ph * NGW + i) + 2 * c;
		if (go_a) {
			int2 o;
			o.x = fold(accl[i][0] + 256 * acch[i][0], l_fold[3 * head_a], l_fold[3 * head_a + 1], l_fold[3 * head_a + 2]);
			o.y = fold(accl[i][1] + 256 * acch[i][1], l_fold[3 * head_a], l_fold[3 * head_a + 1], l_fold[3 * head_a + 2]);
			*(int2*)(b.ctxw + (size_t)(r0 + tok_a) * d.hidden + (size_t)(kvh * G + head_a) * HD + ch) = o;
			lm_a = max(lm_a, max(o.x < 0 ? 0u - (uint32_t)o.x : (uint32_t)o.x, o.y < 0 ? 0u - (uint32_t)o.y : (uint32_t)o.y));
		}
		if (go_b) {
			int2 o;
			o.x = fold(accl[i][2] + 256 * acch[i][2], l_fold[3 * head_b], l_fold[3 * head_b + 1], l_fold[3 * head_b + 2]);
			o.y = fold(accl[i][3] + 256 * acch[i][3], l_fold[3 * head_b], l_fold[3 * head_b + 1], l_fold[3 * head_b + 2]);
			*(int2*)(b.ctxw + (size_t)(r0 + tok_b) * d.hidden + (size_t)(kvh * G + head_b) * HD + ch) = o;
			lm_b = max(lm_b, max(o.x < 0 ? 0u - (uint32_t)o.x : (uint32_t)o.x, o.y < 0 ? 0u - (uint32_t)o.y : (uint32_t)o.y));
		}
	}
	lm_a = max(lm_a, __shfl_xor_sync(0xffffffffu, lm_a, 1));
	lm_a = max(lm_a, __shfl_xor_sync(0xffffffffu, lm_a, 2));
	lm_b = max(lm_b, __shfl_xor_sync(0xffffffffu, lm_b, 1));
	lm_b = max(lm_b, __shfl_xor_sync(0xffffffffu, lm_b, 2));
	if (c == 0) {
		if (go_a && lm_a) atomicMax(&b.rowmax[(size_t)(r0 + tok_a) * 4 + 3], (unsigned long long)lm_a);
		if (go_b && lm_b) atomicMax(&b.rowmax[(size_t)(r0 + tok_b) * 4 + 3], (unsigned long long)lm_b);
	}
}

template <int HD>
static cudaError_t launch_attn_tile(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index, KvPoolDev pool,
                                    cudaStream_t st) {
	const int G = d.heads / d.kv_heads;
	const int tq = kTileRows / G;
	return launch_pdl(k_attention_tile<HD>, dim3(d.kv_heads, (b.m + tq - 1) / tq), dim3(kTileThreads), TileSmem<HD>::kBytes, st, b,
	                  d, layer, layer_index, pool, tq);
}

static int pad64(int w) { return (w + 63) / 64 * 64; }
constexpr int kAttnMaxSlice = 2048;      // positions one block holds at most

struct AttnPlan {
	int splits;       // slices along the width
	int whole_row;    // the cluster spans every kv head of the row (the funnel is fused)
	int cp;           // positions per block (shared-memory capacity)
};
// How a launch over `m` rows of up to `max_width` positions is cut. A cluster has at most 8
// blocks (the portable size), 16 only when a row is too wide for 8 slices; a row's funnel is
// fused when all its kv heads fit into the cluster beside the slices.
static std::atomic<int> g_forced_splits{-1};     // -1: not set yet (the environment decides), 0: automatic
void attn_force_splits(int splits) { g_forced_splits.store(splits < 0 ? 0 : splits); }

static AttnPlan attn_plan(const Dims& d, int m, int max_width, bool one_sequence) {
	AttnPlan p;
	int forced = g_forced_splits.load();
	if (forced < 0) {      // SSLM_B200_ATTN_SPLITS=n fixes the slices per kv head (tuning, tests)
		const char* e = getenv("SSLM_B200_ATTN_SPLITS");
		forced = e ? atoi(e) : 0;
		g_forced_splits.store(forced < 0 ? 0 : forced);
	}
	const int per_kv_max = d.kv_heads <= 8 ? 8 / d.kv_heads : 1;   // slices per kv head with the whole row in one cluster
	int splits = 1;
	if (forced > 0) {
		while (splits * 2 <= forced && splits * 2 <= 16) splits *= 2;
	} else {
		// A block's time is mostly a fixed chain of dependent steps, and blocks of a cluster wait
		// for one another at every exchange, so cutting rows into slices pays only when the rows
		// are so few that most multiprocessors would otherwise idle (a single long sequence): then
		// the width is cut until the blocks fill a fifth of the machine. Otherwise a row is one
		// slice per kv head, unclustered, and the funnel kernel follows.
		const int blocks = m * d.kv_heads;
		int want = 1;
		while (want < 8 && blocks * want * 2 <= sm_count() / 5) want *= 2;
		while (splits * 2 <= want && splits * 2 <= 8) splits *= 2;
		if (splits > per_kv_max) splits = per_kv_max;              // prefer the fused funnel ...
	}
	while (splits > 1 && splits * 64 > pad64(max_width)) splits /= 2;
	// ... unless the width does not fit the slices: then up to 16 slices of one kv head per cluster
	while (splits < 16 && pad64((max_width + splits - 1) / splits) > kAttnMaxSlice) splits *= 2;
	p.whole_row = splits <= per_kv_max ? 1 : 0;
	// The rows of a prefill chunk are many and of very different widths: blocks that wait for one
	// another at cluster barriers cost more there than the separate funnel kernel does.
	if (forced <= 0 && splits == 1) p.whole_row = 0;
	p.splits = splits;
	p.cp = pad64((max_width + splits - 1) / splits);
	return p;
}

template <int HD>
static cudaError_t launch_attn(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index, KvPoolDev pool,
                               const AttnPlan& p, int reverse_rows, cudaStream_t st) {
	const size_t sm = attn_smem_bytes(d.heads / d.kv_heads, p.cp, HD);
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3(d.kv_heads * p.splits, b.m);
	cfg.blockDim = dim3(2 * HD);
	cfg.dynamicSmemBytes = sm;
	cfg.stream = st;
	cudaLaunchAttribute attr[2];
	attr[0].id = cudaLaunchAttributeClusterDimension;
	attr[0].val.clusterDim.x = (unsigned)(p.whole_row ? d.kv_heads * p.splits : p.splits);
	attr[0].val.clusterDim.y = 1;
	attr[0].val.clusterDim.z = 1;
	attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[1].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = attr;
	cfg.numAttrs = pdl_enabled() ? 2 : 1;
	return cudaLaunchKernelEx(&cfg, k_attention<HD>, b, d, layer, layer_index, pool, p.cp, p.splits, p.whole_row, reverse_rows);
}

cudaError_t attn_configure(const Dims& d) {
	const int group = d.heads / d.kv_heads;
	if (group < 1 || group > 8 || d.heads % d.kv_heads != 0) return cudaErrorInvalidConfiguration;
	// widest row the plan can serve: 16 slices of kAttnMaxSlice positions
	if (d.context_cap > 16 * kAttnMaxSlice) return cudaErrorInvalidConfiguration;
	const size_t need = attn_smem_bytes(group, kAttnMaxSlice, d.head_dim);
	if (need > 227 * 1024) return cudaErrorInvalidConfiguration;
	const int n = (int)need;
	const void* f = nullptr;
	if (d.head_dim == 128) f = (const void*)k_attention<128>;
	else if (d.head_dim == 64) f = (const void*)k_attention<64>;
	else if (d.head_dim == 32) f = (const void*)k_attention<32>;
	else return cudaErrorInvalidConfiguration;
	cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, n);
	if (e != cudaSuccess) return e;
	// clusters of 16 blocks (rows wider than 8 slices) are an opt-in size
	e = cudaFuncSetAttribute(f, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
	if (e != cudaSuccess) return e;
	// same carve-out as the kernels around it (see rows_configure)
	e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
	if (e != cudaSuccess) return e;
	const void* ft = nullptr;
	size_t tile_bytes = 0;
	if (d.head_dim == 128) { ft = (const void*)k_attention_tile<128>; tile_bytes = TileSmem<128>::kBytes; }
	else if (d.head_dim == 64) { ft = (const void*)k_attention_tile<64>; tile_bytes = TileSmem<64>::kBytes; }
	else { ft = (const void*)k_attention_tile<32>; tile_bytes = TileSmem<32>::kBytes; }
	e = cudaFuncSetAttribute(ft, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_bytes);
	if (e != cudaSuccess) return e;
	return cudaFuncSetAttribute(ft, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

bool launch_attention(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index,
                      KvPoolDev pool, int max_width, int reverse_rows, cudaStream_t st, cudaError_t* err) {
	// the rows of a prefill chunk (consecutive positions of one sequence) take the query-tiled kernel
	static const bool tile_off = [] {
		const char* e = getenv("SSLM_B200_ATTN_TILE");
		return e && e[0] == '0';
	}();
	// ... once their prefix is long: up to about a thousand positions the per-row kernel, with
	// thousands of independent blocks, is as fast or faster; beyond that re-reading the prefix per
	// token costs more than the tiled kernel's lower parallelism (measured on the 0.5B / 1.5B / 3B widths).
	static const int tile_min = [] {
		const char* e = getenv("SSLM_B200_ATTN_TILE_MIN");      // tuning: the width from which the tiled kernel runs
		return e ? atoi(e) : 1536;
	}();
	if (reverse_rows && b.m >= 4 && max_width >= tile_min && !tile_off) {
		cudaError_t e;
		if (d.head_dim == 128) e = launch_attn_tile<128>(b, d, layer, layer_index, pool, st);
		else if (d.head_dim == 64) e = launch_attn_tile<64>(b, d, layer, layer_index, pool, st);
		else e = launch_attn_tile<32>(b, d, layer, layer_index, pool, st);
		if (err) *err = e;
		return false;
	}
	const AttnPlan p = attn_plan(d, b.m, max_width, reverse_rows != 0);
	cudaError_t e;
	if (d.head_dim == 128) e = launch_attn<128>(b, d, layer, layer_index, pool, p, reverse_rows, st);
	else if (d.head_dim == 64) e = launch_attn<64>(b, d, layer, layer_index, pool, p, reverse_rows, st);
	else e = launch_attn<32>(b, d, layer, layer_index, pool, p, reverse_rows, st);
	if (err) *err = e;
	return p.whole_row != 0;
}

// ------------------------------------------------------------ primitive sweep (tests)
// The integer primitives of the device library evaluated on arrays of operands ON THE DEVICE, so
// that their device-only halves (rcp.approx / rsqrt.approx estimates, 32-bit short forms) are
// compared with the CPU oracle too. Operand meaning per `which`: see sslm_b200_int_sweep.
__global__ void k_int_sweep(int which, const int64_t* a, const int64_t* b, const int64_t* c, const int64_t* e, long long n,
                            int64_t* out0, int64_t* out1, int64_t* out2) {
	for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
		int64_t o0 = 0, o1 = 0, o2 = 0;
		switch (which) {
		case 0: o0 = dyn_recip(a[i]); break;
		case 1: o0 = isqrt64(a[i]); break;
		case 2: o0 = floor_div_h32((int)a[i], b[i], rcp_estimate((double)b[i])); break;
		case 3: {
			o0 = requant_code(a[i], b[i], (int)c[i]);
			const Coder cd = make_coder(b[i], (int)c[i]);       // the per-row coder the kernels use must agree
			o1 = code_of(a[i], cd);
			o2 = fits_i32(a[i]) ? code_of((int32_t)a[i], cd) : o1;
			break;
		}
		case 4: {
			bool sat = false, ex = false;
			o0 = landing_rescale(a[i], b[i], c[i], e[i] >> 32, (int64_t)(int32_t)(uint32_t)e[i], &sat, &ex);
			o1 = (sat ? 1 : 0) | (ex ? 2 : 0);
			break;
		}
		case 5: o0 = (int64_t)udiv_small_quotient((uint64_t)a[i], (uint64_t)b[i], rcp_estimate((double)b[i])); break;
		case 6: {
			const Scale inc{b[i], c[i]}, site{e[i] >> 32, (int64_t)(int32_t)(uint32_t)e[i]};
			const FunnelParams fp = funnel_params((uint64_t)a[i], &inc, 1, site);
			o0 = fp.out.m;
			o1 = fp.out.e;
			o2 = fp.status;
			break;
		}
		case 7: {      // one softmax element on the attention kernels' 32-bit form; peak in the low half of e
			SoftmaxConsts k;
			k.c = IExpConsts{b[i], c[i], e[i] >> 32};
			k.peak = (int64_t)(uint32_t)e[i] << 16;
			const IExpFast f = iexp_fast_prepare(k);
			uint32_t parts = 0;
			const int64_t v = iexp_fast((uint32_t)a[i], f, &parts);
			o0 = v;
			o1 = (v < 0 || v > k.peak) ? 1 : 0;       // the reference's per-element bound
			o2 = iexp_from_parts(parts, f);
			break;
		}
		case 8: {      // Q15 probability: floor((e << 15) / total), 0 <= e <= total
			const unsigned long long tot = (unsigned long long)b[i];
			o0 = prob_q15(a[i], tot, 32768.0f / (float)tot);
			break;
		}
		default: break;
		}
		out0[i] = o0;
		out1[i] = o1;
		out2[i] = o2;
	}
}
void launch_int_sweep(int which, const int64_t* a, const int64_t* b, const int64_t* c, const int64_t* e, long long n, int64_t* out0,
                      int64_t* out1, int64_t* out2, cudaStream_t st) {
	k_int_sweep<<<592, 256, 0, st>>>(which, a, b, c, e, n, out0, out1, out2);
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
