// Integer i-exp softmax attention over the paged int8 KV pool, staged through shared
// memory. One thread block owns one (row, kv head); inside it ONE WARP owns one q head of
// the GQA group, so the heads of a group run side by side with no block-level barrier and
// each K / V byte of the sequence is fetched from HBM once per kv head (the other warps of
// the block hit it in L1/L2).
//
// Per warp (q head):
//   pass 1  scores[k] = q_rot . K[k]   coalesced 16-byte K loads, dp4a, 3 shuffles per row
//   pass 2  max, then total = sum_k e_k (e_k: second-order integer exp, SoftmaxRowQ15)
//   pass 3  p_k = (e_k << 15) / total  exact division, stored over the score
//   pass 4  ctx[d] = sum_k p_k V[k][d]  coalesced V loads, then the per-head fold and row max
//
// Every reduction is an integer max or add, so the result does not depend on the order in
// which lanes, warps or blocks contribute. Restates the attention block of RunLayerLoopImpl
// (src/forward/forward_sites.cpp:1858-1897), SoftmaxRowQ15 (src/intmath.cpp:796-901) and
// GemmProbQ15Accumulate (src/matmul.cpp:522-538).
#include <cuda_runtime.h>

#include "sslm_kernels.h"

namespace sslm {

__device__ __forceinline__ const int8_t* kv_row_ptr(const int8_t* plane, const int32_t* pages, int pos,
                                                    int hd) {
	return plane + ((int64_t)pages[pos / kPageTokens] * kPageTokens + (pos % kPageTokens)) * hd;
}

__device__ __forceinline__ int dot16(const int4& a, const int4& b) {
	int acc = __dp4a(a.x, b.x, 0);
	acc = __dp4a(a.y, b.y, acc);
	acc = __dp4a(a.z, b.z, acc);
	return __dp4a(a.w, b.w, acc);
}

// HD = head_dim (32, 64 or 128)
template <int HD>
__global__ void __launch_bounds__(256)
k_attention(RowBatch b, Dims d, const LayerDev* layer, int layer_index, KvPoolDev pool, int width_pad) {
	extern __shared__ __align__(16) unsigned char smem[];
	const int r = blockIdx.y, kvh = blockIdx.x;
	if (b.status[r] != 0) return;
	const int group = d.heads / d.kv_heads;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int head = kvh * group + warp;               // one warp per q head
	const int width = b.rows[r].pos + 1;
	int32_t* sc = (int32_t*)smem + (size_t)warp * width_pad;   // this warp's scores / probabilities

	const int32_t* pages = b.rows[r].pages;
	const int8_t* kplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 0);
	const int8_t* vplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 1);
	const int8_t* q = b.qrot + (size_t)r * d.hidden + (size_t)head * HD;

	// ---- pass 1: scores. SL lanes share one K row (16 bytes each), RPI rows per load.
	constexpr int SL = HD / 16, RPI = 32 / SL;
	const int sl = lane % SL, sub = lane / SL;
	const int4 qv = *((const int4*)q + sl);
	int mx = INT32_MIN;
	constexpr int U1 = 4;
	for (int k0 = 0; k0 < width; k0 += RPI * U1) {
		int4 kvv[U1];
#pragma unroll
		for (int u = 0; u < U1; ++u) {
			const int k = k0 + u * RPI + sub;
			kvv[u] = make_int4(0, 0, 0, 0);
			if (k < width) kvv[u] = __ldg((const int4*)kv_row_ptr(kplane, pages, k, HD) + sl);
		}
#pragma unroll
		for (int u = 0; u < U1; ++u) {
			int s = dot16(kvv[u], qv);
#pragma unroll
			for (int o = SL / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
			const int k = k0 + u * RPI + sub;
			if (k < width) {
				if (sl == 0) sc[k] = s;
				mx = max(mx, s);
			}
		}
	}
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
	__syncwarp();

	// ---- pass 2: total of the integer exponentials
	const SoftmaxConsts smc = b.smc[(size_t)r * d.kv_heads + kvh];
	unsigned long long tot = 0;
	bool bad = false;
	for (int k = lane; k < width; k += 32) {
		int64_t e;
		if (iexp_element((int64_t)sc[k] - mx, smc.c, smc.peak, &e)) tot += (unsigned long long)e;
		else bad = true;
	}
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
	if (__any_sync(0xffffffffu, bad)) {
		// the reference refuses the row (SoftmaxKernelRefusedAfterGateAccepted)
		if (lane == 0) atomicCAS(&b.status[r], 0, kSoftmaxKernelRefused);
		return;
	}
	// ---- pass 3: Q15 probabilities in place of the scores
	const unsigned long long den = tot > 1ull ? tot : 1ull;
	const double inv = 1.0 / (double)den;
	for (int k = lane; k < width; k += 32) {
		int64_t e;
		iexp_element((int64_t)sc[k] - mx, smc.c, smc.peak, &e);
		sc[k] = (int32_t)udiv_small_quotient((uint64_t)e << 15, den, inv);
	}
	__syncwarp();

	// ---- pass 4: ctx = P V. DL lanes share one V row (4 head-dim elements each).
	constexpr int DL = HD / 4, RPV = 32 / DL;
	const int dl = lane % DL, vsub = lane / DL;
	int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
	constexpr int U4 = 8;
	for (int k0 = 0; k0 < width; k0 += RPV * U4) {
		int vv[U4], pp[U4];
#pragma unroll
		for (int u = 0; u < U4; ++u) {
			const int k = k0 + u * RPV + vsub;
			vv[u] = 0;
			pp[u] = 0;
			if (k < width) {
				vv[u] = __ldg((const int*)kv_row_ptr(vplane, pages, k, HD) + dl);
				pp[u] = sc[k];
			}
		}
#pragma unroll
		for (int u = 0; u < U4; ++u) {
			const int x = vv[u], p = pp[u];
			c0 += p * (int)(int8_t)(x & 0xff);
			c1 += p * (int)(int8_t)((x >> 8) & 0xff);
			c2 += p * (int)(int8_t)((x >> 16) & 0xff);
			c3 += p * (x >> 24);
		}
	}
#pragma unroll
	for (int o = 16; o >= DL; o >>= 1) {
		c0 += __shfl_xor_sync(0xffffffffu, c0, o);
		c1 += __shfl_xor_sync(0xffffffffu, c1, o);
		c2 += __shfl_xor_sync(0xffffffffu, c2, o);
		c3 += __shfl_xor_sync(0xffffffffu, c3, o);
	}
	// per-head context fold (forward_sites.cpp:1889-1896), store, row max for the funnel
	const int32_t fi = layer->f_ctx[3 * head], fm = layer->f_ctx[3 * head + 1], fs = layer->f_ctx[3 * head + 2];
	uint32_t lmax = 0;
	if (vsub == 0) {
		int4 o4;
		o4.x = fold(c0, fi, fm, fs);
		o4.y = fold(c1, fi, fm, fs);
		o4.z = fold(c2, fi, fm, fs);
		o4.w = fold(c3, fi, fm, fs);
		*((int4*)(b.ctxw + (size_t)r * d.hidden + (size_t)head * HD) + dl) = o4;
		const int vals[4] = {o4.x, o4.y, o4.z, o4.w};
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const uint32_t ab = vals[j] < 0 ? 0u - (uint32_t)vals[j] : (uint32_t)vals[j];
			lmax = ab > lmax ? ab : lmax;
		}
	}
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) lmax = max(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
	if (lane == 0 && lmax) atomicMax(&b.rowmax[(size_t)r * 4 + 3], (unsigned long long)lmax);
}

static int pad_width(int w) { return (w + 31) / 32 * 32 + 4; }
static size_t attn_smem(const Dims& d, int width_pad) {
	return (size_t)(d.heads / d.kv_heads) * width_pad * 4;
}

cudaError_t attn_configure(const Dims& d) {
	const size_t need = attn_smem(d, pad_width(d.context_cap));
	if (need > 227 * 1024 || d.heads / d.kv_heads > 8) return cudaErrorInvalidConfiguration;
	const int n = (int)need;
	if (d.head_dim == 128) return cudaFuncSetAttribute(k_attention<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, n);
	if (d.head_dim == 64) return cudaFuncSetAttribute(k_attention<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, n);
	if (d.head_dim == 32) return cudaFuncSetAttribute(k_attention<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, n);
	return cudaErrorInvalidConfiguration;
}

void launch_attention(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index,
                      KvPoolDev pool, int max_width, cudaStream_t st) {
	const int wp = pad_width(max_width);
	const dim3 grid(d.kv_heads, b.m);
	const int threads = 32 * (d.heads / d.kv_heads);
	const size_t sm = attn_smem(d, wp);
	if (d.head_dim == 128) k_attention<128><<<grid, threads, sm, st>>>(b, d, layer, layer_index, pool, wp);
	else if (d.head_dim == 64) k_attention<64><<<grid, threads, sm, st>>>(b, d, layer, layer_index, pool, wp);
	else k_attention<32><<<grid, threads, sm, st>>>(b, d, layer, layer_index, pool, wp);
}

// ------------------------------------------------------------ canonical KV export
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
			const int8_t* src = pool.base + kv_plane_offset(d, pool, layer, kvh, is_v);
			val = *((const int4*)kv_row_ptr(src, pages, pos, hd) + v);
		}
		((int4*)out)[i] = val;
	}
}

void launch_kv_export(const Dims& d, KvPoolDev pool, const int32_t* pages, int context_length,
                      int layer_index, int8_t* out, cudaStream_t st) {
	k_kv_export<<<148 * 4, 256, 0, st>>>(d, pool, pages, context_length, layer_index, out);
}

}  // namespace sslm
