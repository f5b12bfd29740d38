// Integer i-exp softmax attention over the paged int8 KV pool, staged through shared
// memory. One thread block owns one (row, kv head): it serves every q head of the GQA
// group, so each K and V byte of the sequence is read once per kv head.
//
//   pass 1  scores[g][k] = q_rot[g] . K[k]          (dp4a, K rows streamed page by page)
//   pass 2  per head: max, then total = sum_k e_k    (e_k: second-order integer exp)
//   pass 3  p_k = (e_k << 15) / total                (exact division, kept in place of the score)
//   pass 4  ctx[g][d] = sum_k p_k V[k][d]            (V streamed once), per-head fold, row max
//
// Every reduction is an integer max or add, so the result does not depend on the order
// in which threads or blocks contribute. Restates the attention block of RunLayerLoopImpl
// (src/forward/forward_sites.cpp:1858-1897), SoftmaxRowQ15 (src/intmath.cpp:796-901) and
// GemmProbQ15Accumulate (src/matmul.cpp:522-538).
#include <cuda_runtime.h>

#include "sslm_kernels.h"

namespace sslm {

constexpr int kAttnThreads = 256;

__device__ __forceinline__ const int8_t* kv_row_ptr(const int8_t* plane, const int32_t* pages, int pos,
                                                    int hd) {
	return plane + ((int64_t)pages[pos / kPageTokens] * kPageTokens + (pos % kPageTokens)) * hd;
}

__global__ void __launch_bounds__(kAttnThreads)
k_attention(RowBatch b, Dims d, const LayerDev* layer, int layer_index, KvPoolDev pool, int width_pad) {
	extern __shared__ __align__(16) unsigned char smem[];
	const int r = blockIdx.y, kvh = blockIdx.x;
	if (b.status[r] != 0) return;
	const int hd = d.head_dim, group = d.heads / d.kv_heads;
	const int width = b.rows[r].pos + 1;
	// shared layout
	int8_t* sq = (int8_t*)smem;                                    // [group][hd]
	int* smaxv = (int*)(smem + group * hd);                        // [group]
	unsigned long long* stot = (unsigned long long*)(smaxv + 8);   // [group]
	int* sbad = (int*)(stot + 8);                                  // [1] (+pad)
	int32_t* sc = (int32_t*)(sbad + 4);                            // [group][width_pad]
	int32_t* sred = sc + (size_t)group * width_pad;                // [8 warps][group][hd] partial ctx

	const int32_t* pages = b.rows[r].pages;
	const int8_t* kplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 0);
	const int8_t* vplane = pool.base + kv_plane_offset(d, pool, layer_index, kvh, 1);
	const int8_t* qg = b.qrot + (size_t)r * d.hidden + (size_t)kvh * group * hd;
	for (int i = threadIdx.x; i < group * hd / 4; i += blockDim.x) ((int*)sq)[i] = ((const int*)qg)[i];
	if (threadIdx.x < group) {
		smaxv[threadIdx.x] = INT32_MIN;
		stot[threadIdx.x] = 0ull;
	}
	if (threadIdx.x == 0) sbad[0] = 0;
	__syncthreads();

	// pass 1: scores
	const int vec = hd / 16;
	for (int k = threadIdx.x; k < width; k += blockDim.x) {
		const int4* krow = (const int4*)kv_row_ptr(kplane, pages, k, hd);
		int acc[8];
#pragma unroll
		for (int g = 0; g < 8; ++g) acc[g] = 0;
		for (int v = 0; v < vec; ++v) {
			const int4 kvv = __ldg(krow + v);
#pragma unroll
			for (int g = 0; g < 8; ++g) {
				if (g < group) {
					const int4 qv = ((const int4*)(sq + g * hd))[v];
					acc[g] = __dp4a(kvv.x, qv.x, acc[g]);
					acc[g] = __dp4a(kvv.y, qv.y, acc[g]);
					acc[g] = __dp4a(kvv.z, qv.z, acc[g]);
					acc[g] = __dp4a(kvv.w, qv.w, acc[g]);
				}
			}
		}
#pragma unroll
		for (int g = 0; g < 8; ++g)
			if (g < group) sc[(size_t)g * width_pad + k] = acc[g];
	}
	__syncthreads();

	// pass 2a: per-head max
	const int lane = threadIdx.x & 31;
	for (int g = 0; g < group; ++g) {
		int mx = INT32_MIN;
		for (int k = threadIdx.x; k < width; k += blockDim.x) mx = max(mx, sc[(size_t)g * width_pad + k]);
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
		if (lane == 0) atomicMax(&smaxv[g], mx);
	}
	__syncthreads();
	const SoftmaxConsts smc = b.smc[(size_t)r * d.kv_heads + kvh];
	// pass 2b: total of the integer exponentials
	int bad = 0;
	for (int g = 0; g < group; ++g) {
		const int peak = smaxv[g];
		unsigned long long tot = 0;
		for (int k = threadIdx.x; k < width; k += blockDim.x) {
			int64_t e;
			if (iexp_element((int64_t)sc[(size_t)g * width_pad + k] - peak, smc.c, smc.peak, &e)) tot += (unsigned long long)e;
			else bad = 1;
		}
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
		if (lane == 0 && tot) atomicAdd(&stot[g], tot);
	}
	if (bad) sbad[0] = 1;
	__syncthreads();
	if (sbad[0]) {
		if (threadIdx.x == 0) atomicCAS(&b.status[r], 0, kSoftmaxKernelRefused);
		return;
	}
	// pass 3: Q15 probabilities in place of the scores
	for (int g = 0; g < group; ++g) {
		const int peak = smaxv[g];
		const unsigned long long den = stot[g] > 1ull ? stot[g] : 1ull;
		const double inv = 1.0 / (double)den;
		for (int k = threadIdx.x; k < width; k += blockDim.x) {
			int64_t e;
			iexp_element((int64_t)sc[(size_t)g * width_pad + k] - peak, smc.c, smc.peak, &e);
			sc[(size_t)g * width_pad + k] = (int32_t)udiv_small_quotient((uint64_t)e << 15, den, inv);
		}
	}
	__syncthreads();

	// pass 4: ctx = P V. A warp step covers rows_per_step positions; each lane owns 8
	// consecutive head-dim elements of one of them. Four steps are issued back to back so
	// that every lane keeps four independent 8-byte V loads in flight.
	const int lanes_per_row = hd / 8, rows_per_step = 32 / lanes_per_row;
	const int warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
	const int sub = lane / lanes_per_row, dq = lane % lanes_per_row;
	constexpr int kUnroll = 4;
	int cacc[8][8];
#pragma unroll
	for (int g = 0; g < 8; ++g)
#pragma unroll
		for (int j = 0; j < 8; ++j) cacc[g][j] = 0;
	for (int k0 = warp * rows_per_step * kUnroll; k0 < width; k0 += nw * rows_per_step * kUnroll) {
		int2 vv[kUnroll];
#pragma unroll
		for (int u = 0; u < kUnroll; ++u) {
			const int k = k0 + u * rows_per_step + sub;
			vv[u] = make_int2(0, 0);
			if (k < width) vv[u] = __ldg((const int2*)kv_row_ptr(vplane, pages, k, hd) + dq);
		}
#pragma unroll
		for (int u = 0; u < kUnroll; ++u) {
			const int k = k0 + u * rows_per_step + sub;
			if (k >= width) continue;
			int v[8];
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				v[j] = (int8_t)((vv[u].x >> (8 * j)) & 0xff);
				v[4 + j] = (int8_t)((vv[u].y >> (8 * j)) & 0xff);
			}
#pragma unroll
			for (int g = 0; g < 8; ++g) {
				if (g < group) {
					const int p = sc[(size_t)g * width_pad + k];
#pragma unroll
					for (int j = 0; j < 8; ++j) cacc[g][j] += p * v[j];
				}
			}
		}
	}
	// fold the `sub` position lanes of a warp together, then the warps through shared memory
#pragma unroll
	for (int g = 0; g < 8; ++g)
#pragma unroll
		for (int j = 0; j < 8; ++j) {
			int v = cacc[g][j];
			for (int o = 16; o >= lanes_per_row; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
			cacc[g][j] = v;
		}
	if (sub == 0) {
#pragma unroll
		for (int g = 0; g < 8; ++g)
			if (g < group)
#pragma unroll
				for (int j = 0; j < 8; ++j) sred[((size_t)warp * group + g) * hd + dq * 8 + j] = cacc[g][j];
	}
	__syncthreads();
	unsigned long long lmax = 0;
	for (int i = threadIdx.x; i < group * hd; i += blockDim.x) {
		int v = 0;
		for (int w = 0; w < nw; ++w) v += sred[(size_t)w * group * hd + i];
		const int g = i / hd, head = kvh * group + g;
		const int32_t f = fold(v, layer->f_ctx[3 * head], layer->f_ctx[3 * head + 1], layer->f_ctx[3 * head + 2]);
		b.ctxw[(size_t)r * d.hidden + (size_t)head * hd + (i - g * hd)] = f;
		const unsigned long long ab = f < 0 ? (unsigned long long)(-(int64_t)f) : (unsigned long long)f;
		lmax = ab > lmax ? ab : lmax;
	}
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) {
		const unsigned long long t = __shfl_xor_sync(0xffffffffu, lmax, o);
		lmax = t > lmax ? t : lmax;
	}
	if (lane == 0 && lmax) atomicMax(&b.rowmax[(size_t)r * 4 + 3], lmax);
}

static size_t attn_smem(const Dims& d, int width_pad) {
	const int group = d.heads / d.kv_heads;
	return (size_t)group * d.head_dim + 8 * 4 + 8 * 8 + 16 + (size_t)group * width_pad * 4 +
	       (size_t)(kAttnThreads / 32) * group * d.head_dim * 4;
}
static int pad_width(int w) { return (w + 31) / 32 * 32 + 4; }

cudaError_t attn_configure(const Dims& d) {
	const size_t need = attn_smem(d, pad_width(d.context_cap));
	if (need > 227 * 1024) return cudaErrorInvalidConfiguration;
	return cudaFuncSetAttribute(k_attention, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
}

void launch_attention(const RowBatch& b, const Dims& d, const LayerDev* layer, int layer_index,
                      KvPoolDev pool, int max_width, cudaStream_t st) {
	const int wp = pad_width(max_width);
	k_attention<<<dim3(d.kv_heads, b.m), kAttnThreads, attn_smem(d, wp), st>>>(b, d, layer, layer_index,
	                                                                           pool, wp);
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
