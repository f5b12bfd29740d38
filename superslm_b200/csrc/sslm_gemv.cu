// Decode-path int8 linear layer: out[m,n] = fold_n(sum_k x[m,k] w[n,k]) for a handful of
// rows m. HBM-bound: the weights are streamed exactly once with 16-byte coalesced loads,
// multiplied with dp4a against the activation rows held in shared memory, and reduced
// with warp shuffles. The epilogue applies the per-channel weight-scale fold, adds the
// LoRA delta, stores the wide row and reduces the per-row max |x| the funnel needs.
// (GemmInt8AccumulateRow + ApplyWeightScaleFold + AddAmplifyingLoraDelta,
//  src/matmul.cpp:455-464, src/forward/forward_sites.cpp:461-470, :1051-1103.)
// int32 accumulation is exact: K * 127 * 128 < 2^31 for every K the loader accepts.
#include <cuda_runtime.h>

#include "sslm_kernels.h"

namespace sslm {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

__device__ __forceinline__ int dot16(const int4& a, const int4& b, int acc) {
	acc = __dp4a(a.x, b.x, acc);
	acc = __dp4a(a.y, b.y, acc);
	acc = __dp4a(a.z, b.z, acc);
	acc = __dp4a(a.w, b.w, acc);
	return acc;
}

// MT rows per pass, RPW output channels per warp per step.
template <int MT, int RPW>
__global__ void __launch_bounds__(kGemvThreads)
k_gemv(LinearArgs a) {
	extern __shared__ __align__(16) unsigned char smem[];
	int8_t* sx = (int8_t*)smem;                                         // [MT][K]
	unsigned long long* smax = (unsigned long long*)(smem + (size_t)MT * a.K);  // [3][MT] (+ [MT] best)
	const int m0 = blockIdx.y * MT;
	const int mcount = min(MT, a.M - m0);
	const int K = a.K, kv = K / 16;
	pdl_wait();
	pdl_release();
	for (int i = threadIdx.x; i < MT * kv; i += blockDim.x) {
		const int m = i / kv, c = i - m * kv;
		int4 v = make_int4(0, 0, 0, 0);
		if (m < mcount) v = ((const int4*)(a.x + (size_t)(m0 + m) * K))[c];
		((int4*)sx)[i] = v;
	}
	if (threadIdx.x < 4 * MT) smax[threadIdx.x] = 0ull;
	__syncthreads();

	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const int gwarp = blockIdx.x * kGemvWarps + warp, nwarps = gridDim.x * kGemvWarps;
	// this lane's output duty after the reduction: channel c_me of the step, row m_me
	const int c_me = lane / MT, m_me = lane % MT;
	unsigned long long lmax[3] = {0ull, 0ull, 0ull};
	unsigned long long lbest = 0ull;

	for (int n0 = gwarp * RPW; n0 < a.N; n0 += nwarps * RPW) {
		int acc[RPW][MT];
#pragma unroll
		for (int c = 0; c < RPW; ++c)
#pragma unroll
			for (int m = 0; m < MT; ++m) acc[c][m] = 0;
		for (int kc = lane; kc < kv; kc += 32) {
			int4 wv[RPW];
#pragma unroll
			for (int c = 0; c < RPW; ++c) {
				const int n = min(n0 + c, a.N - 1);
				wv[c] = __ldg((const int4*)(a.w + (size_t)n * K) + kc);
			}
#pragma unroll
			for (int m = 0; m < MT; ++m) {
				const int4 xv = ((const int4*)(sx + (size_t)m * K))[kc];
#pragma unroll
				for (int c = 0; c < RPW; ++c) acc[c][m] = dot16(wv[c], xv, acc[c][m]);
			}
		}
		int mine = 0;
#pragma unroll
		for (int c = 0; c < RPW; ++c)
#pragma unroll
			for (int m = 0; m < MT; ++m) {
				int v = acc[c][m];
#pragma unroll
				for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
				if (c == c_me && m == m_me) mine = v;
			}
		const int n = n0 + c_me;
		if (c_me < RPW && n < a.N && m_me < mcount) {
			const int row = m0 + m_me;
			int seg = 0;
			while (seg + 1 < a.nseg && n >= a.seg_end[seg]) ++seg;
			int32_t v32 = mine;
			if (a.fold) v32 = fold(mine, a.fold[3 * n], a.fold[3 * n + 1], a.fold[3 * n + 2]);
			int64_t v = v32;
			if (a.rows != nullptr && a.seg_lora[seg] >= 0) {
				const LoraLayerDev* ll = a.rows[row].lora;
				if (ll != nullptr) {
					const LoraLayerDev& L = ll[a.layer];
					const LoraProjDev& p = L.p[a.seg_lora[seg]];
					if (p.a != nullptr) {
						const int nl = n - (seg ? a.seg_end[seg - 1] : 0);
						const int8_t* brow = p.b + (size_t)nl * L.rank;
						const int8_t* u = a.lora_u + ((size_t)row * 3 + seg) * kMaxLoraRank;
						int dsum = 0;
						for (uint32_t t = 0; t < L.rank; ++t) dsum += (int)brow[t] * (int)u[t];
						v += (int64_t)amp_fold(dsum, p.df[3 * nl], p.df[3 * nl + 1], p.df[3 * nl + 2]);
					}
				}
			}
			if (a.best != nullptr) {
				if (a.row_mask != nullptr) {
					const uint8_t* page = a.row_mask[row];
					if (page != nullptr && !((page[n >> 3] >> (n & 7)) & 1u)) v32 = INT32_MIN;
				}
				const unsigned long long key =
				    ((unsigned long long)((uint32_t)v32 ^ 0x80000000u) << 32) | (0xFFFFFFFFu - (uint32_t)n);
				lbest = key > lbest ? key : lbest;
				if (a.logits) a.logits[(size_t)row * a.N + n] = v32;
			} else {
				if (a.out64) ((int64_t*)a.out)[(size_t)row * a.out_ld + n] = v;
				else ((int32_t*)a.out)[(size_t)row * a.out_ld + n] = (int32_t)v;
				if (a.seg_slot[seg] >= 0) {
					const unsigned long long ab = v < 0 ? (~(unsigned long long)v + 1ull) : (unsigned long long)v;
					lmax[seg] = ab > lmax[seg] ? ab : lmax[seg];
				}
			}
		}
	}
	// block-level reduction of the row maxima / argmax keys, then one global atomic each
	if (c_me < RPW && m_me < mcount) {
		if (a.best != nullptr) {
			if (lbest) atomicMax(&smax[3 * MT + m_me], lbest);
		} else {
#pragma unroll
			for (int s = 0; s < 3; ++s)
				if (lmax[s]) atomicMax(&smax[s * MT + m_me], lmax[s]);
		}
	}
	__syncthreads();
	if (threadIdx.x < 4 * MT) {
		const int s = threadIdx.x / MT, m = threadIdx.x % MT;
		const unsigned long long v = smax[threadIdx.x];
		if (v != 0ull && m < mcount) {
			if (s == 3) atomicMax(&a.best[m0 + m], v);
			else if (a.rowmax != nullptr && s < a.nseg && a.seg_slot[s] >= 0)
				atomicMax(&a.rowmax[(size_t)(m0 + m) * 4 + a.seg_slot[s]], v);
		}
	}
}

template <int MT, int RPW>
static void launch_one(const LinearArgs& a, int grid_x, int grid_y, cudaStream_t st) {
	const size_t smem = (size_t)MT * a.K + 4 * MT * 8 + 16;
	static bool configured = false;
	if (!configured) {
		cudaFuncSetAttribute(k_gemv<MT, RPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
		configured = true;
	}
	launch_pdl(k_gemv<MT, RPW>, dim3(grid_x, grid_y), dim3(kGemvThreads), smem, st, a);
}

template <int MT>
static void launch_mt(const LinearArgs& a, int grid_y, cudaStream_t st) {
	// as many channels per warp step as keeps at least ~2 blocks per SM busy
	const int want_blocks = 296;
	int rpw = 4;
	while (rpw > 1 && (a.N + kGemvWarps * rpw - 1) / (kGemvWarps * rpw) * grid_y < want_blocks) rpw >>= 1;
	if (MT * rpw > 32) rpw = 32 / MT;   // one output per lane
	int gx = (a.N + kGemvWarps * rpw - 1) / (kGemvWarps * rpw);
	if (gx > 148 * 8) gx = 148 * 8;
	if (rpw == 4) launch_one<MT, 4>(a, gx, grid_y, st);
	else if (rpw == 2) launch_one<MT, 2>(a, gx, grid_y, st);
	else launch_one<MT, 1>(a, gx, grid_y, st);
}

void launch_linear_gemv(const LinearArgs& a, cudaStream_t st) {
	if (a.M <= 1) launch_mt<1>(a, 1, st);
	else if (a.M <= 2) launch_mt<2>(a, 1, st);
	else if (a.M <= 4) launch_mt<4>(a, 1, st);
	else launch_mt<8>(a, (a.M + 7) / 8, st);
}

// ---------------------------------------------------------------- LoRA u = A x
// grid (rows, projections); one warp per rank row of A.
__global__ void k_lora_u(RowBatch b, const int8_t* x, int k_in, int layer, int s0, int s1, int s2) {
	const int r = blockIdx.x, pj = blockIdx.y;
	const int slot = pj == 0 ? s0 : (pj == 1 ? s1 : s2);
	pdl_wait();
	pdl_release();
	const LoraLayerDev* ll = b.rows[r].lora;
	if (ll == nullptr) return;
	const LoraLayerDev& L = ll[layer];
	const LoraProjDev& p = L.p[slot];
	if (p.a == nullptr) return;
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
	const int4* xv = (const int4*)(x + (size_t)r * k_in);
	for (uint32_t t = warp; t < L.rank; t += nw) {
		const int4* av = (const int4*)(p.a + (size_t)t * k_in);
		int acc = 0;
		for (int kc = lane; kc < k_in / 16; kc += 32) acc = dot16(__ldg(av + kc), xv[kc], acc);
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
		if (lane == 0) {
			const int32_t u = amp_fold(acc, p.uf[3 * t], p.uf[3 * t + 1], p.uf[3 * t + 2]);
			b.lora_u[((size_t)r * 3 + pj) * kMaxLoraRank + t] = (int8_t)clamp127(u);
		}
	}
}

void launch_lora_u(const RowBatch& b, const int8_t* x, int k_in, int layer, int nproj,
                   const int* slots, cudaStream_t st) {
	launch_pdl(k_lora_u, dim3(b.m, nproj), dim3(256), 0, st, b, x, k_in, layer, slots[0], nproj > 1 ? slots[1] : 0,
	                                            nproj > 2 ? slots[2] : 0);
}

}  // namespace sslm
