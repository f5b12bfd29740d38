// Decode-path int8 linear layer: out[m,n] = fold_n(sum_k x[m,k] w[n,k]) for a handful of
// rows m. HBM-bound: the kernel exists to keep the weight stream at the speed of the memory.
//
// A block owns a contiguous range of output channels; its warps deal those channels among
// themselves (warp w takes channels w, w + W, ...). Every warp streams ITS weight rows through
// its own small ring in shared memory with bulk asynchronous copies (cp.async.bulk, one row or one
// 4 KiB segment of a long row per copy, completion counted on an mbarrier of that ring slot): the
// warp is producer and consumer of its ring, so the main loop has no block-wide synchronisation
// at all, ~100 KiB per block are in flight without holding a register, and a lane's partial sums
// of a channel stay in registers until the channel's last segment -- one warp reduction per
// channel and row of x, whatever K is. The activations sit in shared memory; dp4a does the
// arithmetic.
//
// The weights are written by no kernel, so every ring's first copies and the block's fold rows
// are requested BEFORE the dependency wait: while the kernel in front (a row kernel that moves
// little data) finishes, this kernel's weight stream is already running.
//
// The epilogue applies the per-channel weight-scale fold, adds the LoRA delta, stores the wide
// row and reduces the per-row max |x| the funnel needs (or the argmax key for the head).
// (GemmInt8AccumulateRow + ApplyWeightScaleFold + AddAmplifyingLoraDelta,
//  src/matmul.cpp:455-464, src/forward/forward_sites.cpp:461-470, :1051-1103.)
// int32 accumulation is exact: K * 127 * 128 < 2^31 for every K the loader accepts, and integer
// sums do not depend on the order in which pieces are added.
//
// Every wait on an mbarrier is bounded; a wait that runs out marks the block's rows with an
// internal status, the warp stops issuing copies, waits (bounded again) for the copies it has
// in flight, and the block returns.
#include <cuda_runtime.h>

#include "sslm_kernels.h"

namespace sslm {

// Sixteen warps per block and (shared memory allowing) two blocks per multiprocessor: a warp's
// loop over its items is one dependent chain (wait, load, dp4a, reduce), so the memory system
// is kept busy by the number of warps that run such chains side by side, not by any one of them.
constexpr int kGemvWarps = 16;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kItemBytes = 3072;                    // largest single copy: whole rows, or one segment of a long row
constexpr int kRingBytesPerWarp = 6 * 1024;
constexpr int kMaxSlots = 4;
constexpr uint32_t kGemvMaxPolls = 1u << 22;

__device__ __forceinline__ int dot16(const int4& a, const int4& b, int acc) {
	acc = __dp4a(a.x, b.x, acc);
	acc = __dp4a(a.y, b.y, acc);
	acc = __dp4a(a.z, b.z, acc);
	acc = __dp4a(a.w, b.w, acc);
	return acc;
}

namespace {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint32_t bar, uint32_t parity) {
	uint32_t ok;
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
	    "selp.u32 %0, 1, 0, p;\n\t}"
	    : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
	return ok != 0;
}
// bounded wait: false when the limit ran out
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
	for (uint32_t i = 0; i < kGemvMaxPolls; ++i) {
		if (bar_try_wait(bar, parity)) return true;
		if (i > 1024) __nanosleep(64);
	}
	return false;
}
// contiguous global -> shared copy (both 16-byte aligned, bytes a multiple of 16); completes on `bar`
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
	             ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

}  // namespace

// What the host decides per launch. A work item is one bulk copy: `rows_per_item` whole weight
// rows when a row is short (then nseg = 1), else one of the `nseg` segments of one row. The items
// of a block are dealt round-robin to its warps.
struct GemvPlan {
	int rows_per_block;   // output channels per block
	int rows_per_item;    // whole rows per copy (1 when rows are cut into segments)
	int seg16;            // 16-byte pieces per segment (= K / 16 when nseg == 1)
	int nseg;             // segments per weight row
	int slots;            // ring slots per warp
	int step_g, step_s;   // item index + kGemvWarps = (group + step_g, segment + step_s), segment taken mod nseg
};

// MT rows of x per pass (grid.y walks the row groups).
template <int MT>
__global__ void __launch_bounds__(kGemvThreads)
k_gemv(LinearArgs a, GemvPlan p) {
	extern __shared__ __align__(128) unsigned char smem[];
	const int K = a.K, k16 = K >> 4;
	const int n0 = blockIdx.x * p.rows_per_block;
	const int nrows = min(p.rows_per_block, a.N - n0);
	const int m0 = blockIdx.y * MT;
	const int mcount = min(MT, a.M - m0);
	const int slot_bytes = p.rows_per_item * p.seg16 * 16;
	// carve: rings | x rows | accumulators | fold rows | maxima | barriers
	unsigned char* rings = smem;
	int8_t* sx = (int8_t*)(rings + (size_t)kGemvWarps * p.slots * slot_bytes);
	int* sacc = (int*)(sx + (size_t)MT * K);                                   // [MT][rows_per_block]
	int32_t* sfold = sacc + (size_t)MT * p.rows_per_block;                     // [rows_per_block][3]
	unsigned long long* smax = (unsigned long long*)(((uintptr_t)(sfold + 3 * (size_t)p.rows_per_block) + 7) & ~(uintptr_t)7);   // [4][MT]
	const uint32_t bars = smem_addr(smax + 4 * MT);                            // [warps][kMaxSlots]
	__shared__ int s_timeout;

	const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
	unsigned char* ring = rings + (size_t)warp * p.slots * slot_bytes;
	auto full_bar = [&](int s) { return bars + 8u * (warp * kMaxSlots + s); };
	// the block's items: (row group, segment), item q = group * nseg + segment; this warp takes
	// q = warp, warp + kGemvWarps, ...
	const int groups = (nrows + p.rows_per_item - 1) / p.rows_per_item;
	const int total_items = groups * p.nseg;
	const int items = total_items > warp ? (total_items - warp + kGemvWarps - 1) / kGemvWarps : 0;
	// requests are made in item order, so the request side keeps its own (group, segment, slot) counters
	int q_g = warp / p.nseg, q_s = warp % p.nseg, q_sl = 0;
	auto issue = [&]() {      // (lane 0 only)
		const int row0 = q_g * p.rows_per_item;
		const int nr = min(p.rows_per_item, nrows - row0);
		const int first = q_s * p.seg16, count = min(p.seg16, k16 - first);
		const uint32_t bytes = (uint32_t)nr * (uint32_t)count * 16u;     // (nr > 1 only with whole rows: contiguous)
		bar_expect_tx(full_bar(q_sl), bytes);
		bulk_load(smem_addr(ring + (size_t)q_sl * slot_bytes), a.w + ((size_t)(n0 + row0) * K + (size_t)first * 16), bytes,
		          full_bar(q_sl));
		q_g += p.step_g;
		q_s += p.step_s;
		if (q_s >= p.nseg) {
			q_s -= p.nseg;
			++q_g;
		}
		if (++q_sl == p.slots) q_sl = 0;
	};

	if (lane == 0) {
		for (int s = 0; s < p.slots; ++s) bar_init(full_bar(s), 1);
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (t == 0) s_timeout = 0;
	__syncwarp();
	// ahead of the dependency wait: the first copies of every ring, the block's fold rows, cleared
	// accumulators and maxima
	int issued = items < p.slots ? items : p.slots;      // items whose copies have been requested
	if (lane == 0)
		for (int i = 0; i < issued; ++i) issue();
	if (a.fold != nullptr) {
		const int32_t* f = a.fold + (size_t)n0 * 3;
		for (int i = t; i < nrows * 3; i += kGemvThreads) sfold[i] = __ldg(f + i);
	}
	for (int i = t; i < MT * p.rows_per_block; i += kGemvThreads) sacc[i] = 0;
	if (t < 4 * MT) smax[t] = 0ull;
	pdl_wait();
	pdl_release();
	// the activation rows (written by the kernel in front: read past the L1)
	for (int i = t; i < MT * k16; i += kGemvThreads) {
		const int m = i / k16, c = i - m * k16;
		int4 v = make_int4(0, 0, 0, 0);
		if (m < mcount) v = __ldcg((const int4*)(a.x + (size_t)(m0 + m) * K) + c);
		((int4*)sx)[i] = v;
	}
	__syncthreads();

	bool ok = true;
	// item being consumed: (group c_g, segment c_s) in ring slot sl with wait parity par
	int c_g = warp / p.nseg, c_s = warp % p.nseg, sl = 0;
	uint32_t par = 0;
	for (int i = 0; i < items; ++i) {
		// (the whole warp agrees on the outcome of a wait)
		if (!__all_sync(0xffffffffu, bar_wait(full_bar(sl), par) ? 1 : 0)) {
			atomicExch(&s_timeout, 1);
			ok = false;
			break;
		}
		const int row0 = c_g * p.rows_per_item;
		const int nr = min(p.rows_per_item, nrows - row0);
		const int first = c_s * p.seg16, count = min(p.seg16, k16 - first);
		const int4* wv = (const int4*)(ring + (size_t)sl * slot_bytes);
		for (int rr = 0; rr < nr; ++rr) {
			int acc[MT];
#pragma unroll
			for (int m = 0; m < MT; ++m) acc[m] = 0;
#pragma unroll 2
			for (int c = lane; c < count; c += 32) {
				const int4 w4 = wv[rr * count + c];
#pragma unroll
				for (int m = 0; m < MT; ++m) acc[m] = dot16(w4, ((const int4*)(sx + (size_t)m * K))[first + c], acc[m]);
			}
			// one reduction per (row of x, weight row segment); segments of one weight row may
			// belong to different warps, so the sums meet in shared memory
#pragma unroll
			for (int m = 0; m < MT; ++m) {
				const int v = __reduce_add_sync(0xffffffffu, acc[m]);
				if (lane == 0) {
					if (p.nseg == 1) sacc[m * p.rows_per_block + row0 + rr] = v;
					else atomicAdd(&sacc[m * p.rows_per_block + row0 + rr], v);
				}
			}
		}
		__syncwarp();      // every lane has read the slot: it may be refilled
		if (issued < items) {
			if (lane == 0) issue();
			++issued;
		}
		c_g += p.step_g;
		c_s += p.step_s;
		if (c_s >= p.nseg) {
			c_s -= p.nseg;
			++c_g;
		}
		if (++sl == p.slots) {
			sl = 0;
			par ^= 1u;
		}
	}
	if (!ok && lane == 0) {
		// the copies this warp still has in flight must land before the block's shared memory is given up
		for (int s = 0; s < p.slots && s < issued; ++s) {
			const int last = ((issued - 1 - s) / p.slots) * p.slots + s;     // last requested item that uses slot s
			bar_wait(full_bar(s), (uint32_t)(last / p.slots) & 1u);
		}
	}
	__syncthreads();

	if (*(volatile int*)&s_timeout) {
		if (a.status != nullptr && t < mcount) atomicCAS(&a.status[m0 + t], 0, (int32_t)kInternalWaitTimeout);
		return;
	}
	// ---- epilogue: thread i takes output (m, n) = (i / nrows, i % nrows)
	unsigned long long lmax[3] = {0ull, 0ull, 0ull};
	unsigned long long lbest = 0ull;
	int my_m = -1;
	auto flush = [&]() {
		if (my_m < 0) return;
		if (a.best != nullptr) {
			if (lbest) atomicMax(&smax[3 * MT + my_m], lbest);
		} else {
#pragma unroll
			for (int sg = 0; sg < 3; ++sg)
				if (lmax[sg]) atomicMax(&smax[sg * MT + my_m], lmax[sg]);
		}
		lmax[0] = lmax[1] = lmax[2] = 0ull;
		lbest = 0ull;
	};
	for (int i = t; i < mcount * nrows; i += kGemvThreads) {
		const int m = i / nrows, nl0 = i - m * nrows;
		if (m != my_m) {      // (a thread's outputs belong to one row of x except when the block has few channels)
			flush();
			my_m = m;
		}
		const int n = n0 + nl0, rowg = m0 + m;
		const int mine = sacc[m * p.rows_per_block + nl0];
		int seg = 0;
		while (seg + 1 < a.nseg && n >= a.seg_end[seg]) ++seg;
		int32_t v32 = mine;
		if (a.fold) v32 = fold(mine, sfold[3 * nl0], sfold[3 * nl0 + 1], sfold[3 * nl0 + 2]);
		int64_t v = v32;
		if (a.rows != nullptr && a.seg_lora[seg] >= 0) {
			const LoraLayerDev* ll = a.rows[rowg].lora;
			if (ll != nullptr) {
				const LoraLayerDev& L = ll[a.layer];
				const LoraProjDev& pj = L.p[a.seg_lora[seg]];
				if (pj.a != nullptr) {
					const int nl = n - (seg ? a.seg_end[seg - 1] : 0);
					const int8_t* brow = pj.b + (size_t)nl * L.rank;
					const int8_t* u = a.lora_u + ((size_t)rowg * 3 + seg) * kMaxLoraRank;
					int dsum = 0;
					for (uint32_t r = 0; r < L.rank; ++r) dsum += (int)brow[r] * (int)u[r];
					v += (int64_t)amp_fold(dsum, pj.df[3 * nl], pj.df[3 * nl + 1], pj.df[3 * nl + 2]);
				}
			}
		}
		if (a.best != nullptr) {
			if (a.row_mask != nullptr) {
				const uint8_t* page = a.row_mask[rowg];
				if (page != nullptr && !((page[n >> 3] >> (n & 7)) & 1u)) v32 = INT32_MIN;
			}
			const unsigned long long key =
			    ((unsigned long long)((uint32_t)v32 ^ 0x80000000u) << 32) | (0xFFFFFFFFu - (uint32_t)n);
			lbest = key > lbest ? key : lbest;
			if (a.logits) a.logits[(size_t)rowg * a.N + n] = v32;
		} else {
			if (a.out64) ((int64_t*)a.out)[(size_t)rowg * a.out_ld + n] = v;
			else ((int32_t*)a.out)[(size_t)rowg * a.out_ld + n] = (int32_t)v;
			if (a.seg_slot[seg] >= 0) {
				const unsigned long long ab = v < 0 ? (~(unsigned long long)v + 1ull) : (unsigned long long)v;
				lmax[seg] = ab > lmax[seg] ? ab : lmax[seg];
			}
		}
	}
	flush();
	__syncthreads();
	if (t < 4 * MT) {
		const int sg = t / MT, m = t % MT;
		const unsigned long long v = smax[t];
		if (v != 0ull && m < mcount) {
			if (sg == 3) atomicMax(&a.best[m0 + m], v);
			else if (a.rowmax != nullptr && sg < a.nseg && a.seg_slot[sg] >= 0)
				atomicMax(&a.rowmax[(size_t)(m0 + m) * 4 + a.seg_slot[sg]], v);
		}
	}
}

// shared memory of one block: rings, activation rows, accumulators, fold rows, maxima, barriers
static size_t gemv_smem_bytes(int mt, int K, int rows_per_block, int slots, int slot_bytes) {
	return (size_t)kGemvWarps * slots * slot_bytes + (size_t)mt * K + (size_t)mt * rows_per_block * 4 +
	       (size_t)rows_per_block * 12 + 8 + (size_t)4 * mt * 8 + (size_t)kGemvWarps * kMaxSlots * 8 + 16;
}

template <int MT>
static cudaError_t launch_mt(const LinearArgs& a, int grid_y, cudaStream_t st) {
	static PerDeviceOnce configured;
	cudaError_t e = once_per_device(configured, [] {
		cudaError_t c = cudaFuncSetAttribute(k_gemv<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
		if (c != cudaSuccess) return c;
		return cudaFuncSetAttribute(k_gemv<MT>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
	});
	if (e != cudaSuccess) return e;
	GemvPlan p;
	const int k16 = a.K / 16;
	// a copy carries whole rows while a row is short, else one segment of a row
	if (a.K * 2 <= kItemBytes) {
		p.rows_per_item = kItemBytes / a.K;
		p.nseg = 1;
		p.seg16 = k16;
	} else {
		p.rows_per_item = 1;
		p.nseg = (a.K + kItemBytes - 1) / kItemBytes;
		p.seg16 = (k16 + p.nseg - 1) / p.nseg;
		p.nseg = (k16 + p.seg16 - 1) / p.seg16;
	}
	// Two blocks per multiprocessor when the activation rows leave room for two rings. A block
	// takes whole row groups; it should have at least one item per warp, but never so many rows
	// that blocks are fewer than the multiprocessors while rows remain to hand out.
	const int sms = sm_count();
	const int per_sm = (size_t)MT * a.K <= 16 * 1024 ? 2 : 1;
	int rpb = (a.N + per_sm * sms - 1) / (per_sm * sms);
	const int min_rows = (kGemvWarps + p.nseg - 1) / p.nseg * p.rows_per_item;      // rows that make one item per warp
	if (rpb < min_rows && (a.N + min_rows - 1) / min_rows >= sms) rpb = min_rows;
	rpb = (rpb + p.rows_per_item - 1) / p.rows_per_item * p.rows_per_item;
	if (rpb > a.N) rpb = a.N;
	p.rows_per_block = rpb;
	p.step_g = kGemvWarps / p.nseg;
	p.step_s = kGemvWarps % p.nseg;
	const int slot_bytes = p.rows_per_item * p.seg16 * 16;
	int slots = kRingBytesPerWarp / slot_bytes;
	if (slots > kMaxSlots) slots = kMaxSlots;
	if (slots < 2) slots = 2;
	const int groups = (rpb + p.rows_per_item - 1) / p.rows_per_item;
	const int items_per_warp = (groups * p.nseg + kGemvWarps - 1) / kGemvWarps;
	if (slots > items_per_warp) slots = items_per_warp;
	while (slots > 2 && gemv_smem_bytes(MT, a.K, rpb, slots, slot_bytes) > 220 * 1024) --slots;   // long activation rows: shallower rings
	p.slots = slots;
	const size_t smem = gemv_smem_bytes(MT, a.K, rpb, slots, slot_bytes);
	if (smem > 220 * 1024) return cudaErrorInvalidConfiguration;
	const int gx = (a.N + rpb - 1) / rpb;
	return launch_pdl(k_gemv<MT>, dim3(gx, grid_y), dim3(kGemvThreads), smem, st, a, p);
}

cudaError_t launch_linear_gemv(const LinearArgs& a, cudaStream_t st) {
	if (a.M <= 1) return launch_mt<1>(a, 1, st);
	if (a.M <= 2) return launch_mt<2>(a, 1, st);
	if (a.M <= 4) return launch_mt<4>(a, 1, st);
	return launch_mt<8>(a, (a.M + 7) / 8, st);
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
