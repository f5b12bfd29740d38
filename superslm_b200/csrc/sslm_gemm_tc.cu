// Prefill / batched-decode int8 linear layer on the 5th-generation tensor cores.
//
//   out[m,n] = fold_n( sum_k x[m,k] * w[n,k] ) (+ LoRA delta), per-row max |out| per segment
//
// A = activations [M,K] and B = weights [N,K] are both K-major, which is exactly the
// operand form tcgen05.mma wants, so no repacking happens anywhere: TMA
// (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast) streams 128x128-byte tiles of
// both into a shared-memory ring, one elected thread issues tcgen05.mma.kind::i8
// (M=128, N=128, K=32 per instruction, s8 x s8 -> s32) into a TMEM accumulator, and four
// epilogue warps read the accumulator back with tcgen05.ld, apply the per-channel
// fixed-point fold (ApplyWeightScaleFold, src/forward/forward_sites.cpp:461-470), add the
// runtime LoRA delta (:1082-1102), store the wide row and reduce the row maximum that the
// requant funnel needs (an integer max: order-free, so deterministic).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4) .. +31, one output row per thread).
// Every wait on an mbarrier is bounded; a wait that runs out marks the tile's rows with an
// internal status and the block tears down normally (TMEM is always freed).
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

#include "sslm_kernels.h"

namespace sslm {

namespace {

constexpr int BM = 128, BN = 128, BK = 128, UMMA_K = 32, STAGES = 6;
constexpr int kTcThreads = 192;
constexpr uint32_t kStageBytes = (BM + BN) * BK;          // 32 KiB
constexpr uint32_t kSmemBytes = STAGES * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr uint32_t kMaxPolls = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
	uint32_t ok;
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
	    "selp.u32 %0, 1, 0, p;\n\t}"
	    : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
	return ok != 0;
}
// bounded wait: false when the limit ran out
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
	for (uint32_t i = 0; i < kMaxPolls; ++i) {
		if (mbar_try_wait(bar, parity)) return true;
		if (i > 1024) __nanosleep(64);
	}
	return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
	asm volatile(
	    "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
	    ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// K-major, 128-byte-swizzled operand tile: 8-row groups are 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
	uint64_t d = 0;
	d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address
	d |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzle)
	d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset
	d |= (uint64_t)1 << 46;                               // descriptor version (sm_100)
	d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
	return d;
}
// s8 x s8 -> s32, A and B K-major, M = 128, N = BN
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "setp.ne.b32 p, %4, 0;\n\t"
	    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
	    ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
	asm volatile(
	    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
	    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
	    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
	      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
	      "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
	      "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
	    : "r"(taddr));
	asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kTcThreads, 1)
k_linear_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, LinearArgs a,
            int32_t* row_status) {
	extern __shared__ unsigned char smem_raw[];
	const uint32_t raw = smem_u32(smem_raw);
	const uint32_t base = (raw + 1023u) & ~1023u;            // SW128 tiles want 1024-byte alignment
	unsigned char* smem = smem_raw + (base - raw);
	const uint32_t bars = base + STAGES * kStageBytes;       // full[S], empty[S], acc_full, tmem slot
	auto full_bar = [&](int s) { return bars + 8u * s; };
	auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
	const uint32_t acc_bar = bars + 8u * (2 * STAGES);
	uint32_t* tmem_slot = (uint32_t*)(smem + STAGES * kStageBytes + 8 * (2 * STAGES + 1));
	__shared__ int s_timeout;

	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int tile_n = blockIdx.x, tile_m = blockIdx.y;
	const int m0 = tile_m * BM, n0 = tile_n * BN;
	const int kblocks = (a.K + BK - 1) / BK;

	if (threadIdx.x == 0) {
		for (int s = 0; s < STAGES; ++s) {
			mbar_init(full_bar(s), 1);
			mbar_init(empty_bar(s), 1);
		}
		mbar_init(acc_bar, 1);
		s_timeout = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 1) {
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN));
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem_base = *tmem_slot;

	if (warp == 0) {
		if (lane == 0) {
			for (int kb = 0; kb < kblocks; ++kb) {
				const int s = kb % STAGES;
				const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
				if (!mbar_wait(empty_bar(s), phase ^ 1u)) { s_timeout = 1; break; }
				mbar_expect_tx(full_bar(s), kStageBytes);
				const uint32_t sa = base + s * kStageBytes, sb = sa + BM * BK;
				tma_load_2d(sa, &map_a, full_bar(s), kb * BK, m0);
				tma_load_2d(sb, &map_b, full_bar(s), kb * BK, n0);
			}
		}
	} else if (warp == 1) {
		if (lane == 0) {
			bool ok = true;
			for (int kb = 0; kb < kblocks && ok; ++kb) {
				const int s = kb % STAGES;
				const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
				if (!mbar_wait(full_bar(s), phase)) { s_timeout = 1; ok = false; break; }
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
				const uint32_t sa = base + s * kStageBytes, sb = sa + BM * BK;
				const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sb);
#pragma unroll
				for (int k = 0; k < BK / UMMA_K; ++k) {
					// advancing inside the 128-byte swizzle atom: +32 bytes = +2 in descriptor units
					umma_i8(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), (kb | k) != 0 ? 1u : 0u);
				}
				umma_commit(empty_bar(s));     // frees the stage once these MMAs have read it
			}
			umma_commit(acc_bar);              // accumulator complete (arrives even after a timeout)
		}
	} else {
		// epilogue: this thread owns output row m0 + 32*q + lane
		const int q = warp & 3;
		const int row = m0 + q * 32 + lane;
		const bool acc_ok = mbar_wait(acc_bar, 0);
		asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
		if (!acc_ok) s_timeout = 1;
		const bool row_ok = acc_ok && row < a.M && s_timeout == 0;
		const LoraLayerDev* lora = (row_ok && a.rows != nullptr && a.rows[row].lora != nullptr) ? a.rows[row].lora + a.layer : nullptr;
		unsigned long long lmax[3] = {0ull, 0ull, 0ull};
		unsigned long long lbest = 0ull;
		for (int c0 = 0; c0 < BN; c0 += 32) {
			uint32_t r[32];
			tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);   // warp-collective: never skipped
			if (!row_ok || n0 + c0 >= a.N) continue;
			const bool vec_ok = !a.out64 && (a.out_ld & 3) == 0 && (((uintptr_t)a.out) & 15) == 0;
#pragma unroll
			for (int j4 = 0; j4 < 32; j4 += 4) {
				int64_t v4[4];
#pragma unroll
				for (int jj = 0; jj < 4; ++jj) {
					const int n = n0 + c0 + j4 + jj;
					v4[jj] = 0;
					if (n >= a.N) continue;
					int seg = 0;
					while (seg + 1 < a.nseg && n >= a.seg_end[seg]) ++seg;
					int32_t v32 = (int32_t)r[j4 + jj];
					if (a.fold) v32 = fold(v32, a.fold[3 * n], a.fold[3 * n + 1], a.fold[3 * n + 2]);
					int64_t v = v32;
					if (lora != nullptr && a.seg_lora[seg] >= 0) {
						const LoraProjDev& p = lora->p[a.seg_lora[seg]];
						if (p.a != nullptr) {
							const int nl = n - (seg ? a.seg_end[seg - 1] : 0);
							const int8_t* brow = p.b + (size_t)nl * lora->rank;
							const int8_t* u = a.lora_u + ((size_t)row * 3 + seg) * kMaxLoraRank;
							int dsum = 0;
							for (uint32_t t = 0; t < lora->rank; ++t) dsum += (int)brow[t] * (int)u[t];
							v += (int64_t)amp_fold(dsum, p.df[3 * nl], p.df[3 * nl + 1], p.df[3 * nl + 2]);
						}
					}
					if (a.best != nullptr) {   // head: greedy argmax key, lowest index wins ties
						const unsigned long long key =
						    ((unsigned long long)((uint32_t)v32 ^ 0x80000000u) << 32) | (0xFFFFFFFFu - (uint32_t)n);
						lbest = key > lbest ? key : lbest;
						if (a.logits) a.logits[(size_t)row * a.N + n] = v32;
						continue;
					}
					v4[jj] = v;
					const unsigned long long ab = v < 0 ? (~(unsigned long long)v + 1ull) : (unsigned long long)v;
					if (seg == 0) lmax[0] = ab > lmax[0] ? ab : lmax[0];
					else if (seg == 1) lmax[1] = ab > lmax[1] ? ab : lmax[1];
					else lmax[2] = ab > lmax[2] ? ab : lmax[2];
				}
				const int nb = n0 + c0 + j4;
				if (nb >= a.N || a.best != nullptr) continue;
				if (vec_ok && nb + 3 < a.N) {
					*(int4*)((int32_t*)a.out + (size_t)row * a.out_ld + nb) =
					    make_int4((int)v4[0], (int)v4[1], (int)v4[2], (int)v4[3]);
				} else {
#pragma unroll
					for (int jj = 0; jj < 4; ++jj) {
						if (nb + jj >= a.N) break;
						if (a.out64) ((int64_t*)a.out)[(size_t)row * a.out_ld + nb + jj] = v4[jj];
						else ((int32_t*)a.out)[(size_t)row * a.out_ld + nb + jj] = (int32_t)v4[jj];
					}
				}
			}
		}
		if (row_ok && a.best != nullptr && lbest != 0ull) atomicMax(&a.best[row], lbest);
		if (row_ok && a.rowmax != nullptr) {
			for (int s = 0; s < a.nseg; ++s)
				if (a.seg_slot[s] >= 0 && lmax[s] != 0ull) atomicMax(&a.rowmax[(size_t)row * 4 + a.seg_slot[s]], lmax[s]);
		}
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (s_timeout != 0 && row_status != nullptr && threadIdx.x < BM && m0 + (int)threadIdx.x < a.M)
		atomicCAS(&row_status[m0 + threadIdx.x], 0, (int32_t)kInternalWaitTimeout);
	if (warp == 1) {
		asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN));
	}
}

// ------------------------------------------------------------ host: tensor maps
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
	static EncodeFn fn = [] {
		void* p = nullptr;
		cudaDriverEntryPointQueryResult q;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
		return (EncodeFn)p;
	}();
	return fn;
}

struct MapKey {
	const void* p;
	int rows, k;
	bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && k == o.k; }
};
struct MapKeyHash {
	size_t operator()(const MapKey& k) const {
		return std::hash<const void*>()(k.p) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.k << 40);
	}
};

// [rows, K] int8 row-major -> 2-D map, box 128 bytes x 128 rows, 128-byte swizzle, zero fill
bool tensor_map(const void* ptr, int rows, int k, CUtensorMap* out) {
	static std::mutex mu;
	static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
	const MapKey key{ptr, rows, k};
	std::lock_guard<std::mutex> lock(mu);
	auto it = cache.find(key);
	if (it != cache.end()) {
		*out = it->second;
		return true;
	}
	EncodeFn fn = encode_fn();
	if (!fn) return false;
	const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
	const cuuint64_t strides[1] = {(cuuint64_t)k};
	const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
	const cuuint32_t estr[2] = {1, 1};
	CUtensorMap m;
	if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
	       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
	       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
		return false;
	if (cache.size() > 4096) cache.clear();
	cache.emplace(key, m);
	*out = m;
	return true;
}

}  // namespace

bool launch_linear_tc(const LinearArgs& a, cudaStream_t st) {
	if (a.K % 16 != 0 || ((uintptr_t)a.x & 15) || ((uintptr_t)a.w & 15)) return false;
	static bool configured = false;
	if (!configured) {
		if (cudaFuncSetAttribute(k_linear_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
			return false;
		configured = true;
	}
	CUtensorMap ma, mb;
	if (!tensor_map(a.x, a.M, a.K, &ma) || !tensor_map(a.w, a.N, a.K, &mb)) return false;
	const dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM);
	k_linear_tc<<<grid, kTcThreads, kSmemBytes, st>>>(ma, mb, a, a.status);
	return true;
}

}  // namespace sslm
