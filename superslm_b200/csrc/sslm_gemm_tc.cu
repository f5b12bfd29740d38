// Prefill / batched-decode int8 linear layer on the 5th-generation tensor cores.
//
//   out[m,n] = fold_n( sum_k x[m,k] * w[n,k] ) (+ LoRA delta), per-row max |out| per segment
//
// A = activations [M,K] and B = weights [N,K] are both K-major, which is exactly the
// operand form tcgen05.mma wants, so nothing is repacked: TMA (cp.async.bulk.tensor.2d,
// 128-byte swizzle, loads of this block only) streams 128-byte-wide tiles of both into a shared-memory
// ring, one thread issues tcgen05.mma.kind::i8 (s8 x s8 -> s32, M=128, N=BN, K=32 per
// instruction) into TMEM accumulators, and eight epilogue warps read the accumulators back
// with tcgen05.ld, apply the per-channel fixed-point fold (ApplyWeightScaleFold,
// src/forward/forward_sites.cpp:461-470), add the runtime LoRA delta (:1082-1102), store the
// wide row and reduce the row maximum the requant funnel needs (integer max: order-free).
//
// The kernel is persistent: one block per SM walks a list of output tiles. A tile is BN
// weight rows by MT*128 activation rows (MT = 2 shares every weight tile between two
// accumulators, so a decode batch of up to 256 sequences reads each weight byte once).
// Accumulators are double-buffered in TMEM, so the epilogue of tile i overlaps the main
// loop of tile i+1.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue (warp w reads TMEM lanes 32*(w%4) .. +31, one output row per thread,
// two warps per lane quarter sharing the columns).
// Every wait on an mbarrier is bounded; a wait that runs out marks the rows with an internal
// status and the block tears down normally (TMEM is always freed).
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "sslm_kernels.h"

namespace sslm {

// how often the tensor-core path ran / declined, and why it last declined
// (1 alignment, 2 shared-memory opt-in, 3 no cuTensorMapEncodeTiled, 4 tensor-map encode failed,
// 5 the launch itself was refused)
static std::atomic<unsigned long long> g_tc_launches{0}, g_tc_refusals{0};
static std::atomic<int> g_tc_last_reason{0};
// launches per kernel variant: 0 = 128 x 64 tiles, 1 = 128 x 128, 2 = 256 x 64, 3 = 256 x 128
static std::atomic<unsigned long long> g_tc_variant[8];

namespace {

constexpr int BM = 128, BK = 128, UMMA_K = 32;
constexpr int kTcThreads = 320;   // producer warp, MMA warp, eight epilogue warps
constexpr int kEpiThreads = 256;
constexpr uint32_t kMaxPolls = 1u << 22;
constexpr int kSmemBudget = 200 * 1024;

template <int MT, int BN>
struct TcCfg {
	static constexpr uint32_t kStageBytes = (uint32_t)(MT * BM + BN) * BK;
	static constexpr int kStages = (kSmemBudget / (int)kStageBytes) > 8 ? 8 : (kSmemBudget / (int)kStageBytes);
	static constexpr uint32_t kTmemCols = 2u * MT * BN;                       // two accumulator stages
	static constexpr uint32_t kFoldBytes = 2u * BN * 16;                      // double-buffered per-column fold words
	static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kFoldBytes + 1024 /*align*/ + 256 /*barriers*/;
	// s8 x s8 -> s32, A and B K-major, M = 128, N = BN
	static constexpr uint32_t kInstrDesc =
	    (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
		if (i > 2048) __nanosleep(64);
	}
	return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
	asm volatile(
	    "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
	    ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// the same tile asked into L2 only: no shared memory, no barrier, nothing waits for it
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
	asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
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
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "setp.ne.b32 p, %4, 0;\n\t"
	    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
	    ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
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

// 32-byte store (dst 32-byte aligned)
__device__ __forceinline__ void st_global_v8(int32_t* dst, const int (&v)[8]) {
	asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(v[0]), "r"(v[1]), "r"(v[2]),
	             "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
	             : "memory");
}

// One 32-column chunk of one output row: fold, LoRA delta, store, row max / argmax key.
// sfold: this tile's fold words in shared memory, {multiplier, shift, rounding half, identity}
// per column (or nullptr: no fold), indexed by column offset inside the tile.
__device__ __forceinline__ void epilogue_chunk(const LinearArgs& a, const uint32_t (&r)[32], int row, int n_base,
                                               int col_in_tile, const int4* sfold, const LoraLayerDev* lora,
                                               bool vec_ok, unsigned long long (&lmax)[3], unsigned long long& lbest) {
#pragma unroll
	for (int j4 = 0; j4 < 32; j4 += 4) {
		const int nb = n_base + j4;
		if (nb >= a.N) break;
		int64_t v4[4];
#pragma unroll
		for (int jj = 0; jj < 4; ++jj) {
			const int n = nb + jj;
			v4[jj] = 0;
			if (n >= a.N) continue;
			int32_t v32 = (int32_t)r[j4 + jj];
			if (sfold != nullptr) {
				const int4 f = sfold[col_in_tile + j4 + jj];
				v32 = fold(v32, f.w, f.x, f.y);
			}
			if (a.best != nullptr) {   // head: greedy argmax key, lowest index wins ties
				if (a.row_mask != nullptr) {
					const uint8_t* page = a.row_mask[row];
					if (page != nullptr && !((page[n >> 3] >> (n & 7)) & 1u)) v32 = INT32_MIN;
				}
				const unsigned long long key =
				    ((unsigned long long)((uint32_t)v32 ^ 0x80000000u) << 32) | (0xFFFFFFFFu - (uint32_t)n);
				lbest = key > lbest ? key : lbest;
				if (a.logits) a.logits[(size_t)row * a.N + n] = v32;
				continue;
			}
			int seg = 0;
			if (a.nseg > 1) {
				while (seg + 1 < a.nseg && n >= a.seg_end[seg]) ++seg;
			}
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
			v4[jj] = v;
			const unsigned long long ab = v < 0 ? (~(unsigned long long)v + 1ull) : (unsigned long long)v;
			if (seg == 0) lmax[0] = ab > lmax[0] ? ab : lmax[0];
			else if (seg == 1) lmax[1] = ab > lmax[1] ? ab : lmax[1];
			else lmax[2] = ab > lmax[2] ? ab : lmax[2];
		}
		if (a.best != nullptr) continue;
		if (vec_ok && nb + 3 < a.N) {
			*(int4*)((int32_t*)a.out + (size_t)row * a.out_ld + nb) = make_int4((int)v4[0], (int)v4[1], (int)v4[2], (int)v4[3]);
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

template <int MT, int BN>
__global__ void __launch_bounds__(kTcThreads, 1)
k_linear_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, LinearArgs a) {
	using Cfg = TcCfg<MT, BN>;
	constexpr int S = Cfg::kStages;
	extern __shared__ unsigned char smem_raw[];
	const uint32_t raw = smem_u32(smem_raw);
	const uint32_t base = (raw + 1023u) & ~1023u;            // SW128 tiles want 1024-byte alignment
	unsigned char* smem = smem_raw + (base - raw);
	int4* sfold = (int4*)(smem + S * Cfg::kStageBytes);                             // [2][BN]
	const uint32_t bars = base + S * Cfg::kStageBytes + Cfg::kFoldBytes;            // 8-byte slots
	auto full_bar = [&](int s) { return bars + 8u * s; };
	auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
	auto accf_bar = [&](int s) { return bars + 8u * (2 * S + s); };
	auto acce_bar = [&](int s) { return bars + 8u * (2 * S + 2 + s); };
	uint32_t* tmem_slot = (uint32_t*)(smem + S * Cfg::kStageBytes + Cfg::kFoldBytes + 8 * (2 * S + 4));
	__shared__ volatile int s_timeout;
	__shared__ volatile int s_stop[2];
	__shared__ volatile int s_last[2];

	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int kblocks = (a.K + BK - 1) / BK;
	const int n_tiles = (a.N + BN - 1) / BN;
	const int m_groups = (a.M + MT * BM - 1) / (MT * BM);
	const int tiles = n_tiles * m_groups;
	// split-K: work item w = (tile w % tiles, K slice w / tiles); slice s covers k-blocks
	// [s*kblocks/splits, (s+1)*kblocks/splits). The slices of a tile meet in global scratch.
	const int splits = a.splits > 1 ? a.splits : 1;
	const int items = tiles * splits;

	if (threadIdx.x == 0) {
		for (int s = 0; s < S; ++s) {
			mbar_init(full_bar(s), 1);
			mbar_init(empty_bar(s), 1);
		}
		for (int s = 0; s < 2; ++s) {
			mbar_init(accf_bar(s), 1);
			mbar_init(acce_bar(s), 8);       // one arrival per epilogue warp
		}
		s_timeout = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 1) {
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::kTmemCols));
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem_base = *tmem_slot;
	// everything above touched only this block's shared and tensor memory. The weights are not
	// written by any kernel either: while the previous kernel (a row kernel that moves little
	// data) finishes, the producer warp asks for the weight tiles of this block's work items
	// into L2, so the main loop's first loads do not start a cold trip to HBM. Only the block's
	// first work item: that is the whole weight matrix for the layer projections, and a bounded
	// part of the vocabulary head, which is larger than L2.
	if (warp == 0 && (int)blockIdx.x < items) {
		const int t = (int)blockIdx.x % tiles, ks = (int)blockIdx.x / tiles;
		const int n0 = (t / m_groups) * BN;
		const int kb0 = (int)((long long)ks * kblocks / splits), kb1 = (int)((long long)(ks + 1) * kblocks / splits);
		for (int kb = kb0 + lane; kb < kb1; kb += 32) tma_prefetch_2d(&map_b, kb * BK, n0);
	}
	// from here on the kernel reads what earlier kernels wrote
	pdl_wait();
	pdl_release();

	if (warp == 0) {
		if (lane == 0) {
			uint32_t it = 0;
			for (int w = blockIdx.x; w < items && s_timeout == 0; w += gridDim.x) {
				const int t = w % tiles, ks = w / tiles;
				const int m0 = (t % m_groups) * MT * BM, n0 = (t / m_groups) * BN;
				const int kb0 = (int)((long long)ks * kblocks / splits), kb1 = (int)((long long)(ks + 1) * kblocks / splits);
				for (int kb = kb0; kb < kb1; ++kb, ++it) {
					const int s = (int)(it % S);
					const uint32_t phase = (it / S) & 1u;
					if (!mbar_wait(empty_bar(s), phase ^ 1u)) { s_timeout = 1; break; }
					mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
					const uint32_t sa = base + s * Cfg::kStageBytes;
#pragma unroll
					for (int mt = 0; mt < MT; ++mt) tma_load_2d(sa + mt * BM * BK, &map_a, full_bar(s), kb * BK, m0 + mt * BM);
					// (tests of the bounded waits leave this one request out, once)
					if (!(a.debug_withhold != 0 && blockIdx.x == 0 && it == 0))
						tma_load_2d(sa + MT * BM * BK, &map_b, full_bar(s), kb * BK, n0);
				}
			}
		}
	} else if (warp == 1) {
		if (lane == 0) {
			uint32_t it = 0, tc = 0;
			for (int w = blockIdx.x; w < items && s_timeout == 0; w += gridDim.x, ++tc) {
				const uint32_t as = tc & 1u;
				const int ks = w / tiles;
				const int kb0 = (int)((long long)ks * kblocks / splits), kb1 = (int)((long long)(ks + 1) * kblocks / splits);
				if (!mbar_wait(acce_bar(as), ((tc >> 1) & 1u) ^ 1u)) { s_timeout = 1; break; }
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
				for (int kb = kb0; kb < kb1; ++kb, ++it) {
					const int s = (int)(it % S);
					const uint32_t phase = (it / S) & 1u;
					if (!mbar_wait(full_bar(s), phase)) {
						// the flag must be up before the commit below lets the epilogue look at this tile
						s_timeout = 1;
						__threadfence_block();
						break;
					}
					asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
					const uint32_t sa = base + s * Cfg::kStageBytes;
					const uint64_t db = umma_desc_sw128(sa + MT * BM * BK);
#pragma unroll
					for (int mt = 0; mt < MT; ++mt) {
						const uint64_t da = umma_desc_sw128(sa + mt * BM * BK);
						const uint32_t dcol = tmem_base + (as * MT + mt) * BN;
#pragma unroll
						for (int k = 0; k < BK / UMMA_K; ++k) {
							// advancing inside the 128-byte swizzle atom: +32 bytes = +2 descriptor units
							umma_i8(dcol, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), Cfg::kInstrDesc, (kb > kb0 || k != 0) ? 1u : 0u);
						}
					}
					umma_commit(empty_bar(s));     // frees the stage once these MMAs have read it
				}
				umma_commit(accf_bar(as));         // this tile's accumulators are complete
			}
		}
	} else {
		// epilogue: eight warps. Warp w reads TMEM lanes 32*(w%4)..+31, so this thread owns
		// rows m0 + mt*128 + 32*q + lane of every tile; the two warps of a lane quarter split
		// the tile's 32-column chunks between them (half = 0 / 1).
		const int q = warp & 3;
		const int half = (warp - 2) >> 2;
		const int et = threadIdx.x - 64;           // 0..255 within the epilogue group
		const bool vec_ok = !a.out64 && (a.out_ld & 3) == 0 && (((uintptr_t)a.out) & 15) == 0;
		// straight-line path: int32 rows, fold present, no adapters, not the head
		const bool fast_ok = vec_ok && a.fold != nullptr && a.rows == nullptr && a.best == nullptr;
		const bool wide_ok = (a.out_ld & 7) == 0 && (((uintptr_t)a.out) & 31) == 0;   // 32-byte stores line up
		uint32_t tc = 0;
		for (int w = blockIdx.x; w < items; w += gridDim.x, ++tc) {
			const uint32_t as = tc & 1u;
			const int t = w % tiles, ks = w / tiles;
			const int m0 = (t % m_groups) * MT * BM, n0 = (t / m_groups) * BN;
			int4* sf = nullptr;
			uint32_t odd_column = 0;                           // a column the one-rounding fold does not cover
			if (a.fold != nullptr) {
				sf = sfold + as * BN;
				for (int i = et; i < BN; i += kEpiThreads) {
					const int n = n0 + i;
					int4 f = make_int4(0, 0, 0, 0);
					if (n < a.N) {
						const int32_t* g = a.fold + (size_t)n * 3;
						const int32_t idn = g[0], mult = g[1], shift = g[2];
						const bool plain = fold_is_plain(idn, mult, shift);
						f = make_int4(mult, shift, (plain && shift > 0) ? (int)(1u << (shift - 1)) : 0, idn);
						if (!plain) odd_column = 1u;
					}
					sf[i] = f;
				}
			}
			if (et == 0) s_stop[as] = s_timeout;               // one thread decides, so all eight warps agree
			// fold words + stop flag visible to the epilogue warps; the barrier also tells every
			// thread whether any column of the tile needs the two-step fold
			uint32_t any_odd;
			asm volatile(
			    "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.or.pred p, 1, 256, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
			    : "=r"(any_odd)
			    : "r"(odd_column)
			    : "memory");
			if (s_stop[as] != 0) {
				if (a.status != nullptr) {
					for (int mt = 0; mt < MT; ++mt) {
						const int row = m0 + mt * BM + q * 32 + lane;
						if (row < a.M) atomicCAS(&a.status[row], 0, (int32_t)kInternalWaitTimeout);
					}
				}
				break;
			}
			// (the MMA thread commits a tile it gave up on as well, so that nobody waits out a second
			// limit: the flag, raised before that commit, says the accumulators are not the tile's)
			const bool acc_ok = mbar_wait(accf_bar(as), (tc >> 1) & 1u) && s_timeout == 0;
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
			if (!acc_ok) {
				s_timeout = 1;
				if (a.status != nullptr) {
					for (int mt = 0; mt < MT; ++mt) {
						const int row = m0 + mt * BM + q * 32 + lane;
						if (row < a.M) atomicCAS(&a.status[row], 0, (int32_t)kInternalWaitTimeout);
					}
				}
			}
			bool finish = true;                        // this block runs the tile's epilogue
			if (splits > 1) {
				// every K slice parks its raw accumulators in global scratch and then counts
				// itself in; the slice that arrives last adds the others to its own and runs
				// the epilogue. Nobody waits: the order of arrival decides the roles.
#pragma unroll
				for (int mt = 0; mt < MT; ++mt) {
					const int row = m0 + mt * BM + q * 32 + lane;
					if (m0 + mt * BM < a.M) {
						for (int c0 = half * 32; c0 < BN; c0 += 64) {
							uint32_t r[32];
							tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (as * MT + mt) * BN + c0, r);
								// scratch layout [slice][tile][mt][column quad][128 rows]: the 32 lanes of a
							// warp touch 512 contiguous bytes per access
							int4* dst = (int4*)a.partial +
							            ((((size_t)ks * tiles + t) * MT + mt) * (BN / 4) + (c0 >> 2)) * BM + q * 32 + lane;
#pragma unroll
							for (int j4 = 0; j4 < 32; j4 += 4)
								__stcg(dst + (size_t)(j4 >> 2) * BM, make_int4((int)r[j4], (int)r[j4 + 1], (int)r[j4 + 2], (int)r[j4 + 3]));
						}
					}
				}
				__threadfence();
				asm volatile("bar.sync 1, 256;" ::: "memory");
				if (et == 0) {
					const unsigned int old = atomicAdd(&a.tile_counters[t], 1u);
					const int last = old == (unsigned int)(splits - 1) ? 1 : 0;
					if (last) a.tile_counters[t] = 0u;          // all slices are in: zero for the next launch
					__threadfence();
					s_last[as] = last;
				}
				asm volatile("bar.sync 1, 256;" ::: "memory");
				finish = s_last[as] != 0;
			}
#pragma unroll
			for (int mt = 0; mt < MT; ++mt) {
				if (!finish) break;
				const int row = m0 + mt * BM + q * 32 + lane;
				const bool row_ok = acc_ok && row < a.M;
				const LoraLayerDev* lora =
				    (row_ok && a.rows != nullptr && a.rows[row].lora != nullptr) ? a.rows[row].lora + a.layer : nullptr;
				unsigned long long lmax[3] = {0ull, 0ull, 0ull};
				unsigned long long lbest = 0ull;
				int best_v = INT32_MIN, best_n = -1;
				if (m0 + mt * BM < a.M) {            // warp-uniform: the whole sub-tile is outside M otherwise
					for (int c0 = half * 32; c0 < BN; c0 += 64) {
						uint32_t r[32];
						tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (as * MT + mt) * BN + c0, r);   // warp-collective
						const int nb = n0 + c0;
						if (!row_ok || nb >= a.N) continue;
						if (splits > 1) {
							// the other slices' accumulators, three slices' loads in flight at a time
							constexpr int U = 3;
							const size_t slice_stride = (size_t)tiles * MT * (BN / 4) * BM;
							const int4* src0 = (const int4*)a.partial + (((size_t)t * MT + mt) * (BN / 4) + (c0 >> 2)) * BM + q * 32 + lane;
							for (int s0 = 0; s0 < splits; s0 += U) {
								int4 p[U][8];
#pragma unroll
								for (int u = 0; u < U; ++u) {
									const int s2 = s0 + u;
									const bool live = s2 < splits && s2 != ks;
#pragma unroll
									for (int j = 0; j < 8; ++j)
										p[u][j] = live ? __ldcg(src0 + (size_t)s2 * slice_stride + (size_t)j * BM) : make_int4(0, 0, 0, 0);
								}
#pragma unroll
								for (int u = 0; u < U; ++u) {
#pragma unroll
									for (int j = 0; j < 8; ++j) {
										r[4 * j] += (uint32_t)p[u][j].x;
										r[4 * j + 1] += (uint32_t)p[u][j].y;
										r[4 * j + 2] += (uint32_t)p[u][j].z;
										r[4 * j + 3] += (uint32_t)p[u][j].w;
									}
								}
							}
						}
						const bool full = nb + 32 <= a.N;
						if (a.best != nullptr && a.fold == nullptr && a.logits == nullptr && full) {
							// head: running (value, index) maximum; columns ascend, so a strict
							// comparison keeps the lowest index among equals
							uint32_t allowed = 0xFFFFFFFFu;      // the 32 mask bits of this chunk's columns
							if (a.row_mask != nullptr) {
								const uint8_t* page = a.row_mask[row];
								if (page != nullptr) {
									const uint8_t* pb = page + (nb >> 3);
									allowed = (uint32_t)pb[0] | ((uint32_t)pb[1] << 8) | ((uint32_t)pb[2] << 16) | ((uint32_t)pb[3] << 24);
								}
							}
#pragma unroll
							for (int j = 0; j < 32; ++j) {
								const int v = ((allowed >> j) & 1u) ? (int)r[j] : INT32_MIN;
								const bool gt = v > best_v;
								best_v = gt ? v : best_v;
								best_n = gt ? nb + j : best_n;
							}
							continue;
						}
						int seg = 0;
						while (seg + 1 < a.nseg && nb >= a.seg_end[seg]) ++seg;
						if (fast_ok && any_odd == 0u && full && nb + 32 <= a.seg_end[seg]) {
							// one segment, whole chunk inside N, every column on the one-rounding fold:
							// no branches, one shared-memory word load per element, and the fold's
							// magnitude doubles as the row-maximum candidate
							uint32_t mx = 0;
							int32_t* dst = (int32_t*)a.out + (size_t)row * a.out_ld + nb;
#pragma unroll
							for (int j8 = 0; j8 < 32; j8 += 8) {
								int v[8];
#pragma unroll
								for (int jj = 0; jj < 8; ++jj) {
									const int4 f = sf[c0 + j8 + jj];
									uint32_t mag;
									v[jj] = fold_plain((int32_t)r[j8 + jj], f.x, f.y, (uint32_t)f.z, &mag);
									mx = mag > mx ? mag : mx;
								}
								// a thread owns a row, so a warp's store touches 32 different lines: the
								// 32-byte form halves the number of requests the row's 128 bytes take
								if (wide_ok) {
									st_global_v8(dst + j8, v);
								} else {
									*(int4*)(dst + j8) = make_int4(v[0], v[1], v[2], v[3]);
									*(int4*)(dst + j8 + 4) = make_int4(v[4], v[5], v[6], v[7]);
								}
							}
							if (seg == 0) lmax[0] = mx > lmax[0] ? mx : lmax[0];
							else if (seg == 1) lmax[1] = mx > lmax[1] ? mx : lmax[1];
							else lmax[2] = mx > lmax[2] ? mx : lmax[2];
						} else {
							epilogue_chunk(a, r, row, nb, c0, sf, lora, vec_ok, lmax, lbest);
						}
					}
				}
				if (row_ok) {
					if (best_n >= 0) {
						const unsigned long long key =
						    ((unsigned long long)((uint32_t)best_v ^ 0x80000000u) << 32) | (0xFFFFFFFFu - (uint32_t)best_n);
						lbest = key > lbest ? key : lbest;
					}
					if (a.best != nullptr && lbest != 0ull) atomicMax(&a.best[row], lbest);
					if (a.rowmax != nullptr && a.best == nullptr) {
						for (int s = 0; s < a.nseg; ++s)
							if (a.seg_slot[s] >= 0 && lmax[s] != 0ull) atomicMax(&a.rowmax[(size_t)row * 4 + a.seg_slot[s]], lmax[s]);
					}
				}
			}
			asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
			__syncwarp();
			if (lane == 0) mbar_arrive(acce_bar(as));          // accumulator stage may be overwritten
		}
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (warp == 1) {
		asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols));
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
	int rows, k, box_rows;
	bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && k == o.k && box_rows == o.box_rows; }
};
struct MapKeyHash {
	size_t operator()(const MapKey& k) const {
		return std::hash<const void*>()(k.p) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.k << 40) ^ ((size_t)k.box_rows << 20);
	}
};

// [rows, K] int8 row-major -> 2-D map, box = 128 bytes x box_rows rows, 128-byte swizzle, zero fill
bool tensor_map(const void* ptr, int rows, int k, int box_rows, CUtensorMap* out) {
	static std::mutex mu;
	static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
	const MapKey key{ptr, rows, k, box_rows};
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
	const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
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

// K slices per output tile: only when the tiles alone would leave SMs idle, never fewer than
// eight 128-wide k-blocks per slice (a shorter main loop is cheaper than the exchange), and
// only as many as the scratch can hold.
template <int MT, int BN>
int pick_splits(const LinearArgs& a, int tiles) {
	if (a.partial == nullptr || a.tile_counters == nullptr || tiles > a.n_tile_counters) return 1;
	const int kblocks = (a.K + BK - 1) / BK;
	int s = sm_count() / tiles;
	if (s > kblocks / 8) s = kblocks / 8;
	if (s > 8) s = 8;
	// tuning override: SSLM_B200_TC_SPLITS=n caps the slices (1 turns splitting off)
	static const int cap = [] {
		const char* e = getenv("SSLM_B200_TC_SPLITS");
		return e ? atoi(e) : 0;
	}();
	if (cap > 0 && s > cap) s = cap;
	const size_t per_slice = (size_t)tiles * MT * BM * BN * 4;
	while (s > 1 && (size_t)s * per_slice > a.partial_bytes) --s;
	return s < 2 ? 1 : s;
}

std::atomic<int> g_debug_withhold{0};

template <int MT, int BN>
bool launch_cfg(const LinearArgs& a_in, cudaStream_t st) {
	using Cfg = TcCfg<MT, BN>;
	LinearArgs a = a_in;
	static PerDeviceOnce configured;
	if (once_per_device(configured, [] {
		    return cudaFuncSetAttribute(k_linear_tc<MT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes);
	    }) != cudaSuccess) {
		g_tc_last_reason.store(2);
		return false;
	}
	CUtensorMap ma, mb;
	if (!tensor_map(a.x, a.M, a.K, BM, &ma) || !tensor_map(a.w, a.N, a.K, BN, &mb)) {
		g_tc_last_reason.store(encode_fn() ? 4 : 3);
		return false;
	}
	const int tiles = ((a.N + BN - 1) / BN) * ((a.M + MT * BM - 1) / (MT * BM));
	a.splits = pick_splits<MT, BN>(a, tiles);
	{
		int left = g_debug_withhold.load();
		a.debug_withhold = 0;
		while (left > 0 && !g_debug_withhold.compare_exchange_weak(left, left - 1)) {}
		if (left > 0) a.debug_withhold = 1;
	}
	const int items = tiles * a.splits;
	const int grid = items < sm_count() ? items : sm_count();
	if (launch_pdl(k_linear_tc<MT, BN>, dim3(grid), dim3(kTcThreads), Cfg::kSmemBytes, st, ma, mb, a) != cudaSuccess) {
		g_tc_last_reason.store(5);
		return false;
	}
	return true;
}

}  // namespace

void tc_stats(unsigned long long* launches, unsigned long long* refusals, int* last_reason) {
	*launches = g_tc_launches.load();
	*refusals = g_tc_refusals.load();
	*last_reason = g_tc_last_reason.load();
}
void tc_variant_counts(unsigned long long* counts, int n) {
	for (int i = 0; i < n; ++i) counts[i] = i < 8 ? g_tc_variant[i].load() : 0ull;
}
static bool tc_refuse(int reason) {
	g_tc_refusals.fetch_add(1);
	g_tc_last_reason.store(reason);
	return false;
}

void tc_debug_withhold(int launches) { g_debug_withhold.store(launches < 0 ? 0 : launches); }

bool launch_linear_tc(const LinearArgs& a, cudaStream_t st) {
	if (a.K % 16 != 0 || ((uintptr_t)a.x & 15) || ((uintptr_t)a.w & 15)) return tc_refuse(1);
	// two accumulators per weight tile once there is more than one 128-row group -- unless the
	// output is so small that even 128-row tiles leave SMs idle: then the smaller tile doubles
	// the blocks and halves each block's main loop bytes and epilogue (the second read of a
	// weight tile hits L2). Narrower weight tiles when there would otherwise be clearly fewer tiles
	// than SMs (below 90 % of them; SSLM_B200_TC_NARROW_PCT moves that): every tile re-reads the
	// activation rows from L2, so halving the tile width doubles that traffic, and at 140 tiles
	// on 148 SMs (the gate/up projection of the 1.5B shape) one wide tile per block is faster
	// than two narrow ones even though the narrow ones overlap their epilogues.
	const int n128 = (a.N + 127) / 128;
	const bool two = a.M > BM && n128 * ((a.M + 127) / 128) >= sm_count();
	const int tiles128 = ((a.N + 127) / 128) * ((a.M + (two ? 255 : 127)) / (two ? 256 : 128));
	static const int narrow_pct = [] {
		const char* e = getenv("SSLM_B200_TC_NARROW_PCT");
		return e ? atoi(e) : 90;
	}();
	// (a prefill chunk of several hundred rows has enough work per tile that the wide tile wins
	// until the tiles are fewer than a quarter of the SMs: measured on the 1.5B projections)
	const bool narrow = tiles128 * 100 < sm_count() * (a.M <= 2 * BM ? narrow_pct : (narrow_pct < 25 ? narrow_pct : 25));
	bool ok;
	if (two) ok = narrow ? launch_cfg<2, 64>(a, st) : launch_cfg<2, 128>(a, st);
	else ok = narrow ? launch_cfg<1, 64>(a, st) : launch_cfg<1, 128>(a, st);
	if (!ok) return tc_refuse(g_tc_last_reason.load() ? g_tc_last_reason.load() : 9);
	g_tc_launches.fetch_add(1);
	g_tc_variant[(two ? 2 : 0) + (narrow ? 0 : 1)].fetch_add(1);
	return true;
}

}  // namespace sslm
