// sslm_b200_linear_resident: the standalone int8 linear layer (projection, per-channel
// fold, per-row requant funnel) for operands that already live in device memory, written
// so that the call itself allocates nothing on the host or the device.
//
// Who needs that: a caller that has handed every byte of HBM to its own pools (a serving
// process whose KV pool takes what the weights leave), and a caller that issues work from
// a spot where a device-wide stall is not acceptable. cudaMalloc and cudaFree make the
// whole device wait and may fail late, so such callers reserve memory once at start-up and
// afterwards use only entry points that work inside what they were given.
//
// The layer needs one piece of scratch between its two kernels: per row, the largest
// folded magnitude, which the projection kernel reduces with atomicMax and the funnel
// kernel turns into the row's dynamic scale. Here that scratch is a fixed array in the
// library's own device image (g_row_peak below), not an allocation. Its address is looked
// up once per device, by the first call made with that device current: that first call
// does the set-up (cudaGetSymbolAddress, and the driver's one-time attribute calls for the
// kernels), so make it before any stream capture begins.
//
// Rules that follow from one shared array:
//   * every slot must read zero when a call starts. The array is zero when the module is
//     loaded, and the funnel kernel of this file writes zero back into every slot it
//     consumed, so back-to-back calls on one stream need no clearing in between;
//   * two calls whose kernels can overlap in time (different streams, or different host
//     threads on the same device) race on the array. Give such calls an order.
//   * at most kResidentMaxRows rows per call; more is refused with SSLM_INVALID_ARGUMENT.
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/sslm_b200.h"
#include "sslm_kernels.h"

// The scratch: 4 slots of 8 bytes per row (the projection kernels index row * 4 + slot; this
// layer uses slot 0), 256 rows = 8 KiB of device image. All zero at module load and after
// every completed call.
static __device__ __align__(256) unsigned long long g_row_peak[SSLM_B200_RESIDENT_MAX_ROWS * 4];

namespace sslm {
namespace {

constexpr int kResidentMaxRows = SSLM_B200_RESIDENT_MAX_ROWS;
constexpr int kResidentMaxK = 16384;        // the streaming kernel stages 8 activation rows in shared memory

// Funnel of the projected rows (FunnelProjectedRow's tail, src/forward/forward_sites.cpp:
// 1114-1146): the same arithmetic as the funnel behind sslm_b200_linear, reading the row
// peak from the fixed array and leaving the slot zero for the next call.
__global__ void __launch_bounds__(256)
k_resident_funnel(const int32_t* wide, int n, unsigned long long* row_peak, const Scale* in_scales, Scale site,
                  int8_t* codes, Scale* out_scales, int32_t* status) {
	__shared__ unsigned long long s_peak;
	const int r = blockIdx.x;
	if (threadIdx.x == 0) {
		s_peak = row_peak[(size_t)r * 4];
		row_peak[(size_t)r * 4] = 0ull;
	}
	__syncthreads();
	const FunnelParams fp = funnel_params(s_peak, &in_scales[r], 1, site);
	if (threadIdx.x == 0) {
		if (status != nullptr && status[r] == 0) status[r] = fp.status;
		if (out_scales != nullptr) out_scales[r] = fp.out;
	}
	if (fp.status != kOk || codes == nullptr) return;
	for (int i = threadIdx.x; i < n; i += blockDim.x)
		codes[(size_t)r * n + i] = requant_code((int64_t)wide[(size_t)r * n + i], fp.r, fp.s);
}

// device address of g_row_peak, per device ordinal; resolved by the first call on a device
// (host threads may race through that first call: they all store the same address)
std::atomic<unsigned long long*> g_peak_addr[kMaxDevices];

}  // namespace
}  // namespace sslm

using namespace sslm;

extern "C" sslm_status sslm_b200_linear_resident(const int8_t* d_x, const int8_t* d_w, const int32_t* d_fold,
                                                 int32_t M, int32_t N, int32_t K, const int64_t* d_in_scales,
                                                 int64_t site_m, int64_t site_e, int32_t* d_out_folded,
                                                 int8_t* d_out_codes, int64_t* d_out_scales,
                                                 int32_t* d_row_status, void* stream) {
	if (!d_x || !d_w || !d_fold || !d_in_scales || !d_out_folded) return SSLM_INVALID_ARGUMENT;
	if (M < 1 || N < 1 || K < 16 || K % 16 != 0) return SSLM_INVALID_ARGUMENT;
	if (M > kResidentMaxRows || K > kResidentMaxK) return SSLM_INVALID_ARGUMENT;   // beyond the fixed scratch
	if (((uintptr_t)d_x & 15) || ((uintptr_t)d_w & 15) || ((uintptr_t)d_out_folded & 15)) return SSLM_MISALIGNED_BUFFER;
	// the remaining arrays are read and written as 4- and 8-byte words
	if (((uintptr_t)d_fold & 3) || ((uintptr_t)d_row_status & 3) || ((uintptr_t)d_in_scales & 7) ||
	    ((uintptr_t)d_out_scales & 7))
		return SSLM_MISALIGNED_BUFFER;
	int dev = -1;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SSLM_ALLOCATION_FAILED;
	unsigned long long* peak = g_peak_addr[dev].load(std::memory_order_acquire);
	if (peak == nullptr) {
		// set-up, once per device: where this device keeps its copy of the array
		void* p = nullptr;
		if (cudaGetSymbolAddress(&p, g_row_peak) != cudaSuccess || p == nullptr) return SSLM_ALLOCATION_FAILED;
		peak = (unsigned long long*)p;
		g_peak_addr[dev].store(peak, std::memory_order_release);
	}
	cudaStream_t st = (cudaStream_t)stream;
	if (d_row_status != nullptr && cudaMemsetAsync(d_row_status, 0, (size_t)M * 4, st) != cudaSuccess)
		return SSLM_ALLOCATION_FAILED;

	LinearArgs a{};
	a.x = d_x; a.w = d_w; a.fold = d_fold;
	a.M = M; a.N = N; a.K = K;
	a.out = d_out_folded; a.out_ld = N; a.out64 = 0;
	a.rowmax = peak;
	a.nseg = 1;
	a.seg_end[0] = a.seg_end[1] = a.seg_end[2] = N;
	a.seg_slot[0] = 0; a.seg_slot[1] = a.seg_slot[2] = -1;
	a.seg_lora[0] = a.seg_lora[1] = a.seg_lora[2] = -1;
	a.status = d_row_status;
	// nothing ran yet if the projection's launch is refused: the array still reads zero
	if (launch_linear_gemv(a, st) != cudaSuccess) return SSLM_ALLOCATION_FAILED;
	k_resident_funnel<<<M, 256, 0, st>>>(d_out_folded, N, peak, (const Scale*)d_in_scales, Scale{site_m, site_e},
	                                     d_out_codes, (Scale*)d_out_scales, d_row_status);
	if (cudaGetLastError() != cudaSuccess) {
		// The projection is enqueued and will leave its row peaks in the array, but the kernel that
		// consumes and clears them is not: clear the rows this call used, in stream order, so the
		// next call on this device starts from zero all the same.
		cudaMemsetAsync(peak, 0, (size_t)M * 4 * sizeof(unsigned long long), st);
		return SSLM_ALLOCATION_FAILED;
	}
	return SSLM_OK;
}
