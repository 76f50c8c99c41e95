// 64-neuron ReLU MLP forward on tcgen05 / TMEM (the tcnn FullyFusedMLP::forward of the reference, nerf_network.h:212,271).
// A CTA of 128 threads owns a tile of 128 samples: thread t stages row t of the input into shared memory (core-matrix
// layout), one thread issues the layer's tcgen05.mma chain (M = 128, N = 64 | 16, K = 48 | 64), the accumulator sits in
// tensor memory, every thread then pulls its own row out with tcgen05.ld, applies ReLU, rounds to fp16 and writes it back
// to shared memory as the next layer's A operand.  Weights stay resident in shared memory for the CTA's lifetime.
#include "common.cuh"
#include "tc05.cuh"

namespace n2b {

template <int IN, int NH>
struct TcMlpSmem {
	__half W1[64 * IN];
	__half W2[NH == 2 ? 64 * 64 : 8];
	__half Wo[16 * 64];
	__half X[128 * IN];
	__half H0[128 * 64];
	__half H1[NH == 2 ? 128 * 64 : 8];
	uint64_t mbar;
	uint32_t tmem_base;
	uint32_t pad;
};

__device__ __forceinline__ uint32_t sptr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ReLU + round the thread's 64 accumulator columns to fp16 and store row `row` of a blocked [128][64] tile.
__device__ __forceinline__ void epilogue_hidden(uint32_t taddr, int row, __half* tile, __half* gdst) {
#pragma unroll
	for (int c0 = 0; c0 < 64; c0 += 16) {
		float v[16];
		tc::tmem_ld16(taddr + c0, v);
		tc::tmem_ld_wait();
		__align__(16) __half h[16];
#pragma unroll
		for (int e = 0; e < 16; ++e) h[e] = __float2half_rn(fmaxf(v[e], 0.f));
		*reinterpret_cast<uint4*>(reinterpret_cast<char*>(tile) + tc::blk_off(row, c0, 64)) = reinterpret_cast<const uint4*>(h)[0];
		*reinterpret_cast<uint4*>(reinterpret_cast<char*>(tile) + tc::blk_off(row, c0 + 8, 64)) = reinterpret_cast<const uint4*>(h)[1];
		if (gdst) {
			reinterpret_cast<uint4*>(gdst + c0)[0] = reinterpret_cast<const uint4*>(h)[0];
			reinterpret_cast<uint4*>(gdst + c0)[1] = reinterpret_cast<const uint4*>(h)[1];
		}
	}
}

template <int IN, int NH>
__global__ void __launch_bounds__(128) mlp_forward_tc_kernel(uint32_t n, const __half* __restrict__ weights, const __half* __restrict__ in,
                                                             __half* __restrict__ out, __half* __restrict__ hidden,
                                                             uint32_t* __restrict__ status) {
	extern __shared__ __align__(128) unsigned char smem_raw[];
	auto& sm = *reinterpret_cast<TcMlpSmem<IN, NH>*>(smem_raw);
	const int tid = threadIdx.x, warp = tid >> 5;
	// stage the weights in blocked K-major layout
	for (int e = tid; e < 64 * IN; e += 128)
		*reinterpret_cast<__half*>(reinterpret_cast<char*>(sm.W1) + tc::blk_off(e / IN, e % IN, IN)) = weights[e];
	if (NH == 2)
		for (int e = tid; e < 64 * 64; e += 128)
			*reinterpret_cast<__half*>(reinterpret_cast<char*>(sm.W2) + tc::blk_off(e / 64, e % 64, 64)) = weights[64 * IN + e];
	const int off_o = 64 * IN + (NH - 1) * 4096;
	for (int e = tid; e < 16 * 64; e += 128)
		*reinterpret_cast<__half*>(reinterpret_cast<char*>(sm.Wo) + tc::blk_off(e / 64, e % 64, 64)) = weights[off_o + e];
	if (tid == 0) tc::mbar_init(sptr(&sm.mbar), 1);
	if (warp == 0) tc::tmem_alloc(sptr(&sm.tmem_base), 128);
	tc::fence_before_sync();
	__syncthreads();
	tc::fence_after_sync();
	const uint32_t tmem = sm.tmem_base;
	const uint32_t lane_base = (uint32_t)(warp * 32) << 16;  // this warp's 32 tensor-memory lanes
	uint32_t phase = 0;
	bool ok = true;
	const uint32_t n_tiles = (n + 127u) / 128u;
	for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
		const uint32_t row = tile * 128u + tid;
		// ---- stage the input row
#pragma unroll
		for (int c = 0; c < IN; c += 8) {
			uint4 v = make_uint4(0, 0, 0, 0);
			if (row < n) v = *reinterpret_cast<const uint4*>(in + (size_t)row * IN + c);
			*reinterpret_cast<uint4*>(reinterpret_cast<char*>(sm.X) + tc::blk_off(tid, c, IN)) = v;
		}
		tc::fence_async_smem();
		tc::fence_before_sync();
		__syncthreads();
		// ---- layer 1: [128][IN] x W1^T -> TMEM columns [0, 64)
		if (tid == 0) {
			tc::fence_after_sync();
			tc::issue_gemm_kmajor<64, IN>(tmem, sptr(sm.X), sptr(sm.W1));
			tc::commit(sptr(&sm.mbar));
		}
		ok = tc::mbar_wait(sptr(&sm.mbar), phase);
		phase ^= 1u;
		if (!ok) break;
		tc::fence_after_sync();
		epilogue_hidden(tmem + lane_base, tid, sm.H0, (hidden && row < n) ? hidden + (size_t)row * NH * 64 : nullptr);
		const __half* last = sm.H0;
		if (NH == 2) {
			tc::fence_async_smem();
			tc::fence_before_sync();
			__syncthreads();
			if (tid == 0) {
				tc::fence_after_sync();
				tc::issue_gemm_kmajor<64, 64>(tmem + 64, sptr(sm.H0), sptr(sm.W2));
				tc::commit(sptr(&sm.mbar));
			}
			ok = tc::mbar_wait(sptr(&sm.mbar), phase);
			phase ^= 1u;
			if (!ok) break;
			tc::fence_after_sync();
			epilogue_hidden(tmem + 64 + lane_base, tid, sm.H1, (hidden && row < n) ? hidden + (size_t)row * NH * 64 + 64 : nullptr);
			last = sm.H1;
		}
		tc::fence_async_smem();
		tc::fence_before_sync();
		__syncthreads();
		// ---- output layer: N = 16 -> TMEM columns [0, 16)
		if (tid == 0) {
			tc::fence_after_sync();
			tc::issue_gemm_kmajor<16, 64>(tmem, sptr(last), sptr(sm.Wo));
			tc::commit(sptr(&sm.mbar));
		}
		ok = tc::mbar_wait(sptr(&sm.mbar), phase);
		phase ^= 1u;
		if (!ok) break;
		tc::fence_after_sync();
		{
			float v[16];
			tc::tmem_ld16(tmem + lane_base, v);
			tc::tmem_ld_wait();
			if (row < n) {
				__align__(16) __half h[16];
#pragma unroll
				for (int e = 0; e < 16; ++e) h[e] = __float2half_rn(v[e]);
				reinterpret_cast<uint4*>(out + (size_t)row * 16)[0] = reinterpret_cast<const uint4*>(h)[0];
				reinterpret_cast<uint4*>(out + (size_t)row * 16)[1] = reinterpret_cast<const uint4*>(h)[1];
			}
		}
		tc::fence_before_sync();
		__syncthreads();  // tensor memory and the tiles are free for the next round
	}
	if (!ok && status) atomicOr(status, 1u);
	tc::fence_before_sync();
	__syncthreads();
	if (warp == 0) tc::tmem_dealloc(tmem, 128);
}

template <int IN, int NH>
static int run_tc(uint32_t n, const uint16_t* w, const uint16_t* in, uint16_t* out, uint16_t* hidden, uint32_t* status, cudaStream_t s) {
	const size_t smem = sizeof(TcMlpSmem<IN, NH>) + 128;
	N2B_CHECK_CUDA(cudaFuncSetAttribute(mlp_forward_tc_kernel<IN, NH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	uint32_t ctas = (n + 127u) / 128u;
	if (ctas > 2u * kSMs) ctas = 2u * kSMs;
	mlp_forward_tc_kernel<IN, NH><<<ctas, 128, smem, s>>>(n, (const __half*)w, (const __half*)in, (__half*)out, (__half*)hidden, status);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

}  // namespace n2b

using namespace n2b;

extern "C" int neus2b_mlp_forward_tcgen05(uint32_t n, uint32_t in_width, uint32_t n_hidden, const uint16_t* d_weights, const uint16_t* d_in,
                                          uint16_t* d_out, uint16_t* d_hidden, uint32_t* d_status, neus2b_stream_t stream) {
	if (!d_weights || !d_in || !d_out) return NEUS2B_E_INVALID;
	if (((uintptr_t)d_in | (uintptr_t)d_out | (uintptr_t)d_hidden) & 15u) return NEUS2B_E_INVALID;
	if (n == 0) return NEUS2B_OK;
	if (in_width == 48 && n_hidden == 1) return run_tc<48, 1>(n, d_weights, d_in, d_out, d_hidden, d_status, stream);
	if (in_width == 48 && n_hidden == 2) return run_tc<48, 2>(n, d_weights, d_in, d_out, d_hidden, d_status, stream);
	if (in_width == 64 && n_hidden == 2) return run_tc<64, 2>(n, d_weights, d_in, d_out, d_hidden, d_status, stream);
	return NEUS2B_E_UNSUPPORTED;
}
