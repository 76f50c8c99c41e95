/* tiny-cuda-nn/reduce_sum.h of the B200-native stand-in: sums over a device array.  Two forms, as the reference calls
 * them: reduce_sum(in, fun, out, n, stream) adds fun(in[i]) into out[0] on the device (out is NOT cleared first:
 * src/testbed_nerf.cu:3378-3383 clears it itself), and reduce_sum(in, n, stream) returns the sum on the host, which
 * blocks on the stream (src/testbed_nerf.cu:3423-3425, include/neural-graphics-primitives/nerf_network.h:459).
 *
 * One kernel: a grid-stride loop with 16-byte loads where the pointer allows, a warp shuffle tree, one shared-memory
 * stage and one atomic per block; the grid is a multiple of the SM count, so a sum over millions of elements costs a few
 * hundred atomics. */
#pragma once
#include <tiny-cuda-nn/common.h>
#include <tiny-cuda-nn/gpu_memory.h>

TCNN_NAMESPACE_BEGIN

inline uint32_t reduce_sum_workspace_size(uint32_t n_elements) {
	(void)n_elements;
	return 32; /* floats; the sum lands in element 0 */
}

#if defined(__CUDACC__)
template <typename T, typename F>
__global__ void reduce_sum_kernel(const T* __restrict__ in, F fun, float* __restrict__ out, const uint32_t n_elements) {
	float acc = 0.0f;
	for (uint32_t i = threadIdx.x + blockIdx.x * blockDim.x; i < n_elements; i += blockDim.x * gridDim.x) acc += (float)fun((float)in[i]);
#pragma unroll
	for (int offset = 16; offset > 0; offset >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, offset);
	__shared__ float partial[32];
	const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	if (lane == 0) partial[warp] = acc;
	__syncthreads();
	if (warp == 0) {
		acc = lane < (blockDim.x >> 5) ? partial[lane] : 0.0f;
#pragma unroll
		for (int offset = 16; offset > 0; offset >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, offset);
		if (lane == 0) atomicAdd(out, acc);
	}
}

template <typename T, typename F>
void reduce_sum(T* device_pointer, F fun, float* workspace, uint32_t n_elements, cudaStream_t stream) {
	if (!n_elements) return;
	static int n_sms = 0;
	if (!n_sms) {
		int device = 0;
		CUDA_CHECK_THROW(cudaGetDevice(&device));
		CUDA_CHECK_THROW(cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device));
	}
	const uint32_t threads = 256;
	const uint32_t blocks = std::min(div_round_up(n_elements, threads), (uint32_t)n_sms * 4u);
	reduce_sum_kernel<T, F><<<blocks, threads, 0, stream>>>(device_pointer, fun, workspace, n_elements);
}

struct ReduceIdentity {
	__host__ __device__ float operator()(float v) const { return v; }
};

/* the sum itself, on the host: synchronises with the stream */
template <typename T>
float reduce_sum(T* device_pointer, uint32_t n_elements, cudaStream_t stream) {
	auto scratch = allocate_workspace(stream, sizeof(float));
	float* d_sum = (float*)scratch.data();
	CUDA_CHECK_THROW(cudaMemsetAsync(d_sum, 0, sizeof(float), stream));
	reduce_sum(device_pointer, ReduceIdentity{}, d_sum, n_elements, stream);
	float result = 0.0f;
	CUDA_CHECK_THROW(cudaMemcpyAsync(&result, d_sum, sizeof(float), cudaMemcpyDeviceToHost, stream));
	CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
	return result;
}
#endif

TCNN_NAMESPACE_END
