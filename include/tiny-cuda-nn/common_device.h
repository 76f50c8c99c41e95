/* tiny-cuda-nn/common_device.h of the B200-native stand-in: the small device-side vocabulary the reference's kernels use --
 * vector_t<T, N> (an aligned pack moved with one load or store), scalar helpers, Morton codes of the occupancy grid.
 * Call sites followed: src/testbed_nerf.cu:231, :978, :1568, :1948 (vector_t), :330-420 (morton3D, morton3D_invert,
 * logistic, clamp), include/neural-graphics-primitives/takikawa_encoding.cuh:79-140, envmap.cuh:50-94. */
#pragma once
#include <tiny-cuda-nn/common.h>

#include <type_traits>

TCNN_NAMESPACE_BEGIN

static constexpr float PI = 3.14159265358979323846f;
static constexpr float SQRT2 = 1.41421356237309504880f;

template <typename T>
struct PitchedPtr {
	TCNN_HOST_DEVICE PitchedPtr() : ptr{nullptr}, stride_in_bytes{sizeof(T)} {}
	TCNN_HOST_DEVICE PitchedPtr(T* ptr, size_t stride_in_elements, size_t offset = 0, size_t extra_stride_bytes = 0)
	    : ptr{ptr + offset}, stride_in_bytes{(uint32_t)(stride_in_elements * sizeof(T) + extra_stride_bytes)} {}
	template <typename U>
	TCNN_HOST_DEVICE explicit PitchedPtr(PitchedPtr<U> other) : ptr{(T*)other.ptr}, stride_in_bytes{other.stride_in_bytes} {}
	TCNN_HOST_DEVICE T* operator()(uint32_t y) const { return (T*)((const char*)ptr + y * stride_in_bytes); }
	TCNN_HOST_DEVICE void operator+=(uint32_t y) { ptr = (T*)((const char*)ptr + y * stride_in_bytes); }
	TCNN_HOST_DEVICE void operator-=(uint32_t y) { ptr = (T*)((const char*)ptr - y * stride_in_bytes); }
	TCNN_HOST_DEVICE explicit operator bool() const { return ptr; }
	T* ptr;
	uint32_t stride_in_bytes;
};

#if defined(__CUDACC__)
inline __host__ __device__ float logistic(const float x) { return 1.0f / (1.0f + expf(-x)); }
inline __host__ __device__ float logit(const float x) { return -logf(1.0f / (fminf(fmaxf(x, 1e-9f), 1.0f - 1e-9f)) - 1.0f); }
inline __host__ __device__ float smoothstep(float val) { return val * val * (3.0f - 2.0f * val); }
inline __host__ __device__ float smoothstep_derivative(float val) { return 6 * val * (1.0f - val); }
inline __host__ __device__ float smoothstep_2nd_derivative(float val) { return 6.0f - 12.0f * val; }
inline __host__ __device__ float identity_fun(float val) { return val; }
inline __host__ __device__ float identity_derivative(float) { return 1.0f; }
inline __host__ __device__ float identity_2nd_derivative(float) { return 0.0f; }

/* 10 bits spread to every third bit */
inline __host__ __device__ uint32_t expand_bits(uint32_t v) {
	v = (v * 0x00010001u) & 0xFF0000FFu;
	v = (v * 0x00000101u) & 0x0F00F00Fu;
	v = (v * 0x00000011u) & 0xC30C30C3u;
	v = (v * 0x00000005u) & 0x49249249u;
	return v;
}
inline __host__ __device__ uint32_t morton3D(uint32_t x, uint32_t y, uint32_t z) { return expand_bits(x) | (expand_bits(y) << 1) | (expand_bits(z) << 2); }
inline __host__ __device__ uint32_t morton3D_invert(uint32_t x) {
	x = x & 0x49249249u;
	x = (x | (x >> 2)) & 0xc30c30c3u;
	x = (x | (x >> 4)) & 0x0f00f00fu;
	x = (x | (x >> 8)) & 0xff0000ffu;
	x = (x | (x >> 16)) & 0x0000ffffu;
	return x;
}

template <typename T>
__device__ T warp_reduce(T val) {
#pragma unroll
	for (int offset = 16; offset > 0; offset >>= 1) val += __shfl_xor_sync(0xffffffffu, val, offset);
	return val;
}

/* A compacted batch of *n_input_elements_ptr records (stride values each) is repeated until it fills n_elements records, so
 * that the following kernels run on a full batch (src/testbed_nerf.cu:3908-3916). */
template <typename T>
__global__ void fill_rollover(const uint32_t n_elements, const uint32_t stride, const uint32_t* __restrict__ n_input_elements_ptr, T* inout) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	const uint32_t n_output = n_elements * stride;
	const uint32_t n_input = min(*n_input_elements_ptr, n_elements) * stride;
	if (i < n_input || i >= n_output || n_input == 0) return;
	inout[i] = inout[i % n_input];
}
/* the same for a gradient: every copy, the original included, is scaled by n_input / n_output, so that the repeated batch
 * carries the gradient of the compacted one */
template <typename T>
__global__ void fill_rollover_and_rescale(const uint32_t n_elements, const uint32_t stride, const uint32_t* __restrict__ n_input_elements_ptr, T* inout) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	const uint32_t n_output = n_elements * stride;
	const uint32_t n_input = min(*n_input_elements_ptr, n_elements) * stride;
	if (i >= n_input) return;
	/* one thread per source element writes the element and all its copies: no thread reads what another one writes */
	const float scaled = (float)inout[i] * (float)n_input / (float)n_output;
	for (uint32_t j = i; j < n_output; j += n_input) inout[j] = (T)scaled;
}

template <typename T>
__global__ void cast_kernel(const uint32_t n, const float* __restrict__ in, T* __restrict__ out) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i < n) out[i] = (T)in[i];
}
template <typename T>
__global__ void cast_from_kernel(const uint32_t n, const T* __restrict__ in, float* __restrict__ out) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i < n) out[i] = (float)in[i];
}
template <typename T>
__global__ void add_kernel(const uint32_t n, const T* __restrict__ in, T* __restrict__ out) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i < n) out[i] = (T)((float)out[i] + (float)in[i]);
}
#endif

TCNN_NAMESPACE_END
