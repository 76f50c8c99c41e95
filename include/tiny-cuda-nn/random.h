/* tiny-cuda-nn/random.h of the B200-native stand-in: the pcg32 generator (M. O'Neill's published PCG-XSH-RR 64/32
 * algorithm, restated) usable on host and device, and helpers that fill device arrays with draws of it.  The reference
 * uses it as default_rng_t for sampling training pixels and jittering rays (src/testbed_nerf.cu:1370-1400,
 * include/neural-graphics-primitives/random_val.cuh) and for parameter initialisation (nerf_network.h:805-875). */
#pragma once
#include <tiny-cuda-nn/common.h>
#include <tiny-cuda-nn/gpu_memory.h>

#include <cmath>

#define PCG32_DEFAULT_STATE 0x853c49e6748fea9bULL
#define PCG32_DEFAULT_STREAM 0xda3e39cb94b95bdbULL
#define PCG32_MULT 0x5851f42d4c957f2dULL

TCNN_NAMESPACE_BEGIN

struct pcg32 {
	TCNN_HOST_DEVICE pcg32() : state(PCG32_DEFAULT_STATE), inc(PCG32_DEFAULT_STREAM) {}
	TCNN_HOST_DEVICE pcg32(uint64_t initstate, uint64_t initseq = 1u) { seed(initstate, initseq); }

	TCNN_HOST_DEVICE void seed(uint64_t initstate, uint64_t initseq = 1) {
		state = 0u;
		inc = (initseq << 1u) | 1u;
		next_uint();
		state += initstate;
		next_uint();
	}
	TCNN_HOST_DEVICE uint32_t next_uint() {
		const uint64_t old = state;
		state = old * PCG32_MULT + inc;
		const uint32_t xorshifted = (uint32_t)(((old >> 18u) ^ old) >> 27u);
		const uint32_t rot = (uint32_t)(old >> 59u);
		return (xorshifted >> rot) | (xorshifted << ((~rot + 1u) & 31));
	}
	/* unbiased draw from [0, bound) */
	TCNN_HOST_DEVICE uint32_t next_uint(uint32_t bound) {
		const uint32_t threshold = (~bound + 1u) % bound;
		for (;;) {
			const uint32_t r = next_uint();
			if (r >= threshold) return r % bound;
		}
	}
	/* [0, 1) with 23 random mantissa bits */
	TCNN_HOST_DEVICE float next_float() {
		union {
			uint32_t u;
			float f;
		} x;
		x.u = (next_uint() >> 9) | 0x3f800000u;
		return x.f - 1.0f;
	}
	TCNN_HOST_DEVICE double next_double() {
		union {
			uint64_t u;
			double d;
		} x;
		x.u = ((uint64_t)next_uint() << 20) | 0x3ff0000000000000ULL;
		return x.d - 1.0;
	}
	/* jumps the sequence by delta draws in O(log delta) (F. Brown's published LCG skip-ahead) */
	TCNN_HOST_DEVICE void advance(int64_t delta_ = (1ll << 32)) {
		uint64_t cur_mult = PCG32_MULT, cur_plus = inc, acc_mult = 1u, acc_plus = 0u;
		uint64_t delta = (uint64_t)delta_;
		while (delta > 0) {
			if (delta & 1) {
				acc_mult *= cur_mult;
				acc_plus = acc_plus * cur_mult + cur_plus;
			}
			cur_plus = (cur_mult + 1) * cur_plus;
			cur_mult *= cur_mult;
			delta /= 2;
		}
		state = acc_mult * state + acc_plus;
	}
	TCNN_HOST_DEVICE bool operator==(const pcg32& other) const { return state == other.state && inc == other.inc; }
	TCNN_HOST_DEVICE bool operator!=(const pcg32& other) const { return !(*this == other); }

	uint64_t state, inc;
};

using default_rng_t = pcg32;

static constexpr uint32_t N_RANDOM_VALS_PER_THREAD = 4;

#if defined(__CUDACC__)
template <typename T, typename RNG>
__global__ void generate_random_uniform_kernel(const size_t n_elements, RNG rng, T* __restrict__ out, const T lower, const T upper) {
	const size_t i = threadIdx.x + (size_t)blockIdx.x * blockDim.x;
	const size_t first = i * N_RANDOM_VALS_PER_THREAD;
	if (first >= n_elements) return;
	rng.advance((int64_t)first);
#pragma unroll
	for (uint32_t k = 0; k < N_RANDOM_VALS_PER_THREAD; ++k) {
		if (first + k >= n_elements) return;
		out[first + k] = (T)(rng.next_float() * (float)(upper - lower) + (float)lower);
	}
}
template <typename T, typename RNG>
__global__ void generate_random_logistic_kernel(const size_t n_elements, RNG rng, T* __restrict__ out, const T mean, const T stddev) {
	const size_t i = threadIdx.x + (size_t)blockIdx.x * blockDim.x;
	const size_t first = i * N_RANDOM_VALS_PER_THREAD;
	if (first >= n_elements) return;
	rng.advance((int64_t)first);
	const float scale = (float)stddev * 0.551328895f; /* sqrt(3) / pi: variance of the logistic distribution */
#pragma unroll
	for (uint32_t k = 0; k < N_RANDOM_VALS_PER_THREAD; ++k) {
		if (first + k >= n_elements) return;
		const float u = fminf(fmaxf(rng.next_float(), 1e-7f), 1.0f - 1e-7f);
		out[first + k] = (T)(logf(u / (1.0f - u)) * scale + (float)mean);
	}
}

/* fills out[0, n) on the device with uniform draws of [lower, upper) and moves rng past them */
template <typename T, typename RNG>
void generate_random_uniform(cudaStream_t stream, RNG& rng, size_t n_elements, T* out, const T lower = (T)0.0, const T upper = (T)1.0) {
	if (!n_elements) return;
	const size_t n_threads = div_round_up(n_elements, (size_t)N_RANDOM_VALS_PER_THREAD);
	generate_random_uniform_kernel<T, RNG><<<n_blocks_linear(n_threads), n_threads_linear, 0, stream>>>(n_elements, rng, out, lower, upper);
	rng.advance((int64_t)n_elements);
}
template <typename T, typename RNG>
void generate_random_uniform(RNG& rng, size_t n_elements, T* out, const T lower = (T)0.0, const T upper = (T)1.0) {
	generate_random_uniform(nullptr, rng, n_elements, out, lower, upper);
}
template <typename T, typename RNG>
void generate_random_logistic(cudaStream_t stream, RNG& rng, size_t n_elements, T* out, const T mean = (T)0.0, const T stddev = (T)1.0) {
	if (!n_elements) return;
	const size_t n_threads = div_round_up(n_elements, (size_t)N_RANDOM_VALS_PER_THREAD);
	generate_random_logistic_kernel<T, RNG><<<n_blocks_linear(n_threads), n_threads_linear, 0, stream>>>(n_elements, rng, out, mean, stddev);
	rng.advance((int64_t)n_elements);
}
template <typename T, typename RNG>
void generate_random_logistic(RNG& rng, size_t n_elements, T* out, const T mean = (T)0.0, const T stddev = (T)1.0) {
	generate_random_logistic(nullptr, rng, n_elements, out, mean, stddev);
}
#endif

TCNN_NAMESPACE_END
