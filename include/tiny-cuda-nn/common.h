/* tiny-cuda-nn/common.h of the B200-native stand-in for the reference's un-vendored tiny-cuda-nn fork
 * (dependencies/neus2_tcnn, CMakeLists.txt:88-92): the host-side vocabulary the reference's sources use from this header --
 * namespace macros, error checks, enums, launch helpers, small utilities.  Interfaces follow the call sites in
 * src/testbed_nerf.cu, src/testbed.cu and include/neural-graphics-primitives/*.h; the bodies are this library's own. */
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cctype>
#include <array>
#include <cstdint>
#include <functional>
#include <iostream>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#define TCNN_NAMESPACE_BEGIN namespace tcnn {
#define TCNN_NAMESPACE_END }

#if defined(__CUDACC__)
#define TCNN_HOST_DEVICE __host__ __device__
#define TCNN_DEVICE __device__
#else
#define TCNN_HOST_DEVICE
#define TCNN_DEVICE
#endif

#ifndef TCNN_MIN_GPU_ARCH
#define TCNN_MIN_GPU_ARCH 100 /* this implementation is written for sm_100a only */
#endif

#define TCNN_STRINGIFY(x) #x
#define TCNN_STR(x) TCNN_STRINGIFY(x)
#define TCNN_FILE_LINE __FILE__ ":" TCNN_STR(__LINE__)

/* the reference's error convention: CUDA errors become std::runtime_error (src/testbed_nerf.cu, everywhere) */
#define CUDA_CHECK_THROW(x)                                                                                                  \
	do {                                                                                                                     \
		cudaError_t _tcnn_result = (x);                                                                                      \
		if (_tcnn_result != cudaSuccess)                                                                                     \
			throw std::runtime_error(std::string(TCNN_FILE_LINE " " #x " failed with error ") + cudaGetErrorString(_tcnn_result)); \
	} while (0)
#define CUDA_CHECK_PRINT(x)                                                                                                  \
	do {                                                                                                                     \
		cudaError_t _tcnn_result = (x);                                                                                      \
		if (_tcnn_result != cudaSuccess)                                                                                     \
			std::cout << TCNN_FILE_LINE " " #x " failed with error " << cudaGetErrorString(_tcnn_result) << std::endl;        \
	} while (0)
#define CU_CHECK_THROW(x) CUDA_CHECK_THROW((cudaError_t)(x))

TCNN_NAMESPACE_BEGIN

static constexpr uint32_t MIN_GPU_ARCH = TCNN_MIN_GPU_ARCH;
using network_precision_t = __half; /* TCNN_HALF_PRECISION: the networks run in fp16 */

enum class Activation { ReLU, Exponential, Sine, Sigmoid, Squareplus, Softplus, None };
enum class GridType { Hash, Dense, Tiled };
enum class InterpolationType { Nearest, Linear, Smoothstep };
enum class MatrixLayout { RowMajor = 0, SoA = 0, ColumnMajor = 1, AoS = 1 };
static constexpr MatrixLayout RM = MatrixLayout::RowMajor, SoA = MatrixLayout::SoA, CM = MatrixLayout::ColumnMajor, AoS = MatrixLayout::AoS;
enum class EGradientMode { Ignore = 0, Overwrite = 1, Accumulate = 2 };

inline std::string to_lower(std::string str) {
	std::transform(str.begin(), str.end(), str.begin(), [](unsigned char c) { return (char)std::tolower(c); });
	return str;
}
inline std::string to_upper(std::string str) {
	std::transform(str.begin(), str.end(), str.begin(), [](unsigned char c) { return (char)std::toupper(c); });
	return str;
}
inline bool equals_case_insensitive(const std::string& a, const std::string& b) { return to_lower(a) == to_lower(b); }

inline Activation string_to_activation(const std::string& s) {
	static const std::pair<const char*, Activation> names[] = {{"none", Activation::None},         {"relu", Activation::ReLU},
	                                                            {"exponential", Activation::Exponential}, {"sigmoid", Activation::Sigmoid},
	                                                            {"sine", Activation::Sine},         {"squareplus", Activation::Squareplus},
	                                                            {"softplus", Activation::Softplus}};
	for (const auto& n : names)
		if (to_lower(s) == n.first) return n.second;
	throw std::runtime_error("Invalid activation name: " + s);
}
inline std::string to_string(Activation a) {
	switch (a) {
		case Activation::None: return "None";
		case Activation::ReLU: return "ReLU";
		case Activation::Exponential: return "Exponential";
		case Activation::Sigmoid: return "Sigmoid";
		case Activation::Sine: return "Sine";
		case Activation::Squareplus: return "Squareplus";
		case Activation::Softplus: return "Softplus";
	}
	throw std::runtime_error("Invalid activation");
}
inline InterpolationType string_to_interpolation_type(const std::string& s) {
	if (equals_case_insensitive(s, "Nearest")) return InterpolationType::Nearest;
	if (equals_case_insensitive(s, "Linear")) return InterpolationType::Linear;
	if (equals_case_insensitive(s, "Smoothstep")) return InterpolationType::Smoothstep;
	throw std::runtime_error("Invalid interpolation type: " + s);
}
inline std::string to_string(InterpolationType t) {
	switch (t) {
		case InterpolationType::Nearest: return "Nearest";
		case InterpolationType::Linear: return "Linear";
		case InterpolationType::Smoothstep: return "Smoothstep";
	}
	throw std::runtime_error("Invalid interpolation type");
}

inline int cuda_device() {
	int device = 0;
	CUDA_CHECK_THROW(cudaGetDevice(&device));
	return device;
}
inline uint32_t cuda_compute_capability(int device = -1) {
	if (device < 0) device = cuda_device();
	int major = 0, minor = 0;
	CUDA_CHECK_THROW(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
	CUDA_CHECK_THROW(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
	return (uint32_t)(major * 10 + minor);
}

template <typename T>
TCNN_HOST_DEVICE T div_round_up(T val, T divisor) {
	return (val + divisor - 1) / divisor;
}
template <typename T>
TCNN_HOST_DEVICE T next_multiple(T val, T divisor) {
	return div_round_up(val, divisor) * divisor;
}
template <typename T>
TCNN_HOST_DEVICE T previous_multiple(T val, T divisor) {
	return (val / divisor) * divisor;
}
template <typename T>
constexpr TCNN_HOST_DEVICE bool is_pot(T val) {
	return (val & (val - 1)) == 0;
}
inline constexpr TCNN_HOST_DEVICE uint32_t next_pot(uint32_t v) {
	--v;
	v |= v >> 1;
	v |= v >> 2;
	v |= v >> 4;
	v |= v >> 8;
	v |= v >> 16;
	return v + 1;
}
template <typename T>
TCNN_HOST_DEVICE void host_device_swap(T& a, T& b) {
	T c(a);
	a = b;
	b = c;
}
template <typename T>
TCNN_HOST_DEVICE T clamp(T val, T lower, T upper) {
	return val < lower ? lower : (upper < val ? upper : val);
}

constexpr uint32_t batch_size_granularity = 128;
constexpr uint32_t n_threads_linear = 128;

template <typename T>
constexpr uint32_t n_blocks_linear(T n_elements) {
	return (uint32_t)div_round_up(n_elements, (T)n_threads_linear);
}

#if defined(__CUDACC__)
/* kernel(n_elements, args...) over a 1-D grid of n_threads_linear-wide blocks */
template <typename K, typename T, typename... Types>
inline void linear_kernel(K kernel, uint32_t shmem_size, cudaStream_t stream, T n_elements, Types... args) {
	if (n_elements <= 0) return;
	kernel<<<n_blocks_linear(n_elements), n_threads_linear, shmem_size, stream>>>((uint32_t)n_elements, args...);
}

template <typename F>
__global__ void parallel_for_kernel(const size_t n_elements, F fun) {
	const size_t i = threadIdx.x + (size_t)blockIdx.x * blockDim.x;
	if (i >= n_elements) return;
	fun(i);
}
template <typename F>
inline void parallel_for_gpu(uint32_t shmem_size, cudaStream_t stream, size_t n_elements, F&& fun) {
	if (n_elements <= 0) return;
	parallel_for_kernel<F><<<n_blocks_linear(n_elements), n_threads_linear, shmem_size, stream>>>(n_elements, fun);
}
template <typename F>
inline void parallel_for_gpu(cudaStream_t stream, size_t n_elements, F&& fun) {
	parallel_for_gpu(0, stream, n_elements, std::forward<F>(fun));
}
template <typename F>
inline void parallel_for_gpu(size_t n_elements, F&& fun) {
	parallel_for_gpu(nullptr, n_elements, std::forward<F>(fun));
}
#endif

/* runs a callable when it goes out of scope (src/testbed.cu:2662) */
class ScopeGuard {
public:
	ScopeGuard() = default;
	ScopeGuard(const std::function<void()>& callback) : m_callback{callback} {}
	ScopeGuard(std::function<void()>&& callback) : m_callback{std::move(callback)} {}
	ScopeGuard& operator=(const ScopeGuard&) = delete;
	ScopeGuard(const ScopeGuard&) = delete;
	ScopeGuard& operator=(ScopeGuard&& other) {
		std::swap(m_callback, other.m_callback);
		return *this;
	}
	ScopeGuard(ScopeGuard&& other) { *this = std::move(other); }
	~ScopeGuard() {
		if (m_callback) m_callback();
	}
	void disarm() { m_callback = {}; }

private:
	std::function<void()> m_callback;
};

/* N elements of T in one aligned object (alignment: the pack's size up to 16 bytes), so that a pack travels in one transaction */
template <typename T, uint32_t N_ELEMS>
struct alignas(sizeof(T) * N_ELEMS > 16 ? 16 : sizeof(T) * N_ELEMS) vector_t {
	TCNN_HOST_DEVICE T& operator[](uint32_t idx) { return data[idx]; }
	TCNN_HOST_DEVICE T operator[](uint32_t idx) const { return data[idx]; }
	T data[N_ELEMS];
	static constexpr uint32_t N = N_ELEMS;
};
template <uint32_t N_FLOATS>
using vector_fullp_t = vector_t<float, N_FLOATS>;
template <uint32_t N_HALFS>
using vector_halfp_t = vector_t<__half, N_HALFS>;

template <typename T>
std::string bytes_to_string(T bytes) {
	static const char* suffixes[] = {"B", "KB", "MB", "GB", "TB"};
	double v = (double)bytes;
	int i = 0;
	for (; i < 4 && v >= 1024.0; ++i) v /= 1024.0;
	std::ostringstream o;
	o.precision(2);
	o << std::fixed << v << " " << suffixes[i];
	return o.str();
}

TCNN_NAMESPACE_END

#if defined(__CUDACC__)
/* include/neural-graphics-primitives/nerf_network.h:1088, :1206, :1248 call this unqualified from namespace ngp inside a
 * class template, where a using-directive that appears later in the translation unit is not seen */
using tcnn::parallel_for_gpu;
#endif
