/* C++ host side above the C ABI, shaped like the tiny-cuda-nn objects that NerfNetwork holds for the NeuS training
 * step (include/neural-graphics-primitives/nerf_network.h:36-130: m_pos_encoding, m_density_network, m_rgb_network,
 * m_dir_encoding), with the virtual signatures NerfNetwork itself overrides (nerf_network.h:87, :132, :317-326) and the
 * reference's error convention (exceptions; CUDA_CHECK_THROW).  Header-only; link with libneus2b and cudart.
 *
 * What is mirrored: MatrixLayout, EGradientMode, GPUMemory<T>, GPUMatrixDynamic<T>, Context, Encoding<T>,
 * GridEncoding<T> (hash grid, 2 features per level), SphericalHarmonicsEncoding<T> (degree 4), Network<T>,
 * FullyFusedMLP<T> (64 neurons, ReLU, 16 padded outputs, 1 or 2 hidden layers) and NeusAdamOptimizer (the
 * Ema(ExponentialDecay(Adam)) chain of configs/nerf/base.json as one pass).  T is __half.  Matrices are column-major
 * ("AoS": one sample contiguous), which is the ABI's layout.
 * What is not: the json configuration layer, the memory arena, the out-of-scope encodings and losses. */
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "neus2b.h"

namespace tcnn {

enum class MatrixLayout { RowMajor = 0, SoA = 0, ColumnMajor = 1, AoS = 1 };
static constexpr MatrixLayout RM = MatrixLayout::RowMajor, CM = MatrixLayout::ColumnMajor;
enum class EGradientMode { Ignore = NEUS2B_GRAD_IGNORE, Overwrite = NEUS2B_GRAD_OVERWRITE, Accumulate = NEUS2B_GRAD_ACCUMULATE };

#ifndef CUDA_CHECK_THROW
#define CUDA_CHECK_THROW(x)                                                                                        \
	do {                                                                                                           \
		cudaError_t _e = (x);                                                                                      \
		if (_e != cudaSuccess) throw std::runtime_error(std::string(#x " failed: ") + cudaGetErrorString(_e));      \
	} while (0)
#endif

/* A non-zero return of the C ABI becomes the exception the reference's callers expect. */
inline void neus2b_check(int rc, const char* what) {
	if (rc != 0) throw std::runtime_error(std::string(what) + ": " + neus2b_error_string(rc));
}

template <typename T>
class GPUMemory {
public:
	GPUMemory() = default;
	explicit GPUMemory(size_t n) { resize(n); }
	GPUMemory(const GPUMemory&) = delete;
	GPUMemory& operator=(const GPUMemory&) = delete;
	GPUMemory(GPUMemory&& o) noexcept : m_data(o.m_data), m_size(o.m_size) { o.m_data = nullptr, o.m_size = 0; }
	~GPUMemory() { cudaFree(m_data); }
	void resize(size_t n) {
		if (n == m_size) return;
		free_memory();
		if (n) CUDA_CHECK_THROW(cudaMalloc((void**)&m_data, n * sizeof(T)));
		m_size = n;
	}
	void enlarge(size_t n) {
		if (n > m_size) resize(n);
	}
	void free_memory() {
		if (m_data) CUDA_CHECK_THROW(cudaFree(m_data));
		m_data = nullptr, m_size = 0;
	}
	void memset(int value) { CUDA_CHECK_THROW(cudaMemset(m_data, value, get_bytes())); }
	void copy_from_host(const T* host, size_t n) {
		if (n > m_size) throw std::runtime_error("GPUMemory::copy_from_host: too many elements");
		CUDA_CHECK_THROW(cudaMemcpy(m_data, host, n * sizeof(T), cudaMemcpyHostToDevice));
	}
	void copy_from_host(const std::vector<T>& host) { copy_from_host(host.data(), host.size()); }
	void resize_and_copy_from_host(const std::vector<T>& host) {
		resize(host.size());
		copy_from_host(host);
	}
	void copy_to_host(T* host, size_t n) const {
		if (n > m_size) throw std::runtime_error("GPUMemory::copy_to_host: too many elements");
		CUDA_CHECK_THROW(cudaMemcpy(host, m_data, n * sizeof(T), cudaMemcpyDeviceToHost));
	}
	void copy_to_host(std::vector<T>& host) const {
		host.resize(m_size);
		copy_to_host(host.data(), m_size);
	}
	T* data() const { return m_data; }
	size_t size() const { return m_size; }
	size_t get_bytes() const { return m_size * sizeof(T); }

private:
	T* m_data = nullptr;
	size_t m_size = 0;
};

/* m rows (features) x n columns (samples).  Column-major: column j starts at data + j * stride. */
template <typename T>
class GPUMatrixDynamic {
public:
	GPUMatrixDynamic(T* data, uint32_t m, uint32_t n, MatrixLayout layout = CM, uint32_t stride = 0)
	    : m_data(data), m_rows(m), m_cols(n), m_layout(layout), m_stride(stride ? stride : (layout == CM ? m : n)) {}
	GPUMatrixDynamic(uint32_t m, uint32_t n, MatrixLayout layout = CM)
	    : m_owned(std::make_shared<GPUMemory<T>>((size_t)m * n)), m_data(m_owned->data()), m_rows(m), m_cols(n), m_layout(layout),
	      m_stride(layout == CM ? m : n) {}
	T* data() const { return m_data; }
	uint32_t m() const { return m_rows; }
	uint32_t n() const { return m_cols; }
	uint32_t rows() const { return m_rows; }
	uint32_t cols() const { return m_cols; }
	uint32_t stride() const { return m_stride; }
	MatrixLayout layout() const { return m_layout; }
	size_t n_elements() const { return (size_t)m_rows * m_cols; }
	size_t n_bytes() const { return n_elements() * sizeof(T); }
	void memset_async(cudaStream_t stream, int value) { CUDA_CHECK_THROW(cudaMemsetAsync(m_data, value, n_bytes(), stream)); }
	GPUMatrixDynamic<T> slice_rows(uint32_t offset, uint32_t size) const {  // column-major only: a band of features of every sample
		if (m_layout != CM) throw std::runtime_error("GPUMatrixDynamic::slice_rows: column-major matrices only");
		return GPUMatrixDynamic<T>(m_data + offset, size, m_cols, CM, m_stride);
	}

private:
	std::shared_ptr<GPUMemory<T>> m_owned;
	T* m_data;
	uint32_t m_rows, m_cols;
	MatrixLayout m_layout;
	uint32_t m_stride;
};

struct Context {
	virtual ~Context() {}
};

inline void require_cm(MatrixLayout l, const char* who) {
	if (l != CM) throw std::runtime_error(std::string(who) + ": column-major (AoS) matrices only");
}

/* ---- Encoding<T>: float input, T output (tiny-cuda-nn/encoding.h as NerfNetwork uses it) */
template <typename T>
class Encoding {
public:
	virtual ~Encoding() {}
	virtual std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>* output = nullptr,
	                                              bool use_inference_params = false, bool prepare_input_gradients = false) = 0;
	virtual void backward_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<float>& input, const GPUMatrixDynamic<T>& output,
	                           const GPUMatrixDynamic<T>& dL_doutput, GPUMatrixDynamic<float>* dL_dinput = nullptr,
	                           bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) = 0;
	std::unique_ptr<Context> forward(cudaStream_t s, const GPUMatrixDynamic<float>& in, GPUMatrixDynamic<T>* out = nullptr, bool inf = false,
	                                 bool prep = false) {
		return forward_impl(s, in, out, inf, prep);
	}
	void backward(cudaStream_t s, const Context& c, const GPUMatrixDynamic<float>& in, const GPUMatrixDynamic<T>& out, const GPUMatrixDynamic<T>& dL,
	              GPUMatrixDynamic<float>* dL_din = nullptr, bool inf = false, EGradientMode mode = EGradientMode::Overwrite) {
		backward_impl(s, c, in, out, dL, dL_din, inf, mode);
	}
	virtual void set_params(T* params, T* inference_params, T* backward_params, T* gradients) {
		m_params = params, m_inference_params = inference_params, m_gradients = gradients;
		(void)backward_params;
	}
	virtual size_t n_params() const = 0;
	virtual uint32_t input_width() const = 0;
	virtual uint32_t padded_output_width() const = 0;
	virtual uint32_t output_width() const { return padded_output_width(); }
	virtual MatrixLayout preferred_output_layout() const { return CM; }
	T* params() const { return m_params; }
	T* gradients() const { return m_gradients; }

protected:
	T *m_params = nullptr, *m_inference_params = nullptr, *m_gradients = nullptr;
};

template <typename T>
class GridEncoding : public Encoding<T> {
public:
	struct ForwardContext : public Context {
		GPUMemory<float> dy_dx;  // [n][2L][3], kept when prepare_input_gradients
	};
	/* n_levels, log2_hashmap_size, base_resolution, per_level_scale as in the "encoding" block of configs/nerf/base.json:29-39 */
	GridEncoding(uint32_t n_levels, uint32_t log2_hashmap_size, uint32_t base_resolution, float per_level_scale) {
		m_desc = neus2b_grid_desc{n_levels, log2_hashmap_size, base_resolution, per_level_scale, n_levels};
		uint64_t n = 0;
		neus2b_check(neus2b_grid_n_params(&m_desc, &n), "GridEncoding");
		m_n_params = (size_t)n;
	}
	std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>* output, bool use_inference_params,
	                                      bool prepare_input_gradients) override {
		require_cm(input.layout(), "GridEncoding::forward");
		auto ctx = std::make_unique<ForwardContext>();
		if (!output) return ctx;
		require_cm(output->layout(), "GridEncoding::forward");
		if (output->stride() != padded_output_width()) throw std::runtime_error("GridEncoding::forward: output must be dense");
		if (prepare_input_gradients) ctx->dy_dx.resize((size_t)input.n() * padded_output_width() * 3);
		const T* p = use_inference_params ? this->m_inference_params : this->m_params;
		neus2b_check(neus2b_grid_forward(&m_desc, input.n(), input.data(), input.stride(), (const uint16_t*)p, (uint16_t*)output->data(),
		                                 prepare_input_gradients ? ctx->dy_dx.data() : nullptr, stream),
		             "GridEncoding::forward");
		return ctx;
	}
	void backward_impl(cudaStream_t stream, const Context&, const GPUMatrixDynamic<float>& input, const GPUMatrixDynamic<T>&,
	                   const GPUMatrixDynamic<T>& dL_doutput, GPUMatrixDynamic<float>* dL_dinput, bool use_inference_params,
	                   EGradientMode param_gradients_mode) override {
		require_cm(input.layout(), "GridEncoding::backward");
		const T* p = use_inference_params ? this->m_inference_params : this->m_params;
		if (dL_dinput)
			neus2b_check(neus2b_grid_backward_input(&m_desc, input.n(), input.data(), input.stride(), (const uint16_t*)p,
			                                        (const uint16_t*)dL_doutput.data(), dL_dinput->data(), stream),
			             "GridEncoding::backward (input)");
		if (param_gradients_mode != EGradientMode::Ignore)
			neus2b_check(neus2b_grid_backward_params(&m_desc, input.n(), input.data(), input.stride(), (const uint16_t*)dL_doutput.data(),
			                                         (uint16_t*)this->m_gradients, (int)param_gradients_mode, stream),
			             "GridEncoding::backward (params)");
	}
	/* nerf_network.h:534-544: dL_ddLdinput = dL/d(dy/dx) [3 x n] float, dL_doutput of the first-order pass [2L x n] */
	void backward_backward_input(cudaStream_t stream, const Context&, const GPUMatrixDynamic<float>& input, const GPUMatrixDynamic<float>& dL_ddLdinput,
	                             const GPUMatrixDynamic<T>& dL_doutput, GPUMatrixDynamic<T>* dL_ddLdoutput, GPUMatrixDynamic<float>* dL_dinput = nullptr,
	                             bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		if (dL_dinput) throw std::runtime_error("GridEncoding::backward_backward_input: dL_dinput is not part of the NeuS step");
		const T* p = use_inference_params ? this->m_inference_params : this->m_params;
		neus2b_check(neus2b_grid_backward_backward_input(&m_desc, input.n(), input.data(), input.stride(), (const uint16_t*)p, dL_ddLdinput.data(),
		                                                 (const uint16_t*)dL_doutput.data(), dL_ddLdoutput ? (uint16_t*)dL_ddLdoutput->data() : nullptr,
		                                                 (uint16_t*)this->m_gradients, (int)param_gradients_mode, stream),
		             "GridEncoding::backward_backward_input");
	}
	/* progressive training (nerf_network.h:97-110): number of levels that take part */
	void set_n_active_levels(uint32_t n) { m_desc.n_active_levels = n < m_desc.n_levels ? n : m_desc.n_levels; }
	size_t n_params() const override { return m_n_params; }
	uint32_t input_width() const override { return 3; }
	uint32_t padded_output_width() const override { return 2 * m_desc.n_levels; }
	const neus2b_grid_desc& desc() const { return m_desc; }

private:
	neus2b_grid_desc m_desc;
	size_t m_n_params = 0;
};

template <typename T>
class SphericalHarmonicsEncoding : public Encoding<T> {
public:
	std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>* output, bool, bool) override {
		require_cm(input.layout(), "SphericalHarmonicsEncoding::forward");
		if (output)
			neus2b_check(neus2b_sh4_forward(input.n(), input.data(), input.stride(), (uint16_t*)output->data(), stream), "SphericalHarmonicsEncoding::forward");
		return std::make_unique<Context>();
	}
	void backward_impl(cudaStream_t, const Context&, const GPUMatrixDynamic<float>&, const GPUMatrixDynamic<T>&, const GPUMatrixDynamic<T>&,
	                   GPUMatrixDynamic<float>* dL_dinput, bool, EGradientMode) override {
		if (dL_dinput) throw std::runtime_error("SphericalHarmonicsEncoding: the NeuS step takes no gradient with respect to the view direction");
	}
	size_t n_params() const override { return 0; }
	uint32_t input_width() const override { return 3; }
	uint32_t padded_output_width() const override { return 16; }
};

/* ---- Network<T>: T input, T output (tiny-cuda-nn/network.h as NerfNetwork uses m_density_network / m_rgb_network) */
template <typename T>
class FullyFusedMLP {
public:
	struct ForwardContext : public Context {
		GPUMemory<T> hidden;  // [n][n_hidden][64]
	};
	/* 64 neurons, ReLU, no output activation, 16 padded outputs: the two networks of configs/nerf/base.json:63-80 */
	FullyFusedMLP(uint32_t input_width, uint32_t n_hidden_layers) : m_in(input_width), m_hidden(n_hidden_layers) {
		if ((input_width != 48 && input_width != 32 && input_width != 64) || n_hidden_layers < 1 || n_hidden_layers > 2)
			throw std::runtime_error("FullyFusedMLP: unsupported shape");
	}
	void inference_mixed_precision_impl(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<T>& output, bool use_inference_params = true) {
		require_cm(input.layout(), "FullyFusedMLP::inference");
		const T* p = use_inference_params ? m_inference_params : m_params;
		neus2b_check(neus2b_mlp_forward(input.n(), m_in, m_hidden, (const uint16_t*)p, (const uint16_t*)input.data(), (uint16_t*)output.data(), nullptr, stream),
		             "FullyFusedMLP::inference");
	}
	std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<T>* output = nullptr,
	                                      bool use_inference_params = false, bool prepare_input_gradients = false) {
		(void)prepare_input_gradients;
		require_cm(input.layout(), "FullyFusedMLP::forward");
		auto ctx = std::make_unique<ForwardContext>();
		if (!output) return ctx;
		ctx->hidden.resize((size_t)input.n() * m_hidden * 64);
		const T* p = use_inference_params ? m_inference_params : m_params;
		neus2b_check(neus2b_mlp_forward(input.n(), m_in, m_hidden, (const uint16_t*)p, (const uint16_t*)input.data(), (uint16_t*)output->data(),
		                                (uint16_t*)ctx->hidden.data(), stream),
		             "FullyFusedMLP::forward");
		return ctx;
	}
	void backward_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<T>&, const GPUMatrixDynamic<T>& dL_doutput,
	                   GPUMatrixDynamic<T>* dL_dinput = nullptr, bool use_inference_params = false,
	                   EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		const auto& c = dynamic_cast<const ForwardContext&>(ctx);
		const T* p = use_inference_params ? m_inference_params : m_params;
		neus2b_check(neus2b_mlp_backward(input.n(), m_in, m_hidden, (const uint16_t*)p, (const uint16_t*)input.data(), (const uint16_t*)c.hidden.data(),
		                                 (const uint16_t*)dL_doutput.data(), dL_dinput ? (uint16_t*)dL_dinput->data() : nullptr,
		                                 param_gradients_mode == EGradientMode::Ignore ? nullptr : m_gradients, (int)param_gradients_mode, stream),
		             "FullyFusedMLP::backward");
	}
	/* nerf_network.h:560-571, one hidden layer: dL_ddLdinput = dL/d(dL_dinput) [in x n], dL_doutput of the differentiated pass */
	void backward_backward_input(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<T>&, const GPUMatrixDynamic<T>& dL_ddLdinput,
	                             const GPUMatrixDynamic<T>& dL_doutput, GPUMatrixDynamic<T>* dL_ddLdoutput = nullptr, GPUMatrixDynamic<T>* dL_dinput = nullptr,
	                             bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		if (dL_ddLdoutput || dL_dinput) throw std::runtime_error("FullyFusedMLP::backward_backward_input: only the parameter gradient is part of the NeuS step");
		const auto& c = dynamic_cast<const ForwardContext&>(ctx);
		const T* p = use_inference_params ? m_inference_params : m_params;
		neus2b_check(neus2b_mlp_backward_backward_input(dL_ddLdinput.n(), m_in, (const uint16_t*)p, (const uint16_t*)c.hidden.data(),
		                                                (const uint16_t*)dL_ddLdinput.data(), (const uint16_t*)dL_doutput.data(), m_gradients,
		                                                (int)param_gradients_mode, stream),
		             "FullyFusedMLP::backward_backward_input");
	}
	/* The weight gradient is kept in fp32 (it feeds Adam directly), unlike tcnn's slab of T. */
	void set_params(T* params, T* inference_params, T* backward_params, float* gradients) {
		m_params = params, m_inference_params = inference_params, m_gradients = gradients;
		(void)backward_params;
	}
	size_t n_params() const { return (size_t)64 * m_in + (size_t)(m_hidden - 1) * 64 * 64 + 16 * 64; }
	uint32_t input_width() const { return m_in; }
	uint32_t padded_output_width() const { return 16; }

private:
	uint32_t m_in, m_hidden;
	T *m_params = nullptr, *m_inference_params = nullptr;
	float* m_gradients = nullptr;
};

/* Ema(ExponentialDecay(Adam)) of configs/nerf/base.json:5-27 as one pass over the parameter block
 * [MLP matrices (n_matrix) | grid | 4 variance slots]; Trainer::optimizer_step (src/testbed_nerf.cu:3960). */
class NeusAdamOptimizer {
public:
	NeusAdamOptimizer(uint64_t n_params, uint32_t n_matrix) : m_n(n_params), m_master(n_params), m_m(n_params), m_v(n_params), m_ema(n_params) {
		m_cfg = neus2b_adam_cfg{};
		m_cfg.learning_rate = 1e-2f, m_cfg.beta1 = 0.9f, m_cfg.beta2 = 0.99f, m_cfg.epsilon = 1e-15f, m_cfg.l2_reg = 1e-6f;
		m_cfg.ema_decay = 0.95f, m_cfg.loss_scale = 128.0f, m_cfg.step = 0, m_cfg.n_matrix = n_matrix;
		m_m.memset(0);
		m_v.memset(0);
	}
	void set_learning_rate(float lr) { m_cfg.learning_rate = lr; }
	float learning_rate() const { return m_cfg.learning_rate; }
	uint32_t step() const { return m_cfg.step; }
	neus2b_adam_cfg& hyperparams() { return m_cfg; }
	void set_params_full_precision(const float* host, size_t n) {
		m_master.copy_from_host(host, n);
		m_ema.copy_from_host(host, n);
	}
	float* params_full_precision() const { return m_master.data(); }
	/* gradients: fp32 MLP block, fp16 grid block, fp32 variance slots; all three are cleared by the pass */
	void step(cudaStream_t stream, float loss_scale, __half* params, __half* params_ema, float* grad_mlp, __half* grad_grid, float* grad_variance) {
		m_cfg.loss_scale = loss_scale;
		++m_cfg.step;
		neus2b_check(neus2b_adam_step(&m_cfg, m_n, grad_mlp, (uint16_t*)grad_grid, grad_variance, m_master.data(), m_m.data(), m_v.data(), (uint16_t*)params,
		                              (uint16_t*)params_ema, m_ema.data(), stream),
		             "NeusAdamOptimizer::step");
	}

private:
	uint64_t m_n;
	neus2b_adam_cfg m_cfg;
	GPUMemory<float> m_master, m_m, m_v, m_ema;
};

}  // namespace tcnn
