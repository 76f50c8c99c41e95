/* tiny-cuda-nn/encodings/grid.h of the B200-native stand-in: the multiresolution hash grid as an Encoding<T>.
 * GridEncoding<T> is the interface the testbed reaches through dynamic_cast (src/testbed.cu:1861-1877, :3070-3084);
 * GridEncodingNeus2b<T> implements it over the C interface's grid kernels (neus2b_grid_forward and its backward and
 * second-order passes), for the shape the NeuS path uses: 3 input dimensions, 2 features per level, up to 16 levels,
 * linear interpolation, T = __half.  Other shapes are refused at construction.
 *
 * json keys (configs/nerf/base.json:29-39): n_levels, n_features_per_level, log2_hashmap_size, base_resolution,
 * per_level_scale (the testbed derives it from top_resolution before it creates the encoding, src/testbed.cu:2173-2177),
 * and the progressive mask's base_training_step, valid_level_scale, base_valid_level_scale. */
#pragma once
#include <tiny-cuda-nn/encoding.h>

#include <neus2b.h>

TCNN_NAMESPACE_BEGIN

inline void neus2b_check(int rc, const char* what) {
	if (rc != 0) throw std::runtime_error(std::string(what) + ": " + neus2b_error_string(rc));
}

template <typename T>
class GridEncoding : public Encoding<T> {
public:
	virtual uint32_t n_pos_dims() const = 0;
	virtual uint32_t n_features_per_level() const = 0;
	virtual size_t level_n_params(uint32_t level) const = 0;
	virtual size_t level_params_offset(uint32_t level) const = 0;

	/* fraction of the levels that take part, for all batch elements (the viewer's slider) */
	float max_level() const { return m_max_level; }
	void set_max_level(float value) { m_max_level = value; }
	float* max_level_gpu() const { return m_max_level_gpu; }
	void set_max_level_gpu(float* value) { m_max_level_gpu = value; }
	float quantize_threshold() const { return m_quantize_threshold; }
	void set_quantize_threshold(float value) { m_quantize_threshold = value; }

protected:
	float m_max_level = 1000.f;
	float* m_max_level_gpu = nullptr;
	float m_quantize_threshold = 0.f;
};

template <typename T>
class GridEncodingNeus2b : public GridEncoding<T> {
	static_assert(std::is_same<T, __half>::value, "the grid kernels of this library compute in fp16");

public:
	struct ForwardContext : public Context {
		GPUMemoryArena::Allocation dy_dx; /* [n][2L][3] fp32, kept when prepare_input_gradients */
	};

	GridEncodingNeus2b(const json& params) {
		m_desc = neus2b_grid_desc{};
		m_desc.n_levels = params.value("n_levels", 16u);
		m_desc.log2_hashmap_size = params.value("log2_hashmap_size", 19u);
		m_desc.base_resolution = params.value("base_resolution", 16u);
		m_desc.per_level_scale = params.value("per_level_scale", 2.0f);
		m_desc.n_active_levels = m_desc.n_levels;
		m_base_training_step = params.value("base_training_step", 0u);
		m_valid_level_scale = params.value("valid_level_scale", 0.0f);
		m_base_valid_level_scale = params.value("base_valid_level_scale", 1.0f);
		uint64_t n = 0;
		neus2b_check(neus2b_grid_n_params(&m_desc, &n), "GridEncoding");
		m_n_params = (size_t)n;
		neus2b_check(neus2b_grid_level_table(&m_desc, m_offsets, m_resolutions, m_scales, m_hashed), "GridEncoding");
		m_hyperparams = params;
		m_hyperparams["otype"] = "HashGrid";
		set_training_step(0);
	}

	std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>* output = nullptr,
	                                      bool use_inference_params = false, bool prepare_input_gradients = false) override {
		auto ctx = std::make_unique<ForwardContext>();
		if (!output || input.n() == 0) return ctx;
#if defined(__CUDACC__)
		DenseColumns<float> x{stream, input, true, true};
		DenseColumns<T> y{stream, *output, false};
		if (prepare_input_gradients) ctx->dy_dx = allocate_workspace(stream, (size_t)input.n() * padded_output_width() * 3 * sizeof(float));
		neus2b_check(neus2b_grid_forward(&m_desc, input.n(), x.data(), x_stride(input, x), (const uint16_t*)pick(use_inference_params), (uint16_t*)y.data(),
		                                 prepare_input_gradients ? (float*)ctx->dy_dx.data() : nullptr, stream),
		             "GridEncoding::forward");
		y.scatter();
#else
		throw std::runtime_error("GridEncoding::forward: needs a CUDA translation unit");
#endif
		return ctx;
	}

	void backward_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<float>& input, const GPUMatrixDynamic<T>& output,
	                   const GPUMatrixDynamic<T>& dL_doutput, GPUMatrixDynamic<float>* dL_dinput = nullptr, bool use_inference_params = false,
	                   EGradientMode param_gradients_mode = EGradientMode::Overwrite) override {
		(void)ctx;
		(void)output;
		if (input.n() == 0) return;
#if defined(__CUDACC__)
		DenseColumns<float> x{stream, input, true, true};
		DenseColumns<T> dy{stream, dL_doutput, true};
		if (dL_dinput) {
			DenseColumns<float> dx{stream, *dL_dinput, false};
			neus2b_check(neus2b_grid_backward_input(&m_desc, input.n(), x.data(), x_stride(input, x), (const uint16_t*)pick(use_inference_params),
			                                        (const uint16_t*)dy.data(), dx.data(), stream),
			             "GridEncoding::backward (input)");
			dx.scatter();
		}
		if (param_gradients_mode != EGradientMode::Ignore)
			neus2b_check(neus2b_grid_backward_params(&m_desc, input.n(), x.data(), x_stride(input, x), (const uint16_t*)dy.data(), (uint16_t*)m_gradients,
			                                         (int)param_gradients_mode, stream),
			             "GridEncoding::backward (params)");
#else
		throw std::runtime_error("GridEncoding::backward: needs a CUDA translation unit");
#endif
	}

	/* dL_ddLdinput [3 x n] fp32 = dL/d(dL_dinput of backward); dL_doutput [2L x n] = what backward was given.  Writes
	 * dL_ddLdoutput [2L x n] and adds the parameter gradient (nerf_network.h:534-544). */
	void backward_backward_input_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<float>& input, const GPUMatrixDynamic<float>& dL_ddLdinput,
	                                  const GPUMatrixDynamic<T>& dL_doutput, GPUMatrixDynamic<T>* dL_ddLdoutput = nullptr, GPUMatrixDynamic<float>* dL_dinput = nullptr,
	                                  bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) override {
		(void)ctx;
		if (input.n() == 0) return;
#if defined(__CUDACC__)
		DenseColumns<float> x{stream, input, true, true};
		DenseColumns<float> v{stream, dL_ddLdinput, true};
		DenseColumns<T> g{stream, dL_doutput, true};
		std::unique_ptr<DenseColumns<T>> out;
		if (dL_ddLdoutput) out = std::make_unique<DenseColumns<T>>(stream, *dL_ddLdoutput, false);
		if (dL_dinput) dL_dinput->memset_async(stream, 0); /* linear interpolation: the third derivative along one axis vanishes; the mixed terms are not
		                                                       part of the NeuS step (the caller discards this matrix, nerf_network.h:529-544) */
		neus2b_check(neus2b_grid_backward_backward_input(&m_desc, input.n(), x.data(), x_stride(input, x), (const uint16_t*)pick(use_inference_params), v.data(),
		                                                 (const uint16_t*)g.data(), out ? (uint16_t*)out->data() : nullptr, (uint16_t*)m_gradients,
		                                                 (int)param_gradients_mode, stream),
		             "GridEncoding::backward_backward_input");
		if (out) out->scatter();
#else
		throw std::runtime_error("GridEncoding::backward_backward_input: needs a CUDA translation unit");
#endif
	}

	/* reference keys: levels open with the training step (src/testbed.cu:2641-2647) */
	void set_training_step(int training_step) override {
		neus2b_testbed_config c{};
		c.grid = m_desc;
		c.grid.n_active_levels = m_desc.n_levels;
		c.base_training_step = m_base_training_step;
		c.valid_level_scale = m_valid_level_scale;
		c.base_valid_level_scale = m_base_valid_level_scale;
		m_desc.n_active_levels = neus2b_testbed_config_active_levels(&c, training_step > 0 ? (uint32_t)training_step : 0u);
	}
	uint32_t n_active_levels() const { return m_desc.n_active_levels; }
	void set_n_active_levels(uint32_t n) { m_desc.n_active_levels = std::min(n, m_desc.n_levels); }

	uint32_t input_width() const override { return 3; }
	uint32_t padded_output_width() const override { return next_multiple(2 * m_desc.n_levels, m_alignment); }
	uint32_t output_width() const override { return 2 * m_desc.n_levels; }
	uint32_t required_input_alignment() const override { return 1; }
	void set_alignment(uint32_t alignment) override {
		if ((2 * m_desc.n_levels) % alignment != 0 && next_multiple(2 * m_desc.n_levels, alignment) != 2 * m_desc.n_levels)
			throw std::runtime_error("GridEncoding: the kernels write 2 x n_levels features per element without padding; choose n_levels so that this is a multiple of " + std::to_string(alignment));
		m_alignment = alignment;
	}
	uint32_t min_alignment() const override { return 2; }
	MatrixLayout preferred_output_layout() const override { return AoS; }

	void set_params(T* params, T* inference_params, T* backward_params, T* gradients) override {
		(void)backward_params;
		m_params = params;
		m_inference_params = inference_params;
		m_gradients = gradients;
	}
	/* uniform in [-1e-4, 1e-4] * scale, drawn in full precision */
	void initialize_params(pcg32& rnd, float* params_full_precision, T* params, T* inference_params, T* backward_params, T* gradients, float scale = 1) override {
		set_params(params, inference_params, backward_params, gradients);
#if defined(__CUDACC__)
		generate_random_uniform<float>(rnd, n_params(), params_full_precision, -1e-4f * scale, 1e-4f * scale);
#else
		throw std::runtime_error("GridEncoding::initialize_params: needs a CUDA translation unit");
#endif
	}
	size_t n_params() const override { return m_n_params; }
	T* params() const { return m_params; }
	T* inference_params() const { return m_inference_params; }
	T* gradients() const { return m_gradients; }

	uint32_t n_pos_dims() const override { return 3; }
	uint32_t n_features_per_level() const override { return 2; }
	uint32_t n_levels() const { return m_desc.n_levels; }
	size_t level_n_params(uint32_t level) const override { return level < m_desc.n_levels ? (size_t)(m_offsets[level + 1] - m_offsets[level]) * 2 : 0; }
	size_t level_params_offset(uint32_t level) const override { return level <= m_desc.n_levels ? (size_t)m_offsets[level] * 2 : m_n_params; }
	const neus2b_grid_desc& desc() const { return m_desc; }

	json hyperparams() const override { return m_hyperparams; }

private:
	const T* pick(bool inference) const { return inference ? m_inference_params : m_params; }
	/* a column-major input is read in place with its own stride (coordinates inside a wider record) */
	static uint32_t x_stride(const GPUMatrixDynamic<float>& input, const DenseColumns<float>& x) { return x.copied() ? input.m() : input.stride(); }

	neus2b_grid_desc m_desc;
	uint32_t m_base_training_step = 0;
	float m_valid_level_scale = 0.f, m_base_valid_level_scale = 1.f;
	uint32_t m_alignment = 2;
	size_t m_n_params = 0;
	uint32_t m_offsets[17] = {}, m_resolutions[16] = {}, m_hashed[16] = {};
	float m_scales[16] = {};
	T *m_params = nullptr, *m_inference_params = nullptr, *m_gradients = nullptr;
	json m_hyperparams;
};

template <typename T>
GridEncoding<T>* create_grid_encoding(uint32_t n_dims_to_encode, const json& encoding) {
	if constexpr (!std::is_same<T, __half>::value) {
		throw std::runtime_error("create_grid_encoding: the grid kernels of this library compute in fp16");
	} else {
		if (n_dims_to_encode != 3) throw std::runtime_error("create_grid_encoding: 3 input dimensions only");
		if (encoding.value("n_features_per_level", 2u) != 2) throw std::runtime_error("create_grid_encoding: 2 features per level only");
		if (encoding.value("n_levels", 16u) > 16) throw std::runtime_error("create_grid_encoding: at most 16 levels");
		const std::string otype = to_lower(encoding.value("otype", "HashGrid"));
		if (otype != "hashgrid" && otype != "grid") throw std::runtime_error("create_grid_encoding: hashed grids only (dense coarse levels are chosen per level)");
		if (!equals_case_insensitive(encoding.value("interpolation", "Linear"), "Linear")) throw std::runtime_error("create_grid_encoding: linear interpolation only");
		return new GridEncodingNeus2b<T>{encoding};
	}
}

TCNN_NAMESPACE_END
