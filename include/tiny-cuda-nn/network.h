/* tiny-cuda-nn/network.h of the B200-native stand-in: Network<T, PARAMS_T> (a DifferentiableObject whose input and
 * output share a precision), the json factory, and the one network type the NeuS path instantiates
 * (configs/nerf/base.json:40-47, :63-69): a fully fused MLP of 64 ReLU neurons with 1 or 2 hidden layers, no output
 * activation and 16 padded outputs, bound to the C interface's MLP kernels.  NerfNetwork holds two of them
 * (include/neural-graphics-primitives/nerf_network.h:57, :65) and calls forward, backward and, for the eikonal term,
 * backward_backward_input on the first (:212, :229, :402, :560-571). */
#pragma once
#include <tiny-cuda-nn/object.h>

#include <neus2b.h>

#include <cmath>

TCNN_NAMESPACE_BEGIN

template <typename T, typename PARAMS_T = T>
class Network : public DifferentiableObject<T, PARAMS_T, PARAMS_T> {
public:
	virtual ~Network() {}
	/* width of the activations behind `layer`, their count, and a pointer to them inside a forward context (viewer) */
	virtual uint32_t width(uint32_t layer) const = 0;
	virtual uint32_t num_forward_activations() const = 0;
	virtual std::pair<const PARAMS_T*, MatrixLayout> forward_activations(const Context& ctx, uint32_t layer) const = 0;
};

/* the input alignment a network type asks of the encoding that feeds it */
inline uint32_t minimum_alignment(const json& network) {
	const std::string otype = to_lower(network.value("otype", "FullyFusedMLP"));
	if (otype == "fullyfusedmlp" || otype == "megakernelmlp") return 16u;
	return 8u;
}

#if defined(__CUDACC__)
template <typename T>
__global__ void gradient_from_float_kernel(const uint32_t n, const float* __restrict__ in, T* __restrict__ out, const bool accumulate) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i >= n) return;
	out[i] = (T)(in[i] + (accumulate ? (float)out[i] : 0.0f));
}
#endif

template <typename T>
class FullyFusedMLP : public Network<T> {
	static_assert(std::is_same<T, __half>::value, "the MLP kernels of this library compute in fp16");

public:
	static constexpr uint32_t WIDTH = 64;
	struct ForwardContext : public Context {
		GPUMemoryArena::Allocation hidden;  /* [n][n_hidden][64] */
		GPUMemoryArena::Allocation input;   /* dense copy of the input when it came strided or row-major */
	};

	FullyFusedMLP(uint32_t input_width, uint32_t output_width, uint32_t n_hidden_layers, Activation activation, Activation output_activation)
	    : m_input_width{input_width}, m_output_width{output_width}, m_n_hidden{n_hidden_layers} {
		if (input_width != 32 && input_width != 48 && input_width != 64) throw std::runtime_error("FullyFusedMLP: input widths 32, 48 and 64 only, got " + std::to_string(input_width));
		if (output_width == 0 || output_width > 16) throw std::runtime_error("FullyFusedMLP: at most 16 outputs");
		if (n_hidden_layers < 1 || n_hidden_layers > 2) throw std::runtime_error("FullyFusedMLP: 1 or 2 hidden layers only");
		if (activation != Activation::ReLU || output_activation != Activation::None) throw std::runtime_error("FullyFusedMLP: ReLU hidden and no output activation only");
	}

	void inference_mixed_precision_impl(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<T>& output, bool use_inference_params = true) override {
		if (!input.n()) return;
#if defined(__CUDACC__)
		DenseColumns<T> x{stream, input, true};
		DenseColumns<T> y{stream, output, false};
		neus2b_check_mlp(neus2b_mlp_forward(input.n(), m_input_width, m_n_hidden, (const uint16_t*)pick(use_inference_params), (const uint16_t*)x.data(),
		                                    (uint16_t*)y.data(), nullptr, stream),
		                 "inference");
		y.scatter();
#else
		throw std::runtime_error("FullyFusedMLP: needs a CUDA translation unit");
#endif
	}

	std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<T>* output = nullptr, bool use_inference_params = false,
	                                      bool prepare_input_gradients = false) override {
		(void)prepare_input_gradients;
		auto ctx = std::make_unique<ForwardContext>();
		if (!input.n()) return ctx;
#if defined(__CUDACC__)
		DenseColumns<T> x{stream, input, true};
		GPUMemoryArena::Allocation y_tmp;
		std::unique_ptr<DenseColumns<T>> y;
		T* y_data;
		if (output) {
			y = std::make_unique<DenseColumns<T>>(stream, *output, false);
			y_data = y->data();
		} else {
			y_tmp = allocate_workspace(stream, (size_t)input.n() * 16 * sizeof(T));
			y_data = (T*)y_tmp.data();
		}
		ctx->hidden = allocate_workspace(stream, (size_t)input.n() * m_n_hidden * WIDTH * sizeof(T));
		neus2b_check_mlp(neus2b_mlp_forward(input.n(), m_input_width, m_n_hidden, (const uint16_t*)pick(use_inference_params), (const uint16_t*)x.data(),
		                                    (uint16_t*)y_data, (uint16_t*)ctx->hidden.data(), stream),
		                 "forward");
		if (y) y->scatter();
#else
		throw std::runtime_error("FullyFusedMLP: needs a CUDA translation unit");
#endif
		return ctx;
	}

	void backward_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<T>& output, const GPUMatrixDynamic<T>& dL_doutput,
	                   GPUMatrixDynamic<T>* dL_dinput = nullptr, bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) override {
		(void)output;
		if (!input.n()) return;
#if defined(__CUDACC__)
		const auto& forward = dynamic_cast<const ForwardContext&>(ctx);
		DenseColumns<T> x{stream, input, true};
		DenseColumns<T> dy{stream, dL_doutput, true};
		std::unique_ptr<DenseColumns<T>> dx;
		if (dL_dinput) dx = std::make_unique<DenseColumns<T>>(stream, *dL_dinput, false);
		const bool want_params = param_gradients_mode != EGradientMode::Ignore;
		if (want_params) m_grad_scratch.enlarge(n_params());
		neus2b_check_mlp(neus2b_mlp_backward(input.n(), m_input_width, m_n_hidden, (const uint16_t*)pick(use_inference_params), (const uint16_t*)x.data(),
		                                     (const uint16_t*)forward.hidden.data(), (const uint16_t*)dy.data(), dx ? (uint16_t*)dx->data() : nullptr,
		                                     want_params ? m_grad_scratch.data() : nullptr, want_params ? NEUS2B_GRAD_OVERWRITE : NEUS2B_GRAD_IGNORE, stream),
		                 "backward");
		if (dx) dx->scatter();
		if (want_params) publish_gradients(stream, param_gradients_mode);
#else
		throw std::runtime_error("FullyFusedMLP: needs a CUDA translation unit");
#endif
	}

	/* one hidden layer: the parameter gradient of the eikonal term.  dL_ddLdinput = dL/d(dL_dinput of backward),
	 * dL_doutput = what that backward pass was given (nerf_network.h:560-571). */
	void backward_backward_input_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<T>& dL_ddLdinput,
	                                  const GPUMatrixDynamic<T>& dL_doutput, GPUMatrixDynamic<T>* dL_ddLdoutput = nullptr, GPUMatrixDynamic<T>* dL_dinput = nullptr,
	                                  bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) override {
		if (!input.n()) return;
#if defined(__CUDACC__)
		if (m_n_hidden != 1) throw std::runtime_error("FullyFusedMLP::backward_backward_input: one hidden layer only");
		if (dL_ddLdoutput || dL_dinput)
			throw std::runtime_error("FullyFusedMLP::backward_backward_input: only the parameter gradient is produced (what the NeuS step consumes)");
		if (param_gradients_mode == EGradientMode::Ignore) return;
		const auto& forward = dynamic_cast<const ForwardContext&>(ctx);
		m_grad_scratch.enlarge(n_params());
		DenseColumns<T> u{stream, dL_ddLdinput, true};
		DenseColumns<T> dy{stream, dL_doutput, true};
		neus2b_check_mlp(neus2b_mlp_backward_backward_input(input.n(), m_input_width, (const uint16_t*)pick(use_inference_params), (const uint16_t*)forward.hidden.data(),
		                                                    (const uint16_t*)u.data(), (const uint16_t*)dy.data(), m_grad_scratch.data(), NEUS2B_GRAD_OVERWRITE, stream),
		                 "backward_backward_input");
		publish_gradients(stream, param_gradients_mode);
#else
		throw std::runtime_error("FullyFusedMLP: needs a CUDA translation unit");
#endif
	}

	void set_params(T* params, T* inference_params, T* backward_params, T* gradients) override {
		(void)backward_params;
		m_params = params;
		m_inference_params = inference_params;
		m_gradients = gradients;
	}
	/* every matrix uniform in +-sqrt(6 / (fan_in + fan_out)) * scale */
	void initialize_params(pcg32& rnd, float* params_full_precision, T* params, T* inference_params, T* backward_params, T* gradients, float scale = 1) override {
		set_params(params, inference_params, backward_params, gradients);
#if defined(__CUDACC__)
		size_t offset = 0;
		for (const auto& layer : layer_sizes()) {
			const float bound = std::sqrt(6.0f / (float)(layer.first + layer.second)) * scale;
			generate_random_uniform<float>(rnd, (size_t)layer.first * layer.second, params_full_precision + offset, -bound, bound);
			offset += (size_t)layer.first * layer.second;
		}
#else
		throw std::runtime_error("FullyFusedMLP: needs a CUDA translation unit");
#endif
	}
	size_t n_params() const override {
		size_t n = 0;
		for (const auto& l : layer_sizes()) n += (size_t)l.first * l.second;
		return n;
	}
	/* (rows, columns) = (fan out, fan in) of every matrix, in parameter order; matrices are row-major */
	std::vector<std::pair<uint32_t, uint32_t>> layer_sizes() const override {
		std::vector<std::pair<uint32_t, uint32_t>> r{{WIDTH, m_input_width}};
		for (uint32_t i = 1; i < m_n_hidden; ++i) r.push_back({WIDTH, WIDTH});
		r.push_back({16u, WIDTH});
		return r;
	}
	uint32_t input_width() const override { return m_input_width; }
	uint32_t padded_output_width() const override { return 16; }
	uint32_t output_width() const override { return m_output_width; }
	uint32_t required_input_alignment() const override { return 16; }
	uint32_t width(uint32_t layer) const override {
		(void)layer;
		return WIDTH;
	}
	uint32_t num_forward_activations() const override { return m_n_hidden; }
	std::pair<const T*, MatrixLayout> forward_activations(const Context& ctx, uint32_t layer) const override {
		const auto& forward = dynamic_cast<const ForwardContext&>(ctx);
		/* the hidden activations of one element are contiguous over the layers: layer l of element i sits at (i * n_hidden + l) * 64 */
		return {(const T*)forward.hidden.data() + (size_t)layer * WIDTH, CM};
	}
	T* params() const { return m_params; }
	T* inference_params() const { return m_inference_params; }
	T* gradients() const { return m_gradients; }
	json hyperparams() const override {
		return {{"otype", "FullyFusedMLP"}, {"activation", "ReLU"}, {"output_activation", "None"}, {"n_neurons", WIDTH}, {"n_hidden_layers", m_n_hidden}};
	}

private:
	const T* pick(bool inference) const { return inference ? m_inference_params : m_params; }
	static void neus2b_check_mlp(int rc, const char* what) {
		if (rc) throw std::runtime_error(std::string("FullyFusedMLP::") + what + ": " + neus2b_error_string(rc));
	}
#if defined(__CUDACC__)
	/* the kernels produce the weight gradient in fp32 (one batch's sum); the parameter block's gradient slab is T */
	void publish_gradients(cudaStream_t stream, EGradientMode mode) {
		const uint32_t n = (uint32_t)n_params();
		gradient_from_float_kernel<T><<<n_blocks_linear(n), n_threads_linear, 0, stream>>>(n, m_grad_scratch.data(), m_gradients, mode == EGradientMode::Accumulate);
	}
#endif
	uint32_t m_input_width, m_output_width, m_n_hidden;
	T *m_params = nullptr, *m_inference_params = nullptr, *m_gradients = nullptr;
	GPUMemory<float> m_grad_scratch;
};

template <typename T>
Network<T>* create_network(const json& network) {
	const std::string otype = to_lower(network.value("otype", "FullyFusedMLP"));
	if (otype != "fullyfusedmlp" && otype != "megakernelmlp")
		throw std::runtime_error("create_network: network \"" + network.value("otype", "") + "\" is not part of this library (FullyFusedMLP is)");
	if constexpr (!std::is_same<T, __half>::value) {
		throw std::runtime_error("create_network: the MLP kernels of this library compute in fp16");
	} else {
		if (network.value("n_neurons", 128u) != 64) throw std::runtime_error("create_network: FullyFusedMLP with 64 neurons only");
		return new FullyFusedMLP<T>{network["n_input_dims"], network["n_output_dims"], network.value("n_hidden_layers", 5u),
		                            string_to_activation(network.value("activation", "ReLU")), string_to_activation(network.value("output_activation", "None"))};
	}
}

TCNN_NAMESPACE_END
