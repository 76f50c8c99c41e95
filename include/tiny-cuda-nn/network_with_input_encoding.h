/* tiny-cuda-nn/network_with_input_encoding.h of the B200-native stand-in: an encoding followed by a network, as one
 * Network<float, T> (what the testbed builds for its non-NeRF modes, src/testbed.cu:2279-2290; the NeuS path uses
 * NerfNetwork instead but includes this header). */
#pragma once
#include <tiny-cuda-nn/encoding.h>
#include <tiny-cuda-nn/network.h>

TCNN_NAMESPACE_BEGIN

template <typename T>
class NetworkWithInputEncoding : public Network<float, T> {
public:
	struct ForwardContext : public Context {
		GPUMatrixDynamic<T> network_input;
		std::unique_ptr<Context> encoding_ctx;
		std::unique_ptr<Context> network_ctx;
	};

	NetworkWithInputEncoding(std::shared_ptr<Encoding<T>> encoding, const json& network) : m_encoding{encoding} {
		encoding->set_alignment(minimum_alignment(network));
		json local = network;
		local["n_input_dims"] = m_encoding->padded_output_width();
		m_network.reset(create_network<T>(local));
	}
	NetworkWithInputEncoding(std::shared_ptr<Encoding<T>> encoding, uint32_t n_output_dims, const json& network) : m_encoding{encoding} {
		encoding->set_alignment(minimum_alignment(network));
		json local = network;
		local["n_input_dims"] = m_encoding->padded_output_width();
		local["n_output_dims"] = n_output_dims;
		m_network.reset(create_network<T>(local));
	}
	NetworkWithInputEncoding(uint32_t n_dims_to_encode, uint32_t n_output_dims, const json& encoding, const json& network)
	    : NetworkWithInputEncoding{std::shared_ptr<Encoding<T>>{create_encoding<T>(n_dims_to_encode, encoding, minimum_alignment(network))}, n_output_dims, network} {}

	void inference_mixed_precision_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>& output, bool use_inference_params = true) override {
		GPUMatrixDynamic<T> network_input{m_encoding->padded_output_width(), input.n(), stream, m_encoding->preferred_output_layout()};
		m_encoding->inference_mixed_precision(stream, input, network_input, use_inference_params);
		m_network->inference_mixed_precision(stream, network_input, output, use_inference_params);
	}
	std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>* output = nullptr, bool use_inference_params = false,
	                                      bool prepare_input_gradients = false) override {
		auto forward = std::make_unique<ForwardContext>();
		forward->network_input = GPUMatrixDynamic<T>{m_encoding->padded_output_width(), input.n(), stream, m_encoding->preferred_output_layout()};
		forward->encoding_ctx = m_encoding->forward(stream, input, &forward->network_input, use_inference_params, prepare_input_gradients);
		forward->network_ctx = m_network->forward(stream, forward->network_input, output, use_inference_params, true);
		return forward;
	}
	void backward_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<float>& input, const GPUMatrixDynamic<T>& output, const GPUMatrixDynamic<T>& dL_doutput,
	                   GPUMatrixDynamic<float>* dL_dinput = nullptr, bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) override {
		const auto& forward = dynamic_cast<const ForwardContext&>(ctx);
		GPUMatrixDynamic<T> dL_dnetwork_input;
		const bool need = m_encoding->n_params() > 0 || dL_dinput;
		if (need) dL_dnetwork_input = GPUMatrixDynamic<T>{m_encoding->padded_output_width(), input.n(), stream, m_encoding->preferred_output_layout()};
		m_network->backward(stream, *forward.network_ctx, forward.network_input, output, dL_doutput, need ? &dL_dnetwork_input : nullptr, use_inference_params, param_gradients_mode);
		if (need) m_encoding->backward(stream, *forward.encoding_ctx, input, forward.network_input, dL_dnetwork_input, dL_dinput, use_inference_params, param_gradients_mode);
	}

	void set_params(T* params, T* inference_params, T* backward_params, T* gradients) override {
		size_t offset = 0;
		m_network->set_params(params + offset, inference_params + offset, backward_params + offset, gradients + offset);
		offset += m_network->n_params();
		m_encoding->set_params(params + offset, inference_params + offset, backward_params + offset, gradients + offset);
	}
	void initialize_params(pcg32& rnd, float* params_full_precision, T* params, T* inference_params, T* backward_params, T* gradients, float scale = 1) override {
		size_t offset = 0;
		m_network->initialize_params(rnd, params_full_precision + offset, params + offset, inference_params + offset, backward_params + offset, gradients + offset, scale);
		offset += m_network->n_params();
		m_encoding->initialize_params(rnd, params_full_precision + offset, params + offset, inference_params + offset, backward_params + offset, gradients + offset, scale);
	}
	size_t n_params() const override { return m_encoding->n_params() + m_network->n_params(); }
	uint32_t padded_output_width() const override { return m_network->padded_output_width(); }
	uint32_t output_width() const override { return m_network->output_width(); }
	uint32_t input_width() const override { return m_encoding->input_width(); }
	uint32_t required_input_alignment() const override { return 1; }
	std::vector<std::pair<uint32_t, uint32_t>> layer_sizes() const override { return m_network->layer_sizes(); }
	uint32_t width(uint32_t layer) const override { return layer == 0 ? m_encoding->padded_output_width() : m_network->width(layer - 1); }
	uint32_t num_forward_activations() const override { return m_network->num_forward_activations() + 1; }
	std::pair<const T*, MatrixLayout> forward_activations(const Context& ctx, uint32_t layer) const override {
		const auto& forward = dynamic_cast<const ForwardContext&>(ctx);
		return layer == 0 ? std::make_pair<const T*, MatrixLayout>(forward.network_input.data(), m_encoding->preferred_output_layout())
		                  : m_network->forward_activations(*forward.network_ctx, layer - 1);
	}
	const std::shared_ptr<Encoding<T>>& encoding() const { return m_encoding; }
	json hyperparams() const override { return {{"otype", "NetworkWithInputEncoding"}, {"encoding", m_encoding->hyperparams()}, {"network", m_network->hyperparams()}}; }

private:
	std::shared_ptr<Encoding<T>> m_encoding;
	std::unique_ptr<Network<T>> m_network;
};

TCNN_NAMESPACE_END
