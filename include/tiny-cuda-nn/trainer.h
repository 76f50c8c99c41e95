/* tiny-cuda-nn/trainer.h of the B200-native stand-in: Trainer<T, PARAMS_T, COMPUTE_T> owns one parameter block for a
 * model -- full-precision master weights, the PARAMS_T copy the kernels read, and the gradient slab -- hands slices of
 * it to the model (initialize_params / set_params), and runs the optimizer over it.  Call sites followed:
 * src/testbed.cu:2303 (construction), :2057 (params_* accessors), :2335 (set_params_full_precision), :2689
 * (optimizer()), :3136 / :3240 (serialize / deserialize), src/testbed_nerf.cu:3498-3525 (optimizer_step).
 *
 * Block layout (one device allocation, every array on a 256-byte boundary):
 *   float    params_full_precision[n]   (is the params array itself when PARAMS_T is float)
 *   PARAMS_T params[n]
 *   PARAMS_T params_backward[n]         (kept for interface parity; equal to params)
 *   PARAMS_T param_gradients[n]
 * Inference reads the optimizer's custom weights (the EMA) when it has some, else params. */
#pragma once
#include <tiny-cuda-nn/gpu_memory_json.h>
#include <tiny-cuda-nn/loss.h>
#include <tiny-cuda-nn/object.h>
#include <tiny-cuda-nn/optimizer.h>

#include <random>

TCNN_NAMESPACE_BEGIN

template <typename T, typename PARAMS_T, typename COMPUTE_T = PARAMS_T>
class Trainer : public ObjectWithMutableHyperparams {
public:
	Trainer(std::shared_ptr<DifferentiableObject<T, PARAMS_T, COMPUTE_T>> model, std::shared_ptr<Optimizer<PARAMS_T>> optimizer, std::shared_ptr<Loss<COMPUTE_T>> loss,
	        uint32_t seed = 1337, float perturbation_sigma = 0)
	    : m_model{model}, m_optimizer{optimizer}, m_loss{loss}, m_perturbation_sigma{perturbation_sigma} {
		std::seed_seq seq{seed};
		std::vector<uint32_t> seeds(2);
		seq.generate(std::begin(seeds), std::end(seeds));
		m_rng = pcg32{seeds.front()};
		initialize_params();
	}
	virtual ~Trainer() {}

	void update_hyperparams(const json& params) override {
		if (params.contains("perturbation_sigma")) m_perturbation_sigma = params["perturbation_sigma"];
	}
	json hyperparams() const override { return {{"otype", "Trainer"}, {"perturbation_sigma", m_perturbation_sigma}}; }

	/* allocates the block, lets the model draw its initial weights in full precision, and derives the PARAMS_T copy */
	void initialize_params() {
		const size_t n = m_model->n_params();
		const size_t stride_f = detail::align_to_workspace(n * sizeof(float)), stride_p = detail::align_to_workspace(n * sizeof(PARAMS_T));
		const bool alias = std::is_same<PARAMS_T, float>::value;
		m_params_buffer.resize((alias ? 0 : stride_f) + stride_p * 3 + 256);
		m_params_buffer.memset(0);
		uint8_t* base = (uint8_t*)m_params_buffer.data();
		size_t offset = 0;
		if (!alias) {
			m_params_full_precision = (float*)(base + offset);
			offset += stride_f;
		}
		m_params = (PARAMS_T*)(base + offset);
		offset += stride_p;
		if (alias) m_params_full_precision = (float*)m_params;
		m_params_backward = (PARAMS_T*)(base + offset);
		offset += stride_p;
		m_param_gradients = (PARAMS_T*)(base + offset);
		m_n_params = n;

		m_optimizer->allocate((uint32_t)n, m_model->layer_sizes());
		m_optimizer->set_param_groups(m_model->n_params_canonical(), m_model->n_params_delta(), m_model->n_params_components());
		m_params_inference = m_optimizer->custom_weights() ? m_optimizer->custom_weights() : m_params;
		m_model->initialize_params(m_rng, m_params_full_precision, m_params, m_params_inference, m_params_backward, m_param_gradients);
		sync_from_full_precision();
	}

	/* replaces every copy of the weights by `params` (host memory unless device is set) */
	void set_params_full_precision(const float* params, size_t n_params, bool device = false) {
		if (n_params != m_n_params) throw std::runtime_error("Trainer::set_params_full_precision: the model has " + std::to_string(m_n_params) + " parameters, got " + std::to_string(n_params));
		CUDA_CHECK_THROW(cudaMemcpy(m_params_full_precision, params, sizeof(float) * n_params, device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
		sync_from_full_precision();
	}
	void set_params(const PARAMS_T* params, size_t n_params, bool device = false) {
		if (n_params != m_n_params) throw std::runtime_error("Trainer::set_params: the model has " + std::to_string(m_n_params) + " parameters, got " + std::to_string(n_params));
		CUDA_CHECK_THROW(cudaMemcpy(m_params, params, sizeof(PARAMS_T) * n_params, device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
		sync_to_full_precision();
	}

	/* one optimizer pass over the block with the gradients the model's backward left there */
	void optimizer_step(cudaStream_t stream, float loss_scale) {
		m_optimizer->step(stream, loss_scale, m_params_full_precision, m_params, m_param_gradients);
		++m_n_steps;
	}
	void optimizer_step(float loss_scale) { optimizer_step(nullptr, loss_scale); }

	/* forward, loss, backward and optimizer step on one batch (the generic training loop of the non-NeRF modes) */
	struct ForwardContext : public Context {
		GPUMatrix<COMPUTE_T> perturbed_output;
		GPUMatrix<COMPUTE_T> output;
		GPUMatrix<COMPUTE_T> dL_doutput;
		GPUMatrix<float> L;
		std::unique_ptr<Context> model_ctx;
	};
	std::unique_ptr<ForwardContext> forward(cudaStream_t stream, const float loss_scale, const GPUMatrixDynamic<T>& input, const GPUMatrix<float>& target,
	                                        const GPUMatrix<float>* data_pdf = nullptr, bool use_inference_params = false, bool prepare_input_gradients = false) {
		const uint32_t batch = input.n();
		auto forward = std::make_unique<ForwardContext>();
		forward->output = GPUMatrix<COMPUTE_T>{m_model->padded_output_width(), batch, stream};
		forward->model_ctx = m_model->forward(stream, input, &forward->output, use_inference_params, prepare_input_gradients);
		forward->dL_doutput = GPUMatrix<COMPUTE_T>{m_model->padded_output_width(), batch, stream};
		forward->L = GPUMatrix<float>{m_model->padded_output_width(), batch, stream};
		m_loss->evaluate(stream, m_model->padded_output_width(), m_model->output_width(), loss_scale, forward->output, target, forward->L, forward->dL_doutput, data_pdf);
		return forward;
	}
	void backward(cudaStream_t stream, const ForwardContext& ctx, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<T>* dL_dinput = nullptr,
	              bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		m_model->backward(stream, *ctx.model_ctx, input, ctx.output, ctx.dL_doutput, dL_dinput, use_inference_params, param_gradients_mode);
	}
	std::unique_ptr<ForwardContext> training_step(cudaStream_t stream, const GPUMatrixDynamic<T>& input, const GPUMatrix<float>& target,
	                                              const GPUMatrix<float>* data_pdf = nullptr, bool run_optimizer = true, GPUMatrixDynamic<T>* dL_dinput = nullptr,
	                                              bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		const float loss_scale = default_loss_scale<PARAMS_T>();
		auto ctx = forward(stream, loss_scale, input, target, data_pdf, use_inference_params, dL_dinput != nullptr);
		backward(stream, *ctx, input, dL_dinput, use_inference_params, param_gradients_mode);
		if (run_optimizer) optimizer_step(stream, loss_scale);
		return ctx;
	}
	std::unique_ptr<ForwardContext> training_step(const GPUMatrixDynamic<T>& input, const GPUMatrix<float>& target, const GPUMatrix<float>* data_pdf = nullptr,
	                                              bool run_optimizer = true) {
		return training_step(nullptr, input, target, data_pdf, run_optimizer);
	}
#if defined(__CUDACC__)
	float loss(cudaStream_t stream, const ForwardContext& ctx) const { return reduce_sum_values(ctx.L.data(), ctx.L.n_elements(), stream); }
#endif

	float* params_full_precision() const { return m_params_full_precision; }
	PARAMS_T* params() const { return m_params; }
	PARAMS_T* params_inference() const { return m_params_inference; }
	PARAMS_T* params_backward() const { return m_params_backward; }
	PARAMS_T* param_gradients() const { return m_param_gradients; }
	size_t n_params() const { return m_n_params; }
	uint32_t n_steps() const { return m_n_steps; }
	std::shared_ptr<DifferentiableObject<T, PARAMS_T, COMPUTE_T>> model() { return m_model; }
	std::shared_ptr<Optimizer<PARAMS_T>> optimizer() { return m_optimizer; }
	std::shared_ptr<Loss<COMPUTE_T>> loss() { return m_loss; }

	/* {"n_params", "params_type", "params_binary" (the inference weights), and with optimizer state "optimizer" plus the
	 * master and training copies needed to continue the run exactly} */
	json serialize(bool serialize_optimizer = false) {
		json data;
		data["n_params"] = m_n_params;
		data["params_type"] = type_to_string<PARAMS_T>();
		data["params_binary"] = gpu_memory_to_json_binary(m_params_inference, sizeof(PARAMS_T) * m_n_params);
		if (serialize_optimizer) {
			data["optimizer"] = m_optimizer->serialize();
			data["neus2b"]["params_full_precision_binary"] = gpu_memory_to_json_binary(m_params_full_precision, sizeof(float) * m_n_params);
			data["neus2b"]["params_training_binary"] = gpu_memory_to_json_binary(m_params, sizeof(PARAMS_T) * m_n_params);
		}
		return data;
	}
	void deserialize(const json& data) {
		const std::string type = data.value("params_type", type_to_string<PARAMS_T>());
		if (type != type_to_string<PARAMS_T>()) throw std::runtime_error("Trainer::deserialize: the snapshot holds " + type + " parameters, this trainer " + type_to_string<PARAMS_T>());
		if (data.value("n_params", (size_t)0) != m_n_params)
			throw std::runtime_error("Trainer::deserialize: the snapshot holds " + std::to_string(data.value("n_params", (size_t)0)) + " parameters, the model " + std::to_string(m_n_params));
		json_binary_to_gpu_memory(data["params_binary"].get_binary(), m_params, sizeof(PARAMS_T) * m_n_params);
		sync_to_full_precision();
		if (data.contains("optimizer")) m_optimizer->deserialize(data["optimizer"]);
		if (data.contains("neus2b") && data["neus2b"].contains("params_full_precision_binary")) {
			json_binary_to_gpu_memory(data["neus2b"]["params_full_precision_binary"].get_binary(), m_params_full_precision, sizeof(float) * m_n_params);
			json_binary_to_gpu_memory(data["neus2b"]["params_training_binary"].get_binary(), m_params, sizeof(PARAMS_T) * m_n_params);
			CUDA_CHECK_THROW(cudaMemcpy(m_params_backward, m_params, sizeof(PARAMS_T) * m_n_params, cudaMemcpyDeviceToDevice));
		}
		reset_param_gradients();
	}
	void reset_param_gradients() { CUDA_CHECK_THROW(cudaMemset(m_param_gradients, 0, sizeof(PARAMS_T) * m_n_params)); }

private:
	template <typename U>
	static std::string type_to_string() {
		if (std::is_same<U, float>::value) return "float";
		if (std::is_same<U, __half>::value) return "__half";
		return "unknown";
	}
	template <typename U>
	static float default_loss_scale() {
		return std::is_same<U, __half>::value ? 128.0f : 1.0f;
	}
	/* master weights -> every PARAMS_T copy (and the EMA, so that inference sees the new weights at once) */
	void sync_from_full_precision() {
#if defined(__CUDACC__)
		const uint32_t n = (uint32_t)m_n_params;
		if (!n) return;
		if (!std::is_same<PARAMS_T, float>::value) cast_kernel<PARAMS_T><<<n_blocks_linear(n), n_threads_linear>>>(n, m_params_full_precision, m_params);
		CUDA_CHECK_THROW(cudaMemcpy(m_params_backward, m_params, sizeof(PARAMS_T) * n, cudaMemcpyDeviceToDevice));
		if (m_params_inference != m_params) CUDA_CHECK_THROW(cudaMemcpy(m_params_inference, m_params, sizeof(PARAMS_T) * n, cudaMemcpyDeviceToDevice));
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
#else
		throw std::runtime_error("Trainer: needs a CUDA translation unit");
#endif
	}
	void sync_to_full_precision() {
#if defined(__CUDACC__)
		const uint32_t n = (uint32_t)m_n_params;
		if (!n) return;
		if (!std::is_same<PARAMS_T, float>::value) cast_from_kernel<PARAMS_T><<<n_blocks_linear(n), n_threads_linear>>>(n, m_params, m_params_full_precision);
		CUDA_CHECK_THROW(cudaMemcpy(m_params_backward, m_params, sizeof(PARAMS_T) * n, cudaMemcpyDeviceToDevice));
		if (m_params_inference != m_params) CUDA_CHECK_THROW(cudaMemcpy(m_params_inference, m_params, sizeof(PARAMS_T) * n, cudaMemcpyDeviceToDevice));
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
#else
		throw std::runtime_error("Trainer: needs a CUDA translation unit");
#endif
	}
#if defined(__CUDACC__)
	static float reduce_sum_values(float* values, uint32_t n, cudaStream_t stream);
#endif

	std::shared_ptr<DifferentiableObject<T, PARAMS_T, COMPUTE_T>> m_model;
	std::shared_ptr<Optimizer<PARAMS_T>> m_optimizer;
	std::shared_ptr<Loss<COMPUTE_T>> m_loss;
	GPUMemory<char> m_params_buffer;
	float* m_params_full_precision = nullptr;
	PARAMS_T *m_params = nullptr, *m_params_inference = nullptr, *m_params_backward = nullptr, *m_param_gradients = nullptr;
	size_t m_n_params = 0;
	uint32_t m_n_steps = 0;
	float m_perturbation_sigma;
	pcg32 m_rng;
};

TCNN_NAMESPACE_END

#include <tiny-cuda-nn/reduce_sum.h>

TCNN_NAMESPACE_BEGIN
#if defined(__CUDACC__)
template <typename T, typename PARAMS_T, typename COMPUTE_T>
float Trainer<T, PARAMS_T, COMPUTE_T>::reduce_sum_values(float* values, uint32_t n, cudaStream_t stream) {
	return reduce_sum(values, n, stream);
}
#endif
TCNN_NAMESPACE_END
