/* tiny-cuda-nn/optimizer.h of the B200-native stand-in: Optimizer<T>, the json factory, and the chain the NeuS
 * configuration names (configs/nerf/base.json:5-27): Ema(ExponentialDecay(Adam)).  Each is its own object so that any
 * nesting the json asks for works; Adam is one streaming kernel over the parameter block.
 *
 * Adam's update follows the published tiny-cuda-nn behaviour: the gradient is divided by the loss scale; matrix weights
 * (the first n_matrix_weights parameters: the MLPs) get l2_reg * weight added; non-matrix parameters (hash grid) whose
 * gradient is exactly zero are skipped, moments included; the step uses the bias-corrected learning rate
 * lr * sqrt(1 - beta2^t) / (1 - beta1^t).  Keys of the fork used by the testbed (src/testbed.cu:1965, :2682-2684):
 * optimize_matrix_params, optimize_non_matrix_params, optimize_canonical_params, optimize_delta_params,
 * optimize_params_components {name: bool}; "after_learning_rate" is read by the testbed itself (:2691). */
#pragma once
#include <tiny-cuda-nn/gpu_memory_json.h>
#include <tiny-cuda-nn/object.h>

#include <cmath>

TCNN_NAMESPACE_BEGIN

template <typename T>
class Optimizer : public ObjectWithMutableHyperparams {
public:
	virtual ~Optimizer() {}
	virtual void allocate(uint32_t n_weights, const std::vector<std::pair<uint32_t, uint32_t>>& layer_sizes = {}) = 0;
	/* sized for a model (src/testbed_nerf.cu:4206) */
	void allocate(std::shared_ptr<ParametricObject<T>> target) {
		allocate((uint32_t)target->n_params(), target->layer_sizes());
		set_param_groups(target->n_params_canonical(), target->n_params_delta(), target->n_params_components());
	}
	/* how the block splits into the canonical model and the per-frame motion, and into named parts
	 * ([[index, [name, size]], ...] in block order: NerfNetwork::n_params_components, nerf_network.h:913-925) */
	virtual void set_param_groups(size_t n_canonical, size_t n_delta, const json& components) {
		(void)n_canonical;
		(void)n_delta;
		(void)components;
	}
	virtual void step(cudaStream_t stream, float loss_scale, float* weights_full_precision, T* weights, const T* gradients) = 0;
	virtual float learning_rate() const = 0;
	virtual void set_learning_rate(float val) = 0;
	virtual uint32_t step() const = 0;
	virtual uint32_t n_weights() const = 0;
	/* weights to use for inference instead of the trained ones (the EMA), or nullptr */
	virtual T* custom_weights() const = 0;
	virtual bool supports_nesting() const { return false; }
	virtual json serialize() const { return {}; }
	virtual void deserialize(const json& data) { (void)data; }
};

template <typename T>
Optimizer<T>* create_optimizer(const json& params);

/* up to 8 index ranges of the block that the update leaves alone */
struct FrozenRanges {
	uint32_t n = 0;
	uint32_t begin[8] = {}, end[8] = {};
	TCNN_HOST_DEVICE bool contains(uint32_t i) const {
		for (uint32_t r = 0; r < n; ++r)
			if (i >= begin[r] && i < end[r]) return true;
		return false;
	}
};

#if defined(__CUDACC__)
template <typename T>
__global__ void adam_step_kernel(const uint32_t n_elements, const uint32_t n_matrix_weights, const FrozenRanges frozen, const bool optimize_matrix,
                                 const bool optimize_non_matrix, const float loss_scale, const float learning_rate_t, const float beta1, const float beta2,
                                 const float epsilon, const float l2_reg, float* __restrict__ weights_full_precision, T* __restrict__ weights,
                                 const T* __restrict__ gradients, float* __restrict__ first_moments, float* __restrict__ second_moments) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i >= n_elements) return;
	if (frozen.n && frozen.contains(i)) return;
	float gradient = (float)gradients[i] / loss_scale;
	if (!(fabsf(gradient) <= 3.402823466e+38f)) return; /* an overflowed fp16 sum must not reach the weights */
	const float weight = weights_full_precision[i];
	if (i < n_matrix_weights) {
		if (!optimize_matrix) return;
		gradient += l2_reg * weight;
	} else {
		if (!optimize_non_matrix || gradient == 0.0f) return;
	}
	const float m = first_moments[i] = beta1 * first_moments[i] + (1.0f - beta1) * gradient;
	const float v = second_moments[i] = beta2 * second_moments[i] + (1.0f - beta2) * gradient * gradient;
	const float updated = weight - learning_rate_t * m / (sqrtf(v) + epsilon);
	weights_full_precision[i] = updated;
	weights[i] = (T)updated;
}

template <typename T>
__global__ void ema_step_kernel(const uint32_t n_elements, const float decay, const float old_norm, const float new_norm_inv, const float* __restrict__ weights_full_precision,
                                const T* __restrict__ weights, float* __restrict__ ema_full_precision, T* __restrict__ ema_weights) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i >= n_elements) return;
	const float w = weights_full_precision ? weights_full_precision[i] : (float)weights[i];
	const float e = ((1.0f - decay) * w + decay * ema_full_precision[i] * old_norm) * new_norm_inv;
	ema_full_precision[i] = e;
	ema_weights[i] = (T)e;
}
#endif

template <typename T>
class AdamOptimizer : public Optimizer<T> {
public:
	AdamOptimizer(const json& params) { update_hyperparams(params); }

	void allocate(uint32_t n_weights, const std::vector<std::pair<uint32_t, uint32_t>>& layer_sizes = {}) override {
		m_n_weights = n_weights;
		if (m_first_moments.size() != n_weights) {
			m_first_moments.resize(n_weights);
			m_second_moments.resize(n_weights);
			m_first_moments.memset(0);
			m_second_moments.memset(0);
		}
		m_n_matrix_weights = 0;
		for (const auto& l : layer_sizes) m_n_matrix_weights += l.first * l.second;
		if (m_n_matrix_weights > n_weights) m_n_matrix_weights = n_weights;
	}
	void set_param_groups(size_t n_canonical, size_t n_delta, const json& components) override {
		m_n_canonical = n_canonical;
		m_n_delta = n_delta;
		m_components = components;
	}
	void step(cudaStream_t stream, float loss_scale, float* weights_full_precision, T* weights, const T* gradients) override {
		++m_current_step;
#if defined(__CUDACC__)
		if (!m_n_weights) return;
		const float t = (float)m_current_step;
		const float lr_t = m_learning_rate * std::sqrt(1.0f - std::pow(m_beta2, t)) / (1.0f - std::pow(m_beta1, t));
		adam_step_kernel<T><<<n_blocks_linear(m_n_weights), n_threads_linear, 0, stream>>>(m_n_weights, m_n_matrix_weights, frozen_ranges(), m_optimize_matrix_params,
		                                                                                m_optimize_non_matrix_params, loss_scale, lr_t, m_beta1, m_beta2, m_epsilon, m_l2_reg,
		                                                                                weights_full_precision, weights, gradients, m_first_moments.data(), m_second_moments.data());
#else
		throw std::runtime_error("AdamOptimizer::step: needs a CUDA translation unit");
#endif
	}
	float learning_rate() const override { return m_learning_rate; }
	void set_learning_rate(float val) override { m_learning_rate = val; }
	uint32_t step() const override { return m_current_step; }
	uint32_t n_weights() const override { return m_n_weights; }
	T* custom_weights() const override { return nullptr; }

	void update_hyperparams(const json& params) override {
		if (params.contains("beta1")) m_beta1 = params["beta1"];
		if (params.contains("beta2")) m_beta2 = params["beta2"];
		if (params.contains("epsilon")) m_epsilon = params["epsilon"];
		if (params.contains("learning_rate")) m_learning_rate = params["learning_rate"];
		if (params.contains("l2_reg")) m_l2_reg = params["l2_reg"];
		if (params.contains("optimize_matrix_params")) m_optimize_matrix_params = params["optimize_matrix_params"];
		if (params.contains("optimize_non_matrix_params")) m_optimize_non_matrix_params = params["optimize_non_matrix_params"];
		if (params.contains("optimize_canonical_params")) m_optimize_canonical_params = params["optimize_canonical_params"];
		if (params.contains("optimize_delta_params")) m_optimize_delta_params = params["optimize_delta_params"];
		if (params.contains("optimize_params_components")) m_optimize_components = params["optimize_params_components"];
	}
	json hyperparams() const override {
		return {{"otype", "Adam"},
		        {"beta1", m_beta1},
		        {"beta2", m_beta2},
		        {"epsilon", m_epsilon},
		        {"learning_rate", m_learning_rate},
		        {"l2_reg", m_l2_reg},
		        {"optimize_matrix_params", m_optimize_matrix_params},
		        {"optimize_non_matrix_params", m_optimize_non_matrix_params},
		        {"optimize_canonical_params", m_optimize_canonical_params},
		        {"optimize_delta_params", m_optimize_delta_params},
		        {"optimize_params_components", m_optimize_components}};
	}
	json serialize() const override {
		json data;
		data["otype"] = "Adam";
		data["current_step"] = m_current_step;
		data["learning_rate"] = m_learning_rate;
		data["first_moments_binary"] = m_first_moments;
		data["second_moments_binary"] = m_second_moments;
		return data;
	}
	void deserialize(const json& data) override {
		m_first_moments = data["first_moments_binary"];
		m_second_moments = data["second_moments_binary"];
		m_current_step = data.value("current_step", 0u);
		if (data.contains("learning_rate")) m_learning_rate = data["learning_rate"];
		if (m_n_weights && (m_first_moments.size() != m_n_weights || m_second_moments.size() != m_n_weights))
			throw std::runtime_error("AdamOptimizer::deserialize: the stored moments do not fit the parameter block");
	}

private:
	/* what the group switches leave out: the canonical or the motion part as a whole, and named components that are
	 * switched off (components are laid out in the order the model lists them) */
	FrozenRanges frozen_ranges() const {
		FrozenRanges f;
		auto add = [&f](size_t b, size_t e) {
			if (e > b && f.n < 8) {
				f.begin[f.n] = (uint32_t)b;
				f.end[f.n] = (uint32_t)e;
				++f.n;
			}
		};
		if (m_n_canonical + m_n_delta == m_n_weights && m_n_delta > 0) {
			if (!m_optimize_canonical_params) add(0, m_n_canonical);
			if (!m_optimize_delta_params) add(m_n_canonical, m_n_weights);
		} else if (!m_optimize_canonical_params && m_n_canonical == m_n_weights) {
			add(0, m_n_weights);
		}
		if (m_components.is_array() && m_optimize_components.is_object()) {
			size_t offset = 0;
			for (const auto& entry : m_components) {
				if (!entry.is_array() || entry.size() != 2 || !entry[1].is_array() || entry[1].size() != 2) continue;
				const std::string name = entry[1][0];
				const size_t size = entry[1][1];
				if (m_optimize_components.contains(name) && m_optimize_components[name].is_boolean() && !m_optimize_components[name].get<bool>()) add(offset, offset + size);
				offset += size;
			}
		}
		return f;
	}

	uint32_t m_n_weights = 0, m_n_matrix_weights = 0, m_current_step = 0;
	size_t m_n_canonical = 0, m_n_delta = 0;
	json m_components, m_optimize_components = json::object();
	GPUMemory<float> m_first_moments, m_second_moments;
	float m_learning_rate = 1e-3f, m_beta1 = 0.9f, m_beta2 = 0.999f, m_epsilon = 1e-8f, m_l2_reg = 1e-8f;
	bool m_optimize_matrix_params = true, m_optimize_non_matrix_params = true, m_optimize_canonical_params = true, m_optimize_delta_params = true;
};

/* multiplies the nested optimizer's learning rate by decay_base every decay_interval steps from decay_start on */
template <typename T>
class ExponentialDecayOptimizer : public Optimizer<T> {
public:
	ExponentialDecayOptimizer(const json& params) {
		m_nested.reset(create_optimizer<T>(params.value("nested", json::object())));
		m_base_learning_rate = m_nested->learning_rate();
		update_hyperparams(params);
	}
	void allocate(uint32_t n_weights, const std::vector<std::pair<uint32_t, uint32_t>>& layer_sizes = {}) override { m_nested->allocate(n_weights, layer_sizes); }
	void set_param_groups(size_t n_canonical, size_t n_delta, const json& components) override { m_nested->set_param_groups(n_canonical, n_delta, components); }
	void step(cudaStream_t stream, float loss_scale, float* weights_full_precision, T* weights, const T* gradients) override {
		m_nested->step(stream, loss_scale, weights_full_precision, weights, gradients);
		const uint32_t s = step();
		if (m_decay_interval > 0 && s >= m_decay_start && (s - m_decay_start) % m_decay_interval == 0 && s <= m_decay_end)
			m_nested->set_learning_rate(m_nested->learning_rate() * m_decay_base);
	}
	float learning_rate() const override { return m_nested->learning_rate(); }
	void set_learning_rate(float val) override {
		m_base_learning_rate = val;
		m_nested->set_learning_rate(val);
	}
	uint32_t step() const override { return m_nested->step(); }
	uint32_t n_weights() const override { return m_nested->n_weights(); }
	T* custom_weights() const override { return m_nested->custom_weights(); }
	bool supports_nesting() const override { return true; }
	void update_hyperparams(const json& params) override {
		if (params.contains("decay_base")) m_decay_base = params["decay_base"];
		if (params.contains("decay_start")) m_decay_start = params["decay_start"];
		if (params.contains("decay_end")) m_decay_end = params["decay_end"];
		if (params.contains("decay_interval")) m_decay_interval = params["decay_interval"];
		if (params.contains("nested")) {
			const float before = m_nested->learning_rate();
			m_nested->update_hyperparams(params["nested"]);
			if (m_nested->learning_rate() != before) m_base_learning_rate = m_nested->learning_rate();
		}
	}
	json hyperparams() const override {
		return {{"otype", "ExponentialDecay"}, {"nested", m_nested->hyperparams()}, {"decay_base", m_decay_base}, {"decay_start", m_decay_start},
		        {"decay_end", m_decay_end},     {"decay_interval", m_decay_interval}};
	}
	json serialize() const override {
		json data = m_nested->serialize(); /* transparent: a reader that expects the nested optimizer finds its keys */
		data["base_learning_rate"] = m_base_learning_rate;
		return data;
	}
	void deserialize(const json& data) override {
		m_nested->deserialize(data);
		if (data.contains("base_learning_rate")) m_base_learning_rate = data["base_learning_rate"];
	}

private:
	std::unique_ptr<Optimizer<T>> m_nested;
	float m_base_learning_rate = 0.f, m_decay_base = 0.1f;
	uint32_t m_decay_start = 10000, m_decay_end = 0xFFFFFFFFu, m_decay_interval = 10000;
};

/* keeps a bias-corrected exponential moving average of the nested optimizer's weights and offers it for inference */
template <typename T>
class EmaOptimizer : public Optimizer<T> {
public:
	EmaOptimizer(const json& params) {
		m_nested.reset(create_optimizer<T>(params.value("nested", json::object())));
		update_hyperparams(params);
	}
	void allocate(uint32_t n_weights, const std::vector<std::pair<uint32_t, uint32_t>>& layer_sizes = {}) override {
		m_nested->allocate(n_weights, layer_sizes);
		if (m_ema_full_precision.size() != n_weights) {
			m_ema_full_precision.resize(n_weights);
			m_ema_weights.resize(n_weights);
			m_ema_full_precision.memset(0);
			m_ema_weights.memset(0);
		}
	}
	void set_param_groups(size_t n_canonical, size_t n_delta, const json& components) override { m_nested->set_param_groups(n_canonical, n_delta, components); }
	void step(cudaStream_t stream, float loss_scale, float* weights_full_precision, T* weights, const T* gradients) override {
		m_nested->step(stream, loss_scale, weights_full_precision, weights, gradients);
#if defined(__CUDACC__)
		const uint32_t n = n_weights();
		if (!n) return;
		const float t = (float)step();
		const float old_norm = m_full_precision ? 1.0f - std::pow(m_ema_decay, t - 1.0f) : 1.0f;
		const float new_norm_inv = m_full_precision ? 1.0f / (1.0f - std::pow(m_ema_decay, t)) : 1.0f;
		ema_step_kernel<T><<<n_blocks_linear(n), n_threads_linear, 0, stream>>>(n, m_ema_decay, old_norm, new_norm_inv, weights_full_precision, weights,
		                                                                     m_ema_full_precision.data(), m_ema_weights.data());
#else
		throw std::runtime_error("EmaOptimizer::step: needs a CUDA translation unit");
#endif
	}
	float learning_rate() const override { return m_nested->learning_rate(); }
	void set_learning_rate(float val) override { m_nested->set_learning_rate(val); }
	uint32_t step() const override { return m_nested->step(); }
	uint32_t n_weights() const override { return m_nested->n_weights(); }
	T* custom_weights() const override { return m_ema_weights.data(); }
	bool supports_nesting() const override { return true; }
	void update_hyperparams(const json& params) override {
		if (params.contains("decay")) m_ema_decay = params["decay"];
		if (params.contains("full_precision")) m_full_precision = params["full_precision"];
		if (params.contains("nested")) m_nested->update_hyperparams(params["nested"]);
	}
	json hyperparams() const override { return {{"otype", "Ema"}, {"nested", m_nested->hyperparams()}, {"decay", m_ema_decay}, {"full_precision", m_full_precision}}; }
	json serialize() const override {
		json data;
		data["otype"] = "Ema";
		data["nested"] = m_nested->serialize();
		data["ema_master_binary"] = m_ema_full_precision;
		return data;
	}
	void deserialize(const json& data) override {
		m_ema_full_precision = data["ema_master_binary"];
		m_nested->deserialize(data["nested"]);
#if defined(__CUDACC__)
		m_ema_weights.resize(m_ema_full_precision.size());
		const uint32_t n = (uint32_t)m_ema_full_precision.size();
		if (n) cast_kernel<T><<<n_blocks_linear(n), n_threads_linear>>>(n, m_ema_full_precision.data(), m_ema_weights.data());
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
#endif
	}

private:
	std::unique_ptr<Optimizer<T>> m_nested;
	GPUMemory<float> m_ema_full_precision;
	GPUMemory<T> m_ema_weights;
	float m_ema_decay = 0.99f;
	bool m_full_precision = true; /* debiased running mean kept in fp32 */
};

template <typename T>
Optimizer<T>* create_optimizer(const json& params) {
	const std::string otype = to_lower(params.value("otype", "Adam"));
	if (otype == "adam") return new AdamOptimizer<T>{params};
	if (otype == "exponentialdecay") return new ExponentialDecayOptimizer<T>{params};
	if (otype == "ema") return new EmaOptimizer<T>{params};
	throw std::runtime_error("create_optimizer: optimizer \"" + params.value("otype", "") + "\" is not part of this library (Adam, ExponentialDecay, Ema are)");
}

TCNN_NAMESPACE_END
