/* tiny-cuda-nn/loss.h of the B200-native stand-in: Loss<T> and the json factory.  The NeuS step computes its own loss on
 * composited rays (src/testbed_nerf.cu:1556-1960); a Loss object is still created from the "loss" block and handed to
 * every Trainer (src/testbed.cu:2192, :2303, :2317, :2332).  L2, RelativeL2, L1 and Huber are provided, as one
 * elementwise kernel parameterised by the loss. */
#pragma once
#include <tiny-cuda-nn/object.h>

TCNN_NAMESPACE_BEGIN

template <typename T>
class Loss : public ObjectWithMutableHyperparams {
public:
	virtual ~Loss() {}
	/* prediction [stride x n] (the first `dims` rows count), target [dims x n]; writes per-entry loss values and
	 * d(loss * loss_scale)/d prediction, both divided by the number of entries */
	virtual void evaluate(cudaStream_t stream, const uint32_t stride, const uint32_t dims, const float loss_scale, const GPUMatrix<T>& prediction,
	                      const GPUMatrix<float>& target, GPUMatrix<float>& values, GPUMatrix<T>& gradients, const GPUMatrix<float>* data_pdf = nullptr) const = 0;
	void evaluate(const float loss_scale, const GPUMatrix<T>& prediction, const GPUMatrix<float>& target, GPUMatrix<float>& values, GPUMatrix<T>& gradients,
	              const GPUMatrix<float>* data_pdf = nullptr) const {
		evaluate(nullptr, prediction.m(), prediction.m(), loss_scale, prediction, target, values, gradients, data_pdf);
	}
};

enum class ElementwiseLoss { L2, RelativeL2, L1, Huber };

#if defined(__CUDACC__)
template <typename T>
__global__ void elementwise_loss_kernel(const uint32_t n_elements, const uint32_t stride, const uint32_t dims, const float loss_scale, const ElementwiseLoss kind,
                                        const float huber_delta, const T* __restrict__ predictions, const float* __restrict__ targets, float* __restrict__ values,
                                        T* __restrict__ gradients, const float* __restrict__ data_pdf) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i >= n_elements) return;
	const uint32_t row = i % stride, col = i / stride;
	if (row >= dims) {
		values[i] = 0.0f;
		gradients[i] = (T)0.0f;
		return;
	}
	const uint32_t n_total = n_elements / stride * dims;
	const float prediction = (float)predictions[i];
	const float pdf = data_pdf ? data_pdf[col * dims + row] : 1.0f;
	const float diff = prediction - targets[col * dims + row];
	float value, gradient;
	switch (kind) {
		case ElementwiseLoss::L2:
			value = diff * diff;
			gradient = 2.0f * diff;
			break;
		case ElementwiseLoss::RelativeL2: {
			const float scale = 1.0f / (prediction * prediction + 1e-2f);
			value = diff * diff * scale;
			gradient = 2.0f * diff * scale;
			break;
		}
		case ElementwiseLoss::L1:
			value = fabsf(diff);
			gradient = diff > 0.0f ? 1.0f : (diff < 0.0f ? -1.0f : 0.0f);
			break;
		default: { /* Huber: quadratic inside delta, linear outside, scaled so that the quadratic part is diff^2 / (2 delta) * 2 */
			const float a = fabsf(diff);
			if (a <= huber_delta) {
				value = 0.5f * diff * diff / huber_delta;
				gradient = diff / huber_delta;
			} else {
				value = a - 0.5f * huber_delta;
				gradient = diff > 0.0f ? 1.0f : -1.0f;
			}
		}
	}
	values[i] = value / pdf / (float)n_total;
	gradients[i] = (T)(loss_scale * gradient / pdf / (float)n_total);
}
#endif

template <typename T>
class ElementwiseLossImpl : public Loss<T> {
public:
	ElementwiseLossImpl(ElementwiseLoss kind, const char* name) : m_kind{kind}, m_name{name} {}
	void evaluate(cudaStream_t stream, const uint32_t stride, const uint32_t dims, const float loss_scale, const GPUMatrix<T>& prediction, const GPUMatrix<float>& target,
	              GPUMatrix<float>& values, GPUMatrix<T>& gradients, const GPUMatrix<float>* data_pdf = nullptr) const override {
		if (prediction.n() != target.n() || prediction.m() != stride || target.m() != dims || values.n_elements() != prediction.n_elements() ||
		    gradients.n_elements() != prediction.n_elements())
			throw std::runtime_error(std::string(m_name) + " loss: matrix shapes do not fit together");
#if defined(__CUDACC__)
		const uint32_t n = prediction.n_elements();
		if (n)
			elementwise_loss_kernel<T><<<n_blocks_linear(n), n_threads_linear, 0, stream>>>(n, stride, dims, loss_scale, m_kind, m_huber_delta, prediction.data(), target.data(),
			                                                                             values.data(), gradients.data(), data_pdf ? data_pdf->data() : nullptr);
#else
		throw std::runtime_error("Loss::evaluate: needs a CUDA translation unit");
#endif
	}
	void update_hyperparams(const json& params) override {
		if (params.contains("delta")) m_huber_delta = params["delta"];
	}
	json hyperparams() const override {
		json r = {{"otype", m_name}};
		if (m_kind == ElementwiseLoss::Huber) r["delta"] = m_huber_delta;
		return r;
	}

private:
	ElementwiseLoss m_kind;
	const char* m_name;
	float m_huber_delta = 0.1f;
};

template <typename T>
Loss<T>* create_loss(const json& params) {
	const std::string otype = to_lower(params.value("otype", "RelativeL2"));
	Loss<T>* loss;
	if (otype == "l2")
		loss = new ElementwiseLossImpl<T>{ElementwiseLoss::L2, "L2"};
	else if (otype == "relativel2")
		loss = new ElementwiseLossImpl<T>{ElementwiseLoss::RelativeL2, "RelativeL2"};
	else if (otype == "l1")
		loss = new ElementwiseLossImpl<T>{ElementwiseLoss::L1, "L1"};
	else if (otype == "huber")
		loss = new ElementwiseLossImpl<T>{ElementwiseLoss::Huber, "Huber"};
	else
		throw std::runtime_error("create_loss: loss \"" + params.value("otype", "") + "\" is not part of this library (L2, RelativeL2, L1, Huber are)");
	loss->update_hyperparams(params);
	return loss;
}

TCNN_NAMESPACE_END
