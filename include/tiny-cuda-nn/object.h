/* tiny-cuda-nn/object.h of the B200-native stand-in: the abstract interfaces everything trainable derives from.
 * ParametricObject<PARAMS_T> owns no memory: a Trainer hands it slices of one parameter block (set_params /
 * initialize_params).  DifferentiableObject<T, PARAMS_T, COMPUTE_T> maps input matrices of T to output matrices of
 * COMPUTE_T; the public entry points check shapes and forward to the *_impl virtuals that the concrete classes
 * override (include/neural-graphics-primitives/trainable_buffer.cuh:29-135, nerf_network.h:87-132, :317-326,
 * transform_network.h:26-170 show the overridden set). */
#pragma once
#include <tiny-cuda-nn/common.h>
#include <tiny-cuda-nn/common_device.h>
#include <tiny-cuda-nn/gpu_matrix.h>
#include <tiny-cuda-nn/gpu_memory.h>
#include <tiny-cuda-nn/random.h>

#include <json/json.hpp>

TCNN_NAMESPACE_BEGIN
using json = nlohmann::json;

class Object {
public:
	virtual ~Object() {}
	virtual json hyperparams() const = 0;
};

class ObjectWithMutableHyperparams : public Object {
public:
	virtual ~ObjectWithMutableHyperparams() {}
	virtual void update_hyperparams(const json& params) = 0;
};

template <typename PARAMS_T>
class ParametricObject : public Object {
public:
	virtual ~ParametricObject() {}
	virtual void set_params(PARAMS_T* params, PARAMS_T* inference_params, PARAMS_T* backward_params, PARAMS_T* gradients) = 0;
	virtual void initialize_params(pcg32& rnd, float* params_full_precision, PARAMS_T* params, PARAMS_T* inference_params, PARAMS_T* backward_params,
	                               PARAMS_T* gradients, float scale = 1) = 0;
	virtual size_t n_params() const = 0;
	/* dynamic sequences: the parameters that belong to the canonical model and to the per-frame motion, and the
	 * named parts the optimizer may freeze (nerf_network.h:902-925) */
	virtual size_t n_params_canonical() const { return n_params(); }
	virtual size_t n_params_delta() const { return 0; }
	virtual json n_params_components() const { return json::array(); }
	virtual std::vector<std::pair<uint32_t, uint32_t>> layer_sizes() const = 0;
	virtual std::vector<std::pair<uint32_t, uint32_t>> layer_sizes_canonical() const { return layer_sizes(); }
};

struct Context {
	virtual ~Context() {}
};

#if defined(__CUDACC__)
template <typename C>
__global__ void cast_rows_kernel(const uint32_t n_elements, const uint32_t rows, MatrixView<C> in, MatrixView<float> out) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i >= n_elements) return;
	const uint32_t col = i / rows, row = i - col * rows;
	out(row, col) = (float)in(row, col);
}
template <typename C>
__global__ void one_hot_rows_kernel(const uint32_t batch, const uint32_t dim, MatrixView<C> out) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i < batch) out(dim, i) = (C)1.0f;
}
#endif

template <typename T, typename PARAMS_T, typename COMPUTE_T = PARAMS_T>
class DifferentiableObject : public ParametricObject<PARAMS_T> {
public:
	virtual ~DifferentiableObject() {}

	/* ---- inference */
	virtual void inference_mixed_precision_impl(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<COMPUTE_T>& output,
	                                            bool use_inference_params = true) = 0;
	void inference_mixed_precision(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<COMPUTE_T>& output, bool use_inference_params = true) {
		check_shapes("inference_mixed_precision", input, &output, nullptr);
		inference_mixed_precision_impl(stream, input, output, use_inference_params);
	}
	void inference_mixed_precision(const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<COMPUTE_T>& output, bool use_inference_params = true) {
		inference_mixed_precision(nullptr, input, output, use_inference_params);
	}
	/* full-precision result */
	void inference(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<float>& output) {
		if constexpr (std::is_same<COMPUTE_T, float>::value) {
			inference_mixed_precision(stream, input, output, true);
		} else {
#if defined(__CUDACC__)
			if (output.m() != output_width() || output.n() != input.n()) throw std::runtime_error("inference: the output must be output_width() x batch");
			GPUMatrixDynamic<COMPUTE_T> tmp{padded_output_width(), input.n(), stream, output.layout()};
			inference_mixed_precision(stream, input, tmp, true);
			const uint32_t n = output.n_elements();
			if (n) cast_rows_kernel<COMPUTE_T><<<n_blocks_linear(n), n_threads_linear, 0, stream>>>(n, output.m(), tmp.view(), output.view());
#else
			throw std::runtime_error("inference: needs a CUDA translation unit");
#endif
		}
	}
	void inference(const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<float>& output) { inference(nullptr, input, output); }

	/* ---- forward: keeps what backward needs in the returned context */
	virtual std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<COMPUTE_T>* output = nullptr,
	                                              bool use_inference_params = false, bool prepare_input_gradients = false) = 0;
	std::unique_ptr<Context> forward(cudaStream_t stream, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<COMPUTE_T>* output = nullptr,
	                                 bool use_inference_params = false, bool prepare_input_gradients = false) {
		check_shapes("forward", input, output, nullptr);
		return forward_impl(stream, input, output, use_inference_params, prepare_input_gradients);
	}
	std::unique_ptr<Context> forward(const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<COMPUTE_T>* output = nullptr, bool use_inference_params = false,
	                                 bool prepare_input_gradients = false) {
		return forward(nullptr, input, output, use_inference_params, prepare_input_gradients);
	}

	/* ---- backward */
	virtual void backward_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<COMPUTE_T>& output,
	                           const GPUMatrixDynamic<COMPUTE_T>& dL_doutput, GPUMatrixDynamic<T>* dL_dinput = nullptr, bool use_inference_params = false,
	                           EGradientMode param_gradients_mode = EGradientMode::Overwrite) = 0;
	void backward(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<COMPUTE_T>& output,
	              const GPUMatrixDynamic<COMPUTE_T>& dL_doutput, GPUMatrixDynamic<T>* dL_dinput = nullptr, bool use_inference_params = false,
	              EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		check_shapes("backward", input, &output, &dL_doutput);
		if (dL_dinput && (dL_dinput->m() != input_width() || dL_dinput->n() != input.n()))
			throw std::runtime_error("backward: dL_dinput must be input_width() x batch");
		backward_impl(stream, ctx, input, output, dL_doutput, dL_dinput, use_inference_params, param_gradients_mode);
	}
	void backward(const Context& ctx, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<COMPUTE_T>& output, const GPUMatrixDynamic<COMPUTE_T>& dL_doutput,
	              GPUMatrixDynamic<T>* dL_dinput = nullptr, bool use_inference_params = false, EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		backward(nullptr, ctx, input, output, dL_doutput, dL_dinput, use_inference_params, param_gradients_mode);
	}

	/* ---- second order: the derivative of (dL_dinput of backward) with respect to dL_doutput, the parameters and the
	 * input, contracted with dL_ddLdinput (the eikonal term, nerf_network.h:534-571) */
	virtual void backward_backward_input_impl(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<T>& dL_ddLdinput,
	                                          const GPUMatrixDynamic<COMPUTE_T>& dL_doutput, GPUMatrixDynamic<COMPUTE_T>* dL_ddLdoutput = nullptr,
	                                          GPUMatrixDynamic<T>* dL_dinput = nullptr, bool use_inference_params = false,
	                                          EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		throw std::runtime_error("backward_backward_input: this object has no second-order backward pass");
	}
	void backward_backward_input(cudaStream_t stream, const Context& ctx, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<T>& dL_ddLdinput,
	                             const GPUMatrixDynamic<COMPUTE_T>& dL_doutput, GPUMatrixDynamic<COMPUTE_T>* dL_ddLdoutput = nullptr,
	                             GPUMatrixDynamic<T>* dL_dinput = nullptr, bool use_inference_params = false,
	                             EGradientMode param_gradients_mode = EGradientMode::Overwrite) {
		if (input.m() != input_width() || dL_ddLdinput.n() != input.n() || dL_doutput.n() != input.n())
			throw std::runtime_error("backward_backward_input: matrix shapes do not fit the object");
		backward_backward_input_impl(stream, ctx, input, dL_ddLdinput, dL_doutput, dL_ddLdoutput, dL_dinput, use_inference_params, param_gradients_mode);
	}

	/* ---- d output[dim] / d input, by one forward and one backward pass (src/testbed_nerf.cu:4033) */
	void input_gradient(cudaStream_t stream, uint32_t dim, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<T>& d_dinput, GPUMatrixDynamic<COMPUTE_T>* output = nullptr,
	                    bool use_inference_params = true) {
#if defined(__CUDACC__)
		if (dim >= padded_output_width()) throw std::runtime_error("input_gradient: no such output dimension");
		const uint32_t batch = input.n();
		GPUMatrixDynamic<COMPUTE_T> out_local{padded_output_width(), batch, stream, output ? output->layout() : CM};
		GPUMatrixDynamic<COMPUTE_T>& out = output ? *output : out_local;
		GPUMatrixDynamic<COMPUTE_T> d_doutput{padded_output_width(), batch, stream, out.layout()};
		d_doutput.memset_async(stream, 0);
		if (batch) one_hot_rows_kernel<COMPUTE_T><<<n_blocks_linear(batch), n_threads_linear, 0, stream>>>(batch, dim, d_doutput.view());
		auto ctx = forward(stream, input, &out, use_inference_params, true);
		backward(stream, *ctx, input, out, d_doutput, &d_dinput, use_inference_params, EGradientMode::Ignore);
#else
		throw std::runtime_error("input_gradient: needs a CUDA translation unit");
#endif
	}

	/* ---- one activation of one layer as a grey value, for the viewer (src/testbed_nerf.cu:2774) */
	virtual void visualize_activation(cudaStream_t stream, uint32_t layer, uint32_t dimension, const GPUMatrixDynamic<T>& input, GPUMatrixDynamic<float>& output) {
		throw std::runtime_error("visualize_activation: the viewer is not part of this library");
	}

	virtual uint32_t input_width() const = 0;
	virtual uint32_t padded_output_width() const = 0;
	virtual uint32_t output_width() const = 0;
	virtual uint32_t required_input_alignment() const = 0;

private:
	void check_shapes(const char* who, const GPUMatrixDynamic<T>& input, const GPUMatrixDynamic<COMPUTE_T>* output, const GPUMatrixDynamic<COMPUTE_T>* dL_doutput) const {
		if (input.m() != input_width()) throw std::runtime_error(std::string(who) + ": the input has " + std::to_string(input.m()) + " rows, the object takes " + std::to_string(input_width()));
		if (output && (output->m() != padded_output_width() || output->n() != input.n()))
			throw std::runtime_error(std::string(who) + ": the output must be padded_output_width() x batch");
		if (dL_doutput && (dL_doutput->m() != padded_output_width() || dL_doutput->n() != input.n()))
			throw std::runtime_error(std::string(who) + ": dL_doutput must be padded_output_width() x batch");
	}
};

TCNN_NAMESPACE_END
