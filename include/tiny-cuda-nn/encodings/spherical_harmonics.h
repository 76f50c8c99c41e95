/* Degree-4 spherical harmonics of a direction given in [0,1]^3 (the view-direction encoding of the NeuS path,
 * configs/nerf/base.json:48-62, include/neural-graphics-primitives/nerf_network.h:251) and the identity encoding, as
 * Encoding<T> over the C interface. */
#pragma once
#include <tiny-cuda-nn/encoding.h>

#include <neus2b.h>

TCNN_NAMESPACE_BEGIN

template <typename T>
class SphericalHarmonicsEncoding : public Encoding<T> {
public:
	SphericalHarmonicsEncoding(uint32_t degree, uint32_t n_dims_to_encode) : m_degree{degree} {
		if (n_dims_to_encode != 3) throw std::runtime_error("SphericalHarmonicsEncoding: 3 input dimensions only");
		if (degree != 4) throw std::runtime_error("SphericalHarmonicsEncoding: degree 4 only");
		if (!std::is_same<T, __half>::value) throw std::runtime_error("SphericalHarmonicsEncoding: fp16 output only");
	}
	std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>* output = nullptr,
	                                      bool use_inference_params = false, bool prepare_input_gradients = false) override {
		(void)use_inference_params;
		(void)prepare_input_gradients;
		if (output && input.n()) {
#if defined(__CUDACC__)
			DenseColumns<float> x{stream, input, true, true};
			DenseColumns<T> y{stream, *output, false};
			neus2b_check_sh(neus2b_sh4_forward(input.n(), x.data(), x.copied() ? input.m() : input.stride(), (uint16_t*)y.data(), stream));
			y.scatter();
#else
			throw std::runtime_error("SphericalHarmonicsEncoding::forward: needs a CUDA translation unit");
#endif
		}
		return std::make_unique<Context>();
	}
	void backward_impl(cudaStream_t stream, const Context&, const GPUMatrixDynamic<float>&, const GPUMatrixDynamic<T>&, const GPUMatrixDynamic<T>&,
	                   GPUMatrixDynamic<float>* dL_dinput = nullptr, bool = false, EGradientMode = EGradientMode::Overwrite) override {
		/* the NeuS step takes no gradient with respect to the view direction of a static scene; where a caller asks for
		 * the matrix anyway (dynamic sequences add it to the motion's input gradient) it gets zeros */
		if (dL_dinput) dL_dinput->memset_async(stream, 0);
	}
	uint32_t input_width() const override { return 3; }
	uint32_t padded_output_width() const override { return 16; }
	uint32_t output_width() const override { return 16; }
	uint32_t required_input_alignment() const override { return 1; }
	void set_alignment(uint32_t alignment) override {
		if (16 % alignment) throw std::runtime_error("SphericalHarmonicsEncoding: 16 outputs cannot be aligned to " + std::to_string(alignment));
	}
	uint32_t min_alignment() const override { return 1; }
	MatrixLayout preferred_output_layout() const override { return AoS; }
	void set_params(T*, T*, T*, T*) override {}
	void initialize_params(pcg32&, float*, T*, T*, T*, T*, float = 1) override {}
	size_t n_params() const override { return 0; }
	json hyperparams() const override { return {{"otype", "SphericalHarmonics"}, {"degree", m_degree}}; }

private:
	static void neus2b_check_sh(int rc) {
		if (rc) throw std::runtime_error(std::string("SphericalHarmonicsEncoding::forward: ") + neus2b_error_string(rc));
	}
	uint32_t m_degree;
};

#if defined(__CUDACC__)
template <typename T>
__global__ void identity_kernel(const uint32_t n_elements, const uint32_t n_dims, const uint32_t n_padded, const float scale, const float offset,
                                MatrixView<float> in, MatrixView<T> out) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i >= n_elements) return;
	const uint32_t col = i / n_padded, row = i - col * n_padded;
	out(row, col) = row < n_dims ? (T)(in(row, col) * scale + offset) : (T)1.0f;
}
template <typename T>
__global__ void identity_backward_kernel(const uint32_t n_elements, const uint32_t n_dims, const float scale, MatrixView<T> dL_dy, MatrixView<float> dL_dx) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i >= n_elements) return;
	const uint32_t col = i / n_dims, row = i - col * n_dims;
	dL_dx(row, col) = (float)dL_dy(row, col) * scale;
}
#endif

/* y = x * scale + offset, padded with ones (the constant input lets a following layer learn a bias) */
template <typename T>
class IdentityEncoding : public Encoding<T> {
public:
	IdentityEncoding(uint32_t n_dims_to_encode, float scale = 1.0f, float offset = 0.0f) : m_n_dims{n_dims_to_encode}, m_scale{scale}, m_offset{offset}, m_n_padded{n_dims_to_encode} {}
	std::unique_ptr<Context> forward_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>* output = nullptr,
	                                      bool use_inference_params = false, bool prepare_input_gradients = false) override {
		(void)use_inference_params;
		(void)prepare_input_gradients;
#if defined(__CUDACC__)
		if (output && output->n_elements())
			identity_kernel<T><<<n_blocks_linear(output->n_elements()), n_threads_linear, 0, stream>>>(output->n_elements(), m_n_dims, m_n_padded, m_scale, m_offset,
			                                                                                         input.view(), output->view());
#endif
		return std::make_unique<Context>();
	}
	void backward_impl(cudaStream_t stream, const Context&, const GPUMatrixDynamic<float>& input, const GPUMatrixDynamic<T>&, const GPUMatrixDynamic<T>& dL_doutput,
	                   GPUMatrixDynamic<float>* dL_dinput = nullptr, bool = false, EGradientMode = EGradientMode::Overwrite) override {
#if defined(__CUDACC__)
		if (dL_dinput && dL_dinput->n_elements())
			identity_backward_kernel<T><<<n_blocks_linear(dL_dinput->n_elements()), n_threads_linear, 0, stream>>>(dL_dinput->n_elements(), m_n_dims, m_scale,
			                                                                                                    dL_doutput.view(), dL_dinput->view());
#endif
		(void)input;
	}
	uint32_t input_width() const override { return m_n_dims; }
	uint32_t padded_output_width() const override { return m_n_padded; }
	uint32_t output_width() const override { return m_n_dims; }
	uint32_t required_input_alignment() const override { return 1; }
	void set_alignment(uint32_t alignment) override { m_n_padded = next_multiple(m_n_dims, alignment); }
	uint32_t min_alignment() const override { return 1; }
	MatrixLayout preferred_output_layout() const override { return AoS; }
	void set_params(T*, T*, T*, T*) override {}
	void initialize_params(pcg32&, float*, T*, T*, T*, T*, float = 1) override {}
	size_t n_params() const override { return 0; }
	json hyperparams() const override { return {{"otype", "Identity"}, {"scale", m_scale}, {"offset", m_offset}}; }

private:
	uint32_t m_n_dims;
	float m_scale, m_offset;
	uint32_t m_n_padded;
};

TCNN_NAMESPACE_END
