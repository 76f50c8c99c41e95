/* tiny-cuda-nn/encoding.h of the B200-native stand-in: Encoding<T> (float coordinates in, T features out) and the json
 * factory.  The concrete encodings are the ones the NeuS path instantiates (configs/nerf/base.json:29-62): the
 * multiresolution hash grid (encodings/grid.h), degree-4 spherical harmonics, the identity, and the Composite that
 * NerfNetwork builds for the view direction (include/neural-graphics-primitives/nerf_network.h:41-50).  Anything else
 * is refused by name at construction. */
#pragma once
#include <tiny-cuda-nn/object.h>

TCNN_NAMESPACE_BEGIN

template <typename T>
class Encoding : public DifferentiableObject<float, T, T> {
public:
	virtual ~Encoding() {}

	void inference_mixed_precision_impl(cudaStream_t stream, const GPUMatrixDynamic<float>& input, GPUMatrixDynamic<T>& output,
	                                    bool use_inference_params = true) override {
		this->forward(stream, input, &output, use_inference_params, false);
	}

	/* outputs are padded up to a multiple of the alignment the consumer needs (16 for the fused MLPs) */
	virtual void set_alignment(uint32_t alignment) = 0;
	virtual uint32_t min_alignment() const = 0;
	virtual MatrixLayout preferred_output_layout() const = 0;

	/* progressive training of the fork: the encoding is told the step and masks its fine levels itself
	 * (src/testbed.cu:2641-2647) */
	virtual void set_training_step(int training_step) { (void)training_step; }

	std::vector<std::pair<uint32_t, uint32_t>> layer_sizes() const override { return {}; }
};

template <typename T>
Encoding<T>* create_encoding(uint32_t n_dims_to_encode, const json& params, uint32_t alignment = 8);

TCNN_NAMESPACE_END

#include <tiny-cuda-nn/encodings/grid.h>
#include <tiny-cuda-nn/encodings/spherical_harmonics.h>

TCNN_NAMESPACE_BEGIN

template <typename T>
Encoding<T>* create_encoding(uint32_t n_dims_to_encode, const json& params, uint32_t alignment) {
	const std::string otype = to_lower(params.value("otype", "OneBlob"));
	Encoding<T>* result = nullptr;
	if (otype == "hashgrid" || otype == "grid" || otype == "densegrid" || otype == "tiledgrid") {
		result = create_grid_encoding<T>(n_dims_to_encode, params);
	} else if (otype == "sphericalharmonics") {
		result = new SphericalHarmonicsEncoding<T>{params.value("degree", 4u), n_dims_to_encode};
	} else if (otype == "identity") {
		result = new IdentityEncoding<T>{n_dims_to_encode, params.value("scale", 1.0f), params.value("offset", 0.0f)};
	} else if (otype == "composite") {
		/* the nested encodings split the input dimensions in order; the last one takes what is left.  Only nestings
		 * that reduce to a single encoding with input are built: that is the view-direction encoding of the NeuS
		 * configuration (spherical harmonics over 3 dimensions + an identity over the 0 extra dimensions). */
		if (!params.contains("nested") || !params["nested"].is_array() || params["nested"].empty())
			throw std::runtime_error("create_encoding: a Composite encoding needs a non-empty \"nested\" array");
		uint32_t remaining = n_dims_to_encode;
		const json* live = nullptr;
		uint32_t live_dims = 0;
		const auto& nested = params["nested"];
		for (size_t i = 0; i < nested.size(); ++i) {
			const bool last = i + 1 == nested.size();
			uint32_t dims = last ? remaining : std::min(remaining, nested[i].value("n_dims_to_encode", remaining));
			remaining -= dims;
			if (dims == 0) continue;
			if (live) throw std::runtime_error("create_encoding: a Composite of several non-empty encodings is not part of this library");
			live = &nested[i];
			live_dims = dims;
		}
		if (!live) throw std::runtime_error("create_encoding: the Composite encoding encodes no dimension");
		return create_encoding<T>(live_dims, *live, alignment);
	} else {
		throw std::runtime_error("create_encoding: encoding \"" + params.value("otype", "OneBlob") + "\" is not part of this library (HashGrid, SphericalHarmonics, Identity, Composite are)");
	}
	if (alignment > 0) result->set_alignment(alignment);
	return result;
}

TCNN_NAMESPACE_END
