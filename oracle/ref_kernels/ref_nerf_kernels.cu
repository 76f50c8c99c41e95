/* TEST INFRASTRUCTURE, not product code: the reference's own CUDA kernels of the NeuS training step, made callable.
 *
 * This translation unit includes the reference's src/testbed_nerf.cu where it lies in a reference checkout (given on the
 * include path at build time; nothing of it is copied), so that its file-scope kernels are visible, and wraps the ones
 * on the hot path in extern "C" launchers that take plain device pointers:
 *   generate_training_samples_nerf_with_global_movement   (src/testbed_nerf.cu:1253)
 *   compute_loss_kernel_train_nerf_with_global_movement    (src/testbed_nerf.cu:1465)
 *   generate_grid_samples_nerf_nonuniform, splat_grid_samples_nerf_max_nearest_neighbor, ema_grid_samples_nerf,
 *   grid_to_bitfield, bitfield_max_pool                    (src/testbed_nerf.cu:630-785, launched as in :3287-3391)
 *   Testbed::NerfTracer::init_rays_from_camera / trace + shade_kernel_nerf (src/testbed_nerf.cu:2398-2660, driven as in
 *   Testbed::render_nerf, :2671-2800), with the reference's NerfNetwork<__half> over this repository's layered kernels
 * The launch arguments mirror Testbed::train_nerf_step (:3797-3906) and update_density_grid_nerf (:3327-3391) for a
 * static scene with the default switches.  The reference's tiny-cuda-nn fork is not vendored: the headers under
 * include/tiny-cuda-nn of this repository stand in for it, so pcg32, morton3D_invert, logistic and reduce_sum come from
 * there; everything else the kernels execute is the reference's code.
 *
 * Built by oracle/build_ref_kernels.py into oracle/_ref/libref_nerf_kernels.so (git-ignored; it travels to the GPU
 * machine with the tree).  Only tests load it: they run these kernels and this repository's kernels on the same inputs. */
#include <src/testbed_nerf.cu>

#include <cstring>

using namespace ngp;
using namespace tcnn;
using namespace Eigen;

namespace {

struct RefDataset {
	GPUMemory<TrainingImageMetadata> metadata;
	GPUMemory<TrainingXForm> xforms;
	GPUMemory<Array3f> exposure;
};

/* images of one size, 8-bit RGBA, pinhole cameras: what neus2b_dataset describes */
RefDataset make_dataset(uint32_t n_images, uint32_t width, uint32_t height, const uint32_t* d_pixels, const float* h_xforms, const float* h_focal,
                        const float* h_principal) {
	std::vector<TrainingImageMetadata> meta(n_images);
	std::vector<TrainingXForm> xf(n_images);
	for (uint32_t i = 0; i < n_images; ++i) {
		meta[i].pixels = d_pixels + (size_t)i * width * height;
		meta[i].image_data_type = EImageDataType::Byte;
		meta[i].resolution = Vector2i((int)width, (int)height);
		meta[i].focal_length = Vector2f(h_focal[2 * i], h_focal[2 * i + 1]);
		meta[i].principal_point = Vector2f(h_principal[2 * i], h_principal[2 * i + 1]);
		std::memcpy(xf[i].start.data(), h_xforms + 12 * i, 12 * sizeof(float)); /* 3x4, column major on both sides */
		xf[i].end = xf[i].start;
	}
	RefDataset d;
	d.metadata.resize_and_copy_from_host(meta);
	d.xforms.resize_and_copy_from_host(xf);
	d.exposure.resize(n_images);
	d.exposure.memset(0);
	return d;
}

int guarded(const std::function<void()>& f) {
	try {
		f();
		return cudaGetLastError() == cudaSuccess ? 0 : -2;
	} catch (const std::exception& e) {
		std::fprintf(stderr, "ref_nerf_kernels: %s\n", e.what());
		return -1;
	}
}

}  // namespace

extern "C" {

/* sizes the tests need to lay their buffers out like the reference does */
uint32_t ref_sizeof_nerf_coordinate() { return (uint32_t)sizeof(NerfCoordinate); }
uint32_t ref_sizeof_ray() { return (uint32_t)sizeof(Ray); }
uint32_t ref_nerf_gridsize() { return NERF_GRIDSIZE(); }
uint32_t ref_n_max_random_samples_per_ray() { return N_MAX_RANDOM_SAMPLES_PER_RAY(); }
float ref_loss_scale() { return Testbed::LOSS_SCALE; }

/* Outputs: d_ray_counter[1], d_numsteps_counter[1] (both cleared here), d_ray_indices[n_rays], d_rays[n_rays][6],
 * d_numsteps[n_rays][2] {count, base}, d_coords[max_samples][7].  rotation / transition: fp16 device arrays of the
 * accumulated movement or NULL. */
int ref_generate_training_samples(uint32_t n_rays, uint32_t n_rays_total, uint64_t rng_state, uint64_t rng_inc, uint32_t max_samples, uint32_t n_images,
                                  uint32_t width, uint32_t height, const uint32_t* d_pixels, const float* h_xforms, const float* h_focal,
                                  const float* h_principal, const uint8_t* d_bitfield, int snap_to_pixel_centers, float cone_angle_constant,
                                  uint32_t training_step, const uint16_t* d_rotation, const uint16_t* d_transition, const float* first_frame_offset,
                                  uint32_t* d_ray_counter, uint32_t* d_numsteps_counter, uint32_t* d_ray_indices, float* d_rays, uint32_t* d_numsteps,
                                  float* d_coords) {
	return guarded([&] {
		RefDataset ds = make_dataset(n_images, width, height, d_pixels, h_xforms, h_focal, h_principal);
		default_rng_t rng;
		rng.state = rng_state;
		rng.inc = rng_inc;
		cudaStream_t stream = nullptr;
		CUDA_CHECK_THROW(cudaMemsetAsync(d_ray_counter, 0, sizeof(uint32_t), stream));
		CUDA_CHECK_THROW(cudaMemsetAsync(d_numsteps_counter, 0, sizeof(uint32_t), stream));
		const BoundingBox aabb{Vector3f::Zero(), Vector3f::Ones()};
		linear_kernel(generate_training_samples_nerf_with_global_movement, 0, stream, n_rays, aabb, max_samples, n_rays_total, rng, d_ray_counter,
		              d_numsteps_counter, d_ray_indices, (Ray*)d_rays, d_numsteps, PitchedPtr<NerfCoordinate>((NerfCoordinate*)d_coords, 1, 0, 0), n_images,
		              ds.metadata.data(), ds.xforms.data(), d_bitfield, false, (float*)nullptr, snap_to_pixel_centers != 0, false, cone_angle_constant,
		              (const float*)nullptr, Vector2i::Zero(), (const float*)nullptr, (const float*)nullptr, (const float*)nullptr, Vector2i::Zero(),
		              (const float*)nullptr, 0u, 0u, training_step, (const network_precision_t*)d_rotation, (const network_precision_t*)d_transition,
		              Vector3f(first_frame_offset[0], first_frame_offset[1], first_frame_offset[2]));
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
	});
}

/* The loss pass on what ref_generate_training_samples left behind.  d_network_output [samples][16] fp16.
 * Outputs: d_compacted_counter[1] (cleared here), d_numsteps rewritten to {compacted count, compacted base} per kept ray,
 * d_coords_compacted[target][7], d_dloss_doutput[target][16] fp16 (cleared here), d_loss / d_ek_loss / d_mask_loss [n_rays]
 * (cleared here). */
int ref_compute_loss(uint32_t n_rays, uint32_t n_rays_total, uint64_t rng_state, uint64_t rng_inc, uint32_t target_batch_size, uint32_t n_images,
                     uint32_t width, uint32_t height, const uint32_t* d_pixels, const float* h_xforms, const float* h_focal, const float* h_principal,
                     const uint32_t* d_ray_counter, const uint16_t* d_network_output, const uint32_t* d_ray_indices, const float* d_rays, uint32_t* d_numsteps,
                     const float* d_coords, int random_bg_color, const float* background_color, int snap_to_pixel_centers, float variance,
                     uint32_t training_step, const uint16_t* d_rotation, const uint16_t* d_transition, const float* first_frame_offset,
                     float mask_loss_weight, float ek_loss_weight, float cos_anneal_ratio, uint32_t* d_compacted_counter, float* d_coords_compacted,
                     uint16_t* d_dloss_doutput, float* d_loss, float* d_ek_loss, float* d_mask_loss) {
	return guarded([&] {
		RefDataset ds = make_dataset(n_images, width, height, d_pixels, h_xforms, h_focal, h_principal);
		default_rng_t rng;
		rng.state = rng_state;
		rng.inc = rng_inc;
		cudaStream_t stream = nullptr;
		GPUMemory<float> mean_density(1);
		mean_density.memset(0);
		CUDA_CHECK_THROW(cudaMemsetAsync(d_compacted_counter, 0, sizeof(uint32_t), stream));
		CUDA_CHECK_THROW(cudaMemsetAsync(d_dloss_doutput, 0, (size_t)target_batch_size * 16 * sizeof(uint16_t), stream));
		CUDA_CHECK_THROW(cudaMemsetAsync(d_loss, 0, n_rays * sizeof(float), stream));
		CUDA_CHECK_THROW(cudaMemsetAsync(d_ek_loss, 0, n_rays * sizeof(float), stream));
		CUDA_CHECK_THROW(cudaMemsetAsync(d_mask_loss, 0, n_rays * sizeof(float), stream));
		const BoundingBox aabb{Vector3f::Zero(), Vector3f::Ones()};
		linear_kernel(compute_loss_kernel_train_nerf_with_global_movement, 0, stream, n_rays, aabb, n_rays_total, rng, target_batch_size, d_ray_counter,
		              Testbed::LOSS_SCALE, 16, (const float*)nullptr, (float*)nullptr, Vector2i::Zero(), ELossType::L2,
		              Array3f(background_color[0], background_color[1], background_color[2]), EColorSpace::Linear, random_bg_color != 0, false, n_images,
		              ds.metadata.data(), (const network_precision_t*)d_network_output, d_compacted_counter, d_ray_indices, (const Ray*)d_rays, d_numsteps,
		              PitchedPtr<const NerfCoordinate>((const NerfCoordinate*)d_coords, 1, 0, 0),
		              PitchedPtr<NerfCoordinate>((NerfCoordinate*)d_coords_compacted, 1, 0, 0), (network_precision_t*)d_dloss_doutput, ELossType::Huber, d_loss,
		              d_ek_loss, d_mask_loss, false, (float*)nullptr, ENerfActivation::Logistic, ENerfActivation::Exponential, snap_to_pixel_centers != 0,
		              (float*)nullptr, (const float*)nullptr, (const float*)nullptr, (const float*)nullptr, Vector2i::Zero(), Vector2i::Zero(),
		              (const float*)nullptr, Vector2i::Zero(), (float*)nullptr, (float*)nullptr, mean_density.data(), ds.exposure.data(), (Array3f*)nullptr,
		              0.0f, 0.0f, variance, training_step, (const network_precision_t*)d_rotation, (const network_precision_t*)d_transition,
		              Vector3f(first_frame_offset[0], first_frame_offset[1], first_frame_offset[2]), mask_loss_weight, ek_loss_weight, cos_anneal_ratio);
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
	});
}

/* update_density_grid_nerf, first half: the positions at which the SDF is evaluated (src/testbed_nerf.cu:3327-3353).
 * d_positions [n_uniform + n_nonuniform][3], d_indices [same].  The two generators advance by their default stride. */
int ref_density_grid_samples(uint32_t n_uniform, uint32_t n_nonuniform, uint64_t rng_state, uint64_t rng_inc, uint32_t ema_step, uint32_t n_cascades,
                             const float* d_density_grid, float* d_positions, uint32_t* d_indices, uint64_t* rng_state_out, uint64_t* rng_inc_out) {
	return guarded([&] {
		default_rng_t rng;
		rng.state = rng_state;
		rng.inc = rng_inc;
		cudaStream_t stream = nullptr;
		const BoundingBox aabb{Vector3f::Zero(), Vector3f::Ones()};
		linear_kernel(generate_grid_samples_nerf_nonuniform, 0, stream, n_uniform, rng, ema_step, aabb, d_density_grid, (NerfPosition*)d_positions, d_indices,
		              n_cascades, -0.01f);
		rng.advance();
		linear_kernel(generate_grid_samples_nerf_nonuniform, 0, stream, n_nonuniform, rng, ema_step, aabb, d_density_grid,
		              (NerfPosition*)d_positions + n_uniform, d_indices + n_uniform, n_cascades, NERF_MIN_OPTICAL_THICKNESS());
		rng.advance();
		*rng_state_out = rng.state;
		*rng_inc_out = rng.inc;
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
	});
}

/* Second half (:3355-3391): SDF -> density (NerfNetwork::density, nerf_network.h:711-726), splat, EMA, mean and bitfield with its
 * mip levels.  d_sdf [n] fp16 is overwritten with the densities; d_variance: the 4 fp16 variance parameters.
 * d_density_grid float[128^3 n_cascades] in/out, d_grid_tmp same size, d_bitfield uint8[128^3 / 8 per level], d_mean float[>= 32]. */
int ref_density_grid_update(uint32_t n_samples, const uint32_t* d_indices, uint16_t* d_sdf, const uint16_t* d_variance, float decay, uint32_t ema_step,
                            uint32_t n_cascades, float* d_density_grid, float* d_grid_tmp, uint8_t* d_bitfield, float* d_mean) {
	return guarded([&] {
		cudaStream_t stream = nullptr;
		const uint32_t cells = NERF_GRIDSIZE() * NERF_GRIDSIZE() * NERF_GRIDSIZE();
		const uint32_t n_elements = cells * n_cascades;
		GPUMatrix<network_precision_t, RM> density_matrix((network_precision_t*)d_sdf, 1, n_samples);
		linear_kernel(sdf_to_density_variance_buffer<network_precision_t>, 0, stream, n_samples, (const network_precision_t*)d_variance, density_matrix.view());
		CUDA_CHECK_THROW(cudaMemsetAsync(d_grid_tmp, 0, sizeof(float) * n_elements, stream));
		linear_kernel(splat_grid_samples_nerf_max_nearest_neighbor, 0, stream, n_samples, d_indices, (const network_precision_t*)d_sdf, d_grid_tmp,
		              ENerfActivation::Logistic, ENerfActivation::Exponential);
		linear_kernel(ema_grid_samples_nerf, 0, stream, n_elements, decay, ema_step, d_density_grid, d_grid_tmp);
		/* update_density_grid_mean_and_bitfield (:3370-3391) */
		CUDA_CHECK_THROW(cudaMemsetAsync(d_mean, 0, sizeof(float), stream));
		reduce_sum(d_density_grid, [cells] __device__(float val) { return fmaxf(val, 0.f) / (cells); }, d_mean, cells, stream);
		linear_kernel(grid_to_bitfield, 0, stream, cells / 8 * NERF_CASCADES(), cells / 8 * n_cascades, d_density_grid, d_bitfield, d_mean);
		for (uint32_t level = 1; level < NERF_CASCADES(); ++level)
			linear_kernel(bitfield_max_pool, 0, stream, cells / 64, d_bitfield + (size_t)grid_mip_offset(level - 1) / 8, d_bitfield + (size_t)grid_mip_offset(level) / 8);
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
	});
}

/* One frame through the reference's inference path: NerfTracer::init_rays_from_camera, NerfTracer::trace (rounds of marching,
 * network queries and compositing with compaction of the live rays) and shade_kernel_nerf, Shade mode, pinhole camera.
 * d_params: the fp16 parameter block [SDF MLP | colour MLP | grid | variance]; grid geometry as in the arguments.
 * Outputs: d_frame [h][w][4], d_depth [h][w]. */
int ref_render_frame(uint32_t n_levels, uint32_t log2_hashmap_size, uint32_t base_resolution, float per_level_scale, float sdf_bias, uint16_t* d_params,
                     uint32_t width, uint32_t height, const float* focal_length, const float* camera, const float* screen_center, uint32_t spp,
                     int snap_to_pixel_centers, uint8_t* d_bitfield, float min_transmittance, float cone_angle_constant, float* d_frame, float* d_depth,
                     uint32_t* n_hit_out) {
	return guarded([&] {
		const json pos_encoding = {{"otype", "HashGrid"},          {"n_levels", n_levels},
		                           {"n_features_per_level", 2},   {"log2_hashmap_size", log2_hashmap_size},
		                           {"base_resolution", base_resolution}, {"per_level_scale", per_level_scale}};
		const json dir_encoding = {{"otype", "Composite"},
		                           {"nested", {{{"n_dims_to_encode", 3}, {"otype", "SphericalHarmonics"}, {"degree", 4}}, {{"otype", "Identity"}, {"n_bins", 4}, {"degree", 4}}}}};
		const json density_network = {{"otype", "FullyFusedMLP"}, {"activation", "ReLU"}, {"output_activation", "None"}, {"n_neurons", 64}, {"n_hidden_layers", 1},
		                              {"sdf_bias", sdf_bias}};
		const json rgb_network = {{"otype", "FullyFusedMLP"}, {"activation", "ReLU"}, {"output_activation", "None"}, {"n_neurons", 64}, {"n_hidden_layers", 2}};
		NerfNetwork<network_precision_t> network(3u, 3u, 0u, 4u, pos_encoding, dir_encoding, density_network, rgb_network);
		GPUMemory<network_precision_t> gradients(network.n_params());
		network.set_params((network_precision_t*)d_params, (network_precision_t*)d_params, (network_precision_t*)d_params, gradients.data());
		network.m_training_step = 0;
		network.set_anneal_end(0);  // as the testbed does after it has built the network (src/testbed.cu:2220); the member has no initialiser
		network.m_use_delta = false;
		network.m_train_delta = false;
		cudaStream_t stream;
		CUDA_CHECK_THROW(cudaStreamCreate(&stream));
		{
			Testbed::NerfTracer tracer;
			const BoundingBox aabb{Vector3f::Zero(), Vector3f::Ones()};
			Matrix<float, 3, 4> cam;
			std::memcpy(cam.data(), camera, 12 * sizeof(float));
			const Vector2i resolution((int)width, (int)height);
			const Vector2f focal(focal_length[0], focal_length[1]);
			CUDA_CHECK_THROW(cudaMemsetAsync(d_frame, 0, (size_t)width * height * 4 * sizeof(float), stream));
			tracer.init_rays_from_camera(spp, network.padded_output_width(), network.n_extra_dims(), resolution, focal, cam, cam, Vector4f::Zero(),
			                             Vector2f(screen_center[0], screen_center[1]), Vector3f(0.f, 0.f, 1.f), snap_to_pixel_centers != 0, aabb, 1.0f, 0.0f,
			                             CameraDistortion{}, nullptr, Vector2i::Zero(), nullptr, Vector2i::Zero(), (Array4f*)d_frame, d_depth, d_bitfield, -1,
			                             cone_angle_constant, ERenderMode::Shade, stream, nullptr, nullptr, Vector3f::Zero());
			const uint32_t n_hit = tracer.trace(network, aabb, aabb, 0, nullptr, focal, cone_angle_constant, d_bitfield, ERenderMode::Shade, cam, 1.0f, 0, -1,
			                                    ENerfActivation::Logistic, ENerfActivation::Exponential, -1, min_transmittance, 0.0f, 0, nullptr, stream);
			RaysNerfSoa& rays_hit = tracer.rays_hit();
			linear_kernel(shade_kernel_nerf, 0, stream, n_hit, rays_hit.rgba, rays_hit.depth, rays_hit.payload, ERenderMode::Shade, false, (Array4f*)d_frame, d_depth);
			CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
			if (n_hit_out) *n_hit_out = n_hit;
		}
		CUDA_CHECK_THROW(cudaStreamDestroy(stream));
	});
}

}  // extern "C"
