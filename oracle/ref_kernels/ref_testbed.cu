/* TEST AND MEASUREMENT INFRASTRUCTURE, not product code: the reference's own headless training loop and host code, made callable.
 *
 * oracle/build_ref_kernels.py compiles the reference's sources on the NeuS path where they lie in a reference checkout
 * (src/testbed.cu, testbed_nerf.cu, marching_cubes.cu, nerf_loader.cu, common_device.cu, camera_path.cu, triangle_bvh.cu,
 * thread_pool.cpp, tinyobj_loader_wrapper.cpp; nothing is copied) against include/tiny-cuda-nn of this repository, which
 * stands in for the un-vendored tiny-cuda-nn fork, and links them with this file into oracle/_ref/libref_testbed.so.
 * The parts of the reference that are not compiled (GUI, render buffer, the SDF / image / volume primitives, EXR) are left
 * as stubs that abort: the headless NeRF training path does not reach them.
 *
 * ref_testbed_train does what scripts/run.py does without a window: Testbed(Nerf), load_training_data, network from a
 * json document, then frame() per training step -- the reference's host loop with its stream synchronisations, its own ray
 * marching / loss / occupancy kernels, its NerfNetwork, Trainer and optimizer objects; underneath those objects run this
 * repository's layered kernels.  It is the reference's code path on a B200, not the reference's tiny-cuda-nn kernels.
 *
 * The other entry points hand single pieces of the same library to the tests: ref_load_dataset (ngp::load_nerf),
 * ref_marching_cubes (marching_cubes_gpu), ref_mesh_postprocess (compute_mesh_1ring, save_mesh), ref_testbed_sdf_grid
 * (Testbed::get_density_on_grid) and ref_testbed_snapshot (save_snapshot / load_snapshot / compute_and_save_marching_cubes_mesh). */
#include <neural-graphics-primitives/nerf_loader.h>
#include <neural-graphics-primitives/testbed.h>
#include <tiny-cuda-nn/trainer.h>
#include <neural-graphics-primitives/marching_cubes.h>

#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <vector>

using namespace ngp;

extern "C" {

/* workdir: directory to run in; must hold utils/mlp_weights.txt (the SDF network's initial weights, which
 * NerfNetwork::initialize_params reads relative to the working directory, nerf_network.h:773-803).
 * h_params (optional, n_params floats): full-precision parameters that replace the drawn ones before the first step
 * (Trainer::set_params_full_precision), so that a run can start from the same weights as another implementation's.
 * losses[n_warmup + n_steps]: Testbed::m_loss_scalar.val() after every step (the reference reads the loss back every 16th
 * step).  step_stats (optional) [n_warmup + n_steps][3]: rays_per_batch, measured_batch_size,
 * measured_batch_size_before_compaction after every step.  h_density_grid (optional, n_density_grid floats): the occupancy
 * grid's running densities (Testbed::m_nerf.density_grid) as they stand after grid_after_steps steps; h_bitfield (optional,
 * n_bitfield bytes): the occupancy bits of all cascades (density_grid_bitfield) at the same moment.  step_frames (optional)
 * [n_warmup + n_steps][2]: the frame of a dynamic sequence and the frame's training step after every call of frame() (the data
 * path may be a directory of per-frame transforms files; frame() moves on by itself, src/testbed.cu:1739-1746).  h_motion
 * (optional, 28 fp16 values): the accumulated rotation (12 slots) and transition (4), and the current frame's own 6-D rotation
 * (8) and transition (4), at the end.  wall_ms: host time of the n_steps timed steps (synchronised before
 * and after).  stats[4]: rays_per_batch, measured_batch_size, measured_batch_size_before_compaction, training step at the end. */
int ref_testbed_train(const char* workdir, const char* transforms_json, const char* network_config_json, uint32_t batch_size, uint32_t n_warmup,
                      uint32_t n_steps, const float* h_params, uint64_t n_params, float* losses, uint32_t* step_stats, float* wall_ms, uint32_t* stats,
                      uint32_t grid_after_steps, float* h_density_grid, uint64_t n_density_grid, uint8_t* h_bitfield, uint64_t n_bitfield,
                      uint32_t* step_frames, uint16_t* h_motion) {
	try {
		if (chdir(workdir) != 0) return -3;
		Testbed testbed{ETestbedMode::Nerf};
		testbed.load_training_data(transforms_json);
		testbed.reload_network_from_json(nlohmann::json::parse(network_config_json, nullptr, true, true), "");
		if (h_params) {
			if (n_params != testbed.m_trainer->n_params()) return -4;
			testbed.m_trainer->set_params_full_precision(h_params, n_params);
		}
		testbed.m_train = true;
		testbed.m_training_batch_size = batch_size;
		const auto& c = testbed.m_nerf.training.counters_rgb;
		auto record = [&](uint32_t i) {
			if (h_density_grid && i + 1 == grid_after_steps)
				CUDA_CHECK_THROW(cudaMemcpy(h_density_grid, testbed.m_nerf.density_grid.data(),
				                            sizeof(float) * std::min<uint64_t>(n_density_grid, testbed.m_nerf.density_grid.size()), cudaMemcpyDeviceToHost));
			if (h_bitfield && i + 1 == grid_after_steps)
				CUDA_CHECK_THROW(cudaMemcpy(h_bitfield, testbed.m_nerf.density_grid_bitfield.data(),
				                            std::min<uint64_t>(n_bitfield, testbed.m_nerf.density_grid_bitfield.size()), cudaMemcpyDeviceToHost));
			if (losses) losses[i] = testbed.m_loss_scalar.val();
			if (step_frames) {
				step_frames[2 * i + 0] = (uint32_t)testbed.current_training_time_frame;
				step_frames[2 * i + 1] = testbed.m_training_step;
			}
			if (step_stats) {
				step_stats[3 * i + 0] = c.rays_per_batch;
				step_stats[3 * i + 1] = c.measured_batch_size;
				step_stats[3 * i + 2] = c.measured_batch_size_before_compaction;
			}
		};
		for (uint32_t i = 0; i < n_warmup; ++i) {
			testbed.frame();
			record(i);
		}
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		const auto t0 = std::chrono::steady_clock::now();
		for (uint32_t i = 0; i < n_steps; ++i) {
			testbed.frame();
			record(n_warmup + i);
		}
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		if (wall_ms) *wall_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
		if (h_motion) {  // fp16 bits: accumulated rotation [12 slots], accumulated transition [4], the frame's own rotation [8] and transition [4]
			const auto& net = testbed.m_nerf_network;
			CUDA_CHECK_THROW(cudaMemcpy(h_motion, net->rotation()->params(), sizeof(uint16_t) * std::min<size_t>(12, net->rotation()->n_params()), cudaMemcpyDeviceToHost));
			CUDA_CHECK_THROW(cudaMemcpy(h_motion + 12, net->transition()->params(), sizeof(uint16_t) * std::min<size_t>(4, net->transition()->n_params()), cudaMemcpyDeviceToHost));
			const auto& dn = net->delta_network();
			CUDA_CHECK_THROW(cudaMemcpy(h_motion + 16, dn->rotation()->params(), sizeof(uint16_t) * std::min<size_t>(8, dn->rotation()->n_params()), cudaMemcpyDeviceToHost));
			CUDA_CHECK_THROW(cudaMemcpy(h_motion + 24, dn->transition()->params(), sizeof(uint16_t) * std::min<size_t>(4, dn->transition()->n_params()), cudaMemcpyDeviceToHost));
		}
		if (stats) {
			stats[0] = c.rays_per_batch;
			stats[1] = c.measured_batch_size;
			stats[2] = c.measured_batch_size_before_compaction;
			stats[3] = testbed.m_training_step;
		}
		return 0;
	} catch (const std::exception& e) {
		std::fprintf(stderr, "ref_testbed_train: %s\n", e.what());
		return -1;
	}
}

/* The reference's dataset loader (ngp::load_nerf, src/nerf_loader.cu:197) on one transforms file: what it hands to training.
 * header[8]: n_images, width and height of image 0, bytes per pixel channel (EImageDataType as image_type_size), aabb_scale,
 * is_hdr, from_na, from_mitsuba.  floats[8]: scale, offset xyz, up xyz, 0.  Per image (at most max_images): xforms [12] (the 3x4
 * start matrix, row-major), focal [2], principal [2], and the pixel bytes of image i at pixels + i * width * height * 4 *
 * bytes-per-channel (copied while they fit into pixel_capacity). */
int ref_load_dataset(const char* transforms_json, uint32_t max_images, uint32_t* header, float* floats, float* xforms, float* focal, float* principal,
                     uint8_t* pixels, uint64_t pixel_capacity) {
	try {
		NerfDataset ds = ngp::load_nerf({filesystem::path{transforms_json}}, 0.f);
		const auto& m0 = ds.metadata.at(0);
		header[0] = (uint32_t)ds.n_images;
		header[1] = (uint32_t)m0.resolution.x();
		header[2] = (uint32_t)m0.resolution.y();
		header[3] = (uint32_t)image_type_size(m0.image_data_type);
		header[4] = (uint32_t)ds.aabb_scale;
		header[5] = ds.is_hdr;
		header[6] = ds.from_na;
		header[7] = ds.from_mitsuba;
		floats[0] = ds.scale;
		for (int k = 0; k < 3; ++k) {
			floats[1 + k] = ds.offset[k];
			floats[4 + k] = ds.up[k];
		}
		floats[7] = 0.f;
		const uint64_t image_bytes = (uint64_t)header[1] * header[2] * 4 * header[3];
		for (uint32_t i = 0; i < ds.n_images && i < max_images; ++i) {
			for (int r = 0; r < 3; ++r)
				for (int c = 0; c < 4; ++c) xforms[i * 12 + r * 4 + c] = ds.xforms[i].start(r, c);
			focal[2 * i] = ds.metadata[i].focal_length.x();
			focal[2 * i + 1] = ds.metadata[i].focal_length.y();
			principal[2 * i] = ds.metadata[i].principal_point.x();
			principal[2 * i + 1] = ds.metadata[i].principal_point.y();
			if ((i + 1) * image_bytes <= pixel_capacity)
				CUDA_CHECK_THROW(cudaMemcpy(pixels + i * image_bytes, ds.pixelmemory[i].data(), image_bytes, cudaMemcpyDeviceToHost));
		}
		return 0;
	} catch (const std::exception& e) {
		std::fprintf(stderr, "ref_load_dataset: %s\n", e.what());
		return -1;
	}
}

/* The reference's marching cubes (marching_cubes_gpu, src/marching_cubes.cu:794-822) on a host lattice of rx * ry * rz values
 * (x fastest) in the unit cube.  counts[2]: vertex slots (the reference rounds the count up to 128) and indices; vertices and
 * indices are copied out while they fit.  Vertex numbering follows the arrival order of the reference's atomics. */
int ref_marching_cubes(uint32_t rx, uint32_t ry, uint32_t rz, float thresh, const float* h_density, uint32_t* counts, float* h_verts, uint64_t verts_capacity,
                       uint32_t* h_indices, uint64_t indices_capacity) {
	try {
		tcnn::GPUMemory<float> density;
		density.resize_and_copy_from_host(h_density, (size_t)rx * ry * rz);
		tcnn::GPUMemory<Eigen::Vector3f> verts;
		tcnn::GPUMemory<uint32_t> indices;
		marching_cubes_gpu(nullptr, BoundingBox{Eigen::Vector3f::Zero(), Eigen::Vector3f::Ones()}, Eigen::Vector3i((int)rx, (int)ry, (int)rz), thresh, density, verts,
		                   indices);
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		counts[0] = (uint32_t)verts.size();
		counts[1] = (uint32_t)indices.size();
		if (verts.size() && verts.size() <= verts_capacity) CUDA_CHECK_THROW(cudaMemcpy(h_verts, verts.data(), sizeof(float) * 3 * verts.size(), cudaMemcpyDeviceToHost));
		if (indices.size() && indices.size() <= indices_capacity)
			CUDA_CHECK_THROW(cudaMemcpy(h_indices, indices.data(), sizeof(uint32_t) * indices.size(), cudaMemcpyDeviceToHost));
		return 0;
	} catch (const std::exception& e) {
		std::fprintf(stderr, "ref_marching_cubes: %s\n", e.what());
		return -1;
	}
}

/* The reference's mesh post-processing on a given mesh: compute_mesh_1ring (src/marching_cubes.cu:720-738) -> h_ring [n][4],
 * h_normals [n][3]; then save_mesh (:824-976, no texture unwrap) with the given normals and colours to every file name that is
 * not NULL (the extension selects OBJ or PLY). */
int ref_mesh_postprocess(uint32_t n_verts, const float* h_verts, uint32_t n_indices, const uint32_t* h_indices, float* h_ring, float* h_normals,
                         const float* h_save_normals, const float* h_save_colors, const char* file_a, const char* file_b, float nerf_scale,
                         const float* nerf_offset, int invert_normals) {
	try {
		tcnn::GPUMemory<Eigen::Vector3f> verts(n_verts), normals, save_normals(n_verts), colors(n_verts);
		tcnn::GPUMemory<Eigen::Vector4f> ring;
		tcnn::GPUMemory<uint32_t> indices(n_indices);
		CUDA_CHECK_THROW(cudaMemcpy(verts.data(), h_verts, sizeof(float) * 3 * n_verts, cudaMemcpyHostToDevice));
		CUDA_CHECK_THROW(cudaMemcpy(indices.data(), h_indices, sizeof(uint32_t) * n_indices, cudaMemcpyHostToDevice));
		compute_mesh_1ring(verts, indices, ring, normals);
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		if (ring.size() < n_verts || normals.size() < n_verts) return -2;
		CUDA_CHECK_THROW(cudaMemcpy(h_ring, ring.data(), sizeof(float) * 4 * n_verts, cudaMemcpyDeviceToHost));
		CUDA_CHECK_THROW(cudaMemcpy(h_normals, normals.data(), sizeof(float) * 3 * n_verts, cudaMemcpyDeviceToHost));
		CUDA_CHECK_THROW(cudaMemcpy(save_normals.data(), h_save_normals, sizeof(float) * 3 * n_verts, cudaMemcpyHostToDevice));
		CUDA_CHECK_THROW(cudaMemcpy(colors.data(), h_save_colors, sizeof(float) * 3 * n_verts, cudaMemcpyHostToDevice));
		const Eigen::Vector3f offset(nerf_offset[0], nerf_offset[1], nerf_offset[2]);
		if (file_a) save_mesh(verts, save_normals, colors, indices, file_a, false, nerf_scale, offset, invert_normals != 0);
		if (file_b) save_mesh(verts, save_normals, colors, indices, file_b, false, nerf_scale, offset, invert_normals != 0);
		return 0;
	} catch (const std::exception& e) {
		std::fprintf(stderr, "ref_mesh_postprocess: %s\n", e.what());
		return -1;
	}
}

/* Testbed::get_density_on_grid (src/testbed_nerf.cu:4082-4135; the lattice marching cubes runs on) of a testbed built like in
 * ref_testbed_train, with the given parameters and no training step: h_out [rz][ry][rx] floats over the unit cube. */
int ref_testbed_sdf_grid(const char* workdir, const char* transforms_json, const char* network_config_json, const float* h_params, uint64_t n_params,
                         uint32_t rx, uint32_t ry, uint32_t rz, float* h_out) {
	try {
		if (chdir(workdir) != 0) return -3;
		Testbed testbed{ETestbedMode::Nerf};
		testbed.load_training_data(transforms_json);
		testbed.reload_network_from_json(nlohmann::json::parse(network_config_json, nullptr, true, true), "");
		if (n_params != testbed.m_trainer->n_params()) return -4;
		testbed.m_trainer->set_params_full_precision(h_params, n_params);
		tcnn::GPUMemory<float> grid = testbed.get_density_on_grid(Eigen::Vector3i((int)rx, (int)ry, (int)rz), BoundingBox{Eigen::Vector3f::Zero(), Eigen::Vector3f::Ones()});
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		CUDA_CHECK_THROW(cudaMemcpy(h_out, grid.data(), sizeof(float) * (size_t)rx * ry * rz, cudaMemcpyDeviceToHost));
		return 0;
	} catch (const std::exception& e) {
		std::fprintf(stderr, "ref_testbed_sdf_grid: %s\n", e.what());
		return -1;
	}
}

/* Testbed::save_snapshot / load_snapshot (src/testbed.cu:3134-3244).  With load_path the testbed takes network, parameters,
 * occupancy grid and counters from that file (network_config_json and h_params are not used); otherwise it is built from the
 * configuration and h_params and trained for n_steps.  With save_path the state is then written there (no optimizer state).
 * h_sdf [res]^3: get_density_on_grid afterwards; info[4]: training step, rays per batch, measured batch size, occupied cells of the
 * finest level.  mesh_path (optional): the reference's mesh export of that state (OBJ or PLY by extension). */
int ref_testbed_snapshot(const char* workdir, const char* transforms_json, const char* network_config_json, const float* h_params, uint64_t n_params,
                         uint32_t n_steps, const char* load_path, const char* save_path, uint32_t res, float* h_sdf, uint32_t* info, const char* mesh_path) {
	try {
		if (chdir(workdir) != 0) return -3;
		Testbed testbed{ETestbedMode::Nerf};
		testbed.load_training_data(transforms_json);
		if (load_path) {
			testbed.load_snapshot(load_path);
		} else {
			testbed.reload_network_from_json(nlohmann::json::parse(network_config_json, nullptr, true, true), "");
			if (n_params != testbed.m_trainer->n_params()) return -4;
			testbed.m_trainer->set_params_full_precision(h_params, n_params);
			testbed.m_train = true;
			for (uint32_t i = 0; i < n_steps; ++i) testbed.frame();
			testbed.m_train = false;
		}
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		if (save_path) testbed.save_snapshot(save_path, false);
		tcnn::GPUMemory<float> grid = testbed.get_density_on_grid(Eigen::Vector3i::Constant((int)res), BoundingBox{Eigen::Vector3f::Zero(), Eigen::Vector3f::Ones()});
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		CUDA_CHECK_THROW(cudaMemcpy(h_sdf, grid.data(), sizeof(float) * (size_t)res * res * res, cudaMemcpyDeviceToHost));
		// Testbed::compute_and_save_marching_cubes_mesh (src/testbed.cu:298-306) at the same resolution, threshold 0
		if (mesh_path) testbed.compute_and_save_marching_cubes_mesh(mesh_path, Eigen::Vector3i::Constant((int)res), BoundingBox{}, 0.0f, false);
		info[0] = testbed.m_training_step;
		info[1] = testbed.m_nerf.training.counters_rgb.rays_per_batch;
		info[2] = testbed.m_nerf.training.counters_rgb.measured_batch_size;
		std::vector<uint8_t> bits(NERF_GRIDSIZE() * NERF_GRIDSIZE() * NERF_GRIDSIZE() / 8);
		info[3] = 0;
		if (testbed.m_nerf.density_grid_bitfield.size() >= bits.size()) {
			CUDA_CHECK_THROW(cudaMemcpy(bits.data(), testbed.m_nerf.density_grid_bitfield.data(), bits.size(), cudaMemcpyDeviceToHost));
			for (uint8_t b : bits) info[3] += (uint32_t)__builtin_popcount(b);
		}
		return 0;
	} catch (const std::exception& e) {
		std::fprintf(stderr, "ref_testbed_snapshot: %s\n", e.what());
		return -1;
	}
}

}  // extern "C"
