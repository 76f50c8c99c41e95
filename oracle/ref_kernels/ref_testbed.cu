/* TEST AND MEASUREMENT INFRASTRUCTURE, not product code: the reference's own headless training loop, made callable.
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
 * repository's layered kernels.  It is the reference's code path on a B200, not the reference's tiny-cuda-nn kernels. */
#include <neural-graphics-primitives/testbed.h>

#include <unistd.h>

#include <chrono>
#include <cstdio>

using namespace ngp;

extern "C" {

/* workdir: directory to run in; must hold utils/mlp_weights.txt (the SDF network's initial weights, which
 * NerfNetwork::initialize_params reads relative to the working directory, nerf_network.h:773-803).
 * losses[n_warmup + n_steps]: Testbed::m_loss_scalar after every step.  wall_ms: host time of the n_steps timed steps
 * (synchronised before and after).  stats[4]: rays_per_batch, measured_batch_size, measured_batch_size_before_compaction,
 * training step, after the last step. */
int ref_testbed_train(const char* workdir, const char* transforms_json, const char* network_config_json, uint32_t batch_size, uint32_t n_warmup,
                      uint32_t n_steps, float* losses, float* wall_ms, uint32_t* stats) {
	try {
		if (chdir(workdir) != 0) return -3;
		Testbed testbed{ETestbedMode::Nerf};
		testbed.load_training_data(transforms_json);
		testbed.reload_network_from_json(nlohmann::json::parse(network_config_json, nullptr, true, true), "");
		testbed.m_train = true;
		testbed.m_training_batch_size = batch_size;
		for (uint32_t i = 0; i < n_warmup; ++i) {
			testbed.frame();
			if (losses) losses[i] = testbed.m_loss_scalar.val();
		}
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		const auto t0 = std::chrono::steady_clock::now();
		for (uint32_t i = 0; i < n_steps; ++i) {
			testbed.frame();
			if (losses) losses[n_warmup + i] = testbed.m_loss_scalar.val();
		}
		CUDA_CHECK_THROW(cudaDeviceSynchronize());
		if (wall_ms) *wall_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
		if (stats) {
			const auto& c = testbed.m_nerf.training.counters_rgb;
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

}  // extern "C"
