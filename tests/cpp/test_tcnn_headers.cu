// Drives the tiny-cuda-nn-shaped headers (include/tiny-cuda-nn/*.h) the way the reference's NerfNetwork and Testbed drive
// tiny-cuda-nn -- objects from json, strided slices of wider matrices as operands, a Trainer that owns the parameter
// block -- and checks every result against the same C-ABI entry point called directly (bit for bit where the kernel's
// summation order is fixed), plus the error convention.  Exit code 0 = pass.  With --check-only nothing touches a GPU.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include <tiny-cuda-nn/common.h>
#include <tiny-cuda-nn/common_device.h>
#include <tiny-cuda-nn/cuda_graph.h>
#include <tiny-cuda-nn/encoding.h>
#include <tiny-cuda-nn/encodings/grid.h>
#include <tiny-cuda-nn/gpu_matrix.h>
#include <tiny-cuda-nn/gpu_memory.h>
#include <tiny-cuda-nn/gpu_memory_json.h>
#include <tiny-cuda-nn/loss.h>
#include <tiny-cuda-nn/multi_stream.h>
#include <tiny-cuda-nn/network.h>
#include <tiny-cuda-nn/network_with_input_encoding.h>
#include <tiny-cuda-nn/optimizer.h>
#include <tiny-cuda-nn/random.h>
#include <tiny-cuda-nn/reduce_sum.h>
#include <tiny-cuda-nn/trainer.h>

using namespace tcnn;
using T = network_precision_t;

static int g_failed = 0;
#define EXPECT(cond)                                                      \
	do {                                                                  \
		if (!(cond)) {                                                    \
			std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
			++g_failed;                                                   \
		}                                                                 \
	} while (0)

template <typename F>
static bool throws(F&& f) {
	try {
		f();
	} catch (const std::runtime_error&) {
		return true;
	}
	return false;
}

template <typename U>
static std::vector<U> to_host(const U* dev, size_t n) {
	std::vector<U> v(n);
	CUDA_CHECK_THROW(cudaMemcpy(v.data(), dev, n * sizeof(U), cudaMemcpyDeviceToHost));
	return v;
}
template <typename U>
static bool same(const U* a_dev, const U* b_dev, size_t n) {
	auto a = to_host(a_dev, n), b = to_host(b_dev, n);
	return std::memcmp(a.data(), b.data(), n * sizeof(U)) == 0;
}
static double cosine_half(const T* a_dev, const T* b_dev, size_t n) {
	auto a = to_host(a_dev, n), b = to_host(b_dev, n);
	double ab = 0, aa = 0, bb = 0;
	for (size_t i = 0; i < n; ++i) {
		const double p = __half2float(a[i]), q = __half2float(b[i]);
		ab += p * q, aa += p * p, bb += q * q;
	}
	return aa > 0 && bb > 0 ? ab / std::sqrt(aa * bb) : 0.0;
}

static const json kGrid = {{"otype", "HashGrid"}, {"n_levels", 16},          {"n_features_per_level", 2},
                           {"log2_hashmap_size", 19}, {"base_resolution", 16}, {"per_level_scale", 1.447f}};
static const json kDir = {{"otype", "Composite"},
                          {"nested", {{{"n_dims_to_encode", 3}, {"otype", "SphericalHarmonics"}, {"degree", 4}}, {{"otype", "Identity"}, {"n_bins", 4}, {"degree", 4}}}}};
static const json kSdfNet = {{"otype", "FullyFusedMLP"}, {"activation", "ReLU"}, {"output_activation", "None"}, {"n_neurons", 64},
                             {"n_hidden_layers", 1},     {"n_input_dims", 48},   {"n_output_dims", 16}};
static const json kAdam = {{"otype", "Ema"},
                           {"decay", 0.95f},
                           {"nested",
                            {{"otype", "ExponentialDecay"},
                             {"decay_start", 2},
                             {"decay_interval", 1},
                             {"decay_base", 0.5f},
                             {"nested", {{"otype", "Adam"}, {"learning_rate", 1e-2f}, {"beta1", 0.9f}, {"beta2", 0.99f}, {"epsilon", 1e-15f}, {"l2_reg", 1e-6f}}}}}};

int main(int argc, char** argv) {
	// ---- host-only part: factories, shapes, parameter counts, level tables, error convention
	std::shared_ptr<Encoding<T>> enc{create_encoding<T>(3, kGrid, 16)};
	auto* grid = dynamic_cast<GridEncoding<T>*>(enc.get());
	EXPECT(grid != nullptr);
	EXPECT(enc->n_params() == 12599920u);
	EXPECT(enc->padded_output_width() == 32 && enc->output_width() == 32 && enc->input_width() == 3);
	EXPECT(grid && grid->level_params_offset(0) == 0 && grid->level_n_params(0) == 2u * 4096u);  // the coarsest level is a dense 16^3 lattice
	{
		size_t total = 0;
		for (uint32_t l = 0; l < 16; ++l) total += grid->level_n_params(l);
		EXPECT(total == enc->n_params());
	}
	std::shared_ptr<Encoding<T>> dir{create_encoding<T>(3, kDir, 16)};
	EXPECT(dir->padded_output_width() == 16 && dir->n_params() == 0);
	std::unique_ptr<Network<T>> sdf_net{create_network<T>(kSdfNet)};
	EXPECT(sdf_net->n_params() == 4096 && sdf_net->padded_output_width() == 16 && sdf_net->num_forward_activations() == 1);
	EXPECT(sdf_net->layer_sizes().size() == 2 && sdf_net->layer_sizes()[0] == std::make_pair(64u, 48u));
	EXPECT(minimum_alignment(kSdfNet) == 16);
	EXPECT(throws([] { json j = kSdfNet; j["n_neurons"] = 128; delete create_network<T>(j); }));
	EXPECT(throws([] { delete create_network<T>({{"otype", "CutlassMLP"}, {"n_input_dims", 48}, {"n_output_dims", 16}}); }));
	EXPECT(throws([] { delete create_encoding<T>(3, {{"otype", "Frequency"}}); }));
	EXPECT(throws([] { delete create_encoding<T>(2, kGrid); }));
	EXPECT(throws([] { delete create_optimizer<T>({{"otype", "Shampoo"}}); }));
	EXPECT(throws([] { delete create_loss<T>({{"otype", "Variance"}}); }));
	EXPECT(throws([] { neus2b_check(NEUS2B_E_INVALID, "probe"); }));
	{  // progressive levels under the reference's keys (configs/nerf/base.json:36-38 with 14 levels: 3 levels at step 0)
		json g = kGrid;
		g["n_levels"] = 14, g["base_training_step"] = 100, g["valid_level_scale"] = 0.02f, g["base_valid_level_scale"] = 0.2f;
		std::unique_ptr<Encoding<T>> e{create_encoding<T>(3, g, 2)};
		auto* ge = dynamic_cast<GridEncodingNeus2b<T>*>(e.get());
		EXPECT(ge && ge->n_active_levels() == 3);
		e->set_training_step(2000);
		EXPECT(ge && ge->n_active_levels() == 8);  // 14 * (0.2 + 0.02 * 20) = 8.4
		e->set_training_step(100000);
		EXPECT(ge && ge->n_active_levels() == 14);
	}
	{  // pcg32: skipping ahead equals drawing
		pcg32 a{1337}, b{1337};
		for (int i = 0; i < 1000; ++i) a.next_uint();
		b.advance(1000);
		EXPECT(a == b && a.next_uint() == b.next_uint());
		pcg32 c{1337};
		const float f = c.next_float();
		EXPECT(f >= 0.f && f < 1.f);
	}
	EXPECT(next_multiple(35u, 16u) == 48u && div_round_up(7u, 4u) == 2u && equals_case_insensitive("fullyFUSEDmlp", "FullyFusedMLP"));
	EXPECT(morton3D_invert(morton3D(5, 0, 0)) == 5 && morton3D_invert(morton3D(0, 77, 0) >> 1) == 77 && morton3D_invert(morton3D(0, 0, 127) >> 2) == 127);
	EXPECT(sizeof(vector_t<T, 16>) == 32 && alignof(vector_t<T, 16>) == 16 && alignof(vector_t<T, 4>) == 8);
	if (argc > 1 && std::strcmp(argv[1], "--check-only") == 0) {
		std::printf(g_failed ? "host checks FAILED\n" : "host checks ok\n");
		return g_failed ? 1 : 0;
	}

	// ---- device part
	const uint32_t n = 4096 + 37;
	std::mt19937 rng(7);
	std::uniform_real_distribution<float> u01(0.f, 1.f), small(-1e-2f, 1e-2f), wdist(-0.2f, 0.2f);
	cudaStream_t stream;
	CUDA_CHECK_THROW(cudaStreamCreate(&stream));
	{  // everything allocated in stream order dies before the stream does

	// the input as the training loop holds it: records of 7 floats (position, dt, direction), one per batch element
	std::vector<float> h_coords((size_t)n * 7);
	for (auto& v : h_coords) v = u01(rng);
	GPUMemory<float> coords;
	coords.resize_and_copy_from_host(h_coords);
	GPUMatrix<float> coords_matrix(coords.data(), 7, n);

	std::vector<T> h_grid(enc->n_params()), h_w(sdf_net->n_params()), h_dy((size_t)n * 16);
	for (auto& v : h_grid) v = __float2half(small(rng));
	for (auto& v : h_w) v = __float2half(wdist(rng));
	for (auto& v : h_dy) v = __float2half(small(rng));
	GPUMemory<T> grid_params, grid_grads(enc->n_params()), w, w_grads(sdf_net->n_params()), dy;
	grid_params.resize_and_copy_from_host(h_grid);
	w.resize_and_copy_from_host(h_w);
	dy.resize_and_copy_from_host(h_dy);
	grid_grads.memset(0);
	enc->set_params(grid_params.data(), grid_params.data(), nullptr, grid_grads.data());
	sdf_net->set_params(w.data(), w.data(), nullptr, w_grads.data());

	// forward as in nerf_network.h:137-212: the encoding writes rows [0, 32) of the 48-row network input, the network
	// writes rows [0, 16) of the 48-row input of the next network -- both operands are strided slices
	GPUMatrixDynamic<T> Z{48, n, stream}, next_input{48, n, stream};
	GPUMatrixDynamic<T> E = Z.slice_rows(0, 32), Y = next_input.slice_rows(0, 16);
	EXPECT(!E.is_contiguous() && E.stride() == 48);
	auto X = coords_matrix.slice_rows(0, 3);
	auto enc_ctx = enc->forward(stream, X, &E, false, true);
	auto net_ctx = sdf_net->forward(stream, Z, &Y, false, true);
	GPUMatrixDynamic<T> dY(dy.data(), 16, n), dZ{48, n, stream};
	sdf_net->backward(stream, *net_ctx, Z, Y, dY, &dZ, false, EGradientMode::Overwrite);
	GPUMatrixDynamic<T> dE = dZ.slice_rows(0, 32);
	GPUMatrixDynamic<float> dX{3, n, stream};
	enc->backward(stream, *enc_ctx, X, E, dE, &dX, false, EGradientMode::Overwrite);
	// the direction encoding into rows [16, 32) of the next input
	GPUMatrixDynamic<T> D = next_input.slice_rows(16, 16);
	dir->forward(stream, coords_matrix.slice_rows(4, 3), &D);
	CUDA_CHECK_THROW(cudaStreamSynchronize(stream));

	// the same through the C ABI on dense arrays
	{
		GPUMemory<T> enc2((size_t)n * 32), z2((size_t)n * 48), y2((size_t)n * 16), hid2((size_t)n * 64), dz2((size_t)n * 48), denc2((size_t)n * 32), gg2(enc->n_params()), sh2((size_t)n * 16);
		GPUMemory<float> wg2(sdf_net->n_params()), dx2((size_t)n * 3);
		z2.memset(0), gg2.memset(0);
		neus2b_grid_desc d{16, 19, 16, 1.447f, 16};
		EXPECT(neus2b_grid_forward(&d, n, coords.data(), 7, (const uint16_t*)grid_params.data(), (uint16_t*)enc2.data(), nullptr, stream) == 0);
		CUDA_CHECK_THROW(cudaMemcpy2DAsync(z2.data(), 48 * sizeof(T), enc2.data(), 32 * sizeof(T), 32 * sizeof(T), n, cudaMemcpyDeviceToDevice, stream));
		EXPECT(neus2b_mlp_forward(n, 48, 1, (const uint16_t*)w.data(), (const uint16_t*)z2.data(), (uint16_t*)y2.data(), (uint16_t*)hid2.data(), stream) == 0);
		EXPECT(neus2b_mlp_backward(n, 48, 1, (const uint16_t*)w.data(), (const uint16_t*)z2.data(), (const uint16_t*)hid2.data(), (const uint16_t*)dy.data(),
		                           (uint16_t*)dz2.data(), wg2.data(), NEUS2B_GRAD_OVERWRITE, stream) == 0);
		CUDA_CHECK_THROW(cudaMemcpy2DAsync(denc2.data(), 32 * sizeof(T), dz2.data(), 48 * sizeof(T), 32 * sizeof(T), n, cudaMemcpyDeviceToDevice, stream));
		EXPECT(neus2b_grid_backward_input(&d, n, coords.data(), 7, (const uint16_t*)grid_params.data(), (const uint16_t*)denc2.data(), dx2.data(), stream) == 0);
		EXPECT(neus2b_grid_backward_params(&d, n, coords.data(), 7, (const uint16_t*)denc2.data(), (uint16_t*)gg2.data(), NEUS2B_GRAD_OVERWRITE, stream) == 0);
		EXPECT(neus2b_sh4_forward(n, coords.data() + 4, 7, (uint16_t*)sh2.data(), stream) == 0);
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		EXPECT(same(z2.data(), Z.data(), (size_t)n * 48));    // encoding in rows 0..31, zero padding behind
		EXPECT(same(dz2.data(), dZ.data(), (size_t)n * 48));
		EXPECT(same(dx2.data(), dX.data(), (size_t)n * 3));
		{  // next_input = [network output (16) | direction encoding (16) | zeros (16)] per element
			auto got = to_host(next_input.data(), (size_t)n * 48);
			auto y = to_host(y2.data(), (size_t)n * 16), sh = to_host(sh2.data(), (size_t)n * 16);
			bool ok = true;
			for (uint32_t i = 0; i < n && ok; ++i)
				ok = !std::memcmp(&got[(size_t)i * 48], &y[(size_t)i * 16], 32) && !std::memcmp(&got[(size_t)i * 48 + 16], &sh[(size_t)i * 16], 32) &&
				     __half2float(got[(size_t)i * 48 + 40]) == 0.0f;
			EXPECT(ok);
		}
		{  // the weight gradient is an fp32 sum in arrival order, published as fp16
			auto a = to_host(wg2.data(), wg2.size());
			auto b = to_host(w_grads.data(), w_grads.size());
			double err = 0, ref = 0;
			for (size_t i = 0; i < a.size(); ++i) err = std::fmax(err, std::fabs((double)a[i] - __half2float(b[i]))), ref = std::fmax(ref, std::fabs((double)a[i]));
			EXPECT(ref > 0 && err <= 2e-3 * ref);
		}
		EXPECT(cosine_half(gg2.data(), grid_grads.data(), enc->n_params()) > 0.9999);  // scattered fp16 additions commute only up to rounding
	}
	{  // a row-major operand is accepted too (the occupancy update asks for the SDF as one row, src/testbed_nerf.cu:3274)
		GPUMatrix<T, RM> out_rm{16, n, stream};
		sdf_net->inference_mixed_precision(stream, Z, out_rm, false);
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		auto rm = to_host(out_rm.data(), (size_t)n * 16);
		auto cm = to_host(next_input.data(), (size_t)n * 48);
		bool ok = true;
		for (uint32_t i = 0; i < n && ok; ++i) ok = __half2float(rm[i]) == __half2float(cm[(size_t)i * 48]) && __half2float(rm[(size_t)3 * n + i]) == __half2float(cm[(size_t)i * 48 + 3]);
		EXPECT(ok);
	}
	// misuse comes back as an exception, not as a crash
	EXPECT(throws([&] { GPUMatrixDynamic<T> wrong{24, n, stream}; enc->forward(stream, X, &wrong); }));
	EXPECT(throws([&] { GPUMatrixDynamic<float> wrong{4, n, stream}; enc->forward(stream, wrong, &E); }));

	{  // reduce_sum, both forms
		std::vector<float> h(100003);
		double want = 0;
		for (auto& v : h) v = u01(rng), want += v;
		GPUMemory<float> dvals, out(reduce_sum_workspace_size(100003));
		dvals.resize_and_copy_from_host(h);
		out.memset(0);
		const float got = reduce_sum(dvals.data(), 100003, stream);
		EXPECT(std::fabs(got - want) < 1e-4 * want);
		reduce_sum(dvals.data(), [] __device__(float v) { return 2.0f * v; }, out.data(), 100003, stream);
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		EXPECT(std::fabs(to_host(out.data(), 1)[0] - 2 * want) < 2e-4 * want);
	}
	{  // workspace cut into typed arrays on 256-byte boundaries
		GPUMemoryArena::Allocation alloc;
		auto scratch = allocate_workspace_and_distribute<uint32_t, float, T>(stream, &alloc, 3, 100, 7);
		EXPECT((uint8_t*)std::get<0>(scratch) == alloc.data());
		EXPECT((uint8_t*)std::get<1>(scratch) == alloc.data() + 256 && (uint8_t*)std::get<2>(scratch) == alloc.data() + 256 + 512);
		EXPECT(alloc.size() >= 256 + 512 + 256);
	}
	{  // a captured stream replays: two launches inside a graph
		GPUMemory<float> v(1024);
		v.memset(0);
		CudaGraph graph;
		for (int rep = 0; rep < 3; ++rep) {
			auto guard = graph.capture_guard(stream);
			parallel_for_gpu(stream, 1024, [p = v.data()] __device__(size_t i) { p[i] += 1.0f; });
			parallel_for_gpu(stream, 1024, [p = v.data()] __device__(size_t i) { p[i] *= 2.0f; });
		}
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		EXPECT(to_host(v.data(), 1)[0] == 14.0f);  // ((0+1)*2+1)*2+1)*2
	}
	{  // helper streams join the parent
		GPUMemory<float> v(2);
		v.memset(0);
		{
			SyncedMultiStream streams{stream, 2};
			parallel_for_gpu(streams.get(0), 1, [p = v.data()] __device__(size_t) { p[0] = 1.0f; });
			parallel_for_gpu(streams.get(1), 1, [p = v.data()] __device__(size_t) { p[1] = 2.0f; });
		}
		parallel_for_gpu(stream, 1, [p = v.data()] __device__(size_t) { p[0] += p[1]; });
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		EXPECT(to_host(v.data(), 1)[0] == 3.0f);
	}
	{  // Trainer + Ema(ExponentialDecay(Adam)) over an encoding + network model
		auto model = std::make_shared<NetworkWithInputEncoding<T>>(3, 16, kGrid, [] { json j = kSdfNet; j.erase("n_input_dims"); j["n_hidden_layers"] = 2; return j; }());
		EXPECT(model->n_params() == 64 * 32 + 64 * 64 + 16 * 64 + 12599920u);
		std::shared_ptr<Optimizer<T>> opt{create_optimizer<T>(kAdam)};
		std::shared_ptr<Loss<T>> loss{create_loss<T>({{"otype", "L2"}})};
		auto trainer = std::make_shared<Trainer<float, T, T>>(model, opt, loss, 1337);
		const size_t np = trainer->n_params(), n_matrix = 64 * 32 + 64 * 64 + 16 * 64;
		EXPECT(np == model->n_params() && trainer->params_inference() == opt->custom_weights() && trainer->params() != trainer->params_inference());
		{  // initial weights: matrices spread, grid within +-1e-4, every copy equal
			auto full = to_host(trainer->params_full_precision(), n_matrix + 1000);
			float mx = 0, gmx = 0;
			for (size_t i = 0; i < n_matrix; ++i) mx = std::fmax(mx, std::fabs(full[i]));
			for (size_t i = n_matrix; i < n_matrix + 1000; ++i) gmx = std::fmax(gmx, std::fabs(full[i]));
			EXPECT(mx > 0.1f && mx < 0.3f && gmx > 0 && gmx <= 1e-4f);
			EXPECT(same(trainer->params(), trainer->params_inference(), np));
		}
		// gradient of +1 (times the loss scale) on every matrix weight, one grid entry touched
		std::vector<T> g(np, __float2half(0.0f));
		for (size_t i = 0; i < n_matrix; ++i) g[i] = __float2half(128.0f);
		g[n_matrix + 5] = __float2half(-128.0f);
		CUDA_CHECK_THROW(cudaMemcpy(trainer->param_gradients(), g.data(), np * sizeof(T), cudaMemcpyHostToDevice));
		auto before = to_host(trainer->params_full_precision(), n_matrix + 8);
		trainer->optimizer_step(stream, 128.0f);
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		auto after = to_host(trainer->params_full_precision(), n_matrix + 8);
		EXPECT(std::fabs((before[0] - after[0]) - 1e-2f) < 2e-4f);             // the first Adam step moves by the learning rate
		EXPECT(std::fabs((after[n_matrix + 5] - before[n_matrix + 5]) - 1e-2f) < 2e-4f);
		EXPECT(after[n_matrix + 6] == before[n_matrix + 6]);                   // untouched grid entries keep their weight
		EXPECT(opt->step() == 1 && opt->learning_rate() == 1e-2f);
		trainer->optimizer_step(stream, 128.0f);
		EXPECT(opt->step() == 2 && std::fabs(opt->learning_rate() - 5e-3f) < 1e-9f);  // decay from step 2 on, every step
		{  // the EMA after one step is the weights themselves (bias-corrected), afterwards it lags
			auto ema = to_host(trainer->params_inference(), 4);
			auto cur = to_host(trainer->params(), 4);
			EXPECT(__half2float(ema[0]) != __half2float(cur[0]));
		}
		// snapshot: round trip with optimizer state
		json snap = trainer->serialize(true);
		EXPECT(snap["n_params"] == np && snap["params_type"] == "__half" && snap["params_binary"].get_binary().size() == np * sizeof(T));
		auto params_then = to_host(trainer->params(), 64);
		auto ema_then = to_host(trainer->params_inference(), 64);
		trainer->optimizer_step(stream, 128.0f);
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		EXPECT(to_host(trainer->params(), 1)[0] != params_then[0]);
		// through msgpack, as the reference stores snapshots (src/testbed.cu:3140)
		trainer->deserialize(json::from_msgpack(json::to_msgpack(snap)));
		EXPECT(!std::memcmp(to_host(trainer->params(), 64).data(), params_then.data(), 64 * sizeof(T)));
		EXPECT(!std::memcmp(to_host(trainer->params_inference(), 64).data(), ema_then.data(), 64 * sizeof(T)));
		EXPECT(opt->step() == 2);
		// parameters only: every copy becomes the stored inference weights
		json small_snap = trainer->serialize(false);
		EXPECT(!small_snap.contains("optimizer"));
		trainer->deserialize(small_snap);
		EXPECT(!std::memcmp(to_host(trainer->params(), 64).data(), ema_then.data(), 64 * sizeof(T)));
		EXPECT(throws([&] { json bad = small_snap; bad["n_params"] = 5; trainer->deserialize(bad); }));
		// frozen groups: with the canonical model switched off nothing moves
		opt->update_hyperparams({{"nested", {{"nested", {{"optimize_canonical_params", false}}}}}});
		auto frozen_before = to_host(trainer->params_full_precision(), 4);
		CUDA_CHECK_THROW(cudaMemcpy(trainer->param_gradients(), g.data(), np * sizeof(T), cudaMemcpyHostToDevice));
		trainer->optimizer_step(stream, 128.0f);
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		EXPECT(to_host(trainer->params_full_precision(), 4)[0] == frozen_before[0]);
		// one generic training step runs end to end (forward, L2 loss, backward, optimizer)
		opt->update_hyperparams({{"nested", {{"nested", {{"optimize_canonical_params", true}}}}}});
		GPUMatrix<float> target{16, n, stream};
		auto ctx = trainer->training_step(stream, X, target);
		const float l = trainer->loss(stream, *ctx);
		EXPECT(std::isfinite(l) && l >= 0.0f);
	}
	}
	CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
	cudaStreamDestroy(stream);
	std::printf(g_failed ? "header test FAILED (%d)\n" : "header test ok\n", g_failed);
	return g_failed ? 1 : 0;
}
