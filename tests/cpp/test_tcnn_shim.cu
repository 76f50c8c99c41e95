// Drives the C++ mirror of the tiny-cuda-nn objects (include/neus2b_tcnn.hpp) the way NerfNetwork drives them
// (nerf_network.h:184-234 forward, :388-429 backward) and checks every result against the same C-ABI entry point called
// directly (bit for bit where the kernel's summation order is fixed), plus the error convention.  Exit code 0 = pass.  With --check-only nothing touches a GPU.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "neus2b_tcnn.hpp"

using namespace tcnn;
using T = __half;

static int g_failed = 0;
#define EXPECT(cond)                                                      \
	do {                                                                  \
		if (!(cond)) {                                                    \
			std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
			++g_failed;                                                   \
		}                                                                 \
	} while (0)

template <typename U>
static bool same(const GPUMemory<U>& a, const U* b_dev, size_t n) {
	std::vector<U> x(n), y(n);
	a.copy_to_host(x.data(), n);
	cudaMemcpy(y.data(), b_dev, n * sizeof(U), cudaMemcpyDeviceToHost);
	return std::memcmp(x.data(), y.data(), n * sizeof(U)) == 0;
}

int main(int argc, char** argv) {
	// ---- host-only part: shapes, parameter counts, error convention
	GridEncoding<T> grid(16, 19, 16, 1.447f);
	EXPECT(grid.n_params() == 12599920u);
	EXPECT(grid.padded_output_width() == 32 && grid.input_width() == 3);
	FullyFusedMLP<T> sdf_net(48, 1), rgb_net(48, 2);
	EXPECT(sdf_net.n_params() == 4096 && rgb_net.n_params() == 8192);
	bool threw = false;
	try {
		FullyFusedMLP<T> bad(40, 3);
	} catch (const std::runtime_error&) {
		threw = true;
	}
	EXPECT(threw);
	threw = false;
	try {
		neus2b_check(NEUS2B_E_INVALID, "probe");
	} catch (const std::runtime_error& e) {
		threw = std::strstr(e.what(), "probe") != nullptr;
	}
	EXPECT(threw);
	if (argc > 1 && std::strcmp(argv[1], "--check-only") == 0) {
		std::printf(g_failed ? "host checks FAILED\n" : "host checks ok\n");
		return g_failed ? 1 : 0;
	}

	// ---- device part
	const uint32_t n = 4096 + 37;
	std::mt19937 rng(7);
	std::uniform_real_distribution<float> u01(0.f, 1.f), small(-1e-2f, 1e-2f), wdist(-0.2f, 0.2f);
	std::vector<float> h_x(n * 3);
	for (auto& v : h_x) v = u01(rng);
	std::vector<T> h_grid(grid.n_params());
	for (auto& v : h_grid) v = __float2half(small(rng));
	std::vector<T> h_w(sdf_net.n_params());
	for (auto& v : h_w) v = __float2half(wdist(rng));
	std::vector<T> h_dy(n * 16);
	for (auto& v : h_dy) v = __float2half(small(rng));

	GPUMemory<float> x;
	x.resize_and_copy_from_host(h_x);
	GPUMemory<T> grid_params, grid_grads(grid.n_params()), w, dy;
	grid_params.resize_and_copy_from_host(h_grid);
	w.resize_and_copy_from_host(h_w);
	dy.resize_and_copy_from_host(h_dy);
	GPUMemory<float> w_grads(sdf_net.n_params());
	grid.set_params(grid_params.data(), grid_params.data(), nullptr, grid_grads.data());
	sdf_net.set_params(w.data(), w.data(), nullptr, w_grads.data());
	cudaStream_t stream;
	CUDA_CHECK_THROW(cudaStreamCreate(&stream));

	// forward: encoding -> [enc(32) | pad] -> SDF network
	GPUMatrixDynamic<float> X(x.data(), 3, n);
	GPUMatrixDynamic<T> Z(48, n), Y(16, n);
	Z.memset_async(stream, 0);
	GPUMemory<T> enc(n * 32);
	GPUMatrixDynamic<T> E(enc.data(), 32, n);
	auto enc_ctx = grid.forward(stream, X, &E, false, true);
	CUDA_CHECK_THROW(cudaMemcpy2DAsync(Z.data(), 48 * sizeof(T), E.data(), 32 * sizeof(T), 32 * sizeof(T), n, cudaMemcpyDeviceToDevice, stream));
	auto net_ctx = sdf_net.forward_impl(stream, Z, &Y);
	// backward: network, then encoding (parameter gradients overwritten)
	GPUMatrixDynamic<T> dY(dy.data(), 16, n), dZ(48, n);
	sdf_net.backward_impl(stream, *net_ctx, Z, Y, dY, &dZ, false, EGradientMode::Overwrite);
	GPUMemory<T> denc(n * 32);
	CUDA_CHECK_THROW(cudaMemcpy2DAsync(denc.data(), 32 * sizeof(T), dZ.data(), 48 * sizeof(T), 32 * sizeof(T), n, cudaMemcpyDeviceToDevice, stream));
	GPUMatrixDynamic<T> dE(denc.data(), 32, n);
	GPUMatrixDynamic<float> dX(3, n);
	grid.backward(stream, *enc_ctx, X, E, dE, &dX, false, EGradientMode::Overwrite);
	CUDA_CHECK_THROW(cudaStreamSynchronize(stream));

	// the same through the C ABI
	GPUMemory<T> enc2(n * 32), y2(n * 16), hid2(n * 64), dz2(n * 48), gg2(grid.n_params());
	GPUMemory<float> dydx2((size_t)n * 32 * 3), wg2(sdf_net.n_params()), dx2(n * 3);
	const neus2b_grid_desc d = grid.desc();
	EXPECT(neus2b_grid_forward(&d, n, x.data(), 3, (const uint16_t*)grid_params.data(), (uint16_t*)enc2.data(), dydx2.data(), stream) == 0);
	EXPECT(neus2b_mlp_forward(n, 48, 1, (const uint16_t*)w.data(), (const uint16_t*)Z.data(), (uint16_t*)y2.data(), (uint16_t*)hid2.data(), stream) == 0);
	EXPECT(neus2b_mlp_backward(n, 48, 1, (const uint16_t*)w.data(), (const uint16_t*)Z.data(), (const uint16_t*)hid2.data(), (const uint16_t*)dy.data(),
	                           (uint16_t*)dz2.data(), wg2.data(), NEUS2B_GRAD_OVERWRITE, stream) == 0);
	EXPECT(neus2b_grid_backward_input(&d, n, x.data(), 3, (const uint16_t*)grid_params.data(), (const uint16_t*)denc.data(), dx2.data(), stream) == 0);
	EXPECT(neus2b_grid_backward_params(&d, n, x.data(), 3, (const uint16_t*)denc.data(), (uint16_t*)gg2.data(), NEUS2B_GRAD_OVERWRITE, stream) == 0);
	CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
	EXPECT(same(enc2, E.data(), (size_t)n * 32));
	EXPECT(same(y2, Y.data(), (size_t)n * 16));
	EXPECT(same(dz2, dZ.data(), (size_t)n * 48));
	EXPECT(same(dx2, dX.data(), (size_t)n * 3));
	{
		// fp32 sums over CTAs in arrival order: equal up to rounding
		std::vector<float> a(sdf_net.n_params()), b(sdf_net.n_params());
		wg2.copy_to_host(a.data(), a.size());
		w_grads.copy_to_host(b.data(), b.size());
		double err = 0, ref = 0;
		for (size_t i = 0; i < a.size(); ++i) err = std::fmax(err, std::fabs((double)a[i] - b[i])), ref = std::fmax(ref, std::fabs((double)a[i]));
		EXPECT(ref > 0 && err <= 1e-5 * ref);
	}
	{
		// the scattered fp16 atomics commute only up to rounding: compare the two gradient tables by cosine
		std::vector<T> a(grid.n_params()), b(grid.n_params());
		gg2.copy_to_host(a.data(), a.size());
		grid_grads.copy_to_host(b.data(), b.size());
		double ab = 0, aa = 0, bb = 0;
		for (size_t i = 0; i < a.size(); ++i) {
			const double p = __half2float(a[i]), q = __half2float(b[i]);
			ab += p * q, aa += p * p, bb += q * q;
		}
		EXPECT(aa > 0 && ab / std::sqrt(aa * bb) > 0.9999);
	}
	// SDF output is finite and not constant
	{
		std::vector<T> y(n * 16);
		y2.copy_to_host(y.data(), y.size());
		float mn = 1e30f, mx = -1e30f;
		for (uint32_t i = 0; i < n; ++i) {
			const float v = __half2float(y[i * 16]);
			EXPECT(std::isfinite(v));
			mn = std::fmin(mn, v), mx = std::fmax(mx, v);
		}
		EXPECT(mx > mn);
	}
	// a misuse comes back as an exception, not as a crash
	threw = false;
	try {
		GPUMatrixDynamic<float> bad(x.data(), 3, n, RM);
		grid.forward(stream, bad, &E);
	} catch (const std::runtime_error&) {
		threw = true;
	}
	EXPECT(threw);
	// optimizer: one step moves the weights against the gradient
	{
		const uint64_t np = 12288 + grid.n_params() + 4;
		NeusAdamOptimizer opt(np, 12288);
		std::vector<float> master(np, 0.25f);
		opt.set_params_full_precision(master.data(), np);
		GPUMemory<T> p(np), pe(np), gg(grid.n_params());
		GPUMemory<float> gm(12288), gv(4);
		gm.memset(0), gv.memset(0), gg.memset(0);
		std::vector<float> one(12288, 128.0f);  // loss-scaled gradient of +1 on every MLP weight
		gm.copy_from_host(one);
		opt.step(stream, 128.0f, p.data(), pe.data(), gm.data(), gg.data(), gv.data());
		CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
		std::vector<T> hp(np);
		p.copy_to_host(hp.data(), np);
		EXPECT(__half2float(hp[0]) < 0.25f && __half2float(hp[0]) > 0.23f);  // lr 1e-2, first step moves by about lr
		EXPECT(__half2float(hp[12288 + 5]) == 0.25f);                         // zero gradient on the grid: untouched
		EXPECT(opt.step() == 1);
	}
	cudaStreamDestroy(stream);
	std::printf(g_failed ? "shim test FAILED (%d)\n" : "shim test ok\n", g_failed);
	return g_failed ? 1 : 0;
}
