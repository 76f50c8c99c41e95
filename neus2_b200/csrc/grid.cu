// Stand-alone multiresolution hash-grid kernels: the tcnn GridEncoding entry points the reference calls
// (forward + dy/dx, backward to input, backward to parameters, second-order backward_backward_input).
// One thread per (sample, level) pair; blockIdx.y is the level so a warp gathers from one level for 32
// consecutive samples (neighbouring samples of a ray share cells at the coarse levels).
#include "common.cuh"

namespace n2b {

__global__ void __launch_bounds__(256) grid_forward_kernel(GridLevels lv, uint32_t n, const float* __restrict__ x, uint32_t x_stride,
                                                           const __half* __restrict__ grid, __half* __restrict__ enc,
                                                           float* __restrict__ dy_dx) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	const uint32_t l = blockIdx.y;
	if (i >= n) return;
	const uint32_t W = 2 * lv.n_levels;
	if (l >= lv.n_active) {
		reinterpret_cast<__half2*>(enc)[(size_t)i * lv.n_levels + l] = __floats2half2_rn(0.f, 0.f);
		if (dy_dx) {
			float* o = dy_dx + ((size_t)i * W + 2 * l) * 3;
#pragma unroll
			for (int e = 0; e < 6; ++e) o[e] = 0.f;
		}
		return;
	}
	const float xs[3] = {x[(size_t)i * x_stride], x[(size_t)i * x_stride + 1], x[(size_t)i * x_stride + 2]};
	const Cell c = level_cell(lv, l, xs);
	float a0 = 0.f, a1 = 0.f, j0[3] = {0.f, 0.f, 0.f}, j1[3] = {0.f, 0.f, 0.f};
	__half2 th[8];
#pragma unroll
	for (uint32_t k = 0; k < 8; ++k) th[k] = ldg_h2(grid, corner_index(lv, l, c, k));
#pragma unroll
	for (uint32_t k = 0; k < 8; ++k) {
		const float2 t = __half22float2(th[k]);
		const float w = corner_weight(c, k);
		a0 = __fmaf_rn(w, t.x, a0);
		a1 = __fmaf_rn(w, t.y, a1);
		if (dy_dx) {
			float dw[3];
			corner_dweight(c, lv.scale[l], k, dw);
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				j0[e] = __fmaf_rn(dw[e], t.x, j0[e]);
				j1[e] = __fmaf_rn(dw[e], t.y, j1[e]);
			}
		}
	}
	reinterpret_cast<__half2*>(enc)[(size_t)i * lv.n_levels + l] = __floats2half2_rn(a0, a1);
	if (dy_dx) {
		float* o = dy_dx + ((size_t)i * W + 2 * l) * 3;
#pragma unroll
		for (int e = 0; e < 3; ++e) {
			o[e] = j0[e];
			o[3 + e] = j1[e];
		}
	}
}

// dL/dx[e] = sum_{l,f} (d enc_{l,f} / d x_e) * dL/denc_{l,f};  one thread per sample (the sum runs over levels)
__global__ void __launch_bounds__(128) grid_backward_input_kernel(GridLevels lv, uint32_t n, const float* __restrict__ x,
                                                                  uint32_t x_stride, const __half* __restrict__ grid,
                                                                  const __half* __restrict__ dL_denc, float* __restrict__ dL_dx) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n) return;
	const float xs[3] = {x[(size_t)i * x_stride], x[(size_t)i * x_stride + 1], x[(size_t)i * x_stride + 2]};
	float g[3] = {0.f, 0.f, 0.f};
	for (uint32_t l = 0; l < lv.n_active; ++l) {
		const Cell c = level_cell(lv, l, xs);
		const float2 dy = __half22float2(reinterpret_cast<const __half2*>(dL_denc)[(size_t)i * lv.n_levels + l]);
		float j0[3] = {0.f, 0.f, 0.f}, j1[3] = {0.f, 0.f, 0.f};
#pragma unroll
		for (uint32_t k = 0; k < 8; ++k) {
			const float2 t = __half22float2(ldg_h2(grid, corner_index(lv, l, c, k)));
			float dw[3];
			corner_dweight(c, lv.scale[l], k, dw);
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				j0[e] = __fmaf_rn(dw[e], t.x, j0[e]);
				j1[e] = __fmaf_rn(dw[e], t.y, j1[e]);
			}
		}
#pragma unroll
		for (int e = 0; e < 3; ++e) {
			g[e] = __fmaf_rn(j0[e], dy.x, g[e]);
			g[e] = __fmaf_rn(j1[e], dy.y, g[e]);
		}
	}
#pragma unroll
	for (int e = 0; e < 3; ++e) dL_dx[(size_t)i * 3 + e] = g[e];
}

__global__ void __launch_bounds__(256) grid_backward_params_kernel(GridLevels lv, uint32_t n, const float* __restrict__ x,
                                                                   uint32_t x_stride, const __half* __restrict__ dL_denc,
                                                                   __half* __restrict__ grad) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	const uint32_t l = blockIdx.y;
	if (i >= n || l >= lv.n_active) return;
	const float xs[3] = {x[(size_t)i * x_stride], x[(size_t)i * x_stride + 1], x[(size_t)i * x_stride + 2]};
	const Cell c = level_cell(lv, l, xs);
	const float2 dy = __half22float2(reinterpret_cast<const __half2*>(dL_denc)[(size_t)i * lv.n_levels + l]);
#pragma unroll
	for (uint32_t k = 0; k < 8; ++k) {
		const float w = corner_weight(c, k);
		red_add_h2(grad, corner_index(lv, l, c, k), w * dy.x, w * dy.y);
	}
}

// Second order: coef_k = grad_x(w_k) . v ; grad[k] += coef_k * g_e[l] ; dy_enc[l] = sum_k coef_k * theta_k
__global__ void __launch_bounds__(256) grid_bwd_bwd_kernel(GridLevels lv, uint32_t n, const float* __restrict__ x, uint32_t x_stride,
                                                           const __half* __restrict__ grid, const float* __restrict__ v,
                                                           const __half* __restrict__ g_e, __half* __restrict__ dy_enc,
                                                           __half* __restrict__ grad) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	const uint32_t l = blockIdx.y;
	if (i >= n) return;
	if (l >= lv.n_active) {
		if (dy_enc) reinterpret_cast<__half2*>(dy_enc)[(size_t)i * lv.n_levels + l] = __floats2half2_rn(0.f, 0.f);
		return;
	}
	const float xs[3] = {x[(size_t)i * x_stride], x[(size_t)i * x_stride + 1], x[(size_t)i * x_stride + 2]};
	const float vv[3] = {v[(size_t)i * 3], v[(size_t)i * 3 + 1], v[(size_t)i * 3 + 2]};
	const Cell c = level_cell(lv, l, xs);
	const float2 ge = __half22float2(reinterpret_cast<const __half2*>(g_e)[(size_t)i * lv.n_levels + l]);
	float a0 = 0.f, a1 = 0.f;
#pragma unroll
	for (uint32_t k = 0; k < 8; ++k) {
		const uint32_t idx = corner_index(lv, l, c, k);
		float dw[3];
		corner_dweight(c, lv.scale[l], k, dw);
		const float coef = dw[0] * vv[0] + dw[1] * vv[1] + dw[2] * vv[2];
		if (dy_enc) {
			const float2 t = __half22float2(ldg_h2(grid, idx));
			a0 = __fmaf_rn(coef, t.x, a0);
			a1 = __fmaf_rn(coef, t.y, a1);
		}
		if (grad) red_add_h2(grad, idx, coef * ge.x, coef * ge.y);
	}
	if (dy_enc) reinterpret_cast<__half2*>(dy_enc)[(size_t)i * lv.n_levels + l] = __floats2half2_rn(a0, a1);
}

__global__ void sh4_kernel(uint32_t n, const float* __restrict__ dir01, uint32_t stride, __half* __restrict__ out) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n) return;
	const float d[3] = {dir01[(size_t)i * stride], dir01[(size_t)i * stride + 1], dir01[(size_t)i * stride + 2]};
	float o[16];
	sh4_eval(d, o);
	__half2* dst = reinterpret_cast<__half2*>(out + (size_t)i * 16);
#pragma unroll
	for (int k = 0; k < 8; ++k) dst[k] = __floats2half2_rn(o[2 * k], o[2 * k + 1]);
}

}  // namespace n2b

using namespace n2b;

extern "C" int neus2b_grid_level_table(const neus2b_grid_desc* desc, uint32_t* offsets, uint32_t* resolutions, float* scales,
                                       uint32_t* hashed) {
	GridLevels lv;
	int rc = make_levels(desc, &lv);
	if (rc) return rc;
	for (uint32_t l = 0; l <= NEUS2B_MAX_LEVELS; ++l)
		if (offsets) offsets[l] = lv.offset[l];
	for (uint32_t l = 0; l < NEUS2B_MAX_LEVELS; ++l) {
		if (resolutions) resolutions[l] = lv.res[l];
		if (scales) scales[l] = lv.scale[l];
		if (hashed) hashed[l] = lv.hashed[l];
	}
	return NEUS2B_OK;
}

extern "C" int neus2b_grid_n_params(const neus2b_grid_desc* desc, uint64_t* n_fp16) {
	GridLevels lv;
	int rc = make_levels(desc, &lv);
	if (rc) return rc;
	if (!n_fp16) return NEUS2B_E_INVALID;
	*n_fp16 = (uint64_t)lv.offset[NEUS2B_MAX_LEVELS] * 2u;
	return NEUS2B_OK;
}

extern "C" int neus2b_model_n_params(const neus2b_grid_desc* desc, uint64_t* n_fp16) {
	uint64_t g = 0;
	int rc = neus2b_grid_n_params(desc, &g);
	if (rc) return rc;
	*n_fp16 = NEUS2B_MLP_N + g + 4u;
	return NEUS2B_OK;
}

extern "C" int neus2b_grid_forward(const neus2b_grid_desc* desc, uint32_t n, const float* d_x, uint32_t x_stride,
                                   const uint16_t* d_grid, uint16_t* d_enc, float* d_dy_dx, neus2b_stream_t stream) {
	GridLevels lv;
	int rc = make_levels(desc, &lv);
	if (rc) return rc;
	if (!d_x || !d_grid || !d_enc || x_stride < 3) return NEUS2B_E_INVALID;
	if (n == 0) return NEUS2B_OK;
	dim3 grid(div_up(n, 256), lv.n_levels);
	grid_forward_kernel<<<grid, 256, 0, stream>>>(lv, n, d_x, x_stride, (const __half*)d_grid, (__half*)d_enc, d_dy_dx);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_grid_backward_input(const neus2b_grid_desc* desc, uint32_t n, const float* d_x, uint32_t x_stride,
                                          const uint16_t* d_grid, const uint16_t* d_dL_denc, float* d_dL_dx,
                                          neus2b_stream_t stream) {
	GridLevels lv;
	int rc = make_levels(desc, &lv);
	if (rc) return rc;
	if (!d_x || !d_grid || !d_dL_denc || !d_dL_dx || x_stride < 3) return NEUS2B_E_INVALID;
	if (n == 0) return NEUS2B_OK;
	grid_backward_input_kernel<<<div_up(n, 128), 128, 0, stream>>>(lv, n, d_x, x_stride, (const __half*)d_grid,
	                                                               (const __half*)d_dL_denc, d_dL_dx);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_grid_backward_params(const neus2b_grid_desc* desc, uint32_t n, const float* d_x, uint32_t x_stride,
                                           const uint16_t* d_dL_denc, uint16_t* d_grad, int grad_mode, neus2b_stream_t stream) {
	GridLevels lv;
	int rc = make_levels(desc, &lv);
	if (rc) return rc;
	if (grad_mode == NEUS2B_GRAD_IGNORE) return NEUS2B_OK;
	if (!d_x || !d_dL_denc || !d_grad || x_stride < 3) return NEUS2B_E_INVALID;
	if (grad_mode == NEUS2B_GRAD_OVERWRITE)
		N2B_CHECK_CUDA(cudaMemsetAsync(d_grad, 0, (size_t)lv.offset[NEUS2B_MAX_LEVELS] * 4u, stream));
	if (n == 0) return NEUS2B_OK;
	dim3 grid(div_up(n, 256), lv.n_levels);
	grid_backward_params_kernel<<<grid, 256, 0, stream>>>(lv, n, d_x, x_stride, (const __half*)d_dL_denc, (__half*)d_grad);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_grid_backward_backward_input(const neus2b_grid_desc* desc, uint32_t n, const float* d_x, uint32_t x_stride,
                                                   const uint16_t* d_grid, const float* d_v, const uint16_t* d_g_e,
                                                   uint16_t* d_dy_enc, uint16_t* d_grad, int grad_mode, neus2b_stream_t stream) {
	GridLevels lv;
	int rc = make_levels(desc, &lv);
	if (rc) return rc;
	if (!d_x || !d_grid || !d_v || !d_g_e || x_stride < 3) return NEUS2B_E_INVALID;
	if (grad_mode != NEUS2B_GRAD_IGNORE && !d_grad) return NEUS2B_E_INVALID;
	if (grad_mode == NEUS2B_GRAD_OVERWRITE)
		N2B_CHECK_CUDA(cudaMemsetAsync(d_grad, 0, (size_t)lv.offset[NEUS2B_MAX_LEVELS] * 4u, stream));
	if (n == 0) return NEUS2B_OK;
	dim3 grid(div_up(n, 256), lv.n_levels);
	grid_bwd_bwd_kernel<<<grid, 256, 0, stream>>>(lv, n, d_x, x_stride, (const __half*)d_grid, d_v, (const __half*)d_g_e,
	                                              (__half*)d_dy_enc, grad_mode == NEUS2B_GRAD_IGNORE ? nullptr : (__half*)d_grad);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_sh4_forward(uint32_t n, const float* d_dir01, uint32_t stride, uint16_t* d_out, neus2b_stream_t stream) {
	if (!d_dir01 || !d_out || stride < 3) return NEUS2B_E_INVALID;
	if (n == 0) return NEUS2B_OK;
	sh4_kernel<<<div_up(n, 256), 256, 0, stream>>>(n, d_dir01, stride, (__half*)d_out);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}
