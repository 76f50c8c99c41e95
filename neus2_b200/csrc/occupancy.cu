// Occupancy grid maintenance and the fused optimizer step.
//  * occupancy: src/testbed_nerf.cu:630-785 (kernels) and :3287-3391 (update_density_grid_nerf,
//    update_density_grid_mean_and_bitfield) of the reference; the SDF evaluation in the middle is the fused
//    encoding + SDF-MLP kernel (neus2b_neus_sdf).
//  * optimizer: Ema o ExponentialDecay o Adam of configs/nerf/dtu.json:5-27, one streaming pass that also casts to
//    fp16, maintains the EMA copy and clears the gradients for the next step.
#include "common.cuh"

namespace n2b {

__device__ __forceinline__ uint32_t expand_bits_o(uint32_t v) {
	v = (v * 0x00010001u) & 0xFF0000FFu;
	v = (v * 0x00000101u) & 0x0F00F00Fu;
	v = (v * 0x00000011u) & 0xC30C30C3u;
	v = (v * 0x00000005u) & 0x49249249u;
	return v;
}
__device__ __forceinline__ uint32_t morton3d_o(uint32_t x, uint32_t y, uint32_t z) {
	return expand_bits_o(x) | (expand_bits_o(y) << 1) | (expand_bits_o(z) << 2);
}
__device__ __forceinline__ uint32_t morton3d_invert(uint32_t x) {
	x = x & 0x49249249u;
	x = (x | (x >> 2)) & 0xc30c30c3u;
	x = (x | (x >> 4)) & 0x0f00f00fu;
	x = (x | (x >> 8)) & 0xff0000ffu;
	x = (x | (x >> 16)) & 0x0000ffffu;
	return x;
}

constexpr uint32_t kCells = NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE;

// generate_grid_samples_nerf_nonuniform, src/testbed_nerf.cu:630-659 (unit-cube aabb: warp_position is the identity)
__global__ void occ_samples_kernel(uint32_t n, Pcg32 rng, uint32_t step, const float* __restrict__ grid_in, uint32_t n_cascades,
                                   float thresh, float* __restrict__ pos, uint32_t* __restrict__ indices) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n) return;
	rng.advance((uint64_t)i * 4u);
	const uint32_t level = (uint32_t)(rng.next_float() * (float)n_cascades) % n_cascades;
	uint32_t idx = 0;
	for (uint32_t j = 0; j < 10; ++j) {
		idx = ((i + step * n) * 56924617u + j * 19349663u + 96925573u) % kCells;
		idx += level * kCells;
		if (grid_in[idx] > thresh) break;
	}
	const uint32_t pi = idx % kCells;
	const float c[3] = {(float)morton3d_invert(pi >> 0), (float)morton3d_invert(pi >> 1), (float)morton3d_invert(pi >> 2)};
	float r[3];
#pragma unroll
	for (int e = 0; e < 3; ++e) r[e] = rng.next_float();
#pragma unroll
	for (int e = 0; e < 3; ++e)
		pos[(size_t)i * 3 + e] = __fadd_rn(__fmul_rn(__fsub_rn(__fdiv_rn(__fadd_rn(c[e], r[e]), (float)NEUS2B_GRIDSIZE), 0.5f),
		                                             scalbnf(1.0f, (int)level)), 0.5f);
	indices[i] = idx;
}

// ema_grid_samples_nerf, :700-730
__global__ void occ_ema_kernel(uint32_t n, float decay, float* __restrict__ grid, const float* __restrict__ grid_tmp) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n) return;
	const float prev = grid[i];
	grid[i] = prev < 0.f ? prev : fmaxf(__fmul_rn(prev, decay), grid_tmp[i]);
}

// mean of max(density, 0) over cascade 0 (:3383): fixed-shape double-precision tree, reproducible run to run
__global__ void __launch_bounds__(256) occ_mean_partial_kernel(const float* __restrict__ grid, double* __restrict__ partial) {
	__shared__ double sh[256];
	double acc = 0.0;
	const uint32_t per_block = kCells / 1024u;
	for (uint32_t k = threadIdx.x; k < per_block; k += 256) acc += (double)__fdiv_rn(fmaxf(grid[blockIdx.x * per_block + k], 0.f), (float)kCells);
	sh[threadIdx.x] = acc;
	__syncthreads();
	for (int o = 128; o > 0; o >>= 1) {
		if ((int)threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
		__syncthreads();
	}
	if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
__global__ void occ_mean_final_kernel(const double* __restrict__ partial, float* __restrict__ mean) {
	if (threadIdx.x == 0 && blockIdx.x == 0) {
		double acc = 0.0;
		for (int k = 0; k < 1024; ++k) acc += partial[k];
		*mean = (float)acc;
	}
}

// grid_to_bitfield, :738-762
__global__ void occ_bitfield_kernel(uint32_t n_bytes, uint32_t n_nonzero, const float* __restrict__ grid, uint8_t* __restrict__ bitfield,
                                    const float* __restrict__ mean) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n_bytes) return;
	if (i >= n_nonzero) {
		bitfield[i] = 0;
		return;
	}
	const float thresh = fminf(0.1f, *mean);
	uint8_t bits = 0;
#pragma unroll
	for (uint32_t j = 0; j < 8; ++j) bits |= grid[(size_t)i * 8 + j] > thresh ? (uint8_t)(1u << j) : 0;
	bitfield[i] = bits;
}

// bitfield_max_pool, :764-785
__global__ void occ_maxpool_kernel(uint32_t n, const uint8_t* __restrict__ prev, uint8_t* __restrict__ next) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n) return;
	uint8_t bits = 0;
#pragma unroll
	for (uint32_t j = 0; j < 8; ++j) bits |= prev[(size_t)i * 8 + j] > 0 ? (uint8_t)(1u << j) : 0;
	const uint32_t x = morton3d_invert(i >> 0) + NEUS2B_GRIDSIZE / 8;
	const uint32_t y = morton3d_invert(i >> 1) + NEUS2B_GRIDSIZE / 8;
	const uint32_t z = morton3d_invert(i >> 2) + NEUS2B_GRIDSIZE / 8;
	next[morton3d_o(x, y, z)] |= bits;
}

// ------------------------------------------------------------------------------------------------ Adam
// One element of the Ema o Adam update.  Returns the new weight; m/v are updated in place.
// A gradient that is NaN or infinite counts as absent (bad = true): the parameter keeps its weight and moments.
__device__ __forceinline__ float adam_element(const neus2b_adam_cfg& c, float lr_t, bool matrix, float g, float w, float& m, float& v,
                                              bool& bad) {
	if (!(fabsf(g) <= 3.402823466e+38f)) {
		bad = true;
		return w;
	}
	g = __fdividef(g, c.loss_scale);
	bool upd = true;
	if (matrix) g += c.l2_reg * w;
	else {
		if (g == 0.0f && !(c.flags & NEUS2B_ADAM_UPDATE_UNTOUCHED)) upd = false;  // grid entries no sample touched keep their weight and moments
		if (c.flags & NEUS2B_ADAM_L2_ALL) g += c.l2_reg * w;
	}
	if (upd) {
		m = c.beta1 * m + (1.0f - c.beta1) * g;
		v = c.beta2 * v + (1.0f - c.beta2) * g * g;
		w -= __fdividef(lr_t * m, __fsqrt_rn(v) + c.epsilon);
	}
	return w;
}

// Streaming pass over the parameter block, 4 parameters (8..16-byte accesses) per thread and iteration, enough threads
// resident (<= 32 registers would not buy more: the pass is bound by bytes in flight).  The block is
// [n_matrix MLP weights | grid | 4 variance slots]; n_matrix and the grid size are multiples of 4.
__global__ void __launch_bounds__(256, 8) adam_kernel(neus2b_adam_cfg c, float lr_t, float ema_old, float ema_new_inv, uint64_t n,
                                                      float* __restrict__ grad_mlp, __half* __restrict__ grad_grid,
                                                      float* __restrict__ grad_var, float* __restrict__ master, float* __restrict__ m,
                                                      float* __restrict__ v, __half* __restrict__ params, __half* __restrict__ params_ema,
                                                      float* __restrict__ ema_master) {
	const uint64_t stride = (uint64_t)gridDim.x * blockDim.x * 4u;
	const uint64_t n_grid_end = n - 4u;
	for (uint64_t i0 = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4u; i0 < n; i0 += stride) {
		const bool matrix = i0 < c.n_matrix;
		const bool var = i0 >= n_grid_end;
		float g[4];
		if (matrix) {
			const float4 a = *reinterpret_cast<const float4*>(grad_mlp + i0);
			g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
		} else if (!var) {
			uint2 raw = *reinterpret_cast<const uint2*>(grad_grid + (i0 - c.n_matrix));
			const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
			const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
			g[0] = f0.x; g[1] = f0.y; g[2] = f1.x; g[3] = f1.y;
		} else {
			const float4 a = *reinterpret_cast<const float4*>(grad_var);
			g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
		}
		const float4 w4 = *reinterpret_cast<const float4*>(master + i0);
		const float4 m4 = *reinterpret_cast<const float4*>(m + i0);
		const float4 v4 = *reinterpret_cast<const float4*>(v + i0);
		float w[4] = {w4.x, w4.y, w4.z, w4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
		float em[4] = {0.f, 0.f, 0.f, 0.f};
		if (params_ema) {
			const float4 e4 = *reinterpret_cast<const float4*>(ema_master + i0);
			em[0] = e4.x; em[1] = e4.y; em[2] = e4.z; em[3] = e4.w;
		}
		bool bad = false;
#pragma unroll
		for (int e = 0; e < 4; ++e) w[e] = adam_element(c, lr_t, matrix, g[e], w[e], mm[e], vv[e], bad);
		if (bad && c.d_nonfinite) {
			uint32_t nb = 0;
#pragma unroll
			for (int e = 0; e < 4; ++e) nb += !(fabsf(g[e]) <= 3.402823466e+38f);
			atomicAdd(c.d_nonfinite, nb);
		}
		*reinterpret_cast<float4*>(master + i0) = make_float4(w[0], w[1], w[2], w[3]);
		*reinterpret_cast<float4*>(m + i0) = make_float4(mm[0], mm[1], mm[2], mm[3]);
		*reinterpret_cast<float4*>(v + i0) = make_float4(vv[0], vv[1], vv[2], vv[3]);
		__half2 p01 = __floats2half2_rn(w[0], w[1]), p23 = __floats2half2_rn(w[2], w[3]);
		*reinterpret_cast<uint2*>(params + i0) = make_uint2(*reinterpret_cast<uint32_t*>(&p01), *reinterpret_cast<uint32_t*>(&p23));
		if (params_ema) {
#pragma unroll
			for (int e = 0; e < 4; ++e) em[e] = ((1.0f - c.ema_decay) * w[e] + c.ema_decay * em[e] * ema_old) * ema_new_inv;  // (1, 1 without debiasing)
			*reinterpret_cast<float4*>(ema_master + i0) = make_float4(em[0], em[1], em[2], em[3]);
			__half2 e01 = __floats2half2_rn(em[0], em[1]), e23 = __floats2half2_rn(em[2], em[3]);
			*reinterpret_cast<uint2*>(params_ema + i0) = make_uint2(*reinterpret_cast<uint32_t*>(&e01), *reinterpret_cast<uint32_t*>(&e23));
		}
		// Clear the gradient last, and only where it is set: a store to the address of a load still in flight holds up
		// every later load of the thread until that load has returned (measured: 3.1 instead of 6.1 TB/s for the pass).
		if (g[0] != 0.f || g[1] != 0.f || g[2] != 0.f || g[3] != 0.f) {
			if (matrix) *reinterpret_cast<float4*>(grad_mlp + i0) = make_float4(0.f, 0.f, 0.f, 0.f);
			else if (!var) *reinterpret_cast<uint2*>(grad_grid + (i0 - c.n_matrix)) = make_uint2(0u, 0u);
			else *reinterpret_cast<float4*>(grad_var) = make_float4(0.f, 0.f, 0.f, 0.f);
		}
	}
}

// Same update with the optimizer-private state interleaved per parameter: state[i] = {master, m, v, ema master}, one
// read-modify-write stream of 16 bytes per parameter instead of four arrays.
__global__ void __launch_bounds__(256, 8) adam_packed_kernel(neus2b_adam_cfg c, float lr_t, float ema_old, float ema_new_inv, uint64_t n,
                                                             float* __restrict__ grad_mlp, __half* __restrict__ grad_grid,
                                                             float* __restrict__ grad_var, float4* __restrict__ state,
                                                             __half* __restrict__ params, __half* __restrict__ params_ema) {
	const uint64_t stride = (uint64_t)gridDim.x * blockDim.x * 2u;
	const uint64_t n_grid_end = n - 4u;
	for (uint64_t i0 = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2u; i0 < n; i0 += stride) {
		const bool matrix = i0 < c.n_matrix;
		float g[2];
		if (matrix) {
			const float2 a = *reinterpret_cast<const float2*>(grad_mlp + i0);
			g[0] = a.x; g[1] = a.y;
		} else if (i0 < n_grid_end) {
			const __half2 h = *reinterpret_cast<const __half2*>(grad_grid + (i0 - c.n_matrix));
			const float2 f = __half22float2(h);
			g[0] = f.x; g[1] = f.y;
		} else {
			g[0] = grad_var[i0 - n_grid_end];
			g[1] = grad_var[i0 - n_grid_end + 1];
		}
		float4 s0 = state[i0], s1 = state[i0 + 1];
		bool bad = false;
		s0.x = adam_element(c, lr_t, matrix, g[0], s0.x, s0.y, s0.z, bad);
		s1.x = adam_element(c, lr_t, matrix, g[1], s1.x, s1.y, s1.z, bad);
		if (bad && c.d_nonfinite) atomicAdd(c.d_nonfinite, (uint32_t)!(fabsf(g[0]) <= 3.402823466e+38f) + (uint32_t)!(fabsf(g[1]) <= 3.402823466e+38f));
		s0.w = ((1.0f - c.ema_decay) * s0.x + c.ema_decay * s0.w * ema_old) * ema_new_inv;
		s1.w = ((1.0f - c.ema_decay) * s1.x + c.ema_decay * s1.w * ema_old) * ema_new_inv;
		state[i0] = s0;
		state[i0 + 1] = s1;
		*reinterpret_cast<__half2*>(params + i0) = __floats2half2_rn(s0.x, s1.x);
		if (params_ema) *reinterpret_cast<__half2*>(params_ema + i0) = __floats2half2_rn(s0.w, s1.w);
		if (g[0] != 0.f || g[1] != 0.f) {  // cleared last and only where set, as in adam_kernel
			if (matrix) *reinterpret_cast<float2*>(grad_mlp + i0) = make_float2(0.f, 0.f);
			else if (i0 < n_grid_end) *reinterpret_cast<__half2*>(grad_grid + (i0 - c.n_matrix)) = __floats2half2_rn(0.f, 0.f);
			else grad_var[i0 - n_grid_end] = grad_var[i0 - n_grid_end + 1] = 0.f;
		}
	}
}

// state[i].{x|y|z|w} <-> contiguous array (set / get of the master or EMA parameters)
__global__ void state_scatter_kernel(uint64_t n, const float* __restrict__ src, float4* __restrict__ state, __half* __restrict__ p,
                                     __half* __restrict__ pe) {
	for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
		const float w = src[i];
		state[i] = make_float4(w, 0.f, 0.f, w);
		p[i] = __float2half_rn(w);
		pe[i] = __float2half_rn(w);
	}
}
__global__ void state_gather_kernel(uint64_t n, const float4* __restrict__ state, int field, float* __restrict__ dst) {
	for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
		const float4 sv = state[i];
		dst[i] = field == 0 ? sv.x : (field == 1 ? sv.y : (field == 2 ? sv.z : sv.w));
	}
}

int launch_state_scatter(uint64_t n, const float* src, float4* state, __half* p, __half* pe, cudaStream_t s) {
	state_scatter_kernel<<<kSMs * 8, 256, 0, s>>>(n, src, state, p, pe);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}
int launch_state_gather(uint64_t n, const float4* state, int field, float* dst, cudaStream_t s) {
	state_gather_kernel<<<kSMs * 8, 256, 0, s>>>(n, state, field, dst);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

}  // namespace n2b

using namespace n2b;

extern "C" int neus2b_neus_sdf(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n, const float* d_x,
                               uint32_t x_stride, uint16_t* d_sdf, neus2b_stream_t stream);

namespace {
// sdf_to_density_variance_buffer (common_operation.cuh:310-328, every operation in fp16) followed by
// splat_grid_samples_nerf_max_nearest_neighbor (src/testbed_nerf.cu:661-680)
__global__ void occ_splat_entry(uint32_t n, const uint32_t* __restrict__ indices, const __half* __restrict__ sdf,
                                const __half* __restrict__ variance_ptr, float* __restrict__ grid_tmp) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n) return;
	const __half variance = *variance_ptr;
	const __half s = __float2half_rn(expf(__half2float(__hmul(variance, __float2half_rn(10.0f)))));
	const __half x = __hmul(sdf[i], s);
	const __half sg = __float2half_rn(1.0f / (1.0f + expf(-__half2float(x))));
	const __half dens = __hmul(__hmul(s, sg), __hsub(__float2half_rn(1.0f), sg));
	atomicMax(reinterpret_cast<uint32_t*>(grid_tmp) + indices[i], __float_as_uint(__half2float(dens)));
}
}  // namespace

extern "C" int neus2b_occupancy_update(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n_cascades,
                                       uint32_t n_uniform, uint32_t n_nonuniform, neus2b_pcg32 rng_uniform, neus2b_pcg32 rng_nonuniform,
                                       uint32_t ema_step, float decay, float* d_grid, float* d_grid_tmp, uint8_t* d_bitfield,
                                       float* d_mean, float* d_pos, uint32_t* d_idx, uint16_t* d_sdf, double* d_partial,
                                       neus2b_stream_t stream) {
	return neus2b_occupancy_update_moved(desc, d_params, sdf_bias, n_cascades, n_uniform, n_nonuniform, rng_uniform, rng_nonuniform, ema_step, decay,
	                                     d_grid, d_grid_tmp, d_bitfield, d_mean, d_pos, d_idx, d_sdf, d_partial, nullptr, stream);
}

extern "C" int neus2b_occupancy_update_moved(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n_cascades,
                                             uint32_t n_uniform, uint32_t n_nonuniform, neus2b_pcg32 rng_uniform,
                                             neus2b_pcg32 rng_nonuniform, uint32_t ema_step, float decay, float* d_grid, float* d_grid_tmp,
                                             uint8_t* d_bitfield, float* d_mean, float* d_pos, uint32_t* d_idx, uint16_t* d_sdf,
                                             double* d_partial, const neus2b_motion* motion, neus2b_stream_t stream) {
	if (!desc || !d_params || !d_grid || !d_grid_tmp || !d_bitfield || !d_mean || !d_pos || !d_idx || !d_sdf || !d_partial)
		return NEUS2B_E_INVALID;
	if (n_cascades == 0 || n_cascades > NEUS2B_CASCADES) return NEUS2B_E_INVALID;
	GridLevels lv;
	int rc = make_levels(desc, &lv);
	if (rc) return rc;
	const uint32_t n_elements = kCells * n_cascades;
	const uint32_t n = n_uniform + n_nonuniform;
	N2B_CHECK_CUDA(cudaMemsetAsync(d_grid_tmp, 0, sizeof(float) * (size_t)n_elements, stream));
	if (n_uniform) {
		occ_samples_kernel<<<div_up(n_uniform, 256), 256, 0, stream>>>(n_uniform, Pcg32{rng_uniform.state, rng_uniform.inc}, ema_step,
		                                                               d_grid, n_cascades, -0.01f, d_pos, d_idx);
		N2B_CHECK_LAUNCH();
	}
	if (n_nonuniform) {
		occ_samples_kernel<<<div_up(n_nonuniform, 256), 256, 0, stream>>>(n_nonuniform, Pcg32{rng_nonuniform.state, rng_nonuniform.inc},
		                                                                  ema_step, d_grid, n_cascades, 0.1f, d_pos + (size_t)n_uniform * 3,
		                                                                  d_idx + n_uniform);
		N2B_CHECK_LAUNCH();
	}
	if (n) {
		rc = neus2b_neus_sdf_moved(desc, d_params, sdf_bias, n, d_pos, 3, motion, d_sdf, stream);
		if (rc) return rc;
		const __half* var_ptr = (const __half*)d_params + NEUS2B_GRID_OFF + (size_t)lv.offset[NEUS2B_MAX_LEVELS] * 2;
		occ_splat_entry<<<div_up(n, 256), 256, 0, stream>>>(n, d_idx, (const __half*)d_sdf, var_ptr, d_grid_tmp);
		N2B_CHECK_LAUNCH();
	}
	occ_ema_kernel<<<div_up(n_elements, 256), 256, 0, stream>>>(n_elements, decay, d_grid, d_grid_tmp);
	N2B_CHECK_LAUNCH();
	return neus2b_occupancy_mean_and_bitfield(n_cascades, d_grid, d_bitfield, d_mean, d_partial, stream);
}

extern "C" int neus2b_occupancy_mean_and_bitfield(uint32_t n_cascades, const float* d_grid, uint8_t* d_bitfield, float* d_mean,
                                                  double* d_partial, neus2b_stream_t stream_) {
	cudaStream_t stream = (cudaStream_t)stream_;
	if (!d_grid || !d_bitfield || !d_mean || !d_partial || n_cascades == 0 || n_cascades > NEUS2B_CASCADES) return NEUS2B_E_INVALID;
	occ_mean_partial_kernel<<<1024, 256, 0, stream>>>(d_grid, d_partial);
	N2B_CHECK_LAUNCH();
	occ_mean_final_kernel<<<1, 32, 0, stream>>>(d_partial, d_mean);
	N2B_CHECK_LAUNCH();
	const uint32_t n_bytes = kCells / 8 * NEUS2B_CASCADES, n_nonzero = kCells / 8 * n_cascades;
	occ_bitfield_kernel<<<div_up(n_bytes, 256), 256, 0, stream>>>(n_bytes, n_nonzero, d_grid, d_bitfield, d_mean);
	N2B_CHECK_LAUNCH();
	for (uint32_t level = 1; level < NEUS2B_CASCADES; ++level) {
		occ_maxpool_kernel<<<div_up(kCells / 64, 256), 256, 0, stream>>>(kCells / 64, d_bitfield + (size_t)(kCells / 8) * (level - 1),
		                                                                 d_bitfield + (size_t)(kCells / 8) * level);
		N2B_CHECK_LAUNCH();
	}
	return NEUS2B_OK;
}

extern "C" int neus2b_adam_step(const neus2b_adam_cfg* cfg, uint64_t n, float* d_grad_mlp, uint16_t* d_grad_grid, float* d_grad_variance,
                                float* d_master, float* d_m, float* d_v, uint16_t* d_params, uint16_t* d_params_ema, float* d_ema_master,
                                neus2b_stream_t stream) {
	if (!cfg || !d_grad_mlp || !d_grad_grid || !d_grad_variance || !d_master || !d_m || !d_v || !d_params) return NEUS2B_E_INVALID;
	if (d_params_ema && !d_ema_master) return NEUS2B_E_INVALID;
	if (n < cfg->n_matrix + 4u || cfg->step == 0 || (cfg->n_matrix & 3u) || (n & 3u)) return NEUS2B_E_INVALID;
	if (((uintptr_t)d_grad_variance | (uintptr_t)d_grad_mlp | (uintptr_t)d_grad_grid | (uintptr_t)d_master | (uintptr_t)d_m | (uintptr_t)d_v | (uintptr_t)d_params |
	     (uintptr_t)d_params_ema | (uintptr_t)d_ema_master) & 15u)
		return NEUS2B_E_INVALID;
	const float lr_t = cfg->learning_rate * sqrtf(1.0f - powf(cfg->beta2, (float)cfg->step)) / (1.0f - powf(cfg->beta1, (float)cfg->step));
	const bool debias = !(cfg->flags & NEUS2B_ADAM_EMA_NO_DEBIAS);
	const float ema_old = debias ? 1.0f - powf(cfg->ema_decay, (float)(cfg->step - 1)) : 1.0f;
	const float ema_new_inv = debias ? 1.0f / (1.0f - powf(cfg->ema_decay, (float)cfg->step)) : 1.0f;
	adam_kernel<<<div_up((n + 3) / 4, 256), 256, 0, stream>>>(*cfg, lr_t, ema_old, ema_new_inv, n, d_grad_mlp, (__half*)d_grad_grid, d_grad_variance,
	                                          d_master, d_m, d_v, (__half*)d_params, (__half*)d_params_ema, d_ema_master);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_adam_step_packed(const neus2b_adam_cfg* cfg, uint64_t n, float* d_grad_mlp, uint16_t* d_grad_grid,
                                       float* d_grad_variance, float* d_state, uint16_t* d_params, uint16_t* d_params_ema,
                                       neus2b_stream_t stream) {
	if (!cfg || !d_grad_mlp || !d_grad_grid || !d_grad_variance || !d_state || !d_params) return NEUS2B_E_INVALID;
	if (n < cfg->n_matrix + 4u || cfg->step == 0 || (cfg->n_matrix & 3u) || (n & 3u)) return NEUS2B_E_INVALID;
	if (((uintptr_t)d_grad_variance | (uintptr_t)d_grad_mlp | (uintptr_t)d_grad_grid | (uintptr_t)d_state | (uintptr_t)d_params |
	     (uintptr_t)d_params_ema) & 15u)
		return NEUS2B_E_INVALID;
	const float lr_t = cfg->learning_rate * sqrtf(1.0f - powf(cfg->beta2, (float)cfg->step)) / (1.0f - powf(cfg->beta1, (float)cfg->step));
	const bool debias = !(cfg->flags & NEUS2B_ADAM_EMA_NO_DEBIAS);
	const float ema_old = debias ? 1.0f - powf(cfg->ema_decay, (float)(cfg->step - 1)) : 1.0f;
	const float ema_new_inv = debias ? 1.0f / (1.0f - powf(cfg->ema_decay, (float)cfg->step)) : 1.0f;
	adam_packed_kernel<<<kSMs * 16, 256, 0, stream>>>(*cfg, lr_t, ema_old, ema_new_inv, n, d_grad_mlp, (__half*)d_grad_grid, d_grad_variance,
	                                                  (float4*)d_state, (__half*)d_params, (__half*)d_params_ema);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

namespace {
__global__ void occ_bounds_init_kernel(int32_t* bounds) {
	if (threadIdx.x < 3) bounds[threadIdx.x] = (int32_t)NEUS2B_GRIDSIZE;
	else if (threadIdx.x < 6) bounds[threadIdx.x] = -1;
}
// one thread per byte of the finest level: cell index = Morton code
__global__ void __launch_bounds__(256) occ_bounds_kernel(const uint8_t* __restrict__ bitfield, int32_t* __restrict__ bounds) {
	const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
	int lo[3] = {(int)NEUS2B_GRIDSIZE, (int)NEUS2B_GRIDSIZE, (int)NEUS2B_GRIDSIZE}, hi[3] = {-1, -1, -1};
	if (b < kCells / 8u) {
		uint32_t bits = bitfield[b];
		while (bits) {
			const uint32_t i = b * 8u + (uint32_t)__ffs((int)bits) - 1u;
			bits &= bits - 1u;
			const int c[3] = {(int)morton3d_invert(i >> 0), (int)morton3d_invert(i >> 1), (int)morton3d_invert(i >> 2)};
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				lo[e] = min(lo[e], c[e]);
				hi[e] = max(hi[e], c[e]);
			}
		}
	}
	// warp -> CTA -> one atomic per CTA and bound (thousands of same-address atomics would serialise)
	__shared__ int s_lo[3][8], s_hi[3][8];
	const int warp = threadIdx.x >> 5;
#pragma unroll
	for (int e = 0; e < 3; ++e) {
		const int l = __reduce_min_sync(0xffffffffu, lo[e]), h = __reduce_max_sync(0xffffffffu, hi[e]);
		if ((threadIdx.x & 31) == 0) {
			s_lo[e][warp] = l;
			s_hi[e][warp] = h;
		}
	}
	__syncthreads();
	if (threadIdx.x < 3) {
		const int e = threadIdx.x;
		int l = s_lo[e][0], h = s_hi[e][0];
#pragma unroll
		for (int w = 1; w < 8; ++w) {
			l = min(l, s_lo[e][w]);
			h = max(h, s_hi[e][w]);
		}
		if (l < (int)NEUS2B_GRIDSIZE) atomicMin(&bounds[e], l);
		if (h >= 0) atomicMax(&bounds[3 + e], h);
	}
}
}  // namespace

extern "C" int neus2b_occupancy_bounds(const uint8_t* d_bitfield, int32_t* d_bounds, neus2b_stream_t stream) {
	if (!d_bitfield || !d_bounds) return NEUS2B_E_INVALID;
	occ_bounds_init_kernel<<<1, 32, 0, stream>>>(d_bounds);
	N2B_CHECK_LAUNCH();
	occ_bounds_kernel<<<div_up(kCells / 8u, 256), 256, 0, stream>>>(d_bitfield, d_bounds);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}
