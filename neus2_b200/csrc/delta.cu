// DeltaNetwork as stand-alone entry points: forward, the twelve batch sums of its backward, and its optimizer
// (the reference trains these 12 parameters with a Trainer of their own, src/testbed.cu:2311-2317, stepped next to the main
// one at src/testbed_nerf.cu:3497-3502).  The reference reduces the nine gradients with nine blocking reduce_sum calls of
// per-sample fp16 values (transform_network.h:124-158); here a sample contributes to twelve fp32 sums (dL/dx' and its outer
// product with the unmoved position), reduced in the warp and the CTA, and the 6-D backward -- linear in that outer product --
// runs once on the sums inside the optimizer kernel.
#include "common.cuh"
#include "delta.cuh"

namespace n2b {

__global__ void __launch_bounds__(256) delta_forward_kernel(const __half* __restrict__ delta, float ox, float oy, float oz, uint32_t n,
                                                            const float* __restrict__ in, float* __restrict__ out) {
	const RigidMotion m = load_rigid_motion(delta);
	const float off[3] = {ox, oy, oz};
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
		const float* c = in + (size_t)i * 7;
		float x[3] = {c[0], c[1], c[2]}, d[3] = {c[4], c[5], c[6]};
		move_sample(m.R, m.t, off, x, d);
		float* o = out + (size_t)i * 7;
		o[0] = x[0];
		o[1] = x[1];
		o[2] = x[2];
		o[3] = c[3];
		o[4] = d[0];
		o[5] = d[1];
		o[6] = d[2];
	}
}

// sums[0..2] += sum dL/dx', sums[3..11] += sum dL/dx' (x) (x + t)   (loss_vector, input_vector of common_operation.cuh:810-831)
__global__ void __launch_bounds__(256) delta_backward_kernel(const __half* __restrict__ delta, uint32_t n, const float* __restrict__ in,
                                                             const float* __restrict__ dL_dx, float* __restrict__ sums) {
	__shared__ float acc[12];
	if (threadIdx.x < 12) acc[threadIdx.x] = 0.f;
	__syncthreads();
	const float t[3] = {__half2float(delta[0]), __half2float(delta[1]), __half2float(delta[2])};
	float s[12];
#pragma unroll
	for (int k = 0; k < 12; ++k) s[k] = 0.f;
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
		const float* c = in + (size_t)i * 7;
		const float* l = dL_dx + (size_t)i * 3;
		const float v[3] = {c[0] + t[0], c[1] + t[1], c[2] + t[2]};
#pragma unroll
		for (int r = 0; r < 3; ++r) {
			s[r] += l[r];
#pragma unroll
			for (int k = 0; k < 3; ++k) s[3 + r * 3 + k] += l[r] * v[k];
		}
	}
#pragma unroll
	for (int k = 0; k < 12; ++k) {
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) s[k] += __shfl_xor_sync(0xffffffffu, s[k], o);
		if ((threadIdx.x & 31) == 0 && s[k] != 0.f) atomicAdd(&acc[k], s[k]);
	}
	__syncthreads();
	if (threadIdx.x < 12 && acc[threadIdx.x] != 0.f) atomicAdd(&sums[threadIdx.x], acc[threadIdx.x]);
}

// d normalize(x) / d x applied to a gradient (gradients_for_normalize, common_operation.cuh:68-94)
__device__ inline void normalize_bwd(const float* x, const float* g, float* out) {
	const float n = sqrtf(x[0] * x[0] + x[1] * x[1] + x[2] * x[2]);
	const float b[3] = {x[0] / n, x[1] / n, x[2] / n};
	const float gb = g[0] * b[0] + g[1] * b[1] + g[2] * b[2];
#pragma unroll
	for (int e = 0; e < 3; ++e) out[e] = (g[e] - gb * b[e]) / n;
}

// The twelve sums -> the gradient of the 12 parameters (transition: R^T sum dL/dx', common_operation.cuh:812-820; rotation:
// backward of the Gram-Schmidt construction, gradient_rotation_matrix_to_6d :96-158), then Ema o ExponentialDecay o Adam on
// them (the "globalmove" optimizer block of configs/nerf/*.json).  One thread: twelve numbers.
__global__ void delta_optimizer_kernel(neus2b_adam_cfg c, float lr_t, float ema_old, float ema_new_inv, float* __restrict__ sums,
                                       float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                       __half* __restrict__ params, __half* __restrict__ params_ema, float* __restrict__ ema_master,
                                       float* __restrict__ grad_out) {
	if (threadIdx.x != 0 || blockIdx.x != 0) return;
	float a1[3], a2[3], R[9], g[12];
#pragma unroll
	for (int e = 0; e < 3; ++e) {
		a1[e] = __half2float(params[4 + e]);
		a2[e] = __half2float(params[7 + e]);
	}
	rotation_6d_to_matrix(a1, a2, R);
	const float* L = sums;
	const float* G = sums + 3;  // G[r * 3 + k] = dL / dR(r, k)
#pragma unroll
	for (int k = 0; k < 12; ++k) g[k] = 0.f;
#pragma unroll
	for (int e = 0; e < 3; ++e) g[e] = R[0 * 3 + e] * L[0] + R[1 * 3 + e] * L[1] + R[2 * 3 + e] * L[2];
	{
		const float b1[3] = {R[0], R[3], R[6]}, b2[3] = {R[1], R[4], R[7]};
		const float dt = b1[0] * a2[0] + b1[1] * a2[1] + b1[2] * a2[2];
		const float u2[3] = {a2[0] - dt * b1[0], a2[1] - dt * b1[1], a2[2] - dt * b1[2]};
		const float g1[3] = {G[0], G[3], G[6]}, g2[3] = {G[1], G[4], G[7]}, g3[3] = {G[2], G[5], G[8]};
		// b3 = b1 x b2: dL/db1 += b2 x g3, dL/db2 += g3 x b1
		float db1[3] = {g1[0] + (b2[1] * g3[2] - b2[2] * g3[1]), g1[1] + (b2[2] * g3[0] - b2[0] * g3[2]), g1[2] + (b2[0] * g3[1] - b2[1] * g3[0])};
		const float db2[3] = {g2[0] + (g3[1] * b1[2] - g3[2] * b1[1]), g2[1] + (g3[2] * b1[0] - g3[0] * b1[2]), g2[2] + (g3[0] * b1[1] - g3[1] * b1[0])};
		float du2[3], da1[3];
		normalize_bwd(u2, db2, du2);
		const float du2b1 = du2[0] * b1[0] + du2[1] * b1[1] + du2[2] * b1[2];
#pragma unroll
		for (int e = 0; e < 3; ++e) {
			g[7 + e] = du2[e] - du2b1 * b1[e];  // u2 = a2 - (b1 . a2) b1
			db1[e] -= dt * du2[e] + du2b1 * a2[e];
		}
		normalize_bwd(a1, db1, da1);
#pragma unroll
		for (int e = 0; e < 3; ++e) g[4 + e] = da1[e];
	}
	for (int k = 0; k < 12; ++k) {
		if (grad_out) grad_out[k] = g[k];
		sums[k] = 0.f;
		if (!master) continue;
		float gk = g[k];
		if (!(fabsf(gk) <= 3.402823466e+38f)) {
			if (c.d_nonfinite) atomicAdd(c.d_nonfinite, 1u);
			continue;
		}
		gk /= c.loss_scale;
		float w = master[k];
		if (gk != 0.f || (c.flags & NEUS2B_ADAM_UPDATE_UNTOUCHED)) {  // the unused slots never move
			if (c.flags & NEUS2B_ADAM_L2_ALL) gk += c.l2_reg * w;
			const float mk = c.beta1 * m[k] + (1.0f - c.beta1) * gk, vk = c.beta2 * v[k] + (1.0f - c.beta2) * gk * gk;
			m[k] = mk;
			v[k] = vk;
			w -= lr_t * mk / (sqrtf(vk) + c.epsilon);
			master[k] = w;
		}
		params[k] = __float2half_rn(w);
		if (params_ema) {
			const float e = ((1.0f - c.ema_decay) * w + c.ema_decay * ema_master[k] * ema_old) * ema_new_inv;
			ema_master[k] = e;
			params_ema[k] = __float2half_rn(e);
		}
	}
}

}  // namespace n2b

using namespace n2b;

extern "C" int neus2b_delta_forward(const uint16_t* d_delta, const float first_frame_offset[3], uint32_t n, const float* d_coords_in,
                                    float* d_coords_out, neus2b_stream_t stream) {
	if (!d_delta || !first_frame_offset || !d_coords_in || !d_coords_out) return NEUS2B_E_INVALID;
	if (n == 0) return NEUS2B_OK;
	delta_forward_kernel<<<min(div_up(n, 256), (uint32_t)kSMs * 8u), 256, 0, stream>>>((const __half*)d_delta, first_frame_offset[0],
	                                                                                first_frame_offset[1], first_frame_offset[2], n, d_coords_in,
	                                                                                d_coords_out);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_delta_backward(const uint16_t* d_delta, uint32_t n, const float* d_coords_in, const float* d_dL_dx, float* d_sums,
                                     neus2b_stream_t stream) {
	if (!d_delta || !d_coords_in || !d_dL_dx || !d_sums) return NEUS2B_E_INVALID;
	if (n == 0) return NEUS2B_OK;
	delta_backward_kernel<<<min(div_up(n, 256), (uint32_t)kSMs * 4u), 256, 0, stream>>>((const __half*)d_delta, n, d_coords_in, d_dL_dx, d_sums);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_delta_optimizer_step(const neus2b_adam_cfg* cfg, float* d_sums, float* d_master, float* d_m, float* d_v,
                                           uint16_t* d_delta, uint16_t* d_delta_ema, float* d_ema_master, float* d_grad_out,
                                           neus2b_stream_t stream) {
	if (!d_sums || !d_delta) return NEUS2B_E_INVALID;
	neus2b_adam_cfg c{};
	float lr_t = 0.f, ema_old = 1.f, ema_new_inv = 1.f;
	if (d_master) {
		if (!cfg || !d_m || !d_v || cfg->step == 0 || (d_delta_ema && !d_ema_master)) return NEUS2B_E_INVALID;
		c = *cfg;
		lr_t = cfg->learning_rate * sqrtf(1.0f - powf(cfg->beta2, (float)cfg->step)) / (1.0f - powf(cfg->beta1, (float)cfg->step));
		if (!(cfg->flags & NEUS2B_ADAM_EMA_NO_DEBIAS)) {
			ema_old = 1.0f - powf(cfg->ema_decay, (float)(cfg->step - 1));
			ema_new_inv = 1.0f / (1.0f - powf(cfg->ema_decay, (float)cfg->step));
		}
	} else if (!d_grad_out) {
		return NEUS2B_E_INVALID;
	}
	delta_optimizer_kernel<<<1, 32, 0, stream>>>(c, lr_t, ema_old, ema_new_inv, d_sums, d_master, d_m, d_v, (__half*)d_delta, (__half*)d_delta_ema,
	                                             d_ema_master, d_grad_out);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

// accumulate_global_movement_rotation_6d_kernel (common_operation.cuh:555-589) on the host: a frame switch of a dynamic
// sequence folds the frame's learned motion into the accumulated one, R_acc <- R R_acc, t_acc <- R (t_acc + t).  The reference
// keeps both in fp16 buffers, so the results are rounded to fp16-representable values.
extern "C" int neus2b_movement_accumulate(const uint16_t h_delta[12], float rotation[9], float transition[3]) {
	if (!h_delta || !rotation || !transition) return NEUS2B_E_INVALID;
	float a1[3], a2[3], t[3], R[9], out[9], tv[3], tr[3];
	for (int e = 0; e < 3; ++e) {
		t[e] = __half2float(__ushort_as_half(h_delta[e]));
		a1[e] = __half2float(__ushort_as_half(h_delta[4 + e]));
		a2[e] = __half2float(__ushort_as_half(h_delta[7 + e]));
	}
	rotation_6d_to_matrix(a1, a2, R);
	for (int r = 0; r < 3; ++r)
		for (int k = 0; k < 3; ++k) out[r * 3 + k] = (R[r * 3] * rotation[k] + R[r * 3 + 1] * rotation[3 + k]) + R[r * 3 + 2] * rotation[6 + k];
	for (int e = 0; e < 3; ++e) tv[e] = transition[e] + t[e];
	rotate3(R, tv, tr);
	for (int k = 0; k < 9; ++k) rotation[k] = __half2float(__float2half_rn(out[k]));
	for (int e = 0; e < 3; ++e) transition[e] = __half2float(__float2half_rn(tr[e]));
	return NEUS2B_OK;
}
