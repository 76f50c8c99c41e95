// Inference renderer: camera rays through the occupancy grid, the network on every sample, NeuS alpha compositing front to
// back, blend into the frame buffer (NerfTracer::init_rays_from_camera / trace and Testbed::render_nerf,
// src/testbed_nerf.cu:787-1171, 2147-2332, 2398-2601, 2671-2812 of the reference; accumulate / tonemap,
// src/render_buffer.cu:217-259, 474-500).
//
// The reference marches in rounds: up to 8 steps for every live ray, one network call, one compositing kernel, one
// compaction of the live rays, and a blocking read of the live-ray count on the host -- about a hundred rounds and as many
// host round trips per frame.  Here a frame is: one pass that builds every pixel's ray and counts the samples of its whole
// march, a prefix sum that gives every ray its range, and then, per window of max_samples consecutive samples, one pass
// that writes the sample coordinates, one network call and one compositing pass that carries each ray's colour and
// transmittance from window to window.  A ray's samples are the ones the reference's rounds would take (same recurrence
// of ray parameters, same occupancy tests) until its opacity passes 1 - min_transmittance; the samples behind that
// point are evaluated and then ignored, which costs less than the round trips they replace.  The host reads one number
// per band of rows (the band's sample count, to know how many windows to launch).
//
// Compiled with -fmad=false like the training-side march (see march.cuh).
#include "common.cuh"
#include "march.cuh"
#include "delta.cuh"

namespace n2b {

// ---- low-discrepancy jitter of the first ray parameter (include/neural-graphics-primitives/random_val.cuh:235-290):
// hash-based Owen scrambling of the Sobol sequence (Burley 2020, "Practical Hash-based Owen Scrambling", using the
// Laine-Karras permutation).  Only dimension 0 is needed on the device, where the Sobol point of an index is its bit
// reversal.
__device__ __forceinline__ uint32_t laine_karras(uint32_t x, uint32_t seed) {
	x += seed;
	x ^= x * 0x6c50b47cu;
	x ^= x * 0xb82f1e52u;
	x ^= x * 0xc7afe638u;
	x ^= x * 0x8d22f6e6u;
	return x;
}
__device__ __forceinline__ uint32_t owen_scramble(uint32_t x, uint32_t seed) { return __brev(laine_karras(__brev(x), seed)); }
__device__ __forceinline__ float ld_random_val(uint32_t index, uint32_t seed) {
	index = owen_scramble(index, seed);
	const uint32_t seed0 = seed ^ (0u + (seed << 6) + (seed >> 2));  // hash_combine(seed, dim = 0)
	return (float)owen_scramble(__brev(index), seed0) * 2.3283064365386963e-10f;
}

struct RenderState {  // 8 words per ray
	float rgba[4], depth, max_weight;
	uint32_t done, pad;
};

__device__ __forceinline__ neus2b_train_cfg march_cfg(const neus2b_render_cfg& rc) {
	neus2b_train_cfg c = {};
#pragma unroll
	for (int e = 0; e < 3; ++e) {
		c.aabb_min[e] = rc.aabb_min[e];
		c.aabb_max[e] = rc.aabb_max[e];
	}
	c.cone_angle_constant = rc.cone_angle_constant;
	return c;
}

// init_rays_with_payload_kernel_nerf (:2207-2332) + the jitter of advance_pos_nerf (:787-836), pinhole camera without
// depth of field, distortion, environment map or rolling shutter.  One thread per pixel of the band of rows [y0, y0 + rows).
__global__ void __launch_bounds__(256) render_setup_kernel(neus2b_render_cfg rc, uint32_t y0, uint32_t n_rays, RayTmp* __restrict__ tmp,
                                                           uint64_t* __restrict__ scan_in, RenderState* __restrict__ state,
                                                           float* __restrict__ depth_buffer, const int32_t* __restrict__ occ_bounds,
                                                           uint32_t* __restrict__ hit_list, uint32_t* __restrict__ counters) {
	if (blockIdx.x == 0 && threadIdx.x == 0) scan_in[n_rays + 512] = 0ull;  // the scan's ticket counter
	const CullBox box = cull_box(occ_bounds);
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_rays; i += gridDim.x * blockDim.x) {
		const uint32_t x = i % rc.width, y = y0 + i / rc.width;
		const uint32_t idx = x + rc.width * y;
		RayTmp r;
		r.numsteps = 0;
		r.startt = 0.f;
		// pixel_to_ray (common_device.cuh:246-300)
		const float u = ((float)x + rc.pixel_offset[0]) / (float)rc.width, v = ((float)y + rc.pixel_offset[1]) / (float)rc.height;
		const float dl[3] = {(u - rc.screen_center[0]) * (float)rc.width / rc.focal_length[0],
		                     (v - rc.screen_center[1]) * (float)rc.height / rc.focal_length[1], 1.0f};
		float d[3];
#pragma unroll
		for (int e = 0; e < 3; ++e) {
			r.o[e] = rc.camera[9 + e];
			d[e] = sum3_eigen(rc.camera[0 + e] * dl[0], rc.camera[3 + e] * dl[1], rc.camera[6 + e] * dl[2]);
		}
		normalize3_eigen(d, r.d);
		if (rc.use_global_movement) {  // :2286-2296
			float o2[3], q[3], dq[3];
#pragma unroll
			for (int e = 0; e < 3; ++e) o2[e] = r.o[e] - rc.first_frame_offset[e];
			rotate3(rc.rotation, o2, q);
			rotate3(rc.rotation, r.d, dq);
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				r.o[e] = q[e] + rc.transition[e];
				r.d[e] = dq[e];
			}
		}
		depth_buffer[idx] = 1e10f;
		float tmin, tmax;
		aabb_ray_intersect(rc.aabb_min, rc.aabb_max, r.o, r.d, tmin, tmax);
		float t = fmaxf(tmin, 0.2f) + 1e-6f;  // NERF_RENDERING_NEAR_DISTANCE (:47, :2303)
		const float p0[3] = {r.o[0] + r.d[0] * t, r.o[1] + r.d[1] * t, r.o[2] + r.d[2] * t};
		bool alive = aabb_contains(rc.aabb_min, rc.aabb_max, p0);
		if (alive) {
			t += ld_random_val(rc.sample_index, idx * 786433u) * calc_dt(t, rc.cone_angle_constant);  // (:816-818)
			float t_lo, t_hi;
			alive = cull_ray(box, r.o, r.d, t_lo, t_hi);
		}
		r.startt = t;
		tmp[i] = r;
		scan_in[i] = 0ull;
		RenderState s;
		s.rgba[0] = s.rgba[1] = s.rgba[2] = s.rgba[3] = 0.f;
		s.depth = 0.f;
		s.max_weight = 0.f;
		s.done = 0u;
		s.pad = 0u;
		state[i] = s;
		if (alive) hit_list[atomicAdd(&counters[6], 1u)] = i;
	}
}

// The whole march of one listed ray, counted: advance_pos_nerf's walk to the first occupied cell followed by the steps of
// generate_next_nerf_network_inputs (:867-924) over all rounds.  One warp per ray.
__global__ void __launch_bounds__(128) render_count_kernel(neus2b_render_cfg rc, uint32_t limit, const uint8_t* __restrict__ bitfield,
                                                           RayTmp* __restrict__ tmp, uint64_t* __restrict__ scan_in,
                                                           const int32_t* __restrict__ occ_bounds, const uint32_t* __restrict__ hit_list,
                                                           const uint32_t* __restrict__ counters, uint32_t* __restrict__ masks) {
	const int lane = threadIdx.x & 31;
	const neus2b_train_cfg cfg = march_cfg(rc);
	const CullBox box = cull_box(occ_bounds);
	const uint32_t n_hit = counters[6];
	const uint32_t warps = gridDim.x * (blockDim.x >> 5);
	for (uint32_t h = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); h < n_hit; h += warps) {
		const uint32_t i = hit_list[h];
		const RayTmp r = tmp[i];
		float t_lo, t_hi;
		(void)cull_ray(box, r.o, r.d, t_lo, t_hi);
		uint32_t n_chunks = 0;
		const uint32_t n = march_ray<false>(cfg, r.o, r.d, r.startt, bitfield, limit, nullptr, lane,
		                                    masks ? masks + (size_t)i * kMaskWords : nullptr, &n_chunks, t_lo, t_hi);
		if (lane == 0) {
			scan_in[i] = (uint64_t)n;
			// (top bit: the mask record does not cover this ray, the emit pass marches it again)
			tmp[i].numsteps = n | (n_chunks > kMaskWords ? 0x80000000u : 0u);
		}
	}
}

// Coordinates of the samples whose index over the band falls into the window [s0, s0 + window).
__global__ void __launch_bounds__(128) render_emit_kernel(neus2b_render_cfg rc, uint32_t n_rays, uint32_t s0, uint32_t window,
                                                          const uint8_t* __restrict__ bitfield, const RayTmp* __restrict__ tmp,
                                                          const uint64_t* __restrict__ scan, const int32_t* __restrict__ occ_bounds,
                                                          const uint32_t* __restrict__ hit_list, uint32_t* __restrict__ counters,
                                                          float* __restrict__ coords, const uint32_t* __restrict__ masks) {
	const int lane = threadIdx.x & 31;
	const neus2b_train_cfg cfg = march_cfg(rc);
	const CullBox box = cull_box(occ_bounds);
	const uint32_t total = (uint32_t)scan[n_rays];
	if (blockIdx.x == 0 && threadIdx.x == 0) counters[2] = total > s0 ? min(total - s0, window) : 0u;  // samples of this window
	const uint32_t n_hit = counters[6];
	const uint32_t warps = gridDim.x * (blockDim.x >> 5);
	for (uint32_t h = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); h < n_hit; h += warps) {
		const uint32_t i = hit_list[h];
		RayTmp r = tmp[i];
		const bool long_ray = (r.numsteps & 0x80000000u) != 0;
		r.numsteps &= 0x7fffffffu;
		const uint32_t base = (uint32_t)scan[i];
		if (r.numsteps == 0 || base + r.numsteps <= s0 || base >= s0 + window) continue;
		const uint32_t lo = s0 > base ? s0 - base : 0u, hi = min(r.numsteps, s0 + window - base);
		float* out = coords + ((ptrdiff_t)base - (ptrdiff_t)s0) * 7;
		if (masks && !long_ray) {
			emit_from_masks(cfg, r.o, r.d, r.startt, masks + (size_t)i * kMaskWords, hi, out, lane, lo, hi);
			continue;
		}
		float t_lo, t_hi;
		(void)cull_ray(box, r.o, r.d, t_lo, t_hi);
		march_ray<true>(cfg, r.o, r.d, r.startt, bitfield, hi, out, lane, nullptr, nullptr, t_lo, t_hi, lo, hi);
	}
}

// composite_kernel_nerf (:926-1171), ERenderMode::Shade, for the part of every ray that lies in the window; one thread
// per listed ray, samples front to back like the reference's loop.
__global__ void __launch_bounds__(128) render_composite_kernel(neus2b_render_cfg rc, uint32_t s0, uint32_t window,
                                                               const RayTmp* __restrict__ tmp, const uint64_t* __restrict__ scan,
                                                               const uint32_t* __restrict__ hit_list, const uint32_t* __restrict__ counters,
                                                               const float* __restrict__ coords, const __half* __restrict__ out,
                                                               RenderState* __restrict__ state) {
	const uint32_t n_hit = counters[6];
	const float cam_fwd[3] = {rc.camera[6], rc.camera[7], rc.camera[8]};
	const float cam_pos[3] = {rc.camera[9], rc.camera[10], rc.camera[11]};
	for (uint32_t h = blockIdx.x * blockDim.x + threadIdx.x; h < n_hit; h += gridDim.x * blockDim.x) {
		const uint32_t i = hit_list[h];
		const uint32_t n = tmp[i].numsteps & 0x7fffffffu, base = (uint32_t)scan[i];
		if (n == 0 || base + n <= s0 || base >= s0 + window) continue;
		RenderState s = state[i];
		if (s.done) continue;
		const uint32_t lo = s0 > base ? s0 - base : 0u, hi = min(n, s0 + window - base);
		// the next sample's rows are on their way while this one is composited (the loop is a chain of dependent steps)
		const size_t k0 = (size_t)(base + lo - s0);
		uint4 nx0 = __ldg(reinterpret_cast<const uint4*>(out + k0 * 16)), nx1 = __ldg(reinterpret_cast<const uint4*>(out + k0 * 16) + 1);
		float ndt = __ldg(coords + k0 * 7 + 3);
		for (uint32_t j = lo; j < hi; ++j) {
			const size_t k = (size_t)(base + j - s0);
			__half o[16];
			reinterpret_cast<uint4*>(o)[0] = nx0;
			reinterpret_cast<uint4*>(o)[1] = nx1;
			const float dt_warped = ndt;
			if (j + 1 < hi) {
				nx0 = __ldg(reinterpret_cast<const uint4*>(out + (k + 1) * 16));
				nx1 = __ldg(reinterpret_cast<const uint4*>(out + (k + 1) * 16) + 1);
				ndt = __ldg(coords + (k + 1) * 7 + 3);
			}
			const float* c = coords + k * 7;
			// BENT_DIR (:999-1002): the direction the network saw, renormalised
			float dir[3];
			{
				const float dd[3] = {__half2float(o[8]) * 2.f - 1.f, __half2float(o[9]) * 2.f - 1.f, __half2float(o[10]) * 2.f - 1.f};
				const float nn = sqrtf(dd[0] * dd[0] + dd[1] * dd[1] + dd[2] * dd[2]);
#pragma unroll
				for (int e = 0; e < 3; ++e) dir[e] = dd[e] / nn;
			}
			NeusSample ns;
			neus_sample(o, dt_warped, dir, rc.cos_anneal_ratio, ns);
			const float T = 1.f - s.rgba[3];
			const float weight = ns.alpha * T;
#pragma unroll
			for (int e = 0; e < 3; ++e) s.rgba[e] += ns.rgb[e] * weight;
			s.rgba[3] += weight;
			if (weight > s.max_weight) {
				s.max_weight = weight;
				float dp = 0.f;
#pragma unroll
				for (int e = 0; e < 3; ++e) {
					const float pos = __ldg(c + e) * (rc.aabb_max[e] - rc.aabb_min[e]) + rc.aabb_min[e];  // unwarp_position
					dp += cam_fwd[e] * (pos - cam_pos[e]);
				}
				s.depth = dp;
			}
			if (s.rgba[3] > 1.0f - rc.min_transmittance) {
				const float w = s.rgba[3];
#pragma unroll
				for (int e = 0; e < 4; ++e) s.rgba[e] /= w;
				s.done = 1u;
				break;
			}
		}
		state[i] = s;
	}
}

// shade_kernel_nerf (:2147-2180) for the rays that compact_kernel_nerf (:2182-2205) would have kept (opacity > 0.001).
__global__ void __launch_bounds__(256) render_shade_kernel(neus2b_render_cfg rc, uint32_t y0, const uint32_t* __restrict__ hit_list,
                                                           const uint32_t* __restrict__ counters, const RenderState* __restrict__ state,
                                                           float* __restrict__ frame, float* __restrict__ depth_buffer) {
	const uint32_t n_hit = counters[6];
	for (uint32_t h = blockIdx.x * blockDim.x + threadIdx.x; h < n_hit; h += gridDim.x * blockDim.x) {
		const uint32_t i = hit_list[h];
		const RenderState s = state[i];
		if (!(s.rgba[3] > 0.001f)) continue;
		const uint32_t idx = y0 * rc.width + i;
		float4 tmp = make_float4(s.rgba[0], s.rgba[1], s.rgba[2], s.rgba[3]);
		if (!rc.linear_colors) {
			tmp.x = srgb_to_linear(tmp.x);
			tmp.y = srgb_to_linear(tmp.y);
			tmp.z = srgb_to_linear(tmp.z);
		}
		float4* fb = reinterpret_cast<float4*>(frame) + idx;
		const float4 old = *fb;
		const float k = 1.0f - tmp.w;
		*fb = make_float4(tmp.x + old.x * k, tmp.y + old.y * k, tmp.z + old.z * k, tmp.w + old.w * k);
		if (tmp.w > 0.2f) depth_buffer[idx] = s.depth;
	}
}

// accumulate_kernel, EColorSpace::Linear (src/render_buffer.cu:217-259): running mean over the samples per pixel
__global__ void render_accumulate_kernel(uint32_t n, const float4* __restrict__ frame, float4* __restrict__ acc, float sample_count) {
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
		const float4 c = frame[i];
		float4 t = sample_count > 0.f ? acc[i] : make_float4(0.f, 0.f, 0.f, 0.f);
		t.x = (t.x * sample_count + c.x) / (sample_count + 1.f);
		t.y = (t.y * sample_count + c.y) / (sample_count + 1.f);
		t.z = (t.z * sample_count + c.z) / (sample_count + 1.f);
		t.w = (t.w * sample_count + c.w) / (sample_count + 1.f);
		acc[i] = t;
	}
}

// tonemap_kernel (src/render_buffer.cu:474-500) with the identity curve and a linear working space
__global__ void render_tonemap_kernel(uint32_t n, const float4* __restrict__ acc, float exposure_scale, float4 background, int to_srgb,
                                      float4* __restrict__ outp) {
	background.x = srgb_to_linear(background.x);
	background.y = srgb_to_linear(background.y);
	background.z = srgb_to_linear(background.z);
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
		float4 c = acc[i];
		const float weight = (1.f - c.w) * background.w;
		c.x += background.x * weight;
		c.y += background.y * weight;
		c.z += background.z * weight;
		c.w += weight;
		c.x *= exposure_scale;
		c.y *= exposure_scale;
		c.z *= exposure_scale;
		if (to_srgb) {
			c.x = linear_to_srgb(c.x);
			c.y = linear_to_srgb(c.y);
			c.z = linear_to_srgb(c.z);
		}
		outp[i] = c;
	}
}

}  // namespace n2b

using namespace n2b;

extern "C" int neus2b_render_frame(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, const neus2b_render_cfg* cfg,
                                   const uint8_t* d_bitfield, neus2b_render_workspace* ws, float* d_frame, float* d_depth,
                                   uint64_t* h_n_samples, neus2b_stream_t stream_) {
	cudaStream_t stream = (cudaStream_t)stream_;
	if (!desc || !d_params || !cfg || !d_bitfield || !ws || !d_frame || !d_depth) return NEUS2B_E_INVALID;
	if (!ws->d_ray_tmp || !ws->d_scan_tmp || !ws->d_state || !ws->d_hit_list || !ws->d_coords || !ws->d_out || !ws->d_counters)
		return NEUS2B_E_INVALID;
	if (cfg->width == 0 || cfg->height == 0) return NEUS2B_OK;
	if (ws->max_samples == 0 || (ws->max_samples & 127u) != 0) return NEUS2B_E_INVALID;
	const uint32_t band_cap = ws->max_rays < (1u << 20) ? ws->max_rays : (1u << 20);
	if (cfg->width > band_cap) return NEUS2B_E_TOO_LARGE;
	if ((uint64_t)cfg->width * cfg->height > 0xffffffffull) return NEUS2B_E_TOO_LARGE;
	const uint32_t limit = cfg->max_steps ? cfg->max_steps : 10000u;
	const uint32_t rows_per_band = band_cap / cfg->width;
	uint64_t n_samples = 0;
	for (uint32_t y0 = 0; y0 < cfg->height; y0 += rows_per_band) {
		const uint32_t rows = cfg->height - y0 < rows_per_band ? cfg->height - y0 : rows_per_band;
		const uint32_t n_rays = rows * cfg->width;
		N2B_CHECK_CUDA(cudaMemsetAsync(ws->d_counters, 0, 8 * sizeof(uint32_t), stream));
		render_setup_kernel<<<min(div_up(n_rays, 256), (uint32_t)kSMs * 8u), 256, 0, stream>>>(
		    *cfg, y0, n_rays, (RayTmp*)ws->d_ray_tmp, ws->d_scan_tmp, (RenderState*)ws->d_state, d_depth, ws->d_occupied_bounds, ws->d_hit_list,
		    ws->d_counters);
		N2B_CHECK_LAUNCH();
		const uint32_t ray_ctas = min(div_up(n_rays, 4), (uint32_t)kSMs * 16u);
		render_count_kernel<<<ray_ctas, 128, 0, stream>>>(*cfg, limit, d_bitfield, (RayTmp*)ws->d_ray_tmp, ws->d_scan_tmp, ws->d_occupied_bounds,
		                                                 ws->d_hit_list, ws->d_counters, ws->d_march_masks);
		N2B_CHECK_LAUNCH();
		{
			const int src = launch_scan(n_rays, nullptr, ws->d_scan_tmp, stream);
			if (src) return src;
		}
		// the one read per band: how many windows of max_samples the band's samples fill
		uint64_t total = 0;
		N2B_CHECK_CUDA(cudaMemcpyAsync(&total, ws->d_scan_tmp + n_rays, sizeof(uint64_t), cudaMemcpyDeviceToHost, stream));
		N2B_CHECK_CUDA(cudaStreamSynchronize(stream));
		if (total > 0xffffffffull) return NEUS2B_E_TOO_LARGE;
		n_samples += total;
		for (uint64_t s0 = 0; s0 < total; s0 += ws->max_samples) {
			render_emit_kernel<<<ray_ctas, 128, 0, stream>>>(*cfg, n_rays, (uint32_t)s0, ws->max_samples, d_bitfield, (const RayTmp*)ws->d_ray_tmp,
			                                                ws->d_scan_tmp, ws->d_occupied_bounds, ws->d_hit_list, ws->d_counters, ws->d_coords,
			                                                ws->d_march_masks);
			N2B_CHECK_LAUNCH();
			neus2b_motion motion{};
			motion.d_delta = cfg->d_delta;
			for (int e = 0; e < 3; ++e) motion.first_frame_offset[e] = cfg->first_frame_offset[e];
			const int rc = neus2b_neus_forward_moved(desc, d_params, sdf_bias, ws->max_samples, ws->d_counters + 2, ws->d_coords,
			                                         cfg->d_delta ? &motion : nullptr, ws->d_out, stream_);
			if (rc != NEUS2B_OK) return rc;
			render_composite_kernel<<<min(div_up(n_rays, 128), (uint32_t)kSMs * 16u), 128, 0, stream>>>(
			    *cfg, (uint32_t)s0, ws->max_samples, (const RayTmp*)ws->d_ray_tmp, ws->d_scan_tmp, ws->d_hit_list, ws->d_counters, ws->d_coords,
			    (const __half*)ws->d_out, (RenderState*)ws->d_state);
			N2B_CHECK_LAUNCH();
		}
		render_shade_kernel<<<min(div_up(n_rays, 256), (uint32_t)kSMs * 8u), 256, 0, stream>>>(*cfg, y0, ws->d_hit_list, ws->d_counters,
		                                                                                    (const RenderState*)ws->d_state, d_frame, d_depth);
		N2B_CHECK_LAUNCH();
	}
	if (h_n_samples) *h_n_samples = n_samples;
	return NEUS2B_OK;
}

extern "C" int neus2b_render_accumulate(uint32_t n_pixels, const float* d_frame, float* d_accumulate, uint32_t sample_count,
                                        neus2b_stream_t stream) {
	if (!d_frame || !d_accumulate) return NEUS2B_E_INVALID;
	if (n_pixels == 0) return NEUS2B_OK;
	render_accumulate_kernel<<<min(div_up(n_pixels, 256), (uint32_t)kSMs * 8u), 256, 0, (cudaStream_t)stream>>>(
	    n_pixels, (const float4*)d_frame, (float4*)d_accumulate, (float)sample_count);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_render_tonemap(uint32_t n_pixels, const float* d_accumulate, float exposure, const float background[4], int to_srgb,
                                     float* d_out, neus2b_stream_t stream) {
	if (!d_accumulate || !d_out || !background) return NEUS2B_E_INVALID;
	if (n_pixels == 0) return NEUS2B_OK;
	render_tonemap_kernel<<<min(div_up(n_pixels, 256), (uint32_t)kSMs * 8u), 256, 0, (cudaStream_t)stream>>>(
	    n_pixels, (const float4*)d_accumulate, exp2f(exposure), make_float4(background[0], background[1], background[2], background[3]),
	    to_srgb, (float4*)d_out);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

// Host side of the pixel jitter: two dimensions of the scrambled Sobol sequence.  Direction numbers: 2^(31-k) in
// dimension 0; in dimension 1 (primitive polynomial x + 1) v_k = v_(k-1) xor (v_(k-1) >> 1).
static uint32_t host_reverse_bits(uint32_t x) {
	x = ((x & 0xaaaaaaaau) >> 1) | ((x & 0x55555555u) << 1);
	x = ((x & 0xccccccccu) >> 2) | ((x & 0x33333333u) << 2);
	x = ((x & 0xf0f0f0f0u) >> 4) | ((x & 0x0f0f0f0fu) << 4);
	x = ((x & 0xff00ff00u) >> 8) | ((x & 0x00ff00ffu) << 8);
	return (x >> 16) | (x << 16);
}
static uint32_t host_owen_scramble(uint32_t x, uint32_t seed) {
	x = host_reverse_bits(x) + seed;
	x ^= x * 0x6c50b47cu;
	x ^= x * 0xb82f1e52u;
	x ^= x * 0xc7afe638u;
	x ^= x * 0x8d22f6e6u;
	return host_reverse_bits(x);
}
static void host_ld_random_val_2d(uint32_t index, uint32_t seed, float out[2]) {
	index = host_owen_scramble(index, seed);
	for (uint32_t dim = 0; dim < 2; ++dim) {
		uint32_t v = 0x80000000u, x = 0;
		for (uint32_t bit = 0; bit < 32; ++bit) {
			if ((index >> bit) & 1u) x ^= v;
			v = dim == 0 ? v >> 1 : v ^ (v >> 1);
		}
		const uint32_t sd = seed ^ (dim + (seed << 6) + (seed >> 2));  // hash_combine
		out[dim] = (float)host_owen_scramble(x, sd) * 2.3283064365386963e-10f;
	}
}
extern "C" void neus2b_ld_random_pixel_offset(uint32_t spp, float out_xy[2]) {
	if (!out_xy) return;
	float a[2], b[2];
	host_ld_random_val_2d(0u, 0xdeadbeefu, a);
	host_ld_random_val_2d(spp, 0xdeadbeefu, b);
	for (int e = 0; e < 2; ++e) {
		const float o = 0.5f - a[e] + b[e];
		out_xy[e] = o - floorf(o);
	}
}
