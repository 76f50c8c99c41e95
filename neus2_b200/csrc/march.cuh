// Device code shared by the training-side ray march and the inference renderer: step-size and occupancy-grid helpers,
// box intersection, and the warp-per-ray march over the occupancy grid (src/testbed_nerf.cu:139-154,346-368,474-510,614-628
// of the reference).
//
// Every file that includes this header is compiled with -fmad=false: the DDA decides integer step counts from fp32
// arithmetic, so every operation is a single IEEE operation in a fixed order.
#pragma once
#include "common.cuh"

namespace n2b {

// The reference writes these with Eigen expressions: a reduction over three terms is evaluated as a0 + (a1 + a2) (the unrolled
// redux splits the range in halves), and normalized() divides every component by the root of the squared norm instead of
// multiplying by a reciprocal.  Checked against the reference's kernels running on a GPU: with these the rays and sample
// positions agree bit for bit.
__device__ __forceinline__ float sum3_eigen(float a, float b, float c) { return a + (b + c); }
__device__ __forceinline__ void normalize3_eigen(const float* v, float* out) {
	const float z = sum3_eigen(v[0] * v[0], v[1] * v[1], v[2] * v[2]);
	if (z > 0.0f) {
		const float n = sqrtf(z);
#pragma unroll
		for (int e = 0; e < 3; ++e) out[e] = v[e] / n;
	} else {
#pragma unroll
		for (int e = 0; e < 3; ++e) out[e] = v[e];
	}
}
__device__ __forceinline__ float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ float min_cone_stepsize() { return 1.73205080757f / (float)NEUS2B_STEPS; }
__device__ __forceinline__ float max_cone_stepsize() {
	return min_cone_stepsize() * (float)(1u << (NEUS2B_CASCADES - 1)) * (float)NEUS2B_STEPS / (float)NEUS2B_GRIDSIZE;
}
// calc_dt, src/testbed_nerf.cu:152
__device__ __forceinline__ float calc_dt(float t, float cone_angle) { return clampf(t * cone_angle, min_cone_stepsize(), max_cone_stepsize()); }
// warp_dt / unwarp_dt, src/testbed_nerf.cu:474-482
__device__ __forceinline__ float warp_dt(float dt) {
	const float mx = min_cone_stepsize() * (float)(1u << (NEUS2B_CASCADES - 1));
	return (dt - min_cone_stepsize()) / (mx - min_cone_stepsize());
}
__device__ __forceinline__ float unwarp_dt(float dt) {
	const float mx = min_cone_stepsize() * (float)(1u << (NEUS2B_CASCADES - 1));
	return dt * (mx - min_cone_stepsize()) + min_cone_stepsize();
}
__device__ __forceinline__ uint32_t expand_bits(uint32_t v) {
	v = (v * 0x00010001u) & 0xFF0000FFu;
	v = (v * 0x00000101u) & 0x0F00F00Fu;
	v = (v * 0x00000011u) & 0xC30C30C3u;
	v = (v * 0x00000005u) & 0x49249249u;
	return v;
}
__device__ __forceinline__ uint32_t morton3d(uint32_t x, uint32_t y, uint32_t z) {
	return expand_bits(x) | (expand_bits(y) << 1) | (expand_bits(z) << 2);
}
// mip_from_pos / mip_from_dt, src/testbed_nerf.cu:614-628
__device__ __forceinline__ int mip_from_pos(const float* p) {
	int exponent;
	const float m = fmaxf(fmaxf(fabsf(p[0] - 0.5f), fabsf(p[1] - 0.5f)), fabsf(p[2] - 0.5f));
	frexpf(m, &exponent);
	return min((int)NEUS2B_CASCADES - 1, max(0, exponent + 1));
}
__device__ __forceinline__ int mip_from_dt(float dt, const float* p) {
	const int mip = mip_from_pos(p);
	dt *= 2.f * (float)NEUS2B_GRIDSIZE;
	if (dt < 1.f) return mip;
	int exponent;
	frexpf(dt, &exponent);
	return min((int)NEUS2B_CASCADES - 1, max(exponent, mip));
}
// cascaded_grid_idx_at / density_grid_occupied_at, src/testbed_nerf.cu:484-510
__device__ __forceinline__ bool occupied_at(const float* pos, const uint8_t* __restrict__ bitfield, uint32_t mip) {
	const float mip_scale = scalbnf(1.0f, -(int)mip);
	int c[3];
#pragma unroll
	for (int d = 0; d < 3; ++d) {
		const float p = (pos[d] - 0.5f) * mip_scale + 0.5f;
		const int v = (int)(p * (float)NEUS2B_GRIDSIZE);
		c[d] = v < 0 ? 0 : (v > (int)NEUS2B_GRIDSIZE - 1 ? (int)NEUS2B_GRIDSIZE - 1 : v);
	}
	const uint32_t idx = morton3d((uint32_t)c[0], (uint32_t)c[1], (uint32_t)c[2]);
	const uint32_t cells = NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE;
	return (__ldg(bitfield + idx / 8 + (cells * mip) / 8) & (1u << (idx % 8))) != 0;
}
// distance_to_next_voxel / advance_to_next_voxel, src/testbed_nerf.cu:346-368
__device__ __forceinline__ float advance_to_next_voxel(float t, float cone_angle, const float* pos, const float* dir, const float* idir,
                                                       uint32_t res) {
	float tt[3];
#pragma unroll
	for (int d = 0; d < 3; ++d) {
		const float p = (float)res * pos[d];
		tt[d] = (floorf(p + 0.5f + 0.5f * copysignf(1.0f, dir[d])) - p) * idir[d];
	}
	const float tmin = fminf(fminf(tt[0], tt[1]), tt[2]);
	const float t_target = t + fmaxf(tmin / (float)res, 0.0f);
	do {
		t += calc_dt(t, cone_angle);
	} while (t < t_target);
	return t;
}
// BoundingBox::ray_intersect, include/neural-graphics-primitives/bounding_box.cuh:163-210
__device__ __forceinline__ void aabb_ray_intersect(const float* mn, const float* mx, const float* o, const float* d, float& tmin_out,
                                                   float& tmax_out) {
	const float big = 3.402823466e+38f;
	float tmin = (mn[0] - o[0]) / d[0], tmax = (mx[0] - o[0]) / d[0];
	if (tmin > tmax) { float t = tmin; tmin = tmax; tmax = t; }
	float tymin = (mn[1] - o[1]) / d[1], tymax = (mx[1] - o[1]) / d[1];
	if (tymin > tymax) { float t = tymin; tymin = tymax; tymax = t; }
	if (tmin > tymax || tymin > tmax) { tmin_out = tmax_out = big; return; }
	if (tymin > tmin) tmin = tymin;
	if (tymax < tmax) tmax = tymax;
	float tzmin = (mn[2] - o[2]) / d[2], tzmax = (mx[2] - o[2]) / d[2];
	if (tzmin > tzmax) { float t = tzmin; tzmin = tzmax; tzmax = t; }
	if (tmin > tzmax || tzmin > tmax) { tmin_out = tmax_out = big; return; }
	if (tzmin > tmin) tmin = tzmin;
	if (tzmax < tmax) tmax = tzmax;
	tmin_out = tmin;
	tmax_out = tmax;
}
__device__ __forceinline__ bool aabb_contains(const float* mn, const float* mx, const float* p) {
	return p[0] >= mn[0] && p[0] <= mx[0] && p[1] >= mn[1] && p[1] <= mx[1] && p[2] >= mn[2] && p[2] <= mx[2];
}
// include/neural-graphics-primitives/common_device.cuh:31-77
__device__ __forceinline__ float srgb_to_linear(float s) { return s <= 0.04045f ? s / 12.92f : powf((s + 0.055f) / 1.055f, 2.4f); }
__device__ __forceinline__ float linear_to_srgb(float l) { return l < 0.0031308f ? 12.92f * l : 1.055f * powf(l, 0.41666f) - 0.055f; }
// image_pos / read_rgba for EImageDataType::Byte, common_device.cuh:591-642
__device__ __forceinline__ void read_rgba(const neus2b_dataset& ds, uint32_t img, const float* xy, float* rgba) {
	int px = (int)(xy[0] * (float)ds.width), py = (int)(xy[1] * (float)ds.height);
	px = min(px, (int)ds.width - 1);
	py = min(py, (int)ds.height - 1);
	px = max(px, 0);
	py = max(py, 0);
	const uint32_t v = __ldg(ds.d_pixels + (size_t)img * ds.width * ds.height + (size_t)py * ds.width + px);
	if (v == 0x00FF00FFu) {
		rgba[0] = rgba[1] = rgba[2] = rgba[3] = -1.0f;
		return;
	}
	const float a = (float)(v >> 24) * (1.0f / 255.0f);
	rgba[0] = srgb_to_linear((float)(v & 0xFF) * (1.0f / 255.0f)) * a;
	rgba[1] = srgb_to_linear((float)((v >> 8) & 0xFF) * (1.0f / 255.0f)) * a;
	rgba[2] = srgb_to_linear((float)((v >> 16) & 0xFF) * (1.0f / 255.0f)) * a;
	rgba[3] = a;
}
// image_idx without the error-map CDF, src/testbed_nerf.cu:1231-1251 (32-bit wrap-around like the reference)
__device__ __forceinline__ uint32_t image_idx(uint32_t base_idx, uint32_t n_rays, uint32_t n_rays_total, uint32_t n_images) {
	return (((base_idx + n_rays_total) * n_images) / n_rays) % n_images;
}
// nerf_random_image_pos_training without CDF, src/testbed_nerf.cu:1216-1229
__device__ __forceinline__ void random_image_pos(Pcg32& rng, const neus2b_dataset& ds, bool snap, float* xy) {
	xy[0] = rng.next_float();
	xy[1] = rng.next_float();
	if (snap) {
		int px = (int)(xy[0] * (float)ds.width), py = (int)(xy[1] * (float)ds.height);
		px = max(0, min(px, (int)ds.width - 1));
		py = max(0, min(py, (int)ds.height - 1));
		xy[0] = ((float)px + 0.5f) / (float)ds.width;
		xy[1] = ((float)py + 0.5f) / (float)ds.height;
	}
}

struct RayTmp {  // 8 floats per ray
	float o[3], d[3], startt;
	uint32_t numsteps;
};

// One warp marches one ray.  The reference's loop visits a sequence of ray parameters t defined by the serial recurrence
// t <- t + calc_dt(t); at a visited t it either takes a sample (occupied cell) or jumps: it keeps adding steps until t
// reaches the far side of the empty cell (advance_to_next_voxel).  Here the 32 lanes evaluate 32 consecutive t of that
// same recurrence at once (position, containment, occupancy bit, jump target: the expensive, independent part) and
// where the serial loop would go next from there; then the warp follows that chain over the visited parameters of the
// chunk in ray order (one shuffle per visited parameter), which keeps the result identical to the serial loop: same
// visited set, same samples, same count.
constexpr uint32_t kMaskWords = 64;  // per-ray record of the count pass: one bit per ray parameter that became a sample

// Shortcut for the recurrence t <- t + dt with a constant dt.  While t stays in one binade every t is a multiple of
// u = ulp(t), so t + dt rounds to t + D where D is dt rounded to a multiple of u: the same D at every step, unless dt lies
// exactly halfway between two multiples (then the rounding depends on the parity of t).  If all 32 steps from t0 stay in
// t0's binade, the value after k steps is therefore t0 + k * D, and both the product and the sum are exact in fp32: the
// shortcut returns the very numbers the 32 serial additions produce.  Returns false when it does not apply (a binade
// boundary within the 32 steps, a tie, t0 not a positive normal number); the caller then adds serially.
__device__ __forceinline__ bool const_step_increment(float t0, float dt, float& D, float& t32) {
	const uint32_t b = __float_as_uint(t0);
	const uint32_t e = b & 0x7f800000u;
	if ((b >> 31) != 0u || e < (64u << 23) || e > (190u << 23)) return false;
	const float u = __uint_as_float(e - (23u << 23));
	D = (t0 + dt) - t0;
	t32 = t0 + 32.f * D;
	if ((__float_as_uint(t32) & 0x7f800000u) != e) return false;
	return fabsf(dt - D) * 2.f != u;
}
// t after 32 steps of the recurrence (any cone angle)
__device__ __forceinline__ float advance32(float t, float cone_angle) {
	if (cone_angle == 0.f) {
		const float dt = min_cone_stepsize();
		float D, t32;
		if (const_step_increment(t, dt, D, t32)) return t32;
#pragma unroll
		for (int k = 0; k < 32; ++k) t += dt;
		return t;
	}
#pragma unroll
	for (int k = 0; k < 32; ++k) t += calc_dt(t, cone_angle);
	return t;
}

// First half of a chunk: this lane's ray parameter (t after `lane` steps of the recurrence from the chunk start), its
// position, and the occupancy byte on its way from memory.  Nothing here depends on the visit / jump decisions of earlier
// chunks, so the next chunk's first half is issued before the current chunk is walked and the lookup latency hides there.
struct ChunkHead {
	float my_t, my_dt, t_end, pos[3];
	uint32_t mip, byte, bit;
	bool inside;
};
__device__ __forceinline__ ChunkHead chunk_head(const neus2b_train_cfg& cfg, const float* o, const float* dirn, float t_chunk,
                                                const uint8_t* __restrict__ bitfield, int lane) {
	ChunkHead h;
	const float cone_angle = cfg.cone_angle_constant;
	float t = t_chunk;
	h.my_t = t_chunk;
	h.my_dt = 0.f;
	if (cone_angle == 0.f) {
		// calc_dt(t, 0) = clamp(t * 0, min, max) = the minimum step: same values, same sequence of roundings, a quarter of the
		// dependent operations
		const float dt = min_cone_stepsize();
		h.my_dt = dt;
		float D, t32;
		if (const_step_increment(t, dt, D, t32)) {
			h.my_t = t + (float)lane * D;
			t = t32;
		} else {
#pragma unroll
			for (int k = 0; k < 32; ++k) {
				if (lane == k) h.my_t = t;
				t += dt;
			}
		}
	} else {
#pragma unroll
		for (int k = 0; k < 32; ++k) {
			const float dt = calc_dt(t, cone_angle);
			if (lane == k) {
				h.my_t = t;
				h.my_dt = dt;
			}
			t += dt;
		}
	}
	h.t_end = t;
#pragma unroll
	for (int e = 0; e < 3; ++e) h.pos[e] = o[e] + h.my_t * dirn[e];
	h.inside = aabb_contains(cfg.aabb_min, cfg.aabb_max, h.pos);
	h.mip = 0u;
	h.byte = 0u;
	h.bit = 0u;
	if (h.inside) {
		// cascaded_grid_idx_at / density_grid_occupied_at (:484-510)
		h.mip = (uint32_t)mip_from_dt(h.my_dt, h.pos);
		const float mip_scale = scalbnf(1.0f, -(int)h.mip);
		int c[3];
#pragma unroll
		for (int d = 0; d < 3; ++d) {
			const float p = (h.pos[d] - 0.5f) * mip_scale + 0.5f;
			const int v = (int)(p * (float)NEUS2B_GRIDSIZE);
			c[d] = v < 0 ? 0 : (v > (int)NEUS2B_GRIDSIZE - 1 ? (int)NEUS2B_GRIDSIZE - 1 : v);
		}
		const uint32_t idx = morton3d((uint32_t)c[0], (uint32_t)c[1], (uint32_t)c[2]);
		const uint32_t cells = NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE;
		h.byte = __ldg(bitfield + idx / 8 + (cells * h.mip) / 8);
		h.bit = 1u << (idx % 8);
	}
	return h;
}

template <bool EMIT>
__device__ __forceinline__ uint32_t march_ray(const neus2b_train_cfg& cfg, const float* o, const float* dirn, float startt,
                                              const uint8_t* __restrict__ bitfield, uint32_t limit, float* __restrict__ coords_out,
                                              int lane, uint32_t* __restrict__ masks = nullptr,
                                              uint32_t* n_chunks = nullptr, float t_lo = -3.402823466e+38f,
                                              float t_hi = 3.402823466e+38f, uint32_t slot_lo = 0u, uint32_t slot_hi = 0xffffffffu) {
	const float idir[3] = {1.0f / dirn[0], 1.0f / dirn[1], 1.0f / dirn[2]};
	float skip_until = -3.402823466e+38f;
	uint32_t j = 0;
	bool stop = false;
	// every chunk moves t forward by at least 32 minimum steps, so the ray leaves the box after a bounded number of
	// chunks; the cap only guards against non-finite inputs
	uint32_t chunk = 0;
	// [t_lo, t_hi]: the part of the ray inside the box of occupied cells (one cell of margin), when the caller knows it.
	// Chunks that end well before t_lo only advance the recurrence: nothing there can become a sample, and the chain of
	// visits restarted more than a chunk (seven cells) ahead of the box has long fallen in step with the serial loop's when it
	// gets there -- after a restart the two chains can differ only while they visit different parameters of the same
	// empty cell, and they meet at the next cell unless a parameter falls between two roundings of one boundary (1e-4).
	{
		const float cone_angle = cfg.cone_angle_constant;
		const float guard = 48.f * calc_dt(fmaxf(t_lo, 0.f), cone_angle);
		float t = startt;
		while (chunk < 8192u) {
			const float te = advance32(t, cone_angle);
			if (!(te + guard < t_lo)) break;
			if (!EMIT && masks && chunk < kMaskWords && lane == 0) masks[chunk] = 0u;
			t = te;
			++chunk;
		}
		startt = t;
	}
	ChunkHead cur = chunk_head(cfg, o, dirn, startt, bitfield, lane);
	for (; chunk < 8192u && !stop; ++chunk) {
		const ChunkHead next = chunk_head(cfg, o, dirn, cur.t_end, bitfield, lane);
		const float my_t = cur.my_t, my_dt = cur.my_dt;
		const float* pos = cur.pos;
		const bool inside = cur.inside;
		const bool occ = inside && (cur.byte & cur.bit) != 0;
		float target = 0.f;
		if (inside && !occ) {  // far side of the empty cell: distance_to_next_voxel (:346-354)
			const uint32_t res = NEUS2B_GRIDSIZE >> cur.mip;
			float tt[3];
#pragma unroll
			for (int d = 0; d < 3; ++d) {
				const float p = (float)res * pos[d];
				tt[d] = (floorf(p + 0.5f + 0.5f * copysignf(1.0f, dirn[d])) - p) * idir[d];
			}
			const float tmin = fminf(fminf(tt[0], tt[1]), tt[2]);
			target = my_t + fmaxf(tmin / (float)res, 0.0f);
		}
		const uint32_t in_mask = __ballot_sync(0xffffffffu, inside), occ_mask = __ballot_sync(0xffffffffu, occ);
		// Where the serial loop goes after visiting this lane's parameter when its cell is empty: the first later parameter
		// with t >= target (t grows along the lanes: a binary search over the lanes' my_t).
		uint32_t nxt;
		{
			uint32_t lo = (uint32_t)lane + 1u, hi = 32u;
#pragma unroll
			for (int it = 0; it < 5; ++it) {
				const uint32_t mid = (lo + hi) >> 1;
				const float tm = __shfl_sync(0xffffffffu, my_t, (int)(mid & 31u));
				if (lo < hi) {
					if (tm < target) lo = mid + 1u;
					else hi = mid;
				}
			}
			nxt = lo;
		}
		// Walk the visited parameters in ray order, identically in every lane: a run of occupied cells is taken in one go
		// (every parameter of the run is visited and becomes a sample until the sample limit), an empty cell costs one
		// shuffle for its jump.  Same visited set, same samples and the same count as the serial loop.
		uint32_t emit_mask = 0u;
		int last_empty = -1;
		const uint32_t j0 = j;
		uint32_t k = __ffs(__ballot_sync(0xffffffffu, my_t >= skip_until)) - 1u;  // first parameter not jumped over (0xffffffff: none)
		while (k < 32u) {
			if (!((in_mask >> k) & 1u) || j >= limit) {
				stop = true;
				break;
			}
			if ((occ_mask >> k) & 1u) {
				const uint32_t inv = ~(occ_mask >> k);
				const uint32_t run = inv ? (uint32_t)__ffs((int)inv) - 1u : 32u;  // ones from bit k on
				const uint32_t take = min(run, limit - j);
				emit_mask |= (take >= 32u ? 0xffffffffu : ((1u << take) - 1u)) << k;
				j += take;
				k += take;
			} else {
				last_empty = (int)k;
				k = __shfl_sync(0xffffffffu, nxt, (int)k);
			}
		}
		if (last_empty >= 0) skip_until = __shfl_sync(0xffffffffu, target, last_empty);
		const bool emit = (emit_mask >> lane) & 1u;
		const uint32_t slot = j0 + __popc(emit_mask & ((1u << lane) - 1u));
		if (!EMIT && masks && chunk < kMaskWords) {
			if (lane == 0) masks[chunk] = emit_mask;
		}
		if (EMIT && emit && slot >= slot_lo && slot < slot_hi) {  // (the window: callers that emit a ray's samples in pieces)
			float* c = coords_out + (ptrdiff_t)slot * 7;
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				c[e] = (pos[e] - cfg.aabb_min[e]) / (cfg.aabb_max[e] - cfg.aabb_min[e]);  // warp_position
				c[4 + e] = (dirn[e] + 1.f) * 0.5f;                                          // warp_direction
			}
			c[3] = warp_dt(my_dt);
		}
		if (cur.t_end > t_hi) stop = true;  // the next chunk starts past the occupied cells: no later parameter can become a sample
		cur = next;
	}
	if (n_chunks) *n_chunks = chunk;
	return j;
}

// Emit pass when the count pass recorded which ray parameters became samples: no occupancy lookups and no replay,
// only the t recurrence and the coordinate writes.
__device__ __forceinline__ void emit_from_masks(const neus2b_train_cfg& cfg, const float* o, const float* dirn, float startt,
                                                const uint32_t* __restrict__ masks, uint32_t numsteps, float* __restrict__ coords_out,
                                                int lane, uint32_t slot_lo = 0u, uint32_t slot_hi = 0xffffffffu) {
	const float cone_angle = cfg.cone_angle_constant;
	float t_chunk = startt;
	uint32_t j = 0;
	for (uint32_t chunk = 0; chunk < kMaskWords && j < numsteps; ++chunk) {
		const uint32_t m = masks[chunk];
		float t = t_chunk, my_t = t_chunk, my_dt = 0.f;
		if (cone_angle == 0.f) {  // constant step, see chunk_head
			my_dt = min_cone_stepsize();
			float D, t32;
			if (const_step_increment(t, my_dt, D, t32)) {
				my_t = t + (float)lane * D;
				t = t32;
			} else {
#pragma unroll
				for (int k = 0; k < 32; ++k) {
					if (lane == k) my_t = t;
					t += my_dt;
				}
			}
		} else {
#pragma unroll
			for (int k = 0; k < 32; ++k) {
				const float dt = calc_dt(t, cone_angle);
				if (lane == k) {
					my_t = t;
					my_dt = dt;
				}
				t += dt;
			}
		}
		t_chunk = t;
		const uint32_t slot = j + __popc(m & ((1u << lane) - 1u));
		if (((m >> lane) & 1u) && slot >= slot_lo && slot < slot_hi) {
			float* c = coords_out + (ptrdiff_t)slot * 7;
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				const float pos = o[e] + my_t * dirn[e];
				c[e] = (pos - cfg.aabb_min[e]) / (cfg.aabb_max[e] - cfg.aabb_min[e]);
				c[4 + e] = (dirn[e] + 1.f) * 0.5f;
			}
			c[3] = warp_dt(my_dt);
		}
		j += __popc(m);
	}
}

// Box around the occupied cells of the finest occupancy level, one cell of margin: a ray that misses it cannot take a
// sample, whatever the march would visit, and is not marched (most rays of a converged scene look past the object).
struct CullBox {
	float mn[3], mx[3];
	bool on, nothing;
};
__device__ __forceinline__ CullBox cull_box(const int32_t* __restrict__ occ_bounds) {
	CullBox c;
	c.on = occ_bounds != nullptr;
	c.nothing = false;
#pragma unroll
	for (int e = 0; e < 3; ++e) {
		const int lo = c.on ? occ_bounds[e] : 0, hi = c.on ? occ_bounds[3 + e] : (int)NEUS2B_GRIDSIZE - 1;
		c.nothing = c.nothing || lo > hi;  // nothing occupied
		c.mn[e] = (float)(lo - 1) / (float)NEUS2B_GRIDSIZE;
		c.mx[e] = (float)(hi + 2) / (float)NEUS2B_GRIDSIZE;
	}
	return c;
}
// may the ray take a sample, and between which ray parameters
__device__ __forceinline__ bool cull_ray(const CullBox& c, const float* o, const float* dirn, float& t_lo, float& t_hi) {
	t_lo = -3.402823466e+38f;
	t_hi = 3.402823466e+38f;
	if (!c.on) return true;
	if (c.nothing) return false;
	float c0, c1;
	aabb_ray_intersect(c.mn, c.mx, o, dirn, c0, c1);
	if (c0 >= 3.0e38f || c1 < 0.0f) return false;
	if (c0 == c0 && c1 == c1) {  // (a NaN from a zero direction component keeps the whole ray)
		t_lo = c0;
		t_hi = c1;
	}
	return true;
}

struct NeusSample {
	float alpha, p_div_c, inv_s, iter_cos, true_cos, dt, next_sdf;
	float rgb[3], nrm[3];
};
__device__ __forceinline__ float logisticf(float x) { return 1.0f / (1.0f + __expf(-x)); }

// NeuS alpha of one sample (src/testbed_nerf.cu:1568-1606 == :1779-1805)
__device__ __forceinline__ void neus_sample(const __half* o, float dt_warped, const float* dir, float anneal, NeusSample& s) {
#pragma unroll
	for (int e = 0; e < 3; ++e) s.rgb[e] = logisticf(__half2float(o[e]));
	s.dt = unwarp_dt(dt_warped);
	s.inv_s = __expf(__half2float(__hmul(__float2half_rn(10.0f), o[7])));
	const float sdf = __half2float(o[3]);
#pragma unroll
	for (int e = 0; e < 3; ++e) s.nrm[e] = __half2float(o[4 + e]);
	s.true_cos = dir[0] * s.nrm[0] + dir[1] * s.nrm[1] + dir[2] * s.nrm[2];
	// The reference writes these lines with double literals (0.5, 1.0): the intermediates are fp64 and each line rounds to
	// fp32 once (src/testbed_nerf.cu:1594-1598).  r1 is rounded where it is passed to activation_function(float), the
	// product with the annealing ratio is a float product, the sum and the two sdf estimates are fp64 sums.
	const float r1 = (float)((double)(-s.true_cos) * 0.5 + 0.5), r2 = -s.true_cos;
	const float relu2a = fmaxf(r2, 0.f) * anneal;
	s.iter_cos = (float)(-((double)fmaxf(r1, 0.f) * (1.0 - (double)anneal) + (double)relu2a));
	const float half_step = s.iter_cos * s.dt;  // float product, then * 0.5 in fp64 (exact)
	s.next_sdf = (float)((double)sdf + (double)half_step * 0.5);
	const float prev_sdf = (float)((double)sdf - (double)half_step * 0.5);
	const float next_cdf = logisticf(s.next_sdf * s.inv_s), prev_cdf = logisticf(prev_sdf * s.inv_s);
	s.p_div_c = (prev_cdf - next_cdf + 1e-5f) / (prev_cdf + 1e-5f);
	s.alpha = clampf(s.p_div_c, 0.0f, 1.0f);
}

__device__ __forceinline__ void load_out16(const __half* src, __half* dst) {
	const uint4* p = reinterpret_cast<const uint4*>(src);
	reinterpret_cast<uint4*>(dst)[0] = __ldg(p);
	reinterpret_cast<uint4*>(dst)[1] = __ldg(p + 1);
}

// Exclusive prefix sum of n (<= 2^20) 64-bit keys in place, n read on the device when d_n is given; the total goes to
// data[n_max], data[n_max + 1 .. n_max + 1023] is scratch and data[n_max + 512] must be zero before the launch (it is left
// at zero).
int launch_scan(uint32_t n_max, const uint32_t* d_n, uint64_t* data, cudaStream_t stream);

}  // namespace n2b
