// Pieces shared by the two implementations of the fused NeuS graph kernels (mma.sync warp tiles, tcgen05 CTA tiles).
#pragma once
#include "common.cuh"

namespace n2b {

enum { MODE_FWD = 0, MODE_TRAIN = 1, MODE_SDF = 2 };

struct NeusArgs {
	GridLevels lv;
	const __half* params;
	uint32_t grid_entries;  // total grid entries (2 fp16 each)
	float sdf_bias;
	uint32_t n;
	const uint32_t* d_n;
	const float* coords;
	uint32_t coord_stride;  // floats per sample (7 for NerfCoordinate, >=3 for positions only)
	uint32_t dir_offset;
	__half* out;
	const __half* dL_dout;
	float batch_size;
	float* grad_mlp;
	__half* grad_grid;
	float* grad_var;
	__half* sdf_out;
	// dynamic sequences: the frame's learned rigid motion (DeltaNetwork, nerf_network.h:149-169) is applied to every sample
	// before anything else when delta != nullptr; training adds the twelve sums of its backward to delta_sums when given
	const __half* delta;
	float first_frame_offset[3];
	float* delta_sums;
};

// original column of the SDF-net input for internal column k
__device__ __forceinline__ int sdf_orig_col(int k) { return k < 32 ? 3 + k : (k < 35 ? k - 32 : k); }

// Per (sample, level) geometry, factored so that a corner costs a handful of integer / fp32 operations:
// index = combine(hx[bx], hy[by], hz[bz]), weight = ax[bx] * ay[by] * az[bz].
struct LevelGeom {
	uint32_t hx[2], hy[2], hz[2];
	float ax[2], ay[2], az[2];
	uint32_t mask_or_size, offset;
	bool hashed;
};

// The rare part of level_geom for a dense level: one axis of a cell outside the lattice, both corners, reduced modulo the
// level's size over the integers.  Kept out of line (and free of pointers, so that the caller's arrays stay in registers):
// inlined, its 64-bit divisions sit in the middle of the gather's unrolled loads and cost the fused kernels 5-8 % on samples
// that never take it.
static __device__ __noinline__ uint2 reduce_outside_axis(uint32_t c0, uint32_t stride, uint32_t size_u) {
	const long long size = size_u;
	const long long v0 = ((long long)(int32_t)c0 * stride) % size, v1 = (((long long)(int32_t)c0 + 1) * stride) % size;
	return make_uint2((uint32_t)(v0 < 0 ? v0 + size : v0), (uint32_t)(v1 < 0 ? v1 + size : v1));
}

__device__ __forceinline__ LevelGeom level_geom(const GridLevels& lv, uint32_t l, const float* x) {
	LevelGeom g;
	const Cell c = level_cell(lv, l, x);
	g.ax[0] = 1.0f - c.f[0];
	g.ax[1] = c.f[0];
	g.ay[0] = 1.0f - c.f[1];
	g.ay[1] = c.f[1];
	g.az[0] = 1.0f - c.f[2];
	g.az[1] = c.f[2];
	g.hashed = lv.hashed[l] != 0;
	g.offset = lv.offset[l];
	if (g.hashed) {
		g.hx[0] = c.c0[0];
		g.hx[1] = c.c0[0] + 1u;
		g.hy[0] = c.c0[1] * 2654435761u;
		g.hy[1] = (c.c0[1] + 1u) * 2654435761u;
		g.hz[0] = c.c0[2] * 805459861u;
		g.hz[1] = (c.c0[2] + 1u) * 805459861u;
		g.mask_or_size = lv.size[l] - 1u;
	} else {
		const uint32_t res = lv.res[l];
		g.hx[0] = c.c0[0];
		g.hx[1] = c.c0[0] + 1u;
		g.hy[0] = c.c0[1] * res;
		g.hy[1] = g.hy[0] + res;
		g.hz[0] = c.c0[2] * res * res;
		g.hz[1] = g.hz[0] + res * res;
		g.mask_or_size = lv.size[l];
		// A cell inside the lattice gives a sum below 2 * size (a corner on the far cube face wraps once).  A sample that a
		// learned motion, or a caller's query box, has put outside the unit cube can give anything; the general rule is the
		// lattice index modulo the level's size, over the integers.  The three terms are reduced here, once per level and only
		// for such samples, so that the per-corner combination stays two compare-and-subtract steps.
		if (max(c.c0[0], max(c.c0[1], c.c0[2])) >= res) {
			const uint2 vx = reduce_outside_axis(c.c0[0], 1u, g.mask_or_size), vy = reduce_outside_axis(c.c0[1], res, g.mask_or_size),
			            vz = reduce_outside_axis(c.c0[2], res * res, g.mask_or_size);
			g.hx[0] = vx.x, g.hx[1] = vx.y, g.hy[0] = vy.x, g.hy[1] = vy.y, g.hz[0] = vz.x, g.hz[1] = vz.y;
		}
	}
	return g;
}

__device__ __forceinline__ uint32_t geom_index(const LevelGeom& g, uint32_t k) {
	const uint32_t bx = k & 1u, by = (k >> 1) & 1u, bz = (k >> 2) & 1u;
	uint32_t idx;
	if (g.hashed) {
		idx = (g.hx[bx] ^ g.hy[by] ^ g.hz[bz]) & g.mask_or_size;
	} else {
		idx = g.hx[bx] + g.hy[by] + g.hz[bz];  // < 3 * size (level_geom)
		idx -= idx >= g.mask_or_size ? g.mask_or_size : 0u;
		idx -= idx >= g.mask_or_size ? g.mask_or_size : 0u;
	}
	return g.offset + idx;
}

}  // namespace n2b
