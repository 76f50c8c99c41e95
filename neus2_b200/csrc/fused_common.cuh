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
	}
	return g;
}

__device__ __forceinline__ uint32_t geom_index(const LevelGeom& g, uint32_t k) {
	const uint32_t bx = k & 1u, by = (k >> 1) & 1u, bz = (k >> 2) & 1u;
	uint32_t idx;
	if (g.hashed) {
		idx = (g.hx[bx] ^ g.hy[by] ^ g.hz[bz]) & g.mask_or_size;
	} else {
		// positions inside the unit cube give < 2 * size: a corner on the far cube face wraps once.  Samples a learned motion
		// has carried outside the cube can give anything: then the index is reduced like the general rule says (% size)
		idx = g.hx[bx] + g.hy[by] + g.hz[bz];
		if (idx >= g.mask_or_size) {
			idx -= g.mask_or_size;
			if (idx >= g.mask_or_size) idx %= g.mask_or_size;
		}
	}
	return g.offset + idx;
}

}  // namespace n2b
