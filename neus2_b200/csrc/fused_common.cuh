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
	// forward pass on a list of samples: entry i of the pass reads coords row index[i] and writes out row index[i] (nullptr: i)
	const uint32_t* index;
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
		// A dense level's cell is clamped to the lattice: inside the unit cube that changes nothing (the far face is cell
		// res - 1 with its upper corner at res, which wraps once below); a sample that a learned motion, or a caller's query
		// box, has put outside the cube reads the edge cells instead of whatever index arithmetic on a negative or large
		// coordinate would land on.  Branch-free on purpose: a rare branch here costs the fused kernels 4-8 %.
		const int res = (int)lv.res[l];
		const uint32_t cx = (uint32_t)min(max((int)c.c0[0], 0), res - 1), cy = (uint32_t)min(max((int)c.c0[1], 0), res - 1),
		               cz = (uint32_t)min(max((int)c.c0[2], 0), res - 1);
		g.hx[0] = cx;
		g.hx[1] = cx + 1u;
		g.hy[0] = cy * (uint32_t)res;
		g.hy[1] = g.hy[0] + (uint32_t)res;
		g.hz[0] = cz * (uint32_t)(res * res);
		g.hz[1] = g.hz[0] + (uint32_t)(res * res);
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
		idx = g.hx[bx] + g.hy[by] + g.hz[bz];  // < 2 * size: a corner on the far cube face wraps once
		idx -= idx >= g.mask_or_size ? g.mask_or_size : 0u;
	}
	return g.offset + idx;
}

}  // namespace n2b
