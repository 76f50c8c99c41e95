// Shared device/host helpers of the neus2b kernels (sm_100a).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/neus2b.h"

#define N2B_CHECK_CUDA(expr)                      \
	do {                                          \
		cudaError_t _e = (expr);                  \
		if (_e != cudaSuccess) return (int)_e;    \
	} while (0)
#define N2B_CHECK_LAUNCH()                        \
	do {                                          \
		n2b::count_launch();                      \
		cudaError_t _e = cudaGetLastError();      \
		if (_e != cudaSuccess) return (int)_e;    \
	} while (0)

namespace n2b {
void count_launch();  // capi.cu: every kernel launch of the library passes here (neus2b_launch_count)
}

namespace n2b {

constexpr int kSMs = 148;  // B200: grids are sized in multiples of the SM count

// Level table, passed to kernels by value (lives in constant bank as a kernel parameter).
struct GridLevels {
	uint32_t offset[NEUS2B_MAX_LEVELS + 1];  // in entries of 2 fp16
	uint32_t res[NEUS2B_MAX_LEVELS];
	uint32_t size[NEUS2B_MAX_LEVELS];  // entries in the level
	uint32_t hashed[NEUS2B_MAX_LEVELS];
	float scale[NEUS2B_MAX_LEVELS];
	uint32_t n_levels, n_active;
};

// Level rule the reference uses to report its top resolution (src/testbed.cu:2177): scale = base*b^l - 1,
// res = ceil(scale) + 1; a level is stored densely while res^3 fits in the table, else hashed.
inline int make_levels(const neus2b_grid_desc* d, GridLevels* out) {
	if (!d || d->n_levels == 0 || d->n_levels > NEUS2B_MAX_LEVELS || d->log2_hashmap_size > 24 || d->base_resolution == 0)
		return NEUS2B_E_INVALID;
	const uint32_t T = 1u << d->log2_hashmap_size;
	uint32_t off = 0;
	for (uint32_t l = 0; l < NEUS2B_MAX_LEVELS; ++l) {
		out->res[l] = out->size[l] = out->hashed[l] = 0;
		out->scale[l] = 0.f;
		out->offset[l] = off;
		if (l >= d->n_levels) continue;
		float scale = exp2f((float)l * log2f(d->per_level_scale)) * (float)d->base_resolution - 1.0f;
		uint32_t res = (uint32_t)ceilf(scale) + 1u;
		uint64_t dense = (uint64_t)res * res * res;
		uint32_t n;
		if (dense > (uint64_t)T) {
			out->hashed[l] = 1;
			n = T;
		} else {
			n = (uint32_t)((dense + 7u) / 8u * 8u);
		}
		out->scale[l] = scale;
		out->res[l] = res;
		out->size[l] = n;
		off += n;
	}
	out->offset[NEUS2B_MAX_LEVELS] = off;
	for (uint32_t l = d->n_levels; l <= NEUS2B_MAX_LEVELS; ++l) out->offset[l] = off;
	out->n_levels = d->n_levels;
	out->n_active = d->n_active_levels < d->n_levels ? d->n_active_levels : d->n_levels;
	return NEUS2B_OK;
}

// ---- corner geometry of one (sample, level) pair
struct Cell {
	uint32_t c0[3];
	float f[3];
};

__device__ __forceinline__ Cell level_cell(const GridLevels& lv, uint32_t l, const float* x) {
	Cell c;
	const float scale = lv.scale[l];
#pragma unroll
	for (int d = 0; d < 3; ++d) {
		float pos = __fmaf_rn(x[d], scale, 0.5f);
		float fl = floorf(pos);
		c.f[d] = pos - fl;
		c.c0[d] = (uint32_t)(int32_t)fl;
	}
	return c;
}

// Entry index (level offset included) of corner k (bit d of k = +1 along axis d).
__device__ __forceinline__ uint32_t corner_index(const GridLevels& lv, uint32_t l, const Cell& c, uint32_t k) {
	const uint32_t cx = c.c0[0] + (k & 1u), cy = c.c0[1] + ((k >> 1) & 1u), cz = c.c0[2] + ((k >> 2) & 1u);
	uint32_t idx;
	if (lv.hashed[l]) {
		idx = cx ^ (cy * 2654435761u) ^ (cz * 805459861u);
		idx &= lv.size[l] - 1u;  // hashed levels have a power-of-two size
	} else {
		// dense level: the cell is clamped to the lattice (no change inside the unit cube; samples outside it read the edge
		// cells), a corner on the far cube face wraps once
		const int res = (int)lv.res[l];
		const uint32_t size = lv.size[l];
		const uint32_t bx = k & 1u, by = (k >> 1) & 1u, bz = (k >> 2) & 1u;
		const uint32_t x0 = (uint32_t)min(max((int)c.c0[0], 0), res - 1) + bx, y0 = (uint32_t)min(max((int)c.c0[1], 0), res - 1) + by,
		               z0 = (uint32_t)min(max((int)c.c0[2], 0), res - 1) + bz;
		idx = x0 + y0 * (uint32_t)res + z0 * (uint32_t)(res * res);
		idx -= idx >= size ? size : 0u;
	}
	return lv.offset[l] + idx;
}

__device__ __forceinline__ float corner_weight(const Cell& c, uint32_t k) {
	const float wx = (k & 1u) ? c.f[0] : 1.0f - c.f[0];
	const float wy = (k & 2u) ? c.f[1] : 1.0f - c.f[1];
	const float wz = (k & 4u) ? c.f[2] : 1.0f - c.f[2];
	return wx * wy * wz;
}

// d w_k / d x (level scale included)
__device__ __forceinline__ void corner_dweight(const Cell& c, float scale, uint32_t k, float* dw) {
	const float wx = (k & 1u) ? c.f[0] : 1.0f - c.f[0];
	const float wy = (k & 2u) ? c.f[1] : 1.0f - c.f[1];
	const float wz = (k & 4u) ? c.f[2] : 1.0f - c.f[2];
	dw[0] = ((k & 1u) ? scale : -scale) * wy * wz;
	dw[1] = ((k & 2u) ? scale : -scale) * wx * wz;
	dw[2] = ((k & 4u) ? scale : -scale) * wx * wy;
}

__device__ __forceinline__ __half2 ldg_h2(const __half* grid, uint32_t entry) {
	return __ldg(reinterpret_cast<const __half2*>(grid) + entry);
}

// Packed fp16x2 reduction into global memory (one L2 atomic per grid entry).  Written as `red`: atomicAdd on a __half2
// is an `atom` with a result that travels back from L2 and holds a register until it arrives, whether it is used or not.
__device__ __forceinline__ void red_add_h2(__half* grid_grad, uint32_t entry, float g0, float g1) {
	const __half2 v = __floats2half2_rn(g0, g1);
	asm volatile("red.global.add.noftz.f16x2 [%0], %1;" ::"l"(reinterpret_cast<__half2*>(grid_grad) + entry), "r"(*reinterpret_cast<const uint32_t*>(&v))
	             : "memory");
}
// Two neighbouring entries (entry even: 8-byte aligned) in one reduction.
__device__ __forceinline__ void red_add_h2x2(__half* grid_grad, uint32_t entry, float a0, float a1, float b0, float b1) {
	const __half2 va = __floats2half2_rn(a0, a1), vb = __floats2half2_rn(b0, b1);
	asm volatile("red.global.add.noftz.v2.f16x2 [%0], {%1, %2};" ::"l"(reinterpret_cast<__half2*>(grid_grad) + entry),
	             "r"(*reinterpret_cast<const uint32_t*>(&va)), "r"(*reinterpret_cast<const uint32_t*>(&vb))
	             : "memory");
}

// ---- real spherical harmonics, degree 4, of 2*dir-1
__device__ __forceinline__ void sh4_eval(const float* dir01, float* out) {
	const float x = dir01[0] * 2.f - 1.f, y = dir01[1] * 2.f - 1.f, z = dir01[2] * 2.f - 1.f;
	const float xy = x * y, xz = x * z, yz = y * z, x2 = x * x, y2 = y * y, z2 = z * z;
	out[0] = 0.28209479177387814f;
	out[1] = -0.48860251190291987f * y;
	out[2] = 0.48860251190291987f * z;
	out[3] = -0.48860251190291987f * x;
	out[4] = 1.0925484305920792f * xy;
	out[5] = -1.0925484305920792f * yz;
	out[6] = 0.94617469575755997f * z2 - 0.31539156525251999f;
	out[7] = -1.0925484305920792f * xz;
	out[8] = 0.54627421529603959f * x2 - 0.54627421529603959f * y2;
	out[9] = 0.59004358992664352f * y * (-3.0f * x2 + y2);
	out[10] = 2.8906114426405538f * xy * z;
	out[11] = 0.45704579946446572f * y * (1.0f - 5.0f * z2);
	out[12] = 0.3731763325901154f * z * (5.0f * z2 - 3.0f);
	out[13] = 0.45704579946446572f * x * (1.0f - 5.0f * z2);
	out[14] = 1.4453057213202769f * z * (x2 - y2);
	out[15] = 0.59004358992664352f * x * (-x2 + 3.0f * y2);
}

// ---- PCG32 (tcnn::default_rng_t): 64-bit LCG state, XSH-RR output, O(log n) skip-ahead
struct Pcg32 {
	uint64_t state, inc;
	__host__ __device__ uint32_t next_uint() {
		uint64_t old = state;
		state = old * 0x5851f42d4c957f2dULL + inc;
		uint32_t xorshifted = (uint32_t)(((old >> 18u) ^ old) >> 27u);
		uint32_t rot = (uint32_t)(old >> 59u);
		return (xorshifted >> rot) | (xorshifted << ((~rot + 1u) & 31u));
	}
	__host__ __device__ float next_float() {
		union {
			uint32_t u;
			float f;
		} x;
		x.u = (next_uint() >> 9) | 0x3f800000u;
		return x.f - 1.0f;
	}
	__host__ __device__ void advance(uint64_t delta) {
		uint64_t cur_mult = 0x5851f42d4c957f2dULL, cur_plus = inc, acc_mult = 1u, acc_plus = 0u;
		while (delta > 0) {
			if (delta & 1) {
				acc_mult *= cur_mult;
				acc_plus = acc_plus * cur_mult + cur_plus;
			}
			cur_plus = (cur_mult + 1) * cur_plus;
			cur_mult *= cur_mult;
			delta >>= 1;
		}
		state = acc_mult * state + acc_plus;
	}
};

inline uint32_t div_up(uint64_t a, uint32_t b) { return (uint32_t)((a + b - 1) / b); }

}  // namespace n2b
