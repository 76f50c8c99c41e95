// Marching cubes on an SDF lattice (marching_cubes_gpu, gen_vertices, gen_faces of the reference,
// src/marching_cubes.cu:276-329, 377-718, 794-822).
//
// The reference numbers vertices and triangles with global atomicAdd counters (order changes run to run) and keeps a
// 3 x res^3 int grid of vertex ids (1.5 GiB at 512^3).  Here every cell gets its output ranges from an exclusive prefix
// sum in cell-linear order: vertex and index numbering is canonical and reproducible, and the only scratch is one
// 64-bit key per cell (vertex count | index count).  A face looks the id of a neighbouring cell's edge vertex up as
// "that cell's vertex base + rank of the edge among the cell's crossing edges", recomputed from four SDF values.
// The 256 x 16 case table is data of the caller (the reference carries its own copy next to gen_faces).
#include "common.cuh"

namespace n2b {

struct McGrid {
	uint32_t rx, ry, rz;
	uint64_t res2, res3;
	uint32_t z_off;  // the slab's first lattice layer in the whole grid (vertex positions are those of the whole grid)
	// A slab that is followed by another one carries that slab's first layer pair as a halo: the layers [count_rz, rz) own no
	// vertices, the cells from layer face_rz - 1 on emit no triangles, and the vertices of the layers [own_rz, count_rz) are
	// numbered (exactly as the next slab numbers them) but not written.  Without a halo all four equal rz.
	uint32_t face_rz, count_rz, own_rz;
	uint32_t vertex_offset;  // added to every vertex id written into the index buffer (global numbering)
	float thresh;
	float scale[3], offset[3];
};

__device__ __forceinline__ uint32_t cell_crossings(const McGrid& g, const float* __restrict__ sdf, uint64_t idx, uint32_t x, uint32_t y,
                                                   uint32_t z) {
	const bool inside = sdf[idx] > g.thresh;
	uint32_t m = 0;
	if (x + 1 < g.rx && inside != (sdf[idx + 1] > g.thresh)) m |= 1u;
	if (y + 1 < g.ry && inside != (sdf[idx + g.rx] > g.thresh)) m |= 2u;
	if (z + 1 < g.rz && inside != (sdf[idx + g.res2] > g.thresh)) m |= 4u;
	return m;
}

__device__ __forceinline__ int cube_mask(const McGrid& g, const float* __restrict__ sdf, uint64_t idx) {
	int mask = 0;
	if (sdf[idx] > g.thresh) mask |= 1;
	if (sdf[idx + 1] > g.thresh) mask |= 2;
	if (sdf[idx + 1 + g.rx] > g.thresh) mask |= 4;
	if (sdf[idx + g.rx] > g.thresh) mask |= 8;
	if (sdf[idx + g.res2] > g.thresh) mask |= 16;
	if (sdf[idx + g.res2 + 1] > g.thresh) mask |= 32;
	if (sdf[idx + g.res2 + 1 + g.rx] > g.thresh) mask |= 64;
	if (sdf[idx + g.res2 + g.rx] > g.thresh) mask |= 128;
	return mask;
}

// key = vertices owned by the cell (edges +x, +y, +z from its corner) | triangle indices of the cell << 32
__global__ void __launch_bounds__(256) mc_count_kernel(McGrid g, const float* __restrict__ sdf, const int8_t* __restrict__ tri_table,
                                                       uint64_t* __restrict__ keys) {
	const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (idx >= g.res3) return;
	const uint32_t x = (uint32_t)(idx % g.rx), y = (uint32_t)((idx / g.rx) % g.ry), z = (uint32_t)(idx / g.res2);
	uint64_t key = z < g.count_rz ? (uint64_t)__popc(cell_crossings(g, sdf, idx, x, y, z)) : 0ull;
	if (x + 1 < g.rx && y + 1 < g.ry && z + 1 < g.face_rz) {
		const int mask = cube_mask(g, sdf, idx);
		if (mask && mask != 255) {
			const int8_t* tri = tri_table + mask * 16;
			uint32_t c = 0;
			for (; c < 15; c += 3)
				if (tri[c] < 0) break;
			key |= (uint64_t)c << 32;
		}
	}
	keys[idx] = key;
}

// ---- three-phase exclusive scan of 64-bit keys (two packed 32-bit sums), 4096 keys per CTA
__device__ __forceinline__ uint64_t block_excl_scan(uint64_t sum, uint64_t* warp_sums, uint64_t* total, uint32_t tid) {
	uint64_t incl = sum;
#pragma unroll
	for (int o = 1; o < 32; o <<= 1) {
		const uint64_t u = __shfl_up_sync(0xffffffffu, incl, o);
		if ((tid & 31) >= (uint32_t)o) incl += u;
	}
	if ((tid & 31) == 31) warp_sums[tid >> 5] = incl;
	__syncthreads();
	if (tid < 32) {
		const uint64_t w = warp_sums[tid];
		uint64_t wi = w;
#pragma unroll
		for (int o = 1; o < 32; o <<= 1) {
			const uint64_t u = __shfl_up_sync(0xffffffffu, wi, o);
			if (tid >= (uint32_t)o) wi += u;
		}
		warp_sums[tid] = wi - w;
		if (tid == 31) *total = wi;
	}
	__syncthreads();
	return warp_sums[tid >> 5] + incl - sum;
}

__global__ void __launch_bounds__(1024) scan_local_kernel(uint64_t n, uint64_t* __restrict__ data, uint64_t* __restrict__ block_sums) {
	__shared__ uint64_t warp_sums[32];
	__shared__ uint64_t total;
	const uint32_t tid = threadIdx.x;
	const uint64_t k0 = (uint64_t)blockIdx.x * 4096u + tid * 4u;
	uint64_t v[4];
#pragma unroll
	for (int e = 0; e < 4; ++e) v[e] = (k0 + e < n) ? data[k0 + e] : 0ull;
	uint64_t run = block_excl_scan(v[0] + v[1] + v[2] + v[3], warp_sums, &total, tid);
#pragma unroll
	for (int e = 0; e < 4; ++e) {
		if (k0 + e < n) data[k0 + e] = run;
		run += v[e];
	}
	if (tid == 0) block_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(1024) scan_sums_kernel(uint32_t n, uint64_t* __restrict__ sums, uint64_t* __restrict__ grand_total) {
	__shared__ uint64_t warp_sums[32];
	__shared__ uint64_t total;
	const uint32_t tid = threadIdx.x;
	uint64_t carry = 0;
	for (uint32_t t0 = 0; t0 < n; t0 += 4096u) {
		const uint32_t k0 = t0 + tid * 4u;
		uint64_t v[4];
#pragma unroll
		for (int e = 0; e < 4; ++e) v[e] = (k0 + e < n) ? sums[k0 + e] : 0ull;
		uint64_t run = carry + block_excl_scan(v[0] + v[1] + v[2] + v[3], warp_sums, &total, tid);
#pragma unroll
		for (int e = 0; e < 4; ++e) {
			if (k0 + e < n) sums[k0 + e] = run;
			run += v[e];
		}
		carry += total;
		__syncthreads();
	}
	if (tid == 0) *grand_total = carry;
}

__global__ void __launch_bounds__(1024) scan_add_kernel(uint64_t n, uint64_t* __restrict__ data, const uint64_t* __restrict__ block_sums) {
	const uint64_t k0 = (uint64_t)blockIdx.x * 4096u + threadIdx.x * 4u;
	const uint64_t add = block_sums[blockIdx.x];
#pragma unroll
	for (int e = 0; e < 4; ++e)
		if (k0 + e < n) data[k0 + e] += add;
}

// counts = {vertices, indices} and, for a slab, {vertices owned by the layers before the last one, vertices owned by the
// first layer} (read off the scanned keys: a cell's key is the number of vertices owned by the cells before it)
__global__ void mc_counts_kernel(McGrid g, const uint64_t* __restrict__ keys, const uint64_t* __restrict__ grand_total,
                                 uint32_t* __restrict__ counts, int slab) {
	const uint32_t nv = (uint32_t)(*grand_total & 0xFFFFFFFFull);
	counts[0] = nv;
	counts[1] = (uint32_t)(*grand_total >> 32);
	if (slab == 1) {
		counts[2] = (uint32_t)(keys[(uint64_t)(g.rz - 1) * g.res2] & 0xFFFFFFFFull);
		counts[3] = g.rz > 1 ? (uint32_t)(keys[g.res2] & 0xFFFFFFFFull) : nv;
	} else if (slab == 2) {  // globally numbered slab: vertices this slab owns (= writes)
		counts[2] = g.own_rz < g.rz ? (uint32_t)(keys[(uint64_t)g.own_rz * g.res2] & 0xFFFFFFFFull) : nv;
		counts[3] = 0;
	}
}

// id of the vertex on the edge of cell `c` along `axis` = the cell's vertex base + rank among its crossing edges
__device__ __forceinline__ uint32_t edge_vertex(const McGrid& g, const float* __restrict__ sdf, const uint64_t* __restrict__ keys, uint64_t c,
                                                uint32_t axis) {
	const uint32_t x = (uint32_t)(c % g.rx), y = (uint32_t)((c / g.rx) % g.ry), z = (uint32_t)(c / g.res2);
	const uint32_t m = cell_crossings(g, sdf, c, x, y, z);
	return g.vertex_offset + (uint32_t)(keys[c] & 0xFFFFFFFFull) + __popc(m & ((1u << axis) - 1u));
}

__global__ void __launch_bounds__(256) mc_emit_kernel(McGrid g, const float* __restrict__ sdf, const int8_t* __restrict__ tri_table,
                                                      const uint64_t* __restrict__ keys, float* __restrict__ verts, uint32_t max_verts,
                                                      uint32_t* __restrict__ indices, uint32_t max_indices) {
	const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (idx >= g.res3) return;
	const uint32_t x = (uint32_t)(idx % g.rx), y = (uint32_t)((idx / g.rx) % g.ry), z = (uint32_t)(idx / g.res2);
	const uint64_t key = keys[idx];
	// gen_vertices (:276-329)
	const uint32_t m = z < g.own_rz ? cell_crossings(g, sdf, idx, x, y, z) : 0u;
	if (m) {
		uint32_t vid = (uint32_t)(key & 0xFFFFFFFFull);
		const float f0 = sdf[idx];
		const uint64_t step[3] = {1ull, (uint64_t)g.rx, g.res2};
#pragma unroll
		for (int e = 0; e < 3; ++e) {
			if (!((m >> e) & 1u)) continue;
			const float f1 = sdf[idx + step[e]];
			const float dt = (g.thresh - f0) / (f1 - f0);
			float q[3] = {(float)x, (float)y, (float)(z + g.z_off)};
			q[e] += dt;
			if (vid < max_verts) {
#pragma unroll
				for (int k = 0; k < 3; ++k) verts[(size_t)vid * 3 + k] = q[k] * g.scale[k] + g.offset[k];
			}
			++vid;
		}
	}
	// gen_faces (:377-718)
	if (x + 1 < g.rx && y + 1 < g.ry && z + 1 < g.face_rz) {
		const int mask = cube_mask(g, sdf, idx);
		if (mask && mask != 255) {
			const int8_t* tri = tri_table + mask * 16;
			uint32_t out = (uint32_t)(key >> 32);
			const uint64_t rx = g.rx, r2 = g.res2;
			for (int i = 0; i < 15; ++i) {
				const int j = tri[i];
				if (j < 0) break;
				uint64_t c;
				uint32_t axis;
				switch (j) {
					case 0: c = idx; axis = 0; break;
					case 1: c = idx + 1; axis = 1; break;
					case 2: c = idx + rx; axis = 0; break;
					case 3: c = idx; axis = 1; break;
					case 4: c = idx + r2; axis = 0; break;
					case 5: c = idx + 1 + r2; axis = 1; break;
					case 6: c = idx + rx + r2; axis = 0; break;
					case 7: c = idx + r2; axis = 1; break;
					case 8: c = idx; axis = 2; break;
					case 9: c = idx + 1; axis = 2; break;
					case 10: c = idx + 1 + rx; axis = 2; break;
					default: c = idx + rx; axis = 2; break;
				}
				if (out < max_indices) indices[out] = edge_vertex(g, sdf, keys, c, axis);
				++out;
			}
		}
	}
}

}  // namespace n2b

using namespace n2b;

extern "C" int neus2b_marching_cubes_scratch_bytes(const uint32_t res[3], uint64_t* bytes) {
	if (!res || !bytes || !res[0] || !res[1] || !res[2]) return NEUS2B_E_INVALID;
	const uint64_t cells = (uint64_t)res[0] * res[1] * res[2];
	const uint64_t blocks = (cells + 4095u) / 4096u;
	*bytes = (cells + blocks + 8u) * sizeof(uint64_t);
	return NEUS2B_OK;
}

static int marching_cubes_impl(const float aabb_min[3], const float aabb_max[3], const uint32_t res[3], uint32_t z0, uint32_t n_layers, int slab,
                               float thresh, const float* d_sdf, const int8_t* d_tri_table, uint64_t* d_scratch, float* d_verts,
                               uint32_t max_verts, uint32_t* d_indices, uint32_t max_indices, uint32_t* d_counts, cudaStream_t stream,
                               uint32_t halo = 0, uint32_t vertex_offset = 0) {
	if (!aabb_min || !aabb_max || !res || !d_sdf || !d_tri_table || !d_scratch || !d_counts) return NEUS2B_E_INVALID;
	if (res[0] < 2 || res[1] < 2 || res[2] < 2 || n_layers < 2 || (uint64_t)z0 + n_layers + halo > res[2] || halo > 1) return NEUS2B_E_INVALID;
	McGrid g;
	g.rx = res[0];
	g.ry = res[1];
	g.rz = n_layers + halo;
	g.face_rz = n_layers;
	g.count_rz = n_layers;
	g.own_rz = halo ? n_layers - 1 : n_layers;
	g.vertex_offset = vertex_offset;
	g.z_off = z0;
	g.res2 = (uint64_t)res[0] * res[1];
	g.res3 = g.res2 * g.rz;
	if (g.res3 > (1ull << 32)) return NEUS2B_E_TOO_LARGE;
	g.thresh = thresh;
	for (int k = 0; k < 3; ++k) {
		g.scale[k] = (aabb_max[k] - aabb_min[k]) / (float)res[k];
		g.offset[k] = aabb_min[k];
	}
	const uint64_t cells = g.res3;
	const uint32_t blocks = (uint32_t)((cells + 4095u) / 4096u);
	uint64_t* keys = d_scratch;
	uint64_t* sums = d_scratch + cells;
	uint64_t* total = sums + blocks;
	const bool emit = d_verts && d_indices;
	if (!emit) {  // pass 1: per-cell counts, ranges, totals (the keys stay in d_scratch for the second call)
		mc_count_kernel<<<(uint32_t)((cells + 255u) / 256u), 256, 0, stream>>>(g, d_sdf, d_tri_table, keys);
		N2B_CHECK_LAUNCH();
		scan_local_kernel<<<blocks, 1024, 0, stream>>>(cells, keys, sums);
		N2B_CHECK_LAUNCH();
		scan_sums_kernel<<<1, 1024, 0, stream>>>(blocks, sums, total);
		N2B_CHECK_LAUNCH();
		scan_add_kernel<<<blocks, 1024, 0, stream>>>(cells, keys, sums);
		N2B_CHECK_LAUNCH();
		mc_counts_kernel<<<1, 1, 0, stream>>>(g, keys, total, d_counts, slab);
		N2B_CHECK_LAUNCH();
		return NEUS2B_OK;
	}
	mc_emit_kernel<<<(uint32_t)((cells + 255u) / 256u), 256, 0, stream>>>(g, d_sdf, d_tri_table, keys, d_verts, max_verts, d_indices, max_indices);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_marching_cubes(const float aabb_min[3], const float aabb_max[3], const uint32_t res[3], float thresh, const float* d_sdf,
                                     const int8_t* d_tri_table, uint64_t* d_scratch, float* d_verts, uint32_t max_verts,
                                     uint32_t* d_indices, uint32_t max_indices, uint32_t* d_counts, neus2b_stream_t stream) {
	if (!res) return NEUS2B_E_INVALID;
	return marching_cubes_impl(aabb_min, aabb_max, res, 0, res[2], 0, thresh, d_sdf, d_tri_table, d_scratch, d_verts, max_verts, d_indices,
	                           max_indices, d_counts, stream);
}

extern "C" int neus2b_marching_cubes_slab(const float aabb_min[3], const float aabb_max[3], const uint32_t res[3], uint32_t z0, uint32_t n_layers,
                                          float thresh, const float* d_sdf_slab, const int8_t* d_tri_table, uint64_t* d_scratch, float* d_verts,
                                          uint32_t max_verts, uint32_t* d_indices, uint32_t max_indices, uint32_t* d_counts,
                                          neus2b_stream_t stream) {
	return marching_cubes_impl(aabb_min, aabb_max, res, z0, n_layers, 1, thresh, d_sdf_slab, d_tri_table, d_scratch, d_verts, max_verts, d_indices,
	                           max_indices, d_counts, stream);
}

extern "C" int neus2b_marching_cubes_slab_global(const float aabb_min[3], const float aabb_max[3], const uint32_t res[3], uint32_t z0,
                                                 uint32_t n_layers, uint32_t halo, float thresh, const float* d_sdf_slab,
                                                 const int8_t* d_tri_table, uint64_t* d_scratch, float* d_verts, uint32_t max_verts,
                                                 uint32_t* d_indices, uint32_t max_indices, uint32_t vertex_offset, uint32_t* d_counts,
                                                 neus2b_stream_t stream) {
	return marching_cubes_impl(aabb_min, aabb_max, res, z0, n_layers, 2, thresh, d_sdf_slab, d_tri_table, d_scratch, d_verts, max_verts, d_indices,
	                           max_indices, d_counts, stream, halo, vertex_offset);
}
