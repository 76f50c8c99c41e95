// What follows marching cubes in Testbed::compute_and_save_marching_cubes_mesh (src/testbed.cu:298-306 of the reference):
// area-weighted vertex normals and 1-ring centroids (compute_mesh_1ring, src/marching_cubes.cu:331-375, 720-735), vertex
// colours from the network (Testbed::compute_mesh_vertex_colors, src/testbed_nerf.cu:4057-4080) and the OBJ / PLY writer
// (save_mesh, src/marching_cubes.cu:824-976, without the texture unwrap).
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"

namespace n2b {

// accumulate_1ring (src/marching_cubes.cu:331-367): every triangle adds the other two corners to each of its vertices
// (homogeneous centroid of the 1-ring) and its area-weighted normal (pb - pa) x (pa - pc) to all three.
__global__ void __launch_bounds__(256) mesh_1ring_kernel(uint32_t n_tris, const uint32_t* __restrict__ indices, const float* __restrict__ verts,
                                                         float* __restrict__ ring, float* __restrict__ normals) {
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_tris; i += gridDim.x * blockDim.x) {
		const uint32_t id[3] = {indices[i * 3 + 0], indices[i * 3 + 1], indices[i * 3 + 2]};
		float p[3][3];
#pragma unroll
		for (int k = 0; k < 3; ++k)
#pragma unroll
			for (int e = 0; e < 3; ++e) p[k][e] = __ldg(verts + (size_t)id[k] * 3 + e);
		if (ring) {
#pragma unroll
			for (int k = 0; k < 3; ++k) {
				const int a = (k + 1) % 3, b = (k + 2) % 3;
#pragma unroll
				for (int e = 0; e < 3; ++e) atomicAdd(ring + (size_t)id[k] * 4 + e, p[a][e] + p[b][e]);
				atomicAdd(ring + (size_t)id[k] * 4 + 3, 2.f);
			}
		}
		if (normals) {
			const float u[3] = {p[1][0] - p[0][0], p[1][1] - p[0][1], p[1][2] - p[0][2]};
			const float v[3] = {p[0][0] - p[2][0], p[0][1] - p[2][1], p[0][2] - p[2][2]};
			const float n[3] = {u[1] * v[2] - u[2] * v[1], u[2] * v[0] - u[0] * v[2], u[0] * v[1] - u[1] * v[0]};
#pragma unroll
			for (int k = 0; k < 3; ++k)
#pragma unroll
				for (int e = 0; e < 3; ++e) atomicAdd(normals + (size_t)id[k] * 3 + e, n[e]);
		}
	}
}

// generate_nerf_network_inputs_from_positions (src/testbed_nerf.cu:838-844): the network sees a vertex from the direction
// that points away from the centre of the unit cube, with the smallest step size.
__global__ void __launch_bounds__(256) mesh_color_inputs_kernel(uint32_t n, const float* __restrict__ verts, float3 aabb_min, float3 aabb_max,
                                                                float* __restrict__ coords) {
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
		const float p[3] = {verts[(size_t)i * 3], verts[(size_t)i * 3 + 1], verts[(size_t)i * 3 + 2]};
		float d[3] = {p[0] - 0.5f, p[1] - 0.5f, p[2] - 0.5f};
		const float nn = sqrtf(d[0] * d[0] + d[1] * d[1] + d[2] * d[2]);
		if (nn > 0.f) {
			d[0] /= nn;
			d[1] /= nn;
			d[2] /= nn;
		}
		float* c = coords + (size_t)i * 7;
		c[0] = (p[0] - aabb_min.x) / (aabb_max.x - aabb_min.x);
		c[1] = (p[1] - aabb_min.y) / (aabb_max.y - aabb_min.y);
		c[2] = (p[2] - aabb_min.z) / (aabb_max.z - aabb_min.z);
		c[3] = 0.f;  // warp_dt(MIN_CONE_STEPSIZE)
		c[4] = (d[0] + 1.f) * 0.5f;
		c[5] = (d[1] + 1.f) * 0.5f;
		c[6] = (d[2] + 1.f) * 0.5f;
	}
}

// extract_srgb_with_activation (src/testbed_nerf.cu:522-535) with the logistic colour activation
__global__ void __launch_bounds__(256) mesh_color_extract_kernel(uint32_t n, const __half* __restrict__ out, int from_linear,
                                                                 float* __restrict__ colors) {
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n * 3u; i += gridDim.x * blockDim.x) {
		const uint32_t v = i / 3u, e = i - v * 3u;
		float c = 1.0f / (1.0f + __expf(-__half2float(out[(size_t)v * 16 + e])));
		if (from_linear) c = c < 0.0031308f ? 12.92f * c : 1.055f * powf(c, 0.41666f) - 0.055f;
		colors[i] = c;
	}
}

}  // namespace n2b

using namespace n2b;

extern "C" int neus2b_mesh_1ring(uint32_t n_verts, const float* d_verts, uint32_t n_indices, const uint32_t* d_indices, float* d_ring,
                                 float* d_normals, neus2b_stream_t stream_) {
	cudaStream_t stream = (cudaStream_t)stream_;
	if (n_indices % 3u) return NEUS2B_E_INVALID;
	if (n_verts == 0) return NEUS2B_OK;
	if (!d_verts || (!d_ring && !d_normals) || (n_indices && !d_indices)) return NEUS2B_E_INVALID;
	if (d_ring) N2B_CHECK_CUDA(cudaMemsetAsync(d_ring, 0, (size_t)n_verts * 16, stream));
	if (d_normals) N2B_CHECK_CUDA(cudaMemsetAsync(d_normals, 0, (size_t)n_verts * 12, stream));
	const uint32_t n_tris = n_indices / 3u;
	if (n_tris == 0) return NEUS2B_OK;
	mesh_1ring_kernel<<<min(div_up(n_tris, 256), (uint32_t)kSMs * 8u), 256, 0, stream>>>(n_tris, d_indices, d_verts, d_ring, d_normals);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

extern "C" int neus2b_mesh_vertex_colors(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n_verts,
                                         const float* d_verts, const float aabb_min[3], const float aabb_max[3], int linear_colors,
                                         float* d_coords_scratch, uint16_t* d_out_scratch, uint32_t scratch_samples, float* d_colors,
                                         neus2b_stream_t stream_) {
	cudaStream_t stream = (cudaStream_t)stream_;
	if (n_verts == 0) return NEUS2B_OK;
	if (!desc || !d_params || !d_verts || !aabb_min || !aabb_max || !d_coords_scratch || !d_out_scratch || !d_colors) return NEUS2B_E_INVALID;
	if (scratch_samples < 128u) return NEUS2B_E_INVALID;
	const float3 mn = make_float3(aabb_min[0], aabb_min[1], aabb_min[2]), mx = make_float3(aabb_max[0], aabb_max[1], aabb_max[2]);
	for (uint32_t off = 0; off < n_verts; off += scratch_samples) {
		const uint32_t n = n_verts - off < scratch_samples ? n_verts - off : scratch_samples;
		mesh_color_inputs_kernel<<<min(div_up(n, 256), (uint32_t)kSMs * 8u), 256, 0, stream>>>(n, d_verts + (size_t)off * 3, mn, mx, d_coords_scratch);
		N2B_CHECK_LAUNCH();
		const int rc = neus2b_neus_forward(desc, d_params, sdf_bias, n, nullptr, d_coords_scratch, d_out_scratch, stream_);
		if (rc) return rc;
		mesh_color_extract_kernel<<<min(div_up(n * 3u, 256), (uint32_t)kSMs * 8u), 256, 0, stream>>>(n, (const __half*)d_out_scratch, linear_colors,
		                                                                                       d_colors + (size_t)off * 3);
		N2B_CHECK_LAUNCH();
	}
	return NEUS2B_OK;
}

// ---- save_mesh (src/marching_cubes.cu:824-976): the same text as the reference's fprintf calls, formatted by all host
// threads into one buffer each and written with one fwrite per buffer.
namespace {

template <typename F>
void format_parallel(size_t n, size_t bytes_per_line, std::vector<std::string>& parts, F line) {
	unsigned n_threads = std::thread::hardware_concurrency();
	if (n_threads == 0) n_threads = 1;
	if (n < 4096) n_threads = 1;
	if (n_threads > 64) n_threads = 64;
	const size_t first = parts.size();
	parts.resize(first + n_threads);
	std::vector<std::thread> pool;
	for (unsigned t = 0; t < n_threads; ++t) {
		const size_t b = n * t / n_threads, e = n * (t + 1) / n_threads;
		std::string* out = &parts[first + t];
		auto work = [=]() {
			out->reserve((e - b) * bytes_per_line);
			char buf[256];
			for (size_t i = b; i < e; ++i) {
				const int len = line(i, buf, sizeof(buf));
				if (len > 0) out->append(buf, (size_t)len);
			}
		};
		if (n_threads == 1) work();
		else pool.emplace_back(work);
	}
	for (auto& th : pool) th.join();
}

inline float clamp01(float v) { return v < 0.f ? 0.f : (v > 1.f ? 1.f : v); }

}  // namespace

extern "C" int neus2b_save_mesh(const char* path, uint32_t n_verts, const float* h_verts, const float* h_normals, const float* h_colors,
                                uint32_t n_indices, const uint32_t* h_indices, float nerf_scale, const float nerf_offset[3],
                                int invert_normals) {
	if (!path || n_indices % 3u || (n_verts && (!h_verts || !h_normals || !h_colors)) || (n_indices && !h_indices) || !nerf_offset ||
	    nerf_scale == 0.f)
		return NEUS2B_E_INVALID;
	const size_t len = strlen(path);
	const bool ply = len >= 4 && strcmp(path + len - 4, ".ply") == 0;
	std::vector<std::string> parts;
	auto position = [&](size_t i, float* p) {
		for (int e = 0; e < 3; ++e) p[e] = (h_verts[i * 3 + e] - nerf_offset[e]) / nerf_scale;
	};
	auto unit_normal = [&](size_t i, float* n) {
		const float* v = h_normals + i * 3;
		// Eigen's normalized(): the three squares are summed as a0 + (a1 + a2), every component is divided by the root; unchanged
		// when the length is zero
		const float z = v[0] * v[0] + (v[1] * v[1] + v[2] * v[2]);
		const float inv = z > 0.f ? sqrtf(z) : 1.f;
		for (int e = 0; e < 3; ++e) n[e] = v[e] / inv;
	};
	const uint32_t n_tris = n_indices / 3u;
	if (ply) {
		char head[512];
		const int hl = snprintf(head, sizeof(head),
		                        "ply\nformat ascii 1.0\ncomment output from https://github.com/NVlabs/instant-ngp\nelement vertex %u\n"
		                        "property float x\nproperty float y\nproperty float z\nproperty float nx\nproperty float ny\nproperty float nz\n"
		                        "property uchar red\nproperty uchar green\nproperty uchar blue\nelement face %u\n"
		                        "property list uchar int vertex_index\nend_header\n",
		                        n_verts, n_tris);
		parts.emplace_back(head, (size_t)hl);
		format_parallel(n_verts, 64, parts, [&](size_t i, char* buf, size_t cap) {
			float p[3], n[3];
			position(i, p);
			unit_normal(i, n);
			const float* c = h_colors + i * 3;
			unsigned char c8[3];
			for (int e = 0; e < 3; ++e) {
				const float v = c[e] * 255.f;
				c8[e] = (unsigned char)(v < 0.f ? 0.f : (v > 255.f ? 255.f : v));
			}
			return snprintf(buf, cap, "%0.5f %0.5f %0.5f %0.3f %0.3f %0.3f %d %d %d\n", p[0], p[1], p[2], n[0], n[1], n[2], c8[0], c8[1], c8[2]);
		});
		format_parallel(n_tris, 28, parts, [&](size_t t, char* buf, size_t cap) {
			const uint32_t* k = h_indices + t * 3;
			return invert_normals ? snprintf(buf, cap, "3 %d %d %d\n", (int)k[0], (int)k[1], (int)k[2])
			                      : snprintf(buf, cap, "3 %d %d %d\n", (int)k[2], (int)k[1], (int)k[0]);
		});
	} else {
		format_parallel(n_verts, 56, parts, [&](size_t i, char* buf, size_t cap) {
			float p[3];
			position(i, p);
			const float* c = h_colors + i * 3;
			return snprintf(buf, cap, "v %0.5f %0.5f %0.5f %0.3f %0.3f %0.3f\n", p[0], p[1], p[2], clamp01(c[0]), clamp01(c[1]), clamp01(c[2]));
		});
		format_parallel(n_verts, 32, parts, [&](size_t i, char* buf, size_t cap) {
			float n[3];
			unit_normal(i, n);
			return snprintf(buf, cap, "vn %0.5f %0.5f %0.5f\n", n[0], n[1], n[2]);
		});
		format_parallel(n_tris, 48, parts, [&](size_t t, char* buf, size_t cap) {
			const uint32_t* k = h_indices + t * 3;
			const uint32_t a = invert_normals ? k[0] + 1 : k[2] + 1, b = k[1] + 1, c = invert_normals ? k[2] + 1 : k[0] + 1;
			return snprintf(buf, cap, "f %u//%u %u//%u %u//%u\n", a, a, b, b, c, c);
		});
	}
	FILE* f = fopen(path, "wb");
	if (!f) return NEUS2B_E_IO;
	bool ok = true;
	for (const std::string& s : parts)
		if (!s.empty() && fwrite(s.data(), 1, s.size(), f) != s.size()) ok = false;
	if (fclose(f) != 0) ok = false;
	return ok ? NEUS2B_OK : NEUS2B_E_IO;
}
