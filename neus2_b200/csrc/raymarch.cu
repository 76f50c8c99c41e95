// Ray-march side of the NeuS training step: occupancy-grid DDA sample generation, NeuS compositing + loss + loss
// gradient, compaction and roll-over (src/testbed_nerf.cu:1253-1996, 3908-3916 of the reference).
//
// The reference reserves output ranges with atomicAdd, so its sample order changes from run to run.  Here every
// range comes from an exclusive prefix sum over the ray index: the set of samples, each ray's step count and the
// compaction result are reproducible and identical to the canonical-order CPU restatement.
//
// This file is compiled with -fmad=false: the DDA decides integer step counts from fp32 arithmetic, so every
// operation is a single IEEE operation in a fixed order (fused multiply-adds only where written explicitly).
#include <mutex>

#include "common.cuh"
#include "march.cuh"
#include "delta.cuh"

namespace n2b {

// First half of generate_training_samples_nerf_with_global_movement (:1287-1409), part one: one thread builds one ray
// (pixel, camera, start parameter) and lists it for the march if it can take samples.
__global__ void __launch_bounds__(256) ray_setup_kernel(neus2b_dataset ds, neus2b_train_cfg cfg, uint32_t n_rays_max,
                                                        const uint32_t* __restrict__ d_n_rays, uint32_t n_rays_total,
                                                        const uint32_t* __restrict__ d_n_rays_total, Pcg32 rng0, RayTmp* __restrict__ tmp,
                                                        uint64_t* __restrict__ scan_in, const int32_t* __restrict__ occ_bounds,
                                                        uint32_t* __restrict__ hit_list, uint32_t* __restrict__ hit_count) {
	if (d_n_rays_total) n_rays_total = *d_n_rays_total;
	if (blockIdx.x == 0 && threadIdx.x == 0) scan_in[n_rays_max + 512] = 0ull;  // the scan's ticket counter (see scan_kernel)
	const CullBox box = cull_box(occ_bounds);
	const uint32_t n_rays = d_n_rays ? min(*d_n_rays, n_rays_max) : n_rays_max;
	for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_rays; i += gridDim.x * blockDim.x) {
		RayTmp r;
		r.numsteps = 0;
		r.startt = 0.f;
#pragma unroll
		for (int e = 0; e < 3; ++e) r.o[e] = r.d[e] = 0.f;
		const uint32_t ig = i + cfg.ray_index_offset;
		const uint32_t img = image_idx(ig, n_rays, n_rays_total, ds.n_images);
		Pcg32 rng = rng0;
		rng.advance((uint64_t)ig * 8u);
		float xy[2], rgba[4];
		random_image_pos(rng, ds, cfg.snap_to_pixel_centers != 0, xy);
		read_rgba(ds, img, xy, rgba);
		const bool keep = !(rgba[0] <= 0.0f && rng.next_float() >= 0.9f);
		bool may_hit = false;
		if (keep) {
			(void)rng.next_float();  // motion-blur time (:1307)
			const float* X = ds.d_xforms + (size_t)img * 12;
			const float fx = ds.d_focal[img * 2], fy = ds.d_focal[img * 2 + 1];
			const float ppx = ds.d_principal[img * 2], ppy = ds.d_principal[img * 2 + 1];
			const float dl[3] = {(xy[0] - ppx) * (float)ds.width / fx, (xy[1] - ppy) * (float)ds.height / fy, 1.0f};
			float dirn[3];
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				r.o[e] = X[9 + e];
				r.d[e] = sum3_eigen(X[0 + e] * dl[0], X[3 + e] * dl[1], X[6 + e] * dl[2]);
			}
			normalize3_eigen(r.d, dirn);
			if (cfg.use_global_movement) {  // :1370-1378: the ray is moved; its direction is not normalised again
				float o2[3], q[3], dq[3];
#pragma unroll
				for (int e = 0; e < 3; ++e) o2[e] = r.o[e] - cfg.first_frame_offset[e];
				rotate3(cfg.rotation, o2, q);
				rotate3(cfg.rotation, dirn, dq);
#pragma unroll
				for (int e = 0; e < 3; ++e) {
					r.o[e] = q[e] + cfg.transition[e];
					r.d[e] = dirn[e] = dq[e];  // the later passes take this direction as it is
				}
			}
			float tmin, tmax;
			aabb_ray_intersect(cfg.aabb_min, cfg.aabb_max, r.o, dirn, tmin, tmax);
			tmin = fmaxf(tmin, 0.0f);
			float startt = tmin;
			startt += calc_dt(startt, cfg.cone_angle_constant) * rng.next_float();
			r.startt = startt;
			float t_lo, t_hi;
			may_hit = cull_ray(box, r.o, dirn, t_lo, t_hi);
		}
		tmp[i] = r;
		scan_in[i] = 0ull;
		if (may_hit) hit_list[atomicAdd(hit_count, 1u)] = i;  // any order: the march writes its result under the ray's own index
	}
}

// Part two: one warp marches one listed ray and counts its steps.
__global__ void __launch_bounds__(128) count_steps_kernel(neus2b_train_cfg cfg, const uint8_t* __restrict__ bitfield, RayTmp* __restrict__ tmp,
                                                          uint64_t* __restrict__ scan_in, uint32_t* __restrict__ masks,
                                                          const int32_t* __restrict__ occ_bounds, const uint32_t* __restrict__ hit_list,
                                                          const uint32_t* __restrict__ hit_count) {
	const int lane = threadIdx.x & 31;
	const CullBox box = cull_box(occ_bounds);
	const uint32_t n_hit = *hit_count;
	const uint32_t warps = gridDim.x * (blockDim.x >> 5);
	for (uint32_t h = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); h < n_hit; h += warps) {
		const uint32_t i = hit_list[h];
		RayTmp r = tmp[i];
		float dirn[3];
		if (cfg.use_global_movement) {
#pragma unroll
			for (int e = 0; e < 3; ++e) dirn[e] = r.d[e];
		} else {
			normalize3_eigen(r.d, dirn);
		}
		float t_lo, t_hi;
		(void)cull_ray(box, r.o, dirn, t_lo, t_hi);
		uint32_t n_chunks = 0;
		r.numsteps = march_ray<false>(cfg, r.o, dirn, r.startt, bitfield, NEUS2B_STEPS, nullptr, lane,
		                              masks ? masks + (size_t)i * kMaskWords : nullptr, &n_chunks, t_lo, t_hi);
		if (lane == 0) {
			scan_in[i] = r.numsteps ? ((1ull << 32) | (uint64_t)r.numsteps) : 0ull;
			if (n_chunks > kMaskWords) r.numsteps |= 0x80000000u;  // the mask record does not cover this ray: the emit pass marches again
			tmp[i].numsteps = r.numsteps;
		}
	}
}

// Exclusive prefix sum of n 64-bit keys in place, n read on the device (2^20 at most); the total goes to data[n_max].
// Every CTA scans tiles of 4096 keys; the CTA that finishes last (a ticket, no waiting on other CTAs) scans the tile sums
// and adds the tile offsets.  Scratch lives behind the total: data[n_max + 1 ..] tile sums, data[n_max + 512] the ticket
// counter, zero before the first launch and left at zero (the buffer has max_rays + 1024 entries).
constexpr uint32_t kScanTile = 4096u, kScanMaxTiles = 256u;
__global__ void __launch_bounds__(1024) scan_kernel(uint32_t n_max, const uint32_t* __restrict__ d_n, uint64_t* __restrict__ data) {
	__shared__ uint64_t warp_sums[32];
	__shared__ uint64_t tile_total;
	__shared__ uint64_t offsets[kScanMaxTiles];
	__shared__ bool is_last;
	const uint32_t tid = threadIdx.x;
	const uint32_t n = d_n ? min(*d_n, n_max) : n_max;
	const uint32_t n_tiles = (n + kScanTile - 1u) / kScanTile;
	uint64_t* tile_sums = data + n_max + 1;
	unsigned long long* ticket = reinterpret_cast<unsigned long long*>(data + n_max + 512);
	for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
		const uint32_t k0 = tile * kScanTile + tid * 4u;
		uint64_t v[4];
#pragma unroll
		for (int e = 0; e < 4; ++e) v[e] = (k0 + e < n) ? data[k0 + e] : 0ull;
		const uint64_t sum = v[0] + v[1] + v[2] + v[3];
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
			if (tid == 31) tile_total = wi;
		}
		__syncthreads();
		uint64_t run = warp_sums[tid >> 5] + incl - sum;
#pragma unroll
		for (int e = 0; e < 4; ++e) {
			if (k0 + e < n) data[k0 + e] = run;
			run += v[e];
		}
		if (tid == 0) tile_sums[tile] = tile_total;
		__syncthreads();
	}
	// ticket: the last CTA to get here sees every tile's sum and local scan
	__threadfence();
	if (tid == 0) is_last = atomicAdd(ticket, 1ull) == (unsigned long long)(gridDim.x - 1u);
	__syncthreads();
	if (!is_last) return;
	__threadfence();
	// (what the other CTAs wrote is read through L2, past this SM's L1)
	if (tid == 0) {
		uint64_t run = 0;
		for (uint32_t t = 0; t < n_tiles; ++t) {
			offsets[t] = run;
			run += __ldcg(tile_sums + t);
		}
		data[n_max] = run;
		*ticket = 0ull;
	}
	__syncthreads();
	for (uint32_t k = kScanTile + tid; k < n; k += 1024u) data[k] = __ldcg(data + k) + offsets[k / kScanTile];
}

// The scan holds one offset per tile in shared memory and keeps its tile sums and ticket behind the keys: 2^20 keys at most.
constexpr uint32_t kScanMaxKeys = kScanTile * kScanMaxTiles;
static_assert(kScanMaxKeys == NEUS2B_MAX_RAYS_PER_CALL, "the header states the scan's capacity");

int launch_scan(uint32_t n_max, const uint32_t* d_n, uint64_t* data, cudaStream_t stream) {
	if (n_max > kScanMaxKeys) return NEUS2B_E_TOO_LARGE;
	scan_kernel<<<64, 1024, 0, stream>>>(n_max, d_n, data);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

// Second half of the sample generator (:1410-1445): canonical ranges, then march again and write the coordinates.
__global__ void __launch_bounds__(128) emit_samples_kernel(neus2b_train_cfg cfg, uint32_t n_rays_max, const uint32_t* __restrict__ d_n_rays,
                                                           uint32_t max_samples, const uint32_t* __restrict__ d_prev_samples,
                                                           const uint8_t* __restrict__ bitfield, const RayTmp* __restrict__ tmp,
                                                           const uint64_t* __restrict__ scan, uint32_t* __restrict__ ray_indices,
                                                           float* __restrict__ rays, uint32_t* __restrict__ numsteps,
                                                           float* __restrict__ coords, uint32_t* __restrict__ counters,
                                                           const uint32_t* __restrict__ masks) {
	const int lane = threadIdx.x & 31;
	if (blockIdx.x == 0 && threadIdx.x == 0) counters[1] = (uint32_t)(scan[n_rays_max] & 0xFFFFFFFFull);  // all steps, dropped rays included
	// max_inference of the training loop (:3764-3769): after a step that took samples, the room is the previous step's count
	// rounded up to the batch granularity, and rays beyond it are dropped like rays beyond the buffer
	const uint32_t buffer_samples = max_samples;
	if (d_prev_samples) {
		const uint32_t prev = *d_prev_samples;
		if (prev) max_samples = min(max_samples, (min(prev, max_samples) + 127u) / 128u * 128u);
	}
	const uint32_t n_rays = d_n_rays ? min(*d_n_rays, n_rays_max) : n_rays_max;
	const uint32_t warps = gridDim.x * (blockDim.x >> 5);
	for (uint32_t i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n_rays; i += warps) {
		RayTmp r = tmp[i];
		const bool long_ray = (r.numsteps & 0x80000000u) != 0;
		r.numsteps &= 0x7fffffffu;
		if (r.numsteps == 0) continue;
		const uint64_t key = scan[i];
		const uint32_t base = (uint32_t)(key & 0xFFFFFFFFull), kidx = (uint32_t)(key >> 32);
		if (base + r.numsteps > max_samples) {  // no room left: drop the ray (:1412-1414); the flag reports an exhausted buffer only
			if (lane == 0 && base + r.numsteps > buffer_samples) atomicOr(&counters[3], 1u);
			continue;
		}
		if (lane == 0) {
			atomicMax(&counters[0], kidx + 1u);
			atomicMax(&counters[4], base + r.numsteps);
			ray_indices[kidx] = i;
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				rays[(size_t)kidx * 6 + e] = r.o[e];
				rays[(size_t)kidx * 6 + 3 + e] = r.d[e];
			}
			numsteps[kidx * 2 + 0] = r.numsteps;
			numsteps[kidx * 2 + 1] = base;
		}
		float dirn[3];
		if (cfg.use_global_movement) {
#pragma unroll
			for (int e = 0; e < 3; ++e) dirn[e] = r.d[e];
		} else {
			normalize3_eigen(r.d, dirn);
		}
		// the mask record covers the first kMaskWords * 32 ray parameters; longer rays march again
		if (masks && !long_ray)
			emit_from_masks(cfg, r.o, dirn, r.startt, masks + (size_t)i * kMaskWords, r.numsteps, coords + (size_t)base * 7, lane);
		else
			march_ray<true>(cfg, r.o, dirn, r.startt, bitfield, r.numsteps, coords + (size_t)base * 7, lane);
	}
}

// ------------------------------------------------------------------------------------------------ loss
struct CompTmp {  // 8 floats per kept ray
	float rgb[3], T, weight_sum;
	uint32_t n, full;
	uint32_t state;  // windowed evaluation: bit 0 = the ray is finished (terminated or all samples seen), bits 1.. = samples seen
};

constexpr uint32_t kFull = 0xffffffffu;

// Transmittance in front of each lane's sample, multiplied in ray order exactly like the reference's serial loop
// (T *= 1 - alpha), so the early-termination decision T < 1e-4 does not depend on how the work is parallelised.
__device__ __forceinline__ float serial_transmittance(float T_carry, float one_minus_alpha, int lane) {
	float run = T_carry, mine = 0.f;
#pragma unroll
	for (int k = 0; k < 32; ++k) {
		const float om = __shfl_sync(kFull, one_minus_alpha, k);
		if (lane == k) mine = run;
		run *= om;
	}
	return mine;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
	return v;
}
__device__ __forceinline__ float warp_incl_scan(float v, int lane) {
#pragma unroll
	for (int o = 1; o < 32; o <<= 1) {
		const float u = __shfl_up_sync(kFull, v, o);
		if (lane >= o) v += u;
	}
	return v;
}

// BENT_DIR (:1574-1579): the direction the network saw at the ray's first sample replaces the ray direction; read from
// the second 16-byte half of that sample's output row as lane 0 holds it (halves 8..11 = words x, y).
__device__ __forceinline__ void bent_dir_from_lane0(uint32_t wx, uint32_t wy, float* dir) {
	wx = __shfl_sync(kFull, wx, 0);
	wy = __shfl_sync(kFull, wy, 0);
	const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&wx)), b = __half22float2(*reinterpret_cast<const __half2*>(&wy));
	const float dd[3] = {a.x * 2.f - 1.f, a.y * 2.f - 1.f, b.x * 2.f - 1.f};
	normalize3_eigen(dd, dir);
}

// Pass A (:1563-1617): composite along the ray until transmittance drops below 1e-4; count the surviving samples.
// One warp per kept ray, 32 samples per iteration.
//
// Windowed form: a call composites samples [lo, min(ns, hi)) of every ray that is not finished yet, picking the ray's state
// up from tmp (lo > 0) and leaving it there.  A ray that goes on appends the rows of its next window, samples
// [hi, min(ns, next_hi)), to list (a range reserved with one atomicAdd on *list_len: the order of the list does not matter,
// every row is evaluated on its own) and adds their number to *evaluated.  lo = 0, hi = all, list = nullptr: the whole ray
// in one call, as the reference does.
__global__ void __launch_bounds__(128) composite_kernel(neus2b_train_cfg cfg, const uint32_t* __restrict__ counters,
                                                        const __half* __restrict__ mlp_out, const uint32_t* __restrict__ numsteps,
                                                        const float* __restrict__ coords, CompTmp* __restrict__ tmp,
                                                        uint64_t* __restrict__ scan_in, uint32_t n_rays_max, uint32_t lo, uint32_t hi,
                                                        uint32_t next_hi, uint32_t* __restrict__ list, uint32_t* __restrict__ list_len,
                                                        uint32_t* __restrict__ evaluated) {
	const int lane = threadIdx.x & 31;
	if (blockIdx.x == 0 && threadIdx.x == 0) scan_in[n_rays_max + 512] = 0ull;  // the scan's ticket counter (see scan_kernel)
	const uint32_t n_kept = counters[0];
	const uint32_t warps = gridDim.x * (blockDim.x >> 5);
	for (uint32_t i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n_kept; i += warps) {
		const uint32_t ns = numsteps[i * 2], base = numsteps[i * 2 + 1];
		float T = 1.f, rgb[3] = {0.f, 0.f, 0.f}, ws = 0.f;
		uint32_t n = 0;
		if (lo > 0) {
			const CompTmp c = tmp[i];
			if (c.state & 1u) continue;  // finished in an earlier window: its record stands
			T = c.T, rgb[0] = c.rgb[0], rgb[1] = c.rgb[1], rgb[2] = c.rgb[2], ws = c.weight_sum, n = c.n;
		}
		const uint32_t lim = min(ns, hi);
		bool done = false, terminated = false;
		// the next 32 samples are in flight while the current 32 are composited (a long ray is a serial chain of chunks)
		uint4 q0 = make_uint4(0u, 0u, 0u, 0u), q1 = q0;
		float qdt = 0.f;
		if (lo + (uint32_t)lane < lim) {
			const uint4* p = reinterpret_cast<const uint4*>(mlp_out + (size_t)(base + lo + lane) * 16);
			q0 = __ldg(p);
			q1 = __ldg(p + 1);
			qdt = coords[(size_t)(base + lo + lane) * 7 + 3];
		}
		float dir[3];
		{  // BENT_DIR: the direction the network saw at the ray's first sample (kept rays have at least one sample)
			uint32_t wx = q1.x, wy = q1.y;
			if (lo > 0 && lane == 0) {
				const uint4 f = __ldg(reinterpret_cast<const uint4*>(mlp_out + (size_t)base * 16) + 1);
				wx = f.x, wy = f.y;
			}
			bent_dir_from_lane0(wx, wy, dir);
		}
		for (uint32_t j0 = lo; j0 < lim && !done; j0 += 32) {
			const uint32_t j = j0 + lane;
			const bool valid = j < lim;
			const uint4 c0 = q0, c1 = q1;
			const float cdt = qdt;
			if (j + 32u < lim) {
				const uint4* p = reinterpret_cast<const uint4*>(mlp_out + (size_t)(base + j + 32u) * 16);
				q0 = __ldg(p);
				q1 = __ldg(p + 1);
				qdt = coords[(size_t)(base + j + 32u) * 7 + 3];
			}
			NeusSample s;
			s.alpha = 0.f;
			s.rgb[0] = s.rgb[1] = s.rgb[2] = 0.f;
			if (valid) {
				__align__(16) __half o[16];
				reinterpret_cast<uint4*>(o)[0] = c0;
				reinterpret_cast<uint4*>(o)[1] = c1;
				neus_sample(o, cdt, dir, cfg.cos_anneal_ratio, s);
			}
			const float om = 1.f - s.alpha;
			const float Tb = serial_transmittance(T, om, lane);
			const bool active = valid && !(Tb < 1e-4f);
			const uint32_t cnt = __popc(__ballot_sync(kFull, active)), n_valid = __popc(__ballot_sync(kFull, valid));
			const float w = active ? s.alpha * Tb : 0.f;
#pragma unroll
			for (int e = 0; e < 3; ++e) rgb[e] += warp_sum(w * s.rgb[e]);
			ws += warp_sum(w);
			if (cnt) T = __shfl_sync(kFull, Tb * om, cnt - 1);
			n += cnt;
			terminated = cnt < n_valid;  // a sample inside the window found the ray opaque
			done = terminated || n_valid < 32u;
		}
		const bool finished = terminated || lim == ns;
		if (list && !finished) {  // the rows of this ray's next window
			const uint32_t cnt = min(ns, next_hi) - lim;
			uint32_t off = 0;
			if (lane == 0) {
				off = atomicAdd(list_len, cnt);
				atomicAdd(evaluated, cnt);
			}
			off = __shfl_sync(kFull, off, 0);
			for (uint32_t k = lane; k < cnt; k += 32) list[off + k] = base + lim + k;
		}
		if (lane == 0) {
			CompTmp c;
			c.rgb[0] = rgb[0];
			c.rgb[1] = rgb[1];
			c.rgb[2] = rgb[2];
			c.T = T;
			c.weight_sum = ws;
			c.n = n;
			c.full = n == ns;
			c.state = (lim << 1) | (finished ? 1u : 0u);
			tmp[i] = c;
			scan_in[i] = (uint64_t)n;
		}
	}
}

// The first window's list: samples [0, min(ns, hi)) of every kept ray (later windows' lists come from composite_kernel).
// One warp per ray; lens[0] (the list's length) and *evaluated are zero before the launch.
__global__ void __launch_bounds__(128) window_first_kernel(const uint32_t* __restrict__ counters, const uint32_t* __restrict__ numsteps, uint32_t hi,
                                                           uint32_t* __restrict__ list, uint32_t* __restrict__ list_len,
                                                           uint32_t* __restrict__ evaluated) {
	const int lane = threadIdx.x & 31;
	const uint32_t n_kept = counters[0];
	const uint32_t warps = gridDim.x * (blockDim.x >> 5);
	for (uint32_t i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n_kept; i += warps) {
		const uint32_t ns = numsteps[i * 2], base = numsteps[i * 2 + 1];
		const uint32_t cnt = min(ns, hi);
		uint32_t off = 0;
		if (lane == 0) {
			off = atomicAdd(list_len, cnt);
			atomicAdd(evaluated, cnt);
		}
		off = __shfl_sync(kFull, off, 0);
		for (uint32_t k = lane; k < cnt; k += 32) list[off + k] = base + k;
	}
}

// Target pixel, Huber loss, pass B (:1619-1952): loss gradient w.r.t. the 16 network outputs of every kept sample.
// One warp per kept ray; a lane owns one sample of the current 32-sample chunk.
__global__ void __launch_bounds__(128) loss_kernel(neus2b_dataset ds, neus2b_train_cfg cfg, uint32_t n_rays_max,
                                                   const uint32_t* __restrict__ d_n_rays, uint32_t n_rays_total,
                                                   const uint32_t* __restrict__ d_n_rays_total, Pcg32 rng0,
                                                   uint32_t max_compacted, int rollover, uint32_t* __restrict__ counters,
                                                   const __half* __restrict__ mlp_out, const uint32_t* __restrict__ ray_indices,
                                                   uint32_t* __restrict__ numsteps, const float* __restrict__ coords,
                                                   const CompTmp* __restrict__ tmp, const uint64_t* __restrict__ scan,
                                                   float* __restrict__ coords_out, __half* __restrict__ dloss_dout,
                                                   float* __restrict__ loss_out, float* __restrict__ ek_loss_out) {
	const int lane = threadIdx.x & 31;
	if (d_n_rays_total) n_rays_total = *d_n_rays_total;
	const uint32_t n_compacted = (uint32_t)scan[n_rays_max];
	if (blockIdx.x == 0 && threadIdx.x == 0) counters[2] = n_compacted;
	// fill_rollover_and_rescale (call site :3913-3916): when the batch is padded with copies, every gradient row is scaled by
	// n_valid / n_target.  Done here on the value as it was rounded to fp16, which is what a separate pass over the buffer
	// would read: the same bits, one pass over 8 MB less.
	const uint32_t n_valid = min(n_compacted, max_compacted);
	const bool rescale = rollover && n_valid != 0 && n_valid < max_compacted;
	const float rollover_scale = rescale ? (float)n_valid / (float)max_compacted : 1.0f;
	const uint32_t n_kept = counters[0];
	const uint32_t n_rays = d_n_rays ? min(*d_n_rays, n_rays_max) : n_rays_max;
	const uint32_t warps = gridDim.x * (blockDim.x >> 5);
	for (uint32_t i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n_kept; i += warps) {
		const uint32_t base = numsteps[i * 2 + 1];
		const CompTmp c = tmp[i];
		const uint32_t compacted_base = (uint32_t)scan[i];
		const uint32_t cn = min(max_compacted - min(max_compacted, compacted_base), c.n);
		__syncwarp();
		if (lane == 0) {
			numsteps[i * 2 + 0] = cn;
			numsteps[i * 2 + 1] = compacted_base;
			if (loss_out) loss_out[i] = 0.f;
			if (ek_loss_out) ek_loss_out[i] = 0.f;
		}
		if (cn == 0) continue;
		// this ray's first 32 samples are requested now, the next 32 always one chunk ahead: they arrive behind the target
		// pixel fetch and the compositing of the chunk before
		uint4 q0 = make_uint4(0u, 0u, 0u, 0u), q1 = q0;
		float qc[7] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
		if ((uint32_t)lane < cn) {
			const uint4* p = reinterpret_cast<const uint4*>(mlp_out + (size_t)(base + lane) * 16);
			q0 = __ldg(p);
			q1 = __ldg(p + 1);
			const float* cin = coords + (size_t)(base + lane) * 7;
#pragma unroll
			for (int e = 0; e < 7; ++e) qc[e] = cin[e];
		}
		// target colour (:1619-1667), computed by every lane
		const uint32_t ray_idx = ray_indices[i] + cfg.ray_index_offset;
		Pcg32 rng = rng0;
		rng.advance((uint64_t)ray_idx * 8u);
		const uint32_t img = image_idx(ray_idx, n_rays, n_rays_total, ds.n_images);
		float xy[2], bg[3], tex[4], target[3];
		random_image_pos(rng, ds, cfg.snap_to_pixel_centers != 0, xy);
		if (cfg.random_bg_color) {
#pragma unroll
			for (int e = 0; e < 3; ++e) bg[e] = rng.next_float();
		} else {
#pragma unroll
			for (int e = 0; e < 3; ++e) bg[e] = cfg.background_color[e];
		}
#pragma unroll
		for (int e = 0; e < 3; ++e) bg[e] = srgb_to_linear(bg[e]);
		read_rgba(ds, img, xy, tex);
#pragma unroll
		for (int e = 0; e < 3; ++e) {
			target[e] = linear_to_srgb(tex[e] + (1.0f - tex[3]) * bg[e]);
			bg[e] = linear_to_srgb(bg[e]);
		}
		float rgb_ray[3] = {c.rgb[0], c.rgb[1], c.rgb[2]};
		if (c.full) {
#pragma unroll
			for (int e = 0; e < 3; ++e) rgb_ray[e] += c.T * bg[e];
		}
		// Huber(0.1) / 5 (:301-317, :1459)
		float lgl[3], lgg[3];
#pragma unroll
		for (int e = 0; e < 3; ++e) {
			const float diff = rgb_ray[e] - target[e], ad = fabsf(diff), al = 0.1f;
			lgl[e] = (ad > al ? (ad - 0.5f * al) : 0.5f / al * diff * diff) / 5.0f;
			lgg[e] = (ad > al ? (diff > 0 ? 1.0f : -1.0f) : diff / al) / 5.0f;
		}
		// double literals in the reference (:1690-1702): the comparisons are fp64, the assigned constants round to fp32
		const float mask_gt = (double)tex[3] > 0.9999 ? 1.f : 0.f;
		float gws, ws = c.weight_sum;
		if ((double)ws >= 1.0 - 1e-4) {
			ws = (float)(1.0 - 1e-4);
			gws = 0.f;
		} else if ((double)ws <= 1e-4) {
			ws = (float)1e-4;
			gws = 0.f;
		} else {
			const float sg = 1.0f / (1.0f + expf(-ws));
			gws = (mask_gt - sg) * ws * cfg.mask_loss_weight;
		}
		const float n_rays_f = (float)n_rays * (float)(cfg.ray_count_scale ? cfg.ray_count_scale : 1u);
		if (lane == 0 && loss_out) loss_out[i] = sum3_eigen(lgl[0], lgl[1], lgl[2]) / 3.0f / n_rays_f;  // lg.loss.mean() (:1715)
		const float loss_scale = cfg.loss_scale / n_rays_f;
		float dir[3];
		bent_dir_from_lane0(q1.x, q1.y, dir);
		float rgb2c[3] = {0.f, 0.f, 0.f}, T = 1.f, ek = 0.f;
		for (uint32_t j0 = 0; j0 < cn; j0 += 32) {
			const uint32_t j = j0 + lane;
			const bool valid = j < cn;
			const uint4 c0 = q0, c1 = q1;
			float cs[7];
#pragma unroll
			for (int e = 0; e < 7; ++e) cs[e] = qc[e];
			if (j + 32u < cn) {
				const uint4* p = reinterpret_cast<const uint4*>(mlp_out + (size_t)(base + j + 32u) * 16);
				q0 = __ldg(p);
				q1 = __ldg(p + 1);
				const float* cin = coords + (size_t)(base + j + 32u) * 7;
#pragma unroll
				for (int e = 0; e < 7; ++e) qc[e] = cin[e];
			}
			NeusSample s;
			s.alpha = 0.f;
			s.rgb[0] = s.rgb[1] = s.rgb[2] = 0.f;
			if (valid) {
				__align__(16) __half o[16];
				reinterpret_cast<uint4*>(o)[0] = c0;
				reinterpret_cast<uint4*>(o)[1] = c1;
				float* cout = coords_out + (size_t)(compacted_base + j) * 7;
#pragma unroll
				for (int e = 0; e < 7; ++e) cout[e] = cs[e];
				neus_sample(o, cs[3], dir, cfg.cos_anneal_ratio, s);
			}
			const float om = 1.f - s.alpha;
			const float Tb = serial_transmittance(T, om, lane);
			const float w = valid ? s.alpha * Tb : 0.f;
			const float Ta = Tb * om;  // transmittance after this sample
			float rgb2[3];
#pragma unroll
			for (int e = 0; e < 3; ++e) rgb2[e] = rgb2c[e] + warp_incl_scan(w * s.rgb[e], lane);
			if (valid) {
				float g[16];
#pragma unroll
				for (int k = 0; k < 16; ++k) g[k] = 0.f;
				float dterm[3];
#pragma unroll
				for (int e = 0; e < 3; ++e) {
					const float suffix = rgb_ray[e] - rgb2[e];
					g[e] = loss_scale * (w * lgg[e] * (s.rgb[e] * (1.0f - s.rgb[e])));
					dterm[e] = lgg[e] * (Ta * s.rgb[e] - suffix);
				}
				float dla = sum3_eigen(dterm[0], dterm[1], dterm[2]) + gws * (1.0f - ws);  // gradient.dot(T rgb - suffix) + mask term (:1829-1831)
				dla = (float)((double)dla / ((double)(1.0f - s.alpha) + 1e-5));  // "/ (1.0f - alpha + 1e-5)": fp64 divide (:1829-1832)
				float da_dE = 0, dE_dsdf = 0, dE_ds = 0, da_dP = 0, dP_ds = 0, dP_dic = 0, dE_dic = 0;
				if (!(s.p_div_c <= 0.0f || s.p_div_c >= 1.0f)) {
					const float P = __expf(s.inv_s * s.iter_cos * s.dt);
					const float E = __expf(-s.next_sdf * s.inv_s);
					dE_dsdf = -s.inv_s * E;
					dE_ds = -s.next_sdf * E;
					const float a = 1 + E, b = 1 + P * E, cc = (float)(1e-5 + (double)(1 / (1 + P * E)));  // fp64 sum (:1862)
					const float delta = a * (b * b) * (cc * cc);
					da_dE = -(P / delta - 1 / (a * a * cc));
					da_dP = -E / delta;
					dP_ds = P * s.iter_cos * s.dt;
					dP_dic = P * s.inv_s * s.dt;
					dE_dic = -s.inv_s * E * s.dt * 0.5f;
				}
				const float dl_dinvs = dla * (da_dE * dE_ds + da_dP * dP_ds);
				const float dl_dvar = dl_dinvs * s.inv_s * 10;
				const float dic_dcos = s.true_cos >= 0 ? 0.0f : 1.0f;
				// std::sqrt(float sum + 1e-6): the sum of squares is fp32, the offset and the root are fp64 (:1884)
				const float gn = (float)sqrt((double)(s.nrm[0] * s.nrm[0] + s.nrm[1] * s.nrm[1] + s.nrm[2] * s.nrm[2]) + 1e-6);
				const float gni = 1 - 1 / gn;
				const float dl_dnn = dla * (da_dE * dE_dic + dP_dic * da_dP) * dic_dcos;
				g[3] = loss_scale * (dla * da_dE * dE_dsdf);
				ek += (gn - 1.0f) * (gn - 1.0f);
#pragma unroll
				for (int e = 0; e < 3; ++e) {
					g[4 + e] = cfg.ek_loss_weight * 2 * cfg.loss_scale * gni * s.nrm[e];
					g[8 + e] = loss_scale * dl_dnn * dir[e];
				}
				g[7] = loss_scale * dl_dvar;
				__align__(16) __half gh[16];
#pragma unroll
				for (int k = 0; k < 16; ++k) gh[k] = __float2half_rn(g[k]);
				if (rescale) {
#pragma unroll
					for (int k = 0; k < 16; ++k) gh[k] = __float2half_rn(__half2float(gh[k]) * rollover_scale);
				}
				uint4* dst = reinterpret_cast<uint4*>(dloss_dout + (size_t)(compacted_base + j) * 16);
				dst[0] = reinterpret_cast<const uint4*>(gh)[0];
				dst[1] = reinterpret_cast<const uint4*>(gh)[1];
			}
			// carry to the next chunk
#pragma unroll
			for (int e = 0; e < 3; ++e) rgb2c[e] = __shfl_sync(kFull, rgb2[e], 31);
			T = __shfl_sync(kFull, Ta, 31);
		}
		ek = warp_sum(ek);
		if (lane == 0 && ek_loss_out) ek_loss_out[i] = ek / ((float)cn * n_rays_f);
	}
}

// fill_rollover / fill_rollover_and_rescale (call sites :3908-3916): pad [n_valid, n_target) with wrap-around copies
// of [0, n_valid).  The gradient is also rescaled by n_valid / n_target so the copies do not over-weight the batch: the loss
// pass has written the rows [0, n_valid) already rescaled, so the copies are plain copies.
__global__ void rollover_tail_kernel(uint32_t n_target, const uint32_t* __restrict__ counters, float* __restrict__ coords,
                                     __half* __restrict__ dloss) {
	const uint32_t nv = min(counters[2], n_target);
	if (nv == 0 || nv >= n_target) return;
	const size_t n_tail = (size_t)(n_target - nv);
	for (size_t r = blockIdx.x * (size_t)blockDim.x + threadIdx.x; r < n_tail * 16; r += (size_t)gridDim.x * blockDim.x) {
		const size_t row = nv + r / 16, k = r % 16;
		const size_t src = row % nv;
		dloss[row * 16 + k] = dloss[src * 16 + k];
		if (k < 7) coords[row * 7 + k] = coords[src * 7 + k];
	}
}

}  // namespace n2b

using namespace n2b;

extern "C" void neus2b_pcg32_seed(neus2b_pcg32* rng, uint64_t seed) {
	Pcg32 r;
	r.state = 0u;
	r.inc = (1ull << 1u) | 1u;  // default_rng_t{seed}: the constructor's default stream selector is 1 (src/testbed.cu:2077)
	r.next_uint();
	r.state += seed;
	r.next_uint();
	rng->state = r.state;
	rng->inc = r.inc;
}
extern "C" void neus2b_pcg32_advance(neus2b_pcg32* rng, uint64_t delta) {
	Pcg32 r{rng->state, rng->inc};
	r.advance(delta);
	rng->state = r.state;
}

static int check_ws(const neus2b_ray_workspace* ws) {
	if (!ws || !ws->d_ray_indices || !ws->d_rays || !ws->d_numsteps || !ws->d_coords || !ws->d_counters || !ws->d_scan_tmp ||
	    !ws->d_ray_tmp || ws->max_rays == 0 || ws->max_samples == 0)
		return NEUS2B_E_INVALID;
	return NEUS2B_OK;
}

extern "C" int neus2b_generate_samples(const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays, const uint32_t* d_n_rays,
                                       uint32_t n_rays_total, neus2b_pcg32 rng, const uint8_t* d_bitfield, neus2b_ray_workspace* ws,
                                       neus2b_stream_t stream) {
	if (!ds || !cfg || !d_bitfield || check_ws(ws)) return NEUS2B_E_INVALID;
	if (n_rays == 0 || n_rays > ws->max_rays || ds->n_images == 0) return NEUS2B_E_INVALID;
	if (n_rays > kScanMaxKeys) return NEUS2B_E_TOO_LARGE;
	N2B_CHECK_CUDA(cudaMemsetAsync(ws->d_counters, 0, 8 * sizeof(uint32_t), stream));
	Pcg32 r{rng.state, rng.inc};
	// (the hit list borrows d_ray_indices, which the emit pass fills afterwards; its length is counter 6)
	ray_setup_kernel<<<min(div_up(n_rays, 256), (uint32_t)kSMs * 8u), 256, 0, stream>>>(*ds, *cfg, n_rays, d_n_rays, n_rays_total, ws->d_n_rays_total, r,
	                                                                          (RayTmp*)ws->d_ray_tmp, ws->d_scan_tmp, ws->d_occupied_bounds,
	                                                                          ws->d_ray_indices, ws->d_counters + 6);
	N2B_CHECK_LAUNCH();
	count_steps_kernel<<<min(div_up(n_rays, 4), (uint32_t)kSMs * 16u), 128, 0, stream>>>(*cfg, d_bitfield, (RayTmp*)ws->d_ray_tmp, ws->d_scan_tmp,
	                                                                           ws->d_march_masks, ws->d_occupied_bounds, ws->d_ray_indices,
	                                                                           ws->d_counters + 6);
	N2B_CHECK_LAUNCH();
	scan_kernel<<<64, 1024, 0, stream>>>(n_rays, d_n_rays, ws->d_scan_tmp);
	N2B_CHECK_LAUNCH();
	emit_samples_kernel<<<min(div_up(n_rays, 4), (uint32_t)kSMs * 16u), 128, 0, stream>>>(*cfg, n_rays, d_n_rays, ws->max_samples, ws->d_prev_samples, d_bitfield, (const RayTmp*)ws->d_ray_tmp,
	                                                             ws->d_scan_tmp, ws->d_ray_indices, ws->d_rays, ws->d_numsteps,
	                                                             ws->d_coords, ws->d_counters, ws->d_march_masks);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

static int loss_after_composite(const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays, const uint32_t* d_n_rays, uint32_t n_rays_total,
                                Pcg32 r, uint32_t max_compacted, const uint16_t* d_mlp_out, neus2b_ray_workspace* ws, float* d_coords_out,
                                uint16_t* d_dloss_dout, float* d_loss, float* d_ek_loss, int rollover, cudaStream_t stream);

extern "C" int neus2b_compute_loss(const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays, const uint32_t* d_n_rays,
                                   uint32_t n_rays_total, neus2b_pcg32 rng, uint32_t max_compacted, const uint16_t* d_mlp_out,
                                   neus2b_ray_workspace* ws, float* d_coords_out, uint16_t* d_dloss_dout, float* d_loss, float* d_ek_loss,
                                   int rollover, neus2b_stream_t stream) {
	if (!ds || !cfg || !d_mlp_out || !d_coords_out || !d_dloss_dout || check_ws(ws)) return NEUS2B_E_INVALID;
	if (n_rays == 0 || n_rays > ws->max_rays || max_compacted == 0) return NEUS2B_E_INVALID;
	if (n_rays > kScanMaxKeys) return NEUS2B_E_TOO_LARGE;
	if (((uintptr_t)d_mlp_out | (uintptr_t)d_dloss_dout) & 15u) return NEUS2B_E_INVALID;
	Pcg32 r{rng.state, rng.inc};
	const uint32_t ray_ctas = min(div_up(n_rays, 4), (uint32_t)kSMs * 16u);  // 4 warps per CTA, one warp per ray, grid-stride
	composite_kernel<<<ray_ctas, 128, 0, stream>>>(*cfg, ws->d_counters, (const __half*)d_mlp_out, ws->d_numsteps, ws->d_coords,
	                                               (CompTmp*)ws->d_ray_tmp, ws->d_scan_tmp, n_rays, 0u, 0xffffffffu, 0xffffffffu, nullptr, nullptr, nullptr);
	N2B_CHECK_LAUNCH();
	return loss_after_composite(ds, cfg, n_rays, d_n_rays, n_rays_total, r, max_compacted, d_mlp_out, ws, d_coords_out, d_dloss_dout, d_loss, d_ek_loss,
	                            rollover, stream);
}

// Compaction offsets, loss pass and roll-over on the per-ray records the compositing pass left behind.
static int loss_after_composite(const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays, const uint32_t* d_n_rays, uint32_t n_rays_total,
                                Pcg32 r, uint32_t max_compacted, const uint16_t* d_mlp_out, neus2b_ray_workspace* ws, float* d_coords_out,
                                uint16_t* d_dloss_dout, float* d_loss, float* d_ek_loss, int rollover, cudaStream_t stream) {
	const uint32_t ray_ctas = min(div_up(n_rays, 4), (uint32_t)kSMs * 16u);
	scan_kernel<<<64, 1024, 0, stream>>>(n_rays, ws->d_counters, ws->d_scan_tmp);
	N2B_CHECK_LAUNCH();
	loss_kernel<<<ray_ctas, 128, 0, stream>>>(*ds, *cfg, n_rays, d_n_rays, n_rays_total, ws->d_n_rays_total, r, max_compacted, rollover,
	                                          ws->d_counters, (const __half*)d_mlp_out, ws->d_ray_indices, ws->d_numsteps, ws->d_coords,
	                                          (const CompTmp*)ws->d_ray_tmp, ws->d_scan_tmp, d_coords_out, (__half*)d_dloss_dout, d_loss,
	                                          d_ek_loss);
	N2B_CHECK_LAUNCH();
	if (rollover) {
		rollover_tail_kernel<<<2 * kSMs, 256, 0, stream>>>(max_compacted, ws->d_counters, d_coords_out, (__half*)d_dloss_dout);
		N2B_CHECK_LAUNCH();
	}
	return NEUS2B_OK;
}

// The network pass over the samples and the loss pass as one call that evaluates the network only where its output is
// used.  The reference evaluates every sample the generator drew and then keeps, per ray, the samples in front of the point
// where the ray turns opaque (transmittance below 1e-4): half to five sixths of the evaluations are thrown away.  Here the
// rays are evaluated in windows of consecutive samples: the first window_ends[0] samples of every ray, then samples
// [window_ends[0], window_ends[1]) of the rays that are still transparent, ..., finally the rest of those that remain.
// Between windows the compositing pass continues each ray's record and appends the rows of the ray's next window to the
// list that the fused forward kernel works through next: two launches per window.
// Everything stays on the stream: no host round trip.  The per-ray records, the compacted batch and the loss gradient are
// those of the full pass (every kept sample is evaluated by the same per-sample arithmetic); rows of d_mlp_out behind a
// ray's last evaluated sample keep whatever they held.
extern "C" int neus2b_forward_compute_loss(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, const neus2b_motion* motion,
                                           const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays, const uint32_t* d_n_rays,
                                           uint32_t n_rays_total, neus2b_pcg32 rng, uint32_t max_compacted, neus2b_ray_workspace* ws,
                                           const uint32_t* window_ends, uint32_t n_windows, uint16_t* d_mlp_out, float* d_coords_out,
                                           uint16_t* d_dloss_dout, float* d_loss, float* d_ek_loss, int rollover, neus2b_stream_t stream) {
	if (!desc || !d_params || !ds || !cfg || !d_mlp_out || !d_coords_out || !d_dloss_dout || check_ws(ws)) return NEUS2B_E_INVALID;
	if (n_rays == 0 || n_rays > ws->max_rays || max_compacted == 0) return NEUS2B_E_INVALID;
	if (n_rays > kScanMaxKeys) return NEUS2B_E_TOO_LARGE;
	if (((uintptr_t)d_mlp_out | (uintptr_t)d_dloss_dout) & 15u) return NEUS2B_E_INVALID;
	if (n_windows > NEUS2B_MAX_FORWARD_WINDOWS || (n_windows && !window_ends)) return NEUS2B_E_INVALID;
	for (uint32_t w = 0; w < n_windows; ++w)
		if (window_ends[w] == 0 || (w && window_ends[w] <= window_ends[w - 1])) return NEUS2B_E_INVALID;
	if (n_windows == 0) {  // the reference's order: everything, then the loss pass
		int rc = neus2b_neus_forward_moved(desc, d_params, sdf_bias, ws->max_samples, ws->d_counters + 4, ws->d_coords, motion, d_mlp_out, stream);
		if (rc) return rc;
		return neus2b_compute_loss(ds, cfg, n_rays, d_n_rays, n_rays_total, rng, max_compacted, d_mlp_out, ws, d_coords_out, d_dloss_dout, d_loss,
		                           d_ek_loss, rollover, stream);
	}
	if (!ws->d_window_list || !ws->d_window_lens) return NEUS2B_E_INVALID;
	Pcg32 r{rng.state, rng.inc};
	const uint32_t ray_ctas = min(div_up(n_rays, 4), (uint32_t)kSMs * 16u);
	uint32_t* lens = ws->d_window_lens;        // one list length per window
	uint32_t* evaluated = ws->d_counters + 5;  // (cleared by the generator with the other counters)
	N2B_CHECK_CUDA(cudaMemsetAsync(lens, 0, sizeof(uint32_t) * (NEUS2B_MAX_FORWARD_WINDOWS + 2), stream));
	window_first_kernel<<<ray_ctas, 128, 0, stream>>>(ws->d_counters, ws->d_numsteps, window_ends[0], ws->d_window_list, lens, evaluated);
	N2B_CHECK_LAUNCH();
	uint32_t lo = 0;
	for (uint32_t w = 0; w <= n_windows; ++w) {
		const uint32_t hi = w < n_windows ? window_ends[w] : 0xffffffffu;
		const uint32_t next_hi = w + 1 < n_windows ? window_ends[w + 1] : 0xffffffffu;
		int rc = neus2b_neus_forward_indexed(desc, d_params, sdf_bias, ws->max_samples, lens + w, ws->d_window_list, ws->d_coords, motion, d_mlp_out, stream);
		if (rc) return rc;
		const bool more = w < n_windows;
		composite_kernel<<<ray_ctas, 128, 0, stream>>>(*cfg, ws->d_counters, (const __half*)d_mlp_out, ws->d_numsteps, ws->d_coords,
		                                               (CompTmp*)ws->d_ray_tmp, ws->d_scan_tmp, n_rays, lo, hi, next_hi,
		                                               more ? ws->d_window_list : nullptr, more ? lens + w + 1 : nullptr, more ? evaluated : nullptr);
		N2B_CHECK_LAUNCH();
		lo = hi;
	}
	return loss_after_composite(ds, cfg, n_rays, d_n_rays, n_rays_total, r, max_compacted, d_mlp_out, ws, d_coords_out, d_dloss_dout, d_loss, d_ek_loss,
	                            rollover, stream);
}

// ------------------------------------------------------------------------------------------------
// Sample generation for callers that cannot allocate.
//
// Some hosts of this library own every byte of device memory themselves: a renderer or trainer that carved the whole
// GPU into its own arena at start-up, or a process that is not allowed to call cudaMalloc once it is running because
// the call synchronises the device and can fail late.  Such a caller can hand over buffers for inputs and outputs,
// but it has no pool to take the generator's scratch from (the per-ray staging records and the prefix-sum keys).  For
// them the scratch lives in the two file-scope device arrays below.  Every GPU that loads the library holds them
// (about 2.5 MiB) until the process exits, and the ray count per call is limited to NEUS2B_STATIC_MAX_RAYS.
//
// The arrays are shared by every call on a device: two calls whose kernels overlap on the GPU (different streams,
// different threads) race on them, so issue calls to this entry point one after the other on one stream.  Nothing in
// the scratch has to start at zero: each element a kernel reads was written earlier in the same call, so whatever the
// previous call left behind is harmless.
namespace {
constexpr uint32_t kStaticMaxRays = 65536;  // == NEUS2B_STATIC_MAX_RAYS
static __device__ __align__(256) uint64_t g_static_scan[kStaticMaxRays + 1024];
static __device__ __align__(256) float g_static_ray_tmp[(size_t)kStaticMaxRays * 8];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
uint64_t* g_static_scan_ptr[kMaxDevices] = {};
float* g_static_ray_tmp_ptr[kMaxDevices] = {};

// In host code the array names above are host-side stand-ins, not device addresses; the addresses the kernels need
// come from cudaGetSymbolAddress, looked up once per device with that device current.
int static_scratch(uint64_t** scan, float** ray_tmp) {
	int dev = -1;
	N2B_CHECK_CUDA(cudaGetDevice(&dev));
	if (dev < 0 || dev >= kMaxDevices) return NEUS2B_E_UNSUPPORTED;
	std::lock_guard<std::mutex> lock(g_static_mutex);
	if (!g_static_scan_ptr[dev]) {
		void *a = nullptr, *b = nullptr;
		N2B_CHECK_CUDA(cudaGetSymbolAddress(&a, g_static_scan));
		N2B_CHECK_CUDA(cudaGetSymbolAddress(&b, g_static_ray_tmp));
		g_static_scan_ptr[dev] = (uint64_t*)a;
		g_static_ray_tmp_ptr[dev] = (float*)b;
	}
	*scan = g_static_scan_ptr[dev];
	*ray_tmp = g_static_ray_tmp_ptr[dev];
	return NEUS2B_OK;
}
}  // namespace

extern "C" int neus2b_generate_samples_static(const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays,
                                              const uint32_t* d_n_rays, uint32_t n_rays_total, neus2b_pcg32 rng, const uint8_t* d_bitfield,
                                              uint32_t max_samples, uint32_t* d_ray_indices, float* d_rays, uint32_t* d_numsteps,
                                              float* d_coords, uint32_t* d_counters, neus2b_stream_t stream) {
	if (!ds || !cfg || !d_bitfield || !d_ray_indices || !d_rays || !d_numsteps || !d_coords || !d_counters) return NEUS2B_E_INVALID;
	if (n_rays == 0 || max_samples == 0 || ds->n_images == 0) return NEUS2B_E_INVALID;
	if (n_rays > kStaticMaxRays) return NEUS2B_E_TOO_LARGE;  // the built-in scratch holds NEUS2B_STATIC_MAX_RAYS rays
	uint64_t* scan = nullptr;
	float* ray_tmp = nullptr;
	int rc = static_scratch(&scan, &ray_tmp);
	if (rc) return rc;
	N2B_CHECK_CUDA(cudaMemsetAsync(d_counters, 0, 8 * sizeof(uint32_t), stream));
	Pcg32 r{rng.state, rng.inc};
	ray_setup_kernel<<<min(div_up(n_rays, 256), (uint32_t)kSMs * 8u), 256, 0, stream>>>(*ds, *cfg, n_rays, d_n_rays, n_rays_total, nullptr, r, (RayTmp*)ray_tmp, scan,
	                                                                          nullptr, d_ray_indices, d_counters + 6);
	N2B_CHECK_LAUNCH();
	count_steps_kernel<<<min(div_up(n_rays, 4), (uint32_t)kSMs * 16u), 128, 0, stream>>>(*cfg, d_bitfield, (RayTmp*)ray_tmp, scan, nullptr, nullptr, d_ray_indices,
	                                                                           d_counters + 6);
	N2B_CHECK_LAUNCH();
	scan_kernel<<<64, 1024, 0, stream>>>(n_rays, d_n_rays, scan);
	N2B_CHECK_LAUNCH();
	emit_samples_kernel<<<min(div_up(n_rays, 4), (uint32_t)kSMs * 16u), 128, 0, stream>>>(*cfg, n_rays, d_n_rays, max_samples, nullptr, d_bitfield, (const RayTmp*)ray_tmp, scan,
	                                                             d_ray_indices, d_rays, d_numsteps, d_coords, d_counters, nullptr);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}
