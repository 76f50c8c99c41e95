// Fused NeuS graph kernels (NerfNetwork::forward_impl / backward_impl / sdf of the reference,
// include/neural-graphics-primitives/nerf_network.h:132-709) for sm_100a.
//
// One warp owns a tile of 16 samples from the first gather to the last gradient scatter; nothing but the
// 28-byte coordinate, the 32-byte output / output-gradient and the grid entries ever touches global memory.
//   * encoding: lane = (sample s = lane & 15, level parity = lane >> 4); a lane walks levels parity, parity+2, ...
//     so the 16 lanes of a half-warp gather the same level for 16 consecutive samples of a ray;
//   * MLPs: mma.sync m16n8k16 on the warp's 16-row tiles in shared memory, weights resident in shared memory for the
//     lifetime of the (persistent) CTA;
//   * training: forward and backward run back to back on the same tile (the loss gradient is known before the
//     forward pass, src/testbed_nerf.cu:3846-3932), weight gradients accumulate in shared memory and are flushed
//     once per CTA, grid gradients go out as one packed fp16x2 reduction per corner with the first- and second-order
//     terms merged.
// Internal column order of the SDF-net input is [encoding 0..31 | xyz-0.5 32..34 | zero 35..47] (the weight columns are
// permuted to match while they are staged), so the per-level feature pair is 4-byte aligned.
#include "common.cuh"
#include "fused_common.cuh"
#include "delta.cuh"
#include "mma_tile.cuh"

namespace n2b {

constexpr int kWarps = 8;
constexpr int LD48 = 56;  // halves per row of a 48-wide tile
constexpr int LD64 = 72;  // halves per row of a 64-wide tile
constexpr int LD16 = 24;  // halves per row of a 16-wide tile
constexpr int A56 = 16 * LD48;
constexpr int B72 = 16 * LD64;
constexpr int C24 = 16 * LD16;
// fp32 weight-gradient accumulators: row strides = 4 (mod 8) for conflict-free accumulation
constexpr int GLD48 = 52;
constexpr int GLD64 = 68;

struct WeightsSmem {
	__half W1s[64 * LD48];
	__half W2s[16 * LD64];
	__half W1c[64 * LD48];
	__half W2c[64 * LD64];
	__half W3c[16 * LD64];
};

struct GradSmem {
	float W1s[64 * GLD48];
	float W2s[16 * GLD64];
	float W1c[64 * GLD48];
	float W2c[64 * GLD64];
	float W3c[16 * GLD64];
};

template <int MODE>
struct WarpTiles;
template <>
struct WarpTiles<MODE_FWD> {
	__half a0[A56], a1[A56];  // Zs -> Gz ; Zc
	__half b0[B72], b1[B72];  // Hs -> H1 ; S -> H2
	__half c0[C24];           // colour-net output
	__device__ __half* Zs() { return a0; }
	__device__ __half* Gz() { return a0; }
	__device__ __half* Zc() { return a1; }
	__device__ __half* Hs() { return b0; }
	__device__ __half* H1() { return b0; }
	__device__ __half* S() { return b1; }
	__device__ __half* H2() { return b1; }
	__device__ __half* Y() { return c0; }
};
template <>
struct WarpTiles<MODE_SDF> {
	__half a0[A56];
	__half b0[B72];
	__half c0[C24];
	__device__ __half* Zs() { return a0; }
	__device__ __half* Hs() { return b0; }
	__device__ __half* Y() { return c0; }
};
template <>
struct WarpTiles<MODE_TRAIN> {
	__half a0[A56], a1[A56], a2[A56], a3[A56];  // Zs ; Gz ; Zc -> dZs ; dZc -> U
	__half b0[B72], b1[B72], b2[B72], b3[B72];  // Hs ; S -> H1 -> S ; H2 -> dH1 ; dH2 -> dHs -> T
	__half c0[C24];                             // dY3 -> dYs -> e0
	__device__ __half* Zs() { return a0; }
	__device__ __half* Gz() { return a1; }
	__device__ __half* Zc() { return a2; }
	__device__ __half* dZs() { return a2; }
	__device__ __half* dZc() { return a3; }
	__device__ __half* U() { return a3; }
	__device__ __half* Hs() { return b0; }
	__device__ __half* S() { return b1; }
	__device__ __half* H1() { return b1; }
	__device__ __half* H2() { return b2; }
	__device__ __half* dH1() { return b2; }
	__device__ __half* dH2() { return b3; }
	__device__ __half* dHs() { return b3; }
	__device__ __half* T() { return b3; }
	__device__ __half* Y() { return c0; }
};

template <int MODE>
struct SmemLayout {
	WeightsSmem w;
	WarpTiles<MODE> t[kWarps];
};
template <>
struct SmemLayout<MODE_TRAIN> {
	WeightsSmem w;
	GradSmem g;
	WarpTiles<MODE_TRAIN> t[kWarps];
};

__device__ void stage_weights(WeightsSmem& w, const __half* params, int tid, int nthreads) {
	for (int e = tid; e < 64 * 48; e += nthreads) {
		const int r = e / 48, k = e % 48;
		w.W1s[r * LD48 + k] = params[NEUS2B_SDF_W1 + r * 48 + sdf_orig_col(k)];
		w.W1c[r * LD48 + k] = params[NEUS2B_RGB_W1 + e];
	}
	for (int e = tid; e < 16 * 64; e += nthreads) {
		const int r = e / 64, k = e % 64;
		w.W2s[r * LD64 + k] = params[NEUS2B_SDF_W2 + e];
		w.W3c[r * LD64 + k] = params[NEUS2B_RGB_W3 + e];
	}
	for (int e = tid; e < 64 * 64; e += nthreads) {
		const int r = e / 64, k = e % 64;
		w.W2c[r * LD64 + k] = params[NEUS2B_RGB_W2 + e];
	}
}

// Encoding of the warp's 16 samples into columns [0, 32) of Zs.  With JAC the lane also keeps, per level it owns,
// J[d][f] = d enc_f / d x_d (6 floats): the normal (d sdf/dx), and in the backward pass the second-order term
// dL/d(d sdf/d enc) = J v, come from it without touching the grid again.
template <bool JAC>
__device__ __forceinline__ void encode_tile(const GridLevels& lv, const __half* grid, const float* x, int s, int hl, __half* Zs,
                                            float (&J)[8][6]) {
#pragma unroll
	for (int j = 0; j < 8; ++j) {
		const uint32_t l = 2 * j + hl;
		__half2 feat = __floats2half2_rn(0.f, 0.f);
		if (JAC) {
#pragma unroll
			for (int e = 0; e < 6; ++e) J[j][e] = 0.f;
		}
		if (l < lv.n_active) {
			const LevelGeom g = level_geom(lv, l, x);
			__half2 th[8];
#pragma unroll
			for (uint32_t k = 0; k < 8; ++k) th[k] = ldg_h2(grid, geom_index(g, k));
			const float scale = lv.scale[l];
			float a0 = 0.f, a1 = 0.f;
#pragma unroll
			for (uint32_t k = 0; k < 8; ++k) {
				const uint32_t bx = k & 1u, by = (k >> 1) & 1u, bz = (k >> 2) & 1u;
				const float2 t = __half22float2(th[k]);
				const float w = g.ax[bx] * g.ay[by] * g.az[bz];
				a0 = __fmaf_rn(w, t.x, a0);
				a1 = __fmaf_rn(w, t.y, a1);
				if (JAC) {
					const float dwx = (bx ? scale : -scale) * g.ay[by] * g.az[bz];
					const float dwy = (by ? scale : -scale) * g.ax[bx] * g.az[bz];
					const float dwz = (bz ? scale : -scale) * g.ax[bx] * g.ay[by];
					J[j][0] = __fmaf_rn(dwx, t.x, J[j][0]);
					J[j][1] = __fmaf_rn(dwx, t.y, J[j][1]);
					J[j][2] = __fmaf_rn(dwy, t.x, J[j][2]);
					J[j][3] = __fmaf_rn(dwy, t.y, J[j][3]);
					J[j][4] = __fmaf_rn(dwz, t.x, J[j][4]);
					J[j][5] = __fmaf_rn(dwz, t.y, J[j][5]);
				}
			}
			feat = __floats2half2_rn(a0, a1);
		}
		*reinterpret_cast<__half2*>(Zs + s * LD48 + 2 * l) = feat;
	}
}

// S[r][c] = Hs[r][c] > 0 ? W2s[0][c] : 0   (gradient of y0 w.r.t. the hidden layer)
__device__ __forceinline__ void build_S(const __half* Hs, const __half* W2s_row0, __half* S, int lane) {
	const __half2 zero = __floats2half2_rn(0.f, 0.f);
	const int r = lane >> 1, c0 = (lane & 1) * 32;
#pragma unroll
	for (int c = 0; c < 32; c += 2) {
		const __half2 h = *reinterpret_cast<const __half2*>(Hs + r * LD64 + c0 + c);
		const __half2 w = *reinterpret_cast<const __half2*>(W2s_row0 + c0 + c);
		*reinterpret_cast<__half2*>(S + r * LD64 + c0 + c) = __hmul2(w, __hgt2(h, zero));
	}
}

template <int MODE>
__global__ void __launch_bounds__(kWarps * 32, MODE == MODE_TRAIN ? 1 : 2) neus_kernel(const NeusArgs a) {
	extern __shared__ __align__(16) unsigned char smem_raw[];
	SmemLayout<MODE>& sm = *reinterpret_cast<SmemLayout<MODE>*>(smem_raw);
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const __half* grid = a.params + NEUS2B_GRID_OFF;

	stage_weights(sm.w, a.params, tid, blockDim.x);
	if constexpr (MODE == MODE_TRAIN) {
		float* g = reinterpret_cast<float*>(&sm.g);
		for (int e = tid; e < (int)(sizeof(GradSmem) / 4); e += blockDim.x) g[e] = 0.f;
	}
	{  // zero the warp's tiles once: padding columns are never written afterwards
		uint32_t* t = reinterpret_cast<uint32_t*>(&sm.t[warp]);
		for (int e = lane; e < (int)(sizeof(WarpTiles<MODE>) / 4); e += 32) t[e] = 0u;
	}
	__syncthreads();

	WarpTiles<MODE>& T = sm.t[warp];
	const uint32_t n = a.d_n ? min(*a.d_n, a.n) : a.n;
	const uint32_t n_tiles = (n + 15u) / 16u;
	const int s = lane & 15, hl = lane >> 4;
	const __half variance = a.params[NEUS2B_GRID_OFF + (size_t)a.grid_entries * 2];
	const float bias = __half2float(__float2half_rn(a.sdf_bias));
	float var_grad = 0.f;

	for (uint32_t tile = blockIdx.x * kWarps + warp; tile < n_tiles; tile += gridDim.x * kWarps) {
		const uint32_t i = tile * 16u + (uint32_t)s;
		const bool valid = i < n;
		float x[3] = {0.5f, 0.5f, 0.5f}, dir[3] = {0.5f, 0.5f, 0.5f};
		if (valid) {
			const float* c = a.coords + (size_t)i * a.coord_stride;
			x[0] = c[0];
			x[1] = c[1];
			x[2] = c[2];
			if constexpr (MODE != MODE_SDF) {
				dir[0] = c[a.dir_offset];
				dir[1] = c[a.dir_offset + 1];
				dir[2] = c[a.dir_offset + 2];
			}
		}
		if (a.delta) {  // dynamic sequences: the frame's rigid motion comes first (only the SDF query supports it on this path)
			const RigidMotion rm = load_rigid_motion(a.delta);
			move_sample(rm.R, rm.t, a.first_frame_offset, x, dir);
		}
		// ---- F1: encoding -> Zs[:, 0:32], xyz - 0.5 -> Zs[:, 32:35]
		float J[8][6];
		encode_tile<MODE != MODE_SDF>(a.lv, grid, x, s, hl, T.Zs(), J);
		if (hl == 0) {
#pragma unroll
			for (int e = 0; e < 3; ++e)
				T.Zs()[s * LD48 + 32 + e] = __float2half_rn(__half2float(__float2half_rn(x[e])) - 0.5f);
		} else if constexpr (MODE == MODE_FWD) {
			// Zs shares its buffer with Gz: clear the padding columns the previous tile's Gz filled
#pragma unroll
			for (int e = 35; e < 48; ++e) T.Zs()[s * LD48 + e] = __float2half_rn(0.f);
		}
		__syncwarp();
		// ---- F2: Hs = relu(Zs W1s^T)
		{
			float acc[8][4];
			zero_acc<8>(acc);
			warp_gemm_nt<64, 48>(acc, T.Zs(), LD48, sm.w.W1s, LD48, lane);
			store_acc_half<64, true>(acc, T.Hs(), LD64, lane);
		}
		__syncwarp();
		if constexpr (MODE == MODE_SDF) {
			float acc[2][4];
			zero_acc<2>(acc);
			warp_gemm_nt<16, 64>(acc, T.Hs(), LD64, sm.w.W2s, LD64, lane);
			store_acc_half<16, false>(acc, T.Y(), LD16, lane);
			__syncwarp();
			if (hl == 0 && valid) a.sdf_out[i] = __float2half_rn(__half2float(T.Y()[s * LD16]) + bias);
			__syncwarp();
			continue;
		} else {
			// ---- F3: Ys = Hs W2s^T -> Zc[:, 0:16];  F4: S
			{
				float acc[2][4];
				zero_acc<2>(acc);
				warp_gemm_nt<16, 64>(acc, T.Hs(), LD64, sm.w.W2s, LD64, lane);
				store_acc_half<16, false>(acc, T.Zc(), LD48, lane);
			}
			build_S(T.Hs(), sm.w.W2s, T.S(), lane);
			__syncwarp();
			// ---- F5: Gz = S W1s  (d y0 / d z)
			{
				float acc[6][4];
				zero_acc<6>(acc);
				warp_gemm_nn<48, 64>(acc, T.S(), LD64, sm.w.W1s, LD48, lane);
				store_acc_half<48, false>(acc, T.Gz(), LD48, lane);
			}
			__syncwarp();
			// ---- F6: normal = Gz[xyz] + (d enc / d x)^T Gz[enc]
			float nrm[3] = {0.f, 0.f, 0.f};
#pragma unroll
			for (int j = 0; j < 8; ++j) {
				const uint32_t l = 2 * j + hl;
				const float2 ge = __half22float2(*reinterpret_cast<const __half2*>(T.Gz() + s * LD48 + 2 * l));
#pragma unroll
				for (int e = 0; e < 3; ++e) nrm[e] = __fmaf_rn(J[j][2 * e], ge.x, __fmaf_rn(J[j][2 * e + 1], ge.y, nrm[e]));
			}
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				nrm[e] += __shfl_xor_sync(0xffffffffu, nrm[e], 16);
				nrm[e] += __half2float(T.Gz()[s * LD48 + 32 + e]);
			}
			if (hl == 0) {
#pragma unroll
				for (int e = 0; e < 3; ++e) {
					T.Zc()[s * LD48 + 32 + e] = __float2half_rn(x[e]);
					T.Zc()[s * LD48 + 35 + e] = __float2half_rn(nrm[e]);
				}
				// padding columns: the training layout reuses this buffer for dZs
#pragma unroll
				for (int k = 38; k < 48; k += 2) *reinterpret_cast<__half2*>(T.Zc() + s * LD48 + k) = __floats2half2_rn(0.f, 0.f);
			} else {
				float sh[16];
				sh4_eval(dir, sh);
#pragma unroll
				for (int k = 0; k < 8; ++k)
					*reinterpret_cast<__half2*>(T.Zc() + s * LD48 + 16 + 2 * k) = __floats2half2_rn(sh[2 * k], sh[2 * k + 1]);
			}
			__syncwarp();
			// ---- F7: colour net
			{
				float acc[8][4];
				zero_acc<8>(acc);
				warp_gemm_nt<64, 48>(acc, T.Zc(), LD48, sm.w.W1c, LD48, lane);
				__syncwarp();  // S (train: same buffer as H1) has been consumed by every lane
				store_acc_half<64, true>(acc, T.H1(), LD64, lane);
				__syncwarp();
				zero_acc<8>(acc);
				warp_gemm_nt<64, 64>(acc, T.H1(), LD64, sm.w.W2c, LD64, lane);
				__syncwarp();
				store_acc_half<64, true>(acc, T.H2(), LD64, lane);
			}
			__syncwarp();
			if constexpr (MODE == MODE_FWD) {
				float acc[2][4];
				zero_acc<2>(acc);
				warp_gemm_nt<16, 64>(acc, T.H2(), LD64, sm.w.W3c, LD64, lane);
				store_acc_half<16, false>(acc, T.Y(), LD16, lane);
				__syncwarp();
				if (hl == 0 && valid) {
					__align__(16) __half o[16];
#pragma unroll
					for (int k = 0; k < 16; ++k) o[k] = T.Y()[s * LD16 + k];
					o[3] = __float2half_rn(__half2float(T.Zc()[s * LD48]) + bias);
#pragma unroll
					for (int e = 0; e < 3; ++e) {
						o[4 + e] = __float2half_rn(nrm[e]);
						o[8 + e] = __float2half_rn(dir[e]);
					}
					o[7] = variance;
					uint4* dst = reinterpret_cast<uint4*>(a.out + (size_t)i * 16);
					dst[0] = reinterpret_cast<const uint4*>(o)[0];
					dst[1] = reinterpret_cast<const uint4*>(o)[1];
				}
				__syncwarp();
			}
		}
		if constexpr (MODE == MODE_TRAIN) {
			// ---- B1: colour-net output gradient: rows 0-2 of dL_dout only (nerf_network.h:331-340)
			__align__(16) __half g[16];
			if (hl == 0) {
				if (valid) {
					const uint4* src = reinterpret_cast<const uint4*>(a.dL_dout + (size_t)i * 16);
					reinterpret_cast<uint4*>(g)[0] = __ldg(src);
					reinterpret_cast<uint4*>(g)[1] = __ldg(src + 1);
				} else {
#pragma unroll
					for (int k = 0; k < 16; ++k) g[k] = __float2half_rn(0.f);
				}
#pragma unroll
				for (int k = 0; k < 16; ++k) T.Y()[s * LD16 + k] = k < 3 ? g[k] : __float2half_rn(0.f);
			}
			__syncwarp();
			{
				float acc[8][4];
				zero_acc<8>(acc);
				warp_wgrad_mtile<64>(acc, T.Y(), LD16, 0, T.H2(), LD64, lane);
				smem_accumulate<64>(acc, sm.g.W3c, GLD64, 0, lane);
				zero_acc<8>(acc);
				warp_gemm_nn<64, 16>(acc, T.Y(), LD16, sm.w.W3c, LD64, lane);
				store_acc_half_masked<64>(acc, T.H2(), LD64, T.dH2(), LD64, lane);
			}
			__syncwarp();
			// ---- B2
			{
				float acc[8][4];
#pragma unroll 1
				for (int mt = 0; mt < 4; ++mt) {
					zero_acc<8>(acc);
					warp_wgrad_mtile<64>(acc, T.dH2(), LD64, mt * 16, T.H1(), LD64, lane);
					smem_accumulate<64>(acc, sm.g.W2c, GLD64, mt * 16, lane);
				}
				zero_acc<8>(acc);
				warp_gemm_nn<64, 64>(acc, T.dH2(), LD64, sm.w.W2c, LD64, lane);
				__syncwarp();  // H2 is overwritten by dH1 below; its last reader was B1
				store_acc_half_masked<64>(acc, T.H1(), LD64, T.dH1(), LD64, lane);
			}
			__syncwarp();
			// ---- B3
			{
				float acc[6][4];
#pragma unroll 1
				for (int mt = 0; mt < 4; ++mt) {
					zero_acc<6>(acc);
					warp_wgrad_mtile<48>(acc, T.dH1(), LD64, mt * 16, T.Zc(), LD48, lane);
					smem_accumulate<48>(acc, sm.g.W1c, GLD48, mt * 16, lane);
				}
				zero_acc<6>(acc);
				warp_gemm_nn<48, 64>(acc, T.dH1(), LD64, sm.w.W1c, LD48, lane);
				store_acc_half<48, false>(acc, T.dZc(), LD48, lane);
			}
			__syncwarp();
			// ---- B4: SDF-net output gradient = colour-net input gradient rows 0-15, + dL/dsdf on row 0 (:388-395)
			float v[3] = {0.f, 0.f, 0.f};
			if (hl == 0) {
#pragma unroll
				for (int k = 0; k < 16; ++k) T.Y()[s * LD16 + k] = T.dZc()[s * LD48 + k];
				T.Y()[s * LD16] = __hadd(T.dZc()[s * LD48], g[3]);
#pragma unroll
				for (int e = 0; e < 3; ++e)
					v[e] = __half2float(T.dZc()[s * LD48 + 35 + e]) + __half2float(g[4 + e]) / a.batch_size + __half2float(g[8 + e]);
				var_grad += __half2float(g[7]);
			}
#pragma unroll
			for (int e = 0; e < 3; ++e) v[e] = __shfl_sync(0xffffffffu, v[e], s);
			__syncwarp();
			{
				float acc[8][4];
				zero_acc<8>(acc);
				warp_wgrad_mtile<64>(acc, T.Y(), LD16, 0, T.Hs(), LD64, lane);
				smem_accumulate<64>(acc, sm.g.W2s, GLD64, 0, lane);
				zero_acc<8>(acc);
				warp_gemm_nn<64, 16>(acc, T.Y(), LD16, sm.w.W2s, LD64, lane);
				store_acc_half_masked<64>(acc, T.Hs(), LD64, T.dHs(), LD64, lane);
			}
			__syncwarp();
			// ---- B5
			{
				float acc[6][4];
#pragma unroll 1
				for (int mt = 0; mt < 4; ++mt) {
					zero_acc<6>(acc);
					warp_wgrad_mtile<48>(acc, T.dHs(), LD64, mt * 16, T.Zs(), LD48, lane);
					smem_accumulate<48>(acc, sm.g.W1s, GLD48, mt * 16, lane);
				}
				zero_acc<6>(acc);
				warp_gemm_nn<48, 64>(acc, T.dHs(), LD64, sm.w.W1s, LD48, lane);
				store_acc_half<48, false>(acc, T.dZs(), LD48, lane);
			}
			__syncwarp();
			// ---- B6: grid gradient, first order (w_k * dZs) and second order ((grad w_k . v) * Gz) merged into one
			//      reduction per corner; U = dL/dGz = J v comes from the Jacobian kept since F1 (no second gather)
#pragma unroll
			for (int j = 0; j < 8; ++j) {
				const uint32_t l = 2 * j + hl;
				__half2 dy = __floats2half2_rn(0.f, 0.f);
				if (l < a.lv.n_active) {
					dy = __floats2half2_rn(J[j][0] * v[0] + J[j][2] * v[1] + J[j][4] * v[2], J[j][1] * v[0] + J[j][3] * v[1] + J[j][5] * v[2]);
					if (valid) {
						const LevelGeom g = level_geom(a.lv, l, x);
						const float2 ge = __half22float2(*reinterpret_cast<const __half2*>(T.Gz() + s * LD48 + 2 * l));
						const float2 dz = __half22float2(*reinterpret_cast<const __half2*>(T.dZs() + s * LD48 + 2 * l));
						const float scale = a.lv.scale[l];
						// coef_k = grad w_k . v = q[bx][by] * az[bz] + p[bx][by] * bzv[bz],  w_k = p[bx][by] * az[bz]
						const float bxv[2] = {-scale * v[0], scale * v[0]}, byv[2] = {-scale * v[1], scale * v[1]};
						const float bzv[2] = {-scale * v[2], scale * v[2]};
#pragma unroll
						for (uint32_t k = 0; k < 8; ++k) {
							const uint32_t bx = k & 1u, by = (k >> 1) & 1u, bz = (k >> 2) & 1u;
							const float p = g.ax[bx] * g.ay[by];
							const float q = bxv[bx] * g.ay[by] + g.ax[bx] * byv[by];
							const float w = p * g.az[bz];
							const float coef = q * g.az[bz] + p * bzv[bz];
							red_add_h2(a.grad_grid, geom_index(g, k), __fmaf_rn(w, dz.x, coef * ge.x), __fmaf_rn(w, dz.y, coef * ge.y));
						}
					}
				}
				*reinterpret_cast<__half2*>(T.U() + s * LD48 + 2 * l) = dy;
			}
			if (hl == 0) {
#pragma unroll
				for (int e = 0; e < 3; ++e) T.U()[s * LD48 + 32 + e] = __float2half_rn(v[e]);
				// second-order seed: dy = e0 for every live sample (nerf_network.h:497-503)
#pragma unroll
				for (int k = 0; k < 16; ++k) T.Y()[s * LD16 + k] = __float2half_rn((k == 0 && valid) ? 1.f : 0.f);
			} else {
#pragma unroll
				for (int e = 35; e < 48; ++e) T.U()[s * LD48 + e] = __float2half_rn(0.f);
			}
			__syncwarp();
			// ---- B7: T = D .* (U W1s^T);  dW2s[0,:] += sum_b T;  dW1s += S^T U   (nerf_network.h:560-571)
			{
				float acc[8][4];
				zero_acc<8>(acc);
				warp_gemm_nt<64, 48>(acc, T.U(), LD48, sm.w.W1s, LD48, lane);
				store_acc_half_masked<64>(acc, T.Hs(), LD64, T.T(), LD64, lane);
				build_S(T.Hs(), sm.w.W2s, T.S(), lane);
				__syncwarp();
				zero_acc<8>(acc);
				warp_wgrad_mtile<64>(acc, T.Y(), LD16, 0, T.T(), LD64, lane);
				smem_accumulate<64>(acc, sm.g.W2s, GLD64, 0, lane);
			}
			{
				float acc[6][4];
#pragma unroll 1
				for (int mt = 0; mt < 4; ++mt) {
					zero_acc<6>(acc);
					warp_wgrad_mtile<48>(acc, T.S(), LD64, mt * 16, T.U(), LD48, lane);
					smem_accumulate<48>(acc, sm.g.W1s, GLD48, mt * 16, lane);
				}
			}
			__syncwarp();
		}
	}

	if constexpr (MODE == MODE_TRAIN) {
		// variance gradient = sum over the batch of row 7 (nerf_network.h:452-460)
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) var_grad += __shfl_xor_sync(0xffffffffu, var_grad, o);
		if (lane == 0 && var_grad != 0.f) atomicAdd(a.grad_var, var_grad);
		__syncthreads();
		for (int e = tid; e < 64 * 48; e += blockDim.x) {
			const int r = e / 48, k = e % 48;
			const float gs = sm.g.W1s[r * GLD48 + k], gc = sm.g.W1c[r * GLD48 + k];
			if (gs != 0.f) atomicAdd(a.grad_mlp + NEUS2B_SDF_W1 + r * 48 + sdf_orig_col(k), gs);
			if (gc != 0.f) atomicAdd(a.grad_mlp + NEUS2B_RGB_W1 + e, gc);
		}
		for (int e = tid; e < 16 * 64; e += blockDim.x) {
			const int r = e / 64, k = e % 64;
			const float gs = sm.g.W2s[r * GLD64 + k], gc = sm.g.W3c[r * GLD64 + k];
			if (gs != 0.f) atomicAdd(a.grad_mlp + NEUS2B_SDF_W2 + e, gs);
			if (gc != 0.f) atomicAdd(a.grad_mlp + NEUS2B_RGB_W3 + e, gc);
		}
		for (int e = tid; e < 64 * 64; e += blockDim.x) {
			const int r = e / 64, k = e % 64;
			const float gc = sm.g.W2c[r * GLD64 + k];
			if (gc != 0.f) atomicAdd(a.grad_mlp + NEUS2B_RGB_W2 + e, gc);
		}
	}
}

template <int MODE>
static int launch_neus(const NeusArgs& a, uint32_t n_upper, cudaStream_t stream) {
	static bool configured[8] = {false, false, false, false, false, false, false, false};
	int dev = 0;
	N2B_CHECK_CUDA(cudaGetDevice(&dev));
	const size_t smem = sizeof(SmemLayout<MODE>);
	if (dev < 8 && !configured[dev]) {
		N2B_CHECK_CUDA(cudaFuncSetAttribute(neus_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
		configured[dev] = true;
	} else if (dev >= 8) {
		N2B_CHECK_CUDA(cudaFuncSetAttribute(neus_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	}
	const uint32_t tiles = (n_upper + 15u) / 16u;
	uint32_t ctas = (tiles + kWarps - 1) / kWarps;
	const uint32_t per_sm = MODE == MODE_TRAIN ? 1u : 2u;
	if (ctas > kSMs * per_sm) ctas = kSMs * per_sm;  // persistent: one wave of CTAs, grid-stride over tiles
	if (ctas == 0) return NEUS2B_OK;
	neus_kernel<MODE><<<ctas, kWarps * 32, smem, stream>>>(a);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

static int fill_common(NeusArgs& a, const neus2b_grid_desc* desc, const uint16_t* d_params) {
	int rc = make_levels(desc, &a.lv);
	if (rc) return rc;
	if (!d_params) return NEUS2B_E_INVALID;
	a.params = (const __half*)d_params;
	a.grid_entries = a.lv.offset[NEUS2B_MAX_LEVELS];
	return NEUS2B_OK;
}

// tcgen05 / TMEM implementation of the same two kernels (fused_tc.cu)
int launch_neus_tc_forward(const NeusArgs& a, uint32_t n_upper, cudaStream_t stream);
int launch_neus_tc_train(const NeusArgs& a, uint32_t n_upper, cudaStream_t stream);
int read_tc_error(uint32_t* h_flags);
int write_tc_error(uint32_t flags);
static int g_mma_path = NEUS2B_MMA_TCGEN05;

}  // namespace n2b

using namespace n2b;

extern "C" int neus2b_set_mma_path(int path) {
	if (path != NEUS2B_MMA_SYNC && path != NEUS2B_MMA_TCGEN05) return NEUS2B_E_INVALID;
	g_mma_path = path;
	return NEUS2B_OK;
}
extern "C" int neus2b_get_mma_path(void) { return g_mma_path; }
extern "C" int neus2b_device_error_flags(uint32_t* h_flags) {
	if (!h_flags) return NEUS2B_E_INVALID;
	return read_tc_error(h_flags);
}
extern "C" int neus2b_set_device_error_flags(uint32_t flags) { return write_tc_error(flags); }

static void fill_motion(NeusArgs& a, const neus2b_motion* motion) {
	if (!motion || !motion->d_delta) return;
	a.delta = (const __half*)motion->d_delta;
	for (int e = 0; e < 3; ++e) a.first_frame_offset[e] = motion->first_frame_offset[e];
	a.delta_sums = motion->d_sums;
}

extern "C" int neus2b_neus_forward(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n,
                                   const uint32_t* d_n, const float* d_coords, uint16_t* d_out, neus2b_stream_t stream) {
	return neus2b_neus_forward_moved(desc, d_params, sdf_bias, n, d_n, d_coords, nullptr, d_out, stream);
}

extern "C" int neus2b_neus_forward_moved(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n,
                                         const uint32_t* d_n, const float* d_coords, const neus2b_motion* motion, uint16_t* d_out,
                                         neus2b_stream_t stream) {
	return neus2b_neus_forward_indexed(desc, d_params, sdf_bias, n, d_n, nullptr, d_coords, motion, d_out, stream);
}

extern "C" int neus2b_neus_forward_indexed(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n,
                                           const uint32_t* d_n, const uint32_t* d_index, const float* d_coords, const neus2b_motion* motion,
                                           uint16_t* d_out, neus2b_stream_t stream) {
	NeusArgs a = {};
	a.index = d_index;
	if (d_index && g_mma_path != NEUS2B_MMA_TCGEN05) return NEUS2B_E_UNSUPPORTED;
	int rc = fill_common(a, desc, d_params);
	if (rc) return rc;
	if (!d_coords || !d_out || ((uintptr_t)d_out & 15u)) return NEUS2B_E_INVALID;
	fill_motion(a, motion);
	a.delta_sums = nullptr;
	if (a.delta && g_mma_path != NEUS2B_MMA_TCGEN05) return NEUS2B_E_UNSUPPORTED;
	a.sdf_bias = sdf_bias;
	a.n = n;
	a.d_n = d_n;
	a.coords = d_coords;
	a.coord_stride = 7;
	a.dir_offset = 4;
	a.out = (__half*)d_out;
	if (g_mma_path == NEUS2B_MMA_TCGEN05) return launch_neus_tc_forward(a, n, stream);
	return launch_neus<MODE_FWD>(a, n, stream);
}

extern "C" int neus2b_neus_train(const neus2b_grid_desc* desc, const uint16_t* d_params, uint32_t n, const float* d_coords,
                                 const uint16_t* d_dL_dout, uint32_t indeed_batch_size, float* d_grad_mlp, uint16_t* d_grad_grid,
                                 float* d_grad_variance, neus2b_stream_t stream) {
	if (!d_grad_mlp || !d_grad_grid || !d_grad_variance) return NEUS2B_E_INVALID;
	return neus2b_neus_train_moved(desc, d_params, n, d_coords, nullptr, d_dL_dout, indeed_batch_size, d_grad_mlp, d_grad_grid, d_grad_variance,
	                               stream);
}

extern "C" int neus2b_neus_train_moved(const neus2b_grid_desc* desc, const uint16_t* d_params, uint32_t n, const float* d_coords,
                                       const neus2b_motion* motion, const uint16_t* d_dL_dout, uint32_t indeed_batch_size, float* d_grad_mlp,
                                       uint16_t* d_grad_grid, float* d_grad_variance, neus2b_stream_t stream) {
	NeusArgs a = {};
	int rc = fill_common(a, desc, d_params);
	if (rc) return rc;
	if (!d_coords || !d_dL_dout || ((uintptr_t)d_dL_dout & 15u) || indeed_batch_size == 0) return NEUS2B_E_INVALID;
	// the canonical gradients are all there or all absent (a frame's first steps train the motion alone)
	const bool canonical = d_grad_mlp && d_grad_grid && d_grad_variance;
	if (!canonical && (d_grad_mlp || d_grad_grid || d_grad_variance)) return NEUS2B_E_INVALID;
	fill_motion(a, motion);
	if (!canonical && !a.delta_sums) return NEUS2B_E_INVALID;
	if ((a.delta || !canonical) && g_mma_path != NEUS2B_MMA_TCGEN05) return NEUS2B_E_UNSUPPORTED;
	a.n = n;
	a.coords = d_coords;
	a.coord_stride = 7;
	a.dir_offset = 4;
	a.dL_dout = (const __half*)d_dL_dout;
	a.batch_size = (float)indeed_batch_size;
	a.grad_mlp = d_grad_mlp;
	a.grad_grid = (__half*)d_grad_grid;
	a.grad_var = d_grad_variance;
	if (g_mma_path == NEUS2B_MMA_TCGEN05) return launch_neus_tc_train(a, n, stream);
	return launch_neus<MODE_TRAIN>(a, n, stream);
}

extern "C" int neus2b_neus_sdf(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n, const float* d_x,
                               uint32_t x_stride, uint16_t* d_sdf, neus2b_stream_t stream) {
	return neus2b_neus_sdf_moved(desc, d_params, sdf_bias, n, d_x, x_stride, nullptr, d_sdf, stream);
}

extern "C" int neus2b_neus_sdf_moved(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n, const float* d_x,
                                     uint32_t x_stride, const neus2b_motion* motion, uint16_t* d_sdf, neus2b_stream_t stream) {
	NeusArgs a = {};
	int rc = fill_common(a, desc, d_params);
	if (rc) return rc;
	if (!d_x || !d_sdf || x_stride < 3) return NEUS2B_E_INVALID;
	fill_motion(a, motion);
	a.delta_sums = nullptr;
	a.sdf_bias = sdf_bias;
	a.n = n;
	a.coords = d_x;
	a.coord_stride = x_stride;
	a.sdf_out = (__half*)d_sdf;
	return launch_neus<MODE_SDF>(a, n, stream);
}
