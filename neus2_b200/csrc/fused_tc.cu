// Fused NeuS graph kernels on tcgen05 / TMEM (NerfNetwork::forward_impl / backward_impl of the reference,
// include/neural-graphics-primitives/nerf_network.h:132-641), sm_100a.
//
// A CTA of 512 threads owns a tile of 128 samples.  Thread t works for sample (t & 127): the four threads of a sample
// split the 16 grid levels (gather, Jacobian, scatter: levels p, p + 4, p + 8, p + 12 for part p = t / 128) and the accumulator
// columns (epilogues: 16 each).  The graph's per-sample arithmetic, not the tensor cores, bounds these kernels, and it
// runs at the dependent-issue rate of the resident warps: 16 warps per SM instead of 8 is worth more than anything
// else, while the shared memory stays small enough to leave about 100 KB of L1 for the hash-grid gather.  Every dense
// contraction of the graph is a tcgen05.mma chain issued by one thread with M = 128 (the samples), operands read from
// shared memory in the core-matrix layout (tc05.cuh), fp32 accumulators in tensor memory:
//   forward:  Hs = relu(Zs W1s^T), Ys = Hs W2s^T, Gz = S W1s (d y0 / d z), H1, H2 (, out) of the colour net;
//   backward: input gradients dH2, dH1, dZc, dHs, dZs, the second-order T = D .* (U W1s^T);
//   weight gradients: dW = D^T Z contracts over the 128 samples -- the activation tiles are read a second time as
//             MN-major operands, and the five dW accumulators stay resident in tensor memory for the whole kernel
//             (no shared-memory or register accumulators, no atomics until the final flush).
// Weight matrices are staged once per CTA; as MN-major B operands they also serve the input-gradient GEMMs, so no
// transposed copies exist.  Only rows 0..63 of a weight-gradient accumulator are meaningful (M is 128, the matrices
// have 64 rows): the upper rows are computed from whatever follows the tile in shared memory and are never read.
#include "common.cuh"
#include "fused_common.cuh"
#include "tc05.cuh"
#include "delta.cuh"

namespace n2b {
namespace tcf {

constexpr int kThreads = 512, kParts = 4;
#ifndef N2B_MERGED_J
#define N2B_MERGED_J 2
#endif
constexpr int kMergedJ = N2B_MERGED_J;  // the levels 0 .. 4 * kMergedJ - 1 pre-reduce their grid gradients in the warp

// Part p of a sample's four threads owns the levels p, p + 4, p + 8, p + 12 (a coarse, two middle and a fine one each, so
// the parts carry equal work) and keeps their features in the internal columns 8 p .. 8 p + 7 of the SDF-net input;
// the position follows in columns 32..34.  Original column (reference order: position, then the levels) of internal k:
__device__ __forceinline__ int tc_orig_col(int k) {
	if (k >= 32) return k < 35 ? k - 32 : k;
	const int p = k >> 3, j = (k >> 1) & 3, f = k & 1;
	return 3 + 2 * (p + 4 * j) + f;
}
constexpr int T48 = 128 * 48 * 2, T64 = 128 * 64 * 2, T16 = 128 * 16 * 2;

static __device__ uint32_t g_tc_error;  // bit 0: a bounded completion wait ran out

template <int MODE, bool DYN>
struct Smem {
	alignas(128) unsigned char W1s[64 * 48 * 2];
	unsigned char W2s[16 * 64 * 2];
	unsigned char W1c[64 * 48 * 2];
	unsigned char W2c[64 * 64 * 2];
	unsigned char W3c[16 * 64 * 2];
	unsigned char Zs[T48];  // SDF-net input; training: later U
	unsigned char Zc[T48];  // colour-net input
	unsigned char Hs[T64];  // SDF hidden; inference: later H2
	unsigned char X1[T64];  // S -> H1 -> (training) S again
	unsigned char X2[MODE == MODE_TRAIN ? T64 : 16];  // H2 -> dH1
	unsigned char X3[MODE == MODE_TRAIN ? T64 : 16];  // dH2 -> dHs -> T
	unsigned char dY[MODE == MODE_TRAIN ? T16 : 16];  // dY3 -> dYs
	unsigned char E0[MODE == MODE_TRAIN ? T16 : 16];  // second-order seed e0 (its own tile: the GEMM that reads dYs may still run)
	__half gst[MODE == MODE_TRAIN ? 128 : 1][8];      // rows 3..10 of a sample's output gradient, from part 0 to part 1
	float nrm[kParts][128][3];
	float vbuf[128][4];
	// xyz rows of the colour-net input gradient (for the DeltaNetwork's dL/dx).  Only in the dynamic instantiation: with it the
	// static training kernel's shared memory (plus the 1 KB the system reserves per CTA) would cross 132 KB, the carve-out
	// would move up a step and the L1 that the table gathers live on would shrink from 124 to 92 KB.
	float dxc[(MODE == MODE_TRAIN && DYN) ? 128 : 1][3];
	float motion[12];                            // the frame's rigid motion: R row-major, t
	float dsum[12];                              // this CTA's share of the DeltaNetwork's backward sums
	float red[kThreads / 32];
	uint64_t mbar;
	uint32_t tmem_base;
	uint32_t pad;
};

__device__ __forceinline__ uint32_t sptr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

struct Opnd {
	uint32_t addr, lbo, sbo, kstep, mn;
};
// [rows][C] tile as K-major operand (rows = M or N, columns = K) / as MN-major operand (columns = M or N, rows = K)
__device__ __forceinline__ Opnd kmaj(const void* t, int C) { return Opnd{sptr(t), 128u, (uint32_t)C * 16u, 256u, 0u}; }
__device__ __forceinline__ Opnd mnmaj(const void* t, int C) { return Opnd{sptr(t), (uint32_t)C * 16u, 128u, (uint32_t)C * 32u, 1u}; }

template <int N>
__device__ __forceinline__ void gemm(uint32_t d, const Opnd a, const Opnd b, int ksteps, bool accumulate) {
	const uint32_t id = tc::idesc_f16(128, N, (int)a.mn, (int)b.mn);
	for (int kk = 0; kk < ksteps; ++kk)
		tc::mma_f16(d, tc::smem_desc(a.addr + kk * a.kstep, a.lbo, a.sbo), tc::smem_desc(b.addr + kk * b.kstep, b.lbo, b.sbo), id,
		            (accumulate || kk > 0) ? 1u : 0u);
}

__device__ __forceinline__ void st16(unsigned char* tile, int row, int col, int C, const __half* h8) {
	*reinterpret_cast<uint4*>(tile + tc::blk_off(row, col, C)) = *reinterpret_cast<const uint4*>(h8);
}

// Accumulator columns [c0, c0+16) of this thread's row -> fp16 tile row.  ACT: 1 = ReLU (returns the mask of positive
// outputs), 2 = multiply by the given mask bits (ReLU backward).
template <int ACT>
__device__ __forceinline__ uint32_t epilogue16(uint32_t taddr, int row, int c0, unsigned char* tile, uint32_t mask_in) {
	uint32_t mask_out = 0;
	float v[16];
	tc::tmem_ld16(taddr + c0, v);
	tc::tmem_ld_wait();
	__align__(16) uint32_t w[8];  // 8 fp16 pairs
#pragma unroll
	for (int e = 0; e < 8; ++e) {
		__half2 h = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
		if (ACT == 1) h = __hmax2(h, __floats2half2_rn(0.f, 0.f));  // round(relu(x)) == relu(round(x))
		uint32_t u = *reinterpret_cast<uint32_t*>(&h);
		if (ACT == 1) {
			u &= 0x7fff7fffu;  // nothing negative is left: a -0 becomes +0
			mask_out |= (uint32_t)((u & 0xffffu) != 0u) << (2 * e);
			mask_out |= (uint32_t)((u & 0xffff0000u) != 0u) << (2 * e + 1);
		}
		if (ACT == 2) {
			const uint32_t keep = (((mask_in >> (2 * e)) & 1u) ? 0xffffu : 0u) | (((mask_in >> (2 * e + 1)) & 1u) ? 0xffff0000u : 0u);
			u &= keep;
		}
		w[e] = u;
	}
	*reinterpret_cast<uint4*>(tile + tc::blk_off(row, c0, 64)) = reinterpret_cast<const uint4*>(w)[0];
	*reinterpret_cast<uint4*>(tile + tc::blk_off(row, c0 + 8, 64)) = reinterpret_cast<const uint4*>(w)[1];
	return mask_out;
}

// S[row][c0 .. c0+16) = mask ? W2s[0][c] : 0   (W2s row 0 read from the staged, blocked weight tile)
__device__ __forceinline__ void write_S(const unsigned char* W2s, unsigned char* tile, int row, int c0, uint32_t mask) {
#pragma unroll
	for (int q = 0; q < 2; ++q) {
		const int c = c0 + 8 * q;
		__align__(16) __half w[8];
		*reinterpret_cast<uint4*>(w) = *reinterpret_cast<const uint4*>(W2s + tc::blk_off(0, c, 64));
#pragma unroll
		for (int e = 0; e < 8; ++e)
			if (!((mask >> (8 * q + e)) & 1u)) w[e] = __float2half_rn(0.f);
		st16(tile, row, c, 64, w);
	}
}

// 8 consecutive fp32 columns of the thread's tensor-memory lane
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
	uint32_t r[8];
	asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
	             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
	             : "r"(taddr)
	             : "memory");
#pragma unroll
	for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// DYN compiles the dynamic-sequence parts in (the frame's rigid motion applied to the samples, the motion's backward sums,
// gradient outputs that may be absent while the canonical model is frozen).  Static scenes run the DYN = false
// instantiation: keeping the encoding's Jacobian alive up to the scatter for a flag that is never set costs the static
// kernel 9 % (0.275 -> 0.300 ms at 2^18 samples).
template <int MODE, bool DYN>
__global__ void __launch_bounds__(kThreads, 1) neus_tc_kernel(const NeusArgs a) {
	extern __shared__ __align__(128) unsigned char smem_raw[];
	Smem<MODE, DYN>& sm = *reinterpret_cast<Smem<MODE, DYN>*>(smem_raw);
	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	const int s = tid & 127, part = tid >> 7;
	const __half* grid = a.params + NEUS2B_GRID_OFF;
	constexpr uint32_t kTmemCols = MODE == MODE_TRAIN ? 512u : 128u;

	// A CTA without a tile leaves before the set-up (a windowed forward pass runs on short lists: most of the 148 CTAs of
	// such a launch have nothing to do, and the set-up is the larger part of what a short launch costs).  The whole CTA
	// takes the same branch: no barrier, no tensor memory yet.
	if ((size_t)blockIdx.x * 128u >= (size_t)(a.d_n ? min(*a.d_n, a.n) : a.n)) return;

	// ---- one-time set-up: zero the tiles (padding columns stay zero), stage the weights, allocate tensor memory
	for (int e = tid; e < (int)(sizeof(Smem<MODE, DYN>) / 16); e += kThreads) reinterpret_cast<uint4*>(smem_raw)[e] = make_uint4(0, 0, 0, 0);
	__syncthreads();
	for (int e = tid; e < 64 * 48; e += kThreads) {
		const int r = e / 48, k = e % 48;
		*reinterpret_cast<__half*>(sm.W1s + tc::blk_off(r, k, 48)) = a.params[NEUS2B_SDF_W1 + r * 48 + tc_orig_col(k)];
		*reinterpret_cast<__half*>(sm.W1c + tc::blk_off(r, k, 48)) = a.params[NEUS2B_RGB_W1 + e];
	}
	for (int e = tid; e < 16 * 64; e += kThreads) {
		*reinterpret_cast<__half*>(sm.W2s + tc::blk_off(e / 64, e % 64, 64)) = a.params[NEUS2B_SDF_W2 + e];
		*reinterpret_cast<__half*>(sm.W3c + tc::blk_off(e / 64, e % 64, 64)) = a.params[NEUS2B_RGB_W3 + e];
	}
	for (int e = tid; e < 64 * 64; e += kThreads)
		*reinterpret_cast<__half*>(sm.W2c + tc::blk_off(e / 64, e % 64, 64)) = a.params[NEUS2B_RGB_W2 + e];
	const bool moved = DYN && a.delta != nullptr;
	if (tid == 0 && moved) {
		const RigidMotion rm = load_rigid_motion(a.delta);
#pragma unroll
		for (int k = 0; k < 9; ++k) sm.motion[k] = rm.R[k];
#pragma unroll
		for (int k = 0; k < 3; ++k) sm.motion[9 + k] = rm.t[k];
	}
	const uint32_t mbar = sptr(&sm.mbar);
	if (tid == 0) tc::mbar_init(mbar, 1);
	if (warp == 0) tc::tmem_alloc(sptr(&sm.tmem_base), kTmemCols);
	tc::fence_before_sync();
	__syncthreads();
	tc::fence_after_sync();
	const uint32_t tm = sm.tmem_base;
	const uint32_t lrow = (uint32_t)((warp & 3) * 32) << 16;  // this warp's tensor-memory lanes: rows (warp & 3) * 32 + lane == s
	const uint32_t R0 = tm + lrow, R1 = tm + 64 + lrow;
	const uint32_t WG_W2c = tm + 128, WG_W1c = tm + 192, WG_W1s = tm + 240, WG_W3cT = tm + 288, WG_W2sT = tm + 304;

	const uint32_t n = a.d_n ? min(*a.d_n, a.n) : a.n;
	const uint32_t n_tiles = (n + 127u) / 128u;
	const __half variance = a.params[NEUS2B_GRID_OFF + (size_t)a.grid_entries * 2];
	const float bias = __half2float(__float2half_rn(a.sdf_bias));
	float var_grad = 0.f;
	uint32_t phase = 0;
	bool ok = true, first = true, pending = false;

	// A wait that ran out stays failed for the thread (later waits return at once); nobody leaves the tile loop early, so
	// the barriers always match and the kernel ends by itself with the error flag raised.
#define N2B_ISSUE_NOWAIT(BODY)                           \
	tc::fence_async_smem();                              \
	tc::fence_before_sync();                             \
	__syncthreads();                                     \
	if (tid == 0) {                                      \
		tc::fence_after_sync();                          \
		BODY;                                            \
		tc::commit(mbar);                                \
	}
// BODY is waited for, TAIL (weight-gradient GEMMs, read at the end of the kernel only) runs on behind the wait: the tensor
// pipe works through it while the threads do the stage's epilogue.  MMAs of one thread complete in issue order, so the
// next stage's wait also covers this TAIL.
#define N2B_ISSUE_TAIL(BODY, TAIL)                       \
	tc::fence_async_smem();                              \
	tc::fence_before_sync();                             \
	__syncthreads();                                     \
	if (tid == 0) {                                      \
		tc::fence_after_sync();                          \
		BODY;                                            \
		tc::commit(mbar);                                \
		TAIL;                                            \
	}                                                    \
	N2B_WAIT()
#define N2B_WAIT()                                       \
	if (ok) ok = tc::mbar_wait(mbar, phase);             \
	phase ^= 1u;                                         \
	tc::fence_after_sync();
#define N2B_ISSUE(BODY)    \
	N2B_ISSUE_NOWAIT(BODY) \
	N2B_WAIT()

	for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
		const uint32_t i = tile * 128u + (uint32_t)s;
		const bool valid = i < n;
		// (the forward pass can run on a list of samples: row of the coordinate and output arrays this entry stands for)
		uint32_t row = i;
		if (MODE == MODE_FWD && valid && a.index) row = __ldg(a.index + i);
		float x[3] = {0.5f, 0.5f, 0.5f}, dir[3] = {0.5f, 0.5f, 0.5f};
		if (valid) {
			const float* c = a.coords + (size_t)row * a.coord_stride;
			x[0] = c[0];
			x[1] = c[1];
			x[2] = c[2];
			dir[0] = c[a.dir_offset];
			dir[1] = c[a.dir_offset + 1];
			dir[2] = c[a.dir_offset + 2];
		}
		if (moved) move_sample(sm.motion, sm.motion + 9, a.first_frame_offset, x, dir);
		// ---- gather: features of this thread's 4 levels -> Zs, Jacobian d enc / d x kept in registers.
		// All 32 table loads of the thread are issued before the first is used: one trip to L2 per tile instead of one per level.
		float J[4][6];
		__half2 feats[4];
		__half2 th[4][8];
		float fr[4][3];
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const uint32_t l = (uint32_t)(part + 4 * j);
			if (l < a.lv.n_active) {
				const LevelGeom g = level_geom(a.lv, l, x);
				fr[j][0] = g.ax[1];
				fr[j][1] = g.ay[1];
				fr[j][2] = g.az[1];
#pragma unroll
				for (uint32_t k = 0; k < 8; ++k) th[j][k] = ldg_h2(grid, geom_index(g, k));
			} else {
				fr[j][0] = fr[j][1] = fr[j][2] = 0.f;
#pragma unroll
				for (uint32_t k = 0; k < 8; ++k) th[j][k] = __floats2half2_rn(0.f, 0.f);
			}
		}
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const uint32_t l = (uint32_t)(part + 4 * j);
			__half2 feat = __floats2half2_rn(0.f, 0.f);
#pragma unroll
			for (int e = 0; e < 6; ++e) J[j][e] = 0.f;
			if (l < a.lv.n_active) {
				const float gax[2] = {1.0f - fr[j][0], fr[j][0]}, gay[2] = {1.0f - fr[j][1], fr[j][1]}, gaz[2] = {1.0f - fr[j][2], fr[j][2]};
				const float scale = a.lv.scale[l];
				// Trilinear value and its gradient, factored: along an axis the derivative is the difference of the two faces
				// weighted by the other two axes' products (fp32 throughout, one rounding of the value to fp16).
				float2 t[8];
#pragma unroll
				for (int k = 0; k < 8; ++k) t[k] = __half22float2(th[j][k]);
				float a0 = 0.f, a1 = 0.f;
				float jx0 = 0.f, jx1 = 0.f, jy0 = 0.f, jy1 = 0.f, jz0 = 0.f, jz1 = 0.f;
#pragma unroll
				for (int u = 0; u < 2; ++u)
#pragma unroll
					for (int v = 0; v < 2; ++v) {
						const float pyz = gay[u] * gaz[v], pxz = gax[u] * gaz[v], pxy = gax[u] * gay[v];
						const float2 x0 = t[2 * u + 4 * v], x1 = t[1 + 2 * u + 4 * v];  // bx = 0 | 1 at (by, bz) = (u, v)
						a0 = __fmaf_rn(pyz, __fmaf_rn(gax[1], x1.x, gax[0] * x0.x), a0);
						a1 = __fmaf_rn(pyz, __fmaf_rn(gax[1], x1.y, gax[0] * x0.y), a1);
						jx0 = __fmaf_rn(pyz, x1.x - x0.x, jx0);
						jx1 = __fmaf_rn(pyz, x1.y - x0.y, jx1);
						const float2 y0 = t[u + 4 * v], y1 = t[u + 2 + 4 * v];  // by = 0 | 1 at (bx, bz) = (u, v)
						jy0 = __fmaf_rn(pxz, y1.x - y0.x, jy0);
						jy1 = __fmaf_rn(pxz, y1.y - y0.y, jy1);
						const float2 z0 = t[u + 2 * v], z1 = t[u + 2 * v + 4];  // bz = 0 | 1 at (bx, by) = (u, v)
						jz0 = __fmaf_rn(pxy, z1.x - z0.x, jz0);
						jz1 = __fmaf_rn(pxy, z1.y - z0.y, jz1);
					}
				J[j][0] = scale * jx0;
				J[j][1] = scale * jx1;
				J[j][2] = scale * jy0;
				J[j][3] = scale * jy1;
				J[j][4] = scale * jz0;
				J[j][5] = scale * jz1;
				feat = __floats2half2_rn(a0, a1);
			}
			feats[j] = feat;
		}
		// the previous tile's last GEMMs (weight gradients only) still read the tiles: wait for them here, behind the gather
		if (pending) {
			N2B_WAIT();
			pending = false;
		}
		{
			__align__(16) __half f8[8];
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				f8[2 * j] = __low2half(feats[j]);
				f8[2 * j + 1] = __high2half(feats[j]);
			}
			st16(sm.Zs, s, 8 * part, 48, f8);  // this part's levels = columns 8 p .. 8 p + 7
		}
		if (part == 0) {
#pragma unroll
			for (int e = 0; e < 3; ++e)
				*reinterpret_cast<__half*>(sm.Zs + tc::blk_off(s, 32 + e, 48)) = __float2half_rn(__half2float(__float2half_rn(x[e])) - 0.5f);
		}
		// ---- Hs = relu(Zs W1s^T)
		N2B_ISSUE(gemm<64>(tm, kmaj(sm.Zs, 48), kmaj(sm.W1s, 48), 3, false));
		const uint32_t m_hs = epilogue16<1>(R0, s, part * 16, sm.Hs, 0u);
		write_S(sm.W2s, sm.X1, s, part * 16, m_hs);
		// ---- Ys = Hs W2s^T (R1[0:16]) ; Gz = S W1s (R0[0:48])
		N2B_ISSUE(gemm<16>(tm + 64, kmaj(sm.Hs, 64), kmaj(sm.W2s, 64), 4, false);
		          gemm<48>(tm, kmaj(sm.X1, 64), mnmaj(sm.W1s, 48), 4, false));
		__half2 ge[4];
		float nrm[3] = {0.f, 0.f, 0.f};
		{
			float v[8];
			tmem_ld8(R0 + 8 * part, v);  // d y0 / d (features of this thread's levels)
			tc::tmem_ld_wait();
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				const float g0 = __half2float(__float2half_rn(v[2 * j]));
				const float g1 = __half2float(__float2half_rn(v[2 * j + 1]));
				ge[j] = __floats2half2_rn(g0, g1);
#pragma unroll
				for (int e = 0; e < 3; ++e) nrm[e] = __fmaf_rn(J[j][2 * e], g0, __fmaf_rn(J[j][2 * e + 1], g1, nrm[e]));
			}
		}
		if (part == 0) {
			float v[8];
			tmem_ld8(R0 + 32, v);  // direct position columns of the SDF-net input
			tc::tmem_ld_wait();
#pragma unroll
			for (int e = 0; e < 3; ++e) nrm[e] += __half2float(__float2half_rn(v[e]));
		}
#pragma unroll
		for (int e = 0; e < 3; ++e) sm.nrm[part][s][e] = nrm[e];
		if (part == 1) {
			float v[16];
			tc::tmem_ld16(R1, v);
			tc::tmem_ld_wait();
			__align__(16) __half h[16];
#pragma unroll
			for (int e = 0; e < 16; ++e) h[e] = __float2half_rn(v[e]);
			st16(sm.Zc, s, 0, 48, h);
			st16(sm.Zc, s, 8, 48, h + 8);
		} else if (part == 2) {
			float sh[16];
			sh4_eval(dir, sh);
			__align__(16) __half h[16];
#pragma unroll
			for (int e = 0; e < 16; ++e) h[e] = __float2half_rn(sh[e]);
			st16(sm.Zc, s, 16, 48, h);
			st16(sm.Zc, s, 24, 48, h + 8);
		}
		tc::fence_before_sync();
		__syncthreads();
		if (part == 0) {
			__align__(16) __half h[8];
#pragma unroll
			for (int e = 0; e < 3; ++e) {
				nrm[e] = ((sm.nrm[0][s][e] + sm.nrm[1][s][e]) + sm.nrm[2][s][e]) + sm.nrm[3][s][e];
				h[e] = __float2half_rn(x[e]);
				h[3 + e] = __float2half_rn(nrm[e]);
			}
			h[6] = h[7] = __float2half_rn(0.f);
			st16(sm.Zc, s, 32, 48, h);
		}
		// (training: this sample's output gradient is requested now and used behind the colour net's forward pass)
		uint4 gq0 = make_uint4(0u, 0u, 0u, 0u), gq1 = gq0;
		if constexpr (MODE == MODE_TRAIN) {
			if (part == 0 && valid) {
				const uint4* src = reinterpret_cast<const uint4*>(a.dL_dout + (size_t)i * 16);
				gq0 = __ldg(src);
				gq1 = __ldg(src + 1);
			}
		}
		// ---- colour net
		N2B_ISSUE(gemm<64>(tm + 64, kmaj(sm.Zc, 48), kmaj(sm.W1c, 48), 3, false));
		const uint32_t m_h1 = epilogue16<1>(R1, s, part * 16, sm.X1, 0u);
		N2B_ISSUE(gemm<64>(tm, kmaj(sm.X1, 64), kmaj(sm.W2c, 64), 4, false));
		unsigned char* H2 = MODE == MODE_TRAIN ? sm.X2 : sm.Hs;
		const uint32_t m_h2 = epilogue16<1>(R0, s, part * 16, H2, 0u);
		(void)m_h1;
		(void)m_h2;
		if constexpr (MODE == MODE_FWD) {
			N2B_ISSUE(gemm<16>(tm + 64, kmaj(H2, 64), kmaj(sm.W3c, 64), 4, false));
			if (part == 0) {
				float v[16];
				tc::tmem_ld16(R1, v);
				tc::tmem_ld_wait();
				if (valid) {
					__align__(16) __half o[16];
#pragma unroll
					for (int k = 0; k < 16; ++k) o[k] = __float2half_rn(v[k]);
					o[3] = __float2half_rn(__half2float(*reinterpret_cast<const __half*>(sm.Zc + tc::blk_off(s, 0, 48))) + bias);
#pragma unroll
					for (int e = 0; e < 3; ++e) {
						o[4 + e] = __float2half_rn(nrm[e]);
						o[8 + e] = __float2half_rn(dir[e]);
					}
					o[7] = variance;
					uint4* dst = reinterpret_cast<uint4*>(a.out + (size_t)row * 16);
					dst[0] = reinterpret_cast<const uint4*>(o)[0];
					dst[1] = reinterpret_cast<const uint4*>(o)[1];
				}
			}
		} else {
			// ---- B1: dY3 = rows 0-2 of dL_dout (nerf_network.h:331-340)
			__align__(16) __half g[16];
			reinterpret_cast<uint4*>(g)[0] = gq0;
			reinterpret_cast<uint4*>(g)[1] = gq1;
			if (part == 0) {
				__align__(16) __half d3[16];
#pragma unroll
				for (int k = 0; k < 16; ++k) d3[k] = k < 3 ? g[k] : __float2half_rn(0.f);
				st16(sm.dY, s, 0, 16, d3);
				st16(sm.dY, s, 8, 16, d3 + 8);
				__align__(16) __half gs[8];
#pragma unroll
				for (int e = 0; e < 8; ++e) gs[e] = g[3 + e];
				*reinterpret_cast<uint4*>(&sm.gst[s][0]) = *reinterpret_cast<const uint4*>(gs);  // (read by part 1 behind B3's barrier)
			}
			N2B_ISSUE_TAIL(gemm<64>(tm + 64, kmaj(sm.dY, 16), mnmaj(sm.W3c, 64), 1, false),
			               gemm<16>(WG_W3cT, mnmaj(sm.X2, 64), mnmaj(sm.dY, 16), 8, !first));
			epilogue16<2>(R1, s, part * 16, sm.X3, m_h2);  // dH2
			// ---- B2
			N2B_ISSUE_TAIL(gemm<64>(tm, kmaj(sm.X3, 64), mnmaj(sm.W2c, 64), 4, false),
			               gemm<64>(WG_W2c, mnmaj(sm.X3, 64), mnmaj(sm.X1, 64), 8, !first));
			epilogue16<2>(R0, s, part * 16, sm.X2, m_h1);  // dH1 (over H2)
			// ---- B3
			N2B_ISSUE_TAIL(gemm<48>(tm + 64, kmaj(sm.X2, 64), mnmaj(sm.W1c, 48), 4, false),
			               gemm<48>(WG_W1c, mnmaj(sm.X2, 64), mnmaj(sm.Zc, 48), 8, !first));
			// ---- B4: SDF-net output gradient = colour-net input gradient rows 0-15 (+ dL/dsdf), v = dL/dnormal (:388-395, :465-491)
			if (part == 0) {
				float v[16];
				tc::tmem_ld16(R1, v);
				tc::tmem_ld_wait();
				__align__(16) __half h[16];
#pragma unroll
				for (int e = 0; e < 16; ++e) h[e] = __float2half_rn(v[e]);
				h[0] = __hadd(h[0], g[3]);
				st16(sm.dY, s, 0, 16, h);
				st16(sm.dY, s, 8, 16, h + 8);
				var_grad += __half2float(g[7]);
			} else if (part == 1) {
				float v[8];
				tmem_ld8(R1 + 32, v);
				tc::tmem_ld_wait();
				__align__(16) __half gs[8];  // rows 3..10 of the output gradient
				*reinterpret_cast<uint4*>(gs) = *reinterpret_cast<const uint4*>(&sm.gst[s][0]);
#pragma unroll
				for (int e = 0; e < 3; ++e) {
					sm.vbuf[s][e] = __half2float(__float2half_rn(v[3 + e])) + __half2float(gs[1 + e]) / a.batch_size + __half2float(gs[5 + e]);
					if (DYN) sm.dxc[s][e] = __half2float(__float2half_rn(v[e]));
				}
			}
			N2B_ISSUE_TAIL(gemm<64>(tm, kmaj(sm.dY, 16), mnmaj(sm.W2s, 64), 1, false),
			               gemm<16>(WG_W2sT, mnmaj(sm.Hs, 64), mnmaj(sm.dY, 16), 8, !first));
			epilogue16<2>(R0, s, part * 16, sm.X3, m_hs);  // dHs
			// ---- B5 + B7: U = [J v | v | 0] (dL / d(dy0/dz), :547-557) goes over the colour-net input tile, which is free since B3, so
			// that the second-order GEMMs need not wait for B5: T' = U W1s^T and dW1s += S^T U (:560-571) are issued with it.
			const float v3[3] = {sm.vbuf[s][0], sm.vbuf[s][1], sm.vbuf[s][2]};
			{
				__align__(16) __half u8[8];
#pragma unroll
				for (int j = 0; j < 4; ++j) {
					const uint32_t l = (uint32_t)(part + 4 * j);
					__half2 dy = __floats2half2_rn(0.f, 0.f);
					if (l < a.lv.n_active)
						dy = __floats2half2_rn(J[j][0] * v3[0] + J[j][2] * v3[1] + J[j][4] * v3[2],
						                       J[j][1] * v3[0] + J[j][3] * v3[1] + J[j][5] * v3[2]);
					u8[2 * j] = __low2half(dy);
					u8[2 * j + 1] = __high2half(dy);
				}
				st16(sm.Zc, s, 8 * part, 48, u8);
			}
			if (part == 0) {
				__align__(16) __half h[8];
#pragma unroll
				for (int e = 0; e < 8; ++e) h[e] = __float2half_rn(e < 3 ? v3[e] : 0.f);
				st16(sm.Zc, s, 32, 48, h);
			} else if (part == 1) {
				// second-order seed dy = e0 for every live sample (:497-503)
				__align__(16) __half e0[16];
#pragma unroll
				for (int k = 0; k < 16; ++k) e0[k] = __float2half_rn((k == 0 && valid) ? 1.f : 0.f);
				st16(sm.E0, s, 0, 16, e0);
				st16(sm.E0, s, 8, 16, e0 + 8);
			}
			write_S(sm.W2s, sm.X1, s, part * 16, m_hs);
			N2B_ISSUE_TAIL(gemm<48>(tm + 64, kmaj(sm.X3, 64), mnmaj(sm.W1s, 48), 4, false);
			               gemm<48>(WG_W1s, mnmaj(sm.X3, 64), mnmaj(sm.Zs, 48), 8, !first);
			               gemm<64>(tm, kmaj(sm.Zc, 48), kmaj(sm.W1s, 48), 3, false),
			               gemm<48>(WG_W1s, mnmaj(sm.X1, 64), mnmaj(sm.Zc, 48), 8, true));
			epilogue16<2>(R0, s, part * 16, sm.X3, m_hs);  // T = D .* T'
			// dW2s[0,:] += sum_b T
			N2B_ISSUE_NOWAIT(gemm<16>(WG_W2sT, mnmaj(sm.X3, 64), mnmaj(sm.E0, 16), 8, true));
			// ---- B6: grid gradient (first + second order merged, one reduction per corner); runs while the tensor pipe
			// finishes the tile's last weight-gradient GEMM
			const bool want_dx = DYN && a.delta_sums != nullptr, do_grid = !DYN || a.grad_grid != nullptr;
			float dxp[3] = {0.f, 0.f, 0.f};  // this thread's levels' share of dL/dx (first-order backward of the encoding)
			{
				float dzv[8];
				tmem_ld8(R1 + 8 * part, dzv);
				tc::tmem_ld_wait();
#pragma unroll
				for (int j = 0; j < 4; ++j) {
					const uint32_t l = (uint32_t)(part + 4 * j);
					if (l < a.lv.n_active) {
						const float dz0 = __half2float(__float2half_rn(dzv[2 * j]));
						const float dz1 = __half2float(__float2half_rn(dzv[2 * j + 1]));
						if (want_dx) {
#pragma unroll
							for (int e = 0; e < 3; ++e) dxp[e] = __fmaf_rn(J[j][2 * e], dz0, __fmaf_rn(J[j][2 * e + 1], dz1, dxp[e]));
						}
						if (!do_grid) continue;  // the canonical model is frozen (a frame's first steps train the motion alone)
						const float2 gef = __half22float2(ge[j]);
						const LevelGeom g2 = level_geom(a.lv, l, x);
						const float scale = a.lv.scale[l];
						const float bxv[2] = {-scale * v3[0], scale * v3[0]}, byv[2] = {-scale * v3[1], scale * v3[1]};
						const float bzv[2] = {-scale * v3[2], scale * v3[2]};
						if (j < kMergedJ) {
							// Coarse levels: consecutive samples of a ray sit in the same cell, and thousands of samples hit the same few
							// hundred entries, where the L2 atomics serialise.  Lanes are consecutive samples: sum each run of lanes with
							// the same cell inside the warp (segmented shuffle reduction) and let the run's first lane add the total.
							const uint32_t px = __shfl_up_sync(0xffffffffu, g2.hx[0], 1), py = __shfl_up_sync(0xffffffffu, g2.hy[0], 1);
							const uint32_t pz = __shfl_up_sync(0xffffffffu, g2.hz[0], 1);
							const bool cell_head = lane == 0 || px != g2.hx[0] || py != g2.hy[0] || pz != g2.hz[0];
							const uint32_t hmask = __ballot_sync(0xffffffffu, cell_head);
							const uint32_t after = (hmask >> lane) >> 1;
							const uint32_t run_rest = after ? (uint32_t)__ffs((int)after) - 1u : 31u - (uint32_t)lane;  // lanes behind this one in its run
							// Runs are cut into pieces of kPiece lanes (a ray leaves about a dozen samples in a batch, fewer per cell on
							// the middle levels), so log2(kPiece) shuffle steps do.
							const uint32_t kPiece = j == 0 ? 8u : 4u;  // (j is an unrolled loop index: a constant after unrolling)
							const uint32_t pos = (uint32_t)lane - (31u - (uint32_t)__clz((int)(hmask & (0xffffffffu >> (31 - lane)))));
							const bool head = (pos & (kPiece - 1u)) == 0u;
							const uint32_t rest = min(run_rest, kPiece - 1u - (pos & (kPiece - 1u)));
#pragma unroll
							for (uint32_t k = 0; k < 8; ++k) {
								const uint32_t bx = k & 1u, by = (k >> 1) & 1u, bz = (k >> 2) & 1u;
								const float p = g2.ax[bx] * g2.ay[by];
								const float qq = bxv[bx] * g2.ay[by] + g2.ax[bx] * byv[by];
								const float w = p * g2.az[bz];
								const float coef = qq * g2.az[bz] + p * bzv[bz];
								float v0 = valid ? __fmaf_rn(w, dz0, coef * gef.x) : 0.f, v1 = valid ? __fmaf_rn(w, dz1, coef * gef.y) : 0.f;
#pragma unroll
								for (uint32_t d = 1; d < kPiece; d <<= 1) {
									const float o0 = __shfl_down_sync(0xffffffffu, v0, d), o1 = __shfl_down_sync(0xffffffffu, v1, d);
									if (d <= rest) {
										v0 += o0;
										v1 += o1;
									}
								}
								if (head && (v0 != 0.f || v1 != 0.f)) red_add_h2(a.grad_grid, geom_index(g2, k), v0, v1);
							}
						} else if (valid) {
							// Fine levels: the two x-neighbours of a corner pair are one aligned 8-byte pair of entries whenever their
							// indices differ in bit 0 only (dense: an even index; hashed: an even x, because x ^ h and (x + 1) ^ h then
							// differ in bit 0 only): one vector reduction instead of two.
#pragma unroll
							for (uint32_t k = 0; k < 8; k += 2) {
								const uint32_t by = (k >> 1) & 1u, bz = (k >> 2) & 1u;
								float v[2][2];
#pragma unroll
								for (uint32_t bx = 0; bx < 2; ++bx) {
									const float p = g2.ax[bx] * g2.ay[by];
									const float qq = bxv[bx] * g2.ay[by] + g2.ax[bx] * byv[by];
									const float w = p * g2.az[bz];
									const float coef = qq * g2.az[bz] + p * bzv[bz];
									v[bx][0] = __fmaf_rn(w, dz0, coef * gef.x);
									v[bx][1] = __fmaf_rn(w, dz1, coef * gef.y);
								}
								const uint32_t e0 = geom_index(g2, k), e1 = geom_index(g2, k + 1u);
								if ((e0 ^ e1) == 1u) {
									if (e0 & 1u) red_add_h2x2(a.grad_grid, e1, v[1][0], v[1][1], v[0][0], v[0][1]);
									else red_add_h2x2(a.grad_grid, e0, v[0][0], v[0][1], v[1][0], v[1][1]);
								} else {
									red_add_h2(a.grad_grid, e0, v[0][0], v[0][1]);
									red_add_h2(a.grad_grid, e1, v[1][0], v[1][1]);
								}
							}
						}
					}
				}
			}
			if (want_dx) {
				// ---- gradient for the DeltaNetwork (nerf_network.h:589-612): dL/dx' = encoding dL/dx + xyz rows of both networks'
				// input gradients; its twelve batch sums: sum dL/dx' and sum dL/dx' (x) (x + t) (common_operation.cuh:810-831)
#pragma unroll
				for (int e = 0; e < 3; ++e) sm.nrm[part][s][e] = dxp[e];
				__syncthreads();
				if (part == 0) {
					float dzp[8];
					tmem_ld8(R1 + 32, dzp);  // xyz columns of the SDF-net input gradient
					tc::tmem_ld_wait();
					float sums[12];
#pragma unroll
					for (int k = 0; k < 12; ++k) sums[k] = 0.f;
					if (valid) {
						const float* c = a.coords + (size_t)i * a.coord_stride;
						float l3[3], vv[3];
#pragma unroll
						for (int e = 0; e < 3; ++e) {
							l3[e] = (((sm.nrm[0][s][e] + sm.nrm[1][s][e]) + sm.nrm[2][s][e]) + sm.nrm[3][s][e]) + sm.dxc[s][e] +
							        __half2float(__float2half_rn(dzp[e]));
							vv[e] = c[e] + sm.motion[9 + e];
						}
#pragma unroll
						for (int r = 0; r < 3; ++r) {
							sums[r] = l3[r];
#pragma unroll
							for (int k = 0; k < 3; ++k) sums[3 + r * 3 + k] = l3[r] * vv[k];
						}
					}
#pragma unroll
					for (int k = 0; k < 12; ++k) {
#pragma unroll
						for (int o = 16; o > 0; o >>= 1) sums[k] += __shfl_xor_sync(0xffffffffu, sums[k], o);
						if (lane == 0 && sums[k] != 0.f) atomicAdd(&sm.dsum[k], sums[k]);
					}
				}
			}
			pending = true;
			first = false;
		}
		if constexpr (MODE == MODE_FWD) {
			tc::fence_before_sync();
			__syncthreads();  // the output rows are out of tensor memory: tiles and accumulators are free for the next round
		}
	}
	if (pending) {
		N2B_WAIT();
	}
#undef N2B_ISSUE
#undef N2B_ISSUE_TAIL
#undef N2B_ISSUE_NOWAIT
#undef N2B_WAIT
	if (!ok) atomicOr(&g_tc_error, 1u);
	tc::fence_before_sync();
	__syncthreads();
	tc::fence_after_sync();

	if constexpr (MODE == MODE_TRAIN) {
		// ---- flush the weight gradients held in tensor memory (rows 0..63 of each accumulator)
		if (DYN && a.delta_sums && tid < 12 && sm.dsum[tid] != 0.f) atomicAdd(a.delta_sums + tid, sm.dsum[tid]);
		if (ok && !first && s < 64 && (!DYN || a.grad_mlp)) {
			float v[16];
			if (part == 0) {
#pragma unroll
				for (int q = 0; q < 4; ++q) {
					tc::tmem_ld16(WG_W2c + lrow + 16 * q, v);
					tc::tmem_ld_wait();
#pragma unroll
					for (int e = 0; e < 16; ++e)
						if (v[e] != 0.f) atomicAdd(a.grad_mlp + NEUS2B_RGB_W2 + s * 64 + 16 * q + e, v[e]);
				}
			} else if (part == 1) {
#pragma unroll
				for (int q = 0; q < 3; ++q) {
					tc::tmem_ld16(WG_W1c + lrow + 16 * q, v);
					tc::tmem_ld_wait();
#pragma unroll
					for (int e = 0; e < 16; ++e)
						if (v[e] != 0.f) atomicAdd(a.grad_mlp + NEUS2B_RGB_W1 + s * 48 + 16 * q + e, v[e]);
				}
			} else if (part == 2) {
#pragma unroll
				for (int q = 0; q < 3; ++q) {
					tc::tmem_ld16(WG_W1s + lrow + 16 * q, v);
					tc::tmem_ld_wait();
#pragma unroll
					for (int e = 0; e < 16; ++e)
						if (v[e] != 0.f) atomicAdd(a.grad_mlp + NEUS2B_SDF_W1 + s * 48 + tc_orig_col(16 * q + e), v[e]);
				}
			} else {
				tc::tmem_ld16(WG_W3cT + lrow, v);  // [in = s][out]
				tc::tmem_ld_wait();
#pragma unroll
				for (int e = 0; e < 16; ++e)
					if (v[e] != 0.f) atomicAdd(a.grad_mlp + NEUS2B_RGB_W3 + e * 64 + s, v[e]);
				tc::tmem_ld16(WG_W2sT + lrow, v);
				tc::tmem_ld_wait();
#pragma unroll
				for (int e = 0; e < 16; ++e)
					if (v[e] != 0.f) atomicAdd(a.grad_mlp + NEUS2B_SDF_W2 + e * 64 + s, v[e]);
			}
		}
		// variance gradient = sum of row 7 over the batch (:452-460)
#pragma unroll
		for (int o = 16; o > 0; o >>= 1) var_grad += __shfl_xor_sync(0xffffffffu, var_grad, o);
		if ((tid & 31) == 0) sm.red[warp] = var_grad;
		__syncthreads();
		if (tid == 0) {
			float t = 0.f;
			for (int w = 0; w < kThreads / 32; ++w) t += sm.red[w];
			if (t != 0.f && (!DYN || a.grad_var)) atomicAdd(a.grad_var, t);
		}
	}
	tc::fence_before_sync();
	__syncthreads();
	if (warp == 0) tc::tmem_dealloc(tm, kTmemCols);
}

template <int MODE, bool DYN>
static int launch(const NeusArgs& a, uint32_t n_upper, cudaStream_t stream) {
	const size_t smem = sizeof(Smem<MODE, DYN>) + 128;
	N2B_CHECK_CUDA(cudaFuncSetAttribute(neus_tc_kernel<MODE, DYN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	uint32_t ctas = (n_upper + 127u) / 128u;
	const uint32_t per_sm = 1u;
	if (ctas > kSMs * per_sm) ctas = kSMs * per_sm;
	if (ctas == 0) return NEUS2B_OK;
	neus_tc_kernel<MODE, DYN><<<ctas, kThreads, smem, stream>>>(a);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

}  // namespace tcf

int launch_neus_tc_forward(const NeusArgs& a, uint32_t n_upper, cudaStream_t stream) {
	return a.delta ? tcf::launch<MODE_FWD, true>(a, n_upper, stream) : tcf::launch<MODE_FWD, false>(a, n_upper, stream);
}
int launch_neus_tc_train(const NeusArgs& a, uint32_t n_upper, cudaStream_t stream) {
	const bool dynamic = a.delta || a.delta_sums || !a.grad_grid || !a.grad_mlp || !a.grad_var;
	return dynamic ? tcf::launch<MODE_TRAIN, true>(a, n_upper, stream) : tcf::launch<MODE_TRAIN, false>(a, n_upper, stream);
}
int read_tc_error(uint32_t* h_flags) {
	uint32_t v = 0;
	cudaError_t e = cudaMemcpyFromSymbol(&v, tcf::g_tc_error, sizeof(v));
	if (e != cudaSuccess) return (int)e;
	*h_flags = v;
	return NEUS2B_OK;
}
int write_tc_error(uint32_t flags) {
	cudaError_t e = cudaMemcpyToSymbol(tcf::g_tc_error, &flags, sizeof(flags));
	return e == cudaSuccess ? NEUS2B_OK : (int)e;
}
// Device address of the error word on the current device (for kernels of other translation units that report it).
int tc_error_device_ptr(const uint32_t** d_ptr) {
	void* p = nullptr;
	cudaError_t e = cudaGetSymbolAddress(&p, tcf::g_tc_error);
	if (e != cudaSuccess) return (int)e;
	*d_ptr = (const uint32_t*)p;
	return NEUS2B_OK;
}

}  // namespace n2b
