// Warp-level tensor-core building blocks on 16-row fp16 tiles held in shared memory.
// mma.sync.m16n8k16 (fp16 in, fp32 accumulate) with ldmatrix operand loads.  Every tile is row-major
// [16][ld] with ld a multiple of 8 halves (16-byte rows, as ldmatrix needs) and ld/8 odd, so the 8 row
// addresses of one ldmatrix phase fall in distinct bank groups.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace n2b {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
	asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
	             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
	             : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
	asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
	             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
	             : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
	asm volatile(
	    "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
	    : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
	    : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
	__half2 h = __floats2half2_rn(a, b);
	return *reinterpret_cast<uint32_t*>(&h);
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
	for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
}

// C[16][N] += A[16][K] * W^T, W stored row-major [N][K] (a layer's weight matrix [out][in]).
// N multiple of 16, K multiple of 16.
template <int N, int K>
__device__ __forceinline__ void warp_gemm_nt(float (&acc)[N / 8][4], const __half* A, int lda, const __half* W, int ldw, int lane) {
	const int r = lane & 7, i = lane >> 3;
#pragma unroll
	for (int kk = 0; kk < K / 16; ++kk) {
		uint32_t a[4];
		ldsm_x4(a, A + (r + (i & 1) * 8) * lda + kk * 16 + (i >> 1) * 8);
#pragma unroll
		for (int nt = 0; nt < N / 8; nt += 2) {
			uint32_t b[4];
			ldsm_x4(b, W + (nt * 8 + r + (i >> 1) * 8) * ldw + kk * 16 + (i & 1) * 8);
			mma_16816(acc[nt], a, b[0], b[1]);
			mma_16816(acc[nt + 1], a, b[2], b[3]);
		}
	}
}

// C[16][NIN] += D[16][NOUT] * W, W stored row-major [NOUT][NIN] (input gradient of a layer).
// NIN, NOUT multiples of 16.
template <int NIN, int NOUT>
__device__ __forceinline__ void warp_gemm_nn(float (&acc)[NIN / 8][4], const __half* D, int ldd, const __half* W, int ldw, int lane) {
	const int r = lane & 7, i = lane >> 3;
#pragma unroll
	for (int kk = 0; kk < NOUT / 16; ++kk) {
		uint32_t a[4];
		ldsm_x4(a, D + (r + (i & 1) * 8) * ldd + kk * 16 + (i >> 1) * 8);
#pragma unroll
		for (int nt = 0; nt < NIN / 8; nt += 2) {
			uint32_t b[4];
			ldsm_x4_trans(b, W + (kk * 16 + r + (i & 1) * 8) * ldw + nt * 8 + (i >> 1) * 8);
			mma_16816(acc[nt], a, b[0], b[1]);
			mma_16816(acc[nt + 1], a, b[2], b[3]);
		}
	}
}

// One m-tile (16 output rows m0..m0+15) of dW[M][N] += D^T * Z over the 16 samples of the tile:
// D stored [16 samples][M..], Z stored [16 samples][N..].
template <int N>
__device__ __forceinline__ void warp_wgrad_mtile(float (&acc)[N / 8][4], const __half* D, int ldd, int m0, const __half* Z, int ldz,
                                                 int lane) {
	const int r = lane & 7, i = lane >> 3;
	uint32_t a[4];
	ldsm_x4_trans(a, D + (r + (i >> 1) * 8) * ldd + m0 + (i & 1) * 8);
#pragma unroll
	for (int nt = 0; nt < N / 8; nt += 2) {
		uint32_t b[4];
		ldsm_x4_trans(b, Z + (r + (i & 1) * 8) * ldz + nt * 8 + (i >> 1) * 8);
		mma_16816(acc[nt], a, b[0], b[1]);
		mma_16816(acc[nt + 1], a, b[2], b[3]);
	}
}

// Store a C tile (fp32 accumulators) as fp16 into a row-major tile, optional ReLU.
template <int N, bool RELU>
__device__ __forceinline__ void store_acc_half(const float (&acc)[N / 8][4], __half* T, int ldt, int lane) {
	const int g = lane >> 2, t = lane & 3;
#pragma unroll
	for (int nt = 0; nt < N / 8; ++nt) {
		float v0 = acc[nt][0], v1 = acc[nt][1], v2 = acc[nt][2], v3 = acc[nt][3];
		if (RELU) {
			v0 = fmaxf(v0, 0.f);
			v1 = fmaxf(v1, 0.f);
			v2 = fmaxf(v2, 0.f);
			v3 = fmaxf(v3, 0.f);
		}
		*reinterpret_cast<uint32_t*>(T + g * ldt + nt * 8 + 2 * t) = pack_h2(v0, v1);
		*reinterpret_cast<uint32_t*>(T + (g + 8) * ldt + nt * 8 + 2 * t) = pack_h2(v2, v3);
	}
}

// Store a C tile as fp16 masked by the sign of an activation tile of the same shape (ReLU backward):
// out = act > 0 ? round_half(acc) : 0.
template <int N>
__device__ __forceinline__ void store_acc_half_masked(const float (&acc)[N / 8][4], const __half* act, int lda, __half* T, int ldt,
                                                      int lane) {
	const int g = lane >> 2, t = lane & 3;
	const __half2 zero = __floats2half2_rn(0.f, 0.f);
#pragma unroll
	for (int nt = 0; nt < N / 8; ++nt) {
		__half2 m0 = *reinterpret_cast<const __half2*>(act + g * lda + nt * 8 + 2 * t);
		__half2 m1 = *reinterpret_cast<const __half2*>(act + (g + 8) * lda + nt * 8 + 2 * t);
		__half2 v0 = __floats2half2_rn(acc[nt][0], acc[nt][1]);
		__half2 v1 = __floats2half2_rn(acc[nt][2], acc[nt][3]);
		v0 = __hmul2(v0, __hgt2(m0, zero));  // __hgt2 gives 1.0 / 0.0 per lane
		v1 = __hmul2(v1, __hgt2(m1, zero));
		*reinterpret_cast<__half2*>(T + g * ldt + nt * 8 + 2 * t) = v0;
		*reinterpret_cast<__half2*>(T + (g + 8) * ldt + nt * 8 + 2 * t) = v1;
	}
}

// Add a C tile (one m-tile of a weight gradient) into an fp32 accumulator matrix in shared memory.
// Lanes with odd row group start with the odd column so the 32 lanes of one instruction hit 32 banks
// (needs ldw % 8 == 4).
template <int N>
__device__ __forceinline__ void smem_accumulate(const float (&acc)[N / 8][4], float* dW, int ldw, int m0, int lane) {
	const int g = lane >> 2, t = lane & 3;
	float* r0 = dW + (m0 + g) * ldw + 2 * t;
	float* r1 = dW + (m0 + g + 8) * ldw + 2 * t;
	const int odd = g & 1;
#pragma unroll
	for (int nt = 0; nt < N / 8; ++nt) {
		atomicAdd(r0 + nt * 8 + odd, odd ? acc[nt][1] : acc[nt][0]);
		atomicAdd(r0 + nt * 8 + (odd ^ 1), odd ? acc[nt][0] : acc[nt][1]);
		atomicAdd(r1 + nt * 8 + odd, odd ? acc[nt][3] : acc[nt][2]);
		atomicAdd(r1 + nt * 8 + (odd ^ 1), odd ? acc[nt][2] : acc[nt][3]);
	}
}

}  // namespace n2b
