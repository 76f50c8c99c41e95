// The learned rigid motion of a dynamic sequence's current frame (the reference's DeltaNetwork,
// include/neural-graphics-primitives/transform_network.h:26-170; kernels common_operation.cuh:42-170, 419-474, 793-849):
// 12 fp16 parameters, transition [0..3] (xyz + one unused) and a 6-D rotation [4..11] (two 3-vectors + two unused),
// turned into a rotation matrix by Gram-Schmidt.
#pragma once
#include <cuda_fp16.h>

namespace n2b {

struct RigidMotion {  // x' = R (x + t - off) + off
	float R[9];       // row-major
	float t[3];
};

// Every product and sum below is one rounded fp32 operation in the written order, on the device as on the host (no fused
// multiply-add): the matrix decides where samples and rays land, and it must be the same numbers wherever it is formed.
__host__ __device__ inline float mul_rn(float a, float b) {
#ifdef __CUDA_ARCH__
	return __fmul_rn(a, b);
#else
	volatile float r = a * b;
	return r;
#endif
}
__host__ __device__ inline float add_rn(float a, float b) {
#ifdef __CUDA_ARCH__
	return __fadd_rn(a, b);
#else
	volatile float r = a + b;
	return r;
#endif
}
__host__ __device__ inline float dot3_rn(const float* a, const float* b) {
	return add_rn(add_rn(mul_rn(a[0], b[0]), mul_rn(a[1], b[1])), mul_rn(a[2], b[2]));
}

// rotation_6d_to_matrix (common_operation.cuh:42-66): columns b1 = a1 / |a1|, b2 = normalised (a2 - (b1 . a2) b1), b1 x b2
__host__ __device__ inline void rotation_6d_to_matrix(const float* a1, const float* a2, float* R) {
	const float n1 = sqrtf(dot3_rn(a1, a1));
	const float b1[3] = {a1[0] / n1, a1[1] / n1, a1[2] / n1};
	const float dt = dot3_rn(b1, a2);
	const float u2[3] = {add_rn(a2[0], -mul_rn(dt, b1[0])), add_rn(a2[1], -mul_rn(dt, b1[1])), add_rn(a2[2], -mul_rn(dt, b1[2]))};
	const float n2 = sqrtf(dot3_rn(u2, u2));
	const float b2[3] = {u2[0] / n2, u2[1] / n2, u2[2] / n2};
	const float b3[3] = {add_rn(mul_rn(b1[1], b2[2]), -mul_rn(b1[2], b2[1])), add_rn(mul_rn(b1[2], b2[0]), -mul_rn(b1[0], b2[2])),
	                     add_rn(mul_rn(b1[0], b2[1]), -mul_rn(b1[1], b2[0]))};
#pragma unroll
	for (int r = 0; r < 3; ++r) {
		R[r * 3 + 0] = b1[r];
		R[r * 3 + 1] = b2[r];
		R[r * 3 + 2] = b3[r];
	}
}

__device__ __forceinline__ RigidMotion load_rigid_motion(const __half* delta) {
	RigidMotion m;
	float a1[3], a2[3];
#pragma unroll
	for (int e = 0; e < 3; ++e) {
		m.t[e] = __half2float(delta[e]);
		a1[e] = __half2float(delta[4 + e]);
		a2[e] = __half2float(delta[7 + e]);
	}
	rotation_6d_to_matrix(a1, a2, m.R);
	return m;
}

__host__ __device__ inline void rotate3(const float* R, const float* v, float* out) {
#pragma unroll
	for (int r = 0; r < 3; ++r) out[r] = dot3_rn(R + r * 3, v);
}

// add_global_movement_with_rotation_6d (common_operation.cuh:419-474): position and (unit-cube coded) direction of one sample
__device__ __forceinline__ void move_sample(const float* R, const float* t, const float* off, float* x, float* dir01) {
	float p[3], q[3], d[3], dr[3];
#pragma unroll
	for (int e = 0; e < 3; ++e) {
		p[e] = add_rn(x[e], add_rn(t[e], -off[e]));
		d[e] = add_rn(mul_rn(dir01[e], 2.0f), -1.0f);
	}
	rotate3(R, p, q);
	rotate3(R, d, dr);
#pragma unroll
	for (int e = 0; e < 3; ++e) {
		x[e] = add_rn(q[e], off[e]);
		dir01[e] = mul_rn(add_rn(dr[e], 1.0f), 0.5f);
	}
}

}  // namespace n2b
