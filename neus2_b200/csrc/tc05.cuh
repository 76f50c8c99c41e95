// tcgen05 / TMEM building blocks (sm_100a): 5th-generation tensor-core MMA issued by one thread, operands read from
// shared memory through matrix descriptors, fp32 accumulators in tensor memory, completion through an mbarrier.
//
// Shared-memory tiles use the no-swizzle "core matrix" layout the descriptors describe: a [R][C] fp16 tile is cut into
// 8x8 blocks of 128 contiguous bytes (8 rows of 16 bytes); element (r, c) lives at
//     (r / 8) * (C * 16) + (c / 8) * 128 + (r % 8) * 16 + (c % 8) * 2.
// The same bytes serve two roles:
//   * K-major operand  (rows = M or N, columns = K):   SBO = C * 16 (next 8 rows), LBO = 128 (next 8 columns);
//   * MN-major operand (columns = M or N, rows = K):    SBO = 128 (next 8 columns), LBO = C * 16 (next 8 rows),
// so an activation tile [samples][features] is the A operand of a forward GEMM (K-major) and, untouched, an operand of
// the weight-gradient GEMM that contracts over samples (MN-major).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace n2b {
namespace tc {

__device__ __forceinline__ uint32_t blk_off(int r, int c, int ncols) {  // byte offset inside a blocked tile
	return (uint32_t)((r >> 3) * (ncols * 16) + (c >> 3) * 128 + (r & 7) * 16 + (c & 7) * 2);
}

// 64-bit shared-memory matrix descriptor, SWIZZLE_NONE, version 1 (Blackwell).  Offsets in bytes, multiples of 16.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
	return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) |
	       (1ull << 46);
}

// 32-bit instruction descriptor for kind::f16: fp16 A/B, fp32 accumulate, dense.
__device__ __forceinline__ constexpr uint32_t idesc_f16(int M, int N, int a_mn_major, int b_mn_major) {
	return (1u << 4) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
// Bounded wait: returns false if the phase did not complete (the caller raises an error flag and bails out).
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
	for (uint32_t it = 0; it < (1u << 22); ++it) {
		uint32_t ok;
		asm volatile(
		    "{\n\t.reg .pred p;\n\t"
		    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
		    "selp.u32 %0, 1, 0, p;\n\t}"
		    : "=r"(ok)
		    : "r"(mbar), "r"(parity)
		    : "memory");
		if (ok) return true;
	}
	return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// One full warp allocates / frees `ncols` (power of two >= 32) tensor-memory columns; the base address lands in smem.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[M][N] (+)= A[M][16] * B[N][16]^T, issued by ONE thread.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
	asm volatile(
	    "{\n\t.reg .pred p;\n\t"
	    "setp.ne.b32 p, %4, 0;\n\t"
	    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
	    :
	    : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
	    : "memory");
}
// Arrive on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void commit(uint32_t mbar) {
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}

// Each thread of a warp reads 16 consecutive fp32 columns of its own tensor-memory lane (lane = 32 * (warp % 4) + laneid).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
	uint32_t r[16];
	asm volatile(
	    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
	    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
	      "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
	    : "r"(taddr)
	    : "memory");
#pragma unroll
	for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// C[128][N] = A[128][K] * W[N][K]^T with both operands K-major blocked tiles (A: [128][K], W: [N][K]).
template <int N, int K>
__device__ __forceinline__ void issue_gemm_kmajor(uint32_t d_tmem, uint32_t a_saddr, uint32_t w_saddr, bool accumulate_first = false) {
	constexpr uint32_t id = idesc_f16(128, N, 0, 0);
#pragma unroll
	for (int kk = 0; kk < K / 16; ++kk) {
		const uint64_t ad = smem_desc(a_saddr + kk * 256, 128, K * 16);
		const uint64_t bd = smem_desc(w_saddr + kk * 256, 128, K * 16);
		mma_f16(d_tmem, ad, bd, id, (kk > 0 || accumulate_first) ? 1u : 0u);
	}
}

}  // namespace tc
}  // namespace n2b
