// Stand-alone 64-neuron ReLU MLP kernels (the tcnn FullyFusedMLP entry points the reference calls:
// forward, backward, backward_backward_input).  Same warp-tile scheme as the fused NeuS kernels: a warp owns
// 16 samples, activations stay in shared memory between layers, mma.sync m16n8k16 with fp32 accumulation.
#include "common.cuh"
#include "mma_tile.cuh"

namespace n2b {

constexpr int kMlpWarps = 8;
constexpr int MLD64 = 72;
constexpr int MLD16 = 24;
constexpr int MGLD64 = 68;

template <int IN, int NH>
struct MlpWeights {
	__half W1[64 * (IN + 8)];
	__half W2[(NH == 2 ? 64 : 1) * MLD64];
	__half Wo[16 * MLD64];
};
template <int IN, int NH>
struct MlpGrads {
	float W1[64 * (IN + 4)];
	float W2[(NH == 2 ? 64 : 1) * MGLD64];
	float Wo[16 * MGLD64];
};

template <int IN, int NH>
__device__ void mlp_stage_weights(MlpWeights<IN, NH>& w, const __half* p, int tid, int nt) {
	for (int e = tid; e < 64 * IN; e += nt) w.W1[(e / IN) * (IN + 8) + e % IN] = p[e];
	if (NH == 2)
		for (int e = tid; e < 64 * 64; e += nt) w.W2[(e / 64) * MLD64 + e % 64] = p[64 * IN + e];
	const int off = 64 * IN + (NH - 1) * 4096;
	for (int e = tid; e < 16 * 64; e += nt) w.Wo[(e / 64) * MLD64 + e % 64] = p[off + e];
}

// copy rows [row0, row0+16) of a global [n][W] fp16 matrix (row stride gstride halves) into a tile, zero-filling past n
template <int W>
__device__ __forceinline__ void load_tile(const __half* g, size_t gstride, uint32_t row0, uint32_t n, __half* T, int ld, int lane) {
	for (int e = lane; e < 16 * (W / 8); e += 32) {
		const int r = e / (W / 8), c = (e % (W / 8)) * 8;
		uint4 v = make_uint4(0, 0, 0, 0);
		if (row0 + r < n) v = *reinterpret_cast<const uint4*>(g + (size_t)(row0 + r) * gstride + c);
		*reinterpret_cast<uint4*>(T + r * ld + c) = v;
	}
}
template <int W>
__device__ __forceinline__ void store_tile(__half* g, size_t gstride, uint32_t row0, uint32_t n, const __half* T, int ld, int lane) {
	for (int e = lane; e < 16 * (W / 8); e += 32) {
		const int r = e / (W / 8), c = (e % (W / 8)) * 8;
		if (row0 + r < n) *reinterpret_cast<uint4*>(g + (size_t)(row0 + r) * gstride + c) = *reinterpret_cast<const uint4*>(T + r * ld + c);
	}
}

template <int IN, int NH>
struct FwdSmem {
	MlpWeights<IN, NH> w;
	struct {
		__half X[16 * (IN + 8)], H0[16 * MLD64], H1[16 * MLD64], Y[16 * MLD16];
	} t[kMlpWarps];
};

template <int IN, int NH>
__global__ void __launch_bounds__(kMlpWarps * 32) mlp_forward_kernel(uint32_t n, const __half* __restrict__ weights,
                                                                      const __half* __restrict__ in, __half* __restrict__ out,
                                                                      __half* __restrict__ hidden) {
	extern __shared__ __align__(16) unsigned char smem_raw[];
	auto& sm = *reinterpret_cast<FwdSmem<IN, NH>*>(smem_raw);
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	mlp_stage_weights<IN, NH>(sm.w, weights, tid, blockDim.x);
	__syncthreads();
	auto& T = sm.t[warp];
	const uint32_t n_tiles = (n + 15u) / 16u;
	for (uint32_t tile = blockIdx.x * kMlpWarps + warp; tile < n_tiles; tile += gridDim.x * kMlpWarps) {
		const uint32_t row0 = tile * 16u;
		load_tile<IN>(in, IN, row0, n, T.X, IN + 8, lane);
		__syncwarp();
		float acc[8][4];
		zero_acc<8>(acc);
		warp_gemm_nt<64, IN>(acc, T.X, IN + 8, sm.w.W1, IN + 8, lane);
		store_acc_half<64, true>(acc, T.H0, MLD64, lane);
		__syncwarp();
		if (hidden) store_tile<64>(hidden, (size_t)NH * 64, row0, n, T.H0, MLD64, lane);
		const __half* last = T.H0;
		if (NH == 2) {
			zero_acc<8>(acc);
			warp_gemm_nt<64, 64>(acc, T.H0, MLD64, sm.w.W2, MLD64, lane);
			store_acc_half<64, true>(acc, T.H1, MLD64, lane);
			__syncwarp();
			if (hidden) store_tile<64>(hidden + 64, (size_t)NH * 64, row0, n, T.H1, MLD64, lane);
			last = T.H1;
		}
		float acc2[2][4];
		zero_acc<2>(acc2);
		warp_gemm_nt<16, 64>(acc2, last, MLD64, sm.w.Wo, MLD64, lane);
		store_acc_half<16, false>(acc2, T.Y, MLD16, lane);
		__syncwarp();
		store_tile<16>(out, 16, row0, n, T.Y, MLD16, lane);
		__syncwarp();
	}
}

template <int IN, int NH>
struct BwdSmem {
	MlpWeights<IN, NH> w;
	MlpGrads<IN, NH> g;
	struct {
		__half X[16 * (IN + 8)], H0[16 * MLD64], H1[16 * MLD64], D0[16 * MLD64], D1[16 * MLD64], Y[16 * MLD16];
	} t[kMlpWarps];
};

template <int IN, int NH>
__global__ void __launch_bounds__(kMlpWarps * 32) mlp_backward_kernel(uint32_t n, const __half* __restrict__ weights,
                                                                       const __half* __restrict__ in, const __half* __restrict__ hidden,
                                                                       const __half* __restrict__ dL_dout, __half* __restrict__ dL_din,
                                                                       float* __restrict__ wgrad) {
	extern __shared__ __align__(16) unsigned char smem_raw[];
	auto& sm = *reinterpret_cast<BwdSmem<IN, NH>*>(smem_raw);
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	mlp_stage_weights<IN, NH>(sm.w, weights, tid, blockDim.x);
	{
		float* g = reinterpret_cast<float*>(&sm.g);
		for (int e = tid; e < (int)(sizeof(sm.g) / 4); e += blockDim.x) g[e] = 0.f;
	}
	__syncthreads();
	auto& T = sm.t[warp];
	const uint32_t n_tiles = (n + 15u) / 16u;
	for (uint32_t tile = blockIdx.x * kMlpWarps + warp; tile < n_tiles; tile += gridDim.x * kMlpWarps) {
		const uint32_t row0 = tile * 16u;
		load_tile<IN>(in, IN, row0, n, T.X, IN + 8, lane);
		load_tile<64>(hidden, (size_t)NH * 64, row0, n, T.H0, MLD64, lane);
		if (NH == 2) load_tile<64>(hidden + 64, (size_t)NH * 64, row0, n, T.H1, MLD64, lane);
		load_tile<16>(dL_dout, 16, row0, n, T.Y, MLD16, lane);
		__syncwarp();
		const __half* last = NH == 2 ? T.H1 : T.H0;
		float acc[8][4];
		// output layer
		if (wgrad) {
			zero_acc<8>(acc);
			warp_wgrad_mtile<64>(acc, T.Y, MLD16, 0, last, MLD64, lane);
			smem_accumulate<64>(acc, sm.g.Wo, MGLD64, 0, lane);
		}
		zero_acc<8>(acc);
		warp_gemm_nn<64, 16>(acc, T.Y, MLD16, sm.w.Wo, MLD64, lane);
		store_acc_half_masked<64>(acc, last, MLD64, T.D1, MLD64, lane);
		__syncwarp();
		const __half* dfirst = T.D1;
		if (NH == 2) {
			if (wgrad) {
#pragma unroll 1
				for (int mt = 0; mt < 4; ++mt) {
					zero_acc<8>(acc);
					warp_wgrad_mtile<64>(acc, T.D1, MLD64, mt * 16, T.H0, MLD64, lane);
					smem_accumulate<64>(acc, sm.g.W2, MGLD64, mt * 16, lane);
				}
			}
			zero_acc<8>(acc);
			warp_gemm_nn<64, 64>(acc, T.D1, MLD64, sm.w.W2, MLD64, lane);
			store_acc_half_masked<64>(acc, T.H0, MLD64, T.D0, MLD64, lane);
			__syncwarp();
			dfirst = T.D0;
		}
		float acc1[IN / 8][4];
		if (wgrad) {
#pragma unroll 1
			for (int mt = 0; mt < 4; ++mt) {
				zero_acc<IN / 8>(acc1);
				warp_wgrad_mtile<IN>(acc1, dfirst, MLD64, mt * 16, T.X, IN + 8, lane);
				smem_accumulate<IN>(acc1, sm.g.W1, IN + 4, mt * 16, lane);
			}
		}
		if (dL_din) {
			zero_acc<IN / 8>(acc1);
			warp_gemm_nn<IN, 64>(acc1, dfirst, MLD64, sm.w.W1, IN + 8, lane);
			__syncwarp();  // X is overwritten with its own gradient
			store_acc_half<IN, false>(acc1, T.X, IN + 8, lane);
			__syncwarp();
			store_tile<IN>(dL_din, IN, row0, n, T.X, IN + 8, lane);
		}
		__syncwarp();
	}
	if (wgrad) {
		__syncthreads();
		for (int e = tid; e < 64 * IN; e += blockDim.x) {
			const float v = sm.g.W1[(e / IN) * (IN + 4) + e % IN];
			if (v != 0.f) atomicAdd(wgrad + e, v);
		}
		if (NH == 2)
			for (int e = tid; e < 64 * 64; e += blockDim.x) {
				const float v = sm.g.W2[(e / 64) * MGLD64 + e % 64];
				if (v != 0.f) atomicAdd(wgrad + 64 * IN + e, v);
			}
		const int off = 64 * IN + (NH - 1) * 4096;
		for (int e = tid; e < 16 * 64; e += blockDim.x) {
			const float v = sm.g.Wo[(e / 64) * MGLD64 + e % 64];
			if (v != 0.f) atomicAdd(wgrad + off + e, v);
		}
	}
}

template <int IN>
struct Bwd2Smem {
	MlpWeights<IN, 1> w;
	MlpGrads<IN, 1> g;
	struct {
		__half U[16 * (IN + 8)], H[16 * MLD64], Tt[16 * MLD64], S[16 * MLD64], Y[16 * MLD16];
	} t[kMlpWarps];
};

// t = D .* (W1 u);  dWo += dy^T t;  s = D .* (Wo^T dy);  dW1 += s^T u
template <int IN>
__global__ void __launch_bounds__(kMlpWarps * 32) mlp_bwd_bwd_kernel(uint32_t n, const __half* __restrict__ weights,
                                                                      const __half* __restrict__ hidden, const __half* __restrict__ u,
                                                                      const __half* __restrict__ dy, float* __restrict__ wgrad) {
	extern __shared__ __align__(16) unsigned char smem_raw[];
	auto& sm = *reinterpret_cast<Bwd2Smem<IN>*>(smem_raw);
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	mlp_stage_weights<IN, 1>(sm.w, weights, tid, blockDim.x);
	{
		float* g = reinterpret_cast<float*>(&sm.g);
		for (int e = tid; e < (int)(sizeof(sm.g) / 4); e += blockDim.x) g[e] = 0.f;
	}
	__syncthreads();
	auto& T = sm.t[warp];
	const uint32_t n_tiles = (n + 15u) / 16u;
	for (uint32_t tile = blockIdx.x * kMlpWarps + warp; tile < n_tiles; tile += gridDim.x * kMlpWarps) {
		const uint32_t row0 = tile * 16u;
		load_tile<IN>(u, IN, row0, n, T.U, IN + 8, lane);
		load_tile<64>(hidden, 64, row0, n, T.H, MLD64, lane);
		load_tile<16>(dy, 16, row0, n, T.Y, MLD16, lane);
		__syncwarp();
		float acc[8][4];
		zero_acc<8>(acc);
		warp_gemm_nt<64, IN>(acc, T.U, IN + 8, sm.w.W1, IN + 8, lane);
		store_acc_half_masked<64>(acc, T.H, MLD64, T.Tt, MLD64, lane);
		zero_acc<8>(acc);
		warp_gemm_nn<64, 16>(acc, T.Y, MLD16, sm.w.Wo, MLD64, lane);
		store_acc_half_masked<64>(acc, T.H, MLD64, T.S, MLD64, lane);
		__syncwarp();
		zero_acc<8>(acc);
		warp_wgrad_mtile<64>(acc, T.Y, MLD16, 0, T.Tt, MLD64, lane);
		smem_accumulate<64>(acc, sm.g.Wo, MGLD64, 0, lane);
		float acc1[IN / 8][4];
#pragma unroll 1
		for (int mt = 0; mt < 4; ++mt) {
			zero_acc<IN / 8>(acc1);
			warp_wgrad_mtile<IN>(acc1, T.S, MLD64, mt * 16, T.U, IN + 8, lane);
			smem_accumulate<IN>(acc1, sm.g.W1, IN + 4, mt * 16, lane);
		}
		__syncwarp();
	}
	__syncthreads();
	for (int e = tid; e < 64 * IN; e += blockDim.x) {
		const float v = sm.g.W1[(e / IN) * (IN + 4) + e % IN];
		if (v != 0.f) atomicAdd(wgrad + e, v);
	}
	for (int e = tid; e < 16 * 64; e += blockDim.x) {
		const float v = sm.g.Wo[(e / 64) * MGLD64 + e % 64];
		if (v != 0.f) atomicAdd(wgrad + 64 * IN + e, v);
	}
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
	N2B_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
	return NEUS2B_OK;
}
static uint32_t grid_for(uint32_t n) {
	uint32_t ctas = ((n + 15u) / 16u + kMlpWarps - 1) / kMlpWarps;
	return ctas > 2u * kSMs ? 2u * kSMs : ctas;
}

template <int IN, int NH>
static int run_forward(uint32_t n, const uint16_t* w, const uint16_t* in, uint16_t* out, uint16_t* hidden, cudaStream_t s) {
	int rc = set_smem(mlp_forward_kernel<IN, NH>, sizeof(FwdSmem<IN, NH>));
	if (rc) return rc;
	mlp_forward_kernel<IN, NH><<<grid_for(n), kMlpWarps * 32, sizeof(FwdSmem<IN, NH>), s>>>(n, (const __half*)w, (const __half*)in,
	                                                                                        (__half*)out, (__half*)hidden);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}
template <int IN, int NH>
static int run_backward(uint32_t n, const uint16_t* w, const uint16_t* in, const uint16_t* hidden, const uint16_t* dout, uint16_t* din,
                        float* wgrad, cudaStream_t s) {
	int rc = set_smem(mlp_backward_kernel<IN, NH>, sizeof(BwdSmem<IN, NH>));
	if (rc) return rc;
	mlp_backward_kernel<IN, NH><<<grid_for(n) > (uint32_t)kSMs ? kSMs : grid_for(n), kMlpWarps * 32, sizeof(BwdSmem<IN, NH>), s>>>(
	    n, (const __half*)w, (const __half*)in, (const __half*)hidden, (const __half*)dout, (__half*)din, wgrad);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}
template <int IN>
static int run_bwd_bwd(uint32_t n, const uint16_t* w, const uint16_t* hidden, const uint16_t* u, const uint16_t* dy, float* wgrad,
                       cudaStream_t s) {
	int rc = set_smem(mlp_bwd_bwd_kernel<IN>, sizeof(Bwd2Smem<IN>));
	if (rc) return rc;
	mlp_bwd_bwd_kernel<IN><<<grid_for(n) > (uint32_t)kSMs ? kSMs : grid_for(n), kMlpWarps * 32, sizeof(Bwd2Smem<IN>), s>>>(
	    n, (const __half*)w, (const __half*)hidden, (const __half*)u, (const __half*)dy, wgrad);
	N2B_CHECK_LAUNCH();
	return NEUS2B_OK;
}

static size_t mlp_params(uint32_t in_w, uint32_t nh) { return (size_t)64 * in_w + (size_t)(nh - 1) * 4096 + 1024; }

}  // namespace n2b

using namespace n2b;

#define N2B_DISPATCH(IN_W, NHID, CALL)                                  \
	if (IN_W == 48 && NHID == 1) return CALL(48, 1);                    \
	if (IN_W == 48 && NHID == 2) return CALL(48, 2);                    \
	if (IN_W == 32 && NHID == 1) return CALL(32, 1);                    \
	if (IN_W == 32 && NHID == 2) return CALL(32, 2);                    \
	if (IN_W == 64 && NHID == 1) return CALL(64, 1);                    \
	if (IN_W == 64 && NHID == 2) return CALL(64, 2);                    \
	return NEUS2B_E_UNSUPPORTED;

extern "C" int neus2b_mlp_forward(uint32_t n, uint32_t in_width, uint32_t n_hidden, const uint16_t* d_weights, const uint16_t* d_in,
                                  uint16_t* d_out, uint16_t* d_hidden, neus2b_stream_t stream) {
	if (!d_weights || !d_in || !d_out) return NEUS2B_E_INVALID;
	if (((uintptr_t)d_in | (uintptr_t)d_out | (uintptr_t)d_hidden) & 15u) return NEUS2B_E_INVALID;
	if (n == 0) return NEUS2B_OK;
#define CALL(I, H) run_forward<I, H>(n, d_weights, d_in, d_out, d_hidden, stream)
	N2B_DISPATCH(in_width, n_hidden, CALL)
#undef CALL
}

extern "C" int neus2b_mlp_backward(uint32_t n, uint32_t in_width, uint32_t n_hidden, const uint16_t* d_weights, const uint16_t* d_in,
                                   const uint16_t* d_hidden, const uint16_t* d_dL_dout, uint16_t* d_dL_din, float* d_wgrad,
                                   int grad_mode, neus2b_stream_t stream) {
	if (!d_weights || !d_in || !d_hidden || !d_dL_dout) return NEUS2B_E_INVALID;
	if (((uintptr_t)d_in | (uintptr_t)d_hidden | (uintptr_t)d_dL_dout | (uintptr_t)d_dL_din) & 15u) return NEUS2B_E_INVALID;
	if (grad_mode == NEUS2B_GRAD_IGNORE) d_wgrad = nullptr;
	else if (!d_wgrad) return NEUS2B_E_INVALID;
	if (in_width != 32 && in_width != 48 && in_width != 64) return NEUS2B_E_UNSUPPORTED;
	if (n_hidden != 1 && n_hidden != 2) return NEUS2B_E_UNSUPPORTED;
	if (grad_mode == NEUS2B_GRAD_OVERWRITE)
		N2B_CHECK_CUDA(cudaMemsetAsync(d_wgrad, 0, mlp_params(in_width, n_hidden) * sizeof(float), stream));
	if (n == 0) return NEUS2B_OK;
#define CALL(I, H) run_backward<I, H>(n, d_weights, d_in, d_hidden, d_dL_dout, d_dL_din, d_wgrad, stream)
	N2B_DISPATCH(in_width, n_hidden, CALL)
#undef CALL
}

extern "C" int neus2b_mlp_backward_backward_input(uint32_t n, uint32_t in_width, const uint16_t* d_weights, const uint16_t* d_hidden,
                                                  const uint16_t* d_u, const uint16_t* d_dy, float* d_wgrad, int grad_mode,
                                                  neus2b_stream_t stream) {
	if (!d_weights || !d_hidden || !d_u || !d_dy) return NEUS2B_E_INVALID;
	if (((uintptr_t)d_hidden | (uintptr_t)d_u | (uintptr_t)d_dy) & 15u) return NEUS2B_E_INVALID;
	if (grad_mode == NEUS2B_GRAD_IGNORE) return NEUS2B_OK;
	if (!d_wgrad) return NEUS2B_E_INVALID;
	if (in_width != 32 && in_width != 48 && in_width != 64) return NEUS2B_E_UNSUPPORTED;
	if (grad_mode == NEUS2B_GRAD_OVERWRITE) N2B_CHECK_CUDA(cudaMemsetAsync(d_wgrad, 0, mlp_params(in_width, 1) * sizeof(float), stream));
	if (n == 0) return NEUS2B_OK;
	if (in_width == 48) return run_bwd_bwd<48>(n, d_weights, d_hidden, d_u, d_dy, d_wgrad, stream);
	if (in_width == 32) return run_bwd_bwd<32>(n, d_weights, d_hidden, d_u, d_dy, d_wgrad, stream);
	return run_bwd_bwd<64>(n, d_weights, d_hidden, d_u, d_dy, d_wgrad, stream);
}
