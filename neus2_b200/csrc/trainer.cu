// Host-side training loop: the part of the reference's Testbed that drives one NeuS training step
// (Testbed::train src/testbed.cu:2630-2726, training_prep_nerf / train_nerf / train_nerf_step
// src/testbed_nerf.cu:3434-3990), re-designed so that a step is a fixed sequence of asynchronous launches on one
// stream with no host synchronisation: ray count, sample counts and the batch re-tune live in device memory.
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

namespace n2b {

struct TrainState {  // device resident, one per testbed
	uint32_t rays_per_batch;
	uint32_t n_rays_total;
	uint32_t measured_pre, measured, n_kept, overflow;
	float loss, ek_loss;
	uint32_t nonfinite;     // gradient entries the optimizer pass refused (cumulative; adam_kernel adds to it)
	uint32_t device_error;  // copy of the sticky device error word, taken by the batch tuner
	uint32_t evaluated;     // samples the network pass evaluated (counter 5; 0 = the full pass, which does not count)
};

int tc_error_device_ptr(const uint32_t** d_ptr);  // fused_tc.cu

// Counters::update_after_training (src/testbed_nerf.cu:3406-3432) on the device.
__global__ void tune_kernel(TrainState* st, const uint32_t* __restrict__ counters, uint32_t target, uint32_t max_rays,
                            const uint32_t* __restrict__ device_error) {
	if (threadIdx.x != 0 || blockIdx.x != 0) return;
	st->device_error = *device_error;
	const uint32_t rays = st->rays_per_batch;
	st->n_rays_total += rays;
	st->evaluated = counters[5] ? counters[5] : counters[1];
	st->n_kept = counters[0];
	st->overflow |= counters[3];
	if (counters[1] == 0 || counters[2] == 0) {  // both read as zero (:3411-3416): the batch stays as it is, the next step has the whole buffer
		st->measured_pre = st->measured = 0;
		return;
	}
	st->measured_pre = counters[1];
	st->measured = counters[2];
	uint32_t next = (uint32_t)((float)rays * (float)target / (float)counters[2]);
	next = (next + 127u) / 128u * 128u;
	st->rays_per_batch = max(128u, min(next, max_rays));
}

// loss / ek_loss scalars: sum over the batch's rays, scaled by measured/target (:3423-3425); fixed-shape tree.
__global__ void __launch_bounds__(1024) loss_reduce_kernel(TrainState* st, const float* __restrict__ loss, const float* __restrict__ ek,
                                                           uint32_t target) {
	__shared__ float sl[1024], se[1024];
	const uint32_t n = st->n_kept;
	float a = 0.f, b = 0.f;
	for (uint32_t k = threadIdx.x; k < n; k += 1024) {
		a += loss[k];
		b += ek[k];
	}
	sl[threadIdx.x] = a;
	se[threadIdx.x] = b;
	__syncthreads();
	for (int o = 512; o > 0; o >>= 1) {
		if ((int)threadIdx.x < o) {
			sl[threadIdx.x] += sl[threadIdx.x + o];
			se[threadIdx.x] += se[threadIdx.x + o];
		}
		__syncthreads();
	}
	if (threadIdx.x == 0) {
		const float s = (float)st->measured / (float)target;
		st->loss = sl[0] * s;
		st->ek_loss = se[0] * s;
	}
}

__global__ void master_to_half_kernel(uint64_t n, const float* __restrict__ master, __half* __restrict__ p, __half* __restrict__ pe,
                                      float* __restrict__ ema) {
	for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
		const float w = master[i];
		p[i] = __float2half_rn(w);
		pe[i] = __float2half_rn(w);
		ema[i] = w;
	}
}

// Trainer::deserialize of a snapshot without optimizer state: the stored fp16 parameters become the fp32 master weights and
// the inference (EMA) copies
__global__ void half_to_master_kernel(uint64_t n, const __half* __restrict__ p, float* __restrict__ master, float* __restrict__ ema,
                                      __half* __restrict__ pe) {
	for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
		const __half h = p[i];
		const float w = __half2float(h);
		master[i] = w;
		ema[i] = w;
		pe[i] = h;
	}
}

// generate_grid_samples_nerf_uniform (src/testbed_nerf.cu:586-599): lattice positions x / res, unit aabb
__global__ void sdf_grid_positions_kernel(uint32_t rx, uint32_t ry, uint64_t first, uint32_t n, float ix, float iy, float iz,
                                          float* __restrict__ pos) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= n) return;
	const uint64_t g = first + i;
	const uint32_t x = (uint32_t)(g % rx), y = (uint32_t)((g / rx) % ry), z = (uint32_t)(g / ((uint64_t)rx * ry));
	pos[(size_t)i * 3 + 0] = (float)x * ix;
	pos[(size_t)i * 3 + 1] = (float)y * iy;
	pos[(size_t)i * 3 + 2] = (float)z * iz;
}
// grid_samples_half_to_float (:682-698)
__global__ void half_to_float_kernel(uint32_t n, const __half* __restrict__ src, float* __restrict__ dst) {
	const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i < n) dst[i] = __half2float(src[i]);
}

}  // namespace n2b

using namespace n2b;

struct neus2b_testbed {
	neus2b_testbed_config cfg;
	int device = 0;
	cudaStream_t stream = nullptr;
	uint64_t n_params = 0, n_grid = 0;
	uint32_t max_rays = 1u << 18, max_samples = 0, target = 0;
	uint32_t training_step = 0, ema_step = 0;
	Pcg32 rng, density_rng;
	// parameters / optimizer
	__half *params = nullptr, *params_ema = nullptr, *grad_grid = nullptr;
	float *master = nullptr, *ema_master = nullptr, *adam_m = nullptr, *adam_v = nullptr, *grad_mlp = nullptr, *grad_var = nullptr;
	// occupancy
	float *density_grid = nullptr, *density_tmp = nullptr, *density_mean = nullptr, *occ_pos = nullptr;
	uint8_t* bitfield = nullptr;
	int32_t* occ_bounds = nullptr;  // box of occupied cells (finest level)
	bool occ_bounds_stale = true;   // set by an occupancy update and by handing the bitfield's pointer out
	uint32_t* occ_idx = nullptr;
	__half* occ_sdf = nullptr;
	double* occ_partial = nullptr;
	// batch
	neus2b_ray_workspace ws{};
	__half *mlp_out = nullptr, *dloss = nullptr;
	float *coords_compacted = nullptr, *loss = nullptr, *ek_loss = nullptr;
	TrainState* state = nullptr;
	TrainState* h_state = nullptr;  // pinned
	const uint32_t* d_device_error = nullptr;  // the kernels' sticky error word on this device
	// dataset
	neus2b_dataset ds{};
	float* h_cam = nullptr;  // pinned staging for the camera block
	cudaEvent_t cam_event = nullptr;  // behind the last upload from h_cam
	std::vector<void*> allocs;
	// optional timing of the fused forward+backward kernel inside the step (event pairs on the training stream)
	std::vector<cudaEvent_t> prof_events;
	uint32_t prof_used = 0;
	bool prof_on = false;
	// renderer: buffers for the last requested resolution
	std::vector<void*> render_allocs;
	uint32_t render_pixels = 0;
	neus2b_render_workspace render_ws{};
	float *render_frame = nullptr, *render_depth = nullptr, *render_acc = nullptr, *render_out = nullptr;
	// dynamic sequences (frames after the first): the frame's learned motion and the accumulated movement of the earlier frames
	uint32_t frame = 0;
	bool train_canonical = true, train_delta = false;
	uint32_t canonical_step = 0;  // m_canonical_training_step (src/testbed_nerf.cu:3506-3522)
	uint32_t adam_step = 0, delta_adam_step = 0;  // steps taken by the frame's optimizers (both start afresh with every frame)
	float acc_rotation[9] = {1.f, 0.f, 0.f, 0.f, 1.f, 0.f, 0.f, 0.f, 1.f}, acc_transition[3] = {0.f, 0.f, 0.f};
	__half *delta = nullptr, *delta_ema = nullptr;
	float *delta_master = nullptr, *delta_m = nullptr, *delta_v = nullptr, *delta_ema_master = nullptr, *delta_sums = nullptr;
	bool step_pending = false;  // between a step's backward pass and its optimizer pass
	cudaEvent_t stats_event = nullptr;  // behind the last copy of the step statistics to the host
	uint32_t stats_step = 0;
	bool tuned = false;         // the batch tuner already ran for the step whose optimizer pass is pending
	bool pregenerated = false;  // the next step's samples are already in the ray workspace
	// The next step's samples are drawn on a second stream, next to the optimizer pass: the generator reads the occupancy bits,
	// the cameras and the tuner's ray count, none of which the optimizer touches, and writes the ray workspace, which nothing
	// reads again once the tuner has run.  ev_tuned: behind the tuner on the training stream; ev_generated: behind the
	// generator on the side stream (the training stream waits for it before the next step's network pass).
	cudaStream_t gen_stream = nullptr;
	cudaEvent_t ev_tuned = nullptr, ev_generated = nullptr;
	bool gen_in_flight = false;  // the training stream has not yet waited for ev_generated
	bool cam_on_gen_stream = false;  // the last camera upload went to the side stream
	uint64_t render_samples = 0;  // of the last call
	float render_ms = 0.f;
	cudaEvent_t render_ev[2] = {nullptr, nullptr};
};

template <typename T>
static int dev_alloc(neus2b_testbed* tb, T** p, size_t n) {
	void* q = nullptr;
	cudaError_t e = cudaMalloc(&q, n * sizeof(T));
	if (e != cudaSuccess) return (int)e;
	e = cudaMemsetAsync(q, 0, n * sizeof(T), tb->stream);
	if (e != cudaSuccess) return (int)e;
	tb->allocs.push_back(q);
	*p = (T*)q;
	return NEUS2B_OK;
}
#define TB_ALLOC(ptr, n)                        \
	do {                                        \
		int _rc = dev_alloc(tb, &(ptr), (n));   \
		if (_rc) {                              \
			neus2b_testbed_destroy(tb);         \
			return _rc;                         \
		}                                       \
	} while (0)

extern "C" void neus2b_testbed_default_config(neus2b_testbed_config* c) {
	if (!c) return;
	*c = neus2b_testbed_config{};
	c->grid = neus2b_grid_desc{16, 19, 16, 1.447f, 16};
	c->sdf_bias = -0.1f;
	c->batch_size = 1u << 18;
	c->n_cascades = 1;
	c->seed = 1337;
	c->learning_rate = 1e-2f;
	c->beta1 = 0.9f;
	c->beta2 = 0.99f;
	c->epsilon = 1e-15f;
	c->l2_reg = 1e-6f;
	c->ema_decay = 0.95f;
	c->lr_decay_start = 20000;
	c->lr_decay_interval = 10000;
	c->lr_decay_base = 0.33f;
	c->ek_loss_weight = 0.1f;
	c->mask_loss_weight = 0.f;
	c->anneal_end = 0;
	c->density_grid_decay = 0.95f;
	c->random_bg_color = 1;
	c->snap_to_pixel_centers = 1;  // Nerf::Training::snap_to_pixel_centers (testbed.h:614)
	c->world_size = 1;
	c->rank = 0;
	c->loss_scale = 128.f;
	c->predict_global_movement = 0;
	c->predict_global_movement_training_step = 300;  // src/testbed.cu:2120
	c->finetune_global_movement = 1;
	c->reset_density_grid_after_global_movement = 1;
	c->after_learning_rate = 0.f;
	// "globalmove" optimizer of configs/nerf/base.json:84-110
	c->gm_learning_rate = 5e-3f;
	c->gm_beta1 = 0.9f;
	c->gm_beta2 = 0.99f;
	c->gm_epsilon = 1e-10f;
	c->gm_l2_reg = 1e-10f;
	c->gm_ema_decay = 0.95f;
	c->gm_lr_decay_start = 6000;
	c->gm_lr_decay_interval = 25;
	c->gm_lr_decay_base = 0.99f;
	// samples [0,32), [32,96), then the rest of the rays still transparent.  Multiples of 32 keep the grouping of the fp32 sums
	// along a ray, so the step is bit for bit the full pass's.  Measured on config 1 (steps 520-920): one GPU 0.775 -> 0.777 ms
	// per step (half the evaluations, paid back by four more launches), two GPUs 0.978 -> 0.857 ms (a third of the evaluations).
	c->n_forward_windows = 2;
	c->forward_window_ends[0] = 32;
	c->forward_window_ends[1] = 96;
}

extern "C" void neus2b_testbed_destroy(neus2b_testbed* tb) {
	if (!tb) return;
	if (tb->gen_stream) cudaStreamSynchronize(tb->gen_stream);
	if (tb->stream) cudaStreamSynchronize(tb->stream);
	for (void* p : tb->allocs) cudaFree(p);
	for (void* p : tb->render_allocs) cudaFree(p);
	if (tb->h_state) cudaFreeHost(tb->h_state);
	if (tb->h_cam) cudaFreeHost(tb->h_cam);
	for (cudaEvent_t e : tb->prof_events) cudaEventDestroy(e);
	for (cudaEvent_t e : tb->render_ev)
		if (e) cudaEventDestroy(e);
	if (tb->cam_event) cudaEventDestroy(tb->cam_event);
	if (tb->stats_event) cudaEventDestroy(tb->stats_event);
	if (tb->ev_tuned) cudaEventDestroy(tb->ev_tuned);
	if (tb->ev_generated) cudaEventDestroy(tb->ev_generated);
	if (tb->gen_stream) cudaStreamDestroy(tb->gen_stream);
	if (tb->stream) cudaStreamDestroy(tb->stream);
	delete tb;
}

// DeltaNetwork::initialize_params (transform_network.h:207-246): no translation, the unit 6-D rotation (1 0 0 | 0 1 0), and a
// fresh optimizer for it.
static int write_delta(neus2b_testbed* tb, const float h[12]) {
	float buf[12 * 5] = {};
	uint16_t hb[16] = {};
	for (int k = 0; k < 12; ++k) {
		buf[k] = buf[36 + k] = h[k];
		const __half v = __float2half_rn(h[k]);
		memcpy(&hb[k], &v, 2);
	}
	N2B_CHECK_CUDA(cudaMemcpyAsync(tb->delta_master, buf, sizeof(buf), cudaMemcpyHostToDevice, tb->stream));
	N2B_CHECK_CUDA(cudaMemcpyAsync(tb->delta, hb, sizeof(hb), cudaMemcpyHostToDevice, tb->stream));
	N2B_CHECK_CUDA(cudaMemcpyAsync(tb->delta_ema, hb, sizeof(hb), cudaMemcpyHostToDevice, tb->stream));
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));  // the sources are on this thread's stack
	tb->delta_adam_step = 0;
	return NEUS2B_OK;
}
static int reset_delta(neus2b_testbed* tb) {
	const float ident[12] = {0.f, 0.f, 0.f, 0.f, 1.f, 0.f, 0.f, 0.f, 1.f, 0.f, 0.f, 0.f};
	return write_delta(tb, ident);
}

extern "C" int neus2b_testbed_create(const neus2b_testbed_config* cfg, neus2b_testbed** out) {
	if (!cfg || !out) return NEUS2B_E_INVALID;
	GridLevels lv;
	int rc = make_levels(&cfg->grid, &lv);
	if (rc) return rc;
	if (cfg->batch_size == 0 || cfg->batch_size % 128u || cfg->n_cascades == 0 || cfg->n_cascades > NEUS2B_CASCADES ||
	    cfg->world_size == 0 || cfg->rank >= cfg->world_size || !(cfg->loss_scale > 0.f))
		return NEUS2B_E_INVALID;
	int ndev = 0;
	if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return NEUS2B_E_NO_DEVICE;
	neus2b_testbed* tb = new (std::nothrow) neus2b_testbed();
	if (!tb) return NEUS2B_E_INVALID;
	tb->cfg = *cfg;
	N2B_CHECK_CUDA(cudaGetDevice(&tb->device));
	cudaError_t e = cudaStreamCreateWithFlags(&tb->stream, cudaStreamNonBlocking);
	if (e == cudaSuccess) {  // the generator's small kernels go first where both streams have work ready
		int lo = 0, hi = 0;
		cudaDeviceGetStreamPriorityRange(&lo, &hi);
		e = cudaStreamCreateWithPriority(&tb->gen_stream, cudaStreamNonBlocking, hi);
	}
	if (e == cudaSuccess) e = cudaEventCreateWithFlags(&tb->ev_tuned, cudaEventDisableTiming);
	if (e == cudaSuccess) e = cudaEventCreateWithFlags(&tb->ev_generated, cudaEventDisableTiming);
	if (e != cudaSuccess) {
		neus2b_testbed_destroy(tb);
		return (int)e;
	}
	tb->n_grid = (uint64_t)lv.offset[NEUS2B_MAX_LEVELS] * 2u;
	tb->n_params = NEUS2B_MLP_N + tb->n_grid + 4u;
	tb->target = cfg->batch_size;
	tb->max_samples = cfg->batch_size * 16u;  // "somewhat of a worst case" (src/testbed_nerf.cu:3719)
	// rng streams as in reset_network (src/testbed.cu:2077-2091)
	neus2b_pcg32 r;
	neus2b_pcg32_seed(&r, cfg->seed);
	tb->rng = Pcg32{r.state, r.inc};
	neus2b_pcg32 dr;
	neus2b_pcg32_seed(&dr, tb->rng.next_uint());
	tb->density_rng = Pcg32{dr.state, dr.inc};
	(void)tb->rng.next_uint();  // tv_loss_rng

	TB_ALLOC(tb->params, tb->n_params);
	TB_ALLOC(tb->params_ema, tb->n_params);
	TB_ALLOC(tb->grad_grid, tb->n_grid);
	TB_ALLOC(tb->master, tb->n_params);
	TB_ALLOC(tb->ema_master, tb->n_params);
	TB_ALLOC(tb->adam_m, tb->n_params);
	TB_ALLOC(tb->adam_v, tb->n_params);
	TB_ALLOC(tb->grad_mlp, (size_t)NEUS2B_MLP_N + 4);  // the variance gradient sits right behind: one fp32 exchange for both
	tb->grad_var = tb->grad_mlp + NEUS2B_MLP_N;
	const size_t cells = (size_t)NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE;
	const size_t n_occ = cells * cfg->n_cascades;
	TB_ALLOC(tb->density_grid, n_occ);
	TB_ALLOC(tb->density_tmp, n_occ);
	TB_ALLOC(tb->density_mean, (size_t)1);
	TB_ALLOC(tb->bitfield, cells / 8 * NEUS2B_CASCADES);
	TB_ALLOC(tb->occ_bounds, (size_t)8);
	TB_ALLOC(tb->occ_pos, n_occ * 3);
	TB_ALLOC(tb->occ_idx, n_occ);
	TB_ALLOC(tb->occ_sdf, n_occ);
	TB_ALLOC(tb->occ_partial, (size_t)1024);
	tb->ws.max_rays = tb->max_rays;
	tb->ws.max_samples = tb->max_samples;
	TB_ALLOC(tb->ws.d_ray_indices, (size_t)tb->max_rays);
	TB_ALLOC(tb->ws.d_rays, (size_t)tb->max_rays * 6);
	TB_ALLOC(tb->ws.d_numsteps, (size_t)tb->max_rays * 2);
	TB_ALLOC(tb->ws.d_coords, (size_t)tb->max_samples * 7);
	TB_ALLOC(tb->ws.d_counters, (size_t)8);
	TB_ALLOC(tb->ws.d_scan_tmp, (size_t)tb->max_rays + 1024);
	TB_ALLOC(tb->ws.d_ray_tmp, (size_t)tb->max_rays * 8);
	TB_ALLOC(tb->ws.d_march_masks, (size_t)tb->max_rays * 64);
	TB_ALLOC(tb->ws.d_window_list, (size_t)tb->max_samples);
	TB_ALLOC(tb->ws.d_window_lens, (size_t)8);
	TB_ALLOC(tb->mlp_out, (size_t)tb->max_samples * 16);
	TB_ALLOC(tb->dloss, (size_t)tb->target * 16);
	TB_ALLOC(tb->coords_compacted, (size_t)tb->target * 7);
	TB_ALLOC(tb->loss, (size_t)tb->max_rays);
	TB_ALLOC(tb->ek_loss, (size_t)tb->max_rays);
	TB_ALLOC(tb->state, (size_t)1);
	TB_ALLOC(tb->delta, (size_t)16);
	TB_ALLOC(tb->delta_ema, (size_t)16);
	TB_ALLOC(tb->delta_master, (size_t)12 * 5);  // master, m, v, ema master, sums
	tb->delta_m = tb->delta_master + 12;
	tb->delta_v = tb->delta_master + 24;
	tb->delta_ema_master = tb->delta_master + 36;
	tb->delta_sums = tb->delta_master + 48;
	tb->ws.d_n_rays_total = &tb->state->n_rays_total;
	tb->ws.d_prev_samples = &tb->state->measured_pre;  // max_inference (src/testbed_nerf.cu:3764-3769)
	{
		const int erc = tc_error_device_ptr(&tb->d_device_error);
		if (erc) {
			neus2b_testbed_destroy(tb);
			return erc;
		}
	}
	e = cudaMallocHost((void**)&tb->h_state, sizeof(TrainState));
	if (e != cudaSuccess) {
		neus2b_testbed_destroy(tb);
		return (int)e;
	}
	TrainState init{};
	init.rays_per_batch = 1u << 12;  // Counters::rays_per_batch (testbed.h)
	*tb->h_state = init;
	e = cudaMemcpyAsync(tb->state, tb->h_state, sizeof(TrainState), cudaMemcpyHostToDevice, tb->stream);
	if (e == cudaSuccess) e = cudaStreamSynchronize(tb->stream);
	if (e != cudaSuccess) {
		neus2b_testbed_destroy(tb);
		return (int)e;
	}
	rc = reset_delta(tb);
	if (rc) {
		neus2b_testbed_destroy(tb);
		return rc;
	}
	*out = tb;
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_n_params(const neus2b_testbed* tb, uint64_t* n) {
	if (!tb || !n) return NEUS2B_E_INVALID;
	*n = tb->n_params;
	return NEUS2B_OK;
}

// The training stream waits for samples that are still being drawn on the side stream.
static int join_generation(neus2b_testbed* tb) {
	if (tb->gen_in_flight) {
		N2B_CHECK_CUDA(cudaStreamWaitEvent(tb->stream, tb->ev_generated, 0));
		tb->gen_in_flight = false;
	}
	if (tb->cam_on_gen_stream) {
		N2B_CHECK_CUDA(cudaStreamWaitEvent(tb->stream, tb->cam_event, 0));
		tb->cam_on_gen_stream = false;
	}
	return NEUS2B_OK;
}

static int upload_cameras(neus2b_testbed* tb, const float* h_xforms, const float* h_focal, const float* h_principal, cudaStream_t stream) {
	const uint32_t n = tb->ds.n_images;
	tb->pregenerated = false;  // samples drawn ahead used the previous cameras
	if (!tb->cam_event) N2B_CHECK_CUDA(cudaEventCreateWithFlags(&tb->cam_event, cudaEventDisableTiming));
	else N2B_CHECK_CUDA(cudaEventSynchronize(tb->cam_event));  // the previous upload may still be reading the staging buffer
	memcpy(tb->h_cam, h_xforms, sizeof(float) * 12 * n);
	memcpy(tb->h_cam + 12 * n, h_focal, sizeof(float) * 2 * n);
	memcpy(tb->h_cam + 14 * n, h_principal, sizeof(float) * 2 * n);
	// the three arrays are one allocation, in this order
	N2B_CHECK_CUDA(cudaMemcpyAsync((void*)tb->ds.d_xforms, tb->h_cam, sizeof(float) * 16 * n, cudaMemcpyHostToDevice, stream));
	N2B_CHECK_CUDA(cudaEventRecord(tb->cam_event, stream));
	tb->cam_on_gen_stream = stream == tb->gen_stream;
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_update_cameras(neus2b_testbed* tb, const float* h_xforms, const float* h_focal, const float* h_principal) {
	if (!tb || !tb->ds.n_images || !h_xforms || !h_focal || !h_principal) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	int rc = join_generation(tb);  // samples being drawn ahead still read the old cameras
	if (rc) return rc;
	return upload_cameras(tb, h_xforms, h_focal, h_principal, tb->stream);
}

extern "C" int neus2b_testbed_load_training_data(neus2b_testbed* tb, uint32_t n_images, uint32_t width, uint32_t height,
                                                 const uint32_t* h_pixels, const float* h_xforms, const float* h_focal,
                                                 const float* h_principal) {
	if (!tb || !n_images || !width || !height || !h_pixels || !h_xforms || !h_focal || !h_principal) return NEUS2B_E_INVALID;
	if (tb->ds.n_images) return NEUS2B_E_UNSUPPORTED;  // one dataset per testbed
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	uint32_t* px = nullptr;
	float* cam = nullptr;
	const size_t npx = (size_t)n_images * width * height;
	int rc = dev_alloc(tb, &px, npx);
	if (rc) return rc;
	rc = dev_alloc(tb, &cam, (size_t)16 * n_images);
	if (rc) return rc;
	N2B_CHECK_CUDA(cudaMallocHost((void**)&tb->h_cam, sizeof(float) * 16 * n_images));
	N2B_CHECK_CUDA(cudaMemcpyAsync(px, h_pixels, npx * 4, cudaMemcpyHostToDevice, tb->stream));
	tb->ds.n_images = n_images;
	tb->ds.width = width;
	tb->ds.height = height;
	tb->ds.d_pixels = px;
	tb->ds.d_xforms = cam;
	tb->ds.d_focal = cam + (size_t)12 * n_images;
	tb->ds.d_principal = cam + (size_t)14 * n_images;
	rc = neus2b_testbed_update_cameras(tb, h_xforms, h_focal, h_principal);
	if (rc) return rc;
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_set_params(neus2b_testbed* tb, const float* h_params, uint64_t n) {
	if (!tb || !h_params || n != tb->n_params) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	N2B_CHECK_CUDA(cudaMemcpyAsync(tb->master, h_params, n * sizeof(float), cudaMemcpyHostToDevice, tb->stream));
	master_to_half_kernel<<<kSMs * 4, 256, 0, tb->stream>>>(n, tb->master, tb->params, tb->params_ema, tb->ema_master);
	N2B_CHECK_LAUNCH();
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_get_params(neus2b_testbed* tb, float* h_params, uint64_t n, int ema) {
	if (!tb || !h_params || n != tb->n_params) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaMemcpyAsync(h_params, ema ? tb->ema_master : tb->master, n * sizeof(float), cudaMemcpyDeviceToHost, tb->stream));
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_device_ptrs(neus2b_testbed* tb, uint16_t** d_params, uint16_t** d_params_ema, float** d_master,
                                          float** d_grad_mlp, uint16_t** d_grad_grid, float** d_grad_variance, uint8_t** d_bitfield,
                                          float** d_density_grid, neus2b_stream_t* stream) {
	if (!tb) return NEUS2B_E_INVALID;
	if (int jr = join_generation(tb)) return jr;  // samples may still be drawn on the side stream
	if (d_params) *d_params = (uint16_t*)tb->params;
	if (d_params_ema) *d_params_ema = (uint16_t*)tb->params_ema;
	if (d_master) *d_master = tb->master;
	if (d_grad_mlp) *d_grad_mlp = tb->grad_mlp;
	if (d_grad_grid) *d_grad_grid = (uint16_t*)tb->grad_grid;
	if (d_grad_variance) *d_grad_variance = tb->grad_var;
	if (d_bitfield) {
		*d_bitfield = tb->bitfield;
		tb->occ_bounds_stale = true;  // the caller may write it
		tb->pregenerated = false;
	}
	if (d_density_grid) *d_density_grid = tb->density_grid;
	if (stream) *stream = tb->stream;
	return NEUS2B_OK;
}

extern "C" float neus2b_per_level_scale_from_top_resolution(uint32_t n_levels, uint32_t base_resolution, float top_resolution,
                                                           uint32_t aabb_scale) {
	if (n_levels < 2 || base_resolution == 0 || !(top_resolution > 0.f) || aabb_scale == 0) return 0.f;
	return expf(logf(top_resolution * (float)aabb_scale / (float)base_resolution) / (float)(n_levels - 1));
}

extern "C" uint32_t neus2b_testbed_config_active_levels(const neus2b_testbed_config* c, uint32_t training_step) {
	if (!c) return 0;
	const uint32_t L = c->grid.n_levels;
	uint32_t n = c->grid.n_active_levels < L ? c->grid.n_active_levels : L;
	if (c->base_training_step) {  // the reference's keys (configs/nerf/dtu.json:35-37)
		float frac = c->base_valid_level_scale + c->valid_level_scale * (float)(training_step / c->base_training_step);
		if (!(frac < 1.0f)) frac = 1.0f;
		if (!(frac > 0.f)) frac = 0.f;
		n = (uint32_t)((float)L * frac + 0.5f);  // to the nearest level: 0.2 * 14 = 2.8 -> 3
		n = n < 1u ? 1u : (n > L ? L : n);
	} else if (c->progressive_steps_per_increment) {
		n = c->progressive_start_levels + c->progressive_levels_per_increment * (training_step / c->progressive_steps_per_increment);
		n = n < L ? n : L;
	}
	return n;
}

// After a synchronisation: has any kernel raised the sticky error word (a bounded wait that ran out)?
static int device_error_status() {
	uint32_t flags = 0;
	const int rc = neus2b_device_error_flags(&flags);
	if (rc) return rc;
	return flags ? NEUS2B_E_DEVICE : NEUS2B_OK;
}

// The mask's clock: the training step, and on later frames of a dynamic sequence the steps behind the phase that trains the
// motion alone (set_training_step(m_training_step - m_predict_global_movement_training_step), src/testbed.cu:2642-2647).
static uint32_t predict_steps(const neus2b_testbed* tb) {
	return tb->cfg.predict_global_movement ? tb->cfg.predict_global_movement_training_step : 0u;
}
static neus2b_grid_desc active_desc(const neus2b_testbed* tb) {
	neus2b_grid_desc d = tb->cfg.grid;
	uint32_t step = tb->training_step;
	if (tb->frame >= 1) step = step > predict_steps(tb) ? step - predict_steps(tb) : 0u;
	d.n_active_levels = neus2b_testbed_config_active_levels(&tb->cfg, step);
	return d;
}
// The motion the networks apply to the samples (m_use_delta: a later frame whose motion is being trained, src/testbed.cu:2694-2700).
static const neus2b_motion* step_motion(const neus2b_testbed* tb, neus2b_motion* m, bool with_sums) {
	if (tb->frame == 0 || !tb->train_delta) return nullptr;
	m->d_delta = (const uint16_t*)tb->delta;
	for (int e = 0; e < 3; ++e) m->first_frame_offset[e] = tb->cfg.first_frame_offset[e];
	m->d_sums = with_sums ? tb->delta_sums : nullptr;
	return m;
}

// training_prep_nerf (src/testbed_nerf.cu:3989-4003), called every clamp(step/16, 1, 16) steps (src/testbed.cu:2659)
static int training_prep(neus2b_testbed* tb) {
	const uint32_t cells = NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE, nc = tb->cfg.n_cascades;
	uint32_t n_uniform, n_nonuniform;
	if (tb->training_step < 256) {
		n_uniform = cells * nc;
		n_nonuniform = 0;
	} else {
		n_uniform = cells / 4 * nc;
		n_nonuniform = cells / 4 * nc;
	}
	const neus2b_pcg32 ru{tb->density_rng.state, tb->density_rng.inc};
	tb->density_rng.advance(1ull << 32);
	const neus2b_pcg32 rn{tb->density_rng.state, tb->density_rng.inc};
	tb->density_rng.advance(1ull << 32);
	const neus2b_grid_desc d = active_desc(tb);
	if (tb->training_step == 0) {  // a frame's first update starts from an empty grid (src/testbed_nerf.cu:3308-3325)
		tb->ema_step = 0;
		N2B_CHECK_CUDA(cudaMemsetAsync(tb->density_grid, 0, sizeof(float) * (size_t)cells * nc, tb->stream));
	}
	neus2b_motion mo{};
	int rc = neus2b_occupancy_update_moved(&d, (const uint16_t*)tb->params, tb->cfg.sdf_bias, nc, n_uniform, n_nonuniform, ru, rn, tb->ema_step,
	                                       tb->cfg.density_grid_decay, tb->density_grid, tb->density_tmp, tb->bitfield, tb->density_mean,
	                                       tb->occ_pos, tb->occ_idx, (uint16_t*)tb->occ_sdf, tb->occ_partial, step_motion(tb, &mo, false),
	                                       tb->stream);
	++tb->ema_step;
	tb->occ_bounds_stale = true;
	return rc;
}

static neus2b_train_cfg make_train_cfg(const neus2b_testbed* tb) {
	neus2b_train_cfg c{};
	for (int e = 0; e < 3; ++e) {
		c.aabb_min[e] = 0.f;
		c.aabb_max[e] = 1.f;
	}
	c.cone_angle_constant = 0.f;  // aabb_scale <= 1 (src/testbed_nerf.cu:3084)
	c.snap_to_pixel_centers = tb->cfg.snap_to_pixel_centers;
	c.random_bg_color = tb->cfg.random_bg_color;
	c.loss_scale = tb->cfg.loss_scale;  // LOSS_SCALE (testbed.h:237) = 128 by default
	c.mask_loss_weight = tb->cfg.mask_loss_weight;
	c.ek_loss_weight = tb->cfg.ek_loss_weight;
	// NerfNetwork::cos_anneal_ratio (nerf_network.h:1109-1118)
	c.ray_index_offset = tb->cfg.rank * tb->max_rays;
	c.ray_count_scale = tb->cfg.world_size;
	c.cos_anneal_ratio = tb->cfg.anneal_end == 0 ? 1.0f : fminf(1.0f, (float)tb->training_step / (float)tb->cfg.anneal_end);
	// rays go through the accumulated movement of the earlier frames (m_predict_global_movement, src/testbed_nerf.cu:3830-3832)
	if (tb->cfg.predict_global_movement) {
		c.use_global_movement = 1;
		memcpy(c.rotation, tb->acc_rotation, sizeof(c.rotation));
		memcpy(c.transition, tb->acc_transition, sizeof(c.transition));
		memcpy(c.first_frame_offset, tb->cfg.first_frame_offset, sizeof(c.first_frame_offset));
	}
	return c;
}

// m_canonical_training_step after a step (src/testbed_nerf.cu:3506-3522): the step count, or on later frames the steps behind
// the motion-only phase, during which it stays where the frame switch put it (0: the occupancy grid is updated every step).
static uint32_t next_canonical_step(const neus2b_testbed* tb, uint32_t training_step) {
	if (!tb->cfg.predict_global_movement || tb->frame == 0) return training_step;
	return training_step < predict_steps(tb) ? 0u : training_step - predict_steps(tb);
}

static uint32_t occupancy_skip(uint32_t step) { return step / 16u < 1u ? 1u : (step / 16u > 16u ? 16u : step / 16u); }

// The step's rays and samples (first half of train_nerf_step, src/testbed_nerf.cu:3782-3830).  Depends on the occupancy
// bits, the batch tuner's ray count and the step's random stream, not on the parameters.
static int generate_step_samples(neus2b_testbed* tb, const neus2b_train_cfg& tc, const neus2b_pcg32& rng, cudaStream_t stream) {
	// one cascade: positions map straight to the finest level's cells, so rays that miss the box of occupied cells are
	// not marched; the box is recomputed after every occupancy update (and after the bitfield's pointer was handed out)
	tb->ws.d_occupied_bounds = nullptr;
	if (tb->cfg.n_cascades == 1) {
		if (tb->occ_bounds_stale) {
			int rc = neus2b_occupancy_bounds(tb->bitfield, tb->occ_bounds, stream);
			if (rc) return rc;
			tb->occ_bounds_stale = false;
		}
		tb->ws.d_occupied_bounds = tb->occ_bounds;
	}
	return neus2b_generate_samples(&tb->ds, &tc, tb->max_rays, &tb->state->rays_per_batch, 0, rng, tb->bitfield, &tb->ws, stream);
}

extern "C" int neus2b_testbed_train_backward(neus2b_testbed* tb) {
	if (!tb || !tb->ds.n_images) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	int rc = join_generation(tb);
	if (rc) return rc;
	// a later frame of a dynamic sequence: the canonical model joins once the motion-only phase is over (src/testbed.cu:2649-2657)
	if (tb->frame >= 1 && tb->training_step == predict_steps(tb)) {
		tb->train_canonical = true;
		if (!tb->cfg.finetune_global_movement) tb->train_delta = false;
		if (tb->cfg.reset_density_grid_after_global_movement && predict_steps(tb) > 0) {
			N2B_CHECK_CUDA(cudaMemsetAsync(tb->density_grid, 0,
			                               sizeof(float) * (size_t)NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * tb->cfg.n_cascades, tb->stream));
			tb->ema_step = 0;
		}
	}
	if (tb->canonical_step % occupancy_skip(tb->canonical_step) == 0) {
		if (tb->pregenerated) return NEUS2B_E_INVALID;  // (pregenerate refuses steps that start with an occupancy update)
		rc = training_prep(tb);
		if (rc) return rc;
	}
	const neus2b_grid_desc d = active_desc(tb);
	const neus2b_train_cfg tc = make_train_cfg(tb);
	const neus2b_pcg32 rng{tb->rng.state, tb->rng.inc};
	const uint32_t* d_n_rays = &tb->state->rays_per_batch;
	if (tb->pregenerated) {
		tb->pregenerated = false;  // neus2b_testbed_train_pregenerate already drew this step's samples
	} else {
		// the running ray count that spreads the rays over the images restarts with every frame, and with every step while
		// the canonical step stands at zero (the motion-only phase of a later frame) (src/testbed_nerf.cu:3779-3781);
		// samples are never drawn ahead for such a step (it begins with an occupancy update)
		if (tb->training_step == 0 || tb->canonical_step == 0)
			N2B_CHECK_CUDA(cudaMemsetAsync(&tb->state->n_rays_total, 0, sizeof(uint32_t), tb->stream));
		rc = generate_step_samples(tb, tc, rng, tb->stream);
		if (rc) return rc;
	}
	neus2b_motion mo{};
	const neus2b_motion* motion = step_motion(tb, &mo, true);
	// the network pass over the step's samples and the loss pass; with windows, only the samples in front of the point where
	// a ray turns opaque are evaluated (the mma.sync path has no list form: it evaluates everything)
	const uint32_t n_windows = neus2b_get_mma_path() == NEUS2B_MMA_TCGEN05 ? tb->cfg.n_forward_windows : 0u;
	rc = neus2b_forward_compute_loss(&d, (const uint16_t*)tb->params, tb->cfg.sdf_bias, motion, &tb->ds, &tc, tb->max_rays, d_n_rays, 0, rng, tb->target,
	                                 &tb->ws, tb->cfg.forward_window_ends, n_windows, (uint16_t*)tb->mlp_out, tb->coords_compacted, (uint16_t*)tb->dloss,
	                                 tb->loss, tb->ek_loss, 1, tb->stream);
	if (rc) return rc;
	const bool timed = tb->prof_on && tb->prof_used + 2 <= tb->prof_events.size();
	if (timed) cudaEventRecord(tb->prof_events[tb->prof_used], tb->stream);
	// (the canonical gradients are not formed while the canonical model is frozen: m_train_canonical, nerf_network.h:446)
	const bool canon = tb->train_canonical;
	if (canon || motion)
		rc = neus2b_neus_train_moved(&d, (const uint16_t*)tb->params, tb->target, tb->coords_compacted, motion, (const uint16_t*)tb->dloss,
		                             tb->target * tb->cfg.world_size, canon ? tb->grad_mlp : nullptr, canon ? (uint16_t*)tb->grad_grid : nullptr,
		                             canon ? tb->grad_var : nullptr, tb->stream);
	if (rc) return rc;
	if (timed) {
		cudaEventRecord(tb->prof_events[tb->prof_used + 1], tb->stream);
		tb->prof_used += 2;
	}
	tb->rng.advance(1ull << 32);  // m_rng.advance() (src/testbed_nerf.cu:3981)
	tb->step_pending = true;
	return NEUS2B_OK;
}

// Counters::update_after_training for the step whose optimizer pass is pending, once; the event behind it is what the side
// stream waits for before it touches the ray workspace or the cameras.
static int run_tuner(neus2b_testbed* tb) {
	if (tb->tuned) return NEUS2B_OK;
	tune_kernel<<<1, 32, 0, tb->stream>>>(tb->state, tb->ws.d_counters, tb->target, tb->max_rays, tb->d_device_error);
	N2B_CHECK_LAUNCH();
	N2B_CHECK_CUDA(cudaEventRecord(tb->ev_tuned, tb->stream));
	tb->tuned = true;
	return NEUS2B_OK;
}

// Between neus2b_testbed_train_backward and neus2b_testbed_train_optimizer_step: draws the NEXT step's rays and samples
// now, so that this work overlaps a gradient exchange running on another stream (data-parallel training).  The batch
// tuner of the pending step runs first (it reads the counters the generator is about to reuse).  Returns 1 and does
// nothing when the next step starts with an occupancy-grid update, which needs the updated parameters first.
extern "C" int neus2b_testbed_train_pregenerate(neus2b_testbed* tb) {
	if (!tb || !tb->ds.n_images) return NEUS2B_E_INVALID;
	if (tb->pregenerated) return NEUS2B_OK;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	const uint32_t next = next_canonical_step(tb, tb->training_step + (tb->step_pending ? 1u : 0u));
	if (next % occupancy_skip(next) == 0) return 1;
	if (tb->frame >= 1 && tb->training_step + (tb->step_pending ? 1u : 0u) == predict_steps(tb)) return 1;  // the phase change may clear the grid
	if (tb->step_pending) {
		if (int rc = run_tuner(tb)) return rc;
	} else {  // no optimizer pass to run next to: behind everything the training stream holds
		N2B_CHECK_CUDA(cudaEventRecord(tb->ev_tuned, tb->stream));
	}
	// on the side stream, behind the tuner (and behind a camera upload that went to the training stream)
	N2B_CHECK_CUDA(cudaStreamWaitEvent(tb->gen_stream, tb->ev_tuned, 0));
	if (tb->cam_event && !tb->cam_on_gen_stream) N2B_CHECK_CUDA(cudaStreamWaitEvent(tb->gen_stream, tb->cam_event, 0));
	const neus2b_train_cfg tc = make_train_cfg(tb);  // (nothing the generator reads depends on the step number)
	const neus2b_pcg32 rng{tb->rng.state, tb->rng.inc};  // already advanced to the next step's stream
	int rc = generate_step_samples(tb, tc, rng, tb->gen_stream);
	if (rc) return rc;
	N2B_CHECK_CUDA(cudaEventRecord(tb->ev_generated, tb->gen_stream));
	tb->gen_in_flight = true;
	tb->pregenerated = true;
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_profile(neus2b_testbed* tb, uint32_t max_steps, float* h_ms_sum, uint32_t* h_n) {
	if (!tb) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	if (h_ms_sum && h_n) {  // read back what has been recorded so far
		N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
		float sum = 0.f;
		for (uint32_t i = 0; i + 1 < tb->prof_used; i += 2) {
			float ms = 0.f;
			N2B_CHECK_CUDA(cudaEventElapsedTime(&ms, tb->prof_events[i], tb->prof_events[i + 1]));
			sum += ms;
		}
		*h_ms_sum = sum;
		*h_n = tb->prof_used / 2;
	}
	while (tb->prof_events.size() < 2u * (size_t)max_steps) {
		cudaEvent_t e;
		N2B_CHECK_CUDA(cudaEventCreate(&e));
		tb->prof_events.push_back(e);
	}
	tb->prof_used = 0;
	tb->prof_on = max_steps > 0;
	return NEUS2B_OK;
}

static int optimizer_enqueue(neus2b_testbed* tb, bool want_stats) {
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	const neus2b_testbed_config& c = tb->cfg;
	neus2b_adam_cfg ac{};
	// from the second frame on the canonical model trains at "after_learning_rate" (src/testbed.cu:2684-2692)
	ac.learning_rate = (tb->frame >= 1 && c.after_learning_rate > 0.f) ? c.after_learning_rate : c.learning_rate;
	const uint32_t step = tb->adam_step + 1;  // steps of this frame's optimizer (a new one per frame, src/testbed.cu:2031-2033)
	if (c.lr_decay_interval && step >= c.lr_decay_start)  // ExponentialDecay (configs/nerf/dtu.json:8-12)
		ac.learning_rate *= powf(c.lr_decay_base, (float)((step - c.lr_decay_start) / c.lr_decay_interval + 1));
	ac.beta1 = c.beta1;
	ac.beta2 = c.beta2;
	ac.epsilon = c.epsilon;
	ac.l2_reg = c.l2_reg;
	ac.ema_decay = c.ema_decay;
	ac.loss_scale = c.loss_scale;
	ac.step = step;
	ac.n_matrix = NEUS2B_MLP_N;
	ac.flags = c.adam_flags;
	ac.d_nonfinite = &tb->state->nonfinite;
	int rc = NEUS2B_OK;
	if (tb->train_canonical) {  // src/testbed_nerf.cu:3497-3499
		rc = neus2b_adam_step(&ac, tb->n_params, tb->grad_mlp, (uint16_t*)tb->grad_grid, tb->grad_var, tb->master, tb->adam_m, tb->adam_v,
		                      (uint16_t*)tb->params, (uint16_t*)tb->params_ema, tb->ema_master, tb->stream);
		if (rc) return rc;
		++tb->adam_step;
	}
	if (tb->frame >= 1 && tb->train_delta) {  // m_global_move.trainer->optimizer_step (:3500-3502)
		neus2b_adam_cfg dc{};
		const uint32_t dstep = tb->delta_adam_step + 1;
		dc.learning_rate = c.gm_learning_rate;
		if (c.gm_lr_decay_interval && dstep >= c.gm_lr_decay_start)
			dc.learning_rate *= powf(c.gm_lr_decay_base, (float)((dstep - c.gm_lr_decay_start) / c.gm_lr_decay_interval + 1));
		dc.beta1 = c.gm_beta1;
		dc.beta2 = c.gm_beta2;
		dc.epsilon = c.gm_epsilon;
		dc.l2_reg = c.gm_l2_reg;
		dc.ema_decay = c.gm_ema_decay;
		dc.loss_scale = c.loss_scale;
		dc.step = dstep;
		dc.flags = c.adam_flags;
		dc.d_nonfinite = &tb->state->nonfinite;
		rc = neus2b_delta_optimizer_step(&dc, tb->delta_sums, tb->delta_master, tb->delta_m, tb->delta_v, (uint16_t*)tb->delta,
		                                 (uint16_t*)tb->delta_ema, tb->delta_ema_master, nullptr, tb->stream);
		if (rc) return rc;
		++tb->delta_adam_step;
	}
	if (int rc2 = run_tuner(tb)) return rc2;
	tb->tuned = false;
	tb->step_pending = false;
	++tb->training_step;
	tb->canonical_step = next_canonical_step(tb, tb->training_step);
	if (want_stats) {
		loss_reduce_kernel<<<1, 1024, 0, tb->stream>>>(tb->state, tb->loss, tb->ek_loss, tb->target);
		N2B_CHECK_LAUNCH();
		N2B_CHECK_CUDA(cudaMemcpyAsync(tb->h_state, tb->state, sizeof(TrainState), cudaMemcpyDeviceToHost, tb->stream));
		if (!tb->stats_event) N2B_CHECK_CUDA(cudaEventCreateWithFlags(&tb->stats_event, cudaEventDisableTiming));
		N2B_CHECK_CUDA(cudaEventRecord(tb->stats_event, tb->stream));
		tb->stats_step = tb->training_step;
	}
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_train_wait_stats(neus2b_testbed* tb, neus2b_train_stats* h_stats) {
	if (!tb || !h_stats || !tb->stats_event) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	N2B_CHECK_CUDA(cudaEventSynchronize(tb->stats_event));
	h_stats->training_step = tb->stats_step;
	h_stats->rays_per_batch = tb->h_state->rays_per_batch;
	h_stats->n_rays_kept = tb->h_state->n_kept;
	h_stats->measured_batch_size_before_compaction = tb->h_state->measured_pre;
	h_stats->n_samples_evaluated = tb->h_state->evaluated;
	h_stats->measured_batch_size = tb->h_state->measured;
	h_stats->overflow = tb->h_state->overflow;
	h_stats->loss = tb->h_state->loss;
	h_stats->ek_loss = tb->h_state->ek_loss;
	h_stats->nonfinite_gradients = tb->h_state->nonfinite;
	h_stats->device_error = tb->h_state->device_error;
	// a bounded wait inside a kernel ran out: that step's gradients are not to be trusted
	return tb->h_state->device_error ? NEUS2B_E_DEVICE : NEUS2B_OK;
}

extern "C" int neus2b_testbed_train_optimizer_step(neus2b_testbed* tb, neus2b_train_stats* h_stats) {
	if (!tb) return NEUS2B_E_INVALID;
	const int rc = optimizer_enqueue(tb, h_stats != nullptr);
	if (rc || !h_stats) return rc;
	return neus2b_testbed_train_wait_stats(tb, h_stats);
}

extern "C" int neus2b_testbed_train_optimizer_step_async(neus2b_testbed* tb) {
	if (!tb) return NEUS2B_E_INVALID;
	return optimizer_enqueue(tb, true);
}

extern "C" int neus2b_testbed_train_step(neus2b_testbed* tb, const float* h_next_xforms, const float* h_next_focal,
                                         const float* h_next_principal, neus2b_train_stats* h_stats) {
	if (!tb) return NEUS2B_E_INVALID;
	int rc = neus2b_testbed_train_backward(tb);
	if (rc) return rc;
	// the next step's cameras and samples go to the side stream, behind this step's tuner and next to its optimizer pass
	if (h_next_xforms && h_next_focal && h_next_principal) {
		if (!tb->ds.n_images) return NEUS2B_E_INVALID;
		rc = run_tuner(tb);
		if (rc) return rc;
		N2B_CHECK_CUDA(cudaStreamWaitEvent(tb->gen_stream, tb->ev_tuned, 0));  // this step's loss pass has read the old cameras
		rc = upload_cameras(tb, h_next_xforms, h_next_focal, h_next_principal, tb->gen_stream);
		if (rc) return rc;
	}
	rc = neus2b_testbed_train_pregenerate(tb);
	if (rc != NEUS2B_OK && rc != 1) return rc;
	rc = optimizer_enqueue(tb, h_stats != nullptr);
	if (rc) return rc;
	return h_stats ? neus2b_testbed_train_wait_stats(tb, h_stats) : NEUS2B_OK;
}

extern "C" int neus2b_testbed_train(neus2b_testbed* tb, uint32_t n_steps, neus2b_train_stats* h_stats) {
	if (!tb || n_steps == 0) return NEUS2B_E_INVALID;
	for (uint32_t s = 0; s < n_steps; ++s) {
		int rc = neus2b_testbed_train_backward(tb);
		if (rc) return rc;
		rc = neus2b_testbed_train_pregenerate(tb);  // (1: the next step starts with an occupancy update and draws its samples itself)
		if (rc != NEUS2B_OK && rc != 1) return rc;
		rc = neus2b_testbed_train_optimizer_step(tb, s + 1 == n_steps ? h_stats : nullptr);
		if (rc) return rc;
	}
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_sdf_grid(neus2b_testbed* tb, const uint32_t res[3], uint32_t z0, uint32_t z1, int use_ema, float* d_out) {
	if (!tb || !res || !d_out || z1 <= z0 || z1 > res[2] || !res[0] || !res[1]) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	const uint64_t first = (uint64_t)z0 * res[0] * res[1], total = (uint64_t)(z1 - z0) * res[0] * res[1];
	const uint32_t chunk = NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * tb->cfg.n_cascades;  // reuse the occupancy scratch (>= 2^21)
	neus2b_grid_desc d = tb->cfg.grid;  // every level: inference does not mask
	const float ix = 1.f / (float)res[0], iy = 1.f / (float)res[1], iz = 1.f / (float)res[2];
	for (uint64_t off = 0; off < total; off += chunk) {
		const uint32_t n = (uint32_t)((total - off) < chunk ? (total - off) : chunk);
		sdf_grid_positions_kernel<<<div_up(n, 256), 256, 0, tb->stream>>>(res[0], res[1], first + off, n, ix, iy, iz, tb->occ_pos);
		N2B_CHECK_LAUNCH();
		neus2b_motion mo{};
		const neus2b_motion* motion = step_motion(tb, &mo, false);
		if (motion && use_ema) mo.d_delta = (const uint16_t*)tb->delta_ema;
		int rc = neus2b_neus_sdf_moved(&d, (const uint16_t*)(use_ema ? tb->params_ema : tb->params), tb->cfg.sdf_bias, n, tb->occ_pos, 3,
		                               motion, (uint16_t*)tb->occ_sdf, tb->stream);
		if (rc) return rc;
		half_to_float_kernel<<<div_up(n, 256), 256, 0, tb->stream>>>(n, tb->occ_sdf, d_out + off);
		N2B_CHECK_LAUNCH();
	}
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	return device_error_status();
}

// ------------------------------------------------------------------------------------------------ rendering

template <typename T>
static int render_alloc(neus2b_testbed* tb, T** p, size_t n) {
	void* q = nullptr;
	cudaError_t e = cudaMalloc(&q, n * sizeof(T));
	if (e != cudaSuccess) return (int)e;
	e = cudaMemsetAsync(q, 0, n * sizeof(T), tb->stream);
	if (e != cudaSuccess) {
		cudaFree(q);
		return (int)e;
	}
	tb->render_allocs.push_back(q);
	*p = (T*)q;
	return NEUS2B_OK;
}

static int render_reserve(neus2b_testbed* tb, uint32_t width, uint32_t height) {
	const uint32_t n_pix = width * height;
	if (tb->render_pixels == n_pix && tb->render_ws.max_rays >= width) return NEUS2B_OK;
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	for (void* p : tb->render_allocs) cudaFree(p);
	tb->render_allocs.clear();
	tb->render_pixels = 0;
	neus2b_render_workspace& ws = tb->render_ws;
	ws = neus2b_render_workspace{};
	const uint32_t band = (1u << 20) / width * width;  // whole rows
	ws.max_rays = n_pix < band ? n_pix : band;
	ws.max_samples = 1u << 22;
	int rc = NEUS2B_OK;
	if (!rc) rc = render_alloc(tb, &ws.d_ray_tmp, (size_t)ws.max_rays * 8);
	if (!rc) rc = render_alloc(tb, &ws.d_scan_tmp, (size_t)ws.max_rays + 1024);
	if (!rc) rc = render_alloc(tb, &ws.d_state, (size_t)ws.max_rays * 8);
	if (!rc) rc = render_alloc(tb, &ws.d_hit_list, (size_t)ws.max_rays);
	if (!rc) rc = render_alloc(tb, &ws.d_coords, (size_t)ws.max_samples * 7);
	if (!rc) rc = render_alloc(tb, &ws.d_out, (size_t)ws.max_samples * 16);
	if (!rc) rc = render_alloc(tb, &ws.d_counters, (size_t)8);
	if (!rc) rc = render_alloc(tb, &ws.d_march_masks, (size_t)ws.max_rays * 64);
	if (!rc) rc = render_alloc(tb, &tb->render_frame, (size_t)n_pix * 4);
	if (!rc) rc = render_alloc(tb, &tb->render_depth, (size_t)n_pix);
	if (!rc) rc = render_alloc(tb, &tb->render_acc, (size_t)n_pix * 4);
	if (!rc) rc = render_alloc(tb, &tb->render_out, (size_t)n_pix * 4);
	if (rc) {
		for (void* p : tb->render_allocs) cudaFree(p);
		tb->render_allocs.clear();
		return rc;
	}
	tb->render_pixels = n_pix;
	return NEUS2B_OK;
}

// Testbed::render_to_cpu (src/python_api.cu:123-169) for a fixed camera: spp frames of render_frame
// (src/testbed.cu:2810-2826: clear, render_nerf, accumulate, tonemap), then the surface goes to the host.
extern "C" int neus2b_testbed_render(neus2b_testbed* tb, const neus2b_render_request* req, float* h_rgba, float* h_depth) {
	if (!tb || !req || !h_rgba || req->width == 0 || req->height == 0 || req->spp == 0 || req->fov_axis > 1) return NEUS2B_E_INVALID;
	if ((uint64_t)req->width * req->height > (1ull << 28) || req->width > (1u << 20)) return NEUS2B_E_TOO_LARGE;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	int rc = render_reserve(tb, req->width, req->height);
	if (rc) return rc;
	const uint32_t n_pix = req->width * req->height;
	if (tb->cfg.n_cascades == 1 && tb->occ_bounds_stale) {
		rc = neus2b_occupancy_bounds(tb->bitfield, tb->occ_bounds, tb->stream);
		if (rc) return rc;
		tb->occ_bounds_stale = false;
	}
	tb->render_ws.d_occupied_bounds = tb->cfg.n_cascades == 1 ? tb->occ_bounds : nullptr;
	neus2b_render_cfg c{};
	c.width = req->width;
	c.height = req->height;
	const uint32_t res[2] = {req->width, req->height};
	for (int e = 0; e < 2; ++e) {
		c.focal_length[e] = req->relative_focal_length[e] * (float)res[req->fov_axis] * req->zoom;  // calc_focal_length
		c.screen_center[e] = (0.5f - req->screen_center[e]) * req->zoom + 0.5f;                    // render_screen_center
	}
	memcpy(c.camera, req->camera, sizeof(c.camera));
	const neus2b_train_cfg t = make_train_cfg(tb);
	for (int e = 0; e < 3; ++e) {
		c.aabb_min[e] = t.aabb_min[e];
		c.aabb_max[e] = t.aabb_max[e];
	}
	c.cone_angle_constant = t.cone_angle_constant;
	c.cos_anneal_ratio = t.cos_anneal_ratio;
	c.min_transmittance = req->min_transmittance;
	c.linear_colors = 0;
	c.max_steps = 0;
	if (tb->cfg.predict_global_movement) {  // src/testbed_nerf.cu:2719-2721
		c.use_global_movement = 1;
		memcpy(c.rotation, tb->acc_rotation, sizeof(c.rotation));
		memcpy(c.transition, tb->acc_transition, sizeof(c.transition));
		memcpy(c.first_frame_offset, tb->cfg.first_frame_offset, sizeof(c.first_frame_offset));
	}
	if (tb->frame >= 1 && tb->train_delta) c.d_delta = (const uint16_t*)(req->use_ema ? tb->delta_ema : tb->delta);
	neus2b_grid_desc d = tb->cfg.grid;  // every level, like the SDF lattice
	const uint16_t* params = (const uint16_t*)(req->use_ema ? tb->params_ema : tb->params);
	for (cudaEvent_t& e : tb->render_ev)
		if (!e) N2B_CHECK_CUDA(cudaEventCreate(&e));
	tb->render_samples = 0;
	N2B_CHECK_CUDA(cudaEventRecord(tb->render_ev[0], tb->stream));
	for (uint32_t s = 0; s < req->spp; ++s) {
		c.sample_index = s;
		neus2b_ld_random_pixel_offset(req->snap_to_pixel_centers ? 0u : s, c.pixel_offset);
		N2B_CHECK_CUDA(cudaMemsetAsync(tb->render_frame, 0, (size_t)n_pix * 16, tb->stream));
		uint64_t n_samples = 0;
		rc = neus2b_render_frame(&d, params, tb->cfg.sdf_bias, &c, tb->bitfield, &tb->render_ws, tb->render_frame, tb->render_depth, &n_samples,
		                         tb->stream);
		if (rc) return rc;
		tb->render_samples += n_samples;
		rc = neus2b_render_accumulate(n_pix, tb->render_frame, tb->render_acc, s, tb->stream);
		if (rc) return rc;
	}
	rc = neus2b_render_tonemap(n_pix, tb->render_acc, req->exposure, req->background_color, req->linear ? 0 : 1, tb->render_out, tb->stream);
	if (rc) return rc;
	N2B_CHECK_CUDA(cudaEventRecord(tb->render_ev[1], tb->stream));
	N2B_CHECK_CUDA(cudaMemcpyAsync(h_rgba, tb->render_out, (size_t)n_pix * 16, cudaMemcpyDeviceToHost, tb->stream));
	if (h_depth) N2B_CHECK_CUDA(cudaMemcpyAsync(h_depth, tb->render_depth, (size_t)n_pix * 4, cudaMemcpyDeviceToHost, tb->stream));
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	N2B_CHECK_CUDA(cudaEventElapsedTime(&tb->render_ms, tb->render_ev[0], tb->render_ev[1]));
	return device_error_status();
}

extern "C" int neus2b_testbed_render_stats(const neus2b_testbed* tb, uint64_t* n_samples, float* device_ms) {
	if (!tb) return NEUS2B_E_INVALID;
	if (n_samples) *n_samples = tb->render_samples;
	if (device_ms) *device_ms = tb->render_ms;
	return NEUS2B_OK;
}

// ------------------------------------------------------------------------------------------------ dynamic sequences

extern "C" int neus2b_testbed_next_frame(neus2b_testbed* tb, const uint32_t* h_pixels, const float* h_xforms, const float* h_focal,
                                         const float* h_principal) {
	if (!tb || !tb->ds.n_images || !h_pixels || !h_xforms || !h_focal || !h_principal) return NEUS2B_E_INVALID;
	if (tb->step_pending) return NEUS2B_E_INVALID;  // between the halves of a step
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	if (int jr = join_generation(tb)) return jr;  // samples may still be drawn on the side stream
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	// NerfNetwork::accumulate_global_movement (src/testbed.cu:2044) with the motion as trained (its fp16 parameters)
	if (tb->frame >= 1 && tb->cfg.predict_global_movement) {
		uint16_t hb[12];
		N2B_CHECK_CUDA(cudaMemcpy(hb, tb->delta, sizeof(hb), cudaMemcpyDeviceToHost));
		int rc = neus2b_movement_accumulate(hb, tb->acc_rotation, tb->acc_transition);
		if (rc) return rc;
	}
	// load_nerf(frame): the new images and cameras
	const size_t npx = (size_t)tb->ds.n_images * tb->ds.width * tb->ds.height;
	N2B_CHECK_CUDA(cudaMemcpyAsync((void*)tb->ds.d_pixels, h_pixels, npx * 4, cudaMemcpyHostToDevice, tb->stream));
	int rc = neus2b_testbed_update_cameras(tb, h_xforms, h_focal, h_principal);
	if (rc) return rc;
	// save_snapshot_incremental(no optimizer state) + load_snapshot_incremental (src/testbed.cu:2052-2053, 3169-3256): the fp16
	// parameters become every copy of the weights, Adam starts from zero moments, the EMA from the weights
	half_to_master_kernel<<<kSMs * 4, 256, 0, tb->stream>>>(tb->n_params, tb->params, tb->master, tb->ema_master, tb->params_ema);
	N2B_CHECK_LAUNCH();
	N2B_CHECK_CUDA(cudaMemsetAsync(tb->adam_m, 0, sizeof(float) * tb->n_params, tb->stream));
	N2B_CHECK_CUDA(cudaMemsetAsync(tb->adam_v, 0, sizeof(float) * tb->n_params, tb->stream));
	N2B_CHECK_CUDA(cudaMemsetAsync(tb->grad_grid, 0, sizeof(__half) * tb->n_grid, tb->stream));
	N2B_CHECK_CUDA(cudaMemsetAsync(tb->grad_mlp, 0, sizeof(float) * (NEUS2B_MLP_N + 4), tb->stream));
	rc = reset_delta(tb);  // a new DeltaNetwork trainer: identity motion, fresh optimizer (src/testbed.cu:2559-2568)
	if (rc) return rc;
	N2B_CHECK_CUDA(cudaMemsetAsync(tb->delta_sums, 0, sizeof(float) * 12, tb->stream));
	++tb->frame;
	tb->training_step = 0;
	tb->canonical_step = 0;
	tb->adam_step = 0;
	tb->train_canonical = false;  // src/testbed.cu:2065-2068
	tb->train_delta = tb->cfg.predict_global_movement != 0;
	tb->pregenerated = tb->tuned = false;
	// reset_network_incremental (src/testbed.cu:2341-2352): the ray generator's stream and the ray count restart
	neus2b_pcg32 r;
	neus2b_pcg32_seed(&r, tb->cfg.seed);
	tb->rng = Pcg32{r.state, r.inc};
	TrainState st{};
	N2B_CHECK_CUDA(cudaMemcpyAsync(tb->h_state, tb->state, sizeof(TrainState), cudaMemcpyDeviceToHost, tb->stream));
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	st = *tb->h_state;
	st.rays_per_batch = 1u << 12;
	st.measured_pre = 0;
	*tb->h_state = st;
	N2B_CHECK_CUDA(cudaMemcpyAsync(tb->state, tb->h_state, sizeof(TrainState), cudaMemcpyHostToDevice, tb->stream));
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_get_movement(neus2b_testbed* tb, uint32_t* frame, float rotation[9], float transition[3], float delta[12]) {
	if (!tb) return NEUS2B_E_INVALID;
	if (frame) *frame = tb->frame;
	if (rotation) memcpy(rotation, tb->acc_rotation, sizeof(tb->acc_rotation));
	if (transition) memcpy(transition, tb->acc_transition, sizeof(tb->acc_transition));
	if (delta) {
		N2B_CHECK_CUDA(cudaSetDevice(tb->device));
		N2B_CHECK_CUDA(cudaMemcpyAsync(delta, tb->delta_master, sizeof(float) * 12, cudaMemcpyDeviceToHost, tb->stream));
		N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	}
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_set_movement(neus2b_testbed* tb, uint32_t frame, const float rotation[9], const float transition[3],
                                           const float delta[12]) {
	if (!tb || !rotation || !transition) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	if (int jr = join_generation(tb)) return jr;  // samples may still be drawn on the side stream
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	tb->frame = frame;
	memcpy(tb->acc_rotation, rotation, sizeof(tb->acc_rotation));
	memcpy(tb->acc_transition, transition, sizeof(tb->acc_transition));
	tb->train_delta = frame >= 1 && tb->cfg.predict_global_movement;
	tb->train_canonical = frame == 0 || tb->training_step >= predict_steps(tb);
	tb->canonical_step = next_canonical_step(tb, tb->training_step);
	tb->pregenerated = false;
	return delta ? write_delta(tb, delta) : NEUS2B_OK;
}

// ------------------------------------------------------------------------------------------------ snapshot state

extern "C" int neus2b_testbed_get_training_state(neus2b_testbed* tb, neus2b_training_state* out) {
	if (!tb || !out) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	N2B_CHECK_CUDA(cudaMemcpyAsync(tb->h_state, tb->state, sizeof(TrainState), cudaMemcpyDeviceToHost, tb->stream));
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	out->training_step = tb->training_step;
	out->density_grid_ema_step = tb->ema_step;
	out->rays_per_batch = tb->h_state->rays_per_batch;
	out->n_rays_total = tb->h_state->n_rays_total;
	out->measured_batch_size = tb->h_state->measured;
	out->measured_batch_size_before_compaction = tb->h_state->measured_pre;
	out->loss = tb->h_state->loss;
	out->ek_loss = tb->h_state->ek_loss;
	out->rng = neus2b_pcg32{tb->rng.state, tb->rng.inc};
	out->density_rng = neus2b_pcg32{tb->density_rng.state, tb->density_rng.inc};
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_set_training_state(neus2b_testbed* tb, const neus2b_training_state* in) {
	if (!tb || !in || in->rays_per_batch == 0 || in->rays_per_batch > tb->max_rays) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	if (int jr = join_generation(tb)) return jr;  // samples may still be drawn on the side stream
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	tb->training_step = in->training_step;
	tb->canonical_step = next_canonical_step(tb, tb->training_step);
	tb->train_canonical = tb->frame == 0 || tb->training_step >= predict_steps(tb);
	if (tb->frame >= 1) tb->train_delta = tb->cfg.predict_global_movement && (tb->cfg.finetune_global_movement || tb->training_step < predict_steps(tb));
	if (tb->frame == 0) tb->adam_step = in->training_step;  // the first frame's optimizer has taken every step
	else tb->adam_step = tb->training_step > predict_steps(tb) ? tb->training_step - predict_steps(tb) : 0u;
	tb->pregenerated = tb->tuned = false;
	tb->ema_step = in->density_grid_ema_step;
	tb->rng = Pcg32{in->rng.state, in->rng.inc};
	tb->density_rng = Pcg32{in->density_rng.state, in->density_rng.inc};
	TrainState st{};
	st.rays_per_batch = in->rays_per_batch;
	st.n_rays_total = in->n_rays_total;
	st.measured = in->measured_batch_size;
	st.measured_pre = in->measured_batch_size_before_compaction;
	st.loss = in->loss;
	st.ek_loss = in->ek_loss;
	*tb->h_state = st;
	N2B_CHECK_CUDA(cudaMemcpyAsync(tb->state, tb->h_state, sizeof(TrainState), cudaMemcpyHostToDevice, tb->stream));
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	return NEUS2B_OK;
}

static int state_array(neus2b_testbed* tb, int which, void** ptr, uint64_t* bytes) {
	const uint64_t cells = (uint64_t)NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * NEUS2B_GRIDSIZE * tb->cfg.n_cascades;
	switch (which) {
		case NEUS2B_ARRAY_MASTER: *ptr = tb->master; *bytes = tb->n_params * 4; return NEUS2B_OK;
		case NEUS2B_ARRAY_ADAM_M: *ptr = tb->adam_m; *bytes = tb->n_params * 4; return NEUS2B_OK;
		case NEUS2B_ARRAY_ADAM_V: *ptr = tb->adam_v; *bytes = tb->n_params * 4; return NEUS2B_OK;
		case NEUS2B_ARRAY_EMA_MASTER: *ptr = tb->ema_master; *bytes = tb->n_params * 4; return NEUS2B_OK;
		case NEUS2B_ARRAY_PARAMS: *ptr = tb->params; *bytes = tb->n_params * 2; return NEUS2B_OK;
		case NEUS2B_ARRAY_PARAMS_EMA: *ptr = tb->params_ema; *bytes = tb->n_params * 2; return NEUS2B_OK;
		case NEUS2B_ARRAY_DENSITY_GRID: *ptr = tb->density_grid; *bytes = cells * 4; return NEUS2B_OK;
		default: return NEUS2B_E_INVALID;
	}
}

extern "C" int neus2b_testbed_get_array(neus2b_testbed* tb, int which, void* h_out, uint64_t bytes) {
	if (!tb || !h_out) return NEUS2B_E_INVALID;
	void* p = nullptr;
	uint64_t n = 0;
	int rc = state_array(tb, which, &p, &n);
	if (rc) return rc;
	if (bytes != n) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	N2B_CHECK_CUDA(cudaMemcpyAsync(h_out, p, n, cudaMemcpyDeviceToHost, tb->stream));
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	return NEUS2B_OK;
}

extern "C" int neus2b_testbed_set_array(neus2b_testbed* tb, int which, const void* h_in, uint64_t bytes) {
	if (!tb || !h_in) return NEUS2B_E_INVALID;
	void* p = nullptr;
	uint64_t n = 0;
	int rc = state_array(tb, which, &p, &n);
	if (rc) return rc;
	if (bytes != n) return NEUS2B_E_INVALID;
	N2B_CHECK_CUDA(cudaSetDevice(tb->device));
	if (int jr = join_generation(tb)) return jr;  // samples may still be drawn on the side stream
	N2B_CHECK_CUDA(cudaMemcpyAsync(p, h_in, n, cudaMemcpyHostToDevice, tb->stream));
	if (which == NEUS2B_ARRAY_DENSITY_GRID) {  // update_density_grid_mean_and_bitfield, as load_snapshot does (src/testbed.cu:3228-3230)
		rc = neus2b_occupancy_mean_and_bitfield(tb->cfg.n_cascades, tb->density_grid, tb->bitfield, tb->density_mean, tb->occ_partial, tb->stream);
		if (rc) return rc;
		tb->occ_bounds_stale = true;
		tb->pregenerated = false;  // samples drawn ahead were marched through the previous occupancy bits
	}
	N2B_CHECK_CUDA(cudaStreamSynchronize(tb->stream));
	return NEUS2B_OK;
}

