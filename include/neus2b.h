/*
 * neus2b -- C ABI of the B200-native NeuS2 training-step kernels (libneus2b.so).
 *
 * Plain pointers and sizes only.  Every pointer named d_* is DEVICE memory owned by the caller; nothing in the
 * kernel-level section allocates.  fp16 tensors are passed as `uint16_t*` bit patterns (device `__half`).
 * All matrices are "AoS" (tiny-cuda-nn's column-major GPUMatrix): one sample's values are contiguous, [n][width].
 * Return value: 0 on success, a positive cudaError_t, or a negative NEUS2B_E_* code.  Nothing throws across this ABI
 * and nothing touches the default stream: every call enqueues on the `stream` it is given.
 *
 * Each entry point names the reference interface it stands in for (file:line inside 19reborn/NeuS2).  The bodies of
 * the tiny-cuda-nn methods are not part of that tree (empty submodule dependencies/neus2_tcnn); the citation is the
 * call site that fixes their contract.
 */
#ifndef NEUS2B_H
#define NEUS2B_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* neus2b_stream_t;

#define NEUS2B_OK 0
#define NEUS2B_E_INVALID (-1)     /* bad argument (null pointer, unsupported width, misaligned pointer) */
#define NEUS2B_E_UNSUPPORTED (-2) /* configuration outside what the kernels are built for */
#define NEUS2B_E_NO_DEVICE (-3)
#define NEUS2B_E_OVERFLOW (-4)    /* a device-side capacity was exceeded (flag read back by the caller) */
#define NEUS2B_E_TOO_LARGE (-5)   /* request beyond a fixed compiled-in capacity */
#define NEUS2B_E_IO (-6)          /* a file could not be opened or written */
#define NEUS2B_E_DEVICE (-7)      /* a kernel raised the sticky device error flag (neus2b_device_error_flags) */
#define NEUS2B_E_TIMEOUT (-8)     /* a bounded wait on the host ran out */

#define NEUS2B_MAX_LEVELS 16
#define NEUS2B_GRIDSIZE 128u /* NERF_GRIDSIZE  include/neural-graphics-primitives/nerf.h:24 */
#define NEUS2B_CASCADES 8u   /* NERF_CASCADES  src/testbed_nerf.cu:49 */
#define NEUS2B_STEPS 1024u   /* NERF_STEPS     src/testbed_nerf.cu:48 */

/* tcnn::EGradientMode (include/neural-graphics-primitives/nerf_network.h:229,402,534) */
#define NEUS2B_GRAD_IGNORE 0
#define NEUS2B_GRAD_OVERWRITE 1
#define NEUS2B_GRAD_ACCUMULATE 2

/* Hash-grid geometry: the "encoding" block of configs/nerf/base.json:29-39 (n_features_per_level is fixed at 2). */
typedef struct {
	uint32_t n_levels;          /* <= 16 */
	uint32_t log2_hashmap_size;
	uint32_t base_resolution;
	float per_level_scale;
	uint32_t n_active_levels;   /* progressive mask (Encoding::set_training_step, src/testbed.cu:2643-2647) */
} neus2b_grid_desc;

/* Parameter block order, fp16 scalars (NerfNetwork::set_params, nerf_network.h:728-772):
 * SDF MLP 64x48,16x64 | colour MLP 64x48,64x64,16x64 | grid | variance (4). Weight matrices are row-major [out][in]. */
#define NEUS2B_SDF_W1 0
#define NEUS2B_SDF_W2 3072
#define NEUS2B_RGB_W1 4096
#define NEUS2B_RGB_W2 7168
#define NEUS2B_RGB_W3 11264
#define NEUS2B_MLP_N 12288
#define NEUS2B_GRID_OFF 12288

const char* neus2b_version(void);
/* Kernel launches this library has issued in this process so far (a counter every launch site increments; for callers that
 * want to state how many of the library's kernels ran inside a timed region). */
uint64_t neus2b_launch_count(void);
const char* neus2b_error_string(int code);
/* sizeof of the structures of this header as the loaded library was compiled, in header order: grid_desc, motion, pcg32, dataset,
 * train_cfg, ray_workspace, adam_cfg, testbed_config, train_stats, render_cfg, render_workspace, render_request, training_state.
 * Writes at most `capacity` entries and returns how many there are; a binding compares them with its own before it passes a pointer. */
uint32_t neus2b_abi_struct_sizes(uint32_t* sizes, uint32_t capacity);

/* GridEncoding::level_n_params / level_params_offset (src/testbed.cu:1861-1877).  offsets[17] in grid ENTRIES (2 fp16). */
int neus2b_grid_level_table(const neus2b_grid_desc* desc, uint32_t* offsets, uint32_t* resolutions, float* scales,
                            uint32_t* hashed);
int neus2b_grid_n_params(const neus2b_grid_desc* desc, uint64_t* n_fp16);  /* Encoding::n_params() */
int neus2b_model_n_params(const neus2b_grid_desc* desc, uint64_t* n_fp16); /* NerfNetwork::n_params(), nerf_network.h:902 */

/* ---------------------------------------------------------------- component kernels (tcnn Encoding / Network) */

/* GridEncoding::forward with prepare_input_gradients (nerf_network.h:184-190; inference :671-676).
 * d_x [n][x_stride] fp32 (first 3 used), d_enc [n][2L] fp16, d_dy_dx [n][2L][3] fp32 or NULL. */
int neus2b_grid_forward(const neus2b_grid_desc* desc, uint32_t n, const float* d_x, uint32_t x_stride, const uint16_t* d_grid,
                        uint16_t* d_enc, float* d_dy_dx, neus2b_stream_t stream);
/* GridEncoding::backward(..., &dL_dinput, EGradientMode::Ignore) (nerf_network.h:234). d_dL_dx [n][3] fp32. */
int neus2b_grid_backward_input(const neus2b_grid_desc* desc, uint32_t n, const float* d_x, uint32_t x_stride,
                               const uint16_t* d_grid, const uint16_t* d_dL_denc, float* d_dL_dx, neus2b_stream_t stream);
/* GridEncoding::backward(..., param_gradients_mode) (nerf_network.h:419-429). d_grad [grid n_params] fp16. */
int neus2b_grid_backward_params(const neus2b_grid_desc* desc, uint32_t n, const float* d_x, uint32_t x_stride,
                                const uint16_t* d_dL_denc, uint16_t* d_grad, int grad_mode, neus2b_stream_t stream);
/* GridEncoding::backward_backward_input (nerf_network.h:534-544): d_v = dL/d(dy/dx) [n][3] fp32, d_g_e = dL_doutput of the
 * first-order pass [n][2L] fp16; writes d_dy_enc [n][2L] fp16 (dL/d(dL_doutput)) and adds the parameter gradient. */
int neus2b_grid_backward_backward_input(const neus2b_grid_desc* desc, uint32_t n, const float* d_x, uint32_t x_stride,
                                        const uint16_t* d_grid, const float* d_v, const uint16_t* d_g_e, uint16_t* d_dy_enc,
                                        uint16_t* d_grad, int grad_mode, neus2b_stream_t stream);

/* FullyFusedMLP::forward, 64 neurons, ReLU, no output activation, 16 outputs (nerf_network.h:212 SDF net: in_width 48,
 * n_hidden 1; :271 colour net: in_width 48, n_hidden 2).  d_hidden [n][n_hidden][64] fp16 may be NULL. */
int neus2b_mlp_forward(uint32_t n, uint32_t in_width, uint32_t n_hidden, const uint16_t* d_weights, const uint16_t* d_in,
                       uint16_t* d_out, uint16_t* d_hidden, neus2b_stream_t stream);
/* Same contract as neus2b_mlp_forward, computed with tcgen05.mma on 128-sample tiles with the accumulators in tensor memory
 * (in_width 48 with 1 or 2 hidden layers, or 64 with 2).  d_status (optional, device uint32) gets bit 0 set if a bounded
 * completion wait inside the kernel ran out. */
int neus2b_mlp_forward_tcgen05(uint32_t n, uint32_t in_width, uint32_t n_hidden, const uint16_t* d_weights, const uint16_t* d_in,
                               uint16_t* d_out, uint16_t* d_hidden, uint32_t* d_status, neus2b_stream_t stream);
/* FullyFusedMLP::backward (nerf_network.h:229,340,402,509). d_dL_din [n][in_width] fp16 or NULL; d_wgrad fp32
 * [n_params of the net] or NULL (EGradientMode::Ignore). */
int neus2b_mlp_backward(uint32_t n, uint32_t in_width, uint32_t n_hidden, const uint16_t* d_weights, const uint16_t* d_in,
                        const uint16_t* d_hidden, const uint16_t* d_dL_dout, uint16_t* d_dL_din, float* d_wgrad,
                        int grad_mode, neus2b_stream_t stream);
/* FullyFusedMLP::backward_backward_input, one hidden layer (nerf_network.h:560-571): d_u = dL/d(dL_dinput) [n][in_width],
 * d_dy = dL_doutput of the differentiated pass [n][16]; adds into d_wgrad. */
int neus2b_mlp_backward_backward_input(uint32_t n, uint32_t in_width, const uint16_t* d_weights, const uint16_t* d_hidden,
                                       const uint16_t* d_u, const uint16_t* d_dy, float* d_wgrad, int grad_mode,
                                       neus2b_stream_t stream);
/* SphericalHarmonics degree 4 of 2*dir-1 (configs/nerf/base.json:48-62; nerf_network.h:251). */
int neus2b_sh4_forward(uint32_t n, const float* d_dir01, uint32_t stride, uint16_t* d_out, neus2b_stream_t stream);

typedef struct neus2b_motion neus2b_motion; /* dynamic sequences: the frame's learned rigid motion, defined below */

/* ---------------------------------------------------------------- fused NeuS graph (NerfNetwork) */

/* Two implementations of the fused graph kernels exist: tcgen05.mma on 128-sample CTA tiles with accumulators in tensor
 * memory (default) and mma.sync on 16-sample warp tiles.  Process-wide switch, for A/B measurements and tests. */
#define NEUS2B_MMA_SYNC 0
#define NEUS2B_MMA_TCGEN05 1
int neus2b_set_mma_path(int path);
int neus2b_get_mma_path(void);
/* Sticky device-side error bits (bit 0: a bounded completion wait inside a tcgen05 kernel ran out). Synchronises. */
int neus2b_device_error_flags(uint32_t* h_flags);
/* Overwrites the sticky bits (0 clears them).  For hosts that recovered from an error, and for tests of the error path:
 * the training loop reports NEUS2B_E_DEVICE from its statistics call while a bit is set. */
int neus2b_set_device_error_flags(uint32_t flags);

/* NerfNetwork::inference_mixed_precision == forward_impl (nerf_network.h:87-90,132-315), static scene.
 * d_coords [n][7] fp32 (xyz, dt, dir in [0,1]); d_out [n][16] fp16 rows: 0-2 raw rgb, 3 sdf+bias, 4-6 normal,
 * 7 variance, 8-10 dir.  If d_n is non-NULL the sample count is read from it on the device (clamped to n). */
int neus2b_neus_forward(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n,
                        const uint32_t* d_n, const float* d_coords, uint16_t* d_out, neus2b_stream_t stream);
/* NerfNetwork::forward + backward of one training batch in a single pass (nerf_network.h:132-315 + :317-641,
 * called at src/testbed_nerf.cu:3931-3932).  Gradients are accumulated: d_grad_mlp fp32 [12288], d_grad_grid fp16
 * [grid n_params], d_grad_variance fp32 [1]; zero them first for EGradientMode::Overwrite. */
int neus2b_neus_train(const neus2b_grid_desc* desc, const uint16_t* d_params, uint32_t n, const float* d_coords,
                      const uint16_t* d_dL_dout, uint32_t indeed_batch_size, float* d_grad_mlp, uint16_t* d_grad_grid,
                      float* d_grad_variance, neus2b_stream_t stream);
/* ---- dynamic sequences: the DeltaNetwork (include/neural-graphics-primitives/transform_network.h:26-170), a learned rigid
 * motion applied to every sample ahead of the encoding while the frames after the first are trained (NerfNetwork::forward_impl
 * with m_use_delta, nerf_network.h:149-169; backward :589-625).  d_delta: 12 fp16 parameters in the network's own order,
 * transition [0..3] (xyz, one unused) then the 6-D rotation [4..11] (two 3-vectors, two unused); identity = 0 0 0 0 | 1 0 0 0 1 0 0 0.
 * A sample moves as x' = R (x + t - first_frame_offset) + first_frame_offset, dir' = (R (2 dir - 1) + 1) / 2. */
struct neus2b_motion {
	const uint16_t* d_delta;     /* NULL: no motion (the first frame; m_use_delta false) */
	float first_frame_offset[3]; /* Testbed::m_first_frame_offset (testbed.h:455), 0 */
	float* d_sums;               /* training only, optional: float[12], the backward's batch sums are ADDED here:
	                                [0..2] sum of dL/dx', [3..11] sum of dL/dx' (x) (x + t) row-major; neus2b_delta_optimizer_step
	                                turns them into the parameters' gradients (NULL: m_train_delta false) */
};
/* neus2b_neus_forward / _train / _sdf with the motion applied first (motion may be NULL = the plain call).  In the training
 * call the three canonical gradient pointers may all be NULL: the canonical model is frozen and only motion->d_sums is
 * produced (the reference's m_train_canonical = false while it predicts a frame's global movement). */
int neus2b_neus_forward_moved(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n,
                              const uint32_t* d_n, const float* d_coords, const neus2b_motion* motion, uint16_t* d_out,
                              neus2b_stream_t stream);
/* The same pass on a list of samples: entry i reads row d_index[i] of d_coords and writes row d_index[i] of d_out (d_index NULL:
 * row i; a list needs the tcgen05 path).  n, d_n: capacity and device-side length of the list. */
int neus2b_neus_forward_indexed(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n,
                                const uint32_t* d_n, const uint32_t* d_index, const float* d_coords, const neus2b_motion* motion,
                                uint16_t* d_out, neus2b_stream_t stream);
int neus2b_neus_train_moved(const neus2b_grid_desc* desc, const uint16_t* d_params, uint32_t n, const float* d_coords,
                            const neus2b_motion* motion, const uint16_t* d_dL_dout, uint32_t indeed_batch_size, float* d_grad_mlp,
                            uint16_t* d_grad_grid, float* d_grad_variance, neus2b_stream_t stream);
int neus2b_neus_sdf_moved(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n, const float* d_x,
                          uint32_t x_stride, const neus2b_motion* motion, uint16_t* d_sdf, neus2b_stream_t stream);
/* DeltaNetwork::forward_impl alone (add_global_movement_with_rotation_6d, common_operation.cuh:419-474): coords [n][7]. */
int neus2b_delta_forward(const uint16_t* d_delta, const float first_frame_offset[3], uint32_t n, const float* d_coords_in,
                         float* d_coords_out, neus2b_stream_t stream);
/* DeltaNetwork::backward_impl's per-sample part (add_loss_to_rotation_6d_each, common_operation.cuh:793-849) reduced over the
 * batch on the device: d_dL_dx [n][3] is the gradient w.r.t. the moved positions; the twelve sums are added to d_sums. */
int neus2b_delta_backward(const uint16_t* d_delta, uint32_t n, const float* d_coords_in, const float* d_dL_dx, float* d_sums,
                          neus2b_stream_t stream);
/* NerfNetwork::accumulate_global_movement (nerf_network.h:1153-1167; accumulate_global_movement_rotation_6d_kernel,
 * common_operation.cuh:555-589) on the host: rotation [9] row-major <- R rotation, transition [3] <- R (transition + t), both
 * rounded to fp16-representable values (the reference keeps them in fp16 buffers). */
int neus2b_movement_accumulate(const uint16_t h_delta[12], float rotation[9], float transition[3]);

/* NerfNetwork::sdf (nerf_network.h:643-709): d_sdf [n] fp16 = y0 + bias. */
int neus2b_neus_sdf(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n, const float* d_x,
                    uint32_t x_stride, uint16_t* d_sdf, neus2b_stream_t stream);

/* ---------------------------------------------------------------- ray march, loss, occupancy (src/testbed_nerf.cu) */

typedef struct {
	uint64_t state, inc;
} neus2b_pcg32; /* tcnn::default_rng_t */
void neus2b_pcg32_seed(neus2b_pcg32* rng, uint64_t seed); /* default_rng_t{seed}: stream selector 1, as the constructor defaults */
void neus2b_pcg32_advance(neus2b_pcg32* rng, uint64_t delta);

typedef struct {
	uint32_t n_images, width, height;
	const uint32_t* d_pixels; /* [n_images][height][width] RGBA8 (EImageDataType::Byte) */
	const float* d_xforms;    /* [n_images][12] 3x4 camera-to-world, column major (TrainingXForm::start) */
	const float* d_focal;     /* [n_images][2]  (TrainingImageMetadata::focal_length) */
	const float* d_principal; /* [n_images][2]  (TrainingImageMetadata::principal_point) */
} neus2b_dataset;

typedef struct {
	float aabb_min[3], aabb_max[3];
	float cone_angle_constant;
	uint32_t snap_to_pixel_centers;
	uint32_t random_bg_color;
	float background_color[3];
	float loss_scale; /* LOSS_SCALE, include/neural-graphics-primitives/testbed.h:237 */
	float mask_loss_weight, ek_loss_weight, cos_anneal_ratio;
	/* data-parallel ray sharding: this process draws rays [ray_index_offset, ray_index_offset + n_rays) of a logical
	 * batch that is ray_count_scale times larger (loss normalisation uses n_rays * ray_count_scale); 0 / 1 = single GPU */
	uint32_t ray_index_offset, ray_count_scale;
	/* dynamic sequences: the accumulated global movement of the earlier frames, applied to every ray before the march
	 * (global_movement_with_rotation_6d, src/testbed_nerf.cu:183-203; call sites :1370-1378, :1550-1558):
	 * o = R (o - first_frame_offset) + t, dir = R dir with dir normalised before and not again after.  rotation row-major.
	 * With it the rays written to d_rays are the moved ones (origin, unit direction). */
	uint32_t use_global_movement;
	float rotation[9], transition[3], first_frame_offset[3];
} neus2b_train_cfg;

/* Scratch for one batch of rays; every array is caller-allocated device memory.  One call handles at most
 * NEUS2B_MAX_RAYS_PER_CALL rays (the capacity of the ray-order prefix sum); more returns NEUS2B_E_TOO_LARGE. */
#define NEUS2B_MAX_RAYS_PER_CALL (1u << 20)
typedef struct {
	uint32_t max_rays, max_samples;
	uint32_t* d_ray_indices; /* [max_rays] */
	float* d_rays;           /* [max_rays][6] origin, unnormalised direction */
	uint32_t* d_numsteps;    /* [max_rays][2] {n, base} */
	float* d_coords;         /* [max_samples][7] */
	uint32_t* d_counters;    /* [8]: 0 kept rays, 1 samples, 2 compacted samples (unclipped), 3 overflow flag,
	                            5 samples the windowed network pass evaluated */
	uint64_t* d_scan_tmp;    /* [max_rays + 1024]: keys, the total behind them and 1023 entries of scan scratch */
	float* d_ray_tmp;        /* [max_rays][8] */
	const uint32_t* d_n_rays_total; /* optional: overrides the n_rays_total argument with a device value */
	uint32_t* d_march_masks;        /* optional [max_rays][64]: lets the second march pass skip the occupancy lookups */
	const int32_t* d_occupied_bounds; /* optional int32[6] from neus2b_occupancy_bounds: rays that miss the box of occupied
	                                     cells are not marched (they cannot take a sample; the result is unchanged) */
	uint32_t* d_window_list;          /* optional [max_samples]: sample rows of the current window (neus2b_forward_compute_loss) */
	uint32_t* d_window_lens;          /* optional [8]: the length of each window's list */
	const uint32_t* d_prev_samples;   /* optional: the sample count of the previous training step, read on the device.  When it
	                                     is not zero, rays whose samples end beyond that count rounded up to 128 are dropped
	                                     like rays beyond max_samples: the training loop's max_inference
	                                     (src/testbed_nerf.cu:3764-3769, passed to the generator as its max_samples :3801) */
} neus2b_ray_workspace;

/* generate_training_samples_nerf_with_global_movement (src/testbed_nerf.cu:1253-1446), static scene; sample order is
 * canonical (by ray index, prefix sum) instead of atomicAdd order.  If d_n_rays is non-NULL the ray count is read on
 * the device (clamped to n_rays). */
int neus2b_generate_samples(const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays, const uint32_t* d_n_rays,
                            uint32_t n_rays_total, neus2b_pcg32 rng, const uint8_t* d_bitfield, neus2b_ray_workspace* ws,
                            neus2b_stream_t stream);
/* No counterpart in the reference.  Same result as neus2b_generate_samples, for hosts that cannot give the library any
 * scratch memory: callers that have handed the whole device to their own allocator, or that may not call cudaMalloc
 * after start-up because it synchronises the device and can fail late.  The generator's scratch (per-ray staging
 * records and prefix-sum keys, about 2.5 MiB) sits in static device arrays inside the library, so this call allocates
 * nothing -- no cudaMalloc, no cudaFree, no allocating library routine -- and takes at most NEUS2B_STATIC_MAX_RAYS rays
 * (more returns NEUS2B_E_TOO_LARGE).  The first call on a device looks the arrays' addresses up
 * (cudaGetSymbolAddress); make that first call before any stream capture.  All calls on a device share the arrays:
 * calls that overlap on the GPU race, so issue them one after another on one stream.
 * This is the plain form of the generator: it takes neither the optional record of march masks nor the box of occupied
 * cells that neus2b_ray_workspace can carry, so every ray is marched twice and none is culled (same result, more time).
 * Outputs (caller-allocated): d_ray_indices [n_rays], d_rays [n_rays][6], d_numsteps [n_rays][2],
 * d_coords [max_samples][7], d_counters [8] (layout as in neus2b_ray_workspace). */
#define NEUS2B_STATIC_MAX_RAYS 65536u
int neus2b_generate_samples_static(const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays,
                                   const uint32_t* d_n_rays, uint32_t n_rays_total, neus2b_pcg32 rng, const uint8_t* d_bitfield,
                                   uint32_t max_samples, uint32_t* d_ray_indices, float* d_rays, uint32_t* d_numsteps,
                                   float* d_coords, uint32_t* d_counters, neus2b_stream_t stream);
/* compute_loss_kernel_train_nerf_with_global_movement (src/testbed_nerf.cu:1465-1996) followed by fill_rollover /
 * fill_rollover_and_rescale (:3908-3916).  d_mlp_out [samples][16] fp16 from neus2b_neus_forward on ws->d_coords.
 * Writes d_coords_out [max_compacted][7], d_dloss_dout [max_compacted][16] fp16, per-ray d_loss / d_ek_loss [max_rays]. */
int neus2b_compute_loss(const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays, const uint32_t* d_n_rays,
                        uint32_t n_rays_total, neus2b_pcg32 rng, uint32_t max_compacted, const uint16_t* d_mlp_out,
                        neus2b_ray_workspace* ws, float* d_coords_out, uint16_t* d_dloss_dout, float* d_loss, float* d_ek_loss,
                        int rollover, neus2b_stream_t stream);

/* The network pass over the step's samples (src/testbed_nerf.cu:3840) and the loss pass (:3845-3916) in one call that evaluates
 * the network only on samples whose output is used.  Rays are evaluated in windows of consecutive samples: the first
 * window_ends[0] samples of every ray, then [window_ends[0], window_ends[1]) of the rays that are still transparent, ...,
 * finally the rest of the rays that remain (window_ends: host array, increasing, at most NEUS2B_MAX_FORWARD_WINDOWS entries;
 * n_windows == 0: every sample, then the loss pass, in the reference's order).  Same per-ray records, compacted batch and loss
 * gradient as neus2b_neus_forward on all samples followed by neus2b_compute_loss; rows of d_mlp_out [max_samples][16] behind a
 * ray's last evaluated sample keep what they held.  Needs ws->d_window_list and ws->d_window_lens when n_windows > 0 and the
 * tcgen05 path.  motion: NULL for a static scene. */
#define NEUS2B_MAX_FORWARD_WINDOWS 6
int neus2b_forward_compute_loss(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, const neus2b_motion* motion,
                                const neus2b_dataset* ds, const neus2b_train_cfg* cfg, uint32_t n_rays, const uint32_t* d_n_rays,
                                uint32_t n_rays_total, neus2b_pcg32 rng, uint32_t max_compacted, neus2b_ray_workspace* ws,
                                const uint32_t* window_ends, uint32_t n_windows, uint16_t* d_mlp_out, float* d_coords_out,
                                uint16_t* d_dloss_dout, float* d_loss, float* d_ek_loss, int rollover, neus2b_stream_t stream);

/* Occupancy grid (src/testbed_nerf.cu:630-785, 3287-3391). One call = update_density_grid_nerf's inner step for
 * n_uniform + n_nonuniform samples followed by update_density_grid_mean_and_bitfield.
 * d_grid float[128^3 * n_cascades], d_grid_tmp same size, d_bitfield uint8[128^3], d_mean float[1],
 * scratch: d_pos float[n][3], d_idx uint32[n], d_sdf fp16[n], d_partial double[1024]. */
int neus2b_occupancy_update(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n_cascades,
                            uint32_t n_uniform, uint32_t n_nonuniform, neus2b_pcg32 rng_uniform, neus2b_pcg32 rng_nonuniform,
                            uint32_t ema_step, float decay, float* d_grid, float* d_grid_tmp, uint8_t* d_bitfield,
                            float* d_mean, float* d_pos, uint32_t* d_idx, uint16_t* d_sdf, double* d_partial,
                            neus2b_stream_t stream);

/* The same while a later frame of a dynamic sequence is trained: the SDF is queried through the frame's motion
 * (NerfNetwork::density applies the DeltaNetwork, nerf_network.h:651-662).  motion may be NULL. */
int neus2b_occupancy_update_moved(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n_cascades,
                                  uint32_t n_uniform, uint32_t n_nonuniform, neus2b_pcg32 rng_uniform, neus2b_pcg32 rng_nonuniform,
                                  uint32_t ema_step, float decay, float* d_grid, float* d_grid_tmp, uint8_t* d_bitfield,
                                  float* d_mean, float* d_pos, uint32_t* d_idx, uint16_t* d_sdf, double* d_partial,
                                  const neus2b_motion* motion, neus2b_stream_t stream);

/* Smallest box of cell indices {min x, y, z, max x, y, z} around the set bits of the finest level of the occupancy bitfield
 * (min > max when nothing is occupied); no counterpart in the reference, which marches every ray. */
int neus2b_occupancy_bounds(const uint8_t* d_bitfield, int32_t* d_bounds, neus2b_stream_t stream);
/* update_density_grid_mean_and_bitfield alone (src/testbed_nerf.cu:3371-3391): mean of the finest level, occupancy bits of
 * every level from d_grid float[128^3 * n_cascades]; d_partial double[1024] scratch. */
int neus2b_occupancy_mean_and_bitfield(uint32_t n_cascades, const float* d_grid, uint8_t* d_bitfield, float* d_mean, double* d_partial,
                                       neus2b_stream_t stream);

/* ---------------------------------------------------------------- optimizer (Trainer::optimizer_step, src/testbed_nerf.cu:3498) */
/* What the optimizer does where the un-vendored tiny-cuda-nn fork cannot be read; 0 = the default behaviour of this
 * library (Adam of the public tiny-cuda-nn: weight decay on the matrix weights only, entries without a gradient left
 * alone, bias-corrected EMA).  The flags exist so that each choice can be switched on its own. */
#define NEUS2B_ADAM_UPDATE_UNTOUCHED 1u /* also update non-matrix entries whose gradient is exactly zero (moments decay) */
#define NEUS2B_ADAM_L2_ALL 2u           /* weight decay on every parameter, not only the matrix weights */
#define NEUS2B_ADAM_EMA_NO_DEBIAS 4u    /* plain EMA ema = d * ema + (1 - d) * w, without the 1 / (1 - d^t) correction */
typedef struct {
	float learning_rate, beta1, beta2, epsilon, l2_reg, ema_decay, loss_scale;
	uint32_t step;     /* 1-based */
	uint32_t n_matrix; /* leading MLP-weight entries */
	uint32_t flags;    /* NEUS2B_ADAM_* */
	/* optional device counter: a gradient that is NaN or infinite (an overflowed fp16 sum, a poisoned exchange buffer) is
	 * treated as absent -- that parameter keeps its weight and moments this step, the gradient slot is cleared -- and the
	 * number of such entries is added here, so that one bad value cannot reach the fp32 master weights unnoticed */
	uint32_t* d_nonfinite;
} neus2b_adam_cfg;
/* Ema o ExponentialDecay o Adam (configs/nerf/dtu.json:5-27) over the flat parameter block.  Gradients: d_grad_mlp fp32
 * for [0, n_matrix), d_grad_grid fp16 for [n_matrix, n - 4), d_grad_variance fp32 for the last 4; all are zeroed after
 * use.  Writes fp32 master, Adam moments, fp16 params, and (if d_params_ema) the EMA copies. */
int neus2b_adam_step(const neus2b_adam_cfg* cfg, uint64_t n, float* d_grad_mlp, uint16_t* d_grad_grid, float* d_grad_variance,
                     float* d_master, float* d_m, float* d_v, uint16_t* d_params, uint16_t* d_params_ema, float* d_ema_master,
                     neus2b_stream_t stream);

/* The same step with the optimizer-private state interleaved per parameter: d_state [n][4] fp32 = {master weight, Adam m,
 * Adam v, EMA master}: one read-modify-write stream instead of four arrays (the training loop keeps separate arrays). */
int neus2b_adam_step_packed(const neus2b_adam_cfg* cfg, uint64_t n, float* d_grad_mlp, uint16_t* d_grad_grid,
                            float* d_grad_variance, float* d_state, uint16_t* d_params, uint16_t* d_params_ema,
                            neus2b_stream_t stream);

/* DeltaNetwork's optimizer (dynamic sequences).  The sums -> the 12 parameters' gradients (transition: R^T sum dL/dx'; rotation: backward of the Gram-Schmidt construction,
 * gradient_rotation_matrix_to_6d, common_operation.cuh:96-158) -> one step of the motion's own optimizer (the "globalmove"
 * block of configs/nerf/base.json:84-110; m_global_move.trainer->optimizer_step, src/testbed_nerf.cu:3500-3502).  d_sums is
 * cleared.  d_grad_out (optional, float[12]) receives the gradients; with d_master == NULL only they are computed. */
int neus2b_delta_optimizer_step(const neus2b_adam_cfg* cfg, float* d_sums, float* d_master, float* d_m, float* d_v, uint16_t* d_delta,
                                uint16_t* d_delta_ema, float* d_ema_master, float* d_grad_out, neus2b_stream_t stream);

/* ---------------------------------------------------------------- training loop (Testbed, src/testbed.cu / src/testbed_nerf.cu) */

/* The subset of configs/nerf/base.json + Testbed members that the NeuS training step reads. */
typedef struct {
	neus2b_grid_desc grid;         /* "encoding" */
	float sdf_bias;                /* "network.sdf_bias" (nerf_network.h:74) */
	uint32_t batch_size;           /* hyperparams.batch_size, default 1<<18 (src/testbed.cu:2110) */
	uint32_t n_cascades;           /* max_cascade + 1; 1 when aabb_scale == 1 (src/testbed_nerf.cu:3084) */
	uint32_t seed;                 /* Testbed::m_seed = 1337 (testbed.h:515) */
	float learning_rate, beta1, beta2, epsilon, l2_reg; /* "optimizer" Adam (configs/nerf/dtu.json:14-19) */
	float ema_decay;               /* Ema decay 0.95 */
	uint32_t lr_decay_start, lr_decay_interval; /* ExponentialDecay 20000 / 10000 */
	float lr_decay_base;           /* 0.33 */
	float ek_loss_weight, mask_loss_weight; /* hyperparams (src/testbed.cu:2125-2126) */
	uint32_t anneal_end;           /* hyperparams.anneal_end (nerf_network.h:1109-1118) */
	float density_grid_decay;      /* 0.95 (testbed.h:635) */
	uint32_t random_bg_color, snap_to_pixel_centers;
	/* progressive level mask: n_active = min(L, start + per_increment * (step / steps_per_increment)); 0 steps = off */
	uint32_t progressive_start_levels, progressive_levels_per_increment, progressive_steps_per_increment;
	uint32_t world_size, rank;     /* ray sharding for data-parallel training (one process per GPU) */
	/* The reference's own keys for the progressive mask ("encoding" block, configs/nerf/base.json:36-38, dtu.json:35-37;
	 * consumed by Encoding::set_training_step, src/testbed.cu:2643-2647, inside the un-vendored tiny-cuda-nn fork).
	 * base_training_step > 0 switches this schedule on (it then takes precedence over the triple above):
	 *   fraction = min(1, base_valid_level_scale + valid_level_scale * (step / base_training_step))   (integer division)
	 *   n_active = clamp(round(n_levels * fraction), 1, n_levels)
	 * The formula is this library's reading of the key names; the fork's source is not available. */
	float valid_level_scale, base_valid_level_scale;
	uint32_t base_training_step;
	uint32_t adam_flags;           /* NEUS2B_ADAM_* */
	float loss_scale;              /* LOSS_SCALE (include/neural-graphics-primitives/testbed.h:237): 128 */
	/* dynamic sequences: "hyperparams" of configs/nerf/base.json:70-82 (src/testbed.cu:2108-2122) and its "globalmove" optimizer
	 * block (:84-110).  They matter from the second frame on (neus2b_testbed_next_frame). */
	uint32_t predict_global_movement;                  /* learn a rigid motion per frame (DeltaNetwork); false */
	uint32_t predict_global_movement_training_step;    /* steps of a frame that train the motion alone; 300 in the code, 100 shipped */
	uint32_t finetune_global_movement;                 /* keep training the motion afterwards; true */
	uint32_t reset_density_grid_after_global_movement; /* true in the code, false shipped */
	float after_learning_rate;                         /* the canonical model's learning rate from the second frame on; 0 = unchanged */
	float gm_learning_rate, gm_beta1, gm_beta2, gm_epsilon, gm_l2_reg, gm_ema_decay;
	uint32_t gm_lr_decay_start, gm_lr_decay_interval;
	float gm_lr_decay_base;
	float first_frame_offset[3];                       /* Testbed::m_first_frame_offset (testbed.h:455): 0 */
	/* no counterpart in the reference: the step's network pass over the generated samples runs in windows of consecutive
	 * samples per ray and skips what lies behind the point where a ray turns opaque (neus2b_forward_compute_loss; same
	 * compacted batch and loss).  Cumulative window ends; n_forward_windows = 0 evaluates every sample like the reference. */
	uint32_t n_forward_windows;
	uint32_t forward_window_ends[6];
} neus2b_testbed_config;
/* "top_resolution" -> per_level_scale when the config gives none (src/testbed.cu:2173-2177):
 * exp(log(top_resolution * aabb_scale / base_resolution) / (n_levels - 1)). */
float neus2b_per_level_scale_from_top_resolution(uint32_t n_levels, uint32_t base_resolution, float top_resolution, uint32_t aabb_scale);
/* Active levels at a training step under the testbed's configured schedule (what the step's kernels are launched with). */
uint32_t neus2b_testbed_config_active_levels(const neus2b_testbed_config* cfg, uint32_t training_step);

typedef struct {
	uint32_t training_step;
	uint32_t rays_per_batch;                       /* Counters::rays_per_batch after the step's re-tune */
	uint32_t n_rays_kept;
	uint32_t measured_batch_size_before_compaction;
	uint32_t measured_batch_size;
	uint32_t overflow;
	float loss, ek_loss;                           /* Testbed.loss / ek_loss (python_api.cu:447-449) */
	uint32_t nonfinite_gradients;                  /* gradient entries the optimizer refused so far (NaN / infinite), cumulative */
	uint32_t device_error;                         /* sticky device error bits at the end of the step (neus2b_device_error_flags) */
	uint32_t n_samples_evaluated;                  /* samples the step's network pass evaluated (== ..._before_compaction without
	                                                  forward windows) */
} neus2b_train_stats;

typedef struct neus2b_testbed neus2b_testbed;

void neus2b_testbed_default_config(neus2b_testbed_config* cfg);
/* Testbed(ETestbedMode::Nerf) + reset_network (src/testbed.cu:2074-2339): allocates parameters, optimizer state,
 * occupancy grid and batch scratch on the current device; all later calls run on an internal stream. */
int neus2b_testbed_create(const neus2b_testbed_config* cfg, neus2b_testbed** out);
void neus2b_testbed_destroy(neus2b_testbed* tb);
/* Testbed::load_training_data (src/testbed.cu:83): HOST arrays, copied to the device. */
int neus2b_testbed_load_training_data(neus2b_testbed* tb, uint32_t n_images, uint32_t width, uint32_t height,
                                      const uint32_t* h_pixels, const float* h_xforms, const float* h_focal,
                                      const float* h_principal);
/* Re-upload the camera block only (NerfDataset::update_transforms). */
int neus2b_testbed_update_cameras(neus2b_testbed* tb, const float* h_xforms, const float* h_focal, const float* h_principal);
/* Trainer::set_params_full_precision (src/testbed.cu:2335) / params_full_precision(): HOST fp32 arrays. */
int neus2b_testbed_set_params(neus2b_testbed* tb, const float* h_params, uint64_t n);
int neus2b_testbed_get_params(neus2b_testbed* tb, float* h_params, uint64_t n, int ema);
int neus2b_testbed_n_params(const neus2b_testbed* tb, uint64_t* n);
/* Testbed::train(batch_size) x n_steps (src/testbed.cu:2630-2726): occupancy update when due, sample generation, fused
 * forward, loss + compaction, fused forward+backward, optimizer step, batch re-tune -- enqueued without any host
 * synchronisation.  If h_stats is non-NULL the stream is synchronised once at the end and the last step's counters
 * and losses are copied back. */
int neus2b_testbed_train(neus2b_testbed* tb, uint32_t n_steps, neus2b_train_stats* h_stats);
/* Device views for tests and for the caller's own streams/collectives (valid until destroy).  A caller that writes the
 * occupancy bitfield asks for the pointer again before the next step: the call marks the box of occupied cells stale. */
int neus2b_testbed_device_ptrs(neus2b_testbed* tb, uint16_t** d_params, uint16_t** d_params_ema, float** d_master,
                               float** d_grad_mlp, uint16_t** d_grad_grid, float** d_grad_variance, uint8_t** d_bitfield,
                               float** d_density_grid, neus2b_stream_t* stream);
/* Split one step for data-parallel training: backward leaves the local gradients in place, the caller all-reduces them
 * (NCCL) on the returned stream, then optimizer_step applies Adam.  neus2b_testbed_train == both halves back to back. */
int neus2b_testbed_train_backward(neus2b_testbed* tb);
int neus2b_testbed_train_optimizer_step(neus2b_testbed* tb, neus2b_train_stats* h_stats);
/* Optional, between the two calls above: runs the pending step's batch tuner and draws the NEXT step's rays and samples
 * already (they depend on the occupancy bits and the ray count, not on the parameters), so that this work overlaps the
 * gradient all-reduce running on another stream (it may also be called after the optimizer step, before the next
 * neus2b_testbed_train_backward).  Returns 1 without doing anything when the next step begins with an
 * occupancy-grid update.  The next neus2b_testbed_train_backward then skips its sample generation; camera updates,
 * state changes and handing out the bitfield's address discard the samples drawn ahead.  Results are those of the
 * plain sequence. */
int neus2b_testbed_train_pregenerate(neus2b_testbed* tb);
/* neus2b_testbed_train_optimizer_step in two halves, for hosts that want the step's statistics every step without
 * leaving the GPU idle while they wait: _async enqueues the optimizer pass, the batch tuner, the loss reduction and the
 * copy of the statistics to the host and returns; the host can then enqueue more work (the next step's camera upload and
 * neus2b_testbed_train_pregenerate, which may also follow the optimizer pass) before _wait_stats blocks on an event
 * behind that copy only, not on the stream. */
int neus2b_testbed_train_optimizer_step_async(neus2b_testbed* tb);
int neus2b_testbed_train_wait_stats(neus2b_testbed* tb, neus2b_train_stats* h_stats);
/* One training step through those halves in one call: backward, optimizer pass and statistics copy enqueued, the NEXT
 * step's cameras uploaded (optional: three host arrays as in neus2b_testbed_update_cameras, or NULLs), the next step's
 * samples drawn, then the wait for this step's statistics (h_stats may be NULL: nothing is waited for). */
int neus2b_testbed_train_step(neus2b_testbed* tb, const float* h_next_xforms, const float* h_next_focal, const float* h_next_principal,
                              neus2b_train_stats* h_stats);
/* Testbed::training_network_next_frame (src/testbed.cu:1991-2072) for a dynamic sequence: the next frame's images and cameras
 * replace the current ones (same count and size; HOST arrays as in neus2b_testbed_load_training_data), the frame's learned
 * motion is folded into the accumulated global movement that moves every ray from now on, the parameters are carried over
 * as their fp16 values (the reference goes through a snapshot without optimizer state), both optimizers start afresh, the
 * canonical learning rate becomes after_learning_rate, the step counter, the ray count and the ray generator's random stream
 * restart, and the motion is reset to the identity.  The following steps train the motion alone for
 * predict_global_movement_training_step steps (the canonical model frozen), then both.  The occupancy grid is rebuilt by the
 * frame's first step. */
int neus2b_testbed_next_frame(neus2b_testbed* tb, const uint32_t* h_pixels, const float* h_xforms, const float* h_focal,
                              const float* h_principal);
/* State of the sequence: frame index, accumulated global movement (rotation [9] row-major, transition [3]) and the current
 * frame's motion parameters (12 floats, fp32 master; identity on the first frame).  Any pointer may be NULL. */
int neus2b_testbed_get_movement(neus2b_testbed* tb, uint32_t* frame, float rotation[9], float transition[3], float delta[12]);
/* Restores what neus2b_testbed_get_movement returned (snapshot["rotation"], ["transition"], ["local_rotation"],
 * ["local_transition"] of the reference's snapshots, nerf_network.h:1169-1261). */
int neus2b_testbed_set_movement(neus2b_testbed* tb, uint32_t frame, const float rotation[9], const float transition[3], const float delta[12]);

/* Times the fused forward+backward kernel inside the step (the reference keeps a moving average of the whole step only,
 * m_training_ms, src/testbed.cu:2707-2721): arms CUDA-event pairs around that launch for the next max_steps steps on
 * the training stream (0 = off).  When h_ms_sum and h_n are given, first returns the sum of the durations recorded
 * since the previous call and their count (synchronises the stream). */
int neus2b_testbed_profile(neus2b_testbed* tb, uint32_t max_steps, float* h_ms_sum, uint32_t* h_n);
/* get_density_on_grid (src/testbed_nerf.cu:4082-4133): SDF on a res[0] x res[1] x res[2] lattice x/res (no half-voxel
 * offset), z range [z0, z1), EMA parameters when use_ema.  d_out float[(z1-z0) * res[1] * res[0]] on the device. */
int neus2b_testbed_sdf_grid(neus2b_testbed* tb, const uint32_t res[3], uint32_t z0, uint32_t z1, int use_ema, float* d_out);

/* ---------------------------------------------------------------- mesh extraction (src/marching_cubes.cu) */

/* marching_cubes_gpu (src/marching_cubes.cu:794-822; kernels gen_vertices :276-329, gen_faces :377-718).  Vertex and
 * triangle numbering is canonical (cell-linear order, edges +x, +y, +z inside a cell) instead of atomicAdd order.
 * d_sdf float[res[2]][res[1]][res[0]] (x fastest); d_tri_table int8[256][16] is the caller's case table (the reference keeps
 * its own next to gen_faces); d_scratch from neus2b_marching_cubes_scratch_bytes.
 * Call once with d_verts == NULL: counts -> d_counts[0] vertices, d_counts[1] indices (device).  Call again with the same
 * d_scratch and buffers of at least those sizes: d_verts float[n][3] (scaled into the aabb like the reference,
 * v * (max-min)/res + min), d_indices uint32[n]. */
int neus2b_marching_cubes_scratch_bytes(const uint32_t res[3], uint64_t* bytes);
int neus2b_marching_cubes(const float aabb_min[3], const float aabb_max[3], const uint32_t res[3], float thresh, const float* d_sdf,
                          const int8_t* d_tri_table, uint64_t* d_scratch, float* d_verts, uint32_t max_verts, uint32_t* d_indices,
                          uint32_t max_indices, uint32_t* d_counts, neus2b_stream_t stream);
/* The same for one z-slab of the lattice, for extraction sharded over GPUs (the reference extracts on one GPU): lattice
 * layers z0 .. z0 + n_layers - 1 of the res grid, d_sdf_slab float[n_layers][res[1]][res[0]] holding only those layers
 * (neus2b_testbed_sdf_grid with z0, z1), scratch sized for {res[0], res[1], n_layers}.  Vertex positions are those of the
 * whole grid; numbering is local to the slab.  d_counts[4] = {vertices, indices, vertices owned by the layers before the
 * slab's last, vertices owned by its first layer}: what the host needs to drop the copies of the seam vertices. */
int neus2b_marching_cubes_slab(const float aabb_min[3], const float aabb_max[3], const uint32_t res[3], uint32_t z0, uint32_t n_layers,
                               float thresh, const float* d_sdf_slab, const int8_t* d_tri_table, uint64_t* d_scratch, float* d_verts,
                               uint32_t max_verts, uint32_t* d_indices, uint32_t max_indices, uint32_t* d_counts,
                               neus2b_stream_t stream);

/* One z-slab with GLOBAL numbering, for extraction sharded over GPUs without a merge on the host (the reference extracts on
 * one GPU, src/marching_cubes.cu:794-822).  A slab that is followed by another (halo = 1) gets n_layers + 1 layers of SDF:
 * with the extra layer it can number the vertices of its last own layer exactly as the next slab numbers them (that slab
 * owns and writes them), so every index it writes is already the vertex's final id once vertex_offset = the number of
 * vertices the slabs before it own.  The last slab passes halo = 0 and owns all its vertices.
 * Pass 1 (d_verts == NULL): d_counts[0] = vertex ids the slab refers to, [1] = indices it writes, [2] = vertices it owns.
 * Between the passes the caller exchanges counts [1] and [2] of all slabs (an all-gather of two numbers per rank) and forms
 * the exclusive prefix sums.  Pass 2: d_verts float[owned][3] and d_indices uint32[counts[1]] are this slab's slices of the
 * whole mesh: concatenated in slab order they equal neus2b_marching_cubes on the undivided lattice bit for bit.
 * Scratch sized for {res[0], res[1], n_layers + halo}. */
int neus2b_marching_cubes_slab_global(const float aabb_min[3], const float aabb_max[3], const uint32_t res[3], uint32_t z0,
                                      uint32_t n_layers, uint32_t halo, float thresh, const float* d_sdf_slab,
                                      const int8_t* d_tri_table, uint64_t* d_scratch, float* d_verts, uint32_t max_verts,
                                      uint32_t* d_indices, uint32_t max_indices, uint32_t vertex_offset, uint32_t* d_counts,
                                      neus2b_stream_t stream);

/* ---------------------------------------------------------------- inference rendering (NerfTracer, Testbed::render_nerf) */

typedef struct {
	uint32_t width, height;
	float focal_length[2];  /* in pixels: Testbed::calc_focal_length (src/testbed.cu:2728) */
	float screen_center[2]; /* Testbed::render_screen_center (src/testbed.cu:2732); 0.5, 0.5 = centred */
	float camera[12];       /* 3x4 camera-to-world, column major (camera_matrix1 of render_nerf) */
	float pixel_offset[2];  /* position inside the pixel: ld_random_pixel_offset(sample_index), random_val.cuh:317-322;
	                           {0.5, 0.5} when snapping to pixel centres */
	uint32_t sample_index;  /* index of the sample per pixel (render_buffer.spp()): seeds the jitter of the first ray parameter */
	float aabb_min[3], aabb_max[3]; /* m_render_aabb, taken equal to the training box m_aabb */
	float cone_angle_constant;
	float min_transmittance; /* Testbed::Nerf::rendering_min_transmittance (testbed.h:686), 0.01 */
	float cos_anneal_ratio;
	uint32_t linear_colors; /* Nerf::Training::linear_colors (testbed.h:612); 0: the network's colours are sRGB, the frame
	                           buffer receives srgb_to_linear of them (shade_kernel_nerf) */
	uint32_t max_steps;     /* samples per ray at most; 0 = 10000 (MARCH_ITER, src/testbed_nerf.cu:68, bounds the reference's
	                           rounds) */
	/* dynamic sequences: accumulated global movement applied to the camera rays (src/testbed_nerf.cu:2286-2296), as in
	 * neus2b_train_cfg */
	uint32_t use_global_movement;
	float rotation[9], transition[3], first_frame_offset[3];
	const uint16_t* d_delta; /* the current frame's learned motion applied to the samples (neus2b_motion::d_delta), or NULL */
} neus2b_render_cfg;

/* Scratch of the renderer; every array is caller-allocated device memory.  max_rays pixels (whole rows, at most 2^20) are
 * handled at once, max_samples (a multiple of 128) samples go through the network at once. */
typedef struct {
	uint32_t max_rays, max_samples;
	float* d_ray_tmp;      /* [max_rays][8] */
	uint64_t* d_scan_tmp;  /* [max_rays + 1024], zero before the first use */
	float* d_state;        /* [max_rays][8] */
	uint32_t* d_hit_list;  /* [max_rays] */
	float* d_coords;       /* [max_samples][7] */
	uint16_t* d_out;       /* [max_samples][16] */
	uint32_t* d_counters;  /* [8] */
	const int32_t* d_occupied_bounds; /* optional int32[6] from neus2b_occupancy_bounds (one-cascade scenes): rays that miss
	                                     the box of occupied cells are not marched */
	uint32_t* d_march_masks;          /* optional [max_rays][64]: the counting pass records which ray parameters became
	                                     samples, so that writing their coordinates needs no second march */
} neus2b_render_workspace;

/* Testbed::render_nerf, ERenderMode::Shade (src/testbed_nerf.cu:2671-2812): NerfTracer::init_rays_from_camera (:2398-2478,
 * pinhole camera; no depth of field, lens distortion, environment map, rolling shutter or slice plane), NerfTracer::trace
 * (:2480-2601) and shade_kernel_nerf (:2147-2180).  Blends one sample per pixel into d_frame float[height][width][4]
 * (linear, alpha premultiplied; the caller clears it like CudaRenderBuffer::clear_frame) and writes d_depth
 * float[height][width].  d_params are the weights to render with (the reference renders with its inference = EMA
 * weights).  Instead of the reference's rounds of at most 8 steps with a blocking read of the live-ray count after
 * each, every ray's whole march is counted first and the samples go through the network in windows of max_samples; the
 * host reads one number per band of max_rays pixels.  h_n_samples (optional) receives the number of samples evaluated. */
int neus2b_render_frame(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, const neus2b_render_cfg* cfg,
                        const uint8_t* d_bitfield, neus2b_render_workspace* ws, float* d_frame, float* d_depth, uint64_t* h_n_samples,
                        neus2b_stream_t stream);
/* CudaRenderBuffer::accumulate, EColorSpace::Linear (src/render_buffer.cu:217-259, 540-560): running mean of the frames,
 * sample_count = frames accumulated so far (0 overwrites).  Buffers are float[n_pixels][4]. */
int neus2b_render_accumulate(uint32_t n_pixels, const float* d_frame, float* d_accumulate, uint32_t sample_count,
                             neus2b_stream_t stream);
/* CudaRenderBuffer::tonemap with the identity curve (src/render_buffer.cu:474-500, 562-577): background (sRGB, with alpha)
 * behind the premultiplied colour, exposure in stops, conversion to sRGB when to_srgb. */
int neus2b_render_tonemap(uint32_t n_pixels, const float* d_accumulate, float exposure, const float background[4], int to_srgb,
                          float* d_out, neus2b_stream_t stream);
/* ld_random_pixel_offset (include/neural-graphics-primitives/random_val.cuh:317-322): where inside its pixel the spp-th
 * sample of every pixel lies (Owen-scrambled Sobol point, Burley 2020); host computation. */
void neus2b_ld_random_pixel_offset(uint32_t spp, float out_xy[2]);

typedef struct {
	uint32_t width, height, spp;
	float camera[12];               /* Testbed::m_camera: 3x4 camera-to-world, column major */
	float relative_focal_length[2]; /* Testbed::m_relative_focal_length (set_fov: 0.5 / tan(fov / 2)) */
	uint32_t fov_axis;              /* Testbed::m_fov_axis, 1 */
	float zoom;                     /* Testbed::m_zoom, 1 */
	float screen_center[2];         /* Testbed::m_screen_center, 0.5 0.5 */
	uint32_t snap_to_pixel_centers; /* Testbed::m_snap_to_pixel_centers */
	float exposure;                 /* Testbed::m_exposure, stops */
	float background_color[4];      /* Testbed::m_background_color, sRGB + alpha; 0 0 0 1 */
	uint32_t linear;                /* the `linear` argument of Testbed::render: 1 = linear output, 0 = sRGB */
	float min_transmittance;        /* Testbed::Nerf::rendering_min_transmittance, 0.01 */
	uint32_t use_ema;               /* 1: the EMA (inference) weights, like the reference; 0: the training weights */
} neus2b_render_request;
/* Testbed::render_to_cpu for a fixed camera (src/python_api.cu:123-169 -> Testbed::render_frame src/testbed.cu:2810-2826):
 * spp frames, each cleared, rendered, accumulated; then tone mapping; h_rgba float[height][width][4] on the host,
 * h_depth float[height][width] (optional, of the last frame). */
int neus2b_testbed_render(neus2b_testbed* tb, const neus2b_render_request* req, float* h_rgba, float* h_depth);
/* Of the last neus2b_testbed_render call: samples that went through the network (all spp frames) and the time on the
 * device from the first clear to the end of tone mapping (the copy to the host not included). */
int neus2b_testbed_render_stats(const neus2b_testbed* tb, uint64_t* n_samples, float* device_ms);

/* ---------------------------------------------------------------- mesh post-processing and export */

/* compute_mesh_1ring (src/marching_cubes.cu:331-375, 720-735): per vertex the homogeneous sum of its 1-ring neighbours
 * d_ring float[n_verts][4] (xyz sum, count; optional) and the area-weighted normal d_normals float[n_verts][3] (not
 * normalised; optional).  Both are zeroed first. */
int neus2b_mesh_1ring(uint32_t n_verts, const float* d_verts, uint32_t n_indices, const uint32_t* d_indices, float* d_ring,
                      float* d_normals, neus2b_stream_t stream);
/* Testbed::compute_mesh_vertex_colors (src/testbed_nerf.cu:4057-4080): the network's colour at every vertex, seen from the
 * direction that points away from the centre of the unit cube; logistic activation, then linear_to_srgb when
 * linear_colors (extract_srgb_with_activation, :522-535).  d_colors float[n_verts][3].  Scratch: d_coords_scratch
 * float[scratch_samples][7], d_out_scratch fp16 [scratch_samples][16], scratch_samples >= 128 vertices per network call. */
int neus2b_mesh_vertex_colors(const neus2b_grid_desc* desc, const uint16_t* d_params, float sdf_bias, uint32_t n_verts,
                              const float* d_verts, const float aabb_min[3], const float aabb_max[3], int linear_colors,
                              float* d_coords_scratch, uint16_t* d_out_scratch, uint32_t scratch_samples, float* d_colors,
                              neus2b_stream_t stream);
/* save_mesh without texture unwrap (src/marching_cubes.cu:824-976): HOST arrays in, Wavefront OBJ (or ASCII PLY when the
 * path ends in ".ply") out, the same text as the reference's writer: positions (v - nerf_offset) / nerf_scale, unit
 * normals, colours clamped to [0, 1] (OBJ) or bytes (PLY), triangles reversed unless invert_normals
 * (dataset.from_na, src/testbed.cu:305).  The lines are formatted by all host threads. */
int neus2b_save_mesh(const char* path, uint32_t n_verts, const float* h_verts, const float* h_normals, const float* h_colors,
                     uint32_t n_indices, const uint32_t* h_indices, float nerf_scale, const float nerf_offset[3], int invert_normals);

/* ---------------------------------------------------------------- state for snapshots (Testbed::save_snapshot / load_snapshot,
 * src/testbed.cu:3134-3244: Trainer::serialize + density grid + counters) */

typedef struct {
	uint32_t training_step;          /* snapshot["training_step"] */
	uint32_t density_grid_ema_step;  /* Nerf::density_grid_ema_step */
	uint32_t rays_per_batch, measured_batch_size, measured_batch_size_before_compaction; /* snapshot["nerf"]["rgb"] */
	uint32_t n_rays_total;           /* Counters::n_rays_total */
	float loss, ek_loss;             /* snapshot["loss"] */
	neus2b_pcg32 rng, density_rng;   /* m_rng, m_nerf.density_grid_rng */
} neus2b_training_state;
int neus2b_testbed_get_training_state(neus2b_testbed* tb, neus2b_training_state* out);
int neus2b_testbed_set_training_state(neus2b_testbed* tb, const neus2b_training_state* in);
/* The arrays a snapshot holds, copied to / from HOST memory; `bytes` must be the array's size.  Trainer::serialize stores
 * the fp16 parameters and, with include_optimizer_state, the optimizer's arrays; load_snapshot converts the stored fp16
 * density grid back to fp32 and rebuilds mean and bitfield, which setting NEUS2B_ARRAY_DENSITY_GRID does here too. */
#define NEUS2B_ARRAY_MASTER 0       /* float[n_params]  Trainer::params_full_precision */
#define NEUS2B_ARRAY_ADAM_M 1       /* float[n_params] */
#define NEUS2B_ARRAY_ADAM_V 2       /* float[n_params] */
#define NEUS2B_ARRAY_EMA_MASTER 3   /* float[n_params] */
#define NEUS2B_ARRAY_PARAMS 4       /* fp16[n_params]   Trainer::params */
#define NEUS2B_ARRAY_PARAMS_EMA 5   /* fp16[n_params]   Trainer::params_inference */
#define NEUS2B_ARRAY_DENSITY_GRID 6 /* float[128^3 * n_cascades] */
int neus2b_testbed_get_array(neus2b_testbed* tb, int which, void* h_out, uint64_t bytes);
int neus2b_testbed_set_array(neus2b_testbed* tb, int which, const void* h_in, uint64_t bytes);

#ifdef __cplusplus
}
#endif
#endif
