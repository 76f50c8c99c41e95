/*
 * CPU oracle for the NeuS2 training step.  TEST INFRASTRUCTURE ONLY: it is the checker that the
 * CUDA path is compared against and the timed CPU baseline; nothing in the product links it.
 *
 * Parity status: "parity unpinned" for the arithmetic inside the hash-grid encoding, the fused MLPs, the SH
 * encoding and Adam/EMA, because the reference keeps it in an un-vendored submodule (dependencies/neus2_tcnn,
 * empty; pin unknown).  Those parts restate the published algorithms (multiresolution hash encoding, dense ReLU
 * MLP, real spherical harmonics, Adam) and are anchored on the reference's call sites.  Pinned: the ray-march,
 * NeuS compositing, loss, occupancy-grid, tracer, marching-cubes and mesh parts follow reference source that is
 * present (src/testbed_nerf.cu, src/marching_cubes.cu, include/neural-graphics-primitives/nerf_network.h), cite it
 * per function, and the CUDA path that is checked against this oracle is also run against the reference's own
 * kernels and host code on the GPU (oracle/ref_kernels, tests/test_gpu_reference_*.py); PCG32 is checked against
 * its published known answer, its seeding against the reference's training loop.
 *
 * All matrices are "AoS": one sample's values are contiguous ([n][width]).  fp16 values travel as
 * uint16_t bit patterns.  Every rounding to fp16 that the reference's data flow implies is explicit.
 */
#ifndef NEUS2_ORACLE_H
#define NEUS2_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define N2O_MAX_LEVELS 16
#define N2O_GRIDSIZE 128u   /* NERF_GRIDSIZE, include/neural-graphics-primitives/nerf.h:24 */
#define N2O_CASCADES 8u     /* NERF_CASCADES, src/testbed_nerf.cu:49 */
#define N2O_STEPS 1024u     /* NERF_STEPS,    src/testbed_nerf.cu:48 */

/* Hash-grid geometry.  Level rule scale_l = base*b^l - 1, res_l = ceil(scale_l)+1 is the one the
 * reference itself uses to report the top resolution (src/testbed.cu:2177). */
typedef struct {
	uint32_t n_levels;           /* L <= 16 */
	uint32_t log2_hashmap_size;  /* T = 1 << this */
	uint32_t base_resolution;
	float per_level_scale;
	uint32_t n_active_levels;    /* progressive mask: levels >= this output 0 and get no gradient */
} n2o_grid_desc;

typedef struct {
	uint32_t offset[N2O_MAX_LEVELS + 1]; /* in grid entries (each entry = 2 fp16 features) */
	uint32_t res[N2O_MAX_LEVELS];
	uint32_t hashed[N2O_MAX_LEVELS];
	float scale[N2O_MAX_LEVELS];
} n2o_grid_levels;

/* Parameter block layout (include/neural-graphics-primitives/nerf_network.h:728-772):
 * SDF MLP (64x48 + 16x64) | colour MLP (64x48 + 64x64 + 16x64) | grid | variance (4). */
#define N2O_SDF_W1 0
#define N2O_SDF_W2 (64 * 48)
#define N2O_SDF_N (64 * 48 + 16 * 64)
#define N2O_RGB_W1 N2O_SDF_N
#define N2O_RGB_W2 (N2O_RGB_W1 + 64 * 48)
#define N2O_RGB_W3 (N2O_RGB_W2 + 64 * 64)
#define N2O_MLP_N (N2O_RGB_W3 + 16 * 64)
#define N2O_GRID_OFF N2O_MLP_N

void n2o_set_num_threads(int n); /* OpenMP threads used by every entry point below */

void n2o_grid_make_levels(const n2o_grid_desc* d, n2o_grid_levels* out);
uint32_t n2o_grid_n_params(const n2o_grid_desc* d);  /* fp16 scalars */
uint32_t n2o_model_n_params(const n2o_grid_desc* d); /* whole block incl. 4 variance slots */

/* --- component level (mirrors tcnn Encoding / Network entry points the reference calls) --- */
void n2o_grid_forward(const n2o_grid_desc* d, uint32_t n, const float* x, uint32_t x_stride,
                      const uint16_t* grid, uint16_t* enc /*[n][2L]*/, float* dy_dx /*[n][2L][3] or NULL*/);
void n2o_grid_backward_input(const n2o_grid_desc* d, uint32_t n, const float* x, uint32_t x_stride,
                             const uint16_t* grid, const uint16_t* dL_denc, float* dL_dx /*[n][3]*/);
void n2o_grid_backward_params(const n2o_grid_desc* d, uint32_t n, const float* x, uint32_t x_stride,
                              const uint16_t* dL_denc, double* grad /*[grid_n_params], accumulates*/);
void n2o_grid_backward_backward_input(const n2o_grid_desc* d, uint32_t n, const float* x, uint32_t x_stride,
                                      const uint16_t* grid, const float* v /*[n][3]*/, const uint16_t* g_e /*[n][2L]*/,
                                      double* grad /*accumulates*/, uint16_t* dy_enc /*[n][2L]*/);
/* ReLU MLP in -> 64 (x n_hidden) -> 16, weights fp16 row-major [out][in], layer after layer. */
void n2o_mlp_forward(uint32_t n, uint32_t in_w, uint32_t n_hidden, const uint16_t* w,
                     const uint16_t* in, uint16_t* out /*[n][16]*/, uint16_t* hidden /*[n][n_hidden][64] or NULL*/);
void n2o_mlp_backward(uint32_t n, uint32_t in_w, uint32_t n_hidden, const uint16_t* w, const uint16_t* in,
                      const uint16_t* hidden, const uint16_t* dL_dout, uint16_t* dL_din /*or NULL*/, double* wgrad /*or NULL, accumulates*/);
/* Second-order pass of the one-hidden-layer SDF net (nerf_network.h:560-571): u = dL/d(dy/dz), dy = dL_dout of the
 * first-order pass whose input gradient is being differentiated. */
void n2o_mlp_backward_backward_input(uint32_t n, uint32_t in_w, const uint16_t* w, const uint16_t* hidden,
                                     const uint16_t* u, const uint16_t* dy, double* wgrad);
void n2o_sh4(uint32_t n, const float* dir01, uint32_t stride, uint16_t* out /*[n][16]*/);

/* --- whole NeuS graph (nerf_network.h:132-315 forward, :317-641 backward), static scene --- */
void n2o_neus_forward(const n2o_grid_desc* d, const uint16_t* params, float sdf_bias, uint32_t n,
                      const float* coords /*[n][7]*/, uint16_t* out /*[n][16]*/);
void n2o_neus_backward(const n2o_grid_desc* d, const uint16_t* params, uint32_t n, const float* coords,
                       const uint16_t* dL_dout /*[n][16]*/, uint32_t indeed_batch_size,
                       double* grad /*[model_n_params], accumulates; loss-scaled like dL_dout*/);
/* The same, and the gradient that reaches the sample positions, dL_dx [n][3] (may be NULL): what NerfNetwork::backward_impl
 * hands to the DeltaNetwork (nerf_network.h:589-612) = dL/dx of the encoding's first-order backward + the xyz rows of the
 * colour-net and SDF-net input gradients.  (The second-order term's dL/dx is computed by the reference but never used.) */
void n2o_neus_backward_dx(const n2o_grid_desc* d, const uint16_t* params, uint32_t n, const float* coords,
                          const uint16_t* dL_dout, uint32_t indeed_batch_size, double* grad, float* dL_dx);
/* NerfNetwork::sdf / density (nerf_network.h:643-726) */
void n2o_neus_sdf(const n2o_grid_desc* d, const uint16_t* params, float sdf_bias, uint32_t n, const float* x,
                  uint32_t x_stride, uint16_t* sdf);

/* --- DeltaNetwork: the learned rigid motion of the current frame (include/neural-graphics-primitives/transform_network.h:26-170,
 * kernels common_operation.cuh:42-170, 419-474, 793-849).  delta = 12 fp16 parameters in the network's own order
 * (set_params :183-205): transition [0..3] (xyz + one unused), 6-D rotation [4..11] (a1, a2 + two unused). --- */
void n2o_rotation_6d_to_matrix(const uint16_t* rot6 /*fp16[6]*/, float* R /*[9] row-major*/);
/* add_global_movement_with_rotation_6d: pos' = R (pos + t - off) + off, dir' = (R (2 dir - 1) + 1) / 2; coords [n][7], dt copied */
void n2o_delta_forward(const uint16_t* delta, const float* first_frame_offset, uint32_t n, const float* coords_in, float* coords_out);
/* add_loss_to_rotation_6d_each + the nine batch sums of DeltaNetwork::backward_impl: dL_dx [n][3] = gradient w.r.t. the moved
 * position; grad [12] (+=): transition at [0..2], 6-D rotation at [4..9].  fp32 per sample, fp64 sums (the reference rounds
 * every per-sample value to fp16 before it sums). */
void n2o_delta_backward(const uint16_t* delta, const float* first_frame_offset, uint32_t n, const float* coords_in, const float* dL_dx,
                        double* grad);
/* accumulate_global_movement_rotation_6d_kernel (common_operation.cuh:555-589): R_acc <- R R_acc, t_acc <- R (t_acc + t); both
 * arrays hold fp16-representable values (the reference keeps them in fp16 buffers) */
void n2o_accumulate_global_movement(const uint16_t* delta, float* acc_rotation /*[9]*/, float* acc_transition /*[3]*/);

/* --- ray march / loss (src/testbed_nerf.cu) --- */
typedef struct {
	uint64_t state, inc;
} n2o_pcg32;
void n2o_pcg32_seed(n2o_pcg32* r, uint64_t seed);
void n2o_pcg32_advance(n2o_pcg32* r, uint64_t delta);
uint32_t n2o_pcg32_next_uint(n2o_pcg32* r);
float n2o_pcg32_next_float(n2o_pcg32* r);

typedef struct {
	uint32_t n_images, width, height;
	const uint32_t* pixels;  /* [n_images][height][width] RGBA8, R in the low byte */
	const float* xforms;     /* [n_images][12]: 3x4 camera-to-world, column major (Eigen layout) */
	const float* focal;      /* [n_images][2] */
	const float* principal;  /* [n_images][2] */
} n2o_dataset;

typedef struct {
	float aabb_min[3], aabb_max[3];
	float cone_angle_constant;
	uint32_t snap_to_pixel_centers;
	uint32_t random_bg_color;
	float background_color[3];
	float loss_scale;        /* LOSS_SCALE = 128, include/neural-graphics-primitives/testbed.h:237 */
	float mask_loss_weight, ek_loss_weight, cos_anneal_ratio;
	uint32_t ray_index_offset, ray_count_scale; /* data-parallel ray sharding; 0 / 1 = single process */
	/* accumulated global movement of the earlier frames of a dynamic sequence, applied to every ray before the march
	 * (global_movement_with_rotation_6d, src/testbed_nerf.cu:183-203, call sites :1370-1378, :1550-1558, :2286-2296):
	 * o = R (o - first_frame_offset) + t, dir = R dir (dir normalised before, not after).  R row-major. */
	uint32_t use_global_movement;
	float rotation[9], transition[3], first_frame_offset[3];
} n2o_train_cfg;

/* generate_training_samples_nerf_with_global_movement (src/testbed_nerf.cu:1253-1446), static scene, canonical
 * (ray-index) ordering instead of atomicAdd ordering.  Returns n_rays kept; writes *n_samples. */
uint32_t n2o_generate_samples(const n2o_dataset* ds, const n2o_train_cfg* cfg, uint32_t n_rays, uint32_t n_rays_total,
                              uint32_t max_samples, n2o_pcg32 rng, const uint8_t* bitfield, uint32_t* ray_indices,
                              float* rays /*[n][6] o,d unnormalised*/, uint32_t* numsteps /*[n][2]*/,
                              float* coords /*[max_samples][7]*/, uint32_t* n_samples);
/* compute_loss_kernel_train_nerf_with_global_movement (src/testbed_nerf.cu:1465-1996), canonical compaction order.
 * Returns the compacted sample count (before clipping to max_compacted). */
uint32_t n2o_compute_loss(const n2o_dataset* ds, const n2o_train_cfg* cfg, uint32_t n_rays_kept, uint32_t n_rays,
                          uint32_t n_rays_total, n2o_pcg32 rng, uint32_t max_compacted, const uint16_t* mlp_out,
                          const uint32_t* ray_indices, const float* rays, uint32_t* numsteps, const float* coords,
                          float* coords_out, uint16_t* dloss_dout, float* loss_out, float* ek_loss_out);
/* fill_rollover / fill_rollover_and_rescale (call sites src/testbed_nerf.cu:3908-3916) */
void n2o_fill_rollover(uint32_t n_target, uint32_t width, uint32_t n_valid, float* data);
void n2o_fill_rollover_and_rescale_half(uint32_t n_target, uint32_t width, uint32_t n_valid, uint16_t* data);

/* --- inference rendering (src/testbed_nerf.cu:787-1171, 2147-2332, 2398-2601, 2671-2812; src/render_buffer.cu) --- */
typedef struct {
	uint32_t width, height;
	float focal_length[2], screen_center[2];
	float camera[12];      /* 3x4 camera-to-world, column major */
	float pixel_offset[2]; /* ld_random_pixel_offset(sample_index) */
	uint32_t sample_index;
	float aabb_min[3], aabb_max[3];
	float cone_angle_constant, min_transmittance, cos_anneal_ratio;
	uint32_t linear_colors;
	uint32_t max_steps;    /* 0 = 10000 */
} n2o_render_cfg;
float n2o_ld_random_val(uint32_t index, uint32_t seed); /* random_val.cuh:284-288, dimension 0 */
void n2o_render_march(const n2o_render_cfg* rc, const uint8_t* bitfield, uint64_t max_samples, uint32_t* numsteps /*[h*w]*/,
                      float* coords /*[max_samples][7] or NULL*/, uint64_t* n_samples);
void n2o_render_frame(const n2o_grid_desc* d, const uint16_t* params, float sdf_bias, const n2o_render_cfg* rc, const uint8_t* bitfield,
                      float* frame /*[h][w][4], blended into*/, float* depth /*[h][w]*/, uint64_t* n_samples);
void n2o_render_accumulate(uint32_t n_pixels, const float* frame, float* acc, uint32_t sample_count);
void n2o_render_tonemap(uint32_t n_pixels, const float* acc, float exposure, const float* background /*[4] sRGB*/, int to_srgb,
                        float* out);

/* --- occupancy grid (src/testbed_nerf.cu:630-785, 3287-3391) --- */
uint32_t n2o_morton3d(uint32_t x, uint32_t y, uint32_t z);
uint32_t n2o_morton3d_invert(uint32_t x);
void n2o_occ_generate_samples(uint32_t n, n2o_pcg32 rng, uint32_t step, const float* aabb_min, const float* aabb_max,
                              const float* grid_in, uint32_t n_cascades, float thresh, float* pos /*[n][3]*/, uint32_t* indices);
/* density = s*sigma(s*sdf)*(1-sigma) evaluated in fp16 (common_operation.cuh:310-328) */
void n2o_sdf_to_density(uint32_t n, uint16_t variance, uint16_t* sdf_inout);
void n2o_occ_splat_ema(uint32_t n_samples, const uint32_t* indices, const uint16_t* density, uint32_t n_cells,
                       float decay, float* grid_tmp, float* grid);
void n2o_occ_bitfield(uint32_t n_cascades_used, const float* grid, uint8_t* bitfield, float* mean_out);

/* --- optimizer: Ema o ExponentialDecay o Adam (config configs/nerf/dtu.json:5-27) --- */
typedef struct {
	float learning_rate, beta1, beta2, epsilon, l2_reg, ema_decay, loss_scale;
	uint32_t step;     /* 1-based step being applied */
	uint32_t n_matrix; /* leading MLP-weight entries: L2 applies to them only; other entries with a zero gradient are skipped */
} n2o_adam_cfg;
void n2o_adam_step(const n2o_adam_cfg* c, uint32_t n, const float* grad /*loss-scaled*/, float* master, float* m, float* v,
                   uint16_t* params, uint16_t* params_ema /*or NULL*/, float* ema_master /* or NULL */);

/* --- marching cubes (src/marching_cubes.cu:276-329, 377-718), canonical cell-linear order. tri_table = the 256x16
 * case table, supplied by the caller. Returns counts via pointers; pass NULL outputs to count only. */
void n2o_marching_cubes_slab(const float* aabb_min, const float* aabb_max, const uint32_t res[3], uint32_t z0, uint32_t nz, float thresh,
                             const float* sdf, const int8_t* tri_table, float* verts, uint32_t* indices, uint32_t* counts);
void n2o_marching_cubes(const float* aabb_min, const float* aabb_max, const uint32_t res[3], float thresh, const float* sdf,
                        const int8_t* tri_table, float* verts, uint32_t* indices, uint32_t* n_verts, uint32_t* n_indices);

/* --- mesh post-processing and export (src/marching_cubes.cu:331-375, 824-976; src/testbed_nerf.cu:4057-4080) --- */
void n2o_mesh_1ring(uint32_t n_verts, const float* verts, uint32_t n_indices, const uint32_t* indices, float* ring /*[n][4] or NULL*/,
                    float* normals /*[n][3] or NULL*/);
void n2o_mesh_vertex_colors(const n2o_grid_desc* d, const uint16_t* params, float sdf_bias, uint32_t n_verts, const float* verts,
                            const float* aabb_min, const float* aabb_max, int linear_colors, float* colors /*[n][3]*/);
int n2o_save_mesh(const char* path, uint32_t n_verts, const float* verts, const float* normals, const float* colors, uint32_t n_indices,
                  const uint32_t* indices, float nerf_scale, const float* nerf_offset, int invert_normals);

#ifdef __cplusplus
}
#endif
#endif
