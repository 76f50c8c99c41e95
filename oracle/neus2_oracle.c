/*
 * CPU oracle for the NeuS2 training step -- see neus2_oracle.h for scope and parity status.
 * TEST INFRASTRUCTURE ONLY (checker + timed CPU baseline).  Scalar C with OpenMP over samples/rays.
 */
#include "neus2_oracle.h"

#include <math.h>
#include <omp.h>
#include <stdlib.h>
#include <stdio.h>
#include <string.h>

void n2o_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }

/* ------------------------------------------------------------------ fp16 helpers */
static inline float h2f(uint16_t h) {
	_Float16 x;
	memcpy(&x, &h, 2);
	return (float)x;
}
static inline uint16_t f2h(float f) {
	_Float16 x = (_Float16)f;
	uint16_t h;
	memcpy(&h, &x, 2);
	return h;
}
static inline float rh(float f) { return (float)(_Float16)f; }
static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }
static inline float logisticf(float x) { return 1.0f / (1.0f + expf(-x)); }

/* ------------------------------------------------------------------ hash grid */
void n2o_grid_make_levels(const n2o_grid_desc* d, n2o_grid_levels* out) {
	uint32_t T = 1u << d->log2_hashmap_size;
	uint32_t off = 0;
	memset(out, 0, sizeof(*out));
	for (uint32_t l = 0; l < d->n_levels; ++l) {
		float scale = exp2f((float)l * log2f(d->per_level_scale)) * (float)d->base_resolution - 1.0f;
		uint32_t res = (uint32_t)ceilf(scale) + 1u;
		uint64_t dense = (uint64_t)res * res * res;
		uint32_t n;
		if (dense > (uint64_t)T) {
			out->hashed[l] = 1;
			n = T;
		} else {
			out->hashed[l] = 0;
			n = (uint32_t)((dense + 7u) / 8u * 8u);
		}
		out->scale[l] = scale;
		out->res[l] = res;
		out->offset[l] = off;
		off += n;
	}
	out->offset[d->n_levels] = off;
}

uint32_t n2o_grid_n_params(const n2o_grid_desc* d) {
	n2o_grid_levels lv;
	n2o_grid_make_levels(d, &lv);
	return lv.offset[d->n_levels] * 2u;
}

uint32_t n2o_model_n_params(const n2o_grid_desc* d) { return N2O_MLP_N + n2o_grid_n_params(d) + 4u; }

typedef struct {
	uint32_t idx[8]; /* entry index inside the whole grid (level offset included) */
	float w[8];
	float dw[8][3]; /* d w / d x, level scale included */
} corners_t;

static inline void level_corners(const n2o_grid_levels* lv, uint32_t l, const float* x, corners_t* c) {
	const float scale = lv->scale[l];
	const uint32_t res = lv->res[l];
	const uint32_t n = lv->offset[l + 1] - lv->offset[l];
	float f[3];
	uint32_t c0[3];
	for (int d = 0; d < 3; ++d) {
		float pos = fmaf(x[d], scale, 0.5f);
		float fl = floorf(pos);
		f[d] = pos - fl;
		c0[d] = (uint32_t)(int32_t)fl;
	}
	for (uint32_t k = 0; k < 8; ++k) {
		uint32_t cc[3];
		float wd[3];
		for (int d = 0; d < 3; ++d) {
			uint32_t bit = (k >> d) & 1u;
			cc[d] = c0[d] + bit;
			wd[d] = bit ? f[d] : 1.0f - f[d];
		}
		uint32_t idx;
		if (lv->hashed[l]) {
			idx = (cc[0] * 1u) ^ (cc[1] * 2654435761u) ^ (cc[2] * 805459861u);
			idx %= n;
		} else {
			/* dense level: the cell is clamped to the lattice (no change inside the unit cube, where the far face is cell
			 * res - 1 with its upper corner at res; samples outside the cube read the edge cells), then the plain lattice
			 * index, which wraps once for a corner on the far face (assumption A1) */
			int32_t cl[3];
			for (int d = 0; d < 3; ++d) {
				int32_t v = (int32_t)c0[d];
				cl[d] = v < 0 ? 0 : (v > (int32_t)res - 1 ? (int32_t)res - 1 : v);
			}
			idx = ((uint32_t)cl[0] + (k & 1u)) + ((uint32_t)cl[1] + ((k >> 1) & 1u)) * res + ((uint32_t)cl[2] + ((k >> 2) & 1u)) * res * res;
			idx %= n;
		}
		c->idx[k] = lv->offset[l] + idx;
		c->w[k] = wd[0] * wd[1] * wd[2];
		c->dw[k][0] = ((k & 1u) ? scale : -scale) * wd[1] * wd[2];
		c->dw[k][1] = ((k & 2u) ? scale : -scale) * wd[0] * wd[2];
		c->dw[k][2] = ((k & 4u) ? scale : -scale) * wd[0] * wd[1];
	}
}

/* One sample: features (rounded to fp16, held as float) and optionally J = d enc / d x. */
static void grid_sample_forward(const n2o_grid_desc* d, const n2o_grid_levels* lv, const uint16_t* grid, const float* x,
                                float* enc, float (*J)[3]) {
	for (uint32_t l = 0; l < d->n_levels; ++l) {
		if (l >= d->n_active_levels) {
			enc[2 * l] = enc[2 * l + 1] = 0.f;
			if (J) memset(J[2 * l], 0, sizeof(float) * 6);
			continue;
		}
		corners_t c;
		level_corners(lv, l, x, &c);
		float a0 = 0.f, a1 = 0.f, j0[3] = {0, 0, 0}, j1[3] = {0, 0, 0};
		for (int k = 0; k < 8; ++k) {
			float t0 = h2f(grid[2 * (size_t)c.idx[k]]), t1 = h2f(grid[2 * (size_t)c.idx[k] + 1]);
			a0 = fmaf(c.w[k], t0, a0);
			a1 = fmaf(c.w[k], t1, a1);
			for (int e = 0; e < 3; ++e) {
				j0[e] = fmaf(c.dw[k][e], t0, j0[e]);
				j1[e] = fmaf(c.dw[k][e], t1, j1[e]);
			}
		}
		enc[2 * l] = rh(a0);
		enc[2 * l + 1] = rh(a1);
		if (J) {
			for (int e = 0; e < 3; ++e) {
				J[2 * l][e] = j0[e];
				J[2 * l + 1][e] = j1[e];
			}
		}
	}
}

void n2o_grid_forward(const n2o_grid_desc* d, uint32_t n, const float* x, uint32_t x_stride, const uint16_t* grid,
                      uint16_t* enc, float* dy_dx) {
	n2o_grid_levels lv;
	n2o_grid_make_levels(d, &lv);
	const uint32_t W = 2 * d->n_levels;
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		float e[32], J[32][3];
		grid_sample_forward(d, &lv, grid, x + (size_t)i * x_stride, e, J);
		for (uint32_t k = 0; k < W; ++k) enc[(size_t)i * W + k] = f2h(e[k]);
		if (dy_dx) memcpy(dy_dx + (size_t)i * W * 3, J, sizeof(float) * W * 3);
	}
}

void n2o_grid_backward_input(const n2o_grid_desc* d, uint32_t n, const float* x, uint32_t x_stride, const uint16_t* grid,
                             const uint16_t* dL_denc, float* dL_dx) {
	n2o_grid_levels lv;
	n2o_grid_make_levels(d, &lv);
	const uint32_t W = 2 * d->n_levels;
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		float e[32], J[32][3], g[3] = {0, 0, 0};
		grid_sample_forward(d, &lv, grid, x + (size_t)i * x_stride, e, J);
		for (uint32_t k = 0; k < W; ++k) {
			float dy = h2f(dL_denc[(size_t)i * W + k]);
			for (int e2 = 0; e2 < 3; ++e2) g[e2] = fmaf(J[k][e2], dy, g[e2]);
		}
		memcpy(dL_dx + (size_t)i * 3, g, sizeof(g));
	}
}

static inline void atomic_add_d(double* p, double v) {
#pragma omp atomic
	*p += v;
}

void n2o_grid_backward_params(const n2o_grid_desc* d, uint32_t n, const float* x, uint32_t x_stride, const uint16_t* dL_denc,
                              double* grad) {
	n2o_grid_levels lv;
	n2o_grid_make_levels(d, &lv);
	const uint32_t W = 2 * d->n_levels;
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		for (uint32_t l = 0; l < d->n_levels && l < d->n_active_levels; ++l) {
			corners_t c;
			level_corners(&lv, l, x + (size_t)i * x_stride, &c);
			float g0 = h2f(dL_denc[(size_t)i * W + 2 * l]), g1 = h2f(dL_denc[(size_t)i * W + 2 * l + 1]);
			for (int k = 0; k < 8; ++k) {
				atomic_add_d(&grad[2 * (size_t)c.idx[k]], (double)(c.w[k] * g0));
				atomic_add_d(&grad[2 * (size_t)c.idx[k] + 1], (double)(c.w[k] * g1));
			}
		}
	}
}

/* One sample of the second-order pass: coef_k = grad_x(w_k) . v ;  grad[k,f] += coef_k * g_e[l,f] ;
 * dy_enc[l,f] = sum_k coef_k * theta[k,f]  (nerf_network.h:534-544, derivation from the argument roles). */
static void grid_sample_bwd_bwd(const n2o_grid_desc* d, const n2o_grid_levels* lv, const uint16_t* grid, const float* x,
                                const float* v, const float* ge, double* grad, float* dy_enc) {
	for (uint32_t l = 0; l < d->n_levels; ++l) {
		if (l >= d->n_active_levels) {
			dy_enc[2 * l] = dy_enc[2 * l + 1] = 0.f;
			continue;
		}
		corners_t c;
		level_corners(lv, l, x, &c);
		float a0 = 0.f, a1 = 0.f;
		for (int k = 0; k < 8; ++k) {
			float coef = c.dw[k][0] * v[0] + c.dw[k][1] * v[1] + c.dw[k][2] * v[2];
			float t0 = h2f(grid[2 * (size_t)c.idx[k]]), t1 = h2f(grid[2 * (size_t)c.idx[k] + 1]);
			a0 = fmaf(coef, t0, a0);
			a1 = fmaf(coef, t1, a1);
			if (grad) {
				atomic_add_d(&grad[2 * (size_t)c.idx[k]], (double)(coef * ge[2 * l]));
				atomic_add_d(&grad[2 * (size_t)c.idx[k] + 1], (double)(coef * ge[2 * l + 1]));
			}
		}
		dy_enc[2 * l] = rh(a0);
		dy_enc[2 * l + 1] = rh(a1);
	}
}

void n2o_grid_backward_backward_input(const n2o_grid_desc* d, uint32_t n, const float* x, uint32_t x_stride,
                                      const uint16_t* grid, const float* v, const uint16_t* g_e, double* grad,
                                      uint16_t* dy_enc) {
	n2o_grid_levels lv;
	n2o_grid_make_levels(d, &lv);
	const uint32_t W = 2 * d->n_levels;
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		float ge[32], dy[32];
		for (uint32_t k = 0; k < W; ++k) ge[k] = h2f(g_e[(size_t)i * W + k]);
		grid_sample_bwd_bwd(d, &lv, grid, x + (size_t)i * x_stride, v + (size_t)i * 3, ge, grad, dy);
		if (dy_enc)
			for (uint32_t k = 0; k < W; ++k) dy_enc[(size_t)i * W + k] = f2h(dy[k]);
	}
}

/* ------------------------------------------------------------------ dense ReLU MLP */
static void to_float(const uint16_t* src, float* dst, size_t n) {
	for (size_t i = 0; i < n; ++i) dst[i] = h2f(src[i]);
}
/* y[o] = sum_k W[o][k] z[k], fp32 accumulation */
static inline void matvec(const float* W, int n_out, int n_in, const float* z, float* y) {
	for (int o = 0; o < n_out; ++o) {
		float a = 0.f;
		const float* w = W + (size_t)o * n_in;
		for (int k = 0; k < n_in; ++k) a = fmaf(w[k], z[k], a);
		y[o] = a;
	}
}
/* y[k] = sum_o W[o][k] d[o] */
static inline void matvec_t(const float* W, int n_out, int n_in, const float* dvec, float* y) {
	for (int k = 0; k < n_in; ++k) y[k] = 0.f;
	for (int o = 0; o < n_out; ++o) {
		const float* w = W + (size_t)o * n_in;
		float dv = dvec[o];
		if (dv == 0.f) continue;
		for (int k = 0; k < n_in; ++k) y[k] = fmaf(w[k], dv, y[k]);
	}
}
static inline void relu_round(float* v, int n) {
	for (int i = 0; i < n; ++i) v[i] = rh(v[i] > 0.f ? v[i] : 0.f);
}
static inline void round_vec(float* v, int n) {
	for (int i = 0; i < n; ++i) v[i] = rh(v[i]);
}
static size_t mlp_n_params(uint32_t in_w, uint32_t n_hidden) { return 64u * in_w + (n_hidden - 1) * 64u * 64u + 16u * 64u; }

void n2o_mlp_forward(uint32_t n, uint32_t in_w, uint32_t n_hidden, const uint16_t* w, const uint16_t* in, uint16_t* out,
                     uint16_t* hidden) {
	size_t np = mlp_n_params(in_w, n_hidden);
	float* W = (float*)malloc(np * sizeof(float));
	to_float(w, W, np);
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		float z[64], h[64], y[16];
		for (uint32_t k = 0; k < in_w; ++k) z[k] = h2f(in[(size_t)i * in_w + k]);
		const float* Wl = W;
		int cur_in = (int)in_w;
		for (uint32_t l = 0; l < n_hidden; ++l) {
			matvec(Wl, 64, cur_in, z, h);
			relu_round(h, 64);
			if (hidden)
				for (int j = 0; j < 64; ++j) hidden[((size_t)i * n_hidden + l) * 64 + j] = f2h(h[j]);
			Wl += (size_t)64 * cur_in;
			cur_in = 64;
			memcpy(z, h, sizeof(h));
		}
		matvec(Wl, 16, 64, z, y);
		for (int o = 0; o < 16; ++o) out[(size_t)i * 16 + o] = f2h(y[o]);
	}
	free(W);
}

void n2o_mlp_backward(uint32_t n, uint32_t in_w, uint32_t n_hidden, const uint16_t* w, const uint16_t* in,
                      const uint16_t* hidden, const uint16_t* dL_dout, uint16_t* dL_din, double* wgrad) {
	size_t np = mlp_n_params(in_w, n_hidden);
	float* W = (float*)malloc(np * sizeof(float));
	to_float(w, W, np);
#pragma omp parallel
	{
		double* loc = wgrad ? (double*)calloc(np, sizeof(double)) : NULL;
#pragma omp for schedule(static)
		for (int64_t i = 0; i < (int64_t)n; ++i) {
			float dy[64], dz[64], act[64];
			for (int o = 0; o < 16; ++o) dy[o] = h2f(dL_dout[(size_t)i * 16 + o]);
			/* output layer */
			size_t off_last = (size_t)64 * in_w + (size_t)(n_hidden - 1) * 4096;
			const uint16_t* hl = hidden + ((size_t)i * n_hidden + (n_hidden - 1)) * 64;
			for (int j = 0; j < 64; ++j) act[j] = h2f(hl[j]);
			if (loc)
				for (int o = 0; o < 16; ++o)
					for (int j = 0; j < 64; ++j) loc[off_last + (size_t)o * 64 + j] += (double)(dy[o] * act[j]);
			matvec_t(W + off_last, 16, 64, dy, dz);
			for (int j = 0; j < 64; ++j) dz[j] = act[j] > 0.f ? rh(dz[j]) : 0.f;
			/* hidden layers, last to first */
			for (int l = (int)n_hidden - 1; l >= 0; --l) {
				size_t off = l == 0 ? 0 : (size_t)64 * in_w + (size_t)(l - 1) * 4096;
				int cur_in = l == 0 ? (int)in_w : 64;
				float prev[64];
				if (l == 0)
					for (int k = 0; k < cur_in; ++k) prev[k] = h2f(in[(size_t)i * in_w + k]);
				else
					for (int k = 0; k < 64; ++k) prev[k] = h2f(hidden[((size_t)i * n_hidden + (l - 1)) * 64 + k]);
				memcpy(dy, dz, sizeof(dz));
				if (loc)
					for (int j = 0; j < 64; ++j)
						if (dy[j] != 0.f)
							for (int k = 0; k < cur_in; ++k) loc[off + (size_t)j * cur_in + k] += (double)(dy[j] * prev[k]);
				matvec_t(W + off, 64, cur_in, dy, dz);
				if (l == 0) {
					if (dL_din)
						for (int k = 0; k < cur_in; ++k) dL_din[(size_t)i * in_w + k] = f2h(dz[k]);
				} else {
					for (int k = 0; k < 64; ++k) dz[k] = prev[k] > 0.f ? rh(dz[k]) : 0.f;
				}
			}
		}
		if (loc) {
#pragma omp critical
			for (size_t k = 0; k < np; ++k) wgrad[k] += loc[k];
			free(loc);
		}
	}
	free(W);
}

void n2o_mlp_backward_backward_input(uint32_t n, uint32_t in_w, const uint16_t* w, const uint16_t* hidden, const uint16_t* u,
                                     const uint16_t* dy, double* wgrad) {
	size_t np = mlp_n_params(in_w, 1);
	float* W = (float*)malloc(np * sizeof(float));
	to_float(w, W, np);
	const float* W1 = W;
	const float* W2 = W + (size_t)64 * in_w;
#pragma omp parallel
	{
		double* loc = (double*)calloc(np, sizeof(double));
#pragma omp for schedule(static)
		for (int64_t i = 0; i < (int64_t)n; ++i) {
			float uu[64], t[64], s[64], dyv[16], hh[64];
			for (uint32_t k = 0; k < in_w; ++k) uu[k] = h2f(u[(size_t)i * in_w + k]);
			for (int o = 0; o < 16; ++o) dyv[o] = h2f(dy[(size_t)i * 16 + o]);
			for (int j = 0; j < 64; ++j) hh[j] = h2f(hidden[(size_t)i * 64 + j]);
			matvec(W1, 64, (int)in_w, uu, t);
			matvec_t(W2, 16, 64, dyv, s);
			for (int j = 0; j < 64; ++j) {
				t[j] = hh[j] > 0.f ? rh(t[j]) : 0.f;
				s[j] = hh[j] > 0.f ? rh(s[j]) : 0.f;
			}
			for (int o = 0; o < 16; ++o)
				if (dyv[o] != 0.f)
					for (int j = 0; j < 64; ++j) loc[(size_t)64 * in_w + (size_t)o * 64 + j] += (double)(dyv[o] * t[j]);
			for (int j = 0; j < 64; ++j)
				if (s[j] != 0.f)
					for (uint32_t k = 0; k < in_w; ++k) loc[(size_t)j * in_w + k] += (double)(s[j] * uu[k]);
		}
#pragma omp critical
		for (size_t k = 0; k < np; ++k) wgrad[k] += loc[k];
		free(loc);
	}
	free(W);
}

/* ------------------------------------------------------------------ real spherical harmonics, degree 4 (16 values) */
static void sh4_eval(const float* dir01, float* out) {
	float x = dir01[0] * 2.f - 1.f, y = dir01[1] * 2.f - 1.f, z = dir01[2] * 2.f - 1.f;
	float xy = x * y, xz = x * z, yz = y * z, x2 = x * x, y2 = y * y, z2 = z * z;
	out[0] = 0.28209479177387814f;
	out[1] = -0.48860251190291987f * y;
	out[2] = 0.48860251190291987f * z;
	out[3] = -0.48860251190291987f * x;
	out[4] = 1.0925484305920792f * xy;
	out[5] = -1.0925484305920792f * yz;
	out[6] = 0.94617469575755997f * z2 - 0.31539156525251999f;
	out[7] = -1.0925484305920792f * xz;
	out[8] = 0.54627421529603959f * x2 - 0.54627421529603959f * y2;
	out[9] = 0.59004358992664352f * y * (-3.0f * x2 + y2);
	out[10] = 2.8906114426405538f * xy * z;
	out[11] = 0.45704579946446572f * y * (1.0f - 5.0f * z2);
	out[12] = 0.3731763325901154f * z * (5.0f * z2 - 3.0f);
	out[13] = 0.45704579946446572f * x * (1.0f - 5.0f * z2);
	out[14] = 1.4453057213202769f * z * (x2 - y2);
	out[15] = 0.59004358992664352f * x * (-x2 + 3.0f * y2);
}

void n2o_sh4(uint32_t n, const float* dir01, uint32_t stride, uint16_t* out) {
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		float o[16];
		sh4_eval(dir01 + (size_t)i * stride, o);
		for (int k = 0; k < 16; ++k) out[(size_t)i * 16 + k] = f2h(o[k]);
	}
}

/* ------------------------------------------------------------------ whole NeuS graph */
typedef struct {
	float W1s[64 * 48], W2s[16 * 64], W1c[64 * 48], W2c[64 * 64], W3c[16 * 64];
	float variance;
} weights_t;

static weights_t* load_weights(const n2o_grid_desc* d, const uint16_t* params) {
	weights_t* w = (weights_t*)malloc(sizeof(weights_t));
	to_float(params + N2O_SDF_W1, w->W1s, 64 * 48);
	to_float(params + N2O_SDF_W2, w->W2s, 16 * 64);
	to_float(params + N2O_RGB_W1, w->W1c, 64 * 48);
	to_float(params + N2O_RGB_W2, w->W2c, 64 * 64);
	to_float(params + N2O_RGB_W3, w->W3c, 16 * 64);
	w->variance = h2f(params[N2O_GRID_OFF + n2o_grid_n_params(d)]);
	return w;
}

typedef struct {
	float zs[48], hs[64], ys[16], dh[64], gz[48], n[3];
	float zc[48], h1[64], h2[64], o[16];
	float J[32][3];
} sample_t;

/* nerf_network.h:132-315 for one sample. x = coords[0..2], dir = coords[4..6] (already in [0,1]). */
static void sample_forward(const n2o_grid_desc* d, const n2o_grid_levels* lv, const uint16_t* grid, const weights_t* w,
                           const float* coords, sample_t* s) {
	const float* x = coords;
	const float* dir = coords + 4;
	const uint32_t W = 2 * d->n_levels;
	float enc[32];
	memset(s->zs, 0, sizeof(s->zs));
	memset(s->zc, 0, sizeof(s->zc));
	memset(s->J, 0, sizeof(s->J));
	grid_sample_forward(d, lv, grid, x, enc, s->J);
	for (int e = 0; e < 3; ++e) s->zs[e] = rh(rh(x[e]) - 0.5f); /* fill_positions_view_with_fixed_offset */
	for (uint32_t k = 0; k < W; ++k) s->zs[3 + k] = enc[k];
	matvec(w->W1s, 64, 48, s->zs, s->hs);
	relu_round(s->hs, 64);
	matvec(w->W2s, 16, 64, s->hs, s->ys);
	round_vec(s->ys, 16);
	/* normal = d sdf / d x : backward of the SDF net seeded with dL/dy = e0 (nerf_network.h:215-238) */
	for (int j = 0; j < 64; ++j) s->dh[j] = s->hs[j] > 0.f ? w->W2s[j] : 0.f;
	matvec_t(w->W1s, 64, 48, s->dh, s->gz);
	round_vec(s->gz, 48);
	for (int e = 0; e < 3; ++e) {
		float a = 0.f;
		for (uint32_t k = 0; k < W; ++k) a = fmaf(s->J[k][e], s->gz[3 + k], a);
		s->n[e] = a + s->gz[e];
	}
	/* colour net input: [sdf-net out 16 | SH 16 | xyz 3 | normal 3 | 0] (nerf_network.h:249-267) */
	for (int k = 0; k < 16; ++k) s->zc[k] = s->ys[k];
	float sh[16];
	sh4_eval(dir, sh);
	for (int k = 0; k < 16; ++k) s->zc[16 + k] = rh(sh[k]);
	for (int e = 0; e < 3; ++e) {
		s->zc[32 + e] = rh(x[e]);
		s->zc[35 + e] = rh(s->n[e]);
	}
	matvec(w->W1c, 64, 48, s->zc, s->h1);
	relu_round(s->h1, 64);
	matvec(w->W2c, 64, 64, s->h1, s->h2);
	relu_round(s->h2, 64);
	matvec(w->W3c, 16, 64, s->h2, s->o);
	round_vec(s->o, 16);
}

void n2o_neus_forward(const n2o_grid_desc* d, const uint16_t* params, float sdf_bias, uint32_t n, const float* coords,
                      uint16_t* out) {
	n2o_grid_levels lv;
	n2o_grid_make_levels(d, &lv);
	weights_t* w = load_weights(d, params);
	const uint16_t* grid = params + N2O_GRID_OFF;
	const float bias = rh(sdf_bias);
#pragma omp parallel for schedule(dynamic, 256)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		sample_t s;
		const float* c = coords + (size_t)i * 7;
		sample_forward(d, &lv, grid, w, c, &s);
		uint16_t* o = out + (size_t)i * 16;
		for (int k = 0; k < 16; ++k) o[k] = f2h(s.o[k]);
		o[3] = f2h(s.ys[0] + bias);                    /* extract_sdf_value_view_with_bias */
		for (int e = 0; e < 3; ++e) o[4 + e] = f2h(s.n[e]); /* extract_dSDF_dPos_view */
		o[7] = f2h(w->variance);                        /* extract_single_variance_view */
		for (int e = 0; e < 3; ++e) o[8 + e] = f2h(c[4 + e]);
	}
	free(w);
}

void n2o_neus_sdf(const n2o_grid_desc* d, const uint16_t* params, float sdf_bias, uint32_t n, const float* x,
                  uint32_t x_stride, uint16_t* sdf) {
	n2o_grid_levels lv;
	n2o_grid_make_levels(d, &lv);
	weights_t* w = load_weights(d, params);
	const uint16_t* grid = params + N2O_GRID_OFF;
	const float bias = rh(sdf_bias);
	const uint32_t W = 2 * d->n_levels;
#pragma omp parallel for schedule(dynamic, 256)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		float zs[48], hs[64], enc[32], y0 = 0.f;
		const float* xi = x + (size_t)i * x_stride;
		memset(zs, 0, sizeof(zs));
		grid_sample_forward(d, &lv, grid, xi, enc, NULL);
		for (int e = 0; e < 3; ++e) zs[e] = rh(rh(xi[e]) - 0.5f);
		for (uint32_t k = 0; k < W; ++k) zs[3 + k] = enc[k];
		matvec(w->W1s, 64, 48, zs, hs);
		relu_round(hs, 64);
		for (int j = 0; j < 64; ++j) y0 = fmaf(w->W2s[j], hs[j], y0);
		sdf[i] = f2h(rh(y0) + bias);
	}
	free(w);
}

void n2o_neus_backward(const n2o_grid_desc* d, const uint16_t* params, uint32_t n, const float* coords,
                       const uint16_t* dL_dout, uint32_t indeed_batch_size, double* grad) {
	n2o_neus_backward_dx(d, params, n, coords, dL_dout, indeed_batch_size, grad, NULL);
}

void n2o_neus_backward_dx(const n2o_grid_desc* d, const uint16_t* params, uint32_t n, const float* coords,
                          const uint16_t* dL_dout, uint32_t indeed_batch_size, double* grad, float* dL_dx) {
	n2o_grid_levels lv;
	n2o_grid_make_levels(d, &lv);
	weights_t* w = load_weights(d, params);
	const uint16_t* grid = params + N2O_GRID_OFF;
	double* ggrid = grad + N2O_GRID_OFF;
	const uint32_t W = 2 * d->n_levels;
	const size_t var_off = (size_t)N2O_GRID_OFF + n2o_grid_n_params(d);
#pragma omp parallel
	{
		double* loc = (double*)calloc(N2O_MLP_N + 1, sizeof(double));
#pragma omp for schedule(dynamic, 256)
		for (int64_t i = 0; i < (int64_t)n; ++i) {
			sample_t s;
			const float* c = coords + (size_t)i * 7;
			sample_forward(d, &lv, grid, w, c, &s);
			float g[16];
			for (int k = 0; k < 16; ++k) g[k] = h2f(dL_dout[(size_t)i * 16 + k]);
			/* colour net backward (nerf_network.h:331-340): only rows 0-2 of dL_doutput feed it */
			float dy3[16] = {g[0], g[1], g[2], 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
			float dh2[64], dh1[64], dzc[48];
			for (int o = 0; o < 3; ++o)
				for (int j = 0; j < 64; ++j) loc[N2O_RGB_W3 + o * 64 + j] += (double)(dy3[o] * s.h2[j]);
			matvec_t(w->W3c, 16, 64, dy3, dh2);
			for (int j = 0; j < 64; ++j) dh2[j] = s.h2[j] > 0.f ? rh(dh2[j]) : 0.f;
			for (int j = 0; j < 64; ++j)
				if (dh2[j] != 0.f)
					for (int k = 0; k < 64; ++k) loc[N2O_RGB_W2 + j * 64 + k] += (double)(dh2[j] * s.h1[k]);
			matvec_t(w->W2c, 64, 64, dh2, dh1);
			for (int j = 0; j < 64; ++j) dh1[j] = s.h1[j] > 0.f ? rh(dh1[j]) : 0.f;
			for (int j = 0; j < 64; ++j)
				if (dh1[j] != 0.f)
					for (int k = 0; k < 48; ++k) loc[N2O_RGB_W1 + j * 48 + k] += (double)(dh1[j] * s.zc[k]);
			matvec_t(w->W1c, 64, 48, dh1, dzc);
			round_vec(dzc, 48);
			/* SDF net backward (nerf_network.h:388-402): rows 0-15 of the colour-net input gradient + dL/dsdf */
			float dys[16], dhs[64], dzs[48];
			for (int o = 0; o < 16; ++o) dys[o] = dzc[o];
			dys[0] = rh(dys[0] + g[3]);
			for (int o = 0; o < 16; ++o)
				if (dys[o] != 0.f)
					for (int j = 0; j < 64; ++j) loc[N2O_SDF_W2 + o * 64 + j] += (double)(dys[o] * s.hs[j]);
			matvec_t(w->W2s, 16, 64, dys, dhs);
			for (int j = 0; j < 64; ++j) dhs[j] = s.hs[j] > 0.f ? rh(dhs[j]) : 0.f;
			for (int j = 0; j < 64; ++j)
				if (dhs[j] != 0.f)
					for (int k = 0; k < 48; ++k) loc[N2O_SDF_W1 + j * 48 + k] += (double)(dhs[j] * s.zs[k]);
			matvec_t(w->W1s, 64, 48, dhs, dzs);
			round_vec(dzs, 48);
			/* grid first-order parameter gradient (nerf_network.h:419-429) */
			for (uint32_t l = 0; l < d->n_levels && l < d->n_active_levels; ++l) {
				corners_t cr;
				level_corners(&lv, l, c, &cr);
				for (int k = 0; k < 8; ++k) {
					atomic_add_d(&ggrid[2 * (size_t)cr.idx[k]], (double)(cr.w[k] * dzs[3 + 2 * l]));
					atomic_add_d(&ggrid[2 * (size_t)cr.idx[k] + 1], (double)(cr.w[k] * dzs[3 + 2 * l + 1]));
				}
			}
			/* gradient for the DeltaNetwork (nerf_network.h:589-612): encoding dL/dx (first order) + xyz rows of both input gradients */
			if (dL_dx) {
				for (int e = 0; e < 3; ++e) {
					float a = 0.f;
					for (uint32_t k = 0; k < W; ++k) a = fmaf(s.J[k][e], dzs[3 + k], a);
					dL_dx[(size_t)i * 3 + e] = a + dzc[32 + e] + dzs[e];
				}
			}
			/* variance gradient: sum of row 7 (nerf_network.h:452-460) */
			loc[N2O_MLP_N] += (double)g[7];
			/* v = dL/dnormal (nerf_network.h:465-491) */
			float v[3];
			for (int e = 0; e < 3; ++e) v[e] = dzc[35 + e] + g[4 + e] / (float)indeed_batch_size + g[8 + e];
			/* second order (nerf_network.h:497-587) */
			float dyenc[32], u[48], t[64];
			grid_sample_bwd_bwd(d, &lv, grid, c, v, s.gz + 3, ggrid, dyenc);
			memset(u, 0, sizeof(u));
			for (int e = 0; e < 3; ++e) u[e] = rh(v[e]);
			for (uint32_t k = 0; k < W; ++k) u[3 + k] = dyenc[k];
			matvec(w->W1s, 64, 48, u, t);
			for (int j = 0; j < 64; ++j) {
				float tj = s.hs[j] > 0.f ? rh(t[j]) : 0.f;
				loc[N2O_SDF_W2 + j] += (double)tj; /* dy = e0 */
				float sj = s.dh[j];
				if (sj != 0.f)
					for (int k = 0; k < 48; ++k) loc[N2O_SDF_W1 + j * 48 + k] += (double)(sj * u[k]);
			}
		}
#pragma omp critical
		{
			for (size_t k = 0; k < N2O_MLP_N; ++k) grad[k] += loc[k];
			grad[var_off] += loc[N2O_MLP_N];
		}
		free(loc);
	}
	free(w);
}

/* ------------------------------------------------------------------ DeltaNetwork (transform_network.h, common_operation.cuh) */
static inline void normalize3(const float* a, float* b) {
	const float n = sqrtf(a[0] * a[0] + a[1] * a[1] + a[2] * a[2]);
	for (int e = 0; e < 3; ++e) b[e] = a[e] / n;
}
/* rotation_6d_to_matrix (common_operation.cuh:42-66): Gram-Schmidt on the two 3-vectors, columns b1, b2, b1 x b2 */
void n2o_rotation_6d_to_matrix(const uint16_t* rot6, float* R) {
	float a1[3], a2[3], b1[3], b2[3], u2[3];
	for (int e = 0; e < 3; ++e) {
		a1[e] = h2f(rot6[e]);
		a2[e] = h2f(rot6[3 + e]);
	}
	normalize3(a1, b1);
	const float dt = b1[0] * a2[0] + b1[1] * a2[1] + b1[2] * a2[2];
	for (int e = 0; e < 3; ++e) u2[e] = a2[e] - dt * b1[e];
	normalize3(u2, b2);
	const float b3[3] = {b1[1] * b2[2] - b1[2] * b2[1], b1[2] * b2[0] - b1[0] * b2[2], b1[0] * b2[1] - b1[1] * b2[0]};
	for (int r = 0; r < 3; ++r) {
		R[r * 3 + 0] = b1[r];
		R[r * 3 + 1] = b2[r];
		R[r * 3 + 2] = b3[r];
	}
}
static inline void matvec3(const float* R, const float* v, float* out) {
	for (int r = 0; r < 3; ++r) out[r] = (R[r * 3] * v[0] + R[r * 3 + 1] * v[1]) + R[r * 3 + 2] * v[2];
}

void n2o_delta_forward(const uint16_t* delta, const float* off, uint32_t n, const float* coords_in, float* coords_out) {
	float R[9];
	n2o_rotation_6d_to_matrix(delta + 4, R);
	const float t[3] = {h2f(delta[0]), h2f(delta[1]), h2f(delta[2])};
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		const float* c = coords_in + (size_t)i * 7;
		float* o = coords_out + (size_t)i * 7;
		float p[3], q[3], dd[3], dr[3];
		for (int e = 0; e < 3; ++e) p[e] = c[e] + (t[e] - off[e]); /* pos += transition - first_frame_offset (:443-445) */
		matvec3(R, p, q);
		for (int e = 0; e < 3; ++e) o[e] = q[e] + off[e];
		o[3] = c[3];
		for (int e = 0; e < 3; ++e) dd[e] = c[4 + e] * 2.0f - 1.0f;
		matvec3(R, dd, dr);
		for (int e = 0; e < 3; ++e) o[4 + e] = (dr[e] + 1.0f) * 0.5f;
	}
}

/* d normalize(x) / d x applied to a gradient: (g - (g . b) b) / |x| with b = x / |x| (gradients_for_normalize, :68-94) */
static inline void normalize_bwd(const double* x, const double* g, double* out) {
	const double n = sqrt(x[0] * x[0] + x[1] * x[1] + x[2] * x[2]);
	const double b[3] = {x[0] / n, x[1] / n, x[2] / n};
	const double gb = g[0] * b[0] + g[1] * b[1] + g[2] * b[2];
	for (int e = 0; e < 3; ++e) out[e] = (g[e] - gb * b[e]) / n;
}
/* gradient_rotation_matrix_to_6d (:96-158): backward of the Gram-Schmidt construction; G[r][c] = dL / dR(r, c) */
static void rotation_6d_backward(const uint16_t* rot6, const double* G, double* g6) {
	double a1[3], a2[3], b1[3], b2[3], u2[3];
	for (int e = 0; e < 3; ++e) {
		a1[e] = (double)h2f(rot6[e]);
		a2[e] = (double)h2f(rot6[3 + e]);
	}
	const double n1 = sqrt(a1[0] * a1[0] + a1[1] * a1[1] + a1[2] * a1[2]);
	for (int e = 0; e < 3; ++e) b1[e] = a1[e] / n1;
	const double dt = b1[0] * a2[0] + b1[1] * a2[1] + b1[2] * a2[2];
	for (int e = 0; e < 3; ++e) u2[e] = a2[e] - dt * b1[e];
	const double n2 = sqrt(u2[0] * u2[0] + u2[1] * u2[1] + u2[2] * u2[2]);
	for (int e = 0; e < 3; ++e) b2[e] = u2[e] / n2;
	const double g1[3] = {G[0], G[3], G[6]}, g2[3] = {G[1], G[4], G[7]}, g3[3] = {G[2], G[5], G[8]};
	/* b3 = b1 x b2: dL/db1 += b2 x g3, dL/db2 += g3 x b1 */
	double db1[3] = {g1[0] + (b2[1] * g3[2] - b2[2] * g3[1]), g1[1] + (b2[2] * g3[0] - b2[0] * g3[2]), g1[2] + (b2[0] * g3[1] - b2[1] * g3[0])};
	double db2[3] = {g2[0] + (g3[1] * b1[2] - g3[2] * b1[1]), g2[1] + (g3[2] * b1[0] - g3[0] * b1[2]), g2[2] + (g3[0] * b1[1] - g3[1] * b1[0])};
	double du2[3], da2[3], da1[3];
	normalize_bwd(u2, db2, du2);
	const double du2b1 = du2[0] * b1[0] + du2[1] * b1[1] + du2[2] * b1[2];
	for (int e = 0; e < 3; ++e) {
		da2[e] = du2[e] - du2b1 * b1[e];          /* u2 = a2 - (b1 . a2) b1 */
		db1[e] -= dt * du2[e] + du2b1 * a2[e];
	}
	normalize_bwd(a1, db1, da1);
	for (int e = 0; e < 3; ++e) {
		g6[e] = da1[e];
		g6[3 + e] = da2[e];
	}
}

void n2o_delta_backward(const uint16_t* delta, const float* off, uint32_t n, const float* coords_in, const float* dL_dx, double* grad) {
	(void)off; /* the reference's backward leaves the offset out of the rotated vector (input + transition, :811) */
	float R[9];
	n2o_rotation_6d_to_matrix(delta + 4, R);
	const float t[3] = {h2f(delta[0]), h2f(delta[1]), h2f(delta[2])};
	double G[9] = {0}, L[3] = {0};
	for (uint32_t i = 0; i < n; ++i) {
		const float* c = coords_in + (size_t)i * 7;
		const float* l = dL_dx + (size_t)i * 3;
		const float v[3] = {c[0] + t[0], c[1] + t[1], c[2] + t[2]};
		for (int r = 0; r < 3; ++r) {
			L[r] += (double)l[r];
			for (int k = 0; k < 3; ++k) G[r * 3 + k] += (double)(l[r] * v[k]); /* loss_vector (x) input_vector (:829-831) */
		}
	}
	/* transition: R^-1 dL/dx' summed = R^T sum (:812-820); rotation: the 6-D backward is linear in G, so it is applied to the sum */
	for (int e = 0; e < 3; ++e) grad[e] += (double)R[0 * 3 + e] * L[0] + (double)R[1 * 3 + e] * L[1] + (double)R[2 * 3 + e] * L[2];
	double g6[6];
	rotation_6d_backward(delta + 4, G, g6);
	for (int e = 0; e < 6; ++e) grad[4 + e] += g6[e];
}

void n2o_accumulate_global_movement(const uint16_t* delta, float* acc_R, float* acc_t) {
	float R[9], out[9], tv[3], tr[3];
	n2o_rotation_6d_to_matrix(delta + 4, R);
	for (int r = 0; r < 3; ++r)
		for (int c = 0; c < 3; ++c) out[r * 3 + c] = (R[r * 3] * acc_R[c] + R[r * 3 + 1] * acc_R[3 + c]) + R[r * 3 + 2] * acc_R[6 + c];
	for (int e = 0; e < 3; ++e) tv[e] = acc_t[e] + h2f(delta[e]); /* R (t_acc + t) (:583) */
	matvec3(R, tv, tr);
	for (int k = 0; k < 9; ++k) acc_R[k] = rh(out[k]);
	for (int e = 0; e < 3; ++e) acc_t[e] = rh(tr[e]);
}

/* ------------------------------------------------------------------ PCG32 (published generator; float = 23 mantissa bits) */
#define PCG_MULT 0x5851f42d4c957f2dULL
void n2o_pcg32_seed(n2o_pcg32* r, uint64_t seed) {
	/* default_rng_t{seed} in the reference (src/testbed.cu:2077, :2090): pcg32's constructor takes the stream selector
	 * initseq = 1 by default; the generator's default stream constant belongs to the argument-less constructor only */
	const uint64_t initseq = 1u;
	r->state = 0u;
	r->inc = (initseq << 1u) | 1u;
	n2o_pcg32_next_uint(r);
	r->state += seed;
	n2o_pcg32_next_uint(r);
}
uint32_t n2o_pcg32_next_uint(n2o_pcg32* r) {
	uint64_t old = r->state;
	r->state = old * PCG_MULT + r->inc;
	uint32_t xorshifted = (uint32_t)(((old >> 18u) ^ old) >> 27u);
	uint32_t rot = (uint32_t)(old >> 59u);
	return (xorshifted >> rot) | (xorshifted << ((~rot + 1u) & 31u));
}
float n2o_pcg32_next_float(n2o_pcg32* r) {
	uint32_t u = (n2o_pcg32_next_uint(r) >> 9) | 0x3f800000u;
	float f;
	memcpy(&f, &u, 4);
	return f - 1.0f;
}
void n2o_pcg32_advance(n2o_pcg32* r, uint64_t delta) {
	uint64_t cur_mult = PCG_MULT, cur_plus = r->inc, acc_mult = 1u, acc_plus = 0u;
	while (delta > 0) {
		if (delta & 1) {
			acc_mult *= cur_mult;
			acc_plus = acc_plus * cur_mult + cur_plus;
		}
		cur_plus = (cur_mult + 1) * cur_plus;
		cur_mult *= cur_mult;
		delta >>= 1;
	}
	r->state = acc_mult * r->state + acc_plus;
}

/* ------------------------------------------------------------------ ray march helpers (src/testbed_nerf.cu) */
static inline float min_cone_stepsize(void) { return 1.73205080757f / (float)N2O_STEPS; }
static inline float max_cone_stepsize(void) {
	return min_cone_stepsize() * (float)(1u << (N2O_CASCADES - 1)) * (float)N2O_STEPS / (float)N2O_GRIDSIZE;
}
/* calc_dt, src/testbed_nerf.cu:152 */
static inline float calc_dt(float t, float cone_angle) { return clampf(t * cone_angle, min_cone_stepsize(), max_cone_stepsize()); }
/* warp_dt / unwarp_dt, src/testbed_nerf.cu:474-482 */
static inline float warp_dt(float dt) {
	float mx = min_cone_stepsize() * (float)(1u << (N2O_CASCADES - 1));
	return (dt - min_cone_stepsize()) / (mx - min_cone_stepsize());
}
static inline float unwarp_dt(float dt) {
	float mx = min_cone_stepsize() * (float)(1u << (N2O_CASCADES - 1));
	return dt * (mx - min_cone_stepsize()) + min_cone_stepsize();
}
static inline uint32_t expand_bits(uint32_t v) {
	v = (v * 0x00010001u) & 0xFF0000FFu;
	v = (v * 0x00000101u) & 0x0F00F00Fu;
	v = (v * 0x00000011u) & 0xC30C30C3u;
	v = (v * 0x00000005u) & 0x49249249u;
	return v;
}
uint32_t n2o_morton3d(uint32_t x, uint32_t y, uint32_t z) { return expand_bits(x) | (expand_bits(y) << 1) | (expand_bits(z) << 2); }
uint32_t n2o_morton3d_invert(uint32_t x) {
	x = x & 0x49249249u;
	x = (x | (x >> 2)) & 0xc30c30c3u;
	x = (x | (x >> 4)) & 0x0f00f00fu;
	x = (x | (x >> 8)) & 0xff0000ffu;
	x = (x | (x >> 16)) & 0x0000ffffu;
	return x;
}
/* mip_from_pos / mip_from_dt, src/testbed_nerf.cu:614-628 (max_cascade defaults to NERF_CASCADES-1 at the call sites) */
static inline int mip_from_pos(const float* p) {
	int exponent;
	float m = fmaxf(fmaxf(fabsf(p[0] - 0.5f), fabsf(p[1] - 0.5f)), fabsf(p[2] - 0.5f));
	frexpf(m, &exponent);
	int mip = exponent + 1;
	if (mip < 0) mip = 0;
	if (mip > (int)N2O_CASCADES - 1) mip = (int)N2O_CASCADES - 1;
	return mip;
}
static inline int mip_from_dt(float dt, const float* p) {
	int mip = mip_from_pos(p);
	dt *= 2.f * (float)N2O_GRIDSIZE;
	if (dt < 1.f) return mip;
	int exponent;
	frexpf(dt, &exponent);
	int m = exponent > mip ? exponent : mip;
	return m > (int)N2O_CASCADES - 1 ? (int)N2O_CASCADES - 1 : m;
}
/* cascaded_grid_idx_at / density_grid_occupied_at, src/testbed_nerf.cu:484-510 */
static inline uint32_t cascaded_grid_idx_at(const float* pos, uint32_t mip) {
	float mip_scale = scalbnf(1.0f, -(int)mip);
	int i[3];
	for (int d = 0; d < 3; ++d) {
		float p = (pos[d] - 0.5f) * mip_scale + 0.5f;
		int v = (int)(p * (float)N2O_GRIDSIZE);
		i[d] = v < 0 ? 0 : (v > (int)N2O_GRIDSIZE - 1 ? (int)N2O_GRIDSIZE - 1 : v);
	}
	return n2o_morton3d((uint32_t)i[0], (uint32_t)i[1], (uint32_t)i[2]);
}
static inline int occupied_at(const float* pos, const uint8_t* bitfield, uint32_t mip) {
	uint32_t idx = cascaded_grid_idx_at(pos, mip);
	uint32_t cells = N2O_GRIDSIZE * N2O_GRIDSIZE * N2O_GRIDSIZE;
	return (bitfield[idx / 8 + (cells * mip) / 8] & (1u << (idx % 8))) != 0;
}
static inline float signf(float x) { return copysignf(1.0f, x); }
/* distance_to_next_voxel / advance_to_next_voxel, src/testbed_nerf.cu:346-368 */
static inline float advance_to_next_voxel(float t, float cone_angle, const float* pos, const float* dir, const float* idir,
                                          uint32_t res) {
	float tt[3];
	for (int d = 0; d < 3; ++d) {
		float p = (float)res * pos[d];
		tt[d] = (floorf(p + 0.5f + 0.5f * signf(dir[d])) - p) * idir[d];
	}
	float tmin = fminf(fminf(tt[0], tt[1]), tt[2]);
	float t_target = t + fmaxf(tmin / (float)res, 0.0f);
	do {
		t += calc_dt(t, cone_angle);
	} while (t < t_target);
	return t;
}
/* BoundingBox::ray_intersect, include/neural-graphics-primitives/bounding_box.cuh:163-210 */
static void aabb_ray_intersect(const float* mn, const float* mx, const float* o, const float* d, float* tmin_out, float* tmax_out) {
	float tmin = (mn[0] - o[0]) / d[0], tmax = (mx[0] - o[0]) / d[0];
	if (tmin > tmax) { float t = tmin; tmin = tmax; tmax = t; }
	float tymin = (mn[1] - o[1]) / d[1], tymax = (mx[1] - o[1]) / d[1];
	if (tymin > tymax) { float t = tymin; tymin = tymax; tymax = t; }
	if (tmin > tymax || tymin > tmax) { *tmin_out = *tmax_out = 3.402823466e+38f; return; }
	if (tymin > tmin) tmin = tymin;
	if (tymax < tmax) tmax = tymax;
	float tzmin = (mn[2] - o[2]) / d[2], tzmax = (mx[2] - o[2]) / d[2];
	if (tzmin > tzmax) { float t = tzmin; tzmin = tzmax; tzmax = t; }
	if (tmin > tzmax || tzmin > tmax) { *tmin_out = *tmax_out = 3.402823466e+38f; return; }
	if (tzmin > tmin) tmin = tzmin;
	if (tzmax < tmax) tmax = tzmax;
	*tmin_out = tmin;
	*tmax_out = tmax;
}
static inline int aabb_contains(const float* mn, const float* mx, const float* p) {
	return p[0] >= mn[0] && p[0] <= mx[0] && p[1] >= mn[1] && p[1] <= mx[1] && p[2] >= mn[2] && p[2] <= mx[2];
}
/* colour helpers, include/neural-graphics-primitives/common_device.cuh:31-77 */
static inline float srgb_to_linear(float s) { return s <= 0.04045f ? s / 12.92f : powf((s + 0.055f) / 1.055f, 2.4f); }
static inline float linear_to_srgb(float l) { return l < 0.0031308f ? 12.92f * l : 1.055f * powf(l, 0.41666f) - 0.055f; }
/* image_pos / read_rgba (Byte images), common_device.cuh:591-642 */
static void read_rgba(const n2o_dataset* ds, uint32_t img, const float* xy, float* rgba) {
	int px = (int)(xy[0] * (float)ds->width), py = (int)(xy[1] * (float)ds->height);
	if (px > (int)ds->width - 1) px = (int)ds->width - 1;
	if (py > (int)ds->height - 1) py = (int)ds->height - 1;
	if (px < 0) px = 0;
	if (py < 0) py = 0;
	uint32_t v = ds->pixels[(size_t)img * ds->width * ds->height + (size_t)py * ds->width + px];
	if (v == 0x00FF00FFu) {
		rgba[0] = rgba[1] = rgba[2] = rgba[3] = -1.0f;
		return;
	}
	float a = (float)(v >> 24) * (1.0f / 255.0f);
	rgba[0] = srgb_to_linear((float)(v & 0xFF) * (1.0f / 255.0f)) * a;
	rgba[1] = srgb_to_linear((float)((v >> 8) & 0xFF) * (1.0f / 255.0f)) * a;
	rgba[2] = srgb_to_linear((float)((v >> 16) & 0xFF) * (1.0f / 255.0f)) * a;
	rgba[3] = a;
}
/* image_idx without the error-map CDF, src/testbed_nerf.cu:1231-1251 */
static inline uint32_t image_idx(uint32_t base_idx, uint32_t n_rays, uint32_t n_rays_total, uint32_t n_images) {
	return (uint32_t)((((uint64_t)(uint32_t)(base_idx + n_rays_total) * n_images) & 0xFFFFFFFFu) / n_rays) % n_images;
}
/* nerf_random_image_pos_training without CDF, src/testbed_nerf.cu:1216-1229 */
static inline void random_image_pos(n2o_pcg32* rng, const n2o_dataset* ds, int snap, float* xy) {
	xy[0] = n2o_pcg32_next_float(rng);
	xy[1] = n2o_pcg32_next_float(rng);
	if (snap) {
		int px = (int)(xy[0] * (float)ds->width), py = (int)(xy[1] * (float)ds->height);
		px = px < 0 ? 0 : (px > (int)ds->width - 1 ? (int)ds->width - 1 : px);
		py = py < 0 ? 0 : (py > (int)ds->height - 1 ? (int)ds->height - 1 : py);
		xy[0] = ((float)px + 0.5f) / (float)ds->width;
		xy[1] = ((float)py + 0.5f) / (float)ds->height;
	}
}

/* The reference writes these with Eigen expressions: a reduction over three terms is evaluated as a0 + (a1 + a2) (the
 * unrolled redux splits the range in halves, Eigen/src/Core/Redux.h), and normalized() divides every component by the root of
 * the squared norm (Eigen/src/Core/Dot.h) instead of multiplying by a reciprocal.  Checked against the reference's kernels
 * running on a GPU: with these the rays and sample positions agree bit for bit. */
static inline float sum3_eigen(float a, float b, float c) { return a + (b + c); }
static inline void normalize3_eigen(const float* v, float* out) {
	const float z = sum3_eigen(v[0] * v[0], v[1] * v[1], v[2] * v[2]);
	if (z > 0.0f) {
		const float n = sqrtf(z);
		for (int e = 0; e < 3; ++e) out[e] = v[e] / n;
	} else {
		for (int e = 0; e < 3; ++e) out[e] = v[e];
	}
}

typedef struct {
	uint32_t keep, numsteps;
	float o[3], d[3], dirn[3], startt;
} ray_tmp;

/* First half of generate_training_samples_nerf_with_global_movement (:1287-1409): build the ray, count steps. */
static void ray_setup(const n2o_dataset* ds, const n2o_train_cfg* cfg, uint32_t i, uint32_t n_rays, uint32_t n_rays_total,
                      n2o_pcg32 rng, const uint8_t* bitfield, ray_tmp* r) {
	r->keep = 0;
	r->numsteps = 0;
	const uint32_t ig = i + cfg->ray_index_offset;
	uint32_t img = image_idx(ig, n_rays, n_rays_total, ds->n_images);
	n2o_pcg32_advance(&rng, (uint64_t)ig * 8u);
	float xy[2], rgba[4];
	random_image_pos(&rng, ds, (int)cfg->snap_to_pixel_centers, xy);
	read_rgba(ds, img, xy, rgba);
	if (rgba[0] <= 0.0f && n2o_pcg32_next_float(&rng) >= 0.9f) return;
	(void)n2o_pcg32_next_float(&rng); /* motion-blur time draw (:1307) */
	const float* X = ds->xforms + (size_t)img * 12;
	const float* fl = ds->focal + (size_t)img * 2;
	const float* pp = ds->principal + (size_t)img * 2;
	float dl[3] = {(xy[0] - pp[0]) * (float)ds->width / fl[0], (xy[1] - pp[1]) * (float)ds->height / fl[1], 1.0f};
	for (int e = 0; e < 3; ++e) {
		r->o[e] = X[9 + e];
		r->d[e] = sum3_eigen(X[0 + e] * dl[0], X[3 + e] * dl[1], X[6 + e] * dl[2]);
	}
	normalize3_eigen(r->d, r->dirn);
	if (cfg->use_global_movement) { /* :1370-1378: the ray is moved, its direction is not normalised again */
		float o2[3], q[3], dq[3];
		for (int e = 0; e < 3; ++e) o2[e] = r->o[e] - cfg->first_frame_offset[e];
		matvec3(cfg->rotation, o2, q);
		matvec3(cfg->rotation, r->dirn, dq);
		for (int e = 0; e < 3; ++e) {
			r->o[e] = q[e] + cfg->transition[e];
			r->dirn[e] = r->d[e] = dq[e]; /* (the ray handed on is the moved one) */
		}
	}
	float tmin, tmax;
	aabb_ray_intersect(cfg->aabb_min, cfg->aabb_max, r->o, r->dirn, &tmin, &tmax);
	float cone_angle = cfg->cone_angle_constant;
	tmin = fmaxf(tmin, 0.0f);
	float startt = tmin;
	startt += calc_dt(startt, cone_angle) * n2o_pcg32_next_float(&rng);
	float idir[3] = {1.0f / r->dirn[0], 1.0f / r->dirn[1], 1.0f / r->dirn[2]};
	uint32_t j = 0;
	float t = startt, pos[3];
	for (;;) {
		for (int e = 0; e < 3; ++e) pos[e] = r->o[e] + t * r->dirn[e];
		if (!(aabb_contains(cfg->aabb_min, cfg->aabb_max, pos) && j < N2O_STEPS)) break;
		float dt = calc_dt(t, cone_angle);
		uint32_t mip = (uint32_t)mip_from_dt(dt, pos);
		if (occupied_at(pos, bitfield, mip)) {
			++j;
			t += dt;
		} else {
			t = advance_to_next_voxel(t, cone_angle, pos, r->dirn, idir, N2O_GRIDSIZE >> mip);
		}
	}
	r->startt = startt;
	r->numsteps = j;
	r->keep = j > 0;
}

uint32_t n2o_generate_samples(const n2o_dataset* ds, const n2o_train_cfg* cfg, uint32_t n_rays, uint32_t n_rays_total,
                              uint32_t max_samples, n2o_pcg32 rng, const uint8_t* bitfield, uint32_t* ray_indices, float* rays,
                              uint32_t* numsteps, float* coords, uint32_t* n_samples) {
	ray_tmp* tmp = (ray_tmp*)malloc(sizeof(ray_tmp) * (size_t)n_rays);
#pragma omp parallel for schedule(dynamic, 64)
	for (int64_t i = 0; i < (int64_t)n_rays; ++i) ray_setup(ds, cfg, (uint32_t)i, n_rays, n_rays_total, rng, bitfield, &tmp[i]);
	/* canonical order: exclusive scan over ray index replaces the two atomicAdds (:1411,:1418).  A ray whose samples
	 * would overflow max_samples is dropped but still consumes its range, like the reference's counter does. */
	uint32_t base = 0, kept = 0;
	for (uint32_t i = 0; i < n_rays; ++i) {
		if (!tmp[i].keep) continue;
		uint32_t b = base;
		base += tmp[i].numsteps;
		if (b + tmp[i].numsteps > max_samples) {
			tmp[i].keep = 0;
			continue;
		}
		ray_indices[kept] = i;
		memcpy(rays + (size_t)kept * 6, tmp[i].o, 12);
		memcpy(rays + (size_t)kept * 6 + 3, tmp[i].d, 12);
		numsteps[kept * 2 + 0] = tmp[i].numsteps;
		numsteps[kept * 2 + 1] = b;
		tmp[i].keep = 1 + kept;
		++kept;
	}
	*n_samples = base;
#pragma omp parallel for schedule(dynamic, 64)
	for (int64_t i = 0; i < (int64_t)n_rays; ++i) {
		if (!tmp[i].keep) continue;
		const ray_tmp* r = &tmp[i];
		uint32_t k = r->keep - 1;
		float* co = coords + (size_t)numsteps[k * 2 + 1] * 7;
		float idir[3] = {1.0f / r->dirn[0], 1.0f / r->dirn[1], 1.0f / r->dirn[2]};
		float wd[3] = {(r->dirn[0] + 1.f) * 0.5f, (r->dirn[1] + 1.f) * 0.5f, (r->dirn[2] + 1.f) * 0.5f};
		float t = r->startt, pos[3];
		uint32_t j = 0;
		float cone_angle = cfg->cone_angle_constant;
		for (;;) {
			for (int e = 0; e < 3; ++e) pos[e] = r->o[e] + t * r->dirn[e];
			if (!(aabb_contains(cfg->aabb_min, cfg->aabb_max, pos) && j < r->numsteps)) break;
			float dt = calc_dt(t, cone_angle);
			uint32_t mip = (uint32_t)mip_from_dt(dt, pos);
			if (occupied_at(pos, bitfield, mip)) {
				float* c = co + (size_t)j * 7;
				for (int e = 0; e < 3; ++e) {
					c[e] = (pos[e] - cfg->aabb_min[e]) / (cfg->aabb_max[e] - cfg->aabb_min[e]); /* warp_position */
					c[4 + e] = wd[e];
				}
				c[3] = warp_dt(dt);
				++j;
				t += dt;
			} else {
				t = advance_to_next_voxel(t, cone_angle, pos, r->dirn, idir, N2O_GRIDSIZE >> mip);
			}
		}
	}
	free(tmp);
	return kept;
}

typedef struct {
	float rgb[3], T, weight_sum;
	uint32_t n;
} comp_t;

typedef struct {
	float alpha, p_div_c, inv_s, iter_cos, true_cos, dt, next_sdf;
	float rgb[3], nrm[3];
} neus_sample_t;

/* NeuS alpha of one sample (src/testbed_nerf.cu:1568-1606 == :1779-1805) */
static inline void neus_sample(const uint16_t* o, const float* c, const float* dir, float anneal, neus_sample_t* s) {
	for (int e = 0; e < 3; ++e) s->rgb[e] = logisticf(h2f(o[e]));
	s->dt = unwarp_dt(c[3]);
	s->inv_s = expf(rh(10.0f * h2f(o[7]))); /* (half)10 * half, then __expf */
	float sdf = h2f(o[3]);
	for (int e = 0; e < 3; ++e) s->nrm[e] = h2f(o[4 + e]);
	s->true_cos = dir[0] * s->nrm[0] + dir[1] * s->nrm[1] + dir[2] * s->nrm[2];
	/* The reference writes these lines with double literals (0.5, 1.0), so the intermediates are fp64 and each line rounds
	 * to fp32 once (:1594-1598): r1 is rounded when it is passed to activation_function(float), the product with the
	 * annealing ratio is a float product, the sum and the two sdf estimates are fp64 sums. */
	float r1 = (float)((double)(-s->true_cos) * 0.5 + 0.5), r2 = -s->true_cos;
	float relu2a = (r2 > 0.f ? r2 : 0.f) * anneal;
	s->iter_cos = (float)(-((double)(r1 > 0.f ? r1 : 0.f) * (1.0 - (double)anneal) + (double)relu2a));
	float half_step = s->iter_cos * s->dt; /* float product, then * 0.5 in fp64 (exact) */
	s->next_sdf = (float)((double)sdf + (double)half_step * 0.5);
	float prev_sdf = (float)((double)sdf - (double)half_step * 0.5);
	float next_cdf = logisticf(s->next_sdf * s->inv_s), prev_cdf = logisticf(prev_sdf * s->inv_s);
	s->p_div_c = (prev_cdf - next_cdf + 1e-5f) / (prev_cdf + 1e-5f);
	s->alpha = clampf(s->p_div_c, 0.0f, 1.0f);
}

uint32_t n2o_compute_loss(const n2o_dataset* ds, const n2o_train_cfg* cfg, uint32_t n_rays_kept, uint32_t n_rays,
                          uint32_t n_rays_total, n2o_pcg32 rng0, uint32_t max_compacted, const uint16_t* mlp_out,
                          const uint32_t* ray_indices, const float* rays, uint32_t* numsteps, const float* coords,
                          float* coords_out, uint16_t* dloss_dout, float* loss_out, float* ek_loss_out) {
	comp_t* cp = (comp_t*)malloc(sizeof(comp_t) * (size_t)(n_rays_kept ? n_rays_kept : 1));
	const float anneal = cfg->cos_anneal_ratio;
	/* pass A (:1563-1617): composite, count samples until T < 1e-4 */
#pragma omp parallel for schedule(dynamic, 64)
	for (int64_t i = 0; i < (int64_t)n_rays_kept; ++i) {
		uint32_t ns = numsteps[i * 2], base = numsteps[i * 2 + 1];
		const float* rd = rays + (size_t)i * 6 + 3;
		float dir[3];
		normalize3_eigen(rd, dir);
		comp_t c = {{0, 0, 0}, 1.f, 0.f, 0};
		for (; c.n < ns; ++c.n) {
			if (c.T < 1e-4f) break;
			const uint16_t* o = mlp_out + (size_t)(base + c.n) * 16;
			if (c.n == 0) { /* BENT_DIR (:1574-1579) */
				float dd[3] = {h2f(o[8]) * 2.f - 1.f, h2f(o[9]) * 2.f - 1.f, h2f(o[10]) * 2.f - 1.f};
				normalize3_eigen(dd, dir);
			}
			neus_sample_t s;
			neus_sample(o, coords + (size_t)(base + c.n) * 7, dir, anneal, &s);
			float w = s.alpha * c.T;
			for (int e = 0; e < 3; ++e) c.rgb[e] += w * s.rgb[e];
			c.weight_sum += w;
			c.T *= (1.f - s.alpha);
		}
		cp[i] = c;
	}
	/* canonical compaction: exclusive scan by kept-ray index replaces atomicAdd (:1673) */
	uint32_t total = 0;
	uint32_t* cbase = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(n_rays_kept ? n_rays_kept : 1));
	for (uint32_t i = 0; i < n_rays_kept; ++i) {
		cbase[i] = total;
		total += cp[i].n;
	}
#pragma omp parallel for schedule(dynamic, 64)
	for (int64_t i = 0; i < (int64_t)n_rays_kept; ++i) {
		uint32_t ns = numsteps[i * 2], base = numsteps[i * 2 + 1];
		comp_t c = cp[i];
		uint32_t compacted_base = cbase[i];
		uint32_t mb = max_compacted < compacted_base ? max_compacted : compacted_base;
		uint32_t cn = max_compacted - mb < c.n ? max_compacted - mb : c.n;
		int full = (c.n == ns);
		numsteps[i * 2] = cn;
		numsteps[i * 2 + 1] = compacted_base;
		if (loss_out) loss_out[i] = 0.f;
		if (ek_loss_out) ek_loss_out[i] = 0.f;
		if (cn == 0) continue;
		/* target colour (:1619-1667) */
		uint32_t ray_idx = ray_indices[i] + cfg->ray_index_offset;
		n2o_pcg32 rng = rng0;
		n2o_pcg32_advance(&rng, (uint64_t)ray_idx * 8u);
		uint32_t img = image_idx(ray_idx, n_rays, n_rays_total, ds->n_images);
		float xy[2], bg[3], tex[4], target[3];
		random_image_pos(&rng, ds, (int)cfg->snap_to_pixel_centers, xy);
		if (cfg->random_bg_color) {
			for (int e = 0; e < 3; ++e) bg[e] = n2o_pcg32_next_float(&rng);
		} else {
			for (int e = 0; e < 3; ++e) bg[e] = cfg->background_color[e];
		}
		for (int e = 0; e < 3; ++e) bg[e] = srgb_to_linear(bg[e]);
		read_rgba(ds, img, xy, tex);
		for (int e = 0; e < 3; ++e) {
			target[e] = linear_to_srgb(tex[e] + (1.0f - tex[3]) * bg[e]); /* exposure scale = 1; EColorSpace::Linear, !linear_colors */
			bg[e] = linear_to_srgb(bg[e]);
		}
		float rgb_ray[3] = {c.rgb[0], c.rgb[1], c.rgb[2]};
		if (full)
			for (int e = 0; e < 3; ++e) rgb_ray[e] += c.T * bg[e];
		/* Huber(0.1)/5 (:301-317, :1459) */
		float lgl[3], lgg[3];
		for (int e = 0; e < 3; ++e) {
			float diff = rgb_ray[e] - target[e], ad = fabsf(diff), al = 0.1f;
			lgl[e] = (ad > al ? (ad - 0.5f * al) : 0.5f / al * diff * diff) / 5.0f;
			lgg[e] = (ad > al ? (diff > 0 ? 1.0f : -1.0f) : diff / al) / 5.0f;
		}
		/* double literals in the reference (:1690-1702): the comparisons are fp64, the assigned constants round to fp32 */
		float mask_gt = (double)tex[3] > 0.9999 ? 1.f : 0.f, gws, ws = c.weight_sum;
		if ((double)ws >= 1.0 - 1e-4) { ws = (float)(1.0 - 1e-4); gws = 0.f; }
		else if ((double)ws <= 1e-4) { ws = (float)1e-4; gws = 0.f; }
		else { float sg = 1.0f / (1.0f + expf(-ws)); gws = (mask_gt - sg) * ws * cfg->mask_loss_weight; }
		const float n_rays_f = (float)n_rays * (float)(cfg->ray_count_scale ? cfg->ray_count_scale : 1u);
		if (loss_out) loss_out[i] = sum3_eigen(lgl[0], lgl[1], lgl[2]) / 3.0f / n_rays_f; /* lg.loss.mean() (:1715) */
		const float loss_scale = cfg->loss_scale / n_rays_f;
		/* pass B (:1761-1952) */
		const float* rd = rays + (size_t)i * 6 + 3;
		float dir[3];
		normalize3_eigen(rd, dir);
		{
			const uint16_t* o = mlp_out + (size_t)base * 16;
			float dd[3] = {h2f(o[8]) * 2.f - 1.f, h2f(o[9]) * 2.f - 1.f, h2f(o[10]) * 2.f - 1.f};
			normalize3_eigen(dd, dir);
		}
		float rgb2[3] = {0, 0, 0}, T = 1.f, ek = 0.f;
		for (uint32_t j = 0; j < cn; ++j) {
			const uint16_t* o = mlp_out + (size_t)(base + j) * 16;
			const float* cin = coords + (size_t)(base + j) * 7;
			memcpy(coords_out + (size_t)(compacted_base + j) * 7, cin, 28);
			neus_sample_t s;
			neus_sample(o, cin, dir, anneal, &s);
			float w = s.alpha * T;
			for (int e = 0; e < 3; ++e) rgb2[e] += w * s.rgb[e];
			T *= (1.f - s.alpha);
			float g[16];
			memset(g, 0, sizeof(g));
			float dterm[3];
			for (int e = 0; e < 3; ++e) {
				float suffix = rgb_ray[e] - rgb2[e];
				g[e] = loss_scale * (w * lgg[e] * (s.rgb[e] * (1.0f - s.rgb[e])));
				dterm[e] = lgg[e] * (T * s.rgb[e] - suffix);
			}
			float dla = sum3_eigen(dterm[0], dterm[1], dterm[2]) + gws * (1.0f - ws); /* gradient.dot(T rgb - suffix) + mask term (:1829-1831) */
			dla = (float)((double)dla / ((double)(1.0f - s.alpha) + 1e-5)); /* "/ (1.0f - alpha + 1e-5)": fp64 divide (:1829-1832) */
			float da_dE = 0, dE_dsdf = 0, dE_ds = 0, da_dP = 0, dP_ds = 0, dP_dic = 0, dE_dic = 0;
			if (!(s.p_div_c <= 0.0f || s.p_div_c >= 1.0f)) {
				float P = expf(s.inv_s * s.iter_cos * s.dt);
				float E = expf(-s.next_sdf * s.inv_s);
				dE_dsdf = -s.inv_s * E;
				dE_ds = -s.next_sdf * E;
				float a = 1 + E, b = 1 + P * E, cc = (float)(1e-5 + (double)(1 / (1 + P * E))); /* "1e-5 + 1/(...)": fp64 sum (:1862) */
				float delta = a * (b * b) * (cc * cc);
				da_dE = -(P / delta - 1 / (a * a * cc));
				da_dP = -E / delta;
				dP_ds = P * s.iter_cos * s.dt;
				dP_dic = P * s.inv_s * s.dt;
				dE_dic = -s.inv_s * E * s.dt * 0.5f;
			}
			float dl_dinvs = dla * (da_dE * dE_ds + da_dP * dP_ds);
			float dl_dvar = dl_dinvs * s.inv_s * 10;
			float dic_dcos = s.true_cos >= 0 ? 0.0f : 1.0f;
			/* std::sqrt(float sum + 1e-6): the sum of squares is fp32, the offset and the root are fp64 (:1884) */
			float gn = (float)sqrt((double)(s.nrm[0] * s.nrm[0] + s.nrm[1] * s.nrm[1] + s.nrm[2] * s.nrm[2]) + 1e-6);
			float gni = 1 - 1 / gn;
			float dl_dnn = dla * (da_dE * dE_dic + dP_dic * da_dP) * dic_dcos;
			g[3] = loss_scale * (dla * da_dE * dE_dsdf);
			ek += (gn - 1.0f) * (gn - 1.0f);
			for (int e = 0; e < 3; ++e) {
				g[4 + e] = cfg->ek_loss_weight * 2 * cfg->loss_scale * gni * s.nrm[e];
				g[8 + e] = loss_scale * dl_dnn * dir[e];
			}
			g[7] = loss_scale * dl_dvar;
			uint16_t* go = dloss_dout + (size_t)(compacted_base + j) * 16;
			for (int k = 0; k < 16; ++k) go[k] = f2h(g[k]);
		}
		if (ek_loss_out) ek_loss_out[i] = ek / ((float)cn * n_rays_f);
	}
	free(cp);
	free(cbase);
	return total;
}

/* fill_rollover: pad [n_valid, n_target) by wrap-around copies of [0, n_valid) (call sites :3908-3916; body un-vendored) */
/* ---------------------------------------------------------------- inference rendering */

/* ld_random_val, dimension 0 (include/neural-graphics-primitives/random_val.cuh:235-290): hash-based Owen scrambling of
 * the Sobol sequence (Burley 2020) with the Laine-Karras permutation; the Sobol point of an index in dimension 0 is its
 * bit reversal. */
static inline uint32_t reverse_bits(uint32_t x) {
	x = ((x & 0xaaaaaaaau) >> 1) | ((x & 0x55555555u) << 1);
	x = ((x & 0xccccccccu) >> 2) | ((x & 0x33333333u) << 2);
	x = ((x & 0xf0f0f0f0u) >> 4) | ((x & 0x0f0f0f0fu) << 4);
	x = ((x & 0xff00ff00u) >> 8) | ((x & 0x00ff00ffu) << 8);
	return (x >> 16) | (x << 16);
}
static inline uint32_t laine_karras(uint32_t x, uint32_t seed) {
	x += seed;
	x ^= x * 0x6c50b47cu;
	x ^= x * 0xb82f1e52u;
	x ^= x * 0xc7afe638u;
	x ^= x * 0x8d22f6e6u;
	return x;
}
static inline uint32_t owen_scramble(uint32_t x, uint32_t seed) { return reverse_bits(laine_karras(reverse_bits(x), seed)); }
float n2o_ld_random_val(uint32_t index, uint32_t seed) {
	index = owen_scramble(index, seed);
	uint32_t seed0 = seed ^ (0u + (seed << 6) + (seed >> 2)); /* hash_combine(seed, 0) */
	return (float)owen_scramble(reverse_bits(index), seed0) * (float)(1.0 / 4294967296.0);
}

typedef struct {
	float o[3], d[3], t;
	int alive;
} render_ray;

/* init_rays_with_payload_kernel_nerf (src/testbed_nerf.cu:2207-2332) for a pinhole camera, then the jitter of
 * advance_pos_nerf (:812-818).  The walk to the first occupied cell that follows in advance_pos_nerf is the head of the
 * sampling loop below and is done there. */
static void render_init_ray(const n2o_render_cfg* rc, uint32_t x, uint32_t y, render_ray* r) {
	const uint32_t idx = x + rc->width * y;
	const float u = ((float)x + rc->pixel_offset[0]) / (float)rc->width, v = ((float)y + rc->pixel_offset[1]) / (float)rc->height;
	const float dl[3] = {(u - rc->screen_center[0]) * (float)rc->width / rc->focal_length[0],
	                     (v - rc->screen_center[1]) * (float)rc->height / rc->focal_length[1], 1.0f};
	float d[3];
	for (int e = 0; e < 3; ++e) {
		r->o[e] = rc->camera[9 + e];
		d[e] = sum3_eigen(rc->camera[0 + e] * dl[0], rc->camera[3 + e] * dl[1], rc->camera[6 + e] * dl[2]);
	}
	normalize3_eigen(d, r->d);
	float tmin, tmax;
	aabb_ray_intersect(rc->aabb_min, rc->aabb_max, r->o, r->d, &tmin, &tmax);
	float t = fmaxf(tmin, 0.2f) + 1e-6f; /* NERF_RENDERING_NEAR_DISTANCE */
	const float p0[3] = {r->o[0] + r->d[0] * t, r->o[1] + r->d[1] * t, r->o[2] + r->d[2] * t};
	r->alive = aabb_contains(rc->aabb_min, rc->aabb_max, p0);
	if (r->alive) t += n2o_ld_random_val(rc->sample_index, idx * 786433u) * calc_dt(t, rc->cone_angle_constant);
	r->t = t;
}

/* generate_next_nerf_network_inputs (:867-924): up to n_steps samples from the ray's current parameter; returns how many
 * were taken; *left is set when the ray left the box. */
static uint32_t render_next_inputs(const n2o_render_cfg* rc, render_ray* r, const uint8_t* bitfield, uint32_t n_steps, float* coords,
                                   int* left) {
	const float idir[3] = {1.0f / r->d[0], 1.0f / r->d[1], 1.0f / r->d[2]};
	const float cone_angle = rc->cone_angle_constant;
	float t = r->t;
	*left = 0;
	for (uint32_t j = 0; j < n_steps; ++j) {
		float pos[3], dt;
		for (;;) {
			for (int e = 0; e < 3; ++e) pos[e] = r->o[e] + t * r->d[e];
			if (!aabb_contains(rc->aabb_min, rc->aabb_max, pos)) {
				*left = 1;
				return j;
			}
			dt = calc_dt(t, cone_angle);
			uint32_t mip = (uint32_t)mip_from_dt(dt, pos);
			if (occupied_at(pos, bitfield, mip)) break;
			t = advance_to_next_voxel(t, cone_angle, pos, r->d, idir, N2O_GRIDSIZE >> mip);
		}
		if (coords) {
			float* c = coords + (size_t)j * 7;
			for (int e = 0; e < 3; ++e) {
				c[e] = (pos[e] - rc->aabb_min[e]) / (rc->aabb_max[e] - rc->aabb_min[e]);
				c[4 + e] = (r->d[e] + 1.f) * 0.5f;
			}
			c[3] = warp_dt(dt);
		}
		t += dt;
	}
	r->t = t;
	return n_steps;
}

/* Every pixel's whole march (all rounds of NerfTracer::trace, no early termination by opacity), canonical order by pixel
 * index: what the network would be asked for if no ray ever became opaque. */
void n2o_render_march(const n2o_render_cfg* rc, const uint8_t* bitfield, uint64_t max_samples, uint32_t* numsteps, float* coords,
                      uint64_t* n_samples) {
	const uint32_t limit = rc->max_steps ? rc->max_steps : 10000u;
	const int64_t n_pix = (int64_t)rc->width * rc->height;
#pragma omp parallel for schedule(dynamic, 64)
	for (int64_t i = 0; i < n_pix; ++i) {
		render_ray r;
		render_init_ray(rc, (uint32_t)(i % rc->width), (uint32_t)(i / rc->width), &r);
		int left;
		numsteps[i] = r.alive ? render_next_inputs(rc, &r, bitfield, limit, NULL, &left) : 0u;
	}
	uint64_t base = 0;
	for (int64_t i = 0; i < n_pix; ++i) base += numsteps[i];
	*n_samples = base;
	if (!coords || base > max_samples) return;
	uint64_t* bases = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)n_pix);
	base = 0;
	for (int64_t i = 0; i < n_pix; ++i) {
		bases[i] = base;
		base += numsteps[i];
	}
#pragma omp parallel for schedule(dynamic, 64)
	for (int64_t i = 0; i < n_pix; ++i) {
		if (!numsteps[i]) continue;
		render_ray r;
		render_init_ray(rc, (uint32_t)(i % rc->width), (uint32_t)(i / rc->width), &r);
		int left;
		render_next_inputs(rc, &r, bitfield, numsteps[i], coords + bases[i] * 7, &left);
	}
	free(bases);
}

/* Testbed::render_nerf in ERenderMode::Shade (:2671-2812): init_rays_from_camera, the rounds of NerfTracer::trace
 * (:2480-2601: next inputs -> network -> composite_kernel_nerf :926-1171 -> drop finished rays) with 8 steps per round,
 * shade_kernel_nerf (:2147-2180) for the rays whose opacity passed 0.001 (compact_kernel_nerf :2182-2205).  frame is
 * blended into (float[h][w][4]), depth written (float[h][w]). */
void n2o_render_frame(const n2o_grid_desc* d, const uint16_t* params, float sdf_bias, const n2o_render_cfg* rc, const uint8_t* bitfield,
                      float* frame, float* depth, uint64_t* n_samples_out) {
	const uint32_t limit = rc->max_steps ? rc->max_steps : 10000u;
	const int64_t n_pix = (int64_t)rc->width * rc->height;
	const uint32_t R = 8; /* MAX_STEPS_INBETWEEN_COMPACTION */
	render_ray* rays = (render_ray*)malloc(sizeof(render_ray) * (size_t)n_pix);
	float* rgba = (float*)calloc((size_t)n_pix * 4, sizeof(float));
	float* dep = (float*)calloc((size_t)n_pix, sizeof(float));
	float* max_weight = (float*)calloc((size_t)n_pix, sizeof(float));
	uint32_t* taken = (uint32_t*)calloc((size_t)n_pix, sizeof(uint32_t));
	uint32_t* nsteps = (uint32_t*)calloc((size_t)n_pix, sizeof(uint32_t));
	uint32_t* alive_list = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)n_pix);
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < n_pix; ++i) {
		render_init_ray(rc, (uint32_t)(i % rc->width), (uint32_t)(i / rc->width), &rays[i]);
		depth[i] = 1e10f;
	}
	const float cam_fwd[3] = {rc->camera[6], rc->camera[7], rc->camera[8]};
	const float cam_pos[3] = {rc->camera[9], rc->camera[10], rc->camera[11]};
	uint64_t n_samples = 0;
	float* coords = NULL;
	uint16_t* out = NULL;
	size_t cap = 0;
	for (;;) {
		size_t n_alive = 0;
		for (int64_t i = 0; i < n_pix; ++i)
			if (rays[i].alive) alive_list[n_alive++] = (uint32_t)i;
		if (!n_alive) break;
		if (n_alive * R > cap) {
			cap = n_alive * R;
			free(coords);
			free(out);
			coords = (float*)malloc(cap * 7 * sizeof(float));
			out = (uint16_t*)malloc(cap * 16 * sizeof(uint16_t));
		}
		/* like the reference, sample j of ray a sits at a + j * n_alive */
#pragma omp parallel for schedule(dynamic, 64)
		for (int64_t a = 0; a < (int64_t)n_alive; ++a) {
			const uint32_t i = alive_list[a];
			float c8[8 * 7];
			int left;
			uint32_t want = R;
			if (taken[i] + want > limit) want = limit - taken[i];
			nsteps[i] = render_next_inputs(rc, &rays[i], bitfield, want, c8, &left);
			if (want < R) left = 1; /* step budget used up */
			for (uint32_t j = 0; j < nsteps[i]; ++j) memcpy(coords + ((size_t)a + (size_t)j * n_alive) * 7, c8 + j * 7, 28);
			for (uint32_t j = nsteps[i]; j < R; ++j) memset(coords + ((size_t)a + (size_t)j * n_alive) * 7, 0, 28);
			if (left) rays[i].alive = 2; /* leaves after this round's compositing */
		}
		n2o_neus_forward(d, params, sdf_bias, (uint32_t)(n_alive * R), coords, out);
#pragma omp parallel for schedule(dynamic, 64)
		for (int64_t a = 0; a < (int64_t)n_alive; ++a) {
			const uint32_t i = alive_list[a];
			float* px = rgba + (size_t)i * 4;
			uint32_t j = 0;
			for (; j < nsteps[i]; ++j) {
				const size_t k = (size_t)a + (size_t)j * n_alive;
				const uint16_t* o = out + k * 16;
				const float* c = coords + k * 7;
				float dd[3] = {h2f(o[8]) * 2.f - 1.f, h2f(o[9]) * 2.f - 1.f, h2f(o[10]) * 2.f - 1.f}, dir[3];
				const float nn = sqrtf(dd[0] * dd[0] + dd[1] * dd[1] + dd[2] * dd[2]);
				for (int e = 0; e < 3; ++e) dir[e] = dd[e] / nn; /* BENT_DIR (:999-1002) */
				neus_sample_t ns;
				neus_sample(o, c, dir, rc->cos_anneal_ratio, &ns);
				const float T = 1.f - px[3];
				const float weight = ns.alpha * T;
				for (int e = 0; e < 3; ++e) px[e] += ns.rgb[e] * weight;
				px[3] += weight;
				if (weight > max_weight[i]) {
					max_weight[i] = weight;
					float dp = 0.f;
					for (int e = 0; e < 3; ++e) {
						const float pos = c[e] * (rc->aabb_max[e] - rc->aabb_min[e]) + rc->aabb_min[e];
						dp += cam_fwd[e] * (pos - cam_pos[e]);
					}
					dep[i] = dp;
				}
				if (px[3] > 1.0f - rc->min_transmittance) {
					const float w = px[3];
					for (int e = 0; e < 4; ++e) px[e] /= w;
					break;
				}
			}
			taken[i] += nsteps[i];
			if (j < nsteps[i] || rays[i].alive == 2) rays[i].alive = 0;
		}
		for (size_t a = 0; a < n_alive; ++a) n_samples += nsteps[alive_list[a]];
	}
	for (int64_t i = 0; i < n_pix; ++i) {
		float tmp[4] = {rgba[i * 4], rgba[i * 4 + 1], rgba[i * 4 + 2], rgba[i * 4 + 3]};
		if (!(tmp[3] > 0.001f)) continue;
		if (!rc->linear_colors)
			for (int e = 0; e < 3; ++e) tmp[e] = srgb_to_linear(tmp[e]);
		const float k = 1.0f - tmp[3];
		for (int e = 0; e < 4; ++e) frame[i * 4 + e] = tmp[e] + frame[i * 4 + e] * k;
		if (tmp[3] > 0.2f) depth[i] = dep[i];
	}
	if (n_samples_out) *n_samples_out = n_samples;
	free(rays); free(rgba); free(dep); free(max_weight); free(taken); free(nsteps); free(alive_list); free(coords); free(out);
}

/* accumulate_kernel (EColorSpace::Linear) and tonemap_kernel with the identity curve (src/render_buffer.cu:217-259, 474-500) */
void n2o_render_accumulate(uint32_t n_pixels, const float* frame, float* acc, uint32_t sample_count) {
	const float sc = (float)sample_count;
	for (size_t i = 0; i < (size_t)n_pixels * 4; ++i) acc[i] = ((sample_count ? acc[i] : 0.f) * sc + frame[i]) / (sc + 1.f);
}
void n2o_render_tonemap(uint32_t n_pixels, const float* acc, float exposure, const float* background, int to_srgb, float* out) {
	const float bg[3] = {srgb_to_linear(background[0]), srgb_to_linear(background[1]), srgb_to_linear(background[2])};
	const float scale = exp2f(exposure);
	for (size_t i = 0; i < n_pixels; ++i) {
		float c[4] = {acc[i * 4], acc[i * 4 + 1], acc[i * 4 + 2], acc[i * 4 + 3]};
		const float weight = (1.f - c[3]) * background[3];
		for (int e = 0; e < 3; ++e) {
			c[e] = (c[e] + bg[e] * weight) * scale;
			if (to_srgb) c[e] = linear_to_srgb(c[e]);
		}
		c[3] += weight;
		memcpy(out + i * 4, c, 16);
	}
}

void n2o_fill_rollover(uint32_t n_target, uint32_t width, uint32_t n_valid, float* data) {
	if (n_valid == 0 || n_valid >= n_target) return;
	for (size_t i = (size_t)n_valid * width; i < (size_t)n_target * width; ++i) data[i] = data[i % ((size_t)n_valid * width)];
}
/* ... and rescale every element by n_valid/n_target so the duplicated samples do not over-weight the batch */
void n2o_fill_rollover_and_rescale_half(uint32_t n_target, uint32_t width, uint32_t n_valid, uint16_t* data) {
	if (n_valid == 0 || n_valid >= n_target) return;
	float scale = (float)n_valid / (float)n_target;
	size_t nv = (size_t)n_valid * width;
	for (size_t i = nv; i < (size_t)n_target * width; ++i) data[i] = f2h(h2f(data[i % nv]) * scale);
	for (size_t i = 0; i < nv; ++i) data[i] = f2h(h2f(data[i]) * scale);
}

/* ------------------------------------------------------------------ occupancy grid */
/* generate_grid_samples_nerf_nonuniform, src/testbed_nerf.cu:630-659 */
void n2o_occ_generate_samples(uint32_t n, n2o_pcg32 rng0, uint32_t step, const float* aabb_min, const float* aabb_max,
                              const float* grid_in, uint32_t n_cascades, float thresh, float* pos, uint32_t* indices) {
	const uint32_t cells = N2O_GRIDSIZE * N2O_GRIDSIZE * N2O_GRIDSIZE;
#pragma omp parallel for schedule(static)
	for (int64_t ii = 0; ii < (int64_t)n; ++ii) {
		uint32_t i = (uint32_t)ii;
		n2o_pcg32 rng = rng0;
		n2o_pcg32_advance(&rng, (uint64_t)i * 4u);
		uint32_t level = (uint32_t)(n2o_pcg32_next_float(&rng) * (float)n_cascades) % n_cascades;
		uint32_t idx = 0;
		for (uint32_t j = 0; j < 10; ++j) {
			idx = ((i + step * n) * 56924617u + j * 19349663u + 96925573u) % cells;
			idx += level * cells;
			if (grid_in[idx] > thresh) break;
		}
		uint32_t pi = idx % cells;
		uint32_t x = n2o_morton3d_invert(pi >> 0), y = n2o_morton3d_invert(pi >> 1), z = n2o_morton3d_invert(pi >> 2);
		float r[3], c[3] = {(float)x, (float)y, (float)z};
		for (int e = 0; e < 3; ++e) r[e] = n2o_pcg32_next_float(&rng);
		for (int e = 0; e < 3; ++e) {
			float p = ((c[e] + r[e]) / (float)N2O_GRIDSIZE - 0.5f) * scalbnf(1.0f, (int)level) + 0.5f;
			pos[(size_t)i * 3 + e] = (p - aabb_min[e]) / (aabb_max[e] - aabb_min[e]);
		}
		indices[i] = idx;
	}
}

/* sdf_to_density_variance_buffer, common_operation.cuh:310-328: every operation in fp16 */
void n2o_sdf_to_density(uint32_t n, uint16_t variance, uint16_t* sdf_inout) {
	float s = rh(expf(rh(h2f(variance) * 10.0f)));
	for (uint32_t i = 0; i < n; ++i) {
		float sdf = h2f(sdf_inout[i]);
		float sg = rh(logisticf(rh(sdf * s)));
		float dens = rh(rh(s * sg) * rh(1.0f - sg));
		sdf_inout[i] = f2h(dens);
	}
}

/* splat_grid_samples_nerf_max_nearest_neighbor + ema_grid_samples_nerf, src/testbed_nerf.cu:661-730 */
void n2o_occ_splat_ema(uint32_t n_samples, const uint32_t* indices, const uint16_t* density, uint32_t n_cells, float decay,
                       float* grid_tmp, float* grid) {
	memset(grid_tmp, 0, sizeof(float) * (size_t)n_cells);
	uint32_t* tmp = (uint32_t*)grid_tmp;
	for (uint32_t i = 0; i < n_samples; ++i) {
		float v = h2f(density[i]);
		uint32_t bits;
		memcpy(&bits, &v, 4);
		if (bits > tmp[indices[i]]) tmp[indices[i]] = bits; /* atomicMax on the uint pattern */
	}
	for (uint32_t i = 0; i < n_cells; ++i) {
		float prev = grid[i];
		grid[i] = prev < 0.f ? prev : fmaxf(prev * decay, grid_tmp[i]);
	}
}

/* update_density_grid_mean_and_bitfield, src/testbed_nerf.cu:3371-3391; kernels :738-785 */
void n2o_occ_bitfield(uint32_t n_cascades_used, const float* grid, uint8_t* bitfield, float* mean_out) {
	const uint32_t cells = N2O_GRIDSIZE * N2O_GRIDSIZE * N2O_GRIDSIZE;
	double acc = 0.0;
	for (uint32_t i = 0; i < cells; ++i) acc += (double)(fmaxf(grid[i], 0.f) / (float)cells);
	float mean = (float)acc;
	if (mean_out) *mean_out = mean;
	float thresh = fminf(0.1f, mean);
	uint32_t n_bytes = cells / 8 * N2O_CASCADES, n_nonzero = cells / 8 * n_cascades_used;
	for (uint32_t i = 0; i < n_bytes; ++i) {
		uint8_t bits = 0;
		if (i < n_nonzero)
			for (uint32_t j = 0; j < 8; ++j) bits |= grid[(size_t)i * 8 + j] > thresh ? (uint8_t)(1u << j) : 0;
		bitfield[i] = bits;
	}
	for (uint32_t level = 1; level < N2O_CASCADES; ++level) {
		const uint8_t* prev = bitfield + (size_t)(cells / 8) * (level - 1);
		uint8_t* next = bitfield + (size_t)(cells / 8) * level;
		for (uint32_t i = 0; i < cells / 64; ++i) {
			uint8_t bits = 0;
			for (uint32_t j = 0; j < 8; ++j) bits |= prev[(size_t)i * 8 + j] > 0 ? (uint8_t)(1u << j) : 0;
			uint32_t x = n2o_morton3d_invert(i >> 0) + N2O_GRIDSIZE / 8;
			uint32_t y = n2o_morton3d_invert(i >> 1) + N2O_GRIDSIZE / 8;
			uint32_t z = n2o_morton3d_invert(i >> 2) + N2O_GRIDSIZE / 8;
			next[n2o_morton3d(x, y, z)] |= bits;
		}
	}
}

/* ------------------------------------------------------------------ Adam (+ L2, EMA of the weights) */
void n2o_adam_step(const n2o_adam_cfg* c, uint32_t n, const float* grad, float* master, float* m, float* v, uint16_t* params,
                   uint16_t* params_ema, float* ema_master) {
	const float b1 = c->beta1, b2 = c->beta2;
	const float lr = c->learning_rate * sqrtf(1.0f - powf(b2, (float)c->step)) / (1.0f - powf(b1, (float)c->step));
	const float ema_debias_old = 1.0f - powf(c->ema_decay, (float)(c->step - 1));
	const float ema_debias_new = 1.0f / (1.0f - powf(c->ema_decay, (float)c->step));
#pragma omp parallel for schedule(static)
	for (int64_t i = 0; i < (int64_t)n; ++i) {
		float w = master[i];
		float g = grad[i] / c->loss_scale;
		int upd = 1;
		if ((uint32_t)i < c->n_matrix) g += c->l2_reg * w;
		else if (g == 0.0f) upd = 0; /* grid entries no sample touched stay put */
		if (upd) {
			float mi = m[i] = b1 * m[i] + (1.0f - b1) * g;
			float vi = v[i] = b2 * v[i] + (1.0f - b2) * g * g;
			w -= lr * mi / (sqrtf(vi) + c->epsilon);
			master[i] = w;
		}
		params[i] = f2h(w);
		if (params_ema) {
			float e = ((1.0f - c->ema_decay) * w + c->ema_decay * ema_master[i] * ema_debias_old) * ema_debias_new;
			ema_master[i] = e;
			params_ema[i] = f2h(e);
		}
	}
}

/* ------------------------------------------------------------------ marching cubes, canonical (cell-linear) order */
/* The lattice layers z0 .. z0 + nz - 1 of a res[0] x res[1] x res[2] grid (sdf holds only those layers): vertex positions
 * are those of the whole grid, numbering is local to the slab.  counts = {vertices, indices, vertices owned by the layers
 * before the slab's last one, vertices owned by its first layer}. */
void n2o_marching_cubes_slab(const float* aabb_min, const float* aabb_max, const uint32_t res[3], uint32_t z0, uint32_t nz, float thresh,
                             const float* sdf, const int8_t* tri_table, float* verts, uint32_t* indices, uint32_t* counts) {
	const uint32_t rx = res[0], ry = res[1], rz = nz;
	const size_t res2 = (size_t)rx * ry, res3 = res2 * rz;
	int* vgrid = (int*)calloc(res3 * 3, sizeof(int));
	float scale[3] = {(aabb_max[0] - aabb_min[0]) / (float)rx, (aabb_max[1] - aabb_min[1]) / (float)ry,
	                  (aabb_max[2] - aabb_min[2]) / (float)res[2]};
	uint32_t nv = 0, ni = 0, nv_before_last = 0, nv_first = 0;
	/* gen_vertices, src/marching_cubes.cu:276-329 */
	for (uint32_t z = 0; z < rz; ++z) {
		if (z + 1 == rz) nv_before_last = nv;
		if (z == 1) nv_first = nv;
		for (uint32_t y = 0; y < ry; ++y)
			for (uint32_t x = 0; x < rx; ++x) {
				size_t idx = x + (size_t)y * rx + (size_t)z * res2;
				float f0 = sdf[idx];
				int inside = f0 > thresh;
				const size_t step[3] = {1, rx, res2};
				const uint32_t lim[3] = {rx, ry, rz}, p[3] = {x, y, z};
				for (int e = 0; e < 3; ++e) {
					if (p[e] + 1 >= lim[e]) continue;
					float f1 = sdf[idx + step[e]];
					if (inside != (f1 > thresh)) {
						if (verts) {
							float dt = (thresh - f0) / (f1 - f0);
							float q[3] = {(float)x, (float)y, (float)(z + z0)};
							q[e] += dt;
							for (int k = 0; k < 3; ++k) verts[(size_t)nv * 3 + k] = q[k] * scale[k] + aabb_min[k];
						}
						vgrid[idx + res3 * (size_t)e] = (int)nv + 1;
						++nv;
					}
				}
			}
	}
	if (rz == 1) nv_first = nv;
	/* gen_faces, src/marching_cubes.cu:377-718 */
	for (uint32_t z = 0; z + 1 < rz; ++z)
		for (uint32_t y = 0; y + 1 < ry; ++y)
			for (uint32_t x = 0; x + 1 < rx; ++x) {
				size_t idx = x + (size_t)y * rx + (size_t)z * res2;
				size_t ix = idx, iy = idx + res3, iz = idx + res3 * 2;
				int mask = 0;
				if (sdf[idx] > thresh) mask |= 1;
				if (sdf[idx + 1] > thresh) mask |= 2;
				if (sdf[idx + 1 + rx] > thresh) mask |= 4;
				if (sdf[idx + rx] > thresh) mask |= 8;
				if (sdf[idx + res2] > thresh) mask |= 16;
				if (sdf[idx + res2 + 1] > thresh) mask |= 32;
				if (sdf[idx + res2 + 1 + rx] > thresh) mask |= 64;
				if (sdf[idx + res2 + rx] > thresh) mask |= 128;
				if (!mask || mask == 255) continue;
				int le[12] = {vgrid[ix],        vgrid[iy + 1],        vgrid[ix + rx],        vgrid[iy],
				              vgrid[ix + res2], vgrid[iy + 1 + res2], vgrid[ix + rx + res2], vgrid[iy + res2],
				              vgrid[iz],        vgrid[iz + 1],        vgrid[iz + 1 + rx],    vgrid[iz + rx]};
				const int8_t* tri = tri_table + mask * 16;
				for (int i = 0; i < 15; ++i) {
					int j = tri[i];
					if (j < 0) break;
					if (indices) indices[ni] = (uint32_t)(le[j] - 1);
					++ni;
				}
			}
	free(vgrid);
	counts[0] = nv;
	counts[1] = ni;
	counts[2] = nv_before_last;
	counts[3] = nv_first;
}

void n2o_marching_cubes(const float* aabb_min, const float* aabb_max, const uint32_t res[3], float thresh, const float* sdf,
                        const int8_t* tri_table, float* verts, uint32_t* indices, uint32_t* n_verts, uint32_t* n_indices) {
	uint32_t counts[4];
	n2o_marching_cubes_slab(aabb_min, aabb_max, res, 0, res[2], thresh, sdf, tri_table, verts, indices, counts);
	*n_verts = counts[0];
	*n_indices = counts[1];
}

/* --- mesh post-processing (src/marching_cubes.cu:331-375, 720-735, 824-976; src/testbed_nerf.cu:522-535, 838-844, 4057-4080) */

/* accumulate_1ring: ring [n][4] and normals [n][3] (either may be NULL), accumulated in double and rounded once */
void n2o_mesh_1ring(uint32_t n_verts, const float* verts, uint32_t n_indices, const uint32_t* indices, float* ring, float* normals) {
	double* r = (double*)calloc((size_t)n_verts * 4 + 1, sizeof(double));
	double* nr = (double*)calloc((size_t)n_verts * 3 + 1, sizeof(double));
	for (uint32_t t = 0; t + 2 < n_indices; t += 3) {
		const uint32_t id[3] = {indices[t], indices[t + 1], indices[t + 2]};
		const float* p[3] = {verts + (size_t)id[0] * 3, verts + (size_t)id[1] * 3, verts + (size_t)id[2] * 3};
		for (int k = 0; k < 3; ++k) {
			const int a = (k + 1) % 3, b = (k + 2) % 3;
			for (int e = 0; e < 3; ++e) r[(size_t)id[k] * 4 + e] += (double)(p[a][e] + p[b][e]);
			r[(size_t)id[k] * 4 + 3] += 2.0;
		}
		const float u[3] = {p[1][0] - p[0][0], p[1][1] - p[0][1], p[1][2] - p[0][2]};
		const float v[3] = {p[0][0] - p[2][0], p[0][1] - p[2][1], p[0][2] - p[2][2]};
		const float n[3] = {u[1] * v[2] - u[2] * v[1], u[2] * v[0] - u[0] * v[2], u[0] * v[1] - u[1] * v[0]}; /* (pb-pa) x (pa-pc) */
		for (int k = 0; k < 3; ++k)
			for (int e = 0; e < 3; ++e) nr[(size_t)id[k] * 3 + e] += (double)n[e];
	}
	if (ring)
		for (size_t i = 0; i < (size_t)n_verts * 4; ++i) ring[i] = (float)r[i];
	if (normals)
		for (size_t i = 0; i < (size_t)n_verts * 3; ++i) normals[i] = (float)nr[i];
	free(r);
	free(nr);
}

/* compute_mesh_vertex_colors: generate_nerf_network_inputs_from_positions -> network -> extract_srgb_with_activation */
void n2o_mesh_vertex_colors(const n2o_grid_desc* d, const uint16_t* params, float sdf_bias, uint32_t n_verts, const float* verts,
                            const float* aabb_min, const float* aabb_max, int linear_colors, float* colors) {
	float* coords = (float*)calloc((size_t)(n_verts + 1) * 7, sizeof(float));
	uint16_t* out = (uint16_t*)malloc((size_t)(n_verts + 1) * 16 * sizeof(uint16_t));
	for (uint32_t i = 0; i < n_verts; ++i) {
		const float* p = verts + (size_t)i * 3;
		float dd[3] = {p[0] - 0.5f, p[1] - 0.5f, p[2] - 0.5f};
		const float nn = sqrtf(dd[0] * dd[0] + dd[1] * dd[1] + dd[2] * dd[2]);
		float* c = coords + (size_t)i * 7;
		for (int e = 0; e < 3; ++e) {
			if (nn > 0.f) dd[e] /= nn;
			c[e] = (p[e] - aabb_min[e]) / (aabb_max[e] - aabb_min[e]);
			c[4 + e] = (dd[e] + 1.f) * 0.5f;
		}
		c[3] = warp_dt(min_cone_stepsize());
	}
	n2o_neus_forward(d, params, sdf_bias, n_verts, coords, out);
	for (size_t i = 0; i < (size_t)n_verts * 3; ++i) {
		float c = logisticf(h2f(out[(i / 3) * 16 + i % 3]));
		colors[i] = linear_colors ? linear_to_srgb(c) : c;
	}
	free(coords);
	free(out);
}

/* save_mesh without unwrap: the reference's fprintf calls, one after another.  Returns 0 on success. */
int n2o_save_mesh(const char* path, uint32_t n_verts, const float* verts, const float* normals, const float* colors, uint32_t n_indices,
                  const uint32_t* indices, float nerf_scale, const float* nerf_offset, int invert_normals) {
	const size_t len = strlen(path);
	const int ply = len >= 4 && strcmp(path + len - 4, ".ply") == 0;
	FILE* f = fopen(path, "wb");
	if (!f) return -1;
	if (ply)
		fprintf(f,
		        "ply\nformat ascii 1.0\ncomment output from https://github.com/NVlabs/instant-ngp\nelement vertex %u\n"
		        "property float x\nproperty float y\nproperty float z\nproperty float nx\nproperty float ny\nproperty float nz\n"
		        "property uchar red\nproperty uchar green\nproperty uchar blue\nelement face %u\n"
		        "property list uchar int vertex_index\nend_header\n",
		        n_verts, n_indices / 3);
	for (uint32_t i = 0; i < n_verts; ++i) {
		float p[3], n[3];
		const float* v = normals + (size_t)i * 3;
		const float z = v[0] * v[0] + (v[1] * v[1] + v[2] * v[2]); /* Eigen sums three terms as a0 + (a1 + a2) */
		for (int e = 0; e < 3; ++e) {
			p[e] = (verts[(size_t)i * 3 + e] - nerf_offset[e]) / nerf_scale;
			n[e] = z > 0.f ? v[e] / sqrtf(z) : v[e];
		}
		const float* c = colors + (size_t)i * 3;
		if (ply) {
			unsigned char c8[3];
			for (int e = 0; e < 3; ++e) c8[e] = (unsigned char)clampf(c[e] * 255.f, 0.f, 255.f);
			fprintf(f, "%0.5f %0.5f %0.5f %0.3f %0.3f %0.3f %d %d %d\n", p[0], p[1], p[2], n[0], n[1], n[2], c8[0], c8[1], c8[2]);
		} else {
			fprintf(f, "v %0.5f %0.5f %0.5f %0.3f %0.3f %0.3f\n", p[0], p[1], p[2], clampf(c[0], 0.f, 1.f), clampf(c[1], 0.f, 1.f),
			        clampf(c[2], 0.f, 1.f));
		}
	}
	if (!ply)
		for (uint32_t i = 0; i < n_verts; ++i) {
			const float* v = normals + (size_t)i * 3;
			const float z = v[0] * v[0] + (v[1] * v[1] + v[2] * v[2]); /* Eigen sums three terms as a0 + (a1 + a2) */
			const float s = z > 0.f ? sqrtf(z) : 1.f;
			fprintf(f, "vn %0.5f %0.5f %0.5f\n", v[0] / s, v[1] / s, v[2] / s);
		}
	for (uint32_t t = 0; t + 2 < n_indices; t += 3) {
		const uint32_t a = invert_normals ? indices[t] : indices[t + 2], b = indices[t + 1], c = invert_normals ? indices[t + 2] : indices[t];
		if (ply) fprintf(f, "3 %d %d %d\n", (int)a, (int)b, (int)c);
		else fprintf(f, "f %u//%u %u//%u %u//%u\n", a + 1, a + 1, b + 1, b + 1, c + 1, c + 1);
	}
	return fclose(f);
}
