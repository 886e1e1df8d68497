/*
 * CPU restatement of the reference's fused augmentation path.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It exists so that the CUDA kernels can be
 * checked against an independent, slow and obviously-correct statement of the
 * reference's algorithm, and so that a CPU number can be printed next to the
 * GPU number.  Nothing in the shipped package may call it: only the tests,
 * the smoke check and the benchmark's CPU legs load the library built from it.
 *
 * Every function cites the file:line of yuhezhang-ai/triton-augment v0.3.0 it
 * restates (paths are relative to that project's root).
 *
 * Pinned against the reference itself: tests/golden/make_golden.py runs the
 * reference's own Triton kernels (through its own functional.fused_augment)
 * under the Triton CPU interpreter and stores inputs, parameters and outputs;
 * tests/test_oracle_golden.py requires this file to reproduce those outputs
 * bit-for-bit in fp32 (fma_coords = 0, see below) and within 2 fp16 ulp in
 * fp16.
 *
 * Two arithmetic details are selectable because the reference's result depends
 * on how its kernel was compiled:
 *   fma_coords = 0  a*xc + b*yc is two roundings (what the numpy-backed Triton
 *                   interpreter computes);
 *   fma_coords = 1  fma(xc, a, b*yc), the contraction Triton's GPU compiler
 *                   emits for triton_augment/kernels/geometric_kernel.py:414-415
 *                   (bit fields select other contractions per axis, see map_coords).
 * Compile with -ffp-contract=off so that nothing else is contracted.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

typedef _Float16 f16;

enum { TA_ORACLE_F32 = 0, TA_ORACLE_F16 = 1 };
enum { TA_ORACLE_CONTRAST_FAST = 0, TA_ORACLE_CONTRAST_MEAN = 1 };

/* Mirrors the 27-argument launch at triton_augment/functional.py:1399-1431
 * (kernel signature triton_augment/kernels/fused_kernel.py:60-98). */
typedef struct ta_oracle_params {
    int32_t dtype;              /* TA_ORACLE_F32 / TA_ORACLE_F16 (image, factors, mean, std) */
    int32_t n, c, h, w;         /* input  [n, c, h, w], contiguous NCHW */
    int32_t oh, ow;             /* output [n, c, oh, ow] */
    const void *in;
    void *out;
    const float *top;           /* [n] crop offsets as fp32 (functional.py:1383-1384) */
    const float *left;          /* [n] */
    const uint8_t *flip;        /* [n] 0/1 */
    const float *matrix;        /* [n,6] inverse affine rows, NULL <=> has_affine == False */
    float fill;
    int32_t interp;             /* 0 nearest, 1 bilinear (fused_kernel.py:81) */
    int32_t apply_brightness, apply_contrast, apply_saturation, apply_grayscale, apply_normalize;
    const void *brightness;     /* [n] image dtype (functional.py:1335-1337) */
    const void *contrast;       /* [n] */
    const void *saturation;     /* [n] */
    const uint8_t *gray;        /* [n] 0/1 */
    const void *mean;           /* [3] image dtype (functional.py:1350-1354) */
    const void *std;            /* [3] */
    int32_t fma_coords;         /* see file header */
    int32_t contrast_mode;      /* FAST = fused_kernel.py:245-250; MEAN = color_normalize_kernel.py:37-77 */
    const float *gray_mean;     /* [n] per-image mean for contrast_mode MEAN (fp32 holding image-dtype values) */
    int32_t *src_index;         /* optional [n, oh, ow]: y*w+x of the texel nearest/direct sampling read, -1 = fill */
    int32_t threads;            /* 0 = all available */
} ta_oracle_params;

static inline float h_round(float x) { return (float)(f16)x; }

static inline float ld_px(const ta_oracle_params *p, size_t idx)
{
    return p->dtype == TA_ORACLE_F16 ? (float)((const f16 *)p->in)[idx] : ((const float *)p->in)[idx];
}

static inline float ld_vec(const ta_oracle_params *p, const void *v, int i)
{
    return p->dtype == TA_ORACLE_F16 ? (float)((const f16 *)v)[i] : ((const float *)v)[i];
}

/* triton_augment/kernels/fused_kernel.py:239-241: maximum(0, minimum(1, x)). */
static inline float clamp01(float x) { return fmaxf(0.0f, fminf(1.0f, x)); }

/* triton_augment/kernels/geometric_kernel.py:349-420 apply_fused_geometric_transform:
 * flip in output coordinates, add the crop offset, then the inverse affine map
 * in coordinates centred on the INPUT image. */
static inline void map_coords(const ta_oracle_params *p, int n, int xo, int yo, float *x_in, float *y_in)
{
    float x_f = (float)xo, y_f = (float)yo;
    float x_fl = p->flip[n] ? (float)(p->ow - 1) - x_f : x_f;       /* :390 */
    float x_img = x_fl + p->left[n];                                 /* :393 */
    float y_img = y_f + p->top[n];                                   /* :394 */
    if (!p->matrix) { *x_in = x_img; *y_in = y_img; return; }        /* :416-418 */
    const float *m = p->matrix + (size_t)n * 6;                      /* :399-405 */
    float half_w = (float)p->w * 0.5f, half_h = (float)p->h * 0.5f;  /* :408-409 */
    float xc = (x_img - half_w) + 0.5f;                              /* :410 */
    float yc = (y_img - half_h) + 0.5f;                              /* :411 */
    /* a*xc + b*yc (:414-415): which product, if any, the compiler fused into the addition.
     * Bits 0-1 choose for x, bits 2-3 for y: 0 none, 1 fma(xc, a, b*yc), 2 fma(yc, b, a*xc).
     * Bits 4-5 = k: the reference's kernel handles 1024 consecutive output pixels per program
     * with 128 threads, so a thread's j-th pixel is 128 j further on; when its stores are not
     * vectorised the compiler contracts the x expression of a thread's last k pixels the
     * other way (recipe 1).  Those are the pixels whose linear index has bits 7-9 >= 8 - k. */
    int rx = p->fma_coords & 3;
    const int ry = (p->fma_coords >> 2) & 3, late = (p->fma_coords >> 4) & 3;
    if (late) {
        const uint32_t lin = (uint32_t)n * (uint32_t)(p->oh * p->ow) + (uint32_t)(yo * p->ow + xo);
        if ((int)((lin >> 7) & 7u) >= 8 - late) rx = 1;
    }
    float ux = rx == 1 ? fmaf(xc, m[0], m[1] * yc) : rx == 2 ? fmaf(yc, m[1], m[0] * xc) : m[0] * xc + m[1] * yc;
    float uy = ry == 1 ? fmaf(xc, m[3], m[4] * yc) : ry == 2 ? fmaf(yc, m[4], m[3] * xc) : m[3] * xc + m[4] * yc;
    ux = ux + m[2];
    uy = uy + m[5];
    ux = ux + half_w;
    uy = uy + half_h;
    *x_in = ux - 0.5f;
    *y_in = uy - 0.5f;
}

static inline float fill_as_dtype(const ta_oracle_params *p)
{
    return p->dtype == TA_ORACLE_F16 ? h_round(p->fill) : p->fill;
}

/* triton_augment/kernels/geometric_kernel.py:249-283 sample_nearest:
 * round-half-even, bounds test, out-of-bounds -> fill. */
static inline float sample_nearest(const ta_oracle_params *p, size_t base, float x, float y, int32_t *src)
{
    int xn = (int)rintf(x), yn = (int)rintf(y);                      /* :274-275 */
    if (xn >= 0 && xn < p->w && yn >= 0 && yn < p->h) {              /* :278 */
        if (src) *src = yn * p->w + xn;
        return ld_px(p, base + (size_t)yn * p->w + xn);              /* :282-283 */
    }
    if (src) *src = -1;
    return fill_as_dtype(p);
}

/* triton_augment/kernels/geometric_kernel.py:178-246 sample_bilinear:
 * four independently bounds-checked neighbours, fp32 weights and sum, result
 * cast to the image dtype. */
static inline float sample_bilinear(const ta_oracle_params *p, size_t base, float x, float y)
{
    int x0 = (int)floorf(x), y0 = (int)floorf(y);                    /* :202-203 */
    int x1 = x0 + 1, y1 = y0 + 1;
    float dx = x - (float)x0, dy = y - (float)y0;                    /* :208-209 */
    int vx0 = x0 >= 0 && x0 < p->w, vx1 = x1 >= 0 && x1 < p->w;      /* :212-215 */
    int vy0 = y0 >= 0 && y0 < p->h, vy1 = y1 >= 0 && y1 < p->h;
    float f = fill_as_dtype(p);
    float p00 = (vx0 && vy0) ? ld_px(p, base + (size_t)y0 * p->w + x0) : f;   /* :219-236 */
    float p10 = (vx1 && vy0) ? ld_px(p, base + (size_t)y0 * p->w + x1) : f;
    float p01 = (vx0 && vy1) ? ld_px(p, base + (size_t)y1 * p->w + x0) : f;
    float p11 = (vx1 && vy1) ? ld_px(p, base + (size_t)y1 * p->w + x1) : f;
    float w00 = (1.0f - dx) * (1.0f - dy);                           /* :239-242 */
    float w10 = dx * (1.0f - dy);
    float w01 = (1.0f - dx) * dy;
    float w11 = dx * dy;
    float r = p00 * w00 + p10 * w10 + p01 * w01 + p11 * w11;         /* :245 */
    return p->dtype == TA_ORACLE_F16 ? h_round(r) : r;               /* :246 */
}

/* triton_augment/kernels/fused_kernel.py:216-225: crop/flip coordinates are exact
 * integers, truncated to int32 and loaded.  The reference does not bounds-check
 * here; a window outside the image is undefined behaviour there and reads as 0
 * here. */
static inline float sample_direct(const ta_oracle_params *p, size_t base, float x, float y, int32_t *src)
{
    int xi = (int)x, yi = (int)y;
    if (xi >= 0 && xi < p->w && yi >= 0 && yi < p->h) {
        if (src) *src = yi * p->w + xi;
        return ld_px(p, base + (size_t)yi * p->w + xi);
    }
    if (src) *src = -1;
    return 0.0f;
}

/* Colour tier, fp32 images: triton_augment/kernels/fused_kernel.py:234-283. */
static void colour_f32(const ta_oracle_params *p, int n, float *v, int c)
{
    float bf = ld_vec(p, p->brightness, n), cf = ld_vec(p, p->contrast, n), sf = ld_vec(p, p->saturation, n);
    if (p->apply_brightness)                                         /* :235-241 */
        for (int k = 0; k < c; ++k) v[k] = clamp01(v[k] * bf);
    if (p->apply_contrast) {                                         /* :244-250 */
        if (p->contrast_mode == TA_ORACLE_CONTRAST_MEAN) {
            /* triton_augment/kernels/color_normalize_kernel.py:72-74 */
            float m = p->gray_mean[n];
            for (int k = 0; k < c; ++k) v[k] = clamp01(v[k] * cf + m * (1.0f - cf));
        } else {
            for (int k = 0; k < c; ++k) v[k] = clamp01((v[k] - 0.5f) * cf + 0.5f);
        }
    }
    if (p->apply_saturation && c == 3) {                             /* :253-260 */
        float g = 0.2989f * v[0] + 0.587f * v[1] + 0.114f * v[2];
        for (int k = 0; k < 3; ++k) v[k] = clamp01(v[k] * sf + g * (1.0f - sf));
    }
    if (p->apply_grayscale && c == 3 && p->gray[n]) {                /* :263-269 */
        float g = 0.2989f * v[0] + 0.587f * v[1] + 0.114f * v[2];
        v[0] = v[1] = v[2] = g;
    }
    if (p->apply_normalize)                                          /* :272-283 */
        for (int k = 0; k < c; ++k) v[k] = (v[k] - ld_vec(p, p->mean, k)) / ld_vec(p, p->std, k);
}

/* Colour tier, fp16 images.  The reference's GPU build keeps a value in fp16
 * until the first clamp of an enabled op (minimum/maximum against a Python
 * float promote to fp32) and in fp32 from there to the store; factors, mean
 * and std are fp16 values, and (1 - saturation) is an fp16 subtraction.
 * Same source lines as colour_f32. */
static void colour_f16(const ta_oracle_params *p, int n, float *v, int c)
{
    float bf = ld_vec(p, p->brightness, n), cf = ld_vec(p, p->contrast, n), sf = ld_vec(p, p->saturation, n);
    int wide = 0;   /* 0: v[] holds fp16-representable values, ops round to fp16 */
    if (p->apply_brightness) {
        for (int k = 0; k < c; ++k) v[k] = clamp01(h_round(v[k] * bf));
        wide = 1;
    }
    if (p->apply_contrast) {
        if (p->contrast_mode == TA_ORACLE_CONTRAST_MEAN) {
            float m = p->gray_mean[n];
            if (!wide) {
                float omc = h_round(1.0f - cf), mm = h_round(m * omc);
                for (int k = 0; k < c; ++k) v[k] = clamp01(h_round(h_round(v[k] * cf) + mm));
            } else {
                float omc = h_round(1.0f - cf);
                for (int k = 0; k < c; ++k) v[k] = clamp01(v[k] * cf + m * omc);
            }
        } else if (!wide) {
            for (int k = 0; k < c; ++k)
                v[k] = clamp01(h_round(h_round(h_round(v[k] - 0.5f) * cf) + 0.5f));
        } else {
            for (int k = 0; k < c; ++k) v[k] = clamp01((v[k] - 0.5f) * cf + 0.5f);
        }
        wide = 1;
    }
    if (p->apply_saturation && c == 3) {
        float oms = h_round(1.0f - sf);
        if (!wide) {
            float g = h_round(h_round(h_round(h_round(0.2989f) * v[0]) + h_round(h_round(0.587f) * v[1]))
                              + h_round(h_round(0.114f) * v[2]));
            float gg = h_round(g * oms);
            for (int k = 0; k < 3; ++k) v[k] = clamp01(h_round(h_round(v[k] * sf) + gg));
        } else {
            float g = 0.2989f * v[0] + 0.587f * v[1] + 0.114f * v[2];
            for (int k = 0; k < 3; ++k) v[k] = clamp01(v[k] * sf + g * oms);
        }
        wide = 1;
    }
    if (p->apply_grayscale && c == 3 && p->gray[n]) {
        float g;
        if (!wide)
            g = h_round(h_round(h_round(h_round(0.2989f) * v[0]) + h_round(h_round(0.587f) * v[1]))
                        + h_round(h_round(0.114f) * v[2]));
        else
            g = 0.2989f * v[0] + 0.587f * v[1] + 0.114f * v[2];
        v[0] = v[1] = v[2] = g;
    }
    if (p->apply_normalize) {
        for (int k = 0; k < c; ++k) {
            float m = ld_vec(p, p->mean, k), s = ld_vec(p, p->std, k);
            v[k] = wide ? (v[k] - m) / s : h_round(h_round(v[k] - m) / s);
        }
    }
}

static void fused_rows(const ta_oracle_params *p, long row0, long row1)
{
    const int c = p->c;
    const size_t in_plane = (size_t)p->h * p->w, out_plane = (size_t)p->oh * p->ow;
    for (long row = row0; row < row1; ++row) {
        int n = (int)(row / p->oh), yo = (int)(row % p->oh);
        for (int xo = 0; xo < p->ow; ++xo) {
            float x_in, y_in, v[3];
            map_coords(p, n, xo, yo, &x_in, &y_in);
            int32_t *src = p->src_index ? p->src_index + (size_t)n * out_plane + (size_t)yo * p->ow + xo : NULL;
            for (int k = 0; k < c; ++k) {
                size_t base = ((size_t)n * c + k) * in_plane;        /* fused_kernel.py:200-203 */
                if (!p->matrix)          v[k] = sample_direct(p, base, x_in, y_in, k == 0 ? src : NULL);
                else if (p->interp == 0) v[k] = sample_nearest(p, base, x_in, y_in, k == 0 ? src : NULL);
                else                     v[k] = sample_bilinear(p, base, x_in, y_in);
            }
            if (p->dtype == TA_ORACLE_F16) colour_f16(p, n, v, c); else colour_f32(p, n, v, c);
            for (int k = 0; k < c; ++k) {
                size_t o = ((size_t)n * c + k) * out_plane + (size_t)yo * p->ow + xo;   /* :286-293 */
                if (p->dtype == TA_ORACLE_F16) ((f16 *)p->out)[o] = (f16)v[k];
                else ((float *)p->out)[o] = v[k];
            }
        }
    }
}

typedef struct { const ta_oracle_params *p; long row0, row1; } row_job;

static void *fused_rows_thread(void *arg)
{
    row_job *j = (row_job *)arg;
    fused_rows(j->p, j->row0, j->row1);
    return NULL;
}

int ta_oracle_max_threads(void)
{
    long k = sysconf(_SC_NPROCESSORS_ONLN);
    return k > 0 ? (int)k : 1;
}

/* The whole pass: triton_augment/kernels/fused_kernel.py:159-376.  The reference's
 * SPATIAL (:161-293) and LINEAR (:295-376) paths differ only in how threads are
 * indexed; per output element they compute the same thing, so one loop nest
 * covers both. */
int ta_oracle_fused_augment(const ta_oracle_params *p)
{
    if (!p || !p->in || !p->out || !p->top || !p->left || !p->flip) return -1;
    if (p->c != 1 && p->c != 3) return -2;
    if (p->n < 0 || p->h <= 0 || p->w <= 0 || p->oh <= 0 || p->ow <= 0) return -3;
    if ((p->apply_saturation || p->apply_grayscale) && p->c != 3) return -4;
    if (p->apply_contrast && p->contrast_mode == TA_ORACLE_CONTRAST_MEAN && !p->gray_mean) return -5;
    long rows = (long)p->n * p->oh;
    int nt = p->threads > 0 ? p->threads : ta_oracle_max_threads();
    if (nt > 256) nt = 256;
    if ((long)nt > rows) nt = rows > 0 ? (int)rows : 1;
    if (nt <= 1) { fused_rows(p, 0, rows); return 0; }
    pthread_t tid[256];
    row_job job[256];
    int started = 0;
    for (int t = 0; t < nt; ++t) {
        job[t].p = p;
        job[t].row0 = rows * t / nt;
        job[t].row1 = rows * (t + 1) / nt;
        if (pthread_create(&tid[t], NULL, fused_rows_thread, &job[t]) != 0) break;
        ++started;
    }
    for (int t = started; t < nt; ++t) fused_rows(p, job[t].row0, job[t].row1);   /* could not spawn: do it here */
    for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
    return 0;
}

/* Per-image grayscale mean that torchvision-exact contrast blends towards:
 * triton_augment/functional.py:366-376 (rgb_to_grayscale -> torch.mean over
 * C,H,W -> cast to the image dtype) with the grayscale formula of
 * triton_augment/kernels/color_normalize_kernel.py:248.  Inside the fused
 * pipeline the image whose mean is taken is the output of geometry followed by
 * brightness (what adjust_contrast would be handed in a sequential pipeline),
 * so this walks the same samples as the main pass.  Accumulates in double and
 * rounds once.  mean_out is fp32 holding image-dtype-representable values. */
int ta_oracle_gray_mean(const ta_oracle_params *p, float *mean_out)
{
    if (!p || !mean_out) return -1;
    if (p->c != 1 && p->c != 3) return -2;
    const int c = p->c;
    const size_t in_plane = (size_t)p->h * p->w;
    for (int n = 0; n < p->n; ++n) {
        double acc = 0.0;
        float bf = ld_vec(p, p->brightness, n);
        for (int yo = 0; yo < p->oh; ++yo)
            for (int xo = 0; xo < p->ow; ++xo) {
                float x_in, y_in, v[3];
                map_coords(p, n, xo, yo, &x_in, &y_in);
                for (int k = 0; k < c; ++k) {
                    size_t base = ((size_t)n * c + k) * in_plane;
                    if (!p->matrix)          v[k] = sample_direct(p, base, x_in, y_in, NULL);
                    else if (p->interp == 0) v[k] = sample_nearest(p, base, x_in, y_in, NULL);
                    else                     v[k] = sample_bilinear(p, base, x_in, y_in);
                    if (p->apply_brightness)
                        v[k] = clamp01(p->dtype == TA_ORACLE_F16 ? h_round(v[k] * bf) : v[k] * bf);
                }
                float g = c == 3 ? 0.2989f * v[0] + 0.587f * v[1] + 0.114f * v[2] : v[0];
                if (p->dtype == TA_ORACLE_F16) g = h_round(g);       /* rgb_to_grayscale stores image dtype */
                acc += (double)g;
            }
        float m = (float)(acc / ((double)p->oh * (double)p->ow));
        mean_out[n] = p->dtype == TA_ORACLE_F16 ? h_round(m) : m;
    }
    return 0;
}

/* triton_augment/functional.py:824-892 _get_inverse_affine_matrix, evaluated in
 * fp32 with libm.  The product never uses this (its matrices come from the same
 * torch ops as the reference's so that both kernels see identical inputs); the
 * tests use it to cross-check those torch ops to a tolerance. */
void ta_oracle_inverse_affine_matrix(int n, const float *center, const float *angle, const float *translate,
                                     const float *scale, const float *shear, float *matrix)
{
    const float d2r = (float)(3.141592653589793 / 180.0);
    for (int i = 0; i < n; ++i) {
        float rot = angle[i] * d2r, sx = shear[2 * i] * d2r, sy = shear[2 * i + 1] * d2r;
        float cx = center[2 * i], cy = center[2 * i + 1], tx = translate[2 * i], ty = translate[2 * i + 1];
        float cos_sy = cosf(sy);
        float a = cosf(rot - sy) / cos_sy;
        float b = -cosf(rot - sy) * tanf(sx) / cos_sy - sinf(rot);
        float c = sinf(rot - sy) / cos_sy;
        float d = -sinf(rot - sy) * tanf(sx) / cos_sy + cosf(rot);
        float m0 = d / scale[i], m1 = -b / scale[i], m3 = -c / scale[i], m4 = a / scale[i];
        float m2 = m0 * (-cx - tx) + m1 * (-cy - ty);
        float m5 = m3 * (-cx - tx) + m4 * (-cy - ty);
        float *m = matrix + 6 * (size_t)i;
        m[0] = m0; m[1] = m1; m[2] = m2 + cx; m[3] = m3; m[4] = m4; m[5] = m5 + cy;
    }
}
