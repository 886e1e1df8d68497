// Source footprint of one output tile under flip -> crop offset -> inverse affine.
//
// The staged affine kernel copies the source rows an output tile touches into shared
// memory: one window of columns for all rows when the footprint's bounding box fits it,
// otherwise a window per group of 8 rows that follows the footprint.  This header computes
// the rows and the windows.  It is plain arithmetic shared by the device code and by a
// host-side test hook, so the windows can be checked on a CPU against a brute force walk
// over the tile's pixels.
//
// Geometry restated from triton_augment/kernels/geometric_kernel.py:386-415: an
// output pixel (x, y) maps to x_img = (flip ? ow-1-x : x) + left, y_img = y + top,
// is centred on the input image, multiplied by the 2x3 inverse matrix and
// un-centred.  The map is affine, so a tile (a rectangle) lands on a
// parallelogram; the rows a sampling mode reads from it form a slab in source y,
// and rectangle-intersect-slab is a convex polygon whose extreme source x lie on
// the rectangle's edges.
#pragma once

#if defined(__CUDACC__)
#define TA_HD __host__ __device__ __forceinline__
#else
#define TA_HD inline
#endif

#include <math.h>

namespace ta {

constexpr int kTileW = 64;       // output tile width, pixels
// Output tile height, and the number of source rows one staged tile may span (12 groups of 8):
// a 64 x 64 tile under +-15 degrees of rotation, 5 degrees of shear and scale 0.9 reads ~90 rows.
constexpr int kTileH = 64, kMaxRows = 96;
// The short tile shape of small outputs (64 x 32 pixels, 64 source rows): two thirds of the stage,
// so that the ring holds one stage more than with the tall shape.
constexpr int kTileHShort = 32, kMaxRowsShort = 64;
TA_HD int max_rows_of(int tile_h) { return tile_h == kTileHShort ? kMaxRowsShort : kMaxRows; }
constexpr int kGroupRows = 8;    // rows fetched by one tensor copy
// Staged row pitch = width of every tensor-copy box, in elements.  A pitch that is a multiple
// of 32 words keeps lanes of one warp that sit in different source rows on different banks
// (narrower boxes of 72 / 80 elements were tried: less L2 traffic, but 2-way bank conflicts cost
// more than they saved).  Two-byte elements: 128 (64 words); with 96 (48 words) the lanes of a
// warp, which cover 64 neighbouring columns in pairs, met 2-way conflicts on a third of their
// loads under rotation.  One-byte elements need 128: a copy starts on a 16-byte boundary, i.e.
// up to 15 columns left of the footprint, and a 64-pixel tile under +-15 degrees and scale 1.1
// already spans ~85 columns.  (144 was tried for bytes, to spread rows over the banks: fewer
// conflicts, no gain - the byte kernels are bound by instruction issue.)
constexpr int kPitch = 96;
constexpr int kPitchBytes2 = 128;
constexpr int kPitchBytes1 = 128;
TA_HD int pitch_of(int elem_bytes) { return elem_bytes == 1 ? kPitchBytes1 : elem_bytes == 2 ? kPitchBytes2 : kPitch; }
constexpr float kEps = 1.0f / 64.0f;   // slack (pixels) for the fp32 evaluation of coordinates
constexpr float kCoordLimit = 1.0e6f;  // tiles whose source coordinates exceed this are not staged

struct TileFootprint {
    float sx[4], sy[4];   // source coordinates of the tile's corners (x0y0, x1y0, x1y1, x0y1)
    float inv[4];         // 1 / (sy[j] - sy[i]) per edge, 0 when the edge is level (tile_edges())
    float xmin, xmax;     // extreme source x of the corners
    float dx, dy;         // extent of the tile in centred output coordinates
    int row0;             // first source row
    int rows;             // number of source rows (0 = do not stage)
};

// Corners, rows and bounding box.  mode: 0 nearest (reads row rint(sy)), 1 bilinear (reads rows
// floor(sy), floor(sy)+1).  rows == 0 on return: the tile is not staged.
TA_HD void tile_footprint(TileFootprint &t, int mode, int h, int w, int oh, int ow,
                          float top, float left, bool flip, const float *m, int tile_x, int tile_y,
                          int tile_h = kTileH, int max_rows = kMaxRows)
{
    const int x_first = tile_x * kTileW, y_first = tile_y * tile_h;
    const int x_last = (x_first + kTileW < ow ? x_first + kTileW : ow) - 1;
    const int y_last = (y_first + tile_h < oh ? y_first + tile_h : oh) - 1;
    const float half_w = 0.5f * (float)w, half_h = 0.5f * (float)h;
    const float xi0 = (float)(flip ? ow - 1 - x_last : x_first) + left;
    const float xi1 = (float)(flip ? ow - 1 - x_first : x_last) + left;
    const float xc0 = xi0 - half_w + 0.5f, xc1 = xi1 - half_w + 0.5f;
    const float yc0 = (float)y_first + top - half_h + 0.5f, yc1 = (float)y_last + top - half_h + 0.5f;
    const float cx[4] = {xc0, xc1, xc1, xc0}, cy[4] = {yc0, yc0, yc1, yc1};
    float ymin = INFINITY, ymax = -INFINITY, xmin = INFINITY, xmax = -INFINITY;
    // Per corner and written so that a NaN fails (fminf/fmaxf drop NaNs).
    bool sane = true;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        t.sx[i] = (m[0] * cx[i] + m[1] * cy[i] + m[2]) + half_w - 0.5f;
        t.sy[i] = (m[3] * cx[i] + m[4] * cy[i] + m[5]) + half_h - 0.5f;
        ymin = fminf(ymin, t.sy[i]); ymax = fmaxf(ymax, t.sy[i]);
        xmin = fminf(xmin, t.sx[i]); xmax = fmaxf(xmax, t.sx[i]);
        sane = sane && fabsf(t.sx[i]) < kCoordLimit && fabsf(t.sy[i]) < kCoordLimit;
    }
    t.xmin = xmin; t.xmax = xmax;
    t.dx = xc1 - xc0; t.dy = yc1 - yc0;
    t.rows = 0;
    t.row0 = 0;
    if (!sane) return;
    int r0, r1;
    if (mode == 0) { r0 = (int)ceilf(ymin - kEps - 0.5f); r1 = (int)floorf(ymax + kEps + 0.5f); }
    else           { r0 = (int)floorf(ymin - kEps);       r1 = (int)floorf(ymax + kEps) + 1; }
    const int rows = r1 - r0 + 1;
    if (rows < 1 || rows > max_rows) return;
    t.row0 = r0;
    t.rows = rows;
}

// floor / ceil of a column to a multiple of `chunk`, valid for negative columns
TA_HD int chunk_floor(int c, int chunk) { return (c >= 0 ? c / chunk : -((-c + chunk - 1) / chunk)) * chunk; }
TA_HD int chunk_ceil(int c, int chunk) { return (c >= 0 ? (c + chunk - 1) / chunk : -((-c) / chunk)) * chunk; }

// Inclusive column range read around source x in [lo, hi].
TA_HD void column_range(int mode, float lo, float hi, int &c0, int &c1)
{
    if (mode == 0) { c0 = (int)ceilf(lo - kEps - 0.5f); c1 = (int)floorf(hi + kEps + 0.5f); }
    else           { c0 = (int)floorf(lo - kEps);       c1 = (int)floorf(hi + kEps) + 1; }
}

// The common case: one window of `pitch` columns starting at xs (a multiple of `chunk`) covers
// every row the tile reads, i.e. the bounding box of the corners fits.
TA_HD bool tile_window(const TileFootprint &t, int mode, int chunk, int pitch, int &xs)
{
    int c0, c1;
    column_range(mode, t.xmin, t.xmax, c0, c1);
    xs = chunk_floor(c0, chunk);
    return c1 + 1 - xs <= pitch;
}

// Crop / flip without a matrix: source pixel = (int)(x_img), (int)(y_img) (truncation, as the
// crop kernels do), monotone in x and y, so the tile's first and last pixel give the exact
// range.  Fills xmin / xmax / row0 / rows only; the window always exists (a tile is kTileW wide).
TA_HD void tile_footprint_crop(TileFootprint &t, int oh, int ow, float top, float left, bool flip, int tile_x, int tile_y,
                               int tile_h = kTileH, int max_rows = kMaxRows)
{
    const int x_first = tile_x * kTileW, y_first = tile_y * tile_h;
    const int x_last = (x_first + kTileW < ow ? x_first + kTileW : ow) - 1;
    const int y_last = (y_first + tile_h < oh ? y_first + tile_h : oh) - 1;
    const float xa = (float)(flip ? ow - 1 - x_last : x_first) + left;
    const float xb = (float)(flip ? ow - 1 - x_first : x_last) + left;
    const float ya = (float)y_first + top, yb = (float)y_last + top;
    t.rows = 0;
    t.row0 = 0;
    t.xmin = t.xmax = 0.0f;
    if (!(fabsf(xa) < kCoordLimit && fabsf(xb) < kCoordLimit && fabsf(ya) < kCoordLimit && fabsf(yb) < kCoordLimit)) return;
    t.xmin = (float)(int)xa;
    t.xmax = (float)(int)xb;
    const int r0 = (int)ya, r1 = (int)yb;
    if (r1 - r0 + 1 > max_rows) return;
    t.row0 = r0;
    t.rows = r1 - r0 + 1;
}

TA_HD bool tile_window_crop(const TileFootprint &t, int chunk, int pitch, int &xs)
{
    xs = chunk_floor((int)t.xmin, chunk);
    return (int)t.xmax + 1 - xs <= pitch;
}

// Otherwise rows are fetched in groups with a window each; this prepares the per-edge terms
// tile_rows_range() needs and checks that no group can be wider than a window.  Inside a slab
// of height s in source y, eliminating yc gives sx = (a - b d / e) xc + (b / e) sy + const and
// eliminating xc gives sx = (b - a e / d) yc + (a / d) sy + const; either bounds a row's span.
TA_HD bool tile_edges(TileFootprint &t, int mode, int chunk, int pitch, const float *m)
{
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float d = t.sy[(i + 1) & 3] - t.sy[i];
        t.inv[i] = d != 0.0f ? 1.0f / d : 0.0f;
    }
    const float s = (mode == 0 ? 1.0f : 2.0f) + 2.0f * kEps;
    float span = t.xmax - t.xmin;
    if (m[4] != 0.0f) span = fminf(span, fabsf(m[0] - m[1] * m[3] / m[4]) * t.dx + fabsf(m[1] / m[4]) * s);
    if (m[3] != 0.0f) span = fminf(span, fabsf(m[1] - m[0] * m[4] / m[3]) * t.dy + fabsf(m[0] / m[3]) * s);
    // + 2 eps, + the second tap / rounding to nearest, + rounding both ends to whole chunks
    return span + 2.0f * kEps + 2.0f + 2.0f * (float)(chunk - 1) <= (float)pitch;
}

// Columns [xs, xe) of source rows row0 + r_first .. row0 + r_last that the tile reads, rounded
// outward to whole chunks: the pixels that read any of these rows lie in one slab of the
// parallelogram, which is clipped against its edges.  xs is a multiple of `chunk` (floor
// division, so also for negative columns).  Returns false (and xe == xs == 0) when no pixel
// reads the rows.  Needs tile_edges() first.
TA_HD bool tile_rows_range(const TileFootprint &t, int mode, int chunk, int r_first, int r_last, int &xs, int &xe)
{
    const float ya = (float)(t.row0 + r_first) - (mode == 0 ? 0.5f : 1.0f) - kEps;
    const float yb = (float)(t.row0 + r_last) + (mode == 0 ? 0.5f : 1.0f) + kEps;
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = (i + 1) & 3;
        const float yi = t.sy[i], yj = t.sy[j];
        if ((yi < ya && yj < ya) || (yi > yb && yj > yb)) continue;
        float t0 = 0.0f, t1 = 1.0f;
        if (t.inv[i] != 0.0f) {
            const float ta = (ya - yi) * t.inv[i], tb = (yb - yi) * t.inv[i];
            t0 = fmaxf(0.0f, fminf(ta, tb));
            t1 = fminf(1.0f, fmaxf(ta, tb));
            if (!(t0 <= t1)) continue;
        }
        const float dxs = t.sx[j] - t.sx[i];
        const float xa = t.sx[i] + t0 * dxs, xb = t.sx[i] + t1 * dxs;
        lo = fminf(lo, fminf(xa, xb));
        hi = fmaxf(hi, fmaxf(xa, xb));
    }
    if (!(lo <= hi)) { xs = 0; xe = 0; return false; }
    int c0, c1;   // inclusive column range
    column_range(mode, lo, hi, c0, c1);
    xs = chunk_floor(c0, chunk);
    xe = chunk_ceil(c1 + 1, chunk);
    return true;
}

// What is actually fetched.  Window case: all rows, `pitch` columns from *group_xs.  Otherwise
// rows in groups of kGroupRows, every group `pitch` columns from the smallest xs of its rows
// (group_xs has max_rows / kGroupRows entries).  Scalar restatement of the producer warp's
// decisions; returns false when the tile is not staged.
TA_HD bool tile_plan(TileFootprint &t, int mode, int chunk, int pitch, const float *m, int *group_xs, bool *window,
                     int max_rows = kMaxRows)
{
    if (t.rows == 0) return false;
    int xs;
    *window = tile_window(t, mode, chunk, pitch, xs);
    if (*window) {
        for (int g = 0; g < max_rows / kGroupRows; ++g) group_xs[g] = xs;
        return true;
    }
    if (!tile_edges(t, mode, chunk, pitch, m)) return false;
    for (int g = 0; g < max_rows / kGroupRows; ++g) {
        int lo = 0, hi = chunk;
        const int r_first = g * kGroupRows;
        const int r_last = r_first + kGroupRows - 1 < t.rows - 1 ? r_first + kGroupRows - 1 : t.rows - 1;
        if (r_first >= t.rows || !tile_rows_range(t, mode, chunk, r_first, r_last, lo, hi)) { lo = 0; hi = chunk; }
        if (hi - lo > pitch) return false;
        group_xs[g] = lo;
    }
    return true;
}

}  // namespace ta
