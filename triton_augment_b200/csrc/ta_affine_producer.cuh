// Producer role of the staged affine kernel.  There is one producer warp per stage of the
// ring: warp p fills stage p for the CTA's tiles p, p + stages, p + 2 stages, ...
//
// Per tile the warp (1) works out the source footprint and writes the tile's descriptor, (2)
// waits until the consumers have released the stage, (3) issues the copies.  Only (3) sits
// between "stage free" and "data on its way", so it is kept to one tensor copy per channel in
// the common case; everything else is done ahead of the wait.
#pragma once

namespace ta {

// Two-phase kernel (TWO): the tile sequence of a launch interleaves, image by image, the tiles
// of the grayscale-mean reduction (phase 1) with the tiles of the fused pass (phase 0) of the
// image before: R(0) | R(1) F(0) | R(2) F(1) | ... | F(n-1).  An F tile needs its image's mean,
// which the consumer warp that writes the image's last partial sum finishes; every CTA meets its
// own R tiles of an image before its F tiles of that image, so with all CTAs resident (the
// launch is cooperative) the wait below always ends - and it is bounded like every other wait.
// lag: how many images the fused pass runs behind the reduction (<= the number of images).
// r_start: where the reduction tiles of image n begin in the sequence (they are tpi consecutive numbers).
__device__ __forceinline__ void two_phase_tile(int v, int n_images, int tpi, int lag, int &phase, int &n, int &t, int &r_start)
{
    const int head = lag * tpi, tail_start = head + (n_images - lag) * 2 * tpi;
    if (v < head) { phase = 1; n = v / tpi; t = v - n * tpi; r_start = n * tpi; }
    else if (v < tail_start) {
        const int u = v - head, slot = u / (2 * tpi), w = u - slot * 2 * tpi;
        if (w < tpi) { phase = 1; n = lag + slot; t = w; r_start = v - w; }
        else         { phase = 0; n = slot; t = w - tpi; r_start = 0; }
    } else {
        const int u = v - tail_start, q = u / tpi;
        phase = 0; n = n_images - lag + q; t = u - q * tpi; r_start = 0;
    }
}


template <typename T, int C, int MODE, unsigned F, typename S, bool TWO, int TH>
__device__ __forceinline__ void affine_producer(const KArgs &k, const TMaps &maps, unsigned char *smem,
                                                uint64_t *full, uint64_t *empty, volatile int *abort_flag, int p)
{
    using Info = TileInfo<T, C, F, TH>;
    using Smem = AffineSmem<T, C, F, S, TH>;
    constexpr int CH = Src<S>::chunk, PITCH = Src<S>::pitch, PLANE = Stage<S, TH>::plane;
    constexpr int STAGES = Ring<S, TH>::stages;
    constexpr int TILE_H = Shape<TH>::H, MAX_ROWS = Shape<TH>::ROWS, GROUPS = Shape<TH>::GROUPS;
    static_assert(GROUPS <= 32 && GROUPS <= kNumGroups && MAX_ROWS % kGroupRows == 0, "one lane per row group");
    const int lane = threadIdx.x & 31;
    const int tiles_per_img = k.tiles_x * k.tiles_y;
    S *stage = reinterpret_cast<S *>(smem + p * Smem::stage);
    unsigned long long n_staged = 0, n_direct = 0;
    int cur_n = -1;
    Geom g;
    Colour<T, C, F> col;

    // Tile number -> (image, tile row, tile column), then stepped by STAGES * gridDim.x tiles per
    // round with carries instead of divisions.  Consecutive tile numbers are neighbours along x:
    // the CTAs running at one time then read whole runs of image rows (DRAM page hits) and share
    // the overlap of their boxes in L2; an order that interleaves images was 20-50 % slower.
    const int first = (int)blockIdx.x + p * (int)gridDim.x, step = STAGES * (int)gridDim.x;
    int n = first / tiles_per_img, ty = (first % tiles_per_img) / k.tiles_x, tx = (first % tiles_per_img) % k.tiles_x;
    const int step_n = step / tiles_per_img, step_ty = (step % tiles_per_img) / k.tiles_x,
              step_tx = (step % tiles_per_img) % k.tiles_x;

    int use = 0;
    for (int tile = first; tile < k.num_tiles; tile += step, ++use) {
        int phase = 0, real_tile = tile, r_count = 0;
        if constexpr (TWO) {
            int t, r_start;
            two_phase_tile(tile, k.n, tiles_per_img, min(k.mean_lag, k.n), phase, n, t, r_start);
            if (phase == 1 && tile + (int)gridDim.x >= r_start + tiles_per_img) {
                // this CTA's last reduction tile of the image: tell the consumers, and how many there were
                const int first_own = r_start + (((int)blockIdx.x - r_start) % (int)gridDim.x + (int)gridDim.x) % (int)gridDim.x;
                r_count = (tile - first_own) / (int)gridDim.x + 1;
            }
            ty = t / k.tiles_x;
            tx = t - ty * k.tiles_x;
            real_tile = n * tiles_per_img + t;
            if (2 * n + phase != cur_n) {
                load_geom(g, k, n, MODE != 0);
                if (phase == 0) {
                    // the image's mean must be final (written by another SM: volatile flag, then a fence)
                    int ok = 1;
                    if (lane == 0) {
                        const volatile unsigned *ready = k.mean_ready + n;
                        ok = *ready != 0u;
                        if (!ok) {
                            const unsigned long long t0 = global_ns();
                            for (int i = 0; i < (1 << 24) && !ok; ++i) {
                                ok = *ready != 0u;
                                if (!ok && (i & 63) == 63 && (*abort_flag || global_ns() - t0 > k.wait_ns)) break;
                            }
                        }
                        __threadfence();
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) { *abort_flag = 1; return; }
                }
                col.init(k, n);             // (phase 1 reads no mean: brightness only)
                cur_n = 2 * n + phase;
            }
        } else if (n != cur_n) {                            // per-image parameters: reload on change only
            load_geom(g, k, n, MODE != 0);
            col.init(k, n);
            cur_n = n;
        }
        Info *ti = reinterpret_cast<Info *>(smem + STAGES * Smem::stage + (size_t)(p + STAGES * (use & 1)) * Smem::info);

        // ---- (1) footprint and descriptor
        TileFootprint fp;
        fp.rows = 0;
        fp.row0 = 0;
        const float m[6] = {g.a, g.b, g.c, g.d, g.e, g.f};
        constexpr int FMODE = MODE == 2 ? 1 : 0;            // footprint rule: nearest or bilinear
        if (k.staged_ok) {
            if (MODE == 0) tile_footprint_crop(fp, k.oh, k.ow, g.top, g.left, g.flip, tx, ty, TILE_H, MAX_ROWS);
            else tile_footprint(fp, FMODE, k.h, k.w, k.oh, k.ow, g.top, g.left, g.flip, m, tx, ty, TILE_H, MAX_ROWS);
        }
        bool staged = fp.rows > 0, window = false;
        int gxs = 0;
        const int ngroups = (fp.rows + kGroupRows - 1) / kGroupRows;
        if (staged) {
            window = MODE == 0 ? tile_window_crop(fp, CH, PITCH, gxs) : tile_window(fp, FMODE, CH, PITCH, gxs);
            bool inside;
            if (MODE == 0) {
                staged = window;              // zero outside the image is the crop kernels' rule too
                inside = true;
            } else if (window) {
                int c0, c1;
                column_range(FMODE, fp.xmin, fp.xmax, c0, c1);
                inside = c0 >= 0 && c1 < k.w;
            } else {
                // lanes 0 .. GROUPS-1: columns of row group `lane`; the other lanes hold a neutral entry
                staged = tile_edges(fp, FMODE, CH, PITCH, m);
                int xs = 0, xe = CH;
                const int r_first = lane * kGroupRows, r_last = min(r_first + kGroupRows, fp.rows) - 1;
                const bool have = staged && lane < ngroups && tile_rows_range(fp, FMODE, CH, r_first, r_last, xs, xe);
                if (!have) { xs = 0; xe = CH; }
                gxs = xs;
                staged = staged && __all_sync(0xffffffffu, xe - xs <= PITCH);
                inside = __all_sync(0xffffffffu, !have || (xs >= 0 && xe <= k.w));
                if (staged) {
                    // rowoff[r] = r * PITCH - (first column of r's group); rows lane, lane + 32, ...
#pragma unroll
                    for (int base = 0; base < MAX_ROWS; base += 32) {      // same trip count in every lane
                        const int r = base + lane;
                        const int x_first = __shfl_sync(0xffffffffu, gxs, min(r / kGroupRows, GROUPS - 1));
                        if (r < MAX_ROWS) ti->rowoff[r] = r * PITCH - x_first;
                    }
                    if (lane == 0) ti->rowoff[MAX_ROWS] = 0;
                }
            }
            // fill != 0 cannot rely on the copy's zero fill: stage only tiles that stay inside the image
            inside = inside && fp.row0 >= 0 && fp.row0 + fp.rows <= k.h;
            staged = staged && (MODE == 0 || (k.fill[0] == 0.0f && k.fill[1] == 0.0f && k.fill[2] == 0.0f) || inside);
        }
        // per-row terms of the source coordinates (see TileInfo)
#pragma unroll
        for (int r = lane; r < TILE_H; r += 32) {
            const int y = min(ty * TILE_H + r, k.oh - 1);
            float yv = __fadd_rn(__fadd_rn(__int_as_float(0x4B000000 | y), -8388608.0f), g.top);
            if (MODE == 0) {
                ti->row_y[r] = truncf(yv);
            } else {
                yv = __fadd_rn(__fadd_rn(yv, -g.half_h), 0.5f);
                ti->row_y[r] = yv;
                ti->row_b[r] = __fmul_rn(g.b, yv);
                ti->row_e[r] = __fmul_rn(g.e, yv);
            }
        }
        if (lane == 0) {
            ti->g = g;
            ti->col = col;
            ti->n = n;
            ti->x0 = tx * kTileW;
            ti->y0 = ty * TILE_H;
            ti->rows = staged ? fp.rows : 0;
            ti->row0 = fp.row0;
            ti->window = (window ? 1 : 0) | (phase << 1);
            ti->xs0 = gxs;
            ti->real_tile = real_tile;
            ti->r_count = r_count;
        }
        __syncwarp();

        // ---- (2) the stage must have been released by every consumer warp before it is overwritten
        if (tile == k.skip_arrive_tile) return;      // diagnostics only: lets the consumers' wait run out
        if (use > 0 && !mbar_wait_or_abort(&empty[p], (uint32_t)(use - 1) & 1u, abort_flag, k.wait_ns)) return;

        // ---- (3) copies; the warp's own arrival publishes the descriptor
        if (staged) {
            if (lane == 0)
                mbar_expect_tx(&full[p], (uint32_t)(ngroups * C * PITCH * kGroupRows * (int)sizeof(S)));
            __syncwarp();
            if (window) {
                if (lane < C)         // one box of ngroups * kGroupRows rows per channel
                    tma_load_3d(stage + lane * PLANE, &maps.rows[ngroups - 1], gxs, fp.row0, n * C + lane, &full[p]);
            } else if (lane < ngroups) {
#pragma unroll
                for (int c = 0; c < C; ++c)
                    tma_load_3d(stage + c * PLANE + lane * kGroupRows * PITCH, &maps.rows[0], gxs,
                                fp.row0 + lane * kGroupRows, n * C + c, &full[p]);
            }
            ++n_staged;
        } else {
            ++n_direct;
        }
        if (lane == 0) mbar_arrive(&full[p]);

        // next tile of this warp
        if constexpr (!TWO) {
            tx += step_tx;
            if (tx >= k.tiles_x) { tx -= k.tiles_x; ++ty; }
            ty += step_ty;
            if (ty >= k.tiles_y) { ty -= k.tiles_y; ++n; }
            n += step_n;
        }
    }
    if (lane == 0 && k.counters) {
        if (n_staged) atomicAdd(k.counters + kCntStaged, n_staged);
        if (n_direct) atomicAdd(k.counters + kCntDirect, n_direct);
    }
}

}  // namespace ta
