// Producer role of the staged affine kernel.  There is one producer warp per stage of the
// ring: warp p fills stage p for the CTA's tiles p, p + kStages, p + 2 kStages, ...
//
// Per tile the warp (1) works out the source footprint and writes the tile's descriptor, (2)
// waits until the consumers have released the stage, (3) issues the copies.  Only (3) sits
// between "stage free" and "data on its way", so it is kept to one tensor copy per channel in
// the common case; everything else is done ahead of the wait.
#pragma once

namespace ta {

template <typename T, int C, int MODE, unsigned F, typename S>
__device__ __forceinline__ void affine_producer(const KArgs &k, const TMaps &maps, unsigned char *smem,
                                                uint64_t *full, uint64_t *empty, volatile int *abort_flag, int p)
{
    using Info = TileInfo<T, C, F>;
    using Smem = AffineSmem<T, C, F, S>;
    constexpr int CH = Src<S>::chunk, PITCH = Src<S>::pitch, PLANE = Src<S>::plane;
    static_assert(kNumGroups <= 32 && kMaxRows % kGroupRows == 0, "one lane per row group");
    const int lane = threadIdx.x & 31;
    const int tiles_per_img = k.tiles_x * k.tiles_y;
    S *stage = reinterpret_cast<S *>(smem + p * Smem::stage);
    unsigned long long n_staged = 0, n_direct = 0;
    int cur_n = -1;
    Geom g;
    Colour<T, C, F> col;

    // Tile number -> (image, tile row, tile column), then stepped by kStages * gridDim.x tiles per
    // round with carries instead of divisions.  Consecutive tile numbers are neighbours along x:
    // the CTAs running at one time then read whole runs of image rows (DRAM page hits) and share
    // the overlap of their boxes in L2; an order that interleaves images was 20-50 % slower.
    const int first = (int)blockIdx.x + p * (int)gridDim.x, step = kStages * (int)gridDim.x;
    int n = first / tiles_per_img, ty = (first % tiles_per_img) / k.tiles_x, tx = (first % tiles_per_img) % k.tiles_x;
    const int step_n = step / tiles_per_img, step_ty = (step % tiles_per_img) / k.tiles_x,
              step_tx = (step % tiles_per_img) % k.tiles_x;

    int use = 0;
    for (int tile = first; tile < k.num_tiles; tile += step, ++use) {
        if (n != cur_n) {                                   // per-image parameters: reload on change only
            load_geom(g, k, n, MODE != 0);
            col.init(k, n);
            cur_n = n;
        }
        Info *ti = reinterpret_cast<Info *>(smem + kStages * Smem::stage + (size_t)(p + kStages * (use & 1)) * Smem::info);

        // ---- (1) footprint and descriptor
        TileFootprint fp;
        fp.rows = 0;
        fp.row0 = 0;
        const float m[6] = {g.a, g.b, g.c, g.d, g.e, g.f};
        constexpr int FMODE = MODE == 2 ? 1 : 0;            // footprint rule: nearest or bilinear
        if (k.staged_ok) {
            if (MODE == 0) tile_footprint_crop(fp, k.oh, k.ow, g.top, g.left, g.flip, tx, ty);
            else tile_footprint(fp, FMODE, k.h, k.w, k.oh, k.ow, g.top, g.left, g.flip, m, tx, ty);
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
                // lanes 0 .. kNumGroups-1: columns of row group `lane`; the other lanes hold a neutral entry
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
                    for (int base = 0; base < kMaxRows; base += 32) {      // same trip count in every lane
                        const int r = base + lane;
                        const int x_first = __shfl_sync(0xffffffffu, gxs, min(r / kGroupRows, kNumGroups - 1));
                        if (r < kMaxRows) ti->rowoff[r] = r * PITCH - x_first;
                    }
                    if (lane == 0) ti->rowoff[kMaxRows] = 0;
                }
            }
            // fill != 0 cannot rely on the copy's zero fill: stage only tiles that stay inside the image
            inside = inside && fp.row0 >= 0 && fp.row0 + fp.rows <= k.h;
            staged = staged && (MODE == 0 || k.fill == 0.0f || inside);
        }
        if (lane == 0) {
            ti->g = g;
            ti->col = col;
            ti->n = n;
            ti->x0 = tx * kTileW;
            ti->y0 = ty * kTileH;
            ti->rows = staged ? fp.rows : 0;
            ti->row0 = fp.row0;
            ti->window = window ? 1 : 0;
            ti->xs0 = gxs;
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
        tx += step_tx;
        if (tx >= k.tiles_x) { tx -= k.tiles_x; ++ty; }
        ty += step_ty;
        if (ty >= k.tiles_y) { ty -= k.tiles_y; ++n; }
        n += step_n;
    }
    if (lane == 0 && k.counters) {
        if (n_staged) atomicAdd(k.counters + kCntStaged, n_staged);
        if (n_direct) atomicAdd(k.counters + kCntDirect, n_direct);
    }
}

}  // namespace ta
