// Producer role of the staged affine kernel.  There is one producer warp per stage of the
// ring: warp p fills stage p for the CTA's tiles p, p + kStages, p + 2 kStages, ... so each
// producer has kStages tile-times for the arithmetic of one tile.
#pragma once

namespace ta {

template <typename T, int C, int MODE, unsigned F>
__device__ __forceinline__ void affine_producer(const KArgs &k, const TMaps &maps, unsigned char *smem,
                                                uint64_t *full, uint64_t *empty, volatile int *abort_flag, int p)
{
    using Info = TileInfo<T, C, F>;
    constexpr int CH = 16 / (int)sizeof(T);
    constexpr size_t STAGE = AffineSmem<T, C, F>::stage;
    constexpr int NGROUPS = kMaxRows / kGroupRows;          // lanes 0 .. NGROUPS-1 each own one row group
    static_assert(NGROUPS <= 32 && kMaxRows % kGroupRows == 0, "one lane per row group");
    const int lane = threadIdx.x & 31;
    const int tiles_per_img = k.tiles_x * k.tiles_y;
    T *stage = reinterpret_cast<T *>(smem + p * STAGE);
    Info *ti = reinterpret_cast<Info *>(smem + p * STAGE + (size_t)C * kPlane * sizeof(T));
    unsigned long long n_staged = 0, n_direct = 0;
    int cur_n = -1;
    Geom g;
    Colour<T, C, F> col;

    int use = 0;
    for (long long tile = (long long)blockIdx.x + (long long)p * gridDim.x; tile < k.num_tiles;
         tile += (long long)kStages * gridDim.x, ++use) {
        const int n = (int)(tile / tiles_per_img);
        const int t_in = (int)(tile - (long long)n * tiles_per_img);
        const int ty = t_in / k.tiles_x, tx = t_in - ty * k.tiles_x;
        if (n != cur_n) {                                   // per-image parameters: reload on change only
            load_geom(g, k, n, true);
            col.init(k, n);
            cur_n = n;
        }
        TileFootprint fp;
        fp.rows = 0;
        fp.row0 = 0;
        if (k.staged_ok) {
            const float m[6] = {g.a, g.b, g.c, g.d, g.e, g.f};
            tile_footprint(fp, MODE - 1, CH, k.h, k.w, k.oh, k.ow, g.top, g.left, g.flip, m, tx, ty);
        }
        bool staged = fp.rows > 0;
        int gxs = 0, bw = kPitch, bi = kNumBoxWidths - 1;
        const int ngroups = (fp.rows + kGroupRows - 1) / kGroupRows;
        if (staged) {
            // lanes 0 .. NGROUPS-1: columns of row group `lane`; the other lanes hold a neutral entry
            const int grp = lane;
            int xs = 0, xe = CH;
            const int r_first = grp * kGroupRows, r_last = min(r_first + kGroupRows, fp.rows) - 1;
            if (grp >= ngroups || !tile_rows_range(fp, MODE - 1, CH, r_first, r_last, xs, xe)) { xs = 0; xe = CH; }
            gxs = xs;
            int wmax = xe - xs;
            bool inside = grp >= ngroups || (xs >= 0 && xe <= k.w);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
            inside = __all_sync(0xffffffffu, inside) && fp.row0 >= 0 && fp.row0 + fp.rows <= k.h;
            bi = wmax <= box_width(0) ? 0 : wmax <= box_width(1) ? 1 : 2;
            bw = box_width(bi);
            // fill != 0 cannot rely on TMA's zero fill: stage only tiles that stay inside the image
            staged = wmax <= kPitch && (k.fill == 0.0f || inside);
        }

        // The stage must have been released by every consumer warp before it is overwritten.
        if (use > 0 && !mbar_wait_or_abort(&empty[p], (uint32_t)(use - 1) & 1u, abort_flag)) return;

        if (staged) {
            // rowoff[r] = r * bw - (first column of r's group); rows lane, lane + 32, ...
#pragma unroll
            for (int base = 0; base < kMaxRows; base += 32) {      // same trip count in every lane
                const int r = base + lane;
                const int x_first = __shfl_sync(0xffffffffu, gxs, min(r / kGroupRows, NGROUPS - 1));
                if (r < kMaxRows) ti->rowoff[r] = r * bw - x_first;
            }
            if (lane == 0) {
                ti->rowoff[kMaxRows] = 0;
                mbar_expect_tx(&full[p], (uint32_t)(ngroups * C * bw * kGroupRows * (int)sizeof(T)));
            }
            __syncwarp();
            if (lane < ngroups) {
#pragma unroll
                for (int c = 0; c < C; ++c)
                    tma_load_3d(stage + c * kPlane + lane * kGroupRows * bw, &maps.m[bi], gxs,
                                fp.row0 + lane * kGroupRows, n * C + c, &full[p]);
            }
            ++n_staged;
        } else {
            ++n_direct;
        }
        if (lane == 0) {
            ti->g = g;
            ti->col = col;
            ti->n = n;
            ti->x0 = tx * kTileW;
            ti->y0 = ty * kTileH;
            ti->rows = staged ? fp.rows : 0;
            ti->row0 = fp.row0;
            ti->bw = bw;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[p]);
    }
    if (lane == 0 && k.counters) {
        if (n_staged) atomicAdd(k.counters + kCntStaged, n_staged);
        if (n_direct) atomicAdd(k.counters + kCntDirect, n_direct);
    }
}

}  // namespace ta
