// Fused inverse-affine + crop + flip + colour + normalize kernel (nearest / bilinear).
//
// One CTA walks output tiles of kTileW x kTileH pixels (persistent, grid-stride).  For
// each tile it works out which source rows and, per row, which columns the tile reads
// (ta_footprint.h), brings exactly those row segments into shared memory with bulk
// asynchronous copies that complete on an mbarrier, and then samples from shared
// memory: lanes run along x so reads are bank-conflict-free and every store is a full
// 128-byte line.  Texels outside the image are written as `fill` while staging, so the
// sampling loop has no bounds tests.  A tile whose footprint does not fit (extreme
// zoom-out, rotation near 90 degrees, unaligned rows) is gathered straight from global
// memory with the reference's per-tap bounds tests instead.
#pragma once

#include "ta_common.cuh"

namespace ta {

template <typename T> struct Chunk { static constexpr int value = 16 / (int)sizeof(T); };

template <typename T, int C> constexpr size_t affine_smem_bytes()
{
    return (size_t)C * kMaxRows * kPitch * sizeof(T) + (size_t)(kMaxRows + 4) * sizeof(int);
}

// Gather one tile from global memory (no staging).  MODE 1 nearest, 2 bilinear.
template <typename T, int C, int MODE, unsigned F>
__device__ __forceinline__ void affine_tile_direct(const KArgs &k, const Geom &g, const Colour<T, C, F> &col,
                                                   int n, int x, int y_first, int y_count)
{
    if (x >= k.ow) return;
    const T *img = (const T *)k.in + (size_t)n * C * k.h * k.w;
    T *out = (T *)k.out + (size_t)n * C * k.oh * k.ow;
    const size_t plane = (size_t)k.h * k.w, oplane = (size_t)k.oh * k.ow;
    const T fillv = Elem<T>::from_f(k.fill);
    const float xc = centred(img_x(g, k.ow, x), g.half_w);
    for (int i = 0; i < y_count; ++i) {
        const int y = y_first + i;
        if (y >= k.oh) break;
        const float yc = centred(img_y(g, y), g.half_h);
        const float sx = src_coord(xc, g.a, __fmul_rn(g.b, yc), g.c, g.half_w);
        const float sy = src_coord(xc, g.d, __fmul_rn(g.e, yc), g.f, g.half_h);
        T s[C];
        if (MODE == 1) {
            const int xn = __float2int_rn(sx), yn = __float2int_rn(sy);
#pragma unroll
            for (int c = 0; c < C; ++c) s[c] = tap_global(img + c * plane, k.w, k.h, xn, yn, fillv);
        } else {
            const int x0 = __float2int_rd(sx), y0 = __float2int_rd(sy);
            const float dx = sx - (float)x0, dy = sy - (float)y0;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const T *pl = img + c * plane;
                const float p00 = Elem<T>::to_f(tap_global(pl, k.w, k.h, x0, y0, fillv));
                const float p10 = Elem<T>::to_f(tap_global(pl, k.w, k.h, x0 + 1, y0, fillv));
                const float p01 = Elem<T>::to_f(tap_global(pl, k.w, k.h, x0, y0 + 1, fillv));
                const float p11 = Elem<T>::to_f(tap_global(pl, k.w, k.h, x0 + 1, y0 + 1, fillv));
                s[c] = Elem<T>::from_f(blend4(p00, p10, p01, p11, dx, dy));
            }
        }
        float v[C];
        col.apply(k, s, v);
#pragma unroll
        for (int c = 0; c < C; ++c) Elem<T>::store(out + c * oplane + (size_t)y * k.ow + x, v[c]);
    }
}

template <typename T, int C, int MODE, unsigned F, bool CHECK>
__global__ void __launch_bounds__(kThreads, (sizeof(T) == 4 && C == 3) ? 3 : 4)
affine_kernel(const __grid_constant__ KArgs k)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int CH = Chunk<T>::value;
    constexpr int PLANE = kMaxRows * kPitch;
    T *stage = reinterpret_cast<T *>(smem_raw);
    int *rowoff = reinterpret_cast<int *>(smem_raw + (size_t)C * PLANE * sizeof(T));
    __shared__ __align__(8) uint64_t full_bar;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        mbar_init(&full_bar, kThreads);
        mbar_fence_init();
    }
    __syncthreads();

    uint32_t phase = 0;
    bool poisoned = false;               // a barrier wait ran out: stop staging in this CTA
    unsigned long long n_staged = 0, n_direct = 0, n_viol = 0;
    const int tiles_per_img = k.tiles_x * k.tiles_y;
    const int wx = warp & 1, wy = warp >> 1;          // 2 warps across, 4 down; 8 rows per warp
    constexpr int ROWS_PER_WARP = kTileH / (kWarps / 2);

    for (int tile = blockIdx.x; tile < k.num_tiles; tile += gridDim.x) {
        const int n = tile / tiles_per_img;
        const int t_in = tile - n * tiles_per_img;
        const int ty = t_in / k.tiles_x, tx = t_in - ty * k.tiles_x;
        Geom g;
        load_geom(g, k, n, true);
        Colour<T, C, F> col;
        col.init(k, n);
        const int x = tx * kTileW + wx * 32 + lane;
        const int y_first = ty * kTileH + wy * ROWS_PER_WARP;

        TileFootprint fp;
        fp.rows = 0;
        if (k.staged_ok && !poisoned) {
            const float m[6] = {g.a, g.b, g.c, g.d, g.e, g.f};
            tile_footprint(fp, MODE - 1, CH, k.h, k.w, k.oh, k.ow, g.top, g.left, g.flip, m, tx, ty);
        }
        if (fp.rows == 0) {              // uniform across the CTA
            affine_tile_direct<T, C, MODE, F>(k, g, col, n, x, y_first, ROWS_PER_WARP);
            if (tid == 0) ++n_direct;
            continue;
        }

        // ---- stage: one (source row, channel) segment per thread
        const int nseg = fp.rows * C;
        for (int s = tid; s < nseg; s += kThreads) {
            const int r = s / C, c = s - r * C;
            int xs, xe;
            tile_row_range(fp, MODE - 1, CH, r, xs, xe);
            if (c == 0) rowoff[r] = r * kPitch - xs;
            const int yr = fp.row0 + r;
            T *dst = stage + c * PLANE + r * kPitch;
            const bool row_in = (unsigned)yr < (unsigned)k.h;
            const int cs = row_in ? max(xs, 0) : xe, ce = row_in ? min(xe, k.w) : xe;   // copied part
            const T fillv = Elem<T>::from_f(k.fill);
            for (int q = xs; q < min(cs, xe); ++q) dst[q - xs] = fillv;
            for (int q = max(ce, xs); q < xe; ++q) dst[q - xs] = fillv;
            if (ce > cs) {
                const T *src = (const T *)k.in + (((size_t)n * C + c) * k.h + yr) * k.w + cs;
                const uint32_t bytes = (uint32_t)(ce - cs) * sizeof(T);
                mbar_expect_tx(&full_bar, bytes);
                bulk_copy_g2s(dst + (cs - xs), src, bytes, &full_bar);
            }
        }
        mbar_arrive(&full_bar);
        const bool landed = mbar_wait_bounded(&full_bar, phase);
        if (__syncthreads_or(!landed)) {
            // Should never happen.  The decision is taken by the whole CTA so that no thread
            // is left alone at a barrier: record it, stop staging in this CTA, and produce
            // the tile from global memory so the output is still right.
            poisoned = true;
            if (tid == 0 && k.counters) atomicAdd(k.counters + kCntTimeout, 1ull);
            affine_tile_direct<T, C, MODE, F>(k, g, col, n, x, y_first, ROWS_PER_WARP);
            continue;
        }
        phase ^= 1;
        if (tid == 0) ++n_staged;

        // ---- sample from shared memory
        if (x < k.ow) {
            T *out = (T *)k.out + (size_t)n * C * k.oh * k.ow;
            const size_t oplane = (size_t)k.oh * k.ow;
            const float xc = centred(img_x(g, k.ow, x), g.half_w);
#pragma unroll 2
            for (int i = 0; i < ROWS_PER_WARP; ++i) {
                const int y = y_first + i;
                if (y >= k.oh) break;
                const float yc = centred(img_y(g, y), g.half_h);
                const float sx = src_coord(xc, g.a, __fmul_rn(g.b, yc), g.c, g.half_w);
                const float sy = src_coord(xc, g.d, __fmul_rn(g.e, yc), g.f, g.half_h);
                T s[C];
                if (MODE == 1) {
                    const int xn = __float2int_rn(sx);
                    int r = __float2int_rn(sy) - fp.row0;
                    if (CHECK && (unsigned)r >= (unsigned)fp.rows) { ++n_viol; r = 0; }
                    int idx = rowoff[r] + xn;
                    if (CHECK && (unsigned)(idx - r * kPitch) >= (unsigned)kPitch) { ++n_viol; idx = r * kPitch; }
#pragma unroll
                    for (int c = 0; c < C; ++c) s[c] = stage[c * PLANE + idx];
                } else {
                    const int x0 = __float2int_rd(sx), y0 = __float2int_rd(sy);
                    const float dx = sx - (float)x0, dy = sy - (float)y0;
                    int r = y0 - fp.row0;
                    if (CHECK && (unsigned)r >= (unsigned)(fp.rows - 1)) { ++n_viol; r = 0; }
                    int i0 = rowoff[r] + x0, i1 = rowoff[r + 1] + x0;
                    if (CHECK && ((unsigned)(i0 - r * kPitch) >= (unsigned)(kPitch - 1) ||
                                  (unsigned)(i1 - (r + 1) * kPitch) >= (unsigned)(kPitch - 1))) {
                        ++n_viol; i0 = r * kPitch; i1 = (r + 1) * kPitch;
                    }
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        const T *pl = stage + c * PLANE;
                        s[c] = Elem<T>::from_f(blend4(Elem<T>::to_f(pl[i0]), Elem<T>::to_f(pl[i0 + 1]),
                                                      Elem<T>::to_f(pl[i1]), Elem<T>::to_f(pl[i1 + 1]), dx, dy));
                    }
                }
                float v[C];
                col.apply(k, s, v);
#pragma unroll
                for (int c = 0; c < C; ++c) Elem<T>::store(out + c * oplane + (size_t)y * k.ow + x, v[c]);
            }
        }
        // Everyone is done reading before the next tile's copies and fills overwrite the stage.
        fence_proxy_async();
        __syncthreads();
    }

    // Copies issued before a failed wait may still be in flight: give them one more
    // bounded chance to land before the CTA's shared memory is released.
    if (poisoned) mbar_wait_bounded(&full_bar, phase);

    if (k.counters) {
        if (tid == 0) {
            if (n_staged) atomicAdd(k.counters + kCntStaged, n_staged);
            if (n_direct) atomicAdd(k.counters + kCntDirect, n_direct);
        }
        if (CHECK && n_viol) atomicAdd(k.counters + kCntViolation, n_viol);
    }
}

}  // namespace ta
