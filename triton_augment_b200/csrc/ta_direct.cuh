// Fused crop + flip + colour + normalize kernel (no affine matrix).
//
// Source coordinates are whole pixels, so an output row segment is a source row
// segment (reversed when flipped): nothing to stage.  Each warp owns strips of
// 32 x kRows output pixels, lanes along x, and issues all of a strip's loads
// (kRows x C independent 128-byte warp requests) before it touches the first value,
// which is what keeps enough bytes in flight to cover HBM latency.  Warps walk the
// strips grid-stride.  Restates the has_affine=False branch of
// triton_augment/kernels/fused_kernel.py:215-225 (and :345-350); unlike the reference
// a window that leaves the image reads 0 instead of out-of-bounds memory.
#pragma once

#include "ta_common.cuh"

namespace ta {

constexpr int kDirectRows = 8;

template <typename T, int C, unsigned F>
__global__ void __launch_bounds__(kThreads, 4) direct_kernel(const __grid_constant__ KArgs k)
{
    const int lane = threadIdx.x & 31;
    const int warp_global = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int warps_total = (gridDim.x * kThreads) >> 5;
    const int strips_per_img = k.tiles_x * k.tiles_y;     // tiles_x = ceil(ow/32), tiles_y = ceil(oh/kDirectRows)
    const size_t plane = (size_t)k.h * k.w, oplane = (size_t)k.oh * k.ow;

    for (int strip = warp_global; strip < k.num_tiles; strip += warps_total) {
        const int n = strip / strips_per_img;
        const int s_in = strip - n * strips_per_img;
        const int ty = s_in / k.tiles_x, tx = s_in - ty * k.tiles_x;
        const int x = tx * 32 + lane;
        const int y_first = ty * kDirectRows;
        Geom g;
        load_geom(g, k, n, false);
        Colour<T, C, F> col;
        col.init(k, n);
        if (x >= k.ow) continue;
        const T *img = (const T *)k.in + (size_t)n * C * plane;
        T *out = (T *)k.out + (size_t)n * C * oplane;
        // fused_kernel.py:217-218: float coordinate truncated to int32.
        const int xin = (int)img_x(g, k.ow, x);
        const bool x_ok = (unsigned)xin < (unsigned)k.w;

        T s[kDirectRows][C];
#pragma unroll
        for (int i = 0; i < kDirectRows; ++i) {
            const int yin = (int)img_y(g, y_first + i);
            const bool ok = x_ok && (y_first + i) < k.oh && (unsigned)yin < (unsigned)k.h;
#pragma unroll
            for (int c = 0; c < C; ++c)
                s[i][c] = ok ? __ldg(img + c * plane + (size_t)yin * k.w + xin) : Elem<T>::from_f(0.0f);
        }
#pragma unroll
        for (int i = 0; i < kDirectRows; ++i) {
            const int y = y_first + i;
            if (y < k.oh) {
                float v[C];
                col.apply(k, s[i], v);
#pragma unroll
                for (int c = 0; c < C; ++c) Elem<T>::store(out + c * oplane + (size_t)y * k.ow + x, v[c]);
            }
        }
    }
}

}  // namespace ta
