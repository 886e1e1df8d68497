// Producer and consumer roles of the staged affine kernel, and the kernel itself.
#pragma once

namespace ta {

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// Two source coordinates at once with the packed fp32 pipe; per lane the operation order of
// src_coord(): ((fma(xc, a, b*yc) + c) + half) + (-0.5), each step rounded to nearest.
// R picks which product is fused into the addition (see CoordRecipe).
template <int R>
__device__ __forceinline__ float2 src_coord2(float xc, float a, float b, float2 yc, float c, float half)
{
    float2 u = R == 1 ? pk_fma(f2(xc, xc), f2(a, a), pk_mul(f2(b, b), yc))
                      : pk_fma(yc, f2(b, b), pk_mul(f2(a, a), f2(xc, xc)));
    u = pk_add(u, f2(c, c));
    u = pk_add(f2(half, half), u);
    return pk_add(u, f2(-0.5f, -0.5f));
}

}  // namespace ta

#include "ta_affine_producer.cuh"

namespace ta {

// ----------------------------------------------------------------------------- consumer
template <typename T, int C, int MODE, unsigned F, bool CHECK>
__device__ __forceinline__ void affine_consumer(const KArgs &k, unsigned char *smem, uint64_t *full, uint64_t *empty,
                                                volatile int *abort_flag)
{
    using Info = TileInfo<T, C, F>;
    constexpr size_t STAGE = AffineSmem<T, C, F>::stage;
    constexpr int ROWS_PER_WARP = kTileH / (kConsumerWarps / 2);     // 4
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wx = warp & 1, wy = warp >> 1;
    const unsigned oplane = (unsigned)(k.oh * k.ow);
    unsigned long long n_viol = 0;
    int cur_n = -1;
    Geom g;
    Colour<T, C, F> col;
    int it = 0;
    for (int tile = blockIdx.x; tile < k.num_tiles; tile += gridDim.x, ++it) {
        const int s = it % kStages, use = it / kStages;
        if (!mbar_wait_or_abort(&full[s], (uint32_t)use & 1u, abort_flag)) return;
        const T *stage = reinterpret_cast<const T *>(smem + s * STAGE);
        const Info *ti = reinterpret_cast<const Info *>(smem + s * STAGE + (size_t)C * kPlane * sizeof(T));
        const int n = ti->n, rows = ti->rows, row0 = ti->row0;
        if (n != cur_n) {            // per-image parameters change only every few tiles (warp-uniform branch)
            g = ti->g;
            col = ti->col;
            cur_n = n;
        }
        const int x = ti->x0 + wx * 32 + lane;
        const int y_first = ti->y0 + wy * ROWS_PER_WARP;

        if (rows == 0) {
            affine_rows_direct<T, C, MODE, F>(k, g, col, n, x, y_first, ROWS_PER_WARP);
        } else if (x < k.ow) {
            T *out = (T *)k.out + (size_t)n * C * oplane;
            const float xc = centred(img_x(g, k.ow, x), g.half_w);
#pragma unroll
            for (int pr = 0; pr < ROWS_PER_WARP / 2; ++pr) {
                // No early exit: rows past the image's last row are computed on the last row's
                // geometry (always staged) and only their stores are dropped, so the pairs stay
                // independent and their instructions can interleave.
                const int y_raw = y_first + 2 * pr;
                const bool a_ok = y_raw < k.oh, b_ok = y_raw + 1 < k.oh;
                const int ya = min(y_raw, k.oh - 1), yb = min(y_raw + 1, k.oh - 1);
                const float2 yc = f2(centred(__fadd_rn(float_of_small_uint(ya), g.top), g.half_h),
                                     centred(__fadd_rn(float_of_small_uint(yb), g.top), g.half_h));
                const float2 sx = src_coord2<CoordRecipe<MODE, F>::x>(xc, g.a, g.b, yc, g.c, g.half_w);
                const float2 sy = src_coord2<CoordRecipe<MODE, F>::y>(xc, g.d, g.e, yc, g.f, g.half_h);
                T smp[2][C];
                if (MODE == 1) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int xn = rint_magic(j ? sx.y : sx.x);
                        int r = rint_magic(j ? sy.y : sy.x) - row0;
                        if (CHECK && (unsigned)r >= (unsigned)rows) { ++n_viol; r = 0; }
                        int idx = ti->rowoff[r] + xn;
                        if (CHECK && (unsigned)(idx - r * ti->bw) >= (unsigned)ti->bw) { ++n_viol; idx = 0; }
#pragma unroll
                        for (int c = 0; c < C; ++c) smp[j][c] = stage[c * kPlane + idx];
                    }
                } else {
                    int i0[2], i1[2];
                    float2 dx, dy;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float fx = j ? sx.y : sx.x, fy = j ? sy.y : sy.x;
                        float frac_x, frac_y;
                        const int x0 = floor_magic(fx, frac_x), y0 = floor_magic(fy, frac_y);
                        (j ? dx.y : dx.x) = frac_x;
                        (j ? dy.y : dy.x) = frac_y;
                        int r = y0 - row0;
                        if (CHECK && (unsigned)r >= (unsigned)(rows - 1)) { ++n_viol; r = 0; }
                        i0[j] = ti->rowoff[r] + x0;
                        i1[j] = ti->rowoff[r + 1] + x0;
                        if (CHECK && ((unsigned)(i0[j] - r * ti->bw) >= (unsigned)(ti->bw - 1) ||
                                      (unsigned)(i1[j] - (r + 1) * ti->bw) >= (unsigned)(ti->bw - 1))) {
                            ++n_viol; i0[j] = i1[j] = 0;
                        }
                    }
                    const float2 one = f2(1.0f, 1.0f), neg = f2(-1.0f, -1.0f);
                    const float2 omx = pk_fma(dx, neg, one), omy = pk_fma(dy, neg, one);   // 1 - d, one rounding
                    const float2 w00 = pk_mul(omx, omy), w10 = pk_mul(dx, omy);
                    const float2 w01 = pk_mul(omx, dy), w11 = pk_mul(dx, dy);
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        const T *pl = stage + c * kPlane;
                        float2 acc = pk_mul(f2(Elem<T>::to_f(pl[i0[0]]), Elem<T>::to_f(pl[i0[1]])), w00);
                        acc = pk_fma(f2(Elem<T>::to_f(pl[i0[0] + 1]), Elem<T>::to_f(pl[i0[1] + 1])), w10, acc);
                        acc = pk_fma(f2(Elem<T>::to_f(pl[i1[0]]), Elem<T>::to_f(pl[i1[1]])), w01, acc);
                        acc = pk_fma(f2(Elem<T>::to_f(pl[i1[0] + 1]), Elem<T>::to_f(pl[i1[1] + 1])), w11, acc);
                        smp[0][c] = Elem<T>::from_f(acc.x);
                        smp[1][c] = Elem<T>::from_f(acc.y);
                    }
                }
                const unsigned o = (unsigned)(y_raw * k.ow + x);
                if constexpr (sizeof(T) == 4) {
                    float2 v2[C];
#pragma unroll
                    for (int c = 0; c < C; ++c) v2[c] = f2(smp[0][c], smp[1][c]);
                    col.apply2(k, v2);
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        if (a_ok) Elem<T>::store(out + (size_t)c * oplane + o, v2[c].x);
                        if (b_ok) Elem<T>::store(out + (size_t)c * oplane + o + k.ow, v2[c].y);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        float v[C];
                        col.apply(k, smp[j], v);
                        if (j == 0 ? a_ok : b_ok) {
#pragma unroll
                            for (int c = 0; c < C; ++c) Elem<T>::store(out + (size_t)c * oplane + o + j * k.ow, v[c]);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (CHECK && n_viol && k.counters) atomicAdd(k.counters + kCntViolation, n_viol);
}

// ----------------------------------------------------------------------------- kernel
template <typename T, int C, int MODE, unsigned F, bool CHECK>
__global__ void __launch_bounds__(kAffineThreads, 1)
affine_kernel(const __grid_constant__ KArgs k, const __grid_constant__ TMaps maps)
{
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t full[kStages];
    __shared__ __align__(8) uint64_t empty[kStages];
    __shared__ int abort_flag;
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kConsumerWarps);
        }
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if ((threadIdx.x >> 5) >= kConsumerWarps)
        affine_producer<T, C, MODE, F>(k, maps, smem, full, empty, &abort_flag, (int)(threadIdx.x >> 5) - kConsumerWarps);
    else
        affine_consumer<T, C, MODE, F, CHECK>(k, smem, full, empty, &abort_flag);

    // Leave together.  After an abort, copies may still be in flight towards this CTA's shared
    // memory: give each stage one more bounded chance to settle before the memory is released.
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0 && k.counters) atomicAdd(k.counters + kCntTimeout, 1ull);
        if (threadIdx.x < kStages) {
            for (int i = 0; i < 4096; ++i)
                if (mbar_try_wait(&full[threadIdx.x], 0) || mbar_try_wait(&full[threadIdx.x], 1)) break;
        }
    }
}

}  // namespace ta
