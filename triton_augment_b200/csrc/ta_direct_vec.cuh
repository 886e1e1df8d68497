// Vectorised crop + flip + colour + normalize kernel: 128-bit loads and stores.
//
// Each lane owns EPV = 16 / sizeof(T) consecutive output pixels of a row, so a warp covers
// 512 contiguous output bytes per row and channel and every store is one aligned 16-byte
// vector.  The matching source run starts wherever the crop offset puts it, so each lane
// loads the two ALIGNED 16-byte vectors that cover its run and shifts the wanted elements
// out of the 8 words with funnel shifts (the shift is the same for the whole warp); a flipped
// image reads the mirrored run and reverses it in registers.  Launched only when the host
// has checked that rows of the output are whole vectors, that both tensors are 16-byte
// aligned and that every channel plane of the input is a whole number of vectors (so all
// channels of a strip share one shift); anything else uses direct_kernel.
// Strips whose source run leaves its image row (an invalid crop window) take the scalar
// route with the same read-as-zero rule.
#pragma once

#include "ta_common.cuh"

namespace ta {

constexpr int kVecRows = 2;                    // rows per warp strip

// epv: elements per 16-byte vector.  blocks: resident CTAs per SM the register budget is set
// for; the kernel waits on load latency, so fp32 gains from a third CTA (crop 112 of 224:
// 248 -> 232 us for 4096 images; 256 -> 224: 242 -> 219 us for 1024 images), a fourth spills.
// The fp16 kernel got slower with three (314 -> 329 us on 512 x 3 x 512^2 -> 448^2).
template <typename T> struct VecTraits;
template <> struct VecTraits<float> { static constexpr int epv = 4, blocks = 3; };
template <> struct VecTraits<__half> { static constexpr int epv = 8, blocks = 2; };

// words[q .. q+4] of the 8 loaded words, shifted right by `sh` bits (0 or 16): the 4 output words.
__device__ __forceinline__ void extract4(const uint32_t (&w)[8], int q, int sh, uint32_t (&o)[4])
{
    uint32_t v[5];
    switch (q) {                      // warp-uniform
        case 0: v[0] = w[0]; v[1] = w[1]; v[2] = w[2]; v[3] = w[3]; v[4] = w[4]; break;
        case 1: v[0] = w[1]; v[1] = w[2]; v[2] = w[3]; v[3] = w[4]; v[4] = w[5]; break;
        case 2: v[0] = w[2]; v[1] = w[3]; v[2] = w[4]; v[3] = w[5]; v[4] = w[6]; break;
        default: v[0] = w[3]; v[1] = w[4]; v[2] = w[5]; v[3] = w[6]; v[4] = w[7]; break;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __funnelshift_r(v[j], v[j + 1], sh);
}

template <typename T> __device__ __forceinline__ void reverse_elems(uint32_t (&o)[4]);
template <> __device__ __forceinline__ void reverse_elems<float>(uint32_t (&o)[4])
{
    uint32_t a = o[0], b = o[1];
    o[0] = o[3]; o[1] = o[2]; o[2] = b; o[3] = a;
}
template <> __device__ __forceinline__ void reverse_elems<__half>(uint32_t (&o)[4])
{
    uint32_t a = __byte_perm(o[0], 0, 0x1032), b = __byte_perm(o[1], 0, 0x1032);
    o[0] = __byte_perm(o[3], 0, 0x1032); o[1] = __byte_perm(o[2], 0, 0x1032); o[2] = b; o[3] = a;
}

template <typename T> __device__ __forceinline__ T elem_of(const uint32_t (&o)[4], int i);
template <> __device__ __forceinline__ float elem_of<float>(const uint32_t (&o)[4], int i) { return __uint_as_float(o[i]); }
template <> __device__ __forceinline__ __half elem_of<__half>(const uint32_t (&o)[4], int i)
{
    return __ushort_as_half((unsigned short)((i & 1) ? (o[i >> 1] >> 16) : (o[i >> 1] & 0xffffu)));
}

template <typename T, int C, unsigned F>
__global__ void __launch_bounds__(kThreads, VecTraits<T>::blocks) direct_vec_kernel(const __grid_constant__ KArgs k)
{
    constexpr int EPV = VecTraits<T>::epv;
    constexpr int ES = (int)sizeof(T);
    const int lane = threadIdx.x & 31;
    const int warp_global = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int warps_total = (gridDim.x * kThreads) >> 5;
    const int strips_per_img = k.tiles_x * k.tiles_y;        // tiles_x = ceil(ow / (32 EPV)), tiles_y = ceil(oh / kVecRows)
    const size_t plane = (size_t)k.h * k.w, oplane = (size_t)k.oh * k.ow;
    const size_t total_vecs = (size_t)k.n * C * plane / EPV;  // planes are whole numbers of vectors
    const uint4 *in_vec = reinterpret_cast<const uint4 *>(k.in);

    for (int strip = warp_global; strip < k.num_tiles; strip += warps_total) {
        const int n = strip / strips_per_img;
        const int s_in = strip - n * strips_per_img;
        const int ty = s_in / k.tiles_x, tx = s_in - ty * k.tiles_x;
        const int x = (tx * 32 + lane) * EPV;                 // first of this lane's EPV output pixels
        const int y_first = ty * kVecRows;
        Geom g;
        load_geom(g, k, n, false);
        Colour<T, C, F> col;
        col.init(k, n);
        const bool active = x < k.ow;                          // ow is a multiple of EPV: all-or-nothing per lane
        // Source column of output pixel x (fused_kernel.py:217: float add, truncate), then the
        // lowest column of the run: x itself, or the column of this lane's LAST pixel if flipped.
        const int xin_first = (int)img_x(g, k.ow, x);
        const int run0 = g.flip ? xin_first - (EPV - 1) : xin_first;
        // The runs of neighbouring lanes must be exactly EPV apart (they are, unless `left` is
        // a float so large or odd that x + left rounds differently from lane to lane).
        const int run_lane0 = __shfl_sync(0xffffffffu, run0, 0);
        const bool spaced = run0 == run_lane0 + (g.flip ? -lane * EPV : lane * EPV);
        const bool row_ok = run0 >= 0 && run0 + EPV <= k.w && spaced;
        const bool fast = __all_sync(0xffffffffu, !active || row_ok);
        T *out = (T *)k.out + (size_t)n * C * oplane;

        if (fast) {
            uint32_t w[kVecRows][C][8];
            int q[kVecRows], sh[kVecRows];
#pragma unroll
            for (int i = 0; i < kVecRows; ++i) {
                const int yin = (int)img_y(g, y_first + i);
                const bool ok = active && (y_first + i) < k.oh && (unsigned)yin < (unsigned)k.h;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const size_t e0 = ((size_t)n * C + c) * plane + (size_t)(ok ? yin : 0) * k.w + (ok ? run0 : 0);
                    const size_t v0 = e0 / EPV;
                    const int s = (int)(e0 - v0 * EPV);
                    if (c == 0) { q[i] = (s * ES) >> 2; sh[i] = ((s * ES) & 3) * 8; }
                    const uint4 a = ok ? __ldg(in_vec + v0) : make_uint4(0, 0, 0, 0);
                    const uint4 b = (ok && v0 + 1 < total_vecs) ? __ldg(in_vec + v0 + 1) : make_uint4(0, 0, 0, 0);
                    w[i][c][0] = a.x; w[i][c][1] = a.y; w[i][c][2] = a.z; w[i][c][3] = a.w;
                    w[i][c][4] = b.x; w[i][c][5] = b.y; w[i][c][6] = b.z; w[i][c][7] = b.w;
                }
            }
#pragma unroll
            for (int i = 0; i < kVecRows; ++i) {
                const int y = y_first + i;
                // the shift is uniform over the warp's active lanes (runs are EPV apart); take lane 0's
                const int qq = __shfl_sync(0xffffffffu, q[i], 0), ss = __shfl_sync(0xffffffffu, sh[i], 0);
                uint32_t o[C][4];
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    extract4(w[i][c], qq, ss, o[c]);
                    if (g.flip) reverse_elems<T>(o[c]);
                }
                uint32_t res[C][4];
                if constexpr (ES == 4) {
                    // fp32: two neighbouring pixels per colour-tier evaluation (packed arithmetic)
#pragma unroll
                    for (int e = 0; e < EPV; e += 2) {
                        float2 v2[C];
#pragma unroll
                        for (int c = 0; c < C; ++c) v2[c] = make_float2(__uint_as_float(o[c][e]), __uint_as_float(o[c][e + 1]));
                        col.apply2(k, v2);
#pragma unroll
                        for (int c = 0; c < C; ++c) {
                            res[c][e] = __float_as_uint(v2[c].x);
                            res[c][e + 1] = __float_as_uint(v2[c].y);
                        }
                    }
                } else {
                    // fp16: element pairs through the packed colour tier, results packed as half2 words
#pragma unroll
                    for (int e = 0; e < EPV; e += 2) {
                        __half2 pk[C];
                        float2 v2[C];
#pragma unroll
                        for (int c = 0; c < C; ++c) pk[c] = *reinterpret_cast<const __half2 *>(&o[c][e >> 1]);   // elements e, e + 1
                        col.apply2(k, pk, v2);
#pragma unroll
                        for (int c = 0; c < C; ++c) {
                            const __half2 h = __floats2half2_rn(v2[c].x, v2[c].y);
                            res[c][e >> 1] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                    }
                }
                if (active && y < k.oh) {
#pragma unroll
                    for (int c = 0; c < C; ++c)
                        *reinterpret_cast<uint4 *>(out + c * oplane + (size_t)y * k.ow + x) =
                            make_uint4(res[c][0], res[c][1], res[c][2], res[c][3]);
                }
            }
        } else if (active) {
            // invalid crop window somewhere in this strip: element by element, out of range reads 0
            const T *img = (const T *)k.in + (size_t)n * C * plane;
            for (int i = 0; i < kVecRows; ++i) {
                const int y = y_first + i;
                if (y >= k.oh) break;
                const int yin = (int)img_y(g, y);
                for (int e = 0; e < EPV; ++e) {
                    const int xin = (int)img_x(g, k.ow, x + e);
                    T s[C];
                    float v[C];
#pragma unroll
                    for (int c = 0; c < C; ++c) s[c] = tap_global(img + c * plane, k.w, k.h, xin, yin, Elem<T>::from_f(0.0f));
                    col.apply(k, s, v);
#pragma unroll
                    for (int c = 0; c < C; ++c) Elem<T>::store(out + c * oplane + (size_t)y * k.ow + x + e, v[c]);
                }
            }
        }
    }
}

}  // namespace ta
