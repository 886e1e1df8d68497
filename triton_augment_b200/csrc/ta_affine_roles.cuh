// Producer and consumer roles of the staged affine kernel, and the kernel itself.
#pragma once

namespace ta {

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// A packed operand whose halves hold the same value.  Packed instructions read an aligned
// register pair, so a broadcast scalar costs two register copies wherever it is used unless it
// lives in a pair of its own; hiding the halves from the optimiser (it would otherwise merge
// two copies of one value and re-create the pair at every use) keeps it there.
__device__ __forceinline__ float2 bcast(float v)
{
    float2 p = make_float2(v, v);
    asm volatile("" : "+f"(p.x), "+f"(p.y));
    return p;
}

// Per-image geometry as packed operands.
struct Geom2 {
    float2 a, b, c, d, e, f, half_w, half_h, top, neg_half_h;
    __device__ __forceinline__ void set(const Geom &g)
    {
        a = bcast(g.a); b = bcast(g.b); c = bcast(g.c); d = bcast(g.d); e = bcast(g.e); f = bcast(g.f);
        half_w = bcast(g.half_w); half_h = bcast(g.half_h); top = bcast(g.top); neg_half_h = bcast(-g.half_h);
    }
};

// Literal constants as packed operands, set up once per thread.
struct Const2 {
    float2 half, neg_half, one, neg_one, magic, neg_magic, neg_two23;
    __device__ __forceinline__ void set()
    {
        half = bcast(0.5f); neg_half = bcast(-0.5f); one = bcast(1.0f); neg_one = bcast(-1.0f);
        magic = bcast(kMagic); neg_magic = bcast(-kMagic); neg_two23 = bcast(-8388608.0f);
    }
};

// Two source coordinates at once with the packed fp32 pipe; per lane the operation order of
// src_coord_r(): ((fma + c) + half) + (-0.5), each step rounded to nearest.
// R picks which product is fused into the addition (see CoordRecipe).
template <int R>
__device__ __forceinline__ float2 src_coord2(float2 xc, float2 a, float2 b, float2 yc, float2 c, float2 half,
                                             float2 neg_half)
{
    float2 u = R == 1 ? pk_fma(xc, a, pk_mul(b, yc)) : pk_fma(yc, b, pk_mul(a, xc));
    u = pk_add(u, c);
    u = pk_add(half, u);
    return pk_add(u, neg_half);
}

}  // namespace ta

#include "ta_affine_producer.cuh"

namespace ta {

// ----------------------------------------------------------------------------- consumer
// Texels of one pixel pair (two output rows, same column) from a stage, two ways.
//
// Window path (TileInfo::window): all staged rows start at column xs0, so texel (y, x) lives at
// byte  stage + ES * ((y - row0) * pitch + (x - xs0)).  The integers y and x never exist as
// such: adding 1.5 * 2^23 to a coordinate leaves rint / floor of it in the low bits of the
// float, and address = kb + ES * pitch * bits(y) + ES * bits(x) with every constant (stage
// base, row0, xs0, the two magic offsets) folded into kb once per tile, modulo 2^32.
//
// Table path: each row group has its own first column; rowoff[] translates.
template <typename T, int C, int MODE, bool CHECK, typename S> struct PairSampler {
    static constexpr int PITCH = Src<S>::pitch, PLANE = Src<S>::plane;
    static constexpr uint32_t ES = sizeof(S), ROWB = ES * PITCH, PLANEB = ES * PLANE;
    using P = Px<T, S>;

    // -> smp[j][c], j = 0 / 1 for the pair's first / second row
    static __device__ __forceinline__ void window(const Const2 &k2, uint32_t stage_addr, uint32_t kb, int rows, int row0,
                                                  int xs0, float2 sx, float2 sy, T (&smp)[2][C],
                                                  unsigned long long &n_viol)
    {
        const float2 magic = k2.magic, unmagic = k2.neg_magic;
        if (MODE != 2) {
            const float2 tx = pk_add(sx, magic), ty = pk_add(sy, magic);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t bx = __float_as_uint(j ? tx.y : tx.x), by = __float_as_uint(j ? ty.y : ty.x);
                uint32_t addr = kb + by * ROWB + bx * ES;
                if (CHECK) {
                    const int r = (int)(by - (uint32_t)kMagicBits) - row0, x = (int)(bx - (uint32_t)kMagicBits) - xs0;
                    if ((unsigned)r >= (unsigned)rows || (unsigned)x >= (unsigned)PITCH) { ++n_viol; addr = stage_addr; }
                }
#pragma unroll
                for (int c = 0; c < C; ++c) smp[j][c] = P::from(P::lds(addr + c * PLANEB));
            }
        } else {
            const float2 tx = pk_add_rd(sx, magic), ty = pk_add_rd(sy, magic);
            const float2 neg = k2.neg_one, one = k2.one;
            const float2 dx = pk_fma(pk_add(tx, unmagic), neg, sx);      // s - floor(s), exact
            const float2 dy = pk_fma(pk_add(ty, unmagic), neg, sy);
            uint32_t addr[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t bx = __float_as_uint(j ? tx.y : tx.x), by = __float_as_uint(j ? ty.y : ty.x);
                addr[j] = kb + by * ROWB + bx * ES;
                if (CHECK) {
                    const int r = (int)(by - (uint32_t)kMagicBits) - row0, x = (int)(bx - (uint32_t)kMagicBits) - xs0;
                    if ((unsigned)r >= (unsigned)(rows - 1) || (unsigned)x >= (unsigned)(PITCH - 1)) {
                        ++n_viol; addr[j] = stage_addr;
                    }
                }
            }
            const float2 omx = pk_fma(dx, neg, one), omy = pk_fma(dy, neg, one);   // 1 - d, one rounding
            const float2 w00 = pk_mul(omx, omy), w10 = pk_mul(dx, omy);
            const float2 w01 = pk_mul(omx, dy), w11 = pk_mul(dx, dy);
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const uint32_t a0 = addr[0] + c * PLANEB, a1 = addr[1] + c * PLANEB;
                float2 acc = pk_mul(P::raw_f2(P::lds(a0), P::lds(a1)), w00);
                acc = pk_fma(P::raw_f2(P::lds(a0 + ES), P::lds(a1 + ES)), w10, acc);
                acc = pk_fma(P::raw_f2(P::lds(a0 + ROWB), P::lds(a1 + ROWB)), w01, acc);
                acc = pk_fma(P::raw_f2(P::lds(a0 + ROWB + ES), P::lds(a1 + ROWB + ES)), w11, acc);
                if (P::scaled) acc = pk_mul(acc, f2(kInv255, kInv255));
                smp[0][c] = Elem<T>::from_f(acc.x);
                smp[1][c] = Elem<T>::from_f(acc.y);
            }
        }
    }

    static __device__ __forceinline__ void table(const Const2 &k2, const S *stage, const int *rowoff, int rows,
                                                 int row0, float2 sx, float2 sy, T (&smp)[2][C],
                                                 unsigned long long &n_viol)
    {
        if (MODE != 2) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int xn = rint_magic(j ? sx.y : sx.x);
                int r = rint_magic(j ? sy.y : sy.x) - row0;
                if (CHECK && (unsigned)r >= (unsigned)rows) { ++n_viol; r = 0; }
                int idx = rowoff[r] + xn;
                if (CHECK && (unsigned)(idx - r * PITCH) >= (unsigned)PITCH) { ++n_viol; idx = 0; }
#pragma unroll
                for (int c = 0; c < C; ++c) smp[j][c] = P::from(stage[c * PLANE + idx]);
            }
        } else {
            int i0[2], i1[2];
            float2 dx, dy;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float frac_x, frac_y;
                const int x0 = floor_magic(j ? sx.y : sx.x, frac_x), y0 = floor_magic(j ? sy.y : sy.x, frac_y);
                (j ? dx.y : dx.x) = frac_x;
                (j ? dy.y : dy.x) = frac_y;
                int r = y0 - row0;
                if (CHECK && (unsigned)r >= (unsigned)(rows - 1)) { ++n_viol; r = 0; }
                i0[j] = rowoff[r] + x0;
                i1[j] = rowoff[r + 1] + x0;
                if (CHECK && ((unsigned)(i0[j] - r * PITCH) >= (unsigned)(PITCH - 1) ||
                              (unsigned)(i1[j] - (r + 1) * PITCH) >= (unsigned)(PITCH - 1))) {
                    ++n_viol; i0[j] = i1[j] = 0;
                }
            }
            const float2 one = k2.one, neg = k2.neg_one;
            const float2 omx = pk_fma(dx, neg, one), omy = pk_fma(dy, neg, one);
            const float2 w00 = pk_mul(omx, omy), w10 = pk_mul(dx, omy);
            const float2 w01 = pk_mul(omx, dy), w11 = pk_mul(dx, dy);
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const S *pl = stage + c * PLANE;
                float2 acc = pk_mul(P::raw_f2(pl[i0[0]], pl[i0[1]]), w00);
                acc = pk_fma(P::raw_f2(pl[i0[0] + 1], pl[i0[1] + 1]), w10, acc);
                acc = pk_fma(P::raw_f2(pl[i1[0]], pl[i1[1]]), w01, acc);
                acc = pk_fma(P::raw_f2(pl[i1[0] + 1], pl[i1[1] + 1]), w11, acc);
                if (P::scaled) acc = pk_mul(acc, f2(kInv255, kInv255));
                smp[0][c] = Elem<T>::from_f(acc.x);
                smp[1][c] = Elem<T>::from_f(acc.y);
            }
        }
    }
};

// Colour tier and stores of one pixel pair.  plane[c] points at the thread's pixel in the first
// row of its tile strip, channel c; `row` (a compile-time constant after unrolling) is the
// pair's first row within the strip and row_bytes the byte pitch of an output row, so every
// store address is one multiply-add on a per-tile pointer.
template <typename T, int C, unsigned F>
__device__ __forceinline__ void finish_pair(const KArgs &k, const Colour<T, C, F> &col, T (&smp)[2][C],
                                            T *const (&plane)[C], int row, unsigned row_bytes, bool a_ok, bool b_ok)
{
    auto at = [&](int c, int r) {
        return reinterpret_cast<T *>(reinterpret_cast<char *>(plane[c]) + (size_t)row_bytes * (unsigned)r);
    };
    // fp32: packed colour arithmetic (measured 3 % faster than per-pixel scalar code, although
    // most of its operands are broadcast pairs); fp16 follows the reference's mixed-precision
    // steps per pixel.
    constexpr bool packed_colour = sizeof(T) == 4;
    if constexpr (packed_colour) {
        float2 v2[C];
#pragma unroll
        for (int c = 0; c < C; ++c) v2[c] = f2(smp[0][c], smp[1][c]);
        col.apply2(k, v2);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            if (a_ok) Elem<T>::store(at(c, row), v2[c].x);
            if (b_ok) Elem<T>::store(at(c, row + 1), v2[c].y);
        }
    } else {
        float2 v2[C];
        col.apply2(k, smp[0], smp[1], v2);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            if (a_ok) Elem<T>::store(at(c, row), v2[c].x);
            if (b_ok) Elem<T>::store(at(c, row + 1), v2[c].y);
        }
    }
}

template <typename T, int C, int MODE, unsigned F, bool CHECK, bool MIX, typename S, bool REDUCE>
__device__ __forceinline__ void affine_consumer(const KArgs &k, unsigned char *smem, uint64_t *full, uint64_t *empty,
                                                volatile int *abort_flag)
{
    using Info = TileInfo<T, C, F>;
    using Sampler = PairSampler<T, C, MODE, CHECK, S>;
    using Smem = AffineSmem<T, C, F, S>;
    constexpr int ROWS_PER_WARP = kRowsPerWarp;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wx = warp & 1, wy = warp >> 1;
    const unsigned oplane = (unsigned)(k.oh * k.ow);
    unsigned long long n_viol = 0;
    int cur_n = -1;
    Geom g;
    Geom2 g2;
    Const2 k2;
    k2.set();
    Colour<T, C, F> col;
    int it = 0;
    for (int tile = blockIdx.x; tile < k.num_tiles; tile += gridDim.x, ++it) {
        const int s = it % kStages, use = it / kStages;
        if (!mbar_wait_or_abort(&full[s], (uint32_t)use & 1u, abort_flag, k.wait_ns)) return;
        const S *stage = reinterpret_cast<const S *>(smem + s * Smem::stage);
        const Info *ti = reinterpret_cast<const Info *>(smem + kStages * Smem::stage + (size_t)(it % kInfoSlots) * Smem::info);
        const int4 h0 = *reinterpret_cast<const int4 *>(&ti->n);       // n, x0, y0, rows
        const int4 h1 = *reinterpret_cast<const int4 *>(&ti->row0);    // row0, window, xs0, -
        const int n = h0.x, rows = h0.w, row0 = h1.x;
        if (n != cur_n) {            // per-image parameters change only every few tiles (warp-uniform branch)
            g = ti->g;
            g2.set(g);
            col = ti->col;
            cur_n = n;
        }
        const int x = h0.y + wx * 32 + lane;
        const int y_first = h0.z + wy * ROWS_PER_WARP;
        float mean_acc = 0.0f;               // REDUCE: this lane's share of the tile's sum

        if (rows == 0) {
            affine_rows_direct<T, C, MODE, F, MIX, S, REDUCE>(k, g, col, n, x, y_first, ROWS_PER_WARP, &mean_acc);
        } else if (x < k.ow) {
            T *plane[C];
            plane[0] = (T *)k.out + (size_t)n * C * oplane + (unsigned)(y_first * k.ow + x);
#pragma unroll
            for (int c = 1; c < C; ++c) plane[c] = plane[c - 1] + oplane;
            const unsigned row_bytes = (unsigned)k.ow * (unsigned)sizeof(T);
            // MODE 0 (no matrix): the source column is (int)x_img, as in the crop kernels
            const float2 xc = bcast(MODE == 0 ? truncf(img_x(g, k.ow, x)) : centred(img_x(g, k.ow, x), g.half_w));
            const bool window = h1.y != 0;
            const int xs0 = h1.z;
            const uint32_t stage_addr = smem_u32(stage);
            const uint32_t kb = stage_addr - Sampler::ES * (uint32_t)(row0 * Sampler::PITCH + xs0)
                                - Sampler::ES * (uint32_t)(Sampler::PITCH + 1) * (uint32_t)kMagicBits;
#pragma unroll
            for (int pr = 0; pr < ROWS_PER_WARP / 2; ++pr) {
                // No early exit: rows past the image's last row are computed on the last row's
                // geometry (always staged) and only their stores are dropped, so the pairs stay
                // independent and their instructions can interleave.
                const int y_raw = y_first + 2 * pr;
                const bool a_ok = y_raw < k.oh, b_ok = y_raw + 1 < k.oh;
                const int ya = min(y_raw, k.oh - 1), yb = min(y_raw + 1, k.oh - 1);
                // (float)y as 2^23 + y minus 2^23, then + top, - half_h, + 0.5: img_y() and centred()
                float2 yc = pk_add(f2(__int_as_float(0x4B000000 | ya), __int_as_float(0x4B000000 | yb)), k2.neg_two23);
                yc = pk_add(yc, g2.top);
                float2 sx, sy;
                if (MODE == 0) {
                    sx = xc;
                    sy = f2(truncf(yc.x), truncf(yc.y));
                } else {
                    yc = pk_add(pk_add(yc, g2.neg_half_h), k2.half);
                    sx = src_coord2<CoordRecipe<MODE, F>::x>(xc, g2.a, g2.b, yc, g2.c, g2.half_w, k2.neg_half);
                    sy = src_coord2<CoordRecipe<MODE, F>::y>(xc, g2.d, g2.e, yc, g2.f, g2.half_h, k2.neg_half);
                    if constexpr (MIX) {                  // see late_x()
                        const float2 alt = src_coord2<1>(xc, g2.a, g2.b, yc, g2.c, g2.half_w, k2.neg_half);
                        const uint32_t base = k.lin_base + (uint32_t)n * oplane + (uint32_t)x;
                        if (late_x(k, base + (uint32_t)(ya * k.ow))) sx.x = alt.x;
                        if (late_x(k, base + (uint32_t)(yb * k.ow))) sx.y = alt.y;
                    }
                }
                T smp[2][C];
                if (window) Sampler::window(k2, stage_addr, kb, rows, row0, xs0, sx, sy, smp, n_viol);
                else        Sampler::table(k2, stage, ti->rowoff, rows, row0, sx, sy, smp, n_viol);
                if constexpr (REDUCE) {
                    if (a_ok) mean_acc += mean_term<C, F>(col, smp[0]);
                    if (b_ok) mean_acc += mean_term<C, F>(col, smp[1]);
                } else {
                    finish_pair<T, C, F>(k, col, smp, plane, 2 * pr, row_bytes, a_ok, b_ok);
                }
            }
        }
        __syncwarp();
        if constexpr (REDUCE) {
            // one partial per (tile, warp), lanes added in a fixed order: the mean does not
            // depend on which CTA ran the tile or when
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mean_acc += __shfl_xor_sync(0xffffffffu, mean_acc, o);
            if (lane == 0) k.mean_partials[(size_t)tile * kConsumerWarps + warp] = mean_acc;
        }
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (CHECK && n_viol && k.counters) atomicAdd(k.counters + kCntViolation, n_viol);
}

// ----------------------------------------------------------------------------- kernel
// MIX: the variant of a swapped bilinear kernel (CoordRecipe) that applies late_x() per pixel.
// REDUCE: the grayscale-mean pre-pass on the same machinery (no colour tier, no image output).
template <typename T, int C, int MODE, unsigned F, bool CHECK, bool MIX = false, typename S = T, bool REDUCE = false>
__global__ void __launch_bounds__(kAffineThreads, 1)
affine_kernel(const __grid_constant__ KArgs k, const __grid_constant__ TMaps maps)
{
    // Used as declared (no pointer arithmetic through integers), so the compiler keeps every
    // access in the shared address space.  Tensor copies without swizzle need 16-byte alignment.
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full[kStages];
    __shared__ __align__(8) uint64_t empty[kStages];
    __shared__ int abort_flag;

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
        affine_producer<T, C, MODE, F, S>(k, maps, smem, full, empty, &abort_flag, (int)(threadIdx.x >> 5) - kConsumerWarps);
    else
        affine_consumer<T, C, MODE, F, CHECK, MIX, S, REDUCE>(k, smem, full, empty, &abort_flag);

    // Leave together.  After an abort, copies may still be in flight towards this CTA's shared
    // memory: give each stage one more bounded chance to settle before the memory is released.
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) {
            if (k.counters) atomicAdd(k.counters + kCntTimeout, 1ull);
            if (k.status) {
                *(volatile unsigned *)k.status = 1u;
                __threadfence_system();
            }
        }
        if (threadIdx.x < kStages) {
            for (int i = 0; i < 4096; ++i)
                if (mbar_try_wait(&full[threadIdx.x], 0) || mbar_try_wait(&full[threadIdx.x], 1)) break;
        }
    }
}

}  // namespace ta
