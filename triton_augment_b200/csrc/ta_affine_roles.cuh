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
// The same with the row's terms taken from the tile descriptor: yc and byc = b * yc (TileInfo).
template <int R>
__device__ __forceinline__ float2 src_coord2_rows(float2 xc, float2 a, float2 b, float2 yc, float2 byc, float2 c, float2 half,
                                                  float2 neg_half)
{
    float2 u = R == 1 ? pk_fma(xc, a, byc) : pk_fma(yc, b, pk_mul(a, xc));
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
template <typename T, int C, int MODE, bool CHECK, typename S, int TH> struct PairSampler {
    static constexpr int PITCH = Src<S>::pitch, PLANE = Stage<S, TH>::plane;
    static constexpr uint32_t ES = sizeof(S), ROWB = ES * PITCH, PLANEB = ES * PLANE;
    using P = Px<T, S>;
    using Pair = typename PairOf<T>::type;

    // -> smp[c] = (first pixel of the pair, second pixel)
    static __device__ __forceinline__ void window(const Const2 &k2, uint32_t stage_addr, uint32_t kb, int rows, int row0,
                                                  int xs0, float2 sx, float2 sy, Pair (&smp)[C],
                                                  unsigned long long &n_viol)
    {
        const float2 magic = k2.magic, unmagic = k2.neg_magic;
        if (MODE != 2) {
            const float2 tx = pk_add(sx, magic), ty = pk_add(sy, magic);
            uint32_t addr[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t bx = __float_as_uint(j ? tx.y : tx.x), by = __float_as_uint(j ? ty.y : ty.x);
                addr[j] = kb + by * ROWB + bx * ES;
                if (CHECK) {
                    const int r = (int)(by - (uint32_t)kMagicBits) - row0, x = (int)(bx - (uint32_t)kMagicBits) - xs0;
                    if ((unsigned)r >= (unsigned)rows || (unsigned)x >= (unsigned)PITCH) { ++n_viol; addr[j] = stage_addr; }
                }
            }
#pragma unroll
            for (int c = 0; c < C; ++c) smp[c] = P::pair(P::lds(addr[0] + c * PLANEB), P::lds(addr[1] + c * PLANEB));
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
                smp[c] = PairOf<T>::from_f2(acc);
            }
        }
    }

    static __device__ __forceinline__ void table(const Const2 &k2, const S *stage, const int *rowoff, int rows,
                                                 int row0, float2 sx, float2 sy, Pair (&smp)[C],
                                                 unsigned long long &n_viol)
    {
        if (MODE != 2) {
            int idx[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int xn = rint_magic(j ? sx.y : sx.x);
                int r = rint_magic(j ? sy.y : sy.x) - row0;
                if (CHECK && (unsigned)r >= (unsigned)rows) { ++n_viol; r = 0; }
                idx[j] = rowoff[r] + xn;
                if (CHECK && (unsigned)(idx[j] - r * PITCH) >= (unsigned)PITCH) { ++n_viol; idx[j] = 0; }
            }
#pragma unroll
            for (int c = 0; c < C; ++c) smp[c] = P::pair(stage[c * PLANE + idx[0]], stage[c * PLANE + idx[1]]);
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
                smp[c] = PairOf<T>::from_f2(acc);
            }
        }
    }
};

// Colour tier and stores of one pixel pair of a float image: two rows of one column.  plane[c]
// points at the thread's pixel in the first row of its tile strip, channel c; `row` (a
// compile-time constant after unrolling) is the pair's first row within the strip and row_bytes
// the byte pitch of an output row, so every store address is one multiply-add on a per-tile
// pointer.  Packed colour arithmetic measured 3 % faster than per-pixel scalar code, although
// most of its operands are broadcast pairs.
template <int C, unsigned F, int G = 0>
__device__ __forceinline__ void finish_pair(const KArgs &k, const Colour<float, C, F> &col, float2 (&v2)[C],
                                            float *const (&plane)[C], int row, unsigned row_bytes, bool a_ok, bool b_ok)
{
    auto at = [&](int c, int r) {
        return reinterpret_cast<float *>(reinterpret_cast<char *>(plane[c]) + (size_t)row_bytes * (unsigned)r);
    };
    col.template apply2<G>(k, v2);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        if (a_ok) Elem<float>::store(at(c, row), v2[c].x);
        if (b_ok) Elem<float>::store(at(c, row + 1), v2[c].y);
    }
}

// The same for a half image, whose pair is two neighbouring columns of one row (the reference's
// mixed half / float steps, two pixels at a time): one 32-bit store per channel when the pair
// is whole and output rows keep pairs 4-byte aligned (vec), else element stores.
// whole: every pair of the tile row is inside the image and aligned (uniform over the warp), so
// the stores need no per-lane tests.
template <int C, unsigned F, int G = 0>
__device__ __forceinline__ void finish_pair_x(const KArgs &k, const Colour<__half, C, F> &col, const __half2 (&smp)[C],
                                              __half *const (&plane)[C], int row, unsigned row_bytes, bool whole,
                                              bool row_ok, bool pair_ok)
{
    float2 v2[C];
    col.template apply2<G>(k, smp, v2);
    unsigned h[C];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const __half2 p = __floats2half2_rn(v2[c].x, v2[c].y);       // one packed conversion
        h[c] = *reinterpret_cast<const unsigned *>(&p);
    }
    auto at = [&](int c) { return reinterpret_cast<char *>(plane[c]) + (size_t)row_bytes * (unsigned)row; };
    if (whole || (pair_ok && k.pair_store)) {
        if (row_ok) {
#pragma unroll
            for (int c = 0; c < C; ++c) __stcs(reinterpret_cast<unsigned *>(at(c)), h[c]);
        }
    } else if (row_ok) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            __stcs(reinterpret_cast<unsigned short *>(at(c)), (unsigned short)(h[c] & 0xffffu));
            if (pair_ok) __stcs(reinterpret_cast<unsigned short *>(at(c)) + 1, (unsigned short)(h[c] >> 16));
        }
    }
}

// A consumer warp's share of a tile.  Float pixels: 32 columns x Shape::rows_per_warp rows, a lane owns one
// column and pairs the rows (full 128-byte lines per store instruction).  Half pixels: all 64
// columns x TH / kConsumerWarps rows, a lane owns two neighbouring columns and pairs THEM,
// so that a store is one 32-bit half2, a warp's store a full 128-byte line again, and shared
// memory is read at 4-byte lane stride (no bank conflicts) as in the float case.
// The mean of one image from its partial sums.  The order of the additions is part of the result,
// so it is fixed: 256 chains take the 16-byte groups of partials round-robin (chain t: groups t,
// t + 256, ...) and add each group's four values left to right, in double; a halving tree joins
// the chains (chain t += chain t + 128, then + 64, ... + 1).  Two implementations with the same
// order, hence the same bits: mean_finish_kernel (256 threads, one chain each, after the reduction
// launch) and mean_of_partials_by_warp (one warp, lane l running chains l, l + 32, ... l + 224: the
// two-phase kernel's finisher).  per_image is a multiple of 4 (kConsumerWarps partials per tile),
// the base 16-byte aligned.
__device__ __forceinline__ double chain_sum(const float4 *v, int groups, int chain)
{
    double s = 0.0;
    int m = chain;
    for (; m + 768 < groups; m += 1024) {            // four loads in flight
        const float4 a = __ldcg(v + m), b = __ldcg(v + m + 256), c = __ldcg(v + m + 512), d = __ldcg(v + m + 768);
        s += (double)a.x; s += (double)a.y; s += (double)a.z; s += (double)a.w;
        s += (double)b.x; s += (double)b.y; s += (double)b.z; s += (double)b.w;
        s += (double)c.x; s += (double)c.y; s += (double)c.z; s += (double)c.w;
        s += (double)d.x; s += (double)d.y; s += (double)d.z; s += (double)d.w;
    }
    for (; m < groups; m += 256) {
        const float4 a = __ldcg(v + m);
        s += (double)a.x; s += (double)a.y; s += (double)a.z; s += (double)a.w;
    }
    return s;
}

__device__ __forceinline__ float mean_of_partials_by_warp(const float *base, int per_image, int pixels, int lane)
{
    const float4 *v = reinterpret_cast<const float4 *>(base);
    const int groups = per_image >> 2;
    double a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = chain_sum(v, groups, lane + 32 * j);
#pragma unroll
    for (int j = 0; j < 4; ++j) a[j] += a[j + 4];          // + 128
    a[0] += a[2];                                           // + 64
    a[1] += a[3];
    a[0] += a[1];                                           // + 32
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const double other = __shfl_down_sync(0xffffffffu, a[0], o);
        if (lane < o) a[0] += other;
    }
    return (float)(a[0] / (double)pixels);            // valid in lane 0
}

__device__ __forceinline__ void finish_mean_by_warp(const KArgs &k, int n, int per_image, int lane)
{
    const float mean = mean_of_partials_by_warp(k.mean_partials + (size_t)n * per_image, per_image, k.mean_pixels, lane);
    if (lane == 0) {
        k.mean_out[n] = mean;
        __threadfence();
        *(volatile unsigned *)(k.mean_ready + n) = 1u;
    }
}

// The two-phase kernel's extra warp.  CTA b finishes the means of images b, b + grid, ...: it waits
// until the image's counter says that every partial sum is out, adds them up (mean_of_partials,
// ~10 us of latency that must not sit in any consumer's way: the consumer that happens to be
// last is by definition the slowest, and making it do this work made it slower still, image after
// image), and publishes the mean for the producers of the image's fused-pass tiles.  The wait has no
// fixed limit of its own - the last image's count completes only near the end of the launch - but
// it gives up when this CTA's consumers have made no progress for the wait limit (their heartbeat
// stands still) while the count is incomplete, or when the CTA has aborted.
__device__ __forceinline__ void two_phase_finisher(const KArgs &k, volatile int *abort_flag, volatile unsigned *heartbeat)
{
    const int lane = threadIdx.x & 31;
    const int per_image = k.tiles_x * k.tiles_y * kConsumerWarps;
    for (int n = blockIdx.x; n < k.n; n += gridDim.x) {
        int ok = 1;
        if (lane == 0) {
            const volatile unsigned *done = k.mean_done + n;
            unsigned beat = *heartbeat;
            unsigned long long t0 = global_ns();
            while (*done != (unsigned)per_image) {
                __nanosleep(256);
                if (*abort_flag) { ok = 0; break; }
                const unsigned now = *heartbeat;
                if (now != beat) { beat = now; t0 = global_ns(); }
                else if (global_ns() - t0 > k.wait_ns) { ok = 0; break; }
            }
            __threadfence();
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { *abort_flag = 1; return; }
        finish_mean_by_warp(k, n, per_image, lane);
    }
}

// TWO: tiles of both phases of the two-phase kernel arrive through the same ring; the tile's
// descriptor says which it is.
template <typename T, int C, int MODE, unsigned F, bool CHECK, bool MIX, typename S, bool REDUCE, bool TWO, int TH>
__device__ __forceinline__ void affine_consumer(const KArgs &k, unsigned char *smem, uint64_t *full, uint64_t *empty,
                                                volatile int *abort_flag, unsigned *two_phase_checkin)
{
    using Info = TileInfo<T, C, F, TH>;
    using Sampler = PairSampler<T, C, MODE, CHECK, S, TH>;
    using Smem = AffineSmem<T, C, F, S, TH>;
    using Pair = typename PairOf<T>::type;
    constexpr int STAGES = Ring<S, TH>::stages, INFO_SLOTS = Ring<S, TH>::info_slots;
    constexpr bool PAIR_X = sizeof(T) == 2;
    static_assert(!PAIR_X || (!MIX && !REDUCE && !TWO), "the per-pixel recipe and the mean pre-pass exist for float pixels only");
    static_assert(!TWO || (!REDUCE && !MIX && (F & kMean)), "the two-phase kernel is the mean-contrast pipeline");
    constexpr int ROWS_PER_WARP = PAIR_X ? TH / kConsumerWarps : Shape<TH>::rows_per_warp;
    static_assert(!PAIR_X || (kTileW == 64 && TH % kConsumerWarps == 0), "a warp covers whole tile rows in pairs of columns");
    static_assert(PAIR_X || TH == ROWS_PER_WARP * kConsumerWarps / 2, "two warps side by side per strip of rows");
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
    // the CTA's tile number i uses stage i % STAGES (for the (i / STAGES)-th time) and descriptor i % INFO_SLOTS
    int s = 0, slot = 0;
    uint32_t phase = 0;
    for (int tile = blockIdx.x; tile < k.num_tiles; tile += gridDim.x) {
        if (!mbar_wait_or_abort(&full[s], phase, abort_flag, k.wait_ns)) return;
        const S *stage = reinterpret_cast<const S *>(smem + s * Smem::stage);
        const Info *ti = reinterpret_cast<const Info *>(smem + STAGES * Smem::stage + (size_t)slot * Smem::info);
        const int4 h0 = *reinterpret_cast<const int4 *>(&ti->n);       // n, x0, y0, rows
        const int4 h1 = *reinterpret_cast<const int4 *>(&ti->row0);    // row0, window, xs0, -
        const int n = h0.x, rows = h0.w, row0 = h1.x;
        const bool reduce = REDUCE || (TWO && (h1.y & 2) != 0);          // this tile adds to its image's mean
        const int key = TWO ? 2 * n + (reduce ? 1 : 0) : n;
        if (key != cur_n) {          // per-image parameters change only every few tiles (warp-uniform branch)
            g = ti->g;
            g2.set(g);
            col = ti->col;
            cur_n = key;
        }
        const int x = PAIR_X ? h0.y + 2 * lane : h0.y + wx * 32 + lane;
        const int y_first = h0.z + (PAIR_X ? warp : wy) * ROWS_PER_WARP;
        float mean_acc = 0.0f;               // REDUCE: this lane's share of the tile's sum
        bool released = false;               // the stage has been handed back before the end of the tile

        if (rows == 0) {
            if constexpr (TWO) {
                if (reduce) affine_rows_direct<T, C, MODE, F, MIX, S, true>(k, g, col, n, x, y_first, ROWS_PER_WARP, &mean_acc);
                else        affine_rows_direct<T, C, MODE, F, MIX, S, false>(k, g, col, n, x, y_first, ROWS_PER_WARP, &mean_acc);
            } else {
                affine_rows_direct<T, C, MODE, F, MIX, S, REDUCE>(k, g, col, n, x, y_first, ROWS_PER_WARP, &mean_acc);
                if (PAIR_X) affine_rows_direct<T, C, MODE, F, MIX, S, REDUCE>(k, g, col, n, x + 1, y_first, ROWS_PER_WARP, &mean_acc);
            }
        } else if (x < k.ow) {
            T *plane[C];
            plane[0] = (T *)k.out + (size_t)n * C * oplane + (unsigned)(y_first * k.ow + x);
#pragma unroll
            for (int c = 1; c < C; ++c) plane[c] = plane[c - 1] + oplane;
            const unsigned row_bytes = (unsigned)k.ow * (unsigned)sizeof(T);
            const bool window = (h1.y & 1) != 0;
            const int xs0 = h1.z;
            const uint32_t stage_addr = smem_u32(stage);
            const uint32_t kb = stage_addr - Sampler::ES * (uint32_t)(row0 * Sampler::PITCH + xs0)
                                - Sampler::ES * (uint32_t)(Sampler::PITCH + 1) * (uint32_t)kMagicBits;
            if constexpr (PAIR_X) {
                // The pair: columns x and x + 1 of one row.  A pair cut by the image's right edge is
                // computed on the last column twice (always staged) and stores one element.
                const bool pair_ok = x + 1 < k.ow;
                const float xi0 = img_x(g, k.ow, x), xi1 = img_x(g, k.ow, pair_ok ? x + 1 : x);
                // MODE 0 (no matrix): the source column is (int)x_img, as in the crop kernels
                const float2 xc = MODE == 0 ? f2(truncf(xi0), truncf(xi1)) : f2(centred(xi0, g.half_w), centred(xi1, g.half_w));
                const bool whole = k.pair_store != 0 && h0.y + kTileW <= k.ow;       // the same for every lane
                // The strip's rows, compiled twice: a tile whose rows and pairs all lie inside the
                // image and whose rows share one window (almost all tiles) needs no row clamps, no
                // store predicates and no per-row choice of the sampling path.
                auto rows_of_pairs = [&](auto fast_tile, auto gray_known) {
                    constexpr bool FAST = decltype(fast_tile)::value;
                    constexpr int G = decltype(gray_known)::value;
                    // sample row r of the strip
                    auto sample = [&](int r, Pair (&smp)[C]) {
                        // no early exit: a row past the image's last row is computed on the last row's geometry
                        // (the descriptor's row terms are clamped)
                        const int tr = warp * ROWS_PER_WARP + r;           // row within the tile
                        float2 sx, sy;
                        if (MODE == 0) {
                            sx = xc;
                            sy = bcast(ti->row_y[tr]);
                        } else {
                            const float2 yc = bcast(ti->row_y[tr]);
                            sx = src_coord2_rows<CoordRecipe<MODE, F>::x>(xc, g2.a, g2.b, yc, bcast(ti->row_b[tr]), g2.c, g2.half_w, k2.neg_half);
                            sy = src_coord2_rows<CoordRecipe<MODE, F>::y>(xc, g2.d, g2.e, yc, bcast(ti->row_e[tr]), g2.f, g2.half_h, k2.neg_half);
                        }
                        if (FAST || window) Sampler::window(k2, stage_addr, kb, rows, row0, xs0, sx, sy, smp, n_viol);
                        else                Sampler::table(k2, stage, ti->rowoff, rows, row0, sx, sy, smp, n_viol);
                    };
                    if constexpr (FAST && !REDUCE && MODE != 2) {
                        // Whole tiles, one texel per pixel: all samples first, then the stage goes back to the
                        // producer - its next copies travel while this warp runs the colour tier and the
                        // stores, which touch neither the stage nor the descriptor (512 x 3 x 512^2 -> 448^2
                        // nearest 240 -> 230 us; bilinear: no gain).  FAST means that the tile has all its 64
                        // columns, so all 32 lanes are here, as __syncwarp() requires.
                        Pair smp[ROWS_PER_WARP][C];
#pragma unroll
                        for (int r = 0; r < ROWS_PER_WARP; ++r) sample(r, smp[r]);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&empty[s]);
                        released = true;
#pragma unroll
                        for (int r = 0; r < ROWS_PER_WARP; ++r)
                            finish_pair_x<C, F, G>(k, col, smp[r], plane, r, row_bytes, true, true, true);
                    } else {
#pragma unroll
                        for (int r = 0; r < ROWS_PER_WARP; ++r) {
                            const bool row_ok = FAST || y_first + r < k.oh;
                            Pair smp[C];
                            sample(r, smp);
                            if constexpr (!REDUCE) finish_pair_x<C, F, G>(k, col, smp, plane, r, row_bytes, FAST || whole, row_ok, FAST || pair_ok);
                        }
                    }
                };
                // (the whole-tile copy twice more where grayscale is compiled in: the image's flag is then
                // tested once per tile, not once per pixel pair - 512 x 3 x 512^2 -> 448^2 nearest 260 -> 248 us)
                using g_any = std::integral_constant<int, 0>;
                if (!(window && whole && y_first + ROWS_PER_WARP <= k.oh)) rows_of_pairs(std::false_type{}, g_any{});
                else if (!(C == 3 && (F & kG))) rows_of_pairs(std::true_type{}, g_any{});
                else if (col.gray) rows_of_pairs(std::true_type{}, std::integral_constant<int, 2>{});
                else rows_of_pairs(std::true_type{}, std::integral_constant<int, 1>{});
            } else {
                // MODE 0 (no matrix): the source column is (int)x_img, as in the crop kernels
                const float2 xc = bcast(MODE == 0 ? truncf(img_x(g, k.ow, x)) : centred(img_x(g, k.ow, x), g.half_w));
                // The strip's row pairs, compiled three times: tiles that lie wholly above the image's
                // last row (almost all) need no row clamps and no store predicates; the window /
                // table choice is made once per tile instead of once per pair.
                auto row_pairs = [&](auto inside_rows, auto use_window) {
                    constexpr bool INSIDE = decltype(inside_rows)::value, WINDOW = decltype(use_window)::value;
                    // sample pair pr of the strip (rows 2 pr and 2 pr + 1)
                    auto sample = [&](int pr, Pair (&smp)[C]) {
                        // No early exit: rows past the image's last row are computed on the last row's
                        // geometry (always staged; the descriptor's row terms are clamped) and only their
                        // stores are dropped, so the pairs stay independent and their instructions can interleave.
                        const int tr = wy * ROWS_PER_WARP + 2 * pr;          // first row of the pair within the tile
                        const float2 yc = *reinterpret_cast<const float2 *>(&ti->row_y[tr]);
                        float2 sx, sy;
                        if (MODE == 0) {
                            sx = xc;
                            sy = yc;
                        } else {
                            const float2 byc = *reinterpret_cast<const float2 *>(&ti->row_b[tr]);
                            const float2 eyc = *reinterpret_cast<const float2 *>(&ti->row_e[tr]);
                            // (the reduction uses the contraction of its own stand-alone kernel, whose
                            // flags are brightness or nothing: the two paths must add up the same samples)
                            if (TWO && CoordRecipe<MODE, F>::swapped && reduce) {
                                sx = src_coord2_rows<CoordRecipe<MODE, F & kB>::x>(xc, g2.a, g2.b, yc, byc, g2.c, g2.half_w, k2.neg_half);
                                sy = src_coord2_rows<CoordRecipe<MODE, F & kB>::y>(xc, g2.d, g2.e, yc, eyc, g2.f, g2.half_h, k2.neg_half);
                            } else {
                                sx = src_coord2_rows<CoordRecipe<MODE, F>::x>(xc, g2.a, g2.b, yc, byc, g2.c, g2.half_w, k2.neg_half);
                                sy = src_coord2_rows<CoordRecipe<MODE, F>::y>(xc, g2.d, g2.e, yc, eyc, g2.f, g2.half_h, k2.neg_half);
                            }
                            if constexpr (MIX) {                  // see late_x()
                                const float2 alt = src_coord2_rows<1>(xc, g2.a, g2.b, yc, byc, g2.c, g2.half_w, k2.neg_half);
                                const int y_raw = y_first + 2 * pr;
                                const int ya = INSIDE ? y_raw : min(y_raw, k.oh - 1), yb = INSIDE ? y_raw + 1 : min(y_raw + 1, k.oh - 1);
                                const uint32_t base = k.lin_base + (uint32_t)n * oplane + (uint32_t)x;
                                if (late_x(k, base + (uint32_t)(ya * k.ow))) sx.x = alt.x;
                                if (late_x(k, base + (uint32_t)(yb * k.ow))) sx.y = alt.y;
                            }
                        }
                        if (WINDOW) Sampler::window(k2, stage_addr, kb, rows, row0, xs0, sx, sy, smp, n_viol);
                        else        Sampler::table(k2, stage, ti->rowoff, rows, row0, sx, sy, smp, n_viol);
                    };
                    if constexpr (INSIDE && !REDUCE && !TWO && MODE != 2) {
                        // Whole strips, one texel per pixel: all samples first, then the stage goes back to
                        // the producer - its next copies travel while this warp runs the colour tier and
                        // the stores, which touch neither the stage nor the descriptor (64 x 3 x 1280^2 ->
                        // 1024^2 nearest 260 -> 256 us).  Not for bilinear sampling, where holding every
                        // pair's blended texels until the release measured 1-2 % slower.  INSIDE means that
                        // all 32 lanes are here (see the call), as __syncwarp() requires.
                        Pair smp[ROWS_PER_WARP / 2][C];
#pragma unroll
                        for (int pr = 0; pr < ROWS_PER_WARP / 2; ++pr) sample(pr, smp[pr]);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&empty[s]);
                        released = true;
#pragma unroll
                        for (int pr = 0; pr < ROWS_PER_WARP / 2; ++pr) finish_pair<C, F>(k, col, smp[pr], plane, 2 * pr, row_bytes, true, true);
                    } else {
#pragma unroll
                        for (int pr = 0; pr < ROWS_PER_WARP / 2; ++pr) {
                            const int y_raw = y_first + 2 * pr;
                            const bool a_ok = INSIDE || y_raw < k.oh, b_ok = INSIDE || y_raw + 1 < k.oh;
                            Pair smp[C];
                            sample(pr, smp);
                            if constexpr (REDUCE || TWO) {
                                if (reduce) {
                                    float pa[C], pb[C];
#pragma unroll
                                    for (int c = 0; c < C; ++c) { pa[c] = smp[c].x; pb[c] = smp[c].y; }
                                    if (a_ok) mean_acc += mean_term<C, F>(col, pa);
                                    if (b_ok) mean_acc += mean_term<C, F>(col, pb);
                                }
                            }
                            if constexpr (!REDUCE) {
                                if (!reduce) finish_pair<C, F>(k, col, smp, plane, 2 * pr, row_bytes, a_ok, b_ok);
                            }
                        }
                    }
                };
                using yes = std::true_type;
                using no = std::false_type;
                // (testing the grayscale flag once per tile, as the half-pixel path does, measured no
                // gain here: bilinear 298 -> 297 us, fastest block 275 -> 278 us)
                // (whole strip: all its rows above the image's last row and all 32 columns inside)
                if (!window) row_pairs(no{}, no{});
                else if (y_first + ROWS_PER_WARP <= k.oh && h0.y + wx * 32 + 32 <= k.ow) row_pairs(yes{}, yes{});
                else row_pairs(no{}, yes{});
            }
        }
        __syncwarp();
        if constexpr (REDUCE || TWO) {
            if (reduce) {
                // one partial per (tile, warp), lanes added in a fixed order: the mean does not
                // depend on which CTA ran the tile or when
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mean_acc += __shfl_xor_sync(0xffffffffu, mean_acc, o);
                if (lane == 0) k.mean_partials[(size_t)h1.w * kConsumerWarps + warp] = mean_acc;
                if constexpr (TWO) {
                    // Counting the finished partials: once per image and CTA, not per tile - thousands
                    // of additions to one address per image serialise in the L2.  On the CTA's last
                    // reduction tile of the image every consumer warp checks in at a shared counter;
                    // the last of them adds the CTA's share to the image's global counter.  Nobody
                    // here waits for the count to complete: the image's finisher warp does (below).
                    const int r_count = ti->r_count;
                    if (r_count > 0 && lane == 0) {
                        __threadfence();                                       // this warp's partials are out
                        if (atomicAdd(&two_phase_checkin[n & 3], 1u) == (unsigned)(kConsumerWarps - 1)) {
                            two_phase_checkin[n & 3] = 0u;                     // (no warp can be four images ahead)
                            __threadfence();
                            atomicAdd(k.mean_done + n, (unsigned)(r_count * kConsumerWarps));
                        }
                    }
                }
            }
        }
        if (lane == 0 && !released) mbar_arrive(&empty[s]);
        if (TWO && threadIdx.x == 0) *(volatile unsigned *)&two_phase_checkin[4] += 1u;     // heartbeat for the finisher
        if (++s == STAGES) { s = 0; phase ^= 1u; }
        if (++slot == INFO_SLOTS) slot = 0;
    }
    if (CHECK && n_viol && k.counters) atomicAdd(k.counters + kCntViolation, n_viol);
}

// ----------------------------------------------------------------------------- kernel
// MIX: the variant of a swapped bilinear kernel (CoordRecipe) that applies late_x() per pixel.
// REDUCE: the grayscale-mean pre-pass on the same machinery (no colour tier, no image output).
// TWO: reduction and fused pass of the mean-contrast pipeline in one (cooperative) launch.
template <typename T, int C, int MODE, unsigned F, bool CHECK, bool MIX = false, typename S = T, bool REDUCE = false,
          bool TWO = false, int TH = kTileH>
__global__ void __launch_bounds__(Ring<S, TH>::threads + (TWO ? 32 : 0), 1)
affine_kernel(const __grid_constant__ KArgs k, const __grid_constant__ TMaps maps)
{
    // Used as declared (no pointer arithmetic through integers), so the compiler keeps every
    // access in the shared address space.  Tensor copies without swizzle need 16-byte alignment.
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full[Ring<S, TH>::stages];
    __shared__ __align__(8) uint64_t empty[Ring<S, TH>::stages];
    __shared__ int abort_flag;
    __shared__ unsigned two_phase_checkin[5];       // [0..3] consumer check-ins per image in flight, [4] consumer heartbeat

    if (threadIdx.x == 0) {
        for (int i = 0; i < Ring<S, TH>::stages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kConsumerWarps);
        }
        abort_flag = 0;
        two_phase_checkin[0] = two_phase_checkin[1] = two_phase_checkin[2] = two_phase_checkin[3] = two_phase_checkin[4] = 0u;
        mbar_fence_init();
    }
    __syncthreads();

    if (TWO && (threadIdx.x >> 5) >= kConsumerWarps + Ring<S, TH>::stages)
        two_phase_finisher(k, &abort_flag, &two_phase_checkin[4]);
    else if ((threadIdx.x >> 5) >= kConsumerWarps)
        affine_producer<T, C, MODE, F, S, TWO, TH>(k, maps, smem, full, empty, &abort_flag, (int)(threadIdx.x >> 5) - kConsumerWarps);
    else
        affine_consumer<T, C, MODE, F, CHECK, MIX, S, REDUCE, TWO, TH>(k, smem, full, empty, &abort_flag, two_phase_checkin);

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
        if (threadIdx.x < Ring<S, TH>::stages) {
            for (int i = 0; i < 4096; ++i)
                if (mbar_try_wait(&full[threadIdx.x], 0) || mbar_try_wait(&full[threadIdx.x], 1)) break;
        }
    }
}

}  // namespace ta
