// Fused inverse-affine + crop + flip + colour + normalize kernel (nearest / bilinear; MODE 0:
// the same pipeline without a matrix).
//
// Persistent, warp-specialised, one CTA per SM.  The CTA walks output tiles of
// kTileW x kTileH pixels (grid-stride).  PRODUCER warps (one per stage) work ahead of the
// CONSUMER warps through a ring of shared-memory stages (Ring<S, TH>::stages of them):
//
//   producer  for each tile: map the tile's corners to the source (ta_footprint.h).  When
//             their bounding box fits one window of columns - the usual case - plan one TMA
//             tensor copy per channel (a box of all the tile's source rows); otherwise clip the
//             footprint per group of 8 rows and plan one copy per (group, channel).  Write the
//             tile's descriptor (decoded parameters, window origin) into a slot the consumers
//             are not reading, wait for the stage to be released, issue the copies; they
//             complete on the stage's "full" mbarrier.
//   consumer  wait for "full", sample from shared memory (lanes run along x: conflict-free
//             reads, every store a full 128-byte line), apply the colour tier in registers,
//             store, then release the stage on its "empty" mbarrier.
//
// TMA zero-fills whatever lies outside the image, which is exactly the reference's fill=0
// rule for out-of-range neighbours, so the sampling loop has no bounds tests.  A tile that
// cannot be staged (footprint too large: extreme zoom-out or rotation; rows not 16-byte
// aligned; fill != 0 at the image border) is gathered from global memory with per-tap bounds
// tests instead: the producer marks it and the consumers take that path.
//
// Every wait is bounded (KArgs::wait_ns).  When one runs out the CTA raises an abort flag, leaves
// its remaining tiles unwritten, counts the event in the device counters and sets the host-mapped
// status word, which the library's entry points read without synchronising: the next call on
// the device (and ta_b200_status()) reports the time-out.
#pragma once

#include <cuda.h>

#include "ta_common.cuh"

namespace ta {

// Launch shape, chosen by measurement on the 1280x1280 -> 1024x1024 workload (times: bilinear /
// nearest, power-capped clocks).  About half of a consumer thread's instructions are per-tile
// bookkeeping (barrier wait, descriptor, pointers, the column's coordinates), so the pixels a
// thread handles per tile matter more than the depth of the ring:
//   64x64 tiles, 16 consumer warps x 8 pixels per thread, 96 source rows; float sources fit two
//                such stages in shared memory, half and byte sources three: 298 / 269 us  <- built
//   64x32 tiles, 16 warps x 4 pixels, 64 rows, 3 stages: 322 / 275 us (half pixels: +14 %)
//   64x48 tiles, 16 warps x 6 pixels, 80 rows, 2 stages: 322 / 290 us (48 does not divide 1024)
//   64x40 tiles, 20 warps x 4 pixels, 3 stages: 3 % faster than 64x32, light variants 20 % slower
//   64x36 / 64x28 / 64x24 tiles with 18 / 14 / 24 warps x 4 pixels: equal or slower than 64x32
//   64x32 tiles, 8 warps x 8 pixels: bilinear +2 %, half pixels +12 % (too few warps to hide latency)
// Small outputs take the 64x32 shape with a deeper ring instead (TH = kTileHShort; three stages
// for float sources, four for half): with few tiles per image many are edge tiles with little
// work, and then the depth of the ring - how many tiles' copies are in flight - decides:
// 4096 x 3 x 96^2 float nearest 179 us against 228 us, 1024 x 3 x 256^2 -> 224^2 224 against 236 us;
// above 256 output rows (half pixels: above 96) the tall shape wins.
constexpr int kConsumerWarps = 16;
// Float pixels: two warps side by side per strip of rows, a thread's pixels are rows_per_warp rows
// of one column.  Half pixels: a warp covers whole tile rows.
template <int TH> struct Shape {
    static constexpr int H = TH, ROWS = TH == kTileHShort ? kMaxRowsShort : kMaxRows, GROUPS = ROWS / kGroupRows;
    static constexpr int rows_per_warp = 2 * TH / kConsumerWarps;
    static_assert(TH == kTileH || TH == kTileHShort, "two tile shapes exist");
    static_assert(rows_per_warp % 2 == 0, "rows are handled in pairs");
};

// Source element type S of a staged kernel whose pixels are T: S = T for float and half
// images; S = uint8_t with T = float or half reads bytes and scales them by 1/255 (what ToTensor does
// before the reference's pipeline) on the way from shared memory to registers.
template <typename S> struct Src {
    static constexpr int pitch = sizeof(S) == 1 ? kPitchBytes1 : sizeof(S) == 2 ? kPitchBytes2 : kPitch;   // staged row pitch, elements
    static constexpr int chunk = 16 / (int)sizeof(S);                      // elements per 16 bytes
};
// The ring of a kernel with source elements S and tile height TH.
template <typename S, int TH> struct Ring {
    // depth: what fits 227 KB of shared memory (float sources), four for the short tiles of half images
    static constexpr int stages = sizeof(S) == 4 ? (TH == kTileH ? 2 : 3) : (TH == kTileH ? 3 : 4);
    static constexpr int info_slots = 2 * stages;                          // tile descriptors: two per stage (see AffineSmem)
    static constexpr int threads = (kConsumerWarps + stages) * 32;         // one producer warp per stage
};
// Elements per channel per stage.
template <typename S, int TH> struct Stage { static constexpr int plane = Shape<TH>::ROWS * Src<S>::pitch; };
constexpr float kInv255 = 1.0f / 255.0f;

// Texel of type S -> pixel of type T.
template <typename T, typename S> struct Px {
    static constexpr bool scaled = false;
    static __device__ __forceinline__ T from(S v) { return v; }
    // two texels as a pixel pair
    static __device__ __forceinline__ typename PairOf<T>::type pair(S a, S b) { return PairOf<T>::make(a, b); }
    // two texels as blend operands
    static __device__ __forceinline__ float2 raw_f2(S a, S b) { return make_float2(Elem<T>::to_f(a), Elem<T>::to_f(b)); }
    static __device__ __forceinline__ S lds(uint32_t addr) { return Elem<T>::lds(addr); }
};
// Bytes.  int -> float conversions run on the quarter-rate pipe; for 0..255 the float
// 2^23 + b is the bit pattern 0x4B000000 | b, and both uses below stay exact: b * k as
// fma(2^23 + b, k, -2^23 k) (2^23 k is exact, one rounding, the same value as float(b) * k),
// the blend operand as (2^23 + b) - 2^23, two at once.
template <> struct Px<float, uint8_t> {
    static constexpr bool scaled = true;        // blends run on the raw 0..255 values, scaled once afterwards
    static __device__ __forceinline__ float biased(uint8_t v) { return __uint_as_float(0x4B000000u | (uint32_t)v); }
    static __device__ __forceinline__ float from(uint8_t v) { return __fmaf_rn(biased(v), kInv255, -8388608.0f * kInv255); }
    static __device__ __forceinline__ float2 pair(uint8_t a, uint8_t b)
    {
        return pk_fma(make_float2(biased(a), biased(b)), make_float2(kInv255, kInv255),
                      make_float2(-8388608.0f * kInv255, -8388608.0f * kInv255));
    }
    static __device__ __forceinline__ float2 raw_f2(uint8_t a, uint8_t b)
    {
        return pk_add(make_float2(biased(a), biased(b)), make_float2(-8388608.0f, -8388608.0f));
    }
    static __device__ __forceinline__ uint8_t lds(uint32_t addr)
    {
        uint32_t v;
        asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
        return (uint8_t)v;
    }
};

// Bytes to half pixels: the same exact scaling, rounded once to half; blends run in fp32 on the
// raw values like the float case.
template <> struct Px<__half, uint8_t> {
    static constexpr bool scaled = true;
    static __device__ __forceinline__ __half from(uint8_t v) { return __float2half_rn(Px<float, uint8_t>::from(v)); }
    static __device__ __forceinline__ __half2 pair(uint8_t a, uint8_t b) { return PairOf<__half>::from_f2(Px<float, uint8_t>::pair(a, b)); }
    static __device__ __forceinline__ float2 raw_f2(uint8_t a, uint8_t b) { return Px<float, uint8_t>::raw_f2(a, b); }
    static __device__ __forceinline__ uint8_t lds(uint32_t addr) { return Px<float, uint8_t>::lds(addr); }
};

constexpr int kNumGroups = kMaxRows / kGroupRows;         // tensor maps built per launch

// The input seen as [N*C, H, W].  rows[g] copies a box of Src::pitch columns x (g + 1) * kGroupRows
// rows of one plane: a window tile is one copy per channel.  rows[0] doubles as the per-group
// box of tiles whose groups start at different columns.
struct alignas(64) TMaps {
    CUtensorMap rows[kNumGroups];
};

template <typename T, int C, unsigned F, int TH> struct alignas(16) TileInfo {
    int n, x0, y0;        // image, first output column / row of the tile
    int rows, row0;       // staged source rows (rows == 0: gather this tile from global memory)
    int window;           // bit 0: every row starts at column xs0: texel (y, x) sits at element
    int xs0;              //   (y - row0) * pitch + (x - xs0) of a channel plane.  window bit 1: a tile of the
    int real_tile;        //   reduction phase (two-phase kernel).  real_tile = n * tiles per image + tile in image
    int r_count;          // two-phase kernel: > 0 on this CTA's last reduction tile of an image = how many it had
    int pad3[3];
    // Per tile row (clamped to the image's last row), computed once by the producer because every
    // lane of every consumer warp would otherwise repeat it: row_y = the row's source coordinate
    // term - (int)(y + top) without a matrix, else yc = ((y + top) - h/2) + 0.5, each step rounded as
    // in img_y() and centred() - and the two products of yc that the coordinate recipes fuse nothing
    // into (b * yc, e * yc).  Pairs of rows are read as one 8-byte load.
    float row_y[TH], row_b[TH], row_e[TH];
    Geom g;
    Colour<T, C, F> col;
    int rowoff[Shape<TH>::ROWS + 1];   // otherwise: rowoff[r] + x = element index of texel (row0 + r, x)
};

// Shared memory: Ring::stages pixel stages, then Ring::info_slots tile descriptors.  Tile number i of a CTA
// uses stage i % stages and descriptor i % info_slots, so the producer can write the descriptor
// of the stage's next tile while the consumers still read the current one, and only the copy
// itself has to wait for the stage to be released.
template <typename T, int C, unsigned F, typename S = T, int TH = kTileH> struct AffineSmem {
    static constexpr size_t stage = ((size_t)C * Stage<S, TH>::plane * sizeof(S) + 1023) / 1024 * 1024;
    static constexpr size_t info = (sizeof(TileInfo<T, C, F, TH>) + 15) / 16 * 16;
    static constexpr size_t total = Ring<S, TH>::stages * stage + Ring<S, TH>::info_slots * info;
    static_assert(total <= 227 * 1024, "stages and descriptors must fit one CTA's shared memory");
};

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Wait for a phase of an mbarrier for at most limit_ns, giving up early when another thread
// of the CTA has already given up.  No sleep between polls: a failed poll already parks the
// warp for a while; sleeping on top of it (tried for producers, 256 ns, and for consumers, 64 ns)
// changed nothing for heavy consumers and cost up to 8 % with light ones.
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                                   unsigned long long limit_ns)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (int i = 0; i < (1 << 24); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 63) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit_ns) break;
        }
    }
    *abort_flag = 1;
    return false;
}

// Gather rows [y_first, y_first + y_count) of one tile column from global memory (no staging).
// Value the grayscale-mean pre-pass sums for one pixel: gray(clamp(brightness * sample)), the
// image torchvision's contrast blends towards (fp32 images only).
template <int C, unsigned F>
__device__ __forceinline__ float mean_term(const Colour<float, C, F> &col, const float (&s)[C])
{
    float v[C];
#pragma unroll
    for (int c = 0; c < C; ++c) v[c] = (F & kB) ? __saturatef(s[c] * col.bf) : s[c];
    return C == 3 ? gray_of(v[0], v[C > 1 ? 1 : 0], v[C - 1]) : v[0];
}

// REDUCE: add mean_term() of every pixel to *acc instead of applying the colour tier and storing.
template <typename T, int C, int MODE, unsigned F, bool MIX, typename S, bool REDUCE = false>
__device__ __forceinline__ void affine_rows_direct(const KArgs &k, const Geom &g, const Colour<T, C, F> &col,
                                                   int n, int x, int y_first, int y_count, float *acc = nullptr)
{
    if (x >= k.ow) return;
    const S *img = (const S *)k.in + (size_t)n * C * k.h * k.w;
    T *out = (T *)k.out + (size_t)n * C * k.oh * k.ow;
    const size_t plane = (size_t)k.h * k.w, oplane = (size_t)k.oh * k.ow;
    T fillv[C];
#pragma unroll
    for (int c = 0; c < C; ++c) fillv[c] = Elem<T>::from_f(MODE == 0 ? 0.0f : k.fill[c]);
    // texel (xx, yy) of channel plane c as a pixel value; outside the image: the channel's fill value
    auto tap = [&](const S *pl, int c, int xx, int yy) -> T {
        const bool ok = (unsigned)xx < (unsigned)k.w && (unsigned)yy < (unsigned)k.h;
        return ok ? Px<T, S>::from(__ldg(pl + (size_t)yy * k.w + xx)) : fillv[c];
    };
    const float xi = img_x(g, k.ow, x);
    const float xc = centred(xi, g.half_w);
    for (int i = 0; i < y_count; ++i) {
        const int y = y_first + i;
        if (y >= k.oh) break;
        const float yi = img_y(g, y);
        const float yc = centred(yi, g.half_h);
        // (a reduction adds up the samples of its stand-alone kernel, compiled for brightness or nothing)
        constexpr unsigned RF = REDUCE ? (F & kB) : F;
        float sx = MODE == 0 ? truncf(xi) : src_coord_r<CoordRecipe<MODE, RF>::x>(xc, yc, g.a, g.b, g.c, g.half_w);
        if constexpr (MIX) {
            if (late_x(k, k.lin_base + (uint32_t)n * (uint32_t)oplane + (uint32_t)(y * k.ow + x)))
                sx = src_coord_r<1>(xc, yc, g.a, g.b, g.c, g.half_w);
        }
        const float sy = MODE == 0 ? truncf(yi) : src_coord_r<CoordRecipe<MODE, RF>::y>(xc, yc, g.d, g.e, g.f, g.half_h);
        T s[C];
        if (MODE != 2) {
            const int xn = __float2int_rn(sx), yn = __float2int_rn(sy);
#pragma unroll
            for (int c = 0; c < C; ++c) s[c] = tap(img + c * plane, c, xn, yn);
        } else {
            const int x0 = __float2int_rd(sx), y0 = __float2int_rd(sy);
            const float dx = sx - (float)x0, dy = sy - (float)y0;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const S *pl = img + c * plane;
                s[c] = Elem<T>::from_f(blend4(Elem<T>::to_f(tap(pl, c, x0, y0)), Elem<T>::to_f(tap(pl, c, x0 + 1, y0)),
                                              Elem<T>::to_f(tap(pl, c, x0, y0 + 1)), Elem<T>::to_f(tap(pl, c, x0 + 1, y0 + 1)),
                                              dx, dy));
            }
        }
        if constexpr (REDUCE) {
            *acc += mean_term<C, F>(col, s);
        } else {
            float v[C];
            col.apply(k, s, v);
#pragma unroll
            for (int c = 0; c < C; ++c) Elem<T>::store(out + c * oplane + (size_t)y * k.ow + x, v[c]);
        }
    }
}

}  // namespace ta

#include "ta_affine_roles.cuh"
