// Shared device-side pieces of the sm_100a augmentation kernels: kernel argument
// block, mbarrier / bulk-copy PTX wrappers, exact coordinate arithmetic, texel
// sampling and the colour tier.
#pragma once

#include <cuda_fp16.h>
#include <type_traits>
#include <cuda_runtime.h>
#include <limits.h>
#include <stdint.h>

#include "ta_footprint.h"

namespace ta {

// Colour flags as template bits (same values as TA_B200_APPLY_*), plus the contrast mode.
constexpr unsigned kB = 1u, kC = 2u, kS = 4u, kG = 8u, kN = 16u, kMean = 32u;

constexpr int kThreads = 256;          // per CTA, every kernel
constexpr int kWarps = kThreads / 32;

// Device status words (one block per device, see ta_api.cu).
enum { kCntStaged = 0, kCntDirect = 1, kCntViolation = 2, kCntTimeout = 3 };

struct KArgs {
    const void *in;
    void *out;
    const float *top, *left;
    const uint8_t *flip;
    const float *matrix;
    const void *bf, *cf, *sf;
    const uint8_t *gray;
    const float *gray_mean;
    float *mean_partials;              // staged grayscale-mean pre-pass: [image][tile][consumer warp] sums
    // One-launch mean contrast (two-phase kernel): per image, how many partial sums have been
    // written, whether the image's mean is final, and the means themselves (= gray_mean).
    unsigned *mean_done, *mean_ready;
    float *mean_out;
    int mean_pixels;                   // pixels per output image (divisor of the mean)
    int mean_lag;                      // the fused pass of an image runs this many images behind its reduction
    unsigned long long *counters;
    unsigned *status;                  // host-mapped word: set to 1 when a bounded wait runs out (NULL: not reported)
    unsigned long long wait_ns;        // limit of every barrier wait
    int skip_arrive_tile;              // diagnostics: the producer of this tile leaves without its arrival (-1: never)
    int n, h, w, oh, ow;
    int tiles_x, tiles_y, num_tiles;
    int staged_ok;                     // source rows can be bulk-copied (16-byte aligned pitch and base)
    int late_x_slot;                   // see late_x(): 8 = never
    int pair_store;                    // half output: pairs of columns (x even) are 4-byte aligned in every row
    unsigned lin_base;                 // linear index of this launch's first output element within the caller's batch (late_x())
    float fill[3];                     // per channel: value of texels outside the image (affine only)
    float mean[3], stdv[3];            // image-dtype-rounded values
    float inv_std[3], nbias[3];        // 1/std and -mean/std (fp32 path)
};

// ----------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    // (a suspend-time hint of 1 or 10 us on the poll changed neither the time nor the power draw)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// ----------------------------------------------------------------------------- packed fp32
// Two independent IEEE round-to-nearest operations per instruction on sm_100 (fma.rn.f32x2 and
// friends).
__device__ __forceinline__ float2 pk_fma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 pk_mul(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 pk_add(float2 a, float2 b) { return __fadd2_rn(a, b); }
// Packed addition rounded towards minus infinity (the floor step of floor_magic, two at once).
__device__ __forceinline__ float2 pk_add_rd(float2 a, float2 b) { return __fadd2_rd(a, b); }

// ----------------------------------------------------------------------------- conversions without the XU pipe
// float <-> int conversions issue at a quarter of the FMA rate.  For |v| < 2^22 the same
// integers fall out of one addition of 1.5 * 2^23, whose unit in the last place is 1: the sum
// is rounded to an integer by the adder itself, to nearest-even (= rint) or downwards (= floor)
// depending on the instruction's rounding mode, and the integer sits in the low mantissa bits.
// The staged path only sees coordinates below kCoordLimit, so the results equal
// cvt.rni / cvt.rmi bit for bit there.
constexpr float kMagic = 12582912.0f;            // 1.5 * 2^23, bit pattern 0x4B400000
constexpr int kMagicBits = 0x4B400000;

__device__ __forceinline__ int rint_magic(float v) { return __float_as_int(__fadd_rn(v, kMagic)) - kMagicBits; }

// floor(v) as int, and v - floor(v) (exact, the same value as v - (float)floor)
__device__ __forceinline__ int floor_magic(float v, float &frac)
{
    const float t = __fadd_rd(v, kMagic);
    frac = __fsub_rn(v, __fsub_rn(t, kMagic));
    return __float_as_int(t) - kMagicBits;
}

// ----------------------------------------------------------------------------- element access
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
    // load from a 32-bit shared-memory address (constant offsets fold into the instruction)
    static __device__ __forceinline__ float lds(uint32_t addr)
    {
        float v;
        asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
        return v;
    }
    // plain store: st.global.cs measured no better for float (0-2 % worse)
    static __device__ __forceinline__ void store(float *p, float v) { *p = v; }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ __half lds(uint32_t addr)
    {
        unsigned short v;
        asm("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
        return __ushort_as_half(v);
    }
    static __device__ __forceinline__ void store(__half *p, float v)
    {
        __stcs(reinterpret_cast<unsigned short *>(p), __half_as_ushort(__float2half_rn(v)));
    }
};

// Two pixels that go through the pipeline together (two rows of one column for float images,
// two neighbouring columns of one row for half images): float2 / __half2.
template <typename T> struct PairOf;
template <> struct PairOf<float> {
    using type = float2;
    static __device__ __forceinline__ float2 make(float a, float b) { return make_float2(a, b); }
    static __device__ __forceinline__ float2 from_f2(float2 v) { return v; }
    static __device__ __forceinline__ float first(float2 v) { return v.x; }
    static __device__ __forceinline__ float second(float2 v) { return v.y; }
};
template <> struct PairOf<__half> {
    using type = __half2;
    static __device__ __forceinline__ __half2 make(__half a, __half b) { return __halves2half2(a, b); }
    static __device__ __forceinline__ __half2 from_f2(float2 v) { return __floats2half2_rn(v.x, v.y); }   // one packed conversion
    static __device__ __forceinline__ __half first(__half2 v) { return __low2half(v); }
    static __device__ __forceinline__ __half second(__half2 v) { return __high2half(v); }
};

// ----------------------------------------------------------------------------- geometry
// Per-image geometry, loaded once per tile.
struct Geom {
    float top, left;
    bool flip;
    float a, b, c, d, e, f;
    float half_w, half_h;
};

__device__ __forceinline__ void load_geom(Geom &g, const KArgs &k, int n, bool affine)
{
    g.top = k.top ? __ldg(k.top + n) : 0.0f;
    g.left = k.left ? __ldg(k.left + n) : 0.0f;
    g.flip = k.flip ? __ldg(k.flip + n) != 0 : false;
    g.half_w = (float)k.w * 0.5f;
    g.half_h = (float)k.h * 0.5f;
    if (affine) {
        const float *m = k.matrix + (size_t)n * 6;
        g.a = __ldg(m + 0); g.b = __ldg(m + 1); g.c = __ldg(m + 2);
        g.d = __ldg(m + 3); g.e = __ldg(m + 4); g.f = __ldg(m + 5);
    } else {
        g.a = g.e = 1.0f;
        g.b = g.c = g.d = g.f = 0.0f;
    }
}

// x_img / y_img of triton_augment/kernels/geometric_kernel.py:390-394.
__device__ __forceinline__ float img_x(const Geom &g, int ow, int x)
{
    return __fadd_rn((float)(g.flip ? ow - 1 - x : x), g.left);
}
__device__ __forceinline__ float img_y(const Geom &g, int y) { return __fadd_rn((float)y, g.top); }

// Centred coordinate, geometric_kernel.py:410-411: (v - half) + 0.5.
__device__ __forceinline__ float centred(float v, float half) { return __fadd_rn(__fsub_rn(v, half), 0.5f); }

// Which of the two products of a*xc + b*yc the reference's GPU build fuses into the addition
// is a choice its compiler makes per compiled variant (every flag combination is a separate
// LLVM module).  Measured on a B200 with Triton 3.6 against all 32 colour-flag combinations:
//   nearest  : x and y use fma(xc, a, b*yc)                                   -> recipe 1, 1
//   bilinear : x = fma(xc, a, b*yc), y = fma(yc, e, d*xc)                     -> recipe 1, 2
//              except with (saturation or grayscale) and (brightness or contrast) on,
//              where x = fma(yc, b, a*xc), y = fma(xc, d, e*yc)               -> recipe 2, 1
// MODE 1 nearest, 2 bilinear (0, crop/flip without a matrix, has no coordinate arithmetic); F the colour flags.
template <int MODE, unsigned F> struct CoordRecipe {
    static constexpr bool swapped = MODE == 2 && (F & (kS | kG)) != 0 && (F & (kB | kC)) != 0;
    static constexpr int x = MODE == 2 ? (swapped ? 2 : 1) : 1;
    static constexpr int y = MODE == 2 ? (swapped ? 1 : 2) : 1;
};

// Source coordinate, geometric_kernel.py:414-415, in the reference's operation order:
// ((fma + c) + half) + (-0.5).  Every step is an explicitly rounded intrinsic so the compiler
// cannot re-associate or fuse; R picks the contraction (see CoordRecipe).
// In the swapped bilinear variants the reference's GPU build contracts x the other way
// (recipe 1) for some pixels when its stores are not vectorised, i.e. when neither output
// dimension is divisible by 16: it handles 1024 consecutive output pixels per program with 128
// threads, a thread's j-th pixel lies 128 j further on, and the last 1-3 of a thread's 8 pixels
// are the ones compiled differently.  `lin` is the pixel's index in the [N, oh, ow] output
// (its low 10 bits are enough); the host sets late_x_slot = 8 - (that count), or 8 for never.
__device__ __forceinline__ bool late_x(const KArgs &k, uint32_t lin) { return (int)((lin >> 7) & 7u) >= k.late_x_slot; }

template <int R> __device__ __forceinline__ float src_coord_r(float xc, float yc, float a, float b, float c, float half)
{
    float u = R == 1 ? __fmaf_rn(xc, a, __fmul_rn(b, yc)) : __fmaf_rn(yc, b, __fmul_rn(a, xc));
    u = __fadd_rn(u, c);
    u = __fadd_rn(half, u);
    return __fadd_rn(u, -0.5f);
}

// ----------------------------------------------------------------------------- colour tier
// Restates triton_augment/kernels/fused_kernel.py:234-283.  F holds the compiled-in operations.
template <typename T, int C, unsigned F> struct Colour;

__device__ __forceinline__ float gray_of(float r, float g, float b)
{
    return __fmaf_rn(0.114f, b, __fmaf_rn(0.587f, g, 0.2989f * r));
}

template <int C, unsigned F> struct Colour<float, C, F> {
    float bf, cf, sf, oms, gmt;
    bool gray;
    __device__ __forceinline__ void init(const KArgs &k, int n)
    {
        bf = cf = sf = 1.0f; oms = gmt = 0.0f; gray = false;
        if (F & kB) bf = __ldg((const float *)k.bf + n);
        if (F & kC) {
            cf = __ldg((const float *)k.cf + n);
            if (F & kMean) gmt = __ldcg(k.gray_mean + n) * (1.0f - cf);     // (may have been written by this very launch)
        }
        if (F & kS) { sf = __ldg((const float *)k.sf + n); oms = 1.0f - sf; }
        if (F & kG) gray = __ldg(k.gray + n) != 0;
    }
    // v: texels as sampled; returns values ready to store.
    __device__ __forceinline__ void apply(const KArgs &k, const float (&in)[C], float (&v)[C]) const
    {
#pragma unroll
        for (int i = 0; i < C; ++i) v[i] = in[i];
        if (F & kB) {
#pragma unroll
            for (int i = 0; i < C; ++i) v[i] = __saturatef(v[i] * bf);
        }
        if (F & kC) {
#pragma unroll
            for (int i = 0; i < C; ++i)
                v[i] = (F & kMean) ? __saturatef(__fmaf_rn(v[i], cf, gmt))
                                   : __saturatef(__fmaf_rn(v[i] - 0.5f, cf, 0.5f));
        }
        if (C == 3 && (F & kS)) {
            const float gg = gray_of(v[0], v[1], v[2]) * oms;
#pragma unroll
            for (int i = 0; i < C; ++i) v[i] = __saturatef(__fmaf_rn(v[i], sf, gg));
        }
        if (C == 3 && (F & kG)) {
            if (gray) {
                const float g = gray_of(v[0], v[1], v[2]);
#pragma unroll
                for (int i = 0; i < C; ++i) v[i] = g;
            }
        }
        if (F & kN) {
#pragma unroll
            for (int i = 0; i < C; ++i) v[i] = __fmaf_rn(v[i], k.inv_std[i], k.nbias[i]);
        }
    }
    // Two pixels at once (.x and .y of each channel): everything that does not clamp goes
    // through the packed fp32 pipe, the clamping steps stay scalar because only scalar
    // multiplies / FMAs carry the saturate modifier.  Same arithmetic per pixel as apply().
    // G: what is known about the image's grayscale flag at compile time (0 nothing: test it here,
    // 1 not set, 2 set), for callers that branch on it once per tile instead of once per pixel pair.
    template <int G = 0> __device__ __forceinline__ void apply2(const KArgs &k, float2 (&v)[C]) const
    {
        if (F & kB) {
#pragma unroll
            for (int i = 0; i < C; ++i) v[i] = make_float2(__saturatef(v[i].x * bf), __saturatef(v[i].y * bf));
        }
        if (F & kC) {
#pragma unroll
            for (int i = 0; i < C; ++i) {
                if (F & kMean) {
                    v[i] = make_float2(__saturatef(__fmaf_rn(v[i].x, cf, gmt)), __saturatef(__fmaf_rn(v[i].y, cf, gmt)));
                } else {
                    const float2 d = pk_add(v[i], make_float2(-0.5f, -0.5f));
                    v[i] = make_float2(__saturatef(__fmaf_rn(d.x, cf, 0.5f)), __saturatef(__fmaf_rn(d.y, cf, 0.5f)));
                }
            }
        }
        if (C == 3 && (F & kS)) {
            float2 g = pk_mul(make_float2(0.2989f, 0.2989f), v[0]);
            g = pk_fma(make_float2(0.587f, 0.587f), v[1], g);
            g = pk_fma(make_float2(0.114f, 0.114f), v[C - 1], g);
            g = pk_mul(g, make_float2(oms, oms));
#pragma unroll
            for (int i = 0; i < C; ++i)
                v[i] = make_float2(__saturatef(__fmaf_rn(v[i].x, sf, g.x)), __saturatef(__fmaf_rn(v[i].y, sf, g.y)));
        }
        if (C == 3 && (F & kG)) {
            if (G == 2 || (G == 0 && gray)) {
                float2 g = pk_mul(make_float2(0.2989f, 0.2989f), v[0]);
                g = pk_fma(make_float2(0.587f, 0.587f), v[1], g);
                g = pk_fma(make_float2(0.114f, 0.114f), v[C - 1], g);
#pragma unroll
                for (int i = 0; i < C; ++i) v[i] = g;
            }
        }
        if (F & kN) {
#pragma unroll
            for (int i = 0; i < C; ++i)
                v[i] = pk_fma(v[i], make_float2(k.inv_std[i], k.inv_std[i]), make_float2(k.nbias[i], k.nbias[i]));
        }
    }
};

// fp16 images: the reference's GPU build keeps a value in fp16 until the first clamp of
// an enabled operation and in fp32 from there to the store; factors, mean and std are
// fp16 values and (1 - saturation) is an fp16 subtraction.
template <int C, unsigned F> struct Colour<__half, C, F> {
    __half bh, ch, sh, omsh, gmth;
    float cf, sf, oms, gmt;
    bool gray;
    __device__ __forceinline__ void init(const KArgs &k, int n)
    {
        const __half one = __float2half_rn(1.0f);
        bh = ch = sh = one; omsh = gmth = __float2half_rn(0.0f);
        cf = sf = 1.0f; oms = gmt = 0.0f; gray = false;
        if (F & kB) bh = ((const __half *)k.bf)[n];
        if (F & kC) {
            ch = ((const __half *)k.cf)[n];
            cf = __half2float(ch);
            if (F & kMean) {
                const __half omc = __hsub(one, ch);
                const float m = __ldcg(k.gray_mean + n);
                gmth = __hmul(__float2half_rn(m), omc);
                gmt = m * __half2float(omc);
            }
        }
        if (F & kS) {
            sh = ((const __half *)k.sf)[n];
            sf = __half2float(sh);
            omsh = __hsub(one, sh);
            oms = __half2float(omsh);
        }
        if (F & kG) gray = __ldg(k.gray + n) != 0;
    }
    static __device__ __forceinline__ __half gray_h(__half r, __half g, __half b)
    {
        return __hadd(__hadd(__hmul(__float2half_rn(0.2989f), r), __hmul(__float2half_rn(0.587f), g)),
                      __hmul(__float2half_rn(0.114f), b));
    }
    __device__ __forceinline__ void apply(const KArgs &k, const __half (&in)[C], float (&v)[C]) const
    {
        __half hv[C];
#pragma unroll
        for (int i = 0; i < C; ++i) hv[i] = in[i];
        constexpr bool wide_after_b = (F & kB) != 0;
        constexpr bool wide_after_c = wide_after_b || (F & kC) != 0;
        constexpr bool wide_after_s = wide_after_c || (C == 3 && (F & kS) != 0);
        if (F & kB) {
#pragma unroll
            for (int i = 0; i < C; ++i) v[i] = __saturatef(__half2float(__hmul(hv[i], bh)));
        }
        if (F & kC) {
#pragma unroll
            for (int i = 0; i < C; ++i) {
                if (wide_after_b) {
                    v[i] = (F & kMean) ? __saturatef(__fmaf_rn(v[i], cf, gmt))
                                       : __saturatef(__fmaf_rn(v[i] - 0.5f, cf, 0.5f));
                } else if (F & kMean) {
                    v[i] = __saturatef(__half2float(__hadd(__hmul(hv[i], ch), gmth)));
                } else {
                    const __half hh = __float2half_rn(0.5f);
                    v[i] = __saturatef(__half2float(__hadd(__hmul(__hsub(hv[i], hh), ch), hh)));
                }
            }
        }
        if (C == 3 && (F & kS)) {
            if (wide_after_c) {
                const float gg = gray_of(v[0], v[1], v[2]) * oms;
#pragma unroll
                for (int i = 0; i < C; ++i) v[i] = __saturatef(__fmaf_rn(v[i], sf, gg));
            } else {
                const __half gg = __hmul(gray_h(hv[0], hv[1], hv[2]), omsh);
#pragma unroll
                for (int i = 0; i < C; ++i) v[i] = __saturatef(__half2float(__hadd(__hmul(hv[i], sh), gg)));
            }
        }
        if (C == 3 && (F & kG)) {
            if (gray) {
                if (wide_after_s) {
                    const float g = gray_of(v[0], v[1], v[2]);
#pragma unroll
                    for (int i = 0; i < C; ++i) v[i] = g;
                } else {
                    const __half g = gray_h(hv[0], hv[1], hv[2]);
#pragma unroll
                    for (int i = 0; i < C; ++i) hv[i] = g;
                }
            }
        }
        if (F & kN) {
#pragma unroll
            for (int i = 0; i < C; ++i) {
                if (wide_after_s)
                    v[i] = __fmaf_rn(v[i], k.inv_std[i], k.nbias[i]);      // fp32 from the first clamp on, as for float images
                else
                    v[i] = __half2float(__hdiv(__hsub(hv[i], __float2half_rn(k.mean[i])),
                                               __float2half_rn(k.stdv[i])));
            }
        } else if (!wide_after_s) {
#pragma unroll
            for (int i = 0; i < C; ++i) v[i] = __half2float(hv[i]);
        }
    }
    // Two pixels at once: a[] and b[] are the texels of the pair, v[i] = (result for a, result
    // for b).  Per pixel the same operations in the same precision as apply(): half2 arithmetic
    // where apply() uses half, packed or saturating fp32 where it uses fp32.
    static __device__ __forceinline__ __half2 gray_h2(__half2 r, __half2 g, __half2 b)
    {
        return __hadd2(__hadd2(__hmul2(__float2half2_rn(0.2989f), r), __hmul2(__float2half2_rn(0.587f), g)),
                       __hmul2(__float2half2_rn(0.114f), b));
    }
    static __device__ __forceinline__ float2 sat2(float2 x) { return make_float2(__saturatef(x.x), __saturatef(x.y)); }
    static __device__ __forceinline__ float2 gray_f2(const float2 (&v)[C])
    {
        float2 g = pk_mul(make_float2(0.2989f, 0.2989f), v[0]);
        g = pk_fma(make_float2(0.587f, 0.587f), v[C > 1 ? 1 : 0], g);
        return pk_fma(make_float2(0.114f, 0.114f), v[C - 1], g);
    }
    // half2 product clamped to [0, 1] in one instruction; the clamp of a half value is the same
    // in half and in float (0 and 1 are exact), NaN -> 0 like __saturatef
    static __device__ __forceinline__ __half2 hmul2_sat(__half2 a, __half2 b)
    {
        __half2 r;
        asm("mul.rn.sat.f16x2 %0, %1, %2;" : "=r"(*reinterpret_cast<unsigned *>(&r))
            : "r"(*reinterpret_cast<const unsigned *>(&a)), "r"(*reinterpret_cast<const unsigned *>(&b)));
        return r;
    }
    template <int G = 0> __device__ __forceinline__ void apply2(const KArgs &k, const __half2 (&in)[C], float2 (&v)[C]) const
    {
        __half2 hv[C];
#pragma unroll
        for (int i = 0; i < C; ++i) hv[i] = in[i];
        constexpr bool wide_after_b = (F & kB) != 0;
        constexpr bool wide_after_c = wide_after_b || (F & kC) != 0;
        constexpr bool wide_after_s = wide_after_c || (C == 3 && (F & kS) != 0);
        if (F & kB) {
            const __half2 bh2 = __half2half2(bh);
#pragma unroll
            for (int i = 0; i < C; ++i) v[i] = __half22float2(hmul2_sat(hv[i], bh2));
        }
        if (F & kC) {
#pragma unroll
            for (int i = 0; i < C; ++i) {
                if (wide_after_b) {
                    if (F & kMean) {
                        v[i] = make_float2(__saturatef(__fmaf_rn(v[i].x, cf, gmt)), __saturatef(__fmaf_rn(v[i].y, cf, gmt)));
                    } else {
                        const float2 d = pk_add(v[i], make_float2(-0.5f, -0.5f));
                        v[i] = make_float2(__saturatef(__fmaf_rn(d.x, cf, 0.5f)), __saturatef(__fmaf_rn(d.y, cf, 0.5f)));
                    }
                } else if (F & kMean) {
                    v[i] = sat2(__half22float2(__hadd2(__hmul2(hv[i], __half2half2(ch)), __half2half2(gmth))));
                } else {
                    const __half2 hh = __float2half2_rn(0.5f);
                    v[i] = sat2(__half22float2(__hadd2(__hmul2(__hsub2(hv[i], hh), __half2half2(ch)), hh)));
                }
            }
        }
        if (C == 3 && (F & kS)) {
            if (wide_after_c) {
                const float2 gg = pk_mul(gray_f2(v), make_float2(oms, oms));
#pragma unroll
                for (int i = 0; i < C; ++i)
                    v[i] = make_float2(__saturatef(__fmaf_rn(v[i].x, sf, gg.x)), __saturatef(__fmaf_rn(v[i].y, sf, gg.y)));
            } else {
                const __half2 gg = __hmul2(gray_h2(hv[0], hv[C > 1 ? 1 : 0], hv[C - 1]), __half2half2(omsh));
#pragma unroll
                for (int i = 0; i < C; ++i) v[i] = sat2(__half22float2(__hadd2(__hmul2(hv[i], __half2half2(sh)), gg)));
            }
        }
        if (C == 3 && (F & kG)) {
            if (G == 2 || (G == 0 && gray)) {
                if (wide_after_s) {
                    const float2 g = gray_f2(v);
#pragma unroll
                    for (int i = 0; i < C; ++i) v[i] = g;
                } else {
                    const __half2 g = gray_h2(hv[0], hv[C > 1 ? 1 : 0], hv[C - 1]);
#pragma unroll
                    for (int i = 0; i < C; ++i) hv[i] = g;
                }
            }
        }
        if (F & kN) {
#pragma unroll
            for (int i = 0; i < C; ++i) {
                if (wide_after_s)
                    v[i] = pk_fma(v[i], make_float2(k.inv_std[i], k.inv_std[i]), make_float2(k.nbias[i], k.nbias[i]));
                else
                    v[i] = __half22float2(__h2div(__hsub2(hv[i], __float2half2_rn(k.mean[i])), __float2half2_rn(k.stdv[i])));
            }
        } else if (!wide_after_s) {
#pragma unroll
            for (int i = 0; i < C; ++i) v[i] = __half22float2(hv[i]);
        }
    }
};

// ----------------------------------------------------------------------------- global-memory taps
// Used by the crop/flip kernel and by affine tiles that are not staged.  Bounds-checked;
// texels outside the image read as `fill` (affine) or 0 (crop/flip).
template <typename T>
__device__ __forceinline__ T tap_global(const T *plane, int w, int h, int x, int y, T fillv)
{
    const bool ok = (unsigned)x < (unsigned)w && (unsigned)y < (unsigned)h;
    return ok ? __ldg(plane + (size_t)y * w + x) : fillv;
}

// Bilinear blend, triton_augment/kernels/geometric_kernel.py:239-246 with the fma chain of
// the reference's GPU build: p00*w00, then three fused accumulations.
__device__ __forceinline__ float blend4(float p00, float p10, float p01, float p11, float dx, float dy)
{
    const float omx = 1.0f - dx, omy = 1.0f - dy;
    float r = p00 * (omx * omy);
    r = __fmaf_rn(p10, dx * omy, r);
    r = __fmaf_rn(p01, omx * dy, r);
    r = __fmaf_rn(p11, dx * dy, r);
    return r;
}

}  // namespace ta
