// Kernel tables.  Every (element type, kind, channels, colour flags) combination is its
// own kernel so that disabled operations cost nothing; each translation unit
// instantiates one (element type, kind) slice and exposes it as a table of function
// pointers (and their dynamic shared memory sizes) indexed by the flag bits.
#pragma once

#include <utility>

#include "ta_affine.cuh"
#include "ta_direct.cuh"
#include "ta_direct_vec.cuh"

namespace ta {

constexpr int kNumFlagCombos = 64;   // kB | kC | kS | kG | kN | kMean

struct KernelEntry {
    const void *fn;      // nullptr: combination does not exist
    size_t smem;         // dynamic shared memory
    int threads;         // CTA size
};

struct KernelTable {
    KernelEntry c3[kNumFlagCombos];
    KernelEntry c1[kNumFlagCombos];
    KernelEntry c3_vec[kNumFlagCombos];   // crop/flip only: the 128-bit variant (direct_vec_kernel)
    KernelEntry c1_vec[kNumFlagCombos];
    KernelEntry c3_checked;          // affine only, flags 0, staging assertions on
    KernelEntry c1_checked;
};

constexpr bool flags_valid(int channels, unsigned f)
{
    if ((f & kMean) && !(f & kC)) return false;              // mean mode only qualifies contrast
    if (channels == 1 && (f & (kS | kG))) return false;      // need RGB
    return true;
}

// KIND 0 crop/flip, 1 affine nearest, 2 affine bilinear, 3 crop/flip through the staged kernel,
// 4 affine bilinear with the per-pixel x contraction of late_x() (swapped variants only),
// 5 / 6 / 7 the two-phase kernel (mean reduction + fused pass in one launch) without a matrix /
// nearest / bilinear: exists for the flag combinations with mean-mode contrast.
// S: source element type (uint8_t with T = float or half: bytes scaled by 1/255; staged kernels only).
// TH: tile height of the staged kernels (kTileH, or kTileHShort for small float outputs).
template <typename T, int C, int KIND, unsigned F, bool CHECK = false, typename S = T, int TH = kTileH> KernelEntry kernel_entry()
{
    if constexpr (!flags_valid(C, F)) return KernelEntry{nullptr, 0, 0};
    else if constexpr (KIND == 0) return KernelEntry{(const void *)&direct_kernel<T, C, F>, 0, kThreads};
    else if constexpr (KIND >= 5) {
        if constexpr ((F & kMean) != 0 && !CHECK)
            return KernelEntry{(const void *)&affine_kernel<T, C, KIND - 5, F, false, false, S, false, true>,
                               AffineSmem<T, C, F, S>::total, Ring<S, kTileH>::threads + 32};      // + the finisher warp
        else return KernelEntry{nullptr, 0, 0};
    }
    else if constexpr (KIND == 4) {
        if constexpr (CoordRecipe<2, F>::swapped && !CHECK)
            return KernelEntry{(const void *)&affine_kernel<T, C, 2, F, false, true, S, false, false, TH>,
                               AffineSmem<T, C, F, S, TH>::total, Ring<S, TH>::threads};
        else return KernelEntry{nullptr, 0, 0};
    } else return KernelEntry{(const void *)&affine_kernel<T, C, KIND == 3 ? 0 : KIND, F, CHECK, false, S, false, false, TH>,
                              AffineSmem<T, C, F, S, TH>::total, Ring<S, TH>::threads};
}

template <typename T, int C, unsigned F> KernelEntry vec_entry()
{
    if constexpr (!flags_valid(C, F)) return KernelEntry{nullptr, 0, 0};
    else return KernelEntry{(const void *)&direct_vec_kernel<T, C, F>, 0, kThreads};
}

template <typename T, int KIND, typename S, int TH, unsigned... Fs>
void fill_table(KernelTable &t, std::integer_sequence<unsigned, Fs...>)
{
    ((t.c3[Fs] = kernel_entry<T, 3, KIND, Fs, false, S, TH>()), ...);
    ((t.c1[Fs] = kernel_entry<T, 1, KIND, Fs, false, S, TH>()), ...);
    if constexpr (KIND >= 5) {
        t.c3_checked = t.c1_checked = KernelEntry{nullptr, 0, 0};
    } else if constexpr (KIND != 0) {
        t.c3_checked = kernel_entry<T, 3, KIND, 0u, true, S, TH>();
        t.c1_checked = kernel_entry<T, 1, KIND, 0u, true, S, TH>();
    } else {
        t.c3_checked = t.c1_checked = KernelEntry{nullptr, 0, 0};
        ((t.c3_vec[Fs] = vec_entry<T, 3, Fs>()), ...);
        ((t.c1_vec[Fs] = vec_entry<T, 1, Fs>()), ...);
    }
}

template <typename T, int KIND, typename S = T, int TH = kTileH> const KernelTable &make_table()
{
    static KernelTable t = [] {
        KernelTable x{};
        fill_table<T, KIND, S, TH>(x, std::make_integer_sequence<unsigned, kNumFlagCombos>{});
        return x;
    }();
    return t;
}

// Staged grayscale-mean pre-pass (float32 pixels from float or uint8 images): mode 0 no matrix /
// 1 nearest / 2 bilinear, with or without brightness, 3 or 1 channels.  Defined in ta_inst_f32_mean.cu.
KernelEntry mean_kernel_entry(int mode, bool bright, int channels, bool bytes);

template <int C, int MODE, unsigned F, typename S> KernelEntry mean_entry()
{
    return KernelEntry{(const void *)&affine_kernel<float, C, MODE, F, false, false, S, true>,
                       AffineSmem<float, C, F, S>::total, Ring<S, kTileH>::threads};
}

// Defined one per translation unit (ta_inst_*.cu).
const KernelTable &table_f32_direct();
const KernelTable &table_f32_crop_staged();
const KernelTable &table_f32_bilinear_mix();
const KernelTable &table_f32_two_phase(int mode);    // mode 0 no matrix, 1 nearest, 2 bilinear
const KernelTable &table_u8_crop_staged();
const KernelTable &table_u8_nearest();
const KernelTable &table_u8_bilinear();
const KernelTable &table_u8_bilinear_mix();
const KernelTable &table_u8h_crop_staged();     // bytes in, half out
const KernelTable &table_u8h_nearest();
const KernelTable &table_u8h_bilinear();
const KernelTable &table_f32_nearest();
const KernelTable &table_f32_bilinear();
const KernelTable &table_f32_short_nearest();        // float images on 64 x 32 tiles (small outputs)
const KernelTable &table_f32_short_bilinear();
const KernelTable &table_f32_short_crop_staged();
const KernelTable &table_f32_short_bilinear_mix();
const KernelTable &table_f16_short_nearest();          // half images on 64 x 32 tiles
const KernelTable &table_f16_short_bilinear();
const KernelTable &table_f16_direct();
const KernelTable &table_f16_nearest();
const KernelTable &table_f16_bilinear();

}  // namespace ta
