// Kernel tables.  Every (element type, kind, channels, colour flags) combination is its
// own kernel so that disabled operations cost nothing; each translation unit
// instantiates one (element type, kind) slice and exposes it as a table of function
// pointers indexed by the flag bits.
#pragma once

#include <utility>

#include "ta_affine.cuh"
#include "ta_direct.cuh"

namespace ta {

constexpr int kNumFlagCombos = 64;   // kB | kC | kS | kG | kN | kMean

struct KernelTable {
    const void *c3[kNumFlagCombos];
    const void *c1[kNumFlagCombos];
    const void *c3_checked;          // affine only, flags 0, staging asserts on
    const void *c1_checked;
};

constexpr bool flags_valid(int channels, unsigned f)
{
    if ((f & kMean) && !(f & kC)) return false;              // mean mode only qualifies contrast
    if (channels == 1 && (f & (kS | kG))) return false;      // need RGB
    return true;
}

// KIND 0 crop/flip, 1 affine nearest, 2 affine bilinear
template <typename T, int C, int KIND, unsigned F> const void *kernel_ptr()
{
    if constexpr (!flags_valid(C, F)) return nullptr;
    else if constexpr (KIND == 0) return (const void *)&direct_kernel<T, C, F>;
    else return (const void *)&affine_kernel<T, C, KIND, F, false>;
}

template <typename T, int KIND, unsigned... Fs>
void fill_table(KernelTable &t, std::integer_sequence<unsigned, Fs...>)
{
    ((t.c3[Fs] = kernel_ptr<T, 3, KIND, Fs>()), ...);
    ((t.c1[Fs] = kernel_ptr<T, 1, KIND, Fs>()), ...);
    if constexpr (KIND != 0) {
        t.c3_checked = (const void *)&affine_kernel<T, 3, KIND, 0u, true>;
        t.c1_checked = (const void *)&affine_kernel<T, 1, KIND, 0u, true>;
    } else {
        t.c3_checked = t.c1_checked = nullptr;
    }
}

template <typename T, int KIND> const KernelTable &make_table()
{
    static KernelTable t = [] {
        KernelTable x{};
        fill_table<T, KIND>(x, std::make_integer_sequence<unsigned, kNumFlagCombos>{});
        return x;
    }();
    return t;
}

// Defined one per translation unit (ta_inst_*.cu).
const KernelTable &table_f32_direct();
const KernelTable &table_f32_nearest();
const KernelTable &table_f32_bilinear();
const KernelTable &table_f16_direct();
const KernelTable &table_f16_nearest();
const KernelTable &table_f16_bilinear();

}  // namespace ta
