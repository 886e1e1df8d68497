#include "ta_tables.cuh"
namespace ta {
template <typename S> static KernelEntry pick(int mode, bool bright, int channels)
{
#define TA_ME(CC, MM) (bright ? mean_entry<CC, MM, kB, S>() : mean_entry<CC, MM, 0u, S>())
    if (channels == 3) return mode == 0 ? TA_ME(3, 0) : mode == 1 ? TA_ME(3, 1) : TA_ME(3, 2);
    return mode == 0 ? TA_ME(1, 0) : mode == 1 ? TA_ME(1, 1) : TA_ME(1, 2);
#undef TA_ME
}
KernelEntry mean_kernel_entry(int mode, bool bright, int channels, bool bytes)
{
    return bytes ? pick<uint8_t>(mode, bright, channels) : pick<float>(mode, bright, channels);
}
}
