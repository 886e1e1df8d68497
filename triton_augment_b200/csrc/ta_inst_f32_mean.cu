#include "ta_tables.cuh"
namespace ta {
KernelEntry mean_kernel_entry(int mode, bool bright, int channels)
{
#define TA_ME(CC, MM) (bright ? mean_entry<CC, MM, kB>() : mean_entry<CC, MM, 0u>())
    if (channels == 3) return mode == 0 ? TA_ME(3, 0) : mode == 1 ? TA_ME(3, 1) : TA_ME(3, 2);
    return mode == 0 ? TA_ME(1, 0) : mode == 1 ? TA_ME(1, 1) : TA_ME(1, 2);
#undef TA_ME
}
}
