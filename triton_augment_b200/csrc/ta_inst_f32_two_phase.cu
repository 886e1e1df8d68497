#include "ta_tables.cuh"
namespace ta {
const KernelTable &table_f32_two_phase(int mode)
{
    return mode == 0 ? make_table<float, 5>() : mode == 1 ? make_table<float, 6>() : make_table<float, 7>();
}
}
